// What happens to the queries and keys of softmax attention between the projection and the attention kernel, for the
// forms that the kernel of qk_rope_store.cu does not know, in one pass over the packed rows
// [T, (Hq + Hkv) D + Hkv Dv (+ more)]: an RMS norm of q and of k, the half-split rotation of the first rotary_dim
// channels of every head, and the write of k and v into their pages.
//
//   span 0   no norm
//   span 1   every head by itself: x / sqrt(mean over the head + eps) (* weight[d], one weight for all heads, if given)
//   span 2   q as a whole, and k as a whole: one root mean square over all heads of the projection, weight [H D]
//   after    the norm follows the rotation instead of going before it (span 1 only: per head the order shows only
//            in the rounding, but the design says which)
// A CTA takes one token.  Every head passes through 32-bit shared memory of its warp: loaded, scaled, rotated, scaled,
// stored; q in place, k (and v, copied) to pages[slot_mapping[t] * Hkv + h], a negative slot meaning "do not write".
// Sums run in a fixed order (a head's by warp shuffles, a projection's by a fixed tree over the CTA).
#include "common.cuh"

using namespace mir;

namespace {

constexpr int kThreads = 256;

template <typename T>
__global__ void __launch_bounds__(kThreads)
qk_prepare_kernel(T* __restrict__ qkv, long long row_stride, const int* __restrict__ positions,
                  const int* __restrict__ slot_mapping, const float* __restrict__ inv_freq,
                  const float* __restrict__ q_weight, const float* __restrict__ k_weight, T* __restrict__ k_pages,
                  T* __restrict__ v_pages, int heads, int kv_heads, int head_dim, int value_dim, int rotary_dim, float eps,
                  int span, int after, int write_kv) {
  extern __shared__ float prepare_shared[];          // [rotary_dim] cosines, sines | [warps][head_dim]
  __shared__ float scratch[32];
  grid_launch_dependents();
  const int token = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = kThreads / 32;
  const int half = rotary_dim / 2;
  float* cosines = prepare_shared;
  float* sines = prepare_shared + half;
  float* mine = prepare_shared + rotary_dim + (size_t)warp * head_dim;
  const float position = (float)positions[token];
  const int slot = slot_mapping != nullptr ? slot_mapping[token] : -1;
  for (int pair = threadIdx.x; pair < half; pair += kThreads)
    sincosf(position * inv_freq[pair], &sines[pair], &cosines[pair]);
  grid_dependency_wait();
  T* row = qkv + (size_t)token * (size_t)row_stride;
  const int q_width = heads * head_dim, k_width = kv_heads * head_dim;
  float inverse_q = 1.0f, inverse_k = 1.0f;
  if (span == 2) {
    float sum_q = 0.0f, sum_k = 0.0f;
    for (int d = threadIdx.x; d < q_width; d += kThreads) { const float v = to_float(row[d]); sum_q = fmaf(v, v, sum_q); }
    for (int d = threadIdx.x; d < k_width; d += kThreads) { const float v = to_float(row[q_width + d]); sum_k = fmaf(v, v, sum_k); }
    inverse_q = rsqrtf(block_sum(sum_q, scratch) / (float)q_width + eps);
    inverse_k = rsqrtf(block_sum(sum_k, scratch) / (float)k_width + eps);
  }
  __syncthreads();
  const int units = heads + 2 * kv_heads;
  for (int unit = warp; unit < units; unit += warps) {
    if (unit >= heads + kv_heads) {                  // a value head: copied to its page
      if (write_kv != 1 || slot < 0) continue;
      const int value_head = unit - heads - kv_heads;
      const T* src = row + q_width + k_width + (size_t)value_head * value_dim;
      T* dst = v_pages + ((size_t)slot * kv_heads + value_head) * value_dim;
      for (int d = lane; d < value_dim; d += 32) dst[d] = src[d];
      continue;
    }
    const bool is_query = unit < heads;
    if (!is_query && (write_kv != 1 || slot < 0)) continue;
    const int local = is_query ? unit : unit - heads;
    T* src = row + (size_t)unit * head_dim;
    const float* weight = is_query ? q_weight : k_weight;
    for (int d = lane; d < head_dim; d += 32) mine[d] = to_float(src[d]);
    __syncwarp();
    if (span == 2) {
      const float inverse = is_query ? inverse_q : inverse_k;
      for (int d = lane; d < head_dim; d += 32)
        mine[d] = mine[d] * inverse * (weight != nullptr ? weight[(size_t)local * head_dim + d] : 1.0f);
    } else if (span == 1 && !after) {
      float sum = 0.0f;
      for (int d = lane; d < head_dim; d += 32) sum = fmaf(mine[d], mine[d], sum);
      const float inverse = rsqrtf(warp_sum(sum) / (float)head_dim + eps);
      for (int d = lane; d < head_dim; d += 32) mine[d] = mine[d] * inverse * (weight != nullptr ? weight[d] : 1.0f);
    }
    __syncwarp();
    for (int pair = lane; pair < half; pair += 32) {
      const float first = mine[pair], second = mine[pair + half];
      const float cosine = cosines[pair], sine = sines[pair];
      mine[pair] = first * cosine - second * sine;
      mine[pair + half] = second * cosine + first * sine;
    }
    __syncwarp();
    float late = 1.0f;
    if (span == 1 && after) {
      float sum = 0.0f;
      for (int d = lane; d < head_dim; d += 32) sum = fmaf(mine[d], mine[d], sum);
      late = rsqrtf(warp_sum(sum) / (float)head_dim + eps);
    }
    T* dst = is_query ? src : k_pages + ((size_t)slot * kv_heads + local) * head_dim;
    if (span == 1 && after) {
      for (int d = lane; d < head_dim; d += 32) dst[d] = from_float<T>(mine[d] * late * (weight != nullptr ? weight[d] : 1.0f));
    } else {
      for (int d = lane; d < head_dim; d += 32) dst[d] = from_float<T>(mine[d]);
    }
    __syncwarp();
  }
}

}  // namespace

// qkv: packed rows with row_stride elements from one token to the next (at least the width of q, k and v; what lies
// behind them is left alone).  inv_freq [rotary_dim / 2] (null with rotary_dim 0).  q_weight, k_weight: 32-bit, null
// for a norm without weights; [head_dim] with span 1, [heads * head_dim] and [kv_heads * head_dim] with span 2.
// write_kv 1: keys and values go to their pages; 0: only the queries are treated.
MIR_EXPORT int mir_qk_prepare(int bf16, void* qkv, long long row_stride, const int* positions, const int* slot_mapping,
                              const float* inv_freq, const float* q_weight, const float* k_weight, void* k_pages,
                              void* v_pages, int tokens, int heads, int kv_heads, int head_dim, int value_dim,
                              int rotary_dim, float eps, int span, int after, int write_kv, cudaStream_t stream) {
  if (tokens == 0) return MIR_OK;
  if (tokens < 0 || heads <= 0 || kv_heads <= 0 || head_dim <= 0 || value_dim <= 0 || rotary_dim < 0 ||
      rotary_dim > head_dim || (rotary_dim & 1) || span < 0 || span > 2 || (after && span != 1) ||
      (rotary_dim > 0 && inv_freq == nullptr) ||
      row_stride < (long long)(heads + kv_heads) * head_dim + (long long)kv_heads * value_dim ||
      (write_kv == 1 && (k_pages == nullptr || v_pages == nullptr || slot_mapping == nullptr))) {
    mir_set_error("qk_prepare: bad sizes or arguments (heads %d, kv heads %d, head_dim %d, rotary_dim %d, span %d, "
                  "row stride %lld)", heads, kv_heads, head_dim, rotary_dim, span, row_stride);
    return MIR_BAD_ARGUMENT;
  }
  const size_t smem = ((size_t)rotary_dim + (size_t)(kThreads / 32) * head_dim) * sizeof(float);
  if (smem > 48 * 1024) { mir_set_error("qk_prepare: heads of %d channels are too wide", head_dim); return MIR_BAD_ARGUMENT; }
  if (bf16)
    return mir_launch("qk_prepare", qk_prepare_kernel<__nv_bfloat16>, dim3(tokens), dim3(kThreads), smem, stream, 0,
                      (__nv_bfloat16*)qkv, row_stride, positions, slot_mapping, inv_freq, q_weight, k_weight,
                      (__nv_bfloat16*)k_pages, (__nv_bfloat16*)v_pages, heads, kv_heads, head_dim, value_dim, rotary_dim,
                      eps, span, after, write_kv);
  return mir_launch("qk_prepare", qk_prepare_kernel<float>, dim3(tokens), dim3(kThreads), smem, stream, 0, (float*)qkv,
                    row_stride, positions, slot_mapping, inv_freq, q_weight, k_weight, (float*)k_pages, (float*)v_pages,
                    heads, kv_heads, head_dim, value_dim, rotary_dim, eps, span, after, write_kv);
}
