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
// The kernel for any size and type: a CTA takes one token.  Every head passes through 32-bit shared memory of its warp: loaded, scaled, rotated, scaled,
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

// bf16 heads of 16 L channels, values as wide as keys, 16-byte rows: L lanes take one head, each with two 16-byte pieces
// (channels 8 l .. 8 l + 7 and those half a head further), a warp works on 32 / L heads at once.  The rotation's
// partner of a channel is the lane's other piece (the whole head rotated) or the same piece of the lane rotary_dim / 16
// further or back (at most half the head rotated, in steps of 16 channels).  A CTA takes `units_per_cta` heads of one
// token; with the norm over a projection it takes all of them, and sums the token's q and k rows first.
template <int L>
__global__ void qk_prepare_wide_kernel(__nv_bfloat16* __restrict__ qkv, long long row_stride,
                                       const int* __restrict__ positions, const int* __restrict__ slot_mapping,
                                       const float* __restrict__ inv_freq, const float* __restrict__ q_weight,
                                       const float* __restrict__ k_weight, __nv_bfloat16* __restrict__ k_pages,
                                       __nv_bfloat16* __restrict__ v_pages, int heads, int kv_heads, int rotary_dim,
                                       float eps, int span, int after, int write_kv, int units_per_cta, int resident) {
  constexpr int HALF = 8 * L, DIM = 2 * HALF, GROUPS = 32 / L;
  __shared__ float angles[DIM];                      // [pairs] cosines then [pairs] sines of this token
  __shared__ float scratch[64];
  grid_launch_dependents();
  const int token = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
  const int group = lane / L, l = lane % L;
  const int pairs = rotary_dim / 2, reach = rotary_dim / 16;
  const int units = heads + 2 * kv_heads;
  __nv_bfloat16* row = qkv + (size_t)token * (size_t)row_stride;
  const float position = (float)positions[token];
  const int slot = slot_mapping != nullptr ? slot_mapping[token] : -1;
  for (int pair = threadIdx.x; pair < pairs; pair += blockDim.x)
    sincosf(position * inv_freq[pair], &angles[pairs + pair], &angles[pair]);
  grid_dependency_wait();
  float inverse_q = 1.0f, inverse_k = 1.0f;
  if (span == 2 && !resident) {
    const int q_pieces = heads * DIM / 8, k_pieces = kv_heads * DIM / 8;
    float sum_q = 0.0f, sum_k = 0.0f;
    for (int piece = threadIdx.x; piece < q_pieces + k_pieces; piece += blockDim.x) {
      const uint4 raw = *reinterpret_cast<const uint4*>(row + 8 * (size_t)piece);
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
      float sum = 0.0f;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 x = __bfloat1622float2(h[i]);
        sum = fmaf(x.x, x.x, fmaf(x.y, x.y, sum));
      }
      if (piece < q_pieces) sum_q += sum; else sum_k += sum;
    }
    // both sums through one barrier: a warp's two sums side by side, then every thread adds the warps' in order
    sum_q = warp_sum(sum_q);
    sum_k = warp_sum(sum_k);
    if (lane == 0) { scratch[warp] = sum_q; scratch[32 + warp] = sum_k; }
    __syncthreads();
    sum_q = sum_k = 0.0f;
    for (int w = 0; w < warps; ++w) { sum_q += scratch[w]; sum_k += scratch[32 + w]; }
    inverse_q = rsqrtf(sum_q / (float)(heads * DIM) + eps);
    inverse_k = rsqrtf(sum_k / (float)(kv_heads * DIM) + eps);
  }
  __syncthreads();
  const int unit_begin = blockIdx.y * units_per_cta, unit_end = min(units, unit_begin + units_per_cta);
  // (resident: the CTA's warps hold all the token's heads at once, every warp runs the loop's body exactly once)
  for (int base = unit_begin + warp * GROUPS; resident || base < unit_end; base += warps * GROUPS) {
    const int unit = base + group;
    const bool active = unit < unit_end;
    const bool is_query = unit < heads, is_value = unit >= heads + kv_heads;
    const __nv_bfloat16* src = row + (size_t)unit * DIM;
    uint4 a = make_uint4(0u, 0u, 0u, 0u), b = a;
    if (active) {
      a = *reinterpret_cast<const uint4*>(src + 8 * l);
      b = *reinterpret_cast<const uint4*>(src + HALF + 8 * l);
    }
    const bool writes = active && (is_query || (write_kv == 1 && slot >= 0));
    __nv_bfloat16* dst = nullptr;
    if (writes)
      dst = is_query ? row + (size_t)unit * DIM
                     : (is_value ? v_pages + ((size_t)slot * kv_heads + (unit - heads - kv_heads)) * DIM
                                 : k_pages + ((size_t)slot * kv_heads + (unit - heads)) * DIM);
    float fa[8], fb[8];
    {
      const __nv_bfloat162* ha = reinterpret_cast<const __nv_bfloat162*>(&a);
      const __nv_bfloat162* hb = reinterpret_cast<const __nv_bfloat162*>(&b);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 x = __bfloat1622float2(ha[i]), y = __bfloat1622float2(hb[i]);
        fa[2 * i] = x.x; fa[2 * i + 1] = x.y; fb[2 * i] = y.x; fb[2 * i + 1] = y.y;
      }
    }
    const bool treated = active && !is_value;
    const int local = is_query ? unit : unit - heads;
    if (span == 2 && resident) {
      // the norm over a projection from the pieces in registers: nothing is read twice, and nothing is written
      // before every warp has its pieces
      float sum = 0.0f;
#pragma unroll
      for (int i = 0; i < 8; ++i) sum = fmaf(fa[i], fa[i], fmaf(fb[i], fb[i], sum));
      const float sum_q = warp_sum(treated && is_query ? sum : 0.0f), sum_k = warp_sum(treated && !is_query ? sum : 0.0f);
      if (lane == 0) { scratch[warp] = sum_q; scratch[32 + warp] = sum_k; }
      __syncthreads();
      float total_q = 0.0f, total_k = 0.0f;
      for (int w = 0; w < warps; ++w) { total_q += scratch[w]; total_k += scratch[32 + w]; }
      inverse_q = rsqrtf(total_q / (float)(heads * DIM) + eps);
      inverse_k = rsqrtf(total_k / (float)(kv_heads * DIM) + eps);
    }
    const float* weight = !treated ? nullptr : (is_query ? q_weight : k_weight);
    if (span == 2 || (span == 1 && !after)) {          // the norm before the rotation
      float inverse = is_query ? inverse_q : inverse_k;
      if (span == 1) {
        float sum = 0.0f;
#pragma unroll
        for (int i = 0; i < 8; ++i) sum = fmaf(fa[i], fa[i], fmaf(fb[i], fb[i], sum));
#pragma unroll
        for (int o = L / 2; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);   // every lane takes part
        inverse = rsqrtf(sum / (float)DIM + eps);
      }
      if (treated) {
        const float* w = weight == nullptr ? nullptr : weight + (span == 2 ? (size_t)local * DIM : 0);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          fa[i] *= inverse * (w != nullptr ? w[8 * l + i] : 1.0f);
          fb[i] *= inverse * (w != nullptr ? w[HALF + 8 * l + i] : 1.0f);
        }
      }
    }
    if (rotary_dim == DIM) {                            // a lane's two pieces are each other's partners
      if (treated) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float cosine = angles[8 * l + i], sine = angles[HALF + 8 * l + i];
          const float first = fa[i], second = fb[i];
          fa[i] = first * cosine - second * sine;
          fb[i] = first * sine + second * cosine;
        }
      }
    } else if (rotary_dim > 0) {                        // partners `reach` lanes apart, both in the first piece
      const bool low = l < reach, rotated = l < 2 * reach;
      const int partner = group * L + (low ? l + reach : max(l - reach, 0));
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float other = __shfl_sync(0xffffffffu, fa[i], partner);       // every lane takes part
        if (treated && rotated) {
          const int pair = 8 * (low ? l : l - reach) + i;
          const float cosine = angles[pair], sine = angles[pairs + pair];
          fa[i] = low ? fa[i] * cosine - other * sine : fa[i] * cosine + other * sine;
        }
      }
    }
    if (span == 1 && after) {                           // the norm behind the rotation
      float sum = 0.0f;
#pragma unroll
      for (int i = 0; i < 8; ++i) sum = fmaf(fa[i], fa[i], fmaf(fb[i], fb[i], sum));
#pragma unroll
      for (int o = L / 2; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
      const float inverse = rsqrtf(sum / (float)DIM + eps);
      if (treated) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          fa[i] *= inverse * (weight != nullptr ? weight[8 * l + i] : 1.0f);
          fb[i] *= inverse * (weight != nullptr ? weight[HALF + 8 * l + i] : 1.0f);
        }
      }
    }
    if (writes) {
    if (!is_value) {
      __nv_bfloat162* ha = reinterpret_cast<__nv_bfloat162*>(&a);
      __nv_bfloat162* hb = reinterpret_cast<__nv_bfloat162*>(&b);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        ha[i] = __floats2bfloat162_rn(fa[2 * i], fa[2 * i + 1]);
        hb[i] = __floats2bfloat162_rn(fb[2 * i], fb[2 * i + 1]);
      }
    }
    *reinterpret_cast<uint4*>(dst + 8 * l) = a;                // a value head is copied as it is
    *reinterpret_cast<uint4*>(dst + HALF + 8 * l) = b;
    }
    if (resident) break;
  }
}

// The most warps of a CTA that holds a token's heads in registers for the norm over a projection; wider tokens are
// summed in a pass of their own by CTAs of eight warps (more of which fit an SM).
int g_resident_warps = 16;

template <int L>
int launch_prepare_wide(__nv_bfloat16* qkv, long long row_stride, const int* positions, const int* slot_mapping,
                        const float* inv_freq, const float* q_weight, const float* k_weight, __nv_bfloat16* k_pages,
                        __nv_bfloat16* v_pages, int tokens, int heads, int kv_heads, int rotary_dim, float eps, int span,
                        int after, int write_kv, cudaStream_t stream) {
  const int units = write_kv == 1 ? heads + 2 * kv_heads : heads;
  // one CTA of 8 warps per token, or with few tokens CTAs of 4 warps that share a token's heads; the norm over a
  // projection sums the whole row before any of its heads is overwritten in place, so there a token stays in one CTA
  const bool many = tokens >= 256 || span == 2;
  int threads = many ? 256 : 128;
  const int units_per_cta = many ? units : 4 * (32 / L);
  // the norm over a projection: if the token's heads fit a CTA's warps at once, the pieces stay in registers between
  // the sum and the treatment
  const int warps_for_all = (units + 32 / L - 1) / (32 / L);
  const int resident = span == 2 && warps_for_all <= g_resident_warps;
  if (resident) threads = 32 * warps_for_all;
  const dim3 grid(tokens, (units + units_per_cta - 1) / units_per_cta);
  return mir_launch_with(mir_pdl_for_streaming(), "qk_prepare", qk_prepare_wide_kernel<L>, grid, dim3(threads), 0, stream, 0,
                         qkv, row_stride, positions, slot_mapping, inv_freq, q_weight, k_weight, k_pages, v_pages, heads,
                         kv_heads, rotary_dim, eps, span, after, write_kv, units_per_cta, resident);
}

}  // namespace

// For measurements: the limit described at g_resident_warps (0: always the pass of its own).
MIR_EXPORT int mir_qk_prepare_set_resident_warps(int warps) {
  if (warps < 0 || warps > 32) { mir_set_error("qk_prepare: 0 to 32 warps"); return MIR_BAD_ARGUMENT; }
  g_resident_warps = warps;
  return MIR_OK;
}

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
  const bool wide_rotation = rotary_dim == 0 || rotary_dim == head_dim || (rotary_dim % 16 == 0 && 2 * rotary_dim <= head_dim);
  if (bf16 && wide_rotation && value_dim == head_dim && head_dim % 16 == 0 && row_stride % 8 == 0 &&
      ((uintptr_t)qkv & 15) == 0 && ((uintptr_t)k_pages & 15) == 0 && ((uintptr_t)v_pages & 15) == 0) {
#define MIR_PREPARE_WIDE(L)                                                                                              \
  return launch_prepare_wide<L>((__nv_bfloat16*)qkv, row_stride, positions, slot_mapping, inv_freq, q_weight, k_weight, \
                                (__nv_bfloat16*)k_pages, (__nv_bfloat16*)v_pages, tokens, heads, kv_heads, rotary_dim,  \
                                eps, span, after, write_kv, stream)
    switch (head_dim / 16) {                             // lanes per head
      case 1: MIR_PREPARE_WIDE(1);
      case 2: MIR_PREPARE_WIDE(2);
      case 4: MIR_PREPARE_WIDE(4);
      case 8: MIR_PREPARE_WIDE(8);
      case 16: MIR_PREPARE_WIDE(16);
      default: break;                                    // other head sizes: the kernel below
    }
#undef MIR_PREPARE_WIDE
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
