// Paged grouped-query softmax attention, one code path for portions of prompts and for decoded
// tokens, any head size up to 640 (16-byte loads where it is a multiple of 8), any number of heads and groups,
// optional sliding window, float or bf16 storage.  One warp per (token, query head).
//
// This is the reference kernel of the engine: the 32-bit path always runs it, and the bf16 path
// runs it for the sizes its faster kernels refuse.  The order in which a query's keys are reduced
// depends only on the query's own position and window (32 keys at a time from the first visible
// key), never on how the step was cut or what else is in the batch, so a position's output is
// bit-identical under every work split.
//
// Replaces libmir's paged_attention_bf16.cu:14-93, paged_attention_batch_bf16.cu:14-102 and
// paged_prefill_attention_batch_bf16.cu:14-124: score = (q . k) * scale, running maximum and
// denominator, all in 32-bit; key j is visible to the query at position p iff j <= p and
// (window == 0 or j > p - window or j < keep_first): with a window, the first keep_first keys of a request stay
// visible to every later query (they keep their pages and their true positions).  Values may be narrower or wider
// than keys (value_dim).  A query walks over the kept keys first, then over its window.  Consecutive value rows
// lie value_row_width elements apart: value_dim in a cache of their own, head_dim where the values are the first
// value_dim elements of the keys themselves (a latent that is read both ways; v_pages is then k_pages).
// sinks (one 32-bit number per query head, or none): exp(sink - max) is added to the softmax's denominator once; it
// has no key and no value and is not scaled.  gate (rows of the activations' type with a stride of their own, or
// none): the head's result is multiplied by the sigmoid of its gate elements before it is stored; gate_per_head: a
// gate row holds one number per head instead of one per element.
// softcap > 0: score <- softcap * tanh(score / softcap) after the scale.  rel_bias ([heads, rel_rows] 32-bit, or none):
// the entry min(position - key, rel_rows - 1) of head h is added to the score after the cap (a bias by distance whose
// buckets the host has spread out into one row per distance; from the last row on it no longer changes).
#include <cfloat>
#include "common.cuh"

using namespace mir;

constexpr int kMaxHeadDim = 640;
constexpr int kWarpsPerBlock = 4;

template <typename T>
__global__ void paged_attention_generic_kernel(
    const T* __restrict__ q, size_t q_token_stride, T* __restrict__ out, const T* __restrict__ k_pages,
    const T* __restrict__ v_pages, const int* __restrict__ block_table, int table_width,
    const int* __restrict__ row_of_token, const int* __restrict__ positions, int page_size, int heads, int kv_heads,
    int head_dim, int value_dim, int value_row_width, float scale, int window, int keep_first,
    const float* __restrict__ sinks, const T* __restrict__ gate, size_t gate_stride, int gate_per_head, float softcap,
    const float* __restrict__ rel_bias, int rel_rows) {
  __shared__ float q_shared[kWarpsPerBlock][kMaxHeadDim];
  const int lane = threadIdx.x;
  const int warp = threadIdx.y;
  const int head = blockIdx.y * kWarpsPerBlock + warp;
  const int token = blockIdx.x;
  if (head >= heads) return;
  const int row = row_of_token[token];
  const int position = positions[token];
  const int kv_head = head / (heads / kv_heads);
  const int* table = block_table + (size_t)row * table_width;
  const int first_key = (window > 0 && position + 1 > window) ? position + 1 - window : 0;

  const T* q_row = q + (size_t)token * q_token_stride + (size_t)head * head_dim;
  for (int d = lane; d < head_dim; d += 32) q_shared[warp][d] = to_float(q_row[d]);
  __syncwarp();

  float acc[kMaxHeadDim / 32];
#pragma unroll
  for (int i = 0; i < kMaxHeadDim / 32; ++i) acc[i] = 0.0f;
  float running_max = -FLT_MAX;
  float denominator = 0.0f;

  // the kept first keys that lie before the window, then the window: [0, kept) and [first_key, position]
  const int kept = min(keep_first, first_key);
  const int kept_chunks = (kept + 31) / 32;
  const int chunks = kept_chunks + (position - first_key) / 32 + 1;
  for (int chunk = 0; chunk < chunks; ++chunk) {
    const bool in_kept = chunk < kept_chunks;
    const int base = in_kept ? chunk * 32 : first_key + (chunk - kept_chunks) * 32;
    const int last = in_kept ? kept - 1 : position;
    const int key = base + lane;
    const bool valid = key <= last;
    float score = -FLT_MAX;
    size_t key_offset = 0;
    if (valid) {
      const int page = table[key / page_size];
      key_offset = ((size_t)page * page_size + key % page_size) * kv_heads + kv_head;
      const T* k_row = k_pages + key_offset * head_dim;
      float dot = 0.0f;
      if (head_dim % 8 == 0) {                                // (then every key row starts on a 16-byte boundary)
        for (int d = 0; d < head_dim; d += 8) {
          float k8[8];
          load8(k_row + d, k8);
#pragma unroll
          for (int i = 0; i < 8; ++i) dot = fmaf(q_shared[warp][d + i], k8[i], dot);
        }
      } else {
        for (int d = 0; d < head_dim; ++d) dot = fmaf(q_shared[warp][d], to_float(k_row[d]), dot);
      }
      score = dot * scale;
      if (softcap > 0.0f) score = softcap * tanhf(score / softcap);
      if (rel_bias != nullptr) score += rel_bias[(size_t)head * rel_rows + min(position - key, rel_rows - 1)];
    }
    const float next_max = fmaxf(running_max, warp_max(score));
    const float correction = expf(running_max - next_max);
    const float weight = valid ? expf(score - next_max) : 0.0f;
    denominator = denominator * correction + warp_sum(weight);
#pragma unroll
    for (int i = 0; i < kMaxHeadDim / 32; ++i) acc[i] *= correction;
    const int keys_here = min(32, last - base + 1);
    for (int j = 0; j < keys_here; ++j) {
      const float w = __shfl_sync(0xffffffffu, weight, j);
      const size_t offset = __shfl_sync(0xffffffffu, key_offset, j);
      const T* v_row = v_pages + offset * value_row_width;
#pragma unroll
      for (int i = 0; i < kMaxHeadDim / 32; ++i) {
        const int d = lane + 32 * i;
        if (d < value_dim) acc[i] = fmaf(w, to_float(v_row[d]), acc[i]);
      }
    }
    running_max = next_max;
  }

  if (sinks != nullptr && position >= 0) {
    const float sink = sinks[head];
    const float next_max = fmaxf(running_max, sink);
    const float correction = expf(running_max - next_max);
    denominator = denominator * correction + expf(sink - next_max);
#pragma unroll
    for (int i = 0; i < kMaxHeadDim / 32; ++i) acc[i] *= correction;
  }
  T* out_row = out + ((size_t)token * heads + head) * value_dim;
  const T* gate_row = gate != nullptr ? gate + (size_t)token * gate_stride + (size_t)head * (gate_per_head ? 1 : value_dim)
                                      : nullptr;
  const float inverse = denominator > 0.0f ? 1.0f / denominator : 0.0f;   // a padded row has no keys
#pragma unroll
  for (int i = 0; i < kMaxHeadDim / 32; ++i) {
    const int d = lane + 32 * i;
    if (d < value_dim) {
      float result = acc[i] * inverse;
      if (gate_row != nullptr) result *= 1.0f / (1.0f + expf(-to_float(gate_row[gate_per_head ? 0 : d])));
      out_row[d] = from_float<T>(result);
    }
  }
}

// q: first query element of token 0; q_token_stride in elements (the packed QKV row width).
MIR_EXPORT int mir_paged_attention_generic(int bf16, const void* q, long long q_token_stride, void* out,
                                           const void* k_pages, const void* v_pages, const int* block_table,
                                           int table_width, const int* row_of_token, const int* positions, int tokens,
                                           int page_size, int heads, int kv_heads, int head_dim, int value_dim,
                                           float scale, int window, int keep_first, int value_row_width,
                                           const float* sinks, const void* gate, long long gate_stride,
                                           int gate_per_head, float softcap, const float* rel_bias, int rel_rows,
                                           cudaStream_t stream) {
  if (tokens == 0) return MIR_OK;
  if (tokens < 0 || heads <= 0 || kv_heads <= 0 || heads % kv_heads || page_size <= 0 || table_width <= 0 ||
      window < 0 || keep_first < 0) {
    mir_set_error("paged_attention: bad sizes (tokens %d, heads %d, kv heads %d, page %d, table width %d)", tokens,
                  heads, kv_heads, page_size, table_width);
    return MIR_BAD_ARGUMENT;
  }
  if (head_dim <= 0 || head_dim > kMaxHeadDim) {
    mir_set_error("paged_attention: head_dim %d is not in [1, %d]", head_dim, kMaxHeadDim);
    return MIR_BAD_ARGUMENT;
  }
  if (value_dim <= 0 || value_dim > kMaxHeadDim) {
    mir_set_error("paged_attention: value_dim %d is not in [1, %d]", value_dim, kMaxHeadDim);
    return MIR_BAD_ARGUMENT;
  }
  if (value_row_width <= 0) value_row_width = value_dim;
  if (rel_bias != nullptr && rel_rows <= 0) { mir_set_error("paged_attention: a bias by distance needs rows"); return MIR_BAD_ARGUMENT; }
  const dim3 grid(tokens, (heads + kWarpsPerBlock - 1) / kWarpsPerBlock);
  const dim3 block(32, kWarpsPerBlock);
  if (bf16)
    paged_attention_generic_kernel<<<grid, block, 0, stream>>>(
        (const __nv_bfloat16*)q, (size_t)q_token_stride, (__nv_bfloat16*)out, (const __nv_bfloat16*)k_pages,
        (const __nv_bfloat16*)v_pages, block_table, table_width, row_of_token, positions, page_size, heads, kv_heads,
        head_dim, value_dim, value_row_width, scale, window, keep_first, sinks, (const __nv_bfloat16*)gate,
        (size_t)gate_stride, gate_per_head, softcap, rel_bias, rel_rows);
  else
    paged_attention_generic_kernel<<<grid, block, 0, stream>>>(
        (const float*)q, (size_t)q_token_stride, (float*)out, (const float*)k_pages, (const float*)v_pages,
        block_table, table_width, row_of_token, positions, page_size, heads, kv_heads, head_dim, value_dim,
        value_row_width, scale, window, keep_first, sinks, (const float*)gate, (size_t)gate_stride, gate_per_head, softcap,
        rel_bias, rel_rows);
  return mir_check_launch("paged_attention_generic");
}
