// Kernels of a mixture of gated experts.  P = tokens * top pairs of (token, chosen expert); pair p = token * top + slot.
//
//   moe_route     per token, from the router's 32-bit logits (a product of the framework): sigmoid scores (or a softmax
//                 over all experts), choice among the experts of the best groups by score + correction (a group judged
//                 by the sum of its two largest choice scores, or by its largest), weights = chosen scores / their sum
//                 * scale; and the shared expert's gate.  The last experts of the router may be identity experts, which
//                 have no weights: the sort leaves their pairs out, and moe_combine adds weight * the token's own input
//   moe_sort      the pairs ordered by expert (a stable counting sort: a CTA per expert counts, one CTA scans, a CTA
//                 per expert places), each expert's range, and the list of tiles (8 or 128 pairs of one expert)
//                 that the grouped products walk over
//   moe_grouped   products on the sorted pairs with each pair's own expert's weights: hidden = silu(Wg x) * (Wu x)
//                 from the tokens' rows, and the down projection of the hidden rows into one 32-bit row per pair, as
//                 32-bit multiply-adds on tiles of 8 pairs (any type and size).  bfloat16 rows of 16-byte pieces run
//                 the tcgen05 product of csrc/gemm_tc.cu instead, on tiles of 128 pairs of this file's list, after
//                 moe_gather_rows has brought the tokens' rows into the pairs' order
//   moe_combine   residual[t] += sum over slots of weight * the pair's row (+ gate * the shared expert's row)
// Everything the host needs to launch them is known before the step: no count is read back.
#include <cfloat>
#include "common.cuh"

using namespace mir;

namespace {

constexpr int kExpertTile = 8;        // pairs of one expert that a CTA of the grouped product takes
constexpr int kTensorTile = 128;      // rows of a tile of the tcgen05 grouped product (csrc/gemm_tc.cu)
constexpr int kMaxExperts = 1024;

__device__ __forceinline__ float sigmoid_of(float z) { return 1.0f / (1.0f + expf(-z)); }

// One warp per token, four tokens a CTA.  logits [tokens, >= experts (+ 1)] 32-bit: the router's logits and, behind
// them, the shared expert's gate logit (has_gate).  Shared memory per warp: score[E] | choice[E] | group score[groups].
// Among equal scores the expert (or group) with the lower index wins.
constexpr int kRouteWarps = 4;

__device__ __forceinline__ void warp_best(float& value, int& index, bool want_max) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float other = __shfl_xor_sync(0xffffffffu, value, o);
    const int other_index = __shfl_xor_sync(0xffffffffu, index, o);
    const bool better = want_max ? (other > value || (other == value && other_index < index))
                                 : (other < value || (other == value && other_index > index));
    if (other_index >= 0 && (index < 0 || better)) { value = other; index = other_index; }
  }
}

__global__ void moe_route_kernel(const float* __restrict__ logits, long long ld, const float* __restrict__ correction,
                                 int has_gate, int* __restrict__ ids, float* __restrict__ weights,
                                 float* __restrict__ shared_gate, int tokens, int experts, int top, int groups, int keep,
                                 float scale, int softmax_scores, int group_by_max) {
  extern __shared__ float route_shared[];
  grid_launch_dependents();
  grid_dependency_wait();
  const int lane = threadIdx.x, warp = threadIdx.y;
  const int token = blockIdx.x * kRouteWarps + warp;
  if (token >= tokens) return;
  float* score = route_shared + (size_t)warp * (2 * experts + groups);
  float* choice = score + experts;
  float* group_score = choice + experts;
  const float* z = logits + (size_t)token * ld;
  float softmax_top = 0.0f, softmax_inverse = 1.0f;
  if (softmax_scores) {                                          // over all the router's experts, in 32-bit
    float high = -FLT_MAX;
    for (int e = lane; e < experts; e += 32) high = fmaxf(high, z[e]);
    softmax_top = warp_max(high);
    float sum = 0.0f;
    for (int e = lane; e < experts; e += 32) sum += expf(z[e] - softmax_top);
    softmax_inverse = 1.0f / warp_sum(sum);
  }
  for (int e = lane; e < experts; e += 32) {
    const float s = softmax_scores ? expf(z[e] - softmax_top) * softmax_inverse : sigmoid_of(z[e]);
    score[e] = s;
    choice[e] = correction != nullptr ? s + correction[e] : s;
  }
  if (has_gate && lane == 0) shared_gate[token] = sigmoid_of(z[experts]);
  __syncwarp();
  const int per_group = experts / groups;
  if (keep < groups) {
    // a group's score: the sum of its two largest choice scores (of its one score where a group is one expert)
    for (int g = lane; g < groups; g += 32) {
      float first = -FLT_MAX, second = -FLT_MAX;
      for (int e = g * per_group; e < (g + 1) * per_group; ++e) {
        const float c = choice[e];
        if (c > first) { second = first; first = c; }
        else if (c > second) second = c;
      }
      group_score[g] = (per_group > 1 && !group_by_max) ? first + second : first;
    }
    __syncwarp();
    // experts of all but the `keep` best groups cannot be chosen: their choice scores count as minus infinity
    for (int round = 0; round < groups - keep; ++round) {
      float low = FLT_MAX;
      int worst = -1;
      for (int g = lane; g < groups; g += 32) {
        const float v = group_score[g];
        if (v != FLT_MAX && (worst < 0 || v <= low)) { low = v; worst = g; }     // (among equals the later group goes)
      }
      warp_best(low, worst, false);
      if (worst < 0) break;
      if (lane == 0) group_score[worst] = FLT_MAX;                // marked as dropped
      for (int e = worst * per_group + lane; e < (worst + 1) * per_group; e += 32) choice[e] = -FLT_MAX;
      __syncwarp();
    }
  }
  float total = 0.0f;
  for (int slot = 0; slot < top; ++slot) {
    float high = -FLT_MAX;
    int best = -1;
    for (int e = lane; e < experts; e += 32) {
      const float c = choice[e];
      if (c > high) { high = c; best = e; }
    }
    if (best >= 0 && high == -FLT_MAX) best = -1;
    warp_best(high, best, true);
    if (best < 0) best = 0;                                      // (fewer choosable experts than top: not a valid model)
    if (lane == 0) {
      choice[best] = -FLT_MAX;
      ids[(size_t)token * top + slot] = best;
      weights[(size_t)token * top + slot] = score[best];
    }
    total += score[best];
    __syncwarp();
  }
  const float factor = scale / (total + 1e-20f);
  for (int slot = lane; slot < top; slot += 32) weights[(size_t)token * top + slot] *= factor;
}

// The pairs ordered by expert, in three small kernels.  order[i] = the i-th pair when the pairs are sorted by expert
// (pairs of one expert stay in their own order); offsets[e] .. offsets[e + 1] is expert e's range in it; tiles[2 n],
// tiles[2 n + 1] = expert and first sorted pair of the n-th tile of tile_pairs pairs, tile_count[0] = how many there are.
constexpr int kSortThreads = 256;

// One CTA per expert: how many pairs chose it.
__global__ void moe_count_kernel(const int* __restrict__ ids, int pairs, int* __restrict__ counts) {
  __shared__ float scratch[32];
  grid_launch_dependents();
  grid_dependency_wait();
  const int expert = blockIdx.x;
  int n = 0;
  for (int p = threadIdx.x; p < pairs; p += blockDim.x) n += ids[p] == expert;
  const float total = block_sum((float)n, scratch);              // (exact: fewer than 2^24 pairs)
  if (threadIdx.x == 0) counts[expert] = (int)(total + 0.5f);
}

// One CTA: the experts' ranges and first tiles (an exclusive scan over at most kMaxExperts counts).
__global__ void moe_offsets_kernel(const int* __restrict__ counts, int experts, int tile_pairs, int* __restrict__ offsets,
                                   int* __restrict__ first_tile, int* __restrict__ tile_count) {
  __shared__ int pair_sums[32], tile_sums[32];
  grid_launch_dependents();
  grid_dependency_wait();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;    // 1024 threads: one expert each
  const int e = threadIdx.x;
  const int mine = e < experts ? counts[e] : 0;
  const int my_tiles = (mine + tile_pairs - 1) / tile_pairs;
  int pair_scan = mine, tile_scan = my_tiles;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int a = __shfl_up_sync(0xffffffffu, pair_scan, o), t = __shfl_up_sync(0xffffffffu, tile_scan, o);
    if (lane >= o) { pair_scan += a; tile_scan += t; }
  }
  if (lane == 31) { pair_sums[warp] = pair_scan; tile_sums[warp] = tile_scan; }
  __syncthreads();
  if (warp == 0) {
    int a = pair_sums[lane], t = tile_sums[lane];
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int x = __shfl_up_sync(0xffffffffu, a, o), y = __shfl_up_sync(0xffffffffu, t, o);
      if (lane >= o) { a += x; t += y; }
    }
    pair_sums[lane] = a;
    tile_sums[lane] = t;
  }
  __syncthreads();
  const int pair_base = (warp ? pair_sums[warp - 1] : 0) + pair_scan - mine;
  const int tile_base = (warp ? tile_sums[warp - 1] : 0) + tile_scan - my_tiles;
  if (e < experts) {
    offsets[e] = pair_base;
    first_tile[e] = tile_base;
  }
  if (e == experts - 1) {
    offsets[experts] = pair_base + mine;
    tile_count[0] = tile_base + my_tiles;
  }
}

// One CTA per expert: its pairs into their places, in their own order, and its tiles.
__global__ void moe_place_kernel(const int* __restrict__ ids, int pairs, int tile_pairs, const int* __restrict__ offsets,
                                 const int* __restrict__ first_tile, int* __restrict__ order, int* __restrict__ tiles) {
  __shared__ int warp_counts[kSortThreads / 32];
  grid_launch_dependents();
  grid_dependency_wait();
  const int expert = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int begin = offsets[expert], total = offsets[expert + 1] - begin;
  const int n = (total + tile_pairs - 1) / tile_pairs;
  for (int t = threadIdx.x; t < n; t += kSortThreads) {
    tiles[2 * (first_tile[expert] + t)] = expert;
    tiles[2 * (first_tile[expert] + t) + 1] = begin + t * tile_pairs;
  }
  int placed = 0;
  for (int base = 0; base < pairs && placed < total; base += kSortThreads) {      // (placed is the same for every thread)
    const int p = base + threadIdx.x;
    const bool mine = p < pairs && ids[p] == expert;
    const unsigned ballot = __ballot_sync(0xffffffffu, mine);
    if (lane == 0) warp_counts[warp] = __popc(ballot);
    __syncthreads();
    int before = 0, all = 0;
#pragma unroll
    for (int w = 0; w < kSortThreads / 32; ++w) {
      const int c = warp_counts[w];
      if (w < warp) before += c;
      all += c;
    }
    if (mine) order[begin + placed + before + __popc(ballot & ((1u << lane) - 1u))] = p;
    placed += all;
    __syncthreads();
  }
}

__device__ __forceinline__ void load4(const float* p, float (&out)[4]) {
  const float4 a = *reinterpret_cast<const float4*>(p);
  out[0] = a.x; out[1] = a.y; out[2] = a.z; out[3] = a.w;
}
__device__ __forceinline__ void load4(const __nv_bfloat16* p, float (&out)[4]) {
  const uint2 raw = *reinterpret_cast<const uint2*>(p);
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
  const float2 a = __bfloat1622float2(h[0]), b = __bfloat1622float2(h[1]);
  out[0] = a.x; out[1] = a.y; out[2] = b.x; out[3] = b.y;
}

constexpr int kGroupedWarps = 8;
constexpr int kGroupedPerWarp = 4;                               // outputs a warp computes for the tile's pairs
constexpr int kGroupedChunk = 512;                               // inputs staged at a time

// blockDim (32, kGroupedWarps); grid (tile slots, ceil(N / 32)).  The rows of a tile's pairs are staged in shared
// memory 512 inputs at a time; a warp walks over a weight row with its lanes side by side (4 inputs a lane) and keeps
// one sum per pair.  Every output is the same chain of partial sums and the same tree over the lanes whatever the
// batch holds.  x row of sorted pair i: gather == null ? i : gather[i] / gather_div; out row: scatter == null ? i :
// scatter[i].  GATED: out = silu(w_a x) * (w_b x), else out = w_a x.
template <typename T, typename TO, bool GATED>
__global__ void __launch_bounds__(kGroupedWarps * 32)
moe_grouped_kernel(const T* __restrict__ x, long long ldx, const int* __restrict__ gather, int gather_div,
                   const T* __restrict__ w_a, const T* __restrict__ w_b, TO* __restrict__ out, long long ldo,
                   const int* __restrict__ scatter, const int* __restrict__ tiles, const int* __restrict__ tile_count,
                   const int* __restrict__ offsets, int K, int N) {
  __shared__ __align__(16) float rows[kExpertTile][kGroupedChunk];
  __shared__ int source[kExpertTile];
  grid_launch_dependents();
  grid_dependency_wait();
  if ((int)blockIdx.x >= tile_count[0]) return;
  const int lane = threadIdx.x, warp = threadIdx.y, thread = warp * 32 + lane;
  const int expert = tiles[2 * blockIdx.x], start = tiles[2 * blockIdx.x + 1];
  const int count = min(kExpertTile, offsets[expert + 1] - start);
  if (thread < kExpertTile)
    source[thread] = thread < count ? (gather != nullptr ? gather[start + thread] / gather_div : start + thread) : -1;
  const int first_output = blockIdx.y * (kGroupedWarps * kGroupedPerWarp) + warp * kGroupedPerWarp;
  float acc_a[kGroupedPerWarp][kExpertTile], acc_b[GATED ? kGroupedPerWarp : 1][kExpertTile];
#pragma unroll
  for (int j = 0; j < kGroupedPerWarp; ++j)
#pragma unroll
    for (int r = 0; r < kExpertTile; ++r) {
      acc_a[j][r] = 0.0f;
      if (GATED) acc_b[j][r] = 0.0f;
    }
  const bool wide = K % 4 == 0;
  for (int from = 0; from < K; from += kGroupedChunk) {
    const int here = min(kGroupedChunk, K - from);
    __syncthreads();
    for (int index = thread; index < kExpertTile * here; index += kGroupedWarps * 32) {
      const int r = index / here, i = index - r * here;
      rows[r][i] = source[r] >= 0 ? to_float(x[(size_t)source[r] * ldx + from + i]) : 0.0f;
    }
    __syncthreads();
#pragma unroll
    for (int j = 0; j < kGroupedPerWarp; ++j) {
      const int o = first_output + j;
      if (o >= N) break;
      const T* row_a = w_a + ((size_t)expert * N + o) * K + from;
      const T* row_b = GATED ? w_b + ((size_t)expert * N + o) * K + from : nullptr;
      if (wide) {
        for (int i = lane * 4; i < here; i += 128) {
          float a[4], b[4];
          load4(row_a + i, a);
          if (GATED) load4(row_b + i, b);
#pragma unroll
          for (int r = 0; r < kExpertTile; ++r) {
            const float4 v = *reinterpret_cast<const float4*>(&rows[r][i]);
            acc_a[j][r] = fmaf(a[3], v.w, fmaf(a[2], v.z, fmaf(a[1], v.y, fmaf(a[0], v.x, acc_a[j][r]))));
            if (GATED) acc_b[j][r] = fmaf(b[3], v.w, fmaf(b[2], v.z, fmaf(b[1], v.y, fmaf(b[0], v.x, acc_b[j][r]))));
          }
        }
      } else {
        for (int i = lane; i < here; i += 32) {
          const float a = to_float(row_a[i]);
          const float b = GATED ? to_float(row_b[i]) : 0.0f;
#pragma unroll
          for (int r = 0; r < kExpertTile; ++r) {
            acc_a[j][r] = fmaf(a, rows[r][i], acc_a[j][r]);
            if (GATED) acc_b[j][r] = fmaf(b, rows[r][i], acc_b[j][r]);
          }
        }
      }
    }
  }
#pragma unroll
  for (int j = 0; j < kGroupedPerWarp; ++j) {
    const int o = first_output + j;
#pragma unroll
    for (int r = 0; r < kExpertTile; ++r) {
      const float a = warp_sum(acc_a[j][r]);
      const float b = GATED ? warp_sum(acc_b[j][r]) : 0.0f;
      if (lane == r && r < count && o < N) {
        const int to = scatter != nullptr ? scatter[start + r] : start + r;
        const float value = GATED ? a / (1.0f + expf(-a)) * b : a;
        out[(size_t)to * ldo + o] = from_float<TO>(value);
      }
    }
  }
}

// One CTA per token: residual[t] += sum_s weights[t, s] * pair_rows[t * top + s] (+ shared_gate[t] * shared_rows[t], or
// + shared_rows[t] without a gate), slots in their own order.  A slot whose expert is an identity expert (ids[pair] >=
// real_experts) has no row: it adds weight * the token's own input (identity_rows, in the activations' type).
// overwrite: the sum replaces residual[t] instead of being added to it.
// A thread takes V neighbouring columns of one token (V = 4 where rows and pointers allow 16-byte accesses), a CTA a
// run of columns (blockIdx.y): few tokens still fill the GPU.  A column's sum runs over the slots in ascending order,
// then the shared expert, whatever V is.
template <typename T, int V>
__global__ void moe_combine_kernel(float* __restrict__ residual, const float* __restrict__ pair_rows,
                                   const float* __restrict__ weights, const float* __restrict__ shared_rows,
                                   const float* __restrict__ shared_gate, int width, int top, int overwrite,
                                   const int* __restrict__ ids, int real_experts, const T* __restrict__ identity_rows,
                                   long long identity_stride) {
  grid_launch_dependents();
  grid_dependency_wait();
  const int token = blockIdx.x;
  const int c = (blockIdx.y * blockDim.x + threadIdx.x) * V;
  if (c >= width) return;
  float total[V];
#pragma unroll
  for (int v = 0; v < V; ++v) total[v] = 0.0f;
  for (int s = 0; s < top; ++s) {
    const size_t pair = (size_t)token * top + s;
    const float weight = __ldg(weights + pair);
    alignas(16) float row[V];
    if (ids != nullptr && __ldg(ids + pair) >= real_experts) {
      const T* src = identity_rows + (size_t)token * identity_stride + c;
#pragma unroll
      for (int v = 0; v < V; ++v) row[v] = to_float(src[v]);
    } else if (V == 4) {
      *reinterpret_cast<float4*>(row) = *reinterpret_cast<const float4*>(pair_rows + pair * width + c);
    } else {
      row[0] = pair_rows[pair * width + c];
    }
#pragma unroll
    for (int v = 0; v < V; ++v) total[v] = fmaf(weight, row[v], total[v]);
  }
  const size_t at = (size_t)token * width + c;
  if (shared_rows != nullptr) {
    const float gate = shared_gate != nullptr ? shared_gate[token] : 1.0f;
#pragma unroll
    for (int v = 0; v < V; ++v) total[v] = fmaf(gate, shared_rows[at + v], total[v]);
  }
#pragma unroll
  for (int v = 0; v < V; ++v) residual[at + v] = overwrite ? total[v] : residual[at + v] + total[v];
}

template <typename T, typename TO, bool GATED>
int launch_grouped(cudaStream_t stream, const void* x, long long ldx, const int* gather, int gather_div, const void* w_a,
                   const void* w_b, void* out, long long ldo, const int* scatter, const int* tiles, const int* tile_count,
                   const int* offsets, int pairs, int experts, int K, int N) {
  const int slots = pairs / kExpertTile + experts;               // no more tiles than this, whatever the routing
  const dim3 grid(slots, (N + kGroupedWarps * kGroupedPerWarp - 1) / (kGroupedWarps * kGroupedPerWarp));
  return mir_launch(GATED ? "moe_grouped_gate_up" : "moe_grouped_down", moe_grouped_kernel<T, TO, GATED>, grid,
                    dim3(32, kGroupedWarps), 0, stream, 0, (const T*)x, ldx, gather, gather_div, (const T*)w_a,
                    (const T*)w_b, (TO*)out, ldo, scatter, tiles, tile_count, offsets, K, N);
}

}  // namespace

// logits [tokens, >= experts + has_gate] 32-bit with row stride ld: the router's logits (and the shared expert's gate
// logit behind them); correction [experts] (or null) 32-bit; ids, weights [tokens, top]; shared_gate [tokens].
MIR_EXPORT int mir_moe_route(const float* logits, long long ld, const float* correction, int has_gate, int* ids,
                             float* weights, float* shared_gate, int tokens, int experts, int top, int groups, int keep,
                             float scale, int softmax_scores, int group_by_max, cudaStream_t stream) {
  if (tokens == 0) return MIR_OK;
  if (tokens < 0 || experts <= 0 || experts > kMaxExperts || top <= 0 || top > experts || groups <= 0 ||
      experts % groups || keep <= 0 || keep > groups || (long long)keep * (experts / groups) < top ||
      (has_gate && shared_gate == nullptr)) {
    mir_set_error("moe_route: bad sizes (tokens %d, experts %d, top %d, groups %d of which %d are kept)", tokens, experts,
                  top, groups, keep);
    return MIR_BAD_ARGUMENT;
  }
  const size_t smem = (size_t)kRouteWarps * (2 * experts + groups) * sizeof(float);
  return mir_launch("moe_route", moe_route_kernel, dim3((tokens + kRouteWarps - 1) / kRouteWarps), dim3(32, kRouteWarps),
                    smem, stream, 0, logits, ld, correction, has_gate, ids, weights, shared_gate, tokens, experts, top,
                    groups, keep, scale, softmax_scores, group_by_max);
}

// How many tiles of tile_pairs pairs there can be at most for `pairs` pairs over `experts` experts (`tiles` holds two
// ints for each).
MIR_EXPORT int mir_moe_tile_slots(int pairs, int experts, int tile_pairs) { return pairs / tile_pairs + experts; }

// tile_pairs: 8 for the 32-bit grouped products of this file, 128 for the tcgen05 product (csrc/gemm_tc.cu).
// counts, first_tile: scratch of `experts` ints each.
MIR_EXPORT int mir_moe_sort(const int* ids, int pairs, int experts, int tile_pairs, int* order, int* offsets, int* tiles,
                            int* tile_count, int* counts, int* first_tile, cudaStream_t stream) {
  if (pairs == 0) return MIR_OK;
  if (pairs < 0 || experts <= 0 || experts > kMaxExperts ||
      (tile_pairs != kExpertTile && tile_pairs != kTensorTile)) {
    mir_set_error("moe_sort: bad sizes (pairs %d, experts %d, tiles of %d)", pairs, experts, tile_pairs);
    return MIR_BAD_ARGUMENT;
  }
  int status = mir_launch("moe_count", moe_count_kernel, dim3(experts), dim3(kSortThreads), 0, stream, 0, ids, pairs, counts);
  if (status != MIR_OK) return status;
  status = mir_launch("moe_offsets", moe_offsets_kernel, dim3(1), dim3(kMaxExperts), 0, stream, 0, counts, experts,
                      tile_pairs, offsets, first_tile, tile_count);
  if (status != MIR_OK) return status;
  return mir_launch("moe_place", moe_place_kernel, dim3(experts), dim3(kSortThreads), 0, stream, 0, ids, pairs, tile_pairs,
                    offsets, first_tile, order, tiles);
}

// hidden[i] = silu(w_gate[e] x) * (w_up[e] x) for the i-th sorted pair, x the row of its token (order[i] / top) of h.
// w_gate, w_up [experts, inter, width]; hidden [pairs, inter] in the activations' type.
MIR_EXPORT int mir_moe_gate_up(int bf16, const void* h, long long ld, const int* order, int top, const void* w_gate,
                               const void* w_up, void* hidden, const int* tiles, const int* tile_count,
                               const int* offsets, int pairs, int experts, int width, int inter, int tile_pairs,
                               cudaStream_t stream) {
  if (pairs == 0) return MIR_OK;
  if (tile_pairs != kExpertTile) { mir_set_error("moe_gate_up: this kernel works on tiles of %d pairs", kExpertTile); return MIR_BAD_ARGUMENT; }
  if (bf16)
    return launch_grouped<__nv_bfloat16, __nv_bfloat16, true>(stream, h, ld, order, top, w_gate, w_up, hidden, inter,
                                                              nullptr, tiles, tile_count, offsets, pairs, experts, width,
                                                              inter);
  return launch_grouped<float, float, true>(stream, h, ld, order, top, w_gate, w_up, hidden, inter, nullptr, tiles,
                                            tile_count, offsets, pairs, experts, width, inter);
}

// pair_rows[order[i]] = w_down[e] hidden[i]: one 32-bit row [width] per pair, at the pair's own index.
MIR_EXPORT int mir_moe_down(int bf16, const void* hidden, const int* order, const void* w_down, float* pair_rows,
                            const int* tiles, const int* tile_count, const int* offsets, int pairs, int experts,
                            int width, int inter, int tile_pairs, cudaStream_t stream) {
  if (pairs == 0) return MIR_OK;
  if (tile_pairs != kExpertTile) { mir_set_error("moe_down: this kernel works on tiles of %d pairs", kExpertTile); return MIR_BAD_ARGUMENT; }
  if (bf16)
    return launch_grouped<__nv_bfloat16, float, false>(stream, hidden, inter, nullptr, 1, w_down, nullptr, pair_rows,
                                                       width, order, tiles, tile_count, offsets, pairs, experts, inter,
                                                       width);
  return launch_grouped<float, float, false>(stream, hidden, inter, nullptr, 1, w_down, nullptr, pair_rows, width, order,
                                             tiles, tile_count, offsets, pairs, experts, inter, width);
}

// sorted[i, :] = h[order[i] / top, :]: the tokens' rows in the order of the sorted pairs (16-byte pieces).
__global__ void moe_gather_rows_kernel(const uint4* __restrict__ h, long long ld_pieces, const int* __restrict__ order, int top,
                                       uint4* __restrict__ sorted, int pieces, size_t total,
                                       const int* __restrict__ sorted_count) {
  grid_launch_dependents();
  grid_dependency_wait();
  const size_t index = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (index >= total) return;
  const size_t row = index / pieces;
  if (sorted_count != nullptr && row >= (size_t)sorted_count[0]) return;     // (pairs of identity experts are in no order)
  const int piece = (int)(index - row * pieces);
  sorted[index] = h[(size_t)(order[row] / top) * ld_pieces + piece];
}

// h [tokens, width] bfloat16 (row stride ld, both multiples of 8); sorted [pairs, width].  sorted_count (or null): one
// number on the device, how many of the pairs the order holds (the pairs of identity experts are left out of it).
MIR_EXPORT int mir_moe_gather_rows(const void* h, long long ld, const int* order, int top, void* sorted, int pairs,
                                   int width, const int* sorted_count, cudaStream_t stream) {
  if (pairs == 0) return MIR_OK;
  if (pairs < 0 || width <= 0 || width % 8 || ld % 8 || top <= 0) {
    mir_set_error("moe_gather_rows: rows of 16-byte pieces are needed (width %d, stride %lld)", width, ld);
    return MIR_BAD_ARGUMENT;
  }
  const int pieces = width / 8;
  const size_t total = (size_t)pairs * pieces;
  return mir_launch("moe_gather_rows", moe_gather_rows_kernel, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, stream, 0,
                    (const uint4*)h, ld / 8, order, top, (uint4*)sorted, pieces, total, sorted_count);
}

MIR_EXPORT int mir_moe_combine(float* residual, const float* pair_rows, const float* weights, const float* shared_rows,
                               const float* shared_gate, int tokens, int width, int top, int overwrite, const int* ids,
                               int real_experts, int bf16, const void* identity_rows, long long identity_stride,
                               cudaStream_t stream) {
  if (tokens == 0) return MIR_OK;
  if (ids != nullptr && identity_rows == nullptr) {
    mir_set_error("moe_combine: identity experts need the tokens' input rows");
    return MIR_BAD_ARGUMENT;
  }
  const bool wide = width % 4 == 0 && ((uintptr_t)pair_rows & 15) == 0;
  const int per_thread = wide ? 4 : 1;
  const int threads = width >= 1024 * per_thread ? 256 : 128;
  const dim3 grid(tokens, (width + threads * per_thread - 1) / (threads * per_thread));
#define MIR_COMBINE(T, V)                                                                                             \
  return mir_launch("moe_combine", moe_combine_kernel<T, V>, grid, dim3(threads), 0, stream, 0, residual, pair_rows,   \
                    weights, shared_rows, shared_gate, width, top, overwrite, ids, real_experts, (const T*)identity_rows, \
                    identity_stride)
  if (bf16) {
    if (wide) MIR_COMBINE(__nv_bfloat16, 4);
    MIR_COMBINE(__nv_bfloat16, 1);
  }
  if (wide) MIR_COMBINE(float, 4);
  MIR_COMBINE(float, 1);
#undef MIR_COMBINE
}
