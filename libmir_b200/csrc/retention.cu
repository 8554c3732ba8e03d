// The recurrence of the retention mixer: linear attention with one fixed decay per head and no softmax.
//
//   per head, S [key channel, value channel] (stored per value channel, a column contiguous):
//     S_t = d S_t-1 + k_t v_t^T;   o_t = S_t^T q_t = d (S_t-1^T q_t) + (q_t . k_t) v_t
//   q and k are the projections' results rotated by the token's position (half-split pairs i, i + r/2 of the first r
//   channels; angle = position * inv_freq[i], a 32-bit product), k also times key_scale, both in 32-bit while a chunk
//   of tokens is staged in shared memory: nothing rotated is ever rounded to the storage type.
// The decay, the rotation, the state and every sum are 32-bit; T is the storage type of the projections' results.
// One lane count and one order of sums for every shape of step: a request's 32-bit results do not depend on how it was
// cut into steps.  A row of a captured decode batch whose position is negative is padding: nothing is read or written.
#include "common.cuh"

using namespace mir;

namespace {

constexpr int kWarps = 4;

// A token's q and k of one head, staged by one warp.  Lane `lane` owns the channels i = lane + 32 e.  A channel of the
// first half of the rotated ones is rotated together with its partner i + half by the lane that owns it (one sine and
// cosine for the pair, for q and k alike); the partner's owner has nothing to do there.  `load_token` only issues the
// loads, in the storage type; `stage_token` rotates, scales the key, and writes q at row[i], k at row[PADDED + i] and
// q . k at row[2 PADDED] (32-bit, to shared or global memory).  Every product and sum is spelled out, so that the
// kernels that share this code leave the same bits.
template <typename T, int PER_LANE>
struct TokenInputs {
  static constexpr int PAIRED = (PER_LANE + 1) / 2;              // 32 e < half <= PADDED / 2 for these e alone
  T q[PER_LANE], k[PER_LANE], partner_q[PAIRED], partner_k[PAIRED];
  float position;
};

template <typename T, int PER_LANE>
__device__ __forceinline__ void load_token(TokenInputs<T, PER_LANE>& in, const T* __restrict__ q,
                                           const T* __restrict__ k, size_t source, bool live, float position, int lane,
                                           int dim, int half, int rotary_dim) {
  in.position = live ? position : 0.0f;
#pragma unroll
  for (int e = 0; e < PER_LANE; ++e) {
    const int i = lane + 32 * e;
    const bool mine = live && i < dim && !(i >= half && i < rotary_dim);
    in.q[e] = mine ? q[source + i] : T(0.0f);
    in.k[e] = mine ? k[source + i] : T(0.0f);
    if (e < TokenInputs<T, PER_LANE>::PAIRED) {
      const bool paired = live && i < half;
      in.partner_q[e] = paired ? q[source + i + half] : T(0.0f);
      in.partner_k[e] = paired ? k[source + i + half] : T(0.0f);
    }
  }
}

template <typename T, int PER_LANE>
__device__ __forceinline__ void stage_token(const TokenInputs<T, PER_LANE>& in, const float* frequency, float key_scale,
                                            int lane, int half, int rotary_dim, float* row) {
  constexpr int PADDED = 32 * PER_LANE;
  float sum = 0.0f;
#pragma unroll
  for (int e = 0; e < PER_LANE; ++e) {
    const int i = lane + 32 * e;
    if (32 * e >= half && 32 * e + 32 <= rotary_dim) continue;   // a warp of partners: their owners write them
    const float qi = to_float(in.q[e]), ki = to_float(in.k[e]);
    if (e < TokenInputs<T, PER_LANE>::PAIRED && i < half) {
      // the first of a pair becomes u cos - v sin, the second v cos + u sin
      const float qp = to_float(in.partner_q[e]), kp = to_float(in.partner_k[e]);
      float sine, cosine;
      sincosf(__fmul_rn(in.position, frequency[e]), &sine, &cosine);
      const float q_first = fmaf(qi, cosine, -__fmul_rn(qp, sine)), q_second = fmaf(qp, cosine, __fmul_rn(qi, sine));
      const float k_first = __fmul_rn(fmaf(ki, cosine, -__fmul_rn(kp, sine)), key_scale);
      const float k_second = __fmul_rn(fmaf(kp, cosine, __fmul_rn(ki, sine)), key_scale);
      sum = fmaf(q_first, k_first, sum);
      sum = fmaf(q_second, k_second, sum);
      row[i] = q_first; row[PADDED + i] = k_first;
      row[i + half] = q_second; row[PADDED + i + half] = k_second;
    } else if (!(i >= half && i < rotary_dim)) {                 // not rotated (or beyond dim: zeros)
      const float scaled = __fmul_rn(ki, key_scale);
      sum = fmaf(qi, scaled, sum);
      row[i] = qi; row[PADDED + i] = scaled;
    }
  }
  sum = warp_sum(sum);
  if (lane == 0) row[2 * PADDED] = sum;
}

// blockDim (32, kWarps), grid (rows, heads, ceil(value_dim / (kWarps * 32 / kLanes))).  kLanes lanes share one column of
// the state (a function of the head's width alone: 16 from 33 key channels on, so that a single prompt fills the GPU
// with short chains); lane l of a column holds the key channels 4 (m kLanes + l) .. + 3, m < PER / 4.  The inputs of
// CHUNK tokens at a time are staged in shared memory (every column of a head reads the same q and k): a warp stages
// whole tokens, rotating as it goes, and leaves the token's q . k beside them.  What the next chunk needs is fetched
// into registers before the walk over the current chunk starts.  SHORT: a step of single tokens stages one token a warp.
template <typename T, int PER, int kLanes, bool SHORT>
__global__ void __launch_bounds__(kWarps * 32)
retention_scan_kernel(const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v, long long ld,
                      const float* __restrict__ inv_freq, int rotary_dim, const float* __restrict__ decays,
                      float key_scale, float* __restrict__ state, const int* __restrict__ query_starts,
                      const int* __restrict__ state_slots, const int* __restrict__ positions, float* __restrict__ out,
                      int heads, int dim, int value_dim) {
  constexpr int COLUMNS = 32 / kLanes;
  constexpr int BLOCK_COLUMNS = COLUMNS * kWarps;
  constexpr int PADDED = kLanes * PER;
  constexpr int ROW = 2 * PADDED + 4 + BLOCK_COLUMNS;             // q | k | q . k | v of this CTA's columns
  constexpr int CHUNK = SHORT ? kWarps : (PADDED <= 64 ? 32 : (PADDED <= 128 ? 16 : 8));
  __shared__ __align__(16) float staged[CHUNK * ROW];
  grid_launch_dependents();
  grid_dependency_wait();
  const int lane = threadIdx.x, warp = threadIdx.y;
  const int thread = warp * 32 + lane;
  const int l = lane % kLanes;
  const int row = blockIdx.x, head = blockIdx.y;
  const int first_column = blockIdx.z * BLOCK_COLUMNS;
  const int local_column = warp * COLUMNS + lane / kLanes;
  const int column = first_column + local_column;
  const int start = query_starts[row], end = query_starts[row + 1];
  if (end <= start || positions[start] < 0) return;              // the whole CTA: an empty or padding row
  const bool active = column < value_dim;
  const bool wide = dim % 4 == 0;
  const float decay = decays[head];
  const int half = rotary_dim / 2;
  float* column_state = state + (((size_t)state_slots[row] * heads + head) * value_dim + (active ? column : 0)) * dim;

  float s[PER];
#pragma unroll
  for (int m = 0; m < PER; m += 4) {
    const int i = (m / 4 * kLanes + l) * 4;
    if (wide) {
      const float4 piece = (active && i < dim) ? *reinterpret_cast<const float4*>(column_state + i)
                                               : make_float4(0.f, 0.f, 0.f, 0.f);
      s[m] = piece.x; s[m + 1] = piece.y; s[m + 2] = piece.z; s[m + 3] = piece.w;
    } else {
#pragma unroll
      for (int e = 0; e < 4; ++e) s[m + e] = (active && i + e < dim) ? column_state[i + e] : 0.0f;
    }
  }
  const size_t key_at = (size_t)head * dim, value_at = (size_t)head * value_dim;
  constexpr int TOKENS_PER_WARP = CHUNK / kWarps;
  constexpr int PER_LANE = PADDED / 32;
  constexpr int VALUES_PER_THREAD = (CHUNK * BLOCK_COLUMNS + kWarps * 32 - 1) / (kWarps * 32);
  // `fetch` only issues the loads: nothing waits for them before `commit`, which runs after the walk over the chunk
  // before.
  using Inputs = TokenInputs<T, PER_LANE>;
  Inputs next[TOKENS_PER_WARP];
  T next_v[VALUES_PER_THREAD];
  float frequency[Inputs::PAIRED];                               // of the pairs this lane rotates
#pragma unroll
  for (int e = 0; e < Inputs::PAIRED; ++e) frequency[e] = lane + 32 * e < half ? inv_freq[lane + 32 * e] : 0.0f;
  auto fetch = [&](int from) {
    const int count = min(CHUNK, end - from);
#pragma unroll
    for (int tt = 0; tt < TOKENS_PER_WARP; ++tt) {
      const int t = warp + tt * kWarps;
      const bool live = t < count;
      load_token(next[tt], q, k, (size_t)(from + (live ? t : 0)) * ld + key_at, live,
                 live ? (float)positions[from + t] : 0.0f, lane, dim, half, rotary_dim);
    }
#pragma unroll
    for (int j = 0; j < VALUES_PER_THREAD; ++j) {
      const int index = thread + j * kWarps * 32;
      const int t = index / BLOCK_COLUMNS, c = index - t * BLOCK_COLUMNS;
      next_v[j] = (t < count && first_column + c < value_dim)
                      ? v[(size_t)(from + t) * ld + value_at + first_column + c] : T(0.0f);
    }
  };
  auto commit = [&](int from) {
    const int count = min(CHUNK, end - from);
#pragma unroll
    for (int tt = 0; tt < TOKENS_PER_WARP; ++tt) {
      const int t = warp + tt * kWarps;
      if (t >= count) continue;                                  // (the same for the whole warp)
      stage_token(next[tt], frequency, key_scale, lane, half, rotary_dim, staged + t * ROW);
    }
#pragma unroll
    for (int j = 0; j < VALUES_PER_THREAD; ++j) {
      const int index = thread + j * kWarps * 32;
      const int t = index / BLOCK_COLUMNS, c = index - t * BLOCK_COLUMNS;
      if (t < CHUNK) staged[t * ROW + 2 * PADDED + 4 + c] = to_float(next_v[j]);
    }
  };
  fetch(start);
  const size_t out_width = (size_t)heads * value_dim;
  for (int from = start; from < end; from += CHUNK) {
    const int count = min(CHUNK, end - from);
    __syncthreads();                                             // the chunk before has been read
    commit(from);
    __syncthreads();
    if (from + CHUNK < end) fetch(from + CHUNK);
#pragma unroll 4
    for (int t = 0; t < count; ++t) {
      const float* in = staged + t * ROW;
      const float value = in[2 * PADDED + 4 + local_column];
      float read[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
      for (int m = 0; m < PER; m += 4) {
        const int i = (m / 4 * kLanes + l) * 4;
        const float4 query = *reinterpret_cast<const float4*>(in + i);
        const float4 key = *reinterpret_cast<const float4*>(in + PADDED + i);
        read[0] = fmaf(s[m], query.x, read[0]);
        read[1] = fmaf(s[m + 1], query.y, read[1]);
        read[2] = fmaf(s[m + 2], query.z, read[2]);
        read[3] = fmaf(s[m + 3], query.w, read[3]);
        s[m] = fmaf(s[m], decay, key.x * value);
        s[m + 1] = fmaf(s[m + 1], decay, key.y * value);
        s[m + 2] = fmaf(s[m + 2], decay, key.z * value);
        s[m + 3] = fmaf(s[m + 3], decay, key.w * value);
      }
      float total = (read[0] + read[1]) + (read[2] + read[3]);
#pragma unroll
      for (int step = 1; step < kLanes; step <<= 1) total += __shfl_xor_sync(0xffffffffu, total, step);
      if (l == 0 && active)
        out[(size_t)(from + t) * out_width + value_at + column] = fmaf(in[2 * PADDED], value, decay * total);
    }
  }
  if (!active) return;
#pragma unroll
  for (int m = 0; m < PER; m += 4) {
    const int i = (m / 4 * kLanes + l) * 4;
    if (wide) {
      if (i < dim) *reinterpret_cast<float4*>(column_state + i) = make_float4(s[m], s[m + 1], s[m + 2], s[m + 3]);
    } else {
#pragma unroll
      for (int e = 0; e < 4; ++e)
        if (i + e < dim) column_state[i + e] = s[m + e];
    }
  }
}

// The staging alone, for steps that bring portions of prompts: one warp per (token, head) writes what `stage_token`
// makes into prepared[token, head, 2 PADDED + 4] (32-bit), so that the walk below has nothing but copies between its
// chunks and no CTA of a head repeats another's rotation.  blockDim (32, kWarps), grid ceil(tokens * heads / kWarps).
template <typename T, int PER_LANE>
__global__ void __launch_bounds__(kWarps * 32)
retention_prepare_kernel(const T* __restrict__ q, const T* __restrict__ k, long long ld,
                         const float* __restrict__ inv_freq, int rotary_dim, float key_scale,
                         const int* __restrict__ positions, float* __restrict__ prepared, int tokens, int heads, int dim) {
  constexpr int PADDED = 32 * PER_LANE;
  using Inputs = TokenInputs<T, PER_LANE>;
  grid_launch_dependents();
  grid_dependency_wait();
  const int lane = threadIdx.x;
  const long long unit = (long long)blockIdx.x * kWarps + threadIdx.y;
  if (unit >= (long long)tokens * heads) return;
  const int token = (int)(unit / heads), head = (int)(unit - (long long)token * heads);
  const int position = positions[token];
  if (position < 0) return;                                      // padding
  const int half = rotary_dim / 2;
  float frequency[Inputs::PAIRED];
#pragma unroll
  for (int e = 0; e < Inputs::PAIRED; ++e) frequency[e] = lane + 32 * e < half ? inv_freq[lane + 32 * e] : 0.0f;
  Inputs in;
  load_token(in, q, k, (size_t)token * ld + (size_t)head * dim, true, (float)position, lane, dim, half, rotary_dim);
  stage_token(in, frequency, key_scale, lane, half, rotary_dim, prepared + (size_t)unit * (2 * PADDED + 4));
}

// The walk over prepared rows: as retention_scan_kernel, but a chunk's q, k and q . k arrive by 16-byte asynchronous
// copies into the other half of the staging buffer while the current chunk is walked.  The same lanes, the same order
// of sums: the results are those of the kernel above, bit for bit.
template <typename T, int PER, int kLanes>
__global__ void __launch_bounds__(kWarps * 32)
retention_scan_prepared_kernel(const float* __restrict__ prepared, const T* __restrict__ v, long long ld,
                               const float* __restrict__ decays, float* __restrict__ state,
                               const int* __restrict__ query_starts, const int* __restrict__ state_slots,
                               const int* __restrict__ positions, float* __restrict__ out, int heads, int dim,
                               int value_dim) {
  constexpr int COLUMNS = 32 / kLanes;
  constexpr int BLOCK_COLUMNS = COLUMNS * kWarps;
  constexpr int PADDED = kLanes * PER;
  constexpr int PREPARED = 2 * PADDED + 4;                        // q | k | q . k
  constexpr int ROW = PREPARED + BLOCK_COLUMNS;                   // and v of this CTA's columns
  constexpr int CHUNK = PADDED <= 128 ? 16 : 8;
  constexpr int PIECES = PREPARED / 4;                            // 16-byte pieces of a prepared row
  constexpr int VALUES_PER_THREAD = (CHUNK * BLOCK_COLUMNS + kWarps * 32 - 1) / (kWarps * 32);
  __shared__ __align__(16) float staged[2][CHUNK * ROW];
  __shared__ __align__(16) float partial[CHUNK][kWarps * 32];     // per token: every lane's part of its column's read-out
  grid_launch_dependents();
  grid_dependency_wait();
  const int lane = threadIdx.x, warp = threadIdx.y;
  const int thread = warp * 32 + lane;
  const int l = lane % kLanes;
  const int row = blockIdx.x, head = blockIdx.y;
  const int first_column = blockIdx.z * BLOCK_COLUMNS;
  const int local_column = warp * COLUMNS + lane / kLanes;
  const int column = first_column + local_column;
  const int start = query_starts[row], end = query_starts[row + 1];
  if (end <= start || positions[start] < 0) return;
  const bool active = column < value_dim;
  const bool wide = dim % 4 == 0;
  const float decay = decays[head];
  float* column_state = state + (((size_t)state_slots[row] * heads + head) * value_dim + (active ? column : 0)) * dim;
  float s[PER];
#pragma unroll
  for (int m = 0; m < PER; m += 4) {
    const int i = (m / 4 * kLanes + l) * 4;
    if (wide) {
      const float4 piece = (active && i < dim) ? *reinterpret_cast<const float4*>(column_state + i)
                                               : make_float4(0.f, 0.f, 0.f, 0.f);
      s[m] = piece.x; s[m + 1] = piece.y; s[m + 2] = piece.z; s[m + 3] = piece.w;
    } else {
#pragma unroll
      for (int e = 0; e < 4; ++e) s[m + e] = (active && i + e < dim) ? column_state[i + e] : 0.0f;
    }
  }
  const size_t value_at = (size_t)head * value_dim;
  T next_v[VALUES_PER_THREAD];
  auto issue = [&](int from, int stage) {
    const int count = min(CHUNK, end - from);
    for (int piece = thread; piece < count * PIECES; piece += kWarps * 32) {
      const int t = piece / PIECES, c = piece - t * PIECES;
      const float* source = prepared + ((size_t)(from + t) * heads + head) * PREPARED + 4 * c;
      const unsigned target = (unsigned)__cvta_generic_to_shared(&staged[stage][t * ROW + 4 * c]);
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(target), "l"(source) : "memory");
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
#pragma unroll
    for (int j = 0; j < VALUES_PER_THREAD; ++j) {
      const int index = thread + j * kWarps * 32;
      const int t = index / BLOCK_COLUMNS, c = index - t * BLOCK_COLUMNS;
      next_v[j] = (t < count && first_column + c < value_dim)
                      ? v[(size_t)(from + t) * ld + value_at + first_column + c] : T(0.0f);
    }
  };
  issue(start, 0);
  const size_t out_width = (size_t)heads * value_dim;
  int stage = 0;
  for (int from = start; from < end; from += CHUNK, stage ^= 1) {
    const int count = min(CHUNK, end - from);
    asm volatile("cp.async.wait_group 0;" ::: "memory");
#pragma unroll
    for (int j = 0; j < VALUES_PER_THREAD; ++j) {
      const int index = thread + j * kWarps * 32;
      const int t = index / BLOCK_COLUMNS, c = index - t * BLOCK_COLUMNS;
      if (t < CHUNK) staged[stage][t * ROW + PREPARED + c] = to_float(next_v[j]);
    }
    __syncthreads();                   // this chunk is whole, and every thread has left the chunk before
    if (from + CHUNK < end) issue(from + CHUNK, stage ^ 1);
#pragma unroll 4
    for (int t = 0; t < count; ++t) {
      const float* in = staged[stage] + t * ROW;
      const float value = in[PREPARED + local_column];
      float read[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
      for (int m = 0; m < PER; m += 4) {
        const int i = (m / 4 * kLanes + l) * 4;
        const float4 query = *reinterpret_cast<const float4*>(in + i);
        const float4 key = *reinterpret_cast<const float4*>(in + PADDED + i);
        read[0] = fmaf(s[m], query.x, read[0]);
        read[1] = fmaf(s[m + 1], query.y, read[1]);
        read[2] = fmaf(s[m + 2], query.z, read[2]);
        read[3] = fmaf(s[m + 3], query.w, read[3]);
        s[m] = fmaf(s[m], decay, key.x * value);
        s[m + 1] = fmaf(s[m + 1], decay, key.y * value);
        s[m + 2] = fmaf(s[m + 2], decay, key.z * value);
        s[m + 3] = fmaf(s[m + 3], decay, key.w * value);
      }
      partial[t][thread] = (read[0] + read[1]) + (read[2] + read[3]);
    }
    __syncthreads();
    // the lanes' parts of a column are summed as the butterfly of shuffles in the kernel above sums them (neighbours
    // first, then pairs of pairs, ...), so that the bits are the same; one (token, column) a thread and pass
    for (int index = thread; index < count * BLOCK_COLUMNS; index += kWarps * 32) {
      const int t = index / BLOCK_COLUMNS, c = index - t * BLOCK_COLUMNS;
      float parts[kLanes];
#pragma unroll
      for (int i = 0; i < kLanes; i += 4) {
        const float4 four = *reinterpret_cast<const float4*>(&partial[t][c * kLanes + i]);
        parts[i] = four.x; parts[i + 1] = four.y; parts[i + 2] = four.z; parts[i + 3] = four.w;
      }
#pragma unroll
      for (int width = 1; width < kLanes; width <<= 1)
#pragma unroll
        for (int i = 0; i < kLanes; i += 2 * width) parts[i] += parts[i + width];
      const float* in = staged[stage] + t * ROW;
      if (first_column + c < value_dim)
        out[(size_t)(from + t) * out_width + value_at + first_column + c] =
            fmaf(in[2 * PADDED], in[PREPARED + c], decay * parts[0]);
    }
  }
  if (!active) return;
#pragma unroll
  for (int m = 0; m < PER; m += 4) {
    const int i = (m / 4 * kLanes + l) * 4;
    if (wide) {
      if (i < dim) *reinterpret_cast<float4*>(column_state + i) = make_float4(s[m], s[m + 1], s[m + 2], s[m + 3]);
    } else {
#pragma unroll
      for (int e = 0; e < 4; ++e)
        if (i + e < dim) column_state[i + e] = s[m + e];
    }
  }
}

template <typename T, int PER, int kLanes>
int launch_prepared(cudaStream_t stream, const void* q, const void* k, const void* v, long long ld, const float* inv_freq,
                    int rotary_dim, const float* decays, float key_scale, float* state, const int* query_starts,
                    const int* state_slots, const int* positions, float* out, float* prepared, int tokens, int rows,
                    int heads, int dim, int value_dim) {
  constexpr int columns = kWarps * (32 / kLanes);
  const long long units = (long long)tokens * heads;
  int status = mir_launch("retention_prepare", retention_prepare_kernel<T, kLanes * PER / 32>,
                          dim3((unsigned)((units + kWarps - 1) / kWarps)), dim3(32, kWarps), 0, stream, 0, (const T*)q,
                          (const T*)k, ld, inv_freq, rotary_dim, key_scale, positions, prepared, tokens, heads, dim);
  if (status != MIR_OK) return status;
  return mir_launch("retention_scan", retention_scan_prepared_kernel<T, PER, kLanes>,
                    dim3(rows, heads, (value_dim + columns - 1) / columns), dim3(32, kWarps), 0, stream, 0,
                    (const float*)prepared, (const T*)v, ld, decays, state, query_starts, state_slots, positions, out,
                    heads, dim, value_dim);
}

template <typename T, int PER, int kLanes, bool SHORT>
int launch_scan(cudaStream_t stream, const void* q, const void* k, const void* v, long long ld, const float* inv_freq,
                int rotary_dim, const float* decays, float key_scale, float* state, const int* query_starts,
                const int* state_slots, const int* positions, float* out, int rows, int heads, int dim, int value_dim) {
  constexpr int columns = kWarps * (32 / kLanes);
  return mir_launch("retention_scan", retention_scan_kernel<T, PER, kLanes, SHORT>,
                    dim3(rows, heads, (value_dim + columns - 1) / columns), dim3(32, kWarps), 0, stream, 0, (const T*)q,
                    (const T*)k, (const T*)v, ld, inv_freq, rotary_dim, decays, key_scale, state, query_starts,
                    state_slots, positions, out, heads, dim, value_dim);
}

template <typename T>
int launch_scan_for(cudaStream_t stream, const void* q, const void* k, const void* v, long long ld,
                    const float* inv_freq, int rotary_dim, const float* decays, float key_scale, float* state,
                    const int* query_starts, const int* state_slots, const int* positions, float* out, int rows,
                    int heads, int dim, int value_dim, bool single_tokens, float* prepared, int tokens) {
#define MIR_RETENTION(P, L)                                                                                         \
  if (prepared && !single_tokens)                                                                                   \
    return launch_prepared<T, P, L>(stream, q, k, v, ld, inv_freq, rotary_dim, decays, key_scale, state,           \
                                    query_starts, state_slots, positions, out, prepared, tokens, rows, heads, dim,  \
                                    value_dim);                                                                     \
  if (single_tokens)                                                                                                \
    return launch_scan<T, P, L, true>(stream, q, k, v, ld, inv_freq, rotary_dim, decays, key_scale, state,         \
                                      query_starts, state_slots, positions, out, rows, heads, dim, value_dim);     \
  return launch_scan<T, P, L, false>(stream, q, k, v, ld, inv_freq, rotary_dim, decays, key_scale, state,          \
                                     query_starts, state_slots, positions, out, rows, heads, dim, value_dim);
  if (dim <= 32) { MIR_RETENTION(4, 8) }
  if (dim <= 64) { MIR_RETENTION(4, 16) }
  if (dim <= 128) { MIR_RETENTION(8, 16) }
  if (dim <= 192) { MIR_RETENTION(12, 16) }
  if (dim <= 256) { MIR_RETENTION(16, 16) }
#undef MIR_RETENTION
  mir_set_error("retention_scan: heads of %d key channels are wider than 256", dim);
  return MIR_BAD_ARGUMENT;
}

}  // namespace

// q, k [tokens, heads * dim] and v [tokens, heads * value_dim] with one row stride ld in the activations' type (views
// of one packed projection); inv_freq [rotary_dim / 2] 32-bit (may be null with rotary_dim 0); decays [heads] 32-bit;
// state [slots, heads, value_dim, dim] 32-bit; out [tokens, heads * value_dim] 32-bit: o before the head norm.
// prepared: null, or 32-bit scratch of tokens * heads * (2 * padded + 4) numbers, padded = the key width rounded up to
// 32, 64, 128, 192 or 256: a step that brings more than single tokens then rotates in a kernel of its own first.
MIR_EXPORT int mir_retention_scan(int bf16, const void* q, const void* k, const void* v, long long ld,
                                  const float* inv_freq, int rotary_dim, const float* decays, float key_scale,
                                  float* state, const int* query_starts, const int* state_slots, const int* positions,
                                  float* out, float* prepared, int tokens, int rows, int heads, int dim, int value_dim,
                                  cudaStream_t stream) {
  if (tokens == 0 || rows == 0) return MIR_OK;
  if (tokens < 0 || rows < 0 || heads <= 0 || dim <= 0 || value_dim <= 0 || heads > 65535 || rotary_dim < 0 ||
      rotary_dim > dim || (rotary_dim & 1) || (rotary_dim > 0 && inv_freq == nullptr)) {
    mir_set_error("retention_scan: bad sizes (tokens %d, rows %d, heads %d, dim %d, value_dim %d, rotary_dim %d)",
                  tokens, rows, heads, dim, value_dim, rotary_dim);
    return MIR_BAD_ARGUMENT;
  }
  const bool single_tokens = tokens == rows;                     // a step of decoded tokens: every row brings one
  if (bf16)
    return launch_scan_for<__nv_bfloat16>(stream, q, k, v, ld, inv_freq, rotary_dim, decays, key_scale, state,
                                          query_starts, state_slots, positions, out, rows, heads, dim, value_dim,
                                          single_tokens, prepared, tokens);
  return launch_scan_for<float>(stream, q, k, v, ld, inv_freq, rotary_dim, decays, key_scale, state, query_starts,
                                state_slots, positions, out, rows, heads, dim, value_dim, single_tokens, prepared, tokens);
}
