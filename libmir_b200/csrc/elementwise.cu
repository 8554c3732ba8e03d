// Embedding gather, RMSNorm, SiLU-gate and bias kernels.  The residual stream is 32-bit in both
// engine dtypes; T is the storage type of weights and activations (float or bf16).
//
// What each replaces in libmir: embedding_bf16.cu:3-19, rms_norm_bf16.cu:3-36,
// elementwise_bf16.cu:42-70 (packed gate|up), select_row_bf16.cu (row gather, folded into the norm).
#include <cuda_fp16.h>
#include "common.cuh"

using namespace mir;

// out[r, :] = float(table[ids[r], :]) * scale.  An id outside [0, vocab) gives a row of zeros;
// the host rejects such ids before the launch.
template <typename T>
__global__ void embed_kernel(const T* __restrict__ table, const int* __restrict__ ids, float* __restrict__ out,
                             int hidden, int vocab, float scale) {
  grid_launch_dependents();
  grid_dependency_wait();
  const int row = blockIdx.x;
  const int id = ids[row];
  const bool ok = id >= 0 && id < vocab;
  const T* src = table + (size_t)(ok ? id : 0) * hidden;
  float* dst = out + (size_t)row * hidden;
  for (int c = threadIdx.x; c < hidden; c += blockDim.x) dst[c] = ok ? to_float(src[c]) * scale : 0.0f;
}

// out[r, :] = float(table[ids[r], :]) * scale + float(pairs[bucket(r), :]): a second table indexed by a hash of the
// token and the token before it in its request, bucket = (previous * mul_previous + id * mul_current) mod buckets;
// a request's first token (previous < 0) takes row `buckets`, the table's last.
template <typename T>
__global__ void embed_pairs_kernel(const T* __restrict__ table, const T* __restrict__ pairs, const int* __restrict__ ids,
                                   const int* __restrict__ previous, float* __restrict__ out, int hidden, int vocab,
                                   int buckets, long long mul_previous, long long mul_current, float scale) {
  grid_launch_dependents();
  grid_dependency_wait();
  const int row = blockIdx.x;
  const int id = ids[row];
  const int before = previous[row];
  const bool ok = id >= 0 && id < vocab;
  const long long bucket = before < 0 ? (long long)buckets
                                      : (((long long)before * mul_previous + (long long)id * mul_current) % buckets + buckets) % buckets;
  const T* src = table + (size_t)(ok ? id : 0) * hidden;
  const T* pair = pairs + (size_t)bucket * hidden;
  float* dst = out + (size_t)row * hidden;
  for (int c = threadIdx.x; c < hidden; c += blockDim.x)
    dst[c] = ok ? to_float(src[c]) * scale + to_float(pair[c]) : 0.0f;
}

// x <- 0.5 x (1 + tanh(sqrt(2 / pi) (x + 0.044715 x^3))), in place.
template <typename T>
__global__ void gelu_tanh_kernel(T* __restrict__ x, size_t total) {
  const size_t index = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (index >= total) return;
  const float z = to_float(x[index]);
  const float inner = 0.7978845608028654f * fmaf(0.044715f * z * z, z, z);
  x[index] = from_float<T>(0.5f * z * (1.0f + tanhf(inner)));
}

// residual[r, :] += scale * sum over branches b of branch_b[r, :] * rsqrt(mean(branch_b[r, :]^2) + eps) * weight_b:
// several branch outputs (32-bit rows), each normalised over the model width with a weight of its own, added to the
// residual stream in one pass.  Fixed reduction tree per branch.
struct NormedBranches {
  const float* rows[4];
  const float* weight[4];
  int count;
};
// `rounded` (may be null): the updated residual's rows once more, rounded to bfloat16, for the product that reads them next.
__global__ void add_normed_branches_kernel(NormedBranches branches, float* __restrict__ residual,
                                           __nv_bfloat16* __restrict__ rounded, int hidden, float eps, float scale) {
  __shared__ float scratch[32];
  grid_launch_dependents();
  grid_dependency_wait();
  const int row = blockIdx.x;
  float inverse[4];
  for (int b = 0; b < branches.count; ++b) {
    const float* src = branches.rows[b] + (size_t)row * hidden;
    float sum = 0.0f;
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) sum = fmaf(src[c], src[c], sum);
    sum = block_sum(sum, scratch);
    inverse[b] = rsqrtf(sum / (float)hidden + eps);
  }
  float* dst = residual + (size_t)row * hidden;
  for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
    float total = 0.0f;
    for (int b = 0; b < branches.count; ++b)
      total += branches.rows[b][(size_t)row * hidden + c] * inverse[b] * branches.weight[b][c];
    const float updated = dst[c] + scale * total;
    dst[c] = updated;
    if (rounded) rounded[(size_t)row * hidden + c] = __float2bfloat16(updated);
  }
}

// The same with 16-byte accesses (hidden a multiple of 4, every pointer 16-byte aligned); the second pass finds the
// rows in L1.
__global__ void add_normed_branches_vec4_kernel(NormedBranches branches, float* __restrict__ residual,
                                                __nv_bfloat16* __restrict__ rounded, int hidden, float eps, float scale) {
  __shared__ float scratch[32];
  grid_launch_dependents();
  grid_dependency_wait();
  const int row = blockIdx.x;
  const int quads = hidden >> 2;
  float inverse[4];
  for (int b = 0; b < branches.count; ++b) {
    const float4* src = reinterpret_cast<const float4*>(branches.rows[b] + (size_t)row * hidden);
    float sum = 0.0f;
    for (int c = threadIdx.x; c < quads; c += blockDim.x) {
      const float4 v = src[c];
      sum = fmaf(v.x, v.x, fmaf(v.y, v.y, fmaf(v.z, v.z, fmaf(v.w, v.w, sum))));
    }
    sum = block_sum(sum, scratch);
    inverse[b] = rsqrtf(sum / (float)hidden + eps);
  }
  float4* dst = reinterpret_cast<float4*>(residual + (size_t)row * hidden);
  for (int c = threadIdx.x; c < quads; c += blockDim.x) {
    float4 total = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    for (int b = 0; b < branches.count; ++b) {
      const float4 v = reinterpret_cast<const float4*>(branches.rows[b] + (size_t)row * hidden)[c];
      const float4 w = __ldg(reinterpret_cast<const float4*>(branches.weight[b]) + c);
      total.x += v.x * inverse[b] * w.x; total.y += v.y * inverse[b] * w.y;
      total.z += v.z * inverse[b] * w.z; total.w += v.w * inverse[b] * w.w;
    }
    float4 r = dst[c];
    r.x += scale * total.x; r.y += scale * total.y; r.z += scale * total.z; r.w += scale * total.w;
    dst[c] = r;
    if (rounded) {
      uint2 packed;
      *reinterpret_cast<__nv_bfloat162*>(&packed.x) = __floats2bfloat162_rn(r.x, r.y);
      *reinterpret_cast<__nv_bfloat162*>(&packed.y) = __floats2bfloat162_rn(r.z, r.w);
      reinterpret_cast<uint2*>(rounded + (size_t)row * hidden)[c] = packed;
    }
  }
}

// gelu_tanh on eight bfloat16 values per thread (16-byte accesses).
__global__ void gelu_tanh_bf16x8_kernel(__nv_bfloat16* __restrict__ x, size_t total8) {
  const size_t index = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (index >= total8) return;
  float z[8];
  load8(x + index * 8, z);
  uint4 packed;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&packed);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float a = z[2 * i], b = z[2 * i + 1];
    h[i] = __floats2bfloat162_rn(0.5f * a * (1.0f + tanhf(0.7978845608028654f * fmaf(0.044715f * a * a, a, a))),
                                 0.5f * b * (1.0f + tanhf(0.7978845608028654f * fmaf(0.044715f * b * b, b, b))));
  }
  *reinterpret_cast<uint4*>(x + index * 8) = packed;
}

// y[r, :] = x[src(r), :] * rsqrt(mean(x^2) + eps) * w, src(r) = rows ? rows[r] : r.
// Sum of squares and scaling in 32-bit with a fixed reduction tree.
template <typename Tout>
__global__ void rms_norm_kernel(const float* __restrict__ x, const float* __restrict__ weight,
                                Tout* __restrict__ out, const int* __restrict__ rows, int hidden, float eps) {
  __shared__ float scratch[32];
  grid_launch_dependents();
  grid_dependency_wait();

  const int row = blockIdx.x;
  const float* src = x + (size_t)(rows ? rows[row] : row) * hidden;
  float sum = 0.0f;
  for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
    const float v = src[c];
    sum = fmaf(v, v, sum);
  }
  sum = block_sum(sum, scratch);
  const float inverse = rsqrtf(sum / (float)hidden + eps);
  Tout* dst = out + (size_t)row * hidden;
  for (int c = threadIdx.x; c < hidden; c += blockDim.x) dst[c] = from_float<Tout>(src[c] * inverse * weight[c]);
}

// The same with 16-byte loads (hidden a multiple of 4); the second pass finds the row in L1.
template <typename Tout>
__global__ void rms_norm_vec4_kernel(const float* __restrict__ x, const float* __restrict__ weight,
                                     Tout* __restrict__ out, const int* __restrict__ rows, int hidden, float eps) {
  __shared__ float scratch[32];
  grid_launch_dependents();
  grid_dependency_wait();
  const int row = blockIdx.x;
  const float4* src = reinterpret_cast<const float4*>(x + (size_t)(rows ? rows[row] : row) * hidden);
  const float4* w4 = reinterpret_cast<const float4*>(weight);
  const int quads = hidden >> 2;
  float sum = 0.0f;
  for (int c = threadIdx.x; c < quads; c += blockDim.x) {
    const float4 v = src[c];
    sum = fmaf(v.x, v.x, fmaf(v.y, v.y, fmaf(v.z, v.z, fmaf(v.w, v.w, sum))));
  }
  sum = block_sum(sum, scratch);
  const float inverse = rsqrtf(sum / (float)hidden + eps);
  Tout* dst = out + (size_t)row * hidden;
  for (int c = threadIdx.x; c < quads; c += blockDim.x) {
    const float4 v = src[c];
    const float4 w = __ldg(w4 + c);
    const float a = v.x * inverse * w.x, b = v.y * inverse * w.y, d = v.z * inverse * w.z, e = v.w * inverse * w.w;
    if (sizeof(Tout) == 4) {
      reinterpret_cast<float4*>(dst)[c] = make_float4(a, b, d, e);
    } else {
      const __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(d, e);
      uint2 packed;
      packed.x = *reinterpret_cast<const uint32_t*>(&lo);
      packed.y = *reinterpret_cast<const uint32_t*>(&hi);
      reinterpret_cast<uint2*>(dst)[c] = packed;
    }
  }
}

// out[r, c] = silu(gu[r, c]) * gu[r, inter + c]; gu rows are [gate | up].
template <typename T>
__global__ void silu_mul_kernel(const T* __restrict__ gu, T* __restrict__ out, int inter, size_t total) {
  const size_t index = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (index >= total) return;
  const size_t row = index / inter;
  const int col = (int)(index - row * inter);
  const float g = to_float(gu[row * 2 * inter + col]);
  const float u = to_float(gu[row * 2 * inter + inter + col]);
  out[index] = from_float<T>(g / (1.0f + expf(-g)) * u);
}

// The same, 8 columns per thread with 16-byte loads and stores (inter a multiple of 8, bf16).
__global__ void silu_mul_bf16x8_kernel(const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ out,
                                       int inter, size_t total8) {
  const size_t index = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (index >= total8) return;
  const int per_row = inter / 8;
  const size_t row = index / per_row;
  const int col = (int)(index - row * per_row) * 8;
  float g[8], u[8];
  load8(gu + row * 2 * inter + col, g);
  load8(gu + row * 2 * inter + inter + col, u);
  uint4 packed;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&packed);
#pragma unroll
  for (int i = 0; i < 4; ++i)
    h[i] = __floats2bfloat162_rn(g[2 * i] / (1.0f + expf(-g[2 * i])) * u[2 * i],
                                 g[2 * i + 1] / (1.0f + expf(-g[2 * i + 1])) * u[2 * i + 1]);
  *reinterpret_cast<uint4*>(out + row * inter + col) = packed;
}

// x[r, c] += bias[c]  (32-bit residual; used when a projection that accumulates into the residual has a bias).
template <typename T>
__global__ void add_bias_kernel(float* __restrict__ x, const T* __restrict__ bias, int cols, size_t total) {
  const size_t index = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (index >= total) return;
  x[index] += to_float(bias[index % cols]);
}

// dst[i] = T(src[i]) for the load-time casts (dense_cast.cu:4-18) and for copying logits rows.
template <typename Tin, typename Tout>
__global__ void cast_kernel(const Tin* __restrict__ src, Tout* __restrict__ dst, size_t total) {
  const size_t index = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (index < total) dst[index] = from_float<Tout>(to_float(src[index]));
}

#define LAUNCH_1D(kernel, total, ...)                                                      \
  do {                                                                                     \
    const size_t n_ = (total);                                                             \
    if (n_ == 0) return MIR_OK;                                                            \
    kernel<<<(unsigned)((n_ + 255) / 256), 256, 0, stream>>>(__VA_ARGS__);                 \
  } while (0)

MIR_EXPORT int mir_embed(int bf16, const void* table, const int* ids, float* out, int rows, int hidden, int vocab,
                         float scale, cudaStream_t stream) {
  if (rows == 0) return MIR_OK;
  if (rows < 0 || hidden <= 0 || vocab <= 0) { mir_set_error("embed: bad sizes"); return MIR_BAD_ARGUMENT; }
  if (bf16)
    return mir_launch("embed", embed_kernel<__nv_bfloat16>, dim3(rows), dim3(256), 0, stream, 0,
                      (const __nv_bfloat16*)table, ids, out, hidden, vocab, scale);
  return mir_launch("embed", embed_kernel<float>, dim3(rows), dim3(256), 0, stream, 0, (const float*)table, ids, out,
                    hidden, vocab, scale);
}

MIR_EXPORT int mir_embed_pairs(int bf16, const void* table, const void* pairs, const int* ids, const int* previous,
                               float* out, int rows, int hidden, int vocab, int buckets, long long mul_previous,
                               long long mul_current, float scale, cudaStream_t stream) {
  if (rows == 0) return MIR_OK;
  if (rows < 0 || hidden <= 0 || vocab <= 0 || buckets <= 0) { mir_set_error("embed_pairs: bad sizes"); return MIR_BAD_ARGUMENT; }
  if (bf16)
    return mir_launch("embed_pairs", embed_pairs_kernel<__nv_bfloat16>, dim3(rows), dim3(256), 0, stream, 0,
                      (const __nv_bfloat16*)table, (const __nv_bfloat16*)pairs, ids, previous, out, hidden, vocab,
                      buckets, mul_previous, mul_current, scale);
  return mir_launch("embed_pairs", embed_pairs_kernel<float>, dim3(rows), dim3(256), 0, stream, 0, (const float*)table,
                    (const float*)pairs, ids, previous, out, hidden, vocab, buckets, mul_previous, mul_current, scale);
}

// x <- act(x) in place: kind 1 the exact GELU 0.5 x (1 + erf(x / sqrt 2)), kind 2 tanh, kind 3 the square of relu;
// computed in 32-bit.
template <typename T>
__global__ void activation_kernel(T* __restrict__ x, size_t total, int kind) {
  const size_t index = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (index >= total) return;
  const float z = to_float(x[index]);
  const float positive = fmaxf(z, 0.0f);
  x[index] = from_float<T>(kind == 1 ? 0.5f * z * (1.0f + erff(z * 0.70710678118654752f))
                                     : (kind == 2 ? tanhf(z) : positive * positive));
}

// x <- cap * tanh(x / cap) on 32-bit logits.
__global__ void softcap_kernel(float* __restrict__ x, size_t total, float cap) {
  const size_t index = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (index < total) x[index] = cap * tanhf(x[index] / cap);
}

// residual[r, :] += rows[r, :] (if given) + vector (if given): what a pass of a looped run of layers starts with.
__global__ void add_rows_kernel(float* __restrict__ residual, const float* __restrict__ rows,
                                const float* __restrict__ vector, int hidden, size_t total) {
  const size_t index = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (index >= total) return;
  float v = residual[index];
  if (rows != nullptr) v += rows[index];
  if (vector != nullptr) v += vector[index % hidden];
  residual[index] = v;
}

// Two norms of the same rows: out_a = x * s * weight_a, out_b = x * s * weight_b with one s = rsqrt(mean(x^2) + eps).
template <typename Tout>
__global__ void rms_norm_pair_kernel(const float* __restrict__ x, const float* __restrict__ weight_a,
                                     const float* __restrict__ weight_b, Tout* __restrict__ out_a,
                                     Tout* __restrict__ out_b, int hidden, float eps) {
  __shared__ float scratch[32];
  grid_launch_dependents();
  grid_dependency_wait();
  const int row = blockIdx.x;
  const float* src = x + (size_t)row * hidden;
  float sum = 0.0f;
  for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
    const float v = src[c];
    sum = fmaf(v, v, sum);
  }
  sum = block_sum(sum, scratch);
  const float inverse = rsqrtf(sum / (float)hidden + eps);
  for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
    const float v = src[c] * inverse;
    out_a[(size_t)row * hidden + c] = from_float<Tout>(v * weight_a[c]);
    out_b[(size_t)row * hidden + c] = from_float<Tout>(v * weight_b[c]);
  }
}

MIR_EXPORT int mir_gelu_tanh(int bf16, void* x, size_t total, cudaStream_t stream) {
  if (bf16 && total % 8 == 0 && ((uintptr_t)x & 15) == 0) LAUNCH_1D(gelu_tanh_bf16x8_kernel, total / 8, (__nv_bfloat16*)x, total / 8);
  else if (bf16) LAUNCH_1D(gelu_tanh_kernel, total, (__nv_bfloat16*)x, total);
  else LAUNCH_1D(gelu_tanh_kernel, total, (float*)x, total);
  return mir_check_launch("gelu_tanh");
}

// rows_b, weight_b: `count` (1 to 4) pointers each, to 32-bit [rows, hidden] and [hidden].  rounded: null, or bfloat16
// [rows, hidden] that receives the updated residual.
MIR_EXPORT int mir_add_normed_branches(const float* const* branch_rows, const float* const* branch_weights, int count,
                                       float* residual, void* rounded, int rows, int hidden, float eps, float scale,
                                       cudaStream_t stream) {
  if (rows == 0) return MIR_OK;
  if (rows < 0 || hidden <= 0 || count < 1 || count > 4) { mir_set_error("add_normed_branches: bad sizes"); return MIR_BAD_ARGUMENT; }
  NormedBranches branches = {};
  branches.count = count;
  for (int b = 0; b < count; ++b) { branches.rows[b] = branch_rows[b]; branches.weight[b] = branch_weights[b]; }
  bool aligned = (hidden & 3) == 0 && ((uintptr_t)residual & 15) == 0 && ((uintptr_t)rounded & 7) == 0;
  for (int b = 0; b < count; ++b)
    aligned = aligned && ((uintptr_t)branch_rows[b] & 15) == 0 && ((uintptr_t)branch_weights[b] & 15) == 0;
  if (aligned)
    return mir_launch("add_normed_branches", add_normed_branches_vec4_kernel, dim3(rows), dim3(hidden >= 4096 ? 256 : 128),
                      0, stream, 0, branches, residual, (__nv_bfloat16*)rounded, hidden, eps, scale);
  const int threads = hidden >= 2048 ? 512 : 256;
  return mir_launch("add_normed_branches", add_normed_branches_kernel, dim3(rows), dim3(threads), 0, stream, 0, branches,
                    residual, (__nv_bfloat16*)rounded, hidden, eps, scale);
}

MIR_EXPORT int mir_rms_norm(int bf16, const float* x, const float* weight, void* out, const int* rows, int n_rows,
                            int hidden, float eps, cudaStream_t stream) {
  if (n_rows == 0) return MIR_OK;
  if (n_rows < 0 || hidden <= 0) { mir_set_error("rms_norm: bad sizes"); return MIR_BAD_ARGUMENT; }
  if ((hidden & 3) == 0 && ((uintptr_t)x & 15) == 0 && ((uintptr_t)weight & 15) == 0 && ((uintptr_t)out & 15) == 0) {
    const int vec_threads = hidden >= 1024 ? 256 : 128;
    if (bf16)
      return mir_launch("rms_norm", rms_norm_vec4_kernel<__nv_bfloat16>, dim3(n_rows), dim3(vec_threads), 0, stream, 0,
                        x, weight, (__nv_bfloat16*)out, rows, hidden, eps);
    return mir_launch("rms_norm", rms_norm_vec4_kernel<float>, dim3(n_rows), dim3(vec_threads), 0, stream, 0, x, weight,
                      (float*)out, rows, hidden, eps);
  }
  const int threads = hidden >= 2048 ? 512 : 256;
  if (bf16)
    return mir_launch("rms_norm", rms_norm_kernel<__nv_bfloat16>, dim3(n_rows), dim3(threads), 0, stream, 0, x, weight,
                      (__nv_bfloat16*)out, rows, hidden, eps);
  return mir_launch("rms_norm", rms_norm_kernel<float>, dim3(n_rows), dim3(threads), 0, stream, 0, x, weight,
                    (float*)out, rows, hidden, eps);
}

MIR_EXPORT int mir_activation(int kind, int bf16, void* x, size_t total, cudaStream_t stream) {
  if (kind < 1 || kind > 3) { mir_set_error("activation: unknown kind %d", kind); return MIR_BAD_ARGUMENT; }
  if (bf16) LAUNCH_1D(activation_kernel, total, (__nv_bfloat16*)x, total, kind);
  else LAUNCH_1D(activation_kernel, total, (float*)x, total, kind);
  return mir_check_launch(kind == 1 ? "gelu_erf" : (kind == 2 ? "tanh" : "relu_squared"));
}

MIR_EXPORT int mir_softcap(float* x, size_t total, float cap, cudaStream_t stream) {
  if (!(cap > 0.0f)) { mir_set_error("softcap: the cap must be greater than zero"); return MIR_BAD_ARGUMENT; }
  LAUNCH_1D(softcap_kernel, total, x, total, cap);
  return mir_check_launch("softcap");
}

MIR_EXPORT int mir_add_rows(float* residual, const float* rows, const float* vector, int n_rows, int hidden,
                            cudaStream_t stream) {
  if (n_rows < 0 || hidden <= 0) { mir_set_error("add_rows: bad sizes"); return MIR_BAD_ARGUMENT; }
  const size_t total = (size_t)n_rows * hidden;
  LAUNCH_1D(add_rows_kernel, total, residual, rows, vector, hidden, total);
  return mir_check_launch("add_rows");
}

MIR_EXPORT int mir_rms_norm_pair(int bf16, const float* x, const float* weight_a, const float* weight_b, void* out_a,
                                 void* out_b, int n_rows, int hidden, float eps, cudaStream_t stream) {
  if (n_rows == 0) return MIR_OK;
  if (n_rows < 0 || hidden <= 0) { mir_set_error("rms_norm_pair: bad sizes"); return MIR_BAD_ARGUMENT; }
  const int threads = hidden >= 2048 ? 512 : 256;
  if (bf16)
    return mir_launch("rms_norm_pair", rms_norm_pair_kernel<__nv_bfloat16>, dim3(n_rows), dim3(threads), 0, stream, 0, x,
                      weight_a, weight_b, (__nv_bfloat16*)out_a, (__nv_bfloat16*)out_b, hidden, eps);
  return mir_launch("rms_norm_pair", rms_norm_pair_kernel<float>, dim3(n_rows), dim3(threads), 0, stream, 0, x, weight_a,
                    weight_b, (float*)out_a, (float*)out_b, hidden, eps);
}

MIR_EXPORT int mir_silu_mul(int bf16, const void* gu, void* out, int rows, int inter, cudaStream_t stream) {
  if (rows < 0 || inter <= 0) { mir_set_error("silu_mul: bad sizes"); return MIR_BAD_ARGUMENT; }
  const size_t total = (size_t)rows * inter;
  if (bf16 && inter % 8 == 0 && ((uintptr_t)gu & 15) == 0 && ((uintptr_t)out & 15) == 0)
    LAUNCH_1D(silu_mul_bf16x8_kernel, total / 8, (const __nv_bfloat16*)gu, (__nv_bfloat16*)out, inter, total / 8);
  else if (bf16) LAUNCH_1D(silu_mul_kernel, total, (const __nv_bfloat16*)gu, (__nv_bfloat16*)out, inter, total);
  else LAUNCH_1D(silu_mul_kernel, total, (const float*)gu, (float*)out, inter, total);
  return mir_check_launch("silu_mul");
}

MIR_EXPORT int mir_add_bias(int bf16, float* x, const void* bias, int rows, int cols, cudaStream_t stream) {
  if (rows < 0 || cols <= 0) { mir_set_error("add_bias: bad sizes"); return MIR_BAD_ARGUMENT; }
  const size_t total = (size_t)rows * cols;
  if (bf16) LAUNCH_1D(add_bias_kernel, total, x, (const __nv_bfloat16*)bias, cols, total);
  else LAUNCH_1D(add_bias_kernel, total, x, (const float*)bias, cols, total);
  return mir_check_launch("add_bias");
}

// kind: 0 f32->bf16, 1 bf16->f32, 2 f16->bf16, 3 f16->f32 (what a checkpoint may store, to what the engine keeps).
MIR_EXPORT int mir_cast(int kind, const void* src, void* dst, size_t total, cudaStream_t stream) {
  if (kind == 0) LAUNCH_1D(cast_kernel, total, (const float*)src, (__nv_bfloat16*)dst, total);
  else if (kind == 1) LAUNCH_1D(cast_kernel, total, (const __nv_bfloat16*)src, (float*)dst, total);
  else if (kind == 2) LAUNCH_1D(cast_kernel, total, (const __half*)src, (__nv_bfloat16*)dst, total);
  else if (kind == 3) LAUNCH_1D(cast_kernel, total, (const __half*)src, (float*)dst, total);
  else { mir_set_error("cast: unknown kind %d", kind); return MIR_BAD_ARGUMENT; }
  return mir_check_launch("cast");
}

// Random weights on the device: element i of a tensor is a normal deviate (Box-Muller on two uniforms from the
// SplitMix64 of seed + 2 i and seed + 2 i + 1) times `deviation`: the same for a seed whatever the launch shape.
__device__ __forceinline__ unsigned long long splitmix64(unsigned long long x) {
  x += 0x9E3779B97F4A7C15ull;
  x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
  x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
  return x ^ (x >> 31);
}
template <typename T>
__global__ void random_normal_kernel(T* __restrict__ out, size_t total, unsigned long long seed, float deviation) {
  const size_t index = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (index >= total) return;
  const unsigned long long a = splitmix64(seed + 2ull * index), b = splitmix64(seed + 2ull * index + 1ull);
  const float u = ((float)(a >> 40) + 0.5f) * (1.0f / 16777216.0f);      // (0, 1)
  const float v = (float)(b >> 40) * (1.0f / 16777216.0f);               // [0, 1)
  out[index] = from_float<T>(deviation * sqrtf(-2.0f * logf(u)) * cospif(2.0f * v));
}

MIR_EXPORT int mir_random_normal(int bf16, void* out, size_t total, unsigned long long seed, float deviation,
                                 cudaStream_t stream) {
  if (bf16) LAUNCH_1D(random_normal_kernel, total, (__nv_bfloat16*)out, total, seed, deviation);
  else LAUNCH_1D(random_normal_kernel, total, (float*)out, total, seed, deviation);
  return mir_check_launch("random_normal");
}

// ---- decode batches that run as a captured graph -------------------------------------------------
// Before the layers: where each row's new key/value goes, from its position and block table.  A row
// with a negative position is padding (the batch is smaller than the captured size): no cache write.
__global__ void decode_prepare_kernel(const int* __restrict__ positions, const int* __restrict__ block_table,
                                      int table_width, int page_size, int* __restrict__ slot_mapping,
                                      int* __restrict__ context_lens, int rows) {
  grid_launch_dependents();
  grid_dependency_wait();
  const int row = blockIdx.x * blockDim.x + threadIdx.x;
  if (row >= rows) return;
  const int position = positions[row];
  int slot = -1;
  if (position >= 0) {
    const int block = position / page_size;
    const int page = block < table_width ? block_table[(size_t)row * table_width + block] : -1;
    if (page >= 0) slot = page * page_size + position % page_size;
  }
  slot_mapping[row] = slot;
  context_lens[row] = position >= 0 ? position + 1 : 0;
}

// After sampling: the sampled token is the next step's input, positions move on by one, and the token is
// appended to a log so that several steps can run without the host reading each one.
__global__ void decode_advance_kernel(const int* __restrict__ sampled, int* __restrict__ tokens,
                                      int* __restrict__ positions, int* __restrict__ token_log, int log_steps,
                                      int* __restrict__ step_counter, int rows, int* __restrict__ previous) {
  grid_launch_dependents();
  grid_dependency_wait();
  const int step = *step_counter;
  __syncthreads();
  for (int row = threadIdx.x; row < rows; row += blockDim.x) {
    const int token = sampled[row];
    if (previous) previous[row] = tokens[row];      // the token before the next one, for models that look at pairs
    tokens[row] = token;
    if (positions[row] >= 0) positions[row] += 1;
    if (step < log_steps) token_log[(size_t)step * rows + row] = token;
  }
  if (threadIdx.x == 0) *step_counter = step + 1;
}

MIR_EXPORT int mir_decode_prepare(const int* positions, const int* block_table, int table_width, int page_size,
                                  int* slot_mapping, int* context_lens, int rows, cudaStream_t stream) {
  if (rows <= 0) return MIR_OK;
  return mir_launch("decode_prepare", decode_prepare_kernel, dim3((rows + 127) / 128), dim3(128), 0, stream, 0,
                    positions, block_table, table_width, page_size, slot_mapping, context_lens, rows);
}

MIR_EXPORT int mir_decode_advance(const int* sampled, int* tokens, int* positions, int* token_log, int log_steps,
                                  int* step_counter, int rows, int* previous, cudaStream_t stream) {
  if (rows <= 0) return MIR_OK;
  return mir_launch("decode_advance", decode_advance_kernel, dim3(1), dim3(256), 0, stream, 0, sampled, tokens,
                    positions, token_log, log_steps, step_counter, rows, previous);
}
