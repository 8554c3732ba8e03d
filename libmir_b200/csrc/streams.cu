// Layer norm with weight and bias, and a residual kept as several streams (hyper-connections).
//
// The residual of such a model is S copies per token, x [tokens, S, width] 32-bit.  A sublayer reads one mix of them,
// u = sum_s read[s] x_s, through its norm; its result y then goes back into every stream at once, from the old ones:
//     x_t <- sum_s mix[s, t] x_s + write[t] y          (mix is indexed [from, to])
// At the end the model's residual is the sum of the streams.
//
//   layer_norm      out = (u - mean) / sqrt(var + eps) * w + b, var the mean of the squared deviations (two passes over
//                   the row, which stays in shared memory), u a plain 32-bit row or the mix above of a token's streams
//                   formed on the way in; optional row gather; result in the engine's type
//   streams_write   the update above, in place: a thread takes one column of one token, reads its S old values and
//                   writes the S new ones
//   streams_spread  every stream starts as the embedding's row;  streams_sum  their sum
// Sums run in a fixed order (streams ascending; the row's sums by a fixed tree over a block whose size depends on the
// width alone), so a token's result never depends on what else is in the step.
#include "common.cuh"

using namespace mir;

namespace {

constexpr int kMaxStreams = 16;

template <typename T>
__global__ void layer_norm_kernel(const float* __restrict__ x, int streams, const float* __restrict__ read,
                                  const float* __restrict__ weight, const float* __restrict__ bias, T* __restrict__ out,
                                  const int* __restrict__ rows, int width, float eps) {
  extern __shared__ float row_values[];            // [width]
  __shared__ float scratch[32];
  grid_launch_dependents();
  grid_dependency_wait();
  const int token = rows != nullptr ? rows[blockIdx.x] : blockIdx.x;
  float sum = 0.0f;
  if (read != nullptr) {
    const float* base = x + (size_t)token * streams * width;
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
      float u = 0.0f;
      for (int s = 0; s < streams; ++s) u = fmaf(read[s], base[(size_t)s * width + c], u);
      row_values[c] = u;
      sum += u;
    }
  } else {
    const float* base = x + (size_t)token * width;
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
      const float u = base[c];
      row_values[c] = u;
      sum += u;
    }
  }
  const float mean = block_sum(sum, scratch) / (float)width;
  float squares = 0.0f;
  for (int c = threadIdx.x; c < width; c += blockDim.x) {
    const float d = row_values[c] - mean;
    squares = fmaf(d, d, squares);
  }
  const float inverse = rsqrtf(block_sum(squares, scratch) / (float)width + eps);
  T* dst = out + (size_t)blockIdx.x * width;
  for (int c = threadIdx.x; c < width; c += blockDim.x) {
    float v = (row_values[c] - mean) * inverse * weight[c];
    if (bias != nullptr) v += bias[c];
    dst[c] = from_float<T>(v);
  }
}

__global__ void streams_write_kernel(float* __restrict__ x, const float* __restrict__ y, const float* __restrict__ mix,
                                     const float* __restrict__ write, int streams, int width, size_t total) {
  __shared__ float m[kMaxStreams * kMaxStreams + kMaxStreams];
  grid_launch_dependents();
  grid_dependency_wait();
  for (int i = threadIdx.x; i < streams * streams; i += blockDim.x) m[i] = mix[i];
  for (int i = threadIdx.x; i < streams; i += blockDim.x) m[kMaxStreams * kMaxStreams + i] = write[i];
  __syncthreads();
  const size_t index = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (index >= total) return;
  const size_t token = index / width;
  const int c = (int)(index - token * width);
  float* base = x + token * streams * width + c;
  float old[kMaxStreams];
#pragma unroll
  for (int s = 0; s < kMaxStreams; ++s) old[s] = s < streams ? base[(size_t)s * width] : 0.0f;
  const float branch = y[index];
#pragma unroll
  for (int t = 0; t < kMaxStreams; ++t) {
    if (t >= streams) break;
    float v = 0.0f;
#pragma unroll
    for (int s = 0; s < kMaxStreams; ++s)
      if (s < streams) v = fmaf(m[s * streams + t], old[s], v);
    base[(size_t)t * width] = fmaf(m[kMaxStreams * kMaxStreams + t], branch, v);
  }
}

__global__ void streams_spread_kernel(const float* __restrict__ x, float* __restrict__ out, int streams, int width,
                                      size_t total) {
  grid_launch_dependents();
  grid_dependency_wait();
  const size_t index = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (index >= total) return;
  const size_t token = index / width;
  const int c = (int)(index - token * width);
  const float v = x[index];
  for (int s = 0; s < streams; ++s) out[(token * streams + s) * width + c] = v;
}

__global__ void streams_sum_kernel(const float* __restrict__ x, float* __restrict__ out, int streams, int width,
                                   size_t total) {
  grid_launch_dependents();
  grid_dependency_wait();
  const size_t index = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (index >= total) return;
  const size_t token = index / width;
  const int c = (int)(index - token * width);
  float v = 0.0f;
  for (int s = 0; s < streams; ++s) v += x[(token * streams + s) * width + c];
  out[index] = v;
}

}  // namespace

// x: 32-bit rows [tokens, width], or with `read` ([streams] 32-bit) the streams [tokens, streams, width] whose mix is
// normed.  rows (or null): which tokens, in the order of the result's rows.  bias may be null.
MIR_EXPORT int mir_layer_norm(int bf16, const float* x, int streams, const float* read, const float* weight,
                              const float* bias, void* out, const int* rows, int n_rows, int width, float eps,
                              cudaStream_t stream) {
  if (n_rows == 0) return MIR_OK;
  if (n_rows < 0 || width <= 0 || (read != nullptr && (streams <= 0 || streams > kMaxStreams))) {
    mir_set_error("layer_norm: bad sizes (rows %d, width %d, streams %d)", n_rows, width, streams);
    return MIR_BAD_ARGUMENT;
  }
  const int threads = width >= 2048 ? 512 : 256;
  const size_t smem = (size_t)width * sizeof(float);
  if (smem > 200 * 1024) { mir_set_error("layer_norm: rows of %d numbers do not fit into shared memory", width); return MIR_BAD_ARGUMENT; }
  if (bf16) {
    if (smem > 48 * 1024)
      cudaFuncSetAttribute(layer_norm_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    return mir_launch("layer_norm", layer_norm_kernel<__nv_bfloat16>, dim3(n_rows), dim3(threads), smem, stream, 0, x,
                      streams, read, weight, bias, (__nv_bfloat16*)out, rows, width, eps);
  }
  if (smem > 48 * 1024)
    cudaFuncSetAttribute(layer_norm_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  return mir_launch("layer_norm", layer_norm_kernel<float>, dim3(n_rows), dim3(threads), smem, stream, 0, x, streams, read,
                    weight, bias, (float*)out, rows, width, eps);
}

// x [tokens, streams, width] in place; y [tokens, width]; mix [streams, streams] indexed [from, to]; write [streams].
MIR_EXPORT int mir_streams_write(float* x, const float* y, const float* mix, const float* write, int tokens, int streams,
                                 int width, cudaStream_t stream) {
  if (tokens == 0) return MIR_OK;
  if (tokens < 0 || width <= 0 || streams <= 0 || streams > kMaxStreams) {
    mir_set_error("streams_write: bad sizes (tokens %d, width %d, streams %d of at most %d)", tokens, width, streams,
                  kMaxStreams);
    return MIR_BAD_ARGUMENT;
  }
  const size_t total = (size_t)tokens * width;
  return mir_launch("streams_write", streams_write_kernel, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, stream, 0,
                    x, y, mix, write, streams, width, total);
}

MIR_EXPORT int mir_streams_spread(const float* x, float* out, int tokens, int streams, int width, cudaStream_t stream) {
  if (tokens == 0) return MIR_OK;
  if (tokens < 0 || width <= 0 || streams <= 0) { mir_set_error("streams_spread: bad sizes"); return MIR_BAD_ARGUMENT; }
  const size_t total = (size_t)tokens * width;
  return mir_launch("streams_spread", streams_spread_kernel, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, stream,
                    0, x, out, streams, width, total);
}

MIR_EXPORT int mir_streams_sum(const float* x, float* out, int tokens, int streams, int width, cudaStream_t stream) {
  if (tokens == 0) return MIR_OK;
  if (tokens < 0 || width <= 0 || streams <= 0) { mir_set_error("streams_sum: bad sizes"); return MIR_BAD_ARGUMENT; }
  const size_t total = (size_t)tokens * width;
  return mir_launch("streams_sum", streams_sum_kernel, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, stream, 0, x,
                    out, streams, width, total);
}
