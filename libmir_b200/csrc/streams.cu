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
//   streams_write_norm  that update and the layer norm of the next reader's mix of the new streams in one pass over a
//                   token: the streams are read once and written once, the mix never leaves the chip
//   streams_spread  every stream starts as the embedding's row;  streams_sum  their sum
// Sums run in a fixed order (streams ascending; the row's sums by a fixed tree over a block whose size depends on the
// width alone), so a token's result never depends on what else is in the step.
#include "common.cuh"

using namespace mir;

namespace {

constexpr int kMaxStreams = 16;

// V columns a thread and access: 4 where the width is a multiple of 4 (16-byte loads; 8- or 16-byte stores), else 1.
template <typename T, int V>
__device__ __forceinline__ void store_columns(T* dst, const float (&values)[V]) {
  if constexpr (V == 4 && sizeof(T) == 2) {
    const __nv_bfloat162 low = __floats2bfloat162_rn(values[0], values[1]), high = __floats2bfloat162_rn(values[2], values[3]);
    uint2 packed;
    packed.x = *reinterpret_cast<const uint32_t*>(&low);
    packed.y = *reinterpret_cast<const uint32_t*>(&high);
    *reinterpret_cast<uint2*>(dst) = packed;
  } else if constexpr (V == 4) {
    *reinterpret_cast<float4*>(dst) = make_float4(values[0], values[1], values[2], values[3]);
  } else {
    dst[0] = from_float<T>(values[0]);
  }
}

// A block's sum through one barrier: the warps' sums side by side in `slots` (32 floats that nothing else uses), then
// every thread adds them in the warps' order.  The result depends on the values and on blockDim alone.
__device__ __forceinline__ float block_sum_once(float v, float* slots) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  if (lane == 0) slots[warp] = v;
  __syncthreads();
  float total = 0.0f;
  for (int w = 0; w < warps; ++w) total += slots[w];
  return total;
}

// The second and third pass of a layer norm over the row in shared memory (its sum is known): mean, variance, result.
// A thread reads back only the columns it wrote itself, so the two sums' barriers are the only ones (`scratch`: 64
// floats, one half per sum).
template <typename T, int V>
__device__ __forceinline__ void norm_row(const float* row_values, float sum, float* scratch, const float* __restrict__ weight,
                                         const float* __restrict__ bias, T* __restrict__ dst, int width, float eps) {
  const float mean = block_sum_once(sum, scratch) / (float)width;
  float squares = 0.0f;
  for (int c = threadIdx.x * V; c < width; c += blockDim.x * V) {
#pragma unroll
    for (int v = 0; v < V; ++v) {
      const float d = row_values[c + v] - mean;
      squares = fmaf(d, d, squares);
    }
  }
  const float inverse = rsqrtf(block_sum_once(squares, scratch + 32) / (float)width + eps);
  for (int c = threadIdx.x * V; c < width; c += blockDim.x * V) {
    float values[V];
    alignas(16) float w[V], b[V];
    if constexpr (V == 4) {
      *reinterpret_cast<float4*>(w) = __ldg(reinterpret_cast<const float4*>(weight + c));
      *reinterpret_cast<float4*>(b) = bias != nullptr ? __ldg(reinterpret_cast<const float4*>(bias + c)) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    } else {
      w[0] = weight[c];
      b[0] = bias != nullptr ? bias[c] : 0.0f;
    }
#pragma unroll
    for (int v = 0; v < V; ++v) values[v] = fmaf((row_values[c + v] - mean) * inverse, w[v], b[v]);
    store_columns<T, V>(dst + c, values);
  }
}

template <typename T, int V>
__global__ void __launch_bounds__(512, 3) layer_norm_kernel(const float* __restrict__ x, int streams, const float* __restrict__ read,
                                  const float* __restrict__ weight, const float* __restrict__ bias, T* __restrict__ out,
                                  const int* __restrict__ rows, int width, float eps) {
  extern __shared__ float row_values[];            // [width]
  __shared__ float scratch[64];
  grid_launch_dependents();
  grid_dependency_wait();
  const int token = rows != nullptr ? rows[blockIdx.x] : blockIdx.x;
  const int count = read != nullptr ? streams : 1;
  const float* base = x + (size_t)token * count * width;
  float sum = 0.0f;
  for (int c = threadIdx.x * V; c < width; c += blockDim.x * V) {
    float u[V];
#pragma unroll
    for (int v = 0; v < V; ++v) u[v] = 0.0f;
    for (int s = 0; s < count; ++s) {
      alignas(16) float piece[V];
      if constexpr (V == 4) *reinterpret_cast<float4*>(piece) = *reinterpret_cast<const float4*>(base + (size_t)s * width + c);
      else piece[0] = base[(size_t)s * width + c];
      const float factor = read != nullptr ? read[s] : 1.0f;
#pragma unroll
      for (int v = 0; v < V; ++v) u[v] = read != nullptr ? fmaf(factor, piece[v], u[v]) : piece[v];
    }
#pragma unroll
    for (int v = 0; v < V; ++v) {
      row_values[c + v] = u[v];
      sum += u[v];
    }
  }
  norm_row<T, V>(row_values, sum, scratch, weight, bias, out + (size_t)blockIdx.x * width, width, eps);
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

// streams_write and the layer norm of the next sublayer's input in one pass over a token: the S new values of a column
// are written and, still in registers, mixed by `read` into the row that is normed.  V columns a thread and access
// (V = 4 where the width allows 16-byte accesses).  S = 0: any count up to kMaxStreams.
template <typename T, int S, int V>
__global__ void streams_write_norm_kernel(float* __restrict__ x, const float* __restrict__ y,
                                          const float* __restrict__ mix, const float* __restrict__ write,
                                          const float* __restrict__ read, const float* __restrict__ weight,
                                          const float* __restrict__ bias, T* __restrict__ out, int streams_given,
                                          int width, float eps) {
  extern __shared__ float row_values[];            // [width]
  __shared__ float scratch[64];
  __shared__ float m[kMaxStreams * kMaxStreams + 2 * kMaxStreams];
  constexpr int kCount = S > 0 ? S : kMaxStreams;
  const int streams = S > 0 ? S : streams_given;
  grid_launch_dependents();
  grid_dependency_wait();
  for (int i = threadIdx.x; i < streams * streams; i += blockDim.x) m[i] = mix[i];
  for (int i = threadIdx.x; i < streams; i += blockDim.x) {
    m[kMaxStreams * kMaxStreams + i] = write[i];
    m[kMaxStreams * kMaxStreams + kMaxStreams + i] = read[i];
  }
  __syncthreads();
  const size_t token = blockIdx.x;
  float* base = x + token * streams * width;
  const float* branch_row = y + token * width;
  float sum = 0.0f;
  for (int c = threadIdx.x * V; c < width; c += blockDim.x * V) {
    alignas(16) float old[kCount][V];
    alignas(16) float branch[V];
    float mixed[V];
#pragma unroll
    for (int s = 0; s < kCount; ++s) {
      if (s < streams) {
        if (V == 4) *reinterpret_cast<float4*>(old[s]) = *reinterpret_cast<const float4*>(base + (size_t)s * width + c);
        else old[s][0] = base[(size_t)s * width + c];
      }
    }
    if (V == 4) *reinterpret_cast<float4*>(branch) = *reinterpret_cast<const float4*>(branch_row + c);
    else branch[0] = branch_row[c];
#pragma unroll
    for (int v = 0; v < V; ++v) mixed[v] = 0.0f;
#pragma unroll
    for (int t = 0; t < kCount; ++t) {
      if (t < streams) {
        alignas(16) float fresh[V];
#pragma unroll
        for (int v = 0; v < V; ++v) {
          float value = 0.0f;
#pragma unroll
          for (int s = 0; s < kCount; ++s)
            if (s < streams) value = fmaf(m[s * streams + t], old[s][v], value);
          fresh[v] = fmaf(m[kMaxStreams * kMaxStreams + t], branch[v], value);
          mixed[v] = fmaf(m[kMaxStreams * kMaxStreams + kMaxStreams + t], fresh[v], mixed[v]);
        }
        if (V == 4) *reinterpret_cast<float4*>(base + (size_t)t * width + c) = *reinterpret_cast<const float4*>(fresh);
        else base[(size_t)t * width + c] = fresh[0];
      }
    }
#pragma unroll
    for (int v = 0; v < V; ++v) {
      row_values[c + v] = mixed[v];
      sum += mixed[v];
    }
  }
  if (weight == nullptr) {                         // no norm: the mix itself (the sum of the streams at the model's end)
    T* dst = out + token * width;
    for (int c = threadIdx.x * V; c < width; c += blockDim.x * V) {
      float values[V];
#pragma unroll
      for (int v = 0; v < V; ++v) values[v] = row_values[c + v];    // (this thread's own columns)
      store_columns<T, V>(dst + c, values);
    }
    return;
  }
  norm_row<T, V>(row_values, sum, scratch, weight, bias, out + token * width, width, eps);
}

template <typename T, int S, int V>
int launch_write_norm(float* x, const float* y, const float* mix, const float* write, const float* read,
                      const float* weight, const float* bias, T* out, int tokens, int streams, int width, float eps,
                      cudaStream_t stream) {
  const int threads = width >= 4096 ? 512 : 256;
  const size_t smem = (size_t)width * sizeof(float);
  if (smem > 48 * 1024)
    cudaFuncSetAttribute(streams_write_norm_kernel<T, S, V>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  return mir_launch("streams_write_norm", streams_write_norm_kernel<T, S, V>, dim3(tokens), dim3(threads), smem, stream, 0,
                    x, y, mix, write, read, weight, bias, out, streams, width, eps);
}

template <typename T>
int dispatch_write_norm(float* x, const float* y, const float* mix, const float* write, const float* read,
                        const float* weight, const float* bias, T* out, int tokens, int streams, int width, float eps,
                        cudaStream_t stream) {
#define MIR_WRITE_NORM(S, V) \
  return launch_write_norm<T, S, V>(x, y, mix, write, read, weight, bias, out, tokens, streams, width, eps, stream)
  if (width % 4 == 0) {
    switch (streams) {
      case 1: MIR_WRITE_NORM(1, 4);
      case 2: MIR_WRITE_NORM(2, 4);
      case 3: MIR_WRITE_NORM(3, 4);
      case 4: MIR_WRITE_NORM(4, 4);
      case 6: MIR_WRITE_NORM(6, 4);
      case 8: MIR_WRITE_NORM(8, 4);
      default: break;
    }
  }
  MIR_WRITE_NORM(0, 1);
#undef MIR_WRITE_NORM
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
  const bool wide = width % 4 == 0;
  const int threads = width >= 4096 ? 512 : (width >= 1024 || !wide ? 256 : 128);
  const size_t smem = (size_t)width * sizeof(float);
  if (smem > 200 * 1024) { mir_set_error("layer_norm: rows of %d numbers do not fit into shared memory", width); return MIR_BAD_ARGUMENT; }
#define MIR_LAYER_NORM(T, V)                                                                                              \
  do {                                                                                                                    \
    if (smem > 48 * 1024)                                                                                                 \
      cudaFuncSetAttribute(layer_norm_kernel<T, V>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);              \
    return mir_launch("layer_norm", layer_norm_kernel<T, V>, dim3(n_rows), dim3(threads), smem, stream, 0, x, streams, read, \
                      weight, bias, (T*)out, rows, width, eps);                                                          \
  } while (0)
  if (bf16) {
    if (wide) MIR_LAYER_NORM(__nv_bfloat16, 4);
    MIR_LAYER_NORM(__nv_bfloat16, 1);
  }
  if (wide) MIR_LAYER_NORM(float, 4);
  MIR_LAYER_NORM(float, 1);
#undef MIR_LAYER_NORM
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

// mir_streams_write, and out [tokens, width] = the layer norm (weight, bias or null, eps) of the mix sum_s read[s] x_s of
// the streams as they are after the update; out in bfloat16 or 32-bit.  weight null: out is the mix itself.
MIR_EXPORT int mir_streams_write_norm(int bf16, float* x, const float* y, const float* mix, const float* write,
                                      const float* read, const float* weight, const float* bias, void* out, int tokens,
                                      int streams, int width, float eps, cudaStream_t stream) {
  if (tokens == 0) return MIR_OK;
  if (tokens < 0 || width <= 0 || streams <= 0 || streams > kMaxStreams) {
    mir_set_error("streams_write_norm: bad sizes (tokens %d, width %d, streams %d of at most %d)", tokens, width, streams,
                  kMaxStreams);
    return MIR_BAD_ARGUMENT;
  }
  if ((size_t)width * sizeof(float) > 200 * 1024) {
    mir_set_error("streams_write_norm: rows of %d numbers do not fit into shared memory", width);
    return MIR_BAD_ARGUMENT;
  }
  if (bf16)
    return dispatch_write_norm<__nv_bfloat16>(x, y, mix, write, read, weight, bias, (__nv_bfloat16*)out, tokens, streams,
                                              width, eps, stream);
  return dispatch_write_norm<float>(x, y, mix, write, read, weight, bias, (float*)out, tokens, streams, width, eps, stream);
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
