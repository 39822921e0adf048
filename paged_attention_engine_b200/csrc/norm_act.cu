// Row-wise kernels of decoders that keep their residual stream in float32: the token
// embedding with a learned position table added, LayerNorm (mean and variance, weight and
// bias), and the activations of a plain two-matrix feed-forward (the exact GELU and its tanh
// form). Statistics, sums and the activation's arithmetic are float32; a result is rounded
// once, to the element type of its output.
#include "common.cuh"

using namespace pae;

namespace {

__device__ __forceinline__ double block_sum(double v, double* scratch) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = (blockDim.x + 31) >> 5;
  __syncthreads();                       // scratch may still be read from the call before
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  double total = 0.0;
  for (int i = 0; i < warps; ++i) total += scratch[i];     // every thread adds in the same order
  return total;
}

// out[t, :] = table[id, :] + positions_table[p, :], float32. A negative id stands for the token
// that the request sampled in the step before (last_token[state_slot[seq_index[t]]]).
template <typename T>
__global__ void embedding_positions_kernel(float* __restrict__ out, const T* __restrict__ table,
                                           const T* __restrict__ position_table, const int* __restrict__ ids,
                                           const int* __restrict__ positions, const int* __restrict__ last_token,
                                           const int* __restrict__ state_slot, const int* __restrict__ seq_index,
                                           int rows, int max_positions, int width, float position_scale) {
  dependent_launch_prologue();
  const int t = blockIdx.x;
  int src = ids[t];
  if (src < 0 && last_token != nullptr) src = last_token[state_slot[seq_index[t]]];
  const int p = positions[t];
  const bool ok = src >= 0 && src < rows;
  const bool pos_ok = p >= 0 && p < max_positions;
  const T* from = table + (size_t)(ok ? src : 0) * width;
  const T* pos = position_table + (size_t)(pos_ok ? p : 0) * width;
  float* to = out + (size_t)t * width;
  for (int i = threadIdx.x; i < width; i += blockDim.x)
    to[i] = (ok ? to_float(from[i]) : 0.f) + (pos_ok ? position_scale * to_float(pos[i]) : 0.f);
}

// y = (x - mean) / sqrt(var + eps) * w + b with var the mean of the squared deviations. One block
// per row, three passes over a row that stays in L1; the sums' order depends on the width only.
template <typename TI, typename TO>
__global__ void layer_norm_kernel(TO* __restrict__ out, const TI* __restrict__ x, const float* __restrict__ weight,
                                  const float* __restrict__ bias, int width, float eps) {
  dependent_launch_prologue();
  __shared__ double scratch[32];
  const TI* row = x + (size_t)blockIdx.x * width;
  // The two sums are double: they cost nothing beside the row's traffic, and the mean and the
  // variance then carry no error of their own into every element of the row.
  double sum = 0.0;
  for (int i = threadIdx.x; i < width; i += blockDim.x) sum += (double)to_float(row[i]);
  const float mean = (float)(block_sum(sum, scratch) / (double)width);
  double squares = 0.0;
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    const double dev = (double)to_float(row[i]) - (double)mean;
    squares = fma(dev, dev, squares);
  }
  const float inv = (float)(1.0 / sqrt(block_sum(squares, scratch) / (double)width + (double)eps));
  TO* to = out + (size_t)blockIdx.x * width;
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    float v = (to_float(row[i]) - mean) * inv * weight[i];
    if (bias != nullptr) v += bias[i];
    to[i] = from_float<TO>(v);
  }
}

// kind 0: 0.5 z (1 + erf(z / sqrt 2)); kind 1: 0.5 z (1 + tanh(sqrt(2/pi) (z + 0.044715 z^3))).
template <typename T>
__global__ void gelu_kernel(T* __restrict__ out, const T* __restrict__ x, long long total, int kind) {
  dependent_launch_prologue();
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const float z = to_float(x[i]);
  float y;
  if (kind == 0)
    y = 0.5f * z * (1.f + erff(z * 0.70710678118654752440f));
  else
    y = 0.5f * z * (1.f + tanhf(0.79788456080286535588f * (z + 0.044715f * z * z * z)));
  out[i] = from_float<T>(y);
}

int row_threads(int width) { return width >= 2048 ? 512 : (width >= 1024 ? 256 : (width >= 256 ? 128 : 64)); }

}  // namespace

PAE_EXPORT int pae_embedding_positions(float* out, const void* table, const void* position_table, const int* ids,
                                       const int* positions, const int* last_token, const int* state_slot,
                                       const int* seq_index, int n, int rows, int max_positions, int width,
                                       float position_scale, int dtype, void* stream) {
  if (n == 0) return 0;
  cudaStream_t s = (cudaStream_t)stream;
  const int threads = row_threads(width);
  if (dtype == kF32)
    launch_kernel(embedding_positions_kernel<float>, n, threads, 0, s, out, (const float*)table, (const float*)position_table,
                  ids, positions, last_token, state_slot, seq_index, rows, max_positions, width, position_scale);
  else if (dtype == kBF16)
    launch_kernel(embedding_positions_kernel<__nv_bfloat16>, n, threads, 0, s, out, (const __nv_bfloat16*)table,
                  (const __nv_bfloat16*)position_table, ids, positions, last_token, state_slot, seq_index, rows,
                  max_positions, width, position_scale);
  else
    return fail(1, "embedding_positions: unknown dtype %d", dtype);
  return check_launch("embedding_positions");
}

// x float32 or bfloat16 [rows, width] -> out float32 or bfloat16; weight, bias (may be null) float32.
PAE_EXPORT int pae_layer_norm(void* out, const void* x, const float* weight, const float* bias, int rows, int width,
                              float eps, int in_dtype, int out_dtype, void* stream) {
  if (rows == 0 || width == 0) return 0;
  cudaStream_t s = (cudaStream_t)stream;
  const int threads = row_threads(width);
  using bf = __nv_bfloat16;
  const int key = in_dtype * 10 + out_dtype;
  if (key == 0)
    launch_kernel(layer_norm_kernel<float, float>, rows, threads, 0, s, (float*)out, (const float*)x, weight, bias, width, eps);
  else if (key == 1)
    launch_kernel(layer_norm_kernel<float, bf>, rows, threads, 0, s, (bf*)out, (const float*)x, weight, bias, width, eps);
  else if (key == 10)
    launch_kernel(layer_norm_kernel<bf, float>, rows, threads, 0, s, (float*)out, (const bf*)x, weight, bias, width, eps);
  else if (key == 11)
    launch_kernel(layer_norm_kernel<bf, bf>, rows, threads, 0, s, (bf*)out, (const bf*)x, weight, bias, width, eps);
  else
    return fail(1, "layer_norm: element types in=%d out=%d are not supported", in_dtype, out_dtype);
  return check_launch("layer_norm");
}

PAE_EXPORT int pae_gelu(void* out, const void* x, long long total, int kind, int dtype, void* stream) {
  if (total == 0) return 0;
  if (kind != 0 && kind != 1) return fail(2, "gelu: kind %d (0: erf, 1: tanh)", kind);
  cudaStream_t s = (cudaStream_t)stream;
  const unsigned blocks = (unsigned)((total + 255) / 256);
  if (dtype == kF32)
    launch_kernel(gelu_kernel<float>, blocks, 256, 0, s, (float*)out, (const float*)x, total, kind);
  else if (dtype == kBF16)
    launch_kernel(gelu_kernel<__nv_bfloat16>, blocks, 256, 0, s, (__nv_bfloat16*)out, (const __nv_bfloat16*)x, total, kind);
  else
    return fail(1, "gelu: unknown dtype %d", dtype);
  return check_launch("gelu");
}

PAE_DEFINE_LAST_ERROR()
