// One matrix product per head: out[t, h, 0..N) = w[h] (N x K) . x[t, h, 0..K), for activations and
// outputs whose heads lie at a stride inside a token's row (a head's leading channels are the
// operand; the `tail` channels behind them are copied through unchanged behind the product):
//
//   x   element (t, h, k) at x[t * x_ld + h * x_hs + k]          k < K + tail
//   out element (t, h, n) at out[t * o_ld + h * o_hs + n]        n < N + tail
//   w   [heads, N, K], row-major
//
// Latent attention uses it twice: the queries' unrotated channels times the transposed key
// expansion (the rotated channels pass through as the tail), and the attention's output over
// the latent times the value expansion. On the CUDA cores, any sizes, float32 or bfloat16; a
// float32 product sums in double as the plain product does. An output element sums its K
// products in the same order whatever else is in the batch.
#include "common.cuh"

using namespace pae;

namespace {

constexpr int BM = 32, BN = 32, BK = 16;      // 256 threads, 2 x 2 outputs each

template <typename T, typename TAcc>
__global__ void __launch_bounds__(256) linear_heads_kernel(T* __restrict__ out, const T* __restrict__ x, const T* __restrict__ w,
                                                           int M, int N, int K, int tail, long long x_ld, int x_hs,
                                                           long long o_ld, int o_hs) {
  dependent_launch_prologue();
  __shared__ float xs[BK][BM + 1];
  __shared__ float ws[BK][BN + 1];
  const int h = blockIdx.z, m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  const int tid = threadIdx.x, tx = tid % 16, ty = tid / 16;
  const T* xh = x + (size_t)h * x_hs;
  const T* wh = w + (size_t)h * N * K;
  T* oh = out + (size_t)h * o_hs;
  TAcc acc[2][2] = {{(TAcc)0, (TAcc)0}, {(TAcc)0, (TAcc)0}};
  for (int k0 = 0; k0 < K; k0 += BK) {
    for (int e = tid; e < BM * BK; e += 256) {
      const int r = e / BK, k = e - r * BK;
      xs[k][r] = (m0 + r < M && k0 + k < K) ? to_float(xh[(size_t)(m0 + r) * x_ld + k0 + k]) : 0.f;
      ws[k][r] = (n0 + r < N && k0 + k < K) ? to_float(wh[(size_t)(n0 + r) * K + k0 + k]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < BK; ++k) {
      const TAcc a0 = (TAcc)xs[k][ty * 2], a1 = (TAcc)xs[k][ty * 2 + 1];
      const TAcc b0 = (TAcc)ws[k][tx * 2], b1 = (TAcc)ws[k][tx * 2 + 1];
      acc[0][0] = fma(a0, b0, acc[0][0]);
      acc[0][1] = fma(a0, b1, acc[0][1]);
      acc[1][0] = fma(a1, b0, acc[1][0]);
      acc[1][1] = fma(a1, b1, acc[1][1]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const int m = m0 + ty * 2 + i, n = n0 + tx * 2 + j;
      if (m < M && n < N) oh[(size_t)m * o_ld + n] = from_float<T>((float)acc[i][j]);
    }
  if (blockIdx.x == 0 && tail > 0)
    for (int e = tid; e < BM * tail; e += 256) {
      const int r = e / tail, c = e - r * tail;
      if (m0 + r < M) oh[(size_t)(m0 + r) * o_ld + N + c] = xh[(size_t)(m0 + r) * x_ld + K + c];
    }
}

}  // namespace

PAE_EXPORT int pae_linear_heads(void* out, const void* x, const void* w, int tokens, int heads, int n, int k, int tail,
                                long long x_ld, int x_hs, long long o_ld, int o_hs, int dtype, void* stream) {
  if (tokens == 0 || heads == 0) return 0;
  if (n < 1 || k < 1 || tail < 0) return fail(2, "linear_heads: a product of %d x %d with a tail of %d", n, k, tail);
  if (heads > 65535 || (tokens + BM - 1) / BM > 65535) return fail(3, "linear_heads: %d heads x %d tokens exceed one launch", heads, tokens);
  dim3 grid((n + BN - 1) / BN, (tokens + BM - 1) / BM, heads);
  cudaStream_t s = (cudaStream_t)stream;
  using bf = __nv_bfloat16;
  if (dtype == kF32)
    launch_kernel(linear_heads_kernel<float, double>, grid, 256, 0, s, (float*)out, (const float*)x, (const float*)w, tokens, n, k,
                  tail, x_ld, x_hs, o_ld, o_hs);
  else if (dtype == kBF16)
    launch_kernel(linear_heads_kernel<bf, float>, grid, 256, 0, s, (bf*)out, (const bf*)x, (const bf*)w, tokens, n, k, tail, x_ld,
                  x_hs, o_ld, o_hs);
  else
    return fail(1, "linear_heads: unknown dtype %d", dtype);
  return check_launch("linear_heads");
}

PAE_DEFINE_LAST_ERROR()
