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
// the latent times the value expansion. Two kernels: on the CUDA cores, any sizes, float32 or
// bfloat16 (a float32 product sums in double as the plain product does); and for bfloat16 with K a
// multiple of 16 and 16-byte aligned heads on tensor cores (mma.sync m16n8k16, float32
// accumulation, 64 tokens x 64 outputs a block). An output element sums its K products in the
// same order whatever else is in the batch.
#include "attention_mma.cuh"

using namespace pae;
using namespace pae_attention;

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

// 64 tokens x 64 outputs of one head per block; a warp owns 16 tokens. K goes through shared
// memory 32 channels at a time (rows padded by 16 bytes: conflict-free ldmatrix), two stages.
constexpr int TM = 64, TN = 64, TK = 32, ROW_BYTES = TK * 2 + 16;

__global__ void __launch_bounds__(128) linear_heads_mma_kernel(__nv_bfloat16* __restrict__ out, const __nv_bfloat16* __restrict__ x,
                                                               const __nv_bfloat16* __restrict__ w, int M, int N, int K, int tail,
                                                               long long x_ld, int x_hs, long long o_ld, int o_hs) {
  dependent_launch_prologue();
  __shared__ __align__(128) uint8_t tiles[2][(TM + TN) * ROW_BYTES];
  const int h = blockIdx.z, m0 = blockIdx.y * TM, n0 = blockIdx.x * TN;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const __nv_bfloat16* xh = x + (size_t)h * x_hs;
  const __nv_bfloat16* wh = w + (size_t)h * N * K;
  __nv_bfloat16* oh = out + (size_t)h * o_hs;
  // a thread copies one 16-byte chunk of two rows of each operand per stage: 64 rows x 4 chunks
  const int l_row = tid >> 2, l_chunk = tid & 3;
  auto fetch = [&](int stage, int k0) {
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int r = l_row + half * 32;
      uint8_t* a_dst = tiles[stage] + r * ROW_BYTES + l_chunk * 16;
      uint8_t* b_dst = tiles[stage] + (TM + r) * ROW_BYTES + l_chunk * 16;
      const bool k_ok = k0 + l_chunk * 8 < K;
      if (m0 + r < M && k_ok) cp_async16(smem_u32(a_dst), xh + (size_t)(m0 + r) * x_ld + k0 + l_chunk * 8);
      else *(uint4*)a_dst = make_uint4(0, 0, 0, 0);
      if (n0 + r < N && k_ok) cp_async16(smem_u32(b_dst), wh + (size_t)(n0 + r) * K + k0 + l_chunk * 8);
      else *(uint4*)b_dst = make_uint4(0, 0, 0, 0);
    }
  };
  float acc[TN / 8][4];
#pragma unroll
  for (int n = 0; n < TN / 8; ++n) acc[n][0] = acc[n][1] = acc[n][2] = acc[n][3] = 0.f;
  const int steps = (K + TK - 1) / TK;
  const int mid = lane >> 3, r8 = lane & 7;
  fetch(0, 0);
  cp_async_commit();
  for (int s = 0; s < steps; ++s) {
    if (s + 1 < steps) fetch((s + 1) & 1, (s + 1) * TK);
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();
    const uint32_t base = smem_u32(tiles[s & 1]);
#pragma unroll
    for (int kk = 0; kk < TK / 16; ++kk) {
      uint32_t a[4];
      ldmatrix_x4(a, base + (warp * 16 + ((lane >> 3) & 1) * 8 + r8) * ROW_BYTES + (kk * 2 + (lane >> 4)) * 16);
#pragma unroll
      for (int n = 0; n < TN / 16; ++n) {
        uint32_t b[4];
        ldmatrix_x4(b, base + (TM + n * 16 + (mid >> 1) * 8 + r8) * ROW_BYTES + (kk * 2 + (mid & 1)) * 16);
        mma_16816(acc[2 * n], a, b[0], b[1]);
        mma_16816(acc[2 * n + 1], a, b[2], b[3]);
      }
    }
    __syncthreads();
  }
  cp_async_wait<0>();
  const int c2 = (lane & 3) * 2;
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const int m = m0 + warp * 16 + (lane >> 2) + half * 8;
    if (m >= M) continue;
#pragma unroll
    for (int n = 0; n < TN / 8; ++n) {
      const int col = n0 + n * 8 + c2;
      if (col < N) oh[(size_t)m * o_ld + col] = __float2bfloat16_rn(acc[n][half * 2]);
      if (col + 1 < N) oh[(size_t)m * o_ld + col + 1] = __float2bfloat16_rn(acc[n][half * 2 + 1]);
    }
  }
  if (blockIdx.x == 0 && tail > 0)
    for (int e = tid; e < TM * tail; e += 128) {
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
  cudaStream_t s = (cudaStream_t)stream;
  using bf = __nv_bfloat16;
  if (dtype == kBF16 && k % 16 == 0 && x_ld % 8 == 0 && x_hs % 8 == 0 && (((uintptr_t)x | (uintptr_t)w) & 15) == 0 &&
      (tokens + TM - 1) / TM <= 65535) {
    dim3 tiles((n + TN - 1) / TN, (tokens + TM - 1) / TM, heads);
    launch_kernel(linear_heads_mma_kernel, tiles, 128, 0, s, (bf*)out, (const bf*)x, (const bf*)w, tokens, n, k, tail, x_ld, x_hs,
                  o_ld, o_hs);
    return check_launch("linear_heads");
  }
  dim3 grid((n + BN - 1) / BN, (tokens + BM - 1) / BM, heads);
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
