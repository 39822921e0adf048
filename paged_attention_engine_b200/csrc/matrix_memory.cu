// The matrix memory of xLSTM (mLSTM): a recurrent mixer whose state per head is a d x dv matrix
// S, a vector n of d and a running maximum m of the gates' logarithms. Per token, with the log
// input gate i and the log forget gate f (both capped: i = cap tanh(a / cap), f = logsigmoid(cap
// tanh(b / cap)) from the pre-activations a, b with their biases):
//
//   m' = max(f + m, i)                      (m starts at 0)
//   S' = exp(f + m - m') S + exp(i - m') k v^T
//   n' = exp(f + m - m') n + exp(i - m') k
//   o  = S'^T q / (max(|n' . q|, exp(-m')) + 1e-6)            (q already scaled by d^-1/2)
//
// `scan` walks a request's tokens in order from and into its state slot. The state is stored
// as the augmented matrix [d][dv + 1] (column dv is n) followed by m, float32. A block owns one
// (request, head, range of value columns); thread j keeps column j of S in shared memory (bank j:
// no conflicts), and the last thread of every block keeps the column n, so n . q falls out of the
// same loop as S^T q and every block can divide by itself. The tokens' q, k, v and gates come in
// tiles of 16 tokens; the gates' transcendental functions are computed once per tile in parallel.
// A token's arithmetic is the same instructions in the same order wherever a prompt was cut,
// so the state is carried bit for bit across portions.
//
// `output` divides every head's o by its root mean square, multiplies by a weight and by the
// sigmoid of the gate projection, and rounds to the engine's element type.
#include "common.cuh"

using namespace pae;

namespace {

constexpr int TILE = 16;

struct Scan {
  float* o;               // [tokens, heads, dv]
  float* state;           // [slots, heads, d * (dv + 1) + 1]
  float* carry;           // [requests, heads, d + 1]: the new n and m, put into the state by `commit`
  const float* proj;      // [tokens, ld]
  const float* i_bias;    // [heads]
  const float* f_bias;    // [heads]
  const int* q_start;
  const int* state_slot;
  int ld, q_off, k_off, v_off, i_off, f_off;
  int heads, d, dv, cols;      // cols: value columns per block
  float cap, q_scale;
};

__global__ void matrix_memory_scan_kernel(const Scan p) {
  dependent_launch_prologue();
  extern __shared__ float smem[];
  const int split = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int c0 = split * p.cols;
  const int mine = min(p.cols, p.dv - c0);                 // value columns of this block
  const int first = p.q_start[b], count = p.q_start[b + 1] - first;
  if (mine <= 0 || count <= 0) return;
  const int tid = threadIdx.x;
  const int wide = p.cols + 1;                               // shared-memory row: the block's columns, then n
  const int d = p.d, dv = p.dv;
  float* S = smem;                                           // [d][wide]
  float* qs = S + (size_t)d * wide;                          // [TILE][d]
  float* ks = qs + TILE * d;                                 // [TILE][d]
  float* vs = ks + TILE * d;                                 // [TILE][wide]  (column `cols` holds 1)
  float* gi = vs + TILE * wide;                              // [TILE]
  float* gf = gi + TILE;                                     // [TILE]
  float* below = gf + TILE;                                  // [1]
  const size_t per_head = (size_t)d * (dv + 1) + 1;
  float* st = p.state + ((size_t)p.state_slot[b] * p.heads + h) * per_head;
  // thread j < mine: column c0 + j; thread p.cols: the column n. Others only help with loads.
  const bool is_n = tid == p.cols;
  const bool active = tid < mine || is_n;
  const int col = is_n ? dv : c0 + tid;
  if (active)
    for (int i = 0; i < d; ++i) S[(size_t)i * wide + tid] = st[(size_t)i * (dv + 1) + col];
  float m = st[per_head - 1];
  const int threads = blockDim.x;

  for (int t0 = 0; t0 < count; t0 += TILE) {
    const int n_tok = min(TILE, count - t0);
    __syncthreads();                                         // the tile before is used up
    for (int e = tid; e < n_tok * d; e += threads) {
      const int t = e / d, i = e - t * d;
      const float* row = p.proj + (size_t)(first + t0 + t) * p.ld;
      qs[t * d + i] = row[p.q_off + h * d + i] * p.q_scale;
      ks[t * d + i] = row[p.k_off + h * d + i];
    }
    for (int e = tid; e < n_tok * wide; e += threads) {
      const int t = e / wide, j = e - t * wide;
      const float* row = p.proj + (size_t)(first + t0 + t) * p.ld;
      vs[e] = j == p.cols ? 1.f : (j < mine ? row[p.v_off + h * dv + c0 + j] : 0.f);
    }
    if (tid < n_tok) {
      const float* row = p.proj + (size_t)(first + t0 + tid) * p.ld;
      const float a = row[p.i_off + h] + p.i_bias[h], g = row[p.f_off + h] + p.f_bias[h];
      gi[tid] = p.cap * tanhf(a / p.cap);
      const float z = p.cap * tanhf(g / p.cap);
      gf[tid] = z >= 0.f ? -log1pf(expf(-z)) : z - log1pf(expf(z));      // log sigmoid(z)
    }
    __syncthreads();
    for (int t = 0; t < n_tok; ++t) {
      const float li = gi[t], lf = gf[t];
      const float m_new = fmaxf(lf + m, li);
      const float keep = expf(lf + m - m_new), add = expf(li - m_new);
      m = m_new;
      float num = 0.f;
      if (active) {
        const float av = add * vs[t * wide + tid];
        const float* q = qs + t * d;
        const float* k = ks + t * d;
        for (int i = 0; i < d; ++i) {
          const float s = fmaf(keep, S[(size_t)i * wide + tid], k[i] * av);
          S[(size_t)i * wide + tid] = s;
          num = fmaf(s, q[i], num);
        }
      }
      if (is_n) below[0] = fmaxf(fabsf(num), expf(-m)) + 1e-6f;
      __syncthreads();
      if (tid < mine) p.o[((size_t)(first + t0 + t) * p.heads + h) * dv + c0 + tid] = num / below[0];
      __syncthreads();
    }
  }
  // Every block of a head reads n and m of the state when it starts, and blocks start in any
  // order: the new n and m go to `carry`, and a kernel after this one puts them into the state.
  if (tid < mine)
    for (int i = 0; i < d; ++i) st[(size_t)i * (dv + 1) + col] = S[(size_t)i * wide + tid];
  if (split == 0) {
    float* to = p.carry + ((size_t)b * p.heads + h) * (d + 1);
    if (is_n)
      for (int i = 0; i < d; ++i) to[i] = S[(size_t)i * wide + tid];
    if (tid == 0) to[d] = m;
  }
}

__global__ void matrix_memory_commit_kernel(const Scan p) {
  dependent_launch_prologue();
  const int h = blockIdx.x, b = blockIdx.y;
  if (p.q_start[b + 1] - p.q_start[b] <= 0) return;
  const size_t per_head = (size_t)p.d * (p.dv + 1) + 1;
  float* st = p.state + ((size_t)p.state_slot[b] * p.heads + h) * per_head;
  const float* from = p.carry + ((size_t)b * p.heads + h) * (p.d + 1);
  for (int i = threadIdx.x; i < p.d; i += blockDim.x) st[(size_t)i * (p.dv + 1) + p.dv] = from[i];
  if (threadIdx.x == 0) st[per_head - 1] = from[p.d];
}

// out[t, h, :] = o[t, h, :] / sqrt(mean(o[t, h, :]^2) + eps) * weight[h, :] * sigmoid(gate[t, h, :]).
template <typename TO>
__global__ void matrix_memory_output_kernel(TO* __restrict__ out, const float* __restrict__ o, const float* __restrict__ proj,
                                            int ld, int g_off, const float* __restrict__ weight, int heads, int dv, float eps) {
  dependent_launch_prologue();
  const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
  for (int h = warp; h < heads; h += warps) {
    const float* row = o + ((size_t)t * heads + h) * dv;
    double squares = 0.0;
    for (int i = lane; i < dv; i += 32) squares = fma((double)row[i], (double)row[i], squares);
#pragma unroll
    for (int s = 16; s > 0; s >>= 1) squares += __shfl_xor_sync(0xffffffffu, squares, s);
    const float inv = (float)(1.0 / sqrt(squares / (double)dv + (double)eps));
    for (int i = lane; i < dv; i += 32) {
      const float g = proj[(size_t)t * ld + g_off + h * dv + i];
      out[((size_t)t * heads + h) * dv + i] = from_float<TO>(row[i] * inv * weight[h * dv + i] / (1.f + expf(-g)));
    }
  }
}

size_t scan_smem(int d, int cols) {
  const int wide = cols + 1;
  return sizeof(float) * ((size_t)d * wide + 2 * (size_t)TILE * d + (size_t)TILE * wide + 2 * TILE + 4);
}

}  // namespace

// Floats of one head's state: the augmented matrix and the running maximum.
PAE_EXPORT int pae_matrix_memory_state_floats(int d, int dv) { return d * (dv + 1) + 1; }

// The most blocks that a head's value columns may be shared out over (each keeps at least 32).
PAE_EXPORT int pae_matrix_memory_max_splits(int dv) { return dv / 32 > 1 ? dv / 32 : 1; }

// proj float32 [tokens, ld] holds q, k (heads x d), v (heads x dv) and the gates' pre-activations
// (heads each) at the given column offsets; o float32 [tokens, heads * dv] receives the read-outs;
// carry: seqs * heads * (d + 1) floats of scratch. Two launches.
PAE_EXPORT int pae_matrix_memory_scan(float* o, float* state, float* carry, const float* proj, int ld, int q_off, int k_off, int v_off,
                                      int i_off, int f_off, const float* i_bias, const float* f_bias, const int* q_start,
                                      const int* state_slot, int seqs, int heads, int d, int dv, int splits, float cap,
                                      float q_scale, void* stream) {
  if (seqs == 0) return 0;
  if (heads < 1 || d < 1 || dv < 1) return fail(2, "matrix_memory: %d heads of %d x %d", heads, d, dv);
  if (!(cap > 0.f)) return fail(2, "matrix_memory: the gates' cap %g is not positive", (double)cap);
  if (splits < 1 || splits > dv) return fail(2, "matrix_memory: %d splits of %d value columns", splits, dv);
  if (heads > 65535 || seqs > 65535) return fail(3, "matrix_memory: %d heads x %d requests exceed one launch", heads, seqs);
  int cols = (dv + splits - 1) / splits;
  while (cols + 1 > 1024 || scan_smem(d, cols) > 200 * 1024) {        // narrower blocks until one fits
    if (cols == 1) return fail(2, "matrix_memory: heads of %d key channels do not fit shared memory", d);
    cols = (cols + 1) / 2;
  }
  const int blocks = (dv + cols - 1) / cols;
  const size_t smem = scan_smem(d, cols);
  static size_t raised = 48 * 1024;
  if (smem > raised) {
    cudaError_t err = cudaFuncSetAttribute(matrix_memory_scan_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    if (err != cudaSuccess) return fail(100, "matrix_memory: %s", cudaGetErrorString(err));
    raised = 200 * 1024;
  }
  Scan p{o, state, carry, proj, i_bias, f_bias, q_start, state_slot, ld, q_off, k_off, v_off, i_off, f_off, heads, d, dv, cols, cap, q_scale};
  const int threads = ((cols + 1 + 31) / 32) * 32;
  launch_kernel(matrix_memory_scan_kernel, dim3(blocks, heads, seqs), threads, smem, (cudaStream_t)stream, p);
  if (int err = check_launch("matrix_memory_scan")) return err;
  launch_kernel(matrix_memory_commit_kernel, dim3(heads, seqs), 64, 0, (cudaStream_t)stream, p);
  return check_launch("matrix_memory_commit");
}

PAE_EXPORT int pae_matrix_memory_output(void* out, const float* o, const float* proj, int ld, int g_off, const float* weight,
                                        int tokens, int heads, int dv, float eps, int out_dtype, void* stream) {
  if (tokens == 0) return 0;
  cudaStream_t s = (cudaStream_t)stream;
  const int threads = heads >= 4 ? 128 : 32 * heads;
  if (out_dtype == kF32)
    launch_kernel(matrix_memory_output_kernel<float>, tokens, threads, 0, s, (float*)out, o, proj, ld, g_off, weight, heads, dv, eps);
  else if (out_dtype == kBF16)
    launch_kernel(matrix_memory_output_kernel<__nv_bfloat16>, tokens, threads, 0, s, (__nv_bfloat16*)out, o, proj, ld, g_off, weight, heads, dv, eps);
  else
    return fail(1, "matrix_memory_output: unknown dtype %d", out_dtype);
  return check_launch("matrix_memory_output");
}

PAE_DEFINE_LAST_ERROR()
