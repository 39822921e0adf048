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
// same loop as S^T q and every block can divide by itself (head sizes that are multiples of 16 up to
// 128 take a second form of the kernel, further down, with the columns in registers of four threads). The tokens' q, k, v and gates come in
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

__device__ __forceinline__ void cp_async4(float* dst, const float* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_group1() { asm volatile("cp.async.wait_group 1;" ::: "memory"); }

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

// The same recurrence for head sizes known at compile time: a column of S lives in the registers
// of KS = 4 threads, a quarter of its d key channels each (lanes 8 apart, so that neighbouring lanes
// hold neighbouring columns and the state moves in full sectors); a warp owns 8 value columns and
// needs no other warp (every warp keeps a copy of n, spread over its lanes, and sums n . q by
// shuffles, as it sums a column's four partial read-outs), so a token costs no barrier. Four
// times the warps of a thread-per-column form is what a single request's prompt needs: its
// tokens come one after the other, and heads x dv / 8 warps are all the parallelism there is.
// q is used as projected and d^-1/2 multiplies the two sums.
constexpr int KS = 4;

template <int D>
__global__ void __launch_bounds__(128) matrix_memory_scan_columns_kernel(const Scan p) {
  dependent_launch_prologue();
  extern __shared__ __align__(16) float smem[];
  constexpr int NJ = (D + 31) / 32;
  constexpr int PER = D / KS;                                // key channels of a thread
  constexpr int SEG = PER + 4;                               // a part's channels in shared memory, padded: the four parts' 16-byte loads meet no bank twice
  constexpr int ROW = KS * SEG;                              // a token's q (or k) in shared memory
  constexpr int WARP_COLS = 32 / KS;
  const int h = blockIdx.y, b = blockIdx.z;
  const int c0 = blockIdx.x * p.cols;                        // p.cols = 8 x the block's warps
  const int first = p.q_start[b], count = p.q_start[b + 1] - first;
  if (c0 >= p.dv || count <= 0) return;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, threads = blockDim.x;
  const int dv = p.dv, cols = p.cols;
  const int part = lane / WARP_COLS;                         // which quarter of the key channels
  const int local = warp * WARP_COLS + lane % WARP_COLS;     // the column within the block
  const int col = c0 + local;
  const bool has_col = col < dv;
  auto at = [](int i) { return (i / PER) * SEG + i % PER; };  // where key channel i of a token lies in shared memory
  // two stages of a tile: q [TILE][ROW], k [TILE][ROW], v [TILE][cols], log gates i [TILE], f [TILE]
  const int stage_floats = TILE * (2 * ROW + cols) + 2 * TILE;
  const size_t per_head = (size_t)D * (dv + 1) + 1;
  float* st = p.state + ((size_t)p.state_slot[b] * p.heads + h) * per_head;
  // A tile's q, k and v go to shared memory by asynchronous copies, one tile ahead: a block of
  // a few warps cannot hide a trip to memory per element any other way.
  auto issue = [&](int stage, int t0) {
    float* qs = smem + stage * stage_floats;
    float* ks = qs + TILE * ROW;
    float* vs = ks + TILE * ROW;
    const int n_tok = min(TILE, count - t0);
    for (int e = tid; e < n_tok * D; e += threads) {
      const int t = e / D, i = e - t * D;
      const float* row = p.proj + (size_t)(first + t0 + t) * p.ld;
      cp_async4(qs + t * ROW + at(i), row + p.q_off + h * D + i);
      cp_async4(ks + t * ROW + at(i), row + p.k_off + h * D + i);
    }
    for (int e = tid; e < n_tok * cols; e += threads) {
      const int t = e / cols, j = e - t * cols;
      if (c0 + j < dv) cp_async4(vs + e, p.proj + (size_t)(first + t0 + t) * p.ld + p.v_off + h * dv + c0 + j);
    }
  };
  issue(0, 0);
  cp_async_commit();
  float s[PER];
#pragma unroll
  for (int i = 0; i < PER; ++i) s[i] = has_col ? st[(size_t)(part * PER + i) * (dv + 1) + col] : 0.f;
  float n[NJ];
#pragma unroll
  for (int j = 0; j < NJ; ++j) n[j] = lane + 32 * j < D ? st[(size_t)(lane + 32 * j) * (dv + 1) + dv] : 0.f;
  float m = st[per_head - 1];

  for (int t0 = 0, stage = 0; t0 < count; t0 += TILE, stage ^= 1) {
    const int n_tok = min(TILE, count - t0);
    float* qs = smem + stage * stage_floats;
    float* ks = qs + TILE * ROW;
    float* vs = ks + TILE * ROW;
    float* gi = vs + TILE * cols;
    float* gf = gi + TILE;
    if (t0 + TILE < count) issue(stage ^ 1, t0 + TILE);      // that stage was used up before the barrier that ended the last round
    cp_async_commit();
    if (tid < n_tok) {
      const float* row = p.proj + (size_t)(first + t0 + tid) * p.ld;
      const float a = row[p.i_off + h] + p.i_bias[h], g = row[p.f_off + h] + p.f_bias[h];
      gi[tid] = p.cap * tanhf(a / p.cap);
      const float z = p.cap * tanhf(g / p.cap);
      gf[tid] = z >= 0.f ? -log1pf(expf(-z)) : z - log1pf(expf(z));      // log sigmoid(z)
    }
    cp_async_wait_group1();
    __syncthreads();
    for (int t = 0; t < n_tok; ++t) {
      const float li = gi[t], lf = gf[t];
      const float m_new = fmaxf(lf + m, li);
      const float keep = expf(lf + m - m_new), add = expf(li - m_new);
      m = m_new;
      const float* q = qs + t * ROW;
      const float* k = ks + t * ROW;
      float dot = 0.f;
#pragma unroll
      for (int j = 0; j < NJ; ++j) {
        const int i = lane + 32 * j;
        if (i < D) {
          n[j] = fmaf(keep, n[j], add * k[at(i)]);
          dot = fmaf(n[j], q[at(i)], dot);
        }
      }
      dot = warp_sum(dot) * p.q_scale;                        // n . (q / sqrt(d))
      const float below = fmaxf(fabsf(dot), expf(-m)) + 1e-6f;
      const float av = has_col ? add * vs[t * cols + local] : 0.f;
      const float* kp = k + part * SEG;
      const float* qp = q + part * SEG;
      float num[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int i = 0; i < PER; i += 4) {
        const float4 k4 = *(const float4*)(kp + i), q4 = *(const float4*)(qp + i);
        s[i] = fmaf(keep, s[i], k4.x * av);
        s[i + 1] = fmaf(keep, s[i + 1], k4.y * av);
        s[i + 2] = fmaf(keep, s[i + 2], k4.z * av);
        s[i + 3] = fmaf(keep, s[i + 3], k4.w * av);
        num[0] = fmaf(s[i], q4.x, num[0]);
        num[1] = fmaf(s[i + 1], q4.y, num[1]);
        num[2] = fmaf(s[i + 2], q4.z, num[2]);
        num[3] = fmaf(s[i + 3], q4.w, num[3]);
      }
      float total = (num[0] + num[1]) + (num[2] + num[3]);
      total += __shfl_xor_sync(0xffffffffu, total, WARP_COLS);          // the column's other quarters
      total += __shfl_xor_sync(0xffffffffu, total, 2 * WARP_COLS);
      if (has_col && part == 0) p.o[((size_t)(first + t0 + t) * p.heads + h) * dv + col] = total * p.q_scale / below;
    }
    __syncthreads();
  }
  if (has_col) {
#pragma unroll
    for (int i = 0; i < PER; ++i) st[(size_t)(part * PER + i) * (dv + 1) + col] = s[i];
  }
  // every block of a head read n and m of the state when it started: see the kernel above
  if (blockIdx.x == 0 && warp == 0) {
    float* to = p.carry + ((size_t)b * p.heads + h) * (D + 1);
#pragma unroll
    for (int j = 0; j < NJ; ++j)
      if (lane + 32 * j < D) to[lane + 32 * j] = n[j];
    if (lane == 0) to[D] = m;
  }
}

template <int D>
int launch_columns(Scan p, int seqs, int splits, cudaStream_t s) {
  constexpr int WARP_COLS = 32 / KS, ROW = KS * (D / KS + 4);
  const int warps = (p.dv + WARP_COLS - 1) / WARP_COLS;
  int per_block = (warps + splits - 1) / splits;
  per_block = per_block > 4 ? 4 : per_block;
  p.cols = WARP_COLS * per_block;
  const size_t smem = 2 * sizeof(float) * ((size_t)TILE * (2 * ROW + p.cols) + 2 * TILE);
  static bool raised = false;
  if (smem > 48 * 1024 && !raised) {
    cudaError_t err = cudaFuncSetAttribute(matrix_memory_scan_columns_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, 64 * 1024);
    if (err != cudaSuccess) return fail(100, "matrix_memory: %s", cudaGetErrorString(err));
    raised = true;
  }
  launch_kernel(matrix_memory_scan_columns_kernel<D>, dim3((warps + per_block - 1) / per_block, p.heads, seqs), 32 * per_block, smem, s, p);
  return check_launch("matrix_memory_scan");
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
  for (int h = blockIdx.y * warps + warp; h < heads; h += warps * gridDim.y) {
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
  {
    Scan p{o, state, carry, proj, i_bias, f_bias, q_start, state_slot, ld, q_off, k_off, v_off, i_off, f_off, heads, d, dv, 0, cap, q_scale};
    cudaStream_t s = (cudaStream_t)stream;
    int done = -1;
    switch (d) {
#define PAE_COLUMNS(DD) case DD: done = launch_columns<DD>(p, seqs, splits, s); break;
      PAE_COLUMNS(16) PAE_COLUMNS(32) PAE_COLUMNS(48) PAE_COLUMNS(64) PAE_COLUMNS(80) PAE_COLUMNS(96) PAE_COLUMNS(112) PAE_COLUMNS(128)
#undef PAE_COLUMNS
      default: break;
    }
    if (done > 0) return done;
    if (done == 0) {
      launch_kernel(matrix_memory_commit_kernel, dim3(heads, seqs), 64, 0, s, p);
      return check_launch("matrix_memory_commit");
    }
  }
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
  const dim3 grid(tokens, tokens < 64 ? (heads + 3) / 4 : 1);          // few tokens: a warp per head
  if (out_dtype == kF32)
    launch_kernel(matrix_memory_output_kernel<float>, grid, threads, 0, s, (float*)out, o, proj, ld, g_off, weight, heads, dv, eps);
  else if (out_dtype == kBF16)
    launch_kernel(matrix_memory_output_kernel<__nv_bfloat16>, grid, threads, 0, s, (__nv_bfloat16*)out, o, proj, ld, g_off, weight, heads, dv, eps);
  else
    return fail(1, "matrix_memory_output: unknown dtype %d", out_dtype);
  return check_launch("matrix_memory_output");
}

PAE_DEFINE_LAST_ERROR()
