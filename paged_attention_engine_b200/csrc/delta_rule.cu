// The generalized delta rule: a recurrent mixer whose per-head state S [key channel, value
// channel] is carried from token to token in float32.
//
//   w_t = exp(-c * sigmoid(w~_t + w0))                  decay per key channel (c a constant of the design)
//   a_t = sigmoid(a~_t + a_bias)                        removal rate per key channel
//   u_t = k_t / sqrt(sum(k_t^2) + key_eps)              unit key
//   S_t = diag(w_t) S_(t-1) - (a_t * u_t) (u_t^T S_(t-1)) + k_t v_t^T
//   o_t = S_t^T r_t
//
// Both terms read the old state. A column of S (one value channel) never meets another column:
// u^T S and S^T r are sums over key channels only. So a block owns some value channels of one head
// of one request, a thread owns a run of key channels of one value channel in registers, and the
// two sums are reductions over the few neighbouring lanes that share a value channel. A first
// kernel prepares every token's vectors (w, a u, u, k, w r) once per head, in parallel over the
// tokens; the recurrence then takes a portion's tokens in tiles that asynchronous copies bring
// into shared memory one tile ahead, and walks a tile without a block-wide barrier.
// The state is read at the start of a portion and written back at its end, so a prompt cut into
// portions, or decoded token by token, computes bit for bit what the whole prompt computes.
//
// A second kernel finishes the output: each head's o over its root mean square, times a weight,
// times sigmoid of the gate projection, rounded to the engine's element type.
//
// Everything here is float32: the projections come in as float32 rows, the state is float32.
#include "common.cuh"

using namespace pae;

namespace {

struct DeltaParams {
  const float* proj;       // [tokens, ld]: r, k, v, a~, gate at their column offsets
  int ld, r_off, k_off, v_off, a_off;
  const float* w_pre;      // [tokens, heads * d]: w~
  const float* w0;         // [heads * d]
  const float* a_bias;     // [heads * d]
  float* prepared;         // [tokens, heads, 5 dp + 4]: u, w, a u, k, w r (dp floats each, zero past d), c1, c2, -, -
  float* state;            // [slots, heads, d (value channel), d (key channel)]
  float* o;                // [tokens, heads * d]
  const int* q_start;      // [entries + 1]
  const int* state_slot;   // [entries]
  int tokens, heads, d, columns;   // columns: value channels per block
  int tile;                // tokens in shared memory at a time (twice: the tile after is on its way)
  float decay_scale, key_eps;
};

__device__ __forceinline__ float sigmoidf(float x) { return 1.f / (1.f + expf(-x)); }

__device__ __forceinline__ void copy_async4(float* dst, const float* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void copy_async16(float* dst, const float* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void copy_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void copy_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// What the recurrence needs of a token, once per (token, head), by one warp: the decay w, the unit
// key u, a u, k, w r, and the two sums over key channels that the output needs beside the old
// state, c1 = sum(a u r) and c2 = sum(k r). Those two are where r meets k head on, so they
// cancel hardest; they are summed in double and rounded once. A (token, head) is 5 vectors of
// `dp` floats (d of them real, the rest zero) and four more floats (c1, c2, two unused): every
// vector starts on a 16-byte boundary.
__global__ void delta_prepare_kernel(DeltaParams p, int dp) {
  dependent_launch_prologue();
  const int unit = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (unit >= p.tokens * p.heads) return;
  const int lane = threadIdx.x & 31;
  const int t = unit / p.heads, h = unit - t * p.heads, d = p.d;
  const float* row = p.proj + (size_t)t * p.ld;
  float* out = p.prepared + (size_t)unit * (5 * dp + 4);
  float squares = 0.f;
  for (int i = lane; i < d; i += 32) {
    const float k = row[p.k_off + h * d + i];
    squares = fmaf(k, k, squares);
  }
  const float inv = 1.f / sqrtf(warp_sum(squares) + p.key_eps);
  double c1 = 0.0, c2 = 0.0;
  for (int i = lane; i < dp; i += 32) {
    float u = 0.f, w = 0.f, au = 0.f, k = 0.f, wr = 0.f;
    if (i < d) {
      const int c = h * d + i;
      k = row[p.k_off + c];
      const float r = row[p.r_off + c];
      const float a = sigmoidf(row[p.a_off + c] + p.a_bias[c]);
      w = expf(-p.decay_scale * sigmoidf(p.w_pre[(size_t)t * p.heads * d + c] + p.w0[c]));
      u = k * inv;
      au = a * u;
      wr = w * r;
      c1 += (double)au * (double)r;
      c2 += (double)k * (double)r;
    }
    out[i] = u;
    out[dp + i] = w;
    out[2 * dp + i] = au;
    out[3 * dp + i] = k;
    out[4 * dp + i] = wr;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    c1 += __shfl_xor_sync(0xffffffffu, c1, o);
    c2 += __shfl_xor_sync(0xffffffffu, c2, o);
  }
  if (lane < 4) out[5 * dp + lane] = lane == 0 ? (float)c1 : (lane == 1 ? (float)c2 : 0.f);
}

// RPT key channels per thread (a multiple of 4), P threads per value channel (a power of two of at
// most 32). Thread `part` of a value channel owns the key channels (m P + part) 4 + e for m <
// RPT / 4, e < 4: its reads of a vector in shared memory are 16 bytes wide, and the P threads of a
// value channel read P neighbouring 16-byte words (other value channels read the same words), so
// no two lanes meet in a bank.
template <int RPT, int P>
__global__ void __launch_bounds__(1024) delta_scan_kernel(DeltaParams p) {
  dependent_launch_prologue();
  extern __shared__ __align__(16) float smem[];
  const int e = blockIdx.x, h = blockIdx.y, j0 = blockIdx.z * p.columns;
  constexpr int dp = P * RPT;
  const int d = p.d;
  const int tid = threadIdx.x, threads = blockDim.x;
  const int column = tid / P, part = tid % P;
  const int j = j0 + column;
  const bool owns = column < p.columns && j < d;
  const int first = p.q_start[e], count = p.q_start[e + 1] - first;

  // per tile token: u, w, au, k, wr [dp each], (c1, c2, -, -), v [columns, rounded up to 4]; two tiles take turns
  constexpr int vectors = 5 * dp + 4;
  const int per_token = vectors + (p.columns + 3) / 4 * 4;
  const int tile_floats = p.tile * per_token;
  float S[RPT];
  float* mine = p.state + (((size_t)p.state_slot[e] * p.heads + h) * d + (owns ? j : 0)) * d;
#pragma unroll
  for (int rr = 0; rr < RPT; ++rr) {
    const int i = ((rr >> 2) * P + part) * 4 + (rr & 3);
    S[rr] = (owns && i < d) ? mine[i] : 0.f;
  }

  // A token's prepared vectors are one run of 16-byte words; its values of this block's channels a few floats.
  auto fetch = [&](int t0, float* to) {
    const int n = min(p.tile, count - t0);
    constexpr int chunks = vectors / 4;
    const float* from = p.prepared + ((size_t)(first + t0) * p.heads + h) * vectors;
    const float* values = p.proj + (size_t)(first + t0) * p.ld + p.v_off + h * d + j0;
    for (int tok = 0; tok < n; ++tok) {
      for (int at = tid; at < chunks; at += threads) copy_async16(to + 4 * at, from + 4 * at);
      if (tid < p.columns && j0 + tid < d) copy_async4(to + vectors + tid, values + tid);
      to += per_token;
      from += (size_t)p.heads * vectors;
      values += p.ld;
    }
  };

  if (count > 0) fetch(0, smem);
  copy_async_commit();
  int turn = 0;
  for (int t0 = 0; t0 < count; t0 += p.tile, turn ^= 1) {
    const int n = min(p.tile, count - t0);
    if (t0 + p.tile < count) fetch(t0 + p.tile, smem + (turn ^ 1) * tile_floats);
    copy_async_commit();
    copy_async_wait<1>();
    __syncthreads();
    const float* tile = smem + turn * tile_floats;
    float* o_row = p.o + (size_t)(first + t0) * p.heads * d + h * d + j;
    // o = S_new^T r written over the old state: sum(w r S_old) - (u^T S_old) c1 + v c2, so that both
    // sums over the state's registers run side by side and share one round of shuffles.
#pragma unroll 2
    for (int tok = 0; tok < n; ++tok) {
      const float* at = tile + tok * per_token + part * 4;
      float us[4] = {0.f, 0.f, 0.f, 0.f}, rs[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int m = 0; m < RPT / 4; ++m) {
        const float4 u = *(const float4*)(at + m * P * 4);
        const float4 wr = *(const float4*)(at + 4 * dp + m * P * 4);
        us[0] = fmaf(u.x, S[4 * m], us[0]);
        us[1] = fmaf(u.y, S[4 * m + 1], us[1]);
        us[2] = fmaf(u.z, S[4 * m + 2], us[2]);
        us[3] = fmaf(u.w, S[4 * m + 3], us[3]);
        rs[0] = fmaf(wr.x, S[4 * m], rs[0]);
        rs[1] = fmaf(wr.y, S[4 * m + 1], rs[1]);
        rs[2] = fmaf(wr.z, S[4 * m + 2], rs[2]);
        rs[3] = fmaf(wr.w, S[4 * m + 3], rs[3]);
      }
      float us_all = (us[0] + us[1]) + (us[2] + us[3]), rs_all = (rs[0] + rs[1]) + (rs[2] + rs[3]);
#pragma unroll
      for (int o = P >> 1; o > 0; o >>= 1) {
        us_all += __shfl_xor_sync(0xffffffffu, us_all, o);
        rs_all += __shfl_xor_sync(0xffffffffu, rs_all, o);
      }
      const float* tail = tile + tok * per_token + 5 * dp;
      const float v = owns ? tail[4 + column] : 0.f;
#pragma unroll
      for (int m = 0; m < RPT / 4; ++m) {
        const float4 w = *(const float4*)(at + dp + m * P * 4);
        const float4 au = *(const float4*)(at + 2 * dp + m * P * 4);
        const float4 k = *(const float4*)(at + 3 * dp + m * P * 4);
        S[4 * m] = fmaf(k.x, v, fmaf(-au.x, us_all, w.x * S[4 * m]));
        S[4 * m + 1] = fmaf(k.y, v, fmaf(-au.y, us_all, w.y * S[4 * m + 1]));
        S[4 * m + 2] = fmaf(k.z, v, fmaf(-au.z, us_all, w.z * S[4 * m + 2]));
        S[4 * m + 3] = fmaf(k.w, v, fmaf(-au.w, us_all, w.w * S[4 * m + 3]));
      }
      if (owns && part == 0) *o_row = fmaf(v, tail[1], fmaf(-us_all, tail[0], rs_all));
      o_row += p.heads * d;
    }
    __syncthreads();                              // the tile is read; the fetch after next may refill it
  }
  copy_async_wait<0>();
  if (owns) {
#pragma unroll
    for (int rr = 0; rr < RPT; ++rr) {
      const int i = ((rr >> 2) * P + part) * 4 + (rr & 3);
      if (i < d) mine[i] = S[rr];
    }
  }
}

// out[t, h, :] = o[t, h, :] / rms(o[t, h, :]) * weight[h, :] * sigmoid(gate[t, h, :]); a warp per (token, head).
template <typename T>
__global__ void delta_output_kernel(T* __restrict__ out, const float* __restrict__ o, const float* __restrict__ gate,
                                    int gate_ld, const float* __restrict__ weight, int tokens, int heads, int d, float eps) {
  dependent_launch_prologue();
  const int unit = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (unit >= tokens * heads) return;
  const int lane = threadIdx.x & 31;
  const int t = unit / heads, h = unit - t * heads;
  const float* row = o + ((size_t)t * heads + h) * d;
  float squares = 0.f;
  for (int i = lane; i < d; i += 32) squares = fmaf(row[i], row[i], squares);
  const float inv = 1.f / sqrtf(warp_sum(squares) / (float)d + eps);
  for (int i = lane; i < d; i += 32) {
    float v = row[i] * inv;
    if (weight != nullptr) v *= weight[h * d + i];
    if (gate != nullptr) v *= sigmoidf(gate[(size_t)t * gate_ld + h * d + i]);
    out[((size_t)t * heads + h) * d + i] = from_float<T>(v);
  }
}

// out[t, c] = tanh(x[t, offset + c]) for c < width: the activation between the two small matrices
// of the decay's projection.
template <typename T>
__global__ void tanh_columns_kernel(T* __restrict__ out, const float* __restrict__ x, int ld, int offset, int width, long long total) {
  dependent_launch_prologue();
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const long long t = i / width;
  const int c = (int)(i - t * width);
  out[i] = from_float<T>(tanhf(x[t * ld + offset + c]));
}

int pow2_at_least(int n) {
  int p = 1;
  while (p < n) p *= 2;
  return p;
}

}  // namespace

// How a head of size d is laid out: key channels per thread (0: the size is not taken) and threads
// per value channel.
PAE_EXPORT int pae_delta_rule_layout(int d, int* threads_per_column) {
  if (d < 1 || d > 256) return 0;
  // Few key channels per thread: a warp's instructions per token are what a block's time is made
  // of (one token after the other, a handful of warps an SM), and eight channels a thread
  // with up to 32 threads a value channel keep them fewest. A block then takes at most
  // 1024 / threads-per-channel value channels: pae_delta_rule_min_splits says how many blocks a head needs.
  const int P = pow2_at_least((d + 7) / 8);
  if (threads_per_column != nullptr) *threads_per_column = P;
  return 8;
}

// The fewest blocks that a head's value channels must be shared out over (a block has at most 1,024 threads).
PAE_EXPORT int pae_delta_rule_min_splits(int d) {
  int P = 0;
  if (pae_delta_rule_layout(d, &P) == 0) return 0;
  const int most_columns = 1024 / P;
  return (d + most_columns - 1) / most_columns;
}

PAE_EXPORT long long pae_delta_rule_scratch_floats(int tokens, int heads, int d) {
  int P = 0;
  const int rpt = pae_delta_rule_layout(d, &P);
  return rpt == 0 ? 0 : (long long)tokens * heads * (5 * P * rpt + 4);
}

// proj float32 [tokens, ld] holds r, k, v, a~ at the given column offsets (heads * d columns each);
// w_pre float32 [tokens, heads * d]; state float32 [slots, heads, d, d] (value channel major);
// o float32 [tokens, heads * d]; prepared float32 scratch of pae_delta_rule_scratch_floats(...), 16-byte aligned.
// `column_splits` blocks share a head's value channels.
PAE_EXPORT int pae_delta_rule_scan(float* o, float* state, float* prepared, const float* proj, int ld, int r_off, int k_off,
                                   int v_off, int a_off, const float* w_pre, const float* w0, const float* a_bias,
                                   const int* q_start, const int* state_slot, int tokens, int entries, int heads, int d,
                                   int column_splits, float decay_scale, float key_eps, void* stream) {
  if (entries == 0 || tokens == 0) return 0;
  int P = 0;
  const int rpt = pae_delta_rule_layout(d, &P);
  if (rpt == 0) return fail(2, "delta_rule_scan: head size %d is outside [1, 256]", d);
  if (entries > 2147483647 / 2 || heads > 65535) return fail(3, "delta_rule_scan: %d requests x %d heads exceed one launch", entries, heads);
  if (column_splits < pae_delta_rule_min_splits(d) || column_splits > d)
    return fail(2, "delta_rule_scan: %d blocks for %d value channels (at least %d)", column_splits, d, pae_delta_rule_min_splits(d));
  if (((uintptr_t)prepared | (uintptr_t)state) & 15) return fail(2, "delta_rule_scan: the scratch or the state does not start on a 16-byte boundary");
  DeltaParams p{};
  p.proj = proj; p.ld = ld; p.r_off = r_off; p.k_off = k_off; p.v_off = v_off; p.a_off = a_off;
  p.w_pre = w_pre; p.w0 = w0; p.a_bias = a_bias; p.prepared = prepared; p.state = state; p.o = o;
  p.q_start = q_start; p.state_slot = state_slot;
  p.tokens = tokens; p.heads = heads; p.d = d; p.columns = (d + column_splits - 1) / column_splits;
  p.decay_scale = decay_scale; p.key_eps = key_eps;
  cudaStream_t s = (cudaStream_t)stream;
  const long long units = (long long)tokens * heads;
  const int dp = P * rpt;
  launch_kernel(delta_prepare_kernel, (unsigned)((units + 3) / 4), 128, 0, s, p, dp);
  if (int err = check_launch("delta_rule_prepare")) return err;
  const int per_token = 5 * dp + 4 + (p.columns + 3) / 4 * 4;
  int tile = 16;
  while (tile > 1 && (size_t)2 * tile * per_token * sizeof(float) > 44 * 1024) tile /= 2;
  p.tile = tile;
  const size_t bytes = (size_t)2 * tile * per_token * sizeof(float);
  const int threads = (p.columns * P + 31) / 32 * 32;
  dim3 grid(entries, heads, (d + p.columns - 1) / p.columns);
  switch (P) {
    case 1: launch_kernel(delta_scan_kernel<8, 1>, grid, threads, bytes, s, p); break;
    case 2: launch_kernel(delta_scan_kernel<8, 2>, grid, threads, bytes, s, p); break;
    case 4: launch_kernel(delta_scan_kernel<8, 4>, grid, threads, bytes, s, p); break;
    case 8: launch_kernel(delta_scan_kernel<8, 8>, grid, threads, bytes, s, p); break;
    case 16: launch_kernel(delta_scan_kernel<8, 16>, grid, threads, bytes, s, p); break;
    default: launch_kernel(delta_scan_kernel<8, 32>, grid, threads, bytes, s, p); break;
  }
  return check_launch("delta_rule_scan");
}

// out [tokens, heads * d] (dtype) from o float32; gate float32 rows of pitch gate_ld (the gate's
// columns start at `gate`), weight float32 [heads * d]; either may be null.
PAE_EXPORT int pae_delta_rule_output(void* out, const float* o, const float* gate, int gate_ld, const float* weight,
                                     int tokens, int heads, int d, float eps, int dtype, void* stream) {
  if (tokens == 0 || heads == 0) return 0;
  const long long units = (long long)tokens * heads;
  const unsigned blocks = (unsigned)((units + 3) / 4);
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == kF32)
    launch_kernel(delta_output_kernel<float>, blocks, 128, 0, s, (float*)out, o, gate, gate_ld, weight, tokens, heads, d, eps);
  else if (dtype == kBF16)
    launch_kernel(delta_output_kernel<__nv_bfloat16>, blocks, 128, 0, s, (__nv_bfloat16*)out, o, gate, gate_ld, weight, tokens, heads, d, eps);
  else
    return fail(1, "delta_rule_output: unknown dtype %d", dtype);
  return check_launch("delta_rule_output");
}

PAE_EXPORT int pae_tanh_columns(void* out, const float* x, int tokens, int ld, int offset, int width, int dtype, void* stream) {
  const long long total = (long long)tokens * width;
  if (total == 0) return 0;
  const unsigned blocks = (unsigned)((total + 255) / 256);
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == kF32)
    launch_kernel(tanh_columns_kernel<float>, blocks, 256, 0, s, (float*)out, x, ld, offset, width, total);
  else if (dtype == kBF16)
    launch_kernel(tanh_columns_kernel<__nv_bfloat16>, blocks, 256, 0, s, (__nv_bfloat16*)out, x, ld, offset, width, total);
  else
    return fail(1, "tanh_columns: unknown dtype %d", dtype);
  return check_launch("tanh_columns");
}

PAE_DEFINE_LAST_ERROR()
