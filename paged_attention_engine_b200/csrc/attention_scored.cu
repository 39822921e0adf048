// Paged attention whose scores follow a rule with per-head constants, on the CUDA cores:
//
//   s(i, j) = (q_i . k_j) * scale * temp[h]
//   s      <- cap * tanh(s / cap)                          when cap > 0
//   s      <- s - r1[h] * log(1 + r2[h] * (i - j))         when r1 is given
//   seen:     j <= i and (window <= 0 or i - j < window or j < keep_first)
//   weights:  exp(s - m) / (sum over seen keys of exp(s - m) + exp(sink[h] - m))   (the last term when
//             a sink is given: a learned logit without key or value that counts once)
//
// Every part of the rule is optional (a null pointer or a zero turns it off), so the kernel also
// computes plain causal or windowed attention. Value heads may have another size (dv) than query
// and key heads (d); queries come as their own [tokens, heads, d] tensor. Any d that fits shared
// memory, dv up to 512; the values may be the leading channels of the keys themselves.
// Scores, the rule's arithmetic and the running softmax are float32 for bfloat16 tensors. For
// float32 tensors they are double: a score that is a sum of d float32 products, sharpened by a
// temperature and exponentiated, carries several units of float32 rounding into its weight when
// it is summed in float32, and layers that cancel downstream multiply that; summed and
// transformed in double, a weight is as good as its float32 inputs allow.
//
// A block owns 16 consecutive query tokens of one request and one query head and walks that
// request's pages in place, 32 keys at a time, over two ranges: the kept first keys and the
// window of its queries. Tiles that no query of the block sees are skipped, and a key that none
// sees is not read, so pages that the window has left behind may be gone from the block table.
// A query's result depends on its own keys only.
#include "common.cuh"

#include <cfloat>

using namespace pae;

namespace {

constexpr int BQ = 16;
constexpr int BKEYS = 32;
constexpr int THREADS = 128;

struct ScoreRule {
  float scale;
  float cap;
  const float* temp;     // [heads] or null
  const float* r1;       // [heads] or null
  const float* r2;       // [heads] (with r1)
  const float* sink;     // [heads] or null
  int window;            // 0: every earlier key
  int keep_first;        // keys below this position stay visible under a window
};

__device__ __forceinline__ float exp_of(float x) { return expf(x); }
__device__ __forceinline__ double exp_of(double x) { return exp(x); }
__device__ __forceinline__ float tanh_of(float x) { return tanhf(x); }
__device__ __forceinline__ double tanh_of(double x) { return tanh(x); }
__device__ __forceinline__ float log1p_of(float x) { return log1pf(x); }
__device__ __forceinline__ double log1p_of(double x) { return log1p(x); }

// A: the type of scores, weights and sums (float for bfloat16 tensors, double for float32 ones).
// MAX_D: the most value channels (a thread keeps MAX_D / 8 of them). `vs_row` is the distance
// between two value rows in elements: dv for a value tensor of its own, the key rows' d when
// the values are the leading channels of the keys themselves (values == keys).
template <typename T, typename A, int MAX_D>
__global__ void __launch_bounds__(THREADS) attention_scored_kernel(
    T* __restrict__ out, const T* __restrict__ q, const T* __restrict__ keys, const T* __restrict__ values,
    const int* __restrict__ block_table, int table_width, const int* __restrict__ q_start,
    const int* __restrict__ q_pos0, const int* __restrict__ kv_len, int heads, int kv_heads, int d, int dv,
    int vs_row, int page_size, ScoreRule rule) {
  dependent_launch_prologue();
  extern __shared__ float smem[];
  const int b = blockIdx.z, h = blockIdx.y, tile = blockIdx.x;
  const int first_token = q_start[b];
  const int q_count = q_start[b + 1] - first_token;
  if (tile * BQ >= q_count) return;
  const int p0 = q_pos0[b] + tile * BQ;
  const int rows = min(BQ, q_count - tile * BQ);
  const int kv_end = min(kv_len[b], p0 + rows);
  const int window_begin = rule.window > 0 ? max(0, p0 - rule.window + 1) : 0;   // the first query's; later ones start later
  const int kept_end = rule.window > 0 ? min(rule.keep_first, window_begin) : 0;
  const int g = h / (heads / kv_heads);

  const int dpad = d + 1;
  float* qs = smem;                        // [BQ][d + 1]
  float* ks = qs + BQ * dpad;              // [BKEYS][d + 1]
  float* vs = ks + BKEYS * dpad;           // [BKEYS][dv]
  float* ps = vs + BKEYS * dv;             // [BQ][BKEYS + 1]

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int r = tid >> 3;
  const int cg = tid & 7;

  for (int i = tid; i < BQ * d; i += THREADS) {
    const int row = i / d, k = i - row * d;
    qs[row * dpad + k] = row < rows ? to_float(q[((size_t)(first_token + tile * BQ + row) * heads + h) * d + k]) : 0.f;
  }

  const A lowest = (A)-FLT_MAX;
  const A temp = (A)rule.scale * (rule.temp != nullptr ? (A)rule.temp[h] : (A)1);
  const A cap = (A)rule.cap;
  const A r1 = rule.r1 != nullptr ? (A)rule.r1[h] : (A)0;
  const A r2 = rule.r1 != nullptr ? (A)rule.r2[h] : (A)0;
  A acc[MAX_D / 8];
#pragma unroll
  for (int i = 0; i < MAX_D / 8; ++i) acc[i] = (A)0;
  // The sink is a logit that is always there: the running maximum starts at it, the sum at exp(0).
  A row_max = rule.sink != nullptr ? (A)rule.sink[h] : lowest;
  A row_sum = rule.sink != nullptr ? (A)1 : (A)0;
  const int my_pos = p0 + r;
  const int nd = (dv + 7) >> 3;
  const int* table = block_table + (size_t)b * table_width;

  for (int range = 0; range < 2; ++range) {
    const int begin = range == 0 ? 0 : window_begin;
    const int end = range == 0 ? kept_end : kv_end;
    for (int base = begin; base < end; base += BKEYS) {
      __syncthreads();
      for (int c = warp; c < BKEYS; c += THREADS / 32) {
        const int j = base + c;
        if (j < end) {
          const int page = checked_page(table[checked_table_index(j / page_size, table_width)]);
          const size_t row = ((size_t)page * kv_heads + g) * page_size + (j % page_size);
          for (int k = lane; k < d; k += 32) ks[c * dpad + k] = to_float(keys[row * d + k]);
          for (int k = lane; k < dv; k += 32) vs[c * dv + k] = to_float(values[row * vs_row + k]);
        } else {
          for (int k = lane; k < d; k += 32) ks[c * dpad + k] = 0.f;
          for (int k = lane; k < dv; k += 32) vs[c * dv + k] = 0.f;
        }
      }
      __syncthreads();

      A s[BKEYS / 8];
      A tile_max = lowest;
#pragma unroll
      for (int i = 0; i < BKEYS / 8; ++i) {
        const int c = cg + 8 * i;
        const int j = base + c;
        A dot = (A)0;
        for (int k = 0; k < d; ++k) dot = fma((A)qs[r * dpad + k], (A)ks[c * dpad + k], dot);
        const int distance = my_pos - j;
        const bool seen = r < rows && j < end && distance >= 0 &&
                          (rule.window <= 0 || distance < rule.window || j < rule.keep_first);
        A score = dot * temp;
        if (rule.cap > 0.f) score = cap * tanh_of(score / cap);
        if (rule.r1 != nullptr && seen) score -= r1 * log1p_of(r2 * (A)distance);
        s[i] = seen ? score : lowest;
        tile_max = s[i] > tile_max ? s[i] : tile_max;
      }
#pragma unroll
      for (int o = 4; o > 0; o >>= 1) {
        const A other = __shfl_xor_sync(0xffffffffu, tile_max, o);
        tile_max = other > tile_max ? other : tile_max;
      }
      const A new_max = row_max > tile_max ? row_max : tile_max;
      const A rescale = (row_max == lowest) ? (A)0 : exp_of(row_max - new_max);
      A tile_sum = (A)0;
#pragma unroll
      for (int i = 0; i < BKEYS / 8; ++i) {
        const A p = (s[i] == lowest) ? (A)0 : exp_of(s[i] - new_max);
        ps[r * (BKEYS + 1) + cg + 8 * i] = (float)p;
        tile_sum += p;
      }
#pragma unroll
      for (int o = 4; o > 0; o >>= 1) tile_sum += __shfl_xor_sync(0xffffffffu, tile_sum, o);
      row_sum = row_sum * rescale + tile_sum;
      row_max = new_max;
      __syncwarp();
#pragma unroll
      for (int i = 0; i < MAX_D / 8; ++i) {
        if (i < nd) {
          A v = acc[i] * rescale;
          const int dim = cg + 8 * i;
          if (dim < dv)
            for (int c = 0; c < BKEYS; ++c) v = fma((A)ps[r * (BKEYS + 1) + c], (A)vs[c * dv + dim], v);
          acc[i] = v;
        }
      }
    }
  }

  if (r < rows) {
    const A inv = row_sum > (A)0 ? (A)1 / row_sum : (A)0;
    T* to = out + ((size_t)(first_token + tile * BQ + r) * heads + h) * dv;
#pragma unroll
    for (int i = 0; i < MAX_D / 8; ++i)
      if (i < nd && cg + 8 * i < dv) to[cg + 8 * i] = from_float<T>((float)(acc[i] * inv));
  }
}

constexpr size_t SMEM_LIMIT = 200 * 1024;
constexpr int MOST_CHANNELS = 512;

size_t smem_bytes(int d, int dv) {
  return sizeof(float) * (size_t)(BQ * (d + 1) + BKEYS * (d + 1) + BKEYS * dv + BQ * (BKEYS + 1));
}

template <typename T, typename A, int MAX_D>
int launch_sized(void* out, const void* q, const void* keys, const void* values, const int* block_table, int table_width,
                 const int* q_start, const int* q_pos0, const int* kv_len, int seqs, int max_q_len, int heads, int kv_heads,
                 int d, int dv, int vs_row, int page_size, const ScoreRule& rule, cudaStream_t s) {
  const size_t bytes = smem_bytes(d, dv);
  auto kernel = attention_scored_kernel<T, A, MAX_D>;
  static bool raised = false;
  if (bytes > 48 * 1024 && !raised) {
    cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_LIMIT);
    if (err != cudaSuccess) return fail(100, "paged_attention_scored: %s", cudaGetErrorString(err));
    raised = true;
  }
  dim3 grid((max_q_len + BQ - 1) / BQ, heads, seqs);
  launch_kernel(kernel, grid, THREADS, bytes, s, (T*)out, (const T*)q, (const T*)keys, (const T*)values, block_table,
                table_width, q_start, q_pos0, kv_len, heads, kv_heads, d, dv, vs_row, page_size, rule);
  return check_launch("paged_attention_scored");
}

template <typename T, typename A>
int launch(void* out, const void* q, const void* keys, const void* values, const int* block_table, int table_width,
           const int* q_start, const int* q_pos0, const int* kv_len, int seqs, int max_q_len, int heads, int kv_heads,
           int d, int dv, int vs_row, int page_size, const ScoreRule& rule, cudaStream_t s) {
#define PAE_SIZED(MAXD)                                                                                             \
  if (dv <= MAXD)                                                                                                   \
    return launch_sized<T, A, MAXD>(out, q, keys, values, block_table, table_width, q_start, q_pos0, kv_len, seqs, \
                                    max_q_len, heads, kv_heads, d, dv, vs_row, page_size, rule, s);
  PAE_SIZED(64) PAE_SIZED(128) PAE_SIZED(256) PAE_SIZED(512)
#undef PAE_SIZED
  return fail(2, "paged_attention_scored: value heads of %d channels", dv);
}

}  // namespace

// out [tokens, heads, dv]; q [tokens, heads, d]; keys [pages, kv_heads, page_size, d]; values
// [pages, kv_heads, page_size, dv], or the keys themselves (the same pointer: a key row's first dv
// channels are its value; dv <= d); temp, r1, r2, sink float32 [heads] or null; cap 0: no cap.
PAE_EXPORT int pae_paged_attention_scored(void* out, const void* q, const void* keys, const void* values,
                                          const int* block_table, int table_width, const int* q_start,
                                          const int* q_pos0, const int* kv_len, int seqs, int max_q_len, int heads,
                                          int kv_heads, int d, int dv, int page_size, float scale, float cap,
                                          const float* temp, const float* r1, const float* r2, const float* sink,
                                          int window, int keep_first, int dtype, void* stream) {
  if (seqs == 0 || max_q_len == 0) return 0;
  if (d < 1 || dv < 1 || dv > MOST_CHANNELS || smem_bytes(d, dv) > SMEM_LIMIT)
    return fail(2, "paged_attention_scored: head sizes %d and %d (values up to %d; both must fit shared memory)", d, dv, MOST_CHANNELS);
  const int vs_row = values == keys ? d : dv;
  if (values == keys && dv > d) return fail(2, "paged_attention_scored: values inside keys of %d channels cannot have %d", d, dv);
  if (kv_heads < 1 || heads % kv_heads) return fail(2, "paged_attention_scored: %d heads over %d kv heads", heads, kv_heads);
  if (heads > 65535 || seqs > 65535) return fail(3, "paged_attention_scored: %d heads x %d requests exceed one launch", heads, seqs);
  if (page_size < 1) return fail(2, "paged_attention_scored: page size %d", page_size);
  if ((r1 == nullptr) != (r2 == nullptr)) return fail(2, "paged_attention_scored: the distance bias needs both of its constants");
  if (window < 0 || keep_first < 0) return fail(2, "paged_attention_scored: window %d, kept first keys %d", window, keep_first);
  ScoreRule rule{scale, cap, temp, r1, r2, sink, window, keep_first};
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == kF32)
    return launch<float, double>(out, q, keys, values, block_table, table_width, q_start, q_pos0, kv_len, seqs, max_q_len, heads,
                         kv_heads, d, dv, vs_row, page_size, rule, s);
  if (dtype == kBF16)
    return launch<__nv_bfloat16, float>(out, q, keys, values, block_table, table_width, q_start, q_pos0, kv_len, seqs, max_q_len,
                                 heads, kv_heads, d, dv, vs_row, page_size, rule, s);
  return fail(1, "paged_attention_scored: unknown dtype %d", dtype);
}

PAE_DEFINE_LAST_ERROR()
