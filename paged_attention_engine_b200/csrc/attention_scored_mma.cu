// The scored attention rule of attention_scored.cu on tensor cores, for bfloat16: both products
// are mma.sync m16n8k16 with float32 accumulation (the tile helpers of attention_mma.cuh), the
// rule is applied to the float32 scores between them:
//
//   s = (q . k) * scale * temp[h];  s <- cap * tanh(s / cap);  s <- s - r1[h] * log(1 + r2[h] * (i - j))
//   seen: j <= i and (no window, or i - j < window, or j < keep_first);  a sink logit per head in the denominator
//
// A block owns 64 consecutive query tokens of one request and one head (a single decoded token
// is a tile with one row) and walks 64 keys at a time over two ranges: the kept first keys, and
// from the first query's window to the last query. Keys of a tile that no row of the block can
// see are not read (their pages may have been given back), and 16-key steps that a warp's rows
// cannot see are skipped. Query/key heads and value heads may have different sizes (32, 64 or
// 128 each). tanh and the logarithm use the hardware's exp2 and log2 (relative error about
// 1e-6 on a float32 score); probabilities are rounded to bfloat16 for the second product.
#include "attention_mma.cuh"

using namespace pae;
using namespace pae_attention;

namespace {

struct ScoredParams {
  __nv_bfloat16* out;           // [tokens, heads, DV]
  const __nv_bfloat16* q;       // [tokens, heads, D]
  const __nv_bfloat16* keys;    // [pages, kv_heads, page_size, D]
  const __nv_bfloat16* values;  // [pages, kv_heads, page_size, DV]
  const int* block_table;
  const int* q_start;
  const int* q_pos0;
  const int* kv_len;
  int table_width, heads, kv_heads, page_size, window, keep_first;
  float scale, cap;
  const float* temp;
  const float* r1;
  const float* r2;
  const float* sink;
  // Requests that bring one token (when part_out is given): a block takes one kv head and the
  // query heads that share it as its rows, so every key is read once per kv head; the keys are
  // shared out over `splits` such blocks, which leave unnormalised outputs with their maxima and
  // sums for the merge kernel.
  int splits;
  float* part_out;              // [requests, heads, splits, DV]
  float* part_max;              // [requests, heads, splits]  (in units of log 2)
  float* part_sum;              // [requests, heads, splits]
};

__device__ __forceinline__ float fast_tanh(float x) {
  const float e = fast_exp2(x * (2.f * LOG2E));          // e^(2x); inf and 0 at the ends give +1 and -1
  return 1.f - __fdividef(2.f, e + 1.f);
}

template <int D, int DV>
__global__ void __launch_bounds__(128) scored_kernel(const ScoredParams p) {
  dependent_launch_prologue();
  extern __shared__ __align__(128) uint8_t smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int h = blockIdx.y, b = blockIdx.z;
  const int first_token = p.q_start[b];
  const int q_count = p.q_start[b + 1] - first_token;
  const bool shared_out = p.part_out != nullptr && q_count == 1;
  const int tile = shared_out ? 0 : blockIdx.x;
  const int split = shared_out ? blockIdx.x : 0;
  const int group = p.heads / p.kv_heads;
  if (shared_out ? (split >= p.splits || h >= p.kv_heads) : tile * PREFILL_BQ >= q_count) return;
  const uint32_t smem_base = smem_u32(smem);
  const int g = shared_out ? h : h / group;          // grouped: blockIdx.y counts kv heads
  const int* table = p.block_table + (size_t)b * p.table_width;
  const int warp_row0 = warp * 16;
  constexpr int K_BYTES = PREFILL_BKEYS * D * 2, V_BYTES = PREFILL_BKEYS * DV * 2, STAGE_BYTES = K_BYTES + V_BYTES;

  // grouped: the rows are the group's query heads, all at the one token's position
  const int rows = shared_out ? group : min(PREFILL_BQ, q_count - tile * PREFILL_BQ);
  const int pos0 = p.q_pos0[b] + tile * PREFILL_BQ;
  const int kv_end = shared_out ? min(p.kv_len[b], pos0 + 1) : min(p.kv_len[b], pos0 + rows);
  const int first_key = p.window > 0 ? max(0, pos0 - p.window + 1) : 0;
  int kv_begin = (first_key / 16) * 16;
  // Tiles of the kept first keys come first, unless they touch the window's tiles anyway.
  int kept_end = p.window > 0 ? min(p.keep_first, first_key) : 0;
  int kept_tiles = (kept_end + PREFILL_BKEYS - 1) / PREFILL_BKEYS;
  if (kept_tiles * PREFILL_BKEYS > kv_begin) {
    kv_begin = 0;
    kept_tiles = 0;
    kept_end = 0;
  }
  const int tiles = kept_tiles + (kv_end - kv_begin + PREFILL_BKEYS - 1) / PREFILL_BKEYS;

  uint32_t q[D / 16][4];
  load_query_fragments<D>(q, [&](int r) -> const __nv_bfloat16* {
    const int row = warp_row0 + r;
    if (row >= rows) return nullptr;
    return shared_out ? p.q + ((size_t)first_token * p.heads + g * group + row) * D
                      : p.q + ((size_t)(first_token + tile * PREFILL_BQ + row) * p.heads + h) * D;
  });

  // Rows of a tile that lie at or beyond `limit` are zero-filled and never seen. A thread copies the
  // same 16-byte column of a few rows in every tile. The rows' pages are looked up first, all of
  // them, and the copies issued afterwards: one trip to memory for the lookups instead of one per row.
  constexpr int K_CHUNKS = D / 8, V_CHUNKS = DV / 8;
  constexpr int K_ROWS = 128 / K_CHUNKS, V_ROWS = 128 / V_CHUNKS;               // rows that one pass of the block covers
  constexpr int K_PER = PREFILL_BKEYS / K_ROWS, V_PER = PREFILL_BKEYS / V_ROWS;
  const int k_chunk = threadIdx.x % K_CHUNKS, k_row = threadIdx.x / K_CHUNKS;
  const int v_chunk = threadIdx.x % V_CHUNKS, v_row = threadIdx.x / V_CHUNKS;
  const int page_shift = (p.page_size & (p.page_size - 1)) == 0 ? __ffs(p.page_size) - 1 : -1;
  auto row_of = [&](int key, int limit) -> long long {      // row of the key in the pool, -1: not to be read
    // Keys before the block's window that are not kept first keys may lie in pages that were given back.
    if (key >= limit || (key < first_key && key >= p.keep_first)) return -1;
    const int index = page_shift >= 0 ? key >> page_shift : key / p.page_size;
    const int offset = page_shift >= 0 ? key & (p.page_size - 1) : key - index * p.page_size;
    const int page = checked_page(table[checked_table_index(index, p.table_width)]);
    return ((long long)page * p.kv_heads + g) * p.page_size + offset;
  };
  auto fetch = [&](int stage, int key0, int limit) {
    const uint32_t k_dst = smem_base + stage * STAGE_BYTES;
    long long k_at[K_PER];
#pragma unroll
    for (int j = 0; j < K_PER; ++j) k_at[j] = row_of(key0 + k_row + j * K_ROWS, limit);
#pragma unroll
    for (int j = 0; j < K_PER; ++j) {
      const int offset_in_tile = TileLayout<D>::offset_bytes(k_row + j * K_ROWS, k_chunk);
      if (k_at[j] >= 0)
        cp_async16(k_dst + offset_in_tile, p.keys + (size_t)k_at[j] * D + k_chunk * 8);
      else
        *(uint4*)(smem + stage * STAGE_BYTES + offset_in_tile) = make_uint4(0, 0, 0, 0);
    }
    long long v_at[V_PER];
#pragma unroll
    for (int j = 0; j < V_PER; ++j) v_at[j] = (D == DV) ? k_at[j] : row_of(key0 + v_row + j * V_ROWS, limit);
#pragma unroll
    for (int j = 0; j < V_PER; ++j) {
      const int offset_in_tile = K_BYTES + TileLayout<DV>::offset_bytes(v_row + j * V_ROWS, v_chunk);
      if (v_at[j] >= 0)
        cp_async16(k_dst + offset_in_tile, p.values + (size_t)v_at[j] * DV + v_chunk * 8);
      else
        *(uint4*)(smem + stage * STAGE_BYTES + offset_in_tile) = make_uint4(0, 0, 0, 0);
    }
  };
  auto tile_key0 = [&](int t) { return t < kept_tiles ? t * PREFILL_BKEYS : kv_begin + (t - kept_tiles) * PREFILL_BKEYS; };
  auto tile_limit = [&](int t) { return t < kept_tiles ? kept_end : kv_end; };

  float o[DV / 8][4];
#pragma unroll
  for (int n = 0; n < DV / 8; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;
  // Scores are kept in units of log 2. The sink is a logit that is always there: the running
  // maximum starts at it and the sum at 1.
  const bool has_sink = p.sink != nullptr;
  const float sink2 = has_sink && !shared_out ? p.sink[h] * LOG2E : -FLT_MAX;          // the merge adds it otherwise
  float row_max[2] = {sink2, sink2}, row_sum[2] = {sink2 != -FLT_MAX ? 1.f : 0.f, sink2 != -FLT_MAX ? 1.f : 0.f};
  // The head of each of this lane's two rows: the block's head, or, grouped, the row's own.
  const int my_row[2] = {warp_row0 + (lane >> 2), warp_row0 + (lane >> 2) + 8};
  const int my_head[2] = {shared_out ? min(g * group + my_row[0], p.heads - 1) : h,
                          shared_out ? min(g * group + my_row[1], p.heads - 1) : h};
  const float temp[2] = {p.scale * (p.temp != nullptr ? p.temp[my_head[0]] : 1.f),
                         p.scale * (p.temp != nullptr ? p.temp[my_head[1]] : 1.f)};
  const float inv_cap = p.cap > 0.f ? 1.f / p.cap : 0.f;
  const bool has_bias = p.r1 != nullptr;
  const float r1[2] = {has_bias ? p.r1[my_head[0]] : 0.f, has_bias ? p.r1[my_head[1]] : 0.f};
  const float r2[2] = {has_bias ? p.r2[my_head[0]] : 0.f, has_bias ? p.r2[my_head[1]] : 0.f};
  const int my_pos[2] = {shared_out ? pos0 : pos0 + my_row[0], shared_out ? pos0 : pos0 + my_row[1]};
  const int warp_first_pos = shared_out ? pos0 : pos0 + warp_row0;
  const int warp_last_pos = warp_row0 < rows ? (shared_out ? pos0 : pos0 + min(rows, warp_row0 + 16) - 1) : -1;
  const int c = (lane & 3) * 2;

  int t_begin = 0, t_end = tiles;
  if (shared_out) {
    const int each = (tiles + p.splits - 1) / p.splits;
    t_begin = min(tiles, split * each);
    t_end = min(tiles, t_begin + each);
  }
  if (t_begin < t_end) fetch(t_begin & 1, tile_key0(t_begin), tile_limit(t_begin));
  cp_async_commit();
  for (int t = t_begin; t < t_end; ++t) {
    if (t + 1 < t_end) fetch((t + 1) & 1, tile_key0(t + 1), tile_limit(t + 1));
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();
    const uint32_t k_tile = smem_base + (t & 1) * STAGE_BYTES;
    const int limit = tile_limit(t);
#pragma unroll
    for (int sub = 0; sub < PREFILL_BKEYS / 16; ++sub) {
      const int key0 = tile_key0(t) + sub * 16;
      if (key0 > warp_last_pos || key0 >= limit) continue;
      if (p.window > 0 && key0 + 15 < warp_first_pos - p.window + 1 && key0 >= p.keep_first) continue;
      float s[2][4];
      scores_16_keys<D>(s, q, k_tile, sub * 16);
      float block_max[2] = {-FLT_MAX, -FLT_MAX};
#pragma unroll
      for (int u = 0; u < 2; ++u)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int half = j >> 1, key = key0 + u * 8 + c + (j & 1);
          const int distance = my_pos[half] - key;
          const bool seen = key < limit && distance >= 0 && (p.window <= 0 || distance < p.window || key < p.keep_first);
          float x = s[u][j] * temp[half];
          if (p.cap > 0.f) x = p.cap * fast_tanh(x * inv_cap);
          if (has_bias && seen) x -= r1[half] * __logf(1.f + r2[half] * (float)distance);
          s[u][j] = seen ? x * LOG2E : -FLT_MAX;
          block_max[half] = fmaxf(block_max[half], s[u][j]);
        }
      float rescale[2];
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        block_max[half] = fmaxf(block_max[half], __shfl_xor_sync(0xffffffffu, block_max[half], 1));
        block_max[half] = fmaxf(block_max[half], __shfl_xor_sync(0xffffffffu, block_max[half], 2));
        const float new_max = fmaxf(row_max[half], block_max[half]);
        rescale[half] = row_max[half] == -FLT_MAX ? 0.f : fast_exp2(row_max[half] - new_max);
        row_max[half] = new_max;
      }
      float block_sum[2] = {0.f, 0.f};
#pragma unroll
      for (int u = 0; u < 2; ++u)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int half = j >> 1;
          const float e = s[u][j] == -FLT_MAX ? 0.f : fast_exp2(s[u][j] - row_max[half]);
          s[u][j] = e;
          block_sum[half] += e;
        }
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        block_sum[half] += __shfl_xor_sync(0xffffffffu, block_sum[half], 1);
        block_sum[half] += __shfl_xor_sync(0xffffffffu, block_sum[half], 2);
        row_sum[half] = row_sum[half] * rescale[half] + block_sum[half];
      }
      if (__any_sync(0xffffffffu, rescale[0] != 1.f || rescale[1] != 1.f)) {
#pragma unroll
        for (int n = 0; n < DV / 8; ++n) {
          o[n][0] *= rescale[0];
          o[n][1] *= rescale[0];
          o[n][2] *= rescale[1];
          o[n][3] *= rescale[1];
        }
      }
      uint32_t pa[4];
      pa[0] = pack_bf16(s[0][0], s[0][1]);
      pa[1] = pack_bf16(s[0][2], s[0][3]);
      pa[2] = pack_bf16(s[1][0], s[1][1]);
      pa[3] = pack_bf16(s[1][2], s[1][3]);
      accumulate_16_keys<DV>(o, pa, k_tile + K_BYTES, sub * 16);
    }
    __syncthreads();
  }
  cp_async_wait<0>();

  if (shared_out) {               // a row is a query head of the group
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      if (my_row[half] >= rows) continue;
      const size_t at = ((size_t)b * p.heads + g * group + my_row[half]) * p.splits + split;
#pragma unroll
      for (int n = 0; n < DV / 8; ++n) {
        p.part_out[at * DV + n * 8 + c] = o[n][half * 2];
        p.part_out[at * DV + n * 8 + c + 1] = o[n][half * 2 + 1];
      }
      if ((lane & 3) == 0) {
        p.part_max[at] = row_max[half];
        p.part_sum[at] = row_sum[half];
      }
    }
    return;
  }
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const int row = warp_row0 + (lane >> 2) + half * 8;
    if (row >= rows) continue;
    const float inv = row_sum[half] > 0.f ? 1.f / row_sum[half] : 0.f;
    __nv_bfloat16* out = p.out + ((size_t)(first_token + tile * PREFILL_BQ + row) * p.heads + h) * DV;
#pragma unroll
    for (int n = 0; n < DV / 8; ++n)
      *(uint32_t*)(out + n * 8 + (lane & 3) * 2) = pack_bf16(o[n][half * 2] * inv, o[n][half * 2 + 1] * inv);
  }
}

// out[token of a single-token request, head, :] from the partial results of its blocks, in their
// order, with the sink's logit in the denominator.
__global__ void scored_merge_kernel(const ScoredParams p, int dv) {
  dependent_launch_prologue();
  extern __shared__ float weights[];          // [splits]: what a block's partial result counts for
  __shared__ float stats[2];
  const int h = blockIdx.x, b = blockIdx.y;
  const int first_token = p.q_start[b];
  if (p.q_start[b + 1] - first_token != 1) return;
  const size_t at = ((size_t)b * p.heads + h) * p.splits;
  const int lane = threadIdx.x & 31;
  if (threadIdx.x < 32) {                      // one warp: the maximum, then every block's weight and the sum, in the blocks' order
    const float sink2 = p.sink != nullptr ? p.sink[h] * LOG2E : -FLT_MAX;
    float top = sink2;
    for (int s = lane; s < p.splits; s += 32) top = fmaxf(top, p.part_max[at + s]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) top = fmaxf(top, __shfl_xor_sync(0xffffffffu, top, o));
    for (int s = lane; s < p.splits; s += 32) {
      const float m = p.part_max[at + s];
      weights[s] = m == -FLT_MAX ? 0.f : fast_exp2(m - top);
    }
    __syncwarp();
    if (lane == 0) {
      float sum = sink2 != -FLT_MAX ? fast_exp2(sink2 - top) : 0.f;
      for (int s = 0; s < p.splits; ++s) sum += p.part_sum[at + s] * weights[s];
      stats[0] = sum > 0.f ? 1.f / sum : 0.f;
    }
  }
  __syncthreads();
  const float inv = stats[0];
  for (int c = threadIdx.x; c < dv; c += blockDim.x) {
    float acc = 0.f;
    for (int s = 0; s < p.splits; ++s) acc += p.part_out[(at + s) * dv + c] * weights[s];
    p.out[((size_t)first_token * p.heads + h) * dv + c] = __float2bfloat16_rn(acc * inv);
  }
}

template <int D, int DV>
int launch(const ScoredParams& p, int seqs, int max_q_len, cudaStream_t s) {
  const size_t bytes = (size_t)2 * PREFILL_BKEYS * (D + DV) * 2;
  if (int err = allow_smem(scored_kernel<D, DV>, bytes, "paged_attention_scored_mma")) return err;
  const int q_tiles = (max_q_len + PREFILL_BQ - 1) / PREFILL_BQ;
  dim3 grid(p.part_out != nullptr ? max(q_tiles, p.splits) : q_tiles, p.heads, seqs);
  launch_kernel(scored_kernel<D, DV>, grid, 128, bytes, s, p);
  if (int err = check_launch("paged_attention_scored_mma")) return err;
  if (p.part_out != nullptr) {
    launch_kernel(scored_merge_kernel, dim3(p.heads, seqs), 64, (size_t)p.splits * sizeof(float), s, p, DV);
    return check_launch("paged_attention_scored_merge");
  }
  return 0;
}

bool size_ok(int d) { return d == 32 || d == 64 || d == 128; }

}  // namespace

// 1 when the tensor-core kernel takes these head sizes.
PAE_EXPORT int pae_attention_scored_mma_supports(int d, int dv) { return size_ok(d) && size_ok(dv) ? 1 : 0; }

// bfloat16 only; the arguments of pae_paged_attention_scored without the element type. With
// `scratch` (seqs * heads * splits * (dv + 2) floats) every request that brings ONE token is taken
// by blocks of one kv head each, whose rows are the query heads that share it, its keys shared out
// over `splits` blocks and merged by a second kernel; without scratch a single token is a tile of one row.
PAE_EXPORT int pae_paged_attention_scored_mma(void* out, const void* q, const void* keys, const void* values,
                                              const int* block_table, int table_width, const int* q_start,
                                              const int* q_pos0, const int* kv_len, int seqs, int max_q_len, int heads,
                                              int kv_heads, int d, int dv, int page_size, float scale, float cap,
                                              const float* temp, const float* r1, const float* r2, const float* sink,
                                              int window, int keep_first, int splits, float* scratch, void* stream) {
  if (seqs == 0 || max_q_len == 0) return 0;
  if (splits < 1) return fail(2, "paged_attention_scored_mma: %d splits", splits);
  if (scratch != nullptr && heads / kv_heads > PREFILL_BQ)
    return fail(2, "paged_attention_scored_mma: %d query heads per kv head are more than the %d rows of a block", heads / kv_heads, PREFILL_BQ);
  if (scratch == nullptr && splits != 1) return fail(2, "paged_attention_scored_mma: %d splits without scratch", splits);
  if (!pae_attention_scored_mma_supports(d, dv))
    return fail(2, "paged_attention_scored_mma: head sizes %d and %d are not 32, 64 or 128", d, dv);
  if (kv_heads < 1 || heads % kv_heads) return fail(2, "paged_attention_scored_mma: %d heads over %d kv heads", heads, kv_heads);
  if (heads > 65535 || seqs > 65535) return fail(3, "paged_attention_scored_mma: %d heads x %d requests exceed one launch", heads, seqs);
  if (page_size < 1) return fail(2, "paged_attention_scored_mma: page size %d", page_size);
  if ((r1 == nullptr) != (r2 == nullptr)) return fail(2, "paged_attention_scored_mma: the distance bias needs both of its constants");
  if (window < 0 || keep_first < 0) return fail(2, "paged_attention_scored_mma: window %d, kept first keys %d", window, keep_first);
  if (((uintptr_t)q | (uintptr_t)keys | (uintptr_t)values | (uintptr_t)out) & 15)
    return fail(2, "paged_attention_scored_mma: an operand does not start on a 16-byte boundary");
  ScoredParams p{(__nv_bfloat16*)out, (const __nv_bfloat16*)q, (const __nv_bfloat16*)keys, (const __nv_bfloat16*)values,
                 block_table, q_start, q_pos0, kv_len, table_width, heads, kv_heads, page_size, window, keep_first,
                 scale, cap, temp, r1, r2, sink, splits, nullptr, nullptr, nullptr};
  if (scratch != nullptr) {
    const size_t units = (size_t)seqs * heads * splits;
    p.part_out = scratch;
    p.part_max = scratch + units * dv;
    p.part_sum = p.part_max + units;
  }
  cudaStream_t s = (cudaStream_t)stream;
#define PAE_SCORED_CASE(DD, DDV) \
  if (d == DD && dv == DDV) return launch<DD, DDV>(p, seqs, max_q_len, s);
  PAE_SCORED_CASE(32, 32) PAE_SCORED_CASE(64, 64) PAE_SCORED_CASE(128, 128)
  PAE_SCORED_CASE(32, 64) PAE_SCORED_CASE(64, 32) PAE_SCORED_CASE(64, 128) PAE_SCORED_CASE(128, 64)
  PAE_SCORED_CASE(32, 128) PAE_SCORED_CASE(128, 32)
#undef PAE_SCORED_CASE
  return fail(2, "paged_attention_scored_mma: head sizes %d and %d", d, dv);
}

PAE_DEFINE_LAST_ERROR()
