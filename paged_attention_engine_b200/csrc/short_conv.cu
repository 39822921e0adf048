// A short causal convolution over time on every channel of a fused q|k|v projection, with what
// follows it on the way to attention: the unit-RMS scaling of every query and key head and the
// write of keys and values into their pages.
//
//   y[t, c] = sum_j w[c, j] * u[t - taps + 1 + j, c]        (zeros before the sequence's start)
//
// A request's tokens arrive in portions, so the last taps - 1 projected rows of every request are
// kept as per-request state: a token near the start of a portion reads the rows before the portion
// from there. The state is replaced by a second kernel after the first has read it. The
// projection, the state and all arithmetic are float32; queries leave in the engine's element type
// [tokens, heads * d], keys and values go to pages [pages, kv_heads, page_size, d or dv].
//
// A warp takes one head of one token (query heads, then key heads, then value heads; four warps
// a block), its lanes run along the head's channels, so the sum of squares of a head is one warp
// reduction whose order depends on the head size only.
#include "common.cuh"

using namespace pae;

namespace {

constexpr int MAX_PER_LANE = 8;     // head sizes up to 256

struct ConvParams {
  const float* proj;        // [tokens, channels]
  const float* taps_w;      // [channels, taps], null: no convolution
  const float* state;       // [slots, taps - 1, channels]
  const int* positions;     // [tokens]
  const int* seq_index;     // [tokens]
  const int* q_start;       // [entries + 1]
  const int* q_pos0;        // [entries]
  const int* state_slot;    // [entries]
  const int* slots;         // [tokens]: page * page_size + offset, negative: no write; null: no writes at all
  int taps, heads, kv_heads, d, dv, page_size;
  int normalize;            // unit RMS of q and k heads
  float eps;
};

// TAPS > 0: the number of taps, known when compiled, so that all of a head's loads are asked for
// before the first is used; TAPS 0: any number, a loop. A warp takes one head: blockIdx.y * warps + warp.
template <typename T, int TAPS>
__global__ void __launch_bounds__(128) conv_heads_kernel(T* __restrict__ q_out, T* __restrict__ keys, T* __restrict__ values,
                                                         ConvParams p) {
  dependent_launch_prologue();
  const int t = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
  const int unit = blockIdx.y * warps + warp;
  const int units = p.heads + 2 * p.kv_heads;
  if (unit >= units) return;
  const int channels = (p.heads + p.kv_heads) * p.d + p.kv_heads * p.dv;
  const int e = p.seq_index[t];
  const int pos = p.positions[t];
  const int pos0 = p.q_pos0[e];
  const int taps = TAPS > 0 ? TAPS : p.taps;
  const int kept = taps - 1;
  const float* state = p.state != nullptr ? p.state + (size_t)p.state_slot[e] * kept * channels : nullptr;
  const int slot = p.slots != nullptr ? p.slots[t] : -1;
  const bool writes = slot >= 0 && slot_in_pool(slot, p.page_size);
  const int page = writes ? slot / p.page_size : 0, offset = writes ? slot % p.page_size : 0;
  int first, size;          // the unit's channels in a projected row
  if (unit < p.heads) {
    first = unit * p.d; size = p.d;
  } else if (unit < p.heads + p.kv_heads) {
    first = p.heads * p.d + (unit - p.heads) * p.d; size = p.d;
  } else {
    first = (p.heads + p.kv_heads) * p.d + (unit - p.heads - p.kv_heads) * p.dv; size = p.dv;
  }
  // Where tap j's row lies: in this step's projection, in the state, or before the sequence's start.
  const float* source[TAPS > 0 ? TAPS : 1];
  if (TAPS > 0) {
#pragma unroll
    for (int j = 0; j < TAPS; ++j) {
      const int back = kept - j, at = pos - back;
      source[j] = at < 0 ? nullptr
                  : (at >= pos0 ? p.proj + (size_t)(t - back) * channels : state + (size_t)(at - (pos0 - kept)) * channels);
    }
  }
  float y[MAX_PER_LANE];
  float squares = 0.f;
  if (TAPS > 0 && p.taps_w != nullptr) {
    float u[MAX_PER_LANE][TAPS > 0 ? TAPS : 1], w[MAX_PER_LANE][TAPS > 0 ? TAPS : 1];
#pragma unroll
    for (int i = 0; i < MAX_PER_LANE; ++i) {
      const int c = lane + 32 * i;
#pragma unroll
      for (int j = 0; j < TAPS; ++j) {
        const bool live = c < size && source[j] != nullptr;
        u[i][j] = live ? source[j][first + c] : 0.f;
        w[i][j] = live ? p.taps_w[(size_t)(first + c) * TAPS + j] : 0.f;
      }
    }
#pragma unroll
    for (int i = 0; i < MAX_PER_LANE; ++i) {
      float acc = 0.f;
#pragma unroll
      for (int j = 0; j < TAPS; ++j) acc = fmaf(w[i][j], u[i][j], acc);
      y[i] = acc;
      squares = fmaf(acc, acc, squares);
    }
  } else {
#pragma unroll
    for (int i = 0; i < MAX_PER_LANE; ++i) {
      const int c = lane + 32 * i;
      y[i] = 0.f;
      if (c < size) {
        const int channel = first + c;
        if (p.taps_w == nullptr) {
          y[i] = p.proj[(size_t)t * channels + channel];
        } else {
          float acc = 0.f;
          for (int j = 0; j < taps; ++j) {
            const int back = kept - j;                 // tap j reads the row `back` positions before this token
            const int at = pos - back;
            if (at < 0) continue;
            float u;
            if (at >= pos0)
              u = p.proj[(size_t)(t - back) * channels + channel];
            else                                       // state row i holds position pos0 - kept + i
              u = state[(size_t)(at - (pos0 - kept)) * channels + channel];
            acc = fmaf(p.taps_w[(size_t)channel * taps + j], u, acc);
          }
          y[i] = acc;
        }
        squares = fmaf(y[i], y[i], squares);
      }
    }
  }
  float scale = 1.f;
  if (p.normalize && unit < p.heads + p.kv_heads) scale = 1.f / sqrtf(warp_sum(squares) / (float)size + p.eps);
  T* to = nullptr;
  if (unit < p.heads)
    to = q_out + (size_t)t * p.heads * p.d + unit * p.d;
  else if (!writes)
    to = nullptr;
  else if (unit < p.heads + p.kv_heads)
    to = keys + (((size_t)page * p.kv_heads + (unit - p.heads)) * p.page_size + offset) * p.d;
  else
    to = values + (((size_t)page * p.kv_heads + (unit - p.heads - p.kv_heads)) * p.page_size + offset) * p.dv;
  if (to != nullptr) {
#pragma unroll
    for (int i = 0; i < MAX_PER_LANE; ++i) {
      const int c = lane + 32 * i;
      if (c < size) to[c] = from_float<T>(y[i] * scale);
    }
  }
}

// state[slot, i, :] <- the projected row at position kv_len - kept + i: a row of this step, or a
// row the state already held further back, or zero before the sequence's start. A thread owns a
// channel and walks i upwards, so it reads every old row before it overwrites it.
__global__ void conv_state_update_kernel(float* __restrict__ state, const float* __restrict__ proj,
                                         const int* __restrict__ q_start, const int* __restrict__ q_pos0,
                                         const int* __restrict__ state_slot, int kept, int channels) {
  dependent_launch_prologue();
  const int e = blockIdx.y;
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= channels) return;
  const int first = q_start[e], count = q_start[e + 1] - first, pos0 = q_pos0[e];
  float* mine = state + (size_t)state_slot[e] * kept * channels;
  for (int i = 0; i < kept; ++i) {
    const int source = pos0 + count - kept + i;
    float u = 0.f;
    if (source >= pos0)
      u = proj[(size_t)(first + source - pos0) * channels + c];
    else if (source >= 0)
      u = mine[(size_t)(source - (pos0 - kept)) * channels + c];
    mine[(size_t)i * channels + c] = u;
  }
}

}  // namespace

// proj float32 [tokens, (heads + kv_heads) * d + kv_heads * dv] -> q_out [tokens, heads * d], and
// k, v into pages when `slots` is given. taps_w float32 [channels, taps] or null (then taps is 1 and
// nothing is convolved); state float32 [state slots, taps - 1, channels] (unused when taps is 1).
PAE_EXPORT int pae_conv_heads_cache_write(void* q_out, void* keys, void* values, const float* proj, const float* taps_w,
                                          const float* state, const int* positions, const int* seq_index,
                                          const int* q_start, const int* q_pos0, const int* state_slot,
                                          const int* slots, int tokens, int taps, int heads, int kv_heads, int d, int dv,
                                          int page_size, int normalize, float eps, int dtype, void* stream) {
  if (tokens == 0) return 0;
  if (d < 1 || dv < 1 || d > 32 * MAX_PER_LANE || dv > 32 * MAX_PER_LANE)
    return fail(2, "conv_heads_cache_write: head sizes %d and %d are outside [1, %d]", d, dv, 32 * MAX_PER_LANE);
  if (taps < 1 || (taps_w == nullptr && taps != 1)) return fail(2, "conv_heads_cache_write: %d taps", taps);
  if (taps > 1 && state == nullptr) return fail(2, "conv_heads_cache_write: %d taps need the per-request state", taps);
  if (slots != nullptr && (keys == nullptr || values == nullptr || page_size < 1))
    return fail(2, "conv_heads_cache_write: slots without pages");
  ConvParams p{proj, taps_w, state, positions, seq_index, q_start, q_pos0, state_slot, slots,
               taps, heads, kv_heads, d, dv, page_size, normalize, eps};
  cudaStream_t s = (cudaStream_t)stream;
  const int units = heads + 2 * kv_heads;
  if (units > 4 * 65535) return fail(3, "conv_heads_cache_write: %d heads exceed one launch", units);
  dim3 grid(tokens, (units + 3) / 4);
  const int known = (taps_w != nullptr && taps <= 4) ? taps : 0;
  if (dtype != kF32 && dtype != kBF16) return fail(1, "conv_heads_cache_write: unknown dtype %d", dtype);
#define PAE_CONV_CASE(N)                                                                                              \
  if (known == N) {                                                                                                   \
    if (dtype == kF32)                                                                                                \
      launch_kernel(conv_heads_kernel<float, N>, grid, 128, 0, s, (float*)q_out, (float*)keys, (float*)values, p);    \
    else                                                                                                              \
      launch_kernel(conv_heads_kernel<__nv_bfloat16, N>, grid, 128, 0, s, (__nv_bfloat16*)q_out, (__nv_bfloat16*)keys, \
                    (__nv_bfloat16*)values, p);                                                                       \
  }
  PAE_CONV_CASE(0) PAE_CONV_CASE(1) PAE_CONV_CASE(2) PAE_CONV_CASE(3) PAE_CONV_CASE(4)
#undef PAE_CONV_CASE
  return check_launch("conv_heads_cache_write");
}

PAE_EXPORT int pae_conv_state_update(float* state, const float* proj, const int* q_start, const int* q_pos0,
                                     const int* state_slot, int entries, int taps, int channels, void* stream) {
  if (entries == 0 || taps <= 1) return 0;
  if (entries > 65535) return fail(3, "conv_state_update: %d requests exceed one launch", entries);
  dim3 grid((channels + 127) / 128, entries);
  launch_kernel(conv_state_update_kernel, grid, 128, 0, (cudaStream_t)stream, state, proj, q_start, q_pos0, state_slot,
                taps - 1, channels);
  return check_launch("conv_state_update");
}

PAE_DEFINE_LAST_ERROR()
