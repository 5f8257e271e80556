// Layers that carry a state of fixed size from token to token, and the norms around them.
//
//   * layer norm with scale and shift, alone and fused with the residual sum: the residual stream is
//     float32; r += m * LN_post(delta), then y = LN_pre(r), in one pass over the row;
//   * a table lookup that writes float32 rows (the start of a float32 residual stream);
//   * the causal convolution over a few taps per channel with its SiLU, whose last taps - 1 inputs
//     live in the request's state slot;
//   * the decayed outer-product recurrence  S_t = diag(a_t) S_{t-1} + k_t v_t^T,  o_t = S_t^T q_t
//     per head, S [D, V] float32 in the request's state slot, in two settings: a decay per key channel
//     a = sigmoid(z)^(1/tau) (gated linear attention), and one decay per head a = exp(-exp(A) dt)
//     with k = dt B, q = C and a skip term D x (the state-space form of Mamba-2);
//   * the RMS norm over equal groups of a row with a SiLU gate before or behind it.
//
// Everything that enters the recurrence is float32: decays, their logarithms, softplus, step sizes,
// the state, the sums.  A row's tokens are run in their order, so a result does not depend on how a
// prompt was cut into steps or on what else a step carries.
#include <algorithm>
#include <initializer_list>

#include "common.cuh"

namespace zb {

__device__ __forceinline__ float silu_f(float z) { return z / (1.0f + expf(-z)); }
__device__ __forceinline__ float log_sigmoid_f(float z) { return fminf(z, 0.0f) - log1pf(expf(-fabsf(z))); }
__device__ __forceinline__ float softplus_f(float z) { return fmaxf(z, 0.0f) + log1pf(expf(-fabsf(z))); }

// ------------------------------------------------------------------------------------------------
// Layer norm.  One CTA per row; the row sits in shared memory as float32, mean and variance are
// two passes over it (the variance is the mean of the squared deviations).
// A norm without a shift passes a null pointer for it.
__device__ __forceinline__ float load_shift(const void* b, int w_dtype, int i) {
  return b != nullptr ? load_scale(b, w_dtype, i) : 0.0f;
}

__device__ __forceinline__ void layer_norm_stats(const float* row, int H, float eps, float* scratch, float& mean,
                                                 float& rstd, bool rms = false) {
  if (rms) {          // an RMS norm: no mean is taken off, the statistic is the mean square
    float v = 0.0f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) v = fmaf(row[i], row[i], v);
    mean = 0.0f;
    rstd = 1.0f / sqrtf(block_sum(v, scratch) / static_cast<float>(H) + eps);
    return;
  }
  float s = 0.0f;
  for (int i = threadIdx.x; i < H; i += blockDim.x) s += row[i];
  mean = block_sum(s, scratch) / static_cast<float>(H);
  float v = 0.0f;
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    const float d = row[i] - mean;
    v = fmaf(d, d, v);
  }
  rstd = 1.0f / sqrtf(block_sum(v, scratch) / static_cast<float>(H) + eps);
}

template <typename X, typename T>
__global__ void layer_norm_kernel(T* out, const X* x, const void* w, const void* b, int w_dtype, float eps, int H) {
  extern __shared__ __align__(16) float ln_row[];
  __shared__ float scratch[33];
  const size_t base = static_cast<size_t>(blockIdx.x) * H;
  for (int i = threadIdx.x; i < H; i += blockDim.x) ln_row[i] = to_float(x[base + i]);
  __syncthreads();
  float mean, rstd;
  layer_norm_stats(ln_row, H, eps, scratch, mean, rstd);
  for (int i = threadIdx.x; i < H; i += blockDim.x)
    out[base + i] = from_float<T>(fmaf((ln_row[i] - mean) * rstd, load_scale(w, w_dtype, i), load_shift(b, w_dtype, i)));
}

// residual += mult * LN(delta; w1, b1); then, if `out`, out = LN(residual; w2, b2), or with a null w2
// the sum itself in T (what a part that reads the stream unnormed takes).  RMS: both norms are RMS norms
// (x / sqrt(mean(x^2) + eps) * w, no mean taken off, no shift).
template <typename T, bool RMS>
__global__ void residual_layer_norm_kernel(float* residual, const T* delta, const void* w1, const void* b1, float mult,
                                           T* out, const void* w2, const void* b2, int w_dtype, float eps1, float eps2,
                                           int H) {
  extern __shared__ __align__(16) float ln_row[];
  __shared__ float scratch[33];
  const size_t base = static_cast<size_t>(blockIdx.x) * H;
  for (int i = threadIdx.x; i < H; i += blockDim.x) ln_row[i] = to_float(delta[base + i]);
  __syncthreads();
  float mean, rstd;
  layer_norm_stats(ln_row, H, eps1, scratch, mean, rstd, RMS);
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    const float y = fmaf((ln_row[i] - mean) * rstd, load_scale(w1, w_dtype, i), load_shift(b1, w_dtype, i));
    const float r = fmaf(mult, y, residual[base + i]);
    residual[base + i] = r;
    ln_row[i] = r;              // each thread rewrites only the elements it read
    if (out != nullptr && w2 == nullptr) out[base + i] = from_float<T>(r);     // no second norm: the sum, rounded
  }
  if (out == nullptr || w2 == nullptr) return;
  __syncthreads();
  layer_norm_stats(ln_row, H, eps2, scratch, mean, rstd, RMS);
  for (int i = threadIdx.x; i < H; i += blockDim.x)
    out[base + i] = from_float<T>(fmaf((ln_row[i] - mean) * rstd, load_scale(w2, w_dtype, i), load_shift(b2, w_dtype, i)));
}

// The same two kernels for rows of up to LN_VEC_MAX elements whose length is a multiple of four: a thread
// keeps its share of the row in registers as vectors of four, loads and stores move 8 or 16 bytes, and
// nothing passes through shared memory but the two sums.
constexpr int LN_VEC_THREADS = 256;
constexpr int LN_VEC_ITEMS = 8;
constexpr int LN_VEC_MAX = LN_VEC_THREADS * LN_VEC_ITEMS * 4;

__device__ __forceinline__ float4 load4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 load4(const __nv_bfloat16* p) {
  const uint2 raw = *reinterpret_cast<const uint2*>(p);
  const float2 lo = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
  const float2 hi = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
  return make_float4(lo.x, lo.y, hi.x, hi.y);
}
__device__ __forceinline__ void store4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void store4(__nv_bfloat16* p, float4 v) {
  uint2 raw;
  *reinterpret_cast<__nv_bfloat162*>(&raw.x) = __floats2bfloat162_rn(v.x, v.y);
  *reinterpret_cast<__nv_bfloat162*>(&raw.y) = __floats2bfloat162_rn(v.z, v.w);
  *reinterpret_cast<uint2*>(p) = raw;
}

__device__ __forceinline__ void vec_stats(const float4 (&r)[LN_VEC_ITEMS], int nv, int H, float eps, float* scratch,
                                          float& mean, float& rstd, bool rms = false) {
  if (rms) {
    float v = 0.0f;
#pragma unroll
    for (int j = 0; j < LN_VEC_ITEMS; ++j)
      if (static_cast<int>(threadIdx.x) + j * LN_VEC_THREADS < nv)
        v += (r[j].x * r[j].x + r[j].y * r[j].y) + (r[j].z * r[j].z + r[j].w * r[j].w);
    mean = 0.0f;
    rstd = 1.0f / sqrtf(block_sum(v, scratch) / static_cast<float>(H) + eps);
    return;
  }
  float s = 0.0f;
#pragma unroll
  for (int j = 0; j < LN_VEC_ITEMS; ++j)
    if (static_cast<int>(threadIdx.x) + j * LN_VEC_THREADS < nv) s += (r[j].x + r[j].y) + (r[j].z + r[j].w);
  mean = block_sum(s, scratch) / static_cast<float>(H);
  float v = 0.0f;
#pragma unroll
  for (int j = 0; j < LN_VEC_ITEMS; ++j)
    if (static_cast<int>(threadIdx.x) + j * LN_VEC_THREADS < nv) {
      const float a = r[j].x - mean, b = r[j].y - mean, c = r[j].z - mean, d = r[j].w - mean;
      v += (a * a + b * b) + (c * c + d * d);
    }
  rstd = 1.0f / sqrtf(block_sum(v, scratch) / static_cast<float>(H) + eps);
}

__device__ __forceinline__ float4 vec_affine(float4 x, float mean, float rstd, const float* w, const float* b, int at) {
  const float4 wv = load4(w + at), bv = b != nullptr ? load4(b + at) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
  return make_float4(fmaf((x.x - mean) * rstd, wv.x, bv.x), fmaf((x.y - mean) * rstd, wv.y, bv.y),
                     fmaf((x.z - mean) * rstd, wv.z, bv.z), fmaf((x.w - mean) * rstd, wv.w, bv.w));
}

template <typename X, typename T>
__global__ void __launch_bounds__(LN_VEC_THREADS)
layer_norm_vec_kernel(T* out, const X* x, const float* w, const float* b, float eps, int H) {
  __shared__ float scratch[33];
  const size_t base = static_cast<size_t>(blockIdx.x) * H;
  const int nv = H / 4;
  float4 r[LN_VEC_ITEMS];
#pragma unroll
  for (int j = 0; j < LN_VEC_ITEMS; ++j) {
    const int i = threadIdx.x + j * LN_VEC_THREADS;
    if (i < nv) r[j] = load4(x + base + 4 * i);
  }
  float mean, rstd;
  vec_stats(r, nv, H, eps, scratch, mean, rstd);
#pragma unroll
  for (int j = 0; j < LN_VEC_ITEMS; ++j) {
    const int i = threadIdx.x + j * LN_VEC_THREADS;
    if (i < nv) store4(out + base + 4 * i, vec_affine(r[j], mean, rstd, w, b, 4 * i));
  }
}

template <typename T, bool RMS>
__global__ void __launch_bounds__(LN_VEC_THREADS)
residual_layer_norm_vec_kernel(float* residual, const T* delta, const float* w1, const float* b1, float mult, T* out,
                               const float* w2, const float* b2, float eps1, float eps2, int H) {
  __shared__ float scratch[33];
  const size_t base = static_cast<size_t>(blockIdx.x) * H;
  const int nv = H / 4;
  float4 r[LN_VEC_ITEMS];
#pragma unroll
  for (int j = 0; j < LN_VEC_ITEMS; ++j) {
    const int i = threadIdx.x + j * LN_VEC_THREADS;
    if (i < nv) r[j] = load4(delta + base + 4 * i);
  }
  float mean, rstd;
  vec_stats(r, nv, H, eps1, scratch, mean, rstd, RMS);
#pragma unroll
  for (int j = 0; j < LN_VEC_ITEMS; ++j) {
    const int i = threadIdx.x + j * LN_VEC_THREADS;
    if (i < nv) {
      const float4 y = vec_affine(r[j], mean, rstd, w1, b1, 4 * i), old = load4(residual + base + 4 * i);
      r[j] = make_float4(fmaf(mult, y.x, old.x), fmaf(mult, y.y, old.y), fmaf(mult, y.z, old.z), fmaf(mult, y.w, old.w));
      store4(residual + base + 4 * i, r[j]);
      if (out != nullptr && w2 == nullptr) store4(out + base + 4 * i, r[j]);   // no second norm: the sum, rounded
    }
  }
  if (out == nullptr || w2 == nullptr) return;
  vec_stats(r, nv, H, eps2, scratch, mean, rstd, RMS);
#pragma unroll
  for (int j = 0; j < LN_VEC_ITEMS; ++j) {
    const int i = threadIdx.x + j * LN_VEC_THREADS;
    if (i < nv) store4(out + base + 4 * i, vec_affine(r[j], mean, rstd, w2, b2, 4 * i));
  }
}

// True if rows of H elements and these pointers take the vector kernels (float32 scales).
inline bool ln_vectors(int H, int w_dtype, std::initializer_list<const void*> pointers) {
  if (H % 4 != 0 || H > LN_VEC_MAX || w_dtype != DTYPE_F32) return false;
  for (const void* p : pointers)
    if (p != nullptr && reinterpret_cast<uintptr_t>(p) % 16 != 0) return false;
  return true;
}

// out = scale * table[id] as float32; `rounded` (may be null) gets the same rows in the table's type.
template <typename T>
__global__ void embedding_f32_kernel(float* out, T* rounded, const T* table, const int* ids, float scale, int H, int V,
                                     int* status) {
  const int t = blockIdx.x, id = ids[t];
  const bool ok = id >= 0 && id < V;
  if (!ok && threadIdx.x == 0) report(status, STATUS_TOKEN_OUT_OF_RANGE, id, t);
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    const float v = ok ? scale * to_float(table[static_cast<size_t>(id) * H + i]) : 0.0f;
    out[static_cast<size_t>(t) * H + i] = v;
    if (rounded != nullptr) rounded[static_cast<size_t>(t) * H + i] = from_float<T>(v);
  }
}

// ------------------------------------------------------------------------------------------------
// Causal convolution per channel with SiLU, over all new tokens of the step at once; the inputs before
// a request's first new token come from its state (zeros for a new request), and a second small
// kernel then puts the request's last taps - 1 inputs there.
constexpr int CONV_MAX_TAPS = 8;

struct ConvArgs {
  void* out;                 // [tokens, C]
  const void* x;             // [tokens, x_stride], channel c at column c
  long long x_stride;
  float* state;              // slot s at state + s * slot_stride: [taps - 1][C], oldest input first
  long long slot_stride;
  const int* slots;
  const int* row_q_start;
  const int* row_q_len;
  const void* w;             // [C, taps], the last column weighs the current token
  const void* bias;          // [C]
  int w_dtype, C, taps, num_slots, write_state;
  int* status;
};

// The convolution proper: a thread owns a channel of one token (CONV_TOKENS consecutive ones) of the
// step's stream.  Input i of a request's new tokens is row t0 + i of x for i >= 0 and entry taps - 1 + i of
// the request's state for i < 0; nothing is written to the state here.
constexpr int CONV_TOKENS = 1;

template <typename T>
__global__ void causal_conv_silu_kernel(const ConvArgs a, const int* token_row, int tokens) {
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= a.C) return;
  float w[CONV_MAX_TAPS];
#pragma unroll
  for (int j = 0; j < CONV_MAX_TAPS; ++j) w[j] = j < a.taps ? load_scale(a.w, a.w_dtype, c * a.taps + j) : 0.0f;
  const float bias = load_scale(a.bias, a.w_dtype, c);
  const T* x = static_cast<const T*>(a.x);
  T* out = static_cast<T*>(a.out);
  const int first = blockIdx.x * CONV_TOKENS;
  for (int t = first; t < min(first + CONV_TOKENS, tokens); ++t) {
    const int row = token_row[t];
    const int slot = a.slots[row];
    if (slot < 0 || slot >= a.num_slots) {
      report(a.status, STATUS_ROW_OUT_OF_RANGE, slot, row);
      continue;
    }
    const int i = t - a.row_q_start[row];
    const float* state = a.state + static_cast<long long>(slot) * a.slot_stride;
    float acc = 0.0f;
#pragma unroll
    for (int j = 0; j < CONV_MAX_TAPS; ++j) {          // oldest input first, as the weights lie
      if (j < a.taps) {
        const int back = a.taps - 1 - j;
        const float in = i - back >= 0 ? to_float(x[static_cast<long long>(t - back) * a.x_stride + c])
                                       : state[static_cast<long long>(a.taps - 1 + i - back) * a.C + c];
        acc = fmaf(w[j], in, acc);
      }
    }
    out[static_cast<long long>(t) * a.C + c] = from_float<T>(silu_f(acc + bias));
  }
}

// The form that runs wherever the shapes allow it (bfloat16, an even number of channels, aligned rows):
// a CTA takes CONV_TILE consecutive tokens of the stream and 128 channels, a thread two adjacent
// channels, which it walks down the tile with the last inputs in registers: one 4-byte load and one
// 4-byte store a token.  Where a tile crosses from one request to the next the window starts again
// from that request's state.  The tile's rows, slots and first tokens are looked up once, into shared
// memory.
constexpr int CONV_TILE = 32;

__global__ void __launch_bounds__(64) causal_conv_silu_tile_kernel(const ConvArgs a, const int* token_row, int tokens) {
  __shared__ int first_s[CONV_TILE], slot_s[CONV_TILE];       // per token: index within its request's new tokens, slot
  const int t0 = blockIdx.x * CONV_TILE, nt = min(CONV_TILE, tokens - t0);
  if (threadIdx.x < nt) {
    const int row = token_row[t0 + threadIdx.x];
    const int slot = a.slots[row];
    first_s[threadIdx.x] = t0 + threadIdx.x - a.row_q_start[row];
    slot_s[threadIdx.x] = slot;
    if (slot < 0 || slot >= a.num_slots) report(a.status, STATUS_ROW_OUT_OF_RANGE, slot, row);
  }
  __syncthreads();
  const int c = (blockIdx.y * blockDim.x + threadIdx.x) * 2;
  if (c >= a.C) return;
  const int first = CONV_MAX_TAPS - a.taps;
  const float* wp = static_cast<const float*>(a.w);
  float w[CONV_MAX_TAPS][2], win[CONV_MAX_TAPS][2];
#pragma unroll
  for (int j = 0; j < CONV_MAX_TAPS; ++j) {
    w[j][0] = j >= first ? wp[c * a.taps + (j - first)] : 0.0f;
    w[j][1] = j >= first ? wp[(c + 1) * a.taps + (j - first)] : 0.0f;
    win[j][0] = win[j][1] = 0.0f;
  }
  const float bias0 = static_cast<const float*>(a.bias)[c], bias1 = static_cast<const float*>(a.bias)[c + 1];
  const __nv_bfloat16* x = static_cast<const __nv_bfloat16*>(a.x);
  __nv_bfloat16* out = static_cast<__nv_bfloat16*>(a.out);
  for (int k = 0; k < nt; ++k) {
    const int i = first_s[k], slot = slot_s[k];
    if (slot < 0 || slot >= a.num_slots) continue;
    if (k == 0 || i == 0) {
      // The window before this token: inputs i - taps + 1 .. i - 1, from x or, before the request's first
      // new token, from its state.  win[j + 1] is what win[j] will be after the shift below.
      const float* state = a.state + static_cast<long long>(slot) * a.slot_stride;
#pragma unroll
      for (int j = 0; j < CONV_MAX_TAPS; ++j) {
        if (j > first) {
          const int back = CONV_MAX_TAPS - j;          // win[j] holds the input `back` tokens before this one
          if (i - back >= 0) {
            const float2 v = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(
                x + static_cast<long long>(t0 + k - back) * a.x_stride + c));
            win[j][0] = v.x; win[j][1] = v.y;
          } else {
            const float2 v = *reinterpret_cast<const float2*>(state + static_cast<long long>(a.taps - 1 + i - back) * a.C + c);
            win[j][0] = v.x; win[j][1] = v.y;
          }
        }
      }
    }
#pragma unroll
    for (int j = 0; j + 1 < CONV_MAX_TAPS; ++j) { win[j][0] = win[j + 1][0]; win[j][1] = win[j + 1][1]; }
    const float2 now = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(
        x + static_cast<long long>(t0 + k) * a.x_stride + c));
    win[CONV_MAX_TAPS - 1][0] = now.x; win[CONV_MAX_TAPS - 1][1] = now.y;
    float acc0 = 0.0f, acc1 = 0.0f;
#pragma unroll
    for (int j = 0; j < CONV_MAX_TAPS; ++j) {
      acc0 = fmaf(w[j][0], win[j][0], acc0);
      acc1 = fmaf(w[j][1], win[j][1], acc1);
    }
    *reinterpret_cast<__nv_bfloat162*>(out + static_cast<long long>(t0 + k) * a.C + c) =
        __floats2bfloat162_rn(silu_f(acc0 + bias0), silu_f(acc1 + bias1));
  }
}

// After it: every request's last taps - 1 inputs go to its state.  A thread owns a channel of one request.
template <typename T>
__global__ void conv_state_update_kernel(const ConvArgs a) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x, row = blockIdx.y;
  if (c >= a.C) return;
  const int slot = a.slots[row];
  if (slot < 0 || slot >= a.num_slots) return;       // reported by the convolution
  float* state = a.state + static_cast<long long>(slot) * a.slot_stride;
  const T* x = static_cast<const T*>(a.x);
  const int t0 = a.row_q_start[row], n = a.row_q_len[row], keep = a.taps - 1;
  float last[CONV_MAX_TAPS];
#pragma unroll
  for (int j = 0; j < CONV_MAX_TAPS; ++j) {
    if (j < keep) {
      const int i = n - keep + j;                     // the input that becomes entry j
      last[j] = i >= 0 ? to_float(x[static_cast<long long>(t0 + i) * a.x_stride + c])
                       : state[static_cast<long long>(keep + i) * a.C + c];
    }
  }
#pragma unroll
  for (int j = 0; j < CONV_MAX_TAPS; ++j)
    if (j < keep) state[static_cast<long long>(j) * a.C + c] = last[j];
}

// ------------------------------------------------------------------------------------------------
// The recurrence.  A CTA owns one request, one head and 64 value columns; warp w owns the key
// channels 16 w .. 16 w + 15 of those columns, each lane two columns (32 apart) with their 2 x 16 state
// values in registers, so that a decay, key and query fetched from shared memory serve two columns (two warps per scheduler and more: one warp's shared-memory loads hide behind another's
// multiply-adds).  The tokens of the request are taken SCAN_CHUNK at a time: decays, keys, queries and
// values of the chunk lie in shared memory (all float32), every warp runs the chunk's tokens in
// order, and the warps' partial outputs are added in warp order.  While a chunk runs, the next one's
// inputs are already on their way into registers.  The gated form's decays are made beforehand, in
// place of their logits, by a kernel of their own (every CTA of a head would otherwise repeat them).
constexpr int SCAN_CHUNK = 16;
constexpr int SCAN_ROWS = 16;        // key channels per warp
constexpr int SCAN_COLS = 64;        // value columns per CTA: two a lane, 32 apart
constexpr int SCAN_V_REGS = SCAN_CHUNK * SCAN_COLS / 64;   // values a thread fetches ahead, at most (a CTA has two warps or more)

constexpr int SCAN_GATED = 0;        // a[d] given per key channel (made from the logits by gated_decay_kernel), q scaled
constexpr int SCAN_STATE_SPACE = 1;  // a = exp(-exp(A_log[h]) dt), k = dt B, q = C, o += skip[h] v, dt = softplus(. + dt_bias[h])

struct ScanArgs {
  const void* q; long long q_stride;   // [tokens, .]: head h (or its group) at column h * D
  const void* k; long long k_stride;
  const void* v; long long v_stride;   // [tokens, .]: head h at column h * V
  const float* z; long long z_stride;  // gated: decays [tokens, H * D], float32
  const void* dt; long long dt_stride; // state space: [tokens, H]
  const void* dt_bias; const void* a_log; const void* skip;   // state space: [H] each
  int w_dtype;
  float* state; long long slot_stride; // slot s at state + s * slot_stride: [H][D][V]
  float* out;                          // [tokens, H * V] float32
  const int* slots; const int* row_q_start; const int* row_q_len;
  int H, D, V, heads_per_group, num_slots, write_state;
  float q_scale;
  // Long requests in segments that run side by side (seg_len 0: every request is one piece).  Segment g of
  // a request covers its new tokens g seg_len .. (g + 1) seg_len - 1.  A first pass runs every segment
  // but a request's last from a zero state and leaves the state it ends with and the product of its
  // decays per key channel in ws_state / ws_decay; scan_carry_kernel turns those into the true state at
  // the start of every segment; the second pass runs every segment from there and writes the outputs.
  int seg_len, segs;                   // segs: segments per request in the grid (an upper bound)
  float* ws_state;                     // [rows * segs][H][D][V]
  float* ws_decay;                     // [rows * segs][H][D]
  int* status;
};

constexpr int SCAN_PASS_OUTPUT = 0;  // from the request's state (or a segment's start state), with outputs
constexpr int SCAN_PASS_LOCAL = 1;   // from zero, without outputs: what a segment adds, and its decays' product

// ws_state[g] <- the state at the start of segment g + 1: decay(g) * (state at the start of g) + ws_state[g].
__global__ void scan_carry_kernel(float* ws_state, const float* ws_decay, const float* state, long long slot_stride,
                                  const int* slots, const int* row_q_len, int segs, int seg_len, int H, int D, int V,
                                  int num_slots) {
  const long long per = static_cast<long long>(H) * D * V;
  const long long e = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  const int row = blockIdx.y;
  if (e >= per) return;
  const int slot = slots[row];
  if (slot < 0 || slot >= num_slots) return;
  const int used = (row_q_len[row] + seg_len - 1) / seg_len;
  const long long channel = e / V;                       // h * D + d
  float prev = state[static_cast<long long>(slot) * slot_stride + e];
  for (int g = 0; g + 1 < used; ++g) {
    const long long at = static_cast<long long>(row) * segs + g;
    prev = fmaf(ws_decay[at * H * D + channel], prev, ws_state[at * per + e]);
    ws_state[at * per + e] = prev;
  }
}

// z <- sigmoid(z + bias)^(1/tau), through the logarithm: exp(log_sigmoid(z + bias) / tau).
__global__ void gated_decay_kernel(float* z, long long z_stride, const void* bias, int w_dtype, int width, float inv_tau,
                                   long long count) {
  const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= count) return;
  const long long t = i / width;
  const int c = static_cast<int>(i - t * width);
  float* at = z + t * z_stride + c;
  *at = expf(log_sigmoid_f(*at + load_scale(bias, w_dtype, c)) * inv_tau);
}

template <typename T, int MODE, int PASS>
__global__ void __launch_bounds__(512) decayed_state_scan_kernel(const ScanArgs a) {
  extern __shared__ __align__(16) float scan_smem[];
  const int D = a.D, V = a.V, nwarps = blockDim.x >> 5, Dp = nwarps * SCAN_ROWS;     // blockDim.x == 2 Dp
  float* a_s = scan_smem;                                   // [SCAN_CHUNK][Dp]
  float* k_s = a_s + SCAN_CHUNK * Dp;                       // [SCAN_CHUNK][Dp]
  float* q_s = k_s + SCAN_CHUNK * Dp;                       // [SCAN_CHUNK][Dp]
  float* v_s = q_s + SCAN_CHUNK * Dp;                       // [SCAN_CHUNK][SCAN_COLS]
  float* o_s = v_s + SCAN_CHUNK * SCAN_COLS;                // [SCAN_CHUNK][nwarps][SCAN_COLS]
  float* step_s = o_s + SCAN_CHUNK * nwarps * SCAN_COLS;    // [2][SCAN_CHUNK]: state space: step sizes, decays
  const int v0 = blockIdx.x * SCAN_COLS, h = blockIdx.y;
  const int row = blockIdx.z / a.segs, seg = blockIdx.z - row * a.segs;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int slot = a.slots[row];
  if (slot < 0 || slot >= a.num_slots) {
    if (tid == 0 && seg == 0) report(a.status, STATUS_ROW_OUT_OF_RANGE, slot, row);
    return;
  }
  int t0 = a.row_q_start[row], n = a.row_q_len[row];
  bool last = true;
  if (a.seg_len > 0) {
    const int begin = seg * a.seg_len;
    last = begin + a.seg_len >= n;
    n = min(n, begin + a.seg_len) - begin;
    t0 += begin;
    if (n <= 0 || (PASS == SCAN_PASS_LOCAL && last)) return;      // nothing here, or nobody needs what it adds
  }
  const int col = v0 + lane, col2 = col + 32, d0 = warp * SCAN_ROWS;
  float* state = a.state + static_cast<long long>(slot) * a.slot_stride + static_cast<long long>(h) * D * V;
  const long long piece = static_cast<long long>(row) * a.segs + seg;
  // Where this piece starts from: zero, the state the carry left for it, or the request's slot.
  const float* from = PASS == SCAN_PASS_LOCAL ? nullptr
                      : (a.seg_len > 0 && seg > 0) ? a.ws_state + ((piece - 1) * a.H + h) * D * V : state;
  float S[SCAN_ROWS], S2[SCAN_ROWS], decay_product[PASS == SCAN_PASS_LOCAL ? SCAN_ROWS : 1];
#pragma unroll
  for (int d = 0; d < SCAN_ROWS; ++d) {
    S[d] = (from != nullptr && d0 + d < D && col < V) ? from[static_cast<long long>(d0 + d) * V + col] : 0.0f;
    S2[d] = (from != nullptr && d0 + d < D && col2 < V) ? from[static_cast<long long>(d0 + d) * V + col2] : 0.0f;
    if (PASS == SCAN_PASS_LOCAL) decay_product[d] = 1.0f;
  }

  const T* qp = static_cast<const T*>(a.q);
  const T* kp = static_cast<const T*>(a.k);
  const T* vp = static_cast<const T*>(a.v);
  const int qk_col = (MODE == SCAN_STATE_SPACE ? h / a.heads_per_group : h) * D;
  float head_decay = 0.0f, head_dt_bias = 0.0f, head_skip = 0.0f;
  if (MODE == SCAN_STATE_SPACE) {
    head_decay = -expf(load_scale(a.a_log, a.w_dtype, h));
    head_dt_bias = load_scale(a.dt_bias, a.w_dtype, h);
    head_skip = load_scale(a.skip, a.w_dtype, h);
  }

  // What this thread fetches ahead: one key channel of every second token of the chunk (the threads'
  // two halves take the even and the odd tokens), a share of the values, and (state space, the first
  // SCAN_CHUNK threads) a token's raw step size.
  constexpr int PER = SCAN_CHUNK / 2;
  const int my_d = tid < Dp ? tid : tid - Dp, my_t = tid < Dp ? 0 : 1;
  // Keys, queries, values and step sizes stay in their own type until they are stored to shared memory:
  // a conversion at the load would make the thread wait for the load there and then.
  float pa[PER];
  T pk[PER], pq[PER], pv[SCAN_V_REGS], pdt = from_float<T>(0.0f);
  auto fetch = [&](int c0) {
    const int nc = min(SCAN_CHUNK, n - c0);
#pragma unroll
    for (int j = 0; j < PER; ++j) {
      const int t = 2 * j + my_t;
      pa[j] = 0.0f;
      pk[j] = pq[j] = from_float<T>(0.0f);
      if (t < nc && my_d < D) {
        const long long tok = t0 + c0 + t;
        pk[j] = kp[tok * a.k_stride + qk_col + my_d];
        pq[j] = qp[tok * a.q_stride + qk_col + my_d];
        if (MODE == SCAN_GATED) pa[j] = a.z[tok * a.z_stride + h * D + my_d];
      }
    }
#pragma unroll
    for (int j = 0; j < SCAN_V_REGS; ++j) {
      const int e = tid + j * static_cast<int>(blockDim.x);
      pv[j] = from_float<T>(0.0f);
      if (e < SCAN_CHUNK * SCAN_COLS) {
        const int t = e / SCAN_COLS, c = v0 + (e - t * SCAN_COLS);
        if (t < nc && c < V) pv[j] = vp[static_cast<long long>(t0 + c0 + t) * a.v_stride + h * V + c];
      }
    }
    if (MODE == SCAN_STATE_SPACE && tid < nc)
      pdt = static_cast<const T*>(a.dt)[static_cast<long long>(t0 + c0 + tid) * a.dt_stride + h];
  };

  if (n > 0) fetch(0);
  for (int c0 = 0; c0 < n; c0 += SCAN_CHUNK) {
    const int nc = min(SCAN_CHUNK, n - c0);
    __syncthreads();                      // the chunk before is no longer read
    if (MODE == SCAN_STATE_SPACE) {
      if (tid < nc) {
        const float dt = softplus_f(to_float(pdt) + head_dt_bias);
        step_s[tid] = dt;
        step_s[SCAN_CHUNK + tid] = expf(head_decay * dt);
      }
      __syncthreads();
    }
#pragma unroll
    for (int j = 0; j < PER; ++j) {
      const int t = 2 * j + my_t, e = t * Dp + my_d;
      if (MODE == SCAN_GATED) {
        a_s[e] = pa[j];
        k_s[e] = to_float(pk[j]);
        q_s[e] = to_float(pq[j]) * a.q_scale;
      } else {
        a_s[e] = t < nc ? step_s[SCAN_CHUNK + t] : 0.0f;
        k_s[e] = t < nc ? to_float(pk[j]) * step_s[t] : 0.0f;
        q_s[e] = to_float(pq[j]);
      }
    }
#pragma unroll
    for (int j = 0; j < SCAN_V_REGS; ++j) {
      const int e = tid + j * static_cast<int>(blockDim.x);
      if (e < SCAN_CHUNK * SCAN_COLS) v_s[e] = to_float(pv[j]);
    }
    __syncthreads();
    if (c0 + SCAN_CHUNK < n) fetch(c0 + SCAN_CHUNK);      // lands while this chunk runs
    for (int t = 0; t < nc; ++t) {
      const float vt = v_s[t * SCAN_COLS + lane], vt2 = v_s[t * SCAN_COLS + 32 + lane];
      const float4* at = reinterpret_cast<const float4*>(a_s + t * Dp + d0);
      const float4* kt = reinterpret_cast<const float4*>(k_s + t * Dp + d0);
      const float4* qt = reinterpret_cast<const float4*>(q_s + t * Dp + d0);
      float o0 = 0.0f, o1 = 0.0f, o2 = 0.0f, o3 = 0.0f, p0 = 0.0f, p1 = 0.0f, p2 = 0.0f, p3 = 0.0f;
#pragma unroll
      for (int d4 = 0; d4 < SCAN_ROWS / 4; ++d4) {
        const float4 av = at[d4], kv = kt[d4], qv = qt[d4];
        const int d = 4 * d4;
        S[d] = fmaf(av.x, S[d], kv.x * vt);
        S[d + 1] = fmaf(av.y, S[d + 1], kv.y * vt);
        S[d + 2] = fmaf(av.z, S[d + 2], kv.z * vt);
        S[d + 3] = fmaf(av.w, S[d + 3], kv.w * vt);
        S2[d] = fmaf(av.x, S2[d], kv.x * vt2);
        S2[d + 1] = fmaf(av.y, S2[d + 1], kv.y * vt2);
        S2[d + 2] = fmaf(av.z, S2[d + 2], kv.z * vt2);
        S2[d + 3] = fmaf(av.w, S2[d + 3], kv.w * vt2);
        if (PASS == SCAN_PASS_LOCAL) {
          decay_product[d] *= av.x;
          decay_product[d + 1] *= av.y;
          decay_product[d + 2] *= av.z;
          decay_product[d + 3] *= av.w;
        } else {
          o0 = fmaf(S[d], qv.x, o0);
          o1 = fmaf(S[d + 1], qv.y, o1);
          o2 = fmaf(S[d + 2], qv.z, o2);
          o3 = fmaf(S[d + 3], qv.w, o3);
          p0 = fmaf(S2[d], qv.x, p0);
          p1 = fmaf(S2[d + 1], qv.y, p1);
          p2 = fmaf(S2[d + 2], qv.z, p2);
          p3 = fmaf(S2[d + 3], qv.w, p3);
        }
      }
      if (PASS != SCAN_PASS_LOCAL) {
        o_s[(t * nwarps + warp) * SCAN_COLS + lane] = (o0 + o1) + (o2 + o3);
        o_s[(t * nwarps + warp) * SCAN_COLS + 32 + lane] = (p0 + p1) + (p2 + p3);
      }
    }
    if (PASS == SCAN_PASS_LOCAL) continue;
    __syncthreads();
    for (int e = tid; e < nc * SCAN_COLS; e += blockDim.x) {
      const int t = e / SCAN_COLS, l = e - t * SCAN_COLS, c = v0 + l;
      if (c >= V) continue;
      float o = 0.0f;
      for (int w = 0; w < nwarps; ++w) o += o_s[(t * nwarps + w) * SCAN_COLS + l];
      if (MODE == SCAN_STATE_SPACE) o = fmaf(head_skip, v_s[t * SCAN_COLS + l], o);
      a.out[static_cast<long long>(t0 + c0 + t) * a.H * V + h * V + c] = o;
    }
  }
  if (PASS == SCAN_PASS_LOCAL) {
    float* to = a.ws_state + (piece * a.H + h) * D * V;
#pragma unroll
    for (int d = 0; d < SCAN_ROWS; ++d) {
      if (d0 + d < D && col < V) to[static_cast<long long>(d0 + d) * V + col] = S[d];
      if (d0 + d < D && col2 < V) to[static_cast<long long>(d0 + d) * V + col2] = S2[d];
      if (d0 + d < D && blockIdx.x == 0 && lane == 0) a.ws_decay[(piece * a.H + h) * D + d0 + d] = decay_product[d];
    }
  } else if (a.write_state && last) {
#pragma unroll
    for (int d = 0; d < SCAN_ROWS; ++d) {
      if (d0 + d < D && col < V) state[static_cast<long long>(d0 + d) * V + col] = S[d];
      if (d0 + d < D && col2 < V) state[static_cast<long long>(d0 + d) * V + col2] = S2[d];
    }
  }
}

// ------------------------------------------------------------------------------------------------
// RMS norm over equal groups of a float32 row with a SiLU gate: y = unit_rms(o * silu(g)) * w when the
// gate comes first, y = unit_rms(o) * w * silu(g) otherwise.  w has `w_len` entries and is used
// periodically (a scale per column, or one scale vector shared by all groups).  One warp per group.
template <typename T>
__global__ void gated_group_rms_norm_kernel(T* out, const float* o, const T* gate, long long gate_stride, const void* w,
                                            int w_dtype, int w_len, int width, int group, float eps, int gate_first,
                                            int tokens) {
  const int groups = width / group;
  const long long item = static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (item >= static_cast<long long>(tokens) * groups) return;
  const int lane = threadIdx.x & 31;
  const long long t = item / groups;
  const int c0 = static_cast<int>(item - t * groups) * group;
  float ss = 0.0f;
  for (int i = lane; i < group; i += 32) {
    float val = o[t * width + c0 + i];
    if (gate_first) val *= silu_f(to_float(gate[t * gate_stride + c0 + i]));
    ss = fmaf(val, val, ss);
  }
  const float r = 1.0f / sqrtf(warp_sum(ss) / static_cast<float>(group) + eps);
  for (int i = lane; i < group; i += 32) {
    const float g = silu_f(to_float(gate[t * gate_stride + c0 + i]));
    float val = o[t * width + c0 + i];
    if (gate_first) val *= g;
    val = val * r * load_scale(w, w_dtype, (c0 + i) % w_len);
    if (!gate_first) val *= g;
    out[t * width + c0 + i] = from_float<T>(val);
  }
}

// The same for groups of up to GN_VEC_MAX columns that are a multiple of four, with aligned rows: a lane
// keeps its share of the group in registers, so that o and the gate are read once.
constexpr int GN_VEC_ITEMS = 16;
constexpr int GN_VEC_MAX = 32 * GN_VEC_ITEMS * 4;

template <typename T>
__global__ void __launch_bounds__(128) gated_group_rms_norm_vec_kernel(T* out, const float* o, const T* gate, long long gate_stride,
                                                const float* w, int w_len, int width, int group, float eps,
                                                int gate_first, int tokens) {
  const int groups = width / group;
  const long long item = static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (item >= static_cast<long long>(tokens) * groups) return;
  const int lane = threadIdx.x & 31, nv = group / 4;
  const long long t = item / groups;
  const int c0 = static_cast<int>(item - t * groups) * group;
  // With the gate first only the product is kept; with the gate last, the unit-norm values, and the gate
  // is read again (a second time from the cache) when they are scaled.
  float4 val[GN_VEC_ITEMS];
  float ss = 0.0f;
#pragma unroll
  for (int j = 0; j < GN_VEC_ITEMS; ++j) {
    const int i = lane + 32 * j;
    if (i < nv) {
      val[j] = load4(o + t * width + c0 + 4 * i);
      if (gate_first) {
        const float4 raw = load4(gate + t * gate_stride + c0 + 4 * i);
        val[j] = make_float4(val[j].x * silu_f(raw.x), val[j].y * silu_f(raw.y), val[j].z * silu_f(raw.z),
                             val[j].w * silu_f(raw.w));
      }
      ss += (val[j].x * val[j].x + val[j].y * val[j].y) + (val[j].z * val[j].z + val[j].w * val[j].w);
    }
  }
  const float r = 1.0f / sqrtf(warp_sum(ss) / static_cast<float>(group) + eps);
#pragma unroll
  for (int j = 0; j < GN_VEC_ITEMS; ++j) {
    const int i = lane + 32 * j;
    if (i < nv) {
      const float4 wv = load4(w + (c0 + 4 * i) % w_len);
      float4 y = make_float4(val[j].x * r * wv.x, val[j].y * r * wv.y, val[j].z * r * wv.z, val[j].w * r * wv.w);
      if (!gate_first) {
        const float4 raw = load4(gate + t * gate_stride + c0 + 4 * i);
        y = make_float4(y.x * silu_f(raw.x), y.y * silu_f(raw.y), y.z * silu_f(raw.z), y.w * silu_f(raw.w));
      }
      store4(out + t * width + c0 + 4 * i, y);
    }
  }
}

// out = sa * a + sb * b, float32 arithmetic, one rounding; a and b may be float32 whatever out is.
template <typename IN, typename T>
__global__ void scaled_sum_kernel(T* out, const IN* a, const IN* b, float sa, float sb, long long n) {
  const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i < n) out[i] = from_float<T>(fmaf(sa, to_float(a[i]), sb * to_float(b[i])));
}

inline int norm_threads(int H) { return H >= 2048 ? 512 : (H >= 512 ? 256 : 128); }

template <typename K>
inline int allow_shared(K kernel, size_t bytes) {
  if (bytes > 227 * 1024) return ERR_UNSUPPORTED;
  if (bytes > 48 * 1024 &&
      cuda_failed(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(bytes))))
    return ERR_CUDA;
  return OK;
}

}  // namespace zb

using namespace zb;

// out [rows, H] (out_dtype) = LN(x [rows, H] (x_dtype)); scale and shift in w_dtype.
ZB_API int zb_layer_norm(void* out, const void* x, const void* w, const void* b, int w_dtype, float eps, int rows,
                         int H, int x_dtype, int out_dtype, void* stream) {
  if (rows < 0 || H <= 0) return ERR_BAD_ARGUMENT;
  if (rows == 0) return OK;
  auto s = static_cast<cudaStream_t>(stream);
  if (ln_vectors(H, w_dtype, {out, x, w, b})) {
    const float* wf = static_cast<const float*>(w);
    const float* bf = static_cast<const float*>(b);
    using bf16 = __nv_bfloat16;
    if (x_dtype == DTYPE_F32 && out_dtype == DTYPE_F32)
      layer_norm_vec_kernel<float, float><<<rows, LN_VEC_THREADS, 0, s>>>(static_cast<float*>(out), static_cast<const float*>(x), wf, bf, eps, H);
    else if (x_dtype == DTYPE_F32)
      layer_norm_vec_kernel<float, bf16><<<rows, LN_VEC_THREADS, 0, s>>>(static_cast<bf16*>(out), static_cast<const float*>(x), wf, bf, eps, H);
    else if (out_dtype == DTYPE_F32)
      layer_norm_vec_kernel<bf16, float><<<rows, LN_VEC_THREADS, 0, s>>>(static_cast<float*>(out), static_cast<const bf16*>(x), wf, bf, eps, H);
    else
      layer_norm_vec_kernel<bf16, bf16><<<rows, LN_VEC_THREADS, 0, s>>>(static_cast<bf16*>(out), static_cast<const bf16*>(x), wf, bf, eps, H);
    return launch_result();
  }
  const size_t smem = static_cast<size_t>(H) * sizeof(float);
  const int threads = norm_threads(H);
#define ZB_LN(X, T)                                                                                    \
  {                                                                                                    \
    auto kernel = layer_norm_kernel<X, T>;                                                             \
    if (int rc = allow_shared(kernel, smem)) return rc;                                                \
    kernel<<<rows, threads, smem, s>>>(static_cast<T*>(out), static_cast<const X*>(x), w, b, w_dtype, eps, H); \
  }
  if (x_dtype == DTYPE_F32 && out_dtype == DTYPE_F32) ZB_LN(float, float)
  else if (x_dtype == DTYPE_F32) ZB_LN(float, __nv_bfloat16)
  else if (out_dtype == DTYPE_F32) ZB_LN(__nv_bfloat16, float)
  else ZB_LN(__nv_bfloat16, __nv_bfloat16)
#undef ZB_LN
  return launch_result();
}

template <bool RMS>
static int residual_norm_launch(float* residual, const void* delta, const void* w1, const void* b1, float mult,
                                  void* out, const void* w2, const void* b2, int w_dtype, float eps1, float eps2,
                                  int rows, int H, int dtype, void* stream) {
  if (rows < 0 || H <= 0) return ERR_BAD_ARGUMENT;
  if (rows == 0) return OK;
  auto s = static_cast<cudaStream_t>(stream);
  if (ln_vectors(H, w_dtype, {residual, delta, out, w1, b1, w2, b2})) {
    const float* f1 = static_cast<const float*>(w1);
    const float* g1 = static_cast<const float*>(b1);
    const float* f2 = static_cast<const float*>(w2);
    const float* g2 = static_cast<const float*>(b2);
    if (dtype == DTYPE_F32)
      residual_layer_norm_vec_kernel<float, RMS><<<rows, LN_VEC_THREADS, 0, s>>>(
          residual, static_cast<const float*>(delta), f1, g1, mult, static_cast<float*>(out), f2, g2, eps1, eps2, H);
    else
      residual_layer_norm_vec_kernel<__nv_bfloat16, RMS><<<rows, LN_VEC_THREADS, 0, s>>>(
          residual, static_cast<const __nv_bfloat16*>(delta), f1, g1, mult, static_cast<__nv_bfloat16*>(out), f2, g2,
          eps1, eps2, H);
    return launch_result();
  }
  const size_t smem = static_cast<size_t>(H) * sizeof(float);
  const int threads = norm_threads(H);
  if (dtype == DTYPE_F32) {
    auto kernel = residual_layer_norm_kernel<float, RMS>;
    if (int rc = allow_shared(kernel, smem)) return rc;
    kernel<<<rows, threads, smem, s>>>(residual, static_cast<const float*>(delta), w1, b1, mult,
                                       static_cast<float*>(out), w2, b2, w_dtype, eps1, eps2, H);
  } else {
    auto kernel = residual_layer_norm_kernel<__nv_bfloat16, RMS>;
    if (int rc = allow_shared(kernel, smem)) return rc;
    kernel<<<rows, threads, smem, s>>>(residual, static_cast<const __nv_bfloat16*>(delta), w1, b1, mult,
                                       static_cast<__nv_bfloat16*>(out), w2, b2, w_dtype, eps1, eps2, H);
  }
  return launch_result();
}

ZB_API int zb_residual_layer_norm(float* residual, const void* delta, const void* w1, const void* b1, float mult,
                                  void* out, const void* w2, const void* b2, int w_dtype, float eps1, float eps2,
                                  int rows, int H, int dtype, void* stream) {
  return residual_norm_launch<false>(residual, delta, w1, b1, mult, out, w2, b2, w_dtype, eps1, eps2, rows, H, dtype, stream);
}

// residual += mult * RMSnorm(delta; w1); then out = RMSnorm(residual; w2), or with a null w2 the sum in delta's type.
ZB_API int zb_residual_rms_norm(float* residual, const void* delta, const void* w1, float mult, void* out,
                                const void* w2, int w_dtype, float eps1, float eps2, int rows, int H, int dtype,
                                void* stream) {
  return residual_norm_launch<true>(residual, delta, w1, nullptr, mult, out, w2, nullptr, w_dtype, eps1, eps2, rows, H, dtype, stream);
}

ZB_API int zb_embedding_f32(float* out, void* rounded, const void* table, const int* ids, float scale, int tokens,
                            int H, int V, int dtype, int* status, void* stream) {
  if (tokens < 0 || H <= 0 || V <= 0) return ERR_BAD_ARGUMENT;
  if (tokens == 0) return OK;
  auto s = static_cast<cudaStream_t>(stream);
  if (dtype == DTYPE_F32)
    embedding_f32_kernel<float><<<tokens, 128, 0, s>>>(out, static_cast<float*>(rounded), static_cast<const float*>(table),
                                                       ids, scale, H, V, status);
  else
    embedding_f32_kernel<__nv_bfloat16><<<tokens, 128, 0, s>>>(out, static_cast<__nv_bfloat16*>(rounded),
                                                               static_cast<const __nv_bfloat16*>(table), ids, scale, H, V,
                                                               status);
  return launch_result();
}

ZB_API int zb_causal_conv_silu(void* out, const void* x, long long x_stride, float* state, long long slot_stride,
                               const int* slots, const int* row_q_start, const int* row_q_len, const int* token_row,
                               int tokens, int rows, const void* w,
                               const void* bias, int w_dtype, int C, int taps, int num_slots, int write_state, int dtype,
                               int* status, void* stream) {
  if (rows < 0 || C <= 0 || taps <= 0) return ERR_BAD_ARGUMENT;
  if (taps > CONV_MAX_TAPS) return ERR_UNSUPPORTED;
  if (rows == 0) return OK;
  ConvArgs a;
  a.out = out; a.x = x; a.x_stride = x_stride; a.state = state; a.slot_stride = slot_stride; a.slots = slots;
  a.row_q_start = row_q_start; a.row_q_len = row_q_len; a.w = w; a.bias = bias; a.w_dtype = w_dtype; a.C = C;
  a.taps = taps; a.num_slots = num_slots; a.write_state = write_state; a.status = status;
  auto s = static_cast<cudaStream_t>(stream);
  if (tokens <= 0) return OK;
  const dim3 grid((tokens + CONV_TOKENS - 1) / CONV_TOKENS, (C + 127) / 128), per_row((C + 127) / 128, rows);
  if (dtype == DTYPE_F32) {
    causal_conv_silu_kernel<float><<<grid, 128, 0, s>>>(a, token_row, tokens);
    if (write_state && taps > 1) conv_state_update_kernel<float><<<per_row, 128, 0, s>>>(a);
  } else {
    const bool pairs = C % 2 == 0 && x_stride % 2 == 0 && slot_stride % 2 == 0 && w_dtype == DTYPE_F32 &&
                       reinterpret_cast<uintptr_t>(x) % 4 == 0 && reinterpret_cast<uintptr_t>(out) % 4 == 0 &&
                       reinterpret_cast<uintptr_t>(state) % 8 == 0;
    // Tiles pay where requests bring runs of tokens; a step of single tokens has nothing to slide over.
    if (pairs && tokens >= 4 * rows)
      causal_conv_silu_tile_kernel<<<dim3((tokens + CONV_TILE - 1) / CONV_TILE, (C / 2 + 63) / 64), 64, 0, s>>>(
          a, token_row, tokens);
    else
      causal_conv_silu_kernel<__nv_bfloat16><<<grid, 128, 0, s>>>(a, token_row, tokens);
    if (write_state && taps > 1) conv_state_update_kernel<__nv_bfloat16><<<per_row, 128, 0, s>>>(a);
  }
  return launch_result();
}

// The most key channels a head of the recurrence may have.
ZB_API int zb_state_scan_max_channels() { return 16 * SCAN_ROWS; }

// `z` (gated mode): decay logits [tokens, H * D] float32, overwritten with the decays.
ZB_API int zb_decayed_state_scan(float* out, const void* q, long long q_stride, const void* k, long long k_stride,
                                 const void* v, long long v_stride, float* z, long long z_stride,
                                 const void* z_bias, const void* dt, long long dt_stride, const void* dt_bias,
                                 const void* a_log, const void* skip, int w_dtype, float* state, long long slot_stride,
                                 const int* slots, const int* row_q_start, const int* row_q_len, int rows, int tokens,
                                 int H, int D, int V, int heads_per_group, int num_slots, int write_state,
                                 float q_scale, float inv_tau, int mode, int dtype, int seg_len, float* ws_state,
                                 float* ws_decay, int* status, void* stream) {
  if (rows < 0 || tokens < 0 || H <= 0 || D <= 0 || V <= 0 || heads_per_group <= 0 || seg_len < 0 ||
      (seg_len > 0 && (ws_state == nullptr || ws_decay == nullptr)))
    return ERR_BAD_ARGUMENT;
  if (D > 16 * SCAN_ROWS) return ERR_UNSUPPORTED;
  if (mode != SCAN_GATED && mode != SCAN_STATE_SPACE) return ERR_BAD_ARGUMENT;
  if (rows == 0 || tokens == 0) return OK;
  auto s = static_cast<cudaStream_t>(stream);
  if (mode == SCAN_GATED) {
    const long long count = static_cast<long long>(tokens) * H * D;
    gated_decay_kernel<<<static_cast<unsigned>((count + 255) / 256), 256, 0, s>>>(z, z_stride, z_bias, w_dtype, H * D,
                                                                                inv_tau, count);
  }
  ScanArgs a;
  a.q = q; a.q_stride = q_stride; a.k = k; a.k_stride = k_stride; a.v = v; a.v_stride = v_stride;
  a.z = z; a.z_stride = z_stride; a.dt = dt; a.dt_stride = dt_stride; a.dt_bias = dt_bias;
  a.a_log = a_log; a.skip = skip; a.w_dtype = w_dtype; a.state = state; a.slot_stride = slot_stride; a.out = out;
  a.slots = slots; a.row_q_start = row_q_start; a.row_q_len = row_q_len; a.H = H; a.D = D; a.V = V;
  a.heads_per_group = heads_per_group; a.num_slots = num_slots; a.write_state = write_state; a.q_scale = q_scale;
  a.status = status;
  a.seg_len = seg_len; a.segs = seg_len > 0 ? (tokens + seg_len - 1) / seg_len : 1;
  a.ws_state = ws_state; a.ws_decay = ws_decay;
  if (static_cast<long long>(rows) * a.segs > 65535) return ERR_UNSUPPORTED;
  const int warps = std::max(2, (D + SCAN_ROWS - 1) / SCAN_ROWS);
  const size_t smem = sizeof(float) * (3 * SCAN_CHUNK * warps * SCAN_ROWS + SCAN_CHUNK * SCAN_COLS +
                                       SCAN_CHUNK * warps * SCAN_COLS + 2 * SCAN_CHUNK);
  const dim3 grid((V + SCAN_COLS - 1) / SCAN_COLS, H, rows * a.segs);
#define ZB_SCAN(T, MODE)                                                                                       \
  {                                                                                                            \
    auto kernel = decayed_state_scan_kernel<T, MODE, SCAN_PASS_OUTPUT>;                                        \
    if (int rc = allow_shared(kernel, smem)) return rc;                                                        \
    if (seg_len > 0) {                                                                                         \
      auto local = decayed_state_scan_kernel<T, MODE, SCAN_PASS_LOCAL>;                                        \
      if (int rc = allow_shared(local, smem)) return rc;                                                       \
      local<<<grid, warps * 32, smem, s>>>(a);                                                                 \
      const long long per = static_cast<long long>(H) * D * V;                                                 \
      scan_carry_kernel<<<dim3(static_cast<unsigned>((per + 255) / 256), rows), 256, 0, s>>>(                  \
          ws_state, ws_decay, state, slot_stride, slots, row_q_len, a.segs, seg_len, H, D, V, num_slots);      \
    }                                                                                                          \
    kernel<<<grid, warps * 32, smem, s>>>(a);                                                                  \
  }
  if (dtype == DTYPE_F32) {
    if (mode == SCAN_GATED) ZB_SCAN(float, SCAN_GATED) else ZB_SCAN(float, SCAN_STATE_SPACE)
  } else {
    if (mode == SCAN_GATED) ZB_SCAN(__nv_bfloat16, SCAN_GATED) else ZB_SCAN(__nv_bfloat16, SCAN_STATE_SPACE)
  }
#undef ZB_SCAN
  return launch_result();
}

ZB_API int zb_gated_group_rms_norm(void* out, const float* o, const void* gate, long long gate_stride, const void* w,
                                   int w_dtype, int w_len, int tokens, int width, int group, float eps, int gate_first,
                                   int dtype, void* stream) {
  if (tokens < 0 || width <= 0 || group <= 0 || width % group != 0 || w_len <= 0) return ERR_BAD_ARGUMENT;
  if (tokens == 0) return OK;
  const long long items = static_cast<long long>(tokens) * (width / group);
  const int warps = 4;
  const unsigned blocks = static_cast<unsigned>((items + warps - 1) / warps);
  auto s = static_cast<cudaStream_t>(stream);
  const int elem = dtype == DTYPE_F32 ? 4 : 2;
  if (group % 4 == 0 && group <= GN_VEC_MAX && w_len % 4 == 0 && w_dtype == DTYPE_F32 && (gate_stride * elem) % (4 * elem) == 0 &&
      reinterpret_cast<uintptr_t>(gate) % (4 * elem) == 0 && reinterpret_cast<uintptr_t>(o) % 16 == 0 &&
      reinterpret_cast<uintptr_t>(out) % (4 * elem) == 0 && reinterpret_cast<uintptr_t>(w) % 16 == 0) {
    const float* wf = static_cast<const float*>(w);
    if (dtype == DTYPE_F32)
      gated_group_rms_norm_vec_kernel<float><<<blocks, warps * 32, 0, s>>>(
          static_cast<float*>(out), o, static_cast<const float*>(gate), gate_stride, wf, w_len, width, group, eps,
          gate_first, tokens);
    else
      gated_group_rms_norm_vec_kernel<__nv_bfloat16><<<blocks, warps * 32, 0, s>>>(
          static_cast<__nv_bfloat16*>(out), o, static_cast<const __nv_bfloat16*>(gate), gate_stride, wf, w_len, width,
          group, eps, gate_first, tokens);
    return launch_result();
  }
  if (dtype == DTYPE_F32)
    gated_group_rms_norm_kernel<float><<<blocks, warps * 32, 0, s>>>(
        static_cast<float*>(out), o, static_cast<const float*>(gate), gate_stride, w, w_dtype, w_len, width, group, eps,
        gate_first, tokens);
  else
    gated_group_rms_norm_kernel<__nv_bfloat16><<<blocks, warps * 32, 0, s>>>(
        static_cast<__nv_bfloat16*>(out), o, static_cast<const __nv_bfloat16*>(gate), gate_stride, w, w_dtype, w_len,
        width, group, eps, gate_first, tokens);
  return launch_result();
}

ZB_API int zb_scaled_sum(void* out, const void* a, const void* b, float sa, float sb, long long n, int in_dtype,
                         int dtype, void* stream) {
  if (n < 0) return ERR_BAD_ARGUMENT;
  if (n == 0) return OK;
  auto s = static_cast<cudaStream_t>(stream);
  const unsigned blocks = static_cast<unsigned>((n + 255) / 256);
  using bf16 = __nv_bfloat16;
  if (in_dtype == DTYPE_F32 && dtype == DTYPE_F32)
    scaled_sum_kernel<float, float><<<blocks, 256, 0, s>>>(static_cast<float*>(out), static_cast<const float*>(a),
                                                           static_cast<const float*>(b), sa, sb, n);
  else if (in_dtype == DTYPE_F32)
    scaled_sum_kernel<float, bf16><<<blocks, 256, 0, s>>>(static_cast<bf16*>(out), static_cast<const float*>(a),
                                                          static_cast<const float*>(b), sa, sb, n);
  else if (dtype == DTYPE_BF16)
    scaled_sum_kernel<bf16, bf16><<<blocks, 256, 0, s>>>(static_cast<bf16*>(out), static_cast<const bf16*>(a),
                                                         static_cast<const bf16*>(b), sa, sb, n);
  else
    return ERR_BAD_ARGUMENT;
  return launch_result();
}
