// Small parts around a float32 residual stream whose layers run their mixer and their feed-forward
// side by side on one norm's output.
//
//   hashed pair embedding   x[t] = E[id_t] + B[r_t],  r_t = (id_{t-1} * mul_prev + id_t * mul_cur) mod buckets,
//                           and r_t = buckets (the table's last row) for the first token of a sequence.
//                           The token before a step's first one is read from a per-request slot, which a
//                           second small kernel refreshes with the step's last token.
//   sum + RMS norm          x += (a + b) in float32 (either summand may be absent), then
//                           y = x / sqrt(mean(x^2) + eps) * w in the model's type; also the plain norm of
//                           float32 rows that are a slice of wider rows.
//   clamped gate            g = min(G + b_g, limit), u = clamp(U + b_u, -limit, limit),
//                           y = g * sigmoid(alpha * g) * (u + shift), from a float32 or bfloat16 product.
//   scale                   y *= s on float32 rows (a multiplier on logits).
#include "common.cuh"

#include <algorithm>

namespace zb {

// Four values at once: 16 bytes of float32 or 8 bytes of bfloat16.
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
template <typename T> inline bool aligned_for4(const void* p) {
  return reinterpret_cast<uintptr_t>(p) % (4 * sizeof(T)) == 0;
}

// ------------------------------------------------------------------------------ hashed pair embedding
template <typename T>
__global__ void __launch_bounds__(128)
pair_embedding_kernel(float* out, T* rounded, const T* table, const T* pair_table, const int* ids, const int* positions,
                      const int* token_row, const int* row_q_start, const int* state_slots, const int* last_token,
                      int H, int V, int buckets, long long mul_prev, long long mul_cur, int num_rows, int num_slots,
                      int vectors, int* status) {
  const int t = blockIdx.x;
  const int id = ids[t];
  if (id < 0 || id >= V) {
    if (threadIdx.x == 0) report(status, STATUS_TOKEN_OUT_OF_RANGE, id, t);
    return;
  }
  long long pair_row = buckets;                   // a sequence's first token has no token before it
  if (positions[t] > 0) {
    const int row = token_row[t];
    if (row < 0 || row >= num_rows) {
      if (threadIdx.x == 0) report(status, STATUS_ROW_OUT_OF_RANGE, row, t);
      return;
    }
    int prev;
    if (t == row_q_start[row]) {
      const int slot = state_slots[row];
      if (slot < 0 || slot >= num_slots) {
        if (threadIdx.x == 0) report(status, STATUS_ROW_OUT_OF_RANGE, slot, t);
        return;
      }
      prev = last_token[slot];
    } else {
      prev = ids[t - 1];
    }
    if (prev < 0 || prev >= V) {
      if (threadIdx.x == 0) report(status, STATUS_TOKEN_OUT_OF_RANGE, prev, t);
      return;
    }
    pair_row = (prev * mul_prev + id * mul_cur) % buckets;
  }
  const T* e = table + static_cast<long long>(id) * H;
  const T* p = pair_table + pair_row * H;
  float* o = out + static_cast<long long>(t) * H;
  if (vectors) {          // H a multiple of 4 and every base aligned for four values
    for (int i = 4 * threadIdx.x; i < H; i += 4 * blockDim.x) {
      const float4 a = load4(e + i), b = load4(p + i);
      const float4 v = make_float4(a.x + b.x, a.y + b.y, a.z + b.z, a.w + b.w);
      store4(o + i, v);
      if (rounded != nullptr) store4(rounded + static_cast<long long>(t) * H + i, v);
    }
    return;
  }
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    const float v = to_float(e[i]) + to_float(p[i]);
    o[i] = v;
    if (rounded != nullptr) rounded[static_cast<long long>(t) * H + i] = from_float<T>(v);
  }
}

__global__ void store_last_token_kernel(int* last_token, const int* ids, const int* row_q_start, const int* row_q_len,
                                        const int* state_slots, int num_rows, int num_slots) {
  const int r = blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= num_rows) return;
  const int slot = state_slots[r], n = row_q_len[r];
  if (slot < 0 || slot >= num_slots || n <= 0) return;
  last_token[slot] = ids[row_q_start[r] + n - 1];
}

// ------------------------------------------------------------------------------------ sum + RMS norm
// One CTA a row.  The row is summed into the stream first (and kept in registers where it fits), then
// normed.  PER: elements a thread keeps; rows longer than PER * threads re-read the stream.
constexpr int SN_THREADS = 256;
constexpr int SN_PER = 16;

template <typename A, typename B, typename OUT>
__global__ void __launch_bounds__(SN_THREADS)
sum_rms_norm_kernel(OUT* out, long long out_stride, float* x, long long x_stride, const A* a, const B* b,
                    const float* bias, const void* w, int w_dtype, float eps, int H) {
  __shared__ float scratch[33];
  const long long r = blockIdx.x;
  float* xr = x + r * x_stride;
  const A* ar = a != nullptr ? a + r * H : nullptr;
  const B* br = b != nullptr ? b + r * H : nullptr;
  const bool sums = ar != nullptr || br != nullptr;
  auto summed = [&](int i) {
    float v = xr[i];
    if (sums) {
      float s = (ar != nullptr ? to_float(ar[i]) : 0.0f) + (br != nullptr ? to_float(br[i]) : 0.0f);
      if (bias != nullptr) s += bias[i];
      v += s;
      xr[i] = v;
    }
    return v;
  };
  float keep[SN_PER];
  float ss = 0.0f;
#pragma unroll
  for (int k = 0; k < SN_PER; ++k) {
    const int i = threadIdx.x + k * SN_THREADS;
    keep[k] = i < H ? summed(i) : 0.0f;
    ss += keep[k] * keep[k];
  }
  for (int i = threadIdx.x + SN_PER * SN_THREADS; i < H; i += SN_THREADS) {
    const float v = summed(i);
    ss += v * v;
  }
  if (out == nullptr) return;
  const float inv = 1.0f / sqrtf(block_sum(ss, scratch) / static_cast<float>(H) + eps);
  OUT* o = out + r * out_stride;
#pragma unroll
  for (int k = 0; k < SN_PER; ++k) {
    const int i = threadIdx.x + k * SN_THREADS;
    if (i < H) o[i] = from_float<OUT>(keep[k] * inv * load_scale(w, w_dtype, i));
  }
  for (int i = threadIdx.x + SN_PER * SN_THREADS; i < H; i += SN_THREADS)
    o[i] = from_float<OUT>(xr[i] * inv * load_scale(w, w_dtype, i));
}

// The same with four values a thread and step: H a multiple of 4, every row and base aligned for that.
template <typename A, typename B, typename OUT>
__global__ void __launch_bounds__(SN_THREADS)
sum_rms_norm_vec_kernel(OUT* out, long long out_stride, float* x, long long x_stride, const A* a, const B* b,
                        const float* bias, const void* w, int w_dtype, float eps, int H) {
  __shared__ float scratch[33];
  const long long r = blockIdx.x;
  float* xr = x + r * x_stride;
  const A* ar = a != nullptr ? a + r * H : nullptr;
  const B* br = b != nullptr ? b + r * H : nullptr;
  const bool sums = ar != nullptr || br != nullptr;
  auto summed = [&](int i) {
    float4 v = load4(xr + i);
    if (sums) {
      const float4 p = ar != nullptr ? load4(ar + i) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
      const float4 q = br != nullptr ? load4(br + i) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
      float4 s = make_float4(p.x + q.x, p.y + q.y, p.z + q.z, p.w + q.w);
      if (bias != nullptr) {
        const float4 c = load4(bias + i);
        s.x += c.x; s.y += c.y; s.z += c.z; s.w += c.w;
      }
      v.x += s.x; v.y += s.y; v.z += s.z; v.w += s.w;
      store4(xr + i, v);
    }
    return v;
  };
  auto scaled = [&](float4 v, float inv, int i) {
    const float4 s = w_dtype == DTYPE_F32 ? load4(static_cast<const float*>(w) + i)
                                          : load4(static_cast<const __nv_bfloat16*>(w) + i);
    return make_float4(v.x * inv * s.x, v.y * inv * s.y, v.z * inv * s.z, v.w * inv * s.w);
  };
  constexpr int PER = SN_PER / 4;
  float4 keep[PER];
  float ss = 0.0f;
#pragma unroll
  for (int k = 0; k < PER; ++k) {
    const int i = 4 * (threadIdx.x + k * SN_THREADS);
    keep[k] = i < H ? summed(i) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    ss += keep[k].x * keep[k].x + keep[k].y * keep[k].y + keep[k].z * keep[k].z + keep[k].w * keep[k].w;
  }
  for (int i = 4 * (threadIdx.x + PER * SN_THREADS); i < H; i += 4 * SN_THREADS) {
    const float4 v = summed(i);
    ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
  }
  if (out == nullptr) return;
  const float inv = 1.0f / sqrtf(block_sum(ss, scratch) / static_cast<float>(H) + eps);
  OUT* o = out + r * out_stride;
#pragma unroll
  for (int k = 0; k < PER; ++k) {
    const int i = 4 * (threadIdx.x + k * SN_THREADS);
    if (i < H) store4(o + i, scaled(keep[k], inv, i));
  }
  for (int i = 4 * (threadIdx.x + PER * SN_THREADS); i < H; i += 4 * SN_THREADS) store4(o + i, scaled(load4(xr + i), inv, i));
}

// -------------------------------------------------------------------------------------- clamped gate
// One 16-byte load of gates and one of ups a thread and step (four outputs from float32 sums, eight from
// bfloat16): a warp's loads cover whole 32-byte sectors in either column order.  I a multiple of 8 and every
// base aligned to 16 bytes.
template <typename IN, typename OUT>
__global__ void __launch_bounds__(256)
clamped_gate_vec_kernel(OUT* out, const IN* gu, const float* bias, int T, int I, int blocked, float limit,
                        float alpha, float shift) {
  constexpr int PIECE = 16 / sizeof(IN);
  // A CTA walks rows, a thread pieces of its row: no division, and a row's pieces are neighbours.
  const int per_row = I / PIECE;
  const GateForm form{GATE_BOUNDED, bias, limit, alpha, shift};
  for (long long t = blockIdx.x; t < T; t += gridDim.x)
  for (int j = threadIdx.x; j < per_row; j += blockDim.x) {
    const int o0 = PIECE * j;
    const int gi = blocked ? (o0 >> 3) * 16 + (o0 & 7) : o0;
    const int ui = blocked ? gi + 8 : I + o0;
    const IN* row = gu + t * 2 * I;
    float g[PIECE], u[PIECE];
#pragma unroll
    for (int h = 0; h < PIECE / 4; ++h) {
      const float4 gv = load4(row + gi + 4 * h), uv = load4(row + ui + 4 * h);
      g[4 * h] = gv.x; g[4 * h + 1] = gv.y; g[4 * h + 2] = gv.z; g[4 * h + 3] = gv.w;
      u[4 * h] = uv.x; u[4 * h + 1] = uv.y; u[4 * h + 2] = uv.z; u[4 * h + 3] = uv.w;
    }
    if (bias != nullptr) {
#pragma unroll
      for (int h = 0; h < PIECE / 4; ++h) {
        const float4 gb = load4(bias + gi + 4 * h), ub = load4(bias + ui + 4 * h);
        g[4 * h] += gb.x; g[4 * h + 1] += gb.y; g[4 * h + 2] += gb.z; g[4 * h + 3] += gb.w;
        u[4 * h] += ub.x; u[4 * h + 1] += ub.y; u[4 * h + 2] += ub.z; u[4 * h + 3] += ub.w;
      }
    }
    float y[PIECE];
#pragma unroll
    for (int e = 0; e < PIECE; ++e)      // the fast exponential's 2^-21 vanishes in a bfloat16 result
      y[e] = sizeof(OUT) == 4 ? bounded_gate<false>(g[e], u[e], form) : bounded_gate<true>(g[e], u[e], form);
    OUT* dst = out + t * I + o0;
#pragma unroll
    for (int h = 0; h < PIECE / 4; ++h) store4(dst + 4 * h, make_float4(y[4 * h], y[4 * h + 1], y[4 * h + 2], y[4 * h + 3]));
  }
}

template <typename IN, typename OUT>
__global__ void __launch_bounds__(256)
clamped_gate_kernel(OUT* out, const IN* gu, const float* bias, long long total, int I, int blocked, float limit,
                    float alpha, float shift) {
  for (long long at = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; at < total;
       at += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long t = at / I;
    const int i = static_cast<int>(at - t * I);
    const int gi = blocked ? (i / 8) * 16 + (i % 8) : i;
    const int ui = blocked ? gi + 8 : I + i;
    float g = to_float(gu[t * 2 * I + gi]), u = to_float(gu[t * 2 * I + ui]);
    if (bias != nullptr) {
      g += bias[gi];
      u += bias[ui];
    }
    g = fminf(g, limit);
    u = fminf(fmaxf(u, -limit), limit);
    out[at] = from_float<OUT>(g / (1.0f + expf(-alpha * g)) * (u + shift));
  }
}

__global__ void scale_rows_kernel(float* y, long long total, float scale) {
  for (long long at = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; at < total;
       at += static_cast<long long>(gridDim.x) * blockDim.x)
    y[at] *= scale;
}

inline int grid_for(long long total, int threads) {
  return static_cast<int>(std::min<long long>((total + threads - 1) / threads, 148LL * 16));
}

}  // namespace zb

using namespace zb;

// out [T, H] float32 (and `rounded`, the same rows in the tables' type, unless null) = table[ids[t]] +
// pair_table[r_t]; pair_table has buckets + 1 rows.  last_token: int32 [num_slots].
ZB_API int zb_pair_embedding(float* out, void* rounded, const void* table, const void* pair_table, const int* ids,
                             const int* positions, const int* token_row, const int* row_q_start,
                             const int* state_slots, const int* last_token, int T, int H, int V, int buckets,
                             long long mul_prev, long long mul_cur, int num_rows, int num_slots, int dtype, int* status,
                             void* stream) {
  if (T < 0 || H <= 0 || V <= 0 || buckets <= 0 || mul_prev < 0 || mul_cur < 0 || num_rows < 0 || num_slots <= 0)
    return ERR_BAD_ARGUMENT;
  if (T == 0) return OK;
  auto s = static_cast<cudaStream_t>(stream);
  if (dtype == DTYPE_F32) {
    const int vectors = H % 4 == 0 && aligned_for4<float>(out) && aligned_for4<float>(table) &&
                        aligned_for4<float>(pair_table) && aligned_for4<float>(rounded);
    pair_embedding_kernel<float><<<T, 128, 0, s>>>(out, (float*)rounded, (const float*)table, (const float*)pair_table,
                                                   ids, positions, token_row, row_q_start, state_slots, last_token, H,
                                                   V, buckets, mul_prev, mul_cur, num_rows, num_slots, vectors, status);
  } else {
    using bf16 = __nv_bfloat16;
    const int vectors = H % 4 == 0 && aligned_for4<float>(out) && aligned_for4<bf16>(table) &&
                        aligned_for4<bf16>(pair_table) && aligned_for4<bf16>(rounded);
    pair_embedding_kernel<bf16><<<T, 128, 0, s>>>(
        out, (bf16*)rounded, (const bf16*)table, (const bf16*)pair_table, ids, positions, token_row, row_q_start,
        state_slots, last_token, H, V, buckets, mul_prev, mul_cur, num_rows, num_slots, vectors, status);
  }
  return launch_result();
}

// last_token[state_slots[r]] = the last of row r's new tokens.
ZB_API int zb_store_last_token(int* last_token, const int* ids, const int* row_q_start, const int* row_q_len,
                               const int* state_slots, int num_rows, int num_slots, void* stream) {
  if (num_rows < 0 || num_slots <= 0) return ERR_BAD_ARGUMENT;
  if (num_rows == 0) return OK;
  store_last_token_kernel<<<(num_rows + 127) / 128, 128, 0, static_cast<cudaStream_t>(stream)>>>(
      last_token, ids, row_q_start, row_q_len, state_slots, num_rows, num_slots);
  return launch_result();
}

// x [rows, H] float32 (rows x_stride apart) += (a + b + bias), a and b contiguous [rows, H] of their own types
// or null, bias float32 [H] (a shift of one of the summands, added to every row; only beside a summand) or
// null; then, unless out is null, out [rows, H] (rows out_stride apart) = rmsnorm(x) * w.
ZB_API int zb_sum_rms_norm(void* out, long long out_stride, int out_dtype, float* x, long long x_stride, const void* a,
                           int a_dtype, const void* b, int b_dtype, const float* bias, const void* w, int w_dtype,
                           float eps, int rows, int H, void* stream) {
  if (rows < 0 || H <= 0 || x_stride < H || (out != nullptr && (out_stride < H || w == nullptr)) ||
      (bias != nullptr && a == nullptr && b == nullptr))
    return ERR_BAD_ARGUMENT;
  if (rows == 0) return OK;
  auto s = static_cast<cudaStream_t>(stream);
  using bf16 = __nv_bfloat16;
  const int a_bytes = a_dtype == DTYPE_F32 ? 16 : 8, b_bytes = b_dtype == DTYPE_F32 ? 16 : 8;
  const int o_bytes = out_dtype == DTYPE_F32 ? 16 : 8, w_bytes = w_dtype == DTYPE_F32 ? 16 : 8;
  auto fits = [](const void* p, int bytes) { return reinterpret_cast<uintptr_t>(p) % bytes == 0; };
  const bool vectors = H % 4 == 0 && x_stride % 4 == 0 && out_stride % 4 == 0 && fits(x, 16) && fits(a, a_bytes) &&
                       fits(b, b_bytes) && fits(out, o_bytes) && fits(w, w_bytes) && fits(bias, 16);
#define ZB_SN(A_, B_, OUT_)                                                                                          \
  {                                                                                                                  \
    if (vectors)                                                                                                     \
      sum_rms_norm_vec_kernel<A_, B_, OUT_><<<rows, SN_THREADS, 0, s>>>((OUT_*)out, out_stride, x, x_stride,         \
                                                                         (const A_*)a, (const B_*)b, bias, w, w_dtype, eps, H); \
    else                                                                                                             \
      sum_rms_norm_kernel<A_, B_, OUT_><<<rows, SN_THREADS, 0, s>>>((OUT_*)out, out_stride, x, x_stride, (const A_*)a, \
                                                                     (const B_*)b, bias, w, w_dtype, eps, H);        \
  }
#define ZB_SN_OUT(A_, B_)                              \
  {                                                    \
    if (out_dtype == DTYPE_F32) ZB_SN(A_, B_, float)   \
    else ZB_SN(A_, B_, bf16)                           \
  }
  const bool a32 = a == nullptr || a_dtype == DTYPE_F32, b32 = b == nullptr || b_dtype == DTYPE_F32;
  if (a32 && b32) ZB_SN_OUT(float, float)
  else if (a32) ZB_SN_OUT(float, bf16)
  else if (b32) ZB_SN_OUT(bf16, float)
  else ZB_SN_OUT(bf16, bf16)
#undef ZB_SN_OUT
#undef ZB_SN
  return launch_result();
}

// out [T, I] = g * sigmoid(alpha g) * (u + shift) with g = min(G + bias_g, limit), u = clamp(U + bias_u, +-limit);
// gu [T, 2I] holds G then U, or with `blocked` blocks of 8 gate columns each followed by its 8 up columns;
// bias (float32 [2I], in gu's column order) may be null.
ZB_API int zb_clamped_gate(void* out, int out_dtype, const void* gu, int in_dtype, const float* bias, int T, int I,
                           int blocked, float limit, float alpha, float shift, void* stream) {
  if (T < 0 || I < 0 || (blocked && I % 8 != 0) || !(limit > 0.0f)) return ERR_BAD_ARGUMENT;
  if (out_dtype == DTYPE_F32 && in_dtype != DTYPE_F32) return ERR_BAD_ARGUMENT;
  const long long total = static_cast<long long>(T) * I;
  if (total == 0) return OK;
  auto s = static_cast<cudaStream_t>(stream);
  using bf16 = __nv_bfloat16;
  if (I % 8 == 0 && reinterpret_cast<uintptr_t>(gu) % 16 == 0 && reinterpret_cast<uintptr_t>(out) % 16 == 0 &&
      reinterpret_cast<uintptr_t>(bias) % 16 == 0) {
    int threads = (I / (in_dtype == DTYPE_F32 ? 4 : 8) + 31) / 32 * 32;
    threads = threads > 256 ? 256 : threads;
    const int blocks8 = T < 148 * 32 ? T : 148 * 32;
    if (out_dtype == DTYPE_F32)
      clamped_gate_vec_kernel<float, float><<<blocks8, threads, 0, s>>>((float*)out, (const float*)gu, bias, T, I, blocked, limit, alpha, shift);
    else if (in_dtype == DTYPE_F32)
      clamped_gate_vec_kernel<float, bf16><<<blocks8, threads, 0, s>>>((bf16*)out, (const float*)gu, bias, T, I, blocked, limit, alpha, shift);
    else
      clamped_gate_vec_kernel<bf16, bf16><<<blocks8, threads, 0, s>>>((bf16*)out, (const bf16*)gu, bias, T, I, blocked, limit, alpha, shift);
    return launch_result();
  }
  const int blocks = grid_for(total, 256);
  if (out_dtype == DTYPE_F32)
    clamped_gate_kernel<float, float><<<blocks, 256, 0, s>>>((float*)out, (const float*)gu, bias, total, I, blocked, limit, alpha, shift);
  else if (in_dtype == DTYPE_F32)
    clamped_gate_kernel<float, bf16><<<blocks, 256, 0, s>>>((bf16*)out, (const float*)gu, bias, total, I, blocked, limit, alpha, shift);
  else
    clamped_gate_kernel<bf16, bf16><<<blocks, 256, 0, s>>>((bf16*)out, (const bf16*)gu, bias, total, I, blocked, limit, alpha, shift);
  return launch_result();
}

ZB_API int zb_scale_rows(float* y, long long total, float scale, void* stream) {
  if (total < 0) return ERR_BAD_ARGUMENT;
  if (total == 0) return OK;
  scale_rows_kernel<<<grid_for(total, 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(y, total, scale);
  return launch_result();
}
