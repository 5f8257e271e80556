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

// ------------------------------------------------------------------------------ hashed pair embedding
template <typename T>
__global__ void __launch_bounds__(128)
pair_embedding_kernel(float* out, T* rounded, const T* table, const T* pair_table, const int* ids, const int* positions,
                      const int* token_row, const int* row_q_start, const int* state_slots, const int* last_token,
                      int H, int V, int buckets, long long mul_prev, long long mul_cur, int num_rows, int num_slots,
                      int* status) {
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
                    const void* w, int w_dtype, float eps, int H) {
  __shared__ float scratch[33];
  const long long r = blockIdx.x;
  float* xr = x + r * x_stride;
  const A* ar = a != nullptr ? a + r * H : nullptr;
  const B* br = b != nullptr ? b + r * H : nullptr;
  float keep[SN_PER];
  float ss = 0.0f;
  int k = 0;
  for (int i = threadIdx.x; i < H; i += SN_THREADS, ++k) {
    float v = xr[i];
    if (ar != nullptr || br != nullptr) {
      const float s = (ar != nullptr ? to_float(ar[i]) : 0.0f) + (br != nullptr ? to_float(br[i]) : 0.0f);
      v += s;
      xr[i] = v;
    }
    if (k < SN_PER) keep[k] = v;
    ss += v * v;
  }
  if (out == nullptr) return;
  const float inv = 1.0f / sqrtf(block_sum(ss, scratch) / static_cast<float>(H) + eps);
  OUT* o = out + r * out_stride;
  k = 0;
  for (int i = threadIdx.x; i < H; i += SN_THREADS, ++k) {
    const float v = k < SN_PER ? keep[k] : xr[i];
    o[i] = from_float<OUT>(v * inv * load_scale(w, w_dtype, i));
  }
}

// -------------------------------------------------------------------------------------- clamped gate
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
  if (dtype == DTYPE_F32)
    pair_embedding_kernel<float><<<T, 128, 0, s>>>(out, (float*)rounded, (const float*)table, (const float*)pair_table,
                                                   ids, positions, token_row, row_q_start, state_slots, last_token, H,
                                                   V, buckets, mul_prev, mul_cur, num_rows, num_slots, status);
  else
    pair_embedding_kernel<__nv_bfloat16><<<T, 128, 0, s>>>(
        out, (__nv_bfloat16*)rounded, (const __nv_bfloat16*)table, (const __nv_bfloat16*)pair_table, ids, positions,
        token_row, row_q_start, state_slots, last_token, H, V, buckets, mul_prev, mul_cur, num_rows, num_slots, status);
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

// x [rows, H] float32 (rows x_stride apart) += (a + b), a and b contiguous [rows, H] of their own types or
// null; then, unless out is null, out [rows, H] (rows out_stride apart) = rmsnorm(x) * w.
ZB_API int zb_sum_rms_norm(void* out, long long out_stride, int out_dtype, float* x, long long x_stride, const void* a,
                           int a_dtype, const void* b, int b_dtype, const void* w, int w_dtype, float eps, int rows,
                           int H, void* stream) {
  if (rows < 0 || H <= 0 || x_stride < H || (out != nullptr && (out_stride < H || w == nullptr)))
    return ERR_BAD_ARGUMENT;
  if (rows == 0) return OK;
  auto s = static_cast<cudaStream_t>(stream);
  using bf16 = __nv_bfloat16;
#define ZB_SN(A_, B_, OUT_)                                                                                     \
  sum_rms_norm_kernel<A_, B_, OUT_><<<rows, SN_THREADS, 0, s>>>((OUT_*)out, out_stride, x, x_stride, (const A_*)a, \
                                                                 (const B_*)b, w, w_dtype, eps, H)
#define ZB_SN_OUT(A_, B_)                              \
  {                                                    \
    if (out_dtype == DTYPE_F32) ZB_SN(A_, B_, float);  \
    else ZB_SN(A_, B_, bf16);                          \
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
  const int blocks = grid_for(total, 256);
  using bf16 = __nv_bfloat16;
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
