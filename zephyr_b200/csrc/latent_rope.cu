// Latent attention with a rotated part: what a position keeps, and the rotated part of its queries.
//
// A position's projection holds `rank` latent values and behind them `rot` values of a key part that all
// heads share.  The latent is RMS-normed (float32, with a scale), the key part is rotated by the
// position's angles, and the two together form the one cached row of rank + rot values (a cache that
// keeps keys only; its first `rank` values serve as the values).  Every query head's last `rot` values
// are rotated the same way and written behind that head's `rank` latent-space values, so that one dot
// product over rank + rot values gives q_latent . c + q_rot . k_rot.
//
// Rotation of halves: value i pairs with value i + rot/2,
//   (u, v) -> (u c - v s, v c + u s),  c = m cos(p f_i), s = m sin(p f_i),
// the angle p f_i a float32 product, f a table of float32 frequencies made by the host, m one
// multiplier on both cosine and sine.  One CTA per token: the position's cosines and sines once, then a
// (head, pair) a thread for the queries, and the first warp for the cached row.
#include "common.cuh"

namespace zb {

constexpr int LR_THREADS = 128;
constexpr int LR_MAX_HALF = 256;     // rotated parts of up to 512 values

struct LatentRopeArgs {
  const float* kv;          // [T, kv_stride]: rank latent values, then rot key values
  long long kv_stride;
  const float* q;           // [T, q_stride]: heads of q_head_stride values, the rotated part at q_rot_offset
  long long q_stride;
  int q_head_stride, q_rot_offset;
  void* q_out;              // [T, nh * (rank + rot)]: this kernel fills the last rot values of every head
  const float* norm_w;      // [rank]
  float eps;
  const float* freqs;       // [rot / 2]
  float mult;
  const int* positions;
  const int* token_row;
  void* cache;              // null: the queries only
  const int* block_table;
  int max_blocks, page_size, num_pages, num_rows;
  int nh, rank, rot;
  int* status;
};

template <typename T>
__global__ void __launch_bounds__(LR_THREADS) latent_rope_kernel(const LatentRopeArgs a) {
  __shared__ float cos_of[LR_MAX_HALF], sin_of[LR_MAX_HALF];
  const int t = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int pos = a.positions[t], half = a.rot / 2, width = a.rank + a.rot;
  // The position's angles once for all heads.
  for (int i = threadIdx.x; i < half; i += LR_THREADS) {
    float s, c;
    sincosf(static_cast<float>(pos) * a.freqs[i], &s, &c);
    cos_of[i] = c * a.mult;
    sin_of[i] = s * a.mult;
  }
  __syncthreads();
  // The queries' rotated parts: one (head, pair) a thread and step.
  const float* q_row = a.q + static_cast<long long>(t) * a.q_stride + a.q_rot_offset;
  T* q_dst = static_cast<T*>(a.q_out) + static_cast<long long>(t) * a.nh * width + a.rank;
  for (int item = threadIdx.x; item < a.nh * half; item += LR_THREADS) {
    const int h = item / half, i = item - h * half;
    const float* src = q_row + static_cast<long long>(h) * a.q_head_stride;
    const float u = src[i], v = src[i + half], c = cos_of[i], s = sin_of[i];
    T* dst = q_dst + static_cast<long long>(h) * width;
    dst[i] = from_float<T>(u * c - v * s);
    dst[i + half] = from_float<T>(v * c + u * s);
  }
  if (a.cache == nullptr || warp != 0) return;
  // The cached row, by the first warp: the normed latent, then the rotated key part.
  const int row = a.token_row[t], block = pos / a.page_size;
  if (row < 0 || row >= a.num_rows || block >= a.max_blocks || pos < 0) {
    if (lane == 0) report(a.status, STATUS_ROW_OUT_OF_RANGE, row, t);
    return;
  }
  const int page = a.block_table[static_cast<long long>(row) * a.max_blocks + block];
  if (page <= 0 || page >= a.num_pages) {      // page 0 is the null page and is never written
    if (lane == 0) report(a.status, STATUS_PAGE_OUT_OF_RANGE, page, t);
    return;
  }
  T* dst = static_cast<T*>(a.cache) + (static_cast<long long>(page) * a.page_size + pos % a.page_size) * width;
  const bool swizzled = (width * static_cast<int>(sizeof(T))) % 16 == 0;
  const float* src = a.kv + static_cast<long long>(t) * a.kv_stride;
  float ss = 0.0f;
  for (int i = lane; i < a.rank; i += 32) ss += src[i] * src[i];
  const float inv = 1.0f / sqrtf(warp_sum(ss) / static_cast<float>(a.rank) + a.eps);
  for (int i = lane; i < a.rank; i += 32) {
    const int at = swizzled ? kv_element_index(i, pos, width, sizeof(T)) : i;
    dst[at] = from_float<T>(src[i] * inv * a.norm_w[i]);
  }
  for (int i = lane; i < half; i += 32) {
    const float u = src[a.rank + i], v = src[a.rank + i + half], c = cos_of[i], s = sin_of[i];
    const int lo = a.rank + i, hi = a.rank + i + half;
    dst[swizzled ? kv_element_index(lo, pos, width, sizeof(T)) : lo] = from_float<T>(u * c - v * s);
    dst[swizzled ? kv_element_index(hi, pos, width, sizeof(T)) : hi] = from_float<T>(v * c + u * s);
  }
}

}  // namespace zb

using namespace zb;

ZB_API int zb_latent_rope(void* q_out, const float* q, long long q_stride, int q_head_stride, int q_rot_offset,
                          const float* kv, long long kv_stride, const float* norm_w, float eps, const float* freqs,
                          float mult, const int* positions, const int* token_row, void* cache, const int* block_table,
                          int max_blocks, int page_size, int num_pages, int num_rows, int tokens, int nh, int rank,
                          int rot, int dtype, int* status, void* stream) {
  if (tokens < 0 || nh < 0 || rank <= 0 || rot < 0 || rot % 2 != 0 || page_size <= 0 || (rot > 0 && freqs == nullptr) ||
      (nh > 0 && (q == nullptr || q_out == nullptr)) || (cache != nullptr && (kv == nullptr || norm_w == nullptr)))
    return ERR_BAD_ARGUMENT;
  if (rot > 2 * LR_MAX_HALF) return ERR_UNSUPPORTED;
  if (tokens == 0) return OK;
  LatentRopeArgs a;
  a.kv = kv; a.kv_stride = kv_stride; a.q = q; a.q_stride = q_stride; a.q_head_stride = q_head_stride;
  a.q_rot_offset = q_rot_offset; a.q_out = q_out; a.norm_w = norm_w; a.eps = eps; a.freqs = freqs; a.mult = mult;
  a.positions = positions; a.token_row = token_row; a.cache = cache; a.block_table = block_table;
  a.max_blocks = max_blocks; a.page_size = page_size; a.num_pages = num_pages; a.num_rows = num_rows; a.nh = nh;
  a.rank = rank; a.rot = rot; a.status = status;
  auto s = static_cast<cudaStream_t>(stream);
  if (dtype == DTYPE_F32) latent_rope_kernel<float><<<tokens, LR_THREADS, 0, s>>>(a);
  else latent_rope_kernel<__nv_bfloat16><<<tokens, LR_THREADS, 0, s>>>(a);
  return launch_result();
}
