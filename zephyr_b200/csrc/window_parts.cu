// The pieces around attention whose rotation turns halves of part of a head, whose window is followed by
// pooled blocks, and whose heads' weights are mixed behind the softmax.
//
//   qkv_halves   from a fused q/k/v projection (float32 or the model's type) to queries and cache entries:
//                  an RMS norm of q and of k, either per head with one scale vector shared by the heads,
//                  or over ALL heads of the projection at once with a scale per column, or none;
//                  the rotation of halves on the first `rot_dims` values of every q and k head: value i
//                  pairs with value i + rot_dims / 2, (u, v) -> (u c - v s, v c + u s), c, s = cos, sin of
//                  position * f_i (float32 products, f a table the host made);
//                  optionally every value head divided by its root mean square (no scales);
//                  and the write of k and v into the pages.  One CTA per token; everything in float32
//                  with one rounding at the store.
//   pool_blocks  entry b of a pooled store = the mean over positions b P .. b P + P - 1 of the keys and
//                  values as the pages hold them, summed in float32 in the order of the positions; the
//                  CTA of the token that completes a block writes it.
//   head_mix     out[t, h] = sum_g M[h, g] * a[t, g, kv(h)], with a [T, heads, kv_heads, vd] float32 what
//                  every head's softmax weights make of every key/value head's values.
//   sigmoid_gate x[t, c] *= 1 / (1 + exp(-gate[t, c])), the gate float32 with strided rows.
#include "common.cuh"

namespace zb {

constexpr int QH_THREADS = 256;
constexpr int QH_WARPS = QH_THREADS / 32;

constexpr int NORM_NONE = 0;
constexpr int NORM_PER_HEAD = 1;     // scales [dim], shared by the heads (null: no scales)
constexpr int NORM_WHOLE = 2;        // one statistic over all heads, scales [heads * dim] (null: no scales)

struct QkvHalvesArgs {
  void* q_out;               // [T, nh * kd]
  const void* qkv;           // [T, stride]: q heads, k heads, v heads
  long long stride;
  int norm_mode;
  const float* q_norm_w;
  const float* k_norm_w;
  float eps;
  const float* freqs;        // null or [rot_dims / 2]
  int rot_dims;
  float rot_mult;            // a multiplier on cosine and sine
  int value_unit_norm;
  const int* positions;
  const int* token_row;
  void* cache;               // null: only the queries are made
  const int* block_table;
  int max_blocks, page_size, num_pages, num_rows;
  int nh, nkv, kd, vd;
  int* status;
};

template <typename IN, typename T>
__global__ void __launch_bounds__(QH_THREADS) qkv_halves_kernel(const QkvHalvesArgs a) {
  extern __shared__ __align__(16) float qh_smem[];
  const int t = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int kv_heads = a.cache != nullptr ? a.nkv : 0;
  const int q_cols = a.nh * a.kd, k_cols = kv_heads * a.kd, v_cols = kv_heads * a.vd;
  const int cols = q_cols + k_cols + v_cols, heads = a.nh + 2 * kv_heads;
  float* x = qh_smem;                    // [cols]
  float* head_ss = qh_smem + cols;       // [heads]
  const IN* src = static_cast<const IN*>(a.qkv) + static_cast<long long>(t) * a.stride;
  for (int i = threadIdx.x; i < cols; i += QH_THREADS) x[i] = to_float(src[i]);
  __syncthreads();
  // Every head's sum of squares, by one warp in lane order.
  for (int h = warp; h < heads; h += QH_WARPS) {
    const bool is_v = h >= a.nh + kv_heads;
    const int dim = is_v ? a.vd : a.kd;
    const float* row = x + (h < a.nh ? h * a.kd : (is_v ? q_cols + k_cols + (h - a.nh - kv_heads) * a.vd
                                                        : q_cols + (h - a.nh) * a.kd));
    float ss = 0.0f;
    for (int i = lane; i < dim; i += 32) ss = fmaf(row[i], row[i], ss);
    ss = warp_sum(ss);
    if (lane == 0) head_ss[h] = ss;
  }
  __syncthreads();
  const int pos = a.positions[t];
  int page = 0;
  if (a.cache != nullptr) {
    const int row = a.token_row[t], block = pos / a.page_size;
    if (row < 0 || row >= a.num_rows || block >= a.max_blocks) {
      if (threadIdx.x == 0) report(a.status, STATUS_ROW_OUT_OF_RANGE, row, t);
      return;
    }
    page = a.block_table[static_cast<long long>(row) * a.max_blocks + block];
    if (page <= 0 || page >= a.num_pages) {      // page 0 is the null page and is never written
      if (threadIdx.x == 0) report(a.status, STATUS_PAGE_OUT_OF_RANGE, page, t);
      return;
    }
  }
  const long long page_elems = static_cast<long long>(a.nkv) * a.page_size * (a.kd + a.vd);
  const int half = a.rot_dims / 2;
  for (int h = warp; h < heads; h += QH_WARPS) {
    const bool is_q = h < a.nh, is_v = h >= a.nh + kv_heads;
    const int dim = is_v ? a.vd : a.kd;
    const int own = is_q ? h : (is_v ? h - a.nh - kv_heads : h - a.nh);
    float* row = x + (is_q ? h * a.kd : (is_v ? q_cols + k_cols + own * a.vd : q_cols + own * a.kd));
    // The statistic: the head's own, or (q and k, whole mode) the sum over the projection's heads in head order.
    float inv = 1.0f;
    const float* w = nullptr;
    if (is_v) {
      if (a.value_unit_norm) inv = 1.0f / sqrtf(head_ss[h] / static_cast<float>(dim) + a.eps);
    } else if (a.norm_mode == NORM_PER_HEAD) {
      inv = 1.0f / sqrtf(head_ss[h] / static_cast<float>(dim) + a.eps);
      w = is_q ? a.q_norm_w : a.k_norm_w;
    } else if (a.norm_mode == NORM_WHOLE) {
      const int h0 = is_q ? 0 : a.nh, n = is_q ? a.nh : kv_heads;
      float total = 0.0f;
      for (int j = 0; j < n; ++j) total += head_ss[h0 + j];
      inv = 1.0f / sqrtf(total / static_cast<float>(n * dim) + a.eps);
      w = is_q ? a.q_norm_w : a.k_norm_w;
      if (w != nullptr) w += own * dim;
    }
    for (int i = lane; i < dim; i += 32) row[i] = row[i] * inv * (w != nullptr ? w[i] : 1.0f);
    __syncwarp();
    T* dst;
    int swizzle_pos = -1;          // -1: the row is stored as it is
    if (is_q) {
      dst = static_cast<T*>(a.q_out) + (static_cast<long long>(t) * a.nh + h) * a.kd;
    } else {
      const long long part = is_v ? static_cast<long long>(a.nkv) * a.page_size * a.kd : 0;
      dst = static_cast<T*>(a.cache) + static_cast<long long>(page) * page_elems + part +
            (static_cast<long long>(own) * a.page_size + pos % a.page_size) * dim;
      if ((dim * static_cast<int>(sizeof(T))) % 16 == 0) swizzle_pos = pos;
    }
    for (int i = lane; i < dim; i += 32) {
      float y = row[i];
      if (!is_v && a.freqs != nullptr && i < a.rot_dims) {
        const int f = i < half ? i : i - half;
        float s, c;
        sincosf(static_cast<float>(pos) * a.freqs[f], &s, &c);
        s *= a.rot_mult;
        c *= a.rot_mult;
        y = i < half ? row[i] * c - row[i + half] * s : row[i] * c + row[i - half] * s;
      }
      dst[swizzle_pos >= 0 ? kv_element_index(i, swizzle_pos, dim, sizeof(T)) : i] = from_float<T>(y);
    }
  }
}

// ------------------------------------------------------------------------------------------------
struct PoolBlocksArgs {
  const void* cache;          // the tokens' pages
  const int* block_table;     // [R, max_blocks]
  int max_blocks, num_pages;
  void* pool_cache;           // the pooled store's pages (same heads, widths and page size)
  const int* pool_table;      // [R, pool_max_blocks]
  int pool_max_blocks, pool_num_pages;
  const int* positions;
  const int* token_row;
  int num_rows, page_size, nkv, kd, vd, pool;
  int* status;
};

constexpr int POOL_PAGES_KEPT = 256;     // a block's pages are looked up once, up to this many positions

template <typename T>
__global__ void __launch_bounds__(128) pool_blocks_kernel(const PoolBlocksArgs a) {
  __shared__ int page_of[POOL_PAGES_KEPT];
  const int t = blockIdx.x;
  const int pos = a.positions[t];
  if ((pos + 1) % a.pool != 0) return;           // only the token that completes a block has work
  const int b = pos / a.pool, row = a.token_row[t];
  if (row < 0 || row >= a.num_rows) {
    if (threadIdx.x == 0) report(a.status, STATUS_ROW_OUT_OF_RANGE, row, t);
    return;
  }
  const int out_block = b / a.page_size;
  const int out_page = out_block < a.pool_max_blocks
                           ? a.pool_table[static_cast<long long>(row) * a.pool_max_blocks + out_block] : -1;
  if (out_page <= 0 || out_page >= a.pool_num_pages) {
    if (threadIdx.x == 0) report(a.status, STATUS_PAGE_OUT_OF_RANGE, out_page, t);
    return;
  }
  auto lookup = [&](int p) {
    const int block = p / a.page_size;
    const int page = block < a.max_blocks ? a.block_table[static_cast<long long>(row) * a.max_blocks + block] : -1;
    if (page <= 0 || page >= a.num_pages) {
      report(a.status, STATUS_PAGE_OUT_OF_RANGE, page, t);
      return 0;
    }
    return page;
  };
  for (int j = threadIdx.x; j < min(a.pool, POOL_PAGES_KEPT); j += blockDim.x) page_of[j] = lookup(b * a.pool + j);
  __syncthreads();
  const long long page_elems = static_cast<long long>(a.nkv) * a.page_size * (a.kd + a.vd);
  const long long value_part = static_cast<long long>(a.nkv) * a.page_size * a.kd;
  const T* cache = static_cast<const T*>(a.cache);
  T* pooled = static_cast<T*>(a.pool_cache);
  const float inv = 1.0f / static_cast<float>(a.pool);
  constexpr int vec = 16 / static_cast<int>(sizeof(T));
  if (a.kd % vec == 0 && a.vd % vec == 0) {
    // Rows of whole 16-byte pieces: a thread owns one piece of one head's key or value and walks the block.
    const int k_pieces = a.kd / vec, v_pieces = a.vd / vec, per_head = k_pieces + v_pieces;
    for (int e = threadIdx.x; e < a.nkv * per_head; e += blockDim.x) {
      const int kvh = e / per_head, c = e - kvh * per_head;
      const bool is_v = c >= k_pieces;
      const int dim = is_v ? a.vd : a.kd, pieces = is_v ? v_pieces : k_pieces, piece = is_v ? c - k_pieces : c;
      float sum[vec];
#pragma unroll
      for (int u = 0; u < vec; ++u) sum[u] = 0.0f;
      for (int j = 0; j < a.pool; ++j) {
        const int p = b * a.pool + j;
        const int page = j < POOL_PAGES_KEPT ? page_of[j] : lookup(p);
        if (page == 0) continue;
        const long long base = static_cast<long long>(page) * page_elems + (is_v ? value_part : 0) +
                               (static_cast<long long>(kvh) * a.page_size + p % a.page_size) * dim;
        const uint4 raw = *reinterpret_cast<const uint4*>(cache + base + (piece ^ kv_swizzle(p, pieces)) * vec);
        const T* values = reinterpret_cast<const T*>(&raw);
#pragma unroll
        for (int u = 0; u < vec; ++u) sum[u] += to_float(values[u]);
      }
      uint4 raw;
      T* values = reinterpret_cast<T*>(&raw);
#pragma unroll
      for (int u = 0; u < vec; ++u) values[u] = from_float<T>(sum[u] * inv);
      const long long base = static_cast<long long>(out_page) * page_elems + (is_v ? value_part : 0) +
                             (static_cast<long long>(kvh) * a.page_size + b % a.page_size) * dim;
      *reinterpret_cast<uint4*>(pooled + base + (piece ^ kv_swizzle(b, pieces)) * vec) = raw;
    }
    return;
  }
  const int per_head = a.kd + a.vd;
  for (int e = threadIdx.x; e < a.nkv * per_head; e += blockDim.x) {
    const int kvh = e / per_head, c = e - kvh * per_head;
    const bool is_v = c >= a.kd;
    const int dim = is_v ? a.vd : a.kd, i = is_v ? c - a.kd : c;
    const bool permuted = (dim * static_cast<int>(sizeof(T))) % 16 == 0;
    float sum = 0.0f;
    for (int j = 0; j < a.pool; ++j) {
      const int p = b * a.pool + j;
      const int page = j < POOL_PAGES_KEPT ? page_of[j] : lookup(p);
      if (page == 0) continue;
      const long long base = static_cast<long long>(page) * page_elems + (is_v ? value_part : 0) +
                             (static_cast<long long>(kvh) * a.page_size + p % a.page_size) * dim;
      sum += to_float(cache[base + (permuted ? kv_element_index(i, p, dim, sizeof(T)) : i)]);
    }
    const long long base = static_cast<long long>(out_page) * page_elems + (is_v ? value_part : 0) +
                           (static_cast<long long>(kvh) * a.page_size + b % a.page_size) * dim;
    pooled[base + (permuted ? kv_element_index(i, b, dim, sizeof(T)) : i)] = from_float<T>(sum * inv);
  }
}

// ------------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256)
head_mix_kernel(T* out, const float* a, const float* mix, int nh, int nkv, int vd) {
  extern __shared__ float mix_s[];       // [nh * nh]
  for (int i = threadIdx.x; i < nh * nh; i += blockDim.x) mix_s[i] = mix[i];
  __syncthreads();
  const long long t = blockIdx.x;
  const int g = nh / nkv;
  for (int e = threadIdx.x; e < nh * vd; e += blockDim.x) {
    const int h = e / vd, d = e - h * vd, own = h / g;
    float sum = 0.0f;
    for (int j = 0; j < nh; ++j)
      sum = fmaf(mix_s[h * nh + j], a[((t * nh + j) * nkv + own) * vd + d], sum);
    out[t * nh * vd + e] = from_float<T>(sum);
  }
}

template <typename T>
__global__ void __launch_bounds__(256)
sigmoid_gate_kernel(T* x, const float* gate, long long gate_stride, int width) {
  const long long t = blockIdx.x;
  for (int c = threadIdx.x; c < width; c += blockDim.x) {
    const float g = 1.0f / (1.0f + expf(-gate[t * gate_stride + c]));
    x[t * width + c] = from_float<T>(to_float(x[t * width + c]) * g);
  }
}

}  // namespace zb

using namespace zb;

ZB_API int zb_qkv_halves(void* q_out, const void* qkv, long long stride, int norm_mode, const float* q_norm_w,
                         const float* k_norm_w, float eps, const float* freqs, int rot_dims, float rot_mult,
                         int value_unit_norm, const int* positions, const int* token_row, void* cache,
                         const int* block_table, int max_blocks, int page_size, int num_pages, int num_rows,
                         int tokens, int nh, int nkv, int kd, int vd, int in_dtype, int dtype, int* status,
                         void* stream) {
  if (tokens < 0 || nh <= 0 || nkv <= 0 || kd <= 0 || vd <= 0 || rot_dims < 0 || rot_dims > kd || rot_dims % 2 != 0 ||
      page_size <= 0 || norm_mode < NORM_NONE || norm_mode > NORM_WHOLE || (norm_mode == NORM_NONE && (q_norm_w || k_norm_w)) ||
      ((q_norm_w == nullptr) != (k_norm_w == nullptr)))
    return ERR_BAD_ARGUMENT;
  if (dtype == DTYPE_F32 && in_dtype != DTYPE_F32) return ERR_BAD_ARGUMENT;
  if (tokens == 0) return OK;
  QkvHalvesArgs a;
  a.q_out = q_out; a.qkv = qkv; a.stride = stride; a.norm_mode = norm_mode; a.q_norm_w = q_norm_w;
  a.k_norm_w = k_norm_w; a.eps = eps; a.freqs = freqs; a.rot_dims = freqs != nullptr ? rot_dims : 0;
  a.rot_mult = rot_mult; a.value_unit_norm = value_unit_norm; a.positions = positions; a.token_row = token_row;
  a.cache = cache; a.block_table = block_table; a.max_blocks = max_blocks; a.page_size = page_size;
  a.num_pages = num_pages; a.num_rows = num_rows; a.nh = nh; a.nkv = nkv; a.kd = kd; a.vd = vd; a.status = status;
  const int kv_heads = cache != nullptr ? nkv : 0;
  const size_t smem = sizeof(float) * (static_cast<size_t>(nh) * kd + static_cast<size_t>(kv_heads) * (kd + vd) +
                                       nh + 2 * kv_heads);
  if (smem > 200 * 1024) return ERR_UNSUPPORTED;
  auto s = static_cast<cudaStream_t>(stream);
#define ZB_QH(IN, T)                                                                                            \
  {                                                                                                             \
    auto kernel = qkv_halves_kernel<IN, T>;                                                                     \
    if (smem > 48 * 1024 && cuda_failed(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                                                             static_cast<int>(smem))))                           \
      return ERR_CUDA;                                                                                          \
    kernel<<<tokens, QH_THREADS, smem, s>>>(a);                                                                 \
  }
  if (dtype == DTYPE_F32) ZB_QH(float, float)
  else if (in_dtype == DTYPE_F32) ZB_QH(float, __nv_bfloat16)
  else ZB_QH(__nv_bfloat16, __nv_bfloat16)
#undef ZB_QH
  return launch_result();
}

ZB_API int zb_pool_blocks(const void* cache, const int* block_table, int max_blocks, int num_pages, void* pool_cache,
                          const int* pool_table, int pool_max_blocks, int pool_num_pages, const int* positions,
                          const int* token_row, int tokens, int num_rows, int page_size, int nkv, int kd, int vd,
                          int pool, int dtype, int* status, void* stream) {
  if (tokens < 0 || nkv <= 0 || kd <= 0 || vd <= 0 || pool <= 0 || page_size <= 0 || max_blocks <= 0 ||
      pool_max_blocks <= 0)
    return ERR_BAD_ARGUMENT;
  if (tokens == 0) return OK;
  PoolBlocksArgs a;
  a.cache = cache; a.block_table = block_table; a.max_blocks = max_blocks; a.num_pages = num_pages;
  a.pool_cache = pool_cache; a.pool_table = pool_table; a.pool_max_blocks = pool_max_blocks;
  a.pool_num_pages = pool_num_pages; a.positions = positions; a.token_row = token_row; a.num_rows = num_rows;
  a.page_size = page_size; a.nkv = nkv; a.kd = kd; a.vd = vd; a.pool = pool; a.status = status;
  auto s = static_cast<cudaStream_t>(stream);
  if (dtype == DTYPE_F32) pool_blocks_kernel<float><<<tokens, 128, 0, s>>>(a);
  else pool_blocks_kernel<__nv_bfloat16><<<tokens, 128, 0, s>>>(a);
  return launch_result();
}

ZB_API int zb_head_mix(void* out, const float* a, const float* mix, int tokens, int nh, int nkv, int vd, int dtype,
                       void* stream) {
  if (tokens < 0 || nh <= 0 || nkv <= 0 || nh % nkv != 0 || vd <= 0) return ERR_BAD_ARGUMENT;
  const size_t smem = sizeof(float) * nh * nh;
  if (smem > 48 * 1024) return ERR_UNSUPPORTED;
  if (tokens == 0) return OK;
  auto s = static_cast<cudaStream_t>(stream);
  if (dtype == DTYPE_F32) head_mix_kernel<float><<<tokens, 256, smem, s>>>(static_cast<float*>(out), a, mix, nh, nkv, vd);
  else head_mix_kernel<__nv_bfloat16><<<tokens, 256, smem, s>>>(static_cast<__nv_bfloat16*>(out), a, mix, nh, nkv, vd);
  return launch_result();
}

ZB_API int zb_sigmoid_gate(void* x, const float* gate, long long gate_stride, int tokens, int width, int dtype,
                           void* stream) {
  if (tokens < 0 || width <= 0 || gate_stride < width) return ERR_BAD_ARGUMENT;
  if (tokens == 0) return OK;
  auto s = static_cast<cudaStream_t>(stream);
  if (dtype == DTYPE_F32) sigmoid_gate_kernel<float><<<tokens, 256, 0, s>>>(static_cast<float*>(x), gate, gate_stride, width);
  else sigmoid_gate_kernel<__nv_bfloat16><<<tokens, 256, 0, s>>>(static_cast<__nv_bfloat16*>(x), gate, gate_stride, width);
  return launch_result();
}
