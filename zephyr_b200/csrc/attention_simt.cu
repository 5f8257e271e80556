// Paged causal attention on CUDA cores, float32 arithmetic throughout: the kernel of the true
// 32-bit path, and the general one (any head size up to 512, and up to 768 where the keys are the
// values too; any head and group counts, any page size, with or without a window, any mixture of
// prompt portions and single decoded tokens).
//
// Math (reference: deps/ttl/src/kernels/attention/attention.cu:46-56,76-77,90-166): query head j
// uses key/value head j / g; s = scale * (q . k) with scale = 1/sqrt(hd); a query at absolute
// position p sees the keys of its own sequence at positions <= p (and > p - window when the
// layer has a window); softmax with a running maximum; o = sum softmax * v.  There is no epsilon
// in the denominator and exp is expf.  A position encoding that is a bias on the scores, linear
// in the distance (a slope per query head), is added here; the one architecture has none, and
// the faster kernels do not take one.
//
// Keys and values may differ in width (kd, vd): a page holds its keys [nkv][page_size][kd] and behind
// them its values [nkv][page_size][vd].  Two more masks and one more term of the softmax are taken as
// parameters: `chunk` > 0 lets a query at position p see only keys j with j / chunk == p / chunk
// (chunks counted from position 0 of the sequence); `sinks` (one float32 per query head) adds
// exp(sink) to the softmax's denominator, a term without key or value that is not scaled.
//
// `softcap` > 0 bounds the scaled scores smoothly: s <- softcap * tanh(s / softcap).  `shared_kv`: the
// cache keeps keys only and they serve as the values too (kd = vd; a page is [nkv][page_size][kd]).
//
// A window may keep the first tokens of a sequence for good (`keep_first` = n: key j < n is seen by every
// later query, at its true position), and may be followed by pooled blocks (`pool` = P: a second paged
// store holds one entry per block of P positions, entry b standing for positions b P .. b P + P - 1; a
// query at position i sees entry b if b P + P - 1 <= i - window, that is the first
// floor((i - window + 1) / P) entries, in the same softmax as the tokens of its window).
//
// `cross_values`: every query head's weights are applied to the values of EVERY key/value head, not
// only its own: the result is [T, nh, nkv, vd] (a mixing of the heads' weights behind the softmax is a
// linear map of these).  `out_f32`: the result is written as float32 whatever the cache's type.
//
// One CTA serves one tile: a run of consecutive new tokens of one request, one key/value head,
// and a chunk of that head's query heads.  The (token, head) pairs of the tile are dealt to the
// warps; key/value tiles of 32 positions are staged in shared memory once and used by all pairs.
#include "common.cuh"

namespace zb {

constexpr int ATT_WARPS = 4;
constexpr int ATT_PAIRS_PER_WARP = 4;
constexpr int ATT_MAX_PAIRS = ATT_WARPS * ATT_PAIRS_PER_WARP;   // 16 (token, head) pairs per CTA
constexpr int ATT_TILE = 32;                                    // keys per shared-memory tile

struct AttentionArgs {
  const void* q;            // [T, nh*kd]
  void* out;                // [T, nh*vd]
  const void* kv_cache;     // [num_pages]{[nkv][page_size][kd], [nkv][page_size][vd]}
  const int* block_table;   // [R, max_blocks]
  const int* tile_row;      // [n_tiles] request row of the tile
  const int* tile_q0;       // [n_tiles] offset of the tile's first token within the row's new tokens
  const int* row_q_start;   // [R] index of the row's first new token in the flattened stream
  const int* row_q_len;     // [R]
  const int* row_ctx;       // [R] tokens already in the cache before this step
  int max_blocks, page_size, num_pages, num_rows;
  int nh, nkv, kd, vd, window, chunk, tile_tokens, heads_per_chunk;
  float scale;
  float softcap;             // 0: none
  int shared_kv;             // the keys are the values
  int keep_first;            // with a window: keys below this position stay visible
  int pool;                  // 0, or the positions per entry of the pooled store
  const void* pool_cache;    // the pooled store's pages, laid out as kv_cache
  const int* pool_table;     // [R, pool_max_blocks]
  int pool_max_blocks, pool_num_pages;
  int cross_values;          // grid y = nkv * nkv: (key head, value head) pairs; out [T, nh, nkv, vd]
  int out_f32;
  const float* sinks;        // null, or [nh]: exp(sinks[h]) joins the denominator of head h's softmax
  const float* head_slopes;  // null, or [nh]: query head h adds head_slopes[h] * (key position - query position) to its scores
  int* status;
};

template <typename T> struct KPad;
template <> struct KPad<float> { static constexpr int N = 1; };
template <> struct KPad<__nv_bfloat16> { static constexpr int N = 2; };

// Rows k0 .. k0 + ATT_TILE - 1 of one key/value head (keys or values: `part` is where that half
// begins inside a page, `dim` its width) into shared memory, un-permuted; zeros outside [lo, hi).
// Rows whose bytes are a multiple of 16 are stored with permuted 16-byte chunks (common.cuh:
// kv_swizzle) and move as vectors; any other width is stored as it is and moves element by element.
template <typename T>
__device__ __forceinline__ void stage_rows(T* dst, int dst_stride, const T* cache, const int* table, int max_blocks,
                                           int num_pages, const AttentionArgs& a, int row,
                                           int kvh, int k0, int lo, int hi, int dim, long long page_elems,
                                           long long part, int tok0) {
  constexpr int vec = 16 / static_cast<int>(sizeof(T));
  const bool vectors = dim % vec == 0;
  const int per_row = vectors ? dim / vec : dim;
  for (int e = threadIdx.x; e < ATT_TILE * per_row; e += blockDim.x) {
    const int j = e / per_row, c = e - j * per_row;
    const int pos = k0 + j;
    bool ok = pos >= lo && pos < hi;
    long long base = 0;
    if (ok) {
      const int block = pos / a.page_size;
      const int page = block < max_blocks ? table[static_cast<size_t>(row) * max_blocks + block] : -1;
      if (page <= 0 || page >= num_pages) {
        report(a.status, STATUS_PAGE_OUT_OF_RANGE, page, tok0);
        ok = false;
      } else {
        base = static_cast<long long>(page) * page_elems + part +
               (static_cast<long long>(kvh) * a.page_size + pos % a.page_size) * dim;
      }
    }
    if (vectors) {
      uint4 r = make_uint4(0, 0, 0, 0);
      if (ok) r = *reinterpret_cast<const uint4*>(cache + base + ((c ^ kv_swizzle(pos, per_row)) * vec));
      const T* re = reinterpret_cast<const T*>(&r);
#pragma unroll
      for (int u = 0; u < vec; ++u) dst[j * dst_stride + c * vec + u] = re[u];
    } else {
      dst[j * dst_stride + c] = ok ? cache[base + c] : from_float<T>(0.0f);
    }
  }
}

template <typename T, int ACC>
__global__ void __launch_bounds__(ATT_WARPS * 32)
paged_attention_simt_kernel(const AttentionArgs a) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int kd = a.kd, vd = a.vd, g = a.nh / a.nkv;
  const int kstride = kd + KPad<T>::N;
  float* q_s = reinterpret_cast<float*>(smem_raw);                       // [ATT_MAX_PAIRS][kd]
  T* k_s = reinterpret_cast<T*>(q_s + ATT_MAX_PAIRS * kd);               // [ATT_TILE][kstride]
  T* v_s = a.shared_kv ? k_s : k_s + ATT_TILE * kstride;                  // [ATT_TILE][vd], or the keys again
  const int vstride = a.shared_kv ? kstride : vd;

  const int tile = blockIdx.x, chunk = blockIdx.z;
  const int kvh = a.cross_values ? blockIdx.y % a.nkv : blockIdx.y;      // whose keys
  const int vh = a.cross_values ? blockIdx.y / a.nkv : kvh;              // whose values
  const int row = a.tile_row[tile], q0 = a.tile_q0[tile];
  if (row < 0 || row >= a.num_rows) {
    if (threadIdx.x == 0) report(a.status, STATUS_ROW_OUT_OF_RANGE, row, tile);
    return;
  }
  const int q_len = a.row_q_len[row], ctx = a.row_ctx[row], tok0 = a.row_q_start[row] + q0;
  const int n_tok = min(a.tile_tokens, q_len - q0);
  const int n_heads = min(a.heads_per_chunk, g - chunk * a.heads_per_chunk);
  if (n_tok <= 0 || n_heads <= 0) return;
  const int n_pairs = n_tok * n_heads;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const T* q = static_cast<const T*>(a.q);
  const T* cache = static_cast<const T*>(a.kv_cache);

  // Queries of all pairs, as float32.
  for (int e = threadIdx.x; e < n_pairs * kd; e += blockDim.x) {
    const int p = e / kd, d = e - p * kd;
    const int qi = p / n_heads, hj = p - qi * n_heads;
    const int head = kvh * g + chunk * a.heads_per_chunk + hj;
    q_s[p * kd + d] = to_float(q[(static_cast<size_t>(tok0 + qi) * a.nh + head) * kd + d]);
  }

  float m[ATT_PAIRS_PER_WARP], l[ATT_PAIRS_PER_WARP], acc[ATT_PAIRS_PER_WARP][ACC];
#pragma unroll
  for (int i = 0; i < ATT_PAIRS_PER_WARP; ++i) {
    m[i] = -INFINITY;
    l[i] = 0.0f;
#pragma unroll
    for (int c = 0; c < ACC; ++c) acc[i][c] = 0.0f;
  }

  // Keys any pair of this tile may see: [lo, hi), before them the kept first tokens [0, kept) and the
  // first `entries` entries of the pooled store.
  const int hi = ctx + q0 + n_tok;
  int lo = a.window > 0 ? max(0, ctx + q0 - a.window + 1) : 0;
  if (a.chunk > 0) lo = max(lo, (ctx + q0) / a.chunk * a.chunk);
  const int kept = a.window > 0 ? min(a.keep_first, lo) : 0;
  const int entries = (a.pool > 0 && a.window > 0) ? max(0, (hi - 1 - a.window + 1) / a.pool) : 0;
  const long long page_elems = static_cast<long long>(a.nkv) * a.page_size * (a.shared_kv ? kd : kd + vd);
  const long long value_part = static_cast<long long>(a.nkv) * a.page_size * kd;

  // Three runs of keys share the softmax: pooled entries, kept first tokens, the window.
  for (int run = 0; run < 3; ++run) {
    const int run_lo = run == 2 ? lo : 0;
    const int run_hi = run == 0 ? entries : (run == 1 ? kept : hi);
    if (run_hi <= run_lo) continue;
    const T* source = run == 0 ? static_cast<const T*>(a.pool_cache) : cache;
    const int* table = run == 0 ? a.pool_table : a.block_table;
    const int max_blocks = run == 0 ? a.pool_max_blocks : a.max_blocks;
    const int num_pages = run == 0 ? a.pool_num_pages : a.num_pages;
    for (int k0 = run_lo / ATT_TILE * ATT_TILE; k0 < run_hi; k0 += ATT_TILE) {
      __syncthreads();     // the previous tile is no longer read (and q_s is complete on the first pass)
      // Positions outside [run_lo, run_hi) hold zeros: a page that was given back, or one that another
      // request used before, is never read.
      stage_rows<T>(k_s, kstride, source, table, max_blocks, num_pages, a, row, kvh, k0, run_lo, run_hi, kd,
                    page_elems, 0, tok0);
      if (!a.shared_kv)
        stage_rows<T>(v_s, vd, source, table, max_blocks, num_pages, a, row, vh, k0, run_lo, run_hi, vd, page_elems,
                      value_part, tok0);
      __syncthreads();

      const int kp = k0 + lane;
#pragma unroll
      for (int i = 0; i < ATT_PAIRS_PER_WARP; ++i) {
        const int p = warp + i * ATT_WARPS;
        if (p >= n_pairs) continue;                       // uniform over the warp
        const int qpos = ctx + q0 + p / n_heads;
        const float slope = a.head_slopes != nullptr
                                ? a.head_slopes[kvh * g + chunk * a.heads_per_chunk + (p - p / n_heads * n_heads)] : 0.0f;
        int first = a.window > 0 ? max(0, qpos - a.window + 1) : 0;
        if (a.chunk > 0) first = max(first, qpos / a.chunk * a.chunk);
        bool valid;
        if (run == 0) {
          const int seen = max(0, (qpos - a.window + 1) / a.pool);      // entries this query sees
          if (k0 >= seen) continue;
          valid = kp < seen;
        } else if (run == 1) {
          valid = kp < kept;                                            // below every window of the tile
        } else {
          if (k0 > qpos || (k0 + ATT_TILE <= first && k0 >= a.keep_first)) continue;  // no key of this tile is visible
          valid = kp >= lo && kp <= qpos && (kp >= first || kp < a.keep_first);
        }
        float s = 0.0f;
        const float* qp = q_s + p * kd;
        const T* kr = k_s + lane * kstride;
        for (int d = 0; d + 1 < kd; d += 2) {
          s = fmaf(qp[d], to_float(kr[d]), s);
          s = fmaf(qp[d + 1], to_float(kr[d + 1]), s);
        }
        if (kd & 1) s = fmaf(qp[kd - 1], to_float(kr[kd - 1]), s);
        s *= a.scale;
        if (a.softcap > 0.0f) s = a.softcap * tanhf(s / a.softcap);
        s = valid ? (run == 2 ? fmaf(slope, static_cast<float>(kp - qpos), s) : s) : -INFINITY;
        const float tile_m = warp_max(s);
        if (tile_m == -INFINITY) continue;                 // (a tile of the window that this query has passed)
        const float new_m = fmaxf(m[i], tile_m);
        const float pr = valid ? expf(s - new_m) : 0.0f;
        const float corr = expf(m[i] - new_m);             // exp(-inf) = 0 on the first tile
        l[i] = l[i] * corr + warp_sum(pr);
        m[i] = new_m;
#pragma unroll
        for (int c = 0; c < ACC; ++c) acc[i][c] *= corr;
        for (int j = 0; j < ATT_TILE; ++j) {
          const float pj = __shfl_sync(0xffffffffu, pr, j);
          if (pj == 0.0f) continue;                         // uniform over the warp
#pragma unroll
          for (int c = 0; c < ACC; ++c) {
            const int d = lane + 32 * c;
            if (d < vd) acc[i][c] = fmaf(pj, to_float(v_s[j * vstride + d]), acc[i][c]);
          }
        }
      }
    }
  }

  T* out = static_cast<T*>(a.out);
#pragma unroll
  for (int i = 0; i < ATT_PAIRS_PER_WARP; ++i) {
    const int p = warp + i * ATT_WARPS;
    if (p >= n_pairs) continue;
    const int qi = p / n_heads, hj = p - qi * n_heads;
    const int head = kvh * g + chunk * a.heads_per_chunk + hj;
    float denominator = l[i], keep = 1.0f;
    if (a.sinks != nullptr) {
      // The sink joins the sum as one more exponential: rescale to the larger of the two maxima.
      const float sink = a.sinks[head], top = fmaxf(m[i], sink);
      keep = expf(m[i] - top);
      denominator = l[i] * keep + expf(sink - top);
    }
    const float inv = denominator > 0.0f ? keep / denominator : 0.0f;   // a fully masked row gives zeros
    const size_t at = a.cross_values ? (static_cast<size_t>(tok0 + qi) * a.nh + head) * a.nkv + vh
                                     : static_cast<size_t>(tok0 + qi) * a.nh + head;
#pragma unroll
    for (int c = 0; c < ACC; ++c) {
      const int d = lane + 32 * c;
      if (d >= vd) continue;
      if (a.out_f32) static_cast<float*>(a.out)[at * vd + d] = acc[i][c] * inv;
      else out[at * vd + d] = from_float<T>(acc[i][c] * inv);
    }
  }
}

template <typename T, int ACC>
int attention_simt_launch(const AttentionArgs& a, int n_tiles, int head_chunks, cudaStream_t stream) {
  const size_t smem = static_cast<size_t>(ATT_MAX_PAIRS) * a.kd * sizeof(float) +
                      static_cast<size_t>(ATT_TILE) * (a.kd + (a.shared_kv ? 0 : a.vd) + KPad<T>::N) * sizeof(T);
  auto kernel = paged_attention_simt_kernel<T, ACC>;
  if (smem > 227 * 1024) return ERR_UNSUPPORTED;      // (float32 keys and values of more than 512 each)
  if (smem > 48 * 1024 &&
      cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)) != cudaSuccess)
    return ERR_CUDA;
  kernel<<<dim3(n_tiles, a.cross_values ? a.nkv * a.nkv : a.nkv, head_chunks), ATT_WARPS * 32, smem, stream>>>(a);
  return launch_result();
}

template <typename T>
int attention_simt_dispatch(const AttentionArgs& a, int n_tiles, int head_chunks, cudaStream_t stream) {
  switch ((a.vd + 31) / 32) {
    case 1: return attention_simt_launch<T, 1>(a, n_tiles, head_chunks, stream);
    case 2: return attention_simt_launch<T, 2>(a, n_tiles, head_chunks, stream);
    case 3: return attention_simt_launch<T, 3>(a, n_tiles, head_chunks, stream);
    case 4: return attention_simt_launch<T, 4>(a, n_tiles, head_chunks, stream);
    case 5: return attention_simt_launch<T, 5>(a, n_tiles, head_chunks, stream);
    case 6: return attention_simt_launch<T, 6>(a, n_tiles, head_chunks, stream);
    case 7: return attention_simt_launch<T, 7>(a, n_tiles, head_chunks, stream);
    case 8: return attention_simt_launch<T, 8>(a, n_tiles, head_chunks, stream);
    case 9: case 10: return attention_simt_launch<T, 10>(a, n_tiles, head_chunks, stream);
    case 11: case 12: return attention_simt_launch<T, 12>(a, n_tiles, head_chunks, stream);
    case 13: case 14: case 15: case 16: return attention_simt_launch<T, 16>(a, n_tiles, head_chunks, stream);
    case 17: case 18: case 19: case 20: return attention_simt_launch<T, 20>(a, n_tiles, head_chunks, stream);
    case 21: case 22: case 23: case 24: return attention_simt_launch<T, 24>(a, n_tiles, head_chunks, stream);
    default: return ERR_UNSUPPORTED;
  }
}

}  // namespace zb

using namespace zb;

// How many consecutive new tokens of one request a tile of the general kernel covers, for a
// model with `group` query heads per key/value head.  The host cuts each row's new tokens into
// tiles of this many tokens.
ZB_API int zb_attention_simt_tile_tokens(int group) {
  const int heads_per_chunk = group < ATT_MAX_PAIRS ? group : ATT_MAX_PAIRS;
  const int t = ATT_MAX_PAIRS / heads_per_chunk;
  return t < 1 ? 1 : t;
}

ZB_API int zb_paged_attention_simt(void* out, const void* q, const void* kv_cache, const int* block_table,
                                   int max_blocks, int page_size, int num_pages, int num_rows, const int* tile_row,
                                   const int* tile_q0, int n_tiles, int tile_tokens, const int* row_q_start,
                                   const int* row_q_len, const int* row_ctx, int nh, int nkv, int kd, int vd,
                                   int window, int chunk, float scale, float softcap, int shared_kv,
                                   const float* head_slopes, const float* sinks, int keep_first, int pool,
                                   const void* pool_cache, const int* pool_table, int pool_max_blocks,
                                   int pool_num_pages, int cross_values, int out_f32, int dtype, int* status,
                                   void* stream) {
  if (nh <= 0 || nkv <= 0 || nh % nkv != 0 || kd <= 0 || vd <= 0 || page_size <= 0 || n_tiles < 0 || window < 0 ||
      chunk < 0 || softcap < 0.0f || (shared_kv && kd != vd) || keep_first < 0 || pool < 0 ||
      (pool > 0 && (window <= 0 || pool_cache == nullptr || pool_table == nullptr || pool_max_blocks <= 0)) ||
      (cross_values && shared_kv))
    return ERR_BAD_ARGUMENT;
  if (kd > 768 || vd > 768) return ERR_UNSUPPORTED;
  if (n_tiles == 0) return OK;
  const int g = nh / nkv;
  const int heads_per_chunk = g < ATT_MAX_PAIRS ? g : ATT_MAX_PAIRS;
  if (tile_tokens <= 0 || tile_tokens * heads_per_chunk > ATT_MAX_PAIRS) return ERR_BAD_ARGUMENT;
  const int head_chunks = (g + heads_per_chunk - 1) / heads_per_chunk;
  AttentionArgs a;
  a.q = q; a.out = out; a.kv_cache = kv_cache; a.block_table = block_table;
  a.tile_row = tile_row; a.tile_q0 = tile_q0;
  a.row_q_start = row_q_start; a.row_q_len = row_q_len; a.row_ctx = row_ctx;
  a.max_blocks = max_blocks; a.page_size = page_size; a.num_pages = num_pages; a.num_rows = num_rows;
  a.nh = nh; a.nkv = nkv; a.kd = kd; a.vd = vd; a.window = window; a.chunk = chunk; a.tile_tokens = tile_tokens;
  a.heads_per_chunk = heads_per_chunk; a.scale = scale; a.softcap = softcap; a.shared_kv = shared_kv; a.head_slopes = head_slopes; a.sinks = sinks;
  a.keep_first = keep_first; a.pool = pool; a.pool_cache = pool_cache; a.pool_table = pool_table;
  a.pool_max_blocks = pool_max_blocks; a.pool_num_pages = pool_num_pages; a.cross_values = cross_values;
  a.out_f32 = out_f32;
  a.status = status;
  auto s = static_cast<cudaStream_t>(stream);
  return dtype == DTYPE_F32 ? attention_simt_dispatch<float>(a, n_tiles, head_chunks, s)
                            : attention_simt_dispatch<__nv_bfloat16>(a, n_tiles, head_chunks, s);
}
