// Paged causal attention for prompt portions (rows with several new tokens), bfloat16, on tensor
// cores: a flash-attention loop that reads keys and values straight from the cache pages, so a
// portion attends to everything its request has cached without any gather copy (the reference
// gathers the whole context of every row into packed tensors for each portion,
// src/layer/paged_attention.cpp:118-296, and then runs one scalar kernel per query row,
// deps/ttl/src/kernels/attention/attention.cu:58-170).
//
// One CTA = up to 128 consecutive new tokens of one request x one query head; 8 warps of 16 query
// rows.  Key/value tiles of 64 positions stream through a two-stage shared-memory ring filled by
// 16-byte asynchronous copies; S = Q K^T and O += P V run as m16n8k16 tensor-core products with
// float32 accumulators; the softmax is online, in float32, in base 2 with scale*log2(e) folded
// in; probabilities are rounded to bfloat16 for the second product.  Math and masking as in
// attention_simt.cu (causal, lower-right aligned on the cached context, optional window).
//
// Further masks, as in attention_simt.cu: a window that keeps the first tokens (`keep_first`), and a window
// followed by pooled blocks (`pool`: a second paged store of one entry per block of positions, of which a
// query at position i sees the first floor((i - window + 1) / pool)).  The tiles of keys then come in three
// runs that share the softmax: pooled entries, kept first tokens, the window.  `cross_values`: the grid
// covers every (query head, key/value head) pair and head h's weights are applied to the values of head c,
// the result being [T, nh, nkv, hd] (what a mixing of the heads' weights behind the softmax is a linear map
// of); `out_f32` writes the result unrounded.
//
// `by_group` (template DEC): a tile is ONE new token of a request and the CTA's query rows are the heads that
// share a key/value head (row r = head kvh * g + r, all at the token's position), so a decoded token's keys
// and values stream once for the whole group and the products fill the tensor cores' rows with heads; the
// grid's x counts key/value heads (times value heads with `cross_values`).
//
// Head sizes: every multiple of 32 up to 256 (a query tile's outputs stay in registers: 16 float32
// values a thread for every 32 of the head).  A tile may hold a single token (one warp works, the
// others help to fetch): latent attention serves decoded tokens this way where the split-context
// kernel does not take the cached row's width.
#include "common.cuh"
#include "mma.cuh"

namespace zb {

constexpr int PRE_BM = 128;     // query rows per CTA
constexpr int PRE_BN = 64;      // keys per tile
constexpr int PRE_WARPS = 8;

struct PrefillArgs {
  const __nv_bfloat16* q;        // [T, nh*hd]
  __nv_bfloat16* out;            // [T, nh*hd]
  const __nv_bfloat16* kv_cache; // [num_pages][2][nkv][page_size][hd]
  const int* block_table;        // [R, max_blocks]
  const int* tile_row;           // [n_tiles]
  const int* tile_q0;            // [n_tiles]
  const int* row_q_start;        // [R]
  const int* row_q_len;          // [R]
  const int* row_ctx;            // [R]
  int max_blocks, page_size, num_pages, num_rows;
  int page_shift;                // page_size = 1 << page_shift, or -1 where it is no power of two
  int nh, nkv, window;
  int chunk;                     // n > 0: a query at position p sees only keys >= (p / n) * n
  const float* sinks;            // null, or [nh]: exp(sinks[h]) joins the softmax's denominator of head h
  float scale_log2;
  float softcap_log2;            // > 0: scores are softcap * tanh(scale * s / softcap); this is softcap * log2(e)
  float scale_over_cap;          // scale / softcap
  int keys_only;                 // a page holds keys alone, [nkv][page_size][hd], and they are the values too
  int keep_first;                // with a window: keys below this position stay visible
  int pool;                      // 0, or the positions per entry of the pooled store
  const __nv_bfloat16* pool_cache;   // laid out as kv_cache
  const int* pool_table;         // [R, pool_max_blocks]
  int pool_max_blocks, pool_num_pages;
  int cross_values;              // grid x = nh * nkv: head + nh * value head
  int out_f32;
  int* status;
};

// NS: stages of the ring of key/value tiles.  Two leave room for two CTAs an SM; three and four were measured
// for tiles of one token (a decode step of 8 requests: 2.63 against 2.59 ms) and are not used.
template <int HD, bool DEC, int NS>
__global__ void __launch_bounds__(PRE_WARPS * 32, 1)
paged_prefill_kernel(const PrefillArgs a) {
  static_assert(HD % 32 == 0 && HD <= 256, "head sizes that are multiples of 32, up to 256");
  constexpr int KROW = HD + 8;                      // padded rows: conflict-free ldmatrix
  constexpr int CHUNKS = HD / 8;
  constexpr int STAGE = 2 * PRE_BN * KROW;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __nv_bfloat16* q_s = reinterpret_cast<__nv_bfloat16*>(smem_raw);     // [PRE_BM][KROW]
  __nv_bfloat16* ring = q_s + PRE_BM * KROW;                             // [2][keys, values][PRE_BN][KROW]

  // The host lists the tiles by the number of keys they see, fewest first: take the list back to
  // front, and all heads of a tile before the next tile, so that the longest work of the whole
  // launch starts first and the short tiles fill the gaps at the end.
  const int tile = gridDim.y - 1 - blockIdx.y;
  const int across = DEC ? a.nkv : a.nh;           // what the grid's x counts: key/value heads, or query heads
  const int head = DEC ? (blockIdx.x % across) * (a.nh / a.nkv) : blockIdx.x % across;   // (DEC: the group's first head)
  const int row = a.tile_row[tile], q0 = a.tile_q0[tile];
  if (row < 0 || row >= a.num_rows) {
    if (threadIdx.x == 0) report(a.status, STATUS_ROW_OUT_OF_RANGE, row, tile);
    return;
  }
  const int g = a.nh / a.nkv, kvh = head / g;
  const int vh = a.cross_values ? blockIdx.x / across : kvh;      // whose values
  const int q_len = a.row_q_len[row], ctx = a.row_ctx[row], tok0 = a.row_q_start[row] + q0;
  const int n_tok = DEC ? min(1, q_len - q0) : min(PRE_BM, q_len - q0);
  if (n_tok <= 0) return;
  const int n_rows = DEC ? min(g, PRE_BM) : n_tok;       // query rows of this CTA: heads of the group, or tokens
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int quad_row = lane >> 2, quad_col = (lane & 3) * 2;
  const int* table = a.block_table + static_cast<size_t>(row) * a.max_blocks;

  // Keys any query of this tile may see: [lo, hi).
  const int hi = ctx + q0 + n_tok;
  int lo = a.window > 0 ? max(0, ctx + q0 - a.window + 1) : 0;
  if (a.chunk > 0) lo = max(lo, (ctx + q0) / a.chunk * a.chunk);
  const int first_tile = lo / PRE_BN * PRE_BN;
  // Three runs of tiles: the pooled entries the tile's last query sees, the kept first tokens that lie
  // below every window of the tile, the window.
  const int entries = (a.pool > 0 && a.window > 0) ? max(0, (hi - a.window) / a.pool) : 0;
  const int kept = a.window > 0 ? min(a.keep_first, lo) : 0;
  const int pool_tiles = (entries + PRE_BN - 1) / PRE_BN, kept_tiles = (kept + PRE_BN - 1) / PRE_BN;
  const int n_tiles = pool_tiles + kept_tiles + (hi - first_tile + PRE_BN - 1) / PRE_BN;
  const int* pool_table = a.pool > 0 ? a.pool_table + static_cast<size_t>(row) * a.pool_max_blocks : nullptr;

  for (int e = threadIdx.x; e < PRE_BM * CHUNKS; e += PRE_WARPS * 32) {
    const int j = e / CHUNKS, c = (e - j * CHUNKS) * 8;
    const bool ok = j < n_rows;
    const size_t from = DEC ? static_cast<size_t>(tok0) * a.nh + head + (ok ? j : 0)
                            : static_cast<size_t>(tok0 + (ok ? j : 0)) * a.nh + head;
    cp_async_16(q_s + j * KROW + c, a.q + from * HD + c, ok);
  }
  auto load_tile = [&](int t) {
    __nv_bfloat16* ks = ring + (t % NS) * STAGE;
    __nv_bfloat16* vs = ks + PRE_BN * KROW;
    const int run = t < pool_tiles ? 0 : (t < pool_tiles + kept_tiles ? 1 : 2);
    const int k0 = run == 0 ? t * PRE_BN : (run == 1 ? (t - pool_tiles) * PRE_BN
                                                     : first_tile + (t - pool_tiles - kept_tiles) * PRE_BN);
    const int run_lo = run == 2 ? lo : 0, run_hi = run == 0 ? entries : (run == 1 ? kept : hi);
    const __nv_bfloat16* source = run == 0 ? a.pool_cache : a.kv_cache;
    const int* pages = run == 0 ? pool_table : table;
    const int max_blocks = run == 0 ? a.pool_max_blocks : a.max_blocks;
    const int num_pages = run == 0 ? a.pool_num_pages : a.num_pages;
    for (int e = threadIdx.x; e < PRE_BN * CHUNKS; e += PRE_WARPS * 32) {
      const int j = e / CHUNKS, c = (e - j * CHUNKS) * 8;
      const int pos = k0 + j;
      bool ok = pos >= run_lo && pos < run_hi;
      const __nv_bfloat16* src = source;
      const __nv_bfloat16* vsrc = source;
      if (ok) {
        // (a division by a size only known at run time costs tens of instructions, here for every 16 bytes)
        const int block = a.page_shift >= 0 ? pos >> a.page_shift : pos / a.page_size;
        const int in_page = a.page_shift >= 0 ? pos & (a.page_size - 1) : pos % a.page_size;
        const int page = block < max_blocks ? pages[block] : -1;
        if (page <= 0 || page >= num_pages) {
          report(a.status, STATUS_PAGE_OUT_OF_RANGE, page, tok0);
          ok = false;
        } else {
          // logical chunk c / 8 of the row sits at the permuted chunk (common.cuh: kv_swizzle)
          const long long in_row = ((c >> 3) ^ kv_swizzle(pos, CHUNKS)) << 3;
          const long long page_heads = static_cast<long long>(page) * (a.keys_only ? 1 : 2) * a.nkv;
          src += ((page_heads + kvh) * a.page_size + in_page) * HD + in_row;
          vsrc += ((page_heads + (a.keys_only ? kvh : a.nkv + vh)) * a.page_size + in_page) * HD + in_row;
        }
      }
      cp_async_16(ks + j * KROW + c, src, ok);
      cp_async_16(vs + j * KROW + c, vsrc, ok);
    }
  };
#pragma unroll
  for (int t = 0; t < NS - 1; ++t) {         // one group of copies a tile, empty ones past the end
    if (t < n_tiles) load_tile(t);
    cp_async_commit();
  }

  // This warp's 16 query rows; this lane's two rows sit at positions qpos[0] and qpos[1].
  const int warp_row0 = DEC ? 0 : warp * 16;
  const bool warp_active = warp_row0 < n_rows;
  const int warp_pos0 = DEC ? ctx + q0 : ctx + q0 + warp_row0;      // the position of the warp's first row
  const int qpos[2] = {DEC ? warp_pos0 : warp_pos0 + quad_row, DEC ? warp_pos0 : warp_pos0 + quad_row + 8};
  const int warp_last_pos = DEC ? warp_pos0 : ctx + q0 + min(warp_row0 + 15, n_tok - 1);
  int warp_first_visible = a.window > 0 ? max(0, warp_pos0 - a.window + 1) : 0;
  if (a.chunk > 0) warp_first_visible = max(warp_first_visible, warp_pos0 / a.chunk * a.chunk);
  const int chunk_start[2] = {a.chunk > 0 ? qpos[0] / a.chunk * a.chunk : 0, a.chunk > 0 ? qpos[1] / a.chunk * a.chunk : 0};
  // Pooled entries in sight of this lane's two rows, and of the warp's last row: worked out once, not per score.
  const int seen[2] = {a.pool > 0 ? (qpos[0] - a.window + 1) / a.pool : 0, a.pool > 0 ? (qpos[1] - a.window + 1) / a.pool : 0};
  const int warp_seen = a.pool > 0 ? (warp_last_pos - a.window + 1) / a.pool : 0;
  const int warp_seen_first = a.pool > 0 ? (warp_pos0 - a.window + 1) / a.pool : 0;      // what the warp's first row sees

  unsigned qa[HD / 16][4];
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.0f, 0.0f};
  float o[HD / 8][4];
#pragma unroll
  for (int n = 0; n < HD / 8; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.0f;

  for (int t = 0; t < n_tiles; ++t) {
    cp_async_wait<NS - 2>();
    __syncthreads();                 // tile t (and, the first time, Q) has landed; tile t-1 is no longer read
    if (t + NS - 1 < n_tiles) load_tile(t + NS - 1);
    cp_async_commit();
    if (t == 0) {
#pragma unroll
      for (int ks = 0; ks < HD / 16; ++ks)
        ldmatrix_x4(qa[ks], q_s + (warp_row0 + (lane & 7) + ((lane >> 3) & 1) * 8) * KROW + ks * 16 + (lane >> 4) * 8);
    }
    const int run = t < pool_tiles ? 0 : (t < pool_tiles + kept_tiles ? 1 : 2);
    const int k0 = run == 0 ? t * PRE_BN : (run == 1 ? (t - pool_tiles) * PRE_BN
                                                     : first_tile + (t - pool_tiles - kept_tiles) * PRE_BN);
    if (!warp_active) continue;                          // uniform over the warp, as are the next two
    if (run == 0 && k0 >= warp_seen) continue;
    if (run == 2 && (k0 > warp_last_pos || (k0 + PRE_BN <= warp_first_visible && k0 >= a.keep_first))) continue;
    const __nv_bfloat16* ks_tile = ring + (t % NS) * STAGE;
    const __nv_bfloat16* vs_tile = ks_tile + PRE_BN * KROW;

    // The key tiles of 8 this warp works on: all eight of the 64 keys, or (DEC) the warp's own one.
    constexpr int NTS = DEC ? 1 : PRE_BN / 8;
    float s[NTS][4];
#pragma unroll
    for (int i = 0; i < NTS; ++i) {
      const int nt = DEC ? warp : i;
      s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.0f;
#pragma unroll
      for (int kk = 0; kk < HD / 32; ++kk) {
        unsigned b[4];
        ldmatrix_x4(b, ks_tile + (nt * 8 + (lane & 7)) * KROW + kk * 32 + (lane >> 3) * 8);
        mma_bf16_16816(s[i], qa[2 * kk], b[0], b[1]);
        mma_bf16_16816(s[i], qa[2 * kk + 1], b[2], b[3]);
      }
    }

    float tile_max[2] = {-INFINITY, -INFINITY};
    // A tile that every row of the warp sees whole needs no mask: most tiles of a long window are such.
    const bool whole_tile =
        run == 0 ? k0 + PRE_BN <= warp_seen_first
      : run == 1 ? k0 + PRE_BN <= kept
                 : k0 + PRE_BN - 1 <= warp_pos0 && k0 >= lo && (a.window == 0 || k0 > warp_last_pos - a.window) &&
                       (a.chunk == 0 || k0 >= warp_last_pos / a.chunk * a.chunk);
    if (whole_tile) {
#pragma unroll
      for (int i = 0; i < NTS; ++i) {
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          s[i][c] = a.softcap_log2 > 0.0f ? a.softcap_log2 * tanhf(s[i][c] * a.scale_over_cap) : s[i][c] * a.scale_log2;
          tile_max[c >> 1] = fmaxf(tile_max[c >> 1], s[i][c]);
        }
      }
    } else {
#pragma unroll
      for (int i = 0; i < NTS; ++i) {
        const int nt = DEC ? warp : i;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const int pos = k0 + nt * 8 + quad_col + (c & 1);
          const int qp = qpos[c >> 1];
          const bool valid = run == 0 ? pos < seen[c >> 1]
                           : run == 1 ? pos < kept
                                      : pos <= qp && pos >= lo &&
                                            (a.window == 0 || pos > qp - a.window || pos < a.keep_first) &&
                                            pos >= chunk_start[c >> 1];
          const float scaled = a.softcap_log2 > 0.0f ? a.softcap_log2 * tanhf(s[i][c] * a.scale_over_cap)
                                                     : s[i][c] * a.scale_log2;
          s[i][c] = valid ? scaled : -INFINITY;
          tile_max[c >> 1] = fmaxf(tile_max[c >> 1], s[i][c]);
        }
      }
    }
    float corr[2], m_use[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      tile_max[h] = fmaxf(tile_max[h], __shfl_xor_sync(0xffffffffu, tile_max[h], 1));
      tile_max[h] = fmaxf(tile_max[h], __shfl_xor_sync(0xffffffffu, tile_max[h], 2));
      const float new_m = fmaxf(m_run[h], tile_max[h]);
      m_use[h] = new_m == -INFINITY ? 0.0f : new_m;      // a row that has seen no key yet: keep exp2 finite
      corr[h] = exp2f(m_run[h] - m_use[h]);              // 0 while the running maximum is -inf
      m_run[h] = new_m;
    }
    float row_sum[2] = {0.0f, 0.0f};
#pragma unroll
    for (int i = 0; i < NTS; ++i) {
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        s[i][c] = exp2f(s[i][c] - m_use[c >> 1]);
        row_sum[c >> 1] += s[i][c];
      }
    }
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      row_sum[h] += __shfl_xor_sync(0xffffffffu, row_sum[h], 1);
      row_sum[h] += __shfl_xor_sync(0xffffffffu, row_sum[h], 2);
      l_run[h] = l_run[h] * corr[h] + row_sum[h];
    }
#pragma unroll
    for (int n = 0; n < HD / 8; ++n) {
      o[n][0] *= corr[0]; o[n][1] *= corr[0]; o[n][2] *= corr[1]; o[n][3] *= corr[1];
    }
    if (DEC) {
      // 8 keys: the product's second half of 8 takes zero weights (and reads the same 8 value rows again).
      unsigned pa[4] = {pack_bf16(s[0][0], s[0][1]), pack_bf16(s[0][2], s[0][3]), 0u, 0u};
#pragma unroll
      for (int n2 = 0; n2 < HD / 16; ++n2) {
        unsigned b[4];
        ldmatrix_x4_trans(b, vs_tile + (warp * 8 + (lane & 7)) * KROW + n2 * 16 + (lane >> 4) * 8);
        mma_bf16_16816(o[2 * n2], pa, b[0], b[1]);
        mma_bf16_16816(o[2 * n2 + 1], pa, b[2], b[3]);
      }
    } else {
#pragma unroll
      for (int ks = 0; ks < NTS / 2; ++ks) {
        unsigned pa[4];
        pa[0] = pack_bf16(s[2 * ks][0], s[2 * ks][1]);
        pa[1] = pack_bf16(s[2 * ks][2], s[2 * ks][3]);
        pa[2] = pack_bf16(s[(2 * ks + 1) % NTS][0], s[(2 * ks + 1) % NTS][1]);
        pa[3] = pack_bf16(s[(2 * ks + 1) % NTS][2], s[(2 * ks + 1) % NTS][3]);
#pragma unroll
        for (int n2 = 0; n2 < HD / 16; ++n2) {
          unsigned b[4];
          ldmatrix_x4_trans(b, vs_tile + (ks * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * KROW + n2 * 16 + (lane >> 4) * 8);
          mma_bf16_16816(o[2 * n2], pa, b[0], b[1]);
          mma_bf16_16816(o[2 * n2 + 1], pa, b[2], b[3]);
        }
      }
    }
  }
  cp_async_wait<0>();

  if (DEC) {
    // The eight warps' partial results meet in shared memory (the ring is no longer read): each row's
    // maxima and sums, and its outputs, then 256 threads share the rows' values.
    __syncthreads();
    float* part_o = reinterpret_cast<float*>(ring);                 // [warps][16][HD]
    float* part_m = reinterpret_cast<float*>(q_s);                  // [warps][16], then the sums
    float* part_l = part_m + PRE_WARPS * 16;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int r = quad_row + 8 * h;
      if ((lane & 3) == 0) {
        part_m[warp * 16 + r] = m_run[h];
        part_l[warp * 16 + r] = l_run[h];
      }
#pragma unroll
      for (int n = 0; n < HD / 8; ++n)
        *reinterpret_cast<float2*>(part_o + (warp * 16 + r) * HD + n * 8 + quad_col) = make_float2(o[n][2 * h], o[n][2 * h + 1]);
    }
    __syncthreads();
    for (int e = threadIdx.x; e < n_rows * HD; e += PRE_WARPS * 32) {
      const int r = e / HD, d = e - r * HD;
      float top = -INFINITY;
#pragma unroll
      for (int w = 0; w < PRE_WARPS; ++w) top = fmaxf(top, part_m[w * 16 + r]);
      float denominator = 0.0f, value = 0.0f;
#pragma unroll
      for (int w = 0; w < PRE_WARPS; ++w) {
        const float weight = top == -INFINITY ? 0.0f : exp2f(part_m[w * 16 + r] - top);
        denominator = fmaf(part_l[w * 16 + r], weight, denominator);
        value = fmaf(part_o[(w * 16 + r) * HD + d], weight, value);
      }
      const int row_head = head + r;
      if (a.sinks != nullptr) denominator += exp2f(a.sinks[row_head] * 1.4426950408889634f - top);
      const float result = denominator > 0.0f ? value / denominator : 0.0f;
      const size_t at = (a.cross_values ? (static_cast<size_t>(tok0) * a.nh + row_head) * a.nkv + vh
                                        : static_cast<size_t>(tok0) * a.nh + row_head) * HD + d;
      if (a.out_f32) reinterpret_cast<float*>(a.out)[at] = result;
      else a.out[at] = __float2bfloat16_rn(result);
    }
    return;
  }
  if (!warp_active) return;
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int r = warp_row0 + quad_row + 8 * h;
    if (r >= n_rows) continue;
    const int row_head = DEC ? head + r : head;
    const size_t row_token = DEC ? tok0 : tok0 + r;
    float denominator = l_run[h];
    if (a.sinks != nullptr)      // one more exponential, relative to the running maximum (both in powers of two)
      denominator += exp2f(a.sinks[row_head] * 1.4426950408889634f - m_run[h]);
    const float inv = denominator > 0.0f ? 1.0f / denominator : 0.0f;
    const size_t at = (a.cross_values ? (row_token * a.nh + row_head) * a.nkv + vh
                                      : row_token * a.nh + row_head) * HD + quad_col;
    if (a.out_f32) {
      float* dst = reinterpret_cast<float*>(a.out) + at;
#pragma unroll
      for (int n = 0; n < HD / 8; ++n)
        *reinterpret_cast<float2*>(dst + n * 8) = make_float2(o[n][2 * h] * inv, o[n][2 * h + 1] * inv);
    } else {
      __nv_bfloat16* dst = a.out + at;
#pragma unroll
      for (int n = 0; n < HD / 8; ++n)
        *reinterpret_cast<unsigned*>(dst + n * 8) = pack_bf16(o[n][2 * h] * inv, o[n][2 * h + 1] * inv);
    }
  }
}

template <int HD>
int prefill_launch(const PrefillArgs& a, int n_tiles, cudaStream_t stream, bool by_group = false) {
  constexpr int GROUP_STAGES = 2;
  const int stages = by_group ? GROUP_STAGES : 2;
  const size_t smem = (static_cast<size_t>(PRE_BM) + 2 * stages * PRE_BN) * (HD + 8) * sizeof(__nv_bfloat16);
  auto kernel = by_group ? paged_prefill_kernel<HD, true, GROUP_STAGES> : paged_prefill_kernel<HD, false, 2>;
  if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)) != cudaSuccess)
    return ERR_CUDA;
  const int across = by_group ? a.nkv : a.nh;
  kernel<<<dim3(a.cross_values ? across * a.nkv : across, n_tiles), PRE_WARPS * 32, smem, stream>>>(a);
  return launch_result();
}

}  // namespace zb

using namespace zb;

// Tokens of one request that a tile of this kernel covers (the host cuts rows into such tiles).
ZB_API int zb_paged_prefill_tile_tokens() { return PRE_BM; }

ZB_API int zb_paged_prefill_supported(int nh, int nkv, int hd, int dtype) {
  if (dtype != DTYPE_BF16 || nkv <= 0 || nh <= 0 || nh % nkv != 0 || nh > 65535) return 0;
  return hd % 32 == 0 && hd >= 32 && hd <= 256 ? 1 : 0;
}

// Attention of the tiles' tokens over their requests' pages; writes those tokens' rows of `out`.
// `chunk` and `sinks` as in the general kernel (attention_simt.cu).
// `keep_first`, `pool` with its store, `cross_values` and `out_f32` as the comment at the top says.
ZB_API int zb_paged_prefill_windowed(void* out, const void* q, const void* kv_cache, const int* block_table,
                                     int max_blocks, int page_size, int num_pages, int num_rows, const int* tile_row,
                                     const int* tile_q0, int n_tiles, const int* row_q_start, const int* row_q_len,
                                     const int* row_ctx, int nh, int nkv, int hd, int window, int chunk, float scale,
                                     float softcap, int keys_only, const float* sinks, int keep_first, int pool,
                                     const void* pool_cache, const int* pool_table, int pool_max_blocks,
                                     int pool_num_pages, int cross_values, int out_f32, int by_group, int* status,
                                     void* stream) {
  if (n_tiles < 0 || page_size <= 0 || window < 0 || chunk < 0 || softcap < 0.0f || keep_first < 0 || pool < 0 ||
      (pool > 0 && (window <= 0 || pool_cache == nullptr || pool_table == nullptr || pool_max_blocks <= 0 || keys_only)) ||
      (cross_values && keys_only) || nh * (cross_values ? nkv : 1) > 65535 || (by_group && nh / (nkv > 0 ? nkv : 1) > 16))
    return ERR_BAD_ARGUMENT;
  if (!zb_paged_prefill_supported(nh, nkv, hd, DTYPE_BF16)) return ERR_UNSUPPORTED;
  if (n_tiles == 0) return OK;
  if (n_tiles > 65535) return ERR_UNSUPPORTED;
  PrefillArgs a;
  a.q = static_cast<const __nv_bfloat16*>(q);
  a.out = static_cast<__nv_bfloat16*>(out);
  a.kv_cache = static_cast<const __nv_bfloat16*>(kv_cache);
  a.block_table = block_table; a.tile_row = tile_row; a.tile_q0 = tile_q0;
  a.row_q_start = row_q_start; a.row_q_len = row_q_len; a.row_ctx = row_ctx;
  a.max_blocks = max_blocks; a.page_size = page_size; a.num_pages = num_pages; a.num_rows = num_rows;
  a.page_shift = -1;
  for (int shift = 0; shift < 31; ++shift)
    if (page_size == (1 << shift)) a.page_shift = shift;
  a.nh = nh; a.nkv = nkv; a.window = window; a.chunk = chunk; a.sinks = sinks;
  a.scale_log2 = scale * 1.4426950408889634f;
  a.softcap_log2 = softcap * 1.4426950408889634f;
  a.scale_over_cap = softcap > 0.0f ? scale / softcap : 0.0f;
  a.keys_only = keys_only;
  a.keep_first = window > 0 ? keep_first : 0; a.pool = pool;
  a.pool_cache = static_cast<const __nv_bfloat16*>(pool_cache);
  a.pool_table = pool_table; a.pool_max_blocks = pool_max_blocks; a.pool_num_pages = pool_num_pages;
  a.cross_values = cross_values; a.out_f32 = out_f32;
  a.status = status;
  auto s = static_cast<cudaStream_t>(stream);
  switch (hd) {
    case 32: return prefill_launch<32>(a, n_tiles, s, by_group != 0);
    case 64: return prefill_launch<64>(a, n_tiles, s, by_group != 0);
    case 96: return prefill_launch<96>(a, n_tiles, s, by_group != 0);
    case 128: return prefill_launch<128>(a, n_tiles, s, by_group != 0);
    case 160: return prefill_launch<160>(a, n_tiles, s, by_group != 0);
    case 192: return prefill_launch<192>(a, n_tiles, s, by_group != 0);
    case 224: return prefill_launch<224>(a, n_tiles, s, by_group != 0);
    default: return prefill_launch<256>(a, n_tiles, s, by_group != 0);
  }
}

ZB_API int zb_paged_prefill_masked(void* out, const void* q, const void* kv_cache, const int* block_table,
                                   int max_blocks, int page_size, int num_pages, int num_rows, const int* tile_row,
                                   const int* tile_q0, int n_tiles, const int* row_q_start, const int* row_q_len,
                                   const int* row_ctx, int nh, int nkv, int hd, int window, int chunk, float scale,
                                   float softcap, int keys_only, const float* sinks, int* status, void* stream) {
  return zb_paged_prefill_windowed(out, q, kv_cache, block_table, max_blocks, page_size, num_pages, num_rows, tile_row,
                                   tile_q0, n_tiles, row_q_start, row_q_len, row_ctx, nh, nkv, hd, window, chunk, scale,
                                   softcap, keys_only, sinks, 0, 0, nullptr, nullptr, 0, 0, 0, 0, 0, status, stream);
}

ZB_API int zb_paged_prefill(void* out, const void* q, const void* kv_cache, const int* block_table, int max_blocks,
                            int page_size, int num_pages, int num_rows, const int* tile_row, const int* tile_q0,
                            int n_tiles, const int* row_q_start, const int* row_q_len, const int* row_ctx, int nh,
                            int nkv, int hd, int window, float scale, int* status, void* stream) {
  return zb_paged_prefill_masked(out, q, kv_cache, block_table, max_blocks, page_size, num_pages, num_rows, tile_row,
                                 tile_q0, n_tiles, row_q_start, row_q_len, row_ctx, nh, nkv, hd, window, 0, scale, 0.0f, 0,
                                 nullptr, status, stream);
}
