// A routed feed-forward (mixture of experts), token choice:
//
//   s = softmax(z) over all router outputs          (float32; z = router logits)
//   choice = s + correction                         (moves the choice only)
//   the `top` outputs with the largest choice are taken (ties: the lower index), each with weight s
//   (not renormalised);
//   out = sum over the taken outputs of  s_e * expert_e(x),
//
// where the first `experts` outputs are gated feed-forwards down_e(act(gate_e x) * (up_e x)) and the
// remaining ones are identity experts, expert(x) = x, which have no weights.
//
// Four steps, all shapes fixed by the step's token count (nothing is read back by the host):
//   route     one warp per token: softmax, choice, selection -> ids [T, top], weights [T, top]
//   align     one CTA: the (token, choice) slots sorted by expert, every expert's run cut into tiles of
//             32 (float32) or 64 (bfloat16) rows -> slot list, tile list
//   products  one CTA per (tile, 64 outputs): gate and up together with the activation, then down,
//             each row's sums in the order of k, so a token's result does not depend on what else
//             was routed to its expert; float32 on CUDA cores, bfloat16 on the tensor cores
//   combine   out[t] = sum_j weight[t, j] * (expert output of slot (t, j), or x[t] for an identity
//             expert), in float32 and in the order of j, rounded once.
#include "tile_product.cuh"
#include "tile_product_mma.cuh"

namespace zb {

constexpr int ROUTE_PER_LANE = 8;      // up to 256 router outputs
constexpr int ROUTE_WARPS = 4;

// ---------------------------------------------------------------------------------------------- route
// Further forms, each a parameter: scores that are the logistic function of each logit on its own
// (`sigmoid_scores`) instead of a softmax over all; a choice limited to groups (the outputs form `groups`
// equal runs of neighbours; a group's mark is the sum of its `group_top` largest choice values, and only
// outputs of the `keep` groups with the largest marks can be taken; ties: the lower group); and a
// multiplier on the weights (`weight_scale`); a bias on the logits (`logit_bias`, part of the logit for the
// choice and for the weight alike); and scores that are the logits themselves (`score_kind` 2): the `top`
// largest logits are taken and weigh their outputs by the softmax over the taken logits only.
constexpr int ROUTE_GROUP_TOP_MAX = 4;
constexpr int SCORES_SOFTMAX = 0, SCORES_SIGMOID = 1, SCORES_TOP_SOFTMAX = 2;

__global__ void __launch_bounds__(ROUTE_WARPS * 32)
route_kernel(int* ids, float* weights, const float* logits, long long logits_stride, const float* correction,
             int tokens, int outputs, int top, int score_kind, int groups, int keep, int group_top,
             float weight_scale, const float* logit_bias) {
  __shared__ float choice_of[ROUTE_WARPS][32 * ROUTE_PER_LANE];
  __shared__ float mark_of[ROUTE_WARPS][32 * ROUTE_PER_LANE];
  const int warp = threadIdx.x >> 5;
  const int t = blockIdx.x * ROUTE_WARPS + warp, lane = threadIdx.x & 31;
  if (t >= tokens) return;
  const float* z = logits + t * logits_stride;
  float s[ROUTE_PER_LANE], c[ROUTE_PER_LANE];
  const bool biased = logit_bias != nullptr;
  if (score_kind == SCORES_SIGMOID) {
#pragma unroll
    for (int i = 0; i < ROUTE_PER_LANE; ++i) {
      const int e = lane + 32 * i;
      s[i] = e < outputs ? 1.0f / (1.0f + expf(-(z[e] + (biased ? logit_bias[e] : 0.0f)))) : 0.0f;
    }
  } else if (score_kind == SCORES_TOP_SOFTMAX) {
#pragma unroll
    for (int i = 0; i < ROUTE_PER_LANE; ++i) {
      const int e = lane + 32 * i;
      s[i] = e < outputs ? z[e] + (biased ? logit_bias[e] : 0.0f) : -INFINITY;
    }
  } else {
    float top_z = -INFINITY;
#pragma unroll
    for (int i = 0; i < ROUTE_PER_LANE; ++i) {
      const int e = lane + 32 * i;
      s[i] = e < outputs ? z[e] + (biased ? logit_bias[e] : 0.0f) : -INFINITY;
      top_z = fmaxf(top_z, s[i]);
    }
    top_z = warp_max(top_z);
    float sum = 0.0f;
#pragma unroll
    for (int i = 0; i < ROUTE_PER_LANE; ++i) {
      const int e = lane + 32 * i;
      s[i] = e < outputs ? expf(s[i] - top_z) : 0.0f;
      sum += s[i];
    }
    sum = warp_sum(sum);
#pragma unroll
    for (int i = 0; i < ROUTE_PER_LANE; ++i) s[i] = s[i] / sum;
  }
#pragma unroll
  for (int i = 0; i < ROUTE_PER_LANE; ++i) {
    const int e = lane + 32 * i;
    c[i] = e < outputs ? s[i] + (correction != nullptr ? correction[e] : 0.0f) : -INFINITY;
  }
  if (groups > 1 && keep < groups) {
    const int members = outputs / groups;
#pragma unroll
    for (int i = 0; i < ROUTE_PER_LANE; ++i)
      if (lane + 32 * i < outputs) choice_of[warp][lane + 32 * i] = c[i];
    __syncwarp();
    for (int g = lane; g < groups; g += 32) {
      // The group's largest `group_top` values, by repeated search (the groups are small).
      int taken[ROUTE_GROUP_TOP_MAX];
      float mark = 0.0f;
      for (int k = 0; k < group_top && k < members; ++k) {
        float best = -INFINITY;
        int best_m = -1;
        for (int m = 0; m < members; ++m) {
          bool used = false;
          for (int j = 0; j < k; ++j) used = used || taken[j] == m;
          const float v = choice_of[warp][g * members + m];
          if (!used && (best_m < 0 || v > best)) {
            best = v;
            best_m = m;
          }
        }
        taken[k] = best_m;
        mark += best;
      }
      mark_of[warp][g] = mark;
    }
    __syncwarp();
#pragma unroll
    for (int i = 0; i < ROUTE_PER_LANE; ++i) {
      const int e = lane + 32 * i;
      if (e >= outputs) continue;
      const int g = e / members;
      const float mine = mark_of[warp][g];
      int ahead = 0;
      for (int o = 0; o < groups; ++o) {
        const float other = mark_of[warp][o];
        ahead += (other > mine || (other == mine && o < g)) ? 1 : 0;
      }
      if (ahead >= keep) c[i] = -INFINITY;
    }
  }
  for (int j = 0; j < top; ++j) {
    // The largest remaining choice; among equals the lowest index.
    float best = -INFINITY;
    int best_e = 0x7fffffff;
#pragma unroll
    for (int i = 0; i < ROUTE_PER_LANE; ++i) {
      const int e = lane + 32 * i;
      if (c[i] > best || (c[i] == best && e < best_e && c[i] > -INFINITY)) {
        best = c[i];
        best_e = e;
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float other = __shfl_xor_sync(0xffffffffu, best, o);
      const int other_e = __shfl_xor_sync(0xffffffffu, best_e, o);
      if (other > best || (other == best && other_e < best_e)) {
        best = other;
        best_e = other_e;
      }
    }
    float w = 0.0f;
#pragma unroll
    for (int i = 0; i < ROUTE_PER_LANE; ++i)
      if (lane + 32 * i == best_e) {
        w = s[i];
        c[i] = -INFINITY;
      }
    w = __shfl_sync(0xffffffffu, w, best_e & 31);
    if (lane == 0) {
      ids[static_cast<size_t>(t) * top + j] = best_e;
      weights[static_cast<size_t>(t) * top + j] = score_kind == SCORES_TOP_SOFTMAX ? w : w * weight_scale;
    }
  }
  if (score_kind == SCORES_TOP_SOFTMAX && lane == 0) {
    // The taken logits lie in the order of choice, the largest first: their softmax among themselves.
    float* w = weights + static_cast<size_t>(t) * top;
    const float largest = w[0];
    float sum = 0.0f;
    for (int j = 0; j < top; ++j) {
      w[j] = expf(w[j] - largest);
      sum += w[j];
    }
    for (int j = 0; j < top; ++j) w[j] = w[j] / sum * weight_scale;
  }
}

// ---------------------------------------------------------------------------------------------- align
// plan: [0] = number of tiles; then per tile (expert, first place in `slots`, rows).  slots: the slot
// numbers (t * top + j) of all choices of real experts, expert after expert.  place_of_slot[slot] says
// where the slot landed (-1 for an identity expert).
constexpr int ALIGN_THREADS = 1024;

__global__ void __launch_bounds__(ALIGN_THREADS)
align_kernel(int* plan, int* slots, int* place_of_slot, const int* ids, int num_slots, int experts, int max_tiles,
             int tile_rows) {
  extern __shared__ int align_smem[];
  int* count = align_smem;                 // [experts]
  int* start = count + experts;            // [experts + 1]
  int* fill = start + experts + 1;         // [experts]
  for (int e = threadIdx.x; e < experts; e += blockDim.x) count[e] = fill[e] = 0;
  __syncthreads();
  for (int i = threadIdx.x; i < num_slots; i += blockDim.x) {
    const int e = ids[i];
    if (e >= 0 && e < experts) atomicAdd(&count[e], 1);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int at = 0, tiles = 0;
    for (int e = 0; e < experts; ++e) {
      start[e] = at;
      for (int r = 0; r < count[e] && tiles < max_tiles; r += tile_rows, ++tiles) {
        plan[1 + 3 * tiles] = e;
        plan[2 + 3 * tiles] = at + r;
        plan[3 + 3 * tiles] = min(tile_rows, count[e] - r);
      }
      at += count[e];
    }
    start[experts] = at;
    plan[0] = tiles;
  }
  __syncthreads();
  // Which place a slot gets inside its expert's run depends on the order of arrival; no result does:
  // every row of a product is summed on its own.
  for (int i = threadIdx.x; i < num_slots; i += blockDim.x) {
    const int e = ids[i];
    int place = -1;
    if (e >= 0 && e < experts) {
      place = start[e] + atomicAdd(&fill[e], 1);
      slots[place] = i;
    }
    place_of_slot[i] = place;
  }
}

// The same for products that run as one grouped launch of the tcgen05 kernel (gemm_tc.cu): every expert's
// run begins on a multiple of `tile_rows` places, tile_group[i] names the expert of tile i (-1: unused),
// and slots[place] is -1 where a place pads a run.
__global__ void __launch_bounds__(ALIGN_THREADS)
align_padded_kernel(int* tile_group, int* slots, int* place_of_slot, const int* ids, int num_slots, int experts,
                    int max_tiles, int tile_rows) {
  extern __shared__ int align_smem[];
  int* count = align_smem;                 // [experts]
  int* start = count + experts;            // [experts + 1]
  int* fill = start + experts + 1;         // [experts]
  for (int e = threadIdx.x; e < experts; e += blockDim.x) count[e] = fill[e] = 0;
  for (int i = threadIdx.x; i < max_tiles * tile_rows; i += blockDim.x) slots[i] = -1;
  __syncthreads();
  for (int i = threadIdx.x; i < num_slots; i += blockDim.x) {
    const int e = ids[i];
    if (e >= 0 && e < experts) atomicAdd(&count[e], 1);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int tiles = 0;
    for (int e = 0; e < experts; ++e) {
      start[e] = tiles * tile_rows;
      for (int r = 0; r < count[e] && tiles < max_tiles; r += tile_rows) tile_group[tiles++] = e;
    }
    for (; tiles < max_tiles; ++tiles) tile_group[tiles] = -1;
  }
  __syncthreads();
  for (int i = threadIdx.x; i < num_slots; i += blockDim.x) {
    const int e = ids[i];
    int place = -1;
    if (e >= 0 && e < experts) {
      place = start[e] + atomicAdd(&fill[e], 1);
      slots[place] = i;
    }
    place_of_slot[i] = place;
  }
}

// out[place, :] = x[slots[place] / top, :], zeros where the place pads an expert's run.  16-byte pieces.
__global__ void gather_places_kernel(uint4* out, const uint4* x, long long x_stride16, const int* slots, int pieces, int top) {
  const int place = blockIdx.x, slot = slots[place];
  const uint4* src = slot >= 0 ? x + static_cast<long long>(slot / top) * x_stride16 : nullptr;
  for (int i = threadIdx.x; i < pieces; i += blockDim.x)
    out[static_cast<size_t>(place) * pieces + i] = src != nullptr ? src[i] : make_uint4(0, 0, 0, 0);
}

// ------------------------------------------------------------------------------------------- products
struct ExpertProductArgs {
  void* out;               // gate/up: hidden [places, ff] in T; down: y [places, width] in float32
  const void* x;           // gate/up: the tokens [T, width]; down: hidden [places, ff]
  const void* w0;          // [experts, N, K]
  const void* w1;          // the up matrices (gate/up only)
  const int* plan;
  const int* slots;
  long long x_stride;
  int N, K, top, act;
  int interleaved;         // gate/up: w0 is [experts, 2 N, K], blocks of 8 gate rows each followed by its 8 up rows
};

// Where the tile's first gate row and first up row lie.
template <typename T>
__device__ __forceinline__ void gate_up_rows(const ExpertProductArgs& a, int expert, int n0, const T*& gate, const T*& up) {
  if (a.interleaved) {
    gate = static_cast<const T*>(a.w0) + (static_cast<size_t>(expert) * 2 * a.N + 2 * n0) * a.K;
    up = gate + static_cast<size_t>(8) * a.K;
  } else {
    const size_t at = (static_cast<size_t>(expert) * a.N + n0) * a.K;
    gate = static_cast<const T*>(a.w0) + at;
    up = static_cast<const T*>(a.w1) + at;
  }
}

__device__ __forceinline__ float expert_act(float g, int act) {
  return act == 1 ? fmaxf(g, 0.0f) : g / (1.0f + expf(-g));
}

// hidden[place, n] = act(gate_e x_t) * (up_e x_t) for the tile's places; x_t is gathered by slot / top.
template <typename T>
__global__ void __launch_bounds__(TP_THREADS) expert_gate_up_kernel(const ExpertProductArgs a) {
  __shared__ TileProductSmem sm;
  const int tile = blockIdx.x;
  if (tile >= a.plan[0]) return;
  const int expert = a.plan[1 + 3 * tile], place0 = a.plan[2 + 3 * tile], rows = a.plan[3 + 3 * tile];
  const int n0 = blockIdx.y * TP_BN;
  if (threadIdx.x < TP_BM) {
    const T* src = nullptr;
    if (static_cast<int>(threadIdx.x) < rows)
      src = static_cast<const T*>(a.x) + static_cast<long long>(a.slots[place0 + threadIdx.x] / a.top) * a.x_stride;
    sm.row[threadIdx.x] = src;
  }
  const T *gate, *up;
  gate_up_rows(a, expert, n0, gate, up);
  float acc[2][2][4];
  tile_product<T, true>(sm, gate, up, a.N - n0, a.K, acc, a.interleaved != 0);
  const int ty = threadIdx.x >> 4, tx = threadIdx.x & 15;
#pragma unroll
  for (int m = 0; m < 2; ++m) {
    const int r = 2 * ty + m;
    if (r >= rows) continue;
    T* dst = static_cast<T*>(a.out) + static_cast<size_t>(place0 + r) * a.N;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx + 16 * j;
      // The gate is rounded to the model's type before its activation, as a separate product would leave it.
      if (n < a.N) dst[n] = from_float<T>(expert_act(to_float(from_float<T>(acc[m][0][j])), a.act) *
                                          to_float(from_float<T>(acc[m][1][j])));
    }
  }
}

// y[place, n] = down_e hidden[place]  (float32).
template <typename T>
__global__ void __launch_bounds__(TP_THREADS) expert_down_kernel(const ExpertProductArgs a) {
  __shared__ TileProductSmem sm;
  const int tile = blockIdx.x;
  if (tile >= a.plan[0]) return;
  const int expert = a.plan[1 + 3 * tile], place0 = a.plan[2 + 3 * tile], rows = a.plan[3 + 3 * tile];
  const int n0 = blockIdx.y * TP_BN;
  if (threadIdx.x < TP_BM)
    sm.row[threadIdx.x] = static_cast<int>(threadIdx.x) < rows
                              ? static_cast<const T*>(a.x) + static_cast<long long>(place0 + threadIdx.x) * a.x_stride
                              : nullptr;
  const size_t w_at = (static_cast<size_t>(expert) * a.N + n0) * a.K;
  float acc[2][2][4];
  tile_product<T, false>(sm, static_cast<const T*>(a.w0) + w_at, nullptr, a.N - n0, a.K, acc);
  const int ty = threadIdx.x >> 4, tx = threadIdx.x & 15;
#pragma unroll
  for (int m = 0; m < 2; ++m) {
    const int r = 2 * ty + m;
    if (r >= rows) continue;
    float* dst = static_cast<float*>(a.out) + static_cast<size_t>(place0 + r) * a.N;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx + 16 * j;
      if (n < a.N) dst[n] = acc[m][0][j];
    }
  }
}

// The same two products on the tensor cores (bfloat16): tiles of TM_BM rows.
__global__ void __launch_bounds__(TM_THREADS) expert_gate_up_mma_kernel(const ExpertProductArgs a, int vectors) {
  __shared__ TileMmaSmem sm;
  using T = __nv_bfloat16;
  const int tile = blockIdx.x;
  if (tile >= a.plan[0]) return;
  const int expert = a.plan[1 + 3 * tile], place0 = a.plan[2 + 3 * tile], rows = a.plan[3 + 3 * tile];
  const int n0 = blockIdx.y * TM_BN;
  if (threadIdx.x < TM_BM) {
    const T* src = nullptr;
    if (static_cast<int>(threadIdx.x) < rows)
      src = static_cast<const T*>(a.x) + static_cast<long long>(a.slots[place0 + threadIdx.x] / a.top) * a.x_stride;
    sm.row[threadIdx.x] = src;
  }
  __syncthreads();
  const T *gate, *up;
  gate_up_rows(a, expert, n0, gate, up);
  float acc[2][4][4];
  tile_product_mma<true, T>(sm, gate, up, a.N - n0, a.K, vectors != 0, vectors != 0, acc, a.interleaved != 0);
#pragma unroll
  for (int nt = 0; nt < 4; ++nt)
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      const int r = tm_row(c), n = n0 + tm_col(nt, c);
      if (r < rows && n < a.N)
        static_cast<T*>(a.out)[static_cast<size_t>(place0 + r) * a.N + n] =
            from_float<T>(expert_act(to_float(from_float<T>(acc[0][nt][c])), a.act) * to_float(from_float<T>(acc[1][nt][c])));
    }
}

__global__ void __launch_bounds__(TM_THREADS) expert_down_mma_kernel(const ExpertProductArgs a, int vectors) {
  __shared__ TileMmaSmem sm;
  using T = __nv_bfloat16;
  const int tile = blockIdx.x;
  if (tile >= a.plan[0]) return;
  const int expert = a.plan[1 + 3 * tile], place0 = a.plan[2 + 3 * tile], rows = a.plan[3 + 3 * tile];
  const int n0 = blockIdx.y * TM_BN;
  if (threadIdx.x < TM_BM)
    sm.row[threadIdx.x] = static_cast<int>(threadIdx.x) < rows
                              ? static_cast<const T*>(a.x) + static_cast<long long>(place0 + threadIdx.x) * a.x_stride
                              : nullptr;
  __syncthreads();
  const size_t w_at = (static_cast<size_t>(expert) * a.N + n0) * a.K;
  float acc[2][4][4];
  tile_product_mma<false, T>(sm, static_cast<const T*>(a.w0) + w_at, nullptr, a.N - n0, a.K, vectors != 0, vectors != 0, acc);
#pragma unroll
  for (int nt = 0; nt < 4; ++nt)
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      const int r = tm_row(c), n = n0 + tm_col(nt, c);
      if (r < rows && n < a.N) static_cast<float*>(a.out)[static_cast<size_t>(place0 + r) * a.N + n] = acc[0][nt][c];
    }
}

// -------------------------------------------------------------------------------------------- combine
// Y: the type the experts' outputs come in, float32 sums (rounded to T here) or T itself.
template <typename T, typename Y>
__global__ void combine_kernel(T* out, const Y* y, long long y_stride, const T* x, long long x_stride, const int* ids,
                               const float* weights, const int* place_of_slot, int width, int top) {
  const int t = blockIdx.x;
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    float sum = 0.0f;
    for (int j = 0; j < top; ++j) {
      const int slot = t * top + j, place = place_of_slot[slot];
      const float w = weights[slot];
      // An expert's output takes the model's type before it is weighted, as a layer of its own would leave it.
      const float v = place >= 0 ? to_float(from_float<T>(to_float(y[static_cast<size_t>(place) * y_stride + i])))
                                 : to_float(x[t * x_stride + i]);
      sum = fmaf(w, v, sum);
    }
    out[static_cast<size_t>(t) * width + i] = from_float<T>(sum);
  }
}

// The same for bfloat16 rows of a multiple of 8 elements on 16-byte boundaries: a thread owns 8 neighbouring
// elements and moves them as one piece; the choices' places are read once per token.
constexpr int COMBINE_MAX_TOP = 16;
__global__ void combine_pieces_kernel(uint4* out, const uint4* y, long long y_stride16, const uint4* x, long long x_stride16,
                                      const float* weights, const int* place_of_slot, int pieces, int top) {
  const int t = blockIdx.x;
  __shared__ int place_s[COMBINE_MAX_TOP];
  __shared__ float weight_s[COMBINE_MAX_TOP];
  if (threadIdx.x < top) {
    place_s[threadIdx.x] = place_of_slot[t * top + threadIdx.x];
    weight_s[threadIdx.x] = weights[t * top + threadIdx.x];
  }
  __syncthreads();
  for (int i = threadIdx.x; i < pieces; i += blockDim.x) {
    float sum[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) sum[u] = 0.0f;
    for (int j = 0; j < top; ++j) {
      const int place = place_s[j];
      const uint4 v = place >= 0 ? y[static_cast<long long>(place) * y_stride16 + i] : x[t * x_stride16 + i];
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const float2 f = __bfloat1622float2(h[u]);
        sum[2 * u] = fmaf(weight_s[j], f.x, sum[2 * u]);
        sum[2 * u + 1] = fmaf(weight_s[j], f.y, sum[2 * u + 1]);
      }
    }
    uint4 o;
    o.x = pack_bf16(sum[0], sum[1]); o.y = pack_bf16(sum[2], sum[3]);
    o.z = pack_bf16(sum[4], sum[5]); o.w = pack_bf16(sum[6], sum[7]);
    out[static_cast<size_t>(t) * pieces + i] = o;
  }
}

}  // namespace zb

using namespace zb;

ZB_API int zb_route_max_outputs() { return 32 * ROUTE_PER_LANE; }
ZB_API int zb_expert_tile_rows(int dtype) { return dtype == DTYPE_F32 ? TP_BM : TM_BM; }

// sigmoid_scores: 0 softmax over all outputs, 1 the logistic function of each, 2 the logits themselves with
// the softmax over the taken ones as weights.  logit_bias: null, or one float32 per output.  groups <= 1: no limit on the
// choice; else the outputs form `groups` equal runs and only the `keep` best runs (by the sum of their
// `group_top` largest choice values) can be taken from: keep * (outputs / groups) must reach `top`.
ZB_API int zb_route_biased(int* ids, float* weights, const float* logits, long long logits_stride,
                           const float* correction, int tokens, int outputs, int top, int sigmoid_scores, int groups,
                           int keep, int group_top, float weight_scale, const float* logit_bias, void* stream) {
  if (tokens < 0 || outputs <= 0 || top <= 0 || top > outputs || sigmoid_scores < 0 || sigmoid_scores > 2)
    return ERR_BAD_ARGUMENT;
  if (groups > 1 && (outputs % groups != 0 || keep <= 0 || keep > groups || group_top <= 0 ||
                     keep * (outputs / groups) < top))
    return ERR_BAD_ARGUMENT;
  if (outputs > 32 * ROUTE_PER_LANE || (groups > 1 && group_top > ROUTE_GROUP_TOP_MAX)) return ERR_UNSUPPORTED;
  if (tokens == 0) return OK;
  route_kernel<<<(tokens + ROUTE_WARPS - 1) / ROUTE_WARPS, ROUTE_WARPS * 32, 0, static_cast<cudaStream_t>(stream)>>>(
      ids, weights, logits, logits_stride, correction, tokens, outputs, top, sigmoid_scores, groups, keep, group_top,
      weight_scale, logit_bias);
  return launch_result();
}

ZB_API int zb_route_grouped(int* ids, float* weights, const float* logits, long long logits_stride,
                            const float* correction, int tokens, int outputs, int top, int sigmoid_scores, int groups,
                            int keep, int group_top, float weight_scale, void* stream) {
  return zb_route_biased(ids, weights, logits, logits_stride, correction, tokens, outputs, top, sigmoid_scores, groups,
                         keep, group_top, weight_scale, nullptr, stream);
}

ZB_API int zb_route(int* ids, float* weights, const float* logits, long long logits_stride, const float* correction,
                    int tokens, int outputs, int top, void* stream) {
  return zb_route_grouped(ids, weights, logits, logits_stride, correction, tokens, outputs, top, 0, 1, 1, 1, 1.0f,
                          stream);
}

ZB_API int zb_route_align(int* plan, int* slots, int* place_of_slot, const int* ids, int num_slots, int experts,
                          int max_tiles, int tile_rows, void* stream) {
  if (num_slots < 0 || experts <= 0 || max_tiles < 0 || tile_rows <= 0) return ERR_BAD_ARGUMENT;
  const size_t smem = (3 * static_cast<size_t>(experts) + 1) * sizeof(int);
  if (smem > 48 * 1024) return ERR_UNSUPPORTED;
  align_kernel<<<1, ALIGN_THREADS, smem, static_cast<cudaStream_t>(stream)>>>(plan, slots, place_of_slot, ids,
                                                                                num_slots, experts, max_tiles, tile_rows);
  return launch_result();
}

// `down` = 0: hidden = act(gate x) * (up x), N = ff, K = width; 1: y = down hidden, N = width, K = ff.
// Without w1 the gate/up product reads w0 as [experts, 2 N, K] in blocks of 8 gate rows and their 8 up rows.
ZB_API int zb_expert_product(void* out, const void* x, long long x_stride, const void* w0, const void* w1,
                             const int* plan, const int* slots, int max_tiles, int N, int K, int top, int act,
                             int down, int dtype, void* stream) {
  if (max_tiles < 0 || N <= 0 || K <= 0 || top <= 0 || (act != 0 && act != 1)) return ERR_BAD_ARGUMENT;
  if (!down && w1 == nullptr && N % 8 != 0) return ERR_BAD_ARGUMENT;
  if (max_tiles == 0) return OK;
  ExpertProductArgs a;
  a.out = out; a.x = x; a.w0 = w0; a.w1 = w1; a.plan = plan; a.slots = slots; a.x_stride = x_stride;
  a.N = N; a.K = K; a.top = top; a.act = act;
  a.interleaved = !down && w1 == nullptr;
  const dim3 grid(max_tiles, (N + TP_BN - 1) / TP_BN);       // both tile forms are 64 outputs wide
  static_assert(TP_BN == TM_BN, "one grid for both forms");
  auto s = static_cast<cudaStream_t>(stream);
  if (dtype == DTYPE_F32) {
    if (down) expert_down_kernel<float><<<grid, TP_THREADS, 0, s>>>(a);
    else expert_gate_up_kernel<float><<<grid, TP_THREADS, 0, s>>>(a);
    return launch_result();
  }
  // Vector loads where every row of x and of the matrices starts on a 16-byte boundary.
  const int vectors = K % 8 == 0 && x_stride % 8 == 0 && tm_aligned(x, 16) && tm_aligned(w0, 16) &&
                      (w1 == nullptr || tm_aligned(w1, 16));
  if (down) expert_down_mma_kernel<<<grid, TM_THREADS, 0, s>>>(a, vectors);
  else expert_gate_up_mma_kernel<<<grid, TM_THREADS, 0, s>>>(a, vectors);
  return launch_result();
}

ZB_API int zb_route_align_padded(int* tile_group, int* slots, int* place_of_slot, const int* ids, int num_slots,
                                 int experts, int max_tiles, int tile_rows, void* stream) {
  if (num_slots < 0 || experts <= 0 || max_tiles <= 0 || tile_rows <= 0) return ERR_BAD_ARGUMENT;
  const size_t smem = (3 * static_cast<size_t>(experts) + 1) * sizeof(int);
  if (smem > 48 * 1024) return ERR_UNSUPPORTED;
  align_padded_kernel<<<1, ALIGN_THREADS, smem, static_cast<cudaStream_t>(stream)>>>(tile_group, slots, place_of_slot, ids,
                                                                                       num_slots, experts, max_tiles, tile_rows);
  return launch_result();
}

// out [places, width] = the tokens' rows in the order of `slots` (bfloat16; width a multiple of 8, 16-byte aligned rows).
ZB_API int zb_gather_places(void* out, const void* x, long long x_stride, const int* slots, int places, int width,
                            int top, void* stream) {
  if (places < 0 || width <= 0 || width % 8 != 0 || x_stride % 8 != 0 || top <= 0 ||
      reinterpret_cast<uintptr_t>(out) % 16 != 0 || reinterpret_cast<uintptr_t>(x) % 16 != 0)
    return ERR_BAD_ARGUMENT;
  if (places == 0) return OK;
  gather_places_kernel<<<places, 128, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<uint4*>(out), static_cast<const uint4*>(x), x_stride / 8, slots, width / 8, top);
  return launch_result();
}

// `y_dtype`: float32 sums, or the model's type (what the grouped tcgen05 product writes).
ZB_API int zb_route_combine(void* out, const void* y, long long y_stride, int y_dtype, const void* x, long long x_stride,
                            const int* ids, const float* weights, const int* place_of_slot, int tokens, int width, int top,
                            int dtype, void* stream) {
  if (tokens < 0 || width <= 0 || top <= 0) return ERR_BAD_ARGUMENT;
  if (tokens == 0) return OK;
  auto s = static_cast<cudaStream_t>(stream);
  const int threads = width >= 1024 ? 256 : 128;
  using bf16 = __nv_bfloat16;
  if (dtype == DTYPE_F32) {
    if (y_dtype != DTYPE_F32) return ERR_BAD_ARGUMENT;
    combine_kernel<float, float><<<tokens, threads, 0, s>>>(static_cast<float*>(out), static_cast<const float*>(y), y_stride,
                                                            static_cast<const float*>(x), x_stride, ids, weights,
                                                            place_of_slot, width, top);
  } else if (y_dtype == DTYPE_F32) {
    combine_kernel<bf16, float><<<tokens, threads, 0, s>>>(static_cast<bf16*>(out), static_cast<const float*>(y), y_stride,
                                                           static_cast<const bf16*>(x), x_stride, ids, weights, place_of_slot,
                                                           width, top);
  } else if (width % 8 == 0 && y_stride % 8 == 0 && x_stride % 8 == 0 && top <= COMBINE_MAX_TOP && tm_aligned(out, 16) &&
             tm_aligned(y, 16) && tm_aligned(x, 16)) {
    combine_pieces_kernel<<<tokens, width >= 2048 ? 256 : 128, 0, s>>>(
        static_cast<uint4*>(out), static_cast<const uint4*>(y), y_stride / 8, static_cast<const uint4*>(x), x_stride / 8,
        weights, place_of_slot, width / 8, top);
  } else {
    combine_kernel<bf16, bf16><<<tokens, threads, 0, s>>>(static_cast<bf16*>(out), static_cast<const bf16*>(y), y_stride,
                                                          static_cast<const bf16*>(x), x_stride, ids, weights, place_of_slot,
                                                          width, top);
  }
  return launch_result();
}
