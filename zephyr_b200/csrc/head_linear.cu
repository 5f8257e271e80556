// A product that is block-diagonal over heads:  y[t, h, n] = sum_k x[t, h, k] * W[h, n, k], every head
// with a matrix of its own ([heads, N, K], rows K apart).  Optionally each head's output is multiplied
// by the logistic function of one number per token and head (a gate on the head's output).
//
// Latent attention uses it twice: the queries of a head are carried into the latent space by the
// transposed key map of that head (so that scores are taken against the cached latent itself), and the
// attention's result, a weighted sum of latents per head, is carried out of it by the head's value map.
//
// float32 sums in the order of k; W and y in the model's type (y may be float32), x in that type or in
// float32 (a projection that was left unrounded).  float32 matrices run on CUDA cores, bfloat16 ones on
// the tensor cores (x rounded to bfloat16 as it is staged).
//
// The op moves far more bytes than it multiplies (K and N are a head's sizes), so the bfloat16 form that
// serves whole models stages ALL of K at once: a CTA asks for its 64 rows of x and up to 128 rows of the
// head's matrix in one go (asynchronous 16-byte copies, or 16-byte loads that round float32 rows on
// their way), waits once, multiplies out of shared memory and stores pairs of outputs.  Shapes whose rows
// do not start on 16-byte boundaries, or whose K is no multiple of 16, and fewer than a few hundred rows take
// the tile walk in steps of 32.
#include "tile_product.cuh"
#include "tile_product_mma.cuh"

namespace zb {

struct HeadLinearArgs {
  void* y;                // [T, heads * N], rows y_stride apart
  const void* x;          // [T, heads * K], rows x_stride apart
  const void* w;          // [heads, N, K]
  const float* gate;      // null, or one logit per (token, head): gate[t * gate_stride + h]; with
                          // gate_per_element one per output: gate[t * gate_stride + h * N + n]
  long long x_stride, y_stride, gate_stride;
  int tokens, heads, N, K;
  int x_head_stride, y_head_stride;     // a head's K inputs and N outputs may be slices of wider heads
  int gate_per_element;
};

template <typename X, typename T, typename OUT>
__global__ void __launch_bounds__(TP_THREADS) head_linear_kernel(const HeadLinearArgs a) {
  __shared__ TileProductSmem sm;
  const int t0 = blockIdx.x * TP_BM, n0 = blockIdx.y * TP_BN, head = blockIdx.z;
  if (threadIdx.x < TP_BM) {
    const int t = t0 + threadIdx.x;
    sm.row[threadIdx.x] = t < a.tokens ? static_cast<const X*>(a.x) + t * a.x_stride + static_cast<long long>(head) * a.x_head_stride
                                       : nullptr;
  }
  const T* w = static_cast<const T*>(a.w) + (static_cast<size_t>(head) * a.N + n0) * a.K;
  float acc[2][2][4];
  tile_product<T, false, X>(sm, w, w, a.N - n0, a.K, acc);
  const int ty = threadIdx.x >> 4, tx = threadIdx.x & 15;
#pragma unroll
  for (int m = 0; m < 2; ++m) {
    const int t = t0 + 2 * ty + m;
    if (t >= a.tokens) continue;
    float mult = 1.0f;
    const float* gate = a.gate != nullptr ? a.gate + t * a.gate_stride : nullptr;
    if (gate != nullptr && !a.gate_per_element) mult = 1.0f / (1.0f + expf(-gate[head]));
    OUT* dst = static_cast<OUT*>(a.y) + t * a.y_stride + static_cast<long long>(head) * a.y_head_stride;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx + 16 * j;
      if (n >= a.N) continue;
      if (gate != nullptr && a.gate_per_element) mult = 1.0f / (1.0f + expf(-gate[static_cast<long long>(head) * a.N + n]));
      dst[n] = from_float<OUT>(acc[m][0][j] * mult);
    }
  }
}

template <typename X, typename OUT>
__global__ void __launch_bounds__(TM_THREADS) head_linear_mma_kernel(const HeadLinearArgs a, int a_vectors, int w_vectors) {
  __shared__ TileMmaSmem sm;
  const int t0 = blockIdx.x * TM_BM, n0 = blockIdx.y * TM_BN, head = blockIdx.z;
  if (threadIdx.x < TM_BM) {
    const int t = t0 + threadIdx.x;
    sm.row[threadIdx.x] = t < a.tokens ? static_cast<const X*>(a.x) + t * a.x_stride + static_cast<long long>(head) * a.x_head_stride
                                       : nullptr;
  }
  __syncthreads();
  const __nv_bfloat16* w = static_cast<const __nv_bfloat16*>(a.w) + (static_cast<size_t>(head) * a.N + n0) * a.K;
  float acc[2][4][4];
  tile_product_mma<false, X>(sm, w, nullptr, a.N - n0, a.K, a_vectors != 0, w_vectors != 0, acc);
  // All gates first, then the stores: a load behind a store would wait for it.
  float raw[4][4];
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    const int t = t0 + tm_row(c);
    const float* gate = a.gate != nullptr && t < a.tokens ? a.gate + t * a.gate_stride : nullptr;
#pragma unroll
    for (int nt = 0; nt < 4; ++nt) {
      const int n = n0 + tm_col(nt, c);
      raw[c][nt] = 0.0f;
      if (gate != nullptr && a.gate_per_element && n < a.N) raw[c][nt] = gate[static_cast<long long>(head) * a.N + n];
      else if (gate != nullptr && !a.gate_per_element && nt == 0) raw[c][0] = gate[head];
    }
  }
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    const int t = t0 + tm_row(c);
    if (t >= a.tokens) continue;
    OUT* dst = static_cast<OUT*>(a.y) + t * a.y_stride + static_cast<long long>(head) * a.y_head_stride;
#pragma unroll
    for (int nt = 0; nt < 4; ++nt) {
      const int n = n0 + tm_col(nt, c);
      if (n >= a.N) continue;
      float mult = 1.0f;
      if (a.gate != nullptr) mult = 1.0f / (1.0f + expf(-raw[c][a.gate_per_element ? nt : 0]));
      dst[n] = from_float<OUT>(acc[0][nt][c] * mult);
    }
  }
}

__device__ __forceinline__ void store_pair(float* p, float lo, float hi) { *reinterpret_cast<float2*>(p) = make_float2(lo, hi); }
__device__ __forceinline__ void store_pair(__nv_bfloat16* p, float lo, float hi) {
  *reinterpret_cast<__nv_bfloat162*>(p) = __floats2bfloat162_rn(lo, hi);
}

constexpr int HW_BN = 128;       // outputs of the head a CTA
constexpr int HW_THREADS = 256;
constexpr int HW_MAX_K = 512;    // (64 + 128) rows of K + 8 bfloat16 values fit shared memory
// Which form runs (the sums are the same to the bit): 64 rows a CTA from HW_ROWS_64 rows on, 32 rows a CTA from
// HW_ROWS_32 on (more and smaller CTAs while there are few), below that the walk, whose still smaller tiles
// fill the SMs better.  Measured at 16 heads of 128 x 128.
constexpr int HW_ROWS_64 = 1536;
constexpr int HW_ROWS_32 = 384;

// BM rows of x a CTA (64, or 32 for more and smaller CTAs).  8 warps: BM / 16 of them along the rows, the others
// along the outputs, each with 16 rows and 128 / (8 / (BM / 16)) outputs: eight or four m16n8 tiles.
// Rows of shared memory are K + 8 values apart, which spreads the fragment loads over all banks for
// every K that is a multiple of 16.  `pairs` bit 0: every output row starts on an even element and on a
// boundary of two elements' bytes, so two neighbouring outputs go out as one store; bit 1: the same for
// the gates per output value, which then come in as pairs.
template <typename X, typename OUT, int BM>
__global__ void __launch_bounds__(HW_THREADS, BM == 32 ? 5 : 4) head_linear_whole_k_kernel(const HeadLinearArgs a, int pairs) {
  extern __shared__ __align__(16) unsigned char hw_smem[];
  const int K = a.K, ld = K + 8, pieces = K / 8;
  __nv_bfloat16* sa = reinterpret_cast<__nv_bfloat16*>(hw_smem);      // [BM][ld]
  __nv_bfloat16* sb = sa + BM * ld;                                 // [HW_BN][ld]
  const int t0 = blockIdx.x * BM, n0 = blockIdx.y * HW_BN, head = blockIdx.z, tid = threadIdx.x;
  const int n_here = min(HW_BN, a.N - n0), rows_here = min(BM, a.tokens - t0);
  const int n_tiles = (n_here + 7) / 8 * 8;                            // rows of the matrix that are multiplied at all
  const __nv_bfloat16* w = static_cast<const __nv_bfloat16*>(a.w) + (static_cast<size_t>(head) * a.N + n0) * K;
  if (a.gate != nullptr && a.gate_per_element) {
    // The gates are read last, when the sums are there: ask for their lines now, so that they wait in L2.
    for (int e = tid; e < rows_here * ((n_here + 31) / 32); e += HW_THREADS) {
      const int r = e / ((n_here + 31) / 32), line = e - r * ((n_here + 31) / 32);
      const float* p = a.gate + (t0 + r) * a.gate_stride + static_cast<long long>(head) * a.N + n0 + min(line * 32, n_here - 1);
      asm volatile("prefetch.L2 [%0];\n" ::"l"(p));
    }
  }
  for (int e = tid; e < n_tiles * pieces; e += HW_THREADS) {
    const int r = e / pieces, c = e - r * pieces;
    cp_async_16(sb + r * ld + c * 8, w + static_cast<size_t>(r < n_here ? r : 0) * K + c * 8, r < n_here);
  }
  const X* x = static_cast<const X*>(a.x) + static_cast<long long>(t0) * a.x_stride + static_cast<long long>(head) * a.x_head_stride;
  if (sizeof(X) == 2) {
    for (int e = tid; e < BM * pieces; e += HW_THREADS) {
      const int r = e / pieces, c = e - r * pieces;
      cp_async_16(sa + r * ld + c * 8, x + static_cast<long long>(r < rows_here ? r : 0) * a.x_stride + c * 8, r < rows_here);
    }
  } else {
    // float32 rows: four pieces a thread are on their way before the first is rounded and stored.
    for (int e0 = tid; e0 < BM * pieces; e0 += 4 * HW_THREADS) {
      uint4 v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int e = e0 + u * HW_THREADS, r = e / pieces, c = e - r * pieces;
        v[u] = e < BM * pieces && r < rows_here ? tm_load8(x + static_cast<long long>(r) * a.x_stride + c * 8)
                                                   : make_uint4(0, 0, 0, 0);
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int e = e0 + u * HW_THREADS, r = e / pieces, c = e - r * pieces;
        if (e < BM * pieces) *reinterpret_cast<uint4*>(sa + r * ld + c * 8) = v[u];
      }
    }
  }
  cp_async_commit();
  cp_async_wait<0>();
  __syncthreads();

  const int warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
  constexpr int MW = BM / 16, NT = HW_BN / (8 / MW) / 8;     // warps along the rows; m16n8 tiles a warp
  const int m0 = (warp % MW) * 16, nb = (warp / MW) * (NT * 8);
  float acc[NT][4];
#pragma unroll
  for (int nt = 0; nt < NT; ++nt)
#pragma unroll
    for (int c = 0; c < 4; ++c) acc[nt][c] = 0.0f;
  if (m0 < rows_here && nb < n_here) {
    const __nv_bfloat16* a_lo = sa + (m0 + g) * ld + 2 * t;
    const __nv_bfloat16* a_hi = a_lo + 8 * ld;
    const __nv_bfloat16* b_row = sb + (nb + g) * ld + 2 * t;
    for (int kk = 0; kk < K; kk += 16) {
      unsigned af[4];
      af[0] = *reinterpret_cast<const unsigned*>(a_lo + kk);
      af[1] = *reinterpret_cast<const unsigned*>(a_hi + kk);
      af[2] = *reinterpret_cast<const unsigned*>(a_lo + kk + 8);
      af[3] = *reinterpret_cast<const unsigned*>(a_hi + kk + 8);
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        if (nb + nt * 8 >= n_here) break;                     // uniform over the warp
        const __nv_bfloat16* b = b_row + nt * 8 * ld + kk;
        mma_bf16_16816(acc[nt], af, *reinterpret_cast<const unsigned*>(b), *reinterpret_cast<const unsigned*>(b + 8));
      }
    }
  }
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const int row = t0 + m0 + g + 8 * half;
    if (row >= a.tokens) continue;
    const float* gate = a.gate != nullptr ? a.gate + row * a.gate_stride : nullptr;
    // All of the row's gates first, then the stores: a load behind a store would wait for it.
    float mult[NT][2];
    if (gate != nullptr && a.gate_per_element) {
      float raw[NT][2];
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        const int n = n0 + nb + nt * 8 + 2 * t;
        const float* gv = gate + static_cast<long long>(head) * a.N + n;
        raw[nt][0] = raw[nt][1] = 0.0f;
        if ((pairs & 2) && n + 1 < a.N) {
          const float2 two = *reinterpret_cast<const float2*>(gv);
          raw[nt][0] = two.x;
          raw[nt][1] = two.y;
        } else {
          if (n < a.N) raw[nt][0] = gv[0];
          if (n + 1 < a.N) raw[nt][1] = gv[1];
        }
      }
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        mult[nt][0] = 1.0f / (1.0f + expf(-raw[nt][0]));
        mult[nt][1] = 1.0f / (1.0f + expf(-raw[nt][1]));
      }
    } else {
      const float head_mult = gate != nullptr ? 1.0f / (1.0f + expf(-gate[head])) : 1.0f;
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) mult[nt][0] = mult[nt][1] = head_mult;
    }
    OUT* dst = static_cast<OUT*>(a.y) + row * a.y_stride + static_cast<long long>(head) * a.y_head_stride;
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      const int n = n0 + nb + nt * 8 + 2 * t;
      if (n >= a.N) continue;
      const float v0 = acc[nt][2 * half] * mult[nt][0], v1 = acc[nt][2 * half + 1] * mult[nt][1];
      if ((pairs & 1) && n + 1 < a.N) {
        store_pair(dst + n, v0, v1);
      } else {
        dst[n] = from_float<OUT>(v0);
        if (n + 1 < a.N) dst[n + 1] = from_float<OUT>(v1);
      }
    }
  }
}

template <typename X, typename OUT, int BM>
int head_linear_whole_k_launch(const HeadLinearArgs& a, cudaStream_t s) {
  const size_t smem = static_cast<size_t>(BM + HW_BN) * (a.K + 8) * sizeof(__nv_bfloat16);
  auto kernel = head_linear_whole_k_kernel<X, OUT, BM>;
  static size_t allowed = 48 * 1024;         // of this instantiation; raised once per larger K
  if (smem > allowed) {
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)) != cudaSuccess)
      return ERR_CUDA;
    allowed = smem;
  }
  const bool pairs = tm_aligned(a.y, 2 * sizeof(OUT)) && a.y_stride % 2 == 0 && a.y_head_stride % 2 == 0;
  const bool gate_pairs = a.gate != nullptr && a.gate_per_element && tm_aligned(a.gate, 8) && a.gate_stride % 2 == 0 && a.N % 2 == 0;
  const dim3 grid((a.tokens + BM - 1) / BM, (a.N + HW_BN - 1) / HW_BN, a.heads);
  kernel<<<grid, HW_THREADS, smem, s>>>(a, (pairs ? 1 : 0) | (gate_pairs ? 2 : 0));
  return launch_result();
}

}  // namespace zb

using namespace zb;

// The general form: head h reads K values from x[t, h * x_head_stride ...] and writes N values to
// y[t, h * y_head_stride ...]; gate_per_element: one gate logit per output value instead of one per head;
// walk: 0 the form that suits the shape and the row count; for comparison, where the shape allows all of K at
// once: 1 the tile walk in steps along k, 2 all of K with 32 rows a CTA, 3 with 64.
ZB_API int zb_head_linear_strided(void* y, const void* x, const void* w, const float* gate, long long x_stride,
                                  long long y_stride, long long gate_stride, int x_head_stride, int y_head_stride,
                                  int gate_per_element, int tokens, int heads, int N, int K, int x_dtype, int dtype,
                                  int out_dtype, int walk, void* stream) {
  if (tokens < 0 || heads <= 0 || N <= 0 || K <= 0 || heads > 65535 || x_head_stride < K || y_head_stride < N)
    return ERR_BAD_ARGUMENT;
  if (tokens == 0) return OK;
  HeadLinearArgs a;
  a.y = y; a.x = x; a.w = w; a.gate = gate; a.x_stride = x_stride; a.y_stride = y_stride; a.gate_stride = gate_stride;
  a.tokens = tokens; a.heads = heads; a.N = N; a.K = K;
  a.x_head_stride = x_head_stride; a.y_head_stride = y_head_stride; a.gate_per_element = gate_per_element;
  const dim3 grid((tokens + TP_BM - 1) / TP_BM, (N + TP_BN - 1) / TP_BN, heads);
  auto s = static_cast<cudaStream_t>(stream);
  using bf16 = __nv_bfloat16;
  if (dtype == DTYPE_F32) {
    if (out_dtype != DTYPE_F32 || x_dtype != DTYPE_F32) return ERR_BAD_ARGUMENT;
    head_linear_kernel<float, float, float><<<grid, TP_THREADS, 0, s>>>(a);
    return launch_result();
  }
  const dim3 wide((tokens + TM_BM - 1) / TM_BM, (N + TM_BN - 1) / TM_BN, heads);
  const int w_vectors = K % 8 == 0 && tm_aligned(w, 16);
  const int per16 = x_dtype == DTYPE_F32 ? 4 : 8;          // elements of x in 16 bytes
  const bool all_of_k = K % 16 == 0 && K <= HW_MAX_K && w_vectors && x_stride % per16 == 0 && x_head_stride % per16 == 0 &&
                        tm_aligned(x, 16);
  if (all_of_k && walk != 1 && (walk >= 2 || tokens >= HW_ROWS_32)) {
    if (walk == 2 || (walk == 0 && tokens < HW_ROWS_64)) {
      if (x_dtype == DTYPE_F32)
        return out_dtype == DTYPE_F32 ? head_linear_whole_k_launch<float, float, 32>(a, s) : head_linear_whole_k_launch<float, bf16, 32>(a, s);
      return out_dtype == DTYPE_F32 ? head_linear_whole_k_launch<bf16, float, 32>(a, s) : head_linear_whole_k_launch<bf16, bf16, 32>(a, s);
    }
    if (x_dtype == DTYPE_F32)
      return out_dtype == DTYPE_F32 ? head_linear_whole_k_launch<float, float, 64>(a, s) : head_linear_whole_k_launch<float, bf16, 64>(a, s);
    return out_dtype == DTYPE_F32 ? head_linear_whole_k_launch<bf16, float, 64>(a, s) : head_linear_whole_k_launch<bf16, bf16, 64>(a, s);
  }
  if (x_dtype == DTYPE_F32) {
    const int a_vectors = K % 8 == 0 && x_stride % 4 == 0 && x_head_stride % 4 == 0 && tm_aligned(x, 16);
    if (out_dtype == DTYPE_F32) head_linear_mma_kernel<float, float><<<wide, TM_THREADS, 0, s>>>(a, a_vectors, w_vectors);
    else head_linear_mma_kernel<float, bf16><<<wide, TM_THREADS, 0, s>>>(a, a_vectors, w_vectors);
  } else {
    const int a_vectors = K % 8 == 0 && x_stride % 8 == 0 && x_head_stride % 8 == 0 && tm_aligned(x, 16);
    if (out_dtype == DTYPE_F32) head_linear_mma_kernel<bf16, float><<<wide, TM_THREADS, 0, s>>>(a, a_vectors, w_vectors);
    else head_linear_mma_kernel<bf16, bf16><<<wide, TM_THREADS, 0, s>>>(a, a_vectors, w_vectors);
  }
  return launch_result();
}

ZB_API int zb_head_linear(void* y, const void* x, const void* w, const float* gate, long long x_stride,
                          long long y_stride, long long gate_stride, int tokens, int heads, int N, int K, int x_dtype,
                          int dtype, int out_dtype, void* stream) {
  return zb_head_linear_strided(y, x, w, gate, x_stride, y_stride, gate_stride, K, N, 0, tokens, heads, N, K, x_dtype,
                                dtype, out_dtype, 0, stream);
}
