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
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    const int t = t0 + tm_row(c);
    if (t >= a.tokens) continue;
    float mult = 1.0f;
    const float* gate = a.gate != nullptr ? a.gate + t * a.gate_stride : nullptr;
    if (gate != nullptr && !a.gate_per_element) mult = 1.0f / (1.0f + expf(-gate[head]));
    OUT* dst = static_cast<OUT*>(a.y) + t * a.y_stride + static_cast<long long>(head) * a.y_head_stride;
#pragma unroll
    for (int nt = 0; nt < 4; ++nt) {
      const int n = n0 + tm_col(nt, c);
      if (n >= a.N) continue;
      if (gate != nullptr && a.gate_per_element) mult = 1.0f / (1.0f + expf(-gate[static_cast<long long>(head) * a.N + n]));
      dst[n] = from_float<OUT>(acc[0][nt][c] * mult);
    }
  }
}

}  // namespace zb

using namespace zb;

// The general form: head h reads K values from x[t, h * x_head_stride ...] and writes N values to
// y[t, h * y_head_stride ...]; gate_per_element: one gate logit per output value instead of one per head.
ZB_API int zb_head_linear_strided(void* y, const void* x, const void* w, const float* gate, long long x_stride,
                                  long long y_stride, long long gate_stride, int x_head_stride, int y_head_stride,
                                  int gate_per_element, int tokens, int heads, int N, int K, int x_dtype, int dtype,
                                  int out_dtype, void* stream) {
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
                                dtype, out_dtype, stream);
}
