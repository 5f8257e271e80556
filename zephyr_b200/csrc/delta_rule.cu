// The gated delta rule: per head a state S [D key channels x V value channels], float32, and per token
//
//   S <- g S;   u = beta (v - S^T k);   S <- S + k u^T;   o = S^T q
//
// with one decay g and one step beta per head and token.  Two kernels:
//
//   delta_gates   per token: q and k heads (the model's type, as a convolution left them) made unit
//                 vectors, x / sqrt(sum(x^2) + unit_eps), q also times `q_scale`, both written as
//                 float32; beta = sigmoid(b); g = exp(-exp(A_log) softplus(a + dt_bias)), from float32
//                 projections b and a.
//   delta_scan    a CTA owns a request, a head and a run of value columns; a column is shared by L
//                 lanes that hold D / L key channels of it each.  With r_k = S^T k and r_q = S^T q of
//                 the state BEFORE the token, u = beta (v - g r_k) and o = g r_q + u (k . q): both
//                 reductions run side by side on the old state, and the write S <- g S + k u^T
//                 follows.  A request's tokens run in their order, 16 at a time staged in shared memory;
//                 the state is read from the request's slot at the start of the step's portion and
//                 written back at its end, so a prompt may be cut anywhere.  In the slot a head's state
//                 lies [V][D] (a column's channels together).
//
// Everything here is float32; the values v are read in the model's type.
#include "common.cuh"

namespace zb {

__device__ __forceinline__ float softplus_d(float z) { return fmaxf(z, 0.0f) + log1pf(expf(-fabsf(z))); }

struct DeltaGatesArgs {
  float* q_out;            // [T, qk_heads * D]
  float* k_out;            // [T, qk_heads * D]
  float* beta;             // [T, heads]
  float* decay;            // [T, heads]
  const void* q;           // [T, q_stride] the model's type
  const void* k;
  long long q_stride, k_stride;
  const float* b;          // [T, ba_stride]
  const float* a;
  long long ba_stride;
  const float* a_log;      // [heads]
  const float* dt_bias;    // [heads]
  int qk_heads, heads, D;
  float q_scale, unit_eps;
};

template <typename T>
__global__ void __launch_bounds__(128) delta_gates_kernel(const DeltaGatesArgs a) {
  const long long t = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int h = warp; h < 2 * a.qk_heads; h += 4) {
    const bool is_q = h < a.qk_heads;
    const int own = is_q ? h : h - a.qk_heads;
    const T* src = is_q ? static_cast<const T*>(a.q) + t * a.q_stride + own * a.D
                        : static_cast<const T*>(a.k) + t * a.k_stride + own * a.D;
    float ss = 0.0f;
    for (int i = lane; i < a.D; i += 32) {
      const float x = to_float(src[i]);
      ss = fmaf(x, x, ss);
    }
    const float inv = (is_q ? a.q_scale : 1.0f) / sqrtf(warp_sum(ss) + a.unit_eps);
    float* dst = (is_q ? a.q_out : a.k_out) + (t * a.qk_heads + own) * a.D;
    for (int i = lane; i < a.D; i += 32) dst[i] = to_float(src[i]) * inv;
  }
  for (int h = threadIdx.x; h < a.heads; h += blockDim.x) {
    a.beta[t * a.heads + h] = 1.0f / (1.0f + expf(-a.b[t * a.ba_stride + h]));
    a.decay[t * a.heads + h] = expf(-expf(a.a_log[h]) * softplus_d(a.a[t * a.ba_stride + h] + a.dt_bias[h]));
  }
}

// ------------------------------------------------------------------------------------------------
constexpr int DS_THREADS = 128;
constexpr int DS_TOKENS = 16;       // tokens staged at a time

struct DeltaScanArgs {
  float* out;              // [T, heads * V]
  const float* q;          // [T, qk_heads * D]
  const float* k;
  const void* v;           // [T, v_stride], head h at column h * V, the model's type
  long long v_stride;
  const float* beta;       // [T, heads]
  const float* decay;
  float* state;            // slot s at state + s * slot_stride: [heads][V][D]
  long long slot_stride;
  const int* slots;
  const int* row_q_start;
  const int* row_q_len;
  int heads, heads_per_group, D, V, num_slots, write_state;
  int* status;
};

// KPL: key channels a lane holds; L = lanes of a column (a power of two, L * KPL >= D); channel
// d = l + L * i lies with lane l as its i-th.
template <typename T, int KPL>
__global__ void __launch_bounds__(DS_THREADS) delta_scan_kernel(const DeltaScanArgs a, int L) {
  extern __shared__ __align__(16) float ds_smem[];
  const int D = a.D, V = a.V;
  float* q_s = ds_smem;                          // [DS_TOKENS][D]
  float* k_s = q_s + DS_TOKENS * D;              // [DS_TOKENS][D]
  const int cols = DS_THREADS / L;               // value columns of this CTA
  float* v_s = k_s + DS_TOKENS * D;              // [DS_TOKENS][cols]
  float* beta_s = v_s + DS_TOKENS * cols;        // [DS_TOKENS]
  float* decay_s = beta_s + DS_TOKENS;
  float* kq_s = decay_s + DS_TOKENS;

  const int row = blockIdx.x, head = blockIdx.y, col0 = blockIdx.z * cols;
  const int slot = a.slots[row];
  if (slot < 0 || slot >= a.num_slots) {
    if (threadIdx.x == 0) report(a.status, STATUS_ROW_OUT_OF_RANGE, slot, row);
    return;
  }
  const int t0 = a.row_q_start[row], n = a.row_q_len[row];
  const int l = threadIdx.x % L, col = col0 + threadIdx.x / L;
  const bool live = col < V;
  const int group = head / a.heads_per_group, qk_heads = a.heads / a.heads_per_group;
  float* mine = a.state + static_cast<long long>(slot) * a.slot_stride +
                (static_cast<long long>(head) * V + (live ? col : 0)) * D;
  float S[KPL];
#pragma unroll
  for (int i = 0; i < KPL; ++i) {
    const int d = l + L * i;
    S[i] = (live && d < D) ? mine[d] : 0.0f;
  }
  const T* v = static_cast<const T*>(a.v);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int base = 0; base < n; base += DS_TOKENS) {
    const int nt = min(DS_TOKENS, n - base);
    __syncthreads();            // the tokens staged before are no longer read
    for (int e = threadIdx.x; e < nt * D; e += DS_THREADS) {
      const int j = e / D, d = e - j * D;
      const long long at = (static_cast<long long>(t0 + base + j) * qk_heads + group) * D + d;
      q_s[j * D + d] = a.q[at];
      k_s[j * D + d] = a.k[at];
    }
    for (int e = threadIdx.x; e < nt * cols; e += DS_THREADS) {
      const int j = e / cols, c = e - j * cols;
      v_s[e] = col0 + c < V ? to_float(v[static_cast<long long>(t0 + base + j) * a.v_stride + head * V + col0 + c]) : 0.0f;
    }
    if (threadIdx.x < nt) {
      beta_s[threadIdx.x] = a.beta[static_cast<long long>(t0 + base + threadIdx.x) * a.heads + head];
      decay_s[threadIdx.x] = a.decay[static_cast<long long>(t0 + base + threadIdx.x) * a.heads + head];
    }
    __syncthreads();
    for (int j = warp; j < nt; j += DS_THREADS / 32) {      // k . q of every staged token, in lane order
      float s = 0.0f;
      for (int d = lane; d < D; d += 32) s = fmaf(k_s[j * D + d], q_s[j * D + d], s);
      s = warp_sum(s);
      if (lane == 0) kq_s[j] = s;
    }
    __syncthreads();
    for (int j = 0; j < nt; ++j) {
      const float* kj = k_s + j * D;
      const float* qj = q_s + j * D;
      float rk = 0.0f, rq = 0.0f;
#pragma unroll
      for (int i = 0; i < KPL; ++i) {
        const int d = l + L * i;
        if (d < D) {
          rk = fmaf(S[i], kj[d], rk);
          rq = fmaf(S[i], qj[d], rq);
        }
      }
      for (int o = L >> 1; o > 0; o >>= 1) {
        rk += __shfl_xor_sync(0xffffffffu, rk, o);
        rq += __shfl_xor_sync(0xffffffffu, rq, o);
      }
      const float g = decay_s[j];
      const float u = beta_s[j] * (v_s[j * cols + threadIdx.x / L] - g * rk);
#pragma unroll
      for (int i = 0; i < KPL; ++i) {
        const int d = l + L * i;
        if (d < D) S[i] = fmaf(kj[d], u, g * S[i]);
      }
      if (l == 0 && live)
        a.out[static_cast<long long>(t0 + base + j) * a.heads * V + head * V + col] = fmaf(u, kq_s[j], g * rq);
    }
  }
  if (a.write_state && live) {
#pragma unroll
    for (int i = 0; i < KPL; ++i) {
      const int d = l + L * i;
      if (d < D) mine[d] = S[i];
    }
  }
}

}  // namespace zb

using namespace zb;

ZB_API int zb_delta_max_channels() { return 512; }

ZB_API int zb_delta_gates(float* q_out, float* k_out, float* beta, float* decay, const void* q, long long q_stride,
                          const void* k, long long k_stride, const float* b, const float* a, long long ba_stride,
                          const float* a_log, const float* dt_bias, int tokens, int qk_heads, int heads, int D,
                          float q_scale, float unit_eps, int dtype, void* stream) {
  if (tokens < 0 || qk_heads <= 0 || heads <= 0 || D <= 0) return ERR_BAD_ARGUMENT;
  if (tokens == 0) return OK;
  DeltaGatesArgs g;
  g.q_out = q_out; g.k_out = k_out; g.beta = beta; g.decay = decay; g.q = q; g.k = k; g.q_stride = q_stride;
  g.k_stride = k_stride; g.b = b; g.a = a; g.ba_stride = ba_stride; g.a_log = a_log; g.dt_bias = dt_bias;
  g.qk_heads = qk_heads; g.heads = heads; g.D = D; g.q_scale = q_scale; g.unit_eps = unit_eps;
  auto s = static_cast<cudaStream_t>(stream);
  if (dtype == DTYPE_F32) delta_gates_kernel<float><<<tokens, 128, 0, s>>>(g);
  else delta_gates_kernel<__nv_bfloat16><<<tokens, 128, 0, s>>>(g);
  return launch_result();
}

template <typename T, int KPL>
static int delta_scan_launch(const DeltaScanArgs& a, int L, int rows, cudaStream_t s) {
  const int cols = DS_THREADS / L;
  const size_t smem = sizeof(float) * (2 * DS_TOKENS * a.D + DS_TOKENS * cols + 3 * DS_TOKENS);
  auto kernel = delta_scan_kernel<T, KPL>;
  if (smem > 48 * 1024 &&
      cuda_failed(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem))))
    return ERR_CUDA;
  kernel<<<dim3(rows, a.heads, (a.V + cols - 1) / cols), DS_THREADS, smem, s>>>(a, L);
  return launch_result();
}

ZB_API int zb_delta_scan(float* out, const float* q, const float* k, const void* v, long long v_stride,
                         const float* beta, const float* decay, float* state, long long slot_stride, const int* slots,
                         const int* row_q_start, const int* row_q_len, int rows, int heads, int heads_per_group, int D,
                         int V, int num_slots, int write_state, int dtype, int* status, void* stream) {
  if (rows < 0 || heads <= 0 || heads_per_group <= 0 || heads % heads_per_group != 0 || D <= 0 || V <= 0)
    return ERR_BAD_ARGUMENT;
  if (D > zb_delta_max_channels()) return ERR_UNSUPPORTED;
  if (rows == 0) return OK;
  DeltaScanArgs a;
  a.out = out; a.q = q; a.k = k; a.v = v; a.v_stride = v_stride; a.beta = beta; a.decay = decay; a.state = state;
  a.slot_stride = slot_stride; a.slots = slots; a.row_q_start = row_q_start; a.row_q_len = row_q_len;
  a.heads = heads; a.heads_per_group = heads_per_group; a.D = D; a.V = V; a.num_slots = num_slots;
  a.write_state = write_state; a.status = status;
  auto s = static_cast<cudaStream_t>(stream);
  // Few channels: 4 a lane, so that a column still spreads over several lanes; many: 16 a lane.
  const int kpl = D <= 64 ? 4 : 16;
  int L = 1;
  while (L * kpl < D) L *= 2;
  if (L > 32) return ERR_UNSUPPORTED;
  if (dtype == DTYPE_F32)
    return kpl == 4 ? delta_scan_launch<float, 4>(a, L, rows, s) : delta_scan_launch<float, 16>(a, L, rows, s);
  return kpl == 4 ? delta_scan_launch<__nv_bfloat16, 4>(a, L, rows, s)
                  : delta_scan_launch<__nv_bfloat16, 16>(a, L, rows, s);
}
