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
#include "mma.cuh"

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

// KPL: key channels a lane holds (a multiple of 4); L: lanes of a column (a power of two, L * KPL >= D);
// lane l holds the channels l * KPL .. l * KPL + KPL - 1.  Both are compile-time, so every address inside the
// token loop is a base plus a constant.  Tokens are staged 16 at a time into one of two buffers: while a
// portion's 16 tokens are worked on, the next 16 are on their way (q and k by 16-byte asynchronous copies
// where D is a multiple of 4, else by plain loads; v, beta and the decays through registers).  In shared
// memory a token's q (and k) is L runs of KPL + 4 floats (the 4 keep the lanes' 16-byte loads on separate
// banks); what lies beyond D is zero, so the token loop needs no bounds.  Inside the 16 tokens a lane holds
// the NEXT token's k and q in registers while the chain S -> S^T k -> u -> S of the present token runs, and
// sums its products in four separate sums, so the chain a token adds is the reduction over the L lanes, one
// multiply-add and the write, not the loads.  k . q is summed over the same lanes beside the two read-outs.
// CPT: value columns a thread holds (its group's column and the one `groups` further on): two columns are two
// chains whose waits overlap; a step of single tokens keeps one, so that its CTAs stay many.
template <typename T, int KPL, int L, int CPT, bool ASYNC>
__global__ void __launch_bounds__(DS_THREADS) delta_scan_kernel(const DeltaScanArgs a) {
  extern __shared__ __align__(16) float ds_smem[];
  constexpr int RUN = KPL + 4, DP = L * RUN;      // a lane's run and a token's row in shared memory
  constexpr int groups = DS_THREADS / L;          // groups of L lanes
  constexpr int cols = groups * CPT;              // value columns of this CTA: CPT a group (column group + c * groups)
  constexpr int stage_floats = 2 * DS_TOKENS * DP + DS_TOKENS * cols + 2 * DS_TOKENS;
  // one stage: q [DS_TOKENS][DP], k [DS_TOKENS][DP], v [DS_TOKENS][cols], beta [DS_TOKENS], decay [DS_TOKENS]
  const int D = a.D, V = a.V;

  const int row = blockIdx.x, head = blockIdx.y, col0 = blockIdx.z * cols;
  const int slot = a.slots[row];
  if (slot < 0 || slot >= a.num_slots) {
    if (threadIdx.x == 0) report(a.status, STATUS_ROW_OUT_OF_RANGE, slot, row);
    return;
  }
  const int t0 = a.row_q_start[row], n = a.row_q_len[row];
  const int l = threadIdx.x % L, my_group = threadIdx.x / L;
  const int group = head / a.heads_per_group, qk_heads = a.heads / a.heads_per_group;
  // A thread's CPT columns are separate chains: one column's exchanges and writes run under the other's sums.
  bool live[CPT];
  float* mine[CPT];
  float S[CPT][KPL];
  const bool state_vectors = ASYNC && D % 4 == 0;
#pragma unroll
  for (int c = 0; c < CPT; ++c) {
    const int col = col0 + my_group + c * groups;
    live[c] = col < V;
    mine[c] = a.state + static_cast<long long>(slot) * a.slot_stride +
              (static_cast<long long>(head) * V + (live[c] ? col : 0)) * D + l * KPL;
    if (state_vectors) {
#pragma unroll
      for (int i = 0; i < KPL; i += 4) {
        float4 x = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        if (live[c] && l * KPL + i < D) x = *reinterpret_cast<const float4*>(mine[c] + i);
        S[c][i] = x.x; S[c][i + 1] = x.y; S[c][i + 2] = x.z; S[c][i + 3] = x.w;
      }
    } else {
#pragma unroll
      for (int i = 0; i < KPL; ++i) S[c][i] = (live[c] && l * KPL + i < D) ? mine[c][i] : 0.0f;
    }
  }
  for (int e = threadIdx.x; e < 2 * stage_floats; e += DS_THREADS) ds_smem[e] = 0.0f;
  __syncthreads();
  const T* v = static_cast<const T*>(a.v);
  const int chunks = (n + DS_TOKENS - 1) / DS_TOKENS;
  const int vec = D / 4;                         // 16-byte pieces of a row of q or k (ASYNC: D % 4 == 0)

  auto fetch_v = [&](int base, int nt, int e) -> float {
    const int j = e / cols, c = e - j * cols;
    return (j < nt && col0 + c < V)
               ? to_float(v[static_cast<long long>(t0 + base + j) * a.v_stride + head * V + col0 + c]) : 0.0f;
  };
  auto issue_qk = [&](int base, int nt, float* stage) {
    float* q_s = stage;
    float* k_s = stage + DS_TOKENS * DP;
    if (ASYNC) {
      for (int e = threadIdx.x; e < nt * vec; e += DS_THREADS) {
        const int j = e / vec, c = (e - j * vec) * 4;
        const long long at = (static_cast<long long>(t0 + base + j) * qk_heads + group) * D + c;
        const int to = j * DP + (c / KPL) * RUN + c % KPL;
        cp_async_16(q_s + to, a.q + at, true);
        cp_async_16(k_s + to, a.k + at, true);
      }
    } else {
      for (int e = threadIdx.x; e < nt * D; e += DS_THREADS) {
        const int j = e / D, d = e - j * D;
        const long long at = (static_cast<long long>(t0 + base + j) * qk_heads + group) * D + d;
        const int to = j * DP + (d / KPL) * RUN + d % KPL;
        q_s[to] = a.q[at];
        k_s[to] = a.k[at];
      }
    }
    cp_async_commit();
  };
  constexpr int V_PER = (DS_TOKENS * cols + DS_THREADS - 1) / DS_THREADS;
  float v_next[V_PER], beta_next = 0.0f, decay_next = 0.0f;
  auto fetch_rest = [&](int base, int nt) {
#pragma unroll
    for (int r = 0; r < V_PER; ++r) {
      const int e = threadIdx.x + r * DS_THREADS;
      v_next[r] = e < DS_TOKENS * cols ? fetch_v(base, nt, e) : 0.0f;
    }
    if (threadIdx.x < nt) {
      beta_next = a.beta[static_cast<long long>(t0 + base + threadIdx.x) * a.heads + head];
      decay_next = a.decay[static_cast<long long>(t0 + base + threadIdx.x) * a.heads + head];
    }
  };
  auto store_rest = [&](float* stage) {
    float* v_s = stage + 2 * DS_TOKENS * DP;
#pragma unroll
    for (int r = 0; r < V_PER; ++r) {
      const int e = threadIdx.x + r * DS_THREADS;
      if (e < DS_TOKENS * cols) v_s[e] = v_next[r];
    }
    if (threadIdx.x < DS_TOKENS) {
      v_s[DS_TOKENS * cols + threadIdx.x] = beta_next;
      v_s[DS_TOKENS * cols + DS_TOKENS + threadIdx.x] = decay_next;
    }
  };
  auto load_run = [&](float (&x)[KPL], const float* from) {
#pragma unroll
    for (int i = 0; i < KPL; i += 4) {
      const float4 r = *reinterpret_cast<const float4*>(from + i);
      x[i] = r.x; x[i + 1] = r.y; x[i + 2] = r.z; x[i + 3] = r.w;
    }
  };
  float* out = a.out + static_cast<long long>(t0) * a.heads * V + head * V + col0 + my_group;
  const long long out_stride = static_cast<long long>(a.heads) * V;
  // One token: the read-outs of the old state, the write, the output, for each of the thread's columns.
  auto token = [&](const float (&kr)[KPL], const float (&qr)[KPL], float g, float beta, const float* vj, long long at) {
    float kq[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
    for (int i = 0; i < KPL; ++i) kq[i & 3] = fmaf(kr[i], qr[i], kq[i & 3]);
    float skq = (kq[0] + kq[1]) + (kq[2] + kq[3]);
    float sk[CPT], sq[CPT];
#pragma unroll
    for (int c = 0; c < CPT; ++c) {
      float rk[4] = {0.0f, 0.0f, 0.0f, 0.0f}, rq[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
      for (int i = 0; i < KPL; ++i) {
        rk[i & 3] = fmaf(S[c][i], kr[i], rk[i & 3]);
        rq[i & 3] = fmaf(S[c][i], qr[i], rq[i & 3]);
      }
      sk[c] = (rk[0] + rk[1]) + (rk[2] + rk[3]);
      sq[c] = (rq[0] + rq[1]) + (rq[2] + rq[3]);
    }
#pragma unroll
    for (int o = L >> 1; o > 0; o >>= 1) {
      skq += __shfl_xor_sync(0xffffffffu, skq, o);
#pragma unroll
      for (int c = 0; c < CPT; ++c) {
        sk[c] += __shfl_xor_sync(0xffffffffu, sk[c], o);
        sq[c] += __shfl_xor_sync(0xffffffffu, sq[c], o);
      }
    }
#pragma unroll
    for (int c = 0; c < CPT; ++c) {
      const float u = beta * (vj[c * groups] - g * sk[c]);
#pragma unroll
      for (int i = 0; i < KPL; ++i) S[c][i] = fmaf(kr[i], u, g * S[c][i]);
      if (l == 0 && live[c]) out[at * out_stride + c * groups] = fmaf(u, skq, g * sq[c]);
    }
  };

  if (chunks > 0) {
    issue_qk(0, min(DS_TOKENS, n), ds_smem);
    fetch_rest(0, min(DS_TOKENS, n));
    store_rest(ds_smem);
  }
  for (int chunk = 0; chunk < chunks; ++chunk) {
    const int base = chunk * DS_TOKENS, nt = min(DS_TOKENS, n - base);
    float* stage = ds_smem + (chunk & 1) * stage_floats;
    float* other = ds_smem + ((chunk + 1) & 1) * stage_floats;
    cp_async_wait<0>();
    __syncthreads();             // this portion has landed, and the other buffer is no longer read
    const bool more = chunk + 1 < chunks;
    if (more) {
      issue_qk(base + DS_TOKENS, min(DS_TOKENS, n - base - DS_TOKENS), other);
      fetch_rest(base + DS_TOKENS, min(DS_TOKENS, n - base - DS_TOKENS));
    }
    const float* q_s = stage + l * RUN;
    const float* k_s = stage + DS_TOKENS * DP + l * RUN;
    const float* v_s = stage + 2 * DS_TOKENS * DP + my_group;
    const float* beta_s = stage + 2 * DS_TOKENS * DP + DS_TOKENS * cols;
    const float* decay_s = beta_s + DS_TOKENS;
    // Tokens in pairs: while one token's chain runs on one set of registers, the next token's k and q are
    // fetched into the other set.
    float k0[KPL], q0[KPL], k1[KPL], q1[KPL];
    load_run(k0, k_s);
    load_run(q0, q_s);
    for (int j = 0; j < nt; j += 2) {
      const int j1 = j + 1 < DS_TOKENS ? j + 1 : j, j2 = j + 2 < DS_TOKENS ? j + 2 : j;
      load_run(k1, k_s + j1 * DP);
      load_run(q1, q_s + j1 * DP);
      token(k0, q0, decay_s[j], beta_s[j], v_s + j * cols, base + j);
      if (j + 1 >= nt) break;
      load_run(k0, k_s + j2 * DP);
      load_run(q0, q_s + j2 * DP);
      token(k1, q1, decay_s[j + 1], beta_s[j + 1], v_s + (j + 1) * cols, base + j + 1);
    }
    if (more) store_rest(other);
  }
  cp_async_wait<0>();
#pragma unroll
  for (int c = 0; c < CPT; ++c) {
    if (!a.write_state || !live[c]) continue;
    if (state_vectors) {
#pragma unroll
      for (int i = 0; i < KPL; i += 4)
        if (l * KPL + i < D)
          *reinterpret_cast<float4*>(mine[c] + i) = make_float4(S[c][i], S[c][i + 1], S[c][i + 2], S[c][i + 3]);
    } else {
#pragma unroll
      for (int i = 0; i < KPL; ++i)
        if (l * KPL + i < D) mine[c][i] = S[c][i];
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

template <typename T, int KPL, int L, int CPT>
static int delta_scan_launch(const DeltaScanArgs& a, int rows, cudaStream_t s) {
  constexpr int cols = DS_THREADS / L * CPT;
  const size_t smem = 2 * sizeof(float) * (2 * DS_TOKENS * L * (KPL + 4) + DS_TOKENS * cols + 2 * DS_TOKENS);
  const bool async = a.D % 4 == 0 && reinterpret_cast<uintptr_t>(a.q) % 16 == 0 && reinterpret_cast<uintptr_t>(a.k) % 16 == 0 &&
                     reinterpret_cast<uintptr_t>(a.state) % 16 == 0 && a.slot_stride % 4 == 0;
  auto kernel = async ? delta_scan_kernel<T, KPL, L, CPT, true> : delta_scan_kernel<T, KPL, L, CPT, false>;
  if (smem > 48 * 1024 &&
      cuda_failed(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem))))
    return ERR_CUDA;
  kernel<<<dim3(rows, a.heads, (a.V + cols - 1) / cols), DS_THREADS, smem, s>>>(a);
  return launch_result();
}

template <typename T, int KPL, int L>
static int delta_scan_columns(const DeltaScanArgs& a, int rows, int tokens, cudaStream_t s) {
  // Two columns a thread where requests bring runs of tokens (the chains hide each other's waits) and a head has
  // columns enough; one where a step is single tokens, whose time is the state's bytes.
  const bool runs = tokens >= 4 * rows && a.V >= 2 * (DS_THREADS / L);
  return runs ? delta_scan_launch<T, KPL, L, 2>(a, rows, s) : delta_scan_launch<T, KPL, L, 1>(a, rows, s);
}

template <typename T>
static int delta_scan_dispatch(const DeltaScanArgs& a, int rows, int tokens, cudaStream_t s) {
  // Channels a lane holds and lanes a column: a column spreads over 4 lanes up to 64 channels (two rounds of
  // exchanges a token), over 8 up to 128, 16 up to 256, a whole warp beyond.
  const int D = a.D;
  if (D <= 16) return delta_scan_columns<T, 4, 4>(a, rows, tokens, s);
  if (D <= 32) return delta_scan_columns<T, 8, 4>(a, rows, tokens, s);
  if (D <= 64) return delta_scan_columns<T, 16, 4>(a, rows, tokens, s);
  if (D <= 128) return delta_scan_columns<T, 16, 8>(a, rows, tokens, s);
  if (D <= 256) return delta_scan_columns<T, 16, 16>(a, rows, tokens, s);
  return delta_scan_columns<T, 16, 32>(a, rows, tokens, s);
}

ZB_API int zb_delta_scan(float* out, const float* q, const float* k, const void* v, long long v_stride,
                         const float* beta, const float* decay, float* state, long long slot_stride, const int* slots,
                         const int* row_q_start, const int* row_q_len, int rows, int tokens, int heads,
                         int heads_per_group, int D, int V, int num_slots, int write_state, int dtype, int* status,
                         void* stream) {
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
  return dtype == DTYPE_F32 ? delta_scan_dispatch<float>(a, rows, tokens, s)
                            : delta_scan_dispatch<__nv_bfloat16>(a, rows, tokens, s);
}
