// The gated delta rule: a recurrence whose state is corrected towards each new value.
//
//   per head, S: [dim, vdim] fp32, per request:
//     S <- g_t S                                  g_t = exp(-exp(A_log_h) softplus(a_t + dt_bias_h))
//     u  = beta_t (v_t - S^T k_t)                 beta_t = sigmoid(b_t)
//     S <- S + k_t u^T
//     o_t = S^T q_t                               (the read-out sees the token's own write)
//
// q and k arrive as activations (after their convolution and silu) of `kv_heads` heads; the kernel makes
// them unit vectors per head, x / sqrt(sum x^2 + 1e-6), and multiplies q by `q_scale`; head h reads
// q/k head h / (heads / kv_heads).  a_t and b_t are raw projections, one per head.  Everything here is
// fp32.  The state is read from and written back to the request's state slot, and the walk is token
// by token in the same order whatever the cut, so a step of one token per sequence (decode) is the
// same kernel.
//
// A block owns (sequence, head, a slice of value columns).  A value column's rows are dealt to P
// lanes (row i belongs to lane part i % P), DPT rows each in registers; the two sums over rows of a
// token are P-lane shuffles, so a token costs no block-wide barrier.  Tokens are staged 16 at a time.
//
// Then `group_gate_norm`: every head's output is divided by its root mean square over vdim,
// multiplied by a weight [vdim] shared by the heads and by act(gate), and stored in the run dtype.
#include "common.cuh"

namespace leone {

constexpr int kDeltaTokens = 16;
constexpr int kDeltaThreads = 128;

template <int P> __device__ __forceinline__ float part_sum(float v) {
#pragma unroll
  for (int o = P / 2; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

template <int DPT, int P>
__global__ void __launch_bounds__(kDeltaThreads)
gated_delta_kernel(const float* __restrict__ act, int lda, int q_off, int k_off, int v_off,
                   const float* __restrict__ raw, int ldr, int a_off, int b_off,
                   const float* __restrict__ a_log, const float* __restrict__ dt_bias, float q_scale,
                   float* __restrict__ out, int ldo, float* state, const int* __restrict__ q_start,
                   const int* __restrict__ slot_ids, int heads, int kv_heads, int dim, int vdim, int n_slots,
                   int* status) {
  pdl_trigger();
  pdl_wait();
  constexpr int DIMP = DPT * P;                 // rows with padding
  constexpr int CW = 32 / P;                    // value columns per warp
  constexpr int COLS = CW * (kDeltaThreads / 32);
  extern __shared__ __align__(16) float smem[];
  float* q_s = smem;                            // [tokens][DIMP]
  float* k_s = q_s + kDeltaTokens * DIMP;       // [tokens][DIMP]
  float* v_s = k_s + kDeltaTokens * DIMP;       // [tokens][COLS]
  float* g_s = v_s + kDeltaTokens * COLS;       // [tokens]
  float* b_s = g_s + kDeltaTokens;              // [tokens]
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int part = lane % P;
  const int col_local = warp * CW + lane / P;
  const int h = blockIdx.y, s = blockIdx.z;
  const int v0 = blockIdx.x * COLS;
  const int col = v0 + col_local;
  const int t0 = q_start[s], t1 = q_start[s + 1];
  if (t0 >= t1) return;
  const int slot = slot_ids[s];
  if (slot < 0 || slot >= n_slots) {
    if (tid == 0) set_status(status, kBadSequence, s, slot);
    return;
  }
  const int kvh = h / (heads / kv_heads);
  float* st = state + ((size_t)slot * heads + h) * (size_t)dim * vdim;
  float S[DPT];
#pragma unroll
  for (int r = 0; r < DPT; ++r) {
    const int i = part + P * r;
    S[r] = (i < dim && col < vdim) ? st[(size_t)i * vdim + col] : 0.f;
  }
  const float rate = expf(a_log[h]), bias = dt_bias[h];
  for (int tb = t0; tb < t1; tb += kDeltaTokens) {
    const int nt = min(kDeltaTokens, t1 - tb);
    __syncthreads();
    for (int i = tid; i < nt * DIMP; i += kDeltaThreads) {
      const int tt = i / DIMP, d = i - tt * DIMP;
      const float* row = act + (size_t)(tb + tt) * lda + (size_t)kvh * dim + d;
      q_s[i] = d < dim ? row[q_off] : 0.f;
      k_s[i] = d < dim ? row[k_off] : 0.f;
    }
    for (int i = tid; i < nt * COLS; i += kDeltaThreads) {
      const int tt = i / COLS, c = i - tt * COLS;
      v_s[i] = v0 + c < vdim ? act[(size_t)(tb + tt) * lda + v_off + (size_t)h * vdim + v0 + c] : 0.f;
    }
    if (tid < nt) {
      const float* row = raw + (size_t)(tb + tid) * ldr;
      const float z = row[a_off + h] + bias;
      const float sp = z > 20.f ? z : log1pf(expf(z));           // softplus
      g_s[tid] = expf(-rate * sp);
      b_s[tid] = 1.f / (1.f + expf(-row[b_off + h]));
    }
    __syncthreads();
    // unit vectors: a warp takes every fourth token
    for (int tt = warp; tt < nt; tt += kDeltaThreads / 32) {
      float sq = 0.f, sk = 0.f;
      for (int d = lane; d < dim; d += 32) {
        sq = fmaf(q_s[tt * DIMP + d], q_s[tt * DIMP + d], sq);
        sk = fmaf(k_s[tt * DIMP + d], k_s[tt * DIMP + d], sk);
      }
      sq = warp_sum(sq);
      sk = warp_sum(sk);
      const float rq = q_scale / sqrtf(sq + 1e-6f), rk = 1.f / sqrtf(sk + 1e-6f);
      for (int d = lane; d < dim; d += 32) {
        q_s[tt * DIMP + d] *= rq;
        k_s[tt * DIMP + d] *= rk;
      }
    }
    __syncthreads();
    for (int tt = 0; tt < nt; ++tt) {
      const float g = g_s[tt], beta = b_s[tt], vj = v_s[tt * COLS + col_local];
      const float* kk = k_s + tt * DIMP + part;
      const float* qq = q_s + tt * DIMP + part;
      float kv[DPT];
      float r0 = 0.f, r1 = 0.f;
#pragma unroll
      for (int r = 0; r < DPT; ++r) {
        kv[r] = kk[P * r];
        if (r & 1) r1 = fmaf(S[r], kv[r], r1);
        else r0 = fmaf(S[r], kv[r], r0);
      }
      const float dot = part_sum<P>(r0 + r1);
      const float u = beta * (vj - g * dot);
      float o0 = 0.f, o1 = 0.f;
#pragma unroll
      for (int r = 0; r < DPT; ++r) {
        S[r] = fmaf(g, S[r], kv[r] * u);
        if (r & 1) o1 = fmaf(S[r], qq[P * r], o1);
        else o0 = fmaf(S[r], qq[P * r], o0);
      }
      const float o = part_sum<P>(o0 + o1);
      if (part == 0 && col < vdim) out[(size_t)(tb + tt) * ldo + (size_t)h * vdim + col] = o;
    }
  }
  if (col < vdim) {
#pragma unroll
    for (int r = 0; r < DPT; ++r) {
      const int i = part + P * r;
      if (i < dim) st[(size_t)i * vdim + col] = S[r];
    }
  }
}

// gate_act: 0 sigmoid, 1 silu.  One block per token, a warp per head in turn.
template <typename T, typename TW>
__global__ void __launch_bounds__(256)
group_gate_norm_kernel(const float* __restrict__ o, int ldo, int heads, int vdim, const TW* __restrict__ w,
                       const float* __restrict__ gate, int ldg, int gate_act, T* __restrict__ out, int ldout, float eps) {
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int h = warp; h < heads; h += 8) {
    const float* row = o + (size_t)t * ldo + (size_t)h * vdim;
    float ss = 0.f;
    for (int c = lane; c < vdim; c += 32) ss = fmaf(row[c], row[c], ss);
    ss = warp_sum(ss);
    const float r = 1.f / sqrtf(ss / (float)vdim + eps);
    for (int c = lane; c < vdim; c += 32) {
      float f = 1.f;
      if (gate != nullptr) {
        const float z = gate[(size_t)t * ldg + (size_t)h * vdim + c];
        const float sg = 1.f / (1.f + expf(-z));
        f = gate_act == 1 ? z * sg : sg;
      }
      out[(size_t)t * ldout + (size_t)h * vdim + c] = from_float<T>(row[c] * r * to_float<TW>(w[c]) * f);
    }
  }
}

}  // namespace leone

using namespace leone;

// act: fp32 [n_tokens, lda] with the activations of q and k (kv_heads x dim each) and v (heads x vdim) at
// the given column offsets; raw: fp32 [n_tokens, ldr] with one a and one b per head at theirs.
// out: fp32 [n_tokens, ldo], head h at columns h * vdim.  state: fp32 [n_slots, heads, dim, vdim].
extern "C" int leone_gated_delta(const float* act, int lda, int q_off, int k_off, int v_off, const float* raw, int ldr,
                                 int a_off, int b_off, const float* a_log, const float* dt_bias, float q_scale,
                                 float* out, int ldo, float* state, const int* q_start, const int* slot_ids,
                                 int n_seqs, int heads, int kv_heads, int dim, int vdim, int n_slots, int* status,
                                 cudaStream_t stream) {
  if (n_seqs <= 0) return 0;
  if (heads <= 0 || kv_heads <= 0 || heads % kv_heads != 0 || dim <= 0 || vdim <= 0 || dim > 512 || heads > 65535 ||
      n_seqs > 65535)
    return kRefusedSize;
#define DELTA(DPT, P)                                                                                                 \
  {                                                                                                                   \
    constexpr int cols = (32 / P) * (kDeltaThreads / 32);                                                             \
    const size_t smem = sizeof(float) * (size_t)(kDeltaTokens * (2 * DPT * P + cols) + 2 * kDeltaTokens);             \
    static bool configured = false;                                                                                   \
    if (!configured && smem > 48 * 1024) {                                                                            \
      cudaFuncSetAttribute(gated_delta_kernel<DPT, P>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);       \
      configured = true;                                                                                              \
    }                                                                                                                 \
    return launch_kernel(gated_delta_kernel<DPT, P>, dim3((vdim + cols - 1) / cols, heads, n_seqs),                   \
                         dim3(kDeltaThreads), smem, stream, act, lda, q_off, k_off, v_off, raw, ldr, a_off, b_off,    \
                         a_log, dt_bias, q_scale, out, ldo, state, q_start, slot_ids, heads, kv_heads, dim, vdim,     \
                         n_slots, status);                                                                            \
  }
  if (dim <= 16) DELTA(4, 4)
  if (dim <= 32) DELTA(8, 4)
  if (dim <= 64) DELTA(16, 4)
  if (dim <= 128) DELTA(32, 4)
  if (dim <= 256) DELTA(64, 4)
  DELTA(16, 32)
#undef DELTA
}

// out[t, h, c] = o[t, h, c] / sqrt(mean_c o[t, h, :]^2 + eps) * w[c] * act(gate[t, h, c]); o and gate fp32
// (gate may be null), out in `dtype`, w in `w_dtype`.  gate_act: 0 sigmoid, 1 silu.
extern "C" int leone_group_gate_norm(int dtype, const float* o, int ldo, int n_tokens, int heads, int vdim, const void* w,
                                     int w_dtype, const float* gate, int ldg, int gate_act, void* out, int ldout,
                                     float eps, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (heads <= 0 || vdim <= 0) return kRefusedSize;
#define GGN(T, TW)                                                                                                  \
  return launch_kernel(group_gate_norm_kernel<T, TW>, dim3(n_tokens), dim3(256), 0, stream, o, ldo, heads, vdim,    \
                       (const TW*)w, gate, ldg, gate_act, (T*)out, ldout, eps)
  if (dtype == 0 && w_dtype == 0) GGN(float, float);
  if (dtype == 1 && w_dtype == 0) GGN(__nv_bfloat16, float);
  if (dtype == 1 && w_dtype == 1) GGN(__nv_bfloat16, __nv_bfloat16);
  if (dtype == 0 && w_dtype == 1) GGN(float, __nv_bfloat16);
#undef GGN
  return kRefusedDtype;
}
