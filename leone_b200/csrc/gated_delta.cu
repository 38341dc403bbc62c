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
// token are P-lane shuffles, so a token costs no block-wide barrier.  Tokens are staged 16 at a time, the
// next 16 requested while the current ones are walked.
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
  // two stages of: q [tokens][DIMP], k [tokens][DIMP], v [tokens][COLS], decay [tokens], beta [tokens]
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
  // The raw rows of the next 16 tokens are requested (cp.async, 4 bytes each: no alignment is asked of the
  // rows) before the current 16 are walked, so the walk hides their latency; stage = which half of the
  // doubled buffers holds the current tokens.
  constexpr int kStage = kDeltaTokens * (2 * DIMP + COLS) + 2 * kDeltaTokens;
  auto request = [&](int tb, int stage) {
    const int nt = min(kDeltaTokens, t1 - tb);
    float* qd = smem + stage * kStage;
    float* kd = qd + kDeltaTokens * DIMP;
    float* vd = kd + kDeltaTokens * DIMP;
    for (int i = tid; i < nt * DIMP; i += kDeltaThreads) {
      const int tt = i / DIMP, d = i - tt * DIMP;
      if (d < dim) {
        const float* row = act + (size_t)(tb + tt) * lda + (size_t)kvh * dim + d;
        asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((uint32_t)__cvta_generic_to_shared(qd + i)), "l"(row + q_off));
        asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((uint32_t)__cvta_generic_to_shared(kd + i)), "l"(row + k_off));
      } else {
        qd[i] = 0.f;
        kd[i] = 0.f;
      }
    }
    for (int i = tid; i < nt * COLS; i += kDeltaThreads) {
      const int tt = i / COLS, c = i - tt * COLS;
      if (v0 + c < vdim)
        asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((uint32_t)__cvta_generic_to_shared(vd + i)),
                     "l"(act + (size_t)(tb + tt) * lda + v_off + (size_t)h * vdim + v0 + c));
      else vd[i] = 0.f;
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  // gates of the tokens and unit vectors, in place, once the rows have landed
  auto finish = [&](int tb, int stage) {
    const int nt = min(kDeltaTokens, t1 - tb);
    float* qd = smem + stage * kStage;
    float* kd = qd + kDeltaTokens * DIMP;
    float* gd = kd + kDeltaTokens * DIMP + kDeltaTokens * COLS;
    if (tid < nt) {
      const float* row = raw + (size_t)(tb + tid) * ldr;
      const float z = row[a_off + h] + bias;
      const float sp = z > 20.f ? z : log1pf(expf(z));           // softplus
      gd[tid] = expf(-rate * sp);
      gd[kDeltaTokens + tid] = 1.f / (1.f + expf(-row[b_off + h]));
    }
    for (int tt = warp; tt < nt; tt += kDeltaThreads / 32) {
      float sq = 0.f, sk = 0.f;
      for (int d = lane; d < dim; d += 32) {
        sq = fmaf(qd[tt * DIMP + d], qd[tt * DIMP + d], sq);
        sk = fmaf(kd[tt * DIMP + d], kd[tt * DIMP + d], sk);
      }
      sq = warp_sum(sq);
      sk = warp_sum(sk);
      const float rq = q_scale / sqrtf(sq + 1e-6f), rk = 1.f / sqrtf(sk + 1e-6f);
      for (int d = lane; d < dim; d += 32) {
        qd[tt * DIMP + d] *= rq;
        kd[tt * DIMP + d] *= rk;
      }
    }
  };
  request(t0, 0);
  asm volatile("cp.async.wait_group 0;" ::: "memory");
  __syncthreads();
  finish(t0, 0);
  __syncthreads();
  int stage = 0;
  for (int tb = t0; tb < t1; tb += kDeltaTokens, stage ^= 1) {
    const int nt = min(kDeltaTokens, t1 - tb);
    const bool more = tb + kDeltaTokens < t1;
    if (more) request(tb + kDeltaTokens, stage ^ 1);
    const float* q_c = smem + stage * kStage;
    const float* k_c = q_c + kDeltaTokens * DIMP;
    const float* v_c = k_c + kDeltaTokens * DIMP;
    const float* g_c = v_c + kDeltaTokens * COLS;
    for (int tt = 0; tt < nt; ++tt) {
      const float g = g_c[tt], beta = g_c[kDeltaTokens + tt], vj = v_c[tt * COLS + col_local];
      const float* kk = k_c + tt * DIMP + part;
      const float* qq = q_c + tt * DIMP + part;
      float kv[DPT];
      float r4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int r = 0; r < DPT; ++r) {
        kv[r] = kk[P * r];
        r4[r & 3] = fmaf(S[r], kv[r], r4[r & 3]);
      }
      const float dot = part_sum<P>((r4[0] + r4[1]) + (r4[2] + r4[3]));
      const float u = beta * (vj - g * dot);
      float o4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int r = 0; r < DPT; ++r) {
        S[r] = fmaf(g, S[r], kv[r] * u);
        o4[r & 3] = fmaf(S[r], qq[P * r], o4[r & 3]);
      }
      const float o = part_sum<P>((o4[0] + o4[1]) + (o4[2] + o4[3]));
      if (part == 0 && col < vdim) out[(size_t)(tb + tt) * ldo + (size_t)h * vdim + col] = o;
    }
    if (more) {
      asm volatile("cp.async.wait_group 0;" ::: "memory");
      __syncthreads();
      finish(tb + kDeltaTokens, stage ^ 1);
      __syncthreads();
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
    const size_t smem = 2 * sizeof(float) * (size_t)(kDeltaTokens * (2 * DPT * P + cols) + 2 * kDeltaTokens);             \
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
  // rows dealt to 16 lanes from 33 rows on: a token's cost is the latency of its chain of sums and shuffles,
  // not its multiply-adds (dim 128: 0.48 us a token with 16 lanes a column, 0.59 with 4), and two columns a warp
  // give a prompt of one sequence 8 blocks a head
  if (dim <= 16) DELTA(4, 4)
  if (dim <= 32) DELTA(8, 4)
  if (dim <= 64) DELTA(4, 16)
  if (dim <= 128) DELTA(8, 16)
  if (dim <= 256) DELTA(16, 16)
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
