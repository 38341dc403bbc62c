// A short causal convolution over time on every channel, with the last taps - 1 inputs of every
// sequence kept as fixed-size state between steps; and the minGRU recurrence.
//
//   leone_short_conv:        y_t[c] = (add_input & 1 ? x_t[c] : 0) + sum_j w[c, j] x_(t - taps + 1 + j)[c],
//                            then y * sigmoid(y) if add_input & 2,
//                            inputs before a sequence's start are zero; an input before the step's
//                            first token comes from the state
//   leone_short_conv_state:  the state after the step: the last taps - 1 inputs of every sequence
//                            (older rows move up when the step brought fewer than taps - 1 tokens)
//   leone_min_gru:           z = sigmoid(pz + bz), u = px + bx, c = u >= 0 ? u + 1/2 : sigmoid(u),
//                            S_t = (1 - z) S_(t-1) + z c element by element, state fp32 per slot,
//                            out_t = out_scale * S_t * silu(pg)
//   leone_scale_rows:        a[t, :] *= scale * sigmoid(gate[t])  (gate: one fp32 logit per row)
//   leone_add_scaled:        x += scale * y  (fp32)
//
// The state is [slots, taps - 1, channels] fp32, row taps - 2 the newest input.  Weights are fp32
// [channels, taps].  All sums are fp32 in ascending j, so a token's result does not depend on how
// its sequence was cut into steps.  The convolution does not write the state (tokens at a step's
// start still read it); the state kernel runs after it.  In a step where every sequence brings one
// token (update_state) the convolution's thread of (token, channel) is the only reader and writer of
// its state column and moves it on itself.
#include "common.cuh"

namespace leone {

constexpr int kConvThreads = 128;
constexpr int kMaxTaps = 16;

template <typename TI, typename TO>
__global__ void __launch_bounds__(kConvThreads)
short_conv_kernel(const TI* __restrict__ x, int ldx, const float* __restrict__ w, float* state,
                  TO* __restrict__ out, int ldo, const int* __restrict__ q_start, const int* __restrict__ seq_of_token,
                  const int* __restrict__ slot_ids, int channels, int taps, int add_input, int update_state, int n_seqs,
                  int n_slots, int* status) {
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x, c = blockIdx.y * kConvThreads + threadIdx.x;
  if (c >= channels) return;
  const int s = seq_of_token[t];
  if (s < 0 || s >= n_seqs) {
    if (threadIdx.x == 0) set_status(status, kBadSequence, t, s);
    return;
  }
  const int slot = taps > 1 ? slot_ids[s] : 0;      // one tap: no state, no slot
  if (slot < 0 || (taps > 1 && slot >= n_slots)) {
    if (threadIdx.x == 0) set_status(status, kBadSequence, t, slot);
    return;
  }
  const int local = t - q_start[s];                 // tokens of the sequence in this step before this one
  float* st = state + (size_t)slot * (taps - 1) * channels;
  float acc = 0.f;
  for (int j = 0; j < taps; ++j) {
    const int back = taps - 1 - j;
    float v;
    if (back <= local) v = to_float<TI>(x[(size_t)(t - back) * ldx + c]);
    else v = st[(size_t)(taps - 1 + local - back) * channels + c];
    acc = fmaf(w[(size_t)c * taps + j], v, acc);
  }
  if (add_input & 1) acc += to_float<TI>(x[(size_t)t * ldx + c]);
  if (add_input & 2) acc = acc / (1.f + expf(-acc));
  out[(size_t)t * ldo + c] = from_float<TO>(acc);
  if (update_state && taps > 1 && local == 0 && q_start[s + 1] - q_start[s] == 1) {
    for (int r = 0; r + 2 < taps; ++r) st[(size_t)r * channels + c] = st[(size_t)(r + 1) * channels + c];
    st[(size_t)(taps - 2) * channels + c] = to_float<TI>(x[(size_t)t * ldx + c]);
  }
}

// The same for kConvTile consecutive tokens of V neighbouring channels per thread (steps of many
// tokens): where the tile's tokens belong to one sequence, the kConvTile + taps - 1 inputs they read
// are loaded once (V = 4: as 16- or 8-byte vectors) and every output is formed from registers; a tile
// that spans sequences falls back to token-by-token.  kT is the most taps the form takes (its
// register arrays are sized by it).  Per channel the sum is the one of short_conv_kernel, in the same order.
constexpr int kConvTile = 8;

template <typename T, int V> struct ConvVec;
template <> struct ConvVec<float, 1> {
  static __device__ __forceinline__ void load(const float* p, float* v) { v[0] = *p; }
  static __device__ __forceinline__ void store(float* p, const float* v) { *p = v[0]; }
};
template <> struct ConvVec<__nv_bfloat16, 1> {
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, float* v) { v[0] = __bfloat162float(*p); }
  static __device__ __forceinline__ void store(__nv_bfloat16* p, const float* v) { *p = __float2bfloat16_rn(v[0]); }
};
template <> struct ConvVec<float, 4> {
  static __device__ __forceinline__ void load(const float* p, float* v) {
    const float4 r = *reinterpret_cast<const float4*>(p);
    v[0] = r.x, v[1] = r.y, v[2] = r.z, v[3] = r.w;
  }
  static __device__ __forceinline__ void store(float* p, const float* v) {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
  }
};
template <> struct ConvVec<__nv_bfloat16, 4> {
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, float* v) {
    const uint2 r = *reinterpret_cast<const uint2*>(p);
    const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&r.x), b = *reinterpret_cast<const __nv_bfloat162*>(&r.y);
    v[0] = __low2float(a), v[1] = __high2float(a), v[2] = __low2float(b), v[3] = __high2float(b);
  }
  static __device__ __forceinline__ void store(__nv_bfloat16* p, const float* v) {
    const __nv_bfloat162 a = __floats2bfloat162_rn(v[0], v[1]), b = __floats2bfloat162_rn(v[2], v[3]);
    uint2 r;
    r.x = *reinterpret_cast<const uint32_t*>(&a);
    r.y = *reinterpret_cast<const uint32_t*>(&b);
    *reinterpret_cast<uint2*>(p) = r;
  }
};

template <typename TI, typename TO, int V, int kT>
__global__ void __launch_bounds__(kConvThreads)
short_conv_tile_kernel(const TI* __restrict__ x, int ldx, const float* __restrict__ w, const float* __restrict__ state,
                       TO* __restrict__ out, int ldo, const int* __restrict__ q_start,
                       const int* __restrict__ seq_of_token, const int* __restrict__ slot_ids, int n_tokens, int channels,
                       int taps, int add_input, int n_seqs, int n_slots, int* status) {
  pdl_trigger();
  const int t0 = blockIdx.x * kConvTile, c = (blockIdx.y * kConvThreads + threadIdx.x) * V;
  if (c >= channels) return;
  // the weights are not written during a step: fetched before the wait for the kernel ahead
  float wt[kT][V];
#pragma unroll
  for (int j = 0; j < kT; ++j)
#pragma unroll
    for (int e = 0; e < V; ++e) wt[j][e] = j < taps ? w[(size_t)(c + e) * taps + j] : 0.f;
  pdl_wait();
  const int t_end = min(t0 + kConvTile, n_tokens);
  // Input r of the tile is row t0 - (taps - 1) + r of the step.  The rows are asked for before anything is
  // known about the sequence (a row of the step is there to be read whichever sequence it belongs to), so
  // that the look-ups below do not stand in front of them; a row from before the sequence's first token of
  // this step is then replaced by its state row.
  float v[kConvTile + kT - 1][V];
#pragma unroll
  for (int r = 0; r < kConvTile + kT - 1; ++r) {
#pragma unroll
    for (int e = 0; e < V; ++e) v[r][e] = 0.f;
    const int row = t0 - (taps - 1) + r;
    if (r < kConvTile + taps - 1 && row >= 0 && row < t_end) ConvVec<TI, V>::load(x + (size_t)row * ldx + c, v[r]);
  }
  const int s0 = seq_of_token[t0], s1 = seq_of_token[t_end - 1];
  if (s0 == s1 && s0 >= 0 && s0 < n_seqs) {
    const int slot = taps > 1 ? slot_ids[s0] : 0;
    if (slot < 0 || (taps > 1 && slot >= n_slots)) {
      if (threadIdx.x == 0) set_status(status, kBadSequence, t0, slot);
      return;
    }
    const int local0 = t0 - q_start[s0];
    if (local0 < taps - 1) {                             // block-uniform: the tile starts within taps - 1 of the step's start
      const float* st = state + (size_t)slot * (taps - 1) * channels;
#pragma unroll
      for (int r = 0; r < kT - 1; ++r) {
        const int i = local0 - (taps - 1) + r;           // the sequence's token i of this step; negative: state row taps - 1 + i
        if (r < taps - 1 && i < 0) ConvVec<float, V>::load(st + (size_t)(taps - 1 + i) * channels + c, v[r]);
      }
    }
#pragma unroll
    for (int i = 0; i < kConvTile; ++i) {
      if (t0 + i < t_end) {
        float acc[V];
#pragma unroll
        for (int e = 0; e < V; ++e) acc[e] = 0.f;
#pragma unroll
        for (int j = 0; j < kT; ++j)
          if (j < taps) {
#pragma unroll
            for (int e = 0; e < V; ++e) acc[e] = fmaf(wt[j][e], v[i + j][e], acc[e]);
          }
        // the token's own input is v[i + taps - 1]: picked by a static index
        if (add_input & 1) {
#pragma unroll
          for (int j = 0; j < kT; ++j)
            if (j == taps - 1) {
#pragma unroll
              for (int e = 0; e < V; ++e) acc[e] += v[i + j][e];
            }
        }
        if (add_input & 2) {
#pragma unroll
          for (int e = 0; e < V; ++e) acc[e] = acc[e] / (1.f + expf(-acc[e]));
        }
        ConvVec<TO, V>::store(out + (size_t)(t0 + i) * ldo + c, acc);
      }
    }
    return;
  }
  for (int t = t0; t < t_end; ++t) {
    const int s = seq_of_token[t];
    if (s < 0 || s >= n_seqs) {
      if (threadIdx.x == 0) set_status(status, kBadSequence, t, s);
      continue;
    }
    const int slot = taps > 1 ? slot_ids[s] : 0;
    if (slot < 0 || (taps > 1 && slot >= n_slots)) {
      if (threadIdx.x == 0) set_status(status, kBadSequence, t, slot);
      continue;
    }
    const int local = t - q_start[s];
    const float* st = state + (size_t)slot * (taps - 1) * channels;
#pragma unroll
    for (int e = 0; e < V; ++e) {
      float acc = 0.f;
      for (int j = 0; j < taps; ++j) {
        const int back = taps - 1 - j;
        const float u = back <= local ? to_float<TI>(x[(size_t)(t - back) * ldx + c + e])
                                      : st[(size_t)(taps - 1 + local - back) * channels + c + e];
        acc = fmaf(w[(size_t)(c + e) * taps + j], u, acc);
      }
      if (add_input & 1) acc += to_float<TI>(x[(size_t)t * ldx + c + e]);
      if (add_input & 2) acc = acc / (1.f + expf(-acc));
      out[(size_t)(t * (size_t)ldo) + c + e] = from_float<TO>(acc);
    }
  }
}

template <typename TI>
__global__ void __launch_bounds__(kConvThreads)
short_conv_state_kernel(const TI* __restrict__ x, int ldx, float* __restrict__ state, const int* __restrict__ q_start,
                        const int* __restrict__ slot_ids, int channels, int taps, int n_slots, int* status) {
  pdl_trigger();
  pdl_wait();
  const int s = blockIdx.x, c = blockIdx.y * kConvThreads + threadIdx.x;
  if (c >= channels) return;
  const int slot = slot_ids[s];
  if (slot < 0 || slot >= n_slots) {
    if (threadIdx.x == 0) set_status(status, kBadSequence, s, slot);
    return;
  }
  const int first = q_start[s], len = q_start[s + 1] - first, keep = taps - 1;
  float* st = state + (size_t)slot * keep * channels;
  float rows[kMaxTaps];
#pragma unroll
  for (int r = 0; r < kMaxTaps; ++r) {
    if (r < keep) {
      const int local = len - keep + r;             // which of the step's tokens lands in row r
      rows[r] = local >= 0 ? to_float<TI>(x[(size_t)(first + local) * ldx + c]) : st[(size_t)(r + len) * channels + c];
    }
  }
#pragma unroll
  for (int r = 0; r < kMaxTaps; ++r)
    if (r < keep) st[(size_t)r * channels + c] = rows[r];
}

__device__ __forceinline__ float sigmoid_f(float v) { return 1.f / (1.f + expf(-v)); }

// Tokens first .. last - 1 of one channel.  The loads of kGruAhead tokens are issued before their
// arithmetic, so that a thread has that many rows in flight instead of one; the arithmetic per token
// and its order are the same however the tokens are grouped.
constexpr int kGruAhead = 8;

template <typename TP, typename TO, bool kOut, bool kProduct>
__device__ __forceinline__ void min_gru_walk(const TP* __restrict__ proj, int ldp, int z_off, int x_off, int g_off,
                                             float bz, float bx, int c, int first, int last, float& S, float& A,
                                             TO* __restrict__ out, int ldo, float out_scale) {
  for (int t0 = first; t0 < last; t0 += kGruAhead) {
    float pz[kGruAhead], px[kGruAhead], pg[kGruAhead];
#pragma unroll
    for (int i = 0; i < kGruAhead; ++i) {
      const TP* row = proj + (size_t)min(t0 + i, last - 1) * ldp;
      pz[i] = to_float<TP>(row[z_off + c]);
      px[i] = to_float<TP>(row[x_off + c]);
      if (kOut) pg[i] = to_float<TP>(row[g_off + c]);
    }
#pragma unroll
    for (int i = 0; i < kGruAhead; ++i) {
      if (t0 + i < last) {
        const float z = sigmoid_f(pz[i] + bz);
        const float u = px[i] + bx;
        const float cand = u >= 0.f ? u + 0.5f : sigmoid_f(u);
        S = (1.f - z) * S + z * cand;
        if (kProduct) A *= 1.f - z;
        if (kOut) {
          const float g = pg[i];
          out[(size_t)(t0 + i) * ldo + c] = from_float<TO>(out_scale * S * (g * sigmoid_f(g)));
        }
      }
    }
  }
}

// The same walk for four neighbouring channels of a thread (16- or 8-byte loads and stores), four rows in
// flight.  Per channel the arithmetic and its order are those of min_gru_walk.
constexpr int kGruVec = 4, kGruVecAhead = 4;

template <typename TP, typename TO, bool kOut, bool kProduct>
__device__ __forceinline__ void min_gru_walk4(const TP* __restrict__ proj, int ldp, int z_off, int x_off, int g_off,
                                              const float* bz, const float* bx, int c, int first, int last, float* S,
                                              float* A, TO* __restrict__ out, int ldo, float out_scale) {
  for (int t0 = first; t0 < last; t0 += kGruVecAhead) {
    float pz[kGruVecAhead][kGruVec], px[kGruVecAhead][kGruVec], pg[kGruVecAhead][kGruVec];
#pragma unroll
    for (int i = 0; i < kGruVecAhead; ++i) {
      const TP* row = proj + (size_t)min(t0 + i, last - 1) * ldp + c;
      ConvVec<TP, kGruVec>::load(row + z_off, pz[i]);
      ConvVec<TP, kGruVec>::load(row + x_off, px[i]);
      if (kOut) ConvVec<TP, kGruVec>::load(row + g_off, pg[i]);
    }
#pragma unroll
    for (int i = 0; i < kGruVecAhead; ++i) {
      if (t0 + i < last) {
        float o[kGruVec];
#pragma unroll
        for (int e = 0; e < kGruVec; ++e) {
          const float z = sigmoid_f(pz[i][e] + bz[e]);
          const float u = px[i][e] + bx[e];
          const float cand = u >= 0.f ? u + 0.5f : sigmoid_f(u);
          S[e] = (1.f - z) * S[e] + z * cand;
          if (kProduct) A[e] *= 1.f - z;
          if (kOut) {
            const float g = pg[i][e];
            o[e] = out_scale * S[e] * (g * sigmoid_f(g));
          }
        }
        if (kOut) ConvVec<TO, kGruVec>::store(out + (size_t)(t0 + i) * ldo + c, o);
      }
    }
  }
}

template <typename TP, typename TO>
__global__ void __launch_bounds__(kConvThreads)
min_gru_kernel(const TP* __restrict__ proj, int ldp, int z_off, int x_off, int g_off, const float* __restrict__ z_b,
               const float* __restrict__ x_b, float* __restrict__ state, TO* __restrict__ out, int ldo,
               const int* __restrict__ q_start, const int* __restrict__ slot_ids, int width, int n_slots,
               float out_scale, int* status) {
  pdl_trigger();
  pdl_wait();
  const int s = blockIdx.y, c = blockIdx.x * kConvThreads + threadIdx.x;
  if (c >= width) return;
  const int slot = slot_ids[s];
  if (slot < 0 || slot >= n_slots) {
    if (threadIdx.x == 0) set_status(status, kBadSequence, s, slot);
    return;
  }
  const int first = q_start[s], last = q_start[s + 1];
  const float bz = z_b != nullptr ? z_b[c] : 0.f, bx = x_b != nullptr ? x_b[c] : 0.f;
  float S = state[(size_t)slot * width + c], A = 1.f;
  min_gru_walk<TP, TO, true, false>(proj, ldp, z_off, x_off, g_off, bz, bx, c, first, last, S, A, out, ldo, out_scale);
  state[(size_t)slot * width + c] = S;
}

// The recurrence cut into chunks that run side by side.  S_t = a_t S_(t-1) + b_t with a = 1 - z, b = z c:
// pass 1 gives every chunk its (product of a, S at its end from a zero start); pass 2 walks a sequence's
// chunks in order and leaves the state at each chunk's start; pass 3 walks every chunk from there and
// writes the outputs.  The per-token arithmetic of pass 3 is that of the unchunked kernel.
template <typename TP, int V>
__global__ void __launch_bounds__(kConvThreads)
min_gru_chunk_sums_kernel(const TP* __restrict__ proj, int ldp, int z_off, int x_off, const float* __restrict__ z_b,
                          const float* __restrict__ x_b, const int* __restrict__ chunk_first,
                          const int* __restrict__ chunk_last, float* __restrict__ chunk_a, float* __restrict__ chunk_s,
                          int width) {
  pdl_trigger();
  pdl_wait();
  const int k = blockIdx.y, c = (blockIdx.x * kConvThreads + threadIdx.x) * V;
  if (c >= width) return;
  if (V == kGruVec) {
    float bz[kGruVec], bx[kGruVec], A[kGruVec], S[kGruVec];
#pragma unroll
    for (int e = 0; e < kGruVec; ++e) {
      bz[e] = z_b != nullptr ? z_b[c + e] : 0.f;
      bx[e] = x_b != nullptr ? x_b[c + e] : 0.f;
      A[e] = 1.f, S[e] = 0.f;
    }
    min_gru_walk4<TP, float, false, true>(proj, ldp, z_off, x_off, 0, bz, bx, c, chunk_first[k], chunk_last[k], S, A,
                                          nullptr, 0, 0.f);
    ConvVec<float, kGruVec>::store(chunk_a + (size_t)k * width + c, A);
    ConvVec<float, kGruVec>::store(chunk_s + (size_t)k * width + c, S);
    return;
  }
  const float bz = z_b != nullptr ? z_b[c] : 0.f, bx = x_b != nullptr ? x_b[c] : 0.f;
  float A = 1.f, S = 0.f;
  min_gru_walk<TP, float, false, true>(proj, ldp, z_off, x_off, 0, bz, bx, c, chunk_first[k], chunk_last[k], S, A,
                                       nullptr, 0, 0.f);
  chunk_a[(size_t)k * width + c] = A;
  chunk_s[(size_t)k * width + c] = S;
}

// Pass 2 for 32 channels of one sequence by 32 x kPrefixGroups threads: the sequence's chunks are cut
// into kPrefixGroups runs; a thread composes its run's chunks into one (a, b), the runs' starting states
// follow from those in shared memory, and the thread walks its run again from there.  The chain of
// dependent steps is two runs long instead of the whole sequence.
constexpr int kPrefixGroups = 16;

__global__ void __launch_bounds__(32 * kPrefixGroups)
min_gru_chunk_prefix_kernel(const int* __restrict__ seq_chunk_start, const int* __restrict__ slot_ids,
                            const float* __restrict__ chunk_a, float* __restrict__ chunk_s, float* __restrict__ state,
                            int width, int n_slots, int* status) {
  pdl_trigger();
  pdl_wait();
  __shared__ float run_a[kPrefixGroups][32], run_b[kPrefixGroups][32];
  const int s = blockIdx.y, c = blockIdx.x * 32 + threadIdx.x, gy = threadIdx.y;
  const int slot = slot_ids[s];
  if (slot < 0 || slot >= n_slots) {                     // block-uniform
    if (threadIdx.x == 0 && gy == 0) set_status(status, kBadSequence, s, slot);
    return;
  }
  const bool live = c < width;
  const int k_first = seq_chunk_start[s], k_last = seq_chunk_start[s + 1];
  const int per = (k_last - k_first + kPrefixGroups - 1) / kPrefixGroups;
  const int k0 = min(k_first + gy * per, k_last), k1 = min(k0 + per, k_last);
  float A = 1.f, B = 0.f;
  if (live) {
    for (int kk = k0; kk < k1; kk += kGruAhead) {
      float a[kGruAhead], b[kGruAhead];
#pragma unroll
      for (int i = 0; i < kGruAhead; ++i) {
        const int k = min(kk + i, k1 - 1);
        a[i] = chunk_a[(size_t)k * width + c];
        b[i] = chunk_s[(size_t)k * width + c];
      }
#pragma unroll
      for (int i = 0; i < kGruAhead; ++i) {
        if (kk + i < k1) {
          B = a[i] * B + b[i];
          A *= a[i];
        }
      }
    }
  }
  run_a[gy][threadIdx.x] = A;
  run_b[gy][threadIdx.x] = B;
  __syncthreads();
  if (!live) return;
  float S = state[(size_t)slot * width + c];
  for (int g = 0; g < gy; ++g) S = run_a[g][threadIdx.x] * S + run_b[g][threadIdx.x];
  if (gy == kPrefixGroups - 1) state[(size_t)slot * width + c] = A * S + B;      // the state after the step
  for (int kk = k0; kk < k1; kk += kGruAhead) {
    float a[kGruAhead], b[kGruAhead];
#pragma unroll
    for (int i = 0; i < kGruAhead; ++i) {
      const int k = min(kk + i, k1 - 1);
      a[i] = chunk_a[(size_t)k * width + c];
      b[i] = chunk_s[(size_t)k * width + c];
    }
#pragma unroll
    for (int i = 0; i < kGruAhead; ++i) {
      if (kk + i < k1) {
        chunk_s[(size_t)(kk + i) * width + c] = S;         // from here on: the state at the chunk's start
        S = a[i] * S + b[i];
      }
    }
  }
}

template <typename TP, typename TO, int V>
__global__ void __launch_bounds__(kConvThreads)
min_gru_chunk_out_kernel(const TP* __restrict__ proj, int ldp, int z_off, int x_off, int g_off,
                         const float* __restrict__ z_b, const float* __restrict__ x_b, const int* __restrict__ chunk_first,
                         const int* __restrict__ chunk_last, const float* __restrict__ chunk_s, TO* __restrict__ out,
                         int ldo, int width, float out_scale) {
  pdl_trigger();
  pdl_wait();
  const int k = blockIdx.y, c = (blockIdx.x * kConvThreads + threadIdx.x) * V;
  if (c >= width) return;
  if (V == kGruVec) {
    float bz[kGruVec], bx[kGruVec], A[kGruVec], S[kGruVec];
#pragma unroll
    for (int e = 0; e < kGruVec; ++e) {
      bz[e] = z_b != nullptr ? z_b[c + e] : 0.f;
      bx[e] = x_b != nullptr ? x_b[c + e] : 0.f;
      A[e] = 1.f;
    }
    ConvVec<float, kGruVec>::load(chunk_s + (size_t)k * width + c, S);
    min_gru_walk4<TP, TO, true, false>(proj, ldp, z_off, x_off, g_off, bz, bx, c, chunk_first[k], chunk_last[k], S, A,
                                       out, ldo, out_scale);
    return;
  }
  const float bz = z_b != nullptr ? z_b[c] : 0.f, bx = x_b != nullptr ? x_b[c] : 0.f;
  float S = chunk_s[(size_t)k * width + c], A = 1.f;
  min_gru_walk<TP, TO, true, false>(proj, ldp, z_off, x_off, g_off, bz, bx, c, chunk_first[k], chunk_last[k], S, A, out,
                                    ldo, out_scale);
}

template <typename T>
__global__ void __launch_bounds__(256)
scale_rows_kernel(T* __restrict__ a, int lda, int cols, const float* __restrict__ gate, int ldg, float scale) {
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x;
  const float f = gate != nullptr ? scale * sigmoid_f(gate[(size_t)t * ldg]) : scale;
  for (int c = threadIdx.x; c < cols; c += blockDim.x)
    a[(size_t)t * lda + c] = from_float<T>(to_float<T>(a[(size_t)t * lda + c]) * f);
}

__global__ void __launch_bounds__(256)
add_scaled_kernel(float* __restrict__ x, const float* __restrict__ y, long long n, float scale) {
  pdl_trigger();
  pdl_wait();
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
    x[i] = fmaf(scale, y[i], x[i]);
}

}  // namespace leone

using namespace leone;

extern "C" int leone_add_scaled(float* x, const float* y, long long n, float scale, cudaStream_t stream) {
  if (n <= 0) return 0;
  const long long blocks = (n + 255) / 256;
  return launch_kernel(add_scaled_kernel, dim3((unsigned)(blocks < 148 * 8 ? blocks : 148 * 8)), dim3(256), 0, stream, x, y,
                       n, scale);
}

// in_dtype / out_dtype: 0 float32, 1 bfloat16.
// update_state: every sequence of the step brings one token, and the kernel moves the state on too.
extern "C" int leone_short_conv(int in_dtype, int out_dtype, const void* x, int ldx, const float* w, float* state,
                                void* out, int ldo, const int* q_start, const int* seq_of_token, const int* slot_ids,
                                int n_tokens, int channels, int taps, int add_input, int update_state, int n_seqs,
                                int n_slots, int* status, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (channels <= 0 || taps < 1 || taps > kMaxTaps || ldx < channels || ldo < channels) return kRefusedSize;
  if (taps > 1 && state == nullptr) return kRefusedSize;
  const dim3 grid(n_tokens, (channels + kConvThreads - 1) / kConvThreads);
  const bool tiled = n_tokens >= 16 * kConvTile && !update_state;      // a decode step's tokens each belong to another sequence
  // four channels a thread where every row starts on a 16-byte boundary and the taps fit the small form
  const bool vec = tiled && taps <= 4 && channels % 4 == 0 && ldx % 4 == 0 && ldo % 4 == 0 &&
                   (((uintptr_t)x | (uintptr_t)out | (uintptr_t)state) & 15) == 0;
  const dim3 tile_grid((n_tokens + kConvTile - 1) / kConvTile, grid.y);
  const dim3 vec_grid(tile_grid.x, (channels / 4 + kConvThreads - 1) / kConvThreads);
#define LAUNCH(TI, TO)                                                                                              \
  {                                                                                                                 \
    if (vec)                                                                                                        \
      return launch_kernel(short_conv_tile_kernel<TI, TO, 4, 4>, vec_grid, dim3(kConvThreads), 0, stream,           \
                           (const TI*)x, ldx, w, state, (TO*)out, ldo, q_start, seq_of_token, slot_ids, n_tokens,  \
                           channels, taps, add_input, n_seqs, n_slots, status);                                     \
    if (tiled)                                                                                                      \
      return launch_kernel(short_conv_tile_kernel<TI, TO, 1, kMaxTaps>, tile_grid, dim3(kConvThreads), 0, stream,   \
                           (const TI*)x, ldx, w, state, (TO*)out, ldo, q_start, seq_of_token, slot_ids, n_tokens,  \
                           channels, taps, add_input, n_seqs, n_slots, status);                                     \
    return launch_kernel(short_conv_kernel<TI, TO>, grid, dim3(kConvThreads), 0, stream, (const TI*)x, ldx, w,      \
                         state, (TO*)out, ldo, q_start, seq_of_token, slot_ids, channels, taps, add_input,          \
                         update_state, n_seqs, n_slots, status);                                                    \
  }
  if (in_dtype == 0 && out_dtype == 0) LAUNCH(float, float);
  if (in_dtype == 0 && out_dtype == 1) LAUNCH(float, __nv_bfloat16);
  if (in_dtype == 1 && out_dtype == 1) LAUNCH(__nv_bfloat16, __nv_bfloat16);
  if (in_dtype == 1 && out_dtype == 0) LAUNCH(__nv_bfloat16, float);
#undef LAUNCH
  return kRefusedDtype;
}

extern "C" int leone_short_conv_state(int in_dtype, const void* x, int ldx, float* state, const int* q_start,
                                      const int* slot_ids, int n_seqs, int channels, int taps, int n_slots, int* status,
                                      cudaStream_t stream) {
  if (n_seqs <= 0 || taps <= 1) return 0;
  if (channels <= 0 || taps > kMaxTaps || ldx < channels) return kRefusedSize;
  const dim3 grid(n_seqs, (channels + kConvThreads - 1) / kConvThreads);
  if (in_dtype == 0)
    return launch_kernel(short_conv_state_kernel<float>, grid, dim3(kConvThreads), 0, stream, (const float*)x, ldx, state,
                         q_start, slot_ids, channels, taps, n_slots, status);
  if (in_dtype == 1)
    return launch_kernel(short_conv_state_kernel<__nv_bfloat16>, grid, dim3(kConvThreads), 0, stream,
                         (const __nv_bfloat16*)x, ldx, state, q_start, slot_ids, channels, taps, n_slots, status);
  return kRefusedDtype;
}

// n_chunks == 0: one thread walks all of a sequence's tokens.  Otherwise chunk_first / chunk_last (token rows)
// [n_chunks] and seq_chunk_start [n_seqs + 1] describe the cut, and chunk_a / chunk_s are fp32 [n_chunks, width].
extern "C" int leone_min_gru(int proj_dtype, int out_dtype, const void* proj, int ldp, int z_off, int x_off, int g_off,
                             const float* z_b, const float* x_b, float* state, void* out, int ldo, const int* q_start,
                             const int* slot_ids, int n_seqs, int width, int n_slots, float out_scale, int n_chunks,
                             const int* chunk_first, const int* chunk_last, const int* seq_chunk_start, float* chunk_a,
                             float* chunk_s, int* status, cudaStream_t stream) {
  if (n_seqs <= 0) return 0;
  if (width <= 0 || ldp < width || ldo < width || n_seqs > 65535 || n_chunks > 65535) return kRefusedSize;
  const unsigned cols = (width + kConvThreads - 1) / kConvThreads;
  // four channels a thread in the chunk kernels where every vector starts on a 16-byte boundary
  const bool vec = n_chunks > 0 && width % 4 == 0 && ldp % 4 == 0 && ldo % 4 == 0 && z_off % 4 == 0 && x_off % 4 == 0 &&
                   g_off % 4 == 0 && (((uintptr_t)proj | (uintptr_t)out | (uintptr_t)chunk_a | (uintptr_t)chunk_s) & 15) == 0;
  const unsigned vcols = (width / 4 + kConvThreads - 1) / kConvThreads;
#define LAUNCH(TP, TO)                                                                                                  \
  {                                                                                                                     \
    if (n_chunks == 0)                                                                                                  \
      return launch_kernel(min_gru_kernel<TP, TO>, dim3(cols, n_seqs), dim3(kConvThreads), 0, stream, (const TP*)proj,  \
                           ldp, z_off, x_off, g_off, z_b, x_b, state, (TO*)out, ldo, q_start, slot_ids, width, n_slots, \
                           out_scale, status);                                                                          \
    if (vec)                                                                                                            \
      launch_kernel(min_gru_chunk_sums_kernel<TP, 4>, dim3(vcols, n_chunks), dim3(kConvThreads), 0, stream,             \
                    (const TP*)proj, ldp, z_off, x_off, z_b, x_b, chunk_first, chunk_last, chunk_a, chunk_s, width);    \
    else                                                                                                                \
      launch_kernel(min_gru_chunk_sums_kernel<TP, 1>, dim3(cols, n_chunks), dim3(kConvThreads), 0, stream,              \
                    (const TP*)proj, ldp, z_off, x_off, z_b, x_b, chunk_first, chunk_last, chunk_a, chunk_s, width);    \
    launch_kernel(min_gru_chunk_prefix_kernel, dim3((width + 31) / 32, n_seqs), dim3(32, kPrefixGroups), 0, stream,     \
                  seq_chunk_start, slot_ids, (const float*)chunk_a, chunk_s, state, width, n_slots, status);            \
    if (vec)                                                                                                            \
      return launch_kernel(min_gru_chunk_out_kernel<TP, TO, 4>, dim3(vcols, n_chunks), dim3(kConvThreads), 0, stream,   \
                           (const TP*)proj, ldp, z_off, x_off, g_off, z_b, x_b, chunk_first, chunk_last,                \
                           (const float*)chunk_s, (TO*)out, ldo, width, out_scale);                                     \
    return launch_kernel(min_gru_chunk_out_kernel<TP, TO, 1>, dim3(cols, n_chunks), dim3(kConvThreads), 0, stream,      \
                         (const TP*)proj, ldp, z_off, x_off, g_off, z_b, x_b, chunk_first, chunk_last,                  \
                         (const float*)chunk_s, (TO*)out, ldo, width, out_scale);                                       \
  }
  if (proj_dtype == 0 && out_dtype == 0) LAUNCH(float, float);
  if (proj_dtype == 0 && out_dtype == 1) LAUNCH(float, __nv_bfloat16);
  if (proj_dtype == 1 && out_dtype == 1) LAUNCH(__nv_bfloat16, __nv_bfloat16);
#undef LAUNCH
  return kRefusedDtype;
}

extern "C" int leone_scale_rows(int dtype, void* a, int lda, int n_rows, int cols, const float* gate, int ldg,
                                float scale, cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  if (cols <= 0 || lda < cols) return kRefusedSize;
  if (dtype == 0)
    return launch_kernel(scale_rows_kernel<float>, dim3(n_rows), dim3(256), 0, stream, (float*)a, lda, cols, gate, ldg, scale);
  if (dtype == 1)
    return launch_kernel(scale_rows_kernel<__nv_bfloat16>, dim3(n_rows), dim3(256), 0, stream, (__nv_bfloat16*)a, lda,
                         cols, gate, ldg, scale);
  return kRefusedDtype;
}
