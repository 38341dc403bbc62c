// Softmax attention whose scores are mixed across the heads before the softmax.
//
//   raw_g(i, j)  = (q_g(i) . k(j)) * scale * temp_g            temp: one number per query head, or none
//   raw_g       <- cap * tanh(raw_g / cap)                      a soft cap, or none
//   s_h(i, j)    = sum_g M[h, g] raw_g(i, j)                    M: [heads, heads], or none
//   w_h(i, j)    = exp(s_h(i, j)) / (exp(sink_h) + sum over seen j' of exp(s_h(i, j')))
//   out_h(i)     = sum_j w_h(i, j) v(j)
//
// The sink is a member of the softmax without key or value (a number per head, or none).  What the
// query at position p sees besides j <= p is the mask: everything, the last `size` positions, or the
// keys of its own chunk of `size` positions (chunks counted from position 0 of the sequence).
//
// Because a head's score needs every head's product with the key, a block owns one query token and
// all of its heads: a tile of keys and values of all key/value heads is copied from the pages into
// shared memory once, every (head, key) pair gets its raw score, the scores are mixed, a warp per
// head keeps the running maximum and sum (started at (sink, 1) where there is a sink), and every
// thread keeps R of the token's heads x vdim outputs in registers.  Scores, weights and sums are fp32.
// The key range of a token may be split over several blocks (steps of few tokens); their partial
// (maximum, sum, outputs) are merged by a second kernel, the sink counted once.
//
// q, k and v come as the preparation kernel left them: q in the step's rows, k and v in the pages.
#include "common.cuh"

namespace leone {

constexpr int kMixThreads = 256;

template <typename T> __host__ __device__ inline int padded_row(int d) {
  // elements per shared-memory row so that consecutive rows start an odd number of 32-bit words apart
  if (sizeof(T) == 4) return (d % 2 == 0) ? d + 1 : d;
  int e = (d + 1) / 2 * 2;
  if ((e / 2) % 2 == 0) e += 2;
  return e;
}

// Rows j0 .. j0 + nt - 1 of every key/value head from the pages into shared memory ([head][kt][pitch] elements):
// 16 bytes a load where the rows allow it (the shared rows are only 4-byte aligned, so four stores), else
// element by element.  A key without a valid page is a row of zeros.
template <typename T>
__device__ __forceinline__ void copy_tile(T* dst, int pitch, const T* __restrict__ pool, int d, const int* page_s, int j0,
                                          int nt, int n_kv, int kt, int page_tokens, int tid) {
  constexpr int V = 16 / (int)sizeof(T);
  if (d % V == 0 && (pitch * (int)sizeof(T)) % 4 == 0 && (((uintptr_t)pool) & 15) == 0) {
    const int chunks = d / V;
    for (int i = tid; i < n_kv * nt * chunks; i += kMixThreads) {
      const int c = i % chunks, row = i / chunks;
      const int j = row % nt, g = row / nt;
      const int page = page_s[j];
      uint4 val = make_uint4(0, 0, 0, 0);
      if (page >= 0)
        val = *reinterpret_cast<const uint4*>(pool + (((size_t)page * n_kv + g) * page_tokens + (j0 + j) % page_tokens) * d + c * V);
      uint32_t* out = reinterpret_cast<uint32_t*>(dst + ((size_t)g * kt + j) * pitch + c * V);
      out[0] = val.x;
      out[1] = val.y;
      out[2] = val.z;
      out[3] = val.w;
    }
    return;
  }
  for (int i = tid; i < n_kv * nt * d; i += kMixThreads) {
    const int e = i % d, row = i / d;
    const int j = row % nt, g = row / nt;
    const int page = page_s[j];
    dst[((size_t)g * kt + j) * pitch + e] =
        page < 0 ? from_float<T>(0.f) : pool[(((size_t)page * n_kv + g) * page_tokens + (j0 + j) % page_tokens) * d + e];
  }
}

// mask: 0 causal, 1 window, 2 chunk
template <typename T, int R>
__global__ void __launch_bounds__(kMixThreads)
attention_mixed_heads_kernel(const T* __restrict__ q, int ldq, T* __restrict__ out, int ldo, float* __restrict__ partial,
                             const T* __restrict__ k_pool, const T* __restrict__ v_pool,
                             const int* __restrict__ block_table, int bt_width, const int* __restrict__ seq_of_token,
                             const int* __restrict__ positions, int n_q, int n_kv, int dk, int dv, float scale,
                             const float* __restrict__ temp, float cap, const float* __restrict__ mix,
                             const float* __restrict__ sink, int mask, int mask_size, int page_tokens, int n_pages,
                             int n_seqs, int kt, int splits, int* status) {
  pdl_trigger();
  pdl_wait();
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int t = blockIdx.x, split = blockIdx.y;
  const int dkp = padded_row<T>(dk);
  float* q_s = reinterpret_cast<float*>(smem_raw);          // [n_q][dk], times scale * temp
  float* mix_s = q_s + n_q * dk;                            // [n_q][n_q]
  float* raw_s = mix_s + n_q * n_q;                         // [n_q][kt]
  float* p_s = raw_s + n_q * kt;                            // [n_q][kt]
  float* m_s = p_s + n_q * kt;                              // [n_q] running maximum
  float* l_s = m_s + n_q;                                   // [n_q] running sum
  float* c_s = l_s + n_q;                                   // [n_q] factor on what was summed before
  int* page_s = reinterpret_cast<int*>(c_s + n_q);          // [kt]
  T* k_s = reinterpret_cast<T*>(page_s + kt);               // [n_kv][kt][dkp]
  T* v_s = k_s + (size_t)n_kv * kt * dkp;                   // [n_kv][kt][dv]
  const int s = seq_of_token[t];
  if (s < 0 || s >= n_seqs) {
    if (tid == 0) set_status(status, kBadSequence, t, s);
    return;
  }
  const int p = positions[t];
  int lo = 0;
  if (mask == 1) lo = max(0, p - mask_size + 1);
  else if (mask == 2) lo = (p / mask_size) * mask_size;
  const int group = n_q / n_kv;
  for (int i = tid; i < n_q * dk; i += kMixThreads) {
    const int h = i / dk;
    q_s[i] = to_float<T>(q[(size_t)t * ldq + i]) * (scale * (temp != nullptr ? temp[h] : 1.f));
  }
  for (int i = tid; i < n_q * n_q; i += kMixThreads) mix_s[i] = mix != nullptr ? mix[i] : ((i / n_q == i % n_q) ? 1.f : 0.f);
  for (int h = tid; h < n_q; h += kMixThreads) {
    const bool with_sink = sink != nullptr && split == 0;
    m_s[h] = with_sink ? sink[h] : -INFINITY;
    l_s[h] = with_sink ? 1.f : 0.f;
  }
  float acc[R];
#pragma unroll
  for (int r = 0; r < R; ++r) acc[r] = 0.f;
  const int n_out = n_q * dv;
  const int* table = block_table + (size_t)s * bt_width;
  for (int j0 = lo + split * kt; j0 <= p; j0 += splits * kt) {
    const int nt = min(kt, p + 1 - j0);
    __syncthreads();
    if (tid < nt) {
      const int pos = j0 + tid;
      const int blk = pos / page_tokens;
      const int page = blk < bt_width ? table[blk] : -1;
      if (page < 0 || page >= n_pages) set_status(status, kBadPage, t, page);
      page_s[tid] = (page < 0 || page >= n_pages) ? -1 : page;
    }
    __syncthreads();
    copy_tile<T>(k_s, dkp, k_pool, dk, page_s, j0, nt, n_kv, kt, page_tokens, tid);
    copy_tile<T>(v_s, dv, v_pool, dv, page_s, j0, nt, n_kv, kt, page_tokens, tid);
    __syncthreads();
    for (int i = tid; i < n_q * kt; i += kMixThreads) {
      const int h = i / kt, j = i - h * kt;
      float dot = 0.f;
      if (j < nt) {
        const float* qq = q_s + h * dk;
        const T* kk = k_s + ((size_t)(h / group) * kt + j) * dkp;
        for (int d = 0; d < dk; ++d) dot = fmaf(qq[d], to_float<T>(kk[d]), dot);
        if (cap > 0.f) dot = cap * tanhf(dot / cap);
      }
      raw_s[i] = dot;
    }
    __syncthreads();
    for (int i = tid; i < n_q * kt; i += kMixThreads) {
      const int h = i / kt, j = i - h * kt;
      float v = -INFINITY;
      if (j < nt) {
        v = 0.f;
        const float* row = mix_s + h * n_q;
        for (int g = 0; g < n_q; ++g) v = fmaf(row[g], raw_s[g * kt + j], v);
      }
      p_s[i] = v;
    }
    __syncthreads();
    for (int h = warp; h < n_q; h += kMixThreads / 32) {
      float mx = -INFINITY;
      for (int j = lane; j < kt; j += 32) mx = fmaxf(mx, p_s[h * kt + j]);
      mx = warp_max(mx);
      const float m_old = m_s[h];
      const float m_new = fmaxf(m_old, mx);
      float sum = 0.f;
      for (int j = lane; j < kt; j += 32) {
        const float e = j < nt ? expf(p_s[h * kt + j] - m_new) : 0.f;
        p_s[h * kt + j] = e;
        sum += e;
      }
      sum = warp_sum(sum);
      if (lane == 0) {
        const float c = m_old == -INFINITY ? 0.f : expf(m_old - m_new);
        c_s[h] = c;
        l_s[h] = l_s[h] * c + sum;
        m_s[h] = m_new;
      }
    }
    __syncthreads();
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const int e = tid + r * kMixThreads;
      if (e < n_out) {
        const int h = e / dv, c = e - h * dv;
        const float* pp = p_s + h * kt;
        const T* vv = v_s + (size_t)(h / group) * kt * dv + c;
        float a = acc[r] * c_s[h];
        for (int j = 0; j < nt; ++j) a = fmaf(pp[j], to_float<T>(vv[(size_t)j * dv]), a);
        acc[r] = a;
      }
    }
  }
  __syncthreads();
  if (splits == 1) {
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const int e = tid + r * kMixThreads;
      if (e < n_out) {
        const float l = l_s[e / dv];
        out[(size_t)t * ldo + e] = from_float<T>(l > 0.f ? acc[r] / l : 0.f);
      }
    }
    return;
  }
  // partial: [token][split][n_q * (dv + 2)]: outputs, then maximum and sum per head
  float* mine = partial + ((size_t)t * splits + split) * (size_t)(n_out + 2 * n_q);
#pragma unroll
  for (int r = 0; r < R; ++r) {
    const int e = tid + r * kMixThreads;
    if (e < n_out) mine[e] = acc[r];
  }
  for (int h = tid; h < n_q; h += kMixThreads) {
    mine[n_out + h] = m_s[h];
    mine[n_out + n_q + h] = l_s[h];
  }
}

template <typename T>
__global__ void __launch_bounds__(kMixThreads)
attention_mixed_heads_merge_kernel(const float* __restrict__ partial, T* __restrict__ out, int ldo, int n_q, int dv,
                                   int splits) {
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x, n_out = n_q * dv;
  const size_t per = (size_t)(n_out + 2 * n_q);
  const float* base = partial + (size_t)t * splits * per;
  for (int e = threadIdx.x; e < n_out; e += kMixThreads) {
    const int h = e / dv;
    float m = -INFINITY;
    for (int sp = 0; sp < splits; ++sp) m = fmaxf(m, base[sp * per + n_out + h]);
    float l = 0.f, a = 0.f;
    for (int sp = 0; sp < splits; ++sp) {
      const float ms = base[sp * per + n_out + h];
      const float f = ms == -INFINITY ? 0.f : expf(ms - m);
      l = fmaf(base[sp * per + n_out + n_q + h], f, l);
      a = fmaf(base[sp * per + e], f, a);
    }
    out[(size_t)t * ldo + e] = from_float<T>(l > 0.f ? a / l : 0.f);
  }
}

template <typename T> size_t mixed_heads_smem(int n_q, int n_kv, int dk, int dv, int kt) {
  const size_t floats = (size_t)n_q * (dk + n_q + 2 * kt + 3) + kt;
  return sizeof(float) * floats + sizeof(T) * (size_t)n_kv * kt * (padded_row<T>(dk) + dv);
}

template <typename T>
int launch_mixed_heads(const void* q, int ldq, void* out, int ldo, float* partial, const void* k_pool, const void* v_pool,
                       const int* block_table, int bt_width, const int* seq_of_token, const int* positions, int n_tokens,
                       int n_q, int n_kv, int dk, int dv, float scale, const float* temp, float cap, const float* mix,
                       const float* sink, int mask, int mask_size, int page_tokens, int n_pages, int n_seqs, int splits,
                       int* status, cudaStream_t stream) {
  int kt = 32;
  while (kt > 4 && mixed_heads_smem<T>(n_q, n_kv, dk, dv, kt) > 200 * 1024) kt /= 2;
  const size_t smem = mixed_heads_smem<T>(n_q, n_kv, dk, dv, kt);
  if (smem > 200 * 1024) return kRefusedSize;
  const int per_thread = (n_q * dv + kMixThreads - 1) / kMixThreads;
  const dim3 grid(n_tokens, splits);
#define MIXED(R)                                                                                                       \
  {                                                                                                                    \
    static size_t configured = 0;                                                                                      \
    if (smem > configured) {                                                                                           \
      cudaFuncSetAttribute(attention_mixed_heads_kernel<T, R>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
      configured = smem;                                                                                               \
    }                                                                                                                  \
    const int code = launch_kernel(attention_mixed_heads_kernel<T, R>, grid, dim3(kMixThreads), smem, stream,          \
                                   (const T*)q, ldq, (T*)out, ldo, partial, (const T*)k_pool, (const T*)v_pool,        \
                                   block_table, bt_width, seq_of_token, positions, n_q, n_kv, dk, dv, scale, temp,     \
                                   cap, mix, sink, mask, mask_size, page_tokens, n_pages, n_seqs, kt, splits, status); \
    if (code != 0 || splits == 1) return code;                                                                         \
    return launch_kernel(attention_mixed_heads_merge_kernel<T>, dim3(n_tokens), dim3(kMixThreads), 0, stream,          \
                         (const float*)partial, (T*)out, ldo, n_q, dv, splits);                                        \
  }
  if (per_thread <= 1) MIXED(1)
  if (per_thread <= 2) MIXED(2)
  if (per_thread <= 4) MIXED(4)
  if (per_thread <= 8) MIXED(8)
  if (per_thread <= 16) MIXED(16)
  if (per_thread <= 32) MIXED(32)
#undef MIXED
  return kRefusedSize;
}

}  // namespace leone

using namespace leone;

// q: [n_tokens, ldq] with the heads' queries side by side (n_q * dk); out: [n_tokens, ldo] (n_q * dv).
// temp, mix, sink: fp32, each may be null; cap <= 0: no soft cap.  mask: 0 causal, 1 window, 2 chunk.
// splits > 1: the key tiles of a token are dealt to that many blocks and `partial` holds fp32
// [n_tokens, splits, n_q * (dv + 2)].
extern "C" int leone_attention_mixed_heads(int dtype, const void* q, int ldq, void* out, int ldo, float* partial,
                                           const void* k_pool, const void* v_pool, const int* block_table, int bt_width,
                                           const int* seq_of_token, const int* positions, int n_tokens, int n_q, int n_kv,
                                           int dk, int dv, float scale, const float* temp, float cap, const float* mix,
                                           const float* sink, int mask, int mask_size, int page_tokens, int n_pages,
                                           int n_seqs, int splits, int* status, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (n_q <= 0 || n_kv <= 0 || n_q % n_kv != 0 || dk <= 0 || dv <= 0 || page_tokens <= 0 || splits < 1 || splits > 65535 ||
      (splits > 1 && partial == nullptr) || (mask != 0 && mask_size <= 0) || mask < 0 || mask > 2)
    return kRefusedSize;
  if (dtype == 0)
    return launch_mixed_heads<float>(q, ldq, out, ldo, partial, k_pool, v_pool, block_table, bt_width, seq_of_token,
                                     positions, n_tokens, n_q, n_kv, dk, dv, scale, temp, cap, mix, sink, mask, mask_size,
                                     page_tokens, n_pages, n_seqs, splits, status, stream);
  if (dtype == 1)
    return launch_mixed_heads<__nv_bfloat16>(q, ldq, out, ldo, partial, k_pool, v_pool, block_table, bt_width,
                                             seq_of_token, positions, n_tokens, n_q, n_kv, dk, dv, scale, temp, cap, mix,
                                             sink, mask, mask_size, page_tokens, n_pages, n_seqs, splits, status, stream);
  return kRefusedDtype;
}
