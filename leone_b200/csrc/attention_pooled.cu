// Grouped-query attention over a sliding window of cached keys plus, for everything before the window,
// one mean key and mean value per block of `pool` positions; with the step's preparation (a short
// convolution on the projected q, k and v, rotation, a unit RMS norm per head, cache write).
//
//   the query at position p sees the keys j with 0 <= p - j < window, and every block b of positions
//   b pool .. b pool + pool - 1 that lies wholly before the window: b pool + pool - 1 <= p - window, i.e.
//   the first floor((p - window + 1) / pool) blocks.  A block's key (value) is the mean of its pool cached
//   keys (values).  Tokens and blocks share one softmax.  s = (q . k) * scale, kv_head = head / (n_q / n_kv).
//
// Two caches: the token rows in pages of page_tokens positions (given back once window + pool positions
// lie behind them), and the block means in pages found through a block table of the same kind, where the
// page of a block's last position e holds its row at (e % page_tokens) / pool; a page has pool_rows rows.
//
// leone_attention_pooled_prepare (a block per token, fp32 throughout): row = [q heads x dk | k heads x dk |
// v heads x dv] of the projection (fp32 or bfloat16); an optional causal convolution over time on every
// column (weights fp32 [cols, taps], inputs before the step from the state [slots, taps - 1, cols], see
// short_conv.cu; the state is advanced by leone_short_conv_state afterwards); the rotation of the first
// rot_dims elements of every q and k head by position * freq[pair] with cos and sin times `magnitude`
// (pair i = elements (i, i + rot_dims/2), or (2i, 2i + 1) with `adjacent`); then, with unit_norm, every q
// and k head divided by its root mean square (eps inside the root); q to q_out, k and v into their pages.
//
// leone_attention_pool_blocks (a block per (token, kv head)): a token whose position ends a block writes
// the block's mean key and value (fp32 sums over the rows as the cache holds them: every eighth row in
// ascending position by each of eight warps, then the eight sums in order).
//
// leone_attention_pooled: a block per (token, head); scores and weights fp32, online over tiles of 128
// members (blocks first, then tokens, ascending).  A row depends on its own sequence only.
#include "common.cuh"

namespace leone {

constexpr int kPoolPrepThreads = 256;
constexpr int kPrepTaps = 4, kPrepCols = 4;      // the convolution's unrolled form: taps it takes, columns a thread has in flight

template <typename TP, typename T>
__global__ void __launch_bounds__(kPoolPrepThreads)
attention_pooled_prepare_kernel(const TP* __restrict__ proj, int ldp, int n_q, int n_kv, int dk, int dv,
                                const float* __restrict__ conv_w, int taps, float* conv_state, int update_state,
                                const float* __restrict__ freqs, int rot_dims, int adjacent, float magnitude,
                                int unit_norm, float eps, T* __restrict__ q_out, int ldq,
                                const int* __restrict__ positions, const int* __restrict__ seq_of_token,
                                const int* __restrict__ q_start, const int* __restrict__ slot_ids, int n_slots,
                                const int* __restrict__ block_table, int table_width, int n_seqs,
                                T* __restrict__ k_pool, T* __restrict__ v_pool, int num_pages, int page_tokens,
                                int* status) {
  pdl_trigger();
  pdl_wait();
  extern __shared__ __align__(16) float smem[];
  const int heads = n_q + n_kv;
  const int qk = heads * dk, cols = qk + n_kv * dv;
  float* buf = smem;                    // [cols] the token's row after the convolution
  float* head_f = buf + cols;           // [heads] the heads' norm factors
  float* cs = head_f + heads;           // [rot_dims] cos, sin per pair (times the magnitude)
  const int t = blockIdx.x, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, warps = kPoolPrepThreads / 32;
  // A token's heads do not depend on one another: gridDim.y blocks share them (a step of few tokens has
  // few blocks otherwise).  The units are the q heads, the k heads and the v heads in the order of the
  // row's columns; this block takes units u_lo .. u_hi - 1, that is columns c_lo .. c_hi - 1 and, of the
  // heads that are rotated and normed, h_lo .. h_hi - 1.
  const int units = heads + n_kv, per = (units + gridDim.y - 1) / gridDim.y;
  const int u_lo = blockIdx.y * per, u_hi = min(units, u_lo + per);
  if (u_lo >= units) return;
  const int c_lo = u_lo <= heads ? u_lo * dk : qk + (u_lo - heads) * dv;
  const int c_hi = u_hi <= heads ? u_hi * dk : qk + (u_hi - heads) * dv;
  const int h_lo = min(u_lo, heads), h_hi = min(u_hi, heads);
  const int pos = positions[t], s = seq_of_token[t];
  if (pos < 0 || s < 0 || s >= n_seqs) {
    if (tid == 0) set_status(status, pos < 0 ? kBadPosition : kBadSequence, t, pos < 0 ? pos : s);
    return;
  }
  const TP* row = proj + (size_t)t * ldp;
  if (taps > 1) {
    const int slot = slot_ids[s];
    if (slot < 0 || slot >= n_slots) {
      if (tid == 0) set_status(status, kBadSequence, t, slot);
      return;
    }
    const int local = t - q_start[s];
    float* st = conv_state + (size_t)slot * (taps - 1) * cols;
    // a step in which every sequence brings one token: the thread that reads a state column also moves it on
    const bool move_on = update_state && local == 0 && q_start[s + 1] - q_start[s] == 1;
    if (taps <= kPrepTaps) {
      // up to four taps: the inputs and weights of four columns a thread are asked for together, then the
      // sums are formed (in ascending j, as below)
      for (int c0 = c_lo + tid; c0 < c_hi; c0 += kPoolPrepThreads * kPrepCols) {
        float v[kPrepCols][kPrepTaps], w[kPrepCols][kPrepTaps];
#pragma unroll
        for (int u = 0; u < kPrepCols; ++u) {
          const int c = min(c0 + u * kPoolPrepThreads, c_hi - 1);
#pragma unroll
          for (int j = 0; j < kPrepTaps; ++j) {
            v[u][j] = 0.f, w[u][j] = 0.f;
            if (j < taps) {
              const int back = taps - 1 - j;
              v[u][j] = back <= local ? to_float<TP>(proj[(size_t)(t - back) * ldp + c])
                                      : st[(size_t)(taps - 1 + local - back) * cols + c];
              w[u][j] = conv_w[(size_t)c * taps + j];
            }
          }
        }
#pragma unroll
        for (int u = 0; u < kPrepCols; ++u) {
          const int c = c0 + u * kPoolPrepThreads;
          if (c < c_hi) {
            float acc = 0.f;
#pragma unroll
            for (int j = 0; j < kPrepTaps; ++j)
              if (j < taps) acc = fmaf(w[u][j], v[u][j], acc);
            buf[c] = acc;
            if (move_on) {                               // v[u][1 .. taps - 1]: the state's rows 1 .. and the token's own input
#pragma unroll
              for (int j = 1; j < kPrepTaps; ++j)
                if (j < taps) st[(size_t)(j - 1) * cols + c] = v[u][j];
            }
          }
        }
      }
    } else {
      for (int c = c_lo + tid; c < c_hi; c += kPoolPrepThreads) {
        float acc = 0.f;
        for (int j = 0; j < taps; ++j) {
          const int back = taps - 1 - j;
          const float v = back <= local ? to_float<TP>(proj[(size_t)(t - back) * ldp + c])
                                        : st[(size_t)(taps - 1 + local - back) * cols + c];
          acc = fmaf(conv_w[(size_t)c * taps + j], v, acc);
        }
        buf[c] = acc;
        if (move_on) {
          for (int r = 0; r + 2 < taps; ++r) st[(size_t)r * cols + c] = st[(size_t)(r + 1) * cols + c];
          st[(size_t)(taps - 2) * cols + c] = to_float<TP>(row[c]);
        }
      }
    }
  } else if (taps == 1) {
    for (int c = c_lo + tid; c < c_hi; c += kPoolPrepThreads) buf[c] = conv_w[c] * to_float<TP>(row[c]);
  } else {
    for (int c = c_lo + tid; c < c_hi; c += kPoolPrepThreads) buf[c] = to_float<TP>(row[c]);
  }
  const int half = rot_dims >> 1;
  for (int i = tid; i < (h_lo < h_hi ? half : 0); i += kPoolPrepThreads) {
    const float angle = (float)pos * freqs[i];
    float sn, co;
    sincosf(angle, &sn, &co);
    cs[2 * i] = co * magnitude;
    cs[2 * i + 1] = sn * magnitude;
  }
  __syncthreads();
  // rotation: every thread forms both members of its pairs, so nothing is read after it was written
  for (int i = h_lo * half + tid; i < h_hi * half; i += kPoolPrepThreads) {
    const int h = i / half, pair = i - h * half;
    const int ia = h * dk + (adjacent ? 2 * pair : pair), ib = h * dk + (adjacent ? 2 * pair + 1 : pair + half);
    const float a = buf[ia], b = buf[ib], co = cs[2 * pair], sn = cs[2 * pair + 1];
    buf[ia] = a * co - b * sn;
    buf[ib] = b * co + a * sn;
  }
  __syncthreads();
  for (int h = h_lo + warp; h < h_hi; h += warps) {
    float f = 1.f;
    if (unit_norm) {
      float ss = 0.f;
      for (int c = lane; c < dk; c += 32) ss = fmaf(buf[h * dk + c], buf[h * dk + c], ss);
      ss = warp_sum(ss);
      f = 1.f / sqrtf(ss / (float)dk + eps);
    }
    if (lane == 0) head_f[h] = f;
  }
  __syncthreads();
  long long key_at = -1, value_at = -1;
  if (k_pool != nullptr) {
    const int blk = pos / page_tokens;
    const int page = blk < table_width ? block_table[(size_t)s * table_width + blk] : -1;
    if (page < 0 || page >= num_pages) {
      if (tid == 0) set_status(status, kBadPage, t, page, pos);
      return;
    }
    const long long at = (long long)page * n_kv * page_tokens + (pos % page_tokens);
    key_at = at * dk;
    value_at = at * dv;
  }
  for (int c = c_lo + tid; c < min(c_hi, qk); c += kPoolPrepThreads) {
    const int h = c / dk, e = c - h * dk;
    const T o = from_float<T>(buf[c] * head_f[h]);
    if (h < n_q) q_out[(size_t)t * ldq + c] = o;
    else if (key_at >= 0) k_pool[key_at + (long long)(h - n_q) * page_tokens * dk + e] = o;
  }
  if (value_at >= 0) {
    for (int c = max(c_lo, qk) - qk + tid; c < max(c_hi, qk) - qk; c += kPoolPrepThreads) {
      const int h = c / dv, e = c - h * dv;
      v_pool[value_at + (long long)h * page_tokens * dv + e] = from_float<T>(buf[qk + c]);
    }
  }
}

constexpr int kBlockMeanThreads = 256, kBlockMeanWarps = kBlockMeanThreads / 32, kBlockMeanSlab = 256;
constexpr int kBlockMeanAhead = 8;     // rows of a warp whose loads are issued before their sums

// A thread block looks through `scan` tokens of the step for those that end a pooled block (one in
// `pool`).  For such a token its eight warps take every eighth row of the pooled block each, lanes over
// columns (in slabs of kBlockMeanSlab); the warps' sums meet in shared memory in ascending order.  A warp
// finds the pages of its rows with one look-up per lane and has the loads of kBlockMeanAhead rows in
// flight at a time; the sums are formed in ascending position whatever the grouping.
template <typename T>
__global__ void __launch_bounds__(kBlockMeanThreads)
attention_pool_blocks_kernel(const T* __restrict__ k_pool, const T* __restrict__ v_pool,
                             const int* __restrict__ block_table, int table_width, int num_pages, int page_tokens,
                             T* __restrict__ kb_pool, T* __restrict__ vb_pool, const int* __restrict__ pool_table,
                             int pool_table_width, int pool_pages, int pool_rows, const int* __restrict__ positions,
                             const int* __restrict__ seq_of_token, int n_tokens, int scan, int n_seqs, int n_kv, int dk,
                             int dv, int pool, int* status) {
  pdl_trigger();
  pdl_wait();
  __shared__ float part[kBlockMeanWarps][kBlockMeanSlab];
  __shared__ int bad;
  const int g = blockIdx.y, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int t_end = min((int)(blockIdx.x + 1) * scan, n_tokens);
  for (int t = blockIdx.x * scan; t < t_end; ++t) {          // every branch on t, pos and s is block-uniform
    const int pos = positions[t], s = seq_of_token[t];
    if (pos < 0 || s < 0 || s >= n_seqs) continue;           // the preparation reported it
    if ((pos + 1) % pool != 0) continue;                     // this token ends no block
    const int blk = pos / page_tokens;
    const int dst_page = blk < pool_table_width ? pool_table[(size_t)s * pool_table_width + blk] : -1;
    if (dst_page < 0 || dst_page >= pool_pages) {
      if (tid == 0) set_status(status, kBadPage, t, dst_page, pos);
      continue;
    }
    if (tid == 0) bad = 0;
    __syncthreads();
    const long long dst = ((long long)dst_page * n_kv + g) * pool_rows + (pos % page_tokens) / pool;
    const int first = pos - pool + 1, width = dk + dv;
    const int n_w = pool > warp ? (pool - warp + kBlockMeanWarps - 1) / kBlockMeanWarps : 0;    // rows of this warp
    for (int c0 = 0; c0 < width; c0 += kBlockMeanSlab) {
      const int cn = min(kBlockMeanSlab, width - c0);
      float sum[kBlockMeanSlab / 32];
#pragma unroll
      for (int i = 0; i < kBlockMeanSlab / 32; ++i) sum[i] = 0.f;
      for (int i0 = 0; i0 < n_w; i0 += 32) {
        // lane l: where row i0 + l of this warp (position first + warp + 8 (i0 + l)) lies in the token pools
        long long my_at = -1;
        if (i0 + lane < n_w) {
          const int j = first + warp + kBlockMeanWarps * (i0 + lane);
          const int b = j / page_tokens;
          const int page = b < table_width ? block_table[(size_t)s * table_width + b] : -1;
          if (page < 0 || page >= num_pages) {
            set_status(status, kBadPage, t, page, j);
            bad = 1;
          } else {
            my_at = ((long long)page * n_kv + g) * page_tokens + (j % page_tokens);
          }
        }
        const int n_here = min(32, n_w - i0);
        for (int r0 = 0; r0 < n_here; r0 += kBlockMeanAhead) {
          float val[kBlockMeanAhead][kBlockMeanSlab / 32];
#pragma unroll
          for (int u = 0; u < kBlockMeanAhead; ++u) {
            const long long at = __shfl_sync(0xffffffffu, my_at, min(r0 + u, n_here - 1));
            const bool use = r0 + u < n_here && at >= 0;
#pragma unroll
            for (int i = 0; i < kBlockMeanSlab / 32; ++i) {
              const int c = c0 + lane + 32 * i;
              val[u][i] = 0.f;
              if (use && lane + 32 * i < cn)
                val[u][i] = c < dk ? to_float<T>(k_pool[at * dk + c]) : to_float<T>(v_pool[at * dv + (c - dk)]);
            }
          }
#pragma unroll
          for (int u = 0; u < kBlockMeanAhead; ++u)
#pragma unroll
            for (int i = 0; i < kBlockMeanSlab / 32; ++i) sum[i] += val[u][i];     // a row past the end adds 0
        }
      }
#pragma unroll
      for (int i = 0; i < kBlockMeanSlab / 32; ++i)
        if (lane + 32 * i < cn) part[warp][lane + 32 * i] = sum[i];
      __syncthreads();
      if (!bad) {
        for (int cc = tid; cc < cn; cc += kBlockMeanThreads) {
          float total = 0.f;
#pragma unroll
          for (int w = 0; w < kBlockMeanWarps; ++w) total += part[w][cc];
          const int c = c0 + cc;
          if (c < dk) kb_pool[dst * dk + c] = from_float<T>(total / (float)pool);
          else vb_pool[dst * dv + (c - dk)] = from_float<T>(total / (float)pool);
        }
      }
      __syncthreads();
    }
  }
}

constexpr int kPooledThreads = 128;
constexpr int kPooledAcc = 8;          // value width <= 1024

template <typename T>
__global__ void __launch_bounds__(kPooledThreads)
attention_pooled_kernel(const T* __restrict__ q, int ldq, T* __restrict__ out, int out_stride,
                        const T* __restrict__ k_pool, const T* __restrict__ v_pool,
                        const int* __restrict__ block_table, int table_width, int num_pages, int page_tokens,
                        const T* __restrict__ kb_pool, const T* __restrict__ vb_pool,
                        const int* __restrict__ pool_table, int pool_table_width, int pool_pages, int pool_rows,
                        const int* __restrict__ seq_of_token, const int* __restrict__ positions, int n_q, int n_kv,
                        int dk, int dv, float scale, int window, int pool, float out_scale, int n_seqs, int* status) {
  pdl_trigger();
  pdl_wait();
  extern __shared__ __align__(16) float smem[];
  const T** krow_s = (const T**)smem;                               // [128] the member's key row
  const T** vrow_s = krow_s + kPooledThreads;                       // [128] its value row (null: not seen)
  float* p_s = (float*)(vrow_s + kPooledThreads);                   // [128]
  float* q_s = p_s + kPooledThreads;                                // [dk]
  __shared__ float scratch[33];
  __shared__ int bad;

  const int t = blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
  const int pos = positions[t], s = seq_of_token[t];
  const int kvh = h / (n_q / n_kv);
  T* dst = out + (size_t)t * out_stride + (size_t)h * dv;
  if (tid == 0) bad = 0;
  if (s < 0 || s >= n_seqs || pos < 0) {
    if (tid == 0) set_status(status, s < 0 || s >= n_seqs ? kBadSequence : kBadPosition, t, s < 0 || s >= n_seqs ? s : pos);
    for (int c = tid; c < dv; c += kPooledThreads) dst[c] = from_float<T>(0.f);
    return;
  }
  const T* qr = q + (size_t)t * ldq + (size_t)h * dk;
  for (int c = tid; c < dk; c += kPooledThreads) q_s[c] = to_float<T>(qr[c]);
  __syncthreads();

  const int lo = max(0, pos - window + 1);
  const int n_blocks = pool > 0 && pos - window + 1 >= pool ? (pos - window + 1) / pool : 0;
  const int members = n_blocks + (pos - lo + 1);
  float m_run = -INFINITY, l_run = 0.f;
  float acc[kPooledAcc];
#pragma unroll
  for (int i = 0; i < kPooledAcc; ++i) acc[i] = 0.f;

  for (int i0 = 0; i0 < members; i0 += kPooledThreads) {
    const int i = i0 + tid;
    float score = -INFINITY;
    const T* krow = nullptr;
    const T* vrow = nullptr;
    if (i < members) {
      if (i < n_blocks) {
        const int e = i * pool + pool - 1;
        const int blk = e / page_tokens;
        const int page = blk < pool_table_width ? pool_table[(size_t)s * pool_table_width + blk] : -1;
        if (page < 0 || page >= pool_pages) {
          set_status(status, kBadPage, t, page, e);
          bad = 1;
        } else {
          const long long at = ((long long)page * n_kv + kvh) * pool_rows + (e % page_tokens) / pool;
          krow = kb_pool + at * dk;
          vrow = vb_pool + at * dv;
        }
      } else {
        const int j = lo + (i - n_blocks);
        const int blk = j / page_tokens;
        const int page = blk < table_width ? block_table[(size_t)s * table_width + blk] : -1;
        if (page < 0 || page >= num_pages) {
          set_status(status, kBadPage, t, page, j);
          bad = 1;
        } else {
          const long long at = ((long long)page * n_kv + kvh) * page_tokens + (j % page_tokens);
          krow = k_pool + at * dk;
          vrow = v_pool + at * dv;
        }
      }
      if (krow != nullptr) {
        float dot = 0.f;
        for (int c = 0; c < dk; ++c) dot = fmaf(q_s[c], to_float<T>(krow[c]), dot);
        score = dot * scale;
      }
    }
    vrow_s[tid] = krow != nullptr ? vrow : nullptr;
    const float tile_max = block_max(score, scratch);
    const float m_new = fmaxf(m_run, tile_max);
    const float p = krow != nullptr ? expf(score - m_new) : 0.f;
    p_s[tid] = p;
    const float tile_sum = block_sum(p, scratch);       // also orders the shared writes before the reads
    const float alpha = m_run == -INFINITY ? 0.f : expf(m_run - m_new);
    l_run = l_run * alpha + tile_sum;
    m_run = m_new;
    const int count = min(kPooledThreads, members - i0);
#pragma unroll
    for (int a = 0; a < kPooledAcc; ++a) {
      const int c = tid + a * kPooledThreads;
      if (c < dv) {
        float v = acc[a] * alpha;
        for (int jj = 0; jj < count; ++jj) {
          const T* r = vrow_s[jj];
          if (r != nullptr) v = fmaf(p_s[jj], to_float<T>(r[c]), v);
        }
        acc[a] = v;
      }
    }
    __syncthreads();
  }
  float inv = l_run > 0.f ? out_scale / l_run : 0.f;
  if (bad) inv = 0.f;
#pragma unroll
  for (int a = 0; a < kPooledAcc; ++a) {
    const int c = tid + a * kPooledThreads;
    if (c < dv) dst[c] = from_float<T>(acc[a] * inv);
  }
}

}  // namespace leone

using namespace leone;

// proj_dtype: dtype of the projection rows; dtype: of q_out and the pages.  conv_w null or taps 0: no
// convolution.  freqs null: no rotation.  k_pool null: nothing is written into pages.
extern "C" int leone_attention_pooled_prepare(int proj_dtype, int dtype, const void* proj, int ldp, int n_tokens, int n_q,
                                              int n_kv, int dk, int dv, const float* conv_w, int taps,
                                              float* conv_state, int update_state, const float* freqs, int rot_dims, int adjacent,
                                              float magnitude, int unit_norm, float eps, void* q_out, int ldq,
                                              const int* positions, const int* seq_of_token, const int* q_start,
                                              const int* slot_ids, int n_slots, const int* block_table, int table_width,
                                              int n_seqs, void* k_pool, void* v_pool, int num_pages, int page_tokens,
                                              int* status, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (dk <= 0 || dv <= 0 || n_q <= 0 || n_kv <= 0) return kRefusedSize;
  if (conv_w == nullptr) taps = 0;
  if (taps < 0 || taps > 16 || (taps > 1 && conv_state == nullptr)) return kRefusedSize;
  if (freqs == nullptr) rot_dims = 0;
  if (rot_dims < 0 || rot_dims > dk || (rot_dims & 1)) return kRefusedSize;
  if (k_pool != nullptr && (v_pool == nullptr || page_tokens <= 0 || table_width <= 0)) return kRefusedSize;
  const int cols = (n_q + n_kv) * dk + n_kv * dv;
  if (ldp < cols || ldq < n_q * dk) return kRefusedSize;
  const size_t smem = ((size_t)cols + (n_q + n_kv) + rot_dims + 2) * sizeof(float);
  if (smem > 200 * 1024) return kRefusedSize;
  // a step of few tokens: the heads of a token are shared out over blocks until the SMs have two blocks each
  const int units = n_q + 2 * n_kv;
  const int parts = n_tokens >= 296 ? 1 : min(units, max(1, 296 / n_tokens));
#define LAUNCH(TP, T)                                                                                                 \
  {                                                                                                                   \
    if (smem > 48 * 1024)                                                                                             \
      cudaFuncSetAttribute(attention_pooled_prepare_kernel<TP, T>, cudaFuncAttributeMaxDynamicSharedMemorySize,       \
                           (int)smem);                                                                                \
    return launch_kernel(attention_pooled_prepare_kernel<TP, T>, dim3(n_tokens, parts), dim3(kPoolPrepThreads), smem, stream, \
                         (const TP*)proj, ldp, n_q, n_kv, dk, dv, conv_w, taps, conv_state, update_state, freqs, rot_dims, adjacent, \
                         magnitude, unit_norm, eps, (T*)q_out, ldq, positions, seq_of_token, q_start, slot_ids,       \
                         n_slots, block_table, table_width, n_seqs, (T*)k_pool, (T*)v_pool, num_pages, page_tokens,   \
                         status);                                                                                     \
  }
  if (proj_dtype == 0 && dtype == 0) LAUNCH(float, float);
  if (proj_dtype == 0 && dtype == 1) LAUNCH(float, __nv_bfloat16);
  if (proj_dtype == 1 && dtype == 1) LAUNCH(__nv_bfloat16, __nv_bfloat16);
#undef LAUNCH
  return kRefusedDtype;
}

extern "C" int leone_attention_pool_blocks(int dtype, const void* k_pool, const void* v_pool, const int* block_table,
                                           int table_width, int num_pages, int page_tokens, void* kb_pool,
                                           void* vb_pool, const int* pool_table, int pool_table_width, int pool_pages,
                                           int pool_rows, const int* positions, const int* seq_of_token, int n_tokens,
                                           int n_seqs, int n_kv, int dk, int dv, int pool, int* status,
                                           cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (dk <= 0 || dv <= 0 || n_kv <= 0 || n_kv > 65535 || pool <= 0 || page_tokens <= 0 || pool_rows <= 0 ||
      pool_rows < (page_tokens + pool - 1) / pool)
    return kRefusedSize;
  // a long step: a thread block looks through several tokens, of which one in `pool` ends a block
  const int scan = n_tokens >= 4096 ? 32 : (n_tokens >= 512 ? 8 : 1);
  const dim3 grid((n_tokens + scan - 1) / scan, n_kv);
#define LAUNCH(T)                                                                                                    \
  return launch_kernel(attention_pool_blocks_kernel<T>, grid, dim3(kBlockMeanThreads), 0, stream, (const T*)k_pool, (const T*)v_pool, \
                       block_table, table_width, num_pages, page_tokens, (T*)kb_pool, (T*)vb_pool, pool_table,       \
                       pool_table_width, pool_pages, pool_rows, positions, seq_of_token, n_tokens, scan, n_seqs, n_kv, dk, dv, pool, \
                       status)
  if (dtype == 0) LAUNCH(float);
  if (dtype == 1) LAUNCH(__nv_bfloat16);
#undef LAUNCH
  return kRefusedDtype;
}

extern "C" int leone_attention_pooled(int dtype, const void* q, int ldq, void* out, int out_stride, const void* k_pool,
                                      const void* v_pool, const int* block_table, int table_width, int num_pages,
                                      int page_tokens, const void* kb_pool, const void* vb_pool, const int* pool_table,
                                      int pool_table_width, int pool_pages, int pool_rows, const int* seq_of_token,
                                      const int* positions, int n_tokens, int n_q, int n_kv, int dk, int dv, float scale,
                                      int window, int pool, float out_scale, int n_seqs, int* status,
                                      cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (dk <= 0 || dk > 8192 || dv <= 0 || dv > kPooledThreads * kPooledAcc || n_q <= 0 || n_kv <= 0 ||
      n_q % n_kv != 0 || n_q > 65535 || page_tokens <= 0 || table_width <= 0 || window <= 0 || pool < 0)
    return kRefusedSize;
  if (pool > 0 && (kb_pool == nullptr || vb_pool == nullptr || pool_table == nullptr || pool_rows <= 0)) return kRefusedSize;
  const dim3 grid(n_tokens, n_q);
  const size_t smem = (size_t)(dk + kPooledThreads) * sizeof(float) + 2 * kPooledThreads * sizeof(void*) + 8;
#define LAUNCH(T)                                                                                                      \
  return launch_kernel(attention_pooled_kernel<T>, grid, dim3(kPooledThreads), smem, stream, (const T*)q, ldq, (T*)out, \
                       out_stride, (const T*)k_pool, (const T*)v_pool, block_table, table_width, num_pages, page_tokens, \
                       (const T*)kb_pool, (const T*)vb_pool, pool_table, pool_table_width, pool_pages, pool_rows,      \
                       seq_of_token, positions, n_q, n_kv, dk, dv, scale, window, pool, out_scale, n_seqs, status)
  if (dtype == 0) LAUNCH(float);
  if (dtype == 1) LAUNCH(__nv_bfloat16);
#undef LAUNCH
  return kRefusedDtype;
}
