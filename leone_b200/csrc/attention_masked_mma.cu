// The attention of attention_masked.cu on tensor cores (bfloat16, mma.sync m16n8k16, fp32 sums):
// masks causal / window / chunk / window with pooled blocks before it, weights softmax / softmax with
// a silent member of score 0 / sigmoid with a bias per head, keys of dk and values of dv elements
// (multiples of 16 up to 128).
//
// Window with pooled blocks (mask 3, the rule of attention_pooled.cu): the query at position p sees
// the keys j with 0 <= p - j < size and the first floor((p - size + 1) / pool) rows of a second cache
// that holds one mean key and mean value per block of `pool` positions.  The walk over key tiles has
// two parts, tiles of block rows first and tiles of token rows after them; both feed the same running
// maximum, denominator and sums, so blocks and tokens share one softmax.
//
// Rows of a tile are (token, query head of the KV head's group) pairs of one sequence and one KV
// head; a warp owns 16 rows.  S = Q K^T and O += P V are MMAs with Q, a tile of 64 keys and the
// tile's values in shared memory (copied from the pages with 16-byte cp.async, rows padded by 16
// bytes so that ldmatrix finds eight rows in eight banks); P is rounded to bfloat16 as the second
// product's operand while maxima, exponentials and denominators stay fp32.
//
//  * prompt form: a block of four warps owns 64 rows and walks the key tiles its rows can see
//    (from the first key the tile's first token sees to the last token's position), the tiles
//    double-buffered;
//  * decode form (every sequence brings one token, so a KV head has g <= 16 rows): the four warps
//    of a block share the 16 rows and take every fourth key tile each, with tiles of their own;
//    the key range may also be split over several blocks.  Partial results (running maximum,
//    denominator, sums) are merged in shared memory, and across blocks by a second kernel.
//
// The silent member of "softmax plus one" is one more partial result (maximum 0, denominator 1,
// sums 0): the prompt form starts from it, the decode form adds it in the last merge.
#include "common.cuh"
#include "mma_tile.cuh"

namespace leone {

constexpr int kMmRows = 64, kMmKeys = 64, kMmThreads = 128;
constexpr int kDecKeys = 32;      // keys per tile in the decode form: smaller tiles, more blocks per SM

__device__ __forceinline__ void ldsm4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ uint32_t pack_bf16(float a, float b) {
  __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}
// 2^x by the special-function unit (2^-inf = 0); scores are kept in units of log 2 so that a weight
// costs one subtraction and one of these.
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
constexpr float kLog2e = 1.4426950408889634f;
__device__ __forceinline__ int mm_first_seen(int mask, int size, int pos) {
  if (mask == 1 || mask == 3) return max(0, pos - size + 1);
  if (mask == 2) return (pos / size) * size;
  return 0;
}

// block rows the query at `pos` sees (mask 3 only): the blocks that lie wholly before its window
__device__ __forceinline__ int mm_blocks_seen(int mask, int size, int pool, int pos) {
  return mask == 3 && pos - size + 1 >= pool ? (pos - size + 1) / pool : 0;
}

struct MaskedArgs {
  const __nv_bfloat16* qkv;
  int row_stride;
  __nv_bfloat16* out;
  int out_stride;
  const __nv_bfloat16* k_pool;
  const __nv_bfloat16* v_pool;
  const int* block_table;
  int table_width;
  const int* q_start;      // [n_seqs + 1] first row of each sequence in the step
  const int* ctx_len;      // [n_seqs] keys of the sequence after the step
  int n_q, n_kv, dk, dv;
  float scale;
  int mask, mask_size, weights;
  const float* bias;
  int page_tokens, num_pages;
  int splits;
  float* partial;          // decode form with splits > 1: [seq][kv head][split][16][dv + 2]
  int* status;
  // mask 3: the cache of block means.  The page of a block's last position e (found through
  // pool_table like a token's page) holds its row at (e % page_tokens) / pool; a page has pool_rows rows.
  const __nv_bfloat16* kb_pool = nullptr;
  const __nv_bfloat16* vb_pool = nullptr;
  const int* pool_table = nullptr;
  int pool_table_width = 0, pool_pages = 0, pool_rows = 0, pool = 0;
  float out_scale = 1.f;  // the output rows are multiplied by this
};

// The place of member j of (sequence, kv head) in its pool, in rows: token j, or block j with `blocks`.
// -1 and a status word if the table has no page for it.
__device__ __forceinline__ long long mm_member_slot(const MaskedArgs& a, bool blocks, int seq, int kvh, int j, int tok_row) {
  if (blocks) {
    const int e = j * a.pool + a.pool - 1;
    const int blk = e / a.page_tokens;
    const int page = blk < a.pool_table_width ? a.pool_table[(size_t)seq * a.pool_table_width + blk] : -1;
    if (page < 0 || page >= a.pool_pages) {
      set_status(a.status, kBadPage, tok_row, page, e);
      return -1;
    }
    return ((long long)page * a.n_kv + kvh) * a.pool_rows + (e - blk * a.page_tokens) / a.pool;
  }
  const int blk = j / a.page_tokens;
  const int page = blk < a.table_width ? a.block_table[(size_t)seq * a.table_width + blk] : -1;
  if (page < 0 || page >= a.num_pages) {
    set_status(a.status, kBadPage, tok_row, page, j);
    return -1;
  }
  return ((long long)page * a.n_kv + kvh) * a.page_tokens + (j - blk * a.page_tokens);
}

// Copies keys j0 .. j0 + keys - 1 of (sequence, kv head) into a tile: K rows of dk, V rows of dv elements.
// Keys outside [lo, hi] become zeros.  `lanes` threads take part, this one is `me`.  With `blocks` the
// members are rows of the cache of block means.
__device__ __forceinline__ void load_kv_tile(const MaskedArgs& a, int seq, int kvh, int j0, int lo, int hi,
                                             uint32_t k_s, uint32_t v_s, int pitch_k, int pitch_v, int me, int lanes,
                                             int tok_row, int keys, bool blocks = false) {
  const __nv_bfloat16* k_src = blocks ? a.kb_pool : a.k_pool;
  const __nv_bfloat16* v_src = blocks ? a.vb_pool : a.v_pool;
  const int kc = a.dk >> 3, vc = a.dv >> 3;         // 16-byte chunks per row
  // a block's threads pair up on a key row, a warp's lanes take whole rows: one look-up of the
  // row's page per thread, then copies that depend on nothing else
  const int tpr = lanes >= 128 ? 2 : 1, sub = me % tpr;
  for (int r = me / tpr; r < keys; r += lanes / tpr) {
    const int j = j0 + r;
    bool ok = j >= lo && j <= hi;
    long long slot = 0;
    if (ok) {
      slot = mm_member_slot(a, blocks, seq, kvh, j, tok_row);
      if (slot < 0) {
        ok = false;
        slot = 0;
      }
    }
    const __nv_bfloat16* ks = k_src + slot * a.dk;
    const __nv_bfloat16* vs = v_src + slot * a.dv;
    const uint32_t kd = k_s + r * pitch_k * 2, vd = v_s + r * pitch_v * 2;
    for (int w = sub; w < kc; w += tpr) cp_async16_zfill(kd + w * 16, ok ? (const void*)(ks + w * 8) : (const void*)k_src, ok);
    for (int w = sub; w < vc; w += tpr) cp_async16_zfill(vd + w * 16, ok ? (const void*)(vs + w * 8) : (const void*)v_src, ok);
  }
}

// The same by one warp for a tile of up to 32 keys, with coalesced copies: lane r first finds the place
// of key row r (one look-up in the block table) and leaves it in `slot_s` (32 entries of the warp's
// own); then consecutive lanes copy consecutive 16-byte pieces of a row, so that one instruction
// covers whole rows instead of a piece of 32 different ones.
__device__ __forceinline__ void load_kv_tile_warp(const MaskedArgs& a, int seq, int kvh, int j0, int lo, int hi,
                                                  uint32_t k_s, uint32_t v_s, int pitch_k, int pitch_v, int lane,
                                                  int tok_row, int keys, long long* slot_s, bool blocks = false) {
  {
    const int j = j0 + lane;
    long long slot = -1;
    if (lane < keys && j >= lo && j <= hi) slot = mm_member_slot(a, blocks, seq, kvh, j, tok_row);
    __syncwarp();                  // the last tile's readers of slot_s are done
    slot_s[lane] = slot;
    __syncwarp();
  }
  auto copy = [&](const __nv_bfloat16* pool, int width, uint32_t dst, int pitch) {
    const int chunks = width >> 3;                       // 16-byte pieces per row
    int r = lane / chunks, w = lane - r * chunks;
    const int dr = 32 / chunks, dw = 32 - dr * chunks;
    while (r < keys) {
      const long long slot = slot_s[r];
      const bool ok = slot >= 0;
      cp_async16_zfill(dst + (r * pitch + w * 8) * 2, ok ? (const void*)(pool + slot * width + w * 8) : (const void*)pool, ok);
      r += dr;
      w += dw;
      if (w >= chunks) {
        w -= chunks;
        r += 1;
      }
    }
  };
  copy(blocks ? a.kb_pool : a.k_pool, a.dk, k_s, pitch_k);
  copy(blocks ? a.vb_pool : a.v_pool, a.dv, v_s, pitch_v);
}

// One warp, 16 rows, one tile of NT * 8 keys (64 in the prompt form, 32 in the decode form): scores,
// weights, and the sums into o.  Row `g` (and g + 8)
// of the warp sees keys [lo_r, hi_r] (absolute positions); the tile starts at key j0.  `full`
// (uniform in the warp): every row sees every key of the tile, so no key is tested.  `scale2` is
// the score scale times log2(e), the bias and the running maximum are in the same units.
template <int DKT, int DVT, int NT>
__device__ __forceinline__ void tile_step(uint32_t q_s, uint32_t k_s, uint32_t v_s, int pitch_k, int pitch_v, int dkt,
                                          int dvt, int lane, int j0, bool full, const int (&lo_r)[2],
                                          const int (&hi_r)[2], float scale2, int weights, const float (&bias_r)[2],
                                          float (&m_run)[2], float (&l_run)[2], float (&o)[2 * DVT][4]) {
  float s[NT][4];
#pragma unroll
  for (int n = 0; n < NT; ++n) s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f;
  const int mi = lane >> 3;
#pragma unroll
  for (int kt = 0; kt < DKT; ++kt) {
    if (kt < dkt) {
      uint32_t a0, a1, a2, a3;
      ldsm4(q_s + ((lane & 15) * pitch_k + kt * 16 + (lane >> 4) * 8) * 2, a0, a1, a2, a3);
#pragma unroll
      for (int np = 0; np < NT / 2; ++np) {
        uint32_t b0, b1, b2, b3;
        ldsm4(k_s + ((np * 16 + (lane & 7) + (mi >> 1) * 8) * pitch_k + kt * 16 + (mi & 1) * 8) * 2, b0, b1, b2, b3);
        mma16816(s[2 * np], a0, a1, a2, a3, b0, b1);
        mma16816(s[2 * np + 1], a0, a1, a2, a3, b2, b3);
      }
    }
  }
  const int tq = lane & 3;
  // scores -> weights; element i of n-tile n: row half i >> 1, key j0 + n * 8 + 2 * tq + (i & 1).
  // Keys a row does not see get the score -inf (scale2 > 0 keeps it), which every rule turns into 0.
  if (!full) {
#pragma unroll
    for (int n = 0; n < NT; ++n)
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int h = i >> 1, j = j0 + n * 8 + 2 * tq + (i & 1);
        if (j < lo_r[h] || j > hi_r[h]) s[n][i] = -INFINITY;
      }
  }
  if (weights == 2) {
#pragma unroll
    for (int n = 0; n < NT; ++n)
#pragma unroll
      for (int i = 0; i < 4; ++i)      // the reciprocal of 1 + 2^+inf is 0
        s[n][i] = __frcp_rn(1.f + fast_exp2(-fmaf(s[n][i], scale2, bias_r[i >> 1])));
  } else {
    float tile_max[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int n = 0; n < NT; ++n)
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        s[n][i] *= scale2;
        tile_max[i >> 1] = fmaxf(tile_max[i >> 1], s[n][i]);
      }
    float alpha[2], m_use[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      tile_max[h] = fmaxf(tile_max[h], __shfl_xor_sync(0xffffffffu, tile_max[h], 1));
      tile_max[h] = fmaxf(tile_max[h], __shfl_xor_sync(0xffffffffu, tile_max[h], 2));
      const float m_new = fmaxf(m_run[h], tile_max[h]);
      m_use[h] = m_new == -INFINITY ? 0.f : m_new;
      alpha[h] = m_run[h] == -INFINITY ? 0.f : fast_exp2(m_run[h] - m_use[h]);
      m_run[h] = m_new;
      l_run[h] *= alpha[h];
    }
#pragma unroll
    for (int n = 0; n < 2 * DVT; ++n) {
      o[n][0] *= alpha[0];
      o[n][1] *= alpha[0];
      o[n][2] *= alpha[1];
      o[n][3] *= alpha[1];
    }
#pragma unroll
    for (int n = 0; n < NT; ++n)
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float p = fast_exp2(s[n][i] - m_use[i >> 1]);      // 2^-inf = 0 for keys the row does not see
        s[n][i] = p;
        l_run[i >> 1] += p;
      }
  }
  // O += P V: P as A fragments (16 keys a step), V^T fragments through ldmatrix.trans
#pragma unroll
  for (int kk = 0; kk < NT / 2; ++kk) {
    const uint32_t a0 = pack_bf16(s[2 * kk][0], s[2 * kk][1]), a1 = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
    const uint32_t a2 = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]), a3 = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
    for (int nd = 0; nd < DVT; ++nd) {
      if (nd < dvt) {
        uint32_t b0, b1, b2, b3;
        ldsm4_trans(v_s + ((kk * 16 + (mi & 1) * 8 + (lane & 7)) * pitch_v + nd * 16 + (mi >> 1) * 8) * 2, b0, b1, b2, b3);
        mma16816(o[2 * nd], a0, a1, a2, a3, b0, b1);
        mma16816(o[2 * nd + 1], a0, a1, a2, a3, b2, b3);
      }
    }
  }
}

// ---- prompt form ------------------------------------------------------------------------------------
// grid (row tiles of the longest sequence, kv heads, sequences)
template <int DKT, int DVT>
__global__ void __launch_bounds__(kMmThreads)
attention_masked_prefill_kernel(const MaskedArgs a) {
  pdl_trigger();
  pdl_wait();
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int seq = blockIdx.z, kvh = blockIdx.y;
  const int g = a.n_q / a.n_kv;
  const int toks_per_tile = kMmRows / g;
  const int row0 = a.q_start[seq], q_len = a.q_start[seq + 1] - row0;
  const int tok0 = blockIdx.x * toks_per_tile;
  if (tok0 >= q_len) return;
  const int n_tok = min(toks_per_tile, q_len - tok0);
  const int start = a.ctx_len[seq] - q_len;          // position of the sequence's first token of this step
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int pitch_k = a.dk + 8, pitch_v = a.dv + 8;
  const uint32_t base = (uint32_t)__cvta_generic_to_shared(smem_raw);
  const uint32_t q_s = base;
  const uint32_t kv_s = q_s + kMmRows * pitch_k * 2;
  const uint32_t stage_bytes = kMmKeys * (pitch_k + pitch_v) * 2;
  const int dkt = a.dk >> 4, dvt = a.dv >> 4;

  // Q rows: row r = token r / g, head r % g of the group
  {
    const int kc = a.dk >> 3;
    for (int c = tid; c < kMmRows * kc; c += kMmThreads) {
      const int r = c / kc, w = c - r * kc;
      const int tl = r / g, hg = r - tl * g;
      const bool ok = tl < n_tok;
      const __nv_bfloat16* src = a.qkv + (size_t)(row0 + tok0 + tl) * a.row_stride + (size_t)(kvh * g + hg) * a.dk + w * 8;
      cp_async16_zfill(q_s + (r * pitch_k + w * 8) * 2, ok ? (const void*)src : (const void*)a.qkv, ok);
    }
  }
  const int pos_first = start + tok0, pos_last = start + tok0 + n_tok - 1;
  const int k_lo = mm_first_seen(a.mask, a.mask_size, pos_first);
  // tiles of block rows (mask 3: the blocks the tile's last token sees) come before the tiles of token rows
  const int nb_last = mm_blocks_seen(a.mask, a.mask_size, a.pool, pos_last);
  const int nbt = (nb_last + kMmKeys - 1) / kMmKeys;
  const int n_tiles = nbt + (pos_last - k_lo) / kMmKeys + 1;
  auto load_tile = [&](int t, uint32_t dst) {
    if (t < nbt)
      load_kv_tile(a, seq, kvh, t * kMmKeys, 0, nb_last - 1, dst, dst + kMmKeys * pitch_k * 2, pitch_k, pitch_v, tid,
                   kMmThreads, row0 + tok0, kMmKeys, true);
    else
      load_kv_tile(a, seq, kvh, k_lo + (t - nbt) * kMmKeys, k_lo, pos_last, dst, dst + kMmKeys * pitch_k * 2, pitch_k,
                   pitch_v, tid, kMmThreads, row0 + tok0, kMmKeys);
  };
  load_tile(0, kv_s);
  asm volatile("cp.async.commit_group;" ::: "memory");

  // this thread's two rows
  int lo_r[2], hi_r[2], blo_r[2] = {0, 0}, bhi_r[2];
  float bias_r[2];
  const int gq = lane >> 2;
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int r = warp * 16 + gq + 8 * h;
    const int tl = r / g, hg = r - tl * g;
    const bool ok = tl < n_tok;
    const int pos = start + tok0 + tl;
    hi_r[h] = ok ? pos : -1;
    lo_r[h] = ok ? mm_first_seen(a.mask, a.mask_size, pos) : 0;
    bhi_r[h] = ok ? mm_blocks_seen(a.mask, a.mask_size, a.pool, pos) - 1 : -1;
    bias_r[h] = (a.weights == 2 && ok) ? a.bias[kvh * g + hg] * kLog2e : 0.f;
  }
  // the warp's rows: the tokens they belong to, for tiles that every row sees in full
  const int w_tok_first = (warp * 16) / g, w_tok_last = min((warp * 16 + 15) / g, n_tok - 1);
  const bool w_all_valid = (warp * 16 + 15) / g < n_tok;
  const int w_lo_max = mm_first_seen(a.mask, a.mask_size, start + tok0 + max(w_tok_last, 0));
  const int w_hi_min = start + tok0 + w_tok_first;
  // block rows: those the warp's last token sees, and those all its rows see
  const int w_nb_any = mm_blocks_seen(a.mask, a.mask_size, a.pool, start + tok0 + max(w_tok_last, 0));
  const int w_nb_all = mm_blocks_seen(a.mask, a.mask_size, a.pool, start + tok0 + w_tok_first);
  float m_run[2], l_run[2];
  // the silent member: maximum 0 and, in one of the four lanes that share a row, denominator 1
  m_run[0] = m_run[1] = a.weights == 1 ? 0.f : -INFINITY;
  l_run[0] = l_run[1] = (a.weights == 1 && (lane & 3) == 0) ? 1.f : 0.f;
  float o[2 * DVT][4];
#pragma unroll
  for (int n = 0; n < 2 * DVT; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;

  for (int t = 0; t < n_tiles; ++t) {
    const uint32_t cur = kv_s + (t & 1) * stage_bytes, nxt = kv_s + ((t + 1) & 1) * stage_bytes;
    if (t + 1 < n_tiles) load_tile(t + 1, nxt);
    asm volatile("cp.async.commit_group;" ::: "memory");
    asm volatile("cp.async.wait_group 1;" ::: "memory");
    __syncthreads();
    if (t < nbt) {
      const int b0 = t * kMmKeys;
      if ((warp * 16) / g < n_tok && b0 < w_nb_any)
        tile_step<DKT, DVT, 8>(q_s + warp * 16 * pitch_k * 2, cur, cur + kMmKeys * pitch_k * 2, pitch_k, pitch_v, dkt, dvt,
                               lane, b0, w_all_valid && b0 + kMmKeys <= w_nb_all, blo_r, bhi_r, a.scale * kLog2e,
                               a.weights, bias_r, m_run, l_run, o);
      __syncthreads();
      continue;
    }
    const int j0 = k_lo + (t - nbt) * kMmKeys;
    // a warp whose rows see nothing of this tile skips it (uniform per warp)
    const int w_hi = min(start + tok0 + min((warp * 16 + 15) / g, n_tok - 1), pos_last);
    const int w_first_tok = (warp * 16) / g;
    const bool any = w_first_tok < n_tok && j0 <= w_hi &&
                     j0 + kMmKeys - 1 >= mm_first_seen(a.mask, a.mask_size, start + tok0 + w_first_tok);
    const bool full = w_all_valid && j0 >= w_lo_max && j0 + kMmKeys - 1 <= w_hi_min;
    if (any)
      tile_step<DKT, DVT, 8>(q_s + warp * 16 * pitch_k * 2, cur, cur + kMmKeys * pitch_k * 2, pitch_k, pitch_v, dkt, dvt, lane,
                          j0, full, lo_r, hi_r, a.scale * kLog2e, a.weights, bias_r, m_run, l_run, o);
    __syncthreads();
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");
  // finish: the row's denominator is spread over the four lanes that share the row
  const int tq = lane & 3;
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    float l = l_run[h];
    l += __shfl_xor_sync(0xffffffffu, l, 1);
    l += __shfl_xor_sync(0xffffffffu, l, 2);
    const float inv = a.weights == 2 ? a.out_scale : (l > 0.f ? a.out_scale / l : 0.f);
    const int r = warp * 16 + gq + 8 * h;
    const int tl = r / g, hg = r - tl * g;
    if (tl >= n_tok) continue;
    __nv_bfloat16* dst = a.out + (size_t)(row0 + tok0 + tl) * a.out_stride + (size_t)(kvh * g + hg) * a.dv;
#pragma unroll
    for (int n = 0; n < 2 * DVT; ++n)
      if (n < 2 * dvt)
        *reinterpret_cast<__nv_bfloat162*>(dst + n * 8 + 2 * tq) =
            __floats2bfloat162_rn(o[n][2 * h] * inv, o[n][2 * h + 1] * inv);
  }
}

// ---- decode form -------------------------------------------------------------------------------------
// grid (splits, kv heads, sequences); every sequence brings one token (row q_start[seq]).
template <int DKT, int DVT>
__global__ void __launch_bounds__(kMmThreads)
attention_masked_decode_kernel(const MaskedArgs a) {
  pdl_trigger();
  pdl_wait();
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __shared__ long long slot_s[4][32];
  const int split = blockIdx.x, kvh = blockIdx.y, seq = blockIdx.z;
  const int g = a.n_q / a.n_kv;
  const int row = a.q_start[seq];
  const int pos = a.ctx_len[seq] - 1;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int pitch_k = a.dk + 8, pitch_v = a.dv + 8;
  const uint32_t base = (uint32_t)__cvta_generic_to_shared(smem_raw);
  const uint32_t q_s = base;
  const uint32_t tile_bytes = kDecKeys * (pitch_k + pitch_v) * 2;
  const uint32_t my_k = q_s + 16 * pitch_k * 2 + warp * tile_bytes, my_v = my_k + kDecKeys * pitch_k * 2;
  const int dkt = a.dk >> 4, dvt = a.dv >> 4;
  {
    const int kc = a.dk >> 3;
    for (int c = tid; c < 16 * kc; c += kMmThreads) {
      const int r = c / kc, w = c - r * kc;
      const bool ok = r < g;
      const __nv_bfloat16* src = a.qkv + (size_t)row * a.row_stride + (size_t)(kvh * g + r) * a.dk + w * 8;
      cp_async16_zfill(q_s + (r * pitch_k + w * 8) * 2, ok ? (const void*)src : (const void*)a.qkv, ok);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncthreads();
  }
  const int k_lo = mm_first_seen(a.mask, a.mask_size, pos);
  const int nb = mm_blocks_seen(a.mask, a.mask_size, a.pool, pos);     // tiles of block rows come first
  const int nbt = (nb + kDecKeys - 1) / kDecKeys;
  const int n_tiles = nbt + (pos - k_lo) / kDecKeys + 1;
  const int per_split = (n_tiles + a.splits - 1) / a.splits;
  const int t_begin = split * per_split, t_end = min(n_tiles, t_begin + per_split);
  const int gq = lane >> 2;
  int lo_r[2], hi_r[2], blo_r[2] = {0, 0}, bhi_r[2];
  float bias_r[2];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int r = gq + 8 * h;
    hi_r[h] = r < g ? pos : -1;
    bhi_r[h] = r < g ? nb - 1 : -1;
    lo_r[h] = k_lo;
    bias_r[h] = (a.weights == 2 && r < g) ? a.bias[kvh * g + r] * kLog2e : 0.f;
  }
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
  float o[2 * DVT][4];
#pragma unroll
  for (int n = 0; n < 2 * DVT; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;
  for (int t = t_begin + warp; t < t_end; t += 4) {
    const bool blocks = t < nbt;
    const int j0 = blocks ? t * kDecKeys : k_lo + (t - nbt) * kDecKeys;
    load_kv_tile_warp(a, seq, kvh, j0, blocks ? 0 : k_lo, blocks ? nb - 1 : pos, my_k, my_v, pitch_k, pitch_v, lane, row,
                      kDecKeys, slot_s[warp], blocks);
    asm volatile("cp.async.commit_group;" ::: "memory");
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncwarp();
    tile_step<DKT, DVT, kDecKeys / 8>(q_s, my_k, my_v, pitch_k, pitch_v, dkt, dvt, lane, j0, false, blocks ? blo_r : lo_r,
                                      blocks ? bhi_r : hi_r, a.scale * kLog2e, a.weights, bias_r, m_run, l_run, o);
    __syncwarp();
  }
  // the four warps' partial results into shared memory (over the tiles, which are done with)
  __syncthreads();
  float* part = reinterpret_cast<float*>(smem_raw);        // [4 warps][16 rows][dv + 2]
  const int pw = a.dv + 2, tq = lane & 3;
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    float l = l_run[h];
    l += __shfl_xor_sync(0xffffffffu, l, 1);
    l += __shfl_xor_sync(0xffffffffu, l, 2);
    float* dst = part + ((size_t)warp * 16 + gq + 8 * h) * pw;
#pragma unroll
    for (int n = 0; n < 2 * DVT; ++n)
      if (n < 2 * dvt) {
        dst[n * 8 + 2 * tq] = o[n][2 * h];
        dst[n * 8 + 2 * tq + 1] = o[n][2 * h + 1];
      }
    if (tq == 0) {
      dst[a.dv] = m_run[h];
      dst[a.dv + 1] = l;
    }
  }
  __syncthreads();
  // merge: thread -> (row, column) pairs
  float* out_part = a.splits > 1 ? a.partial + (((size_t)seq * a.n_kv + kvh) * a.splits + split) * 16 * pw : nullptr;
  for (int r = warp; r < g; r += 4) {
    float m = -INFINITY;
    if (a.weights != 2)
      for (int w = 0; w < 4; ++w) m = fmaxf(m, part[((size_t)w * 16 + r) * pw + a.dv]);
    const bool last = a.splits == 1;
    if (a.weights == 1 && last) m = fmaxf(m, 0.f);
    float f[4], l = 0.f;
    for (int w = 0; w < 4; ++w) {
      const float mw = part[((size_t)w * 16 + r) * pw + a.dv];
      f[w] = a.weights == 2 ? 1.f : (mw == -INFINITY ? 0.f : fast_exp2(mw - m));
      l += f[w] * part[((size_t)w * 16 + r) * pw + a.dv + 1];
    }
    if (a.weights == 1 && last) l += fast_exp2(-m);
    if (last) {
      const float inv = a.weights == 2 ? a.out_scale : (l > 0.f ? a.out_scale / l : 0.f);
      __nv_bfloat16* dst = a.out + (size_t)row * a.out_stride + (size_t)(kvh * g + r) * a.dv;
      for (int c = lane; c < a.dv; c += 32) {
        float v = 0.f;
        for (int w = 0; w < 4; ++w) v += f[w] * part[((size_t)w * 16 + r) * pw + c];
        dst[c] = __float2bfloat16_rn(v * inv);
      }
    } else {
      float* dst = out_part + (size_t)r * pw;
      for (int c = lane; c < a.dv; c += 32) {
        float v = 0.f;
        for (int w = 0; w < 4; ++w) v += f[w] * part[((size_t)w * 16 + r) * pw + c];
        dst[c] = v;
      }
      if (lane == 0) {
        dst[a.dv] = m;
        dst[a.dv + 1] = l;
      }
    }
  }
}

// The splits of a (sequence, query head) into the output row.  grid (query heads, sequences).
__global__ void __launch_bounds__(128)
attention_masked_merge_kernel(const MaskedArgs a) {
  pdl_trigger();
  pdl_wait();
  const int h = blockIdx.x, seq = blockIdx.y;
  const int g = a.n_q / a.n_kv, kvh = h / g, r = h - kvh * g;
  const int pw = a.dv + 2;
  const float* src = a.partial + (((size_t)seq * a.n_kv + kvh) * a.splits) * 16 * pw + (size_t)r * pw;
  const size_t step = (size_t)16 * pw;
  float m = a.weights == 1 ? 0.f : -INFINITY;
  if (a.weights != 2)
    for (int s = 0; s < a.splits; ++s) m = fmaxf(m, src[s * step + a.dv]);
  float l = a.weights == 1 ? fast_exp2(-m) : 0.f;      // maxima are in units of log 2
  for (int s = 0; s < a.splits; ++s) {
    const float ms = src[s * step + a.dv];
    if (a.weights != 2 && ms != -INFINITY) l += fast_exp2(ms - m) * src[s * step + a.dv + 1];
  }
  const float inv = a.weights == 2 ? a.out_scale : (l > 0.f ? a.out_scale / l : 0.f);
  __nv_bfloat16* dst = a.out + (size_t)a.q_start[seq] * a.out_stride + (size_t)h * a.dv;
  for (int c = threadIdx.x; c < a.dv; c += blockDim.x) {
    float v = 0.f;
    for (int s = 0; s < a.splits; ++s) {
      const float ms = src[s * step + a.dv];
      const float f = a.weights == 2 ? 1.f : (ms == -INFINITY ? 0.f : fast_exp2(ms - m));
      v += f * src[s * step + c];
    }
    dst[c] = __float2bfloat16_rn(v * inv);
  }
}

template <int DKT, int DVT>
static int launch_masked(const MaskedArgs& a, int n_seqs, int max_q_len, bool decode, cudaStream_t stream) {
  const int pitch_k = a.dk + 8, pitch_v = a.dv + 8;
  const int g = a.n_q / a.n_kv;
  if (decode) {
    size_t smem = (size_t)16 * pitch_k * 2 + 4 * (size_t)kDecKeys * (pitch_k + pitch_v) * 2;
    const size_t merge = (size_t)4 * 16 * (a.dv + 2) * sizeof(float);
    if (merge > smem) smem = merge;
    static size_t configured = 0;
    if (smem > configured) {
      cudaFuncSetAttribute(attention_masked_decode_kernel<DKT, DVT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      configured = smem;
    }
    int r = launch_kernel(attention_masked_decode_kernel<DKT, DVT>, dim3(a.splits, a.n_kv, n_seqs), dim3(kMmThreads), smem,
                          stream, a);
    if (r != 0 || a.splits == 1) return r;
    return launch_kernel(attention_masked_merge_kernel, dim3(a.n_q, n_seqs), dim3(128), 0, stream, a);
  }
  const size_t smem = (size_t)kMmRows * pitch_k * 2 + 2 * (size_t)kMmKeys * (pitch_k + pitch_v) * 2;
  static size_t configured = 0;
  if (smem > configured) {
    cudaFuncSetAttribute(attention_masked_prefill_kernel<DKT, DVT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    configured = smem;
  }
  const int toks_per_tile = kMmRows / g;
  return launch_kernel(attention_masked_prefill_kernel<DKT, DVT>, dim3((max_q_len + toks_per_tile - 1) / toks_per_tile, a.n_kv, n_seqs),
                       dim3(kMmThreads), smem, stream, a);
}

}  // namespace leone

using namespace leone;

extern "C" int leone_attention_masked_mma_supported(int n_q, int n_kv, int dk, int dv, int decode) {
  if (n_q <= 0 || n_kv <= 0 || n_q % n_kv != 0) return 0;
  const int g = n_q / n_kv;
  return dk % 16 == 0 && dv % 16 == 0 && dk >= 16 && dv >= 16 && dk <= 128 && dv <= 128 && g <= (decode ? 16 : 64);
}

extern "C" long long leone_attention_masked_mma_scratch(int n_seqs, int n_kv, int dv, int splits) {
  return splits > 1 ? (long long)n_seqs * n_kv * splits * 16 * (dv + 2) : 0;
}

// decode != 0: every sequence brings exactly one token; `splits` blocks share a (sequence, kv head)'s
// keys and `partial` holds leone_attention_masked_mma_scratch floats if splits > 1.
extern "C" int leone_attention_masked_mma(const void* qkv, int row_stride, void* out, int out_stride, const void* k_pool,
                                          const void* v_pool, const int* block_table, int table_width,
                                          const int* q_start, const int* ctx_len, int n_seqs, int max_q_len, int n_q,
                                          int n_kv, int dk, int dv, float scale, int mask, int mask_size, int weights,
                                          const float* bias, int page_tokens, int num_pages, int decode, int splits,
                                          float* partial, int* status, cudaStream_t stream) {
  if (n_seqs <= 0 || max_q_len <= 0) return 0;
  if (!leone_attention_masked_mma_supported(n_q, n_kv, dk, dv, decode)) return kRefusedSize;
  if (mask < 0 || mask > 2 || weights < 0 || weights > 2 || (mask != 0 && mask_size <= 0)) return kRefusedSize;
  if (weights == 2 && bias == nullptr) return kRefusedSize;
  if (row_stride % 8 != 0 || out_stride % 2 != 0 || ((uintptr_t)qkv & 15) || ((uintptr_t)k_pool & 15) || ((uintptr_t)v_pool & 15) ||
      ((uintptr_t)out & 3))
    return kRefusedAlignment;
  if (n_kv > 65535 || n_seqs > 65535 || page_tokens <= 0 || table_width <= 0) return kRefusedSize;
  if (!decode) splits = 1;
  if (splits < 1 || splits > 64 || (splits > 1 && partial == nullptr)) return kRefusedSize;
  MaskedArgs a{(const __nv_bfloat16*)qkv, row_stride, (__nv_bfloat16*)out, out_stride, (const __nv_bfloat16*)k_pool,
               (const __nv_bfloat16*)v_pool, block_table, table_width, q_start, ctx_len, n_q, n_kv, dk, dv, scale, mask,
               mask_size, weights, bias, page_tokens, num_pages, splits, partial, status};
  const bool wide_k = dk > 64, wide_v = dv > 64;
  if (wide_k && wide_v) return launch_masked<8, 8>(a, n_seqs, max_q_len, decode != 0, stream);
  if (wide_k) return launch_masked<8, 4>(a, n_seqs, max_q_len, decode != 0, stream);
  if (wide_v) return launch_masked<4, 8>(a, n_seqs, max_q_len, decode != 0, stream);
  return launch_masked<4, 4>(a, n_seqs, max_q_len, decode != 0, stream);
}

// The same with mask 3, a window of `window` token rows and before it the rows of the cache of block
// means (pool positions a row); `q` holds the query heads only, the output rows are multiplied by
// out_scale.  Softmax weights.
extern "C" int leone_attention_pooled_mma(const void* q, int ldq, void* out, int out_stride, const void* k_pool,
                                          const void* v_pool, const int* block_table, int table_width, int num_pages,
                                          int page_tokens, const void* kb_pool, const void* vb_pool,
                                          const int* pool_table, int pool_table_width, int pool_pages, int pool_rows,
                                          const int* q_start, const int* ctx_len, int n_seqs, int max_q_len, int n_q,
                                          int n_kv, int dk, int dv, float scale, int window, int pool, float out_scale,
                                          int decode, int splits, float* partial, int* status, cudaStream_t stream) {
  if (n_seqs <= 0 || max_q_len <= 0) return 0;
  if (!leone_attention_masked_mma_supported(n_q, n_kv, dk, dv, decode)) return kRefusedSize;
  if (window <= 0 || pool <= 0 || kb_pool == nullptr || vb_pool == nullptr || pool_table == nullptr ||
      pool_table_width <= 0 || pool_rows < (page_tokens + pool - 1) / pool)
    return kRefusedSize;
  if (ldq % 8 != 0 || out_stride % 2 != 0 || ((uintptr_t)q & 15) || ((uintptr_t)k_pool & 15) || ((uintptr_t)v_pool & 15) ||
      ((uintptr_t)kb_pool & 15) || ((uintptr_t)vb_pool & 15) || ((uintptr_t)out & 3))
    return kRefusedAlignment;
  if (n_kv > 65535 || n_seqs > 65535 || page_tokens <= 0 || table_width <= 0) return kRefusedSize;
  if (!decode) splits = 1;
  if (splits < 1 || splits > 64 || (splits > 1 && partial == nullptr)) return kRefusedSize;
  MaskedArgs a{(const __nv_bfloat16*)q, ldq, (__nv_bfloat16*)out, out_stride, (const __nv_bfloat16*)k_pool,
               (const __nv_bfloat16*)v_pool, block_table, table_width, q_start, ctx_len, n_q, n_kv, dk, dv, scale, 3,
               window, 0, nullptr, page_tokens, num_pages, splits, partial, status};
  a.kb_pool = (const __nv_bfloat16*)kb_pool;
  a.vb_pool = (const __nv_bfloat16*)vb_pool;
  a.pool_table = pool_table;
  a.pool_table_width = pool_table_width;
  a.pool_pages = pool_pages;
  a.pool_rows = pool_rows;
  a.pool = pool;
  a.out_scale = out_scale;
  const bool wide_k = dk > 64, wide_v = dv > 64;
  if (wide_k && wide_v) return launch_masked<8, 8>(a, n_seqs, max_q_len, decode != 0, stream);
  if (wide_k) return launch_masked<8, 4>(a, n_seqs, max_q_len, decode != 0, stream);
  if (wide_v) return launch_masked<4, 8>(a, n_seqs, max_q_len, decode != 0, stream);
  return launch_masked<4, 4>(a, n_seqs, max_q_len, decode != 0, stream);
}
