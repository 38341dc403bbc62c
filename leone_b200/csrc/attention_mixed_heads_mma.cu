// Attention with scores mixed across heads (see attention_mixed_heads.cu for the rule), prompt portions
// on tensor cores (bfloat16, key width a multiple of 16, value width 32, 64, 96 or 128).
//
// A block of 16 warps owns a tile of 16 consecutive query rows of one sequence and ALL query heads'
// scores, because a head's score needs every head's product with the key:
//   (1) a tile of 32 keys and values of all key/value heads is copied from the pages into shared memory
//       (16-byte cp.async, one page look-up per key);
//   (2) the heads are dealt to the warps; a warp forms raw = Q_h K^T for its heads with mma.sync (Q
//       fragments from shared memory, fp32 sums), multiplies by scale * temp_h, applies the soft cap and
//       leaves the 16 x 32 raw scores in shared memory;
//   (3) every thread owns one (row, key) pair, takes the raw scores of all heads into registers and mixes:
//       s_h = sum_g M[h, g] raw_g for the heads of the block's head group, fp32 on CUDA cores, applies the
//       mask (-inf) and writes the mixed scores over the raw ones of those heads;
//   (4) a warp takes the mixed scores of its head in accumulator layout, keeps the running maximum and
//       sum (started at (sink, 1)), and adds P V with mma.sync.  The weights stay fp32: P is split into
//       two bfloat16 terms (P = hi + lo, two MMAs), so that the product sees 16 bits of it.
// Outputs of one head fill 64 registers of a thread at value width 128, so a block accumulates at most
// 16 heads x 128 columns; with more, several blocks share a query tile: each forms all raw scores and
// mixes, normalises and accumulates the heads of its group only.  Where the query tile of all heads does not
// fit beside the key, value and score tiles (32 heads of 128), its fragments are read from global memory
// (the L2) for every key tile instead of from shared memory (QS = false).  At most 32 query heads.
#include "common.cuh"
#include "mma_tile.cuh"

namespace leone {

constexpr int kMmThreads = 512, kMmWarps = 16, kMmRows = 16, kMmKeys = 32;
constexpr int kRawPitch = kMmKeys + 1;      // floats per row of a head's score tile
constexpr int kMmMaxHeads = 32;             // raw scores of one (row, key) pair a thread holds while it mixes

__device__ __forceinline__ void ldsm4_t(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ uint32_t pack2(float a, float b) {
  __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}

struct MixedMmaArgs {
  const __nv_bfloat16* q;
  int ldq;
  __nv_bfloat16* out;
  int ldo;
  const __nv_bfloat16* k_pool;
  const __nv_bfloat16* v_pool;
  const int* block_table;
  int bt_width;
  const int* positions;
  const int* tiles;          // [n_tiles][3]: sequence, first row of the step, rows
  int n_q, n_kv, dk, dv;
  float scale;
  const float* temp;
  float cap;
  const float* mix;
  const float* sink;
  int mask, mask_size, page_tokens, n_pages, n_seqs;
  int group_heads;           // heads a block accumulates (the head group of blockIdx.y)
  int* status;
};

// DV16: value width / 16.  HPW: heads of the group a warp accumulates.  QS: the query tile is in shared memory.
// MH: 16 or 32, at least the number of query heads (the raw scores a thread holds while it mixes).
template <int DV16, int HPW, bool QS, int MH>
__global__ void __launch_bounds__(kMmThreads, 1)
attention_mixed_heads_mma_kernel(MixedMmaArgs a) {
  pdl_trigger();
  pdl_wait();
  extern __shared__ __align__(16) unsigned char smem[];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int seq = a.tiles[blockIdx.x * 3], row0 = a.tiles[blockIdx.x * 3 + 1], n_rows = a.tiles[blockIdx.x * 3 + 2];
  const int n_q = a.n_q, n_kv = a.n_kv, dk = a.dk, dv = DV16 * 16;
  const int hg0 = blockIdx.y * a.group_heads, hg1 = min(n_q, hg0 + a.group_heads);
  const int q_pitch = n_q * dk * 2 + 16, k_pitch = dk * 2 + 16, v_pitch = dv * 2 + 16;      // bytes
  unsigned char* q_s = smem;                                             // [16][n_q * dk] (QS only)
  unsigned char* k_s = q_s + (QS ? (size_t)kMmRows * q_pitch : 0);       // [n_kv][32][dk]
  unsigned char* v_s = k_s + (size_t)n_kv * kMmKeys * k_pitch;           // [n_kv][32][dv]
  float* raw_s = reinterpret_cast<float*>(v_s + (size_t)n_kv * kMmKeys * v_pitch);      // [n_q][16][33]
  float* mix_s = raw_s + (size_t)n_q * kMmRows * kRawPitch;              // [group_heads][n_q4], rows 16-byte aligned
  int* page_s = reinterpret_cast<int*>(mix_s + (size_t)a.group_heads * ((n_q + 3) / 4 * 4));      // [32]
  const int n_q4 = (n_q + 3) / 4 * 4;
  if (seq < 0 || seq >= a.n_seqs || n_rows <= 0) return;
  const int p0 = a.positions[row0];
  const int p_last = p0 + n_rows - 1;
  int lo = 0;
  if (a.mask == 1) lo = max(0, p0 - a.mask_size + 1);
  else if (a.mask == 2) lo = (p0 / a.mask_size) * a.mask_size;
  const int group = n_q / n_kv;
  const int* table = a.block_table + (size_t)seq * a.bt_width;
  // Q tile (rows past the tile are zeros) and the group's rows of the mixing matrix
  {
    const int chunks = QS ? n_q * dk / 8 : 0;
    for (int i = tid; i < kMmRows * chunks; i += kMmThreads) {
      const int r = i / chunks, c = i - r * chunks;
      const bool ok = r < n_rows;
      cp_async16_zfill((uint32_t)__cvta_generic_to_shared(q_s + (size_t)r * q_pitch + c * 16),
                       ok ? (const void*)(a.q + (size_t)(row0 + r) * a.ldq + c * 8) : (const void*)a.q, ok);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
    for (int i = tid; i < (hg1 - hg0) * n_q4; i += kMmThreads) {
      const int h = i / n_q4, g = i - h * n_q4;
      mix_s[i] = g < n_q ? (a.mix != nullptr ? a.mix[(size_t)(hg0 + h) * n_q + g] : (hg0 + h == g ? 1.f : 0.f)) : 0.f;
    }
  }
  // accumulators of this warp's heads: head hg0 + warp + 16 * u
  float o[HPW][DV16 * 2][4];
  float m_run[HPW][2], l_run[HPW][2];
#pragma unroll
  for (int u = 0; u < HPW; ++u) {
    const int h = hg0 + warp + kMmWarps * u;
    const bool with_sink = a.sink != nullptr && h < hg1;
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      m_run[u][r] = with_sink ? a.sink[h] : -INFINITY;
      l_run[u][r] = (with_sink && (lane & 3) == 0) ? 1.f : 0.f;       // counted once per row of the quad
    }
#pragma unroll
    for (int n = 0; n < DV16 * 2; ++n)
#pragma unroll
      for (int i = 0; i < 4; ++i) o[u][n][i] = 0.f;
  }
  const uint32_t q_base = (uint32_t)__cvta_generic_to_shared(q_s), k_base = (uint32_t)__cvta_generic_to_shared(k_s),
                 v_base = (uint32_t)__cvta_generic_to_shared(v_s);
  const int mi = lane >> 3;
  for (int j0 = lo; j0 <= p_last; j0 += kMmKeys) {
    __syncthreads();                       // the tile before is used up
    if (tid < kMmKeys) {
      const int pos = j0 + tid;
      int page = -1;
      if (pos <= p_last) {
        const int blk = pos / a.page_tokens;
        page = blk < a.bt_width ? table[blk] : -1;
        if (page < 0 || page >= a.n_pages) {
          set_status(a.status, kBadPage, row0, page);
          page = -1;
        }
      }
      page_s[tid] = page;
    }
    __syncthreads();
    {
      const int kc = dk / 8, vc = dv / 8;
      for (int i = tid; i < n_kv * kMmKeys * kc; i += kMmThreads) {
        const int c = i % kc, row = i / kc;
        const int j = row % kMmKeys, g = row / kMmKeys;
        const int page = page_s[j];
        const bool ok = page >= 0;
        const __nv_bfloat16* src = a.k_pool + (((size_t)(ok ? page : 0) * n_kv + g) * a.page_tokens + (j0 + j) % a.page_tokens) * dk + c * 8;
        cp_async16_zfill(k_base + (uint32_t)((g * kMmKeys + j) * k_pitch + c * 16), src, ok);
      }
      for (int i = tid; i < n_kv * kMmKeys * vc; i += kMmThreads) {
        const int c = i % vc, row = i / vc;
        const int j = row % kMmKeys, g = row / kMmKeys;
        const int page = page_s[j];
        const bool ok = page >= 0;
        const __nv_bfloat16* src = a.v_pool + (((size_t)(ok ? page : 0) * n_kv + g) * a.page_tokens + (j0 + j) % a.page_tokens) * dv + c * 8;
        cp_async16_zfill(v_base + (uint32_t)((g * kMmKeys + j) * v_pitch + c * 16), src, ok);
      }
      asm volatile("cp.async.commit_group;" ::: "memory");
      asm volatile("cp.async.wait_group 0;" ::: "memory");
    }
    __syncthreads();
    // (2) raw scores of every head, the heads dealt to the warps
    for (int h = warp; h < n_q; h += kMmWarps) {
      float s[4][4];
#pragma unroll
      for (int n = 0; n < 4; ++n)
#pragma unroll
        for (int i = 0; i < 4; ++i) s[n][i] = 0.f;
      const uint32_t qh = q_base + (uint32_t)(h * dk * 2), kg = k_base + (uint32_t)((h / group) * kMmKeys * k_pitch);
      // without the query tile in shared memory: this lane's elements of the A fragments, rows g and g + 8
      const __nv_bfloat16* qg0 = a.q + (size_t)(row0 + (lane >> 2)) * a.ldq + (size_t)h * dk + 2 * (lane & 3);
      const __nv_bfloat16* qg1 = qg0 + (size_t)8 * a.ldq;
      const bool ok0 = (lane >> 2) < n_rows, ok1 = (lane >> 2) + 8 < n_rows;
      for (int ks = 0; ks < dk / 16; ++ks) {
        uint32_t a0, a1, a2, a3;
        if (QS) {
          ldsm4(qh + (lane & 15) * q_pitch + (lane >> 4) * 16 + ks * 32, a0, a1, a2, a3);
        } else {
          a0 = ok0 ? __ldg(reinterpret_cast<const uint32_t*>(qg0 + ks * 16)) : 0u;
          a1 = ok1 ? __ldg(reinterpret_cast<const uint32_t*>(qg1 + ks * 16)) : 0u;
          a2 = ok0 ? __ldg(reinterpret_cast<const uint32_t*>(qg0 + ks * 16 + 8)) : 0u;
          a3 = ok1 ? __ldg(reinterpret_cast<const uint32_t*>(qg1 + ks * 16 + 8)) : 0u;
        }
#pragma unroll
        for (int np = 0; np < 2; ++np) {
          uint32_t b0, b1, b2, b3;
          ldsm4(kg + (np * 16 + (lane & 7) + (mi >> 1) * 8) * k_pitch + (mi & 1) * 16 + ks * 32, b0, b1, b2, b3);
          mma16816(s[2 * np], a0, a1, a2, a3, b0, b1);
          mma16816(s[2 * np + 1], a0, a1, a2, a3, b2, b3);
        }
      }
      const float f = a.scale * (a.temp != nullptr ? a.temp[h] : 1.f);
      float* dst = raw_s + (size_t)h * kMmRows * kRawPitch;
#pragma unroll
      for (int n = 0; n < 4; ++n)
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          float v = s[n][i] * f;
          if (a.cap > 0.f) v = a.cap * tanhf(v / a.cap);
          dst[((lane >> 2) + 8 * (i >> 1)) * kRawPitch + n * 8 + 2 * (lane & 3) + (i & 1)] = v;
        }
    }
    __syncthreads();
    // (3) mixing and mask: one (row, key) pair a thread
    {
      const int r = tid >> 5, j = tid & 31;
      const int p = p0 + r, key = j0 + j;
      bool seen = r < n_rows && key <= p;
      if (a.mask == 1) seen = seen && p - key < a.mask_size;
      else if (a.mask == 2) seen = seen && key / a.mask_size == p / a.mask_size;
      float* src = raw_s + r * kRawPitch + j;
      float rv[MH];
#pragma unroll
      for (int g = 0; g < MH; ++g) rv[g] = g < n_q ? src[(size_t)g * kMmRows * kRawPitch] : 0.f;
      for (int h = 0; h < hg1 - hg0; ++h) {
        float v = -INFINITY;
        if (seen) {
          v = 0.f;
          const float4* row = reinterpret_cast<const float4*>(mix_s + h * n_q4);
#pragma unroll
          for (int g4 = 0; g4 < MH / 4; ++g4) {
            if (g4 * 4 < n_q) {
              const float4 w = row[g4];          // the matrix's row is padded with zeros
              v = fmaf(w.x, rv[g4 * 4], v);
              v = fmaf(w.y, rv[g4 * 4 + 1], v);
              v = fmaf(w.z, rv[g4 * 4 + 2], v);
              v = fmaf(w.w, rv[g4 * 4 + 3], v);
            }
          }
        }
        src[(size_t)(hg0 + h) * kMmRows * kRawPitch] = v;      // over the raw score of that head: this thread alone reads this pair
      }
    }
    __syncthreads();
    // (4) softmax and P V for this warp's heads
#pragma unroll
    for (int u = 0; u < HPW; ++u) {
      const int hl = warp + kMmWarps * u;
      if (hg0 + hl >= hg1) continue;
      const float* src = raw_s + (size_t)(hg0 + hl) * kMmRows * kRawPitch;
      float s[4][4];
      float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
      for (int n = 0; n < 4; ++n)
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          s[n][i] = src[((lane >> 2) + 8 * (i >> 1)) * kRawPitch + n * 8 + 2 * (lane & 3) + (i & 1)];
          mx[i >> 1] = fmaxf(mx[i >> 1], s[n][i]);
        }
      float corr[2], m_use[2];
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
        mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
        const float m_new = fmaxf(m_run[u][r], mx[r]);
        corr[r] = m_run[u][r] == -INFINITY ? 0.f : __expf(m_run[u][r] - m_new);
        m_use[r] = m_new == -INFINITY ? 0.f : m_new;
        m_run[u][r] = m_new;
        l_run[u][r] *= corr[r];
      }
#pragma unroll
      for (int n = 0; n < 4; ++n)
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          s[n][i] = __expf(s[n][i] - m_use[i >> 1]);          // exp(-inf) = 0 for unseen keys
          l_run[u][i >> 1] += s[n][i];
        }
#pragma unroll
      for (int n = 0; n < DV16 * 2; ++n) {
        o[u][n][0] *= corr[0];
        o[u][n][1] *= corr[0];
        o[u][n][2] *= corr[1];
        o[u][n][3] *= corr[1];
      }
      const uint32_t vg = v_base + (uint32_t)(((hg0 + hl) / group) * kMmKeys * v_pitch);
#pragma unroll
      for (int ks = 0; ks < 2; ++ks) {            // 16 keys a step
        uint32_t hi[4], lw[4];
#pragma unroll
        for (int x = 0; x < 4; ++x) {
          // a0: rows r, keys 0-7 of the step; a1: rows r + 8; a2, a3: keys 8-15
          const float p0v = s[2 * ks + (x >> 1)][(x & 1) * 2], p1v = s[2 * ks + (x >> 1)][(x & 1) * 2 + 1];
          const float h0 = __bfloat162float(__float2bfloat16_rn(p0v)), h1 = __bfloat162float(__float2bfloat16_rn(p1v));
          hi[x] = pack2(h0, h1);
          lw[x] = pack2(p0v - h0, p1v - h1);
        }
#pragma unroll
        for (int np = 0; np < DV16; ++np) {
          uint32_t b0, b1, b2, b3;
          ldsm4_t(vg + (ks * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * v_pitch + np * 32 + (lane >> 4) * 16, b0, b1, b2, b3);
          mma16816(o[u][2 * np], hi[0], hi[1], hi[2], hi[3], b0, b1);
          mma16816(o[u][2 * np + 1], hi[0], hi[1], hi[2], hi[3], b2, b3);
          mma16816(o[u][2 * np], lw[0], lw[1], lw[2], lw[3], b0, b1);
          mma16816(o[u][2 * np + 1], lw[0], lw[1], lw[2], lw[3], b2, b3);
        }
      }
    }
  }
#pragma unroll
  for (int u = 0; u < HPW; ++u) {
    const int h = hg0 + warp + kMmWarps * u;
    if (h >= hg1) continue;
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      float l = l_run[u][r];
      l += __shfl_xor_sync(0xffffffffu, l, 1);
      l += __shfl_xor_sync(0xffffffffu, l, 2);
      const float inv = l > 0.f ? 1.f / l : 0.f;
      const int row = (lane >> 2) + 8 * r;
      if (row < n_rows) {
        __nv_bfloat16* dst = a.out + (size_t)(row0 + row) * a.ldo + (size_t)h * dv + 2 * (lane & 3);
#pragma unroll
        for (int n = 0; n < DV16 * 2; ++n)
          *reinterpret_cast<__nv_bfloat162*>(dst + n * 8) = __floats2bfloat162_rn(o[u][n][2 * r] * inv, o[u][n][2 * r + 1] * inv);
      }
    }
  }
}

}  // namespace leone

using namespace leone;

// 1 if the tensor-core form takes these sizes; *groups: blocks that share a query tile, *smem: bytes a block needs
extern "C" int leone_attention_mixed_heads_mma_plan(int n_q, int n_kv, int dk, int dv, int* groups, int* smem) {
  if (n_q <= 0 || n_q > kMmMaxHeads || n_kv <= 0 || n_q % n_kv != 0 || dk % 16 != 0 || dk <= 0 ||
      (dv != 32 && dv != 64 && dv != 96 && dv != 128))
    return 0;
  int hg = 1;
  while (((n_q + hg - 1) / hg + kMmWarps - 1) / kMmWarps * dv > 128) ++hg;
  const int gh = (n_q + hg - 1) / hg;
  const long long q_bytes = (long long)kMmRows * (n_q * dk * 2 + 16);
  const long long rest = (long long)n_kv * kMmKeys * (dk * 2 + 16 + dv * 2 + 16) + 4LL * n_q * kMmRows * kRawPitch +
                         4LL * gh * ((n_q + 3) / 4 * 4) + 4 * kMmKeys;
  if (rest > 220 * 1024) return 0;
  *groups = hg;
  // negative: without the query tile (its fragments come from global memory)
  *smem = q_bytes + rest <= 220 * 1024 ? (int)(q_bytes + rest) : -(int)rest;
  return 1;
}

// tiles: int [n_tiles][3] on the device: sequence, first row of the step, rows (at most 16, consecutive positions).
extern "C" int leone_attention_mixed_heads_mma(const void* q, int ldq, void* out, int ldo, const void* k_pool,
                                               const void* v_pool, const int* block_table, int bt_width,
                                               const int* positions, const int* tiles, int n_tiles, int n_q, int n_kv,
                                               int dk, int dv, float scale, const float* temp, float cap, const float* mix,
                                               const float* sink, int mask, int mask_size, int page_tokens, int n_pages,
                                               int n_seqs, int* status, cudaStream_t stream) {
  if (n_tiles <= 0) return 0;
  int groups = 0, smem = 0;
  if (!leone_attention_mixed_heads_mma_plan(n_q, n_kv, dk, dv, &groups, &smem)) return kRefusedSize;
  if ((ldq % 8) != 0 || (ldo % 2) != 0 || ((uintptr_t)q % 16) != 0 || ((uintptr_t)k_pool % 16) != 0 ||
      ((uintptr_t)v_pool % 16) != 0 || ((uintptr_t)out % 4) != 0)
    return kRefusedAlignment;
  if ((mask != 0 && mask_size <= 0) || mask < 0 || mask > 2 || groups > 65535) return kRefusedSize;
  const int gh = (n_q + groups - 1) / groups;
  MixedMmaArgs a{(const __nv_bfloat16*)q, ldq, (__nv_bfloat16*)out, ldo, (const __nv_bfloat16*)k_pool,
                 (const __nv_bfloat16*)v_pool, block_table, bt_width, positions, tiles, n_q, n_kv, dk, dv, scale, temp,
                 cap, mix, sink, mask, mask_size, page_tokens, n_pages, n_seqs, gh, status};
  const int hpw = (gh + kMmWarps - 1) / kMmWarps;
  const bool q_in_smem = smem > 0;
  if (!q_in_smem) smem = -smem;
#define MM1(DV16, HPW, QS, MH)                                                                                       \
  {                                                                                                                  \
    static int configured = 0;                                                                                       \
    if (smem > configured) {                                                                                         \
      cudaFuncSetAttribute(attention_mixed_heads_mma_kernel<DV16, HPW, QS, MH>,                                      \
                           cudaFuncAttributeMaxDynamicSharedMemorySize, smem);                                       \
      configured = smem;                                                                                             \
    }                                                                                                                \
    return launch_kernel(attention_mixed_heads_mma_kernel<DV16, HPW, QS, MH>, dim3(n_tiles, groups),                 \
                         dim3(kMmThreads), (size_t)smem, stream, a);                                                 \
  }
#define MM(DV16, HPW)                                                                                                \
  {                                                                                                                  \
    if (q_in_smem && n_q <= 16) MM1(DV16, HPW, true, 16)                                                             \
    if (q_in_smem) MM1(DV16, HPW, true, 32)                                                                          \
    if (n_q <= 16) MM1(DV16, HPW, false, 16)                                                                         \
    MM1(DV16, HPW, false, 32)                                                                                        \
  }
  if (dv == 128 && hpw == 1) MM(8, 1)
  if (dv == 96 && hpw == 1) MM(6, 1)
  if (dv == 64 && hpw == 1) MM(4, 1)
  if (dv == 64 && hpw == 2) MM(4, 2)
  if (dv == 32 && hpw == 1) MM(2, 1)
  if (dv == 32 && hpw == 2) MM(2, 2)
  if (dv == 32 && hpw <= 4) MM(2, 4)
#undef MM
#undef MM1
  return kRefusedSize;
}
