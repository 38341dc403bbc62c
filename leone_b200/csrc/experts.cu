// Routed experts: router, grouping of (token, choice) pairs by expert, grouped products, combine.
//
//   z = W_router x (an fp32 product of the framework's own),  s = sigmoid(z) or softmax(z),  the `top` largest s are chosen
//   (lowest index first on equal scores); a pair's weight is its s, optionally divided by the sum
//   of the chosen.  The weight multiplies the expert's input (`scale_input`) or its output.
//   Optionally the choice is restricted to the best groups: the experts form `groups` equal runs of
//   neighbours, a run is worth its largest score, only experts of the `keep` best runs (the lowest
//   index among equal ones) can be chosen; and the chosen weights are multiplied by `weight_scale`.
//   expert_e(a) = W_down_e (silu(W_gate_e a) * (W_up_e a)), or, without a gate matrix,
//   expert_e(a) = W_down_e max(W_up_e a, 0)^2
//   out[t] += sum over the token's pairs, in the order of choice.
//
// Nothing is read back by the host: the pairs are counted and placed per expert on the device, and
// the grouped products take a grid that is large enough for any assignment (row tiles that turn out
// to be empty return at once).  A row of the grouped products is computed from its own token only,
// with k ascending, so a token's result does not depend on what else is in the step.
#include "common.cuh"
#include "mma_tile.cuh"

namespace leone {

__device__ __forceinline__ float silu_e(float z) { return z / (1.f + expf(-z)); }

// One warp per token: scores from the router's fp32 logits, then the `top` largest.
__global__ void __launch_bounds__(128)
select_kernel(const float* __restrict__ logits, int ldl, const float* __restrict__ bias,
              const float* __restrict__ correction, int n_tokens, int experts,
              int top, int softmax, int renormalize, int groups, int keep, float weight_scale,
              int* __restrict__ chosen, float* __restrict__ weight) {
  pdl_trigger();      // the next kernel may be scheduled; it waits for this one before it touches data
  pdl_wait();
  extern __shared__ __align__(16) float smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x * 4 + warp;
  if (t >= n_tokens) return;
  float* sc = smem + (size_t)warp * experts;
  const float* row = logits + (size_t)t * ldl;
  for (int e = lane; e < experts; e += 32) sc[e] = row[e] + (bias != nullptr ? bias[e] : 0.f);
  __syncwarp();
  if (softmax == 1) {
    float m = -INFINITY;
    for (int e = lane; e < experts; e += 32) m = fmaxf(m, sc[e]);
    m = warp_max(m);
    float sum = 0.f;
    for (int e = lane; e < experts; e += 32) sum += expf(sc[e] - m);
    sum = warp_sum(sum);
    for (int e = lane; e < experts; e += 32) sc[e] = expf(sc[e] - m) / sum;
  } else if (softmax == 0) {
    for (int e = lane; e < experts; e += 32) sc[e] = 1.f / (1.f + expf(-sc[e]));
  }                              // softmax == 2: the logits themselves are compared
  __syncwarp();
  // a correction moves the scores for the choice only: the weights come from the scores kept aside
  float* plain = smem + (size_t)4 * (experts + groups) + (size_t)warp * experts;
  if (correction != nullptr) {
    for (int e = lane; e < experts; e += 32) {
      plain[e] = sc[e];
      sc[e] += correction[e];
    }
    __syncwarp();
  }
  if (groups > 1 && keep < groups) {
    // what every group is worth, then the groups that are not kept lose their experts
    float* worth = smem + (size_t)4 * experts + (size_t)warp * groups;
    const int per = experts / groups;
    for (int g = lane; g < groups; g += 32) {
      float w = -INFINITY;
      for (int e = g * per; e < (g + 1) * per; ++e) w = fmaxf(w, sc[e]);
      worth[g] = w;
    }
    __syncwarp();
    for (int g = lane; g < groups; g += 32) {
      int better = 0;             // groups that come before this one: worth more, or the same at a lower index
      for (int o = 0; o < groups; ++o) better += (worth[o] > worth[g] || (worth[o] == worth[g] && o < g)) ? 1 : 0;
      if (better >= keep)
        for (int e = g * per; e < (g + 1) * per; ++e) sc[e] = -INFINITY;
    }
    __syncwarp();
  }
  float total = 0.f, first = 0.f;
  for (int j = 0; j < top; ++j) {
    float best = -INFINITY;
    int at = 0x7fffffff;
    for (int e = lane; e < experts; e += 32) {
      const float v = sc[e];
      if (v > best) { best = v; at = e; }          // ascending e: the lowest index of equal scores
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oa = __shfl_xor_sync(0xffffffffu, at, o);
      if (ob > best || (ob == best && oa < at)) { best = ob; at = oa; }
    }
    if (softmax == 2) {          // the weights are the softmax over the chosen logits only
      if (j == 0) first = best;  // the largest of them
      best = expf(best - first);
    } else if (correction != nullptr) {
      best = plain[at];
    }
    if (lane == 0) {
      chosen[(size_t)t * top + j] = at;
      weight[(size_t)t * top + j] = best;
      sc[at] = -INFINITY;
    }
    total += best;
    __syncwarp();
  }
  if (renormalize || softmax == 2)
    for (int j = lane; j < top; j += 32) weight[(size_t)t * top + j] /= total;
  if (weight_scale != 1.f) {
    __syncwarp();
    for (int j = lane; j < top; j += 32) weight[(size_t)t * top + j] *= weight_scale;
  }
}

// One block: counts per expert, their prefix sums, and every pair's row among its expert's.
// offsets: [experts + 1]; order: [pairs] (sorted row -> pair).
__global__ void __launch_bounds__(1024)
group_pairs_kernel(const int* __restrict__ chosen, int pairs, int experts, int* __restrict__ offsets,
                   int* __restrict__ order) {
  pdl_trigger();      // the next kernel may be scheduled; it waits for this one before it touches data
  pdl_wait();
  extern __shared__ int count_s[];      // [experts] counts, then cursors
  for (int e = threadIdx.x; e < experts; e += blockDim.x) count_s[e] = 0;
  __syncthreads();
  for (int p = threadIdx.x; p < pairs; p += blockDim.x) {
    const int e = chosen[p];
    if (e >= 0 && e < experts) atomicAdd(&count_s[e], 1);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int run = 0;
    for (int e = 0; e < experts; ++e) {
      const int c = count_s[e];
      offsets[e] = run;
      count_s[e] = run;
      run += c;
    }
    offsets[experts] = run;
  }
  __syncthreads();
  for (int p = threadIdx.x; p < pairs; p += blockDim.x) {
    const int e = chosen[p];
    if (e >= 0 && e < experts) order[atomicAdd(&count_s[e], 1)] = p;
  }
}

constexpr int GM = 32, GN = 64, GK = 16;

// Which expert and which of its rows the row tile `tile` covers; false if past the last tile.
__device__ __forceinline__ bool find_tile(const int* __restrict__ offsets, int experts, int tile, int& expert,
                                          int& row0, int& row1) {
  int before = 0;
  for (int e = 0; e < experts; ++e) {
    const int b = offsets[e], n = offsets[e + 1] - b;
    const int tiles = (n + GM - 1) / GM;
    if (tile < before + tiles) {
      expert = e;
      row0 = b + (tile - before) * GM;
      row1 = min(row0 + GM, b + n);
      return true;
    }
    before += tiles;
  }
  return false;
}

// act[sorted row, :] = silu(a W_gate_e^T) * (a W_up_e^T) with a = x[token of the pair] (* the pair's
// weight if scale_input).  w_gate, w_up: [experts, ff, width].
template <typename T>
__global__ void __launch_bounds__(256)
experts_gate_up_kernel(const T* __restrict__ x, int ldx, const T* __restrict__ w_gate, const T* __restrict__ w_up,
                       T* __restrict__ act, const int* __restrict__ offsets, const int* __restrict__ order,
                       const float* __restrict__ weight, int experts, int top, int width, int ff,
                       int scale_input) {
  pdl_trigger();      // the next kernel may be scheduled; it waits for this one before it touches data
  pdl_wait();
  __shared__ float As[GK][GM + 4];
  __shared__ float Gs[GK][GN + 4];
  __shared__ float Us[GK][GN + 4];
  int expert, row0, row1;
  if (!find_tile(offsets, experts, blockIdx.y, expert, row0, row1)) return;
  const int tid = threadIdx.x;
  const int n0 = blockIdx.x * GN;
  const int ty = tid >> 4, tx = tid & 15;        // 16 x 16 threads: 2 rows x 4 cols each
  float g[2][4], u[2][4];
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) g[i][j] = u[i][j] = 0.f;
  // loaders: A 32 rows x 16 k = 512 values (2 a thread); W 64 rows x 16 k = 1024 values (4 a thread)
  const int ar = tid >> 3, ak = (tid & 7) * 2;
  const int wr = tid >> 2, wk = (tid & 3) * 4;
  const int a_sorted = row0 + ar;
  const bool a_ok = a_sorted < row1;
  const int pair = a_ok ? order[a_sorted] : 0;
  const float a_scale = (a_ok && scale_input) ? weight[pair] : 1.f;
  const T* a_row = x + (size_t)(pair / top) * ldx;
  const bool w_ok = n0 + wr < ff;
  const T* g_row = w_gate + ((size_t)expert * ff + n0 + wr) * width;
  const T* u_row = w_up + ((size_t)expert * ff + n0 + wr) * width;
  for (int k0 = 0; k0 < width; k0 += GK) {
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int k = k0 + ak + i;
      As[ak + i][ar] = (a_ok && k < width) ? to_float<T>(a_row[k]) * a_scale : 0.f;
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int k = k0 + wk + i;
      const bool ok = w_ok && k < width;
      Gs[wk + i][wr] = (ok && w_gate != nullptr) ? to_float<T>(g_row[k]) : 0.f;
      Us[wk + i][wr] = ok ? to_float<T>(u_row[k]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < GK; ++k) {
      float a[2], bg[4], bu[4];
#pragma unroll
      for (int i = 0; i < 2; ++i) a[i] = As[k][ty * 2 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        bg[j] = Gs[k][tx * 4 + j];
        bu[j] = Us[k][tx * 4 + j];
      }
#pragma unroll
      for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          g[i][j] = fmaf(a[i], bg[j], g[i][j]);
          u[i][j] = fmaf(a[i], bu[j], u[i][j]);
        }
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int r = row0 + ty * 2 + i;
    if (r >= row1) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n >= ff) continue;
      const float uu = round_to<T>(u[i][j]);
      // without a gate matrix the expert is ungated: the squared ReLU of its one product
      act[(size_t)r * ff + n] = from_float<T>(w_gate != nullptr ? silu_e(round_to<T>(g[i][j])) * uu
                                                                : fmaxf(uu, 0.f) * fmaxf(uu, 0.f));
    }
  }
}

// pair_out[pair of the sorted row, :] = act[sorted row, :] W_down_e^T (* the pair's weight unless
// scale_input).  w_down: [experts, width, ff]; pair_out fp32 [pairs, width].
template <typename T>
__global__ void __launch_bounds__(256)
experts_down_kernel(const T* __restrict__ act, const T* __restrict__ w_down, float* __restrict__ pair_out,
                    const int* __restrict__ offsets, const int* __restrict__ order,
                    const float* __restrict__ weight, int experts, int width, int ff, int scale_input) {
  pdl_trigger();      // the next kernel may be scheduled; it waits for this one before it touches data
  pdl_wait();
  __shared__ float As[GK][GM + 4];
  __shared__ float Ws[GK][GN + 4];
  int expert, row0, row1;
  if (!find_tile(offsets, experts, blockIdx.y, expert, row0, row1)) return;
  const int tid = threadIdx.x;
  const int n0 = blockIdx.x * GN;
  const int ty = tid >> 4, tx = tid & 15;
  float acc[2][4];
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
  const int ar = tid >> 3, ak = (tid & 7) * 2;
  const int wr = tid >> 2, wk = (tid & 3) * 4;
  const bool a_ok = row0 + ar < row1;
  const T* a_row = act + (size_t)(row0 + ar) * ff;
  const bool w_ok = n0 + wr < width;
  const T* w_row = w_down + ((size_t)expert * width + n0 + wr) * ff;
  for (int k0 = 0; k0 < ff; k0 += GK) {
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int k = k0 + ak + i;
      As[ak + i][ar] = (a_ok && k < ff) ? to_float<T>(a_row[k]) : 0.f;
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int k = k0 + wk + i;
      Ws[wk + i][wr] = (w_ok && k < ff) ? to_float<T>(w_row[k]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < GK; ++k) {
      float a[2], b[4];
#pragma unroll
      for (int i = 0; i < 2; ++i) a[i] = As[k][ty * 2 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = Ws[k][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int r = row0 + ty * 2 + i;
    if (r >= row1) continue;
    const int pair = order[r];
    const float f = scale_input ? 1.f : weight[pair];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n < width) pair_out[(size_t)pair * width + n] = acc[i][j] * f;
    }
  }
}

// hidden[t, :] (+)= sum_j pair_out[t * top + j, :], j ascending; top < 0: written, not added (|top| pairs).
// A pair whose choice is past the last expert is an identity expert and contributes weight * x[t, :] instead
// (x null: there are none).
template <typename T>
__global__ void experts_combine_kernel(float* __restrict__ hidden, const float* __restrict__ pair_out,
                                       long long total, int width, int top, const T* __restrict__ x, int ldx,
                                       const int* __restrict__ chosen, const float* __restrict__ weight, int experts) {
  pdl_trigger();      // the next kernel may be scheduled; it waits for this one before it touches data
  pdl_wait();
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const long long t = i / width;
    const int c = (int)(i - t * width);
    float sum = 0.f;
    const int n = top < 0 ? -top : top;
    for (int j = 0; j < n; ++j) {
      const size_t p = (size_t)t * n + j;
      if (x != nullptr && chosen[p] >= experts) sum += weight[p] * to_float<T>(x[(size_t)t * ldx + c]);
      else sum += pair_out[p * width + c];
    }
    hidden[i] = top < 0 ? sum : hidden[i] + sum;
  }
}


// ---- the grouped products on tensor cores (bfloat16) ----------------------------------------------
// A row tile of 64 sorted pairs of one expert times 64 output columns; four warps of 16 rows each;
// operands come through a three-stage cp.async ring in shared memory (rows of 32 k-values, padded
// so that ldmatrix finds eight rows in eight different banks).  NB = 2: gate and up together, with
// the activation in the epilogue; NB = 1: the down product.  Because the products are linear, the
// pair's weight multiplies the fp32 sums in the epilogue instead of the gathered input rows.
__device__ __forceinline__ bool find_tile_m(const int* __restrict__ offsets, int experts, int tile, int& expert,
                                            int& row0, int& row1) {
  int before = 0;
  for (int e = 0; e < experts; ++e) {
    const int b = offsets[e], n = offsets[e + 1] - b;
    const int tiles = (n + TM - 1) / TM;
    if (tile < before + tiles) {
      expert = e;
      row0 = b + (tile - before) * TM;
      row1 = min(row0 + TM, b + n);
      return true;
    }
    before += tiles;
  }
  return false;
}

__global__ void __launch_bounds__(128)
experts_gate_up_mma_kernel(const __nv_bfloat16* __restrict__ x, int ldx, const __nv_bfloat16* __restrict__ w_gate,
                           const __nv_bfloat16* __restrict__ w_up, __nv_bfloat16* __restrict__ act,
                           const int* __restrict__ offsets, const int* __restrict__ order,
                           const float* __restrict__ weight, int experts, int top, int width, int ff,
                           int scale_input) {
  pdl_trigger();      // the next kernel may be scheduled; it waits for this one before it touches data
  pdl_wait();
  extern __shared__ __align__(16) unsigned char smem_m[];
  __shared__ int a_index[TM];
  __shared__ float a_weight[TM];
  int expert, row0, row1;
  if (!find_tile_m(offsets, experts, blockIdx.y, expert, row0, row1)) return;
  const int n0 = blockIdx.x * TN;
  for (int r = threadIdx.x; r < TM; r += 128) {
    const bool ok = row0 + r < row1;
    const int pair = ok ? order[row0 + r] : 0;
    a_index[r] = ok ? pair / top : -1;
    a_weight[r] = (ok && scale_input) ? weight[pair] : 1.f;
  }
  __syncthreads();
  float acc[2][2][4][4];
#pragma unroll
  for (int m = 0; m < 2; ++m)
#pragma unroll
    for (int mt = 0; mt < 2; ++mt)
#pragma unroll
      for (int n = 0; n < 4; ++n)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[m][mt][n][i] = 0.f;
  grouped_mainloop<2>(smem_m, x, a_index, ldx, w_gate + ((size_t)expert * ff + n0) * width,
                      w_up + ((size_t)expert * ff + n0) * width, min(TN, ff - n0), width, acc);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, tq = lane & 3;
  const int wm = warp >> 1, wn = warp & 1;
#pragma unroll
  for (int mt = 0; mt < 2; ++mt)
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int r = wm * 32 + mt * 16 + g + 8 * i;
      if (row0 + r >= row1) continue;
      const float w = a_weight[r];
#pragma unroll
      for (int n = 0; n < 4; ++n) {
        const int col = n0 + wn * 32 + n * 8 + 2 * tq;
        if (col >= ff) continue;
        float v[2];
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          const float gg = round_to<__nv_bfloat16>(acc[0][mt][n][2 * i + j] * w);
          const float uu = round_to<__nv_bfloat16>(acc[1][mt][n][2 * i + j] * w);
          v[j] = silu_e(gg) * uu;
        }
        *reinterpret_cast<__nv_bfloat162*>(act + (size_t)(row0 + r) * ff + col) = __floats2bfloat162_rn(v[0], v[1]);
      }
    }
}

// The ungated expert's first product with the squared ReLU in the epilogue.
__global__ void __launch_bounds__(128)
experts_up_mma_kernel(const __nv_bfloat16* __restrict__ x, int ldx, const __nv_bfloat16* __restrict__ w_up,
                      __nv_bfloat16* __restrict__ act, const int* __restrict__ offsets,
                      const int* __restrict__ order, int experts, int top, int width, int ff) {
  pdl_trigger();      // the next kernel may be scheduled; it waits for this one before it touches data
  pdl_wait();
  extern __shared__ __align__(16) unsigned char smem_m[];
  __shared__ int a_index[TM];
  int expert, row0, row1;
  if (!find_tile_m(offsets, experts, blockIdx.y, expert, row0, row1)) return;
  const int n0 = blockIdx.x * TN;
  for (int r = threadIdx.x; r < TM; r += 128) {
    const bool ok = row0 + r < row1;
    a_index[r] = ok ? order[row0 + r] / top : -1;
  }
  __syncthreads();
  float acc[1][2][4][4];
#pragma unroll
  for (int mt = 0; mt < 2; ++mt)
#pragma unroll
    for (int n = 0; n < 4; ++n)
#pragma unroll
      for (int i = 0; i < 4; ++i) acc[0][mt][n][i] = 0.f;
  grouped_mainloop<1>(smem_m, x, a_index, ldx, w_up + ((size_t)expert * ff + n0) * width, nullptr,
                      min(TN, ff - n0), width, acc);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, tq = lane & 3;
  const int wm = warp >> 1, wn = warp & 1;
#pragma unroll
  for (int mt = 0; mt < 2; ++mt)
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int r = wm * 32 + mt * 16 + g + 8 * i;
      if (row0 + r >= row1) continue;
#pragma unroll
      for (int n = 0; n < 4; ++n) {
        const int col = n0 + wn * 32 + n * 8 + 2 * tq;
        if (col >= ff) continue;
        float v[2];
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          const float uu = fmaxf(round_to<__nv_bfloat16>(acc[0][mt][n][2 * i + j]), 0.f);
          v[j] = uu * uu;
        }
        *reinterpret_cast<__nv_bfloat162*>(act + (size_t)(row0 + r) * ff + col) = __floats2bfloat162_rn(v[0], v[1]);
      }
    }
}

__global__ void __launch_bounds__(128)
experts_down_mma_kernel(const __nv_bfloat16* __restrict__ act, const __nv_bfloat16* __restrict__ w_down,
                        float* __restrict__ pair_out, const int* __restrict__ offsets,
                        const int* __restrict__ order, const float* __restrict__ weight, int experts, int width,
                        int ff, int scale_input) {
  pdl_trigger();      // the next kernel may be scheduled; it waits for this one before it touches data
  pdl_wait();
  extern __shared__ __align__(16) unsigned char smem_m[];
  __shared__ int a_index[TM];
  __shared__ int a_pair[TM];
  int expert, row0, row1;
  if (!find_tile_m(offsets, experts, blockIdx.y, expert, row0, row1)) return;
  const int n0 = blockIdx.x * TN;
  for (int r = threadIdx.x; r < TM; r += 128) {
    const bool ok = row0 + r < row1;
    a_index[r] = ok ? row0 + r : -1;
    a_pair[r] = ok ? order[row0 + r] : 0;
  }
  __syncthreads();
  float acc[1][2][4][4];
#pragma unroll
  for (int mt = 0; mt < 2; ++mt)
#pragma unroll
    for (int n = 0; n < 4; ++n)
#pragma unroll
      for (int i = 0; i < 4; ++i) acc[0][mt][n][i] = 0.f;
  grouped_mainloop<1>(smem_m, act, a_index, ff, w_down + ((size_t)expert * width + n0) * ff, nullptr,
                      min(TN, width - n0), ff, acc);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, tq = lane & 3;
  const int wm = warp >> 1, wn = warp & 1;
#pragma unroll
  for (int mt = 0; mt < 2; ++mt)
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int r = wm * 32 + mt * 16 + g + 8 * i;
      if (row0 + r >= row1) continue;
      const int pair = a_pair[r];
      const float f = scale_input ? 1.f : weight[pair];
#pragma unroll
      for (int n = 0; n < 4; ++n) {
        const int col = n0 + wn * 32 + n * 8 + 2 * tq;
        if (col >= width) continue;
        *reinterpret_cast<float2*>(pair_out + (size_t)pair * width + col) =
            make_float2(acc[0][mt][n][2 * i] * f, acc[0][mt][n][2 * i + 1] * f);
      }
    }
}

}  // namespace leone

using namespace leone;

// logits: fp32 [n_tokens, ldl] (the router's product); chosen, weight: [n_tokens * top].
// groups <= 1 (or keep == groups): every expert can be chosen.
// softmax: 0 sigmoid scores, 1 softmax over all experts, 2 the logits are ranked and the weights are the
// softmax over the chosen ones.  bias: fp32 [experts] added to the logits first, or null.  correction: fp32
// [experts] added to the scores for the choice (and the groups' worth) only, or null: the weights are the
// scores without it.
extern "C" int leone_experts_select(const float* logits, int ldl, const float* bias, const float* correction,
                                    int n_tokens, int experts, int top,
                                    int softmax, int renormalize, int groups, int keep, float weight_scale, int* chosen,
                                    float* weight, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (experts <= 0 || top <= 0 || top > experts || experts > 2048 || ldl < experts) return kRefusedSize;
  if (groups < 1) groups = 1;
  if (experts % groups != 0 || keep < 1 || keep > groups || top > experts / groups * keep) return kRefusedSize;
  if (correction != nullptr && softmax == 2) return kRefusedSize;      // ranked logits have no scores to keep aside
  launch_kernel(select_kernel, dim3((n_tokens + 3) / 4), dim3(128), sizeof(float) * 4 * (size_t)(2 * experts + groups), stream,
      logits, ldl, bias, correction, n_tokens, experts, top, softmax, renormalize, groups, keep, weight_scale, chosen, weight);
  return launch_result();
}

// w_gate null: ungated experts (see the top of the file).  identity: choices `experts .. experts + identity - 1`
// are experts without tensors whose output is their input (weighted at the output).  fresh: hidden is
// written, not added to.
// x: [n_tokens, ldx]; chosen, weight: [n_tokens * top]; scratch: offsets int [experts + 1], order int
// [pairs], act [pairs, ff] in the run dtype, pair_out fp32 [pairs, width]; hidden fp32 [n_tokens, width].
extern "C" int leone_experts_forward(int dtype, const void* x, int ldx, const void* w_gate, const void* w_up,
                                     const void* w_down, const int* chosen, const float* weight, int n_tokens,
                                     int width, int ff, int experts, int top, int scale_input, int* offsets,
                                     int* order, void* act, float* pair_out, float* hidden, int tensor_cores,
                                     int identity, int fresh, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (identity < 0 || (identity > 0 && scale_input)) return kRefusedSize;
  if (width <= 0 || ff <= 0 || experts <= 0 || top <= 0 || experts > 8192) return kRefusedSize;
  if (w_gate == nullptr && scale_input) return kRefusedSize;      // an ungated expert is weighted at its output
  const long long pairs = (long long)n_tokens * top;
  if (pairs > (1 << 30)) return kRefusedSize;
  launch_kernel(group_pairs_kernel, dim3(1), dim3(1024), sizeof(int) * (size_t)experts, stream, chosen, (int)pairs, experts, offsets, order);
  const int combine_top = fresh ? -top : top;
  if (tensor_cores && dtype == 1 && width % 8 == 0 && ff % 8 == 0 && ldx % 8 == 0) {
    const long long tiles = (pairs + TM - 1) / TM + (experts < pairs ? experts : pairs);
    if (tiles > 65535) return kRefusedSize;
    const size_t smem_up = (size_t)TSTAGES * (TM + 2 * TN) * TPITCH, smem_down = (size_t)TSTAGES * (TM + TN) * TPITCH;
    static bool configured = false;
    if (!configured) {
      cudaFuncSetAttribute(experts_gate_up_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_up);
      cudaFuncSetAttribute(experts_down_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_down);
      cudaFuncSetAttribute(experts_up_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_down);
      configured = true;
    }
    if (w_gate == nullptr)
      launch_kernel(experts_up_mma_kernel, dim3((ff + TN - 1) / TN, (unsigned)tiles), dim3(128), smem_down, stream,
          (const __nv_bfloat16*)x, ldx, (const __nv_bfloat16*)w_up, (__nv_bfloat16*)act, offsets, order, experts, top,
          width, ff);
    else
    launch_kernel(experts_gate_up_mma_kernel, dim3((ff + TN - 1) / TN, (unsigned)tiles), dim3(128), smem_up, stream, 
        (const __nv_bfloat16*)x, ldx, (const __nv_bfloat16*)w_gate, (const __nv_bfloat16*)w_up, (__nv_bfloat16*)act,
        offsets, order, weight, experts, top, width, ff, scale_input);
    launch_kernel(experts_down_mma_kernel, dim3((width + TN - 1) / TN, (unsigned)tiles), dim3(128), smem_down, stream, 
        (const __nv_bfloat16*)act, (const __nv_bfloat16*)w_down, pair_out, offsets, order, weight, experts, width, ff,
        scale_input);
    const long long total = (long long)n_tokens * width;
    const long long blocks = (total + 255) / 256;
    launch_kernel(experts_combine_kernel<__nv_bfloat16>, dim3((unsigned)(blocks < 148 * 8 ? blocks : 148 * 8)), dim3(256), 0, stream,
                  hidden, pair_out, total, width, combine_top, identity > 0 ? (const __nv_bfloat16*)x : nullptr, ldx, chosen,
                  weight, experts);
    return launch_result();
  }
  // every expert may end with a partly filled tile
  const long long max_tiles = (pairs + GM - 1) / GM + (experts < pairs ? experts : pairs);
  if (max_tiles > 65535) return kRefusedSize;
  const dim3 grid_up((ff + GN - 1) / GN, (unsigned)max_tiles), grid_down((width + GN - 1) / GN, (unsigned)max_tiles);
  if (dtype == 0) {
    launch_kernel(experts_gate_up_kernel<float>, grid_up, dim3(256), 0, stream, (const float*)x, ldx, (const float*)w_gate,
                                                               (const float*)w_up, (float*)act, offsets, order,
                                                               weight, experts, top, width, ff, scale_input);
    launch_kernel(experts_down_kernel<float>, grid_down, dim3(256), 0, stream, (const float*)act, (const float*)w_down, pair_out,
                                                              offsets, order, weight, experts, width, ff,
                                                              scale_input);
  } else if (dtype == 1) {
    launch_kernel(experts_gate_up_kernel<__nv_bfloat16>, grid_up, dim3(256), 0, stream, 
        (const __nv_bfloat16*)x, ldx, (const __nv_bfloat16*)w_gate, (const __nv_bfloat16*)w_up,
        (__nv_bfloat16*)act, offsets, order, weight, experts, top, width, ff, scale_input);
    launch_kernel(experts_down_kernel<__nv_bfloat16>, grid_down, dim3(256), 0, stream, 
        (const __nv_bfloat16*)act, (const __nv_bfloat16*)w_down, pair_out, offsets, order, weight, experts, width,
        ff, scale_input);
  } else {
    return kRefusedDtype;
  }
  const long long total = (long long)n_tokens * width;
  const long long blocks = (total + 255) / 256;
  const dim3 cgrid((unsigned)(blocks < 148 * 8 ? blocks : 148 * 8));
  if (dtype == 0)
    launch_kernel(experts_combine_kernel<float>, cgrid, dim3(256), 0, stream, hidden, pair_out, total, width, combine_top,
                  identity > 0 ? (const float*)x : nullptr, ldx, chosen, weight, experts);
  else
    launch_kernel(experts_combine_kernel<__nv_bfloat16>, cgrid, dim3(256), 0, stream, hidden, pair_out, total, width,
                  combine_top, identity > 0 ? (const __nv_bfloat16*)x : nullptr, ldx, chosen, weight, experts);
  return launch_result();
}
