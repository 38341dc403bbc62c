// Small kernels shared by several parts: two RMS norms of the same rows in one pass, the squared
// ReLU, a product batched over heads, the norm of a sublayer's output added to the residual stream,
// elementwise gates.
#include "common.cuh"
#include "mma_tile.cuh"

namespace leone {

// out_a = x * r * w_a, out_b = x * r * w_b with r = 1/sqrt(mean(x^2) + eps): both norms of a layer
// whose branches read the same residual rows share the row's sum of squares.
template <typename T, typename TW>
__global__ void __launch_bounds__(256)
rms_norm_pair_kernel(const float* __restrict__ x, const TW* __restrict__ w_a, const TW* __restrict__ w_b,
                     T* __restrict__ out_a, T* __restrict__ out_b, int width, float eps) {
  pdl_trigger();      // the next kernel may be scheduled; it waits for this one before it touches data
  pdl_wait();
  __shared__ float scratch[33];
  const size_t base = (size_t)blockIdx.x * width;
  float ss = 0.f;
  for (int c = threadIdx.x; c < width; c += blockDim.x) ss = fmaf(x[base + c], x[base + c], ss);
  ss = block_sum(ss, scratch);
  const float r = 1.f / sqrtf(ss / (float)width + eps);
  for (int c = threadIdx.x; c < width; c += blockDim.x) {
    const float v = x[base + c] * r;
    out_a[base + c] = from_float<T>(v * to_float<TW>(w_a[c]));
    out_b[base + c] = from_float<T>(v * to_float<TW>(w_b[c]));
  }
}

template <typename T>
__global__ void relu_squared_kernel(T* __restrict__ x, long long n) {
  pdl_trigger();      // the next kernel may be scheduled; it waits for this one before it touches data
  pdl_wait();
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const float v = fmaxf(to_float<T>(x[i]), 0.f);
    x[i] = from_float<T>(v * v);
  }
}

// C_b[M, N] = A_b[M, K] W_b[N, K]^T for b < batch, fp32 accumulation with k ascending; the three
// operands of batch b start b * (their batch stride) elements after those of batch 0.
constexpr int BM = 64, BN = 64, BK = 16;

template <typename T>
__global__ void __launch_bounds__(256)
gemm_batched_kernel(const T* __restrict__ A, const T* __restrict__ W, T* __restrict__ C, int M, int N, int K,
                    int lda, int ldw, int ldc, long long a_bs, long long w_bs, long long c_bs) {
  pdl_trigger();      // the next kernel may be scheduled; it waits for this one before it touches data
  pdl_wait();
  __shared__ float As[BK][BM + 4];
  __shared__ float Ws[BK][BN + 4];
  A += (size_t)blockIdx.z * a_bs;
  W += (size_t)blockIdx.z * w_bs;
  C += (size_t)blockIdx.z * c_bs;
  const int tid = threadIdx.x;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  const int ty = tid >> 4, tx = tid & 15;
  const int lr = tid >> 2, lk = (tid & 3) * 4;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
  const T* a_row = A + (size_t)(m0 + lr) * lda;
  const T* w_row = W + (size_t)(n0 + lr) * ldw;
  const bool a_ok = m0 + lr < M, w_ok = n0 + lr < N;
  for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int k = k0 + lk + i;
      As[lk + i][lr] = (a_ok && k < K) ? to_float<T>(a_row[k]) : 0.f;
      Ws[lk + i][lr] = (w_ok && k < K) ? to_float<T>(w_row[k]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < BK; ++k) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = As[k][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = Ws[k][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int m = m0 + ty * 4 + i;
    if (m >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n < N) C[(size_t)m * ldc + n] = from_float<T>(acc[i][j]);
    }
  }
}

// The same product on tensor cores (bfloat16): a block owns 64 rows x 64 columns of one batch.
__global__ void __launch_bounds__(128)
gemm_batched_mma_kernel(const __nv_bfloat16* __restrict__ A, const __nv_bfloat16* __restrict__ W,
                        __nv_bfloat16* __restrict__ C, int M, int N, int K, int lda, int ldw, int ldc, long long a_bs,
                        long long w_bs, long long c_bs) {
  pdl_trigger();      // the next kernel may be scheduled; it waits for this one before it touches data
  pdl_wait();
  extern __shared__ __align__(16) unsigned char smem_m[];
  __shared__ int a_index[TM];
  A += (size_t)blockIdx.z * a_bs;
  W += (size_t)blockIdx.z * w_bs;
  C += (size_t)blockIdx.z * c_bs;
  const int m0 = blockIdx.y * TM, n0 = blockIdx.x * TN;
  for (int r = threadIdx.x; r < TM; r += 128) a_index[r] = m0 + r < M ? m0 + r : -1;
  __syncthreads();
  float acc[1][2][4][4];
#pragma unroll
  for (int mt = 0; mt < 2; ++mt)
#pragma unroll
    for (int n = 0; n < 4; ++n)
#pragma unroll
      for (int i = 0; i < 4; ++i) acc[0][mt][n][i] = 0.f;
  grouped_mainloop<1>(smem_m, A, a_index, lda, W + (size_t)n0 * ldw, nullptr, min(TN, N - n0), K, acc, ldw);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, tq = lane & 3;
  const int wm = warp >> 1, wn = warp & 1;
#pragma unroll
  for (int mt = 0; mt < 2; ++mt)
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int m = m0 + wm * 32 + mt * 16 + g + 8 * i;
      if (m >= M) continue;
#pragma unroll
      for (int n = 0; n < 4; ++n) {
        const int col = n0 + wn * 32 + n * 8 + 2 * tq;
        if (col >= N) continue;
        *reinterpret_cast<__nv_bfloat162*>(C + (size_t)m * ldc + col) =
            __floats2bfloat162_rn(acc[0][mt][n][2 * i], acc[0][mt][n][2 * i + 1]);
      }
    }
}


// dst[t, :] (+)= coef * (a[t, :] / rms(a[t, :]) * w_a  [+ b[t, :] / rms(b[t, :]) * w_b]), every norm over its own
// row with eps inside the root.  The norm of a sublayer's *output*, added to the residual stream (or
// written, if not `accumulate`); with two sources, the normed outputs of two branches side by side.
// `rounded`: also the new dst row in the run dtype, for the next reader of the stream.  `w_then`: the
// combination is itself RMS-normed with that weight before it is added (a norm on the sum of normed branches).
template <typename TW, typename TR>
__global__ void __launch_bounds__(256)
rms_norm_add_kernel(float* __restrict__ dst, const float* __restrict__ a, const TW* __restrict__ w_a,
                    const float* __restrict__ b, const TW* __restrict__ w_b, int width, float coef, float eps,
                    int accumulate, TR* __restrict__ rounded, const TW* __restrict__ w_then) {
  pdl_trigger();
  pdl_wait();
  __shared__ float scratch[33];
  extern __shared__ float row_s[];      // [width], only with w_then
  const size_t base = (size_t)blockIdx.x * width;
  float sa = 0.f, sb = 0.f;
  for (int c = threadIdx.x; c < width; c += blockDim.x) {
    sa = fmaf(a[base + c], a[base + c], sa);
    if (b != nullptr) sb = fmaf(b[base + c], b[base + c], sb);
  }
  sa = block_sum(sa, scratch);
  const float ra = 1.f / sqrtf(sa / (float)width + eps);
  float rb = 0.f;
  if (b != nullptr) {
    sb = block_sum(sb, scratch);
    rb = 1.f / sqrtf(sb / (float)width + eps);
  }
  float rt = 1.f;
  if (w_then != nullptr) {
    // the combined row is itself normed (with w_then) before it is added: a second pass over the row in shared memory
    float st = 0.f;
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
      float v = a[base + c] * ra * to_float<TW>(w_a[c]);
      if (b != nullptr) v += b[base + c] * rb * to_float<TW>(w_b[c]);
      v *= coef;
      row_s[c] = v;
      st = fmaf(v, v, st);
    }
    st = block_sum(st, scratch);
    rt = 1.f / sqrtf(st / (float)width + eps);
  }
  for (int c = threadIdx.x; c < width; c += blockDim.x) {
    float v;
    if (w_then != nullptr) {
      v = row_s[c] * rt * to_float<TW>(w_then[c]);
    } else {
      v = a[base + c] * ra * to_float<TW>(w_a[c]);
      if (b != nullptr) v += b[base + c] * rb * to_float<TW>(w_b[c]);
      v *= coef;
    }
    if (accumulate) v += dst[base + c];
    dst[base + c] = v;
    if (rounded != nullptr) rounded[base + c] = from_float<TR>(v);
  }
}

// a[t, c] *= act(gate[t, c]): act 0 sigmoid, 1 silu.
template <typename T>
__global__ void __launch_bounds__(256)
gate_rows_kernel(T* __restrict__ a, int lda, const T* __restrict__ gate, int ldg, int n_rows, int cols, int act) {
  pdl_trigger();
  pdl_wait();
  const long long total = (long long)n_rows * cols;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long t = i / cols;
    const int c = (int)(i - t * cols);
    const float z = to_float<T>(gate[t * ldg + c]);
    const float sg = 1.f / (1.f + expf(-z));
    a[t * lda + c] = from_float<T>(to_float<T>(a[t * lda + c]) * (act == 1 ? z * sg : sg));
  }
}

// out[t, c] = gelu_tanh(z[t, c]) * rows[t, off + c]: a projection's fp32 result gates a slice of a
// per-token row.  gelu_tanh(z) = z/2 (1 + tanh(sqrt(2/pi) (z + 0.044715 z^3))).
template <typename T>
__global__ void __launch_bounds__(256)
gelu_gate_kernel(const float* __restrict__ z, int ldz, const float* __restrict__ rows, int ldr, int off,
                 T* __restrict__ out, int ldo, int n_rows, int cols) {
  pdl_trigger();
  pdl_wait();
  const long long total = (long long)n_rows * cols;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long t = i / cols;
    const int c = (int)(i - t * cols);
    const float v = z[t * ldz + c];
    const float g = 0.5f * v * (1.f + tanhf(0.7978845608028654f * (v + 0.044715f * v * v * v)));
    out[t * ldo + c] = from_float<T>(g * rows[t * ldr + off + c]);
  }
}

}  // namespace leone

using namespace leone;

extern "C" void leone_mixers_set_pdl(int enabled) { pdl_flag() = enabled ? 1 : 0; }

extern "C" int leone_rms_norm_pair(const float* x, const void* w_a, const void* w_b, int w_dtype, void* out_a,
                                   void* out_b, int out_dtype, int n, int width, float eps, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (width <= 0) return kRefusedSize;
#define NP(T, TW)                                                                                            \
  launch_kernel(rms_norm_pair_kernel<T, TW>, dim3(n), dim3(256), 0, stream, x, (const TW*)w_a, (const TW*)w_b, (T*)out_a, (T*)out_b, \
                                                     width, eps)
  if (out_dtype == 0 && w_dtype == 0) NP(float, float);
  else if (out_dtype == 1 && w_dtype == 0) NP(__nv_bfloat16, float);
  else if (out_dtype == 1 && w_dtype == 1) NP(__nv_bfloat16, __nv_bfloat16);
  else if (out_dtype == 0 && w_dtype == 1) NP(float, __nv_bfloat16);
  else return kRefusedDtype;
#undef NP
  return launch_result();
}

extern "C" int leone_relu_squared(int dtype, void* x, long long n, cudaStream_t stream) {
  if (n <= 0) return 0;
  const long long want = (n + 255) / 256;
  const unsigned blocks = (unsigned)(want < 148 * 16 ? want : 148 * 16);
  if (dtype == 0) launch_kernel(relu_squared_kernel<float>, dim3(blocks), dim3(256), 0, stream, (float*)x, n);
  else if (dtype == 1) launch_kernel(relu_squared_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, stream, (__nv_bfloat16*)x, n);
  else return kRefusedDtype;
  return launch_result();
}

extern "C" int leone_gemm_batched(int dtype, const void* a, const void* w, void* c, int m, int n, int k, int lda,
                                  int ldw, int ldc, long long a_bs, long long w_bs, long long c_bs, int batch,
                                  cudaStream_t stream) {
  if (m <= 0 || n <= 0 || batch <= 0) return 0;
  if (k <= 0 || lda < k || ldw < k || ldc < n || batch > 65535) return kRefusedSize;
  const dim3 grid((n + BN - 1) / BN, (m + BM - 1) / BM, batch);
  if (grid.y > 65535) return kRefusedSize;
  // bfloat16 with 16-byte aligned rows: tensor cores
  if (dtype == 1 && k % 8 == 0 && n % 2 == 0 && lda % 8 == 0 && ldw % 8 == 0 && ldc % 2 == 0 && a_bs % 8 == 0 &&
      w_bs % 8 == 0 && c_bs % 2 == 0 && ((uintptr_t)a % 16) == 0 && ((uintptr_t)w % 16) == 0 && ((uintptr_t)c % 4) == 0) {
    const dim3 tgrid((n + TN - 1) / TN, (m + TM - 1) / TM, batch);
    if (tgrid.y > 65535) return kRefusedSize;
    const size_t smem = (size_t)TSTAGES * (TM + TN) * TPITCH;
    static bool configured = false;
    if (!configured) {
      cudaFuncSetAttribute(gemm_batched_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      configured = true;
    }
    launch_kernel(gemm_batched_mma_kernel, tgrid, dim3(128), smem, stream, (const __nv_bfloat16*)a, (const __nv_bfloat16*)w,
                                                          (__nv_bfloat16*)c, m, n, k, lda, ldw, ldc, a_bs, w_bs, c_bs);
    return launch_result();
  }
  if (dtype == 0)
    launch_kernel(gemm_batched_kernel<float>, grid, dim3(256), 0, stream, (const float*)a, (const float*)w, (float*)c, m, n, k, lda,
                                                         ldw, ldc, a_bs, w_bs, c_bs);
  else if (dtype == 1)
    launch_kernel(gemm_batched_kernel<__nv_bfloat16>, grid, dim3(256), 0, stream, (const __nv_bfloat16*)a, (const __nv_bfloat16*)w,
                                                                 (__nv_bfloat16*)c, m, n, k, lda, ldw, ldc, a_bs,
                                                                 w_bs, c_bs);
  else
    return kRefusedDtype;
  return launch_result();
}

// dst: fp32 [n, width]; a, b: fp32 [n, width] (b and w_b may be null); w in `w_dtype`; rounded: [n, width] in
// `rounded_dtype`, or null; w_then: [width] in `w_dtype`, or null (width at most 12,000 with it).
extern "C" int leone_rms_norm_add(float* dst, const float* a, const void* w_a, const float* b, const void* w_b,
                                  int w_dtype, int n, int width, float coef, float eps, int accumulate, void* rounded,
                                  int rounded_dtype, const void* w_then, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (width <= 0 || (b != nullptr) != (w_b != nullptr) || (w_then != nullptr && width > 12000)) return kRefusedSize;
  const size_t smem = w_then != nullptr ? sizeof(float) * (size_t)width : 0;
#define NA(TW, TR)                                                                                                    \
  return launch_kernel(rms_norm_add_kernel<TW, TR>, dim3(n), dim3(256), smem, stream, dst, a, (const TW*)w_a, b,      \
                       (const TW*)w_b, width, coef, eps, accumulate, (TR*)rounded, (const TW*)w_then)
  if (w_dtype == 0 && rounded_dtype == 0) NA(float, float);
  if (w_dtype == 0 && rounded_dtype == 1) NA(float, __nv_bfloat16);
  if (w_dtype == 1 && rounded_dtype == 0) NA(__nv_bfloat16, float);
  if (w_dtype == 1 && rounded_dtype == 1) NA(__nv_bfloat16, __nv_bfloat16);
#undef NA
  return kRefusedDtype;
}

extern "C" int leone_gate_rows(int dtype, void* a, int lda, const void* gate, int ldg, int n_rows, int cols, int act,
                               cudaStream_t stream) {
  if (n_rows <= 0 || cols <= 0) return 0;
  const long long want = ((long long)n_rows * cols + 255) / 256;
  const unsigned blocks = (unsigned)(want < 148 * 16 ? want : 148 * 16);
  if (dtype == 0)
    return launch_kernel(gate_rows_kernel<float>, dim3(blocks), dim3(256), 0, stream, (float*)a, lda, (const float*)gate,
                         ldg, n_rows, cols, act);
  if (dtype == 1)
    return launch_kernel(gate_rows_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, stream, (__nv_bfloat16*)a, lda,
                         (const __nv_bfloat16*)gate, ldg, n_rows, cols, act);
  return kRefusedDtype;
}

extern "C" int leone_gelu_gate(int dtype, const float* z, int ldz, const float* rows, int ldr, int off, void* out, int ldo,
                               int n_rows, int cols, cudaStream_t stream) {
  if (n_rows <= 0 || cols <= 0) return 0;
  const long long want = ((long long)n_rows * cols + 255) / 256;
  const unsigned blocks = (unsigned)(want < 148 * 16 ? want : 148 * 16);
  if (dtype == 0)
    return launch_kernel(gelu_gate_kernel<float>, dim3(blocks), dim3(256), 0, stream, z, ldz, rows, ldr, off, (float*)out,
                         ldo, n_rows, cols);
  if (dtype == 1)
    return launch_kernel(gelu_gate_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, stream, z, ldz, rows, ldr, off,
                         (__nv_bfloat16*)out, ldo, n_rows, cols);
  return kRefusedDtype;
}

extern "C" int leone_zero(void* p, long long bytes, cudaStream_t stream) {
  if (bytes <= 0) return 0;
  return (int)cudaMemsetAsync(p, 0, (size_t)bytes, stream);
}
