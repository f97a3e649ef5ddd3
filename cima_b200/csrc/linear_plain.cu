// Plain matrix product for the true 32-bit path and for weights that are stored in 32-bit:
//   out[m,n] = sum_k A[m,k] * W[n,k] (+ bias[n])        weights are [out, in], as in the checkpoint
// FFMA only, no tensor cores and no reduced-precision mode.  Each output element is accumulated
// by one thread over k = 0..K-1 in ascending order, so its value depends on its own row of A and
// row of W only: the same bits whether the row comes alone, in a prompt or in a batch.
//
// Counterpart in the reference: k_gemm_f16 (src/kernels.cu:1410-1431; 16x16 tiles, one output per
// thread, f32 accumulate) with k_bias (:390-393) and k_add (:75-78) behind it.
#include "common.cuh"

enum { LIN_STORE = 0, LIN_ACCUM = 1 };

template <typename TA, typename TW, typename TO, int MODE>
__global__ void __launch_bounds__(256)
k_linear_plain(const TA* __restrict__ A, const TW* __restrict__ W, const float* __restrict__ bias,
               TO* __restrict__ out, int M, int N, int K, int lda, int ldo) {
  cima_pdl_wait();
  constexpr int BM = 64, BN = 64, BK = 16;
  __shared__ float As[BK][BM + 4];
  __shared__ float Ws[BK][BN + 4];
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;       // 16 x 16 threads, 4 x 4 outputs each
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; i++)
#pragma unroll
    for (int j = 0; j < 4; j++) acc[i][j] = 0.f;

  for (int k0 = 0; k0 < K; k0 += BK) {
    // 64 x 16 elements of each operand, 4 per thread: thread -> (row = idx / 16, k = idx % 16)
#pragma unroll
    for (int r = 0; r < 4; r++) {
      const int idx = threadIdx.x + r * 256;
      const int row = idx >> 4, kk = idx & 15;
      const int k = k0 + kk;
      float a = 0.f, w = 0.f;
      if (k < K) {
        if (m0 + row < M) a = cima_to_f32<TA>(A[(size_t)(m0 + row) * lda + k]);
        if (n0 + row < N) w = cima_to_f32<TW>(W[(size_t)(n0 + row) * K + k]);
      }
      As[kk][row] = a;
      Ws[kk][row] = w;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < BK; kk++) {
      float a[4], w[4];
#pragma unroll
      for (int i = 0; i < 4; i++) a[i] = As[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; j++) w[j] = Ws[kk][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; i++) {
    const int m = m0 + ty * 4 + i;
    if (m >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; j++) {
      const int n = n0 + tx * 4 + j;
      if (n >= N) continue;
      float v = acc[i][j];
      if (bias) v += bias[n];
      TO* o = out + (size_t)m * ldo + n;
      if (MODE == LIN_ACCUM) *o = cima_from_f32<TO>(cima_to_f32<TO>(*o) + v);
      else *o = cima_from_f32<TO>(v);
    }
  }
}

// The same for at most 8 rows (a decode step): one thread per output feature walks its row of W once, 64 k at a
// time (sixteen independent 16-byte loads in flight per thread, then the products in ascending k), with one
// accumulator per row of A.  The sequence of fused multiply-adds of an output element is exactly that of the
// tiled kernel above, so the two give the same bits; this one streams the weights (a thread per output feature
// is all the parallelism the fixed order leaves: some 1 TB/s at 3,584 features, 3 TB/s at 37,888) where the tiled
// kernel, with a sixty-fourth of its tile in use, reaches a few percent of the memory's bandwidth.
// The block's rows of A go through shared memory, 64 k at a time (every thread reads the same values).
constexpr int FEW_ROWS = 8;
constexpr int FEW_THREADS = 64;
constexpr int FEW_K = 64;

template <typename TA, typename TW, typename TO, int MODE, bool VEC>
__global__ void __launch_bounds__(FEW_THREADS)
k_linear_plain_few(const TA* __restrict__ A, const TW* __restrict__ W, const float* __restrict__ bias,
                   TO* __restrict__ out, int M, int N, int K, int lda, int ldo) {
  cima_pdl_wait();
  __shared__ __align__(16) float As[FEW_ROWS][FEW_K];
  const int n = blockIdx.x * FEW_THREADS + threadIdx.x;
  const bool live = n < N;
  const TW* wr = W + (size_t)(live ? n : 0) * K;
  float acc[FEW_ROWS];
#pragma unroll
  for (int m = 0; m < FEW_ROWS; m++) acc[m] = 0.f;
  for (int k0 = 0; k0 < K; k0 += FEW_K) {
    const int kn = min(FEW_K, K - k0);
    float w[FEW_K];
    if (VEC && kn == FEW_K) {
#pragma unroll
      for (int q = 0; q < FEW_K / 4; q++) {
        const float4 v = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(wr) + k0 + 4 * q);
        w[4 * q] = v.x; w[4 * q + 1] = v.y; w[4 * q + 2] = v.z; w[4 * q + 3] = v.w;
      }
    } else {
#pragma unroll
      for (int q = 0; q < FEW_K; q++) w[q] = q < kn ? cima_to_f32<TW>(wr[k0 + q]) : 0.f;
    }
    __syncthreads();                                    // the previous chunk of A has been used
    for (int e = threadIdx.x; e < M * FEW_K; e += FEW_THREADS) {
      const int m = e / FEW_K, q = e - m * FEW_K;
      As[m][q] = q < kn ? cima_to_f32<TA>(A[(size_t)m * lda + k0 + q]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int m = 0; m < FEW_ROWS; m++) {
      if (m < M) {
        if (kn == FEW_K) {
#pragma unroll
          for (int q = 0; q < FEW_K; q += 4) {
            const float4 a = *reinterpret_cast<const float4*>(&As[m][q]);
            acc[m] = fmaf(a.x, w[q], acc[m]);
            acc[m] = fmaf(a.y, w[q + 1], acc[m]);
            acc[m] = fmaf(a.z, w[q + 2], acc[m]);
            acc[m] = fmaf(a.w, w[q + 3], acc[m]);
          }
        } else {
          for (int q = 0; q < kn; q++) acc[m] = fmaf(As[m][q], w[q], acc[m]);
        }
      }
    }
  }
  if (!live) return;
#pragma unroll
  for (int m = 0; m < FEW_ROWS; m++) {
    if (m >= M) break;
    float v = acc[m];
    if (bias) v += bias[n];
    TO* o = out + (size_t)m * ldo + n;
    if (MODE == LIN_ACCUM) *o = cima_from_f32<TO>(cima_to_f32<TO>(*o) + v);
    else *o = cima_from_f32<TO>(v);
  }
}

template <typename TA, typename TW, typename TO, int MODE>
static int launch_few(const void* A, const void* W, const float* bias, void* out, int M, int N, int K, int lda, int ldo,
                      cudaStream_t stream) {
  const dim3 g((N + FEW_THREADS - 1) / FEW_THREADS);
  const bool vec = sizeof(TW) == 4 && K % 4 == 0 && ((uintptr_t)W & 15) == 0;
  int rc;
  if (vec) rc = cima_launch(k_linear_plain_few<TA, TW, TO, MODE, true>, g, dim3(FEW_THREADS), (size_t)0, stream, 1, (const TA*)A, (const TW*)W, bias, (TO*)out, M, N, K, lda, ldo);
  else rc = cima_launch(k_linear_plain_few<TA, TW, TO, MODE, false>, g, dim3(FEW_THREADS), (size_t)0, stream, 1, (const TA*)A, (const TW*)W, bias, (TO*)out, M, N, K, lda, ldo);
  if (rc) return rc;
  return cima_launch_result();
}

template <typename TA, typename TW, typename TO>
static int launch_plain(const void* A, const void* W, const float* bias, void* out, int mode, int M, int N, int K,
                        int lda, int ldo, cudaStream_t stream) {
  // (only the all-float32 combination, the 32-bit path's: each instantiation of that kernel costs seconds to compile)
  if constexpr (sizeof(TA) == 4 && sizeof(TW) == 4 && sizeof(TO) == 4) {
    if (M <= FEW_ROWS) {
      if (mode == LIN_STORE) return launch_few<TA, TW, TO, LIN_STORE>(A, W, bias, out, M, N, K, lda, ldo, stream);
      return launch_few<TA, TW, TO, LIN_ACCUM>(A, W, bias, out, M, N, K, lda, ldo, stream);
    }
  }
  dim3 grid((N + 63) / 64, (M + 63) / 64);
  if (mode == LIN_STORE)
    { int rc_ = cima_launch(k_linear_plain<TA, TW, TO, LIN_STORE>, dim3(grid), dim3(256), (size_t)(0), stream, 1, (const TA*)A, (const TW*)W, bias, (TO*)out, M, N, K, lda, ldo); if (rc_) return rc_; }
  else
    { int rc_ = cima_launch(k_linear_plain<TA, TW, TO, LIN_ACCUM>, dim3(grid), dim3(256), (size_t)(0), stream, 1, (const TA*)A, (const TW*)W, bias, (TO*)out, M, N, K, lda, ldo); if (rc_) return rc_; }
  return cima_launch_result();
}

// mode 0: out = A W^T (+ bias), stored as out_dtype.  mode 1: out += A W^T (+ bias); out must be float32.
extern "C" int cima_linear_plain(const void* A, int a_dtype, const void* W, int w_dtype, const float* bias,
                                 void* out, int out_dtype, int mode, int M, int N, int K, int lda, int ldo,
                                 cudaStream_t stream) {
  if (M <= 0) return 0;
  if (N <= 0 || K <= 0) return cima_fail(CIMA_E_SIZE, "linear_plain: N %d and K %d must be positive", N, K);
  if (lda < K || ldo < N) return cima_fail(CIMA_E_SIZE, "linear_plain: leading dimensions (%d, %d) are smaller than the rows (%d, %d)", lda, ldo, K, N);
  if (mode != LIN_STORE && mode != LIN_ACCUM) return cima_fail(CIMA_E_ARG, "linear_plain: mode %d is neither store (0) nor accumulate (1)", mode);
  if (mode == LIN_ACCUM && out_dtype != CIMA_F32) return cima_fail(CIMA_E_DTYPE, "linear_plain: accumulation needs a float32 output");
  if ((long long)((M + 63) / 64) > 65535) return cima_fail(CIMA_E_SIZE, "linear_plain: %d rows exceed one launch; the caller cuts them", M);
  const int key = a_dtype * 4 + w_dtype * 2 + out_dtype;
  switch (key) {
    case 0: return launch_plain<float, float, float>(A, W, bias, out, mode, M, N, K, lda, ldo, stream);
    case 4 + 0 + 0: return launch_plain<__nv_bfloat16, float, float>(A, W, bias, out, mode, M, N, K, lda, ldo, stream);
    case 4 + 0 + 1: return launch_plain<__nv_bfloat16, float, __nv_bfloat16>(A, W, bias, out, mode, M, N, K, lda, ldo, stream);
    case 4 + 2 + 0: return launch_plain<__nv_bfloat16, __nv_bfloat16, float>(A, W, bias, out, mode, M, N, K, lda, ldo, stream);
    case 4 + 2 + 1: return launch_plain<__nv_bfloat16, __nv_bfloat16, __nv_bfloat16>(A, W, bias, out, mode, M, N, K, lda, ldo, stream);
    default:
      return cima_fail(CIMA_E_DTYPE, "linear_plain: dtypes (A %d, W %d, out %d) are not a supported combination", a_dtype, w_dtype, out_dtype);
  }
}
