// Matrix product for few rows (decode): out[m,n] = sum_k X[m,k] * W[n,k], M <= 64, bfloat16 operands,
// float32 accumulation.  The step is bound by reading W once from HBM, so the kernel is built
// around the weight stream: every thread keeps several 16-byte loads of W in flight, the weights
// are the 16-row operand of the tensor-core instruction and the few activation rows are its 8-wide
// operand ("swap A/B"), so M = 1..8 costs one instruction per 16x16 weights and M = 64 costs eight.
//
// Work split.  One block owns 16 output features (or 16 gate and the 16 matching up features for
// the gated epilogue).  Its 8 warps split K in interleaved chunks; their partial sums are added in
// shared memory in warp order 0..7, so a result never depends on scheduling, and a row of X gives
// the same bits whatever else is in the batch.
//
// Operand order.  mma.m16n8k16 wants, per thread, k = {2t, 2t+1, 2t+8, 2t+9} of rows g and g+8.
// A sum over k does not care in which order k is visited as long as both operands agree, so a
// thread instead loads 8 consecutive k (16 bytes) of its W rows and of its X row and feeds the
// first four to one instruction and the last four to the next: all loads are 16-byte and
// row-contiguous, no shared-memory staging of W is needed.
//
// Epilogues (the reference's GEMV has the same three, src/kernels.cu:502-538):
//   0 store bf16 (+ bias)      1 accumulate into the float32 residual      2 silu(gate) * up -> bf16
//   3 store float32 (+ bias), used for logits
#include "common.cuh"

enum { SK_STORE = 0, SK_ACCUM = 1, SK_SWIGLU = 2, SK_STORE_F32 = 3 };

__device__ __forceinline__ uint4 ld_stream16(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}

__device__ __forceinline__ uint4 ld_cached16(const void* p) {
  return __ldg(reinterpret_cast<const uint4*>(p));
}

__device__ __forceinline__ void mma_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                          uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

constexpr int SK_WARPS = 8;
constexpr int SK_ROWS = 16;      // output features per m-tile
constexpr int SK_PAD = 17;       // row stride of the reduction buffer (bank spread)

// NT: 8-row tiles of X (M <= 8 * NT).  MT: m-tiles per block (1, or 2 for the gated epilogue).
// U: 32-wide k steps kept in flight per warp iteration.
template <int NT, int MT, int U, int MODE>
__global__ void __launch_bounds__(SK_WARPS * 32)
k_linear_skinny(const __nv_bfloat16* __restrict__ X, const __nv_bfloat16* __restrict__ W,
                const float* __restrict__ bias, void* __restrict__ out,
                int M, int N, int K, int ldx, int ldo, int up_offset) {
  extern __shared__ float red[];                       // [warps][MT][NT*8][SK_PAD]
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int n0 = blockIdx.x * SK_ROWS;

  float acc[MT][NT][4];
#pragma unroll
  for (int a = 0; a < MT; a++)
#pragma unroll
    for (int j = 0; j < NT; j++)
#pragma unroll
      for (int e = 0; e < 4; e++) acc[a][j][e] = 0.f;

  // rows of W this thread reads: g and g + 8 of each m-tile; the second m-tile (up) starts up_offset further
  const __nv_bfloat16* wrow[MT][2];
  bool wok[MT][2];
#pragma unroll
  for (int a = 0; a < MT; a++)
#pragma unroll
    for (int h = 0; h < 2; h++) {
      const int r = n0 + g + 8 * h;
      wok[a][h] = r < N;
      wrow[a][h] = W + (size_t)((wok[a][h] ? r : 0) + a * up_offset) * K;
    }

  // A warp owns chunks of 128 consecutive k, interleaved with the other warps' chunks; this split,
  // and so the order of summation, is the same for every instantiation.  U only says how many of a
  // chunk's four 32-wide steps are loaded before they are multiplied.
  constexpr int CHUNK = 128;
  for (int k0 = warp * CHUNK; k0 < K; k0 += SK_WARPS * CHUNK) {
#pragma unroll
    for (int sub = 0; sub < 4; sub += U) {
      uint4 w[MT][2][U];
#pragma unroll
      for (int s = 0; s < U; s++) {
        const int k = k0 + (sub + s) * 32 + 8 * t;
#pragma unroll
        for (int a = 0; a < MT; a++)
#pragma unroll
          for (int h = 0; h < 2; h++)
            w[a][h][s] = (wok[a][h] && k < K) ? ld_stream16(wrow[a][h] + k) : make_uint4(0u, 0u, 0u, 0u);
      }
#pragma unroll
      for (int s = 0; s < U; s++) {
        const int k = k0 + (sub + s) * 32 + 8 * t;
#pragma unroll
        for (int j = 0; j < NT; j++) {
          const int m = j * 8 + g;
          const uint4 x = (m < M && k < K) ? ld_cached16(X + (size_t)m * ldx + k) : make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
          for (int a = 0; a < MT; a++) {
            mma_16816(acc[a][j], w[a][0][s].x, w[a][1][s].x, w[a][0][s].y, w[a][1][s].y, x.x, x.y);
            mma_16816(acc[a][j], w[a][0][s].z, w[a][1][s].z, w[a][0][s].w, w[a][1][s].w, x.z, x.w);
          }
        }
      }
    }
  }

  // partial sums -> shared memory: red[warp][a][col = j*8 + 2t (+1)][row = g (+8)]
  constexpr int COLS = NT * 8;
  float* mine = red + (size_t)warp * MT * COLS * SK_PAD;
#pragma unroll
  for (int a = 0; a < MT; a++)
#pragma unroll
    for (int j = 0; j < NT; j++) {
      float* base = mine + ((size_t)a * COLS + j * 8 + 2 * t) * SK_PAD;
      base[g] = acc[a][j][0];
      base[SK_PAD + g] = acc[a][j][1];
      base[g + 8] = acc[a][j][2];
      base[SK_PAD + g + 8] = acc[a][j][3];
    }
  __syncthreads();

  for (int e = threadIdx.x; e < COLS * SK_ROWS; e += SK_WARPS * 32) {
    const int r = e % SK_ROWS, m = e / SK_ROWS;
    const int n = n0 + r;
    if (m >= M || n >= N) continue;
    float v[MT];
#pragma unroll
    for (int a = 0; a < MT; a++) {
      float s = 0.f;
#pragma unroll
      for (int wi = 0; wi < SK_WARPS; wi++) s += red[(((size_t)wi * MT + a) * COLS + m) * SK_PAD + r];
      v[a] = s;
    }
    const size_t o = (size_t)m * ldo + n;
    if (MODE == SK_STORE) {
      ((__nv_bfloat16*)out)[o] = __float2bfloat16_rn(v[0] + (bias ? bias[n] : 0.f));
    } else if (MODE == SK_ACCUM) {
      ((float*)out)[o] += v[0] + (bias ? bias[n] : 0.f);
    } else if (MODE == SK_STORE_F32) {
      ((float*)out)[o] = v[0] + (bias ? bias[n] : 0.f);
    } else {
      const float gate = v[0], up = v[MT - 1];
      ((__nv_bfloat16*)out)[o] = __float2bfloat16_rn(gate / (1.0f + expf(-gate)) * up);
    }
  }
}

template <int NT, int MT, int U, int MODE>
static int launch_skinny(const void* X, const void* W, const float* bias, void* out, int M, int N, int K, int ldx,
                         int ldo, int up_offset, cudaStream_t stream) {
  auto kern = k_linear_skinny<NT, MT, U, MODE>;
  const size_t smem = (size_t)SK_WARPS * MT * NT * 8 * SK_PAD * sizeof(float);
  if (smem > 48 * 1024) {
    static bool raised = false;     // one attribute per instantiation
    if (!raised) {
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e != cudaSuccess) return cima_fail((int)e, "linear_skinny: cannot raise shared memory to %zu bytes: %s", smem, cudaGetErrorString(e));
      raised = true;
    }
  }
  kern<<<(N + SK_ROWS - 1) / SK_ROWS, SK_WARPS * 32, smem, stream>>>(
      (const __nv_bfloat16*)X, (const __nv_bfloat16*)W, bias, out, M, N, K, ldx, ldo, up_offset);
  return cima_launch_result();
}

template <int NT>
static int dispatch_mode(int mode, const void* X, const void* W, const float* bias, void* out, int M, int N, int K,
                         int ldx, int ldo, cudaStream_t stream) {
  constexpr int U = NT <= 2 ? 4 : 2;
  switch (mode) {
    case SK_STORE: return launch_skinny<NT, 1, U, SK_STORE>(X, W, bias, out, M, N, K, ldx, ldo, 0, stream);
    case SK_ACCUM: return launch_skinny<NT, 1, U, SK_ACCUM>(X, W, bias, out, M, N, K, ldx, ldo, 0, stream);
    case SK_STORE_F32: return launch_skinny<NT, 1, U, SK_STORE_F32>(X, W, bias, out, M, N, K, ldx, ldo, 0, stream);
    case SK_SWIGLU: return launch_skinny<NT, 2, (NT <= 2 ? 2 : 1), SK_SWIGLU>(X, W, bias, out, M, N, K, ldx, ldo, N, stream);
    default: return cima_fail(CIMA_E_ARG, "linear_skinny: mode %d is not one of 0..3", mode);
  }
}

// X [M, K] bf16 (row stride ldx), W [N, K] bf16 (for mode 2: [2N, K], gate rows then up rows),
// bias float32 [N] or null, out [M, N] (row stride ldo) in the dtype of the mode.
// Accepts 1 <= M <= 64, any N, K a multiple of 8 (16-byte rows), 16-byte aligned X, W and ldx % 8 == 0.
extern "C" int cima_linear_skinny(const void* X, const void* W, const float* bias, void* out, int mode, int M, int N,
                                  int K, int ldx, int ldo, cudaStream_t stream) {
  if (M <= 0) return 0;
  if (M > 64) return cima_fail(CIMA_E_SIZE, "linear_skinny: %d rows; this kernel takes at most 64", M);
  if (N <= 0 || K <= 0) return cima_fail(CIMA_E_SIZE, "linear_skinny: N %d and K %d must be positive", N, K);
  if (K % 8 || ldx % 8) return cima_fail(CIMA_E_SIZE, "linear_skinny: K %d and the row stride %d must be multiples of 8 (16-byte loads)", K, ldx);
  if (((uintptr_t)X | (uintptr_t)W) & 15) return cima_fail(CIMA_E_ARG, "linear_skinny: X and W must be 16-byte aligned");
  if (mode == SK_SWIGLU && bias) return cima_fail(CIMA_E_ARG, "linear_skinny: the gated epilogue takes no bias");
  if (M <= 8) return dispatch_mode<1>(mode, X, W, bias, out, M, N, K, ldx, ldo, stream);
  if (M <= 16) return dispatch_mode<2>(mode, X, W, bias, out, M, N, K, ldx, ldo, stream);
  if (M <= 32) return dispatch_mode<4>(mode, X, W, bias, out, M, N, K, ldx, ldo, stream);
  return dispatch_mode<8>(mode, X, W, bias, out, M, N, K, ldx, ldo, stream);
}
