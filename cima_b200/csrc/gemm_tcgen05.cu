// Matrix product on the fifth-generation tensor cores (tcgen05) for bfloat16:
//     D[i, j] = sum_k P[i, k] * Q[j, k]          P [p_rows, K], Q [q_rows, K], both row-major (K contiguous)
// One block computes a 128 x BN tile of D.  Operand tiles of 64 k (128 bytes per row) are brought by TMA
// (cp.async.bulk.tensor, 128-byte swizzle) into a ring of shared-memory stages guarded by mbarriers;
// one elected thread issues tcgen05.mma (128 x BN x 16 per instruction) with the accumulator in tensor
// memory (TMEM, 128 lanes x BN float32 columns); tcgen05.commit frees a stage and, at the end, tells the
// epilogue warps that the accumulator is complete; they read it back with tcgen05.ld and apply the
// epilogue in float32 before the one rounding of the store.
//
// Warp roles (192 threads): warp 0 = TMA producer, warp 1 = TMEM allocation + MMA issue,
// warps 2..5 = epilogue (each owns the 32 TMEM lanes its index modulo 4 may access).
//
// Who is P and who is Q decides the use:
//   * prefill (many rows): P = activations [M, K], Q = weights [N, K]; out[i, j]      (row = token)
//   * decode with up to 64 rows ("swap A/B"): P = weights, Q = activations; out[j, i]   (transposed store)
// Epilogues: 0 store bf16 (+ bias)   1 accumulate into the float32 residual (+ bias)
//            2 silu(gate) * up -> bf16 (Q = [gate rows | up rows]; a tile takes BN/2 rows of each)
//            3 store float32 (+ bias)
// Tails in every dimension: TMA fills what lies outside a matrix with zeros, stores are masked.
// K must be a multiple of 8 (16-byte row pitch for TMA).
//
// Every wait on an mbarrier is bounded (2 s); a wait that runs out sets *error_flag, and all roles
// leave their loops, free the tensor memory and return.
//
// The reference has no kernel of this kind: its only tensor-core path is cublasGemmEx
// (src/cuda.rs:2484-2541), its own k_gemm_f16 is a 16x16 shared-memory tile on CUDA cores
// (src/kernels.cu:1410-1431).
#include "tcgen05.cuh"

namespace {

using namespace cima_tc;

constexpr int BM = 128;          // rows of P per tile = TMEM lanes
constexpr int BK = 64;           // k per stage: 64 bf16 = 128 bytes = one swizzle row
constexpr int UMMA_K = 16;
constexpr int THREADS = 192;

enum { EPI_STORE = 0, EPI_ACCUM = 1, EPI_SWIGLU = 2, EPI_STORE_F32 = 3 };

struct GemmArgs {
  int p_rows, q_rows, K;      // extents of P, Q and of the sum
  int up_offset;              // EPI_SWIGLU: row of Q where the "up" half starts
  const float* bias;          // per feature, or null
  void* out;
  int ldo;
  int transposed;             // 0: out[i * ldo + j] (i = P row)   1: out[j * ldo + i]
  int bias_on_p;              // bias indexed by the P row (swap A/B) instead of the Q row
  int* error_flag;
};


// Persistent: the grid has at most one block per SM; a block takes tiles blockIdx.x, blockIdx.x + gridDim.x, ...
// Tile t -> (t % p_tiles, t / p_tiles): the blocks that run together cover all tiles of P (few) times a few
// tiles of Q, so a tile of Q (weights) is fetched from HBM once and shared through L2.
// Two accumulators in tensor memory (2 x BN columns): the epilogue warps drain one while the tensor cores
// fill the other; the ring of shared-memory stages runs on across tiles.
template <int BN, int STAGES, int EPI>
__global__ void __launch_bounds__(THREADS, 1)
k_gemm_tcgen05(const __grid_constant__ CUtensorMap map_p, const __grid_constant__ CUtensorMap map_q, GemmArgs a,
               int p_tiles, int n_tiles) {
  cima_pdl_wait();
  constexpr int P_BYTES = BM * BK * 2, Q_BYTES = BN * BK * 2;
  constexpr int QH = EPI == EPI_SWIGLU ? BN / 2 : BN;          // rows of Q per TMA box
  constexpr int TMEM_COLS = 2 * BN < 32 ? 32 : 2 * BN;
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = (unsigned char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);     // 1024-byte tiles
  unsigned char* sp = smem;                                    // [STAGES][BM x 128 B]
  unsigned char* sq = smem + (size_t)STAGES * P_BYTES;         // [STAGES][BN x 128 B]
  unsigned long long* full = (unsigned long long*)(sq + (size_t)STAGES * Q_BYTES);
  unsigned long long* empty = full + STAGES;
  unsigned long long* acc_full = empty + STAGES;               // [2] accumulator complete
  unsigned long long* acc_free = acc_full + 2;                 // [2] accumulator drained
  unsigned* tmem_slot = (unsigned*)(acc_free + 2);
  volatile int* abort_flag = (volatile int*)(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kblocks = (a.K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; s++) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    for (int b = 0; b < 2; b++) { mbar_init(&acc_full[b], 1); mbar_init(&acc_free[b], 4); }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const unsigned tmem_base = *tmem_slot;

  if (warp == 0) {
    // ---------------------------------------------------------------- TMA producer
    if (lane == 0) {
      int g = 0;                                        // k-blocks issued so far, over all tiles
      bool ok = true;
      for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x) {
        const int p0 = (tile % p_tiles) * BM, q0 = (tile / p_tiles) * QH;
        for (int kb = 0; kb < kblocks; kb++, g++) {
          const int s = g % STAGES;
          if (g >= STAGES && !mbar_wait(&empty[s], ((g / STAGES) - 1) & 1, a.error_flag, abort_flag)) { ok = false; break; }
          mbar_expect_tx(&full[s], P_BYTES + Q_BYTES);
          tma_load_2d(sp + (size_t)s * P_BYTES, &map_p, kb * BK, p0, &full[s]);
          if (EPI == EPI_SWIGLU) {
            tma_load_2d(sq + (size_t)s * Q_BYTES, &map_q, kb * BK, q0, &full[s]);
            tma_load_2d(sq + (size_t)s * Q_BYTES + QH * BK * 2, &map_q, kb * BK, a.up_offset + q0, &full[s]);
          } else {
            tma_load_2d(sq + (size_t)s * Q_BYTES, &map_q, kb * BK, q0, &full[s]);
          }
        }
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issue (one thread)
    if (lane == 0) {
      const unsigned idesc = umma_idesc(BM, BN);
      int g = 0, it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x, it++) {
        const int ab = it & 1;
        if (it >= 2) ok = mbar_wait(&acc_free[ab], ((it >> 1) - 1) & 1, a.error_flag, abort_flag);
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const unsigned acc = tmem_base + (unsigned)(ab * BN);
        for (int kb = 0; kb < kblocks; kb++, g++) {
          const int s = g % STAGES;
          ok = mbar_wait(&full[s], (g / STAGES) & 1, a.error_flag, abort_flag);
          if (!ok) break;
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const unsigned long long pd = umma_smem_desc(smem_u32(sp + (size_t)s * P_BYTES));
          const unsigned long long qd = umma_smem_desc(smem_u32(sq + (size_t)s * Q_BYTES));
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; k++)         // 32 bytes further along the swizzled row per step
            umma_bf16(acc, pd + (unsigned long long)(k * 2), qd + (unsigned long long)(k * 2), idesc, (kb | k) ? 1u : 0u);
          umma_commit(&empty[s]);                       // the stage is free when these instructions have read it
        }
        if (ok) umma_commit(&acc_full[ab]);             // arrives when every instruction of the tile has completed
      }
    }
  } else {
    // ---------------------------------------------------------------- epilogue: 4 warps x 32 TMEM lanes
    const int quarter = warp & 3;                       // the TMEM lanes this warp may read
    int it = 0;
    for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x, it++) {
      const int ab = it & 1;
      const int p0 = (tile % p_tiles) * BM, q0 = (tile / p_tiles) * QH;
      if (!mbar_wait(&acc_full[ab], (it >> 1) & 1, a.error_flag, abort_flag)) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const int i = p0 + quarter * 32 + lane;           // row of P = row of the accumulator
      const unsigned acc = tmem_base + (unsigned)(ab * BN) + ((unsigned)(quarter * 32) << 16);
      constexpr int COLS = EPI == EPI_SWIGLU ? BN / 2 : BN;
#pragma unroll 1
      for (int c0 = 0; c0 < COLS; c0 += 32) {
        float v[32];
        tmem_ld32(acc + (unsigned)c0, v);
        if (EPI == EPI_SWIGLU) {
          float u[32];
          tmem_ld32(acc + (unsigned)(BN / 2 + c0), u);
#pragma unroll
          for (int e = 0; e < 32; e++) v[e] = v[e] / (1.0f + expf(-v[e])) * u[e];
        }
        if (i < a.p_rows) {
          const int jmax = EPI == EPI_SWIGLU ? a.up_offset : a.q_rows;
          const int j0 = q0 + c0;
          // a thread holds 32 consecutive columns of its row: whole 16-byte pieces when the row allows it
          const bool wide = !a.transposed && j0 + 32 <= jmax && (a.ldo & 7) == 0 && ((uintptr_t)a.out & 15) == 0;
          if (wide) {
            if (a.bias && !a.bias_on_p) {
#pragma unroll
              for (int e = 0; e < 32; e++) v[e] += a.bias[j0 + e];
            } else if (a.bias) {
              const float b = a.bias[i];
#pragma unroll
              for (int e = 0; e < 32; e++) v[e] += b;
            }
            const size_t o = (size_t)i * a.ldo + j0;
            if (EPI == EPI_ACCUM || EPI == EPI_STORE_F32) {
              float4* dst = reinterpret_cast<float4*>((float*)a.out + o);
#pragma unroll
              for (int e = 0; e < 8; e++) {
                float4 t = make_float4(v[4 * e], v[4 * e + 1], v[4 * e + 2], v[4 * e + 3]);
                if (EPI == EPI_ACCUM) { const float4 old = dst[e]; t.x += old.x; t.y += old.y; t.z += old.z; t.w += old.w; }
                dst[e] = t;
              }
            } else {
              uint4* dst = reinterpret_cast<uint4*>((__nv_bfloat16*)a.out + o);
#pragma unroll
              for (int e = 0; e < 4; e++) {
                uint4 t;
                __nv_bfloat162* h2 = reinterpret_cast<__nv_bfloat162*>(&t);
#pragma unroll
                for (int k = 0; k < 4; k++) h2[k] = __floats2bfloat162_rn(v[8 * e + 2 * k], v[8 * e + 2 * k + 1]);
                dst[e] = t;
              }
            }
          } else {
#pragma unroll
            for (int e = 0; e < 32; e++) {
              const int j = j0 + e;                     // row of Q = column of the accumulator
              if (j >= jmax) continue;
              float r = v[e];
              if (a.bias) r += a.bias[a.bias_on_p ? i : j];
              const size_t o = a.transposed ? (size_t)j * a.ldo + i : (size_t)i * a.ldo + j;
              if (EPI == EPI_ACCUM) ((float*)a.out)[o] += r;
              else if (EPI == EPI_STORE_F32) ((float*)a.out)[o] = r;
              else ((__nv_bfloat16*)a.out)[o] = __float2bfloat16_rn(r);
            }
          }
        }
      }
      // the accumulator may be overwritten: one arrival per epilogue warp
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_free[ab]);
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  }
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
}

// ---------------------------------------------------------------------------------------- host side

int sm_count() {
  static int n = 0;
  if (!n) {
    int dev = 0;
    cudaGetDevice(&dev);
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
  }
  return n;
}

template <int BN, int STAGES, int EPI>
int launch(const CUtensorMap& mp, const CUtensorMap& mq, const GemmArgs& a, int tiles_q, cudaStream_t stream) {
  auto kern = k_gemm_tcgen05<BN, STAGES, EPI>;
  const size_t smem = 1024 + (size_t)STAGES * (BM + BN) * BK * 2 + (2 * STAGES + 4) * 8 + 16;
  static bool raised = false;
  if (!raised) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return cima_fail((int)e, "gemm_tcgen05: cannot raise shared memory to %zu bytes: %s", smem, cudaGetErrorString(e));
    raised = true;
  }
  const int p_tiles = (a.p_rows + BM - 1) / BM, n_tiles = p_tiles * tiles_q;
  const int grid = n_tiles < sm_count() ? n_tiles : sm_count();
  { int rc_ = cima_launch(kern, dim3(grid), dim3(THREADS), (size_t)(smem), stream, 1, mp, mq, a, p_tiles, n_tiles); if (rc_) return rc_; }
  return cima_launch_result();
}

template <int BN, int STAGES>
int dispatch_epi(int epi, const CUtensorMap& mp, const CUtensorMap& mq, const GemmArgs& a, int tiles_q, cudaStream_t stream) {
  switch (epi) {
    case EPI_STORE: return launch<BN, STAGES, EPI_STORE>(mp, mq, a, tiles_q, stream);
    case EPI_ACCUM: return launch<BN, STAGES, EPI_ACCUM>(mp, mq, a, tiles_q, stream);
    case EPI_SWIGLU: return launch<BN, STAGES, EPI_SWIGLU>(mp, mq, a, tiles_q, stream);
    case EPI_STORE_F32: return launch<BN, STAGES, EPI_STORE_F32>(mp, mq, a, tiles_q, stream);
  }
  return cima_fail(CIMA_E_ARG, "gemm_tcgen05: epilogue %d is not one of 0..3", epi);
}

}  // namespace

// out = epilogue(P Q^T).  P [p_rows, K], Q [q_rows, K] bf16 row-major, 16-byte aligned, K % 8 == 0.
// For epilogue 2, Q is [2 * up_offset, K] (gate rows, then up rows) and q_rows = 2 * up_offset.
// bn: columns of D per tile (64, 128 or 256; for epilogue 2 a tile holds bn/2 gate and bn/2 up features).
// error_flag: device int that a wait that ran out sets to 1 (never cleared here).
extern "C" int cima_gemm_tcgen05(const void* P, const void* Q, const float* bias, void* out, int epi, int p_rows,
                                 int q_rows, int K, int ldo, int transposed, int bias_on_p, int up_offset, int bn,
                                 int* error_flag, cudaStream_t stream) {
  if (p_rows <= 0 || q_rows <= 0) return 0;
  if (K <= 0 || K % 8) return cima_fail(CIMA_E_SIZE, "gemm_tcgen05: K %d must be a positive multiple of 8 (16-byte rows for TMA)", K);
  if (((uintptr_t)P | (uintptr_t)Q) & 15) return cima_fail(CIMA_E_ARG, "gemm_tcgen05: P and Q must be 16-byte aligned");
  if (!error_flag) return cima_fail(CIMA_E_ARG, "gemm_tcgen05: an error flag on the device is needed");
  if (epi == EPI_SWIGLU && (up_offset <= 0 || q_rows != 2 * up_offset)) return cima_fail(CIMA_E_SIZE, "gemm_tcgen05: the gated epilogue needs Q = [gate | up] with q_rows = 2 * up_offset");
  if (epi == EPI_SWIGLU && bias) return cima_fail(CIMA_E_ARG, "gemm_tcgen05: the gated epilogue takes no bias");
  if (bn != 64 && bn != 128 && bn != 256) return cima_fail(CIMA_E_SIZE, "gemm_tcgen05: tile width %d is not 64, 128 or 256", bn);
  const int qh = epi == EPI_SWIGLU ? bn / 2 : bn;                 // rows of Q per TMA box
  const int q_feat = epi == EPI_SWIGLU ? up_offset : q_rows;
  const int tiles_q = (q_feat + qh - 1) / qh;
  CUtensorMap mp, mq;
  int rc = make_map(&mp, P, p_rows, K, K, BM);
  if (rc) return rc;
  rc = make_map(&mq, Q, q_rows, K, K, qh);
  if (rc) return rc;
  GemmArgs a{p_rows, q_rows, K, up_offset, bias, out, ldo, transposed, bias_on_p, error_flag};
  switch (bn) {
    case 64: return dispatch_epi<64, 8>(epi, mp, mq, a, tiles_q, stream);
    case 128: return dispatch_epi<128, 6>(epi, mp, mq, a, tiles_q, stream);
    default: return dispatch_epi<256, 4>(epi, mp, mq, a, tiles_q, stream);
  }
}
