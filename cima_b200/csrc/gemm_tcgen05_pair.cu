// The tcgen05 matrix product on PAIRS of SMs (cta_group::2), for many rows (prefill):
//     D[i, j] = sum_k P[i, k] * Q[j, k]      P [p_rows, K] activations, Q [q_rows, K] weights, both K-major
// A cluster of two blocks computes a 256 x BN tile.  Each block loads its own 128 rows of P and only HALF of the
// tile of Q (BN/2 rows) into its shared memory; the leader block's elected thread issues
// tcgen05.mma.cta_group::2, which reads A from both blocks' shared memory, the two halves of B from the two
// blocks, and writes each block's 128 x BN part of D into that block's tensor memory.  Per multiply-add an SM
// so reads a third less operand bytes from shared memory than alone, which is what bounds a kernel of single
// blocks with 128 x 256 tiles (1,404 TFLOP/s on the gated projection against 1,493 here).  The design: persistent
// blocks, TMA with 128-byte swizzle into a ring of stages, two accumulators in tensor memory so that the
// epilogue warps drain one while the tensor cores fill the other, 16-byte stores, every wait bounded.
//
// Barriers.  The TMA loads of both blocks complete on the LEADER's "full" barrier of the stage (the peer passes
// that barrier's cluster address); the leader's tcgen05.commit arrives, multicast, on both blocks' "empty"
// barrier of the stage and, after a tile, on both blocks' "accumulator full" barrier; every epilogue warp of
// both blocks arrives on the leader's "accumulator free" barrier (8 arrivals).
//
// With the gated epilogue the tile of Q is [BN/2 gate rows | BN/2 up rows]: the leader holds the gate half,
// the peer the up half.
#include "tcgen05.cuh"
#include <cooperative_groups.h>

namespace cg = cooperative_groups;

namespace {

using namespace cima_tc;


constexpr int BM = 128;          // rows of P per tile = TMEM lanes
constexpr int BK = 64;           // k per stage: 64 bf16 = 128 bytes = one swizzle row
constexpr int UMMA_K = 16;
constexpr int THREADS = 192;

enum { EPI_STORE = 0, EPI_ACCUM = 1, EPI_SWIGLU = 2, EPI_STORE_F32 = 3 };

__device__ __forceinline__ unsigned cluster_addr(const void* p, unsigned rank) {      // address of p in block `rank`
  unsigned a = smem_u32(p), r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(rank));
  return r;
}
__device__ __forceinline__ void tma_load_2d_pair(void* smem, const CUtensorMap* map, int x, int y, unsigned bar_cluster_addr) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(smem_u32(smem)), "l"(map), "r"(x), "r"(y), "r"(bar_cluster_addr) : "memory");
}
__device__ __forceinline__ void umma_bf16_pair(unsigned tmem_d, unsigned long long adesc, unsigned long long bdesc,
                                               unsigned idesc, unsigned accumulate) {
  asm volatile(
      "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n}\n"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit_pair(void* bar) {       // arrives on `bar` in both blocks of the pair
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
               ::"r"(smem_u32(bar)), "h"((unsigned short)3) : "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(unsigned bar_cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(bar_cluster_addr) : "memory");
}

struct PairArgs {
  int p_rows, q_rows, K;
  int up_offset;              // gated epilogue: row of Q where the "up" half starts
  const float* bias;          // per feature (row of Q), or null
  void* out;                  // out[i * ldo + j]
  int ldo;
  int* error_flag;
  int act;                    // gated epilogue: the gate's activation (CIMA_ACT_*)
};

// The rows a tile loads: its own 256, but the last tile of a matrix of at least 256 rows starts early enough to end
// with the matrix.  A TMA box that reaches beyond the tensor is filled with zeros much more slowly than one is loaded
// (300 rows took 151 us where 512 take 115); the rows before the tile's own are computed again and not stored.
__device__ __forceinline__ int tile_rows(int first, int p_rows) {
  return p_rows >= 2 * BM ? min(first, p_rows - 2 * BM) : first;
}

template <int BN, int STAGES, int EPI>
__global__ void __launch_bounds__(THREADS, 1)
k_gemm_tcgen05_pair(const __grid_constant__ CUtensorMap map_p, const __grid_constant__ CUtensorMap map_q, PairArgs a,
                    int p_tiles, int n_tiles) {
  cima_pdl_wait();
  constexpr bool GATED = EPI == EPI_SWIGLU;
  constexpr int QH = BN / 2;                                   // rows of Q that one block holds
  constexpr int P_BYTES = BM * BK * 2, Q_BYTES = QH * BK * 2;
  constexpr int TMEM_COLS = 2 * BN;                            // two accumulators
  constexpr int OUT_COLS = GATED ? BN / 2 : BN;
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = (unsigned char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  unsigned char* sp = smem;                                    // [STAGES][128 x 128 B]
  unsigned char* sq = smem + (size_t)STAGES * P_BYTES;         // [STAGES][BN/2 x 128 B]
  unsigned long long* full = (unsigned long long*)(sq + (size_t)STAGES * Q_BYTES);
  unsigned long long* empty = full + STAGES;
  unsigned long long* acc_full = empty + STAGES;               // [2]
  unsigned long long* acc_free = acc_full + 2;                 // [2], used in the leader only
  unsigned* tmem_slot = (unsigned*)(acc_free + 2);
  volatile int* abort_flag = (volatile int*)(tmem_slot + 1);

  cg::cluster_group cluster = cg::this_cluster();
  const unsigned rank = cluster.block_rank();                  // 0 = leader
  const int pair = blockIdx.x >> 1, pairs = gridDim.x >> 1;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kblocks = (a.K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; s++) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    for (int b = 0; b < 2; b++) { mbar_init(&acc_full[b], 1); mbar_init(&acc_free[b], 8); }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  cluster.sync();                                              // both blocks' barriers exist before anyone signals them
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const unsigned tmem_base = *tmem_slot;

  if (warp == 0) {
    // ---------------------------------------------------------------- TMA producer (one in each block)
    if (lane == 0) {
      int g = 0;
      bool ok = true;
      for (int tile = pair; tile < n_tiles && ok; tile += pairs) {
        const int p0 = tile_rows((tile % p_tiles) * (2 * BM), a.p_rows) + (int)rank * BM;
        const int qt = (tile / p_tiles) * (GATED ? QH : BN);
        const int q0 = GATED ? (rank ? a.up_offset + qt : qt) : qt + (int)rank * QH;
        for (int kb = 0; kb < kblocks; kb++, g++) {
          const int s = g % STAGES;
          if (g >= STAGES && !mbar_wait(&empty[s], ((g / STAGES) - 1) & 1, a.error_flag, abort_flag)) { ok = false; break; }
          const unsigned bar = cluster_addr(&full[s], 0);      // the leader's barrier collects both blocks' bytes
          if (rank == 0) mbar_expect_tx(&full[s], 2 * (P_BYTES + Q_BYTES));
          tma_load_2d_pair(sp + (size_t)s * P_BYTES, &map_p, kb * BK, p0, bar);
          tma_load_2d_pair(sq + (size_t)s * Q_BYTES, &map_q, kb * BK, q0, bar);
        }
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issue: the leader's elected thread
    if (rank == 0 && lane == 0) {
      const unsigned idesc = umma_idesc(2 * BM, BN);
      int g = 0, it = 0;
      bool ok = true;
      for (int tile = pair; tile < n_tiles && ok; tile += pairs, it++) {
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
          for (int k = 0; k < BK / UMMA_K; k++)
            umma_bf16_pair(acc, pd + (unsigned long long)(k * 2), qd + (unsigned long long)(k * 2), idesc, (kb | k) ? 1u : 0u);
          umma_commit_pair(&empty[s]);                         // frees the stage in both blocks
        }
        if (ok) umma_commit_pair(&acc_full[ab]);               // tells both blocks' epilogues
      }
    }
  } else {
    // ---------------------------------------------------------------- epilogue: this block's 128 rows of the tile
    const int quarter = warp & 3;
    const unsigned free_bar[2] = {cluster_addr(&acc_free[0], 0), cluster_addr(&acc_free[1], 0)};
    int it = 0;
    for (int tile = pair; tile < n_tiles; tile += pairs, it++) {
      const int ab = it & 1;
      const int p_first = (tile % p_tiles) * (2 * BM);         // the tile's own rows start here
      const int p0 = tile_rows(p_first, a.p_rows) + (int)rank * BM;
      const int q0 = (tile / p_tiles) * OUT_COLS;              // first output column of the tile
      if (!mbar_wait(&acc_full[ab], (it >> 1) & 1, a.error_flag, abort_flag)) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const int i = p0 + quarter * 32 + lane;
      const unsigned acc = tmem_base + (unsigned)(ab * BN) + ((unsigned)(quarter * 32) << 16);
#pragma unroll 1
      for (int c0 = 0; c0 < OUT_COLS; c0 += 32) {
        float v[32];
        tmem_ld32(acc + (unsigned)c0, v);
        if (GATED) {
          float u[32];
          tmem_ld32(acc + (unsigned)(BN / 2 + c0), u);
#pragma unroll
          for (int e = 0; e < 32; e++) v[e] = (a.act == CIMA_ACT_SILU ? v[e] / (1.0f + expf(-v[e])) : cima_gate_act(v[e], a.act)) * u[e];
        }
        if (i >= p_first && i < a.p_rows) {
          const int jmax = GATED ? a.up_offset : a.q_rows;
          const int j0 = q0 + c0;
          const bool wide = j0 + 32 <= jmax && (a.ldo & 7) == 0 && ((uintptr_t)a.out & 15) == 0;
          if (wide) {
            if (a.bias) {
#pragma unroll
              for (int e = 0; e < 32; e++) v[e] += a.bias[j0 + e];
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
              const int j = j0 + e;
              if (j >= jmax) continue;
              float r = v[e];
              if (a.bias) r += a.bias[j];
              const size_t o = (size_t)i * a.ldo + j;
              if (EPI == EPI_ACCUM) ((float*)a.out)[o] += r;
              else if (EPI == EPI_STORE_F32) ((float*)a.out)[o] = r;
              else ((__nv_bfloat16*)a.out)[o] = __float2bfloat16_rn(r);
            }
          }
        }
      }
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(free_bar[ab]);        // 4 warps x 2 blocks arrive on the leader's barrier
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  }
  __syncthreads();
  cluster.sync();                  // nobody leaves while the peer may still read its shared memory or signal its barriers
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
}

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
int launch(const CUtensorMap& mp, const CUtensorMap& mq, const PairArgs& a, int p_tiles, int tiles_q, cudaStream_t stream) {
  auto kern = k_gemm_tcgen05_pair<BN, STAGES, EPI>;
  const size_t smem = 1024 + (size_t)STAGES * (BM + BN / 2) * BK * 2 + (2 * STAGES + 4) * 8 + 16;
  static bool raised = false;
  if (!raised) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return cima_fail((int)e, "gemm_tcgen05_pair: cannot raise shared memory to %zu bytes: %s", smem, cudaGetErrorString(e));
    raised = true;
  }
  const int n_tiles = p_tiles * tiles_q;
  int pairs = sm_count() / 2;
  if (n_tiles < pairs) pairs = n_tiles;
  { int rc_ = cima_launch(kern, dim3(2 * pairs), dim3(THREADS), (size_t)(smem), stream, 2, mp, mq, a, p_tiles, n_tiles); if (rc_) return rc_; }
  return cima_launch_result();
}

}  // namespace

// out[i, j] = epilogue(sum_k P[i, k] Q[j, k]); P [p_rows, K], Q [q_rows, K] bf16, 16-byte aligned, K % 8 == 0.
// Tiles of 256 rows x 256 columns per pair of SMs.  Epilogues: 0 store bf16 (+ bias), 1 accumulate into float32, 2 act(gate) * up (Q = [gate | up]; act: CIMA_ACT_*), 3 store float32.
extern "C" int cima_gemm_tcgen05_pair(const void* P, const void* Q, const float* bias, void* out, int epi, int p_rows,
                                      int q_rows, int K, int ldo, int up_offset, int act, int* error_flag, cudaStream_t stream) {
  if (p_rows <= 0 || q_rows <= 0) return 0;
  if (act < 0 || act >= CIMA_ACT_COUNT) return cima_fail(CIMA_E_ARG, "gemm_tcgen05_pair: activation code %d is not one of 0..%d", act, CIMA_ACT_COUNT - 1);
  if (K <= 0 || K % 8) return cima_fail(CIMA_E_SIZE, "gemm_tcgen05_pair: K %d must be a positive multiple of 8", K);
  if (((uintptr_t)P | (uintptr_t)Q) & 15) return cima_fail(CIMA_E_ARG, "gemm_tcgen05_pair: P and Q must be 16-byte aligned");
  if (!error_flag) return cima_fail(CIMA_E_ARG, "gemm_tcgen05_pair: an error flag on the device is needed");
  if (epi == EPI_SWIGLU && (up_offset <= 0 || q_rows != 2 * up_offset || bias))
    return cima_fail(CIMA_E_SIZE, "gemm_tcgen05_pair: the gated epilogue needs Q = [gate | up], q_rows = 2 * up_offset, no bias");
  constexpr int BN = 256;
  const int q_feat = epi == EPI_SWIGLU ? up_offset : q_rows;
  const int out_cols = epi == EPI_SWIGLU ? BN / 2 : BN;
  const int tiles_q = (q_feat + out_cols - 1) / out_cols;
  const int p_tiles = (p_rows + 2 * BM - 1) / (2 * BM);
  CUtensorMap mp, mq;
  int rc = make_map(&mp, P, p_rows, K, K, BM);
  if (rc) return rc;
  rc = make_map(&mq, Q, q_rows, K, K, BN / 2);
  if (rc) return rc;
  PairArgs a{p_rows, q_rows, K, up_offset, bias, out, ldo, error_flag, act};
  switch (epi) {
    case EPI_STORE: return launch<BN, 6, EPI_STORE>(mp, mq, a, p_tiles, tiles_q, stream);
    case EPI_ACCUM: return launch<BN, 6, EPI_ACCUM>(mp, mq, a, p_tiles, tiles_q, stream);
    case EPI_SWIGLU: return launch<BN, 6, EPI_SWIGLU>(mp, mq, a, p_tiles, tiles_q, stream);
    case EPI_STORE_F32: return launch<BN, 6, EPI_STORE_F32>(mp, mq, a, p_tiles, tiles_q, stream);
  }
  return cima_fail(CIMA_E_ARG, "gemm_tcgen05_pair: epilogue %d is not one of 0..3", epi);
}
