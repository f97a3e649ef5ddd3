// Causal (and windowed) attention of ragged prompts on the fifth-generation tensor cores, head_dim 64 or 128
// (whole 128-byte rows of 64 bfloat16 for the swizzled tiles).
//
// One block computes 128 query rows of one head.  Both products of a tile of 64 keys run as tcgen05.mma with
// their results in tensor memory:
//     S = Q K^T      128 x 64, K-major operands straight from the q/k/v buffer by TMA
//     O += P V       P stays in tensor memory: a softmax thread writes its row's 64 probabilities (bfloat16, 32
//                    words) over the first columns of the S it has just read, and the tensor core takes them from
//                    there as the A operand; V is taken as it lies in the buffer ([keys, dims], dims contiguous):
//                    for this product the dims are N, so the operand is MN-major
// Warp roles (192 threads): warps 0..3 softmax, one thread per query row (a row's maximum and sum need no
// shuffles; each warp reads the 32 TMEM lanes it may access); warp 4 TMA producer; warp 5 TMEM allocation and
// MMA issue.  S has two buffers in TMEM, so the tensor cores compute S of the next tile while the softmax of the
// current one runs (a buffer is free for the tile after next once P V of its tile has completed).  Two blocks
// share an SM (98 KB of shared memory at head_dim 128 and 256 TMEM columns each): a softmax warp alone on its
// scheduler issues one instruction every four cycles, two hide each other's latencies, and the tensor cores
// serve one block while the other exponentiates.  Scores, maxima, exponentials and sums are float32 in the
// base-2 domain; P is rounded to bfloat16 only as operand of P V, the row sums are taken before that rounding.
// O is rescaled in TMEM only when a row's maximum has grown by more than 2^8 over the reference of its
// exponentials.
//
// Two sources of keys and values, as in the mma.sync kernel: the step's own q/k/v buffer (prompts that start at
// position 0), or the layer's pages in the cache (sequences that go on by many tokens: their rows stand at positions
// seq_len - rows .. seq_len - 1, a tile of 64 keys is a page, fetched by TMA through the slot's block table).
//
// Every wait on an mbarrier is bounded (2 s); a wait that runs out sets *error_flag, and all roles leave their
// loops, free the tensor memory and return.
//
// The reference's prefill attention is k_attn_prefill_tiled (src/kernels.cu:659-753): one warp per query row,
// online softmax on CUDA cores; it has no tensor-core attention.
#include "tcgen05.cuh"

namespace {

using namespace cima_tc;

constexpr int BM = 128;            // query rows per block = TMEM lanes
constexpr int BN = 64;             // keys per tile
constexpr int UMMA_K = 16;
constexpr int THREADS = 192;
constexpr int HALF_BYTES = 128 * 64 * 2;     // 128 rows of 64 bf16: one 128-byte-swizzled block, 16 KB
constexpr int KHALF_BYTES = BN * 64 * 2;     // 64 keys of 64 dims: 8 KB

__device__ __forceinline__ float ex2(float x) {          // 2^x, float32, about 2 ulp; 2^(-inf) = 0
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

struct AttnArgs {
  const int* tile_seq;          // [tiles] sequence of the block of 128 query rows
  const int* tile_row0;         // [tiles] first query row of the block among the sequence's rows
  const int* seq_first_row;     // [seqs + 1]
  const int* seq_len;           // keys from the cache: [seqs] positions held after the step
  const int* seq_slot;          //                      [seqs]
  const int* table;             //                      [slots, table_width] pages
  int table_width, ring;
  __nv_bfloat16* out;           // [T, ldo]
  int ldo, nh, nkv, window;
  float scale;
  int* error_flag;
};

// Keys of a query block whose rows stand at positions p0 .. (at most p0 + 127, below len): tiles [first, last] of 64.
__device__ __forceinline__ void key_tiles(int p0, int len, int window, int& first, int& last) {
  const int q_hi = min(p0 + BM, len) - 1;                      // last query position of the block
  const int lo = window > 0 ? max(0, p0 - window + 1) : 0;      // first key any row of the block sees
  first = lo / BN;
  last = q_hi / BN;
}

template <int HD, bool FROM_CACHE>
__global__ void __launch_bounds__(THREADS, 2)
k_attention_prefill_tc(const __grid_constant__ CUtensorMap map_qkv, const __grid_constant__ CUtensorMap map_k,
                       AttnArgs a) {
  cima_pdl_wait();
  extern __shared__ __align__(1024) unsigned char smem[];      // tiles of 1024-byte groups: checked below
  constexpr int NH = HD / 64;                                  // blocks of 64 dims in a row of Q or K
  constexpr int V_BYTES = HD * 64 * 2;                         // V of a tile: NH blocks of [64 keys][64 dims]
  unsigned char* sq = smem;                                    // Q: NH blocks (dims 0..63, 64..127) of 16 KB
  unsigned char* sk = sq + NH * HALF_BYTES;                    // K: [2 stages][NH blocks of 64 dims][64 keys]
  unsigned char* sv = sk + 2 * NH * KHALF_BYTES;               // V: [2 stages][NH blocks of 64 dims][64 keys]
  unsigned long long* bars = (unsigned long long*)(sv + 2 * V_BYTES);
  unsigned long long* q_full = bars;                           // [1]
  unsigned long long* k_full = bars + 1;                       // [2]
  unsigned long long* k_empty = bars + 3;                      // [2]  K's place is free once S of its tile is done,
  unsigned long long* v_full = bars + 5;                       // [2]  long before V's (after P V): the two rings run
  unsigned long long* v_empty = bars + 7;                      // [2]  apart, so K is fetched two tiles ahead
  unsigned long long* s_full = bars + 9;                       // [2]
  unsigned long long* p_full = bars + 11;                      // [2]  one per buffer of S, as s_full: see the softmax warps
  unsigned long long* pv_done = bars + 13;                     // [1]
  unsigned* tmem_slot = (unsigned*)(bars + 14);
  volatile int* abort_flag = (volatile int*)(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // blocks are numbered (tile, head) with the head running fastest, the tiles heaviest first: the hardware hands
  // blocks out in that order, so every head's heaviest tile starts before any lighter one
  const int tile = blockIdx.x / a.nh, h = blockIdx.x % a.nh, kvh = h / (a.nh / a.nkv);
  const int seq = a.tile_seq[tile], r0 = a.tile_row0[tile];
  const int row_base = a.seq_first_row[seq];
  const int rows = a.seq_first_row[seq + 1] - row_base;       // rows of the sequence in this step
  const int len = FROM_CACHE ? a.seq_len[seq] : rows;         // positions it holds after the step
  const int q0 = len - rows + r0;                             // position of the block's first query row
  const int slot = FROM_CACHE ? a.seq_slot[seq] : 0;
  int first, last;
  key_tiles(q0, len, a.window, first, last);
  const int n = last - first + 1;

  if (threadIdx.x == 0 && (smem_u32(smem) & 1023u)) atomicExch(a.error_flag, 2);   // never seen; the tiles would be misread
  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < 2; s++) {
      mbar_init(&k_full[s], 1); mbar_init(&k_empty[s], 1); mbar_init(&v_full[s], 1); mbar_init(&v_empty[s], 1);
      mbar_init(&s_full[s], 1);
      mbar_init(&p_full[s], 4);
    }
    mbar_init(pv_done, 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 5) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(256) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const unsigned tmem_base = *tmem_slot;
  const unsigned tm_s[2] = {tmem_base, tmem_base + 64u};
  const unsigned tm_o = tmem_base + 128u;

  if (warp == 4) {
    // ---------------------------------------------------------------- TMA producers: lane 0 Q and K, lane 1 V
    auto page_of = [&](int tile) -> int {               // the page that holds positions [64 tile, 64 tile + 64)
      int e = tile;
      if (a.ring) e %= a.ring;
      return a.table[(size_t)slot * a.table_width + e];
    };
    if (lane == 0) {
      mbar_expect_tx(q_full, NH * HALF_BYTES);
#pragma unroll
      for (int kb = 0; kb < NH; kb++) tma_load_2d(sq + (size_t)kb * HALF_BYTES, &map_qkv, h * HD + 64 * kb, row_base + r0, q_full);
      for (int j = 0; j < n; j++) {
        const int s = j & 1, k0 = (first + j) * BN;
        if (j >= 2 && !mbar_wait(&k_empty[s], ((j >> 1) - 1) & 1, a.error_flag, abort_flag)) break;
        mbar_expect_tx(&k_full[s], NH * KHALF_BYTES);
        // from the cache, map_k covers the layer's pages as rows of head_dim values: page, k or v, kv head, position
        const int x = FROM_CACHE ? 0 : (a.nh + kvh) * HD, y = FROM_CACHE ? (page_of(first + j) * 2 * a.nkv + kvh) * BN : row_base + k0;
#pragma unroll
        for (int kb = 0; kb < NH; kb++)
          tma_load_2d(sk + (size_t)(NH * s + kb) * KHALF_BYTES, &map_k, x + 64 * kb, y, &k_full[s]);
      }
    } else if (lane == 1) {
      for (int j = 0; j < n; j++) {
        const int s = j & 1, k0 = (first + j) * BN;
        if (j >= 2 && !mbar_wait(&v_empty[s], ((j >> 1) - 1) & 1, a.error_flag, abort_flag)) break;
        mbar_expect_tx(&v_full[s], V_BYTES);
        const int x = FROM_CACHE ? 0 : (a.nh + a.nkv + kvh) * HD;
        const int y = FROM_CACHE ? ((page_of(first + j) * 2 + 1) * a.nkv + kvh) * BN : row_base + k0;
#pragma unroll
        for (int kb = 0; kb < NH; kb++)
          tma_load_2d(sv + (size_t)s * V_BYTES + (size_t)kb * KHALF_BYTES, &map_k, x + 64 * kb, y, &v_full[s]);
      }
    }
  } else if (warp == 5) {
    // ---------------------------------------------------------------- MMA issue (one thread)
    if (lane == 0) {
      const unsigned idesc_s = umma_idesc(BM, BN), idesc_o = umma_idesc(BM, HD) | (1u << 16);   // B of P V is MN-major
      auto issue_s = [&](int j) {                       // S(j) = Q K(j)^T into buffer j & 1
        const int s = j & 1;
#pragma unroll
        for (int kb = 0; kb < NH; kb++) {
          const unsigned long long qd = umma_smem_desc(smem_u32(sq + (size_t)kb * HALF_BYTES));
          const unsigned long long kd = umma_smem_desc(smem_u32(sk + (size_t)(NH * s + kb) * KHALF_BYTES));
#pragma unroll
          for (int k = 0; k < 64 / UMMA_K; k++)
            umma_bf16(tm_s[s], qd + (unsigned long long)(k * 2), kd + (unsigned long long)(k * 2), idesc_s, (kb | k) ? 1u : 0u);
        }
        umma_commit(&s_full[s]);
        umma_commit(&k_empty[s]);                       // K's place is free when these have read it
      };
      bool ok = mbar_wait(q_full, 0, a.error_flag, abort_flag) && mbar_wait(&k_full[0], 0, a.error_flag, abort_flag);
      if (ok) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        issue_s(0);
      }
      for (int j = 0; j < n && ok; j++) {
        if (j + 1 < n) {
          const int s1 = (j + 1) & 1;
          ok = mbar_wait(&k_full[s1], ((j + 1) >> 1) & 1, a.error_flag, abort_flag);
          // buffer s1 held S of tile j - 1 and then its P: free once P V of tile j - 1 has completed
          if (ok && j + 1 >= 2) ok = mbar_wait(pv_done, (j - 1) & 1, a.error_flag, abort_flag);
          if (!ok) break;
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          issue_s(j + 1);
        }
        ok = mbar_wait(&v_full[j & 1], (j >> 1) & 1, a.error_flag, abort_flag) && mbar_wait(&p_full[j & 1], (j >> 1) & 1, a.error_flag, abort_flag);
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const int s = j & 1;
        {                                               // O += P V(j): 64 keys; P from tensor memory (the first 32 columns of S's buffer)
          // V as it lies in the buffer, [keys][dims]: the dims (N) are contiguous, 16 keys further is 16 rows of 128 bytes
          const unsigned long long vd = umma_smem_desc_mn(smem_u32(sv + (size_t)s * V_BYTES), KHALF_BYTES);
#pragma unroll
          for (int k = 0; k < BN / UMMA_K; k++)
            umma_bf16_ts(tm_o, tm_s[s] + (unsigned)(k * (UMMA_K / 2)), vd + (unsigned long long)(k * (UMMA_K * 128 >> 4)), idesc_o, (j | k) ? 1u : 0u);
        }
        umma_commit(&v_empty[s]);
        umma_commit(pv_done);
      }
    }
  } else {
    // ---------------------------------------------------------------- softmax: thread = query row
    const int r = warp * 32 + lane;                     // row of the block = TMEM lane
    const int pos = q0 + r;                             // its position in the sequence
    const unsigned lane_off = (unsigned)(warp * 32) << 16;
    const float sc2 = a.scale * 1.4426950408889634f;
    float m_run = -INFINITY, l_run = 0.f;
    bool ok = true;
    for (int j = 0; j < n && ok; j++) {
      const int s = j & 1, k0 = (first + j) * BN;
      ok = mbar_wait(&s_full[s], (j >> 1) & 1, a.error_flag, abort_flag);
      if (!ok) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      // does any key of this tile need the mask for any row of the block?
      const bool masked = k0 + BN > q0 + 1 || k0 + BN > len || (a.window > 0 && k0 < q0 + BM - a.window);
      const int key_hi = min(pos, len - 1);             // last key this row sees
      const int key_lo = a.window > 0 ? pos - a.window + 1 : 0;
      // the row's scores: the loads in flight together, one wait
      constexpr int NC = BN / 32;
      unsigned raw[NC][32];
#pragma unroll
      for (int c = 0; c < NC; c++) tmem_ld32_issue(tm_s[s] + lane_off + (unsigned)(c * 32), raw[c]);
      tmem_ld_wait();
      // maxima of the raw scores (the scale is positive): four chains instead of one
      float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
      if (masked) {
#pragma unroll
        for (int c = 0; c < NC; c++)
#pragma unroll
          for (int e = 0; e < 32; e++) {
            const int key = k0 + c * 32 + e;
            if (key > key_hi || key < key_lo) raw[c][e] = 0xff800000u;            // -inf
            mx4[e & 3] = fmaxf(mx4[e & 3], __uint_as_float(raw[c][e]));
          }
      } else {
#pragma unroll
        for (int c = 0; c < NC; c++)
#pragma unroll
          for (int e = 0; e < 32; e++) mx4[e & 3] = fmaxf(mx4[e & 3], __uint_as_float(raw[c][e]));
      }
      const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * sc2;
      // The reference point of the exponentials moves only when the row's maximum has grown by more than 2^8
      // since it was set: O and the sum stay consistent with whatever reference they were made with, the
      // probabilities stay below 2^8 (no harm in float32 or bfloat16), and O is rarely rescaled.
      float alpha = 1.0f;
      if (mx > m_run + 8.0f) {                          // also the first tile with a visible key (m_run = -inf)
        alpha = ex2(m_run - mx);                        // 2^(-inf) = 0 while nothing was seen
        m_run = mx;
      }
      const float neg_m = m_run == -INFINITY ? 0.f : -m_run;
      l_run *= alpha;
      // probabilities 2^(s * scale - m), summed in float32, packed as bfloat16 pairs in place
      float ps4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int c = 0; c < NC; c++)
#pragma unroll
        for (int e = 0; e < 32; e += 2) {
          const float p0 = ex2(fmaf(__uint_as_float(raw[c][e]), sc2, neg_m));
          const float p1 = ex2(fmaf(__uint_as_float(raw[c][e + 1]), sc2, neg_m));
          ps4[(e >> 1) & 3] += p0 + p1;
          const __nv_bfloat162 h2 = __floats2bfloat162_rn(p0, p1);
          raw[c][e >> 1] = *reinterpret_cast<const unsigned*>(&h2);
        }
      l_run += (ps4[0] + ps4[1]) + (ps4[2] + ps4[3]);
      // O may be touched once the previous tile's P V has completed
      if (j > 0 && __any_sync(0xffffffffu, alpha != 1.0f)) {
        ok = mbar_wait(pv_done, (j - 1) & 1, a.error_flag, abort_flag);
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        {
#pragma unroll 1
          for (int c = 0; c < HD / 32; c++) {
            float o[32];
            tmem_ld32(tm_o + lane_off + (unsigned)(c * 32), o);
#pragma unroll
            for (int e = 0; e < 32; e++) o[e] *= alpha;
            tmem_st32(tm_o + lane_off + (unsigned)(c * 32), o);
          }
        }
      }
      // P of the row, 64 bfloat16 as 32 words, over the first 32 columns of its S (this thread alone reads and
      // writes its lane of the buffer): the A operand of P V, read by the tensor core from tensor memory
      {
        unsigned pk[32];
#pragma unroll
        for (int c = 0; c < NC; c++)
#pragma unroll
          for (int e = 0; e < 16; e++) pk[c * 16 + e] = raw[c][e];
        tmem_st32_words(tm_s[s] + lane_off, pk);
      }
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      // P of tile j is announced on the barrier of its buffer, j & 1.  That barrier's last phase was tile j - 2, and S of
      // tile j was issued only after P V of tile j - 2 had completed: all four warps had arrived for it and the issuing
      // thread had seen that phase, so no waiter can be a phase behind.  (One barrier for both buffers would let the
      // warps, when no row rescales, announce tiles j and j + 1 while the issuing thread still waits for V of tile j;
      // its wait on the parity of tile j would then be answered by tile j + 2, which never comes.)
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_full[s]);
    }
    // A wait on a parity answers for the last phase of that parity.  This warp has S of tile n - 1, so P V of tile
    // n - 3 is complete, but that of tile n - 2 need not be: asked for tile n - 1 alone, the barrier would answer for
    // tile n - 3.  (Inside the loop a warp with S of tile j asks for tile j - 1 and cannot be answered for j - 3.)
    if (ok && n > 1) ok = mbar_wait(pv_done, (n - 2) & 1, a.error_flag, abort_flag);
    if (ok && n > 0) ok = mbar_wait(pv_done, (n - 1) & 1, a.error_flag, abort_flag);
    if (ok && n > 0) {
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const float inv = l_run > 0.f ? 1.0f / l_run : 0.f;
      __nv_bfloat16* dst = a.out + (size_t)(row_base + r0 + r) * a.ldo + (size_t)h * HD;
#pragma unroll 1
      for (int c = 0; c < HD / 32; c++) {
        float o[32];
        tmem_ld32(tm_o + lane_off + (unsigned)(c * 32), o);
        if (pos < len) {
#pragma unroll
          for (int q = 0; q < 4; q++) {
            uint4 t;
            __nv_bfloat162* h2 = reinterpret_cast<__nv_bfloat162*>(&t);
#pragma unroll
            for (int k = 0; k < 4; k++) h2[k] = __floats2bfloat162_rn(o[8 * q + 2 * k] * inv, o[8 * q + 2 * k + 1] * inv);
            *reinterpret_cast<uint4*>(dst + c * 32 + q * 8) = t;
          }
        }
      }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  }
  __syncthreads();
  if (warp == 5) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(256) : "memory");
  }
}

struct CacheSource {              // keys and values from a layer's pages; cache == nullptr: from the q/k/v buffer
  const void* cache;
  long long n_pages;
  const int *table, *seq_slot, *seq_len;
  int table_width, ring;
};

template <int HD, bool FROM_CACHE>
int launch_attention_tc(const void* qkv, int ld, const int* tile_seq, const int* tile_row0, const int* seq_first_row,
                        const CacheSource& c, void* out, int ldo, int T, int n_tiles, int nh, int nkv, float scale,
                        int window, int* error_flag, cudaStream_t stream) {
  if ((long long)n_tiles * nh > 0x7fffffffll) return cima_fail(CIMA_E_SIZE, "attention_prefill_tc: %d blocks of rows x %d heads exceed one launch", n_tiles, nh);
  CUtensorMap mq, mk;                                  // boxes of 128 rows (Q) and of 64 rows (K and V) by 64 columns
  int rc = make_map(&mq, qkv, T, (long long)(nh + 2 * nkv) * HD, ld);
  if (rc) return rc;
  if (FROM_CACHE) rc = make_map(&mk, c.cache, c.n_pages * 2 * nkv * BN, HD, HD, BN);
  else rc = make_map(&mk, qkv, T, (long long)(nh + 2 * nkv) * HD, ld, BN);
  if (rc) return rc;
  constexpr int NH = HD / 64;
  const size_t smem = NH * (size_t)HALF_BYTES + 2 * NH * (size_t)KHALF_BYTES + 2 * (size_t)HD * 128 + 14 * 8 + 16;
  static_assert(14 * 8 + 8 <= 14 * 8 + 16, "barriers and flags fit their place");
  static bool raised = false;
  if (!raised) {
    cudaError_t e = cudaFuncSetAttribute(k_attention_prefill_tc<HD, FROM_CACHE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return cima_fail((int)e, "attention_prefill_tc: cannot raise shared memory to %zu bytes: %s", smem, cudaGetErrorString(e));
    raised = true;
  }
  AttnArgs a{tile_seq, tile_row0, seq_first_row, c.seq_len, c.seq_slot, c.table, c.table_width, c.ring,
             (__nv_bfloat16*)out, ldo, nh, nkv, window, scale, error_flag};
  { int rc_ = cima_launch(k_attention_prefill_tc<HD, FROM_CACHE>, dim3((unsigned)n_tiles * (unsigned)nh), dim3(THREADS), smem, stream, 1, mq, mk, a); if (rc_) return rc_; }
  return cima_launch_result();
}

}  // namespace

static int tc_checks(const char* who, const void* qkv, int ld, const void* out, int ldo, int nh, int nkv, int hd, const int* error_flag) {
  if (hd != 64 && hd != 128) return cima_fail(CIMA_E_SIZE, "%s: head_dim %d; this kernel takes 64 or 128", who, hd);
  if (nh <= 0 || nkv <= 0 || nh % nkv) return cima_fail(CIMA_E_SIZE, "%s: %d heads are not a multiple of %d kv heads", who, nh, nkv);
  if (ld % 8 || ldo % 8) return cima_fail(CIMA_E_SIZE, "%s: row strides (%d, %d) must be multiples of 8", who, ld, ldo);
  if (ld < (nh + 2 * nkv) * hd) return cima_fail(CIMA_E_SIZE, "%s: row stride %d is smaller than (heads + 2 kv heads) * head_dim", who, ld);
  if ((((uintptr_t)qkv | (uintptr_t)out) & 15)) return cima_fail(CIMA_E_ARG, "%s: qkv and out must be 16-byte aligned", who);
  if (!error_flag) return cima_fail(CIMA_E_ARG, "%s: an error flag on the device is needed", who);
  if (nh > 65535 || nkv > 65535) return cima_fail(CIMA_E_SIZE, "%s: %d heads exceed one launch", who, nh);
  return 0;
}

// qkv [T, ld] bf16: q heads, k heads, v heads of each row, q and k already rotated.  tile_seq / tile_row0: the
// blocks of 128 query rows, heaviest first.  out [T, ldo].  head_dim is 64 or 128.
// error_flag: device int that a wait that ran out sets to 1 (never cleared here).
extern "C" int cima_attention_prefill_tc(const void* qkv, int ld, const int* tile_seq, const int* tile_row0,
                                         const int* seq_first_row, void* out, int ldo, int T, int n_tiles, int nh,
                                         int nkv, int hd, float scale, int window, int* error_flag, cudaStream_t stream) {
  if (T <= 0 || n_tiles <= 0) return 0;
  if (int rc = tc_checks("attention_prefill_tc", qkv, ld, out, ldo, nh, nkv, hd, error_flag)) return rc;
  const CacheSource none{nullptr, 0, nullptr, nullptr, nullptr, 0, 0};
  if (hd == 64)
    return launch_attention_tc<64, false>(qkv, ld, tile_seq, tile_row0, seq_first_row, none, out, ldo, T, n_tiles, nh, nkv, scale, window, error_flag, stream);
  return launch_attention_tc<128, false>(qkv, ld, tile_seq, tile_row0, seq_first_row, none, out, ldo, T, n_tiles, nh, nkv, scale, window, error_flag, stream);
}

// The same for sequences that go on: the rows of sequence s are the positions seq_len[s] - rows .. seq_len[s] - 1, and
// every key, the step's own included, is read from the layer's pages: cache [n_pages, 2, nkv, 64, head_dim] bf16.
extern "C" int cima_attention_extend_tc(const void* qkv, int ld, const int* tile_seq, const int* tile_row0,
                                        const int* seq_first_row, const void* cache, long long n_pages, const int* table,
                                        int table_width, int ring, int page_size, const int* seq_slot, const int* seq_len,
                                        void* out, int ldo, int T, int n_tiles, int nh, int nkv, int hd, float scale,
                                        int window, int* error_flag, cudaStream_t stream) {
  if (T <= 0 || n_tiles <= 0) return 0;
  if (int rc = tc_checks("attention_extend_tc", qkv, ld, out, ldo, nh, nkv, hd, error_flag)) return rc;
  if (page_size != BN) return cima_fail(CIMA_E_SIZE, "attention_extend_tc: page size %d; this kernel takes %d", page_size, BN);
  if (!cache || !table || !seq_slot || !seq_len || ((uintptr_t)cache & 15) || n_pages <= 0)
    return cima_fail(CIMA_E_ARG, "attention_extend_tc: the cache (16-byte aligned), its block table, slots and lengths are needed");
  if (n_pages * 2 * nkv * BN >= (1ll << 31)) return cima_fail(CIMA_E_SIZE, "attention_extend_tc: %lld pages exceed a tensor map's 32-bit row coordinate", n_pages);
  const CacheSource c{cache, n_pages, table, seq_slot, seq_len, table_width, ring};
  if (hd == 64)
    return launch_attention_tc<64, true>(qkv, ld, tile_seq, tile_row0, seq_first_row, c, out, ldo, T, n_tiles, nh, nkv, scale, window, error_flag, stream);
  return launch_attention_tc<128, true>(qkv, ld, tile_seq, tile_row0, seq_first_row, c, out, ldo, T, n_tiles, nh, nkv, scale, window, error_flag, stream);
}
