// Causal grouped-query flash attention for several query rows per sequence (bfloat16): ragged batches in
// one launch.  Two sources of keys and values:
//   step  - the step's own qkv buffer (every sequence of the step starts at position 0, so key j of a
//           sequence is its row j): prompts;
//   cache - the layer's pages through the slot's block table (the step has appended its keys first): sequences
//           that go on by several tokens, at positions seq_len - rows .. seq_len - 1; a key tile is a page.
//
// One block = 64 query rows of one sequence x one head; its 4 warps own 16 rows each.  Key tiles
// of 64 rows stream through shared memory with cp.async (two in flight).  S = Q K^T and O += P V run
// on the tensor cores (mma.m16n8k16, bf16 in, f32 out); scores, running maximum, exponentials and
// sums are float32 (exponentials as 2^(s * scale * log2 e - m) by ex2.approx, whose error is far below
// the bfloat16 rounding of P);
// P is rounded to bfloat16 only as the operand of P V.  Key tiles wholly above the
// diagonal or wholly below the window are skipped.  The list of (sequence, first row) of the blocks
// comes from the host, heaviest first.
//
// Counterpart in the reference: k_attn_prefill_tiled (src/kernels.cu:659-753), one warp per query
// row on CUDA cores, same mask (:700-712).
//
// Accepts head_dim in {16, ..., 128} step 16; other sizes are refused and the caller takes the
// plain kernel.
#include "common.cuh"

namespace {

constexpr int BM = 64, BN = 64, WARPS = 4;

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(s), "l"(gmem));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* smem) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* smem) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ float ex2(float x) {          // 2^x, float32, about 2 ulp; 2^(-inf) = 0
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

template <int HD, bool FROM_CACHE>
__global__ void __launch_bounds__(WARPS * 32, 3)      // 3 blocks per SM: at most 168 registers
k_attention_prefill(const __nv_bfloat16* __restrict__ qkv, int ld, const int* __restrict__ tile_seq,
                    const int* __restrict__ tile_row0, const int* __restrict__ seq_first_row,
                    const __nv_bfloat16* __restrict__ cache, CimaPaged pg, const int* __restrict__ seq_slot,
                    const int* __restrict__ seq_len,
                    __nv_bfloat16* __restrict__ out, int ldo, int T, int nh, int nkv, float scale, int window) {
  cima_pdl_wait();
  constexpr int ROW = HD + 8;
  constexpr int TILE = BN * ROW;
  constexpr int KSTEPS = HD / 16, NTILES = HD / 8, CPR = HD / 8;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __nv_bfloat16* tiles = reinterpret_cast<__nv_bfloat16*>(smem_raw);     // [2 stages][K|V][BN][ROW]

  // blocks are numbered (tile, head) with the head running fastest, the tiles heaviest first: the hardware hands
  // blocks out in that order, so every head's heaviest tile starts before any lighter one
  const int tile = blockIdx.x / nh;
  const int seq = tile_seq[tile];
  const int q0 = tile_row0[tile];                     // first query row of this block among the sequence's rows
  const int first = seq_first_row[seq];
  const int len = seq_first_row[seq + 1] - first;     // rows of the sequence in this step
  const int start = FROM_CACHE ? seq_len[seq] - len : 0;       // position of the sequence's first row
  const int slot = FROM_CACHE ? seq_slot[seq] : 0;
  const int h = blockIdx.x % nh, kvh = h / (nh / nkv);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int kcol = (nh + kvh) * HD, vcol = (nh + nkv + kvh) * HD;
  const float sc2 = scale * 1.4426950408889634f;       // scores are kept in the base-2 domain

  // this thread's two query rows (among the sequence's rows; their positions are start + row)
  const int r0 = q0 + warp * 16 + g, r1 = r0 + 8;
  uint32_t q[KSTEPS][4];
  {
    const __nv_bfloat16* qa = qkv + (size_t)(first + min(r0, len - 1)) * ld + (size_t)h * HD;
    const __nv_bfloat16* qb = qkv + (size_t)(first + min(r1, len - 1)) * ld + (size_t)h * HD;
#pragma unroll
    for (int kk = 0; kk < KSTEPS; kk++) {
      const int d = kk * 16 + 2 * t;
      q[kk][0] = *reinterpret_cast<const uint32_t*>(qa + d);
      q[kk][1] = *reinterpret_cast<const uint32_t*>(qb + d);
      q[kk][2] = *reinterpret_cast<const uint32_t*>(qa + d + 8);
      q[kk][3] = *reinterpret_cast<const uint32_t*>(qb + d + 8);
    }
  }
  float o[NTILES][4];
#pragma unroll
  for (int j = 0; j < NTILES; j++)
#pragma unroll
    for (int e = 0; e < 4; e++) o[j][e] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};

  // key tiles the block needs: from the first key in any row's window to the last row's diagonal
  const int last_q = min(q0 + BM, len) - 1;
  const int lo_key = (window > 0 && start + q0 + 1 > window) ? start + q0 + 1 - window : 0;
  const int t0 = lo_key / BN, t1 = (start + last_q) / BN + 1;

  auto issue = [&](int kt, int stage) {
    __nv_bfloat16* dst = tiles + (size_t)stage * 2 * TILE;
    if constexpr (FROM_CACHE) {
      // tile kt is the page of positions [64 kt, 64 kt + 64): K then V, each [64][HD] contiguous.  What a page holds
      // beyond the sequence's end is finite (zeros or an earlier sequence's keys) and lies above every row's diagonal
      int e = kt;
      if (pg.ring) e %= pg.ring;
      const int page = pg.table[(size_t)slot * pg.width + e];
      const __nv_bfloat16* src = cache + (((size_t)page * 2) * pg.kv_heads + kvh) * (size_t)(BN * HD);
      const size_t vofs = (size_t)pg.kv_heads * BN * HD;
      for (int c = threadIdx.x; c < BN * CPR; c += WARPS * 32) {
        const int r = c / CPR, cc = c % CPR;
        cp_async16(dst + r * ROW + cc * 8, src + r * HD + cc * 8);
        cp_async16(dst + TILE + r * ROW + cc * 8, src + vofs + r * HD + cc * 8);
      }
    } else {
      for (int c = threadIdx.x; c < BN * CPR; c += WARPS * 32) {
        const int r = c / CPR, cc = c % CPR;
        const int grow = first + kt * BN + r;         // global row of this key
        if (grow < T) {
          const __nv_bfloat16* src = qkv + (size_t)grow * ld;
          cp_async16(dst + r * ROW + cc * 8, src + kcol + cc * 8);
          cp_async16(dst + TILE + r * ROW + cc * 8, src + vcol + cc * 8);
        } else {                                      // beyond the step's rows: zeros, so that 0 * V stays 0
          *reinterpret_cast<uint4*>(dst + r * ROW + cc * 8) = make_uint4(0u, 0u, 0u, 0u);
          *reinterpret_cast<uint4*>(dst + TILE + r * ROW + cc * 8) = make_uint4(0u, 0u, 0u, 0u);
        }
      }
    }
  };

  issue(t0, 0);
  cp_async_commit();
  for (int kt = t0; kt < t1; kt++) {
    const int stage = (kt - t0) & 1;
    if (kt + 1 < t1) issue(kt + 1, stage ^ 1);
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();
    const __nv_bfloat16* Kt = tiles + (size_t)stage * 2 * TILE;
    const __nv_bfloat16* Vt = Kt + TILE;

    float s[8][4];
#pragma unroll
    for (int j = 0; j < 8; j++)
#pragma unroll
      for (int e = 0; e < 4; e++) s[j][e] = 0.f;
    // fragments of the next k-step are fetched while the tensor cores work on the current one
    uint32_t kb[2][4][4];
#pragma unroll
    for (int jp = 0; jp < 4; jp++)
      ldmatrix_x4(kb[0][jp], Kt + (jp * 16 + (lane & 7) + 8 * (lane >> 4)) * ROW + 8 * ((lane >> 3) & 1));
#pragma unroll
    for (int kk = 0; kk < KSTEPS; kk++) {
      const int cur = kk & 1;
      if (kk + 1 < KSTEPS) {
#pragma unroll
        for (int jp = 0; jp < 4; jp++)
          ldmatrix_x4(kb[cur ^ 1][jp], Kt + (jp * 16 + (lane & 7) + 8 * (lane >> 4)) * ROW + (kk + 1) * 16 + 8 * ((lane >> 3) & 1));
      }
#pragma unroll
      for (int jp = 0; jp < 4; jp++) {
        mma_bf16(s[2 * jp], q[kk][0], q[kk][1], q[kk][2], q[kk][3], kb[cur][jp][0], kb[cur][jp][1]);
        mma_bf16(s[2 * jp + 1], q[kk][0], q[kk][1], q[kk][2], q[kk][3], kb[cur][jp][2], kb[cur][jp][3]);
      }
    }
    // Scores in the base-2 domain: t = s * scale * log2(e), p = 2^(t - m).  Only tiles that touch the
    // diagonal or the window's lower edge need the mask (a warp-uniform choice).
    const int key_base = kt * BN;
    const int wr0 = start + q0 + warp * 16;            // this warp's first query position
    const bool masked = key_base + BN - 1 > wr0 || (window > 0 && wr0 + 15 - key_base >= window);
    float mx[2] = {-INFINITY, -INFINITY};
    if (masked) {
#pragma unroll
      for (int j = 0; j < 8; j++)
#pragma unroll
        for (int e = 0; e < 4; e++) {
          const int key = key_base + j * 8 + 2 * t + (e & 1);
          const int qp = start + ((e >> 1) ? r1 : r0);
          const bool seen = key <= qp && (window <= 0 || qp - key < window);
          const float v = seen ? s[j][e] * sc2 : -INFINITY;
          s[j][e] = v;
          mx[e >> 1] = fmaxf(mx[e >> 1], v);
        }
    } else {
#pragma unroll
      for (int j = 0; j < 8; j++)
#pragma unroll
        for (int e = 0; e < 4; e++) {
          const float v = s[j][e] * sc2;
          s[j][e] = v;
          mx[e >> 1] = fmaxf(mx[e >> 1], v);
        }
    }
    float corr[2], msafe[2];
#pragma unroll
    for (int r = 0; r < 2; r++) {
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
      const float mnew = fmaxf(m_run[r], mx[r]);
      msafe[r] = mnew == -INFINITY ? 0.f : mnew;
      corr[r] = ex2(m_run[r] - msafe[r]);
      m_run[r] = mnew;
    }
    float psum[2] = {0.f, 0.f};
#pragma unroll
    for (int j = 0; j < 8; j++)
#pragma unroll
      for (int e = 0; e < 4; e++) {
        const float pv = ex2(s[j][e] - msafe[e >> 1]);
        s[j][e] = pv;
        psum[e >> 1] += pv;
      }
#pragma unroll
    for (int r = 0; r < 2; r++) {
      psum[r] += __shfl_xor_sync(0xffffffffu, psum[r], 1);
      psum[r] += __shfl_xor_sync(0xffffffffu, psum[r], 2);
      l_run[r] = l_run[r] * corr[r] + psum[r];
    }
    // the accumulator is rescaled only when some row's maximum moved (after the first tiles it rarely does)
    if (__any_sync(0xffffffffu, corr[0] != 1.0f || corr[1] != 1.0f)) {
#pragma unroll
      for (int j = 0; j < NTILES; j++) {
        o[j][0] *= corr[0]; o[j][1] *= corr[0];
        o[j][2] *= corr[1]; o[j][3] *= corr[1];
      }
    }
#pragma unroll
    for (int ks = 0; ks < 4; ks++) {                  // 16 keys per k-step
      const uint32_t a0 = pack_bf16(s[2 * ks][0], s[2 * ks][1]), a1 = pack_bf16(s[2 * ks][2], s[2 * ks][3]);
      const uint32_t a2 = pack_bf16(s[2 * ks + 1][0], s[2 * ks + 1][1]), a3 = pack_bf16(s[2 * ks + 1][2], s[2 * ks + 1][3]);
#pragma unroll
      for (int j = 0; j < NTILES; j += 2) {
        uint32_t vb[4];
        ldmatrix_x4_trans(vb, Vt + (ks * 16 + (lane & 7) + 8 * ((lane >> 3) & 1)) * ROW + j * 8 + 8 * (lane >> 4));
        mma_bf16(o[j], a0, a1, a2, a3, vb[0], vb[1]);
        mma_bf16(o[j + 1], a0, a1, a2, a3, vb[2], vb[3]);
      }
    }
    __syncthreads();
  }
  cp_async_wait<0>();

  const float inv0 = l_run[0] > 0.f ? 1.0f / l_run[0] : 0.f, inv1 = l_run[1] > 0.f ? 1.0f / l_run[1] : 0.f;
#pragma unroll
  for (int j = 0; j < NTILES; j++) {
    const int d = j * 8 + 2 * t;
    if (r0 < len)
      *reinterpret_cast<uint32_t*>(out + (size_t)(first + r0) * ldo + (size_t)h * HD + d) = pack_bf16(o[j][0] * inv0, o[j][1] * inv0);
    if (r1 < len)
      *reinterpret_cast<uint32_t*>(out + (size_t)(first + r1) * ldo + (size_t)h * HD + d) = pack_bf16(o[j][2] * inv1, o[j][3] * inv1);
  }
}

template <int HD, bool FROM_CACHE>
int launch_prefill(const void* qkv, int ld, const int* tile_seq, const int* tile_row0, const int* seq_first_row,
                   const void* cache, const CimaPaged& pg, const int* seq_slot, const int* seq_len,
                   void* out, int ldo, int T, int n_tiles, int nh, int nkv, float scale, int window, cudaStream_t stream) {
  if ((long long)n_tiles * nh > 0x7fffffffll) return cima_fail(CIMA_E_SIZE, "attention_prefill: %d blocks of rows x %d heads exceed one launch", n_tiles, nh);
  auto kern = k_attention_prefill<HD, FROM_CACHE>;
  const size_t smem = (size_t)2 * 2 * BN * (HD + 8) * sizeof(__nv_bfloat16);
  static bool raised = false;
  if (smem > 48 * 1024 && !raised) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return cima_fail((int)e, "attention_prefill: cannot raise shared memory to %zu bytes: %s", smem, cudaGetErrorString(e));
    raised = true;
  }
  { int rc_ = cima_launch(kern, dim3((unsigned)n_tiles * (unsigned)nh), dim3(WARPS * 32), (size_t)(smem), stream, 1, (const __nv_bfloat16*)qkv, ld, tile_seq, tile_row0, seq_first_row,
                                                        (const __nv_bfloat16*)cache, pg, seq_slot, seq_len,
                                                        (__nv_bfloat16*)out, ldo, T, nh, nkv, scale, window); if (rc_) return rc_; }
  return cima_launch_result();
}

}  // namespace

static int prefill_checks(const char* who, const void* qkv, int ld, const void* out, int ldo, int hd, int nh, int nkv) {
  if (hd % 16 || hd < 16 || hd > 128) return cima_fail(CIMA_E_SIZE, "%s: head_dim %d; this kernel takes multiples of 16 up to 128", who, hd);
  if (nh <= 0 || nkv <= 0 || nh % nkv || nh > 65535) return cima_fail(CIMA_E_SIZE, "%s: %d heads / %d kv heads are not accepted", who, nh, nkv);
  if (ld % 8 || ldo % 2 || ((uintptr_t)qkv & 15) || ((uintptr_t)out & 3))
    return cima_fail(CIMA_E_ARG, "%s: qkv rows must be 16-byte aligned (row stride %d a multiple of 8)", who, ld);
  return 0;
}

// tile_seq / tile_row0 [n_tiles]: the sequence and the first query row of each block of 64 rows.
extern "C" int cima_attention_prefill(const void* qkv, int ld, const int* tile_seq, const int* tile_row0,
                                      const int* seq_first_row, void* out, int ldo, int T, int n_tiles, int nh, int nkv,
                                      int hd, float scale, int window, cudaStream_t stream) {
  if (T <= 0 || n_tiles <= 0) return 0;
  if (int rc = prefill_checks("attention_prefill", qkv, ld, out, ldo, hd, nh, nkv)) return rc;
  const CimaPaged none{nullptr, 0, 0, BN, nkv, hd};
#define CASE(H) case H: return launch_prefill<H, false>(qkv, ld, tile_seq, tile_row0, seq_first_row, nullptr, none, nullptr, nullptr, out, ldo, T, n_tiles, nh, nkv, scale, window, stream)
  switch (hd) {
    CASE(16); CASE(32); CASE(48); CASE(64); CASE(80); CASE(96); CASE(112); CASE(128);
  }
#undef CASE
  return cima_fail(CIMA_E_SIZE, "attention_prefill: head_dim %d is not instantiated", hd);
}

// The same for sequences that go on: the rows of sequence s are the positions seq_len[s] - rows .. seq_len[s] - 1,
// and every key, the step's own included, is read from the layer's pages (64 positions each).
extern "C" int cima_attention_extend(const void* qkv, int ld, const int* tile_seq, const int* tile_row0,
                                     const int* seq_first_row, const void* cache, const int* table, int table_width,
                                     int ring, int page_size, const int* seq_slot, const int* seq_len, void* out, int ldo,
                                     int T, int n_tiles, int nh, int nkv, int hd, float scale, int window,
                                     cudaStream_t stream) {
  if (T <= 0 || n_tiles <= 0) return 0;
  if (int rc = prefill_checks("attention_extend", qkv, ld, out, ldo, hd, nh, nkv)) return rc;
  if (page_size != BN) return cima_fail(CIMA_E_SIZE, "attention_extend: page size %d; this kernel takes %d", page_size, BN);
  if (!cache || !table || !seq_slot || !seq_len || ((uintptr_t)cache & 15)) return cima_fail(CIMA_E_ARG, "attention_extend: the cache (16-byte aligned), its block table, slots and lengths are needed");
  const CimaPaged pg{table, table_width, ring, page_size, nkv, hd};
#define CASE(H) case H: return launch_prefill<H, true>(qkv, ld, tile_seq, tile_row0, seq_first_row, cache, pg, seq_slot, seq_len, out, ldo, T, n_tiles, nh, nkv, scale, window, stream)
  switch (hd) {
    CASE(16); CASE(32); CASE(48); CASE(64); CASE(80); CASE(96); CASE(112); CASE(128);
  }
#undef CASE
  return cima_fail(CIMA_E_SIZE, "attention_extend: head_dim %d is not instantiated", hd);
}
