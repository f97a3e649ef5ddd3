// Decode attention over the paged cache (bfloat16): one new query per sequence, grouped-query,
// keys split across blocks ("split-KV") so that few sequences still fill the GPU.
//
// Grid (split, kv head x m-tile, sequence).  A block streams its share of the sequence's pages
// through shared memory with cp.async (two pages in flight) and serves ALL query heads of the
// kv head's group at once, so every key and value byte is read from HBM once per step: the group's
// heads are the 16 rows of the tensor-core tile (mma.m16n8k16, bf16 in, f32 out), the page's 64 keys
// are split over the 4 warps.  Scores, the running maximum, the exponentials and the sums are
// float32; probabilities are rounded to bfloat16 only as the operand of P.V.  Each warp keeps
// (max, sum, accumulator) of its keys; the warps, and then the splits, are merged by
// log-sum-exp in a fixed order (warp 0..3, split 0..S-1).
//
// The reference's decode attention has the same shape without tensor cores or batches: a block
// per (head, 128-key chunk) writing {m, l, acc[dim]} partials (k_attn_decode_split,
// src/kernels.cu:547-611) and a merge per head (k_attn_reduce, :615-639).
//
// Accepts head_dim in {16, 32, ..., 128}, page_size 64, any group size (16 heads per m-tile), any
// window; other sizes are refused with a sentence and the caller takes the plain kernel.
#include "common.cuh"

namespace {

constexpr int PS = 64;            // keys per page
constexpr int WARPS = 4;
constexpr int KEYS_PER_WARP = PS / WARPS;   // 16

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

constexpr int MAX_SPLITS = 64;
// Pages in flight per block: as many as fill about 104 KB of shared memory with their padded tiles, so that two blocks
// fit an SM whatever the head size and hold the same bytes in flight (3 pages of 34 KB at head_dim 128, 5 of 18 KB at
// 64; with 3 at every head size a block of 64-wide heads drew half the bandwidth).
__host__ __device__ constexpr int decode_stages(int hd) {
  const int n = (104 * 1024) / (2 * PS * (hd + 8) * 2);
  return n < 3 ? 3 : (n > 8 ? 8 : n);
}

// The splits that get pages of a sequence with ``len`` positions: at most one per page of the visible keys.
__device__ __forceinline__ int live_splits(int len, int window, int n_splits) {
  const int lo = (window > 0 && len > window) ? len - window : 0;
  return min(n_splits, (len - 1) / PS - lo / PS + 1);
}

// early: the sequence's lengths, slots and block table, and every page before the one that holds the newest
// position, are not written by the kernel launched just before this one (the q/k/v projection with its cache
// append writes the newest position only); the first pages are then fetched before the wait on that kernel.
template <int HD>
__global__ void __launch_bounds__(WARPS * 32)
k_attention_decode(const __nv_bfloat16* __restrict__ qkv, int ld, const __nv_bfloat16* __restrict__ cache,
                   CimaPaged pg, const int* __restrict__ seq_slot, const int* __restrict__ seq_len,
                   float* __restrict__ part_o, float* __restrict__ part_ml, __nv_bfloat16* __restrict__ out, int ldo,
                   int nh, int nkv, int mtiles, float scale, int window, int n_splits, int early) {
  if (!early) cima_pdl_wait();
  constexpr int ROW = HD + 8;                         // padded row of a tile, in elements (16 bytes of padding)
  constexpr int TILE = PS * ROW;                      // elements of one K or V tile
  constexpr int KSTEPS = HD / 16, NTILES = HD / 8;
  constexpr int STAGES = decode_stages(HD);
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __nv_bfloat16* tiles = reinterpret_cast<__nv_bfloat16*>(smem_raw);     // [STAGES][K|V][PS][ROW]

  const int split = blockIdx.x;
  const int kvh = blockIdx.y / mtiles, mt = blockIdx.y % mtiles;
  const int b = blockIdx.z;
  const int G = nh / nkv;
  const int h0 = kvh * G + mt * 16;                   // first query head of this m-tile
  const int rows = min(16, G - mt * 16);              // heads in this m-tile
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, t = lane & 3;

  const int len = seq_len[b];
  const float sc2 = scale * 1.4426950408889634f;        // scores, running maxima and partial m are in the base-2 domain
  const int slot = seq_slot[b];
  const int lo = (window > 0 && len > window) ? len - window : 0;
  const int pf = lo / PS, pl = (len - 1) / PS;
  const int npages = pl - pf + 1;
  // The pages are shared evenly among S = min(n_splits, pages) splits: split s takes pages [s n / S, (s + 1) n / S).
  // A launch sized for a long context (a captured step keeps its grid while the sequences grow) leaves the
  // blocks beyond S without work; the merge reads the first S partial results only (live_splits there).
  const int S = live_splits(len, window, n_splits);
  if (split >= S) return;
  const int p0 = pf + (int)((long long)split * npages / S);
  const int p1 = pf + (int)((long long)(split + 1) * npages / S);

  auto page_of = [&](int page_index) -> int {
    int e = page_index;
    if (pg.ring) e %= pg.ring;
    return pg.table[(size_t)slot * pg.width + e];
  };
  auto issue = [&](int page, int stage) {
    // one page: K then V, each [PS][HD] contiguous in the cache -> padded rows in shared memory
    const __nv_bfloat16* src = cache + (((size_t)page * 2) * pg.kv_heads + kvh) * (size_t)(PS * HD);
    const size_t vofs = (size_t)pg.kv_heads * PS * HD;
    __nv_bfloat16* dst = tiles + (size_t)stage * 2 * TILE;
    constexpr int CPR = HD / 8;                       // 16-byte chunks per row
    for (int c = threadIdx.x; c < PS * CPR; c += WARPS * 32) {
      const int r = c / CPR, cc = c % CPR;
      cp_async16(dst + r * ROW + cc * 8, src + r * HD + cc * 8);
      cp_async16(dst + TILE + r * ROW + cc * 8, src + vofs + r * HD + cc * 8);
    }
  };

  // Prologue: the first STAGES - 1 pages, one commit group each (empty past the end, so that the groups
  // count the same for every block).
  int ahead = 0;                                      // groups committed so far
  if (early) {
    while (ahead < STAGES - 1 && p0 + ahead < p1 && p0 + ahead < pl) {
      issue(page_of(p0 + ahead), ahead);
      cp_async_commit();
      ahead++;
    }
    cima_pdl_wait();
  }
  for (; ahead < STAGES - 1; ahead++) {
    if (p0 + ahead < p1) issue(page_of(p0 + ahead), ahead);
    cp_async_commit();
  }
  // the id of the page that the next iteration issues is looked up one iteration ahead, so that the table's
  // latency is not on the way of the copies
  int page_next = p0 + STAGES - 1 < p1 ? page_of(p0 + STAGES - 1) : 0;

  // the group's queries as A fragments: row g and g + 8 of the m-tile, 16 dims per k-step
  uint32_t q[KSTEPS][4];
  {
    const __nv_bfloat16* qb = qkv + (size_t)b * ld + (size_t)h0 * HD;
#pragma unroll
    for (int kk = 0; kk < KSTEPS; kk++) {
      const int d = kk * 16 + 2 * t;
      q[kk][0] = g < rows ? *reinterpret_cast<const uint32_t*>(qb + (size_t)g * HD + d) : 0u;
      q[kk][1] = g + 8 < rows ? *reinterpret_cast<const uint32_t*>(qb + (size_t)(g + 8) * HD + d) : 0u;
      q[kk][2] = g < rows ? *reinterpret_cast<const uint32_t*>(qb + (size_t)g * HD + d + 8) : 0u;
      q[kk][3] = g + 8 < rows ? *reinterpret_cast<const uint32_t*>(qb + (size_t)(g + 8) * HD + d + 8) : 0u;
    }
  }

  float o[NTILES][4];
#pragma unroll
  for (int j = 0; j < NTILES; j++)
#pragma unroll
    for (int e = 0; e < 4; e++) o[j][e] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};

  for (int p = p0; p < p1; p++) {
    const int stage = (p - p0) % STAGES;
    cp_async_wait<STAGES - 2>();                      // page p has landed (this thread's part of it)
    __syncthreads();                                   // ... everyone's; and page p - 1 is computed: its stage is free
    if (p + STAGES - 1 < p1) issue(page_next, (p - p0 + STAGES - 1) % STAGES);
    cp_async_commit();
    if (p + STAGES < p1) page_next = page_of(p + STAGES);
    const __nv_bfloat16* Kt = tiles + (size_t)stage * 2 * TILE;
    const __nv_bfloat16* Vt = Kt + TILE;
    const int kw = warp * KEYS_PER_WARP;              // this warp's keys within the page

    // S = Q K^T for 16 keys: two n-tiles of 8 keys
    float s[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
    for (int kk = 0; kk < KSTEPS; kk++) {
      uint32_t kb[4];
      ldmatrix_x4(kb, Kt + (kw + (lane & 7) + 8 * (lane >> 4)) * ROW + kk * 16 + 8 * ((lane >> 3) & 1));
      mma_bf16(s[0], q[kk][0], q[kk][1], q[kk][2], q[kk][3], kb[0], kb[1]);
      mma_bf16(s[1], q[kk][0], q[kk][1], q[kk][2], q[kk][3], kb[2], kb[3]);
    }
    // scale, mask what lies outside [lo, len), running softmax per row (rows g and g + 8)
    const int key0 = p * PS + kw;
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int j = 0; j < 2; j++)
#pragma unroll
      for (int e = 0; e < 4; e++) {
        const int key = key0 + j * 8 + 2 * t + (e & 1);
        const float v = (key >= lo && key < len) ? s[j][e] * sc2 : -INFINITY;
        s[j][e] = v;
        mx[e >> 1] = fmaxf(mx[e >> 1], v);
      }
    float corr[2], msafe[2];
#pragma unroll
    for (int r = 0; r < 2; r++) {
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
      const float mnew = fmaxf(m_run[r], mx[r]);
      msafe[r] = mnew == -INFINITY ? 0.f : mnew;
      corr[r] = ex2(m_run[r] - msafe[r]);               // 2^(-inf) = 0 while nothing was seen
      m_run[r] = mnew;
    }
    float psum[2] = {0.f, 0.f};
#pragma unroll
    for (int j = 0; j < 2; j++)
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
#pragma unroll
    for (int j = 0; j < NTILES; j++) {
      o[j][0] *= corr[0]; o[j][1] *= corr[0];
      o[j][2] *= corr[1]; o[j][3] *= corr[1];
    }
    // O += P V: P (16 x 16 keys) straight from the score registers
    const uint32_t a0 = pack_bf16(s[0][0], s[0][1]), a1 = pack_bf16(s[0][2], s[0][3]);
    const uint32_t a2 = pack_bf16(s[1][0], s[1][1]), a3 = pack_bf16(s[1][2], s[1][3]);
#pragma unroll
    for (int j = 0; j < NTILES; j += 2) {
      uint32_t vb[4];
      ldmatrix_x4_trans(vb, Vt + (kw + (lane & 7) + 8 * ((lane >> 3) & 1)) * ROW + j * 8 + 8 * (lane >> 4));
      mma_bf16(o[j], a0, a1, a2, a3, vb[0], vb[1]);
      mma_bf16(o[j + 1], a0, a1, a2, a3, vb[2], vb[3]);
    }
  }
  cp_async_wait<0>();
  __syncthreads();
  cima_pdl_trigger();

  // merge the 4 warps (fixed order) through shared memory, reusing the tiles' space
  float* so = reinterpret_cast<float*>(smem_raw);      // [WARPS][16][HD]
  float* sml = so + WARPS * 16 * HD;                   // [WARPS][16][2]
#pragma unroll
  for (int j = 0; j < NTILES; j++) {
    float* base = so + ((size_t)warp * 16 + g) * HD + j * 8 + 2 * t;
    base[0] = o[j][0]; base[1] = o[j][1];
    base[8 * HD] = o[j][2]; base[8 * HD + 1] = o[j][3];
  }
  if (t == 0) {
    sml[(warp * 16 + g) * 2] = m_run[0]; sml[(warp * 16 + g) * 2 + 1] = l_run[0];
    sml[(warp * 16 + g + 8) * 2] = m_run[1]; sml[(warp * 16 + g + 8) * 2 + 1] = l_run[1];
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < rows * HD; idx += WARPS * 32) {
    const int r = idx / HD, d = idx - r * HD;
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < WARPS; w++) M = fmaxf(M, sml[(w * 16 + r) * 2]);
    const float Ms = M == -INFINITY ? 0.f : M;
    float acc = 0.f, l = 0.f;
#pragma unroll
    for (int w = 0; w < WARPS; w++) {
      const float f = ex2(sml[(w * 16 + r) * 2] - Ms);
      acc += f * so[((size_t)w * 16 + r) * HD + d];
      l += f * sml[(w * 16 + r) * 2 + 1];
    }
    const int h = h0 + r;
    if (n_splits == 1) {
      out[(size_t)b * ldo + (size_t)h * HD + d] = __float2bfloat16_rn(l > 0.f ? acc / l : 0.f);
    } else {
      const size_t pi = ((size_t)b * nh + h) * n_splits + split;
      part_o[pi * HD + d] = acc;
      if (d == 0) { part_ml[pi * 2] = M; part_ml[pi * 2 + 1] = l; }
    }
  }
}

// out[b, h, :] = sum_s 2^(m_s - M) o_s / sum_s 2^(m_s - M) l_s over the splits that have pages.
// One block per (head, sequence).  The first warp loads every split's (m, l) at once (a lane per split, all loads
// independent), makes the weights 2^(m_s - M) and their sum with l by a shuffle tree (a fixed order, whatever the
// timing), and leaves them in shared memory; then a thread per dimension sums the splits' accumulators, eight
// independent loads at a time.  (A loop of one thread over the splits' l, as this kernel once had, costs a trip to
// L2 per split: 8 us at 32 splits.)
__global__ void __launch_bounds__(128)
k_attention_combine(const float* __restrict__ part_o, const float* __restrict__ part_ml, const int* __restrict__ seq_len,
                    __nv_bfloat16* __restrict__ out, int ldo, int nh, int hd, int window, int splits_launched) {
  cima_pdl_wait();
  __shared__ float w[MAX_SPLITS];
  __shared__ float s_inv;
  const int b = blockIdx.y, h = blockIdx.x;
  const size_t base = ((size_t)b * nh + h) * splits_launched;
  const int n_splits = live_splits(seq_len[b], window, splits_launched);
  if (threadIdx.x < 32) {
    float m[MAX_SPLITS / 32], l[MAX_SPLITS / 32];
    float M = -INFINITY;
#pragma unroll
    for (int i = 0; i < MAX_SPLITS / 32; i++) {
      const int s = threadIdx.x + 32 * i;
      const float2 ml = s < n_splits ? *reinterpret_cast<const float2*>(part_ml + (base + s) * 2) : make_float2(-INFINITY, 0.f);
      m[i] = ml.x;
      l[i] = ml.y;
      M = fmaxf(M, m[i]);
    }
    for (int o = 16; o > 0; o >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, o));
    const float Ms = M == -INFINITY ? 0.f : M;
    float L = 0.f;
#pragma unroll
    for (int i = 0; i < MAX_SPLITS / 32; i++) {
      const int s = threadIdx.x + 32 * i;
      const float ws = ex2(m[i] - Ms);                 // 0 for a split beyond n_splits or without keys
      if (s < n_splits) w[s] = ws;
      L += ws * l[i];
    }
    for (int o = 16; o > 0; o >>= 1) L += __shfl_xor_sync(0xffffffffu, L, o);
    if (threadIdx.x == 0) s_inv = L > 0.f ? 1.0f / L : 0.f;
  }
  __syncthreads();
  const float inv = s_inv;
  for (int d = threadIdx.x; d < hd; d += blockDim.x) {
    float acc = 0.f;
    int s = 0;
    for (; s + 8 <= n_splits; s += 8) {
      float o[8];
#pragma unroll
      for (int q = 0; q < 8; q++) o[q] = part_o[(base + s + q) * hd + d];
#pragma unroll
      for (int q = 0; q < 8; q++) acc += w[s + q] * o[q];
    }
    for (; s < n_splits; s++) acc += w[s] * part_o[(base + s) * hd + d];
    out[(size_t)b * ldo + (size_t)h * hd + d] = __float2bfloat16_rn(acc * inv);
  }
}

template <int HD>
int launch_decode(const void* qkv, int ld, const void* cache, CimaPaged pg, const int* seq_slot, const int* seq_len,
                  float* part_o, float* part_ml, void* out, int ldo, int B, int nh, int nkv, float scale, int window,
                  int n_splits, int early, cudaStream_t stream) {
  auto kern = k_attention_decode<HD>;
  constexpr int STAGES = decode_stages(HD);
  const size_t tiles = (size_t)STAGES * 2 * PS * (HD + 8) * sizeof(__nv_bfloat16);
  const size_t merge = (size_t)WARPS * 16 * (HD + 2) * sizeof(float);
  const size_t smem = tiles > merge ? tiles : merge;
  static bool raised = false;
  if (smem > 48 * 1024 && !raised) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return cima_fail((int)e, "attention_decode: cannot raise shared memory to %zu bytes: %s", smem, cudaGetErrorString(e));
    raised = true;
  }
  const int G = nh / nkv, mtiles = (G + 15) / 16;
  dim3 grid(n_splits, nkv * mtiles, B);
  { int rc_ = cima_launch(kern, dim3(grid), dim3(WARPS * 32), (size_t)(smem), stream, 1, (const __nv_bfloat16*)qkv, ld, (const __nv_bfloat16*)cache, pg, seq_slot,
                                           seq_len, part_o, part_ml, (__nv_bfloat16*)out, ldo, nh, nkv, mtiles, scale,
                                           window, n_splits, early); if (rc_) return rc_; }
  int rc = cima_launch_result();
  if (rc || n_splits == 1) return rc;
  { int rc_ = cima_launch(k_attention_combine, dim3(dim3(nh, B)), dim3(128), (size_t)(0), stream, 1, part_o, part_ml, seq_len, (__nv_bfloat16*)out, ldo, nh, HD, window, n_splits); if (rc_) return rc_; }
  return cima_launch_result();
}

}  // namespace

// One query row per sequence (row b of qkv belongs to sequence b).  part_o [B, nh, n_splits, hd] and
// part_ml [B, nh, n_splits, 2] float32 are scratch, needed when n_splits > 1.  early != 0: the caller states
// that the kernel launched just before this one writes neither seq_slot, seq_len, the block table nor any
// cache page before the one of each sequence's newest position; the first pages are then fetched before that
// kernel has finished.
extern "C" int cima_attention_decode(const void* qkv, int ld, const void* cache, const int* table, int table_width,
                                     int ring, int page_size, const int* seq_slot, const int* seq_len, float* part_o,
                                     float* part_ml, void* out, int ldo, int B, int nh, int nkv, int hd, float scale,
                                     int window, int n_splits, int early, cudaStream_t stream) {
  if (B <= 0) return 0;
  if (page_size != PS) return cima_fail(CIMA_E_SIZE, "attention_decode: page size %d; this kernel takes 64", page_size);
  if (hd % 16 || hd < 16 || hd > 128) return cima_fail(CIMA_E_SIZE, "attention_decode: head_dim %d; this kernel takes multiples of 16 up to 128", hd);
  if (nh <= 0 || nkv <= 0 || nh % nkv) return cima_fail(CIMA_E_SIZE, "attention_decode: %d heads are not a multiple of %d kv heads", nh, nkv);
  if (n_splits < 1 || n_splits > MAX_SPLITS || B > 65535) return cima_fail(CIMA_E_SIZE, "attention_decode: %d splits / %d sequences exceed one launch", n_splits, B);
  if (n_splits > 1 && (!part_o || !part_ml)) return cima_fail(CIMA_E_ARG, "attention_decode: more than one split needs the scratch buffers");
  if (ld % 2 || ((uintptr_t)qkv & 3) || ((uintptr_t)cache & 15)) return cima_fail(CIMA_E_ARG, "attention_decode: qkv rows must be 4-byte and the cache 16-byte aligned");
  CimaPaged pg{table, table_width, ring, page_size, nkv, hd};
#define CASE(H) case H: return launch_decode<H>(qkv, ld, cache, pg, seq_slot, seq_len, part_o, part_ml, out, ldo, B, nh, nkv, scale, window, n_splits, early != 0, stream)
  switch (hd) {
    CASE(16); CASE(32); CASE(48); CASE(64); CASE(80); CASE(96); CASE(112); CASE(128);
  }
#undef CASE
  return cima_fail(CIMA_E_SIZE, "attention_decode: head_dim %d is not instantiated", hd);
}

// ---------------------------------------------------------------------------------------------
// The same kernel for callers that cannot allocate (see attention_decode_static.h): the splits'
// partial results go to a fixed array of this library's device image instead of caller scratch.
// ---------------------------------------------------------------------------------------------
#include "attention_decode_static.h"

static __device__ __align__(256) float g_decode_static_scratch[CIMA_DECODE_STATIC_FLOATS];

// In host code the array's name is only a handle; kernels need its device address, which differs
// per device.  Looked up once per device, with that device current.
static float* decode_static_scratch_address(int* status) {
  constexpr int MAX_DEVICES = 64;
  static float* addr[MAX_DEVICES] = {nullptr};
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) { *status = cima_fail((int)e, "attention_decode_static: cudaGetDevice failed: %s", cudaGetErrorString(e)); return nullptr; }
  if (dev < 0 || dev >= MAX_DEVICES) { *status = cima_fail(CIMA_E_ARG, "attention_decode_static: device ordinal %d is beyond %d", dev, MAX_DEVICES); return nullptr; }
  if (!addr[dev]) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_decode_static_scratch);
    if (e != cudaSuccess || !p) {
      *status = cima_fail(e != cudaSuccess ? (int)e : CIMA_E_ARG, "attention_decode_static: cannot find the scratch array on device %d: %s", dev, cudaGetErrorString(e));
      return nullptr;
    }
    addr[dev] = static_cast<float*>(p);
  }
  *status = 0;
  return addr[dev];
}

extern "C" int cima_attention_decode_static(const void* qkv, int ld, const void* cache, const int* table, int table_width,
                                            int ring, int page_size, const int* seq_slot, const int* seq_len, void* out,
                                            int ldo, int B, int nh, int nkv, int hd, float scale, int window,
                                            int n_splits, cudaStream_t stream) {
  if (B <= 0) return 0;
  if (n_splits < 1 || nh <= 0 || hd <= 0) return cima_fail(CIMA_E_SIZE, "attention_decode_static: splits %d, heads %d and head_dim %d must be positive", n_splits, nh, hd);
  const unsigned long long cells = (unsigned long long)B * nh * n_splits;
  const unsigned long long need = cells * (unsigned long long)(hd + 2);
  if (need > (unsigned long long)CIMA_DECODE_STATIC_FLOATS)
    return cima_fail(CIMA_E_SIZE, "attention_decode_static: %d sequences x %d heads x %d splits x (head_dim %d + 2) = %llu floats of scratch; "
                     "the fixed array holds %d", B, nh, n_splits, hd, need, CIMA_DECODE_STATIC_FLOATS);
  int status = 0;
  float* scratch = decode_static_scratch_address(&status);
  if (!scratch) return status;
  float* part_o = scratch;                       // [B, nh, n_splits, hd]
  float* part_ml = scratch + cells * hd;         // [B, nh, n_splits, 2]
  return cima_attention_decode(qkv, ld, cache, table, table_width, ring, page_size, seq_slot, seq_len, part_o, part_ml,
                               out, ldo, B, nh, nkv, hd, scale, window, n_splits, 0, stream);
}
