// Matrix product for few rows (decode): out[m,n] = sum_k X[m,k] * W[n,k], M <= 8, bfloat16 operands,
// float32 accumulation.  The step is bound by reading W once from HBM, so the kernel is built
// around the weight stream: every thread keeps several 16-byte loads of W in flight, the weights
// are the 16-row operand of the tensor-core instruction and the few activation rows are its 8-wide
// operand ("swap A/B"), so M = 1..8 costs one instruction per 16x16 weights.  (With a second 8-row tile
// for 9 to 16 rows the kernel lost to the library product on B200 and is not instantiated.)
//
// Work split.  One block owns 16 output features (or 16 gate and the 16 matching up features for
// the gated epilogue).  Its 8 warps split K in interleaved chunks; their partial sums are added in
// shared memory in warp order 0..7, so a result never depends on scheduling, and a row of X gives
// the same bits whatever else is in the batch.  A matrix with few output features and a long K
// (the down projection) would leave most of the GPU idle that way, so the blocks of a thread-block
// cluster (1 to 8, chosen from the matrix's shape alone) split K further; block 0 of the
// cluster adds the blocks' sums in rank order through distributed shared memory and stores.
// A warp issues the loads of its first chunk of W before it waits for the kernel in front of it
// (programmatic dependent launch): weights depend on no kernel, and the stream then starts while that
// kernel's last blocks are finishing.
//
// Operand order.  mma.m16n8k16 wants, per thread, k = {2t, 2t+1, 2t+8, 2t+9} of rows g and g+8.
// A sum over k does not care in which order k is visited as long as both operands agree, so a
// thread instead loads 8 consecutive k (16 bytes) of its W rows and of its X row and feeds the
// first four to one instruction and the last four to the next: all loads are 16-byte and
// row-contiguous, no shared-memory staging of W is needed.
//
// Epilogues (the reference's GEMV has the first three, src/kernels.cu:502-538):
//   0 store bf16 (+ bias)      1 accumulate into the float32 residual      2 act(gate) * up -> bf16 (act: CIMA_ACT_*)
//   3 store float32 (+ bias), used for logits      4 q/k/v with rotation and cache append (see SkinnyRope)
#include "common.cuh"
#include <cooperative_groups.h>
namespace cg = cooperative_groups;

enum { SK_STORE = 0, SK_ACCUM = 1, SK_SWIGLU = 2, SK_STORE_F32 = 3, SK_QKV_ROPE = 4 };

__device__ __forceinline__ uint4 ld_stream16(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}

__device__ __forceinline__ uint4 ld_cached16(const void* p) {
  return __ldg(reinterpret_cast<const uint4*>(p));
}

__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
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

// RMSNorm folded into the product.  With inv = 1 / sqrt(sum(x^2) / K + eps) a normed row is inv * (x * w), so
// the product of the normed row is inv * sum_k bf16(x_k * w_k) W[n, k]: the kernel that wrote the residual row x
// also leaves xw = bf16(x * w) (w = the weight of the norm that follows) and partial sums of x^2; the product
// after the norm (NORM = true) reads xw as plain bf16 activations and applies the row's factor to its finished
// sums.  Against bf16(x * inv * w) as operand this differs by bfloat16 rounding only, and no separate norm
// kernel runs between the two.  The partial sums (ssq [M, parts]) are added in a fixed order at the kernel's
// start.  An accumulating product leaves, for the rows it has updated, one partial sum
// per 16-feature tile (ssq_out [M, tiles]) and xw_out [M, N] = bf16(x_new * w_next).
struct SkinnyNorm {
  const float* ssq;      // [M, parts] (NORM kernels)
  int parts;
  float eps;
  float* ssq_out;        // [M, tiles] or null (accumulating epilogue only)
  const float* w_next;   // [N] weight of the norm that follows, with xw_out; both null = not wanted
  __nv_bfloat16* xw_out;
  int act;               // gated epilogue: the gate's activation (CIMA_ACT_*)
};

// Mode 4: the q/k/v projection of a decode step with the rotary encoding and the append to the cache in its
// epilogue.  W is [q heads | k heads | v heads] x head_dim rows.  A block's 16 rows are then not 16
// consecutive features: for a head that rotates they are features 8s..8s+7 and their rotation partners
// head_dim/2 + 8s.., so that both halves of every pair (i, i + head_dim/2) meet in one block.  The rotated q
// goes to the qkv buffer (decode attention reads it there), the rotated k and the v straight to their place
// in the layer's pages.  Angles, sine and cosine are float32 as in rope_cache.cu; the projection is rotated
// before its one rounding to bfloat16.
struct SkinnyRope {
  const float* inv_freq;      // [head_dim / 2]
  const int* row_pos;         // [M] position of each row
  const int* row_seq;         // [M] sequence of each row
  const int* seq_slot;        // [sequences]
  __nv_bfloat16* cache;       // this layer's pages
  CimaPaged pg;
  int nh, nkv, hd;
};

// NT: 8-row tiles of X (M <= 8 * NT).  MT: m-tiles per block (1, or 2 for the gated epilogue).
// U: 32-wide k steps kept in flight per warp iteration.  NORM: X is bf16(x * w), see above.
template <int NT, int MT, int U, int MODE, bool NORM>
__global__ void __launch_bounds__(SK_WARPS * 32)
k_linear_skinny(const __nv_bfloat16* __restrict__ X, const __nv_bfloat16* __restrict__ W,
                const float* __restrict__ bias, void* __restrict__ out,
                int M, int N, int K, int ldx, int ldo, int up_offset, SkinnyNorm nm, SkinnyRope rp) {
  extern __shared__ float red[];                       // [warps][MT][NT*8][SK_PAD], then part [MT][NT*8][SK_ROWS]
  cg::cluster_group cluster = cg::this_cluster();
  const int S = (int)cluster.num_blocks();              // blocks that share this tile's K
  const int crank = (int)cluster.block_rank();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int n0 = (blockIdx.x / S) * SK_ROWS;
  // mode 4: which head this block works on, which 8 pairs of it, and whether the head rotates
  int rp_head = 0, rp_sub = 0;
  bool rp_rot = false;
  if (MODE == SK_QKV_ROPE) {
    const int tph = rp.hd / 16;
    rp_head = (blockIdx.x / S) / tph;
    rp_sub = (blockIdx.x / S) % tph;
    rp_rot = rp_head < rp.nh + rp.nkv;
  }
  // feature (row of W, column of the output) of row r in 0..15 of this block
  auto feature = [&](int r) -> int {
    if (MODE != SK_QKV_ROPE) return n0 + r;
    if (rp_rot) return rp_head * rp.hd + (r < 8 ? rp_sub * 8 + r : rp.hd / 2 + rp_sub * 8 + (r - 8));
    return rp_head * rp.hd + rp_sub * 16 + r;
  };
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
      const int r = feature(g + 8 * h);
      wok[a][h] = r < N;
      wrow[a][h] = W + (size_t)((wok[a][h] ? r : 0) + a * up_offset) * K;
    }

  // A warp owns chunks of 128 consecutive k, interleaved with the other warps' chunks; this split,
  // and so the order of summation, is the same for every instantiation.  U only says how many of a
  // chunk's four 32-wide steps are loaded before they are multiplied.
  constexpr int CHUNK = 128;
  uint4 w[MT][2][U];
  auto load_w = [&](int k0, int sub) {
#pragma unroll
    for (int s = 0; s < U; s++) {
      const int k = k0 + (sub + s) * 32 + 8 * t;
#pragma unroll
      for (int a = 0; a < MT; a++)
#pragma unroll
        for (int h = 0; h < 2; h++)
          w[a][h][s] = (wok[a][h] && k < K) ? ld_stream16(wrow[a][h] + k) : make_uint4(0u, 0u, 0u, 0u);
    }
  };
  auto multiply = [&](int k0, int sub) {
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
  };
  // The weights do not depend on the kernel before this one: the first loads of every warp are issued before
  // the wait for it, so that the weight stream starts while that kernel's last blocks are still finishing.
  const int k_first = (crank * SK_WARPS + warp) * CHUNK;
  if (k_first < K) load_w(k_first, 0);
  cima_pdl_wait();
  // Folded norm: a row's factor inv = 1 / sqrt(sum / K + eps) is made now, from the partial sums of squares that
  // the writer of the rows left, by the warp whose number is the row's: its loads (eight per lane, independent)
  // are answered by L2 while the warp's first weights are still on their way from memory.  The factor is applied
  // to the finished dot products (the operand of the tensor core is bf16(x * w)).
  __shared__ float inv_s[NT * 8];
  if (NORM) {
    for (int m = warp; m < M; m += SK_WARPS) {
      const float* ps = nm.ssq + (size_t)m * nm.parts;
      float p[8];
#pragma unroll
      for (int i = 0; i < 8; i++) p[i] = lane + 32 * i < nm.parts ? __ldg(ps + lane + 32 * i) : 0.f;
      float a = ((p[0] + p[1]) + (p[2] + p[3])) + ((p[4] + p[5]) + (p[6] + p[7]));     // a fixed order
      for (int pidx = 256 + lane; pidx < nm.parts; pidx += 32) a += __ldg(ps + pidx);
      for (int o = 16; o > 0; o >>= 1) a += __shfl_xor_sync(0xffffffffu, a, o);
      if (lane == 0) inv_s[m] = 1.0f / sqrtf(a / (float)K + nm.eps);
    }
  }
  if (k_first < K) {
    multiply(k_first, 0);
#pragma unroll
    for (int sub = U; sub < 4; sub += U) {
      load_w(k_first, sub);
      multiply(k_first, sub);
    }
    for (int k0 = k_first + S * SK_WARPS * CHUNK; k0 < K; k0 += S * SK_WARPS * CHUNK) {
#pragma unroll
      for (int sub = 0; sub < 4; sub += U) {
        load_w(k0, sub);
        multiply(k0, sub);
      }
    }
  }

  cima_pdl_trigger();      // the weights are read: the next kernel may be scheduled while the sums are merged
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

  // this block's sums over its 8 warps, in warp order
  float* part = red + (size_t)SK_WARPS * MT * COLS * SK_PAD;          // [MT][COLS][SK_ROWS]
  for (int e = threadIdx.x; e < COLS * SK_ROWS; e += SK_WARPS * 32) {
    const int r = e % SK_ROWS, m = e / SK_ROWS;
#pragma unroll
    for (int a = 0; a < MT; a++) {
      float s = 0.f;
#pragma unroll
      for (int wi = 0; wi < SK_WARPS; wi++) s += red[(((size_t)wi * MT + a) * COLS + m) * SK_PAD + r];
      part[((size_t)a * COLS + m) * SK_ROWS + r] = s;
    }
  }
  if (S > 1) cluster.sync(); else __syncthreads();

  if (crank == 0) {
    for (int e = threadIdx.x; e < COLS * SK_ROWS; e += SK_WARPS * 32) {
      const int r = e % SK_ROWS, m = e / SK_ROWS;
      const int n = feature(r);
      const bool live = m < M && n < N;
      if (MODE == SK_QKV_ROPE) {
        float s = part[(size_t)m * SK_ROWS + r];
        for (int cr = 1; cr < S; cr++) s += cluster.map_shared_rank(part, cr)[(size_t)m * SK_ROWS + r];
        float v = (NORM ? s * inv_s[m < M ? m : 0] : s) + (bias ? bias[n] : 0.f);
        const int pos = live ? rp.row_pos[m] : 0;
        if (rp_rot) {
          const float other = __shfl_xor_sync(0xffffffffu, v, 8);     // the pair's other half, 8 lanes away
          float sn, cs;
          sincosf((float)pos * rp.inv_freq[rp_sub * 8 + (r & 7)], &sn, &cs);
          v = r < 8 ? v * cs - other * sn : other * sn + v * cs;
        }
        if (live) {
          const __nv_bfloat16 o16 = __float2bfloat16_rn(v);
          if (rp_head < rp.nh) {
            ((__nv_bfloat16*)out)[(size_t)m * ldo + n] = o16;
          } else {
            const int slot = rp.seq_slot[rp.row_seq[m]];
            const bool is_v = rp_head >= rp.nh + rp.nkv;
            const int kvh = rp_head - rp.nh - (is_v ? rp.nkv : 0);
            rp.cache[rp.pg.offset(slot, pos, is_v ? 1 : 0, kvh) + (n - rp_head * rp.hd)] = o16;
          }
        }
        continue;
      }
      if (MODE == SK_ACCUM && nm.ssq_out) {
        // the 16 features of a row sit in 16 consecutive lanes: their squares are summed by shuffles
        float xn = 0.f;
        if (live) {
          float s = part[(size_t)m * SK_ROWS + r];
          for (int cr = 1; cr < S; cr++) s += cluster.map_shared_rank(part, cr)[(size_t)m * SK_ROWS + r];
          const size_t o = (size_t)m * ldo + n;
          xn = ((float*)out)[o] + (s + (bias ? bias[n] : 0.f));
          ((float*)out)[o] = xn;
          if (nm.xw_out) nm.xw_out[o] = __float2bfloat16_rn(xn * nm.w_next[n]);
        }
        float sq = xn * xn;
        for (int o = 8; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
        if (r == 0 && m < M) nm.ssq_out[(size_t)m * gridDim.x / S + blockIdx.x / S] = sq;
        continue;
      }
      if (!live) continue;
      float v[MT];
#pragma unroll
      for (int a = 0; a < MT; a++) {
        float s = part[((size_t)a * COLS + m) * SK_ROWS + r];
        for (int cr = 1; cr < S; cr++)                                // the other blocks' sums, in rank order
          s += cluster.map_shared_rank(part, cr)[((size_t)a * COLS + m) * SK_ROWS + r];
        v[a] = NORM ? s * inv_s[m] : s;
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
        ((__nv_bfloat16*)out)[o] = __float2bfloat16_rn(cima_gate_act(gate, nm.act) * up);
      }
    }
  }
  if (S > 1) cluster.sync();            // a block's shared memory must outlive block 0's reads of it
}

// Blocks per cluster for a matrix of `tiles` 16-feature tiles and K: the largest power of two that keeps all
// blocks resident at once (four blocks of 256 threads per SM) and leaves every warp at least one chunk of 128.
// Measured inside the decode step of a 3584-wide model on B200 (tokens per second at batch 8, K 18944, 224
// tiles): 2 blocks 2496, 4 blocks 2414, 1, 3, 5, 6 or 8 blocks 2230 to 2290: a second, partly filled wave
// costs more than its parallelism brings, and clusters of odd size were slower than their neighbours.
// Depends on the matrix and the device only, never on the rows of X, so that a row's sum has the same order
// whatever the batch.
static int cluster_size(int tiles, int K) {
  static int resident = 0;
  if (!resident) {
    int dev = 0, sms = 0;
    cudaGetDevice(&dev);
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) sms = 148;
    resident = sms * 4;
  }
  int s = 1;
  while (s < 8 && tiles * (2 * s) <= resident && (2 * s) * SK_WARPS * 128 <= K) s *= 2;
  return s;
}

template <int NT, int MT, int U, int MODE, bool NORM>
static int launch_skinny(const void* X, const void* W, const float* bias, void* out, int M, int N, int K, int ldx,
                         int ldo, int up_offset, const SkinnyNorm& nm, cudaStream_t stream,
                         const SkinnyRope& rp = SkinnyRope{}) {
  auto kern = k_linear_skinny<NT, MT, U, MODE, NORM>;
  const size_t smem = ((size_t)SK_WARPS * MT * NT * 8 * SK_PAD + (size_t)MT * NT * 8 * SK_ROWS) * sizeof(float);
  if (smem > 48 * 1024) {
    static bool raised = false;     // one attribute per instantiation
    if (!raised) {
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e != cudaSuccess) return cima_fail((int)e, "linear_skinny: cannot raise shared memory to %zu bytes: %s", smem, cudaGetErrorString(e));
      raised = true;
    }
  }
  const int tiles = (N + SK_ROWS - 1) / SK_ROWS;
  const int S = cluster_size(tiles, K);
  int rc = cima_launch(kern, dim3(tiles * S), dim3(SK_WARPS * 32), smem, stream, S, (const __nv_bfloat16*)X,
                       (const __nv_bfloat16*)W, bias, out, M, N, K, ldx, ldo, up_offset, nm, rp);
  if (rc) return rc;
  return cima_launch_result();
}

template <int NT, bool NORM>
static int dispatch_mode(int mode, const void* X, const void* W, const float* bias, void* out, int M, int N, int K,
                         int ldx, int ldo, const SkinnyNorm& nm, cudaStream_t stream) {
  constexpr int U = 4;
  switch (mode) {
    case SK_STORE: return launch_skinny<NT, 1, U, SK_STORE, NORM>(X, W, bias, out, M, N, K, ldx, ldo, 0, nm, stream);
    case SK_ACCUM: return launch_skinny<NT, 1, U, SK_ACCUM, NORM>(X, W, bias, out, M, N, K, ldx, ldo, 0, nm, stream);
    case SK_STORE_F32: return launch_skinny<NT, 1, U, SK_STORE_F32, NORM>(X, W, bias, out, M, N, K, ldx, ldo, 0, nm, stream);
    case SK_SWIGLU: return launch_skinny<NT, 2, 2, SK_SWIGLU, NORM>(X, W, bias, out, M, N, K, ldx, ldo, N, nm, stream);
    default: return cima_fail(CIMA_E_ARG, "linear_skinny: mode %d is not one of 0..3", mode);
  }
}

static int skinny_checks(const void* X, const void* W, const float* bias, int mode, int M, int N, int K, int ldx) {
  if (M > 8) return cima_fail(CIMA_E_SIZE, "linear_skinny: %d rows; this kernel takes at most 8 (the library product streams the weights faster for more)", M);
  if (N <= 0 || K <= 0) return cima_fail(CIMA_E_SIZE, "linear_skinny: N %d and K %d must be positive", N, K);
  if (K % 8 || ldx % 8) return cima_fail(CIMA_E_SIZE, "linear_skinny: K %d and the row stride %d must be multiples of 8 (16-byte loads)", K, ldx);
  if (((uintptr_t)X | (uintptr_t)W) & 15) return cima_fail(CIMA_E_ARG, "linear_skinny: X and W must be 16-byte aligned");
  if (mode == SK_SWIGLU && bias) return cima_fail(CIMA_E_ARG, "linear_skinny: the gated epilogue takes no bias");
  return 0;
}

// X [M, K] bf16 (row stride ldx), W [N, K] bf16 (for mode 2: [2N, K], gate rows then up rows),
// bias float32 [N] or null, out [M, N] (row stride ldo) in the dtype of the mode.
// Accepts 1 <= M <= 8, any N, K a multiple of 8 (16-byte rows), 16-byte aligned X, W and ldx % 8 == 0.
// ssq_out (mode 1 only, may be null): [M, ceil(N / 16)] partial sums of squares of the updated rows.
// w_next / xw_out (mode 1 with ssq_out, may be null): weight [N] of the norm that follows, and where to put
// bf16(updated row * that weight), [M, N] with row stride ldo.
extern "C" int cima_linear_skinny(const void* X, const void* W, const float* bias, void* out, int mode, int M, int N,
                                  int K, int ldx, int ldo, float* ssq_out, const float* w_next, void* xw_out, int act,
                                  cudaStream_t stream) {
  if (M <= 0) return 0;
  if (act < 0 || act >= CIMA_ACT_COUNT) return cima_fail(CIMA_E_ARG, "linear_skinny: activation code %d is not one of 0..%d", act, CIMA_ACT_COUNT - 1);
  int rc = skinny_checks(X, W, bias, mode, M, N, K, ldx);
  if (rc) return rc;
  if (xw_out && (mode != SK_ACCUM || !ssq_out || !w_next)) return cima_fail(CIMA_E_ARG, "linear_skinny: the scaled rows go with mode 1, the partial sums and the next norm's weight");
  SkinnyNorm nm{nullptr, 0, 0.f, mode == SK_ACCUM ? ssq_out : nullptr,
                mode == SK_ACCUM ? w_next : nullptr, mode == SK_ACCUM ? (__nv_bfloat16*)xw_out : nullptr, act};
  return dispatch_mode<1, false>(mode, X, W, bias, out, M, N, K, ldx, ldo, nm, stream);
}

// The same with RMSNorm folded in: xw [M, K] bf16 = bf16(x * w) as cima_embed or an accumulating product left
// it (row stride ldx), ssq [M, parts] the partial sums of squares of the rows x, and eps.  At most 8 rows.
extern "C" int cima_linear_skinny_norm(const void* xw, const float* ssq, int parts, float eps, const void* W,
                                       const float* bias, void* out, int mode, int M, int N, int K, int ldx, int ldo,
                                       int act, cudaStream_t stream) {
  if (M <= 0) return 0;
  if (act < 0 || act >= CIMA_ACT_COUNT) return cima_fail(CIMA_E_ARG, "linear_skinny_norm: activation code %d is not one of 0..%d", act, CIMA_ACT_COUNT - 1);
  if (M > 8) return cima_fail(CIMA_E_SIZE, "linear_skinny_norm: %d rows; the folded norm takes at most 8", M);
  if (!ssq || parts <= 0) return cima_fail(CIMA_E_ARG, "linear_skinny_norm: the partial sums of squares are needed");
  if (mode == SK_ACCUM) return cima_fail(CIMA_E_ARG, "linear_skinny_norm: the accumulating epilogue reads activations, not the residual");
  int rc = skinny_checks(xw, W, bias, mode, M, N, K, ldx);
  if (rc) return rc;
  SkinnyNorm nm{ssq, parts, eps, nullptr, nullptr, nullptr, act};
  return dispatch_mode<1, true>(mode, xw, W, bias, out, M, N, K, ldx, ldo, nm, stream);
}

// Mode 4 (see SkinnyRope): qkv [M, (nh + 2 nkv) * hd] receives the rotated q; k and v go to the cache.
// X: bf16 activations, or (ssq != null) bf16(x * w) with the partial sums of the rows: the norm folded in.
// At most 8 rows; head_dim a multiple of 16; every dimension of a head rotates (rotary_dim == head_dim).
extern "C" int cima_qkv_rope_skinny(const void* X, const float* ssq, int parts, float eps, const void* W,
                                    const float* bias, void* qkv, int M, int K, int ldx, int ldo,
                                    const float* inv_freq, const int* row_pos, const int* row_seq,
                                    const int* seq_slot, void* cache, const int* table, int table_width, int ring,
                                    int page_size, int nh, int nkv, int hd, cudaStream_t stream) {
  if (M <= 0) return 0;
  if (M > 8) return cima_fail(CIMA_E_SIZE, "qkv_rope_skinny: %d rows; this kernel takes at most 8", M);
  if (hd <= 0 || hd % 16 || nh <= 0 || nkv <= 0) return cima_fail(CIMA_E_SIZE, "qkv_rope_skinny: head_dim %d must be a multiple of 16 and the head counts positive", hd);
  if (!cache || !table || !inv_freq || !row_pos || !row_seq || !seq_slot) return cima_fail(CIMA_E_ARG, "qkv_rope_skinny: positions, frequencies and the cache are needed");
  const int N = (nh + 2 * nkv) * hd;
  const bool norm = ssq != nullptr;
  if (norm && parts <= 0) return cima_fail(CIMA_E_ARG, "qkv_rope_skinny: the folded norm needs the number of partial sums");
  int rc = skinny_checks(X, W, bias, SK_STORE, M, N, K, ldx);
  if (rc) return rc;
  SkinnyNorm nm{ssq, parts, eps, nullptr, nullptr, nullptr, 0};
  SkinnyRope rp{inv_freq, row_pos, row_seq, seq_slot, (__nv_bfloat16*)cache,
                CimaPaged{table, table_width, ring, page_size, nkv, hd}, nh, nkv, hd};
  if (norm) return launch_skinny<1, 1, 4, SK_QKV_ROPE, true>(X, W, bias, qkv, M, N, K, ldx, ldo, 0, nm, stream, rp);
  return launch_skinny<1, 1, 4, SK_QKV_ROPE, false>(X, W, bias, qkv, M, N, K, ldx, ldo, 0, nm, stream, rp);
}
