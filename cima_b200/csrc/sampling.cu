// Token selection on the device.
//
// argmax: a cluster of blocks per row of float32 logits; ties go to the higher index, the order the
// reference gets from packing (orderable float bits << 32 | index) into one u64 maximum
// (src/kernels.cu:244-262).
#include "common.cuh"
#include <cooperative_groups.h>

__device__ __forceinline__ unsigned long long cima_pack_key(float v, int i) {
  unsigned int b = __float_as_uint(v);
  b = (b & 0x80000000u) ? ~b : (b | 0x80000000u);
  return ((unsigned long long)b << 32) | (unsigned int)i;
}

__device__ __forceinline__ unsigned long long cima_block_max_u64(unsigned long long v, unsigned long long* red) {
  for (int o = 16; o > 0; o >>= 1) {
    const unsigned long long w = __shfl_xor_sync(0xffffffffu, v, o);
    v = w > v ? w : v;
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = (blockDim.x + 31) >> 5;
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  unsigned long long t = lane < nwarp ? red[lane] : 0ULL;
  for (int o = 16; o > 0; o >>= 1) {
    const unsigned long long w = __shfl_xor_sync(0xffffffffu, t, o);
    t = w > t ? w : t;
  }
  return t;
}

// A row is shared by the ARGMAX_BLOCKS blocks of a thread-block cluster (a block alone takes 75 us for a
// vocabulary of 152,064: one SM's load latency, not the memory's bandwidth, is the bound); block 0 takes the
// maximum of the blocks' maxima through distributed shared memory.  A maximum of packed keys does not depend
// on the order in which it is taken.
constexpr int ARGMAX_BLOCKS = 8;

__global__ void __launch_bounds__(512)
k_argmax(const float* __restrict__ logits, int ld, int V, int* __restrict__ tokens) {
  cima_pdl_wait();
  namespace cg = cooperative_groups;
  cg::cluster_group cluster = cg::this_cluster();
  __shared__ unsigned long long red[32];
  __shared__ unsigned long long mine;
  const int C = gridDim.x, c = blockIdx.x;
  const float* x = logits + (size_t)blockIdx.y * ld;
  const int per = (((V + C - 1) / C) + 3) & ~3;         // a multiple of 4, so that a block's share starts aligned
  const int lo = min(V, c * per), hi = min(V, lo + per);
  unsigned long long best = 0ULL;
  if ((((uintptr_t)x) & 15) == 0) {
    const int n4 = (hi - lo) >> 2;
    const float4* x4 = reinterpret_cast<const float4*>(x + lo);
    for (int i = threadIdx.x; i < n4; i += blockDim.x) {
      const float4 v = __ldg(x4 + i);
      const int at = lo + 4 * i;
      unsigned long long k = cima_pack_key(v.x, at);
      best = k > best ? k : best;
      k = cima_pack_key(v.y, at + 1); best = k > best ? k : best;
      k = cima_pack_key(v.z, at + 2); best = k > best ? k : best;
      k = cima_pack_key(v.w, at + 3); best = k > best ? k : best;
    }
    for (int i = lo + 4 * n4 + threadIdx.x; i < hi; i += blockDim.x) {
      const unsigned long long k = cima_pack_key(x[i], i);
      best = k > best ? k : best;
    }
  } else {
    for (int i = lo + threadIdx.x; i < hi; i += blockDim.x) {
      const unsigned long long k = cima_pack_key(x[i], i);
      best = k > best ? k : best;
    }
  }
  best = cima_block_max_u64(best, red);
  if (threadIdx.x == 0) mine = best;
  cluster.sync();
  if (c == 0 && threadIdx.x == 0) {
    for (int r = 1; r < C; r++) {
      const unsigned long long k = *cluster.map_shared_rank(&mine, r);
      best = k > best ? k : best;
    }
    tokens[blockIdx.y] = (int)(unsigned int)best;
  }
  cluster.sync();                                        // a block's shared memory must outlive block 0's reads
}

extern "C" int cima_argmax(const float* logits, int ld, int n, int V, int* tokens, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (V <= 0 || ld < V) return cima_fail(CIMA_E_SIZE, "argmax: vocabulary %d must be positive and fit the row stride %d", V, ld);
  if (n > 65535) return cima_fail(CIMA_E_SIZE, "argmax: %d rows exceed one launch", n);
  { int rc_ = cima_launch(k_argmax, dim3(ARGMAX_BLOCKS, n), dim3(512), (size_t)(0), stream, ARGMAX_BLOCKS, logits, ld, V, tokens); if (rc_) return rc_; }
  return cima_launch_result();
}

// ---------------------------------------------------------------------------------------------
// The sampling chain of the reference's DefaultSampler (src/models/mod.rs:86-201), whole, on the
// device, one block per row:
//   1. repeat penalty over the last 64 tokens of the sequence's history, once per occurrence:
//      l > 0 ? l / rp : l * rp                                                    (:149-160)
//   2. temperature <= 0 -> argmax, ties to the higher index                        (:163-169)
//   3. top-k (0 = all) in the order (value descending, index descending)           (:171-194)
//   4. p = exp((l - max) / max(T, 1e-4)), normalised over the kept                 (:104-109)
//   5. top-p: the shortest prefix of that order whose mass reaches top_p           (:110-119)
//   6. r = u * mass(kept); the first token of the order whose cumulated mass reaches r (:121-130)
//      u from xorshift64* (state max(seed, 1)), u = (x * 0x2545F4914F6CDD1D >> 40) / 2^24 (:69-78)
// The reference sorts on the host.  Here nothing is sorted: every token has the 64-bit key
// (orderable value bits << 32 | index), whose order is the order above, and steps 3, 5 and 6 are
// each a search for the largest key T such that {tokens with key >= T} has at least k members, or
// at least the wanted mass.  A search fixes T bit by bit from the top; each bit is one pass over
// the row.  Sums of masses run in a fixed order, so a row's draw is the same whatever else is in
// the batch; they differ from the host's sequential sums by rounding only.
//
// Per-sequence state (by slot): rng state, the ring of the last 64 tokens and the count of tokens
// pushed so far.  The drawn token is pushed into the ring before the kernel ends.
// ---------------------------------------------------------------------------------------------

constexpr int SAMPLE_THREADS = 1024;
constexpr int SAMPLE_RING = 64;

struct SampleRow {
  const float* l;     // penalised logits of the row
  int V;
  float maxl, inv_t;
};

// number of tokens with key >= T
__device__ int sample_count(const SampleRow& r, unsigned long long T, float* redf) {
  int c = 0;
  for (int i = threadIdx.x; i < r.V; i += blockDim.x) c += cima_pack_key(r.l[i], i) >= T ? 1 : 0;
  return (int)(cima_block_sum((float)c, redf) + 0.5f);     // counts below 2^24 are exact in float32
}

// mass of the tokens with key in [T, ...) that are also kept (key >= floor)
__device__ float sample_mass(const SampleRow& r, unsigned long long T, float* redf) {
  float s = 0.f;
  for (int i = threadIdx.x; i < r.V; i += blockDim.x) {
    const float v = r.l[i];
    if (cima_pack_key(v, i) >= T) s += expf((v - r.maxl) * r.inv_t);
  }
  return cima_block_sum(s, redf);
}

__global__ void __launch_bounds__(SAMPLE_THREADS)
k_sample(const float* __restrict__ logits, int ld, int V, const int* __restrict__ row_slot,
         const float* __restrict__ params, unsigned long long* __restrict__ rng, int* __restrict__ ring,
         int* __restrict__ ring_count, float* __restrict__ work, int* __restrict__ tokens, int only_unresolved) {
  cima_pdl_wait();
  __shared__ float redf[32];
  __shared__ unsigned long long redk[32];
  __shared__ float s_u;
  const int row = blockIdx.x;
  if (only_unresolved && tokens[row] >= 0) return;      // the fast kernel has settled this row
  const int slot = row_slot[row];
  const float temperature = params[row * 4 + 0];
  const int top_k = (int)params[row * 4 + 1];
  const float top_p = params[row * 4 + 2];
  const float rp = params[row * 4 + 3];
  const float* x = logits + (size_t)row * ld;
  float* l = work + (size_t)row * V;
  int* myring = ring + (size_t)slot * SAMPLE_RING;

  // 1. working copy, then the penalty, entry by entry as the host loop does
  for (int i = threadIdx.x; i < V; i += blockDim.x) l[i] = x[i];
  __syncthreads();
  const int pushed = ring_count[slot];
  if (threadIdx.x == 0 && rp != 1.0f) {
    const int n = pushed < SAMPLE_RING ? pushed : SAMPLE_RING;
    for (int j = 0; j < n; j++) {
      // oldest first, as a history slice is walked
      const int t = myring[(pushed - n + j) % SAMPLE_RING];
      if (t >= 0 && t < V) l[t] = l[t] > 0.f ? l[t] / rp : l[t] * rp;
    }
  }
  __syncthreads();

  // the largest key (needed by both the greedy and the sampled way)
  unsigned long long best = 0ULL;
  for (int i = threadIdx.x; i < V; i += blockDim.x) {
    const unsigned long long k = cima_pack_key(l[i], i);
    best = k > best ? k : best;
  }
  best = cima_block_max_u64(best, redk);
  int token = (int)(unsigned int)best;

  if (temperature > 0.f) {
    SampleRow r;
    r.l = l; r.V = V;
    r.maxl = l[token];
    r.inv_t = 1.0f / fmaxf(temperature, 1e-4f);
    int idx_bits = 1;
    while ((1 << idx_bits) < V) idx_bits++;

    // 3. floor of the kept keys: the k-th largest key
    unsigned long long floor_key = 0ULL;
    if (top_k > 0 && top_k < V) {
      for (int b = 63; b >= 0; b--) {
        if (b < 32 && b >= idx_bits) continue;               // index bits that no token has
        const unsigned long long cand = floor_key | (1ULL << b);
        const int c = sample_count(r, cand, redf);
        if (c >= top_k) floor_key = cand;
        if (c == top_k) break;                                // the kept set is settled
      }
    }
    // 4./5. mass of the kept, then the top-p floor.  A search builds, bit by bit from the top, the
    // largest T for which "T <= floor, or the tokens with key >= T are some and weigh enough" holds.
    const float total = sample_mass(r, floor_key, redf);
    if (top_p < 1.0f) {
      unsigned long long T = 0ULL;
      for (int b = 63; b >= 0; b--) {
        if (b < 32 && b >= idx_bits) continue;
        const unsigned long long cand = T | (1ULL << b);
        if (cand <= floor_key) { T = cand; continue; }
        if (cand > best) continue;
        if (sample_mass(r, cand, redf) / total >= top_p) T = cand;
      }
      floor_key = T > floor_key ? T : floor_key;
    }
    const float kept = sample_mass(r, floor_key, redf) / total;
    // 6. the draw
    if (threadIdx.x == 0) {
      unsigned long long s = rng[slot];
      s ^= s >> 12; s ^= s << 25; s ^= s >> 27;
      rng[slot] = s;
      s_u = (float)((s * 0x2545F4914F6CDD1DULL) >> 40) / 16777216.0f;
    }
    __syncthreads();
    const float target = s_u * kept;
    unsigned long long T = 0ULL;
    for (int b = 63; b >= 0; b--) {
      if (b < 32 && b >= idx_bits) continue;
      const unsigned long long cand = T | (1ULL << b);
      if (cand <= floor_key) { T = cand; continue; }
      if (cand > best) continue;
      if (sample_mass(r, cand, redf) / total >= target) T = cand;
    }
    if (T < floor_key) T = floor_key;
    // the token is the one with the smallest key >= T (T itself whenever T is a token's key)
    unsigned long long m = 0ULL;
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
      const unsigned long long k = cima_pack_key(l[i], i);
      if (k >= T) { const unsigned long long c = ~k; m = c > m ? c : m; }
    }
    m = cima_block_max_u64(m, redk);
    token = (int)(unsigned int)(~m);
  }
  if (threadIdx.x == 0) {
    tokens[row] = token;
    myring[pushed % SAMPLE_RING] = token;
    ring_count[slot] = pushed + 1;
  }
}

// ---------------------------------------------------------------------------------------------
// The same chain, fast, for the common case that few tokens are kept (the reference's default top_k is 40).
// A row is shared by the 8 blocks of a thread-block cluster; every block keeps its slice of the penalised
// logits in shared memory.  The k-th largest key is found by a radix select (one histogram of 256 bins per
// byte of the key, merged over the cluster through distributed shared memory; it stops as soon as a bin holds
// exactly what is still wanted), the kept tokens are gathered and sorted in block 0, and one thread then does
// what the reference's host loop does, in its order and in float32: probabilities, their sum, the top-p cut,
// the renormalised draw (src/models/mod.rs:100-130).
//
// With top_k = 0 (or at least the vocabulary) the 1024 largest tokens stand in for the whole row (the sum of
// all masses is taken over the whole row): if the top-p cut and the draw both fall inside them the row is
// settled; else, and for a top_k between 1025 and the vocabulary, the blocks search the whole row together
// (the bisection of k_sample, over the slices in shared memory: about 2 us a pass instead of 20).
// ---------------------------------------------------------------------------------------------
constexpr int FAST_BLOCKS = 8;
constexpr int FAST_THREADS = 512;
constexpr int FAST_MAXK = 1024;

__device__ __forceinline__ float cima_key_value(unsigned long long key) {
  const unsigned int hi = (unsigned int)(key >> 32);
  return __uint_as_float((hi & 0x80000000u) ? (hi ^ 0x80000000u) : ~hi);
}

__global__ void __launch_bounds__(FAST_THREADS)
k_sample_fast(const float* __restrict__ logits, int ld, int V, const int* __restrict__ row_slot,
              const float* __restrict__ params, unsigned long long* __restrict__ rng, int* __restrict__ ring,
              int* __restrict__ ring_count, int* __restrict__ tokens) {
  cima_pdl_wait();
  namespace cg = cooperative_groups;
  cg::cluster_group cluster = cg::this_cluster();
  extern __shared__ float sl[];                       // this block's slice of the (penalised) row
  __shared__ float pr_s[FAST_MAXK];                   // block 0: probabilities of the kept tokens, in order
  __shared__ int hist[256];
  __shared__ int merged[256];
  __shared__ unsigned long long cand[FAST_MAXK];      // this block's kept keys, any order
  __shared__ unsigned long long sorted[FAST_MAXK];    // block 0: all kept keys
  __shared__ unsigned long long redk[32];
  __shared__ float redf[32];
  __shared__ unsigned long long s_best;
  __shared__ int ncand, s_sel, s_above, s_cnt, s_total_n;
  __shared__ float s_mass, s_total_all;
  __shared__ float s_part[2];
  __shared__ int s_resolved;
  const int C = FAST_BLOCKS, c = blockIdx.x, row = blockIdx.y, tid = threadIdx.x;
  const int slot = row_slot[row];
  const float temperature = params[row * 4 + 0];
  const int top_k = (int)params[row * 4 + 1];
  const float top_p = params[row * 4 + 2];
  const float rp = params[row * 4 + 3];
  const float* x = logits + (size_t)row * ld;
  int* myring = ring + (size_t)slot * SAMPLE_RING;
  const int per = (((V + C - 1) / C) + 3) & ~3;
  const int lo = min(V, c * per), hi = min(V, lo + per), n_loc = hi - lo;

  // 1. the slice, then the penalty on it, entry by entry as the host loop does
  for (int i = tid; i < n_loc; i += FAST_THREADS) sl[i] = x[lo + i];
  const int pushed = ring_count[slot];
  __syncthreads();
  if (tid == 0 && rp != 1.0f) {
    const int n = pushed < SAMPLE_RING ? pushed : SAMPLE_RING;
    for (int j = 0; j < n; j++) {
      const int t = myring[(pushed - n + j) % SAMPLE_RING];
      if (t >= lo && t < hi) sl[t - lo] = sl[t - lo] > 0.f ? sl[t - lo] / rp : sl[t - lo] * rp;
    }
  }
  __syncthreads();
  // 2. the largest key of the row
  unsigned long long best = 0ULL;
  for (int i = tid; i < n_loc; i += FAST_THREADS) {
    const unsigned long long k = cima_pack_key(sl[i], lo + i);
    best = k > best ? k : best;
  }
  best = cima_block_max_u64(best, redk);
  if (tid == 0) s_best = best;
  cluster.sync();
  for (int r = 0; r < C; r++) {
    const unsigned long long k = *cluster.map_shared_rank(&s_best, r);
    best = k > best ? k : best;
  }
  if (temperature <= 0.f) {
    if (c == 0 && tid == 0) {
      const int token = (int)(unsigned int)best;
      tokens[row] = token;
      myring[pushed % SAMPLE_RING] = token;
      ring_count[slot] = pushed + 1;
    }
    cluster.sync();                                   // a block's shared memory must outlive the others' reads
    return;
  }
  const float maxl = cima_key_value(best);
  const float inv_t = 1.0f / fmaxf(temperature, 1e-4f);
  const int kk = (top_k <= 0 || top_k > V) ? V : top_k;
  const bool exact = kk <= FAST_MAXK;                 // the kept set is gathered whole
  const int want = exact ? kk : FAST_MAXK;
  // more than 1024 kept, but not the whole row: the head cannot stand in (the sum of the kept masses is not at
  // hand there); the search over the whole row below does it
  const bool try_head = exact || kk == V;

  if (try_head) {
    // 3. T = the want-th largest key, byte by byte from the top
    unsigned long long prefix = 0ULL;
    int remaining = want;
    for (int b = 7; b >= 0; b--) {
      if (b == 3) continue;                             // indices stay below 2^24: this byte is zero in every key
      const int shift = 8 * b;
      for (int j = tid; j < 256; j += FAST_THREADS) hist[j] = 0;
      __syncthreads();
      for (int i = tid; i < n_loc; i += FAST_THREADS) {
        const unsigned long long k = cima_pack_key(sl[i], lo + i);
        if (b == 7 || (k >> (shift + 8)) == (prefix >> (shift + 8))) atomicAdd(&hist[(int)((k >> shift) & 255ULL)], 1);
      }
      __syncthreads();
      cluster.sync();
      if (tid < 256) {
        int sum = 0;
        for (int r = 0; r < C; r++) sum += cluster.map_shared_rank(hist, r)[tid];
        merged[tid] = sum;
      }
      __syncthreads();
      if (tid == 0) {
        int cum = 0, bin = 255;
        for (; bin > 0; bin--) {
          if (cum + merged[bin] >= remaining) break;
          cum += merged[bin];
        }
        s_sel = bin; s_above = cum; s_cnt = merged[bin];
      }
      __syncthreads();
      prefix |= (unsigned long long)s_sel << shift;
      remaining -= s_above;
      const bool settled = s_cnt == remaining;          // the whole bin is kept: every lower bit of T is zero
      cluster.sync();                                   // everyone has read this block's histogram
      if (settled) break;
    }
    const unsigned long long T = prefix;

    // 4. the kept keys of this slice; the mass of the whole slice when the kept set is not gathered whole
    if (tid == 0) ncand = 0;
    __syncthreads();
    float mass = 0.f;
    for (int i = tid; i < n_loc; i += FAST_THREADS) {
      const float v = sl[i];
      const unsigned long long k = cima_pack_key(v, lo + i);
      if (k >= T) {
        const int at = atomicAdd(&ncand, 1);
        if (at < FAST_MAXK) cand[at] = k;
      }
      if (!exact) mass += expf((v - maxl) * inv_t);
    }
    if (!exact) {
      mass = cima_block_sum(mass, redf);
      if (tid == 0) s_mass = mass;
    }
    __syncthreads();
    cluster.sync();
    if (c == 0) {
      int at = 0;
      float total_all = 0.f;
      for (int r = 0; r < C; r++) {                     // ranks in order: a fixed sum, a fixed layout
        const int n_r = min(*cluster.map_shared_rank(&ncand, r), FAST_MAXK);
        const unsigned long long* src = cluster.map_shared_rank(cand, r);
        for (int j = tid; j < n_r && at + j < FAST_MAXK; j += FAST_THREADS) sorted[at + j] = src[j];
        at = min(at + n_r, FAST_MAXK);
        if (!exact) total_all += *cluster.map_shared_rank(&s_mass, r);
      }
      if (tid == 0) { s_total_n = at; s_total_all = total_all; }
    }
    cluster.sync();                                     // block 0 has the kept keys (and the row's mass)
    if (c == 0) {
      __syncthreads();
      const int n = s_total_n;
      int P = 1;
      while (P < n) P <<= 1;
      for (int i = n + tid; i < P; i += FAST_THREADS) sorted[i] = 0ULL;
      __syncthreads();
      // 5. bitonic sort, largest key first: the reference's order (value descending, index descending)
      for (int k2 = 2; k2 <= P; k2 <<= 1)
        for (int j = k2 >> 1; j > 0; j >>= 1) {
          for (int i = tid; i < P; i += FAST_THREADS) {
            const int o = i ^ j;
            if (o > i) {
              const unsigned long long a = sorted[i], bq = sorted[o];
              const bool desc = (i & k2) == 0;
              if (desc ? a < bq : a > bq) { sorted[i] = bq; sorted[o] = a; }
            }
          }
          __syncthreads();
        }
      float* pr = pr_s;
      const float v0 = cima_key_value(sorted[0]);
      for (int i = tid; i < n; i += FAST_THREADS) pr[i] = expf((cima_key_value(sorted[i]) - v0) * inv_t);
      __syncthreads();
      if (tid == 0) {
        // 6. the host loop of the reference, in its order and in float32
        float total = 0.f;
        if (exact) { for (int i = 0; i < n; i++) total += pr[i]; } else total = s_total_all;
        int cut = exact ? n : -1;
        float cum = 0.f;
        for (int i = 0; i < n; i++) {
          const float p = pr[i] / total;
          pr[i] = p;
          cum += p;
          if (cum >= top_p) { cut = i + 1; break; }
        }
        unsigned long long st = rng[slot];
        st ^= st >> 12; st ^= st << 25; st ^= st >> 27;
        const float u = (float)((st * 0x2545F4914F6CDD1DULL) >> 40) / 16777216.0f;
        int token = -1;
        if (cut > 0) {
          float renorm = 0.f;
          for (int i = 0; i < cut; i++) renorm += pr[i];
          float r = u * renorm;
          token = (int)(unsigned int)sorted[cut - 1];
          for (int i = 0; i < cut; i++) {
            r -= pr[i];
            if (r <= 0.f) { token = (int)(unsigned int)sorted[i]; break; }
          }
        } else if (top_p >= 1.0f) {
          // nothing is cut and the kept set is the whole row, of which only the head is here: settled if the
          // draw falls into the head
          float r = u;
          for (int i = 0; i < n; i++) {
            r -= pr[i];
            if (r <= 0.f) { token = (int)(unsigned int)sorted[i]; break; }
          }
        }
        if (token >= 0) {
          tokens[row] = token;
          rng[slot] = st;
          myring[pushed % SAMPLE_RING] = token;
          ring_count[slot] = pushed + 1;
        }
        s_resolved = token >= 0;
      }
    }

  }
  // ---- what the head could not settle: the search over the whole row, by all blocks of the cluster.  The order
  // (value descending, index descending) is the order of the 64-bit keys; the k-th largest key, the top-p floor
  // and the drawn token are each the largest key T for which "the tokens with key >= T are at least k" (or
  // "weigh at least so much") holds, found bit by bit from the top; each bit is one pass over the slices in
  // shared memory and one exchange through the cluster.  Sums run in a fixed order (thread, block, rank).
  if (try_head) {
    cluster.sync();                                   // block 0 has said whether the head settled the row
    const int resolved = *cluster.map_shared_rank(&s_resolved, 0);
    cluster.sync();                                   // ... and everyone has heard it
    if (resolved) return;
  }
  int pass = 0;
  auto cl_count = [&](unsigned long long T) -> int {
    int cnt = 0;
    for (int i = tid; i < n_loc; i += FAST_THREADS) cnt += cima_pack_key(sl[i], lo + i) >= T ? 1 : 0;
    const float tot = cima_block_sum((float)cnt, redf);          // below 2^24: exact
    if (tid == 0) s_part[pass & 1] = tot;
    cluster.sync();
    float sum = 0.f;
    for (int r = 0; r < C; r++) sum += cluster.map_shared_rank(s_part, r)[pass & 1];
    pass++;
    return (int)(sum + 0.5f);
  };
  auto cl_mass = [&](unsigned long long T) -> float {
    float m = 0.f;
    for (int i = tid; i < n_loc; i += FAST_THREADS) {
      const float v = sl[i];
      if (cima_pack_key(v, lo + i) >= T) m += expf((v - maxl) * inv_t);
    }
    m = cima_block_sum(m, redf);
    if (tid == 0) s_part[pass & 1] = m;
    cluster.sync();
    float sum = 0.f;
    for (int r = 0; r < C; r++) sum += cluster.map_shared_rank(s_part, r)[pass & 1];
    pass++;
    return sum;
  };
  int idx_bits = 1;
  while ((1 << idx_bits) < V) idx_bits++;
  unsigned long long floor_key = 0ULL;
  if (kk < V) {
    for (int b = 63; b >= 0; b--) {
      if (b < 32 && b >= idx_bits) continue;               // index bits that no token has
      const unsigned long long cand = floor_key | (1ULL << b);
      const int cnt = cl_count(cand);
      if (cnt >= kk) floor_key = cand;
      if (cnt == kk) break;                                 // the kept set is settled
    }
  }
  const float total = cl_mass(floor_key);
  if (top_p < 1.0f) {
    unsigned long long T = 0ULL;
    for (int b = 63; b >= 0; b--) {
      if (b < 32 && b >= idx_bits) continue;
      const unsigned long long cand = T | (1ULL << b);
      if (cand <= floor_key) { T = cand; continue; }
      if (cand > best) continue;
      if (cl_mass(cand) / total >= top_p) T = cand;
    }
    floor_key = T > floor_key ? T : floor_key;
  }
  const float kept = cl_mass(floor_key) / total;
  unsigned long long st = rng[slot];                        // every block draws the same number
  st ^= st >> 12; st ^= st << 25; st ^= st >> 27;
  const float target = (float)((st * 0x2545F4914F6CDD1DULL) >> 40) / 16777216.0f * kept;
  unsigned long long T = 0ULL;
  for (int b = 63; b >= 0; b--) {
    if (b < 32 && b >= idx_bits) continue;
    const unsigned long long cand = T | (1ULL << b);
    if (cand <= floor_key) { T = cand; continue; }
    if (cand > best) continue;
    if (cl_mass(cand) / total >= target) T = cand;
  }
  if (T < floor_key) T = floor_key;
  // the token is the one with the smallest key >= T (T itself whenever T is a token's key)
  unsigned long long m = 0ULL;
  for (int i = tid; i < n_loc; i += FAST_THREADS) {
    const unsigned long long k = cima_pack_key(sl[i], lo + i);
    if (k >= T) { const unsigned long long cm = ~k; m = cm > m ? cm : m; }
  }
  m = cima_block_max_u64(m, redk);
  if (tid == 0) s_best = m;
  cluster.sync();                                     // (every block has read rng[slot] by now)
  if (c == 0 && tid == 0) {
    for (int r = 1; r < C; r++) {
      const unsigned long long k = *cluster.map_shared_rank(&s_best, r);
      m = k > m ? k : m;
    }
    const int token = (int)(unsigned int)(~m);
    tokens[row] = token;
    rng[slot] = st;
    myring[pushed % SAMPLE_RING] = token;
    ring_count[slot] = pushed + 1;
  }
  cluster.sync();                                     // a block's shared memory must outlive block 0's reads
}

// logits [n, V] float32 (row stride ld); row_slot [n]; params [n, 4] = temperature, top_k, top_p,
// repeat_penalty; rng [slots] u64; ring [slots, 64]; ring_count [slots]; work [n, V] float32 scratch.
extern "C" int cima_sample(const float* logits, int ld, int n, int V, const int* row_slot, const float* params,
                           unsigned long long* rng, int* ring, int* ring_count, float* work, int* tokens,
                           cudaStream_t stream) {
  if (n <= 0) return 0;
  if (V <= 0 || ld < V) return cima_fail(CIMA_E_SIZE, "sample: vocabulary %d must be positive and fit the row stride %d", V, ld);
  if (V >= (1 << 24)) return cima_fail(CIMA_E_SIZE, "sample: vocabulary %d exceeds 2^24 (counts are summed in float32)", V);
  if (n > 65535) return cima_fail(CIMA_E_SIZE, "sample: %d rows exceed one launch", n);
  // the fast kernel keeps an eighth of a row in shared memory; rows too long for that go to the general kernel,
  // one block per row
  const int per = (((V + FAST_BLOCKS - 1) / FAST_BLOCKS) + 3) & ~3;
  const size_t smem = (size_t)(per > 4 ? per : 4) * sizeof(float);
  if (smem <= 160 * 1024) {
    static bool raised = false;
    if (!raised) {
      cudaError_t e = cudaFuncSetAttribute(k_sample_fast, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024);
      if (e != cudaSuccess) return cima_fail((int)e, "sample: cannot raise shared memory: %s", cudaGetErrorString(e));
      raised = true;
    }
    { int rc_ = cima_launch(k_sample_fast, dim3(FAST_BLOCKS, n), dim3(FAST_THREADS), smem, stream, FAST_BLOCKS, logits, ld, V, row_slot, params, rng, ring, ring_count, tokens); if (rc_) return rc_; }
    return cima_launch_result();
  }
  const int only_unresolved = 0;
  { int rc_ = cima_launch(k_sample, dim3(n), dim3(SAMPLE_THREADS), (size_t)(0), stream, 1, logits, ld, V, row_slot, params, rng, ring, ring_count, work, tokens, only_unresolved); if (rc_) return rc_; }
  return cima_launch_result();
}

// The general kernel alone (one block per row, any vocabulary below 2^24), whatever the size: what cima_sample
// takes for rows too long for the fast kernel's shared memory, callable by itself so that it can be tested at
// small sizes.
extern "C" int cima_sample_general(const float* logits, int ld, int n, int V, const int* row_slot, const float* params,
                                   unsigned long long* rng, int* ring, int* ring_count, float* work, int* tokens,
                                   cudaStream_t stream) {
  if (n <= 0) return 0;
  if (V <= 0 || ld < V) return cima_fail(CIMA_E_SIZE, "sample: vocabulary %d must be positive and fit the row stride %d", V, ld);
  if (V >= (1 << 24)) return cima_fail(CIMA_E_SIZE, "sample: vocabulary %d exceeds 2^24 (counts are summed in float32)", V);
  { int rc_ = cima_launch(k_sample, dim3(n), dim3(SAMPLE_THREADS), (size_t)(0), stream, 1, logits, ld, V, row_slot, params, rng, ring, ring_count, work, tokens, 0); if (rc_) return rc_; }
  return cima_launch_result();
}
