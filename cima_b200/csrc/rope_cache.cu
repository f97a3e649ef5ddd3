// Rotary position encoding of q and k, and the append of k and v to the paged cache, in one pass
// over a step's rows.
//
// qkv is [T, ld]: q heads, then k heads, then v heads of each row.  q and k are rotated in place
// (prefill attention reads them from this buffer); the rotated k and the v are also written to the
// position's place in the layer's pages.  The angle p * inv_freq[i] and its sine and cosine are
// float32 (sincosf, not the fast approximations); inv_freq[i] = theta^(-2i / rotary_dim) comes from
// the host, computed in float64.  Pair (i, i + rotary_dim/2) of a head rotates:
//   u_i' = u_i cos a - u_j sin a,   u_j' = u_i sin a + u_j cos a        (src/kernels.cu:397-414)
// Dimensions from rotary_dim on pass through.  Append: src/kernels.cu:440-454 (one sequence,
// [kv_heads, max_seq, dim]); here the place comes from the slot's block table.
#include "common.cuh"

template <typename TA>
__global__ void __launch_bounds__(256)
k_rope_append(TA* __restrict__ qkv, int ld, const float* __restrict__ inv_freq, int rotary_dim,
              const int* __restrict__ row_pos, const int* __restrict__ row_seq, const int* __restrict__ seq_slot,
              const int* __restrict__ seq_len, TA* __restrict__ cache_in, CimaPaged pg, int nh, int nkv, int hd) {
  cima_pdl_wait();
  __shared__ float cs[128], sn[128];
  const int row = blockIdx.x;
  const int pos = row_pos[row];
  const int half = rotary_dim >> 1;
  for (int i = threadIdx.x; i < half; i += blockDim.x) {
    float s, c;
    sincosf((float)pos * inv_freq[i], &s, &c);
    cs[i] = c;
    sn[i] = s;
  }
  __syncthreads();
  TA* base = qkv + (size_t)row * ld;
  // In a ring of pages a long prompt wraps: a position whose place a later position of the same
  // step takes is not written at all (two rows of one launch must not write one place).
  TA* cache = cache_in;
  if (cache && pg.ring && pos + pg.ring * pg.page_size < seq_len[row_seq[row]]) cache = nullptr;
  const int slot = cache ? seq_slot[row_seq[row]] : 0;
  // rotation pairs of q heads [0, nh) and k heads [nh, nh + nkv)
  const int npairs = (nh + nkv) * half;
  for (int idx = threadIdx.x; idx < npairs; idx += blockDim.x) {
    const int head = idx / half, i = idx - head * half;
    TA* u = base + (size_t)head * hd;
    const float a = cima_to_f32<TA>(u[i]), b = cima_to_f32<TA>(u[i + half]);
    const TA ra = cima_from_f32<TA>(a * cs[i] - b * sn[i]);
    const TA rb = cima_from_f32<TA>(a * sn[i] + b * cs[i]);
    u[i] = ra;
    u[i + half] = rb;
    if (cache && head >= nh) {
      TA* dst = cache + pg.offset(slot, pos, 0, head - nh);
      dst[i] = ra;
      dst[i + half] = rb;
    }
  }
  if (!cache) return;
  // k dimensions that do not rotate
  const int rest = hd - rotary_dim;
  for (int idx = threadIdx.x; idx < nkv * rest; idx += blockDim.x) {
    const int head = idx / rest, d = rotary_dim + (idx - head * rest);
    cache[pg.offset(slot, pos, 0, head) + d] = base[(size_t)(nh + head) * hd + d];
  }
  // v
  for (int idx = threadIdx.x; idx < nkv * hd; idx += blockDim.x) {
    const int head = idx / hd, d = idx - head * hd;
    cache[pg.offset(slot, pos, 1, head) + d] = base[(size_t)(nh + nkv + head) * hd + d];
  }
}

// The same for bfloat16 rows whose halves are multiples of 8: a thread takes 8 consecutive pairs, i.e. two
// 16-byte pieces of a head, and every access to the row and to the cache is 16 bytes wide.  Same arithmetic,
// element by element, as the kernel above.
__global__ void __launch_bounds__(256)
k_rope_append_bf16x8(__nv_bfloat16* __restrict__ qkv, int ld, const float* __restrict__ inv_freq, int rotary_dim,
                     const int* __restrict__ row_pos, const int* __restrict__ row_seq, const int* __restrict__ seq_slot,
                     const int* __restrict__ seq_len, __nv_bfloat16* __restrict__ cache_in, CimaPaged pg, int nh, int nkv,
                     int hd) {
  cima_pdl_wait();
  __shared__ float cs[128], sn[128];
  const int row = blockIdx.x;
  const int pos = row_pos[row];
  const int half = rotary_dim >> 1;
  for (int i = threadIdx.x; i < half; i += blockDim.x) {
    float s, c;
    sincosf((float)pos * inv_freq[i], &s, &c);
    cs[i] = c;
    sn[i] = s;
  }
  __syncthreads();
  __nv_bfloat16* base = qkv + (size_t)row * ld;
  __nv_bfloat16* cache = cache_in;
  if (cache && pg.ring && pos + pg.ring * pg.page_size < seq_len[row_seq[row]]) cache = nullptr;
  const int slot = cache ? seq_slot[row_seq[row]] : 0;
  const int h8 = half >> 3;                              // groups of 8 pairs per head
  for (int idx = threadIdx.x; idx < (nh + nkv) * h8; idx += blockDim.x) {
    const int head = idx / h8, i = (idx - head * h8) * 8;
    __nv_bfloat16* u = base + (size_t)head * hd;
    uint4 av = *reinterpret_cast<const uint4*>(u + i), bv = *reinterpret_cast<const uint4*>(u + i + half);
    __nv_bfloat16* a = reinterpret_cast<__nv_bfloat16*>(&av);
    __nv_bfloat16* b = reinterpret_cast<__nv_bfloat16*>(&bv);
#pragma unroll
    for (int e = 0; e < 8; e++) {
      const float x = __bfloat162float(a[e]), y = __bfloat162float(b[e]);
      a[e] = __float2bfloat16_rn(x * cs[i + e] - y * sn[i + e]);
      b[e] = __float2bfloat16_rn(x * sn[i + e] + y * cs[i + e]);
    }
    *reinterpret_cast<uint4*>(u + i) = av;
    *reinterpret_cast<uint4*>(u + i + half) = bv;
    if (cache && head >= nh) {
      __nv_bfloat16* dst = cache + pg.offset(slot, pos, 0, head - nh);
      *reinterpret_cast<uint4*>(dst + i) = av;
      *reinterpret_cast<uint4*>(dst + i + half) = bv;
    }
  }
  if (!cache) return;
  const int rest8 = (hd - rotary_dim) >> 3;              // k dimensions that do not rotate
  for (int idx = threadIdx.x; idx < nkv * rest8; idx += blockDim.x) {
    const int head = idx / rest8, d = rotary_dim + (idx - head * rest8) * 8;
    *reinterpret_cast<uint4*>(cache + pg.offset(slot, pos, 0, head) + d) =
        *reinterpret_cast<const uint4*>(base + (size_t)(nh + head) * hd + d);
  }
  const int hd8 = hd >> 3;
  for (int idx = threadIdx.x; idx < nkv * hd8; idx += blockDim.x) {
    const int head = idx / hd8, d = (idx - head * hd8) * 8;
    *reinterpret_cast<uint4*>(cache + pg.offset(slot, pos, 1, head) + d) =
        *reinterpret_cast<const uint4*>(base + (size_t)(nh + nkv + head) * hd + d);
  }
}

// cache may be null (a layer that reads another layer's keys and values writes none).
// seq_len[i] is the length of sequence i after this step.
extern "C" int cima_rope_append(void* qkv, int dtype, int ld, const float* inv_freq, int rotary_dim,
                                const int* row_pos, const int* row_seq, const int* seq_slot, const int* seq_len,
                                void* cache, const int* table, int table_width, int ring, int page_size,
                                int T, int nh, int nkv, int hd, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (hd <= 0 || hd > 256 || rotary_dim < 0 || rotary_dim > hd || (rotary_dim & 1))
    return cima_fail(CIMA_E_SIZE, "rope_append: head_dim %d (at most 256) and an even rotary_dim %d <= head_dim are needed", hd, rotary_dim);
  if (ld < (nh + 2 * nkv) * hd) return cima_fail(CIMA_E_SIZE, "rope_append: row stride %d is smaller than (heads + 2 kv heads) * head_dim = %d", ld, (nh + 2 * nkv) * hd);
  if (cache && (page_size <= 0 || table_width <= 0)) return cima_fail(CIMA_E_SIZE, "rope_append: page size %d and table width %d must be positive", page_size, table_width);
  CimaPaged pg{table, table_width, ring, page_size, nkv, hd};
  if (dtype == CIMA_F32)
    { int rc_ = cima_launch(k_rope_append<float>, dim3(T), dim3(256), (size_t)(0), stream, 1, (float*)qkv, ld, inv_freq, rotary_dim, row_pos, row_seq, seq_slot, seq_len, (float*)cache, pg, nh, nkv, hd); if (rc_) return rc_; }
  else if (dtype == CIMA_BF16 && rotary_dim % 16 == 0 && hd % 8 == 0 && ld % 8 == 0 && rotary_dim <= 256 &&
           (((uintptr_t)qkv | (uintptr_t)cache) & 15) == 0)
    { int rc_ = cima_launch(k_rope_append_bf16x8, dim3(T), dim3(256), (size_t)(0), stream, 1, (__nv_bfloat16*)qkv, ld, inv_freq, rotary_dim, row_pos, row_seq, seq_slot, seq_len, (__nv_bfloat16*)cache, pg, nh, nkv, hd); if (rc_) return rc_; }
  else if (dtype == CIMA_BF16)
    { int rc_ = cima_launch(k_rope_append<__nv_bfloat16>, dim3(T), dim3(256), (size_t)(0), stream, 1, (__nv_bfloat16*)qkv, ld, inv_freq, rotary_dim, row_pos, row_seq, seq_slot, seq_len, (__nv_bfloat16*)cache, pg, nh, nkv, hd); if (rc_) return rc_; }
  else return cima_fail(CIMA_E_DTYPE, "rope_append: dtype code %d is neither float32 nor bfloat16", dtype);
  return cima_launch_result();
}
