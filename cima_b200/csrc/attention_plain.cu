// Plain causal grouped-query attention: one warp per (query row, head), keys visited one by one
// with a running (max, sum, accumulator) in float32.  It is the attention of the true 32-bit path
// and the fallback for head sizes the fast kernels do not take.  Two sources of keys and values:
//   step  - the step's own qkv buffer (a prompt that starts at position 0: key j of a sequence is
//           its row j), used for prefill;
//   cache - the layer's pages through the slot's block table, used for decoding.
// Head h reads kv head h / (heads / kv_heads); score = q.k * scale; a query at position p sees
// keys j <= p, and with window w > 0 only p - j < w (src/kernels.cu:458-491, :700-712).
// A row's result depends only on its own sequence: same bits alone or in any batch.
#include "common.cuh"

template <typename TA, bool FROM_CACHE>
__global__ void __launch_bounds__(128)
k_attention_plain(const TA* __restrict__ qkv, int ld, const TA* __restrict__ cache, CimaPaged pg,
                  const int* __restrict__ row_pos, const int* __restrict__ row_seq,
                  const int* __restrict__ seq_slot, const int* __restrict__ seq_first_row,
                  TA* __restrict__ out, int ldo, int T, int nh, int nkv, int hd, float scale, int window) {
  cima_pdl_wait();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int row = blockIdx.x * (blockDim.x >> 5) + warp;
  const int h = blockIdx.y;
  if (row >= T) return;
  const int kvh = h / (nh / nkv);
  const int pos = row_pos[row];
  const int seq = row_seq[row];
  const int slot = FROM_CACHE ? seq_slot[seq] : 0;
  const int first = FROM_CACHE ? 0 : seq_first_row[seq];
  const int kcol = (nh + kvh) * hd, vcol = (nh + nkv + kvh) * hd;

  float q[8], acc[8];
  const TA* qp = qkv + (size_t)row * ld + (size_t)h * hd;
#pragma unroll
  for (int i = 0; i < 8; i++) {
    const int d = lane + 32 * i;
    q[i] = d < hd ? cima_to_f32<TA>(qp[d]) : 0.f;
    acc[i] = 0.f;
  }
  float m = -1e30f, l = 0.f;
  const int lo = (window > 0 && pos + 1 > window) ? pos + 1 - window : 0;
  for (int j = lo; j <= pos; j++) {
    const TA *kp, *vp;
    if (FROM_CACHE) {
      kp = cache + pg.offset(slot, j, 0, kvh);
      vp = cache + pg.offset(slot, j, 1, kvh);
    } else {
      kp = qkv + (size_t)(first + j) * ld + kcol;
      vp = qkv + (size_t)(first + j) * ld + vcol;
    }
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < 8; i++) {
      const int d = lane + 32 * i;
      if (d < hd) s = fmaf(q[i], cima_to_f32<TA>(kp[d]), s);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    s *= scale;
    const float m2 = fmaxf(m, s);
    const float corr = expf(m - m2), p = expf(s - m2);
#pragma unroll
    for (int i = 0; i < 8; i++) {
      const int d = lane + 32 * i;
      if (d < hd) acc[i] = acc[i] * corr + p * cima_to_f32<TA>(vp[d]);
    }
    l = l * corr + p;
    m = m2;
  }
  TA* op = out + (size_t)row * ldo + (size_t)h * hd;
  const float inv = l > 0.f ? 1.0f / l : 0.f;
#pragma unroll
  for (int i = 0; i < 8; i++) {
    const int d = lane + 32 * i;
    if (d < hd) op[d] = cima_from_f32<TA>(acc[i] * inv);
  }
}

// from_cache 0: keys/values of the step (seq_first_row needed); 1: of the cache (table, seq_slot needed).
extern "C" int cima_attention_plain(const void* qkv, int dtype, int ld, const void* cache, const int* table,
                                    int table_width, int ring, int page_size, const int* row_pos,
                                    const int* row_seq, const int* seq_slot, const int* seq_first_row, void* out,
                                    int ldo, int T, int nh, int nkv, int hd, float scale, int window,
                                    int from_cache, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (hd <= 0 || hd > 256) return cima_fail(CIMA_E_SIZE, "attention_plain: head_dim %d is outside 1..256", hd);
  if (nh <= 0 || nkv <= 0 || nh % nkv) return cima_fail(CIMA_E_SIZE, "attention_plain: %d heads are not a multiple of %d kv heads", nh, nkv);
  if (nh > 65535) return cima_fail(CIMA_E_SIZE, "attention_plain: %d heads exceed one launch", nh);
  if (from_cache && (!cache || !table)) return cima_fail(CIMA_E_ARG, "attention_plain: decoding needs the cache and its block table");
  CimaPaged pg{table, table_width, ring, page_size, nkv, hd};
  dim3 grid((T + 3) / 4, nh);
#define LAUNCH(TA, FC) { int rc_ = cima_launch(k_attention_plain<TA, FC>, dim3(grid), dim3(128), (size_t)(0), stream, 1, (const TA*)qkv, ld, (const TA*)cache, pg, \
    row_pos, row_seq, seq_slot, seq_first_row, (TA*)out, ldo, T, nh, nkv, hd, scale, window); if (rc_) return rc_; }
  if (dtype == CIMA_F32) { if (from_cache) LAUNCH(float, true) else LAUNCH(float, false) }
  else if (dtype == CIMA_BF16) { if (from_cache) LAUNCH(__nv_bfloat16, true) else LAUNCH(__nv_bfloat16, false) }
  else return cima_fail(CIMA_E_DTYPE, "attention_plain: dtype code %d is neither float32 nor bfloat16", dtype);
#undef LAUNCH
  return cima_launch_result();
}
