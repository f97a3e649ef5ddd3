// Embedding gather, RMSNorm, gated activation, residual add, row gather.
//
// The residual stream is float32 in both precisions; what the matrix products read and write
// ("activations") is float32 or bfloat16.  Norm weights and biases are float32 vectors.
//
// Counterparts in the reference (f16 storage, f32 arithmetic): k_gather_* src/kernels.cu:10-21,
// k_rmsnorm :37-50, k_swiglu :81-84, k_add :75-78.
#include "common.cuh"

// ---------------------------------------------------------------- embedding: x[t,:] = scale * E[ids[t],:]
template <typename TW>
__global__ void k_embed(const int* __restrict__ ids, const TW* __restrict__ table, float* __restrict__ x,
                        int H, int V, float scale, float* __restrict__ ssq, const float* __restrict__ w_next,
                        __nv_bfloat16* __restrict__ xw) {
  cima_pdl_wait();
  __shared__ float red[32];
  const int row = blockIdx.x;
  int id = ids[row];
  id = id < 0 ? 0 : (id >= V ? V - 1 : id);    // ids are checked on the host; never read outside the table
  const TW* src = table + (size_t)id * H;
  float* dst = x + (size_t)row * H;
  float acc = 0.f;
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    const float v = cima_to_f32<TW>(src[i]) * scale;
    dst[i] = v;
    if (xw) xw[(size_t)row * H + i] = __float2bfloat16_rn(v * w_next[i]);      // for a norm folded into the next product
    acc += v * v;
  }
  if (ssq) {                                    // the row's sum of squares, for a norm folded into the next product
    const float total = cima_block_sum(acc, red);
    if (threadIdx.x == 0) ssq[row] = total;
  }
}

// ssq (may be null): [T] sum of squares of each row written.  w_next / xw (may be null): weight [H] of the norm
// that follows and where to put bf16(row * weight), [T, H].
extern "C" int cima_embed(const int* ids, const void* table, int table_dtype, float* x, int T, int H, int V,
                          float scale, float* ssq, const float* w_next, void* xw, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (H <= 0 || V <= 0) return cima_fail(CIMA_E_SIZE, "embed: hidden %d and vocab %d must be positive", H, V);
  if (table_dtype == CIMA_F32) { int rc_ = cima_launch(k_embed<float>, dim3(T), dim3(256), (size_t)(0), stream, 1, ids, (const float*)table, x, H, V, scale, ssq, w_next, (__nv_bfloat16*)xw); if (rc_) return rc_; }
  else if (table_dtype == CIMA_BF16) { int rc_ = cima_launch(k_embed<__nv_bfloat16>, dim3(T), dim3(256), (size_t)(0), stream, 1, ids, (const __nv_bfloat16*)table, x, H, V, scale, ssq, w_next, (__nv_bfloat16*)xw); if (rc_) return rc_; }
  else return cima_fail(CIMA_E_DTYPE, "embed: table dtype code %d is neither float32 nor bfloat16", table_dtype);
  return cima_launch_result();
}

// ---------------------------------------------------------------- RMSNorm: y = x * rsqrt(mean(x^2) + eps) * w
// One block per row.  Sum of squares, reciprocal root and the products are float32; one rounding
// at the store.  1/sqrtf rather than rsqrtf: the latter is an approximation.
// With ADD the row is first updated, x += d (the residual sum in float32), and the norm is of the updated row:
// bit for bit what add_residual followed by rmsnorm gives, in one pass over the row less.
//
// Rows of up to 8192 values whose width is a multiple of 4 are read once, 16 bytes at a time, and kept in
// registers between the sum and the scaling; other rows take the loop that reads them twice.  Both walk the
// row in the same order per thread (element i belongs to thread (i / 4) % 256 on the first path, i % 256 on
// the second), so which path a width takes is fixed by the width alone.
constexpr int NORM_THREADS = 256;
constexpr int NORM_VEC = 8;                  // float4 per thread: 256 * 8 * 4 = 8192 values

template <typename TO> __device__ __forceinline__ void cima_store4(TO* p, float a, float b, float c, float d);
template <> __device__ __forceinline__ void cima_store4<float>(float* p, float a, float b, float c, float d) {
  *reinterpret_cast<float4*>(p) = make_float4(a, b, c, d);
}
template <> __device__ __forceinline__ void cima_store4<__nv_bfloat16>(__nv_bfloat16* p, float a, float b, float c, float d) {
  uint2 v;
  *reinterpret_cast<__nv_bfloat162*>(&v.x) = __floats2bfloat162_rn(a, b);
  *reinterpret_cast<__nv_bfloat162*>(&v.y) = __floats2bfloat162_rn(c, d);
  *reinterpret_cast<uint2*>(p) = v;
}
template <typename TA> __device__ __forceinline__ float4 cima_load4(const TA* p);
template <> __device__ __forceinline__ float4 cima_load4<float>(const float* p) { return *reinterpret_cast<const float4*>(p); }
template <> __device__ __forceinline__ float4 cima_load4<__nv_bfloat16>(const __nv_bfloat16* p) {
  const uint2 v = *reinterpret_cast<const uint2*>(p);
  const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&v.x));
  const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&v.y));
  return make_float4(a.x, a.y, b.x, b.y);
}

template <typename TA, bool ADD, bool VEC>
__global__ void __launch_bounds__(NORM_THREADS)
k_rmsnorm(float* __restrict__ x, const TA* __restrict__ d, const float* __restrict__ w, TA* __restrict__ y,
          int H, float eps) {
  cima_pdl_wait();
  __shared__ float red[32];
  float* xi = x + (size_t)blockIdx.x * H;
  const TA* di = ADD ? d + (size_t)blockIdx.x * H : nullptr;
  TA* yo = y + (size_t)blockIdx.x * H;
  if (VEC) {
    float4 v[NORM_VEC];
    const int H4 = H >> 2;
    float acc = 0.f;
#pragma unroll
    for (int j = 0; j < NORM_VEC; j++) {
      const int i4 = threadIdx.x + j * NORM_THREADS;
      if (i4 < H4) {
        v[j] = *reinterpret_cast<const float4*>(xi + 4 * i4);
        if (ADD) {
          const float4 a = cima_load4<TA>(di + 4 * i4);
          v[j].x += a.x; v[j].y += a.y; v[j].z += a.z; v[j].w += a.w;
          *reinterpret_cast<float4*>(xi + 4 * i4) = v[j];
        }
        acc += v[j].x * v[j].x; acc += v[j].y * v[j].y; acc += v[j].z * v[j].z; acc += v[j].w * v[j].w;
      }
    }
    const float total = cima_block_sum(acc, red);
    const float inv = 1.0f / sqrtf(total / (float)H + eps);
#pragma unroll
    for (int j = 0; j < NORM_VEC; j++) {
      const int i4 = threadIdx.x + j * NORM_THREADS;
      if (i4 < H4) {
        const float4 ww = *reinterpret_cast<const float4*>(w + 4 * i4);
        cima_store4<TA>(yo + 4 * i4, v[j].x * inv * ww.x, v[j].y * inv * ww.y, v[j].z * inv * ww.z, v[j].w * inv * ww.w);
      }
    }
    return;
  }
  float acc = 0.f;
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    float v = xi[i];
    if (ADD) { v += cima_to_f32<TA>(di[i]); xi[i] = v; }
    acc += v * v;
  }
  const float total = cima_block_sum(acc, red);
  const float inv = 1.0f / sqrtf(total / (float)H + eps);
  for (int i = threadIdx.x; i < H; i += blockDim.x) yo[i] = cima_from_f32<TA>(xi[i] * inv * w[i]);
}

template <typename TA, bool ADD>
static int launch_rmsnorm(float* x, const void* d, const float* w, void* y, int T, int H, float eps, cudaStream_t stream) {
  const bool vec = H % 4 == 0 && H <= NORM_THREADS * NORM_VEC * 4 &&
                   (((uintptr_t)x | (uintptr_t)w) & 15) == 0 && (((uintptr_t)y | (uintptr_t)d) & (4 * sizeof(TA) - 1)) == 0;
  int rc;
  if (vec) rc = cima_launch(k_rmsnorm<TA, ADD, true>, dim3(T), dim3(NORM_THREADS), (size_t)0, stream, 1, x, (const TA*)d, w, (TA*)y, H, eps);
  else rc = cima_launch(k_rmsnorm<TA, ADD, false>, dim3(T), dim3(NORM_THREADS), (size_t)0, stream, 1, x, (const TA*)d, w, (TA*)y, H, eps);
  if (rc) return rc;
  return cima_launch_result();
}

extern "C" int cima_rmsnorm(const float* x, const float* w, void* y, int y_dtype, int T, int H, float eps,
                            cudaStream_t stream) {
  if (T <= 0) return 0;
  if (H <= 0) return cima_fail(CIMA_E_SIZE, "rmsnorm: width %d must be positive", H);
  if (y_dtype == CIMA_F32) return launch_rmsnorm<float, false>(const_cast<float*>(x), nullptr, w, y, T, H, eps, stream);
  if (y_dtype == CIMA_BF16) return launch_rmsnorm<__nv_bfloat16, false>(const_cast<float*>(x), nullptr, w, y, T, H, eps, stream);
  return cima_fail(CIMA_E_DTYPE, "rmsnorm: output dtype code %d is neither float32 nor bfloat16", y_dtype);
}

// ---------------------------------------------------------------- gated activation: a = act(g) * u (act: CIMA_ACT_*)
// gu is [T, 2I] with the gate in columns [0, I) and the up projection in [I, 2I).
// The bfloat16 kernel moves 16 bytes per access when I is a multiple of 8; otherwise element by element.
template <typename TA>
__global__ void k_swiglu(const TA* __restrict__ gu, TA* __restrict__ a, size_t total, int I, int act) {
  cima_pdl_wait();
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
    const size_t row = idx / I;
    const int c = (int)(idx - row * I);
    const float g = cima_to_f32<TA>(gu[row * 2 * I + c]);
    const float u = cima_to_f32<TA>(gu[row * 2 * I + I + c]);
    a[idx] = cima_from_f32<TA>(cima_gate_act(g, act) * u);
  }
}

__global__ void k_swiglu_bf16x8(const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ a, size_t groups, int I8, int act) {
  cima_pdl_wait();
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < groups; idx += (size_t)gridDim.x * blockDim.x) {
    const size_t row = idx / I8;
    const int c = (int)(idx - row * I8);
    const uint4 gv = *reinterpret_cast<const uint4*>(gu + (row * 2 * I8 + c) * 8);
    const uint4 uv = *reinterpret_cast<const uint4*>(gu + (row * 2 * I8 + I8 + c) * 8);
    const __nv_bfloat162* gp = reinterpret_cast<const __nv_bfloat162*>(&gv);
    const __nv_bfloat162* up = reinterpret_cast<const __nv_bfloat162*>(&uv);
    uint4 ov;
    __nv_bfloat162* op = reinterpret_cast<__nv_bfloat162*>(&ov);
#pragma unroll
    for (int e = 0; e < 4; e++) {
      const float2 g = __bfloat1622float2(gp[e]), u = __bfloat1622float2(up[e]);
      op[e] = __floats2bfloat162_rn(cima_gate_act(g.x, act) * u.x, cima_gate_act(g.y, act) * u.y);
    }
    *reinterpret_cast<uint4*>(a + idx * 8) = ov;
  }
}

extern "C" int cima_swiglu(const void* gu, void* a, int dtype, int T, int I, int act, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (act < 0 || act >= CIMA_ACT_COUNT) return cima_fail(CIMA_E_ARG, "swiglu: activation code %d is not one of 0..%d", act, CIMA_ACT_COUNT - 1);
  if (I <= 0) return cima_fail(CIMA_E_SIZE, "swiglu: intermediate width %d must be positive", I);
  const size_t total = (size_t)T * I;
  if (dtype == CIMA_BF16 && I % 8 == 0 && (((uintptr_t)gu | (uintptr_t)a) & 15) == 0) {
    const size_t groups = total / 8;
    const int grid = (int)((groups + 255) / 256 > 148 * 16 ? 148 * 16 : (groups + 255) / 256);
    { int rc_ = cima_launch(k_swiglu_bf16x8, dim3(grid), dim3(256), (size_t)0, stream, 1, (const __nv_bfloat16*)gu, (__nv_bfloat16*)a, groups, I / 8, act); if (rc_) return rc_; }
    return cima_launch_result();
  }
  const int grid = (int)((total + 255) / 256 > 148 * 32 ? 148 * 32 : (total + 255) / 256);
  if (dtype == CIMA_F32) { int rc_ = cima_launch(k_swiglu<float>, dim3(grid), dim3(256), (size_t)(0), stream, 1, (const float*)gu, (float*)a, total, I, act); if (rc_) return rc_; }
  else if (dtype == CIMA_BF16) { int rc_ = cima_launch(k_swiglu<__nv_bfloat16>, dim3(grid), dim3(256), (size_t)(0), stream, 1, (const __nv_bfloat16*)gu, (__nv_bfloat16*)a, total, I, act); if (rc_) return rc_; }
  else return cima_fail(CIMA_E_DTYPE, "swiglu: dtype code %d is neither float32 nor bfloat16", dtype);
  return cima_launch_result();
}

// ---------------------------------------------------------------- residual: x += d  (sum in float32)
template <typename TA>
__global__ void k_add_residual(float* __restrict__ x, const TA* __restrict__ d, size_t total) {
  cima_pdl_wait();
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x)
    x[idx] += cima_to_f32<TA>(d[idx]);
}

extern "C" int cima_add_residual(float* x, const void* d, int d_dtype, size_t total, cudaStream_t stream) {
  if (total == 0) return 0;
  const int grid = (int)((total + 255) / 256 > 148 * 32 ? 148 * 32 : (total + 255) / 256);
  if (d_dtype == CIMA_F32) { int rc_ = cima_launch(k_add_residual<float>, dim3(grid), dim3(256), (size_t)(0), stream, 1, x, (const float*)d, total); if (rc_) return rc_; }
  else if (d_dtype == CIMA_BF16) { int rc_ = cima_launch(k_add_residual<__nv_bfloat16>, dim3(grid), dim3(256), (size_t)(0), stream, 1, x, (const __nv_bfloat16*)d, total); if (rc_) return rc_; }
  else return cima_fail(CIMA_E_DTYPE, "add_residual: dtype code %d is neither float32 nor bfloat16", d_dtype);
  return cima_launch_result();
}

// ---------------------------------------------------------------- residual + norm: x += d; h = RMSNorm(x)
// k_rmsnorm with ADD (see there).
extern "C" int cima_add_rmsnorm(float* x, const void* d, const float* w, void* h, int dtype, int T, int H, float eps,
                                cudaStream_t stream) {
  if (T <= 0) return 0;
  if (H <= 0) return cima_fail(CIMA_E_SIZE, "add_rmsnorm: width %d must be positive", H);
  if (dtype == CIMA_F32) return launch_rmsnorm<float, true>(x, d, w, h, T, H, eps, stream);
  if (dtype == CIMA_BF16) return launch_rmsnorm<__nv_bfloat16, true>(x, d, w, h, T, H, eps, stream);
  return cima_fail(CIMA_E_DTYPE, "add_rmsnorm: dtype code %d is neither float32 nor bfloat16", dtype);
}

// ---------------------------------------------------------------- row gather: out[i,:] = x[rows[i],:]
__global__ void k_gather_rows(const float* __restrict__ x, const int* __restrict__ rows, float* __restrict__ out, int H) {
  cima_pdl_wait();
  const float* src = x + (size_t)rows[blockIdx.x] * H;
  float* dst = out + (size_t)blockIdx.x * H;
  for (int i = threadIdx.x; i < H; i += blockDim.x) dst[i] = src[i];
}

extern "C" int cima_gather_rows(const float* x, const int* rows, float* out, int n, int H, cudaStream_t stream) {
  if (n <= 0) return 0;
  { int rc_ = cima_launch(k_gather_rows, dim3(n), dim3(256), (size_t)(0), stream, 1, x, rows, out, H); if (rc_) return rc_; }
  return cima_launch_result();
}

// ---------------------------------------------------------------- end of a decode step on the device
// The chosen tokens become the next step's input and every sequence moves on by one position, so
// that a captured step replays without the host touching its inputs (the reference closes its
// captured step the same way: k_argmax_extract and k_pos_bump, src/kernels.cu:309-318).
__global__ void k_decode_advance(const int* __restrict__ chosen, int* __restrict__ tokens, int* __restrict__ row_pos,
                                 int* __restrict__ seq_len, int B) {
  cima_pdl_wait();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < B) {
    tokens[i] = chosen[i];
    row_pos[i] += 1;
    seq_len[i] += 1;
  }
}

extern "C" int cima_decode_advance(const int* chosen, int* tokens, int* row_pos, int* seq_len, int B, cudaStream_t stream) {
  if (B <= 0) return 0;
  { int rc_ = cima_launch(k_decode_advance, dim3((B + 127) / 128), dim3(128), (size_t)(0), stream, 1, chosen, tokens, row_pos, seq_len, B); if (rc_) return rc_; }
  return cima_launch_result();
}
