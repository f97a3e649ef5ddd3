// Shared declarations of the kernel library: dtype codes, conversions, status codes.
//
// Every entry point is `extern "C" int cima_<name>(..., cudaStream_t stream)`.  It returns 0 when
// the launch was issued, a positive cudaError_t when CUDA refused it, and a negative CIMA_E_* code
// when the arguments are outside what the kernel accepts; `cima_last_error()` then holds a sentence
// that names the argument.  Nothing here allocates memory or synchronises.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>

enum { CIMA_F32 = 0, CIMA_BF16 = 1 };
enum { CIMA_E_ARG = -1, CIMA_E_DTYPE = -2, CIMA_E_SIZE = -3 };

extern "C" const char* cima_last_error();
int cima_fail(int code, const char* fmt, ...);

// Programmatic dependent launch.  Every kernel of this library starts with cima_pdl_wait(), which
// returns once the kernels before it in the stream have completed and their writes are visible.
// The long kernels call cima_pdl_trigger() when their main loop is over: from then on the next
// kernel may be scheduled into the space that this one's finishing blocks leave, and sits in its
// own wait until this one is done, so its launch latency hides behind this one's tail.  (A trigger
// at the top of a kernel would let a whole chain of waiting kernels crowd out the running one.)
// Launched without the attribute, both are no-ops.
__device__ __forceinline__ void cima_pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void cima_pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
bool cima_pdl_enabled();      // false when the environment has CIMA_NO_PDL=1

static inline int cima_launch_result() {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return cima_fail((int)e, "CUDA launch failed: %s", cudaGetErrorString(e));
  return 0;
}

template <typename T> __device__ __forceinline__ float cima_to_f32(T v);
template <> __device__ __forceinline__ float cima_to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float cima_to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T cima_from_f32(float v);
template <> __device__ __forceinline__ float cima_from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 cima_from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// The activation of a gated feed-forward's gate, float32.  The reference has SiLU only (src/kernels.cu:81-84);
// the others are what architectures of the same build use in its place.
enum { CIMA_ACT_SILU = 0, CIMA_ACT_GELU_TANH = 1, CIMA_ACT_GELU = 2, CIMA_ACT_RELU = 3, CIMA_ACT_COUNT = 4 };
__device__ __forceinline__ float cima_gate_act(float g, int act) {
  switch (act) {
    case CIMA_ACT_GELU_TANH: return 0.5f * g * (1.0f + tanhf(0.7978845608028654f * (g + 0.044715f * g * g * g)));
    case CIMA_ACT_GELU: return 0.5f * g * (1.0f + erff(g * 0.7071067811865476f));
    case CIMA_ACT_RELU: return fmaxf(g, 0.f);
    default: return g / (1.0f + expf(-g));
  }
}

// Sum over the threads of a block in a fixed order (warp shuffles, then warp 0 over the warps'
// partial sums), so that a row's result never depends on what else is launched with it.
// `red` is shared memory of at least 32 floats.  Every thread gets the total.
__device__ __forceinline__ float cima_block_sum(float v, float* red) {
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = (blockDim.x + 31) >> 5;
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = (lane < nwarp) ? red[lane] : 0.f;
  for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
  return t;
}

__device__ __forceinline__ float cima_block_max(float v, float* red) {
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = (blockDim.x + 31) >> 5;
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = (lane < nwarp) ? red[lane] : -INFINITY;
  for (int o = 16; o > 0; o >>= 1) t = fmaxf(t, __shfl_xor_sync(0xffffffffu, t, o));
  return t;
}

// Where position `pos` of slot `slot` lives in a layer's paged keys/values.
// storage: [pages][2][kv_heads][page_size][head_dim]; table: [slots][width].
struct CimaPaged {
  const int* table;
  int width;        // entries per slot in the table
  int ring;         // 0: entry = pos / page_size; R > 0: entry = (pos / page_size) % R
  int page_size;
  int kv_heads;
  int head_dim;
  __device__ __forceinline__ size_t offset(int slot, int pos, int kv, int head) const {
    int e = pos / page_size;
    if (ring) e %= ring;
    const int page = table[(size_t)slot * width + e];
    return ((((size_t)page * 2 + kv) * kv_heads + head) * page_size + (pos % page_size)) * (size_t)head_dim;
  }
};

// One launch path for all kernels: programmatic stream serialisation (see above) and, for cluster_x > 1,
// thread-block clusters of that many blocks along x.
template <typename... KArgs, typename... Args>
static inline int cima_launch(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                              int cluster_x, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  int n = 0;
  if (cima_pdl_enabled()) {
    attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[n].val.programmaticStreamSerializationAllowed = 1;
    n++;
  }
  if (cluster_x > 1) {
    attr[n].id = cudaLaunchAttributeClusterDimension;
    attr[n].val.clusterDim.x = cluster_x;
    attr[n].val.clusterDim.y = 1;
    attr[n].val.clusterDim.z = 1;
    n++;
  }
  cfg.attrs = attr;
  cfg.numAttrs = n;
  cudaError_t e = cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);
  if (e != cudaSuccess) return cima_fail((int)e, "CUDA launch failed: %s", cudaGetErrorString(e));
  return 0;
}
