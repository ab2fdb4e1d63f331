// Shared device/host helpers for the sm_100a kernels.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

typedef __nv_bfloat16 bf16;
typedef __nv_bfloat162 bf162;

#define MLB_API extern "C" __attribute__((visibility("default")))

// Error word shared by every kernel that can give up on a bounded wait (mbarrier, peer flag).
// 0 = ok.  Layout of a non-zero value: (code << 24) | detail.  Host reads it with mlb_get_error().
enum : int {
  MLB_ERR_NONE = 0,
  MLB_ERR_MBAR_TIMEOUT = 1,   // an mbarrier wait in a TMA/tcgen05 pipeline ran out
  MLB_ERR_FLAG_TIMEOUT = 2,   // a wait on a peer/host flag ran out
  MLB_ERR_BOUNDS = 3,         // a self-check found an index out of range
};
// Each translation unit owns one copy (no relocatable device code is used); MLB_DEFINE_ERROR_WORD(tag) also
// exports mlb_get_error_<tag>() / mlb_clear_error_<tag>() for the host.
#define MLB_DEFINE_ERROR_WORD(tag)                                             \
  MLB_API int mlb_get_error_##tag() {                                          \
    int v = 0;                                                                 \
    cudaMemcpyFromSymbol(&v, g_mlb_error, sizeof(int));                        \
    return v;                                                                  \
  }                                                                            \
  MLB_API void mlb_clear_error_##tag() {                                       \
    int v = 0;                                                                 \
    cudaMemcpyToSymbol(g_mlb_error, &v, sizeof(int));                          \
  }                                                                            \
  /* the word copied to (pinned) host memory behind the work already in `st`: no synchronisation of its own */ \
  MLB_API int mlb_read_error_async_##tag(int* host_dst, cudaStream_t st) {     \
    void* p = nullptr;                                                         \
    cudaError_t e = cudaGetSymbolAddress(&p, g_mlb_error);                     \
    if (e != cudaSuccess) return (int)e;                                       \
    return (int)cudaMemcpyAsync(host_dst, p, sizeof(int), cudaMemcpyDeviceToHost, st); \
  }
static __device__ int g_mlb_error = 0;

// ------------------------------------------------------------------ programmatic dependent launch
// Kernels started through mlb_launch() may become resident while the kernel before them in the stream is still
// draining: they run their own set-up, then mlb_pdl_sync() blocks until that kernel has completed and its writes are
// visible (and lets the kernel after this one start its set-up in turn).  Every global-memory access of such a
// kernel comes after the call.  Launched the ordinary way the instructions are no-ops.
__device__ __forceinline__ void mlb_pdl_sync() {
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
#ifdef __CUDACC__
#include <cstdlib>
#include <utility>
// MLB_PDL: 0 (default) no kernel starts early; 1 every kernel launched through mlb_launch / mlb_launch_tmem may (measured
// slower inside a captured step, 20.6 vs 19.8 ms: a kernel that allocates tensor memory or most of an SM's shared memory
// cannot become resident next to its predecessor anyway, and one that does delays it); 2 only the kernels launched
// through mlb_launch - the element-wise ones, whose CTAs fit beside a tensor-core kernel's (also measured slower in the
// captured step: 18.1-18.5 against 17.75 ms, the early-resident CTAs take issue slots and registers from the kernel
// they wait for).
inline int mlb_pdl_mode() {
  static int mode = -1;
  if (mode < 0) {
    const char* e = getenv("MLB_PDL");
    mode = (e != nullptr && (e[0] == '1' || e[0] == '2')) ? e[0] - '0' : 0;
  }
  return mode;
}
inline bool mlb_pdl_enabled() { return mlb_pdl_mode() == 1; }
template <typename... KArgs, typename... Args>
inline cudaError_t mlb_launch_attr(bool early, void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = early ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kern, std::forward<Args>(args)...);
}
template <typename... KArgs, typename... Args>
inline cudaError_t mlb_launch(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args&&... args) {
  return mlb_launch_attr(mlb_pdl_mode() != 0, kern, grid, block, smem, st, std::forward<Args>(args)...);
}
// for kernels that allocate tensor memory (GEMMs, attention): they start early only in mode 1
template <typename... KArgs, typename... Args>
inline cudaError_t mlb_launch_tmem(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args&&... args) {
  return mlb_launch_attr(mlb_pdl_mode() == 1, kern, grid, block, smem, st, std::forward<Args>(args)...);
}
#endif

__device__ __forceinline__ void mlb_set_error(int code, int detail) {
  atomicCAS(&g_mlb_error, 0, (code << 24) | (detail & 0xFFFFFF));
}

static inline int ceil_div_i(long a, long b) { return (int)((a + b - 1) / b); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Block-wide sum for blockDim.x <= 1024 (multiple of 32). `red` needs 32 floats of shared memory.
__device__ __forceinline__ float block_sum(float v, float* red) {
  int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = blockDim.x >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) red[w] = v;
  __syncthreads();
  float t = (lane < nw) ? red[lane] : 0.f;
  t = warp_sum(t);
  return t;
}
__device__ __forceinline__ float block_max(float v, float* red) {
  int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = blockDim.x >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) red[w] = v;
  __syncthreads();
  float t = (lane < nw) ? red[lane] : -INFINITY;
  t = warp_max(t);
  return t;
}

struct __align__(16) bf16x8 { bf162 v[4]; };

__device__ __forceinline__ uint32_t pack_bf16(float a, float b) {
  bf162 t = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&t);
}
