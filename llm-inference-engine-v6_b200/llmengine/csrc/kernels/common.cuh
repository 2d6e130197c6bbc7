// Shared helpers of the sm_100a kernels: element types, loads/stores that widen to float,
// warp and block reductions, and the launch-status convention of the exported C functions.
//
// Every exported function is `extern "C"`, takes raw device pointers, sizes and a stream, launches
// on that stream and returns 0 or a non-zero code (see LLM_ERR_*); the text of the last error is
// kept for llm_last_error(). Nothing here allocates device memory.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <cstdint>
#include <cstdio>

#define LLM_OK 0
#define LLM_ERR_ARG 1     // a size or option this kernel does not take
#define LLM_ERR_LAUNCH 2  // the CUDA runtime refused the launch

// element type codes shared with the Python side
#define LLM_F32 0
#define LLM_BF16 1

typedef __nv_bfloat16 bf16;

extern "C" const char* llm_last_error();
void llm_set_error(const char* fmt, ...);

#define LLM_REQUIRE(cond, ...)            \
  do {                                    \
    if (!(cond)) {                        \
      llm_set_error(__VA_ARGS__);         \
      return LLM_ERR_ARG;                 \
    }                                     \
  } while (0)

#define LLM_CHECK_LAUNCH(name)                                            \
  do {                                                                    \
    cudaError_t e__ = cudaGetLastError();                                 \
    if (e__ != cudaSuccess) {                                             \
      llm_set_error("%s: launch failed: %s", name, cudaGetErrorString(e__)); \
      return LLM_ERR_LAUNCH;                                              \
    }                                                                     \
  } while (0)

__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(bf16 v) { return __bfloat162float(v); }

template <typename T>
__device__ __forceinline__ T from_f32(float v);
template <>
__device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <>
__device__ __forceinline__ bf16 from_f32<bf16>(float v) { return __float2bfloat16_rn(v); }

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

// Sum over a block of up to 1024 threads; every thread gets the result. `red` holds 33 floats.
// The order of additions depends only on blockDim, never on the batch.
__device__ __forceinline__ float block_sum(float v, float* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float t = lane < nw ? red[lane] : 0.f;
    t = warp_sum(t);
    if (lane == 0) red[32] = t;
  }
  __syncthreads();
  return red[32];
}

static inline int ceil_div(long long a, long long b) { return (int)((a + b - 1) / b); }

// ---------------------------------------------------------------------------------------------
// Programmatic dependent launch. Kernels of a step run back to back on one stream; each is
// launched with the attribute that lets its blocks start while the previous kernel is still
// draining. A kernel may do work that depends on nothing the stream produced (setting up shared
// memory, fetching weights) before dep_wait(); after dep_wait() every earlier kernel of the stream
// has finished and its writes are visible. EVERY kernel calls dep_wait() before it reads what an
// earlier kernel wrote and before its first global write. dep_launch() lets the next kernel's
// blocks be scheduled once all blocks of this one have called it (or left).
// A per-row scalar that a consumer of partial sums multiplies in: 1 / sqrt(sum_j sumsq[row, j] * inv_dim + eps),
// the 1/rms of a norm whose weight the producer of the operand has already applied (a per-row scalar
// commutes with a product over the row). sumsq null: 1.
struct RowScale {
  const float* sumsq;
  int n;
  float inv_dim, eps;
};
__device__ __forceinline__ float row_scale(const RowScale& rs, size_t row) {
  if (rs.sumsq == nullptr) return 1.0f;
  const float* part = rs.sumsq + row * (size_t)rs.n;
  float sum = 0.f;
  for (int j = 0; j < rs.n; ++j) sum += part[j];  // index order
  return 1.0f / sqrtf(sum * rs.inv_dim + rs.eps);
}

__device__ __forceinline__ void dep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void dep_launch() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

extern "C" void llm_set_dependent_launch(int on);
bool llm_dependent_launch();

template <typename... KArgs, typename... Args>
inline cudaError_t launch_kernel(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                 Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = llm_dependent_launch() ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// The same for a kernel whose CTAs form clusters (every grid dimension a multiple of the cluster's).
template <typename... KArgs, typename... Args>
inline cudaError_t launch_kernel_cluster(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, dim3 cluster,
                                         cudaStream_t stream, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = cluster.x;
  attr[0].val.clusterDim.y = cluster.y;
  attr[0].val.clusterDim.z = cluster.z;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = llm_dependent_launch() ? 2 : 1;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}
