// Next-token choice on the device: greedy argmax, or a temperature draw.
//
// Greedy is the reference's rule: the first index of the maximum (strict '>', src/engine.cpp:52-58).
// The reference has no other sampler. The temperature draw here is argmax_i(logit_i / T + g_i)
// with Gumbel noise g_i = -log(-log(u_i)), which is a draw from softmax(logits / T); u_i comes from
// an integer hash of (request seed, index of the draw in that request, i), so the draw depends on
// nothing else: not on the batch, the step or the row it happens to occupy. All arithmetic float32.
#include "common.cuh"

#include <cmath>

namespace {

__device__ __forceinline__ unsigned mix32(unsigned x) {
  x ^= x >> 16;
  x *= 0x7FEB352Du;
  x ^= x >> 15;
  x *= 0x846CA68Bu;
  x ^= x >> 16;
  return x;
}

// Stage 1: block (row, chunk) scans its chunk of the vocabulary and leaves its best (value, index).
__global__ void __launch_bounds__(256) sample_scan_kernel(const float* __restrict__ logits, long long ld,
                                                          const float* __restrict__ temperature,
                                                          const int* __restrict__ seeds, const int* __restrict__ draws,
                                                          float* __restrict__ best_val, int* __restrict__ best_idx, int vocab,
                                                          int chunk) {
  __shared__ float best_v[8];
  __shared__ int best_i[8];
  dep_launch();
  dep_wait();
  const int row = blockIdx.y;
  const float* lr = logits + (size_t)row * ld;
  const float temp = temperature ? temperature[row] : 0.f;
  const int begin = blockIdx.x * chunk, end = min(vocab, begin + chunk);
  float bv = -INFINITY;
  int bi = 0x7fffffff;
  if (temp > 0.f) {
    const float inv_t = 1.0f / temp;
    unsigned k = mix32((unsigned)seeds[row] ^ 0x9E3779B9u);
    k = mix32(k + (unsigned)draws[row]);
    for (int i = begin + threadIdx.x; i < end; i += blockDim.x) {
      const unsigned r = mix32(k ^ ((unsigned)i * 0x85EBCA6Bu));
      const float u = __fmul_rn((float)(r >> 9) + 0.5f, 1.0f / 8388608.0f);
      const float g = -logf(-logf(u));
      const float z = __fadd_rn(__fmul_rn(lr[i], inv_t), g);
      if (z > bv) { bv = z; bi = i; }  // ascending i per thread: first maximum kept
    }
  } else {
    for (int i = begin + threadIdx.x; i < end; i += blockDim.x) {
      const float z = lr[i];
      if (z > bv) { bv = z; bi = i; }
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  if (lane == 0) { best_v[warp] = bv; best_i[warp] = bi; }
  __syncthreads();
  if (warp == 0) {
    bv = lane < nw ? best_v[lane] : -INFINITY;
    bi = lane < nw ? best_i[lane] : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    if (lane == 0) {
      best_val[(size_t)row * gridDim.x + blockIdx.x] = bv;
      best_idx[(size_t)row * gridDim.x + blockIdx.x] = bi;
    }
  }
}

// Stage 2: one warp per row merges the chunks (largest value, lowest index among equals).
__global__ void sample_merge_kernel(const float* __restrict__ best_val, const int* __restrict__ best_idx, int n_chunks,
                                    int* __restrict__ out, int n_rows) {
  dep_launch();
  dep_wait();
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= n_rows) return;
  float bv = -INFINITY;
  int bi = 0x7fffffff;
  for (int c = lane; c < n_chunks; c += 32) {
    const float v = best_val[(size_t)row * n_chunks + c];
    const int i = best_idx[(size_t)row * n_chunks + c];
    if (v > bv || (v == bv && i < bi)) { bv = v; bi = i; }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
  }
  // NaN-free inputs assumed; a row of only -inf or NaN yields index 0.
  if (lane == 0) out[row] = (bi == 0x7fffffff) ? 0 : bi;
}

}  // namespace

// Chunks of the vocabulary that llm_sample scans per row; scratch must hold 2 * rows * chunks words.
extern "C" int llm_sample_chunks(int vocab) {
  int c = (vocab + 4095) / 4096;
  return c < 1 ? 1 : (c > 64 ? 64 : c);
}

// temperature/seeds/draws: one per row; temperature may be null (all greedy).
// scratch: 2 * n_rows * llm_sample_chunks(vocab) 4-byte words.
extern "C" int llm_sample(const float* logits, long long ld, const float* temperature, const int* seeds,
                          const int* draws, int* out, int n_rows, int vocab, void* scratch, cudaStream_t stream) {
  if (n_rows == 0) return LLM_OK;
  LLM_REQUIRE(n_rows > 0 && vocab > 0 && ld >= vocab, "sample: bad sizes rows=%d vocab=%d", n_rows, vocab);
  LLM_REQUIRE(!temperature || (seeds && draws), "sample: temperature needs seeds and draw indices");
  LLM_REQUIRE(scratch != nullptr && n_rows <= 65535, "sample: scratch missing or too many rows");
  const int chunks = llm_sample_chunks(vocab);
  const int chunk = (vocab + chunks - 1) / chunks;
  float* best_val = (float*)scratch;
  int* best_idx = (int*)scratch + (size_t)n_rows * chunks;
  launch_kernel(sample_scan_kernel, dim3(chunks, n_rows), 256, 0, stream, logits, ld, temperature, seeds, draws, best_val, best_idx, vocab, chunk);
  launch_kernel(sample_merge_kernel, ceil_div(n_rows, 4), 128, 0, stream, (const float*)best_val, (const int*)best_idx, chunks, out, n_rows);
  LLM_CHECK_LAUNCH("sample");
  return LLM_OK;
}

// ------------------------------------------------------------------------------------------------
// The variant that allocates nothing (see sampling_no_alloc.h for who needs it and its contract).
#include "sampling_no_alloc.h"

#include <mutex>

namespace {

// Scratch of the two-stage argmax for the largest request this entry point takes. It is part of
// the library's device image: every GPU that loads the library keeps it until the process ends.
static __device__ __align__(256) unsigned char g_sample_scratch[LLM_SAMPLE_NO_ALLOC_SCRATCH_BYTES];

constexpr int kMaxDevices = 64;
void* g_sample_scratch_addr[kMaxDevices] = {};  // device address of the array, per device ordinal
std::mutex g_sample_scratch_mu;

// In host code `g_sample_scratch` is only a handle for the runtime, not a device address: the
// address has to be asked for, once per device, while that device is current.
int sample_scratch_for_current_device(void** addr) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
    llm_set_error("sample_no_alloc: cannot tell the current device (%s)", e == cudaSuccess ? "ordinal out of range" : cudaGetErrorString(e));
    return LLM_ERR_LAUNCH;
  }
  std::lock_guard<std::mutex> lock(g_sample_scratch_mu);
  if (!g_sample_scratch_addr[dev]) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_sample_scratch);
    if (e != cudaSuccess || !p) {
      llm_set_error("sample_no_alloc: cudaGetSymbolAddress failed on device %d: %s", dev, cudaGetErrorString(e));
      return LLM_ERR_LAUNCH;
    }
    g_sample_scratch_addr[dev] = p;
  }
  *addr = g_sample_scratch_addr[dev];
  return LLM_OK;
}

}  // namespace

extern "C" int llm_sample_no_alloc(const float* logits, long long ld, const float* temperature, const int* seeds,
                                   const int* draws, int* out, int n_rows, int vocab, cudaStream_t stream) {
  if (n_rows == 0) return LLM_OK;
  LLM_REQUIRE(n_rows > 0 && vocab > 0 && ld >= vocab, "sample_no_alloc: bad sizes rows=%d vocab=%d", n_rows, vocab);
  LLM_REQUIRE(n_rows <= LLM_SAMPLE_NO_ALLOC_MAX_ROWS, "sample_no_alloc: %d rows exceed the built-in scratch (at most %d rows a call)",
              n_rows, LLM_SAMPLE_NO_ALLOC_MAX_ROWS);
  LLM_REQUIRE(!temperature || (seeds && draws), "sample_no_alloc: temperature needs seeds and draw indices");
  const int chunks = llm_sample_chunks(vocab);
  LLM_REQUIRE(chunks <= LLM_SAMPLE_NO_ALLOC_MAX_CHUNKS, "sample_no_alloc: %d chunks exceed the built-in scratch", chunks);
  void* scratch = nullptr;
  const int rc = sample_scratch_for_current_device(&scratch);
  if (rc != LLM_OK) return rc;
  const int chunk = (vocab + chunks - 1) / chunks;
  float* best_val = (float*)scratch;
  int* best_idx = (int*)scratch + (size_t)n_rows * chunks;
  // every (row, chunk) word read by the merge is written by the scan of this same call
  launch_kernel(sample_scan_kernel, dim3(chunks, n_rows), 256, 0, stream, logits, ld, temperature, seeds, draws, best_val, best_idx, vocab, chunk);
  launch_kernel(sample_merge_kernel, ceil_div(n_rows, 4), 128, 0, stream, (const float*)best_val, (const int*)best_idx, chunks, out, n_rows);
  LLM_CHECK_LAUNCH("sample_no_alloc");
  return LLM_OK;
}
