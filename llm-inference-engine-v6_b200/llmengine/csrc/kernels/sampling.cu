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

__global__ void __launch_bounds__(1024) sample_kernel(const float* __restrict__ logits, long long ld,
                                                       const float* __restrict__ temperature,
                                                       const int* __restrict__ seeds, const int* __restrict__ draws,
                                                       int* __restrict__ out, int vocab) {
  __shared__ float best_v[32];
  __shared__ int best_i[32];
  const int row = blockIdx.x;
  const float* lr = logits + (size_t)row * ld;
  const float temp = temperature ? temperature[row] : 0.f;
  float bv = -INFINITY;
  int bi = 0x7fffffff;
  if (temp > 0.f) {
    const float inv_t = 1.0f / temp;
    unsigned k = mix32((unsigned)seeds[row] ^ 0x9E3779B9u);
    k = mix32(k + (unsigned)draws[row]);
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
      const unsigned r = mix32(k ^ ((unsigned)i * 0x85EBCA6Bu));
      const float u = __fmul_rn((float)(r >> 9) + 0.5f, 1.0f / 8388608.0f);
      const float g = -logf(-logf(u));
      const float z = __fadd_rn(__fmul_rn(lr[i], inv_t), g);
      if (z > bv) { bv = z; bi = i; }  // ascending i per thread: first maximum kept
    }
  } else {
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
      const float z = lr[i];
      if (z > bv) { bv = z; bi = i; }
    }
  }
  // NaN-free inputs assumed; a row of only -inf or NaN yields index 0 below.
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
    if (lane == 0) out[row] = (bi == 0x7fffffff) ? 0 : bi;
  }
}

}  // namespace

// temperature/seeds/draws: one per row; temperature may be null (all greedy).
extern "C" int llm_sample(const float* logits, long long ld, const float* temperature, const int* seeds,
                          const int* draws, int* out, int n_rows, int vocab, cudaStream_t stream) {
  if (n_rows == 0) return LLM_OK;
  LLM_REQUIRE(n_rows > 0 && vocab > 0 && ld >= vocab, "sample: bad sizes rows=%d vocab=%d", n_rows, vocab);
  LLM_REQUIRE(!temperature || (seeds && draws), "sample: temperature needs seeds and draw indices");
  const int threads = vocab >= 8192 ? 1024 : 256;
  sample_kernel<<<n_rows, threads, 0, stream>>>(logits, ld, temperature, seeds, draws, out, vocab);
  LLM_CHECK_LAUNCH("sample");
  return LLM_OK;
}
