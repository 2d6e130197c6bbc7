// Causal grouped-query attention over the paged cache, CUDA cores, float32 arithmetic.
//
// One warp owns one (token, query head) of the step's flat batch. The token's keys are the cache
// positions lo..pos of its request (pos = the token's absolute position, lo = 0 or pos-window+1),
// read through the request's block table, so prompt portions and single decoded tokens are the
// same case. Keys are taken in chunks of 32 aligned to absolute positions with a running
// (max, sum) softmax; the chunking depends only on (lo, pos), hence a token's output does not
// depend on how its request was cut into steps, on the rest of the batch, or on page numbers.
//
// Formula of the reference's attention_f32 (src/kernels.cpp:413-474): kv head = q head / (nq/nkv),
// score = (q . k) * (1/sqrt(head_dim)) with the scale applied after the dot, softmax in float32,
// output = sum_t p_t * V[t].
#include "common.cuh"

#include <cfloat>
#include <cmath>

namespace {

constexpr int WARPS = 4;
constexpr int MAX_HD = 256;

template <typename T, int R>  // R = ceil(hd / 32) output registers per lane
__global__ void __launch_bounds__(WARPS * 32)
    paged_attention_simt_kernel(const T* __restrict__ q, long long ld_q, const T* __restrict__ kcache,
                                const T* __restrict__ vcache, const int* __restrict__ positions,
                                const int* __restrict__ token_seq, const int* __restrict__ block_table,
                                int max_blocks, T* __restrict__ out, long long ld_out, int n_tokens, int nq,
                                int nkv, int hd, int page_size, float scale, int window) {
  __shared__ float q_s[WARPS][MAX_HD];
  dep_launch();
  dep_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long item = (long long)blockIdx.x * WARPS + warp;
  if (item >= (long long)n_tokens * nq) return;  // whole warp leaves together
  const int tok = (int)(item / nq), head = (int)(item - (long long)tok * nq);
  const int kvh = head / (nq / nkv);
  const int pos = positions[tok];
  const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
  const int* table = block_table + (size_t)token_seq[tok] * max_blocks;

  const T* qv = q + (size_t)tok * ld_q + (size_t)head * hd;
  for (int d = lane; d < hd; d += 32) q_s[warp][d] = to_f32(qv[d]);
  __syncwarp();

  float acc[R];
#pragma unroll
  for (int i = 0; i < R; ++i) acc[i] = 0.f;
  float m = -INFINITY, l = 0.f;
  const size_t head_stride = (size_t)page_size * hd;

  for (int c = lo / 32; c <= pos / 32; ++c) {
    const int t = c * 32 + lane;
    const bool valid = (t >= lo) && (t <= pos);
    float s = -INFINITY;
    size_t v_off = 0;
    if (valid) {
      const int page = table[t / page_size];
      const size_t off = ((size_t)page * nkv + kvh) * head_stride + (size_t)(t % page_size) * hd;
      v_off = off;
      const T* kr = kcache + off;
      float dot = 0.f;
      for (int d = 0; d < hd; ++d) dot = fmaf(q_s[warp][d], to_f32(kr[d]), dot);
      s = dot * scale;
    }
    const float m_new = fmaxf(m, warp_max(s));  // finite: the chunk holds at least one valid key
    const float alpha = (m == -INFINITY) ? 0.f : expf(m - m_new);
    const float p = valid ? expf(s - m_new) : 0.f;
    l = l * alpha + warp_sum(p);
#pragma unroll
    for (int i = 0; i < R; ++i) acc[i] *= alpha;
    const int j_end = min(32, pos - c * 32 + 1);
    const int j_begin = max(0, lo - c * 32);
    for (int j = j_begin; j < j_end; ++j) {
      const float pj = __shfl_sync(0xffffffffu, p, j);
      const size_t off_j = __shfl_sync(0xffffffffu, (unsigned long long)v_off, j);
      const T* vr = vcache + off_j;
#pragma unroll
      for (int i = 0; i < R; ++i) {
        const int d = lane + 32 * i;
        if (d < hd) acc[i] = fmaf(pj, to_f32(vr[d]), acc[i]);
      }
    }
    m = m_new;
  }
  const float inv = 1.0f / l;
  T* o = out + (size_t)tok * ld_out + (size_t)head * hd;
#pragma unroll
  for (int i = 0; i < R; ++i) {
    const int d = lane + 32 * i;
    if (d < hd) o[d] = from_f32<T>(acc[i] * inv);
  }
}

template <typename T>
int launch(const void* q, long long ld_q, const void* kc, const void* vc, const int* positions,
           const int* token_seq, const int* block_table, int max_blocks, void* out, long long ld_out,
           int n_tokens, int nq, int nkv, int hd, int page_size, float scale, int window, cudaStream_t stream) {
  const long long items = (long long)n_tokens * nq;
  const int grid = ceil_div(items, WARPS);
#define LLM_ATT_CASE(R)                                                                                     \
  launch_kernel(paged_attention_simt_kernel<T, R>, grid, WARPS * 32, 0, stream, (const T*)q, ld_q, (const T*)kc, \
                (const T*)vc, positions, token_seq, block_table, max_blocks, (T*)out, ld_out, n_tokens, nq, nkv, hd, \
                page_size, scale, window)
  if (hd <= 32) LLM_ATT_CASE(1);
  else if (hd <= 64) LLM_ATT_CASE(2);
  else if (hd <= 128) LLM_ATT_CASE(4);
  else LLM_ATT_CASE(8);
#undef LLM_ATT_CASE
  return 0;
}

}  // namespace

extern "C" int llm_paged_attention_simt(const void* q, long long ld_q, const void* kcache, const void* vcache,
                                        int dtype, const int* positions, const int* token_seq,
                                        const int* block_table, int max_blocks, void* out, long long ld_out,
                                        int n_tokens, int nq, int nkv, int hd, int page_size, float scale,
                                        int window, cudaStream_t stream) {
  if (n_tokens == 0) return LLM_OK;
  LLM_REQUIRE(n_tokens > 0 && nq > 0 && nkv > 0 && nq % nkv == 0, "attention: bad head counts nq=%d nkv=%d", nq, nkv);
  LLM_REQUIRE(hd > 0 && hd <= MAX_HD, "attention: head_dim %d not in 1..%d", hd, MAX_HD);
  LLM_REQUIRE(page_size > 0 && max_blocks > 0 && window >= 0, "attention: bad page_size/max_blocks/window");
  if (dtype == LLM_F32)
    launch<float>(q, ld_q, kcache, vcache, positions, token_seq, block_table, max_blocks, out, ld_out, n_tokens,
                  nq, nkv, hd, page_size, scale, window, stream);
  else if (dtype == LLM_BF16)
    launch<bf16>(q, ld_q, kcache, vcache, positions, token_seq, block_table, max_blocks, out, ld_out, n_tokens,
                 nq, nkv, hd, page_size, scale, window, stream);
  else
    LLM_REQUIRE(false, "attention: unknown dtype %d", dtype);
  LLM_CHECK_LAUNCH("paged_attention_simt");
  return LLM_OK;
}
