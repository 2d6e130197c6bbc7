// Rotary position encoding of q and k, fused with the write of k (rotated) and v (raw) into the
// paged cache.
//
// Rotation is the half-split form of the reference's apply_rope_inplace (src/kernels.cpp:189-203):
//   x[i] = a*cos[i] - b*sin[i];  x[i+half] = b*cos[i] + a*sin[i],   a = x[i], b = x[i+half]
// with cos/sin read from float32 tables indexed by the token's absolute position. The tables are
// built on the host in float64 exactly as build_rope_tables does (src/kernels.cpp:162-187). K is
// cached after rotation, V untouched (src/engine.cpp:343-353).
//
// Cache layout of one layer: [page, kv_head, slot_in_page, head_dim]; the page of position p of a
// request is block_table[request_row][p / page_size].
#include "common.cuh"

template <typename T>
__global__ void rope_kv_write_kernel(T* __restrict__ qkv, long long ld_qkv, const int* __restrict__ positions,
                                     const int* __restrict__ token_seq, const int* __restrict__ block_table,
                                     int max_blocks, const float* __restrict__ cos_t,
                                     const float* __restrict__ sin_t, T* __restrict__ kcache,
                                     T* __restrict__ vcache, int nq, int nkv, int hd, int page_size) {
  const int t = blockIdx.x;
  const int pos = positions[t];
  const int half = hd >> 1;
  T* row = qkv + (size_t)t * ld_qkv;
  T* q = row;
  T* k = row + (size_t)nq * hd;
  T* v = k + (size_t)nkv * hd;

  size_t cache_base = 0;
  if (kcache) {
    const int page = block_table[(size_t)token_seq[t] * max_blocks + pos / page_size];
    cache_base = ((size_t)page * nkv * page_size + (pos % page_size)) * hd;  // + kv_head*page_size*hd
  }
  const size_t head_stride = (size_t)page_size * hd;

  // q and k heads: (nq + nkv) * half pairs
  const int n_pairs = (nq + nkv) * half;
  for (int idx = threadIdx.x; idx < n_pairs; idx += blockDim.x) {
    const int head = idx / half, i = idx - head * half;
    T* x = (head < nq) ? q + (size_t)head * hd : k + (size_t)(head - nq) * hd;
    float a = to_f32(x[i]), b = to_f32(x[i + half]);
    float ra = a, rb = b;
    if (cos_t) {
      const float c = cos_t[(size_t)pos * half + i], s = sin_t[(size_t)pos * half + i];
      ra = a * c - b * s;
      rb = b * c + a * s;
    }
    const T oa = from_f32<T>(ra), ob = from_f32<T>(rb);
    if (head < nq) {
      x[i] = oa;
      x[i + half] = ob;
    } else if (kcache) {
      T* dst = kcache + cache_base + (size_t)(head - nq) * head_stride;
      dst[i] = oa;
      dst[i + half] = ob;
    } else {
      x[i] = oa;
      x[i + half] = ob;
    }
  }
  if (vcache) {
    const int n_v = nkv * hd;
    for (int idx = threadIdx.x; idx < n_v; idx += blockDim.x) {
      const int head = idx / hd, i = idx - head * hd;
      vcache[cache_base + (size_t)head * head_stride + i] = v[idx];
    }
  }
}

// cos_t/sin_t may be null (no rotation); kcache/vcache may be null (a layer that reads another
// layer's cache writes nothing, and k is then rotated in place in qkv).
extern "C" int llm_rope_kv_write(void* qkv, long long ld_qkv, int dtype, const int* positions,
                                 const int* token_seq, const int* block_table, int max_blocks,
                                 const float* cos_t, const float* sin_t, void* kcache, void* vcache,
                                 int n_tokens, int nq, int nkv, int hd, int page_size, cudaStream_t stream) {
  if (n_tokens == 0) return LLM_OK;
  LLM_REQUIRE(n_tokens > 0 && nq > 0 && nkv > 0 && hd > 0 && hd % 2 == 0 && page_size > 0,
              "rope_kv_write: bad sizes tokens=%d nq=%d nkv=%d hd=%d page=%d", n_tokens, nq, nkv, hd, page_size);
  LLM_REQUIRE((cos_t == nullptr) == (sin_t == nullptr), "rope_kv_write: cos and sin tables go together");
  LLM_REQUIRE((kcache == nullptr) == (vcache == nullptr), "rope_kv_write: k and v caches go together");
  const int threads = 256;
  if (dtype == LLM_F32)
    rope_kv_write_kernel<float><<<n_tokens, threads, 0, stream>>>((float*)qkv, ld_qkv, positions, token_seq,
                                                                  block_table, max_blocks, cos_t, sin_t,
                                                                  (float*)kcache, (float*)vcache, nq, nkv, hd, page_size);
  else if (dtype == LLM_BF16)
    rope_kv_write_kernel<bf16><<<n_tokens, threads, 0, stream>>>((bf16*)qkv, ld_qkv, positions, token_seq,
                                                                 block_table, max_blocks, cos_t, sin_t,
                                                                 (bf16*)kcache, (bf16*)vcache, nq, nkv, hd, page_size);
  else
    LLM_REQUIRE(false, "rope_kv_write: unknown dtype %d", dtype);
  LLM_CHECK_LAUNCH("rope_kv_write");
  return LLM_OK;
}
