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

// With `parts` (float32 [n_parts, tokens, width] partial sums of the q|k|v product) the values are
// the sums over parts in index order and only the q section of qkv is written.
//
// grid (tokens, chunks of 128 items); an item is one rotation pair of a q or k head, or two
// neighbouring elements of v. Eight partial-sum loads are in flight per thread.
template <typename T>
__global__ void __launch_bounds__(128)
    rope_kv_write_kernel(T* __restrict__ qkv, long long ld_qkv, const float* __restrict__ parts, int n_parts, size_t part_stride,
                         const int* __restrict__ positions, const int* __restrict__ token_seq,
                         const int* __restrict__ block_table, int max_blocks, const float* __restrict__ cos_t,
                         const float* __restrict__ sin_t, T* __restrict__ kcache, T* __restrict__ vcache, int nq, int nkv,
                         int hd, int page_size, const RowScale rs) {
  dep_launch();
  dep_wait();
  const int t = blockIdx.x;
  const int half = hd >> 1;
  const int n_pairs = (nq + nkv) * half, n_vpairs = vcache ? nkv * half : 0;
  const int item = blockIdx.y * blockDim.x + threadIdx.x;
  if (item >= n_pairs + n_vpairs) return;
  const int pos = positions[t];
  const int width = (nq + 2 * nkv) * hd;
  T* row = qkv + (size_t)t * ld_qkv;

  // the two columns of the q|k|v row that this thread owns
  int col_a, col_b, head = 0, i = 0;
  const bool is_v = item >= n_pairs;
  if (!is_v) {
    head = item / half;
    i = item - head * half;
    col_a = head * hd + i;
    col_b = col_a + half;
  } else {
    col_a = (nq + nkv) * hd + 2 * (item - n_pairs);
    col_b = col_a + 1;
  }
  float a, b;
  if (parts) {
    const float* pa = parts + (size_t)t * width + col_a;
    const float* pb = parts + (size_t)t * width + col_b;
    a = 0.f;
    b = 0.f;
    for (int p0 = 0; p0 < n_parts; p0 += 8) {
      float va[8], vb[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const bool in = p0 + u < n_parts;
        va[u] = in ? pa[(size_t)(p0 + u) * part_stride] : 0.f;
        vb[u] = in ? pb[(size_t)(p0 + u) * part_stride] : 0.f;
      }
#pragma unroll
      for (int u = 0; u < 8; ++u) {  // index order; the zeros of a short last batch change nothing
        a += va[u];
        b += vb[u];
      }
    }
    const float sc = row_scale(rs, (size_t)t);  // the norm before the product, when its 1/rms is still owed
    a *= sc;
    b *= sc;
  } else {
    a = to_f32(row[col_a]);
    b = to_f32(row[col_b]);
  }

  size_t cache_base = 0;
  if (kcache) {
    const int page = block_table[(size_t)token_seq[t] * max_blocks + pos / page_size];
    cache_base = ((size_t)page * nkv * page_size + (pos % page_size)) * hd;  // + kv_head*page_size*hd
  }
  const size_t head_stride = (size_t)page_size * hd;

  if (is_v) {
    const int e = 2 * (item - n_pairs), vh = e / hd, vi = e - vh * hd;  // hd is even: both elements in one head
    T* dst = vcache + cache_base + (size_t)vh * head_stride + vi;
    dst[0] = from_f32<T>(a);
    dst[1] = from_f32<T>(b);
    return;
  }
  float ra = a, rb = b;
  if (cos_t) {
    const float c = cos_t[(size_t)pos * half + i], s = sin_t[(size_t)pos * half + i];
    ra = a * c - b * s;
    rb = b * c + a * s;
  }
  const T oa = from_f32<T>(ra), ob = from_f32<T>(rb);
  if (head < nq || !kcache) {
    row[col_a] = oa;
    row[col_b] = ob;
  } else {
    T* dst = kcache + cache_base + (size_t)(head - nq) * head_stride;
    dst[i] = oa;
    dst[i + half] = ob;
  }
}

// bfloat16 rows without partial sums, 16 bytes at a time: an item is 8 neighbouring rotation pairs
// of a q or k head (8 elements of the first half with their 8 partners of the second half), or 8
// neighbouring elements of v. Needs head_dim % 16 == 0 and 16-byte aligned rows.
__global__ void __launch_bounds__(128)
    rope_kv_write_vec_kernel(bf16* __restrict__ qkv, long long ld_qkv, const int* __restrict__ positions,
                             const int* __restrict__ token_seq, const int* __restrict__ block_table, int max_blocks,
                             const float* __restrict__ cos_t, const float* __restrict__ sin_t, bf16* __restrict__ kcache,
                             bf16* __restrict__ vcache, int nq, int nkv, int hd, int page_size) {
  dep_launch();
  dep_wait();
  const int t = blockIdx.x;
  const int half = hd >> 1, groups = half >> 3;  // groups of 8 pairs per head
  const int n_rot = (nq + nkv) * groups, n_v = vcache ? nkv * (hd >> 3) : 0;
  const int item = blockIdx.y * blockDim.x + threadIdx.x;
  if (item >= n_rot + n_v) return;
  const int pos = positions[t];
  bf16* row = qkv + (size_t)t * ld_qkv;
  size_t cache_base = 0;
  if (kcache) {
    const int page = block_table[(size_t)token_seq[t] * max_blocks + pos / page_size];
    cache_base = ((size_t)page * nkv * page_size + (pos % page_size)) * hd;
  }
  const size_t head_stride = (size_t)page_size * hd;
  if (item >= n_rot) {  // 8 elements of v, copied as they are
    const int e = (item - n_rot) * 8, vh = e / hd, vi = e - vh * hd;
    *reinterpret_cast<uint4*>(vcache + cache_base + (size_t)vh * head_stride + vi) =
        *reinterpret_cast<const uint4*>(row + (size_t)(nq + nkv) * hd + e);
    return;
  }
  const int head = item / groups, i0 = (item - head * groups) * 8;
  bf16* x = row + (size_t)head * hd;
  union { uint4 u; __nv_bfloat162 h[4]; } a, b;
  a.u = *reinterpret_cast<const uint4*>(x + i0);
  b.u = *reinterpret_cast<const uint4*>(x + i0 + half);
  if (cos_t) {
    const float4* c4 = reinterpret_cast<const float4*>(cos_t + (size_t)pos * half + i0);
    const float4* s4 = reinterpret_cast<const float4*>(sin_t + (size_t)pos * half + i0);
    float c[8], sn[8];
    *reinterpret_cast<float4*>(c) = c4[0];
    *reinterpret_cast<float4*>(c + 4) = c4[1];
    *reinterpret_cast<float4*>(sn) = s4[0];
    *reinterpret_cast<float4*>(sn + 4) = s4[1];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 av = __bfloat1622float2(a.h[j]), bv = __bfloat1622float2(b.h[j]);
      const float ra0 = av.x * c[2 * j] - bv.x * sn[2 * j], rb0 = bv.x * c[2 * j] + av.x * sn[2 * j];
      const float ra1 = av.y * c[2 * j + 1] - bv.y * sn[2 * j + 1], rb1 = bv.y * c[2 * j + 1] + av.y * sn[2 * j + 1];
      a.h[j] = __floats2bfloat162_rn(ra0, ra1);
      b.h[j] = __floats2bfloat162_rn(rb0, rb1);
    }
  }
  bf16* dst = (head < nq || !kcache) ? x : kcache + cache_base + (size_t)(head - nq) * head_stride;
  *reinterpret_cast<uint4*>(dst + i0) = a.u;
  *reinterpret_cast<uint4*>(dst + i0 + half) = b.u;
}

// cos_t/sin_t may be null (no rotation); kcache/vcache may be null (a layer that reads another
// layer's cache writes nothing, and k is then rotated in place in qkv).
extern "C" int llm_rope_kv_write(void* qkv, long long ld_qkv, int dtype, const float* parts, int n_parts,
                                 long long part_stride, const int* positions,
                                 const int* token_seq, const int* block_table, int max_blocks,
                                 const float* cos_t, const float* sin_t, void* kcache, void* vcache,
                                 int n_tokens, int nq, int nkv, int hd, int page_size, const float* sumsq, int n_sumsq,
                                 float inv_dim, float eps, cudaStream_t stream) {
  if (n_tokens == 0) return LLM_OK;
  const RowScale rs{sumsq, n_sumsq, inv_dim, eps};
  LLM_REQUIRE(!sumsq || (parts && n_sumsq > 0), "rope_kv_write: a row scale goes with partial sums");
  LLM_REQUIRE(n_tokens > 0 && nq > 0 && nkv > 0 && hd > 0 && hd % 2 == 0 && page_size > 0,
              "rope_kv_write: bad sizes tokens=%d nq=%d nkv=%d hd=%d page=%d", n_tokens, nq, nkv, hd, page_size);
  LLM_REQUIRE((cos_t == nullptr) == (sin_t == nullptr), "rope_kv_write: cos and sin tables go together");
  LLM_REQUIRE((kcache == nullptr) == (vcache == nullptr), "rope_kv_write: k and v caches go together");
  LLM_REQUIRE(!parts || (n_parts >= 1 && kcache), "rope_kv_write: partial sums need n_parts >= 1 and a cache to write to");
  const int threads = 128;
  auto al = [](const void* ptr) { return (reinterpret_cast<uintptr_t>(ptr) & 15u) == 0; };
  if (dtype == LLM_BF16 && !parts && hd % 16 == 0 && ld_qkv % 8 == 0 && al(qkv) && al(kcache) && al(vcache) && al(cos_t) && al(sin_t)) {
    const int vitems = (nq + nkv) * (hd / 16) + (vcache ? nkv * (hd / 8) : 0);
    const dim3 vgrid(n_tokens, ceil_div(vitems, threads));
    LLM_REQUIRE(vgrid.y <= 65535, "rope_kv_write: too many heads");
    launch_kernel(rope_kv_write_vec_kernel, vgrid, threads, 0, stream, (bf16*)qkv, ld_qkv, positions, token_seq, block_table,
                  max_blocks, cos_t, sin_t, (bf16*)kcache, (bf16*)vcache, nq, nkv, hd, page_size);
    LLM_CHECK_LAUNCH("rope_kv_write");
    return LLM_OK;
  }
  const int items = (nq + nkv) * (hd / 2) + (vcache ? nkv * (hd / 2) : 0);
  const dim3 grid(n_tokens, ceil_div(items, threads));
  LLM_REQUIRE(grid.y <= 65535, "rope_kv_write: too many heads");
  if (dtype == LLM_F32)
    launch_kernel(rope_kv_write_kernel<float>, grid, threads, 0, stream, (float*)qkv, ld_qkv, parts, n_parts,
                  (size_t)part_stride, positions, token_seq, block_table, max_blocks, cos_t, sin_t, (float*)kcache,
                  (float*)vcache, nq, nkv, hd, page_size, rs);
  else if (dtype == LLM_BF16)
    launch_kernel(rope_kv_write_kernel<bf16>, grid, threads, 0, stream, (bf16*)qkv, ld_qkv, parts, n_parts,
                  (size_t)part_stride, positions, token_seq, block_table, max_blocks, cos_t, sin_t, (bf16*)kcache,
                  (bf16*)vcache, nq, nkv, hd, page_size, rs);
  else
    LLM_REQUIRE(false, "rope_kv_write: unknown dtype %d", dtype);
  LLM_CHECK_LAUNCH("rope_kv_write");
  return LLM_OK;
}
