// Embedding gather, RMSNorm (with the residual sum fused in), SiLU*up, residual add, sums of
// K-split partials. The residual stream is float32 in both engine precisions; sums of squares, the
// reciprocal root and the activation are computed in float32.
//
// Formulas follow the reference CPU ops: rmsnorm_f32 (src/kernels.cpp:18-24: out = w*x*inv_rms,
// inv_rms = 1/sqrt(sum(x^2)/dim + eps)), silu_f32 (src/kernels.cpp:26-31: v/(1+exp(-v))) with the
// product by `up` as a separate multiply (src/engine.cpp:388-389), embed_lookup_f32
// (src/kernels.cpp:59-66).
#include "common.cuh"

// ------------------------------------------------------------------------------------ embedding
// sumsq (may be null): sumsq[row] = sum of the squares of the row, for a norm that is folded into
// the product after it; scaled (may be null): the row times next_w in bfloat16, that product's operand.
template <typename T>
__global__ void embed_kernel(const T* __restrict__ table, const int* __restrict__ ids,
                             float* __restrict__ out, float* __restrict__ sumsq, int dim, int vocab,
                             const float* __restrict__ next_w, bf16* __restrict__ scaled, long long ld_scaled) {
  __shared__ float red[33];
  dep_launch();
  dep_wait();
  const int row = blockIdx.x;
  int id = ids[row];
  if (id < 0 || id >= vocab) id = 0;  // ids are validated on the host; never read out of range
  const T* src = table + (size_t)id * dim;
  float* dst = out + (size_t)row * dim;
  float ss = 0.f;
  for (int i = threadIdx.x; i < dim; i += blockDim.x) {
    const float v = to_f32(src[i]);
    dst[i] = v;
    ss += v * v;
    if (scaled) scaled[(size_t)row * ld_scaled + i] = __float2bfloat16_rn(v * next_w[i]);
  }
  if (sumsq) {
    ss = block_sum(ss, red);
    if (threadIdx.x == 0) sumsq[row] = ss;
  }
}

// next_w, scaled (both or neither): scaled [rows, ld_scaled] bf16 = next_w * row, the operand of the
// product behind a norm with weight next_w whose 1/rms the product's consumer applies from sumsq.
extern "C" int llm_embed(const void* table, int table_dtype, const int* ids, float* out, float* sumsq, int n_rows,
                         int dim, int vocab, const float* next_w, void* scaled, long long ld_scaled, cudaStream_t stream) {
  if (n_rows == 0) return LLM_OK;
  LLM_REQUIRE((next_w == nullptr) == (scaled == nullptr), "embed: the scaled copy needs the weight it is scaled with");
  LLM_REQUIRE(n_rows > 0 && dim > 0 && vocab > 0, "embed: bad sizes rows=%d dim=%d vocab=%d", n_rows, dim, vocab);
  const int threads = dim >= 1024 ? 256 : 128;
  if (table_dtype == LLM_F32)
    launch_kernel(embed_kernel<float>, n_rows, threads, 0, stream, (const float*)table, ids, out, sumsq, dim, vocab, next_w, (bf16*)scaled, ld_scaled);
  else if (table_dtype == LLM_BF16)
    launch_kernel(embed_kernel<bf16>, n_rows, threads, 0, stream, (const bf16*)table, ids, out, sumsq, dim, vocab, next_w, (bf16*)scaled, ld_scaled);
  else
    LLM_REQUIRE(false, "embed: unknown table dtype %d", table_dtype);
  LLM_CHECK_LAUNCH("embed");
  return LLM_OK;
}

// ------------------------------------------------------------------------------------ RMSNorm
// One block per output row. Source row r = rows ? rows[blockIdx.x] : blockIdx.x.
// x = h[r] + sum_p delta[p][r] (partials added in index order); if write_back, h[r] = x.
// out[blockIdx.x] = (w * x) * inv_rms.
template <typename T>
__device__ __forceinline__ void store4(T* dst, float a, float b, float c, float d);
template <>
__device__ __forceinline__ void store4<float>(float* dst, float a, float b, float c, float d) {
  *reinterpret_cast<float4*>(dst) = make_float4(a, b, c, d);
}
template <>
__device__ __forceinline__ void store4<bf16>(bf16* dst, float a, float b, float c, float d) {
  __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
  uint2 v;
  v.x = *reinterpret_cast<uint32_t*>(&lo);
  v.y = *reinterpret_cast<uint32_t*>(&hi);
  *reinterpret_cast<uint2*>(dst) = v;
}

// dim % 4 == 0 and dim <= 4 * R * blockDim: the row stays in registers between the two passes.
template <typename TOut, int R>
__global__ void __launch_bounds__(1024) rmsnorm_vec_kernel(float* __restrict__ h, const float* __restrict__ delta, int n_partials,
                                                           size_t partial_stride, const float* __restrict__ w,
                                                           const int* __restrict__ rows, TOut* __restrict__ out, int dim,
                                                           float eps, int write_back) {
  __shared__ float red[33];
  dep_launch();
  float4 wv[R];
#pragma unroll
  for (int k = 0; k < R; ++k) {  // the norm weight is not produced by the stream: fetch it before waiting
    const int i = (threadIdx.x + k * blockDim.x) * 4;
    wv[k] = i < dim ? *reinterpret_cast<const float4*>(w + i) : make_float4(0, 0, 0, 0);
  }
  dep_wait();
  const int r = rows ? rows[blockIdx.x] : blockIdx.x;
  float* hr = h + (size_t)r * dim;
  const float* dr = delta ? delta + (size_t)r * dim : nullptr;
  float4 x[R];
  float ss = 0.f;
  if (R > 1 && dr && n_partials == 1) {
    // many rows a launch (a prompt), one product to add: every load of the thread is asked for before
    // any is used, so that a row costs one trip to memory, not one per quarter of it
    float4 d[R];
#pragma unroll
    for (int k = 0; k < R; ++k) {
      const int i = (threadIdx.x + k * blockDim.x) * 4;
      x[k] = i < dim ? *reinterpret_cast<const float4*>(hr + i) : make_float4(0, 0, 0, 0);
      d[k] = i < dim ? *reinterpret_cast<const float4*>(dr + i) : make_float4(0, 0, 0, 0);
    }
#pragma unroll
    for (int k = 0; k < R; ++k) {
      const int i = (threadIdx.x + k * blockDim.x) * 4;
      x[k].x += d[k].x; x[k].y += d[k].y; x[k].z += d[k].z; x[k].w += d[k].w;
      if (i < dim) {
        if (write_back) *reinterpret_cast<float4*>(hr + i) = x[k];
        ss += x[k].x * x[k].x + x[k].y * x[k].y + x[k].z * x[k].z + x[k].w * x[k].w;
      }
    }
  } else
#pragma unroll
  for (int k = 0; k < R; ++k) {
    const int i = (threadIdx.x + k * blockDim.x) * 4;
    x[k] = make_float4(0, 0, 0, 0);
    if (i < dim) {
      x[k] = *reinterpret_cast<const float4*>(hr + i);
      if (dr) {
        for (int p0 = 0; p0 < n_partials; p0 += 8) {  // eight loads in flight, then added in index order
          float4 d[8];
#pragma unroll
          for (int u = 0; u < 8; ++u)
            d[u] = (p0 + u < n_partials) ? *reinterpret_cast<const float4*>(dr + (size_t)(p0 + u) * partial_stride + i)
                                         : make_float4(0, 0, 0, 0);
#pragma unroll
          for (int u = 0; u < 8; ++u) {
            if (p0 + u < n_partials) { x[k].x += d[u].x; x[k].y += d[u].y; x[k].z += d[u].z; x[k].w += d[u].w; }
          }
        }
        if (write_back) *reinterpret_cast<float4*>(hr + i) = x[k];
      }
      ss += x[k].x * x[k].x + x[k].y * x[k].y + x[k].z * x[k].z + x[k].w * x[k].w;
    }
  }
  ss = block_sum(ss, red);
  const float inv = 1.0f / sqrtf(ss / (float)dim + eps);
  TOut* o = out + (size_t)blockIdx.x * dim;
#pragma unroll
  for (int k = 0; k < R; ++k) {
    const int i = (threadIdx.x + k * blockDim.x) * 4;
    if (i < dim)
      store4<TOut>(o + i, (wv[k].x * x[k].x) * inv, (wv[k].y * x[k].y) * inv, (wv[k].z * x[k].z) * inv, (wv[k].w * x[k].w) * inv);
  }
}

template <typename TOut>
__global__ void rmsnorm_kernel(float* __restrict__ h, const float* __restrict__ delta, int n_partials,
                               size_t partial_stride, const float* __restrict__ w,
                               const int* __restrict__ rows, TOut* __restrict__ out, int dim, float eps,
                               int write_back) {
  __shared__ float red[33];
  dep_launch();
  dep_wait();
  const int r = rows ? rows[blockIdx.x] : blockIdx.x;
  float* hr = h + (size_t)r * dim;
  const float* dr = delta ? delta + (size_t)r * dim : nullptr;
  float ss = 0.f;
  for (int i = threadIdx.x; i < dim; i += blockDim.x) {
    float x = hr[i];
    if (dr) {
      for (int p = 0; p < n_partials; ++p) x += dr[(size_t)p * partial_stride + i];
      if (write_back) hr[i] = x;
    }
    ss += x * x;
  }
  ss = block_sum(ss, red);
  const float inv = 1.0f / sqrtf(ss / (float)dim + eps);
  TOut* o = out + (size_t)blockIdx.x * dim;
  for (int i = threadIdx.x; i < dim; i += blockDim.x) {
    float x = hr[i];
    if (dr && !write_back)
      for (int p = 0; p < n_partials; ++p) x += dr[(size_t)p * partial_stride + i];
    o[i] = from_f32<TOut>((w[i] * x) * inv);
  }
}

template <typename TOut>
static void launch_rmsnorm(float* h, const float* delta, int n_partials, size_t partial_stride, const float* w, const int* rows,
                           TOut* out, int n_out_rows, int dim, float eps, int write_back, cudaStream_t stream) {
  auto al = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; };
  const bool vec = dim % 4 == 0 && dim <= 16384 && al(h) && al(w) && al(out) && (!delta || (al(delta) && partial_stride % 4 == 0));
  if (vec) {
    const int quads = dim / 4;
    int threads = quads <= 1024 ? ((quads + 31) / 32) * 32 : 1024;
    // Many rows (a prompt): a quarter of the threads with four float4 each, so that every row of the
    // launch is resident at once and all of its bytes are on their way together.
    if (n_out_rows >= 512 && quads >= 256 && quads <= 4096) threads = ((quads / 4 + 31) / 32) * 32;
    const int per_thread = (quads + threads - 1) / threads;
    if (per_thread == 1)
      launch_kernel(rmsnorm_vec_kernel<TOut, 1>, n_out_rows, threads, 0, stream, h, delta, n_partials, partial_stride, w, rows, out, dim, eps, write_back);
    else if (per_thread == 2)
      launch_kernel(rmsnorm_vec_kernel<TOut, 2>, n_out_rows, threads, 0, stream, h, delta, n_partials, partial_stride, w, rows, out, dim, eps, write_back);
    else
      launch_kernel(rmsnorm_vec_kernel<TOut, 4>, n_out_rows, threads, 0, stream, h, delta, n_partials, partial_stride, w, rows, out, dim, eps, write_back);
    return;
  }
  int threads = 128;
  while (threads < 1024 && threads * 4 < dim) threads *= 2;
  launch_kernel(rmsnorm_kernel<TOut>, n_out_rows, threads, 0, stream, h, delta, n_partials, partial_stride, w, rows, out, dim, eps, write_back);
}

extern "C" int llm_rmsnorm(float* h, const float* delta, int n_partials, long long partial_stride,
                           const float* w, const int* rows, void* out, int out_dtype, int n_out_rows,
                           int dim, float eps, int write_back, cudaStream_t stream) {
  if (n_out_rows == 0) return LLM_OK;
  LLM_REQUIRE(n_out_rows > 0 && dim > 0, "rmsnorm: bad sizes rows=%d dim=%d", n_out_rows, dim);
  LLM_REQUIRE(!(rows && write_back), "rmsnorm: write_back with a row list is not allowed");
  LLM_REQUIRE(!delta || n_partials >= 1, "rmsnorm: delta needs n_partials >= 1");
  if (out_dtype == LLM_F32)
    launch_rmsnorm<float>(h, delta, n_partials, (size_t)partial_stride, w, rows, (float*)out, n_out_rows, dim, eps, write_back, stream);
  else if (out_dtype == LLM_BF16)
    launch_rmsnorm<bf16>(h, delta, n_partials, (size_t)partial_stride, w, rows, (bf16*)out, n_out_rows, dim, eps, write_back, stream);
  else
    LLM_REQUIRE(false, "rmsnorm: unknown out dtype %d", out_dtype);
  LLM_CHECK_LAUNCH("rmsnorm");
  return LLM_OK;
}

// ------------------------------------------------------------------------------------ residual add
__global__ void residual_add_kernel(float* __restrict__ h, const float* __restrict__ delta, int n_partials,
                                    size_t partial_stride, size_t n) {
  dep_launch();
  dep_wait();
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  float x = h[i];
  for (int p = 0; p < n_partials; ++p) x += delta[(size_t)p * partial_stride + i];
  h[i] = x;
}

extern "C" int llm_residual_add(float* h, const float* delta, int n_partials, long long partial_stride,
                                long long n, cudaStream_t stream) {
  if (n == 0) return LLM_OK;
  LLM_REQUIRE(n > 0 && n_partials >= 1, "residual_add: bad sizes");
  launch_kernel(residual_add_kernel, ceil_div(n, 256), 256, 0, stream, h, delta, n_partials, (size_t)partial_stride, (size_t)n);
  LLM_CHECK_LAUNCH("residual_add");
  return LLM_OK;
}

// ------------------------------------------------------------------------------------ SiLU(gate) * up
// in: [rows, 2*ff]; out: [rows, ff]. Column layout of `in`: block == 0: gate in columns [0,ff), up in
// [ff,2ff); block == b > 0: blocks of 2b columns, b of gate followed by the b matching ones of up.
__device__ __forceinline__ void gate_up_columns(int c, int ff, int block, size_t* gate, size_t* up) {
  if (block == 0) {
    *gate = c;
    *up = (size_t)ff + c;
  } else {
    *gate = (size_t)(c / block) * 2 * block + (c % block);
    *up = *gate + block;
  }
}

template <typename T>
__global__ void silu_mul_kernel(const T* __restrict__ in, T* __restrict__ out, int ff, size_t total, int block) {
  dep_launch();
  dep_wait();
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const size_t r = i / ff;
  const int c = (int)(i - r * ff);
  size_t gc, uc;
  gate_up_columns(c, ff, block, &gc, &uc);
  const float g = to_f32(in[r * 2 * ff + gc]);
  const float u = to_f32(in[r * 2 * ff + uc]);
  float s = g / (1.0f + expf(-g));
  out[i] = from_f32<T>(s * u);
}

extern "C" int llm_silu_mul(const void* in, void* out, int dtype, int n_rows, int ff, int block, cudaStream_t stream) {
  if (n_rows == 0) return LLM_OK;
  LLM_REQUIRE(n_rows > 0 && ff > 0, "silu_mul: bad sizes rows=%d ff=%d", n_rows, ff);
  LLM_REQUIRE(block >= 0 && (block == 0 || ff % block == 0), "silu_mul: column block %d does not divide %d", block, ff);
  const size_t total = (size_t)n_rows * ff;
  const int blocks = ceil_div((long long)total, 256);
  if (dtype == LLM_F32)
    launch_kernel(silu_mul_kernel<float>, blocks, 256, 0, stream, (const float*)in, (float*)out, ff, total, block);
  else if (dtype == LLM_BF16)
    launch_kernel(silu_mul_kernel<bf16>, blocks, 256, 0, stream, (const bf16*)in, (bf16*)out, ff, total, block);
  else
    LLM_REQUIRE(false, "silu_mul: unknown dtype %d", dtype);
  LLM_CHECK_LAUNCH("silu_mul");
  return LLM_OK;
}

// ------------------------------------------------------------------------------------ partial sums
// K-split matrix products leave float32 partials [parts, rows, width]; these kernels add them in
// index order (a fixed order: the result does not depend on timing) while doing their own work.
template <typename T>
__global__ void reduce_partials_kernel(const float* __restrict__ partials, int n_partials, size_t stride,
                                       T* __restrict__ out, size_t total) {
  dep_launch();
  dep_wait();
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  float x = partials[i];
  for (int p = 1; p < n_partials; ++p) x += partials[(size_t)p * stride + i];
  out[i] = from_f32<T>(x);
}

extern "C" int llm_reduce_partials(const float* partials, int n_partials, long long stride, void* out, int out_dtype,
                                   long long total, cudaStream_t stream) {
  if (total == 0) return LLM_OK;
  LLM_REQUIRE(total > 0 && n_partials >= 1, "reduce_partials: bad sizes");
  const int blocks = ceil_div(total, 256);
  if (out_dtype == LLM_F32)
    launch_kernel(reduce_partials_kernel<float>, blocks, 256, 0, stream, partials, n_partials, (size_t)stride, (float*)out, (size_t)total);
  else if (out_dtype == LLM_BF16)
    launch_kernel(reduce_partials_kernel<bf16>, blocks, 256, 0, stream, partials, n_partials, (size_t)stride, (bf16*)out, (size_t)total);
  else
    LLM_REQUIRE(false, "reduce_partials: unknown dtype %d", out_dtype);
  LLM_CHECK_LAUNCH("reduce_partials");
  return LLM_OK;
}

// partials: [parts, rows, 2*ff] float32 (gate | up); out [rows, ff] = silu(sum gate) * (sum up).
template <typename T>
__global__ void silu_mul_partials_kernel(const float* __restrict__ partials, int n_partials, size_t stride,
                                         T* __restrict__ out, int ff, size_t total, int block, const RowScale rs) {
  dep_launch();
  dep_wait();
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const size_t r = i / ff;
  const int c = (int)(i - r * ff);
  size_t gc, uc;
  gate_up_columns(c, ff, block, &gc, &uc);
  const size_t gi = r * 2 * ff + gc, ui = r * 2 * ff + uc;
  float g = 0.f, u = 0.f;
  for (int p0 = 0; p0 < n_partials; p0 += 4) {  // four parts' loads in flight, added in index order
    float gv[4], uv[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const bool in = p0 + k < n_partials;
      gv[k] = in ? partials[(size_t)(p0 + k) * stride + gi] : 0.f;
      uv[k] = in ? partials[(size_t)(p0 + k) * stride + ui] : 0.f;
    }
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      g += gv[k];
      u += uv[k];
    }
  }
  const float sc = row_scale(rs, r);  // the norm before the product, when its 1/rms is still owed
  g *= sc;
  u *= sc;
  const float s = g / (1.0f + expf(-g));
  out[i] = from_f32<T>(s * u);
}

extern "C" int llm_silu_mul_partials(const float* partials, int n_partials, long long stride, void* out, int out_dtype,
                                     int n_rows, int ff, int block, const float* sumsq, int n_sumsq, float inv_dim, float eps,
                                     cudaStream_t stream) {
  if (n_rows == 0) return LLM_OK;
  const RowScale rs{sumsq, n_sumsq, inv_dim, eps};
  LLM_REQUIRE(n_rows > 0 && ff > 0 && n_partials >= 1, "silu_mul_partials: bad sizes");
  LLM_REQUIRE(block >= 0 && (block == 0 || ff % block == 0), "silu_mul_partials: column block %d does not divide %d", block, ff);
  const size_t total = (size_t)n_rows * ff;
  const int blocks = ceil_div((long long)total, 256);
  if (out_dtype == LLM_F32)
    launch_kernel(silu_mul_partials_kernel<float>, blocks, 256, 0, stream, partials, n_partials, (size_t)stride, (float*)out, ff, total, block, rs);
  else if (out_dtype == LLM_BF16)
    launch_kernel(silu_mul_partials_kernel<bf16>, blocks, 256, 0, stream, partials, n_partials, (size_t)stride, (bf16*)out, ff, total, block, rs);
  else
    LLM_REQUIRE(false, "silu_mul_partials: unknown dtype %d", out_dtype);
  LLM_CHECK_LAUNCH("silu_mul_partials");
  return LLM_OK;
}
