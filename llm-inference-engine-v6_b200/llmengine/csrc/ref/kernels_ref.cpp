// Plain C++ twins of the CUDA kernels: one scalar loop per kernel, host memory, float32 (rotation
// set-up in float64), the same arguments and meaning as the kernel of the same name under
// csrc/kernels. They are what the kernel tests compare with; nothing of the engine calls them.
// Every function restates the formula of the reference engine that its kernel implements and names
// where that formula stands in the reference's sources.
//
// bf16 inputs are passed as float32 holding bf16-representable values; "round to bf16" below is
// round-to-nearest-even, as the kernels' conversions do.
#include <cmath>
#include <cstdint>
#include <cstring>
#include <limits>
#include <vector>

#define REF_API extern "C" __attribute__((visibility("default")))

namespace {

inline float bf16_round(float x) {
  std::uint32_t u;
  std::memcpy(&u, &x, 4);
  if ((u & 0x7f800000u) == 0x7f800000u) return x;  // inf / nan stay
  u += 0x7fffu + ((u >> 16) & 1u);
  u &= 0xffff0000u;
  float y;
  std::memcpy(&y, &u, 4);
  return y;
}

inline std::uint32_t mix32(std::uint32_t x) {
  x ^= x >> 16;
  x *= 0x7FEB352Du;
  x ^= x >> 15;
  x *= 0x846CA68Bu;
  x ^= x >> 16;
  return x;
}

}  // namespace

// out[n, :] = table[ids[n], :]   (embed_lookup_f32, src/kernels.cpp:59-66)
REF_API void ref_embed(const float* table, const int* ids, float* out, int n_rows, int dim) {
  for (int n = 0; n < n_rows; ++n) std::memcpy(out + (size_t)n * dim, table + (size_t)ids[n] * dim, sizeof(float) * dim);
}

// x = h[r] + sum_p delta[p][r] (parts added in index order; delta may be null); h[r] = x if write_back;
// out[r, i] = (w[i] * x[i]) * inv, inv = 1 / sqrt(sum(x^2) / dim + eps)   (rmsnorm_f32, src/kernels.cpp:18-24)
REF_API void ref_rmsnorm(float* h, const float* delta, int n_parts, long long part_stride, const float* w, float* out,
                         int n_rows, int dim, float eps, int write_back, int round_bf16) {
  std::vector<float> x(dim);
  for (int r = 0; r < n_rows; ++r) {
    float ss = 0.f;
    for (int i = 0; i < dim; ++i) {
      float v = h[(size_t)r * dim + i];
      for (int p = 0; delta && p < n_parts; ++p) v += delta[(size_t)p * part_stride + (size_t)r * dim + i];
      if (delta && write_back) h[(size_t)r * dim + i] = v;
      x[i] = v;
      ss += v * v;
    }
    const float inv = 1.0f / std::sqrt(ss / (float)dim + eps);
    for (int i = 0; i < dim; ++i) {
      const float y = (w[i] * x[i]) * inv;
      out[(size_t)r * dim + i] = round_bf16 ? bf16_round(y) : y;
    }
  }
}

// out[m, n] = sum_k a[m, k] * w[n, k], k ascending, float32 sum   (matmul_f32, src/kernels.cpp:33-57)
REF_API void ref_gemm(const float* a, const float* w, float* out, int M, int N, int K) {
  for (int m = 0; m < M; ++m)
    for (int n = 0; n < N; ++n) {
      float acc = 0.f;
      for (int k = 0; k < K; ++k) acc += a[(size_t)m * K + k] * w[(size_t)n * K + k];
      out[(size_t)m * N + n] = acc;
    }
}

// out = silu(gate) * up, silu(v) = v / (1 + exp(-v))   (silu_f32, src/kernels.cpp:26-31; the product with
// `up` is a multiply of its own, src/engine.cpp:388-389)
REF_API void ref_silu_mul(const float* gate, const float* up, float* out, long long n) {
  for (long long i = 0; i < n; ++i) {
    const float g = gate[i];
    out[i] = (g / (1.0f + std::exp(-g))) * up[i];
  }
}

// Inverse frequencies in float64 with the Llama-3 wavelength bands, rounded to float32
// (llama3_inv_freq, src/kernels.cpp:114-160; pi is the float constant of src/kernels.cpp:110-112), then
// cos/sin of double(p) * double(inv_freq_f32), rounded to float32: tables [max_pos, head_dim / 2]
// (build_rope_tables, src/kernels.cpp:162-187, which stores each half twice).
REF_API void ref_rope_tables(int head_dim, float theta, int has_scaling, float factor, float low_f, float high_f, int orig_max_pos,
                             int max_pos, float* cos_t, float* sin_t) {
  const int half = head_dim / 2;
  const double pi_f = (double)3.14159265358979323846f;
  std::vector<float> inv(half);
  for (int i = 0; i < half; ++i) {
    double fr = 1.0 / std::pow((double)theta, (double)(2 * i) / (double)head_dim);
    if (has_scaling) {
      const double low_wl = (double)orig_max_pos / (double)low_f, high_wl = (double)orig_max_pos / (double)high_f;
      const double wl = 2.0 * pi_f / fr;
      if (wl > low_wl) fr = fr / (double)factor;
      else if (wl >= high_wl) {
        const double smooth = ((double)orig_max_pos / wl - (double)low_f) / ((double)high_f - (double)low_f);
        fr = (1.0 - smooth) * fr / (double)factor + smooth * fr;
      }
    }
    inv[i] = (float)fr;
  }
  for (int p = 0; p < max_pos; ++p)
    for (int i = 0; i < half; ++i) {
      const double ang = (double)p * (double)inv[i];
      cos_t[(size_t)p * half + i] = (float)std::cos(ang);
      sin_t[(size_t)p * half + i] = (float)std::sin(ang);
    }
}

// Rotation of q and k heads of every token by its position's row of the tables, half-split form
// (apply_rope_inplace, src/kernels.cpp:189-203), and the write of k (rotated) and v (raw) into the
// paged cache [pages, nkv, page_size, hd] (src/engine.cpp:343-353). qkv: [n, (nq + 2 nkv) * hd].
REF_API void ref_rope_kv_write(float* qkv, const int* positions, const int* token_seq, const int* block_table, int max_blocks,
                               const float* cos_t, const float* sin_t, float* kcache, float* vcache, int n_tokens, int nq, int nkv,
                               int hd, int page_size, int round_bf16) {
  const int half = hd / 2, width = (nq + 2 * nkv) * hd;
  for (int t = 0; t < n_tokens; ++t) {
    float* row = qkv + (size_t)t * width;
    const int pos = positions[t];
    for (int h = 0; h < nq + nkv; ++h)
      for (int i = 0; i < half; ++i) {
        const float a = row[h * hd + i], b = row[h * hd + i + half];
        float ra = a, rb = b;
        if (cos_t) {
          const float c = cos_t[(size_t)pos * half + i], s = sin_t[(size_t)pos * half + i];
          ra = a * c - b * s;
          rb = b * c + a * s;
        }
        row[h * hd + i] = round_bf16 ? bf16_round(ra) : ra;
        row[h * hd + i + half] = round_bf16 ? bf16_round(rb) : rb;
      }
    if (!kcache) continue;
    const int page = block_table[(size_t)token_seq[t] * max_blocks + pos / page_size];
    for (int kh = 0; kh < nkv; ++kh) {
      const size_t at = (((size_t)page * nkv + kh) * page_size + pos % page_size) * hd;
      std::memcpy(kcache + at, row + (size_t)(nq + kh) * hd, sizeof(float) * hd);
      std::memcpy(vcache + at, row + (size_t)(nq + nkv + kh) * hd, sizeof(float) * hd);
    }
  }
}

// Causal grouped-query attention of every token over cache positions lo..pos of its request:
// kv head = q head / (nq / nkv); score = (q . k) * scale, scale applied after the dot; p = exp(s - max);
// p *= 1 / sum; out = sum p * v, keys in index order   (attention_f32, src/kernels.cpp:413-474; the causal
// range from src/engine.cpp:358-362). window > 0: only the last `window` keys.
REF_API void ref_paged_attention(const float* q, long long ld_q, const float* kcache, const float* vcache, const int* positions,
                                 const int* token_seq, const int* block_table, int max_blocks, float* out, long long ld_out,
                                 int n_tokens, int nq, int nkv, int hd, int page_size, float scale, int window) {
  const int g = nq / nkv;
  std::vector<float> s;
  for (int t = 0; t < n_tokens; ++t) {
    const int pos = positions[t], lo = window > 0 ? std::max(0, pos - window + 1) : 0, n_keys = pos - lo + 1;
    const int* table = block_table + (size_t)token_seq[t] * max_blocks;
    s.assign(n_keys, 0.f);
    for (int h = 0; h < nq; ++h) {
      const float* qh = q + (size_t)t * ld_q + (size_t)h * hd;
      const int kh = h / g;
      float mx = -std::numeric_limits<float>::infinity();
      for (int j = 0; j < n_keys; ++j) {
        const int p = lo + j;
        const float* k = kcache + (((size_t)table[p / page_size] * nkv + kh) * page_size + p % page_size) * hd;
        float dot = 0.f;
        for (int d = 0; d < hd; ++d) dot += qh[d] * k[d];
        s[j] = dot * scale;
        mx = std::max(mx, s[j]);
      }
      float sum = 0.f;
      for (int j = 0; j < n_keys; ++j) {
        s[j] = std::exp(s[j] - mx);
        sum += s[j];
      }
      const float inv = 1.0f / sum;
      float* o = out + (size_t)t * ld_out + (size_t)h * hd;
      for (int d = 0; d < hd; ++d) o[d] = 0.f;
      for (int j = 0; j < n_keys; ++j) {
        const int p = lo + j;
        const float* v = vcache + (((size_t)table[p / page_size] * nkv + kh) * page_size + p % page_size) * hd;
        const float pj = s[j] * inv;
        for (int d = 0; d < hd; ++d) o[d] += pj * v[d];
      }
    }
  }
}

// Token choice: greedy = first index of the maximum (argmax with strict '>', src/engine.cpp:52-58).
// temperature > 0 (no counterpart in the reference): argmax_i(logit_i / T + g_i), g_i = -log(-log(u_i)),
// u_i from the integer hash of (seed, draw, i) that the kernel uses.
REF_API void ref_sample(const float* logits, long long ld, const float* temperature, const int* seeds, const int* draws, int* out,
                        int n_rows, int vocab) {
  for (int r = 0; r < n_rows; ++r) {
    const float* lr = logits + (size_t)r * ld;
    const float temp = temperature ? temperature[r] : 0.f;
    float bv = -std::numeric_limits<float>::infinity();
    int bi = 0;
    std::uint32_t k = 0;
    const float inv_t = temp > 0.f ? 1.0f / temp : 0.f;
    if (temp > 0.f) {
      k = mix32((std::uint32_t)seeds[r] ^ 0x9E3779B9u);
      k = mix32(k + (std::uint32_t)draws[r]);
    }
    for (int i = 0; i < vocab; ++i) {
      float z = lr[i];
      if (temp > 0.f) {
        const std::uint32_t h = mix32(k ^ ((std::uint32_t)i * 0x85EBCA6Bu));
        const float u = ((float)(h >> 9) + 0.5f) * (1.0f / 8388608.0f);
        z = lr[i] * inv_t + (-std::log(-std::log(u)));
      }
      if (z > bv) {
        bv = z;
        bi = i;
      }
    }
    out[r] = bi;
  }
}
