// Causal grouped-query attention over the paged cache on tensor cores (bfloat16 operands, float32
// scores, statistics and accumulators), for prompt portions and decoded tokens alike.
//
// A CTA owns one (request of the batch, key/value head, tile of query tokens): its 64 rows are the
// (token, query head of the group) pairs that share that key/value head, so the group's heads
// reuse every key and value tile that is fetched (a decoded token fills `group` rows, a prompt
// portion 64/group tokens). Keys are walked in tiles of 64 aligned to absolute positions, fetched
// page by page through the block table with cp.async into double-buffered shared memory; scores and
// the running (max, sum) softmax live in registers; each row is masked by its own token's position
// (and window), so the result for a token does not depend on what else is in the step.
// For decoding, the key range is also cut into splits of a fixed number of keys (absolute
// boundaries); every split writes a normalised partial output with its (max, sum) and a second
// kernel merges the splits in index order.
//
// Formula: the reference's attention_f32 (src/kernels.cpp:413-474): kv head = q head / group,
// score = (q . k) * scale applied after the dot, softmax, weighted sum of values.
#include "common.cuh"
#include "mma_common.cuh"

#include <cmath>

namespace {

constexpr int M_TILE = 64, N_TILE = 64, THREADS = 128;

struct AttnParams {
  const bf16* q; long long ld_q;
  const bf16* kcache; const bf16* vcache;
  const int* seq_start; const int* seq_ntok; const int* seq_qoff; const int* block_table;
  int max_blocks, nq, nkv, page_size, window;
  float scale;
  bf16* out; long long ld_out;
  // split mode (decode): partial outputs [split][token][head][HD] and (max, sum) [split][token][head][2]
  float* part_o; float* part_ml; int split_keys, n_splits; long long part_stride_tokens;
};

template <int HD, bool SPLIT>
__global__ void __launch_bounds__(THREADS) paged_attention_mma_kernel(const AttnParams p) {
  constexpr int LD = HD + 8;  // padded row (elements): 16-byte shifts keep ldmatrix free of bank conflicts
  constexpr int KSTEPS = HD / 16, DTILES = HD / 8;
  extern __shared__ __align__(16) uint8_t smem_raw[];
  bf16* q_s = reinterpret_cast<bf16*>(smem_raw);     // [M_TILE][LD]
  bf16* k_s = q_s + M_TILE * LD;                     // [2][N_TILE][LD]
  bf16* v_s = k_s + 2 * N_TILE * LD;                 // [2][N_TILE][LD]

  dep_launch();
  dep_wait();
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int seq = blockIdx.y;
  const int g = p.nq / p.nkv;
  const int tq_cap = M_TILE / g;  // query tokens per tile
  const int kvh = blockIdx.z % p.nkv;
  const int split = blockIdx.z / p.nkv;
  const int ntok = p.seq_ntok[seq];
  const int q0 = blockIdx.x * tq_cap;
  if (q0 >= ntok) return;
  const int n_tq = min(tq_cap, ntok - q0);
  const int n_rows = n_tq * g;
  const int tok_base = p.seq_qoff[seq] + q0;
  const int pos0 = p.seq_start[seq] + q0;      // position of the tile's first token
  const int pos_last = pos0 + n_tq - 1;
  int lo = (p.window > 0) ? max(0, pos0 - p.window + 1) : 0;  // oldest key any row reads
  int hi = pos_last;                                          // newest key any row reads
  if (SPLIT) {
    lo = max(lo, split * p.split_keys);
    hi = min(hi, (split + 1) * p.split_keys - 1);
  }
  const int* table = p.block_table + (size_t)seq * p.max_blocks;
  const size_t head_stride = (size_t)p.page_size * HD;

  // ---- Q tile -> shared memory (rows beyond n_rows are zeros)
  for (int c = tid; c < M_TILE * (HD / 8); c += THREADS) {
    const int r = c / (HD / 8), ch = c % (HD / 8);
    uint4 val = make_uint4(0, 0, 0, 0);
    if (r < n_rows) {
      const int tq = r / g, hg = r % g;
      val = *reinterpret_cast<const uint4*>(p.q + (size_t)(tok_base + tq) * p.ld_q + (size_t)(kvh * g + hg) * HD + ch * 8);
    }
    *reinterpret_cast<uint4*>(q_s + r * LD + ch * 8) = val;
  }

  auto load_tile = [&](int kt, int buf) {
    bf16* kd = k_s + buf * N_TILE * LD;
    bf16* vd = v_s + buf * N_TILE * LD;
    for (int c = tid; c < N_TILE * (HD / 8); c += THREADS) {
      const int r = c / (HD / 8), ch = c % (HD / 8);
      const int key = kt * N_TILE + r;
      const bool valid = key >= lo && key <= hi;
      size_t off = 0;
      if (valid) {
        const int page = table[key / p.page_size];
        off = ((size_t)page * p.nkv + kvh) * head_stride + (size_t)(key % p.page_size) * HD + ch * 8;
      }
      cp_async16(kd + r * LD + ch * 8, p.kcache + off, valid);
      cp_async16(vd + r * LD + ch * 8, p.vcache + off, valid);
    }
  };

  const int kt_first = lo / N_TILE, kt_last = hi / N_TILE;
  const bool any = hi >= lo;
  if (any) load_tile(kt_first, 0);
  cp_async_commit();
  __syncthreads();  // Q tile visible

  // ---- this warp's 16 rows: A fragments of Q, per-row positions
  uint32_t qa[KSTEPS][4];
#pragma unroll
  for (int ks = 0; ks < KSTEPS; ++ks) ldmatrix_x4(qa[ks], q_s + (warp * 16 + (lane % 16)) * LD + ks * 16 + (lane / 16) * 8);
  const int row_a = warp * 16 + lane / 4, row_b = row_a + 8;  // the two rows this thread holds
  const int pos_a = (row_a < n_rows) ? pos0 + row_a / g : -1;  // -1: padding row, sees no key
  const int pos_b = (row_b < n_rows) ? pos0 + row_b / g : -1;
  const int lo_a = (p.window > 0) ? pos_a - p.window + 1 : 0, lo_b = (p.window > 0) ? pos_b - p.window + 1 : 0;

  float o_acc[DTILES][4];
#pragma unroll
  for (int d = 0; d < DTILES; ++d) o_acc[d][0] = o_acc[d][1] = o_acc[d][2] = o_acc[d][3] = 0.f;
  float m_a = -INFINITY, m_b = -INFINITY, l_a = 0.f, l_b = 0.f;
  const float sl2 = p.scale * 1.4426950408889634f;  // scores are kept in units of log2(e)

  if (any) {
    for (int kt = kt_first; kt <= kt_last; ++kt) {
      const int buf = (kt - kt_first) & 1;
      if (kt < kt_last) load_tile(kt + 1, buf ^ 1);
      cp_async_commit();
      cp_async_wait<1>();
      __syncthreads();
      const bf16* kb = k_s + buf * N_TILE * LD;
      const bf16* vb = v_s + buf * N_TILE * LD;
      if (warp * 16 < n_rows) {  // a warp whose rows are all padding only helps with the copies

      // S = Q K^T : 16 rows x 64 keys per warp
      float s[N_TILE / 8][4];
#pragma unroll
      for (int j = 0; j < N_TILE / 8; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
#pragma unroll
      for (int ks = 0; ks < KSTEPS; ++ks) {
#pragma unroll
        for (int j2 = 0; j2 < N_TILE / 16; ++j2) {
          uint32_t b[4];
          ldmatrix_x4(b, kb + (j2 * 16 + (lane % 8) + (lane / 16) * 8) * LD + ks * 16 + ((lane / 8) % 2) * 8);
          mma_bf16(s[2 * j2], qa[ks], b[0], b[1]);
          mma_bf16(s[2 * j2 + 1], qa[ks], b[2], b[3]);
        }
      }
      // mask and running softmax (float32)
      const int key0 = kt * N_TILE + 2 * (lane % 4);
      float mx_a = -INFINITY, mx_b = -INFINITY;
#pragma unroll
      for (int j = 0; j < N_TILE / 8; ++j) {
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int key = key0 + j * 8 + e;
          const bool in_split = !SPLIT || (key >= lo && key <= hi);
          const bool va = in_split && key <= pos_a && key >= lo_a;
          const bool vb2 = in_split && key <= pos_b && key >= lo_b;
          s[j][e] = va ? s[j][e] * sl2 : -INFINITY;
          s[j][2 + e] = vb2 ? s[j][2 + e] * sl2 : -INFINITY;
          mx_a = fmaxf(mx_a, s[j][e]);
          mx_b = fmaxf(mx_b, s[j][2 + e]);
        }
      }
      mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 1));
      mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 2));
      mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 1));
      mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 2));
      const float mn_a = fmaxf(m_a, mx_a), mn_b = fmaxf(m_b, mx_b);
      const float base_a = (mn_a == -INFINITY) ? 0.f : mn_a, base_b = (mn_b == -INFINITY) ? 0.f : mn_b;
      const float al_a = exp2f(m_a - base_a), al_b = exp2f(m_b - base_b);  // exp2(-inf) = 0 on the first tile
      float sum_a = 0.f, sum_b = 0.f;
#pragma unroll
      for (int j = 0; j < N_TILE / 8; ++j) {
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          s[j][e] = exp2f(s[j][e] - base_a);
          s[j][2 + e] = exp2f(s[j][2 + e] - base_b);
          sum_a += s[j][e];
          sum_b += s[j][2 + e];
        }
      }
      sum_a += __shfl_xor_sync(0xffffffffu, sum_a, 1);
      sum_a += __shfl_xor_sync(0xffffffffu, sum_a, 2);
      sum_b += __shfl_xor_sync(0xffffffffu, sum_b, 1);
      sum_b += __shfl_xor_sync(0xffffffffu, sum_b, 2);
      l_a = l_a * al_a + sum_a;
      l_b = l_b * al_b + sum_b;
      m_a = mn_a;
      m_b = mn_b;
#pragma unroll
      for (int d = 0; d < DTILES; ++d) {
        o_acc[d][0] *= al_a; o_acc[d][1] *= al_a;
        o_acc[d][2] *= al_b; o_acc[d][3] *= al_b;
      }
      // O += P V : P (16 x 64, bf16 from the score registers) times V (64 keys x HD)
#pragma unroll
      for (int kk = 0; kk < N_TILE / 16; ++kk) {
        uint32_t pa[4];
        pa[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
        pa[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
        pa[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
        pa[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
        for (int d2 = 0; d2 < DTILES / 2; ++d2) {
          uint32_t b[4];
          ldmatrix_x4_trans(b, vb + (kk * 16 + (lane % 8) + ((lane / 8) % 2) * 8) * LD + d2 * 16 + (lane / 16) * 8);
          mma_bf16(o_acc[2 * d2], pa, b[0], b[1]);
          mma_bf16(o_acc[2 * d2 + 1], pa, b[2], b[3]);
        }
      }
      }
      __syncthreads();  // everyone is done with this buffer before it is filled again
    }
  }
  cp_async_wait<0>();

  // ---- write: rows a and b of this thread, columns 2*(lane%4)+{0,1} of every 8-wide tile
  const float inv_a = l_a > 0.f ? 1.f / l_a : 0.f, inv_b = l_b > 0.f ? 1.f / l_b : 0.f;
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const int row = half ? row_b : row_a;
    if (row >= n_rows) continue;
    const int tq = row / g, hg = row % g;
    const float inv = half ? inv_b : inv_a;
    if (!SPLIT) {
      bf16* dst = p.out + (size_t)(tok_base + tq) * p.ld_out + (size_t)(kvh * g + hg) * HD + 2 * (lane % 4);
#pragma unroll
      for (int d = 0; d < DTILES; ++d)
        *reinterpret_cast<uint32_t*>(dst + d * 8) = pack_bf16(o_acc[d][2 * half] * inv, o_acc[d][2 * half + 1] * inv);
    } else {
      const size_t slot = ((size_t)split * p.part_stride_tokens + (tok_base + tq)) * p.nq + (kvh * g + hg);
      float* dst = p.part_o + slot * HD + 2 * (lane % 4);
#pragma unroll
      for (int d = 0; d < DTILES; ++d) {
        dst[d * 8] = o_acc[d][2 * half] * inv;
        dst[d * 8 + 1] = o_acc[d][2 * half + 1] * inv;
      }
      if ((lane % 4) == 0) {
        p.part_ml[slot * 2] = half ? m_b : m_a;  // log2 units; -inf when this split saw no key of the row
        p.part_ml[slot * 2 + 1] = half ? l_b : l_a;
      }
    }
  }
}

// Merges the splits of every (token, head) in index order: out = sum_s w_s o_s / sum_s w_s,
// w_s = l_s * 2^(m_s - max m).
template <int HD>
__global__ void attention_combine_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml, int n_splits,
                                         long long part_stride_tokens, int nq, bf16* __restrict__ out, long long ld_out,
                                         int n_tokens) {
  dep_launch();
  dep_wait();
  const int item = blockIdx.x * (blockDim.x / 32) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (item >= n_tokens * nq) return;
  const int tok = item / nq, head = item % nq;
  const size_t split_stride = (size_t)part_stride_tokens * nq;  // slots from one split to the next
  const size_t slot0 = (size_t)tok * nq + head;
  float mx = -INFINITY;
  for (int s = lane; s < n_splits; s += 32) mx = fmaxf(mx, part_ml[(slot0 + s * split_stride) * 2]);
  mx = warp_max(mx);
  constexpr int R = (HD + 31) / 32;
  float acc[R];
#pragma unroll
  for (int i = 0; i < R; ++i) acc[i] = 0.f;
  float den = 0.f;
  for (int s0 = 0; s0 < n_splits; s0 += 4) {  // four splits' loads in flight; added in index order
    float w[4], v[4][R];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int s = s0 + u;
      w[u] = 0.f;
      if (s < n_splits) {
        const size_t slot = slot0 + s * split_stride;
        const float m = part_ml[slot * 2], l = part_ml[slot * 2 + 1];
        w[u] = (m == -INFINITY) ? 0.f : l * exp2f(m - mx);  // -inf: the split held no key of the row
#pragma unroll
        for (int i = 0; i < R; ++i) {
          const int d = lane + 32 * i;
          v[u][i] = (d < HD && w[u] != 0.f) ? part_o[slot * HD + d] : 0.f;
        }
      }
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      if (s0 + u < n_splits && w[u] != 0.f) {
        den += w[u];
#pragma unroll
        for (int i = 0; i < R; ++i) acc[i] = fmaf(w[u], v[u][i], acc[i]);
      }
    }
  }
  const float inv = den > 0.f ? 1.f / den : 0.f;
#pragma unroll
  for (int i = 0; i < R; ++i) {
    const int d = lane + 32 * i;
    if (d < HD) out[(size_t)tok * ld_out + (size_t)head * HD + d] = __float2bfloat16_rn(acc[i] * inv);
  }
}

template <int HD>
int launch(const AttnParams& p, int n_seqs, int max_new_tokens, int n_tokens, bool split, cudaStream_t stream) {
  constexpr int LD = HD + 8;
  const int g = p.nq / p.nkv;
  auto set_attr = [&](auto kernel, size_t smem) {
    if (smem > 48 * 1024) return cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) == cudaSuccess;
    return true;
  };
  const size_t smem = (size_t)(M_TILE + 4 * N_TILE) * LD * sizeof(bf16);
  const int tq_cap = M_TILE / g;
  dim3 grid((max_new_tokens + tq_cap - 1) / tq_cap, n_seqs, p.nkv * (split ? p.n_splits : 1));
  if (split) {
    if (!set_attr(paged_attention_mma_kernel<HD, true>, smem)) return 1;
    launch_kernel(paged_attention_mma_kernel<HD, true>, grid, THREADS, smem, stream, p);
    const int items = n_tokens * p.nq;
    launch_kernel(attention_combine_kernel<HD>, (items + 3) / 4, 128, 0, stream, (const float*)p.part_o, (const float*)p.part_ml,
                  p.n_splits, p.part_stride_tokens, p.nq, p.out, p.ld_out, n_tokens);
  } else {
    if (!set_attr(paged_attention_mma_kernel<HD, false>, smem)) return 1;
    launch_kernel(paged_attention_mma_kernel<HD, false>, grid, THREADS, smem, stream, p);
  }
  return 0;
}

}  // namespace

// Whether the tensor-core attention takes this geometry (else the caller uses the CUDA-core kernel).
extern "C" int llm_attention_mma_supported(int nq, int nkv, int hd, long long ld_q, long long ld_out) {
  if (nkv <= 0 || nq % nkv) return 0;
  const int g = nq / nkv;
  return (hd == 16 || hd == 32 || hd == 64 || hd == 128) && g <= M_TILE && (ld_q % 8) == 0 && (ld_out % 2) == 0;
}

// Floats of scratch that the split form needs: partial outputs and (max, sum) pairs.
extern "C" long long llm_attention_mma_scratch_floats(int n_tokens, int nq, int hd, int n_splits) {
  return (long long)n_splits * n_tokens * nq * (hd + 2);
}

// q: rows of [nq*hd] bf16 (ld_q elements apart); caches [pages, nkv, page_size, hd] bf16;
// seq_* and block_table as in the step's batch; out [n_tokens, nq*hd] bf16.
// n_splits > 1: keys are cut every split_keys (a multiple of 64) positions; every split writes a
// partial into scratch (llm_attention_mma_scratch_floats floats) and a second kernel merges them.
// max_new_tokens: longest portion of the batch.
extern "C" int llm_paged_attention_mma(const void* q, long long ld_q, const void* kcache, const void* vcache, const int* seq_start,
                                       const int* seq_ntok, const int* seq_qoff, const int* block_table, int max_blocks, void* out,
                                       long long ld_out, int n_seqs, int n_tokens, int max_new_tokens, int nq, int nkv, int hd,
                                       int page_size, float scale, int window, int n_splits, int split_keys, float* scratch,
                                       cudaStream_t stream) {
  if (n_tokens == 0 || n_seqs == 0) return LLM_OK;
  LLM_REQUIRE(llm_attention_mma_supported(nq, nkv, hd, ld_q, ld_out), "attention_mma: geometry not supported (nq=%d nkv=%d hd=%d)", nq, nkv, hd);
  LLM_REQUIRE(page_size > 0 && max_blocks > 0 && window >= 0 && max_new_tokens > 0, "attention_mma: bad sizes");
  LLM_REQUIRE((reinterpret_cast<uintptr_t>(q) & 15u) == 0 && (reinterpret_cast<uintptr_t>(kcache) & 15u) == 0 &&
              (reinterpret_cast<uintptr_t>(vcache) & 15u) == 0, "attention_mma: q and the caches must be 16-byte aligned");
  LLM_REQUIRE(n_splits >= 1 && (n_splits == 1 || (split_keys > 0 && split_keys % N_TILE == 0 && scratch != nullptr)),
              "attention_mma: splits need split_keys %% 64 == 0 and scratch");
  LLM_REQUIRE((long long)n_seqs <= 65535 && (long long)nkv * n_splits <= 65535, "attention_mma: batch too large for the grid");
  AttnParams p;
  p.q = (const bf16*)q; p.ld_q = ld_q; p.kcache = (const bf16*)kcache; p.vcache = (const bf16*)vcache;
  p.seq_start = seq_start; p.seq_ntok = seq_ntok; p.seq_qoff = seq_qoff; p.block_table = block_table;
  p.max_blocks = max_blocks; p.nq = nq; p.nkv = nkv; p.page_size = page_size; p.window = window; p.scale = scale;
  p.out = (bf16*)out; p.ld_out = ld_out;
  p.n_splits = n_splits; p.split_keys = split_keys; p.part_stride_tokens = n_tokens;
  p.part_o = scratch; p.part_ml = scratch ? scratch + (size_t)n_splits * n_tokens * nq * hd : nullptr;
  const bool split = n_splits > 1;
  int rc = 0;
  if (hd == 16) rc = launch<16>(p, n_seqs, max_new_tokens, n_tokens, split, stream);
  else if (hd == 32) rc = launch<32>(p, n_seqs, max_new_tokens, n_tokens, split, stream);
  else if (hd == 64) rc = launch<64>(p, n_seqs, max_new_tokens, n_tokens, split, stream);
  else rc = launch<128>(p, n_seqs, max_new_tokens, n_tokens, split, stream);
  LLM_REQUIRE(rc == 0, "attention_mma: cannot raise the shared memory limit");
  LLM_CHECK_LAUNCH("paged_attention_mma");
  return LLM_OK;
}
