// Causal grouped-query attention of prompt portions on the 5th-generation tensor cores.
//
// A CTA owns 128 rows = (query token, query head of the group) pairs that share one key/value
// head, i.e. 128/group tokens of one request, and walks the request's cached keys in tiles of KEYS
// (absolute positions; 128 keys at head size 64, 64 keys at head size 128, so that two CTAs fit an
// SM either way), fetched page by page with TMA through the block table:
//
//   S = Q K^T        tcgen05.mma, Q and K in shared memory (128-byte swizzle), S in tensor memory
//   softmax          thread t owns row t: it reads its 128 scores from tensor memory, masks them by
//                    its own token's position (and window), keeps the running max and sum in
//                    float32 and writes P = exp2(S - max) as bfloat16 back to tensor memory
//   O += P V         tcgen05.mma with P read from tensor memory and V from shared memory (V is
//                    [key][dim], i.e. the "MN-major" operand form); O stays in tensor memory and is
//                    rescaled by the owner of each row when its max moves
//
// Warps 0-3 are the softmax threads; one thread of a fifth warp issues the TMA loads and the MMAs
// and runs ahead of them: the scores of tile i + 1 are queued as soon as the softmax threads have
// READ the scores of tile i (not when they have finished with them), so they are waiting when the
// softmax of tile i ends, and P V of tile i runs under the softmax of tile i + 1. Keys and values
// have their own stage barriers: a key stage is free once its scores are done, long before the
// value stage, so the next keys are requested a whole softmax earlier. Two CTAs per SM fill each
// other's gaps. Every
// wait on an mbarrier is bounded (see tc_common.cuh). head_dim 64 or 128 (rows of 128 dims are two
// 64-dim blocks of 128-byte swizzled rows: Q K^T runs over both, P V is one product per block),
// page sizes that are multiples of 8 and divide the tile, groups of up to 128 heads (a CTA takes
// floor(128 / group) tokens; rows beyond them are padding); the caller uses the mma.sync kernel otherwise.
//
// Formula: the reference's attention_f32 (src/kernels.cpp:413-474): kv head = q head / group,
// score = (q . k) * scale applied after the dot, softmax in float32, weighted sum of values.
#include "tc_common.cuh"

#include <cmath>

namespace {

constexpr int ROWS = 128;
constexpr int TMEM_COLS_ATT = 256;
enum : int { ERR_ATT_KV = 11, ERR_ATT_S = 12, ERR_ATT_O = 13 };

template <int HD_>
struct AttLayout {
  static constexpr int HD = HD_;
  static constexpr int KEYS = HD == 64 ? 128 : 64;   // keys per tile
  static constexpr int DBLK = HD / 64;               // 64-dim blocks of a row
  static constexpr int Q_BYTES = ROWS * HD * 2, KV_BYTES = KEYS * HD * 2;  // KV_BYTES: one of K or V of a tile
  static constexpr int S_COL = 0, P_COL = KEYS, O_COL = KEYS + KEYS / 2;   // tensor-memory columns: S f32, P bf16 pairs, O f32
  static_assert(O_COL + HD <= TMEM_COLS_ATT, "the accumulators do not fit the allocation");
};

struct AttnTcParams {
  const bf16* q; long long ld_q;
  const int* seq_start; const int* seq_ntok; const int* seq_qoff; const int* block_table;
  int max_blocks, nq, nkv, page_size, window, null_page;
  float scale;
  bf16* out; long long ld_out;
  int* error_out;
};

__device__ __forceinline__ void tmem_load32(uint32_t taddr, float* v) {
  uint32_t r[32];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, "
      "%18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
        "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]),
        "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
        "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
#pragma unroll
  for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}
// The registers of tmem_load32 calls may be read only after this.
__device__ __forceinline__ void tmem_load_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

__device__ __forceinline__ void tmem_store32(uint32_t taddr, const uint32_t* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, "
      "%18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]),
      "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]),
      "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]),
      "r"(r[31])
      : "memory");
}

// Largest of three, one instruction.
__device__ __forceinline__ float max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}

// 2^x on the special-function unit, one instruction (exp2f adds range handling that is not needed here).
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Two float32 lanes in one 64-bit register pair, for the packed instructions of sm_100 (fma.rn.f32x2,
// add.rn.f32x2: one issue slot for two results, each lane rounded as the scalar instruction rounds).
__device__ __forceinline__ uint64_t pack2(float a, float b) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(a), "f"(b));
  return r;
}
__device__ __forceinline__ void unpack2(uint64_t v, float& a, float& b) { asm("mov.b64 {%0, %1}, %2;" : "=f"(a), "=f"(b) : "l"(v)); }
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
__device__ __forceinline__ uint64_t add2(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}

// The probabilities of a row's scores of one key tile: p[j] = 2^(s[j] * sl2 - base) as bfloat16 pairs,
// and their float32 sum (of the unrounded values; eight chains of additions joined in a fixed order).
// The multiply-adds and the additions run two lanes an instruction.
template <int KEYS>
__device__ __forceinline__ float exp_row(const float* s, float sl2, float base, uint32_t* packed) {
  const uint64_t sl2_2 = pack2(sl2, sl2), nbase2 = pack2(-base, -base);
  uint64_t sum2[4] = {0ull, 0ull, 0ull, 0ull};  // (0.f, 0.f) pairs
#pragma unroll
  for (int j = 0; j < KEYS; j += 2) {
    float x0, x1;
    unpack2(fma2(pack2(s[j], s[j + 1]), sl2_2, nbase2), x0, x1);
    const float p0 = fast_exp2(x0), p1 = fast_exp2(x1);
    sum2[(j / 2) & 3] = add2(sum2[(j / 2) & 3], pack2(p0, p1));
    __nv_bfloat162 t = __floats2bfloat162_rn(p0, p1);
    packed[j / 2] = *reinterpret_cast<uint32_t*>(&t);
  }
  float a0, a1;
  unpack2(add2(add2(sum2[0], sum2[1]), add2(sum2[2], sum2[3])), a0, a1);
  return a0 + a1;
}

// tcgen05.mma with the A operand in tensor memory.
__device__ __forceinline__ void mma_f16_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}" ::"r"(tmem_d),
      "r"(tmem_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}

// bf16 x bf16 -> f32, M = 128; b_mn_major: the B operand is stored with N contiguous ([k][n]).
__host__ __device__ constexpr uint32_t instr_desc_att(int n, bool b_mn_major) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((b_mn_major ? 1u : 0u) << 16) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
}

constexpr int ATT_THREADS = 160;  // warps 0-3: one softmax thread per row; warp 4: one thread issues TMA and MMA

template <int HD>
__global__ void __launch_bounds__(ATT_THREADS, 2)  // two CTAs per SM: at most 200 registers a thread
    paged_attention_tc_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v, const AttnTcParams p) {
  using L = AttLayout<HD>;
  constexpr int KEYS = L::KEYS, DBLK = L::DBLK, Q_BYTES = L::Q_BYTES, KV_BYTES = L::KV_BYTES;
  constexpr int S_COL = L::S_COL, P_COL = L::P_COL, O_COL = L::O_COL;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint8_t* q_s = smem;                  // [DBLK blocks][128 rows][128 B], 128-byte swizzle
  uint8_t* kv_s = smem + Q_BYTES;       // [2 stages][K | V], each [DBLK blocks][KEYS rows][128 B], 128-byte swizzle
  uint64_t* full_k = reinterpret_cast<uint64_t*>(kv_s + 4 * KV_BYTES);  // [2] the keys of a tile have landed
  uint64_t* full_v = full_k + 2;        // [2] the values of a tile have landed
  uint64_t* s_bar = full_v + 2;         // the scores of a tile are in tensor memory
  uint64_t* s_free = s_bar + 1;         // all 128 rows have read their scores: the S columns may be overwritten (an arrival a warp)
  uint64_t* p_bar = s_free + 1;         // all 128 rows of P are in tensor memory (an arrival a warp)
  uint64_t* o_bar = p_bar + 1;          // the P V product of a tile is done
  uint64_t* done_bar = o_bar + 1;       // every product that was issued has finished (committed last, also after giving up)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(done_bar + 2);  // (+1 spare word: the ints after it stay 16-byte aligned)
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  int* page_s = reinterpret_cast<int*>(tmem_slot + 4);  // the tile range's slice of the block table

  dep_launch();
  const int tid = threadIdx.x, warp = tid >> 5;
  const int seq = blockIdx.y, kvh = blockIdx.x;
  const int g = p.nq / p.nkv;
  const int tq_cap = ROWS / g;
  // the batch arrays came with the step's host-to-device copy: they may be read before the wait
  const int ntok = p.seq_ntok[seq];
  // Late query tiles see the most keys. CTAs start in the order x, y, z, so the query tile is the z
  // index, latest first: the long CTAs of every head and request run before any short one, and
  // the grid's tail is made of short CTAs.
  const int q0 = (int)(gridDim.z - 1 - blockIdx.z) * tq_cap;
  if (q0 >= ntok) return;
  const int n_tq = min(tq_cap, ntok - q0);
  const int n_rows = n_tq * g;
  const int tok_base = p.seq_qoff[seq] + q0;
  const int pos0 = p.seq_start[seq] + q0;
  const int pos_last = pos0 + n_tq - 1;
  const int lo = (p.window > 0) ? max(0, pos0 - p.window + 1) : 0;
  const int hi = pos_last;
  const int kt_first = lo / KEYS, kt_last = hi / KEYS;
  const int n_tiles = kt_last - kt_first + 1;
  const int* table = p.block_table + (size_t)seq * p.max_blocks;
  const int pages_per_tile = KEYS / p.page_size;

  if (tid == 0) {
    for (int b = 0; b < 2; ++b) {
      mbar_init(&full_k[b], 1);
      mbar_init(&full_v[b], 1);
    }
    mbar_init(s_bar, 1);
    mbar_init(s_free, ROWS / 32);  // one arrival a softmax warp
    mbar_init(p_bar, ROWS / 32);
    mbar_init(o_bar, 1);
    mbar_init(done_bar, 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(TMEM_COLS_ATT) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  // The pages of this CTA's key tiles, read once by all threads: the thread that issues the copies
  // would otherwise wait for a global read before every single one of them. Every tile is fetched
  // whole: pages that the request does not hold (beyond its newest key, or given back behind a
  // window) are read from the pool's null page, whose values are finite and meet probabilities of
  // exactly zero, so no stage has to be cleared and no copy depends on a fill convention.
  const int page_lo = (kt_first * KEYS) / p.page_size;
  {
    const int n_pages_all = (kt_last + 1) * pages_per_tile - page_lo;
    for (int i = tid; i < n_pages_all; i += ATT_THREADS) {
      const int idx = page_lo + i;
      const int page = (idx < p.max_blocks && idx * p.page_size <= hi) ? table[idx] : -1;
      page_s[i] = page >= 0 ? page : p.null_page;
    }
  }
  __syncthreads();
  auto issue_part = [&](int i, bool values) {  // keys or values of tile i -> stage i % 2
    const int first_page = (kt_first + i) * pages_per_tile - page_lo;
    uint8_t* dst = kv_s + (size_t)(i & 1) * 2 * KV_BYTES + (values ? KV_BYTES : 0);
    uint64_t* bar = values ? &full_v[i & 1] : &full_k[i & 1];
    const CUtensorMap* map = values ? &map_v : &map_k;
    mbar_expect_tx(bar, (uint32_t)KV_BYTES);
    for (int pg = 0; pg < pages_per_tile; ++pg) {
      const int row = (page_s[first_page + pg] * p.nkv + kvh) * p.page_size;
#pragma unroll
      for (int b = 0; b < DBLK; ++b) tma_load_2d(dst + b * (KEYS * 128) + (size_t)pg * p.page_size * 128, map, b * 64, row, bar);
    }
  };
  dep_wait();
  // the first two tiles are on their way while the query rows are fetched
  if (tid == 4 * 32) {
    issue_part(0, false);
    issue_part(0, true);
    if (n_tiles > 1) {
      issue_part(1, false);
      issue_part(1, true);
    }
  }
  // ---- Q rows -> shared memory in the swizzled K-major layout (16-byte chunk c of row r at c ^ (r % 8))
  if (tid < ROWS) {
    const int r = tid;
    uint4 vals[HD / 8];
    if (r < n_rows) {
      const int tq = r / g, hg = r % g;
      const uint4* src = reinterpret_cast<const uint4*>(p.q + (size_t)(tok_base + tq) * p.ld_q + (size_t)(kvh * g + hg) * HD);
#pragma unroll
      for (int c = 0; c < HD / 8; ++c) vals[c] = src[c];
    } else {
#pragma unroll
      for (int c = 0; c < HD / 8; ++c) vals[c] = make_uint4(0, 0, 0, 0);
    }
#pragma unroll
    for (int c = 0; c < HD / 8; ++c)
      *reinterpret_cast<uint4*>(q_s + (c / 8) * (ROWS * 128) + r * 128 + (((c % 8) ^ (r & 7)) << 4)) = vals[c];
  }
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // generic-proxy writes -> visible to TMA / MMA
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_slot;
  bool ok = true;

  if (warp == 4) {
    if (tid == 4 * 32) {
      // ------------------------------------------------------------ the thread that issues TMA and MMA
      auto issue_scores = [&](int i) {  // S = Q K^T of tile i
        constexpr uint32_t idesc_s = instr_desc_att(KEYS, false);
#pragma unroll
        for (int k = 0; k < HD / 16; ++k) {  // 16 dims a step: block k / 4, 32 bytes further along the swizzled row each step
          const uint64_t dq = smem_desc_sw128(smem_u32(q_s + (k / 4) * (ROWS * 128)));
          const uint64_t dk = smem_desc_sw128(smem_u32(kv_s + (size_t)(i & 1) * 2 * KV_BYTES + (k / 4) * (KEYS * 128)));
          mma_f16(tmem_base + S_COL, dq + (uint64_t)(2 * (k % 4)), dk + (uint64_t)(2 * (k % 4)), idesc_s, k > 0 ? 1u : 0u);
        }
        mma_commit(s_bar);
      };
      // what was requested and what has arrived, keys and values apart (for the drain after giving up)
      int k_issued = n_tiles > 1 ? 2 : 1, v_issued = k_issued, k_landed = 0, v_landed = 0;
      ok = mbar_wait(&full_k[0], 0, abort_flag, p.error_out, ERR_ATT_KV);
      if (ok) {
        k_landed = 1;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        issue_scores(0);
      }
      for (int i = 0; i < n_tiles && ok; ++i) {
        if (i + 1 < n_tiles) {
          // every row has READ the scores of tile i: the S columns are free, and so is the key stage
          // of tile i (its scores are done). Queue the next scores now, under the softmax of tile i.
          ok = mbar_wait(s_free, (uint32_t)i & 1u, abort_flag, p.error_out, ERR_ATT_S);
          if (!ok) break;
          if (i + 2 < n_tiles) {
            issue_part(i + 2, false);
            k_issued = i + 3;
          }
          ok = mbar_wait(&full_k[(i + 1) & 1], (uint32_t)((i + 1) >> 1) & 1u, abort_flag, p.error_out, ERR_ATT_KV);
          if (!ok) break;
          k_landed = i + 2;
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          issue_scores(i + 1);
        }
        // P of tile i is in tensor memory
        ok = mbar_wait(p_bar, (uint32_t)i & 1u, abort_flag, p.error_out, ERR_ATT_S);
        if (ok) ok = mbar_wait(&full_v[i & 1], (uint32_t)(i >> 1) & 1u, abort_flag, p.error_out, ERR_ATT_KV);
        if (!ok) break;
        v_landed = i + 1;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        constexpr uint32_t idesc_o = instr_desc_att(64, true);
#pragma unroll
        for (int b = 0; b < DBLK; ++b) {  // one product per 64-dim block of V: 64 columns of O each
          const uint64_t dv = smem_desc_sw128(smem_u32(kv_s + (size_t)(i & 1) * 2 * KV_BYTES + KV_BYTES + b * (KEYS * 128)));
#pragma unroll
          for (int k = 0; k < KEYS / 16; ++k)  // 16 keys = 16 rows of 128 B further down the V block; 8 columns further along P
            mma_f16_ts(tmem_base + O_COL + (uint32_t)(b * 64), tmem_base + P_COL + (uint32_t)(k * 8), dv + (uint64_t)(k * (16 * 128 >> 4)),
                       idesc_o, (i > 0 || k > 0) ? 1u : 0u);
        }
        mma_commit(o_bar);
        if (i + 2 < n_tiles) {  // the value stage of tile i is free once its product is done
          ok = mbar_wait(o_bar, (uint32_t)i & 1u, abort_flag, p.error_out, ERR_ATT_O);
          if (ok) {
            issue_part(i + 2, true);
            v_issued = i + 3;
          }
        }
      }
      mma_commit(done_bar);
      // gave up: the copies still on their way land (bounded) before the CTA gives its shared memory back
      for (int t = k_landed; !ok && t < k_issued; ++t) mbar_drain(&full_k[t & 1], (uint32_t)(t >> 1) & 1u, p.error_out);
      for (int t = v_landed; !ok && t < v_issued; ++t) mbar_drain(&full_v[t & 1], (uint32_t)(t >> 1) & 1u, p.error_out);
    }
  } else {
    // -------------------------------------------------------------- softmax: thread t owns row t
    const uint32_t lane_base = (uint32_t)(warp * 32) << 16;
    const int tq_row = tid / g;
    const int pos_r = (tid < n_rows) ? pos0 + tq_row : -1;  // -1: padding row, sees no key
    const int lo_r = (p.window > 0) ? pos_r - p.window + 1 : 0;
    const float sl2 = p.scale * 1.4426950408889634f;
    float m_run = -INFINITY, l_run = 0.f;
    for (int i = 0; i < n_tiles; ++i) {
      ok = mbar_wait(s_bar, (uint32_t)i & 1u, abort_flag, p.error_out, ERR_ATT_S);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      float s[KEYS];
#pragma unroll
      for (int c = 0; c < KEYS / 32; ++c) tmem_load32(tmem_base + lane_base + S_COL + c * 32, s + c * 32);
      tmem_load_wait();  // four loads in flight, one wait
      // the scores are in registers: the tensor cores may write the next tile's scores over them
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if ((tid & 31) == 0) mbar_arrive(s_free);  // the loads above are warp-wide: one arrival stands for the 32 rows
      const int key0 = (kt_first + i) * KEYS;
      const bool full_tile = (key0 + KEYS - 1 <= pos_r) && (key0 >= lo_r);
      // s stays unscaled: max(s * c) = c * max(s) for c > 0, and the scale folds into the exponent's
      // multiply-add below, which saves an instruction per score in a loop that is bound by issue slots
      float mx = -INFINITY;
      if (!full_tile) {
#pragma unroll
        for (int j = 0; j < KEYS; ++j) {
          const int key = key0 + j;
          s[j] = (key <= pos_r && key >= lo_r) ? s[j] : -INFINITY;
        }
      }
      {  // eight independent chains instead of one of KEYS dependent maxima, three inputs an instruction
        float m8[8];
#pragma unroll
        for (int c = 0; c < 8; ++c) m8[c] = max3(s[c], s[c + 8], s[c + 16]);
#pragma unroll
        for (int j = 24; j + 16 <= KEYS; j += 16) {
#pragma unroll
          for (int c = 0; c < 8; ++c) m8[c] = max3(m8[c], s[j + c], s[j + c + 8]);
        }
        static_assert((KEYS - 24) % 16 == 8, "the tail below takes the last eight scores");
#pragma unroll
        for (int c = 0; c < 8; ++c) m8[c] = fmaxf(m8[c], s[KEYS - 8 + c]);
        mx = fmaxf(max3(m8[0], m8[1], m8[2]), fmaxf(max3(m8[3], m8[4], m8[5]), fmaxf(m8[6], m8[7])));
      }
      mx *= sl2;  // (-inf stays -inf)
      // The running max is only moved when it would grow by more than 2^8: until then the row keeps
      // its older, smaller reference (probabilities up to 256 instead of 1, harmless in float32 and
      // bfloat16) and its sum and output need no rescaling. Sum and output always share one reference.
      const bool move = (mx > m_run + 8.0f) || (m_run == -INFINITY && mx > -INFINITY);
      const float m_new = move ? mx : m_run;
      const float base = (m_new == -INFINITY) ? 0.f : m_new;
      const float alpha = move ? fast_exp2(m_run - base) : 1.0f;  // 0 when the row had seen no key yet
      uint32_t packed[KEYS / 2];
      l_run = l_run * alpha + exp_row<KEYS>(s, sl2, base, packed);
      m_run = m_new;
      if (i > 0) {
        // The product P V of the tile before reads the P columns and adds into O: both are touched
        // below. It was queued when that tile's P was complete, a whole softmax ago, so this wait
        // is over before it starts in all but the shortest tiles.
        ok = mbar_wait(o_bar, (uint32_t)(i - 1) & 1u, abort_flag, p.error_out, ERR_ATT_O);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      }
#pragma unroll
      for (int c = 0; c < KEYS / 64; ++c) tmem_store32(tmem_base + lane_base + P_COL + c * 32, packed + c * 32);
      if (i > 0 && __any_sync(0xffffffffu, move)) {  // rescale the warp's rows of O (the product of the tile before is done)
#pragma unroll
        for (int c = 0; c < HD / 64; ++c) {  // 64 columns at a time keeps the registers within the two-CTA budget
          float o[64];
          tmem_load32(tmem_base + lane_base + O_COL + c * 64, o);
          tmem_load32(tmem_base + lane_base + O_COL + c * 64 + 32, o + 32);
          tmem_load_wait();
          uint32_t ou[64];
#pragma unroll
          for (int d = 0; d < 64; ++d) ou[d] = __float_as_uint(o[d] * alpha);
          tmem_store32(tmem_base + lane_base + O_COL + c * 64, ou);
          tmem_store32(tmem_base + lane_base + O_COL + c * 64 + 32, ou + 32);
        }
      }
      asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if ((tid & 31) == 0) mbar_arrive(p_bar);
    }
    // ---- the rows of O, normalised
    if (ok && n_tiles > 0) ok = mbar_wait(o_bar, (uint32_t)(n_tiles - 1) & 1u, abort_flag, p.error_out, ERR_ATT_O);
    ok = __all_sync(0xffffffffu, ok);
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    if (ok) {  // every thread of a warp takes part in the tensor-memory loads; only real rows are stored
      const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
      const int tq = tid / g, hg = tid % g;
      uint4* dst = reinterpret_cast<uint4*>(p.out + (size_t)(tok_base + tq) * p.ld_out + (size_t)(kvh * g + hg) * HD);
#pragma unroll
      for (int b = 0; b < HD / 64; ++b) {
        float o[64];
        tmem_load32(tmem_base + lane_base + O_COL + b * 64, o);
        tmem_load32(tmem_base + lane_base + O_COL + b * 64 + 32, o + 32);
        tmem_load_wait();
        if (tid < n_rows) {
#pragma unroll
          for (int c = 0; c < 8; ++c) {
            uint32_t w[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              __nv_bfloat162 t = __floats2bfloat162_rn(o[c * 8 + 2 * e] * inv, o[c * 8 + 2 * e + 1] * inv);
              w[e] = *reinterpret_cast<uint32_t*>(&t);
            }
            dst[b * 8 + c] = make_uint4(w[0], w[1], w[2], w[3]);
          }
        }
      }
    }
  }
  // tensor memory and the stages are the products' until the last one issued is done (at once when
  // every tile's output was waited for above; what counts when a role gave up)
  if (tid == 0) mbar_drain(done_bar, 0, p.error_out);
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS_ATT) : "memory");
}

// ---------------------------------------------------------------------------------------------
// Persistent form of the kernel above. A CTA of the kernel above lives for one query tile, and about
// a third of its life at 2,048 tokens is not softmax: it sets up barriers and tensor memory, reads
// its slice of the block table, waits for its first keys and its query rows, and at the end waits
// for the last product, writes its rows and leaves, before the next CTA can start the same on its
// slot. Here two CTAs an SM stay and take query tiles from a counter, longest first, and the warp
// that issues copies and products runs ahead of the softmax warps ACROSS tiles of queries: while
// they finish the last keys of one query tile and write its rows, the first keys and the query rows
// of the next are already there and its first scores are done.
//   * warp 5: lane 0 waits, fetches work items and issues the query rows' copy; every lane below
//     pages-per-tile reads its page of a key tile from the block table and issues that copy; warp 4:
//     one thread issues the products (a trip to L2 for a page number never delays a product);
//   * query rows come by TMA, a box of (tokens of the tile) x 64 dims per head, so row r of the
//     tile is (head r / tokens-per-tile, token r % tokens-per-tile);
//   * every barrier completes once a key tile (keys, values: once a tile and stage), so the parities
//     follow one counter of key tiles that runs on through the query tiles; the first product of a
//     query tile overwrites the output of the one before, which its rows have long read out: they
//     wrote this tile's probabilities, which the product waits for, after that;
//   * work items travel from lane 0 of warp 5 to the other warps through a ring of eight in shared
//     memory, one barrier a slot: the copying warp is at most four items ahead of the softmax warps.
struct AttItem {
  int seq, kvh, tok_base, pos0, n_tq, kt_first, n_tiles, hi;  // n_tiles 0: no more work
};

// Tokens of a query tile: a head's rows start 1,024 bytes apart or a multiple of it (the swizzle
// pattern's period), so a multiple of 8 tokens; 0: the group is too large for this form.
__host__ __device__ inline int persistent_tq_cap(int g) { return (ROWS / g) / 8 * 8; }

// Work item `it` of a step: the kv head runs fastest, then the query tiles of request 0 from its last
// (which sees the most keys) to its first, then those of request 1, and so on. seq_first[s] is the
// number of query tiles of the requests before s (seq_first[n_seqs]: of all), so that requests with a
// single token beside a long prompt portion add one item a kv head each and no empty ones.
template <int HD>
__device__ __forceinline__ void att_item(const AttnTcParams& p, int it, int n_seqs, const int* seq_first, AttItem* out) {
  constexpr int KEYS = AttLayout<HD>::KEYS;
  const int g = p.nq / p.nkv, tq_cap = persistent_tq_cap(g);
  const int kvh = it % p.nkv, j = it / p.nkv;
  int lo_s = 0, hi_s = n_seqs;  // the request whose tiles hold j: seq_first[lo_s] <= j < seq_first[lo_s + 1]
  while (hi_s - lo_s > 1) {
    const int mid = (lo_s + hi_s) >> 1;
    if (seq_first[mid] <= j) lo_s = mid;
    else hi_s = mid;
  }
  const int seq = lo_s, tiles = seq_first[seq + 1] - seq_first[seq];
  const int q0 = (tiles - 1 - (j - seq_first[seq])) * tq_cap, ntok = p.seq_ntok[seq];
  out->seq = seq;
  out->kvh = kvh;
  out->n_tq = min(tq_cap, ntok - q0);
  out->tok_base = p.seq_qoff[seq] + q0;
  out->pos0 = p.seq_start[seq] + q0;
  out->hi = out->pos0 + out->n_tq - 1;
  const int lo = (p.window > 0) ? max(0, out->pos0 - p.window + 1) : 0;
  out->kt_first = lo / KEYS;
  out->n_tiles = out->hi / KEYS - out->kt_first + 1;
}

enum : int { ERR_ATT_ITEM = 14 };

constexpr int ATT_PERSISTENT_THREADS = 192;  // warps 0-3: softmax; warp 4: one thread issues the products; warp 5: work items and copies

template <int HD>
__global__ void __launch_bounds__(ATT_PERSISTENT_THREADS, 2)
    paged_attention_tc_persistent_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                                         const __grid_constant__ CUtensorMap map_v, const AttnTcParams p, int n_seqs,
                                         int* __restrict__ work) {  // work[0]: next item, work[1]: CTAs that are done
  using L = AttLayout<HD>;
  constexpr int KEYS = L::KEYS, DBLK = L::DBLK, Q_BYTES = L::Q_BYTES, KV_BYTES = L::KV_BYTES;
  constexpr int S_COL = L::S_COL, P_COL = L::P_COL, O_COL = L::O_COL;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint8_t* q_s = smem;             // [DBLK blocks][128 rows][128 B], 128-byte swizzle
  uint8_t* kv_s = smem + Q_BYTES;  // [2 stages][K | V], each [DBLK blocks][KEYS rows][128 B]
  uint64_t* full_k = reinterpret_cast<uint64_t*>(kv_s + 4 * KV_BYTES);  // [2] the keys of a tile have landed in the stage
  uint64_t* full_v = full_k + 2;   // [2] the values
  uint64_t* empty_k = full_v + 2;  // [2] the scores that read the stage's keys are done
  uint64_t* empty_v = empty_k + 2; // [2] the product that read the stage's values is done
  uint64_t* q_full = empty_v + 2;  // the query rows of an item have landed
  uint64_t* q_empty = q_full + 1;  // the last scores of an item are done: its query rows may be overwritten
  uint64_t* s_bar = q_empty + 1;   // the scores of a key tile are in tensor memory
  uint64_t* s_free = s_bar + 1;    // every row has read them (an arrival a softmax warp)
  uint64_t* p_bar = s_free + 1;    // every row's probabilities are in tensor memory (an arrival a warp)
  uint64_t* o_bar = p_bar + 1;     // the P V product of a key tile is done
  uint64_t* done_bar = o_bar + 1;  // every product that was issued has finished
  uint64_t* item_bar = done_bar + 1;  // [8] ring slot holds an item
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(item_bar + 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  AttItem* ring = reinterpret_cast<AttItem*>(tmem_slot + 4);  // [8]
  int* seq_first = reinterpret_cast<int*>(ring + 8);          // [n_seqs + 1] query tiles of the requests before (used by warp 5 only)

  dep_launch();
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = p.nq / p.nkv, tq_cap = persistent_tq_cap(g);
  const int pages_per_tile = KEYS / p.page_size;

  if (tid == 0) {
    for (int b = 0; b < 2; ++b) {
      mbar_init(&full_k[b], 1);
      mbar_init(&full_v[b], 1);
      mbar_init(&empty_k[b], 1);
      mbar_init(&empty_v[b], 1);
    }
    mbar_init(q_full, 1);
    mbar_init(q_empty, 1);
    mbar_init(s_bar, 1);
    mbar_init(s_free, ROWS / 32);
    mbar_init(p_bar, ROWS / 32);
    mbar_init(o_bar, 1);
    mbar_init(done_bar, 1);
    for (int b = 0; b < 8; ++b) mbar_init(&item_bar[b], 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(TMEM_COLS_ATT) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  // rows of the query tile that no copy writes (128 is no multiple of every group size) read as zeros
  for (int i = tid; i < Q_BYTES / 16; i += ATT_PERSISTENT_THREADS) reinterpret_cast<uint4*>(q_s)[i] = make_uint4(0, 0, 0, 0);
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_slot;
  dep_wait();  // queries, keys and values come from the kernels before; the work counter was left at zero by the launch before

  if (warp == 5) {
    // ------------------------------------------------------------------ the warp that fetches work and issues the copies
    // Lane 0 waits and takes items from the counter; every lane below pages-per-tile issues its page's
    // copy of a key tile. The stream of key tiles runs on through the items: keys of tile gt go to
    // stage gt % 2 once the scores of tile gt - 2 are done (empty_k of the stage), values once the
    // product of tile gt - 2 is done (empty_v), the query rows of an item once the last scores of the
    // item before are done (q_empty). Each of these barriers belongs to one buffer and cannot complete
    // again before this warp has filled the buffer again, so a wait here is never a phase behind.
    struct Cur {  // a key tile of the CTA's stream: ring slot of its item, index in the item, tiles of the item (0: no more)
      int slot, i, n;
    };
    int n_fetched = 0;
    bool ok = true;
    int n_items = 0;
    {  // the query tiles of every request, summed up (the batch arrays came with the step's host-to-device copy)
      int run = 0;
      for (int base = 0; base < n_seqs; base += 32) {
        const int sq = base + lane;
        const int cnt = sq < n_seqs ? (p.seq_ntok[sq] + tq_cap - 1) / tq_cap : 0;
        int incl = cnt;
#pragma unroll
        for (int off = 1; off < 32; off <<= 1) {
          const int v = __shfl_up_sync(0xffffffffu, incl, off);
          if (lane >= off) incl += v;
        }
        if (sq < n_seqs) seq_first[sq] = run + incl - cnt;
        run += __shfl_sync(0xffffffffu, incl, 31);
      }
      if (lane == 0) seq_first[n_seqs] = run;
      __syncwarp();
      n_items = run * p.nkv;
    }
    auto fetch = [&]() -> Cur {  // the first key tile of the next item
      int slot = n_fetched & 7, n = 0;
      if (lane == 0) {
        AttItem item;
        item.n_tiles = 0;
        const int it = atomicAdd(&work[0], 1);
        if (it < n_items) att_item<HD>(p, it, n_seqs, seq_first, &item);
        ring[slot] = item;
        n = item.n_tiles;
        __threadfence_block();
        mbar_arrive(&item_bar[slot]);
      }
      ++n_fetched;
      n = __shfl_sync(0xffffffffu, n, 0);
      __syncwarp();
      return Cur{slot, 0, n};
    };
    auto next = [&](const Cur& c) -> Cur {
      if (c.n == 0) return c;
      if (c.i + 1 < c.n) return Cur{c.slot, c.i + 1, c.n};
      return fetch();
    };
    // The first cache row of this lane's page of key tile c, through the block table; asked for a key
    // tile ahead of its use.
    auto page_row = [&](const Cur& c) -> int {
      if (c.n == 0 || lane >= pages_per_tile) return 0;
      const AttItem& item = ring[c.slot];
      const int idx = ((item.kt_first + c.i) * KEYS) / p.page_size + lane;
      int page = (idx < p.max_blocks && idx * p.page_size <= item.hi) ? p.block_table[(size_t)item.seq * p.max_blocks + idx] : -1;
      if (page < 0) page = p.null_page;  // not held (beyond the newest key, or given back behind a window): finite values, probabilities of zero
      return (page * p.nkv + item.kvh) * p.page_size;
    };
    auto issue_part = [&](int row, int gt, bool values) {  // keys or values of key tile gt of the stream -> stage gt % 2
      uint8_t* dst = kv_s + (size_t)(gt & 1) * 2 * KV_BYTES + (values ? KV_BYTES : 0);
      uint64_t* bar = values ? &full_v[gt & 1] : &full_k[gt & 1];
      if (lane == 0) mbar_expect_tx(bar, (uint32_t)KV_BYTES);
      __syncwarp();
      if (lane < pages_per_tile) {
        const CUtensorMap* map = values ? &map_v : &map_k;
#pragma unroll
        for (int b = 0; b < DBLK; ++b) tma_load_2d(dst + b * (KEYS * 128) + (size_t)lane * p.page_size * 128, map, b * 64, row, bar);
      }
      __syncwarp();
    };
    auto issue_q = [&](const Cur& c) {  // the query rows of c's item: a box of tq_cap tokens x 64 dims per head and block
      if (lane == 0) {
        const AttItem& item = ring[c.slot];
        mbar_expect_tx(q_full, (uint32_t)(g * DBLK * tq_cap * 128));
        for (int hg = 0; hg < g; ++hg)
#pragma unroll
          for (int b = 0; b < DBLK; ++b)
            tma_load_2d(q_s + b * (ROWS * 128) + (size_t)hg * tq_cap * 128, &map_q, (item.kvh * g + hg) * HD + b * 64, item.tok_base, q_full);
      }
      __syncwarp();
    };
    auto wait0 = [&](uint64_t* bar, uint32_t parity, int code) -> bool {  // lane 0 waits, the warp learns the outcome
      bool r = true;
      if (lane == 0) r = mbar_wait(bar, parity, abort_flag, p.error_out, code);
      return __shfl_sync(0xffffffffu, r, 0);
    };
    int kv_issued = 0, q_issued = 0;  // key tiles and items whose copies have been asked for (for the drain after giving up)
    Cur c = fetch(), c1 = next(c);
    int row = page_row(c);
    for (int gt = 0; c.n > 0 && ok; ++gt) {
      const int row1 = page_row(c1);  // used a key tile from now
      if (c.i == 0) {  // a new item: its query rows, once the scores of the item before are done with theirs
        if (q_issued > 0) {
          ok = wait0(q_empty, (uint32_t)(q_issued - 1) & 1u, ERR_ATT_S);
          if (!ok) break;
        }
        issue_q(c);
        ++q_issued;
      }
      if (gt >= 2) {
        ok = wait0(&empty_k[gt & 1], (uint32_t)((gt >> 1) - 1) & 1u, ERR_ATT_S);
        if (!ok) break;
      }
      issue_part(row, gt, false);
      if (gt >= 2) {
        ok = wait0(&empty_v[gt & 1], (uint32_t)((gt >> 1) - 1) & 1u, ERR_ATT_O);
        if (!ok) {
          if (lane == 0) mbar_drain(&full_k[gt & 1], (uint32_t)(gt >> 1) & 1u, p.error_out);  // the keys just asked for
          break;
        }
      }
      issue_part(row, gt, true);
      kv_issued = gt + 1;
      c = c1;
      c1 = next(c1);
      row = row1;
    }
    if (!ok && lane == 0) {
      // gave up: what was asked for lands (bounded) before the CTA gives its shared memory back; the other
      // roles see the abort flag
      for (int t = max(0, kv_issued - 2); t < kv_issued; ++t) {
        mbar_drain(&full_k[t & 1], (uint32_t)(t >> 1) & 1u, p.error_out);
        mbar_drain(&full_v[t & 1], (uint32_t)(t >> 1) & 1u, p.error_out);
      }
      if (q_issued > 0) mbar_drain(q_full, (uint32_t)(q_issued - 1) & 1u, p.error_out);
    }
  } else if (warp == 4) {
    // ------------------------------------------------------------------ the thread that issues the products
    if (lane == 0) {
      bool ok = true;
      int gt = 0;          // key tiles of the stream whose scores have been issued
      int prev_first = 0;  // whether tile gt - 1 was the first of its item (its product overwrites the output)
      auto issue_pv = [&](int t, bool first) {  // O (+)= P V of key tile t
        ok = mbar_wait(p_bar, (uint32_t)t & 1u, abort_flag, p.error_out, ERR_ATT_S);
        if (ok) ok = mbar_wait(&full_v[t & 1], (uint32_t)(t >> 1) & 1u, abort_flag, p.error_out, ERR_ATT_KV);
        if (!ok) return;
        // (the first product of an item overwrites the output of the item before: its rows wrote P of this
        // tile after they had read that output out)
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        constexpr uint32_t idesc_o = instr_desc_att(64, true);
#pragma unroll
        for (int b = 0; b < DBLK; ++b) {
          const uint64_t dv = smem_desc_sw128(smem_u32(kv_s + (size_t)(t & 1) * 2 * KV_BYTES + KV_BYTES + b * (KEYS * 128)));
#pragma unroll
          for (int k = 0; k < KEYS / 16; ++k)
            mma_f16_ts(tmem_base + O_COL + (uint32_t)(b * 64), tmem_base + P_COL + (uint32_t)(k * 8), dv + (uint64_t)(k * (16 * 128 >> 4)),
                       idesc_o, (!first || k > 0) ? 1u : 0u);
        }
        mma_commit(o_bar);
        mma_commit(&empty_v[t & 1]);  // the value stage may be filled again once this product is done
      };
      for (int n_item = 0; ok; ++n_item) {
        ok = mbar_wait(&item_bar[n_item & 7], (uint32_t)(n_item >> 3) & 1u, abort_flag, p.error_out, ERR_ATT_ITEM);
        if (!ok) break;
        const int n_tiles = ring[n_item & 7].n_tiles;
        if (n_tiles == 0) break;
        for (int i = 0; i < n_tiles && ok; ++i, ++gt) {
          // the scores of tile gt: the S columns are free once every row has read those of the tile before;
          // the first tile of an item also needs the item's query rows
          if (gt > 0) ok = mbar_wait(s_free, (uint32_t)(gt - 1) & 1u, abort_flag, p.error_out, ERR_ATT_S);
          if (ok && i == 0) ok = mbar_wait(q_full, (uint32_t)n_item & 1u, abort_flag, p.error_out, ERR_ATT_KV);
          if (ok) ok = mbar_wait(&full_k[gt & 1], (uint32_t)(gt >> 1) & 1u, abort_flag, p.error_out, ERR_ATT_KV);
          if (!ok) break;
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          constexpr uint32_t idesc_s = instr_desc_att(KEYS, false);
#pragma unroll
          for (int k = 0; k < HD / 16; ++k) {  // 16 dims a step: block k / 4, 32 bytes further along the swizzled row each step
            const uint64_t dq = smem_desc_sw128(smem_u32(q_s + (k / 4) * (ROWS * 128)));
            const uint64_t dk = smem_desc_sw128(smem_u32(kv_s + (size_t)(gt & 1) * 2 * KV_BYTES + (k / 4) * (KEYS * 128)));
            mma_f16(tmem_base + S_COL, dq + (uint64_t)(2 * (k % 4)), dk + (uint64_t)(2 * (k % 4)), idesc_s, k > 0 ? 1u : 0u);
          }
          mma_commit(s_bar);
          mma_commit(&empty_k[gt & 1]);              // the key stage may be filled again once these scores are done,
          if (i == n_tiles - 1) mma_commit(q_empty);  // and after an item's last scores, the query rows
          // and under the softmax of tile gt, the product of the tile before
          if (gt > 0) issue_pv(gt - 1, prev_first != 0);
          prev_first = (i == 0);
        }
      }
      if (ok && gt > 0) issue_pv(gt - 1, prev_first != 0);
      mma_commit(done_bar);  // also after giving up: arrives once every product that was issued has finished
    }
    } else {
    // ------------------------------------------------------------------ softmax: thread t owns row t
    const uint32_t lane_base = (uint32_t)(warp * 32) << 16;
    const int hg = tid / tq_cap, tq_row = tid - hg * tq_cap;  // rows are (head, token): the query rows came a head a box
    const float sl2 = p.scale * 1.4426950408889634f;
    bool ok = true;
    int gt = 0;  // key tiles of the CTA's stream so far
    for (int n_item = 0; ok; ++n_item) {
      ok = mbar_wait(&item_bar[n_item & 7], (uint32_t)(n_item >> 3) & 1u, abort_flag, p.error_out, ERR_ATT_ITEM);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      const AttItem item = ring[n_item & 7];
      if (item.n_tiles == 0) break;
      const bool row_ok = hg < g && tq_row < item.n_tq;
      const int pos_r = row_ok ? item.pos0 + tq_row : -1;  // -1: padding row, sees no key
      const int lo_r = (p.window > 0) ? pos_r - p.window + 1 : 0;
      float m_run = -INFINITY, l_run = 0.f;
      for (int i = 0; i < item.n_tiles; ++i, ++gt) {
        ok = mbar_wait(s_bar, (uint32_t)gt & 1u, abort_flag, p.error_out, ERR_ATT_S);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        float s[KEYS];
#pragma unroll
        for (int c = 0; c < KEYS / 32; ++c) tmem_load32(tmem_base + lane_base + S_COL + c * 32, s + c * 32);
        tmem_load_wait();
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncwarp();
        if (lane == 0) mbar_arrive(s_free);
        const int key0 = (item.kt_first + i) * KEYS;
        const bool full_tile = (key0 + KEYS - 1 <= pos_r) && (key0 >= lo_r);
        float mx = -INFINITY;
        if (!full_tile) {
#pragma unroll
          for (int j = 0; j < KEYS; ++j) {
            const int key = key0 + j;
            s[j] = (key <= pos_r && key >= lo_r) ? s[j] : -INFINITY;
          }
        }
        {
          float m8[8];
#pragma unroll
          for (int c = 0; c < 8; ++c) m8[c] = max3(s[c], s[c + 8], s[c + 16]);
#pragma unroll
          for (int j = 24; j + 16 <= KEYS; j += 16) {
#pragma unroll
            for (int c = 0; c < 8; ++c) m8[c] = max3(m8[c], s[j + c], s[j + c + 8]);
          }
#pragma unroll
          for (int c = 0; c < 8; ++c) m8[c] = fmaxf(m8[c], s[KEYS - 8 + c]);
          mx = fmaxf(max3(m8[0], m8[1], m8[2]), fmaxf(max3(m8[3], m8[4], m8[5]), fmaxf(m8[6], m8[7])));
        }
        mx *= sl2;
        const bool move = (mx > m_run + 8.0f) || (m_run == -INFINITY && mx > -INFINITY);
        const float m_new = move ? mx : m_run;
        const float base = (m_new == -INFINITY) ? 0.f : m_new;
        const float alpha = move ? fast_exp2(m_run - base) : 1.0f;
        uint32_t packed[KEYS / 2];
        l_run = l_run * alpha + exp_row<KEYS>(s, sl2, base, packed);
        m_run = m_new;
        if (gt > 0) {
          // the product of the key tile before (of this item, or the last of the item before) reads the P columns
          ok = mbar_wait(o_bar, (uint32_t)(gt - 1) & 1u, abort_flag, p.error_out, ERR_ATT_O);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        }
#pragma unroll
        for (int c = 0; c < KEYS / 64; ++c) tmem_store32(tmem_base + lane_base + P_COL + c * 32, packed + c * 32);
        if (i > 0 && __any_sync(0xffffffffu, move)) {
#pragma unroll
          for (int c = 0; c < HD / 64; ++c) {
            float o[64];
            tmem_load32(tmem_base + lane_base + O_COL + c * 64, o);
            tmem_load32(tmem_base + lane_base + O_COL + c * 64 + 32, o + 32);
            tmem_load_wait();
            uint32_t ou[64];
#pragma unroll
            for (int d = 0; d < 64; ++d) ou[d] = __float_as_uint(o[d] * alpha);
            tmem_store32(tmem_base + lane_base + O_COL + c * 64, ou);
            tmem_store32(tmem_base + lane_base + O_COL + c * 64 + 32, ou + 32);
          }
        }
        asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncwarp();
        if (lane == 0) mbar_arrive(p_bar);
      }
      if (!ok) break;
      // ---- the rows of the item's output, normalised
      ok = mbar_wait(o_bar, (uint32_t)(gt - 1) & 1u, abort_flag, p.error_out, ERR_ATT_O);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
      uint4* dst = reinterpret_cast<uint4*>(p.out + (size_t)(item.tok_base + tq_row) * p.ld_out + (size_t)(item.kvh * g + hg) * HD);
#pragma unroll
      for (int b = 0; b < HD / 64; ++b) {
        float o[64];
        tmem_load32(tmem_base + lane_base + O_COL + b * 64, o);
        tmem_load32(tmem_base + lane_base + O_COL + b * 64 + 32, o + 32);
        tmem_load_wait();
        if (row_ok) {
#pragma unroll
          for (int c = 0; c < 8; ++c) {
            uint32_t w[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              __nv_bfloat162 t = __floats2bfloat162_rn(o[c * 8 + 2 * e] * inv, o[c * 8 + 2 * e + 1] * inv);
              w[e] = *reinterpret_cast<uint32_t*>(&t);
            }
            dst[b * 8 + c] = make_uint4(w[0], w[1], w[2], w[3]);
          }
        }
      }
      // (the output has left tensor memory; the next item's first product, which overwrites it, waits for
      // probabilities that these threads write later)
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    }
  }
  __syncwarp();
  if (tid == 0) mbar_drain(done_bar, 0, p.error_out);
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS_ATT) : "memory");
  if (tid == 0) {  // the CTA that leaves last puts the counters back to zero for the next launch
    __threadfence();
    if (atomicAdd(&work[1], 1) == (int)gridDim.x - 1) {
      work[0] = 0;
      work[1] = 0;
      __threadfence();
    }
  }
}

template <int HD>
bool launch_att(const CUtensorMap& mk, const CUtensorMap& mv, const AttnTcParams& p, dim3 grid, int max_blocks, cudaStream_t stream) {
  using L = AttLayout<HD>;
  // Q, two stages of K and V, ten 8-byte words of barriers, four ints, the block-table slice (whole tiles: up to 16
  // pages beyond the table's width), alignment slack
  const size_t smem = L::Q_BYTES + 4 * L::KV_BYTES + 10 * sizeof(uint64_t) + 16 + (size_t)(max_blocks + 16) * sizeof(int) + 1024;
  static size_t attr_smem = 0;
  if (smem > attr_smem) {
    if (cudaFuncSetAttribute(paged_attention_tc_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) return false;
    attr_smem = smem;
  }
  launch_kernel(paged_attention_tc_kernel<HD>, grid, ATT_THREADS, smem, stream, mk, mv, p);
  return true;
}

template <int HD>
bool launch_att_persistent(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, const AttnTcParams& p, int n_seqs,
                           long long max_items, int* work, int n_sms, cudaStream_t stream) {
  using L = AttLayout<HD>;
  const size_t smem = L::Q_BYTES + 4 * L::KV_BYTES + 24 * sizeof(uint64_t) + 16 + 8 * sizeof(AttItem) + (size_t)(n_seqs + 1) * sizeof(int) + 1024;
  static size_t attr_smem = 0;
  if (smem > attr_smem) {
    if (cudaFuncSetAttribute(paged_attention_tc_persistent_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) return false;
    attr_smem = smem;
  }
  const int grid = (int)std::min<long long>(max_items, 2 * n_sms);  // (the step may hold fewer items than max_items: CTAs without one leave at once)
  launch_kernel(paged_attention_tc_persistent_kernel<HD>, grid, ATT_PERSISTENT_THREADS, smem, stream, mq, mk, mv, p, n_seqs, work);
  return true;
}

int att_sm_count() {
  static int n = 0;
  if (!n) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
  }
  return n;
}

}  // namespace

static int g_att_persistent = 1;
// 1 (the default): query tiles are taken from a counter by CTAs that stay (where the group allows);
// 0: a CTA a query tile. For comparisons; the results are the same sums in the same order.
extern "C" void llm_attention_tc_persistent(int on) { g_att_persistent = on; }

// Whether the tcgen05 attention takes this geometry (else the caller uses the mma.sync kernel).
extern "C" int llm_attention_tc_supported(int nq, int nkv, int hd, int page_size, long long ld_q, long long ld_out) {
  if (nkv <= 0 || nq % nkv) return 0;
  const int g = nq / nkv;
  if (hd != 64 && hd != 128) return 0;
  const int keys = hd == 64 ? AttLayout<64>::KEYS : AttLayout<128>::KEYS;
  return g <= ROWS && page_size % 8 == 0 && keys % page_size == 0 && (ld_q % 8) == 0 && (ld_out % 8) == 0 &&
         encode_fn() != nullptr;
}

// q: rows of [nq*hd] bf16; caches [pages, nkv, page_size, hd] bf16 (n_cache_pages pages each, the LAST of
// them the null page: finite values, never a request's);
// seq_* and block_table as in the step's batch; out [n_tokens, nq*hd] bf16. n_tokens: rows of q. work: two ints
// that are zero between launches (the persistent form's counters: next query tile, CTAs that are done; the
// kernel leaves them at zero), or null for the form with a CTA a query tile.
extern "C" int llm_paged_attention_tc(const void* q, long long ld_q, const void* kcache, const void* vcache, long long n_cache_pages,
                                      const int* seq_start, const int* seq_ntok, const int* seq_qoff, const int* block_table,
                                      int max_blocks, void* out, long long ld_out, int n_seqs, int max_new_tokens, int nq, int nkv,
                                      int hd, int page_size, float scale, int window, int n_tokens, int* work, cudaStream_t stream) {
  if (n_seqs == 0 || max_new_tokens == 0) return LLM_OK;
  LLM_REQUIRE(llm_attention_tc_supported(nq, nkv, hd, page_size, ld_q, ld_out), "attention_tc: geometry not supported (nq=%d nkv=%d hd=%d page=%d)", nq, nkv, hd, page_size);
  auto al = [](const void* ptr) { return (reinterpret_cast<uintptr_t>(ptr) & 15u) == 0; };
  LLM_REQUIRE(al(q) && al(kcache) && al(vcache) && al(out), "attention_tc: q, the caches and out must be 16-byte aligned");
  LLM_REQUIRE(max_blocks > 0 && window >= 0 && n_seqs <= 65535 && nkv <= 65535, "attention_tc: bad sizes");
  LLM_REQUIRE((long long)max_new_tokens * (nq / nkv) <= 65535LL * ROWS, "attention_tc: portion too long for the grid");
  LLM_REQUIRE(error_word() != nullptr, "attention_tc: cannot allocate the error word");
  CUtensorMap mk, mv;
  const long long rows = n_cache_pages * nkv * page_size;
  LLM_REQUIRE(tensor_map_for(kcache, rows, hd, hd, page_size, &mk) && tensor_map_for(vcache, rows, hd, hd, page_size, &mv),
              "attention_tc: cuTensorMapEncodeTiled failed");
  AttnTcParams p;
  p.q = (const bf16*)q; p.ld_q = ld_q; p.seq_start = seq_start; p.seq_ntok = seq_ntok; p.seq_qoff = seq_qoff; p.block_table = block_table;
  p.max_blocks = max_blocks; p.nq = nq; p.nkv = nkv; p.page_size = page_size; p.window = window; p.scale = scale;
  p.out = (bf16*)out; p.ld_out = ld_out; p.error_out = error_word();
  p.null_page = (int)(n_cache_pages - 1);
  LLM_REQUIRE(max_blocks <= 4096, "attention_tc: block tables wider than 4096 pages are not supported");
  const int g = nq / nkv, tq_cap = ROWS / g;
  const int ptq = persistent_tq_cap(g);
  if (g_att_persistent && ptq >= 8 && n_tokens >= ptq && (ld_q % 8) == 0 && work != nullptr) {  // (a box of query rows is no taller than q)
    // the persistent form: query rows by TMA (rows of q: the step's tokens), work items from a counter
    CUtensorMap mq;
    LLM_REQUIRE(tensor_map_for(q, n_tokens, (long long)nq * hd, ld_q, ptq, &mq), "attention_tc: cuTensorMapEncodeTiled failed for q");
    // at most: every token a query tile of its own, or every request as many as the longest portion
    const long long max_items = std::min<long long>((long long)n_tokens, (long long)n_seqs * ((max_new_tokens + ptq - 1) / ptq)) * nkv;
    LLM_REQUIRE(max_items < (1LL << 30) && n_seqs < 40000, "attention_tc: too many query tiles");
    const bool ok = hd == 64 ? launch_att_persistent<64>(mq, mk, mv, p, n_seqs, max_items, work, att_sm_count(), stream)
                             : launch_att_persistent<128>(mq, mk, mv, p, n_seqs, max_items, work, att_sm_count(), stream);
    LLM_REQUIRE(ok, "attention_tc: cannot raise the shared memory limit");
    LLM_CHECK_LAUNCH("paged_attention_tc");
    return LLM_OK;
  }
  dim3 grid(nkv, n_seqs, (max_new_tokens + tq_cap - 1) / tq_cap);
  bool attr_ok = true;
  if (hd == 64) attr_ok = launch_att<64>(mk, mv, p, grid, max_blocks, stream);
  else attr_ok = launch_att<128>(mk, mv, p, grid, max_blocks, stream);
  LLM_REQUIRE(attr_ok, "attention_tc: cannot raise the shared memory limit");
  LLM_CHECK_LAUNCH("paged_attention_tc");
  return LLM_OK;
}
