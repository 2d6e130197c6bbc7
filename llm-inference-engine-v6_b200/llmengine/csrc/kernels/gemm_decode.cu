// Matrix products of a step with few tokens (decoding): weights stream once, and everything that
// used to be a small kernel of its own around the product happens inside it.
//
//   D[n, t] = sum_k W[n, k] * X[t, k]          W: weights [N, K] bf16; X: activations of T <= 64 tokens
//
// 128 weight rows fill the 128 accumulator lanes of a tcgen05 tile (two tiles per CTA where a gate
// and an up projection must meet), the tokens are the tile's columns. One output tile has too few
// bytes to keep a B200 busy, so the K range is cut into `splits` pieces; the CTAs of one output tile
// are ONE thread-block cluster and add their partial sums through distributed shared memory: every
// CTA sends each row of its partial to the CTA that finishes that row (asynchronous stores whose
// bytes are counted on an mbarrier there, so no fence and no arrival is needed), and finishes its
// own rows by adding what it received in the order of the K pieces (a fixed order: the result does
// not depend on timing). No partial sum goes to global memory.
//
// The other way for the K pieces to meet (chosen by the caller, who then brings scratch memory):
// every CTA writes its partial to global memory and counts itself in per output tile; the CTA that
// arrives last adds the pieces of the whole tile in index order and runs the epilogue. No clusters:
// any number of pieces, CTAs are placed one by one (a cluster waits until all its CTAs fit at once,
// which costs a chain of small kernels most of the overlap that programmatic dependent launch
// gives), at the price of one trip through the L2 for the partials.
//
// Where the activations come from (the tile's B operand):
//   * bf16 rows in global memory, fetched by TMA; or
//   * an RMSNorm that has not run: float32 rows x of the residual stream, the parts of their sums
//     of squares, the norm's weight and eps. The four epilogue warps, idle until the products end,
//     write (w * x) * inv_rms as bf16 straight into the operand stage (128-byte swizzle), so the
//     norm is no kernel of its own. Formula and order of operations: rmsnorm_f32 of the reference
//     (src/kernels.cpp:18-24). A row list (the rows whose logits are wanted) may pick the rows.
//
// What happens to the finished sums (the epilogue of the rows' owner):
//   * PLAIN:    out[t, n] = d, float32 or bf16;
//   * RESIDUAL: h[t, n] += d (the residual stream, float32) and the part of sum_n h[t, n]^2 that
//               these rows hold goes to sumsq[t, part]: what the next norm needs, so that the norm
//               can be folded into the product after it;
//   * SWIGLU:   the CTA holds 128 gate rows and the 128 matching up rows;
//               act[t, c] = silu(gate) * up as bf16, silu(v) = v / (1 + exp(-v)) as the reference's
//               silu_f32 (src/kernels.cpp:26-31).
//
// Roles: warps 0-3 produce normalised activations (if asked) and run the epilogue; warp 4 lane 0
// issues the TMA loads (weights before the wait on the previous kernel); warp 5 lane 0 issues
// tcgen05.mma. Every wait is bounded (tc_common.cuh); the hardware cluster barrier is used once,
// split in two as in attention_decode.cu, before the first access to a peer's shared memory.
#include "tc_common.cuh"

namespace {

constexpr int GD_THREADS = 192;
constexpr int GD_EPI = 128;  // epilogue / activation-producer threads (warps 0-3)
enum : int { GD_PLAIN = 0, GD_RESIDUAL = 1, GD_SWIGLU = 2 };
enum : int { ERR_GD_PRODUCER = 31, ERR_GD_MMA = 32, ERR_GD_EPILOGUE = 33, ERR_GD_PEERS = 34, ERR_GD_ACT = 35 };

struct GdParams {
  int N, K, T;              // weight rows, inner size, tokens (T <= BN)
  int k_tiles, k_per_split;
  int csize;                // CTAs per cluster = K pieces
  int rows_per;             // accumulator rows each CTA of the cluster finishes: ceil(128 / csize)
  int stages;
  // activations by norm (x != nullptr) -- else they come by TMA
  const float* x; long long ld_x;
  const float* sumsq; int n_sumsq;     // [rows of x][n_sumsq] parts of the rows' sums of squares
  const float* norm_w; float eps;
  const int* rows;                     // x row of token t (nullptr: t)
  // outputs
  void* out; long long ld_out;         // PLAIN / SWIGLU
  float* h; long long ld_h;            // RESIDUAL
  float* sumsq_out; int n_sumsq_out;   // RESIDUAL: [T][n_sumsq_out]; in a cluster this CTA writes part blockIdx.x * csize + rank, else the last CTA of a tile writes part blockIdx.x
  int in_cluster;                      // the K pieces meet in shared memory of a cluster (1) or in global memory (0)
  float* parts; int* counters;         // in_cluster == 0: [tiles][csize][128][TILES][t4] floats; [tiles] ints, zero between launches
  int* error;
};

__device__ __forceinline__ void gd_cluster_arrive() { asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory"); }
__device__ __forceinline__ void gd_cluster_wait() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }

__device__ __forceinline__ uint32_t gd_map(uint32_t smem_addr, int rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
  return r;
}
// Four floats into a peer's shared memory, their 16 bytes counted on the mbarrier `bar` (an address
// in that peer's shared memory) when they have landed.
__device__ __forceinline__ void gd_store4_async(uint32_t cluster_addr, uint32_t bar, float a, float b, float c, float d) {
  asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.v4.f32 [%0], {%1, %2, %3, %4}, [%5];" ::"r"(cluster_addr),
               "f"(a), "f"(b), "f"(c), "f"(d), "r"(bar)
               : "memory");
}
// Bounded wait for what the peers send (acquire at cluster scope); it does not leave early on
// another kernel's error: no CTA may exit while a peer can still reach its shared memory.
__device__ __forceinline__ bool gd_wait_peers(uint64_t* bar, int* error_out) {
  const long long t0 = clock64();
  for (uint32_t i = 0;; ++i) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(0u)
        : "memory");
    if (ok) return true;
    if ((i & 255u) == 255u && clock64() - t0 > 2 * WAIT_CYCLES) {
      atomicCAS(error_out, 0, (int)ERR_GD_PEERS);
      return false;
    }
  }
}

// Barrier over the 128 threads of warps 0-3 that also tells whether `mine` held for all of them.
__device__ __forceinline__ bool gd_all_epilogue_threads(bool mine) {
  uint32_t all;
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t"
      "setp.ne.u32 q, %1, 0;\n\t"
      "bar.red.and.pred p, 1, %2, q;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(all)
      : "r"((uint32_t)mine), "n"(GD_EPI)
      : "memory");
  return all != 0;
}

template <int BN, int TILES>
struct GdLayout {
  static constexpr int A_STAGE = TILES * A_BYTES;
  static constexpr int B_STAGE = BN * BK * 2;
  static constexpr int STAGE_BYTES = A_STAGE + B_STAGE;
  static constexpr int TMEM_COLS = (BN * TILES) < 32 ? 32 : BN * TILES;
};

// Bytes of shared memory behind the stages: barriers, flags, the reciprocal roots, what the peers send.
__host__ __device__ inline size_t gd_tail_bytes(int stages, int csize, int rows_per, int tiles, int t4, int mode, int in_cluster) {
  size_t b = (size_t)(3 * stages + 2 + (stages & 1)) * 8 + 16 + 64 * 4;
  if (csize > 1 && in_cluster) b += (size_t)csize * rows_per * tiles * t4 * 4;
  if (mode == GD_RESIDUAL) b += (size_t)(in_cluster ? rows_per : 4) * t4 * 4;
  return b + 16;
}

template <int BN, int TILES, int MODE, typename TO>
__global__ void __launch_bounds__(GD_THREADS)
    gemm_decode_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x, const GdParams p) {
  using L = GdLayout<BN, TILES>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  const int stages = p.stages;
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + (size_t)stages * L::STAGE_BYTES);  // [stages] the copies of a stage have landed
  uint64_t* full_x = full + stages;       // [stages] the stage's activations have been written (norm form)
  uint64_t* empty = full_x + stages;      // [stages] the products have read the stage
  uint64_t* acc_ready = empty + stages;   // every product of this CTA has finished (committed last, also after giving up)
  uint64_t* peers_in = acc_ready + 1;     // the bytes of this CTA's rows, sent by every CTA of the cluster, have all landed
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(peers_in + 1 + (stages & 1));  // (an even number of 8-byte words: what follows stays 16-byte aligned)
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  int* issued_slot = const_cast<int*>(abort_flag) + 1;
  float* inv_s = reinterpret_cast<float*>(tmem_slot + 4);  // [64] reciprocal root mean squares of the tokens' rows
  float* recv = inv_s + 64;                                // [csize][rows_per][TILES][t4]
  const int t4 = (p.T + 3) & ~3;
  float* sq_s = recv + (p.csize > 1 && p.in_cluster ? (size_t)p.csize * p.rows_per * TILES * t4 : 0);  // RESIDUAL: [rows finished here][t4]

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int tile = blockIdx.x, rank = blockIdx.z;  // cluster (1, 1, csize): the rank is the K piece
  const int w_row0 = tile * (128 * TILES);
  const int kt_begin = rank * p.k_per_split;
  const int kt_end = min(p.k_tiles, kt_begin + p.k_per_split);
  const int n_iter = max(kt_end - kt_begin, 0);
  const bool by_norm = p.x != nullptr;

  if (tid == 0) {
    for (int s = 0; s < stages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&full_x[s], 1);
      mbar_init(&empty[s], 1);
    }
    mbar_init(acc_ready, 1);
    mbar_init(peers_in, 1);
    *abort_flag = 0;
    *issued_slot = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    if (p.csize > 1 && p.in_cluster) {  // what the CTAs of the cluster (this one too) will send here: every one its part of this CTA's rows
      const int mine = max(0, min(p.rows_per, 128 - (int)blockIdx.z * p.rows_per));
      mbar_expect_tx(peers_in, (uint32_t)(p.csize * mine * TILES * ((p.T + 3) & ~3) * 4));
    }
  }
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(L::TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  if (by_norm && BN > 8) {  // token rows that no token fills: zeros (they meet columns that are never stored)
    for (int i = tid; i < stages * (L::B_STAGE / 16); i += GD_THREADS) {
      const int s = i / (L::B_STAGE / 16), c = i - s * (L::B_STAGE / 16);
      reinterpret_cast<uint4*>(smem + (size_t)s * L::STAGE_BYTES + L::A_STAGE)[c] = make_uint4(0, 0, 0, 0);
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  // This CTA runs and its barriers exist: the peers learn it at their gd_cluster_wait().
  const bool clustered = p.csize > 1 && p.in_cluster;
  if (clustered) gd_cluster_arrive();
  const uint32_t tmem_base = *tmem_slot;

  dep_launch();
  if (warp == 4) {
    if (lane == 0) {
      // ---------------------------------------------------------------- TMA: weights, and activations if they are bf16 rows
      const uint32_t tx = by_norm ? (uint32_t)L::A_STAGE : (uint32_t)L::STAGE_BYTES;
      const int early = min(stages, n_iter);
      for (int it = 0; it < early; ++it) {  // the weights do not depend on the kernel before
        mbar_expect_tx(&full[it], tx);
#pragma unroll
        for (int a = 0; a < TILES; ++a)
          tma_load_2d(smem + (size_t)it * L::STAGE_BYTES + a * A_BYTES, &map_w, (kt_begin + it) * BK, w_row0 + a * 128, &full[it]);
      }
      *issued_slot = early;
      dep_wait();
      if (!by_norm)
        for (int it = 0; it < early; ++it)
          tma_load_2d(smem + (size_t)it * L::STAGE_BYTES + L::A_STAGE, &map_x, (kt_begin + it) * BK, 0, &full[it]);
      bool ok = true;
      RingPos ring(stages, 0, 1u);
      for (int it = early; it < n_iter && ok; ++it, ring.next()) {
        const int s = ring.s;
        ok = mbar_wait(&empty[s], ring.ph ^ 1u, abort_flag, p.error, ERR_GD_PRODUCER);
        if (!ok) break;
        uint8_t* st = smem + (size_t)s * L::STAGE_BYTES;
        mbar_expect_tx(&full[s], tx);
#pragma unroll
        for (int a = 0; a < TILES; ++a) tma_load_2d(st + a * A_BYTES, &map_w, (kt_begin + it) * BK, w_row0 + a * 128, &full[s]);
        if (!by_norm) tma_load_2d(st + L::A_STAGE, &map_x, (kt_begin + it) * BK, 0, &full[s]);
        *issued_slot = it + 1;
      }
    }
  } else if (warp == 5) {
    if (lane == 0) {
      // ---------------------------------------------------------------- tensor-core issue
      constexpr uint32_t idesc = instr_desc(BN);
      bool ok = true;
      RingPos ring(stages);
      for (int it = 0; it < n_iter && ok; ++it, ring.next()) {
        const int s = ring.s;
        ok = mbar_wait(&full[s], ring.ph, abort_flag, p.error, ERR_GD_MMA);
        if (ok && by_norm) ok = mbar_wait(&full_x[s], ring.ph, abort_flag, p.error, ERR_GD_MMA);
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t sa = smem_u32(smem + (size_t)s * L::STAGE_BYTES);
        const uint64_t db = smem_desc_sw128(sa + L::A_STAGE);
#pragma unroll
        for (int a = 0; a < TILES; ++a) {
          const uint64_t da = smem_desc_sw128(sa + a * A_BYTES);
#pragma unroll
          for (int k = 0; k < BK / 16; ++k)
            mma_f16(tmem_base + (uint32_t)(a * BN), da + (uint64_t)(2 * k), db + (uint64_t)(2 * k), idesc, (it > 0 || k > 0) ? 1u : 0u);
        }
        mma_commit(&empty[s]);
      }
      mma_commit(acc_ready);  // also after giving up: arrives when every product issued above is done
    }
  } else {
    // ------------------------------------------------------------------ warps 0-3
    dep_wait();  // x, the sums of squares and everything this kernel writes belong to the stream
    bool ok = true;
    if (by_norm) {
      // The activation tile of every k-block of this CTA: (w * x) * inv as bf16, 16-byte chunk c of token
      // row r at c ^ (r % 8). Thread (tq, c) = (tid / 16, tid % 16) owns the four consecutive k at 4 c of
      // tokens tq, tq + 8, ...: one norm-weight quad serves all its tokens. The loads of the next k-block
      // are issued before this one is written, so that their latency hides behind the barrier round.
      constexpr int QPT = BN / 8;  // tokens a thread may own
      const int c4 = (tid & 15) * 4, tq = tid >> 4;
      const int chunk = c4 >> 3, within = (c4 & 7) * 2;
      float4 xa[QPT], xb[QPT], wa, wb;
      auto fetch = [&](int it, float4* xv, float4& wv) {
        const int k = (kt_begin + it) * BK + c4;
        const bool in_k = k < p.K;  // K % 4 == 0 (checked by the launcher)
        wv = in_k ? *reinterpret_cast<const float4*>(p.norm_w + k) : make_float4(0, 0, 0, 0);
#pragma unroll
        for (int j = 0; j < QPT; ++j) {
          const int t = tq + 8 * j;
          xv[j] = make_float4(0, 0, 0, 0);
          if (in_k && t < p.T) {
            const size_t r = p.rows ? (size_t)p.rows[t] : (size_t)t;
            xv[j] = *reinterpret_cast<const float4*>(p.x + r * p.ld_x + k);
          }
        }
      };
      if (n_iter > 0) fetch(0, xa, wa);  // on their way while the reciprocal roots are worked out
      // reciprocal root mean square of every token's row, from the parts of its sum of squares (index order)
      for (int t = warp; t < p.T; t += 4) {
        const size_t r = p.rows ? (size_t)p.rows[t] : (size_t)t;
        const float* ss = p.sumsq + r * p.n_sumsq;
        float acc = 0.f;
        for (int j0 = 0; j0 < p.n_sumsq; j0 += 32) {  // 32 parts at a time: a fixed tree over the lanes, then the running sum
          float v = (j0 + lane < p.n_sumsq) ? ss[j0 + lane] : 0.f;
          v = warp_sum(v);
          acc += v;
        }
        if (lane == 0) inv_s[t] = 1.0f / sqrtf(acc / (float)p.K + p.eps);
      }
      asm volatile("bar.sync 1, %0;" ::"n"(GD_EPI) : "memory");
      RingPos ring(stages);
      for (int it = 0; it < n_iter && ok; ++it, ring.next()) {
        const int s = ring.s;
        if (it + 1 < n_iter) fetch(it + 1, xb, wb);
        if (it >= stages) {
          // the 128 threads decide together whether to go on: they meet at a barrier in every round
          ok = gd_all_epilogue_threads(mbar_wait(&empty[s], ring.ph ^ 1u, abort_flag, p.error, ERR_GD_ACT));
          if (!ok) break;
        }
        uint8_t* bt = smem + (size_t)s * L::STAGE_BYTES + L::A_STAGE;
#pragma unroll
        for (int j = 0; j < QPT; ++j) {
          const int t = tq + 8 * j;
          if (t < p.T) {
            const float inv = inv_s[t];
            __nv_bfloat162 lo = __floats2bfloat162_rn((wa.x * xa[j].x) * inv, (wa.y * xa[j].y) * inv);
            __nv_bfloat162 hi = __floats2bfloat162_rn((wa.z * xa[j].z) * inv, (wa.w * xa[j].w) * inv);
            uint2 v;
            v.x = *reinterpret_cast<uint32_t*>(&lo);
            v.y = *reinterpret_cast<uint32_t*>(&hi);
            *reinterpret_cast<uint2*>(bt + t * 128 + ((chunk ^ (t & 7)) << 4) + within) = v;
          }
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // generic-proxy writes -> visible to the tensor cores
        asm volatile("bar.sync 1, %0;" ::"n"(GD_EPI) : "memory");
        if (tid == 0) mbar_arrive(&full_x[s]);
        wa = wb;
#pragma unroll
        for (int j = 0; j < QPT; ++j) xa[j] = xb[j];
      }
    }
    // ------------------------------------------------------------------ epilogue
    bool ready = ok;
    if (ready) ready = mbar_wait(acc_ready, 0, abort_flag, p.error, ERR_GD_EPILOGUE);
    ready = __all_sync(0xffffffffu, ready);
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const int row = warp * 32 + lane;  // accumulator lane = weight row of the tile
    const uint32_t lane_addr = tmem_base + ((uint32_t)(warp * 32) << 16);
    if (p.csize == 1 && MODE != GD_RESIDUAL) {
      // one K piece: the accumulator holds the finished sums; lanes write consecutive n
      if (ready) {
#pragma unroll 1
        for (int c0 = 0; c0 < BN; c0 += 16) {
          float v[TILES][16];
#pragma unroll
          for (int a = 0; a < TILES; ++a) {
            if (n_iter > 0) tmem_load16(lane_addr + (uint32_t)(a * BN + c0), v[a]);
            else {
#pragma unroll
              for (int i = 0; i < 16; ++i) v[a][i] = 0.f;
            }
          }
          if (MODE == GD_SWIGLU) {
            const int col = tile * 128 + row;
            if (col < p.N / 2)
#pragma unroll
              for (int i = 0; i < 16; ++i)
                if (c0 + i < p.T) {
                  const float g = v[0][i], u = v[TILES - 1][i];
                  reinterpret_cast<TO*>(p.out)[(size_t)(c0 + i) * p.ld_out + col] = from_f32<TO>((g / (1.0f + expf(-g))) * u);
                }
          } else {
            const int n = w_row0 + row;
            if (n < p.N)
#pragma unroll
              for (int i = 0; i < 16; ++i)
                if (c0 + i < p.T) reinterpret_cast<TO*>(p.out)[(size_t)(c0 + i) * p.ld_out + n] = from_f32<TO>(v[0][i]);
          }
        }
      }
    } else if (!p.in_cluster) {
      // ---- the K pieces meet in global memory: write this piece, count it in, and if it is the last
      // of its tile, add all pieces in index order and run the epilogue for the whole tile
      float* mine = p.parts + (((size_t)tile * p.csize + rank) * 128 + row) * (TILES * t4);
#pragma unroll 1
      for (int c0 = 0; c0 < t4; c0 += 16) {
#pragma unroll
        for (int a = 0; a < TILES; ++a) {
          float v[16];
          if (ready && n_iter > 0) tmem_load16(lane_addr + (uint32_t)(a * BN + c0), v);
          else {
#pragma unroll
            for (int i = 0; i < 16; ++i) v[i] = 0.f;
          }
#pragma unroll
          for (int i = 0; i < 16; i += 4)
            if (c0 + i < t4) *reinterpret_cast<float4*>(mine + a * t4 + c0 + i) = make_float4(v[i], v[i + 1], v[i + 2], v[i + 3]);
        }
      }
      __threadfence();  // the piece is out before it is counted
      asm volatile("bar.sync 1, %0;" ::"n"(GD_EPI) : "memory");
      int* last_flag = issued_slot + 1;
      if (tid == 0) {
        const int old = atomicAdd(&p.counters[tile], 1);
        *last_flag = old == p.csize - 1;
        if (*last_flag) p.counters[tile] = 0;  // ready for the next launch
      }
      asm volatile("bar.sync 1, %0;" ::"n"(GD_EPI) : "memory");
      if (*last_flag) {
        __threadfence();
        const float* tile_parts = p.parts + (size_t)tile * p.csize * 128 * (TILES * t4);
        const int n = w_row0 + row, col = tile * 128 + row;  // this thread finishes accumulator row `row` for every token
        const bool live = MODE == GD_SWIGLU ? col < p.N / 2 : n < p.N;
        for (int t0 = 0; t0 < p.T; t0 += 4) {  // four tokens at a time: 16-byte loads of every piece, eight pieces in flight
          float4 acc[TILES];
#pragma unroll
          for (int a = 0; a < TILES; ++a) acc[a] = make_float4(0, 0, 0, 0);
          for (int s0 = 0; s0 < p.csize && live; s0 += 8) {
            float4 v[8][TILES];
#pragma unroll
            for (int u = 0; u < 8; ++u)
#pragma unroll
              for (int a = 0; a < TILES; ++a)
                v[u][a] = (s0 + u < p.csize) ? __ldcg(reinterpret_cast<const float4*>(tile_parts + ((size_t)(s0 + u) * 128 + row) * (TILES * t4) + a * t4 + t0))
                                             : make_float4(0, 0, 0, 0);
#pragma unroll
            for (int u = 0; u < 8; ++u)
#pragma unroll
              for (int a = 0; a < TILES; ++a) {
                acc[a].x += v[u][a].x; acc[a].y += v[u][a].y; acc[a].z += v[u][a].z; acc[a].w += v[u][a].w;
              }
          }
          const float g4[4] = {acc[0].x, acc[0].y, acc[0].z, acc[0].w};
          const float u4[4] = {acc[TILES - 1].x, acc[TILES - 1].y, acc[TILES - 1].z, acc[TILES - 1].w};
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const int t = t0 + i;
            if (t < p.T) {  // (uniform over the warp)
              float sq = 0.f;
              if (live) {
                if (MODE == GD_SWIGLU) {
                  reinterpret_cast<TO*>(p.out)[(size_t)t * p.ld_out + col] = from_f32<TO>((g4[i] / (1.0f + expf(-g4[i]))) * u4[i]);
                } else if (MODE == GD_RESIDUAL) {
                  float* hp = p.h + (size_t)t * p.ld_h + n;
                  const float xn = *hp + g4[i];
                  *hp = xn;
                  sq = xn * xn;
                } else {
                  reinterpret_cast<TO*>(p.out)[(size_t)t * p.ld_out + n] = from_f32<TO>(g4[i]);
                }
              }
              if (MODE == GD_RESIDUAL) {  // the warp's 32 rows, a fixed tree; the four warps are added below
                sq = warp_sum(sq);
                if (lane == 0) sq_s[warp * t4 + t] = sq;
              }
            }
          }
        }
        if (MODE == GD_RESIDUAL) {
          asm volatile("bar.sync 1, %0;" ::"n"(GD_EPI) : "memory");
          for (int t = tid; t < p.T; t += GD_EPI)  // the tile's part of the rows' sums of squares
            p.sumsq_out[(size_t)t * p.n_sumsq_out + tile] = (sq_s[t] + sq_s[t4 + t]) + (sq_s[2 * t4 + t] + sq_s[3 * t4 + t]);
        }
      }
    } else {
      // ---- send every row of the partial to the CTA that finishes it: asynchronous stores into its
      // shared memory that count their bytes on its `peers_in` barrier, so that neither side needs a
      // fence or an arrival of its own
      gd_cluster_wait();  // (all 128 threads of these warps and the 64 of the others wait below, converged per warp)
      const int owner = row / p.rows_per, r_local = row - owner * p.rows_per;
      const uint32_t dst0 = gd_map(smem_u32(recv), owner) + (uint32_t)(((rank * p.rows_per + r_local) * TILES) * t4) * 4u;
      const uint32_t owner_bar = gd_map(smem_u32(peers_in), owner);
#pragma unroll 1
      for (int c0 = 0; c0 < t4; c0 += 16) {
#pragma unroll
        for (int a = 0; a < TILES; ++a) {
          float v[16];
          if (ready && n_iter > 0) tmem_load16(lane_addr + (uint32_t)(a * BN + c0), v);
          else {  // nothing was computed (an empty K piece, or a role gave up): the owner still counts these bytes
#pragma unroll
            for (int i = 0; i < 16; ++i) v[i] = 0.f;
          }
#pragma unroll
          for (int i = 0; i < 16; i += 4)
            if (c0 + i < t4) gd_store4_async(dst0 + (uint32_t)(a * t4 + c0 + i) * 4u, owner_bar, v[i], v[i + 1], v[i + 2], v[i + 3]);
        }
      }
      const int rows_mine = max(0, min(p.rows_per, 128 - rank * p.rows_per));
      const int n_el = rows_mine * p.T;
      // RESIDUAL: the stream's values that this thread will add to are on their way while the peers' rows arrive
      constexpr int HPRE = 8;
      float hv[HPRE];
      if (MODE == GD_RESIDUAL) {
#pragma unroll
        for (int j = 0; j < HPRE; ++j) {
          const int e = tid + j * GD_EPI;
          hv[j] = 0.f;
          if (e < n_el) {
            const int t = e / rows_mine, r = e - t * rows_mine;
            const int n = w_row0 + rank * p.rows_per + r;
            if (n < p.N) hv[j] = p.h[(size_t)t * p.ld_h + n];
          }
        }
        for (int e = tid; e < p.rows_per * t4; e += GD_EPI) sq_s[e] = 0.f;
      }
      const bool peers_ok = gd_wait_peers(peers_in, p.error);  // every thread sees the phase complete before it reads what arrived
      asm volatile("bar.sync 1, %0;" ::"n"(GD_EPI) : "memory");
      (void)peers_ok;
      // ---- finish this CTA's rows: the K pieces added in index order
      auto finish = [&](int e, bool have_h, float h_old) {
        const int t = e / rows_mine, r = e - t * rows_mine;  // rows fastest: neighbouring threads write neighbouring n
        float d[TILES];
#pragma unroll
        for (int a = 0; a < TILES; ++a) {
          float acc = 0.f;
          for (int src = 0; src < p.csize; ++src) acc += recv[(size_t)((src * p.rows_per + r) * TILES + a) * t4 + t];
          d[a] = acc;
        }
        const int tile_row = rank * p.rows_per + r;
        if (MODE == GD_SWIGLU) {
          const int col = tile * 128 + tile_row;
          if (col < p.N / 2) reinterpret_cast<TO*>(p.out)[(size_t)t * p.ld_out + col] = from_f32<TO>((d[0] / (1.0f + expf(-d[0]))) * d[TILES - 1]);
        } else {
          const int n = w_row0 + tile_row;
          if (n < p.N) {
            if (MODE == GD_RESIDUAL) {
              float* hp = p.h + (size_t)t * p.ld_h + n;
              const float xn = (have_h ? h_old : *hp) + d[0];
              *hp = xn;
              sq_s[r * t4 + t] = xn * xn;
            } else {
              reinterpret_cast<TO*>(p.out)[(size_t)t * p.ld_out + n] = from_f32<TO>(d[0]);
            }
          }
        }
      };
#pragma unroll
      for (int j = 0; j < HPRE; ++j)
        if (tid + j * GD_EPI < n_el) finish(tid + j * GD_EPI, MODE == GD_RESIDUAL, hv[j]);
      for (int e = tid + HPRE * GD_EPI; e < n_el; e += GD_EPI) finish(e, false, 0.f);
      if (MODE == GD_RESIDUAL) {
        asm volatile("bar.sync 1, %0;" ::"n"(GD_EPI) : "memory");
        for (int t = tid; t < p.T; t += GD_EPI) {  // this CTA's part of the rows' sums of squares, rows in index order
          float acc = 0.f;
          for (int r = 0; r < rows_mine; ++r) acc += sq_s[r * t4 + t];
          p.sumsq_out[(size_t)t * p.n_sumsq_out + tile * p.csize + rank] = acc;
        }
      }
    }
    // the stages and tensor memory belong to the products in flight until acc_ready completes
    if (!ready && tid == 0) mbar_drain(acc_ready, 0, p.error);
  }
  if (clustered && warp >= 4) {
    __syncwarp();  // the lanes went different ways; the cluster barrier wants whole warps
    gd_cluster_wait();  // every arrive is matched by a wait
  }
  // a role gave up: let the copies that were issued land (bounded) before the shared memory is given back
  __syncthreads();
  if (*abort_flag && tid == 0) {
    const int issued = *issued_slot;
    for (int it = max(0, issued - stages); it < issued; ++it) mbar_drain(&full[it % stages], (uint32_t)(it / stages) & 1u, p.error);
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(L::TMEM_COLS) : "memory");
}

struct GdPlan {
  int bn, tiles, csize, rows_per, stages, k_tiles, k_per_split, n_ctas_x;
  size_t smem;
};

// splits: K pieces wanted; the plan gives what the kernel will really use (in a cluster: 1, 2, 4 or 8).
bool gd_plan(int N, int K, int T, int mode, int splits, int in_cluster, GdPlan* pl) {
  pl->bn = T > 32 ? 64 : (T > 16 ? 32 : 16);
  pl->tiles = mode == GD_SWIGLU ? 2 : 1;
  pl->k_tiles = (K + BK - 1) / BK;
  int pieces = 1;
  if (in_cluster) {
    // CTAs of a cluster: a power of two up to the portable cluster size of 8 (measured on B200: 16 pieces,
    // a non-portable size, and odd sizes such as 5 run slower than 8 and 4)
    while (pieces * 2 <= std::min(splits, 8) && pieces * 2 <= pl->k_tiles) pieces *= 2;
  } else {
    pieces = std::max(1, std::min(splits, std::min(32, pl->k_tiles)));
  }
  pl->k_per_split = (pl->k_tiles + pieces - 1) / pieces;
  pl->csize = (pl->k_tiles + pl->k_per_split - 1) / pl->k_per_split;
  if (mode == GD_RESIDUAL && pl->csize == 1 && in_cluster) return false;
  pl->rows_per = in_cluster ? (128 + pl->csize - 1) / pl->csize : 128;
  pl->n_ctas_x = (N + 128 * pl->tiles - 1) / (128 * pl->tiles);
  const int stage_bytes = pl->tiles * A_BYTES + pl->bn * BK * 2;
  const int t4 = (T + 3) & ~3;
  const size_t tail = gd_tail_bytes(8, pl->csize, pl->rows_per, pl->tiles, t4, mode, in_cluster);
  // a short ring, so that several CTAs share an SM: weights stream fastest that way (measured on B200)
  int stages = std::min(pl->tiles == 2 ? 3 : 4, std::max(2, pl->k_per_split));
  while (stages > 2 && (size_t)stages * stage_bytes + tail + 1024 > 200 * 1024) --stages;
  pl->stages = stages;
  pl->smem = (size_t)stages * stage_bytes + gd_tail_bytes(stages, pl->csize, pl->rows_per, pl->tiles, t4, mode, in_cluster) + 1024;
  return pl->smem <= 227 * 1024;
}

template <int BN, int TILES, int MODE, typename TO>
int gd_launch(const CUtensorMap& mw, const CUtensorMap& mx, const GdParams& p, const GdPlan& pl, cudaStream_t stream) {
  auto kernel = gemm_decode_kernel<BN, TILES, MODE, TO>;
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024) != cudaSuccess) {
      llm_set_error("gemm_decode: cannot set the kernel's attributes");
      return LLM_ERR_LAUNCH;
    }
    attr_set = true;
  }
  const dim3 grid(pl.n_ctas_x, 1, pl.csize);
  if (p.in_cluster && pl.csize > 1) launch_kernel_cluster(kernel, grid, GD_THREADS, pl.smem, dim3(1, 1, pl.csize), stream, mw, mx, p);
  else launch_kernel(kernel, grid, GD_THREADS, pl.smem, stream, mw, mx, p);
  return LLM_OK;
}

template <int MODE, typename TO>
int gd_dispatch(const CUtensorMap& mw, const CUtensorMap& mx, const GdParams& p, const GdPlan& pl, cudaStream_t stream) {
  constexpr int TILES = MODE == GD_SWIGLU ? 2 : 1;
  if (pl.bn == 16) return gd_launch<16, TILES, MODE, TO>(mw, mx, p, pl, stream);
  if (pl.bn == 32) return gd_launch<32, TILES, MODE, TO>(mw, mx, p, pl, stream);
  return gd_launch<64, TILES, MODE, TO>(mw, mx, p, pl, stream);
}

}  // namespace

// K pieces (= CTAs per cluster) that llm_gemm_decode will use for these sizes and this wish, 0 if it
// does not take them.
extern "C" int llm_gemm_decode_splits(int N, int K, int T, int mode, int splits, int in_cluster) {
  GdPlan pl;
  if (T < 1 || T > 64 || N < 1 || K < 1 || mode < 0 || mode > 2) return 0;
  return gd_plan(N, K, T, mode, splits, in_cluster, &pl) ? pl.csize : 0;
}

// Floats of scratch that llm_gemm_decode needs when the K pieces meet in global memory (the
// counters beside it: one int per tile, llm_gemm_decode_tiles of them, zero before the first use).
extern "C" long long llm_gemm_decode_scratch_floats(int N, int K, int T, int mode, int splits) {
  GdPlan pl;
  if (T < 1 || T > 64 || N < 1 || K < 1 || mode < 0 || mode > 2 || !gd_plan(N, K, T, mode, splits, 0, &pl)) return 0;
  return (long long)pl.n_ctas_x * pl.csize * 128 * pl.tiles * ((T + 3) & ~3);
}
extern "C" int llm_gemm_decode_tiles(int N, int mode) { return (N + (mode == GD_SWIGLU ? 256 : 128) - 1) / (mode == GD_SWIGLU ? 256 : 128); }

// out/h[t, n] (see the modes above) from W [N, K] bf16 (row stride ldw) and T <= 64 tokens' activations:
//   x_bf16 != null: bf16 rows [T, K] (row stride ld_x); else the norm: x_f32 rows (stride ld_x, row of
//   token t = rows ? rows[t] : t), sumsq [rows of x][n_sumsq], norm_w [K], eps.
// mode 0 PLAIN: out float32 (out_dtype 0) or bf16 (1) [T, N] (stride ld_out);
// mode 1 RESIDUAL: h float32 [T, N] (stride ld_out) updated in place, sumsq_out [T][n_sumsq_out] with
//        n_sumsq_out = tiles of 128 rows x llm_gemm_decode_splits(...) in a cluster, tiles of 128 rows otherwise;
// mode 2 SWIGLU: W rows are blocks of 128 gate rows followed by the 128 matching up rows (N counts both),
//        out bf16 [T, N / 2].
// parts == null: the K pieces meet inside a thread-block cluster; else in `parts`
// (parts_floats >= llm_gemm_decode_scratch_floats floats) with `counters` (llm_gemm_decode_tiles ints, zero, left zero).
extern "C" int llm_gemm_decode(const void* w, long long ldw, int N, int K, int T, const void* x_bf16, const float* x_f32,
                               long long ld_x, const float* sumsq, int n_sumsq, const float* norm_w, float eps, const int* rows,
                               int mode, void* out, long long ld_out, int out_dtype, float* sumsq_out, int n_sumsq_out, int splits,
                               float* parts, long long parts_floats, int* counters, cudaStream_t stream) {
  if (T == 0 || N == 0) return LLM_OK;
  LLM_REQUIRE(T >= 1 && T <= 64 && N > 0 && K > 0 && K % 8 == 0 && ldw % 8 == 0, "gemm_decode: bad sizes T=%d N=%d K=%d", T, N, K);
  LLM_REQUIRE(mode >= GD_PLAIN && mode <= GD_SWIGLU, "gemm_decode: unknown mode %d", mode);
  LLM_REQUIRE((x_bf16 != nullptr) != (x_f32 != nullptr), "gemm_decode: activations come as bf16 rows or as a norm's inputs, one of the two");
  auto al = [](const void* ptr) { return (reinterpret_cast<uintptr_t>(ptr) & 15u) == 0; };
  LLM_REQUIRE(al(w) && al(out), "gemm_decode: w and out must be 16-byte aligned");
  if (x_f32) LLM_REQUIRE(sumsq && n_sumsq >= 1 && norm_w && al(x_f32) && al(norm_w) && ld_x % 4 == 0, "gemm_decode: the norm needs sums of squares, a weight and aligned rows");
  else LLM_REQUIRE(al(x_bf16) && ld_x % 8 == 0 && rows == nullptr, "gemm_decode: bf16 rows must be 16-byte aligned, without a row list");
  LLM_REQUIRE(mode != GD_SWIGLU || (N % 256 == 0 && out_dtype == LLM_BF16), "gemm_decode: SwiGLU needs gate|up blocks of 128 rows and a bf16 output");
  LLM_REQUIRE(mode != GD_RESIDUAL || (sumsq_out != nullptr && out_dtype == LLM_F32), "gemm_decode: the residual form needs float32 rows and a place for the sums of squares");
  LLM_REQUIRE(out_dtype == LLM_F32 || out_dtype == LLM_BF16, "gemm_decode: unknown out dtype %d", out_dtype);
  LLM_REQUIRE(error_word() != nullptr && encode_fn() != nullptr, "gemm_decode: no error word or no tensor-map encoder");
  const int in_cluster = parts == nullptr;
  LLM_REQUIRE(in_cluster || counters != nullptr, "gemm_decode: scratch for the K pieces comes with counters");
  GdPlan pl;
  LLM_REQUIRE(gd_plan(N, K, T, mode, splits, in_cluster, &pl), "gemm_decode: no plan for N=%d K=%d T=%d mode=%d splits=%d", N, K, T, mode, splits);
  LLM_REQUIRE(in_cluster || parts_floats >= (long long)pl.n_ctas_x * pl.csize * 128 * pl.tiles * ((T + 3) & ~3),
              "gemm_decode: the scratch for the K pieces is too small (%lld floats)", parts_floats);
  const int want_parts = in_cluster ? pl.n_ctas_x * pl.csize : pl.n_ctas_x;
  LLM_REQUIRE(mode != GD_RESIDUAL || n_sumsq_out == want_parts, "gemm_decode: sumsq_out must hold %d parts a token, not %d", want_parts, n_sumsq_out);
  CUtensorMap mw, mx;
  LLM_REQUIRE(tensor_map_for(w, N, K, ldw, BM, &mw), "gemm_decode: cuTensorMapEncodeTiled failed for the weights");
  if (x_bf16) LLM_REQUIRE(tensor_map_for(x_bf16, T, K, ld_x, pl.bn, &mx), "gemm_decode: cuTensorMapEncodeTiled failed for the activations");
  else mx = mw;
  GdParams p = {};
  p.N = N; p.K = K; p.T = T; p.k_tiles = pl.k_tiles; p.k_per_split = pl.k_per_split; p.csize = pl.csize; p.rows_per = pl.rows_per;
  p.stages = pl.stages;
  p.x = x_f32; p.ld_x = ld_x; p.sumsq = sumsq; p.n_sumsq = n_sumsq; p.norm_w = norm_w; p.eps = eps; p.rows = rows;
  p.out = out; p.ld_out = ld_out; p.h = (float*)out; p.ld_h = ld_out; p.sumsq_out = sumsq_out; p.n_sumsq_out = n_sumsq_out;
  p.in_cluster = in_cluster; p.parts = parts; p.counters = counters;
  p.error = error_word();
  int rc;
  if (mode == GD_SWIGLU) rc = gd_dispatch<GD_SWIGLU, bf16>(mw, mx, p, pl, stream);
  else if (mode == GD_RESIDUAL) rc = gd_dispatch<GD_RESIDUAL, float>(mw, mx, p, pl, stream);
  else if (out_dtype == LLM_F32) rc = gd_dispatch<GD_PLAIN, float>(mw, mx, p, pl, stream);
  else rc = gd_dispatch<GD_PLAIN, bf16>(mw, mx, p, pl, stream);
  if (rc != LLM_OK) return rc;
  LLM_CHECK_LAUNCH("gemm_decode");
  return LLM_OK;
}
