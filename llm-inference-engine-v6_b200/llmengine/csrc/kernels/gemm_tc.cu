// bfloat16 matrix product on the 5th-generation tensor cores (tcgen05), operands brought to shared
// memory by TMA, float32 accumulator in tensor memory.
//
//   D[ra, rb] = sum_k A[ra, k] * B[rb, k]        A: [RA, K], B: [RB, K], both with k contiguous
//
// Both uses of the engine are this one kernel:
//   * many tokens (prompt portions): A = activations [tokens, K], B = weights [N, K],
//     out[token, n] = D[token, n]; tiles of 128 tokens x BN outputs;
//   * few tokens (decoding): A = weights [N, K] (128 weight rows fill the 128 accumulator lanes),
//     B = activations [tokens <= BN, K], out[token, n] = D[n, token] ("swapped"); the K range can be
//     cut into splits, each writing its own float32 partial [split, tokens, N]; the consumer adds
//     the partials in index order, so the result does not depend on timing.
//
// One CTA computes one output tile: warp 0 lane 0 issues the TMA loads into a ring of stages,
// warp 1 lane 0 issues tcgen05.mma (one instruction covers 128 x BN x 16) and commits each
// stage back to the producer, all four warps read the accumulator with tcgen05.ld and store it.
// Every wait on an mbarrier is bounded: after about a second it records an error code, the
// other roles see the abort flag, outstanding copies are waited for (bounded too), tensor memory is
// freed and the kernel returns; the host reports the code.
//
// The reference computes the same products with a scalar loop (matmul_f32, src/kernels.cpp:33-57).
#include "tc_common.cuh"

#include <type_traits>

int* llm_tc_error_word() {
  // One int of device memory per process for the kernels' error codes, made at first use.
  static int* word = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    if (cudaMalloc(&word, sizeof(int)) == cudaSuccess) cudaMemset(word, 0, sizeof(int));
    else word = nullptr;
  });
  return word;
}


namespace {

// Walks the (tile, k-block) pairs of a persistent CTA: tiles first, first + step, ...; inside a tile
// the k-blocks in order. The one thread that issues copies or products has a k-block's time for
// each of its iterations, so the loop holds no division: the tile's rows are worked out once a tile.
struct TileWalk {
  int tile, kt, a_row0, b_row0;
  int step, k_tiles, m_tiles, a_rows, b_rows, a_off, b_off;
  __device__ __forceinline__ TileWalk(int first, int step_, int k_tiles_, int m_tiles_, int a_rows_, int b_rows_, int a_off_ = 0,
                                      int b_off_ = 0)
      : kt(0), step(step_), k_tiles(k_tiles_), m_tiles(m_tiles_), a_rows(a_rows_), b_rows(b_rows_), a_off(a_off_), b_off(b_off_) {
    set_tile(first);
  }
  __device__ __forceinline__ void set_tile(int t) {
    tile = t;
    const int n = t / m_tiles;
    a_row0 = (t - n * m_tiles) * a_rows + a_off;
    b_row0 = n * b_rows + b_off;
  }
  __device__ __forceinline__ void next() {
    if (++kt == k_tiles) {
      kt = 0;
      set_tile(tile + step);
    }
  }
};

template <typename TO>
__device__ __forceinline__ void store_row16(TO* dst, const float* v, int valid, bool aligned);

template <>
__device__ __forceinline__ void store_row16<float>(float* dst, const float* v, int valid, bool aligned) {
  if (valid == 16 && aligned) {
#pragma unroll
    for (int i = 0; i < 4; ++i) reinterpret_cast<float4*>(dst)[i] = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
  } else {
    for (int i = 0; i < valid; ++i) dst[i] = v[i];
  }
}

template <>
__device__ __forceinline__ void store_row16<bf16>(bf16* dst, const float* v, int valid, bool aligned) {
  if (valid == 16 && aligned) {
    uint32_t p[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      __nv_bfloat162 t = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
      p[i] = *reinterpret_cast<uint32_t*>(&t);
    }
    reinterpret_cast<uint4*>(dst)[0] = make_uint4(p[0], p[1], p[2], p[3]);
    reinterpret_cast<uint4*>(dst)[1] = make_uint4(p[4], p[5], p[6], p[7]);
  } else {
    for (int i = 0; i < valid; ++i) dst[i] = __float2bfloat16_rn(v[i]);
  }
}

// v += dst (float32 outputs that are added into what is there, e.g. the residual stream).
template <typename TO>
__device__ __forceinline__ void add_from16(const TO* dst, float* v, int valid, bool aligned) {}
template <>
__device__ __forceinline__ void add_from16<float>(const float* dst, float* v, int valid, bool aligned) {
  if (valid == 16 && aligned) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float4 t = reinterpret_cast<const float4*>(dst)[i];
      v[4 * i] += t.x; v[4 * i + 1] += t.y; v[4 * i + 2] += t.z; v[4 * i + 3] += t.w;
    }
  } else {
    for (int i = 0; i < valid; ++i) v[i] += dst[i];
  }
}

// A thread's accumulator row (BN columns from tensor-memory address `acc`) added into row `dst_row` of a
// float32 matrix: out[c] += acc[c] for columns col0 .. col0 + BN - 1 below n_cols. The old values of 64
// columns are requested together before the accumulator is read: fetched 16 at a time, behind each
// tensor-memory load, they would be BN / 16 dependent trips to L2.
template <int BN>
__device__ __forceinline__ void add_accumulator_row(uint32_t acc, float* dst_row, bool row_ok, int col0, int n_cols) {
  constexpr int G = BN >= 64 ? 64 : 16;
#pragma unroll 1
  for (int c0 = 0; c0 < BN; c0 += G) {
    float old[G];
#pragma unroll
    for (int q = 0; q < G / 16; ++q) {
      const int c = col0 + c0 + 16 * q;
      float* dst = dst_row + c;
#pragma unroll
      for (int i = 0; i < 16; ++i) old[16 * q + i] = 0.f;
      if (row_ok && c < n_cols) add_from16<float>(dst, old + 16 * q, min(16, n_cols - c), (reinterpret_cast<uintptr_t>(dst) & 15u) == 0);
    }
#pragma unroll
    for (int q = 0; q < G / 16; ++q) {
      float v[16];
      tmem_load16(acc + (uint32_t)(c0 + 16 * q), v);
      const int c = col0 + c0 + 16 * q;
      if (row_ok && c < n_cols) {
#pragma unroll
        for (int i = 0; i < 16; ++i) v[i] += old[16 * q + i];
        float* dst = dst_row + c;
        store_row16<float>(dst, v, min(16, n_cols - c), (reinterpret_cast<uintptr_t>(dst) & 15u) == 0);
      }
    }
  }
}

// What the swapped form (few tokens) can do behind its product, so that no kernel of its own has to:
//   EPI_MEET   the K splits of a tile of outputs meet: each CTA writes its partial sums, the one that
//              arrives last adds them in index order, adds the sum into the float32 residual stream
//              h, writes bf16(next_w * h) for the product that follows the next norm, and this
//              tile's part of every token's sum of squares of the new stream (the norm's 1/rms is
//              then applied by whoever consumes that product: a per-token scalar commutes with it);
//   EPI_SCALE  every token's results are divided by the root mean square that the parts of its sum
//              of squares give (the norm before this product, whose weight is already in the operand).
enum : int { EPI_NONE = 0, EPI_MEET = 1, EPI_SCALE = 2 };
struct EpiArgs {
  float* h = nullptr; long long ld_h = 0;              // MEET: residual stream [tokens, ld_h]
  const float* next_w = nullptr;                       // MEET: weight of the norm that follows (null: no scaled copy)
  bf16* scaled = nullptr; long long ld_scaled = 0;     // MEET: bf16(next_w * h) [tokens, ld_scaled]
  float* sumsq = nullptr; int n_sumsq = 0;             // MEET: [tokens, n_sumsq], column = this tile of outputs
  int* counters = nullptr;                             // MEET: one per tile of outputs, zero between launches
  const float* in_sumsq = nullptr; int n_in_sumsq = 0; // SCALE: [tokens, n_in_sumsq] parts of the sums of squares
  float inv_dim = 0.f, eps = 0.f;                      // SCALE: 1 / sqrt(sum * inv_dim + eps)
};

// grid: (tiles of A rows, tiles of B rows, K splits); block: 128 threads.
// SWIGLU (token tiles of 256 outputs only): the weight rows come in blocks of 256 = 128 rows of the
// gate projection followed by the 128 matching rows of the up projection, so one accumulator tile
// holds both; the epilogue writes silu(gate) * up, 128 columns per tile, and the 2x wider
// intermediate never goes to memory.
template <int BN, bool SWAP, typename TO, bool SWIGLU = false, int EPI = EPI_NONE>
__global__ void __launch_bounds__(128)
    gemm_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, TO* __restrict__ out,
                   int RA, int RB, int k_tiles, int k_tiles_per_split, long long ldo, long long split_stride, int stages,
                   int* __restrict__ error_out, const EpiArgs epi, int add_into) {
  static_assert(EPI == EPI_NONE || (SWAP && !SWIGLU && BN <= 64), "the epilogue options belong to the swapped form with few tokens");
  __shared__ float s_tok[EPI == EPI_NONE ? 1 : 4 * 64];  // SCALE: 1/rms of the tokens; MEET: the warps' parts of the sums of squares
  __shared__ int s_last;
  constexpr int B_BYTES = BN * BK * 2;
  constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  constexpr int TMEM_COLS = BN < 32 ? 32 : BN;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + (size_t)stages * STAGE_BYTES);
  uint64_t* empty = full + stages;
  uint64_t* acc_ready = empty + stages;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_ready + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int a_row0 = blockIdx.x * BM, b_row0 = blockIdx.y * BN;
  const int kt_begin = blockIdx.z * k_tiles_per_split;
  const int kt_end = min(k_tiles, kt_begin + k_tiles_per_split);
  const int n_iter = kt_end - kt_begin;

  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    mbar_init(acc_ready, 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_slot;

  dep_launch();
  if (warp == 0 && lane == 0) {
    // ---------------------------------------------------------------- producer: TMA loads
    // The weight operand is not produced by the stream: its first tiles are requested before the
    // wait on the previous kernel, the activation tiles after it.
    const CUtensorMap* weight_map = SWAP ? &map_a : &map_b;
    const CUtensorMap* act_map = SWAP ? &map_b : &map_a;
    const int weight_row0 = SWAP ? a_row0 : b_row0, act_row0 = SWAP ? b_row0 : a_row0;
    constexpr int WEIGHT_OFF = SWAP ? 0 : A_BYTES, ACT_OFF = SWAP ? A_BYTES : 0;
    const int early = min(stages, n_iter);
    for (int it = 0; it < early; ++it) {
      mbar_expect_tx(&full[it], STAGE_BYTES);
      tma_load_2d(smem + (size_t)it * STAGE_BYTES + WEIGHT_OFF, weight_map, (kt_begin + it) * BK, weight_row0, &full[it]);
    }
    dep_wait();
    for (int it = 0; it < early; ++it)
      tma_load_2d(smem + (size_t)it * STAGE_BYTES + ACT_OFF, act_map, (kt_begin + it) * BK, act_row0, &full[it]);
    int issued = early;
    bool ok = true;
    RingPos ring(stages, 0, 1u);  // iteration `stages` is the first to use a stage again
    for (int it = early; it < n_iter && ok; ++it, ring.next()) {
      const int s = ring.s;
      ok = mbar_wait(&empty[s], ring.ph ^ 1u, abort_flag, error_out, ERR_PRODUCER);
      if (!ok) break;
      uint8_t* sa = smem + (size_t)s * STAGE_BYTES;
      mbar_expect_tx(&full[s], STAGE_BYTES);
      tma_load_2d(sa, &map_a, (kt_begin + it) * BK, a_row0, &full[s]);
      tma_load_2d(sa + A_BYTES, &map_b, (kt_begin + it) * BK, b_row0, &full[s]);
      issued = it + 1;
    }
    if (!ok || *abort_flag) {
      // wait (bounded) for the copies already issued, so that none lands after the CTA has left
      const int first = issued > stages ? issued - stages : 0;
      for (int it = first; it < issued; ++it) {
        const long long t0 = clock64();
        while (!mbar_try_wait(&full[it % stages], (uint32_t)(it / stages) & 1u)) {
          if (clock64() - t0 > WAIT_CYCLES) {
            atomicCAS(error_out, 0, ERR_DRAIN);
            break;
          }
        }
      }
    }
  } else if (warp == 1 && lane == 0) {
    // ---------------------------------------------------------------- tensor-core issue
    constexpr uint32_t idesc = instr_desc(BN);
    bool ok = true;
    RingPos ring(stages);
    for (int it = 0; it < n_iter && ok; ++it, ring.next()) {
      const int s = ring.s;
      ok = mbar_wait(&full[s], ring.ph, abort_flag, error_out, ERR_MMA);
      if (!ok) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const uint32_t sa = smem_u32(smem + (size_t)s * STAGE_BYTES);
      const uint64_t da = smem_desc_sw128(sa), db = smem_desc_sw128(sa + A_BYTES);
#pragma unroll
      for (int k = 0; k < BK / 16; ++k)  // 16 bf16 = 32 bytes further along the swizzled row: +2 in the address field
        mma_f16(tmem_base, da + (uint64_t)(2 * k), db + (uint64_t)(2 * k), idesc, (it > 0 || k > 0) ? 1u : 0u);
      mma_commit(&empty[s]);  // arrives when the MMAs above have read the stage
    }
    mma_commit(acc_ready);  // also when a wait gave up: arrives once every product issued above has finished
  }
  __syncwarp();
  dep_wait();  // every thread: no global write before the previous kernels have finished

  // ------------------------------------------------------------------ epilogue: all four warps
  if (EPI == EPI_SCALE) {
    if ((int)threadIdx.x < RB - b_row0 && threadIdx.x < BN) {
      const float* part = epi.in_sumsq + (size_t)(b_row0 + threadIdx.x) * epi.n_in_sumsq;
      float sum = 0.f;
      for (int j = 0; j < epi.n_in_sumsq; ++j) sum += part[j];  // index order
      s_tok[threadIdx.x] = 1.0f / sqrtf(sum * epi.inv_dim + epi.eps);
    }
    __syncthreads();
  }
  bool ready = n_iter > 0;
  if (ready) ready = mbar_wait(acc_ready, 0, abort_flag, error_out, ERR_EPILOGUE);
  ready = __all_sync(0xffffffffu, ready);  // a warp reads tensor memory together or not at all
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  TO* o = out + (size_t)blockIdx.z * split_stride;
  const int ra = a_row0 + warp * 32 + lane;
  if (SWIGLU) {
    if (ready) {
#pragma unroll 1
      for (int c0 = 0; c0 < BN / 2; c0 += 16) {
        float gv[16], uv[16];
        tmem_load16(tmem_base + ((uint32_t)(warp * 32) << 16) + (uint32_t)c0, gv);
        tmem_load16(tmem_base + ((uint32_t)(warp * 32) << 16) + (uint32_t)(c0 + BN / 2), uv);
#pragma unroll
        for (int i = 0; i < 16; ++i) gv[i] = (gv[i] / (1.0f + expf(-gv[i]))) * uv[i];
        const int col0 = b_row0 / 2 + c0;  // column of the activation matrix [tokens, RB / 2]
        if (ra < RA && col0 < RB / 2) {
          TO* dst = o + (size_t)ra * ldo + col0;
          store_row16<TO>(dst, gv, min(16, RB / 2 - col0), (reinterpret_cast<uintptr_t>(dst) & 15u) == 0);
        }
      }
    }
  } else if (!SWAP && add_into && ready) {
    if constexpr (!SWAP && std::is_same<TO, float>::value)  // out += product
      add_accumulator_row<BN>(tmem_base + ((uint32_t)(warp * 32) << 16), reinterpret_cast<float*>(o) + (size_t)ra * ldo, ra < RA, b_row0, RB);
  } else if (ready || n_iter == 0) {
#pragma unroll 1
    for (int c0 = 0; c0 < BN; c0 += 16) {
      float v[16];
      if (n_iter > 0) {
        tmem_load16(tmem_base + ((uint32_t)(warp * 32) << 16) + (uint32_t)c0, v);
      } else {
#pragma unroll
        for (int i = 0; i < 16; ++i) v[i] = 0.f;
      }
      const int rb0 = b_row0 + c0;
      if (!SWAP) {
        if (ra < RA && rb0 < RB) {
          TO* dst = o + (size_t)ra * ldo + rb0;
          const bool aligned = (reinterpret_cast<uintptr_t>(dst) & 15u) == 0;
          store_row16<TO>(dst, v, min(16, RB - rb0), aligned);
        }
      } else {
        if (ra < RA) {
#pragma unroll
          for (int i = 0; i < 16; ++i)
            if (rb0 + i < RB) {
              const float r = EPI == EPI_SCALE ? v[i] * s_tok[c0 + i] : v[i];
              o[(size_t)(rb0 + i) * ldo + ra] = from_f32<TO>(r);  // lanes write consecutive addresses
            }
        }
      }
    }
  }
  if (EPI == EPI_MEET) {
    // The K splits of this tile of outputs meet. Every CTA has written its partial sums above; the
    // one that counts itself last (also one that gave up: nobody may wait for it) finishes the tile.
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) s_last = atomicAdd(&epi.counters[blockIdx.x], 1) == (int)gridDim.z - 1;
    __syncthreads();
    if (s_last) {
      __threadfence();
      const int splits = (int)gridDim.z, n_tok = min(RB, BN);
      float acc[BN];
#pragma unroll
      for (int t = 0; t < BN; ++t) acc[t] = 0.f;
      if (ra < RA) {
        // a round of 64 loads is issued before any of them is added: added one by one as they come
        // they would be so many dependent trips to L2
        constexpr int U = BN <= 16 ? 4 : (BN <= 32 ? 2 : 1);
        const float* part = reinterpret_cast<const float*>(out) + ra;
        for (int z0 = 0; z0 < splits; z0 += U) {
          float v[U][BN];
#pragma unroll
          for (int u = 0; u < U; ++u)
#pragma unroll
            for (int t = 0; t < BN; ++t)
              v[u][t] = (z0 + u < splits && t < n_tok) ? __ldcg(part + (size_t)(z0 + u) * split_stride + (size_t)t * ldo) : 0.f;
#pragma unroll
          for (int u = 0; u < U; ++u)  // index order; the zeros of a short last round change nothing
#pragma unroll
            for (int t = 0; t < BN; ++t) acc[t] += v[u][t];
        }
      }
      const float wn = (epi.next_w != nullptr && ra < RA) ? epi.next_w[ra] : 0.f;
#pragma unroll
      for (int t = 0; t < BN; ++t) {
        float sq = 0.f;
        if (t < n_tok && ra < RA) {
          float* hp = epi.h + (size_t)t * epi.ld_h + ra;
          const float hn = *hp + acc[t];
          *hp = hn;
          if (epi.scaled != nullptr) epi.scaled[(size_t)t * epi.ld_scaled + ra] = __float2bfloat16_rn(hn * wn);
          sq = hn * hn;
        }
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, off);
        if (lane == 0) s_tok[warp * 64 + t] = sq;
      }
      __syncthreads();
      if ((int)threadIdx.x < n_tok && epi.sumsq != nullptr)
        epi.sumsq[(size_t)threadIdx.x * epi.n_sumsq + blockIdx.x] =
            (s_tok[threadIdx.x] + s_tok[64 + threadIdx.x]) + (s_tok[128 + threadIdx.x] + s_tok[192 + threadIdx.x]);
      if (threadIdx.x == 0) epi.counters[blockIdx.x] = 0;  // left at zero for the next launch
    }
  }
  // a role gave up: products that were issued may still run; the stages and tensor memory are theirs until then
  if (!ready && n_iter > 0 && threadIdx.x == 0) mbar_drain(acc_ready, 0, error_out);
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 0) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
}

// Persistent form of the token-tile product with 256 outputs a tile: one CTA per SM walks the tiles
// blockIdx.x, blockIdx.x + gridDim.x, ... (tiles of one weight column block are neighbours, so the
// CTAs that run together share it in L2). The accumulator is double: tensor memory holds two tiles
// of 256 columns, and the four epilogue warps drain one while the tensor cores fill the other, so
// the tensor pipe does not idle during the 64-128 KB write-out and the ring of operand stages never
// runs empty between tiles. Warps 0-3: epilogue (a warp reads its own 32 accumulator lanes); warp 4
// lane 0: TMA; warp 5 lane 0: tcgen05.mma. Waits are bounded as in the one-tile kernel.
constexpr int PERSIST_THREADS = 192;

template <typename TO, bool SWIGLU, int BN>
__global__ void __launch_bounds__(PERSIST_THREADS)
    gemm_tc_persistent_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                              TO* __restrict__ out, int RA, int RB, int k_tiles, long long ldo, int stages, int m_tiles,
                              int n_tiles, int* __restrict__ error_out, int add_into) {
  static_assert(BN == 256 || BN == 192, "two accumulators of BN columns, 256 columns apart, in 512 columns of tensor memory");
  static_assert(!SWIGLU || BN == 256, "the gate|up blocks are 256 rows");
  constexpr int ACC_STRIDE = 256;  // tensor-memory columns from one accumulator to the other
  constexpr int B_BYTES = BN * BK * 2;
  constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + (size_t)stages * STAGE_BYTES);
  uint64_t* empty = full + stages;
  uint64_t* acc_full = empty + stages;   // [2] the tensor cores have finished a tile in accumulator b
  uint64_t* acc_empty = acc_full + 2;    // [2] the epilogue warps have read accumulator b
  uint64_t* mma_done = acc_empty + 2;    // every product this CTA issued has finished (committed last, also after giving up)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(mma_done + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  int* issued_slot = const_cast<int*>(abort_flag) + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int total = m_tiles * n_tiles;
  const int my_tiles = (int)blockIdx.x < total ? (total - 1 - (int)blockIdx.x) / (int)gridDim.x + 1 : 0;

  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&acc_full[b], 1);
      mbar_init(&acc_empty[b], 4);  // one arrival per epilogue warp
    }
    mbar_init(mma_done, 1);
    *abort_flag = 0;
    *issued_slot = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(512) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_slot;

  dep_launch();
  if (warp == 4) {
    if (lane == 0) {
      // ---------------------------------------------------------------- producer: TMA loads
      // The weight tiles of the first stages are asked for before the wait on the previous kernel.
      const long long n_iter = (long long)my_tiles * k_tiles;
      const int early = (int)(n_iter < stages ? n_iter : stages);
      TileWalk first(blockIdx.x, gridDim.x, k_tiles, m_tiles, BM, BN), walk = first;
      for (int it = 0; it < early; ++it, first.next()) {
        mbar_expect_tx(&full[it], STAGE_BYTES);
        tma_load_2d(smem + (size_t)it * STAGE_BYTES + A_BYTES, &map_b, first.kt * BK, first.b_row0, &full[it]);
      }
      dep_wait();
      for (int it = 0; it < early; ++it, walk.next())
        tma_load_2d(smem + (size_t)it * STAGE_BYTES, &map_a, walk.kt * BK, walk.a_row0, &full[it]);
      long long issued = early;
      bool ok = true;
      RingPos ring(stages, 0, 1u);  // iteration `stages` is the first to use a stage again
      for (long long it = early; it < n_iter && ok; ++it, ring.next(), walk.next()) {
        const int s = ring.s;
        ok = mbar_wait(&empty[s], ring.ph ^ 1u, abort_flag, error_out, ERR_PRODUCER);
        if (!ok) break;
        uint8_t* sa = smem + (size_t)s * STAGE_BYTES;
        mbar_expect_tx(&full[s], STAGE_BYTES);
        tma_load_2d(sa, &map_a, walk.kt * BK, walk.a_row0, &full[s]);
        tma_load_2d(sa + A_BYTES, &map_b, walk.kt * BK, walk.b_row0, &full[s]);
        issued = it + 1;
      }
      if (!ok || *abort_flag) {
        // wait (bounded) for the copies already issued, so that none lands after the CTA has left
        const long long first = issued > stages ? issued - stages : 0;
        for (long long it = first; it < issued; ++it) {
          const long long t0 = clock64();
          while (!mbar_try_wait(&full[it % stages], (uint32_t)(it / stages) & 1u)) {
            if (clock64() - t0 > WAIT_CYCLES) {
              atomicCAS(error_out, 0, ERR_DRAIN);
              break;
            }
          }
        }
      }
    }
  } else if (warp == 5) {
    if (lane == 0) {
      // ---------------------------------------------------------------- tensor-core issue
      constexpr uint32_t idesc = instr_desc(BN);
      bool ok = true;
      RingPos ring(stages);
      for (int t = 0; t < my_tiles && ok; ++t) {
        const int b = t & 1;
        if (t >= 2) {  // the epilogue of the tile that used this accumulator two tiles ago
          ok = mbar_wait(&acc_empty[b], (uint32_t)((t >> 1) - 1) & 1u, abort_flag, error_out, ERR_MMA);
          if (!ok) break;
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        }
        const uint32_t acc = tmem_base + (uint32_t)(b * ACC_STRIDE);
        for (int kt = 0; kt < k_tiles && ok; ++kt, ring.next()) {
          const int s = ring.s;
          ok = mbar_wait(&full[s], ring.ph, abort_flag, error_out, ERR_MMA);
          if (!ok) break;
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const uint32_t sa = smem_u32(smem + (size_t)s * STAGE_BYTES);
          const uint64_t da = smem_desc_sw128(sa), db = smem_desc_sw128(sa + A_BYTES);
#pragma unroll
          for (int k = 0; k < BK / 16; ++k)
            mma_f16(acc, da + (uint64_t)(2 * k), db + (uint64_t)(2 * k), idesc, (kt > 0 || k > 0) ? 1u : 0u);
          mma_commit(&empty[s]);
        }
        if (ok) mma_commit(&acc_full[b]);
      }
      mma_commit(mma_done);
    }
  } else {
    // ------------------------------------------------------------------ epilogue: warps 0-3
    dep_wait();  // no global write before the previous kernels have finished
    bool ok = true;
    for (int t = 0; t < my_tiles; ++t) {
      const int b = t & 1;
      ok = mbar_wait(&acc_full[b], (uint32_t)(t >> 1) & 1u, abort_flag, error_out, ERR_EPILOGUE);
      ok = __all_sync(0xffffffffu, ok);  // a warp reads tensor memory together or not at all
      if (!ok) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const int tile = blockIdx.x + t * gridDim.x;
      const int a_row0 = (tile % m_tiles) * BM, b_row0 = (tile / m_tiles) * BN;
      const int ra = a_row0 + warp * 32 + lane;
      const uint32_t acc = tmem_base + ((uint32_t)(warp * 32) << 16) + (uint32_t)(b * ACC_STRIDE);
      if (SWIGLU) {
#pragma unroll 1
        for (int c0 = 0; c0 < BN / 2; c0 += 16) {
          float gv[16], uv[16];
          tmem_load16(acc + (uint32_t)c0, gv);
          tmem_load16(acc + (uint32_t)(c0 + BN / 2), uv);
#pragma unroll
          for (int i = 0; i < 16; ++i) gv[i] = (gv[i] / (1.0f + expf(-gv[i]))) * uv[i];
          const int col0 = b_row0 / 2 + c0;  // column of the activation matrix [tokens, RB / 2]
          if (ra < RA && col0 < RB / 2) {
            TO* dst = out + (size_t)ra * ldo + col0;
            store_row16<TO>(dst, gv, min(16, RB / 2 - col0), (reinterpret_cast<uintptr_t>(dst) & 15u) == 0);
          }
        }
      } else if (add_into) {
        if constexpr (std::is_same<TO, float>::value)  // out += product
          add_accumulator_row<BN>(acc, reinterpret_cast<float*>(out) + (size_t)ra * ldo, ra < RA, b_row0, RB);
      } else {
#pragma unroll 1
        for (int c0 = 0; c0 < BN; c0 += 16) {
          float v[16];
          tmem_load16(acc + (uint32_t)c0, v);
          const int rb0 = b_row0 + c0;
          if (ra < RA && rb0 < RB) {
            TO* dst = out + (size_t)ra * ldo + rb0;
            store_row16<TO>(dst, v, min(16, RB - rb0), (reinterpret_cast<uintptr_t>(dst) & 15u) == 0);
          }
        }
      }
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[b]);
    }
    // Tensor memory and the stages belong to the products in flight until the last of them is done
    // (at once when every tile was drained above; what counts when a role gave up).
    if (threadIdx.x == 0) mbar_drain(mma_done, 0, error_out);
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 0) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512) : "memory");
  }
}

// ---------------------------------------------------------------------------------------------
// CTA pairs (cta_group::2). Two CTAs of a cluster, on neighbouring SMs, compute one 256 x 256 output
// tile with ONE tcgen05.mma stream issued by the even CTA (the leader): the instruction reads the
// 128 A rows that each CTA holds in its own shared memory and the B tile half from each of them
// (128 of the 256 weight rows), and writes 128 accumulator rows into each CTA's tensor memory. Per
// k-block a CTA so loads 16 KB of A and 16 KB of B instead of 16 + 32 KB for the same products per SM
// (measured: 0.455 us a k-block against 0.50 us, tensor pipe busy 72 % of the active cycles).
//   * both producers wait for their own `empty` barrier and issue their TMA loads with the leader's
//     `full` barrier as the completion barrier; the leader's producer announces the bytes of both;
//   * the leader's MMA thread commits every stage to the `empty` barriers of both CTAs, and every
//     finished tile to both `acc_full` barriers (tcgen05.commit with a CTA mask);
//   * the epilogue warps of both CTAs drain their own 128 rows and arrive on the leader's
//     `acc_empty` barrier (8 arrivals);
//   * nobody leaves before a cluster barrier: a CTA that has exited cannot be arrived on or read.
// Persistent and double-buffered like the kernel above; waits are bounded the same way.
__device__ __forceinline__ uint32_t cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t map_to_cta(uint32_t smem_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void mbar_arrive_remote(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void tma_load_2d_pair(void* dst, const CUtensorMap* map, int x, int y, uint32_t leader_bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(
          smem_u32(dst)),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(leader_bar), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void mma_f16_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
      "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void mma_commit_pair(uint64_t* bar) {  // arrives on `bar` of both CTAs of the pair
  const uint16_t both = 3;
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(smem_u32(bar)),
               "h"(both)
               : "memory");
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// bf16 x bf16 -> f32, both operands K-major, M = 256 over the pair, N = n.
__host__ __device__ constexpr uint32_t instr_desc_pair(int n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(256 >> 4) << 24);
}

template <typename TO, bool SWIGLU>
__global__ void __launch_bounds__(PERSIST_THREADS)
    gemm_tc_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, TO* __restrict__ out,
                        int RA, int RB, int k_tiles, long long ldo, int stages, int mp_tiles, int n_tiles,
                        int* __restrict__ error_out) {
  constexpr int BN = 256;                  // outputs per tile; each CTA holds BN / 2 weight rows of it
  constexpr int B_HALF_BYTES = (BN / 2) * BK * 2;
  constexpr int STAGE_BYTES = A_BYTES + B_HALF_BYTES;  // per CTA
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + (size_t)stages * STAGE_BYTES);  // used in the leader only
  uint64_t* empty = full + stages;
  uint64_t* acc_full = empty + stages;   // [2]
  uint64_t* acc_empty = acc_full + 2;    // [2] used in the leader only: 8 arrivals
  uint64_t* mma_done = acc_empty + 2;    // in both CTAs: every product the leader issued has finished
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(mma_done + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_rank();  // 0: leader
  const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
  const int total = mp_tiles * n_tiles;
  const int my_tiles = pair < total ? (total - 1 - pair) / n_pairs + 1 : 0;

  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&acc_full[b], 1);
      mbar_init(&acc_empty[b], 8);  // four epilogue warps in each CTA of the pair
    }
    mbar_init(mma_done, 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(512) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  cluster_sync_all();  // the peer's barriers exist before anything arrives on them
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_slot;

  dep_launch();
  if (warp == 4) {
    if (lane == 0) {
      // ---------------------------------------------------------------- producer (both CTAs)
      const long long n_iter = (long long)my_tiles * k_tiles;
      // this CTA's 128 token rows and 128 weight rows of each tile of 256 x 256
      TileWalk first(pair, n_pairs, k_tiles, mp_tiles, 256, BN, (int)rank * BM, (int)rank * (BN / 2)), walk = first;
      const int early = (int)(n_iter < stages ? n_iter : stages);
      for (int it = 0; it < early; ++it, first.next()) {  // weights first: they do not depend on the kernel before
        if (rank == 0) mbar_expect_tx(&full[it], 2 * STAGE_BYTES);
        tma_load_2d_pair(smem + (size_t)it * STAGE_BYTES + A_BYTES, &map_b, first.kt * BK, first.b_row0, map_to_cta(smem_u32(&full[it]), 0));
      }
      dep_wait();
      for (int it = 0; it < early; ++it, walk.next())
        tma_load_2d_pair(smem + (size_t)it * STAGE_BYTES, &map_a, walk.kt * BK, walk.a_row0, map_to_cta(smem_u32(&full[it]), 0));
      long long issued = early;
      bool ok = true;
      RingPos ring(stages, 0, 1u);
      for (long long it = early; it < n_iter && ok; ++it, ring.next(), walk.next()) {
        const int s = ring.s;
        ok = mbar_wait(&empty[s], ring.ph ^ 1u, abort_flag, error_out, ERR_PRODUCER);
        if (!ok) break;
        uint8_t* sa = smem + (size_t)s * STAGE_BYTES;
        const uint32_t bar = map_to_cta(smem_u32(&full[s]), 0);
        if (rank == 0) mbar_expect_tx(&full[s], 2 * STAGE_BYTES);
        tma_load_2d_pair(sa, &map_a, walk.kt * BK, walk.a_row0, bar);
        tma_load_2d_pair(sa + A_BYTES, &map_b, walk.kt * BK, walk.b_row0, bar);
        issued = it + 1;
      }
      if (rank == 0 && (!ok || *abort_flag)) {
        // wait (bounded) for the copies of both CTAs that were announced, before anybody leaves
        const long long first = issued > stages ? issued - stages : 0;
        for (long long it = first; it < issued; ++it) {
          const long long t0 = clock64();
          while (!mbar_try_wait(&full[it % stages], (uint32_t)(it / stages) & 1u)) {
            if (clock64() - t0 > WAIT_CYCLES) {
              atomicCAS(error_out, 0, ERR_DRAIN);
              break;
            }
          }
        }
      }
    }
  } else if (warp == 5) {
    if (lane == 0 && rank == 0) {
      // ---------------------------------------------------------------- tensor-core issue (leader)
      constexpr uint32_t idesc = instr_desc_pair(BN);
      bool ok = true;
      RingPos ring(stages);
      for (int t = 0; t < my_tiles && ok; ++t) {
        const int b = t & 1;
        if (t >= 2) {
          ok = mbar_wait(&acc_empty[b], (uint32_t)((t >> 1) - 1) & 1u, abort_flag, error_out, ERR_MMA);
          if (!ok) break;
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        }
        const uint32_t acc = tmem_base + (uint32_t)(b * BN);
        for (int kt = 0; kt < k_tiles && ok; ++kt, ring.next()) {
          const int s = ring.s;
          ok = mbar_wait(&full[s], ring.ph, abort_flag, error_out, ERR_MMA);
          if (!ok) break;
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const uint32_t sa = smem_u32(smem + (size_t)s * STAGE_BYTES);
          const uint64_t da = smem_desc_sw128(sa), db = smem_desc_sw128(sa + A_BYTES);
#pragma unroll
          for (int k = 0; k < BK / 16; ++k)
            mma_f16_pair(acc, da + (uint64_t)(2 * k), db + (uint64_t)(2 * k), idesc, (kt > 0 || k > 0) ? 1u : 0u);
          mma_commit_pair(&empty[s]);
        }
        if (ok) mma_commit_pair(&acc_full[b]);
      }
      mma_commit_pair(mma_done);  // also after giving up: the stages and tensor memory of BOTH CTAs are the products' until then
    }
  } else {
    // ------------------------------------------------------------------ epilogue: warps 0-3 of both CTAs
    dep_wait();
    bool ok = true;
    for (int t = 0; t < my_tiles; ++t) {
      const int b = t & 1;
      ok = mbar_wait(&acc_full[b], (uint32_t)(t >> 1) & 1u, abort_flag, error_out, ERR_EPILOGUE);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const int tile = pair + t * n_pairs;
      const int a_row0 = (tile % mp_tiles) * 256 + (int)rank * BM, b_row0 = (tile / mp_tiles) * BN;
      const int ra = a_row0 + warp * 32 + lane;
      const uint32_t acc = tmem_base + ((uint32_t)(warp * 32) << 16) + (uint32_t)(b * BN);
      if (SWIGLU) {
#pragma unroll 1
        for (int c0 = 0; c0 < BN / 2; c0 += 16) {
          float gv[16], uv[16];
          tmem_load16(acc + (uint32_t)c0, gv);
          tmem_load16(acc + (uint32_t)(c0 + BN / 2), uv);
#pragma unroll
          for (int i = 0; i < 16; ++i) gv[i] = (gv[i] / (1.0f + expf(-gv[i]))) * uv[i];
          const int col0 = b_row0 / 2 + c0;
          if (ra < RA && col0 < RB / 2) {
            TO* dst = out + (size_t)ra * ldo + col0;
            store_row16<TO>(dst, gv, min(16, RB / 2 - col0), (reinterpret_cast<uintptr_t>(dst) & 15u) == 0);
          }
        }
      } else {
#pragma unroll 1
        for (int c0 = 0; c0 < BN; c0 += 16) {
          float v[16];
          tmem_load16(acc + (uint32_t)c0, v);
          const int rb0 = b_row0 + c0;
          if (ra < RA && rb0 < RB) {
            TO* dst = out + (size_t)ra * ldo + rb0;
            store_row16<TO>(dst, v, min(16, RB - rb0), (reinterpret_cast<uintptr_t>(dst) & 15u) == 0);
          }
        }
      }
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive_remote(map_to_cta(smem_u32(&acc_empty[b]), 0));
    }
    if (threadIdx.x == 0) mbar_drain(mma_done, 0, error_out);
  }
  __syncwarp();  // lanes of the producer and issue warps went different ways; the cluster barrier wants whole warps
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  cluster_sync_all();  // both CTAs are done with each other's shared memory, tensor memory and barriers
  if (warp == 0) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512) : "memory");
  }
  // The pair leaves together, after BOTH halves of the pair-wide release: without this barrier one
  // CTA can release and exit while the other has not yet executed its half, and with programmatic
  // dependent launch the next kernel's CTA is placed on the freed SM at once and allocates tensor
  // memory there while the pair-wide release that covers this SM is still half done. (A precaution:
  // it did not end the rare stop for which this kernel is off by default.)
  cluster_sync_all();
}

template <typename TO, bool SWIGLU>
int launch_tc_pair(const CUtensorMap& ma, const CUtensorMap& mb, void* out, int RA, int RB, int K, long long ldo, int n_sms,
                   cudaStream_t stream) {
  constexpr int STAGE_BYTES = A_BYTES + 128 * BK * 2;
  const int k_tiles = (K + BK - 1) / BK;
  const int stages = 6;
  const size_t smem = (size_t)stages * STAGE_BYTES + (2 * stages + 5) * sizeof(uint64_t) + 16 + 1024;
  auto kernel = gemm_tc_pair_kernel<TO, SWIGLU>;
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024) != cudaSuccess) {
      llm_set_error("gemm_tc: cannot raise the shared memory limit");
      return LLM_ERR_LAUNCH;
    }
    attr_set = true;
  }
  const int mp_tiles = (RA + 255) / 256, n_tiles = (RB + 255) / 256;
  const int pairs = std::min(mp_tiles * n_tiles, n_sms / 2);
  launch_kernel_cluster(kernel, 2 * pairs, PERSIST_THREADS, smem, dim3(2, 1, 1), stream, ma, mb, (TO*)out, RA, RB, k_tiles, ldo, stages, mp_tiles,
                        n_tiles, error_word());
  return LLM_OK;
}

template <typename TO, bool SWIGLU, int BN = 256>
int launch_tc_persistent(const CUtensorMap& ma, const CUtensorMap& mb, void* out, int RA, int RB, int K, long long ldo,
                         int n_sms, cudaStream_t stream, int add_into = 0) {
  constexpr int STAGE_BYTES = A_BYTES + BN * BK * 2;
  const int k_tiles = (K + BK - 1) / BK;
  const int stages = BN == 256 ? 4 : 5;
  const size_t smem = (size_t)stages * STAGE_BYTES + (2 * stages + 5) * sizeof(uint64_t) + 16 + 1024;
  auto kernel = gemm_tc_persistent_kernel<TO, SWIGLU, BN>;
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024) != cudaSuccess) {
      llm_set_error("gemm_tc: cannot raise the shared memory limit");
      return LLM_ERR_LAUNCH;
    }
    attr_set = true;
  }
  const int m_tiles = (RA + BM - 1) / BM, n_tiles = (RB + BN - 1) / BN;
  const int grid = std::min(m_tiles * n_tiles, n_sms);
  launch_kernel(kernel, grid, PERSIST_THREADS, smem, stream, ma, mb, (TO*)out, RA, RB, k_tiles, ldo, stages, m_tiles, n_tiles,
                error_word(), add_into);
  return LLM_OK;
}

int sm_count() {
  static int n = 0;
  if (!n) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
      n = 148;
  }
  return n;
}

// The persistent form pays when an SM gets several tiles.
inline bool use_persistent(int M, int N) { return ((M + BM - 1) / BM) * ((N + 255) / 256) >= 2 * sm_count(); }

// Tiles of 192 outputs instead of 256 when that shortens the last round: the product takes
// (rounds of tiles over the SMs) x (tile width), e.g. 2,048 tokens x 3,072 outputs: 192 tiles of 256
// are two rounds (512), 256 tiles of 192 also two (384).
inline bool prefer_192(int M, int N) {
  const int m_tiles = (M + BM - 1) / BM, sms = sm_count();
  const int t256 = m_tiles * ((N + 255) / 256), t192 = m_tiles * ((N + 191) / 192);
  const int cost256 = (t256 + sms - 1) / sms * 256, cost192 = (t192 + sms - 1) / sms * 192;
  return t192 > sms && cost192 < cost256;
}

// CTA pairs (tiles of 256 x 256 on two SMs) against one-CTA tiles. Measured on B200, a pair spends
// about 0.92 of the time of two single CTAs on the same k-blocks (each SM loads a third less), but
// starts and ends later (cluster launch, barriers across the pair), which short products of one
// round do not earn back; and 256 x 256 tiles can leave more of the last round empty.
// mode: 0 never, 1 wherever the shape allows, -1 by this estimate. allow_192: the one-CTA kernels
// may use tiles of 192 outputs (not with SwiGLU in the epilogue).
inline bool prefer_pairs(int mode, int M, int N, int K, bool allow_192 = true) {
  if (mode == 0 || M <= BM || N < 256) return false;
  if (mode == 1) return true;
  const int sms = sm_count(), k_tiles = (K + BK - 1) / BK, m_tiles = (M + BM - 1) / BM;
  const int t_pair = ((M + 255) / 256) * ((N + 255) / 256), pairs = sms / 2 > 0 ? sms / 2 : 1;
  const int rounds_pair = (t_pair + pairs - 1) / pairs;
  const int t256 = m_tiles * ((N + 255) / 256), t192 = m_tiles * ((N + 191) / 192);
  int cost_single = (t256 + sms - 1) / sms * 256;
  if (allow_192 && prefer_192(M, N)) cost_single = (t192 + sms - 1) / sms * 192;
  return rounds_pair * 256 * 0.92f < (float)cost_single && rounds_pair * k_tiles >= 64;
}

template <int BN, bool SWAP, typename TO, bool SWIGLU = false, int EPI = EPI_NONE>
int launch_tc(const CUtensorMap& ma, const CUtensorMap& mb, void* out, int RA, int RB, int K, int splits, long long ldo,
              long long split_stride, int stages, cudaStream_t stream, const EpiArgs& epi = EpiArgs(), int add_into = 0) {
  constexpr int STAGE_BYTES = A_BYTES + BN * BK * 2;
  const int k_tiles = (K + BK - 1) / BK;
  int per_split = (k_tiles + splits - 1) / splits;
  splits = (k_tiles + per_split - 1) / per_split;
  stages = std::min(stages, (227 * 1024 - 4096) / STAGE_BYTES);
  if (stages > per_split) stages = per_split < 2 ? 2 : per_split;
  const size_t smem = (size_t)stages * STAGE_BYTES + (2 * stages + 1) * sizeof(uint64_t) + 16 + 1024;
  auto kernel = gemm_tc_kernel<BN, SWAP, TO, SWIGLU, EPI>;
  static bool attr_set = false;
  if (!attr_set) {
    cudaFuncAttributes fa;  // static and dynamic shared memory share the 227 KB
    const int fixed = cudaFuncGetAttributes(&fa, kernel) == cudaSuccess ? (int)((fa.sharedSizeBytes + 1023) / 1024) * 1024 : 4096;
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024 - fixed) != cudaSuccess) {
      llm_set_error("gemm_tc: cannot raise the shared memory limit");
      return LLM_ERR_LAUNCH;
    }
    attr_set = true;
  }
  dim3 grid((RA + BM - 1) / BM, (RB + BN - 1) / BN, splits);
  launch_kernel(kernel, grid, 128, smem, stream, ma, mb, (TO*)out, RA, RB, k_tiles, per_split, ldo, split_stride, stages, error_word(), epi,
                add_into);
  return LLM_OK;
}

}  // namespace

static int g_persistent = 1, g_pair = 0;
// CTA pairs (cta_group::2) for products of more than 128 tokens and at least 256 outputs:
// 1 always, 0 never (the default), -1 where they are estimated to be faster.
// Off by default: a prompt step at the Llama 3.2 3B layer sizes (2,048 tokens, gate|up with 3,072
// inputs) was seen to stop inside this kernel once in a few dozen launches, for a cause not found;
// the one-CTA persistent kernels take its shapes about 8 % slower.
extern "C" void llm_gemm_tc_pair(int mode) { g_pair = mode; }
// 0: never the persistent form (for comparisons); 1: where an SM gets at least two tiles.
extern "C" void llm_gemm_tc_persistent(int on) { g_persistent = on; }

enum : int { FORM_ONE_TILE = 0, FORM_PERSISTENT_256 = 1, FORM_PERSISTENT_192 = 2, FORM_PAIRS = 3 };

// Which kernel the token-tile form (tiles of 128 tokens) runs for these sizes: one output tile a
// CTA, the persistent kernel with tiles of 256 or of 192 outputs, or CTA pairs. swiglu: the gate|up
// product with the activation in the epilogue (N counts gate and up rows).
extern "C" int llm_gemm_tc_form(int M, int N, int K, int swiglu) {
  if (N < 256) return FORM_ONE_TILE;
  if (prefer_pairs(g_pair, M, N, K, !swiglu)) return FORM_PAIRS;
  if (!g_persistent) return FORM_ONE_TILE;
  if (!swiglu && prefer_192(M, N)) return FORM_PERSISTENT_192;
  return use_persistent(M, N) ? FORM_PERSISTENT_256 : FORM_ONE_TILE;
}

// Number of K splits llm_gemm_tc will really use for (K, wanted splits).
extern "C" int llm_gemm_tc_splits(int K, int splits) {
  const int k_tiles = (K + BK - 1) / BK;
  if (splits < 1) splits = 1;
  const int per_split = (k_tiles + splits - 1) / splits;
  return (k_tiles + per_split - 1) / per_split;
}

// Whether the tensor-core kernel takes these operands (else the caller uses the CUDA-core one).
extern "C" int llm_gemm_tc_supported(const void* a, const void* w, int M, int N, int K, long long lda, long long ldw) {
  auto al = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; };
  return M > 0 && N > 0 && K > 0 && (K % 8) == 0 && (lda % 8) == 0 && (ldw % 8) == 0 && al(a) && al(w) && encode_fn() != nullptr;
}

// out[m, n] = sum_k a[m, k] * w[n, k], a [M, K] and w [N, K] bfloat16.
// swap = 0: tiles of 128 tokens; out dtype bf16 or f32; splits must be 1.
// swap = 1: M <= 256 tokens; weights fill the accumulator lanes; with splits > 1, out is float32
//           [splits, M, ldo] partials (split_stride elements apart) to be added by the consumer.
static int gemm_tc_impl(const void* a, const void* w, void* out, int M, int N, int K, long long lda, long long ldw,
                        long long ldo, int out_dtype, int swap, int splits, long long split_stride, int stages,
                        cudaStream_t stream, int add_into) {
  if (M == 0 || N == 0) return LLM_OK;
  LLM_REQUIRE(!add_into || (!swap && out_dtype == LLM_F32), "gemm_tc: adding into the output needs token tiles and float32");
  LLM_REQUIRE(llm_gemm_tc_supported(a, w, M, N, K, lda, ldw), "gemm_tc: operands must be 16-byte aligned with K and row strides multiples of 8");
  LLM_REQUIRE(out_dtype == LLM_F32 || out_dtype == LLM_BF16, "gemm_tc: unknown out dtype %d", out_dtype);
  LLM_REQUIRE(splits >= 1 && (splits == 1 || (swap && out_dtype == LLM_F32)), "gemm_tc: K splits need the swapped form and float32 partials");
  LLM_REQUIRE(stages >= 2 && stages <= 12, "gemm_tc: stages %d not in 2..12", stages);
  LLM_REQUIRE(error_word() != nullptr, "gemm_tc: cannot allocate the error word");
  CUtensorMap ma, mb;
  int rc = LLM_OK;
  if (!swap) {
    const int bn = N >= 256 ? 256 : (N > 64 ? 128 : (N > 32 ? 64 : (N > 16 ? 32 : 16)));
    LLM_REQUIRE(tensor_map_for(a, M, K, lda, BM, &ma) && tensor_map_for(w, N, K, ldw, bn, &mb), "gemm_tc: cuTensorMapEncodeTiled failed");
#define LLM_TC_CASE(BN_)                                                                                                   \
  rc = (out_dtype == LLM_F32) ? launch_tc<BN_, false, float>(ma, mb, out, M, N, K, 1, ldo, 0, std::min(stages, BN_ == 256 ? 4 : 6), stream, EpiArgs(), add_into) \
                              : launch_tc<BN_, false, bf16>(ma, mb, out, M, N, K, 1, ldo, 0, std::min(stages, BN_ == 256 ? 4 : 6), stream)
    int form = llm_gemm_tc_form(M, N, K, 0);
    if (form == FORM_PAIRS && add_into) form = use_persistent(M, N) ? FORM_PERSISTENT_256 : FORM_ONE_TILE;  // the pair kernel only stores
    if (form == FORM_PAIRS) {
      LLM_REQUIRE(tensor_map_for(w, N, K, ldw, 128, &mb), "gemm_tc: cuTensorMapEncodeTiled failed");
      rc = (out_dtype == LLM_F32) ? launch_tc_pair<float, false>(ma, mb, out, M, N, K, ldo, sm_count(), stream)
                                  : launch_tc_pair<bf16, false>(ma, mb, out, M, N, K, ldo, sm_count(), stream);
    } else if (form == FORM_PERSISTENT_192) {
      LLM_REQUIRE(tensor_map_for(w, N, K, ldw, 192, &mb), "gemm_tc: cuTensorMapEncodeTiled failed");
      rc = (out_dtype == LLM_F32) ? launch_tc_persistent<float, false, 192>(ma, mb, out, M, N, K, ldo, sm_count(), stream, add_into)
                                  : launch_tc_persistent<bf16, false, 192>(ma, mb, out, M, N, K, ldo, sm_count(), stream);
    } else if (form == FORM_PERSISTENT_256)
      rc = (out_dtype == LLM_F32) ? launch_tc_persistent<float, false>(ma, mb, out, M, N, K, ldo, sm_count(), stream, add_into)
                                  : launch_tc_persistent<bf16, false>(ma, mb, out, M, N, K, ldo, sm_count(), stream);
    else if (bn == 256) LLM_TC_CASE(256);
    else if (bn == 128) LLM_TC_CASE(128);
    else if (bn == 64) LLM_TC_CASE(64);
    else if (bn == 32) LLM_TC_CASE(32);
    else LLM_TC_CASE(16);
#undef LLM_TC_CASE
  } else {
    LLM_REQUIRE(M <= 256, "gemm_tc: the swapped form takes at most 256 tokens, got %d", M);
    const int bn = M > 128 ? 256 : (M > 64 ? 128 : (M > 32 ? 64 : (M > 16 ? 32 : 16)));
    LLM_REQUIRE(tensor_map_for(w, N, K, ldw, BM, &ma) && tensor_map_for(a, M, K, lda, bn, &mb), "gemm_tc: cuTensorMapEncodeTiled failed");
#define LLM_TC_CASE(BN_)                                                                                                        \
  rc = (out_dtype == LLM_F32) ? launch_tc<BN_, true, float>(ma, mb, out, N, M, K, splits, ldo, split_stride, std::min(stages, BN_ == 256 ? 4 : 8), stream) \
                              : launch_tc<BN_, true, bf16>(ma, mb, out, N, M, K, 1, ldo, 0, std::min(stages, BN_ == 256 ? 4 : 8), stream)
    if (bn == 256) LLM_TC_CASE(256);
    else if (bn == 128) LLM_TC_CASE(128);
    else if (bn == 64) LLM_TC_CASE(64);
    else if (bn == 32) LLM_TC_CASE(32);
    else LLM_TC_CASE(16);
#undef LLM_TC_CASE
  }
  if (rc != LLM_OK) return rc;
  LLM_CHECK_LAUNCH("gemm_tc");
  return LLM_OK;
}

extern "C" int llm_gemm_tc(const void* a, const void* w, void* out, int M, int N, int K, long long lda, long long ldw,
                           long long ldo, int out_dtype, int swap, int splits, long long split_stride, int stages,
                           cudaStream_t stream) {
  return gemm_tc_impl(a, w, out, M, N, K, lda, ldw, ldo, out_dtype, swap, splits, split_stride, stages, stream, 0);
}

// out [M, ldo] float32 += a . w^T in tiles of 128 tokens (every output element is read, added to and
// written by the one thread that holds its accumulator: the same float32 sum as a kernel that adds
// the product afterwards, without the product ever going to memory).
extern "C" int llm_gemm_tc_add(const void* a, const void* w, float* out, int M, int N, int K, long long lda, long long ldw,
                               long long ldo, int stages, cudaStream_t stream) {
  return gemm_tc_impl(a, w, out, M, N, K, lda, ldw, ldo, LLM_F32, 0, 1, 0, stages, stream, 1);
}

// The swapped form (at most 64 tokens) with the K splits meeting inside the product (EPI_MEET):
// parts [splits, M, N] float32 scratch; h [M, ld_h] float32 += a . w^T; scaled [M, ld_scaled] bf16 =
// next_w * h (skipped when next_w or scaled is null); sumsq [M, n_sumsq] float32 with n_sumsq =
// ceil(N / 128): column j is the part of the rows' sums of squares that outputs 128 j .. 128 j + 127
// contribute; counters: ceil(N / 128) ints, zero before the first launch and left at zero.
extern "C" int llm_gemm_tc_meet(const void* a, const void* w, float* parts, int M, int N, int K, long long lda, long long ldw,
                                int splits, float* h, long long ld_h, const float* next_w, void* scaled, long long ld_scaled,
                                float* sumsq, int n_sumsq, int* counters, int stages, cudaStream_t stream) {
  if (M == 0 || N == 0) return LLM_OK;
  LLM_REQUIRE(llm_gemm_tc_supported(a, w, M, N, K, lda, ldw), "gemm_tc_meet: operands must be 16-byte aligned with K and row strides multiples of 8");
  LLM_REQUIRE(M <= 64, "gemm_tc_meet: at most 64 tokens, got %d", M);
  LLM_REQUIRE(splits >= 1 && stages >= 2 && stages <= 12, "gemm_tc_meet: splits %d, stages %d", splits, stages);
  LLM_REQUIRE(h != nullptr && counters != nullptr && parts != nullptr, "gemm_tc_meet: stream, counters and scratch are needed");
  LLM_REQUIRE(sumsq == nullptr || n_sumsq == (N + BM - 1) / BM, "gemm_tc_meet: %d parts of the sums of squares for %d outputs", n_sumsq, N);
  LLM_REQUIRE(error_word() != nullptr, "gemm_tc_meet: cannot allocate the error word");
  const int bn = M > 32 ? 64 : (M > 16 ? 32 : 16);
  CUtensorMap ma, mb;
  LLM_REQUIRE(tensor_map_for(w, N, K, ldw, BM, &ma) && tensor_map_for(a, M, K, lda, bn, &mb), "gemm_tc_meet: cuTensorMapEncodeTiled failed");
  EpiArgs epi;
  epi.h = h; epi.ld_h = ld_h; epi.next_w = next_w; epi.scaled = static_cast<bf16*>(scaled); epi.ld_scaled = ld_scaled;
  epi.sumsq = sumsq; epi.n_sumsq = n_sumsq; epi.counters = counters;
  int rc;
  const long long split_stride = (long long)M * N;
  if (bn == 64) rc = launch_tc<64, true, float, false, EPI_MEET>(ma, mb, parts, N, M, K, splits, N, split_stride, std::min(stages, 8), stream, epi);
  else if (bn == 32) rc = launch_tc<32, true, float, false, EPI_MEET>(ma, mb, parts, N, M, K, splits, N, split_stride, std::min(stages, 8), stream, epi);
  else rc = launch_tc<16, true, float, false, EPI_MEET>(ma, mb, parts, N, M, K, splits, N, split_stride, std::min(stages, 8), stream, epi);
  if (rc != LLM_OK) return rc;
  LLM_CHECK_LAUNCH("gemm_tc_meet");
  return LLM_OK;
}

// The swapped form (at most 64 tokens, no K splits) with every token's results divided by the root
// mean square that in_sumsq [M, n_in] gives: out [M, ldo] float32 = (a . w^T) / sqrt(sum_j in_sumsq[m, j] * inv_dim + eps).
extern "C" int llm_gemm_tc_scaled(const void* a, const void* w, float* out, int M, int N, int K, long long lda, long long ldw,
                                  long long ldo, const float* in_sumsq, int n_in, float inv_dim, float eps, int stages,
                                  cudaStream_t stream) {
  if (M == 0 || N == 0) return LLM_OK;
  LLM_REQUIRE(llm_gemm_tc_supported(a, w, M, N, K, lda, ldw), "gemm_tc_scaled: operands must be 16-byte aligned with K and row strides multiples of 8");
  LLM_REQUIRE(M <= 64, "gemm_tc_scaled: at most 64 tokens, got %d", M);
  LLM_REQUIRE(in_sumsq != nullptr && n_in > 0 && stages >= 2 && stages <= 12, "gemm_tc_scaled: the parts of the sums of squares are needed");
  LLM_REQUIRE(error_word() != nullptr, "gemm_tc_scaled: cannot allocate the error word");
  const int bn = M > 32 ? 64 : (M > 16 ? 32 : 16);
  CUtensorMap ma, mb;
  LLM_REQUIRE(tensor_map_for(w, N, K, ldw, BM, &ma) && tensor_map_for(a, M, K, lda, bn, &mb), "gemm_tc_scaled: cuTensorMapEncodeTiled failed");
  EpiArgs epi;
  epi.in_sumsq = in_sumsq; epi.n_in_sumsq = n_in; epi.inv_dim = inv_dim; epi.eps = eps;
  int rc;
  if (bn == 64) rc = launch_tc<64, true, float, false, EPI_SCALE>(ma, mb, out, N, M, K, 1, ldo, 0, std::min(stages, 8), stream, epi);
  else if (bn == 32) rc = launch_tc<32, true, float, false, EPI_SCALE>(ma, mb, out, N, M, K, 1, ldo, 0, std::min(stages, 8), stream, epi);
  else rc = launch_tc<16, true, float, false, EPI_SCALE>(ma, mb, out, N, M, K, 1, ldo, 0, std::min(stages, 8), stream, epi);
  if (rc != LLM_OK) return rc;
  LLM_CHECK_LAUNCH("gemm_tc_scaled");
  return LLM_OK;
}

// act[m, c] = silu(g[m, c]) * u[m, c] with g | u = a . w^T, for w [2*FF, K] whose rows are blocks of
// 128 gate rows followed by the 128 matching up rows (FF a multiple of 128). act: bf16 [M, FF].
extern "C" int llm_gemm_tc_swiglu(const void* a, const void* w, void* act, int M, int FF, int K, long long lda, long long ldw,
                                  long long ld_act, cudaStream_t stream) {
  if (M == 0 || FF == 0) return LLM_OK;
  LLM_REQUIRE(llm_gemm_tc_supported(a, w, M, 2 * FF, K, lda, ldw), "gemm_tc_swiglu: operands must be 16-byte aligned with K and row strides multiples of 8");
  LLM_REQUIRE(FF % 128 == 0, "gemm_tc_swiglu: the intermediate size %d must be a multiple of 128", FF);
  LLM_REQUIRE(error_word() != nullptr, "gemm_tc_swiglu: cannot allocate the error word");
  CUtensorMap ma, mb;
  LLM_REQUIRE(tensor_map_for(a, M, K, lda, BM, &ma) && tensor_map_for(w, 2 * FF, K, ldw, 256, &mb), "gemm_tc_swiglu: cuTensorMapEncodeTiled failed");
  const int form = llm_gemm_tc_form(M, 2 * FF, K, 1);
  if (form == FORM_PAIRS) {
    LLM_REQUIRE(tensor_map_for(w, 2 * FF, K, ldw, 128, &mb), "gemm_tc_swiglu: cuTensorMapEncodeTiled failed");
    const int rc2 = launch_tc_pair<bf16, true>(ma, mb, act, M, 2 * FF, K, ld_act, sm_count(), stream);
    if (rc2 != LLM_OK) return rc2;
    LLM_CHECK_LAUNCH("gemm_tc_swiglu");
    return LLM_OK;
  }
  const int rc = form == FORM_PERSISTENT_256
                     ? launch_tc_persistent<bf16, true>(ma, mb, act, M, 2 * FF, K, ld_act, sm_count(), stream)
                     : launch_tc<256, false, bf16, true>(ma, mb, act, M, 2 * FF, K, 1, ld_act, 0, 4, stream);
  if (rc != LLM_OK) return rc;
  LLM_CHECK_LAUNCH("gemm_tc_swiglu");
  return LLM_OK;
}

// Queues a copy of the error word into `host_word` (pinned host memory) on `stream`, behind the
// kernels already launched there: after the stream is synchronized the host reads the code of the
// step without a transfer of its own. May be captured in a CUDA graph.
extern "C" int llm_tc_error_copy_async(int* host_word, cudaStream_t stream) {
  int* w = error_word();
  LLM_REQUIRE(w != nullptr && host_word != nullptr, "tc_error_copy: no error word");
  if (cudaMemcpyAsync(host_word, w, sizeof(int), cudaMemcpyDeviceToHost, stream) != cudaSuccess) {
    llm_set_error("tc_error_copy: cudaMemcpyAsync failed");
    return LLM_ERR_LAUNCH;
  }
  return LLM_OK;
}

// Writes the error word from the host (0 clears it). For tests of the host's error handling, which
// must not make a kernel fail in order to see the code. Synchronizes.
extern "C" int llm_tc_error_set(int code) {
  int* w = error_word();
  if (!w) return -1;
  return cudaMemcpy(w, &code, sizeof(int), cudaMemcpyHostToDevice) == cudaSuccess ? 0 : -2;
}

// Reads and clears the error code that a tensor-core kernel may have left (0 = none). Synchronizes.
extern "C" int llm_gemm_tc_error() {
  int* w = error_word();
  if (!w) return -1;
  int v = 0;
  if (cudaMemcpy(&v, w, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return -2;
  if (v) cudaMemset(w, 0, sizeof(int));
  return v;
}
