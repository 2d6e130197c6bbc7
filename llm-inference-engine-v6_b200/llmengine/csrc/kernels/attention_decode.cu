// Decoding attention over the paged cache: every request of the step brings ONE token.
//
// A CTA owns (request, key/value head, split of the key range); its 16 rows hold the `group` query
// heads that share the key/value head, so a key or value is fetched once for all of them. Keys and
// values arrive by TMA: one producer thread walks the split in tiles of 32 keys (absolute
// positions), looks the pages up in a copy of the block-table slice in shared memory and issues
// one box per page into a ring of stages with 128-byte swizzle; the four consumer warps take the
// tiles in turn (warp w: tiles w, w+4, ...) and never compute an address in global memory. Tiles
// that hold only keys of earlier steps are requested before the wait on the previous kernel; the
// tile that holds the token's own key (written just before this kernel) after it. Pages that the
// table does not hold (beyond the request's last page, or given back behind a window) are read from
// the pool's null page, so every tile is complete; their scores are masked by position.
//
// Scores (bf16 mma.sync, float32 accumulators), the running (max, sum) softmax in log2 units and
// the output sums are float32 registers. The four warps' partials are merged in warp order, the
// splits' partials in index order: a token's result does not depend on the batch or on page numbers.
// Up to eight splits of a (request, key/value head) run as ONE thread-block cluster (CLUSTER): each
// CTA finishes a slice of the output; every CTA stores its partial's shares into the shared memory
// of the CTAs that finish them (distributed shared memory, asynchronous stores whose bytes are
// counted on an mbarrier of the receiver); a CTA that has seen all bytes counted in finds all it
// needs in its own shared memory. The
// hardware cluster barrier is used once, split in two: every thread arrives right after the CTA's
// own barriers are initialised (nothing conditional comes before that) and waits just before the
// first access to a peer's shared memory, which CUDA allows only once the peer has started. Every
// other wait on a peer is a bounded wait on an mbarrier. More splits run as
// several clusters of eight: every cluster merges its own splits the same way into ONE partial in
// global memory, and the cluster that arrives last (a fence and a counter) merges those. Without
// clusters every split's partial goes through global memory (about 2 us slower at six splits, and
// growing with their number: the merging CTA reads them all).
//
// Fused form (FUSED): the kernel before this one is the q|k|v product itself, given as float32 K-split
// partial sums [parts][token][q|k|v]. The computing warps add the parts in index order, rotate q
// (and k) by the position's cos/sin row as the separate rotation kernel does (half-split form of
// the reference's apply_rope_inplace, src/kernels.cpp:189-203) and keep q in shared memory only;
// the CTA whose key range holds the token's own position also writes the new key (rotated) and
// value to the cache for later steps and patches them into its last tile in shared memory, since
// the copy of that tile read the cache before they were there. No copy then depends on the kernel
// before, so all of them are requested ahead of the dependency wait.
//
// Formula: the reference's attention_f32 (src/kernels.cpp:413-474).
#include "tc_common.cuh"
#include "mma_common.cuh"

#include <cmath>

namespace {

constexpr int DEC_THREADS = 160;  // warps 0-3 compute, warp 4 lane 0 issues the copies
constexpr int DEC_CONSUMERS = 128;
constexpr int TK = 32;            // keys per tile
constexpr int ROWS = 16;          // query rows (heads of the group; zeros beyond)
enum : int { ERR_DEC_PRODUCER = 21, ERR_DEC_CONSUMER = 22, ERR_DEC_DRAIN = 23, ERR_DEC_PEERS = 24 };

struct DecParams {
  const bf16* q; long long ld_q;
  const int* seq_start; const int* seq_qoff; const int* block_table;
  int max_blocks, nq, nkv, page_size, page_shift, window, null_page;  // page_shift: log2(page_size), -1 if no power of two
  float scale;
  bf16* out; long long ld_out;
  float* part_o; float* part_ml; int split_keys, n_splits; long long part_stride_tokens;
  int cluster_size;  // CLUSTER: splits per cluster (n_splits is a multiple of it); more than one cluster -> their results meet in global memory
  int* done_count;
  int* error;
  // fused form only
  const float* qkv_parts; int n_parts; long long part_stride;  // [n_parts][tokens][(nq + 2 nkv) * hd], parts part_stride floats apart
  RowScale rs;  // the 1/rms that the q|k|v sums are still owed (sumsq null: none)
  const float* cos_t; const float* sin_t;                       // [positions][hd / 2], or null: no rotation
  bf16* kcache; bf16* vcache;                                   // where the token's own key and value are written
};

// DEEP: a longer ring for launches that fill the GPU with fewer, latency-bound CTAs; the short ring
// lets four CTAs (head size 64) share an SM, which is what streams the cache fastest.
template <int HD, bool DEEP>
struct DecLayout {
  static constexpr int HALVES = HD / 64;               // 64-element (128-byte) column blocks of a row
  static constexpr int TILE_BYTES = TK * HD * 2;       // one of K or V
  static constexpr int STAGE_BYTES = 2 * TILE_BYTES;
  static constexpr int STAGES = HD == 64 ? (DEEP ? 8 : 6) : (DEEP ? 5 : 4);  // 64 / 48 KB and 80 / 64 KB of ring
  static_assert(STAGES >= 4, "the consumers' wait on the stage's previous tile needs a ring of at least four stages");
  static constexpr int Q_LD = HD + 8;
};

// Byte offset of (row, 16-byte chunk) inside a [TK][64] tile written by TMA with 128-byte swizzle.
__device__ __forceinline__ uint32_t sw128(int row, int chunk) { return (uint32_t)(row * 128 + ((chunk ^ (row & 7)) << 4)); }

// One float into the shared memory of CTA `rank` of this cluster, at the address `smem_addr` has here;
// its 4 bytes are counted on that CTA's mbarrier `bar` when they have landed, so the receiver needs no
// arrival from the sender and the sender no fence.
__device__ __forceinline__ void send_to_cta(uint32_t smem_addr, uint64_t* bar, int rank, float v) {
  uint32_t remote, remote_bar;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(smem_addr), "r"(rank));
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote_bar) : "r"(smem_u32(bar)), "r"(rank));
  asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.b32 [%0], %1, [%2];" ::"r"(remote), "r"(__float_as_uint(v)),
               "r"(remote_bar)
               : "memory");
}

// The two halves of the hardware cluster barrier (all threads of the CTA, converged).
__device__ __forceinline__ void cluster_arrive() { asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_wait() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }

// One arrival on the mbarrier that CTA `rank` of this cluster keeps at the address `bar` has here.
// Release at cluster scope: what this CTA stored into that CTA's shared memory before (ordered
// before this thread by a CTA barrier) is visible to whoever sees the phase complete.
__device__ __forceinline__ void mbar_arrive_cta(uint64_t* bar, int rank) {
  uint32_t remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(smem_u32(bar)), "r"(rank));
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(remote) : "memory");
}

// Bounded wait for arrivals from the peers of the cluster (acquire at cluster scope). The bound is
// twice that of the waits inside a CTA: a peer that gives up one of those still arrives here, and
// must find this CTA running. Unlike mbar_wait it does not leave early when another kernel has
// already recorded an error: a CTA may not exit while a peer can still reach its shared memory.
__device__ __forceinline__ bool mbar_wait_peers(uint64_t* bar, uint32_t parity, int* error_out, int code) {
  const long long t0 = clock64();
  for (uint32_t i = 0;; ++i) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    if (ok) return true;
    if ((i & 255u) == 255u && clock64() - t0 > 2 * WAIT_CYCLES) {
      atomicCAS(error_out, 0, code);
      return false;
    }
  }
}

// (Four CTAs of head size 64 share an SM when the launch is larger than one wave: at most 96
// registers a thread, which the second number asks the compiler to keep; head size 128: two.)
template <int HD, bool FUSED, bool DEEP, bool CLUSTER>
__global__ void __launch_bounds__(DEC_THREADS, (HD == 64 ? 4 : 2)) paged_attention_decode_tma_kernel(const __grid_constant__ CUtensorMap map_k,
                                                                                 const __grid_constant__ CUtensorMap map_v,
                                                                                 const DecParams p) {
  using L = DecLayout<HD, DEEP>;
  constexpr int KSTEPS = HD / 16, DTILES = HD / 8, NS = L::STAGES;
  extern __shared__ uint8_t smem_dyn[];
  uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~(uintptr_t)1023);
  uint8_t* ring = base;                                                     // [NS][K tile | V tile]
  bf16* q_s = reinterpret_cast<bf16*>(ring + (size_t)NS * L::STAGE_BYTES);  // [ROWS][Q_LD]
  uint64_t* full = reinterpret_cast<uint64_t*>(q_s + ROWS * L::Q_LD);       // [NS]
  uint64_t* empty = full + NS;                                              // [NS]
  uint64_t* peers_in = empty + NS;   // CLUSTER: the bytes of the shares that every CTA of the cluster sends here have all landed
  uint64_t* slices_out = peers_in + 1;  // CLUSTER, in the cluster's first CTA: every CTA's slice of the cluster's partial is in global memory
  int* flags = reinterpret_cast<int*>(slices_out + 1);                      // [0] abort, [1] tiles issued, [2] is_last
  bf16* kv_new = reinterpret_cast<bf16*>(flags + 4);                        // [2][HD]: the token's own key and value (fused form)
  // CLUSTER: where the peers store their shares of the partials. It must be memory that this CTA
  // uses for nothing else: a faster peer writes here while this CTA's ring is still in use.
  float* recv = reinterpret_cast<float*>(kv_new + 2 * HD);                  // [size][epo] outputs, then [size][g][2] (max, sum)
  int* page_s = reinterpret_cast<int*>(recv + (CLUSTER ? (p.nq / p.nkv) * (HD + 16) + 8 : 0));  // (+8: shares are rounded up per rank)  // the split's slice of the block table
  volatile int* abort_flag = flags;

  dep_launch();
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int seq = blockIdx.x, kvh = blockIdx.y, split = blockIdx.z;
  const int g = p.nq / p.nkv;
  // The batch arrays came with the step's host-to-device copy and every key before the token's own
  // position was written by an earlier step: both may be read before the dependency wait.
  const int pos = p.seq_start[seq];
  const int tok = p.seq_qoff[seq];
  int lo = (p.window > 0) ? max(0, pos - p.window + 1) : 0;
  int hi = pos;
  lo = max(lo, split * p.split_keys);
  hi = min(hi, (split + 1) * p.split_keys - 1);
  const bool any = hi >= lo;
  const int kt_first = lo / TK;
  const int n_tiles = any ? hi / TK - kt_first + 1 : 0;
  const int page_first = kt_first * TK / p.page_size;  // page of the first tile's first key

  if (tid == 0) {
    for (int s = 0; s < NS; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    if (CLUSTER) {
      mbar_init(peers_in, 1);
      mbar_init(slices_out, (uint32_t)p.cluster_size);
    }
    flags[0] = 0;
    flags[1] = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    if (CLUSTER) {
      // what the CTAs of the cluster (this one too) will send here: every one its share of the output
      // elements that this CTA finishes (e = rank, rank + size, ...) and its (max, sum) of every row
      const int cs = p.cluster_size, rk = split % cs, n_el = (p.nq / p.nkv) * HD;
      const int mine = rk < n_el ? (n_el - rk + cs - 1) / cs : 0;
      mbar_expect_tx(peers_in, (uint32_t)(cs * (mine + 2 * (p.nq / p.nkv)) * 4));
    }
  }
  if (any) {
    const int* table = p.block_table + (size_t)seq * p.max_blocks;
    const int n_pages = ((kt_first + n_tiles) * TK - 1) / p.page_size - page_first + 1;
    for (int i = tid; i < n_pages; i += DEC_THREADS) {
      const int idx = page_first + i;
      const int page = idx < p.max_blocks ? table[idx] : -1;
      page_s[i] = page >= 0 ? page : p.null_page;
    }
  }
  __syncthreads();
  // This CTA runs and its barriers exist: the peers learn it at their cluster_wait(), which every
  // thread passes before the CTA's first access to a peer's shared memory.
  if (CLUSTER) cluster_arrive();

  if (warp == 4) {
    // ------------------------------------------------------------------ producer
    // Lane b issues box b of every tile (a box = the tile's keys of one page); lane 0 also waits for
    // the stage and announces the bytes. Boxes per tile: 32 / page_size for small pages, else 1.
    const int rows_per_box = min(p.page_size, TK);
    const int boxes = TK / rows_per_box;
    bool waited = false, ok = true;
    for (int t = 0; t < n_tiles; ++t) {
      const int stage = t % NS;
      if (t >= NS) {
        if (lane == 0) ok = mbar_wait(&empty[stage], ((t / NS) - 1) & 1, abort_flag, p.error, ERR_DEC_PRODUCER);
        ok = __shfl_sync(0xffffffffu, ok, 0);
        if (!ok) break;
      }
      const int key0 = (kt_first + t) * TK;
      if (!FUSED && !waited && key0 + TK > pos) {  // the tile of the token's own key, written by the kernel before this one
        dep_wait();
        waited = true;
      }
      if (lane == 0) mbar_expect_tx(&full[stage], L::STAGE_BYTES);
      __syncwarp();
      if (lane < boxes) {
        const int key = key0 + lane * rows_per_box;
        int page_idx, in_page;
        if (p.page_shift >= 0) {
          page_idx = key >> p.page_shift;
          in_page = key & (p.page_size - 1);
        } else {
          page_idx = key / p.page_size;
          in_page = key - page_idx * p.page_size;
        }
        const int row = (page_s[page_idx - page_first] * p.nkv + kvh) * p.page_size + in_page;
        uint8_t* kb = ring + (size_t)stage * L::STAGE_BYTES + lane * rows_per_box * 128;
        uint8_t* vb = kb + L::TILE_BYTES;
#pragma unroll
        for (int h = 0; h < L::HALVES; ++h) {
          tma_load_2d(kb + h * (TK * 128), &map_k, h * 64, row, &full[stage]);
          tma_load_2d(vb + h * (TK * 128), &map_v, h * 64, row, &full[stage]);
        }
      }
      if (lane == 0) flags[1] = t + 1;
    }
  } else {
    // ------------------------------------------------------------------ consumers
    dep_wait();  // q comes from the kernel before this one
    const bool own_key_here = any && pos >= lo && pos <= hi;  // this CTA's range holds the token's own position
    if constexpr (FUSED) {
      // items: rotation pairs of the group's q heads, then (own_key_here) of the k head, then pairs of
      // neighbouring v elements; sums over the parts in index order, eight loads in flight
      constexpr int HALF = HD / 2;
      const int n_items = g * HALF + (own_key_here ? 2 * HALF : 0);
      const int width = (p.nq + 2 * p.nkv) * HD;
      const float* prow = p.qkv_parts + (size_t)tok * width;
      const float row_sc = row_scale(p.rs, (size_t)tok);
      for (int c = tid; c < (ROWS - g) * (HD / 8); c += DEC_CONSUMERS)  // rows beyond the group are zeros
        *reinterpret_cast<uint4*>(q_s + (g + c / (HD / 8)) * L::Q_LD + (c % (HD / 8)) * 8) = make_uint4(0, 0, 0, 0);
      for (int item = tid; item < n_items; item += DEC_CONSUMERS) {
        int col_a, col_b, i = 0, kind;  // kind 0: q, 1: k, 2: v
        int r = 0;
        if (item < g * HALF) {
          kind = 0; r = item / HALF; i = item - r * HALF;
          col_a = (kvh * g + r) * HD + i; col_b = col_a + HALF;
        } else if (item < g * HALF + HALF) {
          kind = 1; i = item - g * HALF;
          col_a = (p.nq + kvh) * HD + i; col_b = col_a + HALF;
        } else {
          kind = 2; i = item - g * HALF - HALF;
          col_a = (p.nq + p.nkv + kvh) * HD + 2 * i; col_b = col_a + 1;
        }
        float a = 0.f, b = 0.f;
        for (int p0 = 0; p0 < p.n_parts; p0 += 8) {
          float va[8], vb[8];
#pragma unroll
          for (int u = 0; u < 8; ++u) {
            const bool in = p0 + u < p.n_parts;
            va[u] = in ? prow[(size_t)(p0 + u) * p.part_stride + col_a] : 0.f;
            vb[u] = in ? prow[(size_t)(p0 + u) * p.part_stride + col_b] : 0.f;
          }
#pragma unroll
          for (int u = 0; u < 8; ++u) {
            a += va[u];
            b += vb[u];
          }
        }
        a *= row_sc;
        b *= row_sc;
        float ra = a, rb = b;
        if (kind != 2 && p.cos_t) {
          const float cs = p.cos_t[(size_t)pos * HALF + i], sn = p.sin_t[(size_t)pos * HALF + i];
          ra = a * cs - b * sn;
          rb = b * cs + a * sn;
        }
        const bf16 oa = __float2bfloat16_rn(ra), ob = __float2bfloat16_rn(rb);
        if (kind == 0) {
          q_s[r * L::Q_LD + i] = oa;
          q_s[r * L::Q_LD + i + HALF] = ob;
        } else {
          int page_idx, in_page;
          if (p.page_shift >= 0) {
            page_idx = pos >> p.page_shift;
            in_page = pos & (p.page_size - 1);
          } else {
            page_idx = pos / p.page_size;
            in_page = pos - page_idx * p.page_size;
          }
          const size_t at = ((size_t)(page_s[page_idx - page_first] * p.nkv + kvh) * p.page_size + in_page) * HD;
          if (kind == 1) {
            kv_new[i] = oa; kv_new[i + HALF] = ob;
            p.kcache[at + i] = oa; p.kcache[at + i + HALF] = ob;
          } else {
            kv_new[HD + 2 * i] = oa; kv_new[HD + 2 * i + 1] = ob;
            p.vcache[at + 2 * i] = oa; p.vcache[at + 2 * i + 1] = ob;
          }
        }
      }
    } else {
      for (int c = tid; c < ROWS * (HD / 8); c += DEC_CONSUMERS) {
        const int r = c / (HD / 8), ch = c % (HD / 8);
        cp_async16(q_s + r * L::Q_LD + ch * 8, p.q + (size_t)tok * p.ld_q + (size_t)(kvh * g + min(r, g - 1)) * HD + ch * 8, r < g);
      }
      cp_async_commit();
      cp_async_wait<0>();
    }
    asm volatile("bar.sync 1, %0;" ::"n"(DEC_CONSUMERS) : "memory");
    uint32_t qa[KSTEPS][4];
#pragma unroll
    for (int ks = 0; ks < KSTEPS; ++ks) ldmatrix_x4(qa[ks], q_s + (lane % 16) * L::Q_LD + ks * 16 + (lane / 16) * 8);
    const int row_a = lane / 4, row_b = row_a + 8;
    const bool va_row = row_a < g, vb_row = row_b < g;

    float o_acc[DTILES][4];
#pragma unroll
    for (int d = 0; d < DTILES; ++d) o_acc[d][0] = o_acc[d][1] = o_acc[d][2] = o_acc[d][3] = 0.f;
    float m_a = -INFINITY, m_b = -INFINITY, l_a = 0.f, l_b = 0.f;
    const float sl2 = p.scale * 1.4426950408889634f;

    for (int t = warp; t < n_tiles; t += 4) {
      const int stage = t % NS;
      // A parity wait tells the current phase from the one before it, not from older ones. When the
      // ring length is no multiple of the four warps, the tile that used this stage before (t - NS)
      // belongs to another warp and may not even have landed: wait until it has been consumed
      // (that phase is at most one behind, since this warp's own tile t - 4 was issued after tile
      // t - 4 - NS had been consumed), and only then for this tile's copy.
      if (NS % 4 != 0 && t >= NS && !mbar_wait(&empty[stage], ((t / NS) - 1) & 1, abort_flag, p.error, ERR_DEC_CONSUMER)) break;
      if (!mbar_wait(&full[stage], (t / NS) & 1, abort_flag, p.error, ERR_DEC_CONSUMER)) break;
      const uint32_t kb = smem_u32(ring + (size_t)stage * L::STAGE_BYTES);
      const uint32_t vb = kb + L::TILE_BYTES;
      if (FUSED && own_key_here && (kt_first + t) * TK + TK > pos) {
        // the copy of this tile read the cache before the token's own key and value were there
        const int r = pos - (kt_first + t) * TK;
        if (lane < 2 * (HD / 8)) {
          const int which = lane / (HD / 8), chunk = lane % (HD / 8);  // 0: key, 1: value; 16 bytes each lane
          uint8_t* dst = ring + (size_t)stage * L::STAGE_BYTES + which * L::TILE_BYTES + (chunk / 8) * (TK * 128) + sw128(r, chunk % 8);
          *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(kv_new + which * HD + chunk * 8);
        }
        __syncwarp();
      }

      float s[TK / 8][4];
#pragma unroll
      for (int i = 0; i < TK / 8; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
#pragma unroll
      for (int ks = 0; ks < KSTEPS; ++ks) {
#pragma unroll
        for (int j2 = 0; j2 < TK / 16; ++j2) {
          uint32_t b[4];
          const int row = j2 * 16 + (lane % 8) + (lane / 16) * 8;
          const int chunk = (ks % 4) * 2 + ((lane / 8) % 2);
          ldmatrix_x4_addr(b, kb + (ks / 4) * (TK * 128) + sw128(row, chunk));
          mma_bf16(s[2 * j2], qa[ks], b[0], b[1]);
          mma_bf16(s[2 * j2 + 1], qa[ks], b[2], b[3]);
        }
      }
      const int tile_key0 = (kt_first + t) * TK;
      const int key0 = tile_key0 + 2 * (lane % 4);
      float mx_a = -INFINITY, mx_b = -INFINITY;
      if (tile_key0 >= lo && tile_key0 + TK - 1 <= hi) {  // every key of the tile counts: only the rows are masked
#pragma unroll
        for (int i = 0; i < TK / 8; ++i) {
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            s[i][e] = va_row ? s[i][e] * sl2 : -INFINITY;
            s[i][2 + e] = vb_row ? s[i][2 + e] * sl2 : -INFINITY;
            mx_a = fmaxf(mx_a, s[i][e]);
            mx_b = fmaxf(mx_b, s[i][2 + e]);
          }
        }
      } else {
#pragma unroll
        for (int i = 0; i < TK / 8; ++i) {
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const int key = key0 + i * 8 + e;
            const bool in = key >= lo && key <= hi;
            s[i][e] = (in && va_row) ? s[i][e] * sl2 : -INFINITY;
            s[i][2 + e] = (in && vb_row) ? s[i][2 + e] * sl2 : -INFINITY;
            mx_a = fmaxf(mx_a, s[i][e]);
            mx_b = fmaxf(mx_b, s[i][2 + e]);
          }
        }
      }
      mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 1));
      mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 2));
      mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 1));
      mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 2));
      const float mn_a = fmaxf(m_a, mx_a), mn_b = fmaxf(m_b, mx_b);
      const float base_a = (mn_a == -INFINITY) ? 0.f : mn_a, base_b = (mn_b == -INFINITY) ? 0.f : mn_b;
      const float al_a = exp2f(m_a - base_a), al_b = exp2f(m_b - base_b);
      float sum_a = 0.f, sum_b = 0.f;
#pragma unroll
      for (int i = 0; i < TK / 8; ++i) {
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          s[i][e] = exp2f(s[i][e] - base_a);
          s[i][2 + e] = exp2f(s[i][2 + e] - base_b);
          sum_a += s[i][e];
          sum_b += s[i][2 + e];
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
#pragma unroll
      for (int kk = 0; kk < TK / 16; ++kk) {
        uint32_t pa[4];
        pa[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
        pa[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
        pa[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
        pa[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
        for (int d2 = 0; d2 < DTILES / 2; ++d2) {
          uint32_t b[4];
          const int row = kk * 16 + (lane % 8) + ((lane / 8) % 2) * 8;
          const int chunk = d2 * 2 + lane / 16;  // 16-byte chunk of the row over all halves
          ldmatrix_x4_trans_addr(b, vb + (chunk / 8) * (TK * 128) + sw128(row, chunk % 8));
          mma_bf16(o_acc[2 * d2], pa, b[0], b[1]);
          mma_bf16(o_acc[2 * d2 + 1], pa, b[2], b[3]);
        }
      }
      __syncwarp();  // the whole warp has read the stage
      if (lane == 0) mbar_arrive(&empty[stage]);
    }
    // hand the warp's partial to the merge below (after every copy of the ring has landed and been read)
    asm volatile("bar.sync 1, %0;" ::"n"(DEC_CONSUMERS) : "memory");
    if (!*abort_flag) {
      float* mg = reinterpret_cast<float*>(ring);  // [warp][row][HD + 2]
      constexpr int MLD = HD + 2;
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        const int row = half ? row_b : row_a;
        float* dst = mg + ((size_t)warp * ROWS + row) * MLD;
#pragma unroll
        for (int d = 0; d < DTILES; ++d) {
          dst[d * 8 + 2 * (lane % 4)] = o_acc[d][2 * half];
          dst[d * 8 + 2 * (lane % 4) + 1] = o_acc[d][2 * half + 1];
        }
        if ((lane % 4) == 0) {
          dst[HD] = half ? m_b : m_a;
          dst[HD + 1] = half ? l_b : l_a;
        }
      }
    }
  }
  __syncthreads();
  if (CLUSTER) cluster_wait();  // every CTA of the cluster runs and has initialised its barriers
  const int csize = CLUSTER ? p.cluster_size : 1, rank = CLUSTER ? split % csize : 0;
  if (*abort_flag) {
    // A wait gave up. The peers wait for this CTA's shares: tell them at once that there are none
    // (the error word is set; the output of this launch is void), then let the copies that were
    // issued land (bounded), and leave only when no peer can reach this CTA's shared memory any more.
    if (CLUSTER) {  // shares that weigh nothing: a maximum of -inf and a sum of 0
      const int epo = (g * HD + csize - 1) / csize;
      const uint32_t recv_a = smem_u32(recv);
      for (int e = tid; e < g * HD; e += DEC_THREADS) {
        send_to_cta(recv_a + (uint32_t)(rank * epo + e / csize) * 4u, peers_in, e % csize, 0.f);
        if (e % HD == 0)
          for (int c = 0; c < csize; ++c) {
            send_to_cta(recv_a + (uint32_t)(csize * epo + (rank * g + e / HD) * 2) * 4u, peers_in, c, -INFINITY);
            send_to_cta(recv_a + (uint32_t)(csize * epo + (rank * g + e / HD) * 2 + 1) * 4u, peers_in, c, 0.f);
          }
      }
    }
    if (CLUSTER && tid == 0 && p.n_splits > csize) mbar_arrive_cta(slices_out, 0);
    if (tid == 0) {
      const int issued = flags[1];
      for (int t = max(0, issued - NS); t < issued; ++t) {
        const long long t0 = clock64();
        while (!mbar_try_wait(&full[t % NS], (t / NS) & 1)) {
          if (clock64() - t0 > WAIT_CYCLES) {
            atomicCAS(p.error, 0, (int)ERR_DEC_DRAIN);
            break;
          }
        }
      }
      if (CLUSTER) {
        mbar_wait_peers(peers_in, 0, p.error, ERR_DEC_PEERS);
        if (p.n_splits > csize && rank == 0) mbar_wait_peers(slices_out, 0, p.error, ERR_DEC_PEERS);
      }
    }
    __syncthreads();
    return;
  }
  // ---- merge the four warps (in warp order)
  const float* mg = reinterpret_cast<const float*>(ring);
  constexpr int MLD = HD + 2;
  static_assert(4 * ROWS * MLD * 4 <= NS * L::STAGE_BYTES, "the warps' partials do not fit the ring");
  for (int e = tid; e < g * HD; e += DEC_THREADS) {
    const int row = e / HD, d = e - row * HD;
    float mx = -INFINITY;
#pragma unroll
    for (int w = 0; w < 4; ++w) mx = fmaxf(mx, mg[((size_t)w * ROWS + row) * MLD + HD]);
    float acc = 0.f, den = 0.f;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const float* src = mg + ((size_t)w * ROWS + row) * MLD;
      const float m = src[HD];
      if (m == -INFINITY) continue;
      const float sc = exp2f(m - mx);
      den += src[HD + 1] * sc;
      acc = fmaf(sc, src[d], acc);  // src[d] is the warp's unnormalised sum of p * v
    }
    const float inv = den > 0.f ? 1.f / den : 0.f;
    const int head = kvh * g + row;
    if (p.n_splits == 1) {
      p.out[(size_t)tok * p.ld_out + (size_t)head * HD + d] = __float2bfloat16_rn(acc * inv);
    } else if (CLUSTER) {
      // element e of the cluster's output is finished by rank e % size: send it this split's share
      const int epo = (g * HD + csize - 1) / csize;
      const uint32_t recv_a = smem_u32(recv);
      send_to_cta(recv_a + (uint32_t)(rank * epo + e / csize) * 4u, peers_in, e % csize, acc * inv);
      if (d == 0) {
        for (int c = 0; c < csize; ++c) {
          send_to_cta(recv_a + (uint32_t)(csize * epo + (rank * g + row) * 2) * 4u, peers_in, c, mx);
          send_to_cta(recv_a + (uint32_t)(csize * epo + (rank * g + row) * 2 + 1) * 4u, peers_in, c, den);
        }
      }
    } else {
      const size_t slot = ((size_t)split * p.part_stride_tokens + tok) * p.nq + head;
      p.part_o[slot * HD + d] = acc * inv;
      if (d == 0) {
        p.part_ml[slot * 2] = mx;
        p.part_ml[slot * 2 + 1] = den;
      }
    }
  }
  if (p.n_splits == 1) return;
  int n_merge = p.n_splits;  // partials that meet in global memory
  if constexpr (CLUSTER) {
    // ---- eight (or fewer) neighbouring splits are the CTAs of this cluster: every CTA has sent each
    // peer its share (asynchronous stores above, counted on the receiver's barrier) and, once all
    // bytes are in, finishes the elements e = rank, rank + size, ... from what it received, in index order
    const int group = split / csize;
    n_merge = p.n_splits / csize;
    // every thread sees the bytes of all shares counted in before it reads them
    const bool peers_ok = __syncthreads_and(mbar_wait_peers(peers_in, 0, p.error, ERR_DEC_PEERS));
    // (after this no peer touches this CTA's shared memory again; the first CTA of a cluster also
    // waits for `slices_out` below)
    if (!peers_ok) {
      if (n_merge > 1) {
        if (tid == 0) {
          mbar_arrive_cta(slices_out, 0);
          if (rank == 0) mbar_wait_peers(slices_out, 0, p.error, ERR_DEC_PEERS);
        }
        __syncthreads();
      }
      return;
    }
    const int epo = (g * HD + csize - 1) / csize;
    const float* recv_o = recv;
    const float* recv_ml = recv_o + csize * epo;
    for (int k = tid; k * csize + rank < g * HD; k += DEC_THREADS) {
      const int e = k * csize + rank;
      const int row = e / HD, d = e - row * HD;
      float m[8], l[8], v[8];
#pragma unroll
      for (int sp = 0; sp < 8; ++sp) {
        m[sp] = -INFINITY; l[sp] = 0.f; v[sp] = 0.f;
        if (sp < csize) {
          m[sp] = recv_ml[(sp * g + row) * 2];
          l[sp] = recv_ml[(sp * g + row) * 2 + 1];
          v[sp] = recv_o[sp * epo + k];
        }
      }
      float mx = -INFINITY;
#pragma unroll
      for (int sp = 0; sp < 8; ++sp) mx = fmaxf(mx, m[sp]);
      float acc = 0.f, den = 0.f;
#pragma unroll
      for (int sp = 0; sp < 8; ++sp) {
        if (sp < csize && m[sp] != -INFINITY) {
          const float w = l[sp] * exp2f(m[sp] - mx);
          den += w;
          acc = fmaf(w, v[sp], acc);
        }
      }
      const float inv = den > 0.f ? 1.f / den : 0.f;
      const int head = kvh * g + row;
      if (n_merge == 1) {
        p.out[(size_t)tok * p.ld_out + (size_t)head * HD + d] = __float2bfloat16_rn(acc * inv);
      } else {  // this cluster's partial: slot `group`
        const size_t slot = ((size_t)group * p.part_stride_tokens + tok) * p.nq + head;
        p.part_o[slot * HD + d] = acc * inv;
        if (d == 0) {
          p.part_ml[slot * 2] = mx;
          p.part_ml[slot * 2 + 1] = den;
        }
      }
    }
    if (n_merge == 1) return;  // (a CTA may leave at once: its peers read their own shared memory only)
    __threadfence();  // every CTA's slice of the cluster's partial is out before the leader counts it
    __syncthreads();
    if (tid == 0) mbar_arrive_cta(slices_out, 0);
    if (rank != 0) return;
    bool slices_ok = true;
    if (tid == 0) slices_ok = mbar_wait_peers(slices_out, 0, p.error, ERR_DEC_PEERS);
    if (!__syncthreads_and(slices_ok)) return;
  }
  // ---- the CTA (the cluster's leader) that arrives last for this (request, key/value head) merges
  // the partials, in index order whichever one that is
  __threadfence();  // (CLUSTER: what the leader has seen of its peers' slices goes on to whoever sees its count)
  __syncthreads();
  if (tid == 0) {
    const int old = atomicAdd(&p.done_count[seq * p.nkv + kvh], 1);
    flags[2] = (old == n_merge - 1);
    if (flags[2]) p.done_count[seq * p.nkv + kvh] = 0;  // ready for the next launch
  }
  __syncthreads();
  if (!flags[2]) return;
  __threadfence();
  const size_t split_stride = (size_t)p.part_stride_tokens * p.nq;
  float* m_s = reinterpret_cast<float*>(ring);  // [g][n_splits]
  float* l_s = m_s + ROWS * n_merge;         // [g][n_splits]
  __syncthreads();
  for (int idx = tid; idx < g * n_merge; idx += DEC_THREADS) {
    const int row = idx / n_merge, sp = idx - row * n_merge;
    const size_t slot = (size_t)tok * p.nq + kvh * g + row + sp * split_stride;
    m_s[row * n_merge + sp] = __ldcg(&p.part_ml[slot * 2]);
    l_s[row * n_merge + sp] = __ldcg(&p.part_ml[slot * 2 + 1]);
  }
  __syncthreads();
  for (int e = tid; e < g * HD; e += DEC_THREADS) {
    const int row = e / HD, d = e - row * HD;
    const size_t slot0 = (size_t)tok * p.nq + kvh * g + row;
    float mx = -INFINITY;
    for (int sp = 0; sp < n_merge; ++sp) mx = fmaxf(mx, m_s[row * n_merge + sp]);
    float acc = 0.f, den = 0.f;
    for (int s0 = 0; s0 < n_merge; s0 += 8) {  // eight splits' loads in flight; added in index order
      float v[8];
#pragma unroll
      for (int u = 0; u < 8; ++u)
        v[u] = (s0 + u < n_merge) ? __ldcg(&p.part_o[(slot0 + (s0 + u) * split_stride) * HD + d]) : 0.f;
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        if (s0 + u < n_merge) {
          const float m = m_s[row * n_merge + s0 + u];
          if (m != -INFINITY) {
            const float w = l_s[row * n_merge + s0 + u] * exp2f(m - mx);
            den += w;
            acc = fmaf(w, v[u], acc);
          }
        }
      }
    }
    const float inv = den > 0.f ? 1.f / den : 0.f;
    p.out[(size_t)tok * p.ld_out + (size_t)(kvh * g + row) * HD + d] = __float2bfloat16_rn(acc * inv);
  }
}

int g_cluster_merge = 1;  // 0: splits always merge through global memory (for comparisons)

template <int HD, bool DEEP>
size_t decode_smem_bytes(int keys_per_cta, int page_size, int cluster_group) {  // cluster_group: heads per kv head, 0 without clusters
  using L = DecLayout<HD, DEEP>;
  return (cluster_group ? (size_t)(cluster_group * (HD + 16) + 8) * sizeof(float) : 0) + 1024 + (size_t)L::STAGES * L::STAGE_BYTES + (size_t)ROWS * L::Q_LD * 2 + (2 * L::STAGES + 2) * 8 + 16 + 2 * HD * 2 +
         (size_t)((keys_per_cta + 2 * TK) / page_size + 4) * sizeof(int);
}

template <int HD, bool FUSED, bool DEEP, bool CLUSTER>
int launch_decode_ring(const CUtensorMap& mk, const CUtensorMap& mv, const DecParams& p, int n_seqs, cudaStream_t stream) {
  const int keys_per_cta = p.n_splits > 1 ? p.split_keys : p.max_blocks * p.page_size;
  const size_t smem = decode_smem_bytes<HD, DEEP>(keys_per_cta, p.page_size, CLUSTER ? p.nq / p.nkv : 0);
  if (smem > 200 * 1024) return 2;
  auto kernel = paged_attention_decode_tma_kernel<HD, FUSED, DEEP, CLUSTER>;
  static size_t attr_bytes = 0;  // the largest size asked for so far
  if (smem > attr_bytes) {
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) return 1;
    attr_bytes = smem;
  }
  const dim3 grid(n_seqs, p.nkv, p.n_splits);
  if (CLUSTER) launch_kernel_cluster(kernel, grid, DEC_THREADS, smem, dim3(1, 1, p.cluster_size), stream, mk, mv, p);
  else launch_kernel(kernel, grid, DEC_THREADS, smem, stream, mk, mv, p);
  return 0;
}

template <int HD, bool FUSED>
int launch_decode(const CUtensorMap& mk, const CUtensorMap& mv, DecParams p, int n_seqs, cudaStream_t stream) {
  const bool cluster = g_cluster_merge && p.n_splits >= 2;
  if (cluster) {  // 8 is the portable cluster size; more splits: whole clusters of 8 (the splits added are empty)
    p.cluster_size = p.n_splits <= 8 ? p.n_splits : 8;
    p.n_splits = (p.n_splits + p.cluster_size - 1) / p.cluster_size * p.cluster_size;
  }
  // at most three (head size 64) or two (128) CTAs with the long ring fit an SM of 148
  const long long ctas = (long long)n_seqs * p.nkv * p.n_splits;
  const bool deep = ctas <= (HD == 64 ? 444 : 296);
  if (cluster) return deep ? launch_decode_ring<HD, FUSED, true, true>(mk, mv, p, n_seqs, stream)
                           : launch_decode_ring<HD, FUSED, false, true>(mk, mv, p, n_seqs, stream);
  return deep ? launch_decode_ring<HD, FUSED, true, false>(mk, mv, p, n_seqs, stream)
              : launch_decode_ring<HD, FUSED, false, false>(mk, mv, p, n_seqs, stream);
}

}  // namespace

extern "C" void llm_attention_decode_cluster_merge(int on) { g_cluster_merge = on; }

// Whether the TMA decoding kernel takes this geometry: head size 64 or 128, a group of at most 16
// query heads, pages of 8, 16 or a multiple of 32 keys (a tile of 32 keys is whole pages or lies
// inside one).
extern "C" int llm_attention_decode_supported(int nq, int nkv, int hd, int page_size, long long ld_q, long long ld_out) {
  if (nkv <= 0 || nq % nkv || nq / nkv > ROWS) return 0;
  if (hd != 64 && hd != 128) return 0;
  if (!(page_size == 8 || page_size == 16 || (page_size > 0 && page_size % TK == 0))) return 0;
  return (ld_q % 8) == 0 && (ld_out % 2) == 0 && encode_fn() != nullptr;
}

namespace {

int decode_common(DecParams& p, const void* kcache, const void* vcache, long long n_cache_pages, int n_seqs, int hd,
                  float* scratch, bool fused, cudaStream_t stream) {
  LLM_REQUIRE(p.max_blocks > 0 && p.window >= 0 && n_cache_pages >= 1, "attention_decode: bad sizes");
  LLM_REQUIRE((reinterpret_cast<uintptr_t>(kcache) & 15u) == 0 && (reinterpret_cast<uintptr_t>(vcache) & 15u) == 0,
              "attention_decode: the caches must be 16-byte aligned");
  LLM_REQUIRE(p.n_splits >= 1 && p.n_splits <= 128 &&
              (p.n_splits == 1 || (p.split_keys > 0 && p.split_keys % 64 == 0 && scratch != nullptr && p.done_count != nullptr)),  // (the cluster form uses neither)
              "attention_decode: splits need split_keys %% 64 == 0, scratch and counters");
  LLM_REQUIRE((long long)n_seqs <= 65535 * 32768LL && p.nkv <= 65535, "attention_decode: batch too large for the grid");
  const long long rows = n_cache_pages * p.nkv * p.page_size;
  LLM_REQUIRE(rows < (1LL << 31), "attention_decode: the cache has too many rows for a tensor map coordinate");
  CUtensorMap mk, mv;
  const int box_rows = p.page_size < TK ? p.page_size : TK;
  LLM_REQUIRE(tensor_map_for(kcache, rows, hd, hd, box_rows, &mk) && tensor_map_for(vcache, rows, hd, hd, box_rows, &mv),
              "attention_decode: cannot encode the tensor maps of the cache");
  p.page_shift = -1;
  for (int sft = 0; sft < 30; ++sft)
    if ((1 << sft) == p.page_size) p.page_shift = sft;
  p.null_page = (int)(n_cache_pages - 1);
  const int split_keys_asked = p.split_keys;
  if (p.n_splits == 1) p.split_keys = p.max_blocks * p.page_size + TK;
  p.part_stride_tokens = n_seqs;
  p.part_o = scratch;
  p.part_ml = scratch ? scratch + (size_t)p.n_splits * n_seqs * p.nq * hd : nullptr;
  p.error = error_word();
  int rc;
  if (fused) rc = hd == 64 ? launch_decode<64, true>(mk, mv, p, n_seqs, stream) : launch_decode<128, true>(mk, mv, p, n_seqs, stream);
  else rc = hd == 64 ? launch_decode<64, false>(mk, mv, p, n_seqs, stream) : launch_decode<128, false>(mk, mv, p, n_seqs, stream);
  LLM_REQUIRE(rc != 2, "attention_decode: %d keys per split with pages of %d do not fit the block-table copy in shared memory",
              p.n_splits > 1 ? split_keys_asked : p.max_blocks * p.page_size, p.page_size);
  LLM_REQUIRE(rc == 0, "attention_decode: cannot raise the shared memory limit");
  LLM_CHECK_LAUNCH("paged_attention_decode");
  return LLM_OK;
}

}  // namespace

// One token per request. q: rows of [nq*hd] bf16 (ld_q elements apart); caches
// [n_cache_pages, nkv, page_size, hd] bf16, whose LAST page is the null page (finite values, never a
// request's); seq_start[i]: the token's position; seq_qoff[i]: its row; out [n_seqs, nq*hd] bf16.
// n_splits > 1: keys are cut every split_keys (a multiple of 64) positions, scratch holds
// llm_attention_mma_scratch_floats floats and done_count n_seqs * nkv zeroed ints (left at zero).
extern "C" int llm_paged_attention_decode(const void* q, long long ld_q, const void* kcache, const void* vcache,
                                          long long n_cache_pages, const int* seq_start, const int* seq_qoff,
                                          const int* block_table, int max_blocks, void* out, long long ld_out, int n_seqs,
                                          int nq, int nkv, int hd, int page_size, float scale, int window, int n_splits,
                                          int split_keys, float* scratch, int* done_count, cudaStream_t stream) {
  if (n_seqs == 0) return LLM_OK;
  LLM_REQUIRE(llm_attention_decode_supported(nq, nkv, hd, page_size, ld_q, ld_out),
              "attention_decode: geometry not supported (nq=%d nkv=%d hd=%d page=%d)", nq, nkv, hd, page_size);
  LLM_REQUIRE((reinterpret_cast<uintptr_t>(q) & 15u) == 0, "attention_decode: q must be 16-byte aligned");
  DecParams p = {};
  p.q = (const bf16*)q; p.ld_q = ld_q; p.seq_start = seq_start; p.seq_qoff = seq_qoff; p.block_table = block_table;
  p.max_blocks = max_blocks; p.nq = nq; p.nkv = nkv; p.page_size = page_size; p.window = window;
  p.scale = scale; p.out = (bf16*)out; p.ld_out = ld_out;
  p.n_splits = n_splits; p.split_keys = split_keys; p.done_count = done_count;
  return decode_common(p, kcache, vcache, n_cache_pages, n_seqs, hd, scratch, false, stream);
}

// The same with the q|k|v product, rotation and cache write folded in: qkv_parts float32
// [n_parts][tokens][(nq + 2 nkv) * hd] partial sums (parts part_stride floats apart; the values are
// their sums in index order), cos/sin float32 [positions][hd / 2] or both null for no rotation. The
// token's own key (rotated) and value are written into the caches at its position.
extern "C" int llm_paged_attention_decode_fused(const float* qkv_parts, int n_parts, long long part_stride, const float* cos_t,
                                                const float* sin_t, void* kcache, void* vcache, long long n_cache_pages,
                                                const int* seq_start, const int* seq_qoff, const int* block_table,
                                                int max_blocks, void* out, long long ld_out, int n_seqs, int nq, int nkv, int hd,
                                                int page_size, float scale, int window, int n_splits, int split_keys,
                                                float* scratch, int* done_count, const float* sumsq, int n_sumsq,
                                                float inv_dim, float eps, cudaStream_t stream) {
  if (n_seqs == 0) return LLM_OK;
  LLM_REQUIRE(llm_attention_decode_supported(nq, nkv, hd, page_size, 8, ld_out),
              "attention_decode: geometry not supported (nq=%d nkv=%d hd=%d page=%d)", nq, nkv, hd, page_size);
  LLM_REQUIRE(sumsq == nullptr || n_sumsq > 0, "attention_decode: a row scale needs its parts");
  LLM_REQUIRE(qkv_parts != nullptr && n_parts >= 1 && part_stride >= (long long)n_seqs * (nq + 2 * nkv) * hd,
              "attention_decode: bad partial sums");
  LLM_REQUIRE((cos_t == nullptr) == (sin_t == nullptr), "attention_decode: cos and sin come together");
  DecParams p = {};
  p.seq_start = seq_start; p.seq_qoff = seq_qoff; p.block_table = block_table;
  p.max_blocks = max_blocks; p.nq = nq; p.nkv = nkv; p.page_size = page_size; p.window = window;
  p.scale = scale; p.out = (bf16*)out; p.ld_out = ld_out;
  p.n_splits = n_splits; p.split_keys = split_keys; p.done_count = done_count;
  p.qkv_parts = qkv_parts; p.n_parts = n_parts; p.part_stride = part_stride; p.cos_t = cos_t; p.sin_t = sin_t;
  p.rs = RowScale{sumsq, n_sumsq, inv_dim, eps};
  p.kcache = (bf16*)kcache; p.vcache = (bf16*)vcache;
  return decode_common(p, kcache, vcache, n_cache_pages, n_seqs, hd, scratch, true, stream);
}
