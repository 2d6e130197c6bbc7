// Helpers shared by the tcgen05 / TMA kernels: mbarriers with bounded waits, TMA loads, shared-memory
// matrix descriptors, tensor-memory loads and stores, tensor maps (made on the host, kept by
// address and shape) and the per-process error word that a kernel sets when it gives up a wait.
#pragma once

#include <cuda.h>

#include <algorithm>
#include <mutex>
#include <tuple>
#include <unordered_map>

#include "common.cuh"

int* llm_tc_error_word();  // one int of device memory per process for the kernels' error codes (gemm_tc.cu)

namespace {

constexpr int BM = 128;  // accumulator lanes = rows of A per tile
constexpr int BK = 64;   // 64 bf16 = 128 bytes = one row of the 128-byte swizzle
constexpr int A_BYTES = BM * BK * 2;
constexpr long long WAIT_CYCLES = 2000000000LL;  // about one second

enum : int { ERR_PRODUCER = 1, ERR_MMA = 2, ERR_EPILOGUE = 3, ERR_DRAIN = 4 };

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}

__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}

// Bounded wait. Returns false if the phase did not complete in time or another role aborted. Once
// any kernel of the process has recorded an error, a wait that has lasted longer than any wait of
// a healthy kernel (RECHECK_CYCLES) gives up instead of waiting out its full second: everything
// computed since that error is void anyway (the host raises when it reads the word), and a fault
// that repeats in every launch then costs tens of microseconds, not seconds, per launch. The word
// lives in global memory, so it is looked at only that rarely: a load of it stalls the polling
// thread for a microsecond, which the roles of a pipeline cannot spare in every wait.
constexpr long long RECHECK_CYCLES = 100000;  // about 50 us
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag, int* error_out, int code) {
  if (mbar_try_wait(bar, parity)) return true;  // the usual case costs one instruction
  const long long t0 = clock64();
  long long next_check = t0 + RECHECK_CYCLES;
  for (uint32_t i = 0;; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((i & 255u) == 255u) {
      if (*abort_flag) return false;
      const long long now = clock64();
      if (now > next_check) {
        next_check = now + RECHECK_CYCLES;
        if (*reinterpret_cast<volatile int*>(error_out) != 0) {
          *abort_flag = code;
          return false;
        }
        if (now - t0 > WAIT_CYCLES) {
          *abort_flag = code;
          atomicCAS(error_out, 0, code);
          return false;
        }
      }
    }
  }
}

// Last wait of a role that is leaving early: for copies or products that it (or its CTA) issued and
// that still write shared or tensor memory. It looks at no abort flag and at no error word, since
// the memory may not be given up before they are done; twice the bound of the waits above, so that
// a role which itself waits out a full bound still gets here in time.
__device__ __forceinline__ void mbar_drain(uint64_t* bar, uint32_t parity, int* error_out) {
  const long long t0 = clock64();
  while (!mbar_try_wait(bar, parity)) {
    if (clock64() - t0 > 2 * WAIT_CYCLES) {
      atomicCAS(error_out, 0, (int)ERR_DRAIN);
      return;
    }
  }
}

__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(
          smem_u32(dst)),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(x), "r"(y)
      : "memory");
}

// Shared-memory matrix descriptor: K-major tile with 128-byte swizzle; rows are 128 bytes apart,
// groups of 8 rows 1024 bytes apart.
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t addr) {
  uint64_t d = 0;
  d |= (uint64_t)((addr & 0x3FFFFu) >> 4);  // start address, bits [0,14)
  d |= (uint64_t)1 << 16;                   // leading byte offset (unused with swizzle), bits [16,30)
  d |= (uint64_t)(1024 >> 4) << 32;         // stride byte offset, bits [32,46)
  d |= (uint64_t)1 << 46;                   // descriptor version of sm_100
  d |= (uint64_t)2 << 61;                   // 128-byte swizzle
  return d;
}

// Instruction descriptor of kind::f16: bf16 x bf16 -> f32, both operands K-major, M = 128, N = n.
__host__ __device__ constexpr uint32_t instr_desc(int n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
}

__device__ __forceinline__ void mma_f16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
      "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}

__device__ __forceinline__ void mma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ void tmem_load16(uint32_t taddr, float* v) {
  uint32_t r[16];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}

// Stage and phase of a ring, stepped without a division.
struct RingPos {
  int s;
  uint32_t ph;
  int stages;
  __device__ __forceinline__ RingPos(int stages_, int s_ = 0, uint32_t ph_ = 0) : s(s_), ph(ph_), stages(stages_) {}
  __device__ __forceinline__ void next() {
    if (++s == stages) {
      s = 0;
      ph ^= 1u;
    }
  }
};

// ------------------------------------------------------------------------------------ host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

struct MapKey {
  const void* ptr;
  long long rows, cols, ld;
  int box_rows;
  bool operator==(const MapKey& o) const { return ptr == o.ptr && rows == o.rows && cols == o.cols && ld == o.ld && box_rows == o.box_rows; }
};
struct MapKeyHash {
  size_t operator()(const MapKey& k) const {
    size_t h = reinterpret_cast<size_t>(k.ptr);
    for (long long v : {k.rows, k.cols, k.ld, (long long)k.box_rows}) h = h * 1000003u ^ (size_t)v;
    return h;
  }
};

// Tensor map of a row-major bf16 matrix [rows, cols] with row stride ld (elements): boxes of
// box_rows x 64 elements, 128-byte swizzle, zeros outside the matrix. Encoding is host-only work;
// maps are kept by (pointer, shape) since weights and workspaces keep their addresses.
bool tensor_map_for(const void* ptr, long long rows, long long cols, long long ld, int box_rows, CUtensorMap* out) {
  static std::mutex mu;
  static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
  const MapKey key{ptr, rows, cols, ld, box_rows};
  std::lock_guard<std::mutex> lock(mu);
  auto it = cache.find(key);
  if (it != cache.end()) {
    *out = it->second;
    return true;
  }
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUtensorMap m;
  CUresult r = fn(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return false;
  if (cache.size() > 8192) cache.clear();
  cache.emplace(key, m);
  *out = m;
  return true;
}

inline int* error_word() { return llm_tc_error_word(); }


}  // namespace
