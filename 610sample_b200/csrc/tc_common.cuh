// Definitions shared by the tensor-core kernel files: tile sizes, warp roles,
// tensor-map bundle and small device helpers.
#pragma once

#include "attn_common.cuh"
#include "tc_primitives.cuh"

namespace attn {
namespace tc {

constexpr int BM = 128;            // stationary rows per CTA
constexpr int BN = 64;             // streamed rows per iteration
constexpr int kMathWarps = 8;
constexpr int kMathThreads = kMathWarps * 32;
constexpr int kProducerWarp = 8;   // the MMA-issuing warps follow it
constexpr int kTmemCols = 512;
constexpr uint32_t kAtomBytesStat = BM * 128;   // [128 rows][64 halves], 16 KB
constexpr uint32_t kAtomBytesStrm = BN * 128;   // [ 64 rows][64 halves],  8 KB

// Kernel ids inside device status codes (the backward kernels use 18 and 19, the forward kernel
// 20, the self-test 0x6f); the values are documented with the C ABI and do not change.
enum Kind { HVP_PRE = 4, HVP_ROW = 5, HVP_COL = 6 };
enum TensorId { T_Q = 0, T_K, T_V, T_dO, T_gQ, T_gK, T_gV, T_COUNT };

// Output tensors by operation: forward {O}; backward {dQ, dK, dV}; double backward
// {g_dO, g_Q, g_K, g_V}.  Output maps have a box of 64 columns x 128 rows.
enum OutId { TO_O = 0, TO_dQ = 0, TO_dK = 1, TO_dV = 2, TO_gdO = 0, TO_gQ = 1, TO_gK = 2, TO_gV = 3, TO_COUNT = 4 };

struct TmaMaps { CUtensorMap m[T_COUNT]; CUtensorMap out[TO_COUNT]; };

// Control block of the single-tile self-test kernel (every attention kernel has its own).
struct Control {
  uint64_t stat_full;
  uint64_t acc_done;
  uint32_t tmem_base;
  volatile uint32_t abort_flag;
};

// status codes: (kind + 1) << 8 | wait id
__device__ __forceinline__ uint32_t wait_code(int kind, int id) { return ((uint32_t)(kind + 1) << 8) | (uint32_t)id; }

template <typename T> struct Pack;
template <> struct Pack<__nv_bfloat16> {
  static constexpr int kIsBf16 = 1;
  static __device__ __forceinline__ uint32_t pack(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
  }
  static __device__ __forceinline__ float2 unpack(uint32_t w) {
    return __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&w));
  }
};
template <> struct Pack<__half> {
  static constexpr int kIsBf16 = 0;
  static __device__ __forceinline__ uint32_t pack(float lo, float hi) {
    __half2 v = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
  }
  static __device__ __forceinline__ float2 unpack(uint32_t w) {
    return __half22float2(*reinterpret_cast<__half2*>(&w));
  }
};

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// 16 packed halves (two 16-byte chunks) of operand-tile row `row`, columns
// [col0, col0+16), into a 128-byte-swizzled [128][64] tile.
__device__ __forceinline__ void store_op16(uint32_t tile, int row, int col0, const uint32_t (&v)[8]) {
  const uint32_t a0 = tile + sw128_offset(row, col0);
  const uint32_t a1 = tile + sw128_offset(row, col0 + 8);
  asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(a0), "r"(v[0]), "r"(v[1]), "r"(v[2]),
               "r"(v[3])
               : "memory");
  asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(a1), "r"(v[4]), "r"(v[5]), "r"(v[6]),
               "r"(v[7])
               : "memory");
}


// Epilogue of the tensor-core kernels.  The 256 math threads have written a [128 rows][cols]
// half-precision result tile to shared memory at `tile`, one 128-byte-swizzled 16 KB atom per 64
// columns (store_op16).  All of them call this; `leader` (one thread) then writes the tile to
// rows [row0, row0 + 128) of plane `plane` with one TMA store per atom (rows and columns beyond
// the tensor are clipped by the map) and returns once shared memory has been read.
__device__ __forceinline__ void store_tile_tma(const CUtensorMap* map, uint32_t tile, int cols, int row0, int plane,
                                               bool leader) {
  fence_proxy_async_smem();
  named_barrier_sync(2, kMathWarps * 32);
  if (leader) {
    for (int a = 0; a * 64 < cols; ++a) tma_store_3d(map, tile + (uint32_t)a * kAtomBytesStat, a * 64, row0, plane);
    bulk_commit_group();
    bulk_wait_group_read_all();
  }
}

}  // namespace tc
}  // namespace attn
