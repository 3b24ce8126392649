// Blackwell (sm_100a) primitives used by the tensor-core attention kernels:
// mbarriers with bounded waits, TMA tile loads, tensor-memory allocation,
// tcgen05.mma issue/commit, tcgen05.ld, and the shared-memory / instruction
// descriptors those need.  Everything is inline PTX; nothing here depends on a
// library.
#pragma once

#include <cuda_runtime.h>
#include <cuda.h>
#include <stdint.h>

namespace attn {
namespace tc {

// ---------------------------------------------------------------------------
// addresses
// ---------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// ---------------------------------------------------------------------------
// mbarrier
// ---------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}

// Every wait in these kernels is bounded.  A wait that is still unsatisfied
// after kWaitLimitCycles SM clocks (about two seconds) stores `code` in the
// device status word, raises the CTA's abort flag and returns false; the other
// roles see the flag in their own waits and leave as well.
constexpr long long kWaitLimitCycles = 4000000000LL;

// The device status word is the first member of this block (one per device, owned by the
// library).  `host_mirror`, when set, is a page-locked host word that a kernel giving up on a wait
// writes its code to as well, so that the host can notice a time-out by reading its own memory,
// without a copy or a synchronisation.
struct StatusBlock {
  unsigned int word;
  unsigned int reserved;
  unsigned int* host_mirror;
};

__device__ __forceinline__ void report_timeout(unsigned int* status, uint32_t code) {
  if (status == nullptr) return;
  atomicCAS(status, 0u, code);
  unsigned int* mirror = *reinterpret_cast<unsigned int* volatile*>(&reinterpret_cast<StatusBlock*>(status)->host_mirror);
  if (mirror != nullptr) {
    *reinterpret_cast<volatile unsigned int*>(mirror) = code;
    __threadfence_system();
  }
}

__device__ __forceinline__ bool mbar_wait_limit(uint32_t bar, uint32_t parity, volatile uint32_t* abort_flag,
                                                unsigned int* status, uint32_t code, long long limit_cycles) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  while (true) {
    if (mbar_try_wait(bar, parity)) return true;
    if (*abort_flag != 0u) return false;
    if (clock64() - t0 > limit_cycles) {
      *abort_flag = 1u;
      report_timeout(status, code);
      return false;
    }
  }
}

__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile uint32_t* abort_flag,
                                          unsigned int* status, uint32_t code) {
  return mbar_wait_limit(bar, parity, abort_flag, status, code, kWaitLimitCycles);
}

__device__ __forceinline__ void fence_barrier_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
// generic-proxy writes to shared memory -> visible to the async proxy (TMA, tcgen05.mma)
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void named_barrier_sync(uint32_t id, uint32_t threads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

// ---------------------------------------------------------------------------
// TMA: 3-D tiled load, global -> shared, completion on an mbarrier.
// The innermost coordinate x is always a multiple of 64 half-precision elements
// here (128 bytes), which satisfies the 16-byte rule for TMA start addresses.
// ---------------------------------------------------------------------------
__device__ __forceinline__ void tma_load_3d(uint32_t smem_dst, const CUtensorMap* map, int x, int y,
                                            int z, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%2, %3, %4}], [%5];"
      ::"r"(smem_dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(z), "r"(bar)
      : "memory");
}
// 3-D tiled store, shared -> global, as part of the thread's current bulk group.  Elements of
// the box that fall outside the tensor are not written.  x is a multiple of 64 elements and no
// coordinate is negative wherever this is used.
__device__ __forceinline__ void tma_store_3d(const CUtensorMap* map, uint32_t smem_src, int x, int y, int z) {
  asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];"
               ::"l"(reinterpret_cast<uint64_t>(map)), "r"(smem_src), "r"(x), "r"(y), "r"(z)
               : "memory");
}
__device__ __forceinline__ void bulk_commit_group() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// returns once the bulk groups of this thread have finished reading shared memory
__device__ __forceinline__ void bulk_wait_group_read_all() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
}

// ---------------------------------------------------------------------------
// tensor memory
// ---------------------------------------------------------------------------
// One full warp allocates `cols` (power of two, >= 32) columns; the base address
// is written to shared memory at `dst_smem`.
__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem),
               "r"(cols)
               : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols)
               : "memory");
}
__device__ __forceinline__ void tc_fence_before_sync() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after_sync() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// Load 16 consecutive 32-bit columns of this thread's lane, then wait for the
// data.  The wait names the registers so that no use can be scheduled above it.
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait(uint32_t (&r)[16]) {
  asm volatile("tcgen05.wait::ld.sync.aligned;"
               : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]),
                 "+r"(r[7]), "+r"(r[8]), "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]),
                 "+r"(r[13]), "+r"(r[14]), "+r"(r[15])
               :
               : "memory");
}

// Store 8 consecutive 32-bit columns of this thread's lane (16 packed halves).
__device__ __forceinline__ void tmem_st8(uint32_t taddr, const uint32_t (&r)[8]) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
               ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]),
                 "r"(r[7])
               : "memory");
}
__device__ __forceinline__ void tmem_st_wait() {
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

// ---------------------------------------------------------------------------
// descriptors
// ---------------------------------------------------------------------------
// Shared-memory matrix descriptor, 128-byte swizzle.  Bit fields:
//   [0,14)  start address >> 4        [16,30) leading byte offset >> 4
//   [32,46) stride byte offset >> 4   [46,48) version (1 on sm_100)
//   [61,64) layout type (2 = 128-byte swizzle)
// K-major operand ([rows][64 elements], rows 128 bytes apart, 8-row groups 1024
// bytes apart): SBO = 1024, LBO unused.  MN-major operand (same bytes read with
// the contiguous direction as M/N): SBO = 1024 between 8-row K groups, LBO =
// distance between successive 64-element blocks along M/N.
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t addr, uint32_t lbo_bytes,
                                                    uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= (uint64_t)((addr >> 4) & 0x3FFFu);
  d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFFu) << 16;
  d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFFu) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}

// Instruction descriptor for kind::f16 (f16/bf16 operands, fp32 accumulate):
//   [4,6) D format (1 = f32)   [7,10) A format   [10,13) B format (0 f16, 1 bf16)
//   [15] A major   [16] B major (0 = K-major, 1 = MN-major)
//   [17,23) N >> 3             [24,29) M >> 4
// A and B have to be given the same format: on this hardware an instruction whose descriptor
// names f16 for A and bf16 for B raises "illegal instruction".
__host__ __device__ constexpr uint32_t make_idesc(int M, int N, int is_bf16, int a_mn_major,
                                                  int b_mn_major) {
  return (1u << 4) | ((uint32_t)is_bf16 << 7) | ((uint32_t)is_bf16 << 10) |
         ((uint32_t)a_mn_major << 15) | ((uint32_t)b_mn_major << 16) | ((uint32_t)(N >> 3) << 17) |
         ((uint32_t)(M >> 4) << 24);
}

// D[tmem] (+)= A[smem] * B[smem]; one K = 16 step.  Issued by a single thread.
__device__ __forceinline__ void mma_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                       uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// Same with the A operand read from tensor memory: lane = row of A, one 32-bit
// column holds two consecutive K elements, so a K = 16 step reads 8 columns
// starting at a_tmem.  A must be K-major.
__device__ __forceinline__ void mma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                       uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// One lane of a converged warp (true in exactly one lane).  The MMA warps run
// their loops converged and issue through the elected lane, which lets the
// compiler keep descriptors in uniform registers.
__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile("{\n\t.reg .pred P;\n\telect.sync _|P, 0xffffffff;\n\tselp.u32 %0, 1, 0, P;\n\t}" : "=r"(pred));
  return pred != 0;
}

// The mbarrier receives one arrival once every tcgen05.mma issued so far by this
// thread has completed (implies tcgen05.fence::before_thread_sync).
__device__ __forceinline__ void mma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
               : "memory");
}

// Byte offset of element (row, col) of a [rows][64] half-precision tile stored
// with the 128-byte swizzle (tile base 1024-byte aligned): the 16-byte chunk
// index is XORed with row % 8.
__host__ __device__ constexpr uint32_t sw128_offset(uint32_t row, uint32_t col) {
  return row * 128u + ((((col >> 3) ^ (row & 7u)) & 7u) << 4) + ((col & 7u) << 1);
}

}  // namespace tc
}  // namespace attn
