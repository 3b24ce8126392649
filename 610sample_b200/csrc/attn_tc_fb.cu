// First-backward attention kernels on sm_100a (f16/bf16, D a multiple of 16 up to 128).
//
// Two kinds of one kernel.  A CTA owns 128 STATIONARY rows of one (batch, head) and streams
// 64-row tiles of the other axis through as many TMA stages as fit in shared memory (five to eight):
//
//   kind      stationary     streamed   tensor-memory score regions        produces
//   BWD_ROW   Q, dO          K, V       RA = S, RB = dP        (x2 each)   dQ = s dS K
//   BWD_COL   K, V           Q, dO      RA = S^T, RB = dP^T    (x1 each)   dV = P^T dO, dK = s dS^T Q
//
// The stationary operands are copied once from shared memory into TENSOR MEMORY and serve from
// there as the A operand of every score product (a stationary operand left in shared memory
// would be re-read by each MMA instruction: measured 48 instead of 32 clocks for N = 64).  The
// math warps read a score region with tcgen05.ld, evaluate P = exp(S - L) from the saved
// log-sum-exp, and write the half-precision operands of the output products (P, dS) back over the
// score columns they have read; the output products take them from there as their A operand.
// BWD_COL computes transposed scores (keys on the TMEM lanes) so that operand roles are the same
// as in the row kind; its per-query scalars (L, Dv) are staged in shared memory per tile.
// Two warps issue the MMAs, each batch by one elected lane inside a single branch: one the score
// products S (a region is free again as soon as its scores are in the math warps' registers), the
// other the outputs of a tile followed by the dP products that overwrite their operands (its own
// program order is the only ordering needed).  In the row kind the eight math warps form two
// groups of four that take alternate tiles (= alternate buffers of the two regions), a thread
// owning a whole row of its tile, so that one group computes while the other waits for its
// products or for tensor-memory reads (clock stamps: tile period 1 479 -> 1 281 clk with the
// groups alone, the issuing warp then being the limit; with the second issuing warp the row
// kernel takes 368 instead of 408 us at B4 H16 N4096 D128).  The column kind has no room for
// second buffers at D = 128 and keeps all eight warps on one tile.  Head dimensions
// below the tile width run zero-padded (TMA fills the padding) with the padding k-steps and
// columns skipped.  Result tiles leave through shared memory and TMA stores.
// (The forward pass is in attn_tc_fwd.cu.)
// Reference kernels: csrc/flash_double_backward_v7.cu:649-1016.
#include "attn_launch.h"
#include "tc_common.cuh"

namespace attn {
namespace tc {

enum FbKind { FB_BWD_ROW = 2, FB_BWD_COL = 3 };   // numbering of launch_fwd_bwd

constexpr int kFbMmaWarp = 9;
constexpr int kFbThreads = 352;    // 8 math warps, TMA producer, two MMA issuers
constexpr int kFbMaxStages = 8;

struct FbControl {
  uint64_t staging_full;
  uint64_t stat_ready;
  uint64_t stream_full[kFbMaxStages];
  uint64_t stream_empty[kFbMaxStages];
  uint64_t ra_full[2];
  uint64_t rb_full[2];
  uint64_t op_full[2];       // math warps are done with the regions of a tile (operands written)
  uint64_t ra_free[2];       // the scores of a tile are in the math warps' registers
  uint64_t acc_done;
  uint64_t stats_ready[2];
  uint32_t tmem_base;
  volatile uint32_t abort_flag;
};

template <int KIND, int D>
struct FbCfg {
  static constexpr bool kCol = (KIND == FB_BWD_COL);
  static constexpr int kAtoms = D / 64;
  static constexpr int kNStat = 2;
  static constexpr int kNStream = 2;
  static constexpr int kBufs = kCol ? 1 : 2;
  static constexpr int kNOut = kCol ? 2 : 1;
  static constexpr uint32_t kStagingBytes = kNStat * kAtoms * kAtomBytesStat;
  static constexpr uint32_t kStageBytes = kNStream * kAtoms * kAtomBytesStrm;
  static constexpr uint32_t kAuxBytes = 512 + 2048;   // control; per-query scalars / L exchange
  // as many stream stages as fit (at most eight): a TMA load takes about 2 000 clocks from request
  // to arrival and a tile of these kernels much less, so the loads have to run several tiles ahead
  static constexpr uint32_t kMaxSmem = 232448;
  static constexpr int kFit = (int)((kMaxSmem - 1024 - kStagingBytes - kAuxBytes) / kStageBytes);
  static constexpr int kStages = kFit < kFbMaxStages ? kFit : kFbMaxStages;
  static_assert(kStages >= 3, "too few stream stages");
  static constexpr uint32_t kContentBytes = kStagingBytes + kStages * kStageBytes + kAuxBytes;
  static constexpr uint32_t kSmemBytes = kContentBytes + 1024;
  // tensor-memory columns
  static constexpr int kRA = 0;
  static constexpr int kRB = kCol ? 64 : 128;
  static constexpr int kStat = kCol ? 128 : 384;      // stationary operand x at kStat + 64 x
  static constexpr int kOut = 256;
  static_assert(kOut + kNOut * D <= (kCol ? 512 : 384), "tensor memory over-subscribed");
  __host__ __device__ static constexpr uint32_t stream_off(int slot, int atom) {
    return (uint32_t)(slot * kAtoms + atom) * kAtomBytesStrm;
  }
  __host__ __device__ static constexpr int stat_tensor(int x) { return kCol ? (x == 0 ? T_K : T_V) : (x == 0 ? T_Q : T_dO); }
  __host__ __device__ static constexpr int stream_tensor(int s) { return kCol ? (s == 0 ? T_Q : T_dO) : (s == 0 ? T_K : T_V); }
};

template <int KIND, int D, typename T>
__global__ void __launch_bounds__(kFbThreads, 1)
fb_kernel(const __grid_constant__ TmaMaps maps, const Geometry g, const Tensors t) {
  using CF = FbCfg<KIND, D>;
  constexpr int kAtoms = CF::kAtoms;
  constexpr int kBufs = CF::kBufs;
  constexpr int KCODE = 16 + KIND;     // kernel id inside device status codes
  constexpr uint32_t kIdesc64 = make_idesc(BM, 64, Pack<T>::kIsBf16, 0, 0);

  extern __shared__ __align__(1024) uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  {
    uint32_t dyn_size;
    asm("mov.u32 %0, %%dynamic_smem_size;" : "=r"(dyn_size));
    if (smem_base - smem_u32(smem_raw) + CF::kContentBytes > dyn_size) {   // uniform over the CTA
      if (threadIdx.x == 0 && t.status != nullptr) atomicCAS(t.status, 0u, wait_code(KCODE, 15));
      return;
    }
  }
  const uint32_t staging = smem_base;
  const uint32_t strm_base = staging + CF::kStagingBytes;
  const uint32_t aux_off = CF::kStagingBytes + CF::kStages * CF::kStageBytes;
  FbControl* ctl = reinterpret_cast<FbControl*>(smem_gen + aux_off);
  float* aux_f = reinterpret_cast<float*>(smem_gen + aux_off + 512);   // 512 floats

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_stat = CF::kCol ? g.N_kv : g.N_q;
  const int tiles = (n_stat + BM - 1) / BM;
  int bh, rank;
  cta_to_head_and_rank(g, tiles, bh, rank);
  const int tile = (CF::kCol || g.mask_mode != 0) ? rank : (tiles - 1 - rank);   // heavy tiles first
  const int r0 = tile * BM;

  int lo, hi;
  if (CF::kCol) query_range_for_keys(g, r0, r0 + BM, lo, hi);
  else key_range_for_queries(g, r0, r0 + BM, lo, hi);
  const int t_begin = lo / BN;
  const int n_iter = (hi > lo) ? ((hi + BN - 1) / BN - t_begin) : 0;

  const uint32_t bar_staging_full = smem_u32(&ctl->staging_full), bar_stat_ready = smem_u32(&ctl->stat_ready);
  const uint32_t bar_acc_done = smem_u32(&ctl->acc_done);
  auto bar_ra_free = [&](int b) { return smem_u32(&ctl->ra_free[b]); };
  auto bar_stream_full = [&](int s) { return smem_u32(&ctl->stream_full[s]); };
  auto bar_stream_empty = [&](int s) { return smem_u32(&ctl->stream_empty[s]); };
  auto bar_ra_full = [&](int b) { return smem_u32(&ctl->ra_full[b]); };
  auto bar_rb_full = [&](int b) { return smem_u32(&ctl->rb_full[b]); };
  auto bar_op_full = [&](int b) { return smem_u32(&ctl->op_full[b]); };

  if (threadIdx.x == 0) {
    mbar_init(bar_staging_full, 1);
    mbar_init(bar_stat_ready, kMathWarps);
    for (int s = 0; s < CF::kStages; ++s) {
      mbar_init(bar_stream_full(s), 1);
      mbar_init(bar_stream_empty(s), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(bar_ra_full(b), 1);
      mbar_init(bar_rb_full(b), 1);
      // row kind: a tile belongs to one group of four math warps
      mbar_init(bar_op_full(b), CF::kCol ? kMathWarps : kMathWarps / 2);
      mbar_init(bar_ra_free(b), CF::kCol ? kMathWarps : kMathWarps / 2);
      mbar_init(smem_u32(&ctl->stats_ready[b]), kMathWarps);
    }
    mbar_init(bar_acc_done, 1);
    ctl->abort_flag = 0u;
    ctl->tmem_base = 0u;
    fence_barrier_init();
    fence_proxy_async_smem();
  }
  __syncthreads();
  if (warp == kFbMmaWarp) tmem_alloc(smem_u32(&ctl->tmem_base), kTmemCols);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = ctl->tmem_base;
  volatile uint32_t* abort_flag = &ctl->abort_flag;

  // =========================================================================
  // TMA producer
  // =========================================================================
  if (warp == kProducerWarp) {
    if (lane == 0 && n_iter > 0) {
      for (int i = 0; i < T_COUNT; ++i) tma_prefetch_desc(&maps.m[i]);
      mbar_arrive_expect_tx(bar_staging_full, CF::kStagingBytes);
#pragma unroll
      for (int x = 0; x < CF::kNStat; ++x)
#pragma unroll
        for (int a = 0; a < kAtoms; ++a)
#pragma unroll
          for (int h = 0; h < 2; ++h)
            tma_load_3d(staging + (x * kAtoms + a) * kAtomBytesStat + h * kAtomBytesStrm,
                        &maps.m[CF::stat_tensor(x)], a * 64, r0 + h * 64, bh, bar_staging_full);
      bool ok = true;
      for (int it = 0; it < n_iter; ++it) {
        const int st = it % CF::kStages;
        ok = mbar_wait(bar_stream_empty(st), ((it / CF::kStages) & 1) ^ 1, abort_flag, t.status, wait_code(KCODE, 1));
        if (!ok) break;
        mbar_arrive_expect_tx(bar_stream_full(st), CF::kStageBytes);
        const uint32_t stage = strm_base + st * CF::kStageBytes;
#pragma unroll
        for (int s = 0; s < CF::kNStream; ++s)
#pragma unroll
          for (int a = 0; a < kAtoms; ++a)
            tma_load_3d(stage + CF::stream_off(s, a), &maps.m[CF::stream_tensor(s)], a * 64,
                        (t_begin + it) * BN, bh, bar_stream_full(st));
      }
      if (!ok) {   // give copies already in flight a bounded chance to land before the CTA exits
        const long long t0 = clock64();
        while (clock64() - t0 < 2000000LL) { }
      }
    }
  }
  // =========================================================================
  // MMA issuer (converged warp, one elected lane issues)
  // =========================================================================
  else if (warp == kFbMmaWarp || warp == kFbMmaWarp + 1) {
    if (n_iter > 0) {
      bool ok = mbar_wait(bar_stat_ready, 0, abort_flag, t.status, wait_code(KCODE, 2));
      ok = __all_sync(0xffffffffu, ok);
      tc_fence_after_sync();
      // descriptor offsets (16-byte units) within a stage: K-major B, k-step ks of slot; MN-major B,
      // 16 rows per k-step
      auto koff = [](int slot, int ks) { return (uint64_t)((CF::stream_off(slot, ks >> 2) + (ks & 3) * 32) >> 4); };
      auto moff = [](int slot, int ks) { return (uint64_t)((CF::stream_off(slot, 0) + ks * 2048) >> 4); };
      // operand written by the math warps over a score region: the 16 elements of k-step ks sit in
      // 8 columns at col0 + 32*(ks/2) + 8*(ks%2) (owner half, then chunk)
      auto op_tmem = [&](int col0, int ks) { return tmem_base + (uint32_t)(col0 + 32 * (ks >> 1) + 8 * (ks & 1)); };
      auto commit = [&](uint32_t bar) { if (elect_one()) mma_commit(bar); };
      constexpr int KS = D / 16, KO = BN / 16;
      // a head dimension below the tile width: skip the k-steps and output columns that are padding
      const int ks_n = g.D >> 4;
      const uint32_t idesc_out = make_idesc(BM, g.D, Pack<T>::kIsBf16, 0, 1);
      const uint32_t stat0 = tmem_base + CF::kStat, stat1 = stat0 + 64;
      const uint32_t out0 = tmem_base + CF::kOut, out1 = out0 + D;
      (void)stat1; (void)out1;

      auto stage_of = [&](int j) { return strm_base + (uint32_t)(j % CF::kStages) * CF::kStageBytes; };
      auto wait_stream = [&](int j) {
        bool w = mbar_wait(bar_stream_full(j % CF::kStages), (j / CF::kStages) & 1, abort_flag, t.status, wait_code(KCODE, 3));
        return (bool)__all_sync(0xffffffffu, w);
      };
      // Every batch of products is issued by the elected lane inside one branch, with the
      // descriptor of the stage built once: the instruction stream between two MMAs is an add.
      auto issue_ra = [&](int j) {     // S = Q K^T   |   S^T = K Q^T
        const int b = j % kBufs;
        const uint64_t dk = smem_desc_sw128(stage_of(j), 16, 1024);
        const uint32_t acc = tmem_base + CF::kRA + 64 * b;
        if (elect_one()) {
          _Pragma("unroll") for (int ks = 0; ks < KS; ++ks)
            if (ks < ks_n) mma_ts(acc, stat0 + 8 * ks, dk + koff(0, ks), kIdesc64, ks > 0);
          mma_commit(bar_ra_full(b));
        }
        __syncwarp();
      };
      auto issue_rb = [&](int j) {     // dP = dO V^T |   dP^T = V dO^T
        const int b = j % kBufs;
        const uint64_t dk = smem_desc_sw128(stage_of(j), 16, 1024);
        const uint32_t acc = tmem_base + CF::kRB + 64 * b;
        if (elect_one()) {
          _Pragma("unroll") for (int ks = 0; ks < KS; ++ks)
            if (ks < ks_n) mma_ts(acc, stat1 + 8 * ks, dk + koff(1, ks), kIdesc64, ks > 0);
          mma_commit(bar_rb_full(b));
        }
        __syncwarp();
      };
      auto issue_out = [&](int j) {
        const int b = j % kBufs;
        const uint64_t dm = smem_desc_sw128(stage_of(j), kAtomBytesStrm, 1024);
        const bool first = (j == 0);
        if (elect_one()) {
          if constexpr (KIND == FB_BWD_ROW) {          // dQ += dS K
            _Pragma("unroll") for (int ks = 0; ks < KO; ++ks)
              mma_ts(out0, op_tmem(CF::kRB + 64 * b, ks), dm + moff(0, ks), idesc_out, !(first && ks == 0));
          } else {                                     // dV += P^T dO ; dK += dS^T Q
            _Pragma("unroll") for (int ks = 0; ks < KO; ++ks)
              mma_ts(out0, op_tmem(CF::kRB, ks), dm + moff(1, ks), idesc_out, !(first && ks == 0));
            _Pragma("unroll") for (int ks = 0; ks < KO; ++ks)
              mma_ts(out1, op_tmem(CF::kRB + 16, ks), dm + moff(0, ks), idesc_out, !(first && ks == 0));
          }
        }
        __syncwarp();
      };

      // Two barriers in one round: the even lanes wait for the first, the odd lanes for the second
      auto wait_two = [&](uint32_t bar0, uint32_t par0, int id0, bool has1, uint32_t bar1, uint32_t par1, int id1) {
        const bool second = has1 && (lane & 1);
        bool w = mbar_wait(second ? bar1 : bar0, second ? par1 : par0, abort_flag, t.status, wait_code(KCODE, second ? id1 : id0));
        return (bool)__all_sync(0xffffffffu, w);
      };
      if (warp == kFbMmaWarp) {
        // ---- first warp: the score products, as soon as the region's previous scores have been read
        for (int j = 0; j < n_iter && ok; ++j) {
          const int b = j % kBufs;
          ok = wait_two(bar_stream_full(j % CF::kStages), (j / CF::kStages) & 1, 3,
                        j >= kBufs, bar_ra_free(b), ((j / kBufs) & 1) ^ 1, 4);
          if (!ok) break;
          tc_fence_after_sync();
          issue_ra(j);
        }
      } else {
        // ---- second warp: outputs of a tile, then the dP products that overwrite their operands
        for (int i = 0; i < kBufs && i < n_iter && ok; ++i) {
          ok = wait_stream(i);
          if (!ok) break;
          tc_fence_after_sync();
          issue_rb(i);
        }
        for (int j = 0; j < n_iter && ok; ++j) {
          const int b = j % kBufs, nj = j + kBufs;
          ok = wait_two(bar_op_full(b), (j / kBufs) & 1, 5,
                        nj < n_iter, bar_stream_full(nj % CF::kStages), (nj / CF::kStages) & 1, 3);
          if (!ok) break;
          tc_fence_after_sync();
          issue_out(j);
          // every product reading this stage has been issued (the score product of the tile, issued by
          // the first warp, completed before the math warps could write the operands waited for above)
          commit(bar_stream_empty(j % CF::kStages));
          if (nj < n_iter) issue_rb(nj);
        }
        if (ok) commit(bar_acc_done);
      }
    }
  }
  // =========================================================================
  // math warps
  // =========================================================================
  else {
    const int quarter = warp & 3, half = warp >> 2;
    const int row = quarter * 32 + lane;         // stationary row within the tile == TMEM lane
    const int gidx = r0 + row;
    const uint32_t lane_addr = tmem_base + ((uint32_t)(quarter * 32) << 16);
    const size_t row_off = (size_t)bh * g.N_q;

    int vlo, vhi;                                // streamed indices visible to this stationary row
    if (CF::kCol) query_range_for_keys(g, gidx, gidx + 1, vlo, vhi);
    else key_range_for_queries(g, gidx, gidx + 1, vlo, vhi);
    if (gidx >= n_stat) { vlo = 0; vhi = 0; }
    const uint32_t vspan = (uint32_t)(vhi - vlo);

    // ---- one-time copy of the stationary rows from the staging buffer to tensor memory.
    // Shared-memory tile: per 64-column atom, row r at r*128 bytes, 16-byte chunks XOR-swizzled
    // by r % 8.  Tensor-memory A operand: lane = row, one 32-bit column per pair of K elements.
    bool ok = true;
    if (n_iter > 0) {
      ok = mbar_wait(bar_staging_full, 0, abort_flag, t.status, wait_code(KCODE, 6));
      ok = __all_sync(0xffffffffu, ok);
      if (ok) {
        constexpr int kChunksPerHalf = D / 16;
#pragma unroll
        for (int x = 0; x < CF::kNStat; ++x) {
          const uint32_t src = staging + x * kAtoms * kAtomBytesStat;
          const uint32_t dst = lane_addr + CF::kStat + 64 * x;
#pragma unroll
          for (int c = 0; c < kChunksPerHalf; c += 2) {
            uint32_t w[8];
#pragma unroll
            for (int u = 0; u < 2; ++u) {
              const int gc = half * kChunksPerHalf + c + u;
              const uint32_t addr = src + (gc >> 3) * kAtomBytesStat + row * 128 + ((((uint32_t)(gc & 7)) ^ (row & 7)) << 4);
              asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];"
                           : "=r"(w[4 * u]), "=r"(w[4 * u + 1]), "=r"(w[4 * u + 2]), "=r"(w[4 * u + 3])
                           : "r"(addr));
            }
            tmem_st8(dst + 4 * (half * kChunksPerHalf + c), w);
          }
        }
        tmem_st_wait();
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_stat_ready);
    }

    // per-row scalars (row kinds), negated so that every use is a packed add / fma
    float2 nL2 = make_float2(-INFINITY, -INFINITY), nDv = make_float2(0.f, 0.f);
    if constexpr (KIND == FB_BWD_ROW) {
      if (gidx < g.N_q) {
        const float L2 = t.L[row_off + gidx] * kLog2e, Dv = t.Dv[row_off + gidx];
        nL2 = make_float2(-L2, -L2);
        nDv = make_float2(-Dv, -Dv);
      }
    }
    const float2 sl2 = make_float2(g.scale_log2e, g.scale_log2e);
    float2 p_[16];                               // carried from S to dP

    // BWD_COL: per-query scalars of a streamed tile, fetched one tile ahead by the first four warps
    // (thread -> (which, query)) and handed over in shared memory; every warp arrives on the barrier.
    // The load is issued a tile ahead and its value is only touched when it is published, so that
    // its latency never stalls the warp.
    auto fetch_stat = [&](int tile_it) {
      const int which = (threadIdx.x >> 6) & 1, c = threadIdx.x & 63;
      const int qi = (t_begin + tile_it) * BN + c;
      float raw = (which == 0) ? INFINITY : 0.f;      // beyond N_q: L = +inf (p = 0), Dv = 0
      if (CF::kCol && threadIdx.x < 128 && tile_it < n_iter && qi < g.N_q)
        raw = (which == 0) ? __ldg(t.L + row_off + qi) : __ldg(t.Dv + row_off + qi);
      return raw;
    };
    auto publish_stat = [&](int tile_it, float raw) {
      const int which = (threadIdx.x >> 6) & 1;
      if (threadIdx.x < 128)
        aux_f[(tile_it & 1) * 128 + which * 64 + (threadIdx.x & 63)] = (which == 0) ? -raw * kLog2e : -raw;
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&ctl->stats_ready[tile_it & 1]));
    };
    if constexpr (CF::kCol) { if (n_iter > 0) publish_stat(0, fetch_stat(0)); }

    if constexpr (!CF::kCol) {
      // ---- row kind: the eight math warps form two groups of four; group w takes the tiles of
      // parity w (= score buffer w), a thread its whole row of the tile (64 scores).  While one
      // group waits for its products or for tensor-memory reads, the other one computes.
      const int grp = half;
      for (int it = grp; it < n_iter && ok; it += 2) {
        const int b = it & 1;
        const int j0 = (t_begin + it) * BN;
        const bool masked = !(j0 >= vlo && j0 + BN - 1 < vhi);
        const uint32_t ra = lane_addr + CF::kRA + 64 * b;
        const uint32_t rb = lane_addr + CF::kRB + 64 * b;
        ok = mbar_wait(bar_ra_full(b), (it >> 1) & 1, abort_flag, t.status, wait_code(KCODE, 7));
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after_sync();
        float2 pw[32];                               // p of the whole row, carried from S to dP
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
          uint32_t s_[2][16];
          tmem_ld16(ra + hh * 32, s_[0]);
          tmem_ld16(ra + hh * 32 + 16, s_[1]);
          tmem_ld_wait(s_[0]);
          tmem_ld_wait(s_[1]);
          if (hh == 1) {       // the whole row is in registers: the score product of tile it + 2 may overwrite the buffer
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_ra_free(b));
          }
#pragma unroll
          for (int ch = 0; ch < 2; ++ch)
#pragma unroll
            for (int e = 0; e < 16; e += 2) {
              const int cc = hh * 32 + ch * 16 + e;
              const float2 x = __ffma2_rn(make_float2(__uint_as_float(s_[ch][e]), __uint_as_float(s_[ch][e + 1])), sl2, nL2);
              float2 pp = make_float2(ex2(x.x), ex2(x.y));
              if (masked) {
                pp.x = ((uint32_t)(j0 + cc - vlo) < vspan) ? pp.x : 0.f;
                pp.y = ((uint32_t)(j0 + cc + 1 - vlo) < vspan) ? pp.y : 0.f;
              }
              pw[hh * 16 + ch * 8 + (e >> 1)] = pp;
            }
        }
        ok = mbar_wait(bar_rb_full(b), (it >> 1) & 1, abort_flag, t.status, wait_code(KCODE, 8));
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after_sync();
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
          uint32_t d_[2][16];
          tmem_ld16(rb + hh * 32, d_[0]);
          tmem_ld16(rb + hh * 32 + 16, d_[1]);
          tmem_ld_wait(d_[0]);
          tmem_ld_wait(d_[1]);
          uint32_t kds[2][8];
#pragma unroll
          for (int ch = 0; ch < 2; ++ch)
#pragma unroll
            for (int e = 0; e < 16; e += 2) {
              const float2 dpd = __fadd2_rn(make_float2(__uint_as_float(d_[ch][e]), __uint_as_float(d_[ch][e + 1])), nDv);
              const float2 ds = __fmul2_rn(pw[hh * 16 + ch * 8 + (e >> 1)], dpd);
              kds[ch][e >> 1] = Pack<T>::pack(ds.x, ds.y);
            }
          // dS over the dP columns this thread has just read (the layout the output product expects:
          // 16 elements of k-step ks in 8 columns at 32 * (ks / 2) + 8 * (ks % 2))
          tmem_st8(rb + hh * 32, kds[0]);
          tmem_st8(rb + hh * 32 + 8, kds[1]);
        }
        tmem_st_wait();
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_op_full(b));
      }
    } else
    for (int it = 0; it < n_iter && ok; ++it) {
      const int b = it % kBufs;
      const int j0 = (t_begin + it) * BN;
      const int first = j0 + half * 32;
      const bool masked = !(first >= vlo && first + 31 < vhi);
      const uint32_t ra = lane_addr + CF::kRA + 64 * b + half * 32;
      const uint32_t rb = lane_addr + CF::kRB + 64 * b + half * 32;
      const float* cs = aux_f + (it & 1) * 128;   // BWD_COL: [-L*log2(e) | -Dv] x 64 queries
      float next_stat = 0.f;
      if constexpr (CF::kCol) {
        // the scalars of tile it+1 are fetched now and published at the end of this tile
        next_stat = fetch_stat(it + 1);
        ok = mbar_wait(smem_u32(&ctl->stats_ready[it & 1]), (it >> 1) & 1, abort_flag, t.status, wait_code(KCODE, 9));
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
      }

      // ---------------- scores: S -> p ------------------------------------------
      ok = mbar_wait(bar_ra_full(b), (it / kBufs) & 1, abort_flag, t.status, wait_code(KCODE, 7));
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after_sync();
      uint32_t s_[2][16];
      tmem_ld16(ra, s_[0]);
      tmem_ld16(ra + 16, s_[1]);
      tmem_ld_wait(s_[0]);
      tmem_ld_wait(s_[1]);
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_ra_free(b));
      {
        uint32_t kp[2][8];
#pragma unroll
        for (int ch = 0; ch < 2; ++ch)
#pragma unroll
          for (int e = 0; e < 16; e += 2) {
            const int cc = half * 32 + ch * 16 + e;
            float2 l2 = nL2;
            if constexpr (CF::kCol) l2 = *reinterpret_cast<const float2*>(cs + cc);
            const float2 x = __ffma2_rn(make_float2(__uint_as_float(s_[ch][e]), __uint_as_float(s_[ch][e + 1])), sl2, l2);
            float2 pp = make_float2(ex2(x.x), ex2(x.y));
            if (masked) {
              pp.x = ((uint32_t)(j0 + cc - vlo) < vspan) ? pp.x : 0.f;
              pp.y = ((uint32_t)(j0 + cc + 1 - vlo) < vspan) ? pp.y : 0.f;
            }
            p_[ch * 8 + (e >> 1)] = pp;
            kp[ch][e >> 1] = Pack<T>::pack(pp.x, pp.y);
          }
        {
          // ---------------- dP -> dS (and P^T for the column kind) ------------------
          ok = mbar_wait(bar_rb_full(b), (it / kBufs) & 1, abort_flag, t.status, wait_code(KCODE, 8));
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
          tc_fence_after_sync();
          uint32_t d_[2][16];
          tmem_ld16(rb, d_[0]);
          tmem_ld16(rb + 16, d_[1]);
          tmem_ld_wait(d_[0]);
          tmem_ld_wait(d_[1]);
          uint32_t kds[2][8];
#pragma unroll
          for (int ch = 0; ch < 2; ++ch)
#pragma unroll
            for (int e = 0; e < 16; e += 2) {
              const int cc = half * 32 + ch * 16 + e;
              float2 dv = nDv;
              if constexpr (CF::kCol) dv = *reinterpret_cast<const float2*>(cs + 64 + cc);
              const float2 dpd = __fadd2_rn(make_float2(__uint_as_float(d_[ch][e]), __uint_as_float(d_[ch][e + 1])), dv);
              const float2 ds = __fmul2_rn(p_[ch * 8 + (e >> 1)], dpd);
              kds[ch][e >> 1] = Pack<T>::pack(ds.x, ds.y);
            }
          // over the dP columns this thread has read: [P^T (column kind) | dS]
          if constexpr (CF::kCol) {
            tmem_st8(rb, kp[0]);
            tmem_st8(rb + 8, kp[1]);
            tmem_st8(rb + 16, kds[0]);
            tmem_st8(rb + 24, kds[1]);
          } else {
            tmem_st8(rb, kds[0]);
            tmem_st8(rb + 8, kds[1]);
          }
          tmem_st_wait();
        }
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_op_full(b));
      // every warp has finished the previous tile (its operands were consumed before this tile's
      // dP^T product was queued), so the other scalar buffer is free
      if constexpr (CF::kCol) { if (it + 1 < n_iter) publish_stat(it + 1, next_stat); }
    }

    // ---------------- results ------------------------------------------------------
    {
      if (n_iter > 0 && ok) ok = mbar_wait(bar_acc_done, 0, abort_flag, t.status, wait_code(KCODE, 10));
      ok = __all_sync(0xffffffffu, ok);
      tc_fence_after_sync();
      constexpr int kColsPerHalf = D / 2;
      constexpr int kChunks = kColsPerHalf / 16;
      // The result tiles go out through the staging buffer of the stationary operands (they
      // have been in tensor memory since the prologue).
#pragma unroll
      for (int o = 0; o < CF::kNOut; ++o) {
        float mul = 1.f;
        if constexpr (KIND == FB_BWD_ROW) mul = g.scale;
        else mul = (o == 0) ? 1.f : g.scale;
        const uint32_t tile = staging + (uint32_t)o * kAtoms * kAtomBytesStat;
        uint32_t v[kChunks][16];
#pragma unroll
        for (int ch = 0; ch < kChunks; ++ch) {
          if (n_iter > 0 && ok) {
            tmem_ld16(lane_addr + CF::kOut + o * D + half * kColsPerHalf + ch * 16, v[ch]);
          } else {
#pragma unroll
            for (int e = 0; e < 16; ++e) v[ch][e] = 0u;
          }
        }
        if (n_iter > 0 && ok) {
#pragma unroll
          for (int ch = 0; ch < kChunks; ++ch) tmem_ld_wait(v[ch]);
        }
#pragma unroll
        for (int ch = 0; ch < kChunks; ++ch) {
          const int col = half * kColsPerHalf + ch * 16;
          if (col >= g.D) break;   // padding columns (uniform over the warp)
          uint32_t w[8];
#pragma unroll
          for (int e = 0; e < 8; ++e)
            w[e] = Pack<T>::pack(__uint_as_float(v[ch][2 * e]) * mul, __uint_as_float(v[ch][2 * e + 1]) * mul);
          store_op16(tile + (uint32_t)(col >> 6) * kAtomBytesStat, row, col & 63, w);
        }
      }
      fence_proxy_async_smem();
      named_barrier_sync(2, kMathWarps * 32);
      if (threadIdx.x == 0) {
        for (int o = 0; o < CF::kNOut; ++o) {
          const int id = (KIND == FB_BWD_ROW) ? TO_dQ : (o == 0 ? TO_dV : TO_dK);
          for (int a = 0; a * 64 < g.D; ++a)
            tma_store_3d(&maps.out[id], staging + (uint32_t)(o * kAtoms + a) * kAtomBytesStat, a * 64, r0, bh);
        }
        bulk_commit_group();
        bulk_wait_group_read_all();
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == kFbMmaWarp) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

template <int KIND, int D, typename T>
static cudaError_t launch_fb(const TmaMaps& maps, const Geometry& g_in, const Tensors& t, cudaStream_t s) {
  using CF = FbCfg<KIND, D>;
  Geometry g = g_in;
  const int n_stat = CF::kCol ? g.N_kv : g.N_q;
  const long long ctas = (long long)g.BH * ((n_stat + BM - 1) / BM);
  if (ctas <= 0) return cudaSuccess;
  if (ctas > 0x7fffffffLL) return cudaErrorInvalidValue;
  g.head_group = pick_head_group(ctas, g.BH, 2ll * (KIND == FB_BWD_COL ? g.N_q : g.N_kv) * g.D * 2);
  // more than half of an SM's shared memory: one CTA per SM, so the 512-column
  // tensor-memory allocation never waits for a co-resident CTA
  const size_t smem = CF::kSmemBytes < 122880u ? 122880u : CF::kSmemBytes;
  auto kern = fb_kernel<KIND, D, T>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return e;
  kern<<<(unsigned)ctas, kFbThreads, smem, s>>>(maps, g, t);
  return cudaGetLastError();
}

template <int D, typename T>
static cudaError_t launch_fb_kind(int kind, const TmaMaps& maps, const Geometry& g, const Tensors& t, cudaStream_t s) {
  return kind == FB_BWD_ROW ? launch_fb<FB_BWD_ROW, D, T>(maps, g, t, s) : launch_fb<FB_BWD_COL, D, T>(maps, g, t, s);
}

// kind: 2 backward dQ, 3 backward dK and dV
cudaError_t launch_fwd_bwd(int kind, int D, int is_bf16, const TmaMaps& maps, const Geometry& g, const Tensors& t,
                           cudaStream_t s) {
  if (D <= 64) return is_bf16 ? launch_fb_kind<64, __nv_bfloat16>(kind, maps, g, t, s) : launch_fb_kind<64, __half>(kind, maps, g, t, s);
  return is_bf16 ? launch_fb_kind<128, __nv_bfloat16>(kind, maps, g, t, s) : launch_fb_kind<128, __half>(kind, maps, g, t, s);
}

}  // namespace tc
}  // namespace attn
