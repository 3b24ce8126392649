// Row-side kernels of the double backward (Hessian-vector product) on sm_100a.
//
// The query side of the HVP needs two [128 x D] fp32 accumulators (g_Q, g_dO).  At
// D = 128 they would fill half of tensor memory.  The work is therefore split over two
// kernels with ONE accumulator each, which leaves 128 columns for the stationary operands:
//
//   ROW_PREDO  per-row scalars Dv, dot2, dot3 (to scratch) and
//                g_dO = P g_dV + (P o gdS) V - dot2 o O
//              (g_dp = P o (gdS - dot2), and P V = O is an input, so the unknown dot2 is
//              applied in the epilogue instead of inside the loop)
//   ROW_Q      g_Q = s (dS g_dK + g_S K), given the scalars
//
// Both stream K, g_dK, V, g_dV in 64-row tiles (three TMA stages, six at D = 64) past 128 stationary
// rows of Q, dO, g_dQ.  Q and dO are copied once into TENSOR MEMORY and used from there
// as the A operand of their score products (an A operand in shared memory is re-read by
// every MMA instruction: measured 48 instead of 32 clocks for an N = 64 product); g_dQ
// stays in shared memory.
// Tensor memory:  RA [0,128) = [S | gdS] = [Q K^T | Q g_dK^T + g_dQ K^T];
// RB [128,256) = [dP | gPdV] = dO [V; g_dV]^T;  OUT [256,256+D);  Q at [384,384+D/2),
// dO at [448,448+D/2) (two halves per 32-bit column).  Per tile the math warps run two
// half-steps:
//   half-step 1 reads RA:  p = exp(S - L) and either p*gdS (ROW_PREDO, accumulating dot2)
//               or a = gdS - dot2 (ROW_Q); both are kept in registers and RA is released at once;
//   half-step 2 reads RB:  ROW_PREDO accumulates Dv, A, E (dot3 = A - 2 Dv dot2 + E) and
//               writes the operands P and P o gdS over RB; ROW_Q writes dS = p (dP - Dv) and
//               g_S = p (a (dP - Dv) + gPdV - c3), c3 = dot2 Dv + dot3, over RB.
// Output products take their A operand from RB.  Two warps issue the MMAs, each batch by one
// elected lane inside a single branch: the first warp the RA products of every tile, the second
// the outputs of a tile followed by the RB products of the next (so RB is overwritten only after
// the outputs that read it).  With one issuing warp the latency of each of its waits (about 150
// clocks even when satisfied) fell on an empty tensor pipe.  At D = 64 tensor memory has room for
// a second RB region and the RB products run a tile ahead of the outputs.  The result tile leaves
// through shared memory and a TMA store, which clips rows and columns beyond the tensor.
// Formulas: reference csrc/flash_double_backward_v7.cu:1257-1454.
#include "attn_launch.h"
#include "tc_common.cuh"

namespace attn {
namespace tc {

enum RowMode { ROW_PREDO = 0, ROW_Q = 1 };

constexpr int kRowMmaWarp = 9;
constexpr int kRowThreads = 352;    // 8 math warps, TMA producer, two MMA issuers

constexpr int kRowMaxStages = 6;

struct RowControl {
  uint64_t stat_full;          // g_dQ tile in shared memory
  uint64_t staging_full;       // Q and dO tiles in the staging buffer (the last stage)
  uint64_t stat_tmem_ready;    // Q and dO copied to tensor memory
  // a stage has two halves with their own barriers: [K, g_dK] (index 0) and [V, g_dV] (index 1)
  uint64_t stream_full[2][kRowMaxStages];
  uint64_t stream_empty[2][kRowMaxStages];
  uint64_t ra_full;
  uint64_t ra_free;
  uint64_t rb_full[2];         // per RB buffer
  uint64_t op_full[2];         // per RB buffer: operands of a tile written
  uint64_t acc_done;
  // second issuing warp -> first: the RB products of a tile are queued.  Two barriers used in
  // turn (tile parity): the first warp may fall a whole tile behind the second (it also waits for
  // the [K, g_dK] load), and a single barrier completing twice before it is looked at would show
  // the waited-for parity as pending again.
  uint64_t rb_issued[2];
  uint32_t tmem_base;
  volatile uint32_t abort_flag;
};

static_assert(sizeof(RowControl) <= 512, "control block larger than its slot");

template <int D>
struct RowCfg {
  static constexpr int kAtoms = D / 64;
  static constexpr int kNStream = 4;    // K, g_dK, V, g_dV (pairs back to back)
  // A TMA load takes about 2 000 clocks from request to arrival, whatever its size.  At D = 128
  // a tile takes longer than that and three stages (all that fits) keep the loads ahead; at
  // D = 64 a tile takes about 1 600 clocks and the stages are half the size: six of them.
  static constexpr int kStages = (D == 64) ? 6 : 3;
  static_assert(kStages <= kRowMaxStages, "control block too small");
  static constexpr uint32_t kStatBytes = kAtoms * kAtomBytesStat;            // g_dQ only
  static constexpr uint32_t kStageBytes = kNStream * kAtoms * kAtomBytesStrm;
  static_assert(kStageBytes == 2 * kAtoms * kAtomBytesStat, "Q and dO are staged in one stream stage");
  static constexpr uint32_t kAuxBytes = 512;          // control block
  static constexpr uint32_t kContentBytes = kStatBytes + kStages * kStageBytes + kAuxBytes;
  static constexpr uint32_t kMaxSmem = 232448;
  static_assert(kContentBytes <= kMaxSmem, "shared memory over-subscribed");
  static constexpr uint32_t kSmemBytes = (kContentBytes + 1024 <= kMaxSmem) ? kContentBytes + 1024 : kMaxSmem;
  // At D = 64 the accumulator and the stationary operands take half the columns, which leaves
  // room for a second RB region: the RB products then run a tile ahead of the outputs instead of
  // waiting behind them, and the math warps (the bound at D = 64) never wait for RB.
  static constexpr int kRbBufs = (D == 64) ? 2 : 1;
  static constexpr int kRA = 0, kRB = 128, kOut = 128 + 128 * kRbBufs;
  static constexpr int kQT = (D == 64) ? 448 : 384, kDOT = (D == 64) ? 480 : 448;
  static_assert(kOut + D <= kQT && kQT + D / 2 <= kDOT && kDOT + D / 2 <= kTmemCols, "tensor memory over-subscribed");
  __host__ __device__ static constexpr uint32_t stream_off(int slot, int atom) {
    return (uint32_t)(slot >> 1) * (2u * kAtoms * kAtomBytesStrm) + (uint32_t)atom * 2u * kAtomBytesStrm +
           (uint32_t)(slot & 1) * kAtomBytesStrm;
  }
  __host__ __device__ static constexpr int stream_tensor(int slot) {
    return slot == 0 ? T_K : slot == 1 ? T_gK : slot == 2 ? T_V : T_gV;
  }
};

template <int MODE, int D, typename T>
__global__ void __launch_bounds__(kRowThreads, 1)
hvp_row_kernel(const __grid_constant__ TmaMaps maps, const Geometry g, const Tensors t) {
  using CF = RowCfg<D>;
  constexpr int KIND = (MODE == ROW_PREDO) ? HVP_PRE : HVP_ROW;
  constexpr int kAtoms = CF::kAtoms;
  constexpr uint32_t kIdesc64 = make_idesc(BM, 64, Pack<T>::kIsBf16, 0, 0);
  constexpr uint32_t kIdesc128 = make_idesc(BM, 128, Pack<T>::kIsBf16, 0, 0);

  extern __shared__ __align__(1024) uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  {
    uint32_t dyn_size;
    asm("mov.u32 %0, %%dynamic_smem_size;" : "=r"(dyn_size));
    if (smem_base - smem_u32(smem_raw) + CF::kContentBytes > dyn_size) {   // uniform over the CTA
      if (threadIdx.x == 0 && t.status != nullptr) atomicCAS(t.status, 0u, wait_code(KIND, 15));
      return;
    }
  }
  const uint32_t stat_base = smem_base;
  const uint32_t strm_base = stat_base + CF::kStatBytes;
  const uint32_t aux_off = CF::kStatBytes + CF::kStages * CF::kStageBytes;
  const uint32_t staging = strm_base + (CF::kStages - 1) * CF::kStageBytes;   // Q then dO, before the last stage is used
  RowControl* ctl = reinterpret_cast<RowControl*>(smem_gen + aux_off);
  // [2 halves][4][128] floats of row sums, exchanged after the last product has read the
  // g_dQ tile: its shared memory is reused
  float* row_sums = reinterpret_cast<float*>(smem_gen);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tiles = (g.N_q + BM - 1) / BM;
  int bh, rank;
  cta_to_head_and_rank(g, tiles, bh, rank);
  const int tile = (g.mask_mode != 0) ? rank : (tiles - 1 - rank);   // heavy tiles first
  const int r0 = tile * BM;

  int lo, hi;
  key_range_for_queries(g, r0, r0 + BM, lo, hi);
  const int t_begin = lo / BN;
  const int n_iter = (hi > lo) ? ((hi + BN - 1) / BN - t_begin) : 0;

  const uint32_t bar_stat_full = smem_u32(&ctl->stat_full);
  const uint32_t bar_staging_full = smem_u32(&ctl->staging_full);
  const uint32_t bar_stat_tmem_ready = smem_u32(&ctl->stat_tmem_ready);
  const uint32_t bar_ra_full = smem_u32(&ctl->ra_full), bar_ra_free = smem_u32(&ctl->ra_free);
  auto bar_rb_full = [&](int b) { return smem_u32(&ctl->rb_full[b]); };
  auto bar_op_full = [&](int b) { return smem_u32(&ctl->op_full[b]); };
  const uint32_t bar_acc_done = smem_u32(&ctl->acc_done);
  constexpr int LA = CF::kRbBufs;     // tiles the RB products run ahead of the outputs
  auto bar_rb_issued = [&](int tile) { return smem_u32(&ctl->rb_issued[tile & 1]); };
  auto bar_stream_full = [&](int h, int s) { return smem_u32(&ctl->stream_full[h][s]); };
  auto bar_stream_empty = [&](int h, int s) { return smem_u32(&ctl->stream_empty[h][s]); };

  if (threadIdx.x == 0) {
    mbar_init(bar_stat_full, 1);
    mbar_init(bar_staging_full, 1);
    mbar_init(bar_stat_tmem_ready, kMathWarps);
    for (int s = 0; s < CF::kStages; ++s) {
      for (int h = 0; h < 2; ++h) {
        mbar_init(bar_stream_full(h, s), 1);
        mbar_init(bar_stream_empty(h, s), 1);
      }
    }
    mbar_init(bar_ra_full, 1);
    mbar_init(bar_ra_free, kMathWarps);
    for (int b = 0; b < 2; ++b) {
      mbar_init(bar_rb_full(b), 1);
      mbar_init(bar_op_full(b), kMathWarps);
    }
    mbar_init(bar_acc_done, 1);
    mbar_init(bar_rb_issued(0), 1);
    mbar_init(bar_rb_issued(1), 1);
    ctl->abort_flag = 0u;
    ctl->tmem_base = 0u;
    fence_barrier_init();
    fence_proxy_async_smem();
  }
  __syncthreads();
  // the stationary tiles and the first streamed tile are requested before the tensor-memory
  // allocation and the second barrier: their latency is the longest item of the prologue
  if (warp == kProducerWarp && lane == 0 && n_iter > 0) {
    mbar_arrive_expect_tx(bar_staging_full, CF::kStageBytes);
#pragma unroll
    for (int x = 0; x < 2; ++x)       // Q then dO: they are copied to tensor memory first
#pragma unroll
      for (int a = 0; a < kAtoms; ++a)
#pragma unroll
        for (int h = 0; h < 2; ++h)
          tma_load_3d(staging + (x * kAtoms + a) * kAtomBytesStat + h * kAtomBytesStrm, &maps.m[x == 0 ? T_Q : T_dO],
                      a * 64, r0 + h * 64, bh, bar_staging_full);
    mbar_arrive_expect_tx(bar_stream_full(0, 0), CF::kStageBytes / 2);
    mbar_arrive_expect_tx(bar_stream_full(1, 0), CF::kStageBytes / 2);
#pragma unroll
    for (int sl = 0; sl < CF::kNStream; ++sl)
#pragma unroll
      for (int a = 0; a < kAtoms; ++a)
        tma_load_3d(strm_base + CF::stream_off(sl, a), &maps.m[CF::stream_tensor(sl)], a * 64, t_begin * BN, bh,
                    bar_stream_full(sl >> 1, 0));
    mbar_arrive_expect_tx(bar_stat_full, CF::kStatBytes);
#pragma unroll
    for (int a = 0; a < kAtoms; ++a)
#pragma unroll
      for (int h = 0; h < 2; ++h)
        tma_load_3d(stat_base + a * kAtomBytesStat + h * kAtomBytesStrm, &maps.m[T_gQ], a * 64, r0 + h * 64, bh,
                    bar_stat_full);
  }
  if (warp == kRowMmaWarp) tmem_alloc(smem_u32(&ctl->tmem_base), kTmemCols);
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
      bool ok = true;
      // The two halves of a stage are released at different times: [K, g_dK] is last read by the
      // RA products in the scalar pass (long before the outputs of the tile), [V, g_dV] by the RB
      // products in the g_Q pass.  Each half is requested as soon as its own buffer is free, so the
      // loads the first issuing warp waits for leave a tile earlier than a whole-stage release would
      // allow (a load takes about as long as a tile).
      for (int it = 1; it < n_iter; ++it) {     // tile 0 was requested above
        const int st = it % CF::kStages;
        const uint32_t stage = strm_base + st * CF::kStageBytes;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          ok = mbar_wait(bar_stream_empty(h, st), ((it / CF::kStages) & 1) ^ 1, abort_flag, t.status, wait_code(KIND, 1));
          // the last stage doubles as the staging buffer of Q and dO until they are in tensor memory
          if (ok && it == CF::kStages - 1) ok = mbar_wait(bar_stat_tmem_ready, 0, abort_flag, t.status, wait_code(KIND, 10));
          if (!ok) break;
          mbar_arrive_expect_tx(bar_stream_full(h, st), CF::kStageBytes / 2);
#pragma unroll
          for (int s2 = 0; s2 < 2; ++s2)
#pragma unroll
            for (int a = 0; a < kAtoms; ++a)
              tma_load_3d(stage + CF::stream_off(2 * h + s2, a), &maps.m[CF::stream_tensor(2 * h + s2)], a * 64,
                          (t_begin + it) * BN, bh, bar_stream_full(h, st));
        }
        if (!ok) break;
      }
      if (!ok) {   // give copies already in flight a bounded chance to land before the CTA exits
        const long long t0 = clock64();
        while (clock64() - t0 < 2000000LL) { }
      }
    }
  }
  // =========================================================================
  // MMA issuers (converged warps, one elected lane issues)
  // =========================================================================
  else if (warp == kRowMmaWarp || warp == kRowMmaWarp + 1) {
    if (n_iter > 0) {
      bool ok = mbar_wait(bar_stat_full, 0, abort_flag, t.status, wait_code(KIND, 2));
      if (ok) ok = mbar_wait(bar_stat_tmem_ready, 0, abort_flag, t.status, wait_code(KIND, 11));
      ok = __all_sync(0xffffffffu, ok);
      tc_fence_after_sync();
      const uint64_t d_stat = smem_desc_sw128(stat_base, 16, 1024);
      auto gq_desc = [&](int ks) {   // K-major A from shared memory: the g_dQ tile
        return d_stat + (uint64_t)(((ks >> 2) * kAtomBytesStat + (ks & 3) * 32) >> 4);
      };
      // descriptor offsets (16-byte units) within a stage: K-major B, k-step ks of slot; MN-major B,
      // 16 rows per k-step
      auto koff = [](int slot, int ks) { return (uint64_t)((CF::stream_off(slot, ks >> 2) + (ks & 3) * 32) >> 4); };
      auto moff = [](int slot, int ks) { return (uint64_t)((CF::stream_off(slot, 0) + ks * 2048) >> 4); };
      // operand written by the math warps over a 64-column score slot: the 16 elements of
      // k-step ks sit in 8 columns at 32*(ks/2) + 8*(ks%2) (owner half, then chunk)
      auto op_tmem = [&](int col0, int ks) { return tmem_base + (uint32_t)(col0 + 32 * (ks >> 1) + 8 * (ks & 1)); };
      auto commit = [&](uint32_t bar) { if (elect_one()) mma_commit(bar); };
      constexpr int KS = D / 16, KO = BN / 16;
      // a head dimension below the tile width: skip the k-steps and output columns that are padding
      const int ks_n = g.D >> 4;
      const uint32_t idesc_out = make_idesc(BM, g.D, Pack<T>::kIsBf16, 0, 1);
      const uint32_t out = tmem_base + CF::kOut;
      const uint32_t ra = tmem_base + CF::kRA, rb = tmem_base + CF::kRB;
      const uint32_t qt = tmem_base + CF::kQT, dot = tmem_base + CF::kDOT;

      // Every batch of products is issued by the elected lane inside one branch, with the
      // descriptor of the stage built once: the instruction stream between two MMAs is an add.
      // The RA batch goes out in two elected branches, the last kTail k-steps and the commit in the
      // second: measured, the scalar pass loses 10 % when the whole batch is issued in one branch
      // (the short gap lets the other issuing warp's products into the queue in between).
      constexpr int kTail = (D == 128) ? 2 : 0;
      auto issue_ra = [&](uint32_t stage) {           // ends with the commit of the batch
        const uint64_t dk = smem_desc_sw128(stage, 16, 1024);
        if (elect_one()) {
          _Pragma("unroll") for (int ks = 0; ks < KS; ++ks)
            if (ks < ks_n) mma_ts(ra, qt + 8 * ks, dk + koff(0, ks), kIdesc128, ks > 0);
          _Pragma("unroll") for (int ks = 0; ks < KS - kTail; ++ks)
            if (ks < ks_n) mma_ss(ra + 64, gq_desc(ks), dk + koff(0, ks), kIdesc64, 1);
        }
        __syncwarp();
        if (elect_one()) {
          _Pragma("unroll") for (int ks = KS - kTail; ks < KS; ++ks)
            if (ks < ks_n) mma_ss(ra + 64, gq_desc(ks), dk + koff(0, ks), kIdesc64, 1);
          mma_commit(bar_ra_full);
        }
        __syncwarp();
      };
      auto issue_rb = [&](uint32_t stage, int b) {    // into RB buffer b; ends with its commit
        const uint64_t dk = smem_desc_sw128(stage, 16, 1024);
        const uint32_t acc = rb + 128u * (uint32_t)b;
        if (elect_one()) {
          _Pragma("unroll") for (int ks = 0; ks < KS; ++ks)
            if (ks < ks_n) mma_ts(acc, dot + 8 * ks, dk + koff(2, ks), kIdesc128, ks > 0);
          mma_commit(bar_rb_full(b));
        }
        __syncwarp();
      };
      auto issue_out = [&](uint32_t stage, bool first, int b) {   // operands in RB buffer b
        const uint64_t dm = smem_desc_sw128(stage, 2u * kAtomBytesStrm, 1024);
        constexpr int s0 = (MODE == ROW_PREDO) ? 3 : 1;     // g_dO' += P g_dV      | g_Q += dS g_dK
        constexpr int s1 = (MODE == ROW_PREDO) ? 2 : 0;     // g_dO' += (P o gdS) V | g_Q += g_S K
        if (elect_one()) {
          _Pragma("unroll") for (int ks = 0; ks < KO; ++ks)
            mma_ts(out, op_tmem(CF::kRB + 128 * b, ks), dm + moff(s0, ks), idesc_out, !(first && ks == 0));
          _Pragma("unroll") for (int ks = 0; ks < KO; ++ks)
            mma_ts(out, op_tmem(CF::kRB + 128 * b + 64, ks), dm + moff(s1, ks), idesc_out, 1);
        }
        __syncwarp();
      };

      // Two issuing warps, so that the latency of one warp's waits falls while the products of the
      // other are queued.  The tensor pipe needs no order between the two streams: RA(j+1) only
      // waits for RA(j) to have been read, and RB(j+1) follows OUT(j), which reads RB, in the
      // second warp's own order.
      auto wait_stream = [&](int h, int tile) {   // half h of the stage of `tile` has landed
        return mbar_wait(bar_stream_full(h, tile % CF::kStages), (tile / CF::kStages) & 1, abort_flag, t.status, wait_code(KIND, 3));
      };
      // which issuing warp releases which half: the one whose products read it last
      constexpr bool kRaReleasesKG = (MODE == ROW_PREDO);   // scalar pass: the outputs read V, g_dV only
      if (warp == kRowMmaWarp) {
        // ---- first warp: the RA products of every tile
        for (int j = 0; j < n_iter && ok; ++j) {
          ok = wait_stream(0, j);
          if (ok && j > 0) ok = mbar_wait(bar_ra_free, (j - 1) & 1, abort_flag, t.status, wait_code(KIND, 4));
          // ROW_Q keeps the pipe's order OUT(j-2), RB(j-1), RA(j): its second half-step is the long
          // one, and RA(j) queued any earlier delays the outputs that half-step waits behind.  The
          // scalar pass is faster with the two streams left to run freely (both measured).
          if (MODE == ROW_Q && LA == 1 && ok && j > 0) ok = mbar_wait(bar_rb_issued(j - 1), ((j - 1) >> 1) & 1, abort_flag, t.status, wait_code(KIND, 13));
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
          tc_fence_after_sync();
          const uint32_t stage = strm_base + (j % CF::kStages) * CF::kStageBytes;
          issue_ra(stage);
          if (kRaReleasesKG) commit(bar_stream_empty(0, j % CF::kStages));
        }
      } else {
        // ---- second warp: RB products (LA tiles ahead) and outputs
        for (int i = 0; i < LA && i < n_iter && ok; ++i) {
          ok = wait_stream(1, i);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
          tc_fence_after_sync();
          issue_rb(strm_base + (i % CF::kStages) * CF::kStageBytes, i % LA);
          if (!kRaReleasesKG) commit(bar_stream_empty(1, i % CF::kStages));
          if (LA == 1 && lane == 0) mbar_arrive(bar_rb_issued(i));
        }
        for (int j = 0; j < n_iter && ok; ++j) {
          const int st = j % CF::kStages, b = j % LA;
          const int nj = j + LA;
          ok = mbar_wait(bar_op_full(b), (j / LA) & 1, abort_flag, t.status, wait_code(KIND, 6));
          if (ok && nj < n_iter) ok = wait_stream(1, nj);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
          tc_fence_after_sync();
          issue_out(strm_base + st * CF::kStageBytes, j == 0, b);
          commit(bar_stream_empty(kRaReleasesKG ? 1 : 0, st));   // the half the outputs read
          if (nj < n_iter) {
            // buffer b again: after the outputs that read it, in this warp's own order
            issue_rb(strm_base + (nj % CF::kStages) * CF::kStageBytes, b);
            if (!kRaReleasesKG) commit(bar_stream_empty(1, nj % CF::kStages));
            if (LA == 1 && lane == 0) mbar_arrive(bar_rb_issued(nj));
          }
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
    const int row = quarter * 32 + lane;
    const int gidx = r0 + row;
    const uint32_t lane_addr = tmem_base + ((uint32_t)(quarter * 32) << 16);
    const size_t row_off = (size_t)bh * g.N_q;

    int vlo, vhi;
    key_range_for_queries(g, gidx, gidx + 1, vlo, vhi);
    if (gidx >= g.N_q) { vlo = 0; vhi = 0; }
    const uint32_t vspan = (uint32_t)(vhi - vlo);

    // scalars of this thread's query row, negated so that every use is a packed add / fma
    float2 nL2 = make_float2(-INFINITY, -INFINITY), nDv = make_float2(0.f, 0.f);
    float2 nD2 = make_float2(0.f, 0.f), nC3 = make_float2(0.f, 0.f);
    if (gidx < g.N_q) {
      const float L2 = t.L[row_off + gidx] * kLog2e;
      nL2 = make_float2(-L2, -L2);
      if constexpr (MODE == ROW_Q) {
        const float Dv = t.Dv[row_off + gidx], d2 = t.dot2[row_off + gidx];
        const float c3 = fmaf(d2, Dv, t.dot3[row_off + gidx]);
        nDv = make_float2(-Dv, -Dv); nD2 = make_float2(-d2, -d2); nC3 = make_float2(-c3, -c3);
      }
    }
    const float2 sl2 = make_float2(g.scale_log2e, g.scale_log2e);
    const float2 sc2 = make_float2(g.scale, g.scale);
    const float2 zero2 = make_float2(0.f, 0.f);

    // ---- one-time copy of the stationary Q and dO rows from the staging buffer to tensor memory.
    // Tile layout in shared memory: per 64-column atom, row r at r*128 bytes with its 16-byte
    // chunks XOR-swizzled by r % 8.  Tensor-memory layout of an A operand: lane = row, one
    // 32-bit column per pair of consecutive K elements.  This thread moves its row's half.
    bool ok = true;
    if (n_iter > 0) {
      ok = mbar_wait(bar_staging_full, 0, abort_flag, t.status, wait_code(KIND, 12));
      ok = __all_sync(0xffffffffu, ok);
      if (ok) {
        constexpr int kChunksPerHalf = D / 16;    // 16-byte chunks (8 halves) of this thread's half row
#pragma unroll
        for (int x = 0; x < 2; ++x) {             // 0: Q, 1: dO
          const uint32_t src = staging + x * kAtoms * kAtomBytesStat;
          const uint32_t dst = lane_addr + (x == 0 ? CF::kQT : CF::kDOT);
#pragma unroll
          for (int c = 0; c < kChunksPerHalf; c += 2) {
            uint32_t w[8];
#pragma unroll
            for (int u = 0; u < 2; ++u) {
              const int gc = half * kChunksPerHalf + c + u;   // chunk index within the row
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
      if (lane == 0) mbar_arrive(bar_stat_tmem_ready);
    }

    float2 p_[16], a_[16];   // carried from half-step 1 to half-step 2 (ROW_PREDO: a_ = p * gdS)
    float2 acc_D = zero2, acc_2 = zero2, acc_A = zero2, acc_E = zero2;   // ROW_PREDO row sums
    const uint32_t ra = lane_addr + CF::kRA;
    for (int it = 0; it < n_iter && ok; ++it) {
      const uint32_t rb = lane_addr + CF::kRB + 128u * (uint32_t)(it % LA);
      const int j0 = (t_begin + it) * BN;
      const int first = j0 + half * 32;
      const bool masked = !(first >= vlo && first + 31 < vhi);

      // ---------------- half-step 1: RA ------------------------------------------
      ok = mbar_wait(bar_ra_full, it & 1, abort_flag, t.status, wait_code(KIND, 7));
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after_sync();
      // Read this thread's 2 x 32 columns of RA in one go and release the region before the
      // arithmetic: the next tile's RA products are what the math warps wait for next.
      uint32_t s_[2][16], g_[2][16];
      tmem_ld16(ra + half * 32, s_[0]);
      tmem_ld16(ra + half * 32 + 16, s_[1]);
      tmem_ld16(ra + 64 + half * 32, g_[0]);
      tmem_ld16(ra + 64 + half * 32 + 16, g_[1]);
      tmem_ld_wait(s_[0]);
      tmem_ld_wait(s_[1]);
      tmem_ld_wait(g_[0]);
      tmem_ld_wait(g_[1]);
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_ra_free);
#pragma unroll
      for (int ch = 0; ch < 2; ++ch) {
        const int c0 = half * 32 + ch * 16;
#pragma unroll
        for (int e = 0; e < 16; e += 2) {
          const int cc = c0 + e;
          const float2 x = __ffma2_rn(make_float2(__uint_as_float(s_[ch][e]), __uint_as_float(s_[ch][e + 1])), sl2, nL2);
          float2 pp = make_float2(ex2(x.x), ex2(x.y));
          if (masked) {
            pp.x = ((uint32_t)(j0 + cc - vlo) < vspan) ? pp.x : 0.f;
            pp.y = ((uint32_t)(j0 + cc + 1 - vlo) < vspan) ? pp.y : 0.f;
          }
          const float2 gg = make_float2(__uint_as_float(g_[ch][e]), __uint_as_float(g_[ch][e + 1]));
          p_[ch * 8 + (e >> 1)] = pp;
          if constexpr (MODE == ROW_PREDO) {
            const float2 pg = __fmul2_rn(pp, __fmul2_rn(gg, sc2));     // p * gdS
            a_[ch * 8 + (e >> 1)] = pg;
            acc_2 = __fadd2_rn(acc_2, pg);
          } else {
            a_[ch * 8 + (e >> 1)] = __ffma2_rn(gg, sc2, nD2);           // gdS - dot2
          }
        }
      }

      // ---------------- half-step 2: RB ------------------------------------------
      ok = mbar_wait(bar_rb_full(it % LA), (it / LA) & 1, abort_flag, t.status, wait_code(KIND, 8));
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after_sync();
#pragma unroll
      for (int ch = 0; ch < 2; ++ch) {
        const int c0 = half * 32 + ch * 16;
        uint32_t dp_[16], gp_[16];
        tmem_ld16(rb + c0, dp_);
        tmem_ld16(rb + 64 + c0, gp_);
        tmem_ld_wait(dp_);
        tmem_ld_wait(gp_);
        uint32_t k0[8], k1[8];
#pragma unroll
        for (int e = 0; e < 16; e += 2) {
          const float2 pp = p_[ch * 8 + (e >> 1)], aa = a_[ch * 8 + (e >> 1)];
          const float2 dp = make_float2(__uint_as_float(dp_[e]), __uint_as_float(dp_[e + 1]));
          const float2 gp = make_float2(__uint_as_float(gp_[e]), __uint_as_float(gp_[e + 1]));
          if constexpr (MODE == ROW_PREDO) {
            acc_D = __ffma2_rn(pp, dp, acc_D);
            acc_A = __ffma2_rn(aa, dp, acc_A);
            acc_E = __ffma2_rn(pp, gp, acc_E);
            k0[e >> 1] = Pack<T>::pack(pp.x, pp.y);      // P
            k1[e >> 1] = Pack<T>::pack(aa.x, aa.y);      // P o gdS
          } else {
            const float2 dpd = __fadd2_rn(dp, nDv);
            const float2 ds = __fmul2_rn(pp, dpd);
            const float2 gs = __fmul2_rn(pp, __ffma2_rn(aa, dpd, __fadd2_rn(gp, nC3)));
            k0[e >> 1] = Pack<T>::pack(ds.x, ds.y);      // dS
            k1[e >> 1] = Pack<T>::pack(gs.x, gs.y);      // g_S
          }
        }
        // over columns this thread has just read (first half of its dP and gPdV ranges)
        tmem_st8(rb + half * 32 + ch * 8, k0);
        tmem_st8(rb + 64 + half * 32 + ch * 8, k1);
      }
      tmem_st_wait();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_op_full(it % LA));
    }

    // ---------------- results ------------------------------------------------------
    float dot2_row = 0.f;
    if constexpr (MODE == ROW_PREDO) {
      // each row is summed by two threads (column halves): exchange through shared memory
      float* mine = row_sums + half * 512;
      const float sD = acc_D.x + acc_D.y, s2 = acc_2.x + acc_2.y, sA = acc_A.x + acc_A.y, sE = acc_E.x + acc_E.y;
      mine[row] = sD; mine[128 + row] = s2; mine[256 + row] = sA; mine[384 + row] = sE;
      named_barrier_sync(1, kMathThreads);
      const float* other = row_sums + (half ^ 1) * 512;
      const float Dv = sD + other[row], d2 = s2 + other[128 + row];
      const float A = sA + other[256 + row], E = sE + other[384 + row];
      dot2_row = d2;
      if (half == 0 && gidx < g.N_q) {
        t.Dv[row_off + gidx] = Dv;
        t.dot2[row_off + gidx] = d2;
        t.dot3[row_off + gidx] = A - 2.f * Dv * d2 + E;
      }
    }
    constexpr int kColsPerHalf = D / 2;
    constexpr int kChunks = kColsPerHalf / 16;
    const float mul = (MODE == ROW_PREDO) ? 1.f : g.scale;
    // D is the padded head dimension of the tiles; the tensors in global memory have g.D columns
    const size_t elem0 = ((size_t)bh * g.N_q + gidx) * g.D + half * kColsPerHalf;
    // g_dO = g_dO' - dot2 * O: this thread's part of the O row is fetched while the last
    // products are still running
    uint4 o_[MODE == ROW_PREDO ? 2 * kChunks : 1];
    if constexpr (MODE == ROW_PREDO) {
#pragma unroll
      for (int ch = 0; ch < kChunks; ++ch) {
        const bool in = gidx < g.N_q && half * kColsPerHalf + ch * 16 < g.D;
        const uint4* orow = reinterpret_cast<const uint4*>((const T*)t.O + elem0 + ch * 16);
        o_[2 * ch] = in ? __ldg(orow) : make_uint4(0u, 0u, 0u, 0u);
        o_[2 * ch + 1] = in ? __ldg(orow + 1) : make_uint4(0u, 0u, 0u, 0u);
      }
    }
    if (n_iter > 0 && ok) ok = mbar_wait(bar_acc_done, 0, abort_flag, t.status, wait_code(KIND, 9));
    ok = __all_sync(0xffffffffu, ok);
    tc_fence_after_sync();
    // all accumulator columns of this thread first, then the arithmetic and the stores
    uint32_t v[kChunks][16];
#pragma unroll
    for (int ch = 0; ch < kChunks; ++ch) {
      if (n_iter > 0 && ok) {
        tmem_ld16(lane_addr + CF::kOut + half * kColsPerHalf + ch * 16, v[ch]);
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
      if (half * kColsPerHalf + ch * 16 >= g.D) break;   // padding columns (uniform over the warp)
      if (gidx < g.N_q) {
        float f[16];
#pragma unroll
        for (int e = 0; e < 16; ++e) f[e] = __uint_as_float(v[ch][e]) * mul;
        if constexpr (MODE == ROW_PREDO) {
          const uint4 o0 = o_[2 * ch], o1 = o_[2 * ch + 1];
          const uint32_t ow[8] = {o0.x, o0.y, o0.z, o0.w, o1.x, o1.y, o1.z, o1.w};
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            const float2 of = Pack<T>::unpack(ow[e]);
            f[2 * e] = fmaf(-dot2_row, of.x, f[2 * e]);
            f[2 * e + 1] = fmaf(-dot2_row, of.y, f[2 * e + 1]);
          }
        }
        uint32_t w[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) w[e] = Pack<T>::pack(f[2 * e], f[2 * e + 1]);
        const int col = half * kColsPerHalf + ch * 16;
        store_op16(strm_base + (uint32_t)(col >> 6) * kAtomBytesStat, row, col & 63, w);
      }
    }
    // the result tile goes out through the first stream stage (every product has completed)
    store_tile_tma(&maps.out[MODE == ROW_PREDO ? TO_gdO : TO_gQ], strm_base, g.D, r0, bh, threadIdx.x == 0);
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == kRowMmaWarp) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

template <int MODE, int D, typename T>
static cudaError_t launch_row(const TmaMaps& maps, const Geometry& g_in, const Tensors& t, cudaStream_t s) {
  using CF = RowCfg<D>;
  Geometry g = g_in;
  const long long ctas = (long long)g.BH * ((g.N_q + BM - 1) / BM);
  if (ctas <= 0) return cudaSuccess;
  if (ctas > 0x7fffffffLL) return cudaErrorInvalidValue;
  g.head_group = pick_head_group(ctas, g.BH, 4ll * g.N_kv * g.D * 2);   // K, g_dK, V, g_dV
  // more than half of an SM's shared memory: one CTA per SM, so the 512-column
  // tensor-memory allocation never waits for a co-resident CTA
  const size_t smem = CF::kSmemBytes < 122880u ? 122880u : CF::kSmemBytes;
  auto kern = hvp_row_kernel<MODE, D, T>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return e;
  kern<<<(unsigned)ctas, kRowThreads, smem, s>>>(maps, g, t);
  return cudaGetLastError();
}

// mode 0: per-row scalars + g_dO;  mode 1: g_Q
cudaError_t launch_hvp_row(int mode, int D, int is_bf16, const TmaMaps& maps, const Geometry& g,
                           const Tensors& t, cudaStream_t s) {
  if (mode == 0) {
    if (D <= 64) return is_bf16 ? launch_row<ROW_PREDO, 64, __nv_bfloat16>(maps, g, t, s) : launch_row<ROW_PREDO, 64, __half>(maps, g, t, s);
    return is_bf16 ? launch_row<ROW_PREDO, 128, __nv_bfloat16>(maps, g, t, s) : launch_row<ROW_PREDO, 128, __half>(maps, g, t, s);
  }
  if (D <= 64) return is_bf16 ? launch_row<ROW_Q, 64, __nv_bfloat16>(maps, g, t, s) : launch_row<ROW_Q, 64, __half>(maps, g, t, s);
  return is_bf16 ? launch_row<ROW_Q, 128, __nv_bfloat16>(maps, g, t, s) : launch_row<ROW_Q, 128, __half>(maps, g, t, s);
}

}  // namespace tc
}  // namespace attn
