// Main kernels of the double backward (Hessian-vector product) on sm_100a:
// the row side (g_Q, g_dO) and the column side (g_K, g_V), given the per-row
// scalars Dv, dot2, dot3 of the pre-pass.
//
// Tile shapes and warp roles are those of attn_tc.cu (128 stationary rows, 64
// streamed rows per step, 8 math warps + TMA warp, here with two MMA warps).  What differs is
// the pipeline, built for the two constraints of this kernel at D = 128 --
// 512 tensor-memory columns and 227 KB of shared memory:
//
// * Tensor memory holds two 128-column score regions and two output accumulators:
//       RA [  0,128)  = [ S | gdS ]        RB [128,256) = [ dP | gPdV ]
//       OUT0 [256,256+D)                   OUT1 [256+D,256+2D)
//   The math warps work in two half-steps per tile.  Half-step 1 reads RA,
//   computes p = exp(S - L) and a = s*gdS - dot2, keeps both in registers and
//   writes the half-precision operands P and g_dp = p*a back INTO RA.  Half-step
//   2 reads RB and writes dS = p*(dP - Dv) and g_S = p*(a*(dP - Dv) + gPdV - c3),
//   c3 = dot2*Dv + dot3, into RB.  The output products read those operands
//   straight from tensor memory (A operand in TMEM), so no operand tile goes
//   through shared memory.  While the math warps are in half-step 1 of tile j
//   the tensor core runs the RB products of tile j and the RB-operand outputs of
//   tile j-1; during half-step 2 it runs the RA-operand outputs of tile j and the
//   RA products of tile j+1.  Each thread overwrites only columns it has itself
//   already read, so the two column halves of a row never race.
// * Shared memory holds the stationary operands and TWO stages of streamed
//   tiles, so the TMA loads of tile j+1 overlap everything of tile j.
//
// Row side   (stationary Q, dO, g_dQ; streamed K, g_dK, V, g_dV):
//   RA: [S | Q g_dK^T] = Q [K; g_dK]^T (one N = 128 product), gdS += g_dQ K^T
//   RB: [dP | gPdV] = dO [V; g_dV]^T
//   OUT1 = g_dO += P g_dV + g_dp V          OUT0 = g_Q += dS g_dK + g_S K
// Column side (stationary K, V, g_dK, g_dV; streamed Q, g_dQ, dO), scores transposed:
//   RA: [S^T | K g_dQ^T] = K [Q; g_dQ]^T, gdS^T += g_dK Q^T
//   RB: dP^T = V dO^T, gPdV^T = g_dV dO^T
//   OUT1 = g_V += g_dp^T dO                 OUT0 = g_K += dS^T g_dQ + g_S^T Q
// Formulas: reference csrc/flash_double_backward_v7.cu:1354-1454 (rows),
// :1583-1675 (columns).
#include "attn_launch.h"
#include "tc_common.cuh"

namespace attn {
namespace tc {

constexpr int kMmaWarpA = 9;     // issues everything that touches score region RA
constexpr int kMmaWarpB = 10;    // issues everything that touches score region RB
constexpr int kHvpThreads = 352;

struct HvpControl {
  uint64_t stat_full;
  uint64_t stream_full[2];
  uint64_t stream_empty[2];
  uint64_t ra_full, rb_full;      // score regions written by the tensor core
  uint64_t opa_full, opb_full;    // operands written back by the math warps
  uint64_t acc_done;
  uint64_t stats_ready[2];
  uint32_t tmem_base;
  volatile uint32_t abort_flag;
};

template <bool COL, int D>
struct HvpCfg {
  static constexpr int kAtoms = D / 64;
  static constexpr int kNStat = COL ? 4 : 3;
  static constexpr int kNStream = COL ? 3 : 4;
  static constexpr uint32_t kStatBytes = kNStat * kAtoms * kAtomBytesStat;
  static constexpr uint32_t kStageBytes = kNStream * kAtoms * kAtomBytesStrm;
  static constexpr uint32_t kAuxBytes = 256 + (COL ? 2048 : 0);
  static constexpr uint32_t kContentBytes = kStatBytes + 2 * kStageBytes + kAuxBytes;
  static constexpr uint32_t kMaxSmem = 232448;
  static_assert(kContentBytes + 768 <= kMaxSmem, "shared memory over-subscribed");
  static constexpr uint32_t kSmemBytes = (kContentBytes + 1024 <= kMaxSmem) ? kContentBytes + 1024 : kMaxSmem;
  static constexpr int kRA = 0, kRB = 128, kOut0 = 256, kOut1 = 256 + D;
  static_assert(kOut1 + D <= kTmemCols, "tensor memory over-subscribed");
  static constexpr int kKind = COL ? HVP_COL : HVP_ROW;

  // streamed slots.  row side: 0 K, 1 g_dK, 2 V, 3 g_dV (pairs back to back);
  // column side: 0 Q, 1 g_dQ (pair), 2 dO
  __host__ __device__ static constexpr uint32_t stream_off(int slot, int atom) {
    if (!COL)
      return (uint32_t)(slot >> 1) * (2u * kAtoms * kAtomBytesStrm) + (uint32_t)atom * 2u * kAtomBytesStrm +
             (uint32_t)(slot & 1) * kAtomBytesStrm;
    if (slot < 2) return (uint32_t)atom * 2u * kAtomBytesStrm + (uint32_t)slot * kAtomBytesStrm;
    return 2u * kAtoms * kAtomBytesStrm + (uint32_t)atom * kAtomBytesStrm;
  }
  __host__ __device__ static constexpr uint32_t stream_atom_stride(int slot) {
    return (!COL || slot < 2) ? 2u * kAtomBytesStrm : kAtomBytesStrm;
  }
  __host__ __device__ static constexpr int stat_tensor(int slot) {
    if (COL) return slot == 0 ? T_K : slot == 1 ? T_V : slot == 2 ? T_gK : T_gV;
    return slot == 0 ? T_Q : slot == 1 ? T_dO : T_gQ;
  }
  __host__ __device__ static constexpr int stream_tensor(int slot) {
    if (COL) return slot == 0 ? T_Q : slot == 1 ? T_gQ : T_dO;
    return slot == 0 ? T_K : slot == 1 ? T_gK : slot == 2 ? T_V : T_gV;
  }
};

template <bool COL, int D, typename T>
__global__ void __launch_bounds__(kHvpThreads, 1)
hvp_main_kernel(const __grid_constant__ TmaMaps maps, const Geometry g, const Tensors t) {
  using CF = HvpCfg<COL, D>;
  constexpr int KIND = CF::kKind;
  constexpr int kAtoms = CF::kAtoms;
  constexpr uint32_t kIdesc64 = make_idesc(BM, 64, Pack<T>::kIsBf16, 0, 0);
  constexpr uint32_t kIdesc128 = make_idesc(BM, 128, Pack<T>::kIsBf16, 0, 0);
  constexpr uint32_t kIdescOut = make_idesc(BM, D, Pack<T>::kIsBf16, 0, 1);

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
  const uint32_t aux_off = CF::kStatBytes + 2 * CF::kStageBytes;
  HvpControl* ctl = reinterpret_cast<HvpControl*>(smem_gen + aux_off);
  float* col_stats = reinterpret_cast<float*>(smem_gen + aux_off + 256);   // [2][4][64], column side only

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
#ifdef ATTN_EXPERIMENT
  const bool dbg_skip_math = (g.debug & 1) != 0, dbg_skip_mma = (g.debug & 2) != 0;
#else
  constexpr bool dbg_skip_math = false, dbg_skip_mma = false;
#endif
  const int n_stat = COL ? g.N_kv : g.N_q;
  const int tiles = (n_stat + BM - 1) / BM;
  const int bh = g.tile_major ? (int)(blockIdx.x % g.BH) : (int)(blockIdx.x / tiles);
  const int rank = g.tile_major ? (int)(blockIdx.x / g.BH) : (int)(blockIdx.x - bh * tiles);
  const int tile = (COL || g.mask_mode != 0) ? rank : (tiles - 1 - rank);   // heavy tiles first
  const int r0 = tile * BM;

  int lo, hi;
  if (COL) query_range_for_keys(g, r0, r0 + BM, lo, hi);
  else key_range_for_queries(g, r0, r0 + BM, lo, hi);
  const int t_begin = lo / BN;
  const int n_iter = (hi > lo) ? ((hi + BN - 1) / BN - t_begin) : 0;

  const uint32_t bar_stat_full = smem_u32(&ctl->stat_full);
  const uint32_t bar_ra_full = smem_u32(&ctl->ra_full), bar_rb_full = smem_u32(&ctl->rb_full);
  const uint32_t bar_opa_full = smem_u32(&ctl->opa_full), bar_opb_full = smem_u32(&ctl->opb_full);
  const uint32_t bar_acc_done = smem_u32(&ctl->acc_done);
  auto bar_stream_full = [&](int s) { return smem_u32(&ctl->stream_full[s]); };
  auto bar_stream_empty = [&](int s) { return smem_u32(&ctl->stream_empty[s]); };

  if (threadIdx.x == 0) {
    mbar_init(bar_stat_full, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(bar_stream_full(s), 1);
      mbar_init(bar_stream_empty(s), 2);
      mbar_init(smem_u32(&ctl->stats_ready[s]), kMathWarps);
    }
    mbar_init(bar_ra_full, 1);
    mbar_init(bar_rb_full, 1);
    mbar_init(bar_opa_full, kMathWarps);
    mbar_init(bar_opb_full, kMathWarps);
    mbar_init(bar_acc_done, 2);
    ctl->abort_flag = 0u;
    ctl->tmem_base = 0u;
    fence_barrier_init();
    fence_proxy_async_smem();
  }
  __syncthreads();
  if (warp == kMmaWarpA) tmem_alloc(smem_u32(&ctl->tmem_base), kTmemCols);
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
      mbar_arrive_expect_tx(bar_stat_full, CF::kStatBytes);
#pragma unroll
      for (int s = 0; s < CF::kNStat; ++s)
#pragma unroll
        for (int a = 0; a < kAtoms; ++a)
#pragma unroll
          for (int h = 0; h < 2; ++h)
            tma_load_3d(stat_base + (s * kAtoms + a) * kAtomBytesStat + h * kAtomBytesStrm,
                        &maps.m[CF::stat_tensor(s)], a * 64, r0 + h * 64, bh, bar_stat_full);
      bool ok = true;
      for (int it = 0; it < n_iter; ++it) {
        const int st = it & 1;
        ok = mbar_wait(bar_stream_empty(st), ((it >> 1) & 1) ^ 1, abort_flag, t.status, wait_code(KIND, 1));
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
  // MMA issuers.  Warp A owns score region RA (its products and the outputs whose
  // operands live there), warp B owns RB.  Products issued by one warp execute in
  // order, which is what makes overwriting a region right after the outputs that
  // read it safe; the two warps never touch the same columns.  Two issuing warps
  // are used because one warp cannot issue tcgen05.mma fast enough to keep the
  // tensor core busy with N <= 128 instructions.
  // =========================================================================
  else if (warp == kMmaWarpA || warp == kMmaWarpB) {
    if (n_iter > 0) {
      const bool is_a = (warp == kMmaWarpA);
      bool ok = mbar_wait(bar_stat_full, 0, abort_flag, t.status, wait_code(KIND, 2));
      const uint64_t d_stat = smem_desc_sw128(stat_base, 16, 1024);
      auto stat_desc = [&](int slot, int ks) {   // K-major A from shared memory
        return d_stat + (uint64_t)(((slot * kAtoms + (ks >> 2)) * kAtomBytesStat + (ks & 3) * 32) >> 4);
      };
      auto strm_desc_k = [&](uint32_t stage, int slot, int ks) {   // K-major B
        return smem_desc_sw128(stage, 16, 1024) + (uint64_t)((CF::stream_off(slot, ks >> 2) + (ks & 3) * 32) >> 4);
      };
      auto strm_desc_mn = [&](uint32_t stage, int slot, int ks) {  // MN-major B, 16 rows per k-step
        return smem_desc_sw128(stage, CF::stream_atom_stride(slot), 1024) +
               (uint64_t)((CF::stream_off(slot, 0) + ks * 2048) >> 4);
      };
      // operand written by the math warps into a 64-column score slot: the 16 elements of
      // k-step ks sit in 8 columns at 32*(ks/2) + 8*(ks%2) (owner half, then chunk)
      auto op_tmem = [&](int col0, int ks) { return tmem_base + (uint32_t)(col0 + 32 * (ks >> 1) + 8 * (ks & 1)); };
      auto ss = [&](uint32_t d, uint64_t a, uint64_t b, uint32_t idesc, uint32_t acc) {
        if (elect_one()) mma_ss(d, a, b, idesc, acc);
      };
      auto ts = [&](uint32_t d, uint32_t a, uint64_t b, uint32_t idesc, uint32_t acc) {
        if (elect_one()) mma_ts(d, a, b, idesc, acc);
      };
      auto commit = [&](uint32_t bar) { if (elect_one()) mma_commit(bar); };
      constexpr int KS = D / 16, KO = BN / 16;
      const uint32_t ra = tmem_base + CF::kRA, rb = tmem_base + CF::kRB;
      const uint32_t out0 = tmem_base + CF::kOut0, out1 = tmem_base + CF::kOut1;

      auto issue_ra = [&](uint32_t stage) {
        if (dbg_skip_mma) return;
        _Pragma("unroll") for (int ks = 0; ks < KS; ++ks)   // [S | Q g_dK^T] = Q [K; g_dK]^T   | [S^T | K g_dQ^T] = K [Q; g_dQ]^T
          ss(ra, stat_desc(0, ks), strm_desc_k(stage, 0, ks), kIdesc128, ks > 0);
        _Pragma("unroll") for (int ks = 0; ks < KS; ++ks)   // gdS += g_dQ K^T                 | gdS^T += g_dK Q^T
          ss(ra + 64, stat_desc(2, ks), strm_desc_k(stage, 0, ks), kIdesc64, 1);
      };
      auto issue_rb = [&](uint32_t stage) {
        if (dbg_skip_mma) return;
        if constexpr (!COL) {
          _Pragma("unroll") for (int ks = 0; ks < KS; ++ks)   // [dP | gPdV] = dO [V; g_dV]^T
            ss(rb, stat_desc(1, ks), strm_desc_k(stage, 2, ks), kIdesc128, ks > 0);
        } else {
          _Pragma("unroll") for (int ks = 0; ks < KS; ++ks)   // dP^T = V dO^T
            ss(rb, stat_desc(1, ks), strm_desc_k(stage, 2, ks), kIdesc64, ks > 0);
          _Pragma("unroll") for (int ks = 0; ks < KS; ++ks)   // gPdV^T = g_dV dO^T
            ss(rb + 64, stat_desc(3, ks), strm_desc_k(stage, 2, ks), kIdesc64, ks > 0);
        }
      };
      auto issue_out_a = [&](uint32_t stage, bool first) {    // operands living in RA
        if (dbg_skip_mma) return;
        if constexpr (!COL) {
          _Pragma("unroll") for (int ks = 0; ks < KO; ++ks)   // g_dO += P g_dV
            ts(out1, op_tmem(CF::kRA, ks), strm_desc_mn(stage, 3, ks), kIdescOut, !(first && ks == 0));
          _Pragma("unroll") for (int ks = 0; ks < KO; ++ks)   // g_dO += g_dp V
            ts(out1, op_tmem(CF::kRA + 64, ks), strm_desc_mn(stage, 2, ks), kIdescOut, 1);
        } else {
          _Pragma("unroll") for (int ks = 0; ks < KO; ++ks)   // g_V += g_dp^T dO
            ts(out1, op_tmem(CF::kRA + 64, ks), strm_desc_mn(stage, 2, ks), kIdescOut, !(first && ks == 0));
        }
      };
      auto issue_out_b = [&](uint32_t stage, bool first) {    // operands living in RB
        if (dbg_skip_mma) return;
        _Pragma("unroll") for (int ks = 0; ks < KO; ++ks)     // g_Q += dS g_dK      | g_K += dS^T g_dQ
          ts(out0, op_tmem(CF::kRB, ks), strm_desc_mn(stage, 1, ks), kIdescOut, !(first && ks == 0));
        _Pragma("unroll") for (int ks = 0; ks < KO; ++ks)     // g_Q += g_S K        | g_K += g_S^T Q
          ts(out0, op_tmem(CF::kRB + 64, ks), strm_desc_mn(stage, 0, ks), kIdescOut, 1);
      };

      if (ok) ok = mbar_wait(bar_stream_full(0), 0, abort_flag, t.status, wait_code(KIND, 3));
      ok = __all_sync(0xffffffffu, ok);
      if (ok) {
        tc_fence_after_sync();
        if (is_a) { issue_ra(strm_base); commit(bar_ra_full); }
        else { issue_rb(strm_base); commit(bar_rb_full); }
      }
      for (int j = 0; j < n_iter && ok; ++j) {
        const int st = j & 1;
        const uint32_t stage = strm_base + st * CF::kStageBytes;
        const uint32_t nstage = strm_base + (st ^ 1) * CF::kStageBytes;
        const bool more = (j + 1 < n_iter);
        // the math warps have written this tile's operands into the region this warp owns
        ok = mbar_wait(is_a ? bar_opa_full : bar_opb_full, j & 1, abort_flag, t.status, wait_code(KIND, is_a ? 4 : 5));
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after_sync();
        if (is_a) issue_out_a(stage, j == 0); else issue_out_b(stage, j == 0);
        commit(bar_stream_empty(st));     // this warp's last product reading stage st (two arrivals free it)
        if (more) {
          ok = mbar_wait(bar_stream_full(st ^ 1), ((j + 1) >> 1) & 1, abort_flag, t.status, wait_code(KIND, 3));
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
          tc_fence_after_sync();
          // overwrites the region after the outputs above have read it (same warp: in order)
          if (is_a) { issue_ra(nstage); commit(bar_ra_full); }
          else { issue_rb(nstage); commit(bar_rb_full); }
        }
      }
      if (ok) commit(bar_acc_done);
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
    if (COL) query_range_for_keys(g, gidx, gidx + 1, vlo, vhi);
    else key_range_for_queries(g, gidx, gidx + 1, vlo, vhi);
    if (gidx >= n_stat) { vlo = 0; vhi = 0; }
    const uint32_t vspan = (uint32_t)(vhi - vlo);

    // Per-query-row scalars enter the element algebra negated, so that every use is a
    // packed add or fused multiply-add:  nL2 = -L*log2(e), nD2 = -dot2, nDv = -Dv,
    // nC3 = -(dot2*Dv + dot3).  Row side: this thread's own query row (beyond N_q:
    // nL2 = -inf, which makes p = 0).  Column side: per streamed column, from shared memory.
    float2 rnL2 = make_float2(-INFINITY, -INFINITY), rnDv = make_float2(0.f, 0.f);
    float2 rnD2 = make_float2(0.f, 0.f), rnC3 = make_float2(0.f, 0.f);
    if constexpr (!COL) {
      if (gidx < g.N_q) {
        const float L2 = t.L[row_off + gidx] * kLog2e, Dv = t.Dv[row_off + gidx];
        const float d2 = t.dot2[row_off + gidx], c3 = fmaf(d2, Dv, t.dot3[row_off + gidx]);
        rnL2 = make_float2(-L2, -L2); rnDv = make_float2(-Dv, -Dv);
        rnD2 = make_float2(-d2, -d2); rnC3 = make_float2(-c3, -c3);
      }
    }
    const float2 sl2 = make_float2(g.scale_log2e, g.scale_log2e);
    const float2 sc2 = make_float2(g.scale, g.scale);

    float2 p_[16], a_[16];   // carried from half-step 1 to half-step 2
    bool ok = true;
    for (int it = 0; it < n_iter; ++it) {
      const int j0 = (t_begin + it) * BN;
      const float* cs = col_stats + (it & 1) * 256;   // [-L2 | -dot2 | -Dv | -c3] x 64 columns
      if constexpr (COL) {
        const int which = threadIdx.x >> 6, c = threadIdx.x & 63;
        const int qi = j0 + c;
        float v = (which == 0) ? -INFINITY : 0.f;
        if (qi < g.N_q) {
          if (which == 0) v = -t.L[row_off + qi] * kLog2e;
          else if (which == 1) v = -t.dot2[row_off + qi];
          else if (which == 2) v = -t.Dv[row_off + qi];
          else v = -fmaf(t.dot2[row_off + qi], t.Dv[row_off + qi], t.dot3[row_off + qi]);
        }
        col_stats[(it & 1) * 256 + which * 64 + c] = v;
        __syncwarp();
        const uint32_t bar = smem_u32(&ctl->stats_ready[it & 1]);
        if (lane == 0) mbar_arrive(bar);
        ok = mbar_wait(bar, (it >> 1) & 1, abort_flag, t.status, wait_code(KIND, 9));
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
      }
      // all 32 columns this thread handles in this tile are visible: no per-element predicate
      const int first = j0 + half * 32;
      const bool masked = !(first >= vlo && first + 31 < vhi);

      // ---------------- half-step 1: RA -> p, a; operands P, g_dp -----------------
      ok = mbar_wait(bar_ra_full, it & 1, abort_flag, t.status, wait_code(KIND, 6));
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after_sync();
      if (!dbg_skip_math)
#pragma unroll
      for (int ch = 0; ch < 2; ++ch) {
        const int c0 = half * 32 + ch * 16;
        uint32_t s_[16], g_[16];
        tmem_ld16(lane_addr + CF::kRA + c0, s_);
        tmem_ld16(lane_addr + CF::kRA + 64 + c0, g_);
        tmem_ld_wait(s_);
        tmem_ld_wait(g_);
        uint32_t kp[8], kgdp[8];
#pragma unroll
        for (int e = 0; e < 16; e += 2) {
          const int cc = c0 + e;
          float2 nL2 = rnL2, nD2 = rnD2;
          if constexpr (COL) {
            nL2 = *reinterpret_cast<const float2*>(cs + cc);
            nD2 = *reinterpret_cast<const float2*>(cs + 64 + cc);
          }
          const float2 x = __ffma2_rn(make_float2(__uint_as_float(s_[e]), __uint_as_float(s_[e + 1])), sl2, nL2);
          float2 pp = make_float2(ex2(x.x), ex2(x.y));
          if (masked) {
            pp.x = ((uint32_t)(j0 + cc - vlo) < vspan) ? pp.x : 0.f;
            pp.y = ((uint32_t)(j0 + cc + 1 - vlo) < vspan) ? pp.y : 0.f;
          }
          const float2 aa = __ffma2_rn(make_float2(__uint_as_float(g_[e]), __uint_as_float(g_[e + 1])), sc2, nD2);
          const float2 pa = __fmul2_rn(pp, aa);
          p_[ch * 8 + (e >> 1)] = pp;
          a_[ch * 8 + (e >> 1)] = aa;
          kp[e >> 1] = Pack<T>::pack(pp.x, pp.y);
          kgdp[e >> 1] = Pack<T>::pack(pa.x, pa.y);
        }
        if constexpr (!COL) tmem_st8(lane_addr + CF::kRA + half * 32 + ch * 8, kp);
        tmem_st8(lane_addr + CF::kRA + 64 + half * 32 + ch * 8, kgdp);
      }
      tmem_st_wait();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_opa_full);

      // ---------------- half-step 2: RB -> operands dS, g_S ------------------------
      ok = mbar_wait(bar_rb_full, it & 1, abort_flag, t.status, wait_code(KIND, 7));
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after_sync();
      if (!dbg_skip_math)
#pragma unroll
      for (int ch = 0; ch < 2; ++ch) {
        const int c0 = half * 32 + ch * 16;
        uint32_t dp_[16], gp_[16];
        tmem_ld16(lane_addr + CF::kRB + c0, dp_);
        tmem_ld16(lane_addr + CF::kRB + 64 + c0, gp_);
        tmem_ld_wait(dp_);
        tmem_ld_wait(gp_);
        uint32_t kds[8], kgs[8];
#pragma unroll
        for (int e = 0; e < 16; e += 2) {
          const int cc = c0 + e;
          float2 nDv = rnDv, nC3 = rnC3;
          if constexpr (COL) {
            nDv = *reinterpret_cast<const float2*>(cs + 128 + cc);
            nC3 = *reinterpret_cast<const float2*>(cs + 192 + cc);
          }
          const float2 pp = p_[ch * 8 + (e >> 1)], aa = a_[ch * 8 + (e >> 1)];
          const float2 dpd = __fadd2_rn(make_float2(__uint_as_float(dp_[e]), __uint_as_float(dp_[e + 1])), nDv);
          const float2 ds = __fmul2_rn(pp, dpd);
          const float2 tt = __fadd2_rn(make_float2(__uint_as_float(gp_[e]), __uint_as_float(gp_[e + 1])), nC3);
          const float2 gs = __fmul2_rn(pp, __ffma2_rn(aa, dpd, tt));
          kds[e >> 1] = Pack<T>::pack(ds.x, ds.y);
          kgs[e >> 1] = Pack<T>::pack(gs.x, gs.y);
        }
        tmem_st8(lane_addr + CF::kRB + half * 32 + ch * 8, kds);
        tmem_st8(lane_addr + CF::kRB + 64 + half * 32 + ch * 8, kgs);
      }
      tmem_st_wait();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_opb_full);
    }

    // ---------------- outputs --------------------------------------------------------
    if (n_iter > 0 && ok) ok = mbar_wait(bar_acc_done, 0, abort_flag, t.status, wait_code(KIND, 8));
    ok = __all_sync(0xffffffffu, ok);
    tc_fence_after_sync();
    constexpr int kColsPerHalf = D / 2;
    const int n_rows = COL ? g.N_kv : g.N_q;
#pragma unroll
    for (int o = 0; o < 2; ++o) {
      T* dst;
      if constexpr (!COL) dst = (T*)(o == 0 ? t.out_g_Q : t.out_g_dO);
      else dst = (T*)(o == 0 ? t.out_g_K : t.out_g_V);
      const float mul = (o == 0) ? g.scale : 1.f;
      T* prow = dst + ((size_t)bh * n_rows + gidx) * D + half * kColsPerHalf;
#pragma unroll
      for (int ch = 0; ch < kColsPerHalf / 16; ++ch) {
        uint32_t v[16];
        if (n_iter > 0 && ok) {
          tmem_ld16(lane_addr + (o == 0 ? CF::kOut0 : CF::kOut1) + half * kColsPerHalf + ch * 16, v);
          tmem_ld_wait(v);
        } else {
#pragma unroll
          for (int e = 0; e < 16; ++e) v[e] = 0u;
        }
        if (gidx < n_rows) {
          uint4 w0, w1;
          w0.x = Pack<T>::pack(__uint_as_float(v[0]) * mul, __uint_as_float(v[1]) * mul);
          w0.y = Pack<T>::pack(__uint_as_float(v[2]) * mul, __uint_as_float(v[3]) * mul);
          w0.z = Pack<T>::pack(__uint_as_float(v[4]) * mul, __uint_as_float(v[5]) * mul);
          w0.w = Pack<T>::pack(__uint_as_float(v[6]) * mul, __uint_as_float(v[7]) * mul);
          w1.x = Pack<T>::pack(__uint_as_float(v[8]) * mul, __uint_as_float(v[9]) * mul);
          w1.y = Pack<T>::pack(__uint_as_float(v[10]) * mul, __uint_as_float(v[11]) * mul);
          w1.z = Pack<T>::pack(__uint_as_float(v[12]) * mul, __uint_as_float(v[13]) * mul);
          w1.w = Pack<T>::pack(__uint_as_float(v[14]) * mul, __uint_as_float(v[15]) * mul);
          reinterpret_cast<uint4*>(prow + ch * 16)[0] = w0;
          reinterpret_cast<uint4*>(prow + ch * 16)[1] = w1;
        }
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == kMmaWarpA) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

template <bool COL, int D, typename T>
static cudaError_t launch_one(const TmaMaps& maps, const Geometry& g_in, const Tensors& t, cudaStream_t s) {
  using CF = HvpCfg<COL, D>;
  Geometry g = g_in;
  const int n_stat = COL ? g.N_kv : g.N_q;
  const long long ctas = (long long)g.BH * ((n_stat + BM - 1) / BM);
  if (ctas <= 0) return cudaSuccess;
  if (ctas > 0x7fffffffLL) return cudaErrorInvalidValue;
  g.tile_major = ctas < 8 * 148 ? 1 : 0;
  // more than half of an SM's shared memory: one CTA per SM, so the 512-column
  // tensor-memory allocation never waits for a co-resident CTA
  const size_t smem = CF::kSmemBytes < 122880u ? 122880u : CF::kSmemBytes;
  auto kern = hvp_main_kernel<COL, D, T>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return e;
  kern<<<(unsigned)ctas, kHvpThreads, smem, s>>>(maps, g, t);
  return cudaGetLastError();
}

cudaError_t launch_hvp_main(bool col, int D, int is_bf16, const TmaMaps& maps, const Geometry& g,
                            const Tensors& t, cudaStream_t s) {
  if (D == 64) {
    if (is_bf16) return col ? launch_one<true, 64, __nv_bfloat16>(maps, g, t, s) : launch_one<false, 64, __nv_bfloat16>(maps, g, t, s);
    return col ? launch_one<true, 64, __half>(maps, g, t, s) : launch_one<false, 64, __half>(maps, g, t, s);
  }
  if (is_bf16) return col ? launch_one<true, 128, __nv_bfloat16>(maps, g, t, s) : launch_one<false, 128, __nv_bfloat16>(maps, g, t, s);
  return col ? launch_one<true, 128, __half>(maps, g, t, s) : launch_one<false, 128, __half>(maps, g, t, s);
}

}  // namespace tc
}  // namespace attn
