// Tensor-core (tcgen05 / TMEM / TMA) kernels for attention forward, backward
// and double-backward on sm_100a, f16/bf16 inputs, head dimension 64 or 128.
//
// One engine, seven instantiations ("kinds").  A CTA owns a tile of 128
// STATIONARY rows of one (batch, head) -- query rows in the row kinds, key rows in
// the column kinds -- and streams 64-row tiles of the other axis:
//
//   kind      stationary (A operands)   streamed (B operands)    produces
//   FWD_LSE   Q                         K                        L
//   FWD_OUT   Q                         K, V                     O = P V
//   BWD_ROW   Q, dO                     K, V                     dQ = s dS K
//   BWD_COL   K, V                      Q, dO                    dV = P^T dO, dK = s dS^T Q
//   HVP_PRE   Q, dO, g_dQ               K, g_dK, V, g_dV         Dv, dot2, dot3 per row
//   HVP_ROW   Q, dO, g_dQ               K, g_dK, V, g_dV         g_Q, g_dO
//   HVP_COL   K, V, g_dK, g_dV          Q, g_dQ, dO              g_K, g_V
//
// In the column kinds the score tile is computed transposed (keys on the TMEM
// lanes), so every kind has the same operand structure:
//   score  [128 x 64]  = stationary[128 x D] * streamed[64 x D]^T     (both K-major)
//   output [128 x D]  += elementwise(score)[128 x 64] * streamed[64 x D]  (B MN-major)
// and the same 64 x D shared-memory tile serves as K-major B of a score product
// and as MN-major B of an output product.
//
// Warp roles (320 threads): warps 0-7 do the element-wise math (warp w reads
// TMEM lanes 32*(w%4).., columns 32*(w/4).. of each 64-column score slot, i.e.
// one thread per (row, half-tile)); warp 8 is the TMA producer; warp 9 allocates
// tensor memory and issues every tcgen05.mma.  They hand tiles to one another
// through mbarriers; every wait is bounded (tc_primitives.cuh).
//
// Determinism: each output element is accumulated by one CTA in a fixed order;
// there are no atomics.
#include "attn_common.cuh"
#include "attn_launch.h"
#include "tc_common.cuh"

#include <cstdio>
#include <cstring>
#include <mutex>

namespace attn {
namespace tc {

// ---------------------------------------------------------------------------
// per-kind configuration
// ---------------------------------------------------------------------------
template <int KIND, int D>
struct Traits {
  static constexpr bool kCol = (KIND == BWD_COL || KIND == HVP_COL);
  static constexpr bool kReduce = (KIND == FWD_LSE || KIND == HVP_PRE);   // row sums only
  static constexpr int kNStat = (KIND == FWD_LSE || KIND == FWD_OUT) ? 1
                                : (KIND == BWD_ROW || KIND == BWD_COL) ? 2
                                : (KIND == HVP_COL) ? 4 : 3;
  static constexpr int kNStream = (KIND == FWD_LSE) ? 1
                                  : (KIND == FWD_OUT || KIND == BWD_ROW || KIND == BWD_COL) ? 2
                                  : (KIND == HVP_COL) ? 3 : 4;
  // 64-column fp32 score slots in tensor memory
  static constexpr int kNScore = (KIND == FWD_LSE || KIND == FWD_OUT) ? 1
                                 : (KIND == BWD_ROW || KIND == BWD_COL) ? 2 : 4;
  static constexpr int kNOp = kReduce ? 0
                              : (KIND == FWD_OUT || KIND == BWD_ROW) ? 1
                              : (KIND == BWD_COL) ? 2 : (KIND == HVP_ROW) ? 4 : 3;
  static constexpr int kNOut = kReduce ? 0 : (KIND == FWD_OUT || KIND == BWD_ROW) ? 1 : 2;
  static constexpr int kAtoms = D / 64;
  // pairs of streamed tensors laid out back to back so that one N = 128 MMA
  // covers both (same A operand): (K, g_dK) and (V, g_dV) in the HVP row kinds,
  // (Q, g_dQ) in HVP_COL
  static constexpr bool kPaired = (KIND == HVP_PRE || KIND == HVP_ROW);

  static constexpr int kScoreBufs =
      ((kNScore * 64 * 2 + kNOut * D) <= kTmemCols) ? 2 : 1;
  static constexpr uint32_t kStatBytes = kNStat * kAtoms * kAtomBytesStat;
  static constexpr uint32_t kStageBytes = kNStream * kAtoms * kAtomBytesStrm;
  static constexpr uint32_t kOpBytes = kNOp * kOpTileBytes;
  // control block (256 B) + 2 KB of floats: per-column statistics (column kinds)
  // or the cross-half reduction scratch (reduction kinds)
  static constexpr uint32_t kAuxBytes = 256 + ((kCol || kReduce) ? 2048 : 0);
  static constexpr uint32_t kMaxSmem = 232448;              // 227 KB opt-in limit per CTA
  static constexpr uint32_t kBudget = kMaxSmem - 768;       // room to round the base up to 1024
  static constexpr int kStages =
      (kStatBytes + 2 * kStageBytes + kOpBytes + kAuxBytes <= kBudget) ? 2 : 1;
  static constexpr uint32_t kContentBytes = kStatBytes + kStages * kStageBytes + kOpBytes + kAuxBytes;
  static constexpr uint32_t kSmemBytes =
      (kContentBytes + 1024 <= kMaxSmem) ? kContentBytes + 1024 : kMaxSmem;
  // issue the next tile's score products before the current tile's output products
  static constexpr bool kLookahead = (!kReduce) && (kStages >= 2);
  static constexpr int kScoreCol0 = 0;
  static constexpr int kOutCol0 = kScoreBufs * kNScore * 64;
  static_assert(kOutCol0 + kNOut * D <= kTmemCols, "tensor memory over-subscribed");
  static_assert(kStatBytes + kStageBytes + kOpBytes + kAuxBytes <= kBudget, "shared memory over-subscribed");

  // byte offset of (slot, atom) inside one stage of streamed tiles
  __host__ __device__ static constexpr uint32_t stream_off(int slot, int atom) {
    if (kPaired)
      return (uint32_t)(slot >> 1) * (2u * kAtoms * kAtomBytesStrm) + (uint32_t)atom * 2u * kAtomBytesStrm +
             (uint32_t)(slot & 1) * kAtomBytesStrm;
    if (KIND == HVP_COL) {
      if (slot < 2) return (uint32_t)atom * 2u * kAtomBytesStrm + (uint32_t)slot * kAtomBytesStrm;
      return 2u * kAtoms * kAtomBytesStrm + (uint32_t)atom * kAtomBytesStrm;
    }
    return (uint32_t)slot * kAtoms * kAtomBytesStrm + (uint32_t)atom * kAtomBytesStrm;
  }
  // distance between successive 64-column atoms of one streamed slot
  __host__ __device__ static constexpr uint32_t stream_atom_stride(int slot) {
    if (kPaired) return 2u * kAtomBytesStrm;
    if (KIND == HVP_COL) return slot < 2 ? 2u * kAtomBytesStrm : kAtomBytesStrm;
    return kAtomBytesStrm;
  }
  __host__ __device__ static constexpr int stat_tensor(int slot) {
    if (KIND == FWD_LSE || KIND == FWD_OUT) return T_Q;
    if (KIND == BWD_ROW) return slot == 0 ? T_Q : T_dO;
    if (KIND == BWD_COL) return slot == 0 ? T_K : T_V;
    if (KIND == HVP_COL) return slot == 0 ? T_K : slot == 1 ? T_V : slot == 2 ? T_gK : T_gV;
    return slot == 0 ? T_Q : slot == 1 ? T_dO : T_gQ;
  }
  __host__ __device__ static constexpr int stream_tensor(int slot) {
    if (KIND == FWD_LSE) return T_K;
    if (KIND == FWD_OUT || KIND == BWD_ROW) return slot == 0 ? T_K : T_V;
    if (KIND == BWD_COL) return slot == 0 ? T_Q : T_dO;
    if (KIND == HVP_COL) return slot == 0 ? T_Q : slot == 1 ? T_gQ : T_dO;
    return slot == 0 ? T_K : slot == 1 ? T_gK : slot == 2 ? T_V : T_gV;
  }
};

// ---------------------------------------------------------------------------
// the engine
// ---------------------------------------------------------------------------
template <int KIND, int D, typename T>
__global__ void __launch_bounds__(kThreads, 1)
attn_tc_kernel(const __grid_constant__ TmaMaps maps, const Geometry g, const Tensors t) {
  using TR = Traits<KIND, D>;
  constexpr int kAtoms = TR::kAtoms;
  constexpr uint32_t kIdesc64 = make_idesc(BM, 64, Pack<T>::kIsBf16, 0, 0);
  constexpr uint32_t kIdesc128 = make_idesc(BM, 128, Pack<T>::kIsBf16, 0, 0);
  constexpr uint32_t kIdescOut = make_idesc(BM, D, Pack<T>::kIsBf16, 0, 1);

  extern __shared__ __align__(1024) uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  {
    uint32_t dyn_size;
    asm("mov.u32 %0, %%dynamic_smem_size;" : "=r"(dyn_size));
    if (smem_base - smem_u32(smem_raw) + TR::kContentBytes > dyn_size) {   // uniform over the CTA
      if (threadIdx.x == 0 && t.status != nullptr) atomicCAS(t.status, 0u, wait_code(KIND, 15));
      return;
    }
  }
  const uint32_t stat_base = smem_base;
  const uint32_t strm_base = stat_base + TR::kStatBytes;
  const uint32_t op_base = strm_base + TR::kStages * TR::kStageBytes;
  const uint32_t aux_off = TR::kStatBytes + TR::kStages * TR::kStageBytes + TR::kOpBytes;
  Control* ctl = reinterpret_cast<Control*>(smem_gen + aux_off);
  float* aux_f = reinterpret_cast<float*>(smem_gen + aux_off + 256);   // 512 floats when present

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
#ifdef ATTN_EXPERIMENT
  const bool dbg_skip_math = (g.debug & 1) != 0, dbg_skip_mma = (g.debug & 2) != 0;
#else
  constexpr bool dbg_skip_math = false, dbg_skip_mma = false;
#endif
  const int n_stat = TR::kCol ? g.N_kv : g.N_q;
  const int tiles = (n_stat + BM - 1) / BM;
  const int bh = g.tile_major ? (int)(blockIdx.x % g.BH) : (int)(blockIdx.x / tiles);
  const int rank = g.tile_major ? (int)(blockIdx.x / g.BH) : (int)(blockIdx.x - bh * tiles);
  // heavy tiles first within a head: late query tiles / early key tiles see the most work
  const int tile = (TR::kCol || g.mask_mode != 0) ? rank : (tiles - 1 - rank);
  const int r0 = tile * BM;

  int lo, hi;
  if (TR::kCol) query_range_for_keys(g, r0, r0 + BM, lo, hi);
  else key_range_for_queries(g, r0, r0 + BM, lo, hi);
  const int t_begin = lo / BN;
  const int n_iter = (hi > lo) ? ((hi + BN - 1) / BN - t_begin) : 0;

  const uint32_t bar_stat_full = smem_u32(&ctl->stat_full);
  const uint32_t bar_opnd_full = smem_u32(&ctl->opnd_full);
  const uint32_t bar_opnd_free = smem_u32(&ctl->opnd_free);
  const uint32_t bar_acc_done = smem_u32(&ctl->acc_done);
  auto bar_stream_full = [&](int s) { return smem_u32(&ctl->stream_full[s]); };
  auto bar_stream_empty = [&](int s) { return smem_u32(&ctl->stream_empty[s]); };
  auto bar_score_full = [&](int s) { return smem_u32(&ctl->score_full[s]); };
  auto bar_score_free = [&](int s) { return smem_u32(&ctl->score_free[s]); };

  if (threadIdx.x == 0) {
    mbar_init(bar_stat_full, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(bar_stream_full(s), 1);
      mbar_init(bar_stream_empty(s), 1);
      mbar_init(bar_score_full(s), 1);
      mbar_init(bar_score_free(s), kMathWarps);
    }
    mbar_init(bar_opnd_full, kMathWarps);
    mbar_init(bar_opnd_free, 1);
    mbar_init(bar_acc_done, 1);
    mbar_init(smem_u32(&ctl->stats_ready[0]), kMathWarps);
    mbar_init(smem_u32(&ctl->stats_ready[1]), kMathWarps);
    ctl->abort_flag = 0u;
    ctl->tmem_base = 0u;
    fence_barrier_init();
    fence_proxy_async_smem();
  }
  __syncthreads();
  if (warp == kMmaWarp) tmem_alloc(smem_u32(&ctl->tmem_base), kTmemCols);
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
      mbar_arrive_expect_tx(bar_stat_full, TR::kStatBytes);
#pragma unroll
      for (int s = 0; s < TR::kNStat; ++s)
#pragma unroll
        for (int a = 0; a < kAtoms; ++a)
#pragma unroll
          for (int h = 0; h < 2; ++h)
            tma_load_3d(stat_base + (s * kAtoms + a) * kAtomBytesStat + h * kAtomBytesStrm,
                        &maps.m[TR::stat_tensor(s)], a * 64, r0 + h * 64, bh, bar_stat_full);
      bool ok = true;
      for (int it = 0; it < n_iter && ok; ++it) {
        const int st = it % TR::kStages;
        ok = mbar_wait(bar_stream_empty(st), ((it / TR::kStages) & 1) ^ 1, abort_flag, t.status,
                       wait_code(KIND, 1));
        if (!ok) break;
        mbar_arrive_expect_tx(bar_stream_full(st), TR::kStageBytes);
        const uint32_t stage = strm_base + st * TR::kStageBytes;
#pragma unroll
        for (int s = 0; s < TR::kNStream; ++s)
#pragma unroll
          for (int a = 0; a < kAtoms; ++a)
            tma_load_3d(stage + TR::stream_off(s, a), &maps.m[TR::stream_tensor(s)], a * 64,
                        (t_begin + it) * BN, bh, bar_stream_full(st));
      }
      if (!ok) {
        // give copies already in flight a bounded chance to land before the CTA exits
        const long long t0 = clock64();
        while (clock64() - t0 < 2000000LL) { }
      }
    }
  }
  // =========================================================================
  // MMA issuer
  // =========================================================================
  else if (warp == kMmaWarp) {
    // the whole warp runs this loop converged; one elected lane issues (keeps the descriptors in
    // uniform registers: a single diverged lane issues about 1.5x slower)
    if (n_iter > 0) {
      bool ok = mbar_wait(bar_stat_full, 0, abort_flag, t.status, wait_code(KIND, 2));
      ok = __all_sync(0xffffffffu, ok);
      auto mma_ss_e = [&](uint32_t d, uint64_t a_, uint64_t b_, uint32_t idesc, uint32_t acc) {
        if (elect_one()) mma_ss(d, a_, b_, idesc, acc);
      };
      auto commit_e = [&](uint32_t bar) { if (elect_one()) mma_commit(bar); };
      // Descriptor of (base + byte offset) == descriptor of base + (offset >> 4): shared-memory
      // addresses stay below 2^18, so the 14-bit start-address field never carries.
      const uint64_t d_stat = smem_desc_sw128(stat_base, 16, 1024);
      const uint64_t d_op = smem_desc_sw128(op_base, 16, 1024);
      auto stat_desc = [&](int slot, int ks) {   // K-major A, k-step ks of 16 columns
        return d_stat + (uint64_t)(((slot * kAtoms + (ks >> 2)) * kAtomBytesStat + (ks & 3) * 32) >> 4);
      };
      auto strm_desc_k = [&](uint32_t stage, int slot, int ks) {   // K-major B
        return smem_desc_sw128(stage, 16, 1024) + (uint64_t)((TR::stream_off(slot, ks >> 2) + (ks & 3) * 32) >> 4);
      };
      auto strm_desc_mn = [&](uint32_t stage, int slot, int ks) {  // MN-major B, 16 rows per k-step
        return smem_desc_sw128(stage, TR::stream_atom_stride(slot), 1024) +
               (uint64_t)((TR::stream_off(slot, 0) + ks * 2048) >> 4);
      };
      auto op_desc = [&](int o, int ks) {                          // K-major A, operand tile
        return d_op + (uint64_t)((o * kOpTileBytes + ks * 32) >> 4);
      };
      // score products of one tile into score buffer sb
      auto issue_scores = [&](uint32_t stage, int sb) {
        const uint32_t c0 = tmem_base + TR::kScoreCol0 + sb * TR::kNScore * 64;
        constexpr int KS = D / 16;
        if constexpr (KIND == FWD_LSE || KIND == FWD_OUT) {
          _Pragma("unroll") for (int ks = 0; ks < KS; ++ks) mma_ss_e(c0, stat_desc(0, ks), strm_desc_k(stage, 0, ks), kIdesc64, ks > 0);
        } else if constexpr (KIND == BWD_ROW || KIND == BWD_COL) {
          // slot 0: S (or S^T), slot 1: dP (or dP^T)
          _Pragma("unroll") for (int ks = 0; ks < KS; ++ks) mma_ss_e(c0, stat_desc(0, ks), strm_desc_k(stage, 0, ks), kIdesc64, ks > 0);
          _Pragma("unroll") for (int ks = 0; ks < KS; ++ks) mma_ss_e(c0 + 64, stat_desc(1, ks), strm_desc_k(stage, 1, ks), kIdesc64, ks > 0);
        } else if constexpr (KIND == HVP_PRE || KIND == HVP_ROW) {
          // slots: 0 S | 1 gdS | 2 dP | 3 gPdV.  stat: 0 Q, 1 dO, 2 g_dQ.  stream: 0 K, 1 g_dK, 2 V, 3 g_dV
          _Pragma("unroll") for (int ks = 0; ks < KS; ++ks)   // [S | Q g_dK^T] = Q [K ; g_dK]^T
            mma_ss_e(c0, stat_desc(0, ks), strm_desc_k(stage, 0, ks), kIdesc128, ks > 0);
          _Pragma("unroll") for (int ks = 0; ks < KS; ++ks)   // [dP | gPdV] = dO [V ; g_dV]^T
            mma_ss_e(c0 + 128, stat_desc(1, ks), strm_desc_k(stage, 2, ks), kIdesc128, ks > 0);
          _Pragma("unroll") for (int ks = 0; ks < KS; ++ks)   // gdS += g_dQ K^T
            mma_ss_e(c0 + 64, stat_desc(2, ks), strm_desc_k(stage, 0, ks), kIdesc64, 1);
        } else {   // HVP_COL.  stat: 0 K, 1 V, 2 g_dK, 3 g_dV.  stream: 0 Q, 1 g_dQ, 2 dO
          _Pragma("unroll") for (int ks = 0; ks < KS; ++ks)   // [S^T | K g_dQ^T] = K [Q ; g_dQ]^T
            mma_ss_e(c0, stat_desc(0, ks), strm_desc_k(stage, 0, ks), kIdesc128, ks > 0);
          _Pragma("unroll") for (int ks = 0; ks < KS; ++ks)   // gdS^T += g_dK Q^T
            mma_ss_e(c0 + 64, stat_desc(2, ks), strm_desc_k(stage, 0, ks), kIdesc64, 1);
          _Pragma("unroll") for (int ks = 0; ks < KS; ++ks)   // dP^T = V dO^T
            mma_ss_e(c0 + 128, stat_desc(1, ks), strm_desc_k(stage, 2, ks), kIdesc64, ks > 0);
          _Pragma("unroll") for (int ks = 0; ks < KS; ++ks)   // gPdV^T = g_dV dO^T
            mma_ss_e(c0 + 192, stat_desc(3, ks), strm_desc_k(stage, 2, ks), kIdesc64, ks > 0);
        }
      };
      // output products of one tile; `first` clears the accumulators
      auto issue_outs = [&](uint32_t stage, bool first) {
        const uint32_t o0 = tmem_base + TR::kOutCol0, o1 = o0 + D;
        constexpr int KS = BN / 16;
        (void)o1;
        if constexpr (KIND == FWD_OUT) {          // O += P V
          _Pragma("unroll") for (int ks = 0; ks < KS; ++ks) mma_ss_e(o0, op_desc(0, ks), strm_desc_mn(stage, 1, ks), kIdescOut, !(first && ks == 0));
        } else if constexpr (KIND == BWD_ROW) {   // dQ += dS K
          _Pragma("unroll") for (int ks = 0; ks < KS; ++ks) mma_ss_e(o0, op_desc(0, ks), strm_desc_mn(stage, 0, ks), kIdescOut, !(first && ks == 0));
        } else if constexpr (KIND == BWD_COL) {   // dV += P^T dO ; dK += dS^T Q
          _Pragma("unroll") for (int ks = 0; ks < KS; ++ks) mma_ss_e(o0, op_desc(0, ks), strm_desc_mn(stage, 1, ks), kIdescOut, !(first && ks == 0));
          _Pragma("unroll") for (int ks = 0; ks < KS; ++ks) mma_ss_e(o1, op_desc(1, ks), strm_desc_mn(stage, 0, ks), kIdescOut, !(first && ks == 0));
        } else if constexpr (KIND == HVP_ROW) {   // ops: 0 dS, 1 g_S, 2 P, 3 g_dp
          _Pragma("unroll") for (int ks = 0; ks < KS; ++ks) mma_ss_e(o0, op_desc(0, ks), strm_desc_mn(stage, 1, ks), kIdescOut, !(first && ks == 0));  // dS g_dK
          _Pragma("unroll") for (int ks = 0; ks < KS; ++ks) mma_ss_e(o0, op_desc(1, ks), strm_desc_mn(stage, 0, ks), kIdescOut, 1);                    // g_S K
          _Pragma("unroll") for (int ks = 0; ks < KS; ++ks) mma_ss_e(o1, op_desc(2, ks), strm_desc_mn(stage, 3, ks), kIdescOut, !(first && ks == 0));  // P g_dV
          _Pragma("unroll") for (int ks = 0; ks < KS; ++ks) mma_ss_e(o1, op_desc(3, ks), strm_desc_mn(stage, 2, ks), kIdescOut, 1);                    // g_dp V
        } else if constexpr (KIND == HVP_COL) {   // ops: 0 dS^T, 1 g_S^T, 2 g_dp^T
          _Pragma("unroll") for (int ks = 0; ks < KS; ++ks) mma_ss_e(o0, op_desc(0, ks), strm_desc_mn(stage, 1, ks), kIdescOut, !(first && ks == 0));  // dS^T g_dQ
          _Pragma("unroll") for (int ks = 0; ks < KS; ++ks) mma_ss_e(o0, op_desc(1, ks), strm_desc_mn(stage, 0, ks), kIdescOut, 1);                    // g_S^T Q
          _Pragma("unroll") for (int ks = 0; ks < KS; ++ks) mma_ss_e(o1, op_desc(2, ks), strm_desc_mn(stage, 2, ks), kIdescOut, !(first && ks == 0));  // g_dp^T dO
        }
      };
      auto do_out = [&](int k) -> bool {
        bool okw = mbar_wait(bar_opnd_full, k & 1, abort_flag, t.status, wait_code(KIND, 5));
        okw = __all_sync(0xffffffffu, okw);
        if (!okw) return false;
        tc_fence_after_sync();
        const int st = k % TR::kStages;
        if (!dbg_skip_mma) issue_outs(strm_base + st * TR::kStageBytes, k == 0);
        commit_e(bar_opnd_free);
        commit_e(bar_stream_empty(st));
        return true;
      };

      for (int it = 0; it < n_iter && ok; ++it) {
        const int st = it % TR::kStages, sb = it % TR::kScoreBufs;
        ok = mbar_wait(bar_stream_full(st), (it / TR::kStages) & 1, abort_flag, t.status, wait_code(KIND, 3));
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        ok = mbar_wait(bar_score_free(sb), ((it / TR::kScoreBufs) & 1) ^ 1, abort_flag, t.status, wait_code(KIND, 4));
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after_sync();
        if (!dbg_skip_mma) issue_scores(strm_base + st * TR::kStageBytes, sb);
        commit_e(bar_score_full(sb));
        if constexpr (TR::kReduce) {
          commit_e(bar_stream_empty(st));
        } else if constexpr (TR::kLookahead) {
          if (it > 0) ok = do_out(it - 1);
        } else {
          ok = do_out(it);
        }
      }
      if constexpr (!TR::kReduce) {
        if constexpr (TR::kLookahead) { if (ok) ok = do_out(n_iter - 1); }
        if (ok) commit_e(bar_acc_done);
      }
    }
  }
  // =========================================================================
  // math warps
  // =========================================================================
  else {
    const int quarter = warp & 3, half = warp >> 2;
    const int row = quarter * 32 + lane;         // stationary row within the tile == TMEM lane
    const int gidx = r0 + row;                   // global stationary index
    const uint32_t lane_addr = tmem_base + ((uint32_t)(quarter * 32) << 16);
    const size_t row_off = (size_t)bh * g.N_q;

    // visible range of streamed indices for this thread's stationary row
    int vlo, vhi;
    if (TR::kCol) query_range_for_keys(g, gidx, gidx + 1, vlo, vhi);
    else key_range_for_queries(g, gidx, gidx + 1, vlo, vhi);
    if (gidx >= n_stat) { vlo = 0; vhi = 0; }
    const uint32_t vspan = (uint32_t)(vhi - vlo);

    // per-row statistics (row kinds: this thread's query row)
    RowStats rs{INFINITY, 0.f, 0.f, 0.f};
    if constexpr (!TR::kCol && KIND != FWD_LSE) {
      if (gidx < g.N_q) {
        rs.L2 = t.L[row_off + gidx] * kLog2e;
        if constexpr (KIND == BWD_ROW || KIND == HVP_ROW) rs.Dv = t.Dv[row_off + gidx];
        if constexpr (KIND == HVP_ROW) { rs.dot2 = t.dot2[row_off + gidx]; rs.dot3 = t.dot3[row_off + gidx]; }
      }
    }
    // column kinds: statistics of the 64 streamed query rows, double-buffered in the aux area
    // layout: aux_f[buf*256 + which*64 + col], which = 0 L2, 1 Dv, 2 dot2, 3 dot3
    float* col_stats = aux_f;

    // running reductions
    float acc_m = -INFINITY, acc_l = 0.f;                       // FWD_LSE
    float acc_D = 0.f, acc_2 = 0.f, acc_A = 0.f, acc_E = 0.f;   // HVP_PRE

    bool ok = true;
    for (int it = 0; it < n_iter && ok; ++it) {
      const int sb = it % TR::kScoreBufs;
      const int j0 = (t_begin + it) * BN;      // first streamed index of this tile
      if constexpr (TR::kCol) {
        // one value per math thread: 4 arrays x 64 columns
        const int which = threadIdx.x >> 6, c = threadIdx.x & 63;
        const int qi = j0 + c;
        float v = (which == 0) ? INFINITY : 0.f;
        if (qi < g.N_q) {
          if (which == 0) v = t.L[row_off + qi] * kLog2e;
          else if (which == 1) v = t.Dv[row_off + qi];
          else if (KIND == HVP_COL) v = (which == 2) ? t.dot2[row_off + qi] : t.dot3[row_off + qi];
        }
        col_stats[(it & 1) * 256 + which * 64 + c] = v;
        __syncwarp();
        const uint32_t bar = smem_u32(&ctl->stats_ready[it & 1]);
        if (lane == 0) mbar_arrive(bar);
        ok = mbar_wait(bar, (it >> 1) & 1, abort_flag, t.status, wait_code(KIND, 9));
        ok = __all_sync(0xffffffffu, ok);   // keep the warp converged for the .sync.aligned TMEM loads
        if (!ok) break;
      }
      ok = mbar_wait(bar_score_full(sb), (it / TR::kScoreBufs) & 1, abort_flag, t.status, wait_code(KIND, 6));
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after_sync();
      const uint32_t sc = lane_addr + TR::kScoreCol0 + sb * TR::kNScore * 64 + half * 32;
      const float* cs = col_stats + (it & 1) * 256;
      (void)cs;

      if (dbg_skip_math) {
        if constexpr (!TR::kReduce) {
          if (it > 0) ok = mbar_wait(bar_opnd_free, (it - 1) & 1, abort_flag, t.status, wait_code(KIND, 7));
        }
      } else
#pragma unroll
      for (int ch = 0; ch < 2; ++ch) {
        const int c0 = half * 32 + ch * 16;    // column inside the 64-wide tile
        uint32_t s_[16];
        tmem_ld16(sc + ch * 16, s_);
        if constexpr (KIND == FWD_LSE) {
          tmem_ld_wait(s_);
          float x[16], mx = -INFINITY;
#pragma unroll
          for (int e = 0; e < 16; ++e) {
            const bool vis = (uint32_t)(j0 + c0 + e - vlo) < vspan;
            x[e] = vis ? __uint_as_float(s_[e]) * g.scale_log2e : -INFINITY;
            mx = fmaxf(mx, x[e]);
          }
          if (mx > -INFINITY) {
            const float mn = fmaxf(acc_m, mx);
            float sum = 0.f;
#pragma unroll
            for (int e = 0; e < 16; ++e) sum += ex2(x[e] - mn);
            acc_l = acc_l * ex2(acc_m - mn) + sum;
            acc_m = mn;
          }
        } else if constexpr (KIND == FWD_OUT) {
          tmem_ld_wait(s_);
          uint32_t pk[8];
#pragma unroll
          for (int e = 0; e < 16; e += 2) {
            const float p0 = prob(__uint_as_float(s_[e]), g.scale_log2e, rs.L2, (uint32_t)(j0 + c0 + e - vlo) < vspan);
            const float p1 = prob(__uint_as_float(s_[e + 1]), g.scale_log2e, rs.L2, (uint32_t)(j0 + c0 + e + 1 - vlo) < vspan);
            pk[e >> 1] = Pack<T>::pack(p0, p1);
          }
          if (ch == 0 && it > 0) ok = mbar_wait(bar_opnd_free, (it - 1) & 1, abort_flag, t.status, wait_code(KIND, 7));
          store_op16(op_base, row, c0, pk);
        } else if constexpr (KIND == BWD_ROW || KIND == BWD_COL) {
          uint32_t d_[16];
          tmem_ld16(sc + 64 + ch * 16, d_);
          tmem_ld_wait(s_);
          tmem_ld_wait(d_);
          uint32_t pk0[8], pk1[8];
#pragma unroll
          for (int e = 0; e < 16; e += 2) {
            float pr[2], ds[2];
#pragma unroll
            for (int u = 0; u < 2; ++u) {
              const int cc = c0 + e + u;
              const bool vis = (uint32_t)(j0 + cc - vlo) < vspan;
              const float L2 = TR::kCol ? cs[cc] : rs.L2;
              const float Dv = TR::kCol ? cs[64 + cc] : rs.Dv;
              pr[u] = prob(__uint_as_float(s_[e + u]), g.scale_log2e, L2, vis);
              ds[u] = pr[u] * (__uint_as_float(d_[e + u]) - Dv);
            }
            pk0[e >> 1] = Pack<T>::pack(pr[0], pr[1]);
            pk1[e >> 1] = Pack<T>::pack(ds[0], ds[1]);
          }
          if (ch == 0 && it > 0) ok = mbar_wait(bar_opnd_free, (it - 1) & 1, abort_flag, t.status, wait_code(KIND, 7));
          if constexpr (KIND == BWD_ROW) {
            store_op16(op_base, row, c0, pk1);                  // dS
          } else {
            store_op16(op_base, row, c0, pk0);                  // P^T
            store_op16(op_base + kOpTileBytes, row, c0, pk1);   // dS^T
          }
        } else {   // HVP kinds: slots 0 S | 1 gdS | 2 dP | 3 gPdV
          uint32_t gs_[16], dp_[16], gp_[16];
          tmem_ld16(sc + 64 + ch * 16, gs_);
          tmem_ld16(sc + 128 + ch * 16, dp_);
          tmem_ld16(sc + 192 + ch * 16, gp_);
          tmem_ld_wait(s_);
          tmem_ld_wait(gs_);
          tmem_ld_wait(dp_);
          tmem_ld_wait(gp_);
          if constexpr (KIND == HVP_PRE) {
#pragma unroll
            for (int e = 0; e < 16; ++e) {
              const bool vis = (uint32_t)(j0 + c0 + e - vlo) < vspan;
              const float pr = prob(__uint_as_float(s_[e]), g.scale_log2e, rs.L2, vis);
              const float gds = __uint_as_float(gs_[e]) * g.scale;
              const float dp = __uint_as_float(dp_[e]);
              acc_D = fmaf(pr, dp, acc_D);
              acc_2 = fmaf(pr, gds, acc_2);
              acc_A = fmaf(pr * gds, dp, acc_A);
              acc_E = fmaf(pr, __uint_as_float(gp_[e]), acc_E);
            }
          } else {
            uint32_t k_dS[8], k_gS[8], k_p[8], k_gdp[8];
#pragma unroll
            for (int e = 0; e < 16; e += 2) {
              HvpTerms h[2];
#pragma unroll
              for (int u = 0; u < 2; ++u) {
                const int cc = c0 + e + u;
                const bool vis = (uint32_t)(j0 + cc - vlo) < vspan;
                RowStats r = rs;
                if constexpr (TR::kCol) { r.L2 = cs[cc]; r.Dv = cs[64 + cc]; r.dot2 = cs[128 + cc]; r.dot3 = cs[192 + cc]; }
                const float pr = prob(__uint_as_float(s_[e + u]), g.scale_log2e, r.L2, vis);
                h[u] = hvp_terms(pr, __uint_as_float(dp_[e + u]), __uint_as_float(gs_[e + u]),
                                 __uint_as_float(gp_[e + u]), g.scale, r);
              }
              k_dS[e >> 1] = Pack<T>::pack(h[0].dS, h[1].dS);
              k_gS[e >> 1] = Pack<T>::pack(h[0].g_S, h[1].g_S);
              k_p[e >> 1] = Pack<T>::pack(h[0].p, h[1].p);
              k_gdp[e >> 1] = Pack<T>::pack(h[0].g_dp, h[1].g_dp);
            }
            if (ch == 0 && it > 0) ok = mbar_wait(bar_opnd_free, (it - 1) & 1, abort_flag, t.status, wait_code(KIND, 7));
            store_op16(op_base, row, c0, k_dS);
            store_op16(op_base + kOpTileBytes, row, c0, k_gS);
            if constexpr (KIND == HVP_ROW) {
              store_op16(op_base + 2 * kOpTileBytes, row, c0, k_p);
              store_op16(op_base + 3 * kOpTileBytes, row, c0, k_gdp);
            } else {
              store_op16(op_base + 2 * kOpTileBytes, row, c0, k_gdp);
            }
          }
        }
      }
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      // every tcgen05.ld of this tile has completed: the score buffer may be overwritten
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_score_free(sb));
      if constexpr (!TR::kReduce) {
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_opnd_full);
      }
    }

    // ---------------- results -------------------------------------------------
    if constexpr (KIND == FWD_LSE) {
      // combine the two column halves of each row
      float* xm = aux_f;                // [128]
      float* xl = aux_f + 128;          // [128]
      if (half == 1) { xm[row] = acc_m; xl[row] = acc_l; }
      named_barrier_sync(1, kMathThreads);
      if (half == 0 && gidx < g.N_q) {
        const float m1 = xm[row], l1 = xl[row];
        const float mt = fmaxf(acc_m, m1);
        float L = -INFINITY;
        if (mt > -INFINITY) {
          const float lt = acc_l * ex2(acc_m - mt) + l1 * ex2(m1 - mt);
          L = (mt + log2f(lt)) * kLn2;
        }
        t.out_L[row_off + gidx] = L;
      }
    } else if constexpr (KIND == HVP_PRE) {
      float* x = aux_f;                 // [4][128]
      if (half == 1) { x[row] = acc_D; x[128 + row] = acc_2; x[256 + row] = acc_A; x[384 + row] = acc_E; }
      named_barrier_sync(1, kMathThreads);
      if (half == 0 && gidx < g.N_q) {
        const float Dv = acc_D + x[row], d2 = acc_2 + x[128 + row];
        const float A = acc_A + x[256 + row], E = acc_E + x[384 + row];
        t.Dv[row_off + gidx] = Dv;
        t.dot2[row_off + gidx] = d2;
        t.dot3[row_off + gidx] = A - 2.f * Dv * d2 + E;
      }
    } else {
      // outputs: [128 x D] fp32 accumulators in tensor memory -> scaled, rounded, stored
      if (n_iter > 0 && ok) ok = mbar_wait(bar_acc_done, 0, abort_flag, t.status, wait_code(KIND, 8));
      ok = __all_sync(0xffffffffu, ok);
      tc_fence_after_sync();
      constexpr int kColsPerHalf = D / 2;
      const int n_rows = TR::kCol ? g.N_kv : g.N_q;
#pragma unroll
      for (int o = 0; o < TR::kNOut; ++o) {
        T* dst;
        float mul = 1.f;
        if constexpr (KIND == FWD_OUT) dst = (T*)t.out_O;
        else if constexpr (KIND == BWD_ROW) { dst = (T*)t.out_dQ; mul = g.scale; }
        else if constexpr (KIND == BWD_COL) { dst = (T*)(o == 0 ? t.out_dV : t.out_dK); mul = (o == 0) ? 1.f : g.scale; }
        else if constexpr (KIND == HVP_ROW) { dst = (T*)(o == 0 ? t.out_g_Q : t.out_g_dO); mul = (o == 0) ? g.scale : 1.f; }
        else { dst = (T*)(o == 0 ? t.out_g_K : t.out_g_V); mul = (o == 0) ? g.scale : 1.f; }
        T* prow = dst + ((size_t)bh * n_rows + gidx) * D + half * kColsPerHalf;
#pragma unroll
        for (int ch = 0; ch < kColsPerHalf / 16; ++ch) {
          uint32_t v[16];
          if (n_iter > 0 && ok) {
            tmem_ld16(lane_addr + TR::kOutCol0 + o * D + half * kColsPerHalf + ch * 16, v);
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
  }

  // teardown: every role arrives here, also after an abort
  tc_fence_before_sync();
  __syncthreads();
  if (warp == kMmaWarp) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

// ---------------------------------------------------------------------------
// D_i = sum_d dO * O  (one warp per query row), used by the first backward.
// Reference: csrc/flash_double_backward_v7.cu:721-739.
// ---------------------------------------------------------------------------
template <typename T>
__global__ void rowdot_kernel(const T* __restrict__ a, const T* __restrict__ b, float* __restrict__ out,
                              long long rows, int D) {
  const long long r = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (r >= rows) return;
  const int lane = threadIdx.x & 31;
  float acc = 0.f;
  for (int d = lane * 2; d < D; d += 64) {
    acc += Elem<T>::to_float(a[r * D + d]) * Elem<T>::to_float(b[r * D + d]);
    acc += Elem<T>::to_float(a[r * D + d + 1]) * Elem<T>::to_float(b[r * D + d + 1]);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if (lane == 0) out[r] = acc;
}

// ---------------------------------------------------------------------------
// primitive self-test: C[128 x N] = A[128 x K] * B, one CTA
// ---------------------------------------------------------------------------
struct SelftestMaps { CUtensorMap a, b; };

template <typename T>
__global__ void __launch_bounds__(128, 1)
selftest_gemm_kernel(const __grid_constant__ SelftestMaps maps, const T* __restrict__ A_gmem, float* __restrict__ C,
                     int N, int K, int flags, unsigned int* status) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* gen = smem_raw + (base - smem_u32(smem_raw));
  const uint32_t a_base = base;                 // K/64 atoms x [128][64]
  const uint32_t b_base = base + 2 * 16384;     // up to 32 KB
  Control* ctl = reinterpret_cast<Control*>(gen + 4 * 16384);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const bool b_mn = (flags & 1) != 0, a_manual = (flags & 2) != 0, a_tmem = (flags & 4) != 0;
  const uint32_t bar_full = smem_u32(&ctl->stat_full), bar_done = smem_u32(&ctl->acc_done);
  if (threadIdx.x == 0) {
    mbar_init(bar_full, 1);
    mbar_init(bar_done, 1);
    ctl->abort_flag = 0u;
    fence_barrier_init();
    fence_proxy_async_smem();
  }
  __syncthreads();
  if (warp == 0) tmem_alloc(smem_u32(&ctl->tmem_base), 256);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = ctl->tmem_base;
  volatile uint32_t* abort_flag = &ctl->abort_flag;

  if (a_tmem) {
    // every thread stores its own row of A into tensor memory, two halves per 32-bit column,
    // starting at column 128
    const int row = threadIdx.x;
    for (int w0 = 0; w0 < K / 2; w0 += 8) {
      uint32_t v[8];
      const uint4 x0 = *reinterpret_cast<const uint4*>(A_gmem + (size_t)row * K + 2 * w0);
      const uint4 x1 = *reinterpret_cast<const uint4*>(A_gmem + (size_t)row * K + 2 * w0 + 8);
      v[0] = x0.x; v[1] = x0.y; v[2] = x0.z; v[3] = x0.w; v[4] = x1.x; v[5] = x1.y; v[6] = x1.z; v[7] = x1.w;
      tmem_st8(tmem_base + ((uint32_t)(warp * 32) << 16) + 128 + w0, v);
    }
    tmem_st_wait();
    tc_fence_before_sync();
  } else if (a_manual) {
    // every thread writes its own row of A with the software swizzle
    const int row = threadIdx.x;
    for (int c = 0; c < K; c += 8) {
      const uint4 v = *reinterpret_cast<const uint4*>(A_gmem + (size_t)row * K + c);
      const uint32_t addr = a_base + (c >> 6) * 16384 + sw128_offset(row, c & 63);
      asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
    }
    fence_proxy_async_smem();
  }
  __syncthreads();

  const int ka = K / 64;
  if (threadIdx.x == 0) {
    uint32_t bytes = 0;
    const bool a_tma = !a_manual && !a_tmem;
    if (a_tma) bytes += 128 * K * 2;
    bytes += N * K * 2;
    mbar_arrive_expect_tx(bar_full, bytes);
    if (a_tma)
      for (int a = 0; a < ka; ++a)
        for (int h = 0; h < 2; ++h) tma_load_3d(a_base + a * 16384 + h * 8192, &maps.a, a * 64, h * 64, 0, bar_full);
    if (!b_mn) {
      // B given as [N][K]: K/64 atoms, each [N rows][128 bytes]
      for (int a = 0; a < ka; ++a)
        for (int h = 0; h < N / 64; ++h)
          tma_load_3d(b_base + a * (N * 128) + h * 8192, &maps.b, a * 64, h * 64, 0, bar_full);
    } else {
      // B given as [K][N]: N/64 atoms, each [K rows][128 bytes]
      for (int a = 0; a < N / 64; ++a)
        for (int h = 0; h < ka; ++h)
          tma_load_3d(b_base + a * (K * 128) + h * 8192, &maps.b, a * 64, h * 64, 0, bar_full);
    }
    if (mbar_wait(bar_full, 0, abort_flag, status, 0x7001u)) {
      tc_fence_after_sync();
      const uint32_t idesc = make_idesc(128, N, Pack<T>::kIsBf16, 0, b_mn ? 1 : 0);
      for (int ks = 0; ks < K / 16; ++ks) {
        const uint64_t ad = smem_desc_sw128(a_base + (ks >> 2) * 16384 + (ks & 3) * 32, 16, 1024);
        uint64_t bd;
        if (!b_mn) bd = smem_desc_sw128(b_base + (ks >> 2) * (N * 128) + (ks & 3) * 32, 16, 1024);
        else bd = smem_desc_sw128(b_base + ks * 2048, K * 128, 1024);
        if (a_tmem) mma_ts(tmem_base, tmem_base + 128 + ks * 8, bd, idesc, ks > 0);
        else mma_ss(tmem_base, ad, bd, idesc, ks > 0);
      }
      mma_commit(bar_done);
    }
  }
  __syncwarp();
  const bool ok = mbar_wait(bar_done, 0, abort_flag, status, 0x7002u);
  tc_fence_after_sync();
  if (ok) {
    const int row = warp * 32 + lane;
    for (int c = 0; c < N; c += 16) {
      uint32_t v[16];
      tmem_ld16(tmem_base + ((uint32_t)(warp * 32) << 16) + c, v);
      tmem_ld_wait(v);
      for (int e = 0; e < 16; ++e) C[(size_t)row * N + c + e] = __uint_as_float(v[e]);
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 256);
  }
}

// ---------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

// [planes][rows][cols] half-precision tensor, box = 64 cols x 64 rows x 1 plane, 128-byte swizzle.
static thread_local char tl_encode_error[160] = "";

static bool encode_map(CUtensorMap* map, const void* ptr, int is_bf16, long long planes, long long rows,
                       long long cols) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) {
    snprintf(tl_encode_error, sizeof(tl_encode_error), "driver entry point cuTensorMapEncodeTiled not found");
    return false;
  }
  cuuint64_t dims[3] = {(cuuint64_t)cols, (cuuint64_t)rows, (cuuint64_t)planes};
  cuuint64_t strides[2] = {(cuuint64_t)cols * 2, (cuuint64_t)rows * (cuuint64_t)cols * 2};
  cuuint32_t box[3] = {64, 64, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(map, is_bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3,
                  const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    snprintf(tl_encode_error, sizeof(tl_encode_error),
             "cuTensorMapEncodeTiled returned %d for ptr=%p dims=[%lld,%lld,%lld]", (int)r, ptr, planes, rows, cols);
  return r == CUDA_SUCCESS;
}

bool encode_all_maps(TmaMaps* maps, const Geometry& g, const Tensors& t, int is_bf16, const char** err) {
  memset(maps, 0, sizeof(*maps));
  const void* ptrs[T_COUNT] = {t.Q, t.K, t.V, t.dO, t.g_dQ, t.g_dK, t.g_dV};
  const int rows[T_COUNT] = {g.N_q, g.N_kv, g.N_kv, g.N_q, g.N_q, g.N_kv, g.N_kv};
  for (int i = 0; i < T_COUNT; ++i) {
    const void* p = ptrs[i] ? ptrs[i] : t.Q;   // unused maps still need a valid encoding
    const int r = ptrs[i] ? rows[i] : g.N_q;
    if (!encode_map(&maps->m[i], p, is_bf16, g.BH, r, g.D)) {
      *err = tl_encode_error;
      return false;
    }
  }
  return true;
}

cudaError_t launch_hvp_col(int D, int is_bf16, const TmaMaps& maps, const Geometry& g, const Tensors& t,
                           cudaStream_t s);
cudaError_t launch_hvp_row(int mode, int D, int is_bf16, const TmaMaps& maps, const Geometry& g,
                           const Tensors& t, cudaStream_t s);

template <int KIND, int D, typename T>
static cudaError_t launch_kind(const TmaMaps& maps, const Geometry& g_in, const Tensors& t, cudaStream_t s) {
  using TR = Traits<KIND, D>;
  Geometry g = g_in;
  const int n_stat = TR::kCol ? g.N_kv : g.N_q;
  const long long ctas = (long long)g.BH * ((n_stat + BM - 1) / BM);
  if (ctas <= 0) return cudaSuccess;
  if (ctas > 0x7fffffffLL) return cudaErrorInvalidValue;
  // Few waves: order CTAs heaviest-tile-first across all heads so the tail is made of light
  // tiles.  Many waves: keep the CTAs of one head adjacent so its K/V tiles stay in L2.
  g.tile_major = ctas < 8 * 148 ? 1 : 0;
  // at least 120 KB of shared memory per CTA keeps one CTA per SM, so the
  // 512-column tensor-memory allocation can never wait for a co-resident CTA
  const size_t smem = TR::kSmemBytes < 122880u ? 122880u : TR::kSmemBytes;
  auto kern = attn_tc_kernel<KIND, D, T>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return e;
  kern<<<(unsigned)ctas, kThreads, smem, s>>>(maps, g, t);
  return cudaGetLastError();
}

template <int D, typename T>
static cudaError_t launch_op(int op, const TmaMaps& maps, const Geometry& g, const Tensors& t, cudaStream_t s,
                             int* n, int phases) {
  cudaError_t e = cudaSuccess;
  *n = 0;
  if (op == OP_FORWARD) {
    e = launch_kind<FWD_LSE, D, T>(maps, g, t, s);
    Tensors t2 = t;
    t2.L = t.out_L;
    if (e == cudaSuccess) e = launch_kind<FWD_OUT, D, T>(maps, g, t2, s);
    *n = 2;
  } else if (op == OP_BACKWARD) {
    const long long rows = (long long)g.BH * g.N_q;
    if (rows > 0) {
      rowdot_kernel<T><<<(unsigned)((rows + 7) / 8), 256, 0, s>>>((const T*)t.dO, (const T*)t.O, t.Dv, rows, g.D);
      e = cudaGetLastError();
    }
    if (e == cudaSuccess) e = launch_kind<BWD_ROW, D, T>(maps, g, t, s);
    if (e == cudaSuccess) e = launch_kind<BWD_COL, D, T>(maps, g, t, s);
    *n = 3;
  } else {
    if (phases & HVP_PHASE_PRE) { e = launch_hvp_row(0, D, Pack<T>::kIsBf16, maps, g, t, s); ++*n; }   // scalars + g_dO
    if (e == cudaSuccess && (phases & HVP_PHASE_ROW)) { e = launch_hvp_row(1, D, Pack<T>::kIsBf16, maps, g, t, s); ++*n; }  // g_Q
    if (e == cudaSuccess && (phases & HVP_PHASE_COL)) { e = launch_hvp_col(D, Pack<T>::kIsBf16, maps, g, t, s); ++*n; }     // g_K, g_V
  }
  return e;
}

}  // namespace tc

bool tc_supported(int dtype, int D) { return (dtype == 0 || dtype == 1) && (D == 64 || D == 128); }

cudaError_t launch_tc(int op, int dtype, const Geometry& g, const Tensors& t, cudaStream_t s, int* launches,
                      const char** err, int phases) {
  using namespace tc;
  *err = nullptr;
  TmaMaps maps;
  const int bf = dtype == 1;
  if (!encode_all_maps(&maps, g, t, bf, err)) return cudaErrorInvalidValue;
  if (g.D == 64) {
    return bf ? launch_op<64, __nv_bfloat16>(op, maps, g, t, s, launches, phases)
              : launch_op<64, __half>(op, maps, g, t, s, launches, phases);
  }
  return bf ? launch_op<128, __nv_bfloat16>(op, maps, g, t, s, launches, phases)
            : launch_op<128, __half>(op, maps, g, t, s, launches, phases);
}

cudaError_t launch_tc_selftest(const void* A, const void* B, float* C, int N, int K, int dtype, int flags,
                               unsigned int* status, cudaStream_t s, const char** err) {
  using namespace tc;
  *err = nullptr;
  SelftestMaps maps;
  memset(&maps, 0, sizeof(maps));
  const int bf = dtype == 1;
  const bool b_mn = (flags & 1) != 0;
  if (!encode_map(&maps.a, A, bf, 1, 128, K) ||
      !encode_map(&maps.b, B, bf, 1, b_mn ? K : N, b_mn ? N : K)) {
    *err = tl_encode_error;
    return cudaErrorInvalidValue;
  }
  const size_t smem = 4 * 16384 + 1024 + 1024;
  cudaError_t e;
  if (bf) {
    e = cudaFuncSetAttribute(selftest_gemm_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    selftest_gemm_kernel<__nv_bfloat16><<<1, 128, smem, s>>>(maps, (const __nv_bfloat16*)A, C, N, K, flags, status);
  } else {
    e = cudaFuncSetAttribute(selftest_gemm_kernel<__half>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    selftest_gemm_kernel<__half><<<1, 128, smem, s>>>(maps, (const __half*)A, C, N, K, flags, status);
  }
  return cudaGetLastError();
}

}  // namespace attn
