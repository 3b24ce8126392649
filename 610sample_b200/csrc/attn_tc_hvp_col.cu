// Column side of the double backward (Hessian-vector product) on sm_100a: g_K and g_V,
// given the per-row scalars Dv, dot2, dot3 of the row-side pre-pass.
//
// A CTA owns 128 key rows (stationary K, V, g_dK, g_dV in shared memory) and streams 64-row
// query tiles (Q, g_dQ, dO; two TMA stages at D = 128, six at D = 64).  Scores are computed TRANSPOSED (keys on the
// tensor-memory lanes), so the operand roles are those of the row kernels.
// Tensor memory (512 columns):
//     RA [  0,128) = [ S^T | gdS^T ] = K [Q; g_dQ]^T (one N = 128 product), gdS^T += g_dK Q^T
//     RB [128,256) = [ dP^T | gPdV^T ] = V dO^T, g_dV dO^T
//     OUT0 [256,256+D) = g_K += dS^T g_dQ + g_S^T Q        OUT1 [256+D,256+2D) = g_V += g_dp^T dO
// Per tile the math warps run two half-steps.  Half-step 1 reads RA, releases it at once and
// keeps p = exp(S - L) and a = gdS - dot2 in registers.  Half-step 2 reads RB and writes the
// half-precision operands dS = p (dP - Dv), g_dp = p a and g_S = p (a (dP - Dv) + gPdV - c3),
// c3 = dot2 Dv + dot3, over the RB columns the thread has just read; the output products take
// them from there (A operand in tensor memory), so no operand tile goes through shared memory
// and the two column halves of a row never race.  The per-query scalars (L, Dv, dot2, c3) of a
// streamed tile are fetched by the math warps one tile ahead and handed over in shared memory.
// Two warps issue the MMAs, each batch by one elected lane inside a single branch: the first warp
// the RA products of every tile (they need only Q and g_dQ, which land on their own barrier), the
// second the output products of a tile -- in two halves, the even k-steps as soon as their
// operands are written -- followed by the RB products of the next tile, so RB is overwritten only
// after the outputs that read it.  Shared memory holds 128 KB of stationary operands, so there is
// room for two stream stages only: the load of tile j+2 starts when the outputs of tile j have
// completed, and that latency is what the tensor pipe idles on in this kernel.
// The two result tiles leave through shared memory and TMA stores.
// Formulas: reference csrc/flash_double_backward_v7.cu:1583-1675.
#include "attn_launch.h"
#include "tc_common.cuh"

namespace attn {
namespace tc {

constexpr int kColMmaWarp = 9;
constexpr int kColMaxStages = 6;

constexpr int kColThreads = 352;    // 8 math warps, TMA producer, two MMA issuers

struct ColControl {   // lives in the first 256 bytes of the aux area
  uint64_t stat_full;
  uint64_t stream_full[kColMaxStages];     // Q and g_dQ of a streamed tile have landed
  uint64_t stream_full_do[kColMaxStages];  // its dO has landed
  uint64_t stream_empty[kColMaxStages];
  uint64_t ra_full, ra_free;
  uint64_t rb_full;
  uint64_t op_half;            // operands of the even k-steps (first 16 queries of each half) written
  uint64_t op_full;
  uint64_t acc_done;
  uint64_t stats_ready[2];
  uint32_t tmem_base;
  volatile uint32_t abort_flag;
};

static_assert(sizeof(ColControl) <= 256, "control block larger than its slot");

template <int D>
struct ColCfg {
  static constexpr int kAtoms = D / 64;
  static constexpr int kNStat = 4;      // K, V, g_dK, g_dV
  static constexpr int kNStream = 3;    // Q, g_dQ (back to back), dO
  static constexpr uint32_t kStatBytes = kNStat * kAtoms * kAtomBytesStat;
  static constexpr uint32_t kStageBytes = kNStream * kAtoms * kAtomBytesStrm;
  static constexpr uint32_t kAuxBytes = 256 + 2048;   // control block + [2][4][64] per-query scalars
  // 128 KB of stationary operands leave room for two 48 KB stages at D = 128; at D = 64 both halve
  // and six stages fit, which covers the latency of a TMA load (about 2 000 clocks)
  static constexpr int kStages = (D == 64) ? 6 : 2;
  static_assert(kStages <= kColMaxStages, "control block too small");
  static constexpr uint32_t kContentBytes = kStatBytes + kStages * kStageBytes + kAuxBytes;
  static constexpr uint32_t kMaxSmem = 232448;
  static_assert(kContentBytes + 768 <= kMaxSmem, "shared memory over-subscribed");
  static constexpr uint32_t kSmemBytes = (kContentBytes + 1024 <= kMaxSmem) ? kContentBytes + 1024 : kMaxSmem;
  static constexpr int kRA = 0, kRB = 128, kOut0 = 256, kOut1 = 256 + D;
  static_assert(kOut1 + D <= kTmemCols, "tensor memory over-subscribed");
  __host__ __device__ static constexpr uint32_t stream_off(int slot, int atom) {
    if (slot < 2) return (uint32_t)atom * 2u * kAtomBytesStrm + (uint32_t)slot * kAtomBytesStrm;
    return 2u * kAtoms * kAtomBytesStrm + (uint32_t)atom * kAtomBytesStrm;
  }
  __host__ __device__ static constexpr uint32_t stream_atom_stride(int slot) {
    return slot < 2 ? 2u * kAtomBytesStrm : kAtomBytesStrm;
  }
  __host__ __device__ static constexpr int stat_tensor(int slot) {
    return slot == 0 ? T_K : slot == 1 ? T_V : slot == 2 ? T_gK : T_gV;
  }
  __host__ __device__ static constexpr int stream_tensor(int slot) { return slot == 0 ? T_Q : slot == 1 ? T_gQ : T_dO; }
};

template <int D, typename T>
__global__ void __launch_bounds__(kColThreads, 1)
hvp_col_kernel(const __grid_constant__ TmaMaps maps, const Geometry g, const Tensors t) {
  using CF = ColCfg<D>;
  constexpr int KIND = HVP_COL;
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
  ColControl* ctl = reinterpret_cast<ColControl*>(smem_gen + aux_off);
  float* col_stats = reinterpret_cast<float*>(smem_gen + aux_off + 256);   // [2][4][64]

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tiles = (g.N_kv + BM - 1) / BM;
  int bh, tile;   // early key tiles are the heavy ones
  cta_to_head_and_rank(g, tiles, bh, tile);
  const int r0 = tile * BM;

  int lo, hi;
  query_range_for_keys(g, r0, r0 + BM, lo, hi);
  const int t_begin = lo / BN;
  const int n_iter = (hi > lo) ? ((hi + BN - 1) / BN - t_begin) : 0;

  const uint32_t bar_stat_full = smem_u32(&ctl->stat_full);
  const uint32_t bar_ra_full = smem_u32(&ctl->ra_full), bar_ra_free = smem_u32(&ctl->ra_free);
  const uint32_t bar_rb_full = smem_u32(&ctl->rb_full);
  const uint32_t bar_op_full = smem_u32(&ctl->op_full), bar_acc_done = smem_u32(&ctl->acc_done);
  const uint32_t bar_op_half = smem_u32(&ctl->op_half);
  auto bar_stream_full = [&](int s) { return smem_u32(&ctl->stream_full[s]); };
  auto bar_stream_full_do = [&](int s) { return smem_u32(&ctl->stream_full_do[s]); };
  auto bar_stream_empty = [&](int s) { return smem_u32(&ctl->stream_empty[s]); };

  if (threadIdx.x == 0) {
    mbar_init(bar_stat_full, 1);
    for (int s = 0; s < CF::kStages; ++s) {
      mbar_init(bar_stream_full(s), 1);
      mbar_init(bar_stream_full_do(s), 1);
      mbar_init(bar_stream_empty(s), 1);
    }
    for (int s = 0; s < 2; ++s) mbar_init(smem_u32(&ctl->stats_ready[s]), kMathWarps);
    mbar_init(bar_ra_full, 1);
    mbar_init(bar_ra_free, kMathWarps);
    mbar_init(bar_rb_full, 1);
    mbar_init(bar_op_full, kMathWarps);
    mbar_init(bar_op_half, kMathWarps);
    mbar_init(bar_acc_done, 1);
    ctl->abort_flag = 0u;
    ctl->tmem_base = 0u;
    fence_barrier_init();
    fence_proxy_async_smem();
  }
  __syncthreads();
  // the stationary tiles and the first streamed tile are requested before the tensor-memory
  // allocation and the second barrier: their latency is the longest item of the prologue
  if (warp == kProducerWarp && lane == 0 && n_iter > 0) {
    mbar_arrive_expect_tx(bar_stat_full, CF::kStatBytes);
    mbar_arrive_expect_tx(bar_stream_full(0), 2 * kAtoms * kAtomBytesStrm);
    mbar_arrive_expect_tx(bar_stream_full_do(0), kAtoms * kAtomBytesStrm);
#pragma unroll
    for (int s = 0; s < CF::kNStat; ++s) {
#pragma unroll
      for (int a = 0; a < kAtoms; ++a)
#pragma unroll
        for (int h = 0; h < 2; ++h)
          tma_load_3d(stat_base + (s * kAtoms + a) * kAtomBytesStat + h * kAtomBytesStrm,
                      &maps.m[CF::stat_tensor(s)], a * 64, r0 + h * 64, bh, bar_stat_full);
      if (s == 0) {     // the first product needs K and the streamed tile
#pragma unroll
        for (int sl = 0; sl < CF::kNStream; ++sl)
#pragma unroll
          for (int a = 0; a < kAtoms; ++a)
            tma_load_3d(strm_base + CF::stream_off(sl, a), &maps.m[CF::stream_tensor(sl)], a * 64, t_begin * BN, bh,
                        sl < 2 ? bar_stream_full(0) : bar_stream_full_do(0));
      }
    }
  }
  if (warp == kColMmaWarp) tmem_alloc(smem_u32(&ctl->tmem_base), kTmemCols);
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
      for (int it = 1; it < n_iter; ++it) {     // tile 0 was requested above
        const int st = it % CF::kStages;
        ok = mbar_wait(bar_stream_empty(st), ((it / CF::kStages) & 1) ^ 1, abort_flag, t.status, wait_code(KIND, 1));
        if (!ok) break;
        // Q and g_dQ first, on their own barrier: the RA products of the tile need only them
        mbar_arrive_expect_tx(bar_stream_full(st), 2 * kAtoms * kAtomBytesStrm);
        mbar_arrive_expect_tx(bar_stream_full_do(st), kAtoms * kAtomBytesStrm);
        const uint32_t stage = strm_base + st * CF::kStageBytes;
#pragma unroll
        for (int s = 0; s < CF::kNStream; ++s)
#pragma unroll
          for (int a = 0; a < kAtoms; ++a)
            tma_load_3d(stage + CF::stream_off(s, a), &maps.m[CF::stream_tensor(s)], a * 64,
                        (t_begin + it) * BN, bh, s < 2 ? bar_stream_full(st) : bar_stream_full_do(st));
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
  else if (warp == kColMmaWarp || warp == kColMmaWarp + 1) {
    if (n_iter > 0) {
      bool ok = mbar_wait(bar_stat_full, 0, abort_flag, t.status, wait_code(KIND, 2));
      ok = __all_sync(0xffffffffu, ok);
      const uint64_t d_stat = smem_desc_sw128(stat_base, 16, 1024);
      auto stat_desc = [&](int slot, int ks) {   // K-major A from shared memory
        return d_stat + (uint64_t)(((slot * kAtoms + (ks >> 2)) * kAtomBytesStat + (ks & 3) * 32) >> 4);
      };
      // descriptor offsets (16-byte units) within a stage: K-major B, k-step ks of slot; MN-major B,
      // 16 rows per k-step
      auto koff = [](int slot, int ks) { return (uint64_t)((CF::stream_off(slot, ks >> 2) + (ks & 3) * 32) >> 4); };
      auto moff = [](int slot, int ks) { return (uint64_t)((CF::stream_off(slot, 0) + ks * 2048) >> 4); };
      // operand written by the math warps over RB: the 16 elements of k-step ks sit in 8
      // columns at col0 + 32*(ks/2) + 8*(ks%2) (owner half, then chunk)
      auto op_tmem = [&](int col0, int ks) { return tmem_base + (uint32_t)(col0 + 32 * (ks >> 1) + 8 * (ks & 1)); };
      auto commit = [&](uint32_t bar) { if (elect_one()) mma_commit(bar); };
      constexpr int KS = D / 16, KO = BN / 16;
      // a head dimension below the tile width: skip the k-steps and output columns that are padding
      const int ks_n = g.D >> 4;
      const uint32_t idesc_out = make_idesc(BM, g.D, Pack<T>::kIsBf16, 0, 1);
      const uint32_t ra = tmem_base + CF::kRA, rb = tmem_base + CF::kRB;
      const uint32_t out0 = tmem_base + CF::kOut0, out1 = tmem_base + CF::kOut1;

      // Every batch of products is issued by the elected lane inside one branch, with the
      // descriptor of the stage built once: the instruction stream between two MMAs is an add.
      // The last kTail k-steps of a score batch are issued after the wait that follows the batch
      // in program order: the wait's latency then falls while the tensor pipe still has work queued.
      constexpr int kTail = (D == 128) ? 2 : 0;
      auto issue_ra_head = [&](uint32_t stage) {
        const uint64_t dk = smem_desc_sw128(stage, 16, 1024);
        if (elect_one()) {
          _Pragma("unroll") for (int ks = 0; ks < KS; ++ks)   // [S^T | K g_dQ^T] = K [Q; g_dQ]^T
            if (ks < ks_n) mma_ss(ra, stat_desc(0, ks), dk + koff(0, ks), kIdesc128, ks > 0);
          _Pragma("unroll") for (int ks = 0; ks < KS - kTail; ++ks)   // gdS^T += g_dK Q^T
            if (ks < ks_n) mma_ss(ra + 64, stat_desc(2, ks), dk + koff(0, ks), kIdesc64, 1);
        }
        __syncwarp();
      };
      auto issue_ra_tail = [&](uint32_t stage) {      // ends with the commit of the whole batch
        const uint64_t dk = smem_desc_sw128(stage, 16, 1024);
        if (elect_one()) {
          _Pragma("unroll") for (int ks = KS - kTail; ks < KS; ++ks)
            if (ks < ks_n) mma_ss(ra + 64, stat_desc(2, ks), dk + koff(0, ks), kIdesc64, 1);
          mma_commit(bar_ra_full);
        }
        __syncwarp();
      };
      auto issue_rb_head = [&](uint32_t stage) {
        const uint64_t dk = smem_desc_sw128(stage, 16, 1024);
        if (elect_one()) {
          _Pragma("unroll") for (int ks = 0; ks < KS; ++ks)   // dP^T = V dO^T
            if (ks < ks_n) mma_ss(rb, stat_desc(1, ks), dk + koff(2, ks), kIdesc64, ks > 0);
          _Pragma("unroll") for (int ks = 0; ks < KS - kTail; ++ks)   // gPdV^T = g_dV dO^T
            if (ks < ks_n) mma_ss(rb + 64, stat_desc(3, ks), dk + koff(2, ks), kIdesc64, ks > 0);
        }
        __syncwarp();
      };
      auto issue_rb_tail = [&](uint32_t stage) {      // ends with the commit of the whole batch
        const uint64_t dk = smem_desc_sw128(stage, 16, 1024);
        if (elect_one()) {
          _Pragma("unroll") for (int ks = KS - kTail; ks < KS; ++ks)
            if (ks < ks_n) mma_ss(rb + 64, stat_desc(3, ks), dk + koff(2, ks), kIdesc64, ks > 0);
          mma_commit(bar_rb_full);
        }
        __syncwarp();
      };
      // The output products of one tile in two parts: the k-steps of parity `par` (the math warps
      // write the operands of the even k-steps first and announce them on their own barrier).
      // Operands: dS^T at RB, g_dp^T at RB+16, g_S^T at RB+64.
      auto issue_out = [&](uint32_t stage, bool first, int par) {
        // the atoms of Q and g_dQ are interleaved, those of dO follow one another
        const uint64_t dm01 = smem_desc_sw128(stage, CF::stream_atom_stride(0), 1024);
        const uint64_t dm2 = smem_desc_sw128(stage, CF::stream_atom_stride(2), 1024);
        static_assert(CF::stream_atom_stride(0) == CF::stream_atom_stride(1), "Q and g_dQ share a layout");
        if (elect_one()) {
          _Pragma("unroll") for (int ks = 0; ks < KO; ++ks)   // g_K += dS^T g_dQ
            if ((ks & 1) == par) mma_ts(out0, op_tmem(CF::kRB, ks), dm01 + moff(1, ks), idesc_out, !(first && ks == 0));
          _Pragma("unroll") for (int ks = 0; ks < KO; ++ks)   // g_K += g_S^T Q
            if ((ks & 1) == par) mma_ts(out0, op_tmem(CF::kRB + 64, ks), dm01 + moff(0, ks), idesc_out, 1);
          _Pragma("unroll") for (int ks = 0; ks < KO; ++ks)   // g_V += g_dp^T dO
            if ((ks & 1) == par) mma_ts(out1, op_tmem(CF::kRB + 16, ks), dm2 + moff(2, ks), idesc_out, !(first && ks == 0));
        }
        __syncwarp();
      };

      // Two issuing warps, so that the latency of one warp's waits falls while the products of the
      // other are queued.  The tensor pipe needs no order between the two streams: RA(j+1) only
      // waits for RA(j) to have been read, and RB(j+1) follows OUT(j), which reads RB, in the
      // second warp's own order.
      auto wait_stream = [&](int tile) {       // Q and g_dQ of the tile
        return mbar_wait(bar_stream_full(tile % CF::kStages), (tile / CF::kStages) & 1, abort_flag, t.status, wait_code(KIND, 3));
      };
      auto wait_stream_do = [&](int tile) {    // dO of the tile
        return mbar_wait(bar_stream_full_do(tile % CF::kStages), (tile / CF::kStages) & 1, abort_flag, t.status, wait_code(KIND, 13));
      };
      if (warp == kColMmaWarp) {
        // ---- first warp: the RA products of every tile
        for (int j = 0; j < n_iter && ok; ++j) {
          ok = wait_stream(j);
          if (ok && j > 0) ok = mbar_wait(bar_ra_free, (j - 1) & 1, abort_flag, t.status, wait_code(KIND, 4));
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
          tc_fence_after_sync();
          const uint32_t stage = strm_base + (j % CF::kStages) * CF::kStageBytes;
          issue_ra_head(stage);
          issue_ra_tail(stage);
        }
      } else {
        // ---- second warp: RB products and outputs
        ok = ok && wait_stream_do(0);
        ok = __all_sync(0xffffffffu, ok);
        if (ok) {
          tc_fence_after_sync();
          issue_rb_head(strm_base); issue_rb_tail(strm_base);
        }
        for (int j = 0; j < n_iter && ok; ++j) {
          const int st = j % CF::kStages, nst = (j + 1) % CF::kStages;
          const bool more = j + 1 < n_iter;
          ok = mbar_wait(bar_op_half, j & 1, abort_flag, t.status, wait_code(KIND, 14));
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
          tc_fence_after_sync();
          issue_out(strm_base + st * CF::kStageBytes, j == 0, 0);
          ok = mbar_wait(bar_op_full, j & 1, abort_flag, t.status, wait_code(KIND, 5));
          if (ok && more) ok = wait_stream_do(j + 1);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
          tc_fence_after_sync();
          issue_out(strm_base + st * CF::kStageBytes, j == 0, 1);
          commit(bar_stream_empty(st));
          if (more) {
            const uint32_t nstage = strm_base + nst * CF::kStageBytes;
            issue_rb_head(nstage); issue_rb_tail(nstage);
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
    const int row = quarter * 32 + lane;       // key row within the tile == TMEM lane
    const int gidx = r0 + row;
    const uint32_t lane_addr = tmem_base + ((uint32_t)(quarter * 32) << 16);
    const size_t row_off = (size_t)bh * g.N_q;

    int vlo, vhi;                              // query rows that see this thread's key row
    query_range_for_keys(g, gidx, gidx + 1, vlo, vhi);
    if (gidx >= g.N_kv) { vlo = 0; vhi = 0; }
    const uint32_t vspan = (uint32_t)(vhi - vlo);
    const float2 sl2 = make_float2(g.scale_log2e, g.scale_log2e);
    const float2 sc2 = make_float2(g.scale, g.scale);
    const uint32_t ra = lane_addr + CF::kRA, rb = lane_addr + CF::kRB;

    float2 p_[16], a_[16];   // carried from half-step 1 to half-step 2
    bool ok = true;
    // Per-query scalars of a streamed tile, negated so that every use is a packed add / fma:
    // [-L*log2(e) | -dot2 | -Dv | -(dot2*Dv + dot3)] x 64 queries; beyond N_q: -inf, 0, 0, 0 (p = 0).
    // Thread (which, c) fetches one of them; the values of tile it+1 are fetched during tile it and
    // published at its end, so that neither the global loads nor the hand-over are waited for.
    const int which = threadIdx.x >> 6, qc = threadIdx.x & 63;
    // The loads are issued a tile ahead and their values are only touched when they are
    // published, so that their latency never stalls the warp.
    auto fetch_stat = [&](int tile_it) {
      const int qi = (t_begin + tile_it) * BN + qc;
      float3 raw = make_float3((which == 0) ? INFINITY : 0.f, 0.f, 0.f);   // beyond N_q: L = +inf (p = 0), the rest 0
      if (tile_it < n_iter && qi < g.N_q) {
        if (which == 0) raw.x = __ldg(t.L + row_off + qi);
        else if (which == 1) raw.x = __ldg(t.dot2 + row_off + qi);
        else if (which == 2) raw.x = __ldg(t.Dv + row_off + qi);
        else { raw.x = __ldg(t.dot2 + row_off + qi); raw.y = __ldg(t.Dv + row_off + qi); raw.z = __ldg(t.dot3 + row_off + qi); }
      }
      return raw;
    };
    auto publish_stat = [&](int tile_it, float3 raw) {
      const float v = (which == 0) ? -raw.x * kLog2e : (which == 3) ? -fmaf(raw.x, raw.y, raw.z) : -raw.x;
      col_stats[(tile_it & 1) * 256 + which * 64 + qc] = v;
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&ctl->stats_ready[tile_it & 1]));
    };
    if (n_iter > 0) publish_stat(0, fetch_stat(0));
    for (int it = 0; it < n_iter; ++it) {
      const int j0 = (t_begin + it) * BN;
      const float* cs = col_stats + (it & 1) * 256;
      const float3 next_stat = fetch_stat(it + 1);
      ok = mbar_wait(smem_u32(&ctl->stats_ready[it & 1]), (it >> 1) & 1, abort_flag, t.status, wait_code(KIND, 9));
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      const int first = j0 + half * 32;
      const bool masked = !(first >= vlo && first + 31 < vhi);

      // ---------------- half-step 1: RA -> p, a ----------------------------------
      ok = mbar_wait(bar_ra_full, it & 1, abort_flag, t.status, wait_code(KIND, 6));
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after_sync();
      {
        uint32_t s_[2][16], g_[2][16];
        tmem_ld16(ra + half * 32, s_[0]);
        tmem_ld16(ra + half * 32 + 16, s_[1]);
        tmem_ld16(ra + 64 + half * 32, g_[0]);
        tmem_ld16(ra + 64 + half * 32 + 16, g_[1]);
        tmem_ld_wait(s_[0]);
        tmem_ld_wait(s_[1]);
        tmem_ld_wait(g_[0]);
        tmem_ld_wait(g_[1]);
        // the region may be overwritten by the next tile's products
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_ra_free);
#pragma unroll
        for (int ch = 0; ch < 2; ++ch)
#pragma unroll
          for (int e = 0; e < 16; e += 2) {
            const int cc = half * 32 + ch * 16 + e;
            const float2 nL2 = *reinterpret_cast<const float2*>(cs + cc);
            const float2 nD2 = *reinterpret_cast<const float2*>(cs + 64 + cc);
            const float2 x = __ffma2_rn(make_float2(__uint_as_float(s_[ch][e]), __uint_as_float(s_[ch][e + 1])), sl2, nL2);
            float2 pp = make_float2(ex2(x.x), ex2(x.y));
            if (masked) {
              pp.x = ((uint32_t)(j0 + cc - vlo) < vspan) ? pp.x : 0.f;
              pp.y = ((uint32_t)(j0 + cc + 1 - vlo) < vspan) ? pp.y : 0.f;
            }
            p_[ch * 8 + (e >> 1)] = pp;
            a_[ch * 8 + (e >> 1)] =
                __ffma2_rn(make_float2(__uint_as_float(g_[ch][e]), __uint_as_float(g_[ch][e + 1])), sc2, nD2);
          }
      }

      // ---------------- half-step 2: RB -> operands dS, g_dp, g_S ------------------
      ok = mbar_wait(bar_rb_full, it & 1, abort_flag, t.status, wait_code(KIND, 7));
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after_sync();
      {
        uint32_t dp_[2][16], gp_[2][16];
        tmem_ld16(rb + half * 32, dp_[0]);
        tmem_ld16(rb + half * 32 + 16, dp_[1]);
        tmem_ld16(rb + 64 + half * 32, gp_[0]);
        tmem_ld16(rb + 64 + half * 32 + 16, gp_[1]);
        tmem_ld_wait(dp_[0]);
        tmem_ld_wait(dp_[1]);
        tmem_ld_wait(gp_[0]);
        tmem_ld_wait(gp_[1]);
        // All of this thread's RB columns have been read; the operands go over them:
        // dS at [32h, 32h+16), g_dp at [32h+16, 32h+32), g_S at [64+32h, 64+32h+16).
#pragma unroll
        for (int ch = 0; ch < 2; ++ch) {
          uint32_t kds[8], kgdp[8], kgs[8];
#pragma unroll
          for (int e = 0; e < 16; e += 2) {
            const int cc = half * 32 + ch * 16 + e;
            const float2 nDv = *reinterpret_cast<const float2*>(cs + 128 + cc);
            const float2 nC3 = *reinterpret_cast<const float2*>(cs + 192 + cc);
            const float2 pp = p_[ch * 8 + (e >> 1)], aa = a_[ch * 8 + (e >> 1)];
            const float2 dpd = __fadd2_rn(make_float2(__uint_as_float(dp_[ch][e]), __uint_as_float(dp_[ch][e + 1])), nDv);
            const float2 ds = __fmul2_rn(pp, dpd);
            const float2 gdp = __fmul2_rn(pp, aa);
            const float2 tt = __fadd2_rn(make_float2(__uint_as_float(gp_[ch][e]), __uint_as_float(gp_[ch][e + 1])), nC3);
            const float2 gs = __fmul2_rn(pp, __ffma2_rn(aa, dpd, tt));
            kds[e >> 1] = Pack<T>::pack(ds.x, ds.y);
            kgdp[e >> 1] = Pack<T>::pack(gdp.x, gdp.y);
            kgs[e >> 1] = Pack<T>::pack(gs.x, gs.y);
          }
          tmem_st8(rb + half * 32 + ch * 8, kds);
          tmem_st8(rb + half * 32 + 16 + ch * 8, kgdp);
          tmem_st8(rb + 64 + half * 32 + ch * 8, kgs);
          if (ch == 0) {     // the even k-steps of the output products can start
            tmem_st_wait();
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_op_half);
          }
        }
      }
      tmem_st_wait();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_op_full);
      // every warp has finished the previous tile (its operands were consumed before this tile's
      // RB products were queued), so the other scalar buffer is free
      if (it + 1 < n_iter) publish_stat(it + 1, next_stat);
    }

    // ---------------- outputs --------------------------------------------------------
    if (n_iter > 0 && ok) ok = mbar_wait(bar_acc_done, 0, abort_flag, t.status, wait_code(KIND, 8));
    ok = __all_sync(0xffffffffu, ok);
    tc_fence_after_sync();
    constexpr int kColsPerHalf = D / 2;
    constexpr int kChunks = kColsPerHalf / 16;
    // Both result tiles go out through the shared memory of the stationary operands (every
    // product has completed): g_K over the K tile, g_V over the V tile.
#pragma unroll
    for (int o = 0; o < 2; ++o) {
      const float mul = (o == 0) ? g.scale : 1.f;
      const uint32_t tile = stat_base + (uint32_t)o * kAtoms * kAtomBytesStat;
      uint32_t v[kChunks][16];
#pragma unroll
      for (int ch = 0; ch < kChunks; ++ch) {
        if (n_iter > 0 && ok) {
          tmem_ld16(lane_addr + (o == 0 ? CF::kOut0 : CF::kOut1) + half * kColsPerHalf + ch * 16, v[ch]);
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
      for (int o = 0; o < 2; ++o)
        for (int a = 0; a * 64 < g.D; ++a)
          tma_store_3d(&maps.out[o == 0 ? TO_gK : TO_gV], stat_base + (uint32_t)(o * kAtoms + a) * kAtomBytesStat,
                       a * 64, r0, bh);
      bulk_commit_group();
      bulk_wait_group_read_all();
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == kColMmaWarp) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

template <int D, typename T>
static cudaError_t launch_col(const TmaMaps& maps, const Geometry& g_in, const Tensors& t, cudaStream_t s) {
  using CF = ColCfg<D>;
  Geometry g = g_in;
  const long long ctas = (long long)g.BH * ((g.N_kv + BM - 1) / BM);
  if (ctas <= 0) return cudaSuccess;
  if (ctas > 0x7fffffffLL) return cudaErrorInvalidValue;
  g.head_group = pick_head_group(ctas, g.BH, 3ll * g.N_q * g.D * 2);   // Q, g_dQ, dO
  // more than half of an SM's shared memory: one CTA per SM, so the 512-column
  // tensor-memory allocation never waits for a co-resident CTA
  const size_t smem = CF::kSmemBytes < 122880u ? 122880u : CF::kSmemBytes;
  auto kern = hvp_col_kernel<D, T>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return e;
  kern<<<(unsigned)ctas, kColThreads, smem, s>>>(maps, g, t);
  return cudaGetLastError();
}

cudaError_t launch_hvp_col(int D, int is_bf16, const TmaMaps& maps, const Geometry& g, const Tensors& t,
                           cudaStream_t s) {
  if (D <= 64) return is_bf16 ? launch_col<64, __nv_bfloat16>(maps, g, t, s) : launch_col<64, __half>(maps, g, t, s);
  return is_bf16 ? launch_col<128, __nv_bfloat16>(maps, g, t, s) : launch_col<128, __half>(maps, g, t, s);
}

}  // namespace tc
}  // namespace attn
