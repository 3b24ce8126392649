// Forward attention (O, L) on sm_100a in ONE pass: online softmax with the running maximum kept
// per row, O accumulated in tensor memory and rescaled there only when the maximum has grown by
// more than a threshold (f16/bf16, D a multiple of 16 up to 128).
//
// A CTA owns 128 query rows (Q copied once into TENSOR MEMORY) and streams 64-row tiles of K and V
// through a ring of TMA stages; the K half and the V half of a stage have their own barriers.
// Per tile:   S = Q K^T  (N = 64)   ->   P = exp2(S * s * log2 e - m)   ->   O += P V.
// Eight math warps form two groups of four; a thread owns one query row (= tensor-memory lane) and
// all 64 scores of a tile.  Group 0 takes the even tiles, group 1 the odd ones, and each group has
// its OWN running maximum m, running sum l and O accumulator, i.e. the keys are split in two
// interleaved streams that never have to agree on a maximum while the loop runs; the epilogue
// merges them: O = (O_0 2^(m_0 - m) + O_1 2^(m_1 - m)) / (l_0 2^(m_0 - m) + l_1 2^(m_1 - m)).
// Rescaling is lazy: m only moves when a tile's maximum exceeds it by more than kTau (in log2
// units), so P <= 2^kTau, and the O row is then multiplied in tensor memory by 2^(m_old - m_new)
// (a read-modify-write of the row by its owner thread, after the group's previous P V product has
// completed).  With inputs of ordinary scale that happens in the first tile or two of a row only.
// Tensor memory (512 columns): three score buffers S0, S1, S2 [0,192), Q [192,192+D/2),
// O_0 [256,256+D), O_1 [256+D, 256+2D).  P is written (two halves per 32-bit column) over the
// first 32 columns of the score buffer it was computed from and read from there as the A operand
// of P V.  Two warps issue the MMAs, each batch by one elected lane inside a single branch: one
// the score products (three tiles ahead: a buffer is free again once the P V product that read it
// has completed), the other the P V products.  Every wait is bounded.
// The reference computes the same in two passes with the maximum and sum first
// (csrc/flash_double_backward_v7.cu:380-530).
#include "attn_launch.h"
#include "tc_common.cuh"

namespace attn {
namespace tc {

constexpr int kFwdSWarp = 9;        // issues S = Q K^T
constexpr int kFwdPvWarp = 10;      // issues O += P V
constexpr int kFwdThreads = 352;    // 8 math warps, TMA producer, two MMA issuers
constexpr int kFwdMaxStages = 8;
constexpr int kFwdSBufs = 3;
constexpr float kTau = 8.f;         // log2 units: P <= 256
constexpr int KFWD = 20;            // kernel id inside device status codes

struct FwdControl {
  uint64_t staging_full;               // Q tile in the staging buffer
  uint64_t q_ready;                    // Q copied to tensor memory
  uint64_t stream_full[2][kFwdMaxStages];    // [0] K half, [1] V half
  uint64_t stream_empty[2][kFwdMaxStages];
  uint64_t s_full[kFwdSBufs];          // score product complete
  uint64_t p_full[kFwdSBufs];          // P written by the owning math group
  uint64_t pv_done[kFwdSBufs];         // the P V product that read the buffer has completed
  uint64_t acc_done;
  uint32_t tmem_base;
  volatile uint32_t abort_flag;
};

static_assert(sizeof(FwdControl) <= 512, "control block larger than its slot");

template <int D>
struct FwdCfg {
  static constexpr int kAtoms = D / 64;
  static constexpr uint32_t kStagingBytes = kAtoms * kAtomBytesStat;        // Q, later the O tile
  static constexpr uint32_t kStageBytes = 2 * kAtoms * kAtomBytesStrm;      // K then V
  static constexpr uint32_t kAuxBytes = 512 + 2 * 2 * BM * 4;               // control; (m, l) of both groups
  static constexpr uint32_t kMaxSmem = 232448;
  static constexpr int kFit = (int)((kMaxSmem - 1024 - kStagingBytes - kAuxBytes) / kStageBytes);
  static constexpr int kStages = kFit < kFwdMaxStages ? kFit : kFwdMaxStages;
  static_assert(kStages >= 4, "too few stream stages");
  static constexpr uint32_t kContentBytes = kStagingBytes + kStages * kStageBytes + kAuxBytes;
  static constexpr uint32_t kSmemBytes = kContentBytes + 1024;
  static constexpr int kS = 0, kQT = 192, kO = 256;       // O of group w at kO + w * D
  static_assert(kQT + D / 2 <= kO && kO + 2 * D <= kTmemCols, "tensor memory over-subscribed");
  __host__ __device__ static constexpr uint32_t stream_off(int slot, int atom) {   // slot 0 K, 1 V
    return (uint32_t)(slot * kAtoms + atom) * kAtomBytesStrm;
  }
};

template <int D, typename T>
__global__ void __launch_bounds__(kFwdThreads, 1)
fwd_kernel(const __grid_constant__ TmaMaps maps, const Geometry g, const Tensors t) {
  using CF = FwdCfg<D>;
  constexpr int kAtoms = CF::kAtoms;
  constexpr uint32_t kIdesc64 = make_idesc(BM, 64, Pack<T>::kIsBf16, 0, 0);

  extern __shared__ __align__(1024) uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  {
    uint32_t dyn_size;
    asm("mov.u32 %0, %%dynamic_smem_size;" : "=r"(dyn_size));
    if (smem_base - smem_u32(smem_raw) + CF::kContentBytes > dyn_size) {   // uniform over the CTA
      if (threadIdx.x == 0 && t.status != nullptr) atomicCAS(t.status, 0u, wait_code(KFWD, 15));
      return;
    }
  }
  const uint32_t staging = smem_base;
  const uint32_t strm_base = staging + CF::kStagingBytes;
  const uint32_t aux_off = CF::kStagingBytes + CF::kStages * CF::kStageBytes;
  FwdControl* ctl = reinterpret_cast<FwdControl*>(smem_gen + aux_off);
  float* ml = reinterpret_cast<float*>(smem_gen + aux_off + 512);   // [2 groups][m | l][128]

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

  const uint32_t bar_staging_full = smem_u32(&ctl->staging_full), bar_q_ready = smem_u32(&ctl->q_ready);
  const uint32_t bar_acc_done = smem_u32(&ctl->acc_done);
  auto bar_stream_full = [&](int h, int s) { return smem_u32(&ctl->stream_full[h][s]); };
  auto bar_stream_empty = [&](int h, int s) { return smem_u32(&ctl->stream_empty[h][s]); };
  auto bar_s_full = [&](int b) { return smem_u32(&ctl->s_full[b]); };
  auto bar_p_full = [&](int b) { return smem_u32(&ctl->p_full[b]); };
  auto bar_pv_done = [&](int b) { return smem_u32(&ctl->pv_done[b]); };

  if (threadIdx.x == 0) {
    mbar_init(bar_staging_full, 1);
    mbar_init(bar_q_ready, kMathWarps);
    for (int s = 0; s < CF::kStages; ++s)
      for (int h = 0; h < 2; ++h) {
        mbar_init(bar_stream_full(h, s), 1);
        mbar_init(bar_stream_empty(h, s), 1);
      }
    for (int b = 0; b < kFwdSBufs; ++b) {
      mbar_init(bar_s_full(b), 1);
      mbar_init(bar_p_full(b), kMathWarps / 2);
      mbar_init(bar_pv_done(b), 1);
    }
    mbar_init(bar_acc_done, 1);
    ctl->abort_flag = 0u;
    ctl->tmem_base = 0u;
    fence_barrier_init();
    fence_proxy_async_smem();
  }
  __syncthreads();

  // one half of the stage of tile `it`: K (h = 0) or V (h = 1)
  auto request_half = [&](int it, int h) {
    const int st = it % CF::kStages;
    const uint32_t stage = strm_base + st * CF::kStageBytes;
    mbar_arrive_expect_tx(bar_stream_full(h, st), CF::kStageBytes / 2);
#pragma unroll
    for (int a = 0; a < kAtoms; ++a)
      tma_load_3d(stage + CF::stream_off(h, a), &maps.m[h == 0 ? T_K : T_V], a * 64, (t_begin + it) * BN, bh,
                  bar_stream_full(h, st));
  };
  // Q and the first K tile are requested before the tensor-memory allocation and the second
  // barrier: their latency is the longest item of the prologue
  if (warp == kProducerWarp && lane == 0 && n_iter > 0) {
    tma_prefetch_desc(&maps.m[T_Q]); tma_prefetch_desc(&maps.m[T_K]); tma_prefetch_desc(&maps.m[T_V]);
    mbar_arrive_expect_tx(bar_staging_full, CF::kStagingBytes);
#pragma unroll
    for (int a = 0; a < kAtoms; ++a)
#pragma unroll
      for (int h = 0; h < 2; ++h)
        tma_load_3d(staging + a * kAtomBytesStat + h * kAtomBytesStrm, &maps.m[T_Q], a * 64, r0 + h * 64, bh, bar_staging_full);
    request_half(0, 0);
  }
  if (warp == kFwdSWarp) tmem_alloc(smem_u32(&ctl->tmem_base), kTmemCols);
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
      auto wait_free = [&](int it, int h) {
        if (it < CF::kStages) return true;
        return mbar_wait(bar_stream_empty(h, it % CF::kStages), ((it / CF::kStages) & 1) ^ 1, abort_flag, t.status, wait_code(KFWD, 1));
      };
      // K runs ahead of V by the three tiles the score products run ahead of the P V products
      for (int u = 1; u < kFwdSBufs && u < n_iter; ++u) request_half(u, 0);
      for (int u = 0; u < n_iter && ok; ++u) {
        ok = wait_free(u, 1);
        if (!ok) break;
        request_half(u, 1);
        if (u + kFwdSBufs < n_iter) {
          ok = wait_free(u + kFwdSBufs, 0);
          if (!ok) break;
          request_half(u + kFwdSBufs, 0);
        }
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
  else if (warp == kFwdSWarp || warp == kFwdPvWarp) {
    if (n_iter > 0) {
      constexpr int KS = D / 16, KO = BN / 16;
      const int ks_n = g.D >> 4;      // a head dimension below the tile width: skip the padding k-steps
      auto wait_stream = [&](int h, int tile_it) {
        bool w = mbar_wait(bar_stream_full(h, tile_it % CF::kStages), (tile_it / CF::kStages) & 1, abort_flag, t.status, wait_code(KFWD, 3));
        return (bool)__all_sync(0xffffffffu, w);
      };
      bool ok = true;
      if (warp == kFwdSWarp) {
        ok = mbar_wait(bar_q_ready, 0, abort_flag, t.status, wait_code(KFWD, 2));
        ok = __all_sync(0xffffffffu, ok);
        const uint32_t qt = tmem_base + CF::kQT;
        auto koff = [](int ks) { return (uint64_t)((CF::stream_off(0, ks >> 2) + (ks & 3) * 32) >> 4); };
        for (int j = 0; j < n_iter && ok; ++j) {
          const int b = j % kFwdSBufs, st = j % CF::kStages;
          ok = wait_stream(0, j);
          // the buffer was read (as P) by the P V product of tile j - 3
          if (ok && j >= kFwdSBufs) {
            ok = mbar_wait(bar_pv_done(b), ((j / kFwdSBufs) & 1) ^ 1, abort_flag, t.status, wait_code(KFWD, 4));
            ok = __all_sync(0xffffffffu, ok);
          }
          if (!ok) break;
          tc_fence_after_sync();
          const uint64_t dk = smem_desc_sw128(strm_base + st * CF::kStageBytes, 16, 1024);
          const uint32_t sbuf = tmem_base + CF::kS + 64u * (uint32_t)b;
          if (elect_one()) {
            _Pragma("unroll") for (int ks = 0; ks < KS; ++ks)
              if (ks < ks_n) mma_ts(sbuf, qt + 8 * ks, dk + koff(ks), kIdesc64, ks > 0);
            mma_commit(bar_s_full(b));
            mma_commit(bar_stream_empty(0, st));
          }
          __syncwarp();
        }
      } else {
        const uint32_t idesc_out = make_idesc(BM, g.D, Pack<T>::kIsBf16, 0, 1);
        auto moff = [](int ks) { return (uint64_t)((CF::stream_off(1, 0) + ks * 2048) >> 4); };
        for (int j = 0; j < n_iter && ok; ++j) {
          const int b = j % kFwdSBufs, st = j % CF::kStages, w = j & 1;
          ok = mbar_wait(bar_p_full(b), (j / kFwdSBufs) & 1, abort_flag, t.status, wait_code(KFWD, 5));
          ok = __all_sync(0xffffffffu, ok);
          if (ok) ok = wait_stream(1, j);
          if (!ok) break;
          tc_fence_after_sync();
          const uint64_t dm = smem_desc_sw128(strm_base + st * CF::kStageBytes, kAtomBytesStrm, 1024);
          const uint32_t acc = tmem_base + CF::kO + (uint32_t)(w * D);
          const uint32_t pbuf = tmem_base + CF::kS + 64u * (uint32_t)b;
          const bool first = j < 2;       // the first tile of either group overwrites its accumulator
          if (elect_one()) {
            _Pragma("unroll") for (int ks = 0; ks < KO; ++ks)
              mma_ts(acc, pbuf + 8 * ks, dm + moff(ks), idesc_out, !(first && ks == 0));
            mma_commit(bar_pv_done(b));
            mma_commit(bar_stream_empty(1, st));
            if (j + 1 == n_iter) mma_commit(bar_acc_done);
          }
          __syncwarp();
        }
      }
    }
  }
  // =========================================================================
  // math warps: group w = warp / 4 takes the tiles of parity w, one thread per query row
  // =========================================================================
  else {
    const int quarter = warp & 3, grp = warp >> 2;
    const int row = quarter * 32 + lane;
    const int gidx = r0 + row;
    const uint32_t lane_addr = tmem_base + ((uint32_t)(quarter * 32) << 16);
    const size_t row_off = (size_t)bh * g.N_q;

    int vlo, vhi;
    key_range_for_queries(g, gidx, gidx + 1, vlo, vhi);
    if (gidx >= g.N_q) { vlo = 0; vhi = 0; }
    const uint32_t vspan = (uint32_t)(vhi - vlo);

    // ---- one-time copy of the Q rows from the staging buffer to tensor memory: the two groups
    // move one column half each (shared-memory tile: row r at r*128 bytes per 64-column atom,
    // 16-byte chunks XOR-swizzled by r % 8; tensor-memory A operand: lane = row, one 32-bit
    // column per pair of K elements)
    bool ok = true;
    if (n_iter > 0) {
      ok = mbar_wait(bar_staging_full, 0, abort_flag, t.status, wait_code(KFWD, 6));
      ok = __all_sync(0xffffffffu, ok);
      if (ok) {
        constexpr int kChunksPerHalf = D / 16;
#pragma unroll
        for (int c = 0; c < kChunksPerHalf; c += 2) {
          uint32_t w[8];
#pragma unroll
          for (int u = 0; u < 2; ++u) {
            const int gc = grp * kChunksPerHalf + c + u;
            const uint32_t addr = staging + (gc >> 3) * kAtomBytesStat + row * 128 + ((((uint32_t)(gc & 7)) ^ (row & 7)) << 4);
            asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];"
                         : "=r"(w[4 * u]), "=r"(w[4 * u + 1]), "=r"(w[4 * u + 2]), "=r"(w[4 * u + 3])
                         : "r"(addr));
          }
          tmem_st8(lane_addr + CF::kQT + 4 * (grp * kChunksPerHalf + c), w);
        }
        tmem_st_wait();
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_q_ready);
    }

    float m_ref = -INFINITY, l_sum = 0.f;     // this group's running maximum (log2 units) and sum for the row
    const uint32_t oacc = lane_addr + CF::kO + (uint32_t)(grp * D);
    for (int it = grp; it < n_iter && ok; it += 2) {
      const int b = it % kFwdSBufs;
      const uint32_t sbuf = lane_addr + CF::kS + 64u * (uint32_t)b;
      const int j0 = (t_begin + it) * BN;
      const bool masked = !(j0 >= vlo && j0 + BN - 1 < vhi);

      ok = mbar_wait(bar_s_full(b), (it / kFwdSBufs) & 1, abort_flag, t.status, wait_code(KFWD, 7));
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after_sync();
      uint32_t s_[4][16];
#pragma unroll
      for (int c = 0; c < 4; ++c) tmem_ld16(sbuf + 16 * c, s_[c]);
#pragma unroll
      for (int c = 0; c < 4; ++c) tmem_ld_wait(s_[c]);

      // maximum of the raw scores (-inf where masked) in eight independent chains; the scale
      // (positive) is applied to the maximum here and to the scores inside the exponent's fma
      if (masked) {
#pragma unroll
        for (int c = 0; c < 4; ++c)
#pragma unroll
          for (int e = 0; e < 16; ++e)
            if (!((uint32_t)(j0 + 16 * c + e - vlo) < vspan)) s_[c][e] = 0xff800000u;   // -inf
      }
      float mx8[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) mx8[e] = fmaxf(__uint_as_float(s_[0][e]), __uint_as_float(s_[0][8 + e]));
#pragma unroll
      for (int c = 1; c < 4; ++c)
#pragma unroll
        for (int e = 0; e < 8; ++e) mx8[e] = fmaxf(mx8[e], fmaxf(__uint_as_float(s_[c][e]), __uint_as_float(s_[c][8 + e])));
      const float mx = fmaxf(fmaxf(fmaxf(mx8[0], mx8[1]), fmaxf(mx8[2], mx8[3])), fmaxf(fmaxf(mx8[4], mx8[5]), fmaxf(mx8[6], mx8[7]))) *
                       g.scale_log2e;
      // lazy rescale: the reference moves only when this tile exceeds it by more than kTau
      const bool grow = mx > m_ref + kTau || (m_ref == -INFINITY && mx > -INFINITY);
      if (__any_sync(0xffffffffu, grow)) {
        const float m_new = grow ? mx : m_ref;
        const float f = (m_ref == -INFINITY) ? 0.f : ex2(m_ref - m_new);   // 1 for the rows that do not move
        l_sum *= f;
        m_ref = m_new;
        if (it >= 2) {
          // multiply this row of the group's O accumulator by f, once its previous P V product is complete
          const int pb = (it - 2) % kFwdSBufs;
          ok = mbar_wait(bar_pv_done(pb), ((it - 2) / kFwdSBufs) & 1, abort_flag, t.status, wait_code(KFWD, 8));
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
          tc_fence_after_sync();
#pragma unroll
          for (int c = 0; c < D / 16; ++c) {
            if (16 * c >= g.D) break;       // padding columns (uniform)
            uint32_t o_[16];
            tmem_ld16(oacc + 16 * c, o_);
            tmem_ld_wait(o_);
            uint32_t lo8[8], hi8[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) {
              lo8[e] = __float_as_uint(__uint_as_float(o_[e]) * f);
              hi8[e] = __float_as_uint(__uint_as_float(o_[8 + e]) * f);
            }
            tmem_st8(oacc + 16 * c, lo8);
            tmem_st8(oacc + 16 * c + 8, hi8);
          }
        }
      }
      const float nm = (m_ref == -INFINITY) ? 0.f : -m_ref;    // no visible key yet: every p below is masked to 0
      const float2 sc2 = make_float2(g.scale_log2e, g.scale_log2e), nm2 = make_float2(nm, nm);
      float2 sum_a = make_float2(0.f, 0.f), sum_b = make_float2(0.f, 0.f);
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t kp[8];
#pragma unroll
        for (int e = 0; e < 16; e += 4) {
          const float2 xa = __ffma2_rn(make_float2(__uint_as_float(s_[c][e]), __uint_as_float(s_[c][e + 1])), sc2, nm2);
          const float2 xb = __ffma2_rn(make_float2(__uint_as_float(s_[c][e + 2]), __uint_as_float(s_[c][e + 3])), sc2, nm2);
          const float2 pa = make_float2(ex2(xa.x), ex2(xa.y)), pb = make_float2(ex2(xb.x), ex2(xb.y));
          sum_a = __fadd2_rn(sum_a, pa);
          sum_b = __fadd2_rn(sum_b, pb);
          kp[e >> 1] = Pack<T>::pack(pa.x, pa.y);
          kp[(e >> 1) + 1] = Pack<T>::pack(pb.x, pb.y);
        }
        tmem_st8(sbuf + 8 * c, kp);      // over score columns this thread has read
      }
      l_sum += (sum_a.x + sum_a.y) + (sum_b.x + sum_b.y);
      tmem_st_wait();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_p_full(b));
    }

    // ---------------- merge of the two groups and output ------------------------------
    float* mine = ml + grp * 2 * BM;
    const float* other = ml + (grp ^ 1) * 2 * BM;
    mine[row] = m_ref; mine[BM + row] = l_sum;
    named_barrier_sync(1, kMathThreads);
    const float m_o = other[row], l_o = other[BM + row];
    const float m_all = fmaxf(m_ref, m_o);
    float f_me = 0.f, f_ot = 0.f, l_all = 0.f;
    if (m_all > -INFINITY) {
      f_me = (m_ref > -INFINITY) ? ex2(m_ref - m_all) : 0.f;
      f_ot = (m_o > -INFINITY) ? ex2(m_o - m_all) : 0.f;
      l_all = l_sum * f_me + l_o * f_ot;
    }
    const float inv = l_all > 0.f ? 1.f / l_all : 0.f;
    if (grp == 0 && gidx < g.N_q) t.out_L[row_off + gidx] = (l_all > 0.f) ? (m_all + log2f(l_all)) * kLn2 : -INFINITY;

    if (n_iter > 0 && ok) ok = mbar_wait(bar_acc_done, 0, abort_flag, t.status, wait_code(KFWD, 9));
    ok = __all_sync(0xffffffffu, ok);
    tc_fence_after_sync();
    // this thread finishes column half `grp` of its row from both accumulators
    const float f0 = (grp == 0 ? f_me : f_ot) * inv, f1 = (grp == 0 ? f_ot : f_me) * inv;
    const bool use0 = f0 > 0.f, use1 = f1 > 0.f && n_iter > 1;      // an accumulator nothing was added to is never read as a number
    constexpr int kColsPerHalf = D / 2;
#pragma unroll
    for (int c = 0; c < kColsPerHalf / 16; ++c) {
      const int col = grp * kColsPerHalf + 16 * c;
      if (col >= g.D) break;     // padding columns (uniform over the warp)
      uint32_t a_[16], b_[16];
      if (n_iter > 0 && ok) {
        tmem_ld16(lane_addr + CF::kO + col, a_);
        tmem_ld16(lane_addr + CF::kO + D + col, b_);
        tmem_ld_wait(a_);
        tmem_ld_wait(b_);
      }
      uint32_t w[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        float v0 = 0.f, v1 = 0.f;
        if (n_iter > 0 && ok) {
          if (use0) { v0 = __uint_as_float(a_[2 * e]) * f0; v1 = __uint_as_float(a_[2 * e + 1]) * f0; }
          if (use1) { v0 = fmaf(__uint_as_float(b_[2 * e]), f1, v0); v1 = fmaf(__uint_as_float(b_[2 * e + 1]), f1, v1); }
        }
        w[e] = Pack<T>::pack(v0, v1);
      }
      if (gidx < g.N_q) store_op16(staging + (uint32_t)(col >> 6) * kAtomBytesStat, row, col & 63, w);
    }
    // the O tile leaves through the staging buffer (Q has been in tensor memory since the prologue)
    store_tile_tma(&maps.out[TO_O], staging, g.D, r0, bh, threadIdx.x == 0);
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == kFwdSWarp) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

template <int D, typename T>
static cudaError_t launch_fwd_one(const TmaMaps& maps, const Geometry& g_in, const Tensors& t, cudaStream_t s) {
  using CF = FwdCfg<D>;
  Geometry g = g_in;
  const long long ctas = (long long)g.BH * ((g.N_q + BM - 1) / BM);
  if (ctas <= 0) return cudaSuccess;
  if (ctas > 0x7fffffffLL) return cudaErrorInvalidValue;
  g.head_group = pick_head_group(ctas, g.BH, 2ll * g.N_kv * g.D * 2);   // K, V
  // more than half of an SM's shared memory: one CTA per SM, so the 512-column
  // tensor-memory allocation never waits for a co-resident CTA
  const size_t smem = CF::kSmemBytes < 122880u ? 122880u : CF::kSmemBytes;
  auto kern = fwd_kernel<D, T>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return e;
  kern<<<(unsigned)ctas, kFwdThreads, smem, s>>>(maps, g, t);
  return cudaGetLastError();
}

// forward: O and L in one launch
cudaError_t launch_fwd(int D, int is_bf16, const TmaMaps& maps, const Geometry& g, const Tensors& t, cudaStream_t s) {
  if (D <= 64) return is_bf16 ? launch_fwd_one<64, __nv_bfloat16>(maps, g, t, s) : launch_fwd_one<64, __half>(maps, g, t, s);
  return is_bf16 ? launch_fwd_one<128, __nv_bfloat16>(maps, g, t, s) : launch_fwd_one<128, __half>(maps, g, t, s);
}

}  // namespace tc
}  // namespace attn
