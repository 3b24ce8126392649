// fp32 SIMT kernels for attention forward / backward / double-backward.
//
// This family serves float32 inputs (where results must agree with an fp64
// oracle to 1e-4) and half-precision inputs whose head dimension has no
// tensor-core kernel.  All arithmetic is fp32 on CUDA cores; inputs are widened
// when a tile is staged in shared memory.  Nothing here materialises more than
// a 32 x 32 score tile per CTA.
//
// Tiling: a CTA of 256 threads owns 32 "stationary" rows of one (batch, head)
// -- query rows in the row kernels, key rows in the column kernels -- and streams
// 32-row tiles of the other axis.  Thread (ty, tx), ty = tid/16, tx = tid%16,
// holds score elements (ty + 16a, tx + 16b) and output elements
// (ty + 16a, tx + 16c).  Every output element is produced by exactly one thread
// in a fixed order, so results are bitwise reproducible.
#include "attn_common.cuh"
#include "attn_launch.h"

namespace attn {
namespace simt {

constexpr int TS = 32;        // stationary rows per CTA
constexpr int TT = 32;        // streamed rows per iteration
constexpr int NT = 256;       // threads per CTA
constexpr int OPLD = 33;      // leading dimension of an operand tile
constexpr int MAXC = 8;       // output columns per thread = D/16 <= 8

enum Kind { K_FWD = 0, K_BWD_ROW, K_BWD_COL, K_HVP_ROW, K_HVP_COL };

// Stage rows [row0, row0+32) of a [n_rows, D] matrix as fp32, zero beyond n_rows.
template <typename T>
__device__ __forceinline__ void stage_tile(float* dst, int ldd, const T* src, int row0, int n_rows,
                                           int D) {
  const int per_row = D >> 1;
  for (int idx = threadIdx.x; idx < 32 * per_row; idx += NT) {
    const int r = idx / per_row, c = (idx - r * per_row) << 1;
    float v0 = 0.f, v1 = 0.f;
    const int gr = row0 + r;
    if (gr >= 0 && gr < n_rows) {
      const T* p = src + (size_t)gr * D + c;
      v0 = Elem<T>::to_float(p[0]);
      v1 = Elem<T>::to_float(p[1]);
    }
    dst[r * ldd + c] = v0;
    dst[r * ldd + c + 1] = v1;
  }
}

// acc[a][b] += <A[ty+16a, :], B[tx+16b, :]>
__device__ __forceinline__ void score_fma(const float* A, const float* Bm, int D, int ldd, int ty,
                                          int tx, float acc[2][2]) {
  const float4* a0 = reinterpret_cast<const float4*>(A + ty * ldd);
  const float4* a1 = reinterpret_cast<const float4*>(A + (ty + 16) * ldd);
  const float4* b0 = reinterpret_cast<const float4*>(Bm + tx * ldd);
  const float4* b1 = reinterpret_cast<const float4*>(Bm + (tx + 16) * ldd);
  for (int k = 0; k < (D >> 2); ++k) {
    const float4 x0 = a0[k], x1 = a1[k], y0 = b0[k], y1 = b1[k];
    acc[0][0] += x0.x * y0.x + x0.y * y0.y + x0.z * y0.z + x0.w * y0.w;
    acc[0][1] += x0.x * y1.x + x0.y * y1.y + x0.z * y1.z + x0.w * y1.w;
    acc[1][0] += x1.x * y0.x + x1.y * y0.y + x1.z * y0.z + x1.w * y0.w;
    acc[1][1] += x1.x * y1.x + x1.y * y1.y + x1.z * y1.z + x1.w * y1.w;
  }
}

// out[a][c] += sum_j Op[ty+16a, j] * Z[j, tx+16c]
__device__ __forceinline__ void out_fma(const float* Op, const float* Z, int ncol, int ldd, int ty,
                                        int tx, float out[2][MAXC]) {
  for (int j = 0; j < TT; ++j) {
    const float o0 = Op[ty * OPLD + j], o1 = Op[(ty + 16) * OPLD + j];
#pragma unroll
    for (int c = 0; c < MAXC; ++c) {
      if (c < ncol) {
        const float z = Z[j * ldd + tx + 16 * c];
        out[0][c] = fmaf(o0, z, out[0][c]);
        out[1][c] = fmaf(o1, z, out[1][c]);
      }
    }
  }
}

__device__ __forceinline__ float half_warp_sum(float v) {
#pragma unroll
  for (int o = 8; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float half_warp_max(float v) {
#pragma unroll
  for (int o = 8; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

template <typename T>
__device__ __forceinline__ void store_rows(T* dst, int row0, int n_rows, int D, int ncol, int ty,
                                           int tx, const float out[2][MAXC], float mul) {
#pragma unroll
  for (int a = 0; a < 2; ++a) {
    const int r = row0 + ty + 16 * a;
    if (r < n_rows) {
#pragma unroll
      for (int c = 0; c < MAXC; ++c)
        if (c < ncol) dst[(size_t)r * D + tx + 16 * c] = Elem<T>::from_float(out[a][c] * mul);
    }
  }
}

// One kernel per Kind.  Row kinds: stationary = query rows.  Column kinds:
// stationary = key rows and the score tile is held transposed.
template <int KIND, typename T>
__global__ void __launch_bounds__(NT) attn_simt_kernel(const Geometry g, const Tensors t) {
  extern __shared__ __align__(16) float smem[];
  constexpr bool kCol = (KIND == K_BWD_COL || KIND == K_HVP_COL);
  constexpr int kNStat = (KIND == K_FWD) ? 1 : (KIND == K_BWD_ROW) ? 2 : (KIND == K_BWD_COL) ? 2
                         : (KIND == K_HVP_ROW) ? 3 : 4;
  constexpr int kNStream = (KIND == K_FWD) ? 2 : (KIND == K_BWD_ROW) ? 2 : (KIND == K_BWD_COL) ? 2
                           : (KIND == K_HVP_ROW) ? 4 : 3;
  constexpr int kNOp = (KIND == K_FWD) ? 1 : (KIND == K_BWD_ROW) ? 1 : (KIND == K_BWD_COL) ? 2
                       : (KIND == K_HVP_ROW) ? 4 : 3;
  const int D = g.D, ldd = D + 4, ncol = D >> 4;
  const int n_stat = kCol ? g.N_kv : g.N_q;
  const int tiles = (n_stat + TS - 1) / TS;
  const int bh = blockIdx.x / tiles;
  const int r0 = (blockIdx.x - bh * tiles) * TS;
  const int tid = threadIdx.x, ty = tid >> 4, tx = tid & 15;

  float* stat[4];
  float* strm[4];
  float* op[4];
  float* p = smem;
  for (int i = 0; i < kNStat; ++i) { stat[i] = p; p += TS * ldd; }
  for (int i = 0; i < kNStream; ++i) { strm[i] = p; p += TT * ldd; }
  for (int i = 0; i < kNOp; ++i) { op[i] = p; p += TS * OPLD; }
  float* sL2 = p;  p += 32;   // per query row of the current tile (stationary or streamed)
  float* sDv = p;  p += 32;
  float* sD2 = p;  p += 32;
  float* sD3 = p;  p += 32;

  const size_t q_off = (size_t)bh * g.N_q * D, kv_off = (size_t)bh * g.N_kv * D;
  const T* Q = (const T*)t.Q + q_off;
  const T* K = (const T*)t.K + kv_off;
  const T* V = (const T*)t.V + kv_off;
  const T* dO = t.dO ? (const T*)t.dO + q_off : nullptr;
  const T* gQ = t.g_dQ ? (const T*)t.g_dQ + q_off : nullptr;
  const T* gK = t.g_dK ? (const T*)t.g_dK + kv_off : nullptr;
  const T* gV = t.g_dV ? (const T*)t.g_dV + kv_off : nullptr;
  const size_t row_off = (size_t)bh * g.N_q;

  // ---- stationary tiles -----------------------------------------------------
  if constexpr (KIND == K_FWD) {
    stage_tile<T>(stat[0], ldd, Q, r0, g.N_q, D);
  } else if constexpr (KIND == K_BWD_ROW) {
    stage_tile<T>(stat[0], ldd, Q, r0, g.N_q, D);
    stage_tile<T>(stat[1], ldd, dO, r0, g.N_q, D);
  } else if constexpr (KIND == K_BWD_COL) {
    stage_tile<T>(stat[0], ldd, K, r0, g.N_kv, D);
    stage_tile<T>(stat[1], ldd, V, r0, g.N_kv, D);
  } else if constexpr (KIND == K_HVP_ROW) {
    stage_tile<T>(stat[0], ldd, Q, r0, g.N_q, D);
    stage_tile<T>(stat[1], ldd, dO, r0, g.N_q, D);
    stage_tile<T>(stat[2], ldd, gQ, r0, g.N_q, D);
  } else {
    stage_tile<T>(stat[0], ldd, K, r0, g.N_kv, D);
    stage_tile<T>(stat[1], ldd, V, r0, g.N_kv, D);
    stage_tile<T>(stat[2], ldd, gK, r0, g.N_kv, D);
    stage_tile<T>(stat[3], ldd, gV, r0, g.N_kv, D);
  }

  // ---- range of streamed tiles ---------------------------------------------
  int lo, hi;
  if constexpr (kCol) query_range_for_keys(g, r0, r0 + TS, lo, hi);
  else key_range_for_queries(g, r0, r0 + TS, lo, hi);
  const int t_begin = lo / TT, t_end = (hi + TT - 1) / TT;

  float out0[2][MAXC], out1[2][MAXC];
#pragma unroll
  for (int a = 0; a < 2; ++a)
#pragma unroll
    for (int c = 0; c < MAXC; ++c) out0[a][c] = out1[a][c] = 0.f;

  // ======================= forward =========================================
  if constexpr (KIND == K_FWD) {
    // pass 1: log-sum-exp per row, in the log2 domain
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
    for (int tt = t_begin; tt < t_end; ++tt) {
      __syncthreads();
      stage_tile<T>(strm[0], ldd, K, tt * TT, g.N_kv, D);
      __syncthreads();
      float s[2][2] = {{0.f, 0.f}, {0.f, 0.f}};
      score_fma(stat[0], strm[0], D, ldd, ty, tx, s);
#pragma unroll
      for (int a = 0; a < 2; ++a)
#pragma unroll
        for (int b = 0; b < 2; ++b) {
          if (visible(g, r0 + ty + 16 * a, tt * TT + tx + 16 * b)) {
            const float x = s[a][b] * g.scale_log2e;
            const float mn = fmaxf(m[a], x);
            l[a] = l[a] * exp2f(m[a] - mn) + exp2f(x - mn);
            m[a] = mn;
          }
        }
    }
#pragma unroll
    for (int a = 0; a < 2; ++a) {
      const float mt = half_warp_max(m[a]);
      const float lt = half_warp_sum(mt == -INFINITY ? 0.f : l[a] * exp2f(m[a] - mt));
      const float L2 = (lt > 0.f) ? mt + log2f(lt) : -INFINITY;
      const int r = r0 + ty + 16 * a;
      if (tx == 0) {
        sL2[ty + 16 * a] = (r < g.N_q) ? L2 : INFINITY;
        if (r < g.N_q) t.out_L[row_off + r] = L2 * kLn2;
      }
    }
    // pass 2: O = P V
    for (int tt = t_begin; tt < t_end; ++tt) {
      __syncthreads();
      stage_tile<T>(strm[0], ldd, K, tt * TT, g.N_kv, D);
      stage_tile<T>(strm[1], ldd, V, tt * TT, g.N_kv, D);
      __syncthreads();
      float s[2][2] = {{0.f, 0.f}, {0.f, 0.f}};
      score_fma(stat[0], strm[0], D, ldd, ty, tx, s);
#pragma unroll
      for (int a = 0; a < 2; ++a)
#pragma unroll
        for (int b = 0; b < 2; ++b) {
          const int i = ty + 16 * a, j = tx + 16 * b;
          op[0][i * OPLD + j] = prob(s[a][b], g.scale_log2e, sL2[i], visible(g, r0 + i, tt * TT + j));
        }
      __syncthreads();
      out_fma(op[0], strm[1], ncol, ldd, ty, tx, out0);
    }
    store_rows<T>((T*)t.out_O + q_off, r0, g.N_q, D, ncol, ty, tx, out0, 1.f);
    return;
  }

  // ======================= first backward, row side ========================
  if constexpr (KIND == K_BWD_ROW) {
    // D_i = sum_d dO * O from the stored (rounded) O; kept for the column kernel
    __syncthreads();
    {
      const T* O = (const T*)t.O + q_off;
#pragma unroll
      for (int a = 0; a < 2; ++a) {
        const int i = ty + 16 * a, r = r0 + i;
        float acc = 0.f;
        if (r < g.N_q)
          for (int d = tx; d < D; d += 16) acc += stat[1][i * ldd + d] * Elem<T>::to_float(O[(size_t)r * D + d]);
        acc = half_warp_sum(acc);
        if (tx == 0) {
          sDv[i] = acc;
          sL2[i] = (r < g.N_q) ? t.L[row_off + r] * kLog2e : INFINITY;
          if (r < g.N_q) t.Dv[row_off + r] = acc;
        }
      }
    }
    for (int tt = t_begin; tt < t_end; ++tt) {
      __syncthreads();
      stage_tile<T>(strm[0], ldd, K, tt * TT, g.N_kv, D);
      stage_tile<T>(strm[1], ldd, V, tt * TT, g.N_kv, D);
      __syncthreads();
      float s[2][2] = {{0.f, 0.f}, {0.f, 0.f}}, dp[2][2] = {{0.f, 0.f}, {0.f, 0.f}};
      score_fma(stat[0], strm[0], D, ldd, ty, tx, s);
      score_fma(stat[1], strm[1], D, ldd, ty, tx, dp);
#pragma unroll
      for (int a = 0; a < 2; ++a)
#pragma unroll
        for (int b = 0; b < 2; ++b) {
          const int i = ty + 16 * a, j = tx + 16 * b;
          const float pr = prob(s[a][b], g.scale_log2e, sL2[i], visible(g, r0 + i, tt * TT + j));
          op[0][i * OPLD + j] = pr * (dp[a][b] - sDv[i]);
        }
      __syncthreads();
      out_fma(op[0], strm[0], ncol, ldd, ty, tx, out0);
    }
    store_rows<T>((T*)t.out_dQ + q_off, r0, g.N_q, D, ncol, ty, tx, out0, g.scale);
    return;
  }

  // ======================= first backward, column side =====================
  if constexpr (KIND == K_BWD_COL) {
    for (int tt = t_begin; tt < t_end; ++tt) {
      __syncthreads();
      stage_tile<T>(strm[0], ldd, Q, tt * TT, g.N_q, D);
      stage_tile<T>(strm[1], ldd, dO, tt * TT, g.N_q, D);
      if (tid < 32) {
        const int r = tt * TT + tid;
        sL2[tid] = (r < g.N_q) ? t.L[row_off + r] * kLog2e : INFINITY;
        sDv[tid] = (r < g.N_q) ? t.Dv[row_off + r] : 0.f;
      }
      __syncthreads();
      float s[2][2] = {{0.f, 0.f}, {0.f, 0.f}}, dp[2][2] = {{0.f, 0.f}, {0.f, 0.f}};
      score_fma(stat[0], strm[0], D, ldd, ty, tx, s);    // S^T  = K Q^T
      score_fma(stat[1], strm[1], D, ldd, ty, tx, dp);   // dP^T = V dO^T
#pragma unroll
      for (int a = 0; a < 2; ++a)
#pragma unroll
        for (int b = 0; b < 2; ++b) {
          const int jk = ty + 16 * a, iq = tx + 16 * b;
          const float pr = prob(s[a][b], g.scale_log2e, sL2[iq], visible(g, tt * TT + iq, r0 + jk));
          op[0][jk * OPLD + iq] = pr;
          op[1][jk * OPLD + iq] = pr * (dp[a][b] - sDv[iq]);
        }
      __syncthreads();
      out_fma(op[0], strm[1], ncol, ldd, ty, tx, out0);   // dV += P^T dO
      out_fma(op[1], strm[0], ncol, ldd, ty, tx, out1);   // dK += dS^T Q
    }
    store_rows<T>((T*)t.out_dV + kv_off, r0, g.N_kv, D, ncol, ty, tx, out0, 1.f);
    store_rows<T>((T*)t.out_dK + kv_off, r0, g.N_kv, D, ncol, ty, tx, out1, g.scale);
    return;
  }

  // ======================= double backward, row side =======================
  if constexpr (KIND == K_HVP_ROW) {
    __syncthreads();
    if (tid < 32) {
      const int r = r0 + tid;
      sL2[tid] = (r < g.N_q) ? t.L[row_off + r] * kLog2e : INFINITY;
    }
    // pass 1: Dv, dot2, dot3 per row
    float aD[2] = {0.f, 0.f}, a2[2] = {0.f, 0.f}, aA[2] = {0.f, 0.f}, aE[2] = {0.f, 0.f};
    for (int tt = t_begin; tt < t_end; ++tt) {
      __syncthreads();
      stage_tile<T>(strm[0], ldd, K, tt * TT, g.N_kv, D);
      stage_tile<T>(strm[1], ldd, V, tt * TT, g.N_kv, D);
      stage_tile<T>(strm[2], ldd, gK, tt * TT, g.N_kv, D);
      stage_tile<T>(strm[3], ldd, gV, tt * TT, g.N_kv, D);
      __syncthreads();
      float s[2][2] = {{0.f, 0.f}, {0.f, 0.f}}, dp[2][2] = {{0.f, 0.f}, {0.f, 0.f}};
      float gs[2][2] = {{0.f, 0.f}, {0.f, 0.f}}, gp[2][2] = {{0.f, 0.f}, {0.f, 0.f}};
      score_fma(stat[0], strm[0], D, ldd, ty, tx, s);    // Q K^T
      score_fma(stat[1], strm[1], D, ldd, ty, tx, dp);   // dO V^T
      score_fma(stat[2], strm[0], D, ldd, ty, tx, gs);   // g_dQ K^T
      score_fma(stat[0], strm[2], D, ldd, ty, tx, gs);   // + Q g_dK^T
      score_fma(stat[1], strm[3], D, ldd, ty, tx, gp);   // dO g_dV^T
#pragma unroll
      for (int a = 0; a < 2; ++a)
#pragma unroll
        for (int b = 0; b < 2; ++b) {
          const int i = ty + 16 * a, j = tx + 16 * b;
          const float pr = prob(s[a][b], g.scale_log2e, sL2[i], visible(g, r0 + i, tt * TT + j));
          const float gds = gs[a][b] * g.scale;
          aD[a] = fmaf(pr, dp[a][b], aD[a]);
          a2[a] = fmaf(pr, gds, a2[a]);
          aA[a] = fmaf(pr * gds, dp[a][b], aA[a]);
          aE[a] = fmaf(pr, gp[a][b], aE[a]);
        }
    }
    __syncthreads();
#pragma unroll
    for (int a = 0; a < 2; ++a) {
      const float Dv = half_warp_sum(aD[a]), d2 = half_warp_sum(a2[a]);
      const float A = half_warp_sum(aA[a]), E = half_warp_sum(aE[a]);
      const float d3 = A - 2.f * Dv * d2 + E;
      const int i = ty + 16 * a, r = r0 + i;
      if (tx == 0) {
        sDv[i] = Dv; sD2[i] = d2; sD3[i] = d3;
        if (r < g.N_q) { t.Dv[row_off + r] = Dv; t.dot2[row_off + r] = d2; t.dot3[row_off + r] = d3; }
      }
    }
    // pass 2: g_Q and g_dO
    for (int tt = t_begin; tt < t_end; ++tt) {
      __syncthreads();
      stage_tile<T>(strm[0], ldd, K, tt * TT, g.N_kv, D);
      stage_tile<T>(strm[1], ldd, V, tt * TT, g.N_kv, D);
      stage_tile<T>(strm[2], ldd, gK, tt * TT, g.N_kv, D);
      stage_tile<T>(strm[3], ldd, gV, tt * TT, g.N_kv, D);
      __syncthreads();
      float s[2][2] = {{0.f, 0.f}, {0.f, 0.f}}, dp[2][2] = {{0.f, 0.f}, {0.f, 0.f}};
      float gs[2][2] = {{0.f, 0.f}, {0.f, 0.f}}, gp[2][2] = {{0.f, 0.f}, {0.f, 0.f}};
      score_fma(stat[0], strm[0], D, ldd, ty, tx, s);
      score_fma(stat[1], strm[1], D, ldd, ty, tx, dp);
      score_fma(stat[2], strm[0], D, ldd, ty, tx, gs);
      score_fma(stat[0], strm[2], D, ldd, ty, tx, gs);
      score_fma(stat[1], strm[3], D, ldd, ty, tx, gp);
#pragma unroll
      for (int a = 0; a < 2; ++a)
#pragma unroll
        for (int b = 0; b < 2; ++b) {
          const int i = ty + 16 * a, j = tx + 16 * b;
          const float pr = prob(s[a][b], g.scale_log2e, sL2[i], visible(g, r0 + i, tt * TT + j));
          const RowStats rs{sL2[i], sDv[i], sD2[i], sD3[i]};
          const HvpTerms h = hvp_terms(pr, dp[a][b], gs[a][b], gp[a][b], g.scale, rs);
          op[0][i * OPLD + j] = h.dS;
          op[1][i * OPLD + j] = h.g_S;
          op[2][i * OPLD + j] = h.p;
          op[3][i * OPLD + j] = h.g_dp;
        }
      __syncthreads();
      out_fma(op[0], strm[2], ncol, ldd, ty, tx, out0);   // g_Q  += dS g_dK
      out_fma(op[1], strm[0], ncol, ldd, ty, tx, out0);   //       + g_S K
      out_fma(op[2], strm[3], ncol, ldd, ty, tx, out1);   // g_dO += P g_dV
      out_fma(op[3], strm[1], ncol, ldd, ty, tx, out1);   //       + g_dp V
    }
    store_rows<T>((T*)t.out_g_Q + q_off, r0, g.N_q, D, ncol, ty, tx, out0, g.scale);
    store_rows<T>((T*)t.out_g_dO + q_off, r0, g.N_q, D, ncol, ty, tx, out1, 1.f);
    return;
  }

  // ======================= double backward, column side ====================
  if constexpr (KIND == K_HVP_COL) {
    for (int tt = t_begin; tt < t_end; ++tt) {
      __syncthreads();
      stage_tile<T>(strm[0], ldd, Q, tt * TT, g.N_q, D);
      stage_tile<T>(strm[1], ldd, dO, tt * TT, g.N_q, D);
      stage_tile<T>(strm[2], ldd, gQ, tt * TT, g.N_q, D);
      if (tid < 32) {
        const int r = tt * TT + tid;
        const bool in = r < g.N_q;
        sL2[tid] = in ? t.L[row_off + r] * kLog2e : INFINITY;
        sDv[tid] = in ? t.Dv[row_off + r] : 0.f;
        sD2[tid] = in ? t.dot2[row_off + r] : 0.f;
        sD3[tid] = in ? t.dot3[row_off + r] : 0.f;
      }
      __syncthreads();
      float s[2][2] = {{0.f, 0.f}, {0.f, 0.f}}, dp[2][2] = {{0.f, 0.f}, {0.f, 0.f}};
      float gs[2][2] = {{0.f, 0.f}, {0.f, 0.f}}, gp[2][2] = {{0.f, 0.f}, {0.f, 0.f}};
      score_fma(stat[0], strm[0], D, ldd, ty, tx, s);    // K Q^T
      score_fma(stat[1], strm[1], D, ldd, ty, tx, dp);   // V dO^T
      score_fma(stat[0], strm[2], D, ldd, ty, tx, gs);   // K g_dQ^T
      score_fma(stat[2], strm[0], D, ldd, ty, tx, gs);   // + g_dK Q^T
      score_fma(stat[3], strm[1], D, ldd, ty, tx, gp);   // g_dV dO^T
#pragma unroll
      for (int a = 0; a < 2; ++a)
#pragma unroll
        for (int b = 0; b < 2; ++b) {
          const int jk = ty + 16 * a, iq = tx + 16 * b;
          const float pr = prob(s[a][b], g.scale_log2e, sL2[iq], visible(g, tt * TT + iq, r0 + jk));
          const RowStats rs{sL2[iq], sDv[iq], sD2[iq], sD3[iq]};
          const HvpTerms h = hvp_terms(pr, dp[a][b], gs[a][b], gp[a][b], g.scale, rs);
          op[0][jk * OPLD + iq] = h.dS;
          op[1][jk * OPLD + iq] = h.g_S;
          op[2][jk * OPLD + iq] = h.g_dp;
        }
      __syncthreads();
      out_fma(op[0], strm[2], ncol, ldd, ty, tx, out0);   // g_K += dS^T g_dQ
      out_fma(op[1], strm[0], ncol, ldd, ty, tx, out0);   //      + g_S^T Q
      out_fma(op[2], strm[1], ncol, ldd, ty, tx, out1);   // g_V += g_dp^T dO
    }
    store_rows<T>((T*)t.out_g_K + kv_off, r0, g.N_kv, D, ncol, ty, tx, out0, g.scale);
    store_rows<T>((T*)t.out_g_V + kv_off, r0, g.N_kv, D, ncol, ty, tx, out1, 1.f);
    return;
  }
}

template <int KIND>
static size_t smem_bytes(int D) {
  constexpr int nStat = (KIND == K_FWD) ? 1 : (KIND == K_BWD_ROW) ? 2 : (KIND == K_BWD_COL) ? 2
                        : (KIND == K_HVP_ROW) ? 3 : 4;
  constexpr int nStream = (KIND == K_FWD) ? 2 : (KIND == K_BWD_ROW) ? 2 : (KIND == K_BWD_COL) ? 2
                          : (KIND == K_HVP_ROW) ? 4 : 3;
  constexpr int nOp = (KIND == K_FWD) ? 1 : (KIND == K_BWD_ROW) ? 1 : (KIND == K_BWD_COL) ? 2
                      : (KIND == K_HVP_ROW) ? 4 : 3;
  return sizeof(float) * ((size_t)(nStat + nStream) * 32 * (D + 4) + (size_t)nOp * 32 * OPLD + 128);
}

template <int KIND, typename T>
static cudaError_t launch_one(const Geometry& g, const Tensors& t, cudaStream_t stream) {
  constexpr bool kCol = (KIND == K_BWD_COL || KIND == K_HVP_COL);
  const int n_stat = kCol ? g.N_kv : g.N_q;
  const long long ctas = (long long)g.BH * ((n_stat + TS - 1) / TS);
  if (ctas <= 0) return cudaSuccess;
  if (ctas > 0x7fffffffLL) return cudaErrorInvalidValue;
  const size_t smem = smem_bytes<KIND>(g.D);
  auto kern = attn_simt_kernel<KIND, T>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return e;
  kern<<<(unsigned)ctas, NT, smem, stream>>>(g, t);
  return cudaGetLastError();
}

template <typename T>
static cudaError_t dispatch(int op, const Geometry& g, const Tensors& t, cudaStream_t s, int* n, int phases) {
  cudaError_t e = cudaSuccess;
  *n = 0;
  if (op == OP_FORWARD) {
    e = launch_one<K_FWD, T>(g, t, s); *n = 1;
  } else if (op == OP_BACKWARD) {
    e = launch_one<K_BWD_ROW, T>(g, t, s);
    if (e == cudaSuccess) e = launch_one<K_BWD_COL, T>(g, t, s);
    *n = 2;
  } else {
    // the row kernel computes the per-row scalars itself (its first pass)
    if (phases & (HVP_PHASE_PRE | HVP_PHASE_ROW)) { e = launch_one<K_HVP_ROW, T>(g, t, s); ++*n; }
    if (e == cudaSuccess && (phases & HVP_PHASE_COL)) { e = launch_one<K_HVP_COL, T>(g, t, s); ++*n; }
  }
  return e;
}

}  // namespace simt

cudaError_t launch_simt(int op, int dtype, const Geometry& g, const Tensors& t, cudaStream_t s,
                        int* launches, int phases) {
  switch (dtype) {
    case 0: return simt::dispatch<__half>(op, g, t, s, launches, phases);
    case 1: return simt::dispatch<__nv_bfloat16>(op, g, t, s, launches, phases);
    default: return simt::dispatch<float>(op, g, t, s, launches, phases);
  }
}

}  // namespace attn
