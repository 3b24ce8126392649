// Shared host/device definitions for the attention kernels: launch parameters,
// the visibility predicate and the per-element double-backward algebra.
//
// Notation (per batch*head), s = 1/sqrt(D):
//   S = s Q K^T (masked)      L_i = ln sum_j exp(S_ij)      P = exp(S - L)
//   dP = dO V^T               Dv_i = sum_j P dP              dS = P (dP - Dv)
//   gdS = s (g_dQ K^T + Q g_dK^T)        gPdV = dO g_dV^T
//   dot2_i = sum_j P gdS      g_dp = P (gdS - dot2)
//   g_P = gdS (dP - Dv) - dP dot2 + gPdV
//   dot3_i = sum_j P g_P      g_S = P (g_P - dot3)
// The same expressions are what the reference's double-backward kernels
// evaluate (csrc/flash_double_backward_v7.cu:1257-1454, 1583-1675).
#pragma once

#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <cuda_bf16.h>
#include <stdint.h>

namespace attn {

constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;

// Everything a kernel needs to know about the problem besides its pointers.
struct Geometry {
  int BH;        // batch * heads
  int N_q, N_kv, D;
  int qi_base;   // absolute index of query row 0  (= chunk_id * N_q)
  int ki_base;   // absolute index of key row 0    (= chunk_id * N_q + N_q - N_kv)
  int window;    // clamped to 2^30 so qi < ki + window never overflows
  int mask_mode; // 0 reference mask, 1 none
  // CTA order: heads are taken in groups of `head_group`; within a group the CTAs go tile by
  // tile, heavy tiles first, over all heads of the group.  Large groups balance the SMs (longest
  // work first), small groups keep the streamed tensors of the heads in flight inside the L2.
  int head_group;
  float scale;       // 1/sqrt(D)
  float scale_log2e; // scale * log2(e)
};

// Visibility of (query row i, key row j), both local indices.  Out-of-range
// rows are never visible.  Reference predicate: flash_double_backward_v7.cu:100-102.
__host__ __device__ __forceinline__ bool visible(const Geometry& g, int i, int j) {
  if (i >= g.N_q || j >= g.N_kv) return false;
  if (g.mask_mode != 0) return true;
  const int qi = g.qi_base + i, ki = g.ki_base + j;
  return (ki >= 0) && (qi >= ki) && (qi < ki + g.window);
}

// Range [j_lo, j_hi) of key rows that can be visible to query rows [i0, i1).
__host__ __device__ __forceinline__ void key_range_for_queries(const Geometry& g, int i0, int i1,
                                                               int& j_lo, int& j_hi) {
  if (i1 > g.N_q) i1 = g.N_q;
  if (g.mask_mode != 0) { j_lo = 0; j_hi = (i0 < i1) ? g.N_kv : 0; return; }
  if (i0 >= i1) { j_lo = j_hi = 0; return; }
  const int qi_min = g.qi_base + i0, qi_max = g.qi_base + i1 - 1;
  int ki_lo = qi_min - g.window + 1; if (ki_lo < 0) ki_lo = 0;
  int ki_hi = qi_max + 1;                       // exclusive
  j_lo = ki_lo - g.ki_base; if (j_lo < 0) j_lo = 0;
  j_hi = ki_hi - g.ki_base; if (j_hi > g.N_kv) j_hi = g.N_kv;
  if (j_hi < j_lo) j_hi = j_lo;
}

// Range [i_lo, i_hi) of query rows that can see key rows [j0, j1).
__host__ __device__ __forceinline__ void query_range_for_keys(const Geometry& g, int j0, int j1,
                                                              int& i_lo, int& i_hi) {
  if (j1 > g.N_kv) j1 = g.N_kv;
  if (g.mask_mode != 0) { i_lo = 0; i_hi = (j0 < j1) ? g.N_q : 0; return; }
  if (j0 >= j1) { i_lo = i_hi = 0; return; }
  int ki_min = g.ki_base + j0; const int ki_max = g.ki_base + j1 - 1;
  if (ki_max < 0) { i_lo = i_hi = 0; return; }
  if (ki_min < 0) ki_min = 0;
  i_lo = ki_min - g.qi_base; if (i_lo < 0) i_lo = 0;
  long long hi = (long long)ki_max + g.window - g.qi_base;   // exclusive
  i_hi = hi > g.N_q ? g.N_q : (int)hi;
  if (i_hi < i_lo) i_hi = i_lo;
}

// True when every (i, j) of the tile [i0,i1) x [j0,j1) is visible, so the
// per-element predicate can be skipped.
__host__ __device__ __forceinline__ bool tile_fully_visible(const Geometry& g, int i0, int i1,
                                                            int j0, int j1) {
  if (i1 > g.N_q || j1 > g.N_kv) return false;
  if (g.mask_mode != 0) return true;
  const int qi_min = g.qi_base + i0, qi_max = g.qi_base + i1 - 1;
  const int ki_min = g.ki_base + j0, ki_max = g.ki_base + j1 - 1;
  return ki_min >= 0 && qi_min >= ki_max && qi_max < ki_min + g.window;
}

// Per-query-row scalars consumed by the element algebra.
struct RowStats {
  float L2;    // L * log2(e);  +inf for rows beyond N_q (forces P = 0)
  float Dv;
  float dot2;
  float dot3;
};

__device__ __forceinline__ float prob(float s_raw, float scale_log2e, float L2, bool vis) {
  return vis ? exp2f(fmaf(s_raw, scale_log2e, -L2)) : 0.f;
}

// Second-order element terms from the four raw score accumulators.
struct HvpTerms { float p, dS, g_dp, g_S; };
__device__ __forceinline__ HvpTerms hvp_terms(float p, float dP, float gdS_raw, float gPdV,
                                              float scale, const RowStats& r) {
  HvpTerms t;
  const float gds = gdS_raw * scale;
  const float dpd = dP - r.Dv;
  t.p = p;
  t.dS = p * dpd;
  t.g_dp = p * (gds - r.dot2);
  const float gP = fmaf(gds, dpd, fmaf(-dP, r.dot2, gPdV));
  t.g_S = p * (gP - r.dot3);
  return t;
}

// dtype helpers -------------------------------------------------------------
template <typename T> struct Elem;
template <> struct Elem<float> {
  static __device__ __forceinline__ float to_float(float v) { return v; }
  static __device__ __forceinline__ float from_float(float v) { return v; }
};
template <> struct Elem<__half> {
  static __device__ __forceinline__ float to_float(__half v) { return __half2float(v); }
  static __device__ __forceinline__ __half from_float(float v) { return __float2half_rn(v); }
};
template <> struct Elem<__nv_bfloat16> {
  static __device__ __forceinline__ float to_float(__nv_bfloat16 v) { return __bfloat162float(v); }
  static __device__ __forceinline__ __nv_bfloat16 from_float(float v) { return __float2bfloat16_rn(v); }
};

// Pointer bundle shared by every launcher.  Unused members stay null.
// blockIdx -> (head, rank of the tile within the head) under the grouped order
__device__ __forceinline__ void cta_to_head_and_rank(const Geometry& g, int tiles, int& bh, int& rank) {
  const int per_group = g.head_group * tiles;
  const int grp = (int)(blockIdx.x / (unsigned)per_group);
  const int rem = (int)(blockIdx.x - (unsigned)(grp * per_group));
  const int first = grp * g.head_group;
  const int gsize = min(g.head_group, g.BH - first);
  rank = rem / gsize;
  bh = first + (rem - rank * gsize);
}

// heads per group: as many as keep `streamed_bytes_per_head` of every head of the group within
// about 16 MB of L2, all heads when the grid is small anyway
inline int pick_head_group(long long ctas, int BH, long long streamed_bytes_per_head) {
  if (ctas < 8 * 148) return BH > 0 ? BH : 1;
  long long n = (16ll << 20) / (streamed_bytes_per_head > 0 ? streamed_bytes_per_head : 1);
  if (n < 1) n = 1;
  if (n > BH) n = BH;
  return (int)n;
}

struct Tensors {
  const void *Q, *K, *V, *dO, *O, *g_dQ, *g_dK, *g_dV;   // inputs
  const float* L;                                        // [BH, N_q]
  void *out_O, *out_dQ, *out_dK, *out_dV, *out_g_dO, *out_g_Q, *out_g_K, *out_g_V;
  float* out_L;
  float *Dv, *dot2, *dot3;                               // scratch, [BH, N_q] each
  unsigned int* status;  // device status word: a kernel that gives up on a bounded
                         // wait stores a non-zero code here and returns
};

}  // namespace attn
