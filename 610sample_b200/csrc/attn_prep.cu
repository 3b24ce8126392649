// Step before the attention kernels, fused: per-head RMS normalisation of Q / K rows, rotary
// position embedding, and the change of layout from the projections' [T, H, d] to the kernels'
// [1, H, T, d], in one pass over the data (the reference does these as separate eager PyTorch
// operations followed by permute + contiguous: e2e/ttt_pytorch/model.py:76-84, 96-116, 260-263,
// 309-316, 182-184).  Arithmetic in fp32 with the reference's rounding points:
// (x * rsqrt(mean(x^2) + eps)) rounded to the input type, times the weight rounded again, rotated
// pairwise by (cos, sin) of the position in fp32, rounded.
//
// Algorithmically the kernel is one read and one write of the tensor (the table of angles is
// shared by all heads and stays in L2); what it has to avoid is being bound by instruction issue
// instead: about 14 instructions per element go through the SM for 4 bytes of traffic.  Main kernel: a group of 8 or 16 lanes owns one token,
// a lane eight consecutive elements (16-byte accesses for the half types); the group walks over
// four heads of its token with all four loads in flight, so the (cos, sin) values and the weight
// are fetched once per token instead of once per head, and a CTA of 256 threads reads 1 KB runs of
// x and writes 4 to 8 KB runs of the output.  Head dimensions that are not a multiple of 8, or
// pointers that are not 16-byte aligned, take the pairwise kernel (one warp per vector).
#include "attn_b200.h"
#include "attn_common.cuh"

namespace attn {

// two consecutive elements as one aligned access (d is even, so every pair is aligned)
template <typename T> struct PairIO;
template <> struct PairIO<float> {
  static __device__ __forceinline__ float2 load(const float* p) { return *reinterpret_cast<const float2*>(p); }
  static __device__ __forceinline__ void store(float* p, float a, float b) { *reinterpret_cast<float2*>(p) = make_float2(a, b); }
};
template <> struct PairIO<__half> {
  static __device__ __forceinline__ float2 load(const __half* p) { return __half22float2(*reinterpret_cast<const __half2*>(p)); }
  static __device__ __forceinline__ void store(__half* p, float a, float b) { *reinterpret_cast<__half2*>(p) = __floats2half2_rn(a, b); }
};
template <> struct PairIO<__nv_bfloat16> {
  static __device__ __forceinline__ float2 load(const __nv_bfloat16* p) { return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p)); }
  static __device__ __forceinline__ void store(__nv_bfloat16* p, float a, float b) { *reinterpret_cast<__nv_bfloat162*>(p) = __floats2bfloat162_rn(a, b); }
};

template <typename T>
__global__ void qk_norm_rope_kernel(const T* __restrict__ x, const T* __restrict__ weight,
                                    const float* __restrict__ freqs,   // [positions][d/2][cos, sin]
                                    T* __restrict__ out, int n_tok, int H, int d, int pos0, int norm_from,
                                    float eps) {
  const long long vec = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (vec >= (long long)n_tok * H) return;
  const int lane = threadIdx.x & 31;
  const int tok = (int)(vec / H), h = (int)(vec % H);
  const T* src = x + ((size_t)tok * H + h) * d;
  T* dst = out + ((size_t)h * n_tok + tok) * d;
  const int pairs = d >> 1;
  float a[2], b[2];            // up to two pairs per lane (d <= 128)
  float ss = 0.f;
#pragma unroll
  for (int u = 0; u < 2; ++u) {
    const int p = lane + 32 * u;
    a[u] = b[u] = 0.f;
    if (p < pairs) {
      const float2 v = PairIO<T>::load(src + 2 * p);
      a[u] = v.x; b[u] = v.y;
      ss += a[u] * a[u] + b[u] * b[u];
    }
  }
  if (weight != nullptr && tok >= norm_from) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    const float inv = rsqrtf(ss / (float)d + eps);
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      const int p = lane + 32 * u;
      if (p < pairs) {
        const float2 w = PairIO<T>::load(weight + 2 * p);
        a[u] = Elem<T>::to_float(Elem<T>::from_float(Elem<T>::to_float(Elem<T>::from_float(a[u] * inv)) * w.x));
        b[u] = Elem<T>::to_float(Elem<T>::from_float(Elem<T>::to_float(Elem<T>::from_float(b[u] * inv)) * w.y));
      }
    }
  }
  const float* f = freqs + (size_t)(pos0 + tok) * pairs * 2;
#pragma unroll
  for (int u = 0; u < 2; ++u) {
    const int p = lane + 32 * u;
    if (p < pairs) {
      const float2 cs = *reinterpret_cast<const float2*>(f + 2 * p);
      PairIO<T>::store(dst + 2 * p, a[u] * cs.x - b[u] * cs.y, a[u] * cs.y + b[u] * cs.x);
    }
  }
}

// Eight consecutive elements as four packed pairs.  The half types stay packed in registers (one
// 16-byte access) and are widened pair by pair where fp32 arithmetic needs them; "normalised value
// times weight, rounded" is one packed multiply (the fp32 product of two half-precision numbers is
// exact, so rounding it once is what the packed instruction does).  The single-element
// conversions are avoided throughout: they run on the quarter-rate conversion pipe, which was the
// busiest unit of the kernel when it used them (64 % against 47 % of the DRAM bandwidth).
template <typename T> struct Pairs;
template <> struct Pairs<float> {
  using P = float2;
  static __device__ __forceinline__ void load(const float* p, P (&v)[4]) {
    const float4 a = __ldg(reinterpret_cast<const float4*>(p)), b = __ldg(reinterpret_cast<const float4*>(p) + 1);
    v[0] = make_float2(a.x, a.y); v[1] = make_float2(a.z, a.w); v[2] = make_float2(b.x, b.y); v[3] = make_float2(b.z, b.w);
  }
  static __device__ __forceinline__ void store(float* p, const P (&v)[4]) {
    reinterpret_cast<float4*>(p)[0] = make_float4(v[0].x, v[0].y, v[1].x, v[1].y);
    reinterpret_cast<float4*>(p)[1] = make_float4(v[2].x, v[2].y, v[3].x, v[3].y);
  }
  static __device__ __forceinline__ P zero() { return make_float2(0.f, 0.f); }
  static __device__ __forceinline__ float2 widen(P v) { return v; }
  static __device__ __forceinline__ P narrow(float a, float b) { return make_float2(a, b); }
  static __device__ __forceinline__ P mul(P a, P b) { return make_float2(a.x * b.x, a.y * b.y); }
};
template <> struct Pairs<__half> {
  using P = __half2;
  static __device__ __forceinline__ void load(const __half* p, P (&v)[4]) {
    const uint4 q = __ldg(reinterpret_cast<const uint4*>(p));
    v[0] = *reinterpret_cast<const P*>(&q.x); v[1] = *reinterpret_cast<const P*>(&q.y);
    v[2] = *reinterpret_cast<const P*>(&q.z); v[3] = *reinterpret_cast<const P*>(&q.w);
  }
  static __device__ __forceinline__ void store(__half* p, const P (&v)[4]) {
    *reinterpret_cast<uint4*>(p) = make_uint4(*reinterpret_cast<const uint32_t*>(&v[0]), *reinterpret_cast<const uint32_t*>(&v[1]),
                                              *reinterpret_cast<const uint32_t*>(&v[2]), *reinterpret_cast<const uint32_t*>(&v[3]));
  }
  static __device__ __forceinline__ P zero() { return __floats2half2_rn(0.f, 0.f); }
  static __device__ __forceinline__ float2 widen(P v) { return __half22float2(v); }
  static __device__ __forceinline__ P narrow(float a, float b) { return __floats2half2_rn(a, b); }
  static __device__ __forceinline__ P mul(P a, P b) { return __hmul2(a, b); }
};
template <> struct Pairs<__nv_bfloat16> {
  using P = __nv_bfloat162;
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, P (&v)[4]) {
    const uint4 q = __ldg(reinterpret_cast<const uint4*>(p));
    v[0] = *reinterpret_cast<const P*>(&q.x); v[1] = *reinterpret_cast<const P*>(&q.y);
    v[2] = *reinterpret_cast<const P*>(&q.z); v[3] = *reinterpret_cast<const P*>(&q.w);
  }
  static __device__ __forceinline__ void store(__nv_bfloat16* p, const P (&v)[4]) {
    *reinterpret_cast<uint4*>(p) = make_uint4(*reinterpret_cast<const uint32_t*>(&v[0]), *reinterpret_cast<const uint32_t*>(&v[1]),
                                              *reinterpret_cast<const uint32_t*>(&v[2]), *reinterpret_cast<const uint32_t*>(&v[3]));
  }
  static __device__ __forceinline__ P zero() { return __floats2bfloat162_rn(0.f, 0.f); }
  static __device__ __forceinline__ float2 widen(P v) {
    const uint32_t w = *reinterpret_cast<const uint32_t*>(&v);
    return make_float2(__uint_as_float(w << 16), __uint_as_float(w & 0xffff0000u));
  }
  static __device__ __forceinline__ P narrow(float a, float b) { return __floats2bfloat162_rn(a, b); }
  static __device__ __forceinline__ P mul(P a, P b) { return __hmul2(a, b); }
};

constexpr int kPrepThreads = 256;
constexpr int kPrepHeads = 4;      // heads a lane group walks over for its token

// G lanes per token (8 when d <= 64, else 16), eight elements per lane.  One-dimensional grid with
// the head blocks of a token block next to one another, so that the CTAs running at one time read
// whole rows of x and write long runs of every head
// kFast: every CTA is full (n_tok a multiple of the tokens per CTA, H of kPrepHeads, d = 8 G) and
// the normalisation, when there is one, covers every token; the guards and the selects they turn
// into are then compiled out (they were a third of the instructions of an issue-bound kernel).
template <typename T, int G, bool kFast>
__global__ void __launch_bounds__(kPrepThreads)
qk_norm_rope_vec8_kernel(const T* __restrict__ x, const T* __restrict__ weight, const float* __restrict__ freqs,
                         T* __restrict__ out, int n_tok, int H, int d, int pos0, int norm_from, float eps) {
  using PR = Pairs<T>;
  using P = typename PR::P;
  const unsigned head_blocks = (unsigned)(H + kPrepHeads - 1) / kPrepHeads;
  const int sub = threadIdx.x % G;
  const int tok = (int)(blockIdx.x / head_blocks) * (kPrepThreads / G) + threadIdx.x / G;
  const int h0 = (int)(blockIdx.x % head_blocks) * kPrepHeads;
  const bool active = kFast || (tok < n_tok && sub * 8 < d);      // the shuffles below need every lane of the warp
  const bool norm = weight != nullptr && (kFast || tok >= norm_from);
  const float inv_d = 1.f / (float)d;

  P v[kPrepHeads][4];
  const T* src = x + ((size_t)tok * H + h0) * d + sub * 8;
#pragma unroll
  for (int i = 0; i < kPrepHeads; ++i) {
    if (kFast || (active && h0 + i < H)) {
      PR::load(src + (size_t)i * d, v[i]);
    } else {
#pragma unroll
      for (int q = 0; q < 4; ++q) v[i][q] = PR::zero();
    }
  }
  float cs[8];                // (cos, sin) of this lane's four pairs
  P w[4];                     // its eight weights
  if (active) {
    const float4* f = reinterpret_cast<const float4*>(freqs + ((size_t)(pos0 + tok) * (d >> 1) + sub * 4) * 2);
    const float4 f0 = __ldg(f), f1 = __ldg(f + 1);
    cs[0] = f0.x; cs[1] = f0.y; cs[2] = f0.z; cs[3] = f0.w; cs[4] = f1.x; cs[5] = f1.y; cs[6] = f1.z; cs[7] = f1.w;
    if (norm) PR::load(weight + sub * 8, w);
  }
  T* dst = out + ((size_t)h0 * n_tok + tok) * d + sub * 8;
#pragma unroll
  for (int i = 0; i < kPrepHeads; ++i) {
    float2 e[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) e[q] = PR::widen(v[i][q]);
    if (weight != nullptr) {   // uniform over the grid: every lane of the warp takes part in the shuffles
      float ss = 0.f;
#pragma unroll
      for (int q = 0; q < 4; ++q) ss += e[q].x * e[q].x + e[q].y * e[q].y;
#pragma unroll
      for (int o = G / 2; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);   // stays inside the lane group
      const float inv = rsqrtf(ss * inv_d + eps);
      if (norm && active) {
#pragma unroll
        for (int q = 0; q < 4; ++q) e[q] = PR::widen(PR::mul(PR::narrow(e[q].x * inv, e[q].y * inv), w[q]));
      }
    }
    if (kFast || (active && h0 + i < H)) {
      P r[4];
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const float c = cs[2 * q], sn = cs[2 * q + 1];
        r[q] = PR::narrow(e[q].x * c - e[q].y * sn, e[q].x * sn + e[q].y * c);
      }
      PR::store(dst + (size_t)i * n_tok * d, r);
    }
  }
}

template <typename T>
static void launch_vec8(const void* x, const void* weight, const float* freqs, void* out, int n_tok, int H, int d, int pos0,
                        int norm_from, float eps, cudaStream_t s) {
  const int G = d <= 64 ? 8 : 16;
  const int tok_per_cta = kPrepThreads / G;
  const unsigned grid = (unsigned)((n_tok + tok_per_cta - 1) / tok_per_cta) * (unsigned)((H + kPrepHeads - 1) / kPrepHeads);
  const bool fast = n_tok % tok_per_cta == 0 && H % kPrepHeads == 0 && d == 8 * G && (weight == nullptr || norm_from <= 0);
  auto go = [&](auto kern) {
    kern<<<grid, kPrepThreads, 0, s>>>((const T*)x, (const T*)weight, freqs, (T*)out, n_tok, H, d, pos0, norm_from, eps);
  };
  if (G == 8) { if (fast) go(qk_norm_rope_vec8_kernel<T, 8, true>); else go(qk_norm_rope_vec8_kernel<T, 8, false>); }
  else        { if (fast) go(qk_norm_rope_vec8_kernel<T, 16, true>); else go(qk_norm_rope_vec8_kernel<T, 16, false>); }
}

}  // namespace attn

extern "C" int attn_b200_qk_norm_rope(const void* x, const void* weight, const float* freqs, void* out, int32_t n_tok,
                                      int32_t H, int32_t d, int32_t pos0, int32_t norm_from, float eps, int32_t dtype,
                                      void* stream) {
  if (n_tok < 0 || H < 0 || d <= 0 || (d & 1) || d > 128 || pos0 < 0) return ATTN_EINVAL;
  if (dtype != ATTN_F16 && dtype != ATTN_BF16 && dtype != ATTN_F32) return ATTN_EUNSUPPORTED;
  const long long vecs = (long long)n_tok * H;
  if (vecs == 0) return ATTN_OK;
  if (x == nullptr || freqs == nullptr || out == nullptr) return ATTN_EINVAL;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  auto aligned16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; };
  const long long vec8_ctas = ((long long)n_tok + 15) / 16 * ((H + attn::kPrepHeads - 1) / attn::kPrepHeads);
  if (d % 8 == 0 && aligned16(x) && aligned16(out) && aligned16(freqs) && aligned16(weight) && vec8_ctas <= 0x7fffffffLL) {
    if (dtype == ATTN_BF16) attn::launch_vec8<__nv_bfloat16>(x, weight, freqs, out, n_tok, H, d, pos0, norm_from, eps, s);
    else if (dtype == ATTN_F16) attn::launch_vec8<__half>(x, weight, freqs, out, n_tok, H, d, pos0, norm_from, eps, s);
    else attn::launch_vec8<float>(x, weight, freqs, out, n_tok, H, d, pos0, norm_from, eps, s);
    return cudaGetLastError() == cudaSuccess ? ATTN_OK : ATTN_ECUDA;
  }
  if ((vecs + 7) / 8 > 0x7fffffffLL) return ATTN_ETOOLARGE;
  const unsigned blocks = (unsigned)((vecs + 7) / 8);
  if (dtype == ATTN_BF16)
    attn::qk_norm_rope_kernel<__nv_bfloat16><<<blocks, 256, 0, s>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)weight, freqs,
                                                                   (__nv_bfloat16*)out, n_tok, H, d, pos0, norm_from, eps);
  else if (dtype == ATTN_F16)
    attn::qk_norm_rope_kernel<__half><<<blocks, 256, 0, s>>>((const __half*)x, (const __half*)weight, freqs, (__half*)out, n_tok, H, d,
                                                             pos0, norm_from, eps);
  else
    attn::qk_norm_rope_kernel<float><<<blocks, 256, 0, s>>>((const float*)x, (const float*)weight, freqs, (float*)out, n_tok, H, d, pos0,
                                                            norm_from, eps);
  return cudaGetLastError() == cudaSuccess ? ATTN_OK : ATTN_ECUDA;
}
