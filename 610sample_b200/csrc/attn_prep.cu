// Step before the attention kernels, fused: per-head RMS normalisation of Q / K rows, rotary
// position embedding, and the change of layout from the projections' [T, H, d] to the kernels'
// [1, H, T, d], in one pass over the data (the reference does these as separate eager PyTorch
// operations followed by permute + contiguous: e2e/ttt_pytorch/model.py:76-84, 96-116, 260-263,
// 309-316, 182-184).  One warp per (token, head) vector; arithmetic in fp32 with the reference's
// rounding points: (x * rsqrt(mean(x^2) + eps)) rounded to the input type, times the weight rounded
// again, rotated pairwise by (cos, sin) of the position in fp32, rounded.
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
