// Host side of the tensor-core (tcgen05 / TMEM / TMA) attention kernels on sm_100a:
// tensor-map encoding, dispatch of the forward / backward / double-backward launches to the
// kernel files (attn_tc_fwd.cu, attn_tc_fb.cu, attn_tc_hvp_row.cu, attn_tc_hvp_col.cu), the row-dot helper of
// the first backward and the tcgen05 primitive self-test.
#include "attn_common.cuh"
#include "attn_launch.h"
#include "tc_common.cuh"

#include <cstdio>
#include <cstring>
#include <mutex>

namespace attn {
namespace tc {

// ---------------------------------------------------------------------------
// D_i = sum_d dO * O, used by the first backward.  Reference: csrc/flash_double_backward_v7.cu:721-739.
// Bound by HBM traffic (one read of dO and of O): G lanes own a row, a lane eight consecutive
// elements of it (one 16-byte load per tensor), and every lane group walks over kRowdotRows rows
// with all its loads in flight.  D is a multiple of 16, so every 16-byte load is aligned.
// ---------------------------------------------------------------------------
constexpr int kRowdotRows = 4;

template <typename T> __device__ __forceinline__ float2 widen_pair(uint32_t w);
template <> __device__ __forceinline__ float2 widen_pair<__nv_bfloat16>(uint32_t w) {
  return make_float2(__uint_as_float(w << 16), __uint_as_float(w & 0xffff0000u));
}
template <> __device__ __forceinline__ float2 widen_pair<__half>(uint32_t w) {
  return __half22float2(*reinterpret_cast<const __half2*>(&w));
}

template <typename T, int G>
__global__ void __launch_bounds__(256)
rowdot_kernel(const T* __restrict__ a, const T* __restrict__ b, float* __restrict__ out, long long rows, int D) {
  const int sub = threadIdx.x % G;
  const long long r0 = ((long long)blockIdx.x * (256 / G) + threadIdx.x / G) * kRowdotRows;
  const bool lane_on = sub * 8 < D;
  uint4 va[kRowdotRows], vb[kRowdotRows];
#pragma unroll
  for (int i = 0; i < kRowdotRows; ++i) {
    va[i] = vb[i] = make_uint4(0u, 0u, 0u, 0u);
    if (lane_on && r0 + i < rows) {
      va[i] = __ldg(reinterpret_cast<const uint4*>(a + (r0 + i) * D + sub * 8));
      vb[i] = __ldg(reinterpret_cast<const uint4*>(b + (r0 + i) * D + sub * 8));
    }
  }
#pragma unroll
  for (int i = 0; i < kRowdotRows; ++i) {
    const uint32_t wa[4] = {va[i].x, va[i].y, va[i].z, va[i].w}, wb[4] = {vb[i].x, vb[i].y, vb[i].z, vb[i].w};
    float acc = 0.f;
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const float2 x = widen_pair<T>(wa[q]), y = widen_pair<T>(wb[q]);
      acc = fmaf(x.x, y.x, acc);
      acc = fmaf(x.y, y.y, acc);
    }
#pragma unroll
    for (int o = G / 2; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);   // every lane of the warp takes part
    if (sub == 0 && r0 + i < rows) out[r0 + i] = acc;
  }
}

template <typename T>
static cudaError_t launch_rowdot(const T* a, const T* b, float* out, long long rows, int D, cudaStream_t s) {
  const int G = D <= 32 ? 4 : D <= 64 ? 8 : 16;
  const long long rows_per_cta = (long long)(256 / G) * kRowdotRows;
  const long long ctas = (rows + rows_per_cta - 1) / rows_per_cta;
  if (ctas > 0x7fffffffLL) return cudaErrorInvalidValue;
  if (G == 4) rowdot_kernel<T, 4><<<(unsigned)ctas, 256, 0, s>>>(a, b, out, rows, D);
  else if (G == 8) rowdot_kernel<T, 8><<<(unsigned)ctas, 256, 0, s>>>(a, b, out, rows, D);
  else rowdot_kernel<T, 16><<<(unsigned)ctas, 256, 0, s>>>(a, b, out, rows, D);
  return cudaGetLastError();
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
  const bool timeout_test = (flags & 8) != 0;
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
  if (timeout_test) {
    // Exercise of the time-out path: thread 0 waits, with a limit of about a millisecond, on a
    // barrier nothing will ever arrive on.  It stores its code in the status word and raises the
    // abort flag; the other threads leave their wait below through that flag, and everybody goes
    // through the common teardown, which frees the tensor memory.  Nothing is computed.
    if (threadIdx.x == 0) (void)mbar_wait_limit(bar_full, 0, abort_flag, status, 0x7003u, 1000000LL);
  } else
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
                       long long cols, int box_rows = 64) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) {
    snprintf(tl_encode_error, sizeof(tl_encode_error), "driver entry point cuTensorMapEncodeTiled not found");
    return false;
  }
  cuuint64_t dims[3] = {(cuuint64_t)cols, (cuuint64_t)rows, (cuuint64_t)planes};
  cuuint64_t strides[2] = {(cuuint64_t)cols * 2, (cuuint64_t)rows * (cuuint64_t)cols * 2};
  cuuint32_t box[3] = {64, (cuuint32_t)box_rows, 1};
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

bool encode_all_maps(TmaMaps* maps, int op, const Geometry& g, const Tensors& t, int is_bf16, const char** err) {
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
  // outputs of this operation, stored by TMA in boxes of 64 columns x 128 rows
  void* outs[TO_COUNT] = {nullptr, nullptr, nullptr, nullptr};
  int out_rows[TO_COUNT] = {g.N_q, g.N_q, g.N_kv, g.N_kv};
  if (op == OP_FORWARD) {
    outs[TO_O] = t.out_O;
  } else if (op == OP_BACKWARD) {
    outs[TO_dQ] = t.out_dQ; outs[TO_dK] = t.out_dK; outs[TO_dV] = t.out_dV;
    out_rows[TO_dK] = g.N_kv; out_rows[TO_dV] = g.N_kv;
  } else {
    outs[TO_gdO] = t.out_g_dO; outs[TO_gQ] = t.out_g_Q; outs[TO_gK] = t.out_g_K; outs[TO_gV] = t.out_g_V;
  }
  for (int i = 0; i < TO_COUNT; ++i) {
    void* p = outs[i] ? outs[i] : const_cast<void*>(t.Q);
    const int r = outs[i] ? out_rows[i] : g.N_q;
    if (!encode_map(&maps->out[i], p, is_bf16, g.BH, r, g.D, 128)) {
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

cudaError_t launch_fwd_bwd(int kind, int D, int is_bf16, const TmaMaps& maps, const Geometry& g, const Tensors& t,
                           cudaStream_t s);
cudaError_t launch_fwd(int D, int is_bf16, const TmaMaps& maps, const Geometry& g, const Tensors& t, cudaStream_t s);

// Kernels of one operation that do not depend on one another (g_Q and g_K/g_V of the double
// backward; dQ and dK/dV of the backward) run side by side: the second is launched on a helper
// stream of the device between an event fork and an event join on the caller's stream, so the
// SMs that one kernel's last CTAs leave idle take CTAs of the other.  One helper stream and two
// events per device, created on first use and shared by every caller stream and host thread (the
// mutex covers one fork ... join enqueue).  A stream that is being captured is never forked: a
// capture would pull the shared helper stream into the graph until the capture ends, long after
// the mutex is released, and an eager call of another thread in that window would either
// invalidate the capture or be merged into it.  Under capture, and whenever the helper cannot be
// had, both launches stay on the caller's stream.
struct Helper {
  cudaStream_t stream = nullptr;
  cudaEvent_t fork = nullptr, join = nullptr;
  bool tried = false;
  std::mutex in_use;   // host threads share the events: one fork ... join sequence at a time
};

static Helper* helper_for_current_device() {
  static Helper helpers[64];
  static std::mutex mu;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  std::lock_guard<std::mutex> lock(mu);
  Helper& h = helpers[dev];
  if (!h.tried) {
    h.tried = true;
    if (cudaStreamCreateWithFlags(&h.stream, cudaStreamNonBlocking) != cudaSuccess ||
        cudaEventCreateWithFlags(&h.fork, cudaEventDisableTiming) != cudaSuccess ||
        cudaEventCreateWithFlags(&h.join, cudaEventDisableTiming) != cudaSuccess) {
      (void)cudaGetLastError();
      h.stream = nullptr;
    }
  }
  return h.stream != nullptr ? &h : nullptr;
}

// first(s) and second(helper stream) between fork and join; serial on s without a helper
template <typename F1, typename F2>
static cudaError_t run_side_by_side(cudaStream_t s, bool allow_helper, F1 first, F2 second) {
  if (allow_helper) {
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(s, &cap) != cudaSuccess) {   // e.g. the legacy stream while another stream captures
      (void)cudaGetLastError();
      allow_helper = false;
    } else if (cap != cudaStreamCaptureStatusNone) {
      allow_helper = false;
    }
  }
  Helper* h = allow_helper ? helper_for_current_device() : nullptr;
  if (h == nullptr) {
    cudaError_t e = first(s);
    return e == cudaSuccess ? second(s) : e;
  }
  std::lock_guard<std::mutex> lock(h->in_use);
  if (cudaEventRecord(h->fork, s) != cudaSuccess || cudaStreamWaitEvent(h->stream, h->fork, 0) != cudaSuccess) {
    (void)cudaGetLastError();
    cudaError_t e = first(s);
    return e == cudaSuccess ? second(s) : e;
  }
  cudaError_t e1 = first(s);
  cudaError_t e2 = second(h->stream);
  // the join is made even after a failed launch, so that the helper stream never outlives the call
  cudaError_t ej = cudaEventRecord(h->join, h->stream);
  if (ej == cudaSuccess) ej = cudaStreamWaitEvent(s, h->join, 0);
  return e1 != cudaSuccess ? e1 : e2 != cudaSuccess ? e2 : ej;
}

template <typename T>
static cudaError_t launch_op(int op, const TmaMaps& maps, const Geometry& g, const Tensors& t, cudaStream_t s,
                             int* n, int phases) {
  cudaError_t e = cudaSuccess;
  const int D = g.D, bf = Pack<T>::kIsBf16;
  *n = 0;
  if (op == OP_FORWARD) {
    e = launch_fwd(D, bf, maps, g, t, s);                              // O and L in one pass (online softmax)
    *n = 1;
  } else if (op == OP_BACKWARD) {
    const long long rows = (long long)g.BH * g.N_q;
    if (rows > 0) {
      e = launch_rowdot<T>((const T*)t.dO, (const T*)t.O, t.Dv, rows, g.D, s);
    }
    if (e == cudaSuccess)
      e = run_side_by_side(s, true,
                           [&](cudaStream_t q) { return launch_fwd_bwd(2, D, bf, maps, g, t, q); },     // dQ
                           [&](cudaStream_t q) { return launch_fwd_bwd(3, D, bf, maps, g, t, q); });    // dK, dV
    *n = 3;
  } else {
    if (phases & HVP_PHASE_PRE) { e = launch_hvp_row(0, D, bf, maps, g, t, s); ++*n; }                        // scalars + g_dO
    const bool row = (phases & HVP_PHASE_ROW) != 0, col = (phases & HVP_PHASE_COL) != 0;
    if (e == cudaSuccess && row && col) {
      e = run_side_by_side(s, (phases & HVP_PHASE_SERIAL) == 0,
                           [&](cudaStream_t q) { return launch_hvp_col(D, bf, maps, g, t, q); },        // g_K, g_V
                           [&](cudaStream_t q) { return launch_hvp_row(1, D, bf, maps, g, t, q); });    // g_Q
      *n += 2;
    } else {
      if (e == cudaSuccess && row) { e = launch_hvp_row(1, D, bf, maps, g, t, s); ++*n; }  // g_Q
      if (e == cudaSuccess && col) { e = launch_hvp_col(D, bf, maps, g, t, s); ++*n; }     // g_K, g_V
    }
  }
  return e;
}

}  // namespace tc

// Head dimensions that are not 64 or 128 run in the next larger of the two tile widths: the TMA
// loads fill the padding columns with zeros and the epilogues store g.D columns only.
bool tc_supported(int dtype, int D) { return (dtype == 0 || dtype == 1) && D >= 16 && D <= 128 && D % 16 == 0; }

cudaError_t launch_tc(int op, int dtype, const Geometry& g, const Tensors& t, cudaStream_t s, int* launches,
                      const char** err, int phases) {
  using namespace tc;
  *err = nullptr;
  TmaMaps maps;
  const int bf = dtype == 1;
  if (!encode_all_maps(&maps, op, g, t, bf, err)) return cudaErrorInvalidValue;
  return bf ? launch_op<__nv_bfloat16>(op, maps, g, t, s, launches, phases)
            : launch_op<__half>(op, maps, g, t, s, launches, phases);
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
