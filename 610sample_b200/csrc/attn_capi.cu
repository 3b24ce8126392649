// C ABI of libattn_b200.so (see include/attn_b200.h): argument checks, geometry,
// kernel-family dispatch, per-thread error text and the device status word.
#include "attn_b200.h"
#include "attn_launch.h"
#include "tc_primitives.cuh"

#include <cmath>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>

namespace {

thread_local char tl_error[512] = "";
thread_local int tl_launches = 0;

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(tl_error, sizeof(tl_error), fmt, ap);
  va_end(ap);
  return code;
}

// One status block per device, in device global memory owned by this library; the status word
// is its first member.
__device__ attn::tc::StatusBlock g_status_block = {0u, 0u, nullptr};

constexpr int kMaxDevices = 64;
unsigned int* g_status_ptr[kMaxDevices] = {nullptr};
std::mutex g_status_mutex;

int status_pointer(unsigned int** out) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return fail(ATTN_ECUDA, "cudaGetDevice: %s", cudaGetErrorString(e));
  if (dev < 0 || dev >= kMaxDevices) return fail(ATTN_EINVAL, "device index %d out of range", dev);
  std::lock_guard<std::mutex> lock(g_status_mutex);
  if (g_status_ptr[dev] == nullptr) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_status_block);
    if (e != cudaSuccess) return fail(ATTN_ECUDA, "cudaGetSymbolAddress: %s", cudaGetErrorString(e));
    g_status_ptr[dev] = static_cast<unsigned int*>(p);
  }
  *out = g_status_ptr[dev];
  return ATTN_OK;
}

int check_shape(const attn_shape_t* s) {
  if (s == nullptr) return fail(ATTN_EINVAL, "shape is null");
  if (s->B < 0 || s->H < 0 || s->N_q < 0 || s->N_kv < 0) return fail(ATTN_EINVAL, "negative size");
  if (s->dtype != ATTN_F16 && s->dtype != ATTN_BF16 && s->dtype != ATTN_F32)
    return fail(ATTN_EUNSUPPORTED, "dtype %d: expected ATTN_F16, ATTN_BF16 or ATTN_F32", s->dtype);
  if (s->D <= 0 || s->D % 16 != 0) return fail(ATTN_EINVAL, "D must be a positive multiple of 16 (got %d)", s->D);
  if (s->D > 128) return fail(ATTN_EUNSUPPORTED, "unsupported head dimension D=%d (maximum 128)", s->D);
  if (s->mask_mode != ATTN_MASK_REFERENCE && s->mask_mode != ATTN_MASK_NONE)
    return fail(ATTN_EINVAL, "mask_mode %d unknown", s->mask_mode);
  if (s->window_size < 0) return fail(ATTN_EINVAL, "window_size must be >= 0");
  if (s->chunk_id < 0) return fail(ATTN_EINVAL, "chunk_id must be >= 0");
  if ((long long)s->chunk_id * s->N_q + s->N_q > (1LL << 30)) return fail(ATTN_EINVAL, "chunk_id * N_q too large");
  if ((long long)s->B * s->H > (1LL << 24)) return fail(ATTN_EINVAL, "B * H too large");
  if (s->impl < ATTN_IMPL_AUTO || s->impl > ATTN_IMPL_TENSOR) return fail(ATTN_EINVAL, "impl %d unknown", s->impl);
  if (s->impl == ATTN_IMPL_TENSOR && !attn::tc_supported(s->dtype, s->D))
    return fail(ATTN_EUNSUPPORTED, "tensor-core kernels need f16 or bf16 inputs");
  return ATTN_OK;
}

bool shape_is_empty(const attn_shape_t* s) { return s->B == 0 || s->H == 0 || s->N_q == 0 || s->N_kv == 0; }

attn::Geometry make_geometry(const attn_shape_t* s) {
  attn::Geometry g;
  g.BH = s->B * s->H;
  g.N_q = s->N_q;
  g.N_kv = s->N_kv;
  g.D = s->D;
  g.qi_base = s->chunk_id * s->N_q;
  g.ki_base = s->chunk_id * s->N_q + s->N_q - s->N_kv;
  g.window = s->window_size > (1 << 30) ? (1 << 30) : s->window_size;
  g.mask_mode = s->mask_mode;
  g.head_group = 1;
  g.scale = 1.0f / sqrtf((float)s->D);
  g.scale_log2e = g.scale * attn::kLog2e;
  return g;
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// Empty problems (N_q == 0 or N_kv == 0) launch no attention kernel: whatever outputs exist
// are all-masked, i.e. zero, and L is -inf.
__global__ void fill_f32_kernel(float* p, size_t n, float v) {
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) p[i] = v;
}

cudaError_t fill_zero(void* p, size_t elems, int dtype, cudaStream_t s) {
  if (p == nullptr || elems == 0) return cudaSuccess;
  return cudaMemsetAsync(p, 0, elems * (dtype == ATTN_F32 ? 4 : 2), s);
}

int run_empty(int op, const attn_shape_t* s, attn::Tensors& t, cudaStream_t cs) {
  const size_t nq = (size_t)s->B * s->H * s->N_q * s->D, nkv = (size_t)s->B * s->H * s->N_kv * s->D;
  cudaError_t e = cudaSuccess;
  void* q_outs[] = {t.out_O, t.out_dQ, t.out_g_dO, t.out_g_Q};
  void* kv_outs[] = {t.out_dK, t.out_dV, t.out_g_K, t.out_g_V};
  for (void* p : q_outs) if (e == cudaSuccess) e = fill_zero(p, nq, s->dtype, cs);
  for (void* p : kv_outs) if (e == cudaSuccess) e = fill_zero(p, nkv, s->dtype, cs);
  const size_t rows = (size_t)s->B * s->H * s->N_q;
  if (e == cudaSuccess && op == attn::OP_FORWARD && t.out_L != nullptr && rows > 0) {
    fill_f32_kernel<<<(unsigned)((rows + 255) / 256 > 1024 ? 1024 : (rows + 255) / 256), 256, 0, cs>>>(t.out_L, rows, -INFINITY);
    e = cudaGetLastError();
    tl_launches = 1;
  }
  if (e != cudaSuccess) return fail(ATTN_ECUDA, "empty-problem fill failed: %s", cudaGetErrorString(e));
  tl_error[0] = 0;
  return ATTN_OK;
}

int run(int op, const attn_shape_t* s, attn::Tensors& t, void* stream, int phases = attn::HVP_PHASE_ALL) {
  const attn::Geometry g = make_geometry(s);
  tl_launches = 0;
  if (g.BH == 0 || (g.N_q == 0 && g.N_kv == 0)) return ATTN_OK;
  if (g.N_q == 0 || g.N_kv == 0) return run_empty(op, s, t, static_cast<cudaStream_t>(stream));
  // Bind the device's primary context to this host thread.  Tensor-map encoding is a
  // driver call and fails with "invalid context" on a thread that has made no runtime
  // call yet (e.g. a freshly started autograd worker thread).  cudaSetDevice on the current
  // device does that and, unlike a null cudaFree, is legal while a stream is being captured.
  {
    int dev = 0;
    cudaError_t e0 = cudaGetDevice(&dev);
    if (e0 == cudaSuccess) e0 = cudaSetDevice(dev);
    if (e0 != cudaSuccess) return fail(ATTN_ECUDA, "binding the device context: %s", cudaGetErrorString(e0));
  }
  int rc = status_pointer(&t.status);
  if (rc != ATTN_OK) return rc;
  const bool use_tc = s->impl == ATTN_IMPL_TENSOR ||
                      (s->impl == ATTN_IMPL_AUTO && attn::tc_supported(s->dtype, s->D));
  cudaStream_t cs = static_cast<cudaStream_t>(stream);
  cudaError_t e;
  if (use_tc) {
    const char* why = nullptr;
    e = attn::launch_tc(op, s->dtype, g, t, cs, &tl_launches, &why, phases);
    if (e != cudaSuccess)
      return fail(ATTN_ECUDA, "tensor-core launch failed: %s%s%s", cudaGetErrorString(e), why ? ": " : "", why ? why : "");
  } else {
    e = attn::launch_simt(op, s->dtype, g, t, cs, &tl_launches, phases);
    if (e != cudaSuccess) return fail(ATTN_ECUDA, "SIMT launch failed: %s", cudaGetErrorString(e));
  }
  tl_error[0] = 0;
  return ATTN_OK;
}

// A tensor without elements (B, H, N or the other side's N is 0) may be passed as null.
#define REQUIRE_PTR(p)                                                                        \
  do {                                                                                        \
    if ((p) == nullptr) {                                                                     \
      if (!shape_is_empty(shape)) return fail(ATTN_EINVAL, #p " is null");                    \
    } else if (!aligned16(p)) return fail(ATTN_EINVAL, #p " is not 16-byte aligned");          \
  } while (0)

}  // namespace

extern "C" {

int attn_b200_forward(const attn_shape_t* shape, const void* Q, const void* K, const void* V, void* O,
                      float* L, void* stream) {
  int rc = check_shape(shape);
  if (rc != ATTN_OK) return rc;
  REQUIRE_PTR(Q); REQUIRE_PTR(K); REQUIRE_PTR(V); REQUIRE_PTR(O);
  if (L == nullptr && !shape_is_empty(shape)) return fail(ATTN_EINVAL, "L is null");
  attn::Tensors t;
  memset(&t, 0, sizeof(t));
  t.Q = Q; t.K = K; t.V = V; t.out_O = O; t.out_L = L;
  return run(attn::OP_FORWARD, shape, t, stream);
}

size_t attn_b200_backward_scratch_bytes(const attn_shape_t* s) {
  if (s == nullptr || s->B < 0 || s->H < 0 || s->N_q < 0) return 0;
  return sizeof(float) * (size_t)s->B * s->H * s->N_q;
}

int attn_b200_backward(const attn_shape_t* shape, const void* dO, const void* Q, const void* K, const void* V,
                       const void* O, const float* L, void* dQ, void* dK, void* dV, float* scratch,
                       void* stream) {
  int rc = check_shape(shape);
  if (rc != ATTN_OK) return rc;
  REQUIRE_PTR(dO); REQUIRE_PTR(Q); REQUIRE_PTR(K); REQUIRE_PTR(V); REQUIRE_PTR(O);
  REQUIRE_PTR(dQ); REQUIRE_PTR(dK); REQUIRE_PTR(dV);
  if (L == nullptr && !shape_is_empty(shape)) return fail(ATTN_EINVAL, "L is null");
  if (scratch == nullptr && !shape_is_empty(shape)) return fail(ATTN_EINVAL, "scratch is null");
  attn::Tensors t;
  memset(&t, 0, sizeof(t));
  t.dO = dO; t.Q = Q; t.K = K; t.V = V; t.O = O; t.L = L;
  t.out_dQ = dQ; t.out_dK = dK; t.out_dV = dV;
  t.Dv = scratch;
  return run(attn::OP_BACKWARD, shape, t, stream);
}

size_t attn_b200_double_backward_scratch_bytes(const attn_shape_t* s) {
  if (s == nullptr || s->B < 0 || s->H < 0 || s->N_q < 0) return 0;
  return 3 * sizeof(float) * (size_t)s->B * s->H * s->N_q;
}

int attn_b200_double_backward(const attn_shape_t* shape, const void* g_dQ, const void* g_dK, const void* g_dV,
                              const void* dO, const void* Q, const void* K, const void* V, const void* O,
                              const float* L, void* g_dO, void* g_Q, void* g_K, void* g_V, float* scratch,
                              void* stream) {
  return attn_b200_double_backward_phases(shape, g_dQ, g_dK, g_dV, dO, Q, K, V, O, L, g_dO, g_Q, g_K, g_V, scratch,
                                          stream, attn::HVP_PHASE_ALL);
}

int attn_b200_double_backward_phases(const attn_shape_t* shape, const void* g_dQ, const void* g_dK,
                                     const void* g_dV, const void* dO, const void* Q, const void* K, const void* V,
                                     const void* O, const float* L, void* g_dO, void* g_Q, void* g_K, void* g_V,
                                     float* scratch, void* stream, int32_t phases) {
  if (phases <= 0 || phases > attn::HVP_PHASE_ALL) return fail(ATTN_EINVAL, "phases must be a mask in 1..7");
  int rc = check_shape(shape);
  if (rc != ATTN_OK) return rc;
  REQUIRE_PTR(g_dQ); REQUIRE_PTR(g_dK); REQUIRE_PTR(g_dV);
  REQUIRE_PTR(dO); REQUIRE_PTR(Q); REQUIRE_PTR(K); REQUIRE_PTR(V); REQUIRE_PTR(O);
  REQUIRE_PTR(g_dO); REQUIRE_PTR(g_Q); REQUIRE_PTR(g_K); REQUIRE_PTR(g_V);
  if (L == nullptr && !shape_is_empty(shape)) return fail(ATTN_EINVAL, "L is null");
  if (scratch == nullptr && !shape_is_empty(shape)) return fail(ATTN_EINVAL, "scratch is null");
  attn::Tensors t;
  memset(&t, 0, sizeof(t));
  t.g_dQ = g_dQ; t.g_dK = g_dK; t.g_dV = g_dV;
  t.dO = dO; t.Q = Q; t.K = K; t.V = V; t.O = O; t.L = L;
  t.out_g_dO = g_dO; t.out_g_Q = g_Q; t.out_g_K = g_K; t.out_g_V = g_V;
  const size_t rows = (size_t)shape->B * shape->H * shape->N_q;
  t.Dv = scratch;
  t.dot2 = scratch + rows;
  t.dot3 = scratch + 2 * rows;
  return run(attn::OP_DOUBLE_BACKWARD, shape, t, stream, phases);
}

// ---------------------------------------------------------------------------
// Double backward for callers that must not allocate
// ---------------------------------------------------------------------------
namespace {

// Per-row scalars (Dv, dot2, dot3) of the double backward for at most
// ATTN_B200_STATIC_SCRATCH_ROWS query rows in total (B * H * N_q), 12 MB.  The array
// belongs to the loaded library image: every GPU that loads the library holds its own
// copy until the process exits.
static __device__ __align__(256) float g_static_hvp_scratch[3 * ATTN_B200_STATIC_SCRATCH_ROWS];

// Device address of the array per device.  In host code the name of a __device__
// variable is only a handle; a kernel needs the address cudaGetSymbolAddress returns
// while the device in question is current.
float* g_static_scratch_ptr[kMaxDevices] = {nullptr};
std::mutex g_static_scratch_mutex;

int static_scratch_pointer(int dev, float** out) {
  std::lock_guard<std::mutex> lock(g_static_scratch_mutex);
  if (g_static_scratch_ptr[dev] == nullptr) {
    void* p = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&p, g_static_hvp_scratch);
    if (e != cudaSuccess)
      return fail(ATTN_ECUDA, "cudaGetSymbolAddress(static scratch): %s", cudaGetErrorString(e));
    g_static_scratch_ptr[dev] = static_cast<float*>(p);
  }
  *out = g_static_scratch_ptr[dev];
  return ATTN_OK;
}

}  // namespace

int attn_b200_double_backward_static(const attn_shape_t* shape, const void* g_dQ, const void* g_dK,
                                     const void* g_dV, const void* dO, const void* Q, const void* K,
                                     const void* V, const void* O, const float* L, void* g_dO, void* g_Q,
                                     void* g_K, void* g_V, void* stream) {
  int rc = check_shape(shape);
  if (rc != ATTN_OK) return rc;
  REQUIRE_PTR(g_dQ); REQUIRE_PTR(g_dK); REQUIRE_PTR(g_dV);
  REQUIRE_PTR(dO); REQUIRE_PTR(Q); REQUIRE_PTR(K); REQUIRE_PTR(V); REQUIRE_PTR(O);
  REQUIRE_PTR(g_dO); REQUIRE_PTR(g_Q); REQUIRE_PTR(g_K); REQUIRE_PTR(g_V);
  if (L == nullptr && !shape_is_empty(shape)) return fail(ATTN_EINVAL, "L is null");
  const long long rows = (long long)shape->B * shape->H * shape->N_q;
  // an empty problem launches nothing and needs no scratch, whatever its nominal row count
  if (!shape_is_empty(shape) && rows > (long long)ATTN_B200_STATIC_SCRATCH_ROWS)
    return fail(ATTN_ETOOLARGE,
                "B*H*N_q = %lld query rows exceed the built-in scratch of %d rows; use "
                "attn_b200_double_backward with caller-provided scratch",
                rows, (int)ATTN_B200_STATIC_SCRATCH_ROWS);
  attn::Tensors t;
  memset(&t, 0, sizeof(t));
  t.g_dQ = g_dQ; t.g_dK = g_dK; t.g_dV = g_dV;
  t.dO = dO; t.Q = Q; t.K = K; t.V = V; t.O = O; t.L = L;
  t.out_g_dO = g_dO; t.out_g_Q = g_Q; t.out_g_K = g_K; t.out_g_V = g_V;
  if (!shape_is_empty(shape)) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return fail(ATTN_ECUDA, "cudaGetDevice: %s", cudaGetErrorString(e));
    if (dev < 0 || dev >= kMaxDevices) return fail(ATTN_EINVAL, "device index %d out of range", dev);
    float* scratch = nullptr;
    rc = static_scratch_pointer(dev, &scratch);
    if (rc != ATTN_OK) return rc;
    // Nothing in the scratch has to start at zero: the first kernel writes all three
    // scalars of every row in range before the later kernels read them.
    t.Dv = scratch;
    t.dot2 = scratch + (size_t)rows;
    t.dot3 = scratch + 2 * (size_t)rows;
  }
  // the common tail of every entry point (context binding, empty problems, kernel-family
  // dispatch); SERIAL keeps every launch on the caller's stream, so no helper stream is created
  return run(attn::OP_DOUBLE_BACKWARD, shape, t, stream, attn::HVP_PHASE_ALL | attn::HVP_PHASE_SERIAL);
}

int attn_b200_last_launch_count(void) { return tl_launches; }

int attn_b200_device_status(uint32_t* code) {
  unsigned int* p = nullptr;
  int rc = status_pointer(&p);
  if (rc != ATTN_OK) return rc;
  cudaError_t e = cudaDeviceSynchronize();
  if (e != cudaSuccess) return fail(ATTN_ECUDA, "cudaDeviceSynchronize: %s", cudaGetErrorString(e));
  unsigned int v = 0;
  e = cudaMemcpy(&v, p, sizeof(v), cudaMemcpyDeviceToHost);
  if (e != cudaSuccess) return fail(ATTN_ECUDA, "cudaMemcpy: %s", cudaGetErrorString(e));
  if (v != 0u) {
    const unsigned int zero = 0u;
    cudaMemcpy(p, &zero, sizeof(zero), cudaMemcpyHostToDevice);
  }
  if (code != nullptr) *code = v;
  if (v != 0u) return fail(ATTN_EDEVICE, "kernel gave up on a bounded wait (status 0x%x)", v);
  return ATTN_OK;
}

int attn_b200_set_status_mirror(uint32_t* host_word) {
  unsigned int* p = nullptr;
  int rc = status_pointer(&p);
  if (rc != ATTN_OK) return rc;
  unsigned int* dev_view = nullptr;
  if (host_word != nullptr) {
    void* d = nullptr;
    cudaError_t e = cudaHostGetDevicePointer(&d, host_word, 0);
    if (e != cudaSuccess) return fail(ATTN_EINVAL, "host_word is not page-locked, mapped host memory: %s", cudaGetErrorString(e));
    dev_view = static_cast<unsigned int*>(d);
  }
  attn::tc::StatusBlock* blk = reinterpret_cast<attn::tc::StatusBlock*>(p);
  cudaError_t e = cudaMemcpy(&blk->host_mirror, &dev_view, sizeof(dev_view), cudaMemcpyHostToDevice);
  if (e != cudaSuccess) return fail(ATTN_ECUDA, "cudaMemcpy(status mirror): %s", cudaGetErrorString(e));
  return ATTN_OK;
}

const char* attn_b200_last_error(void) { return tl_error; }

const char* attn_b200_version(void) { return "attn_b200 0.1 (sm_100a)"; }

int attn_b200_selftest_gemm(const void* A, const void* B, float* C, int32_t N, int32_t K, int32_t dtype,
                            int32_t flags, void* stream) {
  if (A == nullptr || B == nullptr || C == nullptr) return fail(ATTN_EINVAL, "null pointer");
  if (!aligned16(A) || !aligned16(B)) return fail(ATTN_EINVAL, "operands must be 16-byte aligned");
  if ((N != 64 && N != 128) || (K != 64 && K != 128)) return fail(ATTN_EINVAL, "N and K must be 64 or 128");
  if (dtype != ATTN_F16 && dtype != ATTN_BF16) return fail(ATTN_EUNSUPPORTED, "dtype must be f16 or bf16");
  cudaError_t e0 = cudaFree(nullptr);
  if (e0 != cudaSuccess) return fail(ATTN_ECUDA, "cudaFree(0): %s", cudaGetErrorString(e0));
  unsigned int* status = nullptr;
  int rc = status_pointer(&status);
  if (rc != ATTN_OK) return rc;
  const char* why = nullptr;
  cudaError_t e = attn::launch_tc_selftest(A, B, C, N, K, dtype, flags, status,
                                           static_cast<cudaStream_t>(stream), &why);
  if (e != cudaSuccess)
    return fail(ATTN_ECUDA, "selftest launch failed: %s%s%s", cudaGetErrorString(e), why ? ": " : "", why ? why : "");
  tl_launches = 1;
  return ATTN_OK;
}

}  // extern "C"
