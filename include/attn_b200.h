/*
 * attn_b200.h -- C ABI of the B200 (sm_100a) attention forward / backward /
 * double-backward (Hessian-vector product) library, libattn_b200.so.
 *
 * Every entry point takes plain device pointers and sizes; no framework types
 * cross this boundary.  All tensors are dense row-major:
 *     Q, dO, O, dQ, g_dQ, g_Q, g_dO : [B, H, N_q , D]
 *     K, V, dK, dV, g_dK, g_dV, g_K, g_V : [B, H, N_kv, D]
 *     L : [B, H, N_q] float32, natural-log log-sum-exp of the scaled scores
 * Element type is selected by `dtype` (ATTN_F16 / ATTN_BF16 / ATTN_F32); L and
 * every scratch buffer are always float32.  The softmax scale is 1/sqrt(D).
 *
 * Visibility of key j for query i (mask_mode == ATTN_MASK_REFERENCE):
 *     qi = chunk_id*N_q + i,  ki = chunk_id*N_q + N_q - N_kv + j
 *     visible  <=>  ki >= 0  &&  qi >= ki  &&  qi < ki + window_size
 * which is the predicate of the reference kernels
 * (csrc/flash_double_backward_v7.cu:100-102 with the index bases of :356, :377).
 * mask_mode == ATTN_MASK_NONE makes every pair visible (an extension; the
 * reference cannot express it).  Rows with no visible key give O = 0,
 * L = -inf and zero gradients.
 *
 * Launches are asynchronous on `stream` (a cudaStream_t passed as void*;
 * NULL = the legacy default stream) of the CURRENT device; inputs are never
 * written.  Return value: ATTN_OK or a negative ATTN_E* code;
 * attn_b200_last_error() gives a message for the calling thread.
 *
 * These three functions are what the reference's pybind shim binds
 * (csrc/attention_ext.cpp:4-17: v7_forward_cuda, v7_backward_cuda,
 * v7_double_backward_cuda) with the tensors flattened to pointers + sizes and
 * the outputs / scratch allocated by the caller instead of by ATen
 * (csrc/flash_double_backward_v7.cu:600-601, 1078-1081, 1770-1776).
 */
#ifndef ATTN_B200_H
#define ATTN_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum { ATTN_F16 = 0, ATTN_BF16 = 1, ATTN_F32 = 2 };
enum { ATTN_MASK_REFERENCE = 0, ATTN_MASK_NONE = 1 };
enum {
  ATTN_OK = 0,
  ATTN_EINVAL = -1,      /* bad size / dtype / null pointer / misaligned pointer */
  ATTN_EUNSUPPORTED = -2, /* head dimension or dtype without a kernel */
  ATTN_ECUDA = -3,       /* a CUDA runtime/driver call failed */
  ATTN_EDEVICE = -4,     /* a kernel reported a bounded-wait timeout (see attn_b200_device_status) */
  ATTN_ETOOLARGE = -5    /* problem exceeds a fixed capacity */
};

/* Which kernel family serves a call.  AUTO picks the tcgen05 tensor-core
 * kernels for f16/bf16 inputs (every supported D; head dimensions other than
 * 64 and 128 run zero-padded to the next of the two) and the fp32 SIMT kernels
 * for f32 inputs. */
enum { ATTN_IMPL_AUTO = 0, ATTN_IMPL_SIMT = 1, ATTN_IMPL_TENSOR = 2 };

typedef struct attn_shape {
  int32_t B, H, N_q, N_kv, D;
  int32_t window_size, chunk_id;
  int32_t mask_mode;  /* ATTN_MASK_* */
  int32_t dtype;      /* ATTN_F16 / ATTN_BF16 / ATTN_F32 */
  int32_t impl;       /* ATTN_IMPL_* */
} attn_shape_t;

/* Forward: O = softmax(mask(Q K^T / sqrt(D))) V and L.
 * Replaces v7_forward_cuda (reference csrc/flash_double_backward_v7.cu:619-644,
 * kernel :307-552).  No scratch. */
int attn_b200_forward(const attn_shape_t* shape, const void* Q, const void* K, const void* V,
                      void* O, float* L, void* stream);

/* Bytes of float32 scratch attn_b200_backward needs (B*H*N_q floats: the row
 * term D_i = sum_d dO*O, reference scratch `D_vec`, :1078). */
size_t attn_b200_backward_scratch_bytes(const attn_shape_t* shape);

/* First backward: dQ, dK, dV from dO and the saved (Q, K, V, O, L).
 * Replaces v7_backward_cuda (reference :1113-1138, kernels :649-1016). */
int attn_b200_backward(const attn_shape_t* shape, const void* dO, const void* Q, const void* K,
                       const void* V, const void* O, const float* L, void* dQ, void* dK, void* dV,
                       float* scratch, void* stream);

/* Bytes of float32 scratch attn_b200_double_backward needs (3*B*H*N_q floats:
 * D_i, dot2, dot3 per query row; reference scratch :1770-1772). */
size_t attn_b200_double_backward_scratch_bytes(const attn_shape_t* shape);

/* Double backward (Hessian-vector product).  Given tangents g_dQ, g_dK, g_dV
 * on the first backward's outputs, returns the gradients with respect to dO, Q,
 * K and V (O and L are treated as functions of Q, K, V).  The N_q x N_kv score
 * matrix is never materialised.  D_i is recomputed as sum_j P*dP in float32; the
 * saved O enters only as P V in g_dO = P g_dV + (P o gdS) V - dot2 o O.
 * Replaces v7_double_backward_cuda (reference :1815-1842, kernels :1145-1702);
 * output order as :1809. */
int attn_b200_double_backward(const attn_shape_t* shape, const void* g_dQ, const void* g_dK,
                              const void* g_dV, const void* dO, const void* Q, const void* K,
                              const void* V, const void* O, const float* L, void* g_dO, void* g_Q,
                              void* g_K, void* g_V, float* scratch, void* stream);

/* The same computation restricted to some of its kernels, for profiling one
 * kernel at a time: `phases` is a bit mask of 1 (per-row scalars Dv, dot2, dot3
 * into scratch, and g_dO), 2 (g_Q; needs the scalars in scratch) and 4 (g_K and
 * g_V; needs the scalars too).  7 is attn_b200_double_backward.  In the fp32 CUDA-core
 * family the scalars and both row-side outputs come from ONE kernel, so there masks 1
 * and 2 each run that kernel whole (scalars, g_dO and g_Q are all written).  The reference
 * splits its double backward the same way into kernel A (rows, two passes) and
 * kernel B (columns), csrc/flash_double_backward_v7.cu:1778-1807. */
int attn_b200_double_backward_phases(const attn_shape_t* shape, const void* g_dQ, const void* g_dK,
                                     const void* g_dV, const void* dO, const void* Q, const void* K,
                                     const void* V, const void* O, const float* L, void* g_dO,
                                     void* g_Q, void* g_K, void* g_V, float* scratch, void* stream,
                                     int32_t phases);

/* Double backward without any allocation: same inputs, outputs and results as
 * attn_b200_double_backward, but the per-row scratch lives in a fixed array inside
 * the library instead of being passed in.  It has no counterpart in the reference
 * (whose launcher allocates its scratch through ATen on every call).
 *
 * Who needs it: code that may not call an allocator where the kernel is launched --
 * a host thread inside a real-time or interrupt-like section, a plugin whose host
 * application owns all device memory and forbids cudaMalloc after start-up, a
 * runtime whose memory plan is frozen before execution begins.  This call issues no
 * cudaMalloc / cudaFree and no allocating library routine; the caller still owns Q,
 * K, V, ..., and the four outputs.
 *
 * Limit: B * H * N_q <= ATTN_B200_STATIC_SCRATCH_ROWS (1,048,576 query rows; the
 * array is 12 MB and each GPU that loads the library keeps its copy until the process
 * exits).  Larger problems are rejected with ATTN_ETOOLARGE before anything is
 * launched; use attn_b200_double_backward with your own scratch for those.
 *
 * The first call on a device looks up the device address of the array (one
 * cudaGetSymbolAddress, cached afterwards), and the first launch of each kernel variant
 * (input type x head-dimension class x kernel family) makes the driver load that
 * kernel's code; both are driver-side work at the call site.  So make one warm-up call
 * per variant you will use at start-up, outside any stream capture: from the second
 * call on, nothing is allocated or loaded.  An empty problem (B, H, N_q or N_kv zero)
 * launches nothing and is accepted whatever its row count.
 * All calls on one device share the one array and it keeps whatever the
 * last call left there; nothing in it needs clearing, since each call rewrites every
 * value it later reads.  Because of the sharing, two calls whose kernels can overlap
 * on the GPU (different streams, or different host threads) race on the scratch and
 * corrupt each other: keep calls on one device ordered on one stream. */
#define ATTN_B200_STATIC_SCRATCH_ROWS (1 << 20)
int attn_b200_double_backward_static(const attn_shape_t* shape, const void* g_dQ, const void* g_dK,
                                     const void* g_dV, const void* dO, const void* Q, const void* K,
                                     const void* V, const void* O, const float* L, void* g_dO,
                                     void* g_Q, void* g_K, void* g_V, void* stream);

/* The step in front of the attention calls, fused into one pass: per-(token, head) RMS
 * normalisation with a learned weight, rotary position embedding, and the layout change
 * from the projections' [n_tok, H, d] to the kernels' [1, H, n_tok, d].  The reference does
 * these as separate eager operations followed by permute + contiguous
 * (e2e/ttt_pytorch/model.py:76-84 RMSNorm, :96-116 apply_rotary_emb, :260-263 and
 * :309-316 their use, :182-184 the permutes).  x: [n_tok, H, d] contiguous; weight: [d] in
 * the input type, or NULL for no normalisation; rows below `norm_from` are rotated only
 * (keys that come from the cache are stored normalised); freqs: float32
 * [positions, d/2, 2] = (cos, sin) of position * theta^(-2i/d), token t uses position
 * pos0 + t; out: [1, H, n_tok, d].  d even, <= 128.  Arithmetic in fp32 with the
 * reference's rounding points. */
int attn_b200_qk_norm_rope(const void* x, const void* weight, const float* freqs, void* out,
                           int32_t n_tok, int32_t H, int32_t d, int32_t pos0, int32_t norm_from,
                           float eps, int32_t dtype, void* stream);

/* Number of kernels the last successful call of the calling thread launched. */
int attn_b200_last_launch_count(void);

/* Reads (and clears) the current device's kernel status word: 0 when no kernel
 * has given up on a bounded wait since the last read, otherwise a code naming
 * the kernel and the wait.  Synchronises the device.  Kernels never spin
 * forever: each wait has an iteration limit, after which the kernel records its
 * code here and returns.  Code = (kernel id + 1) << 8 | wait id, kernel ids:
 * 4 / 5 / 6 double-backward scalar + g_dO / g_Q / g_K + g_V kernel, 18 / 19
 * backward row / column kernel, 20 forward, 0x6f the primitive self-test (codes
 * 0x7001..0x7003); wait id 15 = the launch gave the kernel less shared memory
 * than its layout needs. */
int attn_b200_device_status(uint32_t* code);

/* Registers a page-locked host word (cudaHostAlloc / cudaHostRegister memory, mapped into
 * the device's address space) as a mirror of the current device's status word: a kernel
 * that gives up on a bounded wait writes its code there as well as into the device word.
 * A caller can then notice a time-out at the start of its next call by reading its own
 * memory -- no copy, no synchronisation, nothing on the good path -- and fetch and clear
 * the device word with attn_b200_device_status.  The module `attention_cuda` does exactly
 * this, so a time-out surfaces as a Python exception of a following call.  NULL
 * unregisters.  Synchronous (one 8-byte copy); call it at start-up.  Has no counterpart in
 * the reference (whose kernels have no bounded waits). */
int attn_b200_set_status_mirror(uint32_t* host_word);

/* Message for the last error of the calling thread ("" if none). */
const char* attn_b200_last_error(void);

/* Library version string. */
const char* attn_b200_version(void);

/* Tensor-core primitive self-test used by the GPU tests: C[M=128, N] (float32,
 * row-major) = A[128, K] * Bop, with f16/bf16 operands in 128-byte-swizzled
 * shared memory and one tcgen05.mma chain.  flags bit 0: B is given as [K, N]
 * (N contiguous, read as an MN-major operand) instead of [N, K]; bit 1: A is
 * staged by the threads with the software swizzle instead of by TMA; bit 2: A is
 * copied to tensor memory and read from there; bit 3: nothing is computed -- one
 * thread waits, with a limit of about a millisecond, on a barrier that nothing
 * signals, so that the time-out path runs (status word 0x7003, abort flag, common
 * teardown that frees tensor memory) without any fault.
 * N in {64, 128}, K in {64, 128}.  Has no counterpart in the reference. */
int attn_b200_selftest_gemm(const void* A, const void* B, float* C, int32_t N, int32_t K,
                            int32_t dtype, int32_t flags, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* ATTN_B200_H */
