// Internal launcher interface between the C ABI (attn_capi.cu) and the two
// kernel families (attn_simt.cu, attn_tc.cu).
#pragma once
#include "attn_common.cuh"

namespace attn {

enum Op { OP_FORWARD = 0, OP_BACKWARD = 1, OP_DOUBLE_BACKWARD = 2 };

// Phases of the double backward, as a bit mask (all = 7).  PRE computes the
// per-row scalars into scratch, ROW the query-side outputs, COL the key-side ones.
enum HvpPhase { HVP_PHASE_PRE = 1, HVP_PHASE_ROW = 2, HVP_PHASE_COL = 4, HVP_PHASE_ALL = 7,
                // internal: keep every launch on the caller's stream (no helper stream is created)
                HVP_PHASE_SERIAL = 8 };

// fp32 CUDA-core kernels: any dtype, D a multiple of 16 up to 128.
cudaError_t launch_simt(int op, int dtype, const Geometry& g, const Tensors& t, cudaStream_t s,
                        int* launches, int phases);

// tcgen05 tensor-core kernels: f16/bf16, D a multiple of 16 up to 128 (tiles of width 64 or 128,
// zero-padded).
bool tc_supported(int dtype, int D);
cudaError_t launch_tc(int op, int dtype, const Geometry& g, const Tensors& t, cudaStream_t s,
                      int* launches, const char** err, int phases);

// Primitive self-test (one TMA + tcgen05.mma chain), see attn_b200_selftest_gemm.
cudaError_t launch_tc_selftest(const void* A, const void* B, float* C, int N, int K, int dtype,
                               int b_layout, unsigned int* status, cudaStream_t s,
                               const char** err);

}  // namespace attn
