"""Thin helpers that call the C ABI on PyTorch CUDA tensors (pointers only cross
the boundary; PyTorch is used for allocation and streams).  Used by the GPU tests
and the bench to exercise ``libattn_b200.so`` without the pybind module."""
from __future__ import annotations

import torch

from . import capi

_DT = {torch.float16: capi.ATTN_F16, torch.bfloat16: capi.ATTN_BF16, torch.float32: capi.ATTN_F32}


def _shape(Q, K, window_size, chunk_id, mask_mode, impl):
    B, H, N_q, D = Q.shape
    return capi.make_shape(B, H, N_q, K.shape[2], D, window_size, chunk_id, mask_mode, _DT[Q.dtype], impl)


def _stream():
    return torch.cuda.current_stream().cuda_stream


def _p(t):
    return None if t is None else t.data_ptr()


def forward(Q, K, V, window_size, chunk_id, mask_mode=0, impl=0):
    s = _shape(Q, K, window_size, chunk_id, mask_mode, impl)
    O = torch.empty_like(Q)
    L = torch.empty(Q.shape[:3], dtype=torch.float32, device=Q.device)
    capi.check(capi.lib().attn_b200_forward(s, _p(Q), _p(K), _p(V), _p(O), _p(L), _stream()), "attn_b200_forward")
    return O, L


def backward(dO, Q, K, V, O, L, window_size, chunk_id, mask_mode=0, impl=0, scratch=None):
    s = _shape(Q, K, window_size, chunk_id, mask_mode, impl)
    dQ, dK, dV = torch.empty_like(Q), torch.empty_like(K), torch.empty_like(V)
    if scratch is None:
        n = capi.lib().attn_b200_backward_scratch_bytes(s) // 4
        scratch = torch.empty(n + 4, dtype=torch.float32, device=Q.device)
    capi.check(capi.lib().attn_b200_backward(s, _p(dO), _p(Q), _p(K), _p(V), _p(O), _p(L), _p(dQ), _p(dK), _p(dV),
                                             _p(scratch), _stream()), "attn_b200_backward")
    return dQ, dK, dV


def double_backward(g_dQ, g_dK, g_dV, dO, Q, K, V, O, L, window_size, chunk_id, mask_mode=0, impl=0,
                    scratch=None, out=None):
    s = _shape(Q, K, window_size, chunk_id, mask_mode, impl)
    if out is None:
        out = (torch.empty_like(Q), torch.empty_like(Q), torch.empty_like(K), torch.empty_like(V))
    g_dO, g_Q, g_K, g_V = out
    if scratch is None:
        n = capi.lib().attn_b200_double_backward_scratch_bytes(s) // 4
        scratch = torch.empty(n + 4, dtype=torch.float32, device=Q.device)
    capi.check(capi.lib().attn_b200_double_backward(
        s, _p(g_dQ), _p(g_dK), _p(g_dV), _p(dO), _p(Q), _p(K), _p(V), _p(O), _p(L),
        _p(g_dO), _p(g_Q), _p(g_K), _p(g_V), _p(scratch), _stream()), "attn_b200_double_backward")
    return g_dO, g_Q, g_K, g_V


def double_backward_phases(g_dQ, g_dK, g_dV, dO, Q, K, V, O, L, window_size, chunk_id, mask_mode=0, impl=0,
                           scratch=None, out=None, phases=7):
    """One or more kernels of the double backward (bit mask: 1 scalars, 2 row side, 4 column side)."""
    s = _shape(Q, K, window_size, chunk_id, mask_mode, impl)
    g_dO, g_Q, g_K, g_V = out
    capi.check(capi.lib().attn_b200_double_backward_phases(
        s, _p(g_dQ), _p(g_dK), _p(g_dV), _p(dO), _p(Q), _p(K), _p(V), _p(O), _p(L),
        _p(g_dO), _p(g_Q), _p(g_K), _p(g_V), _p(scratch), _stream(), phases), "attn_b200_double_backward_phases")
    return out


def double_backward_static(g_dQ, g_dK, g_dV, dO, Q, K, V, O, L, window_size, chunk_id, mask_mode=0, impl=0, out=None):
    """The allocation-free entry point: the scratch is the library's built-in array.  The four
    outputs must be passed in (`out`) by a caller that really cannot allocate; they are created
    here only when omitted."""
    s = _shape(Q, K, window_size, chunk_id, mask_mode, impl)
    if out is None:
        out = (torch.empty_like(Q), torch.empty_like(Q), torch.empty_like(K), torch.empty_like(V))
    g_dO, g_Q, g_K, g_V = out
    capi.check(capi.lib().attn_b200_double_backward_static(
        s, _p(g_dQ), _p(g_dK), _p(g_dV), _p(dO), _p(Q), _p(K), _p(V), _p(O), _p(L),
        _p(g_dO), _p(g_Q), _p(g_K), _p(g_V), _stream()), "attn_b200_double_backward_static")
    return out


def selftest_gemm(A, B, N, K, flags):
    Cout = torch.zeros(128, N, dtype=torch.float32, device=A.device)
    capi.check(capi.lib().attn_b200_selftest_gemm(_p(A), _p(B), _p(Cout), N, K, _DT[A.dtype], flags, _stream()),
               "attn_b200_selftest_gemm")
    return Cout
