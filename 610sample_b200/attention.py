"""Autograd surface of the B200 attention kernels.

Mirrors the reference's ``attention.py`` (``attention.py:12-71``): the same two
chained ``torch.autograd.Function`` classes, the same argument order and the same
``None`` gradients, so code written against the reference runs unchanged:

    from attention import flash_attention_v7
    O = flash_attention_v7(Q, K, V, window_size, chunk_id)

``FlashAttentionV7.backward`` calls ``FlashAttentionV7Backward.apply`` so that the
first backward is itself differentiable; its ``backward`` is the double backward
(Hessian-vector product) kernel.  Gradients are total derivatives with O and L
treated as functions of Q, K, V, hence ``None`` for the saved O and L.  Third
order is not supported.

Additive extension: ``mask_mode`` (0 = reference mask, 1 = no mask) as a trailing
keyword of ``flash_attention_v7``.

There is no fallback: importing this module fails if the compiled extension
``attention_cuda`` is missing.
"""
import torch

try:  # used as part of the package
    from . import attention_cuda as _attention_cuda
except ImportError:  # used the reference's way: this directory on sys.path
    import attention_cuda as _attention_cuda


class FlashAttentionV7Backward(torch.autograd.Function):
    @staticmethod
    def forward(ctx, dO, Q, K, V, O, L, window_size, chunk_id, mask_mode=0):
        dQ, dK, dV = _attention_cuda.v7_backward(dO, Q, K, V, O, L, window_size, chunk_id, mask_mode)
        ctx.set_materialize_grads(False)
        ctx.save_for_backward(dO, Q, K, V, O, L)
        ctx.window_size = window_size
        ctx.chunk_id = chunk_id
        ctx.mask_mode = mask_mode
        return dQ, dK, dV

    @staticmethod
    def backward(ctx, g_dQ, g_dK, g_dV):
        if g_dQ is None and g_dK is None and g_dV is None:
            return (None,) * 9
        dO, Q, K, V, O, L = ctx.saved_tensors
        if g_dQ is None:
            g_dQ = torch.zeros_like(Q)
        if g_dK is None:
            g_dK = torch.zeros_like(K)
        if g_dV is None:
            g_dV = torch.zeros_like(V)
        g_dO, g_Q, g_K, g_V = _attention_cuda.v7_double_backward(
            g_dQ, g_dK, g_dV, dO, Q, K, V, O, L, ctx.window_size, ctx.chunk_id, ctx.mask_mode)
        # gradients for: dO, Q, K, V, O, L, window_size, chunk_id, mask_mode
        return g_dO, g_Q, g_K, g_V, None, None, None, None, None


class FlashAttentionV7(torch.autograd.Function):
    @staticmethod
    def forward(ctx, Q, K, V, window_size, chunk_id, mask_mode=0):
        O, L = _attention_cuda.v7_forward(Q, K, V, window_size, chunk_id, mask_mode)
        # The saved O is an input of the differentiable backward below, whose own backward
        # returns no gradient for it.  Without this flag the engine would turn that missing
        # gradient into zeros and run a whole first-order backward on them during the
        # second-order pass.
        ctx.set_materialize_grads(False)
        ctx.save_for_backward(Q, K, V, O, L)
        ctx.window_size = window_size
        ctx.chunk_id = chunk_id
        ctx.mask_mode = mask_mode
        return O

    @staticmethod
    def backward(ctx, grad_output):
        if grad_output is None:
            return (None,) * 6
        Q, K, V, O, L = ctx.saved_tensors
        return (*FlashAttentionV7Backward.apply(
            grad_output, Q, K, V, O, L, ctx.window_size, ctx.chunk_id, ctx.mask_mode
        ), None, None, None)


def flash_attention_v7(Q, K, V, window_size, chunk_id, mask_mode=0):
    """Rectangular sliding-window attention with double-backward support.

    Q: (B, H, N_q, D); K, V: (B, H, N_kv, D); fp16, bf16 or fp32 CUDA tensors.
    Key j is visible to query i when, with ``qi = chunk_id*N_q + i`` and
    ``ki = chunk_id*N_q + N_q - N_kv + j``: ``ki >= 0 and qi >= ki and
    qi < ki + window_size``.  Plain causal attention over N tokens is
    ``N_q == N_kv == N, window_size >= N, chunk_id == 0``.
    Returns O: (B, H, N_q, D).
    """
    return FlashAttentionV7.apply(Q, K, V, window_size, chunk_id, mask_mode)
