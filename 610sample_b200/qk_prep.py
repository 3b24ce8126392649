"""Fused preparation of Q / K for the attention kernels: per-head RMS normalisation, rotary
position embedding and the layout change [n_tok, H, d] -> [1, H, n_tok, d] in one CUDA pass
(`attention_cuda.qk_norm_rope`).

The reference does these steps as separate eager operations (`RMSNorm.forward`,
`apply_rotary_emb`, then `permute` + `contiguous` inside `v7_kernel_attention`:
e2e/ttt_pytorch/model.py:76-84, 96-116, 182-184, used at :260-263 and :309-316).  This is an
additive entry point: the reference surface (`attention.py`) does not depend on it.

`qk_norm_rope` is differentiable to second order, as test-time training needs: the forward
runs the fused kernel; the backward re-evaluates the same formulas with ordinary PyTorch
operations on the saved inputs, under the caller's grad mode, so its own derivative exists.
"""
import torch

try:  # used as part of the package
    from . import attention_cuda as _attention_cuda
except ImportError:  # used the reference's way: this directory on sys.path
    import attention_cuda as _attention_cuda


def rope_table(head_dim: int, positions: int, theta: float = 10000.0, device=None) -> torch.Tensor:
    """float32 [positions, head_dim/2, 2] = (cos, sin) of position * theta^(-2i/head_dim): the real
    view of the reference's `precompute_freqs_cis` (model.py:87-93)."""
    freqs = 1.0 / (theta ** (torch.arange(0, head_dim, 2, device=device).float() / head_dim))
    ang = torch.outer(torch.arange(positions, device=device).float(), freqs)
    return torch.stack([torch.cos(ang), torch.sin(ang)], dim=-1).contiguous()


def qk_norm_rope_torch(x, weight, freqs, pos0=0, eps=1e-6, norm_from=0):
    """The same computation in plain PyTorch operations (the formulas of model.py:82-84 and
    :102-116, with their rounding points), returning [1, H, n_tok, d]."""
    n_tok, H, d = x.shape
    y = x
    if weight is not None:
        xf = x.float()
        normed = (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)).to(x.dtype) * weight.to(x.dtype)
        if norm_from > 0:
            keep = (torch.arange(n_tok, device=x.device) < norm_from).view(n_tok, 1, 1)
            normed = torch.where(keep, x, normed)
        y = normed
    f = freqs[pos0:pos0 + n_tok].unsqueeze(1)                         # [n_tok, 1, d/2, 2]
    pair = y.float().reshape(n_tok, H, d // 2, 2)
    a, b = pair[..., 0], pair[..., 1]
    c, s = f[..., 0], f[..., 1]
    out = torch.stack([a * c - b * s, a * s + b * c], dim=-1).reshape(n_tok, H, d).to(x.dtype)
    return out.permute(1, 0, 2).unsqueeze(0)


class _QKNormRope(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, freqs, pos0, eps, norm_from):
        ctx.save_for_backward(x, weight if weight is not None else x.new_empty(0), freqs)
        ctx.has_weight = weight is not None
        ctx.args = (pos0, eps, norm_from)
        return _attention_cuda.qk_norm_rope(x, weight, freqs, pos0, eps, norm_from)

    @staticmethod
    def backward(ctx, g):
        x, weight, freqs = ctx.saved_tensors
        weight = weight if ctx.has_weight else None
        pos0, eps, norm_from = ctx.args
        with torch.enable_grad():
            xs = x if x.requires_grad else x.detach().requires_grad_(True)
            ws = None
            if weight is not None:
                ws = weight if weight.requires_grad else weight.detach().requires_grad_(True)
            y = qk_norm_rope_torch(xs, ws, freqs, pos0, eps, norm_from)
            wrt = [xs] + ([ws] if ws is not None else [])
            grads = torch.autograd.grad(y, wrt, g, create_graph=torch.is_grad_enabled(), allow_unused=True)
        gx = grads[0]
        gw = grads[1] if ws is not None else None
        return gx, gw, None, None, None, None


def qk_norm_rope(x, weight, freqs, pos0=0, eps=1e-6, norm_from=0):
    """x: [n_tok, H, d] (fp16 / bf16 / fp32, CUDA); weight: [d] or None; freqs: `rope_table(...)`.
    Rows below `norm_from` are only rotated (keys taken from a cache are stored normalised).
    Returns [1, H, n_tok, d], ready for `flash_attention_v7`."""
    return _QKNormRope.apply(x, weight, freqs, pos0, eps, norm_from)
