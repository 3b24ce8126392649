"""CPU oracle for the attention forward / backward / double-backward (HVP) path.

TEST INFRASTRUCTURE ONLY.  Nothing in the product package imports this file; it
is used by ``tests/``, by ``__graft_entry__.smoke()`` and by the CPU-baseline /
``--impl reference`` legs of ``bench.py`` as the checker and the timed CPU path.

It restates, in plain PyTorch on the CPU, the algorithm that the reference
project uses as its own ground truth:

* the visibility mask ``(qi >= ki) & (qi < ki + window_size) & (ki >= 0)`` with
  ``qi = chunk_id*N_q + i`` and ``ki = chunk_id*N_q + N_q - N_kv + j``
  (reference ``e2e/ttt_pytorch/model.py:141-156``,
  ``tests/test_v7_correctness.py:23-33``, device twin
  ``csrc/flash_double_backward_v7.cu:100-102``);
* the five-line math attention ``S = QK^T*scale -> masked_fill(-inf) -> softmax
  -> NaN->0 -> P@V`` (reference ``e2e/ttt_pytorch/model.py:159-171`` ==
  ``tests/test_v7_correctness.py:36-44``);
* first backward via ``torch.autograd.grad(..., create_graph=True)`` and the
  Hessian-vector product via a second ``torch.autograd.grad`` of
  ``<dQ,g_dQ> + <dK,g_dK> + <dV,g_dV>`` (pattern of reference
  ``tests/test_v7_correctness.py:136-145``, extended to random ``dO`` and to the
  gradient with respect to ``dO``);
* a closed form of the same HVP (the row/column formulas that the reference
  kernels implement, ``csrc/flash_double_backward_v7.cu:1257-1454`` and
  ``:1583-1675``), evaluated block-wise in fp64 so that N=4096..16384 does not
  need an N x N autograd graph.

Parity pin: ``tests/golden/make_golden.py`` imports the reference's own
``make_sw_causal_mask`` and ``reference_attention`` and stores their outputs;
``tests/test_oracle.py`` checks this file against those fixtures.
"""
from __future__ import annotations

import math
from typing import Dict, Optional, Sequence

import torch

MASK_REFERENCE = 0   # causal + sliding window + validity (the reference's mask)
MASK_NONE = 1        # every (i, j) visible (extension used by the non-causal config)

OUTPUT_NAMES = ("O", "L", "dQ", "dK", "dV", "g_dO", "g_Q", "g_K", "g_V")


# --------------------------------------------------------------------------
# mask
# --------------------------------------------------------------------------
def visibility_mask(chunk_id: int, N_q: int, N_kv: int, window_size: int,
                    mask_mode: int = MASK_REFERENCE, device="cpu") -> torch.Tensor:
    """Boolean [N_q, N_kv] visibility (True = attend).

    Follows reference ``e2e/ttt_pytorch/model.py:141-156``.
    """
    if mask_mode == MASK_NONE:
        return torch.ones(N_q, N_kv, dtype=torch.bool, device=device)
    q0 = chunk_id * N_q
    qi = (torch.arange(N_q, device=device, dtype=torch.int64) + q0).unsqueeze(1)
    ki = (torch.arange(-N_kv, 0, device=device, dtype=torch.int64) + q0 + N_q).unsqueeze(0)
    return (qi >= ki) & (qi < ki + window_size) & (ki >= 0)


def visible_pairs(chunk_id: int, N_q: int, N_kv: int, window_size: int,
                  mask_mode: int = MASK_REFERENCE) -> int:
    """Number of unmasked (i, j) pairs: the unit of the algorithmic flop count."""
    if mask_mode == MASK_NONE:
        return N_q * N_kv
    i = torch.arange(N_q, dtype=torch.int64) + chunk_id * N_q
    k_base = chunk_id * N_q + N_q - N_kv
    lo = torch.clamp(i - window_size + 1, min=0)          # smallest visible ki
    lo = torch.maximum(lo, torch.tensor(max(k_base, 0)))
    hi = torch.minimum(i, torch.tensor(k_base + N_kv - 1))  # largest visible ki
    return int(torch.clamp(hi - lo + 1, min=0).sum())


# --------------------------------------------------------------------------
# the reference's math attention and its double autograd
# --------------------------------------------------------------------------
def math_attention(Q: torch.Tensor, K: torch.Tensor, V: torch.Tensor,
                   mask: torch.Tensor) -> torch.Tensor:
    """``softmax(QK^T/sqrt(D) + mask) V`` exactly as reference
    ``e2e/ttt_pytorch/model.py:159-171`` writes it (fully masked rows give 0)."""
    scale = 1.0 / math.sqrt(Q.shape[-1])
    S = torch.matmul(Q, K.transpose(-2, -1)) * scale
    S = S.masked_fill(~mask, float("-inf"))
    P = torch.softmax(S, dim=-1)
    P = P.masked_fill(torch.isnan(P), 0.0)
    return torch.matmul(P, V)


def logsumexp_rows(Q, K, mask):
    """Natural-log LSE of the scaled, masked scores (-inf for fully masked rows);
    the quantity the reference forward kernel stores as ``L``
    (``csrc/flash_double_backward_v7.cu:452-461``)."""
    scale = 1.0 / math.sqrt(Q.shape[-1])
    S = torch.matmul(Q, K.transpose(-2, -1)) * scale
    S = S.masked_fill(~mask, float("-inf"))
    return torch.logsumexp(S, dim=-1)


def autograd_all(Q, K, V, dO, g_dQ, g_dK, g_dV, mask,
                 compute_dtype: torch.dtype = torch.float64) -> Dict[str, torch.Tensor]:
    """Forward, first backward and HVP by PyTorch double autograd in
    ``compute_dtype`` on the (already rounded) inputs.  Returns the nine tensors
    of ``OUTPUT_NAMES`` in ``compute_dtype``."""
    c = lambda t: t.detach().to(compute_dtype)
    q, k, v, do = (c(t).requires_grad_(True) for t in (Q, K, V, dO))
    O = math_attention(q, k, v, mask)
    dQ, dK, dV = torch.autograd.grad(O, [q, k, v], grad_outputs=do, create_graph=True)
    h = (dQ * c(g_dQ)).sum() + (dK * c(g_dK)).sum() + (dV * c(g_dV)).sum()
    g_dO, g_Q, g_K, g_V = torch.autograd.grad(h, [do, q, k, v])
    with torch.no_grad():
        L = logsumexp_rows(q, k, mask)
    out = dict(O=O, L=L, dQ=dQ, dK=dK, dV=dV, g_dO=g_dO, g_Q=g_Q, g_K=g_K, g_V=g_V)
    return {n: t.detach() for n, t in out.items()}


# --------------------------------------------------------------------------
# closed form, block-wise (no autograd graph, O(block x N_kv) memory)
# --------------------------------------------------------------------------
@torch.no_grad()
def closed_form_all(Q, K, V, dO, g_dQ, g_dK, g_dV, *, window_size: int, chunk_id: int,
                    mask_mode: int = MASK_REFERENCE,
                    compute_dtype: torch.dtype = torch.float64,
                    row_block: int = 512,
                    heads: Optional[Sequence[int]] = None,
                    device="cpu") -> Dict[str, torch.Tensor]:
    """Same nine outputs from the closed-form expressions, one (batch, head) and
    one block of query rows at a time.

    With ``s = 1/sqrt(D)``, ``P = softmax(s QK^T)``, ``dP = dO V^T``,
    ``Dv_i = sum_j P dP``, ``dS = P (dP - Dv)``:

      dQ = s dS K          dK = s dS^T Q          dV = P^T dO
      gdS  = s (g_dQ K^T + Q g_dK^T)       gPdV = dO g_dV^T
      dot2 = sum_j P gdS
      g_dp = P (gdS - dot2)
      g_P  = gdS (dP - Dv) - dP dot2 + gPdV
      dot3 = sum_j P g_P
      g_S  = P (g_P - dot3)
      g_Q  = s (dS g_dK + g_S K)           g_K = s (dS^T g_dQ + g_S^T Q)
      g_V  = g_dp^T dO                     g_dO = P g_dV + g_dp V

    (reference ``csrc/flash_double_backward_v7.cu:1257-1454, 1583-1675``).
    ``heads`` optionally restricts the flattened (batch*head) indices computed;
    the others are left zero.  ``device`` is where the arithmetic runs (the same
    PyTorch expressions; a GPU only makes N = 16384 in fp64 finish in seconds);
    the results come back on the CPU.
    """
    B, H, N_q, D = Q.shape
    N_kv = K.shape[2]
    s = 1.0 / math.sqrt(D)
    cd = compute_dtype
    f = lambda t, n: t.detach().reshape(B * H, n, D).to(device)
    Qf, dOf, gQf = f(Q, N_q), f(dO, N_q), f(g_dQ, N_q)
    Kf, Vf, gKf, gVf = f(K, N_kv), f(V, N_kv), f(g_dK, N_kv), f(g_dV, N_kv)
    z = lambda n: torch.zeros(B * H, n, D, dtype=cd, device=device)
    O, dQ, g_dO, g_Q = z(N_q), z(N_q), z(N_q), z(N_q)
    dK, dV, g_K, g_V = z(N_kv), z(N_kv), z(N_kv), z(N_kv)
    L = torch.zeros(B * H, N_q, dtype=cd, device=device)
    mask_full = visibility_mask(chunk_id, N_q, N_kv, window_size, mask_mode, device=device)
    todo = range(B * H) if heads is None else heads
    for bh in todo:
        k, v, gk, gv = (t[bh].to(cd) for t in (Kf, Vf, gKf, gVf))
        for r0 in range(0, N_q, row_block):
            r1 = min(N_q, r0 + row_block)
            q, do, gq = (t[bh, r0:r1].to(cd) for t in (Qf, dOf, gQf))
            m = mask_full[r0:r1]
            S = (q @ k.T) * s
            S = S.masked_fill(~m, float("-inf"))
            Lr = torch.logsumexp(S, dim=-1)
            P = torch.exp(S - Lr.unsqueeze(1))
            P = torch.where(m, P, torch.zeros_like(P))
            P = torch.nan_to_num(P, nan=0.0)           # fully masked rows
            dP = do @ v.T
            Dv = (P * dP).sum(-1, keepdim=True)
            dS = P * (dP - Dv)
            gdS = s * (gq @ k.T + q @ gk.T)
            gPdV = do @ gv.T
            dot2 = (P * gdS).sum(-1, keepdim=True)
            g_dp = P * (gdS - dot2)
            g_P = gdS * (dP - Dv) - dP * dot2 + gPdV
            dot3 = (P * g_P).sum(-1, keepdim=True)
            g_S = P * (g_P - dot3)
            L[bh, r0:r1] = Lr
            O[bh, r0:r1] = P @ v
            dQ[bh, r0:r1] = s * (dS @ k)
            dK[bh] += s * (dS.T @ q)
            dV[bh] += P.T @ do
            g_Q[bh, r0:r1] = s * (dS @ gk + g_S @ k)
            g_dO[bh, r0:r1] = P @ gv + g_dp @ v
            g_K[bh] += s * (dS.T @ gq + g_S.T @ q)
            g_V[bh] += g_dp.T @ do
    r = lambda t, n: t.reshape(B, H, n, D).cpu()
    return dict(O=r(O, N_q), L=L.reshape(B, H, N_q).cpu(), dQ=r(dQ, N_q), dK=r(dK, N_kv),
                dV=r(dV, N_kv), g_dO=r(g_dO, N_q), g_Q=r(g_Q, N_q), g_K=r(g_K, N_kv),
                g_V=r(g_V, N_kv))


# --------------------------------------------------------------------------
# the step before attention: per-head RMS norm and rotary embedding
# --------------------------------------------------------------------------
def rope_freqs_cis(head_dim: int, positions: int, theta: float = 10000.0) -> torch.Tensor:
    """complex64 [positions, head_dim/2], as reference ``e2e/ttt_pytorch/model.py:87-93``."""
    freqs = 1.0 / (theta ** (torch.arange(0, head_dim, 2).float() / head_dim))
    ang = torch.outer(torch.arange(positions).float(), freqs)
    return torch.polar(torch.ones_like(ang), ang)


def qk_norm_rope_oracle(x: torch.Tensor, weight: Optional[torch.Tensor], freqs_cis: torch.Tensor,
                        pos0: int = 0, eps: float = 1e-6, norm_from: int = 0) -> torch.Tensor:
    """x [n_tok, H, d] -> [1, H, n_tok, d].  RMS normalisation exactly as the reference's
    ``RMSNorm.forward`` (``model.py:82-84``: fp32 statistics, result cast to the input type, then
    multiplied by the weight) on rows >= ``norm_from``; rotary embedding exactly as its
    ``apply_rotary_emb`` (``model.py:96-116``: pairs of consecutive elements as complex numbers
    times ``freqs_cis`` in fp32, cast back); then the permutation of ``model.py:182-184``."""
    n_tok = x.shape[0]
    y = x
    if weight is not None:
        xf = x.float()
        normed = (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)).to(x.dtype) * weight.to(x.dtype)
        y = torch.cat([x[:norm_from], normed[norm_from:]], dim=0)
    xc = torch.view_as_complex(y.float().reshape(*y.shape[:-1], -1, 2).contiguous())
    fc = freqs_cis[pos0:pos0 + n_tok].unsqueeze(-2)
    out = torch.view_as_real(xc * fc).flatten(-2).to(x.dtype)
    return out.permute(1, 0, 2).unsqueeze(0)


# --------------------------------------------------------------------------
# seeded inputs and error metrics
# --------------------------------------------------------------------------
INPUT_NAMES = ("Q", "K", "V", "dO", "g_dQ", "g_dK", "g_dV")


def make_inputs(B: int, H: int, N_q: int, N_kv: int, D: int, *, seed: int = 0,
                dtype: torch.dtype = torch.float32, qk_scale: float = 1.0,
                v_scale: float = 1.0) -> Dict[str, torch.Tensor]:
    """Seeded synthetic inputs.  A CPU generator seeded with ``seed`` draws fp32
    N(0,1) tensors in the order Q, K, V, dO, g_dQ, g_dK, g_dV; Q and K are
    multiplied by ``qk_scale`` and V by ``v_scale``; everything is then cast to
    ``dtype``.  The same function feeds the GPU tests, the bench and the CPU
    baseline so that all of them see identical values."""
    g = torch.Generator(device="cpu").manual_seed(seed)
    shp = dict(Q=N_q, K=N_kv, V=N_kv, dO=N_q, g_dQ=N_q, g_dK=N_kv, g_dV=N_kv)
    out = {}
    for name in INPUT_NAMES:
        t = torch.randn(B, H, shp[name], D, generator=g, dtype=torch.float32)
        if name in ("Q", "K"):
            t = t * qk_scale
        elif name == "V":
            t = t * v_scale
        out[name] = t.to(dtype)
    return out


def max_abs_err(a: torch.Tensor, ref: torch.Tensor) -> float:
    return float((a.double() - ref.double()).abs().max())


def rel_err(a: torch.Tensor, ref: torch.Tensor) -> float:
    """Norm-wise relative error ``||a - ref||_F / ||ref||_F``."""
    num = (a.double() - ref.double()).norm()
    den = ref.double().norm()
    return float(num / den) if den > 0 else float(num)
