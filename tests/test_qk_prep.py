"""The fused step before attention (RMS norm + rotary embedding + layout change): the oracle
restatement against the fixture made by the reference's own RMSNorm / apply_rotary_emb (CPU), and
the CUDA kernel and its differentiable wrapper against the oracle (GPU)."""
import importlib
import os
import sys

import pytest
import torch

import attention_oracle as orc
from _util import load_prep_golden

PKG_DIR = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "610sample_b200")


def test_oracle_matches_the_reference_fixture():
    m, x, w, want = load_prep_golden()
    fc = orc.rope_freqs_cis(m["d"], 128)
    got = orc.qk_norm_rope_oracle(x, w, fc, pos0=m["pos0"], eps=1e-6, norm_from=m["norm_from"])
    assert got.shape == want.shape == (1, m["H"], m["n_tok"], m["d"])
    assert torch.equal(got.float(), want)          # same operations in the same order: bit-exact


def test_oracle_without_weight_only_rotates():
    x = torch.randn(5, 2, 16)
    fc = orc.rope_freqs_cis(16, 8)
    y = orc.qk_norm_rope_oracle(x, None, fc)
    assert torch.allclose(y.norm(dim=-1)[0].T, x.norm(dim=-1), atol=1e-5)      # a rotation keeps the length
    assert torch.allclose(y[0, :, 0], x[0])                                    # position 0: identity


@pytest.fixture(scope="module")
def prep():
    if PKG_DIR not in sys.path:
        sys.path.insert(0, PKG_DIR)
    return importlib.import_module("qk_prep")


@pytest.mark.gpu
def test_kernel_matches_reference_fixture_and_oracle(prep):
    m, x, w, want = load_prep_golden()
    table = prep.rope_table(m["d"], 128, device="cuda")
    got = prep.qk_norm_rope(x.cuda(), w.cuda(), table, pos0=m["pos0"], eps=1e-6, norm_from=m["norm_from"])
    # fp32 arithmetic in a different summation order: at most one bf16 unit in the last place
    err = (got.float().cpu() - want).abs()
    assert float((err / want.abs().clamp_min(1e-3)).max()) <= 2 ** -7
    assert float((err > 0).float().mean()) < 0.02
    # the last three: a head count that is not a multiple of the four a lane group walks over, a
    # width of 8 lanes with a partly filled last CTA, and a head dimension (not a multiple of 8)
    # that takes the pairwise kernel
    for dtype, D, H, n in ((torch.float16, 128, 4, 300), (torch.float32, 80, 2, 77), (torch.bfloat16, 96, 16, 1024),
                           (torch.float16, 64, 5, 130), (torch.bfloat16, 16, 7, 33), (torch.bfloat16, 20, 3, 65)):
        xx = torch.randn(n, H, D).to(dtype)
        ww = (1 + 0.1 * torch.randn(D)).to(dtype)
        fc = orc.rope_freqs_cis(D, n + 9)
        ref = orc.qk_norm_rope_oracle(xx, ww, fc, pos0=9, norm_from=n // 3)
        out = prep.qk_norm_rope(xx.cuda(), ww.cuda(), prep.rope_table(D, n + 9, device="cuda"), pos0=9, norm_from=n // 3)
        tol = {torch.float16: 2 ** -9, torch.bfloat16: 2 ** -7, torch.float32: 1e-5}[dtype]      # a unit or two in the last place
        # a rotated element is a difference of two rounded products: its error scales with the inputs (O(1)), not with itself
        assert float(((out.float().cpu() - ref.float()).abs() / (1.0 + ref.float().abs())).max()) <= tol, dtype
        no_norm = prep.qk_norm_rope(xx.cuda(), None, prep.rope_table(D, n + 9, device="cuda"), pos0=9)
        ref2 = orc.qk_norm_rope_oracle(xx, None, fc, pos0=9)
        assert float((no_norm.float().cpu() - ref2.float()).abs().max()) <= tol * float(ref2.float().abs().max())


@pytest.mark.gpu
def test_kernel_full_tile_variant_matches_oracle(prep):
    """Shapes whose CTAs are all full and whose normalisation covers every token take the
    guard-free variant of the kernel; the same shapes with one token more take the guarded one,
    and the two agree bit for bit on the tokens they share."""
    for dtype, D, H, n in ((torch.bfloat16, 128, 8, 256), (torch.float16, 64, 4, 96), (torch.float32, 128, 4, 32),
                           (torch.bfloat16, 64, 12, 1024)):
        xx = torch.randn(n + 1, H, D).to(dtype)
        ww = (1 + 0.1 * torch.randn(D)).to(dtype)
        fc = orc.rope_freqs_cis(D, n + 4)
        table = prep.rope_table(D, n + 4, device="cuda")
        tol = {torch.float16: 2 ** -9, torch.bfloat16: 2 ** -7, torch.float32: 1e-5}[dtype]
        for weight in (ww, None):
            ref = orc.qk_norm_rope_oracle(xx[:n], weight, fc, pos0=3)
            wc = None if weight is None else weight.cuda()
            full = prep.qk_norm_rope(xx[:n].cuda(), wc, table, pos0=3)
            assert float(((full.float().cpu() - ref.float()).abs() / (1.0 + ref.float().abs())).max()) <= tol, (dtype, D)
            ragged = prep.qk_norm_rope(xx.cuda(), wc, table, pos0=3)
            assert torch.equal(ragged[:, :, :n], full), (dtype, D)


@pytest.mark.gpu
def test_wrapper_is_differentiable_to_second_order_and_feeds_attention(prep):
    """Gradients of the fused call equal those of the plain PyTorch formulas, first and second
    order, and its output goes straight into flash_attention_v7 (layout [1, H, n_tok, d])."""
    from attention import flash_attention_v7
    torch.manual_seed(5)
    n, H, D = 192, 2, 64
    x0 = torch.randn(n, H, D, device="cuda", dtype=torch.float32)
    w0 = (1 + 0.1 * torch.randn(D, device="cuda"))
    table = prep.rope_table(D, n, device="cuda")
    u = torch.randn(1, H, n, D, device="cuda")

    def second_order(fn):
        x = x0.clone().requires_grad_(True)
        w = w0.clone().requires_grad_(True)
        y = fn(x, w, table)
        gx, gw = torch.autograd.grad((y * u).sum() + (y * y).sum(), [x, w], create_graph=True)
        hx, hw = torch.autograd.grad(gx.pow(2).sum() + gw.pow(2).sum(), [x, w])
        return y, gx, gw, hx, hw

    got = second_order(prep.qk_norm_rope)
    want = second_order(prep.qk_norm_rope_torch)
    for a, b, name in zip(got, want, ("y", "gx", "gw", "hx", "hw")):
        assert torch.allclose(a, b, rtol=1e-4, atol=1e-4 * float(b.abs().max())), name

    xq = torch.randn(n, H, D, device="cuda").to(torch.bfloat16).requires_grad_(True)
    wq = torch.ones(D, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    Q = prep.qk_norm_rope(xq, wq, table)
    O = flash_attention_v7(Q, Q.detach(), Q.detach(), n, 0)
    g, = torch.autograd.grad(O.float().sum(), [xq])
    assert g.shape == xq.shape and torch.isfinite(g.float()).all() and float(g.float().abs().max()) > 0
