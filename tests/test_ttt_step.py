"""The end-to-end TTT step harness (bench_ttt.py): structure on CPU with the math attention,
and on the GPU parity of the whole meta step between the CUDA attention path and the math
path, the way the reference's integration test compares its two attention back ends
(reference e2e/tests/test_ttt_e2e_pytorch.py:479-604: loss difference < 0.1, every parameter
gradient within 5e-2)."""
import os
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
import bench_ttt as bt  # noqa: E402


def _step(cfg, dev, dtype, attention):
    slow, fast = bt.init_params(cfg, dev, dtype, seed=1)
    ids, targets = bt.make_batch(cfg, dev, seed=2)
    loss = bt.ttt_step(cfg, slow, fast, ids, targets, attention)
    loss.backward()
    grads = {n: p.grad.detach().float().cpu() for n, p in {**slow, **fast}.items()}
    return float(loss.detach()), grads


def test_meta_step_runs_on_cpu_with_math_attention():
    cfg = dict(bt.SMALL, seq=64, batch=1)
    loss, grads = _step(cfg, torch.device("cpu"), torch.float32, bt.math_attention_fn(cfg["seq"]))
    assert abs(loss - torch.log(torch.tensor(float(cfg["vocab"]))).item()) < 0.5     # random init: ~ln(vocab)
    assert all(torch.isfinite(g).all() for g in grads.values())
    # the outer gradient reaches the attention projections through the inner update
    assert float(grads["blk0.qkv"].abs().max()) > 0 and float(grads["blk1.proj"].abs().max()) > 0


@pytest.mark.gpu
def test_meta_step_matches_math_attention_path():
    sys.path.insert(0, os.path.join(ROOT, "610sample_b200"))
    from attention import flash_attention_v7
    cfg = dict(bt.SMALL)
    dev = torch.device("cuda")
    N = cfg["seq"]
    ours = _step(cfg, dev, torch.bfloat16, lambda q, k, v: flash_attention_v7(q, k, v, N, 0))
    ref = _step(cfg, dev, torch.bfloat16, bt.math_attention_fn(N))
    assert abs(ours[0] - ref[0]) < 0.1
    for n in ref[1]:
        scale = max(1.0, float(ref[1][n].abs().max()))
        assert torch.allclose(ours[1][n], ref[1][n], atol=5e-2 * scale, rtol=5e-2), n


@pytest.mark.gpu
def test_attention_only_meta_step_matches_math_attention_path():
    """The reference's attention-only meta-step (e2e/tests/test_ttt_e2e_pytorch.py:754-818: chunks of
    a token stream, K/V history left-padded with zeros, gradient of sum(O) with respect to the three
    projections under create_graph, meta-loss = sum of those gradients, one backward) on its `small`
    and `med` shapes: the kernel arm against the PyTorch math-attention arm of bench_attn_meta.py."""
    import bench_attn_meta as bam
    dev = torch.device("cuda")
    kern, math_ = bam.kernel_attention(), bam.math_attention()
    for name in ("small", "med"):
        shape = bam.SHAPES[name]
        loss_k, g_k = bam.run_step(torch, kern, 2, shape, dev, torch.bfloat16, seed=3)
        loss_m, g_m = bam.run_step(torch, math_, 2, shape, dev, torch.bfloat16, seed=3)
        assert abs(float(loss_k) - float(loss_m)) <= 5e-2 * max(1.0, abs(float(loss_m)))
        for a, b, n in zip(g_k, g_m, ("W_q", "W_k", "W_v")):
            scale = max(1e-6, float(b.float().abs().max()))
            assert float((a.float() - b.float()).abs().max()) <= 5e-2 * scale, (name, n)
