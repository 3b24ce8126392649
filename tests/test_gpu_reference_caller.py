"""Drop-in check through the reference's OWN caller code.

`oracle/build_ref.py` byte-compiles the reference's TTT model file (e2e/ttt_pytorch/model.py)
into oracle/_ref/; here that module is imported with THIS repository's `610sample_b200/` first
on `sys.path`, so its `v7_kernel_attention` (`from attention import flash_attention_v7`, permuted
non-contiguous [1, H, N, d] views, model.py:174-191) and its `meta_step` with
`use_v7_kernels=True` run on this repository's `attention.py` / `attention_cuda` unchanged.
The two tests are the reference's own integration tests with their tolerances
(e2e/tests/test_ttt_e2e_pytorch.py:415-476 and :479-604): the kernel path against the reference's
matmul attention on the [N, H, d] layout (forward < 5e-3, first-order gradients < 2e-2), and the
whole meta-step with the kernel path on and off (loss difference < 0.1, every parameter gradient
within 5e-2 absolute / relative).
"""
import os
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, "oracle"))
import build_ref  # noqa: E402

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ref_model():
    mod = build_ref.load_python_reference()
    if mod is None:
        pytest.skip("oracle/_ref/ref_ttt_model.bin has not been compiled (python oracle/build_ref.py <checkout>)")
    pkg = os.path.join(ROOT, "610sample_b200")
    sys.path.insert(0, pkg)            # `from attention import flash_attention_v7` finds this repository's module
    sys.modules.pop("attention", None)
    import attention
    assert os.path.dirname(os.path.abspath(attention.__file__)) == pkg
    yield mod
    sys.path.remove(pkg)


@pytest.mark.parametrize("cfg", [
    dict(H=1, N_q=32, N_kv=128, D=64, ws=96, cid=1),
    dict(H=4, N_q=64, N_kv=256, D=64, ws=192, cid=2),
])
def test_reference_v7_kernel_attention_on_nhd_layout(ref_model, cfg):
    H, N_q, N_kv, D, ws, cid = (cfg[k] for k in ("H", "N_q", "N_kv", "D", "ws", "cid"))
    dev, dtype = "cuda", torch.bfloat16
    torch.manual_seed(42)
    Q = torch.randn(N_q, H, D, device=dev, dtype=dtype, requires_grad=True)
    K = torch.randn(N_kv, H, D, device=dev, dtype=dtype, requires_grad=True)
    V = torch.randn(N_kv, H, D, device=dev, dtype=dtype, requires_grad=True)

    mask = ref_model.make_sw_causal_mask(cid, N_q, N_kv, ws, dev)
    Q_h, K_h, V_h = (t.detach().clone().float().permute(1, 0, 2).requires_grad_(True) for t in (Q, K, V))
    ref_O = ref_model.reference_attention(Q_h, K_h, V_h, mask)

    O = ref_model.v7_kernel_attention(Q, K, V, chunk_id=cid, window_size=ws)
    assert O.shape == (N_q, H, D)
    assert float((O.float() - ref_O.permute(1, 0, 2).detach()).abs().max()) < 5e-3

    ref_O.sum().backward()
    grads = torch.autograd.grad(O.sum(), [Q, K, V])
    for name, g, r in zip(("dQ", "dK", "dV"), grads, (Q_h.grad, K_h.grad, V_h.grad)):
        assert float((g.float() - r.permute(1, 0, 2)).abs().max()) < 2e-2, name


def test_reference_meta_step_with_and_without_the_kernels(ref_model):
    dev = "cuda"

    def make_config(use_v7):
        return ref_model.TTTConfig(vocab_size=64, hidden_size=64, intermediate_size=128, num_hidden_layers=2,
                                   num_attention_heads=1, mini_batch_size=64, sliding_window_size=192, seq_len=256,
                                   suffix_len=1, prime=False, inner_lr=0.01, use_v7_kernels=use_v7)

    T = 64 * 4     # four chunks
    torch.manual_seed(123)
    input_ids = torch.randint(0, 64, (T,), device=dev)
    targets = torch.randint(0, 64, (T,), device=dev)
    loss_masks = torch.ones(T, device=dev)

    def run(use_v7):
        cfg = make_config(use_v7)
        torch.manual_seed(42)
        model = ref_model.CausalLM(cfg).to(dev).to(torch.bfloat16)
        loss = ref_model.meta_step(model, input_ids, targets, loss_masks, cfg)
        loss.backward()
        return float(loss), {n: p.grad.float().clone() for n, p in model.named_parameters() if p.grad is not None}

    ref_loss, ref_grads = run(False)
    loss, grads = run(True)
    assert loss > 0 and loss == loss
    assert abs(loss - ref_loss) < 0.1
    assert len(grads) == len(ref_grads) > 0
    for n, g in grads.items():
        assert torch.isfinite(g).all(), n
        assert torch.allclose(g, ref_grads[n], atol=5e-2, rtol=5e-2), (n, float((g - ref_grads[n]).abs().max()))
