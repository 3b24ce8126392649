"""GPU tests of the reference-facing surface: the attention_cuda module and the
flash_attention_v7 autograd functions, used the way the reference's own tests
use them (reference tests/test_v7_correctness.py)."""
import importlib
import os
import sys

import pytest
import torch

import attention_oracle as orc

pytestmark = pytest.mark.gpu

PKG_DIR = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "610sample_b200")
DEV = "cuda"


@pytest.fixture(scope="module")
def mods():
    # the reference's way of importing: the directory on sys.path
    if PKG_DIR not in sys.path:
        sys.path.insert(0, PKG_DIR)
    import attention_cuda
    from attention import flash_attention_v7
    return attention_cuda, flash_attention_v7


REF_CONFIGS = [  # reference tests/test_v7_correctness.py:255-266 (D = 80, 96 go to the SIMT kernels)
    (1, 1, 32, 128, 64, 96, 1), (1, 2, 64, 256, 64, 192, 2), (2, 4, 64, 256, 64, 192, 3),
    (1, 1, 64, 256, 80, 192, 1), (1, 1, 64, 256, 96, 192, 2), (1, 1, 64, 256, 64, 192, 0),
    (1, 2, 32, 128, 64, 96, 0),
]


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("cfg", REF_CONFIGS)
def test_scalar_probe_double_backward(mods, cfg, dtype):
    """The reference's double-backward check (scalar probe, dO = ones), with its
    tolerances (bf16 1.5e-2, fp16 5e-3), plus the gradient with respect to dO."""
    _, flash = mods
    B, H, Nq, Nkv, D, ws, cid = cfg
    torch.manual_seed(42)
    Qr = torch.randn(B, H, Nq, D).to(dtype)
    Kr = torch.randn(B, H, Nkv, D).to(dtype)
    Vr = torch.randn(B, H, Nkv, D).to(dtype)
    uQ, uK, uV = torch.randn(B, H, Nq, D).to(dtype), torch.randn(B, H, Nkv, D).to(dtype), torch.randn(B, H, Nkv, D).to(dtype)
    ones = torch.ones_like(Qr)
    ref = orc.closed_form_all(Qr, Kr, Vr, ones, uQ, uK, uV, window_size=ws, chunk_id=cid)

    Q, K, V = (t.to(DEV).requires_grad_(True) for t in (Qr, Kr, Vr))
    O = flash(Q, K, V, window_size=ws, chunk_id=cid)
    grads = torch.autograd.grad(O.sum(), [Q, K, V], create_graph=True)
    h = sum((g_ * u.to(DEV)).sum() for g_, u in zip(grads, (uQ, uK, uV)))
    g2 = torch.autograd.grad(h, [Q, K, V])
    tol = 1.5e-2 if dtype == torch.bfloat16 else 5e-3
    for got, n in zip(list(grads) + list(g2), ("dQ", "dK", "dV", "g_Q", "g_K", "g_V")):
        assert torch.allclose(got.detach().float().cpu(), ref[n].float(), atol=tol, rtol=tol), n
    assert torch.allclose(O.detach().float().cpu(), ref["O"].float(), atol=5e-3 if dtype == torch.float16 else 1.5e-2, rtol=1e-2)


def test_random_dO_and_grad_wrt_dO(mods):
    _, flash = mods
    inp = orc.make_inputs(2, 2, 320, 320, 128, seed=8, dtype=torch.bfloat16)
    ref = orc.closed_form_all(*(inp[n] for n in orc.INPUT_NAMES), window_size=320, chunk_id=0)
    Q, K, V, dO = (inp[n].to(DEV).requires_grad_(True) for n in ("Q", "K", "V", "dO"))
    O = flash(Q, K, V, 320, 0)
    dQ, dK, dV = torch.autograd.grad(O, [Q, K, V], grad_outputs=dO, create_graph=True)
    h = (dQ * inp["g_dQ"].to(DEV)).sum() + (dK * inp["g_dK"].to(DEV)).sum() + (dV * inp["g_dV"].to(DEV)).sum()
    g_dO, g_Q, g_K, g_V = torch.autograd.grad(h, [dO, Q, K, V])
    for got, n in ((g_dO, "g_dO"), (g_Q, "g_Q"), (g_K, "g_K"), (g_V, "g_V")):
        r = ref[n].float()
        assert float((got.float().cpu() - r).abs().max()) <= 2e-2 * float(r.abs().max()), n


def test_module_functions_and_return_order(mods):
    ac, _ = mods
    inp = orc.make_inputs(1, 2, 128, 256, 64, seed=9, dtype=torch.bfloat16)
    g = {n: t.to(DEV) for n, t in inp.items()}
    r = ac.v7_forward(Q=g["Q"], K=g["K"], V=g["V"], window_size=200, chunk_id=1)
    assert isinstance(r, list) and len(r) == 2
    O, L = r
    assert O.dtype == torch.bfloat16 and L.dtype == torch.float32 and L.shape == (1, 2, 128)
    r = ac.v7_backward(dO=g["dO"], Q=g["Q"], K=g["K"], V=g["V"], O=O, L=L, window_size=200, chunk_id=1)
    assert [t.shape for t in r] == [g["Q"].shape, g["K"].shape, g["V"].shape]
    r = ac.v7_double_backward(g_dQ=g["g_dQ"], g_dK=g["g_dK"], g_dV=g["g_dV"], dO=g["dO"], Q=g["Q"], K=g["K"],
                              V=g["V"], O=O, L=L, window_size=200, chunk_id=1)
    assert [t.shape for t in r] == [g["Q"].shape, g["Q"].shape, g["K"].shape, g["V"].shape]
    ref = orc.closed_form_all(*(inp[n] for n in orc.INPUT_NAMES), window_size=200, chunk_id=1)
    for got, n in zip(r, ("g_dO", "g_Q", "g_K", "g_V")):
        rr = ref[n].float()
        assert float((got.float().cpu() - rr).abs().max()) <= 2e-2 * float(rr.abs().max()), n
    assert ac.last_launch_count() == 3


def test_non_contiguous_and_offset_inputs(mods):
    ac, _ = mods
    base = torch.randn(1, 2, 130, 3, 64, device=DEV).to(torch.bfloat16)
    Q, K, V = base[:, :, 1:129, 0], base[:, :, 1:129, 1], base[:, :, 1:129, 2]     # strided views
    O, L = ac.v7_forward(Q, K, V, 128, 0)
    O2, L2 = ac.v7_forward(Q.contiguous(), K.contiguous(), V.contiguous(), 128, 0)
    assert torch.equal(O, O2) and torch.equal(L, L2)


def test_errors_are_runtime_errors(mods):
    ac, _ = mods
    q = torch.randn(1, 1, 64, 64)
    with pytest.raises(RuntimeError):
        ac.v7_forward(q, q, q, 64, 0)                                   # not CUDA
    qc = torch.randn(1, 1, 64, 64, device=DEV, dtype=torch.float64)
    with pytest.raises(RuntimeError):
        ac.v7_forward(qc, qc, qc, 64, 0)                                # dtype
    qb = torch.randn(1, 1, 64, 72, device=DEV).to(torch.bfloat16)
    with pytest.raises(RuntimeError):
        ac.v7_forward(qb, qb, qb, 64, 0)                                # D % 16
    qd = torch.randn(1, 1, 64, 256, device=DEV).to(torch.bfloat16)
    with pytest.raises(RuntimeError):
        ac.v7_forward(qd, qd, qd, 64, 0)                                # D too large
    a = torch.randn(1, 1, 64, 64, device=DEV).to(torch.bfloat16)
    b = torch.randn(1, 2, 64, 64, device=DEV).to(torch.bfloat16)
    with pytest.raises(RuntimeError):
        ac.v7_forward(a, b, b, 64, 0)                                   # shape mismatch


def test_memory_scales_linearly(mods):
    """Peak memory of forward, backward and double backward grows with N, not N^2
    (reference tests/test_v7_correctness.py:188-249)."""
    ac, flash = mods
    ws, cid, D = 192, 2, 64

    def peak(fn):
        torch.cuda.synchronize(); torch.cuda.empty_cache(); torch.cuda.reset_peak_memory_stats()
        base = torch.cuda.memory_allocated()
        fn(); torch.cuda.synchronize()
        return torch.cuda.max_memory_allocated() - base

    def run(Nq, Nkv):
        def f():
            Q = torch.randn(1, 1, Nq, D, device=DEV).to(torch.bfloat16).requires_grad_(True)
            K = torch.randn(1, 1, Nkv, D, device=DEV).to(torch.bfloat16).requires_grad_(True)
            V = torch.randn(1, 1, Nkv, D, device=DEV).to(torch.bfloat16).requires_grad_(True)
            O = flash(Q, K, V, window_size=ws, chunk_id=cid)
            grads = torch.autograd.grad(O.sum(), [Q, K, V], create_graph=True)
            torch.autograd.grad(sum(g_.sum() for g_ in grads), [Q, K, V])
        return f
    small, large = peak(run(256, 1024)), peak(run(1024, 4096))
    assert large < 8 * max(small, 1), (small, large)


def test_multi_stream_and_device_guard(mods):
    ac, _ = mods
    inp = orc.make_inputs(1, 2, 256, 256, 64, seed=10, dtype=torch.bfloat16)
    g = {n: t.to(DEV) for n, t in inp.items()}
    O0, L0 = ac.v7_forward(g["Q"], g["K"], g["V"], 256, 0)
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        O1, L1 = ac.v7_forward(g["Q"], g["K"], g["V"], 256, 0)
    s.synchronize()
    assert torch.equal(O0, O1) and torch.equal(L0, L1)


def test_empty_inputs(mods):
    """No keys: every row is fully masked (O = 0, L = -inf, zero gradients).  No queries: the
    key-side gradients are zero.  No kernel of the attention families is launched."""
    ac, _ = mods
    q = torch.randn(2, 3, 40, 64, device=DEV).to(torch.bfloat16)
    k0 = torch.empty(2, 3, 0, 64, device=DEV, dtype=torch.bfloat16)
    O, L = ac.v7_forward(q, k0, k0, 16, 0)
    assert O.shape == q.shape and float(O.float().abs().max()) == 0.0
    assert bool(torch.isinf(L).all()) and bool((L < 0).all())
    dQ, dK, dV = ac.v7_backward(torch.ones_like(q), q, k0, k0, O, L, 16, 0)
    assert float(dQ.float().abs().max()) == 0.0 and dK.numel() == 0 and dV.numel() == 0
    g = ac.v7_double_backward(q, k0, k0, q, q, k0, k0, O, L, 16, 0)
    assert float(g[0].float().abs().max()) == 0.0 and float(g[1].float().abs().max()) == 0.0
    q0 = torch.empty(2, 3, 0, 64, device=DEV, dtype=torch.bfloat16)
    k = torch.randn(2, 3, 50, 64, device=DEV).to(torch.bfloat16)
    O0, L0 = ac.v7_forward(q0, k, k, 16, 0)
    assert O0.numel() == 0 and L0.numel() == 0
    dQ, dK, dV = ac.v7_backward(q0, q0, k, k, O0, L0, 16, 0)
    assert dQ.numel() == 0 and float(dK.float().abs().max()) == 0.0 and float(dV.float().abs().max()) == 0.0
    none = torch.empty(0, 3, 8, 64, device=DEV, dtype=torch.bfloat16)
    O1, L1 = ac.v7_forward(none, none, none, 16, 0)
    assert O1.numel() == 0 and ac.last_launch_count() == 0


def test_double_backward_under_cuda_graph_capture():
    """The call is capturable: under capture every launch stays on the capturing stream (the
    library's helper stream is used by eager calls only), tensor maps travel as kernel parameters,
    nothing is allocated by the library.  The replayed graph must reproduce the eager results bit
    for bit."""
    tcapi = importlib.import_module("610sample_b200.torch_capi")
    capi = importlib.import_module("610sample_b200.capi")
    inp = orc.make_inputs(1, 4, 512, 512, 128, seed=21, dtype=torch.bfloat16)
    g = {n: t.to(DEV) for n, t in inp.items()}
    O, L = tcapi.forward(g["Q"], g["K"], g["V"], 512, 0)
    s = tcapi._shape(g["Q"], g["K"], 512, 0, 0, 0)
    scratch = torch.empty(capi.lib().attn_b200_double_backward_scratch_bytes(s) // 4 + 4, dtype=torch.float32, device=DEV)
    eager = tuple(torch.empty_like(g[n]) for n in ("Q", "Q", "K", "V"))
    tcapi.double_backward(g["g_dQ"], g["g_dK"], g["g_dV"], g["dO"], g["Q"], g["K"], g["V"], O, L, 512, 0,
                          scratch=scratch, out=eager)
    torch.cuda.synchronize()
    out = tuple(torch.zeros_like(t) for t in eager)
    graph = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        with torch.cuda.graph(graph, stream=side):
            tcapi.double_backward(g["g_dQ"], g["g_dK"], g["g_dV"], g["dO"], g["Q"], g["K"], g["V"], O, L, 512, 0,
                                  scratch=scratch, out=out)
    torch.cuda.current_stream().wait_stream(side)
    for _ in range(2):
        for t in out:
            t.zero_()
        graph.replay()
        torch.cuda.synchronize()
        for a, b in zip(eager, out):
            assert torch.equal(a, b)
    assert capi.device_status() == 0


def test_two_host_threads_on_their_own_streams():
    """Two host threads call the C ABI at the same time on different streams (ctypes drops the
    GIL).  They share the device's helper stream and its fork / join events; each must still get
    exactly the results of a serial call."""
    import threading
    tcapi = importlib.import_module("610sample_b200.torch_capi")
    capi = importlib.import_module("610sample_b200.capi")
    cases = []
    for seed in (31, 32):
        inp = orc.make_inputs(1, 8, 1024, 1024, 128, seed=seed, dtype=torch.bfloat16)
        g = {n: t.to(DEV) for n, t in inp.items()}
        O, L = tcapi.forward(g["Q"], g["K"], g["V"], 1024, 0)
        ref = tcapi.double_backward(g["g_dQ"], g["g_dK"], g["g_dV"], g["dO"], g["Q"], g["K"], g["V"], O, L, 1024, 0)
        cases.append((g, O, L, ref))
    torch.cuda.synchronize()
    results = [None, None]
    errors = []

    def work(i):
        try:
            g, O, L, _ = cases[i]
            st = torch.cuda.Stream()
            with torch.cuda.stream(st):
                for _ in range(20):
                    r = tcapi.double_backward(g["g_dQ"], g["g_dK"], g["g_dV"], g["dO"], g["Q"], g["K"], g["V"], O, L, 1024, 0)
            st.synchronize()
            results[i] = r
        except Exception as e:  # noqa: BLE001
            errors.append(e)

    th = [threading.Thread(target=work, args=(i,)) for i in range(2)]
    for x in th:
        x.start()
    for x in th:
        x.join()
    assert not errors, errors
    for i in range(2):
        for a, b in zip(cases[i][3], results[i]):
            assert torch.equal(a, b)
    assert capi.device_status() == 0
