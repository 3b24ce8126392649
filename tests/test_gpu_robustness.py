"""Robustness of the CUDA path, with nothing that faults a GPU:

* the bounded-wait time-out path runs once, through the primitive self-test (one thread waits
  about a millisecond on a barrier nothing signals): the status word carries the code, the kernel
  returns, and the library works bit-identically afterwards;
* a time-out reaches a caller of the `attention_cuda` module as an exception of its next call (the
  kernel writes its code to a page-locked host word the module looks at; nothing on the good path);
* the tcgen05 primitive self-test (TMA + MMA chain, every operand placement) against torch.matmul;
* guard bands: every output, L and the scratch are carved out of NaN-filled buffers at ragged
  shapes; after the calls the bands are untouched (plain stores and TMA stores alike);
* the phase masks of the double backward reproduce the one-call result bit for bit;
* a call captured into a CUDA graph on one host thread while another thread calls eagerly;
* a thousand back-to-back calls of the three operations at shapes with many CTAs per SM: no
  wait runs out and every result is bit-identical to the first (the hand-offs between the issuing
  warps and the math groups are the kind of protocol whose faults show once in 10^5 CTAs).
"""
import importlib
import os
import sys
import threading

import pytest
import torch

import attention_oracle as orc

pytestmark = pytest.mark.gpu

tcapi = importlib.import_module("610sample_b200.torch_capi")
capi = importlib.import_module("610sample_b200.capi")
PKG_DIR = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "610sample_b200")
DEV = "cuda"
ATTN_EDEVICE = -4


def _hvp_case(seed=41, B=1, H=2, N=384, D=128, dtype=torch.bfloat16, impl=0):
    inp = orc.make_inputs(B, H, N, N, D, seed=seed, dtype=dtype)
    g = {n: t.to(DEV) for n, t in inp.items()}
    O, L = tcapi.forward(g["Q"], g["K"], g["V"], N, 0, 0, impl)
    return (g["g_dQ"], g["g_dK"], g["g_dV"], g["dO"], g["Q"], g["K"], g["V"], O, L, N, 0, 0, impl)


def _run_timeout_selftest():
    A = torch.zeros(128, 64, device=DEV, dtype=torch.bfloat16)
    B = torch.zeros(64, 64, device=DEV, dtype=torch.bfloat16)
    tcapi.selftest_gemm(A, B, 64, 64, 8)        # flag 8: a wait that nothing satisfies, limit about 1 ms
    torch.cuda.synchronize()


def test_bounded_wait_runs_out_and_the_library_keeps_working():
    args = _hvp_case()
    before = tcapi.double_backward(*args)
    torch.cuda.synchronize()
    assert capi.device_status() == 0
    _run_timeout_selftest()                      # returns: the kernel did not hang
    code = capi.C.c_uint32(0)
    rc = capi.lib().attn_b200_device_status(capi.C.byref(code))
    assert rc == ATTN_EDEVICE and code.value == 0x7003
    assert b"bounded wait" in capi.lib().attn_b200_last_error()
    assert capi.device_status() == 0             # reading cleared it
    after = tcapi.double_backward(*args)         # tensor memory was freed by the teardown: the next kernels get theirs
    torch.cuda.synchronize()
    for a, b in zip(before, after):
        assert torch.equal(a, b)
    assert capi.device_status() == 0


def test_timeout_surfaces_as_an_exception_of_a_following_module_call():
    if PKG_DIR not in sys.path:
        sys.path.insert(0, PKG_DIR)
    import attention_cuda
    q = torch.randn(1, 1, 64, 64, device=DEV, dtype=torch.bfloat16)
    attention_cuda.v7_forward(q, q, q, 64, 0)    # registers the module's host mirror of the status word
    torch.cuda.synchronize()
    _run_timeout_selftest()                      # the kernel that gives up writes its code to the mirror too
    with pytest.raises(RuntimeError, match="bounded wait"):
        attention_cuda.v7_forward(q, q, q, 64, 0)
    O, _ = attention_cuda.v7_forward(q, q, q, 64, 0)     # reported once, cleared
    torch.cuda.synchronize()
    assert torch.isfinite(O.float()).all()
    assert capi.device_status() == 0


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("flags", [0, 1, 2, 3, 4, 5])
@pytest.mark.parametrize("N,K", [(64, 64), (128, 128), (64, 128)])
def test_selftest_gemm_against_matmul(N, K, flags, dtype):
    g = torch.Generator(device="cpu").manual_seed(7)
    A = torch.randn(128, K, generator=g).to(dtype).to(DEV)
    Bnk = torch.randn(N, K, generator=g).to(dtype).to(DEV)
    Bop = Bnk.t().contiguous() if flags & 1 else Bnk       # flag 1: B handed over as [K, N]
    C = tcapi.selftest_gemm(A, Bop, N, K, flags)
    torch.cuda.synchronize()
    ref = A.float() @ Bnk.float().t()
    assert float((C - ref).abs().max()) <= 1e-3 * max(1.0, float(ref.abs().max()))
    assert capi.device_status() == 0


GUARD = 256    # elements of guard band on either side (multiples of 16 bytes for every dtype)


def _banded(shape, dtype):
    n = 1
    for s in shape:
        n *= s
    buf = torch.full((n + 2 * GUARD,), float("nan"), device=DEV, dtype=dtype)
    return buf, buf[GUARD:GUARD + n].view(*shape)


def _bands_intact(buf):
    return bool(torch.isnan(buf[:GUARD]).all()) and bool(torch.isnan(buf[-GUARD:]).all())


@pytest.mark.parametrize("impl", [1, 2])
@pytest.mark.parametrize("shape", [(1, 3, 129, 65, 80, 1000, 0), (2, 1, 65, 129, 128, 70, 1), (1, 2, 200, 200, 64, 200, 0)])
def test_guard_bands_stay_untouched(shape, impl):
    B, H, Nq, Nkv, D, ws, cid = shape
    dt = torch.bfloat16
    inp = orc.make_inputs(B, H, Nq, Nkv, D, seed=9, dtype=dt)
    g = {n: t.to(DEV) for n, t in inp.items()}
    s = capi.make_shape(B, H, Nq, Nkv, D, ws, cid, 0, capi.ATTN_BF16, impl)
    lib = capi.lib()
    st = torch.cuda.current_stream().cuda_stream
    bufs = {}

    def band(name, shp, dtype=dt):
        bufs[name], view = _banded(shp, dtype)
        return view

    O, L = band("O", (B, H, Nq, D)), band("L", (B, H, Nq), torch.float32)
    capi.check(lib.attn_b200_forward(s, g["Q"].data_ptr(), g["K"].data_ptr(), g["V"].data_ptr(), O.data_ptr(), L.data_ptr(), st), "forward")
    dQ, dK, dV = band("dQ", (B, H, Nq, D)), band("dK", (B, H, Nkv, D)), band("dV", (B, H, Nkv, D))
    sb = band("bwd_scratch", (lib.attn_b200_backward_scratch_bytes(s) // 4,), torch.float32)
    capi.check(lib.attn_b200_backward(s, g["dO"].data_ptr(), g["Q"].data_ptr(), g["K"].data_ptr(), g["V"].data_ptr(), O.data_ptr(),
                                      L.data_ptr(), dQ.data_ptr(), dK.data_ptr(), dV.data_ptr(), sb.data_ptr(), st), "backward")
    outs = [band(n, (B, H, Nq if n in ("g_dO", "g_Q") else Nkv, D)) for n in ("g_dO", "g_Q", "g_K", "g_V")]
    sh = band("hvp_scratch", (lib.attn_b200_double_backward_scratch_bytes(s) // 4,), torch.float32)
    capi.check(lib.attn_b200_double_backward(s, g["g_dQ"].data_ptr(), g["g_dK"].data_ptr(), g["g_dV"].data_ptr(), g["dO"].data_ptr(),
                                             g["Q"].data_ptr(), g["K"].data_ptr(), g["V"].data_ptr(), O.data_ptr(), L.data_ptr(),
                                             *(t.data_ptr() for t in outs), sh.data_ptr(), st), "double_backward")
    torch.cuda.synchronize()
    assert capi.device_status() == 0
    for name, buf in bufs.items():
        assert _bands_intact(buf), f"{name}: a guard band was written"
    ref = orc.closed_form_all(*(inp[n] for n in orc.INPUT_NAMES), window_size=ws, chunk_id=cid)
    for t, n in zip([O, dQ, dK, dV] + outs, ("O", "dQ", "dK", "dV", "g_dO", "g_Q", "g_K", "g_V")):
        assert torch.isfinite(t.float()).all(), n             # every element inside the bands was written
        r = ref[n].float()
        assert float((t.float().cpu() - r).abs().max()) <= 2e-2 * max(1.0, float(r.abs().max())), n


@pytest.mark.parametrize("impl,D,dtype", [(2, 128, torch.bfloat16), (2, 64, torch.float16), (1, 64, torch.float32)])
def test_phase_masks_reproduce_the_single_call(impl, D, dtype):
    """Scalars (1), then the row side (2), then the column side (4) -- and 1 followed by 6 -- into
    NaN-filled outputs with one scratch give bit for bit what phases = 7 gives."""
    args = _hvp_case(seed=43, B=1, H=3, N=320, D=D, dtype=dtype, impl=impl)
    g_dQ, g_dK, g_dV, dO, Q, K, V, O, L = args[:9]
    want = tcapi.double_backward(*args)
    s = tcapi._shape(Q, K, 320, 0, 0, impl)
    scratch = torch.empty(capi.lib().attn_b200_double_backward_scratch_bytes(s) // 4 + 4, dtype=torch.float32, device=DEV)
    for seq in ((1, 2, 4), (1, 6), (1, 4, 2)):
        out = tuple(torch.full_like(t, float("nan")) for t in want)
        scratch.fill_(float("nan"))
        for ph in seq:
            tcapi.double_backward_phases(*args, scratch=scratch, out=out, phases=ph)
        torch.cuda.synchronize()
        for a, b, n in zip(out, want, ("g_dO", "g_Q", "g_K", "g_V")):
            assert torch.equal(a, b), (seq, n)
    assert capi.device_status() == 0


def test_capture_on_one_thread_while_another_calls_eagerly():
    """The shared helper stream is not used under capture, so a capture in progress on one host
    thread and eager calls of another thread cannot touch each other."""
    a_args, b_args = _hvp_case(seed=51, H=4, N=512), _hvp_case(seed=52, H=4, N=512)
    want_a, want_b = tcapi.double_backward(*a_args), tcapi.double_backward(*b_args)
    s = tcapi._shape(a_args[4], a_args[5], 512, 0, 0, 0)
    scratch = torch.empty(capi.lib().attn_b200_double_backward_scratch_bytes(s) // 4 + 4, dtype=torch.float32, device=DEV)
    out_a = tuple(torch.zeros_like(t) for t in want_a)
    torch.cuda.synchronize()
    errors, eager_results = [], []
    in_capture, eager_done = threading.Event(), threading.Event()

    def eager():
        try:
            in_capture.wait(timeout=30)
            st = torch.cuda.Stream()
            with torch.cuda.stream(st):
                for _ in range(5):
                    r = tcapi.double_backward(*b_args)
            st.synchronize()
            eager_results.append(r)
        except Exception as e:  # noqa: BLE001
            errors.append(e)
        finally:
            eager_done.set()

    th = threading.Thread(target=eager)
    th.start()
    graph = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        with torch.cuda.graph(graph, stream=side, capture_error_mode="thread_local"):
            tcapi.double_backward(*a_args, scratch=scratch, out=out_a)
            in_capture.set()
            eager_done.wait(timeout=60)          # the other thread runs its eager calls while this capture is open
            tcapi.double_backward(*a_args, scratch=scratch, out=out_a)
    th.join()
    torch.cuda.current_stream().wait_stream(side)
    assert not errors, errors
    graph.replay()
    torch.cuda.synchronize()
    for x, y in zip(out_a, want_a):
        assert torch.equal(x, y)
    for x, y in zip(eager_results[0], want_b):
        assert torch.equal(x, y)
    assert capi.device_status() == 0


@pytest.mark.parametrize("shape", [(96, 1024, 1024, 64, 1024, 0, torch.bfloat16), (24, 768, 2304, 128, 2000, 2, torch.float16)])
def test_repeated_calls_stay_bit_identical_and_never_time_out(shape):
    BH, N_q, N_kv, D, ws, cid, dtype = shape
    inp = orc.make_inputs(1, BH, N_q, N_kv, D, seed=17, dtype=dtype)
    g = {n: t.to(DEV) for n, t in inp.items()}

    def once():
        O, L = tcapi.forward(g["Q"], g["K"], g["V"], ws, cid)
        b = tcapi.backward(g["dO"], g["Q"], g["K"], g["V"], O, L, ws, cid)
        h = tcapi.double_backward(g["g_dQ"], g["g_dK"], g["g_dV"], g["dO"], g["Q"], g["K"], g["V"], O, L, ws, cid)
        return (O, L) + tuple(b) + tuple(h)

    first = [t.clone() for t in once()]
    for _ in range(20):
        for _ in range(50):
            outs = once()
        assert capi.device_status() == 0
        for a, b in zip(outs, first):
            assert torch.equal(a, b)
