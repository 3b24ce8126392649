"""GPU test of the allocation-free double-backward entry point
(`attn_b200_double_backward_static`).

It is for callers that cannot allocate device memory at the point of the call (a
host application that owns all GPU memory, a runtime with a frozen memory plan):
the per-row scratch is a fixed array inside the library.  The file name sorts last
so that a run that stops at the first failure has already run every other test.

Checked here, through the C ABI: results equal those of the regular entry point
(same kernels, so bitwise) on two calls in a row with different problems -- the
second call finds the first call's values in the shared scratch and must not be
affected by them -- and a problem beyond the fixed capacity is refused.
"""
import importlib

import pytest
import torch

import attention_oracle as orc

pytestmark = pytest.mark.gpu

tcapi = importlib.import_module("610sample_b200.torch_capi")
capi = importlib.import_module("610sample_b200.capi")
DEV = "cuda"


def _problem(B, H, Nq, Nkv, D, ws, cid, seed, dtype):
    inp = orc.make_inputs(B, H, Nq, Nkv, D, seed=seed, dtype=dtype)
    g = {n: t.to(DEV) for n, t in inp.items()}
    O, L = tcapi.forward(g["Q"], g["K"], g["V"], ws, cid)
    args = (g["g_dQ"], g["g_dK"], g["g_dV"], g["dO"], g["Q"], g["K"], g["V"], O, L, ws, cid)
    return inp, args


def test_static_scratch_matches_regular_entry_point_twice_in_a_row():
    # call 1: tensor-core kernels, causal;  call 2: a different shape, rectangular window
    for (B, H, Nq, Nkv, D, ws, cid, seed) in [(2, 3, 384, 384, 128, 384, 0, 21), (1, 2, 200, 456, 64, 300, 1, 22)]:
        inp, args = _problem(B, H, Nq, Nkv, D, ws, cid, seed, torch.bfloat16)
        want = tcapi.double_backward(*args)
        outs = tuple(torch.full_like(t, float("nan")) for t in want)      # pre-allocated by the caller
        got = tcapi.double_backward_static(*args, out=outs)
        torch.cuda.synchronize()
        for a, b, n in zip(got, want, ("g_dO", "g_Q", "g_K", "g_V")):
            assert torch.equal(a, b), n
        ref = orc.closed_form_all(*(inp[n] for n in orc.INPUT_NAMES), window_size=ws, chunk_id=cid)
        for a, n in zip(got, ("g_dO", "g_Q", "g_K", "g_V")):
            r = ref[n].float()
            assert float((a.float().cpu() - r).abs().max()) <= 2e-2 * max(1.0, float(r.abs().max())), n
    assert capi.device_status() == 0


def test_static_scratch_fp32_kernels_and_repeat():
    inp, args = _problem(1, 2, 96, 160, 80, 120, 1, 23, torch.float32)     # SIMT family
    want = tcapi.double_backward(*args)
    first = tcapi.double_backward_static(*args)
    second = tcapi.double_backward_static(*args)                           # same problem again
    torch.cuda.synchronize()
    for a, b, c in zip(first, second, want):
        assert torch.equal(a, c) and torch.equal(b, c)


def test_static_scratch_at_exactly_its_capacity_and_without_allocating():
    """The largest accepted problem (B*H*N_q == ATTN_B200_STATIC_SCRATCH_ROWS: every element of
    the fixed array is used) gives the regular entry point's results bit for bit, and a second
    call with caller-provided outputs leaves the device's free memory and PyTorch's allocation
    counter exactly where they were."""
    B, H, N, D = 16, 16, 4096, 16
    assert B * H * N == capi.STATIC_SCRATCH_ROWS
    inp, args = _problem(B, H, N, N, D, N, 0, 24, torch.bfloat16)
    want = tcapi.double_backward(*args)
    outs = tuple(torch.full_like(t, float("nan")) for t in want)
    tcapi.double_backward_static(*args, out=outs)          # first call: kernels and the array's address are loaded
    torch.cuda.synchronize()
    for a, b, n in zip(outs, want, ("g_dO", "g_Q", "g_K", "g_V")):
        assert torch.equal(a, b), n
    for t in outs:
        t.fill_(float("nan"))
    torch.cuda.synchronize()
    free0, _ = torch.cuda.mem_get_info()
    alloc0, reserved0 = torch.cuda.memory_allocated(), torch.cuda.memory_reserved()
    tcapi.double_backward_static(*args, out=outs)
    torch.cuda.synchronize()
    free1, _ = torch.cuda.mem_get_info()
    assert free1 == free0 and torch.cuda.memory_allocated() == alloc0 and torch.cuda.memory_reserved() == reserved0
    for a, b, n in zip(outs, want, ("g_dO", "g_Q", "g_K", "g_V")):
        assert torch.equal(a, b), n
    assert capi.device_status() == 0


def test_static_scratch_empty_problem_beyond_capacity_is_not_refused():
    """N_kv == 0: nothing to compute, the outputs are zero, and the row limit does not apply."""
    rows_over = capi.STATIC_SCRATCH_ROWS // 64 + 1
    q = torch.full((rows_over, 1, 64, 64), float("nan"), device=DEV, dtype=torch.bfloat16)
    kv = torch.empty(rows_over, 1, 0, 64, device=DEV, dtype=torch.bfloat16)
    L = torch.zeros(rows_over, 1, 64, device=DEV)
    s = capi.make_shape(rows_over, 1, 64, 0, 64, 64, 0, 0, capi.ATTN_BF16)
    g_dO, g_Q = torch.full_like(q, float("nan")), torch.full_like(q, float("nan"))
    p = q.data_ptr()
    rc = capi.lib().attn_b200_double_backward_static(s, p, None, None, p, p, None, None, p, L.data_ptr(),
                                                     g_dO.data_ptr(), g_Q.data_ptr(), None, None, torch.cuda.current_stream().cuda_stream)
    assert rc == capi.ATTN_OK, capi.lib().attn_b200_last_error()
    torch.cuda.synchronize()
    assert float(g_dO.float().abs().max()) == 0.0 and float(g_Q.float().abs().max()) == 0.0


def test_static_scratch_rejects_problems_beyond_its_capacity():
    q = torch.zeros(1, 1, 64, 64, device=DEV, dtype=torch.bfloat16)
    L = torch.zeros(1, 1, 64, device=DEV)
    too_many = capi.STATIC_SCRATCH_ROWS // 64 + 1                          # B*H*N_q just over the limit
    s = capi.make_shape(too_many, 1, 64, 64, 64, 64, 0, 0, capi.ATTN_BF16)
    p = q.data_ptr()
    rc = capi.lib().attn_b200_double_backward_static(s, p, p, p, p, p, p, p, p, L.data_ptr(), p, p, p, p, None)
    assert rc == capi.ATTN_ETOOLARGE
    assert b"exceed" in capi.lib().attn_b200_last_error()
    torch.cuda.synchronize()
    assert capi.device_status() == 0                                       # and nothing was launched or broken
