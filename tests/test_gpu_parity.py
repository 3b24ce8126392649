"""GPU parity tests: the CUDA kernels, called through the C ABI, against the CPU
oracle and the golden fixtures produced by the reference's own code.

Tolerances
  * fp32 inputs (SIMT kernels): norm-wise relative error < 1e-4 against the fp64 oracle.
  * bf16 / fp16 inputs: every output within `HALF_RTOL * max|ref| ` max-abs of the fp64
    oracle evaluated on the same rounded inputs (bf16 2.0e-2, fp16 3e-3: output rounding
    alone is 2^-9 resp. 2^-12 relative), and, for bf16, max-abs error no worse than 2x that
    of the reference path (PyTorch math attention differentiated twice in bf16).
"""
import importlib
import math

import pytest
import torch

import attention_oracle as orc
from _util import golden_case_names, load_config1_head, load_golden, record_errors

pytestmark = pytest.mark.gpu

tcapi = importlib.import_module("610sample_b200.torch_capi")
capi = importlib.import_module("610sample_b200.capi")

HALF_RTOL = {torch.bfloat16: 2.0e-2, torch.float16: 3.0e-3}
DEV = "cuda"


def run_all(inp, ws, cid, mm, impl):
    g = {n: t.to(DEV) for n, t in inp.items()}
    O, L = tcapi.forward(g["Q"], g["K"], g["V"], ws, cid, mm, impl)
    dQ, dK, dV = tcapi.backward(g["dO"], g["Q"], g["K"], g["V"], O, L, ws, cid, mm, impl)
    g_dO, g_Q, g_K, g_V = tcapi.double_backward(g["g_dQ"], g["g_dK"], g["g_dV"], g["dO"], g["Q"], g["K"], g["V"],
                                                O, L, ws, cid, mm, impl)
    torch.cuda.synchronize()
    assert capi.device_status() == 0
    out = dict(O=O, L=L, dQ=dQ, dK=dK, dV=dV, g_dO=g_dO, g_Q=g_Q, g_K=g_K, g_V=g_V)
    return {n: t.float().cpu() for n, t in out.items()}


def check_half(got, ref, dtype, what=""):
    for n in orc.OUTPUT_NAMES:
        r = torch.nan_to_num(ref[n].double(), neginf=0.0)
        v = got[n].double()
        if n == "L":
            assert torch.equal(torch.isinf(got[n]), torch.isinf(ref[n].float())), f"{what} L: -inf rows differ"
            v = torch.nan_to_num(v, neginf=0.0)
            assert (v - r).abs().max() <= 1e-4 * max(1.0, float(r.abs().max())), f"{what} L"
            continue
        assert torch.isfinite(v).all(), f"{what} {n}: non-finite values"
        tol = HALF_RTOL[dtype] * max(1.0, float(r.abs().max()))
        err = float((v - r).abs().max())
        assert err <= tol, f"{what} {n}: max-abs {err:.3e} > {tol:.3e}"


@pytest.mark.parametrize("name", golden_case_names())
@pytest.mark.parametrize("impl", ["simt", "tensor"])
def test_golden_fixtures(name, impl):
    meta, inp, ref, _ = load_golden(name)
    got = run_all(inp, meta["window_size"], meta["chunk_id"], 0, 1 if impl == "simt" else 2)
    check_half(got, ref, torch.bfloat16, f"{name}/{impl}")


def test_fp32_reference_config_within_1e4():
    """CPU-runnable reference case: causal, fp32, B2 H4 N256 D64, seed 0."""
    (b, h), _, head_ref, norms, _ = load_config1_head()
    inp = orc.make_inputs(2, 4, 256, 256, 64, seed=0, dtype=torch.float32)
    got = run_all(inp, 256, 0, 0, 0)
    for n in orc.OUTPUT_NAMES:
        assert orc.rel_err(got[n][b, h], head_ref[n]) < 1e-4, n
        assert abs(float(got[n].double().norm()) - norms[n]) < 1e-4 * norms[n], n
    ref = orc.closed_form_all(*(inp[n] for n in orc.INPUT_NAMES), window_size=256, chunk_id=0)
    for n in orc.OUTPUT_NAMES:
        assert orc.rel_err(got[n], ref[n]) < 1e-4, n


def reference_path_errors(inp, mask, oracle):
    """max-abs error of the reference path (math attention, double autograd) run in the
    inputs' own half precision on the GPU, against the fp64 oracle."""
    dt = inp["Q"].dtype
    out = orc.autograd_all(*(inp[n].to(DEV) for n in orc.INPUT_NAMES), mask.to(DEV), compute_dtype=dt)
    return {n: orc.max_abs_err(out[n].float().cpu(), oracle[n]) for n in orc.OUTPUT_NAMES if n != "L"}


@pytest.mark.parametrize("shape", [
    # B, H, N_q, N_kv, D, window, chunk, mask_mode, qk_scale
    (2, 2, 512, 512, 128, 512, 0, 0, 1.0),       # causal, the headline head dimension
    (1, 4, 512, 512, 64, 512, 0, 1, 0.5),        # no mask, inputs scaled like the non-causal config
    (1, 2, 384, 640, 64, 300, 2, 0, 1.0),        # rectangular sliding window
    (1, 2, 512, 512, 128, 512, 0, 0, 2.0),       # peaked softmax rows
])
def test_bf16_error_within_twice_reference_path(shape):
    B, H, Nq, Nkv, D, ws, cid, mm, qk = shape
    inp = orc.make_inputs(B, H, Nq, Nkv, D, seed=1, dtype=torch.bfloat16, qk_scale=qk, v_scale=0.5 if mm else 1.0)
    oracle = orc.closed_form_all(*(inp[n] for n in orc.INPUT_NAMES), window_size=ws, chunk_id=cid, mask_mode=mm)
    got = run_all(inp, ws, cid, mm, 2)
    ref_err = reference_path_errors(inp, orc.visibility_mask(cid, Nq, Nkv, ws, mm), oracle)
    for n, e_ref in ref_err.items():
        e = orc.max_abs_err(got[n], oracle[n])
        assert e <= 2.0 * e_ref + 1e-6, f"{n}: ours {e:.3e} vs reference path {e_ref:.3e}"


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("shape", [
    (1, 1, 1, 1, 64, 1, 0, 0), (1, 1, 129, 65, 64, 1000, 0, 0), (1, 2, 200, 333, 128, 77, 3, 0),
    (1, 1, 64, 512, 128, 512, 0, 0), (2, 1, 300, 300, 64, 300, 0, 1), (1, 1, 96, 40, 128, 1000, 0, 0),
    (1, 3, 640, 640, 128, 1, 0, 0),
])
def test_ragged_and_edge_shapes_tensor(shape, dtype):
    B, H, Nq, Nkv, D, ws, cid, mm = shape
    inp = orc.make_inputs(B, H, Nq, Nkv, D, seed=2, dtype=dtype)
    oracle = orc.closed_form_all(*(inp[n] for n in orc.INPUT_NAMES), window_size=ws, chunk_id=cid, mask_mode=mm)
    got = run_all(inp, ws, cid, mm, 2)
    check_half(got, oracle, dtype, str(shape))


@pytest.mark.parametrize("impl", [1, 2])
@pytest.mark.parametrize("D", [16, 48, 80, 96, 112])
def test_other_head_dims(D, impl):
    """Head dimensions between the two tile widths (the reference builds 64, 80 and 96): the
    tensor-core kernels run them zero-padded to the next tile width."""
    inp = orc.make_inputs(1, 2, 70, 150, D, seed=3, dtype=torch.bfloat16)
    oracle = orc.closed_form_all(*(inp[n] for n in orc.INPUT_NAMES), window_size=100, chunk_id=1)
    got = run_all(inp, 100, 1, 0, impl)
    check_half(got, oracle, torch.bfloat16, f"D={D}")


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("D,cid", [(64, 0), (64, 3), (64, 7), (96, 5), (80, 8)])
def test_chunked_sliding_window_shapes(D, cid, dtype):
    """The reference's own workload (tests/test_ttt_e2e_bench.py:156-161): 1024 queries of chunk
    `cid` against 9216 keys (8192 of history, left-padded while the history is shorter) under a
    sliding window of 8192.  Two heads against the fp64 oracle."""
    Nq, Nkv, ws = 1024, 9216, 8192
    inp = orc.make_inputs(1, 2, Nq, Nkv, D, seed=11 + cid, dtype=dtype)
    oracle = orc.closed_form_all(*(inp[n] for n in orc.INPUT_NAMES), window_size=ws, chunk_id=cid)
    got = run_all(inp, ws, cid, 0, 0)
    check_half(got, oracle, dtype, f"chunk {cid} D={D}")


def _full_size_case(name, B, H, N, D, heads, qk_scale):
    """One BASELINE configuration at its full sequence length: `heads` (batch*head indices of the
    seeded workload the bench uses) through forward, backward and double backward; every output
    against the fp64 closed form evaluated on the GPU, and against the stated tolerance: bf16
    max-abs error no worse than 2x that of the reference path (math attention differentiated
    twice by PyTorch in bf16), both measured against the fp64 oracle."""
    full = orc.make_inputs(1, B * H, N, N, D, seed=0, dtype=torch.bfloat16, qk_scale=qk_scale)
    inp = {n: t[:, list(heads)].contiguous() for n, t in full.items()}
    del full
    got = run_all(inp, N, 0, 0, 2)
    mask = orc.visibility_mask(0, N, N, N, device=DEV)
    table = {}
    for i, h in enumerate(heads):
        one = {n: t[:, i:i + 1] for n, t in inp.items()}
        oracle = orc.closed_form_all(*(one[n] for n in orc.INPUT_NAMES), window_size=N, chunk_id=0, device=DEV)
        sub = {n: t[:, i:i + 1] for n, t in got.items()}
        check_half(sub, oracle, torch.bfloat16, f"{name} head {h}")
        ref_out = orc.autograd_all(*(one[n].to(DEV) for n in orc.INPUT_NAMES), mask, compute_dtype=torch.bfloat16)
        for n in orc.OUTPUT_NAMES:
            if n == "L":
                continue
            e_ref = orc.max_abs_err(ref_out[n].float().cpu(), oracle[n])
            e = orc.max_abs_err(sub[n], oracle[n])
            table[f"head{h}/{n}"] = dict(ours=e, reference_path=e_ref, max_abs_oracle=float(oracle[n].abs().max()))
            assert e <= 2.0 * e_ref + 1e-6, f"{name} head {h} {n}: ours {e:.3e} vs reference path {e_ref:.3e}"
        del ref_out, oracle
        torch.cuda.empty_cache()
    record_errors(name, table)


def test_headline_config_against_fp64_oracle_and_twice_reference_path():
    """BASELINE configs[2], the configuration the metric is quoted on: bf16 causal, B=4, H=16,
    N=4096, D=128, inputs N(0,1) from seed 0 (the tensors bench.py times).  Two of the 64 heads."""
    _full_size_case("headline_N4096_D128", 4, 16, 4096, 128, (0, 37), 1.0)


def test_long_context_config_against_fp64_oracle_and_twice_reference_path():
    """BASELINE configs[3]: bf16 causal, B=1, H=32, N=16384, D=128, Q and K scaled by 2 (peaked
    softmax rows).  One of the 32 heads; the fp64 oracle and the bf16 double-autograd reference
    path both run on the GPU (the latter holds about ten N x N bf16 matrices)."""
    _full_size_case("long_context_N16384_D128", 1, 32, 16384, 128, (5,), 2.0)


def test_bitwise_reproducible():
    inp = orc.make_inputs(2, 3, 700, 700, 128, seed=4, dtype=torch.bfloat16)
    a = run_all(inp, 700, 0, 0, 2)
    b = run_all(inp, 700, 0, 0, 2)
    for n in orc.OUTPUT_NAMES:
        assert torch.equal(a[n], b[n]), n


def test_tensor_kernels_agree_with_simt_at_n2048():
    """Larger than the oracle finishes quickly on a CPU: the fp32 SIMT kernels (pinned
    against the oracle above) check the tensor-core kernels on the same bf16 inputs."""
    inp = orc.make_inputs(1, 2, 2048, 2048, 128, seed=5, dtype=torch.bfloat16)
    a = run_all(inp, 2048, 0, 0, 2)
    b = run_all(inp, 2048, 0, 0, 1)
    for n in orc.OUTPUT_NAMES:
        if n == "L":
            assert (a[n] - b[n]).abs().max() < 1e-4
        else:
            tol = HALF_RTOL[torch.bfloat16] * float(b[n].abs().max())
            assert float((a[n] - b[n]).abs().max()) <= tol, n


def test_grouped_cta_order_with_a_partial_last_group():
    """300 (batch, head) slices of 4 row tiles: more than 8 waves of CTAs, so the kernels take the
    heads in groups of 64 with a last group of 44.  Tensor-core kernels against the SIMT kernels."""
    inp = orc.make_inputs(3, 100, 512, 512, 64, seed=8, dtype=torch.bfloat16)
    a = run_all(inp, 512, 0, 0, 2)
    b = run_all(inp, 512, 0, 0, 1)
    for n in orc.OUTPUT_NAMES:
        if n == "L":
            assert (a[n] - b[n]).abs().max() < 1e-4
        else:
            tol = HALF_RTOL[torch.bfloat16] * max(1.0, float(b[n].abs().max()))
            assert float((a[n] - b[n]).abs().max()) <= tol, n


def test_linearity_in_tangents_at_headline_size():
    """Size-independent property at N=4096, D=128 causal: the HVP is linear in the tangents,
    HVP(a*g) == a*HVP(g) exactly for a power of two, and HVP(0) == 0."""
    inp = orc.make_inputs(1, 2, 4096, 4096, 128, seed=6, dtype=torch.bfloat16)
    g = {n: t.to(DEV) for n, t in inp.items()}
    O, L = tcapi.forward(g["Q"], g["K"], g["V"], 4096, 0)
    base = tcapi.double_backward(g["g_dQ"], g["g_dK"], g["g_dV"], g["dO"], g["Q"], g["K"], g["V"], O, L, 4096, 0)
    twice = tcapi.double_backward(2 * g["g_dQ"], 2 * g["g_dK"], 2 * g["g_dV"], g["dO"], g["Q"], g["K"], g["V"], O, L, 4096, 0)
    z = torch.zeros_like
    zero = tcapi.double_backward(z(g["Q"]), z(g["K"]), z(g["V"]), g["dO"], g["Q"], g["K"], g["V"], O, L, 4096, 0)
    torch.cuda.synchronize()
    for a, b, c in zip(base, twice, zero):
        assert torch.equal((2 * a.float()), b.float())
        assert float(c.float().abs().max()) == 0.0
    # softmax rows sum to one: with V = 1 the forward output is exactly 1 up to rounding
    O1, _ = tcapi.forward(g["Q"], g["K"], torch.ones_like(g["V"]), 4096, 0)
    assert float((O1.float() - 1).abs().max()) < 1e-2
    assert capi.device_status() == 0


def test_noncausal_config_full_size_heads_against_fp64_oracle():
    """BASELINE configs[1]: bf16, no mask, N=2048, D=64, Q/K/V scaled by 0.5, fp32 LSE.  All 64
    (batch, head) slices run on the GPU; two of them are checked against the fp64 oracle."""
    B, H, N, D = 4, 16, 2048, 64
    inp = orc.make_inputs(B, H, N, N, D, seed=0, dtype=torch.bfloat16, qk_scale=0.5, v_scale=0.5)
    got = run_all(inp, N, 0, 1, 0)
    for (b, h) in ((0, 0), (3, 11)):
        one = {n: t[b:b + 1, h:h + 1] for n, t in inp.items()}
        ref = orc.closed_form_all(*(one[n] for n in orc.INPUT_NAMES), window_size=N, chunk_id=0, mask_mode=1)
        sub = {n: t[b:b + 1, h:h + 1] for n, t in got.items()}
        check_half(sub, ref, torch.bfloat16, f"config2 head {b},{h}")


def test_long_context_peaked_softmax_config():
    """BASELINE configs[3] shape (N=16384, D=128, causal, Q and K scaled by 2) on two heads:
    tensor-core kernels against the fp32 SIMT kernels on the same bf16 inputs, and exact
    linearity of the HVP in the tangents."""
    N, D = 16384, 128
    inp = orc.make_inputs(1, 2, N, N, D, seed=0, dtype=torch.bfloat16, qk_scale=2.0)
    a = run_all(inp, N, 0, 0, 2)
    b = run_all(inp, N, 0, 0, 1)
    for n in orc.OUTPUT_NAMES:
        assert torch.isfinite(a[n]).all(), n
        if n == "L":
            assert (a[n] - b[n]).abs().max() < 2e-4 * float(b[n].abs().max())
        else:
            tol = HALF_RTOL[torch.bfloat16] * max(1.0, float(b[n].abs().max()))
            assert float((a[n] - b[n]).abs().max()) <= tol, n
    g = {n: t.to(DEV) for n, t in inp.items()}
    O, L = tcapi.forward(g["Q"], g["K"], g["V"], N, 0)
    base = tcapi.double_backward(g["g_dQ"], g["g_dK"], g["g_dV"], g["dO"], g["Q"], g["K"], g["V"], O, L, N, 0)
    half = tcapi.double_backward(0.5 * g["g_dQ"], 0.5 * g["g_dK"], 0.5 * g["g_dV"], g["dO"], g["Q"], g["K"], g["V"], O, L, N, 0)
    torch.cuda.synchronize()
    for x, y in zip(base, half):
        assert torch.equal(0.5 * x.float(), y.float())
    assert capi.device_status() == 0
