"""CPU tests of the host side: the autograd wiring of attention.py (run against
an oracle-backed stand-in for the compiled module) and the sharding helpers,
including a two-process gloo run."""
import importlib
import os
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import attention_oracle as orc

att = importlib.import_module("610sample_b200.attention")
sharding = importlib.import_module("610sample_b200.sharding")


class OracleBackend:
    """CPU stand-in with the attention_cuda call surface, used only to exercise the
    autograd.Function plumbing without a GPU."""
    calls = []

    @staticmethod
    def _all(Q, K, V, dO, gq, gk, gv, ws, cid, mm):
        return orc.closed_form_all(Q, K, V, dO, gq, gk, gv, window_size=ws, chunk_id=cid, mask_mode=mm)

    def v7_forward(self, Q, K, V, ws, cid, mm=0):
        self.calls.append("fwd")
        z = torch.zeros_like
        r = self._all(Q, K, V, z(Q), z(Q), z(K), z(V), ws, cid, mm)
        return [r["O"].to(Q.dtype), r["L"].float()]

    def v7_backward(self, dO, Q, K, V, O, L, ws, cid, mm=0):
        self.calls.append("bwd")
        z = torch.zeros_like
        r = self._all(Q, K, V, dO, z(Q), z(K), z(V), ws, cid, mm)
        return [r[n].to(Q.dtype) for n in ("dQ", "dK", "dV")]

    def v7_double_backward(self, gq, gk, gv, dO, Q, K, V, O, L, ws, cid, mm=0):
        self.calls.append("dbl")
        r = self._all(Q, K, V, dO, gq, gk, gv, ws, cid, mm)
        return [r[n].to(Q.dtype) for n in ("g_dO", "g_Q", "g_K", "g_V")]


@pytest.fixture()
def oracle_backend(monkeypatch):
    b = OracleBackend()
    b.calls = []
    monkeypatch.setattr(att, "_attention_cuda", b)
    return b


def test_autograd_wiring_matches_double_autograd(oracle_backend):
    inp = orc.make_inputs(1, 2, 24, 40, 16, seed=3, dtype=torch.float64)
    ws, cid = 30, 1
    Q, K, V = (inp[n].clone().requires_grad_(True) for n in ("Q", "K", "V"))
    dO = inp["dO"].clone().requires_grad_(True)
    O = att.flash_attention_v7(Q, K, V, ws, cid)
    dQ, dK, dV = torch.autograd.grad(O, [Q, K, V], grad_outputs=dO, create_graph=True)
    h = (dQ * inp["g_dQ"]).sum() + (dK * inp["g_dK"]).sum() + (dV * inp["g_dV"]).sum()
    g_dO, g_Q, g_K, g_V = torch.autograd.grad(h, [dO, Q, K, V])
    assert oracle_backend.calls == ["fwd", "bwd", "dbl"]
    mask = orc.visibility_mask(cid, 24, 40, ws)
    ref = orc.autograd_all(*(inp[n] for n in orc.INPUT_NAMES), mask)
    for got, n in ((O, "O"), (dQ, "dQ"), (dK, "dK"), (dV, "dV"), (g_dO, "g_dO"), (g_Q, "g_Q"), (g_K, "g_K"), (g_V, "g_V")):
        assert torch.allclose(got.detach(), ref[n], rtol=1e-9, atol=1e-10), n


def test_missing_tangents_become_zeros(oracle_backend):
    inp = orc.make_inputs(1, 1, 16, 16, 16, seed=4, dtype=torch.float64)
    Q, K, V = (inp[n].clone().requires_grad_(True) for n in ("Q", "K", "V"))
    O = att.flash_attention_v7(Q, K, V, 16, 0)
    (dQ,) = torch.autograd.grad(O.sum(), [Q], create_graph=True)      # dK, dV unused -> None tangents
    (gK,) = torch.autograd.grad((dQ * inp["g_dQ"]).sum(), [K])
    z = torch.zeros_like
    ref = orc.closed_form_all(inp["Q"], inp["K"], inp["V"], torch.ones_like(inp["Q"]), inp["g_dQ"], z(inp["K"]),
                              z(inp["V"]), window_size=16, chunk_id=0)
    assert torch.allclose(gK, ref["g_K"], rtol=1e-9, atol=1e-10)


def test_mask_mode_keyword_reaches_backend(oracle_backend):
    inp = orc.make_inputs(1, 1, 8, 8, 16, seed=5, dtype=torch.float64)
    O = att.flash_attention_v7(inp["Q"], inp["K"], inp["V"], 1, 0, mask_mode=1)
    ref = orc.math_attention(inp["Q"], inp["K"], inp["V"], torch.ones(8, 8, dtype=torch.bool))
    assert torch.allclose(O, ref, rtol=1e-9, atol=1e-10)


def test_shard_range_partitions():
    for n in (0, 1, 7, 64, 65):
        for world in (1, 2, 3, 8):
            got = [sharding.shard_range(n, world, r) for r in range(world)]
            assert got[0][0] == 0 and got[-1][1] == n
            assert all(a[1] == b[0] for a, b in zip(got, got[1:]))
            sizes = [e - b for b, e in got]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        sharding.shard_range(4, 2, 2)


def _gloo_worker(rank, world, port, out):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        # each rank computes the HVP of its own (batch, head) slices with the oracle; the
        # concatenation over ranks must equal the unsharded result (no collective on the path)
        inp = orc.make_inputs(1, 6, 16, 16, 16, seed=11, dtype=torch.float64)
        b, e = sharding.shard_range(6, world, rank)
        mine = {n: t[:, b:e] for n, t in inp.items()}
        r = orc.closed_form_all(*(mine[n] for n in orc.INPUT_NAMES), window_size=16, chunk_id=0)
        parts = [None] * world
        dist.all_gather_object(parts, (b, e, r["g_Q"]))
        slow = sharding.max_over_ranks(1.0 + rank)
        if rank == 0:
            full = orc.closed_form_all(*(inp[n] for n in orc.INPUT_NAMES), window_size=16, chunk_id=0)
            cat = torch.cat([p[2] for p in sorted(parts, key=lambda p: p[0])], dim=1)
            out.put((bool(torch.equal(cat, full["g_Q"])), slow))
    finally:
        dist.destroy_process_group()


def test_two_rank_gloo_sharding():
    ctx = mp.get_context("spawn")
    out = ctx.SimpleQueue()
    port = 29500 + (os.getpid() % 2000)
    procs = [ctx.Process(target=_gloo_worker, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    same, slow = out.get()
    assert same and slow == 2.0
