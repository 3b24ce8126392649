"""Generate the golden fixtures in this folder from the reference project itself.

Run once, in a container that has the reference checkout:

    python tests/golden/make_golden.py /path/to/reference

It imports the reference's own ``make_sw_causal_mask`` and ``reference_attention``
(``e2e/ttt_pytorch/model.py:141-171``), runs forward, first backward
(``create_graph=True``) and the Hessian-vector product by double autograd in
fp64 on seeded inputs, and stores inputs + outputs as compressed ``.npz`` files.
The GPU box has no reference checkout, so the tests read only these files.

Cases:
  * the seven shape tuples of the reference's kernel unit tests
    (``tests/test_v7_correctness.py:255-266``), inputs rounded to bf16 first;
  * one (batch, head) slice of the CPU-runnable config (B2 H4 N256 D64 causal,
    fp32, seed 0), plus per-tensor fp64 norms over all of its heads;
  * edge cases: ragged N, window smaller than N, N_kv < N_q (fully masked rows).
"""
from __future__ import annotations

import importlib.util
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "..", "..", "oracle"))
from attention_oracle import INPUT_NAMES, OUTPUT_NAMES, make_inputs  # noqa: E402


def load_reference_module(ref_root: str):
    path = os.path.join(ref_root, "e2e", "ttt_pytorch", "model.py")
    spec = importlib.util.spec_from_file_location("ref_model", path)
    mod = importlib.util.module_from_spec(spec)
    sys.modules["ref_model"] = mod          # dataclasses look their module up by name
    spec.loader.exec_module(mod)
    return mod


def load_reference(ref_root: str):
    mod = load_reference_module(ref_root)
    return mod.make_sw_causal_mask, mod.reference_attention


def run_reference(ref, inp, window_size, chunk_id):
    make_mask, ref_attn = ref
    Q, K, V, dO = (inp[n].double().requires_grad_(True) for n in ("Q", "K", "V", "dO"))
    gq, gk, gv = (inp[n].double() for n in ("g_dQ", "g_dK", "g_dV"))
    B, H, N_q, D = Q.shape
    N_kv = K.shape[2]
    mask = make_mask(chunk_id, N_q, N_kv, window_size, "cpu")
    O = torch.stack([ref_attn(Q[b], K[b], V[b], mask) for b in range(B)])
    dQ, dK, dV = torch.autograd.grad(O, [Q, K, V], grad_outputs=dO, create_graph=True)
    h = (dQ * gq).sum() + (dK * gk).sum() + (dV * gv).sum()
    g_dO, g_Q, g_K, g_V = torch.autograd.grad(h, [dO, Q, K, V])
    scale = 1.0 / (D ** 0.5)
    S = (Q.detach() @ K.detach().transpose(-2, -1)) * scale
    L = torch.logsumexp(S.masked_fill(~mask, float("-inf")), dim=-1)
    out = dict(O=O, L=L, dQ=dQ, dK=dK, dV=dV, g_dO=g_dO, g_Q=g_Q, g_K=g_K, g_V=g_V)
    return {k: v.detach() for k, v in out.items()}, mask


# (name, B, H, N_q, N_kv, D, window_size, chunk_id, seed, input rounding dtype)
CASES = [
    ("ref_unit_0", 1, 1, 32, 128, 64, 96, 1, 42, torch.bfloat16),
    ("ref_unit_1", 1, 2, 64, 256, 64, 192, 2, 42, torch.bfloat16),
    ("ref_unit_2", 2, 4, 64, 256, 64, 192, 3, 42, torch.bfloat16),
    ("ref_unit_3", 1, 1, 64, 256, 80, 192, 1, 42, torch.bfloat16),
    ("ref_unit_4", 1, 1, 64, 256, 96, 192, 2, 42, torch.bfloat16),
    ("ref_unit_5", 1, 1, 64, 256, 64, 192, 0, 42, torch.bfloat16),
    ("ref_unit_6", 1, 2, 32, 128, 64, 96, 0, 42, torch.bfloat16),
    ("edge_ragged", 1, 2, 100, 100, 64, 100, 0, 7, torch.bfloat16),
    ("edge_window", 1, 1, 192, 192, 128, 50, 0, 8, torch.bfloat16),
    ("edge_masked_rows", 1, 1, 96, 40, 64, 1000, 0, 9, torch.bfloat16),
    ("edge_d128_rect", 1, 2, 72, 200, 128, 150, 1, 10, torch.bfloat16),
]


def main():
    if len(sys.argv) != 2:
        raise SystemExit("usage: python tests/golden/make_golden.py <path-to-reference-checkout>")
    ref_root = sys.argv[1]
    ref = load_reference(ref_root)
    torch.set_num_threads(8)
    for name, B, H, N_q, N_kv, D, ws, cid, seed, rdt in CASES:
        inp = make_inputs(B, H, N_q, N_kv, D, seed=seed, dtype=rdt)
        out, mask = run_reference(ref, inp, ws, cid)
        blob = {"meta": np.array([B, H, N_q, N_kv, D, ws, cid, seed], dtype=np.int64),
                "mask": mask.numpy()}
        for n in INPUT_NAMES:   # bf16 values, stored exactly as their 16-bit patterns
            blob["in_" + n] = inp[n].view(torch.int16).numpy().view(np.uint16)
        for n in OUTPUT_NAMES:
            blob["out_" + n] = out[n].float().numpy()
        np.savez_compressed(os.path.join(HERE, name + ".npz"), **blob)
        print(name, "ok")

    # CPU-runnable config: full run, store one head + norms of every tensor
    B, H, N, D = 2, 4, 256, 64
    inp = make_inputs(B, H, N, N, D, seed=0, dtype=torch.float32)
    out, mask = run_reference(ref, inp, N, 0)
    assert bool((mask == torch.ones(N, N, dtype=torch.bool).tril()).all())
    b, h = 1, 2
    blob = {"meta": np.array([B, H, N, N, D, N, 0, 0], dtype=np.int64),
            "head": np.array([b, h], dtype=np.int64)}
    for n in INPUT_NAMES:
        blob["in_" + n] = inp[n][b, h].numpy()
    for n in OUTPUT_NAMES:
        blob["out_" + n] = out[n][b, h].float().numpy()
        blob["norm_" + n] = np.array(float(out[n].double().norm()))
        blob["sum_" + n] = np.array(float(out[n].double().sum()))
    np.savez_compressed(os.path.join(HERE, "config1_head.npz"), **blob)
    print("config1_head ok")

    # the step before attention: the reference's own RMSNorm and apply_rotary_emb on [n_tok, H, d]
    mod = load_reference_module(ref_root)
    g = torch.Generator(device="cpu").manual_seed(11)
    n_tok, H, d, pos0, norm_from = 48, 3, 64, 5, 16
    x = torch.randn(n_tok, H, d, generator=g).to(torch.bfloat16)
    w = (1.0 + 0.1 * torch.randn(d, generator=g)).to(torch.bfloat16)
    norm = mod.RMSNorm(d, eps=1e-6).to(torch.bfloat16)
    with torch.no_grad():
        norm.weight.copy_(w)
        fc = mod.precompute_freqs_cis(d, 128)
        y = torch.cat([x[:norm_from], norm(x[norm_from:])], dim=0)
        out = mod.apply_rotary_emb(y, fc[pos0:pos0 + n_tok]).permute(1, 0, 2).unsqueeze(0)
    np.savez_compressed(os.path.join(HERE, "prep_qk_norm_rope.npz"),
                        meta=np.array([n_tok, H, d, pos0, norm_from], dtype=np.int64),
                        x=x.view(torch.int16).numpy().view(np.uint16), w=w.view(torch.int16).numpy().view(np.uint16),
                        out=out.float().numpy())
    print("prep_qk_norm_rope ok")


if __name__ == "__main__":
    main()
