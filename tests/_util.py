"""Shared helpers for the tests: fixture loading and tolerance bookkeeping."""
import glob
import json
import os

import numpy as np
import torch

from attention_oracle import INPUT_NAMES, OUTPUT_NAMES

GOLDEN_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def golden_case_names():
    names = sorted(os.path.basename(p)[:-4] for p in glob.glob(os.path.join(GOLDEN_DIR, "*.npz")))
    return [n for n in names if n != "config1_head" and not n.startswith("prep_")]


def load_prep_golden():
    """(meta, x bf16 [n_tok, H, d], weight bf16 [d], out fp32 [1, H, n_tok, d]) produced by the
    reference's own RMSNorm and apply_rotary_emb."""
    z = np.load(os.path.join(GOLDEN_DIR, "prep_qk_norm_rope.npz"))
    n_tok, H, d, pos0, norm_from = (int(v) for v in z["meta"])
    x = torch.from_numpy(z["x"].view(np.int16).copy()).view(torch.bfloat16)
    w = torch.from_numpy(z["w"].view(np.int16).copy()).view(torch.bfloat16)
    return dict(n_tok=n_tok, H=H, d=d, pos0=pos0, norm_from=norm_from), x, w, torch.from_numpy(z["out"])


def load_golden(name):
    """Returns (meta dict, inputs dict of bf16 tensors, outputs dict of fp32 tensors, mask)."""
    z = np.load(os.path.join(GOLDEN_DIR, name + ".npz"))
    B, H, N_q, N_kv, D, ws, cid, seed = (int(x) for x in z["meta"])
    meta = dict(B=B, H=H, N_q=N_q, N_kv=N_kv, D=D, window_size=ws, chunk_id=cid, seed=seed)
    inp = {n: torch.from_numpy(z["in_" + n].view(np.int16).copy()).view(torch.bfloat16)
           for n in INPUT_NAMES}
    out = {n: torch.from_numpy(z["out_" + n]) for n in OUTPUT_NAMES}
    return meta, inp, out, torch.from_numpy(z["mask"])


def load_config1_head():
    z = np.load(os.path.join(GOLDEN_DIR, "config1_head.npz"))
    inp = {n: torch.from_numpy(z["in_" + n]) for n in INPUT_NAMES}
    out = {n: torch.from_numpy(z["out_" + n]) for n in OUTPUT_NAMES}
    norms = {n: float(z["norm_" + n]) for n in OUTPUT_NAMES}
    sums = {n: float(z["sum_" + n]) for n in OUTPUT_NAMES}
    return tuple(int(x) for x in z["head"]), inp, out, norms, sums


def record_errors(name, table):
    """Appends a per-output error table (ours / reference path / magnitude) as one JSON line to
    the file named by $ATTN_PARITY_REPORT, when that is set; the tests pass or fail without it."""
    path = os.environ.get("ATTN_PARITY_REPORT")
    if path:
        with open(path, "a") as f:
            f.write(json.dumps({"case": name, "errors": table}) + "\n")
