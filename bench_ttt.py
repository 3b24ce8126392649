#!/usr/bin/env python
"""End-to-end test-time-training (TTT) step benchmark: the caller of the attention path.

    python bench_ttt.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--small]

Workload (BASELINE.json configs[4]): a random-init 12-layer pre-norm decoder, d_model 768,
12 heads (D = 64), GELU MLP 3072, vocabulary 32000, sequence 2048, batch 8 per GPU, bf16,
token ids uniform over the vocabulary.  One step = one inner SGD step (lr 1e-2) on the fast
weights (every block's parameters) followed by the outer loss on the updated weights, which
is differentiated THROUGH the inner step (`create_graph=True`), so every layer runs attention
forward, backward and double backward.  Under torchrun the outer gradient is all-reduced with
NCCL; nothing else is communicated.

The pattern (functional forward with a parameter dict, `autograd.grad(..., create_graph=True)`,
`w <- w - lr*g`, outer `backward`) follows the reference's `meta_step`
(`e2e/ttt_pytorch/model.py:540-671`); the model itself is the plain decoder BASELINE names,
not the reference's SwiGLU/RoPE model.  Attention goes through `flash_attention_v7`
(`--impl ours`) or through the reference's math attention (`--impl reference`, on the CPU,
on a reduced sample that is stated in the output).

Prints one JSON line: metric `ttt_tokens_per_s`.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "oracle"))

FULL = dict(layers=12, d_model=768, heads=12, d_ff=3072, vocab=32000, seq=2048, batch=8)
SMALL = dict(layers=2, d_model=128, heads=2, d_ff=256, vocab=512, seq=256, batch=2)
INNER_LR = 1e-2


def init_params(cfg, device, dtype, seed=0):
    import torch
    g = torch.Generator(device="cpu").manual_seed(seed)
    d, f, v = cfg["d_model"], cfg["d_ff"], cfg["vocab"]

    def w(*shape):
        return (torch.randn(*shape, generator=g) * 0.02).to(dtype).to(device).requires_grad_(True)

    def ones(n):
        return torch.ones(n, dtype=dtype, device=device, requires_grad=True)

    def zeros(n):
        return torch.zeros(n, dtype=dtype, device=device, requires_grad=True)

    slow = {"embed": w(v, d), "ln_f.w": ones(d), "ln_f.b": zeros(d), "head": w(v, d)}
    fast = {}
    for i in range(cfg["layers"]):
        p = f"blk{i}."
        fast[p + "ln1.w"] = ones(d); fast[p + "ln1.b"] = zeros(d)
        fast[p + "qkv"] = w(3 * d, d); fast[p + "proj"] = w(d, d)
        fast[p + "ln2.w"] = ones(d); fast[p + "ln2.b"] = zeros(d)
        fast[p + "fc1"] = w(f, d); fast[p + "fc2"] = w(d, f)
    return slow, fast


def forward_loss(cfg, slow, fast, ids, targets, attention):
    """Mean cross entropy of the decoder with the given fast weights."""
    import torch
    import torch.nn.functional as F
    B, N = ids.shape
    d, H = cfg["d_model"], cfg["heads"]
    hd = d // H
    x = slow["embed"][ids]                                              # [B, N, d]
    for i in range(cfg["layers"]):
        p = f"blk{i}."
        h = F.layer_norm(x, (d,), fast[p + "ln1.w"], fast[p + "ln1.b"])
        # one GEMM for the three projections, then three 25 MB copies into the attention layout
        # (about 10 us each at this size, under 1 % of the step; per-head GEMMs that write
        # [B, H, N, hd] directly have N = 64 outputs and cost more than the copies they save)
        qkv = F.linear(h, fast[p + "qkv"]).view(B, N, 3, H, hd).permute(2, 0, 3, 1, 4)   # [3, B, H, N, hd]
        o = attention(qkv[0].contiguous(), qkv[1].contiguous(), qkv[2].contiguous())     # [B, H, N, hd]
        x = x + F.linear(o.transpose(1, 2).reshape(B, N, d), fast[p + "proj"])
        h = F.layer_norm(x, (d,), fast[p + "ln2.w"], fast[p + "ln2.b"])
        x = x + F.linear(F.gelu(F.linear(h, fast[p + "fc1"])), fast[p + "fc2"])
    x = F.layer_norm(x, (d,), slow["ln_f.w"], slow["ln_f.b"])
    logits = F.linear(x, slow["head"])
    return F.cross_entropy(logits.float().view(B * N, -1), targets.reshape(B * N))


def ttt_step(cfg, slow, fast, ids, targets, attention):
    """One meta step; returns the outer loss (call .backward() on it)."""
    import torch
    names = list(fast.keys())
    inner = forward_loss(cfg, slow, fast, ids, targets, attention)
    grads = torch.autograd.grad(inner, [fast[n] for n in names], create_graph=True)
    updated = {n: fast[n] - INNER_LR * g for n, g in zip(names, grads)}
    return forward_loss(cfg, slow, updated, ids, targets, attention)


def make_batch(cfg, device, seed):
    import torch
    g = torch.Generator(device="cpu").manual_seed(seed)
    ids = torch.randint(0, cfg["vocab"], (cfg["batch"], cfg["seq"] + 1), generator=g)
    return ids[:, :-1].contiguous().to(device), ids[:, 1:].contiguous().to(device)


def math_attention_fn(N):
    import torch
    import attention_oracle as orc
    mask = None

    def f(q, k, v):
        nonlocal mask
        if mask is None or mask.device != q.device:
            mask = orc.visibility_mask(0, N, N, N, device=q.device)
        return orc.math_attention(q, k, v, mask)
    return f


class AttentionTimer:
    """CUDA events around every call of the attention plugin (forward, backward, double backward),
    so that a step's device time can be split into attention and everything else."""

    NAMES = ("v7_forward", "v7_backward", "v7_double_backward")

    def __init__(self, module):
        import torch
        self.torch, self.module = torch, module
        self.orig = {n: getattr(module, n) for n in self.NAMES}
        self.events = {n: [] for n in self.NAMES}
        self.enabled = False
        for n in self.NAMES:
            setattr(module, n, self._wrap(n))

    def _wrap(self, name):
        fn = self.orig[name]

        def timed(*a, **k):
            if not self.enabled:
                return fn(*a, **k)
            e0, e1 = self.torch.cuda.Event(enable_timing=True), self.torch.cuda.Event(enable_timing=True)
            e0.record()
            r = fn(*a, **k)
            e1.record()
            self.events[name].append((e0, e1))
            return r
        return timed

    def restore(self):
        for n in self.NAMES:
            setattr(self.module, n, self.orig[n])

    def totals_ms(self):
        return {n: sum(a.elapsed_time(b) for a, b in ev) for n, ev in self.events.items()}


def measure(args, init_process_group=True):
    """Runs the workload and returns the JSON line as a dict (None on ranks other than 0).  With
    `init_process_group` false the caller has already set the device and the NCCL group up."""
    import torch
    import torch.distributed as dist
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    cfg = dict(SMALL if args.small else FULL)
    reference = args.impl == "reference"
    sample = None
    if reference:
        # CPU arm: the reference's math attention; a reduced sample of the workload, stated below
        if rank != 0:
            return None
        dev = torch.device("cpu")
        torch.set_num_threads(os.cpu_count() or 1)
        if not args.small:
            cfg.update(layers=2, batch=1, seq=1024)
            sample = "2 of 12 layers, batch 1, sequence 1024, fp32, math attention on the host cores"
        dtype = torch.float32
        attention = math_attention_fn(cfg["seq"])
        world = 1
    else:
        if not torch.cuda.is_available():
            raise SystemExit("bench_ttt.py needs a CUDA device (there is no CPU fallback)")
        torch.cuda.set_device(local)
        dev = torch.device("cuda", local)
        if world > 1 and init_process_group:
            os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
            dist.init_process_group("nccl", device_id=dev)
        sys.path.insert(0, os.path.join(ROOT, "610sample_b200"))
        import attention_cuda
        from attention import flash_attention_v7
        timer = AttentionTimer(attention_cuda)
        dtype = torch.bfloat16
        N = cfg["seq"]
        attention = lambda q, k, v: flash_attention_v7(q, k, v, N, 0)

    slow, fast = init_params(cfg, dev, dtype)
    params = list(slow.values()) + list(fast.values())
    ids, targets = make_batch(cfg, dev, seed=rank)

    def step():
        for p in params:
            p.grad = None
        loss = ttt_step(cfg, slow, fast, ids, targets, attention)
        loss.backward()
        if world > 1:
            flat = torch.cat([p.grad.reshape(-1) for p in params])
            dist.all_reduce(flat)
            flat /= world
        return loss

    for _ in range(args.warmup):
        loss = step()
    if dev.type == "cuda":
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        timer.enabled = True
        a.record()
        for _ in range(args.steps):
            loss = step()
        b.record()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        timer.enabled = False
        attn_ms = {n: v / args.steps for n, v in timer.totals_ms().items()}
        timer.restore()
        tm = torch.tensor([a.elapsed_time(b)], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(tm, op=dist.ReduceOp.MAX)
        ms = float(tm.item()) / args.steps
        peak_mb = torch.cuda.max_memory_allocated() / 2**20
    else:
        t0 = time.perf_counter()
        for _ in range(args.steps):
            loss = step()
        ms = (time.perf_counter() - t0) * 1e3 / args.steps
        peak_mb = None
        attn_ms = None
    tokens = cfg["batch"] * cfg["seq"] * world
    line = None
    if rank == 0:
        line = {
            "metric": "ttt_tokens_per_s", "value": tokens / (ms * 1e-3), "unit": "tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32" if reference else "bf16", "data": "synthetic",
            "impl": args.impl,
            "config": {"workload": "ttt_step_12L_d768_h12_seq2048_b8" if not args.small else "ttt_step_small",
                       **{k: cfg[k] for k in ("layers", "d_model", "heads", "d_ff", "vocab", "seq", "batch")},
                       "inner_lr": INNER_LR, "sample": sample},
            "outer_loss": float(loss.detach()), "peak_memory_mb": peak_mb,
        }
        if attn_ms is not None:
            # device time of the attention plugin calls of rank 0, per step (12 layers x two passes)
            line["attention_ms_per_step"] = attn_ms
            line["attention_share"] = sum(attn_ms.values()) / ms
        if reference:
            line["cpu_baseline"] = {"value": line["value"], "unit": "tokens/s", "cores": torch.get_num_threads(),
                                    "kind": "port", "sample": sample or "small configuration, whole"}
    if world > 1 and not reference and init_process_group:
        dist.destroy_process_group()
    return line


def run(args):
    line = measure(args)
    if line is not None:
        print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=2)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--small", action="store_true", help="2-layer toy configuration (tests)")
    run(ap.parse_args())


if __name__ == "__main__":
    main()
