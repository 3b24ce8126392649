#!/usr/bin/env python
"""Attention-only meta-step on the reference's chunked sliding-window workload, and the
largest batch that fits a memory budget.

    python bench_attn_meta.py [--shapes 125M,760M,3B] [--budget-mb 75000] [--trials 5] [--no-math]

Workload (the reference's `benchmark_attention_only` / `benchmark_max_throughput`,
e2e/tests/test_ttt_e2e_pytorch.py:743-1103; shapes `ATTN_CONFIGS`, :743-751): per (batch, head)
a token stream of `chunks * N_q` vectors of width D (N(0,1) * 0.1) and three D x D projections
(N(0,1) * 0.02, the "fast weights").  For every chunk c: Q from the chunk's N_q tokens, K and V
from the last N_kv tokens up to the chunk's end (left-padded with zeros while the history is
shorter), O = sliding-window attention(window, chunk c), chunk loss = sum(O), its gradient with
respect to the three projections taken with `create_graph=True`; the meta-loss is the sum of all
those gradients' sums, and one backward through it ends the step.  Every chunk therefore runs
attention forward, backward and double backward at N_q = 1024, N_kv = 9216, window 8192.

Two arms on the same inputs: `kernels` (this repository's `flash_attention_v7`) and `math`
(PyTorch matmul attention differentiated twice by autograd, the reference's comparison arm; it
materialises the N_q x N_kv matrices).  Reported per shape: median step time (CUDA events) and
peak memory at batch 1, then the largest batch <= 64 whose peak memory stays within the budget
(binary search, as the reference does) with its step time and tokens/s.  One JSON line per
measurement.  (The reference's own record of these workloads was taken on an A100, 75 000 MB
budget; nothing here reads it.)
"""
from __future__ import annotations

import argparse
import json
import os
import sys

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "oracle"))

# name: (H, N_q, N_kv, D, window_size, chunks)
SHAPES = {
    "small": (4, 64, 256, 64, 192, 4),
    "med": (8, 128, 1024, 64, 896, 4),
    "125M": (12, 1024, 9216, 64, 8192, 8),
    "D80": (8, 1024, 9216, 80, 8192, 8),
    "760M": (16, 1024, 9216, 96, 8192, 8),
    "3B": (32, 1024, 9216, 80, 8192, 8),
}


def make_inputs(torch, B, shape, device, dtype, seed=0):
    H, N_q, N_kv, D, ws, chunks = shape
    g = torch.Generator(device=device).manual_seed(seed)
    w = lambda: (torch.randn(B, H, D, D, device=device, dtype=torch.float32, generator=g) * 0.02).to(dtype).requires_grad_(True)
    W_q, W_k, W_v = w(), w(), w()
    tokens = (torch.randn(B, H, chunks * N_q, D, device=device, dtype=torch.float32, generator=g) * 0.1).to(dtype)
    return W_q, W_k, W_v, tokens


def meta_step(torch, attention, W_q, W_k, W_v, tokens, shape):
    """Returns the meta-loss; the caller runs .backward() on it."""
    H, N_q, N_kv, D, ws, chunks = shape
    B = tokens.shape[0]
    meta = torch.zeros((), device=tokens.device, dtype=torch.float32)
    for c in range(chunks):
        end = (c + 1) * N_q
        x_q = tokens[:, :, end - N_q:end]
        x_kv = tokens[:, :, max(0, end - N_kv):end]
        if x_kv.shape[2] < N_kv:
            pad = torch.zeros(B, H, N_kv - x_kv.shape[2], D, device=tokens.device, dtype=tokens.dtype)
            x_kv = torch.cat([pad, x_kv], dim=2)
        Q, K, V = torch.matmul(x_q, W_q), torch.matmul(x_kv, W_k), torch.matmul(x_kv, W_v)
        O = attention(Q, K, V, ws, c)
        grads = torch.autograd.grad(O.sum(), [W_q, W_k, W_v], create_graph=True)
        meta = meta + sum(g.float().sum() for g in grads)
    return meta


def kernel_attention():
    sys.path.insert(0, os.path.join(ROOT, "610sample_b200"))
    from attention import flash_attention_v7
    return lambda Q, K, V, ws, c: flash_attention_v7(Q, K, V, ws, c)


def math_attention():
    import attention_oracle as orc
    masks = {}

    def f(Q, K, V, ws, c):
        key = (c, Q.shape[2], K.shape[2], ws, Q.device)
        if key not in masks:
            masks[key] = orc.visibility_mask(c, Q.shape[2], K.shape[2], ws, device=Q.device)
        return orc.math_attention(Q, K, V, masks[key])
    return f


def run_step(torch, attention, B, shape, device, dtype, seed=0):
    W_q, W_k, W_v, tokens = make_inputs(torch, B, shape, device, dtype, seed)
    loss = meta_step(torch, attention, W_q, W_k, W_v, tokens, shape)
    loss.backward()
    return loss, (W_q.grad, W_k.grad, W_v.grad)


def measure(torch, attention, B, shape, device, dtype, warmup, trials):
    """(median ms, peak MB) of the whole step at batch B."""
    for _ in range(warmup):
        run_step(torch, attention, B, shape, device, dtype)
    torch.cuda.synchronize()
    torch.cuda.empty_cache()
    torch.cuda.reset_peak_memory_stats()
    times = []
    for i in range(trials):
        W_q, W_k, W_v, tokens = make_inputs(torch, B, shape, device, dtype, seed=i)
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        meta_step(torch, attention, W_q, W_k, W_v, tokens, shape).backward()
        b.record()
        torch.cuda.synchronize()
        times.append(a.elapsed_time(b))
        del W_q, W_k, W_v, tokens
    return sorted(times)[len(times) // 2], torch.cuda.max_memory_allocated() / 2**20


def peak_mb(torch, attention, B, shape, device, dtype):
    torch.cuda.empty_cache()
    torch.cuda.reset_peak_memory_stats()
    try:
        run_step(torch, attention, B, shape, device, dtype)
        torch.cuda.synchronize()
    except torch.cuda.OutOfMemoryError:
        torch.cuda.empty_cache()
        return float("inf")
    return torch.cuda.max_memory_allocated() / 2**20


def max_batch(torch, attention, shape, device, dtype, budget_mb, cap=64):
    """Largest batch <= cap whose peak memory stays within budget_mb (0 when batch 1 does not fit)."""
    one = peak_mb(torch, attention, 1, shape, device, dtype)
    if one > budget_mb:
        return 0
    lo, hi, best = 2, min(cap, max(1, int(budget_mb / one))), 1
    while lo <= hi:
        mid = (lo + hi) // 2
        if peak_mb(torch, attention, mid, shape, device, dtype) <= budget_mb:
            best, lo = mid, mid + 1
        else:
            hi = mid - 1
    return best


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--shapes", default="125M,760M,3B")
    ap.add_argument("--budget-mb", type=float, default=75000.0, help="memory budget of the max-batch search (the reference's A100 run used 75 000 MB)")
    ap.add_argument("--trials", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=2)
    ap.add_argument("--no-math", action="store_true", help="skip the PyTorch math-attention arm")
    ap.add_argument("--no-max-batch", action="store_true")
    args = ap.parse_args()
    import torch
    if not torch.cuda.is_available():
        raise SystemExit("bench_attn_meta.py needs a CUDA device (there is no CPU fallback)")
    device, dtype = torch.device("cuda", 0), torch.bfloat16
    arms = [("kernels", kernel_attention())] + ([] if args.no_math else [("math", math_attention())])
    for name in args.shapes.split(","):
        shape = SHAPES[name]
        H, N_q, N_kv, D, ws, chunks = shape
        for arm, attention in arms:
            ms, mb = measure(torch, attention, 1, shape, device, dtype, args.warmup, args.trials)
            print(json.dumps({"bench": "attn_meta_step", "shape": name, "arm": arm, "batch": 1, "H": H, "N_q": N_q, "N_kv": N_kv, "D": D,
                              "window": ws, "chunks": chunks, "ms": ms, "peak_mb": mb}), flush=True)
            if args.no_max_batch:
                continue
            Bmax = max_batch(torch, attention, shape, device, dtype, args.budget_mb)
            if Bmax == 0:
                print(json.dumps({"bench": "attn_max_batch", "shape": name, "arm": arm, "batch": 0, "budget_mb": args.budget_mb}), flush=True)
                continue
            ms, mb = measure(torch, attention, Bmax, shape, device, dtype, 1, max(3, args.trials // 2))
            print(json.dumps({"bench": "attn_max_batch", "shape": name, "arm": arm, "batch": Bmax, "budget_mb": args.budget_mb, "ms": ms,
                              "peak_mb": mb, "tokens_per_s": Bmax * chunks * N_q / (ms * 1e-3)}), flush=True)


if __name__ == "__main__":
    main()
