#!/usr/bin/env python
"""Benchmark of the double-backward (Hessian-vector product) attention path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (BASELINE.json configs[2], the configuration the metric is quoted on):
bf16 causal attention double backward, B=4, H=16, N=4096, D=128, all inputs
N(0,1) from the seeded generator shared with the tests.  One "step" is one
``v7_double_backward`` call over the whole batch (three kernel launches).

Multi-GPU (``torchrun``, one rank per GPU): the 64 (batch, head) slices are
partitioned over the ranks with no collective on the kernel path (strong
scaling: total work fixed); NCCL is used only for the start barrier and the
max-over-ranks of the measured times.

Printed JSON line: metric = algorithmic TFLOP/s of the HVP
(2 * D * 12 * visible_pairs * B * H flop per step, recompute not counted).
``value`` is measured with the inputs resident in HBM; ``e2e`` through the
``attention_cuda.v7_double_backward`` plugin call with pinned host buffers copied
in and the four results copied back inside the timed region.

``--impl reference`` times the reference's CPU path (its PyTorch math attention
differentiated twice) on the host cores: the reference's own ``reference_attention``
when oracle/build_ref.py has byte-compiled it into oracle/_ref/, else the restatement
in oracle/attention_oracle.py (the reference checkout itself is not on the GPU box).
"""
from __future__ import annotations

import argparse
import importlib
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WORKLOAD = dict(name="hvp_bf16_causal_B4_H16_N4096_D128", B=4, H=16, N=4096, D=128,
                window_size=4096, chunk_id=0, mask_mode=0)
HVP_GEMMS = 12          # algorithmic contractions of the double backward
ROW_KERNEL_GEMMS = 7    # contractions the g_Q kernel executes (5 score + 2 output)
PRE_KERNEL_GEMMS = 7    # scalars + g_dO kernel (5 score + 2 output)
COL_KERNEL_GEMMS = 8
# dram__bytes_read.sum + dram__bytes_write.sum per launch of each kernel, from an `ncu --set full`
# capture of this bench at 16 (batch, head) slices; traffic grows in proportion to the number of
# slices, so the bench scales it by BH / 16.  To be refreshed whenever a kernel changes.
NCU_TRAFFIC_BYTES_16_SLICES = {"pre": 193.3e6, "row": 173.6e6, "col": 137.3e6}
# the same for one launch of the fused norm + rotary kernel (part of the output is still in L2 when it ends)
NCU_PREP_TRAFFIC_BYTES = {"16384x32x128": 232.2e6}


def visible_pairs_causal(n: int) -> int:
    return n * (n + 1) // 2


def read_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return dict(bf16_tflops=float(p["bf16_tflops"]), bf16_tflops_sustained=float(p.get("bf16_tflops_sustained", 0)),
                    hbm_gbs=float(p["hbm_gbs"]), source="measured")
    return dict(bf16_tflops=1590.0, bf16_tflops_sustained=1400.0, hbm_gbs=6650.0, source="fallback")


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.lines = []
        self.proc = None
        self.thread = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.gpu), "--query-gpu=" + self.Q, "--format=csv,noheader,nounits", "-lms", "50"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        def pump():
            for line in self.proc.stdout:
                self.lines.append(line.strip())
        self.thread = threading.Thread(target=pump, daemon=True)
        self.thread.start()

    def stop(self):
        if self.proc is None:
            return dict(sm_mhz=None, sm_max_mhz=None, reasons=["nvidia-smi unavailable"])
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, smax, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); smax.append(float(f[2]))
            except ValueError:
                continue
            for name, v in zip(names, f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return dict(sm_mhz=statistics.median(sm) if sm else None, sm_max_mhz=max(smax) if smax else None,
                    samples=len(sm), reasons=sorted(reasons))


def usable_cores() -> int:
    """Cores this process may run on (its affinity mask), not the machine's total."""
    try:
        return len(os.sched_getaffinity(0))
    except AttributeError:
        return os.cpu_count() or 1


def cpu_path(orc):
    """The CPU implementation that is timed: the reference's own `reference_attention` and
    `make_sw_causal_mask` (e2e/ttt_pytorch/model.py, byte-compiled into oracle/_ref/ by
    oracle/build_ref.py) when that file is present -- kind "reference" -- and otherwise the
    restatement of the same five lines in oracle/attention_oracle.py -- kind "port"."""
    try:
        import build_ref
        ref = build_ref.load_python_reference()
    except Exception:  # noqa: BLE001
        ref = None
    if ref is not None:
        return ref.reference_attention, (lambda N: ref.make_sw_causal_mask(0, N, N, N, "cpu")), "reference"
    return orc.math_attention, (lambda N: orc.visibility_mask(0, N, N, N)), "port"


def cpu_hvp_seconds(orc, torch, n_heads: int, N: int, D: int, seed: int = 0):
    """Time the reference CPU path (math attention, double autograd) on `n_heads`
    (batch, head) slices of the workload; returns (seconds for the HVP step, threads, kind)."""
    attention, make_mask, kind = cpu_path(orc)
    inp = orc.make_inputs(1, n_heads, N, N, D, seed=seed, dtype=torch.float32)
    mask = make_mask(N)
    total = 0.0
    for h in range(n_heads):
        q, k, v, do = (inp[n][:, h:h + 1].clone().requires_grad_(True) for n in ("Q", "K", "V", "dO"))
        O = attention(q, k, v, mask)
        dQ, dK, dV = torch.autograd.grad(O, [q, k, v], grad_outputs=do, create_graph=True)
        hsum = (dQ * inp["g_dQ"][:, h:h + 1]).sum() + (dK * inp["g_dK"][:, h:h + 1]).sum() + (dV * inp["g_dV"][:, h:h + 1]).sum()
        t0 = time.perf_counter()
        torch.autograd.grad(hsum, [do, q, k, v])
        total += time.perf_counter() - t0
    return total, torch.get_num_threads(), kind


def reference_kernels_block(torch, tcapi, orc):
    """Secondary, like-for-like comparison: the reference's own CUDA kernels (compiled unchanged for
    sm_100a into oracle/_ref/ by oracle/build_ref.py; they exist for D in {64, 80, 96} only, so not
    for the headline D = 128) and this repository's kernels on the same GPU and inputs: bf16 causal
    N = 4096, D = 64, 64 (batch, head) slices.  None when the reference build is absent."""
    try:
        import build_ref
        ref = build_ref.load_module()
    except Exception:  # noqa: BLE001
        ref = None
    if ref is None:
        return None
    B, H, N, D = 4, 16, 4096, 64
    g = torch.Generator(device="cuda").manual_seed(0)
    mk = lambda: torch.randn(B, H, N, D, device="cuda", generator=g).to(torch.bfloat16)
    Q, K, V, dO, gQ, gK, gV = (mk() for _ in range(7))

    def timeit(f, n=5):
        for _ in range(2):
            f()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(n):
            f()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) / n

    out = {"workload": "bf16 causal B4 H16 N4096 D64", "note": "the reference builds D in {64, 80, 96}; no D = 128 kernel exists to compare the headline with"}
    O, L = tcapi.forward(Q, K, V, N, 0)
    Or, Lr = ref.v7_forward(Q, K, V, N, 0)
    for tag, fwd, bwd, hvp, o, l in (("ours", tcapi.forward, tcapi.backward, tcapi.double_backward, O, L),
                                     ("reference", ref.v7_forward, ref.v7_backward, ref.v7_double_backward, Or, Lr)):
        out[tag] = {"fwd_ms": timeit(lambda: fwd(Q, K, V, N, 0)), "bwd_ms": timeit(lambda: bwd(dO, Q, K, V, o, l, N, 0)),
                    "hvp_ms": timeit(lambda: hvp(gQ, gK, gV, dO, Q, K, V, o, l, N, 0))}
    out["speedup"] = {k: out["reference"][k] / out["ours"][k] for k in ("fwd_ms", "bwd_ms", "hvp_ms")}
    return out


def prep_block(torch, peaks):
    """The fused RMS-norm + rotary + layout kernel in front of the attention calls
    (`attention_cuda.qk_norm_rope`), bf16, at the K/V stream of the reference's largest model shape
    (16384 tokens x 32 heads x 128) and of its 125M shape (9216 x 12 x 64): device time against the
    HBM roofline (algorithmic bytes = one read and one write of the tensor; the table of angles is
    shared by the heads and stays in L2), and the same computation as eager PyTorch operations."""
    sys.path.insert(0, os.path.join(ROOT, "610sample_b200"))
    import attention_cuda
    qk_prep = importlib.import_module("610sample_b200.qk_prep")
    dev = torch.device("cuda", torch.cuda.current_device())
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    out = {}
    for name, (n_tok, H, d) in (("16384x32x128", (16384, 32, 128)), ("9216x12x64", (9216, 12, 64))):
        gen = torch.Generator(device="cpu").manual_seed(0)
        x = torch.randn(n_tok, H, d, generator=gen).to(torch.bfloat16).to(dev)
        w = (1.0 + 0.1 * torch.randn(d, generator=gen)).to(torch.bfloat16).to(dev)
        freqs = qk_prep.rope_table(d, n_tok, device=dev)

        def med(fn, reps=20):
            for _ in range(3):
                fn()
            evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(reps)]
            for a, b in evs:
                flush.zero_()
                a.record()
                fn()
                b.record()
            torch.cuda.synchronize()
            return statistics.median(a.elapsed_time(b) for a, b in evs)
        ms = med(lambda: attention_cuda.qk_norm_rope(x, w, freqs, 0, 1e-6, 0))
        eager_ms = med(lambda: qk_prep.qk_norm_rope_torch(x, w, freqs), reps=5)
        nbytes = 2 * x.numel() * x.element_size()
        gbs = nbytes / (ms * 1e-3) / 1e9
        out[name] = {"us": ms * 1e3, "eager_torch_us": eager_ms * 1e3, "algorithmic_bytes": nbytes,
                     "roofline": {"bound": "hbm", "achieved": gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                                  "frac": gbs / peaks["hbm_gbs"], "traffic": NCU_PREP_TRAFFIC_BYTES.get(name)}}
        del x, w, freqs
    return out


def run_reference(args):
    """CPU arm: the reference's own CPU implementation of the path on the host cores."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import torch
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import attention_oracle as orc
    w = WORKLOAD
    torch.set_num_threads(usable_cores())
    heads_per_step = 4
    flops_head = 2.0 * w["D"] * HVP_GEMMS * visible_pairs_causal(w["N"])
    for _ in range(args.warmup if args.warmup < 2 else 1):
        cpu_hvp_seconds(orc, torch, 1, w["N"], w["D"])
    times = []
    for s in range(args.steps):
        sec, threads, kind = cpu_hvp_seconds(orc, torch, heads_per_step, w["N"], w["D"], seed=s)
        times.append(sec)
    sec = sum(times) / len(times)
    value = flops_head * heads_per_step / sec / 1e12
    sample = f"{heads_per_step} of {w['B'] * w['H']} (batch, head) slices per step, fp32, second autograd.grad only"
    line = {
        "impl": "reference", "metric": "hvp_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": sec * 1e3, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": w["name"], "sample": sample},
        "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": threads, "kind": kind, "sample": sample},
        "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def bind_to_gpu_cpus(gpu_index: int):
    """Restricts this process to the CPU cores next to its GPU (the driver's own affinity mask for
    the device), so that the page-locked host buffers of the end-to-end leg are allocated on the
    GPU's NUMA node: with eight ranks on one box the host-side copies otherwise all cross the
    same memory controller.  Best effort; returns the number of cores kept or None."""
    try:
        import pynvml
        pynvml.nvmlInit()
        h = pynvml.nvmlDeviceGetHandleByIndex(gpu_index)
        n_cpu = os.cpu_count() or 1
        words = pynvml.nvmlDeviceGetCpuAffinity(h, (n_cpu + 63) // 64)
        cpus = {64 * i + b for i, w in enumerate(words) for b in range(64) if (w >> b) & 1}
        cpus &= os.sched_getaffinity(0)
        if cpus:
            os.sched_setaffinity(0, cpus)
            return len(cpus)
    except Exception:  # noqa: BLE001
        pass
    return None


def run_ours(args):
    import torch
    import torch.distributed as dist
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import attention_oracle as orc

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback)")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    numa = bind_to_gpu_cpus(local)      # before any page-locked allocation
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)

    pkg_dir = os.path.join(ROOT, "610sample_b200")
    sys.path.insert(0, pkg_dir)
    import attention_cuda                                   # the plugin module (fails loudly if not built)
    tcapi = importlib.import_module("610sample_b200.torch_capi")
    capi = importlib.import_module("610sample_b200.capi")

    sharding = importlib.import_module("610sample_b200.sharding")

    w = WORKLOAD
    BH = args.bh if args.bh > 0 else w["B"] * w["H"]
    N, D = w["N"], w["D"]
    # every rank draws the full seeded workload and keeps its contiguous range of (batch, head) slices
    full = orc.make_inputs(1, BH, N, N, D, seed=0, dtype=torch.bfloat16)
    begin, end = sharding.shard_range(BH, world, rank)
    bh_local = end - begin
    sl = slice(begin, end)
    host = {n: full[n][:, sl].contiguous().pin_memory() for n in orc.INPUT_NAMES}
    del full
    g = {n: t.to(dev, non_blocking=True) for n, t in host.items()}
    ws, cid, mm = w["window_size"], w["chunk_id"], w["mask_mode"]

    O, L = tcapi.forward(g["Q"], g["K"], g["V"], ws, cid, mm)
    host_O = torch.empty_like(O, device="cpu").pin_memory(); host_O.copy_(O)
    host_L = torch.empty_like(L, device="cpu").pin_memory(); host_L.copy_(L)
    s = tcapi._shape(g["Q"], g["K"], ws, cid, mm, 0)
    scratch = torch.empty(capi.lib().attn_b200_double_backward_scratch_bytes(s) // 4 + 4, dtype=torch.float32, device=dev)
    outs = tuple(torch.empty_like(g[n]) for n in ("Q", "Q", "K", "V"))
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)       # > 126 MB L2

    def step():
        tcapi.double_backward(g["g_dQ"], g["g_dK"], g["g_dV"], g["dO"], g["Q"], g["K"], g["V"], O, L, ws, cid, mm,
                              scratch=scratch, out=outs)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # the clock sampler runs from before the warm-up, so that short timed regions still get samples
    sampler = ClockSampler(local)
    sampler.start()
    for _ in range(max(args.warmup, 3)):
        step()
    launches_per_step = capi.lib().attn_b200_last_launch_count()
    torch.cuda.synchronize()

    # ---- kernel-resident timing ------------------------------------------------
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
    barrier()
    for a, b in ev:
        flush.zero_()
        a.record()
        step()
        b.record()
    barrier()
    clocks = sampler.stop()
    ms = sum(a.elapsed_time(b) for a, b in ev)
    ms_per_step = sharding.max_over_ranks(ms, dev) / args.steps

    # ---- per-kernel timing (single-GPU roofline): the three kernels of a pass, launched one after
    # the other as in a step (serially, each between its own pair of events), L2 flushed before
    # each pass, no host synchronisation inside the loop -- the regime of the timed region above
    phase_ms = {}
    if hasattr(capi.lib(), "attn_b200_double_backward_phases"):
        reps = max(3, min(args.steps, 20))
        names = (("pre", 1), ("row", 2), ("col", 4))
        pev = {n: [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(reps)] for n, _ in names}
        for r in range(reps):
            flush.zero_()
            for name, mask_bits in names:
                a, b = pev[name][r]
                a.record()
                tcapi.double_backward_phases(g["g_dQ"], g["g_dK"], g["g_dV"], g["dO"], g["Q"], g["K"], g["V"], O, L,
                                             ws, cid, mm, scratch=scratch, out=outs, phases=mask_bits)
                b.record()
        torch.cuda.synchronize()
        for name, _ in names:
            phase_ms[name] = sum(a.elapsed_time(b) for a, b in pev[name]) / reps

    # ---- forward and first backward at the same shape (rank-local slices) ----------
    def time_call(fn, reps):
        evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(reps)]
        for a, b in evs:
            flush.zero_()
            a.record()
            fn()
            b.record()
        torch.cuda.synchronize()
        return sum(a.elapsed_time(b) for a, b in evs) / reps

    bwd_scratch = torch.empty(capi.lib().attn_b200_backward_scratch_bytes(s) // 4 + 4, dtype=torch.float32, device=dev)
    fb_reps = max(3, min(args.steps, 20))
    fwd_fn = lambda: tcapi.forward(g["Q"], g["K"], g["V"], ws, cid, mm)
    bwd_fn = lambda: tcapi.backward(g["dO"], g["Q"], g["K"], g["V"], O, L, ws, cid, mm, scratch=bwd_scratch)
    for _ in range(2):
        fwd_fn(); bwd_fn()
    fwd_ms = sharding.max_over_ranks(time_call(fwd_fn, fb_reps), dev)
    bwd_ms = sharding.max_over_ranks(time_call(bwd_fn, fb_reps), dev)

    # ---- the same step looped for >= 2 s: the board's power cap pulls the SM clock down ----
    sustained = None
    if not args.no_sustained:
        n_sus = max(20, int(2000.0 / max(ms_per_step, 1e-3)) + 1)
        sus_sampler = ClockSampler(local)
        barrier()
        sus_sampler.start()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(n_sus):
            step()                       # no L2 flush: the inputs of a step (806 MB) exceed the 126 MB L2
        b.record()
        barrier()
        sus_clocks = sus_sampler.stop()
        sus_ms = sharding.max_over_ranks(a.elapsed_time(b), dev) / n_sus
        sustained = {"steps": n_sus, "ms_per_step": sus_ms, "clocks": sus_clocks,
                     "l2": "no flush between steps; the step's inputs exceed L2"}

    # ---- end to end through the plugin call, host buffers ------------------------
    e2e_steps = max(1, min(args.steps, 5))
    in_names = ("g_dQ", "g_dK", "g_dV", "dO", "Q", "K", "V")
    host_out = [torch.empty_like(t, device="cpu").pin_memory() for t in outs]
    h2d = sum(host[n].numel() * host[n].element_size() for n in in_names) + host_O.numel() * 2 + host_L.numel() * 4
    d2h = sum(t.numel() * t.element_size() for t in host_out)

    # The (batch, head) slices are independent, so the host-buffer path is pipelined over
    # chunks of slices on three streams: upload of chunk c+1, kernels of chunk c and download
    # of chunk c-1 overlap (PCIe is full duplex).  Every byte still crosses inside the timed region.
    # chunks of at least four slices (128 CTAs per kernel), sizes differing by at most one
    n_chunks = max(1, min(args.e2e_chunks, bh_local // 4 if bh_local >= 4 else 1))
    chunk_bounds = [sharding.shard_range(bh_local, n_chunks, c) for c in range(n_chunks)]
    s_in, s_cmp, s_out = torch.cuda.Stream(), torch.cuda.Stream(), torch.cuda.Stream()

    def e2e_step():
        main = torch.cuda.current_stream()
        s_in.wait_stream(main); s_cmp.wait_stream(main); s_out.wait_stream(main)
        for c0, c1 in chunk_bounds:
            sl_c = slice(c0, c1)
            with torch.cuda.stream(s_in):
                d = {n: host[n][:, sl_c].to(dev, non_blocking=True) for n in in_names}
                dO_ = host_O[:, sl_c].to(dev, non_blocking=True)
                dL_ = host_L[:, sl_c].to(dev, non_blocking=True)
                up = torch.cuda.Event(); up.record(s_in)
            with torch.cuda.stream(s_cmp):
                s_cmp.wait_event(up)
                for tns in list(d.values()) + [dO_, dL_]:
                    tns.record_stream(s_cmp)
                r = attention_cuda.v7_double_backward(d["g_dQ"], d["g_dK"], d["g_dV"], d["dO"], d["Q"], d["K"], d["V"],
                                                      dO_, dL_, ws, cid)
                done = torch.cuda.Event(); done.record(s_cmp)
            with torch.cuda.stream(s_out):
                s_out.wait_event(done)
                for dst, src in zip(host_out, r):
                    src.record_stream(s_out)
                    dst[:, sl_c].copy_(src, non_blocking=True)
        main.wait_stream(s_out); main.wait_stream(s_cmp); main.wait_stream(s_in)

    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if args.no_e2e:
        a.record(); b.record()
    else:
        e2e_step()
        barrier()
        a.record()
        for _ in range(e2e_steps):
            e2e_step()
        b.record()
    barrier()
    e2e_ms = sharding.max_over_ranks(max(a.elapsed_time(b), 1e-9), dev) / e2e_steps
    status = capi.device_status()

    # ---- the caller: TTT meta-step (bench_ttt.py) on the same GPUs, NCCL all-reduce of the outer gradient
    ttt = None
    if not args.no_ttt:
        torch.cuda.empty_cache()
        import bench_ttt
        ttt_line = bench_ttt.measure(argparse.Namespace(gpus=world, steps=3, warmup=1, impl="ours", small=False),
                                     init_process_group=False)
        if ttt_line is not None:
            ttt = {k: ttt_line[k] for k in ("value", "unit", "ms_per_step", "steps", "warmup", "scaling",
                                            "attention_ms_per_step", "attention_share", "peak_memory_mb")}
            ttt["workload"] = ttt_line["config"]["workload"]

    flops_step = 2.0 * D * HVP_GEMMS * visible_pairs_causal(N) * BH          # whole job, all ranks
    value = flops_step / (ms_per_step * 1e-3) / 1e12
    e2e_value = flops_step / (e2e_ms * 1e-3) / 1e12
    peaks = read_peaks()

    if rank == 0:
        line = {
            "metric": "hvp_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": w["name"] if args.bh <= 0 else f"{w['name']} reduced to {BH} (batch, head) slices", "parallelism": f"batch*head sharded over {world} GPU(s), no collective",
                       "l2": "256 MB buffer written between timed steps", "heads_on_rank0": bh_local,
                       "flop_model": "2*D*12*visible_pairs*B*H"},
            "pct_of_bf16_peak": 100.0 * value / (peaks["bf16_tflops"] * world),
            "pct_of_bf16_peak_sustained": (100.0 * value / (peaks["bf16_tflops_sustained"] * world)
                                           if peaks["bf16_tflops_sustained"] else None),
            "peaks": peaks, "clocks": clocks,
            "e2e": {"value": e2e_value, "unit": "TFLOP/s", "ms_per_step": e2e_ms, "steps": e2e_steps,
                    "h2d_bytes_per_step": int(h2d) // bh_local * BH, "d2h_bytes_per_step": int(d2h) // bh_local * BH,
                    "pipeline": f"{n_chunks} chunks of (batch, head) slices on upload / compute / download streams",
                    "cpu_cores_bound_to_gpu": numa},
            "gpu_launches": int(launches_per_step) * args.steps,
            "device_status": status,
        }
        pairs_all = visible_pairs_causal(N) * BH
        for key, gemms, t_ms in (("fwd", 2, fwd_ms), ("bwd", 5, bwd_ms)):
            tf = 2.0 * D * gemms * pairs_all / (t_ms * 1e-3) / 1e12
            line[key] = {"ms": t_ms, "tflops": tf, "gemms": gemms, "pct_of_bf16_peak": 100.0 * tf / (peaks["bf16_tflops"] * world)}
        if sustained is not None:
            sv = flops_step / (sustained["ms_per_step"] * 1e-3) / 1e12
            mhz = sustained["clocks"].get("sm_mhz")
            sustained.update(value=sv, pct_of_bf16_peak=100.0 * sv / (peaks["bf16_tflops"] * world),
                             pct_of_bf16_peak_sustained=(100.0 * sv / (peaks["bf16_tflops_sustained"] * world)
                                                         if peaks["bf16_tflops_sustained"] else None),
                             ms_times_mhz=(sustained["ms_per_step"] * mhz if mhz else None))
            line["sustained"] = sustained
        if ttt is not None:
            line["ttt"] = ttt
        if phase_ms and world == 1:
            # One pass of the path = three launches (scalars + g_dO, g_Q, g_K + g_V).  `achieved` counts
            # the 12 ALGORITHMIC contractions of the pass over the summed device time of the three
            # kernels, each timed alone; `executed` adds what the tensor pipe really ran per kernel
            # (score products are recomputed by each kernel), to be compared with ncu's
            # sm__pipe_tensor_cycles_active.
            pairs = visible_pairs_causal(N) * BH
            k_gemms = {"pre": PRE_KERNEL_GEMMS, "row": ROW_KERNEL_GEMMS, "col": COL_KERNEL_GEMMS}
            total_ms = sum(phase_ms.values())
            ach_serial = 2.0 * D * HVP_GEMMS * pairs / (total_ms * 1e-3) / 1e12
            dom = max(phase_ms, key=phase_ms.get)
            executed = {k: {"gemms": k_gemms[k], "tflops": 2.0 * D * k_gemms[k] * pairs / (phase_ms[k] * 1e-3) / 1e12}
                        for k in phase_ms}
            for k in executed:
                executed[k]["frac"] = executed[k]["tflops"] / peaks["bf16_tflops"]
            # `achieved`: the 12 algorithmic contractions of a pass over the duration of the pass in the
            # timed region above (its own CUDA events; g_Q and g_K/g_V kernels side by side as the
            # library launches them).  `achieved_kernels_serial`: the same over the SUM of the three
            # kernels' own durations (each between its own events, launched one after the other).
            line["roofline"] = {"bound": "tensor", "kernel": "hvp pass = hvp_row<PREDO> + hvp_row<Q> + hvp_col",
                                "achieved": value, "peak": peaks["bf16_tflops"],
                                "unit": "TFLOP/s", "frac": value / peaks["bf16_tflops"],
                                "achieved_kernels_serial": ach_serial, "frac_kernels_serial": ach_serial / peaks["bf16_tflops"],
                                "traffic": sum(NCU_TRAFFIC_BYTES_16_SLICES.values()) * BH / 16.0,
                                "traffic_note": "dram bytes of the three launches, scaled from an ncu capture at 16 slices; "
                                                "algorithmic bytes of the pass: %.0f" % ((12 * N * D * 2 + 4 * N) * BH),
                                "peak_source": peaks["source"], "kernel_ms": phase_ms,
                                "dominant_kernel": "hvp_" + dom, "executed": executed}
        if world == 1 and not args.no_prep:
            line["prep"] = prep_block(torch, peaks)
        if world == 1 and not args.no_ref_kernels:
            rk = reference_kernels_block(torch, tcapi, orc)
            if rk is not None:
                line["vs_reference_kernels"] = rk
        if world == 1 and not args.no_cpu_baseline:
            torch.set_num_threads(usable_cores())
            n_cpu = 16
            sec, threads, kind = cpu_hvp_seconds(orc, torch, n_cpu, N, D)
            cpu_val = 2.0 * D * HVP_GEMMS * visible_pairs_causal(N) * n_cpu / sec / 1e12
            line["cpu_baseline"] = {"value": cpu_val, "unit": "TFLOP/s", "cores": threads, "kind": kind,
                                    "sample": f"{n_cpu} of {BH} (batch, head) slices, fp32 math attention, "
                                              f"second autograd.grad only ({sec:.2f} s timed)"}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20,
                    help="timed steps; the SM clock falls under the power limit as a run gets longer, so `value` depends on it "
                         "(the `sustained` key is the long-run figure)")
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--e2e-chunks", type=int, default=8, help="chunks of slices the host-buffer leg is pipelined over")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer leg (profiling runs)")
    ap.add_argument("--no-sustained", action="store_true", help="skip the >= 2 s loop under the power cap")
    ap.add_argument("--no-ttt", action="store_true", help="skip the TTT meta-step of bench_ttt.py")
    ap.add_argument("--no-prep", action="store_true", help="skip the timing of the fused norm + rotary kernel")
    ap.add_argument("--no-ref-kernels", action="store_true", help="skip the comparison with the reference's own CUDA kernels")
    ap.add_argument("--bh", type=int, default=0,
                    help="profiling only: number of (batch, head) slices instead of the workload's 64")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
