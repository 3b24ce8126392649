"""Times this repository's kernels against the reference's own CUDA kernels on the same GPU.

The reference's extension must have been built by oracle/build_ref.py (oracle/_ref/).  Shapes:
the reference's benchmark configurations (tests/test_ttt_e2e_bench.py:156-161, chunk 8 = full
window) and the causal N = 4096 case at the head dimensions the reference builds.  bf16, CUDA
events, 2 warm-up + 5 timed calls each.  Checker tooling: nothing in the package uses it.

    python oracle/compare_with_ref_kernels.py
"""
import importlib, json, sys, os
import torch
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "oracle"))
import attention_oracle as orc, build_ref
ref = build_ref.load_module()
if ref is None:
    raise SystemExit("build the reference's extension first: python oracle/build_ref.py")
tcapi = importlib.import_module("610sample_b200.torch_capi")
def timeit(f, n=5):
    for _ in range(2): f()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(n): f()
    b.record(); torch.cuda.synchronize()
    return a.elapsed_time(b) / n
CASES = [("125M chunk 8", 1, 12, 1024, 9216, 64, 8192, 8), ("760M chunk 8", 1, 16, 1024, 9216, 96, 8192, 8), ("3B chunk 8", 1, 32, 1024, 9216, 80, 8192, 8),
         ("125M b8 chunk 8", 8, 12, 1024, 9216, 64, 8192, 8), ("causal N4096 D64 64 heads", 4, 16, 4096, 4096, 64, 4096, 0), ("causal N4096 D96 64 heads", 4, 16, 4096, 4096, 96, 4096, 0)]
for name, B, H, Nq, Nkv, D, ws, cid in CASES:
    g = torch.Generator(device='cuda').manual_seed(0)
    mk = lambda n: torch.randn(B, H, n, D, device='cuda', generator=g).to(torch.bfloat16)
    Q, K, V, dO, gQ, gK, gV = mk(Nq), mk(Nkv), mk(Nkv), mk(Nq), mk(Nq), mk(Nkv), mk(Nkv)
    O, L = tcapi.forward(Q, K, V, ws, cid)
    Or, Lr = ref.v7_forward(Q, K, V, ws, cid)
    pairs = orc.visible_pairs(cid, Nq, Nkv, ws) * B * H
    res = dict(case=name)
    for tag, fwd, bwd, hvp, o, l in (("ours", tcapi.forward, tcapi.backward, tcapi.double_backward, O, L), ("ref", ref.v7_forward, ref.v7_backward, ref.v7_double_backward, Or, Lr)):
        tf = timeit(lambda: fwd(Q, K, V, ws, cid))
        tb = timeit(lambda: bwd(dO, Q, K, V, o, l, ws, cid))
        th = timeit(lambda: hvp(gQ, gK, gV, dO, Q, K, V, o, l, ws, cid))
        res[tag] = dict(fwd_ms=round(tf, 3), bwd_ms=round(tb, 3), hvp_ms=round(th, 3), hvp_tflops=round(2 * D * 12 * pairs / (th * 1e-3) / 1e12, 1))
    res["speedup"] = {k: round(res["ref"][k] / res["ours"][k], 1) for k in ("fwd_ms", "bwd_ms", "hvp_ms")}
    print(json.dumps(res), flush=True)
