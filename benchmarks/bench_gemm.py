"""Throughput of the tcgen05 grouped GEMM at the per-rank shapes of the EP=8 MoE layer
(32 experts x 1024 rows, H=7168, H'=2048) on ONE GPU, against the measured cuBLAS bf16 peak.

  python benchmarks/bench_gemm.py [--rows-per-group 1024 --groups 32 --H 7168 --Hp 2048]
"""
import argparse
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from moonep_b200.ops import elementwise as ew  # noqa: E402
from moonep_b200.ops import gemm  # noqa: E402


def timeit(fn, iters=10, warmup=3, flush=None):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        if flush is not None:
            flush.zero_()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        ts.append(a.elapsed_time(b))
    ts.sort()
    return ts[len(ts) // 2]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--groups", type=int, default=32)
    ap.add_argument("--rows-per-group", type=int, default=1024)
    ap.add_argument("--H", type=int, default=7168)
    ap.add_argument("--Hp", type=int, default=2048)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--only", default="")
    ap.add_argument("--ab", action="store_true",
                    help="interleaved A/B of the kernel variants (single CTA / CTA pair, TMA-store / plain "
                         "epilogue, weight grad with and without the fused SGD step): best of 6 rounds each, "
                         "run back to back so that all variants see the same clocks")
    args = ap.parse_args()
    G, rpg, H, Hp = args.groups, args.rows_per_group, args.H, args.Hp
    rows = G * rpg
    dev = "cuda"
    peaks = {}
    try:
        peaks = json.load(open(os.path.join(os.path.dirname(__file__), "..", "MEASURED_PEAKS.json")))
    except OSError:
        pass
    peak = peaks.get("bf16_tflops", 1590.0)
    hbm = peaks.get("hbm_gbs", 6650.0)
    g = torch.Generator(device=dev).manual_seed(0)
    cu = (torch.arange(1, G + 1, device=dev) * rpg).to(torch.int32)
    x = torch.randn(rows, H, device=dev, generator=g).bfloat16()
    wg = (torch.randn(G, H, Hp, device=dev, generator=g) * 0.02).bfloat16()
    wu = (torch.randn(G, H, Hp, device=dev, generator=g) * 0.02).bfloat16()
    wd = (torch.randn(G, H, Hp, device=dev, generator=g) * 0.02).bfloat16()
    rs = torch.rand(rows, device=dev, generator=g)
    act, gate, up = gemm.gateup_swiglu(x, wg, wu, cu, row_scale=rs)
    y = torch.empty(rows, H, dtype=torch.bfloat16, device=dev)
    grad = torch.zeros(G, H, Hp, device=dev)
    flush = torch.empty(256 * 2 ** 20, dtype=torch.uint8, device=dev)   # > L2
    F = 2.0 * rows * H * Hp
    ops = {
        "gateup_swiglu": (lambda: gemm.gateup_swiglu(x, wg, wu, cu, row_scale=rs), 2 * F),
        "down": (lambda: gemm.down(act, wd, cu, out=y), F),
        "down_dgrad": (lambda: gemm.down_dgrad(y, wd, cu), F),
        "gateup_dgrad": (lambda: gemm.gateup_dgrad(gate, up, wg, wu, cu, out=y), 2 * F),
        "wgrad": (lambda: gemm.wgrad(x, act, cu, grad), F),
        "cublas_ref_down(torch.bmm)": (lambda: torch.bmm(act.view(G, rpg, Hp), wd.transpose(1, 2)), F),
    }
    out = {"shape": dict(groups=G, rows_per_group=rpg, H=H, Hp=Hp), "peak_tflops_measured": peak}
    if args.ab:
        return ab(args, ops, x, act, cu, grad, wg, out)
    for name, (fn, flops) in ops.items():
        if args.only and args.only not in name:
            continue
        ms = timeit(fn, args.iters, flush=flush)
        out[name] = {"ms": round(ms, 4), "tflops": round(flops / ms / 1e9, 1),
                     "frac_of_measured_peak": round(flops / ms / 1e9 / peak, 3)}
    n = G * H * Hp
    if not args.only:
        nbytes = rows * Hp * 2 * 5 + rows * 4
        ms = timeit(lambda: ew.swiglu_bwd(act, gate, up, rs), args.iters, flush=flush)
        out["swiglu_bwd"] = {"ms": round(ms, 4), "gbs": round(nbytes / ms / 1e6, 1),
                             "frac_of_measured_hbm": round(nbytes / ms / 1e6 / hbm, 3)}
        ms = timeit(lambda: ew.sgd_update_(wg, grad, 1e-6), args.iters, flush=flush)
        out["sgd_update"] = {"ms": round(ms, 4), "gbs": round(n * 8 / ms / 1e6, 1),
                             "frac_of_measured_hbm": round(n * 8 / ms / 1e6 / hbm, 3)}
    if not args.only:
        ms = timeit(lambda: grad.zero_(), args.iters, flush=flush)
        out["hbm_write_only(torch zero_)"] = {"ms": round(ms, 4), "gbs": round(n * 4 / ms / 1e6, 1)}
    torch.cuda.synchronize()
    gemm.check_status()
    print(json.dumps(out))


def ab(args, ops, x, act, cu, grad, w, out):
    def run(fn, n=6):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(n):
            fn()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) / n

    variants = [("single", 0, False), ("single_plain_epilogue", 0, True), ("pair", 1, False), ("pair_plain_epilogue", 1, True)]
    ops = dict(ops)
    ops.pop("cublas_ref_down(torch.bmm)", None)
    flops_w = ops["wgrad"][1]
    ops["wgrad_fused_sgd"] = (lambda: gemm.wgrad(x, act, cu, grad, sgd=(w, 1e-6, None)), flops_w)
    for name, (fn, flops) in ops.items():
        if args.only and args.only not in name:
            continue
        vs = [v for v in variants if "wgrad" not in name or not v[2]]
        for _, two, dbg in vs:
            gemm.TWO_CTA, gemm.PLAIN_EPILOGUE = two, dbg
            fn()
        torch.cuda.synchronize()
        best = {v[0]: 1e9 for v in vs}
        for _ in range(6):
            for v, two, dbg in vs:
                gemm.TWO_CTA, gemm.PLAIN_EPILOGUE = two, dbg
                best[v] = min(best[v], run(fn))
        out[name] = {v: {"ms": round(t, 4), "tflops": round(flops / t / 1e9)} for v, t in best.items()}
    gemm.TWO_CTA, gemm.PLAIN_EPILOGUE = 2, False
    gemm.check_status()
    print(json.dumps(out))


if __name__ == "__main__":
    main()
