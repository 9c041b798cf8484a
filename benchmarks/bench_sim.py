"""Configuration 1 without a GPU: R simulated ranks in one process (CPU oracle + simulator).

  python benchmarks/bench_sim.py [--R 8 --S 512 --K 8 --E 64 --H 256 --token-padding 16]

For every target MaxVio it plans, dispatches and combines through plain arrays, checks the
guarantees (every rank receives exactly S*K rows; at most epn prefetch slots per rank, all from one
remote home group; ``combine(dispatch(x)) == sum_k w_k x``) and prints the plan's telemetry and the
wall-clock time of the CPU planner, as one JSON line per MaxVio.  The reference has no GPU-less
mode; its oracle needs a process group to see other ranks (tests/planning_reference.py:44-52).
"""
import argparse
import json
import os
import sys
import time

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from moonep_b200.reference import SimGroup  # noqa: E402
from moonep_b200.utils.routing import routing_for_maxvio  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--R", type=int, default=8)
    ap.add_argument("--S", type=int, default=512)
    ap.add_argument("--K", type=int, default=8)
    ap.add_argument("--E", type=int, default=64)
    ap.add_argument("--H", type=int, default=256)
    ap.add_argument("--token-padding", type=int, default=16)
    ap.add_argument("--maxvio", default="0,1,4")
    a = ap.parse_args()
    R, S, K, E, H = a.R, a.S, a.K, a.E, a.H
    epn = E // R
    sim = SimGroup(S, H, K, E, R, a.token_padding)
    x = torch.randn(R, S, H, generator=torch.Generator().manual_seed(11))
    for target in (float(t) for t in a.maxvio.split(",")):
        topk, w, mv, _ = routing_for_maxvio(S, K, E, R, target, seed=7)
        t0 = time.perf_counter()
        tables, dst = sim.plan(topk)
        t_plan = time.perf_counter() - t0
        t0 = time.perf_counter()
        hidden, w_nvs, cu, plans = sim.dispatch(x, w, topk)
        out, w_back = sim.combine(plans, hidden * w_nvs[:, :, None], w_nvs)
        t_rt = time.perf_counter() - t0
        etc = tables.experts_to_copy
        rows = tables.alloc.sum(0).tolist()
        homes_ok = all(len(set((etc[d][etc[d] >= 0] // epn).tolist())) <= 1 for d in range(R))
        err = float((out - x * w.sum(dim=2, keepdim=True)).abs().max())
        ok = rows == [S * K] * R and homes_ok and err < 1e-4 and torch.equal(w_back, w)
        print(json.dumps({
            "config": dict(R=R, S=S, K=K, E=E, H=H, token_padding=a.token_padding),
            "maxvio_target": target, "maxvio_achieved": round(float(mv), 3), "ok": bool(ok),
            "rows_per_rank": rows[0], "redundant_experts_total": int((etc >= 0).sum()),
            "redundant_experts_max_per_rank": int((etc >= 0).sum(1).max()),
            "dedup_ratio": round(float((dst >= 0).sum()) / dst.numel(), 3),
            "padding_rows_total": int(tables.zero_fill[:, :, 1].sum()),
            "round_trip_max_abs_err": err,
            "cpu_plan_ms": round(t_plan * 1e3, 2), "cpu_dispatch_combine_ms": round(t_rt * 1e3, 2)}))
        if not ok:
            sys.exit(1)


if __name__ == "__main__":
    main()
