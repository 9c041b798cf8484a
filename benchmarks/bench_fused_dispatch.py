"""A/B of the dispatch fused into the consuming GEMM against the stand-alone dispatch kernel
followed by the same GEMM, on 1 GPU (one rank, local copies) or under torch.distributed.run.

Per-rank workload: S tokens, top-K of E experts (E / R local groups), gate/up GEMM with SwiGLU
(forward) and the down-dgrad GEMM (backward).  Rows printed (device time, CUDA events, max over
ranks, best of ``--rounds`` interleaved rounds so that all variants see the same clocks):

  dispatch            stand-alone dispatch (plan excluded; saved-plan launch + expansion)
  gemm                the GEMM alone on rows that are in place
  gemm_disp_idle      the fused kernel variant (one operand stage fewer, copy warp present) on rows
                      that are in place: it only checks arrival counters that are already full
  fused               the fused launch: the GEMM carries the dispatch
  dispatch+gemm       the sum of the first two, what the fused launch replaces

  python benchmarks/bench_fused_dispatch.py --E 32
  python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 benchmarks/bench_fused_dispatch.py --E 64
"""
import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from moonep_b200.api import Buffer  # noqa: E402
from moonep_b200.ops import gemm  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--S", type=int, default=4096)
    ap.add_argument("--H", type=int, default=7168)
    ap.add_argument("--Hp", type=int, default=2048)
    ap.add_argument("--K", type=int, default=8)
    ap.add_argument("--E", type=int, default=32, help="total experts (E / world size per rank)")
    ap.add_argument("--rounds", type=int, default=5)
    ap.add_argument("--iters", type=int, default=4)
    ap.add_argument("--grid", type=int, default=0, help="CTA limit of the GEMM launches (0: all SMs)")
    a = ap.parse_args()
    R = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if R > 1:
        dist.init_process_group("nccl", device_id=dev)
    S, H, Hp, K, E = a.S, a.H, a.Hp, a.K, a.E
    epn = E // R
    buf = Buffer(S, H, K, E, R, num_sms=32 if R > 1 else 96, token_padding=128)
    g = torch.Generator(device=dev).manual_seed(rank)
    x = torch.randn(S, H, device=dev, generator=g).bfloat16()
    logits = torch.randn(S, E, device=dev, generator=g)
    val, idx = logits.topk(K, dim=1)
    topk, w = idx.to(torch.int32).contiguous(), torch.softmax(val, dim=1).contiguous()
    tpe = torch.bincount(topk.flatten().long(), minlength=E).to(torch.int32)
    wg = (torch.randn(epn, H, Hp, device=dev, generator=g) * 0.02).bfloat16()
    wu = (torch.randn(epn, H, Hp, device=dev, generator=g) * 0.02).bfloat16()
    wd = (torch.randn(epn, H, Hp, device=dev, generator=g) * 0.02).bfloat16()
    hid, wv, cu, plan = buf.dispatch(x, w, topk, tpe, zero_copy=True, router_weights_zero_copy=True)
    cul = cu[:epn].contiguous()
    rows = buf.NvS
    act = torch.empty(rows, Hp, dtype=torch.bfloat16, device=dev)
    gate, up = torch.empty_like(act), torch.empty_like(act)
    dact = torch.empty_like(act)

    def fused_fwd():
        h, wv2, _, _, disp = buf.dispatch_fused_begin(x, w, plan=plan)
        gemm.gateup_swiglu(h, wg, wu, cul, row_scale=wv2, out=(act, gate, up), dispatch=disp, grid=a.grid)

    def fused_bwd():
        h, _, _, _, disp = buf.dispatch_fused_begin(x, plan=plan)
        gemm.down_dgrad(h, wd, cul, out=dact, dispatch=disp, grid=a.grid)

    idle = dict(mode=1, ctx=buf._ctx, fresh=0, shard=0)
    variants = {
        "dispatch": lambda: buf.dispatch(x, plan=plan, zero_copy=True),
        "gateup.gemm": lambda: gemm.gateup_swiglu(hid, wg, wu, cul, row_scale=wv, out=(act, gate, up), grid=a.grid),
        "gateup.gemm_disp_idle": lambda: gemm.gateup_swiglu(hid, wg, wu, cul, row_scale=wv, out=(act, gate, up),
                                                            dispatch=idle, grid=a.grid),
        "gateup.fused": fused_fwd,
        "dgrad.gemm": lambda: gemm.down_dgrad(hid, wd, cul, out=dact, grid=a.grid),
        "dgrad.gemm_disp_idle": lambda: gemm.down_dgrad(hid, wd, cul, out=dact, dispatch=idle, grid=a.grid),
        "dgrad.fused": fused_bwd,
    }

    filler = torch.randn(8192, 8192, device=dev, dtype=torch.bfloat16)

    def run(fn):
        if R > 1:
            dist.barrier()
        torch.cuda.synchronize()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        filler @ filler            # keeps the GPU busy while the host queues the timed launches
        s.record()
        for _ in range(a.iters):
            fn()
        e.record()
        torch.cuda.synchronize()
        t = torch.tensor([s.elapsed_time(e) / a.iters], device=dev)
        if R > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t)

    fused_fwd()                      # leaves every arrival counter full for the "idle" variants
    for fn in variants.values():
        fn()
    best = {k: 1e9 for k in variants}
    for _ in range(a.rounds):
        for k, fn in variants.items():
            if k.endswith("idle"):
                fused_fwd()          # counters full again (a saved-plan entry clears them)
                torch.cuda.synchronize()
            best[k] = min(best[k], run(fn))
    buf.check()
    gemm.check_status()
    if os.environ.get("MOONEP_B200_FD_EXPERIMENT") is not None:
        # a build with -DMEP_GEMM_EXPERIMENTS records the longest copy-warp run and the summed
        # arrival waits of the last launches in the GEMM status words 7 and 6 (microseconds)
        for name, fn in (("gateup.fused", fused_fwd), ("dgrad.fused", fused_bwd)):
            gemm.reset_status()
            fn()
            torch.cuda.synchronize()
            st = gemm.status_word(dev).tolist()
            print(f"[experiment] {name}: longest copy warp {st[7]} us, arrival waits summed over CTAs {st[6]} us",
                  flush=True)
        gemm.reset_status()
    real = int(cu[-1])
    fl_gu = 2.0 * real * H * 2 * Hp
    fl_dg = 2.0 * real * H * Hp
    out = {"R": R, "S": S, "H": H, "Hp": Hp, "K": K, "E": E, "rows": real, "grid": a.grid,
           "ms": {k: round(v, 4) for k, v in best.items()}}
    out["ms"]["gateup.dispatch+gemm"] = round(best["dispatch"] + best["gateup.gemm"], 4)
    out["ms"]["dgrad.dispatch+gemm"] = round(best["dispatch"] + best["dgrad.gemm"], 4)
    out["tflops"] = {"gateup.gemm": round(fl_gu / best["gateup.gemm"] / 1e9), "gateup.fused": round(fl_gu / best["gateup.fused"] / 1e9),
                     "dgrad.gemm": round(fl_dg / best["dgrad.gemm"] / 1e9), "dgrad.fused": round(fl_dg / best["dgrad.fused"] / 1e9)}
    if rank == 0:
        print(json.dumps(out), flush=True)
    buf.destroy()
    if R > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
