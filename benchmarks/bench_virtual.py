"""Dispatch / combine on a single-GPU virtual EP group (all R ranks in one cooperative launch per
kernel).  Peer traffic stays inside one device's HBM, so the timings are NOT NVLink numbers; the
script exists to profile the comm kernels' instruction and memory behaviour under ncu on one GPU
(multi-rank commands must not be profiled) and to smoke-test large shapes.

  python benchmarks/bench_virtual.py [--R 4 --S 2048 --H 7168 --K 8 --E 32 --iters 3]
"""
import argparse
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from moonep_b200 import Buffer  # noqa: E402
from moonep_b200.utils.routing import routing_for_maxvio, tokens_per_expert  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--R", type=int, default=4)
    ap.add_argument("--S", type=int, default=2048)
    ap.add_argument("--H", type=int, default=7168)
    ap.add_argument("--K", type=int, default=8)
    ap.add_argument("--E", type=int, default=32)
    ap.add_argument("--num-sms", type=int, default=16)
    ap.add_argument("--maxvio", type=float, default=2.0)
    ap.add_argument("--iters", type=int, default=3)
    a = ap.parse_args()
    buf = Buffer(a.S, a.H, a.K, a.E, a.R, num_sms=a.num_sms, token_padding=128, virtual=True, timeout_s=5.0)
    topk, w, mv, _ = routing_for_maxvio(a.S, a.K, a.E, a.R, a.maxvio, seed=3)
    tpe = torch.stack([tokens_per_expert(topk[r], a.E) for r in range(a.R)]).cuda()
    topk, w = topk.cuda(), w.cuda()
    x = torch.randn(a.R, a.S, a.H, device="cuda").bfloat16()
    res = {}
    h, _, _, plan = buf.dispatch(x, w, topk, tpe, zero_copy=True, router_weights_zero_copy=True)
    out, _, _ = buf.combine(plan, h, None, zero_copy=True)
    ref = (x.float() * a.K).bfloat16().float()
    res["identity_max_err"] = float((out.float() - ref).abs().max())
    # timing loops below re-run combine on an already pre-reduced shard: times only, no checks
    for name in ("dispatch", "combine"):
        ts = []
        for _ in range(a.iters + 1):
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            if name == "dispatch":
                s.record()
                h, wn, cu, plan = buf.dispatch(x, w, topk, tpe, zero_copy=True, router_weights_zero_copy=True)
                e.record()
            else:
                s.record()
                out, _, _ = buf.combine(plan, h, None, zero_copy=True)
                e.record()
            torch.cuda.synchronize()
            ts.append(s.elapsed_time(e) * 1e3)
        res[name + "_us"] = round(min(ts[1:]), 1)
    # the two local duplicate kernels on their own (bytes: rows read + rows written, all ranks)
    from moonep_b200 import _native as nat
    st = torch.cuda.current_stream().cuda_stream
    link = plan.link
    n_dup = int(((link & 0x40000000) != 0).sum())
    n_prim = int((((link & 0x40000000) == 0) & ((link & 0x00FFFFFF) != 0x00FFFFFF)).sum())
    for name, call, nbytes in (
            ("k_expand", lambda: nat.call("mep_launch_expand", buf._ctx, plan.link.data_ptr(),
                                          plan.cu_seqlens.data_ptr(), 0, st), (n_prim + n_dup) * a.H * 2),
            ("k_prologue", lambda: nat.call("mep_launch_combine_prologue", buf._ctx, plan.link.data_ptr(),
                                            plan.cu_seqlens.data_ptr(), st), (2 * n_prim + n_dup) * a.H * 2)):
        ts = []
        for _ in range(a.iters + 2):
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            call()
            e.record()
            torch.cuda.synchronize()
            ts.append(s.elapsed_time(e) * 1e3)
        res[name + "_us"] = round(min(ts[1:]), 1)
        res[name + "_gbs"] = round(nbytes / min(ts[1:]) / 1e3, 1)
    res["dup_groups"], res["dup_rows"] = n_prim, n_dup
    buf.check()
    res.update(R=a.R, S=a.S, H=a.H, K=a.K, E=a.E, maxvio=round(mv, 2), rows_per_rank=int(plan.cu_seqlens[0, -1]))
    print(json.dumps(res))
    buf.destroy()


if __name__ == "__main__":
    main()
