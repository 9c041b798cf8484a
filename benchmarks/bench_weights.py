"""prefetch_weight / reduce_grad microbenchmark (run under torch.distributed.run).

Gate, up and down projections per expert with H=7168, H'=2048: bf16 weights ~N(0, 0.02) pushed
into the ``[R, epn, H, H']`` prefetch pools, fp32 grads ~N(0, 1e-3) pulled from the reduce pools.
The plan comes from Zipf-skewed routing at the requested MaxVio (default 4).  Reports, per op, the
worst rank's device time, the bytes the busiest owner moves and the resulting GB/s against the
NVLink per-GPU bandwidth.  Counterpart of the reference's bench_prefetch.py / bench_grad_reduce.py.

  python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 benchmarks/bench_weights.py
"""
import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from moonep_b200.api import Buffer  # noqa: E402
from moonep_b200.models.moe_layer import ExpertPools  # noqa: E402
from moonep_b200.utils.routing import routing_for_maxvio, tokens_per_expert  # noqa: E402

NVLINK_MEASURED_GBS, NVLINK_NOMINAL_GBS = 770.0, 900.0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--S", type=int, default=512)
    ap.add_argument("--K", type=int, default=8)
    ap.add_argument("--E", type=int, default=256)
    ap.add_argument("--H", type=int, default=7168)
    ap.add_argument("--Hp", type=int, default=2048)
    ap.add_argument("--maxvio", type=float, default=4.0)
    ap.add_argument("--num-sms", type=int, default=32)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--no-zero", action="store_true", help="reduce_grad without clearing the consumed slots")
    a = ap.parse_args()
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    R, rank = dist.get_world_size(), dist.get_rank()
    epn = a.E // R
    buf = Buffer(a.S, 256, a.K, a.E, R, num_sms=a.num_sms, token_padding=16)   # the plan only needs routing
    pools = ExpertPools(R, epn, a.H, a.Hp, buf.group, rank)
    g = torch.Generator(device=dev).manual_seed(rank)
    w = {n: (torch.randn(epn, a.H, a.Hp, device=dev, generator=g) * 0.02).bfloat16() for n in pools.names}
    gl = {n: torch.zeros(epn, a.H, a.Hp, device=dev) for n in pools.names}
    topk_all, w_all, mv, _ = routing_for_maxvio(a.S, a.K, a.E, R, a.maxvio, seed=7)
    topk = topk_all[rank].to(dev)
    tpe = tokens_per_expert(topk_all[rank], a.E).to(dev)
    x = torch.zeros(a.S, 256, device=dev, dtype=torch.bfloat16)
    _, _, _, plan = buf.dispatch(x, None, topk, tpe)
    etc = plan.experts_to_copy.cpu()
    owners = torch.bincount((etc[etc >= 0] // epn).long(), minlength=R)      # slots per owner rank
    per_expert = a.H * a.Hp

    def fill_reduce():
        for n in pools.names:
            pools.reduce[n][rank].normal_(0.0, 1e-3, generator=g)

    def timed(fn, prep=None):
        ts = []
        for i in range(a.warmup + a.iters):
            if prep is not None:
                prep()
            dist.barrier()
            torch.cuda.synchronize()
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            fn()
            e.record()
            torch.cuda.synchronize()
            if i >= a.warmup:
                ts.append(s.elapsed_time(e) * 1e3)
        t = torch.tensor([sum(ts) / len(ts)], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t)

    pf = lambda: buf.prefetch_weight(
        plan, local_gate_weight=w["gate"], local_up_weight=w["up"], local_down_weight=w["down"],
        gate_prefetch_buffer=pools.prefetch["gate"], up_prefetch_buffer=pools.prefetch["up"],
        down_prefetch_buffer=pools.prefetch["down"])
    rg = lambda: buf.reduce_grad(
        plan, local_gate_grad=gl["gate"], local_up_grad=gl["up"], local_down_grad=gl["down"],
        gate_reduce_buffer=pools.reduce["gate"], up_reduce_buffer=pools.reduce["up"],
        down_reduce_buffer=pools.reduce["down"], zero_consumed=not a.no_zero)
    us_pf = timed(pf)
    us_rg = timed(rg, prep=fill_reduce)
    buf.check()
    busiest = int(owners.max())
    push_bytes = busiest * 3 * per_expert * 2
    pull_bytes = busiest * 3 * per_expert * 4
    if rank == 0:
        out = {"bench": "prefetch_weight+reduce_grad", "R": R, "E": a.E, "epn": epn, "H": a.H, "Hp": a.Hp,
               "maxvio": round(mv, 3), "remote_slots_total": int((etc >= 0).sum()),
               "slots_of_busiest_owner": busiest,
               "prefetch_us_worst_rank": round(us_pf, 1), "prefetch_bytes_busiest_owner": push_bytes,
               "prefetch_gbs": round(push_bytes / us_pf / 1e3, 1) if us_pf > 0 else None,
               "reduce_grad_us_worst_rank": round(us_rg, 1), "reduce_clears_slots": not a.no_zero, "reduce_bytes_busiest_owner": pull_bytes,
               "reduce_gbs": round(pull_bytes / us_rg / 1e3, 1) if us_rg > 0 else None,
               "nvlink_measured_gbs": NVLINK_MEASURED_GBS, "nvlink_nominal_gbs": NVLINK_NOMINAL_GBS}
        if out["prefetch_gbs"]:
            out["prefetch_frac_of_measured"] = round(out["prefetch_gbs"] / NVLINK_MEASURED_GBS, 3)
            out["reduce_frac_of_measured"] = round(out["reduce_gbs"] / NVLINK_MEASURED_GBS, 3)
        print(json.dumps(out), flush=True)
    buf.destroy()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
