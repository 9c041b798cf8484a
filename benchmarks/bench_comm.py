"""Communication benchmark (run under torch.distributed.run, one process per GPU):
plan + dispatch, prefetch_weight, combine, their backward variants and reduce_grad at the
DeepSeek-V3 shape (S=4096 tokens/rank, H=7168, K=8, E=256, token_padding=128, num_sms=32),
swept over routing imbalance, next to the NCCL ``all_to_all_single`` + permute baseline.
Counterpart of the reference's benchmarks/bench_comm.py and bench_vs_deepep.py; timing is
CUDA events on the launching stream, warm-up first, MAX over ranks.

  python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 benchmarks/bench_comm.py
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
from moonep_b200.parallel.nccl_baseline import NcclAllToAllEP  # noqa: E402
from moonep_b200.utils.routing import routing_for_maxvio, tokens_per_expert  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--S", type=int, default=4096)
    ap.add_argument("--H", type=int, default=7168)
    ap.add_argument("--Hp", type=int, default=2048)
    ap.add_argument("--K", type=int, default=8)
    ap.add_argument("--E", type=int, default=256)
    ap.add_argument("--num-sms", type=int, default=32)
    ap.add_argument("--maxvio", default="0,0.5,1,2,4,8")
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--no-weights", action="store_true", help="skip prefetch / reduce_grad pools")
    ap.add_argument("--out", default="")
    args = ap.parse_args()
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    R, rank = dist.get_world_size(), dist.get_rank()
    S, H, Hp, K, E = args.S, args.H, args.Hp, args.K, args.E
    epn = E // R
    buf = Buffer(S, H, K, E, R, num_sms=args.num_sms, token_padding=128)
    pools = None if (args.no_weights or R == 1) else ExpertPools(R, epn, H, Hp, buf.group, rank)
    g = torch.Generator(device=dev).manual_seed(rank)
    x = torch.randn(S, H, device=dev, generator=g).bfloat16()
    if pools is not None:
        w_loc = {n: (torch.randn(epn, H, Hp, device=dev, generator=g) * 0.02).bfloat16() for n in pools.names}
        g_loc = {n: torch.zeros(epn, H, Hp, device=dev) for n in pools.names}
    nccl = NcclAllToAllEP(S, H, K, E)

    def timed(fn):
        for _ in range(args.warmup):
            fn()
        dist.barrier()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(args.iters):
            fn()
        b.record()
        torch.cuda.synchronize()
        t = torch.tensor([a.elapsed_time(b) / args.iters * 1e3], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return round(float(t), 1)

    results = []
    for target in [float(v) for v in args.maxvio.split(",")]:
        topk_all, w_all, mv, _ = routing_for_maxvio(S, K, E, R, target, seed=7)
        topk, w = topk_all[rank].to(dev), w_all[rank].to(dev)
        tpe = tokens_per_expert(topk_all[rank], E).to(dev)
        st = {}

        def fwd_dispatch():
            st["h"], st["w"], st["cu"], st["plan"] = buf.dispatch(
                x, w, topk, tpe, zero_copy=True, router_weights_zero_copy=True)

        fwd_dispatch()
        plan = st["plan"]
        row = {"R": R, "maxvio_target": target, "maxvio": round(mv, 3),
               "dispatch_fwd_us": timed(fwd_dispatch),
               "dispatch_bwd_us": timed(lambda: buf.dispatch(x, plan=plan, zero_copy=True)),
               "combine_fwd_us": timed(lambda: buf.combine(plan, st["h"], None, zero_copy=True)),
               "combine_bwd_us": timed(lambda: buf.combine(plan, st["h"], st["w"], zero_copy=True,
                                                            router_weights_zero_copy=True))}
        if pools is not None:
            pf = lambda: buf.prefetch_weight(
                plan, local_gate_weight=w_loc["gate"], local_up_weight=w_loc["up"],
                local_down_weight=w_loc["down"], gate_prefetch_buffer=pools.prefetch["gate"],
                up_prefetch_buffer=pools.prefetch["up"], down_prefetch_buffer=pools.prefetch["down"])
            rg = lambda: buf.reduce_grad(
                plan, local_gate_grad=g_loc["gate"], local_up_grad=g_loc["up"], local_down_grad=g_loc["down"],
                gate_reduce_buffer=pools.reduce["gate"], up_reduce_buffer=pools.reduce["up"],
                down_reduce_buffer=pools.reduce["down"])
            row["prefetch_us"] = timed(pf)
            row["reduce_grad_us"] = timed(rg)

            def roundtrip():
                fwd_dispatch()
                pf()
                buf.combine(st["plan"], st["h"], None, zero_copy=True)
        else:
            def roundtrip():
                fwd_dispatch()
                buf.combine(st["plan"], st["h"], None, zero_copy=True)
        row["roundtrip_us"] = timed(roundtrip)
        # per-kernel breakdown (the launchers the API calls, timed one by one)
        from moonep_b200 import _native as nat
        stream = lambda: torch.cuda.current_stream().cuda_stream
        out_sh = torch.empty(S, H, dtype=torch.bfloat16, device=dev)
        row["k_sync_us"] = timed(lambda: nat.call("mep_launch_sync", buf._ctx, stream()))
        row["k_plan_us"] = timed(lambda: (nat.call(
            "mep_launch_plan", buf._ctx, topk.data_ptr(), tpe.data_ptr(), plan.dst.data_ptr(),
            plan.cu_seqlens.data_ptr(), plan.zero_fill_ranges.data_ptr(), plan.experts_to_copy.data_ptr(),
            plan.remote_stats.data_ptr(), plan.send_order.data_ptr(), stream()),
            nat.call("mep_launch_sync", buf._ctx, stream())))
        row["k_dispatch_us"] = timed(lambda: nat.call(
            "mep_launch_dispatch", buf._ctx, x.data_ptr(), 0, plan.dst.data_ptr(),
            plan.zero_fill_ranges.data_ptr(), 0, 0, 1, 0, 0, stream()))
        row["k_expand_us"] = timed(lambda: nat.call(
            "mep_launch_expand", buf._ctx, plan.link.data_ptr(), plan.cu_seqlens.data_ptr(), 0, stream()))
        row["k_prologue_us"] = timed(lambda: nat.call(
            "mep_launch_combine_prologue", buf._ctx, plan.link.data_ptr(), plan.cu_seqlens.data_ptr(), stream()))
        row["k_combine_us"] = timed(lambda: nat.call(
            "mep_launch_combine", buf._ctx, plan.dst.data_ptr(), out_sh.data_ptr(), 0, stream()))
        etc = plan.experts_to_copy
        row["remote_experts_max_per_rank"] = int((etc >= 0).sum(1).max())
        row["remote_experts_total"] = int((etc >= 0).sum())
        dstv = plan.dst
        sent = (dstv >= 0) & (dstv // buf.NvS != rank)
        row["nvlink_rows_sent"] = int(sent.sum())
        row["dispatch_nvlink_gbs"] = round(int(sent.sum()) * H * 2 / (row["dispatch_bwd_us"] * 1e-6) / 1e9, 1)
        if R > 1:
            ns = {}

            def nccl_rt():
                rows, _, s2 = nccl.dispatch(x, topk)
                ns["rows"] = s2.rows
                nccl.combine(rows, s2)

            try:
                row["nccl_a2a_roundtrip_us"] = timed(nccl_rt)
                mx = torch.tensor([ns["rows"]], device=dev)
                dist.all_reduce(mx, op=dist.ReduceOp.MAX)
                row["nccl_max_recv_rows"] = int(mx)
            except RuntimeError as exc:               # e.g. out of memory under heavy skew
                row["nccl_a2a_roundtrip_us"] = None
                row["nccl_error"] = str(exc)[:120]
        buf.check()
        results.append(row)
        if rank == 0:
            print(json.dumps(row), flush=True)
    if rank == 0 and args.out:
        with open(args.out, "w") as fh:
            json.dump(results, fh, indent=1)
    buf.destroy()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
