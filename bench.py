"""Headline benchmark: MoE-layer training throughput (tokens/s) at EP = N GPUs.

One DeepSeek-V3-shaped MoE layer (router 7168->256, top-8 softmax, 256 SwiGLU experts with
H=7168, H'=2048, bf16 weights / fp32 grads), S=4096 tokens per rank drawn ~N(0,1) with a
Zipf-skewed router bias, forward + backward + SGD step.  Weak scaling: every rank keeps its 4096
tokens, the experts are sharded E/N per rank.  Alongside it the communication round trip
(plan + dispatch + prefetch_weight + combine) is timed at the same shape and reported in µs.

  python bench.py --gpus 1 --steps 10 --warmup 3
  python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
      --master-port 29500 bench.py --gpus 8 --steps 10 --warmup 3
  python bench.py --impl reference ...      # the unmodified reference under baseline/_ref

Prints ONE JSON line on rank 0.  Data are synthetic and weights random-init.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import tempfile
import time

REPO = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, REPO)

S, H, HP, K, E = 4096, 7168, 2048, 8, 256
TOKEN_PADDING, NUM_SMS = 128, 32


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--maxvio", type=float, default=2.0, help="target routing imbalance")
    ap.add_argument("--lr", type=float, default=1e-3)
    ap.add_argument("--small", action="store_true", help="reduced shape for profiling captures (not a bench)")
    ap.add_argument("--no-graph", action="store_true", help="issue the step eagerly instead of replaying a CUDA graph")
    ap.add_argument("--trace", action="store_true", help="also print a per-span device-time table")
    ap.add_argument("--weight-sms", type=int, default=16,
                    help="CTAs of prefetch_weight / reduce_grad, which run next to the GEMMs")
    ap.add_argument("--comm-sms", type=int, default=0,
                    help="CTAs of dispatch / combine (default: 32 with peers, 96 on one GPU, where they are local copies)")
    ap.add_argument("--no-fused-combine", action="store_true",
                    help="down GEMM into the shard + pull combine instead of the push epilogue")
    ap.add_argument("--no-fused-dispatch", action="store_true",
                    help="stand-alone dispatch kernels (all-to-all, barrier, duplicate expansion) before the "
                         "gate/up and down-dgrad GEMMs instead of the dispatch carried by those GEMM launches")
    ap.add_argument("--ab-dispatch", action="store_true",
                    help="also time the step with the other dispatch variant (fused into the GEMMs / stand-alone) "
                         "in the same process, interleaved round by round, and report both under 'ab_dispatch'")
    ap.add_argument("--copy-dispatch-out", action="store_true",
                    help="forward dispatch copies its rows out of the shard (instead of keeping them in a "
                         "second shard until backward is done)")
    ap.add_argument("--no-fused-sgd", action="store_true",
                    help="store fp32 weight grads and run the SGD kernel over all experts, instead of "
                         "applying SGD in the weight-grad epilogues (bit-identical results)")
    ap.add_argument("--experts", type=int, default=E,
                    help="total experts; anything but 256 is a profiling shape, not the benchmark")
    return ap.parse_args()


class ClockSampler:
    """nvidia-smi clock / throttle-reason samples during the timed region (read-only query)."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, device_index: int):
        self.path = tempfile.mktemp(prefix="clocks_", suffix=".csv")
        self.proc = None
        self.index = device_index

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.index)], stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], 0.0, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        try:
            for line in open(self.path):
                f = [x.strip() for x in line.split(",")]
                if len(f) < 9:
                    continue
                try:
                    sm.append(float(f[1]))
                    mx = max(mx, float(f[2]))
                except ValueError:
                    continue
                for n, v in zip(names, f[5:9]):
                    if v.lower().startswith("active"):
                        reasons.add(n)
            os.unlink(self.path)
        except OSError:
            pass
        sm.sort()
        med = sm[len(sm) // 2] if sm else None
        return {"sm_mhz": med, "sm_max_mhz": mx or None, "reasons": sorted(reasons), "samples": len(sm)}


def calibrate_bias(layer, x, target, dist, R):
    """Zipf router bias whose exponent is searched so that the global MaxVio hits ``target``."""
    import torch

    from moonep_b200.ops import elementwise as ew
    from moonep_b200.ops import gemm
    if target <= 0:
        return None, 0.0
    dev = x.device
    g = torch.Generator().manual_seed(1234)
    n_exp = layer.w_router.shape[1]
    order = torch.randperm(n_exp, generator=g)
    ranks = torch.empty(n_exp)
    ranks[order] = torch.arange(1, n_exp + 1, dtype=torch.float32)
    logpop = -torch.log(ranks).to(dev)
    logits = gemm.dense(x, layer.w_router)
    lo, hi, best = 0.0, 8.0, (None, 1e9)
    for _ in range(20):
        mid = 0.5 * (lo + hi)
        bias = (mid * logpop).contiguous()
        _, _, tpe = ew.router_topk(logits, K, bias)
        tot = tpe.to(torch.float32)
        if R > 1:
            dist.all_reduce(tot)
        mv = float(tot.max() / tot.mean() - 1.0)
        if abs(mv - target) < abs(best[1] - target):
            best = (bias, mv)
        if mv < target:
            lo = mid
        else:
            hi = mid
    return best


def run_ours(args):
    import torch
    import torch.distributed as dist

    from moonep_b200 import _native as nat
    from moonep_b200.api import Buffer
    from moonep_b200.models.moe_layer import ExpertPools, MoELayer

    R = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    assert R == args.gpus, f"--gpus {args.gpus} but WORLD_SIZE={R}"
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if R > 1:
        dist.init_process_group("nccl", device_id=dev)
    s, h, hp, k, e = (512, 1024, 512, 4, 32) if args.small else (S, H, HP, K, args.experts)
    buf = Buffer(s, h, k, e, R, num_sms=args.comm_sms or (NUM_SMS if R > 1 else 96), token_padding=TOKEN_PADDING,
                 num_sms_weights=args.weight_sms)
    pools = ExpertPools(R, e // R, h, hp, buf.group, rank) if R > 1 else None
    layer = MoELayer(buf, hp, pools, seed=0, fused_combine=not args.no_fused_combine,
                     hidden_in_place=not args.copy_dispatch_out,
                     fused_dispatch=False if args.no_fused_dispatch else None)
    gen = torch.Generator(device=dev).manual_seed(100 + rank)
    n_batches = 4
    host = [torch.randn(s, h, generator=torch.Generator().manual_seed(1000 * rank + i)).bfloat16().pin_memory()
            for i in range(n_batches)]
    xs = [t.to(dev) for t in host]
    if not args.small:
        bias, mv = calibrate_bias(layer, xs[0], args.maxvio, dist, R)
    else:
        bias, mv = None, 0.0
    layer.router_bias = bias
    if not args.no_fused_sgd:
        layer.fuse_sgd(args.lr)

    def step(x):
        x = x.detach().requires_grad_(True)
        y = layer(x)
        loss = y.float().pow(2).mean()
        loss.backward()
        layer.sgd_step(args.lr)
        return loss

    def barrier():
        if R > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps):
        barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for i in range(steps):
            fn(i)
        b.record()
        barrier()
        ms = torch.tensor([a.elapsed_time(b)], device=dev)
        if R > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms) / steps

    for i in range(max(args.warmup, 3)):
        step(xs[i % n_batches])
    buf.check()
    # The whole step (forward + backward + SGD, ~300 launches) is captured into one CUDA graph;
    # the timed loops replay it.  Falls back to eager issue if capture is not possible.
    eager_step, graphed = step, False
    nat.LAUNCHES = 0
    eager_step(xs[0])
    launches_per_step = nat.LAUNCHES          # kernels of this library launched by one step
    if not args.no_graph:
        try:
            from moonep_b200.utils.graph import GraphedStep
            gs = GraphedStep(lambda x: eager_step(x), [xs[0]], warmup=1)
            step = lambda x: gs(x)
            graphed = True
            for i in range(2):
                step(xs[i % n_batches])
            buf.check()
        except Exception as exc:  # noqa: BLE001
            if rank == 0:
                print(f"[bench] CUDA graph capture failed, running eagerly: {type(exc).__name__}: {exc}",
                      file=sys.stderr, flush=True)
            step = eager_step
            torch.cuda.synchronize()
    # ---- device-timed: inputs resident on the device ------------------------------------------
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    ms_step = timed(lambda i: step(xs[i % n_batches]), args.steps)
    launches = launches_per_step * args.steps   # replayed from the graph when graphed
    # ---- end to end: pinned host batch -> device every step, loss read back every step ---------
    # A two-deep pipeline, as a training loop with a data loader and asynchronous logging runs it:
    # while step i computes, the copy stream uploads batch i+1 from pinned memory, and the host
    # reads the loss of step i-1 (copied to pinned memory behind that step) instead of stalling
    # the GPU on step i's.  Every step still performs its own H2D copy (58.7 MB) and its own D2H
    # loss read inside the timed region; the last step's loss is read before the timer stops.
    # baseline/reference_arm.py times the reference with the same loop.
    copy_stream = torch.cuda.Stream(device=dev)
    stage = [torch.empty(s, h, dtype=torch.bfloat16, device=dev) for _ in range(2)]
    ready = [torch.cuda.Event(), torch.cuda.Event()]
    consumed = [torch.cuda.Event(), torch.cuda.Event()]
    losses = []
    loss_host = [torch.empty((), dtype=torch.float32).pin_memory() for _ in range(2)]
    loss_ready = [torch.cuda.Event(), torch.cuda.Event()]

    def upload(i):
        slot = i % 2
        with torch.cuda.stream(copy_stream):
            copy_stream.wait_event(consumed[slot])          # the step that used this slot is done
            stage[slot].copy_(host[i % n_batches], non_blocking=True)
            ready[slot].record(copy_stream)

    def prime():                # both slots free, batch 0 on its way, nothing read yet
        torch.cuda.synchronize()
        for ev in consumed:
            ev.record()
        upload(0)
        losses.clear()

    def e2e_step(i, n_steps=None):
        n_steps = args.steps if n_steps is None else n_steps
        slot = i % 2
        upload(i + 1)
        torch.cuda.current_stream().wait_event(ready[slot])
        loss = step(stage[slot])
        consumed[slot].record()
        loss_host[slot].copy_(loss.detach().float().reshape(()), non_blocking=True)
        loss_ready[slot].record()
        for j in ([i - 1] if i > 0 else []) + ([i] if i == n_steps - 1 else []):
            loss_ready[j % 2].synchronize()
            losses.append(float(loss_host[j % 2]))

    prime()
    for i in range(3):          # untimed: the loop's own first-use costs (copy stream, pinned reads)
        e2e_step(i, 3)
    prime()
    ms_e2e = timed(e2e_step, args.steps)
    clocks = sampler.stop() if rank == 0 else None
    # ---- optional A/B of the dispatch variant under identical clocks ---------------------------
    ab = None
    if args.ab_dispatch and graphed:
        from moonep_b200.utils.graph import GraphedStep
        layer_b = MoELayer(buf, hp, pools, seed=0, fused_combine=not args.no_fused_combine,
                           hidden_in_place=not args.copy_dispatch_out, fused_dispatch=not layer.fused_dispatch)
        layer_b.router_bias = layer.router_bias
        if not args.no_fused_sgd:
            layer_b.fuse_sgd(args.lr)

        def step_b_eager(x):
            x = x.detach().requires_grad_(True)
            loss = layer_b(x).float().pow(2).mean()
            loss.backward()
            layer_b.sgd_step(args.lr)
            return loss

        for i in range(3):
            step_b_eager(xs[i % n_batches])
        gs_b = GraphedStep(step_b_eager, [xs[0]], warmup=1)
        best = {"a": 1e9, "b": 1e9}
        for _ in range(3):
            best["a"] = min(best["a"], timed(lambda i: step(xs[i % n_batches]), args.steps))
            best["b"] = min(best["b"], timed(lambda i: gs_b(xs[i % n_batches]), args.steps))
        name = lambda fused: "fused_into_gemm_ms" if fused else "standalone_ms"
        ab = {name(layer.fused_dispatch): best["a"], name(layer_b.fused_dispatch): best["b"],
              "what": "ms per step, best of 3 interleaved rounds, both variants in this process"}
        buf.check()
    # ---- communication round trip at the same shape (plan + dispatch + prefetch + combine) -----
    topk_w = {}

    def comm_round(i):
        from moonep_b200.ops import elementwise as ew
        from moonep_b200.ops import gemm
        if not topk_w:
            logits = gemm.dense(xs[0], layer.w_router)
            topk_w["v"] = ew.router_topk(logits, k, layer.router_bias)
        topk, w, tpe = topk_w["v"]
        hid, wn, cu, plan = buf.dispatch(xs[0], w, topk, tpe, zero_copy=True, router_weights_zero_copy=True)
        if pools is not None:
            buf.prefetch_weight(plan, local_gate_weight=layer.w_gate, local_up_weight=layer.w_up,
                                local_down_weight=layer.w_down, gate_prefetch_buffer=pools.prefetch["gate"],
                                up_prefetch_buffer=pools.prefetch["up"], down_prefetch_buffer=pools.prefetch["down"])
        buf.combine(plan, hid, None, zero_copy=True)

    for i in range(3):
        comm_round(i)
    ms_comm = timed(comm_round, max(args.steps, 10))
    buf.check()
    from moonep_b200.ops import gemm as _g
    _g.check_status(dev)
    peak_gb = torch.cuda.max_memory_allocated(dev) / 2 ** 30
    stats = buf.stats()
    tokens = R * s
    out = {
        "metric": "moe_layer_train_tokens_per_s", "value": tokens / (ms_step / 1e3), "unit": "tokens/s",
        "n_gpus": R, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_step,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic (N(0,1) tokens, random-init weights, Zipf router bias)",
        "impl": "ours",
        "config": {"model": "deepseek-v3-style MoE layer: router 7168->256 top-8 softmax, 256 SwiGLU experts H=7168 H'=2048"
                   if not args.small and args.experts == E else f"profiling shape (experts={e})",
                   "global_batch": tokens, "seq_len": s, "parallelism": f"ep{R}",
                   "tokens_per_rank": s, "token_padding": TOKEN_PADDING, "num_sms_comm": buf.num_sms, "num_sms_weight_ops": buf.num_sms_weights,
                   "maxvio_target": args.maxvio, "maxvio_achieved": mv,
                   "step": "forward + backward + SGD update" + (
                       ", fp32 weight grads stored" if args.no_fused_sgd else
                       ", SGD applied in the weight-grad epilogues (fp32 accumulators; experts with "
                       "replicas store fp32 grads, reduce them home, then update)"),
                   "dispatch": "inside the gate/up and down-dgrad GEMM launches (rows consumed as they arrive)"
                   if layer.fused_dispatch else "stand-alone kernel + barrier before the GEMM",
                   "combine": "pull" if args.no_fused_combine else "pushed by the GEMM epilogue",
                   "last_weight_grad": "two launches, travelling grads first" if layer.split_last_wgrad else "one launch",
                   "cuda_graph": graphed,
                   "l2": "working set per step (>= 8 GB of weights, grads and activations) exceeds the 126 MB L2; no explicit flush"},
        "e2e": {"value": tokens / (ms_e2e / 1e3), "unit": "tokens/s", "ms_per_step": ms_e2e,
                "h2d_bytes_per_step": s * h * 2, "d2h_bytes_per_step": 4,
                "loss_last": losses[-1] if losses else None},
        "gpu_launches": launches,
        "ab_dispatch": ab,
        "comm_roundtrip_us": ms_comm * 1e3,
        "comm_roundtrip_what": "plan + dispatch + prefetch_weight + combine, zero-copy, max over ranks",
        "peak_mem_gb": peak_gb,
        "remote_stats": stats.get("remote_stats"), "dedup_ratio": stats.get("dedup_ratio"),
        "clocks": clocks,
    }
    if args.trace:
        from moonep_b200.utils.trace import Tracer
        layer.tracer = Tracer(enabled=True)
        for i in range(5):
            eager_step(xs[i % n_batches])
        spans = layer.tracer.summary()
        names = list(spans)
        t = torch.tensor([spans[n]["mean_ms"] for n in names], device=dev)
        tmin = t.clone()
        if R > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            dist.all_reduce(tmin, op=dist.ReduceOp.MIN)
        if buf.enable_phase_stamps():       # only with a library built with -DMEP_PHASE_STAMPS
            eager_step(xs[0])
            out["phase_stamps_us_rank0"] = buf.phase_stamps()
        out["trace_ms_max_over_ranks"] = {n: round(float(v), 3) for n, v in zip(names, t)}
        out["trace_ms_min_over_ranks"] = {n: round(float(v), 3) for n, v in zip(names, tmin)}
    if rank == 0:
        print(json.dumps(out), flush=True)
    buf.destroy()
    if R > 1:
        dist.destroy_process_group()


def main():
    args = parse()
    if args.impl == "reference":
        sys.path.insert(0, os.path.join(REPO, "baseline"))
        from reference_arm import run_reference
        run_reference(args)
        return
    run_ours(args)


if __name__ == "__main__":
    main()
