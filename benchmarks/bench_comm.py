"""Communication benchmark (run under torch.distributed.run, one process per GPU).

Times the expert-parallel communication ops at the DeepSeek-V3 shape (S=4096 tokens/rank, H=7168,
K=8, E=256, H'=2048, token_padding=128, num_sms=32) over a sweep of routing imbalance, for either
of two implementations behind the same op definitions:

  --impl ours        this repository's ``moonep_b200.Buffer``
  --impl reference   the unmodified reference ``moonep.Buffer`` installed under ``baseline/_ref``
                     (nothing of ``moonep_b200`` is imported in that arm)

Op definitions are the reference's (benchmarks/bench_vs_deepep.py:208-232):
  d_f  dispatch forward : inter-rank sync + planning + dispatch + duplicate expansion (zero copy)
                          followed by ``prefetch_weight``
  d_b  dispatch backward: dispatch with the saved plan followed by ``prefetch_weight``
  c_f  combine forward  : hidden rows only            c_b  combine backward: with route-weight gather
plus each part on its own (dispatch without the prefetch, ``prefetch_weight``, ``reduce_grad``), the
round trip d_f + c_f issued serially, and the same round trip with ``prefetch_weight(async_finish=
True)`` running on the communication stream next to the combine, as the reference's API intends
(moonep/api.py:880-884).  Timing: CUDA events on the launching stream after warm-up, eager issue,
MAX over ranks (the reference's own script reports the mean over ranks; both are printed).
Both arms get the same routing tensors (Zipf-skewed logits searched for the requested MaxVio,
fixed seeds).  Telemetry per row as in the reference's benchmarks/bench_comm.py:303-314:
max_recv / max_send (redundant experts received / sent by the worst rank), dedup_ratio,
dup_group_count, zero_pad_rows.  ``--sweep`` adds H in {3584, 7168} x K in {8, 16}
(bench_comm.py:464-492); ``--csv`` writes one line per row.

  python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 benchmarks/bench_comm.py
  python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 benchmarks/bench_comm.py --impl reference
"""
import argparse
import csv
import datetime
import json
import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


# ---- routing shared by both arms (plain torch) ---------------------------------------------------
def maxvio_of(topk_all, E):
    tot = torch.bincount(topk_all.reshape(-1).long(), minlength=E).float()
    return float(tot.max() / tot.mean() - 1.0)


def routing_for_maxvio(S, K, E, R, target, seed=7):
    """``(topk[R,S,K] int32, weights[R,S,K] fp32, achieved MaxVio)``: top-k of N(0,1) logits plus
    ``alpha * log Zipf popularity``, alpha bisected for the target; ``target <= 0`` is the
    balanced round-robin routing."""
    if target <= 0:
        s = torch.arange(S)[:, None]
        k = torch.arange(K)[None, :]
        tk = torch.stack([((s * K + k + r * 7) % E) for r in range(R)]).to(torch.int32)
        return tk.contiguous(), torch.full((R, S, K), 1.0 / K), maxvio_of(tk, E)
    order = torch.randperm(E, generator=torch.Generator().manual_seed(seed))
    logpop = torch.empty(E)
    logpop[order] = -torch.log(torch.arange(1, E + 1, dtype=torch.float32))
    base = torch.stack([torch.randn(S, E, generator=torch.Generator().manual_seed(seed * 1000003 + r + 1))
                        for r in range(R)])
    lo, hi, best = 0.0, 6.0, None
    for _ in range(24):
        mid = 0.5 * (lo + hi)
        val, idx = torch.topk(base + mid * logpop, K, dim=2)
        mv = maxvio_of(idx, E)
        if best is None or abs(mv - target) < abs(best[2] - target):
            best = (idx.to(torch.int32).contiguous(), torch.softmax(val, dim=2).contiguous(), mv)
        if abs(mv - target) <= 0.05 * max(target, 1.0):
            break
        lo, hi = (mid, hi) if mv < target else (lo, mid)
    return best


# ---- the two arms ---------------------------------------------------------------------------------
class OursArm:
    name = "ours"
    overlap_ok = True     # prefetch_weight / reduce_grad have their own barrier channel

    def __init__(self, S, H, Hp, K, E, R, rank, dev, num_sms, with_weights):
        sys.path.insert(0, ROOT)
        from moonep_b200.api import Buffer
        from moonep_b200.models.moe_layer import ExpertPools
        self.buf = Buffer(S, H, K, E, R, num_sms=num_sms, token_padding=128)
        self.rank, self.R, self.epn, self.NvS = rank, R, E // R, self.buf.NvS
        self.pools = ExpertPools(R, E // R, H, Hp, self.buf.group, rank) if (with_weights and R > 1) else None
        if self.pools is not None:
            g = torch.Generator(device=dev).manual_seed(rank)
            self.w_loc = [(torch.randn(E // R, H, Hp, device=dev, generator=g) * 0.02).bfloat16() for _ in range(3)]
            self.g_loc = [torch.zeros(E // R, H, Hp, device=dev) for _ in range(3)]

    def prepare(self, x, w, topk, tpe):
        self.x, self.w, self.topk, self.tpe = x, w, topk, tpe
        self.hid, self.wn, _, self.plan = self.buf.dispatch(x, w, topk, tpe, zero_copy=True,
                                                           router_weights_zero_copy=True)
        self.buf.check()

    def dispatch_fwd(self):
        self.hid, self.wn, _, self.plan = self.buf.dispatch(self.x, self.w, self.topk, self.tpe, zero_copy=True,
                                                           router_weights_zero_copy=True)

    def dispatch_bwd(self):
        self.buf.dispatch(self.x, plan=self.plan, zero_copy=True)

    def combine_fwd(self):
        self.buf.combine(self.plan, self.hid, None, zero_copy=True)

    def combine_bwd(self):
        self.buf.combine(self.plan, self.hid, self.wn, zero_copy=True, router_weights_zero_copy=True)

    def prefetch(self, async_finish=False):
        p, w = self.pools.prefetch, self.w_loc
        return self.buf.prefetch_weight(self.plan, async_finish, local_gate_weight=w[0], local_up_weight=w[1],
                                        local_down_weight=w[2], gate_prefetch_buffer=p["gate"],
                                        up_prefetch_buffer=p["up"], down_prefetch_buffer=p["down"])

    def reduce_grad(self):
        p, g = self.pools.reduce, self.g_loc
        self.buf.reduce_grad(self.plan, local_gate_grad=g[0], local_up_grad=g[1], local_down_grad=g[2],
                             gate_reduce_buffer=p["gate"], up_reduce_buffer=p["up"], down_reduce_buffer=p["down"])

    def plan_tables(self):
        return self.plan.experts_to_copy, self.plan.dst, self.plan.zero_fill_ranges, int(self.plan.dup_counts[0])

    def kernels(self, timed):
        """Per-kernel breakdown: the launchers that the API calls, timed one by one."""
        from moonep_b200 import _native as nat
        buf, plan, x = self.buf, self.plan, self.x
        st = lambda: torch.cuda.current_stream().cuda_stream
        out_sh = torch.empty_like(x)
        r = {}
        r["k_sync_us"] = timed(lambda: nat.call("mep_launch_sync", buf._ctx, st()))
        r["k_plan_us"] = timed(lambda: (nat.call(
            "mep_launch_plan", buf._ctx, self.topk.data_ptr(), self.tpe.data_ptr(), plan.dst.data_ptr(),
            plan.cu_seqlens.data_ptr(), plan.zero_fill_ranges.data_ptr(), plan.experts_to_copy.data_ptr(),
            plan.remote_stats.data_ptr(), plan.send_order.data_ptr(), st()),
            nat.call("mep_launch_sync", buf._ctx, st())))
        r["k_dispatch_us"] = timed(lambda: nat.call(
            "mep_launch_dispatch", buf._ctx, x.data_ptr(), 0, plan.dst.data_ptr(),
            plan.zero_fill_ranges.data_ptr(), 0, 0, 1, 0, 0, st()))
        r["k_expand_us"] = timed(lambda: nat.call(
            "mep_launch_expand", buf._ctx, plan.link.data_ptr(), plan.cu_seqlens.data_ptr(), 0, st()))
        r["k_prologue_us"] = timed(lambda: nat.call(
            "mep_launch_combine_prologue", buf._ctx, plan.link.data_ptr(), plan.cu_seqlens.data_ptr(), st()))
        r["k_combine_us"] = timed(lambda: nat.call(
            "mep_launch_combine", buf._ctx, plan.dst.data_ptr(), out_sh.data_ptr(), 0, st()))
        if self.R > 1:
            # the conventional exchange at the same shape: all_to_all_single over NCCL + permute
            from moonep_b200.parallel.nccl_baseline import NcclAllToAllEP
            nccl = NcclAllToAllEP(buf.S, buf.H, buf.K, buf.E)

            def nccl_rt():
                rows, _, s2 = nccl.dispatch(x, self.topk)
                nccl.combine(rows, s2)

            try:
                r["nccl_a2a_roundtrip_us"] = timed(nccl_rt)
            except RuntimeError as exc:               # e.g. out of memory under heavy skew
                r["nccl_a2a_roundtrip_us"] = None
                r["nccl_error"] = str(exc)[:120]
        return r

    def check(self):
        self.buf.check()

    def destroy(self):
        self.buf.destroy()


class ReferenceArm:
    name = "reference"
    # The reference's ops share one set of barrier words, so an asynchronous prefetch_weight may
    # only overlap COMPUTE on the main stream: issued next to a combine on the main stream it
    # stopped answering on this box (both kernels wait in the same cross-rank barrier).  The
    # overlapped round trip is therefore not measured for this arm.
    overlap_ok = False
    overlap_note = "not run: the reference's async prefetch_weight next to a main-stream combine hangs (shared barrier words)"

    def __init__(self, S, H, Hp, K, E, R, rank, dev, num_sms, with_weights):
        ref_dir = os.path.join(ROOT, "baseline", "_ref")
        if not os.path.isdir(os.path.join(ref_dir, "moonep")):
            raise RuntimeError("baseline/_ref/moonep is missing (offline install of the reference not present)")
        sys.path.insert(0, ref_dir)
        from moonep import Buffer
        from moonep.buffer import create_nvl_dist_tensor, pad_dim0_for_alignment
        self.buf = Buffer(S, H, K, E, R, num_sms=num_sms, token_padding=128)
        self.rank, self.R, self.epn = rank, R, E // R
        epn = E // R
        self.NvS = (S * K + 127 * 2 * epn + 127) // 128 * 128
        self.pools = None
        if with_weights and R > 1:
            g = torch.Generator(device=dev).manual_seed(rank)
            self.w_loc = [(torch.randn(epn, H, Hp, device=dev, generator=g) * 0.02).bfloat16() for _ in range(3)]
            self.g_loc = [torch.zeros(epn, H, Hp, device=dev) for _ in range(3)]
            self.pools, self.rpools = [], []
            for dt, dstl in ((torch.bfloat16, self.pools), (torch.float32, self.rpools)):
                rows = pad_dim0_for_alignment([epn, H, Hp], dt)
                for _ in range(3):
                    t = create_nvl_dist_tensor([rows, H, Hp], dt, rank, R).view(R, rows, H, Hp)[:, :epn]
                    if dt == torch.float32:
                        t[rank].zero_()
                    dstl.append(t)
            torch.cuda.synchronize()
            dist.barrier()

    def prepare(self, x, w, topk, tpe):
        self.x, self.w, self.topk, self.tpe = x, w, topk, tpe
        self.hid, self.wn, _, self.plan = self.buf.dispatch(x, w, topk, tpe, zero_copy=True,
                                                           router_weights_zero_copy=True)
        torch.cuda.synchronize()
        dist.barrier()

    def dispatch_fwd(self):
        self.hid, self.wn, _, self.plan = self.buf.dispatch(self.x, self.w, self.topk, self.tpe, zero_copy=True,
                                                           router_weights_zero_copy=True)

    def dispatch_bwd(self):
        self.buf.dispatch(self.x, plan=self.plan, zero_copy=True)

    def combine_fwd(self):
        self.buf.combine(plan=self.plan, hidden_nvsh=self.hid, zero_copy=True)

    def combine_bwd(self):
        self.buf.combine(plan=self.plan, hidden_nvsh=self.hid, route_weights_nvs=self.wn, zero_copy=True,
                         router_weights_zero_copy=True)

    def prefetch(self, async_finish=False):
        p, w = self.pools, self.w_loc
        return self.buf.prefetch_weight(plan=self.plan, async_finish=async_finish, local_gate_weight=w[0],
                                        local_up_weight=w[1], local_down_weight=w[2], gate_prefetch_buffer=p[0],
                                        up_prefetch_buffer=p[1], down_prefetch_buffer=p[2])

    def reduce_grad(self):
        p, g = self.rpools, self.g_loc
        self.buf.reduce_grad(plan=self.plan, local_gate_grad=g[0], local_up_grad=g[1], local_down_grad=g[2],
                             gate_reduce_buffer=p[0], up_reduce_buffer=p[1], down_reduce_buffer=p[2])

    def plan_tables(self):
        return self.plan.experts_to_copy, self.plan.dst, self.plan.zero_fill_ranges, int(self.plan.dup_counts[0])

    def kernels(self, timed):
        return {}

    def check(self):
        torch.cuda.synchronize()

    def destroy(self):
        self.buf.destroy()


def run_shape(args, arm_cls, S, H, Hp, K, E, R, rank, dev, rows_out):
    arm = arm_cls(S, H, Hp, K, E, R, rank, dev, args.num_sms, not args.no_weights)
    x = torch.randn(S, H, device=dev, generator=torch.Generator(device=dev).manual_seed(rank)).bfloat16()

    def timed(fn):
        for _ in range(args.warmup):
            fn()
        torch.cuda.synchronize()
        dist.barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(args.iters):
            fn()
        b.record()
        torch.cuda.synchronize()
        t = torch.tensor([a.elapsed_time(b) / args.iters * 1e3], device=dev, dtype=torch.float64)
        tm = t.clone()
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dist.all_reduce(tm)
        timed.mean = round(float(tm) / R, 1)
        if rank == 0:      # progress line: a later failure must not lose what was measured
            print(f"[{arm.name}] op {timed.n}: {float(t):.1f} us", file=sys.stderr, flush=True)
        timed.n += 1
        return round(float(t), 1)

    timed.n = 0

    for target in [float(v) for v in args.maxvio.split(",")]:
        topk_all, w_all, mv = routing_for_maxvio(S, K, E, R, target)
        topk, w = topk_all[rank].to(dev).contiguous(), w_all[rank].to(dev).contiguous()
        tpe = torch.bincount(topk_all[rank].reshape(-1).long(), minlength=E).to(torch.int32).to(dev)
        arm.prepare(x, w, topk, tpe)
        row = {"impl": arm.name, "R": R, "S": S, "H": H, "K": K, "E": E, "Hp": Hp, "num_sms": args.num_sms,
               "maxvio_target": target, "maxvio": round(mv, 3)}
        row["dispatch_fwd_us"] = timed(arm.dispatch_fwd)
        row["dispatch_bwd_us"] = timed(arm.dispatch_bwd)
        row["combine_fwd_us"] = timed(arm.combine_fwd)
        row["c_f_mean_us"] = timed.mean
        row["combine_bwd_us"] = timed(arm.combine_bwd)
        if arm.pools is not None:
            row["prefetch_us"] = timed(arm.prefetch)
            row["reduce_grad_us"] = timed(arm.reduce_grad)
            row["d_f_us"] = timed(lambda: (arm.dispatch_fwd(), arm.prefetch()))
            row["d_f_mean_us"] = timed.mean
            row["d_b_us"] = timed(lambda: (arm.dispatch_bwd(), arm.prefetch()))
            row["roundtrip_serial_us"] = timed(lambda: (arm.dispatch_fwd(), arm.prefetch(), arm.combine_fwd()))

            def overlapped():
                arm.dispatch_fwd()
                ev = arm.prefetch(async_finish=True)
                arm.combine_fwd()
                torch.cuda.current_stream().wait_event(ev)

            if arm.overlap_ok:
                row["roundtrip_overlapped_us"] = timed(overlapped)
            else:
                row["roundtrip_overlapped_us"] = None
                row["roundtrip_overlapped_note"] = arm.overlap_note
        else:
            row["roundtrip_serial_us"] = timed(lambda: (arm.dispatch_fwd(), arm.combine_fwd()))
        row.update(arm.kernels(timed))
        # ---- telemetry (reference: benchmarks/bench_comm.py:303-314) ---------------------------
        etc, dstv, zf, dup_groups = arm.plan_tables()
        etc_cpu = etc.cpu()
        valid = etc_cpu >= 0
        row["max_recv"] = int(valid.sum(dim=1).max())
        row["max_send"] = int(torch.bincount((etc_cpu[valid] // (E // R)).long(), minlength=R).max()) if bool(valid.any()) else 0
        row["remote_experts_total"] = int(valid.sum())
        sent = (dstv >= 0) & (torch.div(dstv, arm.NvS, rounding_mode="floor") != rank)
        agg = torch.tensor([int(sent.sum()), int((dstv >= 0).sum()), int(zf.reshape(-1, 2)[:, 1].sum()), dup_groups],
                           device=dev, dtype=torch.float64)
        mx = agg.clone()
        dist.all_reduce(agg)
        dist.all_reduce(mx, op=dist.ReduceOp.MAX)
        row["dedup_ratio"] = round(float(agg[1]) / (R * S * K), 4)
        row["nvlink_rows_sent_max"] = int(mx[0])
        row["zero_pad_rows_max"] = int(mx[2])
        row["dup_group_count_max"] = int(mx[3])
        row["dispatch_nvlink_gbs"] = round(float(mx[0]) * H * 2 / (row["dispatch_bwd_us"] * 1e-6) / 1e9, 1)
        row["combine_nvlink_gbs"] = round(float(mx[0]) * H * 2 / (row["combine_fwd_us"] * 1e-6) / 1e9, 1)
        arm.check()
        rows_out.append(row)
        if rank == 0:
            print(json.dumps(row), flush=True)
    arm.destroy()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--S", type=int, default=4096)
    ap.add_argument("--H", type=int, default=7168)
    ap.add_argument("--Hp", type=int, default=2048)
    ap.add_argument("--K", type=int, default=8)
    ap.add_argument("--E", type=int, default=256)
    ap.add_argument("--num-sms", type=int, default=32)
    ap.add_argument("--maxvio", default="0,0.5,1,2,4,8")
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--sweep", action="store_true", help="H in {3584, 7168} x K in {8, 16} instead of one shape")
    ap.add_argument("--no-weights", action="store_true", help="skip prefetch / reduce_grad pools")
    ap.add_argument("--nccl-timeout", type=int, default=120, help="seconds before a stuck collective ends the run")
    ap.add_argument("--out", default="", help="write all rows as JSON")
    ap.add_argument("--csv", default="", help="write all rows as CSV")
    args = ap.parse_args()
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    # a short collective timeout: a hang in either arm ends the run in minutes, not in ten
    dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(seconds=args.nccl_timeout))
    R, rank = dist.get_world_size(), dist.get_rank()
    arm_cls = OursArm if args.impl == "ours" else ReferenceArm
    shapes = [(h, k) for h in (3584, 7168) for k in (8, 16)] if args.sweep else [(args.H, args.K)]
    rows = []
    for h, k in shapes:
        try:
            run_shape(args, arm_cls, args.S, h, args.Hp, k, args.E, R, rank, dev, rows)
        except Exception as exc:  # noqa: BLE001 - one failed shape must not wedge the others
            if rank == 0:
                print(json.dumps({"impl": args.impl, "H": h, "K": k, "error": f"{type(exc).__name__}: {exc}"[:300]}),
                      flush=True)
            torch.cuda.synchronize()
            dist.barrier()
    if rank == 0 and args.out:
        with open(args.out, "w") as fh:
            json.dump(rows, fh, indent=1)
    if rank == 0 and args.csv and rows:
        keys = sorted({k for r in rows for k in r})
        with open(args.csv, "w", newline="") as fh:
            wr = csv.DictWriter(fh, fieldnames=keys)
            wr.writeheader()
            wr.writerows(rows)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
