"""Reference arm of bench.py.

Runs the UNMODIFIED reference (``moonep``, installed under ``baseline/_ref``) through its own
public API -- ``moonep.Buffer.dispatch / prefetch_weight / combine / reduce_grad`` and
``moonep.buffer.create_nvl_dist_tensor`` -- for the same metric and configuration as the main
arm: one MoE-layer training step (forward + backward + SGD) at S=4096, H=7168, H'=2048, K=8,
E=256, EP = number of GPUs.  The reference is a communication library and leaves the expert
math to the host framework (README.md:43-68), so that part is plain PyTorch here:
``torch._grouped_mm`` over the ``[2*epn, H, H']`` compute view that the README describes (local
experts followed by this rank's prefetch slots, one contiguous tensor per projection), eager
elementwise ops for SwiGLU and the router.  Nothing from ``moonep_b200`` is imported.
"""
from __future__ import annotations

import json
import os
import sys
import time

HERE = os.path.dirname(os.path.abspath(__file__))
S, H, HP, K, E = 4096, 7168, 2048, 8, 256


def _unavailable(why: str):
    print(json.dumps({"impl": "reference", "unavailable": why.replace("\n", " ")[:300]}), flush=True)


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if int(os.environ.get("WORLD_SIZE", "1")) == 1 and os.environ.get("MOONEP_REF_CHILD") != "1":
        # One GPU: the reference's native layer ends the process with exit() on a driver error
        # (csrc/nvl_shared_buffer.cuh:17-39) and it asserts NVLS multicast support even for a
        # single rank, so it runs in a child process whose failure becomes the `unavailable` line.
        import subprocess
        env = dict(os.environ, MOONEP_REF_CHILD="1")
        cmd = [sys.executable, os.path.join(os.path.dirname(HERE), "bench.py"), "--impl", "reference",
               "--gpus", "1", "--steps", str(args.steps), "--warmup", str(args.warmup),
               "--maxvio", str(args.maxvio), "--lr", str(args.lr)]
        try:
            res = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=1500)
        except subprocess.TimeoutExpired:
            _unavailable("reference run at 1 GPU did not finish within 1500 s")
            return
        lines = [l for l in res.stdout.splitlines() if l.startswith("{")]
        if res.returncode == 0 and lines:
            print(lines[-1], flush=True)
        else:
            tail = (res.stderr or res.stdout).strip().splitlines()[-1:] or ["no output"]
            _unavailable(f"reference process exited with code {res.returncode} at 1 GPU: {tail[0]}")
        return
    try:
        _run(args)
    except Exception as exc:  # noqa: BLE001 - any failure of the reference is reported, not raised
        if rank == 0:
            _unavailable(f"{type(exc).__name__}: {exc}")
        try:
            import torch.distributed as dist
            if dist.is_initialized():
                dist.destroy_process_group()
        except Exception:  # noqa: BLE001
            pass


def _run(args):
    ref_dir = os.path.join(HERE, "_ref")
    if not os.path.isdir(os.path.join(ref_dir, "moonep")):
        raise RuntimeError("baseline/_ref/moonep is missing (offline install of the reference not present)")
    sys.path.insert(0, ref_dir)
    import torch
    import torch.distributed as dist
    import torch.nn.functional as F

    R = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    assert R == args.gpus
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if not dist.is_initialized():
        if R == 1:
            os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
            os.environ.setdefault("MASTER_PORT", "29577")
            dist.init_process_group("nccl", rank=0, world_size=1, device_id=dev)
        else:
            dist.init_process_group("nccl", device_id=dev)

    from moonep import Buffer
    from moonep.buffer import create_nvl_dist_tensor, pad_dim0_for_alignment

    epn = E // R
    buf = Buffer(S, H, K, E, R, num_sms=32, token_padding=128)

    # [2*epn, H, H'] per rank: rows [0, epn) are the local parameters (or local fp32 grads), rows
    # [epn, 2*epn) this rank's prefetch (or reduce) slots; the communication view is [:, epn:].
    # A lone rank can never receive a redundant expert, so it carries no slots at all.
    nslot = 0 if R == 1 else epn

    def pool(dtype):
        rows = pad_dim0_for_alignment([epn + nslot, H, HP], dtype)
        t = create_nvl_dist_tensor([rows, H, HP], dtype, rank, R).view(R, rows, H, HP)
        return t[rank, : epn + nslot], t[:, epn: epn + nslot]

    g = torch.Generator(device=dev).manual_seed(101 + rank)
    W, Wcomm, G, Gcomm = {}, {}, {}, {}
    for n in ("gate", "up", "down"):
        W[n], Wcomm[n] = pool(torch.bfloat16)
        W[n][:epn].copy_((torch.randn(epn, H, HP, device=dev, generator=g) * 0.02).bfloat16())
        G[n], Gcomm[n] = pool(torch.float32)
        G[n].zero_()
    w_router = (torch.randn(H, E, device=dev, generator=torch.Generator(device=dev).manual_seed(13)) * 0.02).bfloat16()
    g_router = torch.zeros(H, E, device=dev)
    torch.cuda.synchronize()
    dist.barrier()

    host = [torch.randn(S, H, generator=torch.Generator().manual_seed(1000 * rank + i)).bfloat16().pin_memory()
            for i in range(4)]
    xs = [t.to(dev) for t in host]

    # Zipf router bias, exponent searched for the target MaxVio (same procedure as the main arm)
    order = torch.randperm(E, generator=torch.Generator().manual_seed(1234))
    ranks_ = torch.empty(E)
    ranks_[order] = torch.arange(1, E + 1, dtype=torch.float32)
    logpop = -torch.log(ranks_).to(dev)
    bias, mv = None, 0.0
    if args.maxvio > 0:
        logits = (xs[0] @ w_router).float()
        lo, hi, best = 0.0, 8.0, (None, 1e9)
        for _ in range(20):
            mid = 0.5 * (lo + hi)
            b = mid * logpop
            idx = (logits + b).topk(K, dim=1).indices
            tot = torch.bincount(idx.flatten(), minlength=E).float()
            dist.all_reduce(tot)
            m = float(tot.max() / tot.mean() - 1)
            if abs(m - args.maxvio) < abs(best[1] - args.maxvio):
                best = (b, m)
            lo, hi = (mid, hi) if m < args.maxvio else (lo, mid)
        bias, mv = best

    def gmm(a, b, offs, out_dtype=None):
        return torch._grouped_mm(a, b, offs=offs, out_dtype=out_dtype)

    def step(x):
        # ---- forward ----
        logits = (x @ w_router).float()
        sel = logits if bias is None else logits + bias
        topk = sel.topk(K, dim=1).indices
        wsk = torch.softmax(logits.gather(1, topk), dim=1)
        topk32 = topk.to(torch.int32)
        tpe = torch.bincount(topk32.flatten(), minlength=E).to(torch.int32)
        hidden, w_nvs, cu, plan = buf.dispatch(x, wsk, topk32, tpe)
        cu = cu[: epn + nslot]
        if nslot:
            buf.prefetch_weight(plan=plan, local_gate_weight=W["gate"][:epn], local_up_weight=W["up"][:epn],
                                local_down_weight=W["down"][:epn], gate_prefetch_buffer=Wcomm["gate"],
                                up_prefetch_buffer=Wcomm["up"], down_prefetch_buffer=Wcomm["down"])
        gate = gmm(hidden, W["gate"], cu)
        up = gmm(hidden, W["up"], cu)
        act = F.silu(gate.float()).mul_(up.float()).mul_(w_nvs[:, None]).bfloat16()
        y_nvsh = gmm(act, W["down"].transpose(1, 2), cu)
        y, _, _ = buf.combine(plan=plan, hidden_nvsh=y_nvsh)
        loss = y.float().pow(2).mean()
        # ---- backward ----
        dy = (y.float() * (2.0 / y.numel())).bfloat16()
        d_out, _, _, _ = buf.dispatch(dy, plan=plan)
        d_act = gmm(d_out, W["down"], cu)
        G["down"].copy_(gmm(d_out.t(), act, cu, out_dtype=torch.float32) if _F32_OUT[0]
                        else gmm(d_out.t(), act, cu).float())
        gf, uf, da = gate.float(), up.float(), d_act.float()
        sig = torch.sigmoid(gf)
        silu = gf * sig
        d_scale = (da * silu * uf).sum(dim=1)
        d_gate = (da * uf * w_nvs[:, None] * (sig * (1 + gf * (1 - sig)))).bfloat16()
        d_up = (da * silu * w_nvs[:, None]).bfloat16()
        for n, d in (("gate", d_gate), ("up", d_up)):
            G[n].copy_(gmm(hidden.t(), d, cu, out_dtype=torch.float32) if _F32_OUT[0]
                       else gmm(hidden.t(), d, cu).float())
        d_hidden = gmm(d_gate, W["gate"].transpose(1, 2), cu) + gmm(d_up, W["up"].transpose(1, 2), cu)
        dx, dw_sk, _ = buf.combine(plan=plan, hidden_nvsh=d_hidden, route_weights_nvs=d_scale)
        if nslot:
            buf.reduce_grad(plan=plan, local_gate_grad=G["gate"][:epn], local_up_grad=G["up"][:epn],
                            local_down_grad=G["down"][:epn], gate_reduce_buffer=Gcomm["gate"],
                            up_reduce_buffer=Gcomm["up"], down_reduce_buffer=Gcomm["down"])
        dot = (wsk * dw_sk).sum(dim=1, keepdim=True)
        d_logits = torch.zeros(S, E, device=dev).scatter_(1, topk, wsk * (dw_sk - dot)).bfloat16()
        g_router.copy_((x.t() @ d_logits).float())
        dx = dx + d_logits @ w_router.t()
        # ---- SGD ----
        for n in ("gate", "up", "down"):
            W[n][:epn].add_(G[n][:epn].bfloat16(), alpha=-args.lr)
        w_router.add_(g_router.bfloat16(), alpha=-args.lr)
        return loss

    # does this torch build give fp32 outputs from bf16 grouped GEMMs?
    _F32_OUT = [True]
    try:
        offs = torch.tensor([64], dtype=torch.int32, device=dev)
        gmm(torch.zeros(64, 64, device=dev, dtype=torch.bfloat16).t(),
            torch.zeros(64, 64, device=dev, dtype=torch.bfloat16), offs, out_dtype=torch.float32)
    except Exception:  # noqa: BLE001
        _F32_OUT[0] = False

    def barrier():
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
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms) / steps

    for i in range(max(args.warmup, 3)):
        step(xs[i % 4])
    ms_step = timed(lambda i: step(xs[i % 4]), args.steps)
    # end to end, with the same two-deep pipeline as the main arm: batch i+1 is uploaded from
    # pinned memory on a copy stream while step i computes, and the host reads the loss of step
    # i-1 (copied to pinned memory behind that step); the last loss is read before the timer stops
    copy_stream = torch.cuda.Stream(device=dev)
    stage = [torch.empty(S, H, dtype=torch.bfloat16, device=dev) for _ in range(2)]
    ready = [torch.cuda.Event(), torch.cuda.Event()]
    consumed = [torch.cuda.Event(), torch.cuda.Event()]
    loss_host = [torch.empty((), dtype=torch.float32).pin_memory() for _ in range(2)]
    loss_ready = [torch.cuda.Event(), torch.cuda.Event()]
    losses = []

    def upload(i):
        slot = i % 2
        with torch.cuda.stream(copy_stream):
            copy_stream.wait_event(consumed[slot])
            stage[slot].copy_(host[i % 4], non_blocking=True)
            ready[slot].record(copy_stream)

    def prime():                # both slots free, batch 0 on its way, nothing read yet
        torch.cuda.synchronize()
        for ev in consumed:
            ev.record()
        upload(0)
        losses.clear()

    def e2e(i, n_steps=None):
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
        e2e(i, 3)
    prime()

    ms_e2e = timed(e2e, args.steps)
    # ---- communication round trip at the same shape, as the main arm times it: plan + dispatch +
    # prefetch_weight + combine, zero copy, issued serially ------------------------------------
    rt = {}

    def comm_round(i):
        if not rt:
            logits = (xs[0] @ w_router).float()
            sel = logits if bias is None else logits + bias
            topk = sel.topk(K, dim=1).indices
            rt["w"] = torch.softmax(logits.gather(1, topk), dim=1).contiguous()
            rt["topk"] = topk.to(torch.int32).contiguous()
            rt["tpe"] = torch.bincount(rt["topk"].flatten(), minlength=E).to(torch.int32)
        hid, wn, cu, plan = buf.dispatch(xs[0], rt["w"], rt["topk"], rt["tpe"], zero_copy=True,
                                         router_weights_zero_copy=True)
        if nslot:
            buf.prefetch_weight(plan=plan, local_gate_weight=W["gate"][:epn], local_up_weight=W["up"][:epn],
                                local_down_weight=W["down"][:epn], gate_prefetch_buffer=Wcomm["gate"],
                                up_prefetch_buffer=Wcomm["up"], down_prefetch_buffer=Wcomm["down"])
        buf.combine(plan=plan, hidden_nvsh=hid, zero_copy=True)

    for i in range(3):
        comm_round(i)
    ms_comm = timed(comm_round, max(args.steps, 10))
    tokens = R * S
    out = {
        "metric": "moe_layer_train_tokens_per_s", "value": tokens / (ms_step / 1e3), "unit": "tokens/s",
        "n_gpus": R, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_step,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic (N(0,1) tokens, random-init weights, Zipf router bias)",
        "impl": "reference",
        "config": {"model": "deepseek-v3-style MoE layer: router 7168->256 top-8 softmax, 256 SwiGLU experts H=7168 H'=2048",
                   "global_batch": tokens, "seq_len": S, "parallelism": f"ep{R}",
                   "comm": "moonep.Buffer (unmodified reference)", "expert_math": "torch._grouped_mm + eager elementwise",
                   "wgrad_fp32_out": _F32_OUT[0], "maxvio_target": args.maxvio, "maxvio_achieved": mv},
        "e2e": {"value": tokens / (ms_e2e / 1e3), "unit": "tokens/s", "ms_per_step": ms_e2e,
                "h2d_bytes_per_step": S * H * 2, "d2h_bytes_per_step": 4,
                "loss_last": losses[-1] if losses else None},
        "comm_roundtrip_us": ms_comm * 1e3,
        "comm_roundtrip_what": "plan + dispatch + prefetch_weight + combine, zero-copy, max over ranks",
        "peak_mem_gb": torch.cuda.max_memory_allocated(dev) / 2 ** 30,
    }
    if rank == 0:
        print(json.dumps(out), flush=True)
    buf.destroy()
    time.sleep(0.1)
    dist.destroy_process_group()
