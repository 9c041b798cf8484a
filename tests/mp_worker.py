"""Worker for the multi-GPU tests: run under ``python -m torch.distributed.run`` with one process
per GPU.  Checks the real peer-memory paths (VMM handle exchange, NVLink stores / loads, flag
barriers) against the CPU simulator, then the MoE layer against a dense fp32 reference."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from moonep_b200 import reference as ref  # noqa: E402
from moonep_b200.api import Buffer  # noqa: E402
from moonep_b200.utils.routing import routing_for_maxvio, tokens_per_expert  # noqa: E402


def all_ok(ok: bool, what: str, detail=""):
    """Collective assert: every rank learns about a failure, so nobody hangs in a later op."""
    t = torch.tensor([int(ok)], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MIN)
    if int(t) != 1:
        raise AssertionError(f"{what} failed on rank {dist.get_rank()}: {detail}" if not ok
                             else f"{what} failed on another rank")


def comm_checks(R, rank):
    S, H, K, tp = 256, 512, 4, 32
    E = 8 * R
    topk, w, mv, _ = routing_for_maxvio(S, K, E, R, 2.0, seed=11)
    tpe = torch.stack([tokens_per_expert(topk[r], E) for r in range(R)])
    x = torch.randn(R, S, H, generator=torch.Generator().manual_seed(5)).bfloat16()
    sim = ref.SimGroup(S, H, K, E, R, tp)
    h_ref, w_ref, cu_ref, plans_ref = sim.dispatch(x, w, topk)
    buf = Buffer(S, H, K, E, R, num_sms=8, token_padding=tp, timeout_s=10.0)
    xd, wd, td, pd = x[rank].cuda(), w[rank].cuda(), topk[rank].cuda(), tpe[rank].cuda()
    hidden, w_nvs, cu, plan = buf.dispatch(xd, wd, td, pd)
    buf.check()
    rows = int(cu_ref[rank, -1])
    pr = plans_ref[rank]
    all_ok(torch.equal(plan.dst.cpu(), pr.dst), "plan.dst")
    all_ok(torch.equal(cu.cpu(), cu_ref[rank]), "cu_seqlens")
    all_ok(torch.equal(plan.experts_to_copy.cpu(), pr.experts_to_copy), "experts_to_copy")
    all_ok(torch.equal(plan.zero_fill_ranges.cpu(), pr.zero_fill_ranges), "zero_fill")
    all_ok(torch.equal(plan.remote_stats.cpu(), pr.remote_stats), "remote_stats")
    all_ok(torch.equal(hidden.cpu()[:rows], h_ref[rank, :rows]), "dispatched rows")
    all_ok(torch.equal(w_nvs.cpu()[:rows], w_ref[rank, :rows]), "dispatched weights")
    all_ok(torch.equal(plan.link.cpu()[:rows], pr.link[:rows]), "chain links")
    y = (hidden.float() * w_nvs[:, None]).bfloat16()
    out, w_back, _ = buf.combine(plan, y, w_nvs)
    buf.check()
    y_ref = (h_ref.float() * w_ref[:, :, None]).bfloat16()
    out_ref, wb_ref = sim.combine(plans_ref, y_ref, w_ref)
    all_ok(torch.equal(out.cpu().view(torch.int16), out_ref[rank].view(torch.int16)), "combine")
    all_ok(torch.equal(w_back.cpu(), w[rank]), "weight gather")
    # async + plan reuse + zero copy
    h2, _, cu2, plan2, ev = buf.dispatch(xd, None, plan=plan, async_finish=True, zero_copy=True)
    ev.wait()
    all_ok(cu2 is None and plan2 is plan, "plan reuse contract")
    out2, _, ev2 = buf.combine(plan, h2, None, async_finish=True, zero_copy=True)
    ev2.wait()
    torch.cuda.synchronize()
    ident = (x[rank].float() * K).bfloat16()
    err = float((out2.cpu().float() - ident.float()).abs().max())
    all_ok(err <= 2 * 2 ** -7 * float(ident.float().abs().max()), "identity round trip", err)
    # ---- prefetch + reduce_grad with the real plan -------------------------------------------
    from moonep_b200.models.moe_layer import ExpertPools
    epn, Hh, Hp = E // R, 128, 256
    pools = ExpertPools(R, epn, Hh, Hp, buf.group, rank)
    g = torch.Generator(device="cuda").manual_seed(100 + rank)
    loc = {n: torch.randn(epn, Hh, Hp, device="cuda", generator=g).bfloat16() for n in pools.names}
    for n in pools.names:
        pools.prefetch[n][rank].fill_(-3.0)
    torch.cuda.synchronize(); dist.barrier()
    buf.prefetch_weight(plan, local_gate_weight=loc["gate"], local_up_weight=loc["up"],
                        local_down_weight=loc["down"], gate_prefetch_buffer=pools.prefetch["gate"],
                        up_prefetch_buffer=pools.prefetch["up"], down_prefetch_buffer=pools.prefetch["down"])
    buf.check()
    etc = pr.experts_to_copy
    allw = {}
    for n in pools.names:
        lst = [torch.empty_like(loc[n]) for _ in range(R)]
        dist.all_gather(lst, loc[n])
        allw[n] = torch.cat(lst)                                  # [E, Hh, Hp]
    ok = True
    for n in pools.names:
        for b in range(epn):
            e = int(etc[rank, b])
            got = pools.prefetch[n][rank, b]
            ok &= torch.equal(got, allw[n][e]) if e >= 0 else bool((got == -3.0).all())
    all_ok(ok, "prefetch_weight")
    lg = {n: torch.randn(epn, Hh, Hp, device="cuda", generator=g) for n in pools.names}
    lg0 = {n: v.clone() for n, v in lg.items()}
    for n in pools.names:
        pools.reduce[n][rank].copy_(torch.randn(epn, Hh, Hp, device="cuda", generator=g))
    torch.cuda.synchronize(); dist.barrier()
    snap = {n: pools.reduce[n].clone() for n in pools.names}     # all ranks' slots, read over NVLink
    torch.cuda.synchronize(); dist.barrier()
    buf.reduce_grad(plan, local_gate_grad=lg["gate"], local_up_grad=lg["up"], local_down_grad=lg["down"],
                    gate_reduce_buffer=pools.reduce["gate"], up_reduce_buffer=pools.reduce["up"],
                    down_reduce_buffer=pools.reduce["down"])
    buf.check()
    ok = True
    for n in pools.names:
        want = lg0[n].clone()
        for d in range(R):
            for b in range(epn):
                e = int(etc[d, b])
                if e >= 0 and e // epn == rank:
                    want[e % epn] += snap[n][d, b]
        ok &= torch.equal(lg[n], want)
        for b in range(epn):
            if int(etc[rank, b]) >= 0:
                ok &= bool((pools.reduce[n][rank, b] == 0).all())
            else:
                ok &= torch.equal(pools.reduce[n][rank, b], snap[n][rank, b])
    all_ok(ok, "reduce_grad (bitwise)")
    st = buf.stats()
    all_ok(st["dispatch"] == 2 and st["combine"] == 2, "stats")
    buf.destroy()


def layer_check(R, rank):
    from moonep_b200.models.moe_layer import ExpertPools, MoELayer
    from moonep_b200.ops import gemm
    from tests.test_moe_layer import reference_layer
    S, H, Hp, K = 256, 256, 128, 4
    E = 4 * R
    buf = Buffer(S, H, K, E, R, num_sms=8, token_padding=64, timeout_s=10.0)
    pools = ExpertPools(R, E // R, H, Hp, buf.group, rank)
    # a strong bias towards the experts of rank 0 forces redundant experts and prefetch slots
    bias = torch.zeros(E, device="cuda")
    bias[: E // R] = 1.5
    layer = MoELayer(buf, Hp, pools, seed=5, init_std=0.06, router_bias=bias)
    g = torch.Generator(device="cuda").manual_seed(50 + rank)
    x = torch.randn(S, H, device="cuda", generator=g).bfloat16()
    dy = torch.randn(S, H, device="cuda", generator=g).bfloat16()
    xo = x.clone().requires_grad_(True)
    y = layer(xo)
    y.backward(dy)
    buf.check()
    gemm.check_status()
    used = int((layer.last_plan.experts_to_copy >= 0).sum())
    gather = lambda t: torch.cat([u for u in _all_gather(t, R)])
    wg, wu, wd = gather(layer.w_gate), gather(layer.w_up), gather(layer.w_down)
    xs, dys = _all_gather(x, R), _all_gather(dy, R)
    wr = layer.w_router.float().clone().requires_grad_(True)
    wgf, wuf, wdf = [t.float().clone().requires_grad_(True) for t in (wg, wu, wd)]
    mine = None
    for r in range(R):                     # global reference: every rank's tokens through all experts
        xr = xs[r].float().requires_grad_(True)
        yr, _ = reference_layer(xr, wr, wgf, wuf, wdf, K, bias)
        yr.backward(dys[r].float())
        if r == rank:
            mine = (yr.detach(), xr.grad)
    epn = E // R

    def rel(a, b):
        return float((a.float() - b).abs().max()) / (float(b.abs().max()) + 1e-9)

    errs = dict(y=rel(y, mine[0]), dx=rel(xo.grad, mine[1]),
                gate=rel(layer.g_gate, wgf.grad[rank * epn:(rank + 1) * epn]),
                up=rel(layer.g_up, wuf.grad[rank * epn:(rank + 1) * epn]),
                down=rel(layer.g_down, wdf.grad[rank * epn:(rank + 1) * epn]))
    all_ok(max(errs.values()) < 6e-2, "MoE layer vs dense reference", str(errs))
    tot = torch.tensor([used], device="cuda")
    dist.all_reduce(tot)
    all_ok(int(tot) > 0, "skewed routing must create redundant experts", f"slots used {int(tot)}")
    # SGD fused into the weight-grad epilogues gives bit-identical weights, also for the experts
    # whose replicas' grads come home through reduce_grad
    names = ("w_router", "w_gate", "w_up", "w_down")
    w0 = {n: getattr(layer, n).clone() for n in names}
    layer.sgd_step(0.25)
    torch.cuda.synchronize()
    want = {n: getattr(layer, n).clone() for n in names}
    for n in names:
        getattr(layer, n).copy_(w0[n])
    layer.fuse_sgd(0.25)
    xo2 = x.clone().requires_grad_(True)
    y2 = layer(xo2)
    y2.backward(dy)
    layer.sgd_step(0.25)
    buf.check()
    gemm.check_status()
    same = all(torch.equal(getattr(layer, n), want[n]) for n in names)
    same = same and torch.equal(y2, y) and torch.equal(xo2.grad, xo.grad)
    kept = 0 if layer._sgd_keep is None else int(layer._sgd_keep.sum())
    all_ok(same, "fused SGD step", f"weights / outputs differ from the unfused step (kept {kept})")
    layer.fuse_sgd(None)
    if rank == 0:
        print(f"layer R={R}: errs {errs}, prefetch slots in use {int(tot) // R}, fused SGD ok", flush=True)
    buf.destroy()


def fused_dispatch_check(R, rank):
    """The dispatch that runs inside the gate/up (forward) and down-dgrad (backward) GEMM launches
    must give bit-identical results to the stand-alone dispatch kernel, also with redundant
    experts (local groups and prefetch slots are then two launches) and step after step."""
    from moonep_b200.models.moe_layer import ExpertPools, MoELayer
    from moonep_b200.ops import gemm
    S, H, Hp, K = 512, 1024, 256, 4
    E = 4 * R
    buf = Buffer(S, H, K, E, R, num_sms=8, token_padding=128, timeout_s=10.0)
    assert buf.fused_dispatch_supported()
    pools = ExpertPools(R, E // R, H, Hp, buf.group, rank)
    bias = torch.zeros(E, device="cuda")
    bias[: E // R] = 4.0                       # overload rank 0: redundant experts, prefetch slots
    g = torch.Generator(device="cuda").manual_seed(70 + rank)
    x = torch.randn(S, H, device="cuda", generator=g).bfloat16()
    dy = torch.randn(S, H, device="cuda", generator=g).bfloat16()
    res, used = [], 0
    for fused in (False, True):
        layer = MoELayer(buf, Hp, pools, seed=9, init_std=0.05, router_bias=bias, fused_dispatch=fused,
                         hidden_in_place=True)
        assert layer.fused_dispatch == fused
        for _ in range(3):
            xo = x.clone().requires_grad_(True)
            y = layer(xo)
            y.backward(dy)
            layer.sgd_step(0.05)
        buf.check()
        gemm.check_status()
        used = max(used, int((layer.last_plan.experts_to_copy >= 0).sum()))
        res.append([y.detach().clone(), xo.grad.clone(), layer.w_gate.clone(), layer.w_up.clone(),
                    layer.w_down.clone(), layer.w_router.clone(), layer.last_plan.link.clone(),
                    layer.last_plan.src_info.clone()])
        torch.cuda.synchronize(); dist.barrier()
    names = ["y", "dx", "w_gate", "w_up", "w_down", "w_router", "link", "src_info"]
    bad = [n for n, a, b in zip(names, *res) if not torch.equal(a, b)]
    all_ok(not bad, "fused dispatch vs stand-alone dispatch", f"differ: {bad}")
    tot = torch.tensor([used], device="cuda")
    dist.all_reduce(tot)
    all_ok(int(tot) > 0, "fused dispatch check must exercise prefetch slots", f"slots used {int(tot)}")
    if rank == 0:
        print(f"fused dispatch R={R}: bit-identical over 3 steps, prefetch slots in use {int(tot) // R}", flush=True)
    buf.destroy()


def symm_check(R, rank):
    """Symmetric-memory utilities on real GPUs: the handle type the group agrees on, a tensor that
    lives on one rank and is mapped by all, and (when this process runs with the NVLS overlay
    switched on) a multicast store that lands in every rank's copy, with an orderly teardown."""
    from moonep_b200 import buffer as symm
    dev = torch.cuda.current_device()
    kind = symm.handle_type_for_group(dist.group.WORLD, dev)
    all_ok(kind in ("fd", "fabric"), "handle type", kind)
    # ---- single-owner tensor: memory on the last rank, read and written by everyone -------------
    owner = R - 1
    t = symm.create_nvl_single_owner_tensor((4, 256), torch.int32, owner)
    if rank == owner:
        t.fill_(-1)
    torch.cuda.synchronize(); dist.barrier()
    t[rank % 4, rank * 8:(rank + 1) * 8] = rank + 100               # peer stores into the owner's memory
    torch.cuda.synchronize(); dist.barrier()
    want = torch.full((4, 256), -1, dtype=torch.int32, device="cuda")
    for r in range(R):
        want[r % 4, r * 8:(r + 1) * 8] = r + 100
    all_ok(torch.equal(t, want), "single-owner tensor: every rank sees every rank's stores")
    torch.cuda.synchronize(); dist.barrier()
    symm.release(t)
    # ---- NVLS overlay -------------------------------------------------------------------------------
    n = 1024
    tab, alias = symm.create_nvl_dist_multicast_tensor((R * n,), torch.int32)
    rows = tab.shape[0] // R
    if os.environ.get("MOONEP_B200_NVLS") == "1" and kind == "fd" and \
            symm.nat.call("mep_multicast_supported", dev):
        all_ok(alias is not None, "NVLS overlay was requested and is supported but was not built")
    if alias is not None:
        tab[rank * rows:(rank + 1) * rows].zero_()
        torch.cuda.synchronize(); dist.barrier()
        src = (torch.arange(n, device="cuda", dtype=torch.int32) + 1000 * (rank + 1))
        symm.multimem_broadcast(alias, src, offset=rank * n)       # my row into everyone's table
        torch.cuda.synchronize(); dist.barrier()
        mine = tab[rank * rows: rank * rows + R * n].view(R, n)
        want = torch.stack([torch.arange(n, device="cuda", dtype=torch.int32) + 1000 * (r + 1) for r in range(R)])
        all_ok(torch.equal(mine, want), "multimem.st broadcast: my copy holds every rank's row")
        torch.cuda.synchronize(); dist.barrier()
        symm.release(alias)                  # the multicast mapping goes first, then the memory
    dist.barrier()
    symm.release(tab)
    if rank == 0:
        print(f"symm R={R}: handle type {kind}, single-owner ok, NVLS overlay {'ok' if alias is not None else 'not built'}",
              flush=True)


def decoder_check(R, rank):
    """The fused EP path and the NCCL all-to-all path are two implementations of the same model:
    with identical parameters their first loss agrees, and both train."""
    from moonep_b200.models.decoder import MoEDecoder, NcclMoELayer
    from moonep_b200.models.moe_layer import ExpertPools, MoELayer
    S, Hd, K, Hp, V = 256, 256, 4, 128, 211
    E = 4 * R
    g = torch.Generator(device="cuda").manual_seed(7 + rank)
    tok = torch.randint(0, V, (S,), device="cuda", generator=g)
    tgt = torch.randint(0, V, (S,), device="cuda", generator=g)
    bias = torch.zeros(E, device="cuda")
    bias[: E // R] = 1.0
    out, grads, slots = {}, {}, [None]
    for impl in ("fused", "nccl"):
        torch.manual_seed(3)
        if impl == "fused":
            # token_padding 128: the layers use the dispatch fused into their GEMMs, so the backward
            # pass of layer 0 runs re-prefetch + fused dispatch + the two-launch down dgrad together
            buf = Buffer(S, Hd, K, E, R, num_sms=8, token_padding=128, timeout_s=10.0)
            pools = ExpertPools(R, E // R, Hd, Hp, buf.group, rank)
            fac = lambda i: MoELayer(buf, Hp, pools, seed=20 + i, init_std=0.05, router_bias=bias)
        else:
            fac = lambda i: NcclMoELayer(S, Hd, K, E, Hp, seed=20 + i, init_std=0.05, router_bias=bias,
                                         token_padding=64)
        model = MoEDecoder(V, Hd, 2, 4, fac).cuda()
        # one backward pass without an optimizer step: the two models have the same parameters and
        # run the same GEMM kernels, so their gradients can be compared layer by layer.  Layer 0's
        # redundant experts sit in prefetch slots that layer 1's forward pass has refilled by the
        # time layer 0's backward pass needs them.
        loss0 = model(tok, tgt)
        loss0.backward()
        torch.cuda.synchronize()
        grads[impl] = dict(embed=model.embed.weight.grad.float().clone())
        for i, m in enumerate(model.moe_layers()):
            for n in ("g_gate", "g_up", "g_down", "g_router"):
                grads[impl][f"{i}.{n}"] = getattr(m, n).clone()
        if impl == "fused":
            slots[0] = [int((m.last_plan.experts_to_copy >= 0).sum()) for m in model.moe_layers()]
        for p_ in model.parameters():
            p_.grad = None
        out[impl] = [float(model.train_step(tok, tgt, 0.05)) for _ in range(4)]
        if impl == "fused":
            buf.check()
            buf.destroy()
    tot = torch.tensor(slots[0], device="cuda")
    dist.all_reduce(tot)
    all_ok(int(tot[0]) > 0, "layer 0 must use prefetch slots", f"slots per layer {tot.tolist()}")
    worst = {}
    for k, a in grads["fused"].items():
        b = grads["nccl"][k]
        worst[k] = float((a - b).abs().max()) / (float(b.abs().max()) + 1e-12)
    all_ok(max(worst.values()) < 2e-2, "fused vs nccl gradients", str(worst))
    all_ok(max(abs(a - b) for a, b in zip(out["fused"], out["nccl"])) < 3e-2, "fused vs nccl losses", str(out))
    all_ok(out["fused"][-1] < out["fused"][0] and out["nccl"][-1] < out["nccl"][0], "both train", str(out))
    if rank == 0:
        print(f"decoder R={R}: {out}", flush=True)


def leave_check(R, rank):
    """A rank leaves BETWEEN steps (no kernel or collective of its own in flight).  The others
    learn of it on the host, through the heartbeat, before their next launch: they raise
    PeerLostError instead of entering a device barrier that would have to time out, and release
    their Buffer without a group barrier."""
    from moonep_b200.utils.health import Heartbeat, PeerLostError
    S, H, K, tp = 64, 128, 2, 16
    E = 2 * R
    buf = Buffer(S, H, K, E, R, num_sms=2, token_padding=tp, timeout_s=5.0)
    hb = Heartbeat.from_default_group()
    g = torch.Generator(device="cuda").manual_seed(rank)
    x = torch.randn(S, H, device="cuda", generator=g).bfloat16()
    topk = torch.stack([torch.randperm(E, device="cuda", generator=g)[:K] for _ in range(S)]).to(torch.int32)
    tpe = torch.bincount(topk.flatten().long(), minlength=E).to(torch.int32)
    for step in range(2):
        hb.step(step, timeout_s=20.0)
        h, _, _, plan = buf.dispatch(x, None, topk, tpe)
        out, _, _ = buf.combine(plan, h)
        buf.check()
    torch.cuda.synchronize()
    dist.barrier()
    if rank == R - 1:
        os._exit(0)                                  # gone, with nothing in flight
    try:
        hb.step(2, timeout_s=2.0)
        ok = False
    except PeerLostError as exc:
        ok = exc.missing == [R - 1]
    buf.destroy(group_barrier=False)
    if rank == 0:
        print(f"MULTIGPU_OK R={R} leave detected={ok}", flush=True)
    os._exit(0 if ok else 1)


def _all_gather(t, R):
    lst = [torch.empty_like(t) for _ in range(R)]
    dist.all_gather(lst, t.contiguous())
    return lst


def main():
    local = int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    R, rank = dist.get_world_size(), dist.get_rank()
    what = sys.argv[1] if len(sys.argv) > 1 else "all"
    if what in ("all", "comm"):
        comm_checks(R, rank)
    if what in ("all", "layer"):
        layer_check(R, rank)
    if what in ("all", "symm", "nvls"):
        symm_check(R, rank)
    if what in ("all", "fused"):
        fused_dispatch_check(R, rank)
    if what in ("all", "decoder"):
        decoder_check(R, rank)
    if what == "leave":
        leave_check(R, rank)
    dist.barrier()
    if rank == 0:
        print(f"MULTIGPU_OK R={R} {what}", flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
