"""Dispatch fused into the consuming grouped GEMM (one rank; the multi-rank runs are in
tests/mp_worker.py): the rows that the GEMM's copy warps deliver, the plan records and every
result must be bit-identical to the stand-alone dispatch kernel followed by the same GEMM, and
a tile whose rows never arrive must end in a status, not in a hang."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _routing(S, K, E, seed):
    g = torch.Generator().manual_seed(seed)
    pop = torch.exp(torch.randn(E, generator=g))
    topk = torch.stack([torch.multinomial(pop, K, generator=g) for _ in range(S)]).to(torch.int32)
    w = torch.rand(S, K, generator=g) + 0.1
    tpe = torch.bincount(topk.flatten().long(), minlength=E).to(torch.int32)
    return topk.cuda(), w.cuda(), tpe.cuda()


@pytest.mark.parametrize("H,Hp", [(512, 256), (4096, 256), (7168, 128)])
def test_fused_dispatch_gateup_matches_unfused(H, Hp):
    from moonep_b200 import Buffer
    from moonep_b200.ops import gemm
    S, K, E = 384, 4, 8
    buf = Buffer(S, H, K, E, 1, num_sms=8, token_padding=128, timeout_s=5.0)
    assert buf.fused_dispatch_supported()
    topk, w, tpe = _routing(S, K, E, 3)
    g = torch.Generator(device="cuda").manual_seed(1)
    x = torch.randn(S, H, device="cuda", generator=g).bfloat16()
    wg = (torch.randn(E, H, Hp, device="cuda", generator=g) * 0.05).bfloat16()
    wu = (torch.randn(E, H, Hp, device="cuda", generator=g) * 0.05).bfloat16()
    # ---- stand-alone dispatch, then the GEMM ----------------------------------------------------
    hid0, w0, cu0, plan0 = buf.dispatch(x, w, topk, tpe)
    act0, gate0, up0 = gemm.gateup_swiglu(hid0, wg, wu, cu0[:E], row_scale=w0)
    rows = int(cu0[-1])
    torch.cuda.synchronize()
    # ---- the same through the fused launch (twice: counters are reused call after call) --------
    for it in range(2):
        buf.hidden_nvsh_buffer_view.fill_(7.0)          # stale rows must not survive
        hid, wv, cu, plan, disp = buf.dispatch_fused_begin(x, w, topk, tpe)
        act, gate, up = gemm.gateup_swiglu(hid, wg, wu, cu[:E], row_scale=wv, dispatch=disp)
        w1 = buf.dispatch_fused_end(plan, disp)
        buf.check()
        gemm.check_status()
        assert torch.equal(cu, cu0) and torch.equal(plan.dst, plan0.dst)
        assert torch.equal(hid[:rows], hid0[:rows]), "dispatched rows differ"
        assert torch.equal(w1[:rows], w0[:rows])
        assert torch.equal(plan.link[:rows], plan0.link[:rows])
        assert torch.equal(plan.src_info[:rows], plan0.src_info[:rows])
        for a, b in ((act, act0), (gate, gate0), (up, up0)):
            assert torch.equal(a[:rows], b[:rows])
    # ---- saved plan (the backward direction): down-dgrad GEMM carries the dispatch ---------------
    dy = torch.randn(S, H, device="cuda", generator=g).bfloat16()
    wd = (torch.randn(E, H, Hp, device="cuda", generator=g) * 0.05).bfloat16()
    d0, _, _, _ = buf.dispatch(dy, plan=plan0)
    ref = gemm.down_dgrad(d0, wd, cu0[:E])
    torch.cuda.synchronize()
    buf.hidden_nvsh_buffer_view.fill_(-3.0)
    d1, _, cu_none, plan_same, disp = buf.dispatch_fused_begin(dy, plan=plan)
    assert cu_none is None and plan_same is plan
    got = gemm.down_dgrad(d1, wd, cu0[:E], dispatch=disp)
    buf.dispatch_fused_end(plan, disp)
    buf.check()
    gemm.check_status()
    assert torch.equal(d1[:rows], d0[:rows]) and torch.equal(got[:rows], ref[:rows])
    buf.destroy()


def test_send_order_is_the_documented_permutation():
    from moonep_b200 import Buffer
    S, H, K, R = 128, 256, 4, 4
    E = 8 * R
    buf = Buffer(S, H, K, E, R, num_sms=4, token_padding=16, virtual=True, timeout_s=5.0)
    g = torch.Generator().manual_seed(5)
    topk = torch.stack([torch.stack([torch.randperm(E, generator=g)[:K] for _ in range(S)])
                        for _ in range(R)]).to(torch.int32).cuda()
    tpe = torch.stack([torch.bincount(topk[r].flatten().long(), minlength=E) for r in range(R)]).to(torch.int32)
    x = torch.zeros(R, S, H, dtype=torch.bfloat16, device="cuda")
    _, _, _, plan = buf.dispatch(x, None, topk, tpe.cuda())
    buf.check()
    epn = E // R
    for r in range(R):
        e = topk[r].flatten().long().cpu()
        key = (e % epn) * R + ((e // epn - r) % R)
        want = torch.argsort(key, stable=True).to(torch.int32)
        assert torch.equal(plan.send_order[r].cpu(), want)
    buf.destroy()


def test_rows_that_never_arrive_end_in_a_status():
    """A launch that only WAITS for arrivals while nobody sends: the producer's bounded wait runs
    out, the kernel returns, the status names the block, and the next fused dispatch works."""
    from moonep_b200 import Buffer
    from moonep_b200.ops import gemm
    S, H, Hp, K, E = 128, 512, 128, 2, 4
    buf = Buffer(S, H, K, E, 1, num_sms=4, token_padding=128, timeout_s=0.3)
    topk, w, tpe = _routing(S, K, E, 9)
    g = torch.Generator(device="cuda").manual_seed(2)
    x = torch.randn(S, H, device="cuda", generator=g).bfloat16()
    wg = (torch.randn(E, H, Hp, device="cuda", generator=g) * 0.05).bfloat16()
    wu = (torch.randn(E, H, Hp, device="cuda", generator=g) * 0.05).bfloat16()
    hid, wv, cu, plan, disp = buf.dispatch_fused_begin(x, w, topk, tpe)    # counters are now zero
    gemm.gateup_swiglu(hid, wg, wu, cu[:E], row_scale=wv, dispatch=dict(disp, mode=1))
    torch.cuda.synchronize()
    with pytest.raises(RuntimeError, match="never arrived"):
        gemm.check_status()
    gemm.reset_status()
    # the Buffer is still usable: a complete fused dispatch afterwards gives the right rows
    hid0, w0, cu0, plan0 = buf.dispatch(x, w, topk, tpe)
    rows = int(cu0[-1])
    want = hid0[:rows].clone()
    hid, wv, cu, plan, disp = buf.dispatch_fused_begin(x, w, topk, tpe)
    gemm.gateup_swiglu(hid, wg, wu, cu[:E], row_scale=wv, dispatch=disp)
    buf.dispatch_fused_end(plan, disp)
    buf.check()
    gemm.check_status()
    assert torch.equal(hid[:rows], want)
    buf.destroy()
