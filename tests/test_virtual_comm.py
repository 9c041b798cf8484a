"""Single-GPU virtual-group tests: all R ranks of an EP group run as ONE cooperative launch per
kernel on one device, over R VMM chunks mapped back to back.  The device kernels are compared
with the CPU oracle / simulator: the plan bit-exactly, dispatched rows and weights exactly,
combine within bf16 rounding (the reference allows 1 ulp, tests/test_combine.py:177-254)."""
import pytest
import torch

from moonep_b200 import reference as ref
from tests.cases import CASES, case_params

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True)
def _cleanup():
    yield
    from moonep_b200.api import destroy_live_buffers
    destroy_live_buffers()
    torch.cuda.synchronize()


def make_buffer(case, R, **kw):
    from moonep_b200 import Buffer
    H = max(case.H, 8)
    return Buffer(case.S, H, case.K, case.epn * R, R, num_sms=min(case.num_sms, 8),
                  token_padding=case.token_padding, virtual=True, timeout_s=2.0, **kw)


def traceable(R, S, H, K):
    """Row payload encodes (rank, token); weights encode the flat entry index."""
    x = torch.zeros(R, S, H)
    x[:, :, 0] = torch.arange(R)[:, None].float()
    x[:, :, 1] = (torch.arange(S) % 256)[None, :].float()
    x[:, :, 2] = (torch.arange(S) // 256)[None, :].float()
    x[:, :, 3:] = torch.randn(R, S, H - 3, generator=torch.Generator().manual_seed(1))
    w = torch.arange(R * S * K, dtype=torch.float32).view(R, S, K) + 0.5
    return x.bfloat16(), w


@pytest.mark.parametrize("case,R", case_params(Rs=(1, 2, 4, 8)))
def test_plan_dispatch_combine_vs_oracle(case, R):
    S, K, epn, tp = case.S, case.K, case.epn, case.token_padding
    E = epn * R
    buf = make_buffer(case, R)
    H = buf.H
    topk, tpe = case.topk_all(R)
    x, w = traceable(R, S, H, K)
    hidden, w_nvs, cu, plan = buf.dispatch(x.cuda(), w.cuda(), topk.cuda(), tpe.cuda())
    buf.check()
    # ---- plan: bit-exact against the CPU oracle
    tables, dst = ref.plan_all_ranks(topk, S, K, E, tp, tpe)
    assert torch.equal(plan.dst.cpu(), dst)
    assert torch.equal(plan.cu_seqlens.cpu(), tables.cu_seqlens)
    assert torch.equal(plan.zero_fill_ranges.cpu(), tables.zero_fill)
    assert torch.equal(plan.remote_stats.cpu(), tables.remote_stats)
    for r in range(R):
        assert torch.equal(plan.experts_to_copy[r].cpu(), tables.experts_to_copy)
    # ---- dispatch: rows, weights, zero fill, chain links against the simulator
    sim = ref.SimGroup(S, H, K, E, R, tp)
    h_ref, w_ref, _, plans_ref = sim.dispatch(x, w, topk)
    hid, wn, link = hidden.cpu(), w_nvs.cpu(), plan.link.cpu()
    for r in range(R):
        rows = int(tables.cu_seqlens[r, -1])
        assert torch.equal(hid[r, :rows], h_ref[r, :rows])
        assert torch.equal(wn[r, :rows], w_ref[r, :rows])
        assert torch.equal(link[r, :rows], plans_ref[r].link[:rows])
    # ---- identity round trip through combine (unweighted K-sum), weights gathered bit-exactly
    out, w_back, ev = buf.combine(plan, hidden, w_nvs)
    buf.check()
    assert ev is None
    out_ref, wb_ref = sim.combine(plans_ref, h_ref, w_ref)
    assert torch.equal(w_back.cpu(), w)
    assert torch.equal(out.cpu().view(torch.int16), out_ref.view(torch.int16))


def test_combine_scaled_rows_and_plan_reuse():
    """Per-row scaling before combine (a stand-in FFN), then a saved-plan re-dispatch: planning
    is skipped, cu_seqlens is None, the same plan object comes back and the weight slots stay
    untouched when no weights are given (tests/test_e2e.py:253-265)."""
    from moonep_b200 import Buffer
    R, S, K, E, H, tp = 4, 64, 4, 16, 256, 16
    buf = Buffer(S, H, K, E, R, num_sms=4, token_padding=tp, virtual=True, timeout_s=2.0)
    g = torch.Generator().manual_seed(3)
    topk = torch.stack([torch.stack([torch.randperm(E, generator=g)[:K] for _ in range(S)])
                        for _ in range(R)]).to(torch.int32)
    tpe = torch.stack([torch.bincount(topk[r].flatten().long(), minlength=E) for r in range(R)]).to(torch.int32)
    x = torch.randn(R, S, H, generator=g).bfloat16()
    w = torch.rand(R, S, K, generator=g)
    hidden, w_nvs, cu, plan = buf.dispatch(x.cuda(), w.cuda(), topk.cuda(), tpe.cuda())
    y = (hidden.float() * w_nvs[:, :, None]).bfloat16()
    out, _, _ = buf.combine(plan, y, None)
    sim = ref.SimGroup(S, H, K, E, R, tp)
    h_ref, w_ref, _, plans_ref = sim.dispatch(x, w, topk)
    y_ref = (h_ref.float() * w_ref[:, :, None]).bfloat16()
    out_ref, _ = sim.combine(plans_ref, y_ref)
    assert torch.equal(out.cpu().view(torch.int16), out_ref.view(torch.int16))
    dense = (x.float() * w.sum(2, keepdim=True))
    assert float((out.cpu().float() - dense).abs().max()) < 0.1
    # saved-plan re-dispatch of another tensor, hidden only
    before = buf.router_weight_buffer_view.clone()
    g2 = torch.randn(R, S, H, generator=g).bfloat16()
    h2, w2, cu2, plan2 = buf.dispatch(g2.cuda(), plan=plan)
    buf.check()
    assert w2 is None and cu2 is None and plan2 is plan
    assert torch.equal(buf.router_weight_buffer_view, before)
    h2_ref, _, _, _ = sim.dispatch(g2, None, topk)
    for r in range(R):
        rows = int(plan.cu_seqlens[r, -1])
        assert torch.equal(h2.cpu()[r, :rows], h2_ref[r, :rows])


def test_zero_copy_async_and_bad_inputs():
    from moonep_b200 import Buffer
    R, S, K, E, H, tp = 2, 32, 2, 8, 128, 8
    buf = Buffer(S, H, K, E, R, num_sms=2, token_padding=tp, virtual=True, timeout_s=2.0)
    g = torch.Generator().manual_seed(5)
    topk = torch.stack([torch.stack([torch.randperm(E, generator=g)[:K] for _ in range(S)])
                        for _ in range(R)]).to(torch.int32).cuda()
    tpe = torch.stack([torch.bincount(topk[r].flatten().long(), minlength=E) for r in range(R)]).to(torch.int32)
    x = torch.randn(R, S, H, generator=g).bfloat16().cuda()
    w = torch.rand(R, S, K, generator=g).cuda()
    h_sync, w_sync, cu_sync, plan_sync = buf.dispatch(x, w, topk, tpe)
    h_async, w_async, cu_async, plan_async, ev = buf.dispatch(x, w, topk, tpe, async_finish=True)
    ev.wait()
    torch.cuda.synchronize()
    rows = plan_sync.cu_seqlens[:, -1].tolist()
    for r in range(R):
        assert torch.equal(h_sync[r, :rows[r]], h_async[r, :rows[r]])
        assert torch.equal(w_sync[r, :rows[r]], w_async[r, :rows[r]])
    assert torch.equal(plan_sync.dst, plan_async.dst)
    # zero-copy round trip is bit exact with the copying path
    hz, wz, _, planz = buf.dispatch(x, w, topk, tpe, zero_copy=True, router_weights_zero_copy=True)
    assert hz.data_ptr() == buf.hidden_nvsh_buffer_view.data_ptr()
    out_z, wk_z, _ = buf.combine(planz, hz, wz, zero_copy=True, router_weights_zero_copy=True)
    out_c, wk_c, ev2 = buf.combine(plan_sync, h_sync, w_sync, async_finish=True)
    ev2.wait()
    torch.cuda.synchronize()
    assert torch.equal(out_z, out_c) and torch.equal(wk_z, wk_c) and torch.equal(wk_c, w)
    with pytest.raises(AssertionError, match="alias"):
        buf.combine(planz, h_sync, None, zero_copy=True)
    with pytest.raises(AssertionError, match="plan is required"):
        buf.combine(None, h_sync)
    with pytest.raises(TypeError):
        buf.combine(planz, hidden_sh=h_sync)
    with pytest.raises(AssertionError):
        buf.dispatch(x.float(), w, topk, tpe)
    with pytest.raises(AssertionError):
        buf.dispatch(x, w, topk.long(), tpe)
    buf.check()
    st = buf.stats()
    assert st["dispatch"] == 3 and st["combine"] == 2 and 0 < st["dedup_ratio"] <= 1
    buf.destroy()
    buf.destroy()   # idempotent
    assert buf.destroyed


def test_barrier_many_rounds_and_sync_kernel():
    from moonep_b200 import Buffer
    buf = Buffer(8, 64, 2, 8, 8, num_sms=2, token_padding=8, virtual=True, timeout_s=2.0)
    for _ in range(2000):
        buf.inter_rank_sync()
    buf.check()
    assert buf.sync_state[0, :, 1].tolist() == [2000] * 8


def test_bounded_wait_reports_status_and_recovers():
    """Failure detection without a GPU fault: one virtual rank is made to expect a barrier epoch
    that its peer will never publish (a flag that nothing sets).  Its wait runs out after the
    short limit, the kernel RETURNS, the host reads the status block and raises; after
    ``reset_barriers()`` the same Buffer works again."""
    from moonep_b200 import Buffer
    from moonep_b200.api import CommTimeoutError
    buf = Buffer(8, 64, 2, 4, 2, num_sms=1, token_padding=8, virtual=True, timeout_s=0.2)
    buf.inter_rank_sync()
    buf.check()
    buf.sync_state[0, 0, 1] += 5            # rank 0 now waits for an epoch rank 1 never reaches
    torch.cuda.synchronize()
    buf.inter_rank_sync()
    with pytest.raises(CommTimeoutError) as exc:
        buf.check()
    info = exc.value.info
    assert info["kernel"] == "sync" and info["code"] == 2 and info["rank"] == 0 and info["peer"] == 1
    assert info["expected"] - info["observed"] == 5
    buf.reset_barriers()
    for _ in range(3):
        buf.inter_rank_sync()
    buf.check()
    # and a full round trip still works on the recovered Buffer
    x = torch.randn(2, 8, 64, device="cuda").bfloat16()
    topk = torch.tensor([[0, 1]] * 8 + [[2, 3]] * 8, dtype=torch.int32, device="cuda").view(2, 8, 2)
    tpe = torch.stack([torch.bincount(topk[r].flatten().long(), minlength=4) for r in range(2)]).to(torch.int32)
    h, _, _, plan = buf.dispatch(x, None, topk, tpe)
    out, _, _ = buf.combine(plan, h)
    buf.check()
    assert torch.equal(out.float(), (x.float() * 2).bfloat16().float())


@pytest.mark.parametrize("R", [2, 4])
def test_programmatic_dependent_launch_gives_identical_results(R):
    """``enable_pdl`` only changes WHEN the follower kernels of a chain are scheduled (plan ->
    dispatch -> expansion, pre-reduction -> combine); rows, weights, plan and sums are the same."""
    from moonep_b200 import Buffer
    from moonep_b200.utils.routing import routing_for_maxvio, tokens_per_expert
    S, H, K, E, tp = 128, 256, 4, 8 * R, 16
    topk, w, _, _ = routing_for_maxvio(S, K, E, R, 2.0, seed=3)
    tpe = torch.stack([tokens_per_expert(topk[r], E) for r in range(R)]).cuda()
    x = torch.randn(R, S, H, generator=torch.Generator().manual_seed(8)).bfloat16().cuda()
    res = []
    for pdl in (False, True):
        buf = Buffer(S, H, K, E, R, num_sms=4, token_padding=tp, virtual=True, timeout_s=5.0, enable_pdl=pdl)
        for _ in range(3):                                    # back to back: chains overlap their tails
            hidden, w_nvs, cu, plan = buf.dispatch(x, w.cuda(), topk.cuda(), tpe)
            y = (hidden.float() * w_nvs[:, :, None]).bfloat16()
            out, w_back, _ = buf.combine(plan, y, w_nvs)
        buf.check()
        rows = cu[:, -1].tolist()
        res.append((out.clone(), w_back.clone(), plan.dst.clone(), cu.clone(),
                    [hidden[r, :rows[r]].clone() for r in range(R)]))
        buf.destroy()
    a, b = res
    assert torch.equal(a[0], b[0]) and torch.equal(a[1], b[1]) and torch.equal(a[2], b[2]) and torch.equal(a[3], b[3])
    for u, v in zip(a[4], b[4]):
        assert torch.equal(u, v)


def test_phase_stamps_when_compiled_in():
    """With a library built with -DMEP_PHASE_STAMPS the dispatch and combine kernels record
    per-CTA %globaltimer stamps; the phases of a kernel are ordered in time.  A normal build has
    no stamps (the call says so) and the test is skipped."""
    from moonep_b200 import Buffer
    from moonep_b200.utils.routing import routing_for_maxvio, tokens_per_expert
    R, S, H, K, tp = 2, 128, 256, 4, 16
    E = 8 * R
    buf = Buffer(S, H, K, E, R, num_sms=4, token_padding=tp, virtual=True, timeout_s=5.0)
    if not buf.enable_phase_stamps():
        buf.destroy()
        pytest.skip("library built without -DMEP_PHASE_STAMPS")
    topk, w, _, _ = routing_for_maxvio(S, K, E, R, 1.0, seed=2)
    tpe = torch.stack([tokens_per_expert(topk[r], E) for r in range(R)]).cuda()
    x = torch.randn(R, S, H, generator=torch.Generator().manual_seed(1)).bfloat16().cuda()
    h, wn, cu, plan = buf.dispatch(x, w.cuda(), topk.cuda(), tpe)
    buf.combine(plan, h, None)
    st = buf.phase_stamps()
    assert set(st) >= {"dispatch", "combine"}
    d = st["dispatch"]
    assert d["set up"][0] == 0.0 and d["past exit barrier"][1] >= d["rows issued"][0] >= 0.0
    assert st["combine"]["tokens stored"][1] >= st["combine"]["past entry barrier"][0]
    buf.destroy()
