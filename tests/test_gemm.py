"""tcgen05 grouped GEMM against plain PyTorch fp32 references of the same ops."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _mk(rows_per_group, dev="cuda"):
    ends = torch.tensor(rows_per_group).cumsum(0).to(torch.int32).to(dev)
    return ends, int(ends[-1])


def _ref_tokens(a, w_all, ends, fn):
    out = []
    start = 0
    for g, e in enumerate(ends.tolist()):
        if e > start:
            out.append(fn(a[start:e].float(), w_all[g].float()))
        start = e
    return torch.cat(out)


@pytest.fixture(autouse=True)
def _status():
    yield
    from moonep_b200.ops import gemm
    torch.cuda.synchronize()
    gemm.check_status()


def _close(x, ref, tol=2e-2):
    scale = float(ref.abs().max()) + 1e-6
    err = float((x.float() - ref).abs().max()) / scale
    assert err < tol, f"relative max error {err}"


@pytest.mark.parametrize("groups", [[128, 256, 0, 128], [100, 0, 300, 1, 129, 64]])
@pytest.mark.parametrize("H,Hp", [(256, 384), (512, 128)])
def test_down_and_dgrads(groups, H, Hp):
    from moonep_b200.ops import gemm
    g = torch.Generator(device="cuda").manual_seed(0)
    ends, rows = _mk(groups)
    G = len(groups)
    split = G // 2
    w_all = (torch.randn(G, H, Hp, device="cuda", generator=g) * 0.05).bfloat16()
    w_loc, w_slot = w_all[:split].contiguous(), w_all[split:].contiguous()
    act = torch.randn(rows, Hp, device="cuda", generator=g).bfloat16()
    y = gemm.down(act, w_loc, ends, wd_slot=w_slot, split=split)
    _close(y, _ref_tokens(act, w_all, ends, lambda a, w: a @ w.t()))
    dy = torch.randn(rows, H, device="cuda", generator=g).bfloat16()
    dact = gemm.down_dgrad(dy, w_loc, ends, wd_slot=w_slot, split=split)
    _close(dact, _ref_tokens(dy, w_all, ends, lambda a, w: a @ w))
    wu_all = (torch.randn(G, H, Hp, device="cuda", generator=g) * 0.05).bfloat16()
    dg = torch.randn(rows, Hp, device="cuda", generator=g).bfloat16()
    du = torch.randn(rows, Hp, device="cuda", generator=g).bfloat16()
    dx = gemm.gateup_dgrad(dg, du, w_loc, wu_all[:split].contiguous(), ends, wg_slot=w_slot,
                           wu_slot=wu_all[split:].contiguous(), split=split)
    ref = _ref_tokens(dg, w_all, ends, lambda a, w: a @ w.t()) + \
        _ref_tokens(du, wu_all, ends, lambda a, w: a @ w.t())
    _close(dx, ref)


@pytest.mark.parametrize("groups", [[128, 256, 0, 128], [100, 0, 300, 1, 129, 64]])
def test_gateup_swiglu(groups):
    from moonep_b200.ops import gemm
    H, Hp = 256, 384
    g = torch.Generator(device="cuda").manual_seed(1)
    ends, rows = _mk(groups)
    G = len(groups)
    wg = (torch.randn(G, H, Hp, device="cuda", generator=g) * 0.08).bfloat16()
    wu = (torch.randn(G, H, Hp, device="cuda", generator=g) * 0.08).bfloat16()
    x = torch.randn(rows, H, device="cuda", generator=g).bfloat16()
    rs = torch.rand(rows, device="cuda", generator=g) + 0.5
    act, gate, up = gemm.gateup_swiglu(x, wg, wu, ends, row_scale=rs)
    g_ref = _ref_tokens(x, wg, ends, lambda a, w: a @ w)
    u_ref = _ref_tokens(x, wu, ends, lambda a, w: a @ w)
    _close(gate, g_ref)
    _close(up, u_ref)
    gb, ub = gate.float(), up.float()
    a_ref = torch.nn.functional.silu(gb) * ub * rs[:, None]
    _close(act, a_ref, tol=1e-2)


@pytest.mark.parametrize("groups", [[128, 256, 0, 64], [64, 0, 0, 192, 320, 64]])
@pytest.mark.parametrize("accumulate", [False, True])
def test_wgrad(groups, accumulate):
    from moonep_b200.ops import gemm
    M, N = 256, 320
    g = torch.Generator(device="cuda").manual_seed(2)
    ends, rows = _mk(groups)
    G = len(groups)
    split = G // 2
    a = torch.randn(rows, M, device="cuda", generator=g).bfloat16()
    b = torch.randn(rows, N, device="cuda", generator=g).bfloat16()
    gl = torch.randn(split, M, N, device="cuda", generator=g)
    gs = torch.randn(G - split, M, N, device="cuda", generator=g)
    gl0, gs0 = gl.clone(), gs.clone()
    gemm.wgrad(a, b, ends, gl, grad_slot=gs, split=split, accumulate=accumulate)
    start = 0
    for gi, e in enumerate(ends.tolist()):
        ref = a[start:e].float().t() @ b[start:e].float()
        tgt, base = (gl[gi], gl0[gi]) if gi < split else (gs[gi - split], gs0[gi - split])
        if accumulate:
            ref = ref + base
        elif e == start and gi >= split:
            ref = base                      # empty slot groups are left untouched
        _close(tgt, ref, tol=1e-2)
        start = e


def test_dense_router_logits():
    from moonep_b200.ops import gemm
    g = torch.Generator(device="cuda").manual_seed(3)
    a = torch.randn(300, 512, device="cuda", generator=g).bfloat16()
    b = (torch.randn(512, 64, device="cuda", generator=g) * 0.1).bfloat16()
    c = gemm.dense(a, b)
    _close(c, a.float() @ b.float(), tol=5e-3)
    c2 = gemm.dense(a, b.t().contiguous(), b_is_kn=False, out_dtype=torch.bfloat16)
    _close(c2, a.float() @ b.float())


@pytest.mark.parametrize("b_mn", [False, True])
def test_cta_pair_variant_matches(b_mn, monkeypatch):
    """The cta_group::2 kernel (clusters of two CTAs, each staging half of the B tile) gives the
    same results as the single-CTA kernel, including the SwiGLU epilogue."""
    from moonep_b200.ops import gemm
    g = torch.Generator(device="cuda").manual_seed(7)
    groups = [256, 128, 0, 384, 100]
    ends, rows = _mk(groups)
    G, H, Hp = len(groups), 256, 384
    w = (torch.randn(G, H, Hp, device="cuda", generator=g) * 0.06).bfloat16()
    w2 = (torch.randn(G, H, Hp, device="cuda", generator=g) * 0.06).bfloat16()
    if b_mn:
        x = torch.randn(rows, H, device="cuda", generator=g).bfloat16()
        run = lambda: gemm.gateup_swiglu(x, w, w2, ends)
    else:
        x = torch.randn(rows, Hp, device="cuda", generator=g).bfloat16()
        run = lambda: (gemm.down(x, w, ends),)
    monkeypatch.setattr(gemm, "TWO_CTA", 0)
    one = [t.clone() for t in run()]
    monkeypatch.setattr(gemm, "TWO_CTA", 1)
    two = run()
    for a, b in zip(one, two):
        assert torch.equal(a, b)


@pytest.mark.parametrize("accumulate", [False, True])
def test_cta_pair_weight_grad_matches(accumulate, monkeypatch):
    """Weight-grad tiles of a CTA pair (256 weight rows, each CTA 128 of them and half of the B
    tile) are bit-identical to the single-CTA kernel's, with local and slot outputs."""
    from moonep_b200.ops import gemm
    g = torch.Generator(device="cuda").manual_seed(11)
    groups = [192, 64, 0, 320, 128, 0]
    ends, rows = _mk(groups)
    M, N, split = 512, 320, 4
    a = torch.randn(rows, M, device="cuda", generator=g).bfloat16()
    b = torch.randn(rows, N, device="cuda", generator=g).bfloat16()
    base_l = torch.randn(split, M, N, device="cuda", generator=g)
    base_s = torch.randn(len(groups) - split, M, N, device="cuda", generator=g)
    res = []
    for two in (0, 1):
        monkeypatch.setattr(gemm, "TWO_CTA", two)
        gl, gs = base_l.clone(), base_s.clone()
        gemm.wgrad(a, b, ends, gl, grad_slot=gs, split=split, accumulate=accumulate)
        res.append((gl, gs))
    assert torch.equal(res[0][0], res[1][0]) and torch.equal(res[0][1], res[1][1])
    start = 0
    for i, n in enumerate(groups):
        want = a[start:start + n].float().t() @ b[start:start + n].float()
        got = res[1][0][i] if i < split else res[1][1][i - split]
        base = base_l[i] if i < split else base_s[i - split]
        if accumulate:
            want = want + base
        elif n == 0 and i >= split:
            want = base                       # empty slot groups are left untouched
        _close(got, want, tol=5e-3)
        start += n


@pytest.mark.parametrize("two", [0, 1])
def test_weight_grad_fused_sgd(two, monkeypatch):
    """``wgrad(sgd=...)`` updates the unflagged local experts exactly like wgrad + sgd_update_, stores
    fp32 grads for flagged experts and slot groups, and leaves experts without rows alone."""
    from moonep_b200.ops import elementwise as ew
    from moonep_b200.ops import gemm
    monkeypatch.setattr(gemm, "TWO_CTA", two)
    g = torch.Generator(device="cuda").manual_seed(13)
    groups = [192, 0, 64, 320, 128, 0]
    ends, rows = _mk(groups)
    M, N, split, lr = 512, 328, 4, 0.37
    a = torch.randn(rows, M, device="cuda", generator=g).bfloat16()
    b = torch.randn(rows, N, device="cuda", generator=g).bfloat16()
    w0 = torch.randn(split, M, N, device="cuda", generator=g).bfloat16()
    gl = torch.zeros(split, M, N, device="cuda")
    gs = torch.zeros(len(groups) - split, M, N, device="cuda")
    gemm.wgrad(a, b, ends, gl, grad_slot=gs, split=split)
    want = w0.clone()
    ew.sgd_update_(want, gl, lr)
    keep = torch.tensor([0, 0, 1, 0], dtype=torch.int32, device="cuda")
    w = w0.clone()
    gl2 = torch.full_like(gl, 7.0)
    gs2 = torch.full_like(gs, 7.0)
    gemm.wgrad(a, b, ends, gl2, grad_slot=gs2, split=split, sgd=(w, lr, keep))
    torch.cuda.synchronize()
    for e in (0, 1, 3):
        assert torch.equal(w[e], want[e]) and bool((gl2[e] == 7.0).all())     # applied, grad not written
    assert torch.equal(w[1], w0[1])                                           # no rows: untouched
    assert torch.equal(w[2], w0[2]) and torch.equal(gl2[2], gl[2])            # flagged: grad stored
    assert torch.equal(gs2[0], gs[0]) and bool((gs2[1] == 7.0).all())         # slots: stored / empty untouched
    ew.sgd_update_(w, gl2, lr, only=keep)
    assert torch.equal(w, want)


@pytest.mark.parametrize("two", [0, 1])
def test_weight_grad_fused_sgd_in_two_launches(two, monkeypatch):
    """``select=1`` (stored grads only) followed by ``select=2`` (applied tiles only) leaves exactly
    what one launch leaves; after the first launch no weight has changed yet."""
    from moonep_b200.ops import gemm
    monkeypatch.setattr(gemm, "TWO_CTA", two)
    g = torch.Generator(device="cuda").manual_seed(14)
    groups = [128, 256, 0, 64, 192, 64]
    ends, rows = _mk(groups)
    M, N, split, lr = 256, 264, 4, 0.21
    a = torch.randn(rows, M, device="cuda", generator=g).bfloat16()
    b = torch.randn(rows, N, device="cuda", generator=g).bfloat16()
    w0 = torch.randn(split, M, N, device="cuda", generator=g).bfloat16()
    keep = torch.tensor([1, 0, 0, 1], dtype=torch.int32, device="cuda")
    outs = []
    for selects in ((0,), (1, 2)):
        w = w0.clone()
        gl = torch.full((split, M, N), 5.0, device="cuda")
        gs = torch.full((len(groups) - split, M, N), 5.0, device="cuda")
        for i, sel in enumerate(selects):
            gemm.wgrad(a, b, ends, gl, grad_slot=gs, split=split, sgd=(w, lr, keep), select=sel)
            if sel == 1:
                torch.cuda.synchronize()
                assert torch.equal(w, w0)                       # nothing applied yet
                assert not bool((gl[0] == 5.0).all()) and not bool((gs[0] == 5.0).all())
        torch.cuda.synchronize()
        outs.append((w, gl, gs))
    for x, y in zip(*outs):
        assert torch.equal(x, y)
    gemm.check_status()
