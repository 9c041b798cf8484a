"""tcgen05 grouped GEMM at the benchmark's reduction lengths (K = 7168 and K = 2048, N = 2048 and
7168) against an fp32 PyTorch reference, every mode, with a bound derived from bf16 rounding:
each output element may differ from the fp32 result by at most 2^-7 of the largest magnitude in
its row (bf16 output rounding is 2^-9 relative per element; the rest is fp32 accumulation order),
and for fp32 outputs by 2^-12.  A fault in one of the 112 k-blocks, or a tile addressed in the
wrong expert, is far outside that."""
import pytest
import torch

pytestmark = pytest.mark.gpu
H, HP = 7168, 2048
GROUPS = [256, 384, 200]            # incl. a ragged group; single-CTA and CTA-pair kernels both run


@pytest.fixture(autouse=True)
def _status():
    yield
    from moonep_b200.ops import gemm
    torch.cuda.synchronize()
    gemm.check_status()


def _ends(dev="cuda"):
    return torch.tensor(GROUPS).cumsum(0).to(torch.int32).to(dev), sum(GROUPS)


def _per_group(a, w_all, fn):
    out, start = [], 0
    for g, n in enumerate(GROUPS):
        out.append(fn(a[start:start + n].float(), w_all[g].float()))
        start += n
    return torch.cat(out)


def _row_close(got, ref, rel):
    lim = ref.abs().amax(dim=-1, keepdim=True) * rel + 1e-30
    bad = (got.float() - ref).abs() > lim
    assert not bool(bad.any()), f"{int(bad.sum())} elements beyond {rel} of their row's max"


def _data(seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    G = len(GROUPS)
    ends, rows = _ends()
    mk = lambda *s, std=1.0: (torch.randn(*s, device="cuda", generator=g) * std).bfloat16()
    return g, G, ends, rows, mk


@pytest.mark.parametrize("two", [0, 1])
def test_gateup_swiglu_k7168(two, monkeypatch):
    from moonep_b200.ops import gemm
    monkeypatch.setattr(gemm, "TWO_CTA", two)
    g, G, ends, rows, mk = _data(1)
    x, wg, wu = mk(rows, H), mk(G, H, HP, std=0.02), mk(G, H, HP, std=0.02)
    rs = torch.rand(rows, device="cuda", generator=g) + 0.5
    act, gate, up = gemm.gateup_swiglu(x, wg, wu, ends, row_scale=rs)
    _row_close(gate, _per_group(x, wg, lambda a, w: a @ w), 2 ** -7)
    _row_close(up, _per_group(x, wu, lambda a, w: a @ w), 2 ** -7)
    a_ref = torch.nn.functional.silu(gate.float()) * up.float() * rs[:, None]
    _row_close(act, a_ref, 2 ** -7)


@pytest.mark.parametrize("two", [0, 1])
def test_down_and_push_k2048(two, monkeypatch):
    from moonep_b200.ops import gemm
    monkeypatch.setattr(gemm, "TWO_CTA", two)
    g, G, ends, rows, mk = _data(2)
    act, wd = mk(rows, HP), mk(G, H, HP, std=0.02)
    ref = _per_group(act, wd, lambda a, w: a @ w.t())
    y = gemm.down(act, wd, ends)
    _row_close(y, ref, 2 ** -7)
    # the same GEMM with the push epilogue: every row goes to slot (rank 0, entry = row index)
    src = torch.arange(rows, dtype=torch.int32, device="cuda")
    stage = torch.zeros(rows, H, dtype=torch.bfloat16, device="cuda")
    gemm.down(act, wd, ends, push=dict(src_info=src, push_base=stage, push_rank_stride=rows * H,
                                       push_entries=rows, push_ranks=1))
    torch.cuda.synchronize()
    assert torch.equal(stage, y)


@pytest.mark.parametrize("two", [0, 1])
def test_dgrads(two, monkeypatch):
    from moonep_b200.ops import gemm
    monkeypatch.setattr(gemm, "TWO_CTA", two)
    g, G, ends, rows, mk = _data(3)
    dy, wd = mk(rows, H), mk(G, H, HP, std=0.02)
    _row_close(gemm.down_dgrad(dy, wd, ends), _per_group(dy, wd, lambda a, w: a @ w), 2 ** -7)
    dg, du, wg, wu = mk(rows, HP), mk(rows, HP), mk(G, H, HP, std=0.02), mk(G, H, HP, std=0.02)
    ref = _per_group(dg, wg, lambda a, w: a @ w.t()) + _per_group(du, wu, lambda a, w: a @ w.t())
    _row_close(gemm.gateup_dgrad(dg, du, wg, wu, ends), ref, 2 ** -7)


@pytest.mark.parametrize("two", [0, 1])
def test_wgrad_fp32(two, monkeypatch):
    from moonep_b200.ops import gemm
    monkeypatch.setattr(gemm, "TWO_CTA", two)
    global GROUPS
    g, G, ends, rows, mk = _data(4)
    groups = [256, 384, 192]                       # weight-grad groups are multiples of 64
    ends = torch.tensor(groups).cumsum(0).to(torch.int32).cuda()
    rows = sum(groups)
    a, b = mk(rows, H), mk(rows, HP)
    grad = torch.zeros(G, H, HP, device="cuda")
    gemm.wgrad(a, b, ends, grad)
    start = 0
    for i, n in enumerate(groups):
        ref = a[start:start + n].float().t() @ b[start:start + n].float()
        _row_close(grad[i], ref, 2 ** -12)
        start += n
