"""GPU-less multi-rank simulator: R ranks in one process, arrays stand in for peer memory.

Covers the first benchmark configuration (8 simulated ranks, S=512, K=8, E=64, H=256 fp32,
token_padding=16, Zipf-skewed routing swept over MaxVio 0/1/4): every rank receives exactly
S*K rows, each rank's prefetch slots come from one remote home group, and
combine(dispatch(x)) equals the dense weighted top-k sum."""
import pytest
import torch

from moonep_b200.reference import SimGroup
from moonep_b200.utils.routing import maxvio, routing_for_maxvio, tokens_per_expert
from tests.cases import case_params
from tests.test_planner_oracle import check_plan


@pytest.mark.parametrize("target", [0.0, 1.0, 4.0])
def test_config1_roundtrip_weighted(target):
    R, S, K, E, H, tp = 8, 512, 8, 64, 256, 16
    topk, w, mv, _ = routing_for_maxvio(S, K, E, R, target, seed=7)
    if target > 0:
        assert abs(mv - target) < 0.25 * target + 0.05
    sim = SimGroup(S, H, K, E, R, tp)
    g = torch.Generator().manual_seed(11)
    x = torch.randn(R, S, H, generator=g)
    hidden, w_nvs, cu, plans = sim.dispatch(x, w, topk)
    tables, dst = sim.plan(topk)

    class C:  # the invariants helper wants a case-like object
        pass
    c = C(); c.S, c.K, c.epn, c.token_padding = S, K, E // R, tp
    check_plan(c, R, tables, dst)
    # an "expert" that multiplies each row by its route weight; padding rows stay zero
    y = hidden * w_nvs[:, :, None]
    out, w_back = sim.combine(plans, y, w_nvs)
    assert torch.equal(w_back, w)                       # bit-exact weight round trip
    dense = x * w.sum(dim=2, keepdim=True)
    torch.testing.assert_close(out, dense, rtol=1e-5, atol=1e-5)


@pytest.mark.parametrize("case,R", case_params(Rs=(1, 2, 4, 8)))
def test_sim_dispatch_places_every_row(case, R):
    S, K, H, epn, tp = case.S, case.K, case.H, case.epn, case.token_padding
    topk, _ = case.topk_all(R)
    sim = SimGroup(S, H, K, epn * R, R, tp)
    # traceable payload: row encodes (rank, token); weight encodes the flat entry index
    x = (torch.arange(R)[:, None, None] * 1000 + torch.arange(S)[None, :, None]
         + torch.zeros(1, 1, H)).float()
    w = torch.arange(R * S * K, dtype=torch.float32).view(R, S, K)
    hidden, w_nvs, cu, plans = sim.dispatch(x, w, topk, poison=-7.0)
    NvS = sim.NvS
    for r in range(R):
        raw = torch.where(plans[r].dst < 0, -plans[r].dst - 1, plans[r].dst).long()
        dr, lo = raw // NvS, raw % NvS
        tok = torch.arange(S).repeat_interleave(K)
        assert torch.equal(hidden[dr, lo, 0], (r * 1000 + tok).float())   # dups expanded too
        assert torch.equal(w_nvs[dr, lo], w[r].flatten())
    for d in range(R):
        zf = plans[d].zero_fill_ranges
        for g in range(2 * epn):
            a, n = zf[g].tolist()
            assert bool((hidden[d, a:a + n] == 0).all()) and bool((w_nvs[d, a:a + n] == 0).all())
        tail = int(plans[d].cu_seqlens[-1])
        assert bool((hidden[d, tail:] == -7.0).all())                     # tail untouched
    # identity round trip: combine(dispatch(x)) == K * x
    out, w_back = sim.combine(plans, hidden, w_nvs)
    torch.testing.assert_close(out, x * K)
    assert torch.equal(w_back, w)


def test_sim_bf16_prologue_rounding_and_dedup_views():
    R, S, K, E, H, tp = 2, 16, 4, 8, 32, 8
    topk = torch.stack([torch.stack([torch.randperm(E, generator=torch.Generator().manual_seed(s))[:K]
                                     for s in range(S)]) for _ in range(R)]).to(torch.int32)
    sim = SimGroup(S, H, K, E, R, tp)
    x = torch.randn(R, S, H, generator=torch.Generator().manual_seed(5)).bfloat16()
    hidden, _, _, plans = sim.dispatch(x, None, topk)
    out, _ = sim.combine(plans, hidden)
    ref = (x.float() * K).bfloat16()
    # one rounding in the duplicate pre-reduce and one in the final sum: <= 2 bf16 ulp
    assert float((out.float() - ref.float()).abs().max()) <= 2 * 2 ** -7 * float(ref.float().abs().max())
    for d in range(R):
        p = plans[d]
        ng, nd = p.dup_counts.tolist()
        groups = p.dup_groups[:ng]
        assert int(groups[:, 2].sum()) == nd
        # every duplicate row is flagged as such in link and appears once
        dups = p.dup_loffs[:nd].long()
        assert dups.unique().numel() == nd
        assert bool(((p.link[dups] & 0x40000000) != 0).all())
        assert bool(((p.link[groups[:, 0].long()] & 0x40000000) == 0).all())
    # total duplicates = number of negative dst entries
    total = sum(int(p.dup_counts[1]) for p in plans)
    assert total == sum(int((p.dst < 0).sum()) for p in plans)


def test_maxvio_definition():
    tpe = torch.tensor([10, 10, 10, 30])
    assert abs(maxvio(tpe) - 1.0) < 1e-9


def test_cpu_benchmark_script_runs(capsys, monkeypatch):
    """``benchmarks/bench_sim.py`` (configuration 1 on the CPU) exits cleanly and reports ok."""
    import json
    import runpy
    import sys
    monkeypatch.setattr(sys, "argv", ["bench_sim.py", "--R", "4", "--S", "64", "--E", "16", "--H", "32",
                                      "--K", "4", "--maxvio", "0,2"])
    runpy.run_path("benchmarks/bench_sim.py", run_name="__main__")
    lines = [json.loads(line) for line in capsys.readouterr().out.strip().splitlines()]
    assert len(lines) == 2 and all(rec["ok"] and rec["rows_per_rank"] == 64 * 4 for rec in lines)
