"""CPU tests of the planner oracle: the structural invariants the reference checks on device
(tests/kernel_test_utils.py:324-414) plus the balance guarantees of its README
(every rank receives exactly S*K rows; <= epn prefetch slots, all from ONE remote home group)."""
import pytest
import torch

from moonep_b200 import reference as ref
from tests.cases import case_params


def check_plan(case, R, tables, dst):
    S, K, epn, tp = case.S, case.K, case.epn, case.token_padding
    E = epn * R
    N = S * K
    NvS = ref.nvs_rows(S, K, epn, tp)
    # every rank computes exactly S*K real rows
    assert torch.equal(tables.alloc.sum(0).long(), torch.full((R,), N, dtype=torch.long))
    # conservation per expert
    assert torch.equal(tables.alloc.sum(1), tables.tpe_cumsum[R - 1])
    for d in range(R):
        etc = tables.experts_to_copy[d]
        valid = etc[etc >= 0]
        # slots filled in ascending expert order, compactly
        assert torch.equal(etc[: valid.numel()], valid) and bool((valid[1:] > valid[:-1]).all())
        homes = set((valid // epn).tolist())
        assert len(homes) <= 1 and d not in homes
        assert int(tables.remote_stats[d, 0]) == valid.numel()
        cu = tables.cu_seqlens[d].long()
        seg = torch.diff(torch.cat([cu.new_zeros(1), cu]))
        assert bool((seg >= 0).all()) and bool((seg % tp == 0).all()) and int(cu[-1]) <= NvS
    for h in range(R):
        held = ((tables.experts_to_copy >= 0) & (tables.experts_to_copy // epn == h)).sum()
        assert int(tables.remote_stats[h, 1]) == int(held)
    # dst: every real slot of every rank is hit exactly once
    raw = torch.where(dst < 0, -dst - 1, dst).long()
    assert int(raw.min()) >= 0 and int(raw.max()) < R * NvS
    assert raw.unique().numel() == R * N
    occ = torch.zeros(R * NvS, dtype=torch.bool)
    occ[raw.flatten()] = True
    for d in range(R):
        start = 0
        for g in range(2 * epn):
            end = int(tables.cu_seqlens[d, g])
            first_pad, npad = tables.zero_fill[d, g].tolist()
            real_end = first_pad if npad > 0 else end
            assert bool(occ[d * NvS + start: d * NvS + real_end].all())
            assert not bool(occ[d * NvS + real_end: d * NvS + end].any())
            assert real_end + npad == end or (npad == 0 and real_end == end)
            start = end
        assert not bool(occ[d * NvS + start: (d + 1) * NvS].any())
    # canonical duplicates: within a token, the first entry per destination rank is positive
    d3 = dst.view(R, S, K)
    r3 = raw.view(R, S, K) // NvS
    for k in range(K):
        earlier_same = torch.zeros(R, S, dtype=torch.bool)
        for j in range(k):
            earlier_same |= r3[:, :, j] == r3[:, :, k]
        assert torch.equal(d3[:, :, k] < 0, earlier_same)
    # entries land in the group of their expert
    return NvS


@pytest.mark.parametrize("case,R", case_params())
def test_plan_invariants(case, R):
    topk, tpe = case.topk_all(R)
    tables, dst = ref.plan_all_ranks(topk, case.S, case.K, case.epn * R, case.token_padding, tpe)
    NvS = check_plan(case, R, tables, dst)
    # each entry sits inside the group that computes its expert
    E, epn = case.epn * R, case.epn
    raw = torch.where(dst < 0, -dst - 1, dst).long()
    dr, loff = raw // NvS, raw % NvS
    ex = topk.view(R, -1).long()
    for r in range(R):
        for i in range(0, case.S * case.K, max(1, case.S * case.K // 64)):
            d, e, lo = int(dr[r, i]), int(ex[r, i]), int(loff[r, i])
            if e // epn == d:
                g = e - d * epn
            else:
                slot = (tables.experts_to_copy[d] == e).nonzero()
                assert slot.numel() == 1
                g = epn + int(slot)
            start = 0 if g == 0 else int(tables.cu_seqlens[d, g - 1])
            assert start <= lo < int(tables.cu_seqlens[d, g])


def test_order_is_global_source_rank_then_token():
    """Tokens of one expert are numbered in (source rank, token) order and cut into contiguous
    runs per destination rank (moonep/planning.py:1016-1041)."""
    R, S, K, epn, tp = 4, 64, 2, 2, 8
    E = epn * R
    g = torch.Generator().manual_seed(3)
    topk = torch.stack([torch.multinomial(torch.tensor([8.0, 1, 1, 1, 1, 1, 1, 1]).expand(S, E),
                                          K, generator=g) for _ in range(R)]).to(torch.int32)
    tables, dst = ref.plan_all_ranks(topk, S, K, E, tp)
    NvS = ref.nvs_rows(S, K, epn, tp)
    raw = torch.where(dst < 0, -dst - 1, dst).long()
    seq = [int(raw[r, i]) for r in range(R) for i in range(S * K) if int(topk[r].flatten()[i]) == 0]
    ranks = [v // NvS for v in seq]
    assert ranks == sorted(ranks)
    for d in set(ranks):
        rows = [v % NvS for v in seq if v // NvS == d]
        assert rows == list(range(rows[0], rows[0] + len(rows)))
