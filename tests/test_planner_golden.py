"""The CPU planner oracle (csrc/ref/plan_ref.cc) against golden vectors.

``tests/golden_plans.json`` holds, for a selection of the case list and R in {2, 4, 8}, a hash of
every plan field of every rank (dst, cu_seqlens, experts_to_copy, remote_stats, zero_fill) as the
reference's own CPU oracle (tests/planning_reference.py) computes them for the same inputs.  The
hashes are data, produced once; they pin what the invariants of test_planner_oracle.py cannot:
the tie-breaks of the greedy solver (arg-max ties to the smaller rank, ascending slot fill)."""
import hashlib
import json
import os

import pytest
import torch

from moonep_b200 import reference as ref
from tests.cases import CASES

GOLD = json.load(open(os.path.join(os.path.dirname(__file__), "golden_plans.json")))["plans"]


def _h(t):
    return hashlib.sha256(t.to(torch.int32).contiguous().numpy().tobytes()).hexdigest()[:16]


@pytest.mark.parametrize("key", sorted(GOLD))
def test_oracle_reproduces_golden_plan(key):
    name, r_txt = key.rsplit("-R", 1)
    R = int(r_txt)
    c = next(c for c in CASES if c.name == name)
    topk, tpe = c.topk_all(R)
    tables, dst = ref.plan_all_ranks(topk, c.S, c.K, c.epn * R, c.token_padding, tpe)
    assert len(GOLD[key]) == R
    for r, want in enumerate(GOLD[key]):
        got = dict(dst=_h(dst[r]), cu_seqlens=_h(tables.cu_seqlens[r]),
                   experts_to_copy=_h(tables.experts_to_copy), remote_stats=_h(tables.remote_stats[r]),
                   zero_fill=_h(tables.zero_fill[r]))
        assert got == want, f"rank {r}"


def test_golden_set_covers_ties_and_skew():
    names = {k.rsplit("-R", 1)[0] for k in GOLD}
    assert {"balanced_epn16", "duplicate_topk", "near_degenerate_bias", "all_remote"} <= names
    assert len(GOLD) >= 30
