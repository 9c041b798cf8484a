"""Property tests of the planner oracle and the multi-rank simulator (CPU, hypothesis).

Random shapes and adversarial routings (repeated experts inside a token, everything on one
expert, a single hot home group) must keep the guarantees every kernel relies on: exactly S*K
rows per rank, at most epn prefetch slots taken from ONE remote home group, a bijection between
entries and occupied rows, and ``combine(dispatch(x)) == sum_k w_k * x`` through the simulator."""
from dataclasses import dataclass

import torch
from hypothesis import HealthCheck, given, settings
from hypothesis import strategies as st

from moonep_b200 import reference as ref
from tests.test_planner_oracle import check_plan


@dataclass(frozen=True)
class _Shape:
    S: int
    K: int
    epn: int
    token_padding: int


@st.composite
def problems(draw):
    R = draw(st.sampled_from([1, 2, 3, 4, 8]))
    epn = draw(st.integers(1, 5))
    E = R * epn
    K = draw(st.integers(1, min(6, E)))
    S = draw(st.integers(1, 24))
    tp = draw(st.sampled_from([1, 2, 8, 16]))
    mode = draw(st.sampled_from(["uniform", "one_expert", "hot_group", "repeats"]))
    seed = draw(st.integers(0, 2 ** 16))
    g = torch.Generator().manual_seed(seed)
    if mode == "uniform":
        topk = torch.stack([torch.stack([torch.randperm(E, generator=g)[:K] for _ in range(S)]) for _ in range(R)])
    elif mode == "one_expert":
        topk = torch.full((R, S, K), int(torch.randint(E, (1,), generator=g)))
    elif mode == "hot_group":
        h = int(torch.randint(R, (1,), generator=g))
        topk = h * epn + torch.randint(epn, (R, S, K), generator=g)
    else:                                   # arbitrary, repeats allowed inside a token
        topk = torch.randint(E, (R, S, K), generator=g)
    return _Shape(S, K, epn, tp), R, topk.to(torch.int32)


@settings(max_examples=120, deadline=None, suppress_health_check=[HealthCheck.too_slow])
@given(problems())
def test_plan_invariants_hold_for_any_routing(problem):
    shape, R, topk = problem
    tables, dst = ref.plan_all_ranks(topk, shape.S, shape.K, shape.epn * R, shape.token_padding)
    check_plan(shape, R, tables, dst)


@settings(max_examples=40, deadline=None, suppress_health_check=[HealthCheck.too_slow])
@given(problems())
def test_simulated_round_trip_is_the_weighted_sum(problem):
    shape, R, topk = problem
    H = 8
    sim = ref.SimGroup(shape.S, H, shape.K, shape.epn * R, R, shape.token_padding)
    g = torch.Generator().manual_seed(1)
    x = torch.randn(R, shape.S, H, generator=g)
    w = torch.rand(R, shape.S, shape.K, generator=g)
    hidden, w_nvs, _, plans = sim.dispatch(x, w, topk)
    out, _ = sim.combine(plans, hidden * w_nvs[..., None])       # the "expert" multiplies by the weight
    want = x * w.sum(dim=2, keepdim=True)
    assert torch.allclose(out, want, atol=1e-5, rtol=1e-5)
