"""CPU oracle and multi-rank simulator (native C++, ``csrc/ref``), wrapped for torch CPU tensors.

The reference can only be exercised on real GPUs under torchrun (tests/conftest.py:16-33); its
oracle is a Python-loop torch function that needs a process group to see other ranks
(tests/planning_reference.py:44-52).  This module runs all ranks in one process with no GPU:
``plan_all_ranks`` solves the plan, ``SimGroup`` dispatches and combines through plain arrays
that stand in for peer memory.  The same functions are the oracle the CUDA kernels are tested
against.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from . import _native as nat
from ._native import I, L, P
from .plan import CommPlan

nat.declare("mep_ref_plan_solve", I, [P, I, I, I, I, I, L, P, P, P, P, P, P, P, P])
nat.declare("mep_ref_plan_assign", I, [I, P, I, I, I, I, L, P, P, P, P])
nat.declare("mep_sim_dispatch", I, [P, P, P, P, I, I, I, I, I, L, I, P, P, P, I])
nat.declare("mep_sim_combine", I, [P, P, P, P, I, I, I, I, L, I, I, P, P])


def nvs_rows(S: int, K: int, epn: int, token_padding: int) -> int:
    """Rows of the static per-rank dispatch buffer (moonep/api.py:265-266)."""
    raw = S * K + (token_padding - 1) * 2 * epn
    return (raw + token_padding - 1) // token_padding * token_padding


@dataclass
class PlanTables:
    """Everything the solver produces, for all ranks."""
    tpe_cumsum: torch.Tensor       # [R, E]
    alloc: torch.Tensor            # [E, R]
    alloc_cumsum: torch.Tensor     # [E, R]
    expert_off: torch.Tensor       # [R, E]
    cu_seqlens: torch.Tensor       # [R, 2epn]
    zero_fill: torch.Tensor        # [R, 2epn, 2]
    experts_to_copy: torch.Tensor  # [R, epn]
    remote_stats: torch.Tensor     # [R, 2]


def _i32(t: torch.Tensor) -> torch.Tensor:
    return t.detach().to("cpu", torch.int32).contiguous()


def solve_tables(tpe_all: torch.Tensor, S: int, K: int, token_padding: int) -> PlanTables:
    """Planner steps 1-4 for all ranks from the gathered ``tpe[R, E]``."""
    tpe_all = _i32(tpe_all)
    R, E = tpe_all.shape
    epn = E // R
    NvS = nvs_rows(S, K, epn, token_padding)
    z = lambda *s: torch.zeros(*s, dtype=torch.int32)
    t = PlanTables(z(R, E), z(E, R), z(E, R), z(R, E), z(R, 2 * epn), z(R, 2 * epn, 2),
                   z(R, epn), z(R, 2))
    rc = nat.call("mep_ref_plan_solve", tpe_all.data_ptr(), R, E, S, K, token_padding, NvS,
                  t.tpe_cumsum.data_ptr(), t.alloc.data_ptr(), t.alloc_cumsum.data_ptr(),
                  t.expert_off.data_ptr(), t.cu_seqlens.data_ptr(), t.zero_fill.data_ptr(),
                  t.experts_to_copy.data_ptr(), t.remote_stats.data_ptr())
    if rc != 0:
        raise AssertionError(f"planner oracle: invariant violated (code {rc})")
    return t


def assign_dst(rank: int, topk: torch.Tensor, tables: PlanTables, S: int, K: int,
               token_padding: int) -> torch.Tensor:
    """Planner steps 5-6: canonical ``dst[N]`` of one source rank."""
    topk = _i32(topk).reshape(-1)
    R, E = tables.tpe_cumsum.shape
    NvS = nvs_rows(S, K, E // R, token_padding)
    dst = torch.zeros(S * K, dtype=torch.int32)
    rc = nat.call("mep_ref_plan_assign", rank, topk.data_ptr(), R, E, S, K, NvS,
                  tables.tpe_cumsum.data_ptr(), tables.alloc_cumsum.data_ptr(),
                  tables.expert_off.data_ptr(), dst.data_ptr())
    if rc != 0:
        raise AssertionError(f"planner oracle: assignment failed (code {rc})")
    return dst


def plan_all_ranks(topk_all: torch.Tensor, S: int, K: int, E: int, token_padding: int,
                   tpe_all: torch.Tensor | None = None):
    """Plans of all ranks.  ``topk_all`` is ``[R, S, K]``.  Returns ``(tables, dst[R, N])``."""
    topk_all = _i32(topk_all)
    R = topk_all.shape[0]
    if tpe_all is None:
        tpe_all = torch.stack([torch.bincount(topk_all[r].flatten().long(), minlength=E)
                               for r in range(R)]).to(torch.int32)
    tables = solve_tables(tpe_all, S, K, token_padding)
    dst = torch.stack([assign_dst(r, topk_all[r], tables, S, K, token_padding)
                       for r in range(R)])
    return tables, dst


class SimGroup:
    """R simulated ranks in one process: the GPU-less engine.

    ``dispatch`` returns per-rank ``hidden[R, NvS, H]``, ``weights[R, NvS]``, the per-rank
    ``CommPlan`` list and ``cu_seqlens[R, 2epn]``; ``combine`` returns ``out[R, S, H]`` and the
    gathered weights ``[R, S, K]``.  Tensors are fp32 or bf16 on the CPU.
    """

    def __init__(self, S: int, H: int, K: int, E: int, R: int, token_padding: int = 128):
        assert E % R == 0 and min(S, H, K, E, R, token_padding) > 0
        self.S, self.H, self.K, self.E, self.R = S, H, K, E, R
        self.token_padding = token_padding
        self.epn = E // R
        self.NvS = nvs_rows(S, K, self.epn, token_padding)

    def plan(self, topk_all: torch.Tensor):
        tables, dst = plan_all_ranks(topk_all, self.S, self.K, self.E, self.token_padding)
        return tables, dst

    def dispatch(self, x_all, w_all, topk_all, *, expand=True, poison=None):
        R, S, K, H, NvS = self.R, self.S, self.K, self.H, self.NvS
        assert x_all.shape == (R, S, H) and x_all.dtype in (torch.float32, torch.bfloat16)
        tables, dst = self.plan(topk_all)
        x_all = x_all.contiguous()
        hidden = torch.zeros(R, NvS, H, dtype=x_all.dtype)
        w_nvs = torch.zeros(R, NvS, dtype=torch.float32)
        if poison is not None:
            hidden.fill_(poison)
            w_nvs.fill_(poison)
        link = torch.full((R, NvS), 0x00FFFFFF, dtype=torch.int32)
        w_c = None if w_all is None else w_all.to(torch.float32).contiguous()
        rc = nat.call("mep_sim_dispatch", x_all.data_ptr(), nat.ptr(w_c), dst.data_ptr(),
                      tables.zero_fill.data_ptr(), R, S, K, H, self.epn, NvS,
                      x_all.element_size(), hidden.data_ptr(),
                      w_nvs.data_ptr() if w_c is not None else 0, link.data_ptr(),
                      1 if expand else 0)
        if rc != 0:
            raise AssertionError(f"simulated dispatch failed (code {rc})")
        plans = [CommPlan(dst=dst[r], experts_to_copy=tables.experts_to_copy,
                          zero_fill_ranges=tables.zero_fill[r], remote_stats=tables.remote_stats[r],
                          cu_seqlens=tables.cu_seqlens[r], link=link[r], N=S * K, R=R, E=self.E,
                          NvS=NvS, K=K) for r in range(R)]
        return hidden, (w_nvs if w_c is not None else None), tables.cu_seqlens, plans

    def combine(self, plans, hidden, w_nvs=None, *, prologue=True):
        R, S, K, H, NvS = self.R, self.S, self.K, self.H, self.NvS
        hidden = hidden.contiguous().clone()
        dst = torch.stack([p.dst for p in plans]).contiguous()
        link = torch.stack([p.link for p in plans]).contiguous()
        out = torch.zeros(R, S, H, dtype=hidden.dtype)
        w_out = torch.zeros(R, S, K, dtype=torch.float32) if w_nvs is not None else None
        wn = None if w_nvs is None else w_nvs.contiguous()
        rc = nat.call("mep_sim_combine", hidden.data_ptr(), nat.ptr(wn), dst.data_ptr(),
                      link.data_ptr(), R, S, K, H, NvS, hidden.element_size(),
                      1 if prologue else 0, out.data_ptr(), nat.ptr(w_out))
        if rc != 0:
            raise AssertionError(f"simulated combine failed (code {rc})")
        return out, w_out
