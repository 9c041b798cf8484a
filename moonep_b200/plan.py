"""``CommPlan``: the state that links a forward dispatch to prefetch, combine and both
backward passes.  Field-for-field counterpart of the reference's ``MoonEPCommPlan``
(moonep/planning.py:31-86), plus ``link``: the per-slot duplicate chains this
implementation uses in place of the reference's atomics-built dedup arrays.  The
reference-shaped ``dup_groups`` / ``dup_loffs`` / ``dup_counts`` views are derived from
``link`` on demand and, unlike the reference's, come out in a deterministic order.
"""
from __future__ import annotations

from dataclasses import dataclass, field, replace
from typing import Optional

import torch

LINK_NONE = 0x00FFFFFF
LINK_DUP_BIT = 0x40000000
LINK_NEXT_MASK = 0x00FFFFFF


@dataclass(frozen=True)
class CommPlan:
    dst: torch.Tensor               # [N] int32, canonical destinations (negative = duplicate)
    experts_to_copy: torch.Tensor   # [R, epn] int32, replicated on every rank
    zero_fill_ranges: torch.Tensor  # [2*epn, 2] int32
    remote_stats: torch.Tensor      # [2] int32
    cu_seqlens: torch.Tensor        # [2*epn] int32 padded group END rows
    link: torch.Tensor              # [NvS] int32 duplicate chains of MY received rows
    N: int
    R: int
    E: int
    NvS: int
    K: int
    src_info: Optional[torch.Tensor] = None   # [NvS] int32: owner entry of every received row
    # [N] int32: this rank's entries in the order in which the fused dispatch -> GEMM path sends
    # them (by local expert index, then home rank rotated by this rank, then token)
    send_order: Optional[torch.Tensor] = None
    _dedup_cache: dict = field(default_factory=dict, compare=False, repr=False)

    def clone(self) -> "CommPlan":
        return replace(
            self,
            dst=self.dst.clone(),
            experts_to_copy=self.experts_to_copy.clone(),
            zero_fill_ranges=self.zero_fill_ranges.clone(),
            remote_stats=self.remote_stats.clone(),
            cu_seqlens=self.cu_seqlens.clone(),
            link=self.link.clone(),
            src_info=None if self.src_info is None else self.src_info.clone(),
            send_order=None if self.send_order is None else self.send_order.clone(),
            _dedup_cache={},
        )

    # ---- reference-shaped dedup views ---------------------------------------------------
    def _real_row_mask(self) -> torch.Tensor:
        """Boolean [NvS]: rows that hold a dispatched entry (not padding, not the tail)."""
        epn2 = self.cu_seqlens.numel()
        cu = self.cu_seqlens.to(torch.int64)
        starts = torch.cat([cu.new_zeros(1), cu[:-1]])
        zf = self.zero_fill_ranges.to(torch.int64)
        ends = torch.where(zf[:, 1] > 0, zf[:, 0], cu)
        rows = torch.arange(self.NvS, device=cu.device)
        grp = torch.bucketize(rows, cu, right=True).clamp_(max=epn2 - 1)
        return (rows >= starts[grp]) & (rows < ends[grp]) & (rows < cu[-1])

    def _build_dedup(self):
        if "groups" in self._dedup_cache:
            return
        link = self.link.to(torch.int64)
        real = self._real_row_mask()
        nxt = link & LINK_NEXT_MASK
        is_dup = (link & LINK_DUP_BIT) != 0
        prim = real & ~is_dup & (nxt != LINK_NONE)
        prim_rows = torch.nonzero(prim).flatten()
        groups = torch.zeros(self.NvS, 3, dtype=torch.int32, device=link.device)
        loffs = torch.zeros(self.NvS, dtype=torch.int32, device=link.device)
        chains = []
        cur = nxt[prim_rows]
        alive = torch.ones_like(cur, dtype=torch.bool)
        for _ in range(self.K):
            alive = alive & (cur != LINK_NONE)
            if not bool(alive.any()):
                break
            chains.append(torch.where(alive, cur, cur.new_full((), -1)))
            cur = torch.where(alive, nxt[cur.clamp(max=self.NvS - 1)], cur)
        if chains:
            mat = torch.stack(chains, dim=1)             # [G, depth], -1 = past the end
            counts = (mat >= 0).sum(dim=1)
            startv = torch.cumsum(counts, 0) - counts
            flat = mat[mat >= 0]
            loffs[: flat.numel()] = flat.to(torch.int32)
            g = prim_rows.numel()
            groups[:g, 0] = prim_rows.to(torch.int32)
            groups[:g, 1] = startv.to(torch.int32)
            groups[:g, 2] = counts.to(torch.int32)
            cnt = torch.tensor([g, int(flat.numel())], dtype=torch.int32, device=link.device)
        else:
            cnt = torch.zeros(2, dtype=torch.int32, device=link.device)
        self._dedup_cache.update(groups=groups, loffs=loffs, counts=cnt)

    @property
    def dup_groups(self) -> torch.Tensor:
        """[NvS, 3] (primary row, start in ``dup_loffs``, n duplicates); compact prefix valid."""
        self._build_dedup()
        return self._dedup_cache["groups"]

    @property
    def dup_loffs(self) -> torch.Tensor:
        self._build_dedup()
        return self._dedup_cache["loffs"]

    @property
    def dup_counts(self) -> torch.Tensor:
        """[2] (number of groups, number of duplicate rows)."""
        self._build_dedup()
        return self._dedup_cache["counts"]


def plan_num_rows(plan: CommPlan) -> Optional[int]:
    """Rows of the padded layout (``cu_seqlens[-1]``); forces a device sync on CUDA."""
    return int(plan.cu_seqlens[-1].item())
