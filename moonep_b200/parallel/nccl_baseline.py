"""The conventional expert-parallel exchange, used as the baseline the fused path is measured
against: sort the (token, k) entries by expert, exchange counts, ``all_to_all_single`` the rows
over NCCL, and undo it after the experts ran.  No redundant experts: every expert is computed on
its home rank, so a hot expert overloads that rank (and its receive buffer grows with the skew,
which is what makes the reference's competitor run out of memory at high MaxVio,
figure/e2e_vs_deepep.png)."""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.distributed as dist


@dataclass
class A2AState:
    order: torch.Tensor          # [N] entry indices sorted by expert
    send_counts: list
    recv_counts: list
    recv_tpe: torch.Tensor       # [R, epn] rows per (source rank, local expert)
    group_order: torch.Tensor    # [rows] permutation that makes received rows expert-major
    cu_seqlens: torch.Tensor     # [epn] END row of each local expert (unpadded)
    rows: int


class NcclAllToAllEP:
    def __init__(self, S, H, K, E, group=None):
        self.group = group if group is not None else dist.group.WORLD
        self.R = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        self.S, self.H, self.K, self.E = S, H, K, E
        self.epn = E // self.R

    def dispatch(self, x, topk, weights=None):
        """x [S,H] bf16, topk [S,K] int -> (rows [n,H] expert-major, row weights [n] | None, state)."""
        R, epn, K = self.R, self.epn, self.K
        flat = topk.reshape(-1).long()
        order = torch.argsort(flat, stable=True)
        tpe = torch.bincount(flat, minlength=self.E)
        tpe_all = torch.empty(R, self.E, dtype=tpe.dtype, device=x.device)
        dist.all_gather_into_tensor(tpe_all, tpe, group=self.group)
        send_counts = tpe.view(R, epn).sum(1).tolist()                       # host sync, as usual
        recv_tpe = tpe_all[:, self.rank * epn:(self.rank + 1) * epn]          # [R, epn]
        recv_counts = recv_tpe.sum(1).tolist()
        rows = int(sum(recv_counts))
        send = x[order // K]
        recv = torch.empty(rows, self.H, dtype=x.dtype, device=x.device)
        dist.all_to_all_single(recv, send, recv_counts, send_counts, group=self.group)
        # received rows are (source rank, expert)-major; make them expert-major for the GEMM
        src = torch.arange(R, device=x.device).repeat_interleave(epn)
        exp = torch.arange(epn, device=x.device).repeat(R)
        seg_expert = torch.repeat_interleave(exp, recv_tpe.reshape(-1))
        group_order = torch.argsort(seg_expert, stable=True)
        cu = recv_tpe.sum(0).cumsum(0).to(torch.int32)
        wrecv = None
        if weights is not None:
            wsend = weights.reshape(-1)[order]
            wrecv = torch.empty(rows, dtype=weights.dtype, device=x.device)
            dist.all_to_all_single(wrecv, wsend, recv_counts, send_counts, group=self.group)
            wrecv = wrecv[group_order]
        st = A2AState(order, send_counts, recv_counts, recv_tpe, group_order, cu, rows)
        return recv[group_order], wrecv, st

    def combine(self, y, st: A2AState):
        """y [rows,H] expert-major -> [S,H]: reverse exchange and sum the K copies in fp32."""
        inv = torch.empty_like(st.group_order)
        inv[st.group_order] = torch.arange(st.rows, device=y.device)
        back = torch.empty(self.S * self.K, self.H, dtype=y.dtype, device=y.device)
        dist.all_to_all_single(back, y[inv], st.send_counts, st.recv_counts, group=self.group)
        out = torch.zeros(self.S, self.H, dtype=torch.float32, device=y.device)
        out.index_add_(0, st.order // self.K, back.float())
        return out.to(y.dtype)
