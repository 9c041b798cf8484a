"""A small MoE decoder stack for end-to-end training runs: token embedding, N pre-norm blocks of
(causal self-attention, MoE FFN), final norm, LM head, cross-entropy.

The reference contains no model (it is a communication library; its README only reports a
normalised end-to-end figure from a harness that is not in the repository,
figure/e2e_vs_deepep.png).  This stack exists so that the expert-parallel path can be timed inside
a real training step against the conventional NCCL all-to-all path with no redundant experts.
Attention, norms, embedding and the loss are ordinary PyTorch (they are not part of the MoE
path); the MoE FFN is ``MoELayer`` (peer-memory dispatch/combine + tcgen05 grouped GEMM) or
``NcclMoELayer`` (all_to_all_single + permute around the same GEMM kernels).

Parallelism: EP for the experts; everything else is replicated, so dense gradients are averaged
over the group with one flat NCCL all-reduce (the reference leaves that to the host framework,
README.md:67).
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist
import torch.nn as nn
import torch.nn.functional as F

from ..ops import elementwise as ew
from ..ops import gemm
from ..parallel.nccl_baseline import NcclAllToAllEP
from .moe_layer import MoELayer


class _NcclMoEFn(torch.autograd.Function):
    """MoE FFN over the NCCL exchange: every expert is computed on its home rank."""

    @staticmethod
    def forward(ctx, x, layer):
        ep: NcclAllToAllEP = layer.ep
        K, epn, tp = ep.K, ep.epn, layer.token_padding
        logits = gemm.dense(x, layer.w_router)
        topk, w, _ = ew.router_topk(logits, K, layer.router_bias)
        rows, w_rows, st = ep.dispatch(x, topk, w)
        # pad every local expert's rows to a multiple of token_padding (zeros) for the GEMMs
        counts = torch.diff(st.cu_seqlens.long(), prepend=st.cu_seqlens.new_zeros(1).long())
        padded = (counts + tp - 1) // tp * tp
        cu_pad = padded.cumsum(0)
        n_pad = int(cu_pad[-1])                                     # host sync, as the exchange has
        start_pad = cu_pad - padded
        start_raw = st.cu_seqlens.long() - counts
        grp = torch.repeat_interleave(torch.arange(epn, device=x.device), counts)
        pos = torch.arange(st.rows, device=x.device) - start_raw[grp] + start_pad[grp]
        hidden = x.new_zeros(n_pad, x.shape[1])
        hidden.index_copy_(0, pos, rows)
        w_pad = torch.zeros(n_pad, dtype=torch.float32, device=x.device)
        w_pad.index_copy_(0, pos, w_rows)
        cu = cu_pad.to(torch.int32)
        act, gate, up = gemm.gateup_swiglu(hidden, layer.w_gate, layer.w_up, cu, row_scale=w_pad)
        y_pad = gemm.down(act, layer.w_down, cu)
        y = ep.combine(y_pad.index_select(0, pos), st)
        ctx.layer, ctx.st = layer, st
        ctx.save_for_backward(x, hidden, w_pad, cu, act, gate, up, topk, w, pos)
        return y

    @staticmethod
    def backward(ctx, dy):
        layer, st = ctx.layer, ctx.st
        ep: NcclAllToAllEP = layer.ep
        x, hidden, w_pad, cu, act, gate, up, topk, w, pos = ctx.saved_tensors
        K = ep.K
        # backward of combine: send dy of every (token, k) entry to the rank that computed it
        send = dy.contiguous()[st.order // K]
        recv = torch.empty(st.rows, dy.shape[1], dtype=dy.dtype, device=dy.device)
        dist.all_to_all_single(recv, send, st.recv_counts, st.send_counts, group=ep.group)
        d_out = dy.new_zeros(hidden.shape[0], dy.shape[1])
        d_out.index_copy_(0, pos, recv[st.group_order])
        d_act = gemm.down_dgrad(d_out, layer.w_down, cu)
        acc = layer.accumulate_grads
        gemm.wgrad(d_out, act, cu, layer.g_down, accumulate=acc)
        d_gate, d_up, d_scale = ew.swiglu_bwd(d_act, gate, up, w_pad, rows_ptr=cu[-1:])
        gemm.wgrad(hidden, d_gate, cu, layer.g_gate, accumulate=acc)
        gemm.wgrad(hidden, d_up, cu, layer.g_up, accumulate=acc)
        dx_pad = gemm.gateup_dgrad(d_gate, d_up, layer.w_gate, layer.w_up, cu)
        # backward of dispatch: return the rows (and the route-weight grads) to their sources
        inv = torch.empty_like(st.group_order)
        inv[st.group_order] = torch.arange(st.rows, device=dy.device)
        back = torch.empty(ep.S * K, dy.shape[1], dtype=dy.dtype, device=dy.device)
        dist.all_to_all_single(back, dx_pad.index_select(0, pos)[inv], st.send_counts, st.recv_counts,
                               group=ep.group)
        dwb = torch.empty(ep.S * K, dtype=torch.float32, device=dy.device)
        dist.all_to_all_single(dwb, d_scale.index_select(0, pos)[inv], st.send_counts, st.recv_counts,
                               group=ep.group)
        dx = torch.zeros(ep.S, dy.shape[1], dtype=torch.float32, device=dy.device)
        dx.index_add_(0, st.order // K, back.float())
        dw_sk = torch.empty(ep.S * K, dtype=torch.float32, device=dy.device)
        dw_sk[st.order] = dwb
        d_logits = ew.router_topk_bwd(w, dw_sk.view(ep.S, K), topk, ep.E)
        gemm.wgrad(x, d_logits, None, layer.g_router, accumulate=acc)
        dx = dx.to(dy.dtype) + gemm.dense(d_logits, layer.w_router, b_is_kn=False, out_dtype=torch.bfloat16)
        return dx, None


class NcclMoELayer:
    """Baseline MoE layer: same parameters and kernels as ``MoELayer``, NCCL exchange, no
    redundant experts (a hot expert overloads its home rank)."""

    def __init__(self, S, H, K, E, Hp, group=None, *, seed=0, router_bias=None, init_std=0.02,
                 token_padding=128):
        self.ep = NcclAllToAllEP(S, H, K, E, group)
        self.token_padding = token_padding
        self.Hp, self.training, self.accumulate_grads = Hp, True, False
        dev = torch.device("cuda", torch.cuda.current_device())
        epn = self.ep.epn
        g = torch.Generator(device=dev).manual_seed(seed * 7919 + 13)
        ge = torch.Generator(device=dev).manual_seed(seed * 7919 + 101 + self.ep.rank)
        rnd = lambda gen, *s: (torch.randn(*s, device=dev, generator=gen) * init_std).bfloat16()
        self.w_router = rnd(g, H, E)
        self.w_gate, self.w_up, self.w_down = rnd(ge, epn, H, Hp), rnd(ge, epn, H, Hp), rnd(ge, epn, H, Hp)
        self.router_bias = router_bias
        z = lambda *s: torch.zeros(*s, dtype=torch.float32, device=dev)
        self.g_router = z(1, H, E)
        self.g_gate, self.g_up, self.g_down = z(epn, H, Hp), z(epn, H, Hp), z(epn, H, Hp)
        self.max_rows = 0

    def __call__(self, x):
        return _NcclMoEFn.apply(x.contiguous(), self)

    def sgd_step(self, lr):
        ew.sgd_update_(self.w_router, self.g_router[0], lr)
        ew.sgd_update_(self.w_gate, self.g_gate, lr)
        ew.sgd_update_(self.w_up, self.g_up, lr)
        ew.sgd_update_(self.w_down, self.g_down, lr)


class RMSNorm(nn.Module):
    def __init__(self, dim, eps=1e-6):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(dim, dtype=torch.bfloat16))
        self.eps = eps

    def forward(self, x):
        return F.rms_norm(x, (x.shape[-1],), self.weight, self.eps)


class Block(nn.Module):
    def __init__(self, hidden, n_heads, moe):
        super().__init__()
        self.n_heads = n_heads
        self.norm1, self.norm2 = RMSNorm(hidden), RMSNorm(hidden)
        self.qkv = nn.Linear(hidden, 3 * hidden, bias=False, dtype=torch.bfloat16)
        self.proj = nn.Linear(hidden, hidden, bias=False, dtype=torch.bfloat16)
        self.moe = moe                      # not an nn.Module: it owns its own params and grads

    def forward(self, x):                   # x [S, hidden], one sequence per rank
        S, Hd = x.shape
        q, k, v = self.qkv(self.norm1(x)).view(S, 3, self.n_heads, Hd // self.n_heads).unbind(1)
        a = F.scaled_dot_product_attention(q.transpose(0, 1)[None], k.transpose(0, 1)[None],
                                           v.transpose(0, 1)[None], is_causal=True)
        x = x + self.proj(a[0].transpose(0, 1).reshape(S, Hd))
        return x + self.moe(self.norm2(x))


class MoEDecoder(nn.Module):
    """``moe_factory(layer_index)`` builds the MoE FFN of each block (``MoELayer`` or
    ``NcclMoELayer``)."""

    def __init__(self, vocab, hidden, n_layers, n_heads, moe_factory, group=None):
        super().__init__()
        self.group = group
        self.embed = nn.Embedding(vocab, hidden, dtype=torch.bfloat16)
        self.blocks = nn.ModuleList([Block(hidden, n_heads, moe_factory(i)) for i in range(n_layers)])
        self.norm = RMSNorm(hidden)
        self.head = nn.Linear(hidden, vocab, bias=False, dtype=torch.bfloat16)
        for p in self.parameters():
            if p.dim() > 1:
                nn.init.normal_(p, std=0.02)

    def forward(self, tokens, targets):
        x = self.embed(tokens)
        for b in self.blocks:
            x = b(x)
        logits = self.head(self.norm(x))
        return F.cross_entropy(logits.float(), targets)

    def moe_layers(self):
        return [b.moe for b in self.blocks]

    def train_step(self, tokens, targets, lr, fuse_expert_sgd: bool = False):
        """forward + backward + all-reduce of the replicated parameters' grads (dense layers and
        the MoE routers) + SGD on everything; returns the loss.  ``fuse_expert_sgd`` applies the
        expert weights' SGD step inside the weight-grad kernels (``MoELayer.fuse_sgd``)."""
        for m in self.moe_layers():
            if hasattr(m, "fuse_sgd"):
                m.fuse_sgd(lr if fuse_expert_sgd else None)
        loss = self(tokens, targets)
        loss.backward()
        dense = [p for p in self.parameters() if p.grad is not None]
        R = dist.get_world_size(self.group) if dist.is_initialized() else 1
        if R > 1:
            flat = torch.cat([p.grad.reshape(-1) for p in dense])
            dist.all_reduce(flat, group=self.group)
            flat.div_(R)
            off = 0
            for p in dense:
                n = p.numel()
                p.grad.copy_(flat[off:off + n].view_as(p))
                off += n
            # the routers are replicated too (same seed on every rank): average their fp32 grads
            routers = [m.g_router for m in self.moe_layers()]
            rflat = torch.cat([g.reshape(-1) for g in routers])
            dist.all_reduce(rflat, group=self.group)
            rflat.div_(R)
            off = 0
            for g in routers:
                g.copy_(rflat[off:off + g.numel()].view_as(g))
                off += g.numel()
        with torch.no_grad():
            for p in dense:
                p.add_(p.grad, alpha=-lr)
                p.grad = None
        for m in self.moe_layers():
            m.sgd_step(lr)
        return loss

    def state_dict_all(self):
        """Dense parameters plus every MoE layer's home-layout expert weights."""
        sd = {k: v.detach().cpu() for k, v in self.state_dict().items()}
        for i, m in enumerate(self.moe_layers()):
            for k, v in (("router", m.w_router), ("gate", m.w_gate), ("up", m.w_up), ("down", m.w_down)):
                sd[f"moe.{i}.{k}"] = v.detach().cpu()
        return sd

    def load_state_dict_all(self, sd):
        self.load_state_dict({k: v for k, v in sd.items() if not k.startswith("moe.")})
        for i, m in enumerate(self.moe_layers()):
            for k, v in (("router", m.w_router), ("gate", m.w_gate), ("up", m.w_up), ("down", m.w_down)):
                v.copy_(sd[f"moe.{i}.{k}"].to(v.device))
