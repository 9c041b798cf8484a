"""Expert-parallel MoE layer (router -> dispatch -> SwiGLU experts -> combine) with a full
backward pass and an SGD step, built on ``Buffer`` and the tcgen05 grouped GEMM.

The reference stops at the communication API and describes the integration in prose
(README.md:43-156): the framework owns a ``[2*epn, H, H']`` compute view per projection (local
experts followed by this rank's prefetch slots), runs its grouped GEMM over the VM groups of
``cu_seqlens``, accumulates prefetch-slot weight grads in ``[R, epn, H, H']`` reduce buffers and
calls ``reduce_grad``.  This module is that integration:

forward   logits = x Wr -> top-k/softmax/histogram -> ``dispatch`` (fresh plan) ->
          ``prefetch_weight`` -> gate/up GEMM with fused SwiGLU x route weight -> down GEMM whose
          epilogue pushes every result row over NVLink to the token's home rank
          (``fused_combine``) -> ``combine_pushed`` (barrier + local K-sum); or, unfused, down
          GEMM into the Buffer's shard -> ``combine`` (zero copy)
backward  ``dispatch(plan=...)`` of dy -> down dgrad / wgrad -> SwiGLU backward (also yields the
          route-weight grads) -> gate/up wgrad and dgrad (into the shard) -> ``combine`` with the
          weight-gather path (returns d route weights as [S, K]) -> ``reduce_grad`` -> router
          backward.

Weights are bf16, weight grads fp32 ("main grads"), written by the GEMM epilogues.
"""
from __future__ import annotations

import os
from typing import Optional

import torch
import torch.distributed as dist

from .. import buffer as symm
from ..api import Buffer
from ..ops import elementwise as ew
from ..ops import gemm
from ..utils.trace import NULL_TRACER


class ExpertPools:
    """Process-global prefetch (bf16) and reduce (fp32) pools, ``[R, epn, H, H']`` each, mapped on
    every rank.  Shared by all MoE layers of a model (README.md:56-58).  ``None`` when R == 1."""

    def __init__(self, R: int, epn: int, H: int, Hp: int, group=None, rank: int = 0,
                 train: bool = True):
        self.R, self.epn, self.rank = R, epn, rank
        self.names = ("gate", "up", "down")
        self.prefetch = {}
        self.reduce = {}
        # the plan whose redundant experts' weights the prefetch slots hold right now.  Several
        # layers share the pools, so a layer's backward pass finds another layer's weights there
        # unless it was the last one to prefetch; it then prefetches again (see _MoEFn.backward)
        self.prefetch_owner = None
        if R == 1:
            return
        for n in self.names:
            t = symm.create_nvl_dist_tensor((epn, H, Hp), torch.bfloat16, group=group)
            self.prefetch[n] = t.view(R, t.shape[0] // R, H, Hp)[:, :epn]
            if train:
                g = symm.create_nvl_dist_tensor((epn, H, Hp), torch.float32, group=group)
                gv = g.view(R, g.shape[0] // R, H, Hp)[:, :epn]
                gv[rank].zero_()
                self.reduce[n] = gv
        torch.cuda.synchronize()
        dist.barrier(group=group)

    def slot(self, name):
        return self.prefetch[name][self.rank] if self.prefetch else None

    def grad_slot(self, name):
        return self.reduce[name][self.rank] if self.reduce else None


class _MoEFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, layer):
        buf: Buffer = layer.buf
        epn = buf.epn
        tr = layer.tracer
        with tr.span("f.router"):
            logits = gemm.dense(x, layer.w_router)                         # [S, E] fp32
            topk, w, tpe = ew.router_topk(logits, buf.K, layer.router_bias)
        fused = layer.fused_dispatch
        disp = None
        with tr.span("f.dispatch"):
            shard = 1 if layer.hidden_in_place else 0
            if layer.hidden_in_place and ctx.needs_input_grad[0]:
                buf.claim_second_shard(layer)      # rows stay in the second shard until backward has used them
            if fused:
                # only the plan is made here: the rows travel inside the gate/up GEMM launch below
                hidden, w_nvs, cu, plan, disp = buf.dispatch_fused_begin(x, w, topk, tpe, shard=shard)
            elif layer.hidden_in_place:
                hidden, w_nvs, cu, plan = buf.dispatch(x, w, topk, tpe, zero_copy=True, shard=1)
            else:
                hidden, w_nvs, cu, plan = buf.dispatch(x, w, topk, tpe)
        wait_only = None if disp is None else dict(disp, mode=1)
        pools = layer.pools
        if pools is not None and pools.prefetch:
            # the owners push the redundant experts' weights on the comm stream while this stream
            # already runs the gate/up GEMM of the local experts (which need no prefetched weight)
            # on the SMs the copy kernel leaves free; the prefetch slots follow in a second launch
            ev = layer.prefetch(plan)
            slots = dict(g=pools.slot("gate"), u=pools.slot("up"), d=pools.slot("down"))
            split, cu_use = epn, cu
            with tr.span("f.gateup_local"):
                outs = gemm.gateup_swiglu(hidden, layer.w_gate, layer.w_up, cu[:epn], row_scale=w_nvs,
                                          save_gate_up=layer.training, grid=layer.overlap_grid(), dispatch=disp)
            with tr.span("f.wait_prefetch"):
                torch.cuda.current_stream().wait_event(ev)
            with tr.span("f.gateup_slots"):
                act, gate, up = gemm.gateup_swiglu(hidden, layer.w_gate, layer.w_up, cu, wg_slot=slots["g"],
                                                   wu_slot=slots["u"], split=epn, row_scale=w_nvs,
                                                   save_gate_up=layer.training, out=outs, g_begin=epn,
                                                   dispatch=wait_only)
        else:
            slots = dict(g=None, u=None, d=None)
            split, cu_use = None, cu[:epn]
            with tr.span("f.gateup"):
                act, gate, up = gemm.gateup_swiglu(hidden, layer.w_gate, layer.w_up, cu_use, row_scale=w_nvs,
                                                   save_gate_up=layer.training, dispatch=disp)
        if fused:
            w_nvs = buf.dispatch_fused_end(plan, disp)     # plan records + a private copy of the weights
            if not layer.hidden_in_place:
                hidden = hidden.clone()
        if layer.fused_combine:
            # down GEMM fused with the combine all-to-all: the epilogue stores every result row
            # into its entry's slot on the token's home rank while later tiles are still computing
            with tr.span("f.down_push"):
                gemm.down(act, layer.w_down, cu_use, wd_slot=slots["d"], split=split,
                          push=buf.push_target(plan))
            with tr.span("f.combine_pushed"):
                y, _ = buf.combine_pushed(plan)
        else:
            shard = buf.hidden_nvsh_buffer_view
            gemm.down(act, layer.w_down, cu_use, wd_slot=slots["d"], split=split, out=shard)
            y, _, _ = buf.combine(plan, shard, None, zero_copy=True)
        ctx.layer, ctx.plan, ctx.split = layer, plan, split
        ctx.save_for_backward(x, hidden, w_nvs, cu_use, act, gate, up, topk, w)
        layer.last_plan = plan
        return y

    @staticmethod
    def backward(ctx, dy):
        layer, plan, split = ctx.layer, ctx.plan, ctx.split
        buf: Buffer = layer.buf
        pools = layer.pools
        x, hidden, w_nvs, cu, act, gate, up, topk, w = ctx.saved_tensors
        have_slots = split is not None
        slot = (lambda n: pools.slot(n)) if have_slots else (lambda n: None)
        gslot = (lambda n: pools.grad_slot(n)) if have_slots else (lambda n: None)
        dy = dy.contiguous()
        # combine backward = dispatch with the saved plan; the view is consumed before the shard
        # is overwritten further down (same stream)
        tr = layer.tracer
        disp = None
        with tr.span("b.dispatch"):
            if layer.fused_dispatch:    # dy travels inside the down-dgrad GEMM launch below
                d_out, _, _, _, disp = buf.dispatch_fused_begin(dy, plan=plan)
            else:
                d_out, _, _, _ = buf.dispatch(dy, plan=plan, zero_copy=True)
        ev_p = None
        if have_slots and pools.prefetch_owner is not plan:
            # Another layer's forward pass has refilled the shared prefetch slots since this
            # layer's own: bring this plan's redundant experts' weights back before the dgrad
            # GEMMs read them.  Issued after the dispatch entry above, whose barrier guarantees
            # that no rank still reads the slots for a later layer's backward pass.  In fused-SGD
            # mode the experts that have replicas are exactly those that keep their weights until
            # sgd_step, so the copies are the weights forward used.
            with tr.span("b.reprefetch"):
                ev_p = layer.prefetch(plan)
        with tr.span("b.down_dgrad"):
            if ev_p is None:
                d_act = gemm.down_dgrad(d_out, layer.w_down, cu, wd_slot=slot("down"), split=split, dispatch=disp)
            else:      # local experts first, next to the copy kernel; the slot groups once it is done
                d_act = gemm.down_dgrad(d_out, layer.w_down, cu[:buf.epn], grid=layer.overlap_grid(),
                                        dispatch=disp)
                torch.cuda.current_stream().wait_event(ev_p)
                d_act = gemm.down_dgrad(d_out, layer.w_down, cu, wd_slot=slot("down"), split=split,
                                        out=d_act, g_begin=buf.epn,
                                        dispatch=None if disp is None else dict(disp, mode=1))
        if disp is not None:
            buf.dispatch_fused_end(plan, disp)
        acc = layer.accumulate_grads
        fused_lr = layer.fused_sgd_lr
        do_reduce = have_slots and bool(pools.reduce)
        sgd = lambda w: None
        if fused_lr is not None:
            # optimizer step inside the weight-grad epilogues.  Experts that have replicas on
            # other ranks keep an fp32 grad (the replicas' grads are added first, sgd_step then
            # updates only those); every other local expert is updated in place right here.
            assert not acc, "the fused SGD step cannot be combined with grad accumulation"
            keep = None
            if do_reduce:
                etc = plan.experts_to_copy.reshape(-1).long()
                mine = (etc >= 0) & (etc // buf.epn == buf.rank)
                keep = torch.zeros(buf.epn + 1, dtype=torch.int32, device=etc.device)
                keep.index_fill_(0, torch.where(mine, etc % buf.epn, etc.new_full((), buf.epn)), 1)
                keep = keep[:buf.epn]
            layer._sgd_keep = keep
            sgd = lambda w: (w, fused_lr, keep)
        with tr.span("b.wgrad_down"):
            gemm.wgrad(d_out, act, cu, layer.g_down, grad_slot=gslot("down"), split=split, accumulate=acc,
                       sgd=sgd(layer.w_down))
        with tr.span("b.swiglu_bwd"):
            d_gate, d_up, d_scale = ew.swiglu_bwd(d_act, gate, up, w_nvs, rows_ptr=cu[-1:])
        ev_r = None
        zc = layer.accumulate_grads            # the slots are overwritten next step otherwise
        if fused_lr is None:
            with tr.span("b.wgrad_gateup"):
                gemm.wgrad(hidden, d_gate, cu, layer.g_gate, grad_slot=gslot("gate"), split=split, accumulate=acc)
                gemm.wgrad(hidden, d_up, cu, layer.g_up, grad_slot=gslot("up"), split=split, accumulate=acc)
            if layer.hidden_in_place:  # the forward rows have had their last reader
                buf.release_second_shard(layer)
            # the replicas' weight grads travel home on the comm stream while this stream computes dX
            if do_reduce:
                ev_r = buf.reduce_grad(plan, async_finish=True, local_gate_grad=layer.g_gate,
                                       local_up_grad=layer.g_up, local_down_grad=layer.g_down,
                                       gate_reduce_buffer=pools.reduce["gate"], up_reduce_buffer=pools.reduce["up"],
                                       down_reduce_buffer=pools.reduce["down"], zero_consumed=zc)
        elif do_reduce:
            # fused SGD changes w_gate / w_up in their weight-grad epilogues, so dX (which reads
            # them) comes first; meanwhile only the down projection's grads can travel home
            ev_r = buf.reduce_grad_tensors(plan, [layer.g_down], [pools.reduce["down"]], async_finish=True,
                                           zero_consumed=zc)
        grid = layer.overlap_grid() if ev_r is not None else 0
        # dispatch backward = combine; the scalar path returns d(route weights) as [S, K]
        if layer.fused_combine:
            with tr.span("b.gateup_dgrad_push"):
                gemm.gateup_dgrad(d_gate, d_up, layer.w_gate, layer.w_up, cu, wg_slot=slot("gate"),
                                  wu_slot=slot("up"), split=split, push=buf.push_target(plan), grid=grid)
            ev_r = _MoEFn._late_wgrads(layer, plan, hidden, d_gate, d_up, cu, gslot, split, ev_r, do_reduce, sgd)
            with tr.span("b.combine_pushed"):
                dx, dw_sk = buf.combine_pushed(plan, d_scale)
        else:
            shard = buf.hidden_nvsh_buffer_view
            gemm.gateup_dgrad(d_gate, d_up, layer.w_gate, layer.w_up, cu, wg_slot=slot("gate"),
                              wu_slot=slot("up"), split=split, out=shard, grid=grid)
            ev_r = _MoEFn._late_wgrads(layer, plan, hidden, d_gate, d_up, cu, gslot, split, ev_r, do_reduce, sgd)
            dx, dw_sk, _ = buf.combine(plan, shard, d_scale, zero_copy=True)
        # router backward
        with tr.span("b.router"):
            d_logits = ew.router_topk_bwd(w, dw_sk, topk, buf.E)                 # [S, E] bf16
            gemm.wgrad(x, d_logits, None, layer.g_router, accumulate=acc)
            dx_r = gemm.dense(d_logits, layer.w_router, b_is_kn=False, out_dtype=torch.bfloat16)
            dx = dx + dx_r
        if ev_r is not None:
            with tr.span("b.wait_reduce_grad"):
                torch.cuda.current_stream().wait_event(ev_r)      # grads are complete for the optimizer
        return dx, None

    @staticmethod
    def _late_wgrads(layer, plan, hidden, d_gate, d_up, cu, gslot, split, ev_r, do_reduce, sgd):
        """Fused-SGD order only: the gate / up weight grads (which update the weights in their
        epilogues) run after dX.  Returns the event that covers every reduce launched so far."""
        if layer.fused_sgd_lr is None:
            return ev_r
        pools, zc = layer.pools, layer.accumulate_grads
        wg = lambda a, g, w, **kw: gemm.wgrad(hidden, a, cu, g, grad_slot=gslot(w), split=split,
                                              sgd=sgd(getattr(layer, "w_" + w)), **kw)
        with layer.tracer.span("b.wgrad_gateup"):
            wg(d_gate, layer.g_gate, "gate")
            if do_reduce:     # the gate grads travel home under the up projection's weight grad
                ev_r = layer.buf.reduce_grad_tensors(plan, [layer.g_gate], [pools.reduce["gate"]],
                                                     async_finish=True, zero_consumed=zc)
            if do_reduce and layer.split_last_wgrad:
                # The up grads are the last to be computed, and only the combine and the router
                # backward are left to cover their way home.  So the grads that have to travel
                # (experts with replicas elsewhere, this rank's slot groups) are computed first, in
                # a short launch of their own, and leave while the rest is computed and applied.
                wg(d_up, layer.g_up, "up", select=1, grid=layer.overlap_grid())
                ev_r = layer.buf.reduce_grad_tensors(plan, [layer.g_up], [pools.reduce["up"]],
                                                     async_finish=True, zero_consumed=zc)
                wg(d_up, layer.g_up, "up", select=2, grid=layer.overlap_grid())
            else:
                wg(d_up, layer.g_up, "up", grid=layer.overlap_grid() if do_reduce else 0)
                if do_reduce:
                    ev_r = layer.buf.reduce_grad_tensors(plan, [layer.g_up], [pools.reduce["up"]],
                                                         async_finish=True, zero_consumed=zc)
        if layer.hidden_in_place:      # the forward rows have had their last reader
            layer.buf.release_second_shard(layer)
        return ev_r


class MoELayer:
    """One MoE layer of ``E`` SwiGLU experts sharded over the ``R`` ranks of ``buf``."""

    def __init__(self, buf: Buffer, Hp: int, pools: Optional[ExpertPools] = None, *, seed: int = 0,
                 router_bias: Optional[torch.Tensor] = None, init_std: float = 0.02,
                 train: bool = True, fused_combine: bool = True, hidden_in_place: bool = False,
                 fused_dispatch: Optional[bool] = None):
        assert not buf.virtual, "MoELayer runs one rank per process"
        assert buf.token_padding % 64 == 0, "the grouped GEMM needs token_padding % 64 == 0"
        assert buf.H % 128 == 0 and Hp % 64 == 0
        self.buf, self.pools, self.Hp = buf, pools, Hp
        self.training, self.accumulate_grads = train, False
        self.fused_combine = fused_combine
        # dispatch all-to-all inside the consuming GEMM launch (forward: gate/up, backward: down
        # dgrad) instead of a kernel of its own followed by a barrier; default: whenever the
        # Buffer's shape allows it
        ok = buf.fused_dispatch_supported()
        assert not fused_dispatch or ok, "this Buffer's shape cannot use the fused dispatch"
        self.fused_dispatch = ok if fused_dispatch is None else bool(fused_dispatch)
        # set to a learning rate to run the SGD step of the expert weights inside the weight-grad
        # epilogues of the next backward pass (see ``fuse_sgd``)
        self.fused_sgd_lr: Optional[float] = None
        # fused SGD: compute the up projection's travelling grads in a launch of their own, ahead
        # of the rest (see ``_late_wgrads``).  Pays when the last reduce_grad of the step is long
        # enough to stick out behind the combine and the router backward: measured exposed for
        # 0.37 ms at 8 ranks, hidden at 2 and 4, where the extra launch would only cost.
        _e = os.environ.get("MOONEP_B200_SPLIT_WGRAD", "").strip()
        self.split_last_wgrad = (buf.R >= 8) if _e == "" else _e != "0"
        self._sgd_keep = None
        self.tracer = NULL_TRACER
        if fused_combine:
            buf.enable_push()
        # The dispatched rows are an activation that backward needs again, while backward's own
        # dispatch reuses the Buffer's row shard; by default forward therefore copies them out.
        # With ``hidden_in_place`` the Buffer gets a second shard for the forward rows and the copy
        # (NvS x H bf16 read + written) is saved.  The Buffer has ONE second shard: it belongs to
        # this layer from its forward pass until its backward pass has read the rows for the last
        # time, so only one layer per Buffer may use the flag between a forward and its backward
        # (a second layer's forward raises instead of overwriting the rows), and this layer's
        # backward must run before its next forward.
        self.hidden_in_place = hidden_in_place
        if hidden_in_place:
            buf.enable_second_shard()
        dev = torch.device("cuda", buf.device)
        H, E, epn = buf.H, buf.E, buf.epn
        g = torch.Generator(device=dev).manual_seed(seed * 7919 + 13)
        ge = torch.Generator(device=dev).manual_seed(seed * 7919 + 101 + buf.rank)
        rnd = lambda gen, *s: (torch.randn(*s, device=dev, generator=gen) * init_std).bfloat16()
        self.w_router = rnd(g, H, E)                       # replicated (same seed on every rank)
        self.w_gate = rnd(ge, epn, H, Hp)
        self.w_up = rnd(ge, epn, H, Hp)
        self.w_down = rnd(ge, epn, H, Hp)
        self.router_bias = router_bias
        if train:
            z = lambda *s: torch.zeros(*s, dtype=torch.float32, device=dev)
            self.g_router = z(1, H, E)
            self.g_gate, self.g_up, self.g_down = z(epn, H, Hp), z(epn, H, Hp), z(epn, H, Hp)
        self.last_plan = None

    def prefetch(self, plan):
        """``prefetch_weight`` of this layer's experts for ``plan`` on the comm stream; returns the
        event and records the plan as the owner of the shared prefetch slots."""
        pools = self.pools
        ev = self.buf.prefetch_weight(
            plan, async_finish=True, local_gate_weight=self.w_gate, local_up_weight=self.w_up,
            local_down_weight=self.w_down, gate_prefetch_buffer=pools.prefetch["gate"],
            up_prefetch_buffer=pools.prefetch["up"], down_prefetch_buffer=pools.prefetch["down"])
        pools.prefetch_owner = plan
        return ev

    def overlap_grid(self) -> int:
        """CTAs a GEMM may use while a weight op (prefetch / reduce) runs next to it."""
        sms = torch.cuda.get_device_properties(self.buf.device).multi_processor_count
        return max(1, sms - self.buf.num_sms_weights)

    def parameters(self):
        return dict(router=self.w_router, gate=self.w_gate, up=self.w_up, down=self.w_down)

    def grads(self):
        return dict(router=self.g_router[0], gate=self.g_gate, up=self.g_up, down=self.g_down)

    def __call__(self, x: torch.Tensor) -> torch.Tensor:
        assert x.dtype == torch.bfloat16 and tuple(x.shape) == (self.buf.S, self.buf.H)
        return _MoEFn.apply(x.contiguous(), self)

    def fuse_sgd(self, lr: Optional[float]) -> None:
        """Plain SGD fused into backward: with a learning rate set, the weight-grad kernels apply
        ``w = bf16(w - lr * grad)`` to every local expert straight from their accumulators, so the
        fp32 grad is neither written nor read back (12 -> 4 bytes of HBM traffic per parameter).
        Experts that have replicas on other ranks this step still store their grad, receive the
        replicas' grads through ``reduce_grad`` and are updated by ``sgd_step``, which in this
        mode touches only them and the router.  The results are bit-identical to the unfused
        step.  ``grads()`` of the fused experts is stale in this mode; ``None`` switches it off
        (needed for grad accumulation or any optimizer other than plain SGD)."""
        self.fused_sgd_lr = None if lr is None else float(lr)

    def sgd_step(self, lr: float) -> None:
        """``w -= lr * grad`` on every parameter (the router grad is averaged over the group by
        the caller if it wants data-parallel semantics; experts are rank-private)."""
        with self.tracer.span("sgd"):
            ew.sgd_update_(self.w_router, self.g_router[0], lr)
            if self.fused_sgd_lr is not None:
                assert float(lr) == self.fused_sgd_lr, "fuse_sgd() and sgd_step() disagree on the learning rate"
                if self._sgd_keep is None:
                    return                              # every expert was updated in backward
                for w, g in ((self.w_gate, self.g_gate), (self.w_up, self.g_up), (self.w_down, self.g_down)):
                    ew.sgd_update_(w, g, lr, only=self._sgd_keep)
                return
            ew.sgd_update_(self.w_gate, self.g_gate, lr)
            ew.sgd_update_(self.w_up, self.g_up, lr)
            ew.sgd_update_(self.w_down, self.g_down, lr)

    def state_dict(self):
        """Home-layout weights only; prefetch slots are transient and never saved."""
        return {k: v.detach().cpu() for k, v in self.parameters().items()}

    def load_state_dict(self, sd):
        for k, v in self.parameters().items():
            v.copy_(sd[k].to(v.device))
