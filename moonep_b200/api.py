"""``Buffer``: the public expert-parallel communication API.

Same surface as the reference's ``moonep.api.Buffer`` (moonep/api.py:417-1193):
``Buffer(S, H, K, E, num_ep_ranks, num_sms=None, token_padding=128, group=None,
comm_stream_priority=-1, enable_pdl=True, explicitly_destroy=False)`` with ``dispatch`` /
``prefetch_weight`` / ``combine`` / ``reduce_grad`` / ``destroy``, all of them accepting
``async_finish=True`` (work runs on a private high-priority stream and a CUDA event is
returned), plus the views ``hidden_nvsh_buffer_view`` / ``router_weight_buffer_view``.

Additions:

* ``virtual=True`` builds a single-GPU *virtual group*: all ``R`` ranks live on one device,
  every per-rank tensor gains a leading ``[R]`` dimension, and each kernel is ONE cooperative
  launch over all ranks.  The kernels are the same code as on R GPUs (they only see peer
  pointers), which is how multi-rank behaviour is tested on one device.
* every device-side wait is bounded; ``check()`` raises ``CommTimeoutError`` with the recorded
  {kernel, phase, rank, peer} if one ran out, and ``reset_barriers()`` re-synchronises the
  group afterwards.
* ``stats()`` reports bytes moved per op and the last plan's balance figures.
"""
from __future__ import annotations

import ctypes
import logging
import os
import warnings
from typing import Optional

import torch
import torch.distributed as dist

from . import _native as nat
from . import buffer as symm
from ._native import I, L, P
from .plan import CommPlan

log = logging.getLogger("moonep_b200.api")

nat.declare("mep_meta_chunk_ints", L, [L, I, I])
nat.declare("mep_plan_scratch_ints", L, [I, I, I])
nat.declare("mep_sync_state_ints", I, [])
nat.declare("mep_meta_offsets", None, [L, I, I, ctypes.POINTER(ctypes.c_int64)])
nat.declare("mep_ctx_create", P, [I, I, I, I, I, I, I, I, I, I, I, P, L, P, L, P, P, P, L])
nat.declare("mep_ctx_destroy", None, [P])
nat.declare("mep_ctx_set_second_shard", I, [P, P])
nat.declare("mep_ctx_set_pdl", None, [P, I])
nat.declare("mep_phase_stamps_compiled", I, [])
nat.declare("mep_trace_ints64", L, [])
nat.declare("mep_trace_dims", None, [ctypes.POINTER(ctypes.c_int)])
nat.declare("mep_ctx_set_trace", None, [P, P])
nat.declare("mep_launch_plan", I, [P, P, P, P, P, P, P, P, P, P])
nat.declare("mep_launch_arrive_reset", I, [P, P])
nat.declare("mep_launch_plan_snapshot", I, [P, P, P, P])
nat.declare("mep_launch_dispatch", I, [P, P, P, P, P, P, P, I, I, I, P])
nat.declare("mep_launch_push_reduce", I, [P, P, L, P, L, P, P, P, P, P, I, P])
nat.declare("mep_launch_expand", I, [P, P, P, I, P])
nat.declare("mep_launch_combine_prologue", I, [P, P, P, P])
nat.declare("mep_launch_combine", I, [P, P, P, P, P])
nat.declare("mep_launch_prefetch", I, [P, P, I, P, P, P, P, P])
nat.declare("mep_launch_grad_reduce", I, [P, P, I, P, P, P, P, I, I, I, P])
nat.declare("mep_launch_sync", I, [P, P])

_KERNEL_NAMES = {1: "sync", 2: "plan", 3: "dispatch", 4: "expand", 5: "combine_prologue",
                 6: "combine", 7: "prefetch_weight", 8: "reduce_grad", 9: "gemm"}
_STATUS_NAMES = {1: "grid barrier timeout", 2: "peer never arrived", 3: "copy completion timeout",
                 4: "index out of range", 5: "tile rows never arrived"}


class CommTimeoutError(RuntimeError):
    """A bounded device-side wait ran out (or an index check failed); see ``.info``."""

    def __init__(self, info: dict):
        self.info = info
        super().__init__(
            "{what} in kernel {kernel} (phase {phase}) on rank {rank}, peer {peer}: "
            "observed {observed}, expected {expected}".format(**info))


def _default_num_sms_local(sm_count: int) -> int:
    """SMs for the local (non-communicating) kernels; env ``MOONEP_NUM_SMS_DEDUP`` as in the
    reference (moonep/api.py:100-120), validated to ``[1, #SMs]``."""
    env = os.environ.get("MOONEP_NUM_SMS_DEDUP")
    if env is None:
        return sm_count
    try:
        v = int(env)
    except ValueError as exc:
        raise ValueError(f"MOONEP_NUM_SMS_DEDUP must be an integer, got {env!r}") from exc
    if not 1 <= v <= sm_count:
        raise ValueError(f"MOONEP_NUM_SMS_DEDUP must be in [1, {sm_count}], got {v}")
    return v


_LIVE_BUFFERS: "list[Buffer]" = []


class Buffer:
    def __init__(self, S: int, H: int, K: int, E: int, num_ep_ranks: int,
                 num_sms: Optional[int] = None, token_padding: int = 128, group=None,
                 comm_stream_priority: int = -1, enable_pdl: bool = True,
                 explicitly_destroy: bool = False, *, virtual: bool = False,
                 timeout_s: Optional[float] = None, num_sms_weights: Optional[int] = None):
        for name, v in dict(S=S, H=H, K=K, E=E, num_ep_ranks=num_ep_ranks,
                            token_padding=token_padding).items():
            assert isinstance(v, int) and v > 0, f"{name} must be a positive int, got {v!r}"
        R = num_ep_ranks
        assert E % R == 0, f"E={E} must be divisible by num_ep_ranks={R}"
        assert K <= 32 and R <= 128, "K <= 32 and num_ep_ranks <= 128"
        assert H % 8 == 0, "H must be a multiple of 8 (16-byte rows)"
        self._destroyed = True           # until construction succeeds
        self.S, self.H, self.K, self.E, self.R = S, H, K, E, R
        self.epn = E // R
        self.N = S * K
        self.token_padding = token_padding
        self.virtual = bool(virtual)
        # programmatic dependent launch of the kernel chains plan -> dispatch -> expansion and
        # pre-reduction -> pull combine (moonep/_common.py:393-406, api.py:622-626): each follower
        # is scheduled while its predecessor still runs and waits on the device for its completion
        self.enable_pdl = bool(enable_pdl)
        self.explicitly_destroy = explicitly_destroy
        self.device = torch.cuda.current_device()
        dev = torch.device("cuda", self.device)
        props = torch.cuda.get_device_properties(self.device)
        if self.virtual:
            self.group, self.rank = None, 0
            num_sms = 8 if num_sms is None else num_sms
            assert num_sms * R * 1 <= 2 * props.multi_processor_count, \
                "virtual group: num_sms * R CTAs must be co-resident (<= 2 per SM)"
        else:
            if R == 1 and not dist.is_initialized():
                self.group, self.rank = None, 0      # a lone rank needs no process group
            else:
                assert dist.is_initialized(), "construct Buffer after init_process_group"
                self.group = group if group is not None else dist.group.WORLD
                assert dist.get_world_size(self.group) == R, \
                    f"num_ep_ranks={R} != group world size {dist.get_world_size(self.group)}"
                self.rank = dist.get_rank(self.group)
            num_sms = 32 if num_sms is None else num_sms
            assert num_sms <= props.multi_processor_count
        self.num_sms = int(num_sms)
        # CTAs of prefetch_weight / reduce_grad; a small number lets them run next to a GEMM
        self.num_sms_weights = int(num_sms_weights) if num_sms_weights else self.num_sms
        self.num_sms_local = _default_num_sms_local(props.multi_processor_count)
        self.Rv = R if self.virtual else 1
        self.NvS = (self.N + (token_padding - 1) * 2 * self.epn + token_padding - 1) \
            // token_padding * token_padding
        assert self.NvS < (1 << 24) and R * self.NvS < (1 << 31), "NvS exceeds the slot encoding"
        if timeout_s is None:
            timeout_s = float(os.environ.get("MOONEP_B200_TIMEOUT_S", "30"))
        self.timeout_s = timeout_s

        # ---- symmetric buffers ----------------------------------------------------------
        meta_ints = int(nat.call("mep_meta_chunk_ints", self.NvS, R, E))
        self._solo = self.virtual or R == 1
        if self._solo:
            self.hidden_buf = symm.create_local_group_tensor((self.NvS, H), torch.bfloat16, R, self.device)
            self.meta_buf = symm.create_local_group_tensor((meta_ints,), torch.int32, R, self.device)
            self.meta_mc = None
        else:
            self.hidden_buf = symm.create_nvl_dist_tensor((self.NvS, H), torch.bfloat16, group=self.group, device=self.device)
            self.meta_buf, self.meta_mc = symm.create_nvl_dist_multicast_tensor(
                (meta_ints,), torch.int32, group=self.group, device=self.device)
        self.hidden_stride = self.hidden_buf.shape[0] // R
        self.hidden_buf2 = None
        self.meta_stride = self.meta_buf.shape[0] // R
        offs = (ctypes.c_int64 * 6)()
        nat.call("mep_meta_offsets", self.NvS, R, E, offs)
        (self.weights_off, self.link_off, self.tpe_off, self.flags_off, self.arrive_off,
         self.src_off) = list(offs)
        # every rank zeroes ITS OWN chunk, then the group meets: flags start at epoch 0
        if self.virtual:
            self.meta_buf.zero_()
        else:
            self.meta_buf[self.rank * self.meta_stride:(self.rank + 1) * self.meta_stride].zero_()
        torch.cuda.synchronize()
        if not self._solo:
            dist.barrier(group=self.group)

        # ---- local state ------------------------------------------------------------------
        self.sync_state = torch.zeros(2, self.Rv, nat.call("mep_sync_state_ints"), dtype=torch.int32, device=dev)
        self.status = torch.zeros(8, dtype=torch.int32).pin_memory()
        self.plan_scratch = torch.empty(
            self.Rv, int(nat.call("mep_plan_scratch_ints", R, E, self.num_sms)), dtype=torch.int32, device=dev)
        self._ctx = nat.call(
            "mep_ctx_create", self.rank, R, int(self.virtual), E, S, K, H, token_padding,
            self.num_sms, self.num_sms_local, self.num_sms_weights, self.hidden_buf.data_ptr(),
            self.hidden_stride,
            self.meta_buf.data_ptr(), self.meta_stride, self.sync_state.data_ptr(),
            self.status.data_ptr(), self.plan_scratch.data_ptr(), int(self.timeout_s * 1e9))
        if not self._ctx:
            raise RuntimeError(f"Buffer: {nat.last_error()}")
        nat.call("mep_ctx_set_pdl", self._ctx, int(self.enable_pdl))
        self.comm_stream = torch.cuda.Stream(device=dev, priority=comm_stream_priority)
        self._stats = dict(dispatch=0, combine=0, prefetch_weight=0, reduce_grad=0,
                           bytes_dispatch=0, bytes_combine=0)
        self._last_plan: Optional[CommPlan] = None
        self._destroyed = False
        _LIVE_BUFFERS.append(self)
        if self.rank == 0:
            log.info("Buffer S=%d H=%d K=%d E=%d R=%d epn=%d NvS=%d num_sms=%d token_padding=%d "
                     "virtual=%s hidden=%.1f MiB/rank meta=%.2f MiB/rank", S, H, K, E, R, self.epn,
                     self.NvS, self.num_sms, token_padding, self.virtual,
                     self.hidden_stride * H * 2 / 2 ** 20, self.meta_stride * 4 / 2 ** 20)

    # ---- housekeeping ---------------------------------------------------------------------
    @property
    def destroyed(self) -> bool:
        return self._destroyed

    def _require(self):
        assert not self._destroyed, "Buffer has been destroyed"

    def _shape(self, *tail):
        return (self.R, *tail) if self.virtual else tuple(tail)

    def _shards(self, shard: int = 0) -> torch.Tensor:
        """[Rv, NvS, H] view of the local shard(s)."""
        buf = self.hidden_buf if shard == 0 else self.hidden_buf2
        assert buf is not None, "enable_second_shard() first"
        hb = buf.view(self.R, self.hidden_stride, self.H)
        return hb[:, : self.NvS] if self.virtual else hb[self.rank: self.rank + 1, : self.NvS]

    def enable_second_shard(self) -> None:
        """Allocates a second symmetric ``[NvS, H]`` row buffer (collective, once).  ``dispatch(...,
        zero_copy=True, shard=1)`` then lands a forward pass's rows there and returns them in
        place, where they stay valid while later dispatches use shard 0 (a training step's
        backward dispatch): the copy out of the shard that ``zero_copy=False`` pays is saved.
        The caller must be done with the rows before the next ``shard=1`` dispatch."""
        self._require()
        if self.hidden_buf2 is not None:
            return
        if self._solo:
            self.hidden_buf2 = symm.create_local_group_tensor((self.NvS, self.H), torch.bfloat16, self.R, self.device)
        else:
            self.hidden_buf2 = symm.create_nvl_dist_tensor((self.NvS, self.H), torch.bfloat16, group=self.group,
                                                           device=self.device)
        assert self.hidden_buf2.shape[0] // self.R == self.hidden_stride
        self._rc(nat.call("mep_ctx_set_second_shard", self._ctx, self.hidden_buf2.data_ptr()), "second shard")

    def claim_second_shard(self, owner) -> None:
        """Marks the second shard as holding ``owner``'s rows.  A claim by anyone else before
        ``release_second_shard`` raises: the Buffer has one second shard, and a ``shard=1``
        dispatch of another user would silently overwrite rows that are still needed."""
        cur = getattr(self, "_shard1_owner", None)
        if cur is not None and cur is not owner:
            raise RuntimeError(
                "the Buffer's second shard still holds rows that another layer keeps for its backward "
                "pass; give every layer that uses hidden_in_place its own Buffer, or switch the flag off")
        self._shard1_owner = owner

    def release_second_shard(self, owner) -> None:
        if getattr(self, "_shard1_owner", None) is owner:
            self._shard1_owner = None

    def hidden_view(self, shard: int = 0) -> torch.Tensor:
        """``hidden_nvsh_buffer_view`` of the given shard."""
        self._require()
        v = self._shards(shard)
        return v if self.virtual else v[0]

    def _meta_rows(self) -> torch.Tensor:
        mb = self.meta_buf.view(self.R, self.meta_stride)
        return mb if self.virtual else mb[self.rank: self.rank + 1]

    @property
    def hidden_nvsh_buffer_view(self) -> torch.Tensor:
        """``[NvS, H]`` bf16 view of this rank's dispatch shard (``[R, NvS, H]`` when virtual)."""
        self._require()
        v = self._shards()
        return v if self.virtual else v[0]

    @property
    def router_weight_buffer_view(self) -> torch.Tensor:
        """``[NvS]`` fp32 view of this rank's route-weight slots."""
        self._require()
        v = self._meta_rows()[:, self.weights_off: self.weights_off + self.NvS].view(torch.float32)
        return v if self.virtual else v[0]

    def check(self) -> None:
        """Synchronise and raise ``CommTimeoutError`` if any device-side wait ran out."""
        torch.cuda.synchronize(self.device)
        st = self.status.tolist()
        if st[0] != 0:
            info = dict(code=st[0], what=_STATUS_NAMES.get(st[0], f"status {st[0]}"),
                        kernel=_KERNEL_NAMES.get(st[1], str(st[1])), phase=st[2], rank=st[3],
                        peer=st[4], observed=st[5], expected=st[6])
            raise CommTimeoutError(info)

    def reset_barriers(self) -> None:
        """Collective: clear the failure status and re-synchronise the barrier state after a
        ``CommTimeoutError`` (epochs of different ranks may have diverged)."""
        self._require()
        torch.cuda.synchronize(self.device)
        if not self._solo:
            dist.barrier(group=self.group)
        self.status.zero_()
        self.sync_state.zero_()
        rows = self._meta_rows()
        rows[:, self.flags_off: self.flags_off + 2 * ((self.R + 31) // 32 * 32)].zero_()
        torch.cuda.synchronize(self.device)
        if not self._solo:
            dist.barrier(group=self.group)

    def _maybe_check(self):
        if os.environ.get("MOONEP_B200_CHECK") == "1":
            self.check()

    def _rc(self, rc: int, what: str):
        if rc != 0:
            raise RuntimeError(f"{what}: {nat.last_error()} (code {rc})")

    @staticmethod
    def _stream() -> int:
        return torch.cuda.current_stream().cuda_stream

    def inter_rank_sync(self) -> None:
        """Device-side cross-rank barrier on the current stream (moonep/inter_rank_sync.py:119)."""
        self._require()
        self._rc(nat.call("mep_launch_sync", self._ctx, self._stream()), "inter_rank_sync")

    def _run_async(self, tensors, fn):
        """Run ``fn`` on the comm stream after the current stream's work; return its event."""
        main = torch.cuda.current_stream()
        capturing = torch.cuda.is_current_stream_capturing()
        for t in tensors:
            # under graph capture the tensors live in the graph's private pool for its lifetime
            if isinstance(t, torch.Tensor) and t.is_cuda and not capturing:
                t.record_stream(self.comm_stream)
        self.comm_stream.wait_event(main.record_event())
        with torch.cuda.stream(self.comm_stream):
            out = fn()
            ev = self.comm_stream.record_event()
        return out, ev

    # ---- dispatch ---------------------------------------------------------------------------
    def dispatch(self, hidden_sh, route_weights_sk=None, topk_experts_sk=None,
                 tokens_per_expert=None, plan: Optional[CommPlan] = None,
                 async_finish: bool = False, *, inter_rank_sync: bool = True,
                 zero_copy: bool = False, router_weights_zero_copy: bool = False, shard: int = 0):
        """Fused permute + all-to-all.  Returns ``(hidden_nvsh[NvS,H], route_weights_nvs[NvS] |
        None, cu_seqlens[2*epn] | None, plan[, event])`` (moonep/api.py:698-836).
        ``shard=1`` receives into the second row buffer (see ``enable_second_shard``).

        Without ``plan`` a fresh plan is made from ``topk_experts_sk`` / ``tokens_per_expert``.
        With ``plan`` the planner is skipped, ``cu_seqlens`` is ``None``, the same plan object is
        returned and the route weights are only sent when ``route_weights_sk`` is given.
        """
        self._require()
        S, H, K, E = self.S, self.H, self.K, self.E
        assert hidden_sh.dtype == torch.bfloat16 and hidden_sh.is_cuda and hidden_sh.is_contiguous()
        assert tuple(hidden_sh.shape) == self._shape(S, H), \
            f"hidden_sh must be {self._shape(S, H)}, got {tuple(hidden_sh.shape)}"
        assert hidden_sh.data_ptr() % 16 == 0
        if route_weights_sk is not None:
            assert route_weights_sk.dtype == torch.float32 and route_weights_sk.is_contiguous()
            assert tuple(route_weights_sk.shape) == self._shape(S, K)
        fresh = plan is None
        if fresh:
            assert topk_experts_sk is not None and tokens_per_expert is not None, \
                "topk_experts_sk and tokens_per_expert are required for a fresh plan"
            assert topk_experts_sk.dtype == torch.int32 and topk_experts_sk.is_contiguous()
            assert tuple(topk_experts_sk.shape) == self._shape(S, K)
            assert tokens_per_expert.dtype == torch.int32 and tokens_per_expert.is_contiguous()
            assert tuple(tokens_per_expert.shape) == self._shape(E)
        else:
            assert plan.N == self.N and plan.NvS == self.NvS and plan.R == self.R, \
                "plan was made by a Buffer of another shape"

        assert shard == 0 or (shard == 1 and self.hidden_buf2 is not None), \
            "shard must be 0, or 1 after enable_second_shard()"

        def run():
            return self._dispatch_on_current_stream(hidden_sh, route_weights_sk, topk_experts_sk,
                                                    tokens_per_expert, plan, inter_rank_sync,
                                                    zero_copy, router_weights_zero_copy, shard)

        if async_finish:
            out, ev = self._run_async([hidden_sh, route_weights_sk, topk_experts_sk, tokens_per_expert], run)
            for t in out[:3]:
                if isinstance(t, torch.Tensor) and not torch.cuda.is_current_stream_capturing():
                    t.record_stream(torch.cuda.current_stream())
            return (*out, ev)
        return run()

    def _dispatch_on_current_stream(self, x, w, topk, tpe, plan, inter_rank_sync, zero_copy, w_zero_copy,
                                    shard: int = 0):
        dev = x.device
        st = self._stream()
        fresh = plan is None
        i32 = dict(dtype=torch.int32, device=dev)
        if fresh:
            plan = self._fresh_plan(topk, tpe, dev, st)
        self._rc(nat.call("mep_launch_dispatch", self._ctx, x.data_ptr(), nat.ptr(w),
                          plan.dst.data_ptr(), plan.zero_fill_ranges.data_ptr(),
                          plan.link.data_ptr() if fresh else 0,
                          plan.src_info.data_ptr() if fresh else 0,
                          int(bool(inter_rank_sync) and not fresh), int(fresh), shard, st), "dispatch")
        self._rc(nat.call("mep_launch_expand", self._ctx, plan.link.data_ptr(),
                          plan.cu_seqlens.data_ptr(), shard, st), "dispatch expand")
        view = self.hidden_view(shard)
        hidden = view if zero_copy else view.clone()
        weights = None
        if w is not None:
            wv = self.router_weight_buffer_view
            weights = wv if w_zero_copy else wv.clone()
        self._stats["dispatch"] += 1
        self._stats["bytes_dispatch"] += self.N * self.H * 2 * self.Rv
        self._maybe_check()
        return hidden, weights, (plan.cu_seqlens if fresh else None), plan

    def _fresh_plan(self, topk, tpe, dev, st) -> CommPlan:
        i32 = dict(dtype=torch.int32, device=dev)
        dst = torch.empty(self._shape(self.N), **i32)
        cu = torch.empty(self._shape(2 * self.epn), **i32)
        zf = torch.empty(self._shape(2 * self.epn, 2), **i32)
        etc = torch.empty(self._shape(self.R, self.epn), **i32)
        rs = torch.empty(self._shape(2), **i32)
        link = torch.empty(self._shape(self.NvS), **i32)
        src = torch.empty(self._shape(self.NvS), **i32)
        order = torch.empty(self._shape(self.N), **i32)
        self._rc(nat.call("mep_launch_plan", self._ctx, topk.data_ptr(), tpe.data_ptr(),
                          dst.data_ptr(), cu.data_ptr(), zf.data_ptr(), etc.data_ptr(),
                          rs.data_ptr(), order.data_ptr(), st), "plan")
        plan = CommPlan(dst=dst, experts_to_copy=etc, zero_fill_ranges=zf, remote_stats=rs,
                        cu_seqlens=cu, link=link, N=self.N, R=self.R, E=self.E, NvS=self.NvS,
                        K=self.K, src_info=src, send_order=order)
        self._last_plan = plan
        return plan

    # ---- dispatch fused into the consuming GEMM ---------------------------------------------
    def fused_dispatch_supported(self) -> bool:
        """The fused dispatch -> GEMM path needs tiles that never straddle two groups
        (``token_padding % 128 == 0``), rows that split into equal 16-byte multiples of at most
        7 KB, and one rank per process."""
        row = self.H * 2
        nsplit = (row + 7167) // 7168
        return (not self.virtual) and self.token_padding % 128 == 0 and row % (16 * nsplit) == 0

    def dispatch_fused_begin(self, hidden_sh, route_weights_sk=None, topk_experts_sk=None,
                             tokens_per_expert=None, plan: Optional[CommPlan] = None, *, shard: int = 0):
        """First half of a dispatch whose all-to-all runs INSIDE the grouped GEMM that consumes
        the rows (``ops.gemm.gateup_swiglu`` / ``down_dgrad`` with ``dispatch=``): nothing is sent
        here.  A fresh plan is made (or, with ``plan``, the group meets and the arrival counters
        are cleared) and the arguments of the fused launches are returned.

        Returns ``(hidden_nvsh_view, route_weights_view | None, cu_seqlens | None, plan, disp)``.
        The two views alias the Buffer's row buffer ``shard`` and its weight slots; they hold the
        dispatched data only once the GEMM launches that were given ``disp`` (the first one) or
        ``dict(disp, mode=1)`` (any further one over the same rows) have run.  Finish with
        ``dispatch_fused_end``.  The reference has no counterpart: its dispatch ends with a
        barrier before the host framework's GEMM may start (moonep/dispatch.py:687-691)."""
        self._require()
        assert self.fused_dispatch_supported(), "this Buffer's shape cannot use the fused dispatch"
        assert hidden_sh.dtype == torch.bfloat16 and hidden_sh.is_cuda and hidden_sh.is_contiguous()
        assert tuple(hidden_sh.shape) == (self.S, self.H) and hidden_sh.data_ptr() % 16 == 0
        assert shard == 0 or (shard == 1 and self.hidden_buf2 is not None), \
            "shard must be 0, or 1 after enable_second_shard()"
        if route_weights_sk is not None:
            assert route_weights_sk.dtype == torch.float32 and route_weights_sk.is_contiguous()
            assert tuple(route_weights_sk.shape) == (self.S, self.K)
        st = self._stream()
        fresh = plan is None
        if fresh:
            assert topk_experts_sk is not None and tokens_per_expert is not None, \
                "topk_experts_sk and tokens_per_expert are required for a fresh plan"
            assert topk_experts_sk.dtype == torch.int32 and topk_experts_sk.is_contiguous()
            assert tokens_per_expert.dtype == torch.int32 and tokens_per_expert.is_contiguous()
            plan = self._fresh_plan(topk_experts_sk, tokens_per_expert, hidden_sh.device, st)
        else:
            assert plan.N == self.N and plan.NvS == self.NvS and plan.R == self.R
            assert plan.send_order is not None, "plan has no sending order"
            self._rc(nat.call("mep_launch_arrive_reset", self._ctx, st), "dispatch (fused) entry")
        disp = dict(mode=2, ctx=self._ctx, x=hidden_sh, w=route_weights_sk, dst=plan.dst,
                    order=plan.send_order, zero_fill=plan.zero_fill_ranges, fresh=int(fresh), shard=shard)
        self._stats["dispatch"] += 1
        self._stats["bytes_dispatch"] += self.N * self.H * 2
        wv = self.router_weight_buffer_view if route_weights_sk is not None else None
        return self.hidden_view(shard), wv, (plan.cu_seqlens if fresh else None), plan, disp

    def dispatch_fused_end(self, plan: CommPlan, disp: dict, clone_weights: bool = True):
        """Second half: call after the GEMM launches that carried ``disp``.  For a fresh plan the
        plan's chain links and source records are copied out of the meta chunk.  Returns the
        dispatched route weights ``[NvS]`` (a copy unless ``clone_weights=False``) or ``None``."""
        self._require()
        if disp["fresh"]:
            self._rc(nat.call("mep_launch_plan_snapshot", self._ctx, plan.link.data_ptr(),
                              plan.src_info.data_ptr(), self._stream()), "plan snapshot")
        self._maybe_check()
        if disp["w"] is None:
            return None
        wv = self.router_weight_buffer_view
        return wv.clone() if clone_weights else wv

    # ---- combine ----------------------------------------------------------------------------
    def combine(self, plan: Optional[CommPlan] = None, hidden_nvsh=None, route_weights_nvs=None,
                async_finish: bool = False, inter_rank_sync: bool = True, *,
                zero_copy: bool = False, router_weights_zero_copy: bool = False):
        """Pull + K-way fp32 sum.  Returns ``(hidden_sh[S,H], route_weights_sk[S,K] | None,
        event | None)`` -- always a 3-tuple (moonep/api.py:971-1104)."""
        self._require()
        assert plan is not None, "plan is required"
        assert hidden_nvsh is not None, "hidden_nvsh is required"
        assert hidden_nvsh.dtype == torch.bfloat16 and hidden_nvsh.is_cuda
        assert tuple(hidden_nvsh.shape) == self._shape(self.NvS, self.H)
        assert plan.N == self.N and plan.NvS == self.NvS and plan.R == self.R
        if zero_copy:
            assert hidden_nvsh.data_ptr() == self.hidden_nvsh_buffer_view.data_ptr(), \
                "zero_copy combine needs hidden_nvsh to alias the Buffer's dispatch view"
        else:
            assert hidden_nvsh.is_contiguous()
        if route_weights_nvs is not None:
            assert route_weights_nvs.dtype == torch.float32
            assert tuple(route_weights_nvs.shape) == self._shape(self.NvS)
            if router_weights_zero_copy:
                assert route_weights_nvs.data_ptr() == self.router_weight_buffer_view.data_ptr(), \
                    "router_weights_zero_copy needs route_weights_nvs to alias the Buffer's weight view"

        def run():
            return self._combine_on_current_stream(plan, hidden_nvsh, route_weights_nvs,
                                                   inter_rank_sync, zero_copy, router_weights_zero_copy)

        if async_finish:
            (h, w), ev = self._run_async([hidden_nvsh, route_weights_nvs], run)
            for t in (h, w):
                if isinstance(t, torch.Tensor) and not torch.cuda.is_current_stream_capturing():
                    t.record_stream(torch.cuda.current_stream())
            return h, w, ev
        h, w = run()
        return h, w, None

    def _combine_on_current_stream(self, plan, hidden_nvsh, w_nvs, inter_rank_sync, zero_copy, w_zero_copy):
        st = self._stream()
        dev = hidden_nvsh.device
        if inter_rank_sync:
            self._rc(nat.call("mep_launch_sync", self._ctx, st), "inter_rank_sync")
        if not zero_copy:
            self.hidden_nvsh_buffer_view.copy_(hidden_nvsh)
        if w_nvs is not None and not w_zero_copy:
            self.router_weight_buffer_view.copy_(w_nvs)
        self._rc(nat.call("mep_launch_combine_prologue", self._ctx, plan.link.data_ptr(),
                          plan.cu_seqlens.data_ptr(), st), "combine prologue")
        out = torch.empty(self._shape(self.S, self.H), dtype=torch.bfloat16, device=dev)
        w_out = None
        if w_nvs is not None:
            w_out = torch.empty(self._shape(self.S, self.K), dtype=torch.float32, device=dev)
        self._rc(nat.call("mep_launch_combine", self._ctx, plan.dst.data_ptr(), out.data_ptr(),
                          nat.ptr(w_out), st), "combine")
        self._stats["combine"] += 1
        self._stats["bytes_combine"] += self.N * self.H * 2 * self.Rv
        self._maybe_check()
        return out, w_out

    # ---- pushed combine (GEMM fused with the combine all-to-all) ---------------------------------
    def enable_push(self) -> None:
        """Allocate the symmetric staging buffers of the pushed combine: ``[R, S*K, H]`` bf16 rows
        and ``[R, S*K]`` fp32 scalars.  Collective (every rank must call it)."""
        self._require()
        if getattr(self, "push_buf", None) is not None:
            return
        if self._solo:
            self.push_buf = symm.create_local_group_tensor((self.N, self.H), torch.bfloat16, self.R, self.device)
            self.wpush_buf = symm.create_local_group_tensor((self.N,), torch.float32, self.R, self.device)
        else:
            self.push_buf = symm.create_nvl_dist_tensor((self.N, self.H), torch.bfloat16, group=self.group, device=self.device)
            self.wpush_buf = symm.create_nvl_dist_tensor((self.N,), torch.float32, group=self.group, device=self.device)
        self.push_stride = self.push_buf.shape[0] // self.R * self.H       # elements per rank
        self.wpush_stride = self.wpush_buf.shape[0] // self.R

    def push_target(self, plan: CommPlan) -> dict:
        """Arguments the GEMM's push epilogue needs to send each row of this rank's shard to the
        staging slot of its (token, k) entry on the token's home rank."""
        self.enable_push()
        assert plan.src_info is not None, "plan has no source records"
        return dict(src_info=plan.src_info, push_base=self.push_buf, push_rank_stride=self.push_stride,
                    push_entries=self.N, push_ranks=self.R)

    def combine_pushed(self, plan: CommPlan, row_scalar: Optional[torch.Tensor] = None):
        """Finish a combine whose rows were pushed home by the producing GEMM's epilogue: one
        cross-rank barrier, then the local K-way fp32 sum.  ``row_scalar`` ([NvS] fp32, e.g. the
        route-weight grads) is sent home too and returned as ``[S, K]``.
        Returns ``(hidden_sh[S,H], scalars_sk[S,K] | None)``."""
        self._require()
        self.enable_push()
        dev = self.push_buf.device
        out = torch.empty(self._shape(self.S, self.H), dtype=torch.bfloat16, device=dev)
        w_out = None
        if row_scalar is not None:
            assert row_scalar.dtype == torch.float32 and tuple(row_scalar.shape) == self._shape(self.NvS)
            assert row_scalar.is_contiguous()
            w_out = torch.empty(self._shape(self.S, self.K), dtype=torch.float32, device=dev)
        grid_x = self.num_sms if self.virtual else self.num_sms_local
        self._rc(nat.call("mep_launch_push_reduce", self._ctx, self.push_buf.data_ptr(), self.push_stride,
                          self.wpush_buf.data_ptr(), self.wpush_stride, plan.src_info.data_ptr(),
                          nat.ptr(row_scalar), plan.cu_seqlens.data_ptr(), out.data_ptr(),
                          nat.ptr(w_out), grid_x, self._stream()), "combine_pushed")
        self._stats["combine"] += 1
        self._maybe_check()
        return out, w_out

    # ---- prefetch_weight ----------------------------------------------------------------------
    def _pool_args(self, locals_, pools, what):
        n = len(locals_)
        lp = (ctypes.c_void_p * n)()
        pp = (ctypes.c_void_p * n)()
        eb = (ctypes.c_int64 * n)()
        rs = (ctypes.c_int64 * n)()
        for i, (loc, pool) in enumerate(zip(locals_, pools)):
            assert loc.is_cuda and pool.is_cuda and loc.is_contiguous(), f"{what}: tensor {i}"
            assert loc.dtype == pool.dtype, f"{what}: local / pool dtype mismatch for tensor {i}"
            lead = self._shape(self.epn)
            assert tuple(loc.shape[: len(lead)]) == lead, \
                f"{what}: local tensor {i} must start with {lead}, got {tuple(loc.shape)}"
            assert pool.shape[0] == self.R and pool.shape[1] == self.epn, \
                f"{what}: pool {i} must be [R, epn, ...], got {tuple(pool.shape)}"
            per_expert = loc[(0,) * len(lead)].numel() if loc.dim() > len(lead) else 1
            assert pool[0, 0].numel() == per_expert and pool[0].is_contiguous(), \
                f"{what}: pool {i} slots must be contiguous and match the local expert shape"
            assert pool.stride(0) >= self.epn * per_expert
            lp[i], pp[i] = loc.data_ptr(), pool.data_ptr()
            eb[i], rs[i] = per_expert, pool.stride(0)
        return n, lp, pp, eb, rs

    def prefetch_weight(self, plan: CommPlan, async_finish: bool = False, *,
                        local_gate_weight, local_up_weight, local_down_weight,
                        gate_prefetch_buffer, up_prefetch_buffer, down_prefetch_buffer,
                        local_gate_scale=None, local_up_scale=None, local_down_scale=None,
                        gate_scale_prefetch_buffer=None, up_scale_prefetch_buffer=None,
                        down_scale_prefetch_buffer=None):
        """Owners push the weights of redundant experts into the ``[R, epn, ...]`` prefetch slots
        of the ranks that compute them (moonep/api.py:838-969).  Returns ``None`` or an event."""
        self._require()
        assert plan is not None, "plan is required"
        locals_ = [local_gate_weight, local_up_weight, local_down_weight]
        pools = [gate_prefetch_buffer, up_prefetch_buffer, down_prefetch_buffer]
        scales = [local_gate_scale, local_up_scale, local_down_scale]
        spools = [gate_scale_prefetch_buffer, up_scale_prefetch_buffer, down_scale_prefetch_buffer]
        given = [s is not None for s in scales + spools]
        assert all(given) or not any(given), "give all six scale tensors or none"
        if all(given):
            locals_ += scales
            pools += spools
        for t in locals_:
            assert t.dtype in (torch.bfloat16, torch.int8, torch.uint8, torch.float32,
                               torch.float16, torch.float8_e4m3fn, torch.float8_e8m0fnu), \
                f"unsupported prefetch dtype {t.dtype}"
        n, lp, pp, eb, rs = self._pool_args(locals_, pools, "prefetch_weight")
        for i, t in enumerate(locals_):           # kernel works in bytes
            eb[i] *= t.element_size()
            rs[i] *= t.element_size()
            assert eb[i] % 16 == 0, "per-expert byte size must be a multiple of 16"

        def run():
            self._rc(nat.call("mep_launch_prefetch", self._ctx, plan.experts_to_copy.data_ptr(), n,
                              lp, pp, eb, rs, self._stream()), "prefetch_weight")
            self._stats["prefetch_weight"] += 1
            self._maybe_check()

        if async_finish:
            _, ev = self._run_async(locals_ + pools, run)
            return ev
        run()
        return None

    # ---- reduce_grad ----------------------------------------------------------------------------
    def reduce_grad(self, plan: CommPlan, async_finish: bool = False, *,
                    local_gate_grad, local_up_grad, local_down_grad,
                    gate_reduce_buffer, up_reduce_buffer, down_reduce_buffer,
                    entry_sync: bool = True, zero_consumed: bool = True):
        """Home ranks pull the fp32 prefetch-slot grads of their experts from every rank's
        ``[R, epn, ...]`` reduce buffer, add them to the local grad in ascending (rank, slot)
        order, then every rank zeroes its consumed slots (moonep/api.py:1106-1193).

        ``entry_sync=True`` adds a cross-rank barrier first, so that the grads other ranks wrote
        on their streams before calling are visible; the reference leaves that to the caller.
        ``zero_consumed=False`` skips the final clearing for callers whose next backward pass
        overwrites the slots instead of accumulating into them."""
        return self.reduce_grad_tensors(
            plan, [local_gate_grad, local_up_grad, local_down_grad],
            [gate_reduce_buffer, up_reduce_buffer, down_reduce_buffer], async_finish,
            entry_sync=entry_sync, zero_consumed=zero_consumed)

    def reduce_grad_tensors(self, plan: CommPlan, locals_, pools, async_finish: bool = False, *,
                            entry_sync: bool = True, zero_consumed: bool = True, num_sms: int = 0):
        """``reduce_grad`` for any subset of projections: ``locals_[i]`` ``[epn, ...]`` fp32 and its
        ``[R, epn, ...]`` reduce buffer ``pools[i]``.  A training loop that finishes the down
        projection's weight grads long before the gate/up ones can send them home early.
        ``num_sms`` overrides the CTA count of this launch (default: ``num_sms_weights``): the last
        reduce of a step runs next to nothing and may take more SMs."""
        self._require()
        assert plan is not None, "plan is required"
        locals_, pools = list(locals_), list(pools)
        assert len(locals_) == len(pools) and len(locals_) >= 1
        for t in locals_ + pools:
            assert t.dtype == torch.float32, "grads and reduce buffers must be fp32"
        n, lp, pp, eb, rs = self._pool_args(locals_, pools, "reduce_grad")
        for i in range(n):
            assert eb[i] % 4 == 0 and rs[i] % 4 == 0

        def run():
            self._rc(nat.call("mep_launch_grad_reduce", self._ctx, plan.experts_to_copy.data_ptr(), n,
                              lp, pp, eb, rs, int(entry_sync), int(zero_consumed), int(num_sms), self._stream()), "reduce_grad")
            self._stats["reduce_grad"] += 1
            self._maybe_check()

        if async_finish:
            _, ev = self._run_async(locals_ + pools, run)
            return ev
        run()
        return None

    # ---- device-side phase stamps ---------------------------------------------------------------
    _TRACE_NAMES = {
        0: ("dispatch", ["set up", "past entry barrier", "rows issued", "past exit barrier"]),
        1: ("combine", ["set up", "past entry barrier", "tokens stored"]),
        2: ("fused_gemm.producer", ["start", "first group arrived", "last load issued"]),
        3: ("fused_gemm.copy_warp", ["start", "all rows sent"]),
    }

    def enable_phase_stamps(self) -> bool:
        """Start recording per-CTA ``%globaltimer`` stamps in the dispatch, combine and fused-GEMM
        kernels.  Needs a library built with ``MOONEP_B200_NVCC_FLAGS=-DMEP_PHASE_STAMPS`` (a
        normal build compiles the stamps out); returns ``False`` otherwise."""
        self._require()
        if not nat.call("mep_phase_stamps_compiled"):
            return False
        if getattr(self, "_trace", None) is None:
            self._trace = torch.zeros(int(nat.call("mep_trace_ints64")), dtype=torch.int64, device=self.meta_buf.device)
            nat.call("mep_ctx_set_trace", self._ctx, self._trace.data_ptr())
        else:
            self._trace.zero_()
        return True

    def phase_stamps(self) -> dict:
        """``{kernel: {phase: (min_us, max_us)}}`` of the LAST launch of each stamped kernel, in
        microseconds after the kernel's earliest stamp, over the CTAs that ran (synchronises)."""
        if getattr(self, "_trace", None) is None:
            return {}
        torch.cuda.synchronize(self.device)
        dims = (ctypes.c_int * 3)()
        nat.call("mep_trace_dims", dims)
        t = self._trace.view(dims[0], dims[1], dims[2]).cpu()
        out = {}
        for k, (name, phases) in self._TRACE_NAMES.items():
            used = t[k][:, 0] > 0
            if not bool(used.any()):
                continue
            t0 = int(t[k][used][:, 0].min())
            out[name] = {}
            for i, ph in enumerate(phases):
                col = t[k][used][:, i]
                col = col[col > 0]
                if col.numel():
                    out[name][ph] = (round((int(col.min()) - t0) / 1e3, 1), round((int(col.max()) - t0) / 1e3, 1))
        return out

    # ---- telemetry ------------------------------------------------------------------------------
    def stats(self) -> dict:
        """Counters plus, for the last fresh plan: remote_stats, padding rows, dedup ratio.
        Reads device tensors (synchronises)."""
        out = dict(self._stats)
        p = self._last_plan
        if p is not None:
            dst = p.dst.reshape(-1)
            out["remote_stats"] = p.remote_stats.reshape(-1, 2).tolist()
            out["dedup_ratio"] = float((dst >= 0).sum().item()) / max(1, dst.numel())
            out["zero_pad_rows"] = int(p.zero_fill_ranges.reshape(-1, 2)[:, 1].sum().item())
            out["rows_used"] = p.cu_seqlens.reshape(-1, 2 * self.epn)[:, -1].tolist()
        return out

    # ---- teardown ---------------------------------------------------------------------------------
    def destroy(self, group_barrier: bool = True) -> None:
        """Idempotent.  Synchronises, meets the group, then unmaps the symmetric buffers
        (views first, owners last) -- moonep/api.py:512-553.  ``group_barrier=False`` skips the
        collective meeting: the way out when a peer is known to be gone."""
        if self._destroyed:
            return
        self._destroyed = True
        if self in _LIVE_BUFFERS:
            _LIVE_BUFFERS.remove(self)
        try:
            self.comm_stream.synchronize()
            torch.cuda.synchronize(self.device)
            if group_barrier and not self._solo and dist.is_initialized():
                dist.barrier(group=self.group)
        finally:
            nat.call("mep_ctx_destroy", self._ctx)
            self._ctx = None
            for name in ("meta_mc", "meta_buf", "hidden_buf", "hidden_buf2", "push_buf", "wpush_buf"):
                t = getattr(self, name, None)
                setattr(self, name, None)
                if t is not None:
                    symm.release(t)
            self._last_plan = None

    def __del__(self):
        if getattr(self, "_destroyed", True):
            return
        if self.explicitly_destroy:
            warnings.warn("Buffer was created with explicitly_destroy=True but destroy() was "
                          "never called; its peer mappings leak until process exit",
                          ResourceWarning)
            return
        try:
            self.destroy()
        except Exception:  # pragma: no cover
            pass


def destroy_live_buffers() -> None:
    """Destroy every Buffer that is still alive (test fixtures call this)."""
    while _LIVE_BUFFERS:
        _LIVE_BUFFERS[-1].destroy()
