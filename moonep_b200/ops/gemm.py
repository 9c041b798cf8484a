"""Python front end of the tcgen05 grouped GEMM (``csrc/device/grouped_gemm.cu``).

The reference has no GEMM; it leaves the ``[2*epn, H, H']`` "VM group GEMM" to the host
framework (README.md:45-68).  These wrappers are that GEMM for the expert FFN of the MoE layer:

========================  ==========================  =======================================
op                        math                        operands
========================  ==========================  =======================================
``gateup_swiglu``         act = silu(x Wg)*(x Wu)*w   x [rows,H] . Wg/Wu [G,H,H'] (MN-major B)
``down``                  y = act Wd^T                act [rows,H'] . Wd [G,H,H'] (K-major B)
``down_dgrad``            dact = dy Wd                dy [rows,H] . Wd [G,H,H'] (MN-major B)
``gateup_dgrad``          dx = dg Wg^T + du Wu^T      two K segments, K-major B
``wgrad``                 dW[g] (+)= a_g^T b_g        a [rows,H], b [rows,H'] -> fp32 [G,H,H']
``dense``                 c = a b                     one group (router logits)
========================  ==========================  =======================================

Groups are the VM groups of ``cu_seqlens``; ``*_slot`` tensors are this rank's prefetch / reduce
slots and serve groups ``>= split`` (they may be ``None`` when the plan never uses them).
Requirements: bf16 operands, 16-byte aligned, reduction length a multiple of 8, group sizes a
multiple of 64 for ``wgrad``.  Every call raises if the native library is missing; there is no
eager fallback.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from .. import _native as nat
from .._native import I, P

EPI_BF16, EPI_SWIGLU, EPI_F32, EPI_PUSH = 0, 1, 2, 3


class _GemmDesc(ctypes.Structure):
    _fields_ = [
        ("mode", ctypes.c_int32), ("epi", ctypes.c_int32), ("b_mn", ctypes.c_int32),
        ("nseg", ctypes.c_int32), ("ngroups", ctypes.c_int32), ("split", ctypes.c_int32),
        ("total_rows", ctypes.c_int32), ("N", ctypes.c_int32), ("K", ctypes.c_int32),
        ("rows_per_expert", ctypes.c_int32), ("Mw", ctypes.c_int32),
        ("accumulate", ctypes.c_int32), ("zero_empty_below", ctypes.c_int32),
        ("grid", ctypes.c_int32), ("debug", ctypes.c_int32), ("g_begin", ctypes.c_int32),
        ("a_rows", ctypes.c_int64), ("lda", ctypes.c_int64 * 2), ("a", ctypes.c_void_p * 2),
        ("b", (ctypes.c_void_p * 2) * 2), ("b_rows", ctypes.c_int64 * 2), ("ldb", ctypes.c_int64),
        ("cu_seqlens", ctypes.c_void_p), ("out", ctypes.c_void_p * 3), ("ldc", ctypes.c_int64),
        ("row_scale", ctypes.c_void_p), ("status", ctypes.c_void_p), ("timeout_ns", ctypes.c_int64),
        ("src_info", ctypes.c_void_p), ("push_base", ctypes.c_void_p),
        ("push_rank_stride", ctypes.c_int64), ("push_entries", ctypes.c_int32),
        ("push_ranks", ctypes.c_int32), ("two_cta", ctypes.c_int32), ("wg_select", ctypes.c_int32),
        ("sgd_w", ctypes.c_void_p), ("sgd_keep", ctypes.c_void_p), ("sgd_lr", ctypes.c_float),
        ("disp_mode", ctypes.c_int32), ("disp_ctx", ctypes.c_void_p), ("disp_x", ctypes.c_void_p),
        ("disp_w", ctypes.c_void_p), ("disp_dst", ctypes.c_void_p), ("disp_order", ctypes.c_void_p),
        ("disp_zero_fill", ctypes.c_void_p), ("disp_fresh", ctypes.c_int32), ("disp_shard", ctypes.c_int32),
    ]


nat.declare("mep_gemm_desc_bytes", I, [])
nat.declare("mep_gemm_launch", I, [ctypes.POINTER(_GemmDesc), P])

_status: dict[int, torch.Tensor] = {}
_checked_layout = False


def status_word(device) -> torch.Tensor:
    """Per-device int32[8] that GEMM kernels flag on a bounded-wait expiry (0 = healthy)."""
    idx = torch.device(device).index or 0
    if idx not in _status:
        _status[idx] = torch.zeros(8, dtype=torch.int32, device=f"cuda:{idx}")
    return _status[idx]


def check_status(device="cuda") -> None:
    st = status_word(device).tolist()
    if st[0] == 5:
        raise RuntimeError(f"grouped GEMM with fused dispatch: the rows of block {st[4]} never arrived "
                           f"(CTA {st[3]} saw {st[5]} of {st[6]} row parts)")
    if st[0] != 0:
        raise RuntimeError(f"grouped GEMM: bounded wait expired (code {st[0]}, where {st[2]}, CTA {st[3]})")


def reset_status(device="cuda") -> None:
    status_word(device).zero_()


PLAIN_EPILOGUE = False   # A/B switch of benchmarks: per-row 16-byte stores instead of staged TMA stores
# CTA pairs (tcgen05 cta_group::2: clusters of two CTAs issue one 256-row MMA and each stages only
# half of the B tile, which cuts the shared-memory reads per MMA from 12 KB to 8 KB, the limit of
# the single-CTA kernel).  ``MOONEP_B200_TWO_CTA``: ``auto`` (default) uses pairs when the groups
# are long enough on average (see ``_launch``); ``1`` always, ``0`` never.  A launch with a CTA
# limit (one that runs next to a copy kernel) needs an even limit; the copy kernels are placed
# as SM pairs too, so the SMs they leave free can all be paired.
_two = __import__("os").environ.get("MOONEP_B200_TWO_CTA", "auto").strip().lower()
TWO_CTA = {"auto": 2, "": 2}.get(_two, None)
if TWO_CTA is None:
    TWO_CTA = int(_two)
PAIR_MIN_AVG_ROWS = 768
PAIR_MIN_AVG_ROWS_WGRAD = 512   # 64 groups x 512 rows, fused SGD: pairs 1.16 ms, single CTAs 1.44 ms


def _launch(d: _GemmDesc) -> None:
    global _checked_layout
    d.debug = 16 if PLAIN_EPILOGUE else 0
    if TWO_CTA == 2:
        # token-major: a pair covers 256 rows of ONE group, so short groups would leave the second
        # CTA idle; the host only knows the average (over the local groups, the slot groups hold
        # rows taken from those).  Weight-grad tiles split the weight rows instead, but with short
        # groups (a few k-blocks per tile) the pair's extra hand-shakes cost more than they save.
        local_groups = max(1, min(d.ngroups, d.split))
        least = PAIR_MIN_AVG_ROWS_WGRAD if d.mode == 1 else PAIR_MIN_AVG_ROWS
        d.two_cta = int(d.grid % 2 == 0 and d.total_rows >= least * local_groups)
    else:
        d.two_cta = TWO_CTA
    if not _checked_layout:
        assert nat.call("mep_gemm_desc_bytes") == ctypes.sizeof(_GemmDesc), "GemmDesc layout mismatch"
        _checked_layout = True
    rc = nat.call("mep_gemm_launch", ctypes.byref(d), torch.cuda.current_stream().cuda_stream)
    if rc != 0:
        raise RuntimeError(f"grouped GEMM launch failed: {nat.last_error()} (code {rc})")


def _bf16(t: torch.Tensor, name: str) -> torch.Tensor:
    assert t.is_cuda and t.dtype == torch.bfloat16, f"{name} must be a CUDA bf16 tensor"
    assert t.stride(-1) == 1 and t.data_ptr() % 16 == 0, f"{name} must be dense and 16-byte aligned"
    return t


def _groups(cu_seqlens, rows):
    if cu_seqlens is None:
        return None, 1
    assert cu_seqlens.dtype == torch.int32 and cu_seqlens.is_cuda and cu_seqlens.is_contiguous()
    return cu_seqlens.data_ptr(), cu_seqlens.numel()


def _tokens_gemm(a_segs, b_sel, b_slot_sel, cu_seqlens, split, N, K, rows_per_expert, b_mn, epi,
                 outs, ldc, row_scale=None, total_rows=None, grid=0, push=None, g_begin=0, dispatch=None):
    d = _GemmDesc()
    d.mode, d.epi, d.b_mn, d.nseg = 0, epi, int(b_mn), len(a_segs)
    cu_ptr, ngroups = _groups(cu_seqlens, None)
    d.ngroups = ngroups
    d.split = ngroups if split is None else split
    a0 = a_segs[0]
    d.total_rows = a0.shape[0] if total_rows is None else total_rows
    d.N, d.K, d.rows_per_expert, d.Mw = N, K, rows_per_expert, 0
    d.grid = grid
    d.g_begin = g_begin
    d.a_rows = a0.shape[0]
    for i, a in enumerate(a_segs):
        _bf16(a, "A")
        assert a.shape == a0.shape and a.shape[1] == K
        d.a[i] = a.data_ptr()
        d.lda[i] = a.stride(0)
    ld = None
    for i, (b, bs) in enumerate(zip(b_sel, b_slot_sel)):
        _bf16(b, "B")
        assert b.is_contiguous()
        d.b[i][0] = b.data_ptr()
        d.b_rows[0] = b.shape[0] * b.shape[1]
        ld = b.shape[2]
        if bs is not None:
            _bf16(bs, "B slots")
            assert bs.is_contiguous() and bs.shape[1:] == b.shape[1:]
            d.b[i][1] = bs.data_ptr()
            d.b_rows[1] = bs.shape[0] * bs.shape[1]
        else:
            d.b[i][1] = None
            assert d.split >= ngroups, "groups >= split need slot weights"
    d.ldb = ld
    d.cu_seqlens = cu_ptr
    for i, o in enumerate(outs):
        d.out[i] = None if o is None else o.data_ptr()
    d.ldc = ldc
    d.row_scale = None if row_scale is None else row_scale.data_ptr()
    d.status = status_word(a0.device).data_ptr()
    if push is not None:
        d.epi = EPI_PUSH
        d.src_info = push["src_info"].data_ptr()
        d.push_base = push["push_base"].data_ptr()
        d.push_rank_stride = push["push_rank_stride"]
        d.push_entries, d.push_ranks = push["push_entries"], push["push_ranks"]
    if dispatch is not None:
        # the all-to-all that produces A runs inside this launch (``Buffer.dispatch_fused_begin``)
        d.disp_mode, d.disp_ctx = int(dispatch["mode"]), dispatch["ctx"]
        d.disp_fresh, d.disp_shard = int(dispatch["fresh"]), int(dispatch["shard"])
        if d.disp_mode == 2:
            d.disp_x = dispatch["x"].data_ptr()
            d.disp_w = None if dispatch["w"] is None else dispatch["w"].data_ptr()
            d.disp_dst, d.disp_order = dispatch["dst"].data_ptr(), dispatch["order"].data_ptr()
            d.disp_zero_fill = dispatch["zero_fill"].data_ptr()
    _launch(d)


def gateup_swiglu(x, wg, wu, cu_seqlens, *, wg_slot=None, wu_slot=None, split=None,
                  row_scale=None, save_gate_up=True, out=None, g_begin=0, grid=0, dispatch=None):
    """``act[rows,H'] = silu(x Wg[g]) * (x Wu[g]) * row_scale``; also returns bf16 gate / up.

    ``x`` [rows, H]; ``wg``/``wu`` [G0, H, H'] (+ optional slot tensors for groups >= split).
    ``out=(act, gate, up)`` reuses existing outputs and ``g_begin`` skips the first groups, so the
    local experts and the prefetch slots can be computed by two launches; ``grid`` limits the
    number of CTAs (to leave SMs to a concurrent communication kernel).  ``dispatch`` (from
    ``Buffer.dispatch_fused_begin``) makes this launch carry the dispatch all-to-all itself: ``x``
    must be the Buffer's row-buffer view, a seventh warp per CTA sends this rank's tokens, and
    tiles are computed as their rows arrive (``dict(disp, mode=1)`` only waits for arrivals)."""
    rows, H = x.shape
    Hp = wg.shape[2]
    assert wg.shape[1] == H and wu.shape == wg.shape
    if out is not None:
        act, gate, up = out
    else:
        act = torch.empty(rows, Hp, dtype=torch.bfloat16, device=x.device)
        gate = torch.empty_like(act) if save_gate_up else None
        up = torch.empty_like(act) if save_gate_up else None
    if row_scale is not None:
        assert row_scale.dtype == torch.float32 and row_scale.numel() >= rows
    _tokens_gemm([x], [wg, wu], [wg_slot, wu_slot], cu_seqlens, split, Hp, H, H, True, EPI_SWIGLU,
                 [gate, up, act], Hp, row_scale, grid=grid, g_begin=g_begin, dispatch=dispatch)
    return act, gate, up


def down(act, wd, cu_seqlens, *, wd_slot=None, split=None, out=None, push=None):
    """``y[rows,H] = act[rows,H'] Wd[g]^T`` with ``wd`` [G0, H, H'].

    With ``push`` (``Buffer.push_target(plan)``) nothing is written locally: every result row goes
    over NVLink into its entry's slot on the token's home rank (finish with
    ``Buffer.combine_pushed``) and ``None`` is returned."""
    rows, Hp = act.shape
    H = wd.shape[1]
    assert wd.shape[2] == Hp
    if push is not None:
        _tokens_gemm([act], [wd], [wd_slot], cu_seqlens, split, H, Hp, H, False, EPI_BF16, [], H, push=push)
        return None
    y = torch.empty(rows, H, dtype=torch.bfloat16, device=act.device) if out is None else out
    _tokens_gemm([act], [wd], [wd_slot], cu_seqlens, split, H, Hp, H, False, EPI_BF16, [y], y.stride(0))
    return y


def down_dgrad(dy, wd, cu_seqlens, *, wd_slot=None, split=None, out=None, g_begin=0, grid=0, dispatch=None):
    """``dact[rows,H'] = dy[rows,H] Wd[g]``.  ``out`` / ``g_begin`` / ``grid`` / ``dispatch`` as in
    :func:`gateup_swiglu`: the local experts and the prefetch slots may be two launches, and the
    launch may carry the dispatch of ``dy`` itself."""
    rows, H = dy.shape
    Hp = wd.shape[2]
    if out is None:
        out = torch.empty(rows, Hp, dtype=torch.bfloat16, device=dy.device)
    _tokens_gemm([dy], [wd], [wd_slot], cu_seqlens, split, Hp, H, H, True, EPI_BF16, [out], Hp,
                 grid=grid, g_begin=g_begin, dispatch=dispatch)
    return out


def gateup_dgrad(dg, du, wg, wu, cu_seqlens, *, wg_slot=None, wu_slot=None, split=None, out=None,
                 push=None, grid=0):
    """``dx[rows,H] = dg Wg[g]^T + du Wu[g]^T`` (two K segments into one accumulator); ``push`` as
    in :func:`down`."""
    rows, Hp = dg.shape
    H = wg.shape[1]
    if push is not None:
        _tokens_gemm([dg, du], [wg, wu], [wg_slot, wu_slot], cu_seqlens, split, H, Hp, H, False,
                     EPI_BF16, [], H, push=push, grid=grid)
        return None
    dx = torch.empty(rows, H, dtype=torch.bfloat16, device=dg.device) if out is None else out
    _tokens_gemm([dg, du], [wg, wu], [wg_slot, wu_slot], cu_seqlens, split, H, Hp, H, False,
                 EPI_BF16, [dx], dx.stride(0), grid=grid)
    return dx


def wgrad(a, b, cu_seqlens, grad_local, *, grad_slot=None, split=None, accumulate=False, sgd=None,
          grid=0, select=0):
    """``grad[g] (+)= a[rows of g]^T b[rows of g]``; ``a`` [rows, M], ``b`` [rows, N], fp32 grads
    ``[G0, M, N]`` (+ slot grads for groups >= split).  Group sizes must be multiples of 64
    (padding rows must be zero in ``a`` or ``b``).  Empty groups below ``split`` are zeroed
    unless ``accumulate``; empty slot groups are left untouched.

    ``sgd=(weights, lr, keep)`` fuses the optimizer step into the epilogue: for every local group
    whose int32 ``keep`` flag is zero (``keep=None``: all of them) the tile is applied to the bf16
    ``weights`` ``[G0, M, N]`` as ``w = bf16(w - lr * grad)``, bit-identical to ``sgd_update_`` on
    the stored grad, and ``grad_local`` is NOT written for that group.  Groups with a set flag and
    slot groups are stored as fp32 grads as usual.  This saves writing and re-reading the fp32
    grad (8 of the 12 bytes per parameter that weight grad + SGD move).

    With ``sgd``, ``select=1`` computes only the groups whose grads are stored (set flags, slot
    groups) and ``select=2`` only the ones that are applied; the two launches together equal one
    with ``select=0``.  The stored grads are the ones that ``reduce_grad`` has to move, so computing
    them first lets that transfer run beside the rest of the weight grad."""
    _bf16(a, "a"), _bf16(b, "b")
    rows, M = a.shape
    N = b.shape[1]
    assert b.shape[0] == rows and grad_local.dtype == torch.float32 and grad_local.is_contiguous()
    assert grad_local.shape[1:] == (M, N)
    d = _GemmDesc()
    d.mode, d.epi, d.b_mn, d.nseg = 1, EPI_F32, 1, 1
    cu_ptr, ngroups = _groups(cu_seqlens, rows)
    d.ngroups = ngroups
    d.split = ngroups if split is None else split
    d.total_rows, d.N, d.K, d.rows_per_expert, d.Mw = rows, N, 0, 0, M
    d.accumulate = int(accumulate)
    d.zero_empty_below = 0 if accumulate else d.split
    d.a_rows = rows
    d.a[0], d.lda[0] = a.data_ptr(), a.stride(0)
    d.b[0][0], d.ldb = b.data_ptr(), b.stride(0)
    d.cu_seqlens = cu_ptr
    d.out[0] = grad_local.data_ptr()
    if grad_slot is not None:
        assert grad_slot.dtype == torch.float32 and grad_slot.is_contiguous()
        d.out[1] = grad_slot.data_ptr()
    else:
        assert d.split >= ngroups
    d.ldc = N
    d.grid = grid
    assert select in (0, 1, 2) and (select == 0 or sgd is not None), "select splits a fused-SGD weight grad"
    if sgd is not None:
        w, lr, keep = sgd
        _bf16(w, "weights")
        assert not accumulate and w.is_contiguous() and w.shape == grad_local.shape and N % 8 == 0
        d.sgd_w, d.sgd_lr = w.data_ptr(), float(lr)
        d.wg_select = int(select)
        if keep is not None:
            assert keep.dtype == torch.int32 and keep.is_cuda and keep.numel() >= min(d.split, ngroups)
            d.sgd_keep = keep.data_ptr()
    d.status = status_word(a.device).data_ptr()
    _launch(d)
    return grad_local


def dense(a, b, *, out_dtype=torch.float32, b_is_kn=True):
    """``c[M,N] = a[M,K] b`` with ``b`` [K,N] (``b_is_kn``) or [N,K]; one group."""
    M, K = a.shape
    N = b.shape[1] if b_is_kn else b.shape[0]
    out = torch.empty(M, N, dtype=out_dtype, device=a.device)
    epi = EPI_F32 if out_dtype == torch.float32 else EPI_BF16
    _tokens_gemm([a], [b[None]], [None], None, None, N, K, b.shape[0], b_is_kn, epi, [out], N,
                 total_rows=M)
    return out
