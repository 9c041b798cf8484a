"""Wrappers of the bandwidth kernels in ``csrc/device/elementwise.cu`` (router top-k / softmax /
histogram and its backward, SwiGLU backward, fused SGD).  None of these exist in the reference,
which stops at communication; they are the remaining hot ops of the MoE layer."""
from __future__ import annotations

import torch

from .. import _native as nat
from .._native import F, I, L, P

nat.declare("mep_router_topk", I, [P, P, I, I, I, P, P, P, P])
nat.declare("mep_router_topk_bwd", I, [P, P, P, I, I, I, P, P])
nat.declare("mep_swiglu_bwd", I, [P, P, P, P, P, I, I, P, P, P, P])
nat.declare("mep_sgd_update", I, [P, P, L, F, P])
nat.declare("mep_sgd_update_masked", I, [P, P, L, L, P, F, P])


def _st():
    return torch.cuda.current_stream().cuda_stream


def _rc(rc, what):
    if rc != 0:
        raise RuntimeError(f"{what}: {nat.last_error()} (code {rc})")


def router_topk(logits: torch.Tensor, K: int, bias: torch.Tensor | None = None):
    """Top-``K`` experts of ``logits + bias`` per token, softmax gate weights over the selected
    unbiased logits, and the tokens-per-expert histogram.  Returns ``(topk[S,K] int32,
    weights[S,K] fp32, tpe[E] int32)``."""
    assert logits.dtype == torch.float32 and logits.is_contiguous() and logits.is_cuda
    S, E = logits.shape
    topk = torch.empty(S, K, dtype=torch.int32, device=logits.device)
    w = torch.empty(S, K, dtype=torch.float32, device=logits.device)
    tpe = torch.empty(E, dtype=torch.int32, device=logits.device)
    if bias is not None:
        assert bias.dtype == torch.float32 and bias.numel() == E
    _rc(nat.call("mep_router_topk", logits.data_ptr(), nat.ptr(bias), S, E, K, topk.data_ptr(),
                 w.data_ptr(), tpe.data_ptr(), _st()), "router_topk")
    return topk, w, tpe


def router_topk_bwd(weights, dweights, topk, E: int) -> torch.Tensor:
    """``dlogits[S,E]`` bf16 (softmax backward, zero outside the selected experts)."""
    S, K = weights.shape
    assert dweights.dtype == torch.float32 and dweights.is_contiguous()
    out = torch.empty(S, E, dtype=torch.bfloat16, device=weights.device)
    _rc(nat.call("mep_router_topk_bwd", weights.data_ptr(), dweights.data_ptr(), topk.data_ptr(),
                 S, E, K, out.data_ptr(), _st()), "router_topk_bwd")
    return out


def swiglu_bwd(dact, gate, up, row_scale=None, rows_ptr=None, want_dscale=True):
    """Backward of ``act = silu(gate) * up * row_scale``: ``(dgate, dup, dscale[rows] | None)``.
    ``rows_ptr`` (device int32) bounds the rows that are processed without a host sync."""
    rows, Hp = dact.shape
    for t in (dact, gate, up):
        assert t.dtype == torch.bfloat16 and t.is_contiguous()
    dgate, dup = torch.empty_like(dact), torch.empty_like(dact)
    dscale = torch.zeros(rows, dtype=torch.float32, device=dact.device) if want_dscale else None
    _rc(nat.call("mep_swiglu_bwd", dact.data_ptr(), gate.data_ptr(), up.data_ptr(),
                 nat.ptr(row_scale), nat.ptr(rows_ptr), rows, Hp, dgate.data_ptr(), dup.data_ptr(),
                 nat.ptr(dscale), _st()), "swiglu_bwd")
    return dgate, dup, dscale


def sgd_update_(w: torch.Tensor, g: torch.Tensor, lr: float, only: torch.Tensor = None) -> None:
    """In place ``w(bf16) = bf16(w - lr * g(fp32))``.  ``only`` (int32 ``[experts]``, with ``w`` and
    ``g`` shaped ``[experts, ...]``) restricts the update to the experts whose flag is non-zero."""
    assert w.dtype == torch.bfloat16 and g.dtype == torch.float32 and w.numel() == g.numel()
    assert w.is_contiguous() and g.is_contiguous()
    if only is None:
        _rc(nat.call("mep_sgd_update", w.data_ptr(), g.data_ptr(), w.numel(), float(lr), _st()), "sgd_update")
        return
    assert only.dtype == torch.int32 and only.is_cuda and only.numel() >= w.shape[0]
    _rc(nat.call("mep_sgd_update_masked", w.data_ptr(), g.data_ptr(), w.shape[0], w[0].numel(),
                 only.data_ptr(), float(lr), _st()), "sgd_update")
