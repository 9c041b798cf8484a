"""Synthetic top-k routing used by tests and benchmarks.

``generate_topk_routing`` follows the semantics of the reference generator
(tests/generate_topk_routing.py:6-44): ``bias_ratio == 0`` is a deterministic round-robin that
is perfectly balanced; otherwise expert popularity is ``exp(N(0, sigma))`` drawn from a seed
shared by all ranks while every rank draws its own tokens.  ``pattern_topk`` reproduces the
synthetic patterns of tests/kernel_test_utils.py:94-113.  ``zipf_topk`` / ``routing_for_maxvio``
implement the Zipf-skewed router logits the benchmark configurations name, with the skew
searched to hit a target MaxVio (``max_e T_e / mean - 1``, README.md:15-17).
"""
from __future__ import annotations

import torch


def maxvio(tpe_total: torch.Tensor) -> float:
    t = tpe_total.to(torch.float64)
    return float(t.max() / t.mean() - 1.0)


def tokens_per_expert(topk: torch.Tensor, E: int) -> torch.Tensor:
    return torch.bincount(topk.flatten().long(), minlength=E).to(torch.int32)


def generate_topk_routing(S, K, E, R, bias_ratio, dev, seed, rank=0):
    g_shared = torch.Generator(device=dev).manual_seed(seed)
    g_local = torch.Generator(device=dev).manual_seed(rank)
    if bias_ratio == 0.0:
        epn = E // R
        toks = torch.arange(S, device=dev)[:, None]
        ks = torch.arange(K, device=dev)[None, :]
        tgt_rank = (toks + ks) % R
        tgt_local = (toks // R + ks) % epn
        perm = torch.randperm(epn, device=dev, generator=g_local)
        topk = (tgt_rank * epn + perm[tgt_local]).to(torch.int32)
    else:
        pop = torch.exp(torch.normal(0.0, float(bias_ratio), size=(E,), device=dev,
                                     generator=g_shared))
        topk = torch.multinomial(pop[None, :].expand(S, E), K, replacement=False,
                                 generator=g_local).to(torch.int32)
    return topk.contiguous(), tokens_per_expert(topk, E)


def pattern_topk(pattern, S, K, epn, R, rank, dev="cpu"):
    s = torch.arange(S, device=dev)[:, None]
    k = torch.arange(K, device=dev)[None, :]
    if pattern == "all_local":
        topk = rank * epn + (s + k) % epn
    elif pattern == "all_remote":
        topk = ((rank + 1) % R) * epn + (s + k) % epn
    elif pattern == "single_expert":
        topk = torch.zeros(S, K, dtype=torch.long, device=dev)
    elif pattern == "duplicate_topk":
        topk = torch.full((S, K), ((rank + 1) % R) * epn, dtype=torch.long, device=dev)
    else:
        raise ValueError(f"unknown routing pattern {pattern!r}")
    topk = topk.to(torch.int32).contiguous()
    return topk, tokens_per_expert(topk, epn * R)


def zipf_topk(S, K, E, alpha, seed, rank=0, dev="cpu"):
    """Top-k of ``N(0,1) + log Zipf(alpha)`` logits plus softmax gate weights.

    The expert popularity ranking is a seed-shared random permutation so hot experts do not
    all sit on rank 0.
    """
    g_shared = torch.Generator(device="cpu").manual_seed(seed)
    g_local = torch.Generator(device="cpu").manual_seed(seed * 1000003 + rank + 1)
    order = torch.randperm(E, generator=g_shared)
    pop = torch.empty(E)
    pop[order] = torch.arange(1, E + 1, dtype=torch.float32).pow(-float(alpha))
    logits = torch.randn(S, E, generator=g_local) + torch.log(pop)[None, :]
    val, idx = torch.topk(logits, K, dim=1)
    w = torch.softmax(val, dim=1)
    return idx.to(torch.int32).to(dev).contiguous(), w.to(dev).contiguous()


def routing_for_maxvio(S, K, E, R, target, seed=0, dev="cpu", tol=0.05, iters=24):
    """Search the Zipf exponent so that the global MaxVio is close to ``target``.

    Returns ``(topk[R,S,K] int32, weights[R,S,K] fp32, achieved_maxvio, alpha)``.
    ``target <= 0`` returns the balanced round-robin routing with uniform weights.  The N(0,1)
    part of the logits is drawn once; only the popularity term changes during the search.
    """
    if target <= 0:
        tk = torch.stack([generate_topk_routing(S, K, E, R, 0.0, "cpu", seed, r)[0]
                          for r in range(R)])
        w = torch.full((R, S, K), 1.0 / K)
        return tk.to(dev), w.to(dev), maxvio(tokens_per_expert(tk, E)), 0.0
    g_shared = torch.Generator(device="cpu").manual_seed(seed)
    order = torch.randperm(E, generator=g_shared)
    logpop = torch.empty(E)
    logpop[order] = -torch.log(torch.arange(1, E + 1, dtype=torch.float32))
    base = torch.stack([torch.randn(S, E, generator=torch.Generator().manual_seed(seed * 1000003 + r + 1))
                        for r in range(R)])
    lo, hi = 0.0, 6.0
    best = None
    for _ in range(iters):
        mid = 0.5 * (lo + hi)
        val, idx = torch.topk(base + mid * logpop, K, dim=2)
        mv = maxvio(tokens_per_expert(idx, E))
        if best is None or abs(mv - target) < abs(best[2] - target):
            best = (idx.to(torch.int32), torch.softmax(val, dim=2), mv, mid)
        if abs(mv - target) <= tol * max(target, 1.0):
            break
        if mv < target:
            lo = mid
        else:
            hi = mid
    tk, w, mv, alpha = best
    return tk.contiguous().to(dev), w.contiguous().to(dev), mv, alpha
