"""Planner / dispatch case list.  The shapes are the edge cases the reference's suite pins
(tests/test_planning.py:22-204): tiny S=1/K=1, no padding, non-power-of-two epn, heavy skew,
E > 2048, all-local, all-remote, duplicate top-k, single expert with exact / tail padding."""
from dataclasses import dataclass
from typing import Optional

import torch

from moonep_b200.utils.routing import generate_topk_routing, pattern_topk


@dataclass(frozen=True)
class Case:
    name: str
    S: int
    K: int
    epn: int
    H: int = 64
    num_sms: int = 4
    token_padding: int = 128
    routing: str = "balanced"
    bias_ratio: float = 0.0
    seed: int = 1
    min_R: int = 1
    max_R: Optional[int] = None

    def ok_for(self, R: int) -> bool:
        if R < self.min_R or (self.max_R is not None and R > self.max_R):
            return False
        if self.routing in ("balanced", "biased") and self.K > self.epn * R:
            return False
        return True

    def topk_all(self, R: int):
        """(topk[R,S,K], tpe[R,E]) on the CPU."""
        E = self.epn * R
        if self.routing in ("balanced", "biased"):
            bias = self.bias_ratio if self.routing == "biased" else 0.0
            pairs = [generate_topk_routing(self.S, self.K, E, R, bias, "cpu", self.seed, r)
                     for r in range(R)]
        else:
            pairs = [pattern_topk(self.routing, self.S, self.K, self.epn, R, r) for r in range(R)]
        return torch.stack([p[0] for p in pairs]), torch.stack([p[1] for p in pairs])


CASES = [
    Case("balanced_epn16", S=256, K=8, epn=16, H=128, num_sms=8),
    Case("tiny_s1_k1", S=1, K=1, epn=1, H=16, num_sms=1, token_padding=8),
    Case("tiny_biased_with_prefetch", S=3, K=5, epn=3, H=16, num_sms=1, token_padding=32,
         routing="biased", bias_ratio=1.0, seed=9002, min_R=2),
    Case("no_padding", S=33, K=2, epn=2, H=16, num_sms=1, token_padding=1, routing="biased",
         bias_ratio=1.0, seed=10001),
    Case("non_power_mild_bias", S=17, K=3, epn=3, H=16, num_sms=1, token_padding=16,
         routing="biased", bias_ratio=0.5, seed=10501),
    Case("small_balanced_with_prefetch", S=17, K=3, epn=3, H=16, num_sms=1, token_padding=16,
         seed=11001),
    Case("near_degenerate_bias", S=64, K=2, epn=5, H=32, num_sms=8, routing="biased",
         bias_ratio=5.0, seed=12001),
    Case("typical_bias", S=32, K=4, epn=4, H=32, num_sms=8, token_padding=64, routing="biased",
         bias_ratio=1.0, seed=13001),
    Case("heavy_bias", S=96, K=3, epn=7, H=48, num_sms=1, routing="biased", bias_ratio=2.0,
         seed=14001),
    Case("many_experts_k1", S=1024, K=1, epn=256, H=16, num_sms=8, token_padding=1),
    Case("multi_chunk_k1", S=2048, K=1, epn=320, H=16, num_sms=1, token_padding=1),
    Case("segment_tail_k1", S=1536, K=1, epn=320, H=16, num_sms=2, token_padding=1, min_R=4),
    Case("experts_gt_2048", S=256, K=1, epn=1025, H=16, num_sms=8, token_padding=1, max_R=2),
    Case("all_local", S=32, K=4, epn=8, H=32, num_sms=8, token_padding=16, routing="all_local"),
    Case("all_remote", S=32, K=4, epn=8, H=32, num_sms=8, token_padding=16, routing="all_remote",
         min_R=2),
    Case("duplicate_topk", S=16, K=4, epn=4, H=32, num_sms=8, token_padding=8,
         routing="duplicate_topk", min_R=2),
    Case("duplicate_topk_k32", S=8, K=32, epn=2, H=32, num_sms=2, token_padding=8,
         routing="duplicate_topk", min_R=2),
    Case("single_expert_exact_padding", S=8, K=2, epn=4, H=16, num_sms=1, token_padding=8,
         routing="single_expert"),
    Case("single_expert_padding_tail", S=9, K=2, epn=4, H=16, num_sms=1, token_padding=8,
         routing="single_expert"),
    Case("skew_sigma1_k8", S=512, K=8, epn=8, H=256, num_sms=8, token_padding=16,
         routing="biased", bias_ratio=1.0, seed=77),
]


def case_params(Rs=(1, 2, 4, 8)):
    import pytest

    return [pytest.param(c, R, id=f"{c.name}-R{R}") for c in CASES for R in Rs if c.ok_for(R)]
