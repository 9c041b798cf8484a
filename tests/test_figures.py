"""Layout figures: valid SVG whose arrows match the plan they were drawn from (CPU only)."""
import xml.etree.ElementTree as ET

import torch

from moonep_b200.reference import nvs_rows, plan_all_ranks
from moonep_b200.utils import figures
from moonep_b200.utils.routing import generate_topk_routing

NS = "{http://www.w3.org/2000/svg}"


def _plan(R=4, E=16, S=64, K=4, sigma=1.5, tp=8):
    topk = torch.stack([generate_topk_routing(S, K, E, R, sigma, "cpu", 0, rank=r)[0] for r in range(R)])
    tables, _ = plan_all_ranks(topk, S, K, E, tp)
    return tables, nvs_rows(S, K, E // R, tp)


def test_pool_figures_have_one_arrow_per_used_slot():
    tables, _ = _plan()
    etc = tables.experts_to_copy
    used = int((etc >= 0).sum())
    assert used > 0, "the skewed routing should need redundant experts"
    for grads in (False, True):
        root = ET.fromstring(figures.pool_figure(etc.tolist(), grads=grads))
        arrows = [p for p in root.iter(NS + "path") if p.get("class") == "arrow"]
        rects = [r.get("class") for r in root.iter(NS + "rect")]
        assert len(arrows) == used
        assert rects.count("slot-used") == used and rects.count("slot") == etc.numel() - used
        assert rects.count("local") == etc.numel()


def test_dispatch_figure_covers_every_group_and_padding():
    tables, nvs = _plan()
    root = ET.fromstring(figures.dispatch_figure(tables.cu_seqlens.tolist(), tables.zero_fill.tolist(), nvs))
    rects = [r.get("class") for r in root.iter(NS + "rect")]
    cu = tables.cu_seqlens
    prev = torch.cat([torch.zeros(cu.shape[0], 1, dtype=cu.dtype), cu[:, :-1]], dim=1)
    assert rects.count("group") == int((cu > prev).sum())
    assert rects.count("padding") == int(((tables.zero_fill[:, :, 1] > 0) & (cu > prev)).sum())
    assert rects.count("buffer") == cu.shape[0]


def test_cli_writes_three_files(tmp_path):
    figures.main(["--out", str(tmp_path), "--R", "2", "--E", "8", "--S", "32", "--K", "2"])
    names = sorted(p.name for p in tmp_path.iterdir())
    assert names == ["dispatch_buffer.svg", "grad_buffer.svg", "weight_buffer.svg"]
    for p in tmp_path.iterdir():
        ET.parse(p)
