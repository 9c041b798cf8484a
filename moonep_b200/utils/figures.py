"""Layout figures as dependency-free SVG, drawn from an actual plan.

The reference ships a matplotlib script that draws two fixed pictures of its weight / grad
buffers (figure/generate_buffer_figures.py: ``weight_buffer.png``, ``grad_buffer.png``).  Here the
pictures are generated from data: any ``experts_to_copy`` / ``cu_seqlens`` / ``zero_fill_ranges``
(from the CPU oracle or from a ``CommPlan`` of a live ``Buffer``) can be drawn, so the figures
double as a debugging view of what the planner decided.

  python -m moonep_b200.utils.figures --out figure/ [--R 4 --E 16 --S 64 --K 4 --sigma 1.5]

writes ``weight_buffer.svg`` (local experts and the ``[R, epn]`` prefetch pool of every rank, one
arrow per pushed expert), ``grad_buffer.svg`` (the same with the arrows reversed: reduce slots
pulled home) and ``dispatch_buffer.svg`` (every rank's ``[NvS]`` row buffer: expert groups,
padding rows, unused tail).
"""
from __future__ import annotations

import argparse
import os
from typing import Sequence
from xml.sax.saxutils import escape

LOCAL, POOL, USED, PAD, EDGE, TEXT, ARROW = "#FBE7A1", "#F3D6DA", "#C05046", "#E8EAED", "#333333", "#222222", "#555555"
SLOTG = "#BFD7EA"


class _Svg:
    def __init__(self, width: float, height: float):
        self.w, self.h, self.items = width, height, []

    def rect(self, x, y, w, h, fill, stroke=EDGE, cls=None, title=None):
        t = f"<title>{escape(title)}</title>" if title else ""
        c = f' class="{cls}"' if cls else ""
        self.items.append(f'<rect{c} x="{x:.1f}" y="{y:.1f}" width="{w:.1f}" height="{h:.1f}" fill="{fill}" '
                          f'stroke="{stroke}" stroke-width="0.8">{t}</rect>')

    def text(self, x, y, s, size=11, anchor="middle"):
        self.items.append(f'<text x="{x:.1f}" y="{y:.1f}" font-size="{size}" text-anchor="{anchor}" '
                          f'font-family="sans-serif" fill="{TEXT}">{escape(str(s))}</text>')

    def arrow(self, x1, y1, x2, y2, cls="arrow"):
        mx = (x1 + x2) / 2 + (y2 - y1) * 0.15
        my = (y1 + y2) / 2 - (x2 - x1) * 0.15 - 6
        self.items.append(f'<path class="{cls}" d="M{x1:.1f},{y1:.1f} Q{mx:.1f},{my:.1f} {x2:.1f},{y2:.1f}" '
                          f'fill="none" stroke="{ARROW}" stroke-width="1.1" marker-end="url(#head)"/>')

    def render(self) -> str:
        head = (f'<svg xmlns="http://www.w3.org/2000/svg" width="{self.w:.0f}" height="{self.h:.0f}" '
                f'viewBox="0 0 {self.w:.0f} {self.h:.0f}">'
                '<defs><marker id="head" markerWidth="8" markerHeight="8" refX="7" refY="4" orient="auto">'
                f'<path d="M0,0 L8,4 L0,8 z" fill="{ARROW}"/></marker></defs>'
                f'<rect x="0" y="0" width="{self.w:.0f}" height="{self.h:.0f}" fill="white" stroke="none"/>')
        return head + "".join(self.items) + "</svg>"


def pool_figure(experts_to_copy: Sequence[Sequence[int]], *, grads: bool = False, title: str = "") -> str:
    """``experts_to_copy[R][epn]`` (global expert id or -1 per slot) -> SVG.  One row per rank:
    its ``epn`` local experts, then its ``epn`` slots; an arrow per used slot from the expert's
    home (weights: home -> slot; grads: slot -> home)."""
    R, epn = len(experts_to_copy), len(experts_to_copy[0])
    cw, rh, gap, x0, y0 = max(26.0, 360.0 / max(epn, 1)), 30.0, 26.0, 70.0, 56.0
    svg = _Svg(x0 + 2 * epn * cw + gap + 30, y0 + R * (rh + 24) + 20)
    svg.text(svg.w / 2, 20, title or ("grads: reduce slots pulled home" if grads else "weights: experts pushed into prefetch slots"), 13)
    svg.text(x0 + epn * cw / 2, 42, "local grads [epn, H, H']" if grads else "local experts [epn, H, H']", 10)
    svg.text(x0 + epn * cw + gap + epn * cw / 2, 42,
             "reduce slots of this rank [epn, H, H']" if grads else "prefetch slots of this rank [epn, H, H']", 10)
    cell = {}
    for r in range(R):
        y = y0 + r * (rh + 24)
        svg.text(x0 - 8, y + rh / 2 + 4, f"rank {r}", 11, "end")
        for e in range(epn):
            x = x0 + e * cw
            svg.rect(x, y, cw, rh, LOCAL, cls="local", title=f"expert {r * epn + e} (home rank {r})")
            svg.text(x + cw / 2, y + rh / 2 + 4, r * epn + e, 9)
            cell[("L", r * epn + e)] = (x + cw / 2, y)
        for b in range(epn):
            x = x0 + epn * cw + gap + b * cw
            e = int(experts_to_copy[r][b])
            svg.rect(x, y, cw, rh, USED if e >= 0 else POOL, cls="slot-used" if e >= 0 else "slot",
                     title=f"slot ({r}, {b}): " + (f"expert {e}" if e >= 0 else "unused"))
            if e >= 0:
                svg.text(x + cw / 2, y + rh / 2 + 4, e, 9)
            cell[("S", r, b)] = (x + cw / 2, y)
    for r in range(R):
        for b in range(epn):
            e = int(experts_to_copy[r][b])
            if e < 0:
                continue
            (hx, hy), (sx, sy) = cell[("L", e)], cell[("S", r, b)]
            if grads:
                svg.arrow(sx, sy, hx, hy + (rh if hy < sy else 0))
            else:
                svg.arrow(hx, hy + (rh if hy < sy else 0), sx, sy)
    return svg.render()


def dispatch_figure(cu_seqlens: Sequence[Sequence[int]], zero_fill: Sequence[Sequence[Sequence[int]]],
                    nvs: int, *, title: str = "") -> str:
    """Per rank the ``[NvS]`` row buffer: ``cu_seqlens[R][2*epn]`` padded group ends and
    ``zero_fill[R][2*epn][2]`` (start, count) of each group's padding rows."""
    R, G = len(cu_seqlens), len(cu_seqlens[0])
    epn = G // 2
    x0, y0, rh, width = 70.0, 50.0, 26.0, 760.0
    svg = _Svg(x0 + width + 30, y0 + R * (rh + 14) + 40)
    svg.text(svg.w / 2, 20, title or f"dispatch buffer of every rank: {nvs} rows = local groups | slot groups | tail", 13)
    sx = width / float(max(nvs, 1))
    for r in range(R):
        y = y0 + r * (rh + 14)
        svg.text(x0 - 8, y + rh / 2 + 4, f"rank {r}", 11, "end")
        svg.rect(x0, y, width, rh, "white", cls="buffer")
        start = 0
        for g in range(G):
            end = int(cu_seqlens[r][g])
            if end > start:
                zs, zc = int(zero_fill[r][g][0]), int(zero_fill[r][g][1])
                real_end = zs if zc > 0 else end
                svg.rect(x0 + start * sx, y, (real_end - start) * sx, rh, LOCAL if g < epn else SLOTG, cls="group",
                         title=f"group {g} ({'local expert' if g < epn else 'slot'} {g % epn}): rows {start}..{real_end - 1}")
                if zc > 0:
                    svg.rect(x0 + zs * sx, y, zc * sx, rh, PAD, cls="padding", title=f"{zc} zero rows")
            start = max(start, end)
        if start < nvs:
            svg.rect(x0 + start * sx, y, (nvs - start) * sx, rh, "#F7F7F7", stroke="#BBBBBB", cls="tail",
                     title=f"unused tail: {nvs - start} rows")
    ly = y0 + R * (rh + 14) + 8
    for i, (c, name) in enumerate(((LOCAL, "local expert group"), (SLOTG, "redundant expert (slot) group"),
                                   (PAD, "padding rows (zero-filled)"), ("#F7F7F7", "unused tail"))):
        svg.rect(x0 + i * 190, ly, 14, 12, c)
        svg.text(x0 + i * 190 + 20, ly + 10, name, 10, "start")
    return svg.render()


def figures_from_routing(R: int, E: int, S: int, K: int, sigma: float, token_padding: int = 8, seed: int = 0):
    """Plan a skewed synthetic routing with the CPU oracle and draw all three figures."""
    import torch

    from ..reference import nvs_rows, plan_all_ranks
    from .routing import generate_topk_routing
    topk = torch.stack([generate_topk_routing(S, K, E, R, sigma, "cpu", seed, rank=r)[0] for r in range(R)])
    tables, _ = plan_all_ranks(topk, S, K, E, token_padding)
    etc = tables.experts_to_copy.tolist()
    nvs = nvs_rows(S, K, E // R, token_padding)
    return {
        "weight_buffer.svg": pool_figure(etc),
        "grad_buffer.svg": pool_figure(etc, grads=True),
        "dispatch_buffer.svg": dispatch_figure(tables.cu_seqlens.tolist(), tables.zero_fill.tolist(), nvs),
    }


def main(argv=None) -> None:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--out", default="figure")
    ap.add_argument("--R", type=int, default=4)
    ap.add_argument("--E", type=int, default=16)
    ap.add_argument("--S", type=int, default=64)
    ap.add_argument("--K", type=int, default=4)
    ap.add_argument("--sigma", type=float, default=1.5, help="spread of the expert popularity (0 = balanced)")
    ap.add_argument("--token-padding", type=int, default=8)
    ap.add_argument("--seed", type=int, default=0)
    a = ap.parse_args(argv)
    os.makedirs(a.out, exist_ok=True)
    for name, svg in figures_from_routing(a.R, a.E, a.S, a.K, a.sigma, a.token_padding, a.seed).items():
        with open(os.path.join(a.out, name), "w") as f:
            f.write(svg)
        print(os.path.join(a.out, name))


if __name__ == "__main__":
    main()
