"""Dependency-free drawings: Gantt charts of predicted schedules and runtime traces as SVG, and the
algorithm / executable graphs as Graphviz dot text. One lane per GPU; operators are coloured by
model, transfers are hatched grey. Reference: RPEG/utils/visualize.py (dot and Gantt writers) and
RPEG/runtime/plot_trace.py (runtime trace renderer).
"""
from __future__ import annotations

from html import escape
from typing import Dict, Iterable, List, Optional, Sequence, Tuple

from ..core.types import DeviceSpace
from ..passes.lower import ExecNodeType

MODEL_COLOURS = {"Pi": "#4c78a8", "V": "#f58518", "Ref": "#54a24b", "R": "#b279a2", "AC": "#e45756",
                 "actor": "#4c78a8", "critic": "#f58518", "reference": "#54a24b", "reward": "#b279a2", "ac_share": "#e45756"}
ROLE_SHADE = {"GEN": 1.0, "INF": 0.75, "TRAIN": 0.55}
TRANSFER_COLOUR = "#9d9d9d"


def _shade(hex_colour: str, f: float) -> str:
    r, g, b = (int(hex_colour[i:i + 2], 16) for i in (1, 3, 5))
    mix = lambda c: int(255 - (255 - c) * f)
    return f"#{mix(r):02x}{mix(g):02x}{mix(b):02x}"


def gantt_svg(bars: Sequence[Tuple[str, float, float, str, str]], lanes: Sequence[str], path: str, *, title: str = "",
              width: int = 1400, lane_h: int = 18) -> str:
    """``bars``: (lane, start_s, finish_s, colour, label). Writes the SVG and returns its text."""
    lane_index = {l: i for i, l in enumerate(lanes)}
    t_end = max((b[2] for b in bars), default=1.0) or 1.0
    left, top = 110, 34
    h = top + lane_h * len(lanes) + 30
    sx = (width - left - 20) / t_end
    out = [f'<svg xmlns="http://www.w3.org/2000/svg" width="{width}" height="{h}" font-family="monospace" font-size="10">',
           f'<rect width="{width}" height="{h}" fill="white"/>',
           f'<text x="{left}" y="16" font-size="13">{escape(title)} (makespan {t_end:.3f} s)</text>']
    for l, i in lane_index.items():
        y = top + i * lane_h
        out.append(f'<text x="4" y="{y + lane_h - 5}">{escape(l)}</text>')
        out.append(f'<line x1="{left}" y1="{y + lane_h}" x2="{width - 20}" y2="{y + lane_h}" stroke="#eee"/>')
    for k in range(11):
        x = left + (width - left - 20) * k / 10
        out.append(f'<line x1="{x:.1f}" y1="{top}" x2="{x:.1f}" y2="{h - 26}" stroke="#ddd"/>')
        out.append(f'<text x="{x - 14:.1f}" y="{h - 12}">{t_end * k / 10:.3g}s</text>')
    for lane, s, f, colour, label in bars:
        if lane not in lane_index:
            continue
        x, w = left + s * sx, max(0.6, (f - s) * sx)
        y = top + lane_index[lane] * lane_h + 2
        out.append(f'<rect x="{x:.2f}" y="{y}" width="{w:.2f}" height="{lane_h - 4}" fill="{colour}" stroke="#333" '
                   f'stroke-width="0.3"><title>{escape(label)} [{s:.4f}, {f:.4f}] s</title></rect>')
        if w > 7 * len(label) * 0.62:
            out.append(f'<text x="{x + 2:.2f}" y="{y + lane_h - 8}" fill="white">{escape(label)}</text>')
    out.append("</svg>")
    text = "\n".join(out)
    if path:
        with open(path, "w") as fh:
            fh.write(text)
    return text


def _lanes(space: DeviceSpace) -> List[str]:
    return [f"gpu:{r}:{n}:{g}" for r in range(space.R) for n in range(space.N) for g in range(space.G)]


def trace_to_gantt_svg(trace, path: str, space: DeviceSpace, title: str = "predicted schedule") -> str:
    """Gantt chart of a scheduler ``Trace`` (planner prediction)."""
    bars = []
    for node, s in trace.start.items():
        f = trace.finish[node]
        if node.kind is ExecNodeType.OP:
            model = node.model.value if node.model is not None else "Pi"
            colour = _shade(MODEL_COLOURS.get(model, "#777777"), ROLE_SHADE.get(node.role.value if node.role else "INF", 0.8))
            allocs = node.allocs
        else:
            colour = TRANSFER_COLOUR
            allocs = trace.reserved_allocations[node] if trace.reserved_allocations is not None else node.allocs[-1:]
        for a in allocs:
            for r, n, g in a.coords():
                bars.append((f"gpu:{r}:{n}:{g}", s, f, colour, node.id))
    return gantt_svg(bars, _lanes(space), path, title=title)


def runtime_trace_to_gantt_svg(events: Iterable[dict], path: str, space: Optional[DeviceSpace] = None,
                               title: str = "runtime trace") -> str:
    """Gantt chart of a JSONL runtime trace: pairs start/finish events per node and draws the bar on
    every ``gpu:*`` resource the start event lists (or on the worker lane if it lists none)."""
    starts: Dict[str, dict] = {}
    bars, lanes_seen = [], []
    t0 = None
    for e in events:
        if e.get("event") == "start":
            starts[e["node_id"]] = e
            t0 = e["timestamp"] if t0 is None else min(t0, e["timestamp"])
        elif e.get("event") == "finish" and e.get("node_id") in starts:
            s = starts.pop(e["node_id"])
            c = s.get("counters") or {}
            res = [r for r in c.get("resources", ()) if r.startswith("gpu:")] or [f"worker:{s.get('worker_id')}"]
            kind = str(c.get("kind", "op")).lower()
            colour = TRANSFER_COLOUR if kind != "op" else _shade(MODEL_COLOURS.get(c.get("model"), "#777777"),
                                                                 ROLE_SHADE.get(c.get("role"), 0.8))
            if e.get("status") != "ok":
                colour = "#d62728"
            for r in res:
                if r not in lanes_seen:
                    lanes_seen.append(r)
                bars.append((r, s["timestamp"], e["timestamp"], colour, e["node_id"]))
    t0 = t0 or 0.0
    bars = [(l, s - t0, f - t0, c, n) for l, s, f, c, n in bars]
    lanes = _lanes(space) if space is not None else sorted(lanes_seen)
    lanes = lanes + [l for l in lanes_seen if l not in lanes]
    return gantt_svg(bars, lanes, path, title=title)


def rpeg_to_dot(rpeg, path: Optional[str] = None) -> str:
    """The algorithm graph: operators as boxes coloured by model, edges labelled with containers."""
    lines = ["digraph rpeg {", "  rankdir=LR; node [shape=box, style=filled, fontname=monospace];"]
    for v in rpeg.vertices:
        colour = MODEL_COLOURS.get(v.kind.model.value, "#cccccc")
        lines.append(f'  "{v.id}" [label="{v.id}\\n{v.kind.role.value}", fillcolor="{colour}", fontcolor=white];')
    for pub, edges in ((False, rpeg.data_edges), (True, rpeg.pub_edges)):
        for e in edges:
            label = getattr(e.container, "name", str(e.container))
            lines.append(f'  "{e.src.id}" -> "{e.dst.id}" [label="{label}", style={"dashed" if pub else "solid"}];')
    lines.append("}")
    text = "\n".join(lines)
    if path:
        with open(path, "w") as fh:
            fh.write(text)
    return text


def unrolled_to_dot(unrolled, path: Optional[str] = None) -> str:
    """The template unrolled over iterations: one cluster per iteration, publication edges (weights of an earlier
    iteration's training node) dashed and labelled with the iteration they come from."""
    lines = ["digraph unrolled {", "  rankdir=LR; node [shape=box, style=filled, fontname=monospace, fontsize=9];"]
    by_k: Dict[int, list] = {}
    for n in unrolled.nodes:
        by_k.setdefault(n.k, []).append(n)
    for k in sorted(by_k):
        lines.append(f'  subgraph cluster_{k} {{ label="iteration {k}"; color="#bbbbbb";')
        for n in by_k[k]:
            colour = MODEL_COLOURS.get(n.template_vertex.kind.model.value, "#cccccc")
            lines.append(f'    "{n.id}" [fillcolor="{colour}", fontcolor=white];')
        lines.append("  }")
    for pub, edges in ((False, unrolled.data_edges), (True, unrolled.pub_edges)):
        for e in edges:
            name = getattr(e.container, "name", str(e.container))
            label = f"{name}@{e.src.k}" if pub else name
            lines.append(f'  "{e.src.id}" -> "{e.dst.id}" [label="{label}", style={"dashed" if pub else "solid"}];')
    lines.append("}")
    text = "\n".join(lines)
    if path:
        with open(path, "w") as fh:
            fh.write(text)
    return text


def exec_to_dot(executable, path: Optional[str] = None) -> str:
    """The lowered executable graph: operators as boxes, transfers as ellipses."""
    lines = ["digraph exec {", "  rankdir=LR; node [fontname=monospace, fontsize=9];"]
    for n in executable.nodes:
        if n.kind is ExecNodeType.OP:
            colour = MODEL_COLOURS.get(n.model.value if n.model else "", "#cccccc")
            lines.append(f'  "{n.id}" [shape=box, style=filled, fillcolor="{colour}", fontcolor=white];')
        else:
            lines.append(f'  "{n.id}" [shape=ellipse, label="{n.kind.value}\\n{n.label or ""}"];')
    for e in executable.edges:
        lines.append(f'  "{e.src.id}" -> "{e.dst.id}";')
    lines.append("}")
    text = "\n".join(lines)
    if path:
        with open(path, "w") as fh:
            fh.write(text)
    return text


def chart_svg(series: Sequence[Tuple[str, Sequence[Tuple[float, float]]]], path: str, *, title: str = "", xlabel: str = "", ylabel: str = "",
              log_x: bool = False, log_y: bool = False, lines: bool = True, diagonal: bool = False, width: int = 720,
              height: int = 480) -> str:
    """A small line / scatter chart as SVG: ``series`` = [(name, [(x, y), ...])]. ``diagonal`` draws y = x (for
    predicted-against-measured scatters); log axes take positive values only."""
    import math
    pts = [(x, y) for _, s in series for x, y in s if (not log_x or x > 0) and (not log_y or y > 0)]
    if not pts:
        raise ValueError("nothing to plot")
    tx = (lambda v: math.log10(v)) if log_x else (lambda v: v)
    ty = (lambda v: math.log10(v)) if log_y else (lambda v: v)
    x0, x1 = min(tx(x) for x, _ in pts), max(tx(x) for x, _ in pts)
    y0, y1 = min(ty(y) for _, y in pts), max(ty(y) for _, y in pts)
    if diagonal:
        x0 = y0 = min(x0, y0)
        x1 = y1 = max(x1, y1)
    x1, y1 = (x1 if x1 > x0 else x0 + 1.0), (y1 if y1 > y0 else y0 + 1.0)
    left, top, right, bottom = 70, 40, 20, 50
    sx = lambda v: left + (tx(v) - x0) / (x1 - x0) * (width - left - right)
    sy = lambda v: height - bottom - (ty(v) - y0) / (y1 - y0) * (height - top - bottom)
    colours = ["#4c78a8", "#f58518", "#54a24b", "#e45756", "#b279a2", "#72b7b2", "#9d755d", "#bab0ac"]
    out = [f'<svg xmlns="http://www.w3.org/2000/svg" width="{width}" height="{height}" font-family="monospace" font-size="11">',
           f'<rect width="{width}" height="{height}" fill="white"/>', f'<text x="{left}" y="20" font-size="13">{escape(title)}</text>',
           f'<rect x="{left}" y="{top}" width="{width - left - right}" height="{height - top - bottom}" fill="none" stroke="#888"/>',
           f'<text x="{(left + width - right) / 2:.0f}" y="{height - 12}" text-anchor="middle">{escape(xlabel)}</text>',
           f'<text x="14" y="{(top + height - bottom) / 2:.0f}" transform="rotate(-90 14 {(top + height - bottom) / 2:.0f})" text-anchor="middle">{escape(ylabel)}</text>']
    for k in range(6):
        fx, fy = x0 + (x1 - x0) * k / 5, y0 + (y1 - y0) * k / 5
        vx, vy = (10 ** fx if log_x else fx), (10 ** fy if log_y else fy)
        px, py = left + (width - left - right) * k / 5, height - bottom - (height - top - bottom) * k / 5
        out.append(f'<line x1="{px:.1f}" y1="{top}" x2="{px:.1f}" y2="{height - bottom}" stroke="#eee"/>')
        out.append(f'<line x1="{left}" y1="{py:.1f}" x2="{width - right}" y2="{py:.1f}" stroke="#eee"/>')
        out.append(f'<text x="{px:.1f}" y="{height - bottom + 14}" text-anchor="middle">{vx:.3g}</text>')
        out.append(f'<text x="{left - 6}" y="{py + 4:.1f}" text-anchor="end">{vy:.3g}</text>')
    if diagonal:
        out.append(f'<line x1="{left}" y1="{height - bottom}" x2="{width - right}" y2="{top}" stroke="#999" stroke-dasharray="4 3"/>')
    for i, (name, s) in enumerate(series):
        c = colours[i % len(colours)]
        ok = [(x, y) for x, y in s if (not log_x or x > 0) and (not log_y or y > 0)]
        if lines and len(ok) > 1:
            out.append(f'<polyline fill="none" stroke="{c}" stroke-width="1.5" points="' + " ".join(f"{sx(x):.1f},{sy(y):.1f}" for x, y in ok) + '"/>')
        for x, y in ok:
            out.append(f'<circle cx="{sx(x):.1f}" cy="{sy(y):.1f}" r="3" fill="{c}"><title>{escape(name)}: ({x:.4g}, {y:.4g})</title></circle>')
        out.append(f'<rect x="{width - right - 170}" y="{top + 8 + 14 * i}" width="9" height="9" fill="{c}"/>')
        out.append(f'<text x="{width - right - 156}" y="{top + 17 + 14 * i}">{escape(name)}</text>')
    out.append("</svg>")
    text = "\n".join(out)
    if path:
        with open(path, "w") as fh:
            fh.write(text)
    return text


def bars_svg(groups: Sequence[Tuple[str, Sequence[Tuple[str, float]]]], path: str, *, title: str = "", ylabel: str = "",
             width: int = 760, height: int = 420) -> str:
    """Grouped bars as SVG: ``groups`` = [(group label, [(series name, value), ...])]; a series keeps its colour
    across groups (operator-by-operator comparisons of plans, phase times at several GPU counts)."""
    names: List[str] = []
    for _, items in groups:
        for name, _ in items:
            if name not in names:
                names.append(name)
    vals = [v for _, items in groups for _, v in items]
    if not vals:
        raise ValueError("nothing to plot")
    top_v = max(max(vals), 1e-12)
    left, top, right, bottom = 70, 40, 20, 60
    pw, ph = width - left - right, height - top - bottom
    colours = ["#8c8c8c", "#4c78a8", "#e45756", "#54a24b", "#f58518", "#b279a2", "#72b7b2", "#9d755d"]
    out = [f'<svg xmlns="http://www.w3.org/2000/svg" width="{width}" height="{height}" font-family="monospace" font-size="11">',
           f'<rect width="{width}" height="{height}" fill="white"/>', f'<text x="{left}" y="20" font-size="13">{escape(title)}</text>',
           f'<text x="14" y="{top + ph / 2:.0f}" transform="rotate(-90 14 {top + ph / 2:.0f})" text-anchor="middle">{escape(ylabel)}</text>']
    for k in range(6):
        y = top + ph - ph * k / 5
        out.append(f'<line x1="{left}" y1="{y:.1f}" x2="{width - right}" y2="{y:.1f}" stroke="#eee"/>')
        out.append(f'<text x="{left - 6}" y="{y + 4:.1f}" text-anchor="end">{top_v * k / 5:.3g}</text>')
    gw = pw / max(1, len(groups))
    bw = gw * 0.8 / max(1, len(names))
    for gi, (label, items) in enumerate(groups):
        gx = left + gi * gw + gw * 0.1
        have = dict(items)
        for si, name in enumerate(names):
            if name not in have:
                continue
            h = ph * have[name] / top_v
            out.append(f'<rect x="{gx + si * bw:.1f}" y="{top + ph - h:.1f}" width="{bw * 0.92:.1f}" height="{h:.1f}" fill="{colours[si % len(colours)]}">'
                       f'<title>{escape(label)} / {escape(name)}: {have[name]:.4g}</title></rect>')
        for li, part in enumerate(str(label).split("\n")):
            out.append(f'<text x="{gx + gw * 0.4:.1f}" y="{top + ph + 14 + 12 * li}" text-anchor="middle">{escape(part)}</text>')
    for si, name in enumerate(names):
        out.append(f'<rect x="{left + 8 + 150 * si}" y="{height - 16}" width="9" height="9" fill="{colours[si % len(colours)]}"/>')
        out.append(f'<text x="{left + 22 + 150 * si}" y="{height - 7}">{escape(name)}</text>')
    out.append(f'<rect x="{left}" y="{top}" width="{pw}" height="{ph}" fill="none" stroke="#888"/>')
    out.append("</svg>")
    text = "\n".join(out)
    if path:
        with open(path, "w") as fh:
            fh.write(text)
    return text
