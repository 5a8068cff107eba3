"""Self-contained HTML / SVG dashboards (rust-nn src/gui.rs): `ModelDashboard`, `TrainingDashboard`,
`tensor_heatmap_html`, `full_dashboard`, `launch`.

Everything renders to a string of HTML with inline SVG - no window, no display server. `launch`
writes the file; it starts a viewer (`xdg-open` / `open`) only when `open_viewer=True` is passed,
because the usual home of this framework is a headless GPU server. `ModelDashboard.from_model` and
`TrainingDashboard.from_history` build the dashboards from this package's modules and trainers.
"""
from __future__ import annotations

import html as _html
import shutil
import subprocess
import sys
from typing import List, Sequence, Tuple

import torch

_PAGE_CSS = ("body{font-family:sans-serif;background:#10131c;color:#e8e8ee;margin:0;padding:20px}h1,h2{color:#76b900}"
             ".stats{display:flex;gap:20px;margin:20px 0}.stat{background:#1b2030;border-radius:10px;padding:14px 22px}"
             ".stat-value{font-size:26px;font-weight:bold}.stat-label{color:#9aa;font-size:12px}"
             ".sec{background:#161a27;border-radius:12px;padding:16px;margin:16px 0}svg{width:100%;max-width:1100px}")


def _stat(value: str, label: str) -> str:
    return f'<div class="stat"><div class="stat-value">{value}</div><div class="stat-label">{label}</div></div>'


class ModelDashboard:
    """Boxes-and-arrows view of a layer stack. `layer(name, inp, out, init)` appends one box."""

    def __init__(self, title: str):
        self.title = title
        self.layers: List[Tuple[str, int, int]] = []

    @staticmethod
    def new(title: str) -> "ModelDashboard":
        return ModelDashboard(title)

    def layer(self, name: str, inp: int, out: int, _init: str = "") -> "ModelDashboard":
        self.layers.append((name, inp, out))
        return self

    @staticmethod
    def from_model(title: str, model) -> "ModelDashboard":
        d = ModelDashboard(title)
        for m in (model.children() if hasattr(model, "children") else []):
            name = type(m).__name__
            if hasattr(m, "in_features"):
                d.layer(name, m.in_features, m.out_features)
            else:
                d.layer(name, 0, 0)
        return d

    def param_count(self) -> int:
        return sum(i * o + o for n, i, o in self.layers if n.startswith("Linear"))

    def _svg(self) -> Tuple[str, int, int]:
        bw, bh, gap, sh = 160, 60, 50, 200
        sw = len(self.layers) * (bw + gap) + gap
        parts = []
        for i, (name, inp, out) in enumerate(self.layers):
            x, y = gap + i * (bw + gap), (sh - bh) // 2
            col = "#4A90D9" if name.startswith("Linear") else "#D94A4A" if "ReLU" in name else "#2ECC71" if "Norm" in name else "#95A5A6"
            if i > 0:
                px = gap + (i - 1) * (bw + gap) + bw
                parts.append(f'<line x1="{px}" y1="{y + bh // 2}" x2="{x}" y2="{y + bh // 2}" stroke="#555" stroke-width="2"/>')
            parts.append(f'<rect x="{x}" y="{y}" width="{bw}" height="{bh}" rx="8" fill="{col}" stroke="#333"/>')
            parts.append(f'<text x="{x + bw // 2}" y="{y + 22}" text-anchor="middle" fill="white" font-size="14">{_html.escape(name)}</text>')
            if inp > 0:
                parts.append(f'<text x="{x + bw // 2}" y="{y + 42}" text-anchor="middle" fill="#ddd" font-size="11">{inp} to {out}</text>')
        return "".join(parts), sw, sh

    def body(self) -> str:
        svg, sw, sh = self._svg()
        tp = self.param_count()
        return (f'<div class="stats">{_stat(str(len(self.layers)), "Layers")}{_stat(str(tp), "Parameters")}'
                f'{_stat(f"{tp * 4 / 1024:.1f} KB", "Size")}</div>'
                f'<svg viewBox="0 0 {sw} {sh}" xmlns="http://www.w3.org/2000/svg">{svg}</svg>')

    def render(self) -> str:
        t = _html.escape(self.title)
        return f'<!DOCTYPE html><html><head><meta charset="utf-8"><title>{t}</title><style>{_PAGE_CSS}</style></head><body><h1>{t}</h1>{self.body()}</body></html>'


class TrainingDashboard:
    """Loss curve with initial / final / improvement figures."""

    def __init__(self, title: str):
        self.title = title
        self.points: List[Tuple[int, float]] = []

    @staticmethod
    def new(title: str) -> "TrainingDashboard":
        return TrainingDashboard(title)

    def add_point(self, epoch: int, loss: float) -> None:
        self.points.append((int(epoch), float(loss)))

    @staticmethod
    def from_history(title: str, losses: Sequence[float]) -> "TrainingDashboard":
        d = TrainingDashboard(title)
        for i, l in enumerate(losses):
            d.add_point(i + 1, l)
        return d

    def body(self) -> str:
        p = self.points
        me = max(max(e for e, _ in p), 1)
        ml = max(max(l for _, l in p), 0.01)
        mn = min(l for _, l in p)
        r = max(ml - mn, 0.001)
        path = " ".join(f"{40.0 + e / me * 520.0:.1f},{40.0 + (1.0 - (l - mn) / r) * 220.0:.1f}" for e, l in p)
        il, fl = p[0][1], p[-1][1]
        imp = (1.0 - fl / il) * 100.0 if il > 0 else 0.0
        return (f'<p>{len(p)} epochs</p><div class="stats">{_stat(f"{il:.4f}", "Initial")}{_stat(f"{fl:.4f}", "Final")}'
                f'{_stat(f"{imp:.1f}%", "Improvement")}</div>'
                '<svg viewBox="0 0 600 300" xmlns="http://www.w3.org/2000/svg">'
                '<line x1="40" y1="40" x2="40" y2="260" stroke="#333"/><line x1="40" y1="260" x2="560" y2="260" stroke="#333"/>'
                f'<polyline points="{path}" fill="none" stroke="#76b900" stroke-width="2.5"/>'
                f'<text x="30" y="35" fill="#888" font-size="11">{ml:.3f}</text><text x="30" y="275" fill="#888" font-size="11">{mn:.3f}</text>'
                f'<text x="540" y="278" fill="#888" font-size="11">Epoch {me}</text></svg>')

    def render(self) -> str:
        t = _html.escape(self.title)
        if not self.points:
            return f"<html><body><h1>{t}</h1><p>No data.</p></body></html>"
        return f'<!DOCTYPE html><html><head><meta charset="utf-8"><title>Training</title><style>{_PAGE_CSS}</style></head><body><h1>{t}</h1>{self.body()}</body></html>'


def tensor_heatmap_html(tensor: torch.Tensor, max_display: int = 1024) -> str:
    """HTML table colouring the first `max_display` elements from blue (min) to red (max)."""
    flat = tensor.detach().float().reshape(-1)[:max_display].cpu()
    cols = max(tensor.shape[-1] if tensor.dim() else flat.numel(), 1)
    if flat.numel() == 0:
        return '<table style="border-collapse:collapse;font-family:monospace"><tr></tr></table>'
    mn, mx = float(flat.min()), float(flat.max())
    r = max(mx - mn, 1e-8)
    cells = []
    vals = flat.tolist()
    for i, v in enumerate(vals):
        hue = (1.0 - min(max((v - mn) / r, 0.0), 1.0)) * 240.0
        cells.append(f'<td style="background:hsl({hue:.0f},70%,50%);color:#fff;font-size:9px;text-align:center;padding:2px 4px">{v:.2f}</td>')
        if (i + 1) % cols == 0 and i + 1 < len(vals):
            cells.append("</tr><tr>")
    return f'<table style="border-collapse:collapse;font-family:monospace"><tr>{"".join(cells)}</tr></table>'


def full_dashboard(title: str, model: ModelDashboard, training: TrainingDashboard) -> str:
    t = _html.escape(title)
    tr = training.body() if training.points else "<p>No data.</p>"
    return (f'<!DOCTYPE html><html><head><meta charset="utf-8"><title>{t}</title><style>{_PAGE_CSS}</style></head><body><h1>{t}</h1>'
            f'<div class="sec"><h2>Model Architecture</h2>{model.body()}</div>'
            f'<div class="sec"><h2>Training Metrics</h2>{tr}</div></body></html>')


def launch(html: str, path: str, open_viewer: bool = False) -> None:
    """Writes `html` to `path`. With `open_viewer=True` also hands the file to the desktop's opener, if there is one."""
    with open(path, "w", encoding="utf-8") as f:
        f.write(html)
    if open_viewer:
        opener = "open" if sys.platform == "darwin" else "xdg-open"
        exe = shutil.which(opener)
        if exe:
            subprocess.Popen([exe, path], stdout=subprocess.DEVNULL, stderr=subprocess.DEVNULL)


from ._compat import install as _install  # noqa: E402

_install(globals())
