"""Figure helpers of the experiments (counterpart of the reference's ``microbench/plot_style.py``).

Every chart function does two things: it always writes the plotted numbers as an aligned text table
(``<name>.txt``) into the output directory and prints it, and when matplotlib is installed it also writes
``<name>.png`` with a shared style (``Agg`` backend: the machines this runs on have no display).  matplotlib is an
optional dependency: without it the experiments still leave a readable artefact of every figure.
"""

from __future__ import annotations

import math
import os

try:
    import matplotlib

    matplotlib.use("Agg")
    import matplotlib.pyplot as plt

    HAVE_MPL = True
except Exception:  # optional dependency
    plt = None
    HAVE_MPL = False

# one colour per method, used by every figure
COLORS = {
    "muon": "#4c72b0", "himuon": "#c44e52", "legacy": "#dd8452", "himuon+graph": "#937860", "fused": "#55a868",
    "persistent": "#64b5cd", "gemm": "#8172b3", "eager": "#7f7f7f", "compile": "#b0b0b0", "adamw": "#8c8c8c",
    "fp64": "#222222", "fp32": "#4c72b0", "bf16": "#c44e52", "fp8e4m3": "#55a868", "fp8e4m3_native": "#2d7f4f",
    "full": "#4c72b0", "tile": "#c44e52",
}
TILE_COLORS = {128: "#55a868", 256: "#dd8452", 512: "#c44e52", 1024: "#8172b3"}
FIGSIZE = (5.0, 3.6)
FIGSIZE_WIDE = (9.0, 3.6)


def color_of(name, default=None):
    key = str(name).lower()
    if key in COLORS:
        return COLORS[key]
    for k, v in COLORS.items():
        if key.startswith(k):
            return v
    return default


def apply_style():
    if not HAVE_MPL:
        return
    plt.rcParams.update({
        "font.size": 9, "axes.titlesize": 10, "axes.labelsize": 9, "legend.fontsize": 8, "xtick.labelsize": 8,
        "ytick.labelsize": 8, "axes.spines.top": False, "axes.spines.right": False, "axes.grid": True,
        "grid.alpha": 0.25, "grid.linewidth": 0.5, "lines.linewidth": 1.5, "lines.markersize": 4,
        "legend.frameon": False, "figure.dpi": 100, "savefig.dpi": 200, "savefig.bbox": "tight",
    })


def _fmt(v, digits=3):
    if v is None:
        return "-"
    if isinstance(v, float):
        if math.isnan(v):
            return "nan"
        return f"{v:.{digits}g}" if (abs(v) >= 1000 or (abs(v) < 0.01 and v != 0)) else f"{v:.{digits}f}"
    return str(v)


def text_table(header, rows) -> str:
    rows = [[_fmt(c) for c in r] for r in rows]
    header = [str(h) for h in header]
    widths = [max([len(header[i])] + [len(r[i]) for r in rows]) for i in range(len(header))]
    line = "  ".join(f"{{:>{w}}}" for w in widths)
    return "\n".join([line.format(*header)] + [line.format(*r) for r in rows])


def latex_table(header, rows, caption: str = "", label: str = "") -> str:
    """A ``booktabs`` table (the precision-recovery experiment emits one, as the reference does)."""
    cols = "l" + "c" * (len(header) - 1)
    body = [" & ".join(str(h) for h in header) + r" \\", r"\midrule"]
    body += [" & ".join(_fmt(c) if not isinstance(c, str) else c for c in r) + r" \\" for r in rows]
    out = [r"\begin{table}[t]", r"\centering", rf"\begin{{tabular}}{{{cols}}}", r"\toprule", *body, r"\bottomrule",
           r"\end{tabular}"]
    if caption:
        out.append(rf"\caption{{{caption}}}")
    if label:
        out.append(rf"\label{{{label}}}")
    out.append(r"\end{table}")
    return "\n".join(out)


def write_text(out_dir: str, name: str, text: str, ext: str = "txt") -> str:
    os.makedirs(out_dir, exist_ok=True)
    path = os.path.join(out_dir, f"{name}.{ext}")
    with open(path, "w") as f:
        f.write(text + "\n")
    return path


def save_fig(fig, out_dir: str, name: str) -> str:
    os.makedirs(out_dir, exist_ok=True)
    path = os.path.join(out_dir, f"{name}.png")
    fig.savefig(path)
    plt.close(fig)
    return path


def _emit_table(out_dir, name, title, header, rows):
    text = f"# {title}\n" + text_table(header, rows)
    print(text, flush=True)
    return write_text(out_dir, name, text)


def bar_chart(labels, series: dict, ylabel: str, title: str, out_dir: str, name: str, log: bool = False,
              errors: dict | None = None, value_fmt: str | None = None, baseline: float | None = None) -> str:
    """Grouped bars: one group per label, one bar per series.  ``errors[series] = (lo, hi)`` lists draw asymmetric
    error bars (quartiles); ``value_fmt`` prints the value above each bar; ``baseline`` draws a horizontal line."""
    header = ("", *series.keys())
    rows = [(lab, *[vals[i] for vals in series.values()]) for i, lab in enumerate(labels)]
    table = _emit_table(out_dir, name, f"{title} [{ylabel}]", header, rows)
    if not HAVE_MPL:
        return table
    apply_style()
    fig, ax = plt.subplots(figsize=(max(FIGSIZE[0], 1.1 * len(labels) + 2.5), FIGSIZE[1]))
    width = 0.8 / max(1, len(series))
    for i, (sname, vals) in enumerate(series.items()):
        xs = [j + i * width for j in range(len(labels))]
        ys = [float("nan") if v is None else v for v in vals]
        err = None
        if errors and sname in errors:
            lo, hi = errors[sname]
            err = [[max(0.0, y - a) for y, a in zip(ys, lo)], [max(0.0, b - y) for y, b in zip(ys, hi)]]
        ax.bar(xs, ys, width, label=sname, color=color_of(sname), yerr=err, capsize=2, error_kw={"linewidth": 0.8})
        if value_fmt:
            for x, y in zip(xs, ys):
                if y == y:
                    ax.text(x, y, value_fmt.format(y), ha="center", va="bottom", fontsize=6)
    ax.set_xticks([j + 0.4 - width / 2 for j in range(len(labels))])
    ax.set_xticklabels([str(lab) for lab in labels], rotation=15 if len(labels) > 5 else 0)
    ax.set_ylabel(ylabel)
    ax.set_title(title)
    if log:
        ax.set_yscale("log")
    if baseline is not None:
        ax.axhline(baseline, color="#444444", linewidth=0.8, linestyle="--")
    ax.legend()
    return save_fig(fig, out_dir, name)


def line_chart(x, series: dict, xlabel: str, ylabel: str, title: str, out_dir: str, name: str, logx: bool = False,
               logy: bool = False, bands: dict | None = None, hline: float | None = None) -> str:
    """One line per series over ``x``.  ``bands[series] = (lo, hi)`` shades a region (spread over seeds)."""
    header = (xlabel, *series.keys())
    rows = [(xv, *[vals[i] if i < len(vals) else None for vals in series.values()]) for i, xv in enumerate(x)]
    table = _emit_table(out_dir, name, f"{title} [{ylabel}]", header, rows)
    if not HAVE_MPL:
        return table
    apply_style()
    fig, ax = plt.subplots(figsize=FIGSIZE)
    for sname, vals in series.items():
        c = color_of(sname)
        ax.plot(x[:len(vals)], vals, marker="o", label=sname, color=c)
        if bands and sname in bands:
            lo, hi = bands[sname]
            ax.fill_between(x[:len(vals)], lo, hi, alpha=0.15, color=c)
    ax.set_xlabel(xlabel)
    ax.set_ylabel(ylabel)
    ax.set_title(title)
    if logx:
        ax.set_xscale("log")
    if logy:
        ax.set_yscale("log")
    if hline is not None:
        ax.axhline(hline, color="#444444", linewidth=0.8, linestyle="--")
    ax.legend()
    return save_fig(fig, out_dir, name)


def heatmap(row_labels, col_labels, matrix, title: str, out_dir: str, name: str, fmt: str = "{:.2f}",
            center: float | None = None, cbar_label: str = "") -> str:
    """Annotated matrix; ``None`` cells are left blank.  ``center`` puts the middle of a diverging colour map there
    (speed-up maps: 1.0)."""
    header = ("", *col_labels)
    rows = [(r, *[None if v is None else fmt.format(v) for v in matrix[i]]) for i, r in enumerate(row_labels)]
    table = _emit_table(out_dir, name, title, header, rows)
    if not HAVE_MPL:
        return table
    import numpy as np

    apply_style()
    arr = np.array([[float("nan") if v is None else v for v in row] for row in matrix], dtype=float)
    fig, ax = plt.subplots(figsize=(0.7 * len(col_labels) + 2.5, 0.5 * len(row_labels) + 1.8))
    kw = {}
    if center is not None and np.isfinite(arr).any():
        span = max(abs(np.nanmax(arr) - center), abs(center - np.nanmin(arr)), 1e-6)
        kw = {"vmin": center - span, "vmax": center + span, "cmap": "RdBu"}
    im = ax.imshow(arr, aspect="auto", **kw)
    ax.grid(False)
    ax.set_xticks(range(len(col_labels)))
    ax.set_xticklabels([str(c) for c in col_labels])
    ax.set_yticks(range(len(row_labels)))
    ax.set_yticklabels([str(r) for r in row_labels])
    for i in range(arr.shape[0]):
        for j in range(arr.shape[1]):
            if np.isfinite(arr[i, j]):
                ax.text(j, i, fmt.format(arr[i, j]), ha="center", va="center", fontsize=7)
    ax.set_title(title)
    fig.colorbar(im, ax=ax, label=cbar_label)
    return save_fig(fig, out_dir, name)
