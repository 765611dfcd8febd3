"""Headless plotting helpers (matplotlib ``Agg``), used when matplotlib is installed; otherwise the experiments
print their tables as text.  Counterpart of the reference's ``microbench/plot_style.py``."""

from __future__ import annotations

import os

try:
    import matplotlib

    matplotlib.use("Agg")
    import matplotlib.pyplot as plt

    HAVE_MPL = True
except Exception:  # matplotlib is an optional dependency
    plt = None
    HAVE_MPL = False

COLORS = {"muon": "#4c72b0", "himuon": "#c44e52", "legacy": "#dd8452", "fused": "#55a868", "gemm": "#8172b3", "eager": "#7f7f7f"}


def bar_chart(labels, series: dict, ylabel: str, title: str, path: str, log: bool = False) -> str | None:
    """Grouped bars; returns the written path, or None when matplotlib is unavailable."""
    if not HAVE_MPL:
        return None
    os.makedirs(os.path.dirname(path), exist_ok=True)
    fig, ax = plt.subplots(figsize=(1.2 * len(labels) + 3, 3.6))
    width = 0.8 / max(1, len(series))
    for i, (name, vals) in enumerate(series.items()):
        xs = [j + i * width for j in range(len(labels))]
        ax.bar(xs, vals, width, label=name, color=COLORS.get(name))
    ax.set_xticks([j + 0.4 - width / 2 for j in range(len(labels))])
    ax.set_xticklabels(labels, rotation=20)
    ax.set_ylabel(ylabel)
    ax.set_title(title)
    if log:
        ax.set_yscale("log")
    ax.legend(frameon=False)
    fig.tight_layout()
    fig.savefig(path, dpi=150)
    plt.close(fig)
    return path


def line_chart(x, series: dict, xlabel: str, ylabel: str, title: str, path: str, logx: bool = False) -> str | None:
    if not HAVE_MPL:
        return None
    os.makedirs(os.path.dirname(path), exist_ok=True)
    fig, ax = plt.subplots(figsize=(5, 3.6))
    for name, vals in series.items():
        ax.plot(x, vals, marker="o", label=name)
    ax.set_xlabel(xlabel)
    ax.set_ylabel(ylabel)
    ax.set_title(title)
    if logx:
        ax.set_xscale("log")
    ax.legend(frameon=False)
    fig.tight_layout()
    fig.savefig(path, dpi=150)
    plt.close(fig)
    return path


def text_table(header, rows) -> str:
    widths = [max(len(str(h)), *(len(str(r[i])) for r in rows)) for i, h in enumerate(header)]
    fmt = "  ".join(f"{{:>{w}}}" for w in widths)
    return "\n".join([fmt.format(*header)] + [fmt.format(*[str(c) for c in r]) for r in rows])
