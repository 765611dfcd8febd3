"""Re-plot stored results: ``python -m microbench.plot [name ...]`` (counterpart of the reference's ``microbench/plot.py``)."""

from __future__ import annotations

import argparse
import importlib
import os

from .bench_utils import DATA_DIR, load_results


def main(argv=None):
    p = argparse.ArgumentParser()
    p.add_argument("names", nargs="*")
    p.add_argument("--plots", default=os.path.join(os.path.dirname(os.path.abspath(__file__)), "plots"))
    args = p.parse_args(argv)
    names = args.names or sorted(f[:-5] for f in os.listdir(DATA_DIR) if f.endswith(".json"))
    for name in names:
        mod = importlib.import_module(f"microbench.experiments.exp_{name}")
        print(f"=== {name}")
        mod.plot(load_results(name)["data"], args.plots)


if __name__ == "__main__":
    main()
