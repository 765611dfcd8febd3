"""Re-plot stored results without re-running: ``python -m microbench.plot --test shapes`` (or no flag: everything that
has a JSON under ``microbench/data/``).  Counterpart of the reference's ``microbench/plot.py``."""

from __future__ import annotations

import argparse
import importlib
import os

from .bench_utils import DATA_DIR, PLOTS_DIR, load_results
from .run import TESTS, _resolve


def main(argv=None):
    p = argparse.ArgumentParser()
    p.add_argument("--test", nargs="*", default=None, help="tests to re-plot (default: all with stored data)")
    p.add_argument("--data-dir", default=DATA_DIR)
    p.add_argument("--out-dir", default=PLOTS_DIR)
    args = p.parse_args(argv)
    if args.test:
        mods = [TESTS[_resolve(t)] for t in args.test]
    else:
        stored = {f[:-5] for f in os.listdir(args.data_dir) if f.endswith(".json")} if os.path.isdir(args.data_dir) else set()
        mods = [m for m in TESTS.values() if m in stored]
    for name in mods:
        mod = importlib.import_module(f"microbench.experiments.exp_{name}")
        print(f"=== {name}")
        mod.plot(load_results(name, args.data_dir)["data"], args.out_dir)


if __name__ == "__main__":
    main()
