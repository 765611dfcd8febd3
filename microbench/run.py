"""Unified experiment runner: ``python -m microbench.run --test shapes ns_convergence`` (or ``--test all``).

Counterpart of the reference's ``microbench/run.py``: it registers the experiments by short name, forwards the common
flags (``--tile``, ``--ns-steps``, ``--warmup``, ``--repeats``, ``--models``, ``--sizes``) to each one's ``run()``,
stores the results under ``microbench/data/`` and plots them unless ``--no-plot`` is given.  The reference registers
``shapes`` and ``ns_convergence`` and leaves the other experiments stand-alone; here every experiment is registered and
each is also a module of its own with the full set of flags (``python -m microbench.experiments.exp_<name> --help``).
Timing experiments are meant for a GPU; without one ``--test all`` runs the numerics experiments only.
"""

from __future__ import annotations

import argparse
import importlib
import inspect
import sys

from .bench_utils import DATA_DIR, PLOTS_DIR, have_cuda, save_results

# short name -> module suffix; the first two are the reference's registered tests
TESTS = {
    "shapes": "real_shapes_bench",
    "ns_convergence": "ns_convergence",
    "ns_kernel": "ns_kernel_microbench",
    "optimizer_step": "optimizer_step_microbench",
    "ns5_rect": "ns5_rect_bench",
    "tile_shape_quality": "tile_shape_quality",
    "capacity_scaling": "capacity_scaling",
    "topk_recovery": "topk_recovery",
    "precision_recovery": "precision_recovery",
    "precision_descent": "precision_descent",
}
TIMING = ("shapes", "ns_kernel", "optimizer_step", "ns5_rect")      # say nothing without a GPU


def _resolve(name: str) -> str:
    if name in TESTS:
        return name
    for short, mod in TESTS.items():
        if name == mod:
            return short
    raise SystemExit(f"unknown test {name!r}; available: {', '.join(TESTS)}, all")


def _common_kwargs(args, fn) -> dict:
    """The subset of the common flags that ``fn`` takes, under the names it uses."""
    params = inspect.signature(fn).parameters
    given = {"tile": args.tile, "ns_steps": args.ns_steps, "warmup": args.warmup, "repeats": args.repeats,
             "models": args.models, "sizes": args.sizes}
    out = {k: v for k, v in given.items() if v is not None and k in params}
    if args.sizes and "D" in params:                 # ns_convergence takes the matrix side as D
        out["D"] = args.sizes[0]
    return out


def main(argv=None):
    p = argparse.ArgumentParser(description="Run microbenchmark experiments",
                                epilog=f"available tests: {', '.join(TESTS)}, all")
    p.add_argument("--test", nargs="+", required=True, help="tests to run, or 'all'")
    p.add_argument("--sizes", type=int, nargs="+", default=None)
    p.add_argument("--tile", type=int, default=None)
    p.add_argument("--ns-steps", type=int, default=None)
    p.add_argument("--warmup", type=int, default=None)
    p.add_argument("--repeats", type=int, default=None)
    p.add_argument("--models", nargs="+", default=None)
    p.add_argument("--no-plot", action="store_true")
    p.add_argument("--data-dir", default=DATA_DIR)
    p.add_argument("--out-dir", default=PLOTS_DIR)
    args = p.parse_args(argv)
    if "all" in args.test:
        names = [t for t in TESTS if have_cuda() or t not in TIMING]
    else:
        names = [_resolve(t) for t in args.test]
    for short in names:
        mod = importlib.import_module(f"microbench.experiments.exp_{TESTS[short]}")
        print(f"\n{'=' * 72}\n  {short} ({TESTS[short]})\n{'=' * 72}", flush=True)
        data = mod.run(**_common_kwargs(args, mod.run))
        print("saved", save_results(TESTS[short], data, args.data_dir), flush=True)
        if not args.no_plot:
            mod.plot(data, args.out_dir)
    print("\nall done")


if __name__ == "__main__":
    main(sys.argv[1:])
