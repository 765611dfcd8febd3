"""Run experiments and store their results: ``python -m microbench.run [name ...]`` (default: all that fit the
machine; timing experiments need a GPU).  Counterpart of the reference's ``microbench/run.py``."""

from __future__ import annotations

import argparse
import importlib
import os

import torch

from .bench_utils import save_results

GPU_ONLY = ["ns_kernel_microbench", "optimizer_step_microbench", "ns5_rect_bench", "real_shapes_bench"]
ANY = ["ns_convergence", "tile_shape_quality", "capacity_scaling", "topk_recovery", "precision_recovery", "precision_descent"]


def main(argv=None):
    p = argparse.ArgumentParser()
    p.add_argument("names", nargs="*")
    p.add_argument("--plots", default=os.path.join(os.path.dirname(os.path.abspath(__file__)), "plots"))
    args = p.parse_args(argv)
    names = args.names or (GPU_ONLY + ANY if torch.cuda.is_available() else ANY)
    for name in names:
        mod = importlib.import_module(f"microbench.experiments.exp_{name}")
        print(f"=== {name}", flush=True)
        data = mod.run()
        print("saved", save_results(name, data))
        mod.plot(data, args.plots)


if __name__ == "__main__":
    main()
