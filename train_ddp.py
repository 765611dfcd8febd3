#!/usr/bin/env python
"""Data-parallel training, one process per GPU (reference: train_ddp.py). Example: torchrun --standalone --nproc-per-node 8 train_ddp.py --model Qwen3-0.6B --optimizer himuon --dataset synthetic"""

from himuon_b200.trainer import build_arg_parser, run_training

if __name__ == "__main__":
    run_training(build_arg_parser("ddp").parse_args(), "ddp")
