#!/usr/bin/env python
"""Single-process training (reference: train.py). Example: python train.py --model Qwen3-0.6B --optimizer himuon --lr 0.02 --dataset synthetic"""

from himuon_b200.trainer import build_arg_parser, run_training

if __name__ == "__main__":
    run_training(build_arg_parser("single").parse_args(), "single")
