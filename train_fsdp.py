#!/usr/bin/env python
"""Bank-sharded (FSDP) training, one process per GPU (reference: train_fsdp.py). Example: torchrun --standalone --nproc-per-node 8 train_fsdp.py --model Qwen3-4B --optimizer himuon --dataset synthetic --reconfigure-schedule '[{"step":0,"tile_size":1000000000},{"step":200,"tile_size":512}]'"""

from himuon_b200.trainer import build_arg_parser, run_training

if __name__ == "__main__":
    run_training(build_arg_parser("fsdp").parse_args(), "fsdp")
