"""Multi-process CPU (gloo) tests of the engines' host-side logic: bank ownership, gradient accumulation,
reduction, re-gather, un-banked state dict.  Each test shells out to torch.distributed.run, as the reference's
distributed tests do (tests/integration/test_himuon_fsdp_parity.py), but needs no GPU."""

import os
import subprocess
import sys

import pytest

HERE = os.path.dirname(os.path.abspath(__file__))


def _run(nproc, *argv, timeout=300):
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
           "--master-addr", "127.0.0.1", "--master-port", str(29600 + os.getpid() % 300),
           os.path.join(HERE, "_dist_worker.py"), *argv]
    env = dict(os.environ, OMP_NUM_THREADS="2")
    return subprocess.run(cmd, capture_output=True, text=True, timeout=timeout, env=env)


@pytest.mark.distributed
@pytest.mark.parametrize("mode,opt,nproc", [("fsdp", "himuon", 2), ("fsdp", "muon-fsdp", 2), ("ddp", "himuon", 2),
                                            ("fsdp", "himuon", 4), ("fsdp", "adamw", 2),
                                            ("fsdp:ring:replicated", "himuon", 2), ("fsdp:gathered:sharded", "himuon", 2),
                                            ("fsdp:ring:sharded:ckpt:debug", "himuon", 2), ("fsdp:ring:sharded", "adamw", 2),
                                            ("fsdp:ring:sharded", "muon-fsdp", 3), ("ddp:overlap", "adamw", 2),
                                            ("fsdp:gathered:replicated:L7", "himuon", 4), ("fsdp:ring:sharded:L7", "himuon", 3)])
def test_multi_rank_training_matches_single_process(mode, opt, nproc):
    r = _run(nproc, "train", mode, opt)
    assert "PARITY OK" in r.stdout, r.stdout[-2000:] + r.stderr[-3000:]


@pytest.mark.distributed
def test_missing_rank_is_detected_by_collective_timeout():
    r = _run(2, "missing", "-", "-", timeout=120)
    assert "DETECTED" in r.stdout and "UNEXPECTED" not in r.stdout, r.stdout[-2000:] + r.stderr[-2000:]


@pytest.mark.distributed
def test_himuon_on_dtensor_banks_matches_per_matrix():
    r = _run(2, "dtensor", "-", "-")
    assert "PARITY OK dtensor" in r.stdout, r.stdout[-2000:] + r.stderr[-3000:]


def _cli(nproc, script, *argv, timeout=600):
    root = os.path.dirname(HERE)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}", "--master-addr", "127.0.0.1",
           "--master-port", str(29900 + os.getpid() % 90), os.path.join(root, script), *argv]
    return subprocess.run(cmd, capture_output=True, text=True, timeout=timeout, env=dict(os.environ, OMP_NUM_THREADS="2"))


@pytest.mark.distributed
@pytest.mark.parametrize("script", ["train_fsdp.py", "train_ddp.py"])
def test_cli_trains_and_saves_hf_checkpoint(tmp_path, script):
    """The real training scripts on two CPU ranks: metric lines in the reference's format, the reconfigure schedule
    firing, the stop line, and an un-banked Hugging Face checkpoint (reference: test_himuon_fsdp_smoke.py)."""
    import re

    sched = '[{"step": 0, "tile_size": 1000000000}, {"step": 2, "tile_size": 32}]'
    r = subprocess.run(
        [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
         "--master-port", str(29900 + os.getpid() % 90), os.path.join(os.path.dirname(HERE), script),
         "--model", "tiny-qwen3", "--optimizer", "himuon", "--lr", "0.01", "--dataset", "synthetic", "--steps", "4",
         "--batch-size", "2", "--max-length", "32", "--grad-acc", "2", "--device", "cpu", "--no-cuda-graph",
         "--no-gradient-checkpointing", "--reconfigure-schedule", sched, "--save-checkpoint", "--run-name", "cli_test",
         "--time-stats"],
        capture_output=True, text=True, timeout=600, cwd=str(tmp_path), env=dict(os.environ, OMP_NUM_THREADS="2"))
    log = r.stdout + r.stderr
    losses = [float(x) for x in re.findall(r"Step: \d+ LR: [0-9.]+ Training loss: ([0-9.]+), Tokens: [0-9,]+", log)]
    assert len(losses) == 4 and all(l == l for l in losses), log[-3000:]
    assert "Stopping training" in log and "reconfigure @ step 2" in log, log[-3000:]
    ckpt = tmp_path / "checkpoints" / "cli_test_step4"
    assert (ckpt / "config.json").exists() and (ckpt / "model.safetensors").exists(), log[-2000:]
    from safetensors.torch import load_file
    keys = set(load_file(str(ckpt / "model.safetensors")))
    assert "model.layers.1.self_attn.k_proj.weight" in keys and "model.layers.0.mlp.gate_proj.weight" in keys
    assert not any("bank" in k for k in keys)
