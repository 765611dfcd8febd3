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
                                            ("fsdp", "himuon", 4), ("fsdp", "adamw", 2)])
def test_multi_rank_training_matches_single_process(mode, opt, nproc):
    r = _run(nproc, "train", mode, opt)
    assert "PARITY OK" in r.stdout, r.stdout[-2000:] + r.stderr[-3000:]


@pytest.mark.distributed
def test_missing_rank_is_detected_by_collective_timeout():
    r = _run(2, "missing", "-", "-", timeout=120)
    assert "DETECTED" in r.stdout and "UNEXPECTED" not in r.stdout, r.stdout[-2000:] + r.stderr[-2000:]
