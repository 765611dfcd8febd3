"""Multi-GPU tier (needs >= 2 GPUs): the peer-memory collectives, data-parallel and bank-sharded training against a
single-process run, and detection of a missing rank through a bounded device-side wait.  Each case runs as child
processes, one per GPU, like the reference's tests/integration/test_himuon_fsdp_parity.py."""

import os
import subprocess
import sys

import pytest
import torch

pytestmark = [pytest.mark.gpu, pytest.mark.distributed]
HERE = os.path.dirname(os.path.abspath(__file__))
N_GPUS = torch.cuda.device_count() if torch.cuda.is_available() else 0
needs2 = pytest.mark.skipif(N_GPUS < 2, reason="needs at least 2 GPUs")


def _run(nproc, *argv, timeout=600):
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
           "--master-addr", "127.0.0.1", "--master-port", str(29700 + os.getpid() % 200),
           os.path.join(HERE, "_gpu_dist_worker.py"), *argv]
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    return subprocess.run(cmd, capture_output=True, text=True, timeout=timeout, env=env)


# The multicast (NVLS) cases bind every rank's memory to one NVLink multicast object.  They run only when asked for
# (HIMUON_TEST_NVLS=1): a rank that dies while bound can disturb the other GPUs of a shared machine, so the default
# multi-GPU tier, and every failure-detection case, stays on plain peer loads and stores.
nvls_opt_in = pytest.mark.skipif(os.environ.get("HIMUON_TEST_NVLS") != "1", reason="set HIMUON_TEST_NVLS=1 to run the multicast cases")


@needs2
@nvls_opt_in
def test_multicast_collectives():
    r = _run(2, "collectives", "nvls", "-")
    assert "COLLECTIVES OK" in r.stdout, r.stdout[-2000:] + r.stderr[-3000:]


@needs2
@nvls_opt_in
@pytest.mark.parametrize("mode,opt", [("fsdp:gathered:sharded:nvls", "himuon"), ("fsdp:ring:replicated:nvls", "himuon"),
                                      ("ddp:overlap:nvls", "adamw")])
def test_multicast_training_matches_single_process(mode, opt):
    r = _run(2, "train", mode, opt)
    assert "PARITY OK" in r.stdout, r.stdout[-2000:] + r.stderr[-3000:]


@needs2
def test_peer_memory_collectives():
    r = _run(min(N_GPUS, 8), "collectives", "-", "-")
    assert "COLLECTIVES OK" in r.stdout, r.stdout[-2000:] + r.stderr[-3000:]


@needs2
@pytest.mark.parametrize("mode,opt", [("fsdp", "himuon"), ("ddp", "himuon"), ("fsdp", "muon-fsdp"), ("fsdp", "adamw"),
                                      ("fsdp-peer", "himuon"), ("fsdp:ring:replicated", "himuon"),
                                      ("fsdp:gathered:replicated:graph:pull", "himuon"), ("fsdp:ring:replicated:pull", "himuon"),
                                      ("fsdp:gathered:replicated:debug:ckpt:pull", "himuon"),
                                      ("fsdp:ring:replicated:graph", "himuon"), ("fsdp:gathered:sharded", "himuon"),
                                      ("fsdp:ring:sharded:graph:ckpt:debug", "himuon"), ("fsdp:ring:sharded", "adamw"),
                                      ("fsdp:ring:sharded", "muon-fsdp"), ("ddp:overlap:graph", "himuon"),
                                      ("ddp:serial", "adamw"), ("fsdp:ring:replicated:fp32ref", "adamw"),
                                      ("ddp:overlap:fp32ref", "himuon")])
def test_multi_gpu_training_matches_single_process(mode, opt):
    r = _run(2, "train", mode, opt)
    assert "PARITY OK" in r.stdout, r.stdout[-2000:] + r.stderr[-3000:]


@pytest.mark.skipif(N_GPUS < 4, reason="needs at least 4 GPUs")
@pytest.mark.parametrize("mode,opt", [("fsdp:ring:sharded:L20", "adamw"), ("fsdp:ring:replicated:graph:L20", "himuon"),
                                      ("fsdp:gathered:replicated:L20", "himuon")])
def test_many_rank_training_matches_single_process(mode, opt):
    """All GPUs of the machine (up to 8): 20 layers are three layer groups on 8 ranks (five on 4), the last one partly
    made of pad layers, and every rank owns at most three layers of each bank."""
    r = _run(min(N_GPUS, 8), "train", mode, opt, timeout=900)
    assert "PARITY OK" in r.stdout, r.stdout[-2000:] + r.stderr[-3000:]


@needs2
def test_missing_rank_surfaces_as_status_not_hang():
    r = _run(2, "timeout", "-", "-", timeout=300)
    assert "DETECTED" in r.stdout and "UNEXPECTED" not in r.stdout, r.stdout[-2000:] + r.stderr[-2000:]
