"""Peer-memory collectives and the multi-GPU trainer (needs >= 2 GPUs in one box)."""
import os
import subprocess
import sys
from pathlib import Path

import pytest
import torch

pytestmark = pytest.mark.gpu


def _run_ranks(world, port, marker, *args, nvls="0"):
    # the in-switch paths stay off except in the test that is about them
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", PB200_NVLS=nvls, MASTER_ADDR="127.0.0.1")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", str(port),
           str(Path(__file__).parent / "_multi_gpu_worker.py"), *args]
    import signal
    import tempfile

    with tempfile.TemporaryFile("w+") as log:
        proc = subprocess.Popen(cmd, env=env, stdout=log, stderr=subprocess.STDOUT,
                                start_new_session=True)
        try:
            rc = proc.wait(timeout=240)
        except subprocess.TimeoutExpired:
            os.killpg(proc.pid, signal.SIGKILL)      # the whole process group we started
            rc = -9
        log.seek(0)
        text = log.read()
    assert rc == 0 and marker in text, text[-4000:]


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_rank_symmetric_memory_and_trainer():
    _run_ranks(2, 29517, "MULTI_GPU_OK")


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_rank_expert_parallel_moe():
    _run_ranks(2, 29519, "EP_OK", "ep")


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_rank_expert_parallel_trainer():
    _run_ranks(2, 29521, "EP_ENGINE_OK", "ep_engine")


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_rank_context_parallel_delta_rule():
    _run_ranks(2, 29523, "CP_DELTA_OK", "cp_delta")


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_rank_zigzag_context_parallel_layers():
    _run_ranks(2, 29533, "CP_ZIGZAG_OK", "cp_zigzag")


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_rank_all_gather_gemm():
    _run_ranks(2, 29525, "AG_GEMM_OK", "ag_gemm")


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_rank_context_parallel_trainer():
    _run_ranks(2, 29527, "CP_ENGINE_OK", "cp_engine")


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_rank_zero3_trainer():
    _run_ranks(2, 29529, "FSDP_ENGINE_OK", "fsdp_engine")


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_rank_nvls_multicast_paths():
    _run_ranks(2, 29531, "NVLS_OK", "nvls", nvls="1")
