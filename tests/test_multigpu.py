"""Multi-GPU tests: run only where at least two GPUs are visible (one process per GPU via torchrun)."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _torchrun(script, n, port, timeout=600):
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}", "--master-addr", "127.0.0.1",
           "--master-port", str(port), os.path.join(ROOT, "tests", script)]
    return subprocess.run(cmd, capture_output=True, text=True, timeout=timeout, env=env)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_fsdp_fused_matches_nccl_two_ranks():
    r = _torchrun("fsdp_worker.py", 2, 29741)
    assert r.returncode == 0 and "FSDP_WORKER_OK" in r.stdout, r.stdout[-3000:] + r.stderr[-3000:]


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_ddp_fused_bucket_all_reduce_matches_nccl_two_ranks():
    r = _torchrun("ddp_worker.py", 2, 29749)
    assert r.returncode == 0 and "DDP_WORKER_OK" in r.stdout, r.stdout[-3000:] + r.stderr[-3000:]


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_tensor_parallel_fused_matches_nccl_two_ranks():
    r = _torchrun("tp_worker.py", 2, 29743)
    assert r.returncode == 0 and "TP_WORKER_OK" in r.stdout, r.stdout[-3000:] + r.stderr[-3000:]


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_pipeline_1f1b_and_gpipe_over_nccl_two_stages():
    r = _torchrun("pp_worker.py", 2, 29745)
    assert r.returncode == 0 and "PP_WORKER_OK" in r.stdout, r.stdout[-3000:] + r.stderr[-3000:]


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_tensor_parallel_serving_two_ranks():
    r = _torchrun("serve_tp_worker.py", 2, 29747)
    assert r.returncode == 0 and "SERVE_TP_WORKER_OK" in r.stdout, r.stdout[-3000:] + r.stderr[-3000:]
