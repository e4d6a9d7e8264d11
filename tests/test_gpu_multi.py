"""Multi-GPU path: one process per GPU, peers through CUDA IPC, flags with bounded waits, NCCL
allreduce.  Needs at least 2 GPUs; NVLS is switched off so that a failing rank cannot disturb its
peers' GPUs."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _why(out):
    """The failing ranks' own tracebacks (the launcher's report after them says nothing about the cause)."""
    lines = [l for l in out.stderr.splitlines() if l.startswith("[rank") and "Warning" not in l]
    return out.stdout[-1000:] + "\n".join(lines[-40:]) if lines else out.stdout[-1500:] + out.stderr[-3000:]


def _ngpu():
    import torch
    return torch.cuda.device_count()


@pytest.mark.parametrize("world", [2, 4, 8])
def test_multi_gpu_halo_and_host_layer(world):
    if _ngpu() < world:
        pytest.skip(f"needs {world} GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", str(29600 + world), os.path.join(ROOT, "tests", "multi_worker.py")]
    out = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, _why(out)
    assert f"MULTI_OK {world}" in out.stdout


def test_data_parallel_groups_of_spatial_pairs():
    """2 data-parallel groups x 2 strips on 4 GPUs: built-in world-wide gradient exchange (graph replay) against NCCL."""
    if _ngpu() < 4:
        pytest.skip("needs 4 GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", AD_MULTI_PART="hybrid")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=4", "--master-addr", "127.0.0.1",
           "--master-port", "29611", os.path.join(ROOT, "tests", "multi_worker.py")]
    out = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, _why(out)
    assert "HYBRID_OK 4" in out.stdout


@pytest.mark.parametrize("world", [2, 4])
def test_data_parallel_workers_broadcast_and_gradient_sum(world):
    """One unpartitioned replica per GPU: broadcast init and gradient sums over the built-in exchange."""
    if _ngpu() < world:
        pytest.skip(f"needs {world} GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", AD_MULTI_PART="dp")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr", "127.0.0.1",
           "--master-port", str(29620 + world), os.path.join(ROOT, "tests", "multi_worker.py")]
    out = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, _why(out)
    assert f"DP_OK {world}" in out.stdout
