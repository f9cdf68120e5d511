"""Tensor-parallel decode on 2+ GPUs of one box (skipped on a single GPU): sharded model vs the unsharded CPU oracle."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("world", [2, 4, 8])
def test_tensor_parallel_matches_oracle(world):
    import torch
    if torch.cuda.device_count() < world:
        pytest.skip("needs %d GPUs" % world)
    here = os.path.dirname(os.path.abspath(__file__))
    env = dict(os.environ, NCCL_NVLS_ENABLE=os.environ.get("NCCL_NVLS_ENABLE", "0"))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(world), "--master-addr",
           "127.0.0.1", "--master-port", str(29600 + world), os.path.join(here, "tp_worker.py")]
    out = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert out.returncode == 0 and "TP_OK" in out.stdout, out.stdout[-2000:] + out.stderr[-2000:]


@pytest.mark.parametrize("world", [2, 4, 8])
def test_tensor_parallel_13b_shape_matches_oracle(world):
    """The shape the benchmark times (40 heads, 108 hidden groups of 128), cut to 2 layers: logits identical on every
    rank bit for bit and within tolerance of the unsharded CPU oracle."""
    import torch
    if torch.cuda.device_count() < world:
        pytest.skip("needs %d GPUs" % world)
    here = os.path.dirname(os.path.abspath(__file__))
    env = dict(os.environ, NCCL_NVLS_ENABLE=os.environ.get("NCCL_NVLS_ENABLE", "0"), ML2_TP_SHAPE="13b")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(world), "--master-addr",
           "127.0.0.1", "--master-port", str(29620 + world), os.path.join(here, "tp_worker.py")]
    out = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=900)
    assert out.returncode == 0 and "TP_OK" in out.stdout, out.stdout[-2000:] + out.stderr[-2000:]


def test_tensor_parallel_from_model_bin(tmp_path):
    """Two ranks load their shards from one model.bin (the reference's file layout) and match the oracle."""
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    here = os.path.dirname(os.path.abspath(__file__))
    env = dict(os.environ, NCCL_NVLS_ENABLE=os.environ.get("NCCL_NVLS_ENABLE", "0"), ML2_TP_MODEL_BIN=str(tmp_path / "model.bin"))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr",
           "127.0.0.1", "--master-port", "29611", os.path.join(here, "tp_worker.py")]
    out = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert out.returncode == 0 and "TP_OK" in out.stdout, out.stdout[-2000:] + out.stderr[-2000:]


@pytest.mark.parametrize("shape", ["small", "13b"])
def test_late_rank_runs_into_the_wait_limit_and_recovers(shape):
    """Two ranks, one of them calls Forward 1.5 s late while the wait limit is 0.2 s: every rank gets ML2_E_DEVICE from a
    kernel that gave up waiting (no fault, the context stays usable), refuses the next forward, resets, and then decodes
    the same tokens as the CPU oracle. Also on the benchmark's shape, where the roles of a CTA that has given up run
    through tiles and rows that are much larger than whatever the ring last held."""
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    here = os.path.dirname(os.path.abspath(__file__))
    env = dict(os.environ, NCCL_NVLS_ENABLE=os.environ.get("NCCL_NVLS_ENABLE", "0"), ML2_TP_LATE="1")
    if shape == "13b":
        env["ML2_TP_SHAPE"] = "13b"
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr",
           "127.0.0.1", "--master-port", "29631", os.path.join(here, "tp_worker.py")]
    out = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert out.returncode == 0 and "TP_OK" in out.stdout, out.stdout[-2000:] + out.stderr[-2000:]
