"""Multi-GPU test of the peer-memory data-parallel step (needs two CUDA devices on one node)."""

import os
import subprocess
import sys

import pytest
import torch

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_peer_data_parallel_matches_ddp():
    worker = os.path.join(os.path.dirname(os.path.abspath(__file__)), "ddp_worker.py")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    proc = subprocess.run(
        [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
         "--master-port", "29541", worker],
        capture_output=True, text=True, timeout=600, env=env,
    )  # fmt: skip
    assert proc.returncode == 0, proc.stdout[-3000:] + proc.stderr[-3000:]
    assert "identical=True" in proc.stdout, proc.stdout[-2000:]


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("name,width,tol", [("AdamW", 64, 1e-5), ("Muon", 64, 3e-2), ("SOAP", 63, 3e-2), ("PSGDKron", 64, 3e-2)])
def test_real_fsdp_matches_single_process(name, width, tol):
    """``FullyShardedDataParallel(use_orig_params=True)`` + owner repartitioning vs an un-sharded run."""
    worker = os.path.join(os.path.dirname(os.path.abspath(__file__)), "fsdp_worker.py")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    proc = subprocess.run(
        [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
         "--master-port", "29543", worker, name, str(width), "2", "3", str(tol), "norm"],
        capture_output=True, text=True, timeout=600, env=env,
    )  # fmt: skip
    assert proc.returncode == 0, proc.stdout[-3000:] + proc.stderr[-3000:]


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("name,width,tol", [("AdamW", 64, 1e-5), ("Muon", 256, 3e-2), ("SOAP", 256, 3e-2), ("PSGDKron", 256, 3e-2)])
def test_fully_shard_matches_single_process(name, width, tol):
    """``fully_shard`` (FSDP2, DTensor parameters) + owner repartitioning vs an un-sharded run; widths of 256 put the
    matrix stages on the tensor-core kernels."""
    worker = os.path.join(os.path.dirname(os.path.abspath(__file__)), "fsdp_worker.py")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    proc = subprocess.run(
        [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
         "--master-port", "29545", worker, name, str(width), "2", "3", str(tol), "norm", "fsdp2"],
        capture_output=True, text=True, timeout=600, env=env,
    )  # fmt: skip
    assert proc.returncode == 0, proc.stdout[-3000:] + proc.stderr[-3000:]


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_peer_data_parallel_covers_flags_and_second_order_chains():
    """caution, error-corrected state and parameters, ADOPT's warm-up, and owner-partitioned PSGD / SOAP state all run
    through the peer kernels (no collective fallback) with bit-identical replicas."""
    worker = os.path.join(os.path.dirname(os.path.abspath(__file__)), "ddp_variants_worker.py")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    proc = subprocess.run(
        [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
         "--master-port", "29547", worker],
        capture_output=True, text=True, timeout=900, env=env,
    )  # fmt: skip
    assert proc.returncode == 0, proc.stdout[-3000:] + proc.stderr[-3000:]
    assert proc.stdout.count("ok=True") == 5, proc.stdout[-2000:]
