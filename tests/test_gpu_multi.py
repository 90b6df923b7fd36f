"""NCCL ranks on real GPUs (skipped with fewer than two): the step loop with the CUDA kernels, each rank
checking its shard of O, lse, dQ, dK, dV against the full-tensor CPU oracle (reference test.py:164-215)."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(world, schedules, port, extra=()):
    if not torch.cuda.is_available() or torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", TORCH_SYMM_MEM_DISABLE_MULTICAST="1")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", str(port), os.path.join(ROOT, "tests", "_multi_gpu_worker.py"),
           schedules, *extra]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert r.stdout.count("RANK_OK") == world, r.stdout[-3000:]


@pytest.mark.parametrize("world", [2, 4, 8])
def test_ring_nccl(world):
    """The NCCL schedules: all-blocks-per-pass ("gather"), the reference's Q-rotating step loop ("ring") and the
    K/V-rotating ring-attention baseline ("kvring"), all against each other and the oracle."""
    _run(world, "gather,ring,kvring", 29600 + world)


@pytest.mark.parametrize("world", [2, 4, 8])
def test_peer_memory_schedule(world):
    """The exchanges done by the library's own kernels over peer-mapped memory (push form three times in a row,
    so that both buffers of every slot are reused; then the pull form), against the NCCL schedule and the oracle."""
    _run(world, "gather,p2p,p2p,p2p,p2p_pull,p2p_pull", 29650 + world)


@pytest.mark.parametrize("world", [2])
def test_hf_hooks_on_gpu_ranks(world):
    """Both Hugging Face hooks with sharded sequences on GPU ranks (global-position causal mask, per-rank rotary
    slice, K/V recompute) against the unsharded stock modules."""
    _run(world, "gather", 29700 + world, extra=("hf",))


@pytest.mark.parametrize("world", [2])
def test_host_streamed_on_gpu_ranks(world):
    """Pinned host shards in and out on every rank, consecutive steps pipelined, against the device-resident
    schedule and the oracle."""
    _run(world, "gather,hostio", 29750 + world)
