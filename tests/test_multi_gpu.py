"""Sharded training and encoding on 2 GPUs (skipped where fewer are visible)."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _gpus():
    from gpu_bpe_b200 import _lib
    return _lib.lib().b200bpe_device_count()


@pytest.mark.parametrize("world,first_cap", [(2, None), (2, 1025)])
def test_sharded_training_and_encoding_match_oracle(world, first_cap):
    """first_cap: exchange buckets that start far too small, so the run goes through bucket overflow,
    resizing and the recount that follows."""
    if _gpus() < world:
        pytest.skip(f"needs {world} GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    if first_cap:
        env["B200BPE_EXCHANGE_CAP"] = str(first_cap)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", "29611", os.path.join(ROOT, "tests", "multi_gpu_worker.py")]
    r = subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert "multi-gpu ok" in r.stdout
