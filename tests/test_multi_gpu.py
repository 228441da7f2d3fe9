"""Sharded training and encoding on 2, 4 and 8 GPUs (each case is skipped where fewer are visible).

Every case runs tests/multi_gpu_worker.py under torch.distributed.run, one process per GPU, and the
worker checks the merge list, the gathered symbols and the exchanged pair counts against the CPU
oracle.  NVLS is switched off for the NCCL that the processes share.
"""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _gpus():
    from gpu_bpe_b200 import _lib
    return _lib.lib().b200bpe_device_count()


def _run(world, port, **env_extra):
    if _gpus() < world:
        pytest.skip(f"needs {world} GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", **{k: str(v) for k, v in env_extra.items()})
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", str(port), os.path.join(ROOT, "tests", "multi_gpu_worker.py")]
    r = subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=900)
    if r.returncode != 0:   # the ranks' own tracebacks come before the launcher's summary
        lines = [l for l in (r.stdout + r.stderr).splitlines() if l.startswith("[rank")]
        raise AssertionError("\n".join(lines[-40:]) or (r.stdout[-3000:] + r.stderr[-3000:]))
    assert "multi-gpu ok" in r.stdout
    return r.stdout


@pytest.mark.parametrize("world", [2, 4, 8])
def test_peer_exchange_matches_oracle(world):
    """The default exchange: this library's kernels over NVLink peer memory."""
    out = _run(world, 29611)
    assert "exchange=peer" in out


def test_nccl_exchange_matches_oracle():
    out = _run(2, 29612, B200BPE_TEST_EXCHANGE="nccl")
    assert "exchange=nccl" in out


def test_nccl_exchange_bucket_overflow():
    """Exchange buckets that start far too small: the run goes through bucket overflow, resizing and
    the recount that follows."""
    _run(2, 29613, B200BPE_TEST_EXCHANGE="nccl", B200BPE_TEST_EXCHANGE_CAP=1025)


@pytest.mark.parametrize("exchange", ["peer", "nccl"])
def test_small_tables_grow_on_every_rank_together(exchange):
    """Tables forced far too small and one merge per batch: a rank's table fills up in a batch's only
    merge kernel, the status reaches every rank before the host looks at it, and all ranks grow."""
    _run(2, 29614, B200BPE_TEST_EXCHANGE=exchange, B200BPE_TEST_TABLE_LOG2=7, B200BPE_TEST_BATCH=1, B200BPE_TEST_MERGES=40,
         B200BPE_TEST_CORPUS_KIB=256)


def test_one_empty_shard():
    """Fewer word starts than ranks: the last rank's span is empty and it still takes part."""
    _run(2, 29615, B200BPE_TEST_ONE_WORD=1, B200BPE_TEST_MERGES=20)
