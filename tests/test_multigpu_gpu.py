"""Multi-GPU tests of the fused compute+collective paths; need >= 2 GPUs (skipped otherwise)."""
import json
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _torchrun(nproc, script, *args, timeout=420):
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
           "--master-addr", "127.0.0.1", "--master-port", "29531", os.path.join(ROOT, "tests", script), *args]
    return subprocess.run(cmd, capture_output=True, text=True, timeout=timeout, env=env, cwd=ROOT)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_fused_ulysses_and_cfgp_two_gpus():
    r = _torchrun(2, "mp_fused_worker.py", json.dumps([{"cp": 2}, {"cfgp": 2}, {"cp": 2, "cp_mode": "ring"}, {"tp": 2},
                                                      {"tp": 2, "presliced": True}]))
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert r.stdout.count("OK") == 5, r.stdout


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_fused_fsdp_and_allreduce_two_gpus():
    r = _torchrun(2, "mp_train_worker.py")
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert r.stdout.count("OK") == 2, r.stdout


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_fused_comm_kernels_two_gpus():
    """Reduce-scatter pull, all-reduce + residual + RMS-norm (peer loads and multimem), two decoders in turn."""
    r = _torchrun(2, "mp_comm_worker.py")
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert r.stdout.count("OK") == 3, r.stdout


@pytest.mark.skipif(torch.cuda.device_count() < 4, reason="needs 4 GPUs")
def test_fused_cfgp_x_ulysses_four_gpus():
    r = _torchrun(4, "mp_fused_worker.py", json.dumps([{"cfgp": 2, "cp": 2}, {"cp": 4}]))
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert r.stdout.count("OK") == 2, r.stdout
