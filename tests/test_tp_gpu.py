"""Multi-GPU gates (need >= 2 GPUs on one box): bounded push collectives vs NCCL incl. the lost-message path, and the
tensor-parallel model vs the single-GPU model.  Ranks run as child processes, NVLS off, as the reference's
ak_tp_selftest / ak_tp_push_selftest do on real GPUs (kernels/src/tp_ar.cu:377-518)."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


def _run(what, n=2):
    if torch.cuda.device_count() < n:
        pytest.skip(f"needs {n} GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}", "--master-addr", "127.0.0.1",
           "--master-port", "29611", os.path.join(HERE, "tp_worker.py"), what]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=240)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert r.stdout.count(f"{what} ok") == n


def test_push_collectives_match_nccl_and_time_out_cleanly():
    _run("collectives")


def test_tp2_model_matches_single_gpu():
    _run("model")


def test_tp2_engine_leader_follower_and_sampling():
    _run("engine")
