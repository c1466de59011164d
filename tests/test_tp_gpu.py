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


def test_tp2_step_kernel_fused_all_reduce():
    _run("step")


def test_tp4_step_kernel_fused_all_reduce():
    _run("step", n=4)


def test_tp2_engine_leader_follower_and_sampling():
    _run("engine")


def test_tp2_serve_over_http(tmp_path):
    """`serve --tp 2`: rank 0 starts the other rank, schedules, answers over HTTP; a SIGTERM shuts both ranks down."""
    import json
    import time
    import urllib.request
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    from tests.fixtures import tiny_tokenizer_json
    tok = tmp_path / "tokenizer.json"
    tok.write_text(tiny_tokenizer_json())
    root = os.path.dirname(HERE)
    log = open(tmp_path / "serve.log", "w")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    env.pop("RANK", None); env.pop("WORLD_SIZE", None)
    p = subprocess.Popen([sys.executable, "-u", "-m", "agens_engine_b200", "serve", "--random", "oracle-tiny", "--tokenizer", str(tok),
                          "--port", "0", "--wctx", "512", "--max-batch", "2", "--max-convs", "0", "--tp", "2",
                          "--served-model-name", "tiny"], cwd=root, stdout=log, stderr=subprocess.STDOUT, env=env)
    try:
        port = None
        for _ in range(360):
            time.sleep(0.5)
            txt = open(tmp_path / "serve.log").read()
            if "serving tiny on http://" in txt:
                port = int(txt.split("serving tiny on http://127.0.0.1:")[1].split()[0])
                break
            assert p.poll() is None, txt[-3000:]
        assert port, open(tmp_path / "serve.log").read()[-3000:]
        req = urllib.request.Request(f"http://127.0.0.1:{port}/v1/completions", headers={"Content-Type": "application/json"},
                                     data=json.dumps({"model": "tiny", "prompt": "hello there and", "max_tokens": 8, "temperature": 0}).encode())
        with urllib.request.urlopen(req, timeout=120) as r:
            body = json.loads(r.read().decode())
        assert body["usage"]["completion_tokens"] == 8
    finally:
        p.terminate()
        try:
            p.wait(timeout=60)
        except subprocess.TimeoutExpired:
            p.kill()
    assert "Traceback" not in open(tmp_path / "serve.log").read()
