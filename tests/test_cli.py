"""Command line: the checkpoint / planner commands on CPU, the offline gates (run twice -> same hash, kv, spec, batch,
session) on a GPU with random-init weights of the plumbing config."""
import json

import pytest

from agens_engine_b200 import cli
from agens_engine_b200.models import config as C
from agens_engine_b200.models import oracle as O
from agens_engine_b200.utils import checkpoint as K


def _run(capsys, argv):
    rc = cli.main(argv)
    out = capsys.readouterr().out
    return rc, out


def test_cli_cpu_commands(tmp_path, capsys):
    ow = O.random_weights(C.oracle_tiny(), seed=0)
    d = str(tmp_path / "ckpt")
    K.save_oracle(d, ow, shards=2)
    rc, out = _run(capsys, ["validate", d])
    assert rc == 0 and json.loads(out)["ok"]
    rc, out = _run(capsys, ["verify", d])
    assert rc == 0
    rc, out = _run(capsys, ["inspect", d])
    assert rc == 0 and "linears" in out or "tensors" in out
    rc, out = _run(capsys, ["profile", "48gb"])
    assert json.loads(out)["flags"]["max_batch"] == 16
    rc, out = _run(capsys, ["plan", "--random", "dense-32b", "--budget-gib", "64", "--wctx", "131072", "--host-avail-gib", "256"])
    assert rc == 0 and "plan:" in out
    rep = json.loads(out[out.index("{"):])
    assert rep["tier"] == "gpu" and rep["pool_tokens"] >= 131072
    cfg = cli.EngineConfig.resolve(cli.argparse.Namespace(profile="24gb", tp=2, max_batch=None, wctx=4096))
    assert cfg.max_batch == 4 and cfg.wctx == 4096 and cfg.mode == "server"


@pytest.mark.gpu
def test_cli_gates_gpu(capsys):
    base = ["--random", "oracle-tiny", "--wctx", "512", "--prompt-len", "48", "--new-tokens", "24"]
    rc, a = _run(capsys, ["run"] + base)
    rc2, b = _run(capsys, ["run"] + base)
    assert rc == 0 and json.loads(a)["tokens_hash"] == json.loads(b)["tokens_hash"]
    rc, out = _run(capsys, ["kv"] + base)
    assert rc == 0 and json.loads(out)["bitwise_equal"]
    rc, out = _run(capsys, ["spec"] + base)
    assert rc == 0, out
    rc, out = _run(capsys, ["batch"] + base + ["--batch", "2,4"])
    assert rc == 0, out
    rc, out = _run(capsys, ["session"] + base)
    assert rc == 0, out
    rc, out = _run(capsys, ["load"] + base)
    assert rc == 0 and json.loads(out)["tp"] == 1
    rc, out = _run(capsys, ["spec-batch"] + base + ["--sequences", "3", "--draft-depth", "3"])
    assert rc == 0 and all(json.loads(out)[k]["equal"] for k in ("perfect", "corrupt", "garbage")), out
    assert json.loads(out)["perfect"]["tokens_per_step"] > 2.5


@pytest.mark.gpu
def test_cli_agent_replay_gpu(capsys, tmp_path):
    """Agent-session replay: growing multi-turn prompts served from one resident sequence (advance, fork, prefill the
    rest, generate) agree with prefilling every turn from scratch (first tokens; chunk sizes differ, so not bit for bit)."""
    import random
    rnd = random.Random(5)
    sessions = []
    for s_ in range(2):
        ids = [rnd.randrange(1000) for _ in range(40)]
        turns = []
        for t in range(4):
            ids = ids + [rnd.randrange(1000) for _ in range(25 + 7 * t)]       # tool results and the next question
            turns.append(ids + [rnd.randrange(1000) for _ in range(6)])       # the generation prompt of this turn only
        sessions.append(turns)
    (tmp_path / "t.json").write_text(json.dumps(sessions))
    rc, out = _run(capsys, ["agent-replay", "--random", "oracle-tiny", "--wctx", "512", "--new-tokens", "8", str(tmp_path / "t.json"),
                            str(tmp_path / "o.json"), "--check"])
    rep = json.loads(out)
    assert rc == 0 and rep["first_token_agreement"] >= 0.75 and rep["session"]["turns"] == 8, out
    rows = json.load(open(tmp_path / "o.json"))["session"]
    assert all(len(r["tokens"]) == 8 for r in rows)


def test_compare_tools(tmp_path):
    import torch
    from agens_engine_b200.tools import compare as T
    a = torch.randn(4, 100)
    torch.save(a, tmp_path / "a.pt"); torch.save(a + 1e-4 * torch.randn(4, 100), tmp_path / "b.pt")
    rep = T.compare_logits(str(tmp_path / "a.pt"), str(tmp_path / "b.pt"))
    assert rep["top1_agreement"] == 1.0 and rep["mean_kl"] < 1e-6
    (tmp_path / "x.json").write_text(json.dumps([1, 2, 3, 4]))
    (tmp_path / "y.json").write_text(json.dumps({"tokens": [1, 2, 9, 4]}))
    rep = T.compare_tokens(str(tmp_path / "x.json"), str(tmp_path / "y.json"))
    assert not rep["equal"] and rep["first_difference"] == 2 and rep["agreement"] == 0.75
    assert T.main(["tokens", str(tmp_path / "x.json"), str(tmp_path / "x.json")]) == 0


@pytest.mark.gpu
def test_cli_serve_over_http(tmp_path):
    """`serve` end to end: the process loads a model, listens, answers OpenAI requests (plain and streamed)."""
    import os
    import subprocess
    import sys
    import time
    import urllib.request
    from tests.fixtures import tiny_tokenizer_json
    tok = tmp_path / "tokenizer.json"
    tok.write_text(tiny_tokenizer_json())
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    log = open(tmp_path / "serve.log", "w")
    p = subprocess.Popen([sys.executable, "-u", "-m", "agens_engine_b200", "serve", "--random", "oracle-tiny", "--tokenizer", str(tok),
                          "--port", "0", "--wctx", "512", "--max-batch", "4", "--spec-copy", "1", "--served-model-name", "tiny",
                          "--vision", "1"],
                         cwd=root, stdout=log, stderr=subprocess.STDOUT)
    try:
        port = None
        for _ in range(240):
            time.sleep(0.5)
            txt = open(tmp_path / "serve.log").read()
            if "serving tiny on http://" in txt:
                port = int(txt.split("serving tiny on http://127.0.0.1:")[1].split()[0])
                break
            assert p.poll() is None, txt[-2000:]
        assert port, open(tmp_path / "serve.log").read()[-2000:]

        def post(path, body):
            req = urllib.request.Request(f"http://127.0.0.1:{port}{path}", data=json.dumps(body).encode(),
                                         headers={"Content-Type": "application/json"})
            with urllib.request.urlopen(req, timeout=60) as r:
                return r.status, r.read().decode()

        st, txt = post("/v1/chat/completions", {"model": "tiny", "messages": [{"role": "user", "content": "hello there"}],
                                                "max_tokens": 10, "temperature": 0})
        assert st == 200 and json.loads(txt)["usage"]["completion_tokens"] == 10
        st, txt2 = post("/v1/chat/completions", {"model": "tiny", "messages": [{"role": "user", "content": "hello there"}],
                                                 "max_tokens": 10, "temperature": 0})
        assert json.loads(txt2)["choices"][0]["message"] == json.loads(txt)["choices"][0]["message"]
        st, sse = post("/v1/completions", {"model": "tiny", "prompt": "in the", "max_tokens": 6, "stream": True})
        assert st == 200 and sse.strip().endswith("data: [DONE]") and sse.count("data: ") >= 3
        with urllib.request.urlopen(f"http://127.0.0.1:{port}/v1/models", timeout=10) as r:
            assert "tiny" in r.read().decode()
        # an image part: decoded, encoded by the vision tower and prefilled with its rows (PPM payload, 96 x 64 pixels)
        import base64
        ppm = b"P6\n96 64\n255\n" + bytes((i * 7) % 256 for i in range(64 * 96 * 3))
        url = "data:image/x-portable-pixmap;base64," + base64.b64encode(ppm).decode()
        msg = {"role": "user", "content": [{"type": "text", "text": "describe "}, {"type": "image_url", "image_url": {"url": url}}]}
        st, txt3 = post("/v1/chat/completions", {"model": "tiny", "messages": [msg], "max_tokens": 6, "temperature": 0})
        assert st == 200 and json.loads(txt3)["usage"]["completion_tokens"] == 6
        st, txt4 = post("/v1/chat/completions", {"model": "tiny", "messages": [msg], "max_tokens": 6, "temperature": 0})
        assert json.loads(txt4)["choices"][0]["message"] == json.loads(txt3)["choices"][0]["message"]
    finally:
        p.terminate()
        try:
            p.wait(timeout=20)
        except subprocess.TimeoutExpired:
            p.kill()


def test_deploy_entry_and_launcher_command_lines(tmp_path, capsys):
    """Container entry point and host launcher (reference: scripts/agens-entry.sh, scripts/agens-run.sh)."""
    from agens_engine_b200.deploy import entry, run
    a = entry.serve_argv(["--profile", "48gb", "--model", "/m", "--drafter", "/d", "--mtp", "/h", "--images", "on", "--tp", "4",
                          "--", "--max-batch", "8"])
    assert a == ["serve", "--model-dir", "/m", "--host", "0.0.0.0", "--port", "30000", "--profile", "48gb", "--vision", "1",
                 "--spec-drafter", "/d", "--mtp", "/h", "--tp", "4", "--max-batch", "8"]
    assert entry.serve_argv([])[:3] == ["serve", "--model-dir", "/model"] and "--tp" not in entry.serve_argv([])
    for bad in (["--profile", "7gb"], ["--images", "maybe"], ["--tp", "3"], ["--model"]):
        with pytest.raises(SystemExit):
            entry.serve_argv(bad)
    # the flags the entry point emits are flags `serve` knows
    from agens_engine_b200 import cli
    with pytest.raises(SystemExit) as e:
        cli.main(a + ["--help"])
    assert e.value.code == 0
    capsys.readouterr()
    d = run.docker_argv(["--model", str(tmp_path), "--tp", "2", "--gpu", "0,1", "--port", "8000", "--dry-run", "--", "--wctx", "4096"])
    assert d[:2] == ["echo", "docker"] and "--ipc=host" in d and f"{tmp_path}:/model:ro" in d and d[-3:] == ["--", "--wctx", "4096"]
    assert d[d.index("-p") + 1] == "8000:30000" and d[d.index("--tp") + 1] == "2"
    with pytest.raises(SystemExit):
        run.docker_argv(["--model", str(tmp_path), "--tp", "4", "--gpu", "0"])
    assert run.main(["--model", str(tmp_path), "--dry-run"]) == 0 and "docker run" in capsys.readouterr().out
