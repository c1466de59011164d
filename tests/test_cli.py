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
