"""Host-side launcher: builds (and runs) the ``docker run`` command of a serving container.

    python -m agens_engine_b200.deploy.run --profile 48gb --model DIR [--drafter DIR] [--mtp DIR] [--gpu 0 | --tp 4 --gpu 0,1,2,3]
                                           [--port 30000] [--image TAG] [--images on|off] [--dry-run] [-- extra serve flags]

The model, drafter and MTP directories are mounted read-only; ``--ipc=host`` is needed under ``--tp`` (the ranks
exchange CUDA IPC handles).  Reference: scripts/agens-run.sh.
"""
from __future__ import annotations

import argparse
import os
import shlex
import sys
from typing import List

DEFAULT_IMAGE = os.environ.get("B200E_IMAGE", "agens-engine-b200:latest")


def docker_argv(argv) -> List[str]:
    if "--" in argv:
        k = list(argv).index("--")
        argv, extra = list(argv[:k]), list(argv[k + 1:])
    else:
        argv, extra = list(argv), []
    ap = argparse.ArgumentParser(prog="agens_engine_b200.deploy.run")
    ap.add_argument("--profile", default="b200"); ap.add_argument("--model", required=True)
    ap.add_argument("--drafter"); ap.add_argument("--mtp"); ap.add_argument("--gpu", default="0")
    ap.add_argument("--port", type=int, default=30000); ap.add_argument("--image", default=DEFAULT_IMAGE)
    ap.add_argument("--images", choices=["on", "off"]); ap.add_argument("--tp", type=int, default=1)
    ap.add_argument("--dry-run", action="store_true")
    ns = ap.parse_args(argv)
    if ns.tp > 1 and len(ns.gpu.split(",")) != ns.tp:
        raise SystemExit(f"--tp {ns.tp} needs --gpu with {ns.tp} device ids (got {ns.gpu})")
    mounts, inner = ["-v", f"{os.path.abspath(ns.model)}:/model:ro"], ["--profile", ns.profile, "--model", "/model"]
    if ns.drafter:
        mounts += ["-v", f"{os.path.abspath(ns.drafter)}:/drafter:ro"]; inner += ["--drafter", "/drafter"]
    if ns.mtp:
        mounts += ["-v", f"{os.path.abspath(ns.mtp)}:/mtp:ro"]; inner += ["--mtp", "/mtp"]
    if ns.images:
        inner += ["--images", ns.images]
    if ns.tp > 1:
        inner += ["--tp", str(ns.tp)]
    cmd = ["docker", "run", "--rm", "--gpus", f'"device={ns.gpu}"', "--ipc=host", "-p", f"{ns.port}:30000"] + mounts + [ns.image] + inner
    if extra:
        cmd += ["--"] + extra
    return (["echo"] if ns.dry_run else []) + cmd


def main(argv=None) -> int:
    cmd = docker_argv(sys.argv[1:] if argv is None else argv)
    if cmd[0] == "echo":
        print(" ".join(shlex.quote(c) for c in cmd[1:]))
        return 0
    os.execvp(cmd[0], cmd)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
