"""Container entry point.

    python -m agens_engine_b200.deploy.entry --profile 48gb --model /model [--drafter DIR] [--mtp DIR]
                                             [--images on|off] [--tp 1|2|4|8] [-- extra serve flags]

The profiles themselves live in the engine (``serve --profile``), so a server started outside a container gets the same
flags and defaults; this module only maps the container's options onto that command and replaces itself with it.
Environment variables that are already set win over a profile's defaults.  Reference: scripts/agens-entry.sh.
"""
from __future__ import annotations

import os
import sys
from typing import List, Sequence

PORT = 30000
PROFILES = ("12gb", "16gb", "24gb", "48gb", "b200")


def serve_argv(argv: Sequence[str]) -> List[str]:
    """The ``agens_engine_b200 serve`` argument list for the entry point's own arguments (pure: testable on a CPU)."""
    opt = {"profile": "b200", "model": "/model", "drafter": "", "mtp": "", "images": "", "tp": "1"}
    extra: List[str] = []
    i = 0
    while i < len(argv):
        a = argv[i]
        if a == "--":
            extra += list(argv[i + 1:])
            break
        if a.startswith("--") and a[2:] in opt:
            if i + 1 >= len(argv):
                raise SystemExit(f"{a} needs a value")
            opt[a[2:]] = argv[i + 1]
            i += 2
            continue
        extra.append(a)
        i += 1
    if opt["profile"] not in PROFILES:
        raise SystemExit(f"--profile must be one of {', '.join(PROFILES)} (got {opt['profile']})")
    if opt["images"] not in ("", "on", "off"):
        raise SystemExit(f"--images on|off (got {opt['images']})")
    if opt["tp"] not in ("1", "2", "4", "8"):
        raise SystemExit(f"--tp 1|2|4|8 (got {opt['tp']})")
    out = ["serve", "--model-dir", opt["model"], "--host", "0.0.0.0", "--port", str(PORT), "--profile", opt["profile"]]
    if opt["images"]:
        out += ["--vision", "1" if opt["images"] == "on" else "0"]
    if opt["drafter"]:
        out += ["--spec-drafter", opt["drafter"]]
    if opt["mtp"]:
        out += ["--mtp", opt["mtp"]]
    if opt["tp"] != "1":
        out += ["--tp", opt["tp"]]
    return out + extra


def main(argv=None) -> int:
    args = serve_argv(sys.argv[1:] if argv is None else argv)
    os.execv(sys.executable, [sys.executable, "-m", "agens_engine_b200"] + args)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
