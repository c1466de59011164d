"""In-tree build of the native libraries.

Two shared objects are produced under ``agens_engine_b200/lib``:

* ``libagens_b200.so``      - every ``.cu`` under ``csrc/`` compiled by nvcc for sm_100a (kernels, comm, runtime),
  plus the host-only C++ sources.  Linked against cudart only; loads on a machine without a GPU.
* ``libagens_b200_host.so`` - the host-only C++ sources (core, sched, server) compiled by g++, for CPU tests.

The reference builds its kernels with CMake (``kernels/CMakeLists.txt``); here a small dependency-aware driver
compiles translation units in parallel so that a rebuild after touching one kernel takes seconds.
"""
from __future__ import annotations

import concurrent.futures as cf
import hashlib
import os
import shutil
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
CSRC = ROOT / "csrc"
LIBDIR = Path(__file__).resolve().parent / "lib"
OBJDIR = ROOT / "build" / "obj"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
    "-Xcompiler", "-Wall", "-Xcompiler", "-Wno-unused-function",
]
CXX_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-fvisibility=hidden", "-Wall", "-pthread"]


def _nvcc() -> str:
    for c in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", shutil.which("nvcc")):
        if c and os.path.exists(c):
            return c
    raise RuntimeError("nvcc not found")


def _sources():
    cu = sorted(CSRC.rglob("*.cu"))
    cpp = sorted(CSRC.rglob("*.cpp"))
    return cu, cpp


def _headers_digest() -> str:
    h = hashlib.sha256()
    for p in sorted(list(CSRC.rglob("*.cuh")) + list(CSRC.rglob("*.h")) + list(CSRC.rglob("*.hpp"))):
        h.update(p.read_bytes())
    return h.hexdigest()


def _stamp(src: Path, flags, hdig: str) -> str:
    h = hashlib.sha256()
    h.update(src.read_bytes())
    h.update(" ".join(flags).encode())
    h.update(hdig.encode())
    return h.hexdigest()


def _text_with_includes(src: Path, seen=None) -> str:
    """The source's text followed by the text of the headers of this tree that it includes (quoted includes)."""
    import re
    seen = seen if seen is not None else set()
    if src in seen or not src.exists():
        return ""
    seen.add(src)
    text = src.read_text(errors="ignore")
    out = [text]
    for inc in re.findall(r'#include\s+"([^"]+)"', text):
        for base in (src.parent, CSRC):
            h = (base / inc).resolve()
            if h.exists():
                out.append(_text_with_includes(h, seen))
                break
    return "\n".join(out)


def _compile(cmd, obj: Path, stamp: str, verbose: bool, force: bool = False):
    stamp_file = obj.with_suffix(obj.suffix + ".stamp")
    if not force and obj.exists() and stamp_file.exists() and stamp_file.read_text() == stamp:
        return obj, "", False
    obj.parent.mkdir(parents=True, exist_ok=True)
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("compile failed: %s\n%s\n%s" % (" ".join(map(str, cmd)), r.stdout, r.stderr))
    stamp_file.write_text(stamp)
    return obj, (r.stdout + r.stderr) if verbose else "", True


def build(verbose: bool = False, ptxas_info: bool = False, jobs: int | None = None, force: bool = False,
          only: str | None = None) -> dict:
    """Compile everything that changed; returns {"cuda": path, "host": path}."""
    cu, cpp = _sources()
    hdig = _headers_digest()
    nvcc = _nvcc()
    inc = ["-I", str(CSRC)]
    # extra defines for measurement builds (e.g. B200E_NVCC_DEFS="-DB2_STEP_TRACE"); production builds leave it unset
    nv_flags = NVCC_FLAGS + (["-Xptxas", "-v"] if ptxas_info else [])
    extra = os.environ.get("B200E_NVCC_DEFS", "").split()
    tasks = []
    for s in cu:
        rel = s.relative_to(CSRC)
        obj = OBJDIR / "cuda" / rel.with_suffix(".o")
        text = _text_with_includes(s)
        # a measurement define only rebuilds the sources that mention it (themselves or through their own headers)
        flags = nv_flags + [d for d in extra if d[2:].split("=")[0] in text]
        tasks.append(([nvcc, *flags, *inc, "-c", str(s), "-o", str(obj)], obj, _stamp(s, flags, hdig)))
    for s in cpp:
        rel = s.relative_to(CSRC)
        obj = OBJDIR / "host" / rel.with_suffix(".o")
        tasks.append((["g++", *CXX_FLAGS, *inc, "-c", str(s), "-o", str(obj)], obj, _stamp(s, CXX_FLAGS, hdig)))
    logs = []
    rebuilt = False
    with cf.ThreadPoolExecutor(max_workers=jobs or os.cpu_count() or 4) as ex:
        futs = [ex.submit(_compile, cmd, obj, st, verbose or ptxas_info, force and (only is None or only in str(obj)))
                for cmd, obj, st in tasks]
        for f in futs:
            _obj, log, did = f.result()
            rebuilt |= did
            if log:
                logs.append(log)
    LIBDIR.mkdir(parents=True, exist_ok=True)
    cuda_objs = [str(OBJDIR / "cuda" / s.relative_to(CSRC).with_suffix(".o")) for s in cu]
    host_objs = [str(OBJDIR / "host" / s.relative_to(CSRC).with_suffix(".o")) for s in cpp]
    lib_cuda = LIBDIR / "libagens_b200.so"
    lib_host = LIBDIR / "libagens_b200_host.so"
    if rebuilt or not lib_cuda.exists():
        cmd = [nvcc, "-shared", "-o", str(lib_cuda), *cuda_objs, *host_objs, "-lcudart", "-lpthread", "-ldl"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("link failed:\n" + r.stdout + r.stderr)
    if host_objs and (rebuilt or not lib_host.exists()):
        cmd = ["g++", "-shared", "-o", str(lib_host), *host_objs, "-lpthread", "-ldl"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("link failed:\n" + r.stdout + r.stderr)
    if logs and (verbose or ptxas_info):
        sys.stderr.write("\n".join(logs))
    return {"cuda": lib_cuda, "host": lib_host if host_objs else None}


if __name__ == "__main__":
    only = next((a.split("=", 1)[1] for a in sys.argv if a.startswith("--only=")), None)
    out = build(verbose="-v" in sys.argv, ptxas_info="--ptxas" in sys.argv, force="--force" in sys.argv, only=only)
    print(out)
