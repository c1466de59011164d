"""Sanitizer runs of the host-side C++ (no GPU needed).  The reference has no sanitizer configuration; its host side is
Rust.  Here the host side is C++, so the checks Rust gives for free are run as tools:

* ``asan-tests``    build the host sources with AddressSanitizer + UBSan and run the CPU test suite against that build
                    (the tests pick it up through ``B200E_HOST_LIB``);
* ``fuzz-images``   mutate seed images (written with Pillow) and run them through the image decoders of that build;
* ``tsan-listener`` the HTTP listener and the callback backend under ThreadSanitizer with concurrent clients;
* ``tsan-model``    the collectives' inbox protocol model on CPU threads under ThreadSanitizer;
* ``all``           the four above.

    python -m agens_engine_b200.tools.sanitize all [--work DIR] [--iterations N]

Each command prints one line per step and exits non-zero when a sanitizer reported or a check failed."""
from __future__ import annotations

import argparse
import concurrent.futures as cf
import os
import subprocess
import sys
import tempfile
from pathlib import Path

ROOT = Path(__file__).resolve().parents[2]
CSRC = ROOT / "csrc"
DRIVERS = Path(__file__).resolve().parent / "sanitize_drivers"


def _gcc_lib(name: str) -> str:
    return subprocess.run(["gcc", f"-print-file-name={name}"], capture_output=True, text=True, check=True).stdout.strip()


def _run(cmd, env=None, timeout=3600) -> subprocess.CompletedProcess:
    return subprocess.run([str(c) for c in cmd], capture_output=True, text=True, env=env, timeout=timeout)


def _host_sources():
    return sorted(CSRC.rglob("*.cpp"))


def build_asan(work: Path) -> Path:
    """The host library with -fsanitize=address,undefined; objects are compiled in parallel."""
    obj = work / "asan_obj"
    obj.mkdir(parents=True, exist_ok=True)
    flags = ["-std=c++17", "-O1", "-g", "-fsanitize=address,undefined", "-fno-omit-frame-pointer", "-fPIC", "-I", str(CSRC)]

    def one(src: Path):
        o = obj / (src.stem + ".o")
        r = _run(["g++", *flags, "-c", src, "-o", o])
        if r.returncode:
            raise RuntimeError(r.stderr[-4000:])
        return o
    with cf.ThreadPoolExecutor(max_workers=os.cpu_count() or 4) as ex:
        objs = list(ex.map(one, _host_sources()))
    lib = work / "libagens_b200_host_asan.so"
    r = _run(["g++", "-shared", "-fsanitize=address,undefined", "-o", lib, *objs, "-lpthread", "-ldl"])
    if r.returncode:
        raise RuntimeError(r.stderr[-4000:])
    return lib


def _san_env(lib: Path | None = None) -> dict:
    env = dict(os.environ)
    env["ASAN_OPTIONS"] = "detect_leaks=0:allocator_may_return_null=1"
    env["UBSAN_OPTIONS"] = "print_stacktrace=1:halt_on_error=1"
    env["PYTHONPATH"] = str(ROOT) + os.pathsep + env.get("PYTHONPATH", "")
    if lib is not None:
        env["B200E_HOST_LIB"] = str(lib)
        env["LD_PRELOAD"] = _gcc_lib("libasan.so") + ":" + _gcc_lib("libubsan.so")
    return env


def _reported(text: str) -> bool:
    return "ERROR: AddressSanitizer" in text or "runtime error:" in text or "WARNING: ThreadSanitizer" in text


def asan_tests(work: Path) -> bool:
    lib = build_asan(work)
    # the tensor-parallel driver test spawns ranks by re-importing its main module: not under a preloaded runtime
    r = _run([sys.executable, "-m", "pytest", str(ROOT / "tests"), "-x", "-q", "-m", "not gpu", "-p", "no:cacheprovider",
              "--ignore", str(ROOT / "tests" / "test_tp_driver_cpu.py")], env=_san_env(lib))
    out = r.stdout + r.stderr
    ok = r.returncode == 0 and not _reported(out)
    print(f"asan-tests: {'ok' if ok else 'FAILED'}: {out.strip().splitlines()[-1] if out.strip() else ''}")
    if not ok:
        print(out[-6000:])
    return ok


def _seed_images(d: Path):
    import numpy as np
    from PIL import Image
    rng = np.random.default_rng(0)
    d.mkdir(parents=True, exist_ok=True)

    def img(h, w, mode="RGB"):
        y, x = np.mgrid[0:h, 0:w]
        a = np.stack([(x * 7 + y * 3) % 256, (x * 2 + y * 5) % 256, (x + y) % 256], -1).astype(np.uint8)
        return Image.fromarray((a // 2 + rng.integers(0, 128, a.shape)).astype(np.uint8)).convert(mode)
    items = [("jpg", img(33, 47), dict(quality=80)), ("jpg", img(64, 64), dict(quality=90, subsampling=0)),
             ("jpg", img(37, 29), dict(progressive=True, quality=85)), ("jpg", img(64, 48, "L"), {}), ("jpg", img(30, 30, "CMYK"), {}),
             ("jpg", img(50, 70), dict(progressive=True, subsampling=2, quality=50)), ("webp", img(33, 47), dict(lossless=True)),
             ("webp", img(120, 90), dict(lossless=True, quality=100, method=6)), ("webp", img(64, 64).quantize(16).convert("RGB"), dict(lossless=True)),
             ("webp", img(33, 47, "RGBA"), dict(lossless=True)), ("gif", img(33, 47).quantize(64), {}),
             ("gif", img(40, 30).quantize(256), dict(interlace=True)), ("bmp", img(33, 47), {}), ("bmp", img(33, 47, "L"), {}),
             ("bmp", img(33, 47).quantize(16), {})]
    for i, (ext, im, kw) in enumerate(items):
        im.save(d / f"{i:02d}.{ext}", **kw)


def fuzz_images(work: Path, iterations: int) -> bool:
    lib = build_asan(work)
    seeds = work / "image_seeds"
    _seed_images(seeds)
    exe = work / "image_fuzz"
    r = _run(["g++", "-std=c++17", "-O1", "-g", "-fsanitize=address,undefined", DRIVERS / "image_fuzz.cpp", "-o", exe, lib,
              f"-Wl,-rpath,{work}"])
    if r.returncode:
        raise RuntimeError(r.stderr[-4000:])
    env = _san_env()
    ok = True
    with cf.ThreadPoolExecutor(max_workers=4) as ex:
        for seed, res in zip(range(1, 5), ex.map(lambda s: _run([exe, seeds, iterations, s], env=env), range(1, 5))):
            out = res.stdout + res.stderr
            good = res.returncode == 0 and not _reported(out)
            ok &= good
            print(f"fuzz-images seed {seed}: {'ok' if good else 'FAILED'}: {out.strip().splitlines()[-1] if out.strip() else ''}")
            if not good:
                print(out[-4000:])
    return ok


def _tsan(work: Path, name: str, sources, args=()) -> bool:
    exe = work / name
    r = _run(["g++", "-std=c++17", "-O1", "-g", "-fsanitize=thread", "-fPIC", "-pthread", *sources, "-I", CSRC, "-o", exe, "-ldl"])
    if r.returncode:
        raise RuntimeError(r.stderr[-4000:])
    env = dict(os.environ)
    env["TSAN_OPTIONS"] = "halt_on_error=0"
    res = _run([exe, *args], env=env)
    out = res.stdout + res.stderr
    ok = res.returncode == 0 and not _reported(out)
    print(f"{name}: {'ok' if ok else 'FAILED'}: {res.stdout.strip().splitlines()[-1] if res.stdout.strip() else ''}")
    if not ok:
        print(out[-6000:])
    return ok


def tsan_listener(work: Path) -> bool:
    sys.path.insert(0, str(ROOT))
    from tests.fixtures import tiny_tokenizer_json
    tok = work / "tokenizer.json"
    tok.write_text(tiny_tokenizer_json())
    srv = CSRC / "server"
    return _tsan(work, "tsan-listener", [DRIVERS / "listener_tsan.cpp", srv / "server.cpp", srv / "text.cpp", srv / "jinja.cpp"], [tok])


def tsan_model(work: Path) -> bool:
    return _tsan(work, "tsan-model", [DRIVERS / "model_tsan.cpp", CSRC / "comm" / "protocol_model.cpp"])


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="sanitize", description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("what", choices=["asan-tests", "fuzz-images", "tsan-listener", "tsan-model", "all"])
    ap.add_argument("--work", default="", help="build directory (default: a temporary one)")
    ap.add_argument("--iterations", type=int, default=100000, help="mutations per fuzzing seed")
    ns = ap.parse_args(argv)
    with tempfile.TemporaryDirectory() as tmp:
        work = Path(ns.work or tmp)
        work.mkdir(parents=True, exist_ok=True)
        steps = {"asan-tests": lambda: asan_tests(work), "fuzz-images": lambda: fuzz_images(work, ns.iterations),
                 "tsan-listener": lambda: tsan_listener(work), "tsan-model": lambda: tsan_model(work)}
        names = list(steps) if ns.what == "all" else [ns.what]
        ok = all([steps[n]() for n in names])
    return 0 if ok else 1


if __name__ == "__main__":
    sys.exit(main())
