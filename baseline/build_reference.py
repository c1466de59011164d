#!/usr/bin/env python
"""Builds the reference's kernel library, unmodified, for the reference arm of bench.py.

    python baseline/build_reference.py PATH_TO_THE_REFERENCE_CHECKOUT      (or set AGENS_REFERENCE_DIR)

The reference is a Rust workspace plus a CUDA/CMake project; it has no setup.py / pyproject.toml, so `pip install
--target baseline/_ref <reference>` answers "not installable", and cargo / rustc are not available offline.  Its kernel
library and C ABI (`kernels/CMakeLists.txt`, target `agens_kernels_py`) do build with CMake + nvcc: this script
configures that project out of tree for compute capability 10.0 and copies the shared library to
`baseline/_ref/libagens_kernels_py.so`.  Nothing in the reference tree is written or patched.
"""
import shutil
import subprocess
import sys
import tempfile
from pathlib import Path

HERE = Path(__file__).resolve().parent


def main() -> int:
    import os
    where = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("AGENS_REFERENCE_DIR")
    if not where:
        print("usage: python baseline/build_reference.py PATH_TO_THE_REFERENCE_CHECKOUT", file=sys.stderr)
        return 2
    ref = Path(where)
    src = ref / "kernels"
    if not (src / "CMakeLists.txt").exists():
        print(f"{src} has no CMakeLists.txt", file=sys.stderr)
        return 1
    build = Path(tempfile.mkdtemp(prefix="refbuild_"))
    cfg = ["cmake", "-G", "Ninja", "-S", str(src), "-B", str(build), "-DCMAKE_CUDA_ARCHITECTURES=100",
           "-DAGENS_BUILD_ORACLE=OFF", "-DCMAKE_BUILD_TYPE=Release", "-DCMAKE_CUDA_COMPILER=/usr/local/cuda/bin/nvcc"]
    subprocess.check_call(cfg)
    subprocess.check_call(["cmake", "--build", str(build), "--target", "agens_kernels_py", "-j", "16"])
    out = HERE / "_ref"
    out.mkdir(parents=True, exist_ok=True)
    shutil.copy2(build / "libagens_kernels_py.so", out / "libagens_kernels_py.so")
    (out / "BUILD_INFO.txt").write_text("built by baseline/build_reference.py from " + str(src) + " with: " + " ".join(cfg) + "\n")
    print("wrote", out / "libagens_kernels_py.so")
    return 0


if __name__ == "__main__":
    sys.exit(main())
