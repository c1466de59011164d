"""The sanitizer tool (agens_engine_b200/tools/sanitize.py): the protocol model under ThreadSanitizer runs with the
suite; the longer steps (the whole CPU suite against an AddressSanitizer build, image fuzzing, the listener under
ThreadSanitizer: about two minutes) run when B200E_RUN_SANITIZERS=1."""
import os
import shutil
import subprocess

import pytest

from agens_engine_b200.tools import sanitize


def _has(lib: str) -> bool:
    if shutil.which("g++") is None:
        return False
    p = subprocess.run(["gcc", f"-print-file-name={lib}"], capture_output=True, text=True).stdout.strip()
    return os.path.isabs(p) and os.path.exists(p)


@pytest.mark.skipif(not _has("libtsan.so"), reason="no ThreadSanitizer runtime")
def test_protocol_model_under_thread_sanitizer(tmp_path):
    assert sanitize.main(["tsan-model", "--work", str(tmp_path)]) == 0


@pytest.mark.skipif(os.environ.get("B200E_RUN_SANITIZERS") != "1" or not _has("libasan.so"), reason="set B200E_RUN_SANITIZERS=1")
def test_all_sanitizer_steps(tmp_path):
    assert sanitize.main(["all", "--work", str(tmp_path), "--iterations", "30000"]) == 0
