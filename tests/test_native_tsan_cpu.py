"""The C++ host runtime under ThreadSanitizer (no GPU involved): a standalone driver is compiled together with the pool,
token-loader and TCP-store sources with ``-fsanitize=thread`` and must finish without a reported race."""
import os
import shutil
import subprocess

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.skipif(shutil.which("g++") is None, reason="needs g++")
def test_host_runtime_has_no_data_races_under_tsan(tmp_path):
    exe = str(tmp_path / "host_race_check")
    srcs = [os.path.join(ROOT, "tests", "native", "host_race_check.cpp"), os.path.join(ROOT, "csrc", "host", "mempool.cpp"),
            os.path.join(ROOT, "csrc", "host", "token_loader.cpp"), os.path.join(ROOT, "csrc", "host", "tcp_store.cpp"),
            os.path.join(ROOT, "csrc", "host", "watchdog.cpp")]
    cmd = ["g++", "-std=c++17", "-O1", "-g", "-fsanitize=thread", "-pthread", "-I", os.path.join(ROOT, "csrc", "include"),
           "-I", os.path.join(ROOT, "csrc", "host"), *srcs, "-o", exe]
    build = subprocess.run(cmd, capture_output=True, text=True, timeout=300)
    if build.returncode != 0 and "tsan" in build.stderr.lower():
        pytest.skip("ThreadSanitizer runtime not installed")
    assert build.returncode == 0, build.stderr[-2000:]
    tokens = tmp_path / "tokens.bin"
    np.arange(4000, dtype=np.uint16).tofile(tokens)
    run = subprocess.run([exe, str(tokens)], capture_output=True, text=True, timeout=300,
                         env=dict(os.environ, TSAN_OPTIONS="halt_on_error=1 exitcode=66"))
    assert run.returncode == 0, (run.stdout + run.stderr)[-3000:]
    assert "0 inconsistencies" in run.stdout and "WARNING: ThreadSanitizer" not in run.stderr
