"""Host engines under the sanitizers: ``csrc/host/stress/host_stress.cpp`` (threads hammering the host embedding table, its
memory pool and the id mapper) is built with ``-fsanitize=thread`` and with ``-fsanitize=address,undefined`` and must run
clean under both.  No GPU, no Python inside the instrumented binary."""
import os
import shutil
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SRC = os.path.join(ROOT, "csrc", "host", "stress", "host_stress.cpp")


@pytest.mark.parametrize("sanitizer", ["thread", "address,undefined"])
def test_host_engines_run_clean_under_sanitizer(sanitizer, tmp_path):
    if shutil.which("g++") is None:
        pytest.skip("no g++")
    exe = str(tmp_path / "host_stress")
    build = subprocess.run(["g++", "-std=c++17", "-O1", "-g", "-fsanitize=" + sanitizer, "-fno-omit-frame-pointer",
                            "-Wno-unknown-pragmas", "-I", os.path.join(ROOT, "csrc", "host"), SRC, "-o", exe, "-lpthread"],
                           capture_output=True, text=True, timeout=300)
    if build.returncode != 0 and "cannot find" in build.stderr:
        pytest.skip("sanitizer runtime not installed: " + build.stderr.splitlines()[-1])
    assert build.returncode == 0, build.stderr
    env = dict(os.environ, TSAN_OPTIONS="halt_on_error=1", ASAN_OPTIONS="detect_leaks=1", UBSAN_OPTIONS="halt_on_error=1")
    run = subprocess.run([exe], capture_output=True, text=True, timeout=300, env=env)
    if run.returncode != 0 and "unexpected memory mapping" in run.stderr:
        pytest.skip("ThreadSanitizer cannot map its shadow memory on this kernel")
    assert run.returncode == 0, run.stdout + run.stderr
    assert "host_stress: ok" in run.stdout
    assert "WARNING: ThreadSanitizer" not in run.stderr and "ERROR: AddressSanitizer" not in run.stderr
    assert "runtime error" not in run.stderr
