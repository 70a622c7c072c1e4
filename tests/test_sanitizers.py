"""The native host runtime under ThreadSanitizer and AddressSanitizer.

tests/native/host_stress.cpp runs every rank of a job as a thread of one process (engines, progress threads, shared
windows, channel rings) and checks every collective's result; built with each sanitizer it must finish clean.  The
reference's CI builds its extension with sanitizers in the same spirit (tests run against an instrumented .so)."""

import os
import shutil
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CSRC = os.path.join(ROOT, "tandem_b200", "csrc")


@pytest.mark.parametrize("sanitizer", ["thread", "address"])
def test_host_runtime_is_clean_under_sanitizer(sanitizer, tmp_path):
    if shutil.which("g++") is None:
        pytest.skip("no g++")
    exe = str(tmp_path / f"host_stress_{sanitizer}")
    srcs = [os.path.join(ROOT, "tests", "native", "host_stress.cpp")] + [os.path.join(CSRC, s) for s in ("shm.cpp", "channel.cpp", "engine.cpp")]
    build = subprocess.run(["g++", "-O1", "-g", "-std=c++17", f"-fsanitize={sanitizer}", "-fno-omit-frame-pointer", "-Wno-tsan", f"-I{CSRC}",
                            *srcs, "-o", exe, "-lrt", "-lpthread"], capture_output=True, text=True)
    if build.returncode != 0 and "sanitize" in build.stderr and "cannot find" in build.stderr:
        pytest.skip(f"lib{sanitizer[0]}san is not installed")
    assert build.returncode == 0, build.stderr[-2000:]
    env = dict(os.environ, TSAN_OPTIONS="halt_on_error=0 exitcode=66", ASAN_OPTIONS="detect_leaks=1 exitcode=66")
    run = subprocess.run([exe, "4", "30"], capture_output=True, text=True, timeout=600, env=env)
    if "unexpected memory mapping" in run.stderr:  # the sanitizer runtime could not start under this kernel's ASLR settings
        pytest.skip(run.stderr.strip().splitlines()[0])
    sys.stderr.write(run.stderr[-3000:])
    assert "Sanitizer" not in run.stderr, run.stderr[-3000:]
    assert run.returncode == 0, (run.returncode, run.stdout[-500:], run.stderr[-2000:])
    assert "ok" in run.stdout
