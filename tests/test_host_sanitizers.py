"""The native host library (tokenizers, file formats, CPU oracle, threaded batch loader) built
with AddressSanitizer + UndefinedBehaviorSanitizer and with ThreadSanitizer, driven by its own
self-test program with no Python in the process."""
import os
import shutil
import subprocess

import pytest

HOST = os.path.join(os.path.dirname(__file__), "..", "coeus_b200", "csrc", "host")
SOURCES = ["selftest.cpp", "tokenizers.cpp", "io.cpp", "oracle.cpp", "pipeline.cpp"]


@pytest.mark.parametrize("name,flags,env", [
    ("asan_ubsan", ["-fsanitize=address,undefined", "-fno-omit-frame-pointer"],
     {"ASAN_OPTIONS": "detect_leaks=1", "UBSAN_OPTIONS": "halt_on_error=1:print_stacktrace=1"}),
    ("tsan", ["-fsanitize=thread"], {"TSAN_OPTIONS": "halt_on_error=1"}),
])
def test_host_selftest_under_sanitizers(tmp_path, name, flags, env):
    cxx = shutil.which("g++")
    if cxx is None:
        pytest.skip("no g++")
    exe = tmp_path / f"selftest_{name}"
    cmd = [cxx, "-std=c++17", "-O1", "-g", *flags, *[os.path.join(HOST, s) for s in SOURCES],
           "-o", str(exe), "-lpthread"]
    build = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    if build.returncode != 0 and "sanitizer" in build.stderr.lower() and "cannot find" in build.stderr:
        pytest.skip("sanitizer runtime not installed")
    assert build.returncode == 0, build.stderr[-3000:]
    run = subprocess.run([str(exe), str(tmp_path)], capture_output=True, text=True, timeout=600,
                         env={**os.environ, **env})
    assert run.returncode == 0, (run.stdout + run.stderr)[-4000:]
    assert "host selftest ok" in run.stdout
