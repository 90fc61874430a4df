"""The host runtime headers under AddressSanitizer + UndefinedBehaviorSanitizer: the self-test binary
(csrc/selftest/rt_selftest.cpp) drives the scheduler, prefix cache, block table, JSON DOM and schema machine over random,
truncated and corrupted inputs; any report aborts it."""
import shutil
import subprocess
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]


def _compiler_with_sanitizers(tmp_path):
    for cxx in ("/usr/bin/g++", shutil.which("g++"), shutil.which("clang++")):
        if not cxx:
            continue
        probe = tmp_path / "probe.cpp"
        probe.write_text("int main() { return 0; }\n")
        r = subprocess.run([cxx, "-fsanitize=address,undefined", str(probe), "-o", str(tmp_path / "probe")],
                           capture_output=True, text=True)
        if r.returncode == 0:
            return cxx
    return None


def test_runtime_selftest_under_asan_and_ubsan(tmp_path):
    cxx = _compiler_with_sanitizers(tmp_path)
    if cxx is None:
        pytest.skip("no compiler with the sanitizer runtimes on this machine")
    exe = tmp_path / "rt_selftest"
    cmd = [cxx, "-std=c++17", "-O1", "-g", "-fsanitize=address,undefined", "-fno-sanitize-recover=all", "-pthread",
           "-I", str(ROOT / "dgpp_b200" / "csrc"), str(ROOT / "dgpp_b200" / "csrc" / "selftest" / "rt_selftest.cpp"), "-o", str(exe)]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-4000:]
    r = subprocess.run([str(exe)], capture_output=True, text=True, timeout=600,
                       env={"ASAN_OPTIONS": "detect_leaks=1:abort_on_error=0", "UBSAN_OPTIONS": "print_stacktrace=1"})
    assert r.returncode == 0, (r.stdout[-2000:], r.stderr[-4000:])
    assert "rt selftest ok" in r.stdout
