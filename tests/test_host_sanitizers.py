"""The host-side native code (signal protocol simulation, micrograd engine) built and run under the
compiler's sanitizers: ThreadSanitizer for the multi-threaded protocol drive, AddressSanitizer and
UndefinedBehaviorSanitizer for the graph engine. CPU only; skipped where g++ has no sanitizer runtime."""
import shutil
import subprocess
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
SOURCES = [ROOT / "tests" / "native" / "host_sanitize_main.cpp", ROOT / "csrc" / "cpu" / "protocol_sim.cpp",
           ROOT / "csrc" / "cpu" / "micrograd.cpp"]


@pytest.mark.parametrize("sanitizer", ["thread", "address,undefined"])
def test_host_code_is_clean_under_sanitizers(tmp_path, sanitizer):
    gxx = shutil.which("g++")
    if gxx is None:
        pytest.skip("no g++")
    exe = tmp_path / "host_sanitize"
    build = subprocess.run([gxx, "-std=c++17", "-O1", "-g", "-fno-omit-frame-pointer", f"-fsanitize={sanitizer}",
                            "-pthread", "-I", str(ROOT / "csrc"), *map(str, SOURCES), "-o", str(exe)],
                           capture_output=True, text=True)
    if build.returncode != 0 and ("cannot find" in build.stderr or "unrecognized" in build.stderr):
        pytest.skip(f"no runtime for -fsanitize={sanitizer}: {build.stderr[-200:]}")
    assert build.returncode == 0, build.stderr[-2000:]
    run = subprocess.run([str(exe)], capture_output=True, text=True, timeout=300,
                         env={"TSAN_OPTIONS": "halt_on_error=1", "ASAN_OPTIONS": "detect_leaks=1",
                              "UBSAN_OPTIONS": "halt_on_error=1:print_stacktrace=1"})
    report = run.stdout + run.stderr
    assert run.returncode == 0, report[-3000:]
    assert "host sanitize OK" in run.stdout
    for marker in ("ThreadSanitizer", "AddressSanitizer", "LeakSanitizer", "runtime error"):
        assert marker not in report, report[-3000:]
