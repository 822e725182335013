"""The host I/O runtime core (csrc/io/io_core.h: async file writer, mmap token gatherer, sample / blend index
builders) built as a plain program with the address + undefined-behaviour sanitizers and with the thread sanitizer,
and run: concurrent submitters, error paths, part-crossing spans and randomised index checks must come out clean."""

import shutil
import subprocess
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
SRC = ROOT / "csrc" / "io" / "io_selftest.cpp"


@pytest.mark.parametrize("sanitizer", ["address,undefined", "thread"])
def test_io_core_under_sanitizer(tmp_path, sanitizer):
    gxx = shutil.which("g++")
    if gxx is None:
        pytest.skip("no g++")
    exe = tmp_path / "io_selftest"
    build = subprocess.run([gxx, "-std=c++17", "-O1", "-g", "-pthread", f"-fsanitize={sanitizer}",
                            "-fno-sanitize-recover=all", str(SRC), "-o", str(exe)], capture_output=True, text=True, timeout=300)
    if build.returncode != 0 and "sanitize" in build.stderr and "cannot find" in build.stderr:
        pytest.skip(f"sanitizer runtime for {sanitizer} is not installed")
    assert build.returncode == 0, build.stderr[-3000:]
    scratch = tmp_path / "scratch"
    scratch.mkdir()
    run = subprocess.run([str(exe), str(scratch)], capture_output=True, text=True, timeout=300)
    assert run.returncode == 0, run.stdout[-2000:] + run.stderr[-4000:]
    assert "all checks passed" in run.stdout
