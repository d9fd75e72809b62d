"""The host code under the address, thread and undefined-behaviour sanitizers: builds the native
unit tests (csrc/tools/core_tests.cpp: error type, deferred calls and pools, imm counters, sharding,
host buffers, topology helpers, JSON numbers; two transfer engines driven from four threads with a
delayed and reordered domain, two-sided messages and a watched word; the all-to-all host proxy
between two one-rank nodes; the descriptor server under four fetching threads; the tokenizer's
batch encoder on six threads) with -fsanitize=<x> and runs them. The kernels themselves are
not covered: device-side checking is the epoch tags, the bounded waits and the status words."""

from __future__ import annotations

import subprocess
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent


@pytest.mark.parametrize("sanitizer", ["address", "thread", "undefined"])
def test_native_unit_tests_under_sanitizer(sanitizer: str) -> None:
    build = subprocess.run([sys.executable, str(ROOT / "build.py"), "--sanitize", sanitizer],
                           cwd=ROOT, capture_output=True, text=True)
    if build.returncode != 0 and "can link -fsanitize" in build.stderr:
        pytest.skip(f"no {sanitizer} sanitizer runtime in this toolchain")
    assert build.returncode == 0, build.stdout[-2000:] + build.stderr[-2000:]
    env = {"TSAN_OPTIONS": "halt_on_error=1", "UBSAN_OPTIONS": "halt_on_error=1:print_stacktrace=1",
           "ASAN_OPTIONS": "detect_leaks=1", "PATH": "/usr/bin:/bin"}
    run = subprocess.run([str(ROOT / "bin" / f"pplx-core-tests-{sanitizer}")], cwd=ROOT, capture_output=True,
                         text=True, env=env, timeout=300)
    report = run.stdout[-3000:] + run.stderr[-3000:]
    assert run.returncode == 0, report
    assert "0 failed" in run.stdout, report
    for marker in ("WARNING: ThreadSanitizer", "ERROR: AddressSanitizer", "ERROR: LeakSanitizer", "runtime error:"):
        assert marker not in report, report
