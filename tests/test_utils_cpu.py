"""CPU tests of the small utilities: math helpers and Statistics, logging set-up, dtype names,
and the descriptor transport used to share CUDA allocations between processes (exercised here
with a pipe instead of a CUDA handle, so it needs no GPU)."""

import io
import logging
import multiprocessing as mp
import os

import pytest
import torch

from pplx_garden import _native
from pplx_garden.utils import logging_utils
from pplx_garden.utils.math import Statistics, ceil_div, floor_div, mean, mean_and_stddev, round_up, stddev
from pplx_garden.utils.torch import str_to_dtype, type_to_str


def test_integer_helpers():
    assert round_up(0, 8) == 0 and round_up(1, 8) == 8 and round_up(16, 8) == 16
    assert ceil_div(0, 4) == 0 and ceil_div(1, 4) == 1 and ceil_div(8, 4) == 2 and ceil_div(9, 4) == 3
    assert floor_div(9, 4) == 2


def test_mean_and_stddev():
    xs = [1.0, 2.0, 3.0, 4.0]
    assert mean(xs) == 2.5
    m, s = mean_and_stddev(xs)
    assert m == 2.5 and s == pytest.approx(stddev(xs))
    assert stddev([5.0]) == 0.0


def test_statistics_percentiles_are_ordered():
    xs = [float(i) for i in range(1, 1001)]
    st = Statistics.create(xs)
    assert st.min == 1.0 and st.max == 1000.0
    assert st.min <= st.p01 <= st.p25 <= st.p50 <= st.p75 <= st.p95 <= st.p99 <= st.max
    assert st.mean == pytest.approx(500.5)
    assert abs(st.p50 - 500.5) <= 1.0
    assert "p50" in str(st) or "50" in str(st)


def test_dtype_names_round_trip():
    assert str_to_dtype("bfloat16") is torch.bfloat16
    assert str_to_dtype("float8_e4m3fn") is torch.float8_e4m3fn
    with pytest.raises(ValueError):
        str_to_dtype("float7")
    assert type_to_str(torch.bfloat16) == "BFP16"
    assert type_to_str(torch.float8_e4m3fn) == "FP8"


def test_logging_setup_is_idempotent_and_formats(monkeypatch):
    monkeypatch.delenv("DD_ENV", raising=False)
    buf = io.StringIO()
    logging_utils.setup(logging.INFO, stream=buf)
    logging_utils.setup(logging.INFO, stream=buf)
    ours = [h for h in logging.getLogger().handlers if getattr(h, "_pplx_garden", False)]
    assert len(ours) == 1
    logging_utils.get_logger("pplx.test").info("hello %d", 7)
    line = buf.getvalue().strip().splitlines()[-1]
    assert "INFO" in line and "pplx.test" in line and line.endswith("hello 7")
    assert "\x1b[" not in line   # not a terminal: no colour codes
    logging.getLogger().removeHandler(ours[0])


def test_logging_plain_mode(monkeypatch):
    monkeypatch.setenv("DD_ENV", "prod")
    buf = io.StringIO()
    logging_utils.setup(logging.WARNING, stream=buf)
    logging_utils.get_logger("pplx.test").warning("careful")
    assert "WARNING" in buf.getvalue() and "careful" in buf.getvalue()
    for h in list(logging.getLogger().handlers):
        if getattr(h, "_pplx_garden", False):
            logging.getLogger().removeHandler(h)


def _exporter(conn) -> None:
    # child: owns a pipe, registers its read end with the descriptor server and tells the parent
    r, w = os.pipe()
    _native._fd_server_register(r)
    os.write(w, b"through the fence")
    conn.send((os.getpid(), r, _native._fd_server_name()))
    conn.recv()   # stay alive until the parent has fetched
    _native._fd_server_unregister(r)


@pytest.mark.parametrize("mode", ["socket", "auto"])
def test_fd_fetch_from_another_process(mode):
    ctx = mp.get_context("spawn")
    parent, child = ctx.Pipe()
    proc = ctx.Process(target=_exporter, args=(child,))
    proc.start()
    try:
        pid, fd, name = parent.recv()
        _native._fd_fetch_set_mode(mode)
        got = _native._fd_fetch(pid, fd, name)
        assert got >= 0
        assert os.read(got, 64) == b"through the fence"
        os.close(got)
    finally:
        _native._fd_fetch_set_mode("auto")
        parent.send("done")
        proc.join(timeout=20)
    assert proc.exitcode == 0


def test_fd_fetch_refuses_an_unregistered_descriptor():
    ctx = mp.get_context("spawn")
    parent, child = ctx.Pipe()
    proc = ctx.Process(target=_exporter, args=(child,))
    proc.start()
    try:
        pid, fd, name = parent.recv()
        _native._fd_fetch_set_mode("socket")
        with pytest.raises(Exception):
            _native._fd_fetch(pid, fd + 1000, name)
    finally:
        _native._fd_fetch_set_mode("auto")
        parent.send("done")
        proc.join(timeout=20)


def test_fd_fetch_refuses_a_peer_without_the_token():
    """The socket's name is public (/proc/net/unix); the descriptor server only answers a peer
    that presents the secret carried by the export handle (and runs under the same user)."""
    ctx = mp.get_context("spawn")
    parent, child = ctx.Pipe()
    proc = ctx.Process(target=_exporter, args=(child,))
    proc.start()
    try:
        pid, fd, name = parent.recv()
        public_name, token = name.rsplit(":", 1)
        _native._fd_fetch_set_mode("socket")
        for forged in (public_name, public_name + ":0", public_name + ":" + "f" * 16):
            if forged.endswith(token):
                continue
            with pytest.raises(Exception):
                _native._fd_fetch(pid, fd, forged)
        got = _native._fd_fetch(pid, fd, name)    # the real handle still works afterwards
        assert os.read(got, 64) == b"through the fence"
        os.close(got)
    finally:
        _native._fd_fetch_set_mode("auto")
        parent.send("done")
        proc.join(timeout=20)


def test_fd_fetch_inside_one_process_duplicates():
    r, w = os.pipe()
    os.write(w, b"x")
    got = _native._fd_fetch(os.getpid(), r, "")
    assert got != r and os.read(got, 1) == b"x"
    for f in (r, w, got):
        os.close(f)


def test_native_unit_tests_pass():
    """bin/pplx-core-tests: error type, scope guard, object and memory pools, imm counters,
    sharding arithmetic, host buffer reuse, address and CPU-list helpers, JSON numbers."""
    import subprocess
    from pathlib import Path

    exe = Path(__file__).resolve().parent.parent / "bin" / "pplx-core-tests"
    if not exe.exists():
        pytest.skip("run python build.py first")
    res = subprocess.run([str(exe)], capture_output=True, text=True, timeout=120)
    assert res.returncode == 0, res.stdout + res.stderr
    assert "0 failed" in res.stdout


def test_native_profiler_guard_records_a_range():
    """Native entry points open a torch profiler range around their work
    (reference rust/torch-lib/src/torch_lib.cc:121-130)."""
    import torch

    from pplx_garden import _native

    assert _native._profiler_guard_probe("pplx_probe_outside") is False     # no profiler running
    with torch.profiler.profile(activities=[torch.profiler.ProfilerActivity.CPU]) as prof:
        assert _native._profiler_guard_probe("pplx_probe_inside") is True
    names = {e.key for e in prof.key_averages()}
    assert "pplx_probe_inside" in names and "pplx_probe_outside" not in names
