"""The parts of the benchmark contract that can be checked without a GPU."""

import json
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent


def test_reference_arm_reports_unavailable_and_exits_zero():
    res = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--impl", "reference", "--gpus", "1",
                          "--steps", "2", "--warmup", "1"], capture_output=True, text=True, timeout=300, cwd=ROOT)
    assert res.returncode == 0, res.stderr[-500:]
    line = json.loads(res.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference"
    assert isinstance(line.get("unavailable"), str) and len(line["unavailable"]) > 10


def test_bench_help_lists_the_contract_flags():
    res = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--help"], capture_output=True, text=True,
                         timeout=120, cwd=ROOT)
    assert res.returncode == 0
    for flag in ("--gpus", "--steps", "--warmup", "--impl"):
        assert flag in res.stdout


def test_graft_entry_exposes_build_and_smoke():
    sys.path.insert(0, str(ROOT))
    import __graft_entry__ as entry

    assert callable(entry.build) and callable(entry.smoke)
