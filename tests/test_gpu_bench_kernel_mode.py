"""bench.py --kernel: the single-kernel mode that the profiler captures and the per-kernel timings are made with."""
import os
import subprocess
import sys

import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def run(*args):
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), *args], capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert r.returncode == 0, r.stderr[-2000:]
    return r.stdout


def test_gemm_mode_on_each_route_and_without_a_graph():
    for route in ("integer", "tensor"):
        out = run("--kernel", "gemm", "--shape", "128", "4096", "1152", "--route", route, "--reps", "2")
        assert f"route={route}" in out and "us/call" in out
    out = run("--kernel", "gemm", "--shape", "128", "4096", "1152", "--route", "tensor", "--tc-kernel", "2", "--shortcut", "--reps", "2", "--no-graph")
    assert "shortcut=1" in out


def test_pack_mode_reports_both_routes_equal():
    out = run("--kernel", "pack", "--shape", "4", "64", "26", "26", "32", "3", "--reps", "2")
    lines = [l for l in out.splitlines() if l.startswith("pack ")]
    assert len(lines) == 2 and "equal=True" in lines[1]


def test_layer_mode_with_output_and_with_the_shortcut_sum_only():
    out = run("--kernel", "layer", "--shape", "2", "64", "28", "28", "128", "3", "--route", "tensor", "--reps", "2")
    assert "sum_only=0" in out and "us/call" in out
    out = run("--kernel", "layer", "--shape", "2", "64", "28", "28", "128", "3", "2", "--sum-only", "--route", "tensor", "--tc-kernel", "2", "--reps", "2", "--no-graph")
    assert "stride=2" in out and "sum_only=1" in out
