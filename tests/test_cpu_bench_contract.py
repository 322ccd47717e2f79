"""bench.py contract pieces that need no GPU: the reference arm answers with an `unavailable` line
(and exit status 0) when it cannot run, and the bandwidth helper follows the busbw definition."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_reference_arm_single_gpu_is_unavailable():
    proc = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--gpus", "1"],
                          capture_output=True, text=True, timeout=120, env=dict(os.environ, WORLD_SIZE="1", RANK="0"))
    assert proc.returncode == 0, proc.stderr
    line = json.loads(proc.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and "unavailable" in line and "1 rank" in line["unavailable"]


def test_busbw_helper():
    sys.path.insert(0, ROOT)
    import bench
    assert abs(bench.busbw(1e9, 1.0, 8) - 1.75) < 1e-9
    assert abs(bench.busbw(1e9, 1.0, 2) - 1.0) < 1e-9
    assert abs(bench.busbw(1e9, 1.0, 1) - 1.0) < 1e-9  # single GPU: plain bytes/time of the local copy
    assert bench.BASELINE_BUSBW == 23.12 and bench.HEADLINE_BYTES == 64 << 20
