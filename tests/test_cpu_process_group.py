"""The "b200ccl" torch.distributed backend on CPU: registration, collectives (native path and the
all-gather fallbacks), broadcast / barrier built from the three collectives, and torch's own
DistributedDataParallel on top -- one process, and two processes whose stand-in engine travels over gloo."""
import os
import socket
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
WORKER = os.path.join(ROOT, "tests", "pg_worker.py")


def test_single_rank_process_group():
    proc = subprocess.run([sys.executable, WORKER, "solo"], capture_output=True, text=True, timeout=300)
    assert proc.returncode == 0 and "pg worker ok" in proc.stdout, proc.stdout + proc.stderr


def test_two_rank_process_group_and_ddp():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    procs = [subprocess.Popen([sys.executable, WORKER, "pair", str(r), str(port)], stdout=subprocess.PIPE,
                              stderr=subprocess.STDOUT, text=True) for r in range(2)]
    outs = []
    for p in procs:
        try:
            out, _ = p.communicate(timeout=300)
        except subprocess.TimeoutExpired:
            p.kill()
            out, _ = p.communicate()
        outs.append(out)
    for p, out in zip(procs, outs):
        assert p.returncode == 0 and "pg worker ok" in out, out
