"""Tests of the checking build of the library (libb200ccl_check.so: the same sources with the
test-only socket fault hook and the device-side index checks compiled in). Each case runs in a
child process that loads that library instead of the product one. Failures are injected on the
host; the GPU is never made to fault, and every device wait is bounded."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def run(mode, **env):
    full = dict(os.environ, PYTHONPATH=ROOT, B200CCL_LIBRARY="check", **env)
    p = subprocess.run([sys.executable, os.path.join(ROOT, "tests", "check_worker.py"), mode], env=full,
                       stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=240)
    return p.returncode, p.stdout


def test_socket_failure_unblocks_the_kernels_and_names_the_edge():
    # The reference's fault-injection test (tests/mpi_correctness.cu:136-160, 295-310): the send proxy
    # closes its socket after n good slices; pass = the stream wait COMPLETES and the error text names the socket.
    rc, out = run("socket-fault", B200CCL_SOCKET_FAIL_AFTER_SLICES="2")
    assert rc == 0 and "WORKER OK" in out, out


def test_device_index_checks_record_and_skip():
    rc, out = run("bounds", B200CCL_DEBUG_SHRINK_EXTENT="8")
    assert rc == 0 and "WORKER OK" in out, out


def test_canary_pages_around_the_staging_arena():
    rc, out = run("canary")
    assert rc == 0 and "WORKER OK" in out, out
    rc, out = run("canary", B200CCL_DEBUG_SMASH_CANARY="1")
    assert rc == 0 and "WORKER OK" in out and "canary overwritten" in out, out


def test_product_library_has_no_fault_hook():
    # In the product build the environment variable is ignored.
    code = ("import torch, nano_nccl_b200 as nn\n"
            "c = nn.Communicator(devices=[0], loopback_ranks=2, transport='socket', channels=2, wait_timeout_ms=3000)\n"
            "x = [torch.ones(1 << 20, device='cuda') for _ in range(2)]; y = [torch.empty_like(t) for t in x]\n"
            "c.all_reduce(y, x); torch.cuda.synchronize(); c.check_async_error()\n"
            "assert (y[0] == 2).all(); c.close(); print('PRODUCT OK')\n")
    env = dict(os.environ, PYTHONPATH=ROOT, B200CCL_SOCKET_FAIL_AFTER_SLICES="2")
    env.pop("B200CCL_LIBRARY", None)
    p = subprocess.run([sys.executable, "-c", code], env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=240)
    assert p.returncode == 0 and "PRODUCT OK" in p.stdout, p.stdout
