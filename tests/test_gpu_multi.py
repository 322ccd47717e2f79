"""Tests that need two or more GPUs: real peer access in one process, and one process per GPU with
exported allocations (+ NVLS when the driver exposes it). Skipped on a single-GPU machine.
The failure-detection test runs with NVLS off everywhere and makes the failure on the host: a
rank leaves between steps; the survivor's next collective ends with a timeout status after its
bounded wait, and the process stays usable."""
import os
import socket
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def ngpus():
    return torch.cuda.device_count() if torch.cuda.is_available() else 0


def free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def launch(world, mode, extra_env=None, timeout=240):
    port = free_port()
    procs = []
    for rank in range(world):
        env = dict(os.environ, RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1",
                   MASTER_PORT=str(port), B200CCL_PORT=str(port), PYTHONPATH=ROOT)
        env.update(extra_env or {})
        procs.append(subprocess.Popen([sys.executable, os.path.join(ROOT, "tests", "mp_worker.py"), mode], env=env,
                                      stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True))
    outs = []
    for p in procs:
        try:
            out, _ = p.communicate(timeout=timeout)
        except subprocess.TimeoutExpired:
            p.kill()
            out, _ = p.communicate()
            out += "\n[killed after timeout]"
        outs.append((p.returncode, out))
    return outs


@pytest.mark.skipif(ngpus() < 2, reason="needs two GPUs")
def test_single_process_two_gpus():
    import nano_nccl_b200 as nn
    comm = nn.Communicator(devices=[0, 1], wait_timeout_ms=3000)
    try:
        for dtype, tol in ((torch.float32, 1e-5), (torch.bfloat16, 1e-1)):
            for numel in (64, 100003, 1 << 22):
                ins = [torch.randn(numel, device=f"cuda:{d}").to(dtype) for d in (0, 1)]
                outs = [torch.empty_like(t) for t in ins]
                comm.all_reduce(outs, ins, op="sum")
                for d in (0, 1):
                    torch.cuda.synchronize(d)
                comm.check_async_error()
                ref = ins[0].float().cpu() + ins[1].float().cpu()
                for o in outs:
                    assert (o.float().cpu() - ref).abs().max().item() <= tol
    finally:
        comm.close()


@pytest.mark.skipif(ngpus() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("mode", ["collectives", "socket"])
def test_one_process_per_gpu(mode):
    world = min(ngpus(), 4)
    outs = launch(world, mode)
    for rc, out in outs:
        assert rc == 0 and "WORKER OK" in out, out


@pytest.mark.skipif(ngpus() < 2, reason="needs two GPUs")
def test_departed_rank_is_detected_by_bounded_wait():
    outs = launch(2, "departure", extra_env={"B200CCL_NVLS": "0", "NCCL_NVLS_ENABLE": "0"})
    for rc, out in outs:
        assert rc == 0 and "WORKER OK" in out, out
    assert any("timed out" in out for _, out in outs)


@pytest.mark.skipif(ngpus() < 2, reason="needs two GPUs")
def test_torch_distributed_backend_and_ddp():
    # dist.init_process_group("b200ccl") with the real engine: collectives of every kind on CUDA tensors,
    # a misaligned view, and torch's DistributedDataParallel, one process per GPU.
    world = 2
    port = free_port()
    procs = [subprocess.Popen([sys.executable, os.path.join(ROOT, "tests", "pg_worker.py"), "gpu", str(r), str(world), str(port)],
                              env=dict(os.environ, PYTHONPATH=ROOT, B200CCL_WAIT_TIMEOUT_MS="5000"), stdout=subprocess.PIPE,
                              stderr=subprocess.STDOUT, text=True) for r in range(world)]
    for p in procs:
        try:
            out, _ = p.communicate(timeout=240)
        except subprocess.TimeoutExpired:
            p.kill()
            out, _ = p.communicate()
            out += "\n[killed after timeout]"
        assert p.returncode == 0 and "pg worker ok" in out, out
