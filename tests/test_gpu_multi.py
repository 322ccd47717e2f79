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
@pytest.mark.parametrize("mode", ["collectives", "socket", "ring"])
def test_one_process_per_gpu(mode):
    world = min(ngpus(), 4)
    outs = launch(world, mode, extra_env={"B200CCL_PIPELINE_MIN_BYTES": "1M"})
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


@pytest.mark.skipif(ngpus() < 2, reason="needs two GPUs")
def test_ranks_with_different_plans_are_told_so():
    outs = launch(2, "mismatch", extra_env={"B200CCL_NVLS": "0", "NCCL_NVLS_ENABLE": "0"})
    for rc, out in outs:
        assert rc == 0 and "WORKER OK" in out and "disagree on the plan" in out, out


def _pointer_info(lib, address):
    import ctypes
    out = (ctypes.c_int * 2)()
    assert lib.b2_pointer_info(ctypes.c_void_p(address), out) == 0, lib.b2_last_error()
    return out[0], out[1]  # (1 host / 2 device, owning device)


def _ring_round(comm, devices, numel=1 << 20):
    for dtype, tol in ((torch.float32, 1e-5), (torch.bfloat16, 1e-1)):
        ins = [torch.randn(numel, device=f"cuda:{d}").to(dtype) for d in devices]
        outs = [torch.empty_like(t) for t in ins]
        comm.all_reduce(outs, ins, op="avg")
        for d in devices:
            torch.cuda.synchronize(d)
        comm.check_async_error()
        assert comm.last_call()["algo"] == "ring", comm.last_call()
        ref = sum(t.float().cpu() for t in ins) / len(devices)
        for o in outs:
            assert (o.float().cpu() - ref).abs().max().item() <= tol


@pytest.mark.skipif(ngpus() < 2, reason="needs two GPUs")
def test_ring_counters_and_fifos_live_where_the_protocol_says(monkeypatch):
    # Ownership rule of the Simple protocol over peer memory (the reference checks it with
    # cudaPointerGetAttributes, tests/p2p_step_counters.cu:161-183): a rank polls words in its OWN
    # memory (send_head, recv_tail) and keeps its progress there; it publishes into its neighbours'
    # memory (send_tail and the FIFO it fills live on the NEXT rank, recv_head on the PREVIOUS one).
    import nano_nccl_b200 as nn
    from nano_nccl_b200 import _lib
    lib = _lib.load()
    ndev = min(ngpus(), 4)
    devices = list(range(ndev))
    for var in ("B200CCL_SHM_EDGES", "B200CCL_NO_PEER_PAIRS"):
        monkeypatch.delenv(var, raising=False)
    comm = nn.Communicator(devices=devices, algo="ring", channels=4, wait_timeout_ms=3000)
    try:
        _ring_round(comm, devices)
        assert comm.transport == "p2p"
        for r in devices:
            nxt, prv = devices[(r + 1) % ndev], devices[(r - 1) % ndev]
            for c in (0, 3):
                w = comm.ring_channel(r, c)
                for name, owner in (("send_head", r), ("recv_tail", r), ("send_base", r), ("recv_base", r), ("recv_fifo", r),
                                    ("send_tail", nxt), ("send_fifo", nxt), ("recv_head", prv)):
                    kind, dev = _pointer_info(lib, w[name])
                    assert kind == 2 and dev == owner, (r, c, name, kind, dev, owner)
    finally:
        comm.close()


@pytest.mark.skipif(ngpus() < 2, reason="needs two GPUs")
def test_mixed_ring_one_edge_over_host_memory(monkeypatch):
    # `auto` decides edge by edge. Edge 0 (rank 0 -> rank 1) is forced onto host memory: the
    # communicator reports `mixed`, lists both kinds, every collective goes through the ring, and
    # the forced edge's FIFO and counters are host memory while the other edge stays in device memory.
    import nano_nccl_b200 as nn
    from nano_nccl_b200 import _lib
    lib = _lib.load()
    monkeypatch.setenv("B200CCL_SHM_EDGES", "0")
    monkeypatch.delenv("B200CCL_NO_PEER_PAIRS", raising=False)
    comm = nn.Communicator(devices=[0, 1], channels=4, wait_timeout_ms=3000)
    try:
        assert comm.transport == "mixed", comm.transport
        text = comm.describe()
        assert "edge 0->1: shm" in text and "edge 1->0: p2p" in text, text
        _ring_round(comm, [0, 1])
        w0, w1 = comm.ring_channel(0, 0), comm.ring_channel(1, 0)
        for name in ("send_fifo", "send_tail", "send_head"):      # rank 0's outgoing edge: host
            assert _pointer_info(lib, w0[name])[0] == 1, name
        for name in ("recv_fifo", "recv_tail", "recv_head"):      # the same edge seen by rank 1
            assert _pointer_info(lib, w1[name])[0] == 1, name
        assert w0["send_fifo"] == w1["recv_fifo"] and w0["send_tail"] == w1["recv_tail"] and w0["send_head"] == w1["recv_head"]
        for name, owner in (("send_fifo", 0), ("send_tail", 0), ("send_head", 1)):   # rank 1's outgoing edge: peer memory
            assert _pointer_info(lib, w1[name]) == (2, owner), name
        # reduce_scatter and all_gather cross the mixed ring too
        ins = [torch.randn(1 << 16, device=f"cuda:{d}") for d in (0, 1)]
        rs = [torch.empty(1 << 15, device=f"cuda:{d}") for d in (0, 1)]
        ag = [torch.empty(1 << 17, device=f"cuda:{d}") for d in (0, 1)]
        comm.reduce_scatter(rs, ins)
        comm.all_gather(ag, ins)
        for d in (0, 1):
            torch.cuda.synchronize(d)
        comm.check_async_error()
        total = ins[0].cpu() + ins[1].cpu()
        for d in (0, 1):
            assert (rs[d].cpu() - total[d << 15:(d + 1) << 15]).abs().max().item() <= 1e-5
            assert torch.equal(ag[d].cpu(), torch.cat([ins[0].cpu(), ins[1].cpu()]))
    finally:
        comm.close()


@pytest.mark.skipif(ngpus() < 2, reason="needs two GPUs")
def test_pairs_without_peer_access_fall_back_edge_by_edge(monkeypatch):
    # Pretend devices 0 and 1 cannot address each other. With two GPUs every edge then uses host
    # memory (shm); with four, only the edges that touch that pair do, the rest use a FIFO on the
    # receiver reached through peer access enabled for that pair alone: mixed.
    import nano_nccl_b200 as nn
    monkeypatch.setenv("B200CCL_NO_PEER_PAIRS", "0-1")
    monkeypatch.delenv("B200CCL_SHM_EDGES", raising=False)
    ndev = 4 if ngpus() >= 4 else 2
    devices = list(range(ndev))
    comm = nn.Communicator(devices=devices, channels=4, wait_timeout_ms=3000)
    try:
        assert comm.transport == ("mixed" if ndev == 4 else "shm"), comm.transport
        assert "edge 0->1: shm" in comm.describe()
        _ring_round(comm, devices)
        with pytest.raises(Exception):
            comm.empty(1024)  # no symmetric memory without all-pairs peer access
    finally:
        comm.close()
    with pytest.raises(Exception, match="cannot access"):
        nn.Communicator(devices=devices, transport="p2p")  # an explicit request fails rather than falling back


@pytest.mark.skipif(ngpus() < 2, reason="needs two GPUs")
def test_native_benchmark_one_process_per_gpu():
    # The command-line benchmark in its multi-process form (the reference's MPI variant,
    # benchmarks/all_reduce_bench.cu:84-316): constant inputs rank + 1, one table from rank 0,
    # #wrong = 0 and the same exit status in every process.
    binary = os.path.join(ROOT, "build", "bin", "b200ccl_collective_bench")
    if not os.path.exists(binary):
        pytest.skip("native benchmark not built")
    world = min(ngpus(), 4)
    for extra in (["--redop", "avg", "--dtype", "bf16"], ["--collective", "all_gather", "--symmetric"],
                  ["--collective", "reduce_scatter", "--redop", "max"]):
        port = free_port()
        procs = [subprocess.Popen([binary, "--world", str(world), "--rank", str(r), "--addr", f"127.0.0.1:{port}", "-b", "4096",
                                   "-e", "4194304", "-f", "32", "-w", "2", "-n", "5"] + extra,
                                  env=dict(os.environ, B200CCL_WAIT_TIMEOUT_MS="5000"), stdout=subprocess.PIPE,
                                  stderr=subprocess.STDOUT, text=True) for r in range(world)]
        outs = []
        for p in procs:
            try:
                out, _ = p.communicate(timeout=240)
            except subprocess.TimeoutExpired:
                p.kill()
                out, _ = p.communicate()
                out += "\n[killed after timeout]"
            outs.append((p.returncode, out))
        assert all(rc == 0 for rc, _ in outs), outs
        rows = [line.split() for line in outs[0][1].splitlines() if line and not line.startswith("#")]
        assert len(rows) == 3 and all(r[9] == "0" for r in rows), outs[0][1]   # three sizes, #wrong = 0
        assert all(not [l for l in out.splitlines() if l and not l.startswith("#")] for _, out in outs[1:]), "only rank 0 prints rows"
