"""Worker for the multi-process GPU tests (one process per GPU). Modes:
collectives — all_reduce / reduce_scatter / all_gather on plain and symmetric tensors, all dtypes;
socket      — the same ring over TCP proxies between the processes;
departure   — rank 1 leaves between steps (its kernels done, communicator closed); rank 0's next
              collective must end with a timeout status from its bounded wait, not hang;
ring        — the ring + Simple kernels over FIFOs in peer memory between the processes;
mismatch    — rank 0 passes symmetric tensors, the others ordinary ones: the plans differ, and every
              rank must be told so by the first barrier instead of running out its waits."""
import os
import sys
import time

import torch

import nano_nccl_b200 as nn


def expected_sum(world, numel, dtype, seed_base):
    acc = torch.zeros(numel, dtype=torch.float32, device="cuda")
    for r in range(world):
        gen = torch.Generator(device="cuda").manual_seed(seed_base + r)
        acc += torch.randn(numel, device="cuda", generator=gen).to(dtype).float()
    return acc


def my_input(rank, numel, dtype, seed_base):
    gen = torch.Generator(device="cuda").manual_seed(seed_base + rank)
    return torch.randn(numel, device="cuda", generator=gen).to(dtype)


def main():
    mode = sys.argv[1]
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(rank)
    kw = {"wait_timeout_ms": 1500 if mode == "departure" else 5000}
    if mode == "socket":
        kw.update(transport="socket", channels=2)
    if mode == "ring":
        kw.update(algo="ring", channels=8)
    comm = nn.Communicator.from_env(**kw)
    tol = {torch.float32: 1e-5, torch.float16: 1e-2, torch.bfloat16: 1e-1}

    if mode in ("collectives", "socket", "ring"):
        dtypes = [torch.float32, torch.bfloat16] if mode != "collectives" else list(tol)
        for dtype in dtypes:
            for numel in (64, 8 * 12501, 1 << 21):
                x = my_input(rank, numel, dtype, 100)
                out = torch.empty_like(x)
                comm.all_reduce(out, x, op="sum")
                torch.cuda.synchronize()
                comm.check_async_error()
                ref = expected_sum(world, numel, dtype, 100)
                assert (out.float() - ref).abs().max().item() <= tol[dtype] * (2 if dtype != torch.float32 else 1), (dtype, numel, comm.last_call())
                if mode == "ring":
                    assert comm.last_call()["algo"] == "ring" and comm.transport == "p2p", (comm.last_call(), comm.transport)
                if mode == "collectives":
                    # ordinary tensors of another process: small ones ride the flag-in-data kernel, large
                    # ones the tile pipeline (copy in, reduce, copy out inside one launch)
                    # (the caller lowers the pipeline's threshold to 1 MiB so that this test reaches it)
                    nbytes = numel * x.element_size()
                    want = "ll" if nbytes <= (32 << 10) else ("pipeline" if nbytes >= (1 << 20) else None)
                    assert want is None or comm.last_call()["algo"] == want, (numel, comm.last_call())
                    sx, so = comm.empty(numel, dtype), comm.empty(numel, dtype)
                    sx.copy_(x)
                    comm.all_reduce(so, sx, op="avg")
                    torch.cuda.synchronize()
                    comm.check_async_error()
                    assert not comm.last_call()["staged_in"]
                    assert (so.float() - ref / world).abs().max().item() <= tol[dtype], (dtype, numel, comm.last_call())
                    comm.all_reduce(sx, op="sum")  # in place
                    torch.cuda.synchronize()
                    assert (sx.float() - ref).abs().max().item() <= tol[dtype] * 2
                    # ordinary tensors, registered: peers read and write them directly
                    rx, ro = x.clone(), torch.empty_like(x)
                    comm.register(rx)
                    comm.register(ro)
                    comm.all_reduce(ro, rx, op="sum")
                    torch.cuda.synchronize()
                    comm.check_async_error()
                    info = comm.last_call()
                    assert not info["staged_in"] and not info["staged_out"], info
                    assert (ro.float() - ref).abs().max().item() <= tol[dtype] * 2
                    comm.unregister(rx)
                    comm.unregister(ro)
                if numel % world == 0:
                    blk = numel // world
                    rs = torch.empty(blk, device="cuda", dtype=dtype)
                    comm.reduce_scatter(rs, x, op="sum")
                    ag = torch.empty(numel * world, device="cuda", dtype=dtype)
                    comm.all_gather(ag, x)
                    torch.cuda.synchronize()
                    comm.check_async_error()
                    assert (rs.float() - ref[rank * blk:(rank + 1) * blk]).abs().max().item() <= tol[dtype] * 2
                    for r in range(world):
                        assert torch.equal(ag[r * numel:(r + 1) * numel], my_input(r, numel, dtype, 100))
        print(f"rank {rank}: nvls={comm.nvls} transport={comm.transport} last={comm.last_call()}")
    elif mode == "mismatch":
        numel = 1 << 20
        x = my_input(rank, numel, torch.float32, 9)
        if rank == 0:
            sx, so = comm.empty(numel, torch.float32), comm.empty(numel, torch.float32)
        else:
            comm.empty(numel, torch.float32), comm.empty(numel, torch.float32)  # the allocation itself is collective
            sx, so = x, torch.empty_like(x)
        t0 = time.time()
        comm.all_reduce(so, sx)
        torch.cuda.synchronize()
        waited = time.time() - t0
        try:
            comm.check_async_error()
            raise SystemExit("expected a plan mismatch")
        except nn.B200CclError as e:
            assert "disagree on the plan" in str(e), str(e)
            assert waited < 3.0, f"the mismatch must be reported by the first barrier, not by a {waited:.1f} s timeout"
            print("detected:", e)
        assert torch.ones(8, device="cuda").sum().item() == 8  # the context is still usable
    elif mode == "departure":
        x = my_input(rank, 4096, torch.float32, 5)
        out = torch.empty_like(x)
        comm.all_reduce(out, x)           # step 1: both ranks take part
        torch.cuda.synchronize()
        comm.check_async_error()
        if rank == 1:
            comm.close()                  # leaves between steps, nothing of its own in flight
            print("rank 1 left")
            print("WORKER OK")
            return
        time.sleep(1.0)
        comm.all_reduce(out, x)           # step 2: the peer is gone
        torch.cuda.synchronize()          # returns: the wait is bounded
        try:
            comm.check_async_error()
            raise SystemExit("expected a timeout error")
        except nn.B200CclError as e:
            assert "timed out" in str(e) and "rank 1" in str(e), str(e)
            print("detected:", e)
        try:
            comm.all_reduce(out, x)       # a failed communicator rejects new work
            raise SystemExit("expected rejection")
        except nn.B200CclError:
            pass
        assert torch.ones(8, device="cuda").sum().item() == 8  # the context is still usable
    comm.close()
    print("WORKER OK")


if __name__ == "__main__":
    main()
