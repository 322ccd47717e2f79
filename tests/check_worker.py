"""Worker for the tests of the checking build of the library (B200CCL_LIBRARY=check is set by the
caller before this process starts). Every failure here is made on the host; no GPU faults.
socket-fault — a send proxy closes its socket after two slices: the ring kernels must leave their
               waits, the error must name the edge, and the communicator must refuse new work;
bounds       — the host is told to pass extents that are too short: the kernel must record the
               first bad index, skip those accesses and still run to its end;
canary       — the staging arena sits between two pages of canary bytes: they survive staged
               collectives, and a byte overwritten from the host is reported."""
import os
import sys

import torch

import nano_nccl_b200 as nn


def main():
    mode = sys.argv[1]
    torch.cuda.set_device(0)
    assert os.environ.get("B200CCL_LIBRARY") == "check"
    if mode == "socket-fault":
        comm = nn.Communicator(devices=[0], loopback_ranks=2, transport="socket", channels=2, wait_timeout_ms=3000)
        numel = 8 << 20  # 32 MiB per rank: many slices per channel
        ins = [torch.randn(numel, device="cuda") for _ in range(2)]
        outs = [torch.zeros_like(t) for t in ins]
        comm.all_reduce(outs, ins)
        torch.cuda.synchronize()  # returns: the proxy's error raised the abort word, the kernels left their waits
        try:
            comm.check_async_error()
            raise SystemExit("expected the injected socket failure")
        except nn.B200CclError as e:
            text = str(e)
            assert "socket" in text and "injected" in text, text
            for part in ("source=", "destination=", "channel=", "step="):
                assert part in text, text
            print("detected:", text)
        try:
            comm.all_reduce(outs, ins)
            raise SystemExit("a failed communicator must refuse new work")
        except nn.B200CclError:
            pass
        assert torch.ones(8, device="cuda").sum().item() == 8  # the context is still usable
        comm.close()
    elif mode == "bounds":
        comm = nn.Communicator(devices=[0], loopback_ranks=4, algo="twoshot", wait_timeout_ms=3000)
        numel = 1 << 16
        ins = [torch.randn(numel, device="cuda") for _ in range(4)]
        outs = [torch.full_like(t, -7.0) for t in ins]
        comm.all_reduce(outs, ins)
        torch.cuda.synchronize()
        try:
            comm.check_async_error()
            raise SystemExit("expected the self-check to fire")
        except nn.B200CclError as e:
            assert "self-check" in str(e) and "beyond the buffer extent" in str(e), str(e)
            print("detected:", e)
        # packs beyond the (shrunk) extent were skipped, everything below it was reduced
        ref = torch.stack(ins).sum(0)
        shrink_elems = int(os.environ["B200CCL_DEBUG_SHRINK_EXTENT"]) * comm.last_call()["pack_bytes"] // 4
        good = numel - shrink_elems
        for o in outs:
            assert (o[:good] - ref[:good]).abs().max().item() <= 1e-5
            assert (o[good:] == -7.0).all()
        comm.close()
    elif mode == "canary":
        smash = os.environ.pop("B200CCL_DEBUG_SMASH_CANARY", None)
        comm = nn.Communicator(devices=[0], loopback_ranks=4, algo="pipeline", wait_timeout_ms=3000, staging_bytes=8 << 20)
        for numel in (1 << 20, (3 << 20) + 4, 4096):
            ins = [torch.randn(numel, device="cuda") for _ in range(4)]
            outs = [torch.empty_like(t) for t in ins]
            comm.all_reduce(outs, ins)
            torch.cuda.synchronize()
            comm.check_async_error()   # includes the canary check in this build
            ref = torch.stack(ins).sum(0)
            assert all((o - ref).abs().max().item() <= 1e-5 for o in outs)
        if smash:
            os.environ["B200CCL_DEBUG_SMASH_CANARY"] = "1"
            try:
                comm.check_async_error()
                raise SystemExit("expected the canary check to fire")
            except nn.B200CclError as e:
                assert "canary overwritten" in str(e) and "after the arena" in str(e), str(e)
                print("detected:", e)
        comm.close()
    print("WORKER OK")


if __name__ == "__main__":
    main()
