"""Small-case sweep on ONE device (ranks emulated by one launch): element counts 1..64, every
power of two up to 4096 with its neighbours, and primes up to 4096; buffers aligned and
misaligned by one element; 1, 2, 4 and 8 ranks; every dtype and operator. max, min and the
one-rank copy must be exact, sum and avg within the dtype's tolerance of a PyTorch fp32 reference.
The cases cross every boundary of the planner (flag-in-data kernel, one-shot, 16-byte and
element-wise paths) with lengths that leave ragged tails everywhere."""
import pytest
import torch

import nano_nccl_b200 as nn

pytestmark = pytest.mark.gpu

TOL = {torch.float32: 1e-5, torch.float16: 1e-2, torch.bfloat16: 1e-1}


def primes_upto(n):
    sieve = bytearray([1]) * (n + 1)
    sieve[0:2] = b"\x00\x00"
    for i in range(2, int(n ** 0.5) + 1):
        if sieve[i]:
            sieve[i * i::i] = bytearray(len(sieve[i * i::i]))
    return [i for i in range(n + 1) if sieve[i]]


def counts():
    c = set(range(1, 65))
    for k in range(6, 13):
        c.update({(1 << k) - 1, 1 << k, (1 << k) + 1})
    p = primes_upto(4096)
    c.update(p[::9])      # every ninth prime: about sixty of them, spread over the range
    c.update(p[-3:])
    return sorted(c)


@pytest.mark.parametrize("ranks", [1, 2, 4, 8])
@pytest.mark.parametrize("dtype", list(TOL))
def test_small_counts_all_operators_and_alignments(ranks, dtype):
    comm = nn.Communicator(devices=[0], loopback_ranks=ranks, wait_timeout_ms=2000) if ranks > 1 else \
        nn.Communicator(devices=[0], wait_timeout_ms=2000)
    try:
        top = 4096 + 16
        gen = torch.Generator(device="cuda").manual_seed(1234 + ranks)
        base_in = [torch.randn(top, device="cuda", generator=gen).to(dtype) for _ in range(ranks)]
        base_out = [torch.empty(top, device="cuda", dtype=dtype) for _ in range(ranks)]
        stack_all = torch.stack([t.float() for t in base_in])
        bad = []
        for shift in (0, 1):  # 0: 16-byte aligned start; 1: one element past it
            for op in ("sum", "avg", "max", "min"):
                for n in counts():
                    ins = [t[shift:shift + n] for t in base_in]
                    outs = [t[shift:shift + n] for t in base_out]
                    for o in outs:
                        o.fill_(float("nan"))
                    if ranks == 1:
                        comm.all_reduce(outs[0], ins[0], op=op)
                    else:
                        comm.all_reduce(outs, ins, op=op)
                    s = stack_all[:, shift:shift + n]
                    ref = {"sum": s.sum(0), "avg": s.sum(0) / ranks, "max": s.max(0).values, "min": s.min(0).values}[op]
                    for o in outs:
                        if op in ("max", "min") or ranks == 1:
                            okay = torch.equal(o.float(), ref.to(dtype).float())
                        else:
                            okay = bool(((o.float() - ref).abs() <= TOL[dtype]).all())
                        if not okay:
                            bad.append((shift, op, n, comm.last_call()["algo"]))
                            break
        torch.cuda.synchronize()
        comm.check_async_error()
        assert not bad, bad[:10]
    finally:
        comm.close()


@pytest.mark.parametrize("ranks", [2, 8])
def test_neighbouring_elements_are_left_alone(ranks):
    # Canary elements on both sides of every output: a kernel that rounds a length up, or starts a
    # vector access before the buffer, would overwrite them.
    comm = nn.Communicator(devices=[0], loopback_ranks=ranks, wait_timeout_ms=2000)
    try:
        for dtype in TOL:
            for n in (1, 3, 7, 33, 255, 1021, 4093):
                for shift in (8, 9):
                    ins = [torch.randn(n + 32, device="cuda").to(dtype) for _ in range(ranks)]
                    outs = [torch.full((n + 32,), 7.0, device="cuda", dtype=dtype) for _ in range(ranks)]
                    comm.all_reduce([o[shift:shift + n] for o in outs], [t[shift:shift + n] for t in ins], op="sum")
                    torch.cuda.synchronize()
                    for o in outs:
                        assert (o[:shift] == 7.0).all() and (o[shift + n:] == 7.0).all(), (dtype, n, shift, comm.last_call())
        comm.check_async_error()
    finally:
        comm.close()
