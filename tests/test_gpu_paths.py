"""GPU tests of single code paths on ONE device: the single-rank copy kernel (TMA bulk copies), the
256-bit and 128-bit variants of the peer two-shot loop, fp32 accumulation of 16-bit inputs shown by a
case that 16-bit accumulation gets wrong, and the plan fingerprint that the first barrier compares.
Numerics are compared with a plain PyTorch fp32 reference. Every device wait is bounded."""
import pytest
import torch

import nano_nccl_b200 as nn

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def one_rank():
    comm = nn.Communicator(devices=[0], wait_timeout_ms=2000)
    yield comm
    comm.close()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_single_rank_collectives_are_copies(one_rank, dtype):
    comm = one_rank
    esz = torch.empty(0, dtype=dtype).element_size()
    # one 16-byte pack; less than a tile; exactly one tile; a ragged last tile; more tiles than the
    # ring of shared-memory slots holds per CTA; enough for every SM to loop
    for nbytes in (16, 48, 32768, 32768 + 16, 7 * 32768 + 4096, (64 << 20) + 16):
        numel = nbytes // esz
        x = torch.randn(numel, device="cuda").to(dtype)
        for op in ("sum", "avg", "max"):
            y = torch.full_like(x, float("nan"))
            comm.all_reduce(y, x, op=op)
            torch.cuda.synchronize()
            comm.check_async_error()
            assert comm.last_call()["algo"] == "copy", comm.last_call()
            assert torch.equal(y, x), (nbytes, op)
    x = torch.randn(4096, device="cuda").to(dtype)
    y = torch.empty_like(x)
    comm.reduce_scatter(y, x)
    z = torch.empty_like(x)
    comm.all_gather(z, x)
    keep = x.clone()
    comm.all_reduce(x)  # in place: nothing to move
    torch.cuda.synchronize()
    comm.check_async_error()
    assert torch.equal(y, keep) and torch.equal(z, keep) and torch.equal(x, keep)


def test_single_rank_unaligned_buffers_take_the_element_path(one_rank):
    comm = one_rank
    base = torch.randn(1 << 16, device="cuda")
    x = base[1:4098]  # 4 bytes past a 16-byte boundary, 4097 elements
    y = torch.full((4100,), float("nan"), device="cuda")[3:]
    comm.all_reduce(y, x, op="min")
    torch.cuda.synchronize()
    comm.check_async_error()
    assert comm.last_call()["algo"] == "oneshot" and not comm.last_call()["vectorized"]
    assert torch.equal(y, x)


@pytest.mark.parametrize("ranks", [2, 4, 8])
@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
def test_two_shot_pack_widths_agree(ranks, dtype):
    tol = {torch.float32: 1e-5, torch.float16: 1e-2, torch.bfloat16: 1e-1}[dtype]
    esz = torch.empty(0, dtype=dtype).element_size()
    comm = nn.Communicator(devices=[0], loopback_ranks=ranks, algo="twoshot", wait_timeout_ms=2000)
    try:
        numel = (1 << 20) + 96 // esz  # a multiple of 32 bytes that no rank count divides evenly into packs
        gen = torch.Generator(device="cuda").manual_seed(11)
        data = [torch.randn(numel, device="cuda", generator=gen).to(dtype) for _ in range(ranks)]
        raw_in = [torch.empty(numel + 64, device="cuda", dtype=dtype) for _ in range(ranks)]
        raw_out = [torch.full((numel + 64,), float("nan"), device="cuda", dtype=dtype) for _ in range(ranks)]
        results = {}
        for name, shift in (("aligned32", 0), ("aligned16", 16 // esz)):
            ins = [t[shift:shift + numel] for t in raw_in]
            outs = [t[shift:shift + numel] for t in raw_out]
            for view, values in zip(ins, data):
                view.copy_(values)  # the same values behind both alignments
            for op in ("sum", "max"):
                comm.all_reduce(outs, ins, op=op)
                torch.cuda.synchronize()
                comm.check_async_error()
                info = comm.last_call()
                assert info["algo"] == "twoshot" and info["pack_bytes"] == (32 if shift == 0 else 16), info
                stack = torch.stack([t.float() for t in ins])
                ref = stack.sum(0) if op == "sum" else stack.max(0).values
                for o in outs:
                    assert (o.float() - ref).abs().max().item() <= tol, (name, op)
                for o in outs[1:]:
                    assert torch.equal(o, outs[0])
                results[(name, op)] = outs[0].clone()
        # the pack width changes how many elements a thread handles, never the value of an element
        assert torch.equal(results[("aligned32", "max")], results[("aligned16", "max")])
        assert torch.equal(results[("aligned32", "sum")], results[("aligned16", "sum")])
    finally:
        comm.close()


@pytest.mark.parametrize("algo", ["oneshot", "twoshot", "ll"])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_sixteen_bit_inputs_accumulate_in_fp32(algo, dtype):
    # (The ring is not in this list: its partial sums travel through FIFOs of the message's own type,
    # so it adds in fp32 but rounds once per hop, like the FIFO-based ring it re-expresses.)
    # Rank 0 contributes a value whose spacing to the next representable number is larger than what
    # every other rank adds: 256 in bf16 (spacing 2) and 2048 in fp16 (spacing 2), plus seven times
    # 0.5. Adding rank by rank in the 16-bit type leaves the big value unchanged at every step; fp32
    # accumulation with one final rounding gives big + 3.5 -> rounds to big + 4. The result must
    # equal the fp32 sum rounded once, bit for bit.
    ranks = 8
    big = 256.0 if dtype == torch.bfloat16 else 2048.0
    numel = 2048
    comm = nn.Communicator(devices=[0], loopback_ranks=ranks, algo=algo, wait_timeout_ms=2000)
    try:
        ins = [torch.full((numel,), big if r == 0 else 0.5, device="cuda", dtype=dtype) for r in range(ranks)]
        outs = [torch.empty_like(t) for t in ins]
        comm.all_reduce(outs, ins, op="sum")
        torch.cuda.synchronize()
        comm.check_async_error()
        assert comm.last_call()["algo"] == algo
        expect = torch.stack([t.float() for t in ins]).sum(0).to(dtype)
        assert expect[0].item() == big + 4.0
        sixteen_bit_chain = ins[0].clone()
        for t in ins[1:]:
            sixteen_bit_chain = (sixteen_bit_chain + t).to(dtype)
        assert sixteen_bit_chain[0].item() == big, "the case must be one that 16-bit accumulation gets wrong"
        for o in outs:
            assert torch.equal(o, expect), (algo, o[0].item(), expect[0].item())
        # avg: the 1/N scale is applied to the fp32 sum, before the single rounding
        comm.all_reduce(outs, ins, op="avg")
        torch.cuda.synchronize()
        expect_avg = (torch.stack([t.float() for t in ins]).sum(0) / ranks).to(dtype)
        for o in outs:
            assert torch.equal(o, expect_avg)
    finally:
        comm.close()


@pytest.mark.parametrize("ranks", [2, 4, 8])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_staged_pipeline_all_reduce(ranks, dtype):
    # The tile pipeline (copy in / reduce / copy out running at once inside one kernel), forced on
    # buffers that would not need it: sizes from one ragged tile to many tiles per CTA, several calls
    # in a row (the counters only grow), every operator, a small arena (slot reuse), in place.
    tol = {torch.float32: 1e-5, torch.bfloat16: 1e-1}[dtype]
    esz = torch.empty(0, dtype=dtype).element_size()
    comm = nn.Communicator(devices=[0], loopback_ranks=ranks, algo="pipeline", wait_timeout_ms=3000, staging_bytes=16 << 20)
    try:
        sizes = [16, 4096 + 16, (1 << 20) + 48, 1 << 20, (24 << 20) + 16, 3 << 20]
        for i, nbytes in enumerate(sizes):
            numel = nbytes // esz
            op = ["sum", "avg", "max", "min"][i % 4]
            gen = torch.Generator(device="cuda").manual_seed(200 + i)
            ins = [torch.randn(numel, device="cuda", generator=gen).to(dtype) for _ in range(ranks)]
            stack = torch.stack([t.float() for t in ins])
            ref = {"sum": stack.sum(0), "avg": stack.sum(0) / ranks, "max": stack.max(0).values, "min": stack.min(0).values}[op]
            if i % 2:
                outs = ins
                comm.all_reduce(outs, op=op)
            else:
                outs = [torch.full_like(t, float("nan")) for t in ins]
                comm.all_reduce(outs, ins, op=op)
            torch.cuda.synchronize()
            comm.check_async_error()
            info = comm.last_call()
            assert info["algo"] == "pipeline" and info["staged_in"] and info["staged_out"], info
            for o in outs:
                assert (o.float() - ref).abs().max().item() <= tol, (nbytes, op, info)
            for o in outs[1:]:
                assert torch.equal(o, outs[0])
    finally:
        comm.close()


@pytest.mark.parametrize("ranks", [2, 4, 8])
@pytest.mark.parametrize("transport", ["auto", "shm"])
def test_ring_small_slices_return_their_credit_early(ranks, transport):
    # Messages whose slices hold at most one 16-byte vector per thread take the early-credit path
    # of the ring kernel (slot read into registers, credit posted, then combined and forwarded).
    # Many calls in a row reuse every FIFO slot several times, so a credit posted too early would
    # let the sender overwrite a slot that is still being read and corrupt a later call.
    comm = nn.Communicator(devices=[0], loopback_ranks=ranks, algo="ring", transport=transport, channels=4, wait_timeout_ms=3000)
    try:
        for dtype, tol in ((torch.float32, 1e-5), (torch.bfloat16, 1e-1)):
            for i, numel in enumerate([1024, 4096, 16384, 2048, 65536, 4096, 1024, 8192] * 3):
                op = ["sum", "avg", "max", "min"][i % 4]
                gen = torch.Generator(device="cuda").manual_seed(300 + i)
                ins = [torch.randn(numel, device="cuda", generator=gen).to(dtype) for _ in range(ranks)]
                outs = [torch.full_like(t, float("nan")) for t in ins]
                comm.all_reduce(outs, ins, op=op)
                stack = torch.stack([t.float() for t in ins])
                ref = {"sum": stack.sum(0), "avg": stack.sum(0) / ranks, "max": stack.max(0).values, "min": stack.min(0).values}[op]
                for o in outs:
                    assert (o.float() - ref).abs().max().item() <= tol * (2 if dtype != torch.float32 else 1), (numel, op)
        blk = 2048
        ins = [torch.randn(blk * ranks, device="cuda") for _ in range(ranks)]
        rs = [torch.empty(blk, device="cuda") for _ in range(ranks)]
        ag = [torch.empty(blk * ranks * ranks, device="cuda") for _ in range(ranks)]
        comm.reduce_scatter(rs, ins)
        comm.all_gather(ag, ins)
        torch.cuda.synchronize()
        comm.check_async_error()
        total = torch.stack(ins).sum(0)
        for r in range(ranks):
            assert (rs[r] - total[r * blk:(r + 1) * blk]).abs().max().item() <= 1e-5
            assert torch.equal(ag[r], torch.cat(ins))
    finally:
        comm.close()
