"""Worker of tests/test_cpu_process_group.py: drives the "b200ccl" torch.distributed backend on CPU
tensors with a stand-in engine (the real engine needs GPUs), so that the process-group plumbing --
registration, option objects, work objects, fallbacks, DistributedDataParallel -- is exercised.

    python tests/pg_worker.py solo
    python tests/pg_worker.py pair <rank> <port>
    python tests/pg_worker.py gpu <rank> <world> <port>     # the real engine, one process per GPU
"""
import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
from nano_nccl_b200.parallel import process_group as pgmod  # noqa: E402


class SoloEngine:
    """One rank: every collective is a copy."""
    any_device = True

    def __init__(self, store, rank, size):
        assert size == 1
        self.calls = []

    def supports(self, t):
        return t.dtype in (torch.float32, torch.float16, torch.bfloat16)

    def all_reduce(self, out, inp, op):
        self.calls.append(("all_reduce", op, inp.numel()))
        out.copy_(inp)

    def reduce_scatter(self, out, inp, op):
        self.calls.append(("reduce_scatter", op, inp.numel()))
        out.copy_(inp[:out.numel()])

    def all_gather(self, out, inp):
        self.calls.append(("all_gather", "", inp.numel()))
        out.copy_(inp)

    def synchronize(self, device):
        pass

    def close(self):
        self.calls.append(("close", "", 0))


class GlooEngine:
    """Several ranks: the three collectives travel over the default (gloo) group."""
    any_device = True
    OPS = {"sum": dist.ReduceOp.SUM, "max": dist.ReduceOp.MAX, "min": dist.ReduceOp.MIN}

    def __init__(self, store, rank, size):
        self.size = size
        self.calls = []

    def supports(self, t):
        return t.dtype in (torch.float32, torch.float16, torch.bfloat16)

    def _reduce(self, t, op):
        wide = t.float()
        dist.all_reduce(wide, op=self.OPS["sum" if op == "avg" else op])
        if op == "avg":
            wide /= self.size
        return wide.to(t.dtype)

    def all_reduce(self, out, inp, op):
        self.calls.append("all_reduce")
        out.copy_(self._reduce(inp, op))

    def reduce_scatter(self, out, inp, op):
        self.calls.append("reduce_scatter")
        n = out.numel()
        out.copy_(self._reduce(inp, op)[dist.get_rank() * n:(dist.get_rank() + 1) * n])

    def all_gather(self, out, inp):
        self.calls.append("all_gather")
        dist.all_gather_into_tensor(out, inp)

    def synchronize(self, device):
        pass

    def close(self):
        pass


DEV = torch.device("cpu")


def check_collectives(group, rank, world):
    kw = {"group": group} if group is not None else {}
    torch.set_default_device(DEV)
    x = torch.arange(6, dtype=torch.float32) + rank
    dist.all_reduce(x, **kw)
    assert torch.equal(x, torch.arange(6, dtype=torch.float32) * world + sum(range(world)))
    x = torch.full((5,), float(rank + 1), dtype=torch.bfloat16)
    dist.all_reduce(x, op=dist.ReduceOp.AVG, **kw)
    assert torch.allclose(x.float(), torch.full((5,), (world + 1) / 2.0)), x
    t = (torch.arange(6, dtype=torch.float32).reshape(2, 3) + rank).t()  # not contiguous
    assert not t.is_contiguous()
    dist.all_reduce(t, op=dist.ReduceOp.MAX, **kw)
    assert torch.equal(t, (torch.arange(6, dtype=torch.float32).reshape(2, 3) + world - 1).t())
    # other dtypes and operators go through the all-gather fallback
    i = torch.tensor([1, 2, 3], dtype=torch.int64) * (rank + 1)
    dist.all_reduce(i, **kw)
    assert i.tolist() == [s * sum(r + 1 for r in range(world)) for s in (1, 2, 3)]
    b = torch.tensor([rank == 0, True, False])
    dist.all_reduce(b, op=dist.ReduceOp.BAND, **kw)
    assert b.tolist() == [world == 1, True, False]
    p = torch.tensor([2.0, 3.0]) + rank
    dist.all_reduce(p, op=dist.ReduceOp.PRODUCT, **kw)
    expect = torch.tensor([2.0, 3.0])
    for r in range(1, world):
        expect = expect * (torch.tensor([2.0, 3.0]) + r)
    assert torch.equal(p, expect)
    # all-gather: flat tensor, list form, odd sizes, 8-byte elements
    src = torch.arange(7, dtype=torch.float16) + 10 * rank
    out = torch.empty(7 * world, dtype=torch.float16)
    dist.all_gather_into_tensor(out, src, **kw)
    assert torch.equal(out, torch.cat([torch.arange(7, dtype=torch.float16) + 10 * r for r in range(world)]))
    outs = [torch.empty(3, dtype=torch.int64) for _ in range(world)]
    dist.all_gather(outs, torch.tensor([rank, rank + 1, -rank], dtype=torch.int64), **kw)
    for r in range(world):
        assert outs[r].tolist() == [r, r + 1, -r]
    # reduce-scatter
    inp = torch.arange(4 * world, dtype=torch.float32) * (rank + 1)
    got = torch.empty(4, dtype=torch.float32)
    dist.reduce_scatter_tensor(got, inp, **kw)
    scale = sum(r + 1 for r in range(world))
    assert torch.equal(got, torch.arange(4 * world, dtype=torch.float32)[rank * 4:(rank + 1) * 4] * scale)
    blocks = [torch.full((2,), float(rank + 10 * k)) for k in range(world)]
    got = torch.empty(2)
    dist.reduce_scatter(got, blocks, op=dist.ReduceOp.MAX, **kw)
    assert torch.equal(got, torch.full((2,), float(world - 1 + 10 * rank)))
    # broadcast (any dtype) and barrier
    for root in range(world):
        v = torch.tensor([root * 100 + 7, 5], dtype=torch.int32) if rank == root else torch.zeros(2, dtype=torch.int32)
        dist.broadcast(v, src=root, **kw)
        assert v.tolist() == [root * 100 + 7, 5]
    dist.barrier(**kw)
    torch.set_default_device("cpu")


def check_ddp(group, rank, world):
    torch.manual_seed(0)
    model = torch.nn.Sequential(torch.nn.Linear(8, 16), torch.nn.Tanh(), torch.nn.Linear(16, 4)).to(DEV)
    ref = torch.nn.Sequential(torch.nn.Linear(8, 16), torch.nn.Tanh(), torch.nn.Linear(16, 4)).to(DEV)
    ref.load_state_dict(model.state_dict())
    ddp = torch.nn.parallel.DistributedDataParallel(model, process_group=group,
                                                    device_ids=[DEV.index] if DEV.type == "cuda" else None)
    data = [torch.randn(4, 8, generator=torch.Generator().manual_seed(100 + r)).to(DEV) for r in range(world)]
    ddp(data[rank]).pow(2).mean().backward()
    # reference: mean over ranks of each rank's gradient
    for r in range(world):
        ref(data[r]).pow(2).mean().div(world).backward()
    for a, b in zip(model.parameters(), ref.parameters()):
        assert torch.allclose(a.grad, b.grad, atol=1e-5), (a.grad - b.grad).abs().max()


def main():
    global DEV
    mode = sys.argv[1]
    if mode == "gpu":
        rank, world, port = int(sys.argv[2]), int(sys.argv[3]), int(sys.argv[4])
        torch.cuda.set_device(rank)
        DEV = torch.device("cuda", rank)
        dist.init_process_group("b200ccl", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
        pg = dist.distributed_c10d._get_default_group()
        assert isinstance(pg, pgmod.B200ProcessGroup)
        check_collectives(None, rank, world)
        # a view that does not start on a 16-byte boundary goes through an aligned temporary
        odd = (torch.arange(9, dtype=torch.float32, device=DEV) + rank)[1:]
        dist.all_reduce(odd)
        assert torch.equal(odd.cpu(), torch.arange(1, 9, dtype=torch.float32) * world + sum(range(world)))
        check_ddp(None, rank, world)
        assert pg.engine.comm is not None and pg.engine.comm.last_call()["algo"] != ""
        torch.cuda.synchronize()
        dist.barrier()
        pg.shutdown()
        dist.destroy_process_group()
        print("pg worker ok")
        return
    if mode == "solo":
        pgmod.set_engine_factory(SoloEngine)
        dist.init_process_group("b200ccl", store=dist.HashStore(), rank=0, world_size=1)
        pg = dist.distributed_c10d._get_default_group()
        assert isinstance(pg, pgmod.B200ProcessGroup) and dist.get_backend() == "b200ccl"
        check_collectives(None, 0, 1)
        check_ddp(None, 0, 1)
        kinds = {c[0] for c in pg.engine.calls}
        assert {"all_reduce", "all_gather", "reduce_scatter"} <= kinds
        assert ("all_reduce", "avg", 5) in pg.engine.calls  # native dtypes and operators reach the engine as such
        pg.shutdown()
        assert pg.engine.calls[-1][0] == "close"
        dist.destroy_process_group()
        # without a stand-in engine, CPU tensors are refused with a clear message
        pgmod.set_engine_factory(None)
        dist.init_process_group("b200ccl", store=dist.HashStore(), rank=0, world_size=1)
        try:
            dist.all_reduce(torch.ones(2))
            raise SystemExit("a CPU tensor was accepted")
        except RuntimeError as e:
            assert "only CUDA tensors" in str(e)
        dist.destroy_process_group()
    else:
        rank, port = int(sys.argv[2]), int(sys.argv[3])
        world = 2
        dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
        pgmod.set_engine_factory(GlooEngine)
        group = dist.new_group(backend="b200ccl")
        assert isinstance(group, pgmod.B200ProcessGroup)
        check_collectives(group, rank, world)
        check_ddp(group, rank, world)
        assert {"all_reduce", "all_gather", "reduce_scatter"} <= set(group.engine.calls)
        dist.barrier()
        dist.destroy_process_group()
    print("pg worker ok")


if __name__ == "__main__":
    main()
