"""``torch.distributed`` backend ``"b200ccl"``: importing this module registers it, after which

    import nano_nccl_b200.parallel.process_group  # noqa: F401
    torch.distributed.init_process_group("b200ccl", ...)      # or dist.new_group(backend="b200ccl")

routes ``all_reduce`` / ``reduce_scatter_tensor`` / ``all_gather_into_tensor`` (and their list forms) on
CUDA tensors of float32 / float16 / bfloat16 with sum / avg / max / min to this library's kernels, on
the CURRENT stream (work objects are already complete: the next kernel on that stream is ordered after
the collective, which is the guarantee ``Work.wait()`` gives for NCCL). ``torch.nn.parallel.
DistributedDataParallel`` and ``FSDP`` run on it unchanged.

The library has three collectives; what else a process group must answer is built from them:
``broadcast`` = all-gather of the raw bytes + pick the root's block (N times the traffic, meant for
parameter synchronisation at start-up, not for hot loops); ``barrier`` = a one-element all-reduce and a
stream synchronisation; all-reduce of other dtypes or operators (integers, product, bitwise) = all-gather
of the raw bytes + a local reduction. Point-to-point, scatter/gather and all-to-all are not provided.

The reference library has no PyTorch layer; this stands where a user of it would have written glue.
"""
import socket

import torch
import torch.distributed as dist
from torch._C._distributed_c10d import _create_work_from_future
from torch.distributed.distributed_c10d import (AllgatherOptions, AllreduceOptions, BarrierOptions, BroadcastOptions,
                                                ReduceOp, ReduceScatterOptions)
from torch.futures import Future

BACKEND_NAME = "b200ccl"
_NATIVE_DTYPES = (torch.float32, torch.float16, torch.bfloat16)
_PAD = 16  # raw-byte exchanges are padded to whole 16-byte vectors


def _done(result):
    fut = Future()
    fut.set_result(result)
    return _create_work_from_future(fut)


def _native_op(op):
    for torch_op, name in ((ReduceOp.SUM, "sum"), (ReduceOp.AVG, "avg"), (ReduceOp.MAX, "max"), (ReduceOp.MIN, "min")):
        if op == torch_op:
            return name
    return None


def _local_reduce(stacked, op):
    """Reduces dim 0 of ``stacked`` ([world, ...]) with a torch operator (fallback path)."""
    if op == ReduceOp.SUM:
        return stacked.sum(0).to(stacked.dtype)
    if op == ReduceOp.AVG:
        return (stacked.sum(0) / stacked.shape[0]).to(stacked.dtype)
    if op == ReduceOp.PRODUCT:
        return stacked.prod(0).to(stacked.dtype)
    if op == ReduceOp.MAX:
        return stacked.max(0).values
    if op == ReduceOp.MIN:
        return stacked.min(0).values
    out = stacked[0].clone()
    for row in stacked[1:]:
        if op == ReduceOp.BAND:
            out &= row
        elif op == ReduceOp.BOR:
            out |= row
        elif op == ReduceOp.BXOR:
            out ^= row
        else:
            raise NotImplementedError(f"b200ccl: reduction {op} is not supported")
    return out


class CommunicatorEngine:
    """The three collectives on flat CUDA tensors, carried out by a :class:`nano_nccl_b200.Communicator`
    that is created on first use (rank 0 publishes the rendezvous port through the group's store)."""

    def __init__(self, store, rank, size):
        self.store, self.rank, self.world_size = store, rank, size
        self.comm = None

    def supports(self, tensor):
        return tensor.is_cuda and tensor.dtype in _NATIVE_DTYPES

    def _ensure(self, device):
        if self.comm is None:
            import nano_nccl_b200 as nn

            if self.rank == 0:
                s = socket.socket()
                s.bind(("127.0.0.1", 0))
                port = s.getsockname()[1]
                s.close()
                self.store.set("b200ccl_rendezvous_port", str(port))
            else:
                port = int(self.store.get("b200ccl_rendezvous_port"))
            index = device.index if device.index is not None else torch.cuda.current_device()
            self.comm = nn.Communicator(devices=[index], rank=self.rank, world_size=self.world_size, port=port)
        return self.comm

    # Buffers that travel between processes must start on a 16-byte boundary; a view that does not
    # (say ``x[1:]``) goes through an aligned temporary.
    @staticmethod
    def _misaligned(*tensors):
        return any(t.data_ptr() % 16 for t in tensors)

    def all_reduce(self, out, inp, op):
        comm = self._ensure(inp.device)
        if self._misaligned(out, inp):
            tmp = inp.clone()
            comm.all_reduce(tmp, op=op)
            out.copy_(tmp)
        else:
            comm.all_reduce(out, inp, op=op)

    def reduce_scatter(self, out, inp, op):
        comm = self._ensure(inp.device)
        if self._misaligned(out, inp):
            tmp_out = torch.empty_like(out)
            comm.reduce_scatter(tmp_out, inp.clone(), op=op)
            out.copy_(tmp_out)
        else:
            comm.reduce_scatter(out, inp, op=op)

    def all_gather(self, out, inp):
        comm = self._ensure(inp.device)
        if self._misaligned(out, inp):
            tmp_out = torch.empty_like(out)
            comm.all_gather(tmp_out, inp.clone())
            out.copy_(tmp_out)
        else:
            comm.all_gather(out, inp)

    def synchronize(self, device):
        torch.cuda.current_stream(device).synchronize()

    def close(self):
        if self.comm is not None:
            self.comm.close()
            self.comm = None


_engine_factory = CommunicatorEngine


def set_engine_factory(factory):
    """Replaces what carries the collectives out (``factory(store, rank, size)`` → an object with the
    methods of :class:`CommunicatorEngine`). Used by the CPU tests; returns the previous factory."""
    global _engine_factory
    previous, _engine_factory = _engine_factory, (factory or CommunicatorEngine)
    return previous


class B200ProcessGroup(dist.ProcessGroup):
    def __init__(self, store, rank, size, timeout=None):
        super().__init__(rank, size)
        self._rank, self._size = rank, size
        self.engine = _engine_factory(store, rank, size)

    def size(self):
        return self._size

    def rank(self):
        return self._rank

    def getBackendName(self):
        return BACKEND_NAME

    def __repr__(self):
        return f"B200ProcessGroup(rank={self._rank}, size={self._size})"

    # -- helpers -------------------------------------------------------------------------------
    def _check(self, tensor):
        if not tensor.is_cuda and not getattr(self.engine, "any_device", False):
            raise RuntimeError("b200ccl: only CUDA tensors can take part in a collective")

    def _gather_bytes(self, tensor):
        """[world, nbytes] uint8: every rank's copy of ``tensor``, bit for bit."""
        src = tensor.contiguous().view(-1).view(torch.uint8)
        n = src.numel()
        padded = max(-(-n // _PAD) * _PAD, _PAD)
        mine = torch.zeros(padded, dtype=torch.uint8, device=tensor.device)
        mine[:n] = src
        everyone = torch.empty(self._size * padded, dtype=torch.uint8, device=tensor.device)
        self.engine.all_gather(everyone.view(torch.float32), mine.view(torch.float32))
        return everyone.view(self._size, padded), n

    def _gather_like(self, tensor):
        """[world, *tensor.shape] with ``tensor``'s dtype."""
        raw, n = self._gather_bytes(tensor)
        rows = [raw[r, :n].view(tensor.dtype).view(tensor.shape) for r in range(self._size)]
        return torch.stack(rows)

    # -- collectives ---------------------------------------------------------------------------
    def allreduce(self, tensor_list, opts=AllreduceOptions()):
        for t in tensor_list:
            self._check(t)
            name = _native_op(opts.reduceOp)
            if name is not None and self.engine.supports(t) and t.numel() > 0:
                if t.is_contiguous():
                    flat = t.view(-1)
                    self.engine.all_reduce(flat, flat, name)
                else:
                    flat = t.contiguous().view(-1)
                    self.engine.all_reduce(flat, flat, name)
                    t.copy_(flat.view(t.shape))
            else:
                t.copy_(_local_reduce(self._gather_like(t), opts.reduceOp))
        return _done(tensor_list)

    def allreduce_coalesced(self, tensor_list, opts=AllreduceOptions()):
        return self.allreduce(tensor_list, opts)

    def _allgather_base(self, output_tensor, input_tensor, opts=AllgatherOptions()):
        self._check(input_tensor)
        if self.engine.supports(input_tensor) and output_tensor.is_contiguous() and input_tensor.numel() > 0:
            self.engine.all_gather(output_tensor.view(-1), input_tensor.contiguous().view(-1))
        else:
            output_tensor.copy_(self._gather_like(input_tensor).view(output_tensor.shape))
        return _done(output_tensor)

    def allgather(self, output_tensors, input_tensor, opts=AllgatherOptions()):
        for outs, inp in zip(output_tensors, input_tensor):
            self._check(inp)
            gathered = self._gather_like(inp)
            for r, o in enumerate(outs):
                o.copy_(gathered[r])
        return _done(output_tensors)

    def allgather_into_tensor_coalesced(self, output_tensor_list, input_tensor_list, opts=AllgatherOptions()):
        for o, i in zip(output_tensor_list, input_tensor_list):
            self._allgather_base(o, i, opts)
        return _done(output_tensor_list)

    def _reduce_scatter_base(self, output_tensor, input_tensor, opts=ReduceScatterOptions()):
        self._check(input_tensor)
        name = _native_op(opts.reduceOp)
        if name is not None and self.engine.supports(input_tensor) and output_tensor.is_contiguous():
            self.engine.reduce_scatter(output_tensor.view(-1), input_tensor.contiguous().view(-1), name)
        else:
            reduced = _local_reduce(self._gather_like(input_tensor.contiguous().view(self._size, -1)), opts.reduceOp)
            output_tensor.copy_(reduced[self._rank].view(output_tensor.shape))
        return _done(output_tensor)

    def reduce_scatter(self, output_tensors, input_tensors, opts=ReduceScatterOptions()):
        for out, blocks in zip(output_tensors, input_tensors):
            self._reduce_scatter_base(out, torch.cat([b.reshape(-1) for b in blocks]), opts)
        return _done(output_tensors)

    def reduce_scatter_tensor_coalesced(self, output_tensors, input_tensors, opts=ReduceScatterOptions()):
        for o, i in zip(output_tensors, input_tensors):
            self._reduce_scatter_base(o, i, opts)
        return _done(output_tensors)

    def broadcast(self, tensor_list, opts=BroadcastOptions()):
        for t in tensor_list:
            self._check(t)
            if t.numel() == 0:
                continue
            raw, n = self._gather_bytes(t)
            if self._rank != opts.rootRank:
                t.copy_(raw[opts.rootRank, :n].view(t.dtype).view(t.shape))
        return _done(tensor_list)

    def barrier(self, opts=BarrierOptions()):
        device = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")
        token = torch.ones(4, dtype=torch.float32, device=device)
        self.engine.all_reduce(token, token, "sum")
        self.engine.synchronize(device)
        return _done([])

    def shutdown(self):
        self.engine.close()


def _create(store, rank, size, timeout):
    return B200ProcessGroup(store, rank, size, timeout)


if not hasattr(dist.Backend, BACKEND_NAME.upper()):
    dist.Backend.register_backend(BACKEND_NAME, _create, devices=["cuda", "cpu"])
