"""Bucketed all-reduce of a list of tensors (a ProcessGroup-style gradient reducer).

Tensors are assigned, in order, to flat buckets of at most ``bucket_bytes`` (25 MiB by default).
Each bucket is reduced with one collective issued on a side stream, after an event recorded on the
producing stream, so that the reduction of one bucket overlaps whatever the main stream does next.
With the b200ccl backend the buckets are symmetric tensors: peers (and the NVSwitch multicast
engine) address them directly and the all-reduce runs in place, with the avg 1/N scale fused.

The reference library has no such layer; this is the thin PyTorch layer that drives it.
"""
import torch


class BucketPlan:
    """Pure bookkeeping (no device needed): which tensor goes where.

    ``slots[i] = (bucket, offset, numel)`` for tensor i; ``bucket_numel[b]`` is bucket b's size in
    elements, rounded up to a multiple of ``align`` elements so that every bucket is a whole number
    of 16-byte vectors for any supported dtype."""

    def __init__(self, numels, element_size, bucket_bytes=25 << 20, align=8):
        if bucket_bytes <= 0:
            raise ValueError("bucket_bytes must be positive")
        self.slots = []
        self.bucket_numel = []
        cap = max(bucket_bytes // element_size, 1)
        cur = 0
        for n in numels:
            n = int(n)
            if cur > 0 and cur + n > cap:
                self.bucket_numel.append(-(-cur // align) * align)
                cur = 0
            self.slots.append((len(self.bucket_numel), cur, n))
            cur += -(-n // align) * align if n % align else n
        if cur > 0 or not self.bucket_numel:
            self.bucket_numel.append(max(-(-cur // align) * align, align))

    @property
    def num_buckets(self):
        return len(self.bucket_numel)

    def tensors_of(self, bucket):
        return [i for i, s in enumerate(self.slots) if s[0] == bucket]


class CclBackend:
    """Reduces buckets with a b200ccl communicator (one process per GPU)."""

    def __init__(self, comm):
        self.comm = comm
        self.world_size = comm.world_size

    def empty(self, numel, dtype, device):
        return self.comm.empty(numel, dtype)

    def all_reduce_(self, flat, op, stream):
        self.comm.all_reduce(flat, op=op, stream=stream)


class TorchDistBackend:
    """Reduces buckets with torch.distributed (gloo on CPU, NCCL on GPU): comparator and CPU tests."""

    def __init__(self, group=None):
        import torch.distributed as dist
        self.dist = dist
        self.group = group
        self.world_size = dist.get_world_size(group)

    def empty(self, numel, dtype, device):
        return torch.empty(numel, dtype=dtype, device=device)

    def all_reduce_(self, flat, op, stream):
        dist = self.dist
        if op == "avg":
            # gloo has no AVG: sum, then scale (the b200ccl backend fuses the scale instead).
            dist.all_reduce(flat, op=dist.ReduceOp.SUM, group=self.group)
            flat.div_(self.world_size)
        else:
            ops = {"sum": dist.ReduceOp.SUM, "max": dist.ReduceOp.MAX, "min": dist.ReduceOp.MIN}
            dist.all_reduce(flat, op=ops[op], group=self.group)


class BucketAllReducer:
    def __init__(self, backend, numels, dtype, device, bucket_bytes=25 << 20, op="avg"):
        self.backend = backend
        self.op = op
        self.dtype = dtype
        self.device = torch.device(device)
        self.plan = BucketPlan(numels, torch.empty((), dtype=dtype).element_size(), bucket_bytes)
        self.buckets = [backend.empty(n, dtype, self.device) for n in self.plan.bucket_numel]
        for b in self.buckets:
            b.zero_()
        self.cuda = self.device.type == "cuda"
        # High priority: when the reduction is issued beside a stream of matmuls, its CTAs (which spin until
        # the same CTAs of every rank are resident) are placed as soon as an SM frees up instead of after the
        # matmul's whole grid.
        self.stream = torch.cuda.Stream(self.device, priority=-1) if self.cuda else None
        self._ready = [torch.cuda.Event() for _ in self.buckets] if self.cuda else []
        self._done = [torch.cuda.Event() for _ in self.buckets] if self.cuda else []
        self.launches = 0

    def views(self, shapes=None):
        """One view per tensor into its bucket (write gradients here to skip the packing copy)."""
        out = []
        for i, (b, off, n) in enumerate(self.plan.slots):
            v = self.buckets[b][off:off + n]
            out.append(v.view(shapes[i]) if shapes is not None else v)
        return out

    def reduce_bucket(self, bucket):
        """Reduces one bucket in place on the side stream, ordered after the current stream."""
        flat = self.buckets[bucket]
        if self.cuda:
            self._ready[bucket].record(torch.cuda.current_stream(self.device))
            self.stream.wait_event(self._ready[bucket])
            with torch.cuda.stream(self.stream):
                self.backend.all_reduce_(flat, self.op, self.stream)
                self._done[bucket].record(self.stream)
        else:
            self.backend.all_reduce_(flat, self.op, None)
        self.launches += 1

    def wait(self):
        """Makes the current stream wait for every bucket reduced so far."""
        if self.cuda:
            cur = torch.cuda.current_stream(self.device)
            for e in self._done:
                cur.wait_event(e)

    def reduce(self, tensors):
        """Packs ``tensors`` into the buckets, reduces every bucket, unpacks in place and returns
        after ordering the current stream behind the reductions."""
        views = self.views()
        for b in range(self.plan.num_buckets):
            idx = self.plan.tensors_of(b)
            torch._foreach_copy_([views[i] for i in idx], [tensors[i].reshape(-1) for i in idx])
            self.reduce_bucket(b)
        self.wait()
        for b in range(self.plan.num_buckets):
            idx = self.plan.tensors_of(b)
            torch._foreach_copy_([tensors[i].view(-1) for i in idx], [views[i] for i in idx])
        return tensors
