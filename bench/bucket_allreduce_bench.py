#!/usr/bin/env python
"""Gradient-bucket all-reduce from PyTorch, one process per GPU.

A list of bf16 tensors shaped like a GPT-2-small layer stack (124M elements: hidden 768, 12 layers,
vocabulary 50257), values N(0, 0.02) seeded per rank, is packed into 25 MiB buckets and averaged
over the ranks on a side stream, alone and overlapped with a stream of synthetic matmuls.
Reports the time of the reduction alone, of the matmuls alone, and of both together, for this
library (`--impl ours`, symmetric buckets, in-place, avg fused) and for torch.distributed NCCL
(`--impl nccl`). Prints one JSON line from rank 0.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29541 bench/bucket_allreduce_bench.py --impl ours
"""
import argparse
import json
import os
import socket
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from nano_nccl_b200.models import gpt2_small_shapes  # noqa: E402
from nano_nccl_b200.parallel import BucketAllReducer, CclBackend, TorchDistBackend  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--impl", default="ours", choices=["ours", "nccl"])
    ap.add_argument("--bucket-mib", type=int, default=25)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--matmul-n", type=int, default=8192)
    ap.add_argument("--matmuls", type=int, default=12)
    ap.add_argument("--max-ctas", type=int, default=0,
                    help="CTAs a collective may occupy per GPU (0: defaults); small values leave SMs to the matmuls")
    args = ap.parse_args()
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", rank=rank, world_size=world)

    comm = None
    if args.impl == "ours":
        import nano_nccl_b200 as nn
        port = [0]
        if rank == 0:
            s = socket.socket(); s.bind(("127.0.0.1", 0)); port[0] = s.getsockname()[1]; s.close()
        if world > 1:
            dist.broadcast_object_list(port, src=0)
        comm = nn.Communicator(devices=[local], rank=rank, world_size=world, port=port[0], max_ctas=args.max_ctas)
        backend = CclBackend(comm)
    else:
        backend = TorchDistBackend()

    shapes = gpt2_small_shapes()
    gen = torch.Generator(device=dev).manual_seed(1234 + rank)
    grads = [(torch.randn(s, device=dev, generator=gen) * 0.02).to(torch.bfloat16) for s in shapes]
    numels = [g.numel() for g in grads]
    reducer = BucketAllReducer(backend, numels, torch.bfloat16, dev, bucket_bytes=args.bucket_mib << 20, op="avg")
    views = reducer.views()

    # correctness of one reduction against an fp32 reference of the first and last tensors
    ref = []
    for idx in (0, len(grads) - 1):
        acc = torch.zeros(numels[idx], device=dev)
        for r in range(world):
            g = torch.Generator(device=dev).manual_seed(1234 + r)
            t = None
            for k, s in enumerate(shapes):
                x = (torch.randn(s, device=dev, generator=g) * 0.02).to(torch.bfloat16)
                if k == idx:
                    t = x
                    break
            acc += t.float().view(-1)
        ref.append(acc / world)
    work = [g.clone() for g in grads]
    reducer.reduce(work)
    torch.cuda.synchronize()
    err = max((work[0].float().view(-1) - ref[0]).abs().max().item(), (work[-1].float().view(-1) - ref[1]).abs().max().item())

    a = torch.randn(args.matmul_n, args.matmul_n, device=dev, dtype=torch.bfloat16)
    b = torch.randn(args.matmul_n, args.matmul_n, device=dev, dtype=torch.bfloat16)

    def fill():
        torch._foreach_copy_(views, [g.view(-1) for g in grads])

    def reduce_all():
        for bkt in range(reducer.plan.num_buckets):
            reducer.reduce_bucket(bkt)
        reducer.wait()

    def matmuls():
        c = None
        for _ in range(args.matmuls):
            c = a @ b
        return c

    def timed(fn):
        for _ in range(3):
            fill()
            fn()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        total = 0.0
        for _ in range(args.iters):
            fill()  # untimed: fresh gradients (and cold L2) for every iteration
            torch.cuda.synchronize()
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            fn()
            stop.record()
            torch.cuda.synchronize()
            total += start.elapsed_time(stop)
        t = torch.tensor([total / args.iters], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    t_reduce = timed(reduce_all)
    t_matmul = timed(matmuls)

    def both():
        for bkt in range(reducer.plan.num_buckets):
            reducer.reduce_bucket(bkt)
        matmuls()
        reducer.wait()

    t_both = timed(both)
    if comm is not None:
        comm.check_async_error()
    if rank == 0:
        total_bytes = sum(numels) * 2
        factor = 2 * (world - 1) / world if world > 1 else 1.0
        print(json.dumps({
            "bench": "gpt2_small_gradient_buckets", "impl": args.impl, "n_gpus": world, "elements": sum(numels),
            "buckets": reducer.plan.num_buckets, "bucket_mib": args.bucket_mib, "dtype": "bf16", "op": "avg",
            "reduce_ms": round(t_reduce, 3), "matmul_ms": round(t_matmul, 3), "overlapped_ms": round(t_both, 3),
            "busbw_gbs": round(total_bytes / (t_reduce / 1e3) / 1e9 * factor, 2),
            "overlap_hidden_fraction": round(max(0.0, (t_reduce + t_matmul - t_both) / min(t_reduce, t_matmul)), 3),
            "max_abs_error": err, "launches_per_reduction": reducer.plan.num_buckets,
            "algo": comm.last_call()["algo"] if comm is not None else "nccl"}), flush=True)
    if comm is not None:
        del reducer, views
        comm.close()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
