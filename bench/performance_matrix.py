#!/usr/bin/env python
"""AllReduce dtype x reduction matrix against NCCL, rendered as a markdown table.

For float / fp16 / bf16 and sum / avg / max / min, at 256 KiB ... 64 MiB (x4) per rank, with
values N(0,1) seeded per rank: bus bandwidth of this library (symmetric tensors) and of
torch.distributed NCCL on the same GPUs, their ratio, and the number of wrong elements against an
fp32 reference. One process per GPU:

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29551 bench/performance_matrix.py --out performance_n8.md

Covers what the reference's scripts/run_performance_matrix.sh + render_performance_md.py produce
(nano-nccl vs nccl-tests), with device-side timing (CUDA events, maximum over ranks).
"""
import argparse
import os
import socket
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
import nano_nccl_b200 as nn  # noqa: E402

TOL = {"float": 1e-5, "fp16": 1e-2, "bf16": 1e-1}
DT = {"float": torch.float32, "fp16": torch.float16, "bf16": torch.bfloat16}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", default="")
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    args = ap.parse_args()
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", rank=rank, world_size=world)
    port = [0]
    if rank == 0:
        s = socket.socket(); s.bind(("127.0.0.1", 0)); port[0] = s.getsockname()[1]; s.close()
    dist.broadcast_object_list(port, src=0)
    comm = nn.Communicator(devices=[local], rank=rank, world_size=world, port=port[0])
    sizes = [262144, 1048576, 4194304, 16777216, 67108864]
    nccl_ops = {"sum": dist.ReduceOp.SUM, "avg": dist.ReduceOp.AVG, "max": dist.ReduceOp.MAX, "min": dist.ReduceOp.MIN}
    factor = 2 * (world - 1) / world

    def timed(fn):
        for _ in range(args.warmup):
            fn()
        dist.barrier()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(args.iters):
            fn()
        b.record()
        torch.cuda.synchronize()
        t = torch.tensor([a.elapsed_time(b) / 1e3 / args.iters], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    lines = [f"# AllReduce matrix on {world} x B200: this library vs NCCL {'.'.join(map(str, torch.cuda.nccl.version()))}",
             "", "Cell: `ours busbw / NCCL busbw (ratio)` in GB/s; `#wrong` summed over the row. CUDA-event timing, max over ranks,",
             f"{args.warmup} warm-up + {args.iters} timed calls, values N(0,1) seeded per rank, symmetric tensors for this library.", "",
             "| dtype | op | " + " | ".join(f"{s // 1024} KiB" if s < 1 << 20 else f"{s >> 20} MiB" for s in sizes) + " | #wrong |",
             "|---|---|" + "---|" * (len(sizes) + 1)]
    for dname, dtype in DT.items():
        for op in ("sum", "avg", "max", "min"):
            cells, wrong_total = [], 0
            for size in sizes:
                numel = size // torch.empty((), dtype=dtype).element_size()
                gen = torch.Generator(device=dev).manual_seed(7 + rank)
                x = comm.empty(numel, dtype)
                y = comm.empty(numel, dtype)
                x.copy_(torch.randn(numel, device=dev, generator=gen).to(dtype))
                t_ours = timed(lambda: comm.all_reduce(y, x, op=op))
                comm.check_async_error()
                # reference result in fp32 from every rank's seeded input
                acc = None
                for r in range(world):
                    g = torch.Generator(device=dev).manual_seed(7 + r)
                    v = torch.randn(numel, device=dev, generator=g).to(dtype).float()
                    acc = v if acc is None else (acc + v if op in ("sum", "avg") else (torch.maximum(acc, v) if op == "max" else torch.minimum(acc, v)))
                if op == "avg":
                    acc /= world
                wrong = int(((y.float() - acc).abs() > TOL[dname]).sum().item())
                w = torch.tensor([wrong], device=dev)
                dist.all_reduce(w)
                wrong_total += int(w.item())
                z = x.clone()
                t_nccl = timed(lambda: dist.all_reduce(z, op=nccl_ops[op]))
                bo, bn = size / t_ours / 1e9 * factor, size / t_nccl / 1e9 * factor
                cells.append(f"{bo:.1f} / {bn:.1f} ({bo / bn:.2f})")
                del x, y, z
            lines.append(f"| {dname} | {op} | " + " | ".join(cells) + f" | {wrong_total} |")
    if rank == 0:
        text = "\n".join(lines) + "\n"
        print(text)
        if args.out:
            with open(args.out, "w") as f:
                f.write(text)
    comm.close()
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
