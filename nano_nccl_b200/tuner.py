"""Measures every algorithm / CTA-count candidate over message sizes on the GPUs at hand and
writes the table (and the winners per size) to a JSON file; the crossover points in
src/sched/plan.cc (default_tuning) are taken from these tables.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29521 -m nano_nccl_b200.tuner --out tuning/b200_n8.json

Timing: CUDA events around a batch of back-to-back calls (optionally replayed from a CUDA graph
to take the Python call cost out), maximum over ranks; buffers are symmetric tensors, rotated
over several sets for sizes that would otherwise sit in L2.
"""
import argparse
import json
import os
import socket
import sys

import torch
import torch.distributed as dist

import nano_nccl_b200 as nn

L2_BYTES = 126 * 1000 * 1000


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", default="")
    ap.add_argument("--min-bytes", type=int, default=1024)
    ap.add_argument("--max-bytes", type=int, default=1 << 30)
    ap.add_argument("--collective", default="all_reduce", choices=["all_reduce", "reduce_scatter", "all_gather"])
    ap.add_argument("--dtype", default="float", choices=["float", "fp16", "bf16"])
    ap.add_argument("--op", default="sum")
    ap.add_argument("--algos", default="oneshot,twoshot,nvls",
                    help="comma list of oneshot,twoshot,nvls,ring,ll (ll: all_reduce up to 128 KiB, one CTA count)")
    ap.add_argument("--ctas", default="16,32,64,128")
    ap.add_argument("--unrolls", default="", help="comma list of multimem loads in flight per thread (2,4,8) to try for nvls")
    ap.add_argument("--sizes", default="", help="comma list of message sizes in bytes (default: every power of two in range)")
    ap.add_argument("--iters", type=int, default=0, help="calls per timed batch (default: by size)")
    ap.add_argument("--graph", action="store_true", help="replay each batch from a CUDA graph")
    ap.add_argument("--emit-tuning", default="", help="also write the crossovers as a tuning file (B200CCL_TUNING_FILE)")
    ap.add_argument("--buffers", default="symmetric", choices=["symmetric", "plain"])
    ap.add_argument("--impl", default="ours", choices=["ours", "nccl"],
                    help="nccl: time torch.distributed's NCCL collectives on the same sizes (comparator)")
    return ap.parse_args()


def main():
    args = parse_args()
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", rank=rank, world_size=world)
    dtype = {"float": torch.float32, "fp16": torch.float16, "bf16": torch.bfloat16}[args.dtype]
    esize = torch.empty((), dtype=dtype).element_size()

    def max_over_ranks(v):
        if world == 1:
            return v
        t = torch.tensor([v], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    class NcclComm:
        """torch.distributed NCCL behind the small interface the loop below uses."""
        nvls = True

        def empty(self, n, dt):
            return torch.empty(n, dtype=dt, device=dev)

        def all_reduce(self, y, x, op="sum"):
            dist.all_reduce(x, op={"sum": dist.ReduceOp.SUM, "avg": dist.ReduceOp.AVG, "max": dist.ReduceOp.MAX, "min": dist.ReduceOp.MIN}[op])

        def reduce_scatter(self, y, x, op="sum"):
            dist.reduce_scatter_tensor(y, x, op=dist.ReduceOp.SUM if op == "sum" else dist.ReduceOp.AVG)

        def all_gather(self, y, x):
            dist.all_gather_into_tensor(y, x)

        def check_async_error(self):
            pass

        def last_call(self):
            return {"algo": "nccl", "grid": 0}

        def close(self):
            pass

    rows = []
    algos = ["nccl"] if args.impl == "nccl" else args.algos.split(",")
    cta_list = [0] if args.impl == "nccl" else [int(c) for c in args.ctas.split(",")]
    unrolls = [int(u) for u in args.unrolls.split(",")] if args.unrolls else [0]
    size_list = [int(s) for s in args.sizes.split(",")] if args.sizes else None
    for algo, ctas, unroll in [(a, c, u) for a in algos for c in cta_list for u in (unrolls if a == "nvls" else [0])]:
        if True:
            if args.impl == "nccl":
                comm = NcclComm()
                yield_comm = True
            else:
                yield_comm = False
            if not yield_comm:
                if ctas > 0:
                    os.environ["B200CCL_MAX_CTAS"] = str(ctas)  # an explicit cap applies to every algorithm
                else:
                    os.environ.pop("B200CCL_MAX_CTAS", None)    # 0: the library's own per-algorithm caps
                if unroll:
                    os.environ["B200CCL_NVLS_UNROLL"] = str(unroll)
                port = [0]
                if rank == 0:
                    s = socket.socket(); s.bind(("127.0.0.1", 0)); port[0] = s.getsockname()[1]; s.close()
                if world > 1:
                    dist.broadcast_object_list(port, src=0)
                comm = nn.Communicator(devices=[local], rank=rank, world_size=world, port=port[0], algo=algo)
                if algo == "nvls" and not comm.nvls:
                    comm.close()
                    continue
            sizes = size_list if size_list is not None else [args.min_bytes << k for k in range(64) if (args.min_bytes << k) <= args.max_bytes]
            for size in sizes:
                if algo == "oneshot" and size > (8 << 20):
                    break
                if algo == "ll" and (size > (128 << 10) or args.collective != "all_reduce" or ctas != cta_list[0]):
                    break  # fixed grid of 8 CTAs: one pass is enough
                numel = max(size // esize, 1)
                in_mult = world if args.collective == "reduce_scatter" else 1
                out_mult = world if args.collective == "all_gather" else 1
                per_set = numel * esize * (in_mult + out_mult)
                nsets = int(min(8, max(1, -(-4 * L2_BYTES // per_set))))
                alloc = (lambda n: comm.empty(n, dtype)) if args.buffers == "symmetric" else (lambda n: torch.empty(n, dtype=dtype, device=dev))
                try:
                    sets = []
                    for _ in range(nsets):
                        x, y = alloc(numel * in_mult), alloc(numel * out_mult)
                        x.normal_()
                        sets.append((x, y))

                    def call(i):
                        x, y = sets[i % nsets]
                        if args.collective == "all_reduce":
                            comm.all_reduce(y, x, op=args.op)
                        elif args.collective == "reduce_scatter":
                            comm.reduce_scatter(y, x, op=args.op)
                        else:
                            comm.all_gather(y, x)

                    iters = args.iters or (200 if size <= (1 << 20) else (40 if size <= (64 << 20) else 8))
                    for i in range(5):
                        call(i)
                    barrier()
                    comm.check_async_error()
                    graph = None
                    if args.graph:
                        graph = torch.cuda.CUDAGraph()
                        with torch.cuda.graph(graph):
                            for i in range(iters):
                                call(i)
                        graph.replay()
                        barrier()
                    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    start.record()
                    if graph is not None:
                        graph.replay()
                    else:
                        for i in range(iters):
                            call(i)
                    stop.record()
                    barrier()
                    comm.check_async_error()
                    t = max_over_ranks(start.elapsed_time(stop) / 1e3 / iters)
                    info = comm.last_call()
                    total = numel * esize * (1 if args.collective == "all_reduce" else world)
                    factor = (2 * (world - 1) / world if args.collective == "all_reduce" else (world - 1) / world) if world > 1 else 1.0
                    rows.append({"collective": args.collective, "algo": info["algo"], "requested": algo, "max_ctas": ctas, "unroll": unroll,
                                 "grid": info["grid"], "bytes": numel * esize, "time_us": round(t * 1e6, 2),
                                 "busbw_gbs": round(total / t / 1e9 * factor, 2)})
                    del sets, graph
                except Exception as e:  # a candidate that cannot run (e.g. forced algorithm impossible) is skipped
                    if rank == 0:
                        print(f"skip {algo} ctas={ctas} size={size}: {e}", file=sys.stderr)
                    break
            comm.close()
    if rank == 0:
        best = {}
        for r in rows:
            cur = best.get(r["bytes"])
            if cur is None or r["time_us"] < cur["time_us"]:
                best[r["bytes"]] = r
        result = {"n_gpus": world, "dtype": args.dtype, "op": args.op, "collective": args.collective, "graph": args.graph,
                  "buffers": args.buffers, "rows": rows, "best": [best[k] for k in sorted(best)]}
        if args.out:
            os.makedirs(os.path.dirname(os.path.abspath(args.out)), exist_ok=True)
            with open(args.out, "w") as f:
                json.dump(result, f, indent=1)
        if args.emit_tuning and args.collective == "all_reduce":
            from .tuning_file import derive_tuning, format_tuning
            with open(args.emit_tuning, "w") as f:
                f.write(format_tuning(derive_tuning([result]), f"{world} GPUs, {args.dtype} {args.op}, graph={args.graph}"))
        print(f"# best per size ({world} GPUs, {args.collective}, {args.dtype} {args.op}, graph={args.graph})")
        for k in sorted(best):
            b = best[k]
            print(f"{k:>12} {b['time_us']:>10.2f} us {b['busbw_gbs']:>9.2f} GB/s  {b['algo']:<8} ctas<={b['max_ctas']} grid={b['grid']}")
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
