#!/usr/bin/env python
"""Headline benchmark: AllReduce bus bandwidth (GB/s) on N B200s of one node.

One step = one out-of-place float32 sum AllReduce of 64 MiB per rank (the largest size of the
reference's published table, performance.md:28-32) through this package's public API, one process
per GPU. Prints ONE JSON line from rank 0.

    python bench.py --gpus 1 --steps 200 --warmup 20
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29511 bench.py --gpus 8 --steps 200 --warmup 20
    ... bench.py --impl reference   # the unmodified reference's own benchmark binary
    ... bench.py --impl nccl        # torch.distributed NCCL on the same buffers (comparator)
    ... bench.py --impl nccl-ring   # NCCL pinned to Ring + Simple, 4 channels, 32 MiB buffer

Timing: W warm-up steps, then batches of exactly K steps, each batch between a barrier + device
synchronize on both sides and measured with CUDA events on the launching stream, maximum over
ranks; the batch is repeated (7 times by default) and the MEDIAN batch is reported, with the
fastest and slowest beside it. Successive steps rotate over buffer sets whose total exceeds the
126 MB L2. SM clocks and throttle reasons are sampled during the timed batches. A short sweep over
message sizes is measured the same way and printed under "sweep".
"""
import argparse
import json
import os
import socket
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

HEADLINE_BYTES = 64 << 20
BASELINE_BUSBW = 23.12  # nano-nccl, 4x A6000, float sum, 64 MiB (performance.md:32)
L2_BYTES = 126 * 1000 * 1000


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "nccl", "nccl-ring"])
    ap.add_argument("--bytes", type=int, default=HEADLINE_BYTES)
    ap.add_argument("--dtype", default="float", choices=["float", "fp16", "bf16"])
    ap.add_argument("--op", default="sum", choices=["sum", "avg", "max", "min"])
    ap.add_argument("--buffers", default="symmetric", choices=["symmetric", "plain", "registered"],
                    help="symmetric: tensors from Communicator.empty (peer-mapped, NVLS-capable); plain: torch.empty "
                         "(staged inside the kernel); registered: torch.empty + Communicator.register (peer-mapped)")
    ap.add_argument("--algo", default="auto")
    ap.add_argument("--repeats", type=int, default=7, help="timed batches of --steps steps; the median batch is reported")
    ap.add_argument("--sweep", default="short", choices=["short", "full", "none"],
                    help="short: 1 KiB, 64 KiB, 1 MiB, 16 MiB, 64 MiB, 1 GiB; full: every power of two from 1 KiB to --sweep-max")
    ap.add_argument("--sweep-max", type=int, default=1 << 30)
    ap.add_argument("--ref-transport", default="p2p", choices=["auto", "p2p", "shm"])
    return ap.parse_args()


from nano_nccl_b200.utils.clocks import ClockSampler  # noqa: E402  (reads clocks only)


# ---------------------------------------------------------------------------------------------
# helpers

def free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def dist_env():
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", str(rank)))
    return rank, world, local


def init_dist(backend):
    import torch.distributed as dist
    rank, world, _ = dist_env()
    if world > 1 and not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group(backend=backend, rank=rank, world_size=world)
    return dist


def busbw(nbytes, seconds, n):
    alg = nbytes / seconds / 1e9
    return alg * 2 * (n - 1) / n if n > 1 else alg


def link_bytes_per_direction(algo, nbytes, n):
    """Bytes that leave (and that enter) one GPU over NVLink for an AllReduce of nbytes per rank."""
    if n < 2:
        return 0.0
    if algo == "nvls" or (algo == "pipeline" and n >= 3):
        # every shard goes out once to the switch and the result comes back multicast (the tile pipeline
        # reduces through the switch from three ranks up; its staging copies stay inside the GPU)
        return nbytes * (1 + 1.0 / n)
    if algo in ("twoshot", "ring"):  # pull the own shard from n-1 peers, push the result to n-1 peers
        return nbytes * 2.0 * (n - 1) / n
    if algo == "oneshot":            # every peer reads the whole message
        return float(nbytes) * (n - 1)
    if algo == "ll":                 # 8 bytes on the wire per 4 bytes of data, to every peer
        return 2.0 * nbytes * (n - 1)
    return nbytes * 2.0 * (n - 1) / n


def measured_peaks():
    """The machine's measured copy bandwidth (GB/s) if the file is there, else an earlier measurement."""
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


def torch_dtype(name):
    import torch
    return {"float": torch.float32, "fp16": torch.float16, "bf16": torch.bfloat16}[name]


# ---------------------------------------------------------------------------------------------
# our arm and the NCCL comparator share the timing harness

class Runner:
    def __init__(self, args):
        import torch
        self.torch = torch
        self.args = args
        self.rank, self.world, self.local = dist_env()
        if self.world != args.gpus:
            if self.world == 1 and args.gpus > 1:
                raise SystemExit("--gpus N > 1 needs one process per GPU: launch with torch.distributed.run")
        torch.cuda.set_device(self.local)
        self.dev = torch.device("cuda", self.local)
        self.is_nccl = args.impl.startswith("nccl")
        if args.impl == "nccl-ring":
            os.environ.update({"NCCL_ALGO": "Ring", "NCCL_PROTO": "Simple", "NCCL_MIN_NCHANNELS": "4",
                               "NCCL_MAX_NCHANNELS": "4", "NCCL_BUFFSIZE": "33554432"})
        self.dist = init_dist("nccl")
        self.comm = None
        if not self.is_nccl:
            import nano_nccl_b200 as nn
            port = [free_port() if self.rank == 0 else 0]
            if self.world > 1:
                self.dist.broadcast_object_list(port, src=0)
            self.comm = nn.Communicator(devices=[self.local], rank=self.rank, world_size=self.world,
                                        addr=os.environ.get("MASTER_ADDR", "127.0.0.1"), port=port[0], algo=args.algo)
        self.launches = 0

    def barrier(self):
        if self.world > 1:
            self.dist.barrier()
        self.torch.cuda.synchronize()

    def max_over_ranks(self, value):
        if self.world == 1:
            return value
        t = self.torch.tensor([value], dtype=self.torch.float64, device=self.dev)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return float(t.item())

    def alloc(self, numel, dtype):
        if self.comm is not None and self.args.buffers == "symmetric":
            return self.comm.empty(numel, dtype)
        t = self.torch.empty(numel, dtype=dtype, device=self.dev)
        if self.comm is not None and self.args.buffers == "registered":
            self.comm.register(t)
        return t

    def all_reduce(self, out, inp, op):
        if self.is_nccl:
            # NCCL through torch is in-place; reduce `inp` into itself (same traffic as out-of-place).
            ops = {"sum": self.dist.ReduceOp.SUM, "avg": self.dist.ReduceOp.AVG, "max": self.dist.ReduceOp.MAX,
                   "min": self.dist.ReduceOp.MIN}
            if self.world > 1:
                self.dist.all_reduce(inp, op=ops[op])
        else:
            self.comm.all_reduce(out, inp, op=op)
        self.launches += 1

    def make_sets(self, nbytes, dtype):
        esize = self.torch.empty((), dtype=dtype).element_size()
        numel = max(nbytes // esize, 1)
        per_set = 2 * numel * esize
        nsets = int(min(8, max(1, -(-4 * L2_BYTES // per_set))))
        sets = []
        for s in range(nsets):
            inp = self.alloc(numel, dtype)
            out = self.alloc(numel, dtype)
            gen = self.torch.Generator(device=self.dev).manual_seed(1000 * self.rank + s)
            inp.copy_((self.torch.rand(numel, device=self.dev, generator=gen) * 2 - 1).to(dtype))
            sets.append((inp, out))
        return sets, numel, nsets * per_set

    def time_steps(self, sets, op, warmup, steps, repeats=1):
        """W warm-up steps, then `repeats` batches of exactly `steps` steps. Returns the per-batch
        seconds (each the maximum over ranks), in the order measured."""
        torch = self.torch
        for i in range(warmup):
            inp, out = sets[i % len(sets)]
            self.all_reduce(out, inp, op)
        batches = []
        for _ in range(repeats):
            self.barrier()
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            self.launches = 0
            start.record()
            for i in range(steps):
                inp, out = sets[i % len(sets)]
                self.all_reduce(out, inp, op)
            stop.record()
            self.barrier()
            if self.comm is not None:
                self.comm.check_async_error()
            batches.append(self.max_over_ranks(start.elapsed_time(stop) / 1e3))
        return batches

    def release(self, sets):
        """Gives symmetric / registered buffers back (a collective call, like their allocation)."""
        if self.comm is None:
            return
        for inp, out in sets:
            if self.args.buffers == "symmetric":
                self.comm.free(inp)
                self.comm.free(out)
            elif self.args.buffers == "registered":
                self.comm.unregister(inp)
                self.comm.unregister(out)

    def verify(self, sets, numel, dtype, op):
        """Recomputes the expected result of set 0 from every rank's seeded input (fp32) and counts mismatches."""
        torch = self.torch
        if self.is_nccl:
            return None
        inp, out = sets[0]
        self.all_reduce(out, inp, op)
        torch.cuda.synchronize()
        acc = None
        for r in range(self.world):
            gen = torch.Generator(device=self.dev).manual_seed(1000 * r)
            x = (torch.rand(numel, device=self.dev, generator=gen) * 2 - 1).to(dtype).float()
            if acc is None:
                acc = x
            elif op in ("sum", "avg"):
                acc += x
            elif op == "max":
                acc = torch.maximum(acc, x)
            else:
                acc = torch.minimum(acc, x)
        if op == "avg":
            acc /= self.world
        eps = {"float": 1e-5, "fp16": 1e-2, "bf16": 1e-1}[self.args.dtype]
        wrong = int(((out.float() - acc).abs() > eps).sum().item())
        return int(self.max_over_ranks(float(wrong)))

    def time_e2e(self, sets, numel, dtype, op, warmup, steps):
        """Same metric end to end: every step copies its input from pinned host memory, runs the
        collective through the public API and reads a slice of the result back to the host."""
        torch = self.torch
        host_in = [torch.empty(numel, dtype=dtype).pin_memory() for _ in sets]
        for h, (inp, _) in zip(host_in, sets):
            h.copy_(inp)
        res_elems = min(numel, 1024)
        host_out = torch.empty(res_elems, dtype=dtype).pin_memory()
        h2d = numel * host_in[0].element_size()
        d2h = res_elems * host_out.element_size()

        def step(i):
            inp, out = sets[i % len(sets)]
            inp.copy_(host_in[i % len(sets)], non_blocking=True)
            self.all_reduce(out, inp, op)
            src = inp if self.is_nccl else out
            host_out.copy_(src[:res_elems], non_blocking=True)

        for i in range(warmup):
            step(i)
        self.barrier()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for i in range(steps):
            step(i)
        stop.record()
        self.barrier()
        return self.max_over_ranks(start.elapsed_time(stop) / 1e3), h2d, d2h


def median(values):
    v = sorted(values)
    return v[len(v) // 2] if len(v) % 2 else 0.5 * (v[len(v) // 2 - 1] + v[len(v) // 2])


def run_measured(args):
    import torch
    r = Runner(args)
    dtype = torch_dtype(args.dtype)
    sets, numel, working = r.make_sets(args.bytes, dtype)
    nbytes = numel * sets[0][0].element_size()
    wrong = r.verify(sets, numel, dtype, args.op)
    sampler = ClockSampler(r.local)
    if r.rank == 0:
        sampler.start()
        time.sleep(0.05)  # let the sampler come up before the timed region
    t_begin = time.time()
    batches = r.time_steps(sets, args.op, max(args.warmup, 3), args.steps, max(args.repeats, 1))
    t_end = time.time()
    seconds = median(batches)
    launches = r.launches
    clocks = sampler.stop((t_begin, t_end)) if r.rank == 0 else None
    e2e_steps = args.steps
    e2e_seconds, h2d, d2h = r.time_e2e(sets, numel, dtype, args.op, max(args.warmup, 3), e2e_steps)
    info = r.comm.last_call() if r.comm is not None else {"algo": args.impl}
    r.release(sets)
    del sets
    torch.cuda.empty_cache()

    sweep = None
    if args.sweep != "none":
        sweep = []
        if args.sweep == "short":
            sizes = [s for s in (1 << 10, 64 << 10, 1 << 20, 16 << 20, 64 << 20, 1 << 30) if s <= args.sweep_max]
        else:
            sizes = [1 << k for k in range(10, 31) if (1 << k) <= args.sweep_max]
        for size in sizes:
            s_sets, s_numel, _ = r.make_sets(size, dtype)
            iters = 100 if size <= (1 << 20) else (20 if size <= (64 << 20) else 5)
            t = median(r.time_steps(s_sets, args.op, 5, iters, 3)) / iters
            b = s_numel * s_sets[0][0].element_size()
            algo = r.comm.last_call()["algo"] if r.comm is not None else args.impl
            row = {"bytes": b, "time_us": round(t * 1e6, 2), "busbw_gbs": round(busbw(b, t, r.world), 2), "algo": algo}
            if r.world > 1 and r.comm is not None:
                row["link_fraction_of_900"] = round(link_bytes_per_direction(algo, b, r.world) / t / 900e9, 3)
            sweep.append(row)
            r.release(s_sets)
            del s_sets
            torch.cuda.empty_cache()

    if r.rank == 0:
        per_step = seconds / args.steps
        value = busbw(nbytes, per_step, r.world)
        e2e_value = busbw(nbytes, e2e_seconds / e2e_steps, r.world)
        algo = info.get("algo")
        hbm_peak, peak_kind = measured_peaks()
        line = {
            "metric": "allreduce_busbw_gbs_64MiB_float_sum",
            "value": round(value, 2),
            "unit": "GB/s",
            "impl": args.impl,
            "n_gpus": r.world,
            "steps": args.steps,
            "warmup": max(args.warmup, 3),
            "ms_per_step": round(per_step * 1e3, 5),
            "repeats": len(batches),
            "ms_per_step_min": round(min(batches) / args.steps * 1e3, 5),
            "ms_per_step_max": round(max(batches) / args.steps * 1e3, 5),
            "higher_is_better": True,
            "scaling": "weak",
            "vs_baseline": round(value / BASELINE_BUSBW, 2),
            "dtype": args.dtype,
            "data": "synthetic: uniform[-1,1) seeded per rank, device-generated",
            "wrong": wrong,
            "aggregate_gbs": round(value * r.world, 2),
            "config": {
                "model": "AllReduce (collective library; no neural model)",
                "collective": "all_reduce", "redop": args.op, "bytes_per_rank": nbytes, "global_batch": nbytes * r.world,
                "seq_len": numel, "parallelism": f"allreduce{r.world}",
                "buffers": args.buffers if r.comm is not None else "torch.empty (NCCL in place)",
                "algo": algo, "grid": info.get("grid"),
                "process_model": "one process per GPU (torchrun), peer memory shared as exported allocations",
                "l2": f"rotating over {len(sets_desc(nbytes))} buffer sets, {working >> 20} MiB working set > 126 MB L2",
                "busbw_formula": "bytes/time * 2(n-1)/n for n > 1; one GPU has no bus, so at n = 1 the value is bytes/time of "
                                 "the device-to-device copy the collective degenerates to (see hbm_fraction)",
                "timing": f"CUDA events around each batch of K back-to-back steps, max over ranks; median of {len(batches)} batches",
            },
            "clocks": clocks,
            "e2e": {"value": round(e2e_value, 2), "unit": "GB/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "steps": e2e_steps, "ms_per_step": round(e2e_seconds / e2e_steps * 1e3, 5),
                    "note": "each step: pinned-host -> device copy of the whole input, all_reduce via Communicator.all_reduce, device -> pinned-host read of the first 1024 result elements"},
            "gpu_launches": launches if r.comm is not None else 0,
        }
        if r.world > 1:
            per_dir = link_bytes_per_direction(algo, nbytes, r.world)
            line["link_fraction_of_900"] = round(per_dir / per_step / 900e9, 3)
            line["link_model"] = f"{algo}: {per_dir / nbytes:.3f} x message bytes leave and enter every GPU per step"
        else:
            line["hbm_fraction"] = round(2 * nbytes / per_step / 1e9 / hbm_peak, 3)
            line["hbm_peak"] = f"{hbm_peak:.0f} GB/s copy bandwidth ({peak_kind}); the copy reads and writes the message once each"
        if sweep is not None:
            line["sweep"] = sweep
        print(json.dumps(line), flush=True)
    if r.comm is not None:
        r.comm.close()
    if r.world > 1:
        r.dist.barrier()
        r.dist.destroy_process_group()


def sets_desc(nbytes):
    per_set = 2 * nbytes
    return range(int(min(8, max(1, -(-4 * L2_BYTES // per_set)))))


# ---------------------------------------------------------------------------------------------
# reference arm: the unmodified nano-nccl benchmark binary, built by baseline/build_reference.sh

def run_reference(args):
    rank, world, _ = dist_env()
    n = args.gpus
    result = None
    if rank == 0:
        binary = os.path.join(ROOT, "baseline", "_ref", "bin", f"nano_nccl_all_reduce_bench_n{n}")
        if n < 2:
            result = {"impl": "reference", "unavailable": "the reference fixes its rank count at build time and is not built or documented for 1 rank"}
        elif not os.path.exists(binary):
            result = {"impl": "reference", "unavailable": f"{os.path.relpath(binary, ROOT)} missing: run baseline/build_reference.sh"}
        else:
            result = reference_measure(binary, args, n)
    if world > 1:
        dist = init_dist("gloo")
        dist.barrier()
        dist.destroy_process_group()
    if rank == 0:
        print(json.dumps(result), flush=True)


def reference_measure(binary, args, n):
    """Runs (1) the harness baseline/ref_e2e_driver.cu built against the unmodified reference library:
    K all_reduce calls through its public API timed with CUDA events (max over ranks), then the same
    K steps end to end with the host-to-device input copy and a 4 KiB read-back; (2) the reference's
    stock benchmark binary, whose own host-clock row is kept under "stock_benchmark"."""
    warm = max(args.warmup, 3)
    sampler = ClockSampler(0)
    sampler.start()
    t0 = time.time()
    harness = os.path.join(os.path.dirname(binary), f"ref_e2e_n{n}")
    e2e_row = None
    harness_note = None
    if args.dtype == "float" and args.op == "sum" and os.path.exists(harness):
        try:
            proc = subprocess.run([harness, str(args.bytes), str(args.steps), str(warm), args.ref_transport],
                                  capture_output=True, text=True, timeout=600)
            for line in proc.stdout.splitlines():
                if line.startswith("REF_E2E"):
                    parts = line.split()
                    e2e_row = {parts[k]: parts[k + 1] for k in range(1, len(parts) - 1, 2)}
            if e2e_row is None:
                harness_note = f"harness exit {proc.returncode}: {(proc.stderr or proc.stdout).strip()[-200:]}"
        except subprocess.TimeoutExpired:
            harness_note = "harness did not finish within 600 s"
    t1 = time.time()
    cmd = [binary, "--dtype", args.dtype, "--redop", args.op, "--transport", args.ref_transport,
           "-b", str(args.bytes), "-e", str(args.bytes), "-f", "2", "-w", str(warm), "-n", str(args.steps)]
    stock = None
    try:
        proc = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
        for line in proc.stdout.splitlines():
            parts = line.split()
            if not line.startswith("#") and len(parts) >= 11 and parts[4].isdigit():
                stock = {"transport": parts[3], "bytes": int(parts[4]), "time_us": float(parts[6]), "algbw_gbs": float(parts[7]),
                         "busbw_gbs": float(parts[8]), "wrong_ranks": int(parts[9]), "timing": "host steady_clock (its stock method)"}
        if stock is None:
            stock = {"error": f"exit {proc.returncode}: {(proc.stderr or proc.stdout).strip()[-200:]}"}
    except subprocess.TimeoutExpired:
        stock = {"error": "did not finish within 600 s"}
    clocks = sampler.stop((t0, t1))
    # The reference's published range, 256 KiB .. 64 MiB x4, through its stock benchmark (host clock).
    sweep = None
    if args.sweep != "none":
        try:
            proc = subprocess.run([binary, "--dtype", args.dtype, "--redop", args.op, "--transport", args.ref_transport,
                                   "-b", "262144", "-e", "67108864", "-f", "4", "-w", "5", "-n", "20"],
                                  capture_output=True, text=True, timeout=600)
            sweep = []
            for line in proc.stdout.splitlines():
                parts = line.split()
                if not line.startswith("#") and len(parts) >= 11 and parts[4].isdigit():
                    sweep.append({"bytes": int(parts[4]), "time_us": float(parts[6]), "busbw_gbs": float(parts[8]),
                                  "algo": "ring_simple", "timing": "host clock (stock benchmark)"})
        except subprocess.TimeoutExpired:
            sweep = None
    if e2e_row is None and (stock is None or "error" in stock):
        return {"impl": "reference", "unavailable": f"reference gave no result: {harness_note}; stock: {stock}"[:300]}
    if e2e_row is not None:
        per_step = float(e2e_row["kernel_ms_per_step"]) / 1e3
        e2e_step = float(e2e_row["e2e_ms_per_step"]) / 1e3
        value = busbw(args.bytes, per_step, n)
        e2e = {"value": round(busbw(args.bytes, e2e_step, n), 2), "unit": "GB/s", "h2d_bytes_per_step": int(e2e_row["h2d_bytes"]),
               "d2h_bytes_per_step": int(e2e_row["d2h_bytes"]), "steps": args.steps, "ms_per_step": round(e2e_step * 1e3, 5),
               "note": "per step and rank: pinned-host -> device copy of the whole input, Communicator::all_reduce, 4 KiB read-back"}
        wrong, transport = int(e2e_row["wrong"]), e2e_row["transport"]
        timing = "CUDA events on every rank's stream around K back-to-back calls, max over ranks (harness over the reference's public API)"
    else:
        per_step = stock["time_us"] / 1e6
        value, e2e, wrong, transport = stock["busbw_gbs"], None, stock["wrong_ranks"], stock["transport"]
        timing = stock["timing"]
    return {
        "metric": "allreduce_busbw_gbs_64MiB_float_sum", "value": round(value, 2), "unit": "GB/s", "impl": "reference",
        "n_gpus": n, "steps": args.steps, "warmup": warm, "ms_per_step": round(per_step * 1e3, 5),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": round(value / BASELINE_BUSBW, 2), "dtype": args.dtype,
        "data": "synthetic: fixed arithmetic pattern per rank", "wrong": wrong,
        "config": {"model": "AllReduce (collective library; no neural model)", "collective": "all_reduce", "redop": args.op,
                   "bytes_per_rank": args.bytes, "global_batch": args.bytes * n, "seq_len": args.bytes // 4,
                   "parallelism": f"allreduce{n}", "transport": transport, "requested_transport": args.ref_transport,
                   "build": f"unmodified reference, -DNANO_NCCL_NRANKS={n} -DNANO_NCCL_CUDA_ARCH=100, one process driving {n} GPUs",
                   "process_model": f"one process, one host thread driving {n} GPUs (the reference's only single-host model)",
                   "timing": timing, "l2": "single buffer pair of 2 x 64 MiB per GPU (the reference's FIFO traffic adds to it)"},
        "clocks": clocks, "e2e": e2e, "gpu_launches": args.steps * n, "stock_benchmark": stock, "harness_note": harness_note,
        "sweep": sweep,
    }


def main():
    args = parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_measured(args)


if __name__ == "__main__":
    main()
