#!/usr/bin/env python
"""A/B runs of the RDMA transport's modes on one machine: data plane (SEND/RECV vs RDMA WRITE with
clear-to-send grants), progress (one thread per proxy vs one shared engine), FIFO placement (pinned
host memory vs device memory registered with the HCA) and, in a timeline build, the proxy timeline
dump. Every mode runs `--runs` times through build/bin/b200ccl_collective_bench --transport rdma; the
per-size best / median / worst bus bandwidth go to a CSV and a markdown summary.

    python bench/rdma_modes_ab.py --out-dir rdma_ab --runs 3 --nranks 4 [--loopback] [--timeline] [--dry-run]

In one process every ring edge is looped through the proxies (B200CCL_RDMA_BACKEND=fake needs no HCA;
`ibverbs` uses the first active port, or the one of B200CCL_RDMA_IFNAME). It covers, on one host, what
the reference's scripts/ab_rdma_progress.sh, compare_rdma_no_gdr.sh and capture_rdma_proxy_timeline.sh do
between two hosts; host names and interfaces come from the environment only, as there.
"""
import argparse
import csv
import os
import statistics
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

MODES = {
    "send-dedicated": {"B200CCL_RDMA_USE_WRITE": "0", "B200CCL_RDMA_SHARED_PROGRESS": "0", "B200CCL_RDMA_GDR": "0"},
    "send-shared": {"B200CCL_RDMA_USE_WRITE": "0", "B200CCL_RDMA_SHARED_PROGRESS": "1", "B200CCL_RDMA_GDR": "0"},
    "write-dedicated": {"B200CCL_RDMA_USE_WRITE": "1", "B200CCL_RDMA_SHARED_PROGRESS": "0", "B200CCL_RDMA_GDR": "0"},
    "write-shared": {"B200CCL_RDMA_USE_WRITE": "1", "B200CCL_RDMA_SHARED_PROGRESS": "1", "B200CCL_RDMA_GDR": "0"},
    "send-dedicated-gdr": {"B200CCL_RDMA_USE_WRITE": "0", "B200CCL_RDMA_SHARED_PROGRESS": "0", "B200CCL_RDMA_GDR": "1"},
}


def parse_table(text):
    """Rows of the benchmark's table: (bytes, time_us, busbw, wrong)."""
    rows = []
    for line in text.splitlines():
        parts = line.split()
        if len(parts) == 11 and not line.startswith("#"):
            try:
                rows.append((int(parts[4]), float(parts[6]), float(parts[8]), int(parts[9])))
            except ValueError:
                pass
    return rows


def command(args):
    cmd = [args.bin, "--collective", "all_reduce", "--transport", "rdma", "--dtype", args.dtype, "--redop", "sum",
           "-b", args.min_bytes, "-e", args.max_bytes, "-f", str(args.factor), "-w", str(args.warmup), "-n", str(args.iters)]
    if args.nranks:
        cmd += ["--nranks", str(args.nranks)]
    if args.loopback:
        cmd.append("--loopback")
    return cmd


def summarise(samples):
    """samples: {mode: {bytes: [busbw, ...]}} -> list of CSV rows."""
    out = []
    for mode, by_size in samples.items():
        for size in sorted(by_size):
            v = by_size[size]
            out.append({"mode": mode, "bytes": size, "runs": len(v), "best_gbs": max(v), "median_gbs": statistics.median(v),
                        "worst_gbs": min(v)})
    return out


def markdown(rows):
    modes = sorted({r["mode"] for r in rows})
    sizes = sorted({r["bytes"] for r in rows})
    cell = {(r["mode"], r["bytes"]): r for r in rows}
    lines = ["| size (B) | " + " | ".join(f"{m} median (best) GB/s" for m in modes) + " |",
             "|---:|" + "|".join(["---:"] * len(modes)) + "|"]
    for s in sizes:
        cols = []
        for m in modes:
            r = cell.get((m, s))
            cols.append(f"{r['median_gbs']:.2f} ({r['best_gbs']:.2f})" if r else "–")
        lines.append(f"| {s} | " + " | ".join(cols) + " |")
    return "\n".join(lines) + "\n"


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--bin", default=os.path.join(ROOT, "build", "bin", "b200ccl_collective_bench"))
    ap.add_argument("--out-dir", required=True)
    ap.add_argument("--runs", type=int, default=3)
    ap.add_argument("--modes", default="send-dedicated,send-shared,write-dedicated,write-shared",
                    help="comma list of " + ", ".join(MODES))
    ap.add_argument("--nranks", type=int, default=0)
    ap.add_argument("--loopback", action="store_true", help="emulate the ranks on one GPU")
    ap.add_argument("--dtype", default="float")
    ap.add_argument("--min-bytes", default="1M")
    ap.add_argument("--max-bytes", default="64M")
    ap.add_argument("--factor", type=int, default=4)
    ap.add_argument("--warmup", type=int, default=2)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--timeline", action="store_true",
                    help="set B200CCL_RDMA_PROXY_TIMELINE=1 and keep each run's stderr (needs a B200CCL_ENABLE_TIMELINE build)")
    ap.add_argument("--dry-run", action="store_true", help="print the commands and environments, run nothing")
    args = ap.parse_args(argv)
    modes = [m for m in args.modes.split(",") if m]
    for m in modes:
        if m not in MODES:
            ap.error(f"unknown mode '{m}'")
    os.makedirs(args.out_dir, exist_ok=True)
    samples, failures = {}, 0
    for mode in modes:
        env = dict(os.environ)
        env.update(MODES[mode])
        if args.timeline:
            env["B200CCL_RDMA_PROXY_TIMELINE"] = "1"
        for run in range(args.runs):
            cmd = command(args)
            if args.dry_run:
                print(" ".join(f"{k}={v}" for k, v in sorted(MODES[mode].items())), " ".join(cmd))
                continue
            proc = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=1800)
            with open(os.path.join(args.out_dir, f"{mode}_run{run}.log"), "w") as f:
                f.write(proc.stdout)
            if args.timeline or proc.returncode != 0:
                with open(os.path.join(args.out_dir, f"{mode}_run{run}.stderr"), "w") as f:
                    f.write(proc.stderr)
            rows = parse_table(proc.stdout)
            if proc.returncode != 0 or not rows or any(r[3] != 0 for r in rows):
                failures += 1
                print(f"{mode} run {run}: exit {proc.returncode}, {len(rows)} rows, wrong={[r[3] for r in rows]}", file=sys.stderr)
                continue
            for size, _, busbw, _ in rows:
                samples.setdefault(mode, {}).setdefault(size, []).append(busbw)
    if args.dry_run:
        return 0
    rows = summarise(samples)
    with open(os.path.join(args.out_dir, "summary.csv"), "w", newline="") as f:
        w = csv.DictWriter(f, fieldnames=["mode", "bytes", "runs", "best_gbs", "median_gbs", "worst_gbs"])
        w.writeheader()
        w.writerows(rows)
    with open(os.path.join(args.out_dir, "summary.md"), "w") as f:
        f.write(markdown(rows))
    sys.stdout.write(markdown(rows))
    return 1 if failures else 0


if __name__ == "__main__":
    sys.exit(main())
