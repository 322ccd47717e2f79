"""Turns tuner tables into a tuning file for the planner (``B200CCL_TUNING_FILE``).

    python -m nano_nccl_b200.tuning_file tuning/b200_n8_all_reduce_graph.json tuning/b200_n4_all_reduce_graph.json > b200.tuning
    B200CCL_TUNING_FILE=b200.tuning python train.py

The planner picks, per AllReduce call: the low-latency kernel up to ``ll_max_bytes``; the multimem kernel
from ``nvls_min_bytes`` up (when multicast is available); else one-shot up to ``oneshot_max_bytes.<nranks>``
and two-shot above. This module reads those crossovers off measured tables (one per GPU count) and also
the CTA cap that was fastest at large sizes. No GPU is needed.
"""
import json
import sys

LARGE = 32 << 20  # CTA caps are judged on messages of at least this size


def _fastest(rows):
    """{algo: {bytes: (time_us, max_ctas)}} keeping the fastest CTA cap of every algorithm and size."""
    table = {}
    for r in rows:
        if r.get("collective", "all_reduce") != "all_reduce":
            continue
        algo = r.get("requested") or r["algo"]
        cur = table.setdefault(algo, {}).get(r["bytes"])
        if cur is None or r["time_us"] < cur[0]:
            table[algo][r["bytes"]] = (r["time_us"], r.get("max_ctas", 0))
    return table


def _prefix_where_fastest(table, algo, others, slack=1.0):
    """Largest size S such that `algo` is at least as fast as every algorithm of `others` at every
    measured size <= S (0 when it loses at the smallest size already)."""
    limit = 0
    for size in sorted(table.get(algo, {})):
        mine = table[algo][size][0]
        rivals = [table[o][size][0] for o in others if size in table.get(o, {})]
        if rivals and mine > min(rivals) * slack:
            break
        limit = size
    return limit


def _suffix_where_fastest(table, algo, others, slack=1.0):
    """Smallest size S such that `algo` is at least as fast as every other at every measured size >= S
    (None when it loses at the largest size)."""
    start = None
    for size in sorted(table.get(algo, {}), reverse=True):
        mine = table[algo][size][0]
        rivals = [table[o][size][0] for o in others if size in table.get(o, {})]
        if rivals and mine > min(rivals) * slack:
            break
        start = size
    return start


def _best_cta_cap(rows, algo):
    total = {}
    for r in rows:
        if (r.get("requested") or r["algo"]) == algo and r["bytes"] >= LARGE and r.get("max_ctas"):
            total.setdefault(r["max_ctas"], []).append(r["time_us"])
    full = max((len(v) for v in total.values()), default=0)
    total = {c: sum(v) for c, v in total.items() if len(v) == full}  # compare caps measured on the same sizes
    return min(total, key=total.get) if total else None


def derive_tuning(tables):
    """``tables``: parsed tuner outputs (dicts with n_gpus and rows). Returns {key: value} for the file."""
    out = {}
    nvls_starts = []
    for doc in sorted(tables, key=lambda d: d["n_gpus"]):
        n, rows = doc["n_gpus"], doc["rows"]
        if n < 2:
            continue
        t = _fastest(rows)
        if "oneshot" in t:
            out[f"oneshot_max_bytes.{n}"] = _prefix_where_fastest(t, "oneshot", ["twoshot"])
        if "nvls" in t and n >= 3:
            s = _suffix_where_fastest(t, "nvls", ["oneshot", "twoshot"], slack=1.02)
            if s is not None:
                nvls_starts.append(s)
        if "ll" in t:
            out["ll_max_bytes"] = min(out.get("ll_max_bytes", 1 << 40), _prefix_where_fastest(t, "ll", ["oneshot", "twoshot", "nvls"]))
        for algo, key in (("nvls", "nvls_max_ctas"), ("twoshot", "twoshot_max_ctas")):
            cap = _best_cta_cap(rows, algo)
            if cap is not None and n == max(d["n_gpus"] for d in tables):  # caps from the largest machine measured
                out[key] = cap
    if nvls_starts:
        out["nvls_min_bytes"] = max(nvls_starts)  # one threshold for every rank count: the most cautious one
    return out


def format_tuning(values, comment=""):
    lines = ["# b200ccl tuning file (key = value; see src/sched/plan.h)"]
    if comment:
        lines.append("# " + comment)
    for key in sorted(values):
        lines.append(f"{key} = {values[key]}")
    return "\n".join(lines) + "\n"


def main(argv=None):
    argv = sys.argv[1:] if argv is None else argv
    if not argv or argv[0] in ("-h", "--help"):
        print(__doc__)
        return 0 if argv else 2
    tables = [json.load(open(p)) for p in argv]
    sys.stdout.write(format_tuning(derive_tuning(tables), "derived from " + ", ".join(argv)))
    return 0


if __name__ == "__main__":
    sys.exit(main())
