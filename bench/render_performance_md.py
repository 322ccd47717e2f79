#!/usr/bin/env python
"""Renders benchmark results as markdown tables (no GPU needed).

Inputs, any mix, each optionally as LABEL=path:
  * the --json file of build/bin/b200ccl_collective_bench (a list of rows),
  * a tuner table (nano_nccl_b200.tuner --out; the per-size winners are used),
  * a file holding the JSON line(s) printed by bench.py (the 'sweep' list if present, else the headline).

With one input: one table (size, time, algorithm bandwidth, bus bandwidth, #wrong when known).
With several: one column of bus bandwidth per label and the ratio of the first label to each other.

    python bench/render_performance_md.py ours=ours.json nccl=nccl.json --title "AllReduce, 8 GPUs" > performance.md

Stands where the reference has scripts/render_performance_md.py (markdown from its matrix runs).
"""
import argparse
import json
import sys


def human(nbytes):
    for unit, shift in (("GiB", 30), ("MiB", 20), ("KiB", 10)):
        if nbytes >= (1 << shift) and nbytes % (1 << shift) == 0:
            return f"{nbytes >> shift} {unit}"
    return f"{nbytes} B"


def rows_of(doc):
    """Normalises one parsed input to a list of dicts with bytes, time_us, busbw_gbs (+ optional keys)."""
    if isinstance(doc, dict) and "best" in doc and "rows" in doc:  # tuner table
        return [dict(r) for r in doc["best"]]
    if isinstance(doc, dict) and "metric" in doc:  # bench.py line
        if doc.get("sweep"):
            return [dict(r) for r in doc["sweep"]]
        cfg = doc.get("config", {})
        return [{"bytes": cfg.get("bytes", cfg.get("message_bytes", 0)), "time_us": doc.get("ms_per_step", 0) * 1e3,
                 "busbw_gbs": doc.get("value", 0), "algo": cfg.get("algo", doc.get("impl", ""))}]
    if isinstance(doc, list):
        return [dict(r) for r in doc]
    raise ValueError("unrecognised result file")


def load(path):
    text = open(path).read().strip()
    try:
        return rows_of(json.loads(text))
    except json.JSONDecodeError:
        rows = []
        for line in text.splitlines():  # a log with one JSON object per line
            line = line.strip()
            if line.startswith("{") and line.endswith("}"):
                rows.extend(rows_of(json.loads(line)))
        if not rows:
            raise
        return rows


def single_table(rows):
    has_wrong = any("wrong" in r for r in rows)
    has_algbw = any("algbw_gbs" in r for r in rows)
    head = ["size", "algo", "time (us)"] + (["algbw (GB/s)"] if has_algbw else []) + ["busbw (GB/s)"] + (["#wrong"] if has_wrong else [])
    out = ["| " + " | ".join(head) + " |", "|" + "|".join(["---:"] * len(head)) + "|"]
    for r in sorted(rows, key=lambda r: r["bytes"]):
        cells = [human(r["bytes"]), str(r.get("algo", "")), f"{r['time_us']:.2f}"]
        if has_algbw:
            cells.append(f"{r.get('algbw_gbs', 0):.2f}")
        cells.append(f"{r['busbw_gbs']:.2f}")
        if has_wrong:
            cells.append(str(r.get("wrong", "")))
        out.append("| " + " | ".join(cells) + " |")
    return out


def comparison_table(named):
    labels = [n for n, _ in named]
    by_size = {}
    for label, rows in named:
        for r in rows:
            by_size.setdefault(r["bytes"], {})[label] = r
    head = ["size"] + [f"{n} busbw (GB/s)" for n in labels] + [f"{labels[0]} / {n}" for n in labels[1:]]
    out = ["| " + " | ".join(head) + " |", "|" + "|".join(["---:"] * len(head)) + "|"]
    for size in sorted(by_size):
        got = by_size[size]
        cells = [human(size)] + [f"{got[n]['busbw_gbs']:.2f}" if n in got else "–" for n in labels]
        for n in labels[1:]:
            if labels[0] in got and n in got and got[n]["busbw_gbs"] > 0:
                cells.append(f"{got[labels[0]]['busbw_gbs'] / got[n]['busbw_gbs']:.2f}")
            else:
                cells.append("–")
        out.append("| " + " | ".join(cells) + " |")
    return out


def render(inputs, title=""):
    named = []
    for i, spec in enumerate(inputs):
        label, _, path = spec.rpartition("=")
        named.append((label or f"run{i + 1}", load(path)))
    lines = [f"## {title}", ""] if title else []
    lines += single_table(named[0][1]) if len(named) == 1 else comparison_table(named)
    return "\n".join(lines) + "\n"


def main():
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("inputs", nargs="+", help="[LABEL=]path of a result file")
    ap.add_argument("--title", default="")
    args = ap.parse_args()
    sys.stdout.write(render(args.inputs, args.title))


if __name__ == "__main__":
    main()
