#!/usr/bin/env python
"""Turns the JSON-lines records of `bench_shapes --json` into a markdown report.

Counterpart of the reference's docs/generate_report.py (which parses Google-Benchmark console
output and writes docs/gfx11xx_{square,rectangle}.md): one row per (matrix size, input layout
A,B), one column per output layout C, in TFLOP/s, plus the fraction of the chip's dense
half-precision tensor peak — the place the vendor-library column takes in the reference's
tables, since no vendor library is part of this library.  The reference's PNG plots are not
reproduced (no plotting package is assumed); `--json-out` writes the pivoted numbers instead.

    python -m rocm_wmma_gemm_b200.bench_shapes --preset squares --json squares.jsonl
    python -m rocm_wmma_gemm_b200.generate_report squares.jsonl -o sm100_square.md --title "Square FP16 GEMM"
"""
from __future__ import annotations

import argparse
import json
import sys
from collections import OrderedDict

LAYOUT_WORD = {0: "row", 1: "col"}
INPUT_ORDER = [(1, 1), (0, 1), (1, 0), (0, 0)]  # (A, B): the order of the reference's tables
NOMINAL_TFLOPS = 2250.0


def load_records(paths):
    records = []
    for path in paths:
        with open(path) as f:
            for line in f:
                line = line.strip()
                if line:
                    records.append(json.loads(line))
    return records


def pivot(records, metric="tflops_median"):
    """{(type, M, N, K): {(la, lb): {lc: value}}} keeping first-seen size order; a repeated
    (size, layout) keeps the best value."""
    table = OrderedDict()
    for r in records:
        key = (r["type"], r["M"], r["N"], r["K"])
        lay = r["layout"]
        cell = table.setdefault(key, {}).setdefault((lay["A"], lay["B"]), {})
        value = r.get(metric)
        if value is None:
            continue
        cell[lay["C"]] = max(cell.get(lay["C"], 0.0), float(value))
    return table


def render(table, title, system, metric_label, peak=NOMINAL_TFLOPS):
    lines = [f"# {title}", ""]
    lines.append(f"Performance measured on {system} in TFLOP/s ({metric_label}); "
                 f"'% peak' is the better of the two output layouts against {peak:.0f} TFLOP/s dense.")
    lines.append("")
    by_type = OrderedDict()
    for (typ, m, n, k), rows in table.items():
        by_type.setdefault(typ, []).append(((m, n, k), rows))
    for typ, sizes in by_type.items():
        out_t, in_t = typ.split("_")
        lines.append(f"## {in_t.upper()} -> {out_t.upper()} Performance Results")
        lines.append("")
        lines.append("| Matrix Size | Input Layout (A,B) | C=col | C=row | % peak |")
        lines.append("|:------------|:-------------------|------:|------:|-------:|")
        for (m, n, k), rows in sizes:
            for la, lb in INPUT_ORDER:
                if (la, lb) not in rows:
                    continue
                cell = rows[(la, lb)]
                col, row = cell.get(1), cell.get(0)
                best = max(v for v in (col, row) if v is not None)
                fmt = lambda v: f"{v:.2f}" if v is not None else "–"
                lines.append(f"| {m}x{n}x{k} | {LAYOUT_WORD[la]}, {LAYOUT_WORD[lb]} | {fmt(col)} | {fmt(row)} | "
                             f"{100.0 * best / peak:.1f} |")
        lines.append("")
    return "\n".join(lines)


def main(argv=None):
    p = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    p.add_argument("records", nargs="+", help="JSON-lines files written by bench_shapes --json")
    p.add_argument("-o", "--output", help="markdown file (default: stdout)")
    p.add_argument("--title", default="Half-precision GEMM performance")
    p.add_argument("--system", default="NVIDIA B200 (sm_100a)")
    p.add_argument("--metric", default="tflops_median",
                   choices=["tflops_median", "avg_tflops", "tflops_sustained", "tflops_graph"])
    p.add_argument("--json-out", help="also write the pivoted table as JSON")
    a = p.parse_args(argv)
    labels = {"tflops_median": "median of individually timed calls", "avg_tflops": "mean of per-call TFLOP/s",
              "tflops_sustained": "back-to-back calls", "tflops_graph": "CUDA-graph replay, device time only"}
    table = pivot(load_records(a.records), a.metric)
    text = render(table, a.title, a.system, labels[a.metric])
    if a.output:
        with open(a.output, "w") as f:
            f.write(text + "\n")
    else:
        print(text)
    if a.json_out:
        flat = [{"type": t, "M": m, "N": n, "K": k, "A": LAYOUT_WORD[la], "B": LAYOUT_WORD[lb],
                 "C_col": c.get(1), "C_row": c.get(0)}
                for (t, m, n, k), rows in table.items() for (la, lb), c in rows.items()]
        with open(a.json_out, "w") as f:
            json.dump(flat, f, indent=1)
    return 0


if __name__ == "__main__":
    sys.exit(main())
