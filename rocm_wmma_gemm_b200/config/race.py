#!/usr/bin/env python
"""Head-to-head re-timing of two tuned JSON tables, and a row-C vs column-C cross-check.

Counterpart of the reference's rocm_wmma_gemm/config/race.py:65-267.  For every (size, layout)
both tables hold, the two configurations are timed in alternating order for several rounds and
compared by median; the table that wins more entries is reported, and `--merge` writes the
per-entry winners.  `--cross` additionally tries, for each column-major-C entry, the
configuration tuned for the same A/B layouts with row-major C (and vice versa): a faster
result means the tuner was caught in a local optimum for that entry.
"""
from __future__ import annotations

import argparse
import os
import statistics
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from rocm_wmma_gemm_b200.config import tune  # noqa: E402


def race_pair(evaluate, shape, layout, a, b, rounds=5):
    ta, tb = [], []
    for r in range(rounds):
        order = [(a, ta), (b, tb)] if r % 2 == 0 else [(b, tb), (a, ta)]
        for cfg, sink in order:
            sink.append(evaluate(*shape, *layout, cfg))
    wins_a = sum(1 for x, y in zip(ta, tb) if x < y)
    return statistics.median(ta), statistics.median(tb), wins_a, rounds - wins_a


def main(argv=None):
    p = argparse.ArgumentParser()
    p.add_argument("table_a")
    p.add_argument("table_b", nargs="?")
    p.add_argument("--type", default="bf16_bf16", choices=list(tune.TYPE_INDEX))
    p.add_argument("--rounds", type=int, default=5)
    p.add_argument("--merge", help="write the per-entry winners to this JSON")
    p.add_argument("--cross", action="store_true", help="row-C vs column-C cross-check within table_a")
    a = p.parse_args(argv)

    ta = tune.load_table(a.table_a)
    evaluate = tune.InProcessEvaluator(a.type)
    merged = {s: dict(v) for s, v in ta.items()}

    if a.table_b:
        tb = tune.load_table(a.table_b)
        score = [0, 0]
        for shape in sorted(set(ta) & set(tb)):
            for layout in sorted(set(ta[shape]) & set(tb[shape])):
                ca, cb = tune.from_dict(ta[shape][layout]["config"]), tune.from_dict(tb[shape][layout]["config"])
                if ca == cb:
                    continue
                ma, mb, wa, wb = race_pair(evaluate, shape, layout, ca, cb, a.rounds)
                win = 0 if ma <= mb else 1
                score[win] += 1
                if win == 1:
                    merged[shape][layout] = tb[shape][layout]
                print(f"{shape} {layout}: A {ma:.4f} ms ({wa} wins)  B {mb:.4f} ms ({wb} wins)  -> {'AB'[win]}")
        print(f"entries won: A {score[0]}  B {score[1]}")

    if a.cross:
        for shape in sorted(ta):
            for layout in sorted(ta[shape]):
                other = (layout[0], layout[1], 1 - layout[2])
                if other not in ta[shape]:
                    continue
                mine, theirs = tune.from_dict(ta[shape][layout]["config"]), tune.from_dict(ta[shape][other]["config"])
                if mine == theirs or not tune.check_constraints(theirs, *shape, layout[2]):
                    continue
                m1, m2, _, _ = race_pair(evaluate, shape, layout, mine, theirs, a.rounds)
                if m2 < m1 * 0.98:
                    entry = dict(ta[shape][layout])
                    entry["config"] = tune.to_dict(theirs)
                    entry["time_ms"] = round(m2, 5)
                    merged[shape][layout] = entry
                    print(f"{shape} {layout}: config of C-{'rc'[other[2]]} is faster: {m2:.4f} vs {m1:.4f} ms")

    if a.merge:
        tune.save_table(a.merge, merged)
        print("wrote", a.merge)
    return 0


if __name__ == "__main__":
    sys.exit(main())
