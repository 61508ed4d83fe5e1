"""The arithmetic of the balanced (stream-K) schedule, restated in Python and checked by
exhaustion on small cases: the runs of `WorkCursor` (csrc/gemm_kernels.cuh) cover every K step
of every tile exactly once, the workspace slot tile + worker is unique per segment, and the
fix-up pass's closed form for "which workers touch tile t" names exactly the segments written."""
import itertools

import pytest


def run_start(worker, total, workers):
    return worker * total // workers


def segments(worker, tiles, upt, workers):
    """(tile, first K step, last K step (exclusive), slot) of each segment of one worker's run."""
    total = tiles * upt
    nxt, end = run_start(worker, total, workers), run_start(worker + 1, total, workers)
    out = []
    while nxt < end:
        tile = nxt // upt
        first = nxt - tile * upt
        last = min(upt, first + (end - nxt))
        out.append((tile, first, last, tile + worker))
        nxt += last - first
    return out


def fixup_workers(tile, upt, total, workers):
    x0, x1 = tile * upt, tile * upt + upt - 1
    w0 = ((x0 + 1) * workers + total - 1) // total - 1
    w1 = ((x1 + 1) * workers + total - 1) // total - 1
    return w0, w1


@pytest.mark.parametrize("tiles,upt,sms", list(itertools.product([1, 2, 3, 7, 32, 64, 150, 513], [1, 2, 5, 16, 33, 128], [1, 3, 74, 148])))
def test_runs_cover_every_step_once_and_fixup_finds_them(tiles, upt, sms):
    total = tiles * upt
    workers = min(total, sms)
    seen = {}
    slots = {}
    per_tile = {}
    for w in range(workers):
        steps = 0
        for (tile, first, last, slot) in segments(w, tiles, upt, workers):
            assert 0 <= first < last <= upt
            assert slot not in slots, "two segments share a workspace slot"
            slots[slot] = (tile, w)
            per_tile.setdefault(tile, []).append(w)
            for k in range(first, last):
                assert (tile, k) not in seen
                seen[(tile, k)] = w
            steps += last - first
        assert steps in (total // workers, total // workers + 1), "runs differ by more than one step"
    assert len(seen) == total
    assert max(slots) <= tiles + workers - 2
    for tile in range(tiles):
        w0, w1 = fixup_workers(tile, upt, total, workers)
        assert per_tile[tile] == list(range(w0, w1 + 1)), "the fix-up pass would add the wrong partial tiles"
        # partials are added in ascending worker order = ascending K
        firsts = [min(k for (t, k), w in seen.items() if t == tile and w == ww) for ww in range(w0, w1 + 1)]
        assert firsts == sorted(firsts)
