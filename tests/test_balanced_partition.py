"""The arithmetic of the balanced (stream-K) schedule, restated in Python and checked by
exhaustion on small cases.  Whole waves of tiles are dealt round-robin; the tiles of the
incomplete wave (all tiles when there are fewer than workers) are cut into runs, and for them: the runs of `WorkCursor` (csrc/gemm_kernels.cuh) cover every K step
of every tile exactly once; a run has at most two partial segments and their workspace slots
(2 * worker for a segment that starts inside a tile, 2 * worker + 1 for one that ends inside a
tile) never collide; and the fix-up pass (`streamk_reduce_kernel`) - one job per run boundary,
the first boundary inside a tile owning it - visits exactly the tiles that were cut, with
exactly the slots that were written, in K order."""
import itertools

import pytest


def run_start(worker, total, workers):
    return worker * total // workers


def segments(worker, tiles, upt, workers):
    """(tile, first K step, last K step (exclusive), partial, slot or None) of one worker's run."""
    total = tiles * upt
    nxt, end = run_start(worker, total, workers), run_start(worker + 1, total, workers)
    out = []
    while nxt < end:
        tile = nxt // upt
        first = nxt - tile * upt
        last = min(upt, first + (end - nxt))
        partial = first != 0 or last != upt
        slot = (2 * worker + (0 if first != 0 else 1)) if partial else None
        out.append((tile, first, last, partial, slot))
        nxt += last - first
    return out


def fixup_jobs(tiles, upt, workers):
    """What the fix-up kernel does: {tile: [slots in the order they are added]}."""
    total = tiles * upt
    done = {}
    for j in range(1, workers):
        boundary = run_start(j, total, workers)
        tile = boundary // upt
        beg = tile * upt
        if boundary == beg:
            continue
        if j > 1 and run_start(j - 1, total, workers) > beg:
            continue
        x0, x1 = beg, beg + upt - 1
        w0 = ((x0 + 1) * workers + total - 1) // total - 1
        w1 = ((x1 + 1) * workers + total - 1) // total - 1
        assert tile not in done, "two jobs claim one tile"
        done[tile] = [2 * w0 + 1] + [2 * w for w in range(w0 + 1, w1 + 1)]
    return done


@pytest.mark.parametrize("tiles,upt,sms", list(itertools.product([1, 2, 3, 7, 32, 64, 150, 513], [1, 2, 5, 16, 33, 128], [1, 3, 74, 148])))
def test_runs_cover_every_step_once_and_fixup_finds_the_cut_tiles(tiles, upt, sms):
    total = tiles * upt
    workers = min(total, sms)
    seen = {}
    slots = {}
    written = {}   # tile -> [(first K step, slot)] of its partial segments
    whole = set()
    for w in range(workers):
        steps, partials = 0, 0
        for (tile, first, last, partial, slot) in segments(w, tiles, upt, workers):
            assert 0 <= first < last <= upt
            if partial:
                partials += 1
                assert slot not in slots, "two partial segments share a workspace slot"
                slots[slot] = (tile, w)
                written.setdefault(tile, []).append((first, slot))
            else:
                whole.add(tile)
            for k in range(first, last):
                assert (tile, k) not in seen
                seen[(tile, k)] = w
            steps += last - first
        assert partials <= 2
        assert steps in (total // workers, total // workers + 1), "runs differ by more than one step"
    assert len(seen) == total
    assert not slots or max(slots) < 2 * workers
    assert whole.isdisjoint(written), "a tile is both stored whole and cut"
    jobs = fixup_jobs(tiles, upt, workers)
    assert set(jobs) == set(written), "the fix-up pass visits other tiles than the cut ones"
    for tile, order in jobs.items():
        assert order == [slot for _, slot in sorted(written[tile])], "wrong partials, or not in K order"


def geometry(tiles, upt, slots):
    """`balanced_geometry` of csrc/gemm_lib.cu."""
    sk = tiles if tiles <= slots else tiles % slots
    runs = max(1, min(sk * upt, slots))
    grid = slots if tiles >= slots else runs
    return sk, runs, grid


@pytest.mark.parametrize("tiles,upt,slots", list(itertools.product([1, 2, 7, 73, 74, 75, 148, 160, 256, 300, 513], [1, 4, 32, 128], [1, 3, 74, 148])))
def test_whole_waves_round_robin_and_the_rest_in_runs(tiles, upt, slots):
    sk, runs, grid = geometry(tiles, upt, slots)
    assert 0 <= sk <= tiles and (tiles - sk) % slots == 0 or tiles <= slots
    assert 1 <= runs <= grid <= slots or sk == 0
    seen = {}
    for unit in range(grid):
        steps = 0
        if unit < runs:  # the worker's run over the cut tiles (WorkCursor: next / end)
            for (tile, first, last, partial, slot) in (segments(unit, sk, upt, runs) if sk else []):
                assert tile < sk
                for k in range(first, last):
                    assert (tile, k) not in seen
                    seen[(tile, k)] = unit
                steps += last - first
        t = sk + unit     # then whole tiles (WorkCursor: dp)
        while t < tiles:
            for k in range(upt):
                assert (t, k) not in seen
                seen[(t, k)] = unit
            steps += upt
            t += grid
    assert len(seen) == tiles * upt, "a K step of some tile is never computed"
    # every worker's load is within one K step of the others' when the tiles outnumber the workers
    if tiles >= slots and sk * upt >= slots:
        per = [sum(1 for v in seen.values() if v == u) for u in range(grid)]
        assert max(per) - min(per) <= 1
