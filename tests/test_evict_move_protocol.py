"""In-place stable compaction by several CTAs per segment, checked by simulation (no GPU).

``evict_move_kernel`` (trimkv_b200/csrc/tkv_evict.cu) lets C CTAs share the rows of one segment: CTA c owns destination
rows [lo_c, hi_c), stages the rows whose source lies at or beyond hi_c ("tail"), raises a flag, waits for its left
neighbour's flag, moves its remaining rows tile by tile (all loads of a tile, then all its stores) and stores the tail
last.  This file restates that schedule, runs the CTAs under random interleavings at the granularity of those steps on an
array whose rows carry their original index, and checks that every load returns the row's ORIGINAL content and that the
result is the stable compaction.  It also shows that ranges shorter than the largest displacement would be unsafe, which
is why the kernel never makes them shorter than max_len - M rows.
"""
import random

import numpy as np
import pytest


def move_range(m, j0, ctas, tail_max, tile_rows, c, enforce_min=True):
    total = max(m - j0, 0)
    per = -(-(-(-total // ctas)) // tile_rows)                      # ceil(ceil(total / ctas) / tile_rows)
    if enforce_min:
        per = max(per, -(-tail_max // tile_rows))
    per *= tile_rows
    lo = min(m, j0 + c * per)
    return lo, min(m, lo + per)


def cta_program(kept, m, j0, ctas, tail_max, tile_rows, c, enforce_min=True):
    """Steps of CTA c as (kind, rows): 'load' src rows into private storage, 'store' them to dst rows, 'flag', 'wait'."""
    lo, hi = move_range(m, j0, ctas, tail_max, tile_rows, c, enforce_min)
    steps = [("start", None)]                                        # the block has been dispatched, nothing done yet
    if lo >= hi:
        return steps + [("flag", None)]
    jt = hi
    if hi < m:
        jt = lo + int(np.searchsorted(kept[lo:hi], hi, side="left"))   # first row whose source is at or beyond hi
    tail = list(range(jt, hi))
    steps.append(("load", tail))
    steps.append(("flag", None))
    if c > 0:
        steps.append(("wait", None))
    for jb in range(lo, jt, tile_rows):
        rows = list(range(jb, min(jb + tile_rows, jt)))
        steps.append(("load", rows))
        steps.append(("store", rows))
    steps.append(("store", tail))
    return steps


def simulate(n, m, ctas, tile_rows, seed, enforce_min=True):
    rng = random.Random(seed)
    nprng = np.random.default_rng(seed)
    kept = np.sort(nprng.choice(n, size=m, replace=False))
    moved = np.nonzero(kept != np.arange(m))[0]
    j0 = int(moved[0]) if moved.size else m
    tail_max = n - m
    mem = np.arange(n)                                              # row i holds original row i
    progs = [cta_program(kept, m, j0, ctas, tail_max, tile_rows, c, enforce_min) for c in range(ctas)]
    pc, flag, held = [0] * ctas, [False] * ctas, [dict() for _ in range(ctas)]
    while any(pc[c] < len(progs[c]) for c in range(ctas)):
        # blocks are dispatched in index order: a CTA can only run once every lower-numbered one has started
        started = [pc[c] > 0 for c in range(ctas)]
        runnable = []
        for c in range(ctas):
            if pc[c] >= len(progs[c]):
                continue
            if c > 0 and not started[c - 1]:
                continue
            kind, _ = progs[c][pc[c]]
            if kind == "wait" and not flag[c - 1]:
                continue
            runnable.append(c)
        assert runnable, "dead-lock"
        c = rng.choice(runnable)
        kind, rows = progs[c][pc[c]]
        if kind == "load":
            for j in rows:
                if mem[kept[j]] != kept[j]:
                    return f"CTA {c} read row {kept[j]} after it was overwritten (holds {mem[kept[j]]})"
                held[c][j] = mem[kept[j]]
        elif kind == "store":
            for j in rows:
                mem[j] = held[c].pop(j)
        elif kind == "flag":
            flag[c] = True
        pc[c] += 1
    return None if np.array_equal(mem[:m], kept) else "result is not the stable compaction"


@pytest.mark.parametrize("n,m,ctas,tile_rows", [(640, 512, 4, 32), (4224, 4096, 16, 64), (4224, 4096, 32, 64), (4200, 4096, 5, 64),
                                               (133, 100, 8, 16), (130, 129, 2, 64), (300, 7, 3, 8)])
def test_ranges_and_flags_keep_every_source_intact_until_it_is_read(n, m, ctas, tile_rows):
    for seed in range(25):
        assert simulate(n, m, ctas, tile_rows, seed) is None


def test_ranges_shorter_than_the_largest_displacement_are_unsafe():
    """Without the minimum range length, a CTA's sources reach beyond its right neighbour's range, whose owner only
    waits for its direct neighbour: some schedule overwrites a row before it has been read."""
    outcomes = [simulate(700, 600, 32, 8, seed, enforce_min=False) for seed in range(60)]
    assert any(o is not None for o in outcomes)
    assert all(simulate(700, 600, 32, 8, seed) is None for seed in range(60))
