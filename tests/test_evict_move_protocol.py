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


def simulate_grid(nseg_evicting, n, m, ctas, rows_y, resident, tile_rows, seed):
    """The whole move kernel: a grid of ctas x rows_y blocks, block (c, y) taking the evicting segments y, y + rows_y, ...
    in turn (``evict_move_kernel``'s loop over the list written by the selection kernel), with at most ``resident``
    blocks on the device at once, dispatched in index order as earlier ones finish."""
    rng = random.Random(seed)
    nprng = np.random.default_rng(seed)
    kept, mem, progs_of = [], [], {}
    for s in range(nseg_evicting):
        kp = np.sort(nprng.choice(n, size=m, replace=False))
        moved = np.nonzero(kp != np.arange(m))[0]
        j0 = int(moved[0]) if moved.size else m
        kept.append(kp); mem.append(np.arange(n))
        for c in range(ctas):
            progs_of[(s, c)] = cta_program(kp, m, j0, ctas, n - m, tile_rows, c)
    blocks = [(c, y) for y in range(rows_y) for c in range(ctas)]            # linear block index: x fastest
    prog = {}
    for (c, y) in blocks:
        steps = [("start", None, None)]
        for s in range(y, nseg_evicting, rows_y):
            steps += [(kind, rows, s) for kind, rows in progs_of[(s, c)] if kind != "start"]
        prog[(c, y)] = steps
    pc = {b: 0 for b in blocks}
    flag, held = set(), {b: dict() for b in blocks}
    dispatched, next_block = [], 0
    while True:
        dispatched = [b for b in dispatched if pc[b] < len(prog[b])]
        while len(dispatched) < resident and next_block < len(blocks):
            dispatched.append(blocks[next_block]); next_block += 1
        if not dispatched:
            break
        runnable = []
        for b in dispatched:
            kind, _, s = prog[b][pc[b]]
            if kind == "wait" and (s, b[0] - 1) not in flag:
                continue
            runnable.append(b)
        assert runnable, "dead-lock"
        b = rng.choice(runnable)
        kind, rows, s = prog[b][pc[b]]
        if kind == "load":
            for j in rows:
                if mem[s][kept[s][j]] != kept[s][j]:
                    return f"block {b} read row {kept[s][j]} of segment {s} after it was overwritten"
                held[b][(s, j)] = mem[s][kept[s][j]]
        elif kind == "store":
            for j in rows:
                mem[s][j] = held[b].pop((s, j))
        elif kind == "flag":
            flag.add((s, b[0]))
        pc[b] += 1
    for s in range(nseg_evicting):
        if not np.array_equal(mem[s][:m], kept[s]):
            return f"segment {s}: result is not the stable compaction"
    return None


@pytest.mark.parametrize("nseg_evicting,n,m,ctas,rows_y,resident", [
    (16, 640, 512, 4, 37, 444),      # fewer evicting segments than rows of the grid: some blocks find nothing to do
    (9, 640, 512, 4, 4, 16),         # every block walks two or three segments
    (9, 640, 512, 4, 4, 5),          # fewer resident blocks than the grid holds: later blocks start as earlier ones end
    (7, 200, 150, 8, 3, 9),
    (5, 133, 100, 8, 2, 1),          # one block at a time: strictly in index order
])
def test_blocks_walking_a_list_of_segments_cannot_dead_lock(nseg_evicting, n, m, ctas, rows_y, resident):
    for seed in range(12):
        assert simulate_grid(nseg_evicting, n, m, ctas, rows_y, resident, 16, seed) is None
