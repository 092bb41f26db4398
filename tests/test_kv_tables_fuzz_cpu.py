"""Random page-table operations (grow, release a window, share with a cache entry, adopt into a new row, drop entries,
free rows) on plain and context-parallel tables: after every operation each pool page is either free or referenced,
never both, and the reference counts equal the number of owners."""
import random

import pytest
import torch

from stkernel_b200.runtime.kv import GroupTable, OutOfPages


def _check(t: GroupTable, entries):
    owners = [0] * t.num_pages
    for row in range(t.max_requests):
        for lp in range(t.lo[row], t.hi[row]):
            pg = int(t.table_np[row, lp])
            assert pg != -1
            if pg != t.trash:
                assert t.owns(lp)
                owners[pg] += 1
            else:
                assert not t.owns(lp)
        assert all(int(x) == -1 for x in t.table_np[row, :t.lo[row]]) and all(int(x) == -1 for x in t.table_np[row, t.hi[row]:])
        assert t.held(row) == sum(1 for lp in range(t.lo[row], t.hi[row]) if t.owns(lp))
    for pages in entries:
        for pg in pages:
            if pg != t.trash:
                owners[pg] += 1
    assert owners == t.ref
    free = set(t.free)
    assert len(free) == len(t.free)                                   # no page twice in the free list
    assert free == {pg for pg in range(t.num_pages) if owners[pg] == 0}


@pytest.mark.parametrize("dcp", [(0, 1), (0, 2), (2, 3)])
@pytest.mark.parametrize("seed", [0, 1, 2])
def test_random_table_operations_keep_pages_accounted(dcp, seed):
    rng = random.Random(seed)
    t = GroupTable("c4", 24, 4, 20, torch.device("cpu"), 0.25, dcp[0], dcp[1])
    entries = []
    live = set()
    for _ in range(400):
        op = rng.choice(["grow", "grow", "grow", "window", "share", "adopt", "drop", "free"])
        row = rng.randrange(4)
        try:
            if op == "grow":
                last = min(19, t.hi[row] + rng.randint(0, 3))
                t.ensure(row, t.lo[row] if t.hi[row] > t.lo[row] else rng.randint(0, 2), last)
                live.add(row)
            elif op == "window" and t.hi[row] > t.lo[row]:
                t.release_before(row, rng.randint(t.lo[row], t.hi[row]))
            elif op == "share" and t.hi[row] > t.lo[row]:
                a = rng.randint(t.lo[row], t.hi[row] - 1)
                b = rng.randint(a, t.hi[row] - 1)
                entries.append((a, t.share(row, a, b)))
            elif op == "adopt" and entries and t.hi[row] == t.lo[row]:
                first, pages = rng.choice(entries)
                t.release_all(row)
                t.adopt(row, first, pages)
                live.add(row)
            elif op == "drop" and entries:
                _, pages = entries.pop(rng.randrange(len(entries)))
                for pg in pages:
                    t.unref(pg)
            elif op == "free":
                t.release_all(row)
                live.discard(row)
        except OutOfPages:
            pass                                                       # a full pool refuses; the state stays consistent
        _check(t, [p for _, p in entries])
    for row in range(4):
        t.release_all(row)
    for _, pages in entries:
        for pg in pages:
            t.unref(pg)
    _check(t, [])
    assert t.pages_in_use == 0
