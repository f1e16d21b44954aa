"""The cache manager on the host: allocator contract, tables, groups, windows, state slots."""

import ctypes
import random

import numpy as np
import pytest

from miniserve_b200.cache import BlockAllocator, BlockTable, CacheManager, OutOfBlocks
from miniserve_b200.ops import native
from miniserve_b200.parts import FixedState, PagedKV
from miniserve_b200.parts.decoder import EntryCache


# ------------------------------------------------------------------ allocator (miniserve/cache/block_allocator.py contract)
def test_fresh_allocator_hands_out_in_order_and_reuses_lifo():
    a = BlockAllocator(6, 16)
    assert a.allocate(3) == [0, 1, 2]
    a.free([1])
    a.free([0])
    assert a.allocate(3) == [0, 1, 3]
    assert a.num_free == 2 and a.num_used == 4
    a.check_invariants()


def test_allocate_is_all_or_nothing():
    a = BlockAllocator(4, 8)
    a.allocate(3)
    with pytest.raises(OutOfBlocks):
        a.allocate(2)
    assert a.num_free == 1
    with pytest.raises(ValueError):
        a.allocate(-1)
    assert a.allocate(0) == []


def test_free_validates_before_it_changes_anything():
    a = BlockAllocator(4, 8)
    got = a.allocate(3)
    with pytest.raises(ValueError):
        a.free([got[0], got[1], got[1]])  # the second release of block 1 is one too many
    assert a.num_free == 1 and a.refcount(got[0]) == 1
    with pytest.raises(IndexError):
        a.free([7])
    with pytest.raises(ValueError):
        a.free([3])  # never allocated
    a.incref([got[0]])
    a.free([got[0], got[0]])
    assert a.refcount(got[0]) == 0
    with pytest.raises(ValueError):
        a.incref([got[0]])
    a.check_invariants()


def test_bad_sizes_are_refused():
    with pytest.raises(ValueError):
        BlockAllocator(0, 16)
    with pytest.raises(ValueError):
        BlockAllocator(4, 0)


def test_allocator_against_a_model_under_random_operations():
    rng = random.Random(0)
    a = BlockAllocator(32, 4)
    free = list(range(31, -1, -1))
    held: list[int] = []
    for _ in range(2000):
        if rng.random() < 0.5:
            n = rng.randint(0, 6)
            if n > len(free):
                with pytest.raises(OutOfBlocks):
                    a.allocate(n)
            else:
                expect = [free.pop() for _ in range(n)]
                assert a.allocate(n) == expect
                held += expect
        elif held:
            k = rng.randint(1, min(4, len(held)))
            pick = [held.pop(rng.randrange(len(held))) for _ in range(k)]
            a.free(pick)
            free += pick
        assert a.num_free == len(free)
    a.check_invariants()


# ------------------------------------------------------------------ tables (miniserve/cache/block_table.py contract)
def test_table_append_slot_rewind_release():
    a = BlockAllocator(8, 4)
    a.allocate(2)  # so that the table's blocks are not 0, 1, ...
    t = a.new_table()
    assert t.blocks_needed(5) == 2
    t.append_tokens(5)
    assert t.blocks == [2, 3] and t.num_tokens == 5 and t.capacity == 8
    assert t.slot(0) == 8 and t.slot(4) == 12
    with pytest.raises(IndexError):
        t.slot(5)
    assert t.blocks_needed(3) == 0 and t.blocks_needed(4) == 1
    t.rewind(2)
    assert t.num_tokens == 3 and t.blocks == [2, 3]  # blocks stay
    with pytest.raises(IndexError):
        t.rewind(4)
    t.append_tokens(9)
    assert t.num_tokens == 12 and len(t.blocks) == 3
    with pytest.raises(OutOfBlocks):
        t.append_tokens(100)
    assert t.num_tokens == 12 and len(t.blocks) == 3  # nothing changed
    t.release()
    assert t.num_tokens == 0 and t.blocks == [] and a.num_free == 6
    a.check_invariants()


def test_table_gives_back_pages_below_a_position():
    a = BlockAllocator(8, 4)
    t = a.new_table()
    t.append_tokens(14)  # pages 0..3
    assert t.release_below(9) == 2  # pages 0, 1 lie wholly below 9 (page 2 holds 8..11)
    assert t.blocks == [-1, -1, 2, 3] and t.num_blocks == 2 and a.num_free == 6
    assert t.release_below(9) == 0
    with pytest.raises(IndexError):
        t.slot(3)
    assert t.slot(9) == 2 * 4 + 1
    assert t.release_below(1000) == 1  # never the page of the newest token
    assert t.blocks == [-1, -1, -1, 3]
    t.append_tokens(3)  # reuses a freed page for the new tail
    assert t.blocks[:4] == [-1, -1, -1, 3] and t.blocks[4] == 2
    t.release()
    assert a.num_free == 8
    a.check_invariants()


# ------------------------------------------------------------------ the manager
def _entries(n_full=2, n_window=0, n_state=0, shared=False):
    out = []
    for i in range(n_full):
        out.append(EntryCache(len(out), PagedKV(2, 16)))
    for i in range(n_window):
        out.append(EntryCache(len(out), PagedKV(2, 16, window=10)))
    for i in range(n_state):
        out.append(EntryCache(len(out), FixedState((3, 4))))
    if shared:
        out.append(EntryCache(0, PagedKV(2, 16)))
    return out


def test_layers_with_equal_needs_share_a_group_and_windowed_ones_have_their_own():
    cm = CacheManager(_entries(3, 2, 1, shared=True), num_pages=16, page_size=4, max_requests=3)
    assert cm.num_groups == 2
    assert cm.groups[0].entries == [0, 1, 2] and cm.groups[1].entries == [3, 4]
    assert cm.groups[0].allocator is not cm.groups[1].allocator
    views = cm.entry_views
    assert views[0].group == 0 and views[3].group == 1 and views[6].group == 0  # the reader sees its owner's group
    assert views[5].shape == (3, 4)
    with pytest.raises(ValueError):
        CacheManager(_entries(1), num_pages=4, page_size=6, max_requests=1)


def test_reserve_is_all_or_nothing_across_rows_and_groups():
    cm = CacheManager(_entries(1, 1), num_pages=4, page_size=4, max_requests=4)
    a, b = cm.new_request(), cm.new_request()
    cm.reserve([(a, 6)])
    with pytest.raises(OutOfBlocks):
        cm.reserve([(a, 2), (b, 9)])  # 0 + 3 pages > 2 free
    assert a.num_tokens == 6 and b.num_tokens == 0 and cm.num_free() == (2, 2)
    cm.reserve([(a, 2), (b, 5)])
    assert cm.num_free() == (0, 0)
    cm.release(a)
    cm.release(b)
    with pytest.raises(ValueError):
        cm.release(b)
    assert cm.is_idle()
    cm.check_invariants()


def test_window_group_gives_pages_back_while_running_and_reuses_them():
    cm = CacheManager(_entries(1, 1), num_pages=8, page_size=4, max_requests=2)
    r = cm.new_request()
    cm.reserve([(r, 20)])
    assert cm.num_free() == (3, 3)
    freed = cm.trim(r)  # next query at position 20 sees keys from 11 on: pages 0, 1 go (page 2 holds 8..11)
    assert freed == 2 and cm.num_free() == (3, 5)
    assert r.tables[1].blocks[:2] == [-1, -1] and r.tables[0].blocks == [0, 1, 2, 3, 4]
    cm.reserve([(r, 8)])  # positions 20..27 -> two more pages; the windowed group reuses the freed ones
    assert r.tables[1].blocks[5:] == [1, 0]
    cm.trim(r)
    cm.release(r)
    assert cm.is_idle()
    cm.check_invariants()


def test_state_slots_are_handed_out_once_and_returned():
    cm = CacheManager(_entries(1, 0, 1), num_pages=4, page_size=4, max_requests=2)
    a, b = cm.new_request(), cm.new_request()
    assert {a.state_slot, b.state_slot} == {0, 1}
    with pytest.raises(OutOfBlocks):
        cm.new_request()
    cm.release(a)
    c = cm.new_request()
    assert c.state_slot == 0 and cm.num_free_slots == 0
    cm.release(b)
    cm.release(c)
    assert cm.is_idle()


def test_no_page_is_lost_held_twice_or_freed_twice_under_random_orders():
    rng = random.Random(1)
    cm = CacheManager(_entries(2, 1, 1), num_pages=24, page_size=4, max_requests=5)
    live = []
    for step in range(3000):
        op = rng.random()
        if op < 0.25 and cm.num_free_slots:
            live.append(cm.new_request())
        elif op < 0.75 and live:
            rows = [(rc, rng.randint(1, 9)) for rc in rng.sample(live, rng.randint(1, len(live)))]
            before = [(rc.num_tokens, [t.blocks for t in rc.tables]) for rc, _ in rows]
            try:
                cm.reserve(rows)
            except OutOfBlocks:
                assert before == [(rc.num_tokens, [t.blocks for t in rc.tables]) for rc, _ in rows]
            else:
                for rc, _ in rows:
                    cm.trim(rc)
        elif live:
            cm.release(live.pop(rng.randrange(len(live))))
        # every page is either free or held by exactly one table of its group
        for gi, g in enumerate(cm.groups):
            held = [b for rc in live for b in rc.tables[gi].blocks if b >= 0]
            assert len(held) == len(set(held)), "a page is held twice"
            assert len(held) + g.allocator.num_free == g.allocator.num_blocks, "a page was lost"
            assert all(g.allocator.refcount(b) == 1 for b in held)
        assert len({rc.state_slot for rc in live}) == len(live)
        cm.check_invariants()
    for rc in live:
        cm.release(rc)
    assert cm.is_idle()


# ------------------------------------------------------------------ the step packer
def _pack(tables_by_group, q_start, q_len, ids, want, pad_rows=0, pad_page=(99,), indices_cap=0, want_pad=False, pad_len=1,
          page_size=4):
    lib = native.host()
    rows, groups = len(q_len), len(tables_by_group)
    arena = np.full(4096, -7, dtype=np.int32)
    offsets = (ctypes.c_longlong * (9 + 2 * groups))()
    handles = (ctypes.c_void_p * max(rows * groups, 1))()
    for g, tabs in enumerate(tables_by_group):
        for i, t in enumerate(tabs):
            handles[g * rows + i] = t.handle
    arr = lambda x: np.asarray(x, dtype=np.int32)
    qs, ql, tok, ss, wa, pp = arr(q_start), arr(q_len), arr(ids), arr([5] * rows), arr(want), arr(list(pad_page))
    total = lib.ms_pack_step(arena.ctypes.data, arena.size, offsets, rows, pad_rows, qs.ctypes.data, ql.ctypes.data,
                             tok.ctypes.data, ss.ctypes.data, wa.ctypes.data, len(want), groups, handles,
                             pp.ctypes.data, indices_cap, int(want_pad), 64, pad_len, page_size)
    return total, arena, list(offsets)


def test_packer_against_a_naive_layout():
    a = BlockAllocator(16, 4)
    t0, t1 = a.new_table(), a.new_table()
    t1.append_tokens(3)
    t0.append_tokens(6)   # request 0: 6 tokens, all new
    t1.append_tokens(2)   # request 1: 3 cached + 2 new
    total, arena, o = _pack([[t0, t1]], [0, 3], [6, 2], [10, 11, 12, 13, 14, 15, 20, 21], [5, 7], pad_rows=1,
                            want_pad=True)
    assert total > 0
    T, R = 9, 3
    assert arena[o[0]:o[0] + T].tolist() == [10, 11, 12, 13, 14, 15, 20, 21, 0]
    assert arena[o[1]:o[1] + T].tolist() == [0, 1, 2, 3, 4, 5, 3, 4, 0]
    assert arena[o[2]:o[2] + T].tolist() == [0] * 6 + [1, 1, 2]
    assert arena[o[3]:o[3] + R + 1].tolist() == [0, 6, 8, 9]
    assert arena[o[4]:o[4] + R].tolist() == [0, 3, 0]
    assert arena[o[5]:o[5] + R].tolist() == [6, 5, 1]
    assert arena[o[6]:o[6] + R].tolist() == [5, 5, 64]  # the padding row gets the spare state slot
    assert arena[o[7]:o[7] + 3].tolist() == [5, 7, 8]
    assert arena[o[8]:o[8] + R + 1].tolist() == [0, 2, 4, 5]
    assert arena[o[9]:o[9] + 5].tolist() == t0.blocks + t1.blocks + [99]
    assert all(x % 4 == 0 for x in o)


def test_packer_pads_with_a_row_of_several_tokens():
    """A padding row of 6 tokens on pages of 4: positions 0..5, two page entries that both name the page
    outside the allocator, the spare state slot; the real rows are packed as without it."""
    a = BlockAllocator(16, 4)
    t0 = a.new_table()
    t0.append_tokens(5)
    total, arena, o = _pack([[t0]], [2], [3], [7, 8, 9], [2], pad_rows=1, pad_len=6)
    assert total > 0
    T, R = 9, 2
    assert arena[o[0]:o[0] + T].tolist() == [7, 8, 9, 0, 0, 0, 0, 0, 0]
    assert arena[o[1]:o[1] + T].tolist() == [2, 3, 4, 0, 1, 2, 3, 4, 5]
    assert arena[o[2]:o[2] + T].tolist() == [0, 0, 0] + [1] * 6
    assert arena[o[3]:o[3] + R + 1].tolist() == [0, 3, 9]
    assert arena[o[4]:o[4] + R].tolist() == [2, 0] and arena[o[5]:o[5] + R].tolist() == [5, 6]
    assert arena[o[6]:o[6] + R].tolist() == [5, 64]
    assert arena[o[7]:o[7] + 1].tolist() == [2]
    assert arena[o[8]:o[8] + R + 1].tolist() == [0, 2, 4]
    assert arena[o[9]:o[9] + 4].tolist() == t0.blocks + [99, 99]
    total, arena, o = _pack([[t0]], [2], [3], [7, 8, 9], [2], pad_rows=2, pad_len=3, want_pad=True)
    assert arena[o[7]:o[7] + 3].tolist() == [2, 5, 8]  # with their logits wanted: each padding row's last token
    assert _pack([[t0]], [2], [3], [7, 8, 9], [2], pad_rows=1, pad_len=0)[0] < 0


def test_packer_refuses_inconsistent_steps():
    a = BlockAllocator(16, 4)
    t = a.new_table()
    t.append_tokens(5)
    total, _, _ = _pack([[t]], [0], [4], [1, 2, 3, 4], [])  # the table holds 5 tokens, the step ends at 4
    assert total < 0 and "table holds 5" in native.host().ms_host_last_error().decode()
    total, _, _ = _pack([[t]], [0], [5], [1, 2, 3, 4, 5], [9])
    assert total < 0
    total, _, _ = _pack([[t]], [5], [0], [], [])
    assert total < 0
    total, _, o = _pack([[t]], [0], [5], [1, 2, 3, 4, 5], [4], indices_cap=7)
    assert total > 0 and o[10] - o[9] == 8  # fixed room, rounded up to 4 entries
    total, _, _ = _pack([[t]], [0], [5], [1, 2, 3, 4, 5], [4], indices_cap=1)
    assert total < 0


def test_packer_packs_only_the_pages_a_windowed_table_still_holds():
    """A table that has given pages back is packed from the entry below its first live page; the row's
    base is where entry 0 would be, so kernels index by absolute page number all the same."""
    a = BlockAllocator(32, 4)
    t0, t1 = a.new_table(), a.new_table()
    t0.append_tokens(22)          # pages 0..5
    assert t0.release_below(17) == 4  # pages 0..3 lie wholly below 17
    t1.append_tokens(5)
    t0.append_tokens(1)
    t1.append_tokens(2)
    total, arena, o = _pack([[t0, t1]], [22, 5], [1, 2], [1, 2, 3], [0, 2])
    assert total > 0
    base0, base1, end = arena[o[8]:o[8] + 3].tolist()
    packed = arena[o[9]:o[9] + end].tolist()
    blocks0, blocks1 = t0.blocks, t1.blocks
    assert end == (len(blocks0) - 3) + len(blocks1)  # three of the four freed entries are not packed at all
    for page in range(3, len(blocks0)):               # the entry just below the live ones reads -1
        assert packed[base0 + page] == blocks0[page]
    assert packed[base0 + 3] == -1 and base0 == -3
    for page in range(len(blocks1)):
        assert packed[base1 + page] == blocks1[page]
    # long decoding behind a window: the packed size stays bounded by what is held
    for _ in range(200):
        t0.append_tokens(1)
        t0.release_below(t0.num_tokens - 10 + 1)
    total, arena, o = _pack([[t0]], [t0.num_tokens - 1], [1], [7], [0], indices_cap=8)
    assert total > 0 and t0.num_entries > 50 and t0.num_blocks <= 4


def test_groups_may_have_pools_of_different_sizes_and_windows_bound_what_a_request_holds():
    from miniserve_b200.cache.manager import group_needs, window_pages

    entries = _entries(2, 1, 1)
    needs, states = group_needs(entries)
    assert [(n.window, c) for n, c in needs] == [(None, 2), (10, 1)] and len(states) == 1
    cm = CacheManager(entries, num_pages=[24, 6], page_size=4, max_requests=3, step_tokens=8)
    assert cm.group_pages() == (24, 6) and cm.num_pages == 24
    # a long request may hold all its pages in the full group, but only window + step in the windowed one
    assert cm.pages_for(80) == (20, window_pages(10, 4, 8)) == (20, 6)
    assert cm.pages_for(7) == (2, 2)
    with pytest.raises(ValueError, match="page counts"):
        CacheManager(entries, num_pages=[24], page_size=4, max_requests=3)
    r = cm.new_request()
    for _ in range(10):  # 80 tokens in steps of 8: the windowed group never runs out of its 6 pages
        cm.reserve([(r, 8)])
        cm.trim(r)
    assert cm.pages_held(r)[0] == 20 and cm.pages_held(r)[1] <= 6
    cm.release(r)
    assert cm.is_idle()


def test_host_core_under_address_and_undefined_behaviour_sanitizers(tmp_path):
    """The allocator, table and packer tests once more in a process whose host core is compiled with
    -fsanitize=address,undefined (MINISERVE_HOST_SANITIZE=1): an out-of-bounds write, a use after
    free or signed overflow in the C++ would end that process with a report."""
    import os
    import shutil
    import subprocess
    import sys

    gcc = shutil.which("gcc")
    if gcc is None:
        pytest.skip("no gcc to ask for the sanitizer runtime")
    runtime = subprocess.run([gcc, "-print-file-name=libasan.so"], capture_output=True, text=True).stdout.strip()
    if not os.path.isfile(runtime):
        pytest.skip("the AddressSanitizer runtime is not installed")
    env = dict(os.environ, MINISERVE_HOST_SANITIZE="1", MINISERVE_BUILD_DIR=str(tmp_path), LD_PRELOAD=os.path.realpath(runtime),
               ASAN_OPTIONS="detect_leaks=0:abort_on_error=1", UBSAN_OPTIONS="halt_on_error=1:print_stacktrace=1")
    here = os.path.dirname(os.path.abspath(__file__))
    proc = subprocess.run(
        [sys.executable, "-m", "pytest", os.path.join(here, "test_cache.py"), "-q", "-x", "-p", "no:cacheprovider",
         "-k", "not sanitizers"], capture_output=True, text=True, env=env, timeout=600, cwd=os.path.dirname(here))
    assert proc.returncode == 0, proc.stdout[-3000:] + proc.stderr[-3000:]
    assert (tmp_path / "libms_host_san.so").is_file(), "the sanitized host core was not the one that ran"
    assert "AddressSanitizer" not in proc.stderr and "runtime error" not in proc.stderr, proc.stderr[-3000:]
