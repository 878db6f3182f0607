"""Host bookkeeping: the shipped KVCacheManager / BlockTable against
  - the reference's own unit-test scenarios (tests/test_block_allocator.cpp:9-143),
  - the committed golden trace generated from the reference's compiled sources,
  - the pure-Python restatement and, where built, the compiled reference on random traces,
plus the additive copy-on-write operations."""
import json
import os

import numpy as np
import pytest

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def toks(n, base=0):
    return list(range(base, base + n))


def _val(x):
    return x() if callable(x) else x


def snapshot(mgr, tables):
    return {
        "free": _val(mgr.num_free_blocks), "cached": _val(mgr.num_cached_blocks), "used": _val(mgr.num_used_blocks),
        "avail": _val(mgr.num_available_blocks), "stats": _val(mgr.stats),
        "tables": [([int(b) for b in t.blocks], [int(h) for h in t.hashes], int(t.num_committed)) for t in tables],
    }


def random_trace_compare(make_a, make_b, seeds, steps=300):
    """Drives two allocator implementations with the same random operations and
    requires every observable result to be identical after every step."""
    for seed in seeds:
        rng = np.random.default_rng(1000 + seed)
        nb, bs = int(rng.integers(4, 40)), int(rng.choice([1, 2, 4, 16]))
        prefix = bool(seed % 3 != 2)
        A, B = make_a(nb, bs, prefix), make_b(nb, bs, prefix)
        live = []  # [ta, tb, tokens, computed]
        for _ in range(steps):
            r = rng.random()
            if r < 0.35 or not live:
                n = int(rng.integers(1, 5 * bs + 3))
                t = rng.integers(0, 4, size=n).astype(np.int32).tolist()
                if live and rng.random() < 0.5:
                    base = live[int(rng.integers(len(live)))][2]
                    t = (base[:len(base) // bs * bs] + t)[:8 * bs]
                ta, tb = A.new_table(), B.new_table()
                ra, rb = A.allocate_prompt(ta, t), B.allocate_prompt(tb, t)
                assert ra == rb
                if ra is not None:
                    live.append([ta, tb, t, ra])
            elif r < 0.6:
                e = live[int(rng.integers(len(live)))]
                oka, okb = A.ensure_slot(e[0], len(e[2]) + 1), B.ensure_slot(e[1], len(e[2]) + 1)
                assert oka == okb
                if oka:
                    e[2] = e[2] + [int(rng.integers(0, 4))]
            elif r < 0.85:
                e = live[int(rng.integers(len(live)))]
                nc = int(rng.integers(e[3], len(e[2]) + 1))
                A.commit_computed(e[0], e[2], nc)
                B.commit_computed(e[1], e[2], nc)
                e[3] = nc
            else:
                e = live.pop(int(rng.integers(len(live))))
                A.free(e[0])
                B.free(e[1])
            probe = rng.integers(0, 4, size=int(rng.integers(0, 3 * bs + 1))).astype(np.int32).tolist()
            assert A.lookup_cached_prefix(probe) == B.lookup_cached_prefix(probe)
            sa, sb = snapshot(A, [e[0] for e in live]), snapshot(B, [e[1] for e in live])
            assert sa == sb
            assert sa["free"] + sa["cached"] + sa["used"] == nb     # tests/test_stress.cpp's conservation law


# ---- the reference's eight scenarios ---------------------------------------------
def test_prompt_allocation_exhaustion_free_and_reuse(pkv):
    kv = pkv.KVCacheManager(4, 16, False)
    a, b = kv.new_table(), kv.new_table()
    assert kv.allocate_prompt(a, toks(33)) == 0
    assert a.num_blocks() == 3
    assert kv.num_free_blocks() == 1
    assert kv.allocate_prompt(b, toks(17)) is None
    assert b.empty()
    assert kv.num_free_blocks() == 1
    assert kv.stats()["allocation_failures"] == 1
    kv.free(a)
    assert a.empty()
    assert kv.num_free_blocks() == 4
    assert kv.allocate_prompt(b, toks(17)) == 0
    assert b.num_blocks() == 2


def test_ensure_slot_allocates_only_at_block_boundaries(pkv):
    kv = pkv.KVCacheManager(3, 4, False)
    bt = kv.new_table()
    assert kv.allocate_prompt(bt, toks(4)) == 0
    assert bt.num_blocks() == 1
    assert kv.ensure_slot(bt, 5) and bt.num_blocks() == 2
    assert kv.ensure_slot(bt, 6) and bt.num_blocks() == 2
    assert kv.ensure_slot(bt, 8) and bt.num_blocks() == 2
    assert kv.ensure_slot(bt, 9) and bt.num_blocks() == 3
    assert kv.num_free_blocks() == 0
    assert kv.ensure_slot(bt, 12)
    assert kv.ensure_slot(bt, 13) is False
    assert bt.slot(5, 4) == int(bt.blocks[1]) * 4 + 1


def test_shared_prompt_blocks_are_reused_and_refcounted(pkv):
    kv = pkv.KVCacheManager(8, 4, True)
    shared = toks(8, 1000)
    p1, p2 = shared + [1, 2], shared + [3]
    a, b = kv.new_table(), kv.new_table()
    assert kv.allocate_prompt(a, p1) == 0
    assert a.num_blocks() == 3
    assert kv.lookup_cached_prefix(p2) == 0
    kv.commit_computed(a, p1, 5)
    assert kv.lookup_cached_prefix(p2) == 4
    kv.commit_computed(a, p1, 10)
    assert kv.lookup_cached_prefix(p2) == 8
    assert kv.allocate_prompt(b, p2) == 8
    assert b.blocks[0] == a.blocks[0] and b.blocks[1] == a.blocks[1] and b.blocks[2] != a.blocks[2]
    assert kv.num_used_blocks() == 4
    assert kv.stats()["prefix_hit_blocks"] == 2
    assert kv.stats()["prefix_total_blocks"] == 4
    kv.free(a)
    assert kv.num_used_blocks() == 3
    assert kv.num_cached_blocks() == 0
    kv.free(b)
    assert kv.num_used_blocks() == 0
    assert kv.num_cached_blocks() == 2
    assert kv.num_free_blocks() == 6
    c = kv.new_table()
    assert kv.allocate_prompt(c, p1) == 8
    assert kv.num_cached_blocks() == 0


def test_hashes_are_position_aware(pkv):
    kv = pkv.KVCacheManager(8, 4, True)
    p = toks(8, 5)
    q = p[4:]
    a, b = kv.new_table(), kv.new_table()
    assert kv.allocate_prompt(a, p) == 0
    assert kv.lookup_cached_prefix(q) == 0
    assert kv.allocate_prompt(b, q) == 0
    assert b.blocks[0] != a.blocks[1]


def test_decode_fills_blocks_that_later_requests_reuse(pkv):
    kv = pkv.KVCacheManager(8, 4, True)
    a = kv.new_table()
    t = toks(3)
    assert kv.allocate_prompt(a, t) == 0
    kv.commit_computed(a, t, 3)
    t.append(3); assert kv.ensure_slot(a, 4); kv.commit_computed(a, t, 4)
    t.append(4); assert kv.ensure_slot(a, 5); kv.commit_computed(a, t, 5)
    kv.free(a)
    assert kv.num_cached_blocks() == 1
    assert kv.num_free_blocks() == 7
    b = kv.new_table()
    assert kv.allocate_prompt(b, toks(5)) == 4


def test_lru_eviction_oldest_released_first(pkv):
    kv = pkv.KVCacheManager(4, 2, True)
    a, b = kv.new_table(), kv.new_table()
    assert kv.allocate_prompt(a, toks(2, 10)) == 0; kv.commit_computed(a, toks(2, 10), 2)
    assert kv.allocate_prompt(b, toks(2, 20)) == 0; kv.commit_computed(b, toks(2, 20), 2)
    kv.free(a)
    kv.free(b)
    assert kv.num_cached_blocks() == 2
    assert kv.num_available_blocks() == 4
    c = kv.new_table()
    assert kv.allocate_prompt(c, toks(6, 30)) == 0; kv.commit_computed(c, toks(6, 30), 6)
    assert kv.stats()["evictions"] == 1
    assert kv.lookup_cached_prefix(toks(2, 10)) == 0
    assert kv.lookup_cached_prefix(toks(2, 20)) == 2
    kv.free(c)
    d = kv.new_table()
    assert kv.allocate_prompt(d, toks(2, 20)) == 2


def test_cannot_overcommit_against_blocks_about_to_be_reused(pkv):
    kv = pkv.KVCacheManager(2, 2, True)
    a = kv.new_table()
    assert kv.allocate_prompt(a, toks(4)) == 0; kv.commit_computed(a, toks(4), 4)
    kv.free(a)
    b = kv.new_table()
    assert kv.allocate_prompt(b, toks(5)) is None
    assert kv.num_cached_blocks() == 2
    assert kv.allocate_prompt(b, toks(4)) == 4


def test_prefix_caching_disabled_caches_nothing(pkv):
    kv = pkv.KVCacheManager(4, 2, False)
    a = kv.new_table()
    assert kv.allocate_prompt(a, toks(4)) == 0; kv.commit_computed(a, toks(4), 4)
    kv.free(a)
    assert kv.num_cached_blocks() == 0
    assert kv.num_free_blocks() == 4
    b = kv.new_table()
    assert kv.allocate_prompt(b, toks(4)) == 0


def test_constructor_rejects_non_positive_sizes(pkv):
    for nb, bs in ((0, 16), (4, 0), (-1, 4)):
        with pytest.raises(ValueError):
            pkv.KVCacheManager(nb, bs, True)


# ---- golden trace and differential runs ------------------------------------------------
def test_golden_trace_from_compiled_reference(pkv):
    from tests.test_oracle import _replay, check_allocator_state
    trace = json.load(open(os.path.join(GOLD, "allocator_trace.json")))
    count = lambda m, what: getattr(m, f"num_{what}_blocks")()
    n = 0
    for rec, mgr, live in _replay(trace, pkv.KVCacheManager):
        check_allocator_state(rec, mgr, live, count)
        n += 1
    assert n == len(trace["ops"])


def test_hash_block_matches_oracle(pkv, orc):
    rng = np.random.default_rng(5)
    for _ in range(100):
        t = rng.integers(-3, 2 ** 31 - 1, size=int(rng.integers(0, 33))).astype(np.int32)
        prev = int(rng.integers(0, 2 ** 63)) * 2 + int(rng.integers(0, 2))
        assert pkv.KVCacheManager.hash_block(prev, t) == orc.hash_block(prev, t)


def test_random_traces_against_python_restatement(pkv):
    from oracle import kv_oracle
    random_trace_compare(pkv.KVCacheManager, kv_oracle.Allocator, seeds=range(12))


def test_random_traces_against_compiled_reference(pkv, ref):
    if ref is None:
        pytest.skip("oracle/_ref/libpkv_ref.so not built (reference tree absent)")
    import oracle
    random_trace_compare(pkv.KVCacheManager, lambda nb, bs, p: oracle.ref_allocator(nb, bs, p), seeds=range(12))


def test_large_pool_trace_against_python_restatement(pkv):
    """Pool of the largest benchmark configuration (65,536 blocks of 16)."""
    from oracle import kv_oracle
    A, B = pkv.KVCacheManager(65536, 16, True), kv_oracle.Allocator(65536, 16, True)
    rng = np.random.default_rng(8)
    prefix = rng.integers(0, 32000, size=512).astype(np.int32).tolist()
    tabs = []
    for i in range(64):
        t = prefix + rng.integers(0, 32000, size=int(rng.integers(32, 257))).astype(np.int32).tolist()
        ta, tb = A.new_table(), B.new_table()
        assert A.allocate_prompt(ta, t) == B.allocate_prompt(tb, t) == (0 if i == 0 else 512)
        A.commit_computed(ta, t, len(t)); B.commit_computed(tb, t, len(t))
        tabs.append((ta, tb))
        assert ta.blocks.tolist() == tb.blocks
    assert A.num_used_blocks() == B.num_used_blocks
    assert A.ref_count(int(tabs[0][0].blocks[0])) == 64


# ---- copy-on-write (additive; the Python restatement defines the semantics) -------------
def test_fork_and_copy_on_write(pkv):
    from oracle import kv_oracle
    for make in (pkv.KVCacheManager, kv_oracle.Allocator):
        kv = make(8, 4, True)
        parent = kv.new_table()
        t = toks(6)                                  # one full block + a partial one holding 2 tokens
        assert kv.allocate_prompt(parent, t) == 0
        kv.commit_computed(parent, t, 6)
        kids = [kv.new_table() for _ in range(3)]
        for k in kids:
            kv.fork(parent, k)
            assert [int(b) for b in k.blocks] == [int(b) for b in parent.blocks]
        tail = int(parent.blocks[1])
        assert _val(kv.num_used_blocks) == 2
        # first divergent write of each child: position 6 lives in the shared partial block
        moved = []
        for k in kids:
            r = kv.cow(k, 6) if hasattr(kv, "cow") else kv.cow_tail(k, 6)
            assert r[0] == tail and r[1] not in (tail, -1)
            assert int(k.blocks[1]) == r[1] and int(k.blocks[0]) == int(parent.blocks[0])
            moved.append(r[1])
        assert len(set(moved)) == 3
        # the parent is now the block's only owner and writes in place
        r = kv.cow(parent, 6) if hasattr(kv, "cow") else kv.cow_tail(parent, 6)
        assert tuple(r) == (-1, -1)
        # a committed (full, published) block is never copied
        r = kv.cow(kids[0], 2) if hasattr(kv, "cow") else kv.cow_tail(kids[0], 2)
        assert tuple(r) == (-1, -1)
        assert _val(kv.num_used_blocks) == 5
        for k in kids:
            kv.free(k)
        kv.free(parent)
        assert _val(kv.num_used_blocks) == 0


def test_copy_on_write_reports_exhaustion(pkv):
    kv = pkv.KVCacheManager(2, 4, False)
    a, b = kv.new_table(), kv.new_table()
    assert kv.allocate_prompt(a, toks(6)) == 0
    kv.fork(a, b)
    assert kv.cow(b, 6) is None
    assert kv.stats()["allocation_failures"] == 1
