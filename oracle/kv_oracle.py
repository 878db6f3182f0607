"""TEST INFRASTRUCTURE -- NOT PRODUCT CODE.

A small pure-Python restatement of llm-engine's KV block bookkeeping, used to
check the shipped C++ ``KVCacheManager`` on short traces.  Follows
src/kv_cache/block_allocator.cpp (line numbers cited per method) and
include/engine/kv_cache.h:21-32.  Parity status: pinned -- tests/test_oracle.py
replays the reference's own unit-test scenarios (tests/test_block_allocator.cpp)
through it and compares it step by step with the compiled reference on random
traces.

The copy-on-write additions (``fork`` / ``cow_tail``) have no counterpart in the
reference (docs/design.md:36 says sharing is full-block only, so it never copies);
their semantics are defined here and in include/pkv_kv_cache.hpp.
"""
from __future__ import annotations

from collections import OrderedDict

M64 = (1 << 64) - 1
GOLD = 0x9E3779B97F4A7C15


def _mix(z: int) -> int:
    z = (z + GOLD) & M64
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & M64
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & M64
    return z ^ (z >> 31)


def hash_block(prev: int, tokens) -> int:
    """block_allocator.cpp:16-23."""
    h = prev ^ GOLD
    for t in tokens:
        h = _mix(h ^ (int(t) & 0xFFFFFFFF))
    return 1 if h == 0 else h


class Table:
    """include/engine/kv_cache.h:21-32."""

    def __init__(self):
        self.blocks: list[int] = []
        self.hashes: list[int] = []
        self.num_committed = 0

    def slot(self, pos: int, bs: int) -> int:
        return self.blocks[pos // bs] * bs + pos % bs


class Allocator:
    def __init__(self, num_blocks: int, block_size: int, prefix: bool):
        if num_blocks <= 0 or block_size <= 0:
            raise ValueError("num_blocks and block_size must be > 0")
        self.nb, self.bs, self.prefix = num_blocks, block_size, bool(prefix)
        self.free_list = list(range(num_blocks - 1, -1, -1))  # pop() hands out low ids first (:12-13)
        self.ref = [0] * num_blocks
        self.block_hash = [0] * num_blocks
        self.by_hash: dict[int, int] = {}
        self.lru: "OrderedDict[int, None]" = OrderedDict()  # first = least recently released
        self.stats = dict(prefix_queries=0, prefix_hit_blocks=0, prefix_total_blocks=0, evictions=0,
                          allocation_failures=0)

    # kv_cache.h:46-55
    num_free_blocks = property(lambda s: len(s.free_list))
    num_cached_blocks = property(lambda s: len(s.lru))
    num_available_blocks = property(lambda s: len(s.free_list) + len(s.lru))
    num_used_blocks = property(lambda s: s.nb - len(s.free_list) - len(s.lru))

    def new_table(self):
        return Table()

    def _take(self):  # :25-35
        if self.free_list:
            return self.free_list.pop()
        if not self.lru:
            return None
        b, _ = self.lru.popitem(last=False)
        self.by_hash.pop(self.block_hash[b], None)
        self.block_hash[b] = 0
        self.stats["evictions"] += 1
        return b

    def _release(self, b, h):  # :42-52
        assert self.ref[b] > 0
        self.ref[b] -= 1
        if self.ref[b] > 0:
            return
        if self.prefix and h != 0 and self.block_hash[b] == h:
            self.lru[b] = None
        else:
            if self.block_hash[b] != 0:
                self.by_hash.pop(self.block_hash[b], None)
                self.block_hash[b] = 0
            self.free_list.append(b)

    def lookup_cached_prefix(self, tokens):  # :66-76
        if not self.prefix:
            return 0
        prev, hit = 0, 0
        for i in range(len(tokens) // self.bs):
            h = hash_block(prev, tokens[i * self.bs:(i + 1) * self.bs])
            if h not in self.by_hash:
                break
            hit += 1
            prev = h
        return hit * self.bs

    def allocate_prompt(self, bt: Table, tokens):  # :78-116
        assert not bt.blocks
        n = len(tokens)
        needed = (n + self.bs - 1) // self.bs
        full = n // self.bs
        self.stats["prefix_queries"] += 1
        self.stats["prefix_total_blocks"] += full
        hits, prev = [], 0
        if self.prefix:
            for i in range(full):
                h = hash_block(prev, tokens[i * self.bs:(i + 1) * self.bs])
                b = self.by_hash.get(h)
                if b is None:
                    break
                hits.append((h, b))
                prev = h
        cached = len(hits)
        lru_hits = sum(1 for _, b in hits if self.ref[b] == 0)
        if needed - cached > self.num_available_blocks - lru_hits:
            self.stats["allocation_failures"] += 1
            return None
        for h, b in hits:
            self.lru.pop(b, None)
            self.ref[b] += 1
            bt.blocks.append(b)
            bt.hashes.append(h)
        self.stats["prefix_hit_blocks"] += cached
        for _ in range(cached, needed):
            b = self._take()
            assert b is not None
            self.ref[b] = 1
            bt.blocks.append(b)
            bt.hashes.append(0)
        bt.num_committed = cached
        return cached * self.bs

    def ensure_slot(self, bt: Table, num_tokens: int) -> bool:  # :118-128
        needed = (num_tokens + self.bs - 1) // self.bs
        assert needed <= len(bt.blocks) + 1
        if needed > len(bt.blocks):
            b = self._take()
            if b is None:
                self.stats["allocation_failures"] += 1
                return False
            self.ref[b] = 1
            bt.blocks.append(b)
            bt.hashes.append(0)
        return True

    def commit_computed(self, bt: Table, tokens, num_computed: int):  # :130-137 with :54-64
        if not self.prefix:
            return
        assert num_computed <= len(tokens)
        while bt.num_committed < len(bt.blocks) and (bt.num_committed + 1) * self.bs <= num_computed:
            i = bt.num_committed
            prev = 0 if i == 0 else bt.hashes[i - 1]
            if not (i > 0 and prev == 0):
                h = hash_block(prev, tokens[i * self.bs:(i + 1) * self.bs])
                if h not in self.by_hash:
                    b = bt.blocks[i]
                    self.by_hash[h] = b
                    self.block_hash[b] = h
                    bt.hashes[i] = h
            bt.num_committed += 1

    def free(self, bt: Table):  # :139-142
        for i in range(len(bt.blocks) - 1, -1, -1):
            self._release(bt.blocks[i], bt.hashes[i])
        bt.blocks, bt.hashes, bt.num_committed = [], [], 0

    # ---- additive copy-on-write bookkeeping (no reference counterpart) ----
    def fork(self, parent: Table, child: Table):
        """Child shares every block of the parent, the partial tail included."""
        assert not child.blocks
        for b, h in zip(parent.blocks, parent.hashes):
            self.ref[b] += 1
            child.blocks.append(b)
            child.hashes.append(h)
        child.num_committed = parent.num_committed

    def cow_tail(self, bt: Table, write_pos: int):
        """Before writing position write_pos: if its block is shared, move this
        table to a private block.  Returns (src, dst), (-1, -1) when nothing has to
        be copied, or None when the pool is exhausted."""
        i = write_pos // self.bs
        if i >= len(bt.blocks) or i < bt.num_committed:
            return (-1, -1)  # committed (full, published) blocks are only ever re-written identically
        src = bt.blocks[i]
        if self.ref[src] <= 1:
            return (-1, -1)
        dst = self._take()
        if dst is None:
            self.stats["allocation_failures"] += 1
            return None
        self.ref[dst] = 1
        self.ref[src] -= 1
        bt.blocks[i] = dst
        bt.hashes[i] = 0
        return (src, dst)
