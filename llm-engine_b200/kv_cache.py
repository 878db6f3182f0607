"""Host-side mirror of llm-engine's BlockTable / KVCacheManager, backed by libpkv.

Same method names, argument meaning and results as include/engine/kv_cache.h:21-99
of llm-engine; the arithmetic runs in the C++ class of include/pkv_kv_cache.hpp
through the C handles of include/pkv.h (section a0).
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import _lib

kNoBlock = -1


def _i32(tokens) -> np.ndarray:
    return np.ascontiguousarray(tokens, dtype=np.int32)


class BlockTable:
    """include/engine/kv_cache.h:21-32."""

    def __init__(self):
        self._L = _lib.lib()
        self._h = self._L.pkv_table_create()

    def __del__(self):
        try:
            self._L.pkv_table_destroy(self._h)
        except Exception:
            pass

    def num_blocks(self) -> int:
        return self._L.pkv_table_num_blocks(self._h)

    def empty(self) -> bool:
        return self.num_blocks() == 0

    @property
    def num_committed(self) -> int:
        return self._L.pkv_table_num_committed(self._h)

    @property
    def blocks(self) -> np.ndarray:
        """Copy of the physical block ids (int32)."""
        n = self.num_blocks()
        if n == 0:
            return np.zeros(0, dtype=np.int32)
        p = self._L.pkv_table_blocks(self._h)
        return np.ctypeslib.as_array(C.cast(p, C.POINTER(C.c_int32)), shape=(n,)).copy()

    @property
    def hashes(self) -> np.ndarray:
        n = self.num_blocks()
        if n == 0:
            return np.zeros(0, dtype=np.uint64)
        p = self._L.pkv_table_hashes(self._h)
        return np.ctypeslib.as_array(C.cast(p, C.POINTER(C.c_uint64)), shape=(n,)).copy()

    def slot(self, pos: int, block_size: int) -> int:
        s = self._L.pkv_table_slot(self._h, pos, block_size)
        if s < 0:
            raise IndexError(f"position {pos} lies beyond the table's {self.num_blocks()} blocks")
        return int(s)


class KVCacheManager:
    """include/engine/kv_cache.h:42-99."""

    def __init__(self, num_blocks: int, block_size: int, enable_prefix_caching: bool):
        self._L = _lib.lib()
        self._h = self._L.pkv_kvmgr_create(num_blocks, block_size, int(bool(enable_prefix_caching)))
        if not self._h:
            raise ValueError("num_blocks and block_size must be > 0")  # std::invalid_argument in the reference
        self._prefix = bool(enable_prefix_caching)

    def __del__(self):
        try:
            self._L.pkv_kvmgr_destroy(self._h)
        except Exception:
            pass

    def new_table(self) -> BlockTable:
        return BlockTable()

    def block_size(self) -> int:
        return self._L.pkv_kvmgr_block_size(self._h)

    def num_total_blocks(self) -> int:
        return self._L.pkv_kvmgr_num_total_blocks(self._h)

    def capacity_tokens(self) -> int:
        return self._L.pkv_kvmgr_capacity_tokens(self._h)

    def num_free_blocks(self) -> int:
        return self._L.pkv_kvmgr_num_free_blocks(self._h)

    def num_cached_blocks(self) -> int:
        return self._L.pkv_kvmgr_num_cached_blocks(self._h)

    def num_available_blocks(self) -> int:
        return self._L.pkv_kvmgr_num_available_blocks(self._h)

    def num_used_blocks(self) -> int:
        return self._L.pkv_kvmgr_num_used_blocks(self._h)

    def prefix_caching_enabled(self) -> bool:
        return self._prefix

    def ref_count(self, block: int) -> int:
        return self._L.pkv_kvmgr_ref_count(self._h, block)

    def stats(self) -> dict:
        out = (C.c_uint64 * 5)()
        self._L.pkv_kvmgr_stats(self._h, out)
        keys = ("prefix_queries", "prefix_hit_blocks", "prefix_total_blocks", "evictions", "allocation_failures")
        return dict(zip(keys, (int(x) for x in out)))

    @staticmethod
    def blocks_needed(num_tokens: int, block_size: int) -> int:
        return (num_tokens + block_size - 1) // block_size

    @staticmethod
    def hash_block(prev_hash: int, tokens) -> int:
        t = _i32(tokens)
        return int(_lib.lib().pkv_hash_block(C.c_uint64(prev_hash), t.ctypes.data, t.size))

    def allocate_prompt(self, bt: BlockTable, tokens):
        """Cached token count, or None when the pool cannot fit the prompt."""
        t = _i32(tokens)
        r = self._L.pkv_kvmgr_allocate_prompt(self._h, bt._h, t.ctypes.data, t.size)
        if r < -1:
            _lib.check("pkv_kvmgr_allocate_prompt", r)
        return None if r < 0 else r

    def ensure_slot(self, bt: BlockTable, num_tokens: int) -> bool:
        return bool(_lib.check("pkv_kvmgr_ensure_slot", self._L.pkv_kvmgr_ensure_slot(self._h, bt._h, num_tokens)))

    def commit_computed(self, bt: BlockTable, tokens, num_computed: int) -> None:
        t = _i32(tokens)
        if num_computed > t.size:
            raise ValueError("num_computed exceeds the number of tokens")
        self._L.pkv_kvmgr_commit_computed(self._h, bt._h, t.ctypes.data, t.size, num_computed)

    def free(self, bt: BlockTable) -> None:
        self._L.pkv_kvmgr_free(self._h, bt._h)

    def lookup_cached_prefix(self, tokens) -> int:
        t = _i32(tokens)
        return self._L.pkv_kvmgr_lookup_cached_prefix(self._h, t.ctypes.data, t.size)

    # ---- additive copy-on-write bookkeeping --------------------------------
    def fork(self, parent: BlockTable, child: BlockTable) -> None:
        _lib.check("pkv_kvmgr_fork", self._L.pkv_kvmgr_fork(self._h, parent._h, child._h))

    def cow(self, bt: BlockTable, write_pos: int):
        """(src, dst) to copy before writing write_pos, (-1, -1) if none; None when out of blocks."""
        s, d = C.c_int(-1), C.c_int(-1)
        r = self._L.pkv_kvmgr_cow(self._h, bt._h, write_pos, C.byref(s), C.byref(d))
        if r == _lib.PKV_E_NOMEM:
            return None
        _lib.check("pkv_kvmgr_cow", r)
        return (s.value, d.value)
