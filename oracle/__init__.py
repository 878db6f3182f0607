"""TEST INFRASTRUCTURE -- NOT PRODUCT CODE.

ctypes bindings for the two CPU checkers of the paged-KV path:

``orc``  the plain-C restatement in ``oracle/paged_oracle.c`` (``liborc.so``)
``ref``  the reference's own sources compiled behind ``oracle/ref_shim.cpp``
         (``oracle/_ref/libpkv_ref.so``); ``None`` when that file was not built.

Both expose the same functions under the prefixes ``orc_`` / ``ref_``; the
``Checker`` class hides the prefix.  Only the test-suite, the smoke check and the
benchmark's CPU-baseline legs may import this package; the shipped library
(``llm-engine_b200``) never does.

Parity status: pinned (see the header of ``paged_oracle.c``).
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
ORC_PATH = os.path.join(_HERE, "liborc.so")
REF_PATH = os.path.join(_HERE, "_ref", "libpkv_ref.so")


def reference_root() -> str:
    """Where the llm-engine source tree is looked for: $LLM_ENGINE_REFERENCE, else the
    Makefile's default.  It need not exist (a prebuilt ``_ref/libpkv_ref.so`` is used then)."""
    return os.environ.get("LLM_ENGINE_REFERENCE", "/root/reference")


def build(verbose: bool = False) -> None:
    """Compile ``liborc.so`` and, where the reference tree is present, ``_ref/libpkv_ref.so``."""
    out = subprocess.run(["make", "-C", _HERE, "REF=" + reference_root()], capture_output=True, text=True)
    if verbose or out.returncode != 0:
        print(out.stdout + out.stderr)
    if out.returncode != 0:
        raise RuntimeError("building the oracle failed")


def _ptr(a, ctype=None):
    if a is None:
        return None
    assert a.flags["C_CONTIGUOUS"], "oracle arrays must be contiguous"
    return a.ctypes.data_as(C.c_void_p)


class Checker:
    """One of the two CPU implementations, behind a uniform numpy interface."""

    def __init__(self, path: str, prefix: str, kind: str):
        self.lib = C.CDLL(path)
        self.prefix = prefix
        self.kind = kind  # "port" (C restatement) or "reference" (compiled reference)
        L, p = self.lib, prefix
        f = lambda name: getattr(L, p + name)
        f("bf16_to_f32").restype = C.c_float
        f("bf16_to_f32").argtypes = [C.c_uint16]
        f("f32_to_bf16").restype = C.c_uint16
        f("f32_to_bf16").argtypes = [C.c_float]
        f("f16_to_f32").restype = C.c_float
        f("f16_to_f32").argtypes = [C.c_uint16]
        f("f32_to_f16").restype = C.c_uint16
        f("f32_to_f16").argtypes = [C.c_float]
        for n in ("f32_to_bf16_array", "bf16_to_f32_array", "f32_to_f16_array", "f16_to_f32_array"):
            f(n).restype = None
            f(n).argtypes = [C.c_void_p, C.c_void_p, C.c_size_t]
        f("slot").restype = C.c_int64
        f("slot").argtypes = [C.c_void_p, C.c_int, C.c_int]
        f("hash_block").restype = C.c_uint64
        f("hash_block").argtypes = [C.c_uint64, C.c_void_p, C.c_int]
        f("append").restype = None
        f("append").argtypes = [C.c_void_p] * 5 + [C.c_int, C.c_size_t]
        f("paged_attention").restype = None
        f("paged_attention").argtypes = [C.c_void_p] * 8 + [C.c_int] * 5 + [C.c_float, C.c_int]

        f("rope_tables").restype = None
        f("rope_tables").argtypes = [C.c_int, C.c_int, C.c_float, C.c_void_p, C.c_void_p]
        f("rope_inplace").restype = None
        f("rope_inplace").argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_void_p]

    def _f(self, name):
        return getattr(self.lib, self.prefix + name)

    # ---- rope --------------------------------------------------------------
    def rope_tables(self, head_dim: int, max_positions: int, theta: float):
        half = head_dim // 2
        cos = np.zeros((max_positions, half), dtype=np.float32)
        sin = np.zeros((max_positions, half), dtype=np.float32)
        self._f("rope_tables")(head_dim, max_positions, C.c_float(theta), _ptr(cos), _ptr(sin))
        return cos, sin

    def rope(self, x: np.ndarray, heads: int, head_dim: int, positions, cos, sin) -> np.ndarray:
        """x[n_tokens, heads*head_dim] fp32 -> rotated copy, token t at positions[t]."""
        out = np.ascontiguousarray(x, dtype=np.float32).copy()
        for t in range(out.shape[0]):
            row = out[t]
            self._f("rope_inplace")(row.ctypes.data_as(C.c_void_p), heads, head_dim, int(positions[t]), _ptr(cos), _ptr(sin))
        return out

    # ---- scalar casts ------------------------------------------------------
    def f32_to_bf16(self, x: float) -> int:
        return int(self._f("f32_to_bf16")(x))

    def bf16_to_f32(self, h: int) -> float:
        return float(self._f("bf16_to_f32")(h))

    def f32_to_f16(self, x: float) -> int:
        return int(self._f("f32_to_f16")(x))

    def f16_to_f32(self, h: int) -> float:
        return float(self._f("f16_to_f32")(h))

    # ---- array casts -------------------------------------------------------
    def to_bf16_bits(self, a: np.ndarray) -> np.ndarray:
        a = np.ascontiguousarray(a, dtype=np.float32)
        out = np.empty(a.shape, dtype=np.uint16)
        self._f("f32_to_bf16_array")(_ptr(a), _ptr(out), a.size)
        return out

    def from_bf16_bits(self, a: np.ndarray) -> np.ndarray:
        a = np.ascontiguousarray(a, dtype=np.uint16)
        out = np.empty(a.shape, dtype=np.float32)
        self._f("bf16_to_f32_array")(_ptr(a), _ptr(out), a.size)
        return out

    def to_f16_bits(self, a: np.ndarray) -> np.ndarray:
        a = np.ascontiguousarray(a, dtype=np.float32)
        out = np.empty(a.shape, dtype=np.uint16)
        self._f("f32_to_f16_array")(_ptr(a), _ptr(out), a.size)
        return out

    def from_f16_bits(self, a: np.ndarray) -> np.ndarray:
        a = np.ascontiguousarray(a, dtype=np.uint16)
        out = np.empty(a.shape, dtype=np.float32)
        self._f("f16_to_f32_array")(_ptr(a), _ptr(out), a.size)
        return out

    # ---- tables ------------------------------------------------------------
    def slot(self, blocks: np.ndarray, pos: int, block_size: int) -> int:
        blocks = np.ascontiguousarray(blocks, dtype=np.int32)
        return int(self._f("slot")(_ptr(blocks), pos, block_size))

    def hash_block(self, prev: int, tokens) -> int:
        t = np.ascontiguousarray(tokens, dtype=np.int32)
        return int(self._f("hash_block")(C.c_uint64(prev), _ptr(t), t.size))

    # ---- hot path ----------------------------------------------------------
    def append(self, k, v, slots, k_cache, v_cache) -> None:
        """In place: cache[slots[t]] = rows[t] for K and V (any dtype; byte copy)."""
        n = int(slots.shape[0])
        if n == 0:
            return
        row_bytes = k[0].nbytes
        slots = np.ascontiguousarray(slots, dtype=np.int32)
        self._f("append")(_ptr(k), _ptr(v), _ptr(slots), _ptr(k_cache), _ptr(v_cache), n, row_bytes)

    def paged_attention(self, q, k_cache, v_cache, block_tables, table_offset, token_seq, token_pos,
                        q_heads, kv_heads, head_dim, block_size, scale, threads=1) -> np.ndarray:
        """fp32 attention for every packed token; returns out[n_tokens, q_heads*head_dim]."""
        q = np.ascontiguousarray(q, dtype=np.float32)
        k_cache = np.ascontiguousarray(k_cache, dtype=np.float32)
        v_cache = np.ascontiguousarray(v_cache, dtype=np.float32)
        bt = np.ascontiguousarray(block_tables, dtype=np.int32)
        to = np.ascontiguousarray(table_offset, dtype=np.int32)
        ts = np.ascontiguousarray(token_seq, dtype=np.int32)
        tp = np.ascontiguousarray(token_pos, dtype=np.int32)
        n = int(tp.shape[0])
        out = np.zeros((n, q_heads * head_dim), dtype=np.float32)
        if n:
            self._f("paged_attention")(_ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(bt), _ptr(to), _ptr(ts),
                                       _ptr(tp), _ptr(out), n, q_heads, kv_heads, head_dim, block_size,
                                       C.c_float(scale), int(threads))
        return out


class RefAllocator:
    """The reference's KVCacheManager (compiled), driven through ref_shim.cpp handles."""

    class Table:
        def __init__(self, lib):
            self._lib = lib
            self.h = lib.ref_bt_new()

        def __del__(self):
            try:
                self._lib.ref_bt_delete(self.h)
            except Exception:
                pass

        @property
        def blocks(self):
            n = self._lib.ref_bt_num_blocks(self.h)
            out = np.zeros(n, dtype=np.int32)
            self._lib.ref_bt_blocks(self.h, _ptr(out))
            return out.tolist()

        @property
        def hashes(self):
            n = self._lib.ref_bt_num_blocks(self.h)
            out = np.zeros(n, dtype=np.uint64)
            self._lib.ref_bt_hashes(self.h, _ptr(out))
            return [int(x) for x in out]

        @property
        def num_committed(self):
            return self._lib.ref_bt_num_committed(self.h)

        def slot(self, pos, bs):
            return int(self._lib.ref_bt_slot(self.h, pos, bs))

    def __init__(self, lib, num_blocks, block_size, prefix):
        L = self.lib = lib
        L.ref_mgr_new.restype = C.c_void_p
        L.ref_mgr_new.argtypes = [C.c_int, C.c_int, C.c_int]
        L.ref_mgr_delete.argtypes = [C.c_void_p]
        L.ref_bt_new.restype = C.c_void_p
        L.ref_bt_delete.argtypes = [C.c_void_p]
        L.ref_mgr_allocate_prompt.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int]
        L.ref_mgr_ensure_slot.argtypes = [C.c_void_p, C.c_void_p, C.c_int]
        L.ref_mgr_commit_computed.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int]
        L.ref_mgr_commit_computed.restype = None
        L.ref_mgr_free.argtypes = [C.c_void_p, C.c_void_p]
        L.ref_mgr_free.restype = None
        L.ref_mgr_lookup_cached_prefix.argtypes = [C.c_void_p, C.c_void_p, C.c_int]
        L.ref_mgr_count.argtypes = [C.c_void_p, C.c_int]
        L.ref_mgr_stats.argtypes = [C.c_void_p, C.c_void_p]
        L.ref_mgr_stats.restype = None
        for n in ("ref_bt_num_blocks", "ref_bt_num_committed"):
            getattr(L, n).argtypes = [C.c_void_p]
        L.ref_bt_blocks.argtypes = [C.c_void_p, C.c_void_p]
        L.ref_bt_hashes.argtypes = [C.c_void_p, C.c_void_p]
        L.ref_bt_slot.restype = C.c_int64
        L.ref_bt_slot.argtypes = [C.c_void_p, C.c_int, C.c_int]
        self.h = L.ref_mgr_new(num_blocks, block_size, int(bool(prefix)))
        if not self.h:
            raise ValueError("num_blocks and block_size must be > 0")

    def __del__(self):
        try:
            self.lib.ref_mgr_delete(self.h)
        except Exception:
            pass

    def new_table(self):
        return RefAllocator.Table(self.lib)

    def allocate_prompt(self, bt, tokens):
        t = np.ascontiguousarray(tokens, dtype=np.int32)
        r = self.lib.ref_mgr_allocate_prompt(self.h, bt.h, _ptr(t), t.size)
        return None if r < 0 else r

    def ensure_slot(self, bt, num_tokens):
        return bool(self.lib.ref_mgr_ensure_slot(self.h, bt.h, num_tokens))

    def commit_computed(self, bt, tokens, num_computed):
        t = np.ascontiguousarray(tokens, dtype=np.int32)
        self.lib.ref_mgr_commit_computed(self.h, bt.h, _ptr(t), t.size, num_computed)

    def free(self, bt):
        self.lib.ref_mgr_free(self.h, bt.h)

    def lookup_cached_prefix(self, tokens):
        t = np.ascontiguousarray(tokens, dtype=np.int32)
        return self.lib.ref_mgr_lookup_cached_prefix(self.h, _ptr(t), t.size)

    def _count(self, what):
        return self.lib.ref_mgr_count(self.h, what)

    num_free_blocks = property(lambda s: s._count(0))
    num_cached_blocks = property(lambda s: s._count(1))
    num_available_blocks = property(lambda s: s._count(2))
    num_used_blocks = property(lambda s: s._count(3))
    num_total_blocks = property(lambda s: s._count(4))
    block_size = property(lambda s: s._count(5))
    capacity_tokens = property(lambda s: s._count(6))

    @property
    def stats(self):
        out = np.zeros(5, dtype=np.uint64)
        self.lib.ref_mgr_stats(self.h, _ptr(out))
        keys = ("prefix_queries", "prefix_hit_blocks", "prefix_total_blocks", "evictions", "allocation_failures")
        return dict(zip(keys, (int(x) for x in out)))


def load_orc() -> Checker:
    if not os.path.exists(ORC_PATH):
        build()
    return Checker(ORC_PATH, "orc_", "port")


def load_ref():
    """The compiled reference, or None when oracle/_ref/libpkv_ref.so is absent."""
    if not os.path.exists(REF_PATH):
        return None
    return Checker(REF_PATH, "ref_", "reference")


def ref_allocator(num_blocks, block_size, prefix):
    ref = load_ref()
    if ref is None:
        return None
    return RefAllocator(ref.lib, num_blocks, block_size, prefix)


def ref_default_thread_count() -> int:
    ref = load_ref()
    if ref is None:
        return os.cpu_count() or 1
    return int(ref.lib.ref_default_thread_count())
