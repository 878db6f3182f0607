"""ctypes binding of libpkv.so (the C ABI declared in include/pkv.h).

There is no fallback: if the library has not been built, or a call returns a
non-zero status, an exception is raised.
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("PKV_LIB_PATH") or os.path.join(_HERE, "libpkv.so")  # override: developer builds

PKV_OK = 0
PKV_E_ARG, PKV_E_UNSUPPORTED, PKV_E_WORKSPACE, PKV_E_CUDA, PKV_E_NOMEM, PKV_E_STATE = -1, -2, -3, -4, -5, -6


class PkvError(RuntimeError):
    def __init__(self, fn: str, status: int, detail: str):
        self.status = status
        super().__init__(f"{fn}: status {status}: {detail}")


class DecodePlan(C.Structure):
    """Mirror of struct pkv_decode_plan."""
    _fields_ = [("n_tokens", C.c_int), ("q_heads", C.c_int), ("kv_heads", C.c_int), ("head_dim", C.c_int),
                ("chunk", C.c_int), ("n_items", C.c_int), ("exact", C.c_int), ("reserved", C.c_int),
                ("num_blocks", C.c_int), ("cluster", C.c_int), ("pad", C.c_int * 2)]


_vp, _i, _f, _sz, _u64 = C.c_void_p, C.c_int, C.c_float, C.c_size_t, C.c_uint64

# name -> (restype, argtypes); every symbol include/pkv.h declares.
SIGNATURES = {
    "pkv_abi_version": (_i, []),
    "pkv_status_string": (C.c_char_p, [_i]),
    "pkv_last_error": (C.c_char_p, []),
    "pkv_debug_device_flags": (_i, [_vp]),
    "pkv_debug_set_reported_flags": (_i, [C.c_uint]),
    "pkv_debug_cluster_launches": (C.c_ulonglong, []),
    "pkv_mixed_attn_workspace_bytes": (_sz, [_i] * 4),
    **{f"pkv_mixed_attn_{s}": (_i, [_vp] * 8 + [_i] * 6 + [_f, _i, _vp, _sz, _vp]) for s in ("f16", "bf16")},
    **{f"pkv_append_{s}": (_i, [_vp] * 5 + [_i, _i, _vp]) for s in ("f16", "bf16", "f32")},
    **{f"pkv_rope_append_{s}": (_i, [_vp] * 9 + [_i] * 4 + [_vp]) for s in ("f16", "bf16", "f32")},
    "pkv_decode_workspace_bytes": (_sz, [_i] * 4),
    **{f"pkv_decode_attn_{s}": (_i, [_vp] * 8 + [_i] * 5 + [_f, _vp, _sz, _vp]) for s in ("f16", "bf16", "f32")},
    "pkv_decode_attn_bf16_builtin_scratch": (_i, [_vp] * 8 + [_i] * 5 + [_f, _vp]),
    "pkv_decode_plan_staging_bytes": (_sz, [_i, _i]),
    "pkv_decode_plan_host": (_i, [_vp, _i, _i, _i, _i, _vp, _sz, _vp, _sz, _vp, C.POINTER(DecodePlan)]),
    "pkv_decode_plan_host_image": (_i, [_vp, _i, _i, _i, _i, _vp, _sz, _sz, C.POINTER(DecodePlan), C.POINTER(_sz)]),
    "pkv_decode_plan_device": (_i, [_vp, _i, _i, _i, _i, _vp, _sz, _vp, C.POINTER(DecodePlan)]),
    **{f"pkv_decode_attn_planned_peer_{s}": (_i, [C.POINTER(DecodePlan)] + [_vp] * 7 + [_vp, _vp, _i, _i, _i, _i, _i, _f, _vp, _sz, _vp])
       for s in ("f16", "bf16")},
    **{f"pkv_append_decode_attn_planned_{s}": (_i, [C.POINTER(DecodePlan)] + [_vp] * 11 + [_i, _f, _vp, _sz, _vp])
       for s in ("f16", "bf16")},
    "pkv_peer_alloc": (_i, [_sz, _vp, _vp]),
    "pkv_peer_open": (_i, [_vp, _vp]),
    "pkv_peer_close": (_i, [_vp]),
    "pkv_peer_free": (_i, [_vp]),
    "pkv_decode_plan_host_shared": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, C.c_longlong, _vp, _sz, _vp, _sz, _vp,
                                         C.POINTER(DecodePlan)]),
    **{f"pkv_decode_attn_planned_{s}": (_i, [C.POINTER(DecodePlan)] + [_vp] * 8 + [_i, _f, _vp, _sz, _vp])
       for s in ("f16", "bf16", "f32")},
    **{f"pkv_prefill_attn_{s}": (_i, [_vp] * 9 + [_i] * 8 + [_f, _vp]) for s in ("f16", "bf16")},
    **{f"pkv_copy_blocks_{s}": (_i, [_vp, _vp, _vp, _i, _i, _i, _vp]) for s in ("f16", "bf16", "f32")},
    "pkv_copy_blocks_layers": (_i, [_vp, _i, _vp, _i, _sz, _vp]),
    "pkv_step_pack_device": (_i, [_vp, _i, _vp, _i, _vp, _vp, _i, _i, _i, _vp, _vp, _vp, _i, _vp, _i, _vp, _vp, _vp]),
    "pkv_step_pack": (_i, [_i, _vp, _vp, _vp, _vp, _i, _vp, _vp, _vp, _sz, _vp, _sz, _vp, _vp]),
    "pkv_kvmgr_create": (_vp, [_i, _i, _i]),
    "pkv_kvmgr_destroy": (None, [_vp]),
    "pkv_table_create": (_vp, []),
    "pkv_table_destroy": (None, [_vp]),
    "pkv_kvmgr_allocate_prompt": (_i, [_vp, _vp, _vp, _i]),
    "pkv_kvmgr_ensure_slot": (_i, [_vp, _vp, _i]),
    "pkv_kvmgr_commit_computed": (None, [_vp, _vp, _vp, _i, _i]),
    "pkv_kvmgr_free": (None, [_vp, _vp]),
    "pkv_kvmgr_lookup_cached_prefix": (_i, [_vp, _vp, _i]),
    "pkv_hash_block": (_u64, [_u64, _vp, _i]),
    **{f"pkv_kvmgr_{n}": (_i, [_vp]) for n in ("block_size", "num_total_blocks", "capacity_tokens",
                                                "num_free_blocks", "num_cached_blocks", "num_available_blocks",
                                                "num_used_blocks")},
    "pkv_kvmgr_stats": (None, [_vp, _vp]),
    "pkv_kvmgr_ref_count": (_i, [_vp, _i]),
    "pkv_table_num_blocks": (_i, [_vp]),
    "pkv_table_num_committed": (_i, [_vp]),
    "pkv_table_blocks": (_vp, [_vp]),
    "pkv_table_hashes": (_vp, [_vp]),
    "pkv_table_slot": (C.c_int64, [_vp, _i, _i]),
    "pkv_kvmgr_fork": (_i, [_vp, _vp, _vp]),
    "pkv_kvmgr_cow": (_i, [_vp, _vp, _i, _vp, _vp]),
}

_lib = None


def lib() -> C.CDLL:
    """The loaded library.  Raises if it has not been built (python llm-engine_b200/build.py)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(f"{LIB_PATH} is missing: build it with `python llm-engine_b200/build.py` "
                               "(there is no fallback implementation)")
        L = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(L, name)  # AttributeError here means the library is stale
            fn.restype = res
            fn.argtypes = args
        _lib = L
    return _lib


def last_error() -> str:
    return (lib().pkv_last_error() or b"").decode()


def check(fn: str, status: int) -> int:
    if status < 0:
        raise PkvError(fn, status, f"{lib().pkv_status_string(status).decode()}: {last_error()}")
    return status
