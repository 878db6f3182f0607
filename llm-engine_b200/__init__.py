"""B200 (sm_100a) paged-KV hot path for llm-engine: K/V append, paged decode
attention, paged prefill attention and the copy-on-write block copy, behind the C
ABI of include/pkv.h, plus the host bookkeeping that feeds them.

The directory name contains a hyphen, so import it with
``importlib.import_module("llm-engine_b200")``.
"""
from . import _lib
from ._lib import PkvError, lib
from .kv_cache import BlockTable, KVCacheManager, kNoBlock
from .step import DeviceStepPacker, StepIndices, pack_step
from .kernels import (DecodePlan, debug_device_flags, alloc_decode_workspace, decode_workspace_bytes, launch_attention_decode,
                      launch_attention_decode_gqa, launch_attention_mixed, launch_attention_prefill, mixed_workspace_bytes, launch_copy_blocks,
                      launch_copy_blocks_layers, launch_rope_store_kv, launch_store_kv)

__all__ = [
    "PkvError", "lib", "debug_device_flags", "BlockTable", "KVCacheManager", "kNoBlock", "StepIndices", "pack_step", "DeviceStepPacker", "DecodePlan",
    "alloc_decode_workspace", "decode_workspace_bytes", "launch_attention_decode", "launch_attention_decode_gqa",
    "launch_attention_mixed", "mixed_workspace_bytes", "launch_attention_prefill", "launch_copy_blocks", "launch_copy_blocks_layers", "launch_rope_store_kv", "launch_store_kv",
]
