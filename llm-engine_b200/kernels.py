"""Device-side operators of the paged-KV path, named and shaped after llm-engine's
launchers (include/engine/cuda_kernels.h:43-62) and called through the C ABI.

Arguments are torch CUDA tensors (torch is used only for device memory and
streams); element type is taken from the tensors: float16 (the reference's CUDA
dtype), bfloat16 or float32.  Errors raise, as the reference launchers throw; there
is no CPU path.
"""
from __future__ import annotations

import ctypes as C

from . import _lib

_SUFFIX = {"torch.float16": "f16", "torch.bfloat16": "bf16", "torch.float32": "f32"}


def _suffix(t) -> str:
    try:
        return _SUFFIX[str(t.dtype)]
    except KeyError:
        raise TypeError(f"unsupported KV element type {t.dtype}") from None


def _ptr(t):
    if t is None:
        return None
    if not t.is_cuda:
        raise ValueError("paged-KV operators take CUDA tensors; there is no CPU path")
    if not t.is_contiguous():
        raise ValueError("paged-KV operators take contiguous tensors")
    return t.data_ptr()


def _stream(stream):
    if stream is None:
        import torch
        return torch.cuda.current_stream().cuda_stream
    return getattr(stream, "cuda_stream", stream)


def launch_store_kv(k, v, slots, k_cache, v_cache, n_tokens: int, kv_dim: int, stream=None) -> None:
    """k_cache[slots[t]] = k[t], v_cache[slots[t]] = v[t] (engine::launch_store_kv)."""
    fn = f"pkv_append_{_suffix(k_cache)}"
    st = getattr(_lib.lib(), fn)(_ptr(k), _ptr(v), _ptr(slots), _ptr(k_cache), _ptr(v_cache), n_tokens, kv_dim,
                                 _stream(stream))
    _lib.check(fn, st)


def launch_rope_store_kv(q, k, v, positions, cos_table, sin_table, slots, k_cache, v_cache, n_tokens: int,
                         q_heads: int, kv_heads: int, head_dim: int, stream=None) -> None:
    """launch_rope(q) + launch_rope(k) + launch_store_kv in one pass: q rotated in place, rotated k and v
    written to their slots (cos/sin: fp32 tables [max_positions][head_dim/2])."""
    fn = f"pkv_rope_append_{_suffix(k_cache)}"
    st = getattr(_lib.lib(), fn)(_ptr(q), _ptr(k), _ptr(v), _ptr(positions), _ptr(cos_table), _ptr(sin_table),
                                 _ptr(slots), _ptr(k_cache), _ptr(v_cache), n_tokens, q_heads, kv_heads, head_dim,
                                 _stream(stream))
    _lib.check(fn, st)


def decode_workspace_bytes(n_tokens: int, q_heads: int, kv_heads: int, head_dim: int) -> int:
    return int(_lib.lib().pkv_decode_workspace_bytes(n_tokens, q_heads, kv_heads, head_dim))


def alloc_decode_workspace(n_tokens: int, q_heads: int, kv_heads: int, head_dim: int, device="cuda"):
    """A uint8 CUDA tensor large enough for split-K at this step size (256-byte aligned)."""
    import torch
    n = decode_workspace_bytes(n_tokens, q_heads, kv_heads, head_dim)
    return torch.empty(max(n, 256), dtype=torch.uint8, device=device)


def launch_attention_decode(q, k_cache, v_cache, block_tables, table_offset, token_seq, token_pos, out,
                            n_tokens: int, q_heads: int, kv_heads: int, head_dim: int, block_size: int,
                            scale: float, stream=None, workspace=None) -> None:
    """engine::launch_attention_decode; `workspace` (uint8 CUDA tensor) enables split-K."""
    fn = f"pkv_decode_attn_{_suffix(k_cache)}"
    ws_ptr = _ptr(workspace)
    ws_bytes = workspace.numel() * workspace.element_size() if workspace is not None else 0
    st = getattr(_lib.lib(), fn)(_ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(block_tables), _ptr(table_offset),
                                 _ptr(token_seq), _ptr(token_pos), _ptr(out), n_tokens, q_heads, kv_heads,
                                 head_dim, block_size, C.c_float(scale), ws_ptr, ws_bytes, _stream(stream))
    _lib.check(fn, st)


def mixed_workspace_bytes(n_tokens: int, q_heads: int, kv_heads: int, head_dim: int) -> int:
    return int(_lib.lib().pkv_mixed_attn_workspace_bytes(n_tokens, q_heads, kv_heads, head_dim))


def launch_attention_mixed(q, k_cache, v_cache, block_tables, table_offset, token_seq, token_pos, out,
                           n_tokens: int, q_heads: int, kv_heads: int, head_dim: int, block_size: int,
                           scale: float, workspace, num_blocks: int = 0, min_run: int = 0, stream=None) -> None:
    """One call for a step that packs prefill chunks and decode tokens together, the way
    llm-engine's forward pass calls launch_attention_decode (src/model/cuda/cuda_model.cu:362-377):
    runs of at least min_run consecutive tokens of one sequence go to the tensor-core prefill kernel,
    the rest to the decode kernels; the split is made on the device."""
    fn = f"pkv_mixed_attn_{_suffix(k_cache)}"
    st = getattr(_lib.lib(), fn)(_ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(block_tables), _ptr(table_offset),
                                 _ptr(token_seq), _ptr(token_pos), _ptr(out), n_tokens, q_heads, kv_heads, head_dim,
                                 block_size, num_blocks, C.c_float(scale), min_run, _ptr(workspace),
                                 workspace.numel() * workspace.element_size(), _stream(stream))
    _lib.check(fn, st)


# llm-engine keeps two names for the same operation, chosen by ENGINE_ATTN
# (src/model/cuda/cuda_model.cu:554-557); both are one kernel here.
launch_attention_decode_gqa = launch_attention_decode


class DecodePlan:
    """Split-K work list built once per step and shared by every layer's attention call."""

    def __init__(self, n_tokens: int, q_heads: int, kv_heads: int, head_dim: int, workspace=None, device="cuda",
                 num_blocks: int = 0):
        """num_blocks: blocks per K/V pool, if known: the kernels' tensor maps then end at the pool
        (a wrong block id reads zeros); 0 = unknown, as through llm-engine's own launcher signature."""
        import torch
        self.n_tokens, self.q_heads, self.kv_heads, self.head_dim = n_tokens, q_heads, kv_heads, head_dim
        self.num_blocks = num_blocks
        self.workspace = workspace if workspace is not None else alloc_decode_workspace(
            n_tokens, q_heads, kv_heads, head_dim, device)
        nstage = int(_lib.lib().pkv_decode_plan_staging_bytes(n_tokens, kv_heads))
        self.staging = torch.empty(max(nstage, 256), dtype=torch.uint8).pin_memory()
        self.plan = _lib.DecodePlan()

    def _ws(self):
        return self.workspace.data_ptr(), self.workspace.numel()

    def build_host(self, token_pos_host, stream=None) -> "DecodePlan":
        """token_pos_host: int32 numpy array or CPU tensor of the packed tokens' positions."""
        import numpy as np
        pos = np.ascontiguousarray(token_pos_host, dtype=np.int32)
        p, n = self._ws()
        st = _lib.lib().pkv_decode_plan_host(pos.ctypes.data, self.n_tokens, self.q_heads, self.kv_heads,
                                             self.head_dim, self.staging.data_ptr(), self.staging.numel(), p, n,
                                             _stream(stream), C.byref(self.plan))
        _lib.check("pkv_decode_plan_host", st)
        self.plan.num_blocks = self.num_blocks
        return self

    def build_host_image(self, token_pos_host) -> int:
        """The host planner without the upload: the image goes to self.staging (pinned) and its size
        is returned; the caller copies it to the start of self.workspace, typically as a node of a
        captured graph that is replayed every step."""
        import numpy as np
        pos = np.ascontiguousarray(token_pos_host, dtype=np.int32)
        n = C.c_size_t(0)
        st = _lib.lib().pkv_decode_plan_host_image(pos.ctypes.data, self.n_tokens, self.q_heads, self.kv_heads, self.head_dim,
                                                   self.staging.data_ptr(), self.staging.numel(), self.workspace.numel(),
                                                   C.byref(self.plan), C.byref(n))
        _lib.check("pkv_decode_plan_host_image", st)
        self.plan.num_blocks = self.num_blocks
        return int(n.value)

    def build_host_shared(self, idx, block_size: int, min_saved_bytes: int = -1, stream=None) -> "DecodePlan":
        """Shared-prefix-aware plan from the host copies of the step's index arrays (`idx`: a
        StepIndices as returned by pack_step): sequences whose tables start with the same blocks
        have that range read once per group of up to four tokens, if that saves at least
        min_saved_bytes of K/V reads per layer (-1: the library's default; 0: always)."""
        import numpy as np
        pos = np.ascontiguousarray(idx.token_pos, dtype=np.int32)
        seq = np.ascontiguousarray(idx.token_seq, dtype=np.int32)
        tabs = np.ascontiguousarray(idx.block_tables, dtype=np.int32)
        off = np.ascontiguousarray(idx.table_offset, dtype=np.int32)
        p, n = self._ws()
        st = _lib.lib().pkv_decode_plan_host_shared(pos.ctypes.data, seq.ctypes.data, tabs.ctypes.data, off.ctypes.data,
                                                    self.n_tokens, off.size, tabs.size, block_size, self.q_heads,
                                                    self.kv_heads, self.head_dim, min_saved_bytes, self.staging.data_ptr(),
                                                    self.staging.numel(), p, n, _stream(stream), C.byref(self.plan))
        _lib.check("pkv_decode_plan_host_shared", st)
        self.plan.num_blocks = self.num_blocks
        return self

    @property
    def n_shared_units(self) -> int:
        return int(self.plan.reserved) >> 1

    def build_device(self, token_pos, stream=None) -> "DecodePlan":
        p, n = self._ws()
        st = _lib.lib().pkv_decode_plan_device(_ptr(token_pos), self.n_tokens, self.q_heads, self.kv_heads,
                                               self.head_dim, p, n, _stream(stream), C.byref(self.plan))
        _lib.check("pkv_decode_plan_device", st)
        self.plan.num_blocks = self.num_blocks
        return self

    def attention(self, q, k_cache, v_cache, block_tables, table_offset, token_seq, token_pos, out,
                  block_size: int, scale: float, stream=None) -> None:
        fn = f"pkv_decode_attn_planned_{_suffix(k_cache)}"
        p, n = self._ws()
        st = getattr(_lib.lib(), fn)(C.byref(self.plan), _ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(block_tables),
                                     _ptr(table_offset), _ptr(token_seq), _ptr(token_pos), _ptr(out), block_size,
                                     C.c_float(scale), p, n, _stream(stream))
        _lib.check(fn, st)

    def append_attention(self, q, k, v, slots, k_cache, v_cache, block_tables, table_offset, token_seq, token_pos, out,
                         block_size: int, scale: float, stream=None) -> None:
        """launch_store_kv + attention in one chain (decode steps only: one token per sequence)."""
        fn = f"pkv_append_decode_attn_planned_{_suffix(k_cache)}"
        p, n = self._ws()
        st = getattr(_lib.lib(), fn)(C.byref(self.plan), _ptr(q), _ptr(k), _ptr(v), _ptr(slots), _ptr(k_cache), _ptr(v_cache),
                                     _ptr(block_tables), _ptr(table_offset), _ptr(token_seq), _ptr(token_pos), _ptr(out),
                                     block_size, C.c_float(scale), p, n, _stream(stream))
        _lib.check(fn, st)


def launch_attention_prefill(q, k_cache, v_cache, block_tables, table_offset, q_start, q_len, ctx_len, out,
                             n_tokens: int, n_seqs: int, max_q_len: int, q_heads: int, kv_heads: int, head_dim: int,
                             block_size: int, num_blocks: int, scale: float, stream=None) -> None:
    """Causal attention of each sequence's new chunk over its cached plus new tokens."""
    fn = f"pkv_prefill_attn_{_suffix(k_cache)}"
    st = getattr(_lib.lib(), fn)(_ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(block_tables), _ptr(table_offset),
                                 _ptr(q_start), _ptr(q_len), _ptr(ctx_len), _ptr(out), n_tokens, n_seqs, max_q_len, q_heads,
                                 kv_heads, head_dim, block_size, num_blocks, C.c_float(scale), _stream(stream))
    _lib.check(fn, st)


def launch_copy_blocks(k_cache, v_cache, src_dst_pairs, n_pairs: int, block_size: int, kv_dim: int,
                       stream=None) -> None:
    """Copy-on-write: block pairs[2i] -> block pairs[2i+1] in both pools."""
    fn = f"pkv_copy_blocks_{_suffix(k_cache)}"
    st = getattr(_lib.lib(), fn)(_ptr(k_cache), _ptr(v_cache), _ptr(src_dst_pairs), n_pairs, block_size, kv_dim,
                                 _stream(stream))
    _lib.check(fn, st)


def launch_copy_blocks_layers(cache_ptrs, n_caches: int, src_dst_pairs, n_pairs: int, block_bytes: int,
                              stream=None) -> None:
    """Same for every pool at once; cache_ptrs is an int64 CUDA tensor of pool base addresses."""
    st = _lib.lib().pkv_copy_blocks_layers(_ptr(cache_ptrs), n_caches, _ptr(src_dst_pairs), n_pairs, block_bytes,
                                           _stream(stream))
    _lib.check("pkv_copy_blocks_layers", st)


def debug_device_flags() -> int:
    """Reads and clears the word in which kernels record a bounded wait that ran out
    (synchronises the device; 0 = no kernel ever gave up)."""
    v = C.c_uint(0)
    _lib.check("pkv_debug_device_flags", _lib.lib().pkv_debug_device_flags(C.byref(v)))
    return int(v.value)
