"""Multi-GPU sharding of the paged-KV path: by sequence, with no data-path exchange.

Every GPU owns a block pool and a set of sequences; a step on one GPU touches only that
GPU's memory, so the only cross-rank traffic is the benchmark's own bookkeeping (a barrier
and two scalar reductions).  llm-engine itself is single-GPU
(src/model/cuda/cuda_model.cu:239); this is the harness around it.
"""
from __future__ import annotations

import numpy as np


def rank_seed(base_seed: int, rank: int) -> int:
    """Weak scaling: every rank draws its own batch of the same shape."""
    return base_seed + 1000 * rank


def deal_sequences(ctx_lengths, world: int, rank: int, policy: str = "balanced") -> np.ndarray:
    """Strong scaling: indices of the sequences of ONE batch that `rank` owns.

    round_robin: sequence i goes to rank i % world.
    balanced:    longest-first greedy on context length, so every rank reads about the same
                 number of K/V bytes (contexts in one batch can differ by 64x).
    Every sequence is owned by exactly one rank."""
    L = np.asarray(ctx_lengths, dtype=np.int64)
    if world <= 1:
        return np.arange(L.size)
    if policy == "round_robin":
        return np.arange(rank, L.size, world)
    if policy != "balanced":
        raise ValueError(policy)
    load = np.zeros(world, dtype=np.int64)
    owner = np.empty(L.size, dtype=np.int64)
    for i in np.argsort(-L, kind="stable"):
        r = int(np.argmin(load))
        owner[i] = r
        load[r] += L[i] + 1
    return np.nonzero(owner == rank)[0]


def reduce_step(tokens_this_rank: float, ms_this_rank: float, dist=None, device=None):
    """(total tokens over ranks, max time over ranks): whole-job throughput = tokens / time."""
    if dist is None or not dist.is_initialized() or dist.get_world_size() == 1:
        return float(tokens_this_rank), float(ms_this_rank)
    import torch
    t = torch.tensor([tokens_this_rank], dtype=torch.float64, device=device)
    m = torch.tensor([ms_this_rank], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.SUM)
    dist.all_reduce(m, op=dist.ReduceOp.MAX)
    return float(t.item()), float(m.item())


def head_slices(q_heads: int, kv_heads: int, world: int, rank: int):
    """Head-sharded variant: (first query head, query heads, first kv head, kv heads) of `rank`.
    Needs kv_heads % world == 0; a GQA group stays on one rank."""
    if kv_heads % world or q_heads % kv_heads:
        raise ValueError(f"{kv_heads} kv heads do not divide over {world} ranks")
    kvl = kv_heads // world
    ql = q_heads // world
    return rank * ql, ql, rank * kvl, kvl


class _RawCuda:
    """A device allocation that torch did not make, viewed through __cuda_array_interface__."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3}


class HeadShardedExchange:
    """Full-output buffers of the head-sharded decode variant, one per rank, each mapped into every
    other rank (pkv_peer_alloc / pkv_peer_open), and the fused attention + exchange call.

    `dist` is an initialised torch.distributed (any backend: it only carries the 64-byte handles and
    a barrier)."""

    def __init__(self, n_tokens: int, q_heads_total: int, head_dim: int, torch_dtype, dist, device):
        import ctypes as C
        import torch
        from . import _lib
        self.torch, self.dist, self.C, self._lib = torch, dist, C, _lib
        self.world, self.rank = dist.get_world_size(), dist.get_rank()
        self.n_tokens, self.q_heads_total, self.head_dim, self.dtype = n_tokens, q_heads_total, head_dim, torch_dtype
        self.out_bytes = n_tokens * q_heads_total * head_dim * 2
        self.flag_off = (self.out_bytes + 255) // 256 * 256
        total = self.flag_off + 256
        L = _lib.lib()
        ptr, handle = C.c_void_p(), (C.c_ubyte * 64)()
        _lib.check("pkv_peer_alloc", L.pkv_peer_alloc(total, C.byref(ptr), handle))
        self._own = ptr.value
        handles = [None] * self.world
        dist.all_gather_object(handles, bytes(handle))
        self._ptrs = []
        for r, h in enumerate(handles):
            if r == self.rank:
                self._ptrs.append(self._own)
            else:
                p = C.c_void_p()
                hb = (C.c_ubyte * 64).from_buffer_copy(h)
                _lib.check("pkv_peer_open", L.pkv_peer_open(hb, C.byref(p)))
                self._ptrs.append(p.value)
        self._out_arr = (C.c_void_p * self.world)(*self._ptrs)
        self._flag_arr = (C.c_void_p * self.world)(*[p + self.flag_off for p in self._ptrs])
        raw = torch.as_tensor(_RawCuda(self._own, total), device=device)
        self.out = raw[:self.out_bytes].view(torch_dtype).view(n_tokens, q_heads_total * head_dim)
        self.flags = raw[self.flag_off:self.flag_off + 4 * (self.world + 1)].view(torch.int32)
        self.epoch = 0
        dist.barrier()

    def attention(self, plan, q_local, k_cache, v_cache, block_tables, table_offset, token_seq, token_pos,
                  block_size: int, scale: float, stream=None, device_epoch: bool = True):
        """plan: a DecodePlan built for the LOCAL head counts.  Returns this rank's full output
        (valid once the stream has run the call).  device_epoch: the calls are counted on the device
        (replayable in a CUDA graph); otherwise the host passes a growing epoch."""
        from .kernels import _ptr, _stream, _suffix
        self.epoch = 0 if device_epoch else self.epoch + 1
        fn = f"pkv_decode_attn_planned_peer_{_suffix(k_cache)}"
        p, n = plan._ws()
        st = getattr(self._lib.lib(), fn)(self.C.byref(plan.plan), _ptr(q_local), _ptr(k_cache), _ptr(v_cache),
                                          _ptr(block_tables), _ptr(table_offset), _ptr(token_seq), _ptr(token_pos),
                                          self._out_arr, self._flag_arr, self.world, self.rank, self.epoch,
                                          self.q_heads_total, block_size, self.C.c_float(scale), p, n, _stream(stream))
        self._lib.check(fn, st)
        return self.out

    def close(self):
        self.torch.cuda.synchronize()
        self.dist.barrier()
        L = self._lib.lib()
        for r, p in enumerate(self._ptrs):
            if r != self.rank:
                L.pkv_peer_close(p)
        self.dist.barrier()
        L.pkv_peer_free(self._own)
        self._ptrs = []
