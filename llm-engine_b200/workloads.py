"""Seeded synthetic workloads with the shapes of the five benchmark configurations.

No dataset is involved: context lengths, block tables and tensor values are drawn
from a numpy Generator (PCG64) seeded per configuration; values are N(0, 1).  Block
tables are fragmented on purpose: the pool's block ids are shuffled and dealt to
sequences in that order, so consecutive logical blocks are never neighbours.
"""
from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np


@dataclass
class Workload:
    name: str
    layers: int
    q_heads: int
    kv_heads: int
    head_dim: int
    block_size: int
    num_blocks: int
    dtype: str                      # "f32" | "bf16" | "f16"
    ctx: np.ndarray                 # cached tokens per sequence before this step
    new: np.ndarray                 # new tokens per sequence in this step (1 = decode)
    tables: list = field(default_factory=list)   # per-sequence int32 block ids
    seed: int = 0
    shared_prefix_blocks: int = 0   # leading blocks shared by every sequence (cfg5)

    @property
    def n_seqs(self) -> int:
        return int(self.ctx.shape[0])

    @property
    def kv_dim(self) -> int:
        return self.kv_heads * self.head_dim

    @property
    def elem_bytes(self) -> int:
        return 4 if self.dtype == "f32" else 2

    @property
    def scale(self) -> float:
        return 1.0 / float(np.sqrt(np.float32(self.head_dim)))

    def pool_bytes_per_layer(self) -> int:
        return 2 * self.num_blocks * self.block_size * self.kv_dim * self.elem_bytes

    # ---- packed step (one token row per new token) -------------------------
    def step_tokens(self):
        """(tok_tables, tok_pos, tok_seq_index): packed tokens in sequence order."""
        tabs, pos, seq = [], [], []
        for s in range(self.n_seqs):
            for i in range(int(self.new[s])):
                tabs.append(self.tables[s])
                pos.append(int(self.ctx[s]) + i)
                seq.append(s)
        return tabs, np.asarray(pos, dtype=np.int32), np.asarray(seq, dtype=np.int32)

    # ---- algorithmic work -------------------------------------------------
    def decode_bytes_per_layer(self) -> int:
        """K and V read once per kv head, q read, out written, block table and the
        three per-token index arrays: sum_s 2 L_s Hkv D E + 2 N Hq D E + sum_s 4 ceil(L_s/bs) + 12 N."""
        L = (self.ctx + self.new).astype(np.int64)
        n = int(self.new.sum())
        e = self.elem_bytes
        kv = int((2 * L * self.kv_heads * self.head_dim * e).sum())
        qo = 2 * n * self.q_heads * self.head_dim * e
        tbl = int((4 * ((L + self.block_size - 1) // self.block_size)).sum())
        return kv + qo + tbl + 12 * n

    def append_bytes_per_layer(self) -> int:
        n = int(self.new.sum())
        return 4 * n * self.kv_dim * self.elem_bytes + 4 * n

    def prefill_flops_per_layer(self) -> int:
        """QK^T and PV over unmasked (query, key) pairs: 4 D Hq sum_s [C P_s + C (C+1)/2]."""
        C = self.new.astype(np.int64)
        P = self.ctx.astype(np.int64)
        return int((4 * self.head_dim * self.q_heads * (C * P + C * (C + 1) // 2)).sum())

    def prefill_bytes_per_layer(self) -> int:
        L = (self.ctx + self.new).astype(np.int64)
        n = int(self.new.sum())
        e = self.elem_bytes
        return int((2 * L * self.kv_heads * self.head_dim * e).sum()) + 2 * n * self.q_heads * self.head_dim * e


def _deal_tables(rng, num_blocks, blocks_per_seq, shared_prefix_blocks=0):
    perm = rng.permutation(num_blocks).astype(np.int32)
    need = int(sum(blocks_per_seq)) + shared_prefix_blocks
    if need > num_blocks:
        raise ValueError(f"workload needs {need} blocks, pool has {num_blocks}")
    shared = perm[:shared_prefix_blocks]
    at = shared_prefix_blocks
    tables = []
    for nb in blocks_per_seq:
        tables.append(np.concatenate([shared, perm[at:at + nb]]).astype(np.int32))
        at += nb
    return tables


def _blocks_for(tokens, bs):
    return (np.asarray(tokens, dtype=np.int64) + bs - 1) // bs


def make(name: str, seed: int | None = None, n_seqs: int | None = None, layers: int | None = None,
         num_blocks: int | None = None, extra_tokens: int = 0, dtype: str | None = None) -> Workload:
    """Build configuration `name` in {"cfg1".."cfg5"}.  n_seqs / layers / num_blocks shrink
    it for tests; extra_tokens reserves table room for that many further decode steps."""
    idx = int(name[-1])
    rng = np.random.default_rng(1234 + idx if seed is None else seed)
    bs = 16
    if name == "cfg1":      # one Qwen2.5-0.5B attention layer, fp32, 8 seqs, ctx U[64,512]
        S = n_seqs or 8
        ctx = rng.integers(64, 513, size=S)
        w = Workload(name, layers or 1, 14, 2, 64, bs, num_blocks or 4096, dtype or "f32", ctx, np.ones(S, dtype=np.int64))
    elif name == "cfg2":    # Qwen2.5-0.5B decode step, 24 layers, bf16, 64 seqs, ctx U[256,2048]
        S = n_seqs or 64
        ctx = rng.integers(256, 2049, size=S)
        w = Workload(name, layers or 24, 14, 2, 64, bs, num_blocks or 16384, dtype or "bf16", ctx, np.ones(S, dtype=np.int64))
    elif name == "cfg3":    # TinyLlama decode, 22 layers, bf16, 256 seqs, ctx log-uniform [128,8192]
        S = n_seqs or 256
        ctx = np.exp(rng.uniform(np.log(128.0), np.log(8192.0), size=S)).astype(np.int64)
        ctx = np.clip(ctx, 128, 8192)
        w = Workload(name, layers or 22, 32, 4, 64, bs, num_blocks or 65536, dtype or "bf16", ctx, np.ones(S, dtype=np.int64))
    elif name == "cfg4":    # chunked prefill, Qwen shapes, bf16, 32 seqs, prior U[0,1536], chunk 512
        S = n_seqs or 32
        ctx = rng.integers(0, 1537, size=S)
        w = Workload(name, layers or 1, 14, 2, 64, bs, num_blocks or 8192, dtype or "bf16", ctx, np.full(S, 512, dtype=np.int64))
    elif name == "cfg5":    # prefix cache: TinyLlama shapes, 128 seqs share 512 tokens, suffix U[32,256]
        S = n_seqs or 128
        suffix = rng.integers(32, 257, size=S)
        ctx = 512 + suffix
        w = Workload(name, layers or 22, 32, 4, 64, bs, num_blocks or 8192, dtype or "bf16", ctx, np.ones(S, dtype=np.int64),
                     shared_prefix_blocks=32)
    else:
        raise ValueError(name)
    w.ctx = w.ctx.astype(np.int64)
    w.seed = 1234 + idx if seed is None else seed
    total = w.ctx + w.new + extra_tokens
    if w.shared_prefix_blocks:
        own = _blocks_for(total, bs) - w.shared_prefix_blocks
        w.tables = _deal_tables(rng, w.num_blocks, own, w.shared_prefix_blocks)
    else:
        w.tables = _deal_tables(rng, w.num_blocks, _blocks_for(total, bs))
    return w
