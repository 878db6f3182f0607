"""Reader for tests/golden/engine_trace.npz: the steps llm-engine's own Scheduler and KVCacheManager
(compiled from its sources by oracle/Makefile; generator: tests/golden/make_golden.py) built for a
small serving run -- chunked prefill, decode, prefix-cache hits, preemption with recompute."""
import os

import numpy as np

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def content_keys(tokens):
    """key[p] stands for the content of positions 0..p of a sequence (what K/V at p depend on in a real
    model); sequences with a common prefix share the keys of that prefix."""
    keys = np.empty(len(tokens), dtype=np.uint64)
    k = 0
    for p, t in enumerate(tokens):
        k = (k * 6364136223846793005 + int(t) + 1442695040888963407) & 0xFFFFFFFFFFFFFFFF
        keys[p] = k
    return keys


class EngineTrace:
    def __init__(self):
        t = np.load(os.path.join(GOLD, "engine_trace.npz"))
        self.bs, self.num_blocks, self.max_seqs, self.budget, self.chunk = (int(x) for x in t["geometry"])
        self.stats = [int(x) for x in t["scheduler_stats"]]       # steps, preemptions, admitted, finished
        so, to = t["slice_offset"], t["table_offset"]
        self.keys = [content_keys(t["seq_tokens"][a:b]) for a, b in zip(t["seq_token_offset"][:-1], t["seq_token_offset"][1:])]
        self.steps = []
        for s in range(so.size - 1):
            sl = []
            for i in range(int(so[s]), int(so[s + 1])):
                sl.append((int(t["slice_seq"][i]), int(t["slice_start"][i]), int(t["slice_len"][i]),
                           t["tables"][int(to[i]):int(to[i + 1])].astype(np.int32)))
            self.steps.append(sl)

    def packed(self, step):
        """(tok_tables, tok_pos, tok_seq_ids, tok_keys) of one step, slice after slice as the engine packs them
        (src/model/cuda/cuda_model.cu:434-447)."""
        tabs, pos, sid, keys = [], [], [], []
        for seq, start, ln, table in self.steps[step]:
            for p in range(start, start + ln):
                tabs.append(table)
                pos.append(p)
                sid.append(seq)
                keys.append(self.keys[seq][p])
        return tabs, np.asarray(pos, np.int32), np.asarray(sid, np.int64), np.asarray(keys, np.uint64)


def rows_from_keys(keys, width, salt):
    """Deterministic fp32 rows in [-1.7, 1.7) from 64-bit content keys: the K, V or q row of a token is a
    function of its content only, so a recomputed or prefix-shared position gets the same values."""
    k = np.asarray(keys, dtype=np.uint64)[:, None] + np.full(1, salt, dtype=np.uint64) * np.uint64(0x9E3779B97F4A7C15)   # arrays wrap modulo 2^64
    x = k + np.arange(1, width + 1, dtype=np.uint64)[None, :] * np.uint64(0xBF58476D1CE4E5B9)
    x ^= x >> np.uint64(30)
    x *= np.uint64(0xBF58476D1CE4E5B9)
    x ^= x >> np.uint64(27)
    x *= np.uint64(0x94D049BB133111EB)
    x ^= x >> np.uint64(31)
    return ((x >> np.uint64(40)).astype(np.float32) / np.float32(1 << 23) - np.float32(1.0)) * np.float32(1.7)
