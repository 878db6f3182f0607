"""The golden engine trace (steps built by the reference's own Scheduler + KVCacheManager), checked on CPU:
the product's step packing accepts every step, and a cache driven by those steps is read-your-writes
consistent -- every position a token attends holds the content that position should have, including
positions it never wrote itself (prefix-cache hits) and positions rewritten after a preemption."""
import numpy as np

from tests.engine_trace_util import EngineTrace


def test_trace_shape_and_scheduler_behaviour():
    tr = EngineTrace()
    assert tr.bs == 16 and len(tr.steps) == tr.stats[0] == 320
    assert tr.stats[1] >= 3                      # preemptions happened: recompute-on-resume is exercised
    lens = [ln for st in tr.steps for _, _, ln, _ in st]
    starts = [s for st in tr.steps for _, s, ln, _ in st if ln > 1]
    assert max(lens) == tr.chunk and sum(1 for x in lens if x == 1) > 1000
    assert any(s > 0 and s % tr.chunk for s in starts)          # a prefill that starts at a cached prefix or resumes mid-way
    for st in tr.steps:                                          # prefill slices first, then decode (sequence.h:74-89)
        kinds = [ln > 1 for _, _, ln, _ in st]
        assert sum(ln for _, _, ln, _ in st) <= tr.budget and len(st) <= tr.max_seqs
        assert kinds == sorted(kinds, reverse=True) or all(k is False for k in kinds)


def test_cache_driven_by_the_trace_is_read_your_writes_consistent(pkv):
    tr = EngineTrace()
    held = np.zeros(tr.num_blocks * tr.bs, dtype=np.uint64)       # content key currently stored in every slot
    shared_reads = 0
    for s in range(len(tr.steps)):
        tabs, pos, sid, keys = tr.packed(s)
        idx = pkv.pack_step(tabs, pos, tr.bs, tok_keys=sid.tolist())
        assert idx.n_tokens == pos.size
        # append: a slot written twice in one step must get the same content (it never happens with distinct sequences)
        order = np.argsort(idx.slots, kind="stable")
        dup = idx.slots[order][1:] == idx.slots[order][:-1]
        assert np.array_equal(keys[order][1:][dup], keys[order][:-1][dup])
        held[idx.slots] = keys
        # attention: token at position p of its sequence reads positions 0..p through the table it was given
        for seq, start, ln, table in tr.steps[s]:
            p_last = start + ln - 1
            slots = table[np.arange(p_last + 1) // tr.bs].astype(np.int64) * tr.bs + np.arange(p_last + 1) % tr.bs
            assert np.array_equal(held[slots], tr.keys[seq][:p_last + 1]), (s, seq)
            if start > 0 and ln > 1:
                shared_reads += start
    assert shared_reads > 0
