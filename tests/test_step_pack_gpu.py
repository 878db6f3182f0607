"""GPU parity for the device-side step-index build (pkv_step_pack_device): its outputs must be
the CPU checker's orc_step_pack outputs, integer for integer, for the same packed tokens."""
import ctypes

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def oracle_pack(orc, tables, slices, bs):
    """tables: {row: int32 array}; slices: [(row, start, len)] -> dict of numpy arrays."""
    tok_tabs, tok_pos, keys = [], [], []
    for row, start, n in slices:
        for i in range(n):
            tok_tabs.append(tables[row]); tok_pos.append(start + i); keys.append(row)
    n = len(tok_pos)
    karr = np.asarray(keys, dtype=np.uint64)
    ptrs = (ctypes.c_void_p * max(n, 1))(*[t.ctypes.data for t in tok_tabs])
    nblk = np.asarray([t.size for t in tok_tabs], dtype=np.int32)
    pos = np.asarray(tok_pos, dtype=np.int32)
    slots = np.zeros(max(n, 1), np.int32); tseq = np.zeros(max(n, 1), np.int32)
    tabs = np.zeros(max(sum(t.size for t in tables.values()), 1), np.int32); off = np.zeros(max(len(tables), 1), np.int32)
    ntab = ctypes.c_int(0)
    f = orc.lib.orc_step_pack
    f.restype = ctypes.c_int
    f.argtypes = [ctypes.c_int] + [ctypes.c_void_p] * 4 + [ctypes.c_int] + [ctypes.c_void_p] * 5
    nseq = f(n, karr.ctypes.data, ctypes.cast(ptrs, ctypes.c_void_p), nblk.ctypes.data, pos.ctypes.data, bs,
             slots.ctypes.data, tseq.ctypes.data, tabs.ctypes.data, off.ctypes.data, ctypes.byref(ntab))
    assert nseq >= 0
    return dict(n=n, pos=pos, slots=slots[:n], token_seq=tseq[:n], tables=tabs[:ntab.value], table_offset=off[:nseq])


def check(packer, want, n_tokens):
    c = packer.counts.cpu().numpy()
    assert c.tolist() == [want["n"], want["table_offset"].size, want["tables"].size, 0]
    assert n_tokens == want["n"]
    n = want["n"]
    assert np.array_equal(packer.positions[:n].cpu().numpy(), want["pos"])
    assert np.array_equal(packer.token_seq[:n].cpu().numpy(), want["token_seq"])
    assert np.array_equal(packer.slots[:n].cpu().numpy(), want["slots"])
    assert np.array_equal(packer.tables[:want["tables"].size].cpu().numpy(), want["tables"])
    assert np.array_equal(packer.table_offset[:want["table_offset"].size].cpu().numpy(), want["table_offset"])


@pytest.mark.parametrize("bs", [16, 32, 24])
def test_mixed_step_matches_checker(pkv, orc, torch_cuda, bs):
    rng = np.random.default_rng(40 + bs)
    rows = 64
    packer = pkv.DeviceStepPacker(rows, 48, bs, max_tokens=4096, max_table_entries=rows * 48)
    tables = {r: rng.permutation(5000)[:int(rng.integers(1, 48))].astype(np.int32) for r in range(0, rows, 2)}
    for r, t in tables.items():
        packer.set_table(r, t)
    # prefill slices, decode tokens, one sequence revisited by two slices, rows out of order
    order = list(tables)
    rng.shuffle(order)
    slices = []
    for r in order[:20] + order[3:5]:
        cap = tables[r].size * bs
        n = int(rng.integers(1, min(cap, 70) + 1)) if rng.random() < 0.5 else 1
        slices.append((r, int(rng.integers(0, cap - n + 1)), n))
    n = packer.pack(slices)
    check(packer, oracle_pack(orc, tables, slices, bs), n)


def test_tables_follow_the_sequences_from_step_to_step(pkv, orc, torch_cuda):
    """Decode steps: every step each sequence advances by one token, now and then needs a new
    block, and sequences finish (row released) and start (row reused with a new table)."""
    rng = np.random.default_rng(77)
    bs, rows = 16, 32
    packer = pkv.DeviceStepPacker(rows, 64, bs, max_tokens=rows, max_table_entries=rows * 64)
    free_blocks = list(rng.permutation(20000).astype(np.int32))
    tables, length = {}, {}
    for step in range(40):
        for r in range(rows):
            if r not in tables and rng.random() < 0.3:                     # a new sequence takes the row
                length[r] = int(rng.integers(1, 200))
                nb = (length[r] + bs) // bs                                # room for position length[r]
                tables[r] = np.array([free_blocks.pop() for _ in range(nb)], dtype=np.int32)
                packer.release(r)
                packer.set_table(r, tables[r])
        slices = []
        for r in sorted(tables, key=lambda x: (x * 7) % rows):
            pos = length[r]
            if pos // bs >= tables[r].size:                                # ensure_slot: one more block
                b = free_blocks.pop()
                packer.set_block(r, tables[r].size, int(b))
                tables[r] = np.append(tables[r], b).astype(np.int32)
            slices.append((r, pos, 1))
            length[r] += 1
        n = packer.pack(slices)
        check(packer, oracle_pack(orc, tables, slices, bs), n)
        for r in list(tables):
            if length[r] > 900 or rng.random() < 0.05:                      # finished
                packer.release(r)
                del tables[r], length[r]


def test_full_size_steps(pkv, orc, torch_cuda, workloads):
    """Configuration 3 (256 decode tokens over long tables) and configuration 4 (32 chunks of 512)."""
    for name in ("cfg3", "cfg4"):
        w = workloads.make(name)
        S = len(w.tables)
        stride = max(t.size for t in w.tables)
        packer = pkv.DeviceStepPacker(S, stride, w.block_size, max_tokens=int(w.new.sum()),
                                      max_table_entries=int(sum(t.size for t in w.tables)))
        tables = {s: np.ascontiguousarray(w.tables[s], dtype=np.int32) for s in range(S)}
        for s, t in tables.items():
            packer.set_table(s, t)
        slices = [(s, int(w.ctx[s]), int(w.new[s])) for s in range(S)]
        n = packer.pack(slices)
        check(packer, oracle_pack(orc, tables, slices, w.block_size), n)


def test_problems_are_reported_in_the_status_word(pkv, torch_cuda):
    bs = 16
    packer = pkv.DeviceStepPacker(4, 8, bs, max_tokens=16, max_table_entries=8)
    packer.set_table(0, [5, 6])
    packer.pack([(0, 31, 1)], check=True)                 # last position of the second block: fine
    with pytest.raises(RuntimeError, match="status bits 4"):
        packer.pack([(0, 32, 1)], check=True)             # needs a third block
    with pytest.raises(RuntimeError, match="status bits 2"):
        packer.pack([(0, 0, 17)], check=True)             # more tokens than the arrays hold
    packer.set_table(1, list(range(8)))
    with pytest.raises(RuntimeError, match="status bits 1"):
        packer.pack([(0, 0, 1), (1, 0, 1)], check=True)   # 2 + 8 table entries, capacity 8
    with pytest.raises(RuntimeError, match="status bits 8"):
        packer.pack([(7, 0, 1)], check=True)              # no such row
    assert packer.pack([], check=True) == 0
    assert packer.counts.cpu().numpy().tolist() == [0, 0, 0, 0]
