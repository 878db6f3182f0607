"""Pins the CPU checkers before anything is compared with them.

1. known-answer values held by the reference's own unit tests
   (tests/test_tensor.cpp:7-33, tests/test_block_allocator.cpp:39),
2. the committed golden fixtures, generated from the reference's compiled sources
   (tests/golden/make_golden.py),
3. where oracle/_ref/libpkv_ref.so is present, bit-for-bit agreement between the C
   restatement and the reference's own code on fresh seeded inputs.
"""
import json
import math
import os
import struct

import numpy as np
import pytest

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def f32_from_bits(b):
    return struct.unpack("<f", struct.pack("<I", b))[0]


# ---- 1. the reference's own known answers ------------------------------------------
def test_f16_round_trip_on_representable_values(orc):
    for f in (0.0, 1.0, -1.0, 0.5, 65504.0, -65504.0, 6.103515625e-05, 5.960464477539063e-08, 3.140625):
        assert orc.f16_to_f32(orc.f32_to_f16(f)) == f


def test_f16_known_bit_patterns(orc):
    assert orc.f32_to_f16(1.0) == 0x3C00
    assert orc.f32_to_f16(-2.0) == 0xC000
    assert orc.f32_to_f16(65504.0) == 0x7BFF
    assert orc.f32_to_f16(1e5) == 0x7C00
    assert orc.f16_to_f32(0x0001) == 5.960464477539063e-08
    assert math.isnan(orc.f16_to_f32(0x7E00))


def test_f16_rounds_to_nearest_even(orc):
    assert orc.f32_to_f16(1.0 + 0.00048828125) == 0x3C00
    assert orc.f32_to_f16(1.0 + 3 * 0.00048828125) == 0x3C02


def test_bf16_round_trip(orc):
    for f in (0.0, 1.0, -1.0, 3.125, 1024.0, -0.375):
        assert orc.bf16_to_f32(orc.f32_to_bf16(f)) == f
    assert orc.f32_to_bf16(1.0) == 0x3F80
    assert orc.bf16_to_f32(0x4049) == 3.140625


def test_slot_arithmetic(orc):
    blocks = np.asarray([7, 3, 9], dtype=np.int32)
    assert orc.slot(blocks, 5, 4) == 3 * 4 + 1          # tests/test_block_allocator.cpp:39
    assert orc.slot(blocks, 0, 16) == 7 * 16
    assert orc.slot(blocks, 47, 16) == 9 * 16 + 15


# ---- 2. golden fixtures ---------------------------------------------------------------
def test_casts_match_golden(orc):
    g = json.load(open(os.path.join(GOLD, "casts.json")))
    for rec in g["to"]:
        x = f32_from_bits(rec["f32_bits"])
        assert orc.f32_to_bf16(x) == rec["bf16"], hex(rec["f32_bits"])
        assert orc.f32_to_f16(x) == rec["f16"], hex(rec["f32_bits"])
    for h, bits in g["f16_to_f32"].items():
        got = np.float32(orc.f16_to_f32(int(h))).view(np.uint32)
        assert int(got) == bits
    for h, bits in g["bf16_to_f32"].items():
        assert int(np.float32(orc.bf16_to_f32(int(h))).view(np.uint32)) == bits


def test_array_casts_match_scalar(orc):
    x = np.random.default_rng(3).standard_normal(257).astype(np.float32)
    assert orc.to_bf16_bits(x).tolist() == [orc.f32_to_bf16(float(v)) for v in x]
    assert orc.to_f16_bits(x).tolist() == [orc.f32_to_f16(float(v)) for v in x]
    # numpy's own float16 cast is IEEE round-to-nearest-even as well
    assert np.array_equal(orc.to_f16_bits(x), x.astype(np.float16).view(np.uint16))
    assert np.array_equal(orc.from_f16_bits(x.astype(np.float16).view(np.uint16)), x.astype(np.float16).astype(np.float32))


@pytest.mark.parametrize("name", ["attn_qwen_f32", "attn_tiny_f32"])
def test_attention_matches_golden_bit_for_bit(orc, name):
    g = np.load(os.path.join(GOLD, name + ".npz"))
    qh, kvh, hd, bs, nb = (int(x) for x in g["geometry"])
    kc, vc = g["k_cache"].copy(), g["v_cache"].copy()
    slots = np.asarray([orc.slot(g["block_tables"][g["table_offset"][s]:], int(p), bs)
                        for s, p in zip(g["token_seq"], g["token_pos"])], dtype=np.int32)
    assert np.array_equal(slots, g["slots"])
    orc.append(g["k"], g["v"], slots, kc, vc)
    for threads in (1, 3):
        out = orc.paged_attention(g["q"], kc, vc, g["block_tables"], g["table_offset"], g["token_seq"],
                                  g["token_pos"], qh, kvh, hd, bs, float(g["scale"]), threads=threads)
        assert np.array_equal(out.view(np.uint32), g["out"].view(np.uint32))


def _replay(trace, make_mgr):
    """Replays the golden allocator trace; yields (op record, manager, live tables)."""
    mgr = make_mgr(trace["num_blocks"], trace["block_size"], trace["prefix"])
    live = {}
    for rec in trace["ops"]:
        op = rec["op"]
        if op == "allocate_prompt":
            bt = mgr.new_table()
            res = mgr.allocate_prompt(bt, rec["tokens"])
            assert res == rec["result"]
            if res is not None:
                live[rec["id"]] = [bt, list(rec["tokens"])]
        elif op == "ensure_slot":
            bt, toks = live[rec["id"]]
            ok = mgr.ensure_slot(bt, len(toks) + 1)
            assert ok == rec["result"]
            if ok:
                toks.append(rec["token"])
        elif op == "commit_computed":
            bt, toks = live[rec["id"]]
            mgr.commit_computed(bt, toks, rec["num_computed"])
        else:
            bt, _ = live.pop(rec["id"])
            mgr.free(bt)
        yield rec, mgr, live


def check_allocator_state(rec, mgr, live, count):
    st = rec["state"]
    assert mgr.lookup_cached_prefix(rec["probe"]) == rec["probe_hit"]
    assert count(mgr, "free") == st["free"] and count(mgr, "cached") == st["cached"] and count(mgr, "used") == st["used"]
    stats = mgr.stats() if callable(mgr.stats) else mgr.stats
    assert stats == st["stats"]
    assert sorted(live) == sorted(int(k) for k in st["tables"])
    for sid, (bt, _) in live.items():
        want = st["tables"][str(sid)]
        assert [int(b) for b in bt.blocks] == want["blocks"]
        assert [str(int(h)) for h in bt.hashes] == want["hashes"]
        assert bt.num_committed == want["num_committed"]


def test_python_allocator_restatement_matches_golden_trace():
    from oracle import kv_oracle
    trace = json.load(open(os.path.join(GOLD, "allocator_trace.json")))
    count = lambda m, what: getattr(m, f"num_{what}_blocks")
    for rec, mgr, live in _replay(trace, kv_oracle.Allocator):
        check_allocator_state(rec, mgr, live, count)


def test_hash_block_matches_golden_and_python(orc):
    from oracle import kv_oracle
    trace = json.load(open(os.path.join(GOLD, "allocator_trace.json")))
    bs = trace["block_size"]
    seen = 0
    for rec in trace["ops"]:
        for sid, t in rec["state"]["tables"].items():
            pass
        if rec["op"] != "allocate_prompt":
            continue
        toks = rec["tokens"]
        prev = 0
        for i in range(len(toks) // bs):
            h = orc.hash_block(prev, toks[i * bs:(i + 1) * bs])
            assert h == kv_oracle.hash_block(prev, toks[i * bs:(i + 1) * bs])
            prev = h
            seen += 1
    assert seen > 100
    assert orc.hash_block(0, []) == kv_oracle.hash_block(0, [])


# ---- 3. against the reference's compiled sources, where present ---------------------
def test_restatement_equals_compiled_reference(orc, ref):
    if ref is None:
        pytest.skip("oracle/_ref/libpkv_ref.so not built (reference tree absent)")
    rng = np.random.default_rng(99)
    x = np.concatenate([rng.standard_normal(4096).astype(np.float32) * s for s in (1.0, 1e-5, 1e4, 7e4)])
    assert np.array_equal(orc.to_bf16_bits(x), ref.to_bf16_bits(x))
    assert np.array_equal(orc.to_f16_bits(x), ref.to_f16_bits(x))
    h = np.arange(0, 65536, dtype=np.uint16)
    assert np.array_equal(orc.from_f16_bits(h).view(np.uint32), ref.from_f16_bits(h).view(np.uint32))
    assert np.array_equal(orc.from_bf16_bits(h).view(np.uint32), ref.from_bf16_bits(h).view(np.uint32))
    for _ in range(50):
        toks = rng.integers(-5, 50000, size=int(rng.integers(0, 40))).astype(np.int32)
        prev = int(rng.integers(0, 2 ** 63))
        assert orc.hash_block(prev, toks) == ref.hash_block(prev, toks)
    # attention on a fragmented pool, odd geometry included
    for (qh, kvh, hd, bs) in [(14, 2, 64, 16), (32, 4, 64, 16), (6, 3, 40, 4), (4, 4, 128, 8)]:
        nb = 40
        kc = rng.standard_normal((nb * bs, kvh * hd), dtype=np.float32)
        vc = rng.standard_normal((nb * bs, kvh * hd), dtype=np.float32)
        perm = rng.permutation(nb).astype(np.int32)
        lens = [1, bs - 1, bs, bs + 1, 3 * bs + 2]
        tables, at = [], 0
        for L in lens:
            n = (L + bs - 1) // bs
            tables.append(perm[at:at + n])
            at += n
        bt = np.concatenate(tables)
        to = np.cumsum([0] + [t.size for t in tables[:-1]]).astype(np.int32)
        ts = np.arange(len(lens), dtype=np.int32)
        tp = np.asarray([L - 1 for L in lens], dtype=np.int32)
        q = rng.standard_normal((len(lens), qh * hd), dtype=np.float32)
        scale = float(np.float32(1.0) / np.sqrt(np.float32(hd)))
        a = orc.paged_attention(q, kc, vc, bt, to, ts, tp, qh, kvh, hd, bs, scale, threads=2)
        b = ref.paged_attention(q, kc, vc, bt, to, ts, tp, qh, kvh, hd, bs, scale, threads=2)
        assert np.array_equal(a.view(np.uint32), b.view(np.uint32))


def test_python_allocator_equals_compiled_reference_on_random_traces(ref):
    if ref is None:
        pytest.skip("oracle/_ref/libpkv_ref.so not built (reference tree absent)")
    import oracle
    from oracle import kv_oracle
    from tests.test_kv_cache import random_trace_compare
    random_trace_compare(lambda nb, bs, p: oracle.ref_allocator(nb, bs, p), kv_oracle.Allocator, seeds=range(6))


def test_rope_restatement_equals_compiled_reference(orc, ref):
    """RoPE tables (include/engine/ops.h:34-51) and rotate_half rotation (ops.h:56-68), bit for bit."""
    if ref is None:
        pytest.skip("oracle/_ref/libpkv_ref.so not built (reference tree absent)")
    for hd, theta in ((64, 10000.0), (128, 1000000.0), (6, 500.0)):
        ca, sa = orc.rope_tables(hd, 300, theta)
        cb, sb = ref.rope_tables(hd, 300, theta)
        assert np.array_equal(ca.view(np.uint32), cb.view(np.uint32)) and np.array_equal(sa.view(np.uint32), sb.view(np.uint32))
        x = np.random.default_rng(hd).standard_normal((7, 3 * hd)).astype(np.float32)
        pos = [0, 1, 17, 299, 128, 64, 5]
        a, b = orc.rope(x, 3, hd, pos, ca, sa), ref.rope(x, 3, hd, pos, cb, sb)
        assert np.array_equal(a.view(np.uint32), b.view(np.uint32))
    # known answers: position 0 is the identity; a quarter turn swaps the halves with a sign
    c, s = orc.rope_tables(4, 2, 10000.0)
    assert np.array_equal(c[0], np.ones(2, np.float32)) and np.array_equal(s[0], np.zeros(2, np.float32))
    x = np.asarray([[1.0, 2.0, 3.0, 4.0]], dtype=np.float32)
    assert np.array_equal(orc.rope(x, 1, 4, [0], c, s), x)
    c90, s90 = np.zeros((1, 2), np.float32), np.ones((1, 2), np.float32)
    assert orc.rope(x, 1, 4, [0], c90, s90).tolist() == [[-3.0, -4.0, 1.0, 2.0]]
