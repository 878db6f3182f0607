"""Generates the committed golden fixtures from the reference's OWN code.

Runs only where oracle/_ref/libpkv_ref.so exists (i.e. where the reference tree was
available to oracle/Makefile).  Usage, from the repository root:
    python tests/golden/make_golden.py
Outputs:
    tests/golden/attn_qwen_f32.npz    one Qwen2.5-0.5B-shaped attention step
    tests/golden/attn_tiny_f32.npz    one TinyLlama-shaped step, mixed decode + chunk tokens
    tests/golden/allocator_trace.json a random KVCacheManager trace with every observable result
    tests/golden/casts.json           bf16 / f16 conversions of edge-case floats
    tests/golden/engine_trace.npz     the steps the reference's own Scheduler builds for a small serving run
                                      (chunked prefill, decode, prefix-cache hits, preemption with recompute):
                                      per step the slices and every slice's block table at that moment
"""
import json
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
import oracle  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))


def content_keys(tokens):
    """key[p] identifies the content of positions 0..p (K/V at p depend on all of them in a real model): two
    sequences with the same first p + 1 tokens -- a shared, cached prefix -- get the same key."""
    keys = np.empty(len(tokens), dtype=np.uint64)
    k = 0
    for p, t in enumerate(tokens):
        k = (k * 6364136223846793005 + int(t) + 1442695040888963407) & 0xFFFFFFFFFFFFFFFF
        keys[p] = k
    return keys


def engine_trace(ref, path, seed=5):
    """Drives engine::Scheduler + engine::KVCacheManager (compiled from the reference's sources) the way
    Engine::step does -- schedule(), run the step, on_step_done(sampled) -- on a pool small enough to force
    preemptions, with prompts that share cached prefixes, and records what the attention path is handed."""
    import ctypes as C
    L = ref.lib
    L.ref_sched_new.restype = C.c_void_p
    L.ref_sched_new.argtypes = [C.c_int] * 6
    for name, args in (("ref_sched_delete", [C.c_void_p]), ("ref_sched_add", [C.c_void_p, C.c_void_p, C.c_int, C.c_int]),
                       ("ref_sched_step", [C.c_void_p] * 5 + [C.c_int]), ("ref_sched_seq_blocks", [C.c_void_p, C.c_int, C.c_void_p, C.c_int]),
                       ("ref_sched_seq_tokens", [C.c_void_p, C.c_int, C.c_void_p, C.c_int]),
                       ("ref_sched_done", [C.c_void_p, C.c_void_p, C.c_int]), ("ref_sched_has_work", [C.c_void_p]),
                       ("ref_sched_stats", [C.c_void_p, C.c_void_p])):
        getattr(L, name).argtypes = args
        getattr(L, name).restype = C.c_int
    rng = np.random.default_rng(seed)
    bs, num_blocks, max_seqs, budget, chunk = 16, 72, 8, 320, 128
    h = L.ref_sched_new(num_blocks, bs, 1, max_seqs, budget, chunk)
    common = rng.integers(0, 30000, size=3 * bs + 5).astype(np.int32)           # a shared system prompt: 3 full blocks + 5
    prompts = []
    for i in range(14):
        n = int(rng.integers(10, 300))
        own = rng.integers(0, 30000, size=n).astype(np.int32)
        prompts.append(np.concatenate([common, own]) if i % 3 == 0 else own)
    arrivals = {0: [0, 1, 2, 3], 2: [4, 5], 5: [6], 9: [7, 8, 9], 15: [10, 11], 22: [12, 13]}   # step -> requests that arrive before it
    max_new = [int(x) for x in rng.integers(60, 260, size=len(prompts))]
    ids = {}
    steps = []
    cap = 64
    a_seq, a_start, a_len, a_log = (np.zeros(cap, np.int32) for _ in range(4))
    step_no = 0
    while step_no < 320:
        for r in arrivals.get(step_no, []):
            ids[r] = L.ref_sched_add(h, prompts[r].ctypes.data, prompts[r].size, max_new[r])
        if not L.ref_sched_has_work(h) and step_no > max(arrivals):
            break
        n = L.ref_sched_step(h, a_seq.ctypes.data, a_start.ctypes.data, a_len.ctypes.data, a_log.ctypes.data, cap)
        assert n <= cap
        if n == 0:
            step_no += 1
            continue
        rec = {"seq": a_seq[:n].copy(), "start": a_start[:n].copy(), "len": a_len[:n].copy(), "tables": []}
        sampled = []
        for i in range(n):
            sid = int(a_seq[i])
            tb = np.zeros(num_blocks, np.int32)
            nb = L.ref_sched_seq_blocks(h, sid, tb.ctypes.data, num_blocks)
            rec["tables"].append(tb[:nb].copy())
            if a_log[i]:
                sampled.append((sid * 7919 + (int(a_start[i]) + int(a_len[i])) * 104729) % 30000)
        steps.append(rec)
        smp = np.asarray(sampled, dtype=np.int32)
        L.ref_sched_done(h, smp.ctypes.data, smp.size)
        step_no += 1
    st = np.zeros(4, np.uint64)
    L.ref_sched_stats(h, st.ctypes.data)
    # every sequence's tokens as they stand at the end (prompt + what was "sampled"): tokens are only ever
    # appended, so the content of positions 0..p at any earlier step is a prefix of this
    seq_tokens = []
    for sid in range(len(ids)):
        tk = np.zeros(4096, np.int32)
        nt = L.ref_sched_seq_tokens(h, sid, tk.ctypes.data, 4096)
        seq_tokens.append(tk[:nt].copy())
    L.ref_sched_delete(h)
    # flatten
    sl_off = np.cumsum([0] + [r["seq"].size for r in steps]).astype(np.int32)
    tb_all = [t for r in steps for t in r["tables"]]
    tb_off = np.cumsum([0] + [t.size for t in tb_all]).astype(np.int32)
    tok_off = np.cumsum([0] + [t.size for t in seq_tokens]).astype(np.int32)
    np.savez_compressed(path, geometry=np.asarray([bs, num_blocks, max_seqs, budget, chunk], dtype=np.int32),
                        slice_offset=sl_off, slice_seq=np.concatenate([r["seq"] for r in steps]),
                        slice_start=np.concatenate([r["start"] for r in steps]), slice_len=np.concatenate([r["len"] for r in steps]),
                        table_offset=tb_off, tables=np.concatenate(tb_all), seq_token_offset=tok_off,
                        seq_tokens=np.concatenate(seq_tokens), scheduler_stats=st)
    toks = int(sum(int(r["len"].sum()) for r in steps))
    print(path, "steps", len(steps), "tokens", toks, "preemptions", int(st[1]), "admitted", int(st[2]), "finished", int(st[3]),
          "bytes", os.path.getsize(path))


def attention_case(ref, path, seed, q_heads, kv_heads, head_dim, bs, num_blocks, seq_ctx, seq_new):
    rng = np.random.default_rng(seed)
    kv_dim = kv_heads * head_dim
    perm = rng.permutation(num_blocks).astype(np.int32)
    tables, at = [], 0
    for c, n in zip(seq_ctx, seq_new):
        nb = (c + n + bs - 1) // bs
        tables.append(perm[at:at + nb].copy())
        at += nb
    kc = rng.standard_normal((num_blocks * bs, kv_dim), dtype=np.float32)
    vc = rng.standard_normal((num_blocks * bs, kv_dim), dtype=np.float32)
    tok_seq, tok_pos = [], []
    for s, (c, n) in enumerate(zip(seq_ctx, seq_new)):
        for i in range(n):
            tok_seq.append(s)
            tok_pos.append(c + i)
    tok_seq = np.asarray(tok_seq, dtype=np.int32)
    tok_pos = np.asarray(tok_pos, dtype=np.int32)
    N = tok_pos.size
    q = rng.standard_normal((N, q_heads * head_dim), dtype=np.float32)
    k = rng.standard_normal((N, kv_dim), dtype=np.float32)
    v = rng.standard_normal((N, kv_dim), dtype=np.float32)
    block_tables = np.concatenate(tables).astype(np.int32)
    table_offset = np.cumsum([0] + [t.size for t in tables[:-1]]).astype(np.int32)
    slots = np.asarray([ref.slot(tables[s], p, bs) for s, p in zip(tok_seq, tok_pos)], dtype=np.int32)
    kc_after, vc_after = kc.copy(), vc.copy()
    ref.append(k, v, slots, kc_after, vc_after)
    scale = np.float32(1.0) / np.sqrt(np.float32(head_dim))
    out = ref.paged_attention(q, kc_after, vc_after, block_tables, table_offset, tok_seq, tok_pos, q_heads,
                              kv_heads, head_dim, bs, float(scale), threads=1)
    np.savez_compressed(path, q=q, k=k, v=v, k_cache=kc, v_cache=vc, block_tables=block_tables,
                        table_offset=table_offset, token_seq=tok_seq, token_pos=tok_pos, slots=slots,
                        geometry=np.asarray([q_heads, kv_heads, head_dim, bs, num_blocks], dtype=np.int32),
                        scale=np.float32(scale), out=out)
    print(path, "tokens", N, "bytes", os.path.getsize(path))


def allocator_trace(path, seed=7, steps=400):
    rng = np.random.default_rng(seed)
    num_blocks, bs = 24, 4
    mgr = oracle.ref_allocator(num_blocks, bs, True)
    live = {}   # id -> (table, tokens)
    ops, next_id = [], 0
    vocab = 5   # tiny vocabulary so prompts collide and prefix hits, duplicates and evictions all occur
    for _ in range(steps):
        r = rng.random()
        rec = None
        if r < 0.35 or not live:
            n = int(rng.integers(1, 22))
            toks = rng.integers(0, vocab, size=n).astype(np.int32)
            if rng.random() < 0.5 and live:   # extend somebody's prompt: guaranteed shared prefix
                base = live[list(live)[int(rng.integers(len(live)))]][1]
                toks = np.concatenate([base[:len(base) // bs * bs], toks]).astype(np.int32)[:40]
            bt = mgr.new_table()
            res = mgr.allocate_prompt(bt, toks)
            rec = {"op": "allocate_prompt", "id": next_id, "tokens": toks.tolist(), "result": res}
            if res is not None:
                live[next_id] = (bt, toks, res)
            next_id += 1
        elif r < 0.6:
            sid = list(live)[int(rng.integers(len(live)))]
            bt, toks, done = live[sid]
            toks = np.append(toks, np.int32(rng.integers(0, vocab))).astype(np.int32)
            ok = mgr.ensure_slot(bt, len(toks))
            rec = {"op": "ensure_slot", "id": sid, "token": int(toks[-1]), "result": ok}
            if ok:
                live[sid] = (bt, toks, done)
        elif r < 0.85:
            sid = list(live)[int(rng.integers(len(live)))]
            bt, toks, done = live[sid]
            cap = min(len(toks), len(bt.blocks) * bs)
            nc = int(rng.integers(done, cap + 1)) if cap >= done else done
            mgr.commit_computed(bt, toks, nc)
            live[sid] = (bt, toks, nc)
            rec = {"op": "commit_computed", "id": sid, "num_computed": nc}
        else:
            sid = list(live)[int(rng.integers(len(live)))]
            bt, toks, done = live.pop(sid)
            mgr.free(bt)
            rec = {"op": "free", "id": sid}
        probe = rng.integers(0, vocab, size=int(rng.integers(0, 13))).astype(np.int32)
        rec["probe"] = probe.tolist()
        rec["probe_hit"] = mgr.lookup_cached_prefix(probe)
        rec["state"] = {"free": mgr.num_free_blocks, "cached": mgr.num_cached_blocks, "used": mgr.num_used_blocks,
                        "stats": mgr.stats,
                        "tables": {str(i): {"blocks": t.blocks, "hashes": [str(h) for h in t.hashes],
                                            "num_committed": t.num_committed} for i, (t, _, _) in live.items()}}
        ops.append(rec)
    with open(path, "w") as f:
        json.dump({"num_blocks": num_blocks, "block_size": bs, "prefix": True, "ops": ops}, f)
    print(path, "ops", len(ops), "bytes", os.path.getsize(path))


def casts(ref, path):
    vals = [0.0, -0.0, 1.0, -1.0, 0.5, 3.140625, 3.14159265, 65504.0, 65520.0, 1e5, -1e5, 6.103515625e-05,
            5.960464477539063e-08, 2.98e-08, 1e-8, 1.0 + 2 ** -11, 1.0 + 3 * 2 ** -11, 1.0 + 2 ** -8, 1.0 + 3 * 2 ** -9,
            1.00390625, 0.1, -0.3333333, 1e38, 3.3e38, float("inf"), float("-inf")]
    rng = np.random.default_rng(11)
    vals += [float(x) for x in rng.standard_normal(64).astype(np.float32)]
    vals += [float(np.float32(x)) for x in (rng.standard_normal(32) * 1e-6)]
    rec = []
    for x in vals:
        x32 = float(np.float32(x))
        rec.append({"f32_bits": int(np.float32(x32).view(np.uint32)), "bf16": ref.f32_to_bf16(x32), "f16": ref.f32_to_f16(x32)})
    back16 = {str(h): int(np.float32(ref.f16_to_f32(h)).view(np.uint32)) for h in
              [0, 1, 0x3ff, 0x400, 0x3c00, 0x7bff, 0x7c00, 0xfc00, 0x8000, 0x8001, 0xc000, 0x0203, 0x7e00 & 0x7dff]}
    backbf = {str(h): int(np.float32(ref.bf16_to_f32(h)).view(np.uint32)) for h in [0, 0x3f80, 0x4049, 0xbf80, 0x7f80, 0x0001, 0x8000]}
    with open(path, "w") as f:
        json.dump({"to": rec, "f16_to_f32": back16, "bf16_to_f32": backbf}, f)
    print(path, "bytes", os.path.getsize(path))


def main():
    ref = oracle.load_ref()
    if ref is None:
        raise SystemExit("oracle/_ref/libpkv_ref.so is missing: run `make -C oracle` where the reference tree exists")
    # Qwen2.5-0.5B geometry: 14 query heads / 2 kv heads (group 7), head_dim 64, block 16; decode tokens only.
    attention_case(ref, os.path.join(HERE, "attn_qwen_f32.npz"), 101, 14, 2, 64, 16, 24,
                   seq_ctx=[70, 15, 32, 47, 1, 0], seq_new=[1, 1, 1, 1, 1, 1])
    # TinyLlama geometry: 32 / 4 (group 8); two decode tokens and two prefill chunks starting mid-block.
    attention_case(ref, os.path.join(HERE, "attn_tiny_f32.npz"), 202, 32, 4, 64, 16, 12,
                   seq_ctx=[33, 5, 16, 0], seq_new=[1, 9, 1, 20])
    allocator_trace(os.path.join(HERE, "allocator_trace.json"))
    casts(ref, os.path.join(HERE, "casts.json"))
    engine_trace(ref, os.path.join(HERE, "engine_trace.npz"))


if __name__ == "__main__":
    main()
