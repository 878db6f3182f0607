"""Prefix sharing with copy-on-write, end to end on the GPU against the CPU checker:
children forked from a parent share its full blocks AND its partial last block; the first
divergent append of each child triggers KVCacheManager.cow -> a block copy on every pool ->
the append; a few decode steps follow.  Pools must stay byte-identical to the host mirror
(memcpy semantics) and attention within 2e-2."""
import ctypes

import numpy as np
import pytest

from tests.gpu_util import TOL, cast_like_reference, from_device, rel_errors, to_device

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("fused", [False, True], ids=["append then attention", "append inside the attention launch"])
def test_fork_cow_copy_append_decode(pkv, orc, torch_cuda, fused):
    """fused: the attention launch then fetches the pools' older rows -- the copied blocks among them --
    ahead of its dependency wait; the block copy before it does not release its dependents early."""
    torch = torch_cuda
    rng = np.random.default_rng(77)
    qh, kvh, hd, bs, nb, layers = 32, 4, 64, 16, 96, 3
    kv_dim = kvh * hd
    scale = float(np.float32(1.0) / np.sqrt(np.float32(hd)))
    mgr = pkv.KVCacheManager(nb, bs, True)
    parent = mgr.new_table()
    prompt = rng.integers(0, 1000, size=40).astype(np.int32).tolist()   # 2 full blocks + 8 tokens
    assert mgr.allocate_prompt(parent, prompt) == 0
    mgr.commit_computed(parent, prompt, 40)
    kids = [mgr.new_table() for _ in range(5)]
    for k in kids:
        mgr.fork(parent, k)
    seqs = [parent] + kids
    lens = [40] * len(seqs)

    # host mirror (bf16 bits + widened fp32) and device pools, per layer
    h_bits, h_f32, d_pool = [], [], []
    for _ in range(2 * layers):
        bits, f32 = cast_like_reference(orc, rng.standard_normal((nb * bs, kv_dim), dtype=np.float32), "bf16")
        h_bits.append(bits.copy()); h_f32.append(f32.copy()); d_pool.append(to_device(torch, bits, "bf16"))
    ptrs = torch.tensor([p.data_ptr() for p in d_pool], dtype=torch.int64, device="cuda")
    copyf = orc.lib.orc_copy_blocks
    copyf.restype = None
    copyf.argtypes = [ctypes.c_void_p] * 3 + [ctypes.c_int, ctypes.c_size_t]

    for step in range(4):
        # bookkeeping: copy-on-write first, then room for the new token
        pairs = []
        for t, L in zip(seqs, lens):
            r = mgr.cow(t, L)
            assert r is not None
            if r[0] >= 0:
                pairs.append(r)
            assert mgr.ensure_slot(t, L + 1)
        if step == 0:
            assert len(pairs) == 5 and len({d for _, d in pairs}) == 5      # the last owner writes in place
        else:
            assert not pairs
        if pairs:
            pa = np.asarray(pairs, dtype=np.int32)
            pkv.launch_copy_blocks_layers(ptrs, 2 * layers, torch.from_numpy(pa).cuda(), len(pairs), bs * kv_dim * 2)
            for l in range(layers):
                copyf(h_bits[2 * l].ctypes.data, h_bits[2 * l + 1].ctypes.data, pa.ctypes.data, len(pairs), bs * kv_dim * 2)
                copyf(h_f32[2 * l].ctypes.data, h_f32[2 * l + 1].ctypes.data, pa.ctypes.data, len(pairs), bs * kv_dim * 4)
        idx = pkv.pack_step([t.blocks for t in seqs], lens, bs, tok_keys=list(range(len(seqs))))
        N = idx.n_tokens
        i32 = lambda a: torch.from_numpy(np.ascontiguousarray(a, dtype=np.int32)).cuda()
        d_idx = [i32(idx.block_tables), i32(idx.table_offset), i32(idx.token_seq), i32(idx.token_pos)]
        plan = pkv.DecodePlan(N, qh, kvh, hd).build_host(idx.token_pos)
        for l in range(layers):
            qb, qf = cast_like_reference(orc, rng.standard_normal((N, qh * hd), dtype=np.float32), "bf16")
            kb, kf = cast_like_reference(orc, rng.standard_normal((N, kv_dim), dtype=np.float32), "bf16")
            vb, vf = cast_like_reference(orc, rng.standard_normal((N, kv_dim), dtype=np.float32), "bf16")
            out = torch.zeros((N, qh * hd), dtype=torch.bfloat16, device="cuda")
            if fused:
                plan.append_attention(to_device(torch, qb, "bf16"), to_device(torch, kb, "bf16"), to_device(torch, vb, "bf16"),
                                      i32(idx.slots), d_pool[2 * l], d_pool[2 * l + 1], *d_idx, out, bs, scale)
            else:
                pkv.launch_store_kv(to_device(torch, kb, "bf16"), to_device(torch, vb, "bf16"), i32(idx.slots),
                                    d_pool[2 * l], d_pool[2 * l + 1], N, kv_dim)
                plan.attention(to_device(torch, qb, "bf16"), d_pool[2 * l], d_pool[2 * l + 1], *d_idx, out, bs, scale)
            orc.append(kb, vb, idx.slots, h_bits[2 * l], h_bits[2 * l + 1])
            orc.append(kf, vf, idx.slots, h_f32[2 * l], h_f32[2 * l + 1])
            want = orc.paged_attention(qf, h_f32[2 * l], h_f32[2 * l + 1], idx.block_tables, idx.table_offset,
                                       idx.token_seq, idx.token_pos, qh, kvh, hd, bs, scale, threads=4)
            torch.cuda.synchronize()
            _, got = from_device(torch, orc, out, "bf16")
            e_ref, e_row = rel_errors(got.reshape(-1, hd), want.reshape(-1, hd))
            assert e_row <= TOL["bf16"], (step, l, e_ref, e_row)
        lens = [L + 1 for L in lens]
    for l in range(2 * layers):
        bits, _ = from_device(torch, orc, d_pool[l], "bf16")
        assert np.array_equal(bits, h_bits[l]), f"pool {l} differs from the host mirror"
    # children share the two full prefix blocks with the parent, and nothing else
    for k in kids:
        assert k.blocks[:2].tolist() == parent.blocks[:2].tolist() and k.blocks[2] != parent.blocks[2]
    assert mgr.ref_count(int(parent.blocks[0])) == 6 and mgr.ref_count(int(parent.blocks[2])) == 1
