"""The C-ABI library loads without a GPU, exports every symbol include/pkv.h
declares, and rejects bad arguments on the host before touching the device."""
import ctypes as C
import os
import re

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "pkv.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(pkv_[a-z0-9_]+)\s*\(", text)))


def test_every_declared_symbol_is_exported_and_bound(pkv):
    L = pkv.lib()
    names = declared_symbols()
    assert len(names) > 40
    for n in names:
        assert hasattr(L, n), f"{n} declared in pkv.h but not exported by libpkv.so"
        assert n in pkv._lib.SIGNATURES, f"{n} has no ctypes signature"
    assert L.pkv_abi_version() == 2


def test_reference_launcher_symbols_are_exported(pkv):
    """engine::launch_store_kv / launch_attention_decode / launch_attention_decode_gqa with the
    reference's exact C++ signatures (include/engine/cuda_kernels.h:43-62), Itanium-mangled."""
    L = pkv.lib()
    store = "_ZN6engine15launch_store_kvEPK6__halfS2_PKiPS0_S5_iiP11CUstream_st"
    dec = "_ZN6engine23launch_attention_decodeEPK6__halfS2_S2_PKiS4_S4_S4_PS0_iiiiifP11CUstream_st"
    gqa = "_ZN6engine27launch_attention_decode_gqaEPK6__halfS2_S2_PKiS4_S4_S4_PS0_iiiiifP11CUstream_st"
    for sym in (store, dec, gqa):
        assert hasattr(L, sym), sym


def test_status_strings(pkv):
    L = pkv.lib()
    assert L.pkv_status_string(0) == b"ok"
    for code in range(-6, 0):
        assert L.pkv_status_string(code) not in (b"ok", b"unknown status")
    assert L.pkv_status_string(-99) == b"unknown status"


def test_empty_steps_are_silent_noops(pkv):
    """n_tokens <= 0 returns OK without looking at any pointer (src/kernels/store_kv.cu:34,
    src/kernels/attention_decode.cu:138)."""
    L = pkv.lib()
    for s in ("f16", "bf16", "f32"):
        assert getattr(L, f"pkv_append_{s}")(None, None, None, None, None, 0, 128, None) == 0
        assert getattr(L, f"pkv_append_{s}")(None, None, None, None, None, 4, 0, None) == 0
        assert getattr(L, f"pkv_decode_attn_{s}")(None, None, None, None, None, None, None, None, 0, 14, 2, 64, 16,
                                                  C.c_float(0.125), None, 0, None) == 0
        assert getattr(L, f"pkv_copy_blocks_{s}")(None, None, None, 0, 16, 128, None) == 0
    assert L.pkv_copy_blocks_layers(None, 0, None, 0, 4096, None) == 0


def test_bad_arguments_are_rejected_on_the_host(pkv):
    L = pkv.lib()
    one = 0x1000  # a non-null, 16-byte aligned address that is never dereferenced on these paths
    f = C.c_float(0.125)
    # null pointers
    assert L.pkv_append_bf16(None, one, one, one, one, 4, 128, None) == pkv._lib.PKV_E_ARG
    assert L.pkv_decode_attn_bf16(None, one, one, one, one, one, one, one, 4, 14, 2, 64, 16, f, None, 0, None) == pkv._lib.PKV_E_ARG
    # q_heads not a multiple of kv_heads (reference: attention_decode_gqa.cu:212-214 throws)
    assert L.pkv_decode_attn_bf16(one, one, one, one, one, one, one, one, 4, 14, 4, 64, 16, f, None, 0, None) == pkv._lib.PKV_E_UNSUPPORTED
    assert b"multiple" in L.pkv_last_error()
    # head_dim beyond the accumulators
    assert L.pkv_decode_attn_f16(one, one, one, one, one, one, one, one, 4, 8, 8, 512, 16, f, None, 0, None) == pkv._lib.PKV_E_UNSUPPORTED
    # misaligned pool
    assert L.pkv_decode_attn_f16(one, one + 2, one, one, one, one, one, one, 4, 8, 8, 64, 16, f, None, 0, None) == pkv._lib.PKV_E_ARG
    # workspace too small / misaligned
    assert L.pkv_decode_attn_f16(one, one, one, one, one, one, one, one, 4, 8, 8, 64, 16, f, one, 64, None) == pkv._lib.PKV_E_WORKSPACE
    assert L.pkv_decode_attn_f16(one, one, one, one, one, one, one, one, 4, 8, 8, 64, 16, f, one + 16, 1 << 30, None) == pkv._lib.PKV_E_ARG
    assert L.pkv_copy_blocks_bf16(None, one, one, 3, 16, 128, None) == pkv._lib.PKV_E_ARG
    assert L.pkv_copy_blocks_bf16(one, one, one, 70000, 16, 128, None) == pkv._lib.PKV_E_UNSUPPORTED


def test_workspace_size_query(pkv):
    L = pkv.lib()
    assert L.pkv_decode_workspace_bytes(0, 14, 2, 64) == 0
    small = L.pkv_decode_workspace_bytes(8, 14, 2, 64)
    big = L.pkv_decode_workspace_bytes(256, 32, 4, 64)
    assert 0 < small < 256 * 2 ** 20 and 0 < big < 256 * 2 ** 20
    assert small % 256 == 0 and big % 256 == 0
    assert L.pkv_decode_plan_staging_bytes(256, 4) > 256 * 16


def test_host_plan_layout_without_a_device(pkv):
    """The host planner's item list, checked structurally: items tile every token's key range
    exactly once, partial slots are distinct, single-chunk tokens write directly."""
    L = pkv.lib()
    rng = np.random.default_rng(0)
    pos = np.concatenate([rng.integers(0, 9000, size=200), [0, 63, 64, 255, 256, 257, 8192]]).astype(np.int32)
    n, qh, kvh, hd = pos.size, 32, 4, 64
    nstage = L.pkv_decode_plan_staging_bytes(n, kvh)
    staging = np.zeros(nstage, dtype=np.uint8)
    plan = pkv._lib.DecodePlan()
    # a null workspace is refused before any copy is attempted
    st = L.pkv_decode_plan_host(pos.ctypes.data, n, qh, kvh, hd, staging.ctypes.data, nstage, None, 1 << 30, None, C.byref(plan))
    assert st == pkv._lib.PKV_E_ARG
    neg = pos.copy(); neg[3] = -1
    st = L.pkv_decode_plan_host(neg.ctypes.data, n, qh, kvh, hd, staging.ctypes.data, nstage, 0x10000, 1 << 30, None, C.byref(plan))
    assert st == pkv._lib.PKV_E_ARG and b"negative" in L.pkv_last_error()


def test_host_planner_offers_the_cluster_form_for_small_steps_only(pkv, monkeypatch):
    """pkv_decode_plan.cluster: set by the host planner unless the environment has PKV_DECODE_CLUSTER=0
    (read at every call), and only for steps whose (token, kv head) pairs can each have a resident cluster
    (3 blocks on each of the device's SMs; 148 assumed without a device) with at most 256 keys per warp,
    head_dim 64 and at most 8 query heads per kv head."""
    L = pkv.lib()

    def cluster_of(pos, qh, kvh, hd=64):
        pos = np.asarray(pos, dtype=np.int32)
        nstage = L.pkv_decode_plan_staging_bytes(pos.size, kvh)
        staging = np.zeros(nstage, dtype=np.uint8)
        plan = pkv._lib.DecodePlan()
        image = C.c_size_t(0)
        ws = L.pkv_decode_workspace_bytes(pos.size, qh, kvh, hd)
        st = L.pkv_decode_plan_host_image(pos.ctypes.data, pos.size, qh, kvh, hd, staging.ctypes.data, nstage, ws,
                                          C.byref(plan), C.byref(image))
        assert st == 0, L.pkv_last_error()
        return plan.cluster

    monkeypatch.setenv("PKV_DECODE_CLUSTER", "0")
    assert cluster_of([1000] * 8, 32, 4) == 0
    monkeypatch.delenv("PKV_DECODE_CLUSTER")
    assert cluster_of([1000] * 8, 32, 4) == 8            # 32 pairs: the largest portable cluster
    assert cluster_of([1000] * 64, 14, 2) == 3           # 128 pairs on 444 block slots
    assert cluster_of([1000] * 40, 14, 2) == 4           # 80 pairs: 5 would fit; the kernel takes 2, 3, 4 or 8
    assert cluster_of([1000] * 111, 14, 2) == 2          # 222 pairs
    assert cluster_of([1000] * 112, 14, 2) == 0          # 224 pairs: two blocks each would not all be resident
    assert cluster_of([20000] * 8, 32, 4) == 0           # 626 keys per warp
    assert cluster_of([1000] * 8, 32, 2) == 0            # 16 query heads per kv head
    assert cluster_of([1000] * 8, 32, 4, hd=128) == 0
    assert cluster_of([100] * 8, 32, 4) == 0             # nothing to merge: no token is split


def test_step_pack_matches_restatement(pkv, orc):
    import ctypes
    rng = np.random.default_rng(4)
    bs = 16
    tables = [rng.permutation(500)[:int(n)].astype(np.int32) for n in rng.integers(1, 30, size=9)]
    tok_tabs, tok_pos, keys = [], [], []
    # prefill slices first, then decode tokens, sequences interleaved and revisited
    for s in (3, 0, 3, 7, 1, 0, 8, 8, 2):
        n = int(rng.integers(1, 6))
        start = int(rng.integers(0, tables[s].size * bs - n + 1))
        for i in range(n):
            tok_tabs.append(tables[s]); tok_pos.append(start + i); keys.append(1000 + s)
    got = pkv.pack_step(tok_tabs, tok_pos, bs, tok_keys=keys)
    n = len(tok_pos)
    karr = np.asarray(keys, dtype=np.uint64)
    ptrs = (ctypes.c_void_p * n)(*[t.ctypes.data for t in tok_tabs])
    nblk = np.asarray([t.size for t in tok_tabs], dtype=np.int32)
    pos = np.asarray(tok_pos, dtype=np.int32)
    slots = np.zeros(n, np.int32); tseq = np.zeros(n, np.int32)
    tabs = np.zeros(sum(t.size for t in tables), np.int32); off = np.zeros(len(tables), np.int32)
    ntab = ctypes.c_int(0)
    f = orc.lib.orc_step_pack
    f.restype = ctypes.c_int
    f.argtypes = [ctypes.c_int] + [ctypes.c_void_p] * 4 + [ctypes.c_int] + [ctypes.c_void_p] * 5
    nseq = f(n, karr.ctypes.data, ctypes.cast(ptrs, ctypes.c_void_p), nblk.ctypes.data, pos.ctypes.data, bs,
             slots.ctypes.data, tseq.ctypes.data, tabs.ctypes.data, off.ctypes.data, ctypes.byref(ntab))
    assert got.n_seqs == nseq
    assert np.array_equal(got.slots, slots) and np.array_equal(got.token_seq, tseq)
    assert np.array_equal(got.block_tables, tabs[:ntab.value]) and np.array_equal(got.table_offset, off[:nseq])
    assert got.token_seq.tolist()[:1] == [0] and got.n_seqs == 6


def test_step_pack_errors(pkv):
    t = np.asarray([5, 6], dtype=np.int32)
    with pytest.raises(pkv.PkvError):
        pkv.pack_step([t], [32], 16)          # position 32 needs a third block
    with pytest.raises(pkv.PkvError):
        pkv.pack_step([t], [-1], 16)
    e = pkv.pack_step([], [], 16)
    assert e.n_tokens == 0 and e.n_seqs == 0


def test_recorded_give_up_is_reported_once_by_the_next_attention_call(pkv):
    """The contract of include/pkv.h, "Bounded waits": the attention call that follows an incomplete
    launch returns PKV_E_CUDA once and enqueues nothing; the call after that runs normally."""
    L = pkv.lib()
    one = 0x1000
    f = C.c_float(0.125)
    assert L.pkv_debug_set_reported_flags(2 | 8) == 0
    st = L.pkv_decode_attn_bf16(one, one, one, one, one, one, one, one, 4, 14, 2, 64, 16, f, None, 0, None)
    assert st == pkv._lib.PKV_E_CUDA
    msg = L.pkv_last_error().decode()
    assert "gave up" in msg and "0xa" in msg
    # cleared by the report: the same call now gets as far as its argument checks
    st = L.pkv_decode_attn_bf16(None, one, one, one, one, one, one, one, 4, 14, 2, 64, 16, f, None, 0, None)
    assert st == pkv._lib.PKV_E_ARG
    # empty steps never look: they stay silent no-ops
    assert L.pkv_debug_set_reported_flags(4) == 0
    assert L.pkv_decode_attn_f16(None, None, None, None, None, None, None, None, 0, 14, 2, 64, 16, f, None, 0, None) == 0
    plan = pkv._lib.DecodePlan()
    plan.n_tokens, plan.q_heads, plan.kv_heads, plan.head_dim = 4, 14, 2, 64
    st = L.pkv_decode_attn_planned_f16(C.byref(plan), one, one, one, one, one, one, one, one, 16, f, one, 1 << 20, None)
    assert st == pkv._lib.PKV_E_CUDA and "0x4" in L.pkv_last_error().decode()
    assert L.pkv_debug_set_reported_flags(1) == 0
    st = L.pkv_prefill_attn_bf16(one, one, one, one, one, one, one, one, one, 4, 1, 4, 14, 2, 64, 16, 8, f, None)
    assert st == pkv._lib.PKV_E_CUDA
    st = L.pkv_mixed_attn_bf16(one, one, one, one, one, one, one, one, 0, 14, 2, 64, 16, 0, f, 0, None, 0, None)
    assert st == 0


def test_launcher_symbols_throw_what_the_c_abi_returns(pkv, tmp_path):
    """engine::launch_attention_decode turns a refusal into std::runtime_error before anything is
    enqueued, like the reference launchers (src/kernels/attention_decode_gqa.cu:211-224); checked
    without a GPU on the two refusals that need none."""
    from tests.shim_util import build_harness
    H = build_harness(tmp_path)
    err = C.create_string_buffer(600)
    one = 0x1000
    args = lambda n, qh, kvh: (0, 0, one, one, one, one, one, one, one, one, one, one, one, n, qh, kvh, 64, 16, C.c_float(0.125), None, err, 600)
    assert H.harness_layer(*args(4, 14, 4)) == 1 and b"multiple" in err.value
    pkv.lib().pkv_debug_set_reported_flags(8)
    assert H.harness_layer(*args(4, 14, 2)) == 1 and b"gave up" in err.value and b"launch_attention_decode" in err.value
    assert H.harness_layer(*args(0, 14, 2)) == 0          # an empty step is a silent no-op
    assert pkv.lib().pkv_mixed_attn_workspace_bytes(300, 14, 2, 64) > pkv.lib().pkv_decode_workspace_bytes(300, 14, 2, 64)
