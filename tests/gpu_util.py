"""Helpers shared by the GPU parity tests: build a seeded paged-KV step, run it through the
C ABI on the device and through the CPU checker on the host, and compare."""
from __future__ import annotations

import numpy as np

TOL = {"f32": 1e-5, "bf16": 2e-2, "f16": 2e-2}   # max relative error the path must meet per KV dtype


def torch_dtype(torch, dtype):
    return {"f32": torch.float32, "bf16": torch.bfloat16, "f16": torch.float16}[dtype]


def cast_like_reference(orc, x, dtype):
    """fp32 array -> (bits to upload, fp32 values the checker sees): the reference's own
    f32_to_bf16 / f32_to_f16 (include/engine/tensor.h:23-62), then widened back."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    if dtype == "f32":
        return x, x
    if dtype == "bf16":
        bits = orc.to_bf16_bits(x)
        return bits, orc.from_bf16_bits(bits)
    bits = orc.to_f16_bits(x)
    return bits, orc.from_f16_bits(bits)


def to_device(torch, arr, dtype):
    if dtype == "f32":
        return torch.from_numpy(np.ascontiguousarray(arr)).cuda()
    t = torch.from_numpy(np.ascontiguousarray(arr).view(np.int16)).cuda()
    return t.view(torch_dtype(torch, dtype))


def from_device(torch, orc, t, dtype):
    """(raw bits or fp32 array, fp32 values)."""
    if dtype == "f32":
        a = t.cpu().numpy()
        return a, a
    bits = t.view(torch.int16).cpu().numpy().view(np.uint16)
    return bits, (orc.from_bf16_bits(bits) if dtype == "bf16" else orc.from_f16_bits(bits))


def rel_errors(got, want):
    """(reference metric, per-row metric): max|diff| / max(max|want|, 1) as in llm-engine's
    tests/test_golden_ops.cpp:71-79, and the stricter max over rows of max|diff| / max|want_row|."""
    got = np.asarray(got, dtype=np.float64)
    want = np.asarray(want, dtype=np.float64)
    diff = np.abs(got - want)
    ref_metric = diff.max() / max(np.abs(want).max(), 1.0) if diff.size else 0.0
    row = diff.max(axis=-1) / np.maximum(np.abs(want).max(axis=-1), 1e-30) if diff.size else np.zeros(1)
    return float(ref_metric), float(row.max())


class Case:
    """One packed step over a fragmented pool."""

    def __init__(self, orc, dtype, q_heads, kv_heads, head_dim, bs, num_blocks, seq_ctx, seq_new, seed, pkv, share=None):
        """share: [(member sequence indices, n_blocks)]: the members' first n_blocks table entries are
        made those of the first member (a common prompt prefix held once in the pool)."""
        rng = np.random.default_rng(seed)
        self.dtype, self.qh, self.kvh, self.hd, self.bs, self.nb = dtype, q_heads, kv_heads, head_dim, bs, num_blocks
        kv_dim = kv_heads * head_dim
        perm = rng.permutation(num_blocks).astype(np.int32)
        self.tables, at = [], 0
        for c, n in zip(seq_ctx, seq_new):
            k = (c + n + bs - 1) // bs
            assert at + k <= num_blocks
            self.tables.append(perm[at:at + k].copy())
            at += k
        for members, n_shared in (share or []):
            for s in members[1:]:
                assert n_shared * bs <= seq_ctx[s] and n_shared * bs <= seq_ctx[members[0]]   # new tokens land in private blocks
                self.tables[s][:n_shared] = self.tables[members[0]][:n_shared]
        tok_tabs, tok_pos = [], []
        for s, (c, n) in enumerate(zip(seq_ctx, seq_new)):
            for i in range(n):
                tok_tabs.append(self.tables[s])
                tok_pos.append(c + i)
        self.idx = pkv.pack_step(tok_tabs, tok_pos, bs)
        N = self.idx.n_tokens
        self.N = N
        f = lambda *shape: rng.standard_normal(shape, dtype=np.float32)
        self.kc_bits, self.kc = cast_like_reference(orc, f(num_blocks * bs, kv_dim), dtype)
        self.vc_bits, self.vc = cast_like_reference(orc, f(num_blocks * bs, kv_dim), dtype)
        self.q_bits, self.q = cast_like_reference(orc, f(N, q_heads * head_dim), dtype)
        self.k_bits, self.k = cast_like_reference(orc, f(N, kv_dim), dtype)
        self.v_bits, self.v = cast_like_reference(orc, f(N, kv_dim), dtype)
        self.scale = float(np.float32(1.0) / np.sqrt(np.float32(head_dim)))

    def expected(self, orc, threads=4):
        kc, vc = self.kc.copy(), self.vc.copy()
        orc.append(self.k, self.v, self.idx.slots, kc, vc)
        kcb, vcb = self.kc_bits.copy(), self.vc_bits.copy()
        orc.append(self.k_bits, self.v_bits, self.idx.slots, kcb, vcb)
        out = orc.paged_attention(self.q, kc, vc, self.idx.block_tables, self.idx.table_offset, self.idx.token_seq,
                                  self.idx.token_pos, self.qh, self.kvh, self.hd, self.bs, self.scale, threads=threads)
        return kcb, vcb, out

    def upload(self, torch):
        d = {}
        for name in ("kc", "vc", "q", "k", "v"):
            d[name] = to_device(torch, getattr(self, name + "_bits"), self.dtype)
        i32 = lambda a: torch.from_numpy(np.ascontiguousarray(a, dtype=np.int32)).cuda()
        d["slots"], d["token_seq"], d["token_pos"] = i32(self.idx.slots), i32(self.idx.token_seq), i32(self.idx.token_pos)
        d["block_tables"], d["table_offset"] = i32(self.idx.block_tables), i32(self.idx.table_offset)
        d["out"] = torch.zeros((self.N, self.qh * self.hd), dtype=torch_dtype(torch, self.dtype), device="cuda")
        return d

    def run_gpu(self, pkv, torch, mode="split", d=None):
        """mode: direct | split | host_plan | shared_plan | device_plan | fused_append.  Returns (k_cache bits, v_cache bits, out fp32, dev dict)."""
        d = d or self.upload(torch)
        kv_dim = self.kvh * self.hd
        if mode == "fused_append":
            plan = pkv.DecodePlan(self.N, self.qh, self.kvh, self.hd).build_host(self.idx.token_pos)
            plan.append_attention(d["q"], d["k"], d["v"], d["slots"], d["kc"], d["vc"], d["block_tables"], d["table_offset"],
                                  d["token_seq"], d["token_pos"], d["out"], self.bs, self.scale)
            d["plan"] = plan
            torch.cuda.synchronize()
            return d
        pkv.launch_store_kv(d["k"], d["v"], d["slots"], d["kc"], d["vc"], self.N, kv_dim)
        args = (d["q"], d["kc"], d["vc"], d["block_tables"], d["table_offset"], d["token_seq"], d["token_pos"], d["out"])
        if mode == "direct":
            pkv.launch_attention_decode(*args, self.N, self.qh, self.kvh, self.hd, self.bs, self.scale)
        elif mode == "split":
            ws = pkv.alloc_decode_workspace(self.N, self.qh, self.kvh, self.hd)
            pkv.launch_attention_decode_gqa(*args, self.N, self.qh, self.kvh, self.hd, self.bs, self.scale, workspace=ws)
        else:
            plan = pkv.DecodePlan(self.N, self.qh, self.kvh, self.hd)
            if mode == "host_plan":
                plan.build_host(self.idx.token_pos)
            elif mode == "shared_plan":
                plan.build_host_shared(self.idx, self.bs, min_saved_bytes=0)
            else:
                plan.build_device(d["token_pos"])
            plan.attention(*args, self.bs, self.scale)
            d["plan"] = plan
        torch.cuda.synchronize()
        return d


def check_case(case, pkv, torch, orc, mode, tol=None):
    want_kc, want_vc, want_out = case.expected(orc)
    d = case.run_gpu(pkv, torch, mode)
    kcb, _ = from_device(torch, orc, d["kc"], case.dtype)
    vcb, _ = from_device(torch, orc, d["vc"], case.dtype)
    view = (lambda a: a.view(np.uint32)) if case.dtype == "f32" else (lambda a: a)
    assert np.array_equal(view(kcb), view(want_kc)), "K pool differs from the reference append"
    assert np.array_equal(view(vcb), view(want_vc)), "V pool differs from the reference append"
    _, got = from_device(torch, orc, d["out"], case.dtype)
    assert np.isfinite(got).all()
    assert pkv.debug_device_flags() == 0, "a kernel gave up on a bounded wait"
    e_ref, e_row = rel_errors(got.reshape(case.N * case.qh, case.hd), want_out.reshape(case.N * case.qh, case.hd))
    tol = tol or TOL[case.dtype]
    assert e_ref <= tol and e_row <= tol, f"{mode}: rel err {e_ref:.3e} (reference metric) / {e_row:.3e} (per row) > {tol}"
    return e_ref, e_row
