"""GPU parity for the two pure-copy operations: K/V append and the copy-on-write block copy.
Both must reproduce the CPU checker's bytes exactly."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

NP_OF = {"f32": np.float32, "bf16": np.uint16, "f16": np.uint16}


def tdtype(torch, dtype):
    return {"f32": torch.float32, "bf16": torch.bfloat16, "f16": torch.float16}[dtype]


def dev(torch, a, dtype):
    if dtype == "f32":
        return torch.from_numpy(np.ascontiguousarray(a)).cuda()
    return torch.from_numpy(np.ascontiguousarray(a).view(np.int16)).cuda().view(tdtype(torch, dtype))


def host(torch, t, dtype):
    if dtype == "f32":
        return t.cpu().numpy().view(np.uint32)
    return t.view(torch.int16).cpu().numpy().view(np.uint16)


def rand_bits(rng, shape, dtype):
    if dtype == "f32":
        return rng.standard_normal(shape, dtype=np.float32)
    return rng.integers(0, 65536, size=shape, dtype=np.uint16)   # any bit pattern, NaNs included: it is a byte copy


@pytest.mark.parametrize("dtype", ["f32", "bf16", "f16"])
@pytest.mark.parametrize("n_tokens,kv_dim,slots_total", [
    (8, 128, 4096 * 16),        # configuration 1
    (64, 128, 16384 * 16),      # configuration 2
    (256, 256, 65536 * 16),     # configuration 3
    (16384, 128, 8192 * 16),    # configuration 4: a whole prefill step
    (1, 128, 64),
    (5, 24, 100),               # row size not a multiple of 16 bytes (element-wise path)
    (7, 3, 50),
])
def test_append_is_bit_exact(pkv, orc, torch_cuda, dtype, n_tokens, kv_dim, slots_total):
    torch = torch_cuda
    rng = np.random.default_rng(n_tokens * 31 + kv_dim)
    k, v = rand_bits(rng, (n_tokens, kv_dim), dtype), rand_bits(rng, (n_tokens, kv_dim), dtype)
    kc, vc = rand_bits(rng, (slots_total, kv_dim), dtype), rand_bits(rng, (slots_total, kv_dim), dtype)
    slots = rng.permutation(slots_total)[:n_tokens].astype(np.int32)
    d_kc, d_vc = dev(torch, kc, dtype), dev(torch, vc, dtype)
    pkv.launch_store_kv(dev(torch, k, dtype), dev(torch, v, dtype), torch.from_numpy(slots).cuda(), d_kc, d_vc,
                        n_tokens, kv_dim)
    torch.cuda.synchronize()
    orc.append(k, v, slots, kc, vc)
    view = (lambda a: a.view(np.uint32)) if dtype == "f32" else (lambda a: a)
    assert np.array_equal(host(torch, d_kc, dtype), view(kc))
    assert np.array_equal(host(torch, d_vc, dtype), view(vc))


def test_append_duplicate_slots_with_identical_payloads(pkv, orc, torch_cuda):
    """A fully cached prompt recomputes its last token and re-writes a shared full block with the
    same values (llm-engine src/scheduler/scheduler.cpp:60): duplicates are legal when the rows agree."""
    torch = torch_cuda
    rng = np.random.default_rng(2)
    row_k, row_v = rand_bits(rng, (1, 256), "bf16"), rand_bits(rng, (1, 256), "bf16")
    k, v = np.repeat(row_k, 6, 0), np.repeat(row_v, 6, 0)
    slots = np.asarray([40, 40, 7, 40, 7, 40], dtype=np.int32)
    kc, vc = rand_bits(rng, (128, 256), "bf16"), rand_bits(rng, (128, 256), "bf16")
    d_kc, d_vc = dev(torch, kc, "bf16"), dev(torch, vc, "bf16")
    pkv.launch_store_kv(dev(torch, k, "bf16"), dev(torch, v, "bf16"), torch.from_numpy(slots).cuda(), d_kc, d_vc, 6, 256)
    torch.cuda.synchronize()
    orc.append(k, v, slots, kc, vc)
    assert np.array_equal(host(torch, d_kc, "bf16"), kc) and np.array_equal(host(torch, d_vc, "bf16"), vc)


def test_append_empty_step_touches_nothing(pkv, torch_cuda):
    torch = torch_cuda
    kc = torch.full((64, 128), 3.0, device="cuda", dtype=torch.bfloat16)
    vc = kc.clone()
    e = torch.zeros((0, 128), device="cuda", dtype=torch.bfloat16)
    pkv.launch_store_kv(e, e, torch.zeros(0, dtype=torch.int32, device="cuda"), kc, vc, 0, 128)
    torch.cuda.synchronize()
    assert bool((kc == 3.0).all()) and bool((vc == 3.0).all())


def test_launchers_raise_like_the_reference(pkv, torch_cuda):
    """Unsupported geometry is an exception before launch (attention_decode_gqa.cu:211-224), not a trap."""
    torch = torch_cuda
    z = torch.zeros((4, 64 * 14), device="cuda", dtype=torch.float16)
    i = torch.zeros(4, device="cuda", dtype=torch.int32)
    pool = torch.zeros((64, 256), device="cuda", dtype=torch.float16)
    with pytest.raises(pkv.PkvError):
        pkv.launch_attention_decode(z, pool, pool, i, i, i, i, z, 4, 14, 4, 64, 16, 0.125)   # 14 % 4 != 0
    with pytest.raises(ValueError):
        pkv.launch_store_kv(z.cpu(), z, i, pool, pool, 4, 128)                               # no CPU path


@pytest.mark.parametrize("dtype", ["f32", "bf16", "f16"])
@pytest.mark.parametrize("bs,kv_dim,num_blocks,n_pairs", [(16, 256, 2048, 127), (16, 128, 512, 1), (4, 24, 300, 50), (1, 3, 64, 9)])
def test_copy_blocks_is_bit_exact(pkv, orc, torch_cuda, dtype, bs, kv_dim, num_blocks, n_pairs):
    torch = torch_cuda
    rng = np.random.default_rng(bs * 7 + n_pairs)
    kc, vc = rand_bits(rng, (num_blocks * bs, kv_dim), dtype), rand_bits(rng, (num_blocks * bs, kv_dim), dtype)
    perm = rng.permutation(num_blocks)
    # many destinations per source, as when every child of one parent diverges from the same partial block
    srcs = perm[:max(1, n_pairs // 8)]
    pairs = np.stack([rng.choice(srcs, size=n_pairs), perm[len(srcs):len(srcs) + n_pairs]], axis=1).astype(np.int32)
    d_kc, d_vc = dev(torch, kc, dtype), dev(torch, vc, dtype)
    pkv.launch_copy_blocks(d_kc, d_vc, torch.from_numpy(pairs).cuda(), n_pairs, bs, kv_dim)
    torch.cuda.synchronize()
    esz = 4 if dtype == "f32" else 2
    f = orc.lib.orc_copy_blocks
    import ctypes
    f.restype = None
    f.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_size_t]
    f(kc.ctypes.data, vc.ctypes.data, pairs.ctypes.data, n_pairs, bs * kv_dim * esz)
    view = (lambda a: a.view(np.uint32)) if dtype == "f32" else (lambda a: a)
    assert np.array_equal(host(torch, d_kc, dtype), view(kc))
    assert np.array_equal(host(torch, d_vc, dtype), view(vc))


def test_copy_blocks_across_all_layers(pkv, orc, torch_cuda):
    """Configuration 5's wave: 127 children diverge from one shared partial block, 22 layers x {K, V}."""
    torch = torch_cuda
    layers, bs, kv_dim, nb = 22, 16, 256, 512
    g = torch.Generator(device="cuda").manual_seed(5)
    pools = [torch.randint(-32768, 32767, (nb * bs, kv_dim), generator=g, device="cuda", dtype=torch.int16).view(torch.bfloat16)
             for _ in range(2 * layers)]
    before = [p.clone() for p in pools]
    pairs = np.stack([np.full(127, 17), np.arange(100, 227)], axis=1).astype(np.int32)
    ptrs = torch.tensor([p.data_ptr() for p in pools], dtype=torch.int64, device="cuda")
    pkv.launch_copy_blocks_layers(ptrs, len(pools), torch.from_numpy(pairs).cuda(), 127, bs * kv_dim * 2)
    torch.cuda.synchronize()
    for p, b in zip(pools, before):
        pv, bv = p.view(torch.int16).view(nb, -1), b.view(torch.int16).view(nb, -1)
        want = bv.clone()
        want[100:227] = bv[17]
        assert torch.equal(pv, want)
