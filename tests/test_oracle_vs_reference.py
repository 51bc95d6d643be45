"""The oracle against the reference's own host code, live, where the shim was
built (oracle/_ref/libw4ref.so). Skipped on machines without it; the committed
golden vectors cover those."""
import numpy as np
import pytest

import cases


def test_generators_and_scalars(oracle, reference):
    for seed in (0, 1, 0x44A1, 2**63 + 5):
        assert np.array_equal(oracle.normal_f64(3001, seed).view(np.uint64),
                              reference.normal_f64(3001, seed).view(np.uint64))
        assert np.array_equal(oracle.normal_f16(999, seed), reference.normal_f16(999, seed))
    for h in range(0, 65536, 7):
        a, b = oracle.f16_to_f32(h), reference.f16_to_f32(h)
        assert a == b or (a != a and b != b)
    rng = np.random.default_rng(1)
    for x in rng.standard_normal(20000).astype(np.float32) * np.float32(10.0) ** rng.integers(-9, 6, 20000).astype(np.float32):
        assert oracle.f32_to_f16(x) == reference.f32_to_f16(x)
        assert oracle.encode_e4m3(x) == reference.encode_e4m3(x)


def test_dequant_one_exhaustive(oracle, reference):
    # every code against a spread of scales incl. subnormal, tiny, huge and negative
    scales = [0x0001, 0x0200, 0x03FF, 0x0400, 0x1234, 0x2E66, 0x3C00, 0x5555, 0x7BFF, 0x8001, 0xBC00, 0x0000]
    for s in scales:
        for q in range(16):
            for z in range(16):
                assert oracle.dequant_one(s, q, z) == reference.dequant_one(s, q, z)
        for b in range(256):
            assert oracle.dequant_one_f8(s, b) == reference.dequant_one_f8(s, b)
    for se in range(255):
        for q in range(16):
            assert oracle.dequant_one_mx(se, q) == reference.dequant_one_mx(se, q)


@pytest.mark.parametrize("sym", [True, False])
def test_random_shapes_w4(oracle, reference, sym):
    rng = np.random.default_rng(7)
    for _ in range(12):
        N, K = int(rng.integers(1, 40)), int(rng.integers(1, 300))
        gs = int(rng.choice([8, 16, 24, 32, 48, 64, 128]))
        w = rng.standard_normal(N * K) * 10.0 ** rng.integers(-3, 3)
        a, b = oracle.quantize_w4(w, N, K, gs, sym), reference.quantize_w4(w, N, K, gs, sym)
        for key in ("q", "scales", "zeros"):
            assert (a[key] is None and b[key] is None) or np.array_equal(a[key], b[key])
        assert np.array_equal(oracle.dequant_all_w4(a), reference.dequant_all_w4(b))


def test_random_shapes_mx_f8_paged(oracle, reference):
    rng = np.random.default_rng(9)
    for _ in range(8):
        N, K = int(rng.integers(1, 40)), int(rng.integers(1, 300))
        w = rng.standard_normal(N * K) * 2.0 ** rng.integers(-20, 20)
        a, b = oracle.quantize_mx(w, N, K), reference.quantize_mx(w, N, K)
        assert np.array_equal(a["q"], b["q"]) and np.array_equal(a["scales"], b["scales"])
        assert np.array_equal(oracle.dequant_all_mx(a), reference.dequant_all_mx(b))
    for _ in range(6):
        H, S, D = int(rng.integers(1, 4)), int(rng.integers(1, 50)), int(rng.integers(1, 30)) * 4
        gs = int(rng.choice([8, 16, 32]))
        k, v = rng.standard_normal(H * S * D), rng.standard_normal(H * S * D) * 3
        q = rng.standard_normal(H * D).astype(np.float16).view(np.uint16)
        a, b = oracle.quantize_cache_f8(k, v, H, S, D, gs), reference.quantize_cache_f8(k, v, H, S, D, gs)
        for key in ("q_k", "s_k", "q_v", "s_v"):
            assert np.array_equal(a[key], b[key])
        out, kd, vd = reference.attention_f8(q, b)
        assert np.array_equal(oracle.dequant_cache_f8(a, "k"), kd)
        assert np.array_equal(oracle.attention_reference(q, kd, vd, H, S, D), out)
        for sym in (True, False):
            ca, cb = oracle.quantize_cache_w4(k, v, H, S, D, gs, sym), reference.quantize_cache_w4(k, v, H, S, D, gs, sym)
            out, kd, vd = reference.attention_w4(q, cb)
            assert np.array_equal(oracle.dequant_cache_w4(ca, "v"), vd)
            assert np.array_equal(oracle.attention_reference(q, kd, vd, H, S, D), out)
            page = int(rng.choice([1, 4, 16]))
            bt = rng.permutation((S + page - 1) // page).astype(np.int32)
            pa, pb = oracle.paged_from_contiguous(ca, page, bt), reference.paged_from_contiguous(cb, page, bt)
            for key in ("q_k", "s_k", "z_k", "q_v", "s_v", "z_v"):
                assert (pa[key] is None and pb[key] is None) or np.array_equal(pa[key], pb[key])
