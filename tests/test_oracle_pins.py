"""CPU gates for the oracle: the reference's host pins and bounds
(tests/test_oracle.cpp), restated against oracle/w4_oracle.c."""
import numpy as np
import pytest

import cases
from cases import f16

E2M1 = np.array([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0])


def nibbles(words, per_row_words, count):
    w = np.asarray(words, np.uint32).reshape(-1, per_row_words)
    sh = (4 * np.arange(8, dtype=np.uint32))[None, None, :]
    return ((w[:, :, None] >> sh) & 0xF).reshape(w.shape[0], -1)[:, :count].astype(np.int64)


@pytest.mark.parametrize("sym", [True, False])
@pytest.mark.parametrize("i", range(len(cases.HOST_GEMM_CFGS)))
def test_w4_per_element_bound(oracle, i, sym):
    # tests/test_oracle.cpp:23-61: |deq - w| <= (clamped ? 1.1 : 0.52) * scale
    M, N, K, gs = cases.HOST_GEMM_CFGS[i]
    w = oracle.normal_f64(N * K, cases.w4_seed(i, sym))
    p = oracle.quantize_w4(w, N, K, gs, sym)
    wd = f16(oracle.dequant_all_w4(p)).reshape(N, K)
    q = nibbles(p["q"], (K + 7) // 8, K)
    sf = f16(p["scales"]).reshape(N, p["G"])[:, np.arange(K) // gs]
    tol = np.where((q == 0) | (q == 15), 1.1, 0.52) * sf + 1e-12
    assert np.all(np.abs(wd - w.reshape(N, K)) <= tol)


def test_gemm_oracle_known_answer(oracle):
    # tests/test_oracle.cpp:63-78: x=[1,2], W=[[3,4],[5,6]] -> [11,17]
    h = lambda v: np.array(v, np.float16).view(np.uint16)
    c = oracle.gemm_oracle(h([1, 2]), 1, 2, h([3, 4, 5, 6]), 2)
    assert c.tolist() == [11.0, 17.0]
    assert oracle.gemm_oracle(h([1, 2]), 1, 2, h([3, 4, 5, 6]), 2, threads=2).tolist() == [11.0, 17.0]


@pytest.mark.parametrize("sym", [True, False])
def test_w4_zero_groups(oracle, sym):
    # tests/test_oracle.cpp:80-94
    p = oracle.quantize_w4(np.zeros(64 * 64), 64, 64, 32, sym)
    assert not np.any(f16(oracle.dequant_all_w4(p)))


def test_w4_throws(oracle):
    # tests/test_oracle.cpp:96-148
    ok = np.full(64 * 64, 0.5)
    for args in [(0, 64, 8), (64, 64, 0), (64, 64, 7), (64, 64, 9)]:
        with pytest.raises(ValueError):
            oracle.quantize_w4(ok, args[0], args[1], args[2], True)
    with pytest.raises(ValueError):
        oracle.quantize_w4(np.zeros(10), 64, 64, 8, True)
    for sym in (True, False):
        bad = ok.copy()
        bad[3] = np.nan
        with pytest.raises(ValueError):
            oracle.quantize_w4(bad, 64, 64, 8, sym)
        bad[3] = 1e300
        with pytest.raises(ValueError):
            oracle.quantize_w4(bad, 64, 64, 8, sym)
        with pytest.raises(ValueError):
            oracle.quantize_w4(np.full(64 * 64, 1e-12), 64, 64, 8, sym)
    p = oracle.quantize_w4(ok, 64, 64, 8, True)
    bad = dict(p, gs=7)
    with pytest.raises(ValueError):
        oracle.dequant_all_w4(bad)
    bad = dict(p, G=p["G"] + 1)
    with pytest.raises(ValueError):
        oracle.dequant_all_w4(bad)


@pytest.mark.parametrize("i", range(len(cases.MX_HOST_CFGS)))
def test_mx_bound_and_no_saturation(oracle, i):
    # tests/test_oracle.cpp:155-211
    M, N, K = cases.MX_HOST_CFGS[i]
    w = oracle.normal_f64(N * K, cases.mx_host_seed(i)).reshape(N, K)
    p = oracle.quantize_mx(w, N, K)
    wd = f16(oracle.dequant_all_mx(p)).reshape(N, K)
    s = np.ldexp(1.0, p["scales"].astype(np.int64).reshape(N, p["B"]) - 127)
    idx = nibbles(p["q"], (K + 7) // 8, K) & 7
    left = np.where(idx > 0, E2M1[idx] - E2M1[np.maximum(idx - 1, 0)], 0.5)
    right = np.where(idx < 7, E2M1[np.minimum(idx + 1, 7)] - E2M1[idx], left)
    tol = 0.5 * np.maximum(left, right) * s[:, np.arange(K) // 32] + 1e-12
    assert np.all(np.abs(wd - w) <= tol)
    for b in range(p["B"]):
        amax = np.abs(w[:, 32 * b:32 * b + 32]).max(axis=1)
        assert np.all(amax <= 6.0 * s[:, b] * (1 + 1e-12))


def test_mx_pins(oracle):
    # tests/test_oracle.cpp:213-262
    p = oracle.quantize_mx(np.full(64, 3.0), 2, 32)
    assert p["scales"].tolist() == [126, 126]
    assert int(p["q"][0] & 0xF) == 7
    wd = f16(oracle.dequant_all_mx(p))
    assert wd[0] == 3.0 and wd[63] == 3.0
    p = oracle.quantize_mx(np.full(32, -2.0), 1, 32)
    assert f16(oracle.dequant_all_mx(p))[0] == -2.0 and (int(p["q"][0]) & 8)
    p = oracle.quantize_mx(np.zeros(64 * 64), 64, 64)
    assert not np.any(f16(oracle.dequant_all_mx(p)))
    # code 8 is minus zero and must keep its sign bit (include/w4/mx.hpp:61)
    assert oracle.dequant_one_mx(127, 8) == 0x8000
    assert oracle.dequant_one_mx(127, 0) == 0x0000


def test_mx_throws(oracle):
    # tests/test_oracle.cpp:264-301
    ok = np.full(64 * 64, 0.5)
    with pytest.raises(ValueError):
        oracle.quantize_mx(ok, 0, 64)
    with pytest.raises(ValueError):
        oracle.quantize_mx(np.zeros(10), 64, 64)
    bad = ok.copy()
    bad[3] = np.nan
    with pytest.raises(ValueError):
        oracle.quantize_mx(bad, 64, 64)
    bad[3] = 1e300
    with pytest.raises(ValueError):
        oracle.quantize_mx(bad, 64, 64)
    p = oracle.quantize_mx(ok, 64, 64)
    with pytest.raises(ValueError):
        oracle.dequant_all_mx(dict(p, B=p["B"] + 1))


@pytest.mark.parametrize("sym", [True, False])
def test_kv_layout_matches_per_head_quantize(oracle, sym):
    # tests/test_oracle.cpp:313-331
    H, S, D, gs = 3, 5, 24, 8
    k = oracle.normal_f64(H * S * D, 0xC1)
    v = oracle.normal_f64(H * S * D, 0xC2)
    c = oracle.quantize_cache_w4(k, v, H, S, D, gs, sym)
    kd = oracle.dequant_cache_w4(c, "k").reshape(H, S * D)
    for h in range(H):
        p = oracle.quantize_w4(k[h * S * D:(h + 1) * S * D], S, D, gs, sym)
        assert np.array_equal(oracle.dequant_all_w4(p), kd[h])


def test_kv_pins(oracle):
    # tests/test_oracle.cpp:333-379: zero K -> mean of the V rows exactly; huge scores stay finite
    H, S, D = 1, 2, 8
    v = np.concatenate([np.full(D, 1.0), np.full(D, 3.0)])
    c = oracle.quantize_cache_w4(np.zeros(S * D), v, H, S, D, 8, True)
    kd, vd = oracle.dequant_cache_w4(c, "k"), oracle.dequant_cache_w4(c, "v")
    q = np.full(D, 1.0, np.float16).view(np.uint16)
    out = oracle.attention_reference(q, kd, vd, H, S, D)
    want = 0.5 * f16(vd[:D]) + 0.5 * f16(vd[D:])
    assert np.array_equal(out, want)
    c = oracle.quantize_cache_w4(np.full(S * D, 100.0), np.full(S * D, 0.5), H, S, D, 8, True)
    kd, vd = oracle.dequant_cache_w4(c, "k"), oracle.dequant_cache_w4(c, "v")
    q = np.full(D, 100.0, np.float16).view(np.uint16)
    out = oracle.attention_reference(q, kd, vd, H, S, D)
    assert np.isfinite(out[0]) and out[0] == f16(vd[:1])[0]


def test_kv_throws(oracle):
    # tests/test_oracle.cpp:381-428
    ok = np.full(1 * 4 * 8, 0.5)
    for H, gs in [(0, 8), (1, 7), (1, 0)]:
        with pytest.raises(ValueError):
            oracle.quantize_cache_w4(ok, ok, H, 4, 8, gs, True)
    with pytest.raises(ValueError):
        oracle.quantize_cache_w4(np.zeros(10), ok, 1, 4, 8, 8, True)
    c = oracle.quantize_cache_w4(ok, ok, 1, 4, 8, 8, True)
    with pytest.raises(ValueError):
        oracle.dequant_cache_w4(dict(c, G=2), "k")


@pytest.mark.parametrize("i", range(len(cases.F8_HOST_CFGS)))
def test_f8_bounds(oracle, i):
    # tests/test_oracle.cpp:436-508: rounding-interval bound and amax <= 448*s*(1+1e-3)
    S, D = cases.F8_HOST_CFGS[i]
    gs = 32
    k = oracle.normal_f64(S * D, cases.f8_host_seed(i))
    v = oracle.normal_f64(S * D, cases.f8_host_seed(i) + 1)
    c = oracle.quantize_cache_f8(k, v, 1, S, D, gs)
    tab = np.array(sorted({abs(float(np.float32(x))) for x in
                           [_e4m3(b) for b in range(0x7F)]}))
    for side, src in (("k", k), ("v", v)):
        src = src.reshape(S, D)
        s = f16(c["s_" + side]).reshape(S, c["G"])[:, np.arange(D) // gs]
        wd = f16(oracle.dequant_cache_f8(c, side)).reshape(S, D)
        x = np.abs(src / s)
        j = np.clip(np.searchsorted(tab, x), 1, len(tab) - 1)
        gap = tab[j] - tab[j - 1]
        # one E4M3 rounding (half the bracketing gap) plus one FP16 rounding of the product
        assert np.all(np.abs(wd - src) <= (0.5 * gap * s) * (1 + 1e-9) + np.abs(src) * 2.0 ** -10 + 1e-12)
        for g in range(c["G"]):
            amax = np.abs(src[:, g * gs:(g + 1) * gs]).max(axis=1)
            assert np.all(amax <= 448.0 * f16(c["s_" + side]).reshape(S, c["G"])[:, g] * (1 + 1e-3))


def _e4m3(b):
    e, m = (b >> 3) & 0xF, b & 7
    mag = m * 2.0 ** -9 if e == 0 else (8 + m) * 2.0 ** (e - 10)
    return -mag if b & 0x80 else mag


def test_f8_pins(oracle):
    # tests/test_oracle.cpp:510-535: all 1.0 -> code 0x7E, dequant 1.0; all -2.0 -> -2.0 with bit 7
    c = oracle.quantize_cache_f8(np.full(64, 1.0), np.full(64, -2.0), 1, 2, 32, 32)
    assert set(c["q_k"].tolist()) == {0x7E}
    assert np.all(f16(oracle.dequant_cache_f8(c, "k")) == 1.0)
    assert np.all(c["q_v"] & 0x80) and np.all(f16(oracle.dequant_cache_f8(c, "v")) == -2.0)
    z = oracle.quantize_cache_f8(np.zeros(64), np.zeros(64), 1, 2, 32, 32)
    assert not np.any(f16(oracle.dequant_cache_f8(z, "k")))
    for b in range(256):  # decode is the exact table; sign on zero survives
        assert oracle.dequant_one_f8(0x3C00, b) == int(np.float16(_e4m3(b)).view(np.uint16)) or (b & 0x7F) == 0
    assert oracle.dequant_one_f8(0x3C00, 0x80) == 0x8000


def test_f8_throws(oracle):
    ok = np.full(4 * 8, 0.5)
    for H, gs in [(0, 8), (1, 7), (1, 0)]:
        with pytest.raises(ValueError):
            oracle.quantize_cache_f8(ok, ok, H, 4, 8, gs)
    bad = ok.copy()
    bad[1] = np.nan
    with pytest.raises(ValueError):
        oracle.quantize_cache_f8(bad, ok, 1, 4, 8, 8)
    bad[1] = 1e300
    with pytest.raises(ValueError):
        oracle.quantize_cache_f8(ok, bad, 1, 4, 8, 8)


def test_paged_scatter_and_throws(oracle):
    # tests/test_oracle.cpp:612-675: bt-resolved pool row == contiguous row
    H, S, D, gs, page = 2, 37, 24, 8, 16
    bt = [2, 0, 1]
    for sym in (True, False):
        k = oracle.normal_f64(H * S * D, 0xD1)
        v = oracle.normal_f64(H * S * D, 0xD2)
        c = oracle.quantize_cache_w4(k, v, H, S, D, gs, sym)
        p = oracle.paged_from_contiguous(c, page, bt)
        wd = (D + 7) // 8
        pool = p["q_k"].reshape(H, p["npages"] * page, wd)
        src = c["q_k"].reshape(H, S, wd)
        for t in range(S):
            assert np.array_equal(pool[:, bt[t // page] * page + t % page], src[:, t])
        assert not np.any(pool[:, bt[2] * page + (S % page):bt[2] * page + page])  # tail rows stay zero
    with pytest.raises(ValueError):
        oracle.paged_from_contiguous(c, 0, bt)
    with pytest.raises(ValueError):
        oracle.paged_from_contiguous(c, page, [0, 1])
    with pytest.raises(ValueError):
        oracle.paged_from_contiguous(c, page, [0, 0, 1])
    with pytest.raises(ValueError):
        oracle.paged_from_contiguous(c, page, [0, 1, 3])
    assert oracle.validate_block_table([2, 0, 1], S, page, 3)
    assert not oracle.validate_block_table([2, 0, 1], S, page, 2)
    assert not oracle.validate_block_table([1, 0, 1], S, page, 3)
