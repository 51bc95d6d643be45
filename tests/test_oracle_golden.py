"""The oracle against the committed golden vectors (made by the reference's own
host code through tests/golden/make_golden.py): bitwise artefacts by sha256,
FP64 GEMM / attention outputs exactly."""
import os

import numpy as np
import pytest

import cases

GOLD = np.load(os.path.join(os.path.dirname(__file__), "golden", "golden.npz"))


def gold(key):
    v = GOLD[key]
    return str(v) if v.dtype.kind == "U" else v


@pytest.mark.parametrize("sym", [True, False])
@pytest.mark.parametrize("i", range(len(cases.GEMM_CFGS)))
def test_w4_golden(oracle, i, sym):
    M, N, K, gs = cases.GEMM_CFGS[i]
    seed = cases.w4_seed(i, sym)
    w = oracle.normal_f64(N * K, seed)
    x = oracle.normal_f16(M * K, seed + 1)
    p = oracle.quantize_w4(w, N, K, gs, sym)
    wd = oracle.dequant_all_w4(p)
    key = f"w4/{'sym' if sym else 'asym'}/{i}"
    assert cases.digest(p["q"], p["scales"], p["zeros"]) == gold(key + "/packed")
    assert cases.digest(wd) == gold(key + "/dequant")
    assert cases.digest(x) == gold(key + "/x")
    c = oracle.gemm_oracle(x, M, K, wd, N)
    assert np.array_equal(c, gold(key + "/c"))
    assert np.array_equal(oracle.gemm_oracle(x, M, K, wd, N, threads=3), c)


@pytest.mark.parametrize("i", range(len(cases.MX_HOST_CFGS)))
def test_mx_host_golden(oracle, i):
    M, N, K = cases.MX_HOST_CFGS[i]
    p = oracle.quantize_mx(oracle.normal_f64(N * K, cases.mx_host_seed(i)), N, K)
    assert cases.digest(p["q"], p["scales"]) == gold(f"mxhost/{i}/packed")
    assert cases.digest(oracle.dequant_all_mx(p)) == gold(f"mxhost/{i}/dequant")


@pytest.mark.parametrize("i", range(len(cases.GEMM_CFGS)))
def test_mx_golden(oracle, i):
    M, N, K, _ = cases.GEMM_CFGS[i]
    seed = cases.mx_gpu_seed(i)
    p = oracle.quantize_mx(oracle.normal_f64(N * K, seed), N, K)
    wd = oracle.dequant_all_mx(p)
    assert cases.digest(p["q"], p["scales"]) == gold(f"mx/{i}/packed")
    assert cases.digest(wd) == gold(f"mx/{i}/dequant")
    x = oracle.normal_f16(M * K, seed + 1)
    assert np.array_equal(oracle.gemm_oracle(x, M, K, wd, N), gold(f"mx/{i}/c"))


KV_ALL = [("kv", i, c) for i, c in enumerate(cases.KV_CFGS)] + [("kvlong", i, c) for i, c in enumerate(cases.KV_LONG_CFGS)]


@pytest.mark.parametrize("sym", [True, False])
@pytest.mark.parametrize("name,i,cfg", KV_ALL)
def test_kv_golden(oracle, name, i, cfg, sym):
    H, S, D, gs = cfg
    seed = (cases.kv_seed if name == "kv" else cases.kv_long_seed)(i, sym)
    k = oracle.normal_f64(H * S * D, seed)
    v = oracle.normal_f64(H * S * D, seed + 1)
    q = oracle.normal_f16(H * D, seed + 2)
    c = oracle.quantize_cache_w4(k, v, H, S, D, gs, sym)
    kd, vd = oracle.dequant_cache_w4(c, "k"), oracle.dequant_cache_w4(c, "v")
    key = f"{name}/{'sym' if sym else 'asym'}/{i}"
    assert cases.digest(c["q_k"], c["s_k"], c["z_k"], c["q_v"], c["s_v"], c["z_v"]) == gold(key + "/packed")
    assert cases.digest(kd, vd) == gold(key + "/dequant")
    out = oracle.attention_reference(q, kd, vd, H, S, D)
    assert np.array_equal(out, gold(key + "/out"))
    assert np.array_equal(oracle.attention_reference(q, kd, vd, H, S, D, threads=2), out)


@pytest.mark.parametrize("i", range(len(cases.KV_CFGS) + 1))
def test_f8_golden(oracle, i):
    H, S, D, gs = (cases.KV_CFGS + [cases.KV_LONG_CFGS[1]])[i]
    seed = cases.f8_gpu_seed(i)
    k = oracle.normal_f64(H * S * D, seed)
    v = oracle.normal_f64(H * S * D, seed + 1)
    q = oracle.normal_f16(H * D, seed + 2)
    c = oracle.quantize_cache_f8(k, v, H, S, D, gs)
    kd, vd = oracle.dequant_cache_f8(c, "k"), oracle.dequant_cache_f8(c, "v")
    assert cases.digest(c["q_k"], c["s_k"], c["q_v"], c["s_v"]) == gold(f"f8/{i}/packed")
    assert cases.digest(kd, vd) == gold(f"f8/{i}/dequant")
    assert np.array_equal(oracle.attention_reference(q, kd, vd, H, S, D), gold(f"f8/{i}/out"))


@pytest.mark.parametrize("sym", [True, False])
@pytest.mark.parametrize("i", range(len(cases.PAGED_CFGS)))
def test_paged_golden(oracle, i, sym):
    H, S, D, gs, page = cases.PAGED_CFGS[i]
    seed = cases.paged_seed(i, sym)
    c = oracle.quantize_cache_w4(oracle.normal_f64(H * S * D, seed), oracle.normal_f64(H * S * D, seed + 1),
                                 H, S, D, gs, sym)
    bt = np.random.default_rng(seed ^ 0x5ED).permutation((S + page - 1) // page).astype(np.int32)
    p = oracle.paged_from_contiguous(c, page, bt)
    assert cases.digest(p["q_k"], p["s_k"], p["z_k"], p["q_v"], p["s_v"], p["z_v"]) == \
        gold(f"paged/{'sym' if sym else 'asym'}/{i}/pool")
