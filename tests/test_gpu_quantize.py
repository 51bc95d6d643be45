"""GPU parity: the device-side quantizers and the KV append produce the bits of the
host quantizers (quantize, include/w4/pack.hpp:64-130; quantize_mx, include/w4/mx.hpp:71-119;
quantize_cache, include/w4/kvcache.hpp:60-108; quantize_cache_f8, include/w4/kvfp8.hpp:70-128)
on the reference's own shapes and seeds (tests/test_oracle.cpp, tests/test_gpu.cu).
Bar: bit-exact codes, scales and zero points."""
import numpy as np
import pytest
import torch

import cases
import w4a16_dequant_gemm_b200 as w4
from gpu_util import KvF8, KvW4, bits, dev, empty_f16, ptr, sync_ok

pytestmark = pytest.mark.gpu


def words(n):
    return (n + 7) // 8


def junk(n, dtype):
    """A destination that holds stale bits: the kernels must overwrite all of it."""
    return torch.full((int(n),), -1, dtype=dtype, device="cuda")


def u32(t):
    return t.cpu().numpy().view(np.uint32).ravel()


def u16(t):
    return t.cpu().numpy().view(np.uint16).ravel()


def f64_dev(a):
    return torch.from_numpy(np.ascontiguousarray(a, np.float64)).cuda()


def quantize_w4_dev(w_d, N, K, gs, sym, f16=False):
    G = (K + gs - 1) // gs
    q, s = junk(N * words(K), torch.int32), junk(N * G, torch.int16)
    z = None if sym else junk(N * words(G), torch.int32)
    w4.quantize(ptr(w_d), N, K, gs, sym, ptr(q), ptr(s), ptr(z), f16=f16)
    sync_ok()
    return u32(q), u16(s), None if sym else u32(z)


@pytest.mark.parametrize("sym", [True, False])
@pytest.mark.parametrize("i", range(len(cases.GEMM_CFGS)))
def test_quantize_w4_reference_shapes(oracle, i, sym):
    M, N, K, gs = cases.GEMM_CFGS[i]
    w = oracle.normal_f64(N * K, cases.w4_seed(i, sym))
    p = oracle.quantize_w4(w, N, K, gs, sym)
    q, s, z = quantize_w4_dev(f64_dev(w), N, K, gs, sym)
    assert np.array_equal(q, p["q"]) and np.array_equal(s, p["scales"])
    if not sym:
        assert np.array_equal(z, p["zeros"])


@pytest.mark.parametrize("sym", [True, False])
@pytest.mark.parametrize("N,K,gs", [(257, 4096, 128), (64, 1000, 64), (33, 2048, 32), (5, 520, 8), (3, 4100, 128)])
def test_quantize_w4_model_shapes(oracle, N, K, gs, sym):
    """Weight-scale values (sigma 0.02), many groups per row (several zero words), ragged K."""
    w = oracle.normal_f64(N * K, 0xA11 + N + gs) * 0.02
    w[:K // 2] = 0.0                                  # all-zero groups: scale 1, codes = zero point
    p = oracle.quantize_w4(w, N, K, gs, sym)
    q, s, z = quantize_w4_dev(f64_dev(w), N, K, gs, sym)
    assert np.array_equal(q, p["q"]) and np.array_equal(s, p["scales"])
    if not sym:
        assert np.array_equal(z, p["zeros"])


@pytest.mark.parametrize("sym", [True, False])
def test_quantize_w4_from_f16(oracle, sym):
    """FP16 sources are widened exactly: same bits as the host quantizer on the widened values."""
    N, K, gs = 96, 1024, 128
    x16 = oracle.normal_f16(N * K, 0xF16)
    p = oracle.quantize_w4(cases.f16(x16), N, K, gs, sym)
    q, s, z = quantize_w4_dev(dev(x16), N, K, gs, sym, f16=True)
    assert np.array_equal(q, p["q"]) and np.array_equal(s, p["scales"])
    if not sym:
        assert np.array_equal(z, p["zeros"])


@pytest.mark.parametrize("i", range(len(cases.MX_HOST_CFGS) + len(cases.GEMM_CFGS)))
def test_quantize_mx_reference_shapes(oracle, i):
    if i < len(cases.MX_HOST_CFGS):
        _, N, K = cases.MX_HOST_CFGS[i]
        seed = cases.mx_host_seed(i)
    else:
        j = i - len(cases.MX_HOST_CFGS)
        _, N, K, _ = cases.GEMM_CFGS[j]
        seed = cases.mx_gpu_seed(j)
    w = oracle.normal_f64(N * K, seed)
    p = oracle.quantize_mx(w, N, K)
    q, s = junk(N * words(K), torch.int32), junk(N * p["B"], torch.uint8)
    w4.quantize_mx(ptr(f64_dev(w)), N, K, ptr(q), ptr(s))
    sync_ok()
    assert np.array_equal(u32(q), p["q"]) and np.array_equal(s.cpu().numpy(), p["scales"])


def test_quantize_mx_scales_and_ties(oracle):
    """Magnitudes across 60 binades, exact ties between E2M1 steps, block maxima exactly on 6 * 2^e
    (the boundary of the shared exponent), zero blocks, a ragged last block."""
    N, K = 64, 200
    rng = np.random.default_rng(7)
    w = rng.standard_normal(N * K) * np.exp2(rng.integers(-30, 30, N * K).astype(np.float64))
    w = w.reshape(N, K)
    w[0, :] = 0.0
    w[1, :32] = np.tile([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 6.0], 4)   # ties at scale 1
    w[2, :32] = -w[1, :32] * 2.0 ** -9
    w[3, :32] = 6.0 * 2.0 ** 5 * np.sign(rng.standard_normal(32))          # amax on the boundary
    w[4, :32] = np.nextafter(6.0 * 2.0 ** 5, np.inf)                         # just above it
    w = w.ravel()
    p = oracle.quantize_mx(w, N, K)
    q, s = junk(N * words(K), torch.int32), junk(N * p["B"], torch.uint8)
    w4.quantize_mx(ptr(f64_dev(w)), N, K, ptr(q), ptr(s))
    sync_ok()
    assert np.array_equal(s.cpu().numpy(), p["scales"])
    assert np.array_equal(u32(q), p["q"])


@pytest.mark.parametrize("i", range(2 * len(cases.F8_HOST_CFGS)))
def test_quantize_f8_reference_shapes(oracle, i):
    j = i % len(cases.F8_HOST_CFGS)
    S, D = cases.F8_HOST_CFGS[j]
    seed = cases.f8_host_seed(j) if i < len(cases.F8_HOST_CFGS) else cases.f8_gpu_seed(j)
    H, gs = 2, 32
    k, v = oracle.normal_f64(H * S * D, seed), oracle.normal_f64(H * S * D, seed + 1)
    c = oracle.quantize_cache_f8(k, v, H, S, D, gs)
    for side, src in (("k", k), ("v", v)):
        q, s = junk(H * S * D, torch.uint8), junk(H * S * c["G"], torch.int16)
        w4.quantize_f8(ptr(f64_dev(src)), H * S, D, gs, ptr(q), ptr(s))
        sync_ok()
        assert np.array_equal(q.cpu().numpy(), c["q_" + side]) and np.array_equal(u16(s), c["s_" + side])


@pytest.mark.parametrize("sym", [True, False])
@pytest.mark.parametrize("i", [0, 1, 2, 3, 4])
def test_kv_append_w4_contiguous(oracle, i, sym):
    """Appending position after position gives the cache quantize_cache gives all at once."""
    H, S, D, gs = cases.KV_CFGS[i]
    S = min(S, 40)
    seed = cases.kv_seed(i, sym)
    k, v = oracle.normal_f64(H * S * D, seed), oracle.normal_f64(H * S * D, seed + 1)
    c = oracle.quantize_cache_w4(k, v, H, S, D, gs, sym)
    G = c["G"]
    t = {"q_k": junk(H * S * words(D), torch.int32), "s_k": junk(H * S * G, torch.int16),
         "q_v": junk(H * S * words(D), torch.int32), "s_v": junk(H * S * G, torch.int16),
         "z_k": None if sym else junk(H * S * words(G), torch.int32),
         "z_v": None if sym else junk(H * S * words(G), torch.int32)}
    desc = w4.DeviceKVW4(H, S, D, gs, G, int(sym), ptr(t["q_k"]), ptr(t["s_k"]), ptr(t["z_k"]), ptr(t["q_v"]),
                         ptr(t["s_v"]), ptr(t["z_v"]))
    k3, v3 = k.reshape(H, S, D), v.reshape(H, S, D)
    for pos in range(S):
        k_new, v_new = f64_dev(k3[:, pos, :]), f64_dev(v3[:, pos, :])
        w4.kv_append_w4(desc, pos, S, ptr(k_new), ptr(v_new))
    sync_ok()
    for key in t:
        if t[key] is not None:
            got = u16(t[key]) if key.startswith("s_") else u32(t[key])
            assert np.array_equal(got, c[key]), key


@pytest.mark.parametrize("sym", [True, False])
@pytest.mark.parametrize("i", [0, 3])
def test_kv_append_w4_paged_then_attention(oracle, i, sym):
    """A decode loop: FP16 K / V rows appended into a paged pool through a shuffled block table; the
    pool equals the host-quantised cache scattered into pages, and paged attention over it gives the
    bits it gives over that host-built pool."""
    H, S, D, gs, page = cases.PAGED_CFGS[i]
    S = min(S, 70)
    seed = cases.paged_seed(i, sym)
    k16, v16 = oracle.normal_f16(H * S * D, seed), oracle.normal_f16(H * S * D, seed + 1)
    q = oracle.normal_f16(H * D, seed + 2)
    c = oracle.quantize_cache_w4(cases.f16(k16), cases.f16(v16), H, S, D, gs, sym)
    lp = (S + page - 1) // page
    bt = np.random.default_rng(seed ^ 0x5ED).permutation(lp).astype(np.int32)
    pool = oracle.paged_from_contiguous(c, page, bt)
    host, G = KvW4(pool), c["G"]
    rows = lp * page
    zero = lambda n, dt: torch.zeros(int(n), dtype=dt, device="cuda")   # host pools pad unused rows with zero
    t = {"q_k": zero(H * rows * words(D), torch.int32), "s_k": zero(H * rows * G, torch.int16),
         "q_v": zero(H * rows * words(D), torch.int32), "s_v": zero(H * rows * G, torch.int16),
         "z_k": None if sym else zero(H * rows * words(G), torch.int32),
         "z_v": None if sym else zero(H * rows * words(G), torch.int32)}
    desc = w4.DeviceKVW4(H, S, D, gs, G, int(sym), ptr(t["q_k"]), ptr(t["s_k"]), ptr(t["z_k"]), ptr(t["q_v"]),
                         ptr(t["s_v"]), ptr(t["z_v"]))
    k_d, v_d = dev(k16).view(H, S, D), dev(v16).view(H, S, D)
    for pos in range(S):
        row = int(bt[pos // page]) * page + pos % page
        k_new, v_new = k_d[:, pos, :].contiguous(), v_d[:, pos, :].contiguous()
        w4.kv_append_w4(desc, row, rows, ptr(k_new), ptr(v_new), f16=True)
    sync_ok()
    for key in t:
        if t[key] is not None:
            got = u16(t[key]) if key.startswith("s_") else u32(t[key])
            assert np.array_equal(got, pool[key]), key
    q_d, bt_d = dev(q), dev(bt)
    out_a, out_h = empty_f16(H * D), empty_f16(H * D)
    w4.attention_w4_flash_paged(desc, ptr(bt_d), page, lp, ptr(q_d), ptr(out_a))
    w4.attention_w4_flash_paged(host.desc, ptr(bt_d), page, lp, ptr(q_d), ptr(out_h))
    sync_ok()
    assert np.array_equal(bits(out_a), bits(out_h))
    ref = oracle.attention_reference(q, oracle.dequant_cache_w4(c, "k"), oracle.dequant_cache_w4(c, "v"), H, S, D)
    assert cases.rel_l2(cases.f16(bits(out_a)), ref) <= 1e-3


@pytest.mark.parametrize("i", [0, 1, 2, 3, 4])
def test_kv_append_f8(oracle, i):
    S, D = cases.F8_HOST_CFGS[i]
    H, gs = 3, 32
    seed = cases.f8_gpu_seed(i)
    k, v = oracle.normal_f64(H * S * D, seed), oracle.normal_f64(H * S * D, seed + 1)
    c = oracle.quantize_cache_f8(k, v, H, S, D, gs)
    G = c["G"]
    t = {"q_k": junk(H * S * D, torch.uint8), "s_k": junk(H * S * G, torch.int16),
         "q_v": junk(H * S * D, torch.uint8), "s_v": junk(H * S * G, torch.int16)}
    desc = w4.DeviceKVF8(H, S, D, gs, G, ptr(t["q_k"]), ptr(t["s_k"]), ptr(t["q_v"]), ptr(t["s_v"]))
    k3, v3 = k.reshape(H, S, D), v.reshape(H, S, D)
    for pos in range(S):
        k_new, v_new = f64_dev(k3[:, pos, :]), f64_dev(v3[:, pos, :])
        w4.kv_append_f8(desc, pos, ptr(k_new), ptr(v_new))
    sync_ok()
    for key in t:
        got = u16(t[key]) if key.startswith("s_") else t[key].cpu().numpy()
        assert np.array_equal(got, c[key]), key


def test_quantizer_value_errors_reach_status(oracle):
    """What the host quantizer throws on for values (pack.hpp:84-104: a non-finite value, a scale
    beyond FP16) is reported through the device status word; the next call is clean."""
    N, K, gs = 4, 64, 32
    w = oracle.normal_f64(N * K, 5)
    for poison in (np.inf, np.nan, 1e9):   # 1e9 / 7 overflows an FP16 scale
        bad = w.copy()
        bad[70] = poison
        with pytest.raises(ValueError):
            oracle.quantize_w4(bad, N, K, gs, True)
        q, s = junk(N * words(K), torch.int32), junk(N * 2, torch.int16)
        w4.quantize(ptr(f64_dev(bad)), N, K, gs, True, ptr(q), ptr(s), None)
        assert w4.device_status() == 501
        assert w4.device_status() == 0
    q, s = junk(N * words(K), torch.int32), junk(N * 2, torch.int16)
    w4.quantize(ptr(f64_dev(w)), N, K, gs, True, ptr(q), ptr(s), None)
    sync_ok()
    assert np.array_equal(u32(q), oracle.quantize_w4(w, N, K, gs, True)["q"])


def test_quantizer_shape_contract():
    """Shape errors answer as the host quantizers do (pack.hpp:66-75), before any launch."""
    buf = torch.zeros(4096, dtype=torch.float64, device="cuda")
    o = torch.zeros(4096, dtype=torch.int32, device="cuda")
    for N, K, gs in [(0, 64, 32), (4, 0, 32), (4, 64, 4), (4, 64, 12), (4, 64, 0)]:
        with pytest.raises(w4.InvalidArgument):
            w4.quantize(ptr(buf), N, K, gs, True, ptr(o), ptr(o), None)
    with pytest.raises(w4.InvalidArgument):
        w4.quantize(ptr(buf), 4, 64, 32, False, ptr(o), ptr(o), None)   # asymmetric without zeros
    with pytest.raises(w4.InvalidArgument):
        w4.quantize_mx(ptr(buf), 0, 64, ptr(o), ptr(o))
    with pytest.raises(w4.InvalidArgument):
        w4.quantize_f8(ptr(buf), 4, 64, 12, ptr(o), ptr(o))
