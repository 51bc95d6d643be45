"""GPU parity of decode attention through the C ABI: the reference's device gates
for W4 (single-block and flash, tests/test_gpu.cu:506-924), FP16, FP8
(:930-1078) and paged W4 caches (:1085-1467) on its own shapes and seeds.

Gates, as in the reference: the k_out / v_out hooks reproduce dequant_head bit
for bit; the output is within rel L2 <= 1e-3 of the FP64 reference; a paged call
is byte-identical to the contiguous call over the same logical cache."""
import os

import numpy as np
import pytest

import cases
import w4a16_dequant_gemm_b200 as w4
from gpu_util import KvF8, KvW4, bits, dev, empty_f16, ptr, sync_ok

pytestmark = pytest.mark.gpu
TOL = 1e-3
GOLD = np.load(os.path.join(os.path.dirname(__file__), "golden", "golden.npz"))
KV_ALL = [("kv", i, c) for i, c in enumerate(cases.KV_CFGS)] + \
         [("kvlong", i, c) for i, c in enumerate(cases.KV_LONG_CFGS)]


def make_w4(oracle, cfg, seed, sym):
    H, S, D, gs = cfg
    c = oracle.quantize_cache_w4(oracle.normal_f64(H * S * D, seed), oracle.normal_f64(H * S * D, seed + 1),
                                 H, S, D, gs, sym)
    return c, oracle.normal_f16(H * D, seed + 2)


@pytest.mark.parametrize("sym", [True, False])
@pytest.mark.parametrize("name,i,cfg", KV_ALL)
def test_w4_attention(oracle, name, i, cfg, sym):
    H, S, D, gs = cfg
    seed = (cases.kv_seed if name == "kv" else cases.kv_long_seed)(i, sym)
    c, q = make_w4(oracle, cfg, seed, sym)
    kd, vd = oracle.dequant_cache_w4(c, "k"), oracle.dequant_cache_w4(c, "v")
    ref = GOLD[f"{name}/{'sym' if sym else 'asym'}/{i}/out"]  # the reference's own FP64 attention
    kv, q_d = KvW4(c), dev(q)
    entries = [w4.attention_w4_flash] + ([w4.attention_w4] if S <= 4096 else [])
    for fn in entries:
        out, k_out, v_out = empty_f16(H * D), empty_f16(H * S * D), empty_f16(H * S * D)
        fn(kv.desc, ptr(q_d), ptr(out), None, ptr(k_out), ptr(v_out))
        sync_ok()
        assert np.array_equal(bits(k_out), kd) and np.array_equal(bits(v_out), vd), fn.__name__
        assert cases.rel_l2(cases.f16(bits(out)), ref) <= TOL, fn.__name__
        out2 = empty_f16(H * D)
        fn(kv.desc, ptr(q_d), ptr(out2))
        sync_ok()
        assert np.array_equal(bits(out), bits(out2))
    # FP16 cache holding the dequantised values: same reference (tests/test_gpu.cu:700-781)
    out = empty_f16(H * D)
    kd_d, vd_d = dev(kd), dev(vd)  # keep the device buffers alive across the launches
    w4.attention_fp16_flash(ptr(q_d), ptr(kd_d), ptr(vd_d), ptr(out), H, S, D)
    sync_ok()
    assert cases.rel_l2(cases.f16(bits(out)), ref) <= TOL
    if S <= 4096:
        out1 = empty_f16(H * D)
        w4.attention_fp16(ptr(q_d), ptr(kd_d), ptr(vd_d), ptr(out1), H, S, D)
        sync_ok()
        assert cases.rel_l2(cases.f16(bits(out1)), ref) <= TOL


@pytest.mark.parametrize("i", range(len(cases.KV_CFGS) + 1))
def test_f8_attention(oracle, i):
    H, S, D, gs = (cases.KV_CFGS + [cases.KV_LONG_CFGS[1]])[i]
    seed = cases.f8_gpu_seed(i)
    c = oracle.quantize_cache_f8(oracle.normal_f64(H * S * D, seed), oracle.normal_f64(H * S * D, seed + 1),
                                 H, S, D, gs)
    q = oracle.normal_f16(H * D, seed + 2)
    kd, vd = oracle.dequant_cache_f8(c, "k"), oracle.dequant_cache_f8(c, "v")
    ref = GOLD[f"f8/{i}/out"]
    kv, q_d = KvF8(c), dev(q)
    out, k_out, v_out = empty_f16(H * D), empty_f16(H * S * D), empty_f16(H * S * D)
    w4.attention_f8_flash(kv.desc, ptr(q_d), ptr(out), None, ptr(k_out), ptr(v_out))
    sync_ok()
    assert np.array_equal(bits(k_out), kd) and np.array_equal(bits(v_out), vd)
    assert cases.rel_l2(cases.f16(bits(out)), ref) <= TOL


@pytest.mark.parametrize("sym", [True, False])
@pytest.mark.parametrize("i", range(len(cases.PAGED_CFGS)))
def test_paged_equals_contiguous(oracle, i, sym):
    H, S, D, gs, page = cases.PAGED_CFGS[i]
    seed = cases.paged_seed(i, sym)
    c, q = make_w4(oracle, (H, S, D, gs), seed, sym)
    lp = (S + page - 1) // page
    bt = np.random.default_rng(seed ^ 0x5ED).permutation(lp).astype(np.int32)  # shuffled placement
    pool = oracle.paged_from_contiguous(c, page, bt)
    kd, vd = oracle.dequant_cache_w4(c, "k"), oracle.dequant_cache_w4(c, "v")
    ref = oracle.attention_reference(q, kd, vd, H, S, D)
    q_d, bt_d = dev(q), dev(bt)
    flat, paged = KvW4(c), KvW4(pool)
    out_c = empty_f16(H * D)
    w4.attention_w4_flash(flat.desc, ptr(q_d), ptr(out_c))
    out_p, k_out, v_out = empty_f16(H * D), empty_f16(H * S * D), empty_f16(H * S * D)
    w4.attention_w4_flash_paged(paged.desc, ptr(bt_d), page, lp, ptr(q_d), ptr(out_p), None, ptr(k_out), ptr(v_out))
    sync_ok()
    assert np.array_equal(bits(out_p), bits(out_c))          # tests/test_gpu.cu:1085-1310: memcmp
    assert np.array_equal(bits(k_out), kd) and np.array_equal(bits(v_out), vd)  # hooks in logical order
    assert cases.rel_l2(cases.f16(bits(out_p)), ref) <= TOL


def test_prefix_sharing(oracle):
    """One pool holds sequence B (520 positions) and its 200-position prefix A through
    btA = btB[:13]; A is launched with S = 200 but the pool's npages (tests/test_gpu.cu:1316-1467)."""
    H, D, gs, page, S2, S1 = 2, 64, 32, 16, 520, 200
    c, q = make_w4(oracle, (H, S2, D, gs), 0xABCD, True)
    lp = (S2 + page - 1) // page
    bt = np.random.default_rng(3).permutation(lp).astype(np.int32)
    pool = oracle.paged_from_contiguous(c, page, bt)
    kd = oracle.dequant_cache_w4(c, "k").reshape(H, S2, D)
    vd = oracle.dequant_cache_w4(c, "v").reshape(H, S2, D)
    q_d, bt_d, paged = dev(q), dev(bt), KvW4(pool)
    for S in (S2, S1):
        ref = oracle.attention_reference(q, np.ascontiguousarray(kd[:, :S]).ravel(),
                                         np.ascontiguousarray(vd[:, :S]).ravel(), H, S, D)
        desc = KvW4.__new__(KvW4)
        desc.t = paged.t
        d = paged.desc
        desc.desc = w4.DeviceKVW4(H, S, D, gs, d.G, 1, d.q_k, d.s_k, None, d.q_v, d.s_v, None)
        out = empty_f16(H * D)
        w4.attention_w4_flash_paged(desc.desc, ptr(bt_d), page, lp, ptr(q_d), ptr(out))
        sync_ok()
        assert cases.rel_l2(cases.f16(bits(out)), ref) <= TOL, S


@pytest.mark.parametrize("fmt", ["fp16", "w4", "f8"])
def test_baseline_c4_shape(oracle, fmt):
    """BASELINE config 4 geometry (D = 128, gs = 32) at B*H = 8, S = 8192: FP16 / W4 / FP8."""
    H, S, D, gs = 8, 8192, 128, 32
    rng = np.random.default_rng(11)
    k, v = rng.standard_normal(H * S * D), rng.standard_normal(H * S * D)
    q = rng.standard_normal(H * D).astype(np.float16).view(np.uint16)
    q_d, out = dev(q), empty_f16(H * D)
    if fmt == "fp16":
        kd, vd = k.astype(np.float16).view(np.uint16), v.astype(np.float16).view(np.uint16)
        kd_d, vd_d = dev(kd), dev(vd)
        w4.attention_fp16_flash(ptr(q_d), ptr(kd_d), ptr(vd_d), ptr(out), H, S, D)
    elif fmt == "w4":
        c = oracle.quantize_cache_w4(k, v, H, S, D, gs, True)
        kd, vd = oracle.dequant_cache_w4(c, "k"), oracle.dequant_cache_w4(c, "v")
        kv = KvW4(c)
        w4.attention_w4_flash(kv.desc, ptr(q_d), ptr(out))
    else:
        c = oracle.quantize_cache_f8(k, v, H, S, D, gs)
        kd, vd = oracle.dequant_cache_f8(c, "k"), oracle.dequant_cache_f8(c, "v")
        kv = KvF8(c)
        w4.attention_f8_flash(kv.desc, ptr(q_d), ptr(out))
    sync_ok()
    ref = oracle.attention_reference(q, kd, vd, H, S, D, threads=8)
    assert cases.rel_l2(cases.f16(bits(out)), ref) <= TOL


# Every (head size, group size) the tensor-pipe kernel serves, at ragged lengths that leave partial
# 16-position blocks and partial 64-position slices; W4 symmetric / asymmetric and FP8, with hooks.
MMA_MATRIX = [(D, gs, S) for D in (64, 128) for gs in (32, 64, 128) if gs <= D for S in (17, 333)] + \
             [(128, 32, 2049), (64, 32, 1280)]


@pytest.mark.parametrize("fmt", ["w4sym", "w4asym", "f8"])
@pytest.mark.parametrize("D,gs,S", MMA_MATRIX)
def test_tensor_pipe_matrix(oracle, fmt, D, gs, S):
    H = 3
    seed = 0x3A7 + 131 * D + 17 * gs + S
    kf, vf = oracle.normal_f64(H * S * D, seed), oracle.normal_f64(H * S * D, seed + 1)
    q = oracle.normal_f16(H * D, seed + 2)
    q_d = dev(q)
    out, k_out, v_out = empty_f16(H * D), empty_f16(H * S * D), empty_f16(H * S * D)
    if fmt == "f8":
        c = oracle.quantize_cache_f8(kf, vf, H, S, D, gs)
        kd, vd = oracle.dequant_cache_f8(c, "k"), oracle.dequant_cache_f8(c, "v")
        kv = KvF8(c)
        call = lambda o, ko=None, vo=None: w4.attention_f8_flash(kv.desc, ptr(q_d), ptr(o), None, ko, vo)
    else:
        c = oracle.quantize_cache_w4(kf, vf, H, S, D, gs, fmt == "w4sym")
        kd, vd = oracle.dequant_cache_w4(c, "k"), oracle.dequant_cache_w4(c, "v")
        kv = KvW4(c)
        call = lambda o, ko=None, vo=None: w4.attention_w4_flash(kv.desc, ptr(q_d), ptr(o), None, ko, vo)
    call(out, ptr(k_out), ptr(v_out))
    sync_ok()
    assert np.array_equal(bits(k_out), kd) and np.array_equal(bits(v_out), vd)  # hooks: bitwise
    ref = oracle.attention_reference(q, kd, vd, H, S, D)
    assert cases.rel_l2(cases.f16(bits(out)), ref) <= TOL
    out2 = empty_f16(H * D)
    call(out2)
    sync_ok()
    assert np.array_equal(bits(out), bits(out2))  # with and without hooks: the same bits
    # the FP16 entry over the dequantised cache
    out3, kd_d, vd_d = empty_f16(H * D), dev(kd), dev(vd)
    w4.attention_fp16_flash(ptr(q_d), ptr(kd_d), ptr(vd_d), ptr(out3), H, S, D)
    sync_ok()
    assert cases.rel_l2(cases.f16(bits(out3)), ref) <= TOL
    if fmt != "f8":
        # a paged copy with a page size that is no multiple of the kernel's 16-position block
        page = 24
        lp = (S + page - 1) // page
        bt = np.random.default_rng(seed).permutation(lp).astype(np.int32)
        pool = oracle.paged_from_contiguous(c, page, bt)
        paged, bt_d, out_p = KvW4(pool), dev(bt), empty_f16(H * D)
        w4.attention_w4_flash_paged(paged.desc, ptr(bt_d), page, lp, ptr(q_d), ptr(out_p))
        sync_ok()
        assert np.array_equal(bits(out_p), bits(out))
