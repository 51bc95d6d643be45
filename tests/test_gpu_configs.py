"""GPU parity at the sizes the benchmark configurations name, through the C ABI.

The reference's gates (tests/test_gpu.cu:54-62 for the GEMM matrix, :786-924 for long
sequences, :1085-1467 for paged caches and prefix sharing) are applied, with unchanged
tolerances (bitwise hooks, rel L2 <= 1e-3 against the FP64 oracle), to the shapes its
tests do not reach: M = 256 on both orientations of the W4 GEMM, M = 128 / 512 of the
MXFP4 GEMM, the tensor kernel's multi-tile M range, decode attention at S = 32768 with
512 heads and at the small end, the paged geometry of the 70B-shaped decode step, the
peer all-gather (looped back on one GPU) and sharded descriptors.

Where the FP64 oracle over the full output would take minutes, it runs on a sample of
rows / heads; the sampled outputs are compared exactly as the full ones would be."""
import os

import numpy as np
import pytest
import torch

import cases
import w4a16_dequant_gemm_b200 as w4
from gpu_util import KvF8, KvW4, MxWeights, W4Weights, bits, dev, empty_f16, ptr, sync_ok

pytestmark = pytest.mark.gpu
TOL = 1e-3
THREADS = os.cpu_count() or 8


def sample_rows(N, count, seed):
    """Sorted sample of weight rows that always holds the first and the last panel's rows."""
    rng = np.random.default_rng(seed)
    rows = set(rng.choice(N, size=min(count, N), replace=False).tolist())
    rows.update(range(0, min(16, N)))
    rows.update(range(max(0, N - 16), N))
    return np.array(sorted(rows), dtype=np.int64)


def check_sampled(oracle, c_bits, x, M, N, K, wd, rows):
    got = cases.f16(c_bits).reshape(M, N)[:, rows]
    sub = np.ascontiguousarray(wd.reshape(N, K)[rows]).ravel()
    ref = oracle.gemm_oracle(x, M, K, sub, len(rows), threads=THREADS).reshape(M, len(rows))
    assert cases.rel_l2(got, ref) <= TOL


_W4 = {}


def c2_weights(oracle, N, K):
    if (N, K) not in _W4:
        _W4.clear()
        p = oracle.quantize_w4(oracle.normal_f64(N * K, 0) * 0.02, N, K, 128, False)
        _W4[(N, K)] = (p, oracle.dequant_all_w4(p), W4Weights(p))
    return _W4[(N, K)]


@pytest.mark.parametrize("N,K", [(14336, 4096), (4096, 14336)])
def test_c2_m256(oracle, N, K):
    """Config 2 at M = 256 (the tensor kernel's widest accumulator), both orientations."""
    M = 256
    p, wd, wts = c2_weights(oracle, N, K)
    x = oracle.normal_f16(M * K, 1 + M)
    x_d, c = dev(x), empty_f16(M * N)
    c.fill_(float("nan"))
    w4.gemm(wts.desc, ptr(x_d), ptr(c), M)
    sync_ok()
    check_sampled(oracle, bits(c), x, M, N, K, wd, sample_rows(N, 768, N + K))


_MX = {}


@pytest.mark.parametrize("M", [128, 512])
def test_c3_mx_large_m(oracle, M):
    """Config 3 (MXFP4, N = K = 8192) at M = 128 and 512."""
    N = K = 8192
    if "p" not in _MX:
        p = oracle.quantize_mx(oracle.normal_f64(N * K, 0) * 0.02, N, K)
        _MX.update(p=p, wd=oracle.dequant_all_mx(p), wts=MxWeights(p))
    x = oracle.normal_f16(M * K, 1 + M)
    x_d, c = dev(x), empty_f16(M * N)
    c.fill_(float("nan"))
    w4.gemm_mx(_MX["wts"].desc, ptr(x_d), ptr(c), M)
    sync_ok()
    check_sampled(oracle, bits(c), x, M, N, K, _MX["wd"], sample_rows(N, 384, M))


@pytest.mark.parametrize("fmt", ["sym", "asym", "mx"])
@pytest.mark.parametrize("M", [128, 256, 300, 513])
def test_tensor_kernel_large_m(oracle, fmt, M):
    """The tensor kernel with 128..256 accumulator columns, several m-tiles and a short last tile: output
    against the oracle, the hook bitwise, hook and plain launches identical."""
    N, K, gs = 1000, 1024, 64
    w = oracle.normal_f64(N * K, 77 + M) * 0.02
    if fmt == "mx":
        p = oracle.quantize_mx(w, N, K)
        wd, wts, fn = oracle.dequant_all_mx(p), MxWeights(p), w4.gemm_mx
    else:
        p = oracle.quantize_w4(w, N, K, gs, fmt == "sym")
        wd, wts, fn = oracle.dequant_all_w4(p), W4Weights(p), w4.gemm
    x = oracle.normal_f16(M * K, 78 + M)
    x_d = dev(x)
    assert w4.gemm_route(wts.desc, M, w4.PATH_TENSOR, ptr(x_d)) == w4.PATH_TENSOR
    c, w_out = empty_f16(M * N), empty_f16(N * K)
    c.fill_(float("nan"))
    fn(wts.desc, ptr(x_d), ptr(c), M, None, ptr(w_out), path=w4.PATH_TENSOR)
    sync_ok()
    assert np.array_equal(bits(w_out), wd)
    ref = oracle.gemm_oracle(x, M, K, wd, N, threads=THREADS)
    assert cases.rel_l2(cases.f16(bits(c)), ref) <= TOL
    c2 = empty_f16(M * N)
    fn(wts.desc, ptr(x_d), ptr(c2), M, None, None, path=w4.PATH_TENSOR)
    sync_ok()
    assert np.array_equal(bits(c), bits(c2))


def _replicated(t, times):
    """Device tensor holding `times` copies of the head slabs in t (None passes through)."""
    return None if t is None else t.repeat(times)


@pytest.mark.parametrize("fmt", ["fp16", "w4", "f8"])
def test_c4_s32768_512_heads(oracle, fmt):
    """Config 4's largest case: B*H = 512 heads, S = 32768, D = 128, gs = 32. Four distinct head slabs are
    generated and quantised on the host, checked against the FP64 reference, and repeated 128 times on the
    device: every one of the 512 outputs must then carry the bits of its source head (head strides beyond
    2^31 elements included)."""
    H0, REP, S, D, gs = 4, 128, 32768, 128, 32
    H = H0 * REP
    rng = np.random.default_rng(2024)
    k, v = rng.standard_normal(H0 * S * D), rng.standard_normal(H0 * S * D)
    q = rng.standard_normal(H0 * D).astype(np.float16).view(np.uint16)
    q_d = dev(q).repeat(REP)
    out = empty_f16(H * D)
    out.fill_(float("nan"))
    if fmt == "fp16":
        kd, vd = k.astype(np.float16).view(np.uint16), v.astype(np.float16).view(np.uint16)
        kd_d, vd_d = dev(kd).repeat(REP), dev(vd).repeat(REP)
        w4.attention_fp16_flash(ptr(q_d), ptr(kd_d), ptr(vd_d), ptr(out), H, S, D)
    elif fmt == "w4":
        c = oracle.quantize_cache_w4(k, v, H0, S, D, gs, True)
        kd, vd = oracle.dequant_cache_w4(c, "k"), oracle.dequant_cache_w4(c, "v")
        t = {n: _replicated(dev(c[n]), REP) for n in ("q_k", "s_k", "q_v", "s_v")}
        desc = w4.DeviceKVW4(H, S, D, gs, c["G"], 1, ptr(t["q_k"]), ptr(t["s_k"]), None, ptr(t["q_v"]),
                             ptr(t["s_v"]), None)
        w4.attention_w4_flash(desc, ptr(q_d), ptr(out))
    else:
        c = oracle.quantize_cache_f8(k, v, H0, S, D, gs)
        kd, vd = oracle.dequant_cache_f8(c, "k"), oracle.dequant_cache_f8(c, "v")
        t = {n: _replicated(dev(c[n]), REP) for n in ("q_k", "s_k", "q_v", "s_v")}
        desc = w4.DeviceKVF8(H, S, D, gs, c["G"], ptr(t["q_k"]), ptr(t["s_k"]), ptr(t["q_v"]), ptr(t["s_v"]))
        w4.attention_f8_flash(desc, ptr(q_d), ptr(out))
    sync_ok()
    got = bits(out).reshape(REP, H0 * D)
    assert (got == got[0]).all(), "replicated heads disagree"
    ref = oracle.attention_reference(q, kd, vd, H0, S, D, threads=THREADS)
    assert cases.rel_l2(cases.f16(got[0]), ref) <= TOL


@pytest.mark.parametrize("fmt", ["fp16", "w4", "f8"])
def test_c4_small_end(oracle, fmt):
    """Config 4's smallest case: B*H = 8, S = 1024."""
    H, S, D, gs = 8, 1024, 128, 32
    rng = np.random.default_rng(7)
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
    assert cases.rel_l2(cases.f16(bits(out)), oracle.attention_reference(q, kd, vd, H, S, D, threads=8)) <= TOL


def test_c5_paged_geometry_two_sequences(oracle):
    """The paged KV geometry of the 70B-shaped decode step (16-token pages, D = 128, gs = 32, S = 4608 =
    4096 shared prefix + 512 own tokens), two sequences in one pool that share the prefix pages, each
    against its own FP64 reference and bit-identical to a contiguous call over the same logical cache."""
    H, D, gs, page, SP, SU = 4, 128, 32, 16, 4096, 512
    S = SP + SU
    rng = np.random.default_rng(5)
    pk, pv = rng.standard_normal((H, SP, D)), rng.standard_normal((H, SP, D))
    seqs = []
    for _ in range(2):
        uk, uv = rng.standard_normal((H, SU, D)), rng.standard_normal((H, SU, D))
        seqs.append((np.concatenate([pk, uk], axis=1), np.concatenate([pv, uv], axis=1)))
    # logical caches (quantisation is per position, so the shared prefix quantises identically in both)
    caches = [oracle.quantize_cache_w4(k.ravel(), v.ravel(), H, S, D, gs, True) for k, v in seqs]
    npre, nown = SP // page, SU // page
    npages = npre + 2 * nown
    perm = np.random.default_rng(9).permutation(npages).astype(np.int32)
    bts = [np.concatenate([perm[:npre], perm[npre + i * nown: npre + (i + 1) * nown]]).astype(np.int32)
           for i in range(2)]
    # one pool: scatter both logical caches (the prefix pages are written twice with the same bytes)
    wd, G = (D + 7) // 8, caches[0]["G"]
    rows = npages * page
    pool = {n: np.zeros((H, rows, w), dtype=caches[0][n].dtype)
            for n, w in (("q_k", wd), ("q_v", wd), ("s_k", G), ("s_v", G))}
    for c, bt in zip(caches, bts):
        for n, w in (("q_k", wd), ("q_v", wd), ("s_k", G), ("s_v", G)):
            src = c[n].reshape(H, S, w)
            for lp_, phys in enumerate(bt):
                pool[n][:, phys * page:(phys + 1) * page] = src[:, lp_ * page:(lp_ + 1) * page]
    t = {n: dev(a.ravel()) for n, a in pool.items()}
    desc = w4.DeviceKVW4(H, S, D, gs, G, 1, ptr(t["q_k"]), ptr(t["s_k"]), None, ptr(t["q_v"]), ptr(t["s_v"]), None)
    for c, bt in zip(caches, bts):
        q = oracle.normal_f16(H * D, int(bt[-1]) + 1)
        q_d, bt_d = dev(q), dev(bt)
        out_p, out_c = empty_f16(H * D), empty_f16(H * D)
        w4.attention_w4_flash_paged(desc, ptr(bt_d), page, npages, ptr(q_d), ptr(out_p))
        flat = KvW4(c)
        w4.attention_w4_flash(flat.desc, ptr(q_d), ptr(out_c))
        sync_ok()
        assert np.array_equal(bits(out_p), bits(out_c))
        ref = oracle.attention_reference(q, oracle.dequant_cache_w4(c, "k"), oracle.dequant_cache_w4(c, "v"), H, S, D,
                                         threads=8)
        assert cases.rel_l2(cases.f16(bits(out_p)), ref) <= TOL


def test_batched_paged_matches_per_sequence_calls(oracle):
    """The batched paged entry: sequences of different lengths over one pool (all prefixes of one another),
    one launch; every sequence's output must match the FP64 reference and the per-sequence entry (the two cut
    a sequence into different slices, so they agree to rounding, not to the bit), must not depend on the
    company it has in the call, and a call with one sequence must carry the bits of the per-sequence entry."""
    H, D, gs, page = 4, 128, 32, 16
    lens = [4608, 300, 4100, 16, 1]
    rng = np.random.default_rng(21)
    Smax = max(lens)
    k, v = rng.standard_normal((H, Smax, D)), rng.standard_normal((H, Smax, D))
    c = oracle.quantize_cache_w4(k.ravel(), v.ravel(), H, Smax, D, gs, True)  # per position: prefixes agree
    lp = (Smax + page - 1) // page
    npages = lp + 7
    perm = np.random.default_rng(22).permutation(npages).astype(np.int32)
    bt_long = perm[:lp]
    # the pool: the long sequence's pages scattered by its table (more pages than it needs)
    wd, G = (D + 7) // 8, c["G"]
    rows = npages * page
    pool = {}
    for n, w in (("q_k", wd), ("q_v", wd), ("s_k", G), ("s_v", G)):
        a = np.zeros((H, rows, w), dtype=c[n].dtype)
        src = np.zeros((H, lp * page, w), dtype=c[n].dtype)
        src[:, :Smax] = c[n].reshape(H, Smax, w)
        for i, phys in enumerate(bt_long):
            a[:, phys * page:(phys + 1) * page] = src[:, i * page:(i + 1) * page]
        pool[n] = a
    t = {n: dev(np.ascontiguousarray(pool[n]).ravel()) for n in ("q_k", "q_v", "s_k", "s_v")}
    # every sequence is a prefix of the long one: its table is the head of the long table
    nseq, stride = len(lens), lp + 3
    bt = np.zeros((nseq, stride), dtype=np.int32)
    for i, L in enumerate(lens):
        n_i = (L + page - 1) // page
        bt[i, :n_i] = bt_long[:n_i]
    qs = oracle.normal_f16(nseq * H * D, 23)
    q_d, bt_d, lens_d = dev(qs), dev(bt.ravel()), dev(np.array(lens, dtype=np.int32))
    desc = w4.DeviceKVW4(H, Smax, D, gs, G, 1, ptr(t["q_k"]), ptr(t["s_k"]), None, ptr(t["q_v"]), ptr(t["s_v"]), None)
    out_b = empty_f16(nseq * H * D)
    out_b.fill_(float("nan"))
    w4.attention_w4_flash_paged_batched(desc, ptr(bt_d), stride, ptr(lens_d), nseq, Smax, page, npages, ptr(q_d),
                                        ptr(out_b))
    sync_ok()
    got = bits(out_b).reshape(nseq, H * D)
    kd = oracle.dequant_cache_w4(c, "k").reshape(H, Smax, D)
    vd = oracle.dequant_cache_w4(c, "v").reshape(H, Smax, D)
    for i, L in enumerate(lens):
        d_i = w4.DeviceKVW4(H, L, D, gs, G, 1, ptr(t["q_k"]), ptr(t["s_k"]), None, ptr(t["q_v"]), ptr(t["s_v"]), None)
        out_1 = empty_f16(H * D)
        w4.attention_w4_flash_paged(d_i, ptr(bt_d) + 4 * i * stride, page, npages, ptr(q_d) + 2 * i * H * D, ptr(out_1))
        sync_ok()
        ref = oracle.attention_reference(qs[i * H * D:(i + 1) * H * D], np.ascontiguousarray(kd[:, :L]).ravel(),
                                         np.ascontiguousarray(vd[:, :L]).ravel(), H, L, D)
        assert cases.rel_l2(cases.f16(got[i]), ref) <= TOL, f"sequence {i}"
        assert cases.rel_l2(cases.f16(got[i]), cases.f16(bits(out_1))) <= TOL, f"sequence {i} (length {L})"
        # one sequence per batched call: the single-sequence geometry, hence its bits
        out_s = empty_f16(H * D)
        w4.attention_w4_flash_paged_batched(d_i, ptr(bt_d) + 4 * i * stride, stride, ptr(lens_d) + 4 * i, 1, L, page, npages,
                                            ptr(q_d) + 2 * i * H * D, ptr(out_s))
        sync_ok()
        assert np.array_equal(bits(out_s), bits(out_1)), f"sequence {i} alone"
    # the same sequences in another order and company: every output keeps its bits
    order = [2, 0, 4, 1, 3]
    bt2, lens2 = dev(bt[order].ravel()), dev(np.array([lens[i] for i in order], dtype=np.int32))
    q2 = dev(qs.reshape(nseq, H * D)[order].ravel())
    out_2 = empty_f16(nseq * H * D)
    w4.attention_w4_flash_paged_batched(desc, ptr(bt2), stride, ptr(lens2), nseq, Smax, page, npages, ptr(q2), ptr(out_2))
    sync_ok()
    got2 = bits(out_2).reshape(nseq, H * D)
    for j, i in enumerate(order):
        assert np.array_equal(got2[j], got[i]), f"sequence {i} moved to slot {j}"


@pytest.mark.parametrize("sym", [True, False])
@pytest.mark.parametrize("D,gs", [(128, 32), (64, 64)])
def test_batched_paged_shared_prefix_groups(oracle, D, gs, sym):
    """Sequences of equal length that share prefix pages and then own pages (config 5's geometry, scaled down),
    more than eight of them so that a full and a partial group of eight form: the batched entry decodes shared
    blocks once per group; every sequence must match the FP64 reference and its single-sequence call, and must
    carry the bits it gets when the same call serves it without sharing (a pool in which every sequence has
    pages of its own). The length is not a multiple of the page."""
    H, page, nseq = 3, 16, 11
    n_pre, n_own = 21, 5
    S = (n_pre + n_own) * page - 7
    rng = np.random.default_rng(31 + D)
    k_pre, v_pre = rng.standard_normal((H, n_pre * page, D)), rng.standard_normal((H, n_pre * page, D))
    npages = n_pre + nseq * n_own + 4
    perm = np.random.default_rng(32).permutation(npages).astype(np.int32)
    lp = n_pre + n_own
    wd, G = D // 8, D // gs
    rows = npages * page
    names = ("q_k", "q_v", "s_k", "s_v") + (() if sym else ("z_k", "z_v"))
    width = {"q_k": wd, "q_v": wd, "s_k": G, "s_v": G, "z_k": 1, "z_v": 1}
    pool, caches = {}, []
    bt = np.zeros((nseq, lp), dtype=np.int32)
    for i in range(nseq):
        k_i = np.concatenate([k_pre, rng.standard_normal((H, lp * page - n_pre * page, D))], axis=1)[:, :S]
        v_i = np.concatenate([v_pre, rng.standard_normal((H, lp * page - n_pre * page, D))], axis=1)[:, :S]
        c = oracle.quantize_cache_w4(np.ascontiguousarray(k_i).ravel(), np.ascontiguousarray(v_i).ravel(), H, S, D, gs, sym)
        caches.append(c)
        bt[i, :n_pre] = perm[:n_pre]
        bt[i, n_pre:] = perm[n_pre + i * n_own: n_pre + (i + 1) * n_own]
        for n in names:
            if n not in pool:
                pool[n] = np.zeros((H, rows, width[n]), dtype=c[n].dtype)
            src = np.zeros((H, lp * page, width[n]), dtype=c[n].dtype)
            src[:, :S] = c[n].reshape(H, S, width[n])
            for j, phys in enumerate(bt[i]):
                if i == 0 or j >= n_pre:
                    pool[n][:, phys * page:(phys + 1) * page] = src[:, j * page:(j + 1) * page]
    t = {n: dev(np.ascontiguousarray(pool[n]).ravel()) for n in names}
    zk, zv = (None, None) if sym else (ptr(t["z_k"]), ptr(t["z_v"]))
    desc = w4.DeviceKVW4(H, S, D, gs, G, int(sym), ptr(t["q_k"]), ptr(t["s_k"]), zk, ptr(t["q_v"]), ptr(t["s_v"]), zv)
    qs = oracle.normal_f16(nseq * H * D, 33)
    q_d, bt_d, lens_d = dev(qs), dev(bt.ravel()), dev(np.full(nseq, S, dtype=np.int32))
    out_b = empty_f16(nseq * H * D)
    out_b.fill_(float("nan"))
    w4.attention_w4_flash_paged_batched(desc, ptr(bt_d), lp, ptr(lens_d), nseq, S, page, npages, ptr(q_d), ptr(out_b))
    sync_ok()
    got = bits(out_b).reshape(nseq, H * D)
    for i in range(nseq):
        out_1 = empty_f16(H * D)
        w4.attention_w4_flash_paged(desc, ptr(bt_d) + 4 * i * lp, page, npages, ptr(q_d) + 2 * i * H * D, ptr(out_1))
        sync_ok()
        assert cases.rel_l2(cases.f16(got[i]), cases.f16(bits(out_1))) <= TOL, f"sequence {i}"
        if i in (0, 7, 10):
            c = caches[i]
            ref = oracle.attention_reference(qs[i * H * D:(i + 1) * H * D], oracle.dequant_cache_w4(c, "k"),
                                             oracle.dequant_cache_w4(c, "v"), H, S, D)
            assert cases.rel_l2(cases.f16(got[i]), ref) <= TOL, f"sequence {i}"
    # the same sequences without sharing: prefix pages copied per sequence into a larger pool, so that every block
    # runs once per sequence. Same slices, same order of sums: the bits must agree with the shared run.
    npages2 = nseq * lp
    rows2 = npages2 * page
    bt_own = np.arange(npages2, dtype=np.int32).reshape(nseq, lp)
    pool2 = {n: np.zeros((H, rows2, width[n]), dtype=pool[n].dtype) for n in names}
    for i in range(nseq):
        for j in range(lp):
            src, dst = int(bt[i, j]), int(bt_own[i, j])
            for n in names:
                pool2[n][:, dst * page:(dst + 1) * page] = pool[n][:, src * page:(src + 1) * page]
    t2 = {n: dev(np.ascontiguousarray(pool2[n]).ravel()) for n in names}
    zk2, zv2 = (None, None) if sym else (ptr(t2["z_k"]), ptr(t2["z_v"]))
    desc2 = w4.DeviceKVW4(H, S, D, gs, G, int(sym), ptr(t2["q_k"]), ptr(t2["s_k"]), zk2, ptr(t2["q_v"]), ptr(t2["s_v"]), zv2)
    bt_own_d = dev(bt_own.ravel())
    out_o = empty_f16(nseq * H * D)
    w4.attention_w4_flash_paged_batched(desc2, ptr(bt_own_d), lp, ptr(lens_d), nseq, S, page, npages2, ptr(q_d), ptr(out_o))
    sync_ok()
    assert np.array_equal(bits(out_o).reshape(nseq, H * D), got)


def test_peer_allgather_loopback():
    """The exchange kernels on one GPU: two arenas stand for two ranks, the pushes of a step are launched one
    after the other on one stream (a push only waits for the OTHER rank's previous step, which an earlier
    launch has posted), then both ranks wait for the current step. Every slice must land in the peer's
    arena, over more steps than there are slice buffers."""
    world, nbytes = 2, 28672
    lay = w4.peer.arena_layout(nbytes, world)
    arenas = [torch.zeros(lay["bytes"], dtype=torch.uint8, device="cuda") for _ in range(world)]
    base = [a.data_ptr() for a in arenas]

    def slot(arena, buf, owner):
        return base[arena] + (buf * world + owner) * lay["slot"]

    for step in range(1, 8):
        buf = step % w4.peer.NBUF
        want = []
        for r in range(world):
            pattern = torch.full((nbytes,), (17 * step + 5 * r) % 251, dtype=torch.uint8, device="cuda")
            off = (buf * world + r) * lay["slot"]
            arenas[r][off:off + nbytes] = pattern
            want.append(int(pattern[0]))
        for r in range(world):
            o = 1 - r
            dst = [0, 0]
            flag_dst = [0, 0]
            dst[o] = slot(o, buf, r)
            flag_dst[o] = base[o] + lay["flags"] + 8 * r
            w4.capi.allgather_push(slot(r, buf, r), nbytes, dst, flag_dst, base[r] + lay["flags"],
                                   base[r] + lay["counters"], r, world, wait_now=False)
        for r in range(world):
            w4.capi.allgather_wait(base[r] + lay["flags"], base[r] + lay["counters"], r, world)
        sync_ok()
        for r in range(world):
            o = 1 - r
            off = (buf * world + o) * lay["slot"]
            got = arenas[r][off:off + nbytes]
            assert bool((got == want[o]).all()), (step, r)
            flags = arenas[r][lay["flags"]:lay["flags"] + 8 * world].view(torch.int64)
            assert int(flags[o]) == step


def test_gemm_push_loopback(oracle):
    """The GEMM whose epilogue does the exchange, on one GPU: two arenas stand for two ranks that each own half
    of W's rows; a step launches rank 0's GEMM and then rank 1's on one stream (each only waits for the other's
    PREVIOUS step), then both wait. Afterwards every arena must hold both slices, equal to the plain GEMM's
    output bit for bit, over more steps than there are slice buffers."""
    N, K, gs, M, world = 1024, 1024, 128, 4, 2
    p = oracle.quantize_w4(oracle.normal_f64(N * K, 51) * 0.02, N, K, gs, False)
    wts = W4Weights(p)
    shards = [w4.shard.shard_w4(wts.desc, world, r) for r in range(world)]
    nloc = shards[0].N
    assert all(d.N == nloc for d in shards)
    nbytes = M * nloc * 2
    lay = w4.peer.arena_layout(nbytes, world)
    arenas = [torch.zeros(lay["bytes"], dtype=torch.uint8, device="cuda") for _ in range(world)]
    base = [a.data_ptr() for a in arenas]

    def slot(arena, buf, owner):
        return base[arena] + (buf * world + owner) * lay["slot"]

    for step in range(1, 6):
        buf = step % w4.peer.NBUF
        x = oracle.normal_f16(M * K, 60 + step)
        x_d = dev(x)
        want = []
        for r in range(world):
            c = empty_f16(M * nloc)
            w4.gemm(shards[r], ptr(x_d), ptr(c), M, path=w4.PATH_STREAM)
            want.append(bits(c))
        for r in range(world):
            o = 1 - r
            c_peer, flag_dst = [0, 0], [0, 0]
            c_peer[o] = slot(o, buf, r)
            flag_dst[o] = base[o] + lay["flags"] + 8 * r
            w4.capi.gemm_push(shards[r], ptr(x_d), slot(r, buf, r), M, c_peer, flag_dst, base[r] + lay["flags"],
                              base[r] + lay["counters"], base[r] + lay["done"], r, world)
        for r in range(world):
            w4.capi.allgather_wait(base[r] + lay["flags"], base[r] + lay["counters"], r, world)
        sync_ok()
        for arena in range(world):
            for owner in range(world):
                off = (buf * world + owner) * lay["slot"]
                got = arenas[arena][off:off + nbytes].view(torch.int16).cpu().numpy().view(np.uint16)
                assert np.array_equal(got, want[owner]), (step, arena, owner)
            flags = arenas[arena][lay["flags"]:lay["flags"] + 8 * world].view(torch.int64)
            assert int(flags[1 - arena]) == step

def test_gemm_carry_loopback(oracle):
    """The GEMM that carries the previous step's slice to the peers, on one GPU: two arenas stand for two ranks
    that each own half of W's rows. A step launches rank 0's GEMM and then rank 1's on one stream; each delivers
    its slice of the step before and waits only for flags that earlier launches have posted. The last slice goes
    out with the exchange kernel. Afterwards every arena must hold both ranks' slices of every step, equal to
    the plain GEMM's output bit for bit, over more steps than there are slice buffers."""
    N, K, gs, M, world = 1024, 1024, 128, 4, 2
    p = oracle.quantize_w4(oracle.normal_f64(N * K, 71) * 0.02, N, K, gs, False)
    wts = W4Weights(p)
    shards = [w4.shard.shard_w4(wts.desc, world, r) for r in range(world)]
    nloc = shards[0].N
    nbytes = M * nloc * 2
    lay = w4.peer.arena_layout(nbytes, world)
    arenas = [torch.zeros(lay["bytes"], dtype=torch.uint8, device="cuda") for _ in range(world)]
    base = [a.data_ptr() for a in arenas]

    def slot(arena, buf, owner):
        return base[arena] + (buf * world + owner) * lay["slot"]

    def args(r, buf):
        o = 1 - r
        dst, flag_dst = [0, 0], [0, 0]
        dst[o] = slot(o, buf, r)
        flag_dst[o] = base[o] + lay["flags"] + 8 * r
        return dst, flag_dst

    nsteps = 7
    xs = [dev(oracle.normal_f16(M * K, 80 + i)) for i in range(nsteps)]
    want = []
    for i in range(nsteps):
        per_rank = []
        for r in range(world):
            c = empty_f16(M * nloc)
            w4.gemm(shards[r], ptr(xs[i]), ptr(c), M, path=w4.PATH_STREAM)
            per_rank.append(bits(c).copy())
        want.append(per_rank)
    sync_ok()

    def check(i):  # both slices of step i in both arenas
        buf = i % w4.peer.NBUF
        for r in range(world):
            for owner in range(world):
                off = (buf * world + owner) * lay["slot"]
                got = arenas[r][off:off + nbytes].cpu().numpy().view(np.uint16)
                assert np.array_equal(got, want[i][owner]), (i, r, owner)

    for i in range(nsteps):
        buf = i % w4.peer.NBUF
        prev = (i - 1) % w4.peer.NBUF
        for r in range(world):
            dst, flag_dst = args(r, prev)
            w4.capi.gemm_carry(shards[r], ptr(xs[i]), slot(r, buf, r), M, slot(r, prev, r) if i else None, nbytes if i else 0,
                               dst if i else [0, 0], flag_dst, base[r] + lay["flags"], base[r] + lay["counters"],
                               base[r] + lay["done"], r, world)
        if i:
            for r in range(world):  # step i - 1 is complete everywhere once both carries have run
                w4.capi.allgather_wait(base[r] + lay["flags"], base[r] + lay["counters"], r, world)
            sync_ok()
            check(i - 1)
    last = (nsteps - 1) % w4.peer.NBUF
    for r in range(world):
        dst, flag_dst = args(r, last)
        w4.capi.allgather_push(slot(r, last, r), nbytes, dst, flag_dst, base[r] + lay["flags"], base[r] + lay["counters"],
                               r, world, wait_now=False)
    for r in range(world):
        w4.capi.allgather_wait(base[r] + lay["flags"], base[r] + lay["counters"], r, world)
    sync_ok()
    check(nsteps - 1)
    for r in range(world):
        flags = arenas[r][lay["flags"]:lay["flags"] + 8 * world].view(torch.int64)
        assert int(flags[1 - r]) == nsteps


@pytest.mark.parametrize("world", [2, 3, 8])
def test_sharded_descriptors_match_unsharded(oracle, world):
    """Descriptors built by shard.shard_w4 (contiguous row slices of q / scales / zeros): the hook output of the
    shards, concatenated, is dequant_all bit for bit; the GEMM output of the shards against the oracle and
    against the unsharded call. (The shards' K range is cut between CTAs at other places than the unsharded
    matrix's, so FP32 sums may round differently: equal to within one FP16 ulp, not bit for bit.)"""
    N, K, gs, M = 1536, 1024, 128, 4
    p = oracle.quantize_w4(oracle.normal_f64(N * K, 31) * 0.02, N, K, gs, False)
    wd, wts = oracle.dequant_all_w4(p), W4Weights(p)
    x = oracle.normal_f16(M * K, 32)
    x_d = dev(x)
    full = empty_f16(M * N)
    w4.gemm(wts.desc, ptr(x_d), ptr(full), M)
    sync_ok()
    parts, hooks = [], []
    for r in range(world):
        d = w4.shard.shard_w4(wts.desc, world, r)
        n0, n1 = w4.shard.row_range(N, world, r)
        assert d.N == n1 - n0
        if d.N == 0:
            continue
        c, w_out = empty_f16(M * d.N), empty_f16(d.N * K)
        w4.gemm(d, ptr(x_d), ptr(c), M, None, ptr(w_out))
        sync_ok()
        parts.append(bits(c).reshape(M, d.N))
        hooks.append(bits(w_out))
    assert np.array_equal(np.concatenate(hooks), wd)
    got = np.concatenate(parts, axis=1)
    ref = oracle.gemm_oracle(x, M, K, wd, N, threads=8)
    assert cases.rel_l2(cases.f16(got.ravel()), ref) <= TOL
    a, b = cases.f16(got.ravel()), cases.f16(bits(full))
    ulp = np.maximum(np.abs(b), 2.0 ** -14) * 2.0 ** -10
    assert np.all(np.abs(a - b) <= ulp)


def test_device_status_covers_the_no_alloc_entry(oracle):
    """w4b_device_status() also reads (and clears) the status word of the no-allocation entry's fixed array."""
    N, K, gs, M = 256, 512, 128, 2
    p = oracle.quantize_w4(oracle.normal_f64(N * K, 41) * 0.02, N, K, gs, True)
    wts = W4Weights(p)
    x_d, c = dev(oracle.normal_f16(M * K, 42)), empty_f16(M * N)
    w4.gemm_noalloc(wts.desc, ptr(x_d), ptr(c), M)
    assert w4.device_status() == 0
    assert w4.device_status() == 0
