"""CPU tests of the drop-in boundary: the library loads, exports every symbol
include/w4b_abi.h declares, and rejects malformed calls on the host before
touching CUDA -- the reference's entry-contract gates (tests/test_gpu.cu:1473-1864)
with the same dummy pointers that must never be dereferenced. No GPU needed."""
import ctypes
import os
import re

import pytest

import w4a16_dequant_gemm_b200 as w4

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
INT32_MAX = 2**31 - 1
ONE = 1  # the reference's (T*)1 dummy pointer


def test_exports_match_header():
    text = open(os.path.join(ROOT, "include", "w4b_abi.h")).read()
    declared = set(re.findall(r"\b(w4b_[a-z0-9_]+)\s*\(", text))
    assert declared == set(w4.capi.ABI), declared ^ set(w4.capi.ABI)
    dll = ctypes.CDLL(w4.build.LIB)
    for name in declared:
        assert hasattr(dll, name), name


def test_no_oracle_in_product():
    # the shipped path must not reach into oracle/
    pkg = os.path.join(ROOT, "w4a16-dequant-gemm_b200")
    for base, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h")):
                assert "oracle" not in open(os.path.join(base, f)).read().lower(), f


def good():
    return w4.DevicePackedW(2, 32, 8, 4, 1, ONE, ONE, None)


def variants():
    g = good()
    out = {}
    out["gs=0"] = w4.DevicePackedW(2, 32, 0, 4, 1, ONE, ONE, None)
    out["gs=7"] = w4.DevicePackedW(2, 32, 7, 4, 1, ONE, ONE, None)
    out["G wrong"] = w4.DevicePackedW(2, 32, 8, 3, 1, ONE, ONE, None)
    out["q null"] = w4.DevicePackedW(2, 32, 8, 4, 1, None, ONE, None)
    out["asym zeros null"] = w4.DevicePackedW(2, 32, 8, 4, 0, ONE, ONE, None)
    out["sym carries zeros"] = w4.DevicePackedW(2, 32, 8, 4, 1, ONE, ONE, ONE)
    out["N=0"] = w4.DevicePackedW(0, 32, 8, 4, 1, ONE, ONE, None)
    return g, out


@pytest.mark.parametrize("entry", ["dequant", "gemm_fused", "gemm_mma", "gemm"])
def test_w4_structural_rejections(entry):
    g, bad = variants()
    for name, p in bad.items():
        with pytest.raises(w4.InvalidArgument):
            if entry == "dequant":
                w4.dequant(p, ONE)
            else:
                getattr(w4, entry)(p, ONE, ONE, 2)
    if entry == "dequant":
        with pytest.raises(w4.InvalidArgument):  # 2^21 rows x words(8192) = 2^31 exactly
            w4.dequant(w4.DevicePackedW(1 << 21, 8192, 8, 1024, 1, ONE, ONE, None), ONE)
        with pytest.raises(w4.InvalidArgument):
            w4.dequant(g, None)
        return
    fn = getattr(w4, entry)
    for args in [(g, ONE, ONE, 0), (g, None, ONE, 2), (g, ONE, None, 2)]:
        with pytest.raises(w4.InvalidArgument):
            fn(*args)


def test_gemm_launch_bounds():
    g = good()
    with pytest.raises(w4.InvalidArgument):  # fused: M > 65535 * 4
        w4.gemm_fused(g, ONE, ONE, 262141)
    with pytest.raises(w4.InvalidArgument):  # mma: M > 65535 * 64
        w4.gemm_mma(g, ONE, ONE, 4194241)
    huge = w4.DevicePackedW(INT32_MAX, 32, 8, 4, 1, ONE, ONE, None)
    with pytest.raises(w4.InvalidArgument):
        w4.gemm_mma(huge, ONE, ONE, 2)
    with pytest.raises(w4.InvalidArgument):
        w4.gemm_fused(huge, ONE, ONE, 2)
    with pytest.raises(w4.InvalidArgument):
        w4.gemm(g, ONE, ONE, 2, path=7)


@pytest.mark.parametrize("entry", ["dequant_mx", "gemm_fused_mx", "gemm_mma_mx", "gemm_mx"])
def test_mx_rejections(entry):
    ok = w4.DevicePackedWm(2, 32, 1, ONE, ONE)
    bad = [w4.DevicePackedWm(0, 32, 1, ONE, ONE), w4.DevicePackedWm(2, 32, 2, ONE, ONE),
           w4.DevicePackedWm(2, 32, 1, None, ONE), w4.DevicePackedWm(2, 32, 1, ONE, None)]
    for p in bad:
        with pytest.raises(w4.InvalidArgument):
            if entry == "dequant_mx":
                w4.dequant_mx(p, ONE)
            else:
                getattr(w4, entry)(p, ONE, ONE, 2)
    if entry == "dequant_mx":
        with pytest.raises(w4.InvalidArgument):
            w4.dequant_mx(ok, None)
        with pytest.raises(w4.InvalidArgument):
            w4.dequant_mx(w4.DevicePackedWm(1 << 21, 8192, 256, ONE, ONE), ONE)
        return
    fn = getattr(w4, entry)
    for args in [(ok, ONE, ONE, 0), (ok, None, ONE, 2), (ok, ONE, None, 2)]:
        with pytest.raises(w4.InvalidArgument):
            fn(*args)
    with pytest.raises(w4.InvalidArgument):
        w4.gemm_fused_mx(ok, ONE, ONE, 262141)
    with pytest.raises(w4.InvalidArgument):
        w4.gemm_mma_mx(w4.DevicePackedWm(INT32_MAX, 32, 1, ONE, ONE), ONE, ONE, 2)


def kv(H=2, S=4, D=64, gs=32, G=2, sym=1, qk=ONE, sk=ONE, zk=None, qv=ONE, sv=ONE, zv=None):
    return w4.DeviceKVW4(H, S, D, gs, G, sym, qk, sk, zk, qv, sv, zv)


@pytest.mark.parametrize("entry", ["attention_w4", "attention_w4_flash", "paged"])
def test_kv_w4_rejections(entry):
    def call(p, q=ONE, out=ONE, bt=ONE, page=4, npages=1):
        if entry == "paged":
            w4.attention_w4_flash_paged(p, bt, page, npages, q, out)
        else:
            getattr(w4, entry)(p, q, out)

    bad = [kv(H=0), kv(S=0), kv(D=0), kv(D=513, G=17), kv(gs=7), kv(gs=0), kv(G=3), kv(qk=None), kv(sv=None),
           kv(sym=0), kv(zk=ONE, zv=ONE), kv(zk=ONE)]
    for p in bad:
        with pytest.raises(w4.InvalidArgument):
            call(p)
    for a in [dict(q=None), dict(out=None)]:
        with pytest.raises(w4.InvalidArgument):
            call(kv(), **a)
    if entry == "attention_w4":
        with pytest.raises(w4.InvalidArgument):  # single-block bound S <= 4096
            call(kv(S=4097))
    else:
        with pytest.raises(w4.InvalidArgument):  # S > 65535 * 256
            call(kv(S=65535 * 256 + 1), page=65536, npages=256)
    if entry == "paged":
        for a in [dict(bt=None), dict(page=0), dict(npages=0), dict(page=1, npages=3),
                  dict(page=50000, npages=50000)]:
            with pytest.raises(w4.InvalidArgument):
                call(kv(), **a)


@pytest.mark.parametrize("entry", ["attention_fp16", "attention_fp16_flash"])
def test_kv_fp16_rejections(entry):
    fn = getattr(w4, entry)
    for args in [(ONE, ONE, ONE, ONE, 0, 4, 64), (ONE, ONE, ONE, ONE, 2, 0, 64), (ONE, ONE, ONE, ONE, 2, 4, 0),
                 (ONE, ONE, ONE, ONE, 2, 4, 513), (None, ONE, ONE, ONE, 2, 4, 64), (ONE, None, ONE, ONE, 2, 4, 64),
                 (ONE, ONE, None, ONE, 2, 4, 64), (ONE, ONE, ONE, None, 2, 4, 64)]:
        with pytest.raises(w4.InvalidArgument):
            fn(*args)
    with pytest.raises(w4.InvalidArgument):
        if entry == "attention_fp16":
            fn(ONE, ONE, ONE, ONE, 2, 4097, 64)
        else:
            fn(ONE, ONE, ONE, ONE, 2, 65535 * 256 + 1, 64)


def test_f8_rejections():
    def f8(H=2, S=4, D=64, gs=32, G=2, qk=4, sk=ONE, qv=4, sv=ONE):
        return w4.DeviceKVF8(H, S, D, gs, G, qk, sk, qv, sv)

    bad = [f8(H=0), f8(D=513, G=17), f8(gs=7), f8(G=3), f8(qk=None), f8(sv=None), f8(S=65535 * 256 + 1),
           f8(D=66, G=3), f8(qk=1), f8(qv=3)]  # misaligned bases (uint8_t*)1 / 3
    for p in bad:
        with pytest.raises(w4.InvalidArgument):
            w4.attention_f8_flash(p, ONE, ONE)
    with pytest.raises(w4.InvalidArgument):
        w4.attention_f8_flash(f8(), None, ONE)
    for args in [(4, ONE, ONE, 0, 64, 32), (4, ONE, ONE, 4, 64, 7), (None, ONE, ONE, 4, 64, 32),
                 (4, ONE, ONE, 4, 66, 8), (1, ONE, ONE, 4, 64, 32), (4, ONE, ONE, 1 << 24, 512, 32)]:
        with pytest.raises(w4.InvalidArgument):
            w4.dequant_f8(*args)


def test_batched_paged_contract():
    """The batched paged entry rejects malformed calls before touching any pointer (dummy pointers)."""
    kv = w4.DeviceKVW4(2, 64, 128, 32, 4, 1, ONE * 16, ONE * 16, None, ONE * 16, ONE * 16, None)

    def call(desc=kv, bt=ONE * 16, stride=8, lens=ONE * 16, nseq=2, smax=100, page=16, npages=16, q=ONE * 16,
             out=ONE * 16):
        w4.attention_w4_flash_paged_batched(desc, bt, stride, lens, nseq, smax, page, npages, q, out)

    bad = w4.InvalidArgument
    for kw in (dict(bt=None), dict(lens=None), dict(nseq=0), dict(smax=0), dict(page=0), dict(npages=0),
               dict(npages=6),      # 6 pages of 16 rows cannot hold 100 positions
               dict(stride=6),      # the longest sequence needs 7 table entries
               dict(q=None), dict(out=None),
               dict(desc=w4.DeviceKVW4(2, 64, 96, 32, 3, 1, ONE * 16, ONE * 16, None, ONE * 16, ONE * 16, None)),  # D = 96
               dict(desc=w4.DeviceKVW4(2, 64, 128, 32, 4, 0, ONE * 16, ONE * 16, None, ONE * 16, ONE * 16, None))):  # asym, no zeros
        with pytest.raises(bad):
            call(**kw)


def test_relayout_contract():
    """The re-layout and the padded-K entries reject malformed calls on the host (dummy pointers)."""
    assert w4.relayout_k(4100) == 4608 and w4.relayout_k(512) == 512 and w4.relayout_k(1) == 512
    for k in (0, -5, INT32_MAX):
        with pytest.raises(w4.InvalidArgument):
            w4.relayout_k(k)
    TWO = 2  # a second dummy address: the entries compare source and destination pointers
    src = w4.DevicePackedW(2, 36, 8, 5, 0, ONE, ONE, ONE)

    def dst(N=2, K=512, gs=8, G=64, sym=0, q=TWO, s=TWO, z=TWO):
        return w4.DevicePackedW(N, K, gs, G, sym, q, s, z)

    bad = w4.InvalidArgument
    for d in (dst(N=3), dst(K=32, G=4), dst(gs=16, G=32), dst(sym=1, z=None), dst(G=63), dst(q=ONE), dst(s=ONE),
              dst(z=ONE), dst(q=None)):
        with pytest.raises(bad):
            w4.relayout(src, d)
    for name, p in variants()[1].items():          # a malformed source
        with pytest.raises(bad):
            w4.relayout(p, dst())
    msrc = w4.DevicePackedWm(2, 40, 2, ONE, ONE)
    for d in (w4.DevicePackedWm(3, 512, 16, TWO, TWO), w4.DevicePackedWm(2, 32, 1, TWO, TWO),
              w4.DevicePackedWm(2, 512, 15, TWO, TWO), w4.DevicePackedWm(2, 512, 16, ONE, TWO),
              w4.DevicePackedWm(2, 512, 16, TWO, None)):
        with pytest.raises(bad):
            w4.relayout_mx(msrc, d)
    g = good()
    for args in [(g, ONE, 0, ONE, 2), (g, ONE, 33, ONE, 2), (g, None, 32, ONE, 2), (g, ONE, 32, None, 2),
                 (g, ONE, 32, ONE, 0)]:
        with pytest.raises(bad):
            w4.gemm_padded(*args)
    with pytest.raises(bad):
        w4.gemm_padded(g, ONE, 32, ONE, 2, path=9)
    gm = w4.DevicePackedWm(2, 64, 2, ONE, ONE)
    for args in [(gm, ONE, 0, ONE, 2), (gm, ONE, 65, ONE, 2), (gm, None, 64, ONE, 2), (gm, ONE, 64, ONE, 0)]:
        with pytest.raises(bad):
            w4.gemm_mx_padded(*args)
