"""GPU parity of the fused dequant GEMM through the C ABI: the reference's device
gates (tests/test_gpu.cu:68-297 for W4, :305-498 for MXFP4) on its own shapes
and seeds, the stream kernel's shape family, and the BASELINE shapes at full size.

Gates, as in the reference: the w_out hook reproduces dequant_all bit for bit;
the output is within rel L2 <= 1e-3 of the FP64 oracle; the dispatcher's output
is byte-identical to the entry it selects (so kernels are run-to-run
deterministic)."""
import os

import numpy as np
import pytest

import cases
import w4a16_dequant_gemm_b200 as w4
from gpu_util import MxWeights, W4Weights, bits, dev, empty_f16, ptr, sync_ok

pytestmark = pytest.mark.gpu
TOL = 1e-3  # rel L2 against the FP64 oracle (tests/test_gpu.cu:152-158)
GOLD = np.load(os.path.join(os.path.dirname(__file__), "golden", "golden.npz"))


def run_entry(fn, desc, x_d, M, N, K, hook):
    c = empty_f16(M * N)
    c.fill_(float("nan"))
    w_out = empty_f16(N * K) if hook else None
    fn(desc, ptr(x_d), ptr(c), M, None, ptr(w_out))
    sync_ok()
    return bits(c), (bits(w_out) if hook else None)


@pytest.mark.parametrize("sym", [True, False])
@pytest.mark.parametrize("i", range(len(cases.GEMM_CFGS)))
def test_w4_reference_matrix(oracle, i, sym):
    M, N, K, gs = cases.GEMM_CFGS[i]
    seed = cases.w4_seed(i, sym)
    p = oracle.quantize_w4(oracle.normal_f64(N * K, seed), N, K, gs, sym)
    wd = oracle.dequant_all_w4(p)
    x = oracle.normal_f16(M * K, seed + 1)
    c_ref = GOLD[f"w4/{'sym' if sym else 'asym'}/{i}/c"]           # the reference's own FP64 result
    assert np.array_equal(c_ref, oracle.gemm_oracle(x, M, K, wd, N))
    wts, x_d = W4Weights(p), dev(x)
    outs = {}
    for name in ("gemm_fused", "gemm_mma", "gemm"):
        c, w_hook = run_entry(getattr(w4, name), wts.desc, x_d, M, N, K, True)
        assert np.array_equal(w_hook, wd), f"{name}: w_out is not bitwise dequant_all"
        c2, _ = run_entry(getattr(w4, name), wts.desc, x_d, M, N, K, False)
        assert np.array_equal(c, c2), f"{name}: hook and plain launches differ"
        assert cases.rel_l2(cases.f16(c), c_ref) <= TOL, name
        outs[name] = c
    winner = "gemm_fused" if M < w4.DISPATCH_MMA_MIN_M() else "gemm_mma"
    assert np.array_equal(outs["gemm"], outs[winner])  # routing gate, tests/test_gpu.cu:255-286


@pytest.mark.parametrize("i", range(len(cases.GEMM_CFGS)))
def test_mx_reference_matrix(oracle, i):
    M, N, K, _ = cases.GEMM_CFGS[i]
    seed = cases.mx_gpu_seed(i)
    p = oracle.quantize_mx(oracle.normal_f64(N * K, seed), N, K)
    wd = oracle.dequant_all_mx(p)
    x = oracle.normal_f16(M * K, seed + 1)
    c_ref = GOLD[f"mx/{i}/c"]
    wts, x_d = MxWeights(p), dev(x)
    outs = {}
    for name in ("gemm_fused_mx", "gemm_mma_mx", "gemm_mx"):
        c, w_hook = run_entry(getattr(w4, name), wts.desc, x_d, M, N, K, True)
        assert np.array_equal(w_hook, wd), name
        assert cases.rel_l2(cases.f16(c), c_ref) <= TOL, name
        outs[name] = c
    winner = "gemm_fused_mx" if M < w4.DISPATCH_MMA_MIN_M() else "gemm_mma_mx"
    assert np.array_equal(outs["gemm_mx"], outs[winner])


@pytest.mark.parametrize("M", [1, 8, 16, 33])
def test_mx_block_exponents_outside_the_half_range(oracle, M):
    """Blocks whose power of two is no FP16 value (tiny and huge rows beside ordinary ones): the kernels choose
    between the bit-placement decode and the scalar definition - per word, or per chunk by a warp vote in the
    stream kernel - and both must give dequant_one_mx's bits (mx.hpp:52-59) and the oracle's products."""
    N, K = 192, 1024
    w = (oracle.normal_f64(N * K, 0xE8 + M) * 0.02).reshape(N, K)
    rows = np.arange(N)
    w[rows % 5 == 1] *= 2.0 ** -45        # shared exponents far below the half range
    w[rows % 5 == 3] *= 2.0 ** 9          # ... and above the range of the fast form
    w[7, 512:544] *= 2.0 ** -60           # one odd block inside an ordinary row
    p = oracle.quantize_mx(w.ravel(), N, K)
    se = p["scales"]
    assert (se < 89).any() and (se > 128).any() and ((se >= 89) & (se <= 128)).any()
    wd = oracle.dequant_all_mx(p)
    x = oracle.normal_f16(M * K, 0xE9 + M)
    ref = oracle.gemm_oracle(x, M, K, wd, N)
    wts, x_d = MxWeights(p), dev(x)
    for name in ("gemm_fused_mx", "gemm_mma_mx"):
        c, w_hook = run_entry(getattr(w4, name), wts.desc, x_d, M, N, K, True)
        assert np.array_equal(w_hook, wd), name
        assert cases.rel_l2(cases.f16(c), ref) <= TOL, name
        c2, _ = run_entry(getattr(w4, name), wts.desc, x_d, M, N, K, False)
        assert np.array_equal(c2, c), name


# The stream kernel's family: K % 512 == 0, N >= 64 (ragged N tails, several panels, split panels),
# every supported group size, M across the m-tile and multi-pass boundaries.
STREAM_SHAPES = [(64, 512), (128, 512), (200, 512), (333, 1024), (1024, 2048), (2500, 512), (4096, 4096)]


@pytest.mark.parametrize("fmt", ["sym", "asym", "mx"])
@pytest.mark.parametrize("N,K", STREAM_SHAPES)
def test_stream_kernel_family(oracle, N, K, fmt):
    rng_seed = 1000 + N + K
    w = oracle.normal_f64(N * K, rng_seed) * 0.02
    for gs in ([32] if fmt == "mx" else [32, 64, 128]):
        if fmt == "mx":
            p = oracle.quantize_mx(w, N, K)
            wd, wts, fn = oracle.dequant_all_mx(p), MxWeights(p), w4.gemm_mx
        else:
            p = oracle.quantize_w4(w, N, K, gs, fmt == "sym")
            wd, wts, fn = oracle.dequant_all_w4(p), W4Weights(p), w4.gemm
        for M in ([1, 3, 8, 9, 16, 17, 35] if N <= 1024 else [1, 16]):
            x = oracle.normal_f16(M * K, rng_seed + M)
            x_d = dev(x)
            assert w4.gemm_route(wts.desc, M, w4.PATH_STREAM, ptr(x_d)) == w4.PATH_STREAM
            hook = M in (1, 17)
            c, w_hook = run_entry(lambda d, *a: fn(d, *a, path=w4.PATH_STREAM), wts.desc, x_d, M, N, K, hook)
            if hook:
                assert np.array_equal(w_hook, wd), (fmt, gs, M)
            ref = oracle.gemm_oracle(x, M, K, wd, N, threads=8)
            assert cases.rel_l2(cases.f16(c), ref) <= TOL, (fmt, gs, M)
            c2, _ = run_entry(lambda d, *a: fn(d, *a, path=w4.PATH_STREAM), wts.desc, x_d, M, N, K, False)
            assert np.array_equal(c, c2), "stream kernel is not run-to-run deterministic"
            cg, _ = run_entry(lambda d, *a: fn(d, *a, path=w4.PATH_GENERIC), wts.desc, x_d, M, N, K, False)
            assert cases.rel_l2(cases.f16(cg), ref) <= TOL


def test_linearity_at_full_size(oracle):
    """Size-independent property at the BASELINE shape (14336 x 4096, asym gs=128):
    gemm(x1 + x2) == gemm(x1) + gemm(x2) to FP16 rounding, and the hook is bitwise."""
    N, K, gs = 14336, 4096, 128
    p = oracle.quantize_w4(oracle.normal_f64(N * K, 0) * 0.02, N, K, gs, False)
    wts = W4Weights(p)
    rng = np.random.default_rng(5)
    x1 = rng.standard_normal(K).astype(np.float16)
    x2 = (rng.standard_normal(K) * 0.5).astype(np.float16)
    xs = (x1.astype(np.float32) + x2.astype(np.float32)).astype(np.float16)
    outs = []
    for x in (x1, x2, xs):
        x_d = dev(x.view(np.uint16))
        c, _ = run_entry(w4.gemm, wts.desc, x_d, 1, N, K, False)
        outs.append(cases.f16(c))
    # x1 + x2 was rounded to FP16 once more than the two separate products
    assert cases.rel_l2(outs[2], outs[0] + outs[1]) <= 2e-3
    w_out = empty_f16(N * K)
    c = empty_f16(N)
    x_d = dev(x1.view(np.uint16))
    w4.gemm(wts.desc, ptr(x_d), ptr(c), 1, None, ptr(w_out))
    sync_ok()
    assert np.array_equal(bits(w_out), oracle.dequant_all_w4(p))


@pytest.mark.parametrize("N,K", [(14336, 4096), (4096, 14336)])
@pytest.mark.parametrize("M", [1, 4, 8, 9, 16, 64])
def test_baseline_c2_against_oracle(oracle, N, K, M):
    """BASELINE config 2 (W4 asymmetric gs=128, x ~ N(0,1), W ~ N(0, 0.02)) at full size."""
    key = (N, K)
    if key not in _C2:
        p = oracle.quantize_w4(oracle.normal_f64(N * K, 0) * 0.02, N, K, 128, False)
        _C2.clear()
        _C2[key] = (p, oracle.dequant_all_w4(p), W4Weights(p))
    p, wd, wts = _C2[key]
    x = oracle.normal_f16(M * K, 1 + M)
    x_d = dev(x)
    c, _ = run_entry(w4.gemm, wts.desc, x_d, M, N, K, False)
    ref = oracle.gemm_oracle(x, M, K, wd, N, threads=os.cpu_count() or 8)
    assert cases.rel_l2(cases.f16(c), ref) <= TOL


_C2 = {}


def test_baseline_c2_ragged_k(oracle):
    """Config 2's ragged K = 4100 (words = 513, G = 33): served by the generic kernel."""
    N, K, gs, M = 2048, 4100, 128, 4
    p = oracle.quantize_w4(oracle.normal_f64(N * K, 3) * 0.02, N, K, gs, False)
    wd, wts = oracle.dequant_all_w4(p), W4Weights(p)
    x = oracle.normal_f16(M * K, 4)
    x_d = dev(x)
    c, w_hook = run_entry(w4.gemm, wts.desc, x_d, M, N, K, True)
    assert np.array_equal(w_hook, wd)
    assert cases.rel_l2(cases.f16(c), oracle.gemm_oracle(x, M, K, wd, N, threads=8)) <= TOL


@pytest.mark.parametrize("K", [72, 100, 104, 40])
def test_baseline_c3_partial_blocks(oracle, K):
    """Config 3's partial-block K for MXFP4."""
    N, M = 512, 8
    p = oracle.quantize_mx(oracle.normal_f64(N * K, K) * 0.02, N, K)
    wd, wts = oracle.dequant_all_mx(p), MxWeights(p)
    x = oracle.normal_f16(M * K, K + 1)
    x_d = dev(x)
    c, w_hook = run_entry(w4.gemm_mx, wts.desc, x_d, M, N, K, True)
    assert np.array_equal(w_hook, wd)
    assert cases.rel_l2(cases.f16(c), oracle.gemm_oracle(x, M, K, wd, N)) <= TOL


@pytest.mark.parametrize("M", [1, 8, 32])
def test_baseline_c3_mx_8192(oracle, M):
    N = K = 8192
    if "p" not in _C3:
        p = oracle.quantize_mx(oracle.normal_f64(N * K, 0) * 0.02, N, K)
        _C3.update(p=p, wd=oracle.dequant_all_mx(p), wts=MxWeights(p))
    x = oracle.normal_f16(M * K, 1 + M)
    x_d = dev(x)
    c, _ = run_entry(w4.gemm_mx, _C3["wts"].desc, x_d, M, N, K, False)
    ref = oracle.gemm_oracle(x, M, K, _C3["wd"], N, threads=os.cpu_count() or 8)
    assert cases.rel_l2(cases.f16(c), ref) <= TOL


_C3 = {}


def test_hostio_entry(oracle):
    """The host-buffer entry returns the same bytes as the device-pointer entry."""
    import torch
    N, K, M = 1024, 1024, 4
    p = oracle.quantize_w4(oracle.normal_f64(N * K, 9) * 0.02, N, K, 128, True)
    wts = W4Weights(p)
    x = oracle.normal_f16(M * K, 10)
    x_d = dev(x)
    c_dev, _ = run_entry(w4.gemm, wts.desc, x_d, M, N, K, False)
    xh = torch.from_numpy(x.view(np.int16).copy()).pin_memory()
    ch = torch.empty(M * N, dtype=torch.int16).pin_memory()
    w4.gemm_hostio(wts.desc, xh.data_ptr(), ch.data_ptr(), M)  # page-locked: the kernel writes c_host itself
    assert np.array_equal(ch.numpy().view(np.uint16), c_dev)
    # new values at the same page-locked address must be seen by the next call
    x2 = oracle.normal_f16(M * K, 11)
    c2_dev, _ = run_entry(w4.gemm, wts.desc, dev(x2), M, N, K, False)
    xh.copy_(torch.from_numpy(x2.view(np.int16).copy()))
    w4.gemm_hostio(wts.desc, xh.data_ptr(), ch.data_ptr(), M)
    assert np.array_equal(ch.numpy().view(np.uint16), c2_dev)
    # the same with launch overlap on: the GEMM may start early and waits for the copy before it reads x
    prev = w4.set_launch_overlap(True)
    try:
        for xs, want in ((x, c_dev), (x2, c2_dev), (x, c_dev)):
            xh.copy_(torch.from_numpy(xs.view(np.int16).copy()))
            w4.gemm_hostio(wts.desc, xh.data_ptr(), ch.data_ptr(), M)
            assert np.array_equal(ch.numpy().view(np.uint16), want)
    finally:
        w4.set_launch_overlap(prev)
    # a larger M (tensor kernel)
    Mb = 40
    xb = oracle.normal_f16(Mb * K, 12)
    cb_dev, _ = run_entry(w4.gemm, wts.desc, dev(xb), Mb, N, K, False)
    xbh = torch.from_numpy(xb.view(np.int16).copy()).pin_memory()
    cbh = torch.empty(Mb * N, dtype=torch.int16).pin_memory()
    w4.gemm_hostio(wts.desc, xbh.data_ptr(), cbh.data_ptr(), Mb)
    assert np.array_equal(cbh.numpy().view(np.uint16), cb_dev)
    xp, cp = x.copy(), np.zeros(M * N, np.uint16)  # pageable: staged through device memory
    w4.gemm_hostio(wts.desc, xp.ctypes.data, cp.ctypes.data, M)
    assert np.array_equal(cp, c_dev)
