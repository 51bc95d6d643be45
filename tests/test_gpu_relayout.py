"""GPU parity of the offline re-layout (w4b_relayout_w4 / _mx) and the padded-K GEMM entries.

The reference has no such converter (its kernels take any K: include/w4/fused.cuh:175-193), so the checks are
against its definitions: the converted matrix dequantises (dequant, include/w4/dequant.cuh:62-82) to the bits of
the source followed by +0 columns, and the GEMM over it equals gemm_oracle (include/w4/pack.hpp:166-184) on the
ORIGINAL matrix within the project's bar, rel L2 <= 1e-3."""
import numpy as np
import pytest
import torch

import cases
import w4a16_dequant_gemm_b200 as w4
from gpu_util import MxWeights, W4Weights, bits, dev, empty_f16, ptr, sync_ok

pytestmark = pytest.mark.gpu
TOL = 1e-3


def words(n):
    return (n + 7) // 8


def junk(n, dtype):
    return torch.full((int(n),), -1, dtype=dtype, device="cuda")


class PaddedW4:
    """Destination buffers full of stale bits plus the descriptor of the extended matrix."""

    def __init__(self, src, Kp):
        N, gs = src.N, src.gs
        Gp = (Kp + gs - 1) // gs
        self.q, self.s = junk(N * words(Kp), torch.int32), junk(N * Gp, torch.int16)
        self.z = None if src.symmetric else junk(N * words(Gp), torch.int32)
        self.desc = w4.DevicePackedW(N, Kp, gs, Gp, src.symmetric, ptr(self.q), ptr(self.s), ptr(self.z))


class PaddedMx:
    def __init__(self, src, Kp):
        Bp = (Kp + 31) // 32
        self.q, self.s = junk(src.N * words(Kp), torch.int32), junk(src.N * Bp, torch.uint8)
        self.desc = w4.DevicePackedWm(src.N, Kp, Bp, ptr(self.q), ptr(self.s))


W4_SHAPES = [(96, 4100, 128), (64, 1000, 32), (130, 520, 64), (64, 100, 8), (70, 4096, 128), (65, 36, 24)]


def test_relayout_k():
    assert [w4.relayout_k(k) for k in (1, 511, 512, 513, 4100)] == [512, 512, 512, 1024, 4608]
    with pytest.raises(w4.InvalidArgument):
        w4.relayout_k(0)


@pytest.mark.parametrize("sym", [True, False])
@pytest.mark.parametrize("N,K,gs", W4_SHAPES)
def test_relayout_w4_is_the_same_matrix_zero_extended(oracle, N, K, gs, sym):
    w = oracle.normal_f64(N * K, 0x4E1A + N + K + gs)
    p = oracle.quantize_w4(w, N, K, gs, sym)
    src = W4Weights(p)
    Kp = w4.relayout_k(K)
    dst = PaddedW4(src.desc, Kp)
    w4.relayout(src.desc, dst.desc)
    out = empty_f16(N * Kp)
    w4.dequant(dst.desc, ptr(out))
    sync_ok()
    got = bits(out).reshape(N, Kp)
    ref = oracle.dequant_all_w4(p).reshape(N, K)
    assert np.array_equal(got[:, :K], ref)
    assert not got[:, K:].any()            # +0, bit pattern 0x0000
    # the original scales and zero points are carried over unchanged
    s = dst.s.cpu().numpy().view(np.uint16).reshape(N, -1)
    assert np.array_equal(s[:, :p["G"]], p["scales"].reshape(N, -1)) and not s[:, p["G"]:].any()


@pytest.mark.parametrize("M", [1, 8, 16, 40])
@pytest.mark.parametrize("sym", [True, False])
@pytest.mark.parametrize("N,K,gs", [(96, 4100, 128), (64, 1000, 32), (130, 520, 64)])
def test_gemm_padded_w4(oracle, N, K, gs, sym, M):
    w = oracle.normal_f64(N * K, 0x6E44 + N + K)
    p = oracle.quantize_w4(w, N, K, gs, sym)
    x16 = oracle.normal_f16(M * K, 0x77 + M)
    ref = oracle.gemm_oracle(x16, M, K, oracle.dequant_all_w4(p), N)
    src = W4Weights(p)
    dst = PaddedW4(src.desc, w4.relayout_k(K))
    w4.relayout(src.desc, dst.desc)
    x, c = dev(x16), empty_f16(M * N)
    # the padded shape is one of the fast kernels', the source's is not
    xp = empty_f16(M * dst.desc.K)
    assert w4.gemm_route(dst.desc, M, w4.PATH_AUTO, ptr(xp)) in (w4.PATH_STREAM, w4.PATH_TENSOR)
    w4.gemm_padded(dst.desc, ptr(x), K, ptr(c), M)
    sync_ok()
    got = cases.f16(bits(c))
    assert cases.rel_l2(got, ref) <= TOL
    # a caller that pads its own activation rows gets the same bits from the plain entry
    xp.zero_()
    xp.view(M, -1)[:, :K] = x.view(torch.float16).view(M, K)
    c2 = empty_f16(M * N)
    w4.gemm(dst.desc, ptr(xp), ptr(c2), M)
    sync_ok()
    assert np.array_equal(bits(c2), bits(c))


@pytest.mark.parametrize("N,K", [(64, 1000), (96, 4100), (70, 72)])
def test_relayout_mx(oracle, N, K):
    w = oracle.normal_f64(N * K, 0x3A + N + K)
    p = oracle.quantize_mx(w, N, K)
    src = MxWeights(p)
    Kp = w4.relayout_k(K)
    dst = PaddedMx(src.desc, Kp)
    w4.relayout_mx(src.desc, dst.desc)
    out = empty_f16(N * Kp)
    w4.dequant_mx(dst.desc, ptr(out))
    sync_ok()
    got = bits(out).reshape(N, Kp)
    assert np.array_equal(got[:, :K], oracle.dequant_all_mx(p).reshape(N, K))
    assert not got[:, K:].any()
    for M in (1, 16, 33):
        x16 = oracle.normal_f16(M * K, 0x99 + M)
        ref = oracle.gemm_oracle(x16, M, K, oracle.dequant_all_mx(p), N)
        x, c = dev(x16), empty_f16(M * N)
        w4.gemm_mx_padded(dst.desc, ptr(x), K, ptr(c), M)
        sync_ok()
        assert cases.rel_l2(cases.f16(bits(c)), ref) <= TOL


def test_relayout_rejections(oracle):
    N, K, gs = 64, 520, 64
    p = oracle.quantize_w4(oracle.normal_f64(N * K, 5), N, K, gs, False)
    src = W4Weights(p)
    good = PaddedW4(src.desc, 1024)
    with pytest.raises(w4.InvalidArgument):           # shorter than the source
        w4.relayout(src.desc, PaddedW4(src.desc, 512).desc)
    other = PaddedW4(src.desc, 1024)
    other.desc.gs, other.desc.G = 128, 8              # another group size
    with pytest.raises(w4.InvalidArgument):
        w4.relayout(src.desc, other.desc)
    with pytest.raises(w4.InvalidArgument):           # in place
        w4.relayout(src.desc, src.desc)
    x, c = empty_f16(2 * 1024), empty_f16(2 * N)
    w4.relayout(src.desc, good.desc)
    with pytest.raises(w4.InvalidArgument):           # more activation columns than the matrix has
        w4.gemm_padded(good.desc, ptr(x), 1025, ptr(c), 2)
    with pytest.raises(w4.InvalidArgument):
        w4.gemm_padded(good.desc, ptr(x), 0, ptr(c), 2)
    sync_ok()
