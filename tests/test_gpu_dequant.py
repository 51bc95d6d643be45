"""GPU parity: stand-alone dequantisation is bit-identical to the oracle's
dequant_all / dequant_all_mx / dequant_head_f8 (the reference's gates
tests/test_gpu.cu:119-134, 305-360 and its FP8 two-pass), including an
exhaustive sweep of the register decoders over every (scale, code, zero)."""
import numpy as np
import pytest

import cases
import w4a16_dequant_gemm_b200 as w4
from gpu_util import MxWeights, W4Weights, bits, dev, empty_f16, ptr, sync_ok

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("sym", [True, False])
@pytest.mark.parametrize("i", range(len(cases.GEMM_CFGS)))
def test_dequant_w4_reference_shapes(oracle, i, sym):
    M, N, K, gs = cases.GEMM_CFGS[i]
    p = oracle.quantize_w4(oracle.normal_f64(N * K, cases.w4_seed(i, sym)), N, K, gs, sym)
    wts = W4Weights(p)
    out = empty_f16(N * K)
    w4.dequant(wts.desc, ptr(out))
    sync_ok()
    assert np.array_equal(bits(out), oracle.dequant_all_w4(p))


@pytest.mark.parametrize("i", range(len(cases.GEMM_CFGS)))
def test_dequant_mx_reference_shapes(oracle, i):
    M, N, K, _ = cases.GEMM_CFGS[i]
    p = oracle.quantize_mx(oracle.normal_f64(N * K, cases.mx_gpu_seed(i)), N, K)
    wts = MxWeights(p)
    out = empty_f16(N * K)
    w4.dequant_mx(wts.desc, ptr(out))
    sync_ok()
    assert np.array_equal(bits(out), oracle.dequant_all_mx(p))


@pytest.mark.parametrize("sym", [True, False])
@pytest.mark.parametrize("gs", [32, 64, 128])
def test_dequant_w4_vector_path(oracle, gs, sym):
    N, K = 257, 512
    p = oracle.quantize_w4(oracle.normal_f64(N * K, 77 + gs) * 0.02, N, K, gs, sym)
    wts = W4Weights(p)
    out = empty_f16(N * K)
    w4.dequant(wts.desc, ptr(out))
    sync_ok()
    assert np.array_equal(bits(out), oracle.dequant_all_w4(p))


def test_w4_decoder_exhaustive(oracle):
    """Every FP16 scale bit pattern that is finite x every zero-point x every code,
    through the vector kernel (the decoder the GEMM kernels share)."""
    scales = np.arange(65536, dtype=np.uint32)
    scales = scales[(scales & 0x7C00) != 0x7C00].astype(np.uint16)  # drop inf / NaN
    ns = scales.size
    N, K, gs = ns * 16, 32, 32                   # row = (scale, zero); 32 codes per row: 0..15 twice
    q = np.tile(np.array([0x76543210, 0xFEDCBA98, 0x76543210, 0xFEDCBA98], np.uint32), N)
    s = np.repeat(scales, 16)
    z = np.tile(np.arange(16, dtype=np.uint32), ns)  # words(G) = 1: nibble 0 of each row's word
    p = dict(N=N, K=K, gs=gs, G=1, symmetric=False, q=q, scales=s, zeros=z)
    wts = W4Weights(p)
    out = empty_f16(N * K)
    w4.dequant(wts.desc, ptr(out))
    sync_ok()
    assert np.array_equal(bits(out), oracle.dequant_all_w4(p))


def test_mx_decoder_exhaustive(oracle):
    """Every E8M0 byte 0..254 x every code, through the vector kernel (fast form for
    89..128, the scalar definition outside)."""
    N, K = 255, 32
    q = np.tile(np.array([0x76543210, 0xFEDCBA98, 0x76543210, 0xFEDCBA98], np.uint32), N)
    p = dict(N=N, K=K, B=1, q=q, scales=np.arange(255, dtype=np.uint8))
    wts = MxWeights(p)
    out = empty_f16(N * K)
    w4.dequant_mx(wts.desc, ptr(out))
    sync_ok()
    assert np.array_equal(bits(out), oracle.dequant_all_mx(p))


@pytest.mark.parametrize("i", range(len(cases.KV_CFGS)))
def test_dequant_f8(oracle, i):
    H, S, D, gs = cases.KV_CFGS[i]
    seed = cases.f8_gpu_seed(i)
    c = oracle.quantize_cache_f8(oracle.normal_f64(H * S * D, seed), oracle.normal_f64(H * S * D, seed + 1),
                                 H, S, D, gs)
    want = oracle.dequant_cache_f8(c, "k").reshape(H, S * D)
    qd, sd = dev(c["q_k"]), dev(c["s_k"])
    G = c["G"]
    for h in range(H):
        out = empty_f16(S * D)
        w4.dequant_f8(qd.data_ptr() + h * S * D, sd.data_ptr() + h * S * G * 2, ptr(out), S, D, gs)
        sync_ok()
        assert np.array_equal(bits(out), want[h])
