"""GPU test of w4b_gemm_w4_noalloc, the entry for callers that may not allocate
(a process whose memory pool has claimed the whole device, so that cudaMalloc
would fail, or a serving loop that forbids allocations after warm-up): its
output must equal the regular entry's, on two calls in a row (the second call reuses the fixed scratch array
the first one left behind). Collected last on purpose: a failure here stops a
`-x` run only after every other test has run."""
import numpy as np
import pytest

import w4a16_dequant_gemm_b200 as w4
from gpu_util import W4Weights, bits, dev, empty_f16, ptr, sync_ok

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("N,K,gs,sym,M", [(1000, 1024, 128, False, 1), (4096, 4096, 128, True, 8),
                                          (14336, 4096, 128, False, 16), (333, 512, 32, False, 5)])
def test_noalloc_matches_regular_entry(oracle, N, K, gs, sym, M):
    p = oracle.quantize_w4(oracle.normal_f64(N * K, 21 + N) * 0.02, N, K, gs, sym)
    wts = W4Weights(p)
    x_d = dev(oracle.normal_f16(M * K, 22 + N))
    want = empty_f16(M * N)
    w4.gemm(wts.desc, ptr(x_d), ptr(want), M, None, None, w4.PATH_STREAM)
    sync_ok()
    for call in range(2):
        got = empty_f16(M * N)
        got.fill_(float("nan"))
        w4.gemm_noalloc(wts.desc, ptr(x_d), ptr(got), M)
        sync_ok()
        assert np.array_equal(bits(got), bits(want)), f"call {call}"
    ref = oracle.gemm_oracle(oracle.normal_f16(M * K, 22 + N), M, K, oracle.dequant_all_w4(p), N, threads=8)
    assert np.sqrt(((bits(want).view(np.float16).astype(np.float64) - ref) ** 2).sum() / (ref ** 2).sum()) <= 1e-3


def test_noalloc_rejects_large_k_that_outgrows_the_array(oracle):
    """N = 1,100,000 rows need more per-tile counters than the fixed array holds. Rejected on the host,
    before any pointer is touched (dummy pointers)."""
    N, K, gs = 1_100_000, 8192, 128
    desc = w4.DevicePackedW(N, K, gs, K // gs, 1, 256, 256, None)
    with pytest.raises(w4.InvalidArgument):
        w4.gemm_noalloc(desc, 256, 256, 16)


def test_noalloc_rejects_what_it_cannot_serve(oracle):
    p = oracle.quantize_w4(oracle.normal_f64(128 * 100, 5), 128, 100, 8, True)  # ragged K: not a stream shape
    wts = W4Weights(p)
    x_d, c_d = dev(oracle.normal_f16(100, 6)), empty_f16(128)
    with pytest.raises(w4.InvalidArgument):
        w4.gemm_noalloc(wts.desc, ptr(x_d), ptr(c_d), 1)
    big = oracle.quantize_w4(oracle.normal_f64(256 * 512, 7), 256, 512, 128, True)
    wb = W4Weights(big)
    xb, cb = dev(oracle.normal_f16(16384 * 512, 8)), empty_f16(16384 * 256)
    with pytest.raises(w4.InvalidArgument):  # 1024 passes of 16 rows: the fragments outgrow the fixed array
        w4.gemm_noalloc(wb.desc, ptr(xb), ptr(cb), 16384)
