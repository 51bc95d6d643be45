"""Shapes and seeds of the reference's own gates, as (seed, shape) pairs.

The reference stores no vectors: every test input is regenerated from
std::mt19937_64 + std::normal_distribution seeds (include/w4/pack.hpp:186-200).
The oracle restates that generator, so these lists reproduce the reference's
inputs exactly. Citations are to the reference's tests/test_oracle.cpp and
tests/test_gpu.cu.
"""
import hashlib

import numpy as np

# tests/test_oracle.cpp:23-27 (host) and tests/test_gpu.cu:54-62 (device adds the last four)
GEMM_CFGS = [
    (1, 64, 64, 8), (8, 128, 96, 16), (16, 256, 100, 32), (4, 96, 72, 48), (2, 32, 128, 64),
    (3, 40, 256, 128), (5, 72, 40, 8),
    (17, 64, 128, 16), (33, 48, 104, 24), (20, 32, 100, 8), (65, 96, 100, 16),
]
HOST_GEMM_CFGS = GEMM_CFGS[:7]


def w4_seed(i, sym):  # tests/test_oracle.cpp:33, tests/test_gpu.cu:71
    return 0x44A1 ^ (i * 977 + (0 if sym else 1))


# tests/test_oracle.cpp:156-160: (M, N, K); K=100/72/33/40 are the partial-block cases
MX_HOST_CFGS = [(1, 64, 64), (8, 128, 96), (16, 256, 100), (4, 96, 72), (2, 32, 33), (3, 40, 256), (5, 72, 40)]


def mx_host_seed(i):  # tests/test_oracle.cpp:163
    return 0x9E4F ^ (i * 977)


def mx_gpu_seed(i):  # tests/test_gpu.cu (MX section): 0x1E4A ^ (i*977), shapes = GEMM_CFGS with gs ignored
    return 0x1E4A ^ (i * 977)


# tests/test_gpu.cu:506-781: (H, S, D, gs)
KV_CFGS = [(1, 1, 64, 32), (2, 7, 64, 8), (4, 128, 128, 128), (2, 300, 96, 32), (3, 65, 40, 8), (1, 4096, 64, 64)]
KV_LONG_CFGS = [(2, 5000, 64, 32), (1, 9000, 128, 64)]  # tests/test_gpu.cu:786-924


def kv_seed(i, sym):
    return 0x77B5 ^ (i * 977 + (0 if sym else 1))


def kv_long_seed(i, sym):
    return 0x51D0 ^ (i * 977 + (0 if sym else 1))


# tests/test_oracle.cpp:436-508: (S, D) with gs=32
F8_HOST_CFGS = [(64, 64), (7, 96), (16, 100), (5, 40), (3, 72)]


def f8_host_seed(i):
    return 0x8F1D ^ (i * 977)


def f8_gpu_seed(i):  # tests/test_gpu.cu:930-1078
    return 0xF80A ^ (i * 977)


# tests/test_gpu.cu:1085-1310: (H, S, D, gs, page)
PAGED_CFGS = [(2, 300, 96, 32, 16), (2, 520, 64, 32, 16), (1, 1000, 128, 64, 64), (3, 65, 40, 8, 32),
              (1, 5000, 64, 32, 256)]


def paged_seed(i, sym):
    return 0x9A6E ^ (i * 977 + (0 if sym else 1))


def digest(*arrays):
    h = hashlib.sha256()
    for a in arrays:
        if a is not None:
            h.update(np.ascontiguousarray(a).tobytes())
    return h.hexdigest()


def f16(bits):
    """uint16 bit patterns -> float64 values."""
    return np.asarray(bits, np.uint16).view(np.float16).astype(np.float64)


def rel_l2(got, ref):
    """sqrt(sum (got-ref)^2 / sum ref^2), denominator 1 when the reference is all zero
    (tests/test_gpu.cu:145-151)."""
    got = np.asarray(got, np.float64).ravel()
    ref = np.asarray(ref, np.float64).ravel()
    den = float(np.sum(ref * ref))
    return float(np.sqrt(np.sum((got - ref) ** 2) / (den if den > 0 else 1.0)))
