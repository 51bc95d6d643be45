"""ctypes bindings for the CPU oracle (oracle/libw4oracle.so) and, when built,
the reference shim (oracle/_ref/libw4ref.so).

TEST INFRASTRUCTURE ONLY: imported by the test-suite, by the smoke check and by
the benchmark's CPU-baseline / reference arm. The GPU product path never
imports this module.

Both libraries export the same function set under the prefixes ``orc_`` (plain-C
restatement) and ``ref_`` (the reference's own headers); ``Lib`` hides the
prefix so a test can run the same call against either.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ORACLE_SO = os.path.join(HERE, "libw4oracle.so")
REF_SO = os.path.join(HERE, "_ref", "libw4ref.so")

_P = C.c_void_p


def reference_root() -> str:
    """Where the reference project's checkout is looked for: $W4_REFERENCE, else a directory named
    `reference` beside this repository's checkout. It may not exist (then nothing reference-derived is built)."""
    return os.environ.get("W4_REFERENCE") or os.path.normpath(os.path.join(HERE, "..", "..", "reference"))


def build(ref: bool = True) -> None:
    """Compile the oracle; also the reference shim when the reference tree exists."""
    subprocess.run(["make", "-C", HERE, "all"], check=True, stdout=subprocess.DEVNULL)
    root = reference_root()
    if ref and os.path.isfile(os.path.join(root, "include", "w4", "pack.hpp")):
        subprocess.run(["make", "-C", HERE, "ref", "REF=" + root], check=True, stdout=subprocess.DEVNULL)


def words(n: int) -> int:
    return (n + 7) // 8


def _ptr(a):
    if a is None:
        return None
    assert a.flags["C_CONTIGUOUS"]
    return a.ctypes.data_as(_P)


class Lib:
    """One of the two CPU implementations, selected by symbol prefix."""

    def __init__(self, path: str, prefix: str):
        self.path, self.prefix = path, prefix
        self.dll = C.CDLL(path)
        f = self._f
        f("f32_to_f16", C.c_uint16, [C.c_float])
        f("f16_to_f32", C.c_float, [C.c_uint16])
        f("normal_f64", None, [_P, C.c_size_t, C.c_uint64])
        f("normal_f16", None, [_P, C.c_size_t, C.c_uint64])
        f("dequant_one", C.c_uint16, [C.c_uint16, C.c_int, C.c_int])
        f("dequant_one_mx", C.c_uint16, [C.c_uint8, C.c_int])
        f("dequant_one_f8", C.c_uint16, [C.c_uint16, C.c_uint8])
        f("encode_e4m3", C.c_uint8, [C.c_float])
        f("quantize_w4", C.c_int, [_P, C.c_int, C.c_int, C.c_int, C.c_int, _P, _P, _P])
        f("dequant_all_w4", C.c_int, [C.c_int] * 5 + [_P, _P, _P, _P])
        f("gemm_oracle", C.c_int, [_P, C.c_int, C.c_int, _P, C.c_int, _P])
        f("gemm_oracle_mt", C.c_int, [_P, C.c_int, C.c_int, _P, C.c_int, _P, C.c_int])
        f("quantize_mx", C.c_int, [_P, C.c_int, C.c_int, _P, _P])
        f("dequant_all_mx", C.c_int, [C.c_int, C.c_int, C.c_int, _P, _P, _P])
        f("quantize_cache_w4", C.c_int, [_P, _P] + [C.c_int] * 5 + [_P] * 6)
        f("quantize_cache_f8", C.c_int, [_P, _P] + [C.c_int] * 4 + [_P] * 4)

    def _f(self, name, res, args):
        fn = getattr(self.dll, self.prefix + name)
        fn.restype, fn.argtypes = res, args
        setattr(self, "_" + name, fn)

    # ---- scalars -------------------------------------------------------
    def f32_to_f16(self, x):
        return int(self._f32_to_f16(float(x)))

    def f16_to_f32(self, h):
        return float(self._f16_to_f32(int(h)))

    def dequant_one(self, s, q, z):
        return int(self._dequant_one(int(s), int(q), int(z)))

    def dequant_one_mx(self, se, q):
        return int(self._dequant_one_mx(int(se), int(q)))

    def dequant_one_f8(self, s, b):
        return int(self._dequant_one_f8(int(s), int(b)))

    def encode_e4m3(self, x):
        return int(self._encode_e4m3(float(x)))

    # ---- generators ------------------------------------------------------
    def normal_f64(self, count, seed):
        out = np.empty(count, np.float64)
        self._normal_f64(_ptr(out), count, seed & (2**64 - 1))
        return out

    def normal_f16(self, count, seed):
        """FP16 bit patterns (uint16) of the reference's seeded activations."""
        out = np.empty(count, np.uint16)
        self._normal_f16(_ptr(out), count, seed & (2**64 - 1))
        return out

    # ---- W4 ---------------------------------------------------------------
    def quantize_w4(self, w, N, K, gs, symmetric):
        """-> dict(q, scales, zeros|None, G) or raises ValueError (invalid_argument)."""
        w = np.ascontiguousarray(w, np.float64)
        if N < 1 or K < 1 or gs < 8 or gs % 8:
            # shapes the output buffers cannot even be sized for: the call
            # still goes through so the library's own check is what answers
            rc = self._quantize_w4(_ptr(w), N, K, gs, int(symmetric), None, None, None)
            assert rc == 1
            raise ValueError("quantize_w4: invalid argument")
        if w.size != N * K:
            raise ValueError("quantize_w4: size")
        G = (K + gs - 1) // gs
        q = np.zeros(N * words(K), np.uint32)
        s = np.zeros(N * G, np.uint16)
        z = None if symmetric else np.zeros(N * words(G), np.uint32)
        rc = self._quantize_w4(_ptr(w), N, K, gs, int(symmetric), _ptr(q), _ptr(s), _ptr(z))
        if rc:
            raise ValueError("quantize_w4: invalid argument")
        return dict(N=N, K=K, gs=gs, G=G, symmetric=bool(symmetric), q=q, scales=s, zeros=z)

    def dequant_all_w4(self, p):
        w = np.empty(p["N"] * p["K"], np.uint16)
        rc = self._dequant_all_w4(p["N"], p["K"], p["gs"], p["G"], int(p["symmetric"]), _ptr(p["q"]),
                                  _ptr(p["scales"]), _ptr(p["zeros"]), _ptr(w))
        if rc:
            raise ValueError("dequant_all_w4: invalid argument")
        return w

    def gemm_oracle(self, x16, M, K, w16, N, threads=0):
        c = np.empty(M * N, np.float64)
        if threads and threads > 1:
            rc = self._gemm_oracle_mt(_ptr(x16), M, K, _ptr(w16), N, _ptr(c), threads)
        else:
            rc = self._gemm_oracle(_ptr(x16), M, K, _ptr(w16), N, _ptr(c))
        if rc:
            raise ValueError("gemm_oracle: invalid argument")
        return c

    # ---- MX ---------------------------------------------------------------
    def quantize_mx(self, w, N, K):
        w = np.ascontiguousarray(w, np.float64)
        if N < 1 or K < 1:
            rc = self._quantize_mx(_ptr(w), N, K, None, None)
            assert rc == 1
            raise ValueError("quantize_mx: invalid argument")
        if w.size != N * K:
            raise ValueError("quantize_mx: size")
        B = (K + 31) // 32
        q = np.zeros(N * words(K), np.uint32)
        s = np.zeros(N * B, np.uint8)
        rc = self._quantize_mx(_ptr(w), N, K, _ptr(q), _ptr(s))
        if rc:
            raise ValueError("quantize_mx: invalid argument")
        return dict(N=N, K=K, B=B, q=q, scales=s)

    def dequant_all_mx(self, p):
        w = np.empty(p["N"] * p["K"], np.uint16)
        rc = self._dequant_all_mx(p["N"], p["K"], p["B"], _ptr(p["q"]), _ptr(p["scales"]), _ptr(w))
        if rc:
            raise ValueError("dequant_all_mx: invalid argument")
        return w

    # ---- KV caches --------------------------------------------------------
    def quantize_cache_w4(self, k, v, H, S, D, gs, symmetric):
        k = np.ascontiguousarray(k, np.float64)
        v = np.ascontiguousarray(v, np.float64)
        if H < 1 or S < 1 or D < 1 or gs < 8 or gs % 8:
            raise ValueError("quantize_cache_w4: invalid argument")
        if k.size != H * S * D or v.size != H * S * D:
            raise ValueError("quantize_cache_w4: size")
        G = (D + gs - 1) // gs
        mk = lambda n, t: np.zeros(n, t)
        c = dict(H=H, S=S, D=D, gs=gs, G=G, symmetric=bool(symmetric))
        for side in "kv":
            c["q_" + side] = mk(H * S * words(D), np.uint32)
            c["s_" + side] = mk(H * S * G, np.uint16)
            c["z_" + side] = None if symmetric else mk(H * S * words(G), np.uint32)
        rc = self._quantize_cache_w4(_ptr(k), _ptr(v), H, S, D, gs, int(symmetric), _ptr(c["q_k"]),
                                     _ptr(c["s_k"]), _ptr(c["z_k"]), _ptr(c["q_v"]), _ptr(c["s_v"]),
                                     _ptr(c["z_v"]))
        if rc:
            raise ValueError("quantize_cache_w4: invalid argument")
        return c

    def quantize_cache_f8(self, k, v, H, S, D, gs):
        k = np.ascontiguousarray(k, np.float64)
        v = np.ascontiguousarray(v, np.float64)
        if H < 1 or S < 1 or D < 1 or gs < 8 or gs % 8:
            raise ValueError("quantize_cache_f8: invalid argument")
        if k.size != H * S * D or v.size != H * S * D:
            raise ValueError("quantize_cache_f8: size")
        G = (D + gs - 1) // gs
        c = dict(H=H, S=S, D=D, gs=gs, G=G)
        for side in "kv":
            c["q_" + side] = np.zeros(H * S * D, np.uint8)
            c["s_" + side] = np.zeros(H * S * G, np.uint16)
        rc = self._quantize_cache_f8(_ptr(k), _ptr(v), H, S, D, gs, _ptr(c["q_k"]), _ptr(c["s_k"]),
                                     _ptr(c["q_v"]), _ptr(c["s_v"]))
        if rc:
            raise ValueError("quantize_cache_f8: invalid argument")
        return c


class Oracle(Lib):
    """The plain-C restatement, plus the entry points only it has."""

    def __init__(self):
        if not os.path.exists(ORACLE_SO):
            build(ref=False)
        super().__init__(ORACLE_SO, "orc_")
        d = self.dll
        d.orc_dequant_cache_w4.restype = C.c_int
        d.orc_dequant_cache_w4.argtypes = [C.c_int] * 6 + [_P] * 4
        d.orc_dequant_cache_f8.restype = C.c_int
        d.orc_dequant_cache_f8.argtypes = [C.c_int] * 5 + [_P] * 3
        d.orc_attention_reference.restype = C.c_int
        d.orc_attention_reference.argtypes = [_P, _P, _P, C.c_int, C.c_int, C.c_int, _P, C.c_int]
        d.orc_paged_scatter.restype = C.c_int
        d.orc_paged_scatter.argtypes = [_P, _P, C.c_int, C.c_int, C.c_int, _P, C.c_int, C.c_int]
        d.orc_validate_block_table.restype = C.c_int
        d.orc_validate_block_table.argtypes = [_P, C.c_int, C.c_int, C.c_int]

    def dequant_cache_w4(self, c, side):
        out = np.empty(c["H"] * c["S"] * c["D"], np.uint16)
        rc = self.dll.orc_dequant_cache_w4(c["H"], c["S"], c["D"], c["gs"], c["G"], int(c["symmetric"]),
                                           _ptr(c["q_" + side]), _ptr(c["s_" + side]),
                                           _ptr(c["z_" + side]), _ptr(out))
        if rc:
            raise ValueError("dequant_cache_w4: invalid argument")
        return out

    def dequant_cache_f8(self, c, side):
        out = np.empty(c["H"] * c["S"] * c["D"], np.uint16)
        rc = self.dll.orc_dequant_cache_f8(c["H"], c["S"], c["D"], c["gs"], c["G"], _ptr(c["q_" + side]),
                                           _ptr(c["s_" + side]), _ptr(out))
        if rc:
            raise ValueError("dequant_cache_f8: invalid argument")
        return out

    def attention_reference(self, q16, kd16, vd16, H, S, D, threads=1):
        """FP64 decode attention over dequantised FP16 K/V [H][S][D] (uint16 bit patterns)."""
        out = np.empty(H * D, np.float64)
        rc = self.dll.orc_attention_reference(_ptr(q16), _ptr(kd16), _ptr(vd16), H, S, D, _ptr(out), threads)
        if rc:
            raise ValueError("attention_reference: invalid argument")
        return out

    def paged_from_contiguous(self, c, page, bt):
        """Scatter a contiguous W4 cache into a pool of ceil(S/page) pages per head."""
        bt = np.ascontiguousarray(bt, np.int32)
        H, S, D, G = c["H"], c["S"], c["D"], c["G"]
        lp = (S + page - 1) // page if page > 0 else 0
        if page < 1 or bt.size != lp:
            raise ValueError("paged_from_contiguous: invalid argument")
        p = dict(c)
        p.update(page=page, npages=lp, block_table=bt)
        for side in "kv":
            for key, elems, dt in (("q_", words(D), np.uint32), ("s_", G, np.uint16), ("z_", words(G), np.uint32)):
                src = c[key + side]
                if src is None:
                    p[key + side] = None
                    continue
                dst = np.zeros(H * lp * page * elems, dt)
                rc = self.dll.orc_paged_scatter(_ptr(src), _ptr(dst), H, S, page, _ptr(bt), elems,
                                                np.dtype(dt).itemsize)
                if rc:
                    raise ValueError("paged_from_contiguous: bad block table")
                p[key + side] = dst
        return p

    def validate_block_table(self, bt, S, page, npages):
        bt = np.ascontiguousarray(bt, np.int32)
        return self.dll.orc_validate_block_table(_ptr(bt), S, page, npages) == 0


class Reference(Lib):
    """The reference's own headers behind the shim (only where it was built)."""

    def __init__(self):
        super().__init__(REF_SO, "ref_")
        d = self.dll
        d.ref_attention_w4.restype = C.c_int
        d.ref_attention_w4.argtypes = [_P] + [C.c_int] * 6 + [_P] * 9
        d.ref_attention_f8.restype = C.c_int
        d.ref_attention_f8.argtypes = [_P] + [C.c_int] * 5 + [_P] * 7
        d.ref_paged_from_contiguous.restype = C.c_int
        d.ref_paged_from_contiguous.argtypes = [C.c_int] * 6 + [_P] * 6 + [C.c_int, _P, C.c_int] + [_P] * 6
        d.ref_cpu_path_w4.restype = C.c_int
        d.ref_cpu_path_w4.argtypes = [_P, _P] + [C.c_int] * 7 + [_P] * 6

    def attention_w4(self, q16, c, want_dequant=True):
        H, S, D = c["H"], c["S"], c["D"]
        out = np.empty(H * D, np.float64)
        kd = np.empty(H * S * D, np.uint16) if want_dequant else None
        vd = np.empty(H * S * D, np.uint16) if want_dequant else None
        rc = self.dll.ref_attention_w4(_ptr(q16), H, S, D, c["gs"], c["G"], int(c["symmetric"]),
                                       _ptr(c["q_k"]), _ptr(c["s_k"]), _ptr(c["z_k"]), _ptr(c["q_v"]),
                                       _ptr(c["s_v"]), _ptr(c["z_v"]), _ptr(out), _ptr(kd), _ptr(vd))
        if rc:
            raise ValueError("attention_w4: invalid argument")
        return out, kd, vd

    def attention_f8(self, q16, c, want_dequant=True):
        H, S, D = c["H"], c["S"], c["D"]
        out = np.empty(H * D, np.float64)
        kd = np.empty(H * S * D, np.uint16) if want_dequant else None
        vd = np.empty(H * S * D, np.uint16) if want_dequant else None
        rc = self.dll.ref_attention_f8(_ptr(q16), H, S, D, c["gs"], c["G"], _ptr(c["q_k"]), _ptr(c["s_k"]),
                                       _ptr(c["q_v"]), _ptr(c["s_v"]), _ptr(out), _ptr(kd), _ptr(vd))
        if rc:
            raise ValueError("attention_f8: invalid argument")
        return out, kd, vd

    def paged_from_contiguous(self, c, page, bt):
        bt = np.ascontiguousarray(bt, np.int32)
        H, S, D, G = c["H"], c["S"], c["D"], c["G"]
        lp = max(bt.size, 1)
        p = dict(c)
        p.update(page=page, npages=bt.size, block_table=bt)
        rows = H * lp * max(page, 1)
        for side in "kv":
            p["q_" + side] = np.zeros(rows * words(D), np.uint32)
            p["s_" + side] = np.zeros(rows * G, np.uint16)
            p["z_" + side] = None if c["symmetric"] else np.zeros(rows * words(G), np.uint32)
        rc = self.dll.ref_paged_from_contiguous(
            H, S, D, c["gs"], G, int(c["symmetric"]), _ptr(c["q_k"]), _ptr(c["s_k"]), _ptr(c["z_k"]),
            _ptr(c["q_v"]), _ptr(c["s_v"]), _ptr(c["z_v"]), page, _ptr(bt), bt.size, _ptr(p["q_k"]),
            _ptr(p["s_k"]), _ptr(p["z_k"]), _ptr(p["q_v"]), _ptr(p["s_v"]), _ptr(p["z_v"]))
        if rc:
            raise ValueError("paged_from_contiguous: invalid argument")
        return p

    def cpu_path_w4(self, w, x16, M, N, K, gs, symmetric, threads, packed=None):
        """Reference CPU path for one GEMM: (quantize) -> dequant_all -> gemm_oracle.
        Returns (wd16, c64, [t_quantize, t_dequant, t_gemm]) in seconds."""
        wd = np.empty(N * K, np.uint16)
        c = np.empty(M * N, np.float64)
        sec = np.zeros(3, np.float64)
        if packed is None:
            w = np.ascontiguousarray(w, np.float64)
            rc = self.dll.ref_cpu_path_w4(_ptr(w), _ptr(x16), M, N, K, gs, int(symmetric), threads, 1,
                                          None, None, None, _ptr(wd), _ptr(c), _ptr(sec))
        else:
            rc = self.dll.ref_cpu_path_w4(None, _ptr(x16), M, N, K, gs, int(symmetric), threads, 0,
                                          _ptr(packed["q"]), _ptr(packed["scales"]), _ptr(packed["zeros"]),
                                          _ptr(wd), _ptr(c), _ptr(sec))
        if rc:
            raise ValueError("cpu_path_w4: invalid argument")
        return wd, c, sec


def have_reference() -> bool:
    return os.path.exists(REF_SO)
