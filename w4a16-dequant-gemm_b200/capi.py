"""ctypes binding of the C ABI (include/w4b_abi.h) and a host-side mirror of the
reference's GPU entry points (namespace w4::gpu): same names, argument order
and error behaviour, so that tests read like the reference's own.

Contract violations raise ``InvalidArgument`` (the reference's
std::invalid_argument), CUDA failures raise ``CudaError`` (its
std::runtime_error). Device buffers are passed as integers (device addresses),
e.g. ``tensor.data_ptr()``; nothing here allocates or touches device memory.
There is no CPU fallback: without the compiled library the import fails.
"""
from __future__ import annotations

import ctypes as C
import os
from dataclasses import dataclass
from typing import Optional

from . import build as _build

PATH_AUTO, PATH_STREAM, PATH_TENSOR, PATH_GENERIC = 0, 1, 2, 3


class InvalidArgument(ValueError):
    """A contract violation, rejected on the host before any launch."""


class CudaError(RuntimeError):
    """A CUDA runtime failure reported by the library."""


class _PackedW4(C.Structure):
    _fields_ = [("N", C.c_int), ("K", C.c_int), ("gs", C.c_int), ("G", C.c_int), ("symmetric", C.c_int),
                ("q", C.c_void_p), ("scales", C.c_void_p), ("zeros", C.c_void_p)]


class _PackedMx(C.Structure):
    _fields_ = [("N", C.c_int), ("K", C.c_int), ("B", C.c_int), ("q", C.c_void_p), ("scales", C.c_void_p)]


class _KvW4(C.Structure):
    _fields_ = [("H", C.c_int), ("S", C.c_int), ("D", C.c_int), ("gs", C.c_int), ("G", C.c_int),
                ("symmetric", C.c_int), ("q_k", C.c_void_p), ("s_k", C.c_void_p), ("z_k", C.c_void_p),
                ("q_v", C.c_void_p), ("s_v", C.c_void_p), ("z_v", C.c_void_p)]


class _KvF8(C.Structure):
    _fields_ = [("H", C.c_int), ("S", C.c_int), ("D", C.c_int), ("gs", C.c_int), ("G", C.c_int),
                ("q_k", C.c_void_p), ("s_k", C.c_void_p), ("q_v", C.c_void_p), ("s_v", C.c_void_p)]


# Every symbol include/w4b_abi.h declares: name -> (restype, argtypes)
_P, _I = C.c_void_p, C.c_int
ABI = {
    "w4b_last_error": (C.c_char_p, []),
    "w4b_dispatch_mma_min_m": (_I, []),
    "w4b_gemm_w4_route": (_I, [C.POINTER(_PackedW4), _I, _I, _P]),
    "w4b_gemm_mx_route": (_I, [C.POINTER(_PackedMx), _I, _I, _P]),
    "w4b_device_status": (_I, []),
    "w4b_launch_count": (C.c_ulonglong, []),
    "w4b_set_launch_overlap": (_I, [_I]),
    "w4b_launch_overlap": (_I, []),
    "w4b_gemm_w4": (_I, [C.POINTER(_PackedW4), _P, _P, _I, _I, _P, _P]),
    "w4b_gemm_mx": (_I, [C.POINTER(_PackedMx), _P, _P, _I, _I, _P, _P]),
    "w4b_gemm_w4_hostio": (_I, [C.POINTER(_PackedW4), _P, _P, _I, _I, _P]),
    "w4b_gemm_w4_noalloc": (_I, [C.POINTER(_PackedW4), _P, _P, _I, _P]),
    "w4b_dequant_w4": (_I, [C.POINTER(_PackedW4), _P, _P]),
    "w4b_dequant_mx": (_I, [C.POINTER(_PackedMx), _P, _P]),
    "w4b_dequant_f8": (_I, [_P, _P, _P, _I, _I, _I, _P]),
    "w4b_quantize_w4": (_I, [_P, _I, _I, _I, _I, _I, _P, _P, _P, _P]),
    "w4b_quantize_mx": (_I, [_P, _I, _I, _I, _P, _P, _P]),
    "w4b_quantize_f8": (_I, [_P, _I, _I, _I, _I, _P, _P, _P]),
    "w4b_kv_append_w4": (_I, [C.POINTER(_KvW4), C.c_longlong, C.c_longlong, _P, _P, _I, _P]),
    "w4b_kv_append_f8": (_I, [C.POINTER(_KvF8), C.c_longlong, _P, _P, _I, _P]),
    "w4b_relayout_k": (_I, [_I]),
    "w4b_relayout_w4": (_I, [C.POINTER(_PackedW4), C.POINTER(_PackedW4), _P]),
    "w4b_relayout_mx": (_I, [C.POINTER(_PackedMx), C.POINTER(_PackedMx), _P]),
    "w4b_gemm_w4_padded": (_I, [C.POINTER(_PackedW4), _P, _I, _P, _I, _I, _P]),
    "w4b_gemm_mx_padded": (_I, [C.POINTER(_PackedMx), _P, _I, _P, _I, _I, _P]),
    "w4b_attn_flash_fp16": (_I, [_P, _P, _P, _P, _I, _I, _I, _P]),
    "w4b_attn_flash_w4": (_I, [C.POINTER(_KvW4), _P, _P, _P, _P, _P]),
    "w4b_attn_flash_f8": (_I, [C.POINTER(_KvF8), _P, _P, _P, _P, _P]),
    "w4b_attn_flash_w4_paged": (_I, [C.POINTER(_KvW4), _P, _I, _I, _P, _P, _P, _P, _P]),
    "w4b_attn_flash_w4_paged_batched": (_I, [C.POINTER(_KvW4), _P, _I, _P, _I, _I, _I, _I, _P, _P, _P]),
    "w4b_attn_single_fp16": (_I, [_P, _P, _P, _P, _I, _I, _I, _P]),
    "w4b_attn_single_w4": (_I, [C.POINTER(_KvW4), _P, _P, _P, _P, _P]),
    "w4b_peer_alloc": (_I, [C.c_size_t, C.POINTER(_P), _P]),
    "w4b_peer_open": (_I, [_P, C.POINTER(_P)]),
    "w4b_peer_close": (_I, [_P]),
    "w4b_peer_free": (_I, [_P]),
    "w4b_allgather_push": (_I, [_P, C.c_size_t, C.POINTER(_P), C.POINTER(_P), _P, _P, _I, _I, _I, _P]),
    "w4b_allgather_wait": (_I, [_P, _P, _I, _I, _P]),
    "w4b_gemm_w4_push": (_I, [C.POINTER(_PackedW4), _P, _P, _I, C.POINTER(_P), C.POINTER(_P), _P, _P, _P, _I, _I, _P]),
    "w4b_gemm_w4_carry": (_I, [C.POINTER(_PackedW4), _P, _P, _I, _P, C.c_size_t, C.POINTER(_P), C.POINTER(_P), _P, _P, _P,
                               _I, _I, _P]),
}


def _load():
    path = _build.LIB
    if not os.path.exists(path):
        raise ImportError(f"{path} is missing: build it with `python w4a16-dequant-gemm_b200/build.py` "
                          "(there is no CPU fallback)")
    dll = C.CDLL(path)
    for name, (res, args) in ABI.items():
        fn = getattr(dll, name)
        fn.restype, fn.argtypes = res, args
    return dll


lib = _load()


def _check(rc: int):
    if rc == 0:
        return
    msg = lib.w4b_last_error().decode()
    if rc == 1:
        raise InvalidArgument(msg)
    raise CudaError(msg)


# ---- the reference's descriptor structs, as plain Python ------------------

@dataclass
class DevicePackedW:  # include/w4/dequant.cuh:31-37
    N: int
    K: int
    gs: int
    G: int
    symmetric: int
    q: int
    scales: int
    zeros: Optional[int] = None

    def _c(self):
        return _PackedW4(self.N, self.K, self.gs, self.G, int(self.symmetric), self.q, self.scales, self.zeros)


@dataclass
class DevicePackedWm:  # include/w4/mxfused.cuh:26-30
    N: int
    K: int
    B: int
    q: int
    scales: int

    def _c(self):
        return _PackedMx(self.N, self.K, self.B, self.q, self.scales)


@dataclass
class DeviceKVW4:  # include/w4/kvattention.cuh:39-48
    H: int
    S: int
    D: int
    gs: int
    G: int
    symmetric: int
    q_k: int
    s_k: int
    z_k: Optional[int]
    q_v: int
    s_v: int
    z_v: Optional[int]

    def _c(self):
        return _KvW4(self.H, self.S, self.D, self.gs, self.G, int(self.symmetric), self.q_k, self.s_k, self.z_k,
                     self.q_v, self.s_v, self.z_v)


@dataclass
class DeviceKVF8:  # include/w4/kvflash.cuh:390-396
    H: int
    S: int
    D: int
    gs: int
    G: int
    q_k: int
    s_k: int
    q_v: int
    s_v: int

    def _c(self):
        return _KvF8(self.H, self.S, self.D, self.gs, self.G, self.q_k, self.s_k, self.q_v, self.s_v)


# ---- entry points, named as in the reference ------------------------------

def DISPATCH_MMA_MIN_M() -> int:  # include/w4/dispatch.cuh:25
    return lib.w4b_dispatch_mma_min_m()


def gemm(p: DevicePackedW, x, c, M, stream=None, w_out=None, path=PATH_AUTO):  # dispatch.cuh:27
    _check(lib.w4b_gemm_w4(C.byref(p._c()), x, c, M, path, stream, w_out))


def gemm_fused(p, x, c, M, stream=None, w_out=None):  # fused.cuh:172
    gemm(p, x, c, M, stream, w_out, PATH_STREAM)


def gemm_mma(p, x, c, M, stream=None, w_out=None):  # mma.cuh:234
    gemm(p, x, c, M, stream, w_out, PATH_TENSOR)


def gemm_mx(p: DevicePackedWm, x, c, M, stream=None, w_out=None, path=PATH_AUTO):  # dispatch.cuh:36
    _check(lib.w4b_gemm_mx(C.byref(p._c()), x, c, M, path, stream, w_out))


def gemm_fused_mx(p, x, c, M, stream=None, w_out=None):  # mxfused.cuh:166
    gemm_mx(p, x, c, M, stream, w_out, PATH_STREAM)


def gemm_mma_mx(p, x, c, M, stream=None, w_out=None):  # mxfused.cuh:291
    gemm_mx(p, x, c, M, stream, w_out, PATH_TENSOR)


def gemm_hostio(p: DevicePackedW, x_host, c_host, M, stream=None, path=PATH_AUTO):
    """x_host / c_host are HOST addresses (pinned for full speed); weights stay on the device."""
    _check(lib.w4b_gemm_w4_hostio(C.byref(p._c()), x_host, c_host, M, path, stream))


def gemm_noalloc(p: DevicePackedW, x, c, M, stream=None):
    """The stream GEMM with its scratch in a fixed array of the library image: for callers
    that may not allocate (graph capture, pooled memory, no-allocation serving loops)."""
    _check(lib.w4b_gemm_w4_noalloc(C.byref(p._c()), x, c, M, stream))


def gemm_route(p, M, path=PATH_AUTO, x=16) -> int:
    if isinstance(p, DevicePackedWm):
        return lib.w4b_gemm_mx_route(C.byref(p._c()), M, path, x)
    return lib.w4b_gemm_w4_route(C.byref(p._c()), M, path, x)


def dequant(p: DevicePackedW, w, stream=None):  # dequant.cuh:62
    _check(lib.w4b_dequant_w4(C.byref(p._c()), w, stream))


def dequant_mx(p: DevicePackedWm, w, stream=None):  # mxfused.cuh:57
    _check(lib.w4b_dequant_mx(C.byref(p._c()), w, stream))


def dequant_f8(q, s, w, S, D, gs, stream=None):  # kvflash.cuh:435
    _check(lib.w4b_dequant_f8(q, s, w, S, D, gs, stream))


def attention_fp16_flash(q, k16, v16, out, H, S, D, stream=None):  # kvflash.cuh:365
    _check(lib.w4b_attn_flash_fp16(q, k16, v16, out, H, S, D, stream))


def attention_w4_flash(p: DeviceKVW4, q, out, stream=None, k_out=None, v_out=None):  # kvflash.cuh:350
    _check(lib.w4b_attn_flash_w4(C.byref(p._c()), q, out, stream, k_out, v_out))


def attention_f8_flash(p: DeviceKVF8, q, out, stream=None, k_out=None, v_out=None):  # kvflash.cuh:572
    _check(lib.w4b_attn_flash_f8(C.byref(p._c()), q, out, stream, k_out, v_out))


def attention_w4_flash_paged(p: DeviceKVW4, bt, page, npages, q, out, stream=None, k_out=None,
                             v_out=None):  # kvflash.cuh:725
    _check(lib.w4b_attn_flash_w4_paged(C.byref(p._c()), bt, page, npages, q, out, stream, k_out, v_out))


def attention_w4_flash_paged_batched(p: DeviceKVW4, bt, bt_stride, seq_lens, nseq, max_seq_len, page, npages, q, out,
                                     stream=None):
    """nseq sequences over one pool in one launch (no reference counterpart: its paged entry takes one
    sequence per call). Blocks whose page is common to eight consecutive sequences of equal length are
    decoded once for the eight; out[i] is attention_w4_flash_paged on sequence i up to the order of the sums."""
    _check(lib.w4b_attn_flash_w4_paged_batched(C.byref(p._c()), bt, bt_stride, seq_lens, nseq, max_seq_len, page, npages,
                                               q, out, stream))


def attention_fp16(q, k16, v16, out, H, S, D, stream=None):  # kvattention.cuh:226
    _check(lib.w4b_attn_single_fp16(q, k16, v16, out, H, S, D, stream))


def attention_w4(p: DeviceKVW4, q, out, stream=None, k_out=None, v_out=None):  # kvattention.cuh:241
    _check(lib.w4b_attn_single_w4(C.byref(p._c()), q, out, stream, k_out, v_out))


# ---- device-side quantizers and KV append (the reference quantises on the host only) ------------

def quantize(w, N, K, gs, symmetric, q, scales, zeros=None, f16=False, stream=None):  # pack.hpp:64
    _check(lib.w4b_quantize_w4(w, int(f16), N, K, gs, int(symmetric), q, scales, zeros, stream))


def quantize_mx(w, N, K, q, scales, f16=False, stream=None):  # mx.hpp:71
    _check(lib.w4b_quantize_mx(w, int(f16), N, K, q, scales, stream))


def quantize_f8(x, rows, D, gs, q, scales, f16=False, stream=None):  # kvfp8.hpp:70 (one side)
    _check(lib.w4b_quantize_f8(x, int(f16), rows, D, gs, q, scales, stream))


def kv_append_w4(p: DeviceKVW4, row, slab_rows, k_new, v_new, f16=False, stream=None):
    """Quantise one token's K / V (H*D values each) into row `row` of every head slab of a W4 cache."""
    _check(lib.w4b_kv_append_w4(C.byref(p._c()), row, slab_rows, k_new, v_new, int(f16), stream))


def kv_append_f8(p: DeviceKVF8, row, k_new, v_new, f16=False, stream=None):
    _check(lib.w4b_kv_append_f8(C.byref(p._c()), row, k_new, v_new, int(f16), stream))


# ---- offline re-layout: the same matrix zero-extended along K (no counterpart in the reference) ----

def relayout_k(K: int) -> int:
    """The K a matrix is extended to: the next multiple of 512."""
    r = lib.w4b_relayout_k(K)
    if r < 0:
        raise InvalidArgument("relayout_k: bad K")
    return r


def relayout(src: DevicePackedW, dst: DevicePackedW, stream=None):
    """Writes src, zero-extended along K to dst.K, into dst's buffers (same format, every word written)."""
    _check(lib.w4b_relayout_w4(C.byref(src._c()), C.byref(dst._c()), stream))


def relayout_mx(src: DevicePackedWm, dst: DevicePackedWm, stream=None):
    _check(lib.w4b_relayout_mx(C.byref(src._c()), C.byref(dst._c()), stream))


def gemm_padded(p: DevicePackedW, x, K_x, c, M, stream=None, path=PATH_AUTO):
    """gemm for activations of K_x <= p.K columns: x is padded with zeros in library scratch first."""
    _check(lib.w4b_gemm_w4_padded(C.byref(p._c()), x, K_x, c, M, path, stream))


def gemm_mx_padded(p: DevicePackedWm, x, K_x, c, M, stream=None, path=PATH_AUTO):
    _check(lib.w4b_gemm_mx_padded(C.byref(p._c()), x, K_x, c, M, path, stream))


def device_status() -> int:
    """Synchronises and returns (then clears) the kernels' status word; 0 is healthy."""
    return lib.w4b_device_status()


def launch_count() -> int:
    return int(lib.w4b_launch_count())


def set_launch_overlap(on: bool) -> bool:
    """Lets consecutive stream-GEMM launches of a stream overlap (programmatic dependent launch): a launch
    pre-loads its packed weights while the previous kernel is still running. Only for weights that no
    kernel writes directly before the GEMM in the same stream. Returns the previous setting."""
    return bool(lib.w4b_set_launch_overlap(1 if on else 0))


def launch_overlap() -> bool:
    return bool(lib.w4b_launch_overlap())


# ---- all-gather over peer memory (no reference counterpart) ----------------------------------

def peer_alloc(nbytes: int):
    """cudaMalloc + zero-fill an arena on the current device; returns (device address, 64-byte IPC handle)."""
    ptr, handle = _P(), C.create_string_buffer(64)
    _check(lib.w4b_peer_alloc(nbytes, C.byref(ptr), handle))
    return ptr.value, handle.raw


def peer_open(handle: bytes) -> int:
    """Map a peer's arena from its IPC handle; returns its address in this process."""
    ptr = _P()
    _check(lib.w4b_peer_open(C.create_string_buffer(handle, 64), C.byref(ptr)))
    return ptr.value


def peer_close(ptr: int):
    _check(lib.w4b_peer_close(ptr))


def peer_free(ptr: int):
    _check(lib.w4b_peer_free(ptr))


def allgather_push(src, nbytes, dst, flag_dst, flags_local, counters, rank, world, wait_now=True, stream=None):
    """One all-gather step: push the slice at `src` to every peer's `dst[p]` and post the step flag; wait for
    the peers' slices of this step (wait_now) or only of the previous one."""
    arr = _P * world
    _check(lib.w4b_allgather_push(src, nbytes, arr(*dst), arr(*flag_dst), flags_local, counters, rank, world,
                                  1 if wait_now else 0, stream))


def gemm_push(p: DevicePackedW, x, c, M, c_peer, flag_dst, flags_local, counters, done, rank, world, stream=None):
    """The sharded GEMM with the exchange in its epilogue: c (this rank's slice buffer) also goes to c_peer[p]
    in every peer's arena and the step flag is posted, all in the one kernel."""
    arr = _P * world
    _check(lib.w4b_gemm_w4_push(C.byref(p._c()), x, c, M, arr(*c_peer), arr(*flag_dst), flags_local, counters, done,
                                rank, world, stream))


def gemm_carry(p: DevicePackedW, x, c, M, prev, prev_bytes, prev_peer, flag_dst, flags_local, counters, done, rank, world,
               stream=None):
    """The sharded GEMM of a step with the exchange of the previous step inside it: `prev` (this rank's finished
    slice of the previous step) goes to prev_peer[p] in every peer's arena while this step's weights stream."""
    arr = _P * world
    _check(lib.w4b_gemm_w4_carry(C.byref(p._c()), x, c, M, prev, prev_bytes, arr(*prev_peer), arr(*flag_dst), flags_local,
                                 counters, done, rank, world, stream))


def allgather_wait(flags_local, counters, rank, world, stream=None):
    """Wait (on the stream) until every peer's slice of the last pushed step has arrived."""
    _check(lib.w4b_allgather_wait(flags_local, counters, rank, world, stream))

