"""Helpers of the GPU parity tests: device buffers (torch is used for memory
only) and descriptors built from oracle-side packed artefacts."""
import numpy as np
import torch

import w4a16_dequant_gemm_b200 as w4


def dev(a):
    """numpy array -> device tensor holding the same bytes (None passes through)."""
    if a is None:
        return None
    a = np.ascontiguousarray(a)
    if a.dtype == np.uint16:
        return torch.from_numpy(a.view(np.int16)).cuda()
    if a.dtype == np.uint32:
        return torch.from_numpy(a.view(np.int32)).cuda()
    return torch.from_numpy(a).cuda()


def ptr(t):
    return None if t is None else t.data_ptr()


def empty_f16(n):
    return torch.empty(int(n), dtype=torch.float16, device="cuda")


def bits(t):
    """device FP16 tensor -> numpy uint16 bit patterns."""
    return t.detach().cpu().numpy().view(np.uint16).ravel()


class W4Weights:
    """Device copy of an oracle-packed W4 matrix plus its descriptor."""

    def __init__(self, p):
        self.q, self.s, self.z = dev(p["q"]), dev(p["scales"]), dev(p["zeros"])
        self.desc = w4.DevicePackedW(p["N"], p["K"], p["gs"], p["G"], int(p["symmetric"]), ptr(self.q),
                                     ptr(self.s), ptr(self.z))


class MxWeights:
    def __init__(self, p):
        self.q, self.s = dev(p["q"]), dev(p["scales"])
        self.desc = w4.DevicePackedWm(p["N"], p["K"], p["B"], ptr(self.q), ptr(self.s))


class KvW4:
    def __init__(self, c, S=None):
        self.t = {k: dev(c[k]) for k in ("q_k", "s_k", "z_k", "q_v", "s_v", "z_v")}
        self.desc = w4.DeviceKVW4(c["H"], c["S"] if S is None else S, c["D"], c["gs"], c["G"], int(c["symmetric"]),
                                  ptr(self.t["q_k"]), ptr(self.t["s_k"]), ptr(self.t["z_k"]), ptr(self.t["q_v"]),
                                  ptr(self.t["s_v"]), ptr(self.t["z_v"]))


class KvF8:
    def __init__(self, c):
        self.t = {k: dev(c[k]) for k in ("q_k", "s_k", "q_v", "s_v")}
        self.desc = w4.DeviceKVF8(c["H"], c["S"], c["D"], c["gs"], c["G"], ptr(self.t["q_k"]), ptr(self.t["s_k"]),
                                  ptr(self.t["q_v"]), ptr(self.t["s_v"]))


def sync_ok():
    """Synchronise; the kernels' own status word must be clean."""
    st = w4.device_status()
    assert st == 0, f"device status {st}: a bounded wait inside a kernel gave up"
