"""B200 (sm_100a) fused-dequant GEMM and flash-decode attention behind the
reference project's GPU API. The CUDA kernels and the C ABI live in csrc/;
capi.py binds the ABI and mirrors the reference's entry points."""
from . import build  # noqa: F401
from .capi import *  # noqa: F401,F403
from . import capi  # noqa: F401
from . import shard  # noqa: F401
from . import peer  # noqa: F401
