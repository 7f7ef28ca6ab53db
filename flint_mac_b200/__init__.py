"""B200-native attention hot path of flint-mac: sm_100a CUDA kernels behind a C ABI (include/flint_attn.h).

The Python here is only a ctypes mirror of that ABI, in the role the reference's server/src/ffi.rs plays for
src/capi.h.  There is no CPU fallback: without the compiled library, or without a B200, calls fail loudly.
"""
from .capi import Attn, FlintAttnError, load_library, F32, BF16, plan_decode, rollback_restart, decode_noalloc_dev, i32_array  # noqa: F401
from .engine import Engine, write_model_file  # noqa: F401,E402
from .sched import ContinuousBatcher, Router  # noqa: F401,E402
