"""ctypes mirror of include/flint_capi.h: the reference's nine engine entry points (src/capi.h:20-37), bound the way
server/src/ffi.rs:18-98 binds them, plus a writer for the flat model container flint_open reads."""
from __future__ import annotations

import ctypes as C
import struct

import numpy as np

from . import capi

MAGIC = b"FLNTATT1"


class _Config(C.Structure):  # src/capi.h:12-17
    _fields_ = [("model_path", C.c_char_p), ("metallib_dir", C.c_char_p), ("pool_gb", C.c_double), ("n_ctx", C.c_int32)]


SYMBOLS = {
    "flint_open": (C.c_void_p, [C.POINTER(_Config), C.c_char_p, C.c_int32]),
    "flint_close": (None, [C.c_void_p]),
    "flint_n_ctx": (C.c_int32, [C.c_void_p]),
    "flint_n_vocab": (C.c_int32, []),
    "flint_pos": (C.c_int32, [C.c_void_p]),
    "flint_truncate": (C.c_int32, [C.c_void_p, C.c_int32]),
    "flint_prefill": (C.c_int32, [C.c_void_p, C.POINTER(C.c_int32), C.c_int32, C.c_char_p, C.c_int32]),
    "flint_decode": (C.c_int32, [C.c_void_p, C.c_int32, C.c_char_p, C.c_int32]),
    "flint_logits": (C.POINTER(C.c_float), [C.c_void_p]),
}


def _lib():
    lib = capi.load_library()
    if not getattr(lib, "_flint_capi_bound", False):
        for name, (res, args) in SYMBOLS.items():
            fn = getattr(lib, name)
            fn.restype, fn.argtypes = res, args
        lib._flint_capi_bound = True
    return lib


def _bf16_bits(x: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even bf16 bits of an fp32 array."""
    u = np.ascontiguousarray(x, np.float32).view(np.uint32)
    return ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)


def write_model_file(path: str, w: dict) -> None:
    """Write the container of include/flint_capi.h from fp32 arrays: embd [V][E], out_norm [E], w_out [V][E], per layer
    (leading axis) attn_norm [L][E], wq [L][4096][E], wk/wv [L][512][E], q_norm/k_norm [L][128], sinks [L][32],
    wo [L][E][4096], is_swa/has_rope [L].  Matrices are stored as bf16 (rounded to nearest even)."""
    L, E, V = int(w["n_layer"]), int(w["n_embd"]), int(w["n_vocab"])
    with open(path, "wb") as f:
        f.write(MAGIC + struct.pack("<iiii", L, E, V, 0))
        f.write(np.asarray(w["is_swa"], np.int32).tobytes() + np.asarray(w["has_rope"], np.int32).tobytes())
        f.write(_bf16_bits(w["embd"]).tobytes())
        for il in range(L):
            f.write(np.ascontiguousarray(w["attn_norm"][il], np.float32).tobytes())
            for k in ("wq", "wk", "wv"):
                f.write(_bf16_bits(w[k][il]).tobytes())
            for k in ("q_norm", "k_norm", "sinks"):
                f.write(np.ascontiguousarray(w[k][il], np.float32).tobytes())
            f.write(_bf16_bits(w["wo"][il]).tobytes())
        f.write(np.ascontiguousarray(w["out_norm"], np.float32).tobytes())
        f.write(_bf16_bits(w["w_out"]).tobytes())


class Engine:
    """One engine behind the reference's interface.  Single session, not thread-safe (src/capi.h:1)."""

    def __init__(self, model_path: str, n_ctx: int = 4096):
        self._lib = _lib()
        self._err = C.create_string_buffer(capi.ERR_LEN)
        cfg = _Config(model_path.encode(), b"", 0.0, n_ctx)
        self._h = self._lib.flint_open(C.byref(cfg), self._err, capi.ERR_LEN)
        if not self._h:
            raise capi.FlintAttnError(self._err.value.decode(errors="replace"))

    def close(self):
        if getattr(self, "_h", None):
            self._lib.flint_close(self._h)
            self._h = None

    __del__ = close

    def __enter__(self):
        return self

    def __exit__(self, *a):
        self.close()

    @property
    def n_ctx(self) -> int:
        return int(self._lib.flint_n_ctx(self._h))

    @property
    def n_vocab(self) -> int:
        return int(self._lib.flint_n_vocab())

    @property
    def pos(self) -> int:
        return int(self._lib.flint_pos(self._h))

    def truncate(self, pos: int) -> int:
        return int(self._lib.flint_truncate(self._h, pos))

    def prefill(self, tokens) -> int:
        arr = capi.i32_array(list(tokens))
        r = self._lib.flint_prefill(self._h, arr, len(arr), self._err, capi.ERR_LEN)
        if r < 0:
            raise capi.FlintAttnError(self._err.value.decode(errors="replace"))
        return int(r)

    def decode(self, token: int) -> int:
        r = self._lib.flint_decode(self._h, int(token), self._err, capi.ERR_LEN)
        if r < 0:
            raise capi.FlintAttnError(self._err.value.decode(errors="replace"))
        return int(r)

    def logits(self) -> np.ndarray:
        """A copy of the last call's logits (the library's buffer is only valid until the next call, src/capi.h:36)."""
        p = self._lib.flint_logits(self._h)
        return np.ctypeslib.as_array(p, shape=(self.n_vocab,)).copy()
