"""ctypes mirror of include/flint_attn.h (what server/src/ffi.rs:5-98 is to the reference's src/capi.h)."""
from __future__ import annotations

import ctypes as C
import os
from typing import Sequence

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
# FLINT_ATTN_LIB names another build of the same library (an A/B comparison, a debug build)
LIB_PATH = os.environ.get("FLINT_ATTN_LIB") or os.path.join(HERE, "libflint_attn.so")

F32, BF16 = 0, 1
N_HEAD, N_HEAD_KV, HEAD_DIM = 32, 4, 128
QKV_DIM, OUT_DIM, PARTIAL_DIM = 5120, 4096, 130
ERR_LEN = 1024  # server/src/ffi.rs:38


class FlintAttnError(RuntimeError):
    pass


class _Config(C.Structure):
    _fields_ = [("device", C.c_int32), ("n_layers", C.c_int32), ("layer_is_swa", C.POINTER(C.c_int32)),
                ("layer_has_rope", C.POINTER(C.c_int32)), ("max_seqs", C.c_int32), ("n_ctx", C.c_int32),
                ("kv_rank", C.c_int32), ("kv_ranks", C.c_int32), ("kv_pages", C.c_int32)]


SYMBOLS = {
    "flint_attn_open": (C.c_void_p, [C.POINTER(_Config), C.c_char_p, C.c_int32]),
    "flint_attn_close": (None, [C.c_void_p]),
    "flint_attn_n_ctx": (C.c_int32, [C.c_void_p]),
    "flint_attn_pos": (C.c_int32, [C.c_void_p, C.c_int32]),
    "flint_attn_truncate": (C.c_int32, [C.c_void_p, C.c_int32, C.c_int32]),
    "flint_attn_rollback_restart": (C.c_int32, [C.c_int32, C.c_int32]),
    "flint_attn_advance": (C.c_int32, [C.c_void_p, C.c_int32, C.POINTER(C.c_int32), C.c_int32]),
    "flint_attn_set_layer": (C.c_int32, [C.c_void_p, C.c_int32, C.c_void_p, C.c_void_p, C.c_void_p, C.c_char_p, C.c_int32]),
    "flint_attn_decode": (C.c_int32, [C.c_void_p, C.c_int32, C.c_int32, C.POINTER(C.c_int32), C.c_void_p, C.c_int32,
                                      C.c_void_p, C.c_int32, C.c_char_p, C.c_int32]),
    "flint_attn_decode_dev": (C.c_int32, [C.c_void_p, C.c_int32, C.c_int32, C.POINTER(C.c_int32), C.c_void_p, C.c_int32,
                                          C.c_void_p, C.c_int32, C.c_void_p, C.c_char_p, C.c_int32]),
    "flint_attn_decode_partial_dev": (C.c_int32, [C.c_void_p, C.c_int32, C.c_int32, C.POINTER(C.c_int32), C.c_void_p,
                                                  C.c_int32, C.c_void_p, C.c_void_p, C.c_char_p, C.c_int32]),
    "flint_attn_combine_dev": (C.c_int32, [C.c_void_p, C.c_int32, C.c_int32, C.c_int32, C.c_void_p, C.c_void_p, C.c_int32,
                                           C.c_void_p, C.c_char_p, C.c_int32]),
    "flint_attn_xchg_create": (C.c_int32, [C.c_void_p, C.c_int32, C.c_void_p, C.c_char_p, C.c_int32]),
    "flint_attn_xchg_connect": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_char_p, C.c_int32]),
    "flint_attn_xchg_base": (C.c_void_p, [C.c_void_p]),
    "flint_attn_xchg_connect_local": (C.c_int32, [C.c_void_p, C.POINTER(C.c_void_p), C.c_char_p, C.c_int32]),
    "flint_attn_decode_xchg_post_dev": (C.c_int32, [C.c_void_p, C.c_int32, C.c_int32, C.POINTER(C.c_int32), C.c_void_p,
                                                    C.c_int32, C.c_void_p, C.c_char_p, C.c_int32]),
    "flint_attn_combine_xchg_dev": (C.c_int32, [C.c_void_p, C.c_int32, C.c_int32, C.c_void_p, C.c_int32, C.c_void_p,
                                                C.c_char_p, C.c_int32]),
    "flint_attn_prefill": (C.c_int32, [C.c_void_p, C.c_int32, C.c_int32, C.c_int32, C.c_void_p, C.c_int32, C.c_void_p,
                                       C.c_int32, C.c_char_p, C.c_int32]),
    "flint_attn_prefill_dev": (C.c_int32, [C.c_void_p, C.c_int32, C.c_int32, C.c_int32, C.c_void_p, C.c_int32, C.c_void_p,
                                           C.c_int32, C.c_void_p, C.c_char_p, C.c_int32]),
    "flint_attn_set_projections": (C.c_int32, [C.c_void_p, C.c_int32, C.c_int32, C.c_void_p, C.c_void_p, C.c_void_p,
                                               C.c_void_p, C.c_void_p, C.c_char_p, C.c_int32]),
    "flint_attn_decode_block_dev": (C.c_int32, [C.c_void_p, C.c_int32, C.c_int32, C.POINTER(C.c_int32), C.c_void_p,
                                                C.c_void_p, C.c_char_p, C.c_int32]),
    "flint_attn_prefill_block_dev": (C.c_int32, [C.c_void_p, C.c_int32, C.c_int32, C.c_int32, C.c_void_p, C.c_void_p,
                                                 C.c_char_p, C.c_int32]),
    "flint_attn_project_dev": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_int32, C.c_int32, C.c_void_p, C.c_int32,
                                           C.c_void_p, C.c_void_p, C.c_void_p, C.c_char_p, C.c_int32]),
    "flint_attn_prefill_partial_dev": (C.c_int32, [C.c_void_p, C.c_int32, C.c_int32, C.c_int32, C.c_void_p, C.c_int32,
                                                   C.c_void_p, C.c_void_p, C.c_void_p, C.c_char_p, C.c_int32]),
    "flint_attn_prefill_combine_dev": (C.c_int32, [C.c_void_p, C.c_int32, C.c_int32, C.c_void_p, C.c_void_p, C.c_void_p,
                                                   C.c_int32, C.c_void_p, C.c_char_p, C.c_int32]),
    "flint_attn_check": (C.c_int32, [C.c_void_p, C.c_char_p, C.c_int32]),
    "flint_attn_n_slots": (C.c_int32, [C.c_void_p, C.c_int32]),
    "flint_attn_read_kv": (C.c_int32, [C.c_void_p, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_void_p, C.c_void_p,
                                       C.c_char_p, C.c_int32]),
    "flint_attn_write_kv": (C.c_int32, [C.c_void_p, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_void_p, C.c_void_p,
                                        C.c_char_p, C.c_int32]),
    "flint_attn_kv_dev": (C.c_void_p, [C.c_void_p, C.c_int32, C.c_int32]),
    "flint_attn_set_pos": (C.c_int32, [C.c_void_p, C.c_int32, C.c_int32]),
    "flint_attn_seq_release": (C.c_int32, [C.c_void_p, C.c_int32]),
    "flint_attn_pages_free": (C.c_int32, [C.c_void_p]),
    "flint_attn_plan_decode": (C.c_int32, [C.c_int32, C.POINTER(C.c_int32), C.c_int32, C.c_int32, C.c_int32, C.c_int32,
                                           C.POINTER(C.c_int32), C.c_int32]),
    "flint_attn_set_target_items": (C.c_int32, [C.c_void_p, C.c_int32]),
    "flint_attn_launch_count": (C.c_int64, [C.c_void_p]),
    "flint_attn_set_timing": (C.c_int32, [C.c_void_p, C.c_int32]),
    "flint_attn_kernel_ms": (C.c_double, [C.c_void_p, C.POINTER(C.c_int64)]),
    "flint_attn_decode_noalloc_dev": (C.c_int32, [C.c_int32, C.POINTER(C.c_int32), C.c_void_p, C.c_int32, C.c_void_p,
                                                  C.c_int32, C.c_void_p, C.c_void_p, C.c_int32, C.c_int32, C.c_int32,
                                                  C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_char_p, C.c_int32]),
}

_lib = None


def load_library() -> C.CDLL:
    """Load libflint_attn.so (built in-tree by flint_mac_b200/build.py). Fails loudly if it is missing."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise FlintAttnError(f"{LIB_PATH} not built: run `python -m flint_mac_b200.build` (there is no CPU fallback)")
        lib = C.CDLL(LIB_PATH)
        for name, (res, args) in SYMBOLS.items():
            fn = getattr(lib, name)
            fn.restype, fn.argtypes = res, args
        _lib = lib
    return _lib


def _i32(xs):
    """int32 C array for a sequence of ints.  A ctypes int32 array (see i32_array) passes through untouched, so a
    caller that decodes the same batch every step converts its sequence list once."""
    if isinstance(xs, C.Array) and xs._type_ is C.c_int32:
        return xs
    if isinstance(xs, np.ndarray):
        xs = np.ascontiguousarray(xs, np.int32)
        return (C.c_int32 * xs.size).from_buffer_copy(xs)
    return (C.c_int32 * len(xs))(*xs)


def i32_array(xs):
    """Convert once, pass many times: the result is accepted wherever a list of sequence indices is."""
    return _i32(xs)


def _ptr(x) -> int:
    """Address of a numpy array (host) or of anything exposing data_ptr() (a torch tensor, host or device)."""
    if isinstance(x, np.ndarray):
        assert x.flags.c_contiguous
        return x.ctypes.data
    if hasattr(x, "data_ptr"):
        assert x.is_contiguous()
        return x.data_ptr()
    return int(x)


def plan_decode(pos: Sequence[int], is_swa: bool, kv_lo: int = 0, kv_hi: int = 2**31 - 1, target_items: int = 296):
    """Host-only: the decode work list as an int32 array [n_items][8] =
    (token, kv_head, j0, j1, fold_new_token, split, n_split, first_partial)."""
    lib = load_library()
    cap = 1 << 16
    while True:
        out = (C.c_int32 * (8 * cap))()
        n = lib.flint_attn_plan_decode(len(pos), _i32(pos), int(is_swa), kv_lo, kv_hi, target_items, out, cap)
        if n >= 0:
            return np.ctypeslib.as_array(out)[: 8 * n].reshape(n, 8).copy()
        cap *= 4


def rollback_restart(cached_len: int, pos: int) -> int:
    return int(load_library().flint_attn_rollback_restart(cached_len, pos))


def decode_noalloc_dev(pos: Sequence[int], qkv_dev, qkv_dtype: int, out_dev, out_dtype: int, k_cache_dev, v_cache_dev,
                       n_slots: int, is_swa: bool, has_rope: bool, q_norm_dev, k_norm_dev, sinks_dev, stream: int = 0):
    """Handle-free decode attention that allocates nothing (flint_attn_decode_noalloc_dev): every buffer is the
    caller's, the scratch is a fixed array inside the library.  At most 64 tokens per call."""
    err = C.create_string_buffer(ERR_LEN)
    r = load_library().flint_attn_decode_noalloc_dev(
        len(pos), _i32(pos), _ptr(qkv_dev), qkv_dtype, _ptr(out_dev), out_dtype, _ptr(k_cache_dev), _ptr(v_cache_dev),
        n_slots, int(is_swa), int(has_rope), _ptr(q_norm_dev), _ptr(k_norm_dev), _ptr(sinks_dev), stream, err, ERR_LEN)
    if r != 0:
        raise FlintAttnError(err.value.decode(errors="replace"))


class Attn:
    """One attention handle on one GPU. Single owner, not thread-safe (src/capi.h:1)."""

    def __init__(self, layer_is_swa: Sequence[bool], layer_has_rope: Sequence[bool], max_seqs: int, n_ctx: int,
                 device: int = 0, kv_rank: int = 0, kv_ranks: int = 1, kv_pages: int = 0):
        self._lib = load_library()
        self._err = C.create_string_buffer(ERR_LEN)
        self.n_layers = len(layer_is_swa)
        swa, rope = _i32([int(b) for b in layer_is_swa]), _i32([int(b) for b in layer_has_rope])
        cfg = _Config(device, self.n_layers, swa, rope, max_seqs, n_ctx, kv_rank, kv_ranks, kv_pages)
        err = C.create_string_buffer(ERR_LEN)
        self._h = self._lib.flint_attn_open(C.byref(cfg), err, ERR_LEN)
        if not self._h:
            raise FlintAttnError(err.value.decode(errors="replace"))
        self.layer_is_swa = [bool(b) for b in layer_is_swa]
        self.layer_has_rope = [bool(b) for b in layer_has_rope]
        self.max_seqs, self.n_ctx = max_seqs, n_ctx

    def close(self):
        if getattr(self, "_h", None):
            self._lib.flint_attn_close(self._h)
            self._h = None

    __del__ = close

    def __enter__(self):
        return self

    def __exit__(self, *a):
        self.close()

    def _call(self, name, *args):
        err = self._err  # one buffer per handle (single owner, not thread-safe): nothing is allocated per call
        r = getattr(self._lib, name)(self._h, *args, err, ERR_LEN)
        if r != 0:
            raise FlintAttnError(err.value.decode(errors="replace"))

    # ---- state
    def pos(self, seq: int) -> int:
        return int(self._lib.flint_attn_pos(self._h, seq))

    def truncate(self, seq: int, pos: int) -> int:
        return int(self._lib.flint_attn_truncate(self._h, seq, pos))

    def set_pos(self, seq: int, pos: int) -> int:
        return int(self._lib.flint_attn_set_pos(self._h, seq, pos))

    def advance(self, seqs: Sequence[int], n_tokens: int = 1) -> int:
        return int(self._lib.flint_attn_advance(self._h, len(seqs), _i32(seqs), n_tokens))

    def seq_release(self, seq: int) -> int:
        """Retire a sequence slot: position 0, its KV pages back to the pool."""
        return int(self._lib.flint_attn_seq_release(self._h, seq))

    def pages_free(self) -> int:
        return int(self._lib.flint_attn_pages_free(self._h))

    def set_layer(self, layer: int, q_norm: np.ndarray, k_norm: np.ndarray, sinks: np.ndarray):
        q_norm, k_norm, sinks = (np.ascontiguousarray(x, np.float32) for x in (q_norm, k_norm, sinks))
        assert q_norm.size == 128 and k_norm.size == 128 and sinks.size == 32
        self._call("flint_attn_set_layer", layer, q_norm.ctypes.data, k_norm.ctypes.data, sinks.ctypes.data)

    def n_slots(self, layer: int) -> int:
        return int(self._lib.flint_attn_n_slots(self._h, layer))

    def set_target_items(self, n: int) -> int:
        return int(self._lib.flint_attn_set_target_items(self._h, n))

    def launch_count(self) -> int:
        return int(self._lib.flint_attn_launch_count(self._h))

    def set_timing(self, on: bool) -> None:
        self._lib.flint_attn_set_timing(self._h, int(on))

    def kernel_ms(self):
        """(summed milliseconds, number of timed calls) since the last query."""
        n = C.c_int64(0)
        ms = float(self._lib.flint_attn_kernel_ms(self._h, C.byref(n)))
        return ms, int(n.value)

    # ---- host-buffer operators (synchronous)
    def decode(self, layer: int, seqs: Sequence[int], qkv, qkv_dtype: int, out, out_dtype: int):
        self._call("flint_attn_decode", layer, len(seqs), _i32(seqs), _ptr(qkv), qkv_dtype, _ptr(out), out_dtype)

    def prefill(self, layer: int, seq: int, n_tok: int, qkv, qkv_dtype: int, out, out_dtype: int):
        self._call("flint_attn_prefill", layer, seq, n_tok, _ptr(qkv), qkv_dtype, _ptr(out), out_dtype)

    # ---- device-pointer operators (asynchronous on `stream`, a raw cudaStream_t value; 0 = default stream)
    def decode_dev(self, layer, seqs, qkv_dev, qkv_dtype, out_dev, out_dtype, stream: int = 0):
        self._call("flint_attn_decode_dev", layer, len(seqs), _i32(seqs), _ptr(qkv_dev), qkv_dtype, _ptr(out_dev),
                   out_dtype, stream)

    def prepared_decode_dev(self, layer, seqs, qkv_dtype, out_dev, out_dtype, stream: int = 0):
        """For a caller that decodes the same batch every step (a serving loop): every argument except the address
        of the step's q|k|v rows is converted once.  Returns f(qkv_address) that enqueues flint_attn_decode_dev."""
        fn, h, n, arr, outp, err = self._lib.flint_attn_decode_dev, self._h, len(seqs), _i32(seqs), _ptr(out_dev), self._err

        def call(qkv_address: int):
            if fn(h, layer, n, arr, qkv_address, qkv_dtype, outp, out_dtype, stream, err, ERR_LEN) != 0:
                raise FlintAttnError(err.value.decode(errors="replace"))

        return call

    def prepared_advance(self, seqs, n_tokens: int = 1):
        """f() that advances the given sequences by n_tokens, with the index list converted once."""
        fn, h, n, arr = self._lib.flint_attn_advance, self._h, len(seqs), _i32(seqs)

        def call():
            if fn(h, n, arr, n_tokens) != 0:
                raise FlintAttnError("advance failed: a sequence would pass the end of the context")

        return call

    def decode_partial_dev(self, layer, seqs, qkv_dev, qkv_dtype, partial_dev, stream: int = 0):
        self._call("flint_attn_decode_partial_dev", layer, len(seqs), _i32(seqs), _ptr(qkv_dev), qkv_dtype,
                   _ptr(partial_dev), stream)

    def combine_dev(self, layer, n, n_parts, partials_dev, out_dev, out_dtype, stream: int = 0):
        self._call("flint_attn_combine_dev", layer, n, n_parts, _ptr(partials_dev), _ptr(out_dev), out_dtype, stream)

    # ---- exchange of partial records through peer memory (KV-range sharding on the GPUs of one node)
    IPC_HANDLE_BYTES = 64

    def xchg_create(self, n_max: int) -> bytes:
        """Allocate this rank's gather buffer; returns its CUDA IPC handle for the other ranks' xchg_connect."""
        h = C.create_string_buffer(self.IPC_HANDLE_BYTES)
        self._call("flint_attn_xchg_create", n_max, C.cast(h, C.c_void_p))
        return h.raw

    def xchg_connect(self, handles):
        """handles: one IPC handle per rank, in rank order (this rank's own entry is not opened)."""
        blob = b"".join(handles)
        buf = C.create_string_buffer(blob, len(blob))
        self._call("flint_attn_xchg_connect", C.cast(buf, C.c_void_p))

    def xchg_base(self) -> int:
        return int(self._lib.flint_attn_xchg_base(self._h) or 0)

    def xchg_connect_local(self, bases):
        """Ranks that are handles of one process: bases[r] = rank r's xchg_base()."""
        arr = (C.c_void_p * len(bases))(*bases)
        self._call("flint_attn_xchg_connect_local", arr)

    def decode_xchg_post_dev(self, layer, seqs, qkv_dev, qkv_dtype, stream: int = 0):
        self._call("flint_attn_decode_xchg_post_dev", layer, len(seqs), _i32(seqs), _ptr(qkv_dev), qkv_dtype, stream)

    def combine_xchg_dev(self, layer, n, out_dev, out_dtype, stream: int = 0):
        self._call("flint_attn_combine_xchg_dev", layer, n, _ptr(out_dev), out_dtype, stream)

    def prefill_dev(self, layer, seq, n_tok, qkv_dev, qkv_dtype, out_dev, out_dtype, stream: int = 0):
        self._call("flint_attn_prefill_dev", layer, seq, n_tok, _ptr(qkv_dev), qkv_dtype, _ptr(out_dev), out_dtype,
                   stream)

    # ---- the attention block with its projections (residual stream rows in, updated in place)
    def set_projections(self, layer: int, attn_norm: np.ndarray, wq: np.ndarray, wk: np.ndarray, wv: np.ndarray,
                        wo: np.ndarray):
        """attn_norm fp32 [n_embd]; wq [4096][n_embd], wk/wv [512][n_embd], wo [n_embd][4096] as uint16 bf16 bits."""
        attn_norm = np.ascontiguousarray(attn_norm, np.float32)
        wq, wk, wv, wo = (np.ascontiguousarray(x, np.uint16) for x in (wq, wk, wv, wo))
        n_embd = attn_norm.size
        assert wq.shape == (4096, n_embd) and wk.shape == (512, n_embd) and wv.shape == (512, n_embd)
        assert wo.shape == (n_embd, 4096)
        self._call("flint_attn_set_projections", layer, n_embd, attn_norm.ctypes.data, wq.ctypes.data, wk.ctypes.data,
                   wv.ctypes.data, wo.ctypes.data)

    def decode_block_dev(self, layer, seqs, x_dev, stream: int = 0):
        self._call("flint_attn_decode_block_dev", layer, len(seqs), _i32(seqs), _ptr(x_dev), stream)

    def prefill_block_dev(self, layer, seq, n_tok, x_dev, stream: int = 0):
        self._call("flint_attn_prefill_block_dev", layer, seq, n_tok, _ptr(x_dev), stream)

    def project_dev(self, w_dev, n_rows_w, k, x_dev, n, norm_w_dev, out_dev, stream: int = 0):
        self._call("flint_attn_project_dev", _ptr(w_dev), n_rows_w, k, _ptr(x_dev), n,
                   _ptr(norm_w_dev) if norm_w_dev is not None else None, _ptr(out_dev), stream)

    def prefill_partial_dev(self, layer, seq, n_tok, qkv_dev, qkv_dtype, partial_o_dev, partial_ml_dev, stream: int = 0):
        self._call("flint_attn_prefill_partial_dev", layer, seq, n_tok, _ptr(qkv_dev), qkv_dtype, _ptr(partial_o_dev),
                   _ptr(partial_ml_dev), stream)

    def prefill_combine_dev(self, n_tok, n_parts, partials_o_dev, partials_ml_dev, out_dev, out_dtype, stream: int = 0):
        self._call("flint_attn_prefill_combine_dev", n_tok, n_parts, _ptr(partials_o_dev), _ptr(partials_ml_dev),
                   _ptr(out_dev), out_dtype, stream)

    def check(self):
        """Synchronise and raise if any asynchronous call of this handle failed on the device."""
        self._call("flint_attn_check")

    # ---- cache access (tests, cache pre-loading)
    def read_kv(self, layer: int, seq: int, slot0: int, n: int):
        k = np.empty((N_HEAD_KV, n, HEAD_DIM), np.uint16)
        v = np.empty((N_HEAD_KV, n, HEAD_DIM), np.uint16)
        self._call("flint_attn_read_kv", layer, seq, slot0, n, k.ctypes.data, v.ctypes.data)
        return k, v

    def write_kv(self, layer: int, seq: int, slot0: int, k: np.ndarray, v: np.ndarray):
        k, v = np.ascontiguousarray(k, np.uint16), np.ascontiguousarray(v, np.uint16)
        assert k.shape == v.shape and k.shape[0] == N_HEAD_KV and k.shape[2] == HEAD_DIM
        self._call("flint_attn_write_kv", layer, seq, slot0, k.shape[1], k.ctypes.data, v.ctypes.data)

    def kv_dev(self, layer: int, which: int) -> int:
        return int(self._lib.flint_attn_kv_dev(self._h, layer, which) or 0)
