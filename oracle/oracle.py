"""ctypes binding of the CPU oracle (liboracle.so) -- TEST INFRASTRUCTURE ONLY.

Imported by tests/, by the smoke check and by the benchmark's CPU-baseline leg; never by the
shipped package.  Every function is a thin call into oracle/flint_attn_oracle.c, which restates
the reference's src/ref/ref_model.cpp:45-61,107-149.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "liboracle.so")

N_HEAD, N_HEAD_KV, HEAD_DIM, GQA = 32, 4, 128, 8
Q_DIM, KV_DIM, QKV_DIM = 4096, 512, 5120
N_SWA, MAX_CHUNK, SWA_RING = 513, 512, 1024

# Streams of the seeded generator: one per synthetic tensor kind.
STREAM_QKV, STREAM_QNORM, STREAM_KNORM, STREAM_SINKS, STREAM_KCACHE, STREAM_VCACHE, STREAM_CTX = 1, 2, 3, 4, 5, 6, 7


def build(force: bool = False) -> str:
    """Compile liboracle.so with the Makefile beside this file (gcc, a second or two)."""
    src = os.path.join(HERE, "flint_attn_oracle.c")
    if force or not os.path.exists(LIB_PATH) or os.path.getmtime(LIB_PATH) < os.path.getmtime(src):
        subprocess.run(["make", "-C", HERE, "liboracle.so"], check=True, capture_output=True)
    return LIB_PATH


_lib = None
_f32p = np.ctypeslib.ndpointer(np.float32, flags="C_CONTIGUOUS")
_u16p = np.ctypeslib.ndpointer(np.uint16, flags="C_CONTIGUOUS")
_i32p = np.ctypeslib.ndpointer(np.int32, flags="C_CONTIGUOUS")


def lib():
    global _lib
    if _lib is None:
        build()
        L = C.CDLL(LIB_PATH)
        L.fo_gen_normal.argtypes = [C.c_uint64, C.c_uint64, C.c_uint64, C.c_uint64, C.c_float, C.c_float, _f32p]
        L.fo_gen_u64.argtypes = [C.c_uint64, C.c_uint64, C.c_uint64]
        L.fo_gen_u64.restype = C.c_uint64
        L.fo_round_f16.argtypes = [_f32p, C.c_uint64]
        L.fo_round_bf16.argtypes = [_f32p, C.c_uint64]
        L.fo_f32_to_f16_bits.argtypes = [_f32p, _u16p, C.c_uint64]
        L.fo_f16_bits_to_f32.argtypes = [_u16p, _f32p, C.c_uint64]
        L.fo_f32_to_bf16_bits.argtypes = [_f32p, _u16p, C.c_uint64]
        L.fo_bf16_bits_to_f32.argtypes = [_u16p, _f32p, C.c_uint64]
        L.fo_rmsnorm.argtypes = [_f32p, _f32p, _f32p, C.c_int, C.c_float]
        L.fo_rope_neox.argtypes = [_f32p, C.c_int, C.c_int, C.c_float]
        L.fo_inv_freq.argtypes = [C.c_float, _f32p]
        L.fo_qk_norm_rope.argtypes = [_f32p, _f32p, _f32p, C.c_int, C.c_int]
        L.fo_attend.argtypes = [_f32p, _f32p, _f32p, _f32p, C.c_int, C.c_int, _f32p, C.c_int]
        L.fo_layer_forward.argtypes = [_f32p, C.c_int, C.c_int, _f32p, _f32p, _f32p, C.c_int, C.c_int, C.c_int,
                                       _f32p, _f32p, _f32p, C.c_int]
        L.fo_decode_token_f16cache.argtypes = [_f32p, C.c_int, _f32p, _f32p, _f32p, C.c_int, C.c_int, _u16p, _u16p,
                                               C.c_int64, _f32p, C.c_int]
        L.fo_attend_partial.argtypes = [_f32p, _f32p, _f32p, C.c_int, C.c_int, _f32p]
        L.fo_combine.argtypes = [_f32p, C.c_int, _f32p, _f32p]
        L.fo_attend_double_f16.argtypes = [_f32p, C.c_int, _f32p, _f32p, _f32p, C.c_int, C.c_int, _i32p, C.c_int, _i32p,
                                           C.c_int, np.ctypeslib.ndpointer(np.float64, flags="C_CONTIGUOUS")]
        L.fo_gen_grid.argtypes = [C.c_uint64, C.c_uint64, C.c_uint64, C.c_uint64, _f32p]
        L.fo_matvec.argtypes = [_f32p, _f32p, _f32p, C.c_int, C.c_int, C.c_int]
        L.fo_stack_forward.argtypes = [_f32p, _f32p, _f32p, _f32p, _f32p, _f32p, _f32p, _f32p, _f32p, _i32p, _i32p, _f32p,
                                       _f32p, _i32p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_int]
        L.fo_slot.argtypes = [C.c_int32, C.c_int]
        L.fo_slot.restype = C.c_int32
        L.fo_k_begin.argtypes = [C.c_int32, C.c_int]
        L.fo_k_begin.restype = C.c_int32
        L.fo_ref_split_policy.argtypes = [C.c_int32, C.c_int, C.POINTER(C.c_int32), C.POINTER(C.c_int32)]
        L.fo_rollback_restart.argtypes = [C.c_int32, C.c_int32]
        L.fo_rollback_restart.restype = C.c_int32
        L.fo_ring_owners.argtypes = [C.c_int32, _i32p]
        _lib = L
    return _lib


# ---------------------------------------------------------------- generator and conversions
def gen_normal(seed: int, stream: int, n: int, mean: float = 0.0, std: float = 1.0, first: int = 0) -> np.ndarray:
    out = np.empty(n, np.float32)
    lib().fo_gen_normal(seed, stream, first, n, mean, std, out)
    return out


def gen_u64(seed: int, stream: int, index: int) -> int:
    return int(lib().fo_gen_u64(seed, stream, index))


def round_f16(x: np.ndarray) -> np.ndarray:
    y = np.ascontiguousarray(x, np.float32).copy()
    lib().fo_round_f16(y.reshape(-1), y.size)
    return y


def round_bf16(x: np.ndarray) -> np.ndarray:
    y = np.ascontiguousarray(x, np.float32).copy()
    lib().fo_round_bf16(y.reshape(-1), y.size)
    return y


def to_f16_bits(x: np.ndarray) -> np.ndarray:
    x = np.ascontiguousarray(x, np.float32)
    out = np.empty(x.shape, np.uint16)
    lib().fo_f32_to_f16_bits(x.reshape(-1), out.reshape(-1), x.size)
    return out


def from_f16_bits(x: np.ndarray) -> np.ndarray:
    x = np.ascontiguousarray(x, np.uint16)
    out = np.empty(x.shape, np.float32)
    lib().fo_f16_bits_to_f32(x.reshape(-1), out.reshape(-1), x.size)
    return out


def to_bf16_bits(x: np.ndarray) -> np.ndarray:
    x = np.ascontiguousarray(x, np.float32)
    out = np.empty(x.shape, np.uint16)
    lib().fo_f32_to_bf16_bits(x.reshape(-1), out.reshape(-1), x.size)
    return out


def from_bf16_bits(x: np.ndarray) -> np.ndarray:
    x = np.ascontiguousarray(x, np.uint16)
    out = np.empty(x.shape, np.float32)
    lib().fo_bf16_bits_to_f32(x.reshape(-1), out.reshape(-1), x.size)
    return out


# ---------------------------------------------------------------- synthetic layer parameters
def layer_weights(seed: int, layer: int = 0):
    """q_norm, k_norm ~ 1 + N(0, 0.1) [128]; sinks ~ N(0, 1) [32] (the shapes of blk.N.attn_{q,k}_norm / attn_sinks)."""
    qn = gen_normal(seed, STREAM_QNORM + 16 * layer, HEAD_DIM, 1.0, 0.1)
    kn = gen_normal(seed, STREAM_KNORM + 16 * layer, HEAD_DIM, 1.0, 0.1)
    sk = gen_normal(seed, STREAM_SINKS + 16 * layer, N_HEAD, 0.0, 1.0)
    return qn, kn, sk


def raw_qkv(seed: int, layer: int, first_pos: int, n_tok: int, seq: int = 0) -> np.ndarray:
    """Raw (pre-norm) q|k|v rows [n_tok][5120] ~ N(0,1) of positions first_pos.. of sequence `seq`."""
    stream = STREAM_QKV + 16 * layer + 4096 * seq
    return gen_normal(seed, stream, n_tok * QKV_DIM, first=first_pos * QKV_DIM).reshape(n_tok, QKV_DIM)


# ---------------------------------------------------------------- arithmetic
def rmsnorm(x: np.ndarray, w: np.ndarray, eps: float = 1e-6) -> np.ndarray:
    x = np.ascontiguousarray(x, np.float32)
    y = np.empty_like(x)
    lib().fo_rmsnorm(x, np.ascontiguousarray(w, np.float32), y, x.size, eps)
    return y


def inv_freq(theta: float = 10000.0) -> np.ndarray:
    out = np.empty(64, np.float32)
    lib().fo_inv_freq(theta, out)
    return out


def qk_norm_rope(qkv_row: np.ndarray, qn, kn, pos: int, has_rope: bool) -> np.ndarray:
    row = np.ascontiguousarray(qkv_row, np.float32).copy()
    lib().fo_qk_norm_rope(row, qn, kn, pos, int(has_rope))
    return row


def layer_forward(qkv: np.ndarray, qn, kn, sinks, is_swa: bool, has_rope: bool, round_kv_f16: bool = False,
                  p0: int = 0, kc: np.ndarray | None = None, vc: np.ndarray | None = None, n_threads: int = 1):
    """Token-by-token attention of one layer. Returns (att [T][4096], kc, vc) with kc/vc [p0+T][512] fp32."""
    qkv = np.ascontiguousarray(qkv, np.float32)
    T = qkv.shape[0]
    kfull = np.zeros((p0 + T, KV_DIM), np.float32)
    vfull = np.zeros((p0 + T, KV_DIM), np.float32)
    if p0:
        kfull[:p0] = kc[:p0]
        vfull[:p0] = vc[:p0]
    att = np.empty((T, Q_DIM), np.float32)
    lib().fo_layer_forward(qkv.reshape(-1), T, p0, qn, kn, sinks, int(is_swa), int(has_rope), int(round_kv_f16),
                           kfull.reshape(-1), vfull.reshape(-1), att.reshape(-1), n_threads)
    return att, kfull, vfull


def decode_token_f16cache(qkv_row, pos: int, qn, kn, sinks, is_swa: bool, has_rope: bool, k16: np.ndarray,
                          v16: np.ndarray, n_threads: int = 1) -> np.ndarray:
    """k16/v16: uint16 half bits [4][n_slots][128] of one sequence; updated in place with the new token."""
    assert k16.dtype == np.uint16 and k16.flags.c_contiguous and v16.flags.c_contiguous
    n_slots = k16.shape[1]
    att = np.empty(Q_DIM, np.float32)
    lib().fo_decode_token_f16cache(np.ascontiguousarray(qkv_row, np.float32), pos, qn, kn, sinks, int(is_swa),
                                   int(has_rope), k16.reshape(-1), v16.reshape(-1), n_slots, att, n_threads)
    return att


# The probe set of the reference's own attention unit test (src/main.mm:280-281).
PROBE_POS = (0, 1, 31, 32, 200, 511, 512, 513, 600, 1023, 1024, 1100, 1299)
PROBE_HEADS = (0, 7, 8, 31)


def attend_double_f16(qkv: np.ndarray, qn, kn, sinks, is_swa: bool, has_rope: bool, probe_pos=PROBE_POS,
                      probe_heads=PROBE_HEADS) -> np.ndarray:
    """The reference's all-double statement with half-rounded K/V (src/main.mm:253-305) at the probe positions and
    heads: [n_pos][n_heads][128] float64."""
    qkv = np.ascontiguousarray(qkv, np.float32)
    pp, ph = np.asarray(probe_pos, np.int32), np.asarray(probe_heads, np.int32)
    out = np.empty((len(pp), len(ph), HEAD_DIM), np.float64)
    lib().fo_attend_double_f16(qkv.reshape(-1), qkv.shape[0], qn, kn, sinks, int(is_swa), int(has_rope), pp, len(pp), ph,
                               len(ph), out.reshape(-1))
    return out


def grid_qkv(seed: int, n_tok: int) -> np.ndarray:
    """Raw q|k|v rows [n_tok][5120] uniform on the grid {-2, -1.998, ..., 2}, the distribution of src/main.mm:247."""
    out = np.empty(n_tok * QKV_DIM, np.float32)
    lib().fo_gen_grid(seed, STREAM_QKV, 0, out.size, out)
    return out.reshape(n_tok, QKV_DIM)


def attend_partial(q, kc, vc, j0: int, j1: int) -> np.ndarray:
    part = np.empty((N_HEAD, HEAD_DIM + 2), np.float32)
    lib().fo_attend_partial(np.ascontiguousarray(q, np.float32).reshape(-1), kc.reshape(-1), vc.reshape(-1), j0, j1,
                            part.reshape(-1))
    return part


def combine(part: np.ndarray, sinks) -> np.ndarray:
    """part [32][n_split][130] -> out [32][128]."""
    part = np.ascontiguousarray(part, np.float32)
    out = np.empty((N_HEAD, HEAD_DIM), np.float32)
    lib().fo_combine(part.reshape(-1), part.shape[1], sinks, out.reshape(-1))
    return out


# ---------------------------------------------------------------- the attention stack with its projections
STREAM_EMBD, STREAM_ATTN_NORM, STREAM_WQ, STREAM_WK, STREAM_WV, STREAM_WO, STREAM_OUT_NORM, STREAM_WOUT = range(8, 16)


def matvec(w: np.ndarray, x: np.ndarray, n_threads: int = 1) -> np.ndarray:
    """y = W x with a double accumulator per row (src/ref/ref_model.cpp:74-92)."""
    w = np.ascontiguousarray(w, np.float32)
    y = np.empty(w.shape[0], np.float32)
    lib().fo_matvec(w.reshape(-1), np.ascontiguousarray(x, np.float32), y, w.shape[0], w.shape[1], n_threads)
    return y


def stack_weights(seed: int, n_layer: int, n_embd: int, n_vocab: int, layer_kinds):
    """Seeded weights of a small attention stack, every matrix rounded to bf16 (what the GPU holds): projections
    ~ N(0, 0.02), norms ~ 1 + N(0, 0.1), sinks ~ N(0, 1), embeddings ~ N(0, 1).  layer_kinds: [(is_swa, has_rope)].
    Returns a dict of fp32 arrays."""
    E = n_embd
    w = {"n_layer": n_layer, "n_embd": E, "n_vocab": n_vocab,
         "is_swa": np.array([int(k[0]) for k in layer_kinds], np.int32),
         "has_rope": np.array([int(k[1]) for k in layer_kinds], np.int32),
         "embd": round_bf16(gen_normal(seed, STREAM_EMBD, n_vocab * E)).reshape(n_vocab, E),
         "out_norm": gen_normal(seed, STREAM_OUT_NORM, E, 1.0, 0.1),
         "w_out": round_bf16(gen_normal(seed, STREAM_WOUT, n_vocab * E, 0.0, 0.02)).reshape(n_vocab, E)}
    per = {"attn_norm": [], "wq": [], "wk": [], "wv": [], "wo": [], "q_norm": [], "k_norm": [], "sinks": []}
    for il in range(n_layer):
        per["attn_norm"].append(gen_normal(seed, STREAM_ATTN_NORM + 16 * il, E, 1.0, 0.1))
        per["wq"].append(round_bf16(gen_normal(seed, STREAM_WQ + 16 * il, Q_DIM * E, 0.0, 0.02)).reshape(Q_DIM, E))
        per["wk"].append(round_bf16(gen_normal(seed, STREAM_WK + 16 * il, KV_DIM * E, 0.0, 0.02)).reshape(KV_DIM, E))
        per["wv"].append(round_bf16(gen_normal(seed, STREAM_WV + 16 * il, KV_DIM * E, 0.0, 0.02)).reshape(KV_DIM, E))
        per["wo"].append(round_bf16(gen_normal(seed, STREAM_WO + 16 * il, E * Q_DIM, 0.0, 0.02)).reshape(E, Q_DIM))
        qn, kn, sk = layer_weights(seed, il)
        per["q_norm"].append(qn); per["k_norm"].append(kn); per["sinks"].append(sk)
    for k, v in per.items():
        w[k] = np.ascontiguousarray(np.stack(v), np.float32)
    return w


def stack_forward(w: dict, tokens, want_logits: bool = True, want_hidden: bool = True, n_threads: int = 8):
    """The reference's forward pass with a zero feed-forward half (src/ref/ref_model.cpp:95-197), token by token from
    position 0.  Returns (logits [n_tok][n_vocab] or None, hidden [n_tok][n_embd] or None)."""
    tokens = np.ascontiguousarray(tokens, np.int32)
    n = tokens.size
    logits = np.empty((n, w["n_vocab"]), np.float32) if want_logits else None
    hidden = np.empty((n, w["n_embd"]), np.float32) if want_hidden else None
    f = lambda a: np.ascontiguousarray(a, np.float32).reshape(-1)  # noqa: E731
    lib().fo_stack_forward(f(w["embd"]), f(w["attn_norm"]), f(w["wq"]), f(w["wk"]), f(w["wv"]), f(w["q_norm"]),
                           f(w["k_norm"]), f(w["sinks"]), f(w["wo"]), w["is_swa"], w["has_rope"], f(w["out_norm"]),
                           f(w["w_out"]), tokens, n, w["n_layer"], w["n_embd"], w["n_vocab"],
                           logits.ctypes.data if want_logits else None, hidden.ctypes.data if want_hidden else None,
                           n_threads)
    return logits, hidden


# ---------------------------------------------------------------- integer maps
def slot(pos: int, is_swa: bool) -> int:
    return int(lib().fo_slot(pos, int(is_swa)))


def k_begin(pos: int, is_swa: bool) -> int:
    return int(lib().fo_k_begin(pos, int(is_swa)))


def ref_split_policy(pos: int, is_swa: bool):
    a, b = C.c_int32(), C.c_int32()
    lib().fo_ref_split_policy(pos, int(is_swa), C.byref(a), C.byref(b))
    return a.value, b.value


def rollback_restart(cached_len: int, p: int) -> int:
    return int(lib().fo_rollback_restart(cached_len, p))


def ring_owners(n: int) -> np.ndarray:
    out = np.empty(SWA_RING, np.int32)
    lib().fo_ring_owners(n, out)
    return out
