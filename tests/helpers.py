"""Shared helpers for the parity tests: seeded inputs from the oracle's generator and the tolerances of the task."""
from __future__ import annotations

import numpy as np

from oracle import oracle as fo

# Attention outputs vs the fp32 reference arithmetic: max-abs 2e-3, mean-abs 2e-4.
MAX_ABS_TOL = 2e-3
MEAN_ABS_TOL = 2e-4

KINDS = {  # name -> (is_swa, has_rope)
    "swa_rope": (True, True),
    "full_nope": (False, False),
    "full_rope": (False, True),
}


def assert_close(got: np.ndarray, want: np.ndarray, what: str = ""):
    got = np.asarray(got, np.float64).reshape(-1)
    want = np.asarray(want, np.float64).reshape(-1)
    assert np.isfinite(got).all(), f"{what}: non-finite output"
    err = np.abs(got - want)
    assert err.max() <= MAX_ABS_TOL, f"{what}: max-abs {err.max():.3e} > {MAX_ABS_TOL}"
    assert err.mean() <= MEAN_ABS_TOL, f"{what}: mean-abs {err.mean():.3e} > {MEAN_ABS_TOL}"
    return float(err.max()), float(err.mean())


def synth_cache_f16(seed: int, layer: int, seq: int, n_pos: int):
    """fp16 K/V ~ N(0,1) for positions [0, n_pos) of one sequence, position-major [n_pos][4][128] half bits."""
    k = fo.gen_normal(seed, fo.STREAM_KCACHE + 16 * layer + 4096 * seq, n_pos * fo.KV_DIM)
    v = fo.gen_normal(seed, fo.STREAM_VCACHE + 16 * layer + 4096 * seq, n_pos * fo.KV_DIM)
    return (fo.to_f16_bits(k).reshape(n_pos, 4, 128), fo.to_f16_bits(v).reshape(n_pos, 4, 128))


def to_slot_layout(kv_pos_major: np.ndarray, n_slots: int, is_swa: bool) -> np.ndarray:
    """[n_pos][4][128] by position -> [4][n_slots][128] by cache slot (ring: the last writer of a slot wins)."""
    n_pos = kv_pos_major.shape[0]
    out = np.zeros((4, n_slots, 128), np.uint16)
    if is_swa:
        first = max(0, n_pos - n_slots)
        pos = np.arange(first, n_pos)
        out[:, pos & (n_slots - 1)] = kv_pos_major[first:].transpose(1, 0, 2)
    else:
        out[:, :n_pos] = kv_pos_major.transpose(1, 0, 2)
    return out


def bf16_round_rows(x: np.ndarray):
    """(rounded fp32 values, uint16 bf16 bits)."""
    bits = fo.to_bf16_bits(x)
    return fo.from_bf16_bits(bits), bits


def oracle_at_positions(qkv: np.ndarray, weights, is_swa: bool, has_rope: bool, positions, round_kv_f16=False,
                        p0: int = 0):
    """Reference attention (src/ref arithmetic) at selected positions only: norm/RoPE every token to build the K/V
    history, then attend for the chosen ones.  qkv rows are positions p0.. ; returns ([len(positions)][4096], kc, vc)."""
    qn, kn, sinks = weights
    T = qkv.shape[0]
    rows = np.stack([fo.qk_norm_rope(qkv[t], qn, kn, p0 + t, has_rope) for t in range(T)])
    kc = np.zeros((p0 + T, fo.KV_DIM), np.float32)
    vc = np.zeros((p0 + T, fo.KV_DIM), np.float32)
    kc[p0:] = rows[:, fo.Q_DIM:fo.Q_DIM + fo.KV_DIM]
    vc[p0:] = rows[:, fo.Q_DIM + fo.KV_DIM:]
    if round_kv_f16:
        kc, vc = fo.round_f16(kc), fo.round_f16(vc)
    out = np.empty((len(positions), fo.Q_DIM), np.float32)
    for i, p in enumerate(positions):
        att = np.empty(fo.Q_DIM, np.float32)
        fo.lib().fo_attend(np.ascontiguousarray(rows[p - p0, :fo.Q_DIM]), kc.reshape(-1), vc.reshape(-1), sinks, p,
                           int(is_swa), att, 8)
        out[i] = att
    return out, kc, vc


def device_view(torch, ptr: int, numel: int, dtype):
    """A torch view (no copy) of device memory owned by the library, e.g. a layer's K or V cache."""
    class _Holder:
        pass

    itemsize = torch.empty((), dtype=dtype).element_size()
    holder = _Holder()
    holder.__cuda_array_interface__ = {"shape": (numel * itemsize,), "typestr": "|u1", "data": (ptr, False), "version": 3}
    return torch.as_tensor(holder, device="cuda").view(dtype)
