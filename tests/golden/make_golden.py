"""Generate the golden attention vectors from the UNMODIFIED reference CPU model.

Run where the reference tree is mounted (it is not needed afterwards):

    make -C oracle ref            # compiles src/ref/ref_model.cpp etc. where they lie -> oracle/_ref/ref_attn
    python tests/golden/make_golden.py

For each layer kind it writes a synthetic all-F32 GGUF to a temporary directory, runs the reference's
RefModel::forward over 1300 tokens (src/ref/ref_model.cpp:95-197) through oracle/_ref/ref_attn, and stores in
tests/golden/ref_attn_<kind>.npz:

  probe_pos   the positions the reference's own test-attn probes (src/main.mm:280): query-block edges,
              window edges 511/512/513, ring wrap 1023/1024
  probe_att   float32 [n_probe][32][128] attention outputs at those positions, all heads
  row_sum     float64 [1300] sum of all 4096 outputs of every position (covers every position cheaply)
  row_abs     float64 [1300] sum of absolute values likewise
  seed, layer, is_swa, has_rope, n_tok

Inputs are not stored: tests regenerate them from (seed, layer) with the oracle's counter-based generator
and the same embedding-wide RMSNorm the reference applies before its projections (ref_model.cpp:108).

How the GGUF isolates attention.  n_embd = 9216 = 5120 + 4096.  Row t of token_embd is [x_t (5120 values ~ N(0,1)) |
4096 zeros]; attn_norm = 1; attn_q/k/v are selection matrices picking xn[0:4096], xn[4096:4608], xn[4608:5120];
attn_output copies head outputs into dims [5120, 9216), which are zero on input, so the residual add is exact;
the (dense) FFN has zero weights.  last_hidden()[5120:] is then the attention output, bit for bit.
"""
from __future__ import annotations

import os
import struct
import subprocess
import sys
import tempfile

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import oracle as fo  # noqa: E402

E = 9216
N_TOK = 1300
SEED = 0
PROBE_POS = [0, 1, 31, 32, 200, 511, 512, 513, 600, 1023, 1024, 1100, 1299]
KINDS = {  # name -> (layer index used for the generator streams, is_swa, has_rope)
    "swa_rope": (2, True, True),    # the reference's layer 2 (SWA + RoPE)
    "full_nope": (0, False, False),  # the reference's layer 0 (full attention, no RoPE)
    "full_rope": (1, False, True),   # full attention with RoPE (src/ref keeps the two flags independent)
}

U32, F32, BOOL, STR, ARR = 4, 6, 7, 8, 9


def _s(b: str) -> bytes:
    e = b.encode()
    return struct.pack("<Q", len(e)) + e


def _kv(key, typ, val) -> bytes:
    out = _s(key) + struct.pack("<I", typ)
    if typ == U32:
        out += struct.pack("<I", val)
    elif typ == F32:
        out += struct.pack("<f", val)
    elif typ == BOOL:
        out += struct.pack("<B", int(val))
    elif typ == STR:
        out += _s(val)
    elif typ == ARR:  # bool arrays only
        out += struct.pack("<IQ", BOOL, len(val)) + bytes(int(v) for v in val)
    return out


def token_rows(layer: int) -> np.ndarray:
    """x_t for t < N_TOK: [N_TOK][9216], first 5120 dims seeded N(0,1), rest zero."""
    x = np.zeros((N_TOK, E), np.float32)
    x[:, : fo.QKV_DIM] = fo.raw_qkv(SEED, layer, 0, N_TOK)
    return x


def effective_qkv(layer: int) -> np.ndarray:
    """What the reference's projections hand to attention: rows of rmsnorm_E(x_t)[0:5120] (ref_model.cpp:108-111)."""
    x = token_rows(layer)
    ones = np.ones(E, np.float32)
    return np.stack([fo.rmsnorm(x[t], ones)[: fo.QKV_DIM] for t in range(N_TOK)])


def write_gguf(path: str, layer: int, is_swa: bool, has_rope: bool) -> None:
    qn, kn, sinks = fo.layer_weights(SEED, layer)
    a = "flint"
    kvs = [
        _kv("general.architecture", STR, a),
        _kv(a + ".block_count", U32, 1), _kv(a + ".embedding_length", U32, E),
        _kv(a + ".attention.head_count", U32, 32), _kv(a + ".attention.head_count_kv", U32, 4),
        _kv(a + ".attention.key_length", U32, 128), _kv(a + ".feed_forward_length", U32, 1),
        _kv(a + ".expert_feed_forward_length", U32, 1), _kv(a + ".expert_shared_feed_forward_length", U32, 1),
        _kv(a + ".expert_count", U32, 1), _kv(a + ".expert_used_count", U32, 1),
        _kv(a + ".leading_dense_block_count", U32, 1), _kv(a + ".attention.sliding_window", U32, 513),
        _kv(a + ".attention.layer_norm_rms_epsilon", F32, 1e-6), _kv(a + ".rope.freq_base", F32, 10000.0),
        _kv(a + ".attention.sliding_window_pattern", ARR, [is_swa]), _kv(a + ".attention.rope_pattern", ARR, [has_rope]),
        _kv(a + ".expert_gating_func", U32, 2), _kv(a + ".expert_weights_norm", BOOL, True),
        _kv(a + ".expert_weights_scale", F32, 1.0),
    ]
    sel_q = np.zeros((4096, E), np.float32); sel_q[np.arange(4096), np.arange(4096)] = 1
    sel_k = np.zeros((512, E), np.float32); sel_k[np.arange(512), 4096 + np.arange(512)] = 1
    sel_v = np.zeros((512, E), np.float32); sel_v[np.arange(512), 4608 + np.arange(512)] = 1
    w_o = np.zeros((E, 4096), np.float32); w_o[5120 + np.arange(4096), np.arange(4096)] = 1
    ones = np.ones(E, np.float32)
    tensors = [  # (name, array whose LAST axis is ggml dims[0])
        ("token_embd.weight", token_rows(layer)), ("output_norm.weight", ones),
        ("output.weight", np.zeros((1, E), np.float32)),
        ("blk.0.attn_norm.weight", ones), ("blk.0.attn_q.weight", sel_q), ("blk.0.attn_k.weight", sel_k),
        ("blk.0.attn_v.weight", sel_v), ("blk.0.attn_q_norm.weight", qn), ("blk.0.attn_k_norm.weight", kn),
        ("blk.0.attn_sinks.weight", sinks), ("blk.0.attn_output.weight", w_o), ("blk.0.ffn_norm.weight", ones),
        ("blk.0.ffn_gate.weight", np.zeros((1, E), np.float32)), ("blk.0.ffn_up.weight", np.zeros((1, E), np.float32)),
        ("blk.0.ffn_down.weight", np.zeros((E, 1), np.float32)),
    ]
    head = struct.pack("<IIQQ", 0x46554747, 3, len(tensors), len(kvs)) + b"".join(kvs)
    infos, off = b"", 0
    for name, arr in tensors:
        dims = list(reversed(arr.shape))
        infos += _s(name) + struct.pack("<I", len(dims)) + b"".join(struct.pack("<Q", d) for d in dims)
        infos += struct.pack("<IQ", 0, off)
        off += (arr.nbytes + 31) // 32 * 32
    pre = head + infos
    pad = (-len(pre)) % 32
    with open(path, "wb") as f:
        f.write(pre + b"\0" * pad)
        for _, arr in tensors:
            b = np.ascontiguousarray(arr, np.float32).tobytes()
            f.write(b + b"\0" * ((-len(b)) % 32))


def main() -> None:
    ref_bin = os.path.join(ROOT, "oracle", "_ref", "ref_attn")
    if not os.path.exists(ref_bin):
        sys.exit("build the reference first: make -C oracle ref")
    kinds = sys.argv[1:] or list(KINDS)
    for kind in kinds:
        layer, is_swa, has_rope = KINDS[kind]
        with tempfile.TemporaryDirectory() as tmp:
            gg, out = os.path.join(tmp, "m.gguf"), os.path.join(tmp, "att.bin")
            write_gguf(gg, layer, is_swa, has_rope)
            subprocess.run([ref_bin, gg, str(N_TOK), out, str(os.cpu_count() or 8)], check=True)
            att = np.fromfile(out, np.float32).reshape(N_TOK, 32, 128)
        # the oracle on the same inputs, for the record printed below (the test suite repeats this check)
        qn, kn, sinks = fo.layer_weights(SEED, layer)
        mine, _, _ = fo.layer_forward(effective_qkv(layer), qn, kn, sinks, is_swa, has_rope, n_threads=8)
        diff = np.abs(mine.reshape(att.shape) - att)
        print(f"{kind}: reference vs oracle restatement: max|diff| = {diff.max():.3e}, "
              f"bit-identical outputs = {np.mean(mine.reshape(att.shape) == att):.6f}")
        np.savez_compressed(
            os.path.join(ROOT, "tests", "golden", f"ref_attn_{kind}.npz"),
            probe_pos=np.array(PROBE_POS, np.int32), probe_att=att[PROBE_POS],
            row_sum=att.reshape(N_TOK, -1).astype(np.float64).sum(1),
            row_abs=np.abs(att.reshape(N_TOK, -1).astype(np.float64)).sum(1),
            seed=SEED, layer=layer, is_swa=is_swa, has_rope=has_rope, n_tok=N_TOK)


if __name__ == "__main__":
    main()
