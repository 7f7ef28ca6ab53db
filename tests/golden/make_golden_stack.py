"""Golden logits of a small attention stack from the UNMODIFIED reference CPU model.

    make -C oracle ref
    python tests/golden/make_golden_stack.py

Writes a synthetic all-F32 GGUF of a 3-layer model (full/NoPE, sliding-window/RoPE, full/RoPE; n_embd 512, vocabulary
1024) whose attention projections are real matrices (seeded, rounded to bf16 so that a bf16 GPU copy holds the very
same numbers) and whose feed-forward weights are zero, runs the reference's RefModel::forward
(src/ref/ref_model.cpp:95-197) over 700 seeded token ids through `oracle/_ref/ref_attn --stack`, and stores in
tests/golden/ref_stack.npz:

  tokens        int32 [700]
  probe_pos     positions whose full logit rows are kept (query-block edges, the 513-key window edge)
  probe_logits  float32 [n_probe][1024]
  argmax        int32 [700] greedy next token after every position
  logit_sum     float64 [700] sum of the 1024 logits of every position
  hidden_sum    float64 [700] sum of the residual stream after the last layer
  seed, n_layer, n_embd, n_vocab, is_swa, has_rope

Weights are not stored: tests regenerate them with oracle.stack_weights(seed, ...).
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
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from make_golden import ARR, BOOL, F32, STR, U32, _kv, _s  # noqa: E402
from oracle import oracle as fo  # noqa: E402

SEED, N_LAYER, E, N_VOCAB, N_TOK = 5, 3, 512, 1024, 700
KINDS = [(False, False), (True, True), (False, True)]  # (is_swa, has_rope) per layer
PROBE_POS = [0, 1, 31, 32, 200, 511, 512, 513, 600, 699]


def tokens() -> np.ndarray:
    return np.array([fo.gen_u64(SEED, 99, i) % N_VOCAB for i in range(N_TOK)], np.int32)


def write_gguf(path: str, w: dict) -> None:
    a = "flint"
    kvs = [
        _kv("general.architecture", STR, a),
        _kv(a + ".block_count", U32, N_LAYER), _kv(a + ".embedding_length", U32, E),
        _kv(a + ".attention.head_count", U32, 32), _kv(a + ".attention.head_count_kv", U32, 4),
        _kv(a + ".attention.key_length", U32, 128), _kv(a + ".feed_forward_length", U32, 1),
        _kv(a + ".expert_feed_forward_length", U32, 1), _kv(a + ".expert_shared_feed_forward_length", U32, 1),
        _kv(a + ".expert_count", U32, 1), _kv(a + ".expert_used_count", U32, 1),
        _kv(a + ".leading_dense_block_count", U32, N_LAYER), _kv(a + ".attention.sliding_window", U32, 513),
        _kv(a + ".attention.layer_norm_rms_epsilon", F32, 1e-6), _kv(a + ".rope.freq_base", F32, 10000.0),
        _kv(a + ".attention.sliding_window_pattern", ARR, [k[0] for k in KINDS]),
        _kv(a + ".attention.rope_pattern", ARR, [k[1] for k in KINDS]),
        _kv(a + ".expert_gating_func", U32, 2), _kv(a + ".expert_weights_norm", BOOL, True),
        _kv(a + ".expert_weights_scale", F32, 1.0),
    ]
    ones = np.ones(E, np.float32)
    tensors = [("token_embd.weight", w["embd"]), ("output_norm.weight", w["out_norm"]), ("output.weight", w["w_out"])]
    for il in range(N_LAYER):
        b = f"blk.{il}."
        tensors += [
            (b + "attn_norm.weight", w["attn_norm"][il]), (b + "attn_q.weight", w["wq"][il]),
            (b + "attn_k.weight", w["wk"][il]), (b + "attn_v.weight", w["wv"][il]),
            (b + "attn_q_norm.weight", w["q_norm"][il]), (b + "attn_k_norm.weight", w["k_norm"][il]),
            (b + "attn_sinks.weight", w["sinks"][il]), (b + "attn_output.weight", w["wo"][il]),
            (b + "ffn_norm.weight", ones), (b + "ffn_gate.weight", np.zeros((1, E), np.float32)),
            (b + "ffn_up.weight", np.zeros((1, E), np.float32)), (b + "ffn_down.weight", np.zeros((E, 1), np.float32)),
        ]
    head = struct.pack("<IIQQ", 0x46554747, 3, len(tensors), len(kvs)) + b"".join(kvs)
    infos, off = b"", 0
    for name, arr in tensors:
        dims = list(reversed(arr.shape))
        infos += _s(name) + struct.pack("<I", len(dims)) + b"".join(struct.pack("<Q", d) for d in dims)
        infos += struct.pack("<IQ", 0, off)
        off += (arr.nbytes + 31) // 32 * 32
    pre = head + infos
    with open(path, "wb") as f:
        f.write(pre + b"\0" * ((-len(pre)) % 32))
        for _, arr in tensors:
            b = np.ascontiguousarray(arr, np.float32).tobytes()
            f.write(b + b"\0" * ((-len(b)) % 32))


def main() -> None:
    ref_bin = os.path.join(ROOT, "oracle", "_ref", "ref_attn")
    if not os.path.exists(ref_bin):
        sys.exit("build the reference first: make -C oracle ref")
    w = fo.stack_weights(SEED, N_LAYER, E, N_VOCAB, KINDS)
    toks = tokens()
    with tempfile.TemporaryDirectory() as tmp:
        gg = os.path.join(tmp, "m.gguf")
        tk, lo, hi = (os.path.join(tmp, n) for n in ("tok.i32", "logits.bin", "hidden.bin"))
        write_gguf(gg, w)
        toks.tofile(tk)
        subprocess.run([ref_bin, "--stack", gg, tk, lo, hi, str(os.cpu_count() or 8)], check=True)
        logits = np.fromfile(lo, np.float32).reshape(N_TOK, N_VOCAB)
        hidden = np.fromfile(hi, np.float32).reshape(N_TOK, E)
    mine_l, mine_h = fo.stack_forward(w, toks)
    print(f"reference vs oracle restatement: logits max|diff| = {np.abs(mine_l - logits).max():.3e} "
          f"(bit-identical {np.mean(mine_l == logits):.6f}), hidden max|diff| = {np.abs(mine_h - hidden).max():.3e} "
          f"(bit-identical {np.mean(mine_h == hidden):.6f})")
    np.savez_compressed(
        os.path.join(ROOT, "tests", "golden", "ref_stack.npz"), tokens=toks, probe_pos=np.array(PROBE_POS, np.int32),
        probe_logits=logits[PROBE_POS], argmax=logits.argmax(1).astype(np.int32),
        logit_sum=logits.astype(np.float64).sum(1), hidden_sum=hidden.astype(np.float64).sum(1), seed=SEED,
        n_layer=N_LAYER, n_embd=E, n_vocab=N_VOCAB, is_swa=np.array([k[0] for k in KINDS]),
        has_rope=np.array([k[1] for k in KINDS]))


if __name__ == "__main__":
    main()
