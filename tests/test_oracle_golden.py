"""The CPU oracle against the golden vectors produced by the unmodified reference RefModel
(tests/golden/make_golden.py ran src/ref/ref_model.cpp on a synthetic GGUF), and against itself."""
import os

import numpy as np
import pytest

GOLD = os.path.join(os.path.dirname(__file__), "golden")
KINDS = ["swa_rope", "full_nope", "full_rope"]
E = 9216


def effective_qkv(fo, seed, layer, n_tok):
    """rmsnorm over the 9216-wide synthetic embedding row, as the reference applies before projecting
    (src/ref/ref_model.cpp:108); the selection projections then hand its first 5120 values to attention."""
    x = np.zeros((n_tok, E), np.float32)
    x[:, :fo.QKV_DIM] = fo.raw_qkv(seed, layer, 0, n_tok)
    ones = np.ones(E, np.float32)
    return np.stack([fo.rmsnorm(x[t], ones)[:fo.QKV_DIM] for t in range(n_tok)])


@pytest.mark.parametrize("kind", KINDS)
def test_oracle_matches_reference_refmodel(fo, kind):
    g = np.load(os.path.join(GOLD, f"ref_attn_{kind}.npz"))
    seed, layer, n_tok = int(g["seed"]), int(g["layer"]), int(g["n_tok"])
    qn, kn, sinks = fo.layer_weights(seed, layer)
    att, _, _ = fo.layer_forward(effective_qkv(fo, seed, layer, n_tok), qn, kn, sinks, bool(g["is_swa"]),
                                 bool(g["has_rope"]), n_threads=8)
    att = att.reshape(n_tok, 32, 128)
    # Same arithmetic, same order, same compiler flags: the restatement reproduces the reference bit for bit.
    assert np.array_equal(att[g["probe_pos"]], g["probe_att"])
    assert np.array_equal(att.reshape(n_tok, -1).astype(np.float64).sum(1), g["row_sum"])
    assert np.array_equal(np.abs(att.reshape(n_tok, -1).astype(np.float64)).sum(1), g["row_abs"])


def test_threads_do_not_change_results(fo):
    qn, kn, sinks = fo.layer_weights(3, 0)
    qkv = fo.raw_qkv(3, 0, 0, 40)
    a1, _, _ = fo.layer_forward(qkv, qn, kn, sinks, True, True, n_threads=1)
    a8, _, _ = fo.layer_forward(qkv, qn, kn, sinks, True, True, n_threads=8)
    assert np.array_equal(a1, a8)


def test_generator_is_counter_based(fo):
    a = fo.gen_normal(5, 9, 1000)
    b = fo.gen_normal(5, 9, 300, first=500)
    assert np.array_equal(a[500:800], b)
    assert abs(float(a.mean())) < 0.15 and 0.85 < float(a.std()) < 1.15
    assert not np.array_equal(a, fo.gen_normal(6, 9, 1000))


def test_partial_and_combine_match_full(fo):
    """Split-K records merged with the combine formula (src/metal/fused.metal:332-350) equal unsplit attention."""
    seed, T = 11, 700
    qn, kn, sinks = fo.layer_weights(seed, 0)
    qkv = fo.raw_qkv(seed, 0, 0, T)
    att, kc, vc = fo.layer_forward(qkv, qn, kn, sinks, False, True)
    q = fo.qk_norm_rope(qkv[T - 1], qn, kn, T - 1, True)[:fo.Q_DIM]
    for bounds in ([0, T], [0, 256, 512, T], [0, 1, 699, T], [0, 0, T]):
        parts = np.stack([fo.attend_partial(q, kc, vc, a, b) for a, b in zip(bounds[:-1], bounds[1:])], axis=1)
        out = fo.combine(parts, sinks)
        assert np.abs(out.reshape(-1) - att[T - 1]).max() < 2e-6


def test_f16cache_decode_matches_rounded_layer_forward(fo):
    seed, T = 12, 1100
    for is_swa in (True, False):
        qn, kn, sinks = fo.layer_weights(seed, 1)
        qkv = fo.raw_qkv(seed, 1, 0, T)
        att, _, _ = fo.layer_forward(qkv, qn, kn, sinks, is_swa, True, round_kv_f16=True)
        n_slots = 1024 if is_swa else T
        k16 = np.zeros((4, n_slots, 128), np.uint16)
        v16 = np.zeros((4, n_slots, 128), np.uint16)
        for p in range(T):
            a = fo.decode_token_f16cache(qkv[p], p, qn, kn, sinks, is_swa, True, k16, v16)
            assert np.array_equal(a, att[p]), p


@pytest.mark.parametrize("kind", ["full_nope", "swa_rope"])
def test_second_cpu_statement_agrees_with_the_first(fo, kind):
    """The reference states this path twice on the CPU: src/ref (fp32 scores, double accumulators, un-rounded cache)
    and its attention unit test (src/main.mm:253-305: all double, K/V rounded through half).  On the unit test's own
    workload -- 1300 tokens of grid-uniform rows, its probe positions and heads, a full/NoPE and a SWA/RoPE layer --
    the restatements of both agree to fp32 rounding once the first one rounds K/V through half as well, and to the
    size of that rounding when it does not."""
    is_swa, has_rope = {"full_nope": (False, False), "swa_rope": (True, True)}[kind]
    seed, T = 11, 1300
    qn, kn, sinks = fo.layer_weights(seed, 0 if kind == "full_nope" else 2)
    qkv = fo.grid_qkv(seed, T)
    assert qkv.min() >= -2 and qkv.max() <= 2 and len(np.unique(qkv)) == 2001
    second = fo.attend_double_f16(qkv, qn, kn, sinks, is_swa, has_rope)
    pos, heads = list(fo.PROBE_POS), list(fo.PROBE_HEADS)
    rounded, _, _ = fo.layer_forward(qkv, qn, kn, sinks, is_swa, has_rope, round_kv_f16=True, n_threads=8)
    plain, _, _ = fo.layer_forward(qkv, qn, kn, sinks, is_swa, has_rope, round_kv_f16=False, n_threads=8)
    rounded = rounded.reshape(T, 32, 128)[pos][:, heads]
    plain = plain.reshape(T, 32, 128)[pos][:, heads]
    # fp32 norm/RoPE can move a K element across a half rounding boundary: a handful of one-ulp differences in K
    assert np.abs(rounded - second).max() < 1e-4
    rms = np.sqrt((second ** 2).mean())
    assert np.abs(plain - second).max() / rms < 2e-2  # the bar of the reference's test (src/main.mm:309)
    assert np.abs(plain - second).max() < 2e-3


def test_stack_restatement_matches_reference_refmodel(fo):
    """The attention stack with real projections (rmsnorm -> q/k/v matvecs -> attention -> o-proj -> residual, then
    output norm and vocabulary matvec): the restatement reproduces, bit for bit, the logits and residual stream the
    unmodified RefModel produced on the same weights and tokens (tests/golden/make_golden_stack.py)."""
    g = np.load(os.path.join(GOLD, "ref_stack.npz"))
    kinds = list(zip(g["is_swa"].tolist(), g["has_rope"].tolist()))
    w = fo.stack_weights(int(g["seed"]), int(g["n_layer"]), int(g["n_embd"]), int(g["n_vocab"]), kinds)
    logits, hidden = fo.stack_forward(w, g["tokens"])
    assert np.array_equal(logits[g["probe_pos"]], g["probe_logits"])
    assert np.array_equal(logits.argmax(1), g["argmax"])
    assert np.array_equal(logits.astype(np.float64).sum(1), g["logit_sum"])
    assert np.array_equal(hidden.astype(np.float64).sum(1), g["hidden_sum"])
