"""Prefill attention on the GPU (norm/RoPE/cache-write prologue + tcgen05 flash attention), through the C ABI,
against the CPU oracle and the reference's golden vectors."""
import os

import numpy as np
import pytest

from helpers import KINDS, assert_close, bf16_round_rows, oracle_at_positions

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(__file__), "golden")
PROBES = [0, 1, 31, 32, 200, 511, 512, 513, 600, 1023, 1024, 1100, 1299]  # src/main.mm:280


@pytest.fixture(scope="module")
def fa():
    import flint_mac_b200 as fa

    fa.load_library()
    return fa


def _open(fa, kind, n_ctx, max_seqs=1):
    return fa.Attn([KINDS[kind][0]], [KINDS[kind][1]], max_seqs, n_ctx)


def _prefill_chunks(fa, h, qkv, chunk, dtype=None):
    T = qkv.shape[0]
    out = np.empty((T, 4096), np.float32)
    for c0 in range(0, T, chunk):
        n = min(chunk, T - c0)
        o = np.empty((n, 4096), np.float32)
        h.prefill(0, 0, n, np.ascontiguousarray(qkv[c0:c0 + n]), fa.F32, o, fa.F32)
        h.advance([0], n)
        out[c0:c0 + n] = o
    return out


@pytest.mark.parametrize("kind", list(KINDS))
@pytest.mark.parametrize("T", [1, 15, 16, 17, 40, 130])
def test_small_prompts_every_position(fa, fo, kind, T):
    is_swa, has_rope = KINDS[kind]
    w = fo.layer_weights(4, 0)
    qkv = fo.raw_qkv(4, 0, 0, T)
    want, _, _ = fo.layer_forward(qkv, *w, is_swa, has_rope)
    with _open(fa, kind, 256) as h:
        h.set_layer(0, *w)
        got = _prefill_chunks(fa, h, qkv, T)
    assert_close(got, want, f"{kind} T={T}")


@pytest.mark.parametrize("kind", ["full_nope", "swa_rope", "full_rope"])
@pytest.mark.parametrize("chunk", [512, 1300])
def test_attn_1300_tokens_like_the_reference_test(fa, fo, kind, chunk):
    """The reference's test-attn (src/main.mm:240-314): 1300 tokens in chunks of 512 (512/512/276), a full/NoPE and a
    SWA/RoPE layer, probes at query-block, window and ring-wrap edges -- and the same prompt in a single launch."""
    is_swa, has_rope = KINDS[kind]
    seed, T = 0, 1300
    w = fo.layer_weights(seed, 2)
    qkv = fo.raw_qkv(seed, 2, 0, T)
    with _open(fa, kind, 2048) as h:
        h.set_layer(0, *w)
        got = _prefill_chunks(fa, h, qkv, chunk)
        want, kc, vc = fo.layer_forward(qkv, *w, is_swa, has_rope, n_threads=8)
        assert_close(got, want, f"{kind} chunk={chunk} all positions")
        assert_close(got[PROBES], want[PROBES], f"{kind} chunk={chunk} probes")
        # the reference's own pass bar: max_err / rms < 2e-2 (src/main.mm:308)
        rms = np.sqrt((want[PROBES].astype(np.float64) ** 2).mean())
        assert np.abs(got[PROBES] - want[PROBES]).max() / rms < 2e-2
        # cache / ring contents after the prompt: V bit-exact in the slot its position owns
        n_slots = h.n_slots(0)
        k_dev, v_dev = h.read_kv(0, 0, 0, n_slots)
        owners = fo.ring_owners(T) if is_swa else np.arange(T)
        for s in range(len(owners)):
            p = int(owners[s])
            if p < 0:
                continue
            assert np.array_equal(v_dev[:, s].reshape(-1), fo.to_f16_bits(vc[p])), (s, p)
            assert np.abs(fo.from_f16_bits(k_dev[:, s].reshape(-1)) - kc[p]).max() <= np.abs(kc[p]).max() * 2 ** -9


@pytest.mark.parametrize("kind", ["full_nope", "swa_rope"])
def test_attn_against_the_all_double_statement(fa, fo, kind):
    """The reference's test-attn as it is written (src/main.mm:240-314): grid-uniform rows, 1300 tokens prefilled in
    chunks of 512, compared at its probe positions and heads with its all-double CPU statement (K/V rounded through
    half), under its own bar max_err / rms < 2e-2 and under the tolerance of this repo -- and the same through the
    decode path, one token at a time."""
    is_swa, has_rope = KINDS[kind]
    seed, T = 11, 1300
    w = fo.layer_weights(seed, 0 if kind == "full_nope" else 2)
    qkv = fo.grid_qkv(seed, T)
    want = fo.attend_double_f16(qkv, *w, is_swa, has_rope)
    pos, heads = list(fo.PROBE_POS), list(fo.PROBE_HEADS)
    rms = np.sqrt((want ** 2).mean())
    with _open(fa, kind, 2048) as h:
        h.set_layer(0, *w)
        got = _prefill_chunks(fa, h, qkv, 512).reshape(T, 32, 128)[pos][:, heads]
    assert np.abs(got - want).max() / rms < 2e-2
    assert_close(got, want, f"{kind} prefill vs the all-double statement")
    with _open(fa, kind, 2048) as h:
        h.set_layer(0, *w)
        row = np.empty(4096, np.float32)
        dec = np.empty((T, 4096), np.float32)
        for t in range(T):
            h.decode(0, [0], np.ascontiguousarray(qkv[t]), fa.F32, row, fa.F32)
            h.advance([0])
            dec[t] = row
    dec = dec.reshape(T, 32, 128)[pos][:, heads]
    assert np.abs(dec - want).max() / rms < 2e-2
    assert_close(dec, want, f"{kind} decode vs the all-double statement")


@pytest.mark.parametrize("kind", list(KINDS))
def test_golden_vectors_of_the_reference(fa, fo, kind):
    g = np.load(os.path.join(GOLD, f"ref_attn_{kind}.npz"))
    seed, layer, T = int(g["seed"]), int(g["layer"]), int(g["n_tok"])
    x = np.zeros((T, 9216), np.float32)
    x[:, :5120] = fo.raw_qkv(seed, layer, 0, T)
    ones = np.ones(9216, np.float32)
    qkv = np.stack([fo.rmsnorm(x[t], ones)[:5120] for t in range(T)])
    with _open(fa, kind, 1300) as h:
        h.set_layer(0, *fo.layer_weights(seed, layer))
        got = _prefill_chunks(fa, h, qkv, 512).reshape(T, 32, 128)
    assert_close(got[g["probe_pos"]], g["probe_att"], f"{kind} golden probes")
    assert np.abs(got.reshape(T, -1).astype(np.float64).sum(1) - g["row_sum"]).max() < 4096 * 2e-4


def test_config3_4000_token_prompt_swa_bf16(fa, fo):
    """One 4000-token prompt on a SWA layer, bf16 q/k/v, window 512 + sink, K/V into the 1024-slot ring; output
    checked on the last 256 positions, ring contents on all 1024 slots."""
    seed, T = 3, 4000
    w = fo.layer_weights(seed, 0)
    qkv, bits = bf16_round_rows(fo.raw_qkv(seed, 0, 0, T))
    with _open(fa, "swa_rope", 4096) as h:
        h.set_layer(0, *w)
        out = np.empty((T, 4096), np.float32)
        h.prefill(0, 0, T, bits, fa.BF16, out, fa.F32)
        assert np.isfinite(out).all()
        last = list(range(T - 256, T))
        want, kc, vc = oracle_at_positions(qkv, w, True, True, last)
        assert_close(out[last], want, "config 3, last 256 positions")
        k_dev, v_dev = h.read_kv(0, 0, 0, 1024)
        owners = fo.ring_owners(T)
        assert owners.min() == T - 1024
        for s in range(1024):
            p = int(owners[s])
            assert np.array_equal(v_dev[:, s].reshape(-1), fo.to_f16_bits(vc[p])), (s, p)
        # a few earlier positions too (window edges of the first blocks)
        some = [0, 15, 16, 511, 512, 513, 1023, 1024, 2047, 2048]
        want2, _, _ = oracle_at_positions(qkv, w, True, True, some)
        assert_close(out[some], want2, "config 3, early positions")


def test_long_prompt_on_a_full_layer_in_two_chunks(fa, fo):
    """A 6000-token prompt on a full-attention layer (every key back to position 0), given as a 4000-token chunk and a
    2000-token chunk that attends over the first chunk's cache; sampled positions against the oracle, cache rows
    bit for bit through V."""
    seed, T, cut = 5, 6000, 4000
    w = fo.layer_weights(seed, 0)
    qkv, bits = bf16_round_rows(fo.raw_qkv(seed, 0, 0, T))
    with _open(fa, "full_rope", T + 8) as h:
        h.set_layer(0, *w)
        out = np.empty((T, 4096), np.float32)
        h.prefill(0, 0, cut, bits[:cut], fa.BF16, out[:cut], fa.F32)
        assert h.advance([0], cut) == 0
        h.prefill(0, 0, T - cut, np.ascontiguousarray(bits[cut:]), fa.BF16, out[cut:], fa.F32)
        assert np.isfinite(out).all()
        some = [0, 1, 127, 128, 2047, 3999, 4000, 4001, 4127, 5000, 5998, 5999]
        want, kc, vc = oracle_at_positions(qkv, w, False, True, some)
        assert_close(out[some], want, "full layer, long prompt")
        k_dev, v_dev = h.read_kv(0, 0, 0, T)
        for p in (0, 3999, 4000, 5999):
            assert np.array_equal(v_dev[:, p].reshape(-1), fo.to_f16_bits(vc[p])), p


def test_short_chunks_on_a_long_full_layer_history_split_their_key_range(fa, fo):
    """The reference's own call pattern (chunks of at most 512 tokens, src/engine.mm:1080) on a full-attention layer
    with a long history: such a launch has fewer work units than SMs, so the key range of every unit is split and
    merged by log-sum-exp.  A 512-token chunk (2 ranges), a 100-token ragged chunk (8 ranges) and a 7-token chunk
    after 4000 tokens of history; every output row of the short chunks against the oracle, fp32 and bf16 rows out."""
    import torch

    seed, hist = 8, 4000
    chunks = [512, 100, 7]
    T = hist + sum(chunks)
    w = fo.layer_weights(seed, 0)
    qkv, bits = bf16_round_rows(fo.raw_qkv(seed, 0, 0, T))
    with _open(fa, "full_rope", T + 8) as h:
        h.set_layer(0, *w)
        out = np.zeros((T, 4096), np.float32)
        h.prefill(0, 0, hist, bits[:hist], fa.BF16, out[:hist], fa.F32)
        assert h.advance([0], hist) == 0
        p = hist
        out16 = np.zeros((chunks[0], 4096), np.uint16)
        for i, n in enumerate(chunks):
            rows = np.ascontiguousarray(bits[p:p + n])
            if i == 0:  # the same chunk once more with bf16 rows out (the position has not moved yet)
                h.prefill(0, 0, n, rows, fa.BF16, out16, fa.BF16)
            h.prefill(0, 0, n, rows, fa.BF16, out[p:p + n], fa.F32)
            assert h.advance([0], n) == 0
            p += n
        assert np.isfinite(out).all()
        some = list(range(hist, hist + 40)) + list(range(hist + 480, T))
        want, _, _ = oracle_at_positions(qkv, w, False, True, some)
        assert_close(out[some], want, "split key range vs oracle")
        got16 = fo.from_bf16_bits(out16)
        assert np.abs(got16 - out[hist:hist + chunks[0]]).max() <= np.abs(out).max() * 2 ** -8


def test_short_chunks_on_a_sliding_window_history(fa, fo):
    """The reference's call pattern (chunks of at most 512 tokens) on a sliding-window layer: a 512-token chunk behind
    a cached prefix (64 work units whose 544-key bands start in the ring's history), then a 300-token and a 37-token
    chunk.  Rows of every chunk against the oracle, and the ring afterwards bit for bit through V."""
    seed, hist = 9, 1500
    chunks = [512, 300, 37]
    T = hist + sum(chunks)
    w = fo.layer_weights(seed, 0)
    qkv, bits = bf16_round_rows(fo.raw_qkv(seed, 0, 0, T))
    with _open(fa, "swa_rope", T + 8) as h:
        h.set_layer(0, *w)
        out = np.zeros((T, 4096), np.float32)
        h.prefill(0, 0, hist, bits[:hist], fa.BF16, out[:hist], fa.F32)
        assert h.advance([0], hist) == 0
        p = hist
        for n in chunks:
            h.prefill(0, 0, n, np.ascontiguousarray(bits[p:p + n]), fa.BF16, out[p:p + n], fa.F32)
            assert h.advance([0], n) == 0
            p += n
        assert np.isfinite(out).all()
        some = list(range(hist, hist + 40)) + list(range(hist + 490, hist + 530)) + list(range(T - 60, T))
        want, _, vc = oracle_at_positions(qkv, w, True, True, some)
        assert_close(out[some], want, "sliding-window chunks vs oracle")
        k_dev, v_dev = h.read_kv(0, 0, 0, 1024)
        for pos in (T - 1, T - 513, T - 1000):
            assert np.array_equal(v_dev[:, pos % 1024].reshape(-1), fo.to_f16_bits(vc[pos])), pos


@pytest.mark.parametrize("kind", ["swa_rope", "full_rope"])
def test_prefill_then_decode_equals_decode_only(fa, fo, kind):
    """The reference's check-prefill idea (src/main.mm:317-346) at the kernel level: prefill the first part, decode the
    rest token by token; both paths must agree with the oracle, and so with each other."""
    is_swa, has_rope = KINDS[kind]
    seed, T, split = 6, 1200, 700
    w = fo.layer_weights(seed, 0)
    qkv = fo.raw_qkv(seed, 0, 0, T)
    want, _, _ = fo.layer_forward(qkv, *w, is_swa, has_rope, n_threads=8)
    with _open(fa, kind, 2048) as h:
        h.set_layer(0, *w)
        got = np.empty((T, 4096), np.float32)
        got[:split] = _prefill_chunks(fa, h, qkv[:split], 512)
        assert h.pos(0) == split
        row = np.empty(4096, np.float32)
        for t in range(split, T):
            h.decode(0, [0], np.ascontiguousarray(qkv[t]), fa.F32, row, fa.F32)
            h.advance([0])
            got[t] = row
        # then prefill again on top of decoded history (window crosses prefill- and decode-written ring slots)
        extra = fo.raw_qkv(seed, 0, T, 100)
        o2 = np.empty((100, 4096), np.float32)
        h.prefill(0, 0, 100, extra, fa.F32, o2, fa.F32)
    assert_close(got, want, f"{kind} prefill+decode")
    want2, _, _ = fo.layer_forward(np.concatenate([qkv, extra]), *w, is_swa, has_rope, n_threads=8)
    assert_close(o2, want2[T:], f"{kind} prefill on decoded history")


def test_rollback_and_recompute(fa, fo):
    """truncate + the server's rule (server/src/main.rs:96-100): rolling back up to 511 tokens needs nothing; more
    needs a re-prefill from p-512, after which outputs from p on are those of an uninterrupted run."""
    seed, T = 8, 1900
    w = fo.layer_weights(seed, 0)
    qkv = fo.raw_qkv(seed, 0, 0, T)
    want, _, _ = fo.layer_forward(qkv, *w, True, True, n_threads=8)
    for back in (300, 511, 512, 600):
        with _open(fa, "swa_rope", 2048) as h:
            h.set_layer(0, *w)
            _prefill_chunks(fa, h, qkv, 512)
            p = T - back
            restart = fa.rollback_restart(T, p)
            assert restart == (p if back <= 511 else p - 512)
            assert h.truncate(0, restart) == 0 and h.pos(0) == restart
            redo = np.empty((T - restart, 4096), np.float32)
            h.prefill(0, 0, T - restart, np.ascontiguousarray(qkv[restart:]), fa.F32, redo, fa.F32)
            assert_close(redo[p - restart:], want[p:], f"rollback by {back}")


@pytest.mark.parametrize("n_ctx,chunks", [(1008, [700, 300]), (4108, [512, 1500, 37, 2000])])
def test_context_parallel_prefill_of_a_kv_sharded_full_layer(fa, fo, n_ctx, chunks):
    """A full layer whose key range is cut over two ranks (two handles on this GPU): every rank gets the same rows,
    stores the K/V of its own positions, attends all queries to the keys it holds and returns an un-normalised partial
    with (m, l) per row; the merged result equals the reference arithmetic, chunk after chunk (the second rank has no
    key at all for early chunks, a few for the chunk that crosses the boundary), and a decode step through the
    sharded decode path on the caches the prefill built agrees too."""
    import torch

    seed, T = 61, sum(chunks)
    w = fo.layer_weights(seed, 1)
    qkv = fo.raw_qkv(seed, 1, 0, T + 1)
    want, kc, vc = fo.layer_forward(qkv, *w, False, True, n_threads=8)
    handles = [fa.Attn([False], [True], 1, n_ctx, kv_rank=r, kv_ranks=2) for r in range(2)]
    try:
        for h in handles:
            h.set_layer(0, *w)
        with pytest.raises(fa.FlintAttnError, match="prefill_partial"):
            handles[0].prefill(0, 0, 8, np.ascontiguousarray(qkv[:8]), fa.F32, np.empty((8, 4096), np.float32), fa.F32)
        p0 = 0
        for n in chunks:
            rows = torch.from_numpy(np.ascontiguousarray(qkv[p0:p0 + n])).cuda()
            po = torch.full((2, n, 4096), float("nan"), device="cuda")
            pml = torch.full((2, n, 32, 2), float("nan"), device="cuda")
            for r, h in enumerate(handles):
                h.prefill_partial_dev(0, 0, n, rows, fa.F32, po[r], pml[r])
            out = torch.empty(n, 4096, device="cuda")
            handles[1].prefill_combine_dev(n, 2, po, pml, out, fa.F32)
            torch.cuda.synchronize()
            for h in handles:
                h.check()
                h.advance([0], n)
            assert_close(out.cpu().numpy(), want[p0:p0 + n], f"chunk at {p0} (+{n})")
            shard = handles[0].n_slots(0)
            if p0 + n <= shard:  # nothing of this chunk lies in the second rank's range: its partial is empty
                assert float(pml[1, :, :, 1].abs().max()) == 0.0
            p0 += n
        # the caches the sharded prefill left behind: V bit-exact in the slot of its position, on the rank that owns it
        shard = handles[0].n_slots(0)
        for r, h in enumerate(handles):
            lo, hi = r * shard, min(T, (r + 1) * shard)
            if hi > lo:
                _, v_dev = h.read_kv(0, 0, 0, hi - lo)
                assert np.array_equal(v_dev.transpose(1, 0, 2).reshape(hi - lo, 512), fo.to_f16_bits(vc[lo:hi]))
        # one decode step on top, through the sharded decode path
        row = torch.from_numpy(np.ascontiguousarray(qkv[T:T + 1])).cuda()
        parts = torch.zeros(2, 1, 32, 130, device="cuda")
        for r, h in enumerate(handles):
            h.decode_partial_dev(0, [0], row, fa.F32, parts[r])
        dec = torch.empty(1, 4096, device="cuda")
        handles[0].combine_dev(0, 1, 2, parts, dec, fa.F32)
        torch.cuda.synchronize()
        assert_close(dec.cpu().numpy()[0], want[T], "decode after the sharded prefill")
    finally:
        for h in handles:
            h.close()
