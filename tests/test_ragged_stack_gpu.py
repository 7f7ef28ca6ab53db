"""A small version of the ragged serving mix: one decode step over a 4-layer stack (3 sliding-window ring layers +
1 full layer) for sequences of very different lengths, some of them rolled back first -- by up to 511 tokens (nothing
to redo) and by more (the rings are rewritten by a 512-token prefill, server/src/main.rs:96-100)."""
import numpy as np
import pytest

from helpers import bf16_round_rows, synth_cache_f16, to_slot_layout

pytestmark = pytest.mark.gpu
IS_SWA = [True, True, True, False]
HAS_ROPE = [True, True, True, False]  # the reference's layers: SWA + RoPE, full + NoPE (flint_config.h:37-38)


def test_ragged_stack_with_rollback(fo):
    import flint_mac_b200 as fa

    seed, n_ctx = 17, 4096
    ctx = [1, 40, 511, 512, 513, 700, 1023, 1025, 1500, 2600, 3000, 4000]
    back = [0, 10, 0, 300, 0, 600, 511, 512, 0, 599, 0, 1]
    B = len(ctx)
    w = [fo.layer_weights(seed, il) for il in range(4)]
    with fa.Attn(IS_SWA, HAS_ROPE, B, n_ctx) as h:
        pos_major = {}  # (layer, seq) -> (k, v) half bits by position, what the caches are supposed to hold
        for il in range(4):
            h.set_layer(il, *w[il])
            n_slots = h.n_slots(il)
            for s, c in enumerate(ctx):
                k, v = synth_cache_f16(seed, il, s, c)
                h.write_kv(il, s, 0, to_slot_layout(k, n_slots, IS_SWA[il]), to_slot_layout(v, n_slots, IS_SWA[il]))
                pos_major[il, s] = (k.copy(), v.copy())
        for s, c in enumerate(ctx):
            h.set_pos(s, c)
        # ---- rollback
        new_len = list(ctx)
        for s, b in enumerate(back):
            if b == 0:
                continue
            p = ctx[s] - b
            restart = fa.rollback_restart(ctx[s], p)
            assert restart == fo.rollback_restart(ctx[s], p)
            assert h.truncate(s, restart) == 0
            if restart < p:
                T = p - restart
                for il in range(3):  # only the rings lose history; the full layer's slots [restart, p) are intact
                    rows, bits = bf16_round_rows(fo.raw_qkv(seed + 1, il, restart, T, seq=s))
                    out = np.empty((T, 4096), np.float32)
                    h.prefill(il, s, T, bits, fa.BF16, out, fa.F32)
                    k, v = pos_major[il, s]
                    for t in range(T):
                        row = fo.qk_norm_rope(rows[t], w[il][0], w[il][1], restart + t, HAS_ROPE[il])
                        k[restart + t] = fo.to_f16_bits(row[4096:4608]).reshape(4, 128)
                        v[restart + t] = fo.to_f16_bits(row[4608:]).reshape(4, 128)
                assert h.advance([s], T) == 0
            assert h.pos(s) == p
            new_len[s] = p
        # ---- one decode step over the stack, ragged batch
        seqs = list(range(B))
        for il in range(4):
            rows, bits = bf16_round_rows(np.stack([fo.raw_qkv(seed + 2, il, new_len[s], 1, seq=s)[0] for s in seqs]))
            out = np.empty((B, 4096), np.float32)
            h.decode(il, seqs, bits, fa.BF16, out, fa.F32)
            n_slots = h.n_slots(il)
            for s in seqs:
                k, v = pos_major[il, s]
                p = new_len[s]
                ks = to_slot_layout(k[:p], n_slots, IS_SWA[il])
                vs = to_slot_layout(v[:p], n_slots, IS_SWA[il])
                want = fo.decode_token_f16cache(rows[s], p, *w[il], IS_SWA[il], HAS_ROPE[il], ks, vs, n_threads=8)
                err = np.abs(out[s] - want)
                assert err.max() <= 2e-3 and err.mean() <= 2e-4, (il, s, p, float(err.max()))
        assert h.advance(seqs, 1) == 0
        assert [h.pos(s) for s in seqs] == [n + 1 for n in new_len]
