"""Paged KV cache and continuous batching: results must not depend on where K/V rows live or on who shared the batch.

A full-attention layer of a paged handle keeps its K/V in a pool of 64-key pages handed out through a block table;
the reference is the same run on a handle with contiguous per-sequence caches (and the CPU oracle for one case).
"""
import numpy as np
import pytest

from helpers import assert_close, bf16_round_rows

IS_SWA = [True, False, True, False]
HAS_ROPE = [True, False, True, True]


@pytest.fixture(scope="module")
def fa():
    import flint_mac_b200 as fa

    fa.load_library()
    return fa


def test_batcher_bookkeeping():
    """CPU: slots and page reservations of the continuous-batching loop, no GPU involved."""
    from flint_mac_b200.sched import ContinuousBatcher, Router, pages_for

    b = ContinuousBatcher(max_seqs=2, kv_pages=10, n_ctx=512)
    with pytest.raises(ValueError):
        b.submit(0, 600, 1)
    for rid, (p, n) in enumerate([(100, 28), (200, 56), (64, 1), (300, 20)]):  # 2, 4, 2, 5 pages
        b.submit(rid, p, n)
    admitted, retired, steps = [], [], 0
    while not b.idle:
        plan = b.next_step()
        assert len(b.running) <= 2 and b.pages_reserved <= 10
        assert all(r not in plan.decode for r in plan.admit)
        admitted += [r.req_id for r in plan.admit]
        retired += [r.req_id for r in b.complete(plan)]
        steps += 1
        assert steps < 400
    assert admitted == [0, 1, 2, 3]            # first come, first served
    assert sorted(retired) == [0, 1, 2, 3] and retired[0] == 0 and retired.index(2) < retired.index(1)
    assert b.pages_reserved == 0 and sorted(b.free_slots) == [0, 1]
    assert pages_for(1) == 1 and pages_for(64) == 1 and pages_for(65) == 2
    r = Router(2, n_full_layers=1, n_swa_layers=3)
    assert [r.place(i, c, 0) for i, c in enumerate([30000, 100, 200, 40000])] == [0, 1, 1, 1]
    r.retire(0)
    assert r.place(9, 10, 0) == 0


def _rows(fo, seed, layer, req, pos0, n):
    return bf16_round_rows(fo.raw_qkv(seed, layer, pos0, n, seq=req))


def _run_alone(fa, fo, w, seed, req, prompt_len, n_new):
    """One request on its own, contiguous caches: prefill the prompt, then decode token by token.  Returns
    [layer][prompt_len + n_new][4096]."""
    out = np.empty((4, prompt_len + n_new, 4096), np.float32)
    with fa.Attn(IS_SWA, HAS_ROPE, 1, prompt_len + n_new) as h:
        for il in range(4):
            h.set_layer(il, *w[il])
            _, bits = _rows(fo, seed, il, req, 0, prompt_len)
            h.prefill(il, 0, prompt_len, bits, fa.BF16, out[il, :prompt_len], fa.F32)
        h.advance([0], prompt_len)
        for t in range(n_new):
            for il in range(4):
                _, bits = _rows(fo, seed, il, req, prompt_len + t, 1)
                h.decode(il, [0], bits, fa.BF16, out[il, prompt_len + t:prompt_len + t + 1], fa.F32)
            h.advance([0])
    return out


@pytest.mark.gpu
def test_paged_equals_contiguous_and_oracle(fa, fo):
    """Prefill across page boundaries and decode on a paged handle: same outputs as contiguous caches, and the
    full-attention layer against the oracle through the paged read-back (which walks the block table)."""
    seed, P, N = 51, 700, 70  # 700 = 10 pages + 60 keys; the decode steps cross into page 12
    w = [fo.layer_weights(seed, il) for il in range(4)]
    want = _run_alone(fa, fo, w, seed, 0, P, N)
    with fa.Attn(IS_SWA, HAS_ROPE, 3, 1024, kv_pages=40) as h:
        assert h.pages_free() == 40
        for il in range(4):
            h.set_layer(il, *w[il])
        got = np.empty_like(want)
        seq = 2
        for il in range(4):
            _, bits = _rows(fo, seed, il, 0, 0, P)
            h.prefill(il, seq, P, bits, fa.BF16, got[il, :P], fa.F32)
        h.advance([seq], P)
        assert h.pages_free() == 40 - 11
        for t in range(N):
            for il in range(4):
                _, bits = _rows(fo, seed, il, 0, P + t, 1)
                h.decode(il, [seq], bits, fa.BF16, got[il, P + t:P + t + 1], fa.F32)
            h.advance([seq])
        assert h.pages_free() == 40 - 13
        assert np.abs(got - want).max() <= 2e-5
        # oracle on the paged full layer (layer 3): cache read back through the block table, position-ordered
        k16, v16 = h.read_kv(3, seq, 0, P + N)
        rows, _ = _rows(fo, seed, 3, 0, P + N - 1, 1)
        ref = fo.decode_token_f16cache(rows[0], P + N - 1, *w[3], False, True, np.ascontiguousarray(k16),
                                       np.ascontiguousarray(v16), n_threads=8)
        assert_close(got[3, P + N - 1], ref, "paged full layer vs oracle")
        # a slot that never ran reads back as zeros; releasing returns every page
        kz, _ = h.read_kv(1, 0, 0, 128)
        assert not kz.any()
        assert h.seq_release(seq) == 0 and h.pages_free() == 40 and h.pos(seq) == 0


@pytest.mark.gpu
def test_pool_exhaustion_is_an_error_that_changes_nothing(fa, fo):
    seed = 52
    w = fo.layer_weights(seed, 1)
    with fa.Attn([False], [False], 4, 4096, kv_pages=6) as h:
        h.set_layer(0, *w)
        _, bits = _rows(fo, seed, 0, 0, 0, 300)
        out = np.empty((300, 4096), np.float32)
        h.prefill(0, 0, 300, bits, fa.BF16, out, fa.F32)  # 5 pages
        h.advance([0], 300)
        with pytest.raises(fa.FlintAttnError, match="page pool exhausted"):
            h.prefill(0, 1, 300, bits, fa.BF16, out, fa.F32)
        assert h.pages_free() == 1
        row = np.empty((2, 4096), np.float32)
        _, b2 = _rows(fo, seed, 0, 1, 0, 2)
        h.set_pos(1, 0)
        h.set_pos(2, 0)
        with pytest.raises(fa.FlintAttnError, match="page pool exhausted"):
            h.decode(0, [1, 2], b2, fa.BF16, row, fa.F32)  # two new sequences need two pages, one is free
        assert h.pages_free() == 1
        h.decode(0, [1], b2[:1], fa.BF16, row[:1], fa.F32)
        assert h.pages_free() == 0
        h.seq_release(0)
        assert h.pages_free() == 5
    with pytest.raises(fa.FlintAttnError, match="cannot also be sharded"):
        fa.Attn([False], [False], 1, 256, kv_ranks=2, kv_pages=4)


@pytest.mark.gpu
def test_continuous_batching_loop(fa, fo):
    """Nine requests of very different lengths through three sequence slots and a pool that holds only a few of them
    at a time: requests join the running decode batch and leave it, pages are reused by later requests, and every
    request's outputs equal those of the same request run alone on contiguous caches."""
    from flint_mac_b200.sched import ContinuousBatcher

    seed, n_ctx = 53, 2048
    reqs = [(900, 12), (30, 40), (513, 5), (64, 64), (1, 100), (1500, 3), (200, 0), (127, 2), (1023, 9)]
    w = [fo.layer_weights(seed, il) for il in range(4)]
    alone = {rid: _run_alone(fa, fo, w, seed, rid, p, n) for rid, (p, n) in enumerate(reqs)}
    pages = 30  # 1920 keys: the two longest requests together do not fit
    b = ContinuousBatcher(max_seqs=3, kv_pages=pages, n_ctx=n_ctx)
    for rid, (p, n) in enumerate(reqs):
        b.submit(rid, p, n)
    got = {rid: np.empty_like(alone[rid]) for rid in alone}
    max_batch_seen, steps = 0, 0
    with fa.Attn(IS_SWA, HAS_ROPE, 3, n_ctx, kv_pages=pages) as h:
        for il in range(4):
            h.set_layer(il, *w[il])
        while not b.idle:
            plan = b.next_step()
            for r in plan.admit:
                for il in range(4):
                    _, bits = _rows(fo, seed, il, r.req_id, 0, r.prompt_len)
                    h.prefill(il, r.slot, r.prompt_len, bits, fa.BF16, got[r.req_id][il, :r.prompt_len], fa.F32)
                h.advance([r.slot], r.prompt_len)
            if plan.decode:
                slots = [r.slot for r in plan.decode]
                max_batch_seen = max(max_batch_seen, len(slots))
                for il in range(4):
                    bits = np.concatenate([_rows(fo, seed, il, r.req_id, r.prompt_len + r.generated, 1)[1]
                                           for r in plan.decode])
                    out = np.empty((len(slots), 4096), np.float32)
                    h.decode(il, slots, bits, fa.BF16, out, fa.F32)
                    for i, r in enumerate(plan.decode):
                        got[r.req_id][il, r.prompt_len + r.generated] = out[i]
                h.advance(slots)
            for r in b.complete(plan):
                assert h.pos(r.slot) == r.prompt_len + r.max_new
                assert h.seq_release(r.slot) == 0
            assert h.pages_free() >= pages - b.pages_reserved
            steps += 1
            assert steps < 1000
        assert h.pages_free() == pages
    assert max_batch_seen >= 2 and sorted(b.finished) == list(range(len(reqs)))
    for rid in alone:
        assert np.abs(got[rid] - alone[rid]).max() <= 2e-5, rid
