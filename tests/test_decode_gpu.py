"""Decode attention on the GPU, through the C ABI, against the CPU oracle and the reference's golden vectors."""
import os

import numpy as np
import pytest

from helpers import KINDS, assert_close, bf16_round_rows, device_view, synth_cache_f16, to_slot_layout

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(__file__), "golden")


@pytest.fixture(scope="module")
def fa():
    import flint_mac_b200 as fa

    fa.load_library()
    return fa


def _open(fa, kinds, max_seqs, n_ctx, seed=0, **kw):
    names = list(kinds)
    h = fa.Attn([KINDS[k][0] for k in names], [KINDS[k][1] for k in names], max_seqs, n_ctx, **kw)
    return h


def _decode_sequence(fa, fo, h, layer, qkv, weights):
    """Token-by-token decode of one sequence through the host-buffer entry point (how Engine::step drives it)."""
    h.set_layer(layer, *weights)
    out = np.empty((qkv.shape[0], 4096), np.float32)
    row = np.empty(4096, np.float32)
    for t in range(qkv.shape[0]):
        assert h.pos(0) == t
        h.decode(layer, [0], np.ascontiguousarray(qkv[t]), fa.F32, row, fa.F32)
        out[t] = row
        assert h.advance([0]) == 0
    return out


@pytest.mark.parametrize("kind", list(KINDS))
def test_config1_1300_tokens_one_at_a_time(fa, fo, kind):
    """One SWA+RoPE layer and one full layer (and full+RoPE), 1300 tokens decoded one at a time: crosses the
    513-key window and the 1024-slot ring wrap.  Compared at every position and head."""
    is_swa, has_rope = KINDS[kind]
    seed, T = 0, 1300
    w = fo.layer_weights(seed, 2)
    qkv = fo.raw_qkv(seed, 2, 0, T)
    with _open(fa, [kind], 1, 2048) as h:
        got = _decode_sequence(fa, fo, h, 0, qkv, w)
        want, kc, vc = fo.layer_forward(qkv, *w, is_swa, has_rope, round_kv_f16=False, n_threads=8)
        assert_close(got, want, f"{kind} vs fp32 oracle")
        want16, kc16, vc16 = fo.layer_forward(qkv, *w, is_swa, has_rope, round_kv_f16=True, n_threads=8)
        assert_close(got, want16, f"{kind} vs half-rounded oracle")
        # cache contents: V is a pure half rounding of the input, so slot indexing is checked bit for bit;
        # K went through norm/RoPE in fp32 on both sides and may differ in the last half bit.
        n_slots = h.n_slots(0)
        k_dev, v_dev = h.read_kv(0, 0, 0, n_slots)
        owners = fo.ring_owners(T) if is_swa else np.concatenate([np.arange(T), -np.ones(n_slots - T, np.int64)])
        for s in range(n_slots):
            p = int(owners[s])
            if p < 0:
                assert not v_dev[:, s].any() and not k_dev[:, s].any()
                continue
            assert fo.slot(p, is_swa) == s
            assert np.array_equal(v_dev[:, s].reshape(-1), fo.to_f16_bits(vc16[p])), (s, p)
            kd = fo.from_f16_bits(k_dev[:, s].reshape(-1))
            assert np.abs(kd - kc16[p]).max() <= np.abs(kc16[p]).max() * 2 ** -10, (s, p)


@pytest.mark.parametrize("kind", list(KINDS))
def test_golden_vectors_of_the_reference(fa, fo, kind):
    """Same inputs as the run of the unmodified reference RefModel that produced tests/golden/*.npz."""
    g = np.load(os.path.join(GOLD, f"ref_attn_{kind}.npz"))
    seed, layer, T = int(g["seed"]), int(g["layer"]), int(g["n_tok"])
    x = np.zeros((T, 9216), np.float32)
    x[:, :5120] = fo.raw_qkv(seed, layer, 0, T)
    ones = np.ones(9216, np.float32)
    qkv = np.stack([fo.rmsnorm(x[t], ones)[:5120] for t in range(T)])
    with _open(fa, [kind], 1, 1300) as h:
        got = _decode_sequence(fa, fo, h, 0, qkv, fo.layer_weights(seed, layer)).reshape(T, 32, 128)
    assert_close(got[g["probe_pos"]], g["probe_att"], f"{kind} probes")
    rs = got.reshape(T, -1).astype(np.float64).sum(1)
    assert np.abs(rs - g["row_sum"]).max() < 4096 * 2e-4


@pytest.mark.parametrize("kind,target", [("full_rope", 1184), ("full_rope", 37), ("full_rope", 100000),
                                         ("swa_rope", 1184), ("swa_rope", 100000), ("full_nope", 300)])
def test_batched_ragged_decode_bf16(fa, fo, kind, target):
    """Ragged batch over pre-loaded fp16 caches, bf16 q/k/v rows, several split policies (1 split .. many)."""
    is_swa, has_rope = KINDS[kind]
    seed, n_ctx = 21, 4096
    ctx = [0, 1, 63, 64, 65, 511, 512, 513, 1023, 1024, 1025, 2000, 3071, 4095]
    B = len(ctx)
    w = fo.layer_weights(seed, 0)
    with _open(fa, [kind], B, n_ctx) as h:
        h.set_layer(0, *w)
        h.set_target_items(target)
        n_slots = h.n_slots(0)
        caches = []
        for s, c in enumerate(ctx):
            k, v = synth_cache_f16(seed, 0, s, c)
            ks, vs = to_slot_layout(k, n_slots, is_swa), to_slot_layout(v, n_slots, is_swa)
            h.write_kv(0, s, 0, ks, vs)
            h.set_pos(s, c)
            caches.append((ks, vs))
        qkv, qkv_bits = bf16_round_rows(np.stack([fo.raw_qkv(seed, 0, c, 1, seq=s)[0] for s, c in enumerate(ctx)]))
        out_bits = np.empty((B, 4096), np.uint16)
        order = list(range(B))[::-1]  # batch order need not be cache order
        h.decode(0, order, np.ascontiguousarray(qkv_bits[order]), fa.BF16, out_bits, fa.BF16)
        got = fo.from_bf16_bits(out_bits)
        for i, s in enumerate(order):
            ks, vs = caches[s]
            want = fo.decode_token_f16cache(qkv[s], ctx[s], *w, is_swa, has_rope, ks, vs, n_threads=8)
            # bf16 output: half an ulp of the largest output on top of the tolerance
            err = np.abs(got[i] - want)
            assert err.max() <= 2e-3 + np.abs(want).max() * 2 ** -8, (s, ctx[s], err.max())
            # the new token was stored in its slot: V bit-exact
            slot = fo.slot(ctx[s], is_swa)
            k_dev, v_dev = h.read_kv(0, s, slot, 1)
            assert np.array_equal(v_dev, vs[:, slot:slot + 1])
            assert np.abs(fo.from_f16_bits(k_dev) - fo.from_f16_bits(ks[:, slot:slot + 1])).max() <= 2 ** -8


def test_split_invariance_and_sampled_oracle_at_config2_size(fa, fo):
    """Config-2 shape (64 sequences x 8192 cached tokens, one full layer): results do not depend on the split
    policy, and sampled sequences match the oracle."""
    import torch

    B, S, seed = 64, 8192, 5
    w = fo.layer_weights(seed, 0)
    with _open(fa, ["full_rope"], B, S + 8) as h:
        h.set_layer(0, *w)
        n_slots = h.n_slots(0)
        gen = torch.Generator(device="cuda").manual_seed(seed)
        kptr, vptr = h.kv_dev(0, 0), h.kv_dev(0, 1)
        # fill the caches in place with N(0,1) halves (zero-copy views of the library's buffers)
        numel = B * 4 * n_slots * 128
        for ptr in (kptr, vptr):
            buf = device_view(torch, ptr, numel, torch.float16)
            buf.normal_(generator=gen)
        for s in range(B):
            h.set_pos(s, S)
        qkv = torch.randn(B, 5120, generator=gen, device="cuda").to(torch.bfloat16)
        outs = []
        for target in (1184, 200, 5000):
            h.set_target_items(target)
            out = torch.empty(B, 4096, device="cuda", dtype=torch.float32)
            h.decode_dev(0, list(range(B)), qkv, fa.BF16, out, fa.F32)
            torch.cuda.synchronize()
            outs.append(out.cpu().numpy())
        assert np.abs(outs[0] - outs[1]).max() < 2e-5 and np.abs(outs[0] - outs[2]).max() < 2e-5
        qkv_host = fo.from_bf16_bits(qkv.view(torch.int16).cpu().numpy().view(np.uint16))
        for s in (0, 17, 63):
            k16, v16 = h.read_kv(0, s, 0, n_slots)
            # read_kv happened after the decode: the slot of position S already holds the new token; the oracle
            # rewrites it with the same values
            want = fo.decode_token_f16cache(qkv_host[s], S, *w, False, True, k16, v16, n_threads=8)
            assert_close(outs[0][s], want, f"config-2 sequence {s}")


def test_kv_sharded_partials_and_combine(fa, fo):
    """Long-context layout on one device: two handles each holding half of the key range produce partial
    (O, m, l) records; the combine kernel merges them with the sink.  Equals the unsharded result."""
    import torch

    seed, n_ctx, P = 9, 6000, 5000
    w = fo.layer_weights(seed, 0)
    k, v = synth_cache_f16(seed, 0, 0, P)
    qkv = fo.raw_qkv(seed, 0, P, 1)
    parts = []
    for pos_case in (P, 2500):  # new token owned by the second / by the first shard
        with _open(fa, ["full_rope"], 1, n_ctx) as h0:
            h0.set_layer(0, *w)
            h0.write_kv(0, 0, 0, to_slot_layout(k[:pos_case], n_ctx, False), to_slot_layout(v[:pos_case], n_ctx, False))
            h0.set_pos(0, pos_case)
            ref = np.empty((1, 4096), np.float32)
            h0.decode(0, [0], qkv, fa.F32, ref, fa.F32)
        partials = torch.zeros(2, 1, 32, 130, device="cuda")
        q_dev = torch.from_numpy(qkv).cuda()
        out = torch.empty(1, 4096, device="cuda")
        handles = [_open(fa, ["full_rope"], 1, n_ctx, kv_rank=r, kv_ranks=2) for r in range(2)]
        try:
            for r, h in enumerate(handles):
                h.set_layer(0, *w)
                lo, n = r * 3000, h.n_slots(0)
                assert n == 3000
                hi = min(pos_case, lo + n)
                if hi > lo:
                    h.write_kv(0, 0, 0, k[lo:hi].transpose(1, 0, 2).copy(), v[lo:hi].transpose(1, 0, 2).copy())
                h.set_pos(0, pos_case)
                h.decode_partial_dev(0, [0], q_dev, fa.F32, partials[r])
            handles[0].combine_dev(0, 1, 2, partials, out, fa.F32)
            torch.cuda.synchronize()
            assert np.abs(out.cpu().numpy() - ref).max() < 2e-5
            # records follow fused.metal:324-327; compare with the oracle's partial arithmetic
            pr = partials.cpu().numpy()
            assert np.isfinite(pr[..., :128]).all()
            parts.append(pr)
        finally:
            for h in handles:
                h.close()
    # when the first shard owns the token (pos 2500) the second shard has no keys at all: l = 0
    assert (parts[1][1, 0, :, 129] == 0).all()


def test_errors_do_not_cross_the_boundary(fa, fo):
    with _open(fa, ["swa_rope"], 2, 64) as h:
        row, out = np.zeros(5120, np.float32), np.zeros(4096, np.float32)
        with pytest.raises(fa.FlintAttnError, match="weights not set"):
            h.decode(0, [0], row, fa.F32, out, fa.F32)
        h.set_layer(0, *fo.layer_weights(0, 0))
        with pytest.raises(fa.FlintAttnError, match="out of range"):
            h.decode(0, [2], row, fa.F32, out, fa.F32)
        with pytest.raises(fa.FlintAttnError, match="out of range"):
            h.decode(1, [0], row, fa.F32, out, fa.F32)
        h.set_pos(0, 64)
        with pytest.raises(fa.FlintAttnError, match="context full"):
            h.decode(0, [0], row, fa.F32, out, fa.F32)
        assert h.truncate(0, 65) == -1 and h.truncate(0, -1) == -1 and h.truncate(0, 10) == 0 and h.pos(0) == 10
    with pytest.raises(fa.FlintAttnError):
        fa.Attn([True], [True], 1, 128, device=99)


def _sharded_pair(fa, w, n_ctx, k, v, pos):
    """Two KV-range shards of one sequence as two handles on this GPU, exchange buffers connected in-process."""
    handles = [_open(fa, ["full_rope"], 1, n_ctx, kv_rank=r, kv_ranks=2) for r in range(2)]
    for r, h in enumerate(handles):
        h.set_layer(0, *w)
        lo, n = r * (n_ctx // 2), h.n_slots(0)
        hi = min(pos, lo + n)
        if hi > lo:
            h.write_kv(0, 0, 0, k[lo:hi].transpose(1, 0, 2).copy(), v[lo:hi].transpose(1, 0, 2).copy())
        h.set_pos(0, pos)
        h.xchg_create(1)
    bases = [h.xchg_base() for h in handles]
    for h in handles:
        h.xchg_connect_local(bases)
    return handles


def test_kv_sharded_exchange_through_peer_buffers(fa, fo):
    """The decode kernel stores its records into every rank's gather buffer and publishes a step flag; the combine
    kernel waits on the flags and merges.  Both ranks live on this one GPU here, so every rank posts before any
    rank combines (a waiting kernel never runs ahead of its producer).  Three steps in a row cover both record
    buffers and their reuse; every rank's output equals the unsharded decode."""
    import torch

    seed, n_ctx, P, steps = 11, 6000, 2998, 4  # the token's owner changes from shard 0 to shard 1 at position 3000
    w = fo.layer_weights(seed, 0)
    k, v = synth_cache_f16(seed, 0, 0, P)
    rows = fo.raw_qkv(seed, 0, P, steps)
    refs = np.empty((steps, 4096), np.float32)
    with _open(fa, ["full_rope"], 1, n_ctx) as h0:
        h0.set_layer(0, *w)
        h0.write_kv(0, 0, 0, to_slot_layout(k, n_ctx, False), to_slot_layout(v, n_ctx, False))
        h0.set_pos(0, P)
        for s in range(steps):
            h0.decode(0, [0], rows[s], fa.F32, refs[s:s + 1], fa.F32)
            h0.advance([0])
    handles = _sharded_pair(fa, w, n_ctx, k, v, P)
    try:
        with pytest.raises(fa.FlintAttnError, match="nothing was posted"):
            handles[0].combine_xchg_dev(0, 1, torch.empty(1, 4096, device="cuda"), fa.F32)
        # a post that fails validation must not move this rank's step counter (its peers would wait for a step that
        # is never published)
        handles[0].set_pos(0, n_ctx)
        with pytest.raises(fa.FlintAttnError, match="context full"):
            handles[0].decode_xchg_post_dev(0, [0], torch.zeros(1, 5120, device="cuda"), fa.F32)
        handles[0].set_pos(0, P)
        outs = torch.zeros(2, steps, 4096, device="cuda")
        for s in range(steps):
            q_dev = torch.from_numpy(rows[s:s + 1]).cuda()
            for h in handles:
                h.decode_xchg_post_dev(0, [0], q_dev, fa.F32)
            for r, h in enumerate(handles):
                h.combine_xchg_dev(0, 1, outs[r, s:s + 1], fa.F32)
                h.advance([0])
        torch.cuda.synchronize()
        for h in handles:
            h.check()
        got = outs.cpu().numpy()
        assert np.abs(got[0] - refs).max() < 2e-5 and np.abs(got[1] - refs).max() < 2e-5
    finally:
        for h in handles:
            h.close()


def test_exchange_wait_is_bounded(fa, fo):
    """A rank whose peer never posts: the combine kernel gives up after about a second, records the fact, and the
    context stays usable (the next check reports it; nothing hangs or faults)."""
    import torch

    seed, n_ctx, P = 12, 2048, 300
    w = fo.layer_weights(seed, 0)
    k, v = synth_cache_f16(seed, 0, 0, P)
    handles = _sharded_pair(fa, w, n_ctx, k, v, P)
    try:
        q_dev = torch.from_numpy(fo.raw_qkv(seed, 0, P, 1)).cuda()
        out = torch.zeros(1, 4096, device="cuda")
        handles[0].decode_xchg_post_dev(0, [0], q_dev, fa.F32)  # rank 1 stays silent
        handles[0].combine_xchg_dev(0, 1, out, fa.F32)
        with pytest.raises(fa.FlintAttnError, match="ran out"):
            handles[0].check()
        handles[0].check()  # reported once, then cleared: the handle is usable again
        torch.cuda.synchronize()
        assert float((out + 1).sum().item()) == 4096.0  # the device still answers; the output was left alone
    finally:
        for h in handles:
            h.close()


def test_host_entry_with_page_locked_output_rows(fa, fo):
    """flint_attn_decode writes its output rows straight into page-locked host memory (no staging copy); pageable
    rows go through the device staging buffer.  Both give the same bits."""
    import torch

    seed, B, S = 31, 5, 700
    w = fo.layer_weights(seed, 0)
    rows, bits = bf16_round_rows(np.stack([fo.raw_qkv(seed, 0, S, 1, seq=s)[0] for s in range(B)]))
    outs = []
    for pinned in (False, True):
        with _open(fa, ["full_rope"], B, 1024) as h:
            h.set_layer(0, *w)
            for s in range(B):
                k, v = synth_cache_f16(seed, 0, s, S)
                h.write_kv(0, s, 0, to_slot_layout(k, 1024, False), to_slot_layout(v, 1024, False))
                h.set_pos(s, S)
            if pinned:
                q_host = torch.from_numpy(bits.view(np.int16)).pin_memory()
                o_host = torch.zeros(B, 4096, dtype=torch.float32).pin_memory()
                h.decode(0, list(range(B)), q_host, fa.BF16, o_host, fa.F32)
                outs.append(o_host.numpy().copy())
            else:
                o = np.zeros((B, 4096), np.float32)
                h.decode(0, list(range(B)), bits, fa.BF16, o, fa.F32)
                outs.append(o)
    assert np.array_equal(outs[0], outs[1])
    assert np.abs(outs[0]).max() > 0
