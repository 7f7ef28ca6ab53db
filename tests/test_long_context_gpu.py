"""Decode attention at the sizes of the long-context and ragged configurations, against the CPU oracle.

One sequence with 131 072 cached tokens on a full-attention layer is cut into about 70 key ranges per KV head, so the
second level of the split-K merge runs (more than 16 splits per group); every case here is compared with the oracle's
src/ref arithmetic, not with another launch of the same kernel.  The same sequence is also run as two KV-range shards
(two handles on this GPU) through both exchanges: partial records + combine, and the records stored by the decode
kernel into the ranks' gather buffers.  The ragged case puts 20 000-32 767-token sequences next to 1-token ones on the
3 sliding-window + 1 full layer stack.
"""
import numpy as np
import pytest

from helpers import assert_close, device_view

pytestmark = pytest.mark.gpu
S_LONG = 131072


@pytest.fixture(scope="module")
def fa():
    import flint_mac_b200 as fa

    fa.load_library()
    return fa


@pytest.fixture(scope="module")
def long_case(fa, fo):
    """K/V ~ N(0,1) halves for positions [0, 131072) generated on the device, the two query rows (fp32 and the same
    rounded to bf16) and the oracle's outputs for both."""
    import torch

    seed, n_ctx = 41, S_LONG + 8
    gen = torch.Generator(device="cuda").manual_seed(seed)
    k = torch.randn(4, n_ctx, 128, generator=gen, device="cuda").to(torch.float16)
    v = torch.randn(4, n_ctx, 128, generator=gen, device="cuda").to(torch.float16)
    w = fo.layer_weights(seed, 0)
    row32 = fo.raw_qkv(seed, 0, S_LONG, 1)[0]
    row16_bits = fo.to_bf16_bits(row32)
    row16 = fo.from_bf16_bits(row16_bits)
    k16 = k.cpu().numpy().view(np.uint16)
    v16 = v.cpu().numpy().view(np.uint16)
    want32 = fo.decode_token_f16cache(row32, S_LONG, *w, False, True, k16.copy(), v16.copy(), n_threads=16)
    want16 = fo.decode_token_f16cache(row16, S_LONG, *w, False, True, k16.copy(), v16.copy(), n_threads=16)
    return dict(seed=seed, n_ctx=n_ctx, k=k, v=v, w=w, row32=row32, row16_bits=row16_bits, want32=want32, want16=want16)


def _rows(torch, fa, case, dtype):
    if dtype == fa.F32:
        return torch.from_numpy(case["row32"][None]).cuda(), case["want32"]
    return torch.from_numpy(case["row16_bits"].view(np.int16)[None]).cuda().view(torch.bfloat16), case["want16"]


def _check(got, want, dtype, fa, what):
    if dtype == fa.F32:
        assert_close(got, want, what)
    else:  # bf16 output rows: half an ulp of the largest output on top of the tolerance
        err = np.abs(np.asarray(got, np.float32).reshape(-1) - want)
        assert err.max() <= 2e-3 + np.abs(want).max() * 2 ** -8, (what, float(err.max()))
        assert err.mean() <= 2e-4 + np.abs(want).mean() * 2 ** -8, (what, float(err.mean()))


@pytest.mark.parametrize("dtype_name", ["f32", "bf16"])
def test_131072_cached_tokens_on_one_handle(fa, fo, long_case, dtype_name):
    """Unsharded: one handle scans all 131 072 keys; the planner cuts each KV head's range into more than 16 splits,
    so the records are folded in two levels before the sink enters."""
    import torch

    dtype = fa.F32 if dtype_name == "f32" else fa.BF16
    case = long_case
    plan = fa.plan_decode([S_LONG], False, 0, case["n_ctx"], 296)
    assert plan[:, 6].min() > 16, "the second merge level needs more than 16 splits per (token, KV head)"
    with fa.Attn([False], [True], 1, case["n_ctx"]) as h:
        h.set_layer(0, *case["w"])
        n = 4 * h.n_slots(0) * 128
        device_view(torch, h.kv_dev(0, 0), n, torch.float16).copy_(case["k"].reshape(-1))
        device_view(torch, h.kv_dev(0, 1), n, torch.float16).copy_(case["v"].reshape(-1))
        h.set_pos(0, S_LONG)
        rows, want = _rows(torch, fa, case, dtype)
        out = torch.empty(1, 4096, device="cuda", dtype=torch.float32 if dtype == fa.F32 else torch.bfloat16)
        h.decode_dev(0, [0], rows, dtype, out, dtype)
        torch.cuda.synchronize()
        h.check()
        _check(out.float().cpu().numpy(), want, dtype, fa, f"131072 tokens, {dtype_name} rows")
        # the new token landed in slot 131072: V is a pure rounding of the row
        _, v_new = h.read_kv(0, 0, S_LONG, 1)
        src = case["row32"] if dtype == fa.F32 else fo.from_bf16_bits(case["row16_bits"])
        assert np.array_equal(v_new.reshape(-1), fo.to_f16_bits(src[4608:]))


@pytest.mark.parametrize("dtype_name", ["f32", "bf16"])
def test_131072_cached_tokens_as_two_kv_range_shards(fa, fo, long_case, dtype_name):
    """Two handles hold the key ranges [0, 65540) and [65540, 131080).  Each scans its own keys (about 70 splits per KV
    head, two merge levels, no sink), and the per-shard records are merged with the sink by (a) flint_attn_combine_dev
    over records written to a caller buffer and (b) the exchange inside the kernels (records stored into both ranks'
    gather buffers, combine waits on the step flags).  Both are compared with the oracle."""
    import torch

    dtype = fa.F32 if dtype_name == "f32" else fa.BF16
    tdtype = torch.float32 if dtype == fa.F32 else torch.bfloat16
    case = long_case
    n_ctx = case["n_ctx"]
    handles = [fa.Attn([False], [True], 1, n_ctx, kv_rank=r, kv_ranks=2) for r in range(2)]
    try:
        for r, h in enumerate(handles):
            h.set_layer(0, *case["w"])
            n_slots = h.n_slots(0)
            lo = r * n_slots
            assert n_slots == (n_ctx + 1) // 2
            for which, src in ((0, case["k"]), (1, case["v"])):
                dst = device_view(torch, h.kv_dev(0, which), 4 * n_slots * 128, torch.float16).view(4, n_slots, 128)
                dst.copy_(src[:, lo:lo + n_slots])
            h.set_pos(0, S_LONG)
            h.xchg_create(1)
        bases = [h.xchg_base() for h in handles]
        for h in handles:
            h.xchg_connect_local(bases)
        rows, want = _rows(torch, fa, case, dtype)
        # (a) records to a caller buffer, merged by the combine kernel
        partials = torch.zeros(2, 1, 32, 130, device="cuda")
        for r, h in enumerate(handles):
            h.decode_partial_dev(0, [0], rows, dtype, partials[r])
        out_a = torch.empty(1, 4096, device="cuda", dtype=tdtype)
        handles[0].combine_dev(0, 1, 2, partials, out_a, dtype)
        torch.cuda.synchronize()
        pr = partials.cpu().numpy()
        assert np.isfinite(pr).all() and (pr[:, 0, :, 129] > 0).all(), "both shards hold keys of every head"
        _check(out_a.float().cpu().numpy(), want, dtype, fa, f"two shards + combine, {dtype_name}")
        # (b) records exchanged by the kernels; both ranks post before either combines (they share this GPU)
        outs = torch.empty(2, 1, 4096, device="cuda", dtype=tdtype)
        for h in handles:
            h.decode_xchg_post_dev(0, [0], rows, dtype)
        for r, h in enumerate(handles):
            h.combine_xchg_dev(0, 1, outs[r], dtype)
        torch.cuda.synchronize()
        for h in handles:
            h.check()
        for r in range(2):
            _check(outs[r].float().cpu().numpy(), want, dtype, fa, f"two shards, in-kernel exchange, rank {r}, {dtype_name}")
    finally:
        for h in handles:
            h.close()


def test_ragged_batch_with_long_sequences_on_the_layer_stack(fa, fo):
    """One decode step over 3 sliding-window layers + 1 full layer for a batch that mixes sequences of 20 000 to 32 767
    cached tokens with 1- and 2-token ones; bf16 rows in, fp32 rows out, every sequence and layer against the oracle."""
    import torch

    seed, n_ctx = 43, 32768
    ctx = [1, 32767, 20000, 1, 27001, 2, 31111, 513, 24576, 1023]
    B = len(ctx)
    is_swa, has_rope = [True, True, True, False], [True, True, True, False]
    w = [fo.layer_weights(seed, il) for il in range(4)]
    gen = torch.Generator(device="cuda").manual_seed(seed)
    with fa.Attn(is_swa, has_rope, B, n_ctx) as h:
        for il in range(4):
            h.set_layer(il, *w[il])
            n = B * 4 * h.n_slots(il) * 128
            for which in (0, 1):
                device_view(torch, h.kv_dev(il, which), n, torch.float16).normal_(generator=gen)
        for s, c in enumerate(ctx):
            h.set_pos(s, c)
        seqs = list(range(B))
        for il in range(4):
            n_slots = h.n_slots(il)
            before = [h.read_kv(il, s, 0, n_slots) for s in seqs]  # slot layout, as the oracle takes it
            rows = np.stack([fo.raw_qkv(seed, il, ctx[s], 1, seq=s)[0] for s in seqs])
            bits = fo.to_bf16_bits(rows)
            rows = fo.from_bf16_bits(bits)
            out = torch.empty(B, 4096, device="cuda")
            h.decode_dev(il, seqs, torch.from_numpy(bits.view(np.int16)).cuda().view(torch.bfloat16), fa.BF16, out, fa.F32)
            torch.cuda.synchronize()
            got = out.cpu().numpy()
            for s in seqs:
                ks, vs = before[s]
                want = fo.decode_token_f16cache(rows[s], ctx[s], *w[il], is_swa[il], has_rope[il], ks, vs, n_threads=16)
                assert_close(got[s], want, f"layer {il}, sequence {s} ({ctx[s]} cached tokens)")
        h.check()
