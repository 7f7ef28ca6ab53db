"""The allocation-free decode entry point against the handle-based one.

flint_attn_decode_noalloc_dev exists for hosts that cannot allocate device memory when they need attention (their
own arena owns the GPU and the KV caches, or an allocation's implicit synchronisation is not acceptable where they
call from).  It takes caller-owned device buffers for everything and keeps its split-K scratch in a fixed array
inside the library.  Here the caller's buffers are torch tensors made by the test; the call under test allocates
nothing.  Two calls in a row must both agree with flint_attn_decode_dev: the second one finds the first one's
partial records and counters in the shared array.

Collected last on purpose: a run that stops at the first failure has by then run every other test.
"""
import numpy as np
import pytest

from helpers import KINDS, synth_cache_f16, to_slot_layout

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("kind", ["full_rope", "swa_rope"])
def test_noalloc_decode_matches_handle_decode_twice_in_a_row(fo, kind):
    import torch

    import flint_mac_b200 as fa

    is_swa, has_rope = KINDS[kind]
    seed, n_ctx = 31, 6144
    ctx = [0, 5, 300, 513, 1024, 2047, 4000, 6000]  # several splits per sequence for the long ones
    B = len(ctx)
    qn, kn, sinks = fo.layer_weights(seed, 0)
    with fa.Attn([is_swa], [has_rope], B, n_ctx) as h:
        h.set_layer(0, qn, kn, sinks)
        n_slots = h.n_slots(0)
        k_mine = torch.zeros(B, 4, n_slots, 128, dtype=torch.float16, device="cuda")
        v_mine = torch.zeros_like(k_mine)
        for s, c in enumerate(ctx):
            k, v = synth_cache_f16(seed, 0, s, c)
            ks, vs = to_slot_layout(k, n_slots, is_swa), to_slot_layout(v, n_slots, is_swa)
            h.write_kv(0, s, 0, ks, vs)
            h.set_pos(s, c)
            k_mine[s] = torch.from_numpy(ks.view(np.float16)).cuda()
            v_mine[s] = torch.from_numpy(vs.view(np.float16)).cuda()
        qn_d, kn_d, sk_d = (torch.from_numpy(x).cuda() for x in (qn, kn, sinks))
        seqs = list(range(B))
        pos = list(ctx)
        for call in range(2):
            rows = np.stack([fo.raw_qkv(seed, 0, p, 1, seq=s)[0] for s, p in enumerate(pos)])
            qkv = torch.from_numpy(rows).cuda().to(torch.bfloat16)
            want = torch.empty(B, 4096, device="cuda")
            got = torch.full((B, 4096), float("nan"), device="cuda")
            h.decode_dev(0, seqs, qkv, fa.BF16, want, fa.F32)
            fa.decode_noalloc_dev(pos, qkv, fa.BF16, got, fa.F32, k_mine, v_mine, n_slots, is_swa, has_rope, qn_d, kn_d,
                                  sk_d)
            torch.cuda.synchronize()
            # Same kernel and same inputs.  The handle may cut the key ranges a little differently (on the second call
            # it extends its previous work list by one position instead of planning anew), so the two agree to what
            # moving a split boundary does to the half-precision probabilities (a few 1e-5), far inside the 2e-3 of
            # the parity tests, rather than bit for bit.
            assert torch.isfinite(got).all()
            assert (got - want).abs().max().item() <= 1e-4, f"call {call}: outputs differ from flint_attn_decode_dev"
            # both wrote the new token's K/V into its slot
            for s, p in enumerate(pos):
                slot = fo.slot(p, is_swa)
                k_h, v_h = h.read_kv(0, s, slot, 1)
                assert np.array_equal(k_mine[s, :, slot].cpu().numpy().view(np.uint16), k_h[:, 0])
                assert np.array_equal(v_mine[s, :, slot].cpu().numpy().view(np.uint16), v_h[:, 0])
            h.advance(seqs, 1)
            pos = [p + 1 for p in pos]


def test_noalloc_rejects_sizes_beyond_the_fixed_scratch(fo):
    import torch

    import flint_mac_b200 as fa

    dummy = torch.zeros(1024, device="cuda")
    with pytest.raises(fa.FlintAttnError, match="1..64"):
        fa.decode_noalloc_dev([0] * 65, dummy, fa.F32, dummy, fa.F32, dummy, dummy, 1024, True, True, dummy, dummy, dummy)
    with pytest.raises(fa.FlintAttnError, match="outside the cache"):
        fa.decode_noalloc_dev([4096], dummy, fa.F32, dummy, fa.F32, dummy, dummy, 4096, False, True, dummy, dummy, dummy)
