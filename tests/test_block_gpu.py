"""The projections either side of attention and the reference's engine interface on top of them.

Golden data: logits and residual-stream sums that the unmodified reference RefModel produced for a small 3-layer
attention stack (tests/golden/make_golden_stack.py); the CPU oracle reproduces them bit for bit and supplies every
intermediate row here.  The GPU keeps bf16 weights (the golden weights are bf16-representable), fp16 K/V and fp16
probabilities, so comparisons are by tolerance: 2e-3 max-abs / 2e-4 mean-abs on the residual stream, as for attention
outputs.
"""
import os
import subprocess

import numpy as np
import pytest

from helpers import assert_close

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
GOLD = os.path.join(HERE, "golden")
LIB_DIR = os.path.join(ROOT, "flint_mac_b200")


@pytest.fixture(scope="module")
def fa():
    import flint_mac_b200 as fa

    fa.load_library()
    return fa


@pytest.fixture(scope="module")
def stack(fo):
    g = np.load(os.path.join(GOLD, "ref_stack.npz"))
    kinds = list(zip(g["is_swa"].tolist(), g["has_rope"].tolist()))
    w = fo.stack_weights(int(g["seed"]), int(g["n_layer"]), int(g["n_embd"]), int(g["n_vocab"]), kinds)
    logits, hidden = fo.stack_forward(w, g["tokens"])
    return dict(g=g, w=w, kinds=kinds, logits=logits, hidden=hidden)


def _open_stack(fa, fo, w, kinds, max_seqs, n_ctx):
    h = fa.Attn([k[0] for k in kinds], [k[1] for k in kinds], max_seqs, n_ctx)
    for il in range(w["n_layer"]):
        h.set_layer(il, w["q_norm"][il], w["k_norm"][il], w["sinks"][il])
        h.set_projections(il, w["attn_norm"][il], *(fo.to_bf16_bits(w[k][il]) for k in ("wq", "wk", "wv", "wo")))
    return h


@pytest.mark.gpu
@pytest.mark.parametrize("n,rows_w,k,norm", [(1, 5120, 4096, True), (5, 5120, 512, True), (8, 4096, 4096, False),
                                             (9, 512, 4096, False), (33, 5120, 2048, True), (64, 5120, 4096, True),
                                             (100, 1024, 512, False), (1, 150144, 2048, True)])
def test_projection_against_the_reference_matvec(fa, fo, n, rows_w, k, norm):
    """out = W . rmsnorm?(x) for decode-sized and chunked batches, all K-split / batch-group variants of the kernel:
    against src/ref arithmetic (rmsnorm, then a double-accumulated matvec per row) on the same bf16 weights."""
    import torch

    seed = 21
    wmat = fo.round_bf16(fo.gen_normal(seed, 60, rows_w * k, 0.0, 0.02)).reshape(rows_w, k)
    x = fo.gen_normal(seed, 61, n * k).reshape(n, k)
    nw = fo.gen_normal(seed, 62, k, 1.0, 0.1)
    with fa.Attn([False], [False], 1, 64) as h:
        w_dev = torch.from_numpy(fo.to_bf16_bits(wmat).view(np.int16)).cuda()
        x_dev = torch.from_numpy(x).cuda()
        nw_dev = torch.from_numpy(nw).cuda()
        out = torch.full((n, rows_w), float("nan"), device="cuda")
        for _ in range(2):  # the second call finds the arrival counters where the first one left them
            h.project_dev(w_dev, rows_w, k, x_dev, n, nw_dev if norm else None, out)
        torch.cuda.synchronize()
        got = out.cpu().numpy()
    rows = range(n) if rows_w <= 8192 else [0]
    for b in rows:
        xin = fo.rmsnorm(x[b], nw) if norm else x[b]
        want = fo.matvec(wmat, xin, n_threads=8)
        err = np.abs(got[b] - want)
        scale = np.abs(want).max()
        assert err.max() <= 2e-5 * max(1.0, scale) + 1e-5, (b, float(err.max()), float(scale))


@pytest.mark.gpu
def test_config1_block_hidden_4096(fa, fo):
    """Config 1 with its projections: hidden 4096, x ~ N(0,1), Wq [4096 x 4096], Wk/Wv [512 x 4096], Wo [4096 x 4096]
    ~ N(0, 0.02), one sliding-window + RoPE layer and one full layer, tokens one at a time across the 513-key window:
    the residual stream after each block against the reference arithmetic (fp32 un-rounded cache)."""
    import torch

    seed, E, T = 0, 4096, 560
    kinds = [(True, True), (False, False)]
    w = fo.stack_weights(seed, 2, E, 128, kinds)
    x = fo.gen_normal(seed, 77, T * E).reshape(T, E)
    # reference: each layer on its own, from the same inputs (the blocks are checked separately, not chained)
    want = np.empty((2, T, E), np.float32)
    for il, (is_swa, has_rope) in enumerate(kinds):
        rows = np.empty((T, fo.QKV_DIM), np.float32)
        for t in range(T):
            xn = fo.rmsnorm(x[t], w["attn_norm"][il])
            rows[t] = np.concatenate([fo.matvec(w[k][il], xn, 8) for k in ("wq", "wk", "wv")])
        att, _, _ = fo.layer_forward(rows, w["q_norm"][il], w["k_norm"][il], w["sinks"][il], is_swa, has_rope, n_threads=8)
        for t in range(T):
            want[il, t] = x[t] + fo.matvec(w["wo"][il], att[t], 8)
    with _open_stack(fa, fo, w, kinds, 1, T) as h:
        # decode path: token by token
        got = np.empty((2, T, E), np.float32)
        x_dev = torch.empty(2, 1, E, device="cuda")
        for t in range(T):
            for il in range(2):
                x_dev[il, 0] = torch.from_numpy(x[t]).cuda()
                h.decode_block_dev(il, [0], x_dev[il])
            h.advance([0])
            got[:, t] = x_dev[:, 0].cpu().numpy()
        for il in range(2):
            assert_close(got[il] - x, want[il] - x, f"decode block, layer {il}")
        # prefill path: the whole prompt at once
        h.set_pos(0, 0)
        for il in range(2):
            xp = torch.from_numpy(x).cuda()
            h.prefill_block_dev(il, 0, T, xp)
            torch.cuda.synchronize()
            assert_close(xp.cpu().numpy() - x, want[il] - x, f"prefill block, layer {il}")
        h.check()


@pytest.mark.gpu
def test_stack_blocks_against_the_reference_golden(fa, fo, stack):
    """The 3-layer stack of the golden run, chained: prefill 600 tokens, decode 100, residual stream after the last
    layer against the reference's (whose per-token sums are the golden file's)."""
    import torch

    g, w, kinds, hidden = stack["g"], stack["w"], stack["kinds"], stack["hidden"]
    assert np.array_equal(hidden.astype(np.float64).sum(1), g["hidden_sum"])
    toks, T, P = g["tokens"], len(g["tokens"]), 600
    with _open_stack(fa, fo, w, kinds, 1, T) as h:
        x = torch.from_numpy(w["embd"][toks[:P]]).cuda().contiguous()
        for il in range(w["n_layer"]):
            h.prefill_block_dev(il, 0, P, x)
        h.advance([0], P)
        got = [x.cpu().numpy()]
        for t in range(P, T):
            xt = torch.from_numpy(w["embd"][toks[t]][None]).cuda().contiguous()
            for il in range(w["n_layer"]):
                h.decode_block_dev(il, [0], xt)
            h.advance([0])
            got.append(xt.cpu().numpy())
        h.check()
    got = np.concatenate(got)
    emb = w["embd"][toks]
    assert_close(got - emb, hidden - emb, "residual stream after three attention blocks")


def _client(tmp_path_factory):
    exe = str(tmp_path_factory.mktemp("capi") / "flint_capi_client")
    r = subprocess.run(["gcc", "-std=gnu11", "-Wall", "-Wextra", "-Werror", "-O1", "-o", exe,
                        os.path.join(HERE, "flint_capi_client.c"), "-L" + LIB_DIR, "-l:libflint_attn.so",
                        "-Wl,-rpath," + LIB_DIR], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    return exe


def test_engine_interface_links_from_c(fa, tmp_path_factory):
    """The nine symbols of src/capi.h resolve at LINK time from a C program that includes include/flint_capi.h."""
    exe = _client(tmp_path_factory)
    r = subprocess.run([exe, "link-only"], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "linked 9 symbols, n_vocab before any model = 150144" in r.stdout


@pytest.mark.gpu
def test_engine_interface_replays_the_server_sequence(fa, fo, stack, tmp_path_factory):
    """open -> prefill -> decode ... -> truncate -> decode -> logits -> close from plain C, on the golden stack: the
    greedy tokens and logits are the reference's wherever its own top-2 margin is not a rounding matter."""
    g, w, logits = stack["g"], stack["w"], stack["logits"]
    tmp = tmp_path_factory.mktemp("model")
    model, tokf = str(tmp / "stack.flint"), str(tmp / "tok.i32")
    fa.write_model_file(model, w)
    g["tokens"].astype(np.int32).tofile(tokf)
    P, D, back = 600, 100, 7
    exe = _client(tmp_path_factory)
    r = subprocess.run([exe, model, tokf, str(P), str(D), str(back)], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout + r.stderr
    lines = r.stdout.strip().splitlines()
    assert lines[0] == f"n_ctx {P + D + 8} n_vocab {w['n_vocab']} pos 0"
    assert lines[1].startswith("empty prefill refused: empty prefill")
    assert lines[-1] == "client ok" and lines[-2].startswith("context full refused: context full")
    calls = [ln.split() for ln in lines[2:-2] if not ln.startswith("truncated")]
    assert len(calls) == 1 + D + back
    expect_pos = [P] + list(range(P + 1, P + D + 1)) + list(range(P + D - back + 1, P + D + 1))
    for (pos, tok, lg, sm), p in zip(calls, expect_pos):
        ref = logits[p - 1]  # the call that ended at position p saw tokens [0, p): logits of position p - 1
        assert int(pos) == p
        top2 = np.sort(ref)[-2:]
        if top2[1] - top2[0] > 5e-3:
            assert int(tok) == int(ref.argmax()), (p, tok, int(ref.argmax()))
        assert abs(float(lg) - ref[int(tok)]) < 5e-3
        assert abs(float(sm) - float(ref.astype(np.float64).sum())) < 1024 * 1e-3
    # the re-decoded tail equals the first pass over the same positions
    first, again = calls[1 + D - back:1 + D], calls[1 + D:]
    assert [c[1:] for c in first] == [c[1:] for c in again]


@pytest.mark.gpu
def test_engine_mirror_and_error_paths(fa, fo, stack, tmp_path):
    w, g, logits = stack["w"], stack["g"], stack["logits"]
    model = str(tmp_path / "stack.flint")
    fa.write_model_file(model, w)
    with pytest.raises(fa.FlintAttnError, match="cannot open"):
        fa.Engine(str(tmp_path / "missing.flint"))
    bad = str(tmp_path / "bad.gguf")
    open(bad, "wb").write(b"GGUF" + b"\0" * 64)
    with pytest.raises(fa.FlintAttnError, match="GGUF loading is outside"):
        fa.Engine(bad)
    with fa.Engine(model, n_ctx=64) as e:
        assert (e.n_ctx, e.n_vocab, e.pos) == (64, w["n_vocab"], 0)
        with pytest.raises(fa.FlintAttnError, match="out of range"):
            e.prefill([w["n_vocab"]])
        nxt = e.prefill(g["tokens"][:40])
        assert e.pos == 40
        assert np.abs(e.logits() - logits[39]).max() < 5e-3
        assert nxt == int(e.logits().argmax())
        with pytest.raises(fa.FlintAttnError, match="context full"):
            e.prefill(g["tokens"][:30])
        assert e.truncate(41) == -1 and e.truncate(10) == 0 and e.pos == 10
