"""Multi-rank host logic on CPU: placement functions, and the partial-record exchange over a 2-rank gloo group
checked with the oracle's partial/combine arithmetic (src/metal/fused.metal:324-350)."""
import os
import socket

import numpy as np
import pytest


def test_balance_by_kv_bytes_is_a_partition_and_balanced():
    from flint_mac_b200 import shard

    rng = np.random.default_rng(7)
    ctx = [int(x) for x in rng.integers(1, 32769, 256)]
    for n in (1, 2, 4, 8):
        owned = shard.balance_by_kv_bytes(ctx, n, n_full_layers=1, n_swa_layers=3)
        flat = sorted(i for o in owned for i in o)
        assert flat == list(range(256))
        loads = [sum(shard.kv_bytes_per_token_step(ctx[i], 1, 3) for i in o) for o in owned]
        assert max(loads) <= min(loads) + shard.kv_bytes_per_token_step(max(ctx), 1, 3)
        assert max(loads) / (sum(loads) / n) < 1.02


def test_kv_shard_ranges_tile_the_context():
    from flint_mac_b200 import shard

    for n_ctx in (1, 7, 4096, 131072, 131073):
        for n in (1, 2, 3, 8):
            r = [shard.kv_shard_range(n_ctx, k, n) for k in range(n)]
            assert r[0][0] == 0 and r[-1][1] == n_ctx
            assert all(a[1] == b[0] for a, b in zip(r[:-1], r[1:]))
    assert shard.contiguous_blocks(64, 8) == [(8 * i, 8 * i + 8) for i in range(8)]
    assert [e - b for b, e in shard.contiguous_blocks(10, 4)] == [3, 3, 2, 2]


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _rank_main(rank, world, port, results):
    import torch
    import torch.distributed as dist

    from flint_mac_b200 import dist as fdist, shard
    from oracle import oracle as fo

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        seed, P = 13, 1500  # every rank regenerates the same sequence; each attends only to its key range
        w = fo.layer_weights(seed, 0)
        qkv = fo.raw_qkv(seed, 0, 0, P + 1)
        want, kc, vc = fo.layer_forward(qkv, *w, False, True)
        q_vec = fo.qk_norm_rope(qkv[P], w[0], w[1], P, True)[:fo.Q_DIM]
        lo, hi = shard.kv_shard_range(P + 1, rank, world)
        part = fo.attend_partial(q_vec, kc, vc, lo, hi)  # the owner of position P folds the new token: hi == P+1 there
        gathered = fdist.gather_partials(torch.from_numpy(part[None]))  # [world, 1, 32, 130]
        merged = fo.combine(np.ascontiguousarray(gathered.numpy()[:, 0].transpose(1, 0, 2)), w[2])
        err = float(np.abs(merged.reshape(-1) - want[P]).max())
        out = (rank, err, tuple(gathered.shape))
    finally:
        dist.destroy_process_group()
    results.put(out)


def test_partial_exchange_over_gloo_world_size_2():
    import torch.multiprocessing as mp

    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_rank_main, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, err, shape in res:
        assert shape == (2, 1, 32, 130)
        assert err < 2e-6, (rank, err)
