"""CPU-only checks: the C ABI library loads and exports what include/flint_attn.h declares; the split-K planner
and the integer maps are exact."""
import ctypes
import os
import re

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def fa():
    from flint_mac_b200 import build

    build.build()
    import flint_mac_b200 as fa

    return fa


def test_library_exports_every_declared_symbol(fa):
    hdr = open(os.path.join(ROOT, "include", "flint_attn.h")).read()
    declared = set(re.findall(r"\b(flint_attn_[a-z0-9_]+)\s*\(", hdr))
    assert len(declared) >= 20
    lib = ctypes.CDLL(fa.capi.LIB_PATH)
    for name in declared:
        assert hasattr(lib, name), name
    assert declared == set(fa.capi.SYMBOLS), declared ^ set(fa.capi.SYMBOLS)


def test_open_fails_loudly_without_a_gpu(fa):
    import torch

    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    with pytest.raises(fa.FlintAttnError, match="CUDA"):
        fa.Attn([True], [True], 1, 128)


@pytest.mark.parametrize("is_swa", [False, True])
@pytest.mark.parametrize("target", [1, 37, 1184, 100000])
def test_plan_covers_every_key_exactly_once(fa, fo, is_swa, target):
    rng = np.random.default_rng(3)
    pos = [0, 1, 2, 63, 64, 255, 256, 257, 511, 512, 513, 514, 1023, 1024, 1025, 8192, 32767] + \
        [int(x) for x in rng.integers(0, 32768, 40)]
    items = fa.plan_decode(pos, is_swa, target_items=target)
    lengths = items[:, 3] - items[:, 2]
    assert (np.diff(lengths) <= 0).all(), "items are issued longest first"
    for tok, p in enumerate(pos):
        kb = fo.k_begin(p, is_swa)
        for kvh in range(4):
            grp = items[(items[:, 0] == tok) & (items[:, 1] == kvh)]
            grp = grp[np.argsort(grp[:, 5])]
            n_split = len(grp)
            assert (grp[:, 6] == n_split).all() and list(grp[:, 5]) == list(range(n_split))
            assert grp[0, 2] == kb and grp[-1, 3] == p
            assert (grp[1:, 2] == grp[:-1, 3]).all()                # contiguous, no overlap
            assert n_split == 1 or (grp[:, 3] > grp[:, 2]).all()      # no empty split
            assert list(grp[:, 4]) == [0] * (n_split - 1) + [1]       # only the last split folds the new token
            assert len(set(grp[:, 7])) == 1
    # partial records of different groups do not overlap
    multi = items[items[:, 6] > 1]
    recs = set()
    for it in multi:
        r = int(it[7] + it[5])
        assert r not in recs
        recs.add(r)


def test_plan_waves(fa):
    """Equal sequences are cut into one wave of work items; a ragged batch whose one-wave list would leave its longest
    item well above the mean slot load gets two waves of shorter items (and never more)."""
    slots = 296
    for n, ctx in ((8, 8192), (16, 8192), (32, 8192), (64, 8192), (4, 8192), (1, 131072)):
        items = fa.plan_decode([ctx] * n, False, target_items=slots)
        assert len(items) <= slots, (n, ctx, len(items))
    rng = np.random.default_rng(7)
    ragged = [int(x) for x in rng.integers(1, 32769, 32)]
    items = fa.plan_decode(ragged, False, target_items=slots)
    lengths = items[:, 3] - items[:, 2]
    assert slots < len(items) <= 2 * slots
    mean_slot = 4 * sum(ragged) / slots
    assert lengths.max() <= mean_slot            # no item longer than a slot's share of one wave
    # sliding-window layers are never re-planned: one item per (sequence, KV head)
    assert len(fa.plan_decode(ragged, True, target_items=slots)) == 4 * len(ragged)


def test_plan_with_kv_range_sharding(fa, fo):
    pos = [0, 100, 4999, 5000, 5001, 9999]
    shards = [(0, 5000), (5000, 10000)]
    cover = {i: [] for i in range(len(pos))}
    folds = {i: 0 for i in range(len(pos))}
    for lo, hi in shards:
        items = fa.plan_decode(pos, False, kv_lo=lo, kv_hi=hi, target_items=64)
        for it in items[items[:, 1] == 0]:
            if it[2] == it[3] and not it[4]:
                continue  # a shard with no visible key for this token emits one empty record
            assert lo <= it[2] <= it[3] <= hi
            cover[int(it[0])].append((int(it[2]), int(it[3])))
            folds[int(it[0])] += int(it[4])
            if it[4]:
                assert lo <= pos[it[0]] < hi and it[3] == pos[it[0]]
    for i, p in enumerate(pos):
        keys = sorted(j for a, b in cover[i] for j in range(a, b))
        assert keys == list(range(p)), i
        assert folds[i] == 1


def test_integer_maps(fa, fo):
    for p in range(0, 2101):
        assert fo.slot(p, True) == p % 1024 and fo.slot(p, False) == p
        assert fo.k_begin(p, True) == max(0, p - 512) and fo.k_begin(p, False) == 0
    owners = fo.ring_owners(1300)
    assert owners[0] == 1024 and owners[275] == 1299 and owners[276] == 276 and owners[1023] == 1023
    # the reference's own policy (src/engine.mm:742-743)
    assert fo.ref_split_policy(8192, False) == (256, 32)
    assert fo.ref_split_policy(131072, False) == (4096, 32)
    assert fo.ref_split_policy(600, True) == (256, 2)
    assert fo.ref_split_policy(0, True) == (256, 1)
    # rollback rule (server/src/main.rs:96-100) on both sides of the 511 boundary
    for cached, p in [(1000, 489), (1000, 488), (600, 0), (5000, 4489), (5000, 4000), (10, 10), (300, 900)]:
        assert fa.rollback_restart(cached, p) == fo.rollback_restart(cached, p)
    assert fa.rollback_restart(1000, 489) == 489 and fa.rollback_restart(1000, 488) == 0
    assert fa.rollback_restart(5000, 4000) == 3488
