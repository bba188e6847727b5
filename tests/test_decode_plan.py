"""How the decode attention kernel deals a step's pages to its CTAs, checked on the host.

The plan is worked out by one function (``csrc/decode_plan.h``) that the kernels call on the device and that
``csrc/decode_plan_host.cpp`` compiles for the host.  A wrong plan shows on a device only as a wrong logit
somewhere; here every plan of a launch is looked at directly: every unit of work dealt exactly once, in
order, nothing for a CTA past the last, each way of dealing within the limits the kernel's merge has.
No counterpart in the reference (its decode attention cuts every sequence into a fixed number of parts:
engine/kernels/attention.py:140-177).
"""

import ctypes
import random

import numpy as np
import pytest

PAGE = 64
GROUP_COST = 4          # kGroupCost: units in front of a group's pages in equal runs
MOST_PARTS = 64         # kMaxGroupParts: CTAs that may share one group


@pytest.fixture(scope="module")
def planner():
    from dryft_flash_infer_b200.ops import build

    lib = build.load_library("dfi_plan", build.PLAN_SOURCES)
    assert lib.dfi_decode_plan_ints() == 12
    return lib


def plans_of(lib, lengths, n_kv, group, window, launched, cluster, head_dim):
    """``lengths``: keys of each sequence with the step's token.  Rows of (total, n_ctas, parts, tiles, whole, uneven,
    group_cost, first_unit, end_unit, first_seq, -, -), one a CTA."""
    seq_start = np.asarray([l - 1 for l in lengths], dtype=np.int32)
    out = np.full((launched, 12), -7, dtype=np.int32)
    rc = lib.dfi_decode_plan_host(out.ctypes.data_as(ctypes.c_void_p), seq_start.ctypes.data_as(ctypes.c_void_p),
                                  len(lengths), n_kv, group, window, launched, cluster, head_dim)
    assert rc == 0
    return out


def pages_of(length, window):
    pos = length - 1
    first_key = max(0, pos - window + 1) if window > 0 else 0
    return pos // PAGE - first_key // PAGE + 1


def check(plans, lengths, n_kv, group, window, launched, cluster, head_dim):
    tiles = [pages_of(l, window) for l in lengths]
    n, groups = len(lengths), len(lengths) * n_kv
    total, n_ctas, parts, run_tiles, whole, uneven, gc = (int(x) for x in plans[0, :7])
    assert (plans[:, :7] == plans[0, :7]).all()                 # every CTA works out the same launch
    assert gc in (0, GROUP_COST) and total == (sum(tiles) + n * gc) * n_kv
    assert 1 <= n_ctas <= launched
    first, end, first_seq = plans[:, 7].astype(int), plans[:, 8].astype(int), plans[:, 9].astype(int)
    assert (first[n_ctas:] == end[n_ctas:]).all()               # nothing past the last CTA
    assert first[0] == 0 and end[n_ctas - 1] == total           # every unit, once, in order
    assert (first[1:n_ctas] == end[:n_ctas - 1]).all() and (first[:n_ctas] <= end[:n_ctas]).all()
    # where sequences and groups begin in the units
    seq_begin = np.concatenate([[0], np.cumsum([(t + gc) * n_kv for t in tiles])])
    group_begin = np.array([seq_begin[s] + h * (tiles[s] + gc) for s in range(n) for h in range(n_kv)] + [total])
    for c in range(n_ctas):
        if first[c] < end[c] or uneven:
            s = first_seq[c]
            assert 0 <= s < n and seq_begin[s] <= first[c] < seq_begin[s + 1], (c, s)
    merges = cluster > 1 and head_dim % cluster == 0 and (head_dim // cluster) % 4 == 0
    if parts > 0:
        assert gc == 0 and whole == 0 and parts <= MOST_PARTS and n_ctas == groups * parts
        if not uneven:
            assert len(set(tiles)) == 1 and run_tiles == tiles[0]
        for c in range(n_ctas):                                   # a CTA stays inside the group it is a part of
            g = c // parts
            assert group_begin[g] <= first[c] <= end[c] <= group_begin[g + 1], (c, g)
        if uneven and not (merges and parts == cluster):
            assert (first[:n_ctas] < end[:n_ctas]).all()          # parts without pages only meet in a cluster
        if cluster > 1 and parts == cluster:
            assert n_ctas % cluster == 0
    elif whole > 0:
        assert gc == 0 and whole == groups
        edges = set(int(x) for x in group_begin)
        assert all(int(first[c]) in edges and int(end[c]) in edges for c in range(n_ctas))
    else:
        assert gc == GROUP_COST and not uneven
        # CTAs that hold pages of one group (its first gc units are no pages)
        for g in range(groups):
            lo, hi = group_begin[g] + gc, group_begin[g + 1]
            holders = sum(1 for c in range(n_ctas) if max(first[c], lo) < min(end[c], hi))
            assert 1 <= holders <= MOST_PARTS, (g, holders)
    return parts, whole, uneven


def launch_of(rnd):
    cluster = rnd.choice([1, 2, 4, 8, 16])
    launched = rnd.choice([1, 3, 16, 40, 148, 272, 284, 296, 500])
    launched = max(cluster, launched // cluster * cluster)       # a launch in clusters is a whole number of them
    return launched, cluster


@pytest.mark.parametrize("seed", range(6))
def test_every_unit_is_dealt_once_whatever_the_step(planner, seed):
    rnd = random.Random(seed)
    seen = set()
    for _ in range(400):
        n_kv, group = rnd.choice([1, 2, 4, 8]), rnd.choice([1, 2, 4, 8, 16])
        launched, cluster = launch_of(rnd)
        head_dim = rnd.choice([128, 64, 96, 48])
        window = rnd.choice([0, 0, 0, 100, 4096])
        n = rnd.choice([1, 1, 2, 3, 8, 9, 16, 40, 64, 70, 300])
        kind = rnd.choice(["equal", "random", "short", "mixed", "long"])
        if kind == "equal":
            lengths = [rnd.choice([1, 63, 64, 65, 600, 1270, 2100, 4096, 10000, 32768])] * n
        elif kind == "short":
            lengths = [rnd.randint(1, 130) for _ in range(n)]
        elif kind == "mixed":
            lengths = [rnd.choice([1, 64, 65, 300, 1500, 4000]) for _ in range(n)]
        elif kind == "long":
            lengths = [rnd.randint(20000, 40000) for _ in range(min(n, 16))]
        else:
            lengths = [rnd.randint(1, 5000) for _ in range(n)]
        plans = plans_of(planner, lengths, n_kv, group, window, launched, cluster, head_dim)
        parts, whole, uneven = check(plans, lengths, n_kv, group, window, launched, cluster, head_dim)
        seen.add(("parts" if parts else "whole" if whole else "runs", bool(uneven), parts == cluster and cluster > 1))
    # the cases reach every way of dealing
    assert {("runs", False, False), ("parts", False, True), ("parts", True, True), ("whole", False, False),
            ("whole", True, False), ("parts", False, False), ("parts", True, False)} <= seen, seen


def test_the_benchmark_shapes_are_dealt_as_the_design_says(planner):
    # batch 8 at 4,096 keys, 8 key/value heads, clusters of four on a wave of 284 CTAs: 64 groups x 4 parts of 16 pages
    plans = plans_of(planner, [4096] * 8, 8, 4, 0, 284, 4, 128)
    assert tuple(plans[0, :7]) == (4096, 256, 4, 64, 0, 0, 0)
    assert [tuple(plans[c, 7:10]) for c in (0, 1, 255, 256)] == [(0, 16, 0), (16, 32, 0), (4080, 4096, 7), (0, 0, 0)]
    # one sequence of 4,096 keys in clusters of sixteen: 8 groups x 16 parts of 4 pages
    plans = plans_of(planner, [4096], 8, 4, 0, 272, 16, 128)
    assert tuple(plans[0, :7]) == (512, 128, 16, 64, 0, 0, 0)
    # ... and with a head size whose columns sixteen CTAs cannot share in fours, more and shorter parts by ticket
    plans = plans_of(planner, [4096], 8, 4, 0, 272, 16, 96)
    check(plans, [4096], 8, 4, 0, 272, 16, 96)
    # 70 short sequences of two or three pages, more groups than CTAs: whole groups, two or three a CTA
    lengths = [70] * 35 + [170] * 35
    plans = plans_of(planner, lengths, 8, 4, 0, 284, 4, 128)
    parts, whole, uneven = check(plans, lengths, 8, 4, 0, 284, 4, 128)
    assert whole == 560 and uneven
    # places to spare beside long sequences (24 of 4,096 keys, 8 of one): equal runs with a cost for every group
    lengths = [4096] * 24 + [1] * 8
    plans = plans_of(planner, lengths, 8, 4, 0, 284, 4, 128)
    parts, whole, uneven = check(plans, lengths, 8, 4, 0, 284, 4, 128)
    assert not parts and not whole and int(plans[0, 6]) == GROUP_COST


def test_arguments_that_no_launch_has_are_refused(planner):
    out = np.zeros((4, 12), dtype=np.int32)
    seq = np.zeros(1, dtype=np.int32)
    o, s = out.ctypes.data_as(ctypes.c_void_p), seq.ctypes.data_as(ctypes.c_void_p)
    assert planner.dfi_decode_plan_host(o, s, 1, 1, 1, 0, 4, 3, 128) == -1        # no clusters of three
    assert planner.dfi_decode_plan_host(o, s, 0, 1, 1, 0, 4, 1, 128) == -1
    assert planner.dfi_decode_plan_host(None, s, 1, 1, 1, 0, 4, 1, 128) == -1
