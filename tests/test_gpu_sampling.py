"""GPU parity of sampling, relabelling, owner bucketing and sorted unique
against the CPU oracle (bit-exact), through the operator layer over the C ABI."""
import os

import numpy as np
import pytest
import torch

import apt_b200
from apt_b200 import ops
from apt_b200._lib import check, lib
from oracle import oracle as orc
from tests.gpu_util import dev, host, install_graph, reset_world
from tests.helpers import small_graph

pytestmark = pytest.mark.gpu
I64 = np.int64
GOLDEN = os.path.join(os.path.dirname(__file__), "golden")


@pytest.fixture(scope="module")
def graph():
    n, indptr, indices = small_graph(scale=12, edge_factor=8)
    # a few isolated nodes: rebuild without self loops for the last 16 ids
    keep = ~np.isin(np.repeat(np.arange(n), np.diff(indptr)), np.arange(n - 16, n))
    indices2 = indices[keep]
    deg = np.diff(indptr).copy()
    deg[n - 16:] = 0
    indptr2 = np.concatenate([[0], np.cumsum(deg)]).astype(I64)
    return n, indptr2, indices2


@pytest.mark.parametrize("fanout", [1, 5, 10, 15, 25, 40])
@pytest.mark.parametrize("layout", ["hbm", "cached", "pinned"])
def test_sample_matches_oracle(graph, fanout, layout):
    n, indptr, indices = graph
    rng = np.random.default_rng(fanout)
    cached = rng.permutation(n)[: n // 3].astype(I64) if layout == "cached" else None
    dip, dix = install_graph(indptr, indices, cached, pinned_host=(layout == "pinned"))
    adj = orc.build_adj_pos_map(n, cached) if cached is not None else None
    seeds = rng.integers(0, n - 16, 3000).astype(I64)
    ops.set_sampling(key=1234567, call_id=11, replace=True)
    got_seeds, nbr = ops.local_sample_one_layer(dev(seeds), fanout)
    want = orc.sample_csc_fanout(seeds, fanout, adj, dip, dix, indptr, indices, key=1234567, call_id=11)
    assert got_seeds.data_ptr() == got_seeds.data_ptr() and np.array_equal(host(got_seeds), seeds)
    assert np.array_equal(host(nbr), want)
    ops.check_status()
    # the next call uses the next call id
    _, nbr2 = ops.local_sample_one_layer(dev(seeds), fanout)
    assert np.array_equal(host(nbr2), orc.sample_csc_fanout(seeds, fanout, adj, dip, dix, indptr, indices,
                                                            key=1234567, call_id=12))


def test_sample_zero_degree_and_empty(graph):
    n, indptr, indices = graph
    install_graph(indptr, indices)
    seeds = np.array([n - 1, 5, n - 3], dtype=I64)
    ops.set_sampling(key=5, call_id=0)
    _, nbr = ops.local_sample_one_layer(dev(seeds), 4)
    want = orc.sample_csc_fanout(seeds, 4, None, None, None, indptr, indices, key=5, call_id=0)
    assert np.array_equal(host(nbr), want)
    assert host(nbr)[:4].tolist() == [n - 1] * 4
    ops.check_status()  # zero degree is a notice, not an error
    _, e = ops.local_sample_one_layer(torch.empty(0, dtype=torch.int64, device="cuda"), 7)
    assert e.numel() == 0


def test_sample_out_of_range_id_is_flagged(graph):
    n, indptr, indices = graph
    install_graph(indptr, indices)
    ops.local_sample_one_layer(dev(np.array([3, n + 5], dtype=I64)), 3)
    with pytest.raises(RuntimeError, match="outside the registered tables"):
        ops.check_status()
    ops.check_status()  # cleared


@pytest.mark.parametrize("fanout", [3, 10, 32])
def test_sample_without_replacement(graph, fanout):
    n, indptr, indices = graph
    install_graph(indptr, indices)
    rng = np.random.default_rng(2)
    seeds = rng.integers(0, n, 2000).astype(I64)
    ops.set_sampling(key=77, call_id=0, replace=False)
    try:
        _, nbr = ops.local_sample_one_layer(dev(seeds), fanout)
    finally:
        ops.set_sampling(replace=True)
    want = orc.sample_csc_fanout(seeds, fanout, None, None, None, indptr, indices, key=77, call_id=0, replace=False)
    assert np.array_equal(host(nbr), want)


def test_sample_uniformity_chi_square(graph):
    # with replacement every edge slot of a node is equally likely (src/cuda/npc_kernel.cu:280)
    n, indptr, indices = graph
    install_graph(indptr, indices)
    deg = np.diff(indptr)
    v = int(np.argmax(deg == 16)) if (deg == 16).any() else int(np.argmax(deg))
    d = int(deg[v])
    ops.set_sampling(key=42, call_id=0)
    reps = 4000
    _, nbr = ops.local_sample_one_layer(dev(np.full(reps, v, dtype=I64)), 25)
    row = indices[indptr[v]:indptr[v + 1]]
    ids, counts = np.unique(host(nbr), return_counts=True)
    assert np.isin(ids, row).all()
    mult = np.array([np.sum(row == i) for i in ids])
    expected = reps * 25 * mult / d
    chi2 = float(((counts - expected) ** 2 / expected).sum())
    assert chi2 < 3.0 * len(ids) + 30


@pytest.mark.parametrize("S,f,hi", [(1, 1, 5), (100, 10, 300), (1024, 25, 5000), (3000, 15, 1 << 40), (4096, 10, 64)])
def test_relabel_matches_oracle(S, f, hi):
    rng = np.random.default_rng(S + f)
    seeds = rng.integers(0, hi, S).astype(I64)
    nbrs = rng.integers(0, hi, S * f).astype(I64)
    uniq, rel = ops.relabel_csc(dev(seeds), dev(nbrs))
    wu, wr = orc.relabel_csc(seeds, nbrs)
    assert np.array_equal(host(uniq), wu) and np.array_equal(host(rel), wr)


@pytest.mark.parametrize("S,f", [(1, 1), (1024, 5), (1024, 7), (1170, 6), (1171, 6), (3000, 1)])
def test_relabel_one_block_path_equals_multi_block_path(S, f):
    # layers of up to 8192 items run in one block with the table in shared memory; the same
    # call with that path switched off must give the same arrays (8190 and 8197 items straddle the limit)
    rng = np.random.default_rng(S * 31 + f)
    seeds = dev(rng.integers(0, 4000, S).astype(I64))
    nbrs = dev(rng.integers(0, 4000, S * f).astype(I64))
    outs = []
    for small in (1, 0):
        check(lib.apt_set_tunable(b"relabel_small", small))
        try:
            outs.append(ops.relabel_csc(seeds, nbrs))
        finally:
            check(lib.apt_set_tunable(b"relabel_small", 1))
    assert torch.equal(outs[0][0], outs[1][0]) and torch.equal(outs[0][1], outs[1][1])
    wu, wr = orc.relabel_csc(host(seeds), host(nbrs))
    assert np.array_equal(host(outs[0][0]), wu) and np.array_equal(host(outs[0][1]), wr)
    ops.check_status()


def test_relabel_edge_cases():
    e = torch.empty(0, dtype=torch.int64, device="cuda")
    uniq, rel = ops.relabel_csc(e, e)
    assert uniq.numel() == 0 and rel.numel() == 0
    uniq, rel = ops.relabel_csc(dev(np.array([5, 5, 3], dtype=I64)), dev(np.array([3, 9, 5, 9], dtype=I64)))
    assert host(uniq).tolist() == [5, 3, 9] and host(rel).tolist() == [1, 2, 0, 2]
    uniq, rel = ops.relabel_csc(dev(np.array([7, 8], dtype=I64)), e)
    assert host(uniq).tolist() == [7, 8] and rel.numel() == 0


def test_relabel_full_size_properties():
    # outer hop of the papers-shaped run: 67 584 seeds x fanout 15 (about 1.08 M items)
    rng = np.random.default_rng(9)
    S, f, N = 67584, 15, 111_000_000
    seeds = rng.choice(N, S, replace=False).astype(I64)
    z = rng.zipf(1.3, S * f)
    nbrs = (z % N).astype(I64)
    uniq, rel = ops.relabel_csc(dev(seeds), dev(nbrs))
    u, r = host(uniq), host(rel)
    assert np.array_equal(u[r], nbrs)                     # relabel inverts through unique
    assert np.array_equal(u[:S], seeds)                   # dst nodes first, in order
    assert len(np.unique(u)) == len(u) == len(np.unique(np.concatenate([seeds, nbrs])))
    # first-occurrence order: among ids that are not seeds, a smaller new id is first used earlier
    ids, first_pos = np.unique(r, return_index=True)
    fp = first_pos[ids >= S]
    assert np.all(np.diff(fp) > 0)


@pytest.mark.parametrize("n_items", [2048, 2049, 10_000, 300_000])
def test_relabel_many_tiles_repeated_calls(n_items):
    # the ordered compaction hands tiles of 2048 items out by ticket and chains their counts;
    # repeated calls on one workspace reuse the tile states (tagged by call) without clearing
    rng = np.random.default_rng(n_items)
    lib.apt_set_tunable(b"relabel_small", 0)
    try:
        for rep in range(4):
            S = max(1, n_items // 11)
            seeds = rng.choice(10 * n_items, S, replace=False).astype(I64)
            nbrs = rng.integers(0, 3 * n_items, n_items - S).astype(I64)
            uniq, rel = ops.relabel_csc(dev(seeds), dev(nbrs))
            wu, wr = orc.relabel_csc(seeds, nbrs)
            assert np.array_equal(host(uniq), wu) and np.array_equal(host(rel), wr)
    finally:
        lib.apt_set_tunable(b"relabel_small", 1)


@pytest.mark.parametrize("small", [1, 0])
def test_relabel_negative_id_is_not_an_id(small):
    # -1 is what an operator upstream leaves for an id it could not resolve (and the bit pattern of an
    # empty table slot): it gets no new id, is relabelled to -1 and raises the out-of-range flag
    seeds = np.array([7, 3, 9], dtype=I64)
    nbrs = np.array([3, -1, 11, 7, -5, 11, -1, 2], dtype=I64)
    lib.apt_set_tunable(b"relabel_small", small)
    try:
        uniq, rel = ops._relabel_enqueue(dev(seeds), dev(nbrs), None, ops.STATE.word(0))
        with pytest.raises(RuntimeError, match="id outside"):
            ops.check_status()
        n = int(ops.STATE.words()[0].item())
    finally:
        lib.apt_set_tunable(b"relabel_small", 1)
    assert host(uniq)[:n].tolist() == [7, 3, 9, 11, 2]
    assert host(rel).tolist() == [1, -1, 3, 0, -1, 3, -1, 4]
    # the table is empty again: the next call is not disturbed
    u2, r2 = ops.relabel_csc(dev(seeds), dev(np.array([9, 2, 2], dtype=I64)))
    assert host(u2).tolist() == [7, 3, 9, 2] and host(r2).tolist() == [2, 3, 3]


@pytest.mark.parametrize("S,fanout", [(64, 5), (1024, 5), (1200, 10), (6000, 10), (40000, 15)])
@pytest.mark.parametrize("dev_count", [False, True])
def test_sample_and_relabel_in_one_call_equals_the_two_calls(graph, S, fanout, dev_count):
    # apt_sample_relabel_csc (the sampling kernel enters its ids into the relabel table itself; layers of
    # up to 8192 items are one launch) against sampling, then relabelling, then the oracle
    n, indptr, indices = graph
    install_graph(indptr, indices)
    rng = np.random.default_rng(S + fanout)
    seeds = rng.choice(n, min(S, n), replace=False).astype(I64)
    S = len(seeds)
    buf = np.concatenate([seeds, rng.integers(0, n, 50).astype(I64)])    # the buffer is an upper bound
    n_dev = torch.tensor([S], dtype=torch.int64, device="cuda") if dev_count else None
    src = dev(buf) if dev_count else dev(seeds)
    ops.set_sampling(key=31337, call_id=5)
    uniq, rel, nbr = ops._sample_relabel_enqueue(src, fanout, n_dev, ops.STATE.word(3), want_neighbors=True)
    ops.check_status()
    nu = int(ops.STATE.words()[3].item())
    want_nbr = orc.sample_csc_fanout(seeds, fanout, None, None, None, indptr, indices, key=31337, call_id=5)
    wu, wr = orc.relabel_csc(seeds, want_nbr)
    assert np.array_equal(host(nbr)[:S * fanout], want_nbr)
    assert nu == len(wu) and np.array_equal(host(uniq)[:nu], wu)
    assert np.array_equal(host(rel)[:S * fanout], wr)
    # without the neighbour list (what the chained samplers ask for)
    ops.set_sampling(key=31337, call_id=5)
    uniq2, rel2, none = ops._sample_relabel_enqueue(src, fanout, n_dev, ops.STATE.word(4))
    ops.check_status()
    assert none is None and int(ops.STATE.words()[4].item()) == nu
    assert torch.equal(uniq2[:nu], uniq[:nu]) and torch.equal(rel2[:S * fanout], rel[:S * fanout])


@pytest.mark.parametrize("ws", [1, 2, 8, 32])
@pytest.mark.parametrize("n_ids", [0, 1, 1000, 70000])
def test_bucket_matches_oracle(ws, n_ids):
    rng = np.random.default_rng(ws * 7 + n_ids)
    N = 100000
    cuts = np.sort(rng.choice(np.arange(1, N), ws - 1, replace=False)) if ws > 1 else np.array([], dtype=I64)
    mv = np.concatenate([[0], cuts, [N]]).astype(I64)
    ids = rng.integers(0, N, n_ids).astype(I64)
    rank = ws // 2
    reset_world(ws, rank)
    try:
        ops.register_min_vids(torch.from_numpy(mv))
        sorted_ids, perm, sizes, offsets = ops._bucket(dev(ids))
    finally:
        reset_world()
    wsz, wof, wsorted, wperm = orc.bucket_by_owner(ids, mv, ws, rank=rank)
    assert np.array_equal(host(sizes)[:ws], wsz) and np.array_equal(host(offsets), wof)
    assert int(host(sizes)[ws]) == n_ids              # the total follows the sizes
    assert np.array_equal(host(sorted_ids), wsorted) and np.array_equal(host(perm), wperm)


def test_bucket_machine_window_remap():
    ws, rank, node_size = 8, 5, 4
    mv = (np.arange(ws + 1) * 1000).astype(I64)
    ids = np.random.default_rng(1).integers(0, 8000, 5000).astype(I64)
    s = apt_b200.STATE
    reset_world(ws, rank)
    s.node_size = node_size
    try:
        ops.register_min_vids(torch.from_numpy(mv))
        sorted_ids, perm, sizes, offsets = ops._bucket(dev(ids))
    finally:
        reset_world()
    wsz, wof, wsorted, wperm = orc.bucket_by_owner(ids, mv, ws, rank=rank, node_beg=4, node_end=8)
    assert host(sizes)[:4].sum() == 0
    assert np.array_equal(host(sizes)[:ws], wsz) and np.array_equal(host(sorted_ids), wsorted)
    assert np.array_equal(host(perm), wperm)


@pytest.mark.parametrize("n_ids,lo,hi", [(0, 0, 100), (1, 0, 1), (5000, 0, 3000), (70000, 1000, 14_000_000), (300000, 0, 111_000_000)])
def test_unique_sorted_matches_oracle(n_ids, lo, hi):
    rng = np.random.default_rng(n_ids)
    ids = (lo + rng.zipf(1.2, n_ids) % (hi - lo)).astype(I64) if n_ids else np.array([], dtype=I64)
    uniq, inv = ops.unique_sorted(dev(ids), lo, hi)
    wu, wi = orc.unique_sorted(ids)
    assert np.array_equal(host(uniq), wu) and np.array_equal(host(inv), wi)


def test_unique_sorted_alternating_ranges_share_one_workspace():
    rng = np.random.default_rng(77)
    for lo, hi in ((0, 5000), (0, 9000), (100, 4100), (0, 9000), (0, 5000)):
        ids = rng.integers(lo, hi, 3000).astype(I64)
        uniq, inv = ops.unique_sorted(dev(ids), lo, hi)
        wu, wi = orc.unique_sorted(ids)
        assert np.array_equal(host(uniq), wu) and np.array_equal(host(inv), wi)


def test_committed_fixture_on_gpu():
    z = np.load(os.path.join(GOLDEN, "path_small.npz"))
    install_graph(z["indptr"], z["indices"])
    ops.set_sampling(key=int(z["key"]), call_id=int(z["call_id"]))
    _, nbr = ops.local_sample_one_layer(dev(z["seeds"]), int(z["fanout"]))
    assert np.array_equal(host(nbr), z["neighbors"])
    uniq, rel = ops.relabel_csc(dev(z["seeds"]), nbr)
    assert np.array_equal(host(uniq), z["unique"]) and np.array_equal(host(rel), z["relabeled"])
    reset_world(int(z["world_size"]), 1)
    try:
        ops.register_min_vids(torch.from_numpy(z["min_vids"]))
        sorted_ids, perm, sizes, offsets = ops._bucket(uniq)
    finally:
        reset_world()
    assert np.array_equal(host(sorted_ids), z["sorted_idx"]) and np.array_equal(host(perm), z["permutation"])
    assert np.array_equal(host(offsets), z["bucket_offsets"])
