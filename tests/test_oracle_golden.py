"""Pins the CPU oracle: known-answer vectors of Philox, the closed-form cases
of the reference's own collective tests replayed over in-process ranks, the
C restatement against the numpy one, and the committed fixtures."""
import ctypes
import os

import numpy as np
import pytest

from oracle import oracle as orc
from tests.helpers import feature_setup, small_graph

I64 = np.int64
GOLDEN = os.path.join(os.path.dirname(__file__), "golden")


def _p(a):
    return a.ctypes.data_as(ctypes.c_void_p)


# ------------------------------------------------------------------ Philox
@pytest.mark.parametrize("ctr,key,want", [
    ((0, 0, 0, 0), (0, 0), (0x6627E8D5, 0xE169C58D, 0xBC57AC4C, 0x9B00DBD8)),
    ((0xFFFFFFFF,) * 4, (0xFFFFFFFF,) * 2, (0x408F276D, 0x41C83B0E, 0xA20BC7C6, 0x6D5451FD)),
    ((0x243F6A88, 0x85A308D3, 0x13198A2E, 0x03707344), (0xA4093822, 0x299F31D0),
     (0xD16CFE09, 0x94FDCCEB, 0x5001E420, 0x24126EA1)),
])
def test_philox_known_answers(ctr, key, want, c_oracle):
    got = orc.philox4x32_10(*ctr, *key)
    assert tuple(int(x) for x in got) == want
    c = np.array(ctr, dtype=np.uint32)
    k = np.array(key, dtype=np.uint32)
    out = np.zeros(4, dtype=np.uint32)
    c_oracle.oracle_philox(_p(c), _p(k), _p(out))
    assert tuple(int(x) for x in out) == want


# ------------------------------------- the reference's collective test cases
@pytest.mark.parametrize("ws", [1, 2, 4, 8])
def test_alltoall_nccl1(ws):
    # tests/test_alltoall.cc:8-22: send arange(ws), offsets arange(1..ws) -> recv == rank
    arange = np.arange(1, ws + 1)
    out = orc.alltoall([np.arange(ws, dtype=I64)] * ws, [arange] * ws, [arange] * ws)
    for r in range(ws):
        assert np.array_equal(out[r], np.full(ws, r, dtype=I64))


@pytest.mark.parametrize("ws", [2, 4, 8])
@pytest.mark.parametrize("expand", [1, 16])
def test_alltoall_nccl2_and_3(ws, expand):
    # tests/test_alltoall.cc:24-99: size to r = 7(rank-r)^2+100, payload = rank
    k, b = 7, 100
    send_sizes = [[k * (rank - r) ** 2 + b for r in range(ws)] for rank in range(ws)]
    recv_sizes = [[k * (r - rank) ** 2 + b for r in range(ws)] for rank in range(ws)]
    send_off = [np.cumsum(s) for s in send_sizes]
    recv_off = [np.cumsum(s) for s in recv_sizes]
    inputs = [np.full(send_off[rank][-1] * expand, rank, dtype=I64) for rank in range(ws)]
    out = orc.alltoall(inputs, send_off, recv_off, expand=expand)
    for rank in range(ws):
        want = np.concatenate([np.full(recv_sizes[rank][r] * expand, r, dtype=I64) for r in range(ws)])
        assert np.array_equal(out[rank], want)


@pytest.mark.parametrize("ws", [1, 3, 8])
def test_allgather1(ws):
    # tests/test_allgather.cc:8-26
    out = orc.allgather([np.array([r, r * 10], dtype=I64) for r in range(ws)])
    want = np.array([x for r in range(ws) for x in (r, r * 10)], dtype=I64)
    assert all(np.array_equal(o, want) for o in out)


@pytest.mark.parametrize("ws", [2, 5])
def test_allbroadcast1(ws):
    # tests/test_allbroadcast.cc:8-32: rank r sends arange(r+1)
    out = orc.allbroadcast([np.arange(r + 1, dtype=I64) for r in range(ws)])
    want = np.concatenate([np.arange(r + 1, dtype=I64) for r in range(ws)])
    assert all(np.array_equal(o, want) for o in out)


@pytest.mark.parametrize("ws", [2, 4])
def test_allreduce1(ws):
    # tests/test_allreduce.cc:9-26: rank q contributes full(total, q); root r keeps r+1
    # elements, each the sum 0+1+...+(ws-1)
    sizes = [r + 1 for r in range(ws)]
    total = sum(sizes)
    out = orc.allreduce_scatter_v([np.full(total, q, dtype=I64) for q in range(ws)], sizes)
    for r in range(ws):
        assert np.array_equal(out[r], np.full(r + 1, ws * (ws - 1) // 2, dtype=I64))


@pytest.mark.parametrize("ws", [1, 2, 4, 8])
def test_shuffle_seeds1_inputs(ws):
    # tests/test_shuffle_seeds.cc:8-41: min_vids = 100*arange(ws+1), seeds = ws*arange(99)+rank.
    # The reference prints instead of asserting; the contract of src/sampling.cc:159-193 is checked.
    base = 100
    min_vids = base * np.arange(ws + 1)
    seeds = [ws * np.arange(base - 1, dtype=I64) + r for r in range(ws)]
    res = orc.shuffle_seeds(seeds, min_vids)
    for r in range(ws):
        recv, perm, recv_off, dev_off = res[r]
        assert np.all((recv >= min_vids[r]) & (recv < min_vids[r + 1]))
        sizes, offs, sorted_idx, perm2 = orc.bucket_by_owner(seeds[r], min_vids, ws, rank=r)
        assert np.array_equal(sorted_idx[perm], seeds[r]) and np.array_equal(perm, perm2)
        assert np.array_equal(dev_off, offs) and dev_off[-1] == base - 1
        # what r received from s is exactly what s bucketed for r, in s's order
        ro = np.concatenate([[0], recv_off])
        for s in range(ws):
            ssz, soff, ssorted, _ = orc.bucket_by_owner(seeds[s], min_vids, ws, rank=s)
            so = np.concatenate([[0], soff])
            assert np.array_equal(recv[ro[s]:ro[s + 1]], ssorted[so[r]:so[r + 1]])
    # every seed arrives exactly once
    got = np.sort(np.concatenate([res[r][0] for r in range(ws)]))
    assert np.array_equal(got, np.sort(np.concatenate(seeds)))


def test_shuffle_seeds2_inputs():
    # tests/test_shuffle_seeds.cc:43-58 (body commented out there): seeds =
    # cat(arange(ws).flip, arange(ws)), min_vids = arange(ws+1) -> every rank receives 2*ws copies of its id
    ws = 4
    seeds = [np.concatenate([np.arange(ws)[::-1], np.arange(ws)]).astype(I64)] * ws
    res = orc.shuffle_seeds(seeds, np.arange(ws + 1))
    for r in range(ws):
        assert np.array_equal(res[r][0], np.full(2 * ws, r, dtype=I64))


# ------------------------------------------------ numpy oracle vs C restatement
def test_sample_numpy_vs_c(c_oracle):
    n, indptr, indices = small_graph(scale=9)
    rng = np.random.default_rng(3)
    cached = rng.permutation(n)[: n // 4].astype(I64)
    adj = orc.build_adj_pos_map(n, cached)
    dev_indptr = np.concatenate([[0], np.cumsum(indptr[cached + 1] - indptr[cached])]).astype(I64)
    dev_indices = np.concatenate([indices[indptr[v]:indptr[v + 1]] for v in cached]).astype(I64)
    seeds = rng.integers(0, n, 700).astype(I64)
    for fanout in (5, 10, 25, 40):
        want = orc.sample_csc_fanout(seeds, fanout, adj, dev_indptr, dev_indices, indptr, indices, key=99, call_id=7)
        got = np.zeros(len(seeds) * fanout, dtype=I64)
        c_oracle.oracle_sample(_p(seeds), ctypes.c_int64(len(seeds)), fanout, _p(adj), _p(dev_indptr),
                               _p(dev_indices), _p(indptr), _p(indices), ctypes.c_uint64(99), ctypes.c_uint32(7),
                               _p(got))
        assert np.array_equal(got, want)
        # sampler invariant of the reference's debug hook (python/npc/sampler.py:126-130):
        # every (neighbour -> seed) pair is an edge of the graph
        for j in rng.integers(0, len(seeds), 50):
            row = indices[indptr[seeds[j]]:indptr[seeds[j] + 1]]
            assert np.isin(want[j * fanout:(j + 1) * fanout], row).all()
    # cached rows hold the same neighbours, so the map must not change the result
    plain = orc.sample_csc_fanout(seeds, 10, None, None, None, indptr, indices, key=99, call_id=7)
    mapped = orc.sample_csc_fanout(seeds, 10, adj, dev_indptr, dev_indices, indptr, indices, key=99, call_id=7)
    assert np.array_equal(plain, mapped)


def test_sample_without_replacement_properties():
    n, indptr, indices = small_graph(scale=9)
    rng = np.random.default_rng(5)
    seeds = rng.integers(0, n, 300).astype(I64)
    fanout = 10
    out = orc.sample_csc_fanout(seeds, fanout, None, None, None, indptr, indices, key=1, call_id=0,
                                replace=False).reshape(-1, fanout)
    for j, v in enumerate(seeds):
        row = indices[indptr[v]:indptr[v + 1]]
        assert np.isin(out[j], row).all()
        if len(row) > fanout and len(np.unique(row)) == len(row):
            assert len(np.unique(out[j])) == fanout
        if len(row) <= fanout:
            assert np.array_equal(out[j, :len(row)], row)


def test_relabel_numpy_vs_c(c_oracle):
    rng = np.random.default_rng(11)
    for S, f, hi in ((1, 1, 5), (100, 10, 300), (1024, 25, 5000), (50, 5, 1 << 40)):
        seeds = rng.permutation(min(hi, 10 ** 6))[:S].astype(I64) if hi < 10 ** 7 else rng.integers(0, hi, S).astype(I64)
        nbrs = rng.integers(0, hi, S * f).astype(I64)
        uniq, rel = orc.relabel_csc(seeds, nbrs)
        cu = np.zeros(S + S * f, dtype=I64)
        cr = np.zeros(S * f, dtype=I64)
        c_oracle.oracle_relabel.restype = ctypes.c_int64
        U = c_oracle.oracle_relabel(_p(seeds), ctypes.c_int64(S), _p(nbrs), ctypes.c_int64(S * f), _p(cu), _p(cr))
        assert U == len(uniq) and np.array_equal(cu[:U], uniq) and np.array_equal(cr, rel)
        assert np.array_equal(uniq[rel], nbrs)
        if len(np.unique(seeds)) == S:
            assert np.array_equal(uniq[:S], seeds)  # dst nodes are the first src nodes


def test_relabel_empty_and_duplicate_seeds():
    uniq, rel = orc.relabel_csc(np.array([], dtype=I64), np.array([], dtype=I64))
    assert len(uniq) == 0 and len(rel) == 0
    uniq, rel = orc.relabel_csc(np.array([5, 5, 3], dtype=I64), np.array([3, 9, 5, 9], dtype=I64))
    assert uniq.tolist() == [5, 3, 9] and rel.tolist() == [1, 2, 0, 2]


def test_bucket_and_unique_numpy_vs_c(c_oracle):
    rng = np.random.default_rng(13)
    for ws in (1, 2, 8, 32):
        n_nodes = 10000
        cuts = np.sort(rng.choice(np.arange(1, n_nodes), ws - 1, replace=False)) if ws > 1 else np.array([], dtype=I64)
        mv = np.concatenate([[0], cuts, [n_nodes]]).astype(I64)
        ids = rng.integers(0, n_nodes, 5000).astype(I64)
        sizes, offs, sorted_idx, perm = orc.bucket_by_owner(ids, mv, ws, rank=0)
        cs, cp = np.zeros(len(ids), dtype=I64), np.zeros(len(ids), dtype=I64)
        csz, cof = np.zeros(ws, dtype=I64), np.zeros(ws, dtype=I64)
        c_oracle.oracle_bucket(_p(ids), ctypes.c_int64(len(ids)), _p(mv), ws, ctypes.c_int64(0), 0, 0, ws,
                               _p(cs), _p(cp), _p(csz), _p(cof))
        assert np.array_equal(cs, sorted_idx) and np.array_equal(cp, perm)
        assert np.array_equal(csz, sizes) and np.array_equal(cof, offs)
        u, inv = orc.unique_sorted(ids)
        cu, ci = np.zeros(len(ids), dtype=I64), np.zeros(len(ids), dtype=I64)
        c_oracle.oracle_unique_sorted.restype = ctypes.c_int64
        U = c_oracle.oracle_unique_sorted(_p(ids), ctypes.c_int64(len(ids)), _p(cu), _p(ci))
        assert U == len(u) and np.array_equal(cu[:U], u) and np.array_equal(ci, inv)


def test_owner_multi_machine_remap():
    # src/cuda/npc_kernel.cu:340-342: owners outside [node_beg, node_end) fall back to the caller
    mv = np.array([0, 10, 20, 30, 40])
    ids = np.array([1, 11, 21, 31, 39, 45])
    assert orc.owner_of(ids, mv, 4, rank=2, node_beg=2, node_end=4).tolist() == [2, 2, 2, 3, 3, 3]
    assert orc.owner_of(ids, mv, 4).tolist() == [0, 1, 2, 3, 3, 3]


def test_gather_numpy_vs_c_and_cpu_twin(c_oracle):
    rng = np.random.default_rng(17)
    n, dim = 2000, 24
    feats, uva, dev, cached_idx, local_idx, pos_map, cpu_map = feature_setup(n, dim, 0.3, rng)
    ids = rng.integers(0, n, 3000).astype(I64)
    out = orc.load_subtensor(ids, pos_map, dev, uva)
    assert np.array_equal(out, feats[ids])
    # the reference's own CPU op (src/load_subtensor.cc:10-17) reads the host table only
    assert np.array_equal(orc.cpu_load_subtensor(ids, cpu_map, uva), feats[ids])
    got = np.zeros_like(out)
    c_oracle.oracle_gather(_p(ids), ctypes.c_int64(len(ids)), _p(pos_map), _p(dev), ctypes.c_int64(dim * 4),
                           _p(uva), ctypes.c_int64(dim * 4), ctypes.c_int64(0), _p(got))
    assert np.array_equal(got, out)
    # model-parallel column window (feat_dim_offset, src/cuda/npc_kernel.cu:199-201)
    dev_w = np.ascontiguousarray(dev[:, 8:16])
    out_w = orc.load_subtensor(ids, pos_map, dev_w, uva, feat_dim_offset=8)
    assert np.array_equal(out_w, feats[ids][:, 8:16])


def test_feat_shuffle_round_trip():
    # fwd returns rows in the asker's seed order; bwd is its transpose
    rng = np.random.default_rng(19)
    ws, D, n_nodes = 4, 6, 400
    mv = np.linspace(0, n_nodes, ws + 1).astype(I64)
    seeds = [rng.integers(0, n_nodes, 50 + 10 * r).astype(I64) for r in range(ws)]
    table = rng.standard_normal((n_nodes, D)).astype(np.float32)
    res = orc.shuffle_seeds(seeds, mv)
    # owner side: the row of every received id, in receive order
    inputs = [table[res[r][0]] for r in range(ws)]
    send_off = [res[r][2] for r in range(ws)]   # python send_offset = C++ recv_offset (python/npc/sampler.py:147)
    recv_off = [res[r][3] for r in range(ws)]
    perms = [res[r][1] for r in range(ws)]
    out = orc.feat_shuffle(inputs, send_off, recv_off, perms, D, fwd=True)
    for r in range(ws):
        assert np.array_equal(out[r], table[seeds[r]])
    grads = [rng.standard_normal(o.shape).astype(np.float32) for o in out]
    back = orc.feat_shuffle(grads, recv_off, send_off, perms, D, fwd=False)
    # <fwd(x), g> == <x, bwd(g)>
    lhs = sum(float((out[r].astype(np.float64) * grads[r]).sum()) for r in range(ws))
    rhs = sum(float((inputs[r].astype(np.float64) * back[r]).sum()) for r in range(ws))
    assert abs(lhs - rhs) < 1e-6 * max(1.0, abs(lhs))


def test_spmm_sddmm_numpy_vs_c(c_oracle):
    rng = np.random.default_rng(23)
    S, f, D = 64, 5, 12
    n_src = 200
    row = rng.integers(0, n_src, S * f).astype(I64)
    col = np.repeat(np.arange(S, dtype=I64), f)
    x = rng.standard_normal((n_src, D)).astype(np.float32)
    coo, ioff, ooff = np.array([0, S * f], dtype=I64), np.array([0, n_src], dtype=I64), np.array([0, S], dtype=I64)
    want = orc.spmm_sum("copy_u", row, col, x, None, coo, ioff, ooff)
    got = np.zeros((S, D), dtype=np.float32)
    c_oracle.oracle_spmm_copy_u(_p(row), _p(col), ctypes.c_int64(S * f), _p(x), ctypes.c_int64(D), _p(coo),
                                _p(ioff), _p(ooff), 1, _p(got))
    assert np.allclose(got, want, rtol=1e-5, atol=1e-6)
    assert np.allclose(want, x[row].reshape(S, f, D).astype(np.float64).sum(1))
    y = rng.standard_normal((S, D)).astype(np.float32)
    for mul, name in ((0, "u_add_v"), (1, "u_mul_v")):
        want = orc.sddmm(name, row, col, x, y, coo, ioff, ooff, acc=np.float32)
        got = np.zeros((S * f, D), dtype=np.float32)
        c_oracle.oracle_sddmm(mul, _p(row), _p(col), ctypes.c_int64(S * f), _p(x), _p(y), ctypes.c_int64(D), _p(coo),
                              _p(ioff), _p(ooff), 1, _p(got))
        assert np.array_equal(got, want)
    # the reference's UMulESum kernel adds (src/cuda/spmm.cu:78); the operator's meaning is multiply
    e = rng.standard_normal((S * f, D)).astype(np.float32)
    mul_ = orc.spmm_sum("u_mul_e", row, col, x, e, coo, ioff, ooff)
    add_ = orc.spmm_sum("u_add_e", row, col, x, e, coo, ioff, ooff)
    assert np.allclose(mul_, (x[row].astype(np.float64) * e).reshape(S, f, D).sum(1))
    assert np.allclose(add_, (x[row].astype(np.float64) + e).reshape(S, f, D).sum(1))


def test_spmm_segments():
    # two segments with their own row bases (src/cuda/spmm.cu:20-24)
    x = np.arange(12, dtype=np.float32).reshape(6, 2)
    row = np.array([0, 1, 2, 0, 1], dtype=I64)
    col = np.array([0, 0, 1, 0, 0], dtype=I64)
    out = orc.spmm_sum("copy_u", row, col, x, None, [0, 3, 5], [0, 3, 6], [0, 2, 3])
    assert np.array_equal(out, np.array([x[0] + x[1], x[2], x[3] + x[4]], dtype=np.float64))


# ------------------------------------------------------------ committed fixtures
@pytest.mark.parametrize("ws", [1, 2, 3, 8])
@pytest.mark.parametrize("with_dst", [False, True])
def test_virtual_node_path_adds_up(ws, with_dst):
    # SNP with virtual nodes: the partial sums per virtual node, sent back, add up to the direct
    # neighbour sums; sizes are consistent between the ranks; every received virtual node names
    # its sender (python/npc/sampler.py:240-330, src/sampling.cc:71-149)
    n, indptr, indices = small_graph(scale=10, edge_factor=8)
    graph = (None, None, None, indptr, indices)
    mv = np.linspace(0, n, ws + 1).astype(I64)
    rng = np.random.default_rng(ws)
    seeds = [rng.integers(0, n, 40 + 9 * r).astype(I64) for r in range(ws)]
    f, k = 5, (3 if with_dst else 2)
    res = orc.sp_virtual_sample(seeds, f, mv, graph, key=1, call_id=2, num_total_nodes=n, with_dst=with_dst)
    x = rng.standard_normal((n, 4))
    inputs = []
    for r, p in enumerate(res):
        assert np.array_equal(orc.owner_of(p["ori_src"], mv, ws), np.full(len(p["ori_src"]), r))
        assert np.array_equal(np.sort(p["vir_src"] // 10_000_000, kind="stable"), p["vir_src"] // 10_000_000)
        for q in range(ws):
            assert np.array_equal(p["recv_sizes"][k * q:k * q + k], res[q]["send_sizes"][k * r:k * r + k])
        assert p["send_sizes"][k - 2::k].sum() == len(seeds[r]) * f
        assert p["send_sizes"][k - 1::k].sum() == len(p["unique_frontier"])
        assert p["recv_sizes"][k - 1::k].sum() == len(p["unique_dst"])
        h = np.zeros((len(p["unique_dst"]), 4))
        np.add.at(h, p["block2_dst"], x[p["unique_src"]][p["block2_src"]])
        inputs.append(np.concatenate([x[p["recv_dst"]], h]) if with_dst else h)
    got = orc.sp_feat_shuffle(inputs, [p["recv_sizes"] for p in res], [p["send_sizes"] for p in res], with_dst)
    for r, p in enumerate(res):
        g, nd = got[r], len(seeds[r])
        if with_dst:
            assert np.allclose(g[:nd], x[seeds[r][p["perm"][:nd]]])
            g = g[nd:]
        out = np.zeros((nd, 4))
        np.add.at(out, p["block1_dst"], g)
        assert np.allclose(out, x[p["neighbors"]].reshape(nd, f, 4).sum(1))


def test_virtual_send_offsets_closed_form():
    # 2 ranks, 3 destinations, fanout 2: owners of the neighbours 0 1 | 1 1 | 0 0
    mv = np.array([0, 10, 20], dtype=I64)
    src = np.array([1, 11, 12, 13, 2, 3], dtype=I64)
    m = orc.src_to_vir(src, 2, 3, mv, 2)
    assert m.tolist() == [0, 3, 4, 4, 2, 2]
    s, u = np.sort(m), np.unique(m)
    assert orc.vir_send_offset(2, 3, s, u, False).tolist() == [0, 3, 6, 2, 4]
    assert orc.vir_send_sizes(2, 3, s, u, False).tolist() == [3, 2, 3, 2]
    dst = np.array([15, 5, 6], dtype=I64)
    md = orc.srcdst_to_vir(dst, src, 2, mv, 2)
    assert md.tolist() == [3, 1, 2, 6, 9, 10, 10, 8, 8]
    sd = np.sort(md)
    ud = np.unique(sd[3:])
    assert orc.vir_send_offset(2, 3, sd, ud, True).tolist() == [0, 2, 3, 6, 9, 2, 4]
    assert orc.vir_send_sizes(2, 3, sd, ud, True).tolist() == [2, 3, 2, 1, 3, 2]


@pytest.mark.parametrize("ws", [1, 2, 4])
def test_nfp_path_adds_up(ws):
    # NFP: every rank holds a slice of the columns; the multi-segment aggregation of all ranks'
    # blocks followed by the reduce-scatter gives every rank the full-width neighbour sums of its
    # own seeds (python/npc/sampler.py:332-356, python/npc/model/sageconv.py:117-188)
    n, indptr, indices = small_graph(scale=10, edge_factor=8)
    graph = (None, None, None, indptr, indices)
    rng = np.random.default_rng(40 + ws)
    seeds = [rng.permutation(n)[:30 + 11 * r].astype(I64) for r in range(ws)]
    f, width = 4, 3
    res = orc.mp_sample(seeds, f, graph, key=9, call_id=1)
    x = rng.standard_normal((n, ws * width))
    w = rng.standard_normal((ws * width, 5))                # the layer's weight, rows split like the columns
    partial = []
    for r, p in enumerate(res):
        fo = np.concatenate([[0], np.cumsum(p["recv_frontier_size"])])
        co = np.concatenate([[0], np.cumsum(p["recv_coo_size"])])
        so = np.concatenate([[0], np.cumsum(p["recv_size"])])
        assert p["send_size"][0] == len(seeds[r]) and co[-1] == len(p["all_coo_row"]) == len(p["all_coo_col"])
        xs = x[p["all_frontier"], r * width:(r + 1) * width] @ w[r * width:(r + 1) * width]
        partial.append(orc.spmm_sum("copy_u", p["all_coo_row"], p["all_coo_col"], xs, None, co, fo, so))
    got = orc.mp_feat_shuffle_fwd(partial, res[0]["recv_size"], 5)
    for r in range(ws):
        want = (x[res[r]["neighbors"]] @ w).reshape(len(seeds[r]), f, 5).sum(1)
        assert np.allclose(got[r], want)
    back = orc.mp_feat_shuffle_bwd([g.astype(np.float32) for g in got], 5)
    for r in range(ws):
        assert np.array_equal(back[r], np.concatenate(got).astype(np.float32))


def test_cost_model_arithmetic_closed_form():
    # get_cache_miss (python/npc/cost_model/estimator.py:22-30) and the volume formulas (:129-188)
    freq = np.array([5, 0, 9, 9, 1], dtype=np.int32)
    assert orc.hot_order(freq).tolist() == [2, 3, 0, 4, 1]
    assert orc.get_cache_miss(freq, 0, 10) == 240 and orc.get_cache_miss(freq, 2, 10) == 60
    assert orc.get_cache_miss(freq, 99, 10) == 0
    assert orc.get_cache_miss(freq, 1, 10, made_seeds_freq=np.array([0, 7, 0, 0, 0])) == 240
    # rank 1 of 3: sends 4 + 6 rows to the others, receives 1 + 2
    assert orc.np_reshuffle_vol(3, 1, [4, 9, 15], [1, 8, 10], 256) == 2 * 256 * (10 + 3)
    assert orc.sp_reshuffle_vol(2, 0, [7, 3, 9, 4], [1, 2, 5, 6], 8) == 2 * 8 * (4 + 6)
    assert orc.sp_reshuffle_vol(2, 1, [1, 7, 3, 2, 9, 4], [1, 1, 2, 3, 5, 6], 8, with_dst=True) == 2 * 8 * (1 + 3 + 1 + 2)
    assert orc.mp_reshuffle_vol(4, [10], [10, 20, 30, 40], 16) == 2 * 16 * (10 * 2 + 100)
    assert orc.vol_to_seconds(1024 * 1024, 4.0) == 1.0


def test_committed_fixture_matches_oracle():
    z = np.load(os.path.join(GOLDEN, "path_small.npz"))
    indptr, indices = z["indptr"], z["indices"]
    nbr = orc.sample_csc_fanout(z["seeds"], int(z["fanout"]), None, None, None, indptr, indices,
                                key=int(z["key"]), call_id=int(z["call_id"]))
    assert np.array_equal(nbr, z["neighbors"])
    uniq, rel = orc.relabel_csc(z["seeds"], z["neighbors"])
    assert np.array_equal(uniq, z["unique"]) and np.array_equal(rel, z["relabeled"])
    sizes, offs, sorted_idx, perm = orc.bucket_by_owner(z["unique"], z["min_vids"], int(z["world_size"]), rank=1)
    assert np.array_equal(sorted_idx, z["sorted_idx"]) and np.array_equal(perm, z["permutation"])
    assert np.array_equal(offs, z["bucket_offsets"])
    src, dst = orc.rmat_edges(int(z["graph_seed"]), 0, int(z["num_edges"]), int(z["scale"]), int(z["num_nodes"]))
    ip, ix = orc.csc_from_edges(src, dst, int(z["num_nodes"]))
    assert np.array_equal(ip, indptr) and np.array_equal(ix, indices)


def test_committed_strategy_fixture_matches_oracle():
    # tests/golden/strategies_small.npz (tests/golden/make_golden.py): SNP with virtual nodes and NFP
    # on the fixture graph for one and two ranks; the oracle must still produce every array
    import importlib.util
    spec = importlib.util.spec_from_file_location("make_golden", os.path.join(GOLDEN, "make_golden.py"))
    mg = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mg)
    z = np.load(os.path.join(GOLDEN, "path_small.npz"))
    want = np.load(os.path.join(GOLDEN, "strategies_small.npz"))
    got = mg.strategy_cases(z["indptr"], z["indices"], int(z["num_nodes"]))
    assert sorted(got) == sorted(want.files)
    for k in want.files:
        assert np.array_equal(got[k], want[k]), k
