"""The GPU-side generators of the synthetic workloads against the CPU oracle
(R-MAT edges bit-exact), and structural checks of what the benchmark installs."""
import ctypes

import numpy as np
import pytest
import torch

import apt_b200
from apt_b200 import _lib, ops, synthetic
from apt_b200._lib import check, lib
from oracle import oracle as orc
from tests.gpu_util import host

pytestmark = pytest.mark.gpu
I64 = np.int64


@pytest.mark.parametrize("scale,n,first,m", [(10, 1 << 10, 0, 5000), (12, 3000, 777, 20000), (17, 100000, 0, 30000)])
def test_rmat_edges_match_oracle(scale, n, first, m):
    src = torch.empty(m, dtype=torch.int64, device="cuda")
    dst = torch.empty(m, dtype=torch.int64, device="cuda")
    check(lib.apt_rmat_edges(5, first, m, scale, n, 0.57, 0.19, 0.19, src.data_ptr(), dst.data_ptr(), None))
    ws, wd = orc.rmat_edges(5, first, m, scale, n)
    assert np.array_equal(host(src), ws) and np.array_equal(host(dst), wd)
    assert host(src).max() < n and host(dst).max() < n


def test_sort_u64_and_normal_rows():
    g = torch.Generator(device="cuda").manual_seed(0)
    keys = torch.randint(0, 1 << 40, (100003,), generator=g, device="cuda")
    out = torch.empty_like(keys)
    tb = lib.apt_sort_u64_temp_bytes(keys.numel())
    temp = torch.empty(tb, dtype=torch.uint8, device="cuda")
    check(lib.apt_sort_u64(keys.data_ptr(), out.data_ptr(), keys.numel(), temp.data_ptr(), tb, 40, None))
    assert torch.equal(out, torch.sort(keys).values)
    w = synthetic.WORKLOADS["tiny_np"]
    rows = synthetic.normal_rows(w, torch.device("cuda"), first_row=100, num_rows=20000)
    assert abs(float(rows.mean())) < 0.01 and abs(float(rows.std()) - 1.0) < 0.01
    ids = torch.tensor([100, 5000, 20099], device="cuda")
    picked = synthetic.normal_rows(w, torch.device("cuda"), row_ids=ids)
    assert torch.equal(picked, rows[ids - 100])          # a cache row equals the same node's table row
    half = synthetic.normal_rows(synthetic.Workload("x", 10, 10, 128, "bf16", 0.1, [2], 1, 1, 0.1),
                                 torch.device("cuda"), first_row=100, num_rows=64)
    assert half.dtype == torch.bfloat16 and torch.equal(half, rows[:64].bfloat16())


def test_install_tiny_workload_structure():
    w = synthetic.WORKLOADS["tiny_np"]
    ops.init(0, 0, 1, ops.nccl_get_unique_id(), 1)
    inst = synthetic.install(w)
    indptr, indices = host(inst.indptr), host(inst.indices)
    n = w.num_nodes
    assert indptr[0] == 0 and indptr[-1] == len(indices) == w.num_edges + n
    deg = np.diff(indptr)
    assert deg.min() >= 1                                   # one self loop per node
    for v in (0, 1, n // 2, n - 1):
        row = indices[indptr[v]:indptr[v + 1]]
        assert v in row and np.all(np.diff(row) >= 0)       # rows sorted by source id
    k = inst.info["num_cached_rows"]
    assert k == int(n * w.cache_frac)
    cached = host(inst.cached_idx)
    assert deg[cached].min() >= np.sort(deg)[::-1][k - 1]   # the cache holds the highest in-degrees
    pos = host(ops.STATE.feat.feat_pos_map)
    assert (pos >= 0).sum() == k and np.array_equal(pos[cached], np.arange(k))
    # cache rows and host rows of the same node are the same bytes
    ids = torch.from_numpy(cached[:1000]).cuda()
    assert torch.equal(ops.STATE.feat.dev_feats[:1000].cpu(), inst.host_feats[cached[:1000]])
    x = ops.load_subtensor(ids)
    assert torch.equal(x.cpu(), inst.host_feats[cached[:1000]])
    assert inst.train_ids.numel() >= w.batch and int(inst.train_ids.max()) < n
    ops.check_status()


@pytest.mark.parametrize("scale,n,edges,root", [(9, 500, 4000, 7), (12, 4096, 30000, 0), (13, 8000, 20000, 4321)])
def test_bfs_order_and_renumbered_graph_match_oracle(scale, n, edges, root):
    # the locality-preserving partition: breadth-first order, renumbering, share of edges inside a part
    src, dst = orc.rmat_edges(3, 0, edges, scale, n)
    indptr, indices = orc.csc_from_edges(src, dst, n)
    ip, ix = torch.from_numpy(indptr).cuda(), torch.from_numpy(indices).cuda()
    for chunk in (1 << 27, 997):                         # the second forces the frontier to be expanded in pieces
        order = synthetic.bfs_order(ip, ix, root, edge_chunk=chunk)
        want = orc.bfs_order(indptr, indices, root)
        assert np.array_equal(host(order), want)
    assert sorted(host(order).tolist()) == list(range(n)) and int(order[0]) == root
    nip, nix = synthetic.relabel_graph(ip, ix, order)
    wip, wix = orc.relabel_graph(indptr, indices, want)
    assert np.array_equal(host(nip), wip) and np.array_equal(host(nix), wix)
    mv = synthetic.partition_min_vids(n, 4)
    share = synthetic.intra_partition_edge_share(nip, nix, mv)
    assert abs(share - orc.intra_partition_edge_share(wip, wix, mv.numpy())) < 1e-12
    assert share > synthetic.intra_partition_edge_share(ip, ix, mv)        # locality gained over the random ids


@pytest.mark.parametrize("num_ranks,s", [(1000, 1.1), (100_000_000, 1.1), (50, 2.0)])
def test_zipf_ranks_match_oracle(num_ranks, s):
    m = 200_000
    out = torch.empty(m, dtype=torch.int64, device="cuda")
    check(lib.apt_zipf_ranks(9, 12345, m, num_ranks, s, out.data_ptr(), None))
    want = orc.zipf_ranks(9, 12345, m, num_ranks, s)
    got = host(out)
    assert got.min() >= 1 and got.max() <= num_ranks
    assert np.array_equal(got, want)
    # rank 1 is the most likely, and the frequencies fall like k^-s
    c = np.bincount(got, minlength=6)
    assert c[1] > c[2] > c[3] > c[5]
    assert abs(c[1] / c[2] - (1 - 2 ** (1 - s)) / (2 ** (1 - s) - 3 ** (1 - s))) < 0.1


def test_install_stress_and_locality_miniatures():
    ops.init(0, 0, 1, ops.nccl_get_unique_id(), 1)
    w = synthetic.WORKLOADS["tiny_stress"]
    inst = synthetic.install(w)
    n, R = w.num_nodes, inst.info["host_rows"]
    assert R == 5000 and inst.host_feats.shape[0] == R and inst.info["num_cached_rows"] == 6000
    batches = synthetic.seed_batches(inst, 3)
    order = host(inst.degree_order)
    for k, b in enumerate(batches):
        want = orc.zipf_seeds(w.train_seed, k * 4 * w.batch, 4 * w.batch, order, w.zipf_s, w.batch)
        assert np.array_equal(host(b), want) and len(np.unique(want)) == w.batch
    # every node has a row: its own period-R row, from the cache or from host memory
    ids = torch.cat([batches[0], torch.arange(n - 50, n, device="cuda")])
    x = ops.load_subtensor(ids)
    assert torch.equal(x.cpu(), inst.host_feats[(ids % R).cpu()])
    ops.check_status()
    synthetic.cleanup(inst)

    w2 = synthetic.WORKLOADS["tiny_snp_gat"]
    inst2 = synthetic.install(w2)
    assert inst2.info["intra_partition_edge_share"] > 0.7          # three quarters of the edges are planted inside a block
    assert inst2.info["intra_partition_edge_share"] == max(inst2.info["intra_partition_edge_share_as_generated"],
                                                           inst2.info["intra_partition_edge_share_bfs"])
    indptr, indices = host(inst2.indptr), host(inst2.indices)
    assert np.diff(indptr).min() >= 1 and all(v in indices[indptr[v]:indptr[v + 1]] for v in (0, 5, w2.num_nodes - 1))
    synthetic.cleanup(inst2)
