"""SNP with virtual nodes (SAGE / GCN): the id arithmetic kernels against the
oracle for every rank of worlds of 1 to 8, and the whole outermost hop with one
rank. The exchange across real GPUs is checked in tests/multi_gpu_worker.py."""
import ctypes

import numpy as np
import pytest
import torch

import apt_b200
from apt_b200 import ops
from apt_b200._lib import AptError, check, lib
from apt_b200.sampler import SPVirtualSampler
from oracle import oracle as orc
from tests.gpu_util import dev, host, install_graph, reset_world
from tests.helpers import small_graph

pytestmark = pytest.mark.gpu
I64 = np.int64


def _world(ws, rank, n):
    reset_world(ws, rank)
    mv = np.linspace(0, n, ws + 1).astype(I64)
    ops.register_min_vids(torch.from_numpy(mv))
    return mv


@pytest.mark.parametrize("ws", [1, 2, 3, 8])
@pytest.mark.parametrize("fanout", [1, 5, 15])
def test_virtual_ids_match_oracle(ws, fanout):
    n = 10_000
    rng = np.random.default_rng(ws * 31 + fanout)
    for rank in range(ws):
        mv = _world(ws, rank, n)
        num_dst = int(rng.integers(1, 700))
        dst = rng.integers(0, n, num_dst).astype(I64)
        src = rng.integers(0, n, num_dst * fanout).astype(I64)
        got = host(ops.src_to_vir(fanout, num_dst, dev(src)))
        assert np.array_equal(got, orc.src_to_vir(src, fanout, num_dst, mv, ws, rank=rank))
        got = host(ops.srcdst_to_vir(fanout, dev(dst), dev(src)))
        assert np.array_equal(got, orc.srcdst_to_vir(dst, src, fanout, mv, ws, rank=rank))
    reset_world()


@pytest.mark.parametrize("ws", [1, 2, 4, 8])
@pytest.mark.parametrize("with_dst", [0, 1])
def test_send_sizes_match_oracle(ws, with_dst):
    n = 5_000
    rng = np.random.default_rng(ws + 7 * with_dst)
    for rank in range(ws):
        mv = _world(ws, rank, n)
        for num_dst, fanout in ((1, 1), (37, 5), (600, 10)):
            dst = rng.integers(0, n, num_dst).astype(I64)
            # leave one owner without any neighbour in some cases
            src = rng.integers(0, n if num_dst != 37 else n // 2, num_dst * fanout).astype(I64)
            if with_dst:
                m = orc.srcdst_to_vir(dst, src, fanout, mv, ws, rank=rank)
                sorted_all = np.sort(m, kind="stable")
                uniq = np.unique(sorted_all[num_dst:])
            else:
                m = orc.src_to_vir(src, fanout, num_dst, mv, ws, rank=rank)
                sorted_all = np.sort(m, kind="stable")
                uniq = np.unique(m)
            sizes, offs = ops.vir_send_sizes(num_dst, dev(sorted_all), dev(uniq), with_dst, with_offsets=True)
            assert np.array_equal(host(offs), orc.vir_send_offset(ws, num_dst, sorted_all, uniq, with_dst))
            want = orc.vir_send_sizes(ws, num_dst, sorted_all, uniq, with_dst)
            assert np.array_equal(host(sizes), want)
            k = 3 if with_dst else 2
            assert want[k - 2::k].sum() == num_dst * fanout and want[k - 1::k].sum() == len(uniq)
    reset_world()


def test_pack_and_unpack_round_trip():
    _world(4, 3, 1000)
    n_total = 111_059_956
    g = apt_b200.STATE.graph
    saved = g.num_total_nodes
    g.num_total_nodes = n_total
    try:
        rng = np.random.default_rng(5)
        num_dst, m = 977, 20_000
        vir = np.sort(rng.integers(0, 4 * num_dst, m)).astype(I64)
        ids = rng.integers(0, n_total, m).astype(I64)
        packed = ops.sp_pack_frontier(dev(vir), dev(ids), num_dst)
        want = I64(3) * I64(ops.SP_BASE) * I64(n_total) + (vir % num_dst) * I64(n_total) + ids
        assert np.array_equal(host(packed), want)
        out_vir = torch.empty_like(packed)
        out_ori = torch.empty_like(packed)
        check(lib.apt_sp_unpack_frontier(packed.data_ptr(), m, None, n_total, out_vir.data_ptr(), out_ori.data_ptr(),
                                         ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)))
        assert np.array_equal(host(out_ori), ids)
        assert np.array_equal(host(out_vir), 3 * ops.SP_BASE + vir % num_dst)
        # a destination count beyond SP_BASE cannot be packed
        with pytest.raises(AptError):
            ops.sp_pack_frontier(dev(vir), dev(ids), ops.SP_BASE + 1)
    finally:
        g.num_total_nodes = saved
        reset_world()


@pytest.mark.parametrize("with_dst,chained", [(False, True), (False, False), (True, True), (True, False)])
@pytest.mark.parametrize("model", ["SAGE", "GCN"])
def test_outermost_hop_with_one_rank(with_dst, chained, model):
    n, indptr, indices = small_graph(scale=11, edge_factor=6)
    reset_world()
    install_graph(indptr, indices)
    mv = _world(1, 0, n)
    ops.set_sampling(key=77, call_id=5)
    rng = np.random.default_rng(11)
    seeds = rng.permutation(n)[:300].astype(I64)
    fanout = 7
    sampler = SPVirtualSampler(0, [fanout], model=model, shuffle_with_dst=with_dst, chained=chained)
    assert sampler.chained == chained
    input_nodes, output_nodes, blocks, send_sizes, recv_sizes = sampler.sample(None, dev(seeds))
    want = orc.sp_virtual_sample([seeds], fanout, mv, (None, None, None, indptr, indices), key=77, call_id=5,
                                 num_total_nodes=n, with_dst=with_dst, model=model)[0]
    last = sampler.last
    assert np.array_equal(host(last["neighbors"]), want["neighbors"])
    assert np.array_equal(host(last["sorted_allnodes"]), want["sorted_allnodes"])
    assert np.array_equal(host(last["unique_frontier"]), want["unique_frontier"])
    assert np.array_equal(host(last["send_frontier"]), want["send_frontier"])
    assert np.array_equal(host(last["vir_src"]), want["vir_src"])
    assert np.array_equal(host(last["ori_src"]), want["ori_src"])
    assert np.array_equal(send_sizes.numpy(), want["send_sizes"])
    assert np.array_equal(recv_sizes.numpy(), want["recv_sizes"])
    block2, block1 = blocks
    assert np.array_equal(host(block1.coo_col), want["block1_dst"])
    assert np.array_equal(host(block1.coo_row), want["block1_src"])
    assert np.array_equal(host(block2.src_ids), want["unique_src"])
    assert np.array_equal(host(block2.coo_row), want["block2_src"])
    assert np.array_equal(host(block2.coo_col), want["block2_dst"])
    assert np.array_equal(host(last["unique_dst"]), want["unique_dst"])
    assert np.array_equal(host(input_nodes), want["input_nodes"])
    if with_dst:
        assert np.array_equal(host(last["recv_dst"]), want["recv_dst"])

    # sums through the virtual nodes equal the direct sums over the sampled neighbours
    x = rng.standard_normal((n, 16)).astype(np.float32)
    xs = dev(x)[block2.src_ids]
    one = lambda a, b: torch.tensor([a, b], device="cuda")
    e2 = block2.coo_row.numel()
    h_vir = ops.spmm_copy_u_sum(block2.coo_row, block2.coo_col, xs, one(0, e2), one(0, block2.num_src),
                                one(0, block2.num_dst))
    k = 3 if with_dst else 2
    if with_dst:
        h_in = torch.cat((dev(x)[last["recv_dst"]], h_vir))
        total = int(send_sizes[0::3].sum() + send_sizes[2::3].sum())
    else:
        h_in = h_vir
        total = int(send_sizes[1::2].sum())
    got = ops.sp_feat_shuffle(h_in, recv_sizes, send_sizes, total, 16, int(with_dst))
    if with_dst:
        got = got[len(seeds):]
    e1 = block1.coo_row.numel()
    out = ops.spmm_copy_u_sum(block1.coo_row, block1.coo_col, got.contiguous(), one(0, e1), one(0, block1.num_src),
                              one(0, block1.num_dst))
    direct = x[want["neighbors"]].reshape(len(seeds), fanout, 16).astype(np.float64).sum(1)
    assert np.abs(host(out) - direct).max() <= 1e-4
    ops.check_status()
    reset_world()


@pytest.mark.parametrize("with_dst", [False, True])
def test_chained_sampler_equals_operator_by_operator_form(with_dst):
    # three hops, three mini-batches: the chained form (sizes stay on the device, one host read per
    # mini-batch), replayed from a CUDA graph or enqueued kernel by kernel, gives what the
    # operator-by-operator form gives
    n, indptr, indices = small_graph(scale=12, edge_factor=8)
    reset_world()
    install_graph(indptr, indices)
    _world(1, 0, n)
    rng = np.random.default_rng(21)
    batches = [dev(rng.permutation(n)[:128].astype(I64)) for _ in range(3)]
    outs = []
    for chained, use_graph in ((True, True), (True, False), (False, False)):
        ops.set_sampling(key=5, call_id=0)
        smp = SPVirtualSampler(0, [6, 4, 3], model="SAGE", shuffle_with_dst=with_dst, chained=chained,
                               use_graph=use_graph)
        assert smp.use_graph == use_graph and smp.chained == chained
        res = []
        for seeds in batches:
            out = smp.sample(None, seeds)
            res.append((out, {k: (v.clone() if v is not None else None) for k, v in smp.last.items()},
                        [(b.coo_row.clone(), b.coo_col.clone(), b.src_ids.clone(), b.num_src, b.num_dst) for b in out[2]],
                        out[0].clone()))
        outs.append(res)
    for other in outs[1:]:
        for (a, la, ba, ia), (b, lb, bb, ib) in zip(outs[0], other):
            assert torch.equal(ia, ib) and torch.equal(a[3], b[3]) and torch.equal(a[4], b[4])
            assert len(ba) == len(bb) == 4
            for x, y in zip(ba, bb):
                assert x[3:] == y[3:] and all(torch.equal(p, q) for p, q in zip(x[:3], y[:3]))
            for k in ("neighbors", "sorted_allnodes", "unique_frontier", "send_frontier", "vir_src", "ori_src",
                      "unique_dst") + (("recv_dst",) if with_dst else ()):
                assert torch.equal(la[k], lb[k]), k
    ops.check_status()
    reset_world()


@pytest.mark.parametrize("kind", ["snp", "snp_dst", "nfp", "snp_gat"])
def test_pipelined_iterator_of_the_other_samplers(kind):
    # sample_iter with three mini-batches in flight on lanes of their own hands out what sample() returns,
    # for every sampler on the shared replay base
    from apt_b200.sampler import MPSampler, SPGATSampler

    n, indptr, indices = small_graph(scale=12, edge_factor=8)
    reset_world()
    install_graph(indptr, indices)
    _world(1, 0, n)
    rng = np.random.default_rng(77)
    batches = [dev(rng.permutation(n)[:96].astype(I64)) for _ in range(7)]

    def make(lanes):
        if kind == "nfp":
            return MPSampler(0, [5, 3], lanes=lanes)
        if kind == "snp_gat":
            return SPGATSampler(0, [5, 3], prefetch_features=False, lanes=lanes)
        return SPVirtualSampler(0, [5, 3], model="SAGE", shuffle_with_dst=(kind == "snp_dst"), lanes=lanes)

    def flat(out):
        res = [out[0].clone(), out[1].clone()]
        for b in out[2]:
            if isinstance(b, tuple):
                res += [t.clone() for t in b]
            else:
                res += [b.coo_row.clone(), b.coo_col.clone(), b.src_ids.clone(),
                        torch.tensor([b.num_src, b.num_dst])]
        return res + [t.clone() for t in out[3:]]

    ops.set_sampling(key=12, call_id=3)
    one = make(1)
    want = [flat(one.sample(None, b)) for b in batches]
    ops.set_sampling(key=12, call_id=3)
    piped = make(3)
    assert piped.lanes == 3
    got = [flat(out) for out in piped.sample_iter(None, batches)]
    assert len(got) == len(want)
    for g_, w_ in zip(got, want):
        assert len(g_) == len(w_)
        for a, b in zip(g_, w_):
            assert torch.equal(a.cpu(), b.cpu())
    assert ops.STATE.lane == 0
    ops.check_status()
    reset_world()


def test_committed_strategy_fixture_one_rank():
    # tests/golden/strategies_small.npz, one-rank cases: SNP with virtual nodes (both variants) and NFP
    import os

    from apt_b200.sampler import MPSampler

    golden = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
    z = np.load(os.path.join(golden, "path_small.npz"))
    want = np.load(os.path.join(golden, "strategies_small.npz"))
    n = int(z["num_nodes"])
    reset_world()
    install_graph(z["indptr"], z["indices"])
    _world(1, 0, n)
    seeds = dev(want["ws1/0/seeds"])
    for with_dst in (False, True):
        ops.set_sampling(key=99, call_id=4)
        smp = SPVirtualSampler(0, [5], model="SAGE", shuffle_with_dst=with_dst)
        input_nodes, _, (block2, block1), send_sizes, recv_sizes = smp.sample(None, seeds)
        got = dict(smp.last, input_nodes=input_nodes, unique_src=block2.src_ids, block1_dst=block1.coo_col,
                   block2_src=block2.coo_row, block2_dst=block2.coo_col, send_sizes=send_sizes, recv_sizes=recv_sizes)
        for name in ("neighbors", "sorted_allnodes", "unique_frontier", "send_frontier", "vir_src", "ori_src",
                     "send_sizes", "recv_sizes", "unique_src", "unique_dst", "block1_dst", "block2_src", "block2_dst",
                     "input_nodes"):
            assert np.array_equal(host(got[name]), want[f"ws1/0/snp{int(with_dst)}/{name}"]), (with_dst, name)
    ops.set_sampling(key=99, call_id=4)
    in_nodes, _, blocks, send_size, recv_size = MPSampler(0, [5]).sample(None, seeds)
    row, col, fsz, csz, ssz = blocks[0]
    got = dict(all_frontier=in_nodes, all_coo_row=row, all_coo_col=col, send_size=send_size, recv_size=recv_size,
               recv_frontier_size=fsz, recv_coo_size=csz)
    for name, v in got.items():
        assert np.array_equal(host(v), want[f"ws1/0/nfp/{name}"]), name
    ops.check_status()
    reset_world()
