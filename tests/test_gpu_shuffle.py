"""GPU parity of the seed shuffle, the feature shuffle and the peer-to-peer
all-to-all. Several ranks are emulated on one GPU as inbox contexts wired to
each other by pointer; all pushes are issued before any wait, so no kernel
ever waits for one that has not been launched."""
import ctypes

import numpy as np
import pytest
import torch

import apt_b200
from apt_b200 import _lib, ops
from apt_b200._lib import check, lib
from oracle import oracle as orc
from tests.gpu_util import dev, host, install_graph, reset_world
from tests.helpers import small_graph

pytestmark = pytest.mark.gpu
I64 = np.int64


def _stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _raw_bytes(ptr, nbytes):
    """A uint8 tensor over device memory the library owns (no copy)."""

    class _Raw:
        __cuda_array_interface__ = {"shape": (int(nbytes),), "typestr": "|u1", "data": (int(ptr), False), "version": 2}

    return torch.as_tensor(_Raw(), device="cuda")


class Ranks:
    """N inbox contexts in one process, each attached to the others by pointer."""

    def __init__(self, ws, region_bytes=1 << 20):
        self.ws = ws
        self.ctx = []
        for r in range(ws):
            c = ctypes.c_void_p()
            check(lib.apt_p2p_create(r, ws, region_bytes, ctypes.byref(c), None))
            self.ctx.append(c)
        for r in range(ws):
            for q in range(ws):
                if q != r:
                    check(lib.apt_p2p_attach_ptr(self.ctx[r], q, lib.apt_p2p_local_base(self.ctx[q])))
        self.status = torch.zeros(2, dtype=torch.int32, device="cuda")

    def alltoall(self, srcs, send_offsets, row_bytes, src_index=None, index_is_dest=0):
        """One all-to-all of all ranks; returns the per-rank received counts (device tensors)."""
        counts = []
        for r in range(self.ws):
            off = dev(np.asarray(send_offsets[r], dtype=I64))
            idx = None if src_index is None else src_index[r].data_ptr()
            n = int(send_offsets[r][-1])
            check(lib.apt_p2p_push(self.ctx[r], srcs[r].data_ptr() if srcs[r].numel() else None, idx, index_is_dest,
                                   off.data_ptr(), n, row_bytes, self.status.data_ptr(), _stream()))
        for r in range(self.ws):
            c = torch.empty(self.ws + 1, dtype=torch.int64, device="cuda")   # per-peer counts, then their total
            check(lib.apt_p2p_wait(self.ctx[r], c.data_ptr(), self.status.data_ptr(), 0, _stream()))
            assert int(c[:self.ws].sum().item()) == int(c[self.ws].item())
            counts.append(c[:self.ws])
        return counts

    def pull(self, r, counts, dst, row_bytes, index=None, index_is_source=0, num_dst_rows=0):
        total = int(counts.sum().item())
        n = num_dst_rows if index is not None and index_is_source else total
        check(lib.apt_p2p_pull(self.ctx[r], counts.data_ptr(), None if index is None else index.data_ptr(),
                               index_is_source, n, max(n, total), row_bytes, dst.data_ptr() if dst.numel() else None,
                               _stream()))

    def close(self):
        for c in self.ctx:
            lib.apt_p2p_destroy(c)


@pytest.mark.parametrize("ws", [1, 2, 4, 8])
@pytest.mark.parametrize("expand", [1, 16])
def test_p2p_alltoall_reference_cases(ws, expand):
    # the closed-form cases of the reference's tests/test_alltoall.cc:24-99
    k, b = 7, 100
    send_sizes = [[k * (rank - r) ** 2 + b for r in range(ws)] for rank in range(ws)]
    recv_sizes = [[k * (r - rank) ** 2 + b for r in range(ws)] for rank in range(ws)]
    send_off = [np.cumsum(s) for s in send_sizes]
    ranks = Ranks(ws)
    try:
        for rep in range(3):  # three epochs: both parities of the inbox are reused
            srcs = [torch.full((int(send_off[r][-1]) * expand,), r + 10 * rep, dtype=torch.int64, device="cuda")
                    for r in range(ws)]
            counts = ranks.alltoall(srcs, send_off, 8 * expand)
            for r in range(ws):
                assert host(counts[r]).tolist() == recv_sizes[r]
                out = torch.empty(sum(recv_sizes[r]) * expand, dtype=torch.int64, device="cuda")
                ranks.pull(r, counts[r], out, 8 * expand)
                want = np.concatenate([np.full(recv_sizes[r][q] * expand, q + 10 * rep, dtype=I64) for q in range(ws)])
                assert np.array_equal(host(out), want)
        assert int(ranks.status[0].item()) == 0
    finally:
        ranks.close()


@pytest.mark.parametrize("ws", [2, 4, 8])
@pytest.mark.parametrize("dtype,D", [(torch.float32, 256), (torch.bfloat16, 256), (torch.float16, 1024), (torch.float32, 5)])
def test_p2p_seed_and_feature_shuffle_matches_oracle(ws, dtype, D):
    rng = np.random.default_rng(ws * 100 + D)
    n_nodes = 4000
    mv = np.linspace(0, n_nodes, ws + 1).astype(I64)
    seeds = [rng.integers(0, n_nodes, 300 + 17 * r).astype(I64) for r in range(ws)]
    want = orc.shuffle_seeds(seeds, mv)
    table = torch.randn((n_nodes, D), device="cuda").to(dtype)
    esz = table.element_size()
    ranks = Ranks(ws, region_bytes=4 << 20)
    reset_world(ws, 0)
    try:
        ops.register_min_vids(torch.from_numpy(mv))
        parts = []
        for r in range(ws):
            apt_b200.STATE.rank = r
            parts.append(ops._bucket(dev(seeds[r])))     # sorted, perm, sizes, offsets
        # --- seed exchange (ShuffleSeeds, src/sampling.cc:159-193)
        counts = ranks.alltoall([p[0] for p in parts], [host(p[3]) for p in parts], 8)
        recv = []
        for r in range(ws):
            out = torch.empty(int(counts[r].sum().item()), dtype=torch.int64, device="cuda")
            ranks.pull(r, counts[r], out, 8)
            recv.append(out)
            assert np.array_equal(host(out), want[r][0])
            assert np.array_equal(host(parts[r][1]), want[r][1])
            assert np.array_equal(np.cumsum(host(counts[r])), want[r][2])
            assert np.array_equal(host(parts[r][3]), want[r][3])
        # --- feature shuffle forward (FeatShuffle fwd, src/feat_shuffle.cc:9-30)
        inputs = [table[recv[r]] for r in range(ws)]
        send_off = [want[r][2] for r in range(ws)]
        counts_f = ranks.alltoall(inputs, send_off, D * esz)
        outs = []
        for r in range(ws):
            out = torch.empty((len(seeds[r]), D), dtype=dtype, device="cuda")
            ranks.pull(r, counts_f[r], out, D * esz, index=parts[r][1], index_is_source=1, num_dst_rows=len(seeds[r]))
            outs.append(out)
            assert torch.equal(out, table[dev(seeds[r])])   # rows come back in the asker's seed order
        # --- backward: rows scattered by permutation travel back (fwd_flag = 0)
        grads = [torch.randn((len(seeds[r]), D), device="cuda").to(dtype) for r in range(ws)]
        recv_off_b = [want[r][3] for r in range(ws)]
        counts_b = ranks.alltoall(grads, recv_off_b, D * esz, src_index=[p[1] for p in parts], index_is_dest=1)
        want_b = orc.feat_shuffle([host(g) for g in grads], recv_off_b, send_off, [want[r][1] for r in range(ws)], D, fwd=False)
        for r in range(ws):
            out = torch.empty((len(want[r][0]), D), dtype=dtype, device="cuda")
            ranks.pull(r, counts_b[r], out, D * esz)
            assert np.array_equal(host(out), want_b[r])
        assert int(ranks.status[0].item()) == 0
    finally:
        reset_world()
        ranks.close()


def test_p2p_wait_times_out_with_a_status_not_a_hang():
    # rank 1 never pushes: rank 0's wait must give up after its bound and report it
    ranks = Ranks(2)
    try:
        src = torch.arange(8, dtype=torch.int64, device="cuda")
        off = dev(np.array([4, 8], dtype=I64))
        check(lib.apt_p2p_push(ranks.ctx[0], src.data_ptr(), None, 0, off.data_ptr(), 8, 8, ranks.status.data_ptr(), _stream()))
        c = torch.full((3,), -1, dtype=torch.int64, device="cuda")
        check(lib.apt_p2p_wait(ranks.ctx[0], c.data_ptr(), ranks.status.data_ptr(), 50_000_000, _stream()))  # 50 ms
        torch.cuda.synchronize()
        assert host(c).tolist() == [4, 0, 4]
        assert int(ranks.status[0].item()) & _lib.FLAG_PEER_TIMEOUT
        # the GPU context stays usable ...
        assert int((src + 1).sum().item()) == 36
        # ... but the inbox does not: after a wait that ran out, a region could be overwritten before its
        # owner has read it, so the next push stores nothing on any peer and reports the time-out again
        poisoned = ctypes.c_int(0)
        check(lib.apt_p2p_poisoned(ranks.ctx[0], ctypes.byref(poisoned)))
        assert poisoned.value == 1
        check(lib.apt_p2p_poisoned(ranks.ctx[1], ctypes.byref(poisoned)))
        assert poisoned.value == 0
        ranks.status.zero_()
        region = int(lib.apt_p2p_region_bytes(ranks.ctx[1]))
        header = 16384
        peer_inbox = _raw_bytes(lib.apt_p2p_local_base(ranks.ctx[1]), header + 4 * region)
        before = peer_inbox[header:].clone()
        src2 = torch.full((8,), 77, dtype=torch.int64, device="cuda")
        check(lib.apt_p2p_push(ranks.ctx[0], src2.data_ptr(), None, 0, off.data_ptr(), 8, 8, ranks.status.data_ptr(), _stream()))
        check(lib.apt_p2p_wait(ranks.ctx[0], c.data_ptr(), ranks.status.data_ptr(), 50_000_000, _stream()))
        torch.cuda.synchronize()
        assert int(ranks.status[0].item()) & _lib.FLAG_PEER_TIMEOUT
        assert host(c).tolist() == [0, 0, 0]
        assert torch.equal(peer_inbox[header:], before)       # nothing reached the peer
    finally:
        ranks.close()
    # inboxes created anew (behind a host barrier when the ranks are processes) work again
    ranks = Ranks(2)
    try:
        srcs = [torch.arange(6, dtype=torch.int64, device="cuda") + 10 * r for r in range(2)]
        counts = ranks.alltoall(srcs, [[2, 6], [5, 6]], 8)
        out = torch.empty(7, dtype=torch.int64, device="cuda")
        ranks.pull(0, counts[0], out, 8)
        assert host(out).tolist() == [0, 1, 10, 11, 12, 13, 14]
        assert int(ranks.status[0].item()) == 0
    finally:
        ranks.close()


def test_p2p_pull_scatter_index_is_bounded():
    # a scatter index that names a row outside the destination drops that row instead of writing past the end
    ranks = Ranks(1)
    try:
        src = torch.arange(6, dtype=torch.int64, device="cuda") + 100
        counts = ranks.alltoall([src], [[6]], 8)
        dst = torch.full((8,), -1, dtype=torch.int64, device="cuda")   # 4 rows belong to the call, 4 are a guard
        index = dev(np.array([3, 0, 9, 1, -2, 2], dtype=I64))
        check(lib.apt_p2p_pull(ranks.ctx[0], counts[0].data_ptr(), index.data_ptr(), 0, 4, 6, 8, dst.data_ptr(), _stream()))
        torch.cuda.synchronize()
        assert host(dst).tolist() == [101, 103, 105, 100, -1, -1, -1, -1]
    finally:
        ranks.close()


def test_p2p_region_overflow_is_flagged():
    ranks = Ranks(1, region_bytes=256)
    try:
        src = torch.arange(100, dtype=torch.int64, device="cuda")
        off = dev(np.array([100], dtype=I64))
        check(lib.apt_p2p_push(ranks.ctx[0], src.data_ptr(), None, 0, off.data_ptr(), 100, 8, ranks.status.data_ptr(), _stream()))
        c = torch.empty(2, dtype=torch.int64, device="cuda")
        check(lib.apt_p2p_wait(ranks.ctx[0], c.data_ptr(), ranks.status.data_ptr(), 0, _stream()))
        torch.cuda.synchronize()
        assert int(ranks.status[0].item()) & _lib.FLAG_TABLE_FULL
        assert host(c).tolist() == [32, 32]
    finally:
        ranks.close()


@pytest.mark.parametrize("backend", ["local", "p2p"])
def test_operator_layer_single_rank(backend):
    """shuffle_seeds / np_sample_and_shuffle / feat_shuffle / alltoall through the
    operator layer with one rank; with the p2p backend rows loop through the inbox."""
    from apt_b200.exchange import LocalExchange, P2PExchange

    n, indptr, indices = small_graph(scale=11)
    install_graph(indptr, indices)
    reset_world(1, 0)
    s = apt_b200.STATE
    ex = LocalExchange(s) if backend == "local" else P2PExchange.__new__(P2PExchange)
    if backend == "p2p":
        c = ctypes.c_void_p()
        check(lib.apt_p2p_create(0, 1, 8 << 20, ctypes.byref(c), None))
        P2PExchange.__init__(ex, s, 0, ctx=c)
    s.exchange = ex
    try:
        ops.register_min_vids(torch.tensor([0, n]))
        rng = np.random.default_rng(1)
        seeds = rng.integers(0, n, 1500).astype(I64)
        ops.set_sampling(key=9, call_id=0)
        res = ops.np_sample_and_shuffle(dev(seeds), 10)
        want = orc.np_sample_and_shuffle([seeds], 10, np.array([0, n]), (None, None, None, indptr, indices), key=9, call_id=0)[0]
        for g, w in zip(res, want):
            assert np.array_equal(host(g), w)
        assert not res[3].is_cuda and not res[4].is_cuda and res[2].is_cuda
        recv, perm, recv_off, dev_off = ops.shuffle_seeds(dev(seeds))
        assert np.array_equal(host(recv)[host(perm)], seeds)
        D = 64
        h = torch.randn((res[0].numel(), D), device="cuda")
        x = ops.rows_gather(h, res[5])                       # h[inverse_idx]
        y = ops.feat_shuffle(x, res[3], res[4], res[2], D, 1)
        assert torch.equal(y, h[res[5]][res[2]])
        g = torch.randn_like(y)
        gb = ops.feat_shuffle(g, res[4], res[3], res[2], D, 0)
        ref = torch.zeros_like(g)
        ref.index_add_(0, res[2], g)
        assert torch.equal(gb, ref)
        out = torch.empty(40, dtype=torch.int64, device="cuda")
        ops.alltoall(torch.arange(40, device="cuda"), out, torch.tensor([10]), torch.tensor([10]), 4, 0)
        assert torch.equal(out, torch.arange(40, device="cuda"))
        ops.check_status()
    finally:
        if backend == "p2p":
            ex.close()
        reset_world()


@pytest.mark.parametrize("ws", [2, 4, 8])
@pytest.mark.parametrize("dtype,D", [(torch.float32, 256), (torch.bfloat16, 64), (torch.float16, 40), (torch.float32, 3)])
def test_p2p_reduce_scatter_and_allbroadcast(ws, dtype, D):
    """The NFP exchanges over emulated ranks: segment r of every rank's rows summed
    on rank r (receiving half of _AllReduce, src/ops/collective.cc:404-436), and
    every rank's rows to every rank (AllBroadcastV2, :367-402)."""
    rng = np.random.default_rng(ws * 100 + D)
    seg = rng.integers(0, 300, ws).astype(I64)
    seg[rng.integers(0, ws)] = 0                                  # one rank owns no destination
    rows = int(seg.sum())
    esz = torch.empty(0, dtype=dtype).element_size()
    xs = [torch.from_numpy(rng.standard_normal((rows, D)).astype(np.float32)).to(dtype).cuda() for _ in range(ws)]
    ranks = Ranks(ws, region_bytes=4 << 20)
    code = {torch.float32: _lib.F32, torch.bfloat16: _lib.BF16, torch.float16: _lib.F16}[dtype]
    try:
        counts = ranks.alltoall(xs, [np.cumsum(seg)] * ws, D * esz)
        want = orc.mp_feat_shuffle_fwd([host(x) for x in xs], seg, D)
        for r in range(ws):
            c = torch.cat([counts[r], counts[r].sum()[None]])
            out = torch.full((int(seg[r]), D), 7, dtype=dtype, device="cuda")
            check(lib.apt_p2p_pull_sum(ranks.ctx[r], c.data_ptr(), code, int(seg[r]), D,
                                       out.data_ptr() if out.numel() else None, ranks.status.data_ptr(), _stream()))
            tol = 1e-5 if dtype == torch.float32 else 1e-2
            err = np.abs(host(out).astype(np.float64) - want[r]) / np.maximum(np.abs(want[r]), 1.0)
            assert err.size == 0 or err.max() <= tol
        assert int(ranks.status[0].item()) == 0
        # a peer that sent another row count is reported, not summed
        r = int(np.argmax(seg))
        c = torch.cat([counts[r], counts[r].sum()[None]]).clone()
        c[(r + 1) % ws] += 1
        out = torch.empty((int(seg[r]), D), dtype=dtype, device="cuda")
        check(lib.apt_p2p_pull_sum(ranks.ctx[r], c.data_ptr(), code, int(seg[r]), D, out.data_ptr(),
                                   ranks.status.data_ptr(), _stream()))
        assert int(ranks.status[0].item()) & _lib.FLAG_SIZE_MISMATCH
        ranks.status.zero_()

        # all-broadcast: the push index repeats every rank's rows once per peer
        lens = rng.integers(0, 200, ws).astype(I64)
        ys = [torch.from_numpy(rng.standard_normal((int(n_), D)).astype(np.float32)).to(dtype).cuda() for n_ in lens]
        idx = [torch.arange(int(n_), device="cuda").repeat(ws) for n_ in lens]
        counts = ranks.alltoall(ys, [np.arange(1, ws + 1, dtype=I64) * int(n_) for n_ in lens], D * esz,
                                src_index=[i if i.numel() else torch.zeros(1, dtype=torch.int64, device="cuda")
                                           for i in idx], index_is_dest=0)
        cat = np.concatenate([host(y) for y in ys])
        for r in range(ws):
            assert np.array_equal(host(counts[r]), lens)
            out = torch.empty((int(lens.sum()), D), dtype=dtype, device="cuda")
            ranks.pull(r, counts[r], out, D * esz)
            assert np.array_equal(host(out), cat)
        assert int(ranks.status[0].item()) == 0
    finally:
        ranks.close()


@pytest.mark.parametrize("backend", ["local", "p2p"])
def test_nfp_operators_single_rank(backend):
    """mp_sample_shuffle / mp_feat_shuffle_fwd / _bwd and the NFP sampler with one rank."""
    from apt_b200.exchange import LocalExchange, P2PExchange
    from apt_b200.sampler import MPSampler

    n, indptr, indices = small_graph(scale=11)
    install_graph(indptr, indices)
    reset_world(1, 0)
    s = apt_b200.STATE
    ex = LocalExchange(s) if backend == "local" else P2PExchange.__new__(P2PExchange)
    if backend == "p2p":
        c = ctypes.c_void_p()
        check(lib.apt_p2p_create(0, 1, 8 << 20, ctypes.byref(c), None))
        P2PExchange.__init__(ex, s, 0, ctx=c)
    s.exchange = ex
    try:
        rng = np.random.default_rng(3)
        seeds = rng.permutation(n)[:400].astype(I64)
        ops.set_sampling(key=4, call_id=0)
        in_nodes, out_nodes, blocks, send_size, recv_size = MPSampler(0, [6]).sample(None, dev(seeds))
        want = orc.mp_sample([seeds], 6, (None, None, None, indptr, indices), key=4, call_id=0)[0]
        all_coo_row, all_coo_col, recv_frontier_size, recv_coo_size, recv_seed_size = blocks[0]
        assert np.array_equal(host(in_nodes), want["all_frontier"])
        assert np.array_equal(host(all_coo_row), want["all_coo_row"])
        assert np.array_equal(host(all_coo_col), want["all_coo_col"])
        for got, name in ((send_size, "send_size"), (recv_size, "recv_size"), (recv_frontier_size, "recv_frontier_size"),
                          (recv_coo_size, "recv_coo_size"), (recv_seed_size, "recv_size")):
            assert not got.is_cuda and np.array_equal(got.numpy(), want[name])
        # three hops, two mini-batches in a row: the replayed CUDA graph, the chained form enqueued eagerly
        # (one host read per mini-batch) and the operator-by-operator form agree
        seeds3 = [dev(rng.permutation(n)[:100].astype(I64)) for _ in range(2)]
        res3 = []
        for chained, use_graph in ((True, True), (True, False), (False, False)):
            ops.set_sampling(key=4, call_id=10)
            smp = MPSampler(0, [5, 4, 3], chained=chained, use_graph=use_graph)
            assert smp.chained == chained and smp.use_graph == use_graph
            res3.append([smp.sample(None, sd) for sd in seeds3])
        for other in res3[1:]:
            for a, b in zip(res3[0], other):
                assert torch.equal(a[0], b[0]) and torch.equal(a[3], b[3]) and torch.equal(a[4], b[4])
                for x_, y_ in zip(a[2][0], b[2][0]):
                    assert torch.equal(x_, y_)
                for x_, y_ in zip(a[2][1:], b[2][1:]):
                    assert torch.equal(x_.coo_row, y_.coo_row) and torch.equal(x_.src_ids, y_.src_ids)
                    assert (x_.num_src, x_.num_dst) == (y_.num_src, y_.num_dst)
        assert not torch.equal(res3[0][0][0], res3[0][1][0])
        x = torch.randn((400, 48), device="cuda")
        y = ops.mp_feat_shuffle_fwd(x, recv_size, send_size, 48)
        assert torch.equal(y, x)
        z = ops.mp_feat_shuffle_bwd(y, send_size, recv_size, 48)
        assert torch.equal(z, x)
        ops.check_status()
    finally:
        if backend == "p2p":
            ex.close()
        reset_world()


@pytest.mark.parametrize("dtype,D", [(torch.float32, 64), (torch.bfloat16, 256), (torch.float16, 1024)])
def test_direct_placement_single_rank(dtype, D):
    """Opt-in direct placement: the rows land at their final slots of a landing buffer and the
    result is a view of it; same bytes as the push / wait / pull path, forward and backward."""
    from apt_b200.exchange import P2PExchange

    reset_world(1, 0)
    s = apt_b200.STATE
    c = ctypes.c_void_p()
    check(lib.apt_p2p_create_landing(0, 1, 8 << 20, 8 << 20, 2, ctypes.byref(c), None))
    ex = P2PExchange.__new__(P2PExchange)
    P2PExchange.__init__(ex, s, 0, ctx=c)
    ex._landing_slots = 2
    s.exchange = ex
    try:
        g = torch.Generator(device="cuda").manual_seed(D)
        n = 3000
        x = torch.randn((n, D), generator=g, device="cuda").to(dtype)
        perm = torch.randperm(n, generator=g, device="cuda")
        off = torch.tensor([n])
        ex.direct = False
        want_f = ops.feat_shuffle(x, off, off, perm, D, 1)
        want_b = ops.feat_shuffle(x, off, off, perm, D, 0)
        ex.direct = True
        got_f = ops.feat_shuffle(x, off, off, perm, D, 1)
        assert torch.equal(got_f, want_f) and torch.equal(got_f, x[perm])
        got_b = ops.feat_shuffle(x, off, off, perm, D, 0)
        assert torch.equal(got_b, want_b)
        # two landing buffers: the first result is still intact after the second call, and is
        # overwritten by the third
        assert torch.equal(got_f, x[perm])
        y = torch.randn((n, D), generator=g, device="cuda").to(dtype)
        got_f2 = ops.feat_shuffle(y, off, off, perm, D, 1)
        assert got_f2.data_ptr() == got_f.data_ptr() and torch.equal(got_f, y[perm])
        # a result that does not fit the landing buffer is refused on the host
        big = torch.zeros((9 << 20) // (D * x.element_size()) + 1, D, dtype=dtype, device="cuda")
        p2 = torch.arange(big.shape[0], device="cuda")
        with pytest.raises(RuntimeError):
            ops.feat_shuffle(big, torch.tensor([big.shape[0]]), torch.tensor([big.shape[0]]), p2, D, 1)
        ops.check_status()
    finally:
        ex.close()
        reset_world()
