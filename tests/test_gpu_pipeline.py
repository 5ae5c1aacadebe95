"""The whole sampled mini-batch (NP strategy, one rank) against the oracle
composed stage by stage, and the row movers."""
import numpy as np
import pytest
import torch

import apt_b200
from apt_b200 import ops
from oracle import oracle as orc
from tests.gpu_util import dev, host, install_graph, reset_world
from tests.helpers import feature_setup, small_graph

pytestmark = pytest.mark.gpu
I64 = np.int64


@pytest.mark.parametrize("chained", [False, True])
def test_np_minibatch_matches_oracle(chained):
    n, indptr, indices = small_graph(scale=13, edge_factor=8)
    install_graph(indptr, indices)
    reset_world(1, 0)
    ops.register_min_vids(torch.tensor([0, n]))
    rng = np.random.default_rng(3)
    feats, uva, devf, cached_idx, local_idx, pos_map, cpu_map = feature_setup(n, 128, 0.25, rng)
    ops.cache_feats_shared(n, torch.from_numpy(uva).pin_memory(), dev(devf), torch.from_numpy(cached_idx),
                           torch.from_numpy(local_idx), 0)
    fanouts = [15, 10, 5]
    seeds = rng.permutation(n)[:256].astype(I64)
    ops.set_sampling(key=31337, call_id=0)
    sampler = apt_b200.MixedNeighborSampler(0, fanouts, chained=chained)
    input_nodes, output_nodes, blocks, perm, send_off, recv_off, inverse_idx = sampler.sample(None, dev(seeds))
    assert (ops.STATE.prefetched is not None) == chained
    x = ops.load_subtensor(input_nodes)
    assert ops.STATE.prefetched is None

    # oracle: same loop as python/npc/sampler.py:132-156
    graph = (None, None, None, indptr, indices)
    cur, call, want_blocks = seeds, 0, []
    for f in reversed(fanouts[1:]):
        nbr = orc.sample_csc_fanout(cur, f, *graph, key=31337, call_id=call)
        call += 1
        uniq, rel = orc.relabel_csc(cur, nbr)
        want_blocks.insert(0, (rel, np.repeat(np.arange(len(cur)), f), uniq))
        cur = uniq
    res = orc.np_sample_and_shuffle([cur], fanouts[0], np.array([0, n]), graph, key=31337, call_id=call)[0]
    uniq, rel = orc.relabel_csc(res[0], res[1])
    want_blocks.insert(0, (rel, np.repeat(np.arange(len(res[0])), fanouts[0]), uniq))
    assert len(blocks) == 3
    for b, (wr, wc, wu) in zip(blocks, want_blocks):
        assert np.array_equal(host(b.coo_row), wr) and np.array_equal(host(b.coo_col), wc)
        assert np.array_equal(host(b.src_ids), wu) and b.num_src == len(wu)
    assert np.array_equal(host(input_nodes), want_blocks[0][2])
    assert np.array_equal(host(perm), res[2]) and np.array_equal(host(inverse_idx), res[5])
    assert np.array_equal(send_off.numpy(), res[3]) and np.array_equal(recv_off.numpy(), res[4])
    assert np.array_equal(host(x), orc.load_subtensor(want_blocks[0][2], pos_map, devf, uva))
    # every sampled edge exists (the reference's debug hook, python/npc/sampler.py:126-130)
    b = blocks[-1]
    src = host(b.src_ids)[host(b.coo_row)]
    dst = seeds[host(b.coo_col)]
    for s_, d_ in list(zip(src, dst))[:200]:
        assert s_ in indices[indptr[d_]:indptr[d_ + 1]]
    # aggregation over the outermost block equals the dense definition
    h = torch.randn((blocks[0].num_src, 64), device="cuda")
    off = [torch.tensor(v, device="cuda") for v in ([0, blocks[0].coo_row.numel()], [0, blocks[0].num_src], [0, blocks[0].num_dst])]
    agg = ops.spmm_copy_u_sum(blocks[0].coo_row, blocks[0].coo_col, h, *off)
    ref = h[blocks[0].coo_row].view(blocks[0].num_dst, fanouts[0], 64).sum(1)
    assert torch.allclose(agg, ref, rtol=1e-5, atol=1e-5)
    ops.check_status()


def test_graph_replay_equals_eager_over_several_batches():
    """Three consecutive mini-batches: CUDA-graph replay, device-chained eager and one
    host read per operator give the same tensors; with two graph buffers a batch's
    results survive the next batch."""
    n, indptr, indices = small_graph(scale=12, edge_factor=8)
    install_graph(indptr, indices)
    reset_world(1, 0)
    ops.register_min_vids(torch.tensor([0, n]))
    rng = np.random.default_rng(8)
    feats, uva, devf, cached_idx, local_idx, pos_map, cpu_map = feature_setup(n, 32, 0.5, rng)
    ops.cache_feats_shared(n, torch.from_numpy(uva).pin_memory(), dev(devf), torch.from_numpy(cached_idx),
                           torch.from_numpy(local_idx), 0)
    batches = [dev(rng.permutation(n)[:200].astype(I64)) for _ in range(3)]
    results = {}
    for mode, kw in (("plain", dict(chained=False)), ("eager", dict(chained=True, use_graph=False)),
                     ("graph", dict(chained=True, use_graph=True, graph_buffers=2))):
        ops.set_sampling(key=4242, call_id=5)
        smp = apt_b200.MixedNeighborSampler(0, [10, 5], **kw)
        outs = []
        for b in batches:
            res = smp.sample(None, b)
            x = ops.load_subtensor(res[0])
            outs.append((res, x))
        # with two buffers the previous batch is still intact after the next one was sampled
        keep = [(host(r[0]), host(r[2][0].coo_row), host(x_)) for r, x_ in outs[-2:]]
        results[mode] = ([(host(r[0]), host(r[2][0].coo_row), host(r[2][1].coo_row), host(r[3]), host(r[6]),
                           host(x_), r[2][0].num_src) for r, x_ in outs[-2:]], keep)
    for mode in ("eager", "graph"):
        for got, want in zip(results[mode][0], results["plain"][0]):
            for g_, w_ in zip(got, want):
                assert np.array_equal(g_, w_), mode
    assert apt_b200.STATE.sample_calls == 5 + 2 * 3
    ops.check_status()


@pytest.mark.parametrize("use_graph", [False, True])
def test_frontier_rows_gathered_beside_the_outermost_hop(use_graph):
    """The rows of the frontier (the destination nodes of the outermost block) are fetched on a
    second stream while that hop is sampled and relabelled, the other rows afterwards: every way of
    joining the two streams gives the rows of one plain gather."""
    n, indptr, indices = small_graph(scale=12, edge_factor=8)
    install_graph(indptr, indices)
    reset_world(1, 0)
    ops.register_min_vids(torch.tensor([0, n]))
    rng = np.random.default_rng(21)
    feats, uva, devf, cached_idx, local_idx, pos_map, cpu_map = feature_setup(n, 48, 0.4, rng)
    ops.cache_feats_shared(n, torch.from_numpy(uva).pin_memory(), dev(devf), torch.from_numpy(cached_idx),
                           torch.from_numpy(local_idx), 0)
    batches = [dev(rng.permutation(n)[:300].astype(I64)) for _ in range(3)]
    got = {}
    for split in (0, 1, 2):
        ops.set_sampling(key=77, call_id=0)
        smp = apt_b200.MixedNeighborSampler(0, [8, 4], chained=True, use_graph=use_graph)
        smp.gather_split = split
        outs = []
        for b in batches:
            res = smp.sample(None, b)
            x = ops.load_subtensor(res[0])
            outs.append((host(res[0]), host(x)))
        got[split] = outs
    for split in (1, 2):
        for (ids_a, x_a), (ids_b, x_b) in zip(got[split], got[0]):
            assert np.array_equal(ids_a, ids_b) and np.array_equal(x_a, x_b), split
    for ids_a, x_a in got[1]:
        assert np.array_equal(x_a, orc.load_subtensor(ids_a, pos_map, devf, uva))
    ops.check_status()


@pytest.mark.parametrize("lanes,thread", [(1, False), (2, False), (3, False), (1, True), (4, True)])
def test_pipelined_iterator_equals_one_sample_per_batch(lanes, thread):
    """sample_iter enqueues mini-batch k + 1 before it reads mini-batch k back; the tensors it hands
    out are those of sample(), batch by batch, and stay valid while the next batch is in flight.
    With lanes the mini-batches in flight run on streams and scratch of their own; with the launch
    thread the replays are enqueued by a second host thread."""
    n, indptr, indices = small_graph(scale=12, edge_factor=8)
    install_graph(indptr, indices)
    reset_world(1, 0)
    ops.register_min_vids(torch.tensor([0, n]))
    rng = np.random.default_rng(33)
    feats, uva, devf, cached_idx, local_idx, pos_map, cpu_map = feature_setup(n, 32, 0.5, rng)
    ops.cache_feats_shared(n, torch.from_numpy(uva).pin_memory(), dev(devf), torch.from_numpy(cached_idx),
                           torch.from_numpy(local_idx), 0)
    batches = [dev(rng.permutation(n)[:150].astype(I64)) for _ in range(9)]

    def snapshot(res, x):
        return (host(res[0]), host(res[2][0].coo_row), host(res[2][1].coo_row), host(res[3]), host(res[6]),
                res[4].clone().numpy(), host(x))

    ops.set_sampling(key=5150, call_id=2)
    plain = apt_b200.MixedNeighborSampler(0, [7, 3], chained=False)
    want = []
    for b in batches:
        res = plain.sample(None, b)
        want.append(snapshot(res, ops.load_subtensor(res[0])))
    ops.set_sampling(key=5150, call_id=2)
    piped = apt_b200.MixedNeighborSampler(0, [7, 3], chained=True, use_graph=True, lanes=lanes)
    assert piped.lanes == lanes and piped._in_flight() == (2 if lanes == 1 else lanes * piped.plans_per_lane)
    piped.launch_thread = thread          # launches from a thread of their own
    got = []
    for res in piped.sample_iter(None, iter(batches)):
        got.append(snapshot(res, ops.load_subtensor(res[0])))      # the next batch is already in flight here
    assert len(got) == len(want)
    for g_, w_ in zip(got, want):
        for a, b in zip(g_, w_):
            assert np.array_equal(a, b)
    assert apt_b200.STATE.sample_calls == 2 + 2 * len(batches)
    # seed batches handed over in page-locked host memory: same mini-batches, output nodes on the device
    ops.set_sampling(key=5150, call_id=2)
    pinned = [b.cpu().pin_memory() for b in batches]
    for k, res in enumerate(piped.sample_iter(None, pinned)):
        assert res[1].is_cuda and torch.equal(res[1], batches[k])
        for a, c in zip(snapshot(res, ops.load_subtensor(res[0])), want[k]):
            assert np.array_equal(a, c)
    # a consumer that stops early leaves nothing behind
    ops.set_sampling(key=5150, call_id=2)
    for k, res in enumerate(piped.sample_iter(None, iter(batches))):
        if k == 2:
            break
    torch.cuda.synchronize()
    # one call at a time: sample() has plans of its own on the caller's stream
    ops.set_sampling(key=5150, call_id=2)
    for b, w_ in zip(batches[:4], want):
        res = piped.sample(None, b)
        for a, c in zip(snapshot(res, ops.load_subtensor(res[0])), w_):
            assert np.array_equal(a, c)
    assert apt_b200.STATE.lane == 0
    ops.check_status()


def test_gather_rows_from_a_device_side_first_row():
    rng = np.random.default_rng(4)
    n = 3000
    feats, uva, devf, cached_idx, local_idx, pos_map, cpu_map = feature_setup(n, 32, 0.5, rng)
    ops.cache_feats_shared(n, torch.from_numpy(uva).pin_memory(), dev(devf), torch.from_numpy(cached_idx),
                           torch.from_numpy(local_idx), 0)
    ids = rng.integers(0, n, 5000).astype(I64)
    want = orc.load_subtensor(ids, pos_map, devf, uva)
    for first, count in ((0, 5000), (1234, 5000), (4999, 5000), (5000, 5000), (100, 3100), (7000, 5000)):
        out = torch.full((5000, 32), -7.0, device="cuda")
        ops._gather_enqueue(dev(ids), torch.tensor([count], device="cuda"), out=out,
                            first_dev=torch.tensor([first], device="cuda"))
        ops.check_status()
        lo = min(first, count)
        assert np.array_equal(host(out)[lo:count], want[lo:count])
        assert (host(out)[:lo] == -7.0).all() and (host(out)[count:] == -7.0).all()   # rows outside stay untouched


@pytest.mark.parametrize("row_elems,dtype", [(256, torch.float32), (1024, torch.float16), (3, torch.float32), (1, torch.bfloat16)])
def test_row_movers(row_elems, dtype):
    g = torch.Generator(device="cuda").manual_seed(row_elems)
    x = torch.randn((5000, row_elems), generator=g, device="cuda").to(dtype)
    idx = torch.randint(0, 5000, (12345,), generator=g, device="cuda")
    assert torch.equal(ops.rows_gather(x, idx), x[idx])
    p = torch.randperm(5000, generator=g, device="cuda")
    y = ops.rows_scatter(x, p, 5000)
    ref = torch.empty_like(x)
    ref[p] = x
    assert torch.equal(y, ref)
    z = ops.rows_scatter(x[:100], p[:100], 5000)
    ref = torch.zeros_like(x)
    ref[p[:100]] = x[:100]
    assert torch.equal(z, ref)


def test_memory_budget_cuts_the_number_of_buffer_sets():
    """Buffer sets are sized for upper bounds; a budget (APT_SAMPLER_PLAN_GB) keeps a shape's ring from
    taking more device memory, down to two sets, and the mini-batches stay what they were."""
    n, indptr, indices = small_graph(scale=12, edge_factor=8)
    install_graph(indptr, indices)
    reset_world(1, 0)
    ops.register_min_vids(torch.tensor([0, n]))
    rng = np.random.default_rng(8)
    batches = [dev(rng.permutation(n)[:120].astype(I64)) for _ in range(7)]
    runs = []
    for budget in (None, 1):
        ops.set_sampling(key=31, call_id=0)
        smp = apt_b200.MixedNeighborSampler(0, [6, 4], prefetch_features=False, lanes=3)
        if budget is not None:
            smp.plan_budget_bytes = budget
        runs.append([(host(r[0]), host(r[2][0].coo_row), host(r[3])) for r in smp.sample_iter(None, batches)])
        assert smp.buffer_sets() == (2 if budget else 3 * smp.plans_per_lane)
    for a, b in zip(*runs):
        for x, y in zip(a, b):
            assert np.array_equal(x, y)
    ops.check_status()


def test_memcpy_async_both_directions_and_inside_a_captured_graph():
    """apt_memcpy_async between page-locked host memory and the device; as a node of a captured graph it
    reads its host source when the replay runs (what the samplers' plans rely on for the call-id base)."""
    import ctypes

    from apt_b200._lib import check, lib

    host_in = torch.arange(16, dtype=torch.int64).pin_memory()
    host_out = torch.zeros(16, dtype=torch.int64).pin_memory()
    dev_buf = torch.zeros(16, dtype=torch.int64, device="cuda")
    ptr = lambda t: ctypes.c_void_p(t.data_ptr())
    stream = lambda: ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    check(lib.apt_memcpy_async(ptr(dev_buf), ptr(host_in), 128, stream()))
    check(lib.apt_memcpy_async(ptr(host_out), ptr(dev_buf), 128, stream()))
    torch.cuda.synchronize()
    assert torch.equal(host_out, host_in)
    assert lib.apt_memcpy_async(None, ptr(host_in), 8, stream()) != 0          # null pointer: refused
    assert lib.apt_memcpy_async(None, None, 0, stream()) == 0                  # nothing to copy
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        check(lib.apt_memcpy_async(ptr(dev_buf), ptr(host_in), 128, stream()))
        dev_buf.add_(1)
        check(lib.apt_memcpy_async(ptr(host_out), ptr(dev_buf), 128, stream()))
    for base in (100, 200):
        host_in.fill_(base)                                                     # changed between replays
        graph.replay()
        torch.cuda.synchronize()
        assert torch.equal(host_out, torch.full((16,), base + 1, dtype=torch.int64))
