"""One rank of the multi-GPU parity check (launched by tests/test_gpu_multi.py
through torch.distributed.run, one process per GPU).

Every rank builds the same small graph and feature table, the ranks run the
NP mini-batch (seed shuffle to the owner, outer-hop sampling there, feature
shuffle back, backward shuffle) with the peer-to-peer exchange, and rank 0
compares what all ranks got with the CPU oracle replaying all ranks at once.
The library all-to-all (NCCL) must give the same bytes. A timing of a large
feature shuffle with both backends is printed for information.
"""
import json
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import apt_b200  # noqa: E402
from apt_b200 import ops  # noqa: E402
from apt_b200.exchange import NcclExchange  # noqa: E402
from oracle import oracle as orc  # noqa: E402
from tests.helpers import small_graph  # noqa: E402

I64 = np.int64


def gather_objects(obj):
    out = [None] * dist.get_world_size()
    dist.all_gather_object(out, obj)
    return out


def host(t):
    return (t.float() if t.dtype == torch.bfloat16 else t).cpu().numpy()


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    ops.init(rank, local, world, ops.nccl_get_unique_id(), world)
    assert ops.STATE.exchange.name == "p2p"
    p2p = ops.STATE.exchange
    nccl = NcclExchange(ops.STATE)

    n, indptr, indices = small_graph(scale=13, edge_factor=8)
    e = torch.empty(0, dtype=torch.int64)
    ops.mix_cache_graphs(0, e, e, e, torch.from_numpy(indptr).cuda(), torch.from_numpy(indices).cuda())
    mv = np.linspace(0, n, world + 1).astype(I64)
    ops.register_min_vids(torch.from_numpy(mv))
    graph = (None, None, None, indptr, indices)
    report = {}

    # --- the reference's all-to-all cases (tests/test_alltoall.cc:24-99) on real links
    for expand in (1, 16):
        k, b = 7, 100
        send = [k * (rank - r) ** 2 + b for r in range(world)]
        recv = [k * (r - rank) ** 2 + b for r in range(world)]
        inp = torch.full((sum(send) * expand,), rank, dtype=torch.int64, device="cuda")
        out = torch.empty(sum(recv) * expand, dtype=torch.int64, device="cuda")
        ops.alltoall(inp, out, torch.tensor(send).cumsum(0), torch.tensor(recv).cumsum(0), expand, 0)
        want = np.concatenate([np.full(recv[r] * expand, r, dtype=I64) for r in range(world)])
        assert np.array_equal(host(out), want), f"alltoall expand {expand}"

    # --- a rank that arrives late but inside the wait bound (APT_P2P_TIMEOUT_MS, default 30 s): the wait
    # kernels of the others spin until its flags arrive; the result is complete and no status flag is set
    import time
    torch.cuda.synchronize()
    dist.barrier()
    if rank == world - 1:
        time.sleep(3.0)
    send = [50 + rank] * world
    recv = [50 + r for r in range(world)]
    inp = torch.full((sum(send),), rank, dtype=torch.int64, device="cuda")
    out = torch.empty(sum(recv), dtype=torch.int64, device="cuda")
    ops.alltoall(inp, out, torch.tensor(send).cumsum(0), torch.tensor(recv).cumsum(0), 1, 0)
    assert np.array_equal(host(out), np.concatenate([np.full(recv[r], r, dtype=I64) for r in range(world)])), \
        "all-to-all with a late rank"
    ops.check_status()
    assert not p2p.poisoned()

    # --- NP outer hop: shuffle + unique + sample at the owner
    rng = np.random.default_rng(100 + rank)
    seeds = rng.integers(0, n, 3000 + 101 * rank).astype(I64)
    for trial in range(3):  # several epochs of the inbox
        ops.set_sampling(key=555, call_id=7)
        res = ops.np_sample_and_shuffle(torch.from_numpy(seeds).cuda(), 10)
        ops.set_sampling(key=555, call_id=7)
        ops.STATE.exchange = nccl
        res_nccl = ops.np_sample_and_shuffle(torch.from_numpy(seeds).cuda(), 10)
        ops.STATE.exchange = p2p
        for a, b_ in zip(res, res_nccl):
            assert np.array_equal(host(a), host(b_)), "p2p and nccl disagree"
    all_seeds = gather_objects(seeds)
    all_res = gather_objects([host(t) for t in res])
    if rank == 0:
        want = orc.np_sample_and_shuffle(all_seeds, 10, mv, graph, key=555, call_id=7)
        for r in range(world):
            for got, w in zip(all_res[r], want[r]):
                assert np.array_equal(got, w), f"rank {r}: np_sample_and_shuffle differs from the oracle"
    uniq, nbr, perm, send_off, recv_off, inverse_idx = res

    # --- the whole three-hop mini-batch: device-chained sizes against one read per operator
    batch = torch.from_numpy(seeds[:512]).cuda()
    outs = []
    for chained in (False, True):
        ops.set_sampling(key=99, call_id=0)
        smp = apt_b200.MixedNeighborSampler(rank, [10, 5, 5], chained=chained, prefetch_features=False)
        outs.append(smp.sample(None, batch))
    a, b_ = outs
    for i in (0, 1, 3, 4, 5, 6):
        assert np.array_equal(host(a[i]), host(b_[i])), f"chained sampler differs at output {i}"
    for ba, bb in zip(a[2], b_[2]):
        assert np.array_equal(host(ba.coo_row), host(bb.coo_row)) and np.array_equal(host(ba.src_ids), host(bb.src_ids))
        assert np.array_equal(host(ba.coo_col), host(bb.coo_col)) and (ba.num_src, ba.num_dst) == (bb.num_src, bb.num_dst)

    # --- SNP-GAT outermost hop (python/npc/sampler.py:215-238): unique sources go to their owners,
    # their projected rows come back in unique-source order (python/npc/model/gatconv.py:98-105)
    ops.set_sampling(key=321, call_id=0)
    sp = apt_b200.SPGATSampler(rank, [10])
    sp_seeds = seeds[:700]
    in_nodes, _, sp_blocks, sp_perm, sp_send, sp_recv = sp.sample(None, torch.from_numpy(sp_seeds).cuda())
    all_sp_seeds = gather_objects(sp_seeds)
    all_sp = gather_objects((host(in_nodes), host(sp_blocks[0].coo_row), host(sp_blocks[0].src_ids), host(sp_perm),
                             sp_send.numpy(), sp_recv.numpy()))
    if rank == 0:
        want = orc.sp_gat_sample(all_sp_seeds, 10, mv, graph, key=321, call_id=0)
        for r in range(world):
            got = all_sp[r]
            w = want[r]
            names = ("input_nodes", "arange_src", "unique_neigh", "perm", "send_offset", "recv_offset")
            for name, a_ in zip(names, got):
                assert np.array_equal(a_, w[name]), \
                    f"rank {r}: SNP-GAT sampler output {name} differs from the oracle ({a_.shape} vs {w[name].shape})"
    g0 = torch.Generator(device="cuda").manual_seed(11)
    table_sp = torch.randn((n, 256), generator=g0, device="cuda").bfloat16()       # 4 heads x 64, bf16
    projected = table_sp[in_nodes][sp_blocks[0].num_dst:]
    back = ops.feat_shuffle(projected, sp_send, sp_recv, sp_perm, 256, 1)
    assert torch.equal(back, table_sp[sp_blocks[0].src_ids]), "SNP-GAT feature shuffle"

    # --- SNP with virtual nodes for SAGE / GCN (python/npc/sampler.py:240-330), without and with
    # destinations: every intermediate against the oracle replaying all ranks, then the partial sums
    # per virtual node travel back (SPFeatShuffle) and must add up to the direct neighbour sums
    g1 = torch.Generator(device="cuda").manual_seed(13)
    table_v = torch.randn((n, 32), generator=g1, device="cuda")                     # same on every rank
    vseeds = seeds[:500 + 37 * rank]
    all_vseeds = gather_objects(vseeds)
    one = lambda a_, b_: torch.tensor([a_, b_], device="cuda")
    for with_dst in (False, True):
        ops.set_sampling(key=555, call_id=0)
        vs = apt_b200.SPVirtualSampler(rank, [6], model="SAGE", shuffle_with_dst=with_dst)
        v_in, _, (vb2, vb1), v_send, v_recv = vs.sample(None, torch.from_numpy(vseeds).cuda())
        last = vs.last
        names = ["neighbors", "sorted_allnodes", "unique_frontier", "send_frontier", "vir_src", "ori_src", "unique_dst"]
        got_v = {k_: host(last[k_]) for k_ in names}
        got_v.update(send_sizes=v_send.numpy(), recv_sizes=v_recv.numpy(), input_nodes=host(v_in),
                     block1_dst=host(vb1.coo_col), block2_src=host(vb2.coo_row), block2_dst=host(vb2.coo_col),
                     unique_src=host(vb2.src_ids))
        if with_dst:
            got_v["recv_dst"] = host(last["recv_dst"])
        all_v = gather_objects(got_v)
        if rank == 0:
            want_v = orc.sp_virtual_sample(all_vseeds, 6, mv, graph, key=555, call_id=0, num_total_nodes=n,
                                           with_dst=with_dst, model="SAGE")
            for r in range(world):
                for name, a_ in all_v[r].items():
                    assert np.array_equal(a_, want_v[r][name]), \
                        f"rank {r}: SNP virtual-node sampler (with_dst={with_dst}): {name} differs from the oracle"
        h_vir = ops.spmm_copy_u_sum(vb2.coo_row, vb2.coo_col, table_v[vb2.src_ids], one(0, vb2.coo_row.numel()),
                                    one(0, vb2.num_src), one(0, vb2.num_dst))
        if with_dst:
            h_in = torch.cat((table_v[last["recv_dst"]], h_vir))
            total = int(v_send[0::3].sum() + v_send[2::3].sum())
        else:
            h_in = h_vir
            total = int(v_send[1::2].sum())
        part = ops.sp_feat_shuffle(h_in, v_recv, v_send, total, 32, int(with_dst))
        ops.STATE.exchange = nccl
        part_nccl = ops.sp_feat_shuffle(h_in, v_recv, v_send, total, 32, int(with_dst))
        ops.STATE.exchange = p2p
        assert torch.equal(part, part_nccl), "SNP virtual-node feature shuffle: p2p and library all-to-all differ"
        if with_dst:
            h_self, part = part[:len(vseeds)], part[len(vseeds):].contiguous()
            dst_sorted = ops._bucket(torch.from_numpy(vseeds).cuda())[0]
            assert torch.equal(h_self, table_v[dst_sorted]), "SNP virtual nodes: destination rows"
        out_v = ops.spmm_copy_u_sum(vb1.coo_row, vb1.coo_col, part, one(0, vb1.coo_row.numel()), one(0, vb1.num_src),
                                    one(0, vb1.num_dst))
        direct = table_v[last["neighbors"]].view(len(vseeds), 6, 32).double().sum(1)
        assert (out_v.double() - direct).abs().max().item() <= 1e-4, "SNP virtual nodes: sums differ from direct sums"
        # backward direction: gradients of the partial sums travel to the owners
        gpart = torch.randn((total, 32), generator=g1, device="cuda")
        n_back = int(v_recv[0::3].sum() + v_recv[2::3].sum()) if with_dst else int(v_recv[1::2].sum())
        gback = ops.sp_feat_shuffle(gpart, v_send, v_recv, n_back, 32, int(with_dst))
        all_g = gather_objects((host(gpart), host(gback), v_send.numpy(), v_recv.numpy()))
        if rank == 0:
            want_g = orc.sp_feat_shuffle([a_[0] for a_ in all_g], [a_[2] for a_ in all_g], [a_[3] for a_ in all_g],
                                         with_dst)
            for r in range(world):
                assert np.array_equal(all_g[r][1], want_g[r]), f"rank {r}: sp_feat_shuffle backward differs"
    ops.check_status()

    # --- NFP (python/npc/sampler.py:332-356, model/sageconv.py:117-188): every rank holds a slice of the
    # columns, aggregates it for all ranks' blocks (multi-segment SpMM) and the reduce-scatter sums the slices
    ops.set_sampling(key=777, call_id=0)
    mseeds = seeds[:300 + 41 * rank]
    all_mseeds = gather_objects(mseeds)
    # seed counts differ between the ranks here: the operator-by-operator form sizes its buffers from the
    # gathered sizes; the chained form (buffers sized from the own batch) is checked below on equal counts
    m_in, _, m_blocks, m_send, m_recv = apt_b200.MPSampler(rank, [5], chained=False).sample(
        None, torch.from_numpy(mseeds).cuda())
    m_row, m_col, m_fsz, m_csz, m_ssz = m_blocks[0]
    all_m = gather_objects(dict(all_frontier=host(m_in), all_coo_row=host(m_row), all_coo_col=host(m_col),
                                send_size=m_send.numpy(), recv_size=m_recv.numpy(), recv_frontier_size=m_fsz.numpy(),
                                recv_coo_size=m_csz.numpy()))
    if rank == 0:
        want_m = orc.mp_sample(all_mseeds, 5, graph, key=777, call_id=0)
        for r in range(world):
            for name, a_ in all_m[r].items():
                assert np.array_equal(a_, want_m[r][name]), f"rank {r}: NFP sampler: {name} differs from the oracle"
    ops.set_sampling(key=778, call_id=0)
    eq_seeds = seeds[:256]
    all_eq = gather_objects(eq_seeds)
    c_in, _, c_blocks, c_send, c_recv = apt_b200.MPSampler(rank, [4, 3]).sample(None, torch.from_numpy(eq_seeds).cuda())
    c_row, c_col, c_fsz, c_csz, c_ssz = c_blocks[0]
    all_c = gather_objects(dict(all_frontier=host(c_in), all_coo_row=host(c_row), all_coo_col=host(c_col),
                                send_size=c_send.numpy(), recv_size=c_recv.numpy(), recv_frontier_size=c_fsz.numpy(),
                                recv_coo_size=c_csz.numpy()))
    if rank == 0:
        inner = []
        for r in range(world):
            nb_ = orc.sample_csc_fanout(all_eq[r], 3, *graph, key=778, call_id=0)
            inner.append(orc.relabel_csc(all_eq[r], nb_)[0])
        want_c = orc.mp_sample(inner, 4, graph, key=778, call_id=1)
        for r in range(world):
            for name, a_ in all_c[r].items():
                assert np.array_equal(a_, want_c[r][name]), f"rank {r}: chained NFP sampler: {name} differs from the oracle"
    width = 8
    g2 = torch.Generator(device="cuda").manual_seed(17)
    table_m = torch.randn((n, world * width), generator=g2, device="cuda")          # same on every rank
    weight = torch.randn((world * width, 16), generator=g2, device="cuda")
    cum = lambda t: torch.cat([torch.zeros(1, dtype=torch.int64), t.cumsum(0)]).cuda()
    xs_m = table_m[m_in][:, rank * width:(rank + 1) * width] @ weight[rank * width:(rank + 1) * width]
    part_m = ops.spmm_copy_u_sum(m_row, m_col, xs_m.contiguous(), cum(m_csz), cum(m_fsz), cum(m_ssz))
    summed = ops.mp_feat_shuffle_fwd(part_m, m_recv, m_send, 16)
    ops.STATE.exchange = nccl
    summed_nccl = ops.mp_feat_shuffle_fwd(part_m, m_recv, m_send, 16)
    ops.STATE.exchange = p2p
    nb_m = torch.from_numpy(orc.sample_csc_fanout(mseeds, 5, *graph, key=777, call_id=0)).cuda()
    direct_m = (table_m[nb_m].double() @ weight.double()).view(len(mseeds), 5, 16).sum(1)
    assert (summed.double() - direct_m).abs().max().item() <= 1e-3, "NFP: reduce-scatter differs from the direct sums"
    assert (summed - summed_nccl).abs().max().item() <= 1e-4, "NFP: p2p and library reduce-scatter differ"
    all_part = gather_objects(host(part_m))
    all_sum = gather_objects(host(summed))
    back_m = ops.mp_feat_shuffle_bwd(summed, m_send, m_recv, 16)
    ops.STATE.exchange = nccl
    back_nccl = ops.mp_feat_shuffle_bwd(summed, m_send, m_recv, 16)
    ops.STATE.exchange = p2p
    assert torch.equal(back_m, back_nccl), "NFP: p2p and library all-broadcast differ"
    all_back = gather_objects(host(back_m))
    if rank == 0:
        want_sum = orc.mp_feat_shuffle_fwd(all_part, m_recv.numpy(), 16)
        for r in range(world):
            err = np.abs(all_sum[r] - want_sum[r]).max() if len(all_sum[r]) else 0.0
            assert err <= 1e-4, f"rank {r}: mp_feat_shuffle_fwd differs from the oracle by {err}"
            assert np.array_equal(all_back[r], np.concatenate(all_sum)), f"rank {r}: mp_feat_shuffle_bwd"
    ops.check_status()

    # --- dry run and cost model (python/npc/cost_model/estimator.py:283-697): all four strategies in one pass,
    # counters on the device; exchange volumes and input-node frequencies against the oracle replaying all ranks
    from apt_b200 import planner
    rng_p = np.random.default_rng(900 + rank)
    p_batches = [rng_p.permutation(n)[:96].astype(I64) for _ in range(2)]
    ops.set_sampling(key=4242, call_id=0)
    all_sampler = planner.AllStrategySampler(rank, [4, 3], model="SAGE")
    cm = planner.run_costmodel(all_sampler, [[torch.from_numpy(b).cuda() for b in p_batches]], n,
                               cache_memory=500 * 32 * 4, input_dim=32, num_hidden=16)
    all_pb = gather_objects(p_batches)
    all_cm = gather_objects((cm.volumes, cm.best, cm.records))
    if rank == 0:
        want_vol = [dict.fromkeys(("DP", "NP", "SP", "MP"), 0.0) for _ in range(world)]
        for step in range(2):
            o = orc.all_strategy_sample([all_pb[r][step] for r in range(world)], [4, 3], mv, graph, key=4242,
                                        first_call_id=3 * step, num_total_nodes=n)
            for r in range(world):
                want_vol[r]["NP"] += orc.np_reshuffle_vol(world, r, o[r]["np"][1], o[r]["np"][2], 16)
                want_vol[r]["SP"] += orc.sp_reshuffle_vol(world, r, o[r]["sp"][1], o[r]["sp"][2], 16)
                want_vol[r]["MP"] += orc.mp_reshuffle_vol(world, o[r]["mp"][1], o[r]["mp"][2], 16)
        for r in range(world):
            assert all_cm[r][0] == want_vol[r], f"rank {r}: cost model volumes {all_cm[r][0]} != {want_vol[r]}"
            assert all_cm[r][1] == all_cm[0][1] and all_cm[r][2] == all_cm[0][2], "ranks disagree on the best strategy"
    ops.check_status()

    # --- the committed two-rank fixture (tests/golden/strategies_small.npz): SNP with virtual nodes and NFP
    if world == 2:
        gdir = os.path.join(ROOT, "tests", "golden")
        zf = np.load(os.path.join(gdir, "path_small.npz"))
        fx = np.load(os.path.join(gdir, "strategies_small.npz"))
        nf = int(zf["num_nodes"])
        ops.mix_cache_graphs(0, e, e, e, torch.from_numpy(zf["indptr"]).cuda(), torch.from_numpy(zf["indices"]).cuda())
        ops.register_min_vids(torch.from_numpy(np.linspace(0, nf, 3).astype(I64)))
        fseeds = torch.from_numpy(fx[f"ws2/{rank}/seeds"]).cuda()
        for with_dst in (False, True):
            ops.set_sampling(key=99, call_id=4)
            fs = apt_b200.SPVirtualSampler(rank, [5], model="SAGE", shuffle_with_dst=with_dst)
            f_in, _, (fb2, fb1), f_send, f_recv = fs.sample(None, fseeds)
            got_f = dict(fs.last, input_nodes=f_in, unique_src=fb2.src_ids, block1_dst=fb1.coo_col,
                         block2_src=fb2.coo_row, block2_dst=fb2.coo_col, send_sizes=f_send, recv_sizes=f_recv)
            for name in ("neighbors", "sorted_allnodes", "unique_frontier", "send_frontier", "vir_src", "ori_src",
                         "send_sizes", "recv_sizes", "unique_src", "unique_dst", "block1_dst", "block2_src",
                         "block2_dst", "input_nodes"):
                assert np.array_equal(host(got_f[name]), fx[f"ws2/{rank}/snp{int(with_dst)}/{name}"]), \
                    f"rank {rank}: fixture, SNP with_dst={with_dst}: {name}"
        ops.set_sampling(key=99, call_id=4)
        f_in, _, f_blocks, f_send, f_recv = apt_b200.MPSampler(rank, [5], chained=False).sample(None, fseeds)
        f_row, f_col, f_fsz, f_csz, f_ssz = f_blocks[0]
        for name, v in dict(all_frontier=f_in, all_coo_row=f_row, all_coo_col=f_col, send_size=f_send, recv_size=f_recv,
                            recv_frontier_size=f_fsz, recv_coo_size=f_csz).items():
            assert np.array_equal(host(v), fx[f"ws2/{rank}/nfp/{name}"]), f"rank {rank}: fixture, NFP: {name}"
        ops.check_status()
        ops.mix_cache_graphs(0, e, e, e, torch.from_numpy(indptr).cuda(), torch.from_numpy(indices).cuda())
        ops.register_min_vids(torch.from_numpy(mv))

    # --- feature shuffle forward/backward (fp32 1 KiB rows, bf16 512 B rows, odd width)
    for dtype, D in ((torch.float32, 256), (torch.bfloat16, 256), (torch.float32, 3)):
        g = torch.Generator(device="cuda").manual_seed(7)
        table = torch.randn((n, D), generator=g, device="cuda").to(dtype)   # same on every rank
        h = table[uniq]                                                        # "layer-0 output" of owned ids
        x = ops.rows_gather(h, inverse_idx)
        y = ops.feat_shuffle(x, send_off, recv_off, perm, D, 1)
        assert torch.equal(y, table[torch.from_numpy(seeds).cuda()]), "feat_shuffle fwd"
        ops.STATE.exchange = nccl
        y2 = ops.feat_shuffle(x, send_off, recv_off, perm, D, 1)
        ops.STATE.exchange = p2p
        assert torch.equal(y, y2)
        grad = torch.randn(y.shape, generator=g, device="cuda").to(dtype)
        gb = ops.feat_shuffle(grad, recv_off, send_off, perm, D, 0)
        ops.STATE.exchange = nccl
        gb2 = ops.feat_shuffle(grad, recv_off, send_off, perm, D, 0)
        ops.STATE.exchange = p2p
        assert torch.equal(gb, gb2), "feat_shuffle bwd: p2p vs nccl"
        # the same two calls through the single cooperative kernel, buckets cut into 3 chunks
        p2p.use_fused, p2p.chunks = True, 3
        y3 = ops.feat_shuffle(x, send_off, recv_off, perm, D, 1)
        gb3 = ops.feat_shuffle(grad, recv_off, send_off, perm, D, 0)
        p2p.use_fused, p2p.chunks = False, 1
        assert torch.equal(y3, y) and torch.equal(gb3, gb), "fused all-to-all"
        all_grad = gather_objects(host(grad))
        all_gb = gather_objects(host(gb))
        all_meta = gather_objects((host(perm), send_off.numpy(), recv_off.numpy()))
        if rank == 0:
            want = orc.feat_shuffle(all_grad, [m[2] for m in all_meta], [m[1] for m in all_meta],
                                    [m[0] for m in all_meta], D, fwd=False)
            for r in range(world):
                assert np.array_equal(all_gb[r], want[r]), f"rank {r}: feat_shuffle bwd differs from the oracle"
    ops.check_status()

    # --- opt-in direct placement: rows stored at their final slots of a landing buffer on the receiver,
    # no pull pass; same bytes as the three-kernel path, forward and backward
    from apt_b200.exchange import P2PExchange
    os.environ.update(APT_P2P_DIRECT="1", APT_P2P_DIRECT_SLOTS="2", APT_P2P_LANDING_MB="64")
    direct = P2PExchange(ops.STATE, 64 << 20)
    os.environ.pop("APT_P2P_DIRECT")
    assert direct.direct
    for dtype, D in ((torch.float32, 256), (torch.bfloat16, 256)):
        g = torch.Generator(device="cuda").manual_seed(7)
        table = torch.randn((n, D), generator=g, device="cuda").to(dtype)
        x = ops.rows_gather(table[uniq], inverse_idx)
        grad = torch.randn((len(seeds), D), generator=g, device="cuda").to(dtype)
        ops.STATE.exchange = p2p
        want_y = ops.feat_shuffle(x, send_off, recv_off, perm, D, 1)
        want_g = ops.feat_shuffle(grad, recv_off, send_off, perm, D, 0)
        ops.STATE.exchange = direct
        got_y = ops.feat_shuffle(x, send_off, recv_off, perm, D, 1)
        got_g = ops.feat_shuffle(grad, recv_off, send_off, perm, D, 0)
        assert torch.equal(got_y, want_y), "direct placement: forward shuffle differs"
        assert torch.equal(got_g, want_g), "direct placement: backward shuffle differs"
    ops.STATE.exchange = p2p
    ops.check_status()
    dist.barrier()
    direct.close()

    # --- the small NP configuration of the benchmark list (2^20 nodes, 16 M R-MAT edges, fanout [25, 10],
    # 1024 seeds per rank): graph built on every GPU, whole mini-batch against the oracle replaying all ranks
    from apt_b200 import synthetic
    w0 = synthetic.WORKLOADS["c0_small_np"]
    ip0, ix0 = synthetic.build_csc(w0)
    e0_ = torch.empty(0, dtype=torch.int64)
    ops.mix_cache_graphs(0, e0_, e0_, e0_, ip0, ix0)
    mv0 = synthetic.partition_min_vids(w0.num_nodes, world)
    ops.register_min_vids(mv0)
    gsd = torch.Generator(device="cuda").manual_seed(1000 + rank)
    batch0 = torch.randperm(w0.num_nodes, generator=gsd, device="cuda")[:w0.batch]
    ops.set_sampling(key=2026, call_id=0)
    smp0 = apt_b200.MixedNeighborSampler(rank, w0.fanouts, prefetch_features=False)
    out0 = smp0.sample(None, batch0)
    all_b0 = gather_objects(host(batch0))
    all_o0 = gather_objects((host(out0[0]), host(out0[2][0].coo_row), host(out0[2][1].coo_row), host(out0[3]),
                             out0[4].numpy(), out0[5].numpy(), host(out0[6])))
    if rank == 0:
        cip, cix = host(ip0), host(ix0)
        g0 = (None, None, None, cip, cix)
        frontier, inner = [], []
        for r in range(world):
            nb = orc.sample_csc_fanout(all_b0[r], w0.fanouts[1], *g0, key=2026, call_id=0)
            u, rel = orc.relabel_csc(all_b0[r], nb)
            frontier.append(u)
            inner.append(rel)
        outer = orc.np_sample_and_shuffle(frontier, w0.fanouts[0], mv0.numpy(), g0, key=2026, call_id=1)
        for r in range(world):
            uq, nb, pm, so, ro, inv = outer[r]
            u3, rel3 = orc.relabel_csc(uq, nb)
            want0 = (u3, rel3, inner[r], pm, so, ro, inv)
            for name, a_, b_ in zip(("input_nodes", "outer coo_row", "inner coo_row", "perm", "send_offset",
                                     "recv_offset", "inverse_idx"), all_o0[r], want0):
                assert np.array_equal(a_, b_), f"rank {r}: small NP configuration: {name} differs from the oracle"
    # the same configuration through the pipelined iterator, one lane against three: with lanes every
    # mini-batch in flight runs on a stream, scratch and inbox of its own, and gives the same tensors
    batches0 = [torch.randperm(w0.num_nodes, generator=gsd, device="cuda")[:w0.batch] for _ in range(7)]
    runs0 = []
    for lanes in (1, 3):
        ops.set_sampling(key=2027, call_id=0)
        smp_l = apt_b200.MixedNeighborSampler(rank, w0.fanouts, prefetch_features=False, lanes=lanes)
        assert smp_l.lanes == lanes
        runs0.append([(host(o[0]), host(o[2][0].coo_row), host(o[2][1].coo_row), host(o[3]), o[4].numpy().copy(),
                       o[5].numpy().copy(), host(o[6])) for o in smp_l.sample_iter(None, batches0)])
    for k_, (a_, b_) in enumerate(zip(*runs0)):
        for x_, y_ in zip(a_, b_):
            assert np.array_equal(x_, y_), f"rank {rank}: mini-batch {k_} differs between one lane and three"
    assert ops.STATE.lane == 0 and len(ops.STATE._lane_exchange) == 3
    dist.barrier()
    # put the small test graph back for the timing below
    ops.mix_cache_graphs(0, e, e, e, torch.from_numpy(indptr).cuda(), torch.from_numpy(indices).cuda())
    ops.register_min_vids(torch.from_numpy(mv))

    # --- timing of a large forward shuffle (2 KiB fp16 rows), both backends
    rows, D = 200_000, 1024
    ids = torch.randint(0, n, (rows,), device="cuda")
    recv_ids, perm2, roff, doff = ops.shuffle_seeds(ids)
    x = torch.randn((recv_ids.numel(), D), device="cuda").half()
    for name, ex in (("p2p", p2p), ("nccl", nccl)):
        ops.STATE.exchange = ex
        for _ in range(3):
            ops.feat_shuffle(x, roff, doff, perm2, D, 1)
        torch.cuda.synchronize()
        dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(10):
            ops.feat_shuffle(x, roff, doff, perm2, D, 1)
        e1.record()
        torch.cuda.synchronize()
        ms = torch.tensor([e0.elapsed_time(e1) / 10], device="cuda")
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        counts = np.diff(np.concatenate([[0], roff.numpy()]))
        remote = int(counts.sum() - counts[rank]) * D * 2
        report[name] = {"ms": float(ms.item()), "remote_gb_per_s_per_gpu": remote / (float(ms.item()) * 1e-3) / 1e9}
    ops.STATE.exchange = p2p
    ops.check_status()
    if rank == 0:
        print("MULTI_GPU_OK " + json.dumps({"world": world, "shuffle_2KiB_rows": report}))
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
