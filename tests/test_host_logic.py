"""Host-side logic of the multi-rank path on CPU: the rendezvous that swaps
inbox handles (2 gloo ranks), offset bookkeeping, workload sharding."""
import os
import subprocess
import sys
import textwrap

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_counts_from_inclusive_offsets():
    from apt_b200.exchange import _counts

    assert _counts(torch.tensor([3, 3, 10])) == [3, 0, 7]
    assert _counts(torch.tensor([0])) == [0]


def test_partition_and_batches():
    sys.path.insert(0, ROOT)
    import bench
    from apt_b200 import synthetic

    mv = synthetic.partition_min_vids(103, 4)
    assert mv.tolist() == [0, 25, 50, 75, 103]
    w = synthetic.WORKLOADS["c1_papers_np"]
    assert w.scale == 27 and w.fanouts == [15, 10, 5] and w.batch == 1024
    small = synthetic.Workload("x", 1000, 1000, 8, "f32", 0.1, [2], 64, 8, 0.1)
    inst = synthetic.Installed(small, 0, 1, None, None, mv, None, None, torch.arange(1000))
    bs = bench.batches_of(inst, 40)
    assert all(b.numel() == 64 for b in bs) and bs[0][0] == 0 and bs[1][0] == 64
    assert bench.batches_of(inst, 2, offset=3)[0][0] == 192
    # the benchmark's digest is the same number on the host and on the device side
    a = torch.randint(-2 ** 31, 2 ** 31, (5000,), dtype=torch.int64)
    assert bench.digest_np(a.numpy()) == bench.digest_torch(a)
    # every workload of the benchmark list is registered
    for name in ("c0_small_np", "c1_papers_np", "c2_papers_snp_gat", "c3_friendster_np", "c4_stress"):
        assert name in synthetic.WORKLOADS


def test_handle_exchange_two_gloo_ranks(tmp_path):
    """exchange_blobs is what carries the 64-byte IPC handles between ranks."""
    script = tmp_path / "worker.py"
    script.write_text(textwrap.dedent(f"""
        import os, sys
        sys.path.insert(0, {ROOT!r})
        import torch.distributed as dist
        from apt_b200.exchange import exchange_blobs, make_exchange
        from apt_b200.ops import NPCState
        dist.init_process_group("gloo")
        r = dist.get_rank()
        blobs = exchange_blobs(bytes([r]) * 64)
        assert blobs == [bytes([0]) * 64, bytes([1]) * 64], blobs
        s = NPCState(); s.world_size = 1
        assert make_exchange(s).name == "local"
        s.world_size = 2; s.shuffle_backend = "bogus"
        try:
            make_exchange(s)
        except RuntimeError as e:
            assert "unknown" in str(e)
        else:
            raise SystemExit("bad backend accepted")
        dist.barrier()
        print("HOST_OK", r)
    """))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr",
           "127.0.0.1", "--master-port", "29431", str(script)]
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=300, env=dict(os.environ, MASTER_ADDR="127.0.0.1"))
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-2000:]
    assert res.stdout.count("HOST_OK") == 2


def test_library_backend_collectives_two_gloo_ranks(tmp_path):
    """The NFP and SNP collectives of the library back end (all-broadcast, reduce-scatter, fixed-shape
    all-to-all, all-to-all with offsets) over 2 gloo ranks on CPU tensors, against the oracle."""
    script = tmp_path / "worker.py"
    script.write_text(textwrap.dedent(f"""
        import sys
        sys.path.insert(0, {ROOT!r})
        import numpy as np, torch
        import torch.distributed as dist
        from apt_b200.exchange import NcclExchange
        from apt_b200.ops import NPCState
        from oracle import oracle as orc
        dist.init_process_group("gloo")
        r, ws = dist.get_rank(), dist.get_world_size()
        s = NPCState(); s.world_size = ws; s.rank = r
        ex = NcclExchange(s)
        rng = np.random.default_rng(5)
        lens = [3, 5]
        xs = [rng.standard_normal((n, 4)).astype(np.float32) for n in lens]
        got = ex.allbroadcast(torch.from_numpy(xs[r]), lens)
        assert np.array_equal(got.numpy(), orc.allbroadcast_v2(xs, 4)[r])
        seg = np.array([2, 4])
        ys = [rng.standard_normal((6, 3)).astype(np.float32) for _ in range(ws)]
        got = ex.reduce_scatter(torch.from_numpy(ys[r]), torch.from_numpy(seg), int(seg[r]))
        assert np.allclose(got.numpy(), orc.mp_feat_shuffle_fwd(ys, seg, 3)[r], atol=1e-6)
        send = torch.arange(4).view(2, 2) + 10 * r
        recv = torch.empty_like(send)
        ex.exchange_fixed(send, recv)
        assert recv.tolist() == [[2 * r, 2 * r + 1], [10 + 2 * r, 11 + 2 * r]], recv
        # the closed-form all-to-all case of the reference's tests/test_alltoall.cc:24-60 (k = 7, b = 100)
        sizes = [[7 * (q - p) ** 2 + 100 for p in range(ws)] for q in range(ws)]
        inp = torch.cat([torch.full((sizes[r][p],), 10 * r + p, dtype=torch.int64) for p in range(ws)])
        recv_sizes = [sizes[q][r] for q in range(ws)]
        out = torch.empty(sum(recv_sizes), dtype=torch.int64)
        ex.alltoall(inp, out, torch.tensor(sizes[r]).cumsum(0), torch.tensor(recv_sizes).cumsum(0), 1)
        want = torch.cat([torch.full((recv_sizes[q],), 10 * q + r, dtype=torch.int64) for q in range(ws)])
        assert torch.equal(out, want)
        dist.barrier()
        print("COLL_OK", r)
    """))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr",
           "127.0.0.1", "--master-port", "29432", str(script)]
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=300, env=dict(os.environ, MASTER_ADDR="127.0.0.1"))
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-2000:]
    assert res.stdout.count("COLL_OK") == 2


def test_cost_model_host_arithmetic_matches_oracle():
    """The volume and time formulas of the cost model (python/npc/cost_model/estimator.py:112-188) need no GPU."""
    import numpy as np

    from apt_b200 import planner
    from oracle import oracle as orc

    rng = np.random.default_rng(12)
    for ws in (2, 3, 8):
        for rank in range(ws):
            so, ro = np.cumsum(rng.integers(0, 50, ws)), np.cumsum(rng.integers(0, 50, ws))
            assert planner.get_np_reshuffle_vol(ws, rank, torch.from_numpy(so), torch.from_numpy(ro), 128) == \
                orc.np_reshuffle_vol(ws, rank, so, ro, 128)
            for with_dst in (False, True):
                k = 3 if with_dst else 2
                ss, rs = rng.integers(0, 50, k * ws), rng.integers(0, 50, k * ws)
                assert planner.get_sp_reshuffle_vol(ws, rank, torch.from_numpy(ss), torch.from_numpy(rs), 32, "GCN",
                                                    with_dst) == orc.sp_reshuffle_vol(ws, rank, ss, rs, 32, with_dst)
            sizes = rng.integers(1, 50, ws)
            assert planner.get_mp_reshuffle_vol(ws, torch.tensor([int(sizes[rank])]), torch.from_numpy(sizes), 64) == \
                orc.mp_reshuffle_vol(ws, [int(sizes[rank])], sizes, 64)
    # a GAT layer exchanges hidden x heads columns, through the NP formula (estimator.py:121-122, :149-150)
    assert planner.get_reshuffle_dim("GAT", 64, 4) == 256 and planner.get_reshuffle_dim("SAGE", 64, 4) == 64
    so = torch.tensor([4, 9, 15])
    assert planner.get_sp_reshuffle_vol(3, 1, so, so, 256, "GAT") == planner.get_np_reshuffle_vol(3, 1, so, so, 256)
    vol = 3 * 1024 * 1024
    assert planner.cachemiss_vol_to_time(vol) == orc.vol_to_seconds(vol, planner.REFERENCE_BW["pcie"])
    assert planner.reshuffle_vol_to_time(vol) == orc.vol_to_seconds(vol, planner.REFERENCE_BW["network"])
    assert planner.reshuffle_vol_to_time(vol, planner.B200_BW) < planner.reshuffle_vol_to_time(vol)


def test_cache_selection_modes_and_costmodel_log(tmp_path):
    """The cache modes of cache_adj_and_feats (python/npc/ops.py:107-274) and the cost model's log rows
    (python/npc/cost_model/estimator.py:643-689) on closed-form inputs."""
    from apt_b200 import planner

    N = 10
    # costmodel: candidates 0..9 are feature rows (40 bytes each), 10..19 adjacency lists (8 x degree bytes)
    idx_mem = torch.tensor([40] * N + [8 * (v + 1) for v in range(N)])
    order = torch.tensor([3, 12, 7, 19, 0, 10, 5, 11])          # best first
    # prefix sums 40, 64, 104, 184, 224, ...: the first prefix above 190 is the fifth, the reference keeps one less
    # than its index (index 4 -> 3 candidates)
    feats, adj = planner.select_cache_costmodel(order, idx_mem, 190, N)
    assert feats.tolist() == [3, 7] and adj.tolist() == [2]
    feats, adj = planner.select_cache_costmodel(order, idx_mem, 10, N)
    assert feats.numel() == 0 and adj.numel() == 0
    # greedy: half features, half lists; m = 6 fits (3 x 40 + 8 (1 + 2 + 3 + 4) = 200 at the probed indices)
    f_idx, g_idx = torch.arange(N), torch.arange(N)
    feats, adj = planner.select_cache_greedy(f_idx, g_idx, idx_mem, 200, 0.5, N)
    m = 2 * feats.numel()
    assert feats.tolist() == list(range(feats.numel())) and adj.numel() == feats.numel()
    used = 40 * (m // 2 + 1) + sum(8 * (v + 1) for v in range(m // 2 + 1))   # what the search compares (one past)
    assert used <= 200 < 40 * (m // 2 + 2) + sum(8 * (v + 1) for v in range(m // 2 + 2))
    # dryrun: the order depends on the strategy
    fr = [torch.tensor([5, 0, 9, 1, 0, 0, 2, 0, 0, 0]), torch.tensor([0, 7, 0, 1, 8, 0, 0, 0, 3, 0])]
    mv = [0, 5, 10]
    assert planner.dryrun_cache_order("NP", 1, fr)[:3].tolist() == [4, 1, 8]
    assert planner.dryrun_cache_order("DP", 0, fr)[:3].tolist() == [2, 4, 1]
    assert planner.dryrun_cache_order("MP", 1, fr)[:3].tolist() == [2, 4, 1]
    assert planner.dryrun_cache_order("SP", 1, fr, mv)[:2].tolist() == [8, 6]      # only nodes 5..9 count on rank 1
    local = torch.tensor([0, 2, 4, 6, 8])
    feats, adj = planner.cache_adj_and_feats("dryrun", 0, local, N, cache_memory=3 * 16 * 4, input_dim=16, system="DP",
                                             input_freqs=fr)
    assert feats.tolist() == [2, 4, 0] and adj.numel() == 0                       # hottest local rows, 3 fit
    feats, _ = planner.cache_adj_and_feats("dryrun", 0, local, N, cache_memory=16 * 4, input_dim=16, system="MP",
                                           world_size=2, input_freqs=fr)
    assert feats.tolist() == [2, 4]                                               # NFP rows are world_size times narrower
    feats, adj = planner.cache_adj_and_feats("random", 0, local, N, feat_cache_ratio=0.4,
                                             generator=torch.Generator().manual_seed(1))
    assert feats.numel() == 2 and set(feats.tolist()) <= set(local.tolist()) and adj.numel() == 0
    # the log: four rows, one per strategy, sums in the last column
    res = planner.CostModelResult(volumes={})
    res.records = {"DP": [1.234, 5.0, 0.0], "NP": [1.0, 2.0, 3.004], "SP": [2.0, 2.0, 2.0], "MP": [9.0, 0.5, 0.25]}
    log = tmp_path / "costmodel.csv"
    planner.append_costmodel_csv(str(log), res, tag="papers_w8_x", world_size=8, model="SAGE", batch_size=1024,
                                 input_dim=128, num_hidden=256, num_heads=1, fan_out="15,10,5", cache_mode="dryrun",
                                 cache_memory=4 << 30, cache_value="x", warmup_epochs=1, dryrun_epochs=2,
                                 num_record_steps=10, warmup_time=1.234, dryrun_time=2.5)
    import csv
    with open(log) as f:
        rows = list(csv.reader(f))
    assert len(rows) == 4 and [r[-5] for r in rows] == ["DP", "NP", "SP", "MP"]
    assert rows[0][-4:] == ["1.23", "5.0", "0.0", "6.23"] and rows[1][-1] == "6.0" and rows[0][9] == "4GB"
