"""Dry run, cache policy and cost model: the device counters, the order by falling
frequency and the hit volume against numpy, the cache selection and the dry-run
file format, and a whole cost-model run with one rank against the oracle."""
import os

import numpy as np
import pytest
import torch

import apt_b200
from apt_b200 import ops, planner
from oracle import oracle as orc
from tests.gpu_util import dev, host, install_graph, reset_world
from tests.helpers import small_graph

pytestmark = pytest.mark.gpu
I64 = np.int64


@pytest.mark.parametrize("n,draws", [(1, 5), (1000, 20_000), (1 << 20, 300_000)])
def test_counters_order_and_hit_volume(n, draws):
    rng = np.random.default_rng(n)
    hc = planner.HotnessCounter(n, device="cuda")
    want = np.zeros(n, dtype=np.int64)
    for _ in range(3):
        ids = np.minimum((rng.pareto(1.2, draws) * n / 50).astype(I64), n - 1)     # skewed accesses
        hc.add(dev(ids))
        want[ids] += 1                                    # an id named twice in one call counts once
        hc.add(dev(np.unique(ids)), distinct=True)
        want[ids] += 1
    assert np.array_equal(host(hc.counters), want)
    order = host(hc.sorted_idx())
    assert np.array_equal(order, orc.hot_order(want))
    for k in (0, 1, n // 3, n, n + 10):
        total, cached = planner.cached_access(hc.counters, dev(order), k)
        assert total == want.sum() and cached == want[order[:min(k, n)]].sum()
        assert planner.get_cache_miss(hc.counters, k, 128) == orc.get_cache_miss(want, k, 128)
    # the cache order may come from other counters than the accesses (made_seeds_freq)
    other = rng.integers(0, 100, n).astype(np.int32)
    assert planner.get_cache_miss(hc.counters, n // 4, 64, dev(other)) == orc.get_cache_miss(want, n // 4, 64, other)
    ops.check_status()


def test_out_of_range_id_is_flagged():
    hc = planner.HotnessCounter(10, device="cuda")
    hc.add(dev(np.array([1, 2, 10, -1, 2], dtype=I64)))
    assert host(hc.counters).tolist() == [0, 1, 1, 0, 0, 0, 0, 0, 0, 0]
    with pytest.raises(RuntimeError):
        ops.check_status()


def test_cache_selection_and_dryrun_file(tmp_path):
    n = 5000
    rng = np.random.default_rng(2)
    freq = rng.integers(0, 50, n).astype(np.int32)
    local = rng.random(n) < 0.5
    order = planner.hot_order(dev(freq))
    sel = planner.select_cache_nodes(order, dev(local), cache_memory=300 * 128 * 4, input_dim=128)
    want = [v for v in orc.hot_order(freq) if local[v]][:300]
    assert host(sel).tolist() == want
    sel_mp = planner.select_cache_nodes(order, dev(local), cache_memory=300 * 128 * 4, input_dim=128, base=4)
    assert host(sel_mp).tolist() == [v for v in orc.hot_order(freq) if local[v]][:1200]
    path = os.path.join(tmp_path, "rk#0_epo100.pt")
    planner.save_dryrun(path, dev(freq), dev(freq) * 2)
    both = torch.load(path)
    assert isinstance(both, list) and both[0].dtype == torch.int64 and not both[1].is_cuda
    assert np.array_equal(planner.load_dryrun(path).numpy(), freq.astype(np.int64) * 2)


def test_reshuffle_volumes_match_oracle():
    rng = np.random.default_rng(4)
    for ws in (2, 4, 8):
        for rank in range(ws):
            so = np.cumsum(rng.integers(0, 100, ws))
            ro = np.cumsum(rng.integers(0, 100, ws))
            assert planner.get_np_reshuffle_vol(ws, rank, torch.from_numpy(so), torch.from_numpy(ro), 256) == \
                orc.np_reshuffle_vol(ws, rank, so, ro, 256)
            for wd in (False, True):
                k = 3 if wd else 2
                ss, rs = rng.integers(0, 100, k * ws), rng.integers(0, 100, k * ws)
                assert planner.get_sp_reshuffle_vol(ws, rank, torch.from_numpy(ss), torch.from_numpy(rs), 64, "SAGE", wd) \
                    == orc.sp_reshuffle_vol(ws, rank, ss, rs, 64, wd)
            r_ = rng.integers(0, 100, ws)
            assert planner.get_mp_reshuffle_vol(ws, torch.tensor([int(r_[rank])]), torch.from_numpy(r_), 32) == \
                orc.mp_reshuffle_vol(ws, [int(r_[rank])], r_, 32)


def test_cost_model_run_with_one_rank():
    n, indptr, indices = small_graph(scale=12, edge_factor=8)
    reset_world()
    install_graph(indptr, indices)
    ops.register_min_vids(torch.tensor([0, n]))
    graph = (None, None, None, indptr, indices)
    mv = np.array([0, n], dtype=I64)
    rng = np.random.default_rng(8)
    fanouts = [5, 4]
    epochs = [[rng.permutation(n)[:64].astype(I64) for _ in range(3)] for _ in range(2)]
    ops.set_sampling(key=31, call_id=0)
    sampler = planner.AllStrategySampler(0, fanouts, model="SAGE")
    res = planner.run_costmodel(sampler, [[dev(b) for b in e] for e in epochs], n, cache_memory=200 * 16 * 4,
                                input_dim=16, num_hidden=8)
    names = ("DP", "NP", "SP", "MP")
    freq = {k: np.zeros(n, dtype=np.float32) for k in names}
    vols = dict.fromkeys(names, 0.0)
    call = 0
    for e in epochs:
        per = {k: np.zeros(n, dtype=np.int64) for k in names}
        for b in e:
            o = orc.all_strategy_sample([b], fanouts, mv, graph, key=31, first_call_id=call, num_total_nodes=n)[0]
            call += len(fanouts) + 1
            per["DP"][o["dp_seeds"]] += 1
            per["NP"][o["np"][0]] += 1
            per["SP"][o["sp"][0]] += 1
            per["MP"][o["mp"][0]] += 1
            vols["NP"] += orc.np_reshuffle_vol(1, 0, o["np"][1], o["np"][2], 8) / len(epochs)
            vols["SP"] += orc.sp_reshuffle_vol(1, 0, o["sp"][1], o["sp"][2], 8) / len(epochs)
            vols["MP"] += orc.mp_reshuffle_vol(1, o["mp"][1], o["mp"][2], 8) / len(epochs)
        for k in names:
            freq[k] += per[k]
    for k in names:
        assert res.volumes[k] == pytest.approx(vols[k])
    mean = {k: (freq[k] / len(epochs)).astype(np.int32) for k in names}
    order = {"DP": orc.hot_order(mean["DP"]), "NP": orc.hot_order(mean["NP"]), "SP": orc.hot_order(mean["DP"]),
             "MP": orc.hot_order(mean["DP"])}
    for k in names:
        dim = 16
        miss = int(mean[k].astype(np.int64).sum() - mean[k][order[k][:200]].astype(np.int64).sum()) * dim
        want_ms = orc.vol_to_seconds(miss, planner.REFERENCE_BW["pcie"]) / len(epochs) * 1000.0
        assert res.records[k][1] == pytest.approx(want_ms, rel=1e-5)
        want_rs = orc.vol_to_seconds(vols[k], planner.REFERENCE_BW["network"]) / len(epochs) * 1000.0
        assert res.records[k][2] == pytest.approx(want_rs, rel=1e-5)
        assert res.records[k][0] > 0
    assert res.best in names and res.total(res.best) == min(res.total(k) for k in names)
    reset_world()
