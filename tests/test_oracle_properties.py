"""Property tests of the CPU oracle (hypothesis): invariants the reference's
data path guarantees whatever the input, checked on small random cases."""
import numpy as np
from hypothesis import given, settings
from hypothesis import strategies as st

from oracle import oracle as orc

I64 = np.int64
ids = st.lists(st.integers(0, 199), min_size=0, max_size=60)


@settings(max_examples=60, deadline=None)
@given(seeds=ids, nbrs=ids)
def test_relabel_inverts_through_unique(seeds, nbrs):
    # TensorRelabelCSC, src/cuda/relabel.cu:78-185: unique in order of first occurrence, seeds first
    s, m = np.array(seeds, dtype=I64), np.array(nbrs, dtype=I64)
    uniq, rel = orc.relabel_csc(s, m)
    assert len(set(uniq.tolist())) == len(uniq) == len(set(seeds) | set(nbrs))
    assert np.array_equal(uniq[rel], m)
    first = list(dict.fromkeys(seeds + nbrs))
    assert uniq.tolist() == first


@settings(max_examples=60, deadline=None)
@given(values=ids, ws=st.integers(1, 8), rank=st.integers(0, 7))
def test_bucket_is_a_stable_partition(values, ws, rank):
    # ClusterAndPermute, src/cuda/npc_kernel.cu:318-382 (stable order is one of its legal outcomes)
    rank %= ws
    v = np.array(values, dtype=I64)
    mv = np.linspace(0, 200, ws + 1).astype(I64)
    sizes, offs, sorted_ids, perm = orc.bucket_by_owner(v, mv, ws, rank=rank)
    assert sizes.sum() == len(v) and np.array_equal(offs, np.cumsum(sizes))
    assert np.array_equal(sorted_ids[perm], v)
    own = orc.owner_of(sorted_ids, mv, ws, rank=rank)
    assert np.all(np.diff(own) >= 0)
    for r in range(ws):
        assert sorted_ids[own == r].tolist() == [x for x in values if orc.owner_of(np.array([x]), mv, ws, rank=rank)[0] == r]


@settings(max_examples=40, deadline=None)
@given(num_dst=st.integers(1, 20), fanout=st.integers(1, 6), ws=st.integers(1, 6), data=st.data())
def test_virtual_node_sizes_add_up(num_dst, fanout, ws, data):
    # GetVirSendOffset(WithDst) and the sizes SPSampleAndShuffle derives, src/cuda/npc_kernel.cu:119-183,
    # src/sampling.cc:86-106
    src = np.array(data.draw(st.lists(st.integers(0, 199), min_size=num_dst * fanout, max_size=num_dst * fanout)), dtype=I64)
    dst = np.array(data.draw(st.lists(st.integers(0, 199), min_size=num_dst, max_size=num_dst)), dtype=I64)
    mv = np.linspace(0, 200, ws + 1).astype(I64)
    m = orc.src_to_vir(src, fanout, num_dst, mv, ws)
    assert np.array_equal(m % num_dst, np.arange(len(src)) // fanout)
    assert np.array_equal(m // num_dst, orc.owner_of(src, mv, ws))
    sizes = orc.vir_send_sizes(ws, num_dst, np.sort(m), np.unique(m), False)
    assert sizes[0::2].sum() == len(src) and sizes[1::2].sum() == len(np.unique(m))
    for r in range(ws):
        assert sizes[2 * r] == np.sum(m // num_dst == r)
        assert sizes[2 * r + 1] == len(np.unique(m[m // num_dst == r]))
    md = orc.srcdst_to_vir(dst, src, fanout, mv, ws)
    sd = np.sort(md, kind="stable")
    sizes3 = orc.vir_send_sizes(ws, num_dst, sd, np.unique(sd[num_dst:]), True)
    assert sizes3[0::3].sum() == num_dst and sizes3[1::3].sum() == len(src)
    assert sizes3[2::3].sum() == len(np.unique(md[num_dst:]))


@settings(max_examples=40, deadline=None)
@given(freq=st.lists(st.integers(0, 30), min_size=1, max_size=50), k=st.integers(0, 60), dim=st.integers(1, 8))
def test_cache_miss_volume_is_monotone(freq, k, dim):
    # get_cache_miss, python/npc/cost_model/estimator.py:22-30
    f = np.array(freq, dtype=np.int32)
    miss = orc.get_cache_miss(f, k, dim)
    assert 0 <= miss <= int(f.sum()) * dim
    assert orc.get_cache_miss(f, k + 1, dim) <= miss
    assert orc.get_cache_miss(f, len(f), dim) == 0
    order = orc.hot_order(f)
    assert sorted(order.tolist()) == list(range(len(f))) and np.all(np.diff(f[order]) <= 0)
