"""Parity with the REFERENCE ITSELF. tests/golden/ref_*.npz hold the outputs of the
reference's own operators (kaihaoma/APT compiled unmodified by oracle/build_ref.py
and run on a B200 by tests/golden/make_ref_golden.py) on seeded inputs; here the
CPU oracle (no GPU needed) and the CUDA path (``-m gpu``) are compared with them:

  relabel_csc, load_subtensor, cpu_load_subtensor      bit-exact
  SpMM / SDDMM on exactly summable inputs               bit-exact
  SpMM / SDDMM on N(0,1) inputs                         1e-5 relative (fp32; the reference sums with
                                                        float atomics in arbitrary order)
  local_sample_one_layer                                layout, edge membership and uniformity only:
                                                        the reference draws from cuRAND, this library
                                                        from Philox (the specification asks for it)
"""
import os

import numpy as np
import pytest

from oracle import oracle as orc

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
I64 = np.int64


def _load(name):
    return np.load(os.path.join(GOLDEN, name))


def _table(rows, dim, salt):
    r = np.arange(rows, dtype=I64)[:, None]
    c = np.arange(dim, dtype=I64)[None, :]
    return (((r * 131 + c * 7 + salt) % 2001) - 1000).astype(np.float32) / 8.0


def _gather_case(z, name):
    feat_dim, rank_dim, offset, n_nodes, n_cached = [int(v) for v in z[f"{name}_shape"]]
    host = _table(n_nodes, feat_dim, int(z["salt"]))
    cached_idx = z[f"{name}_cached_idx"]
    dev = np.ascontiguousarray(host[cached_idx][:, offset:offset + rank_dim]) if n_cached else \
        np.zeros((0, rank_dim), dtype=np.float32)
    return host, dev, cached_idx, np.arange(n_nodes, dtype=I64), offset, z[f"{name}_ids"]


def _sum_close(got, want, magnitude, rel=1e-5):
    """Error bound of a sum in floating point: |got - want| <= rel * (sum of the |terms|). Where the terms do
    not cancel this is the plain relative error; where they do, no fp32 summation can do better: the
    reference's own fp32 results (float atomics) miss the exact sums of N(0,1) terms by up to about 1e-4
    relative at outputs near 1e-2, while staying inside 1e-5 of the summed magnitudes."""
    return np.all(np.abs(got - want) <= rel * np.maximum(magnitude, 1e-30))


# ----------------------------------------------------------------- CPU: the oracle
def test_oracle_relabel_equals_reference():
    z = _load("ref_relabel.npz")
    for name in z["names"]:
        uniq, rel = orc.relabel_csc(z[f"{name}_seeds"], z[f"{name}_neighbors"])
        assert np.array_equal(uniq, z[f"{name}_unique"]), name
        assert np.array_equal(rel, z[f"{name}_relabeled"]), name


def test_oracle_gather_equals_reference():
    z = _load("ref_gather.npz")
    for name in z["names"]:
        host, dev, cached_idx, local_idx, offset, ids = _gather_case(z, name)
        pos_map, cpu_map = orc.build_feat_pos_maps(len(host), cached_idx, local_idx)
        assert np.array_equal(orc.load_subtensor(ids, pos_map, dev, host, feat_dim_offset=offset), z[f"{name}_out"]), name
        assert np.array_equal(orc.cpu_load_subtensor(ids, cpu_map, host), z[f"{name}_cpu_out"]), name


def test_oracle_spmm_sddmm_equal_reference():
    z = _load("ref_spmm_sddmm.npz")
    for name in z["names"]:
        g = lambda k: z[f"{name}_{k}"]
        row, col, co, io, oo = g("row"), g("col"), g("coo_off"), g("in_off"), g("out_off")
        got = {
            "copy_u": orc.spmm_sum("copy_u", row, col, g("x_src"), None, co, io, oo),
            "copy_e": orc.spmm_sum("copy_e", row, col, None, g("x_edge"), co, None, oo),
            # the reference's kernel adds where its name says multiply (src/cuda/spmm.cu:78)
            "u_mul_e": orc.spmm_sum("u_add_e", row, col, g("x_src"), g("x_edge"), co, io, oo),
            "u_add_v": orc.sddmm("u_add_v", row, col, g("x_src"), g("x_dst"), co, io, oo, acc=np.float32),
            "u_mul_v": orc.sddmm("u_mul_v", row, col, g("x_src"), g("x_dst"), co, io, oo, acc=np.float32),
        }
        for k, v in got.items():
            want = g(k)
            if int(g("exact")) or k in ("u_add_v", "u_mul_v"):   # no summation: one rounding, same on both sides
                assert np.array_equal(v.astype(np.float32), want), (name, k)
            else:
                mag = {"copy_u": lambda: orc.spmm_sum("copy_u", row, col, np.abs(g("x_src")), None, co, io, oo),
                       "copy_e": lambda: orc.spmm_sum("copy_e", row, col, None, np.abs(g("x_edge")), co, None, oo),
                       "u_mul_e": lambda: orc.spmm_sum("u_add_e", row, col, np.abs(g("x_src")), np.abs(g("x_edge")),
                                                       co, io, oo)}[k]()
                assert _sum_close(v.astype(np.float64), want.astype(np.float64), mag), (name, k)


def _sample_graph(z):
    src, dst = orc.rmat_edges(int(z["graph_seed"]), 0, int(z["num_edges"]), int(z["scale"]), int(z["num_nodes"]))
    return orc.csc_from_edges(src, dst, int(z["num_nodes"]))


def _slot_histogram(seeds, nbrs, fanout, indptr, indices, bins=8, whole_bins=False):
    """How often each eighth of a seed's neighbour list was chosen, over seeds whose list has `bins`
    distinct members or more (position of the chosen id inside the list, by value). With whole_bins
    only lists whose length is a multiple of `bins` count, so that a uniform choice fills the bins evenly."""
    hist = np.zeros(bins)
    rows = nbrs.reshape(len(seeds), fanout)
    for v, row in zip(seeds, rows):
        lst = indices[indptr[v]:indptr[v + 1]]
        if len(lst) < bins or len(np.unique(lst)) != len(lst) or (whole_bins and len(lst) % bins):
            continue
        order = {int(u): k for k, u in enumerate(lst)}
        for u in row:
            hist[order[int(u)] * bins // len(lst)] += 1
    return hist


def test_reference_sampler_layout_membership_and_uniformity():
    z = _load("ref_sample.npz")
    indptr, indices = _sample_graph(z)
    seeds, fanout, nbrs = z["seeds"], int(z["fanout"]), z["neighbors"]
    assert np.array_equal(z["out_seeds"], seeds) and nbrs.shape == (len(seeds) * fanout,)   # dense [S, fanout]
    for v, row in zip(seeds[:500], nbrs.reshape(len(seeds), fanout)[:500]):
        assert np.isin(row, indices[indptr[v]:indptr[v + 1]]).all()                         # every pair is an edge
    # with replacement: some seed with more neighbours than the fanout still drew one twice
    rows = nbrs.reshape(len(seeds), fanout)
    deg = np.diff(indptr)[seeds]
    assert any(len(np.unique(r)) < fanout for r, d in zip(rows, deg) if d > fanout)
    # the oracle's draws (Philox) and the reference's (cuRAND) fill the eighths of the neighbour lists alike
    ours = orc.sample_csc_fanout(seeds, fanout, None, None, None, indptr, indices, key=7777777, call_id=0)
    h_ref = _slot_histogram(seeds, nbrs, fanout, indptr, indices)
    h_our = _slot_histogram(seeds, ours, fanout, indptr, indices)
    assert h_ref.sum() == h_our.sum() > 5000
    chi2 = float(((h_ref - h_our) ** 2 / (h_ref + h_our)).sum())     # two-sample, 7 degrees of freedom
    assert chi2 < 30.0, (chi2, h_ref, h_our)
    for picks in (nbrs, ours):                                       # and each is flat by itself
        h = _slot_histogram(seeds, picks, fanout, indptr, indices, whole_bins=True)
        assert h.sum() > 500 and float(((h - h.mean()) ** 2 / h.mean()).sum()) < 30.0, h


# ------------------------------------------------------------ GPU: the CUDA path
@pytest.mark.gpu
def test_cuda_relabel_equals_reference():
    from apt_b200 import ops
    from tests.gpu_util import dev, host

    z = _load("ref_relabel.npz")
    for name in z["names"]:
        uniq, rel = ops.relabel_csc(dev(z[f"{name}_seeds"]), dev(z[f"{name}_neighbors"]))
        assert np.array_equal(host(uniq), z[f"{name}_unique"]), name
        assert np.array_equal(host(rel), z[f"{name}_relabeled"]), name
    ops.check_status()


@pytest.mark.gpu
def test_cuda_gather_equals_reference():
    import torch

    from apt_b200 import ops
    from tests.gpu_util import dev, host

    z = _load("ref_gather.npz")
    for name in z["names"]:
        table, cache, cached_idx, local_idx, offset, ids = _gather_case(z, name)
        ops.cache_feats_shared(len(table), torch.from_numpy(table).pin_memory(), dev(cache),
                               torch.from_numpy(cached_idx), torch.from_numpy(local_idx), offset)
        assert np.array_equal(host(ops.load_subtensor(dev(ids))), z[f"{name}_out"]), name
        assert np.array_equal(ops.cpu_load_subtensor(torch.from_numpy(ids)).numpy(), z[f"{name}_cpu_out"]), name
    ops.check_status()


@pytest.mark.gpu
def test_cuda_spmm_sddmm_equal_reference():
    from apt_b200 import ops
    from tests.gpu_util import dev, host

    z = _load("ref_spmm_sddmm.npz")
    for name in z["names"]:
        g = lambda k: z[f"{name}_{k}"]
        row, col, co, io, oo = [dev(g(k)) for k in ("row", "col", "coo_off", "in_off", "out_off")]
        xs, xd, xe = dev(g("x_src")), dev(g("x_dst")), dev(g("x_edge"))
        got = {
            "copy_u": ops.spmm_copy_u_sum(row, col, xs, co, io, oo),
            "copy_e": ops.spmm_copy_e_sum(row, col, xe, co, oo),
            "u_mul_e": ops.spmm_u_mul_e_sum(row, col, xs, xe, co, io, oo, ref_quirk_add=True),
            "u_add_v": ops.sddmm_u_add_v(row, col, xs, xd, co, io, oo),
            "u_mul_v": ops.sddmm_u_mul_v(row, col, xs, xd, co, io, oo),
        }
        for k, v in got.items():
            want = g(k)
            if int(g("exact")) or k in ("u_add_v", "u_mul_v"):
                assert np.array_equal(host(v), want), (name, k)
            else:
                mag = {"copy_u": lambda: orc.spmm_sum("copy_u", g("row"), g("col"), np.abs(g("x_src")), None,
                                                      g("coo_off"), g("in_off"), g("out_off")),
                       "copy_e": lambda: orc.spmm_sum("copy_e", g("row"), g("col"), None, np.abs(g("x_edge")),
                                                      g("coo_off"), None, g("out_off")),
                       "u_mul_e": lambda: orc.spmm_sum("u_add_e", g("row"), g("col"), np.abs(g("x_src")),
                                                       np.abs(g("x_edge")), g("coo_off"), g("in_off"), g("out_off"))}[k]()
                assert _sum_close(host(v).astype(np.float64), want.astype(np.float64), mag), (name, k)
    ops.check_status()


@pytest.mark.gpu
def test_cuda_sampler_fills_neighbour_lists_like_the_reference():
    from apt_b200 import ops
    from tests.gpu_util import dev, host, install_graph

    z = _load("ref_sample.npz")
    indptr, indices = _sample_graph(z)
    install_graph(indptr, indices, cached=z["cached_nodes"])
    seeds, fanout = z["seeds"], int(z["fanout"])
    ops.set_sampling(key=7777777, call_id=0)
    out_seeds, nbrs = ops.local_sample_one_layer(dev(seeds), fanout)
    assert np.array_equal(host(out_seeds), seeds)
    ours = host(nbrs)
    assert np.array_equal(ours, orc.sample_csc_fanout(seeds, fanout, None, None, None, indptr, indices,
                                                      key=7777777, call_id=0))
    h_ref = _slot_histogram(seeds, z["neighbors"], fanout, indptr, indices)
    h_our = _slot_histogram(seeds, ours, fanout, indptr, indices)
    assert float(((h_ref - h_our) ** 2 / (h_ref + h_our)).sum()) < 30.0
    ops.check_status()
