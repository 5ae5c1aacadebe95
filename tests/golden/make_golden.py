"""Writes tests/golden/path_small.npz (a small seeded workload with the outputs
of every stage of the path) and tests/golden/strategies_small.npz (the
outermost hop of the same graph under SNP with virtual nodes, with and without
destinations, and under NFP, for one rank and for two ranks), produced by the
CPU oracle.

The reference itself cannot produce fixtures in this environment (its hot path
is CUDA-only and its Python package imports DGL), so these vectors freeze the
oracle's behaviour; the closed-form cases of the reference's own tests are
replayed directly in tests/test_oracle_golden.py.

    python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import oracle as orc  # noqa: E402


def main():
    scale, n, num_edges, graph_seed = 9, 500, 4000, 1
    src, dst = orc.rmat_edges(graph_seed, 0, num_edges, scale, n)
    indptr, indices = orc.csc_from_edges(src, dst, n)
    rng = np.random.default_rng(2024)
    seeds = rng.permutation(n)[:64].astype(np.int64)
    fanout, key, call_id = 10, 7777777, 3
    nbr = orc.sample_csc_fanout(seeds, fanout, None, None, None, indptr, indices, key=key, call_id=call_id)
    uniq, rel = orc.relabel_csc(seeds, nbr)
    ws = 4
    min_vids = np.array([0, 100, 250, 380, n], dtype=np.int64)
    sizes, offs, sorted_idx, perm = orc.bucket_by_owner(uniq, min_vids, ws, rank=1)
    out = os.path.join(os.path.dirname(os.path.abspath(__file__)), "path_small.npz")
    np.savez_compressed(
        out, scale=scale, num_nodes=n, num_edges=num_edges, graph_seed=graph_seed, indptr=indptr, indices=indices,
        seeds=seeds, fanout=fanout, key=key, call_id=call_id, neighbors=nbr, unique=uniq, relabeled=rel,
        world_size=ws, min_vids=min_vids, sorted_idx=sorted_idx, permutation=perm, bucket_offsets=offs)
    print(out, os.path.getsize(out), "bytes")
    strategies(indptr, indices, n)


def strategy_cases(indptr, indices, n):
    """The arrays of strategies_small.npz, keyed '<case>/<rank>/<name>'."""
    graph = (None, None, None, indptr, indices)
    rng = np.random.default_rng(77)
    arrays = {}
    for ws in (1, 2):
        mv = np.linspace(0, n, ws + 1).astype(np.int64)
        seeds = [rng.permutation(n)[:40 + 8 * r].astype(np.int64) for r in range(ws)]
        for r in range(ws):
            arrays[f"ws{ws}/{r}/seeds"] = seeds[r]
        for with_dst in (False, True):
            res = orc.sp_virtual_sample(seeds, 5, mv, graph, key=99, call_id=4, num_total_nodes=n, with_dst=with_dst)
            for r, p in enumerate(res):
                for name in ("neighbors", "sorted_allnodes", "unique_frontier", "send_frontier", "vir_src", "ori_src",
                             "send_sizes", "recv_sizes", "unique_src", "unique_dst", "block1_dst", "block2_src",
                             "block2_dst", "input_nodes"):
                    arrays[f"ws{ws}/{r}/snp{int(with_dst)}/{name}"] = np.asarray(p[name])
        for r, p in enumerate(orc.mp_sample(seeds, 5, graph, key=99, call_id=4)):
            for name in ("all_frontier", "all_coo_row", "all_coo_col", "send_size", "recv_size", "recv_frontier_size",
                         "recv_coo_size"):
                arrays[f"ws{ws}/{r}/nfp/{name}"] = np.asarray(p[name])
    return arrays


def strategies(indptr, indices, n):
    out = os.path.join(os.path.dirname(os.path.abspath(__file__)), "strategies_small.npz")
    np.savez_compressed(out, **strategy_cases(indptr, indices, n))
    print(out, os.path.getsize(out), "bytes")


if __name__ == "__main__":
    main()
