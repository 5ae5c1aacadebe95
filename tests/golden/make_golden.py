"""Writes tests/golden/path_small.npz: a small seeded workload with the
outputs of every stage of the path, produced by the CPU oracle.

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


if __name__ == "__main__":
    main()
