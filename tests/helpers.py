"""Shared builders of small seeded workloads for the tests (CPU side)."""
import numpy as np

from oracle import oracle as orc


def small_graph(scale=10, edge_factor=8, seed=1, num_nodes=None):
    n = num_nodes or (1 << scale)
    src, dst = orc.rmat_edges(seed, 0, n * edge_factor, scale, n)
    indptr, indices = orc.csc_from_edges(src, dst, n)
    return n, indptr, indices


def feature_setup(n, dim, cache_frac, rng, dtype=np.float32, host_frac=1.0):
    """Host table for `host_frac` of the nodes (shuffled order), device cache of
    the first cache_frac of a random node order. Returns the tables, index
    lists and the two position maps."""
    feats = rng.standard_normal((n, dim)).astype(dtype)
    local_idx = rng.permutation(n)[: int(n * host_frac)].astype(np.int64)
    uva = feats[local_idx]
    cached_idx = rng.permutation(local_idx)[: int(n * cache_frac)].astype(np.int64)
    dev = feats[cached_idx]
    pos_map, cpu_map = orc.build_feat_pos_maps(n, cached_idx, local_idx)
    return feats, uva, dev, cached_idx, local_idx, pos_map, cpu_map
