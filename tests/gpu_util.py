"""Helpers of the GPU tests: numpy <-> CUDA tensors and state installation."""
import numpy as np
import torch

import apt_b200
from apt_b200 import ops


def dev(a, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(a))
    if dtype is not None:
        t = t.to(dtype)
    return t.cuda()


def host(t):
    if t.dtype == torch.bfloat16:
        return t.float().cpu().numpy()
    return t.cpu().numpy()


def install_graph(indptr, indices, cached=None, pinned_host=False):
    """mix_cache_graphs with the global CSC in HBM (default) or pinned host memory."""
    n = len(indptr) - 1
    if pinned_host:
        gi, gx = torch.from_numpy(indptr).pin_memory(), torch.from_numpy(indices).pin_memory()
    else:
        gi, gx = dev(indptr), dev(indices)
    if cached is None or len(cached) == 0:
        e = torch.empty(0, dtype=torch.int64)
        ops.mix_cache_graphs(0, e, e, e, gi, gx)
        return None, None
    dip = np.concatenate([[0], np.cumsum(indptr[cached + 1] - indptr[cached])]).astype(np.int64)
    dix = np.concatenate([indices[indptr[v]:indptr[v + 1]] for v in cached]).astype(np.int64)
    ops.mix_cache_graphs(len(cached), torch.from_numpy(cached), dev(dip), dev(dix), gi, gx)
    return dip, dix


def reset_world(world_size=1, rank=0):
    s = apt_b200.STATE
    s.rank, s.world_size, s.node_size = rank, world_size, world_size
    s.exchange = None
    s.lane = 0
