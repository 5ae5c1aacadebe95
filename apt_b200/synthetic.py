"""Seeded synthetic workloads with the shapes of the reference's datasets
(ogbn-papers100M, Friendster and IGB are what scripts/preprocess_dataset.py:18-41
loads; none can be downloaded here, so R-MAT graphs of the same sizes stand in).

Everything is derived from counter-based Philox streams in the CUDA library,
so every rank builds bit-identical graphs and feature rows on its own GPU, and
the CPU oracle can regenerate small instances for the tests.

The layout handed to the operators is the reference's: an int64 CSC
(``graph.adj_tensors("csc")``, python/npc/utils/utils.py:311) with one self loop
per node (scripts/load_data.py:71), contiguous id ranges per rank
(``min_vids``), a page-locked host feature table shared by all ranks and a
per-GPU cache of the highest in-degree rows.
"""
import ctypes
import math
import os
from dataclasses import dataclass, field
from typing import List, Optional

import torch

from . import _lib, hostmem, ops
from ._lib import check, lib

_TORCH_DT = {"f32": torch.float32, "bf16": torch.bfloat16, "f16": torch.float16}
_DT_CODE = {"f32": _lib.F32, "bf16": _lib.BF16, "f16": _lib.F16}


@dataclass
class Workload:
    name: str
    num_nodes: int
    num_edges: int           # directed R-MAT edges before the self loops
    feat_dim: int
    dtype: str               # f32 | bf16 | f16
    cache_frac: float        # fraction of rows cached per GPU (by in-degree)
    fanouts: List[int]       # fanouts[0] is the outermost hop
    batch: int               # seeds per GPU per mini-batch
    hidden: int
    train_frac: float
    system: str = "NP"
    cache_bytes: Optional[int] = None
    rmat: tuple = (0.57, 0.19, 0.19)
    graph_seed: int = 1
    feat_seed: int = 2
    perm_seed: int = 3
    train_seed: int = 4
    undirected: bool = False
    notes: str = ""

    @property
    def scale(self):
        return max(1, math.ceil(math.log2(self.num_nodes)))


WORKLOADS = {
    # BASELINE.json configs[0]: the CPU-runnable case
    "c0_small_np": Workload("c0_small_np", 1 << 20, 16_000_000, 128, "f32", 0.25, [25, 10], 1024, 256, 0.10),
    # configs[1]: papers-shaped NPC run (the metric's configuration)
    "c1_papers_np": Workload("c1_papers_np", 111_059_956, 1_600_000_000, 128, "f32", 0.25, [15, 10, 5], 1024, 256, 0.011),
    # configs[3]: friendster-shaped DNP run
    "c3_friendster_np": Workload("c3_friendster_np", 65_608_366, 1_800_000_000, 256, "bf16", 0.40, [20, 15], 2048, 256,
                                 0.01, undirected=True),
    # a miniature of c1 for quick checks and tests
    "tiny_np": Workload("tiny_np", 1 << 16, 1 << 20, 128, "f32", 0.25, [15, 10, 5], 256, 256, 0.05),
}


def _s():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _p(t):
    return ctypes.c_void_p(t.data_ptr())


def node_permutation(w: Workload, device) -> torch.Tensor:
    """Random relabelling of node ids, so that contiguous id ranges are a random
    partition (the reference partitions, then renumbers each part contiguously,
    scripts/preprocess_dataset.py:128-135)."""
    g = torch.Generator(device=device).manual_seed(w.perm_seed)
    return torch.randperm(w.num_nodes, generator=g, device=device)


def build_csc(w: Workload, device=None, chunk=1 << 27):
    """R-MAT edges -> id permutation -> self loops -> CSC sorted by (dst, src).
    Returns (indptr, indices) as int64 CUDA tensors."""
    device = device or torch.device("cuda", torch.cuda.current_device())
    n, bits = w.num_nodes, max(1, (w.num_nodes - 1).bit_length())
    mult = 2 if w.undirected else 1
    total = w.num_edges * mult + n
    keys = torch.empty(total, dtype=torch.int64, device=device)
    perm = node_permutation(w, device)
    a, b, c = w.rmat
    at = 0
    src = torch.empty(min(chunk, w.num_edges), dtype=torch.int64, device=device)
    dst = torch.empty_like(src)
    for first in range(0, w.num_edges, chunk):
        m = min(chunk, w.num_edges - first)
        check(lib.apt_rmat_edges(w.graph_seed, first, m, w.scale, n, a, b, c, _p(src), _p(dst), _s()))
        ps, pd = perm[src[:m]], perm[dst[:m]]
        keys[at:at + m] = (pd << bits) | ps
        at += m
        if w.undirected:
            keys[at:at + m] = (ps << bits) | pd
            at += m
    del src, dst, perm
    loop = torch.arange(n, dtype=torch.int64, device=device)
    keys[at:] = (loop << bits) | loop
    del loop
    out = torch.empty_like(keys)
    tb = lib.apt_sort_u64_temp_bytes(total)
    temp = torch.empty(tb, dtype=torch.uint8, device=device)
    check(lib.apt_sort_u64(_p(keys), _p(out), total, _p(temp), tb, 2 * bits, _s()))
    del keys, temp
    counts = torch.zeros(n, dtype=torch.int64, device=device)
    for first in range(0, total, chunk):
        d = out[first:first + chunk] >> bits
        counts += torch.bincount(d, minlength=n)
    indptr = torch.zeros(n + 1, dtype=torch.int64, device=device)
    torch.cumsum(counts, 0, out=indptr[1:])
    out.bitwise_and_((1 << bits) - 1)
    return indptr, out


def partition_min_vids(num_nodes: int, world_size: int) -> torch.Tensor:
    """Equal contiguous id ranges (ids were randomly relabelled, so this is a
    random partition)."""
    step = num_nodes // world_size
    v = [r * step for r in range(world_size)] + [num_nodes]
    return torch.tensor(v, dtype=torch.int64)


def normal_rows(w: Workload, device, first_row=0, num_rows=0, row_ids=None):
    n = row_ids.numel() if row_ids is not None else num_rows
    out = torch.empty((n, w.feat_dim), dtype=_TORCH_DT[w.dtype], device=device)
    check(lib.apt_normal_rows(w.feat_seed, first_row, _p(row_ids) if row_ids is not None and n else None, n,
                              w.feat_dim, _DT_CODE[w.dtype], _p(out) if n else None, _s()))
    return out


def _shared_host_table(w: Workload, rank: int, world_size: int, tag: str):
    """One host table for all ranks of the box: a /dev/shm file mapped shared and
    page-locked by every process (the reference shares its feature tensor
    between the per-GPU processes and registers it, examples/train.py:43-46)."""
    rows, dim = w.num_nodes, w.feat_dim
    dt = _TORCH_DT[w.dtype]
    if world_size == 1:
        return hostmem.alloc_table(rows, dim, dt), None
    import torch.distributed as dist

    path = f"/dev/shm/apt_b200_{tag}_{w.name}.bin"
    nbytes = rows * dim * torch.empty(0, dtype=dt).element_size()
    if rank == 0:
        with open(path, "wb") as f:
            f.truncate(nbytes)
    dist.barrier()
    # registered with CUDA after the fill (cache_feats_shared does it): registering the still
    # unpopulated shared mapping fails with an operating-system error
    t = torch.from_file(path, shared=True, size=rows * dim, dtype=dt).view(rows, dim)
    return t, path


@dataclass
class Installed:
    workload: Workload
    rank: int
    world_size: int
    indptr: torch.Tensor
    indices: torch.Tensor
    min_vids: torch.Tensor
    host_feats: torch.Tensor
    cached_idx: torch.Tensor
    train_ids: torch.Tensor
    shm_path: Optional[str] = None
    info: dict = field(default_factory=dict)


def install(w: Workload, rank=0, world_size=1, row_chunk=1 << 22, tag="bench") -> Installed:
    """Builds the workload on the current GPU and registers it with the operators
    (mix_cache_graphs, cache_feats_shared, register_min_vids)."""
    device = torch.device("cuda", torch.cuda.current_device())
    indptr, indices = build_csc(w, device)
    n = w.num_nodes
    e = torch.empty(0, dtype=torch.int64)
    # whole topology resident in HBM: no adjacency cache is needed
    ops.mix_cache_graphs(0, e, e, e, indptr, indices)
    min_vids = partition_min_vids(n, world_size)
    ops.register_min_vids(min_vids)

    deg = indptr[1:] - indptr[:-1]
    esz = torch.empty(0, dtype=_TORCH_DT[w.dtype]).element_size()
    k = int(n * w.cache_frac) if w.cache_bytes is None else min(n, w.cache_bytes // (w.feat_dim * esz))
    order = torch.sort(deg, descending=True, stable=True).indices
    cached_idx = order[:k].contiguous()
    del order, deg
    dev_feats = normal_rows(w, device, row_ids=cached_idx)

    host, shm_path = _shared_host_table(w, rank, world_size, tag)
    lo = (n * rank) // world_size
    hi = (n * (rank + 1)) // world_size
    for first in range(lo, hi, row_chunk):
        m = min(row_chunk, hi - first)
        host[first:first + m].copy_(normal_rows(w, device, first_row=first, num_rows=m))
    torch.cuda.synchronize()
    if world_size > 1:
        import torch.distributed as dist

        dist.barrier()
    local_idx = torch.arange(n, dtype=torch.int64)
    ops.cache_feats_shared(n, host, dev_feats, cached_idx.cpu(), local_idx, 0)

    g = torch.Generator(device=device).manual_seed(w.train_seed)
    n_train = max(w.batch * world_size, int(n * w.train_frac))
    train = torch.randperm(n, generator=g, device=device)[:n_train]
    per = n_train // world_size            # rebalanced evenly (python/npc/ops.py:454-462)
    train_ids = train[rank * per:(rank + 1) * per].contiguous()
    return Installed(w, rank, world_size, indptr, indices, min_vids, host, cached_idx, train_ids, shm_path,
                     {"num_cached_rows": k, "num_csc_edges": int(indices.numel())})


def cleanup(inst: Installed):
    if inst.shm_path and inst.rank == 0 and os.path.exists(inst.shm_path):
        os.unlink(inst.shm_path)
