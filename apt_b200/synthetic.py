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
    partition: str = "random"        # "random": contiguous ranges of randomly relabelled ids; "bfs": ranges of a
                                     # breadth-first order from bfs_root (locality-preserving)
    bfs_root_seed: int = 5
    locality: float = 0.0            # share of the R-MAT edges whose source is moved into the destination's block
    locality_blocks: int = 8         # (equal blocks of the id range): R-MAT alone has no community structure
    seed_dist: str = "uniform"       # "uniform": batches out of a seeded training split; "zipf": Zipf(zipf_s) over
    zipf_s: float = 1.1              # the rank by in-degree
    host_rows_cap: Optional[int] = None   # host table rows when the full table does not fit host memory

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
    # configs[2]: the papers-shaped graph with a locality-preserving partition, SNP with a 3-layer GAT
    # (4 heads x 64, bf16): SDDMM edge scores and softmax-weighted SpMM on the sampled blocks
    "c2_papers_snp_gat": Workload("c2_papers_snp_gat", 111_059_956, 1_600_000_000, 128, "f32", 0.25, [15, 10, 5], 1024,
                                  256, 0.011, system="SP", partition="bfs", locality=0.75),
    # configs[4]: skewed large-feature gather / shuffle stress test (1024-dim fp16 rows of 2 KiB, 60 GB of
    # cached rows per GPU, Zipf(1.1) seeds over the degree rank)
    "c4_stress": Workload("c4_stress", 100_000_000, 1_200_000_000, 1024, "f16", 0.0, [10, 10, 10], 4096, 256, 0.0,
                          cache_bytes=60 * 10 ** 9, seed_dist="zipf", zipf_s=1.1, host_rows_cap=16_000_000),
    # miniatures for quick checks and tests
    "tiny_snp_gat": Workload("tiny_snp_gat", 1 << 15, 1 << 19, 64, "f32", 0.25, [6, 5, 4], 128, 256, 0.05,
                             system="SP", partition="bfs", locality=0.75),
    "tiny_stress": Workload("tiny_stress", 1 << 15, 1 << 19, 256, "f16", 0.0, [4, 4, 4], 256, 256, 0.0,
                            cache_bytes=6000 * 512, seed_dist="zipf", zipf_s=1.1, host_rows_cap=5000),
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
        if w.locality > 0:
            # planted locality: a seeded share of the edges keeps its offset inside a block but moves to the
            # block of its destination, so that a partition into those blocks finds most edges inside a part
            block = -(-n // w.locality_blocks)
            e_idx = torch.arange(first, first + m, dtype=torch.int64, device=device)
            pick = ((e_idx * 0x9E3779B97F4A7C15 + w.graph_seed) >> 11) % 1000 < int(round(w.locality * 1000))
            moved = torch.clamp((pd // block) * block + ps % block, max=n - 1)
            ps = torch.where(pick, moved, ps)
            del e_idx, pick, moved
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


def _shared_host_table(w: Workload, rank: int, world_size: int, tag: str, rows: Optional[int] = None):
    """One host table for all ranks of the box: a /dev/shm file mapped shared and
    page-locked by every process (the reference shares its feature tensor
    between the per-GPU processes and registers it, examples/train.py:43-46)."""
    rows, dim = (w.num_nodes if rows is None else rows), w.feat_dim
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



def bfs_order(indptr: torch.Tensor, indices: torch.Tensor, root: int, edge_chunk: int = 1 << 27) -> torch.Tensor:
    """Breadth-first visiting order over the in-neighbour lists from `root` on the GPU: level by
    level, ascending ids inside a level, unreached nodes last in id order. order[k] is the node
    visited k-th. Contiguous blocks of this order are the locality-preserving partition that stands
    in for the reference's METIS partition (scripts/preprocess_dataset.py:76-135)."""
    n = indptr.numel() - 1
    dev = indptr.device
    deg = indptr[1:] - indptr[:-1]
    visited = torch.zeros(n, dtype=torch.bool, device=dev)
    order = torch.empty(n, dtype=torch.int64, device=dev)
    frontier = torch.tensor([root], dtype=torch.int64, device=dev)
    visited[root] = True
    pos = 0
    while frontier.numel():
        k = frontier.numel()
        order[pos:pos + k] = frontier
        pos += k
        mark = torch.zeros(n, dtype=torch.bool, device=dev)
        d = deg[frontier]
        ends = torch.cumsum(d, 0)
        start, done = 0, 0
        while start < k:      # expand the frontier's lists in pieces of about edge_chunk edges
            stop = int(torch.searchsorted(ends, torch.tensor(done + edge_chunk, device=dev), right=True))
            stop = min(max(stop, start + 1), k)
            f, dd = frontier[start:stop], d[start:stop]
            tot = int(ends[stop - 1]) - done
            if tot:
                first = indptr[f] - (torch.cumsum(dd, 0) - dd)
                idx = torch.repeat_interleave(first, dd) + torch.arange(tot, device=dev)
                mark[indices[idx]] = True
                del idx
            done += tot
            start = stop
        mark &= ~visited
        frontier = mark.nonzero().view(-1)
        visited |= mark
    order[pos:] = (~visited).nonzero().view(-1)
    return order


def relabel_graph(indptr: torch.Tensor, indices: torch.Tensor, order: torch.Tensor, chunk: int = 1 << 27):
    """The CSC after renumbering node order[k] to k (dgl.reorder_graph in
    scripts/preprocess_dataset.py:128-130): (indptr, indices) with lists sorted by new source id."""
    n = indptr.numel() - 1
    dev = indptr.device
    bits = max(1, (n - 1).bit_length())
    new_id = torch.empty(n, dtype=torch.int64, device=dev)
    new_id[order] = torch.arange(n, dtype=torch.int64, device=dev)
    total = indices.numel()
    keys = torch.empty(total, dtype=torch.int64, device=dev)
    deg = indptr[1:] - indptr[:-1]
    for first in range(0, n, chunk >> 4):        # by destination ranges, to bound the expanded temporaries
        last = min(n, first + (chunk >> 4))
        lo, hi = int(indptr[first]), int(indptr[last])
        dst = torch.repeat_interleave(new_id[first:last], deg[first:last])
        keys[lo:hi] = (dst << bits) | new_id[indices[lo:hi]]
        del dst
    out = torch.empty_like(keys)
    tb = lib.apt_sort_u64_temp_bytes(total)
    temp = torch.empty(tb, dtype=torch.uint8, device=dev)
    check(lib.apt_sort_u64(_p(keys), _p(out), total, _p(temp), tb, 2 * bits, _s()))
    del keys, temp
    counts = deg[order]                              # the list of new node k is the list of order[k]
    new_indptr = torch.zeros(n + 1, dtype=torch.int64, device=dev)
    torch.cumsum(counts, 0, out=new_indptr[1:])
    out.bitwise_and_((1 << bits) - 1)
    return new_indptr, out


def intra_partition_edge_share(indptr: torch.Tensor, indices: torch.Tensor, min_vids: torch.Tensor,
                               chunk: int = 1 << 22) -> float:
    """Share of the edges whose endpoints have the same owner under the contiguous ranges min_vids."""
    n = indptr.numel() - 1
    dev = indptr.device
    cuts = min_vids[1:-1].to(dev)
    deg = indptr[1:] - indptr[:-1]
    same = 0
    for first in range(0, n, chunk):
        last = min(n, first + chunk)
        lo, hi = int(indptr[first]), int(indptr[last])
        owner_dst = torch.bucketize(torch.arange(first, last, device=dev), cuts, right=True)
        same += int((torch.repeat_interleave(owner_dst, deg[first:last]) ==
                     torch.bucketize(indices[lo:hi], cuts, right=True)).sum())
    return same / max(indices.numel(), 1)


def zipf_seed_batches(w: Workload, degree_order: torch.Tensor, rank: int, count: int, first_batch: int = 0):
    """`count` batches of w.batch distinct seeds drawn Zipf(w.zipf_s) over the rank by in-degree
    (degree_order[0] is the node of highest in-degree): each batch takes 4 x batch draws of its own
    counter range, maps them to nodes, drops repeats keeping the first occurrence (the relabel kernel
    does exactly that) and keeps the first w.batch."""
    dev = degree_order.device
    per = 4 * w.batch
    out = []
    e = torch.empty(0, dtype=torch.int64, device=dev)
    for b in range(first_batch, first_batch + count):
        ranks = torch.empty(per, dtype=torch.int64, device=dev)
        check(lib.apt_zipf_ranks(w.train_seed + 1000 * rank, b * per, per, degree_order.numel(), float(w.zipf_s),
                                 _p(ranks), _s()))
        uniq, _ = ops.relabel_csc(e, degree_order[ranks - 1])
        if uniq.numel() < w.batch:
            raise RuntimeError(f"{uniq.numel()} distinct seeds out of {per} Zipf draws: fewer than the batch of {w.batch}")
        out.append(uniq[:w.batch].contiguous())
    return out


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
    degree_order: Optional[torch.Tensor] = None     # node ids by falling in-degree (seed_dist == "zipf")


def install(w: Workload, rank=0, world_size=1, row_chunk=1 << 22, tag="bench") -> Installed:
    """Builds the workload on the current GPU and registers it with the operators
    (mix_cache_graphs, cache_feats_shared, register_min_vids)."""
    device = torch.device("cuda", torch.cuda.current_device())
    indptr, indices = build_csc(w, device)
    n = w.num_nodes
    min_vids = partition_min_vids(n, world_size)
    info = {}
    if w.partition == "bfs":
        # locality-preserving partition: renumber by breadth-first order from a seeded root, then the
        # same equal contiguous ranges. The share of edges inside one part is measured, not assumed, for
        # the ids as generated and for the breadth-first renumbering, and the better of the two is installed.
        parts = w.locality_blocks if world_size == 1 else world_size
        probe = partition_min_vids(n, parts)
        before = intra_partition_edge_share(indptr, indices, probe)
        g0 = torch.Generator().manual_seed(w.bfs_root_seed)
        root = int(torch.randint(0, n, (1,), generator=g0))
        order = bfs_order(indptr, indices, root)
        b_indptr, b_indices = relabel_graph(indptr, indices, order)
        del order
        after = intra_partition_edge_share(b_indptr, b_indices, probe)
        if after >= before:
            indptr, indices = b_indptr, b_indices
        del b_indptr, b_indices
        info.update(intra_partition_edge_share=round(max(before, after), 4),
                    intra_partition_edge_share_as_generated=round(before, 4),
                    intra_partition_edge_share_bfs=round(after, 4), partition_used="bfs" if after >= before else
                    "as generated", partition_parts_measured=parts, bfs_root=root)
    e = torch.empty(0, dtype=torch.int64)
    # whole topology resident in HBM: no adjacency cache is needed
    ops.mix_cache_graphs(0, e, e, e, indptr, indices)
    ops.register_min_vids(min_vids)

    deg = indptr[1:] - indptr[:-1]
    esz = torch.empty(0, dtype=_TORCH_DT[w.dtype]).element_size()
    k = int(n * w.cache_frac) if w.cache_bytes is None else min(n, w.cache_bytes // (w.feat_dim * esz))
    order = torch.sort(deg, descending=True, stable=True).indices
    cached_idx = order[:k].contiguous()
    degree_order = order if w.seed_dist == "zipf" else None
    del order, deg
    # When the full host table does not fit host memory it holds host_rows rows and the features repeat
    # with that period (node v has the row of node v mod host_rows), in the cache as in host memory:
    # bytes per row, miss rate and access pattern stay those of the full table.
    host_rows = n if w.host_rows_cap is None else min(n, int(w.host_rows_cap))
    dev_feats = normal_rows(w, device, row_ids=cached_idx % host_rows if host_rows < n else cached_idx)

    host, shm_path = _shared_host_table(w, rank, world_size, tag, rows=host_rows)
    lo = (host_rows * rank) // world_size
    hi = (host_rows * (rank + 1)) // world_size
    for first in range(lo, hi, row_chunk):
        m = min(row_chunk, hi - first)
        host[first:first + m].copy_(normal_rows(w, device, first_row=first, num_rows=m))
    torch.cuda.synchronize()
    if world_size > 1:
        import torch.distributed as dist

        dist.barrier()
    local_idx = torch.arange(host_rows, dtype=torch.int64)
    ops.cache_feats_shared(n, host, dev_feats, cached_idx.cpu(), local_idx, 0)
    if host_rows < n:
        m = ops.STATE.feat.feat_pos_map
        absent = (m == -1).nonzero().view(-1)
        m[absent] = -(absent % host_rows) - 2
        del absent
        ops.STATE.feat._cpu_map_args = None      # the CPU twin of the gather does not model the repeating table
        info["host_rows"] = host_rows

    g = torch.Generator(device=device).manual_seed(w.train_seed)
    n_train = max(w.batch * world_size, int(n * w.train_frac))
    train = torch.randperm(n, generator=g, device=device)[:n_train]
    per = n_train // world_size            # rebalanced evenly (python/npc/ops.py:454-462)
    train_ids = train[rank * per:(rank + 1) * per].contiguous()
    info.update(num_cached_rows=k, num_csc_edges=int(indices.numel()))
    return Installed(w, rank, world_size, indptr, indices, min_vids, host, cached_idx, train_ids, shm_path, info,
                     degree_order)


def seed_batches(inst: Installed, count: int, offset: int = 0):
    """`count` consecutive seed batches of this rank: slices of its training ids (wrapping) or, for
    a Zipf workload, batches of distinct Zipf-distributed seeds."""
    w = inst.workload
    if w.seed_dist == "zipf":
        return zipf_seed_batches(w, inst.degree_order, inst.rank, count, first_batch=offset)
    n = inst.train_ids.numel()
    out = []
    for i in range(count):
        lo = ((offset + i) * w.batch) % max(n - w.batch + 1, 1)
        out.append(inst.train_ids[lo:lo + w.batch].contiguous())
    return out


def cleanup(inst: Installed):
    if inst.shm_path and inst.rank == 0 and os.path.exists(inst.shm_path):
        os.unlink(inst.shm_path)
