"""Dry run, cache policy and strategy cost model (the "adaptive" part of APT)
on top of the data path: python/npc/cost_model/estimator.py, the cache
selection of python/npc/ops.py:107-274 and the counters of examples/dryrun.py.

The reference keeps the access counters on the host (``freq[ids.cpu()] += 1``
per mini-batch) and sorts them with torch on the CPU; here the counters live
in HBM, the mini-batch ids never leave the device, and the order and the hit
volume come from kernels (csrc/hotness.cu). The arithmetic that turns volumes
into times is the reference's, with its bandwidth constants as defaults.
"""
import time
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence

import torch
import torch.distributed as dist

from . import ops
from ._lib import check, lib
from .sampler import SPVirtualSampler, create_block

BYTES_PER_ELEMENT = 4
# MiB/s, python/npc/cost_model/estimator.py:16-20 (measured by its authors on their machines)
REFERENCE_BW = {"pcie": 5594.79, "gpu": 5782.60, "network": 4616.41, "pure_network": 3831.46}
# MiB/s on the B200 boxes this library was measured on: cold random 512-byte rows from pinned host
# memory (25 GB/s), HBM copy (6543 GB/s), NVLink peer copy per direction (770 GB/s)
B200_BW = {"pcie": 25e9 / 2 ** 20, "gpu": 6542.7e9 / 2 ** 20, "network": 770e9 / 2 ** 20,
           "pure_network": 770e9 / 2 ** 20}


_COUNT_SLOT = 120   # device word of the state block taking the distinct-id count


def _ptr(t):
    return ops._ptr(t)


class HotnessCounter:
    """int32 access counters of all nodes on the device."""

    def __init__(self, num_nodes: int, device=None):
        self.num_nodes = int(num_nodes)
        self.counters = torch.zeros(self.num_nodes, dtype=torch.int32, device=device or ops.STATE.device())

    def add(self, ids: torch.Tensor, distinct: bool = False) -> None:
        """counters[ids] += 1 as torch's indexed ``+= 1`` does it (estimator.py:433-436):
        an id named several times in one call still counts once. Unless the caller
        vouches for distinct ids they go through the bitmap unique first, whose
        count stays on the device."""
        ids = ops._need_cuda(ids, "ids")
        n_dev = None
        if not distinct and ids.numel():
            n_dev = ops.STATE.word(_COUNT_SLOT)
            ids, _ = ops._unique_enqueue(ids, None, 0, self.num_nodes, n_dev)
        check(lib.apt_hotness_add(_ptr(ids), ids.numel(), _ptr(n_dev), _ptr(self.counters), self.num_nodes,
                                  ops.STATE.status_ptr(), ops._stream()))

    def zero(self) -> None:
        self.counters.zero_()

    def sorted_idx(self) -> torch.Tensor:
        return hot_order(self.counters)


def hot_order(freq: torch.Tensor) -> torch.Tensor:
    """Node ids by falling frequency (``torch.sort(freq, descending=True)[1]``,
    estimator.py:26, :208-209); equal frequencies by rising id."""
    freq = ops._need_cuda(freq, "freq", dtype=torch.int32)
    n = freq.numel()
    out = torch.empty(n, dtype=torch.int64, device=freq.device)
    nbytes = lib.apt_hot_order_workspace_bytes(n)
    ws = torch.empty(nbytes, dtype=torch.uint8, device=freq.device)
    check(lib.apt_hot_order(_ptr(freq), n, _ptr(ws), ws.numel(), _ptr(out), ops._stream()))
    return out


def cached_access(freq: torch.Tensor, sorted_idx: torch.Tensor, num_cache_nodes: int):
    """(all accesses, accesses served by a cache of the first num_cache_nodes of sorted_idx)."""
    freq = ops._need_cuda(freq, "freq", dtype=torch.int32)
    sorted_idx = ops._need_cuda(sorted_idx, "sorted_idx")
    out = torch.empty(2, dtype=torch.int64, device=freq.device)
    check(lib.apt_cached_access(_ptr(freq), freq.numel(), _ptr(sorted_idx), int(num_cache_nodes), _ptr(out),
                                ops._stream()))
    total, cached = out.tolist()
    return total, cached


def get_cache_miss(seeds_freq: torch.Tensor, num_cache_nodes: int, input_dim: int,
                   made_seeds_freq: Optional[torch.Tensor] = None) -> int:
    """get_cache_miss, estimator.py:22-30: elements read past a cache of the
    num_cache_nodes hottest nodes of made_seeds_freq."""
    order = hot_order(seeds_freq if made_seeds_freq is None else made_seeds_freq)
    total, cached = cached_access(seeds_freq, order, min(int(num_cache_nodes), seeds_freq.numel()))
    return (total - cached) * int(input_dim)


def cachemiss_vol_to_time(vol: float, bw: Dict[str, float] = REFERENCE_BW, bytes_per_element: int = BYTES_PER_ELEMENT):
    """estimator.py:112-113."""
    return vol * bytes_per_element / (1024 * 1024 * bw["pcie"])


def reshuffle_vol_to_time(vol: float, bw: Dict[str, float] = REFERENCE_BW,
                          bytes_per_element: int = BYTES_PER_ELEMENT):
    """estimator.py:116-118. The reference picks BW_NETWORK whenever
    args.nproc_per_node is non-zero, and its single-machine value is -1, so every
    run it makes takes BW_NETWORK; kept."""
    return vol * bytes_per_element / (1024 * 1024 * bw["network"])


def get_featload_time(seeds_freq: torch.Tensor, num_gpu_cache_nodes: int, input_dim: int,
                      gpu_sorted_idx: Optional[torch.Tensor] = None, bw: Dict[str, float] = REFERENCE_BW) -> float:
    """get_featload_time on one machine, estimator.py:53-70."""
    if gpu_sorted_idx is None:
        gpu_sorted_idx = hot_order(seeds_freq)
    total, cached = cached_access(seeds_freq, gpu_sorted_idx, min(int(num_gpu_cache_nodes), seeds_freq.numel()))
    return cachemiss_vol_to_time((total - cached) * int(input_dim), bw)


def get_reshuffle_dim(model: str, num_hidden: int, num_heads: int = 1) -> int:
    """estimator.py:121-122."""
    return num_hidden if model != "GAT" else num_hidden * num_heads


def get_dp_reshuffle_vol() -> int:
    return 0


def get_np_reshuffle_vol(world_size: int, rank: int, send_offset, recv_offset, dim: int) -> int:
    """estimator.py:129-144: rows sent to and received from the other ranks, both
    directions of the layer (forward and backward)."""
    so = [int(x) for x in send_offset.tolist()]
    ro = [int(x) for x in recv_offset.tolist()]
    total_send = so[world_size - 1] - so[rank] + (so[rank - 1] if rank > 0 else 0)
    total_recv = ro[world_size - 1] - ro[rank] + (ro[rank - 1] if rank > 0 else 0)
    return 2 * dim * (total_send + total_recv)


def get_sp_reshuffle_vol(world_size: int, rank: int, send_sizes, recv_sizes, dim: int, model: str = "SAGE",
                         shuffle_with_dst: bool = False) -> int:
    """estimator.py:147-178."""
    if model == "GAT":
        return get_np_reshuffle_vol(world_size, rank, send_sizes, recv_sizes, dim)
    ss = [int(x) for x in send_sizes.tolist()]
    rs = [int(x) for x in recv_sizes.tolist()]
    vol = 0
    for r in range(world_size):
        if r == rank:
            continue
        if shuffle_with_dst:
            vol += 2 * dim * (ss[3 * r] + ss[3 * r + 2] + rs[3 * r] + rs[3 * r + 2])
        else:
            vol += 2 * dim * (ss[2 * r + 1] + rs[2 * r + 1])
    return vol


def get_mp_reshuffle_vol(world_size: int, send_size, recv_size, dim: int) -> int:
    """estimator.py:181-188."""
    return 2 * dim * (int(send_size.view(-1)[0]) * (world_size - 2) + int(recv_size.sum()))


def select_cache_nodes(sorted_idx: torch.Tensor, localnode_mask: torch.Tensor, cache_memory: int, input_dim: int,
                       base: int = 1) -> torch.Tensor:
    """The "dryrun" cache mode, python/npc/ops.py:233-243: the hottest nodes whose rows
    this process holds, as many as cache_memory bytes take (base = world_size for
    NFP, whose rows are world_size times narrower)."""
    local_sorted = torch.masked_select(sorted_idx, localnode_mask[sorted_idx])
    k = min(local_sorted.numel(), int(cache_memory * base / (input_dim * BYTES_PER_ELEMENT)))
    return local_sorted[:k]


def select_cache_costmodel(sorted_idx: torch.Tensor, idx_mem: torch.Tensor, cache_memory: int,
                           num_total_nodes: int):
    """The "costmodel" cache mode, python/npc/ops.py:118-142. `sorted_idx` ranks 2 N candidates by
    benefit per byte: entry v < N is node v's feature row, entry N + v node v's adjacency list;
    `idx_mem[c]` is candidate c's size in bytes. The first candidates whose sizes add up to at most
    cache_memory are cached (the reference stops one short of the first prefix that exceeds the
    budget). Returns (feature node ids, adjacency node ids), each in rank order."""
    sorted_idx = sorted_idx.to(torch.int64)
    cumsum = torch.cumsum(idx_mem.to(torch.int64)[sorted_idx], 0)
    over = cumsum > int(cache_memory)
    # torch.max over a bool vector returns the first True (or index 0 when none is set)
    first_over = int(torch.max(over, 0)[1]) if over.numel() else 0
    k = max(0, first_over - 1)
    head = sorted_idx[:k]
    return head[head < num_total_nodes], head[head >= num_total_nodes] - num_total_nodes


def select_cache_greedy(feat_idx: torch.Tensor, graph_idx: torch.Tensor, mem_usage: torch.Tensor, cache_memory: int,
                        feat_ratio: float, num_total_nodes: int):
    """The "greedy" cache mode, python/npc/ops.py:144-180: feature rows and adjacency lists are
    ranked separately; a binary search finds the largest m such that the first m * feat_ratio
    feature rows plus the first m * (1 - feat_ratio) adjacency lists fit cache_memory. Returns
    (feature node ids, adjacency node ids)."""
    mem_usage = mem_usage.to(torch.int64)
    feat_mem = torch.cumsum(mem_usage[feat_idx], 0)
    graph_mem = torch.cumsum(mem_usage[graph_idx + num_total_nodes], 0)
    lb, ub = 0, int(num_total_nodes)
    while ub > lb + 1:
        mid = (ub + lb) // 2
        total = int(feat_mem[int(mid * feat_ratio)]) + int(graph_mem[int(mid * (1 - feat_ratio))])
        if total <= cache_memory:
            lb = mid
        else:
            ub = mid
    return feat_idx[:int(lb * feat_ratio)], graph_idx[:int(lb * (1 - feat_ratio))]


def dryrun_cache_order(system: str, rank: int, input_freqs: Sequence[torch.Tensor], min_vids=None) -> torch.Tensor:
    """Node order the "dryrun" cache mode caches by on one machine, python/npc/ops.py:197-230, from
    the per-rank input-node frequencies of a dry run (entry [1] of every rank's rk#{r}_epo100.pt):
    NP ranks by this rank's own counts; GDP and NFP by the counts summed over the ranks (every rank
    gets the same order); SNP by the summed counts of the nodes this rank owns (the others count as
    never used)."""
    if system == "NP":
        return torch.sort(input_freqs[rank], descending=True)[1]
    total = torch.stack(list(input_freqs), 0).sum(0)
    if system in ("MP", "DP"):
        return torch.sort(total, descending=True)[1]
    if system == "SP":
        own = torch.zeros_like(total)
        lo, hi = int(min_vids[rank]), int(min_vids[rank + 1])
        own[lo:hi] = total[lo:hi]
        return torch.sort(own, descending=True)[1]
    raise ValueError(f"unknown system {system!r}")


def cache_adj_and_feats(cache_mode: str, rank: int, localnode_feats_idx: torch.Tensor, num_total_nodes: int, *,
                        cache_memory: int = 0, input_dim: int = 0, system: str = "NP", world_size: int = 1,
                        sorted_idx: Optional[torch.Tensor] = None, idx_mem: Optional[torch.Tensor] = None,
                        greedy_idx=None, greedy_feat_ratio: float = 0.5, input_freqs=None, min_vids=None,
                        feat_cache_ratio: float = 0.0, generator: Optional[torch.Generator] = None):
    """cache_adj_and_feats, python/npc/ops.py:107-274, with the files it loads handed in as tensors:
    which nodes' feature rows and which nodes' adjacency lists this rank caches. Returns (feature
    node ids, adjacency node ids); the first goes to cache_feats_shared, the second, with the rows
    it names, to mix_cache_graphs. Modes: "costmodel" (sorted_idx + idx_mem), "greedy" (greedy_idx =
    (feature order, adjacency order) + idx_mem), "dryrun" (input_freqs of all ranks; no adjacency
    cache), anything else: a random feat_cache_ratio of the local rows."""
    none = torch.empty(0, dtype=torch.int64)
    if cache_mode == "costmodel":
        return select_cache_costmodel(sorted_idx, idx_mem, cache_memory, num_total_nodes)
    if cache_mode == "greedy":
        return select_cache_greedy(greedy_idx[0], greedy_idx[1], idx_mem, cache_memory, greedy_feat_ratio,
                                   num_total_nodes)
    if cache_mode == "dryrun":
        order = dryrun_cache_order(system, rank, input_freqs, min_vids)
        mask = torch.zeros(num_total_nodes, dtype=torch.bool)
        mask[localnode_feats_idx] = True
        return select_cache_nodes(order, mask, cache_memory, input_dim, world_size if system == "MP" else 1), none
    n_local = localnode_feats_idx.numel()
    k = int(feat_cache_ratio * n_local)
    return localnode_feats_idx[torch.randperm(n_local, generator=generator)[:k]], none


def append_costmodel_csv(path: str, result: "CostModelResult", *, tag: str, world_size: int, model: str,
                         batch_size: int, input_dim: int, num_hidden: int, num_heads: int, fan_out: str,
                         cache_mode: str, cache_memory: int, cache_value, warmup_epochs: int, dryrun_epochs: int,
                         num_record_steps: int, warmup_time: float, dryrun_time: float) -> None:
    """The four rows (one per strategy) the reference's cost model appends to its log,
    python/npc/cost_model/estimator.py:643-689: the run's description, the strategy, its sampling,
    feature-loading and reshuffle milliseconds rounded to 0.01, and their sum."""
    import csv

    info = [tag, world_size, model, batch_size, input_dim, num_hidden, num_heads, fan_out, cache_mode,
            f"{round(cache_memory / (1024 * 1024 * 1024))}GB", cache_value, warmup_epochs, dryrun_epochs,
            num_record_steps, round(warmup_time, 2), round(dryrun_time, 2)]
    with open(path, "a") as f:
        writer = csv.writer(f, lineterminator="\n")
        for system in ("DP", "NP", "SP", "MP"):
            record = result.records[system]
            writer.writerow(info + [system] + [round(v, 2) for v in record] + [round(sum(record), 2)])


def save_dryrun(path: str, seeds_counter: torch.Tensor, input_counter: torch.Tensor) -> None:
    """The file a dry run leaves per rank (rk#{r}_epo{n}.pt, examples/dryrun.py:86-108):
    a list of two int64 CPU tensors, [1] being the input-node frequencies the cache
    policy reads (python/npc/ops.py:196-201)."""
    torch.save([seeds_counter.to("cpu", torch.int64), input_counter.to("cpu", torch.int64)], path)


def load_dryrun(path: str) -> torch.Tensor:
    return torch.load(path)[1]


class AllStrategySampler:
    """AllPSNeighborSampler, python/npc/sampler.py:372-600: the inner hops once,
    then the outermost hop under all four strategies (GDP, NP, SNP, NFP), so that
    one dry run yields every strategy's input nodes and exchange sizes. Returns
    ((dp_seeds,), (np_seeds, send_offset, recv_offset), (sp_seeds, send_sizes,
    recv_sizes), (mp_seeds, send_size, recv_size)). SAGE / GCN only."""

    def __init__(self, rank: int, fanouts: List[int], model: str = "SAGE", shuffle_with_dst: bool = False):
        self.rank = rank
        self.fanouts = list(fanouts)
        self.num_layers = len(fanouts)
        self.model = model
        self._sp = SPVirtualSampler(rank, fanouts, model=model, shuffle_with_dst=shuffle_with_dst)
        self.clear_time_list()

    def clear_time_list(self):
        self.num_sample_times = 0
        self.time_list = [0.0, 0.0, 0.0, 0.0]
        self.sampling_algo_time = [0.0 for _ in range(self.num_layers)]

    def get_time_list(self):
        return self.num_sample_times, self.sampling_algo_time, self.time_list

    @staticmethod
    def _now():
        torch.cuda.synchronize()
        return time.perf_counter()

    def sample(self, graph, seeds: torch.Tensor):
        self.num_sample_times += 1
        now = self._now
        for layer_id, fanout in enumerate(reversed(self.fanouts)):
            last = layer_id == self.num_layers - 1
            if last:
                t0 = now()
                np_seeds, np_neighbors, _, np_send_offset, np_recv_offset, _ = ops.np_sample_and_shuffle(seeds, fanout)
                self.time_list[1] += now() - t0
            t0 = now()
            seeds, neighbors = ops.local_sample_one_layer(seeds, fanout)
            if not last:
                seeds = create_block(seeds, neighbors, fanout).src_ids
                self.sampling_algo_time[layer_id] += now() - t0
                continue
            self.sampling_algo_time[layer_id] += now() - t0
            t0 = now()
            dp_seeds = ops.relabel_csc(seeds, neighbors)[0]
            self.time_list[0] += now() - t0
            t0 = now()
            np_seeds = ops.relabel_csc(np_seeds, np_neighbors)[0]
            self.time_list[1] += now() - t0
            t0 = now()
            sp_seeds, _, _, sp_send_sizes, sp_recv_sizes = self._sp._outer(seeds, neighbors, fanout)
            self.time_list[2] += now() - t0
            t0 = now()
            unique_frontier, coo_row = ops.relabel_csc(seeds, neighbors)
            mp_seeds, _, mp_send_size, mp_recv_size, _, _ = ops.mp_sample_shuffle(seeds, unique_frontier, coo_row)
            self.time_list[3] += now() - t0
        return ((dp_seeds,), (np_seeds, np_send_offset, np_recv_offset), (sp_seeds, sp_send_sizes, sp_recv_sizes),
                (mp_seeds, mp_send_size, mp_recv_size))


@dataclass
class CostModelResult:
    """Milliseconds per dry-run epoch and strategy: [sampling, feature loading, reshuffle]."""
    records: Dict[str, List[float]] = field(default_factory=dict)
    best: str = ""
    volumes: Dict[str, float] = field(default_factory=dict)

    def total(self, name: str) -> float:
        return float(sum(self.records[name]))


def run_costmodel(sampler: AllStrategySampler, epochs: Sequence[Sequence[torch.Tensor]], num_total_nodes: int,
                  cache_memory: int, input_dim: int, num_hidden: int, model: str = "SAGE", num_heads: int = 1,
                  mp_input_dim: Optional[int] = None, sorted_idx: Optional[Dict[str, torch.Tensor]] = None,
                  bw: Dict[str, float] = REFERENCE_BW, group=None) -> CostModelResult:
    """run_costmodel on one machine, estimator.py:283-697: dry-runs `epochs` (a list
    of lists of seed batches) through all four strategies, counts the input nodes,
    adds up the exchange volumes, and estimates per strategy sampling + feature
    loading past a cache of cache_memory bytes + reshuffle; the maximum over the
    ranks decides, the smallest sum wins. `sorted_idx` may carry the cache orders
    of an earlier dry run ("ori", "npc", "sp": estimator.py:191-226); otherwise they
    come from this run's own counters."""
    st = ops.STATE
    rank, ws = st.rank, st.world_size
    multi = ws > 1 and dist.is_initialized()
    names = ("DP", "NP", "SP", "MP")
    dim = get_reshuffle_dim(model, num_hidden, num_heads)
    counters = {k: HotnessCounter(num_total_nodes) for k in names}
    freq_sum = {k: torch.zeros(num_total_nodes, dtype=torch.float32, device=st.device()) for k in names}
    vol_lists = {k: [] for k in names}
    sampler.clear_time_list()
    for batches in epochs:
        vols = dict.fromkeys(names, 0)
        for c in counters.values():
            c.zero()
        for seeds in batches:
            (dp_seeds,), (np_seeds, np_so, np_ro), (sp_seeds, sp_ss, sp_rs), (mp_seeds, mp_s, mp_r) = \
                sampler.sample(None, seeds)
            counters["DP"].add(dp_seeds, distinct=True)
            counters["NP"].add(np_seeds, distinct=True)
            counters["SP"].add(sp_seeds)
            counters["MP"].add(mp_seeds)
            vols["DP"] += get_dp_reshuffle_vol()
            vols["NP"] += get_np_reshuffle_vol(ws, rank, np_so, np_ro, dim)
            vols["SP"] += get_sp_reshuffle_vol(ws, rank, sp_ss, sp_rs, dim, model, sampler._sp.shuffle_with_dst)
            vols["MP"] += get_mp_reshuffle_vol(ws, mp_s, mp_r, dim)
        for k in names:
            freq_sum[k] += counters[k].counters.float()
            vol_lists[k].append(vols[k])
    n_epochs = max(len(epochs), 1)
    # mean over the epochs, truncated to int32 as in estimator.py:471-474
    freq = {k: (freq_sum[k] / n_epochs).to(torch.int32) for k in names}
    vol = {k: float(sum(v)) / n_epochs for k, v in vol_lists.items()}
    _, algo, other = sampler.get_time_list()
    sampling = {"DP": sum(algo) + other[0], "NP": sum(algo[:-1]) + other[1], "SP": sum(algo) + other[2],
                "MP": sum(algo) + other[3]}
    if sorted_idx is None:
        ori = freq["DP"].clone()
        if multi:
            dist.all_reduce(ori, group=group)
        lo, hi = ops._owned_range()
        sp_freq = torch.zeros_like(ori)
        sp_freq[lo:hi] = ori[lo:hi]
        sorted_idx = {"ori": hot_order(ori), "npc": hot_order(freq["NP"]), "sp": hot_order(sp_freq)}
    k_cache = int(cache_memory / (input_dim * BYTES_PER_ELEMENT))
    mp_dim = int(mp_input_dim) if mp_input_dim is not None else input_dim // ws
    load = {"DP": get_featload_time(freq["DP"], k_cache, input_dim, sorted_idx["ori"], bw),
            "NP": get_featload_time(freq["NP"], k_cache, input_dim, sorted_idx["npc"], bw),
            "SP": get_featload_time(freq["SP"], k_cache, input_dim, sorted_idx["sp"], bw),
            "MP": get_featload_time(freq["MP"], k_cache * ws, mp_dim, sorted_idx["ori"], bw)}
    vals = []
    for k in names:
        vals += [sampling[k], load[k], reshuffle_vol_to_time(vol[k], bw)]
    t = torch.tensor(vals, dtype=torch.float32, device=st.device()) / n_epochs
    if multi:
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    ms = [v * 1000.0 for v in t.tolist()]
    res = CostModelResult(volumes=vol)
    for i, k in enumerate(names):
        res.records[k] = ms[3 * i:3 * i + 3]
    res.best = min(names, key=res.total)
    ops.check_status()
    return res
