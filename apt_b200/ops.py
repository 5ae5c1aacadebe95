"""Host side of the data path: the operators of the reference's ``npc`` library
(``TORCH_LIBRARY(npc, m)``, src/pybind.cc:18-48) with the same names, argument
meaning and result layout, implemented on libapt_b200's C ABI.

PyTorch is used for device memory, streams and ``torch.distributed`` only; all
arithmetic of the path runs in the CUDA library. There is no CPU fallback:
every operator except ``cpu_load_subtensor`` requires CUDA tensors.

State lives in one process-wide object like the reference's ``NPCState``
(src/state.h:32-63): one process drives one GPU.
"""
import ctypes
import os
import threading
from typing import List, Optional, Tuple

import torch

from . import _lib
from ._lib import check, lib

_DTYPE_CODE = {torch.float32: _lib.F32, torch.bfloat16: _lib.BF16, torch.float16: _lib.F16}


def _ptr(t: Optional[torch.Tensor]):
    if t is None or t.numel() == 0:
        return None
    return ctypes.c_void_p(t.data_ptr())


def _stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _need_cuda(t: torch.Tensor, name: str, dtype=torch.int64):
    if not t.is_cuda:
        raise RuntimeError(f"{name} must be a CUDA tensor (apt_b200 has no CPU path)")
    if dtype is not None and t.dtype != dtype:
        raise RuntimeError(f"{name} must have dtype {dtype}, got {t.dtype}")
    return t.contiguous()


def _device_visible(t: torch.Tensor, name: str) -> torch.Tensor:
    """A tensor kernels can dereference: CUDA memory, or page-locked host memory
    (registered here if needed, as the reference's pin_tensor does,
    python/npc/utils/utils.py:70-75)."""
    if t.is_cuda:
        return t.contiguous()
    if not t.is_contiguous():
        raise RuntimeError(f"{name} must be contiguous")
    if t.numel() > 0 and not t.is_pinned():
        from . import hostmem

        hostmem.register(t.data_ptr(), t.numel() * t.element_size())
    return t


class FeatStorage:
    """FeatStorage, src/state.h:10-16."""

    def __init__(self):
        self.dev_feats = None
        self.uva_feats = None
        self.feat_pos_map = None
        self._cpu_feat_pos_map = None
        self._cpu_map_args = None
        self.num_total_nodes = 0
        self.feat_dim = 0
        self.rank_feat_dim = 0
        self.feat_dim_offset = 0

    @property
    def cpu_feat_pos_map(self):
        if self._cpu_feat_pos_map is None and self._cpu_map_args is not None:
            n, localnode_idx = self._cpu_map_args
            m = torch.full((n,), -1, dtype=torch.int64)
            m[localnode_idx] = -torch.arange(localnode_idx.numel(), dtype=torch.int64) - 2
            self._cpu_feat_pos_map = m
        return self._cpu_feat_pos_map


class GraphStorage:
    """GraphStorage, src/state.h:18-23."""

    def __init__(self):
        self.dev_indptr = None
        self.dev_indices = None
        self.uva_indptr = None
        self.uva_indices = None
        self.adj_pos_map = None
        self.num_total_nodes = 0
        self.num_cached_nodes = 0


class NPCState:
    """NPCState, src/state.h:32-63, plus what the CUDA library needs from the
    host: cached workspaces, the device status word and the exchange backend."""

    def __init__(self):
        self.rank = 0
        self.local_rank = 0
        self.world_size = 1
        self.node_size = 1
        self.initialized = False
        self.shuffle_min_vids = None
        self._min_vids_host = None
        self.shuffle_id_offset = 0
        self.graph = GraphStorage()
        self.feat = FeatStorage()
        self.sample_key = 7777777  # the reference's seed constant, src/cuda/npc_kernel.cu:292
        self.sample_calls = 0
        self.sample_replace = True
        self._ws = {}
        self._lane_words = {}
        # mini-batches that run beside one another on the GPU (each on a stream of its own) must not
        # share scratch: workspaces, the word block and the exchange context are kept per lane
        self._tls = threading.local()
        self._lane_exchange = {}
        self._lane_streams = {}
        self.prefetched = None  # (input ids, gathered rows) left by a sampler that gathers ahead
        self.generation = 0     # bumped whenever installed state changes; captured graphs check it
        self.profiling = False
        self.exchange = None  # set by apt_b200.exchange.make_exchange at init
        self.exchange_generation = 0
        self._side_stream = None
        self.shuffle_backend = os.environ.get("APT_SHUFFLE_BACKEND", "p2p")
        self.p2p_region_bytes = int(os.environ.get("APT_P2P_REGION_MB", "256")) << 20
        # inboxes of the lanes beside the first carry the samplers' id exchanges only
        self.p2p_lane_region_bytes = int(os.environ.get("APT_P2P_LANE_REGION_MB", "64")) << 20

    @property
    def lane(self) -> int:
        """The lane whose scratch the calling thread's operators use (0: the caller's own)."""
        return getattr(self._tls, "lane", 0)

    @lane.setter
    def lane(self, value: int):
        self._tls.lane = int(value)

    # -- device scratch --------------------------------------------------
    def device(self):
        return torch.device("cuda", torch.cuda.current_device())

    def workspace(self, name: str, nbytes: int) -> torch.Tensor:
        """A cached, 256-byte aligned scratch tensor of at least nbytes."""
        key = (name, torch.cuda.current_device(), self.lane)
        buf = self._ws.get(key)
        if buf is None or buf.numel() < nbytes:
            buf = torch.empty(max(int(nbytes * 1.25), 1 << 16), dtype=torch.uint8, device=self.device())
            self._ws[key] = buf
        return buf

    def side_stream(self) -> torch.cuda.Stream:
        """A second stream of this device for work that runs beside the main chain of a mini-batch."""
        if self._side_stream is None or self._side_stream.device != self.device():
            self._side_stream = torch.cuda.Stream(device=self.device())
        return self._side_stream

    def lane_stream(self, lane: int) -> torch.cuda.Stream:
        """The one stream on which work that uses lane `lane`'s scratch is enqueued: everything on
        a lane runs in order, whichever sampler put it there."""
        key = (lane, torch.cuda.current_device())
        stream = self._lane_streams.get(key)
        if stream is None:
            stream = self._lane_streams[key] = torch.cuda.Stream(device=self.device())
        return stream

    NUM_WORDS = 256

    def words(self) -> torch.Tensor:
        """int64[256] device words: [0..254] small results (counts a kernel leaves for
        the next kernel and, later, for the host), [255] status flags."""
        pair = self._lane_words.get(self.lane)
        if pair is None or pair[0].device != self.device():
            pair = (torch.zeros(self.NUM_WORDS, dtype=torch.int64, device=self.device()),
                    torch.zeros(self.NUM_WORDS, dtype=torch.int64).pin_memory())
            self._lane_words[self.lane] = pair
        return pair[0]

    def word(self, k: int) -> torch.Tensor:
        """One-element view of device word k (a device-side count)."""
        return self.words()[k:k + 1]

    def status_ptr(self):
        return ctypes.c_void_p(self.words().data_ptr() + 8 * (self.NUM_WORDS - 1))

    def read_words(self) -> torch.Tensor:
        """Copies the device words to the host (one stream sync) and raises on
        any status flag except zero-degree, which is only a notice."""
        w = self.words()
        host = self._lane_words[self.lane][1]
        host.copy_(w, non_blocking=True)
        torch.cuda.current_stream().synchronize()
        self.check_host_words(host)
        return host

    def check_host_words(self, host: torch.Tensor):
        """Raises if a host copy of the word block carries a status flag (zero-degree is a notice)."""
        flags = int(host[self.NUM_WORDS - 1]) & 0xFFFFFFFF
        if flags & ~_lib.FLAG_ZERO_DEGREE:
            self.words()[self.NUM_WORDS - 1] = 0
            raise RuntimeError(f"apt_b200 device status flags 0x{flags:x}: " + _flag_text(flags))


def _flag_text(flags):
    names = {
        _lib.FLAG_ID_OUT_OF_RANGE: "id outside the registered tables",
        _lib.FLAG_FEAT_NOT_EXIST: "feature row neither cached nor in host memory",
        _lib.FLAG_ZERO_DEGREE: "node without in-neighbours sampled",
        _lib.FLAG_TABLE_FULL: "workspace or inbox region too small",
        _lib.FLAG_PEER_TIMEOUT: "a peer's data did not arrive within the wait bound (APT_P2P_TIMEOUT_MS); the "
                                "exchange refuses further use: call init() again on every rank, behind a barrier",
        _lib.FLAG_NOT_GROUPED: "edges of a block are not grouped by destination",
        _lib.FLAG_SIZE_MISMATCH: "a peer sent another number of rows than the reduction expects",
    }
    return ", ".join(v for k, v in names.items() if flags & k)


STATE = NPCState()


def _exchange():
    """The exchange backend; a process that never called init() is a world of one. Lanes other
    than the first get a context of their own on first use (a collective step: every rank has to
    reach it, which holds when the ranks run the same sampler), since the flags of one context
    order its exchanges as one sequence."""
    from .exchange import P2PExchange, make_exchange

    if STATE.exchange is None:
        STATE.exchange = make_exchange(STATE)
    if STATE.lane == 0 or STATE.exchange.name != "p2p" or STATE.world_size == 1:
        return STATE.exchange
    ex = STATE._lane_exchange.get(STATE.lane)
    if ex is None or ex.generation != STATE.exchange_generation:
        ex = P2PExchange(STATE, min(STATE.p2p_region_bytes, STATE.p2p_lane_region_bytes))
        ex.generation = STATE.exchange_generation
        STATE._lane_exchange[STATE.lane] = ex
    return ex


def profile_enable(on: bool):
    """Per-kernel CUDA-event timing (apt_profile_enable). Captured CUDA graphs
    cannot hold timing events, so samplers run eagerly while this is on."""
    STATE.profiling = bool(on)
    check(lib.apt_profile_enable(1 if on else 0))


def check_status():
    """Synchronises and raises if any kernel since the last check flagged an error."""
    STATE.read_words()


# ---------------------------------------------------------------- init / state
def nccl_get_unique_id() -> torch.Tensor:
    """NCCLGetUniqueId, src/core.cc:38-44: int64[16] on the CPU. The exchange
    here rides on torch.distributed's process group, so the id is a
    placeholder kept for callers that broadcast it (python/npc/__init__.py:33-49)."""
    return torch.zeros(16, dtype=torch.int64)


def init(rank: int, local_rank: int, world_size: int, nccl_id_tensor_list: torch.Tensor, node_size: int) -> None:
    """Initialize, src/core.cc:54-100."""
    from .exchange import make_exchange

    s = STATE
    s.rank, s.local_rank, s.world_size, s.node_size = int(rank), int(local_rank), int(world_size), int(node_size)
    torch.cuda.set_device(s.local_rank)
    s.exchange = make_exchange(s)
    s.exchange_generation += 1
    for ex in s._lane_exchange.values():
        ex.close()
    s._lane_exchange = {}
    s.initialized = True
    s.generation += 1


def register_min_vids(shuffle_min_vids: torch.Tensor, shuffle_id_offset: int = 0) -> None:
    """RegisterMinVids, src/core.cc:102-108."""
    mv = shuffle_min_vids.to(device=STATE.device(), dtype=torch.int64).contiguous()
    if mv.numel() != STATE.world_size + 1:
        raise RuntimeError(f"min_vids needs world_size+1 = {STATE.world_size + 1} entries, got {mv.numel()}")
    STATE.shuffle_min_vids = mv
    STATE.generation += 1
    STATE._min_vids_host = [int(x) for x in shuffle_min_vids.cpu().tolist()]
    STATE.shuffle_id_offset = int(shuffle_id_offset)


def mix_cache_graphs(num_cached_nodes: int, cached_node_idx: torch.Tensor, cached_indptr: torch.Tensor,
                     cached_indices: torch.Tensor, global_indptr: torch.Tensor, global_indices: torch.Tensor) -> None:
    """MixCacheGraphs, src/cache_graphs.cc:12-49. The global CSC may be pinned
    host memory (read over the host link, as in the reference) or CUDA memory
    (the whole topology resident in HBM)."""
    g = STATE.graph
    STATE.generation += 1
    if int(num_cached_nodes) != cached_node_idx.numel():
        raise RuntimeError("num_cached_nodes != cached_node_idx.numel()")
    g.num_cached_nodes = int(num_cached_nodes)
    g.num_total_nodes = global_indptr.numel() - 1
    g.uva_indptr = _device_visible(global_indptr, "global_indptr")
    g.uva_indices = _device_visible(global_indices, "global_indices")
    if g.num_cached_nodes > 0:
        g.dev_indptr = _need_cuda(cached_indptr, "cached_indptr")
        g.dev_indices = _need_cuda(cached_indices, "cached_indices")
        m = -torch.arange(g.num_total_nodes, dtype=torch.int64, device=STATE.device()) - 2
        m[cached_node_idx.to(STATE.device())] = torch.arange(g.num_cached_nodes, dtype=torch.int64, device=STATE.device())
        g.adj_pos_map = m
    else:
        # Every node reads the global CSC: the position map would be the
        # identity encoding, so it is not materialised.
        g.dev_indptr = g.dev_indices = g.adj_pos_map = None


def cache_feats_shared(num_total_nodes: int, localnode_feats: torch.Tensor, cached_feats: torch.Tensor,
                       cached_idx: torch.Tensor, localnode_idx: torch.Tensor, feat_dim_offset: int = 0) -> None:
    """CacheFeatsShared, src/cache_feats.cc:14-61."""
    f = STATE.feat
    dev = STATE.device()
    STATE.generation += 1
    if localnode_feats.dim() != 2 or cached_feats.dim() != 2:
        raise RuntimeError("feature tables must be 2-D")
    if cached_feats.dtype != localnode_feats.dtype or cached_feats.dtype not in _DTYPE_CODE:
        raise RuntimeError(f"unsupported feature dtypes {localnode_feats.dtype}/{cached_feats.dtype}")
    f.num_total_nodes = int(num_total_nodes)
    f.uva_feats = _device_visible(localnode_feats, "localnode_feats")
    f.dev_feats = _need_cuda(cached_feats, "cached_feats", dtype=None)
    f.feat_dim = localnode_feats.shape[1]
    f.rank_feat_dim = cached_feats.shape[1]
    f.feat_dim_offset = int(feat_dim_offset)
    m = torch.full((f.num_total_nodes,), -1, dtype=torch.int64, device=dev)
    li = localnode_idx.to(dev)
    m[li] = -torch.arange(li.numel(), dtype=torch.int64, device=dev) - 2
    m[cached_idx.to(dev)] = torch.arange(cached_idx.numel(), dtype=torch.int64, device=dev)
    f.feat_pos_map = m
    f._cpu_feat_pos_map = None
    f._cpu_map_args = (f.num_total_nodes, localnode_idx.cpu())


def set_sampling(key: Optional[int] = None, call_id: Optional[int] = None, replace: Optional[bool] = None):
    """Sampler stream control: draws depend only on (key, call_id, seed slot,
    draw slot); call_id advances by one per sampling call."""
    STATE.generation += 1
    if key is not None:
        STATE.sample_key = int(key)
    if call_id is not None:
        STATE.sample_calls = int(call_id)
    if replace is not None:
        STATE.sample_replace = bool(replace)


# -------------------------------------------------------------------- sampling
def _sample(seeds: torch.Tensor, fanout: int, n_dev: Optional[torch.Tensor] = None,
            call_id: Optional[int] = None, call_base_dev: Optional[torch.Tensor] = None) -> torch.Tensor:
    """n_dev: optional one-element device count; seeds.numel() is then an upper bound.
    call_id / call_base_dev: explicit call id (plus a device-side base) instead of the
    process-wide counter, for sequences replayed from a CUDA graph."""
    g = STATE.graph
    if g.uva_indptr is None:
        raise RuntimeError("mix_cache_graphs has not been called")
    seeds = _need_cuda(seeds, "seeds")
    out = torch.empty(seeds.numel() * int(fanout), dtype=torch.int64, device=seeds.device)
    if call_id is None:
        call_id = STATE.sample_calls
        STATE.sample_calls += 1
    check(lib.apt_sample_csc_fanout(
        _ptr(seeds), seeds.numel(), _ptr(n_dev), int(fanout), _ptr(g.adj_pos_map), g.num_total_nodes,
        _ptr(g.dev_indptr), _ptr(g.dev_indices), _ptr(g.uva_indptr), _ptr(g.uva_indices),
        STATE.sample_key, call_id & 0xFFFFFFFF, _ptr(call_base_dev), 1 if STATE.sample_replace else 0,
        _ptr(out), STATE.status_ptr(), _stream()))
    return out


def local_sample_one_layer(seeds: torch.Tensor, fanout: int) -> List[torch.Tensor]:
    """LocalSamplingNeibhorsOneLayer, src/sampling.cc:13-17: [seeds, neighbors]."""
    return [seeds, _sample(seeds, fanout)]


def _relabel_enqueue(seeds, neighbors, n_dev, count_out):
    """Enqueues the relabelling; the number of unique ids lands in the device
    word `count_out`. Returns the full-length (upper bound) buffers."""
    n = seeds.numel() + neighbors.numel()
    uniq = torch.empty(n, dtype=torch.int64, device=seeds.device)
    rel = torch.empty(neighbors.numel(), dtype=torch.int64, device=seeds.device)
    ws = _relabel_workspace(n)
    check(lib.apt_relabel_csc(_ptr(seeds), seeds.numel(), _ptr(n_dev), _ptr(neighbors), neighbors.numel(),
                              _ptr(ws), ws.numel(), _ptr(uniq), _ptr(rel),
                              _ptr(count_out), STATE.status_ptr(), _stream()))
    return uniq, rel


def _relabel_workspace(n):
    ws = STATE.workspace("relabel", lib.apt_relabel_workspace_bytes(n))
    if getattr(ws, "_apt_clean", False) is not True:
        # the table has to be empty once; every call then releases the slots it used
        check(lib.apt_relabel_workspace_init(_ptr(ws), ws.numel(), _stream()))
        ws._apt_clean = True
    return ws


def _sample_relabel_enqueue(seeds, fanout, n_dev, count_out, call_id=None, call_base_dev=None, want_neighbors=False):
    """One sampled layer, sampling and relabelling together (apt_sample_relabel_csc): returns the
    upper-bound buffers (unique ids, relabelled neighbours, neighbours or None); the number of
    unique ids lands in the device word `count_out`."""
    g = STATE.graph
    if g.uva_indptr is None:
        raise RuntimeError("mix_cache_graphs has not been called")
    if not STATE.sample_replace:
        nbr = _sample(seeds, fanout, n_dev, call_id, call_base_dev)
        uniq, rel = _relabel_enqueue(seeds, nbr, n_dev, count_out)
        return uniq, rel, nbr
    seeds = _need_cuda(seeds, "seeds")
    S, f = seeds.numel(), int(fanout)
    uniq = torch.empty(S * (1 + f), dtype=torch.int64, device=seeds.device)
    rel = torch.empty(S * f, dtype=torch.int64, device=seeds.device)
    nbr = torch.empty(S * f, dtype=torch.int64, device=seeds.device) if want_neighbors else None
    ws = _relabel_workspace(S * (1 + f))
    if call_id is None:
        call_id = STATE.sample_calls
        STATE.sample_calls += 1
    check(lib.apt_sample_relabel_csc(
        _ptr(seeds), S, _ptr(n_dev), f, _ptr(g.adj_pos_map), g.num_total_nodes, _ptr(g.dev_indptr),
        _ptr(g.dev_indices), _ptr(g.uva_indptr), _ptr(g.uva_indices), STATE.sample_key, call_id & 0xFFFFFFFF,
        _ptr(call_base_dev), _ptr(ws), ws.numel(), _ptr(nbr), _ptr(uniq), _ptr(rel), _ptr(count_out),
        STATE.status_ptr(), _stream()))
    return uniq, rel, nbr


def relabel_csc(seeds: torch.Tensor, neighbors: torch.Tensor) -> List[torch.Tensor]:
    """RelabelCSC, src/relabel.cc:9-15: [all_unique, relabeled_neighbors]."""
    seeds = _need_cuda(seeds, "seeds")
    neighbors = _need_cuda(neighbors, "neighbors")
    uniq, rel = _relabel_enqueue(seeds, neighbors, None, STATE.word(0))
    num_unique = int(STATE.read_words()[0])
    return [uniq[:num_unique], rel]


# ---------------------------------------------------------------- seed shuffle
def _bucket(seeds: torch.Tensor, n_dev: Optional[torch.Tensor] = None, sizes: Optional[torch.Tensor] = None,
            offsets: Optional[torch.Tensor] = None):
    """Stable partition by owner: (sorted ids, permutation, sizes[world_size + 1]
    with their total last, inclusive offsets[world_size]). `sizes` / `offsets`
    may be given as preallocated device views."""
    s = STATE
    if s.shuffle_min_vids is None:
        raise RuntimeError("register_min_vids has not been called")
    n = seeds.numel()
    dev = seeds.device
    sorted_ids = torch.empty(n, dtype=torch.int64, device=dev)
    perm = torch.empty(n, dtype=torch.int64, device=dev)
    if sizes is None:
        sizes = torch.empty(s.world_size + 1, dtype=torch.int64, device=dev)
    if offsets is None:
        offsets = torch.empty(s.world_size, dtype=torch.int64, device=dev)
    nbytes = lib.apt_bucket_workspace_bytes(n, s.world_size)
    ws = s.workspace("bucket", nbytes)
    node_beg = s.rank - s.rank % s.node_size
    check(lib.apt_bucket_by_owner(_ptr(seeds), n, _ptr(n_dev), _ptr(s.shuffle_min_vids), s.world_size,
                                  s.shuffle_id_offset,
                                  s.rank, node_beg, node_beg + s.node_size, _ptr(ws), ws.numel(),
                                  _ptr(sorted_ids), _ptr(perm), _ptr(sizes), _ptr(offsets), _stream()))
    return sorted_ids, perm, sizes, offsets


def shuffle_seeds(seeds: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
    """ShuffleSeeds, src/sampling.cc:159-193: (recv_frontier [cuda],
    permutation [cuda], recv_offset [cpu], dev_offset [cpu]); offsets are
    inclusive cumulative counts. Ids of one owner keep their input order."""
    seeds = _need_cuda(seeds, "seeds")
    sorted_ids, perm, sizes, offsets = _bucket(seeds)
    recv, recv_offset, dev_offset = _exchange().exchange_ids(sorted_ids, sizes, offsets)
    return recv, perm, recv_offset, dev_offset


def unique_sorted(ids: torch.Tensor, id_lo: int, id_hi: int):
    """Sorted unique + inverse of ids in [id_lo, id_hi): torch::_unique2(sorted,
    return_inverse) of src/sampling.cc:58-59, via a bitmap over the id range."""
    ids = _need_cuda(ids, "ids")
    uniq, inv = _unique_enqueue(ids, None, id_lo, id_hi, STATE.word(0))
    num_unique = int(STATE.read_words()[0])
    return uniq[:num_unique], inv


def _unique_enqueue(ids, n_dev, id_lo, id_hi, count_out, ws_name="unique"):
    """`ws_name` picks the cached bitmap: callers that alternate between id ranges give
    each range its own, so that none is cleared again on every call."""
    n = ids.numel()
    rng = int(id_hi) - int(id_lo)
    uniq = torch.empty(min(n, max(rng, 0)), dtype=torch.int64, device=ids.device)
    inv = torch.empty(n, dtype=torch.int64, device=ids.device)
    nbytes = lib.apt_unique_workspace_bytes(rng)
    if ws_name != "unique":
        # a bitmap of its own per id range: a captured graph that replays this call must find
        # the layout it was captured with, whatever ran on the shared bitmap in between
        ws_name = f"{ws_name}:{rng}"
    ws = STATE.workspace(ws_name, nbytes)
    if getattr(ws, "_apt_clean_range", None) != rng:
        # the bitmap has to be zero once per id range (the layout follows the range);
        # every call then leaves it zero again
        check(lib.apt_unique_workspace_init(_ptr(ws), ws.numel(), _stream()))
        ws._apt_clean_range = rng
    check(lib.apt_unique_sorted(_ptr(ids), n, _ptr(n_dev), int(id_lo), int(id_hi), _ptr(ws), ws.numel(), _ptr(uniq),
                                _ptr(inv), _ptr(count_out), STATE.status_ptr(), _stream()))
    return uniq, inv


def concat_ids(a: torch.Tensor, na_dev: Optional[torch.Tensor], b: torch.Tensor, nb_dev: Optional[torch.Tensor],
               count_out: torch.Tensor) -> torch.Tensor:
    """cat(a[:na], b[:nb]) with device-side lengths (None: the whole tensor); the result buffer holds
    a.numel() + b.numel() ids and the device word `count_out` receives na + nb."""
    out = torch.empty(a.numel() + b.numel(), dtype=torch.int64, device=a.device)
    check(lib.apt_concat_ids(_ptr(a), a.numel(), _ptr(na_dev), _ptr(b), b.numel(), _ptr(nb_dev), _ptr(out),
                             _ptr(count_out), _stream()))
    return out


def _owned_range():
    """Ids this rank can receive from a seed shuffle. On one machine these are
    the ids it owns; with several machines foreign ids are re-mapped to the
    sender itself (src/cuda/npc_kernel.cu:340-342), so any id may arrive."""
    s = STATE
    n_total = s.graph.num_total_nodes
    if s.node_size == s.world_size and s.shuffle_id_offset == 0 and s._min_vids_host is not None:
        lo = int(s._min_vids_host[s.rank])
        hi = int(s._min_vids_host[s.rank + 1])
        if s.rank == 0:
            lo = min(lo, 0)
        if s.rank == s.world_size - 1:
            hi = max(hi, n_total)
        return lo, hi
    return 0, n_total


def np_sample_and_shuffle(seeds: torch.Tensor, fanout: int) -> List[torch.Tensor]:
    """NPSampleAndShuffle, src/sampling.cc:52-69: [unique_frontier, neighbors,
    permutation, recv_offset, dev_offset, inverse_idx]."""
    recv, perm, recv_offset, dev_offset = shuffle_seeds(seeds)
    lo, hi = _owned_range()
    uniq, inverse_idx = unique_sorted(recv, lo, hi)
    neighbors = _sample(uniq, fanout)
    return [uniq, neighbors, perm, recv_offset, dev_offset, inverse_idx]


def sp_sample_shuffle_src(unique_src: torch.Tensor) -> List[torch.Tensor]:
    """SPSampleShuffleSrc, src/sampling.cc:151-157."""
    return list(shuffle_seeds(unique_src))


# ------------------------------------------------- SNP virtual nodes (SAGE / GCN)
SP_BASE = 10_000_000   # python/npc/sampler.py:181: virtual node = sender * SP_BASE + destination index


def _owner_args():
    s = STATE
    if s.shuffle_min_vids is None:
        raise RuntimeError("register_min_vids has not been called")
    node_beg = s.rank - s.rank % s.node_size
    return _ptr(s.shuffle_min_vids), s.world_size, int(s.shuffle_id_offset), s.rank, node_beg, node_beg + s.node_size


def src_to_vir(fanout: int, num_dst: int, src: torch.Tensor) -> torch.Tensor:
    """SrcToVir, src/sampling.cc:19-34: owner(src[i]) * num_dst + i // fanout."""
    src = _need_cuda(src, "src")
    out = torch.empty_like(src)
    check(lib.apt_src_to_vir(_ptr(src), src.numel(), int(fanout), int(num_dst), *_owner_args(), _ptr(out), _stream()))
    return out


def srcdst_to_vir(fanout: int, dst: torch.Tensor, src: torch.Tensor) -> torch.Tensor:
    """SrcDsttoVir, src/sampling.cc:36-50: destinations first, then the
    neighbours shifted by world_size * num_dst."""
    dst = _need_cuda(dst, "dst")
    src = _need_cuda(src, "src")
    out = torch.empty(dst.numel() + src.numel(), dtype=torch.int64, device=src.device)
    check(lib.apt_srcdst_to_vir(_ptr(dst), dst.numel(), _ptr(src), src.numel(), int(fanout), *_owner_args(),
                                _ptr(out), _stream()))
    return out


def vir_send_sizes(num_seeds: int, sorted_allnodes: torch.Tensor, unique_frontier: torch.Tensor,
                   shuffle_with_dst: int, with_offsets: bool = False):
    """Device tensor of the k = 2 (3 with destinations) sizes per receiver that
    SPSampleAndShuffle exchanges (src/sampling.cc:86-106)."""
    ws = STATE.world_size
    k = 3 if shuffle_with_dst else 2
    sizes = torch.empty(k * ws, dtype=torch.int64, device=sorted_allnodes.device)
    offs = torch.empty(k * ws + 1, dtype=torch.int64, device=sorted_allnodes.device) if with_offsets else None
    check(lib.apt_vir_send_sizes(_ptr(sorted_allnodes), sorted_allnodes.numel(), None, _ptr(unique_frontier),
                                 unique_frontier.numel(), None, ws, int(num_seeds), None, int(bool(shuffle_with_dst)),
                                 _ptr(offs), _ptr(sizes), _stream()))
    return (sizes, offs) if with_offsets else sizes


def sp_pack_frontier(sorted_vir: torch.Tensor, sorted_ids: torch.Tensor, num_dst: int) -> torch.Tensor:
    """rank * SP_BASE * N + (sorted_vir % num_dst) * N + sorted_ids, the packed
    (sender, destination index, neighbour id) of python/npc/sampler.py:296-300."""
    out = torch.empty_like(sorted_ids)
    check(lib.apt_sp_pack_frontier(_ptr(sorted_vir), _ptr(sorted_ids), sorted_ids.numel(), int(num_dst), STATE.rank,
                                   SP_BASE, int(STATE.graph.num_total_nodes), _ptr(out), _stream()))
    return out


def _cumsum_cpu(sizes: torch.Tensor) -> torch.Tensor:
    return sizes.cumsum(0) if sizes.numel() else sizes


def sp_sample_and_shuffle(num_dst: int, send_frontier: torch.Tensor, sorted_allnodes: torch.Tensor,
                          unique_frontier: torch.Tensor, shuffle_with_dst: int) -> List[torch.Tensor]:
    """SPSampleAndShuffle, src/sampling.cc:71-149: [vir_src, ori_src, send_sizes,
    recv_sizes] or, with destinations, [recv_dst, vir_src, ori_src, send_sizes,
    recv_sizes]; the size vectors are CPU int64 as in the reference."""
    send_frontier = _need_cuda(send_frontier, "send_frontier")
    sorted_allnodes = _need_cuda(sorted_allnodes, "sorted_allnodes")
    unique_frontier = _need_cuda(unique_frontier, "unique_frontier")
    s = STATE
    ws = s.world_size
    with_dst = int(bool(shuffle_with_dst))
    k = 3 if with_dst else 2
    ex = _exchange()
    send_sizes_dev = vir_send_sizes(num_dst, sorted_allnodes, unique_frontier, with_dst)
    recv_sizes_dev = torch.empty_like(send_sizes_dev)
    steps = torch.arange(1, ws + 1, dtype=torch.int64) * k
    ex.alltoall(send_sizes_dev, recv_sizes_dev, steps, steps, 1)
    both = torch.stack([send_sizes_dev, recv_sizes_dev]).cpu()
    send_sizes, recv_sizes = both[0].contiguous(), both[1].contiguous()
    n_total = int(s.graph.num_total_nodes)
    dev = send_frontier.device
    if with_dst:
        sd, rd = send_sizes[0::3], recv_sizes[0::3]
        ss, rs = send_sizes[1::3], recv_sizes[1::3]
        n_sd, n_rd, n_rs = int(sd.sum()), int(rd.sum()), int(rs.sum())
        recv_all = torch.empty(n_rd + n_rs, dtype=torch.int64, device=dev)
        ex.alltoall(send_frontier[:n_sd], recv_all[:n_rd], _cumsum_cpu(sd), _cumsum_cpu(rd), 1)
        ex.alltoall(send_frontier[n_sd:], recv_all[n_rd:], _cumsum_cpu(ss), _cumsum_cpu(rs), 1)
        recv_src = recv_all[n_rd:]
    else:
        ss, rs = send_sizes[0::2], recv_sizes[0::2]
        n_rs = int(rs.sum())
        recv_src = torch.empty(n_rs, dtype=torch.int64, device=dev)
        ex.alltoall(send_frontier, recv_src, _cumsum_cpu(ss), _cumsum_cpu(rs), 1)
    vir_src = torch.empty(n_rs, dtype=torch.int64, device=dev)
    ori_src = torch.empty(n_rs, dtype=torch.int64, device=dev)
    check(lib.apt_sp_unpack_frontier(_ptr(recv_src), n_rs, None, n_total, _ptr(vir_src), _ptr(ori_src), _stream()))
    if with_dst:
        return [recv_all[:n_rd], vir_src, ori_src, send_sizes, recv_sizes]
    return [vir_src, ori_src, send_sizes, recv_sizes]


def sp_feat_shuffle(inputs: torch.Tensor, send_sizes: torch.Tensor, recv_sizes: torch.Tensor, total_recv_size: int,
                    expand: int, shuffle_with_dst: int) -> torch.Tensor:
    """SPFeatShuffle, src/feat_shuffle.cc:32-52: rows of `expand` elements; per
    peer q the last of its k sizes (partial sums per virtual node), preceded,
    with destinations, by sizes[3 q] destination rows for every q."""
    if inputs.dtype not in _DTYPE_CODE:
        raise RuntimeError(f"sp_feat_shuffle: unsupported dtype {inputs.dtype}")
    inputs = _need_cuda(inputs, "inputs", dtype=None)
    expand = int(expand)
    rows = inputs.numel() // expand
    flat = inputs.view(rows, expand)
    out = torch.empty((int(total_recv_size), expand), dtype=inputs.dtype, device=inputs.device)
    send_sizes, recv_sizes = send_sizes.cpu(), recv_sizes.cpu()
    ex = _exchange()
    if shuffle_with_dst:
        sd, rd = send_sizes[0::3], recv_sizes[0::3]
        sv, rv = send_sizes[2::3], recv_sizes[2::3]
        n_sd, n_rd = int(sd.sum()), int(rd.sum())
        if n_sd + int(sv.sum()) != rows or n_rd + int(rv.sum()) != int(total_recv_size):
            raise RuntimeError("sp_feat_shuffle: sizes do not add up to the rows given")
        ex.alltoall(flat[:n_sd], out[:n_rd], _cumsum_cpu(sd), _cumsum_cpu(rd), expand)
        ex.alltoall(flat[n_sd:], out[n_rd:], _cumsum_cpu(sv), _cumsum_cpu(rv), expand)
    else:
        sv, rv = send_sizes[1::2], recv_sizes[1::2]
        if int(sv.sum()) != rows or int(rv.sum()) != int(total_recv_size):
            raise RuntimeError("sp_feat_shuffle: sizes do not add up to the rows given")
        ex.alltoall(flat, out, _cumsum_cpu(sv), _cumsum_cpu(rv), expand)
    return out


# ------------------------------------------- NFP (feature dimension partitioned)
def mp_sample_shuffle(seeds: torch.Tensor, unique_frontier: torch.Tensor, coo_row: torch.Tensor) -> List[torch.Tensor]:
    """MPSampleShuffle, src/sampling.cc:195-239: every rank receives every
    rank's frontier and relabelled rows. [recv_frontier, recv_coo_row,
    [seeds_size] (cpu), recv_seeds_size (cpu), recv_frontier_size (cpu),
    recv_coo_size (cpu)]."""
    unique_frontier = _need_cuda(unique_frontier, "unique_frontier")
    coo_row = _need_cuda(coo_row, "coo_row")
    ws = STATE.world_size
    ex = _exchange()
    mine = torch.tensor([[seeds.numel(), unique_frontier.numel(), coo_row.numel()]], dtype=torch.int64,
                        device=unique_frontier.device)
    sizes = ex.allbroadcast(mine, [1] * ws).cpu()                       # [ws, 3]
    recv_seeds_size = sizes[:, 0].contiguous()
    recv_frontier_size = sizes[:, 1].contiguous()
    recv_coo_size = sizes[:, 2].contiguous()
    recv_frontier = ex.allbroadcast(unique_frontier.view(-1, 1), recv_frontier_size.tolist()).view(-1)
    recv_coo_row = ex.allbroadcast(coo_row.view(-1, 1), recv_coo_size.tolist()).view(-1)
    return [recv_frontier, recv_coo_row, torch.tensor([seeds.numel()]), recv_seeds_size, recv_frontier_size,
            recv_coo_size]


def mp_feat_shuffle_fwd(inputs: torch.Tensor, send_size: torch.Tensor, recv_size: torch.Tensor,
                        feat_dim: int) -> torch.Tensor:
    """MPFeatShuffleFwd, src/feat_shuffle.cc:54-64 (a reduce-scatter): rows
    [off[r], off[r] + send_size[r]) of every rank's inputs are summed on rank r,
    which gets recv_size rows. The sum runs over the ranks in rank order in fp32."""
    if inputs.dtype not in _DTYPE_CODE:
        raise RuntimeError(f"mp_feat_shuffle_fwd: unsupported dtype {inputs.dtype}")
    inputs = _need_cuda(inputs, "inputs", dtype=None)
    feat_dim = int(feat_dim)
    flat = inputs.view(inputs.numel() // feat_dim, feat_dim)
    send_size = send_size.cpu().to(torch.int64).view(-1)
    mine = int(recv_size.view(-1)[0])
    if int(send_size.sum()) != flat.shape[0] or int(send_size[STATE.rank]) != mine:
        raise RuntimeError("mp_feat_shuffle_fwd: sizes do not match the rows given")
    return _exchange().reduce_scatter(flat, send_size, mine)


def mp_feat_shuffle_bwd(inputs: torch.Tensor, send_size: torch.Tensor, recv_size: torch.Tensor,
                        feat_dim: int) -> torch.Tensor:
    """MPFeatShuffleBwd, src/feat_shuffle.cc:66-79 (an all-gather of blocks of
    different lengths): every rank receives every rank's rows in rank order."""
    inputs = _need_cuda(inputs, "inputs", dtype=None)
    feat_dim = int(feat_dim)
    flat = inputs.view(inputs.numel() // feat_dim, feat_dim)
    if int(send_size.view(-1)[0]) != flat.shape[0]:
        raise RuntimeError("mp_feat_shuffle_bwd: send_size does not match the rows given")
    return _exchange().allbroadcast(flat, [int(x) for x in recv_size.view(-1).tolist()])


# ---------------------------------------------------------------------- gather
def load_subtensor(node_id: torch.Tensor) -> torch.Tensor:
    """LoadSubtensor, src/load_subtensor.cc:19-40: rows of the GPU cache or,
    on a miss, of the page-locked host table, in one call."""
    f = STATE.feat
    if f.feat_pos_map is None:
        raise RuntimeError("cache_feats_shared has not been called")
    node_id = _need_cuda(node_id, "node_id")
    pre = STATE.prefetched
    if pre is not None:
        STATE.prefetched = None
        ids, rows = pre
        if ids.data_ptr() == node_id.data_ptr() and ids.numel() == node_id.numel():
            return rows
    return _gather_enqueue(node_id, None)


def _gather_enqueue(node_id: torch.Tensor, n_dev: Optional[torch.Tensor], out: Optional[torch.Tensor] = None,
                    first_dev: Optional[torch.Tensor] = None, ws_name: str = "gather") -> torch.Tensor:
    """Enqueues the gather of rows [first_dev, n_dev) of node_id (device words; None: 0 and
    node_id.numel()) into `out` (allocated here when None). Calls that may overlap on the GPU
    need workspaces of their own (`ws_name`)."""
    f = STATE.feat
    n = node_id.numel()
    esz = f.dev_feats.element_size()
    if out is None:
        out = torch.empty((n, f.rank_feat_dim), dtype=f.dev_feats.dtype, device=node_id.device)
    nbytes = lib.apt_gather_workspace_bytes(n)
    ws = STATE.workspace(ws_name, nbytes)
    check(lib.apt_gather_rows_from(
        _ptr(node_id), n, _ptr(n_dev), _ptr(first_dev), _ptr(f.feat_pos_map), f.num_total_nodes,
        _ptr(f.dev_feats), f.dev_feats.shape[0], f.rank_feat_dim * esz,
        _ptr(f.uva_feats), f.uva_feats.shape[0], f.feat_dim * esz, f.feat_dim_offset * esz,
        _ptr(out), _ptr(ws), ws.numel(), STATE.status_ptr(), _stream()))
    return out


def cpu_load_subtensor(node_id: torch.Tensor) -> torch.Tensor:
    """CPULoadSubtensor, src/load_subtensor.cc:10-17: host table only, on the
    CPU, as the reference does it (two index_selects)."""
    f = STATE.feat
    pos = -f.cpu_feat_pos_map.index_select(0, node_id.cpu()) - 2
    table = f.uva_feats if not f.uva_feats.is_cuda else f.uva_feats.cpu()
    return table.index_select(0, pos)


# -------------------------------------------------------------- feature shuffle
def feat_shuffle(inputs: torch.Tensor, send_offset: torch.Tensor, recv_offset: torch.Tensor,
                 permutation: torch.Tensor, feat_dim: int, fwd_flag: int) -> torch.Tensor:
    """FeatShuffle, src/feat_shuffle.cc:9-30. Offsets are CPU int64 inclusive
    cumulative row counts. fwd: rows travel to the ranks that asked for them
    and come out in the asker's original seed order (``buf[permutation]``);
    bwd: rows are scattered by permutation and travel back."""
    if inputs.dtype not in _DTYPE_CODE:
        raise RuntimeError(f"feat_shuffle: unsupported dtype {inputs.dtype}")
    inputs = _need_cuda(inputs, "inputs", dtype=None)
    permutation = _need_cuda(permutation, "permutation")
    rows_in = inputs.numel() // int(feat_dim)
    return _exchange().exchange_rows(inputs.view(rows_in, int(feat_dim)), send_offset, recv_offset,
                                        permutation, bool(fwd_flag))


def alltoall(input: torch.Tensor, output: torch.Tensor, send_offset: torch.Tensor, recv_offset: torch.Tensor,
             expand: int = 1, comm_type: int = 0) -> None:
    """AlltoAll, src/ops/collective.cc:252-266: in place into `output`; any
    dtype (the reference silently ignores everything but int64/fp32)."""
    _exchange().alltoall(_need_cuda(input, "input", dtype=None), output, send_offset, recv_offset, int(expand))


# ---------------------------------------------------------------- SpMM / SDDMM
def _spmm(op, coo_row, coo_col, inp, edata, coo_offset, input_offset, output_offset):
    ref = inp if inp is not None else edata
    if ref.dtype not in _DTYPE_CODE:
        raise RuntimeError(f"spmm: unsupported dtype {ref.dtype}")
    coo_row = _need_cuda(coo_row, "coo_row")
    coo_col = _need_cuda(coo_col, "coo_col")
    coo_offset = _need_cuda(coo_offset, "coo_offset")
    output_offset = _need_cuda(output_offset, "output_offset")
    if input_offset is not None:
        input_offset = _need_cuda(input_offset, "input_offset")
    ref = _need_cuda(ref, "input", dtype=None)
    if inp is not None:
        inp = ref
    if edata is not None:
        edata = _need_cuda(edata, "edata", dtype=ref.dtype)
    out_num = int(output_offset[-1].item())  # host read, as in src/spmm.cc:13
    num_edges = coo_row.numel()
    feat_dim = inp.shape[1] if inp is not None else edata.numel() // max(num_edges, 1)
    # edata may be [E, D], [E, H] or [E, H, 1]: one value per column or per head
    edim = edata.numel() // num_edges if edata is not None and num_edges else feat_dim
    out = torch.empty((out_num, feat_dim), dtype=ref.dtype, device=ref.device)
    nbytes = lib.apt_spmm_workspace_bytes(out_num, num_edges)
    ws = STATE.workspace("spmm", nbytes)
    check(lib.apt_spmm_sum(op, _DTYPE_CODE[ref.dtype], _ptr(coo_row), _ptr(coo_col), coo_row.numel(),
                           _ptr(inp), _ptr(edata), int(edim), int(feat_dim), _ptr(coo_offset),
                           _ptr(input_offset), _ptr(output_offset), coo_offset.numel() - 1, out_num,
                           _ptr(out), _ptr(ws), ws.numel(), _stream()))
    return out


def spmm_copy_u_sum(coo_row, coo_col, input, coo_offset, input_offset, output_offset):
    """CopyUSum, src/spmm.cc:9-19."""
    return _spmm(0, coo_row, coo_col, input, None, coo_offset, input_offset, output_offset)


def spmm_copy_e_sum(coo_row, coo_col, input, coo_offset, output_offset):
    """CopyESum, src/spmm.cc:21-29: `input` holds one row per edge."""
    return _spmm(1, coo_row, coo_col, None, input, coo_offset, None, output_offset)


def spmm_u_mul_e_sum(coo_row, coo_col, input, edata, coo_offset, input_offset, output_offset, ref_quirk_add=False):
    """UMulESum, src/spmm.cc:31-42: sum over edges of input[src] * edata[e].
    The reference's kernel adds instead of multiplying (src/cuda/spmm.cu:78);
    ref_quirk_add=True reproduces that."""
    return _spmm(3 if ref_quirk_add else 2, coo_row, coo_col, input, edata, coo_offset, input_offset, output_offset)


def _sddmm(op, coo_row, coo_col, lhs, rhs, coo_offset, lhs_offset, rhs_offset):
    if lhs.dtype not in _DTYPE_CODE or rhs.dtype != lhs.dtype:
        raise RuntimeError(f"sddmm: unsupported dtypes {lhs.dtype}/{rhs.dtype}")
    coo_row = _need_cuda(coo_row, "coo_row")
    coo_col = _need_cuda(coo_col, "coo_col")
    lhs = _need_cuda(lhs, "lhs", dtype=None)
    rhs = _need_cuda(rhs, "rhs", dtype=None)
    coo_offset = _need_cuda(coo_offset, "coo_offset")
    lhs_offset = _need_cuda(lhs_offset, "lhs_offset")
    rhs_offset = _need_cuda(rhs_offset, "rhs_offset")
    out = torch.empty((coo_row.numel(), lhs.shape[1]), dtype=lhs.dtype, device=lhs.device)
    check(lib.apt_sddmm(op, _DTYPE_CODE[lhs.dtype], _ptr(coo_row), _ptr(coo_col), coo_row.numel(), _ptr(lhs),
                        _ptr(rhs), lhs.shape[1], _ptr(coo_offset), _ptr(lhs_offset), _ptr(rhs_offset),
                        coo_offset.numel() - 1, _ptr(out), _stream()))
    return out


def sddmm_u_add_v(coo_row, coo_col, lhs, rhs, coo_offset, lhs_offset, rhs_offset):
    """UAddV, src/sddmm.cc:9-19."""
    return _sddmm(0, coo_row, coo_col, lhs, rhs, coo_offset, lhs_offset, rhs_offset)


def sddmm_u_mul_v(coo_row, coo_col, lhs, rhs, coo_offset, lhs_offset, rhs_offset):
    """UMulV, src/sddmm.cc:21-31."""
    return _sddmm(1, coo_row, coo_col, lhs, rhs, coo_offset, lhs_offset, rhs_offset)


def gat_edge_softmax_sum(coo_row, coo_col, ft, el, er, num_dst: int, negative_slope: float = 0.2,
                         return_attention: bool = False):
    """One sampled block of a GAT layer in one kernel: u_add_v(el, er) -> leaky_relu ->
    edge_softmax -> u_mul_e(ft, a) summed per destination (the DGL calls of
    python/npc/model/gatconv.py:113-124). ft [num_src, H, Dh] or [num_src, H*Dh],
    el [num_src, H(,1)], er [num_dst, H(,1)]; edges grouped by destination.
    Returns out [num_dst, H, Dh] (and the attention [E, H, 1])."""
    if ft.dtype not in _DTYPE_CODE or el.dtype != ft.dtype or er.dtype != ft.dtype:
        raise RuntimeError(f"gat_edge_softmax_sum: unsupported dtypes {ft.dtype}/{el.dtype}/{er.dtype}")
    coo_row = _need_cuda(coo_row, "coo_row")
    coo_col = _need_cuda(coo_col, "coo_col")
    ft = _need_cuda(ft, "ft", dtype=None)
    el = _need_cuda(el, "el", dtype=None)
    er = _need_cuda(er, "er", dtype=None)
    num_src = ft.shape[0]
    heads = el.numel() // max(num_src, 1) if num_src else er.numel() // max(num_dst, 1)
    head_dim = ft.numel() // max(num_src * heads, 1)
    out = torch.empty((num_dst, heads, head_dim), dtype=ft.dtype, device=ft.device)
    attn = torch.empty((coo_row.numel(), heads, 1), dtype=ft.dtype, device=ft.device) if return_attention else None
    nbytes = lib.apt_spmm_workspace_bytes(num_dst, 0)
    ws = STATE.workspace("spmm", nbytes)
    check(lib.apt_gat_edge_softmax_sum(_DTYPE_CODE[ft.dtype], _ptr(coo_row), _ptr(coo_col), coo_row.numel(),
                                       _ptr(ft), _ptr(el), _ptr(er), int(heads), int(head_dim),
                                       float(negative_slope), int(num_dst), _ptr(out), _ptr(attn), _ptr(ws),
                                       ws.numel(), STATE.status_ptr(), _stream()))
    return (out, attn) if return_attention else out


def _spmm_single(op, in_index, out_index, inp, edata, edim, feat_dim, num_in, num_out):
    """apt_spmm_sum over one segment with the sizes known on the host (no read of an
    offset tensor): out[out_index[e]] += f(inp[in_index[e]], edata[e])."""
    ref = inp if inp is not None else edata
    E = in_index.numel()
    off = torch.tensor([0, E, 0, num_in, 0, num_out], dtype=torch.int64).to(ref.device, non_blocking=True)
    out = torch.empty((num_out, feat_dim), dtype=ref.dtype, device=ref.device)
    ws = STATE.workspace("spmm", lib.apt_spmm_workspace_bytes(num_out, E))
    check(lib.apt_spmm_sum(op, _DTYPE_CODE[ref.dtype], _ptr(in_index), _ptr(out_index), E, _ptr(inp), _ptr(edata),
                           int(edim), int(feat_dim), _ptr(off[0:2]), _ptr(off[2:4]), _ptr(off[4:6]), 1, int(num_out),
                           _ptr(out), _ptr(ws), ws.numel(), _stream()))
    return out


def gat_edge_softmax_sum_backward(coo_row, coo_col, ft, el, er, grad_out, negative_slope: float = 0.2):
    """Gradients of gat_edge_softmax_sum with respect to ft, el and er for
    grad_out [num_dst, H, Dh]: one kernel over the destinations (softmax and
    leaky_relu backward per edge, grad_er), then the two sums over the source side
    as SpMM calls in the reverse direction. Returns (grad_ft, grad_el, grad_er)
    shaped like ft, el, er."""
    if ft.dtype not in _DTYPE_CODE or any(t.dtype != ft.dtype for t in (el, er, grad_out)):
        raise RuntimeError("gat_edge_softmax_sum_backward: unsupported or mixed dtypes")
    coo_row = _need_cuda(coo_row, "coo_row")
    coo_col = _need_cuda(coo_col, "coo_col")
    ft = _need_cuda(ft, "ft", dtype=None)
    el = _need_cuda(el, "el", dtype=None)
    er = _need_cuda(er, "er", dtype=None)
    grad_out = _need_cuda(grad_out, "grad_out", dtype=None)
    num_src, num_dst, E = ft.shape[0], grad_out.shape[0], coo_row.numel()
    heads = el.numel() // max(num_src, 1) if num_src else er.numel() // max(num_dst, 1)
    head_dim = ft.numel() // max(num_src * heads, 1)
    dev, dt = ft.device, ft.dtype
    attn = torch.empty((E, heads), dtype=dt, device=dev)
    gscore = torch.empty((E, heads), dtype=dt, device=dev)
    grad_er = torch.empty((num_dst, heads), dtype=dt, device=dev)
    ws = STATE.workspace("spmm", lib.apt_spmm_workspace_bytes(num_dst, 0))
    check(lib.apt_gat_edge_backward(_DTYPE_CODE[dt], _ptr(coo_row), _ptr(coo_col), E, _ptr(ft), _ptr(el), _ptr(er),
                                    _ptr(grad_out), int(heads), int(head_dim), float(negative_slope), int(num_dst),
                                    _ptr(attn), _ptr(gscore), _ptr(grad_er), _ptr(ws), ws.numel(),
                                    STATE.status_ptr(), _stream()))
    if E == 0 or num_src == 0:
        return torch.zeros_like(ft), torch.zeros_like(el), grad_er.view(er.shape)
    width = heads * head_dim
    grad_ft = _spmm_single(2, coo_col, coo_row, grad_out.view(num_dst, width), attn, heads, width, num_dst, num_src)
    grad_el = _spmm_single(1, coo_col, coo_row, None, gscore, heads, heads, num_dst, num_src)
    return grad_ft.view(ft.shape), grad_el.view(el.shape), grad_er.view(er.shape)


class GATEdgeSoftmaxSum(torch.autograd.Function):
    """gat_edge_softmax_sum with its backward, for use inside a model:
    ``out = GATEdgeSoftmaxSum.apply(coo_row, coo_col, ft, el, er, num_dst, slope)``."""

    @staticmethod
    def forward(ctx, coo_row, coo_col, ft, el, er, num_dst, negative_slope=0.2):
        ctx.save_for_backward(coo_row, coo_col, ft, el, er)
        ctx.slope = float(negative_slope)
        return gat_edge_softmax_sum(coo_row, coo_col, ft, el, er, int(num_dst), float(negative_slope))

    @staticmethod
    def backward(ctx, grad_out):
        coo_row, coo_col, ft, el, er = ctx.saved_tensors
        g_ft, g_el, g_er = gat_edge_softmax_sum_backward(coo_row, coo_col, ft, el, er, grad_out.contiguous(), ctx.slope)
        return None, None, g_ft, g_el, g_er, None, None


# ------------------------------------------------------------------ row movers
def rows_gather(inp: torch.Tensor, index: torch.Tensor) -> torch.Tensor:
    """out[i] = inp[index[i]] for 2-D inp (the model's h[inverse_idx],
    python/npc/model/sage_model.py:67)."""
    inp = _need_cuda(inp, "inp", dtype=None)
    index = _need_cuda(index, "index")
    out = torch.empty((index.numel(), inp.shape[1]), dtype=inp.dtype, device=inp.device)
    check(lib.apt_rows_gather(_ptr(inp), _ptr(index), index.numel(), inp.shape[1] * inp.element_size(),
                              _ptr(out), _stream()))
    return out


def rows_scatter(inp: torch.Tensor, index: torch.Tensor, num_out_rows: int) -> torch.Tensor:
    """out[index[i]] = inp[i]; rows of out not named by index are zero."""
    inp = _need_cuda(inp, "inp", dtype=None)
    index = _need_cuda(index, "index")
    alloc = torch.empty if index.numel() == num_out_rows else torch.zeros
    out = alloc((num_out_rows, inp.shape[1]), dtype=inp.dtype, device=inp.device)
    check(lib.apt_rows_scatter(_ptr(inp), _ptr(index), index.numel(), inp.shape[1] * inp.element_size(),
                               _ptr(out), _stream()))
    return out
