"""Multi-layer samplers of the data path without DGL: the loops of
MixedNeighborSampler (NP, python/npc/sampler.py:109-156) and of the DP branch
of MixedPSNeighborSampler (:187-203), returning blocks as plain COO tensors
instead of DGLBlock objects (DGL builds those from the same COO,
python/npc/sampler.py:59-91).

By default the whole mini-batch is enqueued without the host ever waiting for
an intermediate size: each operator takes its element count from the device
word the previous one wrote, buffers are sized for the no-duplicate upper
bound, and one read at the end brings every count to the host, where the
buffers are narrowed to their real lengths. The results are identical to
calling the operators one by one (``chained=False``), which reads a count
after every relabelling like the reference does (src/cuda/relabel.cu:119).
"""
import itertools
import os
import queue
import threading
from dataclasses import dataclass
from typing import List

import torch
import torch.distributed as dist

from . import ops
from ._lib import check, lib


@dataclass
class Block:
    """One sampled bipartite layer: edge e runs src coo_row[e] -> dst coo_col[e];
    src_ids[k] is the global id of local src k, and the first num_dst src nodes
    are the dst nodes (create_dgl_block, python/npc/sampler.py:76-91)."""

    coo_row: torch.Tensor
    coo_col: torch.Tensor
    num_src: int
    num_dst: int
    src_ids: torch.Tensor
    fanout: int


_COL_CACHE = {}


def _coo_col(num_dst_max: int, num_dst: int, fanout: int, device) -> torch.Tensor:
    """arange(num_dst).repeat_interleave(fanout) (python/npc/sampler.py:78) as a
    prefix of a cached longer one."""
    key = (fanout, device)
    col = _COL_CACHE.get(key)
    if col is None or col.numel() < num_dst_max * fanout:
        col = torch.arange(0, num_dst_max, device=device).repeat_interleave(fanout)
        _COL_CACHE[key] = col
    return col[:num_dst * fanout]


def create_block(seeds: torch.Tensor, neighbors: torch.Tensor, fanout: int) -> Block:
    unique_frontier, indices = ops.relabel_csc(seeds, neighbors)
    coo_col = torch.arange(0, seeds.numel(), device=indices.device).repeat_interleave(fanout)
    return Block(indices, coo_col, unique_frontier.numel(), seeds.numel(), unique_frontier, fanout)


# Upper-bound buffers beyond this many bytes of gathered rows are not gathered
# ahead of the size read; the gather then runs right after it with exact sizes.
_PREFETCH_LIMIT_BYTES = 6 << 30


class _Plan:
    """Buffers of one enqueued mini-batch and, when captured, the CUDA graph
    that replays the enqueue."""

    def __init__(self):
        self.seeds_buf = None
        self.bufs = None
        self.graph = None
        self.generation = -1
        self.keepalive = None
        # pipelined use (sample_iter): the batch's own copy of the word block, the event behind that
        # copy, and its own pinned word for the call-id base
        self.host_words = None
        self.done = None
        self.host_base = None
        # the lane whose scratch the plan was built on; with more than one lane, the lane's stream
        # and the event that orders a new launch behind the consumer of the plan's last results
        self.lane = 0
        self.stream = None
        self.ready = None
        self.ring_size = 1      # buffer sets of this plan's shape: as many mini-batches may be in flight


_CALL_BASE_SLOT = 100  # device word holding the sampler's call-id base for graph replays


def _tunable_from_env(name: str, default: int = 0) -> int:
    for pair in os.environ.get("APT_TUNABLES", "").split(","):
        key, _, value = pair.partition("=")
        if key.strip() == name and value.strip():
            return int(value)
    return default


# what the process runs with outside a lane's capture (APT_TUNABLES may have set it)
_MISS_KB_DEFAULT = _tunable_from_env("gather_miss_kb_per_block")


class _Ring:
    """The buffer sets (plans) of one batch shape, taken in turn."""

    def __init__(self, count):
        self.plans = [None] * count
        self.turn = 0
        self.sized = False


class _GraphReplay:
    """What the chained samplers share: the whole mini-batch is enqueued by `_enqueue(seeds, base_dev)`
    without a host read and narrowed by `_finish(seeds, bufs, host)` after one copy of the device word
    block; the enqueue is captured once per batch shape as a CUDA graph and replayed, from
    `graph_buffers` buffer sets in turn. `sample_iter` launches mini-batch k + 1 before it reads
    mini-batch k back. Subclasses set `num_calls` (sampling calls per mini-batch).

    With `lanes` > 1 (APT_SAMPLER_LANES, default 8) the buffer sets of `sample_iter` also get
    scratch of their own (workspaces, word block, exchange context: a "lane" of the operator state)
    and a stream of their own, so that the mini-batches it keeps in flight run beside one another
    on the GPU instead of one behind the other: most kernels of a mini-batch wait on dependent
    loads at low occupancy and leave room for another mini-batch's. sample() is not affected."""

    use_graph = True
    graph_buffers = 2
    lanes = 1
    num_calls = 1

    def _init_replay(self, use_graph, graph_buffers=2, lanes=None):
        if use_graph is None:
            use_graph = os.environ.get("APT_SAMPLER_GRAPH", "1") != "0"
        self.use_graph = bool(use_graph)
        if lanes is None:
            lanes = int(os.environ.get("APT_SAMPLER_LANES", "8"))
        self.lanes = max(1, min(int(lanes), 16))
        self.plans_per_lane = max(1, min(int(os.environ.get("APT_SAMPLER_PLANS_PER_LANE", "2")), 4))
        self.graph_buffers = max(1, int(graph_buffers))
        self._plans = {}
        # device memory the buffer sets of one batch shape may take together (APT_SAMPLER_PLAN_GB)
        self.plan_budget_bytes = int(float(os.environ.get("APT_SAMPLER_PLAN_GB", "40")) * (1 << 30))
        # KiB to fetch per block of the copy from host memory inside a lane's graph (0: all blocks)
        self.miss_kb_per_block = int(os.environ.get("APT_SAMPLER_MISS_KB_PER_BLOCK", "128"))
        # launches of sample_iter on a thread of their own (APT_SAMPLER_THREAD)
        self.launch_thread = os.environ.get("APT_SAMPLER_THREAD", "0") == "1"

    def _graph_ok(self):
        st = ops.STATE
        # the library all-to-all (baseline backend) reads sizes on the host and cannot be captured;
        # timing events cannot live in a captured graph either
        return self.use_graph and not st.profiling and ops._exchange().name in ("local", "p2p")

    def _in_flight(self):
        """Buffer sets sample_iter takes turns with. With lanes every lane has `plans_per_lane` of them:
        a lane's next replay is then already queued on its stream when the running one ends, and the
        lane does not idle while the host reads the finished mini-batch back and hands it out."""
        if self.lanes > 1:
            return max(self.graph_buffers, self.lanes * self.plans_per_lane)
        return self.graph_buffers

    def buffer_sets(self):
        """Buffer sets sample_iter really takes turns with: the number asked for, or fewer once the
        memory budget has cut a shape's ring."""
        sizes = [len(ring.plans) for key, ring in self._plans.items() if key[2]]
        return min(sizes) if sizes else self._in_flight()

    def _plan_for(self, seeds, piped=False):
        """The plan the next mini-batch of this shape runs on. sample() takes `graph_buffers` plans in
        turn on the caller's stream; sample_iter (piped) has plans of its own, on lanes when lanes > 1."""
        st = ops.STATE
        on_lanes = piped and self.lanes > 1
        dev = seeds.device if seeds.is_cuda else st.device()
        key = (seeds.numel(), dev, piped)
        ring = self._plans.get(key)
        if ring is None:
            ring = self._plans[key] = _Ring(self._in_flight() if piped else self.graph_buffers)
        i = ring.turn % len(ring.plans)
        ring.turn += 1
        plan = ring.plans[i]
        if plan is not None and plan.generation == st.generation:
            return plan
        before = torch.cuda.memory_allocated(dev)
        plan = _Plan()
        plan.generation = st.generation
        plan.seeds_buf = torch.empty(seeds.numel(), dtype=torch.int64, device=dev)
        plan.seeds_buf.copy_(seeds)
        plan.host_words = torch.zeros(st.NUM_WORDS, dtype=torch.int64).pin_memory()
        plan.host_base = torch.zeros(1, dtype=torch.int64).pin_memory()
        plan.done = torch.cuda.Event()
        if on_lanes:
            # lane 0 stays with the caller: its exchange context also carries the feature shuffles
            # the model side runs on its own stream while the samplers' lanes are in flight
            plan.lane = 1 + i % self.lanes
            plan.stream = st.lane_stream(plan.lane)
            plan.ready = torch.cuda.Event()
            torch.cuda.synchronize()     # no other lane's mini-batch is in flight while this one is built
        st.lane = plan.lane
        try:
            if on_lanes:
                # a launch's grid is fixed when it is captured: on a lane the copy from host memory keeps
                # only the blocks its bytes ask for, the SM slots of the others go to the kernels of the
                # mini-batches beside it (C1, eight lanes: 6700 -> 7460 mini-batches/s)
                check(lib.apt_set_tunable(b"gather_miss_kb_per_block", self.miss_kb_per_block))
            base_dev = st.word(_CALL_BASE_SLOT)
            # one eager run first: it sizes the cached workspaces and surfaces errors outside capture
            bufs = self._enqueue(plan.seeds_buf, base_dev)
            st.read_words()
            st.prefetched = None
            del bufs
            plan.graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(plan.graph):
                # the two small host copies are nodes of the graph: the call-id base is read from the
                # plan's pinned word when the replay runs, and the word block lands in the plan's
                # pinned copy behind the last kernel
                # (apt_memcpy_async and not Tensor.copy_: the latter also records an event for the
                # pinned block, which may not be queried once it was recorded in a capture)
                check(lib.apt_memcpy_async(ops._ptr(base_dev), ops._ptr(plan.host_base), 8, ops._stream()))
                plan.bufs = self._enqueue(plan.seeds_buf, base_dev)
                check(lib.apt_memcpy_async(ops._ptr(plan.host_words), ops._ptr(st.words()), 8 * st.NUM_WORDS,
                                           ops._stream()))
            plan.keepalive = [v for k, v in st._ws.items() if k[2] == plan.lane]
        finally:
            st.lane = 0
            if on_lanes:
                check(lib.apt_set_tunable(b"gather_miss_kb_per_block", _MISS_KB_DEFAULT))
        ring.plans[i] = plan
        if piped and not ring.sized:
            # the first buffer set of a shape tells what one costs: keep as many as fit the budget
            # (buffers are sized for the no-duplicate upper bound, times world_size for what is received)
            ring.sized = True
            each = max(1, torch.cuda.memory_allocated(dev) - before)
            fit = max(2, int(self.plan_budget_bytes // each))
            if st.world_size > 1 and dist.is_available() and dist.is_initialized():
                # the ranks take their lanes in the same turn: they have to agree on the number
                agreed = torch.tensor([fit], dtype=torch.int64, device=dev)
                dist.all_reduce(agreed, op=dist.ReduceOp.MIN)
                fit = int(agreed.item())
            if i == 0 and fit < len(ring.plans):
                del ring.plans[fit:]
        plan.ring_size = len(ring.plans)
        return plan

    def _replay(self, plan, seeds):
        """Enqueues one replay of `plan` for `seeds` and records `plan.done` behind it: on the current
        stream, or, with lanes, on the plan's own stream behind everything the current stream holds
        so far (the seeds' producer and the consumer of the plan's previous results)."""
        st = ops.STATE
        plan.host_base[0] = st.sample_calls
        st.sample_calls += self.num_calls
        # explicit streams throughout: looking the current stream up costs more host time than a launch
        cur = torch.cuda.current_stream()
        if plan.stream is None:
            plan.seeds_buf.copy_(seeds, non_blocking=True)
            plan.graph.replay()
            plan.done.record(cur)
            return
        plan.ready.record(cur)
        plan.stream.wait_event(plan.ready)
        torch.cuda.set_stream(plan.stream)
        try:
            plan.seeds_buf.copy_(seeds, non_blocking=True)
            plan.graph.replay()
        finally:
            torch.cuda.set_stream(cur)
        plan.done.record(plan.stream)

    def _sample_chained(self, seeds: torch.Tensor):
        seeds = ops._need_cuda(seeds, "seeds")
        if not self._graph_ok():
            return self._finish(seeds, self._enqueue(seeds, None))
        return self._collect(self._launch(seeds, piped=False))

    def sample_iter(self, graph, seed_batches):
        """Yields what sample() returns for every tensor of `seed_batches`, with the next mini-batch
        already enqueued while the previous one is read back and handed out, so that the GPU never
        waits for the host between mini-batches (the role a prefetching DataLoader has around the
        reference's sampler, examples/train.py:85-94). Needs the CUDA-graph path; otherwise it falls
        back to one sample() per batch. A mini-batch's tensors stay valid until the next one has
        been asked for (the buffer sets take turns). The seed batches may be CUDA tensors or int64
        tensors in page-locked host memory; the latter are copied straight into the plan's buffer,
        and the output nodes handed out are then that buffer."""
        depth = self._in_flight()
        if not (getattr(self, "chained", True) and self._graph_ok() and depth >= 2):
            for seeds in seed_batches:
                yield self.sample(graph, seeds if seeds.is_cuda else seeds.to(ops.STATE.device()))
            return
        if self.launch_thread:
            yield from self._iter_threaded(seed_batches, depth)
            return
        # all buffer sets but one are in flight behind the mini-batch the caller holds
        pending = []
        for seeds in seed_batches:
            pending.append(self._launch(seeds))
            if len(pending) >= min(p[0].ring_size for p in pending):
                yield self._collect(pending.pop(0))
        while pending:
            yield self._collect(pending.pop(0))

    def _iter_threaded(self, seed_batches, depth):
        """sample_iter with the launches on a thread of their own: the driver's part of a graph launch
        runs without the interpreter lock, beside the caller's thread narrowing the previous
        mini-batch. A buffer set is launched on again only after the caller asked for the mini-batch
        behind the one it held; plans are built (captured, inboxes created) by the calling thread."""
        out_q, handback = queue.SimpleQueue(), queue.SimpleQueue()
        slots = threading.Semaphore(depth)
        stop = threading.Event()
        device = torch.cuda.current_device()
        stream = torch.cuda.current_stream()

        def launcher():
            try:
                torch.cuda.set_device(device)
                torch.cuda.set_stream(stream)
                for seeds in seed_batches:
                    slots.acquire()
                    if stop.is_set():
                        return
                    if self._has_plan(seeds):
                        out_q.put(("launched", self._launch(seeds)))
                    else:
                        out_q.put(("build", seeds))
                        handback.get()            # the calling thread built the plan and launched on it
                out_q.put(("end", None))
            except BaseException as exc:          # handed to the calling thread, which raises it
                out_q.put(("error", exc))

        thread = threading.Thread(target=launcher, name="apt-sampler-launch", daemon=True)
        thread.start()
        try:
            while True:
                kind, item = out_q.get()
                if kind == "end":
                    break
                if kind == "error":
                    raise item
                if kind == "build":
                    item = self._launch(item)
                    while depth > item[0].ring_size:      # fewer buffer sets than asked for: give permits back
                        slots.acquire()
                        depth -= 1
                    handback.put(None)
                yield self._collect(item)
                slots.release()
        finally:
            stop.set()
            slots.release()
            handback.put(None)
            thread.join(timeout=60)

    def _has_plan(self, seeds):
        """True when the plan the next piped launch of this shape takes exists already."""
        st = ops.STATE
        dev = seeds.device if seeds.is_cuda else st.device()
        ring = self._plans.get((seeds.numel(), dev, True))
        if ring is None:
            return False
        plan = ring.plans[ring.turn % len(ring.plans)]
        return plan is not None and plan.generation == st.generation

    def _launch(self, seeds, piped=True):
        if seeds.is_cuda or not piped:
            seeds = ops._need_cuda(seeds, "seeds")
        elif seeds.dtype != torch.int64 or not seeds.is_contiguous():
            seeds = seeds.to(torch.int64).contiguous()
        plan = self._plan_for(seeds, piped)
        self._replay(plan, seeds)
        # seeds handed over in host memory went straight into the plan's buffer, which then stands for them
        return plan, (seeds if seeds.is_cuda else plan.seeds_buf)

    def _collect(self, launched):
        plan, seeds = launched
        plan.done.synchronize()
        st = ops.STATE
        st.lane = plan.lane
        try:
            st.check_host_words(plan.host_words)
            return self._finish(seeds, plan.bufs, plan.host_words)
        finally:
            st.lane = 0



class MixedNeighborSampler(_GraphReplay):
    """NP ("NPC") strategy: inner hops are sampled locally, the outermost hop at
    the owner of each frontier node (np_sample_and_shuffle). fanouts[0] is the
    outermost hop, as in the reference's --fan_out (python/npc/utils/utils.py:428-432).

    chained            enqueue the whole mini-batch with device-side sizes (one host
                       read per batch) instead of one read per operator
    prefetch_features  also enqueue the feature gather of the input nodes before that
                       read; the next ops.load_subtensor(input_nodes) returns it
    use_graph          capture the enqueue once per batch size as a CUDA graph and
                       replay it (one launch per mini-batch). The results of a batch
                       live in the graph's buffers: they stay valid until
                       `graph_buffers` further batches have been sampled.
    lanes              buffer sets with scratch and a stream of their own, so that the
                       mini-batches sample_iter keeps in flight overlap on the GPU
                       (default: APT_SAMPLER_LANES, else 8)
    """

    def __init__(self, rank: int, fanouts: List[int], chained: bool = None, prefetch_features: bool = True,
                 use_graph: bool = None, graph_buffers: int = 2, lanes: int = None):
        self.rank = rank
        self.fir_fanouts = list(fanouts[1:])
        self.las_fanouts = fanouts[0]
        self.num_layers = len(fanouts)
        if chained is None:
            chained = os.environ.get("APT_CHAINED_SAMPLER", "1") != "0"
        self.chained = chained
        self.prefetch_features = prefetch_features
        self._init_replay(use_graph, graph_buffers, lanes)
        self.use_graph = self.use_graph and chained
        self.num_calls = self.num_layers
        # 0 (default): one gather after the outermost hop; 1: the frontier's rows are gathered on a second
        # stream beside the outermost hop and the two meet before the remaining rows are gathered; 2: they
        # meet at the end. Measured on the papers-shaped run, 1 and 2 are slower (0.371 and 0.374 ms per
        # mini-batch against 0.340): kernels that share SMs with the host-memory reads of the miss copy
        # slow down by more than the overlap wins.
        self.gather_split = int(os.environ.get("APT_GATHER_SPLIT", "0"))

    def sample(self, graph, seeds: torch.Tensor):
        if self.chained:
            return self._sample_chained(seeds)
        output_nodes = seeds
        blocks = []
        for fanout in reversed(self.fir_fanouts):
            seeds, neighbors = ops.local_sample_one_layer(seeds, fanout)
            block = create_block(seeds, neighbors, fanout)
            seeds = block.src_ids
            blocks.insert(0, block)
        seeds, neighbors, perm, send_offset, recv_offset, inverse_idx = ops.np_sample_and_shuffle(
            seeds, self.las_fanouts)
        block = create_block(seeds, neighbors, self.las_fanouts)
        blocks.insert(0, block)
        seeds = block.src_ids
        return seeds, output_nodes, blocks, perm, send_offset, recv_offset, inverse_idx

    # ------------------------------------------------------------ chained path
    def _enqueue(self, seeds: torch.Tensor, call_base_dev):
        """Enqueues every kernel of the mini-batch on the current stream; no host
        read. With call_base_dev the k-th sampling call uses call id base + k."""
        st = ops.STATE
        ws = st.world_size
        if self.num_layers > 14:
            raise RuntimeError("the chained sampler keeps at most 14 hop counts")
        explicit = call_base_dev is not None
        slot = 0
        call = 0
        cur, cur_n = seeds, None
        layers = []                      # (dst buffer, rel, uniq, uniq count slot, fanout)
        for fanout in reversed(self.fir_fanouts):
            cnt = st.word(slot)
            uniq, rel, _ = ops._sample_relabel_enqueue(cur, fanout, cur_n, cnt, call if explicit else None,
                                                       call_base_dev)
            call += 1
            layers.append((cur, rel, uniq, slot, fanout))
            cur, cur_n = uniq, cnt
            slot += 1
        # outermost hop at the owners (NPSampleAndShuffle, src/sampling.cc:52-69)
        # counts the host needs are written straight into the word block by the kernels:
        # [0..15] hop counts, [16..48] ids received per peer (+ total), [64..95] my bucket offsets,
        # [100] call-id base of graph replays, [128..160] bucket sizes when they are not what is received
        words = st.words()
        recv_view = words[16:16 + ws + 1]
        sizes_view = recv_view if ws == 1 else words[128:128 + ws + 1]
        sorted_ids, perm, sizes, offsets = ops._bucket(cur, cur_n, sizes_view, words[64:64 + ws])
        recv, recv_counts = ops._exchange().exchange_ids_enqueue(sorted_ids, sizes, offsets, recv_view)
        total = recv_counts[ws:ws + 1]
        lo, hi = ops._owned_range()
        u_slot, in_slot = slot, slot + 1
        uniq2, inv = ops._unique_enqueue(recv, total, lo, hi, st.word(u_slot), "unique_np")
        # The block of the outermost hop lists its destination nodes (the frontier uniq2, sorted and
        # distinct) first, so input row j is the row of uniq2[j] for j below the frontier's size: those
        # rows are fetched on a second stream while the hop is still being sampled and relabelled,
        # and only the rows of the newly met nodes wait for the relabelling.
        f = st.feat
        prefetch = self.prefetch_features and f.feat_pos_map is not None and \
            uniq2.numel() * (1 + self.las_fanouts) * f.rank_feat_dim * f.dev_feats.element_size() <= _PREFETCH_LIMIT_BYTES
        split = self.gather_split if prefetch and not st.profiling else 0
        rows = None
        side = None
        if prefetch:
            rows = torch.empty((uniq2.numel() * (1 + self.las_fanouts), f.rank_feat_dim), dtype=f.dev_feats.dtype,
                               device=uniq2.device)
        if split:
            main = torch.cuda.current_stream()
            side = st.side_stream()
            side.wait_stream(main)
            with torch.cuda.stream(side):
                ops._gather_enqueue(uniq2, st.word(u_slot), out=rows, ws_name="gather_frontier")
        uniq3, rel3, _ = ops._sample_relabel_enqueue(uniq2, self.las_fanouts, st.word(u_slot), st.word(in_slot),
                                                     call if explicit else None, call_base_dev)
        if split == 1:
            main.wait_stream(side)
        if prefetch:
            ops._gather_enqueue(uniq3, st.word(in_slot), out=rows, first_dev=st.word(u_slot) if split else None)
        if split == 2:
            main.wait_stream(side)
        return dict(layers=layers, perm=perm, inv=inv, uniq2=uniq2, uniq3=uniq3, rel3=rel3, rows=rows,
                    u_slot=u_slot, in_slot=in_slot)

    def _finish(self, seeds, bufs, host=None):
        """The one host read of the mini-batch (or the copy of the word block a pipelined launch
        left in `host`), then buffers narrowed to their real sizes."""
        st = ops.STATE
        ws = st.world_size
        if host is None:
            host = st.read_words()
        u_slot, in_slot = bufs["u_slot"], bufs["in_slot"]
        # one tolist() of the word block: python ints from here on (every slice, clone or int() of the
        # pinned block costs microseconds of host time per mini-batch)
        h = host.tolist()
        count = h[:in_slot + 1]
        recv_cum = list(itertools.accumulate(h[16:16 + ws]))
        recv_offset = torch.tensor(recv_cum, dtype=torch.int64)
        dev_offset = torch.tensor(h[64:64 + ws], dtype=torch.int64)
        total_recv = recv_cum[-1]
        if total_recv > bufs["inv"].numel():
            raise RuntimeError("chained NP sampler: more ids received than the buffer sized from this rank's own "
                               "batch holds; use chained=False for batches that differ this much between the ranks")
        blocks = []
        n_dst = seeds.numel()
        for dst_buf, rel, uniq, u_s, fanout in bufs["layers"]:
            n_src = count[u_s]
            blocks.insert(0, Block(rel[:n_dst * fanout], _coo_col(dst_buf.numel(), n_dst, fanout, rel.device),
                                   n_src, n_dst, uniq[:n_src], fanout))
            n_dst = n_src
        n_frontier = n_dst
        n_owner_dst, n_in = count[u_slot], count[in_slot]
        f0 = self.las_fanouts
        uniq2, uniq3, rel3 = bufs["uniq2"], bufs["uniq3"], bufs["rel3"]
        blocks.insert(0, Block(rel3[:n_owner_dst * f0], _coo_col(uniq2.numel(), n_owner_dst, f0, rel3.device),
                               n_in, n_owner_dst, uniq3[:n_in], f0))
        input_nodes = uniq3[:n_in]
        if bufs["rows"] is not None:
            st.prefetched = (input_nodes, bufs["rows"][:n_in])
        return (input_nodes, seeds, blocks, bufs["perm"][:n_frontier], recv_offset, dev_offset,
                bufs["inv"][:total_recv])


class SPGATSampler(_GraphReplay):
    """SNP strategy with a GAT model (MixedPSNeighborSampler with system "SP",
    model "GAT", shuffle_with_dst False, python/npc/sampler.py:187-238 and
    :358-364): inner hops as in GDP; in the outermost hop the block keeps the
    local dst nodes, its sources are the sorted unique neighbours, and those
    ids travel to their owners, which load and project their features; the
    feature shuffle brings the projected rows back in unique-neighbour order.
    Returns (input_nodes, output_nodes, blocks, perm, send_offset, recv_offset)
    with input_nodes = cat(dst nodes, ids received from the other ranks).

    chained / use_graph as in MixedNeighborSampler: the whole mini-batch enqueued with device-side
    sizes and replayed from a CUDA graph, one host read at the end; prefetch_features also
    enqueues the gather of the input nodes' rows before that read."""

    # word slots of the chained form: [0..13] hop counts, [16..48] ids received per peer (+ total),
    # [64..95] bucket offsets, [50] neighbours drawn, [51] unique neighbours, [52] input nodes,
    # [128..160] bucket sizes
    _N, _U, _IN = 50, 51, 52

    def __init__(self, rank: int, fanouts: List[int], chained: bool = None, use_graph: bool = None,
                 prefetch_features: bool = True, lanes: int = None):
        self.rank = rank
        self.fanouts = list(fanouts)
        if chained is None:
            chained = os.environ.get("APT_CHAINED_SAMPLER", "1") != "0"
        self.chained = bool(chained)
        self.prefetch_features = prefetch_features
        self._init_replay(use_graph, 2, lanes)
        self.use_graph = self.use_graph and self.chained
        self.num_calls = len(self.fanouts)

    def _enqueue(self, seeds: torch.Tensor, call_base_dev):
        """Every kernel of the mini-batch on the current stream, no host read."""
        st = ops.STATE
        ws = st.world_size
        if ws > 31 or len(self.fanouts) > 14:
            raise RuntimeError("the chained SNP-GAT sampler serves at most 31 ranks and 14 hops")
        words = st.words()
        explicit = call_base_dev is not None
        slot = 0
        call = 0
        cur, cur_n = seeds, None
        layers = []
        for fanout in list(reversed(self.fanouts))[:-1]:
            cnt = st.word(slot)
            uniq, rel, _ = ops._sample_relabel_enqueue(cur, fanout, cur_n, cnt, call if explicit else None,
                                                       call_base_dev)
            call += 1
            layers.append((cur, rel, uniq, slot, fanout))
            cur, cur_n = uniq, cnt
            slot += 1
        f = self.fanouts[0]
        nbr = ops._sample(cur, f, cur_n, call if explicit else None, call_base_dev)
        n_word = None
        if cur_n is not None:
            n_word = st.word(self._N)
            torch.mul(cur_n, f, out=n_word)
        # sorted unique of the neighbours + the position of every neighbour in it (torch.unique with
        # return_inverse, python/npc/sampler.py:224-226)
        u_word = st.word(self._U)
        unique_neigh, arange_src = ops._unique_enqueue(nbr, n_word, 0, int(st.graph.num_total_nodes), u_word,
                                                       "unique_gat")
        recv_view = words[16:16 + ws + 1]
        sizes_view = recv_view if ws == 1 else words[128:128 + ws + 1]
        sorted_ids, perm, sizes, offsets = ops._bucket(unique_neigh, u_word, sizes_view, words[64:64 + ws])
        recv, recv_counts = ops._exchange().exchange_ids_enqueue(sorted_ids, sizes, offsets, recv_view)
        in_word = st.word(self._IN)
        input_nodes = ops.concat_ids(cur, cur_n, recv, recv_counts[ws:ws + 1], in_word)
        rows = None
        ft = st.feat
        if self.prefetch_features and ft.feat_pos_map is not None and \
                input_nodes.numel() * ft.rank_feat_dim * ft.dev_feats.element_size() <= _PREFETCH_LIMIT_BYTES:
            rows = ops._gather_enqueue(input_nodes, in_word)
        return dict(layers=layers, slot=slot, cur=cur, arange_src=arange_src, unique_neigh=unique_neigh, perm=perm,
                    input_nodes=input_nodes, rows=rows)

    def _finish(self, seeds, b, host=None):
        st = ops.STATE
        ws = st.world_size
        if host is None:
            host = st.read_words()
        dev = seeds.device
        f = self.fanouts[0]
        blocks = []
        n_dst = seeds.numel()
        for dst_buf, rel, uniq, u_s, fanout in b["layers"]:
            n_src = int(host[u_s])
            blocks.insert(0, Block(rel[:n_dst * fanout], _coo_col(dst_buf.numel(), n_dst, fanout, dev), n_src, n_dst,
                                   uniq[:n_src], fanout))
            n_dst = n_src
        n_u, n_in = int(host[self._U]), int(host[self._IN])
        if n_in > b["input_nodes"].numel():
            raise RuntimeError("chained SNP-GAT sampler: more ids received than the buffer sized from this rank's own "
                               "batch holds; use chained=False for batches that differ this much between the ranks")
        blocks.insert(0, Block(b["arange_src"][:n_dst * f], _coo_col(b["cur"].numel(), n_dst, f, dev), n_u, n_dst,
                               b["unique_neigh"][:n_u], f))
        h = host.tolist()
        send_offset = torch.tensor(list(itertools.accumulate(h[16:16 + ws])), dtype=torch.int64)
        recv_offset = torch.tensor(h[64:64 + ws], dtype=torch.int64)
        input_nodes = b["input_nodes"][:n_in]
        if b["rows"] is not None:
            st.prefetched = (input_nodes, b["rows"][:n_in])
        return input_nodes, seeds, blocks, b["perm"][:n_u], send_offset, recv_offset

    def sample(self, graph, seeds: torch.Tensor):
        if self.chained and ops._exchange().name in ("local", "p2p"):
            return self._sample_chained(seeds)
        output_nodes = seeds
        blocks = []
        n_total = ops.STATE.graph.num_total_nodes
        for layer_id, fanout in enumerate(reversed(self.fanouts)):
            seeds, neighbors = ops.local_sample_one_layer(seeds, fanout)
            if layer_id != len(self.fanouts) - 1:
                block = create_block(seeds, neighbors, fanout)
                seeds = block.src_ids
                blocks.insert(0, block)
                continue
            num_dst = seeds.numel()
            unique_neigh, arange_src = ops.unique_sorted(neighbors, 0, n_total)
            arange_dst = torch.arange(num_dst, device=seeds.device).repeat_interleave(fanout)
            blocks.insert(0, Block(arange_src, arange_dst, unique_neigh.numel(), num_dst, unique_neigh, fanout))
            shuffled_neigh, perm, send_offset, recv_offset = ops.sp_sample_shuffle_src(unique_neigh)
            seeds = torch.cat((seeds, shuffled_neigh))
        return seeds, output_nodes, blocks, perm, send_offset, recv_offset


class SPVirtualSampler(_GraphReplay):
    """SNP strategy with a SAGE or GCN model (MixedPSNeighborSampler with system
    "SP", python/npc/sampler.py:240-330). Inner hops as in GDP. In the outermost
    hop each sampled neighbour becomes a virtual node (owner, local destination):
    block1 joins the sorted unique virtual nodes to the local destinations, the
    packed triples (sender, destination index, neighbour id) travel to the
    neighbour's owner, and block2 there joins the received neighbours to the
    received virtual nodes, so that the owner sums its rows per virtual node
    before anything crosses a link (sp_feat_shuffle carries the partial sums).

    The reference sorts the virtual ids with torch.sort, which leaves equal keys
    in any order; here the order is the stable one, given by the owner bucketing
    (virtual ids rise with the position inside one owner's bucket).

    Returns (input_nodes, output_nodes, blocks, send_sizes, recv_sizes); blocks =
    [block2, block1, inner blocks...]. block2.src_ids are the unique received
    neighbours, its destinations the sorted unique received virtual nodes
    (`self.last["unique_dst"]`)."""

    def __init__(self, rank: int, fanouts: List[int], model: str = "SAGE", shuffle_with_dst: bool = False,
                 chained: bool = None, use_graph: bool = None, lanes: int = None):
        if model not in ("SAGE", "GCN"):
            raise ValueError("SPVirtualSampler serves SAGE and GCN; GAT uses SPGATSampler")
        self.rank = rank
        self.fanouts = list(fanouts)
        self.model = model
        self.shuffle_with_dst = bool(shuffle_with_dst)
        if chained is None:
            chained = os.environ.get("APT_CHAINED_SAMPLER", "1") != "0"
        self.chained = bool(chained)
        self._init_replay(use_graph, 2, lanes)
        self.use_graph = self.use_graph and self.chained
        self.num_calls = len(self.fanouts)
        self.last = {}

    # word slots of the chained form: [0..13] hop counts, [16..48] packed ids received per peer (+ total),
    # [50] neighbours, [51] unique virtual nodes, [52] unique received neighbours, [53] unique received
    # virtual nodes, [54] destinations + neighbours, [64..96] destinations received per peer (+ total),
    # [128..191] send sizes, [192..253] receive sizes
    _N, _UF, _US, _UD, _ALL, _RDST, _SEND, _RECV = 50, 51, 52, 53, 54, 64, 128, 192

    def _enqueue(self, seeds: torch.Tensor, call_base_dev):
        """Every kernel of the mini-batch on the current stream, no host read."""
        st = ops.STATE
        ws = st.world_size
        with_dst = self.shuffle_with_dst
        k = 3 if with_dst else 2
        if k * ws > 62 or len(self.fanouts) > 14:
            raise RuntimeError("the chained SNP sampler serves at most 31 ranks (20 with destinations) and 14 hops")
        dev = seeds.device
        words = st.words()
        explicit = call_base_dev is not None
        slot = 0
        call = 0
        cur, cur_n = seeds, None
        layers = []
        for fanout in list(reversed(self.fanouts))[:-1]:
            cnt = st.word(slot)
            uniq, rel, _ = ops._sample_relabel_enqueue(cur, fanout, cur_n, cnt, call if explicit else None,
                                                       call_base_dev)
            call += 1
            layers.append((cur, rel, uniq, slot, fanout))
            cur, cur_n = uniq, cnt
            slot += 1
        f = self.fanouts[0]
        s_max = cur.numel()
        n_max = s_max * f
        nbr = ops._sample(cur, f, cur_n, call if explicit else None, call_base_dev)
        n_word = None
        if cur_n is not None:
            n_word = st.word(self._N)
            torch.mul(cur_n, f, out=n_word)
        _, pos, _, _ = ops._bucket(nbr, n_word)
        sorted_vir = torch.empty(n_max, dtype=torch.int64, device=dev)
        packed = torch.empty(n_max, dtype=torch.int64, device=dev)
        owner = ops._owner_args()
        n_total = int(st.graph.num_total_nodes)
        check(lib.apt_sp_map_place_pack(ops._ptr(nbr), ops._ptr(pos), s_max, ops._ptr(cur_n), f, *owner, ops.SP_BASE,
                                        n_total, ops._ptr(sorted_vir), ops._ptr(packed), None, ops._stream()))
        uf_word = st.word(self._UF)
        # the unique virtual nodes come from the ids as they stand (owner x num_dst + destination); with
        # destinations every neighbour's id is shifted by world_size x num_dst afterwards, which keeps the order
        unique_frontier, _ = ops._unique_enqueue(sorted_vir, n_word, 0, ws * max(s_max, 1), uf_word, "unique_vir")
        dst_sorted = None
        if with_dst:
            dst_sorted, dst_pos, _, _ = ops._bucket(cur, cur_n)
            dst_vir = torch.empty(s_max, dtype=torch.int64, device=dev)
            scratch = torch.empty(s_max, dtype=torch.int64, device=dev)
            # a destination is a neighbour list of length one: owner(destination) x num_dst + its index,
            # placed by the bucket's positions (MapSrcDsttoVir, src/cuda/npc_kernel.cu:15-70)
            check(lib.apt_sp_map_place_pack(ops._ptr(cur), ops._ptr(dst_pos), s_max, ops._ptr(cur_n), 1, *owner,
                                            ops.SP_BASE, n_total, ops._ptr(dst_vir), ops._ptr(scratch), None,
                                            ops._stream()))
            shift = cur_n * ws if cur_n is not None else ws * s_max
            sorted_src = sorted_vir + shift
            unique_frontier = unique_frontier + shift
            sorted_all = ops.concat_ids(dst_vir, cur_n, sorted_src, n_word, st.word(self._ALL))
            all_word = st.word(self._ALL)
        else:
            sorted_all, all_word = sorted_vir, n_word
        send_sizes = words[self._SEND:self._SEND + k * ws]
        recv_sizes = words[self._RECV:self._RECV + k * ws]
        check(lib.apt_vir_send_sizes(ops._ptr(sorted_all), sorted_all.numel(), ops._ptr(all_word),
                                     ops._ptr(unique_frontier), unique_frontier.numel(), ops._ptr(uf_word), ws, s_max,
                                     ops._ptr(cur_n), int(with_dst), None, ops._ptr(send_sizes), ops._stream()))
        ex = ops._exchange()
        ex.exchange_fixed(send_sizes.view(ws, k), recv_sizes.view(ws, k))
        counts = words[16:16 + ws + 1]
        dst_counts = words[self._RDST:self._RDST + ws + 1]
        recv_dst = None
        ids_at = 1 if with_dst else 0
        if ws == 1:
            recv = packed
            counts[0:1].copy_(send_sizes[ids_at:ids_at + 1])
            counts[1:2].copy_(send_sizes[ids_at:ids_at + 1])
            if with_dst:
                recv_dst = dst_sorted
                dst_counts[0:1].copy_(send_sizes[0:1])
                dst_counts[1:2].copy_(send_sizes[0:1])
        else:
            if with_dst:
                recv_dst, _ = ex.exchange_ids_enqueue(dst_sorted, None, torch.cumsum(send_sizes[0::k], 0), dst_counts)
            recv, _ = ex.exchange_ids_enqueue(packed, None, torch.cumsum(send_sizes[ids_at::k], 0), counts)
        total = counts[ws:ws + 1]
        vir_src = torch.empty(recv.numel(), dtype=torch.int64, device=dev)
        ori_src = torch.empty(recv.numel(), dtype=torch.int64, device=dev)
        check(lib.apt_sp_unpack_frontier(ops._ptr(recv), recv.numel(), ops._ptr(total), n_total,
                                         ops._ptr(vir_src), ops._ptr(ori_src), ops._stream()))
        lo, hi = ops._owned_range()
        unique_src, a_src = ops._unique_enqueue(ori_src, total, lo, hi, st.word(self._US), "unique_sp_src")
        unique_dst, a_dst = ops._unique_enqueue(vir_src, total, 0, ws * ops.SP_BASE, st.word(self._UD), "unique_vdst")
        div = cur_n if cur_n is not None else max(s_max, 1)
        arange_dst = torch.remainder(unique_frontier, div)
        return dict(layers=layers, slot=slot, cur=cur, nbr=nbr, sorted_all=sorted_all, packed=packed,
                    unique_frontier=unique_frontier, arange_dst=arange_dst, vir_src=vir_src, ori_src=ori_src,
                    unique_src=unique_src, a_src=a_src, unique_dst=unique_dst, a_dst=a_dst, dst_sorted=dst_sorted,
                    recv_dst=recv_dst)

    def _finish(self, seeds, b, host=None):
        """The one host read of the mini-batch, then everything is narrowed to its real size."""
        st = ops.STATE
        ws = st.world_size
        dev = seeds.device
        f = self.fanouts[0]
        if host is None:
            host = st.read_words()
        count = [int(host[k]) for k in range(b["slot"])]
        blocks = []
        n_dst = seeds.numel()
        for dst_buf, rel, uniq, u_s, fanout in b["layers"]:
            n_src = count[u_s]
            blocks.insert(0, Block(rel[:n_dst * fanout], _coo_col(dst_buf.numel(), n_dst, fanout, dev), n_src, n_dst,
                                   uniq[:n_src], fanout))
            n_dst = n_src
        num_dst = n_dst
        n_uf, n_us, n_ud = int(host[self._UF]), int(host[self._US]), int(host[self._UD])
        n_recv = int(host[16 + ws])
        with_dst = self.shuffle_with_dst
        k = 3 if with_dst else 2
        n_rdst = int(host[self._RDST + ws]) if with_dst else 0
        if n_recv > b["vir_src"].numel() or (with_dst and n_rdst > b["recv_dst"].numel()):
            raise RuntimeError("chained SNP sampler: more ids received than the buffer sized from this rank's own "
                               "batch holds; use chained=False for batches that differ this much between the ranks")
        h = host.tolist()
        send_sizes_cpu = torch.tensor(h[self._SEND:self._SEND + k * ws], dtype=torch.int64)
        recv_sizes_cpu = torch.tensor(h[self._RECV:self._RECV + k * ws], dtype=torch.int64)
        unique_frontier, unique_src = b["unique_frontier"], b["unique_src"]
        block1 = Block(torch.arange(n_uf, device=dev), b["arange_dst"][:n_uf], n_uf, num_dst, unique_frontier[:n_uf], f)
        block2 = Block(b["a_src"][:n_recv], b["a_dst"][:n_recv], n_us, n_ud, unique_src[:n_us], f)
        blocks.insert(0, block1)
        blocks.insert(0, block2)
        dst_nodes = b["cur"][:num_dst]
        n_all = num_dst * f + (num_dst if with_dst else 0)
        send_frontier = b["packed"][:num_dst * f]
        recv_dst = None
        if with_dst:
            send_frontier = torch.cat((b["dst_sorted"][:num_dst], send_frontier))
            recv_dst = b["recv_dst"][:n_rdst]
        self.last = dict(neighbors=b["nbr"][:num_dst * f], sorted_allnodes=b["sorted_all"][:n_all],
                         unique_frontier=unique_frontier[:n_uf], send_frontier=send_frontier, recv_dst=recv_dst,
                         vir_src=b["vir_src"][:n_recv], ori_src=b["ori_src"][:n_recv],
                         unique_dst=b["unique_dst"][:n_ud])
        if with_dst:
            nxt = torch.cat((recv_dst, unique_src[:n_us]))
        elif self.model == "GCN":
            nxt = unique_src[:n_us]
        else:
            nxt = torch.cat((dst_nodes, unique_src[:n_us]))
        return nxt, seeds, blocks, send_sizes_cpu, recv_sizes_cpu

    def _outer(self, seeds, neighbors, fanout):
        st = ops.STATE
        ws = st.world_size
        num_dst = seeds.numel()
        dev = seeds.device
        n_total = st.graph.num_total_nodes
        nbr_sorted, nbr_pos, _, _ = ops._bucket(neighbors)        # neighbours grouped by owner, input order kept
        if self.shuffle_with_dst:
            map_all = ops.srcdst_to_vir(fanout, seeds, neighbors)
            dst_sorted, dst_pos, _, _ = ops._bucket(seeds)
            pos = torch.cat((dst_pos, nbr_pos + num_dst))
            sorted_all = ops.rows_scatter(map_all.view(-1, 1), pos, pos.numel()).view(-1)
            map_src = sorted_all[num_dst:]
            lo = ws * num_dst
        else:
            map_all = ops.src_to_vir(fanout, num_dst, neighbors)
            sorted_all = ops.rows_scatter(map_all.view(-1, 1), nbr_pos, nbr_pos.numel()).view(-1)
            map_src = sorted_all
            lo = 0
        unique_frontier, _ = ops.unique_sorted(map_src, lo, lo + ws * max(num_dst, 1))
        arange_dst = unique_frontier % max(num_dst, 1)
        arange_src = torch.arange(unique_frontier.numel(), device=dev)
        block1 = Block(arange_src, arange_dst, unique_frontier.numel(), num_dst, unique_frontier, fanout)
        packed = ops.sp_pack_frontier(map_src, nbr_sorted, num_dst)
        if self.shuffle_with_dst:
            send_frontier = torch.cat((dst_sorted, packed))
            recv_dst, recv_seeds, recv_neighbors, send_sizes, recv_sizes = ops.sp_sample_and_shuffle(
                num_dst, send_frontier, sorted_all, unique_frontier, 1)
        else:
            recv_dst = None
            recv_seeds, recv_neighbors, send_sizes, recv_sizes = ops.sp_sample_and_shuffle(
                num_dst, packed, sorted_all, unique_frontier, 0)
        own_lo, own_hi = ops._owned_range()
        unique_src, a_src = ops.unique_sorted(recv_neighbors, own_lo, own_hi)
        unique_dst, a_dst = ops.unique_sorted(recv_seeds, 0, ws * ops.SP_BASE)
        block2 = Block(a_src, a_dst, unique_src.numel(), unique_dst.numel(), unique_src, fanout)
        self.last = dict(neighbors=neighbors, sorted_allnodes=sorted_all, unique_frontier=unique_frontier,
                         send_frontier=send_frontier if self.shuffle_with_dst else packed, recv_dst=recv_dst,
                         vir_src=recv_seeds, ori_src=recv_neighbors, unique_dst=unique_dst)
        if self.shuffle_with_dst:
            nxt = torch.cat((recv_dst, unique_src))
        elif self.model == "GCN":
            nxt = unique_src
        else:
            nxt = torch.cat((seeds, unique_src))
        return nxt, block1, block2, send_sizes, recv_sizes

    def sample(self, graph, seeds: torch.Tensor):
        if self.chained and ops._exchange().name in ("local", "p2p"):
            return self._sample_chained(seeds)
        output_nodes = seeds
        blocks = []
        for layer_id, fanout in enumerate(reversed(self.fanouts)):
            seeds, neighbors = ops.local_sample_one_layer(seeds, fanout)
            if layer_id != len(self.fanouts) - 1:
                block = create_block(seeds, neighbors, fanout)
                seeds = block.src_ids
                blocks.insert(0, block)
                continue
            seeds, block1, block2, send_sizes, recv_sizes = self._outer(seeds, neighbors, fanout)
            blocks.insert(0, block1)
            blocks.insert(0, block2)
        return seeds, output_nodes, blocks, send_sizes, recv_sizes


class MPSampler(_GraphReplay):
    """NFP strategy with a SAGE or GCN model (MixedPSNeighborSampler with system
    "MP", python/npc/sampler.py:332-356): every rank holds a slice of the feature
    columns of all nodes. Inner hops as in GDP; in the outermost hop every rank
    relabels its own block and then receives every rank's frontier and relabelled
    rows, so that it can aggregate its column slice for all ranks' destinations
    (multi-segment spmm_copy_u_sum) before mp_feat_shuffle_fwd sums the slices.

    Returns (input_nodes, output_nodes, blocks, send_size, recv_size); blocks[0] =
    (all_coo_row, all_coo_col, recv_frontier_size, recv_coo_size, recv_size) as in
    the reference, input_nodes = the concatenation of all ranks' frontiers."""

    def __init__(self, rank: int, fanouts: List[int], chained: bool = None, use_graph: bool = None,
                 lanes: int = None):
        self.rank = rank
        self.fanouts = list(fanouts)
        if chained is None:
            chained = os.environ.get("APT_CHAINED_SAMPLER", "1") != "0"
        self.chained = bool(chained)
        self._init_replay(use_graph, 2, lanes)
        self.use_graph = self.use_graph and self.chained
        self.num_calls = len(self.fanouts)

    # word slots of the chained form: [0..13] hop counts (the last one is the frontier of the outermost
    # hop), [54..56] this rank's (seeds, frontier, rows) sizes, [16..48] / [64..96] rows received per peer
    # for the two broadcasts, [128..223] every rank's three sizes
    _MINE, _ALL = 54, 128

    def _enqueue(self, seeds: torch.Tensor, call_base_dev):
        """Every kernel of the mini-batch on the current stream without a host read: sizes stay in the
        device word block, buffers are upper bounds, the broadcasts take device-side counts."""
        st = ops.STATE
        ws = st.world_size
        if ws > 31 or len(self.fanouts) > 13:
            raise RuntimeError("the chained NFP sampler serves at most 31 ranks and 13 hops")
        dev = seeds.device
        words = st.words()
        explicit = call_base_dev is not None
        slot = 0
        call = 0
        cur, cur_n = seeds, None
        layers = []
        for fanout in list(reversed(self.fanouts))[:-1]:
            cnt = st.word(slot)
            uniq, rel, _ = ops._sample_relabel_enqueue(cur, fanout, cur_n, cnt, call if explicit else None,
                                                       call_base_dev)
            call += 1
            layers.append((cur, rel, uniq, slot, fanout))
            cur, cur_n = uniq, cnt
            slot += 1
        f = self.fanouts[0]
        uf_word = st.word(slot)
        unique_frontier, coo_row, _ = ops._sample_relabel_enqueue(cur, f, cur_n, uf_word, call if explicit else None,
                                                                  call_base_dev)
        mine = words[self._MINE:self._MINE + 3]
        if cur_n is None:
            mine[0:1].fill_(cur.numel())
        else:
            mine[0:1].copy_(cur_n)
        mine[1:2].copy_(uf_word)
        torch.mul(mine[0:1], f, out=mine[2:3])
        ex = ops._exchange()
        all_sizes = words[self._ALL:self._ALL + 3 * ws].view(ws, 3)
        if ws == 1:
            all_sizes.copy_(mine.view(1, 3))
        else:
            got, _ = ex.allbroadcast_enqueue(mine.view(1, 3), words[self._MINE + 3:self._MINE + 4].fill_(1),
                                             torch.empty(ws + 1, dtype=torch.int64, device=dev))
            all_sizes.copy_(got[:ws])
        recv_frontier, _ = ex.allbroadcast_enqueue(unique_frontier.view(-1, 1), mine[1:2], words[16:16 + ws + 1])
        recv_coo, _ = ex.allbroadcast_enqueue(coo_row.view(-1, 1), mine[2:3], words[64:64 + ws + 1])
        return dict(layers=layers, slot=slot, recv_frontier=recv_frontier, recv_coo=recv_coo)

    def _finish(self, seeds, b, host=None):
        """The one host read of the mini-batch, then everything is narrowed to its real size."""
        st = ops.STATE
        ws = st.world_size
        dev = seeds.device
        f = self.fanouts[0]
        if host is None:
            host = st.read_words()
        count = [int(host[k]) for k in range(b["slot"])]
        blocks = []
        n_dst = seeds.numel()
        for dst_buf, rel, uniq, u_s, fanout in b["layers"]:
            n_src = count[u_s]
            blocks.insert(0, Block(rel[:n_dst * fanout], _coo_col(dst_buf.numel(), n_dst, fanout, dev), n_src, n_dst,
                                   uniq[:n_src], fanout))
            n_dst = n_src
        sizes = host[self._ALL:self._ALL + 3 * ws].view(ws, 3)
        sizes = torch.tensor(sizes.tolist(), dtype=torch.int64)        # off the pinned block
        recv_size = sizes[:, 0].contiguous()
        recv_frontier_size = sizes[:, 1].contiguous()
        recv_coo_size = sizes[:, 2].contiguous()
        recv_frontier, recv_coo = b["recv_frontier"], b["recv_coo"]
        if int(recv_frontier_size.sum()) > recv_frontier.shape[0] or int(recv_coo_size.sum()) > recv_coo.shape[0]:
            raise RuntimeError("chained NFP sampler: the ranks sent more rows than the buffers sized from this rank's "
                               "own batch hold; it needs the same number of seeds on every rank (or chained=False)")
        all_frontier = recv_frontier.view(-1)[:int(recv_frontier_size.sum())]
        all_coo_row = recv_coo.view(-1)[:int(recv_coo_size.sum())]
        all_coo_col = torch.cat([_coo_col(int(i), int(i), f, dev) for i in recv_size])
        blocks.insert(0, (all_coo_row, all_coo_col, recv_frontier_size, recv_coo_size, recv_size))
        return all_frontier, seeds, blocks, torch.tensor([n_dst]), recv_size

    def sample(self, graph, seeds: torch.Tensor):
        if self.chained and ops._exchange().name in ("local", "p2p"):
            return self._sample_chained(seeds)
        output_nodes = seeds
        blocks = []
        for layer_id, fanout in enumerate(reversed(self.fanouts)):
            seeds, neighbors = ops.local_sample_one_layer(seeds, fanout)
            if layer_id != len(self.fanouts) - 1:
                block = create_block(seeds, neighbors, fanout)
                seeds = block.src_ids
                blocks.insert(0, block)
                continue
            unique_frontier, coo_row = ops.relabel_csc(seeds, neighbors)
            all_frontier, all_coo_row, send_size, recv_size, recv_frontier_size, recv_coo_size = \
                ops.mp_sample_shuffle(seeds, unique_frontier, coo_row)
            all_coo_col = torch.cat([_coo_col(int(i), int(i), fanout, all_coo_row.device) for i in recv_size])
            blocks.insert(0, (all_coo_row, all_coo_col, recv_frontier_size, recv_coo_size, recv_size))
            seeds = all_frontier
        return seeds, output_nodes, blocks, send_size, recv_size


class DPNeighborSampler:
    """GDP strategy: every hop local (python/npc/sampler.py:202-203 with the
    common block construction)."""

    def __init__(self, rank: int, fanouts: List[int]):
        self.rank = rank
        self.fanouts = list(fanouts)

    def sample(self, graph, seeds: torch.Tensor):
        output_nodes = seeds
        blocks = []
        for fanout in reversed(self.fanouts):
            seeds, neighbors = ops.local_sample_one_layer(seeds, fanout)
            block = create_block(seeds, neighbors, fanout)
            seeds = block.src_ids
            blocks.insert(0, block)
        return seeds, output_nodes, blocks
