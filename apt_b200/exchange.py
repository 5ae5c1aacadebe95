"""The exchange step between ranks (seed ids one way, feature rows the other)
behind ShuffleSeeds (src/sampling.cc:176-191), FeatShuffle
(src/feat_shuffle.cc:9-30) and AlltoAll (src/ops/collective.cc:223-266).

Three interchangeable backends with identical results:

``LocalExchange``   world_size == 1: nothing crosses a link; rows are permuted
                    by the local row-mover kernels.
``P2PExchange``     the product path: each rank stores its rows straight into
                    the receiving GPU's inbox over NVLink (apt_p2p_* in the
                    C ABI), one flag per (sender, receiver) pair, no host
                    round trip for sizes.
``NcclExchange``    torch.distributed all_to_all_single, the counterpart of the
                    reference's grouped ncclSend/ncclRecv; kept as the measured
                    baseline (APT_SHUFFLE_BACKEND=nccl).
"""
import ctypes
import os

import torch
import torch.distributed as dist

from . import _lib
from ._lib import check, lib


def _ptr(t):
    return None if t is None or t.numel() == 0 else ctypes.c_void_p(t.data_ptr())


def _stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _counts(offsets_cpu: torch.Tensor):
    """Inclusive cumulative offsets -> per-rank counts (python ints)."""
    o = [int(x) for x in offsets_cpu.tolist()]
    return [o[0]] + [o[i] - o[i - 1] for i in range(1, len(o))]


class LocalExchange:
    name = "local"

    def __init__(self, state):
        self.state = state

    def exchange_ids(self, sorted_ids, sizes, offsets):
        off = offsets.cpu()
        return sorted_ids, off, off.clone()

    def exchange_ids_enqueue(self, sorted_ids, sizes, offsets, counts_out=None):
        """Stream-ordered variant without a host read: (recv buffer, device counts
        int64[world_size + 1] with the total last). With one rank what is
        received is what was bucketed, so the bucket sizes are the counts."""
        if counts_out is not None and counts_out.data_ptr() != sizes.data_ptr():
            counts_out.copy_(sizes)
            return sorted_ids, counts_out
        return sorted_ids, sizes

    def exchange_rows(self, inputs, send_offset, recv_offset, permutation, fwd):
        from . import ops

        if fwd:
            return ops.rows_gather(inputs, permutation)
        return ops.rows_scatter(inputs, permutation, int(recv_offset[-1]))

    def alltoall(self, inp, out, send_offset, recv_offset, expand):
        n = int(send_offset[-1]) * expand
        out.view(-1)[:n].copy_(inp.view(-1)[:n])

    def allbroadcast(self, inp, recv_counts):
        return inp.clone()

    def reduce_scatter(self, inp, seg_sizes, my_rows):
        return inp.clone()

    def exchange_fixed(self, send, recv):
        """All-to-all of one row of send[world_size, k] per peer into recv, stream-ordered."""
        recv.copy_(send)

    def allbroadcast_enqueue(self, inp, n_dev, counts_out):
        """Stream-ordered all-broadcast of the first n_dev rows of inp (device count): (buffer of
        world_size x inp.shape[0] rows holding the received rows in rank order, counts)."""
        counts_out[0:1].copy_(n_dev)
        counts_out[1:2].copy_(n_dev)
        return inp, counts_out


class NcclExchange:
    """Baseline: the collective library's all-to-all-v."""

    name = "nccl"

    def __init__(self, state, group=None):
        self.state = state
        self.group = group

    def _a2a(self, inp, send_counts, recv_counts, width):
        out = inp.new_empty((sum(recv_counts), width))
        dist.all_to_all_single(out, inp.reshape(-1, width), output_split_sizes=recv_counts,
                               input_split_sizes=send_counts, group=self.group)
        return out

    def exchange_ids(self, sorted_ids, sizes, offsets):
        sizes = sizes[:self.state.world_size].contiguous()
        recv_sizes = torch.empty_like(sizes)
        dist.all_to_all_single(recv_sizes, sizes, group=self.group)
        send_counts = [int(x) for x in sizes.tolist()]
        recv_counts = [int(x) for x in recv_sizes.tolist()]
        recv = self._a2a(sorted_ids.view(-1, 1), send_counts, recv_counts, 1).view(-1)
        return recv, torch.tensor(recv_counts).cumsum(0), offsets.cpu()

    def exchange_ids_enqueue(self, sorted_ids, sizes, offsets, counts_out=None):
        # the library all-to-all needs the sizes on the host: this baseline synchronises
        recv, recv_offset, _ = self.exchange_ids(sorted_ids, sizes, offsets)
        counts = torch.cat([torch.tensor(_counts(recv_offset)), recv_offset[-1:]]).to(sorted_ids.device)
        if counts_out is not None:
            counts_out.copy_(counts)
            counts = counts_out
        return recv, counts

    def exchange_rows(self, inputs, send_offset, recv_offset, permutation, fwd):
        from . import ops

        send_counts, recv_counts = _counts(send_offset), _counts(recv_offset)
        if fwd:
            buf = self._a2a(inputs, send_counts, recv_counts, inputs.shape[1])
            return ops.rows_gather(buf, permutation)
        tmp = ops.rows_scatter(inputs, permutation, inputs.shape[0])
        return self._a2a(tmp, send_counts, recv_counts, inputs.shape[1])

    def alltoall(self, inp, out, send_offset, recv_offset, expand):
        send_counts, recv_counts = _counts(send_offset), _counts(recv_offset)
        res = self._a2a(inp.view(-1, expand)[: sum(send_counts)], send_counts, recv_counts, expand)
        out.view(-1)[: res.numel()].copy_(res.view(-1))

    def allbroadcast(self, inp, recv_counts):
        """Every rank's rows to every rank, in rank order (all-gather of blocks of
        different lengths)."""
        ws = self.state.world_size
        n = inp.shape[0]
        return self._a2a(inp.repeat(ws, 1), [n] * ws, [int(c) for c in recv_counts], inp.shape[1])

    def reduce_scatter(self, inp, seg_sizes, my_rows):
        """Segment r of every rank's rows summed on rank r."""
        ws = self.state.world_size
        counts = [int(c) for c in seg_sizes.tolist()]
        buf = self._a2a(inp, counts, [int(my_rows)] * ws, inp.shape[1])
        return buf.view(ws, int(my_rows), inp.shape[1]).float().sum(0).to(inp.dtype)

    def exchange_fixed(self, send, recv):
        dist.all_to_all_single(recv, send.contiguous(), group=self.group)


class P2PExchange:
    """Rows go from the sender's tensor straight into the receiver's inbox with
    16-byte stores over NVLink. Inboxes are created once and mapped into every
    peer through CUDA IPC handles exchanged over torch.distributed."""

    name = "p2p"

    def __init__(self, state, region_bytes, group=None, ctx=None, timeout_ns=0):
        self.state = state
        self.group = group
        self.timeout_ns = int(timeout_ns)
        # The single cooperative kernel (push, wait and pull overlapped by chunks) is opt-in:
        # measured on 4 B200s it moves 67 584 x 1 KiB rows in 146 us against 162 us for the three
        # kernels, but 495 616 x 2 KiB rows in 1.55 ms (1 chunk) to 2.08 ms (8 chunks) against 1.47 ms.
        self.use_fused = os.environ.get("APT_P2P_FUSED", "0") == "1"
        self.chunks = max(1, min(8, int(os.environ.get("APT_P2P_CHUNKS", "1"))))
        self._off_dev = None
        self._off_host = None
        # Direct placement (opt-in, APT_P2P_DIRECT=1): the feature shuffle writes every row to its
        # final slot of a landing buffer on the receiving GPU, and the tensor it returns is a view of
        # that buffer, valid until APT_P2P_DIRECT_SLOTS (default 4) further feature shuffles have run.
        self.direct = os.environ.get("APT_P2P_DIRECT", "0") == "1"
        self._landing_turn = 0
        self._landing_views = {}
        self._landing_slots = max(1, int(os.environ.get("APT_P2P_DIRECT_SLOTS", "4")))
        if ctx is not None:  # same-process ranks (tests): contexts are wired by the caller
            self.ctx = ctx
            self.direct = self.direct and lib.apt_p2p_landing_bytes(ctx) > 0
            return
        handle = ctypes.create_string_buffer(_lib.IPC_HANDLE_BYTES)
        ctx_p = ctypes.c_void_p()
        landing_slots = self._landing_slots if self.direct else 0
        landing_bytes = (int(os.environ.get("APT_P2P_LANDING_MB", "0")) << 20) or int(region_bytes)
        check(lib.apt_p2p_create_landing(state.rank, state.world_size, int(region_bytes),
                                         landing_bytes if landing_slots else 0, landing_slots,
                                         ctypes.byref(ctx_p), handle))
        self.ctx = ctx_p
        handles = exchange_blobs(bytes(handle.raw), group)
        for r, h in enumerate(handles):
            if r != state.rank:
                check(lib.apt_p2p_attach(self.ctx, r, ctypes.c_char_p(h)))
        dist.barrier(group=group)

    @property
    def region_bytes(self):
        return int(lib.apt_p2p_region_bytes(self.ctx))

    def probe_peer_copy(self, peer: int, nbytes: int):
        """Enqueues one plain copy of nbytes from this rank's inbox into `peer`'s (apt_p2p_probe_copy):
        the link rate a shuffle is compared with. Call it only between exchanges, behind a barrier."""
        check(lib.apt_p2p_probe_copy(self.ctx, int(peer), int(nbytes), _stream()))

    def poisoned(self) -> bool:
        """True once a wait of this rank ran out of time. The inbox then refuses every further
        exchange (the kernels set the peer-timeout flag and store nothing): all ranks have to
        build new exchanges (ops.init) behind a host barrier."""
        out = ctypes.c_int(0)
        check(lib.apt_p2p_poisoned(self.ctx, ctypes.byref(out)))
        return bool(out.value)

    def _offsets_to_device(self, send_cpu, recv_cpu=None):
        """CPU offsets -> device, through a pinned staging block so the copy does
        not stall the stream. Four alternating slots let back-to-back calls keep
        their own copy. Returns (send offsets, recv offsets) device views."""
        ws = self.state.world_size
        if self._off_dev is None:
            self._off_host = torch.zeros((4, 64), dtype=torch.int64).pin_memory()
            self._off_dev = torch.zeros((4, 64), dtype=torch.int64, device=self.state.device())
            self._slot = 0
            self._events = [None] * 4
        k = self._slot
        self._slot = (k + 1) % 4
        if self._events[k] is not None:
            self._events[k].synchronize()  # the staging slot's last copy has left the host
        self._off_host[k, :ws].copy_(send_cpu.to(torch.int64))
        if recv_cpu is not None:
            self._off_host[k, 32:32 + ws].copy_(recv_cpu.to(torch.int64))
        self._off_dev[k].copy_(self._off_host[k], non_blocking=True)
        ev = torch.cuda.Event()
        ev.record()
        self._events[k] = ev
        return self._off_dev[k, :32], self._off_dev[k, 32:]

    def _fused(self, src, src_index, index_is_dest, send_cpu, recv_cpu, pull_index, num_dst_rows, row_bytes, dst):
        """One cooperative kernel (push, wait and pull overlapped by chunks) when the
        rows are 16-byte multiples; returns False if the three-kernel path must be
        used. Every rank has to take the same branch with the same chunk count, so
        both depend only on the row size and on configuration, never on this
        rank's own sizes or addresses."""
        if not self.use_fused or row_bytes % 16:
            return False
        if src.numel() and src.data_ptr() % 16:
            src = src.clone()
        assert dst.numel() == 0 or dst.data_ptr() % 16 == 0
        send_dev, recv_dev = self._offsets_to_device(send_cpu, recv_cpu)
        check(lib.apt_p2p_alltoall_fused(self.ctx, _ptr(src), _ptr(src_index), int(index_is_dest), _ptr(send_dev),
                                         _ptr(recv_dev), _ptr(pull_index), int(num_dst_rows), int(row_bytes),
                                         self.chunks, _ptr(dst), self.state.status_ptr(), self.timeout_ns,
                                         _stream()))
        return True

    def _push(self, src, index, index_is_dest, offsets_dev, max_rows, row_bytes):
        check(lib.apt_p2p_push(self.ctx, _ptr(src), _ptr(index), int(index_is_dest), _ptr(offsets_dev),
                               int(max_rows), int(row_bytes), self.state.status_ptr(), _stream()))

    def _wait(self, counts_dev):
        check(lib.apt_p2p_wait(self.ctx, _ptr(counts_dev), self.state.status_ptr(), self.timeout_ns, _stream()))

    def _pull(self, counts_dev, index, index_is_source, num_dst_rows, max_rows, row_bytes, dst):
        check(lib.apt_p2p_pull(self.ctx, _ptr(counts_dev), _ptr(index), int(index_is_source), int(num_dst_rows),
                               int(max_rows), int(row_bytes), _ptr(dst), _stream()))

    def _check_capacity(self, max_rows_per_peer, row_bytes):
        if max_rows_per_peer * row_bytes > self.region_bytes:
            raise RuntimeError(
                f"p2p inbox region of {self.region_bytes} bytes cannot hold {max_rows_per_peer} rows of "
                f"{row_bytes} bytes; raise APT_P2P_REGION_MB (APT_P2P_LANE_REGION_MB for the inboxes of a "
                f"sampler's extra lanes)")

    def exchange_ids(self, sorted_ids, sizes, offsets):
        st = self.state
        ws = st.world_size
        n = sorted_ids.numel()
        self._check_capacity(n, 8)
        counts_dev = torch.empty(ws + 1, dtype=torch.int64, device=sorted_ids.device)
        self._push(sorted_ids, None, 0, offsets, n, 8)
        self._wait(counts_dev)
        # one host read brings the received counts, my bucket offsets and the status word
        host = torch.cat([counts_dev, offsets]).cpu()
        st.read_words()
        recv_counts = host[:ws]
        recv_offset = recv_counts.cumsum(0)
        total = int(recv_offset[-1])
        recv = torch.empty(total, dtype=torch.int64, device=sorted_ids.device)
        self._pull(counts_dev, None, 0, total, total, 8, recv)
        return recv, recv_offset, host[ws + 1:].clone()

    def exchange_ids_enqueue(self, sorted_ids, sizes, offsets, counts_out=None):
        """Stream-ordered seed exchange without a host read. Every rank is taken
        to send at most sorted_ids.numel() ids (the ranks run the same batch
        shape), which bounds what this rank can receive."""
        st = self.state
        ws = st.world_size
        n = sorted_ids.numel()
        self._check_capacity(n, 8)
        counts_dev = counts_out if counts_out is not None else \
            torch.empty(ws + 1, dtype=torch.int64, device=sorted_ids.device)
        self._push(sorted_ids, None, 0, offsets, n, 8)
        self._wait(counts_dev)
        recv = torch.empty(ws * n, dtype=torch.int64, device=sorted_ids.device)
        self._pull(counts_dev, None, 0, ws * n, ws * n, 8, recv)
        return recv, counts_dev

    def _landing_view(self, slot, rows, width, dtype):
        """The first rows x width elements of landing buffer `slot` as a tensor (no copy)."""
        base = self._landing_views.get(slot)
        if base is None:
            nbytes = int(lib.apt_p2p_landing_bytes(self.ctx))
            ptr = lib.apt_p2p_landing(self.ctx, slot)

            class _Raw:
                __cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (int(ptr), False),
                                            "version": 2}

            base = torch.as_tensor(_Raw(), device=self.state.device())
            self._landing_views[slot] = base
        esz = torch.empty(0, dtype=dtype).element_size()
        return base[:rows * width * esz].view(dtype).view(rows, width)

    def _exchange_rows_direct(self, inputs, send_offset, recv_offset, permutation, fwd):
        """Two all-to-alls and no pull: the receiver sends each sender the final slot of every
        row it will get (8 bytes per row), the senders then store the rows at those slots of the
        receiver's landing buffer."""
        st = self.state
        ws = st.world_size
        width = inputs.shape[1]
        row_bytes = width * inputs.element_size()
        total_recv = int(recv_offset[-1])
        out_rows = permutation.numel() if fwd else total_recv
        if out_rows * row_bytes > int(lib.apt_p2p_landing_bytes(self.ctx)):
            raise RuntimeError(f"direct feature shuffle: {out_rows} rows of {row_bytes} bytes do not fit the landing "
                               "buffer; raise APT_P2P_LANDING_MB (every rank must take the same path)")
        self._check_capacity(max(_counts(recv_offset) + _counts(send_offset)), 8)
        dev = inputs.device
        if fwd:   # concatenation row p ends at the row i with permutation[i] == p
            slots = torch.empty(total_recv, dtype=torch.int64, device=dev)
            slots[permutation] = torch.arange(permutation.numel(), device=dev)
        else:     # rows arrive in concatenation order
            slots = torch.arange(total_recv, dtype=torch.int64, device=dev)
        counts_dev = torch.empty(ws + 1, dtype=torch.int64, device=dev)
        ask_off, _ = self._offsets_to_device(recv_offset)
        self._push(slots, None, 0, ask_off, total_recv, 8)
        self._wait(counts_dev)
        slot = self._landing_turn
        self._landing_turn = (slot + 1) % self._landing_slots
        off_dev, _ = self._offsets_to_device(send_offset)
        index, by_dest = (None, 0) if fwd else (permutation, 1)
        check(lib.apt_p2p_push_direct(self.ctx, _ptr(inputs), _ptr(index), by_dest, _ptr(off_dev), inputs.shape[0],
                                      int(row_bytes), slot, st.status_ptr(), _stream()))
        self._wait(counts_dev)
        return self._landing_view(slot, out_rows, width, inputs.dtype)

    def exchange_rows(self, inputs, send_offset, recv_offset, permutation, fwd):
        st = self.state
        ws = st.world_size
        row_bytes = inputs.shape[1] * inputs.element_size()
        if self.direct and row_bytes % 16 == 0:
            return self._exchange_rows_direct(inputs, send_offset, recv_offset, permutation, fwd)
        self._check_capacity(max(_counts(send_offset)), row_bytes)
        rows_in = inputs.shape[0]
        total_out = int(recv_offset[-1])
        if fwd:
            out = torch.empty((permutation.numel(), inputs.shape[1]), dtype=inputs.dtype, device=inputs.device)
            if self._fused(inputs, None, 0, send_offset, recv_offset, permutation, permutation.numel(),
                           row_bytes, out):
                return out
        else:
            out = torch.empty((total_out, inputs.shape[1]), dtype=inputs.dtype, device=inputs.device)
            if self._fused(inputs, permutation, 1, send_offset, recv_offset, None, total_out, row_bytes, out):
                return out
        off_dev, _ = self._offsets_to_device(send_offset)
        counts_dev = torch.empty(ws + 1, dtype=torch.int64, device=inputs.device)
        if fwd:
            self._push(inputs, None, 0, off_dev, rows_in, row_bytes)
            self._wait(counts_dev)
            out = torch.empty((permutation.numel(), inputs.shape[1]), dtype=inputs.dtype, device=inputs.device)
            self._pull(counts_dev, permutation, 1, permutation.numel(), permutation.numel(), row_bytes, out)
        else:
            self._push(inputs, permutation, 1, off_dev, rows_in, row_bytes)
            self._wait(counts_dev)
            out = torch.empty((total_out, inputs.shape[1]), dtype=inputs.dtype, device=inputs.device)
            self._pull(counts_dev, None, 0, total_out, total_out, row_bytes, out)
        return out

    def alltoall(self, inp, out, send_offset, recv_offset, expand):
        st = self.state
        row_bytes = expand * inp.element_size()
        self._check_capacity(max(_counts(send_offset)), row_bytes)
        rows_in = int(send_offset[-1])
        total_out = int(recv_offset[-1])
        if self._fused(inp, None, 0, send_offset, recv_offset, None, total_out, row_bytes, out):
            return
        off_dev, _ = self._offsets_to_device(send_offset)
        counts_dev = torch.empty(st.world_size + 1, dtype=torch.int64, device=inp.device)
        self._push(inp, None, 0, off_dev, rows_in, row_bytes)
        self._wait(counts_dev)
        self._pull(counts_dev, None, 0, total_out, total_out, row_bytes, out)

    def allbroadcast(self, inp, recv_counts):
        """Every rank's rows to every rank, in rank order: one push whose source
        index repeats this rank's rows once per peer."""
        st = self.state
        ws = st.world_size
        n, width = inp.shape
        row_bytes = width * inp.element_size()
        self._check_capacity(max([n] + [int(c) for c in recv_counts]), row_bytes)
        index = torch.arange(n, device=inp.device).repeat(ws)
        off_dev, _ = self._offsets_to_device(torch.arange(1, ws + 1, dtype=torch.int64) * n)
        counts_dev = torch.empty(ws + 1, dtype=torch.int64, device=inp.device)
        self._push(inp, index, 0, off_dev, n * ws, row_bytes)
        self._wait(counts_dev)
        total = int(sum(int(c) for c in recv_counts))
        out = torch.empty((total, width), dtype=inp.dtype, device=inp.device)
        self._pull(counts_dev, None, 0, total, total, row_bytes, out)
        return out

    def reduce_scatter(self, inp, seg_sizes, my_rows):
        """Segment r of every rank's rows summed on rank r: the segments are pushed
        into the owners' inboxes and one kernel there adds the world_size copies
        in rank order."""
        from .ops import _DTYPE_CODE

        st = self.state
        ws = st.world_size
        width = inp.shape[1]
        row_bytes = width * inp.element_size()
        self._check_capacity(max(int(c) for c in seg_sizes.tolist()), row_bytes)
        off_dev, _ = self._offsets_to_device(seg_sizes.cumsum(0))
        counts_dev = torch.empty(ws + 1, dtype=torch.int64, device=inp.device)
        self._push(inp, None, 0, off_dev, inp.shape[0], row_bytes)
        self._wait(counts_dev)
        out = torch.empty((int(my_rows), width), dtype=inp.dtype, device=inp.device)
        check(lib.apt_p2p_pull_sum(self.ctx, _ptr(counts_dev), _DTYPE_CODE[inp.dtype], int(my_rows), width, _ptr(out),
                                   st.status_ptr(), _stream()))
        return out

    def allbroadcast_enqueue(self, inp, n_dev, counts_out):
        """Stream-ordered all-broadcast of the first n_dev rows of inp (a device count) without a
        host read: one push in which every peer's bucket is the same source rows. Every rank is
        taken to send at most inp.shape[0] rows. Returns (buffer of world_size x inp.shape[0] rows
        with the received rows in rank order, counts_out[world_size + 1])."""
        ws = self.state.world_size
        n_max, width = inp.shape
        row_bytes = width * inp.element_size()
        self._check_capacity(n_max, row_bytes)
        if getattr(self, "_steps_dev", None) is None:
            self._steps_dev = torch.arange(1, ws + 1, dtype=torch.int64, device=inp.device)
            self._fixed_counts = torch.empty(ws + 1, dtype=torch.int64, device=inp.device)
        offsets = self._steps_dev * n_dev
        self._push(inp, None, 2, offsets, n_max * ws, row_bytes)
        self._wait(counts_out)
        recv = torch.empty((ws * n_max, width), dtype=inp.dtype, device=inp.device)
        self._pull(counts_out, None, 0, ws * n_max, ws * n_max, row_bytes, recv)
        return recv, counts_out

    def exchange_fixed(self, send, recv):
        """All-to-all of one row of send[world_size, k] per peer into recv[world_size, k]; sizes
        are the same everywhere, so nothing is read on the host."""
        ws = self.state.world_size
        if getattr(self, "_steps_dev", None) is None:
            self._steps_dev = torch.arange(1, ws + 1, dtype=torch.int64, device=send.device)
            self._fixed_counts = torch.empty(ws + 1, dtype=torch.int64, device=send.device)
        row_bytes = send.shape[1] * send.element_size()
        self._push(send, None, 0, self._steps_dev, ws, row_bytes)
        self._wait(self._fixed_counts)
        self._pull(self._fixed_counts, None, 0, ws, ws, row_bytes, recv)

    def close(self):
        if self.ctx is not None:
            lib.apt_p2p_destroy(self.ctx)
            self.ctx = None


def exchange_blobs(blob: bytes, group=None):
    """All-gather of one small bytes object per rank over the process group
    (any backend; gloo on CPU works). Returns the list in rank order."""
    out = [None] * dist.get_world_size(group)
    dist.all_gather_object(out, blob, group=group)
    return out


def make_exchange(state):
    """Backend for this process: local for one rank; otherwise
    APT_SHUFFLE_BACKEND (default p2p; nccl = the library baseline)."""
    if state.world_size == 1:
        return LocalExchange(state)
    if not dist.is_initialized():
        raise RuntimeError("world_size > 1 needs torch.distributed.init_process_group before npc.init")
    if state.shuffle_backend == "nccl":
        return NcclExchange(state)
    if state.shuffle_backend == "p2p":
        return P2PExchange(state, state.p2p_region_bytes)
    raise RuntimeError(f"unknown APT_SHUFFLE_BACKEND {state.shuffle_backend!r}")
