"""Benchmark of the mini-batch data path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl reference]

One step = one mini-batch per GPU of the papers-shaped NPC run: three-hop
fanout sampling (the outermost hop at the owner of each frontier node),
relabelling of every hop, the seed shuffle, and the cache-aware gather of the
input features. The printed JSON line carries
  value      mini-batches/s over all GPUs, seeds already resident in HBM
  e2e        the same through host buffers: seeds copied from pinned host
             memory every step and a digest of the gathered rows read back
  roofline   the HBM-bound gather kernel (cache hits), timed with CUDA events
             on its own stream inside the timed region
  roofline_link  the host-link-bound gather kernel (cache misses)
  cpu_baseline   the C restatement of the path (oracle/) on the host cores
``--impl reference`` times that CPU restatement alone (the reference has no CPU
implementation of its own beyond the gather, and cannot be built here).
"""
import argparse
import ctypes
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

STAGE_TAGS = ("sample_relabel", "sample", "relabel", "bucket", "unique_sorted", "gather_hit", "gather_miss",
              "p2p_push", "p2p_wait", "p2p_pull")
# DRAM bytes (read + written) per algorithmic byte of the hit kernel, from an ncu capture of that kernel
# alone at the mini-batch's size (143 000 rows of 512 bytes out of a 27.8 M-row cache table); None until
# such a capture exists for the current kernel.
HIT_DRAM_BYTES_PER_ALGORITHMIC_BYTE = None
HIT_TRAFFIC_SOURCE = "not captured for this kernel yet"
METRIC = "sampled+gathered mini-batches/sec (whole box)"
UNIT = "mini-batches/s"


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--workload", default="c1_papers_np")
    ap.add_argument("--impl", default="apt_b200", choices=["apt_b200", "reference"])
    ap.add_argument("--cpu-batches", type=int, default=1000,
                    help="batches of the CPU-baseline sample (about 10 s of work on 16 host threads)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--stage", default="minibatch", choices=["minibatch", "gather", "shuffle", "ops", "strategies"],
                    help="gather: the cached feature gather alone on a synthetic table; "
                         "shuffle: the NPC feature shuffle alone (needs --gpus >= 2 under torchrun); "
                         "ops: sampling, relabelling, SpMM, SDDMM and the fused GAT block one by one; "
                         "strategies: the outermost hop and its first-layer exchange under NP, SNP with virtual "
                         "nodes and NFP, side by side (needs --gpus >= 2 under torchrun)")
    ap.add_argument("--hidden", type=int, default=256, help="--stage strategies: width of the exchanged rows")
    ap.add_argument("--rows", type=int, default=1_081_344, help="--stage gather: rows per call")
    ap.add_argument("--table-rows", type=int, default=4_000_000, help="--stage gather: rows of the cached table")
    ap.add_argument("--feat-dim", type=int, default=128)
    ap.add_argument("--feat-dtype", default="f32", choices=["f32", "bf16", "f16"])
    ap.add_argument("--miss-frac", type=float, default=0.0, help="--stage gather: share of rows read from host memory")
    return ap.parse_args()


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """nvidia-smi clocks and throttle reasons of this rank's GPU during the timed region."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index = index
        self.proc = None
        self.path = None

    def start(self):
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, smax, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        with open(self.path) as f:
            for line in f:
                p = [x.strip() for x in line.split(",")]
                if len(p) < 9:
                    continue
                try:
                    sm.append(float(p[1]))
                    smax.append(float(p[2]))
                except ValueError:
                    continue
                for name, val in zip(names, p[5:9]):
                    if val.lower().startswith("active"):
                        reasons.add(name)
        os.unlink(self.path)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(smax) if smax else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def batches_of(train_ids, batch, count, offset=0):
    """`count` consecutive seed batches out of the rank's training ids (wrapping)."""
    n = train_ids.numel()
    out = []
    for i in range(count):
        lo = ((offset + i) * batch) % max(n - batch + 1, 1)
        out.append(train_ids[lo:lo + batch].contiguous())
    return out


# ------------------------------------------------------------------ CPU baseline
class CpuPath:
    """One mini-batch of the same path on the host cores with the C restatement
    (oracle/apt_oracle.c): every hop's sampling and relabelling, the owner
    bucketing + sorted unique of the outermost hop, and the reference's CPU
    gather (host table only, src/load_subtensor.cc:10-17)."""

    def __init__(self, inst):
        import numpy as np

        so = os.path.join(ROOT, "oracle", "libapt_oracle.so")
        if not os.path.exists(so):
            subprocess.run(["make", "-C", os.path.join(ROOT, "oracle")], check=True, capture_output=True)
        self.lib = ctypes.CDLL(so)
        self.lib.oracle_relabel.restype = ctypes.c_int64
        self.lib.oracle_unique_sorted.restype = ctypes.c_int64
        self.np = np
        self.w = inst.workload
        self.indptr = inst.indptr.cpu().numpy()
        self.indices = inst.indices.cpu().numpy()
        self.feats = inst.host_feats.view(torch.uint8).numpy() if inst.host_feats.dtype == torch.bfloat16 \
            else inst.host_feats.numpy()
        self.row_bytes = inst.host_feats.shape[1] * inst.host_feats.element_size()
        n = self.w.num_nodes
        self.pos_map = -np.arange(n, dtype=np.int64) - 2      # every row in the host table
        self.min_vids = inst.min_vids.numpy().astype(np.int64)
        # torchrun hands its workers OMP_NUM_THREADS=1: the baseline takes the host's threads explicitly
        self.lib.oracle_set_threads.restype = ctypes.c_int
        self.cores = int(self.lib.oracle_set_threads(os.cpu_count() or 1))

    @staticmethod
    def _p(a):
        return a.ctypes.data_as(ctypes.c_void_p)

    def _sample(self, seeds, fanout, call_id):
        np = self.np
        out = np.empty(len(seeds) * fanout, dtype=np.int64)
        self.lib.oracle_sample(self._p(seeds), ctypes.c_int64(len(seeds)), fanout, None, None, None,
                               self._p(self.indptr), self._p(self.indices), ctypes.c_uint64(7777777),
                               ctypes.c_uint32(call_id), self._p(out))
        return out

    def _relabel(self, seeds, nbrs):
        np = self.np
        uniq = np.empty(len(seeds) + len(nbrs), dtype=np.int64)
        rel = np.empty(len(nbrs), dtype=np.int64)
        u = self.lib.oracle_relabel(self._p(seeds), ctypes.c_int64(len(seeds)), self._p(nbrs),
                                    ctypes.c_int64(len(nbrs)), self._p(uniq), self._p(rel))
        return uniq[:u], rel

    def batch(self, seeds):
        np = self.np
        cur = np.ascontiguousarray(seeds, dtype=np.int64)
        call = 0
        for f in reversed(self.w.fanouts[1:]):
            nbr = self._sample(cur, f, call)
            call += 1
            cur, _ = self._relabel(cur, nbr)
        ws = len(self.min_vids) - 1
        sorted_ids, perm = np.empty_like(cur), np.empty_like(cur)
        sizes, offs = np.empty(ws, dtype=np.int64), np.empty(ws, dtype=np.int64)
        self.lib.oracle_bucket(self._p(cur), ctypes.c_int64(len(cur)), self._p(self.min_vids), ws, ctypes.c_int64(0),
                               0, 0, ws, self._p(sorted_ids), self._p(perm), self._p(sizes), self._p(offs))
        uniq, inv = np.empty_like(cur), np.empty_like(cur)
        u = self.lib.oracle_unique_sorted(self._p(sorted_ids), ctypes.c_int64(len(cur)), self._p(uniq), self._p(inv))
        uniq = uniq[:u]
        nbr = self._sample(uniq, self.w.fanouts[0], call)
        inputs, _ = self._relabel(uniq, nbr)
        out = np.empty((len(inputs), self.row_bytes), dtype=np.uint8)
        self.lib.oracle_gather(self._p(inputs), ctypes.c_int64(len(inputs)), self._p(self.pos_map), None,
                               ctypes.c_int64(self.row_bytes), self._p(self.feats), ctypes.c_int64(self.row_bytes),
                               ctypes.c_int64(0), self._p(out))
        return len(inputs)

    def time(self, seed_batches, warmup=1):
        for b in seed_batches[:warmup]:
            self.batch(b)
        t0 = time.perf_counter()
        rows = 0
        for b in seed_batches[warmup:]:
            rows += self.batch(b)
        dt = time.perf_counter() - t0
        n = len(seed_batches) - warmup
        return n / dt, dt, rows / max(n, 1)


# ------------------------------------------------------------------ stage: gather
def stage_gather(args):
    """The cached feature gather alone: `rows` random rows out of a cache table of
    `table_rows` rows (larger than L2), a share `miss_frac` of them from pinned
    host memory instead. One JSON line with the hit-copy kernel's roofline."""
    import apt_b200  # noqa: F401
    from apt_b200 import ops
    from apt_b200._lib import lib

    dt = {"f32": torch.float32, "bf16": torch.bfloat16, "f16": torch.float16}[args.feat_dtype]
    torch.cuda.set_device(0)
    n_dev, dim = args.table_rows, args.feat_dim
    n_host = max(16, int(n_dev * 0.25)) if args.miss_frac > 0 else 16
    g = torch.Generator(device="cuda").manual_seed(5)
    dev_feats = torch.randn((n_dev, dim), generator=g, device="cuda").to(dt)
    host = torch.randn((n_host, dim)).to(dt).pin_memory()
    n = n_dev + n_host                       # ids [0, n_dev) cached, [n_dev, n) only in host memory
    ops.cache_feats_shared(n, host, dev_feats, torch.arange(n_dev), torch.arange(n_host) + n_dev, 0)
    row_bytes = dim * dev_feats.element_size()
    n_miss = int(args.rows * args.miss_frac)
    peak, peak_kind = peaks()
    lib.apt_profile_enable(1)
    total_ms = 0.0
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for it in range(args.warmup + args.steps):
        ids = torch.cat([torch.randint(0, n_dev, (args.rows - n_miss,), generator=g, device="cuda"),
                         torch.randint(n_dev, n, (n_miss,), generator=g, device="cuda")])
        ids = ids[torch.randperm(args.rows, generator=g, device="cuda")].contiguous()
        if it == args.warmup:
            for tag in (b"gather_hit", b"gather_miss"):
                t, k = ctypes.c_double(), ctypes.c_int64()
                lib.apt_profile_read(tag, ctypes.byref(t), ctypes.byref(k))
        torch.cuda.nvtx.range_push("apt_timed")
        ev0.record()
        out = ops.load_subtensor(ids)
        ev1.record()
        torch.cuda.nvtx.range_pop()
        torch.cuda.synchronize()
        if it >= args.warmup:
            total_ms += ev0.elapsed_time(ev1)
    ops.check_status()
    res = {}
    for tag in ("gather_hit", "gather_miss"):
        t, k = ctypes.c_double(), ctypes.c_int64()
        lib.apt_profile_read(tag.encode(), ctypes.byref(t), ctypes.byref(k))
        res[tag] = (t.value, k.value)
    hit_ms, hit_n = res["gather_hit"]
    # the hit kernel reads an id and a position-map entry for every requested row (16 bytes) and moves
    # every cached row once in and once out
    hit_bytes = (args.rows - n_miss) * 2 * row_bytes + args.rows * 16
    gbs = hit_bytes / (hit_ms / hit_n * 1e-3) / 1e9
    call_gbs = args.rows * (2 * row_bytes + 16) / (total_ms / args.steps * 1e-3) / 1e9
    print(json.dumps({
        "metric": "cached feature gather GB/s (hit-copy kernel)", "value": gbs, "unit": "GB/s", "n_gpus": 1,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": total_ms / args.steps, "higher_is_better": True,
        "dtype": args.feat_dtype, "data": "synthetic",
        "config": {"workload": "stage gather", "rows": args.rows, "table_rows": n_dev, "row_bytes": row_bytes,
                   "miss_frac": args.miss_frac, "l2": "cache table larger than the 126 MB L2, new random ids every call"},
        "whole_call_gbs": call_gbs,
        "stage_us": {k: 1000.0 * v[0] / max(v[1], 1) for k, v in res.items()},
        "roofline": {"kernel": "k_gather_hits", "bound": "hbm", "achieved": round(gbs, 1), "peak": peak,
                     "peak_kind": peak_kind, "unit": "GB/s", "frac": round(gbs / peak, 4), "traffic": None}}))


# ------------------------------------------------------------------ stage: ops
def stage_ops(args):
    """Every remaining operator of the path alone, at the size of the papers-shaped outermost hop
    (67 584 destination nodes x fanout 15) on the small R-MAT graph (CSC larger than L2):
    time per call (CUDA events) and algorithmic GB/s against the measured HBM peak."""
    import apt_b200  # noqa: F401
    from apt_b200 import ops, synthetic
    from apt_b200._lib import lib

    torch.cuda.set_device(0)
    w = synthetic.WORKLOADS["c0_small_np"]
    indptr, indices = synthetic.build_csc(w)
    e = torch.empty(0, dtype=torch.int64)
    ops.mix_cache_graphs(0, e, e, e, indptr, indices)
    S, f, n = 67_584, 15, w.num_nodes
    g = torch.Generator(device="cuda").manual_seed(9)
    peak, peak_kind = peaks()
    results = {}

    def read_tags(tags):
        out = {}
        for tag in tags:
            t_, k_ = ctypes.c_double(), ctypes.c_int64()
            lib.apt_profile_read(tag.encode(), ctypes.byref(t_), ctypes.byref(k_))
            out[tag] = round(1e6 * t_.value / max(k_.value, 1), 2)
        return out

    def timed(name, fn, algo_bytes, fresh=None, tags=()):
        for _ in range(args.warmup):
            fn(fresh() if fresh else None)
        inputs = [fresh() if fresh else None for _ in range(args.steps)]
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.nvtx.range_push("apt_timed")
        e0.record()
        for x in inputs:
            fn(x)
        e1.record()
        torch.cuda.nvtx.range_pop()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / args.steps
        gbs = algo_bytes / (ms * 1e-3) / 1e9
        results[name] = {"us": round(1000 * ms, 2), "algorithmic_mb": round(algo_bytes / 1e6, 2),
                         "gbs": round(gbs, 1), "frac_of_hbm_peak": round(gbs / peak, 4)}
        if tags:   # a second, untimed pass with an event pair around each launch group
            ops.profile_enable(True)
            read_tags(tags)
            for x in inputs[:5]:
                fn(x)
            torch.cuda.synchronize()
            ops.profile_enable(False)
            results[name]["launch_groups_us"] = read_tags(tags)

    def seeds():
        return torch.randint(0, n, (S,), generator=g, device="cuda")

    # sampling: 32 + 16 f bytes per seed
    timed("sample_csc_fanout (67 584 seeds x 15)", lambda s: ops._sample(s, f), S * (32 + 16 * f), seeds)
    nbr_pool = [ops._sample(seeds(), f) for _ in range(4)]
    seed_pool = [torch.randperm(n, generator=g, device="cuda")[:S].contiguous() for _ in range(4)]
    k = [0]

    def relabel(_):
        k[0] += 1
        ops._relabel_enqueue(seed_pool[k[0] % 4], nbr_pool[k[0] % 4], None, ops.STATE.word(0))

    items = S * (1 + f)
    timed("relabel_csc (1.08 M items, no host read)", relabel, 16 * items)
    uniq, rel = ops.relabel_csc(seed_pool[0], nbr_pool[0])
    n_src, E = uniq.numel(), rel.numel()
    col = torch.arange(S, device="cuda").repeat_interleave(f)
    off = [torch.tensor(v, device="cuda") for v in ([0, E], [0, n_src], [0, S])]
    spmm_tags = ("spmm_ranges", "spmm_group", "spmm_rows", "spmm_long")
    for dt, name in ((torch.float32, "f32"), (torch.bfloat16, "bf16")):
        D = 256
        x = torch.randn((n_src, D), generator=g, device="cuda").to(dt)
        esz = x.element_size()
        ws = ops.STATE.workspace("spmm", 1)
        timed(f"spmm_copy_u_sum {name} D=256 (1.01 M edges, grouped)",
              lambda _: ops._spmm(0, rel, col, x, None, off[0], off[1], off[2]), E * (16 + D * esz) + S * D * esz,
              tags=spmm_tags)
        gsd = torch.randn((S, D), generator=g, device="cuda").to(dt)
        timed(f"spmm_copy_u_sum {name} D=256 backward shape (scattered)",
              lambda _: ops._spmm(0, col, rel, gsd, None, off[0], off[2], off[1]), E * (16 + D * esz) + n_src * D * esz,
              tags=spmm_tags)
    el = torch.randn((n_src, 4), generator=g, device="cuda")
    er = torch.randn((S, 4), generator=g, device="cuda")
    timed("sddmm_u_add_v f32 D=4 (GAT scores)", lambda _: ops.sddmm_u_add_v(rel, col, el, er, *off), E * (16 + 3 * 4 * 4))
    ft = torch.randn((n_src, 4, 64), generator=g, device="cuda").bfloat16()
    elb, erb = el.bfloat16(), er.bfloat16()
    timed("gat_edge_softmax_sum bf16 4 heads x 64",
          lambda _: ops.gat_edge_softmax_sum(rel, col, ft, elb, erb, S), E * (8 + 4 * 2 + 256 * 2) + S * 256 * 2)
    gob = torch.randn((S, 4, 64), generator=g, device="cuda").bfloat16()
    # backward: the edge kernel reads ft twice, then two reverse SpMM calls (u_mul_e over 256 columns, copy_e over 4)
    timed("gat_edge_softmax_sum backward bf16 4 heads x 64 (edge kernel + 2 reverse SpMM)",
          lambda _: ops.gat_edge_softmax_sum_backward(rel, col, ft, elb, erb, gob),
          E * (8 + 4 * 2 * 2 + 2 * 256 * 2) + S * 256 * 2 + E * (16 + 256 * 2 + 4 * 2) + n_src * 256 * 2,
          tags=("gat_bwd_rows",) + spmm_tags)
    ids = torch.randint(0, n, (S,), generator=g, device="cuda")
    ops.register_min_vids(torch.tensor([0, n]))
    timed("unique_sorted (67 584 ids over 2^20)", lambda _: ops._unique_enqueue(ids, None, 0, n, ops.STATE.word(1)),
          16 * S + n // 1024 * 4)
    timed("bucket_by_owner (67 584 ids)", lambda _: ops._bucket(ids), 24 * S)
    ops.check_status()
    print(json.dumps({"metric": "operators of the mini-batch path, one by one", "unit": "us per call", "n_gpus": 1,
                      "steps": args.steps, "warmup": args.warmup, "data": "synthetic",
                      "config": {"workload": "stage ops", "graph": w.name, "dst_nodes": S, "fanout": f,
                                 "block_src_nodes": n_src, "edges": E},
                      "peak": {"hbm_gbs": peak, "kind": peak_kind}, "ops": results}))


# ------------------------------------------------------------------ stage: shuffle
def stage_shuffle(args):
    """The NPC feature shuffle alone (FeatShuffle forward and backward): every rank asks
    for `rows` rows owned uniformly at random by all ranks, the owners send them back.
    Reports GB/s per GPU and direction over NVLink for the peer-to-peer path, split into
    its kernels, next to the library all-to-all on the same rows."""
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world < 2:
        raise SystemExit("--stage shuffle needs at least 2 ranks (torchrun)")
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    import apt_b200  # noqa: F401
    from apt_b200 import ops
    from apt_b200._lib import lib
    from apt_b200.exchange import NcclExchange

    dt = {"f32": torch.float32, "bf16": torch.bfloat16, "f16": torch.float16}[args.feat_dtype]
    dim = args.feat_dim
    row_bytes = dim * torch.empty(0, dtype=dt).element_size()
    rows = args.rows
    ops.STATE.p2p_region_bytes = max(64 << 20, int(2.0 * rows / world * row_bytes) + (8 << 20))
    ops.init(rank, local, world, ops.nccl_get_unique_id(), world)
    p2p, nccl = ops.STATE.exchange, NcclExchange(ops.STATE)
    n = 1 << 24
    ops.register_min_vids(torch.tensor([n * r // world for r in range(world)] + [n]))
    g = torch.Generator(device="cuda").manual_seed(100 + rank)
    ids = torch.randint(0, n, (rows,), generator=g, device="cuda")
    recv_ids, perm, send_off, recv_off = ops.shuffle_seeds(ids)   # python names: send_offset = C++ recv_offset
    x = torch.randn((recv_ids.numel(), dim), generator=g, device="cuda").to(dt)
    grad = torch.randn((rows, dim), generator=g, device="cuda").to(dt)
    counts = [int(c) for c in (send_off - torch.cat([torch.zeros(1, dtype=torch.int64), send_off[:-1]])).tolist()]
    remote_out = (sum(counts) - counts[rank]) * row_bytes          # bytes this rank sends to other GPUs (fwd)

    def run(ex, fwd, profiled):
        ops.STATE.exchange = ex
        fn = (lambda: ops.feat_shuffle(x, send_off, recv_off, perm, dim, 1)) if fwd else \
             (lambda: ops.feat_shuffle(grad, recv_off, send_off, perm, dim, 0))
        for _ in range(args.warmup):
            fn()
        ops.profile_enable(profiled)
        for tag in (b"p2p_push", b"p2p_wait", b"p2p_pull", b"p2p_fused"):
            t_, k_ = ctypes.c_double(), ctypes.c_int64()
            lib.apt_profile_read(tag, ctypes.byref(t_), ctypes.byref(k_))
        torch.cuda.synchronize()
        dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.steps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        ops.profile_enable(False)
        ms = torch.tensor([e0.elapsed_time(e1) / args.steps], device="cuda")
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        stages = {}
        for tag in ("p2p_push", "p2p_wait", "p2p_pull", "p2p_fused"):
            t_, k_ = ctypes.c_double(), ctypes.c_int64()
            lib.apt_profile_read(tag.encode(), ctypes.byref(t_), ctypes.byref(k_))
            stages[tag] = 1000.0 * t_.value / max(k_.value, 1)
        return float(ms.item()), stages

    res = {}
    for name, ex in (("p2p", p2p), ("nccl", nccl)):
        for fwd in (True, False):
            ms, _ = run(ex, fwd, False)
            res[f"{name}_{'fwd' if fwd else 'bwd'}_ms"] = ms
    # the three separate kernels (push, wait, pull), to show what each part costs
    fused_was = p2p.use_fused
    p2p.use_fused = False
    res["p2p_unfused_fwd_ms"], stages = run(p2p, True, True)
    p2p.use_fused = fused_was
    ops.STATE.exchange = p2p
    ops.check_status()
    link_peak = 770.0      # GB/s per direction per GPU, measured peer copy on this pool (900 nominal)
    rem = torch.tensor([float(remote_out)], device="cuda")
    dist.all_reduce(rem, op=dist.ReduceOp.MAX)
    remote = float(rem.item())
    gbs = {k: remote / (v * 1e-3) / 1e9 for k, v in res.items()}
    push_gbs = remote / (stages["p2p_push"] * 1e-6) / 1e9
    if rank == 0:
        print(json.dumps({
            "metric": "NPC feature shuffle GB/s per GPU and direction over NVLink", "value": gbs["p2p_fwd_ms"],
            "unit": "GB/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": res["p2p_fwd_ms"], "higher_is_better": True, "dtype": args.feat_dtype, "data": "synthetic",
            "config": {"workload": "stage shuffle", "rows_per_gpu": rows, "row_bytes": row_bytes,
                       "remote_bytes_per_gpu": remote, "owners": "uniform over ranks",
                       "fused_kernel": bool(p2p.use_fused), "chunks": p2p.chunks},
            "ms": res, "gbs": gbs, "p2p_stage_us": stages,
            "roofline": {"kernel": "k_p2p_push", "bound": "nvlink", "achieved": round(push_gbs, 1), "peak": link_peak,
                         "peak_kind": "measured peer copy per direction (900 nominal)", "unit": "GB/s",
                         "frac": round(push_gbs / link_peak, 4), "traffic": None},
            "whole_op_frac_of_link": round(gbs["p2p_fwd_ms"] / link_peak, 4),
            "nccl_baseline_gbs": gbs["nccl_fwd_ms"]}))
    dist.barrier()
    dist.destroy_process_group()


# -------------------------------------------------------------- stage: strategies
def stage_strategies(args):
    """One mini-batch of the small graph (2^20 nodes, fanout [25, 10], 1024 seeds per GPU) through the
    sampler and the first-layer exchange of three strategies of the reference: NP (seeds to the owner,
    hidden rows back), SNP with virtual nodes (packed neighbour ids to the owner, partial sums per
    virtual node back) and NFP (frontiers and blocks to everyone, column slices summed by a
    reduce-scatter). Reports ms per mini-batch (max over ranks) and the bytes each strategy puts on
    NVLink per GPU, which is what the reference's planner trades off."""
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world < 2:
        raise SystemExit("--stage strategies needs at least 2 ranks (torchrun)")
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    import apt_b200
    from apt_b200 import ops, synthetic

    ops.STATE.p2p_region_bytes = 256 << 20
    ops.init(rank, local, world, ops.nccl_get_unique_id(), world)
    w = synthetic.WORKLOADS["c0_small_np"]
    indptr, indices = synthetic.build_csc(w)
    e = torch.empty(0, dtype=torch.int64)
    ops.mix_cache_graphs(0, e, e, e, indptr, indices)
    ops.register_min_vids(synthetic.partition_min_vids(w.num_nodes, world))
    H = args.hidden
    g = torch.Generator(device="cuda").manual_seed(500 + rank)
    steps = args.warmup + args.steps
    batches = [torch.randperm(w.num_nodes, generator=g, device="cuda")[:w.batch] for _ in range(steps)]
    table = torch.randn((w.num_nodes, H), generator=g, device="cuda")       # stands for the projected rows
    table_slice = table[:, :H // world].contiguous()
    one = lambda a, b: torch.tensor([a, b], device="cuda")
    cum = lambda t: torch.cat([torch.zeros(1, dtype=torch.int64), t.cumsum(0)]).cuda()
    volume = {}

    def np_step(seeds):
        smp = np_step.sampler
        in_nodes, _, blocks, perm, send_off, recv_off, inv = smp.sample(None, seeds)
        h = table[in_nodes[:blocks[0].num_dst]]                         # layer output of the owned frontier
        x = ops.rows_gather(h, inv)
        y = ops.feat_shuffle(x, send_off, recv_off, perm, H, 1)
        sent = int(send_off[-1]) - int(send_off[rank] - (send_off[rank - 1] if rank else 0))
        got = int(recv_off[-1]) - int(recv_off[rank] - (recv_off[rank - 1] if rank else 0))
        volume["NP"] = (got * 8, sent * H * 4)                          # ids out = rows this rank asked for
        return y

    np_step.sampler = apt_b200.MixedNeighborSampler(rank, w.fanouts, prefetch_features=False)

    def sp_step(seeds):
        smp = sp_step.sampler
        in_nodes, _, (b2, b1, *_), send_sizes, recv_sizes = smp.sample(None, seeds)
        h_vir = ops.spmm_copy_u_sum(b2.coo_row, b2.coo_col, table[b2.src_ids], one(0, b2.coo_row.numel()),
                                    one(0, b2.num_src), one(0, b2.num_dst))
        part = ops.sp_feat_shuffle(h_vir, recv_sizes, send_sizes, int(send_sizes[1::2].sum()), H, 0)
        out = ops.spmm_copy_u_sum(b1.coo_row, b1.coo_col, part, one(0, b1.coo_row.numel()), one(0, b1.num_src),
                                  one(0, b1.num_dst))
        ids = int(send_sizes[0::2].sum() - send_sizes[2 * rank])
        rows = int(recv_sizes[1::2].sum() - recv_sizes[2 * rank + 1])
        volume["SNP"] = (ids * 8, rows * H * 4)
        return out

    sp_step.sampler = apt_b200.SPVirtualSampler(rank, w.fanouts, model="SAGE")

    def mp_step(seeds):
        smp = mp_step.sampler
        in_nodes, _, blocks, send_size, recv_size = smp.sample(None, seeds)
        row, col, fsz, csz, ssz = blocks[0]
        xs = table_slice[in_nodes]                                       # this rank's column slice, projected
        part = ops.spmm_copy_u_sum(row, col, xs, cum(csz), cum(fsz), cum(ssz))
        out = ops.mp_feat_shuffle_fwd(part, recv_size, send_size, H // world)
        mine = int(fsz[rank] + csz[rank])
        volume["NFP"] = ((world - 1) * mine * 8, int(ssz.sum() - ssz[rank]) * (H // world) * 4)
        return out

    mp_step.sampler = apt_b200.MPSampler(rank, w.fanouts)

    res = {}
    for name, fn in (("NP", np_step), ("SNP", sp_step), ("NFP", mp_step)):
        ops.set_sampling(key=2026, call_id=0)
        for b in batches[:args.warmup]:
            fn(b)
        torch.cuda.synchronize()
        dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for b in batches[args.warmup:]:
            fn(b)
        e1.record()
        torch.cuda.synchronize()
        ms = torch.tensor([e0.elapsed_time(e1) / args.steps], device="cuda")
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        vol = torch.tensor(volume[name], dtype=torch.float64, device="cuda")
        dist.all_reduce(vol, op=dist.ReduceOp.MAX)
        res[name] = {"ms_per_minibatch": round(float(ms.item()), 4),
                     "id_bytes_out_per_gpu": int(vol[0].item()), "row_bytes_out_per_gpu": int(vol[1].item())}
    ops.check_status()
    if rank == 0:
        print(json.dumps({"metric": "outermost hop + first-layer exchange per strategy", "unit": "ms per mini-batch",
                          "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "data": "synthetic",
                          "config": {"workload": "stage strategies", "graph": w.name, "fanouts": list(w.fanouts),
                                     "seeds_per_gpu": w.batch, "hidden": H, "rows": "f32"},
                          "strategies": res}))
    dist.barrier()
    dist.destroy_process_group()


# ------------------------------------------------------------------------- main
PHASE = ["setup"]     # the part of the run an exception came from


def main():
    """Runs the benchmark; a failing rank prints its traceback as its last lines on stderr and a
    one-line JSON record of the error on stdout before it exits non-zero, so that the cause
    survives the launcher's own summary."""
    try:
        run()
    except BaseException as exc:   # noqa: BLE001  (SystemExit included: say why the rank left)
        if isinstance(exc, SystemExit) and exc.code in (0, None):
            raise
        import traceback

        rank = os.environ.get("RANK", "0")
        text = traceback.format_exc()
        print(json.dumps({"error": f"{type(exc).__name__}: {exc}", "phase": PHASE[0], "rank": int(rank)}), flush=True)
        sys.stderr.write(f"\n[bench.py rank {rank}] failed in phase '{PHASE[0]}':\n{text}")
        sys.stderr.flush()
        os._exit(1)      # do not wait in a collective's destructor for peers that are still running


def run():
    args = parse()
    if args.stage == "gather":
        return stage_gather(args)
    if args.stage == "shuffle":
        return stage_shuffle(args)
    if args.stage == "ops":
        return stage_ops(args)
    if args.stage == "strategies":
        return stage_strategies(args)
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world != max(args.gpus, 1) and world > 1:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}")
    if args.impl == "reference" and rank != 0:
        return  # the CPU arm runs on rank 0 alone

    torch.cuda.set_device(local_rank)
    if world > 1 and args.impl != "reference":
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    import apt_b200
    from apt_b200 import ops, synthetic
    from apt_b200._lib import lib

    ws_eff = 1 if args.impl == "reference" else world
    w = synthetic.WORKLOADS[args.workload]
    ops.init(rank if ws_eff > 1 else 0, local_rank, ws_eff, ops.nccl_get_unique_id(), ws_eff)
    t_setup = time.time()
    inst = synthetic.install(w, rank if ws_eff > 1 else 0, ws_eff)
    torch.cuda.synchronize()
    setup_s = time.time() - t_setup
    esz = inst.host_feats.element_size()
    row_bytes = w.feat_dim * esz
    config = {
        "workload": w.name, "num_nodes": w.num_nodes, "num_edges": w.num_edges, "csc_edges": inst.info["num_csc_edges"],
        "feat_dim": w.feat_dim, "feat_dtype": w.dtype, "cached_rows_per_gpu": inst.info["num_cached_rows"],
        "cache_policy": f"top {w.cache_frac:.0%} rows by in-degree", "fanout": w.fanouts, "seeds_per_gpu": w.batch,
        "strategy": "NP (outermost hop sampled at the owner, random contiguous partition)",
        "topology": "int64 CSC resident in HBM", "host_features": "pinned host memory read by the gather kernel",
        "l2": "inputs (CSC 13.7 GB, feature tables) exceed the 126 MB L2; every step touches other rows",
    }
    run_info = {"setup_s": round(setup_s, 1), "shuffle_backend": ops.STATE.shuffle_backend if ws_eff > 1 else "local"}

    if args.impl == "reference":
        cpu = CpuPath(inst)
        seeds = [b.cpu().numpy() for b in batches_of(inst.train_ids, w.batch, args.warmup + args.steps)]
        rate, dt, rows = cpu.time(seeds, warmup=args.warmup)
        line = {
            "impl": "reference", "metric": METRIC, "value": rate, "unit": UNIT, "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1000.0 / rate, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "int64 ids, " + w.dtype + " rows", "data": "synthetic",
            "config": config, "run_info": run_info,
            "cpu_baseline": {"value": rate, "unit": UNIT, "cores": cpu.cores, "kind": "port",
                             "sample": f"{args.steps} mini-batches of {w.batch} seeds on the full graph, "
                                       f"about {rows:.0f} gathered rows each, OpenMP over all host threads"},
            "e2e": {"value": rate, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        }
        print(json.dumps(line))
        return

    sampler = apt_b200.MixedNeighborSampler(rank, w.fanouts)
    total = args.warmup + args.steps
    dev_batches = batches_of(inst.train_ids, w.batch, total)
    host_batches = [b.cpu().pin_memory() for b in batches_of(inst.train_ids, w.batch, total, offset=total)]

    def step(seeds):
        sample = sampler.sample(None, seeds)
        x = ops.load_subtensor(sample[0])
        return sample, x

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def phase(name):
        PHASE[0] = name

    def reduce_max(x):
        if world == 1:
            return x
        t = torch.tensor([x], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def reduce_sum(x):
        if world == 1:
            return x
        t = torch.tensor([x], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.SUM)
        return float(t.item())

    # ---- device-resident run ------------------------------------------------
    ops.set_sampling(key=7777777, call_id=0)
    clocks = ClockSampler(local_rank)
    clocks.start()          # sampled from the warm-up on: the timed region alone can be shorter than one sample period
    # every phase that exchanges between the ranks starts behind a barrier: host-side work of different
    # length (registering the host table, stopping the clock sampler) must not eat into the wait bound
    phase("warmup")
    barrier()
    for b in dev_batches[:args.warmup]:
        step(b)
    ops.check_status()
    phase("timed")
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    torch.cuda.nvtx.range_push("apt_timed")
    ev0.record()
    for b in dev_batches[args.warmup:]:
        step(b)
    ev1.record()
    torch.cuda.nvtx.range_pop()
    barrier()
    ms = reduce_max(ev0.elapsed_time(ev1))
    graph_mode = bool(sampler._graph_ok())
    value = world * args.steps / (ms / 1000.0)
    ops.check_status()

    # ---- spread of the single steps: an event pair around each of up to 100 of the same steps
    phase("spread")
    n_spread = min(args.steps, 100)
    marks = [torch.cuda.Event(enable_timing=True) for _ in range(n_spread + 1)]
    barrier()
    marks[0].record()
    for k, b in enumerate(dev_batches[args.warmup:args.warmup + n_spread]):
        step(b)
        marks[k + 1].record()
    barrier()
    per_step = sorted(marks[k].elapsed_time(marks[k + 1]) for k in range(n_spread))
    spread = {"steps": n_spread, "median": per_step[n_spread // 2], "p10": per_step[n_spread // 10],
              "p90": per_step[min(n_spread - 1, (9 * n_spread) // 10)]}
    ops.check_status()

    # ---- the same steps once more with per-kernel CUDA events (for the roofline and the
    # launch count). Timing events cannot live inside a captured graph, so this pass
    # enqueues the kernels one by one; its own rate is reported as profiled_value.
    phase("profiled")
    ops.profile_enable(True)
    barrier()
    for b in dev_batches[:args.warmup]:
        step(b)
    for tag in STAGE_TAGS:
        t_, n_ = ctypes.c_double(), ctypes.c_int64()
        lib.apt_profile_read(tag.encode(), ctypes.byref(t_), ctypes.byref(n_))
    lib.apt_launch_count_reset()
    kept = []
    barrier()
    torch.cuda.nvtx.range_push("apt_profiled")
    ev0.record()
    for b in dev_batches[args.warmup:]:
        sample, x = step(b)
        kept.append(sample[0].clone())
    ev1.record()
    torch.cuda.nvtx.range_pop()
    barrier()
    launches = int(lib.apt_launch_count())
    ops.profile_enable(False)
    clock_info = clocks.stop()
    ms_prof = reduce_max(ev0.elapsed_time(ev1))
    ops.check_status()

    def prof(tag):
        t, n = ctypes.c_double(), ctypes.c_int64()
        lib.apt_profile_read(tag.encode(), ctypes.byref(t), ctypes.byref(n))
        return t.value, n.value

    stage_ms = {tag: prof(tag) for tag in STAGE_TAGS}
    pos_map = ops.STATE.feat.feat_pos_map
    rows_total = sum(int(k.numel()) for k in kept)
    hits_total = sum(int((pos_map[k] >= 0).sum().item()) for k in kept)
    miss_total = rows_total - hits_total
    peak, peak_kind = peaks()
    hit_ms, hit_n = stage_ms["gather_hit"]
    miss_ms, miss_n = stage_ms["gather_miss"]
    # algorithmic bytes of one launch of the hit kernel: an id and a position-map entry per requested row
    # (16 bytes), and every cached row once in and once out
    hit_bytes = (hits_total * 2 * row_bytes + rows_total * 16) / max(hit_n, 1)
    hit_gbs = hit_bytes / (hit_ms / max(hit_n, 1) * 1e-3) / 1e9 if hit_ms > 0 else 0.0
    roofline = {"kernel": "k_gather_hits (gather: decode + copy of the cache hits)", "bound": "hbm",
                "achieved": round(hit_gbs, 1), "peak": peak, "peak_kind": peak_kind, "unit": "GB/s",
                "frac": round(hit_gbs / peak, 4),
                "traffic": round(hit_bytes * HIT_DRAM_BYTES_PER_ALGORITHMIC_BYTE)
                if HIT_DRAM_BYTES_PER_ALGORITHMIC_BYTE else None,
                "traffic_source": HIT_TRAFFIC_SOURCE,
                "measured_in": "the pass that enqueues the kernels one by one with an event pair around each "
                               "(one launch over all input rows of the mini-batch; the graph replay of the headline "
                               "splits the same rows into two launches of this kernel)",
                "rows_per_launch": rows_total / max(hit_n, 1),
                "hit_rows_per_launch": hits_total / max(hit_n, 1), "us_per_launch": 1000.0 * hit_ms / max(hit_n, 1)}
    miss_bytes = miss_total * row_bytes / max(miss_n, 1)
    miss_gbs = miss_bytes / (miss_ms / max(miss_n, 1) * 1e-3) / 1e9 if miss_ms > 0 else 0.0

    # ---- measured host-link rate (pinned host -> device copy), the miss kernel's ceiling
    phase("host_link_probe")
    probe_rows = min(w.num_nodes, (1 << 30) // row_bytes)
    dst = torch.empty((probe_rows, w.feat_dim), dtype=inst.host_feats.dtype, device="cuda")
    dst.copy_(inst.host_feats[:probe_rows], non_blocking=True)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    dst.copy_(inst.host_feats[:probe_rows], non_blocking=True)
    e1.record()
    torch.cuda.synchronize()
    link_gbs = probe_rows * row_bytes / (e0.elapsed_time(e1) * 1e-3) / 1e9
    del dst
    roofline_link = {"kernel": "k_copy_miss (gather, rows from pinned host memory)", "bound": "host_link",
                     "achieved": round(miss_gbs, 2), "peak": round(link_gbs, 2),
                     "peak_kind": "pinned host->device copy of 1 GiB measured in this run", "unit": "GB/s",
                     "frac": round(miss_gbs / link_gbs, 4) if link_gbs else None,
                     "miss_rows_per_launch": miss_total / max(miss_n, 1),
                     "us_per_launch": 1000.0 * miss_ms / max(miss_n, 1)}

    # ---- end to end through host buffers --------------------------------------
    def e2e_step(host_seeds):
        seeds = host_seeds.to("cuda", non_blocking=True)
        sample, x = step(seeds)
        digest = torch.cat([x[0], x[-1]]).float().cpu()      # device -> host read of the step's result
        return digest

    phase("e2e")
    barrier()
    for b in host_batches[:args.warmup]:
        e2e_step(b)
    barrier()
    ev0.record()
    for b in host_batches[args.warmup:]:
        e2e_step(b)
    ev1.record()
    barrier()
    ms_e2e = reduce_max(ev0.elapsed_time(ev1))
    e2e = {"value": world * args.steps / (ms_e2e / 1000.0), "unit": UNIT, "ms_per_step": ms_e2e / args.steps,
           "h2d_bytes_per_step": w.batch * 8, "d2h_bytes_per_step": 2 * w.feat_dim * 4 + 64 * 4,
           "note": "seeds come from pinned host memory; a digest (first and last gathered row) and the per-hop "
                   "unique counts are read back; the gathered rows stay on the GPU for the model"}
    ops.check_status()

    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "int64 ids, " + w.dtype + " rows", "data": "synthetic", "config": config, "run_info": run_info,
        "clocks": clock_info,
        "e2e": e2e, "gpu_launches": int(reduce_sum(launches)),
        "launch_mode": "one CUDA graph replay per mini-batch" if graph_mode else
                       "kernels enqueued one by one, sizes chained on the device",
        "step_ms_spread": spread,
        "profiled_value": world * args.steps / (ms_prof / 1000.0),
        "roofline": roofline, "roofline_link": roofline_link,
        "per_step": {"gathered_rows": rows_total / args.steps, "cache_hit_rate": hits_total / max(rows_total, 1),
                     "gather_gb": rows_total / args.steps * row_bytes / 1e9,
                     "stage_ms": {k: round(v[0] / args.steps, 4) for k, v in stage_ms.items()},
                     "stage_launches": {k: v[1] / args.steps for k, v in stage_ms.items()}},
    }

    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        cpu = CpuPath(inst)
        seeds = [b.cpu().numpy() for b in batches_of(inst.train_ids, w.batch, args.cpu_batches + 1)]
        rate, dt, rows = cpu.time(seeds, warmup=1)
        line["cpu_baseline"] = {"value": rate, "unit": UNIT, "cores": cpu.cores, "kind": "port",
                                "sample": f"{args.cpu_batches} mini-batches of {w.batch} seeds on the full graph "
                                          f"({dt:.1f} s, about {rows:.0f} gathered rows each), C restatement with "
                                          "OpenMP over all host threads"}
    if rank == 0:
        print(json.dumps(line))
    synthetic.cleanup(inst)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
