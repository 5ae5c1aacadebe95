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

# Before CUDA starts: one hardware queue per stream. With the default of 8 the caller's stream shares a
# queue with one of the sampler's lane streams, and whatever the caller enqueues (here: the read-back of
# a step's result) waits behind that lane's queued mini-batches.
os.environ.setdefault("CUDA_DEVICE_MAX_CONNECTIONS", "32")

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

STAGE_TAGS = ("sample", "relabel", "bucket", "unique_sorted", "gather_classify", "gather_hit", "gather_miss",
              "p2p_push", "p2p_wait", "p2p_pull")
# DRAM bytes (read + written) per algorithmic byte of the hit kernel, from an ncu capture of that kernel
# alone at the mini-batch's size: 143 000 random rows of 512 bytes out of a 2 GB cache table moved
# 73.3 MB of DRAM reads (every row once) and 21.5 MB of DRAM writes (the rest of the 73.2 MB written was
# still in the 126 MB L2 when the kernel ended) for 147.6 MB algorithmic. Traffic grows with the rows.
HIT_DRAM_BYTES_PER_ALGORITHMIC_BYTE = (73.3 + 21.5) / 147.6
HIT_TRAFFIC_SOURCE = ("ncu dram__bytes_read.sum + dram__bytes_write.sum of k_copy_hits at 143 000 rows x 512 B "
                      "(94.8 MB per 147.6 MB algorithmic), scaled by this launch's algorithmic bytes; writes that "
                      "stay in L2 past the kernel's end are not in it")
# the pool's reference figure for a peer copy over NVLink, GB/s per direction (900 nominal); the benchmark
# also measures a copy-engine peer copy in its own run and reports fractions of all three
POOL_PEER_COPY_GBS = 770.0
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


def batches_of(inst, count, offset=0):
    """`count` consecutive seed batches of the rank (apt_b200.synthetic.seed_batches)."""
    from apt_b200 import synthetic

    return synthetic.seed_batches(inst, count, offset)


def digest_np(a):
    """Order-sensitive 64-bit digest of an integer array: sum of a[i] * (2 i + 1) modulo 2^64."""
    import numpy as np

    flat = np.ascontiguousarray(a).reshape(-1).astype(np.int64).view(np.uint64)
    with np.errstate(over="ignore"):
        k = np.arange(len(flat), dtype=np.uint64) * np.uint64(2) + np.uint64(1)
        return int((flat * k).sum(dtype=np.uint64))


def digest_torch(t):
    """The same digest on the device (int64 arithmetic wraps like uint64)."""
    flat = t.reshape(-1).to(torch.int64)
    k = torch.arange(flat.numel(), dtype=torch.int64, device=flat.device) * 2 + 1
    return int((flat * k).sum().item()) & 0xFFFFFFFFFFFFFFFF


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
        # every row is read from the host table; a table shorter than the node count repeats with its length
        self.pos_map = -(np.arange(n, dtype=np.int64) % inst.host_feats.shape[0]) - 2
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

    def inner_hops(self, seeds):
        """The local hops: returns (frontier, [(unique, relabelled) per hop, innermost first], next call id)."""
        np = self.np
        cur = np.ascontiguousarray(seeds, dtype=np.int64)
        call, layers = 0, []
        for f in reversed(self.w.fanouts[1:]):
            nbr = self._sample(cur, f, call)
            call += 1
            cur, rel = self._relabel(cur, nbr)
            layers.append((cur, rel))
        return cur, layers, call

    def bucket(self, ids, rank):
        np = self.np
        ws = len(self.min_vids) - 1
        sorted_ids, perm = np.empty_like(ids), np.empty_like(ids)
        sizes, offs = np.empty(ws, dtype=np.int64), np.empty(ws, dtype=np.int64)
        self.lib.oracle_bucket(self._p(ids), ctypes.c_int64(len(ids)), self._p(self.min_vids), ws, ctypes.c_int64(0),
                               rank, 0, ws, self._p(sorted_ids), self._p(perm), self._p(sizes), self._p(offs))
        return sorted_ids, perm, sizes, offs

    def outer_hop(self, received, call):
        """Sorted unique of what a rank received, the outermost hop on it, its relabelling."""
        np = self.np
        uniq, inv = np.empty_like(received), np.empty_like(received)
        u = self.lib.oracle_unique_sorted(self._p(received), ctypes.c_int64(len(received)), self._p(uniq), self._p(inv))
        uniq = uniq[:u].copy()
        nbr = self._sample(uniq, self.w.fanouts[0], call)
        inputs, rel = self._relabel(uniq, nbr)
        return uniq, inv, inputs, rel

    def gather(self, inputs):
        np = self.np
        out = np.empty((len(inputs), self.row_bytes), dtype=np.uint8)
        self.lib.oracle_gather(self._p(inputs), ctypes.c_int64(len(inputs)), self._p(self.pos_map), None,
                               ctypes.c_int64(self.row_bytes), self._p(self.feats), ctypes.c_int64(self.row_bytes),
                               ctypes.c_int64(0), self._p(out))
        return out

    def batch(self, seeds):
        cur, _, call = self.inner_hops(seeds)
        sorted_ids, _, _, _ = self.bucket(cur, 0)
        _, _, inputs, _ = self.outer_hop(sorted_ids, call)
        self.gather(inputs)
        return len(inputs)

    def replay(self, seeds_per_rank):
        """One NP mini-batch of every rank at once (the seed exchange is a concatenation of the
        buckets in rank order): per rank a dict of what the sampler and the gather must return."""
        np = self.np
        world = len(seeds_per_rank)
        first = [self.inner_hops(s) for s in seeds_per_rank]
        buckets = [self.bucket(first[r][0], r) for r in range(world)]
        out = []
        for r in range(world):
            parts = []
            for q in range(world):
                sorted_q, _, sizes_q, offs_q = buckets[q]
                lo = int(offs_q[r] - sizes_q[r])
                parts.append(sorted_q[lo:int(offs_q[r])])
            received = np.concatenate(parts) if parts else np.empty(0, dtype=np.int64)
            uniq, inv, inputs, rel = self.outer_hop(received, first[r][2])
            out.append({
                "input_nodes": inputs, "outer_rel": rel, "inner_rel": [l[1] for l in first[r][1]],
                "perm": buckets[r][1], "inverse_idx": inv[:len(received)],
                "recv_counts": np.array([len(p) for p in parts], dtype=np.int64), "bucket_offsets": buckets[r][3],
                "rows_digest": digest_np(self.gather(inputs).view(np.int32)),
            })
        return out

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
            for tag in (b"gather_hit", b"gather_miss", b"gather_classify"):
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
    for tag in ("gather_hit", "gather_miss", "gather_classify"):
        t, k = ctypes.c_double(), ctypes.c_int64()
        lib.apt_profile_read(tag.encode(), ctypes.byref(t), ctypes.byref(k))
        res[tag] = (t.value, k.value)
    hit_ms, hit_n = res["gather_hit"]
    # the hit kernel reads the 8-byte position of every requested row and moves every cached row once in
    # and once out
    hit_bytes = (args.rows - n_miss) * 2 * row_bytes + args.rows * 8
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
        "roofline": {"kernel": "k_copy_hits", "bound": "hbm", "achieved": round(gbs, 1), "peak": peak,
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
            out[tag] = round(1e3 * t_.value / max(k_.value, 1), 2)      # milliseconds -> us per launch
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
    # the form the samplers use: the sampling kernel enters the ids it draws into the table itself
    timed("sample + relabel in the sampler's fused form (67 584 seeds x 15)",
          lambda s: ops._sample_relabel_enqueue(s, f, None, ops.STATE.word(0)), S * (32 + 16 * f) + 16 * items,
          lambda: seed_pool[0], tags=("sample", "relabel"))
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


# ------------------------------------------------------------------ parity check
def parity_check(inst, w, rank, world, cpu_path, barrier):
    """One NP mini-batch of the benchmarked configuration on every rank, compared on rank 0 with the
    CPU restatement (oracle/) replaying all ranks at once: input nodes, every block's relabelled
    neighbours, permutation, inverse index, exchange counts bit for bit, and the gathered rows through
    a 64-bit digest. Then the feature shuffle forward and backward with rows that are a function of the
    node id, so that each rank can tell locally what has to arrive where. Raises on any mismatch."""
    import numpy as np

    import apt_b200
    from apt_b200 import ops

    seeds = batches_of(inst, 1, offset=7)[0]
    ops.set_sampling(key=7777777, call_id=0)
    smp = apt_b200.MixedNeighborSampler(rank, w.fanouts, chained=True, use_graph=False)
    barrier()
    input_nodes, _, blocks, perm, send_off, recv_off, inv = smp.sample(None, seeds)
    x = ops.load_subtensor(input_nodes)
    ops.check_status()
    counts = torch.cat([send_off[:1], send_off[1:] - send_off[:-1]])
    mine = {
        "seeds": seeds.cpu().numpy(), "input_nodes": digest_torch(input_nodes), "n_in": int(input_nodes.numel()),
        "outer_rel": digest_torch(blocks[0].coo_row), "inner_rel": [digest_torch(b.coo_row) for b in blocks[:0:-1]],
        "perm": digest_torch(perm), "inverse_idx": digest_torch(inv), "recv_counts": counts.numpy(),
        "bucket_offsets": recv_off.numpy(), "rows_digest": digest_torch(x.view(torch.int32)),
    }
    if world > 1:
        every = [None] * world
        dist.all_gather_object(every, mine)
    else:
        every = [mine]
    verdict = ["ok"]
    if rank == 0:
        want = cpu_path.replay([e["seeds"] for e in every])
        for r in range(world):
            g, o = every[r], want[r]
            checks = {
                "input_nodes": g["n_in"] == len(o["input_nodes"]) and g["input_nodes"] == digest_np(o["input_nodes"]),
                "outer_rel": g["outer_rel"] == digest_np(o["outer_rel"]),
                "inner_rel": g["inner_rel"] == [digest_np(a) for a in o["inner_rel"]],
                "perm": g["perm"] == digest_np(o["perm"]), "inverse_idx": g["inverse_idx"] == digest_np(o["inverse_idx"]),
                "recv_counts": np.array_equal(g["recv_counts"], o["recv_counts"]),
                "bucket_offsets": np.array_equal(g["bucket_offsets"], o["bucket_offsets"]),
                "rows": g["rows_digest"] == o["rows_digest"],
            }
            bad = [k for k, ok in checks.items() if not ok]
            if bad:
                verdict[0] = f"rank {r}: {', '.join(bad)} differ from the CPU restatement"
                break
    if world > 1:
        dist.broadcast_object_list(verdict, src=0)
    if verdict[0] != "ok":
        raise RuntimeError("parity check of the NP mini-batch failed: " + verdict[0])

    # feature shuffle: the owner's rows are f(node id); forward, each rank gets f(its frontier) in its
    # own order; backward, what arrives at an owner for the k-th id it received is f(that id)
    def rows_of(ids, width=16):
        c = torch.arange(width, device=ids.device, dtype=torch.int64)
        return ((ids.view(-1, 1) * 31 + c * 7) % 65521).to(torch.float32)

    frontier = blocks[1].src_ids if len(blocks) > 1 else seeds
    owned = blocks[0].src_ids[:blocks[0].num_dst]                  # sorted unique of what this rank received
    y = ops.feat_shuffle(ops.rows_gather(rows_of(owned), inv), send_off, recv_off, perm, 16, 1)
    ok_f = torch.equal(y, rows_of(frontier))
    gb = ops.feat_shuffle(rows_of(frontier), recv_off, send_off, perm, 16, 0)
    ok_b = torch.equal(gb, rows_of(owned[inv]))
    ops.check_status()
    flags = torch.tensor([int(ok_f), int(ok_b)], device="cuda")
    if world > 1:
        dist.all_reduce(flags, op=dist.ReduceOp.MIN)
    if not bool(flags[0]) or not bool(flags[1]):
        raise RuntimeError(f"parity check of the feature shuffle failed (forward ok: {bool(flags[0])}, "
                           f"backward ok: {bool(flags[1])})")
    return {"np_minibatch": "ok", "feat_shuffle": "ok", "ranks": world,
            "against": "CPU restatement (oracle/) replaying all ranks; blocks, permutation, inverse index and "
                       "exchange counts bit for bit, gathered rows by 64-bit digest; feature shuffle forward "
                       "and backward in closed form", "input_rows_rank0": every[0]["n_in"]}


# ------------------------------------------------------------- shuffle record
def shuffle_record(args, rank, world, barrier):
    """The NPC feature shuffle alone, inside the benchmark run: forward shuffle of the stress shape
    (495 616 rows of 2 KiB fp16 per GPU) and of the papers-shaped NP run (67 584 rows of 1 KiB fp32),
    through the peer-to-peer path and through the library all-to-all, next to a peer copy measured in
    the same run (every rank copies 256 MiB into its right neighbour's inbox with cudaMemcpyAsync)."""
    import apt_b200  # noqa: F401
    from apt_b200 import ops
    from apt_b200.exchange import NcclExchange, P2PExchange

    st = ops.STATE
    keep = st.exchange
    n_ids = 1 << 24
    saved_mv = (st.shuffle_min_vids, st._min_vids_host, st.shuffle_id_offset)
    ops.register_min_vids(torch.tensor([n_ids * r // world for r in range(world)] + [n_ids]))
    shapes = {"c4_stress_2KiB_f16": (495_616, 1024, torch.float16), "c1_np_1KiB_f32": (67_584, 256, torch.float32)}
    need = max(int(2.0 * rows / world * dim * torch.empty(0, dtype=dt).element_size()) + (8 << 20)
               for rows, dim, dt in shapes.values())
    p2p = keep if isinstance(keep, P2PExchange) and keep.region_bytes >= need else P2PExchange(st, need)
    nccl = NcclExchange(st)
    # a second inbox with two landing buffers for the direct-placement leg (opt-in path of the library)
    rows_c4, dim_c4, dt_c4 = shapes["c4_stress_2KiB_f16"]
    landing_mb = int(1.08 * rows_c4 * dim_c4 * torch.empty(0, dtype=dt_c4).element_size()) >> 20
    env_keep = {k: os.environ.get(k) for k in ("APT_P2P_DIRECT", "APT_P2P_DIRECT_SLOTS", "APT_P2P_LANDING_MB")}
    os.environ.update(APT_P2P_DIRECT="1", APT_P2P_DIRECT_SLOTS="2", APT_P2P_LANDING_MB=str(landing_mb))
    try:
        direct = P2PExchange(st, need)
    finally:
        for k, v in env_keep.items():
            if v is None:
                os.environ.pop(k, None)
            else:
                os.environ[k] = v
    if not direct.direct:
        direct.close()
        direct = None
    steps, warm = 10, 3
    g = torch.Generator(device="cuda").manual_seed(100 + rank)
    out = {}

    def timed(fn):
        for _ in range(warm):
            fn()
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        ms = torch.tensor([e0.elapsed_time(e1) / steps], device="cuda")
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item())

    # peer copy: the denominator, measured here and now
    copy_bytes = min(256 << 20, p2p.region_bytes)
    right = (rank + 1) % world
    copy_ms = timed(lambda: p2p.probe_peer_copy(right, copy_bytes))
    peer_gbs = copy_bytes / (copy_ms * 1e-3) / 1e9
    for name, (rows, dim, dt) in shapes.items():
        row_bytes = dim * torch.empty(0, dtype=dt).element_size()
        st.exchange = p2p
        ids = torch.randint(0, n_ids, (rows,), generator=g, device="cuda")
        recv_ids, perm, send_off, recv_off = ops.shuffle_seeds(ids)
        x = torch.randn((recv_ids.numel(), dim), generator=g, device="cuda").to(dt)
        counts = torch.cat([send_off[:1], send_off[1:] - send_off[:-1]])
        remote = torch.tensor([float((int(counts.sum()) - int(counts[rank])) * row_bytes)], device="cuda")
        dist.all_reduce(remote, op=dist.ReduceOp.MAX)
        rec = {"rows_per_gpu": rows, "row_bytes": row_bytes, "remote_bytes_per_gpu": float(remote.item())}
        for label, ex in (("p2p", p2p), ("nccl", nccl)):
            st.exchange = ex
            ms = timed(lambda: ops.feat_shuffle(x, send_off, recv_off, perm, dim, 1))
            rec[f"{label}_ms"] = round(ms, 4)
            rec[f"{label}_gbs"] = round(float(remote.item()) / (ms * 1e-3) / 1e9, 1)
        rec["frac_of_measured_peer_copy"] = round(rec["p2p_gbs"] / peer_gbs, 4)
        rec["frac_of_900_nominal"] = round(rec["p2p_gbs"] / 900.0, 4)
        rec["frac_of_770_pool_reference"] = round(rec["p2p_gbs"] / POOL_PEER_COPY_GBS, 4)
        if direct is not None and name == "c4_stress_2KiB_f16":
            # the opt-in path of large shuffles: the askers send the final slot of every row first, the owners
            # store the rows there, no pull pass; the result is a view of a landing buffer of the inbox
            st.exchange = direct
            try:
                ms = timed(lambda: ops.feat_shuffle(x, send_off, recv_off, perm, dim, 1))
                ops.check_status()
                gbs = float(remote.item()) / (ms * 1e-3) / 1e9
                rec["direct_placement"] = {"ms": round(ms, 4), "gbs": round(gbs, 1),
                                           "frac_of_measured_peer_copy": round(gbs / peer_gbs, 4),
                                           "frac_of_900_nominal": round(gbs / 900.0, 4),
                                           "frac_of_770_pool_reference": round(gbs / POOL_PEER_COPY_GBS, 4)}
            except RuntimeError as exc:       # an extra leg: its failure is reported, the line stands
                rec["direct_placement"] = {"error": str(exc)[:200]}
        out[name] = rec
        del x, ids, recv_ids
    st.exchange = keep
    if direct is not None:
        barrier()
        direct.close()
    ops.check_status()
    if p2p is not keep:
        barrier()
        p2p.close()
    st.shuffle_min_vids, st._min_vids_host, st.shuffle_id_offset = saved_mv
    st.generation += 1
    head = out["c4_stress_2KiB_f16"]
    return {"gbs": head["p2p_gbs"], "nccl_gbs": head["nccl_gbs"],
            "frac_of_measured_peer_copy": head["frac_of_measured_peer_copy"],
            "frac_of_900_nominal": head["frac_of_900_nominal"],
            "frac_of_770_pool_reference": head["frac_of_770_pool_reference"],
            "direct_placement": head.get("direct_placement"),
            "peer_copy_gbs": round(peer_gbs, 1),
            "peer_copy": f"{copy_bytes >> 20} MiB cudaMemcpyAsync into the right neighbour's inbox, all ranks at once "
                         f"(a copy-engine copy; the pool's reference figure for a peer copy is {POOL_PEER_COPY_GBS:.0f} "
                         "GB/s per direction)",
            "unit": "GB/s per GPU and direction, remote rows only", "direction": "forward (rows back to the askers)",
            "path": "direct placement" if getattr(p2p, "direct", False) else "push + wait + pull", "shapes": out}


# ------------------------------------------------------------- SNP with a GAT model
def run_snp_gat(args, inst, w, rank, world, config, run_info, barrier, reduce_max, phase):
    """One step = one mini-batch per GPU of the SNP strategy with a GAT first layer
    (python/npc/sampler.py:215-238, python/npc/model/gatconv.py:89-135): inner hops local, the
    outermost hop's unique sources travel to their owners, which gather and project their rows
    (bf16, 4 heads x 64; the projection is a library GEMM), the feature shuffle brings the projected
    rows back in unique-source order, and the fused edge kernel (u_add_v scores, leaky_relu, edge
    softmax, weighted sum) produces the layer output of the destination nodes."""
    import apt_b200
    from apt_b200 import ops

    heads, head_dim = 4, 64
    width = heads * head_dim
    gen = torch.Generator(device="cuda").manual_seed(77)
    weight = (torch.randn((w.feat_dim, width), generator=gen, device="cuda") / w.feat_dim ** 0.5).bfloat16()
    attn_l = torch.randn((1, heads, head_dim), generator=gen, device="cuda").bfloat16()
    attn_r = torch.randn((1, heads, head_dim), generator=gen, device="cuda").bfloat16()
    sampler = apt_b200.SPGATSampler(rank, w.fanouts)
    run_info["sampler_lanes"] = sampler.lanes
    total = args.warmup + args.steps
    dev_batches = batches_of(inst, total)
    marks = {}

    def model_side(sample, mark=lambda name: None):
        """Everything behind the sampler for one mini-batch: gather (already enqueued by the sampler when it
        prefetches), projection, feature shuffle, attention block."""
        in_nodes, _, blocks, perm, send_off, recv_off = sample
        x = ops.load_subtensor(in_nodes)
        mark("gather")
        b0 = blocks[0]
        proj = x.bfloat16() @ weight
        mark("project")
        ft_src = ops.feat_shuffle(proj[b0.num_dst:].contiguous(), send_off, recv_off, perm, width, 1)
        mark("feat_shuffle")
        ft_dst = proj[:b0.num_dst]
        el = (ft_src.view(-1, heads, head_dim) * attn_l).sum(-1)
        er = (ft_dst.view(-1, heads, head_dim) * attn_r).sum(-1)
        out = ops.gat_edge_softmax_sum(b0.coo_row, b0.coo_col, ft_src.view(-1, heads, head_dim), el.contiguous(),
                                       er.contiguous(), b0.num_dst)
        mark("gat_block")
        return out, (in_nodes, blocks, perm, send_off, recv_off, x)

    def step(seeds, timed=None):
        def mark(name):
            if timed is not None:
                ev = torch.cuda.Event(enable_timing=True)
                ev.record()
                timed.append((name, ev))

        mark("start")
        sample = sampler.sample(None, seeds)
        mark("sample")
        return model_side(sample, mark)

    def run_steps(batches):
        # the sampler's pipelined iterator: mini-batch k + 1 is on the GPU while k is read back and consumed
        for sample in sampler.sample_iter(None, batches):
            model_side(sample)

    phase("parity_check")
    barrier()
    ops.set_sampling(key=7777777, call_id=0)
    _, (in_nodes, blocks, perm, send_off, recv_off, x) = step(dev_batches[0])
    b0 = blocks[0]
    raw_back = ops.feat_shuffle(x[b0.num_dst:].contiguous(), send_off, recv_off, perm, w.feat_dim, 1)
    ok = torch.equal(raw_back, ops.load_subtensor(b0.src_ids)) and \
        torch.equal(in_nodes[:b0.num_dst], blocks[1].src_ids if len(blocks) > 1 else dev_batches[0])
    flag = torch.tensor([int(ok)], device="cuda")
    if world > 1:
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    if not bool(flag[0]):
        raise RuntimeError("parity check of the SNP-GAT mini-batch failed: the rows that came back are not the rows "
                           "of the block's unique sources")
    ops.check_status()

    # set-up, like the installation of the graph: every buffer set of the sampler's iterator is built (one
    # eager run and one graph capture each) before the warm-up steps, whatever their number
    phase("prime")
    barrier()
    run_steps([dev_batches[0]] * sampler._in_flight())
    phase("warmup")
    clocks = ClockSampler(int(os.environ.get("LOCAL_RANK", "0")))
    clocks.start()
    barrier()
    run_steps(dev_batches[:args.warmup])
    ops.check_status()
    phase("timed")
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    ev0.record()
    run_steps(dev_batches[args.warmup:])
    ev1.record()
    barrier()
    ms = reduce_max(ev0.elapsed_time(ev1))
    graph_mode = bool(sampler._graph_ok())
    phase("profiled")
    ops.profile_enable(True)       # the sampler then enqueues its kernels one by one (no graph), like the NP bench
    sums, n_prof = {}, min(args.steps, 20)
    rows_in = edges = 0
    barrier()
    for b in dev_batches[args.warmup:args.warmup + n_prof]:
        timed = []
        _, (in_nodes, blocks, *_rest) = step(b, timed)
        torch.cuda.synchronize()
        for (_, e_a), (name, e_b) in zip(timed[:-1], timed[1:]):
            sums[name] = sums.get(name, 0.0) + e_a.elapsed_time(e_b)
        rows_in += int(in_nodes.numel())
        edges += int(blocks[0].coo_row.numel())
    ops.profile_enable(False)
    clock_info = clocks.stop()
    ops.check_status()
    line = {
        "metric": METRIC, "value": world * args.steps / (ms / 1000.0), "unit": UNIT, "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "int64 ids, f32 rows gathered, bf16 projected rows",
        "data": "synthetic", "config": dict(config, strategy="SNP with a GAT first layer (4 heads x 64, bf16)"),
        "run_info": run_info, "clocks": clock_info,
        "launch_mode": "sampler and gather: one CUDA graph replay per mini-batch, the next one enqueued before the "
                       "previous one is read back; projection, feature shuffle and attention block enqueued one by one"
                       if graph_mode else "kernels enqueued one by one",
        "parity_check": {"snp_gat_minibatch": "ok", "ranks": world,
                         "against": "closed form: rows shuffled back equal the gathered rows of the block's sources"},
        "per_step": {"input_rows": rows_in / n_prof, "outer_block_edges": edges / n_prof,
                     "stage_ms": {k: round(v / n_prof, 4) for k, v in sums.items()}},
    }
    return line


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
    cache_gb = inst.info["num_cached_rows"] * row_bytes / 1e9
    config = {
        "workload": w.name, "num_nodes": w.num_nodes, "num_edges": w.num_edges, "csc_edges": inst.info["num_csc_edges"],
        "feat_dim": w.feat_dim, "feat_dtype": w.dtype, "cached_rows_per_gpu": inst.info["num_cached_rows"],
        "cache_policy": (f"top {w.cache_frac:.0%} rows by in-degree" if w.cache_bytes is None else
                         f"{cache_gb:.1f} GB of rows by falling in-degree"),
        "fanout": w.fanouts, "seeds_per_gpu": w.batch,
        "seeds": "uniform over a seeded training split" if w.seed_dist == "uniform" else
                 f"Zipf({w.zipf_s}) over the rank by in-degree, distinct within a batch",
        "strategy": "NP (outermost hop sampled at the owner)",
        "partition": "random contiguous ranges" if w.partition == "random" else
                     f"{inst.info['intra_partition_edge_share']:.1%} of the edges inside a part over "
                     f"{inst.info['partition_parts_measured']} contiguous parts (measured); ids as generated "
                     f"({w.locality:.0%} of the R-MAT edges planted inside {w.locality_blocks} blocks): "
                     f"{inst.info['intra_partition_edge_share_as_generated']:.1%}, after a breadth-first "
                     f"renumbering from a seeded root: {inst.info['intra_partition_edge_share_bfs']:.1%}; "
                     f"installed: {inst.info['partition_used']}",
        "topology": "int64 CSC resident in HBM", "host_features": "pinned host memory read by the gather kernel",
        "l2": f"inputs (CSC {inst.info['num_csc_edges'] * 8 / 1e9:.1f} GB, feature tables) exceed the 126 MB L2; "
              "every step touches other rows",
    }
    if "host_rows" in inst.info:
        config["host_table"] = (f"{inst.info['host_rows']} rows: the full table of {w.num_nodes * row_bytes / 1e9:.0f} GB "
                                "does not fit host memory, features repeat with that period; bytes per row, miss "
                                "rate and access pattern are those of the full table")
    run_info = {"setup_s": round(setup_s, 1), "shuffle_backend": ops.STATE.shuffle_backend if ws_eff > 1 else "local"}

    if args.impl == "reference":
        cpu = CpuPath(inst)
        seeds = [b.cpu().numpy() for b in batches_of(inst, args.warmup + args.steps)]
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
    run_info["sampler_lanes"] = sampler.lanes
    total = args.warmup + args.steps
    dev_batches = batches_of(inst, total)
    host_batches = [b.cpu().pin_memory() for b in batches_of(inst, total, offset=total)]

    def step(seeds):
        sample = sampler.sample(None, seeds)
        x = ops.load_subtensor(sample[0])
        return sample, x

    def run_steps(batches, after=None):
        """One step per batch through the sampler's pipelined iterator (the next mini-batch is already
        on the GPU while the previous one is read back, like a prefetching loader around the
        reference's sampler) and load_subtensor; after(k, sample, rows) runs behind every step."""
        for k, sample in enumerate(sampler.sample_iter(None, batches)):
            x = ops.load_subtensor(sample[0])
            if after is not None:
                after(k, sample, x)

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

    if w.system == "SP":
        line = run_snp_gat(args, inst, w, rank, world, config, run_info, barrier, reduce_max, phase)
        if rank == 0:
            print(json.dumps(line))
        synthetic.cleanup(inst)
        if world > 1:
            dist.destroy_process_group()
        return

    # ---- device-resident run ------------------------------------------------
    ops.set_sampling(key=7777777, call_id=0)
    clocks = ClockSampler(local_rank)
    clocks.start()          # sampled from the warm-up on: the timed region alone can be shorter than one sample period
    # every phase that exchanges between the ranks starts behind a barrier: host-side work of different
    # length (registering the host table, stopping the clock sampler) must not eat into the wait bound
    # set-up, like the installation of the graph: every buffer set of the sampler's iterator is built (one
    # eager run and one graph capture each) before the warm-up steps, whatever their number
    phase("prime")
    barrier()
    run_steps([dev_batches[0]] * sampler._in_flight())
    phase("warmup")
    barrier()
    run_steps(dev_batches[:args.warmup])
    ops.check_status()
    phase("timed")
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    torch.cuda.nvtx.range_push("apt_timed")
    ev0.record()
    run_steps(dev_batches[args.warmup:])
    ev1.record()
    torch.cuda.nvtx.range_pop()
    barrier()
    ms = reduce_max(ev0.elapsed_time(ev1))
    graph_mode = bool(sampler._graph_ok())
    value = world * args.steps / (ms / 1000.0)
    ops.check_status()

    # ---- spread: an event behind every step of up to 100 of the same steps. With several mini-batches in
    # flight the steps complete in bursts, so the spread is taken over windows of 10 steps (ms per step).
    phase("spread")
    n_spread = min(args.steps, 100)
    window = 10 if sampler.lanes > 1 and n_spread >= 30 else 1
    marks = [torch.cuda.Event(enable_timing=True) for _ in range(n_spread + 1)]
    barrier()
    marks[0].record()
    run_steps(dev_batches[args.warmup:args.warmup + n_spread], after=lambda k, sample, x: marks[k + 1].record())
    barrier()
    n_win = n_spread // window
    per_step = sorted(marks[k * window].elapsed_time(marks[(k + 1) * window]) / window for k in range(n_win))
    spread = {"steps": n_spread, "window": window, "median": per_step[n_win // 2], "p10": per_step[n_win // 10],
              "p90": per_step[min(n_win - 1, (9 * n_win) // 10)]}
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
    # what an event pair around one launch costs by itself: the same gather with a device-side row count of
    # zero (same grids, every block returns at once), bracketed by the same events
    ops.profile_enable(True)
    zero_rows = torch.zeros(1, dtype=torch.int64, device="cuda")
    for _ in range(20):
        ops._gather_enqueue(kept[-1], zero_rows)
    torch.cuda.synchronize()
    ops.profile_enable(False)
    empty_ms, empty_n = prof("gather_hit")
    for tag in ("gather_classify", "gather_miss"):
        prof(tag)
    bracket_us = 1000.0 * empty_ms / max(empty_n, 1)
    pos_map = ops.STATE.feat.feat_pos_map
    rows_total = sum(int(k.numel()) for k in kept)
    hits_total = sum(int((pos_map[k] >= 0).sum().item()) for k in kept)
    miss_total = rows_total - hits_total
    peak, peak_kind = peaks()
    hit_ms, hit_n = stage_ms["gather_hit"]
    miss_ms, miss_n = stage_ms["gather_miss"]
    # algorithmic bytes of one launch of the hit kernel: each cached row once in and once out, plus the
    # 8-byte position of every requested row
    hit_bytes = (hits_total * 2 * row_bytes + rows_total * 8) / max(hit_n, 1)
    hit_gbs = hit_bytes / (hit_ms / max(hit_n, 1) * 1e-3) / 1e9 if hit_ms > 0 else 0.0
    roofline = {"kernel": "k_copy_hits (gather, cache hits)", "bound": "hbm",
                "achieved": round(hit_gbs, 1), "peak": peak, "peak_kind": peak_kind, "unit": "GB/s",
                "frac": round(hit_gbs / peak, 4),
                # the capture holds for launches of its kind: 512-byte rows, a batch that fits the L2 twice over
                "traffic": round(hit_bytes * HIT_DRAM_BYTES_PER_ALGORITHMIC_BYTE)
                if row_bytes == 512 and hit_bytes < 4e8 else None,
                "traffic_source": HIT_TRAFFIC_SOURCE if row_bytes == 512 and hit_bytes < 4e8 else
                "not captured for launches of this size",
                "measured_in": "the pass that enqueues the kernels one by one with an event pair around each",
                "rows_per_launch": rows_total / max(hit_n, 1),
                "hit_rows_per_launch": hits_total / max(hit_n, 1), "us_per_launch": 1000.0 * hit_ms / max(hit_n, 1),
                "us_per_empty_launch": round(bracket_us, 2),
                "empty_launch": "the same launch with a device-side row count of zero between the same event pair: "
                                "what the events and the launch cost without any row moved"}
    miss_bytes = miss_total * row_bytes / max(miss_n, 1)
    miss_gbs = miss_bytes / (miss_ms / max(miss_n, 1) * 1e-3) / 1e9 if miss_ms > 0 else 0.0

    # ---- measured host-link rate (pinned host -> device copy), the miss kernel's ceiling
    phase("host_link_probe")
    probe_rows = min(int(inst.host_feats.shape[0]), (1 << 30) // row_bytes)
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
    # Every step copies its seeds from pinned host memory and reads a digest of the gathered rows (and,
    # inside the sampler, the 2 KiB block of counts) back into pinned host memory. The digest of step k
    # is looked at once step k + 1 has been enqueued, so that the read does not drain the GPU.
    row_dtype = ops.STATE.feat.dev_feats.dtype
    digests = [torch.empty(w.feat_dim, dtype=row_dtype).pin_memory() for _ in range(2)]
    digest_done = [torch.cuda.Event(), torch.cuda.Event()]
    checksum = [0.0]

    def e2e_run(host_seed_batches):
        def read_back(k, sample, x):
            digests[k % 2].copy_(x[-1], non_blocking=True)     # the last gathered row: device -> host
            digest_done[k % 2].record()
            if k >= 1:
                digest_done[(k - 1) % 2].synchronize()
                checksum[0] += float(digests[(k - 1) % 2][0])
        n = len(host_seed_batches)
        run_steps(host_seed_batches, after=read_back)     # the iterator copies each batch host -> device itself
        if n:
            digest_done[(n - 1) % 2].synchronize()
            checksum[0] += float(digests[(n - 1) % 2][0])

    phase("e2e")
    barrier()
    e2e_run(host_batches[:args.warmup])
    barrier()
    ev0.record()
    e2e_run(host_batches[args.warmup:])
    ev1.record()
    barrier()
    ms_e2e = reduce_max(ev0.elapsed_time(ev1))
    e2e = {"value": world * args.steps / (ms_e2e / 1000.0), "unit": UNIT, "ms_per_step": ms_e2e / args.steps,
           "h2d_bytes_per_step": w.batch * 8, "d2h_bytes_per_step": row_bytes + 8 * ops.STATE.NUM_WORDS,
           "note": "seeds come from pinned host memory; the last gathered row and the block of device-side counts "
                   "(per-hop unique counts, exchange sizes, status flags) are read back into pinned host memory "
                   "every step; the gathered rows stay on the GPU for the model"}
    ops.check_status()

    # ---- parity of this very configuration, outside every timed region ----------------------
    phase("parity_check")
    cpu_path = None
    if rank == 0:
        cpu_path = CpuPath(inst)
    parity = parity_check(inst, w, rank, world, cpu_path, barrier)

    # ---- the feature shuffle alone (N >= 2): GB/s per GPU and direction over NVLink ----------
    shuffle = None
    if world > 1:
        phase("shuffle")
        barrier()
        shuffle = shuffle_record(args, rank, world, barrier)

    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "int64 ids, " + w.dtype + " rows", "data": "synthetic", "config": config, "run_info": run_info,
        "clocks": clock_info,
        "e2e": e2e, "gpu_launches": int(reduce_sum(launches)),
        "launch_mode": (f"one CUDA graph replay per mini-batch, {sampler.buffer_sets()} mini-batches in flight on "
                        f"{min(sampler.lanes, sampler.buffer_sets())} streams with scratch of their own"
                        if sampler.lanes > 1 else
                        "one CUDA graph replay per mini-batch, the next one enqueued before the previous one is "
                        "read back") if graph_mode else
                       "kernels enqueued one by one, sizes chained on the device",
        "step_ms_spread": spread,
        "profiled_value": world * args.steps / (ms_prof / 1000.0),
        "roofline": roofline, "roofline_link": roofline_link, "parity_check": parity,
        "per_step": {"gathered_rows": rows_total / args.steps, "cache_hit_rate": hits_total / max(rows_total, 1),
                     "gather_gb": rows_total / args.steps * row_bytes / 1e9,
                     "stage_ms": {k: round(v[0] / args.steps, 4) for k, v in stage_ms.items()},
                     "stage_launches": {k: v[1] / args.steps for k, v in stage_ms.items()}},
    }

    if shuffle is not None:
        line["shuffle"] = shuffle
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        phase("cpu_baseline")
        cpu = cpu_path
        seeds = [b.cpu().numpy() for b in batches_of(inst, args.cpu_batches + 1)]
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
