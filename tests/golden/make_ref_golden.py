"""Records what the REFERENCE ITSELF computes, as golden vectors for the tests.

Runs on a machine with one CUDA GPU, after ``python oracle/build_ref.py`` has
compiled the reference's own sources into oracle/_ref/libnpc_ref.so:

    python tests/golden/make_ref_golden.py [output directory]

It loads that library with ``torch.classes.load_library`` and calls the
reference's operators exactly as python/npc/ops.py does (``torch.ops.npc.*``),
on seeded, well-formed inputs only (every node has an in-neighbour, every id
has a feature row, no collective is involved), and writes the inputs and the
reference's outputs to ``ref_*.npz``. tests/test_ref_golden.py (CPU: the
oracle; GPU: the CUDA path) compares with these files; nothing else reads them.

Operators recorded (reference file:line of the entry point):
  relabel_csc            src/relabel.cc:9-15, src/cuda/relabel.cu:175-185
  load_subtensor         src/load_subtensor.cc:19-40 (+ cache_feats_shared, src/cache_feats.cc:14-61)
  cpu_load_subtensor     src/load_subtensor.cc:10-17
  local_sample_one_layer src/sampling.cc:13-17 (+ mix_cache_graphs, src/cache_graphs.cc:12-49); its
                         random stream is cuRAND's, so the tests use it for the layout, the
                         edge-membership invariant and the uniformity of the chosen slots only
  spmm_copy_u_sum / spmm_copy_e_sum / spmm_u_mul_e_sum   src/spmm.cc:9-42
  sddmm_u_add_v / sddmm_u_mul_v                          src/sddmm.cc:9-31
shuffle_seeds and feat_shuffle need an NCCL communicator and stay out; they are
pinned by the closed-form cases of the reference's own tests instead.
"""
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import oracle as orc  # noqa: E402  (only its seeded R-MAT graph generator is used here)

REF_LIB = os.path.join(ROOT, "oracle", "_ref", "libnpc_ref.so")


def table(rows, dim, salt):
    """Feature rows made of exactly representable values, a function of (row, column)."""
    r = np.arange(rows, dtype=np.int64)[:, None]
    c = np.arange(dim, dtype=np.int64)[None, :]
    return (((r * 131 + c * 7 + salt) % 2001) - 1000).astype(np.float32) / 8.0


def cuda(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def main():
    out_dir = sys.argv[1] if len(sys.argv) > 1 else os.path.join(ROOT, "tests", "golden")
    os.makedirs(out_dir, exist_ok=True)
    assert torch.cuda.is_available(), "needs a CUDA device"
    torch.cuda.set_device(0)
    torch.classes.load_library(REF_LIB)
    npc = torch.ops.npc
    rng = np.random.default_rng(20261125)

    # ---------------------------------------------------------------- relabel
    cases = {}
    shapes = {"tiny": (16, 4, 40), "small": (256, 10, 900), "dup_seeds": (300, 5, 500), "large": (2048, 5, 6000)}
    for name, (S, f, id_range) in shapes.items():
        if name == "dup_seeds":
            seeds = rng.integers(0, id_range, S).astype(np.int64)       # repeats among the seeds
        else:
            seeds = rng.permutation(id_range)[:S].astype(np.int64) * 3 + 1
        nbrs = rng.integers(0, id_range * 3 + 1, S * f).astype(np.int64)
        uniq, rel = npc.relabel_csc(cuda(seeds), cuda(nbrs))
        torch.cuda.synchronize()
        cases[f"{name}_seeds"], cases[f"{name}_neighbors"] = seeds, nbrs
        cases[f"{name}_unique"], cases[f"{name}_relabeled"] = uniq.cpu().numpy(), rel.cpu().numpy()
    np.savez_compressed(os.path.join(out_dir, "ref_relabel.npz"), names=np.array(list(shapes)), **cases)

    # ---------------------------------------------------- graph for sampling
    n, scale, graph_seed, num_edges = 2000, 11, 5, 30000
    src, dst = orc.rmat_edges(graph_seed, 0, num_edges, scale, n)
    indptr, indices = orc.csc_from_edges(src, dst, n)                   # one self loop per node: deg >= 1
    deg = np.diff(indptr)
    cached_nodes = np.argsort(-deg, kind="stable")[:200].astype(np.int64)
    dip = np.concatenate([[0], np.cumsum(deg[cached_nodes])]).astype(np.int64)
    dix = np.concatenate([indices[indptr[v]:indptr[v + 1]] for v in cached_nodes]).astype(np.int64)
    gi, gx = torch.from_numpy(indptr).pin_memory(), torch.from_numpy(indices).pin_memory()
    npc.mix_cache_graphs(len(cached_nodes), torch.from_numpy(cached_nodes), cuda(dip), cuda(dix), gi, gx)
    seeds = rng.integers(0, n, 4096).astype(np.int64)                   # repeats on purpose
    fanout = 10
    res = npc.local_sample_one_layer(cuda(seeds), fanout)
    torch.cuda.synchronize()
    np.savez_compressed(os.path.join(out_dir, "ref_sample.npz"), num_nodes=n, scale=scale, graph_seed=graph_seed,
                        num_edges=num_edges, cached_nodes=cached_nodes, seeds=seeds, fanout=fanout,
                        out_seeds=res[0].cpu().numpy(), neighbors=res[1].cpu().numpy())

    # ------------------------------------------------------------- gather
    g = {}
    for name, (feat_dim, rank_dim, offset, n_nodes, n_cached, n_ids) in {
            "full_width": (64, 64, 0, 3000, 700, 400),
            "column_slice": (96, 32, 32, 1500, 300, 300),      # NFP: each rank holds a slice of the columns
            "all_cached": (32, 32, 0, 500, 500, 200),
            "none_cached": (32, 32, 0, 500, 0, 200)}.items():
        host = table(n_nodes, feat_dim, 11)
        order = rng.permutation(n_nodes).astype(np.int64)
        cached_idx = np.sort(order[:n_cached])
        local_idx = np.arange(n_nodes, dtype=np.int64)
        dev = np.ascontiguousarray(host[cached_idx][:, offset:offset + rank_dim]) if n_cached else \
            np.zeros((0, rank_dim), dtype=np.float32)
        host_t = torch.from_numpy(host).pin_memory()
        npc.cache_feats_shared(n_nodes, host_t, cuda(dev), torch.from_numpy(cached_idx), torch.from_numpy(local_idx),
                               offset)
        ids = rng.integers(0, n_nodes, n_ids).astype(np.int64)
        out = npc.load_subtensor(cuda(ids))
        torch.cuda.synchronize()
        cpu_out = npc.cpu_load_subtensor(torch.from_numpy(ids))
        g[f"{name}_shape"] = np.array([feat_dim, rank_dim, offset, n_nodes, n_cached], dtype=np.int64)
        g[f"{name}_cached_idx"], g[f"{name}_ids"] = cached_idx, ids
        g[f"{name}_out"] = out.cpu().numpy()
        g[f"{name}_cpu_out"] = cpu_out.numpy()
    np.savez_compressed(os.path.join(out_dir, "ref_gather.npz"), salt=11,
                        names=np.array(["full_width", "column_slice", "all_cached", "none_cached"]), **g)

    # -------------------------------------------------------- SpMM / SDDMM
    s = {}
    for name, (segs, D, exact) in {"one_segment_exact": (1, 16, True), "three_segments_exact": (3, 8, True),
                                   "one_segment_normal": (1, 16, False), "gat_scores": (1, 4, False)}.items():
        n_src = [int(x) for x in rng.integers(40, 80, segs)]
        n_dst = [int(x) for x in rng.integers(20, 40, segs)]
        n_e = [int(x) for x in rng.integers(150, 300, segs)]
        row = np.concatenate([rng.integers(0, a, e) for a, e in zip(n_src, n_e)]).astype(np.int64)
        col = np.concatenate([np.sort(rng.integers(0, b, e)) for b, e in zip(n_dst, n_e)]).astype(np.int64)
        coo_off = np.concatenate([[0], np.cumsum(n_e)]).astype(np.int64)
        in_off = np.concatenate([[0], np.cumsum(n_src)]).astype(np.int64)
        out_off = np.concatenate([[0], np.cumsum(n_dst)]).astype(np.int64)
        E = int(coo_off[-1])
        if exact:   # multiples of 1/8: every partial sum is exact in fp32, so any summation order agrees
            mk = lambda *shape: (rng.integers(-32, 33, shape).astype(np.float32) / 8.0)
        else:
            mk = lambda *shape: rng.standard_normal(shape).astype(np.float32)
        x_src, x_dst, x_edge = mk(int(in_off[-1]), D), mk(int(out_off[-1]), D), mk(E, D)
        t = [cuda(a) for a in (row, col, coo_off, in_off, out_off)]
        r_, c_, co, io, oo = t
        torch.cuda.synchronize()
        outs = {
            "copy_u": npc.spmm_copy_u_sum(r_, c_, cuda(x_src), co, io, oo),
            "copy_e": npc.spmm_copy_e_sum(r_, c_, cuda(x_edge), co, oo),
            "u_mul_e": npc.spmm_u_mul_e_sum(r_, c_, cuda(x_src), cuda(x_edge), co, io, oo),
            "u_add_v": npc.sddmm_u_add_v(r_, c_, cuda(x_src), cuda(x_dst), co, io, oo),
            "u_mul_v": npc.sddmm_u_mul_v(r_, c_, cuda(x_src), cuda(x_dst), co, io, oo),
        }
        torch.cuda.synchronize()   # the reference launches these on the legacy default stream without a sync
        for k, v in (("row", row), ("col", col), ("coo_off", coo_off), ("in_off", in_off), ("out_off", out_off),
                     ("x_src", x_src), ("x_dst", x_dst), ("x_edge", x_edge)):
            s[f"{name}_{k}"] = v
        for k, v in outs.items():
            s[f"{name}_{k}"] = v.cpu().numpy()
        s[f"{name}_exact"] = np.array(int(exact))
    np.savez_compressed(os.path.join(out_dir, "ref_spmm_sddmm.npz"),
                        names=np.array(["one_segment_exact", "three_segments_exact", "one_segment_normal",
                                        "gat_scores"]), **s)
    sizes = {f: os.path.getsize(os.path.join(out_dir, f)) for f in sorted(os.listdir(out_dir)) if f.startswith("ref_")}
    print("reference golden vectors written:", sizes)


if __name__ == "__main__":
    main()
