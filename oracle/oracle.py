"""CPU oracle of APT's mini-batch data path (numpy). TEST INFRASTRUCTURE ONLY.

This file restates, on the CPU, what the reference (kaihaoma/APT) computes on
the path sampling -> relabel -> seed shuffle -> feature gather -> feature
shuffle -> SpMM/SDDMM, one function per reference function, each citing the
reference file:line it follows. Only the tests, the smoke check and the
benchmark's CPU-baseline leg may import it; the product path never does.

Pinning status (what ties this restatement to the reference itself)
  * relabelling, the feature gather (GPU and CPU flavour), SpMM (copy_u, copy_e and the
    reference's u_mul_e kernel, which adds) and SDDMM are pinned by outputs of the
    REFERENCE'S OWN CODE: oracle/build_ref.py compiles the reference's sources unmodified
    (oracle/_ref/libnpc_ref.so), tests/golden/make_ref_golden.py runs its operators on a
    B200 on seeded inputs and records inputs and outputs in tests/golden/ref_*.npz, and
    tests/test_ref_golden.py holds this file (and the CUDA path) to them: bit for bit for
    the integer and byte work and for exactly summable SpMM inputs, within the error
    bound of fp32 summation otherwise.
  * all-to-all / all-gather / all-broadcast / all-reduce and the seed shuffle are pinned
    by the closed-form cases of the reference's own tests (tests/test_alltoall.cc,
    test_allgather.cc, test_allbroadcast.cc, test_allreduce.cc, test_shuffle_seeds.cc),
    replayed over N in-process ranks in tests/test_oracle_golden.py (they need an NCCL
    communicator in the reference, so they are not re-run through the compiled library).
  * sampling is pinned in everything but the random stream: dense [S, fanout] layout,
    the edge-membership invariant, with-replacement semantics and the uniformity of the
    chosen slots are checked against the reference's recorded output
    (tests/golden/ref_sample.npz); the draws themselves differ by design (next paragraph).
  * the operators the reference leaves to DGL (edge softmax, the GAT layer) and the SNP /
    NFP samplers have no reference-side vectors: they follow the cited lines and the public
    operator definitions, cross-checked against an independent C restatement
    (oracle/apt_oracle.c) and torch autograd; for them parity is unpinned.

Deliberate, documented differences from the reference:
  * the sampler draws from Philox4x32-10 (counter-based) instead of cuRAND
    XORWOW re-seeded per call (src/cuda/npc_kernel.cu:258-261); the use of the
    draw, `indices[start + draw % deg]`, is the reference's (:279-282);
  * a zero-degree seed yields its own id (the reference leaves the row
    uninitialised, npc_kernel.cu:277);
  * feat_pos_map == -1 yields a zero row (the reference reads out of bounds,
    npc_kernel.cu:196-205);
  * within-bucket order of the seed shuffle is the stable one (the reference's
    is atomic-order dependent, npc_kernel.cu:345-346).
"""
import numpy as np

U32 = np.uint32
U64 = np.uint64
I64 = np.int64

FEAT_NOT_EXIST = -1  # src/utils.h:20


def encode_id(i):
    """ENCODE_ID, src/utils.h:17: i -> -(i) - 2 (its own inverse)."""
    return -(i) - 2


# --------------------------------------------------------------------- Philox
_M0 = U64(0xD2511F53)
_M1 = U64(0xCD9E8D57)
_W0 = 0x9E3779B9
_W1 = 0xBB67AE85
_MASK = U64(0xFFFFFFFF)


def philox4x32_10(c0, c1, c2, c3, k0, k1):
    """Philox4x32-10 (Salmon et al., SC'11). Inputs broadcast; returns four
    uint32 arrays. Known answers: counter 0/key 0 -> 6627e8d5 e169c58d bc57ac4c
    9b00dbd8; all-ones -> 408f276d 41c83b0e a20bc7c6 6d5451fd."""
    c0, c1, c2, c3 = [np.asarray(x, dtype=U64) & _MASK for x in np.broadcast_arrays(c0, c1, c2, c3)]
    k0 = int(k0) & 0xFFFFFFFF
    k1 = int(k1) & 0xFFFFFFFF
    for _ in range(10):
        p0 = _M0 * c0
        p1 = _M1 * c2
        n0 = (p1 >> U64(32)) ^ c1 ^ U64(k0)
        n1 = p1 & _MASK
        n2 = (p0 >> U64(32)) ^ c3 ^ U64(k1)
        n3 = p0 & _MASK
        c0, c1, c2, c3 = n0, n1, n2, n3
        k0 = (k0 + _W0) & 0xFFFFFFFF
        k1 = (k1 + _W1) & 0xFFFFFFFF
    return c0.astype(U32), c1.astype(U32), c2.astype(U32), c3.astype(U32)


def draw_words(j, i, call_id, key):
    """The sampler's draw(j, i): word (i & 3) of Philox with counter
    (j lo, j hi, i >> 2, call_id) and the 64-bit key split lo/hi."""
    j = np.asarray(j, dtype=U64)
    i = np.asarray(i, dtype=U64)
    j, i = np.broadcast_arrays(j, i)
    w = philox4x32_10(j & _MASK, j >> U64(32), i >> U64(2), call_id, key & 0xFFFFFFFF, (key >> 32) & 0xFFFFFFFF)
    sel = (i & U64(3)).astype(np.int64)
    return np.choose(sel, w)


# ------------------------------------------------------------------- topology
def build_adj_pos_map(num_total_nodes, cached_node_idx):
    """MixCacheGraphs, src/cache_graphs.cc:36-43: every node points at its row
    of the global CSC (encoded), cached nodes at their compact row."""
    m = encode_id(np.arange(num_total_nodes, dtype=I64))
    m[np.asarray(cached_node_idx, dtype=I64)] = np.arange(len(cached_node_idx), dtype=I64)
    return m


def sample_csc_fanout(seeds, fanout, adj_pos_map, dev_indptr, dev_indices, uva_indptr, uva_indices,
                      key, call_id, replace=True):
    """LocalSampleNeighbors / _CSRRowWiseSampleReplaceKernel,
    src/cuda/npc_kernel.cu:248-316: row lookup through adj_pos_map (:263-271),
    deg from the indptr pair (:272-276), out[j*fanout+i] = indices[start +
    draw % deg] (:277-283). replace=False is the optional Floyd selection."""
    seeds = np.asarray(seeds, dtype=I64)
    S = len(seeds)
    out = np.empty(S * fanout, dtype=I64)
    if S == 0:
        return out
    if adj_pos_map is None:
        pos = encode_id(seeds)
    else:
        pos = np.asarray(adj_pos_map, dtype=I64)[seeds]
    on_dev = pos >= 0
    row = np.where(on_dev, pos, encode_id(pos))
    start = np.empty(S, dtype=I64)
    deg = np.empty(S, dtype=I64)
    for mask, indptr in ((on_dev, dev_indptr), (~on_dev, uva_indptr)):
        if mask.any():
            ip = np.asarray(indptr, dtype=I64)
            start[mask] = ip[row[mask]]
            deg[mask] = ip[row[mask] + 1] - start[mask]
    jj = np.repeat(np.arange(S, dtype=I64), fanout)
    ii = np.tile(np.arange(fanout, dtype=I64), S)
    words = draw_words(jj, ii, call_id, key).astype(I64)
    degr = np.repeat(deg, fanout)
    slot = np.where(degr > 0, words % np.maximum(degr, 1), 0)
    if not replace:
        slot = slot.reshape(S, fanout)
        words2 = words.reshape(S, fanout)
        for j in range(S):
            d = int(deg[j])
            if d <= 0:
                continue
            if d <= fanout:
                slot[j, :d] = np.arange(d)
            else:
                picks = []
                for i in range(fanout):
                    t = d - fanout + i
                    r = int(words2[j, i]) % (t + 1)
                    picks.append(t if r in picks else r)
                slot[j, :] = picks
        slot = slot.reshape(-1)
    edge = np.repeat(start, fanout) + slot
    dev_r = np.repeat(on_dev, fanout)
    zero = degr <= 0
    res = np.repeat(seeds, fanout).copy()
    for mask, indices in ((dev_r & ~zero, dev_indices), (~dev_r & ~zero, uva_indices)):
        if mask.any():
            res[mask] = np.asarray(indices, dtype=I64)[edge[mask]]
    return res


# -------------------------------------------------------------------- relabel
def relabel_csc(seeds, neighbors):
    """TensorRelabelCSC, src/cuda/relabel.cu:175-185: total = cat(seeds,
    neighbors) (:177); Unique keeps each id at the position of its first
    occurrence, compacted in order (:89-147); Relabel maps every neighbour to
    that position (:153-173). Returns (all_unique, relabeled_neighbors)."""
    seeds = np.asarray(seeds, dtype=I64)
    neighbors = np.asarray(neighbors, dtype=I64)
    total = np.concatenate([seeds, neighbors])
    if len(total) == 0:
        return total, neighbors.copy()
    uniq_sorted, first_idx, inverse = np.unique(total, return_index=True, return_inverse=True)
    order = np.argsort(first_idx, kind="stable")       # sorted-unique slot -> rank by first occurrence
    new_id_of_sorted = np.empty(len(order), dtype=I64)
    new_id_of_sorted[order] = np.arange(len(order), dtype=I64)
    all_unique = uniq_sorted[order]
    relabeled = new_id_of_sorted[inverse.reshape(-1)[len(seeds):]]
    return all_unique, relabeled


# ------------------------------------------------------------- seed shuffle
def owner_of(ids, min_vids, world_size, shuffle_id_offset=0, rank=0, node_beg=0, node_end=None):
    """_CountDeviceVerticesKernel, src/cuda/npc_kernel.cu:335-342."""
    ids = np.asarray(ids, dtype=I64)
    mv = np.asarray(min_vids, dtype=I64)
    if node_end is None:
        node_end = world_size
    d = np.full(ids.shape, shuffle_id_offset, dtype=I64)
    for r in range(shuffle_id_offset + 1, world_size):
        # the while loop advances only while every earlier boundary also held
        d = np.where((d == r - 1) & (mv[r] <= ids), r, d)
    d = np.where((d < node_beg) | (d >= node_end), rank, d)
    return d


def bucket_by_owner(ids, min_vids, world_size, shuffle_id_offset=0, rank=0, node_beg=0, node_end=None):
    """ClusterAndPermute, src/cuda/npc_kernel.cu:434-470 (+ _PermuteKernel
    :367-382): returns (bucket_size, bucket_offset (inclusive), sorted_idx,
    permutation) with sorted_idx[permutation[i]] == ids[i]; stable order."""
    ids = np.asarray(ids, dtype=I64)
    own = owner_of(ids, min_vids, world_size, shuffle_id_offset, rank, node_beg, node_end)
    order = np.argsort(own, kind="stable")
    perm = np.empty(len(ids), dtype=I64)
    perm[order] = np.arange(len(ids), dtype=I64)
    sizes = np.bincount(own, minlength=world_size).astype(I64)
    return sizes, np.cumsum(sizes), ids[order], perm


def alltoall(inputs, send_offsets, recv_offsets, expand=1):
    """_AlltoAll over N in-process ranks, src/ops/collective.cc:223-250: rank s
    sends rows [send_offsets[s][r-1], send_offsets[s][r]) * expand to rank r,
    which stores them at [recv_offsets[r][s-1], recv_offsets[r][s]) * expand.
    Offsets are inclusive cumulative counts."""
    n = len(inputs)
    outs = []
    for r in range(n):
        total = int(recv_offsets[r][-1]) * expand if len(recv_offsets[r]) else 0
        outs.append(np.zeros(total, dtype=np.asarray(inputs[r]).dtype))
    for s in range(n):
        src = np.asarray(inputs[s]).reshape(-1)
        so = np.concatenate([[0], np.asarray(send_offsets[s], dtype=I64)])
        for r in range(n):
            ro = np.concatenate([[0], np.asarray(recv_offsets[r], dtype=I64)])
            cnt = so[r + 1] - so[r]
            assert cnt == ro[s + 1] - ro[s], "send/recv size mismatch (the reference would hang)"
            outs[r][ro[s] * expand:(ro[s] + cnt) * expand] = src[so[r] * expand:(so[r] + cnt) * expand]
    return outs


def allgather(inputs):
    """AllGather, src/ops/collective.cc:19-36: concatenation in rank order."""
    cat = np.concatenate([np.asarray(x).reshape(-1) for x in inputs])
    return [cat.copy() for _ in inputs]


def allbroadcast(inputs):
    """_AllBroadcast, src/ops/collective.cc:318-339: every rank receives the
    concatenation of all ranks' (variable-length) inputs."""
    return allgather(inputs)


def allreduce_scatter_v(inputs, sizes):
    """_AllReduce, src/ops/collective.cc:404-422: one ncclReduce per root; root
    r receives the sum over ranks of their slice [off[r], off[r]+sizes[r])."""
    off = np.concatenate([[0], np.cumsum(sizes)])
    return [sum(np.asarray(x)[off[r]:off[r + 1]] for x in inputs) for r in range(len(inputs))]


def shuffle_seeds(seeds_per_rank, min_vids, node_size=None):
    """ShuffleSeeds, src/sampling.cc:159-193, for all ranks at once. Per rank:
    (recv_frontier, permutation, recv_offset, dev_offset)."""
    n = len(seeds_per_rank)
    node_size = n if node_size is None else node_size
    parts = []
    for r in range(n):
        beg = r - r % node_size
        parts.append(bucket_by_owner(seeds_per_rank[r], min_vids, n, 0, r, beg, beg + node_size))
    sizes = np.stack([p[0] for p in parts])            # sizes[s][r]: s sends to r
    recv_offsets = [np.cumsum(sizes[:, r]) for r in range(n)]
    recv = alltoall([p[2] for p in parts], [p[1] for p in parts], recv_offsets)
    return [(recv[r], parts[r][3], recv_offsets[r], parts[r][1]) for r in range(n)]


def unique_sorted(ids):
    """torch::_unique2(sorted=true, return_inverse=true), src/sampling.cc:58-59."""
    u, inv = np.unique(np.asarray(ids, dtype=I64), return_inverse=True)
    return u, inv.reshape(-1).astype(I64)


def np_sample_and_shuffle(seeds_per_rank, fanout, min_vids, graph, key, call_id):
    """NPSampleAndShuffle, src/sampling.cc:52-69, for all ranks at once.
    `graph` = (adj_pos_map, dev_indptr, dev_indices, uva_indptr, uva_indices).
    Per rank: [unique_frontier, neighbors, permutation, recv_offset,
    dev_offset, inverse_idx]."""
    out = []
    for recv, perm, recv_off, dev_off in shuffle_seeds(seeds_per_rank, min_vids):
        uniq, inv = unique_sorted(recv)
        nbr = sample_csc_fanout(uniq, fanout, *graph, key=key, call_id=call_id)
        out.append([uniq, nbr, perm, recv_off, dev_off, inv])
    return out


# --------------------------------------------------------------------- gather
def build_feat_pos_maps(num_total_nodes, cached_idx, localnode_idx):
    """CacheFeatsShared, src/cache_feats.cc:45-55: returns (feat_pos_map,
    cpu_feat_pos_map). Host row i of node localnode_idx[i] is ENCODE_ID(i);
    cached node cached_idx[i] is i; everything else FEAT_NOT_EXIST."""
    m = np.full(num_total_nodes, FEAT_NOT_EXIST, dtype=I64)
    m[np.asarray(localnode_idx, dtype=I64)] = encode_id(np.arange(len(localnode_idx), dtype=I64))
    cpu = m.copy()
    m[np.asarray(cached_idx, dtype=I64)] = np.arange(len(cached_idx), dtype=I64)
    return m, cpu


def load_subtensor(node_id, feat_pos_map, dev_feats, uva_feats, feat_dim_offset=0):
    """LoadSubtensor / gather kernel, src/load_subtensor.cc:19-40 and
    src/cuda/npc_kernel.cu:187-224: p < -1 -> host row ENCODE_ID(p), columns
    [offset, offset + rank_feat_dim); p >= 0 -> device-cache row p."""
    node_id = np.asarray(node_id, dtype=I64)
    d = dev_feats.shape[1]
    out = np.zeros((len(node_id), d), dtype=dev_feats.dtype)
    p = np.asarray(feat_pos_map, dtype=I64)[node_id]
    hit = p >= 0
    miss = p < -1
    out[hit] = dev_feats[p[hit]]
    out[miss] = uva_feats[encode_id(p[miss]), feat_dim_offset:feat_dim_offset + d]
    return out


def cpu_load_subtensor(node_id, cpu_feat_pos_map, uva_feats):
    """CPULoadSubtensor, src/load_subtensor.cc:10-17 (the reference's own CPU
    code): uva_feats.index_select(0, ENCODE_ID(cpu_feat_pos_map[node_id]))."""
    pos = encode_id(np.asarray(cpu_feat_pos_map, dtype=I64)[np.asarray(node_id, dtype=I64)])
    return uva_feats[pos]


# ------------------------------------------------------------- feature shuffle
def feat_shuffle(inputs, send_offsets, recv_offsets, permutations, feat_dim, fwd):
    """FeatShuffle, src/feat_shuffle.cc:9-30, for all ranks at once.
    fwd: out = alltoall(flatten(in))[permutation]; bwd: scatter rows by
    permutation (index_select_backward, :13-16), then alltoall."""
    n = len(inputs)
    if fwd:
        flat = [np.asarray(x).reshape(-1) for x in inputs]
    else:
        flat = []
        for r in range(n):
            x = np.asarray(inputs[r])
            tmp = np.zeros_like(x)
            np.add.at(tmp, np.asarray(permutations[r], dtype=I64), x)
            flat.append(tmp.reshape(-1))
    outs = alltoall(flat, send_offsets, recv_offsets, expand=feat_dim)
    outs = [o.reshape(-1, feat_dim) for o in outs]
    if fwd:
        outs = [outs[r][np.asarray(permutations[r], dtype=I64)] for r in range(n)]
    return outs


# -------------------------------------------------------------- SpMM / SDDMM
def _segments(coo_offset, num_edges):
    coo_offset = np.asarray(coo_offset, dtype=I64)
    # cub::UpperBound(coo_off, len, e) - 1, src/cuda/spmm.cu:20
    return np.searchsorted(coo_offset, np.arange(num_edges, dtype=I64), side="right") - 1


def spmm_sum(op, row, col, inp, edata, coo_offset, input_offset, output_offset, acc=np.float64):
    """CopyUSumKernel / CopyESumKernel / UMulESumKernel, src/cuda/spmm.cu:7-83.
    op: 'copy_u', 'copy_e', 'u_mul_e', or 'u_add_e' (what the reference's
    UMulESum kernel computes, :78). Accumulates in `acc`, returns that dtype."""
    row = np.asarray(row, dtype=I64)
    col = np.asarray(col, dtype=I64)
    E = len(row)
    seg = _segments(coo_offset, E)
    n_out = int(np.asarray(output_offset)[-1])
    ref = inp if inp is not None else edata
    D = ref.shape[1]
    out = np.zeros((n_out, D), dtype=acc)
    if E == 0:
        return out
    dst = np.asarray(output_offset, dtype=I64)[seg] + col
    if op != "copy_e":
        src = np.asarray(input_offset, dtype=I64)[seg] + row
        val = inp[src].astype(acc)
    if op == "copy_e":
        val = edata.astype(acc)
    elif op in ("u_mul_e", "u_add_e"):
        e = edata.astype(acc)
        if e.shape[1] != D:
            e = np.repeat(e, D // e.shape[1], axis=1)
        val = val * e if op == "u_mul_e" else val + e
    np.add.at(out, dst, val)
    return out


def sddmm(op, row, col, lhs, rhs, coo_offset, lhs_offset, rhs_offset, acc=np.float64):
    """UAddVKernel / UMulVKernel, src/cuda/sddmm.cu:7-59: out[e] =
    lhs[lhs_off[k]+row[e]] (+|*) rhs[rhs_off[k]+col[e]]."""
    row = np.asarray(row, dtype=I64)
    col = np.asarray(col, dtype=I64)
    seg = _segments(coo_offset, len(row))
    a = lhs[np.asarray(lhs_offset, dtype=I64)[seg] + row].astype(acc)
    b = rhs[np.asarray(rhs_offset, dtype=I64)[seg] + col].astype(acc)
    return a + b if op == "u_add_v" else a * b


def gat_edge_softmax_sum(row, col, ft, el, er, num_dst, negative_slope=0.2):
    """The DGL calls of the reference's SNP-GAT layer, python/npc/model/gatconv.py:113-124,
    restated from the public operator definitions (DGL itself is not available, so
    this stage is parity-unpinned): e = leaky_relu(el[src] + er[dst]) (fn.u_add_v +
    LeakyReLU), a = softmax of e over the incoming edges of each dst per head
    (dgl.ops.edge_softmax), out[dst] = sum_e a * ft[src] (fn.u_mul_e + fn.sum).
    ft [Ns, H, D], el [Ns, H], er [Nd, H]. Returns (out [Nd, H, D], a [E, H]) in fp64."""
    row = np.asarray(row, dtype=I64)
    col = np.asarray(col, dtype=I64)
    ft = np.asarray(ft, dtype=np.float64)
    el = np.asarray(el, dtype=np.float64).reshape(ft.shape[0], -1)
    er = np.asarray(er, dtype=np.float64).reshape(num_dst, -1)
    s = el[row] + er[col]
    s = np.where(s > 0, s, s * negative_slope)
    m = np.full((num_dst, s.shape[1]), -np.inf)
    np.maximum.at(m, col, s)
    ex = np.exp(s - m[col])
    den = np.zeros((num_dst, s.shape[1]))
    np.add.at(den, col, ex)
    a = ex / den[col]
    out = np.zeros((num_dst,) + ft.shape[1:])
    np.add.at(out, col, a[:, :, None] * ft[row])
    return out, a


def gat_edge_softmax_sum_backward(row, col, ft, el, er, grad_out, num_dst, negative_slope=0.2):
    """Gradients of gat_edge_softmax_sum (the chain DGL's autograd runs for
    python/npc/model/gatconv.py:113-124) in float64: with s = el[row] + er[col],
    a = edge_softmax(leaky_relu(s)), out[col] += a * ft[row]:
      grad_ft[row] += a * grad_out[col];   grad_a = <grad_out[col], ft[row]> per head;
      grad_z = a * (grad_a - sum over the destination's edges of a * grad_a);
      grad_s = grad_z * (1 if s > 0 else slope); grad_el[row] += grad_s; grad_er[col] += grad_s.
    Returns (grad_ft, grad_el, grad_er, a, grad_s)."""
    row = np.asarray(row, dtype=I64)
    col = np.asarray(col, dtype=I64)
    ft = np.asarray(ft, dtype=np.float64)
    el = np.asarray(el, dtype=np.float64)
    er = np.asarray(er, dtype=np.float64)
    go = np.asarray(grad_out, dtype=np.float64)
    _, a = gat_edge_softmax_sum(row, col, ft, el, er, num_dst, negative_slope)
    s = el[row] + er[col]
    grad_ft = np.zeros_like(ft)
    np.add.at(grad_ft, row, a[:, :, None] * go[col])
    grad_a = (go[col] * ft[row]).sum(-1)
    t = np.zeros((num_dst, a.shape[1]))
    np.add.at(t, col, a * grad_a)
    grad_s = a * (grad_a - t[col]) * np.where(s > 0, 1.0, negative_slope)
    grad_el = np.zeros_like(el)
    np.add.at(grad_el, row, grad_s)
    grad_er = np.zeros_like(er)
    np.add.at(grad_er, col, grad_s)
    return grad_ft, grad_el, grad_er, a, grad_s


def sp_gat_sample(seeds_per_rank, fanout, min_vids, graph, key, call_id):
    """Outermost hop of the SNP-GAT sampler, python/npc/sampler.py:215-238, for all
    ranks at once: local sampling, sorted unique of the neighbours as block sources,
    shuffle of those ids to their owners (SPSampleShuffleSrc, src/sampling.cc:151-157).
    Per rank: dict(neighbors, unique_neigh, arange_src, shuffled, perm, send_offset,
    recv_offset, input_nodes)."""
    res = []
    uniq = []
    for seeds in seeds_per_rank:
        nbr = sample_csc_fanout(seeds, fanout, *graph, key=key, call_id=call_id)
        u, inv = unique_sorted(nbr)
        uniq.append(u)
        res.append(dict(neighbors=nbr, unique_neigh=u, arange_src=inv))
    shuffled = shuffle_seeds(uniq, min_vids)
    for r, (recv, perm, recv_off, dev_off) in enumerate(shuffled):
        res[r].update(shuffled=recv, perm=perm, send_offset=recv_off, recv_offset=dev_off,
                      input_nodes=np.concatenate([np.asarray(seeds_per_rank[r], dtype=I64), recv]))
    return res


# --------------------------------------- SNP with virtual nodes (SAGE / GCN)
def src_to_vir(src, fanout, num_dst, min_vids, world_size, shuffle_id_offset=0, rank=0, node_beg=0, node_end=None):
    """MapSrctoVir, src/cuda/npc_kernel.cu:71-117 (SrcToVir, src/sampling.cc:19-34):
    neighbour i of destination i // fanout becomes owner * num_dst + i // fanout."""
    src = np.asarray(src, dtype=I64)
    own = owner_of(src, min_vids, world_size, shuffle_id_offset, rank, node_beg, node_end)
    return own * I64(num_dst) + np.arange(len(src), dtype=I64) // I64(fanout)


def srcdst_to_vir(dst, src, fanout, min_vids, world_size, shuffle_id_offset=0, rank=0, node_beg=0, node_end=None):
    """MapSrcDsttoVir, src/cuda/npc_kernel.cu:15-70 (SrcDsttoVir, src/sampling.cc:36-50):
    destinations first (owner * num_dst + index), then the neighbours shifted by
    world_size * num_dst."""
    dst = np.asarray(dst, dtype=I64)
    src = np.asarray(src, dtype=I64)
    num_dst = I64(len(dst))
    od = owner_of(dst, min_vids, world_size, shuffle_id_offset, rank, node_beg, node_end)
    os_ = owner_of(src, min_vids, world_size, shuffle_id_offset, rank, node_beg, node_end)
    return np.concatenate([od * num_dst + np.arange(len(dst), dtype=I64),
                           os_ * num_dst + I64(world_size) * num_dst + np.arange(len(src), dtype=I64) // I64(fanout)])


def vir_send_offset(world_size, base, sorted_nodes, unique_nodes, with_dst):
    """GetVirSendOffset / GetVirSendOffsetWithDst, src/cuda/npc_kernel.cu:119-183:
    lower bounds of base * i in the sorted virtual ids (i in [0, k ws], k = 2 with
    destinations else 1), then in their sorted unique values for the last ws of
    those search values."""
    k = 2 if with_dst else 1
    vals = I64(base) * np.arange(k * world_size + 1, dtype=I64)
    first = np.searchsorted(np.asarray(sorted_nodes, dtype=I64), vals, side="left")
    second = np.searchsorted(np.asarray(unique_nodes, dtype=I64), vals[(k - 1) * world_size + 1:], side="left")
    return np.concatenate([first, second]).astype(I64)


def vir_send_sizes(world_size, base, sorted_nodes, unique_nodes, with_dst):
    """The size vector SPSampleAndShuffle derives from those offsets,
    src/sampling.cc:86-106 with the permutations of src/core.cc:80-95: per
    receiver r, (ids, unique virtual nodes) or (destinations, ids, unique
    virtual nodes) bound for r."""
    k = 3 if with_dst else 2
    off = vir_send_offset(world_size, base, sorted_nodes, unique_nodes, with_dst)
    fir_uni = off[(k - 1) * world_size + 1]
    sizes = np.diff(off)
    sizes[(k - 1) * world_size] = fir_uni
    permute = np.array([i * world_size + r for r in range(world_size) for i in range(k)], dtype=I64)
    return sizes[permute].astype(I64)


def sp_sample_and_shuffle(num_seeds_pr, send_frontier_pr, sorted_pr, unique_pr, with_dst, num_total_nodes):
    """SPSampleAndShuffle, src/sampling.cc:71-149, with the size exchange
    (AlltoAll of k values per peer) and SPSampleAlltoAll(WithDst),
    src/ops/collective.cc:38-133, for all ranks at once. Per rank: dict(recv_dst
    (with destinations only), vir_src, ori_src, send_sizes, recv_sizes)."""
    ws = len(send_frontier_pr)
    k = 3 if with_dst else 2
    send_sizes = [vir_send_sizes(ws, num_seeds_pr[r], sorted_pr[r], unique_pr[r], with_dst) for r in range(ws)]
    recv_sizes = [np.concatenate([send_sizes[q][k * r:k * r + k] for q in range(ws)]) for r in range(ws)]
    out = []
    for r in range(ws):
        parts_dst, parts_src = [], []
        for q in range(ws):
            sz = send_sizes[q]
            fr = np.asarray(send_frontier_pr[q], dtype=I64)
            if with_dst:
                d0 = int(sz[0:3 * r:3].sum())
                parts_dst.append(fr[d0:d0 + int(sz[3 * r])])
                s0 = int(sz[0::3].sum()) + int(sz[1:3 * r:3].sum())
                parts_src.append(fr[s0:s0 + int(sz[3 * r + 1])])
            else:
                s0 = int(sz[0:2 * r:2].sum())
                parts_src.append(fr[s0:s0 + int(sz[2 * r])])
        recv_src = np.concatenate(parts_src) if parts_src else np.zeros(0, dtype=I64)
        res = dict(vir_src=recv_src // I64(num_total_nodes), ori_src=recv_src % I64(num_total_nodes),
                   send_sizes=send_sizes[r], recv_sizes=recv_sizes[r])
        if with_dst:
            res["recv_dst"] = np.concatenate(parts_dst)
        out.append(res)
    return out


def sp_feat_shuffle(inputs_pr, send_sizes_pr, recv_sizes_pr, with_dst):
    """SPFeatShuffle, src/feat_shuffle.cc:32-52 over SPFeatureAlltoAll(WithDst),
    src/ops/collective.cc:135-212: rank r sends send_sizes[k q + k - 1] rows to q
    (after, with destinations, send_sizes[3 q] destination rows to every q) and
    receives in sender order. Returns the received rows per rank."""
    ws = len(inputs_pr)
    k = 3 if with_dst else 2
    out = []
    for r in range(ws):
        parts = []
        passes = (0, 2) if with_dst else (1,)
        for i in passes:
            for q in range(ws):
                sz = np.asarray(send_sizes_pr[q], dtype=I64)
                start = 0
                for j in passes:
                    if j == i:
                        break
                    start += int(sz[j::k].sum())
                start += int(sz[i:k * r:k].sum()) if r > 0 else 0
                n = int(sz[k * r + i])
                assert n == int(recv_sizes_pr[r][k * q + i])
                parts.append(np.asarray(inputs_pr[q])[start:start + n])
        out.append(np.concatenate(parts) if parts else np.zeros((0,) + np.asarray(inputs_pr[r]).shape[1:]))
    return out


def sp_virtual_sample(seeds_pr, fanout, min_vids, graph, key, call_id, num_total_nodes, with_dst=False,
                      model="SAGE", sp_base=10_000_000):
    """Outermost hop of the SNP sampler for SAGE / GCN, python/npc/sampler.py:240-330,
    for all ranks at once. Neighbours are mapped to virtual nodes (owner, local
    destination), sorted (the reference's torch.sort leaves ties in any order; the
    stable order is taken here), block1 joins the unique virtual nodes to the local
    destinations, the packed triples (sender, destination index, neighbour id) go to
    the neighbour's owner, and block2 there joins the received neighbours to the
    received virtual nodes. Per rank a dict of every intermediate."""
    ws = len(seeds_pr)
    pre = []
    for r, seeds in enumerate(seeds_pr):
        seeds = np.asarray(seeds, dtype=I64)
        num_dst = len(seeds)
        nbr = sample_csc_fanout(seeds, fanout, *graph, key=key, call_id=call_id)
        if with_dst:
            m = srcdst_to_vir(seeds, nbr, fanout, min_vids, ws, rank=r)
            perm = np.argsort(m, kind="stable")
            sorted_all = m[perm]
            map_src = sorted_all[num_dst:]
            send = np.concatenate([seeds[perm[:num_dst]],
                                   I64(r) * I64(sp_base) * I64(num_total_nodes) + (map_src % num_dst) * I64(num_total_nodes)
                                   + nbr[perm[num_dst:] - num_dst]])
        else:
            m = src_to_vir(nbr, fanout, num_dst, min_vids, ws, rank=r)
            perm = np.argsort(m, kind="stable")
            sorted_all = m[perm]
            map_src = m
            send = I64(r) * I64(sp_base) * I64(num_total_nodes) + (sorted_all % num_dst) * I64(num_total_nodes) + nbr[perm]
        uniq = np.unique(map_src)
        pre.append(dict(seeds=seeds, neighbors=nbr, sorted_allnodes=sorted_all, perm=perm, unique_frontier=uniq,
                        block1_src=np.arange(len(uniq), dtype=I64), block1_dst=uniq % max(num_dst, 1),
                        send_frontier=send))
    sh = sp_sample_and_shuffle([len(p["seeds"]) for p in pre], [p["send_frontier"] for p in pre],
                               [p["sorted_allnodes"] for p in pre], [p["unique_frontier"] for p in pre],
                               with_dst, num_total_nodes)
    for r, p in enumerate(pre):
        p.update(sh[r])
        usrc, asrc = np.unique(p["ori_src"], return_inverse=True)
        udst, adst = np.unique(p["vir_src"], return_inverse=True)
        p.update(unique_src=usrc, block2_src=asrc.astype(I64), unique_dst=udst, block2_dst=adst.astype(I64))
        if with_dst:
            p["input_nodes"] = np.concatenate([p["recv_dst"], usrc])
        elif model == "GCN":
            p["input_nodes"] = usrc
        else:
            p["input_nodes"] = np.concatenate([p["seeds"], usrc])
    return pre


# ------------------------------------------------ NFP (feature dimension split)
def allbroadcast_v2(inputs, expand=1):
    """AllBroadcastV2, src/ops/collective.cc:367-402: every rank sends its whole
    (variable-length) input to every rank; received in rank order."""
    cat = np.concatenate([np.asarray(x).reshape(-1, expand) for x in inputs]) if inputs else np.zeros((0, expand))
    return [cat.copy() for _ in inputs]


def mp_sample_shuffle(seeds_pr, unique_frontier_pr, coo_row_pr):
    """MPSampleShuffle, src/sampling.cc:195-239, for all ranks at once: sizes
    all-gathered, frontiers and relabelled rows all-broadcast. Per rank:
    (recv_frontier, recv_coo_row, [seeds_size], recv_seeds_size,
    recv_frontier_size, recv_coo_size)."""
    ws = len(seeds_pr)
    seeds_size = np.array([len(x) for x in seeds_pr], dtype=I64)
    frontier_size = np.array([len(x) for x in unique_frontier_pr], dtype=I64)
    coo_size = np.array([len(x) for x in coo_row_pr], dtype=I64)
    fr = np.concatenate([np.asarray(x, dtype=I64) for x in unique_frontier_pr])
    co = np.concatenate([np.asarray(x, dtype=I64) for x in coo_row_pr])
    return [(fr.copy(), co.copy(), np.array([seeds_size[r]], dtype=I64), seeds_size.copy(), frontier_size.copy(),
             coo_size.copy()) for r in range(ws)]


def mp_feat_shuffle_fwd(inputs_pr, seg_sizes, feat_dim, acc=np.float64):
    """MPFeatShuffleFwd, src/feat_shuffle.cc:54-64 over _AllReduce,
    src/ops/collective.cc:404-436: rank r receives the sum over all ranks of
    their rows [off[r], off[r + 1]) (seg_sizes[r] rows of feat_dim)."""
    xs = [np.asarray(x).reshape(-1, feat_dim).astype(acc) for x in inputs_pr]
    return allreduce_scatter_v(xs, seg_sizes)


def mp_feat_shuffle_bwd(inputs_pr, feat_dim):
    """MPFeatShuffleBwd, src/feat_shuffle.cc:66-79: all-broadcast of every
    rank's rows."""
    return allbroadcast_v2(inputs_pr, feat_dim)


def mp_sample(seeds_pr, fanout, graph, key, call_id):
    """Outermost hop of the NFP sampler for SAGE / GCN, python/npc/sampler.py:332-356:
    local sampling and relabelling, then every rank gets every rank's frontier
    and relabelled rows; all_coo_col restarts at 0 for every sender's block."""
    pre = []
    for seeds in seeds_pr:
        seeds = np.asarray(seeds, dtype=I64)
        nbr = sample_csc_fanout(seeds, fanout, *graph, key=key, call_id=call_id)
        u, rel = relabel_csc(seeds, nbr)
        pre.append((seeds, nbr, u, rel))
    sh = mp_sample_shuffle([p[0] for p in pre], [p[2] for p in pre], [p[3] for p in pre])
    out = []
    for r, (fr, co, send_size, recv_size, recv_frontier_size, recv_coo_size) in enumerate(sh):
        col = np.concatenate([np.repeat(np.arange(int(i), dtype=I64), fanout) for i in recv_size])
        out.append(dict(neighbors=pre[r][1], all_frontier=fr, all_coo_row=co, all_coo_col=col, send_size=send_size,
                        recv_size=recv_size, recv_frontier_size=recv_frontier_size, recv_coo_size=recv_coo_size))
    return out


# ------------------------------------------- dry run, cache policy, cost model
def hot_order(freq):
    """torch.sort(freq, descending=True)[1] (python/npc/cost_model/estimator.py:26,
    :208-209) with equal frequencies by rising id."""
    freq = np.asarray(freq)
    return np.lexsort((np.arange(len(freq)), -freq.astype(np.int64))).astype(I64)


def get_cache_miss(seeds_freq, num_cache_nodes, input_dim, made_seeds_freq=None):
    """get_cache_miss, estimator.py:22-30."""
    seeds_freq = np.asarray(seeds_freq).astype(np.int64)
    order = hot_order(seeds_freq if made_seeds_freq is None else made_seeds_freq)
    k = min(int(num_cache_nodes), len(seeds_freq))
    return int(seeds_freq.sum() - seeds_freq[order[:k]].sum()) * int(input_dim)


def np_reshuffle_vol(world_size, rank, send_offset, recv_offset, dim):
    """get_np_reshuffle_vol, estimator.py:129-144."""
    so, ro = [int(x) for x in send_offset], [int(x) for x in recv_offset]
    total_send = so[world_size - 1] - so[rank] + (so[rank - 1] if rank > 0 else 0)
    total_recv = ro[world_size - 1] - ro[rank] + (ro[rank - 1] if rank > 0 else 0)
    return 2 * dim * (total_send + total_recv)


def sp_reshuffle_vol(world_size, rank, send_sizes, recv_sizes, dim, with_dst=False):
    """get_sp_reshuffle_vol for SAGE / GCN, estimator.py:147-178."""
    k = 3 if with_dst else 2
    vol = 0
    for r in range(world_size):
        if r == rank:
            continue
        vol += 2 * dim * int(send_sizes[k * r + k - 1] + recv_sizes[k * r + k - 1])
        if with_dst:
            vol += 2 * dim * int(send_sizes[3 * r] + recv_sizes[3 * r])
    return vol


def mp_reshuffle_vol(world_size, send_size, recv_size, dim):
    """get_mp_reshuffle_vol, estimator.py:181-188."""
    return 2 * dim * (int(send_size[0]) * (world_size - 2) + int(np.sum(recv_size)))


def vol_to_seconds(vol, mib_per_s, bytes_per_element=4):
    """cachemiss_vol_to_time / reshuffle_vol_to_time, estimator.py:112-118."""
    return vol * bytes_per_element / (1024 * 1024 * mib_per_s)


def all_strategy_sample(seeds_pr, fanouts, min_vids, graph, key, first_call_id, num_total_nodes, model="SAGE",
                        with_dst=False):
    """AllPSNeighborSampler.sample, python/npc/sampler.py:403-600, for all ranks at
    once: inner hops, then the outermost hop under GDP, NP, SNP (virtual nodes) and
    NFP. The outermost NP draw comes before the local one (:408-416), which fixes
    the call ids. Per rank: dict(dp_seeds, np=(seeds, send_offset, recv_offset),
    sp=(seeds, send_sizes, recv_sizes), mp=(seeds, send_size, recv_size))."""
    ws = len(seeds_pr)
    cur = [np.asarray(s_, dtype=I64) for s_ in seeds_pr]
    call = first_call_id
    rev = list(reversed(list(fanouts)))
    for f in rev[:-1]:
        nxt = []
        for s_ in cur:
            nb = sample_csc_fanout(s_, f, *graph, key=key, call_id=call)
            nxt.append(relabel_csc(s_, nb)[0])
        cur = nxt
        call += 1
    f = rev[-1]
    npo = np_sample_and_shuffle(cur, f, min_vids, graph, key=key, call_id=call)
    call += 1
    sp = sp_virtual_sample(cur, f, min_vids, graph, key=key, call_id=call, num_total_nodes=num_total_nodes,
                           with_dst=with_dst, model=model)
    mp = mp_sample(cur, f, graph, key=key, call_id=call)
    out = []
    for r in range(ws):
        uq, nb, _, so, ro, _ = npo[r]
        out.append(dict(dp_seeds=relabel_csc(cur[r], sp[r]["neighbors"])[0],
                        np=(relabel_csc(uq, nb)[0], so, ro),
                        sp=(sp[r]["input_nodes"], sp[r]["send_sizes"], sp[r]["recv_sizes"]),
                        mp=(mp[r]["all_frontier"], mp[r]["send_size"], mp[r]["recv_size"])))
    return out


# ------------------------------------------------------- synthetic generators
def rmat_edges(seed, first_edge, num_edges, scale, num_nodes, a=0.57, b=0.19, c=0.19):
    """The benchmark's R-MAT generator (counter-based; same stream as the GPU
    setup kernel): per edge and attempt, one Philox word per level picks the
    quadrant; endpoints >= num_nodes are redrawn (at most 64 attempts)."""
    f32 = np.float32
    a_, ab, abc = f32(a), f32(a) + f32(b), f32(a) + f32(b) + f32(c)
    e = np.arange(first_edge, first_edge + num_edges, dtype=U64)
    src = np.zeros(num_edges, dtype=I64)
    dst = np.zeros(num_edges, dtype=I64)
    todo = np.ones(num_edges, dtype=bool)
    for attempt in range(64):
        if not todo.any():
            break
        ee = e[todo]
        s = np.zeros(len(ee), dtype=I64)
        d = np.zeros(len(ee), dtype=I64)
        for lvl in range(0, scale, 4):
            w = philox4x32_10(ee & _MASK, ee >> U64(32), lvl >> 2, attempt, seed & 0xFFFFFFFF, (seed >> 32) & 0xFFFFFFFF)
            for t in range(4):
                if lvl + t >= scale:
                    break
                u = (w[t] >> U32(8)).astype(f32) * f32(1.0 / 16777216.0)
                sbit = (u >= ab).astype(I64)
                dbit = (((u >= a_) & (u < ab)) | (u >= abc)).astype(I64)
                s = (s << 1) | sbit
                d = (d << 1) | dbit
        ok = (s < num_nodes) & (d < num_nodes)
        idx = np.flatnonzero(todo)
        if attempt == 63:
            s, d, ok = s % num_nodes, d % num_nodes, np.ones_like(ok)
        src[idx[ok]] = s[ok]
        dst[idx[ok]] = d[ok]
        # a rejected draw still leaves its (reduced) value behind, as the kernel does
        src[idx[~ok]] = s[~ok] % num_nodes
        dst[idx[~ok]] = d[~ok] % num_nodes
        todo[idx[ok]] = False
    return src, dst


def csc_from_edges(src, dst, num_nodes, add_self_loops=True):
    """CSC (indptr over destinations, indices = sources) with rows sorted by
    source id; one self loop per node is appended first, like the reference's
    dataset preparation (scripts/load_data.py:71), so every degree is >= 1."""
    src = np.asarray(src, dtype=I64)
    dst = np.asarray(dst, dtype=I64)
    if add_self_loops:
        loop = np.arange(num_nodes, dtype=I64)
        src = np.concatenate([src, loop])
        dst = np.concatenate([dst, loop])
    bits = max(1, int(num_nodes - 1).bit_length())
    key = (dst.astype(U64) << U64(bits)) | src.astype(U64)
    key.sort()
    indices = (key & U64((1 << bits) - 1)).astype(I64)
    d = (key >> U64(bits)).astype(I64)
    indptr = np.zeros(num_nodes + 1, dtype=I64)
    np.cumsum(np.bincount(d, minlength=num_nodes), out=indptr[1:])
    return indptr, indices


# ------------------------------------------------- locality partition / skewed seeds
def bfs_order(indptr, indices, root):
    """Breadth-first visiting order over the in-neighbour lists of a CSC graph from `root`:
    level by level, ascending ids inside a level; nodes the search does not reach follow in
    ascending id order. Stands in for the partitioner of the reference's preprocessing
    (scripts/preprocess_dataset.py:76-135 calls METIS through DGL and then renumbers every
    part contiguously): contiguous blocks of this order are the locality-preserving partition
    of the synthetic graphs. Returns order with order[k] = the node visited k-th."""
    indptr = np.asarray(indptr, dtype=I64)
    indices = np.asarray(indices, dtype=I64)
    n = len(indptr) - 1
    visited = np.zeros(n, dtype=bool)
    order = np.empty(n, dtype=I64)
    frontier = np.array([root], dtype=I64)
    visited[root] = True
    pos = 0
    while len(frontier):
        order[pos:pos + len(frontier)] = frontier
        pos += len(frontier)
        mark = np.zeros(n, dtype=bool)
        for v in frontier:
            mark[indices[indptr[v]:indptr[v + 1]]] = True
        mark &= ~visited
        frontier = np.nonzero(mark)[0].astype(I64)
        visited |= mark
    order[pos:] = np.nonzero(~visited)[0]
    return order


def relabel_graph(indptr, indices, order):
    """The CSC after renumbering node order[k] to k (what dgl.reorder_graph does in
    scripts/preprocess_dataset.py:128-130): in-neighbour lists sorted by new source id."""
    indptr = np.asarray(indptr, dtype=I64)
    indices = np.asarray(indices, dtype=I64)
    n = len(indptr) - 1
    new_id = np.empty(n, dtype=I64)
    new_id[order] = np.arange(n, dtype=I64)
    dst = new_id[np.repeat(np.arange(n, dtype=I64), np.diff(indptr))]
    src = new_id[indices]
    key = np.lexsort((src, dst))
    counts = np.bincount(dst, minlength=n)
    return np.concatenate([[0], np.cumsum(counts)]).astype(I64), src[key]


def intra_partition_edge_share(indptr, indices, min_vids):
    """Share of edges whose two endpoints have the same owner (contiguous ranges min_vids)."""
    indptr = np.asarray(indptr, dtype=I64)
    n = len(indptr) - 1
    cuts = np.asarray(min_vids, dtype=I64)[1:-1]
    dst_owner = np.searchsorted(cuts, np.repeat(np.arange(n, dtype=I64), np.diff(indptr)), side="right")
    src_owner = np.searchsorted(cuts, np.asarray(indices, dtype=I64), side="right")
    return float((dst_owner == src_owner).mean()) if len(indices) else 1.0


def zipf_ranks(seed, first_draw, num_draws, num_ranks, s):
    """Ranks in [1, num_ranks], rank k with the mass of x^-s over [k, k+1): the inverse of that
    integral at u = (53 bits + 0.5) / 2^53, bits from words 0 and 1 of Philox4x32-10 with counter
    (draw, draw >> 32, 0, 'zipf') keyed by `seed` (twin of apt_zipf_ranks)."""
    d = np.arange(first_draw, first_draw + num_draws, dtype=U64)
    w = philox4x32_10(d & _MASK, d >> U64(32), 0, 0x7A697066, seed & 0xFFFFFFFF, (seed >> 32) & 0xFFFFFFFF)
    bits = ((w[0].astype(U64) << U64(32)) | w[1].astype(U64)) >> U64(11)
    u = (bits.astype(np.float64) + 0.5) * (1.0 / 9007199254740992.0)
    e = 1.0 - float(s)
    span = np.power(float(num_ranks) + 1.0, e) - 1.0
    k = np.floor(np.power(1.0 + u * span, 1.0 / e)).astype(I64)
    return np.clip(k, 1, num_ranks)


def zipf_seeds(seed, first_draw, num_draws, degree_order, s, batch):
    """`batch` distinct seed nodes: Zipf(s) ranks over `degree_order` (node ids by falling
    in-degree, ties by id), duplicates dropped keeping the first occurrence."""
    ranks = zipf_ranks(seed, first_draw, num_draws, len(degree_order), s)
    ids = np.asarray(degree_order, dtype=I64)[ranks - 1]
    _, first = np.unique(ids, return_index=True)
    return ids[np.sort(first)][:batch]
