"""The SNP-GAT block (config 2 of the benchmark list: 4 heads x 64, bf16): fused edge
pipeline against the fp64 oracle and against the composition of the separate
operators, and the SNP-GAT sampler against the oracle with one rank."""
import numpy as np
import pytest
import torch

import apt_b200
from apt_b200 import ops
from oracle import oracle as orc
from tests.gpu_util import dev, host, install_graph, reset_world
from tests.helpers import small_graph

pytestmark = pytest.mark.gpu
I64 = np.int64
TOL = {torch.float32: 1e-5, torch.bfloat16: 1e-2, torch.float16: 1e-2}


def _round(x, dtype):
    return torch.from_numpy(x).to(dtype).float().numpy() if dtype != torch.float32 else x


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("S,f,H,Dh", [(512, 10, 4, 64), (100, 5, 1, 8), (333, 25, 8, 16), (64, 15, 3, 5)])
def test_fused_gat_block_matches_oracle(dtype, S, f, H, Dh):
    rng = np.random.default_rng(S + H)
    n_src = 3 * S
    row = rng.integers(0, n_src, S * f).astype(I64)
    col = np.repeat(np.arange(S, dtype=I64), f)
    ft = _round(rng.standard_normal((n_src, H, Dh)).astype(np.float32), dtype)
    el = _round(rng.standard_normal((n_src, H)).astype(np.float32), dtype)
    er = _round(rng.standard_normal((S, H)).astype(np.float32), dtype)
    out, attn = ops.gat_edge_softmax_sum(dev(row), dev(col), dev(ft, dtype), dev(el, dtype), dev(er, dtype), S, 0.2,
                                         return_attention=True)
    want, want_a = orc.gat_edge_softmax_sum(row, col, ft, el, er, S, 0.2)
    assert tuple(out.shape) == (S, H, Dh) and tuple(attn.shape) == (S * f, H, 1)
    tol = TOL[dtype]
    err = np.abs(host(out).astype(np.float64) - want) / np.maximum(np.abs(want), 1.0)
    assert err.max() <= tol, f"out max rel err {err.max():.2e}"
    erra = np.abs(host(attn).astype(np.float64).reshape(S * f, H) - want_a)
    assert erra.max() <= tol
    # attention sums to one over the edges of every destination
    sums = host(attn).astype(np.float64).reshape(S, f, H).sum(1)
    assert np.abs(sums - 1).max() <= (2e-2 if dtype != torch.float32 else 1e-5)
    ops.check_status()


def test_fused_gat_equals_separate_operators():
    # u_add_v -> leaky_relu -> softmax -> u_mul_e + sum with the reference's operator set
    g = torch.Generator(device="cuda").manual_seed(3)
    S, f, H, Dh, n_src = 2048, 15, 4, 64, 9000
    row = torch.randint(0, n_src, (S * f,), generator=g, device="cuda")
    col = torch.arange(S, device="cuda").repeat_interleave(f)
    ft = torch.randn((n_src, H, Dh), generator=g, device="cuda")
    el = torch.randn((n_src, H), generator=g, device="cuda")
    er = torch.randn((S, H), generator=g, device="cuda")
    off = [torch.tensor(v, device="cuda") for v in ([0, S * f], [0, n_src], [0, S])]
    e = ops.sddmm_u_add_v(row, col, el, er, off[0], off[1], off[2])
    a = torch.softmax(torch.nn.functional.leaky_relu(e, 0.2).view(S, f, H), dim=1).reshape(S * f, H)
    ref = ops.spmm_u_mul_e_sum(row, col, ft.view(n_src, H * Dh), a, off[0], off[1], off[2]).view(S, H, Dh)
    out = ops.gat_edge_softmax_sum(row, col, ft, el, er, S, 0.2)
    assert torch.allclose(out, ref, rtol=1e-5, atol=1e-5)


def test_fused_gat_rejects_ungrouped_edges():
    row = dev(np.array([0, 1, 2], dtype=I64))
    col = dev(np.array([1, 0, 1], dtype=I64))
    ft = torch.ones((3, 1, 4), device="cuda")
    out = ops.gat_edge_softmax_sum(row, col, ft, torch.ones((3, 1), device="cuda"), torch.ones((2, 1), device="cuda"), 2)
    torch.cuda.synchronize()
    assert not host(out).any()
    with pytest.raises(RuntimeError, match="not grouped"):
        ops.check_status()


@pytest.mark.parametrize("mode", ["plain", "chained", "graph", "graph_single_hop"])
def test_sp_gat_sampler_one_rank(mode):
    # operator by operator (one host read each), chained on the device (one read per mini-batch), and the
    # chained form replayed from a CUDA graph give the same mini-batch as the oracle
    n, indptr, indices = small_graph(scale=12, edge_factor=8)
    install_graph(indptr, indices)
    reset_world(1, 0)
    ops.register_min_vids(torch.tensor([0, n]))
    rng = np.random.default_rng(4)
    seeds = rng.permutation(n)[:300].astype(I64)
    kw = {"plain": dict(chained=False), "chained": dict(chained=True, use_graph=False),
          "graph": dict(chained=True, use_graph=True), "graph_single_hop": dict(chained=True, use_graph=True)}[mode]
    if mode == "graph_single_hop":
        ops.set_sampling(key=11, call_id=1)
        one = apt_b200.SPGATSampler(0, [10], prefetch_features=False, **kw)
        for _ in range(2):       # the second call replays the captured graph
            ops.set_sampling(key=11, call_id=1)
            in1, out1, b1, p1, so1, ro1 = one.sample(None, dev(seeds))
        w1 = orc.sp_gat_sample([seeds], 10, np.array([0, n]), (None, None, None, indptr, indices), key=11, call_id=1)[0]
        assert np.array_equal(host(in1), w1["input_nodes"]) and np.array_equal(host(b1[0].coo_row), w1["arange_src"])
        assert np.array_equal(host(b1[0].src_ids), w1["unique_neigh"]) and np.array_equal(host(p1), w1["perm"])
        ops.check_status()
        return
    smp = apt_b200.SPGATSampler(0, [10, 5], prefetch_features=False, **kw)
    for _ in range(2 if mode == "graph" else 1):
        ops.set_sampling(key=11, call_id=0)
        input_nodes, output_nodes, blocks, perm, send_off, recv_off = smp.sample(None, dev(seeds))
    graph = (None, None, None, indptr, indices)
    nbr = orc.sample_csc_fanout(seeds, 5, *graph, key=11, call_id=0)
    u1, r1 = orc.relabel_csc(seeds, nbr)
    want = orc.sp_gat_sample([u1], 10, np.array([0, n]), graph, key=11, call_id=1)[0]
    assert np.array_equal(host(blocks[1].coo_row), r1) and np.array_equal(host(blocks[1].src_ids), u1)
    assert np.array_equal(host(blocks[0].coo_row), want["arange_src"])
    assert np.array_equal(host(blocks[0].src_ids), want["unique_neigh"])
    assert blocks[0].num_dst == len(u1) and blocks[0].num_src == len(want["unique_neigh"])
    assert np.array_equal(host(input_nodes), want["input_nodes"])
    assert np.array_equal(host(perm), want["perm"])
    assert np.array_equal(send_off.numpy(), want["send_offset"]) and np.array_equal(recv_off.numpy(), want["recv_offset"])
    # features of the received ids come back in unique-neighbour order through the feature shuffle
    D = 32
    table = torch.randn((n, D), device="cuda")
    proj = table[input_nodes][blocks[0].num_dst:]
    back = ops.feat_shuffle(proj, send_off, recv_off, perm, D, 1)
    assert torch.equal(back, table[blocks[0].src_ids])
    ops.check_status()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("S,f,H,Dh", [(512, 10, 4, 64), (100, 5, 1, 8), (333, 25, 8, 16), (64, 15, 3, 5), (40, 4, 2, 256)])
def test_gat_backward_matches_oracle(dtype, S, f, H, Dh):
    rng = np.random.default_rng(S * 7 + H)
    n_src = 2 * S
    row = rng.integers(0, n_src, S * f).astype(I64)
    col = np.repeat(np.arange(S, dtype=I64), f)
    ft = _round(rng.standard_normal((n_src, H, Dh)).astype(np.float32), dtype)
    el = _round(rng.standard_normal((n_src, H)).astype(np.float32), dtype)
    er = _round(rng.standard_normal((S, H)).astype(np.float32), dtype)
    go = _round(rng.standard_normal((S, H, Dh)).astype(np.float32), dtype)
    g_ft, g_el, g_er = ops.gat_edge_softmax_sum_backward(dev(row), dev(col), dev(ft, dtype), dev(el, dtype),
                                                         dev(er, dtype), dev(go, dtype), 0.2)
    w_ft, w_el, w_er, _, _ = orc.gat_edge_softmax_sum_backward(row, col, ft, el, er, go, S, 0.2)
    assert tuple(g_ft.shape) == (n_src, H, Dh) and tuple(g_el.shape) == (n_src, H) and tuple(g_er.shape) == (S, H)
    tol = TOL[dtype]
    for got, want, name in ((g_ft, w_ft, "grad_ft"), (g_el, w_el, "grad_el"), (g_er, w_er, "grad_er")):
        # per-edge terms are rounded to the storage type before they are summed: scale by the largest value
        err = np.abs(host(got).astype(np.float64) - want).max() / max(np.abs(want).max(), 1.0)
        assert err <= tol, f"{name} max rel err {err:.2e}"
    ops.check_status()


def test_gat_autograd_function_against_torch():
    g = torch.Generator(device="cuda").manual_seed(5)
    S, f, H, Dh, n_src = 300, 7, 4, 32, 900
    row = torch.randint(0, n_src, (S * f,), generator=g, device="cuda")
    col = torch.arange(S, device="cuda").repeat_interleave(f)
    leaves = [torch.randn(shape, generator=g, device="cuda", requires_grad=True)
              for shape in ((n_src, H, Dh), (n_src, H), (S, H))]
    go = torch.randn((S, H, Dh), generator=g, device="cuda")
    out = apt_b200.GATEdgeSoftmaxSum.apply(row, col, *leaves, S, 0.2)
    out.backward(go)
    got = [t.grad.clone() for t in leaves]
    for t in leaves:
        t.grad = None
    ft, el, er = leaves
    s = torch.nn.functional.leaky_relu(el[row] + er[col], 0.2)
    a = torch.softmax(s.view(S, f, H), dim=1).reshape(S * f, H)
    ref = torch.zeros((S, H, Dh), device="cuda").index_add(0, col, a[:, :, None] * ft[row])
    assert (out - ref).abs().max().item() <= 1e-5
    ref.backward(go)
    for a_, b_ in zip(got, leaves):
        assert (a_ - b_.grad).abs().max().item() <= 2e-5 * max(1.0, b_.grad.abs().max().item())
    ops.check_status()
