"""GPU parity of SpMM / SDDMM over sampled blocks against the fp64 CPU oracle: 1e-5 for fp32, 1e-2 for
bf16/fp16. SDDMM (no summation) is held to the plain relative error |got - want| <= tol * |want|. A sum is
held to |got - want| <= tol * (sum of the |terms|), the error bound of floating-point summation: equal to
the relative error where the terms do not cancel, and the most any fp32 summation can promise where they
do (the reference's own float-atomic sums of N(0,1) terms are off by up to 1e-4 relative at small outputs,
tests/test_ref_golden.py)."""
import numpy as np
import pytest
import torch

from apt_b200 import ops
from oracle import oracle as orc
from tests.gpu_util import dev, host

pytestmark = pytest.mark.gpu
I64 = np.int64
TOL = {torch.float32: 1e-5, torch.bfloat16: 1e-2, torch.float16: 1e-2}
# absolute floor of the relative error: the smallest normal number of the type (below it the spacing
# of representable values is fixed, so the error no longer shrinks with the value)
FLOOR = {torch.float32: 1.2e-38, torch.bfloat16: 1.2e-38, torch.float16: 6.2e-5}


def _close(got, want, dtype, magnitude=None):
    """magnitude: the same operator applied to the absolute values of its inputs (sums); None: no sum."""
    got = host(got).astype(np.float64)
    tol = TOL[dtype]
    scale = np.abs(want) if magnitude is None else magnitude
    err = np.abs(got - want) / np.maximum(scale, FLOOR[dtype])
    assert err.max() <= tol, f"max err {err.max():.3e} of the scale > {tol}"


def _mag(op, row, col, x, e, *off):
    return orc.spmm_sum(op, row, col, None if x is None else np.abs(x), None if e is None else np.abs(e), *off)


def _block(S, f, n_src, rng):
    row = rng.integers(0, n_src, S * f).astype(I64)
    col = np.repeat(np.arange(S, dtype=I64), f)
    return row, col


def _round(x, dtype):
    return torch.from_numpy(x).to(dtype).float().numpy() if dtype != torch.float32 else x


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("S,f,D", [(1024, 10, 256), (300, 25, 128), (77, 5, 64), (50, 3, 7), (2000, 15, 4)])
def test_copy_u_sum_sorted_block(dtype, S, f, D):
    rng = np.random.default_rng(S + D)
    n_src = S * 3
    row, col = _block(S, f, n_src, rng)
    x = _round(rng.standard_normal((n_src, D)).astype(np.float32), dtype)
    off = (np.array([0, S * f], dtype=I64), np.array([0, n_src], dtype=I64), np.array([0, S], dtype=I64))
    out = ops.spmm_copy_u_sum(dev(row), dev(col), dev(x, dtype), dev(off[0]), dev(off[1]), dev(off[2]))
    want = orc.spmm_sum("copy_u", row, col, x, None, *off)
    assert out.dtype == dtype and tuple(out.shape) == (S, D)
    _close(out, want, dtype, _mag("copy_u", row, col, x, None, *off))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_copy_u_sum_unsorted_backward_shape(dtype):
    # the backward call swaps row/col and the offsets (python/npc/model/sageconv.py:113):
    # destinations are then the relabelled src ids, in no order
    rng = np.random.default_rng(3)
    S, f, D, n_src = 512, 10, 128, 1500
    row, col = _block(S, f, n_src, rng)
    g = _round(rng.standard_normal((S, D)).astype(np.float32), dtype)
    off = (np.array([0, S * f], dtype=I64), np.array([0, S], dtype=I64), np.array([0, n_src], dtype=I64))
    out = ops.spmm_copy_u_sum(dev(col), dev(row), dev(g, dtype), dev(off[0]), dev(off[1]), dev(off[2]))
    want = orc.spmm_sum("copy_u", col, row, g, None, *off)
    assert tuple(out.shape) == (n_src, D)
    # rows that receive no edge are exactly zero; the others are summed in fp32 and rounded once
    _close(out, want, dtype, np.maximum(_mag("copy_u", col, row, g, None, *off), 1e-30))
    assert not host(out)[np.bincount(row, minlength=n_src) == 0].any()


@pytest.mark.parametrize("grouped", [True, False])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_hub_rows_with_thousands_of_edges(grouped, dtype):
    # power-law destinations (the backward call): a few output rows own most of the edges
    rng = np.random.default_rng(12)
    n_in, n_out, E, D = 3000, 500, 60000, 128
    col = np.minimum((rng.zipf(1.4, E) - 1), n_out - 1).astype(I64)
    if grouped:
        col = np.sort(col)
    row = rng.integers(0, n_in, E).astype(I64)
    x = _round(rng.standard_normal((n_in, D)).astype(np.float32), dtype)
    off = (np.array([0, E], dtype=I64), np.array([0, n_in], dtype=I64), np.array([0, n_out], dtype=I64))
    assert np.bincount(col).max() > 5000
    out = ops.spmm_copy_u_sum(dev(row), dev(col), dev(x, dtype), dev(off[0]), dev(off[1]), dev(off[2]))
    want = orc.spmm_sum("copy_u", row, col, x, None, *off)
    _close(out, want, dtype, _mag("copy_u", row, col, x, None, *off))


def test_empty_rows_and_empty_edges():
    D = 16
    x = np.ones((10, D), dtype=np.float32)
    row = np.array([1, 2, 3], dtype=I64)
    col = np.array([0, 0, 4], dtype=I64)   # rows 1,2,3,5 receive nothing
    off = (np.array([0, 3], dtype=I64), np.array([0, 10], dtype=I64), np.array([0, 6], dtype=I64))
    out = ops.spmm_copy_u_sum(dev(row), dev(col), dev(x), dev(off[0]), dev(off[1]), dev(off[2]))
    assert host(out).sum(1).tolist() == [2 * D, 0, 0, 0, D, 0]
    e = torch.empty(0, dtype=torch.int64, device="cuda")
    out = ops.spmm_copy_u_sum(e, e, dev(x), dev(np.array([0, 0], dtype=I64)), dev(off[1]), dev(off[2]))
    assert tuple(out.shape) == (6, D) and not host(out).any()


def test_segments_batched_blocks():
    # three blocks concatenated the way the NFP callers build them (python/npc/model/sageconv.py:159-161)
    rng = np.random.default_rng(4)
    D = 32
    sizes_e, sizes_in, sizes_out = [300, 0, 500], [100, 50, 200], [30, 10, 50]
    rows, cols = [], []
    for e, ni, no in zip(sizes_e, sizes_in, sizes_out):
        rows.append(rng.integers(0, ni, e))
        cols.append(np.sort(rng.integers(0, no, e)))
    row, col = np.concatenate(rows).astype(I64), np.concatenate(cols).astype(I64)
    coo = np.concatenate([[0], np.cumsum(sizes_e)]).astype(I64)
    ioff = np.concatenate([[0], np.cumsum(sizes_in)]).astype(I64)
    ooff = np.concatenate([[0], np.cumsum(sizes_out)]).astype(I64)
    x = rng.standard_normal((sum(sizes_in), D)).astype(np.float32)
    out = ops.spmm_copy_u_sum(dev(row), dev(col), dev(x), dev(coo), dev(ioff), dev(ooff))
    _close(out, orc.spmm_sum("copy_u", row, col, x, None, coo, ioff, ooff), torch.float32,
           _mag("copy_u", row, col, x, None, coo, ioff, ooff))
    lhs = rng.standard_normal((sum(sizes_in), D)).astype(np.float32)
    rhs = rng.standard_normal((sum(sizes_out), D)).astype(np.float32)
    for name, fn in (("u_add_v", ops.sddmm_u_add_v), ("u_mul_v", ops.sddmm_u_mul_v)):
        got = fn(dev(row), dev(col), dev(lhs), dev(rhs), dev(coo), dev(ioff), dev(ooff))
        want = orc.sddmm(name, row, col, lhs, rhs, coo, ioff, ooff, acc=np.float32)
        assert np.array_equal(host(got), want)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_copy_e_and_u_mul_e(dtype):
    rng = np.random.default_rng(5)
    S, f, H, Dh, n_src = 256, 10, 4, 64, 700
    D = H * Dh
    row, col = _block(S, f, n_src, rng)
    off = (np.array([0, S * f], dtype=I64), np.array([0, n_src], dtype=I64), np.array([0, S], dtype=I64))
    x = _round(rng.standard_normal((n_src, D)).astype(np.float32), dtype)
    e_full = _round(rng.standard_normal((S * f, D)).astype(np.float32), dtype)
    e_head = _round(rng.random((S * f, H)).astype(np.float32), dtype)
    out = ops.spmm_copy_e_sum(dev(row), dev(col), dev(e_full, dtype), dev(off[0]), dev(off[2]))
    _close(out, orc.spmm_sum("copy_e", row, col, None, e_full, *off), dtype, _mag("copy_e", row, col, None, e_full, *off))
    out = ops.spmm_u_mul_e_sum(dev(row), dev(col), dev(x, dtype), dev(e_full, dtype), *[dev(o) for o in off])
    _close(out, orc.spmm_sum("u_mul_e", row, col, x, e_full, *off), dtype, _mag("u_mul_e", row, col, x, e_full, *off))
    # one attention weight per head, broadcast over the head's columns (GAT, python/npc/model/gatconv.py:124)
    out = ops.spmm_u_mul_e_sum(dev(row), dev(col), dev(x, dtype), dev(e_head, dtype), *[dev(o) for o in off])
    _close(out, orc.spmm_sum("u_mul_e", row, col, x, e_head, *off), dtype, _mag("u_mul_e", row, col, x, e_head, *off))
    # what the reference's kernel really computes (src/cuda/spmm.cu:78)
    out = ops.spmm_u_mul_e_sum(dev(row), dev(col), dev(x, dtype), dev(e_full, dtype), *[dev(o) for o in off],
                               ref_quirk_add=True)
    _close(out, orc.spmm_sum("u_add_e", row, col, x, e_full, *off), dtype, _mag("u_add_e", row, col, x, e_full, *off))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("D", [4, 1, 64, 13])
def test_sddmm(dtype, D):
    rng = np.random.default_rng(D)
    S, f, n_src = 500, 10, 900
    row, col = _block(S, f, n_src, rng)
    lhs = _round(rng.standard_normal((n_src, D)).astype(np.float32), dtype)
    rhs = _round(rng.standard_normal((S, D)).astype(np.float32), dtype)
    off = (np.array([0, S * f], dtype=I64), np.array([0, n_src], dtype=I64), np.array([0, S], dtype=I64))
    for name, fn in (("u_add_v", ops.sddmm_u_add_v), ("u_mul_v", ops.sddmm_u_mul_v)):
        got = fn(dev(row), dev(col), dev(lhs, dtype), dev(rhs, dtype), *[dev(o) for o in off])
        want = orc.sddmm(name, row, col, lhs, rhs, *off)
        assert tuple(got.shape) == (S * f, D)
        _close(got, want, dtype)


def test_spmm_linearity_full_size():
    # papers-shaped outer block: 67 584 dst x fanout 15, hidden 256; spmm(a*x + y) == a*spmm(x) + spmm(y)
    g = torch.Generator(device="cuda").manual_seed(2)
    S, f, D, n_src = 67584, 15, 256, 700_000
    row = torch.randint(0, n_src, (S * f,), generator=g, device="cuda")
    col = torch.arange(S, device="cuda").repeat_interleave(f)
    x = torch.randn((n_src, D), generator=g, device="cuda")
    y = torch.randn((n_src, D), generator=g, device="cuda")
    off = [torch.tensor(v, device="cuda") for v in ([0, S * f], [0, n_src], [0, S])]
    sx = ops.spmm_copy_u_sum(row, col, x, *off)
    sy = ops.spmm_copy_u_sum(row, col, y, *off)
    sxy = ops.spmm_copy_u_sum(row, col, 2.0 * x + y, *off)
    assert torch.allclose(sxy, 2.0 * sx + sy, rtol=1e-4, atol=1e-4)
    ref = x[row].view(S, f, D).sum(1)
    assert torch.allclose(sx, ref, rtol=1e-5, atol=1e-5)
