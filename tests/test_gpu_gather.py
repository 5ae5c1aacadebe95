"""GPU parity of the cache-aware feature gather (bit-exact byte copies)."""
import ctypes

import numpy as np
import pytest
import torch

import apt_b200
from apt_b200 import _lib, ops
from oracle import oracle as orc
from tests.gpu_util import dev, host
from tests.helpers import feature_setup

pytestmark = pytest.mark.gpu
I64 = np.int64
TORCH_DT = {"f32": torch.float32, "bf16": torch.bfloat16, "f16": torch.float16}


def _install(n, dim, cache_frac, rng, dtype="f32", host_frac=1.0, offset=0, width=None):
    feats, uva, devf, cached_idx, local_idx, pos_map, cpu_map = feature_setup(n, dim, cache_frac, rng, host_frac=host_frac)
    tdt = TORCH_DT[dtype]
    uva_t = torch.from_numpy(uva).to(tdt).pin_memory()
    width = width or dim
    dev_t = torch.from_numpy(devf).to(tdt)[:, offset:offset + width].contiguous().cuda()
    ops.cache_feats_shared(n, uva_t, dev_t, torch.from_numpy(cached_idx), torch.from_numpy(local_idx), offset)
    table = torch.from_numpy(feats).to(tdt)[:, offset:offset + width]
    return table, pos_map, cpu_map, uva_t


@pytest.mark.parametrize("dtype,dim", [("f32", 128), ("bf16", 256), ("f16", 1024), ("f32", 25), ("bf16", 7), ("f32", 4), ("f16", 1)])
@pytest.mark.parametrize("cache_frac", [0.0, 0.3, 1.0])
def test_gather_matches_table(dtype, dim, cache_frac):
    rng = np.random.default_rng(dim)
    n = 5000
    table, pos_map, cpu_map, _ = _install(n, dim, cache_frac, rng, dtype)
    ids = rng.integers(0, n, 20011).astype(I64)
    out = ops.load_subtensor(dev(ids))
    torch.cuda.synchronize()
    assert out.dtype == TORCH_DT[dtype] and tuple(out.shape) == (len(ids), dim)
    assert torch.equal(out.cpu(), table[torch.from_numpy(ids)])
    ops.check_status()


def test_gather_oracle_and_cpu_twin():
    rng = np.random.default_rng(5)
    n, dim = 3000, 64
    feats, uva, devf, cached_idx, local_idx, pos_map, cpu_map = feature_setup(n, dim, 0.25, rng)
    uva_t = torch.from_numpy(uva).pin_memory()
    ops.cache_feats_shared(n, uva_t, dev(devf), torch.from_numpy(cached_idx), torch.from_numpy(local_idx), 0)
    ids = rng.integers(0, n, 4097).astype(I64)
    want = orc.load_subtensor(ids, pos_map, devf, uva)
    assert np.array_equal(host(ops.load_subtensor(dev(ids))), want)
    # cpu_load_subtensor is the reference's CPU op (src/load_subtensor.cc:10-17)
    assert np.array_equal(ops.cpu_load_subtensor(torch.from_numpy(ids)).numpy(), want)
    assert np.array_equal(host(ops.STATE.feat.feat_pos_map), pos_map)
    assert np.array_equal(ops.STATE.feat.cpu_feat_pos_map.numpy(), cpu_map)


def test_gather_column_window():
    # model-parallel slice: cache holds columns [8,24) of 32; host rows are read at the same offset
    rng = np.random.default_rng(6)
    table, *_ = _install(2000, 32, 0.4, rng, "f32", offset=8, width=16)
    ids = rng.integers(0, 2000, 3333).astype(I64)
    out = ops.load_subtensor(dev(ids))
    assert torch.equal(out.cpu(), table[torch.from_numpy(ids)])
    # odd offset: falls back to narrower vectors
    table, *_ = _install(2000, 32, 0.4, rng, "f32", offset=3, width=9)
    out = ops.load_subtensor(dev(ids))
    assert torch.equal(out.cpu(), table[torch.from_numpy(ids)])


def test_gather_missing_row_is_zero_and_flagged():
    rng = np.random.default_rng(7)
    n, dim = 1000, 16
    feats, uva, devf, cached_idx, local_idx, pos_map, cpu_map = feature_setup(n, dim, 0.2, rng, host_frac=0.5)
    ops.cache_feats_shared(n, torch.from_numpy(uva).pin_memory(), dev(devf), torch.from_numpy(cached_idx),
                           torch.from_numpy(local_idx), 0)
    absent = np.setdiff1d(np.arange(n), local_idx)
    ids = np.concatenate([local_idx[:50], absent[:5]]).astype(I64)
    out = ops.load_subtensor(dev(ids))
    torch.cuda.synchronize()
    assert np.array_equal(host(out)[:50], feats[ids[:50]])
    assert not host(out)[50:].any()
    with pytest.raises(RuntimeError, match="neither cached nor in host memory"):
        ops.check_status()


def test_gather_empty_and_single():
    rng = np.random.default_rng(8)
    table, *_ = _install(100, 128, 0.5, rng)
    out = ops.load_subtensor(torch.empty(0, dtype=torch.int64, device="cuda"))
    assert tuple(out.shape) == (0, 128)
    out = ops.load_subtensor(dev(np.array([42], dtype=I64)))
    assert torch.equal(out.cpu()[0], table[42])


def test_gather_full_size_checksum():
    # papers-shaped outer hop: about 1.08 M rows of 512 B; rows are tagged so that a
    # checksum over columns proves every row landed where it should.
    n, dim, rows = 2_000_000, 128, 1_081_344
    g = torch.Generator(device="cuda").manual_seed(1)
    feats = torch.randn((n, dim), generator=g, device="cuda")
    feats[:, 0] = torch.arange(n, device="cuda", dtype=torch.float32)
    cached = torch.arange(0, n, 2)                       # even ids cached, odd ids in host memory
    local = torch.arange(n)
    uva = torch.empty((n, dim), dtype=torch.float32).pin_memory()
    uva.copy_(feats)
    ops.cache_feats_shared(n, uva, feats[cached.cuda()].contiguous(), cached, local, 0)
    ids = torch.randint(0, n, (rows,), generator=g, device="cuda")
    out = ops.load_subtensor(ids)
    assert torch.equal(out[:, 0].long(), ids)
    assert torch.equal(out.sum(1), feats[ids].sum(1))
    ops.check_status()


def test_gather_direct_abi_call_capacity_error():
    rng = np.random.default_rng(9)
    _install(100, 8, 0.5, rng)
    f = ops.STATE.feat
    ids = dev(np.arange(50, dtype=I64))
    out = torch.empty((50, 8), device="cuda")
    ws = torch.empty(64, dtype=torch.uint8, device="cuda")
    st = _lib.lib.apt_gather_rows(ids.data_ptr(), 50, None, f.feat_pos_map.data_ptr(), 100, f.dev_feats.data_ptr(),
                                  f.dev_feats.shape[0], 32, f.uva_feats.data_ptr(), 100, 32, 0, out.data_ptr(),
                                  ws.data_ptr(), 64, ops.STATE.status_ptr(), None)
    assert st == _lib.APT_ERR_CAPACITY
