"""The C-ABI library loads and exports exactly what include/apt_b200.h declares
(no compute calls: this runs without a GPU)."""
import os
import re
import subprocess

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "apt_b200.h")


def _declared():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(apt_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_are_exported_and_bound():
    from apt_b200 import _lib

    declared = _declared()
    assert len(declared) >= 30
    for name in declared:
        assert hasattr(_lib.lib, name), f"{name} declared in the header but not exported"
    assert sorted(_lib.exported_symbols()) == declared, "ctypes prototypes and header differ"
    out = subprocess.run(["nm", "-D", "--defined-only", _lib.LIB_PATH], capture_output=True, text=True).stdout
    exported = set(re.findall(r"\bT (apt_[a-z0-9_]+)", out))
    assert set(declared) <= exported
    assert exported <= set(declared), f"exported but undeclared: {sorted(exported - set(declared))}"


def test_argument_errors_without_gpu():
    from apt_b200 import _lib

    lib = _lib.lib
    assert lib.apt_version() >= 100
    assert lib.apt_relabel_workspace_bytes(1000) >= 1000 * 8
    assert lib.apt_gather_workspace_bytes(0) > 0
    assert lib.apt_bucket_workspace_bytes(5000, 8) >= 8 * 5 * 4
    # argument checks fire before any CUDA call
    st = lib.apt_sample_csc_fanout(None, 5, None, 0, None, 10, None, None, None, None, 1, 0, None, 1, None, None, None)
    assert st == _lib.APT_ERR_BAD_ARG and b"apt_sample_csc_fanout" in lib.apt_last_error()
    st = lib.apt_bucket_by_owner(None, 5, None, None, 64, 0, 0, 0, 1, None, 0, None, None, None, None, None)
    assert st == _lib.APT_ERR_BAD_ARG
    st = lib.apt_spmm_sum(9, 0, None, None, 0, None, None, 1, 1, None, None, None, 1, 0, None, None, 0, None)
    assert st == _lib.APT_ERR_BAD_ARG


def test_npc_operator_schemas_match_reference_registry():
    # src/pybind.cc:18-48 registers these 29 names
    import torch

    import apt_b200  # noqa: F401

    names = """nccl_get_unique_id init alltoall cache_feats_shared mix_cache_graphs register_min_vids
    register_multi_machines_scheme cpu_load_subtensor load_subtensor crossmachine_load_subtensor cluster_reqs
    local_sample_one_layer srcdst_to_vir src_to_vir np_sample_and_shuffle sp_sample_and_shuffle
    sp_sample_shuffle_src mp_sample_shuffle feat_shuffle sp_feat_shuffle mp_feat_shuffle_fwd mp_feat_shuffle_bwd
    shuffle_seeds relabel_csc spmm_copy_u_sum spmm_copy_e_sum spmm_u_mul_e_sum sddmm_u_add_v sddmm_u_mul_v""".split()
    assert len(names) == 29
    for n in names:
        assert hasattr(torch.ops.npc, n)
    # Argument and return TYPES against what the reference's own library registers:
    # tests/golden/ref_op_schemas.json holds the schema strings the dispatcher reports after
    # loading the compiled reference (tests/golden/make_ref_schemas.py). The reference's arguments
    # are unnamed (_0, _1, ...) because TORCH_LIBRARY infers them from C++ signatures; the names
    # given here are documentation, so only the types are compared.
    import json

    with open(os.path.join(ROOT, "tests", "golden", "ref_op_schemas.json")) as f:
        ref = json.load(f)
    assert sorted(ref) == sorted(names)

    def types_of(schema_text):
        sch = torch._C.parse_schema("npc::" + schema_text if not schema_text.startswith("npc::") else schema_text)
        return [str(a.type) for a in sch.arguments], [str(r.type) for r in sch.returns]

    for n in names:
        ours = torch._C._get_schema("npc::" + n, "")
        got = ([str(a.type) for a in ours.arguments], [str(r.type) for r in ours.returns])
        assert got == types_of(ref[n]), f"npc::{n}: {ours} differs from the reference's {ref[n]}"
    ident = torch.ops.npc.nccl_get_unique_id()
    assert ident.dtype == torch.int64 and ident.numel() == 16 and not ident.is_cuda


def test_ops_refuse_cpu_tensors():
    import pytest
    import torch

    import apt_b200

    with pytest.raises(RuntimeError, match="CUDA tensor"):
        apt_b200.relabel_csc(torch.arange(4), torch.arange(8))
