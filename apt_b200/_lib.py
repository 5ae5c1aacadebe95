"""ctypes binding of libapt_b200.so (the C ABI declared in include/apt_b200.h).

There is no CPU or PyTorch fallback: if the CUDA library has not been built,
importing this module raises. Build it with ``python apt_b200/build.py``.
"""
import ctypes
import os
from ctypes import c_char_p, c_double, c_float, c_int, c_int64, c_size_t, c_uint32, c_uint64, c_void_p

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG, "libapt_b200.so")

if not os.path.exists(LIB_PATH):
    raise ImportError(
        f"{LIB_PATH} is missing: the sm_100a CUDA library has not been built "
        "(run `python apt_b200/build.py`). apt_b200 has no fallback path."
    )

lib = ctypes.CDLL(LIB_PATH)

APT_OK, APT_ERR_BAD_ARG, APT_ERR_CUDA, APT_ERR_TIMEOUT, APT_ERR_OOB, APT_ERR_CAPACITY = range(6)
FLAG_ID_OUT_OF_RANGE, FLAG_FEAT_NOT_EXIST, FLAG_ZERO_DEGREE, FLAG_TABLE_FULL, FLAG_PEER_TIMEOUT = 1, 2, 4, 8, 16
FLAG_NOT_GROUPED = 32
FLAG_SIZE_MISMATCH = 64
F32, BF16, F16 = 0, 1, 2
IPC_HANDLE_BYTES = 64

P = c_void_p
# name -> (restype, argtypes); mirrors include/apt_b200.h line by line.
PROTOTYPES = {
    "apt_last_error": (c_char_p, []),
    "apt_version": (c_int, []),
    "apt_launch_count": (c_int64, []),
    "apt_launch_count_reset": (None, []),
    "apt_memcpy_async": (c_int, [P, P, c_size_t, P]),
    "apt_set_tunable": (c_int, [c_char_p, c_int64]),
    "apt_profile_enable": (c_int, [c_int]),
    "apt_profile_read": (c_int, [c_char_p, ctypes.POINTER(c_double), ctypes.POINTER(c_int64)]),
    "apt_sample_csc_fanout": (c_int, [P, c_int64, P, c_int, P, c_int64, P, P, P, P, c_uint64, c_uint32, P, c_int, P, P, P]),
    "apt_relabel_workspace_bytes": (c_size_t, [c_int64]),
    "apt_relabel_workspace_init": (c_int, [P, c_size_t, P]),
    "apt_relabel_csc": (c_int, [P, c_int64, P, P, c_int64, P, c_size_t, P, P, P, P, P]),
    "apt_sample_relabel_csc": (c_int, [P, c_int64, P, c_int, P, c_int64, P, P, P, P, c_uint64, c_uint32, P, P, c_size_t,
                                       P, P, P, P, P, P]),
    "apt_bucket_workspace_bytes": (c_size_t, [c_int64, c_int]),
    "apt_bucket_by_owner": (c_int, [P, c_int64, P, P, c_int, c_int64, c_int, c_int, c_int, P, c_size_t, P, P, P, P, P]),
    "apt_unique_workspace_bytes": (c_size_t, [c_int64]),
    "apt_unique_workspace_init": (c_int, [P, c_size_t, P]),
    "apt_unique_sorted": (c_int, [P, c_int64, P, c_int64, c_int64, P, c_size_t, P, P, P, P, P]),
    "apt_concat_ids": (c_int, [P, c_int64, P, P, c_int64, P, P, P, P]),
    "apt_gather_workspace_bytes": (c_size_t, [c_int64]),
    "apt_gather_rows": (c_int, [P, c_int64, P, P, c_int64, P, c_int64, c_int64, P, c_int64, c_int64, c_int64, P, P, c_size_t, P, P]),
    "apt_gather_rows_from": (c_int, [P, c_int64, P, P, P, c_int64, P, c_int64, c_int64, P, c_int64, c_int64, c_int64, P, P,
                                     c_size_t, P, P]),
    "apt_gather_static_max_rows": (c_int64, []),
    "apt_gather_rows_static": (c_int, [P, c_int64, P, c_int64, P, c_int64, c_int64, P, c_int64, c_int64, c_int64, P, P, P]),
    "apt_spmm_workspace_bytes": (c_size_t, [c_int64, c_int64]),
    "apt_spmm_sum": (c_int, [c_int, c_int, P, P, c_int64, P, P, c_int64, c_int64, P, P, P, c_int, c_int64, P, P, c_size_t, P]),
    "apt_sddmm": (c_int, [c_int, c_int, P, P, c_int64, P, P, c_int64, P, P, P, c_int, P, P]),
    "apt_gat_edge_softmax_sum": (c_int, [c_int, P, P, c_int64, P, P, P, c_int, c_int64, c_float, c_int64, P, P, P, c_size_t, P, P]),
    "apt_gat_edge_backward": (c_int, [c_int, P, P, c_int64, P, P, P, P, c_int, c_int64, c_float, c_int64, P, P, P, P, c_size_t, P, P]),
    "apt_src_to_vir": (c_int, [P, c_int64, c_int64, c_int64, P, c_int, c_int, c_int, c_int, c_int, P, P]),
    "apt_srcdst_to_vir": (c_int, [P, c_int64, P, c_int64, c_int64, P, c_int, c_int, c_int, c_int, c_int, P, P]),
    "apt_vir_send_sizes": (c_int, [P, c_int64, P, P, c_int64, P, c_int, c_int64, P, c_int, P, P, P]),
    "apt_sp_map_place_pack": (c_int, [P, P, c_int64, P, c_int64, P, c_int, c_int, c_int, c_int, c_int, c_int64, c_int64, P, P, P, P]),
    "apt_sp_pack_frontier": (c_int, [P, P, c_int64, c_int64, c_int, c_int64, c_int64, P, P]),
    "apt_sp_unpack_frontier": (c_int, [P, c_int64, P, c_int64, P, P, P]),
    "apt_hotness_add": (c_int, [P, c_int64, P, P, c_int64, P, P]),
    "apt_hot_order_workspace_bytes": (c_size_t, [c_int64]),
    "apt_hot_order": (c_int, [P, c_int64, P, c_size_t, P, P]),
    "apt_cached_access": (c_int, [P, c_int64, P, c_int64, P, P]),
    "apt_rows_gather": (c_int, [P, P, c_int64, c_int64, P, P]),
    "apt_rows_scatter": (c_int, [P, P, c_int64, c_int64, P, P]),
    "apt_p2p_create": (c_int, [c_int, c_int, c_size_t, ctypes.POINTER(P), P]),
    "apt_p2p_attach": (c_int, [P, c_int, P]),
    "apt_p2p_attach_ptr": (c_int, [P, c_int, P]),
    "apt_p2p_local_base": (P, [P]),
    "apt_p2p_destroy": (c_int, [P]),
    "apt_p2p_region_bytes": (c_size_t, [P]),
    "apt_p2p_push": (c_int, [P, P, P, c_int, P, c_int64, c_int64, P, P]),
    "apt_p2p_wait": (c_int, [P, P, P, c_int64, P]),
    "apt_p2p_default_timeout_ns": (c_int64, []),
    "apt_p2p_probe_copy": (c_int, [P, c_int, c_size_t, P]),
    "apt_p2p_poisoned": (c_int, [P, ctypes.POINTER(c_int)]),
    "apt_p2p_pull": (c_int, [P, P, P, c_int, c_int64, c_int64, c_int64, P, P]),
    "apt_p2p_pull_sum": (c_int, [P, P, c_int, c_int64, c_int64, P, P, P]),
    "apt_p2p_create_landing": (c_int, [c_int, c_int, c_size_t, c_size_t, c_int, ctypes.POINTER(P), P]),
    "apt_p2p_landing_bytes": (c_size_t, [P]),
    "apt_p2p_landing": (P, [P, c_int]),
    "apt_p2p_push_direct": (c_int, [P, P, P, c_int, P, c_int64, c_int64, c_int, P, P]),
    "apt_p2p_alltoall_fused": (c_int, [P, P, P, c_int, P, P, P, c_int64, c_int64, c_int, P, P, c_int64, P]),
    "apt_rmat_edges": (c_int, [c_uint64, c_int64, c_int64, c_int, c_int64, c_float, c_float, c_float, P, P, P]),
    "apt_zipf_ranks": (c_int, [c_uint64, c_int64, c_int64, c_int64, c_double, P, P]),
    "apt_sort_u64_temp_bytes": (c_size_t, [c_int64]),
    "apt_sort_u64": (c_int, [P, P, c_int64, P, c_size_t, c_int, P]),
    "apt_normal_rows": (c_int, [c_uint64, c_int64, P, c_int64, c_int64, c_int, P, P]),
}

for _name, (_res, _args) in PROTOTYPES.items():
    _fn = getattr(lib, _name)  # AttributeError here means header and library disagree
    _fn.restype = _res
    _fn.argtypes = _args


# APT_TUNABLES="name=value,name=value": measurement knobs of apt_set_tunable applied at import.
for _kv in filter(None, os.environ.get("APT_TUNABLES", "").split(",")):
    _k, _, _v = _kv.partition("=")
    if lib.apt_set_tunable(_k.strip().encode(), int(_v)) != APT_OK:
        raise ValueError("APT_TUNABLES: " + lib.apt_last_error().decode("utf-8", "replace"))


class AptError(RuntimeError):
    """A C-ABI call returned a non-zero apt_status."""

    def __init__(self, status, text):
        super().__init__(f"libapt_b200 status {status}: {text}")
        self.status = status


def check(status):
    if status != APT_OK:
        raise AptError(status, lib.apt_last_error().decode("utf-8", "replace"))


def exported_symbols():
    return sorted(PROTOTYPES)
