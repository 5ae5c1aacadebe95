"""Registers the operators under ``torch.ops.npc.*`` with the schemas the
reference's ``TORCH_LIBRARY(npc, m)`` block infers (src/pybind.cc:18-48), so
that the reference's Python package (python/npc/ops.py, sampler.py, model/)
runs on this library unchanged: importing this module takes the place of
``torch.classes.load_library(".../libnpc.so")`` (python/npc/__init__.py:6-12).

Operators of strategies outside the path built here are registered too and
raise NotImplementedError when called, so a missing piece fails loudly.
"""
import torch

from . import ops

_SCHEMAS = {
    "nccl_get_unique_id": "() -> Tensor",
    "init": "(int rank, int local_rank, int world_size, Tensor nccl_id_tensor_list, int node_size) -> ()",
    "alltoall": "(Tensor input, Tensor output, Tensor send_offset, Tensor recv_offset, int expand, int comm_type) -> ()",
    "cache_feats_shared": "(int num_total_nodes, Tensor localnode_feats, Tensor cached_feats, Tensor cached_idx, Tensor localnode_idx, int feat_dim_offset) -> ()",
    "mix_cache_graphs": "(int num_cached_nodes, Tensor cached_node_idx, Tensor cached_indptr, Tensor cached_indices, Tensor global_indptr, Tensor global_indices) -> ()",
    "register_min_vids": "(Tensor shuffle_min_vids, int shuffle_id_offset) -> ()",
    "cpu_load_subtensor": "(Tensor node_id) -> Tensor",
    "load_subtensor": "(Tensor node_id) -> Tensor",
    "local_sample_one_layer": "(Tensor seeds, int fanout) -> Tensor[]",
    "np_sample_and_shuffle": "(Tensor seeds, int fanout) -> Tensor[]",
    "srcdst_to_vir": "(int fanout, Tensor dst, Tensor src) -> Tensor",
    "src_to_vir": "(int fanout, int num_dst, Tensor src) -> Tensor",
    "sp_sample_and_shuffle": "(int num_dst, Tensor send_frontier, Tensor sorted_allnodes, Tensor unique_frontier, int shuffle_with_dst) -> Tensor[]",
    "sp_feat_shuffle": "(Tensor inputs, Tensor send_sizes, Tensor recv_sizes, int total_recv_size, int expand, int shuffle_with_dst) -> Tensor",
    "mp_sample_shuffle": "(Tensor seeds, Tensor unique_frontier, Tensor coo_row) -> Tensor[]",
    "mp_feat_shuffle_fwd": "(Tensor inputs, Tensor send_size, Tensor recv_size, int feat_dim) -> Tensor",
    "mp_feat_shuffle_bwd": "(Tensor inputs, Tensor send_size, Tensor recv_size, int feat_dim) -> Tensor",
    "sp_sample_shuffle_src": "(Tensor unique_src) -> Tensor[]",
    "feat_shuffle": "(Tensor inputs, Tensor send_offset, Tensor recv_offset, Tensor permutation, int feat_dim, int fwd_flag) -> Tensor",
    "shuffle_seeds": "(Tensor seeds) -> (Tensor, Tensor, Tensor, Tensor)",
    "relabel_csc": "(Tensor seeds, Tensor neighbors) -> Tensor[]",
    "spmm_copy_u_sum": "(Tensor coo_row, Tensor coo_col, Tensor input, Tensor coo_offset, Tensor input_offset, Tensor output_offset) -> Tensor",
    "spmm_copy_e_sum": "(Tensor coo_row, Tensor coo_col, Tensor input, Tensor coo_offset, Tensor output_offset) -> Tensor",
    "spmm_u_mul_e_sum": "(Tensor coo_row, Tensor coo_col, Tensor input, Tensor edata, Tensor coo_offset, Tensor input_offset, Tensor output_offset) -> Tensor",
    "sddmm_u_add_v": "(Tensor coo_row, Tensor coo_col, Tensor lhs, Tensor rhs, Tensor coo_offset, Tensor lhs_offset, Tensor rhs_offset) -> Tensor",
    "sddmm_u_mul_v": "(Tensor coo_row, Tensor coo_col, Tensor lhs, Tensor rhs, Tensor coo_offset, Tensor lhs_offset, Tensor rhs_offset) -> Tensor",
}

# Registered by the reference for several machines (src/pybind.cc:25,28-29);
# not part of this path.
_NOT_BUILT = {
    "register_multi_machines_scheme": "(Tensor remote_worker_map, Tensor remote_worker_id) -> ()",
    "crossmachine_load_subtensor": "(Tensor node_id) -> Tensor",
    "cluster_reqs": "(Tensor node_id) -> (Tensor, Tensor, Tensor)",
}

_LIB = torch.library.Library("npc", "DEF")


def _not_built(name):
    def fn(*args, **kwargs):
        raise NotImplementedError(f"torch.ops.npc.{name} belongs to a strategy this library does not implement")

    return fn


for _name, _schema in _SCHEMAS.items():
    _LIB.define(_name + _schema)
    _LIB.impl(_name, getattr(ops, _name), "CompositeExplicitAutograd")
for _name, _schema in _NOT_BUILT.items():
    _LIB.define(_name + _schema)
    _LIB.impl(_name, _not_built(_name), "CompositeExplicitAutograd")


def registered_ops():
    return sorted(_SCHEMAS), sorted(_NOT_BUILT)
