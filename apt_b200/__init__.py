"""apt_b200: the mini-batch data path of APT (sampling, relabelling,
cache-aware feature gather, seed/feature shuffle, SpMM/SDDMM) as hand-written
sm_100a CUDA behind the reference's ``torch.ops.npc`` operator interface.

Importing the package loads libapt_b200.so (raising if it is not built) and
registers the ``npc`` operators.
"""
import os as _os

# The samplers' pipelined iterator runs mini-batches on streams of their own. With CUDA's default of 8
# hardware queues the caller's stream shares a queue with one of them, and the caller's kernels and
# copies then wait behind that lane's queued mini-batches. The setting is read when CUDA starts, so
# it only takes effect when this package is imported before the first CUDA call of the process.
_os.environ.setdefault("CUDA_DEVICE_MAX_CONNECTIONS", "32")

from . import _lib  # noqa: E402,F401  (raises when the CUDA library is missing)
from . import npc_ops  # noqa: F401  (registers torch.ops.npc.*)
from . import ops
from .ops import (  # noqa: F401
    STATE, alltoall, cache_feats_shared, check_status, cpu_load_subtensor, feat_shuffle, init,
    load_subtensor, local_sample_one_layer, mix_cache_graphs, mp_feat_shuffle_bwd, mp_feat_shuffle_fwd,
    mp_sample_shuffle, nccl_get_unique_id, np_sample_and_shuffle,
    register_min_vids, relabel_csc, rows_gather, rows_scatter, sddmm_u_add_v, sddmm_u_mul_v, set_sampling,
    gat_edge_softmax_sum, gat_edge_softmax_sum_backward, GATEdgeSoftmaxSum, shuffle_seeds, sp_feat_shuffle, sp_sample_and_shuffle, sp_sample_shuffle_src, spmm_copy_e_sum, spmm_copy_u_sum, spmm_u_mul_e_sum, src_to_vir,
    srcdst_to_vir, unique_sorted,
)
from .sampler import Block, DPNeighborSampler, MPSampler, MixedNeighborSampler, SPGATSampler, SPVirtualSampler, create_block  # noqa: F401
