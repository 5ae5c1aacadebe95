"""Multi-layer samplers of the data path without DGL: the loops of
MixedNeighborSampler (NP, python/npc/sampler.py:109-156) and of the DP branch
of MixedPSNeighborSampler (:187-203), returning blocks as plain COO tensors
instead of DGLBlock objects (DGL builds those from the same COO,
python/npc/sampler.py:59-91).
"""
from dataclasses import dataclass
from typing import List

import torch

from . import ops


@dataclass
class Block:
    """One sampled bipartite layer: edge e runs src coo_row[e] -> dst coo_col[e];
    src_ids[k] is the global id of local src k, and the first num_dst src nodes
    are the dst nodes (create_dgl_block, python/npc/sampler.py:76-91)."""

    coo_row: torch.Tensor
    coo_col: torch.Tensor
    num_src: int
    num_dst: int
    src_ids: torch.Tensor
    fanout: int


def create_block(seeds: torch.Tensor, neighbors: torch.Tensor, fanout: int) -> Block:
    unique_frontier, indices = ops.relabel_csc(seeds, neighbors)
    coo_col = torch.arange(0, seeds.numel(), device=indices.device).repeat_interleave(fanout)
    return Block(indices, coo_col, unique_frontier.numel(), seeds.numel(), unique_frontier, fanout)


class MixedNeighborSampler:
    """NP ("NPC") strategy: inner hops are sampled locally, the outermost hop at
    the owner of each frontier node (np_sample_and_shuffle). fanouts[0] is the
    outermost hop, as in the reference's --fan_out (python/npc/utils/utils.py:428-432)."""

    def __init__(self, rank: int, fanouts: List[int]):
        self.rank = rank
        self.fir_fanouts = list(fanouts[1:])
        self.las_fanouts = fanouts[0]
        self.num_layers = len(fanouts)

    def sample(self, graph, seeds: torch.Tensor):
        output_nodes = seeds
        blocks = []
        for fanout in reversed(self.fir_fanouts):
            seeds, neighbors = ops.local_sample_one_layer(seeds, fanout)
            block = create_block(seeds, neighbors, fanout)
            seeds = block.src_ids
            blocks.insert(0, block)
        seeds, neighbors, perm, send_offset, recv_offset, inverse_idx = ops.np_sample_and_shuffle(
            seeds, self.las_fanouts)
        block = create_block(seeds, neighbors, self.las_fanouts)
        blocks.insert(0, block)
        seeds = block.src_ids
        return seeds, output_nodes, blocks, perm, send_offset, recv_offset, inverse_idx


class DPNeighborSampler:
    """GDP strategy: every hop local (python/npc/sampler.py:202-203 with the
    common block construction)."""

    def __init__(self, rank: int, fanouts: List[int]):
        self.rank = rank
        self.fanouts = list(fanouts)

    def sample(self, graph, seeds: torch.Tensor):
        output_nodes = seeds
        blocks = []
        for fanout in reversed(self.fanouts):
            seeds, neighbors = ops.local_sample_one_layer(seeds, fanout)
            block = create_block(seeds, neighbors, fanout)
            seeds = block.src_ids
            blocks.insert(0, block)
        return seeds, output_nodes, blocks
