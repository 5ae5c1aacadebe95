// Fanout neighbour sampling over a CSC graph: a group of G lanes (8, 16 or 32,
// the power of two covering the fanout) serves one seed, so a warp serves
// 32/G seeds at once and each lane produces one output slot. Draws come from
// a counter-based Philox stream, so the result depends only on
// (key, call_id, seed slot, draw slot) and not on the launch shape.
//
// With INSERT the kernel is also the first pass of the relabelling that follows
// a sampled layer: every id it handles (the seed at position j, the neighbour of
// draw slot i at position S + j * fanout + i) enters the relabel table while it is
// still in a register, so the neighbour list need not be read back.
#pragma once

#include "relabel_table.cuh"

namespace apt {

__device__ __forceinline__ uint32_t draw_word(uint64_t j, uint32_t i,
                                              uint32_t call_id, uint32_t k0,
                                              uint32_t k1) {
  const Philox4 p = philox4x32_10((uint32_t)j, (uint32_t)(j >> 32), i >> 2,
                                  call_id, k0, k1);
  return p.w[i & 3];
}

__device__ __forceinline__ int64_t mod_deg(uint32_t word, int64_t deg) {
  // word < 2^32, so for deg >= 2^32 the remainder is the word itself.
  return deg <= 0xffffffffll ? (int64_t)(word % (uint32_t)deg) : (int64_t)word;
}

struct SampleInsert {
  Slot* slots;        // relabel table (INSERT only)
  int32_t* slot_of;   // [S + S * fanout] slot of every item
};

template <int G, bool INSERT>
__global__ void __launch_bounds__(256)
sample_replace_kernel(const int64_t* __restrict__ seeds, int64_t num_seeds,
                      const int64_t* __restrict__ num_seeds_dev, int fanout, const int64_t* __restrict__ adj_pos_map,
                      int64_t num_nodes, const int64_t* __restrict__ dev_indptr,
                      const int64_t* __restrict__ dev_indices,
                      const int64_t* __restrict__ uva_indptr,
                      const int64_t* __restrict__ uva_indices, uint32_t k0,
                      uint32_t k1, uint32_t call_id, const int64_t* __restrict__ call_base_dev,
                      int64_t* __restrict__ out, int32_t* status, SampleInsert ins) {
  num_seeds = effective_n(num_seeds, num_seeds_dev);
  if (call_base_dev) call_id += (uint32_t)*call_base_dev;
  const uint32_t cap = INSERT ? relabel_capacity(num_seeds + num_seeds * fanout) : 0u;
  const int sub = threadIdx.x % G;
  const int64_t groups_per_block = blockDim.x / G;
  int64_t j = (int64_t)blockIdx.x * groups_per_block + threadIdx.x / G;
  const int64_t stride = (int64_t)gridDim.x * groups_per_block;
  int flags = 0;
  for (; j < num_seeds; j += stride) {
    const int64_t v = seeds[j];
    int64_t* orow = out ? out + j * fanout : nullptr;
    const int64_t* nbr = nullptr;
    int64_t deg = 0;
    if (v < 0 || v >= num_nodes) {
      flags |= APT_FLAG_ID_OUT_OF_RANGE;
    } else {
      int64_t pos = adj_pos_map ? adj_pos_map[v] : (int64_t)(-v - 2);
      const int64_t* indptr;
      const int64_t* indices;
      if (pos >= 0) {
        indptr = dev_indptr;
        indices = dev_indices;
      } else {
        pos = -pos - 2;
        indptr = uva_indptr;
        indices = uva_indices;
      }
      const int64_t start = indptr[pos];
      deg = indptr[pos + 1] - start;
      if (deg <= 0) flags |= APT_FLAG_ZERO_DEGREE;
      nbr = indices + start;
    }
    if (INSERT && sub == 0) ins.slot_of[j] = table_insert(ins.slots, cap, v, (uint32_t)j, &flags);
    for (int i = sub; i < fanout; i += G) {
      int64_t u = v;   // a seed that is no node, or has no in-neighbour, fills its row with itself
      if (deg > 0) u = nbr[mod_deg(draw_word((uint64_t)j, (uint32_t)i, call_id, k0, k1), deg)];
      if (orow) orow[i] = u;
      if (INSERT) {
        const int64_t item = num_seeds + j * fanout + i;
        ins.slot_of[item] = table_insert(ins.slots, cap, u, (uint32_t)item, &flags);
      }
    }
  }
  if (flags) atomicOr(status, flags);
}

// Without replacement (fanout <= 32): one warp per seed. Lane i ends up holding
// the edge slot of output i. Floyd's selection: for step i, t = deg-fanout+i,
// r = draw(j,i) % (t+1); take r unless an earlier step already took it, then
// take t. Every lane evaluates the same r, the lanes that own earlier picks
// vote on the collision.
__global__ void __launch_bounds__(256)
sample_floyd_kernel(const int64_t* __restrict__ seeds, int64_t num_seeds,
                    const int64_t* __restrict__ num_seeds_dev, int fanout, const int64_t* __restrict__ adj_pos_map,
                    int64_t num_nodes, const int64_t* __restrict__ dev_indptr,
                    const int64_t* __restrict__ dev_indices,
                    const int64_t* __restrict__ uva_indptr,
                    const int64_t* __restrict__ uva_indices, uint32_t k0,
                    uint32_t k1, uint32_t call_id, const int64_t* __restrict__ call_base_dev,
                    int64_t* __restrict__ out, int32_t* status) {
  num_seeds = effective_n(num_seeds, num_seeds_dev);
  if (call_base_dev) call_id += (uint32_t)*call_base_dev;
  const int lane = threadIdx.x & 31;
  const int64_t warps_per_block = blockDim.x >> 5;
  int64_t j = (int64_t)blockIdx.x * warps_per_block + (threadIdx.x >> 5);
  const int64_t stride = (int64_t)gridDim.x * warps_per_block;
  int flags = 0;
  for (; j < num_seeds; j += stride) {
    const int64_t v = seeds[j];
    int64_t* orow = out + j * fanout;
    if (v < 0 || v >= num_nodes) {
      flags |= APT_FLAG_ID_OUT_OF_RANGE;
      if (lane < fanout) orow[lane] = v;
      continue;
    }
    int64_t pos = adj_pos_map ? adj_pos_map[v] : (int64_t)(-v - 2);
    const int64_t* indptr;
    const int64_t* indices;
    if (pos >= 0) {
      indptr = dev_indptr;
      indices = dev_indices;
    } else {
      pos = -pos - 2;
      indptr = uva_indptr;
      indices = uva_indices;
    }
    const int64_t start = indptr[pos];
    const int64_t deg = indptr[pos + 1] - start;
    if (deg <= 0) {
      flags |= APT_FLAG_ZERO_DEGREE;
      if (lane < fanout) orow[lane] = v;
      continue;
    }
    const int64_t* nbr = indices + start;
    int64_t pick = -1;
    if (deg <= fanout) {
      if (lane < deg) {
        pick = lane;
      } else if (lane < fanout) {
        pick = mod_deg(draw_word((uint64_t)j, (uint32_t)lane, call_id, k0, k1), deg);
      }
    } else {
      for (int i = 0; i < fanout; ++i) {
        const int64_t t = deg - fanout + i;
        const int64_t r =
            mod_deg(draw_word((uint64_t)j, (uint32_t)i, call_id, k0, k1), t + 1);
        const unsigned taken = __ballot_sync(0xffffffffu, lane < i && pick == r);
        if (lane == i) pick = taken ? t : r;
      }
    }
    if (lane < fanout) orow[lane] = nbr[pick];
  }
  if (flags) atomicOr(status, flags);
}

}  // namespace apt
