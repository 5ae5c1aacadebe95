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

// The CSC as the sampler sees it: rows of the cached part (dev_*) or of the global graph (uva_*),
// chosen per node by adj_pos_map (NULL: every node reads the global graph).
struct CscView {
  const int64_t* adj_pos_map;
  int64_t num_nodes;
  const int64_t* dev_indptr;
  const int64_t* dev_indices;
  const int64_t* uva_indptr;
  const int64_t* uva_indices;
};

// In-neighbour list of node v: returns its length (0 with a flag for a seed that is no node or
// has no in-neighbour) and points *nbr at it.
__device__ __forceinline__ int64_t csc_row(const CscView& g, int64_t v, const int64_t** nbr, int* flags) {
  if (v < 0 || v >= g.num_nodes) {
    *flags |= APT_FLAG_ID_OUT_OF_RANGE;
    return 0;
  }
  int64_t pos = g.adj_pos_map ? g.adj_pos_map[v] : (int64_t)(-v - 2);
  const int64_t* indptr;
  const int64_t* indices;
  if (pos >= 0) {
    indptr = g.dev_indptr;
    indices = g.dev_indices;
  } else {
    pos = -pos - 2;
    indptr = g.uva_indptr;
    indices = g.uva_indices;
  }
  const int64_t start = indptr[pos];
  const int64_t deg = indptr[pos + 1] - start;
  if (deg <= 0) {
    *flags |= APT_FLAG_ZERO_DEGREE;
    return 0;
  }
  *nbr = indices + start;
  return deg;
}

struct SampleInsert {
  Slot* slots;        // relabel table (INSERT only)
  int32_t* slot_of;   // [S + S * fanout] slot of every item
};

template <int G, bool INSERT>
__global__ void __launch_bounds__(256)
sample_replace_kernel(const int64_t* __restrict__ seeds, int64_t num_seeds,
                      const int64_t* __restrict__ num_seeds_dev, int fanout, CscView g, uint32_t k0,
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
    const int64_t deg = csc_row(g, v, &nbr, &flags);
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

}  // namespace apt
