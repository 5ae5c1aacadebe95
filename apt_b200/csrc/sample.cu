// Entry point of the fanout sampler (kernels in sample_kernels.cuh).
#include "sample_kernels.cuh"

namespace apt {

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


extern "C" int apt_sample_csc_fanout(
    const int64_t* seeds, int64_t num_seeds, const int64_t* num_seeds_dev, int fanout,
    const int64_t* adj_pos_map, int64_t num_nodes, const int64_t* dev_indptr,
    const int64_t* dev_indices, const int64_t* uva_indptr,
    const int64_t* uva_indices, uint64_t key, uint32_t call_id,
    const int64_t* call_id_base_dev, int replace, int64_t* out_neighbors,
    int32_t* status_word, void* stream) {
  using namespace apt;
  APT_CHECK_ARG(num_seeds >= 0 && fanout > 0 && num_nodes >= 0,
                "apt_sample_csc_fanout: bad sizes (seeds %lld fanout %d)",
                (long long)num_seeds, fanout);
  if (num_seeds == 0) return APT_OK;
  APT_CHECK_ARG(seeds && out_neighbors && status_word && uva_indptr && uva_indices,
                "apt_sample_csc_fanout: null pointer");
  APT_CHECK_ARG(replace || fanout <= 32,
                "apt_sample_csc_fanout: selection without replacement needs fanout <= 32");
  cudaStream_t s = (cudaStream_t)stream;
  const uint32_t k0 = (uint32_t)key, k1 = (uint32_t)(key >> 32);
  const CscView g{adj_pos_map, num_nodes, dev_indptr, dev_indices, uva_indptr, uva_indices};
  ProfScope prof("sample", s);
  if (!replace) {
    const int grid = wave_grid(ceil_div(num_seeds, 8), 8);
    APT_LAUNCH(sample_floyd_kernel, grid, 256, 0, s, seeds, num_seeds, num_seeds_dev, fanout,
               adj_pos_map, num_nodes, dev_indptr, dev_indices, uva_indptr,
               uva_indices, k0, k1, call_id, call_id_base_dev, out_neighbors, status_word);
    return APT_OK;
  }
#define APT_SAMPLE_G(G)                                                        \
  do {                                                                         \
    const int grid = wave_grid(ceil_div(num_seeds, 256 / G), 8);               \
    APT_LAUNCH((sample_replace_kernel<G, false>), grid, 256, 0, s, seeds, num_seeds,    \
               num_seeds_dev, fanout, g, k0, k1, call_id, call_id_base_dev,    \
               out_neighbors, status_word, SampleInsert{nullptr, nullptr});    \
  } while (0)
  if (fanout <= 8) {
    APT_SAMPLE_G(8);
  } else if (fanout <= 16) {
    APT_SAMPLE_G(16);
  } else {
    APT_SAMPLE_G(32);
  }
#undef APT_SAMPLE_G
  return APT_OK;
}
