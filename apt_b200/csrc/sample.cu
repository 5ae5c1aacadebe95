// Entry point of the fanout sampler (kernels in sample_kernels.cuh).
#include "sample_kernels.cuh"


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
               num_seeds_dev, fanout, adj_pos_map, num_nodes, dev_indptr, dev_indices,        \
               uva_indptr, uva_indices, k0, k1, call_id, call_id_base_dev,     \
               out_neighbors, status_word, SampleInsert{nullptr, nullptr});          \
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
