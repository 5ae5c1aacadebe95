// Access-frequency counters of the dry run and what the cache policy derives
// from them: the node order by falling frequency and the share of accesses a
// cache of the k hottest nodes would serve.
#include <cub/cub.cuh>

#include "common.cuh"

namespace apt {

__global__ void __launch_bounds__(256)
k_hotness_add(const int64_t* __restrict__ ids, int64_t n, const int64_t* __restrict__ n_dev,
              int32_t* __restrict__ counters, int64_t num_nodes, int32_t* status) {
  n = effective_n(n, n_dev);
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  bool bad = false;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    const int64_t v = ids[i];
    if (v < 0 || v >= num_nodes) {
      bad = true;
      continue;
    }
    atomicAdd(counters + v, 1);
  }
  if (bad) atomicOr(status, APT_FLAG_ID_OUT_OF_RANGE);
}

// Key = (2^32 - 1 - count) in the high word, node id in the low word: ascending keys
// are falling counts, ties by rising id.
__global__ void __launch_bounds__(256)
k_hot_keys(const int32_t* __restrict__ counters, int64_t n, uint64_t* __restrict__ keys) {
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
    keys[i] = ((uint64_t)(0xFFFFFFFFu - (uint32_t)counters[i]) << 32) | (uint64_t)i;
}

__global__ void __launch_bounds__(256)
k_hot_ids(const uint64_t* __restrict__ keys, int64_t n, int64_t* __restrict__ out) {
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
    out[i] = (int64_t)(keys[i] & 0xFFFFFFFFull);
}

// out[0] += sum of counters, out[1] += sum of counters[sorted_idx[0 .. num_cache)]
__global__ void __launch_bounds__(256)
k_cached_access(const int32_t* __restrict__ counters, int64_t n, const int64_t* __restrict__ sorted_idx,
                int64_t num_cache, unsigned long long* __restrict__ out) {
  typedef cub::BlockReduce<unsigned long long, 256> Reduce;
  __shared__ typename Reduce::TempStorage tmp_a, tmp_b;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  unsigned long long total = 0, cached = 0;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    total += (unsigned long long)(uint32_t)counters[i];
    if (i < num_cache) {
      const int64_t v = sorted_idx[i];
      if (v >= 0 && v < n) cached += (unsigned long long)(uint32_t)counters[v];
    }
  }
  total = Reduce(tmp_a).Sum(total);
  cached = Reduce(tmp_b).Sum(cached);
  if (threadIdx.x == 0) {
    atomicAdd(out, total);
    atomicAdd(out + 1, cached);
  }
}

static size_t hot_order_layout(int64_t n, size_t* sort_bytes) {
  size_t temp = 0;
  cub::DeviceRadixSort::SortKeys(nullptr, temp, (const uint64_t*)nullptr, (uint64_t*)nullptr, n > 0 ? n : 1, 0, 64);
  if (sort_bytes) *sort_bytes = temp;
  return 2 * align_up((size_t)(n > 0 ? n : 1) * 8, 256) + align_up(temp, 256);
}

}  // namespace apt

extern "C" int apt_hotness_add(const int64_t* ids, int64_t n, const int64_t* n_dev, int32_t* counters,
                               int64_t num_nodes, int32_t* status_word, void* stream) {
  using namespace apt;
  APT_CHECK_ARG(n >= 0 && num_nodes > 0 && counters && status_word, "apt_hotness_add: bad argument");
  if (n == 0) return APT_OK;
  APT_CHECK_ARG(ids, "apt_hotness_add: null ids");
  cudaStream_t s = (cudaStream_t)stream;
  ProfScope prof("hotness_add", s);
  APT_LAUNCH(k_hotness_add, wave_grid(ceil_div(n, 256), 8), 256, 0, s, ids, n, n_dev, counters, num_nodes,
             status_word);
  return APT_OK;
}

extern "C" size_t apt_hot_order_workspace_bytes(int64_t num_nodes) {
  if (num_nodes < 0) return 0;
  return apt::hot_order_layout(num_nodes, nullptr);
}

extern "C" int apt_hot_order(const int32_t* counters, int64_t num_nodes, void* workspace, size_t workspace_bytes,
                             int64_t* out_sorted_idx, void* stream) {
  using namespace apt;
  APT_CHECK_ARG(num_nodes >= 0 && num_nodes < ((int64_t)1 << 32), "apt_hot_order: bad num_nodes");
  if (num_nodes == 0) return APT_OK;
  APT_CHECK_ARG(counters && workspace && out_sorted_idx, "apt_hot_order: null pointer");
  APT_CHECK_ARG(((uintptr_t)workspace & 255) == 0, "apt_hot_order: workspace must be 256-byte aligned");
  size_t sort_bytes = 0;
  const size_t need = hot_order_layout(num_nodes, &sort_bytes);
  if (workspace_bytes < need) {
    set_error("apt_hot_order: workspace %zu < %zu bytes", workspace_bytes, need);
    return APT_ERR_CAPACITY;
  }
  cudaStream_t s = (cudaStream_t)stream;
  const size_t half = align_up((size_t)num_nodes * 8, 256);
  uint64_t* keys_in = (uint64_t*)workspace;
  uint64_t* keys_out = (uint64_t*)((char*)workspace + half);
  void* temp = (char*)workspace + 2 * half;
  const int grid = wave_grid(ceil_div(num_nodes, 256), 8);
  ProfScope prof("hot_order", s);
  APT_LAUNCH(k_hot_keys, grid, 256, 0, s, counters, num_nodes, keys_in);
  APT_CUDA(cub::DeviceRadixSort::SortKeys(temp, sort_bytes, keys_in, keys_out, num_nodes, 0, 64, s));
  APT_LAUNCH(k_hot_ids, grid, 256, 0, s, keys_out, num_nodes, out_sorted_idx);
  return APT_OK;
}

extern "C" int apt_cached_access(const int32_t* counters, int64_t num_nodes, const int64_t* sorted_idx,
                                 int64_t num_cache, int64_t* out_total_and_cached, void* stream) {
  using namespace apt;
  APT_CHECK_ARG(num_nodes >= 0 && num_cache >= 0 && out_total_and_cached, "apt_cached_access: bad argument");
  cudaStream_t s = (cudaStream_t)stream;
  APT_CUDA(cudaMemsetAsync(out_total_and_cached, 0, 16, s));
  if (num_nodes == 0) return APT_OK;
  APT_CHECK_ARG(counters && (sorted_idx || num_cache == 0), "apt_cached_access: null pointer");
  if (num_cache > num_nodes) num_cache = num_nodes;
  ProfScope prof("cached_access", s);
  APT_LAUNCH(k_cached_access, wave_grid(ceil_div(num_nodes, 256), 8, 2), 256, 0, s, counters, num_nodes, sorted_idx,
             num_cache, (unsigned long long*)out_total_and_cached);
  return APT_OK;
}
