// Virtual nodes of the SNP strategy for SAGE / GCN: a neighbour sampled for
// local destination j and owned by rank o becomes the virtual node (o, j);
// the owner aggregates its neighbours per virtual node before anything
// crosses a link. This file holds the id arithmetic around that exchange.
#include "common.cuh"

namespace apt {

__global__ void __launch_bounds__(256)
k_src_to_vir(const int64_t* __restrict__ dst, int64_t num_dst, const int64_t* __restrict__ src,
             int64_t num_src, int64_t fanout, const int64_t* __restrict__ min_vids, OwnerParams p,
             int with_dst, int64_t* __restrict__ out) {
  __shared__ int64_t mv[kMaxRanks + 1];
  if (threadIdx.x <= p.world_size) mv[threadIdx.x] = min_vids[threadIdx.x];
  __syncthreads();
  const int64_t head = with_dst ? num_dst : 0;
  const int64_t total = head + num_src;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
    int64_t v, offset;
    if (i < head) {
      v = dst[i];
      offset = i;
    } else {
      const int64_t k = i - head;
      v = src[k];
      offset = (with_dst ? (int64_t)p.world_size * num_dst : 0) + k / fanout;
    }
    out[i] = (int64_t)owner_of(v, mv, p) * num_dst + offset;
  }
}

__device__ __forceinline__ int64_t lower_bound_of(const int64_t* __restrict__ a, int64_t n, int64_t v) {
  int64_t lo = 0, hi = n;
  while (lo < hi) {
    const int64_t mid = (lo + hi) >> 1;
    if (a[mid] < v) lo = mid + 1; else hi = mid;
  }
  return lo;
}

// One block. Thread t < K+1 (K = ws or 2 ws) searches base * t in the sorted
// virtual ids, the next ws threads search base * (K - ws + 1 + t') in the unique
// ones; the differences are then laid out receiver-major: (ids, uniques) or
// (destinations, ids, uniques) per receiver.
__global__ void __launch_bounds__(128)
k_vir_send_sizes(const int64_t* __restrict__ sorted_nodes, int64_t num_sorted,
                 const int64_t* __restrict__ num_sorted_dev,
                 const int64_t* __restrict__ unique_nodes, int64_t num_unique,
                 const int64_t* __restrict__ num_unique_dev, int ws, int64_t base,
                 const int64_t* __restrict__ base_dev, int with_dst,
                 int64_t* __restrict__ out_offset, int64_t* __restrict__ out_sizes) {
  __shared__ int64_t off[3 * kMaxRanks + 1];
  const int K = with_dst ? 2 * ws : ws;
  const int total = K + 1 + ws;
  num_sorted = effective_n(num_sorted, num_sorted_dev);
  num_unique = effective_n(num_unique, num_unique_dev);
  if (base_dev) base = *base_dev;
  for (int t = threadIdx.x; t < total; t += blockDim.x) {
    if (t <= K) off[t] = lower_bound_of(sorted_nodes, num_sorted, base * t);
    else off[t] = lower_bound_of(unique_nodes, num_unique, base * (int64_t)(K - ws + (t - K)));
    if (out_offset) out_offset[t] = off[t];
  }
  __syncthreads();
  const int k = with_dst ? 3 : 2;
  for (int t = threadIdx.x; t < k * ws; t += blockDim.x) {
    const int r = t / k, i = t % k;
    const int j = i * ws + r;            // index into the differences, field-major
    int64_t v;
    if (j == K) v = off[K + 1];          // uniques of receiver 0 start at zero
    else v = off[j + 1] - off[j];
    out_sizes[t] = v;
  }
}

__global__ void __launch_bounds__(256)
k_sp_pack(const int64_t* __restrict__ sorted_vir, const int64_t* __restrict__ sorted_ids, int64_t n,
          int64_t num_dst, int64_t rank_term, int64_t num_total_nodes, int64_t* __restrict__ out) {
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
    out[i] = rank_term + (sorted_vir[i] % num_dst) * num_total_nodes + sorted_ids[i];
}

__global__ void __launch_bounds__(256)
k_sp_unpack(const int64_t* __restrict__ packed, int64_t n, const int64_t* __restrict__ n_dev,
            int64_t num_total_nodes, int64_t* __restrict__ out_vir, int64_t* __restrict__ out_ori) {
  n = effective_n(n, n_dev);
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    const int64_t v = packed[i];
    const int64_t q = v / num_total_nodes;
    out_vir[i] = q;
    out_ori[i] = v - q * num_total_nodes;
  }
}

// The whole sender side of the virtual-node hop in one pass over the neighbours:
// neighbour i (of destination i / fanout) has been given slot pos[i] by the stable owner
// bucketing; its virtual id owner * num_dst + i / fanout and its packed triple
// (sender, destination index, neighbour id) are written to that slot, which is the
// order a stable sort of the virtual ids yields. num_dst may come from a device word
// (what the previous relabelling produced); the number of neighbours is then
// num_dst * fanout and is left in out_count for the kernels that follow.
__global__ void __launch_bounds__(256)
k_sp_map_place_pack(const int64_t* __restrict__ nbr, const int64_t* __restrict__ pos, int64_t num_dst,
                    const int64_t* __restrict__ num_dst_dev, int64_t fanout,
                    const int64_t* __restrict__ min_vids, OwnerParams p, int64_t rank_term,
                    int64_t num_total_nodes, int64_t* __restrict__ sorted_vir,
                    int64_t* __restrict__ packed, int64_t* __restrict__ out_count) {
  __shared__ int64_t mv[kMaxRanks + 1];
  if (threadIdx.x <= p.world_size) mv[threadIdx.x] = min_vids[threadIdx.x];
  __syncthreads();
  num_dst = effective_n(num_dst, num_dst_dev);
  const int64_t n = num_dst * fanout;
  if (out_count && blockIdx.x == 0 && threadIdx.x == 0) *out_count = n;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    const int64_t v = nbr[i];
    const int64_t d = i / fanout;
    const int64_t slot = pos[i];
    sorted_vir[slot] = (int64_t)owner_of(v, mv, p) * num_dst + d;
    packed[slot] = rank_term + d * num_total_nodes + v;
  }
}

static int check_owner_args(const char* who, int world_size, int shuffle_id_offset, int rank,
                            int node_beg, int node_end) {
  APT_CHECK_ARG(world_size >= 1 && world_size <= kMaxRanks, "%s: world_size %d outside [1,%d]", who,
                world_size, kMaxRanks);
  APT_CHECK_ARG(rank >= 0 && rank < world_size && shuffle_id_offset >= 0 && shuffle_id_offset < world_size &&
                    node_beg >= 0 && node_beg <= node_end,
                "%s: rank/offset outside the world", who);
  return APT_OK;
}

}  // namespace apt

extern "C" int apt_src_to_vir(const int64_t* src, int64_t num_src, int64_t fanout, int64_t num_dst,
                              const int64_t* min_vids, int world_size, int shuffle_id_offset, int rank,
                              int node_beg, int node_end, int64_t* out_vir, void* stream) {
  using namespace apt;
  if (int rc = check_owner_args("apt_src_to_vir", world_size, shuffle_id_offset, rank, node_beg, node_end)) return rc;
  APT_CHECK_ARG(num_src >= 0 && fanout >= 1 && num_dst >= 0, "apt_src_to_vir: bad sizes");
  if (num_src == 0) return APT_OK;
  APT_CHECK_ARG(src && min_vids && out_vir, "apt_src_to_vir: null pointer");
  cudaStream_t s = (cudaStream_t)stream;
  ProfScope prof("src_to_vir", s);
  OwnerParams p{world_size, shuffle_id_offset, rank, node_beg, node_end};
  APT_LAUNCH(k_src_to_vir, wave_grid(ceil_div(num_src, 256), 8), 256, 0, s, nullptr, num_dst, src, num_src,
             fanout, min_vids, p, 0, out_vir);
  return APT_OK;
}

extern "C" int apt_srcdst_to_vir(const int64_t* dst, int64_t num_dst, const int64_t* src, int64_t num_src,
                                 int64_t fanout, const int64_t* min_vids, int world_size,
                                 int shuffle_id_offset, int rank, int node_beg, int node_end,
                                 int64_t* out_vir, void* stream) {
  using namespace apt;
  if (int rc = check_owner_args("apt_srcdst_to_vir", world_size, shuffle_id_offset, rank, node_beg, node_end))
    return rc;
  APT_CHECK_ARG(num_src >= 0 && fanout >= 1 && num_dst >= 0, "apt_srcdst_to_vir: bad sizes");
  if (num_src + num_dst == 0) return APT_OK;
  APT_CHECK_ARG((dst || num_dst == 0) && (src || num_src == 0) && min_vids && out_vir,
                "apt_srcdst_to_vir: null pointer");
  cudaStream_t s = (cudaStream_t)stream;
  ProfScope prof("src_to_vir", s);
  OwnerParams p{world_size, shuffle_id_offset, rank, node_beg, node_end};
  APT_LAUNCH(k_src_to_vir, wave_grid(ceil_div(num_src + num_dst, 256), 8), 256, 0, s, dst, num_dst, src,
             num_src, fanout, min_vids, p, 1, out_vir);
  return APT_OK;
}

extern "C" int apt_vir_send_sizes(const int64_t* sorted_nodes, int64_t num_sorted,
                                  const int64_t* num_sorted_dev, const int64_t* unique_nodes,
                                  int64_t num_unique, const int64_t* num_unique_dev, int world_size,
                                  int64_t base, const int64_t* base_dev, int with_dst,
                                  int64_t* out_send_offset, int64_t* out_send_sizes, void* stream) {
  using namespace apt;
  APT_CHECK_ARG(world_size >= 1 && world_size <= kMaxRanks, "apt_vir_send_sizes: world_size %d outside [1,%d]",
                world_size, kMaxRanks);
  APT_CHECK_ARG(num_sorted >= 0 && num_unique >= 0 && base >= 0, "apt_vir_send_sizes: bad sizes");
  APT_CHECK_ARG(out_send_sizes && (sorted_nodes || num_sorted == 0) && (unique_nodes || num_unique == 0),
                "apt_vir_send_sizes: null pointer");
  cudaStream_t s = (cudaStream_t)stream;
  ProfScope prof("vir_send_sizes", s);
  APT_LAUNCH(k_vir_send_sizes, 1, 128, 0, s, sorted_nodes, num_sorted, num_sorted_dev, unique_nodes, num_unique,
             num_unique_dev, world_size, base, base_dev, with_dst ? 1 : 0, out_send_offset, out_send_sizes);
  return APT_OK;
}

extern "C" int apt_sp_pack_frontier(const int64_t* sorted_vir, const int64_t* sorted_ids, int64_t n,
                                    int64_t num_dst, int rank, int64_t sp_base, int64_t num_total_nodes,
                                    int64_t* out, void* stream) {
  using namespace apt;
  APT_CHECK_ARG(n >= 0 && num_dst >= 0 && rank >= 0 && sp_base > 0 && num_total_nodes > 0,
                "apt_sp_pack_frontier: bad sizes");
  APT_CHECK_ARG(num_dst <= sp_base, "apt_sp_pack_frontier: %lld destinations exceed sp_base %lld",
                (long long)num_dst, (long long)sp_base);
  // (rank + 1) * sp_base * num_total_nodes has to fit 63 bits
  APT_CHECK_ARG((double)(rank + 1) * (double)sp_base * (double)num_total_nodes < 9.2e18,
                "apt_sp_pack_frontier: packed id overflows 63 bits");
  if (n == 0) return APT_OK;
  APT_CHECK_ARG(sorted_vir && sorted_ids && out && num_dst > 0, "apt_sp_pack_frontier: null pointer");
  cudaStream_t s = (cudaStream_t)stream;
  ProfScope prof("sp_pack", s);
  APT_LAUNCH(k_sp_pack, wave_grid(ceil_div(n, 256), 8), 256, 0, s, sorted_vir, sorted_ids, n, num_dst,
             (int64_t)rank * sp_base * num_total_nodes, num_total_nodes, out);
  return APT_OK;
}

extern "C" int apt_sp_unpack_frontier(const int64_t* packed, int64_t n, const int64_t* n_dev,
                                      int64_t num_total_nodes, int64_t* out_vir, int64_t* out_ori,
                                      void* stream) {
  using namespace apt;
  APT_CHECK_ARG(n >= 0 && num_total_nodes > 0, "apt_sp_unpack_frontier: bad sizes");
  if (n == 0) return APT_OK;
  APT_CHECK_ARG(packed && out_vir && out_ori, "apt_sp_unpack_frontier: null pointer");
  cudaStream_t s = (cudaStream_t)stream;
  ProfScope prof("sp_unpack", s);
  APT_LAUNCH(k_sp_unpack, wave_grid(ceil_div(n, 256), 8), 256, 0, s, packed, n, n_dev, num_total_nodes, out_vir,
             out_ori);
  return APT_OK;
}

extern "C" int apt_sp_map_place_pack(const int64_t* neighbors, const int64_t* positions, int64_t num_dst,
                                     const int64_t* num_dst_dev, int64_t fanout, const int64_t* min_vids,
                                     int world_size, int shuffle_id_offset, int rank, int node_beg, int node_end,
                                     int64_t sp_base, int64_t num_total_nodes, int64_t* out_sorted_vir,
                                     int64_t* out_packed, int64_t* out_count, void* stream) {
  using namespace apt;
  if (int rc = check_owner_args("apt_sp_map_place_pack", world_size, shuffle_id_offset, rank, node_beg, node_end))
    return rc;
  APT_CHECK_ARG(num_dst >= 0 && fanout >= 1 && sp_base > 0 && num_total_nodes > 0, "apt_sp_map_place_pack: bad sizes");
  APT_CHECK_ARG(num_dst <= sp_base, "apt_sp_map_place_pack: %lld destinations exceed sp_base %lld",
                (long long)num_dst, (long long)sp_base);
  APT_CHECK_ARG((double)(rank + 1) * (double)sp_base * (double)num_total_nodes < 9.2e18,
                "apt_sp_map_place_pack: packed id overflows 63 bits");
  cudaStream_t s = (cudaStream_t)stream;
  if (num_dst == 0) {
    if (out_count) APT_CUDA(cudaMemsetAsync(out_count, 0, 8, s));
    return APT_OK;
  }
  APT_CHECK_ARG(neighbors && positions && min_vids && out_sorted_vir && out_packed,
                "apt_sp_map_place_pack: null pointer");
  ProfScope prof("sp_map_place_pack", s);
  OwnerParams p{world_size, shuffle_id_offset, rank, node_beg, node_end};
  APT_LAUNCH(k_sp_map_place_pack, wave_grid(ceil_div(num_dst * fanout, 256), 8), 256, 0, s, neighbors, positions,
             num_dst, num_dst_dev, fanout, min_vids, p, (int64_t)rank * sp_base * num_total_nodes, num_total_nodes,
             out_sorted_vir, out_packed, out_count);
  return APT_OK;
}
