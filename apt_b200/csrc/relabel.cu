// Relabelling of a sampled layer: unique of cat(seeds, neighbours) in order of
// first occurrence, and the new id of every neighbour.
//
// One open-addressing table (linear probing, load <= 2/3) in the caller's
// workspace holds, per distinct id, the smallest position at which it occurs.
// An item is a "first occurrence" iff that minimum equals its own position;
// an ordered compaction (block counts -> one-block scan -> in-block scan) turns
// the first-occurrence flags into new ids, which makes the result independent
// of the table layout and of thread scheduling.
//
//   k_clear    empties the slots this call will use
//   k_insert   items -> table (CAS on the key, atomicMin on the position),
//              remembers each item's slot
//   k_count    per-block number of first occurrences
//   k_scan     exclusive scan of the block counts, writes U
//   k_assign   new id = block offset + in-block rank; writes unique[] and the
//              slot's new id
//   k_relabel  neighbours -> new id through the remembered slot
#include "common.cuh"

namespace apt {

constexpr int kRelabelBlock = 1024;

struct RelabelWs {
  int64_t* keys;     // [cap] -1 = empty
  int32_t* min_pos;  // [cap] 0x7f7f7f7f = none yet
  int32_t* new_id;   // [cap]
  int32_t* slot_of;  // [n]
  int32_t* block_sums;  // [nblocks + 1]
  uint32_t cap;      // capacity for the host-side (upper bound) item count
  int nblocks;
};

// Problem size as the kernels see it. With device-side counts the number of
// seeds comes from a device word and every seed brings `per_seed` neighbours;
// the table then only uses the capacity the real item count needs, so clearing
// and probing cost what the real size costs, not what the upper bound would.
struct RelabelDims {
  int64_t S, n;
  uint32_t cap;
};

__host__ __device__ inline uint32_t relabel_capacity(int64_t n) {
  return (uint32_t)(n + n / 2 + 64);
}

__device__ __forceinline__ RelabelDims relabel_dims(int64_t S_host, int64_t M_host,
                                                    const int64_t* S_dev, int64_t per_seed) {
  RelabelDims d;
  if (S_dev) {
    d.S = effective_n(S_host, S_dev);
    d.n = d.S + d.S * per_seed;
  } else {
    d.S = S_host;
    d.n = S_host + M_host;
  }
  d.cap = relabel_capacity(d.n);
  return d;
}

static size_t relabel_layout(int64_t n, char* base, RelabelWs* ws) {
  const uint32_t cap = relabel_capacity(n);
  const int nblocks = (int)ceil_div(n > 0 ? n : 1, kRelabelBlock);
  size_t off = 0;
  auto take = [&](size_t bytes) {
    size_t o = off;
    off = align_up(off + bytes, 256);
    return o;
  };
  const size_t o_keys = take((size_t)cap * 8);
  const size_t o_min = take((size_t)cap * 4);
  const size_t o_new = take((size_t)cap * 4);
  const size_t o_slot = take((size_t)(n > 0 ? n : 1) * 4);
  const size_t o_sums = take((size_t)(nblocks + 1) * 4);
  if (ws) {
    ws->keys = (int64_t*)(base + o_keys);
    ws->min_pos = (int32_t*)(base + o_min);
    ws->new_id = (int32_t*)(base + o_new);
    ws->slot_of = (int32_t*)(base + o_slot);
    ws->block_sums = (int32_t*)(base + o_sums);
    ws->cap = cap;
    ws->nblocks = nblocks;
  }
  return off;
}

__device__ __forceinline__ uint32_t hash_id(int64_t key) {
  // 64 -> 32 bit finaliser (splitmix64 constants); ids are often dense, so the
  // low bits alone would cluster under linear probing.
  uint64_t x = (uint64_t)key;
  x ^= x >> 30; x *= 0xbf58476d1ce4e5b9ull;
  x ^= x >> 27; x *= 0x94d049bb133111ebull;
  x ^= x >> 31;
  return (uint32_t)x;
}

__device__ __forceinline__ int64_t item_at(const int64_t* seeds, int64_t S,
                                           const int64_t* nbrs, int64_t i) {
  return i < S ? seeds[i] : nbrs[i - S];
}

// Empties the slots the real item count will use (keys = -1, min_pos = none).
__global__ void __launch_bounds__(256)
k_clear(int64_t S_host, int64_t M_host, const int64_t* __restrict__ S_dev, int64_t per_seed,
        RelabelWs ws) {
  const RelabelDims d = relabel_dims(S_host, M_host, S_dev, per_seed);
  // two keys per 16-byte store; cap is rounded up to even inside the padded arrays
  const int64_t pairs = ((int64_t)d.cap + 1) / 2;
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (; i < pairs; i += stride) {
    ((uint4*)ws.keys)[i] = make_uint4(0xffffffffu, 0xffffffffu, 0xffffffffu, 0xffffffffu);
    ((uint2*)ws.min_pos)[i] = make_uint2(0x7f7f7f7fu, 0x7f7f7f7fu);
  }
}

__global__ void __launch_bounds__(kRelabelBlock)
k_insert(const int64_t* __restrict__ seeds, int64_t S_host, const int64_t* __restrict__ nbrs,
         int64_t M_host, const int64_t* __restrict__ S_dev, int64_t per_seed, RelabelWs ws,
         int32_t* status) {
  const RelabelDims d = relabel_dims(S_host, M_host, S_dev, per_seed);
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= d.n) return;
  const int64_t key = item_at(seeds, d.S, nbrs, i);
  uint32_t pos = (uint32_t)(((uint64_t)hash_id(key) * d.cap) >> 32);
  unsigned long long* keys = (unsigned long long*)ws.keys;
  for (uint32_t probe = 0; probe < d.cap; ++probe) {
    unsigned long long prev = keys[pos];
    if (prev == ~0ull) prev = atomicCAS(keys + pos, ~0ull, (unsigned long long)key);
    if (prev == ~0ull || prev == (unsigned long long)key) {
      atomicMin(ws.min_pos + pos, (int32_t)i);
      ws.slot_of[i] = (int32_t)pos;
      return;
    }
    pos = pos + 1 == d.cap ? 0 : pos + 1;
  }
  ws.slot_of[i] = -1;
  atomicOr(status, APT_FLAG_TABLE_FULL);
}

__device__ __forceinline__ int is_first(const RelabelWs& ws, int64_t i, int64_t n) {
  if (i >= n) return 0;
  const int32_t slot = ws.slot_of[i];
  return slot >= 0 && ws.min_pos[slot] == (int32_t)i;
}

__global__ void __launch_bounds__(kRelabelBlock)
k_count(int64_t S_host, int64_t M_host, const int64_t* __restrict__ S_dev, int64_t per_seed,
        RelabelWs ws) {
  const RelabelDims d = relabel_dims(S_host, M_host, S_dev, per_seed);
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int f = is_first(ws, i, d.n);
  const int c = __syncthreads_count(f);
  if (threadIdx.x == 0) ws.block_sums[blockIdx.x] = c;
}

__global__ void __launch_bounds__(kRelabelBlock)
k_assign(const int64_t* __restrict__ seeds, int64_t S_host, const int64_t* __restrict__ nbrs,
         int64_t M_host, const int64_t* __restrict__ S_dev, int64_t per_seed, RelabelWs ws,
         int64_t* __restrict__ out_unique) {
  __shared__ int warp_sums[33];
  const RelabelDims d = relabel_dims(S_host, M_host, S_dev, per_seed);
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int f = is_first(ws, i, d.n);
  int total;
  const int ex = block_exclusive_scan(f, warp_sums, &total);
  if (f) {
    const int32_t id = ws.block_sums[blockIdx.x] + ex;
    out_unique[id] = item_at(seeds, d.S, nbrs, i);
    ws.new_id[ws.slot_of[i]] = id;
  }
}

__global__ void __launch_bounds__(256)
k_relabel(int64_t S_host, int64_t M_host, const int64_t* __restrict__ S_dev, int64_t per_seed,
          RelabelWs ws, int64_t* __restrict__ out) {
  const RelabelDims d = relabel_dims(S_host, M_host, S_dev, per_seed);
  const int64_t M = d.n - d.S;
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (; i < M; i += stride) {
    const int32_t slot = ws.slot_of[d.S + i];
    out[i] = slot >= 0 ? (int64_t)ws.new_id[slot] : -1;
  }
}

}  // namespace apt

extern "C" size_t apt_relabel_workspace_bytes(int64_t num_items) {
  if (num_items < 0) return 0;
  return apt::relabel_layout(num_items, nullptr, nullptr);
}

extern "C" int apt_relabel_csc(const int64_t* seeds, int64_t num_seeds,
                               const int64_t* num_seeds_dev, const int64_t* neighbors,
                               int64_t num_neighbors, void* workspace, size_t workspace_bytes,
                               int64_t* out_unique, int64_t* out_relabeled,
                               int64_t* out_num_unique, int32_t* status_word, void* stream) {
  using namespace apt;
  APT_CHECK_ARG(num_seeds >= 0 && num_neighbors >= 0, "apt_relabel_csc: negative size");
  const int64_t n = num_seeds + num_neighbors;
  APT_CHECK_ARG(n < (int64_t)0x7f000000, "apt_relabel_csc: %lld items exceed the 31-bit position range",
                (long long)n);
  APT_CHECK_ARG(out_num_unique && status_word, "apt_relabel_csc: null output word");
  int64_t per_seed = 0;
  if (num_seeds_dev) {
    APT_CHECK_ARG(num_seeds > 0 && num_neighbors % num_seeds == 0,
                  "apt_relabel_csc: with a device-side seed count the neighbours must be a fixed number per seed");
    per_seed = num_neighbors / num_seeds;
  }
  cudaStream_t s = (cudaStream_t)stream;
  if (n == 0) {
    APT_CUDA(cudaMemsetAsync(out_num_unique, 0, sizeof(int64_t), s));
    return APT_OK;
  }
  APT_CHECK_ARG((num_seeds == 0 || seeds) && (num_neighbors == 0 || (neighbors && out_relabeled)) &&
                    out_unique && workspace,
                "apt_relabel_csc: null pointer");
  APT_CHECK_ARG(((uintptr_t)workspace & 255) == 0, "apt_relabel_csc: workspace must be 256-byte aligned");
  RelabelWs ws;
  const size_t need = relabel_layout(n, (char*)workspace, &ws);
  if (workspace_bytes < need) {
    set_error("apt_relabel_csc: workspace %zu < %zu bytes", workspace_bytes, need);
    return APT_ERR_CAPACITY;
  }
  ProfScope prof("relabel", s);
  {
    const int grid = wave_grid(ceil_div(((int64_t)ws.cap + 1) / 2, 256), 8, 2);
    APT_LAUNCH(k_clear, grid, 256, 0, s, num_seeds, num_neighbors, num_seeds_dev, per_seed, ws);
  }
  APT_LAUNCH(k_insert, ws.nblocks, kRelabelBlock, 0, s, seeds, num_seeds, neighbors, num_neighbors,
             num_seeds_dev, per_seed, ws, status_word);
  APT_LAUNCH(k_count, ws.nblocks, kRelabelBlock, 0, s, num_seeds, num_neighbors, num_seeds_dev, per_seed, ws);
  APT_LAUNCH(k_scan_blocks, 1, 1024, 0, s, ws.block_sums, ws.nblocks, out_num_unique);
  APT_LAUNCH(k_assign, ws.nblocks, kRelabelBlock, 0, s, seeds, num_seeds, neighbors, num_neighbors,
             num_seeds_dev, per_seed, ws, out_unique);
  if (num_neighbors > 0) {
    const int grid = wave_grid(ceil_div(num_neighbors, 256), 8);
    APT_LAUNCH(k_relabel, grid, 256, 0, s, num_seeds, num_neighbors, num_seeds_dev, per_seed, ws,
               out_relabeled);
  }
  return APT_OK;
}
