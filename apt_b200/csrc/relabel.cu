// Relabelling of a sampled layer: unique of cat(seeds, neighbours) in order of
// first occurrence, and the new id of every neighbour.
//
// One open-addressing table (linear probing, load <= 2/3) in the caller's
// workspace holds, per distinct id, the smallest position at which it occurs.
// An item is a "first occurrence" iff that minimum equals its own position;
// an ordered compaction (per-tile counts, then each tile sums the counts of the
// tiles before it) turns the first-occurrence flags into new ids, which makes
// the result independent of the table layout and of thread scheduling.
//
//   k_insert   items -> table (CAS on the key, atomicMin on the position),
//              remembers each item's slot
//   k_count    per-tile number of first occurrences
//   k_assign   new id = offset of the tile + rank inside it; writes unique[],
//              the slot's new id and (last tile) the number of unique ids
//   k_relabel  neighbours -> new id through the remembered slot; every item
//              also empties its slot again
//
// Layers of up to 8192 items run in one block with the table in shared memory
// (k_relabel_small below).
//
// The table is empty between calls (apt_relabel_workspace_init empties it once,
// each call empties the slots it used), so a call costs what its own item count
// costs and no clearing pass is needed.
#include "common.cuh"

namespace apt {

constexpr int kRelabelBlock = 1024;
constexpr unsigned long long kEmptyKey = ~0ull;
constexpr uint32_t kNoPos = 0xffffffffu;

// key, smallest position and new id of one distinct id: 16 bytes, one sector.
struct Slot {
  unsigned long long key;
  uint32_t min_pos;
  uint32_t new_id;
};

struct RelabelWs {
  Slot* slots;          // [cap_ws] all-0xff between calls
  int32_t* slot_of;     // [items_ws]
  int32_t* tile_count;  // [tiles_ws]
  int64_t items_ws;     // items this workspace was sized for
  int tiles;            // tiles of the host-side (upper bound) item count of this call
};

// Problem size as the kernels see it. With device-side counts the number of
// seeds comes from a device word and every seed brings `per_seed` neighbours;
// the table then uses the capacity the real item count needs.
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

static size_t relabel_bytes_for(int64_t items) {
  const int64_t n = items > 0 ? items : 1;
  return align_up((size_t)relabel_capacity(n) * sizeof(Slot), 256) + align_up((size_t)n * 4, 256) +
         align_up((size_t)(ceil_div(n, kRelabelBlock) + 1) * 4, 256);
}

// The layout depends only on the size of the workspace, not on the call, so
// that "empty between calls" holds for one fixed slot region.
static bool relabel_layout(char* base, size_t bytes, RelabelWs* ws) {
  // 16 * 1.5 + 4 bytes per item plus a little: first guess, then shrink until it fits
  int64_t items = bytes > 4096 ? (int64_t)((bytes - 4096) / 281 * 10) : 0;
  while (items > 0 && relabel_bytes_for(items) > bytes) items -= 1 + items / 4096;
  ws->items_ws = items;
  if (items <= 0) return false;
  const size_t o_slot_of = align_up((size_t)relabel_capacity(items) * sizeof(Slot), 256);
  ws->slots = (Slot*)base;
  ws->slot_of = (int32_t*)(base + o_slot_of);
  ws->tile_count = (int32_t*)(base + o_slot_of + align_up((size_t)items * 4, 256));
  return true;
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

__global__ void __launch_bounds__(kRelabelBlock)
k_insert(const int64_t* __restrict__ seeds, int64_t S_host, const int64_t* __restrict__ nbrs,
         int64_t M_host, const int64_t* __restrict__ S_dev, int64_t per_seed, RelabelWs ws,
         int32_t* status) {
  const RelabelDims d = relabel_dims(S_host, M_host, S_dev, per_seed);
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= d.n) return;
  const unsigned long long key = (unsigned long long)item_at(seeds, d.S, nbrs, i);
  uint32_t pos = (uint32_t)(((uint64_t)hash_id((int64_t)key) * d.cap) >> 32);
  for (uint32_t probe = 0; probe < d.cap; ++probe) {
    Slot* s = ws.slots + pos;
    unsigned long long prev = *(volatile unsigned long long*)&s->key;
    if (prev == kEmptyKey) prev = atomicCAS(&s->key, kEmptyKey, key);
    if (prev == kEmptyKey || prev == key) {
      atomicMin(&s->min_pos, (uint32_t)i);
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
  return slot >= 0 && ws.slots[slot].min_pos == (uint32_t)i;
}

__global__ void __launch_bounds__(kRelabelBlock)
k_count(int64_t S_host, int64_t M_host, const int64_t* __restrict__ S_dev, int64_t per_seed,
        RelabelWs ws) {
  const RelabelDims d = relabel_dims(S_host, M_host, S_dev, per_seed);
  // tiles past the real item count (the grid covers the upper bound) have nothing to count,
  // and no tile before them ever reads their count
  if ((int64_t)blockIdx.x * blockDim.x >= d.n) return;
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int f = is_first(ws, i, d.n);
  const int c = __syncthreads_count(f);
  if (threadIdx.x == 0) ws.tile_count[blockIdx.x] = c;
}

__global__ void __launch_bounds__(kRelabelBlock)
k_assign(const int64_t* __restrict__ seeds, int64_t S_host, const int64_t* __restrict__ nbrs,
         int64_t M_host, const int64_t* __restrict__ S_dev, int64_t per_seed, RelabelWs ws,
         int64_t* __restrict__ out_unique, int64_t* __restrict__ out_num_unique) {
  __shared__ int scratch[33];
  const RelabelDims d = relabel_dims(S_host, M_host, S_dev, per_seed);
  const int64_t tile_first = (int64_t)blockIdx.x * blockDim.x;
  if (tile_first >= d.n) {
    // past the real item count; with no item at all the first tile reports zero unique ids
    if (d.n == 0 && blockIdx.x == 0 && threadIdx.x == 0) *out_num_unique = 0;
    return;
  }
  const int before = block_sum_of(ws.tile_count, blockIdx.x, scratch);
  const int64_t i = tile_first + threadIdx.x;
  const int f = is_first(ws, i, d.n);
  int total;
  const int ex = block_exclusive_scan(f, scratch, &total);
  if (f) {
    const int32_t id = before + ex;
    out_unique[id] = item_at(seeds, d.S, nbrs, i);
    ws.slots[ws.slot_of[i]].new_id = (uint32_t)id;
  }
  // the tile that holds the last real item knows the number of unique ids
  if (tile_first + blockDim.x >= d.n && threadIdx.x == 0) *out_num_unique = before + total;
}

__global__ void __launch_bounds__(256)
k_relabel(int64_t S_host, int64_t M_host, const int64_t* __restrict__ S_dev, int64_t per_seed,
          RelabelWs ws, int64_t* __restrict__ out) {
  const RelabelDims d = relabel_dims(S_host, M_host, S_dev, per_seed);
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (; i < d.n; i += stride) {
    const int32_t slot = ws.slot_of[i];
    if (slot < 0) {
      if (i >= d.S) out[i - d.S] = -1;
      continue;
    }
    // one 16-byte load brings the new id and the position of the id's first occurrence
    const uint4 v = ld_plain_16((const uint4*)(ws.slots + slot));
    if (i >= d.S) out[i - d.S] = (int64_t)v.w;
    // Nothing reads keys any more and only the first occurrence itself compares positions:
    // that item empties the slot with one 16-byte store (the new id stays for the others).
    if (v.z == (uint32_t)i) st_plain_16((uint4*)(ws.slots + slot), make_uint4(0xffffffffu, 0xffffffffu, kNoPos, v.w));
  }
}

// ---- small layers: the whole relabelling in one block, table in shared memory ----------
// Up to kSmallItems items (the innermost hops of a mini-batch: 1024 seeds x (1 + 5)) fit a
// table of kSmallCap 16-byte slots in the 227 KB of shared memory of one SM together with
// each item's slot number. One block of 1024 threads then runs the three phases (insert,
// ordered compaction, relabel) with block barriers between them: no global table traffic,
// no clearing, one launch instead of four. The order of first occurrence is decided by
// the minimum position per id exactly as in the multi-block path, so both give the same
// arrays.
static bool g_relabel_small = true;   // apt_set_tunable("relabel_small", 0) forces the multi-block path
void set_relabel_small(bool on) { g_relabel_small = on; }

constexpr int kSmallItems = 8192;
constexpr uint32_t kSmallCap = 12288;
constexpr size_t kSmallSmem = (size_t)kSmallCap * sizeof(Slot) + (size_t)kSmallItems * sizeof(uint16_t);

__global__ void __launch_bounds__(kRelabelBlock)
k_relabel_small(const int64_t* __restrict__ seeds, int64_t S_host, const int64_t* __restrict__ nbrs,
                int64_t M_host, const int64_t* __restrict__ S_dev, int64_t per_seed,
                int64_t* __restrict__ out_unique, int64_t* __restrict__ out_relabeled,
                int64_t* __restrict__ out_num_unique) {
  extern __shared__ __align__(16) unsigned char smem[];
  __shared__ int scratch[33];
  Slot* slots = (Slot*)smem;
  uint16_t* slot_of = (uint16_t*)(smem + (size_t)kSmallCap * sizeof(Slot));
  const RelabelDims d = relabel_dims(S_host, M_host, S_dev, per_seed);
  const int n = (int)d.n;
  for (uint32_t t = threadIdx.x; t < kSmallCap; t += blockDim.x) {
    slots[t].key = kEmptyKey;
    slots[t].min_pos = kNoPos;
    slots[t].new_id = 0;
  }
  __syncthreads();
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const unsigned long long key = (unsigned long long)item_at(seeds, d.S, nbrs, i);
    uint32_t pos = (uint32_t)(((uint64_t)hash_id((int64_t)key) * kSmallCap) >> 32);
    for (;;) {   // at most kSmallItems of the kSmallCap slots are ever taken: an empty one is found
      Slot* s = slots + pos;
      unsigned long long prev = *(volatile unsigned long long*)&s->key;
      if (prev == kEmptyKey) prev = atomicCAS(&s->key, kEmptyKey, key);
      if (prev == kEmptyKey || prev == key) {
        atomicMin(&s->min_pos, (uint32_t)i);
        slot_of[i] = (uint16_t)pos;
        break;
      }
      pos = pos + 1 == kSmallCap ? 0 : pos + 1;
    }
  }
  __syncthreads();
  int running = 0;
  for (int base = 0; base < n; base += blockDim.x) {
    const int i = base + threadIdx.x;
    const int f = i < n && slots[slot_of[i]].min_pos == (uint32_t)i;
    int total;
    const int ex = block_exclusive_scan(f, scratch, &total);
    if (f) {
      const int id = running + ex;
      out_unique[id] = item_at(seeds, d.S, nbrs, i);
      slots[slot_of[i]].new_id = (uint32_t)id;
    }
    running += total;
  }
  if (threadIdx.x == 0) *out_num_unique = running;
  __syncthreads();
  for (int i = (int)d.S + threadIdx.x; i < n; i += blockDim.x)
    out_relabeled[i - d.S] = (int64_t)slots[slot_of[i]].new_id;
}

}  // namespace apt

extern "C" size_t apt_relabel_workspace_bytes(int64_t num_items) {
  if (num_items < 0) return 0;
  // a little headroom so that the size-only layout always fits num_items
  return apt::relabel_bytes_for(num_items + num_items / 256 + 4096);
}

extern "C" int apt_relabel_workspace_init(void* workspace, size_t workspace_bytes, void* stream) {
  using namespace apt;
  APT_CHECK_ARG(workspace && workspace_bytes > 0, "apt_relabel_workspace_init: null workspace");
  APT_CUDA(cudaMemsetAsync(workspace, 0xff, workspace_bytes, (cudaStream_t)stream));
  return APT_OK;
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
  if (n <= kSmallItems && g_relabel_small) {
    static bool attr_set[64] = {};
    int dev = 0;
    APT_CUDA(cudaGetDevice(&dev));
    if (dev < 64 && !attr_set[dev]) {
      APT_CUDA(cudaFuncSetAttribute(k_relabel_small, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmallSmem));
      attr_set[dev] = true;
    }
    ProfScope prof("relabel", s);
    APT_LAUNCH(k_relabel_small, 1, kRelabelBlock, kSmallSmem, s, seeds, num_seeds, neighbors, num_neighbors,
               num_seeds_dev, per_seed, out_unique, out_relabeled, out_num_unique);
    return APT_OK;
  }
  RelabelWs ws;
  if (!relabel_layout((char*)workspace, workspace_bytes, &ws) || ws.items_ws < n) {
    set_error("apt_relabel_csc: workspace of %zu bytes holds %lld items, %lld needed (apt_relabel_workspace_bytes)",
              workspace_bytes, (long long)ws.items_ws, (long long)n);
    return APT_ERR_CAPACITY;
  }
  ws.tiles = (int)ceil_div(n, kRelabelBlock);
  ProfScope prof("relabel", s);
  APT_LAUNCH(k_insert, ws.tiles, kRelabelBlock, 0, s, seeds, num_seeds, neighbors, num_neighbors,
             num_seeds_dev, per_seed, ws, status_word);
  APT_LAUNCH(k_count, ws.tiles, kRelabelBlock, 0, s, num_seeds, num_neighbors, num_seeds_dev, per_seed, ws);
  APT_LAUNCH(k_assign, ws.tiles, kRelabelBlock, 0, s, seeds, num_seeds, neighbors, num_neighbors,
             num_seeds_dev, per_seed, ws, out_unique, out_num_unique);
  const int grid = wave_grid(ceil_div(n, 256), 8);
  APT_LAUNCH(k_relabel, grid, 256, 0, s, num_seeds, num_neighbors, num_seeds_dev, per_seed, ws,
             out_relabeled);
  return APT_OK;
}
