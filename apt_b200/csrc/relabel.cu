// Relabelling of a sampled layer: unique of cat(seeds, neighbours) in order of
// first occurrence, and the new id of every neighbour.
//
// One open-addressing table (linear probing, load <= 2/3) in the caller's
// workspace holds, per distinct id, the smallest position at which it occurs.
// An item is a "first occurrence" iff that minimum equals its own position;
// an ordered compaction turns the first-occurrence flags into new ids, which
// makes the result independent of the table layout and of thread scheduling.
// Three launches:
//
//   k_insert        items -> table (CAS on the key, atomicMin on the position),
//                   remembers each item's slot. When the layer is sampled by this
//                   library the sampling kernel does this itself
//                   (sample_replace_kernel<G, true>, apt_sample_relabel_csc) and the
//                   neighbour list is never read back.
//   k_scan_assign   single-pass ordered compaction (tile counts chained by a
//                   look-back over the tiles before): new id = first occurrences
//                   before the item; writes unique[], the slot's new id and the
//                   number of unique ids
//   k_relabel       neighbours -> new id through the remembered slot; the first
//                   occurrence of every id also empties its slot again
//
// Layers of up to 8192 items run in one block with the table in shared memory
// (k_relabel_small below).
//
// The table is empty between calls (apt_relabel_workspace_init empties it once,
// each call empties the slots it used), so a call costs what its own item count
// costs and no clearing pass is needed.
#include "sample_kernels.cuh"

namespace apt {

constexpr int kRelabelBlock = 1024;

static size_t relabel_bytes_for(int64_t items) {
  const int64_t n = items > 0 ? items : 1;
  return align_up((size_t)relabel_capacity(n) * sizeof(Slot), 256) + align_up((size_t)n * 4, 256) +
         align_up(sizeof(ScanCtrl) + (size_t)(ceil_div(n, kScanTile) + 1) * 8, 256);
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
  const size_t o_ctrl = o_slot_of + align_up((size_t)items * 4, 256);
  ws->slots = (Slot*)base;
  ws->slot_of = (int32_t*)(base + o_slot_of);
  ws->ctrl = (ScanCtrl*)(base + o_ctrl);
  ws->tile_state = (uint64_t*)(base + o_ctrl + sizeof(ScanCtrl));
  return true;
}

__device__ __forceinline__ int64_t item_at(const int64_t* seeds, int64_t S,
                                           const int64_t* nbrs, int64_t i) {
  return i < S ? seeds[i] : nbrs[i - S];
}

// Pass 1 when the ids come from memory (apt_relabel_csc).
__global__ void __launch_bounds__(256)
k_insert(const int64_t* __restrict__ seeds, int64_t S_host, const int64_t* __restrict__ nbrs,
         int64_t M_host, const int64_t* __restrict__ S_dev, int64_t per_seed, RelabelWs ws,
         int32_t* status) {
  const RelabelDims d = relabel_dims(S_host, M_host, S_dev, per_seed);
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  int flags = 0;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < d.n; i += stride)
    ws.slot_of[i] = table_insert(ws.slots, d.cap, item_at(seeds, d.S, nbrs, i), (uint32_t)i, &flags);
  if (flags) atomicOr(status, flags);
}

// ---- pass 2: ordered compaction in one launch ----------------------------------------
// An item is a first occurrence iff its slot's smallest position is its own. Tiles of
// kScanTile consecutive items; their counts are chained by the look-back of common.cuh.
__global__ void __launch_bounds__(kScanThreads)
k_scan_assign(int64_t S_host, int64_t M_host, const int64_t* __restrict__ S_dev, int64_t per_seed,
              RelabelWs ws, int64_t* __restrict__ out_unique, int64_t* __restrict__ out_num_unique,
              int32_t* status) {
  __shared__ int scratch[33];
  __shared__ uint32_t s_tile, s_epoch, s_before;
  const RelabelDims d = relabel_dims(S_host, M_host, S_dev, per_seed);
  if (threadIdx.x == 0) tile_ticket(ws.ctrl, &s_tile, &s_epoch);
  __syncthreads();
  const uint32_t tile = s_tile;
  const int64_t first = (int64_t)tile * kScanTile;
  if (first < d.n || tile == 0) {
    // consecutive items of one thread: the block scan over thread sums keeps item order
    const int64_t i0 = first + (int64_t)threadIdx.x * kScanItems;
    int32_t slot[kScanItems];
    uint4 sv[kScanItems];
    int f[kScanItems];
    int mine = 0;
#pragma unroll
    for (int k = 0; k < kScanItems; ++k) slot[k] = i0 + k < d.n ? ws.slot_of[i0 + k] : -1;
#pragma unroll
    for (int k = 0; k < kScanItems; ++k)
      if (slot[k] >= 0) sv[k] = ld_plain_16((const uint4*)(ws.slots + slot[k]));
#pragma unroll
    for (int k = 0; k < kScanItems; ++k) {
      f[k] = slot[k] >= 0 && sv[k].z == (uint32_t)(i0 + k);
      mine += f[k];
    }
    int total;
    const int ex = block_exclusive_scan(mine, scratch, &total);
    if (threadIdx.x < 32) {
      const uint32_t before = tile_lookback(ws.tile_state, tile, s_epoch, (uint32_t)total, status, APT_FLAG_TABLE_FULL);
      if (threadIdx.x == 0) s_before = before;
    }
    __syncthreads();
    uint32_t id = s_before + (uint32_t)ex;
#pragma unroll
    for (int k = 0; k < kScanItems; ++k) {
      if (f[k]) {
        out_unique[id] = (int64_t)(((uint64_t)sv[k].y << 32) | sv[k].x);   // the slot's key is the id
        ws.slots[slot[k]].new_id = id;
        ++id;
      }
    }
    // the tile that holds the last item (or the only, empty tile) knows the number of unique ids
    if (threadIdx.x == 0 && first + kScanTile >= d.n) *out_num_unique = (int64_t)s_before + total;
  }
  __syncthreads();
  if (threadIdx.x == 0) tile_done(ws.ctrl, s_epoch);
}

// ---- pass 3: neighbours -> new id through the remembered slot; the first occurrence
// of every id also empties its slot again with one 16-byte store.
__global__ void __launch_bounds__(256)
k_relabel(int64_t S_host, int64_t M_host, const int64_t* __restrict__ S_dev, int64_t per_seed,
          RelabelWs ws, int64_t* __restrict__ out) {
  const RelabelDims d = relabel_dims(S_host, M_host, S_dev, per_seed);
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  constexpr int K = 4;
  for (int64_t base = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; base < d.n; base += stride * K) {
    int32_t slot[K];
    uint4 v[K];
#pragma unroll
    for (int k = 0; k < K; ++k) {
      const int64_t i = base + k * stride;
      slot[k] = i < d.n ? ws.slot_of[i] : -2;
    }
#pragma unroll
    for (int k = 0; k < K; ++k)
      if (slot[k] >= 0) v[k] = ld_plain_16((const uint4*)(ws.slots + slot[k]));
#pragma unroll
    for (int k = 0; k < K; ++k) {
      const int64_t i = base + k * stride;
      if (slot[k] == -2) continue;
      if (slot[k] < 0) {
        if (i >= d.S) out[i - d.S] = -1;
        continue;
      }
      if (i >= d.S) out[i - d.S] = (int64_t)v[k].w;
      // Nothing reads keys any more and only the first occurrence itself compares positions:
      // that item empties the slot (the new id stays for the items that have not read it yet).
      if (v[k].z == (uint32_t)i)
        st_plain_16((uint4*)(ws.slots + slot[k]), make_uint4(0xffffffffu, 0xffffffffu, kNoPos, v[k].w));
    }
  }
}

// ---- small layers: the whole relabelling in one block, table in shared memory ----------
// Up to kSmallItems items (the innermost hops of a mini-batch: 1024 seeds x (1 + 5)) fit a
// table of kSmallCap 16-byte slots in the 227 KB of shared memory of one SM together with
// each item's slot number. One block of 1024 threads then runs the three phases (insert,
// ordered compaction, relabel) with block barriers between them: no global table traffic,
// no clearing, one launch. (Drawing the neighbours inside this one block as well was measured
// slower than the separate sampling kernel: 28 us against 22 us for 1024 seeds x 5, because one
// block walks the dependent seed -> row -> neighbour loads in five rounds.) The order of first
// occurrence is decided by the minimum position per id exactly as in the multi-block path, so
// both give the same arrays.
static bool g_relabel_small = true;   // apt_set_tunable("relabel_small", 0) forces the multi-block path
void set_relabel_small(bool on) { g_relabel_small = on; }

constexpr int kSmallItems = 8192;
constexpr uint32_t kSmallCap = 12288;
constexpr uint16_t kSmallNoSlot = 0xffffu;
constexpr size_t kSmallSmem = (size_t)kSmallCap * sizeof(Slot) + (size_t)kSmallItems * sizeof(uint16_t);

// erase_nbrs: the neighbour list sits in the (otherwise unused) table region of the workspace and
// every entry is put back to all-ones once read, so that the table stays empty between calls.
__global__ void __launch_bounds__(kRelabelBlock)
k_relabel_small(const int64_t* __restrict__ seeds, int64_t S_host, int64_t* __restrict__ nbrs,
                int64_t M_host, const int64_t* __restrict__ S_dev, int64_t per_seed, int erase_nbrs,
                int64_t* __restrict__ out_unique, int64_t* __restrict__ out_relabeled,
                int64_t* __restrict__ out_num_unique, int32_t* status) {
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
  int flags = 0;
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const int64_t id = item_at(seeds, d.S, nbrs, i);
    if (erase_nbrs && i >= d.S) nbrs[i - d.S] = -1;
    if (id < 0) {   // not an id (see table_insert): no slot, relabelled to -1
      flags |= APT_FLAG_ID_OUT_OF_RANGE;
      slot_of[i] = kSmallNoSlot;
      continue;
    }
    const unsigned long long key = (unsigned long long)id;
    uint32_t pos = (uint32_t)(((uint64_t)hash_id(id) * kSmallCap) >> 32);
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
  if (flags) atomicOr(status, flags);
  __syncthreads();
  int running = 0;
  for (int base = 0; base < n; base += blockDim.x) {
    const int i = base + threadIdx.x;
    const int f = i < n && slot_of[i] != kSmallNoSlot && slots[slot_of[i]].min_pos == (uint32_t)i;
    int total;
    const int ex = block_exclusive_scan(f, scratch, &total);
    if (f) {
      const int id = running + ex;
      out_unique[id] = (int64_t)slots[slot_of[i]].key;
      slots[slot_of[i]].new_id = (uint32_t)id;
    }
    running += total;
  }
  if (threadIdx.x == 0) *out_num_unique = running;
  __syncthreads();
  for (int i = (int)d.S + threadIdx.x; i < n; i += blockDim.x)
    out_relabeled[i - d.S] = slot_of[i] == kSmallNoSlot ? (int64_t)-1 : (int64_t)slots[slot_of[i]].new_id;
}

static int set_small_smem() {
  static bool attr_set[64] = {};
  int dev = 0;
  APT_CUDA(cudaGetDevice(&dev));
  if (dev < 64 && !attr_set[dev]) {
    APT_CUDA(cudaFuncSetAttribute(k_relabel_small, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmallSmem));
    attr_set[dev] = true;
  }
  return APT_OK;
}

// Passes 2 and 3 of the multi-block path (the table already holds every item).
static int scan_and_relabel(int64_t num_seeds, int64_t num_neighbors, const int64_t* num_seeds_dev,
                            int64_t per_seed, const RelabelWs& ws, int64_t* out_unique, int64_t* out_relabeled,
                            int64_t* out_num_unique, int32_t* status_word, cudaStream_t s) {
  const int64_t n = num_seeds + num_neighbors;
  APT_LAUNCH(k_scan_assign, (int)ceil_div(n, kScanTile), kScanThreads, 0, s, num_seeds, num_neighbors,
             num_seeds_dev, per_seed, ws, out_unique, out_num_unique, status_word);
  const int grid = wave_grid(ceil_div(n, 256 * 4), 8, 1);
  APT_LAUNCH(k_relabel, grid, 256, 0, s, num_seeds, num_neighbors, num_seeds_dev, per_seed, ws, out_relabeled);
  return APT_OK;
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
  // the control words and tile states of the ordered compaction start at zero
  RelabelWs ws;
  if (relabel_layout((char*)workspace, workspace_bytes, &ws)) {
    const size_t off = (size_t)((char*)ws.ctrl - (char*)workspace);
    APT_CUDA(cudaMemsetAsync(ws.ctrl, 0, workspace_bytes - off, (cudaStream_t)stream));
  }
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
    const int rc = set_small_smem();
    if (rc != APT_OK) return rc;
    ProfScope prof("relabel", s);
    APT_LAUNCH(k_relabel_small, 1, kRelabelBlock, kSmallSmem, s, seeds, num_seeds, (int64_t*)neighbors, num_neighbors,
               num_seeds_dev, per_seed, 0, out_unique, out_relabeled, out_num_unique, status_word);
    return APT_OK;
  }
  RelabelWs ws;
  if (!relabel_layout((char*)workspace, workspace_bytes, &ws) || ws.items_ws < n) {
    set_error("apt_relabel_csc: workspace of %zu bytes holds %lld items, %lld needed (apt_relabel_workspace_bytes)",
              workspace_bytes, (long long)ws.items_ws, (long long)n);
    return APT_ERR_CAPACITY;
  }
  ProfScope prof("relabel", s);
  APT_LAUNCH(k_insert, wave_grid(ceil_div(n, 256 * 2), 8, 2), 256, 0, s, seeds, num_seeds, neighbors, num_neighbors,
             num_seeds_dev, per_seed, ws, status_word);
  return scan_and_relabel(num_seeds, num_neighbors, num_seeds_dev, per_seed, ws, out_unique, out_relabeled,
                          out_num_unique, status_word, s);
}

extern "C" int apt_sample_relabel_csc(const int64_t* seeds, int64_t num_seeds, const int64_t* num_seeds_dev,
                                      int fanout, const int64_t* adj_pos_map, int64_t num_nodes,
                                      const int64_t* dev_indptr, const int64_t* dev_indices,
                                      const int64_t* uva_indptr, const int64_t* uva_indices, uint64_t key,
                                      uint32_t call_id, const int64_t* call_id_base_dev, void* workspace,
                                      size_t workspace_bytes, int64_t* out_neighbors, int64_t* out_unique,
                                      int64_t* out_relabeled, int64_t* out_num_unique, int32_t* status_word,
                                      void* stream) {
  using namespace apt;
  APT_CHECK_ARG(num_seeds >= 0 && fanout > 0 && num_nodes >= 0,
                "apt_sample_relabel_csc: bad sizes (seeds %lld fanout %d)", (long long)num_seeds, fanout);
  const int64_t num_neighbors = num_seeds * fanout, n = num_seeds + num_neighbors;
  APT_CHECK_ARG(n < (int64_t)0x7f000000, "apt_sample_relabel_csc: %lld items exceed the 31-bit position range",
                (long long)n);
  APT_CHECK_ARG(out_num_unique && status_word, "apt_sample_relabel_csc: null output word");
  cudaStream_t s = (cudaStream_t)stream;
  if (n == 0) {
    APT_CUDA(cudaMemsetAsync(out_num_unique, 0, sizeof(int64_t), s));
    return APT_OK;
  }
  APT_CHECK_ARG(seeds && out_unique && out_relabeled && workspace && uva_indptr && uva_indices,
                "apt_sample_relabel_csc: null pointer");
  APT_CHECK_ARG(((uintptr_t)workspace & 255) == 0, "apt_sample_relabel_csc: workspace must be 256-byte aligned");
  const uint32_t k0 = (uint32_t)key, k1 = (uint32_t)(key >> 32);
  const CscView g{adj_pos_map, num_nodes, dev_indptr, dev_indices, uva_indptr, uva_indices};
  RelabelWs ws;
  if (!relabel_layout((char*)workspace, workspace_bytes, &ws) || ws.items_ws < n) {
    set_error("apt_sample_relabel_csc: workspace of %zu bytes holds %lld items, %lld needed "
              "(apt_relabel_workspace_bytes)", workspace_bytes, (long long)ws.items_ws, (long long)n);
    return APT_ERR_CAPACITY;
  }
  const bool small = n <= kSmallItems && g_relabel_small;
  // small layers: the neighbours go to the caller's array or, when it wants none, to the table region of the
  // workspace (16 bytes per slot, 1.5 slots per item: always room for 8 bytes per neighbour), which the
  // one-block kernel does not use and wipes again as it reads
  int64_t* nbr_buf = out_neighbors ? out_neighbors : (int64_t*)ws.slots;
  const SampleInsert ins{ws.slots, ws.slot_of};
  {
    ProfScope prof("sample", s);
#define APT_SAMPLE_INSERT(G)                                                                         \
  do {                                                                                               \
    const int grid = wave_grid(ceil_div(num_seeds, 256 / G), 8);                                     \
    if (small)                                                                                       \
      APT_LAUNCH((sample_replace_kernel<G, false>), grid, 256, 0, s, seeds, num_seeds,               \
                 num_seeds_dev, fanout, g, k0, k1, call_id, call_id_base_dev, nbr_buf, status_word,  \
                 SampleInsert{nullptr, nullptr});                                                    \
    else                                                                                             \
      APT_LAUNCH((sample_replace_kernel<G, true>), grid, 256, 0, s, seeds, num_seeds, num_seeds_dev, \
                 fanout, g, k0, k1, call_id, call_id_base_dev, out_neighbors, status_word, ins);     \
  } while (0)
    if (fanout <= 8) {
      APT_SAMPLE_INSERT(8);
    } else if (fanout <= 16) {
      APT_SAMPLE_INSERT(16);
    } else {
      APT_SAMPLE_INSERT(32);
    }
#undef APT_SAMPLE_INSERT
  }
  ProfScope prof("relabel", s);
  if (small) {
    const int rc = set_small_smem();
    if (rc != APT_OK) return rc;
    APT_LAUNCH(k_relabel_small, 1, kRelabelBlock, kSmallSmem, s, seeds, num_seeds, nbr_buf, num_neighbors,
               num_seeds_dev, (int64_t)fanout, out_neighbors ? 0 : 1, out_unique, out_relabeled, out_num_unique,
               status_word);
    return APT_OK;
  }
  return scan_and_relabel(num_seeds, num_neighbors, num_seeds_dev, (int64_t)fanout, ws, out_unique, out_relabeled,
                          out_num_unique, status_word, s);
}
