// Owner bucketing (stable partition of ids by owning rank) and the sorted
// unique + inverse over a bounded id range.
#include "common.cuh"

namespace apt {

constexpr int kBucketBlock = 1024;

__global__ void __launch_bounds__(kBucketBlock)
k_bucket_count(const int64_t* __restrict__ ids, int64_t n, const int64_t* __restrict__ n_dev,
               const int64_t* __restrict__ min_vids, OwnerParams p,
               int32_t* __restrict__ hist /* [world_size][nblocks] */,
               int nblocks) {
  __shared__ int64_t mv[kMaxRanks + 1];
  __shared__ int cnt[kMaxRanks];
  n = effective_n(n, n_dev);
  if (threadIdx.x <= p.world_size) mv[threadIdx.x] = min_vids[threadIdx.x];
  if (threadIdx.x < kMaxRanks) cnt[threadIdx.x] = 0;
  __syncthreads();
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  // one shared-memory add per bucket and warp instead of one per id
  const int b = i < n ? owner_of(ids[i], mv, p) : -1;
  const unsigned peers = __match_any_sync(0xffffffffu, b);
  if (b >= 0 && (threadIdx.x & 31) == __ffs(peers) - 1) atomicAdd(&cnt[b], __popc(peers));
  __syncthreads();
  if (threadIdx.x < p.world_size)
    hist[(int64_t)threadIdx.x * nblocks + blockIdx.x] = cnt[threadIdx.x];
}

// Scatter. hist[k*nblocks + blk] (written by k_bucket_count) is the number of
// ids of block blk owned by rank k. The first output slot of bucket k's ids from
// this block is (ids of all lower buckets) + (ids of bucket k in lower blocks):
// warp k of the block sums row k of hist for that, so no scan kernel sits between
// the two passes. Block 0 also writes the bucket sizes (+ their total) and the
// inclusive offsets.
__global__ void __launch_bounds__(kBucketBlock)
k_bucket_scatter(const int64_t* __restrict__ ids, int64_t n, const int64_t* __restrict__ n_dev,
                 const int64_t* __restrict__ min_vids, OwnerParams p,
                 const int32_t* __restrict__ hist, int nblocks,
                 int64_t* __restrict__ sorted, int64_t* __restrict__ perm,
                 int64_t* __restrict__ sizes, int64_t* __restrict__ offsets) {
  __shared__ int64_t mv[kMaxRanks + 1];
  __shared__ int warp_cnt[kBucketBlock / 32][kMaxRanks];
  __shared__ int row_total[kMaxRanks], row_before[kMaxRanks], bucket_base[kMaxRanks];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  n = effective_n(n, n_dev);
  if (threadIdx.x <= p.world_size) mv[threadIdx.x] = min_vids[threadIdx.x];
  for (int t = threadIdx.x; t < (kBucketBlock / 32) * kMaxRanks; t += blockDim.x)
    (&warp_cnt[0][0])[t] = 0;
  if (warp < p.world_size) {
    const int32_t* row = hist + (int64_t)warp * nblocks;
    int tot = 0, before = 0;
    for (int t = lane; t < nblocks; t += 32) {
      const int c = row[t];
      tot += c;
      if (t < (int)blockIdx.x) before += c;
    }
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) {
      tot += __shfl_down_sync(0xffffffffu, tot, d);
      before += __shfl_down_sync(0xffffffffu, before, d);
    }
    if (lane == 0) {
      row_total[warp] = tot;
      row_before[warp] = before;
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int run = 0;
    for (int k = 0; k < p.world_size; ++k) {
      bucket_base[k] = run + row_before[k];
      run += row_total[k];
      if (blockIdx.x == 0) {
        sizes[k] = row_total[k];
        offsets[k] = run;
      }
    }
    if (blockIdx.x == 0) sizes[p.world_size] = run;
  }
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const bool live = i < n;
  int64_t v = 0;
  int b = -1;
  if (live) {
    v = ids[i];
    b = owner_of(v, mv, p);
  }
  // Rank of this lane among the lanes of its warp that share its bucket.
  const unsigned peers = __match_any_sync(0xffffffffu, b);
  const int rank_in_warp = __popc(peers & ((1u << lane) - 1u));
  if (live && rank_in_warp == 0) warp_cnt[warp][b] = __popc(peers);
  __syncthreads();
  // Exclusive scan over warps for each bucket (32 warps x <=32 buckets).
  if (threadIdx.x < kMaxRanks) {
    int run = 0;
    for (int w = 0; w < kBucketBlock / 32; ++w) {
      const int c = warp_cnt[w][threadIdx.x];
      warp_cnt[w][threadIdx.x] = run;
      run += c;
    }
  }
  __syncthreads();
  if (live) {
    const int64_t slot = (int64_t)bucket_base[b] + warp_cnt[warp][b] + rank_in_warp;
    sorted[slot] = v;
    perm[i] = slot;
  }
}

// out = cat(a[0:na], b[0:nb]) with both lengths taken from device words (the input nodes of an
// SNP-GAT mini-batch: the local destination nodes followed by the ids received from the peers,
// python/npc/sampler.py:230).
__global__ void __launch_bounds__(256)
k_concat_ids(const int64_t* __restrict__ a, int64_t na, const int64_t* __restrict__ na_dev,
             const int64_t* __restrict__ b, int64_t nb, const int64_t* __restrict__ nb_dev,
             int64_t* __restrict__ out, int64_t* __restrict__ out_count) {
  na = effective_n(na, na_dev);
  nb = effective_n(nb, nb_dev);
  const int64_t total = na + nb;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride)
    out[i] = i < na ? a[i] : b[i - na];
  if (out_count && blockIdx.x == 0 && threadIdx.x == 0) *out_count = total;
}

// ------------------------------------------------------------ sorted unique
// A two-level bitmap over the id range stands in for the sort: level 0 has one
// bit per id, level 1 one bit per level-0 word that is not zero. Counting,
// ranking and emitting walk level 1 only (range/1024 words), so the cost of a
// call follows the number of ids, not the width of the range. Both levels are
// all-zero between calls: the call clears exactly the words it set. Four launches:
// mark, emit (count + ordered ranks in one pass), inverse, clear.
constexpr int kUniqBlock = 1024;

__global__ void __launch_bounds__(256)
k_uniq_mark(const int64_t* __restrict__ ids, int64_t n, const int64_t* __restrict__ n_dev,
            int64_t lo, int64_t hi, uint32_t* __restrict__ l0, uint32_t* __restrict__ l1,
            int32_t* status) {
  n = effective_n(n, n_dev);
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  int flags = 0;
  for (; i < n; i += stride) {
    const int64_t v = ids[i];
    if (v < lo || v >= hi) {
      flags |= APT_FLAG_ID_OUT_OF_RANGE;
      continue;
    }
    const int64_t r = v - lo;
    const uint32_t bit = 1u << (r & 31);
    const int64_t w = r >> 5;
    if (*(volatile uint32_t*)(l0 + w) & bit) continue;
    const uint32_t old = atomicOr(l0 + w, bit);
    if (old == 0) atomicOr(l1 + (w >> 5), 1u << (w & 31));  // first bit of this word
  }
  if (flags) atomicOr(status, flags);
}

// Ids under one level-1 word (up to 1024 of them).
__device__ __forceinline__ int l1_word_count(const uint32_t* __restrict__ l0, int64_t w1, uint32_t bits) {
  int c = 0;
  while (bits) {
    const int b = __ffs(bits) - 1;
    bits &= bits - 1;
    c += __popc(l0[(w1 << 5) + b]);
  }
  return c;
}

// Counting, ranking and emitting in one launch: a tile of kUniqBlock level-1 words counts its ids,
// the tiles' counts are chained by the look-back of common.cuh, and the tile writes its ids in order.
__global__ void __launch_bounds__(kUniqBlock)
k_uniq_emit(const uint32_t* __restrict__ l0, const uint32_t* __restrict__ l1, int64_t nwords1,
            int64_t lo, ScanCtrl* ctrl, uint64_t* tile_state,
            uint32_t* __restrict__ word_prefix, int64_t* __restrict__ out_unique,
            int64_t* __restrict__ out_num_unique, int32_t* status) {
  __shared__ int warp_sums[33];
  __shared__ uint32_t s_tile, s_epoch, s_before;
  if (threadIdx.x == 0) tile_ticket(ctrl, &s_tile, &s_epoch);
  __syncthreads();
  const uint32_t tile = s_tile;
  const int64_t w1 = (int64_t)tile * blockDim.x + threadIdx.x;
  uint32_t bits1 = w1 < nwords1 ? l1[w1] : 0u;
  int total;
  const int ex = block_exclusive_scan(l1_word_count(l0, w1, bits1), warp_sums, &total);
  if (threadIdx.x < 32) {
    const uint32_t before = tile_lookback(tile_state, tile, s_epoch, (uint32_t)total, status, APT_FLAG_TABLE_FULL);
    if (threadIdx.x == 0) s_before = before;
  }
  __syncthreads();
  if (tile == gridDim.x - 1 && threadIdx.x == 0) *out_num_unique = (int64_t)s_before + total;
  int64_t at = (int64_t)s_before + ex;
  while (bits1) {
    const int b1 = __ffs(bits1) - 1;
    bits1 &= bits1 - 1;
    const int64_t w = (w1 << 5) + b1;
    uint32_t bits = l0[w];
    word_prefix[w] = (uint32_t)at;      // rank of the word's first id; only non-zero words are ever looked up
    const int64_t base = lo + (w << 5);
    while (bits) {
      const int b = __ffs(bits) - 1;
      bits &= bits - 1;
      out_unique[at++] = base + b;
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) tile_done(ctrl, s_epoch);
}

__global__ void __launch_bounds__(256)
k_uniq_inverse(const int64_t* __restrict__ ids, int64_t n, const int64_t* __restrict__ n_dev,
               int64_t lo, int64_t hi, const uint32_t* __restrict__ l0,
               const uint32_t* __restrict__ word_prefix,
               int64_t* __restrict__ out_inverse) {
  n = effective_n(n, n_dev);
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (; i < n; i += stride) {
    const int64_t v = ids[i];
    if (v < lo || v >= hi) {
      out_inverse[i] = -1;
      continue;
    }
    const int64_t r = v - lo;
    const uint32_t bits = l0[r >> 5];
    out_inverse[i] = (int64_t)word_prefix[r >> 5] +
                     __popc(bits & ((1u << (r & 31)) - 1u));
  }
}

// Puts both levels back to zero by revisiting the ids that set them.
__global__ void __launch_bounds__(256)
k_uniq_clear(const int64_t* __restrict__ ids, int64_t n, const int64_t* __restrict__ n_dev,
             int64_t lo, int64_t hi, uint32_t* __restrict__ l0, uint32_t* __restrict__ l1) {
  n = effective_n(n, n_dev);
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (; i < n; i += stride) {
    const int64_t v = ids[i];
    if (v < lo || v >= hi) continue;
    const int64_t w = (v - lo) >> 5;
    l0[w] = 0u;
    l1[w >> 5] = 0u;
  }
}

}  // namespace apt

extern "C" size_t apt_bucket_workspace_bytes(int64_t num_ids, int world_size) {
  if (num_ids < 0 || world_size < 1) return 0;
  const int64_t nblocks = apt::ceil_div(num_ids > 0 ? num_ids : 1, apt::kBucketBlock);
  return apt::align_up((size_t)(nblocks * world_size + 1) * 4, 256);
}

extern "C" int apt_bucket_by_owner(const int64_t* ids, int64_t num_ids,
                                   const int64_t* num_ids_dev, const int64_t* min_vids, int world_size,
                                   int64_t shuffle_id_offset, int rank,
                                   int node_beg, int node_end, void* workspace,
                                   size_t workspace_bytes, int64_t* out_sorted,
                                   int64_t* out_perm, int64_t* out_bucket_sizes,
                                   int64_t* out_bucket_offsets, void* stream) {
  using namespace apt;
  APT_CHECK_ARG(world_size >= 1 && world_size <= kMaxRanks,
                "apt_bucket_by_owner: world_size %d outside [1,%d]", world_size, kMaxRanks);
  APT_CHECK_ARG(num_ids >= 0 && num_ids < (int64_t)0x7fffffff, "apt_bucket_by_owner: bad num_ids");
  APT_CHECK_ARG(min_vids && out_bucket_sizes && out_bucket_offsets,
                "apt_bucket_by_owner: null pointer");
  APT_CHECK_ARG(rank >= 0 && rank < world_size && shuffle_id_offset >= 0 &&
                    shuffle_id_offset < world_size,
                "apt_bucket_by_owner: rank/offset outside the world");
  cudaStream_t s = (cudaStream_t)stream;
  if (num_ids == 0) {
    APT_CUDA(cudaMemsetAsync(out_bucket_sizes, 0, sizeof(int64_t) * (world_size + 1), s));
    APT_CUDA(cudaMemsetAsync(out_bucket_offsets, 0, sizeof(int64_t) * world_size, s));
    return APT_OK;
  }
  APT_CHECK_ARG(ids && out_sorted && out_perm && workspace, "apt_bucket_by_owner: null pointer");
  const size_t need = apt_bucket_workspace_bytes(num_ids, world_size);
  if (workspace_bytes < need) {
    set_error("apt_bucket_by_owner: workspace %zu < %zu bytes", workspace_bytes, need);
    return APT_ERR_CAPACITY;
  }
  OwnerParams p;
  p.world_size = world_size;
  p.shuffle_id_offset = (int)shuffle_id_offset;
  p.rank = rank;
  p.node_beg = node_beg;
  p.node_end = node_end;
  const int nblocks = (int)ceil_div(num_ids, kBucketBlock);
  int32_t* hist = (int32_t*)workspace;
  ProfScope prof("bucket", s);
  APT_LAUNCH(k_bucket_count, nblocks, kBucketBlock, 0, s, ids, num_ids, num_ids_dev, min_vids, p, hist, nblocks);
  APT_LAUNCH(k_bucket_scatter, nblocks, kBucketBlock, 0, s, ids, num_ids, num_ids_dev, min_vids, p, hist,
             nblocks, out_sorted, out_perm, out_bucket_sizes, out_bucket_offsets);
  return APT_OK;
}

namespace apt {
struct UniqWs {
  uint32_t* l0;           // [nwords0] one bit per id
  uint32_t* l1;           // [nwords1] one bit per level-0 word
  uint32_t* word_prefix;  // [nwords0]
  ScanCtrl* ctrl;         // [1]        control words of the ordered emit, zero once
  uint64_t* tile_state;   // [nblocks]  its tile states, tagged by call
  int64_t nwords0, nwords1;
  int nblocks;
  size_t bitmap_bytes;    // l0 + l1: the part that has to be zero between calls
};
static size_t uniq_layout(int64_t range, char* base, UniqWs* ws) {
  const int64_t nwords0 = ceil_div(range > 0 ? range : 1, 32);
  const int64_t nwords1 = ceil_div(nwords0, 32);
  const int nblocks = (int)ceil_div(nwords1, kUniqBlock);
  const size_t b0 = align_up((size_t)nwords1 * 32 * 4, 256);  // level 0, padded to whole level-1 words
  const size_t b1 = align_up((size_t)nwords1 * 4, 256);
  const size_t b2 = align_up((size_t)nwords0 * 4, 256);
  const size_t b3 = align_up(sizeof(ScanCtrl) + (size_t)nblocks * 8, 256);
  if (ws) {
    ws->l0 = (uint32_t*)base;
    ws->l1 = (uint32_t*)(base + b0);
    ws->word_prefix = (uint32_t*)(base + b0 + b1);
    ws->ctrl = (ScanCtrl*)(base + b0 + b1 + b2);
    ws->tile_state = (uint64_t*)(base + b0 + b1 + b2 + sizeof(ScanCtrl));
    ws->nwords0 = nwords0;
    ws->nwords1 = nwords1;
    ws->nblocks = nblocks;
    ws->bitmap_bytes = b0 + b1;
  }
  return b0 + b1 + b2 + b3;
}
}  // namespace apt

extern "C" size_t apt_unique_workspace_bytes(int64_t id_range) {
  if (id_range < 0) return 0;
  return apt::uniq_layout(id_range, nullptr, nullptr);
}

extern "C" int apt_unique_workspace_init(void* workspace, size_t workspace_bytes, void* stream) {
  using namespace apt;
  APT_CHECK_ARG(workspace && workspace_bytes > 0, "apt_unique_workspace_init: null workspace");
  APT_CUDA(cudaMemsetAsync(workspace, 0, workspace_bytes, (cudaStream_t)stream));
  return APT_OK;
}

extern "C" int apt_unique_sorted(const int64_t* ids, int64_t num_ids,
                                 const int64_t* num_ids_dev, int64_t id_lo,
                                 int64_t id_hi, void* workspace, size_t workspace_bytes,
                                 int64_t* out_unique, int64_t* out_inverse,
                                 int64_t* out_num_unique, int32_t* status_word,
                                 void* stream) {
  using namespace apt;
  APT_CHECK_ARG(num_ids >= 0 && id_hi >= id_lo, "apt_unique_sorted: bad sizes");
  APT_CHECK_ARG(id_hi - id_lo < ((int64_t)1 << 36), "apt_unique_sorted: id range too wide for a bitmap");
  APT_CHECK_ARG(out_num_unique && status_word, "apt_unique_sorted: null output word");
  cudaStream_t s = (cudaStream_t)stream;
  if (num_ids == 0 || id_hi == id_lo) {
    APT_CUDA(cudaMemsetAsync(out_num_unique, 0, sizeof(int64_t), s));
    if (num_ids > 0) {
      APT_CHECK_ARG(out_inverse, "apt_unique_sorted: null pointer");
      APT_CUDA(cudaMemsetAsync(out_inverse, 0xff, sizeof(int64_t) * num_ids, s));
    }
    return APT_OK;
  }
  APT_CHECK_ARG(ids && workspace && out_unique && out_inverse, "apt_unique_sorted: null pointer");
  UniqWs ws;
  const size_t need = uniq_layout(id_hi - id_lo, (char*)workspace, &ws);
  if (workspace_bytes < need) {
    set_error("apt_unique_sorted: workspace %zu < %zu bytes", workspace_bytes, need);
    return APT_ERR_CAPACITY;
  }
  ProfScope prof("unique_sorted", s);
  const int g = wave_grid(ceil_div(num_ids, 256), 8);
  APT_LAUNCH(k_uniq_mark, g, 256, 0, s, ids, num_ids, num_ids_dev, id_lo, id_hi, ws.l0, ws.l1, status_word);
  APT_LAUNCH(k_uniq_emit, ws.nblocks, kUniqBlock, 0, s, ws.l0, ws.l1, ws.nwords1, id_lo, ws.ctrl, ws.tile_state,
             ws.word_prefix, out_unique, out_num_unique, status_word);
  APT_LAUNCH(k_uniq_inverse, g, 256, 0, s, ids, num_ids, num_ids_dev, id_lo, id_hi, ws.l0,
             ws.word_prefix, out_inverse);
  APT_LAUNCH(k_uniq_clear, g, 256, 0, s, ids, num_ids, num_ids_dev, id_lo, id_hi, ws.l0, ws.l1);
  return APT_OK;
}

extern "C" int apt_concat_ids(const int64_t* a, int64_t num_a, const int64_t* num_a_dev, const int64_t* b,
                              int64_t num_b, const int64_t* num_b_dev, int64_t* out, int64_t* out_count_dev,
                              void* stream) {
  using namespace apt;
  APT_CHECK_ARG(num_a >= 0 && num_b >= 0 && (num_a == 0 || a) && (num_b == 0 || b), "apt_concat_ids: bad argument");
  APT_CHECK_ARG(out || num_a + num_b == 0, "apt_concat_ids: null output");
  cudaStream_t s = (cudaStream_t)stream;
  if (num_a + num_b == 0) {
    if (out_count_dev) APT_CUDA(cudaMemsetAsync(out_count_dev, 0, sizeof(int64_t), s));
    return APT_OK;
  }
  APT_LAUNCH(k_concat_ids, wave_grid(ceil_div(num_a + num_b, 256), 8, 1), 256, 0, s, a, num_a, num_a_dev, b, num_b,
             num_b_dev, out, out_count_dev);
  return APT_OK;
}
