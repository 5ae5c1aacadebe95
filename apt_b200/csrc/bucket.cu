// Owner bucketing (stable partition of ids by owning rank) and the sorted
// unique + inverse over a bounded id range.
#include "common.cuh"

namespace apt {

constexpr int kMaxRanks = 32;
constexpr int kBucketBlock = 1024;

struct OwnerParams {
  int world_size;
  int shuffle_id_offset;
  int rank, node_beg, node_end;
};

// Owner of id v: the last rank d with min_vids[d] <= v, starting from
// shuffle_id_offset; owners outside this machine's rank window fall back to
// the calling rank.
__device__ __forceinline__ int owner_of(int64_t v, const int64_t* mv,
                                        const OwnerParams& p) {
  int d = p.shuffle_id_offset;
  while (d + 1 < p.world_size && mv[d + 1] <= v) ++d;
  if (d < p.node_beg || d >= p.node_end) d = p.rank;
  return d;
}

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
  if (i < n) atomicAdd(&cnt[owner_of(ids[i], mv, p)], 1);
  __syncthreads();
  if (threadIdx.x < p.world_size)
    hist[(int64_t)threadIdx.x * nblocks + blockIdx.x] = cnt[threadIdx.x];
}

// After the scan of hist (bucket-major), hist[b*nblocks + blk] is the first
// output slot of bucket b's items from block blk. Bucket sizes and inclusive
// offsets fall out of the same array.
__global__ void k_bucket_sizes(const int32_t* __restrict__ hist, int nblocks,
                               int world_size, int64_t n, const int64_t* __restrict__ n_dev,
                               int64_t* __restrict__ sizes,
                               int64_t* __restrict__ offsets) {
  n = effective_n(n, n_dev);
  const int b = threadIdx.x;
  if (b >= world_size) return;
  const int64_t beg = hist[(int64_t)b * nblocks];
  const int64_t end = b + 1 < world_size ? hist[(int64_t)(b + 1) * nblocks] : n;
  sizes[b] = end - beg;
  offsets[b] = end;
}

__global__ void __launch_bounds__(kBucketBlock)
k_bucket_scatter(const int64_t* __restrict__ ids, int64_t n, const int64_t* __restrict__ n_dev,
                 const int64_t* __restrict__ min_vids, OwnerParams p,
                 const int32_t* __restrict__ hist, int nblocks,
                 int64_t* __restrict__ sorted, int64_t* __restrict__ perm) {
  __shared__ int64_t mv[kMaxRanks + 1];
  __shared__ int warp_cnt[kBucketBlock / 32][kMaxRanks];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  n = effective_n(n, n_dev);
  if (threadIdx.x <= p.world_size) mv[threadIdx.x] = min_vids[threadIdx.x];
  for (int t = threadIdx.x; t < (kBucketBlock / 32) * kMaxRanks; t += blockDim.x)
    (&warp_cnt[0][0])[t] = 0;
  __syncthreads();
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
    const int64_t slot = (int64_t)hist[(int64_t)b * nblocks + blockIdx.x] +
                         warp_cnt[warp][b] + rank_in_warp;
    sorted[slot] = v;
    perm[i] = slot;
  }
}

// ------------------------------------------------------------ sorted unique
constexpr int kUniqBlock = 1024;

__global__ void __launch_bounds__(256)
k_uniq_mark(const int64_t* __restrict__ ids, int64_t n, const int64_t* __restrict__ n_dev,
            int64_t lo, int64_t hi, uint32_t* __restrict__ bitmap, int32_t* status) {
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
    uint32_t* w = bitmap + (r >> 5);
    if (!(*(volatile uint32_t*)w & bit)) atomicOr(w, bit);
  }
  if (flags) atomicOr(status, flags);
}

__global__ void __launch_bounds__(kUniqBlock)
k_uniq_count(const uint32_t* __restrict__ bitmap, int64_t nwords,
             int32_t* __restrict__ block_sums) {
  __shared__ int warp_sums[33];
  const int64_t w = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int c = w < nwords ? __popc(bitmap[w]) : 0;
  int total;
  block_exclusive_scan(c, warp_sums, &total);
  if (threadIdx.x == 0) block_sums[blockIdx.x] = total;
}

__global__ void __launch_bounds__(kUniqBlock)
k_uniq_emit(const uint32_t* __restrict__ bitmap, int64_t nwords, int64_t lo,
            const int32_t* __restrict__ block_sums,
            uint32_t* __restrict__ word_prefix, int64_t* __restrict__ out_unique) {
  __shared__ int warp_sums[33];
  const int64_t w = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  uint32_t bits = w < nwords ? bitmap[w] : 0u;
  int total;
  const int ex = block_exclusive_scan(__popc(bits), warp_sums, &total);
  if (w >= nwords) return;
  int64_t at = (int64_t)block_sums[blockIdx.x] + ex;
  word_prefix[w] = (uint32_t)at;
  const int64_t base = lo + (w << 5);
  while (bits) {
    const int b = __ffs(bits) - 1;
    out_unique[at++] = base + b;
    bits &= bits - 1;
  }
}

__global__ void __launch_bounds__(256)
k_uniq_inverse(const int64_t* __restrict__ ids, int64_t n, const int64_t* __restrict__ n_dev,
               int64_t lo, int64_t hi, const uint32_t* __restrict__ bitmap,
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
    const uint32_t bits = bitmap[r >> 5];
    out_inverse[i] = (int64_t)word_prefix[r >> 5] +
                     __popc(bits & ((1u << (r & 31)) - 1u));
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
    APT_CUDA(cudaMemsetAsync(out_bucket_sizes, 0, sizeof(int64_t) * world_size, s));
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
  APT_LAUNCH(k_scan_blocks, 1, 1024, 0, s, hist, nblocks * world_size, (int64_t*)nullptr);
  APT_LAUNCH(k_bucket_sizes, 1, 32, 0, s, hist, nblocks, world_size, num_ids, num_ids_dev,
             out_bucket_sizes, out_bucket_offsets);
  APT_LAUNCH(k_bucket_scatter, nblocks, kBucketBlock, 0, s, ids, num_ids, num_ids_dev, min_vids, p, hist,
             nblocks, out_sorted, out_perm);
  return APT_OK;
}

namespace apt {
struct UniqWs {
  uint32_t* bitmap;
  uint32_t* word_prefix;
  int32_t* block_sums;
  int64_t nwords;
  int nblocks;
};
static size_t uniq_layout(int64_t range, char* base, UniqWs* ws) {
  const int64_t nwords = ceil_div(range > 0 ? range : 1, 32);
  const int nblocks = (int)ceil_div(nwords, kUniqBlock);
  const size_t b0 = align_up((size_t)nwords * 4, 256);
  const size_t b1 = align_up((size_t)nwords * 4, 256);
  const size_t b2 = align_up((size_t)(nblocks + 1) * 4, 256);
  if (ws) {
    ws->bitmap = (uint32_t*)base;
    ws->word_prefix = (uint32_t*)(base + b0);
    ws->block_sums = (int32_t*)(base + b0 + b1);
    ws->nwords = nwords;
    ws->nblocks = nblocks;
  }
  return b0 + b1 + b2;
}
}  // namespace apt

extern "C" size_t apt_unique_workspace_bytes(int64_t id_range) {
  if (id_range < 0) return 0;
  return apt::uniq_layout(id_range, nullptr, nullptr);
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
  APT_CUDA(cudaMemsetAsync(ws.bitmap, 0, (size_t)ws.nwords * 4, s));
  const int g = wave_grid(ceil_div(num_ids, 256), 8);
  APT_LAUNCH(k_uniq_mark, g, 256, 0, s, ids, num_ids, num_ids_dev, id_lo, id_hi, ws.bitmap, status_word);
  APT_LAUNCH(k_uniq_count, ws.nblocks, kUniqBlock, 0, s, ws.bitmap, ws.nwords, ws.block_sums);
  APT_LAUNCH(k_scan_blocks, 1, 1024, 0, s, ws.block_sums, ws.nblocks, out_num_unique);
  APT_LAUNCH(k_uniq_emit, ws.nblocks, kUniqBlock, 0, s, ws.bitmap, ws.nwords, id_lo,
             ws.block_sums, ws.word_prefix, out_unique);
  APT_LAUNCH(k_uniq_inverse, g, 256, 0, s, ids, num_ids, num_ids_dev, id_lo, id_hi, ws.bitmap,
             ws.word_prefix, out_inverse);
  return APT_OK;
}
