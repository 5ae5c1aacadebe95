// Cache-aware feature-row gather.
//
//   k_classify     id -> feat_pos_map entry of every requested row, kept in a dense
//                  scratch array; rows that live in host memory are also appended
//                  (warp-aggregated) to a miss list. One resident wave, grid-stride.
//   k_copy_hits    HBM -> HBM, register-staged. One resident wave; every warp owns one
//                  contiguous share of the rows, reads 32 positions with one coalesced
//                  load and keeps two groups of four rows in flight: the loads of the
//                  next group are issued before the stores of the current one, so the
//                  warp always has loads outstanding.
//   k_copy_hits_bulk  the same copy staged through shared memory by the SM's bulk-copy
//                  engine (cp.async.bulk global -> shared -> global): a warp has 32 rows
//                  in flight per buffer, two buffers in turn, and moves a row with two
//                  instructions instead of 2 x 32 lanes of vector loads and stores.
//                  Rows must be multiples of 16 bytes on 16-byte boundaries.
//                  (A variant that decoded the ids inside the copy kernel, the two
//                  dependent lookups in front of each share of rows, was measured at
//                  0.47-0.62 of the HBM peak on 143 000 rows against 0.67 for decode
//                  and copy as two kernels: a warp that waits for its lookups has
//                  nothing in flight.)
//   k_copy_miss    pinned host memory -> HBM over the host link, over the miss list.
//                  It runs after the hit copy on the same stream: measured on B200,
//                  running the two at once (second stream, any grid size) slows the
//                  hit copy by 2-4x and the pair finishes later than back to back.
//   k_copy_miss_bulk  variant of the miss copy that stages rows through shared
//                  memory with cp.async.bulk (gather_miss_mode = 1); measured equal
//                  or slower than the vector loads, kept for comparison.
//
// Rows are opaque bytes. The vector width V is the widest of 16/8/4/2/1 bytes
// that divides every row size, column offset and base address involved.
#include <string.h>

#include "common.cuh"

namespace apt {

constexpr int kRowsPerGroup = 4;   // rows whose loads are in flight together
constexpr int kMinMissBlocks = 16; // blocks of the miss copy that always take part
constexpr int kGatherBlock = 256;

struct GatherWs {
  int64_t* src_pos;    // [n]  feat_pos_map[index[r]], -1 = no such row
  int32_t* miss_rows;  // [n]  output rows whose source is host memory
  int32_t* miss_count; // [1]
};

static size_t gather_layout(int64_t n, char* base, GatherWs* ws) {
  const size_t rows = (size_t)(n > 0 ? n : 1);
  const size_t b0 = align_up(rows * 8, 256);
  const size_t b1 = align_up(rows * 4, 256);
  if (ws) {
    ws->src_pos = (int64_t*)base;
    ws->miss_rows = (int32_t*)(base + b0);
    ws->miss_count = (int32_t*)(base + b0 + b1);
  }
  return b0 + b1 + 256;
}

template <typename V>
__device__ __forceinline__ V ld_vec(const V* p) { return __ldg(p); }
template <>
__device__ __forceinline__ uint4 ld_vec<uint4>(const uint4* p) { return ld_stream_16(p); }
template <typename V>
__device__ __forceinline__ void st_vec(V* p, V v) { *p = v; }
template <>
__device__ __forceinline__ void st_vec<uint4>(uint4* p, uint4 v) { st_stream_16(p, v); }
template <typename V>
__device__ __forceinline__ V zero_vec() { return V(0); }
template <>
__device__ __forceinline__ uint4 zero_vec<uint4>() { return make_uint4(0, 0, 0, 0); }
template <>
__device__ __forceinline__ uint2 zero_vec<uint2>() { return make_uint2(0, 0); }

// Rows [first, n) of the request, first from a device word when given.
__device__ __forceinline__ int64_t first_row(const int64_t* first_dev, int64_t n) {
  const int64_t f = first_dev ? *first_dev : 0;
  return f < 0 ? 0 : (f > n ? n : f);
}

// p = feat_pos_map[index[r]]: p >= 0 cache row, p < -1 host row -(p)-2 (queued for
// the miss copy), p == -1 no such row (zeros + flag).
__global__ void __launch_bounds__(256)
k_classify(const int64_t* __restrict__ index, int64_t n, const int64_t* __restrict__ n_dev,
           const int64_t* __restrict__ first_dev, const int64_t* __restrict__ pos_map,
           int64_t num_nodes, int64_t num_dev_rows, int64_t num_uva_rows, GatherWs ws, int32_t* status) {
  const int lane = threadIdx.x & 31;
  n = effective_n(n, n_dev);
  const int64_t first = first_row(first_dev, n);
  int64_t r = first + (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  int flags = 0;
  // Whole warps iterate together so that the ballot below is convergent.
  for (int64_t r0 = r - lane; r0 < n; r0 += stride, r += stride) {
    int64_t p = -1;
    if (r < n) {
      const int64_t id = index[r];
      if (id < 0 || id >= num_nodes) {
        flags |= APT_FLAG_ID_OUT_OF_RANGE;
      } else {
        p = pos_map[id];
        if (p == -1) {
          flags |= APT_FLAG_FEAT_NOT_EXIST;
        } else if (p >= num_dev_rows || (-p - 2) >= num_uva_rows) {
          flags |= APT_FLAG_ID_OUT_OF_RANGE;
          p = -1;
        }
      }
      ws.src_pos[r] = p;
    }
    const bool miss = p < -1;
    const unsigned m = __ballot_sync(0xffffffffu, miss);
    if (m) {
      int base = 0;
      const int leader = __ffs(m) - 1;
      if (lane == leader) base = atomicAdd(ws.miss_count, __popc(m));
      base = __shfl_sync(0xffffffffu, base, leader);
      if (miss) ws.miss_rows[base + __popc(m & ((1u << lane) - 1u))] = (int32_t)r;
    }
  }
  if (flags) atomicOr(status, flags);
}

// The share of rows of one warp: rows [first, n) split evenly over all warps of the grid.
__device__ __forceinline__ void warp_share(int64_t first, int64_t n, int64_t* lo, int64_t* hi) {
  const int64_t warps = (int64_t)gridDim.x * (blockDim.x >> 5);
  const int64_t warp = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int64_t m = n - first;
  *lo = first + m * warp / warps;
  *hi = first + m * (warp + 1) / warps;
}

// Output row r comes from cache row src_pos[r] (>= 0), is zero (src_pos == -1), or
// belongs to the miss copy (src_pos < -1).
template <typename V>
__global__ void __launch_bounds__(kGatherBlock, 4)
k_copy_hits(int64_t n, const int64_t* __restrict__ n_dev, const int64_t* __restrict__ first_dev,
            const int64_t* __restrict__ src_pos, const char* __restrict__ dev_feats, int64_t row_bytes,
            char* __restrict__ out) {
  constexpr int R = kRowsPerGroup;
  n = effective_n(n, n_dev);
  const int lane = threadIdx.x & 31;
  int64_t lo, hi;
  warp_share(first_row(first_dev, n), n, &lo, &hi);
  const int chunks = (int)(row_bytes / (int64_t)sizeof(V));
  if (chunks <= 32) {
    // Rows of up to 32 vectors (512 bytes with 16-byte vectors): one vector per lane and row. The
    // share is walked in groups of R rows with two groups in flight (the loads of group g + 1 are
    // issued before the stores of group g); positions come in windows of 32 rows, one coalesced
    // load each, and the next window is fetched while the current one is being copied, so the warp
    // never runs out of loads in flight before its share ends.
    const bool live = lane < chunks;
    const int64_t rows = hi - lo;
    const int64_t groups = (rows + R - 1) / R;
    // -2 and below: not this kernel's row (a miss, or past the share)
    int64_t p_cur = lane < rows ? src_pos[lo + lane] : (int64_t)-2;
    int64_t p_nxt = 32 + lane < rows ? src_pos[lo + 32 + lane] : (int64_t)-2;
    V cur[R], nxt[R];
#pragma unroll
    for (int k = 0; k < R; ++k) {
      const int64_t pk = __shfl_sync(0xffffffffu, p_cur, k);
      cur[k] = zero_vec<V>();
      if (live && pk >= 0) cur[k] = ld_vec<V>((const V*)(dev_feats + pk * row_bytes) + lane);
    }
    for (int64_t g = 0; g < groups; ++g) {
      const int at = (int)((g * R) & 31);                 // first row of group g inside its window
      const bool turn = at + R == 32;                     // group g + 1 opens the next window
#pragma unroll
      for (int k = 0; k < R; ++k) {
        const int64_t pk = __shfl_sync(0xffffffffu, turn ? p_nxt : p_cur, (at + R + k) & 31);
        nxt[k] = zero_vec<V>();
        if (live && pk >= 0) nxt[k] = ld_vec<V>((const V*)(dev_feats + pk * row_bytes) + lane);
      }
#pragma unroll
      for (int k = 0; k < R; ++k) {
        const int64_t pk = __shfl_sync(0xffffffffu, p_cur, at + k);
        if (live && pk >= -1) st_vec<V>((V*)(out + (lo + g * R + k) * row_bytes) + lane, cur[k]);
      }
#pragma unroll
      for (int k = 0; k < R; ++k) cur[k] = nxt[k];
      if (turn) {
        p_cur = p_nxt;
        const int64_t next_window = (g + 1) * R + 32;     // first row of the window after the one just opened
        p_nxt = next_window + lane < rows ? src_pos[lo + next_window + lane] : (int64_t)-2;
      }
    }
  } else {
    for (int64_t base = lo; base < hi; base += 32) {
      const int cnt = hi - base < 32 ? (int)(hi - base) : 32;
      const int64_t p = lane < cnt ? src_pos[base + lane] : (int64_t)-2;
      for (int k0 = 0; k0 < cnt; k0 += R) {
        // the trip count is the same for all lanes, so that the shuffles are convergent
        for (int c0 = 0; c0 < chunks; c0 += 32) {
          const int c = c0 + lane;
          const bool live = c < chunks;
          V v[R];
#pragma unroll
          for (int k = 0; k < R; ++k) {
            const int64_t pk = __shfl_sync(0xffffffffu, p, (k0 + k) & 31);
            v[k] = zero_vec<V>();
            if (live && k0 + k < cnt && pk >= 0) v[k] = ld_vec<V>((const V*)(dev_feats + pk * row_bytes) + c);
          }
#pragma unroll
          for (int k = 0; k < R; ++k) {
            const int64_t pk = __shfl_sync(0xffffffffu, p, (k0 + k) & 31);
            if (live && k0 + k < cnt && pk >= -1) st_vec<V>((V*)(out + (base + k0 + k) * row_bytes) + c, v[k]);
          }
        }
      }
    }
  }
}

// Grid-stride form of the hit copy: many small blocks, a warp takes R consecutive rows at a time
// (positions, then all loads, then all stores) and strides over the request. The hardware's block
// scheduler spreads the blocks over the SMs as they retire.
template <typename V>
__global__ void __launch_bounds__(kGatherBlock)
k_copy_hits_strided(int64_t n, const int64_t* __restrict__ n_dev, const int64_t* __restrict__ first_dev,
                    const int64_t* __restrict__ src_pos, const char* __restrict__ dev_feats, int64_t row_bytes,
                    char* __restrict__ out) {
  n = effective_n(n, n_dev);
  const int64_t first = first_row(first_dev, n);
  const int lane = threadIdx.x & 31;
  const int64_t warps = (int64_t)gridDim.x * (blockDim.x >> 5);
  const int64_t warp = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int chunks = (int)(row_bytes / (int64_t)sizeof(V));
  for (int64_t r0 = first + warp * kRowsPerGroup; r0 < n; r0 += warps * kRowsPerGroup) {
    int64_t p[kRowsPerGroup];
#pragma unroll
    for (int k = 0; k < kRowsPerGroup; ++k) p[k] = r0 + k < n ? src_pos[r0 + k] : (int64_t)-2;
    for (int c = lane; c < chunks; c += 32) {
      V v[kRowsPerGroup];
#pragma unroll
      for (int k = 0; k < kRowsPerGroup; ++k) {
        v[k] = zero_vec<V>();
        if (p[k] >= 0) v[k] = ld_vec<V>((const V*)(dev_feats + p[k] * row_bytes) + c);
      }
#pragma unroll
      for (int k = 0; k < kRowsPerGroup; ++k)
        if (p[k] >= -1) st_vec<V>((V*)(out + (r0 + k) * row_bytes) + c, v[k]);
    }
  }
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}

// Bounded wait for a phase of an mbarrier in shared memory (about a second).
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t phase) {
  uint32_t done = 0;
  const uint64_t t0 = global_timer_ns();
  for (int it = 0; it < (1 << 22) && !done; ++it) {
    asm volatile(
        "{ .reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }"
        : "=r"(done)
        : "r"(bar), "r"(phase)
        : "memory");
    if (!done && (it & 63) == 63 && global_timer_ns() - t0 > 1000000000ull) break;  // 1 s
  }
  return done != 0;
}

// Bulk-copy variant of the hit copy. A warp owns two buffers of `slots` row slots (up to
// 32) in shared memory. Filling a buffer: lane l asks the SM's copy engine for row l of the
// batch (cp.async.bulk global -> shared), all copies of the batch completing on one
// mbarrier whose expected byte count lane 0 has armed. Draining: after the wait lane l
// sends its row on (shared -> global), one bulk group per batch. Batch t is filled before
// batch t-1 is drained, so a warp has up to 2 x slots rows in flight. Rows without a source
// are zeroed by their lane (src_pos == -1) or skipped (misses). A wait that runs out sets
// APT_FLAG_PEER_TIMEOUT and ends the warp's work after one more bounded wait for the
// copies it still has in flight.
constexpr int kBulkWarps = 6;                 // warps per block
constexpr size_t kBulkSmem = 192 * 1024;      // 6 warps x 2 buffers x 32 rows of 512 bytes

__global__ void __launch_bounds__(kBulkWarps * 32, 1)
k_copy_hits_bulk(int64_t n, const int64_t* __restrict__ n_dev, const int64_t* __restrict__ first_dev,
                 const int64_t* __restrict__ src_pos, const char* __restrict__ dev_feats, int64_t row_bytes,
                 int slots, char* __restrict__ out, int32_t* status) {
  extern __shared__ __align__(128) unsigned char smem[];
  __shared__ __align__(8) uint64_t bars[kBulkWarps * 2];
  n = effective_n(n, n_dev);
  const int lane = threadIdx.x & 31, wib = threadIdx.x >> 5;
  int64_t lo, hi;
  warp_share(first_row(first_dev, n), n, &lo, &hi);
  unsigned char* wbuf = smem + (size_t)wib * 2 * slots * row_bytes;
  uint64_t* wbar = bars + wib * 2;
  if (lane == 0) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_u32(wbar)));
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_u32(wbar + 1)));
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncwarp();
  const int64_t batches = (hi - lo + slots - 1) / slots;
  uint32_t parity0 = 0u, parity1 = 0u;   // phase each buffer's barrier completes next
  int64_t prev_p = -2, prev_row = 0;     // this lane's row of the batch that is in flight
  bool failed = false;
  for (int64_t t = 0; t <= batches && !failed; ++t) {
    const int b = (int)(t & 1);
    int64_t p = -2, row = 0;
    unsigned hits = 0;
    if (t < batches) {
      row = lo + t * slots + lane;
      if (lane < slots && row < hi) p = src_pos[row];
      // the rows this buffer held two batches ago must have been read out of shared memory
      asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
      __syncwarp();
      hits = __ballot_sync(0xffffffffu, p >= 0);
      if (lane == 0 && hits)
        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(wbar + b)),
                     "r"((uint32_t)__popc(hits) * (uint32_t)row_bytes)
                     : "memory");
      __syncwarp();
      unsigned char* slot = wbuf + ((size_t)b * slots + lane) * row_bytes;
      if (p >= 0) {
        asm volatile(
            "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                smem_u32(slot)),
            "l"(dev_feats + p * row_bytes), "r"((uint32_t)row_bytes), "r"(smem_u32(wbar + b))
            : "memory");
      } else if (p == -1) {
        for (int64_t o = 0; o < row_bytes; o += 16) *(uint4*)(slot + o) = make_uint4(0, 0, 0, 0);
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // generic writes, then read by the bulk store
      }
    }
    if (t >= 1) {
      // drain batch t - 1 (buffer b ^ 1)
      const int pb = b ^ 1;
      const unsigned had_hits = __ballot_sync(0xffffffffu, prev_p >= 0);
      bool ok = true;
      if (had_hits) {
        ok = mbar_wait_bounded(smem_u32(wbar + pb), pb ? parity1 : parity0);
        if (pb) parity1 ^= 1u; else parity0 ^= 1u;
      }
      ok = __all_sync(0xffffffffu, ok);
      if (ok && prev_p >= -1)
        asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(out + prev_row * row_bytes),
                     "r"(smem_u32(wbuf + ((size_t)pb * slots + lane) * row_bytes)), "r"((uint32_t)row_bytes)
                     : "memory");
      asm volatile("cp.async.bulk.commit_group;" ::: "memory");
      if (!ok) {
        failed = true;
        // the batch issued above may still be landing: one more bounded wait before the buffers go away
        if (hits) mbar_wait_bounded(smem_u32(wbar + b), b ? parity1 : parity0);
      }
    }
    prev_p = p;
    prev_row = row;
  }
  asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
  if (failed && lane == 0) atomicOr(status, APT_FLAG_PEER_TIMEOUT);
}

template <typename V>
__global__ void __launch_bounds__(kGatherBlock)
k_copy_miss(GatherWs ws, const char* __restrict__ uva_feats, int64_t uva_row_bytes,
            int64_t col_offset_bytes, int64_t row_bytes, int64_t bytes_per_block,
            char* __restrict__ out) {
  const int lane = threadIdx.x & 31;
  const int64_t n = *ws.miss_count;
  // With bytes_per_block set, only as many blocks take part as the bytes to fetch ask for (at least
  // kMinMissBlocks, at most the grid); the others leave at once. A copy from host memory holds its
  // SM slots for a long time without using the SMs; when several mini-batches are in flight the slots
  // it does not need are worth more to their kernels than to the copy.
  int64_t blocks = gridDim.x;
  if (bytes_per_block > 0) {
    const int64_t want = (n * row_bytes + bytes_per_block - 1) / bytes_per_block;
    blocks = want < kMinMissBlocks ? kMinMissBlocks : want;
    if (blocks > (int64_t)gridDim.x) blocks = gridDim.x;
    if ((int64_t)blockIdx.x >= blocks) return;
  }
  const int64_t warps = blocks * (blockDim.x >> 5);
  const int64_t warp = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int chunks = (int)(row_bytes / (int64_t)sizeof(V));
  for (int64_t m0 = warp * kRowsPerGroup; m0 < n; m0 += warps * kRowsPerGroup) {
    int64_t r[kRowsPerGroup], p[kRowsPerGroup];
#pragma unroll
    for (int k = 0; k < kRowsPerGroup; ++k) {
      r[k] = m0 + k < n ? (int64_t)ws.miss_rows[m0 + k] : (int64_t)-1;
      p[k] = r[k] >= 0 ? -ws.src_pos[r[k]] - 2 : (int64_t)0;
    }
    for (int c = lane; c < chunks; c += 32) {
      V v[kRowsPerGroup];
#pragma unroll
      for (int k = 0; k < kRowsPerGroup; ++k) {
        v[k] = zero_vec<V>();
        if (r[k] >= 0)
          v[k] = ld_vec<V>((const V*)(uva_feats + p[k] * uva_row_bytes + col_offset_bytes) + c);
      }
#pragma unroll
      for (int k = 0; k < kRowsPerGroup; ++k)
        if (r[k] >= 0) st_vec<V>((V*)(out + r[k] * row_bytes) + c, v[k]);
    }
  }
}

// ---- tunables (set through apt_set_tunable; defaults are the measured best) ----
static int g_miss_mode = 0;      // 0: 16-byte ld.global.nc, 1: bulk copy staged through shared memory
static int g_miss_blocks = kNumSMs;
static int g_miss_kb_per_block = 0;  // > 0: blocks of the miss copy beyond one per this many KiB to fetch leave at once
static int g_hit_mode = 0;       // 0: one wave, two groups in flight per warp; 1: bulk copies through shared memory;
                                 // 2: grid-stride blocks, one group per warp at a time
static int g_hit_waves = 4;      // mode 2: cap on the grid, in units of 148 x 8 blocks

// Bulk-copy variant: one lane per warp asks the copy engine of the SM for the
// whole row (cp.async.bulk global -> shared, completion on an mbarrier), then
// for the row's way out (shared -> global). Rows must be multiples of 16 bytes
// on 16-byte boundaries. Waits are bounded. A row that does not arrive sets the
// status flag and ends the warp's work: its barrier never completed the phase and
// its copy may still be in flight, so neither the barrier nor the shared-memory
// stage may be used again; the warp gives every outstanding copy one more bounded
// wait and leaves its remaining rows untouched (the flag tells the caller).
constexpr int kBulkStages = 4;  // rows in flight per warp

__global__ void __launch_bounds__(kGatherBlock)
k_copy_miss_bulk(GatherWs ws, const char* uva_feats, int64_t uva_row_bytes, int64_t col_offset_bytes,
                 int64_t row_bytes, char* __restrict__ out, int32_t* status) {
  extern __shared__ __align__(128) unsigned char smem[];
  __shared__ __align__(8) uint64_t bars[(kGatherBlock / 32) * kBulkStages];
  const int lane = threadIdx.x & 31, wib = threadIdx.x >> 5;
  const int64_t warps = (int64_t)gridDim.x * (blockDim.x >> 5);
  const int64_t warp = (int64_t)blockIdx.x * (blockDim.x >> 5) + wib;
  const int64_t n = *ws.miss_count;
  unsigned char* wbuf = smem + (size_t)wib * kBulkStages * row_bytes;
  uint64_t* wbar = bars + wib * kBulkStages;
  if (lane == 0) {
    for (int k = 0; k < kBulkStages; ++k)
      asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_u32(wbar + k)));
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncwarp();
  if (lane != 0) return;   // one lane drives the copies of its warp
  uint32_t phase = 0;
  for (int64_t m0 = warp * kBulkStages; m0 < n; m0 += warps * kBulkStages) {
    const int cnt = n - m0 < kBulkStages ? (int)(n - m0) : kBulkStages;
    for (int k = 0; k < cnt; ++k) {
      const char* src = uva_feats + (-ws.src_pos[ws.miss_rows[m0 + k]] - 2) * uva_row_bytes + col_offset_bytes;
      const uint32_t bar = smem_u32(wbar + k), dst = smem_u32(wbuf + (size_t)k * row_bytes);
      asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"((uint32_t)row_bytes)
                   : "memory");
      asm volatile(
          "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
          "l"(src), "r"((uint32_t)row_bytes), "r"(bar)
          : "memory");
    }
    unsigned arrived = 0;
    for (int k = 0; k < cnt; ++k) {
      if (!mbar_wait_bounded(smem_u32(wbar + k), phase)) continue;
      arrived |= 1u << k;
      const int64_t r = ws.miss_rows[m0 + k];
      asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(out + r * row_bytes),
                   "r"(smem_u32(wbuf + (size_t)k * row_bytes)), "r"((uint32_t)row_bytes)
                   : "memory");
    }
    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
    asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
    if (arrived != (1u << cnt) - 1u) {
      atomicOr(status, APT_FLAG_PEER_TIMEOUT);
      for (int k = 0; k < cnt; ++k)   // one more bounded wait per copy that may still be in flight, then stop
        if (!(arrived & (1u << k))) mbar_wait_bounded(smem_u32(wbar + k), phase);
      return;
    }
    phase ^= 1;
  }
}

static int vec_width(uint64_t bits) {
  for (int w = 16; w > 1; w >>= 1)
    if ((bits & (uint64_t)(w - 1)) == 0) return w;
  return 1;
}

struct GatherArgs {
  const int64_t* index;
  int64_t num_rows;
  const int64_t* num_rows_dev;
  const int64_t* first_row_dev;
  const int64_t* feat_pos_map;
  int64_t num_nodes;
  const char* dev_feats;
  int64_t num_dev_rows, dev_row_bytes;
  const char* uva_feats;
  int64_t num_uva_rows, uva_row_bytes, uva_col_offset_bytes;
  char* out;
  int32_t* status_word;
};

// Blocks of one resident wave of a kernel on the current device (asked once per kernel and device).
template <typename K>
static int wave_blocks(K kernel, int block, size_t smem, int* cache, int* out) {
  int dev = 0;
  APT_CUDA(cudaGetDevice(&dev));
  const bool cacheable = dev >= 0 && dev < 64;
  if (!cacheable || cache[dev] == 0) {
    int per_sm = 0, sms = 0;
    APT_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, block, smem));
    APT_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    const int wave = (per_sm > 0 ? per_sm : 1) * (sms > 0 ? sms : kNumSMs);
    if (!cacheable) {
      *out = wave;
      return APT_OK;
    }
    cache[dev] = wave;
  }
  *out = cache[dev];
  return APT_OK;
}

// The launches shared by the workspace-taking and the allocation-free entry points.
static int gather_launch(const GatherArgs& a, GatherWs ws, cudaStream_t s) {
  uint64_t bits = (uint64_t)a.dev_row_bytes | (uintptr_t)a.out;
  if (a.num_dev_rows > 0) bits |= (uintptr_t)a.dev_feats;
  const int vw_hit = vec_width(bits);
  if (a.num_uva_rows > 0)
    bits |= (uint64_t)a.uva_row_bytes | (uint64_t)a.uva_col_offset_bytes | (uintptr_t)a.uva_feats;
  const int vw_miss = vec_width(bits);
  // the miss counter is the one word that has to start at zero
  APT_CUDA(cudaMemsetAsync(ws.miss_count, 0, sizeof(int32_t), s));

  {
    ProfScope prof("gather_classify", s);
    // one wave at most; a thread takes several rows when the request is larger
    const int grid = wave_grid(ceil_div(a.num_rows, 256), 8, 1);
    APT_LAUNCH(k_classify, grid, 256, 0, s, a.index, a.num_rows, a.num_rows_dev, a.first_row_dev, a.feat_pos_map,
               a.num_nodes, a.num_dev_rows, a.num_uva_rows, ws, a.status_word);
  }
  // blocks of the hit copy: at least 32 rows per warp, at most one resident wave
#define APT_HITS(V)                                                                        \
  do {                                                                                     \
    static int cache[64] = {};                                                             \
    int wave = 0;                                                                          \
    const int rc = wave_blocks(k_copy_hits<V>, kGatherBlock, 0, cache, &wave);             \
    if (rc != APT_OK) return rc;                                                           \
    const int64_t want = ceil_div(a.num_rows, (int64_t)(kGatherBlock / 32) * 32);          \
    const int grid = (int)(want < wave ? (want < 1 ? 1 : want) : wave);                    \
    ProfScope prof("gather_hit", s);                                                       \
    APT_LAUNCH(k_copy_hits<V>, grid, kGatherBlock, 0, s, a.num_rows, a.num_rows_dev,       \
               a.first_row_dev, ws.src_pos, a.dev_feats, a.dev_row_bytes, a.out);          \
  } while (0)
#define APT_HITS_STRIDED(V)                                                                \
  do {                                                                                     \
    const int grid =                                                                       \
        wave_grid(ceil_div(a.num_rows, (kGatherBlock / 32) * kRowsPerGroup), 8, g_hit_waves); \
    ProfScope prof("gather_hit", s);                                                       \
    APT_LAUNCH(k_copy_hits_strided<V>, grid, kGatherBlock, 0, s, a.num_rows, a.num_rows_dev, \
               a.first_row_dev, ws.src_pos, a.dev_feats, a.dev_row_bytes, a.out);          \
  } while (0)
#define APT_MISS(V)                                                                        \
  do {                                                                                     \
    ProfScope prof("gather_miss", s);                                                      \
    APT_LAUNCH(k_copy_miss<V>, g_miss_blocks, kGatherBlock, 0, s, ws, a.uva_feats,         \
               a.uva_row_bytes, a.uva_col_offset_bytes, a.dev_row_bytes,                   \
               (int64_t)g_miss_kb_per_block << 10, a.out);                                 \
  } while (0)
#define APT_BY_WIDTH(W, MACRO)                                                             \
  do {                                                                                     \
    switch (W) {                                                                           \
      case 16: MACRO(uint4); break;                                                        \
      case 8: MACRO(uint2); break;                                                         \
      case 4: MACRO(uint32_t); break;                                                      \
      case 2: MACRO(uint16_t); break;                                                      \
      default: MACRO(uint8_t); break;                                                      \
    }                                                                                      \
  } while (0)
  const int bulk_slots = (int)(kBulkSmem / ((size_t)kBulkWarps * 2 * (size_t)a.dev_row_bytes));
  if (g_hit_mode == 1 && vw_hit == 16 && bulk_slots >= 1) {
    static bool attr_set[64] = {};
    static int cache[64] = {};
    int dev = 0, wave = 0;
    APT_CUDA(cudaGetDevice(&dev));
    if (dev >= 0 && dev < 64 && !attr_set[dev]) {
      APT_CUDA(cudaFuncSetAttribute(k_copy_hits_bulk, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kBulkSmem));
      attr_set[dev] = true;
    }
    const int rc = wave_blocks(k_copy_hits_bulk, kBulkWarps * 32, kBulkSmem, cache, &wave);
    if (rc != APT_OK) return rc;
    const int slots = bulk_slots < 32 ? bulk_slots : 32;
    const int64_t want = ceil_div(a.num_rows, (int64_t)kBulkWarps * slots);
    const int grid = (int)(want < wave ? (want < 1 ? 1 : want) : wave);
    ProfScope prof("gather_hit", s);
    APT_LAUNCH(k_copy_hits_bulk, grid, kBulkWarps * 32, kBulkSmem, s, a.num_rows, a.num_rows_dev, a.first_row_dev,
               ws.src_pos, a.dev_feats, a.dev_row_bytes, slots, a.out, a.status_word);
  } else if (g_hit_mode == 2) {
    APT_BY_WIDTH(vw_hit, APT_HITS_STRIDED);
  } else {
    APT_BY_WIDTH(vw_hit, APT_HITS);
  }
  if (a.num_uva_rows > 0) {
    const size_t smem = (size_t)a.dev_row_bytes * kBulkStages * (kGatherBlock / 32);
    if (vw_miss == 16 && g_miss_mode == 1 && smem <= 200 * 1024) {
      APT_CUDA(cudaFuncSetAttribute(k_copy_miss_bulk, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
      ProfScope prof("gather_miss", s);
      APT_LAUNCH(k_copy_miss_bulk, g_miss_blocks, kGatherBlock, smem, s, ws, a.uva_feats, a.uva_row_bytes,
                 a.uva_col_offset_bytes, a.dev_row_bytes, a.out, a.status_word);
    } else {
      APT_BY_WIDTH(vw_miss, APT_MISS);
    }
  }
#undef APT_HITS
#undef APT_HITS_STRIDED
#undef APT_MISS
#undef APT_BY_WIDTH
  return APT_OK;
}

static int gather_check(const char* who, const GatherArgs& a) {
  APT_CHECK_ARG(a.num_rows >= 0 && a.num_rows < (int64_t)0x7fffffff, "%s: bad num_rows", who);
  APT_CHECK_ARG(a.dev_row_bytes > 0 && a.num_dev_rows >= 0 && a.num_uva_rows >= 0 && a.num_nodes >= 0,
                "%s: bad table sizes", who);
  APT_CHECK_ARG(a.num_uva_rows == 0 || (a.uva_col_offset_bytes >= 0 &&
                                         a.uva_col_offset_bytes + a.dev_row_bytes <= a.uva_row_bytes),
                "%s: column window [%lld,+%lld) outside a %lld-byte host row", who,
                (long long)a.uva_col_offset_bytes, (long long)a.dev_row_bytes, (long long)a.uva_row_bytes);
  if (a.num_rows == 0) return APT_OK;
  APT_CHECK_ARG(a.index && a.feat_pos_map && a.out && a.status_word, "%s: null pointer", who);
  APT_CHECK_ARG((a.num_dev_rows == 0 || a.dev_feats) && (a.num_uva_rows == 0 || a.uva_feats),
                "%s: null feature table", who);
  return APT_OK;
}

}  // namespace apt

extern "C" int apt_set_tunable(const char* name, int64_t value) {
  using namespace apt;
  APT_CHECK_ARG(name, "apt_set_tunable: null name");
  if (!strcmp(name, "gather_miss_mode") && value >= 0 && value <= 1) {
    g_miss_mode = (int)value;
  } else if (!strcmp(name, "gather_miss_blocks") && value >= 1 && value <= 65535) {
    g_miss_blocks = (int)value;
  } else if (!strcmp(name, "gather_miss_kb_per_block") && value >= 0 && value <= (1 << 20)) {
    g_miss_kb_per_block = (int)value;
  } else if (!strcmp(name, "gather_hit_mode") && value >= 0 && value <= 2) {
    g_hit_mode = (int)value;
  } else if (!strcmp(name, "gather_hit_waves") && value >= 1 && value <= 64) {
    g_hit_waves = (int)value;
  } else if (!strcmp(name, "relabel_small") && value >= 0 && value <= 1) {
    set_relabel_small(value != 0);
  } else {
    set_error("apt_set_tunable: unknown name or bad value: %s = %lld", name, (long long)value);
    return APT_ERR_BAD_ARG;
  }
  return APT_OK;
}

extern "C" size_t apt_gather_workspace_bytes(int64_t num_rows) {
  if (num_rows < 0) return 0;
  return apt::gather_layout(num_rows, nullptr, nullptr);
}

extern "C" int apt_gather_rows(const int64_t* index, int64_t num_rows,
                               const int64_t* num_rows_dev, const int64_t* feat_pos_map,
                               int64_t num_nodes, const void* dev_feats, int64_t num_dev_rows,
                               int64_t dev_row_bytes, const void* uva_feats,
                               int64_t num_uva_rows, int64_t uva_row_bytes,
                               int64_t uva_col_offset_bytes, void* out, void* workspace,
                               size_t workspace_bytes, int32_t* status_word, void* stream) {
  return apt_gather_rows_from(index, num_rows, num_rows_dev, nullptr, feat_pos_map, num_nodes, dev_feats,
                              num_dev_rows, dev_row_bytes, uva_feats, num_uva_rows, uva_row_bytes,
                              uva_col_offset_bytes, out, workspace, workspace_bytes, status_word, stream);
}

extern "C" int apt_gather_rows_from(const int64_t* index, int64_t num_rows,
                                    const int64_t* num_rows_dev, const int64_t* first_row_dev,
                                    const int64_t* feat_pos_map,
                                    int64_t num_nodes, const void* dev_feats, int64_t num_dev_rows,
                                    int64_t dev_row_bytes, const void* uva_feats,
                                    int64_t num_uva_rows, int64_t uva_row_bytes,
                                    int64_t uva_col_offset_bytes, void* out, void* workspace,
                                    size_t workspace_bytes, int32_t* status_word, void* stream) {
  using namespace apt;
  const GatherArgs a{index, num_rows, num_rows_dev, first_row_dev, feat_pos_map, num_nodes, (const char*)dev_feats,
                     num_dev_rows, dev_row_bytes, (const char*)uva_feats, num_uva_rows, uva_row_bytes,
                     uva_col_offset_bytes, (char*)out, status_word};
  const int rc = gather_check("apt_gather_rows", a);
  if (rc != APT_OK || num_rows == 0) return rc;
  APT_CHECK_ARG(workspace && ((uintptr_t)workspace & 255) == 0,
                "apt_gather_rows: workspace must be non-null and 256-byte aligned");
  GatherWs ws;
  const size_t need = gather_layout(num_rows, (char*)workspace, &ws);
  if (workspace_bytes < need) {
    set_error("apt_gather_rows: workspace %zu < %zu bytes", workspace_bytes, need);
    return APT_ERR_CAPACITY;
  }
  return gather_launch(a, ws, (cudaStream_t)stream);
}

// ---------------------------------------------------------------------------
// Gather without any allocation, for callers that must not allocate.
//
// The scratch that apt_gather_rows takes from its caller (decoded positions,
// miss list and miss counter) lives here in a fixed array inside the library's device image,
// sized for kStaticGatherMaxRows rows per call. The name g_gather_scratch is a
// host-side stand-in in host code, not a device address; the address kernels can
// use is asked for with cudaGetSymbolAddress while the caller's device is current.
namespace apt {

constexpr int64_t kStaticGatherMaxRows = 1 << 20;
constexpr size_t kStaticGatherBytes =
    (size_t)kStaticGatherMaxRows * 8 + (size_t)kStaticGatherMaxRows * 4 + 256;

static __device__ __align__(256) unsigned char g_gather_scratch[kStaticGatherBytes];

// Asked for on every call (a host-side lookup, no allocation): an address cached per device
// ordinal would go stale when that device's context is torn down and created again.
static int static_scratch(void** out) {
  void* p = nullptr;
  APT_CUDA(cudaGetSymbolAddress(&p, g_gather_scratch));
  APT_CHECK_ARG(p && ((uintptr_t)p & 255) == 0, "apt_gather_rows_static: scratch address %p", p);
  *out = p;
  return APT_OK;
}

}  // namespace apt

extern "C" int64_t apt_gather_static_max_rows(void) { return apt::kStaticGatherMaxRows; }

extern "C" int apt_gather_rows_static(const int64_t* index, int64_t num_rows,
                                      const int64_t* feat_pos_map, int64_t num_nodes,
                                      const void* dev_feats, int64_t num_dev_rows,
                                      int64_t dev_row_bytes, const void* uva_feats,
                                      int64_t num_uva_rows, int64_t uva_row_bytes,
                                      int64_t uva_col_offset_bytes, void* out,
                                      int32_t* status_word, void* stream) {
  using namespace apt;
  APT_CHECK_ARG(num_rows >= 0, "apt_gather_rows_static: negative num_rows");
  if (num_rows > kStaticGatherMaxRows) {
    set_error("apt_gather_rows_static: %lld rows exceed the built-in scratch of %lld rows per call; "
              "split the request or use apt_gather_rows with a caller workspace",
              (long long)num_rows, (long long)kStaticGatherMaxRows);
    return APT_ERR_CAPACITY;
  }
  const GatherArgs a{index, num_rows, nullptr, nullptr, feat_pos_map, num_nodes, (const char*)dev_feats,
                     num_dev_rows, dev_row_bytes, (const char*)uva_feats, num_uva_rows, uva_row_bytes,
                     uva_col_offset_bytes, (char*)out, status_word};
  int rc = gather_check("apt_gather_rows_static", a);
  if (rc != APT_OK || num_rows == 0) return rc;
  void* base = nullptr;
  rc = static_scratch(&base);
  if (rc != APT_OK) return rc;
  GatherWs ws;
  gather_layout(kStaticGatherMaxRows, (char*)base, &ws);
  // The array keeps the previous call's contents: gather_launch zeroes the miss
  // counter; positions and the miss list are rewritten for every row that is read.
  return gather_launch(a, ws, (cudaStream_t)stream);
}
