// Cache-aware feature-row gather.
//
//   k_gather_hits  decodes and copies in one launch. Every warp owns one contiguous
//                  share of the requested rows. For 32 rows at a time lane k looks up
//                  id -> feat_pos_map entry of row k (the two dependent loads happen
//                  once per 32 rows and for all warps of the SM at the same time), rows
//                  that live in host memory are appended (warp-aggregated) to a miss
//                  list, rows in the cache are copied HBM -> HBM, R of them in flight
//                  per warp, each lane one 16-byte vector per row, all loads issued
//                  before the first store. The grid is one resident wave and the rows
//                  are split evenly over its warps, so there is no partial last wave.
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

constexpr int kRowsPerGroup = 4;   // rows whose loads are in flight together (miss copy)
constexpr int kGatherBlock = 256;

struct GatherWs {
  int64_t* miss_pos;   // [n]  host-table row of every miss
  int32_t* miss_rows;  // [n]  output row of every miss
  int32_t* miss_count; // [1]
};

static size_t gather_layout(int64_t n, char* base, GatherWs* ws) {
  const size_t rows = (size_t)(n > 0 ? n : 1);
  const size_t b0 = align_up(rows * 8, 256);
  const size_t b1 = align_up(rows * 4, 256);
  if (ws) {
    ws->miss_pos = (int64_t*)base;
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

// Output rows [first, n) (first from a device word when first_dev is given, else 0):
// p = feat_pos_map[index[r]]: p >= 0 cache row (copied here), p < -1 host row -(p)-2
// (queued for the miss copy), p == -1 no such row (zeros + flag).
template <typename V, int R>
__global__ void __launch_bounds__(kGatherBlock, R >= 8 ? 2 : 4)
k_gather_hits(const int64_t* __restrict__ index, int64_t n, const int64_t* __restrict__ n_dev,
              const int64_t* __restrict__ first_dev, const int64_t* __restrict__ pos_map,
              int64_t num_nodes, int64_t num_dev_rows, int64_t num_uva_rows,
              const char* __restrict__ dev_feats, int64_t row_bytes, char* __restrict__ out,
              GatherWs ws, int32_t* status) {
  n = effective_n(n, n_dev);
  int64_t first = first_dev ? *first_dev : 0;
  first = first < 0 ? 0 : (first > n ? n : first);
  const int lane = threadIdx.x & 31;
  const int64_t warps = (int64_t)gridDim.x * (blockDim.x >> 5);
  const int64_t warp = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int64_t m = n - first;
  const int64_t lo = first + m * warp / warps, hi = first + m * (warp + 1) / warps;
  const int chunks = (int)(row_bytes / (int64_t)sizeof(V));
  int flags = 0;
  for (int64_t base = lo; base < hi; base += 32) {
    const int cnt = hi - base < 32 ? (int)(hi - base) : 32;
    int64_t p = -2;   // lanes past the share: nothing to do (any p < -1 is skipped by the copy below)
    if (lane < cnt) {
      const int64_t id = index[base + lane];
      p = -1;
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
    }
    const bool miss = lane < cnt && p < -1;
    const unsigned mm = __ballot_sync(0xffffffffu, miss);
    if (mm) {
      int at = 0;
      const int leader = __ffs(mm) - 1;
      if (lane == leader) at = atomicAdd(ws.miss_count, __popc(mm));
      at = __shfl_sync(0xffffffffu, at, leader) + __popc(mm & ((1u << lane) - 1u));
      if (miss) {
        ws.miss_rows[at] = (int32_t)(base + lane);
        ws.miss_pos[at] = -p - 2;
      }
    }
    for (int k0 = 0; k0 < cnt; k0 += R) {
      // the trip count is the same for all lanes, so that the shuffles below are convergent
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
  if (flags) atomicOr(status, flags);
}

template <typename V>
__global__ void __launch_bounds__(kGatherBlock)
k_copy_miss(GatherWs ws, const char* __restrict__ uva_feats, int64_t uva_row_bytes,
            int64_t col_offset_bytes, int64_t row_bytes, char* __restrict__ out) {
  const int lane = threadIdx.x & 31;
  const int64_t warps = (int64_t)gridDim.x * (blockDim.x >> 5);
  const int64_t warp = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int64_t n = *ws.miss_count;
  const int chunks = (int)(row_bytes / (int64_t)sizeof(V));
  for (int64_t m0 = warp * kRowsPerGroup; m0 < n; m0 += warps * kRowsPerGroup) {
    int64_t r[kRowsPerGroup], p[kRowsPerGroup];
#pragma unroll
    for (int k = 0; k < kRowsPerGroup; ++k) {
      r[k] = m0 + k < n ? (int64_t)ws.miss_rows[m0 + k] : (int64_t)-1;
      p[k] = m0 + k < n ? ws.miss_pos[m0 + k] : (int64_t)0;
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
static int g_hit_rows = 8;       // rows in flight per warp of the hit copy (4 or 8)

// Bulk-copy variant: one lane per warp asks the copy engine of the SM for the
// whole row (cp.async.bulk global -> shared, completion on an mbarrier), then
// for the row's way out (shared -> global). Rows must be multiples of 16 bytes
// on 16-byte boundaries. Waits are bounded. A row that does not arrive sets the
// status flag and ends the warp's work: its barrier never completed the phase and
// its copy may still be in flight, so neither the barrier nor the shared-memory
// stage may be used again; the warp gives every outstanding copy one more bounded
// wait and leaves its remaining rows untouched (the flag tells the caller).
constexpr int kBulkStages = 4;  // rows in flight per warp

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}

__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t phase) {
  uint32_t done = 0;
  const uint64_t t0 = global_timer_ns();
  for (int it = 0; it < (1 << 20) && !done; ++it) {
    asm volatile(
        "{ .reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }"
        : "=r"(done)
        : "r"(bar), "r"(phase)
        : "memory");
    if (!done && (it & 15) == 15 && global_timer_ns() - t0 > 1000000000ull) break;  // 1 s
  }
  return done != 0;
}

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
      const char* src = uva_feats + ws.miss_pos[m0 + k] * uva_row_bytes + col_offset_bytes;
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

// One resident wave of the hit copy for vector type V and R rows in flight.
template <typename V, int R>
static int hit_wave_blocks(int* out) {
  static int cached[64] = {};
  int dev = 0;
  APT_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64 || cached[dev] == 0) {
    int per_sm = 0, sms = 0;
    APT_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, k_gather_hits<V, R>, kGatherBlock, 0));
    APT_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    const int wave = (per_sm > 0 ? per_sm : 1) * (sms > 0 ? sms : kNumSMs);
    if (dev < 0 || dev >= 64) {
      *out = wave;
      return APT_OK;
    }
    cached[dev] = wave;
  }
  *out = cached[dev];
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

#define APT_HITS_R(V, R)                                                                   \
  do {                                                                                     \
    int wave = 0;                                                                          \
    const int rc = hit_wave_blocks<V, R>(&wave);                                           \
    if (rc != APT_OK) return rc;                                                           \
    /* at least 2 R rows per warp, at most one resident wave */                            \
    const int64_t want = ceil_div(a.num_rows, (int64_t)(kGatherBlock / 32) * 2 * R);       \
    const int grid = (int)(want < wave ? (want < 1 ? 1 : want) : wave);                    \
    ProfScope prof("gather_hit", s);                                                       \
    APT_LAUNCH((k_gather_hits<V, R>), grid, kGatherBlock, 0, s, a.index, a.num_rows,       \
               a.num_rows_dev, a.first_row_dev, a.feat_pos_map, a.num_nodes,               \
               a.num_dev_rows, a.num_uva_rows, a.dev_feats, a.dev_row_bytes, a.out, ws,    \
               a.status_word);                                                             \
  } while (0)
#define APT_HITS(V)                                                                        \
  do {                                                                                     \
    if (g_hit_rows >= 8 && a.dev_row_bytes <= 1024) APT_HITS_R(V, 8);                      \
    else APT_HITS_R(V, 4);                                                                 \
  } while (0)
#define APT_MISS(V)                                                                        \
  do {                                                                                     \
    ProfScope prof("gather_miss", s);                                                      \
    APT_LAUNCH(k_copy_miss<V>, g_miss_blocks, kGatherBlock, 0, s, ws, a.uva_feats,         \
               a.uva_row_bytes, a.uva_col_offset_bytes, a.dev_row_bytes, a.out);           \
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
  APT_BY_WIDTH(vw_hit, APT_HITS);
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
#undef APT_HITS_R
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
  } else if (!strcmp(name, "gather_hit_rows") && (value == 4 || value == 8)) {
    g_hit_rows = (int)value;
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
// The scratch that apt_gather_rows takes from its caller (the miss list: host-table
// row and output row of every miss, and the miss counter) lives here in a fixed array inside the library's device image,
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
  // counter, and only the list entries below the new count are ever read.
  return gather_launch(a, ws, (cudaStream_t)stream);
}
