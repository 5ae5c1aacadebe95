// Shared device/host helpers of libapt_b200: error plumbing, launch counting,
// optional per-kernel event timing, Philox4x32-10, 16-byte row movers and a
// block-wide exclusive scan.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include "../../include/apt_b200.h"

namespace apt {

// ---------------------------------------------------------------- host side
void set_error(const char* fmt, ...);
void count_launch();
// RAII bracket that records events around one tagged kernel when profiling is on.
struct ProfScope {
  ProfScope(const char* tag, cudaStream_t s);
  ~ProfScope();
  const char* tag;
  cudaStream_t stream;
  int slot;
};

#define APT_CHECK_ARG(cond, ...)        \
  do {                                  \
    if (!(cond)) {                      \
      apt::set_error(__VA_ARGS__);      \
      return APT_ERR_BAD_ARG;           \
    }                                   \
  } while (0)

#define APT_CUDA(call)                                                        \
  do {                                                                        \
    cudaError_t e__ = (call);                                                 \
    if (e__ != cudaSuccess) {                                                 \
      apt::set_error("%s:%d %s -> %s", __FILE__, __LINE__, #call,             \
                     cudaGetErrorString(e__));                                \
      return APT_ERR_CUDA;                                                    \
    }                                                                         \
  } while (0)

// Launch + count + launch-error check (cudaPeekAtLastError keeps sticky
// errors visible to the caller's own checks).
#define APT_LAUNCH(kernel, grid, block, smem, stream, ...)                    \
  do {                                                                        \
    kernel<<<(grid), (block), (smem), (stream)>>>(__VA_ARGS__);               \
    apt::count_launch();                                                      \
    cudaError_t e__ = cudaPeekAtLastError();                                  \
    if (e__ != cudaSuccess) {                                                 \
      apt::set_error("%s:%d launch of %s -> %s", __FILE__, __LINE__, #kernel, \
                     cudaGetErrorString(e__));                                \
      return APT_ERR_CUDA;                                                    \
    }                                                                         \
  } while (0)

void set_relabel_small(bool on);   // relabel.cu: one-block shared-memory path for small layers

constexpr int kNumSMs = 148;  // B200: 2 dies x 74 SMs

inline int64_t ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }
inline size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

// Grid for a grid-stride kernel: enough blocks for `work_blocks`, rounded up
// to whole waves of `per_sm` resident blocks on each of the 148 SMs, capped
// at `max_waves` waves.
inline int wave_grid(int64_t work_blocks, int per_sm, int max_waves = 8) {
  if (work_blocks < 1) work_blocks = 1;
  const int64_t wave = (int64_t)kNumSMs * per_sm;
  int64_t waves = ceil_div(work_blocks, wave);
  if (waves > max_waves) waves = max_waves;
  int64_t g = work_blocks < wave ? work_blocks : waves * wave;
  return (int)g;
}

// -------------------------------------------------------------- device side
#ifdef __CUDACC__

// Philox4x32-10 (Salmon et al., "Parallel random numbers: as easy as 1, 2, 3",
// SC'11). Counter-based: the same (key, counter) gives the same four words on
// the GPU and in the CPU oracle.
struct Philox4 {
  uint32_t w[4];
};

__host__ __device__ inline Philox4 philox4x32_10(uint32_t c0, uint32_t c1,
                                                 uint32_t c2, uint32_t c3,
                                                 uint32_t k0, uint32_t k1) {
  const uint32_t M0 = 0xD2511F53u, M1 = 0xCD9E8D57u;
  const uint32_t W0 = 0x9E3779B9u, W1 = 0xBB67AE85u;
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    const uint64_t p0 = (uint64_t)M0 * c0;
    const uint64_t p1 = (uint64_t)M1 * c2;
    const uint32_t n0 = (uint32_t)(p1 >> 32) ^ c1 ^ k0;
    const uint32_t n1 = (uint32_t)p1;
    const uint32_t n2 = (uint32_t)(p0 >> 32) ^ c3 ^ k1;
    const uint32_t n3 = (uint32_t)p0;
    c0 = n0; c1 = n1; c2 = n2; c3 = n3;
    k0 += W0; k1 += W1;
  }
  Philox4 out;
  out.w[0] = c0; out.w[1] = c1; out.w[2] = c2; out.w[3] = c3;
  return out;
}

__device__ __forceinline__ uint4 ld_stream_16(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}
__device__ __forceinline__ void st_stream_16(void* p, uint4 v) {
  asm volatile("st.global.cs.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x),
               "r"(v.y), "r"(v.z), "r"(v.w)
               : "memory");
}
// Plain (coherent) 16-byte store: used for stores into a peer GPU's memory.
__device__ __forceinline__ void st_plain_16(void* p, uint4 v) {
  asm volatile("st.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x),
               "r"(v.y), "r"(v.z), "r"(v.w)
               : "memory");
}
// Coherent 16-byte load (no .nc): for memory another GPU has just written.
__device__ __forceinline__ uint4 ld_plain_16(const void* p) {
  uint4 v;
  asm volatile("ld.global.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p)
               : "memory");
  return v;
}

__device__ __forceinline__ uint64_t global_timer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

constexpr int kMaxRanks = 32;

struct OwnerParams {
  int world_size;
  int shuffle_id_offset;
  int rank, node_beg, node_end;
};

// Owner of id v: the last rank d with min_vids[d] <= v, starting from
// shuffle_id_offset; owners outside this machine's rank window fall back to
// the calling rank.
__device__ __forceinline__ int owner_of(int64_t v, const int64_t* mv, const OwnerParams& p) {
  int d = p.shuffle_id_offset;
  while (d + 1 < p.world_size && mv[d + 1] <= v) ++d;
  if (d < p.node_beg || d >= p.node_end) d = p.rank;
  return d;
}

// Sizes may live on the device: an operator chained behind another one takes
// its element count from a device word (what the previous kernel produced), so
// that the host never has to wait for it. `n_host` is then only an upper bound
// that sized the grid and the buffers.
__device__ __forceinline__ int64_t effective_n(int64_t n_host, const int64_t* n_dev) {
  if (!n_dev) return n_host;
  const int64_t v = *n_dev;
  return v < 0 ? 0 : (v < n_host ? v : n_host);
}

// Exclusive scan of one int per thread over a block of up to 1024 threads.
// Returns the thread's exclusive prefix; *total gets the block sum (all threads).
// `warp_sums` is a shared array of 33 ints. Ends with a __syncthreads().
__device__ __forceinline__ int block_exclusive_scan(int v, int* warp_sums,
                                                    int* total) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int inc = v;
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    int t = __shfl_up_sync(0xffffffffu, inc, d);
    if (lane >= d) inc += t;
  }
  if (lane == 31) warp_sums[warp] = inc;
  __syncthreads();
  if (warp == 0) {
    const int nw = (blockDim.x + 31) >> 5;
    int s = lane < nw ? warp_sums[lane] : 0;
    int sinc = s;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      int t = __shfl_up_sync(0xffffffffu, sinc, d);
      if (lane >= d) sinc += t;
    }
    warp_sums[lane] = sinc - s;  // exclusive warp offset
    if (lane == 31) warp_sums[32] = sinc;
  }
  __syncthreads();
  const int res = warp_sums[warp] + inc - v;
  *total = warp_sums[32];
  __syncthreads();
  return res;
}

// Sum of sums[0..count) computed by the whole block (every thread must call it
// and gets the result). Lets the block that owns tile `b` find the offset of its
// tile from the per-tile counts of an earlier kernel without a scan kernel in
// between. `scratch` is a shared array of 33 ints. Ends with a __syncthreads().
__device__ __forceinline__ int block_sum_of(const int32_t* __restrict__ sums, int count, int* scratch) {
  int acc = 0;
  for (int t = threadIdx.x; t < count; t += blockDim.x) acc += sums[t];
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) acc += __shfl_down_sync(0xffffffffu, acc, d);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) scratch[warp] = acc;
  __syncthreads();
  if (warp == 0) {
    const int nw = (blockDim.x + 31) >> 5;
    int v = lane < nw ? scratch[lane] : 0;
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) v += __shfl_down_sync(0xffffffffu, v, d);
    if (lane == 0) scratch[32] = v;
  }
  __syncthreads();
  const int total = scratch[32];
  __syncthreads();
  return total;
}

// ---- single-pass ordered prefix over tiles (decoupled look-back) ----------------------
// Tiles are handed out in launch order by a ticket, so every tile before a running tile is
// running or finished. A tile publishes its own count as soon as it has it, then looks back
// over the tiles before it (32 at a time, nearest first) until it meets one that has published
// its inclusive prefix; its own inclusive prefix follows. State words carry the epoch of the
// call (epoch << 34 | status << 32 | count), so nothing has to be cleared between calls; the
// control words start at zero once and every call leaves ticket and done at zero.
struct ScanCtrl {
  uint32_t ticket;   // next tile number to hand out
  uint32_t done;     // blocks that have finished
  uint32_t epoch;    // calls completed on this workspace
  uint32_t pad;
};
constexpr uint32_t kTileAggregate = 1u, kTileInclusive = 2u;
constexpr int kLookbackSpinLimit = 1 << 22;   // about a second of polling; never reached unless a block died

__device__ __forceinline__ uint64_t ld_tile_state(const uint64_t* p) {
  uint64_t v;
  asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_tile_state(uint64_t* p, uint64_t v) {
  asm volatile("st.release.gpu.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}

// Thread 0 of the block: takes the block's tile number and the epoch of this call.
__device__ __forceinline__ void tile_ticket(ScanCtrl* ctrl, uint32_t* tile, uint32_t* epoch) {
  *epoch = *(volatile uint32_t*)&ctrl->epoch + 1u;   // moves only after the last block is done
  *tile = atomicAdd(&ctrl->ticket, 1u);
}

// Called by all 32 lanes of one warp: publishes `total` for `tile` and returns the sum of the totals of
// all tiles before it. A look-back that exhausts its polling limit raises `give_up_flag` in *status and
// returns what it has (the ids of this tile are then wrong).
__device__ __forceinline__ uint32_t tile_lookback(uint64_t* tile_state, uint32_t tile, uint32_t epoch_full,
                                                  uint32_t total, int32_t* status, int give_up_flag) {
  const int lane = threadIdx.x & 31;
  const uint32_t epoch = epoch_full & 0x3fffffffu;
  uint32_t before = 0;
  if (lane == 0)
    st_tile_state(tile_state + tile,
                  ((uint64_t)epoch << 34) | ((uint64_t)(tile == 0 ? kTileInclusive : kTileAggregate) << 32) | total);
  if (tile > 0) {
    int64_t look = (int64_t)tile - 1;
    int spins = 0;
    for (;;) {
      const int64_t idx = look - lane;
      const uint64_t w = idx >= 0 ? ld_tile_state(tile_state + idx) : 0ull;
      const bool ready = idx < 0 || (uint32_t)(w >> 34) == epoch;
      const bool incl = idx < 0 || (ready && ((uint32_t)(w >> 32) & 3u) == kTileInclusive);
      const unsigned ready_mask = __ballot_sync(0xffffffffu, ready);
      const unsigned incl_mask = __ballot_sync(0xffffffffu, incl);
      const int stop = incl_mask ? __ffs(incl_mask) - 1 : 31;          // nearest tile with a full prefix
      const unsigned need = stop == 31 ? 0xffffffffu : ((2u << stop) - 1u);
      if ((ready_mask & need) == need) {
        uint32_t v = (lane <= stop && idx >= 0) ? (uint32_t)w : 0u;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
        before += v;
        if (incl_mask) break;
        look -= 32;
        spins = 0;
      } else if (++spins > kLookbackSpinLimit) {
        if (lane == 0) atomicOr(status, give_up_flag);
        break;
      } else {
        __nanosleep(40);
      }
    }
    if (lane == 0)
      st_tile_state(tile_state + tile, ((uint64_t)epoch << 34) | ((uint64_t)kTileInclusive << 32) | (before + total));
  }
  return before;
}

// Thread 0 of every block, at its end: the last block to finish puts the ticket back and advances the epoch.
__device__ __forceinline__ void tile_done(ScanCtrl* ctrl, uint32_t epoch_full) {
  __threadfence();
  if (atomicAdd(&ctrl->done, 1u) == gridDim.x - 1) {
    ctrl->done = 0;
    ctrl->ticket = 0;
    __threadfence();
    *(volatile uint32_t*)&ctrl->epoch = epoch_full;
  }
}

#endif  // __CUDACC__

}  // namespace apt
