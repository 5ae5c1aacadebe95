// Row movers inside one GPU, and the all-to-all between GPUs done with plain
// stores into the receiving GPU's memory over NVLink.
//
// Inbox layout of every rank (one cudaMalloc, exported by CUDA IPC):
//   [0, 4096)             header: flags[2][32] (uint64: epoch << 32 | rows),
//                         the push kernel's block counter, and the two
//                         sequence numbers (pushes and waits completed)
//   [4096, ...)           data[parity][source rank][region_bytes]
// A push writes rows for peer r into data[parity][me] of r's inbox; when the
// last block of the push kernel has finished (block counter) it publishes
// flags[parity][me] on every peer. The wait kernel polls the local flags with
// a time bound; the pull kernel reads the rows out of the local inbox.
// The epoch of an all-to-all is not a kernel argument: push and wait kernels
// derive it from the sequence numbers in the local header and advance them,
// so an enqueued sequence can be captured in a CUDA graph and replayed.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdlib.h>
#include <string.h>

#include "common.cuh"

namespace apt {

constexpr int kMoveRows = 4;   // rows in flight per warp
constexpr int kMoveBlock = 256;
constexpr int kP2pMaxRanks = 32;
constexpr size_t kHeaderBytes = 16384;
constexpr size_t kCounterOffset = 2048;
constexpr size_t kPushSeqOffset = 2112;  // uint32: all-to-alls this rank has pushed
constexpr size_t kWaitSeqOffset = 2120;  // uint32: all-to-alls this rank has waited for
// uint32, sticky: a wait of this rank ran out of time. From then on the two-region rotation no longer
// proves that a peer has read a region before it is written again, so every later push, wait and fused
// all-to-all of this rank refuses to run (status APT_FLAG_PEER_TIMEOUT) until the inbox is created anew.
constexpr size_t kPoisonOffset = 2128;
// fused (chunked) all-to-all: flags[parity][source][chunk], one ticket counter per chunk, one for the end
constexpr int kMaxChunks = 8;
constexpr size_t kChunkFlagOffset = 4096;
constexpr size_t kChunkCounterOffset = 8192;
constexpr size_t kDoneCounterOffset = 8192 + 64;

template <typename V>
__device__ __forceinline__ V mv_load(const V* p) { return *p; }
template <>
__device__ __forceinline__ uint4 mv_load<uint4>(const uint4* p) { return ld_plain_16(p); }
template <typename V>
__device__ __forceinline__ void mv_store(V* p, V v) { *p = v; }
template <>
__device__ __forceinline__ void mv_store<uint4>(uint4* p, uint4 v) { st_plain_16(p, v); }

// Rows narrower than a warp of vectors are moved by a group of G lanes (the power of two covering
// the row's vectors), so that a warp moves 32 / G x kMoveRows rows at a time: an 8-byte id takes one
// lane, not a warp.
__device__ __forceinline__ int lane_group(int chunks) {
  int g = 1;
  while (g < chunks && g < 32) g <<= 1;
  return g;
}
static int lane_group_host(int64_t chunks) {
  int g = 1;
  while (g < chunks && g < 32) g <<= 1;
  return g;
}

// mode 0: out[i] = in[index[i]]   (i < n rows of out)
// mode 1: out[index[i]] = in[i]   (i < n rows of in)
template <typename V, int MODE>
__global__ void __launch_bounds__(kMoveBlock)
k_rows_move(const char* __restrict__ in, const int64_t* __restrict__ index, int64_t n,
            int64_t row_bytes, char* __restrict__ out) {
  const int lane = threadIdx.x & 31;
  const int64_t warps = (int64_t)gridDim.x * (blockDim.x >> 5);
  const int64_t warp = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int chunks = (int)(row_bytes / (int64_t)sizeof(V));
  const int G = lane_group(chunks), sub = lane % G, per = 32 / G;      // `per` rows side by side in a warp
  const int64_t step = (int64_t)per * kMoveRows;
  for (int64_t r0 = warp * step + lane / G; r0 < n; r0 += warps * step) {
    int64_t ix[kMoveRows];
#pragma unroll
    for (int k = 0; k < kMoveRows; ++k) ix[k] = r0 + (int64_t)k * per < n ? index[r0 + (int64_t)k * per] : (int64_t)-1;
    for (int c = sub; c < chunks; c += G) {
      V v[kMoveRows];
#pragma unroll
      for (int k = 0; k < kMoveRows; ++k) {
        const int64_t src = MODE == 0 ? ix[k] : r0 + (int64_t)k * per;
        if (ix[k] >= 0) v[k] = mv_load<V>((const V*)(in + src * row_bytes) + c);
      }
#pragma unroll
      for (int k = 0; k < kMoveRows; ++k) {
        const int64_t dst = MODE == 0 ? r0 + (int64_t)k * per : ix[k];
        if (ix[k] >= 0) mv_store<V>((V*)(out + dst * row_bytes) + c, v[k]);
      }
    }
  }
}

static int vec_width_of(uint64_t bits) {
  for (int w = 16; w > 1; w >>= 1)
    if ((bits & (uint64_t)(w - 1)) == 0) return w;
  return 1;
}

template <int MODE>
static int rows_move(const void* in, const int64_t* index, int64_t n, int64_t row_bytes,
                     void* out, cudaStream_t s, const char* tag) {
  if (n == 0) return APT_OK;
  APT_CHECK_ARG(in && index && out && row_bytes > 0 && n > 0, "%s: bad argument", tag);
  const int w = vec_width_of((uint64_t)row_bytes | (uintptr_t)in | (uintptr_t)out);
  const int64_t rows_per_warp = (int64_t)(32 / lane_group_host(row_bytes / w)) * kMoveRows;
  const int grid = wave_grid(ceil_div(n, (kMoveBlock / 32) * rows_per_warp), 8, 4);
  ProfScope prof(tag, s);
  const char* ip = (const char*)in;
  char* op = (char*)out;
  switch (w) {
    case 16: APT_LAUNCH((k_rows_move<uint4, MODE>), grid, kMoveBlock, 0, s, ip, index, n, row_bytes, op); break;
    case 8: APT_LAUNCH((k_rows_move<uint2, MODE>), grid, kMoveBlock, 0, s, ip, index, n, row_bytes, op); break;
    case 4: APT_LAUNCH((k_rows_move<uint32_t, MODE>), grid, kMoveBlock, 0, s, ip, index, n, row_bytes, op); break;
    case 2: APT_LAUNCH((k_rows_move<uint16_t, MODE>), grid, kMoveBlock, 0, s, ip, index, n, row_bytes, op); break;
    default: APT_LAUNCH((k_rows_move<uint8_t, MODE>), grid, kMoveBlock, 0, s, ip, index, n, row_bytes, op); break;
  }
  return APT_OK;
}

// ---------------------------------------------------------------- all-to-all
struct PeerTable {
  char* base[kP2pMaxRanks];
};

__device__ __forceinline__ void st_release_sys(uint64_t* p, uint64_t v) {
  asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ uint64_t ld_acquire_sys(const uint64_t* p) {
  uint64_t v;
  asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}

template <typename V>
__global__ void __launch_bounds__(kMoveBlock)
k_p2p_push(const char* __restrict__ src, const int64_t* __restrict__ src_index,
           int index_is_dest, const int64_t* __restrict__ send_offsets, int world_size,
           int me, int64_t row_bytes, size_t region_bytes, PeerTable peers, int32_t* status,
           size_t landing_off /* 0: rows go to the inbox region */, size_t landing_bytes) {
  __shared__ int64_t soff[kP2pMaxRanks + 1];
  __shared__ bool is_last;
  if (*(const volatile uint32_t*)(peers.base[me] + kPoisonOffset)) {
    // an earlier wait of this rank timed out: nothing is stored on any peer and no flag is published
    if (blockIdx.x == 0 && threadIdx.x == 0) atomicOr(status, APT_FLAG_PEER_TIMEOUT);
    return;
  }
  // Every block reads the sequence number before it takes its ticket below, and
  // the number only moves after the last ticket, so all blocks see the same epoch.
  uint32_t* push_seq = (uint32_t*)(peers.base[me] + kPushSeqOffset);
  const uint32_t epoch = *(volatile uint32_t*)push_seq + 1u;
  const int parity = (int)(epoch & 1u);
  if (threadIdx.x == 0) soff[0] = 0;
  if (threadIdx.x < world_size) soff[threadIdx.x + 1] = send_offsets[threadIdx.x];
  __syncthreads();
  const int64_t n = soff[world_size];
  const int lane = threadIdx.x & 31;
  const int64_t warps = (int64_t)gridDim.x * (blockDim.x >> 5);
  const int64_t warp = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int chunks = (int)(row_bytes / (int64_t)sizeof(V));
  const size_t slot_off = kHeaderBytes + ((size_t)parity * world_size + me) * region_bytes;
  // Direct placement: the receiver has told this rank, in the all-to-all waited for last, the
  // final row slot of every row it is about to get (8 bytes per row, in the inbox region of that
  // receiver here). Rows then go straight to that slot of the receiver's landing buffer and no
  // pull pass follows.
  const bool direct = landing_off != 0;
  const int64_t cap_rows = direct ? (int64_t)(region_bytes / 8) : (int64_t)(region_bytes / (size_t)row_bytes);
  const int64_t landing_rows = direct ? (int64_t)(landing_bytes / (size_t)row_bytes) : 0;
  const char* slot_lists = peers.base[me] + kHeaderBytes +
                           (size_t)(*(const volatile uint32_t*)(peers.base[me] + kWaitSeqOffset) & 1u) *
                               world_size * region_bytes;
  bool overflow = false;
  // Walking the stream in order would have every sender write to peer 0 first,
  // then peer 1, ...: all senders on one receiver's links at a time. Unless the
  // index names destinations (then the source order already mixes the peers),
  // work item t is row t / N of the bucket of peer (me + 1 + t % N) % N, so that
  // neighbouring warps feed different peers and senders start at different ones.
  const bool interleave = !(src_index && index_is_dest);
  int64_t work = n;
  if (interleave) {
    int64_t longest = 0;
    for (int r = 0; r < world_size; ++r) longest = max(longest, soff[r + 1] - soff[r]);
    work = longest * world_size;
  }
  const int G = lane_group(chunks), sub = lane % G, per = 32 / G;      // `per` rows side by side in a warp
  const int64_t step = (int64_t)per * kMoveRows;
  for (int64_t j0 = warp * step + lane / G; j0 < work; j0 += warps * step) {
    const char* sp[kMoveRows];
    char* dp[kMoveRows];
#pragma unroll
    for (int k = 0; k < kMoveRows; ++k) {
      // t walks the source rows when the index names destinations
      // (stream position j = index[t]) and the stream otherwise.
      const int64_t t = j0 + (int64_t)k * per;
      sp[k] = nullptr;
      dp[k] = nullptr;
      if (t < work) {
        int64_t j;
        int r = 0;
        if (interleave) {
          r = (int)((me + 1 + t % world_size) % world_size);
          const int64_t l = t / world_size;
          if (l >= soff[r + 1] - soff[r]) continue;   // this peer's bucket is shorter
          j = soff[r] + l;
        } else {
          j = src_index[t];
          if (j < 0 || j >= n) {
            overflow = true;
            continue;
          }
          while (soff[r + 1] <= j) ++r;
        }
        const int64_t local = j - soff[r];
        // index_is_dest == 2 (no index): every peer gets the same rows, bucket row l is source row l
        const int64_t srow = index_is_dest == 2 ? local
                             : (src_index && !index_is_dest) ? src_index[j] : (interleave ? j : t);
        if (local >= cap_rows) {
          overflow = true;
        } else if (direct) {
          const int64_t slot = ((const int64_t*)(slot_lists + (size_t)r * region_bytes))[local];
          if (slot < 0 || slot >= landing_rows) {
            overflow = true;
          } else {
            sp[k] = src + srow * row_bytes;
            dp[k] = peers.base[r] + landing_off + slot * row_bytes;
          }
        } else {
          sp[k] = src + srow * row_bytes;
          dp[k] = peers.base[r] + slot_off + local * row_bytes;
        }
      }
    }
    for (int c = sub; c < chunks; c += G) {
      V v[kMoveRows];
#pragma unroll
      for (int k = 0; k < kMoveRows; ++k)
        if (sp[k]) v[k] = mv_load<V>((const V*)sp[k] + c);
#pragma unroll
      for (int k = 0; k < kMoveRows; ++k)
        if (sp[k]) mv_store<V>((V*)dp[k] + c, v[k]);
    }
  }
  if (overflow) atomicOr(status, APT_FLAG_TABLE_FULL);
  // Publish: every thread orders its own stores system-wide, the last block to
  // arrive releases the flags on all peers.
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    int32_t* counter = (int32_t*)(peers.base[me] + kCounterOffset);
    const int ticket = atomicAdd(counter, 1);
    is_last = ticket == (int)gridDim.x - 1;
    if (is_last) *counter = 0;
  }
  __syncthreads();
  if (is_last && threadIdx.x < world_size) {
    __threadfence_system();
    const int r = threadIdx.x;
    int64_t rows = soff[r + 1] - soff[r];
    if (rows > cap_rows) rows = cap_rows;
    uint64_t* flag = (uint64_t*)peers.base[r] + (size_t)parity * kP2pMaxRanks + me;
    st_release_sys(flag, ((uint64_t)epoch << 32) | (uint64_t)(uint32_t)rows);
    if (r == 0) *(volatile uint32_t*)push_seq = epoch;
  }
}

__global__ void k_p2p_wait(char* local_base, int world_size, int64_t timeout_ns,
                           int64_t* __restrict__ out_counts, int32_t* status) {
  uint32_t* wait_seq = (uint32_t*)(local_base + kWaitSeqOffset);
  volatile uint32_t* poison = (volatile uint32_t*)(local_base + kPoisonOffset);
  const int r = threadIdx.x;
  const bool live = r < world_size;
  if (*poison) {   // refused: see kPoisonOffset
    if (live) out_counts[r] = 0;
    if (r == 0) {
      out_counts[world_size] = 0;
      atomicOr(status, APT_FLAG_PEER_TIMEOUT);
    }
    return;
  }
  const uint32_t epoch = *(volatile uint32_t*)wait_seq + 1u;
  const int parity = (int)(epoch & 1u);
  const uint64_t* flag = (const uint64_t*)local_base + (size_t)parity * kP2pMaxRanks + (live ? r : 0);
  const uint64_t t0 = global_timer_ns();
  uint64_t v = live ? ld_acquire_sys(flag) : ((uint64_t)epoch << 32);
  // Bounded both by wall time and by an iteration count, in case the timer stalls.
  for (uint64_t it = 0; (uint32_t)(v >> 32) != epoch && it < (1ull << 34); ++it) {
    if ((it & 63) == 63 && (int64_t)(global_timer_ns() - t0) > timeout_ns) break;
    __nanosleep(64);
    v = ld_acquire_sys(flag);
  }
  if (!live) v = (uint64_t)epoch << 32;  // lanes beyond the world contribute nothing
  int64_t got = 0;
  if ((uint32_t)(v >> 32) == epoch) {
    got = (int64_t)(uint32_t)v;
  } else {
    atomicOr(status, APT_FLAG_PEER_TIMEOUT);
    *poison = 1u;
  }
  if (live) out_counts[r] = got;
  // total over the peers, for operators chained behind the exchange
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) got += __shfl_down_sync(0xffffffffu, got, d);
  if (r == 0) {
    out_counts[world_size] = got;
    *(volatile uint32_t*)wait_seq = epoch;
  }
}

// mode 0: dst row j = concatenation row j; 1: dst row i = concat row index[i];
// 2: concat row j -> dst row index[j].
template <typename V, int MODE>
__global__ void __launch_bounds__(kMoveBlock)
k_p2p_pull(const char* __restrict__ local_base, const int64_t* __restrict__ recv_counts,
           int world_size, size_t region_bytes,
           const int64_t* __restrict__ index, int64_t num_dst_rows, int64_t row_bytes,
           char* __restrict__ dst) {
  __shared__ int64_t roff[kP2pMaxRanks + 1];
  // the all-to-all being read is the last one waited for
  const int parity = (int)(*(const volatile uint32_t*)(local_base + kWaitSeqOffset) & 1u);
  if (threadIdx.x == 0) {
    int64_t run = 0;
    roff[0] = 0;
    for (int r = 0; r < world_size; ++r) {
      run += recv_counts[r];
      roff[r + 1] = run;
    }
  }
  __syncthreads();
  const int64_t total = roff[world_size];
  // never more rows than the destination holds: a caller that sized it by an upper bound of what
  // the peers send loses the excess (and can see it in the counts) instead of writing past the end
  // (with a scatter index every concatenation row is visited; its destination row is checked instead)
  const int64_t n = MODE == 1 ? num_dst_rows : MODE == 2 ? total : (total < num_dst_rows ? total : num_dst_rows);
  const int lane = threadIdx.x & 31;
  const int64_t warps = (int64_t)gridDim.x * (blockDim.x >> 5);
  const int64_t warp = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int chunks = (int)(row_bytes / (int64_t)sizeof(V));
  const char* data = local_base + kHeaderBytes + (size_t)parity * world_size * region_bytes;
  const int G = lane_group(chunks), sub = lane % G, per = 32 / G;      // `per` rows side by side in a warp
  const int64_t step = (int64_t)per * kMoveRows;
  for (int64_t i0 = warp * step + lane / G; i0 < n; i0 += warps * step) {
    const char* sp[kMoveRows];
    char* dp[kMoveRows];
#pragma unroll
    for (int k = 0; k < kMoveRows; ++k) {
      const int64_t i = i0 + (int64_t)k * per;
      sp[k] = nullptr;
      dp[k] = nullptr;
      if (i < n) {
        const int64_t j = MODE == 1 ? index[i] : i;          // concatenation row
        const int64_t d = MODE == 2 ? index[i] : i;          // destination row
        if (j >= 0 && j < total && d >= 0 && d < num_dst_rows) {
          int r = 0;
          while (roff[r + 1] <= j) ++r;
          sp[k] = data + (size_t)r * region_bytes + (j - roff[r]) * row_bytes;
          dp[k] = dst + d * row_bytes;
        }
      }
    }
    for (int c = sub; c < chunks; c += G) {
      V v[kMoveRows];
#pragma unroll
      for (int k = 0; k < kMoveRows; ++k)
        if (sp[k]) v[k] = mv_load<V>((const V*)sp[k] + c);
#pragma unroll
      for (int k = 0; k < kMoveRows; ++k)
        if (sp[k]) mv_store<V>((V*)dp[k] + c, v[k]);
    }
  }
}


// Reduce-scatter epilogue. Every source has pushed the same number of rows (its
// partial results for this rank's segment) into its region of the local inbox;
// element i of dst is their sum, taken in rank order with an fp32 accumulator,
// so the result does not depend on which peer arrived first. A source whose
// count differs from num_rows is left out and APT_FLAG_SIZE_MISMATCH is set.
template <typename T> __device__ __forceinline__ float elem_to_f(T x);
template <> __device__ __forceinline__ float elem_to_f<float>(float x) { return x; }
template <> __device__ __forceinline__ float elem_to_f<__nv_bfloat16>(__nv_bfloat16 x) { return __bfloat162float(x); }
template <> __device__ __forceinline__ float elem_to_f<__half>(__half x) { return __half2float(x); }
template <typename T> __device__ __forceinline__ T elem_from_f(float x);
template <> __device__ __forceinline__ float elem_from_f<float>(float x) { return x; }
template <> __device__ __forceinline__ __nv_bfloat16 elem_from_f<__nv_bfloat16>(float x) { return __float2bfloat16_rn(x); }
template <> __device__ __forceinline__ __half elem_from_f<__half>(float x) { return __float2half_rn(x); }

template <typename T, int VE>
__global__ void __launch_bounds__(256)
k_p2p_pull_sum(const char* __restrict__ local_base, const int64_t* __restrict__ recv_counts,
               int world_size, size_t region_bytes, int64_t num_rows, int64_t row_elems,
               T* __restrict__ dst, int32_t* status) {
  __shared__ int ok[kP2pMaxRanks];
  const int parity = (int)(*(const volatile uint32_t*)(local_base + kWaitSeqOffset) & 1u);
  const char* data = local_base + kHeaderBytes + (size_t)parity * world_size * region_bytes;
  if (threadIdx.x < world_size) {
    ok[threadIdx.x] = recv_counts[threadIdx.x] == num_rows;
    if (!ok[threadIdx.x] && blockIdx.x == 0) atomicOr(status, APT_FLAG_SIZE_MISMATCH);
  }
  __syncthreads();
  struct alignas(sizeof(T) * VE) Vec { T v[VE]; };
  const int64_t nvec = num_rows * row_elems / VE;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += stride) {
    float acc[VE];
#pragma unroll
    for (int t = 0; t < VE; ++t) acc[t] = 0.f;
    for (int s = 0; s < world_size; ++s) {
      if (!ok[s]) continue;
      const Vec x = *((const Vec*)(data + (size_t)s * region_bytes) + i);
#pragma unroll
      for (int t = 0; t < VE; ++t) acc[t] += elem_to_f<T>(x.v[t]);
    }
    Vec o;
#pragma unroll
    for (int t = 0; t < VE; ++t) o.v[t] = elem_from_f<T>(acc[t]);
    *((Vec*)dst + i) = o;
  }
}

// ------------------------------------------------------------ fused all-to-all
// Push, wait and pull in ONE cooperative kernel, so that the local pass that
// permutes received rows to their final place overlaps the NVLink transfer
// instead of following it. Every (sender, receiver) bucket is cut into C chunks
// of rows. All blocks are co-resident (cooperative launch) and run
//     push(0); push(1), pull(0); push(2), pull(1); ... ; pull(C-1)
// where push(c) stores this rank's chunk c into every peer's inbox and the last
// block to finish it releases flag (epoch, rows) for chunk c on every peer, and
// pull(c) waits (bounded) for chunk c of every source and moves those rows from
// the local inbox to `dst`. A flag for chunk k depends only on pushes <= k and
// pulls <= k-2 of its sender, so no wait can close a cycle between GPUs.
struct FusedA2A {
  const char* src;
  const int64_t* src_index;     // as in k_p2p_push
  int index_is_dest;
  const int64_t* send_offsets;  // inclusive, world_size entries (device)
  const int64_t* recv_offsets;  // inclusive, world_size entries (device): rows each source will send
  const int64_t* pull_index;    // NULL: dst row j = concatenation row j; else dst row i = row pull_index[i]
  int64_t num_dst_rows;
  char* dst;
  int64_t row_bytes;
  int chunks, world_size, me;
  size_t region_bytes;
  PeerTable peers;
  int64_t timeout_ns;
  int32_t* status;
};

__device__ __forceinline__ int64_t chunk_lo(int64_t len, int c, int chunks) { return len * c / chunks; }

__global__ void __launch_bounds__(kMoveBlock)
k_p2p_fused(FusedA2A a) {
  __shared__ int64_t soff[kP2pMaxRanks + 1], roff[kP2pMaxRanks + 1];
  __shared__ int flag_ok;
  const int ws = a.world_size, me = a.me;
  if (threadIdx.x == 0) soff[0] = roff[0] = 0;
  if (threadIdx.x < ws) {
    soff[threadIdx.x + 1] = a.send_offsets[threadIdx.x];
    roff[threadIdx.x + 1] = a.recv_offsets[threadIdx.x];
  }
  char* local = a.peers.base[me];
  if (*(const volatile uint32_t*)(local + kPoisonOffset)) {   // refused: see kPoisonOffset
    if (blockIdx.x == 0 && threadIdx.x == 0) atomicOr(a.status, APT_FLAG_PEER_TIMEOUT);
    return;
  }
  uint32_t* push_seq = (uint32_t*)(local + kPushSeqOffset);
  const uint32_t epoch = *(volatile uint32_t*)push_seq + 1u;   // moves only after every block has finished
  const int parity = (int)(epoch & 1u);
  __syncthreads();
  const int64_t n_send = soff[ws], n_recv = roff[ws];
  const int lane = threadIdx.x & 31;
  const int64_t warps = (int64_t)gridDim.x * (blockDim.x >> 5);
  const int64_t warp = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int chunks_per_row = (int)(a.row_bytes / 16);
  const size_t my_slot = kHeaderBytes + ((size_t)parity * ws + me) * a.region_bytes;
  const char* inbox = local + kHeaderBytes + (size_t)parity * ws * a.region_bytes;
  const int64_t cap_rows = (int64_t)(a.region_bytes / (size_t)a.row_bytes);
  const bool by_dest = a.src_index && a.index_is_dest;
  bool overflow = false, timed_out = false;

  for (int step = 0; step <= a.chunks; ++step) {
    // ---------------------------------------------------------------- push(step)
    if (step < a.chunks) {
      const int c = step;
      int64_t work = n_send;
      if (!by_dest) {
        int64_t longest = 0;
        for (int r = 0; r < ws; ++r) {
          const int64_t len = soff[r + 1] - soff[r];
          longest = max(longest, chunk_lo(len, c + 1, a.chunks) - chunk_lo(len, c, a.chunks));
        }
        work = longest * ws;
      }
      for (int64_t t0 = warp * kMoveRows; t0 < work; t0 += warps * kMoveRows) {
        const char* sp[kMoveRows];
        char* dp[kMoveRows];
#pragma unroll
        for (int k = 0; k < kMoveRows; ++k) {
          const int64_t t = t0 + k;
          sp[k] = nullptr;
          dp[k] = nullptr;
          if (t >= work) continue;
          int r;
          int64_t l, srow;
          if (!by_dest) {
            r = (int)((me + 1 + t % ws) % ws);
            const int64_t len = soff[r + 1] - soff[r];
            l = chunk_lo(len, c, a.chunks) + t / ws;
            if (l >= chunk_lo(len, c + 1, a.chunks)) continue;
            const int64_t j = soff[r] + l;
            srow = a.src_index ? a.src_index[j] : j;
          } else {
            const int64_t j = a.src_index[t];
            if (j < 0 || j >= n_send) {
              overflow = true;
              continue;
            }
            r = 0;
            while (soff[r + 1] <= j) ++r;
            l = j - soff[r];
            const int64_t len = soff[r + 1] - soff[r];
            if (l < chunk_lo(len, c, a.chunks) || l >= chunk_lo(len, c + 1, a.chunks)) continue;
            srow = t;
          }
          if (l >= cap_rows) {
            overflow = true;
            continue;
          }
          sp[k] = a.src + srow * a.row_bytes;
          dp[k] = a.peers.base[r] + my_slot + l * a.row_bytes;
        }
        for (int q = lane; q < chunks_per_row; q += 32) {
          uint4 v[kMoveRows];
#pragma unroll
          for (int k = 0; k < kMoveRows; ++k)
            if (sp[k]) v[k] = ld_plain_16((const uint4*)sp[k] + q);
#pragma unroll
          for (int k = 0; k < kMoveRows; ++k)
            if (sp[k]) st_plain_16((uint4*)dp[k] + q, v[k]);
        }
      }
      // chunk c of this rank is complete on every peer once all blocks have passed here
      __threadfence_system();
      __syncthreads();
      if (threadIdx.x == 0) {
        int32_t* counter = (int32_t*)(local + kChunkCounterOffset) + c;
        if (atomicAdd(counter, 1) == (int)gridDim.x - 1) {
          *counter = 0;
          __threadfence_system();
          for (int r = 0; r < ws; ++r) {
            const int64_t len = soff[r + 1] - soff[r];
            int64_t rows = chunk_lo(len, c + 1, a.chunks) - chunk_lo(len, c, a.chunks);
            uint64_t* flag = (uint64_t*)(a.peers.base[r] + kChunkFlagOffset) +
                             ((size_t)parity * kP2pMaxRanks + me) * kMaxChunks + c;
            st_release_sys(flag, ((uint64_t)epoch << 32) | (uint64_t)(uint32_t)rows);
          }
        }
      }
    }
    // ---------------------------------------------------------------- pull(step - 1)
    if (step >= 1) {
      const int c = step - 1;
      if (threadIdx.x == 0) {
        int ok = 1;
        const uint64_t t0 = global_timer_ns();
        for (int s = 0; s < ws && ok; ++s) {
          const uint64_t* flag = (const uint64_t*)(local + kChunkFlagOffset) +
                                 ((size_t)parity * kP2pMaxRanks + s) * kMaxChunks + c;
          uint64_t v = ld_acquire_sys(flag);
          for (uint64_t it = 0; (uint32_t)(v >> 32) != epoch && it < (1ull << 34); ++it) {
            if ((it & 63) == 63 && (int64_t)(global_timer_ns() - t0) > a.timeout_ns) break;
            __nanosleep(64);
            v = ld_acquire_sys(flag);
          }
          if ((uint32_t)(v >> 32) != epoch) ok = 0;
        }
        flag_ok = ok;
      }
      __syncthreads();
      if (!flag_ok) {
        timed_out = true;      // keep going: the other phases must still be signalled
      } else if (a.pull_index) {
        // gather: dst row i takes concatenation row pull_index[i] if that row lies in chunk c
        for (int64_t i0 = warp * kMoveRows; i0 < a.num_dst_rows; i0 += warps * kMoveRows) {
          const char* sp[kMoveRows];
#pragma unroll
          for (int k = 0; k < kMoveRows; ++k) {
            sp[k] = nullptr;
            const int64_t i = i0 + k;
            if (i >= a.num_dst_rows) continue;
            const int64_t j = a.pull_index[i];
            if (j < 0 || j >= n_recv) continue;
            int s = 0;
            while (roff[s + 1] <= j) ++s;
            const int64_t l = j - roff[s], len = roff[s + 1] - roff[s];
            if (l < chunk_lo(len, c, a.chunks) || l >= chunk_lo(len, c + 1, a.chunks) || l >= cap_rows) continue;
            sp[k] = inbox + (size_t)s * a.region_bytes + l * a.row_bytes;
          }
          for (int q = lane; q < chunks_per_row; q += 32) {
            uint4 v[kMoveRows];
#pragma unroll
            for (int k = 0; k < kMoveRows; ++k)
              if (sp[k]) v[k] = ld_plain_16((const uint4*)sp[k] + q);
#pragma unroll
            for (int k = 0; k < kMoveRows; ++k)
              if (sp[k]) st_plain_16((uint4*)(a.dst + (i0 + k) * a.row_bytes) + q, v[k]);
          }
        }
      } else {
        // contiguous: concatenation row roff[s] + l lands at the same dst row
        int64_t longest = 0;
        for (int s = 0; s < ws; ++s) {
          const int64_t len = roff[s + 1] - roff[s];
          longest = max(longest, chunk_lo(len, c + 1, a.chunks) - chunk_lo(len, c, a.chunks));
        }
        const int64_t work = longest * ws;
        for (int64_t t0 = warp * kMoveRows; t0 < work; t0 += warps * kMoveRows) {
          const char* sp[kMoveRows];
          char* dp[kMoveRows];
#pragma unroll
          for (int k = 0; k < kMoveRows; ++k) {
            sp[k] = nullptr;
            dp[k] = nullptr;
            const int64_t t = t0 + k;
            if (t >= work) continue;
            const int s = (int)(t % ws);
            const int64_t len = roff[s + 1] - roff[s];
            const int64_t l = chunk_lo(len, c, a.chunks) + t / ws;
            if (l >= chunk_lo(len, c + 1, a.chunks) || l >= cap_rows) continue;
            sp[k] = inbox + (size_t)s * a.region_bytes + l * a.row_bytes;
            dp[k] = a.dst + (roff[s] + l) * a.row_bytes;
          }
          for (int q = lane; q < chunks_per_row; q += 32) {
            uint4 v[kMoveRows];
#pragma unroll
            for (int k = 0; k < kMoveRows; ++k)
              if (sp[k]) v[k] = ld_plain_16((const uint4*)sp[k] + q);
#pragma unroll
            for (int k = 0; k < kMoveRows; ++k)
              if (sp[k]) st_plain_16((uint4*)dp[k] + q, v[k]);
          }
        }
      }
      __syncthreads();   // flag_ok is rewritten in the next step
    }
  }
  if (overflow) atomicOr(a.status, APT_FLAG_TABLE_FULL);
  if (timed_out && threadIdx.x == 0) atomicOr(a.status, APT_FLAG_PEER_TIMEOUT);
  // the poison word is written by the last block below, after every block has read it above
  // the last block to finish advances both sequence numbers: the next all-to-all, fused or not,
  // then uses the other half of the inbox
  __syncthreads();
  if (threadIdx.x == 0) {
    int32_t* done = (int32_t*)(local + kDoneCounterOffset);
    int32_t* tflag = (int32_t*)(local + kDoneCounterOffset) + 1;   // some block of this launch timed out
    if (timed_out) atomicOr(tflag, 1);
    __threadfence();
    if (atomicAdd(done, 1) == (int)gridDim.x - 1) {
      *done = 0;
      if (atomicExch(tflag, 0)) *(volatile uint32_t*)(local + kPoisonOffset) = 1u;
      *(volatile uint32_t*)push_seq = epoch;
      *(volatile uint32_t*)(local + kWaitSeqOffset) = epoch;
    }
  }
}

}  // namespace apt

struct apt_p2p {
  int rank, world_size, device;
  size_t region_bytes, alloc_bytes;
  size_t landing_bytes;   // bytes of one landing buffer (0: none)
  int landing_slots;      // landing buffers behind the inbox, used in turn
  char* local_base;
  char* peer_base[apt::kP2pMaxRanks];
  bool peer_is_ipc[apt::kP2pMaxRanks];
};

extern "C" int apt_rows_gather(const void* in, const int64_t* index, int64_t num_out_rows,
                               int64_t row_bytes, void* out, void* stream) {
  return apt::rows_move<0>(in, index, num_out_rows, row_bytes, out, (cudaStream_t)stream, "rows_gather");
}
extern "C" int apt_rows_scatter(const void* in, const int64_t* index, int64_t num_in_rows,
                                int64_t row_bytes, void* out, void* stream) {
  return apt::rows_move<1>(in, index, num_in_rows, row_bytes, out, (cudaStream_t)stream, "rows_scatter");
}

extern "C" int apt_p2p_create(int rank, int world_size, size_t region_bytes, apt_p2p** out_ctx,
                              void* out_handle) {
  return apt_p2p_create_landing(rank, world_size, region_bytes, 0, 0, out_ctx, out_handle);
}

extern "C" int apt_p2p_create_landing(int rank, int world_size, size_t region_bytes, size_t landing_bytes,
                                      int landing_slots, apt_p2p** out_ctx, void* out_handle) {
  using namespace apt;
  APT_CHECK_ARG(out_ctx && world_size >= 1 && world_size <= kP2pMaxRanks && rank >= 0 &&
                    rank < world_size && region_bytes > 0,
                "apt_p2p_create: bad argument (rank %d of %d)", rank, world_size);
  APT_CHECK_ARG(landing_slots >= 0 && landing_slots <= 64 && (landing_slots == 0) == (landing_bytes == 0),
                "apt_p2p_create_landing: %d landing buffers of %zu bytes", landing_slots, landing_bytes);
  apt_p2p* c = new apt_p2p();
  c->rank = rank;
  c->world_size = world_size;
  c->region_bytes = align_up(region_bytes, 256);
  c->landing_bytes = align_up(landing_bytes, 256);
  c->landing_slots = landing_slots;
  c->alloc_bytes = kHeaderBytes + 2 * (size_t)world_size * c->region_bytes + (size_t)landing_slots * c->landing_bytes;
  for (int r = 0; r < kP2pMaxRanks; ++r) {
    c->peer_base[r] = nullptr;
    c->peer_is_ipc[r] = false;
  }
  cudaError_t e = cudaGetDevice(&c->device);
  if (e == cudaSuccess) e = cudaMalloc((void**)&c->local_base, c->alloc_bytes);
  if (e == cudaSuccess) e = cudaMemset(c->local_base, 0, kHeaderBytes);
  if (e == cudaSuccess && out_handle) {
    cudaIpcMemHandle_t h;
    e = cudaIpcGetMemHandle(&h, c->local_base);
    if (e == cudaSuccess) memcpy(out_handle, &h, sizeof(h));
  }
  if (e != cudaSuccess) {
    set_error("apt_p2p_create: %s", cudaGetErrorString(e));
    if (c->local_base) cudaFree(c->local_base);
    delete c;
    return APT_ERR_CUDA;
  }
  c->peer_base[rank] = c->local_base;
  *out_ctx = c;
  return APT_OK;
}

extern "C" int apt_p2p_attach(apt_p2p* ctx, int peer, const void* handle) {
  using namespace apt;
  APT_CHECK_ARG(ctx && handle && peer >= 0 && peer < ctx->world_size, "apt_p2p_attach: bad argument");
  if (peer == ctx->rank) return APT_OK;
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, sizeof(h));
  void* p = nullptr;
  APT_CUDA(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
  ctx->peer_base[peer] = (char*)p;
  ctx->peer_is_ipc[peer] = true;
  return APT_OK;
}

extern "C" int apt_p2p_attach_ptr(apt_p2p* ctx, int peer, void* base) {
  using namespace apt;
  APT_CHECK_ARG(ctx && base && peer >= 0 && peer < ctx->world_size, "apt_p2p_attach_ptr: bad argument");
  if (peer == ctx->rank) return APT_OK;
  ctx->peer_base[peer] = (char*)base;
  ctx->peer_is_ipc[peer] = false;
  return APT_OK;
}

extern "C" void* apt_p2p_local_base(apt_p2p* ctx) { return ctx ? ctx->local_base : nullptr; }
extern "C" size_t apt_p2p_region_bytes(const apt_p2p* ctx) { return ctx ? ctx->region_bytes : 0; }
extern "C" size_t apt_p2p_landing_bytes(const apt_p2p* ctx) { return ctx ? ctx->landing_bytes : 0; }
extern "C" void* apt_p2p_landing(apt_p2p* ctx, int slot) {
  if (!ctx || slot < 0 || slot >= ctx->landing_slots) return nullptr;
  return ctx->local_base + apt::kHeaderBytes + 2 * (size_t)ctx->world_size * ctx->region_bytes +
         (size_t)slot * ctx->landing_bytes;
}

extern "C" int apt_p2p_destroy(apt_p2p* ctx) {
  if (!ctx) return APT_OK;
  for (int r = 0; r < ctx->world_size; ++r)
    if (ctx->peer_is_ipc[r] && ctx->peer_base[r]) cudaIpcCloseMemHandle(ctx->peer_base[r]);
  if (ctx->local_base) cudaFree(ctx->local_base);
  delete ctx;
  return APT_OK;
}

static int p2p_push_launch(apt_p2p* ctx, const void* src, const int64_t* src_index, int index_is_dest,
                           const int64_t* send_offsets, int64_t max_rows, int64_t row_bytes, size_t landing_off,
                           int32_t* status_word, void* stream) {
  using namespace apt;
  APT_CHECK_ARG(ctx && send_offsets && status_word && row_bytes > 0 && max_rows >= 0, "apt_p2p_push: bad argument");
  APT_CHECK_ARG(max_rows == 0 || src, "apt_p2p_push: null source");
  APT_CHECK_ARG((size_t)row_bytes <= ctx->region_bytes, "apt_p2p_push: a %lld-byte row exceeds the %zu-byte region",
                (long long)row_bytes, ctx->region_bytes);
  for (int r = 0; r < ctx->world_size; ++r)
    APT_CHECK_ARG(ctx->peer_base[r], "apt_p2p_push: peer %d is not attached", r);
  cudaStream_t s = (cudaStream_t)stream;
  PeerTable pt;
  for (int r = 0; r < kP2pMaxRanks; ++r) pt.base[r] = ctx->peer_base[r];
  const int w = vec_width_of((uint64_t)row_bytes | (uintptr_t)src | (uint64_t)ctx->region_bytes);
  const int64_t rows_per_warp = (int64_t)(32 / lane_group_host(row_bytes / w)) * kMoveRows;
  const int grid = wave_grid(ceil_div(max_rows > 0 ? max_rows : 1, (kMoveBlock / 32) * rows_per_warp), 8, 2);
  ProfScope prof("p2p_push", s);
  const char* sp = (const char*)src;
#define APT_PUSH(V)                                                                       \
  APT_LAUNCH(k_p2p_push<V>, grid, kMoveBlock, 0, s, sp, src_index, index_is_dest, send_offsets,          \
             ctx->world_size, ctx->rank, row_bytes, ctx->region_bytes, pt, status_word, landing_off,     \
             ctx->landing_bytes)
  switch (w) {
    case 16: APT_PUSH(uint4); break;
    case 8: APT_PUSH(uint2); break;
    case 4: APT_PUSH(uint32_t); break;
    case 2: APT_PUSH(uint16_t); break;
    default: APT_PUSH(uint8_t); break;
  }
#undef APT_PUSH
  return APT_OK;
}

extern "C" int apt_p2p_push(apt_p2p* ctx, const void* src, const int64_t* src_index,
                            int index_is_dest, const int64_t* send_offsets, int64_t max_rows, int64_t row_bytes,
                            int32_t* status_word, void* stream) {
  return p2p_push_launch(ctx, src, src_index, index_is_dest, send_offsets, max_rows, row_bytes, 0, status_word,
                         stream);
}

extern "C" int apt_p2p_push_direct(apt_p2p* ctx, const void* src, const int64_t* src_index, int index_is_dest,
                                   const int64_t* send_offsets, int64_t max_rows, int64_t row_bytes,
                                   int landing_slot, int32_t* status_word, void* stream) {
  using namespace apt;
  APT_CHECK_ARG(ctx && landing_slot >= 0 && landing_slot < ctx->landing_slots,
                "apt_p2p_push_direct: landing buffer %d of %d", landing_slot, ctx ? ctx->landing_slots : 0);
  const size_t off = kHeaderBytes + 2 * (size_t)ctx->world_size * ctx->region_bytes +
                     (size_t)landing_slot * ctx->landing_bytes;
  return p2p_push_launch(ctx, src, src_index, index_is_dest, send_offsets, max_rows, row_bytes, off, status_word,
                         stream);
}

// Bound of a device-side wait when the caller passes none: APT_P2P_TIMEOUT_MS (read once), default
// 30 s. It has to exceed the largest skew between ranks that is not a failure (a rank that is still
// registering host memory, loading data or compiling while its peers already wait).
static int64_t default_timeout_ns() {
  static const int64_t ns = [] {
    const char* e = getenv("APT_P2P_TIMEOUT_MS");
    long long ms = e ? atoll(e) : 0;
    if (ms <= 0) ms = 30000;
    if (ms > 600000) ms = 600000;
    return (int64_t)ms * 1000000ll;
  }();
  return ns;
}

extern "C" int64_t apt_p2p_default_timeout_ns(void) { return default_timeout_ns(); }

extern "C" int apt_p2p_probe_copy(apt_p2p* ctx, int peer, size_t nbytes, void* stream) {
  using namespace apt;
  APT_CHECK_ARG(ctx && peer >= 0 && peer < ctx->world_size && ctx->peer_base[peer], "apt_p2p_probe_copy: bad peer");
  APT_CHECK_ARG(nbytes > 0 && nbytes <= ctx->region_bytes, "apt_p2p_probe_copy: %zu bytes exceed a %zu-byte region",
                nbytes, ctx->region_bytes);
  // region [0][me] of the peer's inbox is written by this rank only; the source is the same region here
  const size_t off = kHeaderBytes + (size_t)ctx->rank * ctx->region_bytes;
  APT_CUDA(cudaMemcpyAsync(ctx->peer_base[peer] + off, ctx->local_base + off, nbytes, cudaMemcpyDeviceToDevice,
                           (cudaStream_t)stream));
  return APT_OK;
}

extern "C" int apt_p2p_poisoned(apt_p2p* ctx, int* out_poisoned) {
  using namespace apt;
  APT_CHECK_ARG(ctx && out_poisoned, "apt_p2p_poisoned: bad argument");
  uint32_t v = 0;
  APT_CUDA(cudaMemcpy(&v, ctx->local_base + kPoisonOffset, sizeof(v), cudaMemcpyDeviceToHost));
  *out_poisoned = v != 0;
  return APT_OK;
}

extern "C" int apt_p2p_wait(apt_p2p* ctx, int64_t* out_recv_counts, int32_t* status_word,
                            int64_t timeout_ns, void* stream) {
  using namespace apt;
  APT_CHECK_ARG(ctx && out_recv_counts && status_word, "apt_p2p_wait: bad argument");
  if (timeout_ns <= 0) timeout_ns = default_timeout_ns();
  cudaStream_t s = (cudaStream_t)stream;
  ProfScope prof("p2p_wait", s);
  APT_LAUNCH(k_p2p_wait, 1, 32, 0, s, ctx->local_base, ctx->world_size, timeout_ns, out_recv_counts,
             status_word);
  return APT_OK;
}

extern "C" int apt_p2p_pull(apt_p2p* ctx, const int64_t* recv_counts, const int64_t* dst_index,
                            int index_is_source, int64_t num_dst_rows, int64_t max_rows,
                            int64_t row_bytes, void* dst, void* stream) {
  using namespace apt;
  APT_CHECK_ARG(ctx && recv_counts && row_bytes > 0 && max_rows >= 0, "apt_p2p_pull: bad argument");
  if (max_rows == 0) return APT_OK;
  APT_CHECK_ARG(dst, "apt_p2p_pull: null destination");
  cudaStream_t s = (cudaStream_t)stream;
  const int w = vec_width_of((uint64_t)row_bytes | (uintptr_t)dst | (uint64_t)ctx->region_bytes);
  const int64_t rows_per_warp = (int64_t)(32 / lane_group_host(row_bytes / w)) * kMoveRows;
  const int grid = wave_grid(ceil_div(max_rows, (kMoveBlock / 32) * rows_per_warp), 8, 4);
  const int mode = !dst_index ? 0 : (index_is_source ? 1 : 2);
  ProfScope prof("p2p_pull", s);
  char* dp = (char*)dst;
#define APT_PULL(V, M)                                                                     \
  APT_LAUNCH((k_p2p_pull<V, M>), grid, kMoveBlock, 0, s, ctx->local_base, recv_counts,     \
             ctx->world_size, ctx->region_bytes, dst_index, num_dst_rows,                  \
             row_bytes, dp)
#define APT_PULL_W(V)                                   \
  do {                                                  \
    if (mode == 0) { APT_PULL(V, 0); }                  \
    else if (mode == 1) { APT_PULL(V, 1); }             \
    else { APT_PULL(V, 2); }                            \
  } while (0)
  switch (w) {
    case 16: APT_PULL_W(uint4); break;
    case 8: APT_PULL_W(uint2); break;
    case 4: APT_PULL_W(uint32_t); break;
    case 2: APT_PULL_W(uint16_t); break;
    default: APT_PULL_W(uint8_t); break;
  }
#undef APT_PULL_W
#undef APT_PULL
  return APT_OK;
}

extern "C" int apt_p2p_pull_sum(apt_p2p* ctx, const int64_t* recv_counts, int dtype, int64_t num_rows,
                                int64_t row_elems, void* dst, int32_t* status_word, void* stream) {
  using namespace apt;
  APT_CHECK_ARG(ctx && recv_counts && status_word && num_rows >= 0 && row_elems > 0, "apt_p2p_pull_sum: bad argument");
  APT_CHECK_ARG(dtype >= APT_F32 && dtype <= APT_F16, "apt_p2p_pull_sum: dtype %d", dtype);
  if (num_rows == 0) return APT_OK;
  APT_CHECK_ARG(dst, "apt_p2p_pull_sum: null destination");
  const size_t esz = dtype == APT_F32 ? 4 : 2;
  APT_CHECK_ARG((size_t)num_rows * row_elems * esz <= ctx->region_bytes,
                "apt_p2p_pull_sum: %lld rows of %lld elements exceed the %zu-byte region", (long long)num_rows,
                (long long)row_elems, ctx->region_bytes);
  cudaStream_t s = (cudaStream_t)stream;
  const int64_t total = num_rows * row_elems;
  const bool vec = (((uint64_t)(total * esz) | (uintptr_t)dst) & 15) == 0;
  const int ve = vec ? (int)(16 / esz) : 1;
  const int grid = wave_grid(ceil_div(total / ve, 256), 8, 4);
  ProfScope prof("p2p_pull_sum", s);
#define APT_PULL_SUM(T, VE)                                                                              \
  APT_LAUNCH((k_p2p_pull_sum<T, VE>), grid, 256, 0, s, ctx->local_base, recv_counts, ctx->world_size,    \
             ctx->region_bytes, num_rows, row_elems, (T*)dst, status_word)
  if (dtype == APT_F32) {
    if (vec) { APT_PULL_SUM(float, 4); } else { APT_PULL_SUM(float, 1); }
  } else if (dtype == APT_BF16) {
    if (vec) { APT_PULL_SUM(__nv_bfloat16, 8); } else { APT_PULL_SUM(__nv_bfloat16, 1); }
  } else {
    if (vec) { APT_PULL_SUM(__half, 8); } else { APT_PULL_SUM(__half, 1); }
  }
#undef APT_PULL_SUM
  return APT_OK;
}

extern "C" int apt_p2p_alltoall_fused(apt_p2p* ctx, const void* src, const int64_t* src_index,
                                      int index_is_dest, const int64_t* send_offsets,
                                      const int64_t* recv_offsets, const int64_t* pull_index,
                                      int64_t num_dst_rows, int64_t row_bytes, int chunks, void* dst,
                                      int32_t* status_word, int64_t timeout_ns, void* stream) {
  using namespace apt;
  APT_CHECK_ARG(ctx && send_offsets && recv_offsets && status_word && row_bytes > 0 && num_dst_rows >= 0,
                "apt_p2p_alltoall_fused: bad argument");
  APT_CHECK_ARG(chunks >= 1 && chunks <= kMaxChunks, "apt_p2p_alltoall_fused: chunks %d outside [1,%d]", chunks,
                kMaxChunks);
  // src / dst may be NULL on a rank that sends / receives nothing; it still takes part
  APT_CHECK_ARG(row_bytes % 16 == 0 && ((uintptr_t)src & 15) == 0 && ((uintptr_t)dst & 15) == 0 &&
                    (ctx->region_bytes & 15) == 0,
                "apt_p2p_alltoall_fused: rows must be multiples of 16 bytes on 16-byte boundaries");
  APT_CHECK_ARG((size_t)row_bytes <= ctx->region_bytes, "apt_p2p_alltoall_fused: row larger than an inbox region");
  for (int r = 0; r < ctx->world_size; ++r)
    APT_CHECK_ARG(ctx->peer_base[r], "apt_p2p_alltoall_fused: peer %d is not attached", r);
  if (timeout_ns <= 0) timeout_ns = default_timeout_ns();
  FusedA2A a;
  a.src = (const char*)src;
  a.src_index = src_index;
  a.index_is_dest = index_is_dest;
  a.send_offsets = send_offsets;
  a.recv_offsets = recv_offsets;
  a.pull_index = pull_index;
  a.num_dst_rows = num_dst_rows;
  a.dst = (char*)dst;
  a.row_bytes = row_bytes;
  a.chunks = chunks;
  a.world_size = ctx->world_size;
  a.me = ctx->rank;
  a.region_bytes = ctx->region_bytes;
  for (int r = 0; r < kP2pMaxRanks; ++r) a.peers.base[r] = ctx->peer_base[r];
  a.timeout_ns = timeout_ns;
  a.status = status_word;
  // every block has to be resident at once (blocks wait for each other's chunks): cooperative launch
  int per_sm = 0;
  APT_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, k_p2p_fused, kMoveBlock, 0));
  APT_CHECK_ARG(per_sm >= 1, "apt_p2p_alltoall_fused: kernel does not fit an SM");
  int dev = 0, sms = 0;
  APT_CUDA(cudaGetDevice(&dev));
  APT_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  const int grid = sms * (per_sm < 4 ? per_sm : 4);
  void* args[] = {&a};
  cudaStream_t s = (cudaStream_t)stream;
  ProfScope prof("p2p_fused", s);
  APT_CUDA(cudaLaunchCooperativeKernel((const void*)k_p2p_fused, dim3(grid), dim3(kMoveBlock), args, 0, s));
  count_launch();
  return APT_OK;
}
