// The open-addressing table of the relabelling and its workspace layout, shared
// by the relabel kernels (relabel.cu) and by the sampling kernel that inserts
// the ids it draws while they are still in registers (sample_kernels.cuh).
#pragma once

#include "common.cuh"

namespace apt {

constexpr unsigned long long kEmptyKey = ~0ull;
constexpr uint32_t kNoPos = 0xffffffffu;

// key, smallest position and new id of one distinct id: 16 bytes, one sector.
struct Slot {
  unsigned long long key;
  uint32_t min_pos;
  uint32_t new_id;
};

// Items per tile of the ordered compaction: 512 threads x 4 consecutive items.
constexpr int kScanThreads = 512;
constexpr int kScanItems = 4;
constexpr int kScanTile = kScanThreads * kScanItems;

struct RelabelWs {
  Slot* slots;            // [cap_ws] all-0xff between calls
  int32_t* slot_of;       // [items_ws] slot of every item of the running call, -1: not in the table
  ScanCtrl* ctrl;         // [1]
  uint64_t* tile_state;   // [tiles_ws] epoch << 34 | status << 32 | count
  int64_t items_ws;       // items this workspace was sized for
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

#ifdef __CUDACC__
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

__device__ __forceinline__ uint32_t hash_id(int64_t key) {
  // 64 -> 32 bit finaliser (splitmix64 constants); ids are often dense, so the
  // low bits alone would cluster under linear probing.
  uint64_t x = (uint64_t)key;
  x ^= x >> 30; x *= 0xbf58476d1ce4e5b9ull;
  x ^= x >> 27; x *= 0x94d049bb133111ebull;
  x ^= x >> 31;
  return (uint32_t)x;
}

// Enters item `pos` with id `id` into the table: claims (or finds) the id's slot,
// lowers the slot's smallest position to `pos` and returns the slot number.
// Negative ids are not ids (the all-ones key marks an empty slot, and -1 is what
// an operator upstream writes for an id it could not resolve): they get no slot,
// return -1 and raise APT_FLAG_ID_OUT_OF_RANGE. A full table returns -1 with
// APT_FLAG_TABLE_FULL.
__device__ __forceinline__ int32_t table_insert(Slot* slots, uint32_t cap, int64_t id, uint32_t pos,
                                                int* flags) {
  if (id < 0) {
    *flags |= APT_FLAG_ID_OUT_OF_RANGE;
    return -1;
  }
  const unsigned long long key = (unsigned long long)id;
  uint32_t at = (uint32_t)(((uint64_t)hash_id(id) * cap) >> 32);
  for (uint32_t probe = 0; probe < cap; ++probe) {
    Slot* s = slots + at;
    unsigned long long prev = *(volatile unsigned long long*)&s->key;
    if (prev == kEmptyKey) prev = atomicCAS(&s->key, kEmptyKey, key);
    if (prev == kEmptyKey || prev == key) {
      // the minimum only falls: an id that many items share (a hub) stops costing atomics on one
      // address as soon as an early position has arrived
      if (*(volatile uint32_t*)&s->min_pos > pos) atomicMin(&s->min_pos, pos);
      return (int32_t)at;
    }
    at = at + 1 == cap ? 0 : at + 1;
  }
  *flags |= APT_FLAG_TABLE_FULL;
  return -1;
}
#endif  // __CUDACC__

}  // namespace apt
