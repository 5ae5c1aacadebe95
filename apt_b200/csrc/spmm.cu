// Segment-batched COO SpMM (sum reduce) and SDDMM over sampled blocks.
//
// A sampled block lists its edges grouped by destination (col is
// non-decreasing). SpMM then needs no atomics: k_edge_ranges turns col into a
// CSR-style range per output row (and detects the unsorted case), and
// k_spmm_rows gives each output row to a group of G lanes (G = the power of
// two covering the row's 16-byte vectors, at most a warp) that walks the
// row's edges in order, keeps the running sum in fp32 registers and writes the
// row once. Every output row is written, so the caller's buffer needs no
// zero-fill. For unsorted col (the backward call, which swaps row and col) the
// edges are first grouped by a counting sort on the destination (histogram,
// tile sums, offsets, fill: four small kernels that return at once when col is
// grouped already) and the same row kernel walks them through the resulting
// order. Scattering edge by edge with vector red.add instead took 25 ms for the
// 1.01 M-edge backward block of the benchmark (64 M 16-byte reductions), against
// 0.15 ms for the row kernel. The decision is taken on the device from a flag
// word, so the host never waits.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <math.h>

#include <algorithm>

#include "common.cuh"

namespace apt {

constexpr int kMaxSegments = 64;

static int pow2_at_least_fwd(int64_t x) {
  int g = 1;
  while (g < x && g < 32) g <<= 1;
  return g;
}

struct SegTable {
  // Copied into shared memory by each block: first edge and row bases per segment.
  const int64_t* coo_off;
  const int64_t* in_off;
  const int64_t* out_off;
  int nseg;
};

__device__ __forceinline__ int seg_of(const int64_t* coo, int nseg, int64_t e) {
  int k = 0;
  while (k + 1 < nseg && coo[k + 1] <= e) ++k;
  return k;
}

constexpr int kDstTile = 1024;

struct SpmmWs {
  int64_t* range;     // [num_out_rows + 1] first edge (or first slot of `order`) of each output row
  int32_t* flags;     // [0] = 1 when col is not grouped by output row
  int32_t* cursor;    // [num_out_rows] counting sort: edges per row, then the fill cursor
  int32_t* tile_sum;  // [tiles + 1]
  int32_t* order;     // [num_edges] edge ids grouped by output row (only when col is not grouped)
  int64_t* long_rows; // [num_edges / kLongRow + 2] output rows with more than kLongRow edges
  // flags[2] counts them
};

// Rows with more edges than this (hub nodes of a power-law graph reach tens of
// thousands in the backward call) are left to k_spmm_long, one block per row.
constexpr int kLongRow = 256;

static size_t spmm_layout(int64_t num_out_rows, int64_t num_edges, char* base, SpmmWs* ws) {
  const size_t b0 = align_up((size_t)(num_out_rows + 1) * 8, 256);
  const size_t b1 = 256;
  const size_t b2 = align_up((size_t)(num_out_rows > 0 ? num_out_rows : 1) * 4, 256);
  const size_t b3 = align_up((size_t)(ceil_div(num_out_rows > 0 ? num_out_rows : 1, kDstTile) + 1) * 4, 256);
  const size_t b4 = align_up((size_t)(num_edges > 0 ? num_edges : 1) * 4, 256);
  const size_t b5 = align_up((size_t)(num_edges / 256 + 2) * 8, 256);
  if (ws) {
    ws->long_rows = (int64_t*)(base + b0 + b1 + b2 + b3 + b4);
    ws->range = (int64_t*)base;
    ws->flags = (int32_t*)(base + b0);
    ws->cursor = (int32_t*)(base + b0 + b1);
    ws->tile_sum = (int32_t*)(base + b0 + b1 + b2);
    ws->order = (int32_t*)(base + b0 + b1 + b2 + b3);
  }
  return b0 + b1 + b2 + b3 + b4 + b5;
}

// ---- element <-> fp32 helpers ------------------------------------------------
template <typename T> struct Elem;
template <> struct Elem<float> {
  static __device__ __forceinline__ float to_f(float x) { return x; }
  static __device__ __forceinline__ float from_f(float x) { return x; }
};
template <> struct Elem<__nv_bfloat16> {
  static __device__ __forceinline__ float to_f(__nv_bfloat16 x) { return __bfloat162float(x); }
  static __device__ __forceinline__ __nv_bfloat16 from_f(float x) { return __float2bfloat16_rn(x); }
};
template <> struct Elem<__half> {
  static __device__ __forceinline__ float to_f(__half x) { return __half2float(x); }
  static __device__ __forceinline__ __half from_f(float x) { return __float2half_rn(x); }
};

// A 16-byte (VE > 1) or single-element (VE == 1) slice of a row.
template <typename T, int VE>
struct alignas(sizeof(T) * VE) Pack {
  T v[VE];
};

template <typename T, int VE>
__device__ __forceinline__ Pack<T, VE> load_pack(const T* p) {
  Pack<T, VE> r;
  if constexpr (sizeof(T) * VE == 16) {
    const uint4 u = __ldg((const uint4*)p);
    *(uint4*)&r = u;
  } else {
    r.v[0] = *p;
  }
  return r;
}
template <typename T, int VE>
__device__ __forceinline__ void store_pack(T* p, const Pack<T, VE>& r) {
  if constexpr (sizeof(T) * VE == 16) {
    *(uint4*)p = *(const uint4*)&r;
  } else {
    *p = r.v[0];
  }
}

// ---- edge ranges ---------------------------------------------------------------
// Is col grouped by output row (non-decreasing, inside the output)? Checked on its
// own first: the range kernel below fills the gap between consecutive destinations
// and must not run on unsorted input, where those gaps are arbitrary.
__global__ void __launch_bounds__(256)
k_check_grouped(const int64_t* __restrict__ col, int64_t E, SegTable st, int64_t num_out_rows, SpmmWs ws) {
  __shared__ int64_t coo[kMaxSegments + 1], ooff[kMaxSegments + 1];
  for (int t = threadIdx.x; t <= st.nseg; t += blockDim.x) {
    coo[t] = st.coo_off[t];
    ooff[t] = st.out_off[t];
  }
  __syncthreads();
  int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  bool bad = false;
  for (; e < E; e += stride) {
    const int64_t d = ooff[st.nseg > 1 ? seg_of(coo, st.nseg, e) : 0] + col[e];
    const int64_t prev = e > 0 ? ooff[st.nseg > 1 ? seg_of(coo, st.nseg, e - 1) : 0] + col[e - 1] : (int64_t)-1;
    bad |= d < prev || d < 0 || d >= num_out_rows;
  }
  if (bad) atomicOr(ws.flags, 1);
}

__global__ void __launch_bounds__(256)
k_edge_ranges(const int64_t* __restrict__ col, int64_t E, SegTable st,
              int64_t num_out_rows, SpmmWs ws) {
  if (*ws.flags != 0) return;
  __shared__ int64_t coo[kMaxSegments + 1], ooff[kMaxSegments + 1];
  for (int t = threadIdx.x; t <= st.nseg; t += blockDim.x) {
    coo[t] = st.coo_off[t];
    ooff[t] = st.out_off[t];
  }
  __syncthreads();
  int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  bool bad = false;
  for (; e < E; e += stride) {
    const int64_t d = ooff[seg_of(coo, st.nseg, e)] + col[e];
    const int64_t prev = e > 0 ? ooff[seg_of(coo, st.nseg, e - 1)] + col[e - 1] : (int64_t)-1;
    if (d < prev || d < 0 || d >= num_out_rows) {
      bad = true;
      continue;
    }
    for (int64_t t = prev + 1; t <= d; ++t) ws.range[t] = e;
    if (e == E - 1)
      for (int64_t t = d + 1; t <= num_out_rows; ++t) ws.range[t] = E;
  }
  if (bad) atomicOr(ws.flags, 1);
}

// Single-block variant: col already holds output rows.
__global__ void __launch_bounds__(256)
k_edge_ranges_single(const int64_t* __restrict__ col, int64_t E, int64_t num_out_rows, SpmmWs ws) {
  int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  bool bad = false;
  for (; e < E; e += stride) {
    const int64_t d = col[e];
    const int64_t prev = e > 0 ? col[e - 1] : (int64_t)-1;
    if (d < prev || d < 0 || d >= num_out_rows) {
      bad = true;
      continue;
    }
    for (int64_t t = prev + 1; t <= d; ++t) ws.range[t] = e;
    if (e == E - 1)
      for (int64_t t = d + 1; t <= num_out_rows; ++t) ws.range[t] = E;
  }
  if (bad) atomicOr(ws.flags, 1);
}

// ---- grouping of unsorted edges by destination (counting sort) ---------------------
__global__ void __launch_bounds__(256)
k_dst_hist(const int64_t* __restrict__ col, int64_t E, SegTable st, int64_t num_out_rows, SpmmWs ws) {
  if (*ws.flags == 0) return;
  __shared__ int64_t coo[kMaxSegments + 1], ooff[kMaxSegments + 1];
  for (int t = threadIdx.x; t <= st.nseg; t += blockDim.x) {
    coo[t] = st.coo_off[t];
    ooff[t] = st.out_off[t];
  }
  __syncthreads();
  int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (; e < E; e += stride) {
    const int64_t d = ooff[st.nseg > 1 ? seg_of(coo, st.nseg, e) : 0] + col[e];
    if (d >= 0 && d < num_out_rows) atomicAdd(ws.cursor + d, 1);
  }
}

__global__ void __launch_bounds__(kDstTile)
k_dst_tile_sums(int64_t num_out_rows, SpmmWs ws) {
  if (*ws.flags == 0) return;
  __shared__ int scratch[33];
  const int64_t d = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  int total;
  block_exclusive_scan(d < num_out_rows ? ws.cursor[d] : 0, scratch, &total);
  if (threadIdx.x == 0) ws.tile_sum[blockIdx.x] = total;
}

__global__ void __launch_bounds__(kDstTile)
k_dst_offsets(int64_t num_out_rows, SpmmWs ws) {
  if (*ws.flags == 0) return;
  __shared__ int scratch[33];
  const int before = block_sum_of(ws.tile_sum, blockIdx.x, scratch);
  const int64_t d = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int v = d < num_out_rows ? ws.cursor[d] : 0;
  int total;
  const int ex = block_exclusive_scan(v, scratch, &total);
  if (d < num_out_rows) {
    ws.range[d] = before + ex;
    ws.cursor[d] = before + ex;
    if (d == num_out_rows - 1) ws.range[num_out_rows] = before + ex + v;
  }
}

__global__ void __launch_bounds__(256)
k_dst_fill(const int64_t* __restrict__ col, int64_t E, SegTable st, int64_t num_out_rows, SpmmWs ws) {
  if (*ws.flags == 0) return;
  __shared__ int64_t coo[kMaxSegments + 1], ooff[kMaxSegments + 1];
  for (int t = threadIdx.x; t <= st.nseg; t += blockDim.x) {
    coo[t] = st.coo_off[t];
    ooff[t] = st.out_off[t];
  }
  __syncthreads();
  int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (; e < E; e += stride) {
    const int64_t d = ooff[st.nseg > 1 ? seg_of(coo, st.nseg, e) : 0] + col[e];
    if (d >= 0 && d < num_out_rows) ws.order[atomicAdd(ws.cursor + d, 1)] = (int32_t)e;
  }
}

enum { kCopyU = 0, kCopyE = 1, kUMulE = 2, kUAddE = 3 };

template <typename T, int VE, int OP>
__device__ __forceinline__ void edge_value(float* acc, const T* __restrict__ in,
                                           const T* __restrict__ edata, int64_t src_off /* row * feat_dim */,
                                           int64_t e, int64_t feat_dim, int64_t edata_dim,
                                           int64_t per, int64_t col0, int64_t ecol = -1) {
  float x[VE];
  if constexpr (OP != kCopyE) {
    const Pack<T, VE> p = load_pack<T, VE>(in + src_off + col0);
#pragma unroll
    for (int t = 0; t < VE; ++t) x[t] = Elem<T>::to_f(p.v[t]);
  }
  if constexpr (OP == kCopyE) {
    const Pack<T, VE> p = load_pack<T, VE>(edata + e * feat_dim + col0);
#pragma unroll
    for (int t = 0; t < VE; ++t) x[t] = Elem<T>::to_f(p.v[t]);
  } else if constexpr (OP == kUMulE || OP == kUAddE) {
    if (per == 1) {
      const Pack<T, VE> p = load_pack<T, VE>(edata + e * feat_dim + col0);
#pragma unroll
      for (int t = 0; t < VE; ++t) {
        const float w = Elem<T>::to_f(p.v[t]);
        x[t] = OP == kUMulE ? x[t] * w : x[t] + w;
      }
    } else if (ecol >= 0) {
      // one value per head and the whole slice inside one head: a single load, column found by the caller
      const float w = Elem<T>::to_f(edata[e * edata_dim + ecol]);
#pragma unroll
      for (int t = 0; t < VE; ++t) x[t] = OP == kUMulE ? x[t] * w : x[t] + w;
    } else {
#pragma unroll
      for (int t = 0; t < VE; ++t) {
        const float w = Elem<T>::to_f(edata[e * edata_dim + (col0 + t) / per]);
        x[t] = OP == kUMulE ? x[t] * w : x[t] + w;
      }
    }
  }
#pragma unroll
  for (int t = 0; t < VE; ++t) acc[t] += x[t];
}

template <typename T, int VE, int OP>
__global__ void __launch_bounds__(256)
k_spmm_rows(const int64_t* __restrict__ row, int64_t E, const T* __restrict__ in,
            const T* __restrict__ edata, int64_t edata_dim, int64_t feat_dim,
            SegTable st, int64_t num_out_rows, SpmmWs ws, T* __restrict__ out,
            int group /* lanes per output row, power of two <= 32 */) {
  __shared__ int64_t coo[kMaxSegments + 1], ioff[kMaxSegments + 1];
  for (int t = threadIdx.x; t <= st.nseg; t += blockDim.x) {
    coo[t] = st.coo_off[t];
    ioff[t] = OP == kCopyE ? 0 : st.in_off[t];
  }
  __syncthreads();
  const bool unsorted = *ws.flags != 0;
  const int lane = threadIdx.x & 31;
  const int sub = lane % group;
  // lanes of this group inside the warp: the shuffles below name only them, so groups
  // whose rows differ in length do not wait for each other
  const unsigned gmask = group == 32 ? 0xffffffffu : (((1u << group) - 1u) << (lane - sub));
  const int64_t rows_per_block = blockDim.x / group;
  const int64_t nvec = feat_dim / VE;
  const int64_t per = feat_dim / edata_dim;
  int64_t d = (int64_t)blockIdx.x * rows_per_block + threadIdx.x / group;
  const int64_t stride = (int64_t)gridDim.x * rows_per_block;
  for (; d < num_out_rows; d += stride) {
    const int64_t e0 = ws.range[d];
    const int64_t e1 = ws.range[d + 1];
    if (e1 - e0 > kLongRow) {
      // one lane group would walk this row for too long: queue it for k_spmm_long
      if (sub == 0) ws.long_rows[atomicAdd(ws.flags + 2, 1)] = d;
      continue;
    }
    for (int64_t c0 = 0; c0 < nvec; c0 += group) {
      const int64_t c = c0 + sub;
      const int64_t ecol = (per > 1 && per % VE == 0) ? (c * VE) / per : -1;
      float acc[VE];
#pragma unroll
      for (int t = 0; t < VE; ++t) acc[t] = 0.f;
      // The group resolves `group` edges at a time, one per lane (edge id through the
      // order array when the edges are not grouped, then its source row): two dependent
      // loads for the whole batch instead of two per edge. The values are then handed
      // round by shuffles, and the row loads of one batch do not depend on each other.
      for (int64_t k0 = e0; k0 < e1; k0 += group) {
        int my_e = 0;
        int64_t my_src = 0;
        if (k0 + sub < e1) {
          my_e = unsorted ? ws.order[k0 + sub] : (int)(k0 + sub);
          // element offset of the source row, so that the walk below only adds
          my_src = OP == kCopyE ? 0 : (ioff[st.nseg > 1 ? seg_of(coo, st.nseg, my_e) : 0] + row[my_e]) * feat_dim;
        }
        const int cnt = (int)min((int64_t)group, e1 - k0);
#pragma unroll 4
        for (int j = 0; j < cnt; ++j) {
          const int e = OP == kCopyU ? 0 : __shfl_sync(gmask, my_e, j, group);   // copy_u never looks at the edge id
          const int64_t src = __shfl_sync(gmask, my_src, j, group);
          if (c < nvec) edge_value<T, VE, OP>(acc, in, edata, src, e, feat_dim, edata_dim, per, c * VE, ecol);
        }
      }
      if (c < nvec) {
        Pack<T, VE> o;
#pragma unroll
        for (int t = 0; t < VE; ++t) o.v[t] = Elem<T>::from_f(acc[t]);
        store_pack<T, VE>(out + d * feat_dim + c * VE, o);
      }
    }
  }
}

// ---- SDDMM -------------------------------------------------------------------------
template <typename T, int VE, int OP>
__global__ void __launch_bounds__(256)
k_sddmm(const int64_t* __restrict__ row, const int64_t* __restrict__ col, int64_t E,
        const T* __restrict__ lhs, const T* __restrict__ rhs, int64_t feat_dim,
        SegTable st, const int64_t* __restrict__ rhs_off, T* __restrict__ out) {
  __shared__ int64_t coo[kMaxSegments + 1], loff[kMaxSegments + 1], roff[kMaxSegments + 1];
  for (int t = threadIdx.x; t <= st.nseg; t += blockDim.x) {
    coo[t] = st.coo_off[t];
    loff[t] = st.in_off[t];
    roff[t] = rhs_off[t];
  }
  __syncthreads();
  const int64_t nvec = feat_dim / VE;
  const int64_t total = E * nvec;
  int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (; idx < total; idx += stride) {
    const int64_t e = idx / nvec, c = idx - e * nvec;
    const int k = st.nseg > 1 ? seg_of(coo, st.nseg, e) : 0;
    const Pack<T, VE> a = load_pack<T, VE>(lhs + (loff[k] + row[e]) * feat_dim + c * VE);
    const Pack<T, VE> b = load_pack<T, VE>(rhs + (roff[k] + col[e]) * feat_dim + c * VE);
    Pack<T, VE> o;
#pragma unroll
    for (int t = 0; t < VE; ++t) {
      const float x = Elem<T>::to_f(a.v[t]), y = Elem<T>::to_f(b.v[t]);
      o.v[t] = Elem<T>::from_f(OP == 0 ? x + y : x * y);
    }
    store_pack<T, VE>(out + e * feat_dim + c * VE, o);
  }
}

// ---- fused GAT edge pipeline ---------------------------------------------------------
// For every destination row d with its edges e (src_e -> d) and every head h:
//   s_e = leaky_relu(el[src_e, h] + er[d, h]);  a_e = softmax over the edges of d;
//   out[d, h, :] = sum_e a_e * ft[src_e, h, :]
// which is u_add_v -> leaky_relu -> edge_softmax -> u_mul_e + sum in one pass
// over a grouped block (python/npc/model/gatconv.py:113-124). One lane group per
// destination row as in k_spmm_rows; scores are recomputed per lane (a block has
// at most a few dozen edges per row), sums stay in fp32 registers.
template <typename T, int VE>
__global__ void __launch_bounds__(256)
k_gat_rows(const int64_t* __restrict__ row, const T* __restrict__ ft, const T* __restrict__ el,
           const T* __restrict__ er, int num_heads, int64_t head_dim, float slope,
           int64_t num_dst, SpmmWs ws, T* __restrict__ out, T* __restrict__ attn,
           int group, int32_t* status) {
  const bool unsorted = *ws.flags != 0;
  if (unsorted && blockIdx.x == 0 && threadIdx.x == 0) atomicOr(status, APT_FLAG_NOT_GROUPED);
  const int sub = threadIdx.x % group;
  const int64_t rows_per_block = blockDim.x / group;
  const int64_t feat_dim = (int64_t)num_heads * head_dim;
  const int64_t nvec = feat_dim / VE;
  int64_t d = (int64_t)blockIdx.x * rows_per_block + threadIdx.x / group;
  const int64_t stride = (int64_t)gridDim.x * rows_per_block;
  for (; d < num_dst; d += stride) {
    const int64_t e0 = unsorted ? 0 : ws.range[d];
    const int64_t e1 = unsorted ? 0 : ws.range[d + 1];
    for (int64_t c = sub; c < nvec; c += group) {
      const int h = (int)((c * VE) / head_dim);
      const float r = Elem<T>::to_f(er[d * num_heads + h]);
      float m = -INFINITY;
      for (int64_t e = e0; e < e1; ++e) {
        float s = Elem<T>::to_f(el[row[e] * num_heads + h]) + r;
        s = s > 0.f ? s : s * slope;
        m = fmaxf(m, s);
      }
      float denom = 0.f;
      for (int64_t e = e0; e < e1; ++e) {
        float s = Elem<T>::to_f(el[row[e] * num_heads + h]) + r;
        s = s > 0.f ? s : s * slope;
        denom += expf(s - m);
      }
      const float inv = denom > 0.f ? 1.f / denom : 0.f;
      float acc[VE];
#pragma unroll
      for (int t = 0; t < VE; ++t) acc[t] = 0.f;
      const bool writes_attn = attn != nullptr && (c * VE) % head_dim == 0;
      for (int64_t e = e0; e < e1; ++e) {
        const int64_t src = row[e];
        float s = Elem<T>::to_f(el[src * num_heads + h]) + r;
        s = s > 0.f ? s : s * slope;
        const float a = expf(s - m) * inv;
        if (writes_attn) attn[e * num_heads + h] = Elem<T>::from_f(a);
        const Pack<T, VE> p = load_pack<T, VE>(ft + src * feat_dim + c * VE);
#pragma unroll
        for (int t = 0; t < VE; ++t) acc[t] += a * Elem<T>::to_f(p.v[t]);
      }
      Pack<T, VE> o;
#pragma unroll
      for (int t = 0; t < VE; ++t) o.v[t] = Elem<T>::from_f(acc[t]);
      store_pack<T, VE>(out + d * feat_dim + c * VE, o);
    }
  }
}

// Fast path of the same operator for wide rows (one warp per destination row), up to
// kGatHeads heads and up to 32 edges per row (fixed-fanout blocks): lane j computes the scores
// of edge j for all heads once (one exp per edge and head instead of two per edge and lane),
// the softmax statistics are warp reductions, the attention values and source ids wait in
// shared memory, and the weighted sum then walks the edges with one shared-memory read each.
// Rows with more than 32 edges take the recomputing walk of k_gat_rows.
constexpr int kGatHeads = 8;

template <typename T, int VE>
__global__ void __launch_bounds__(256)
k_gat_rows_warp(const int64_t* __restrict__ row, const T* __restrict__ ft, const T* __restrict__ el,
                const T* __restrict__ er, int num_heads, int64_t head_dim, float slope,
                int64_t num_dst, SpmmWs ws, T* __restrict__ out, T* __restrict__ attn, int32_t* status) {
  __shared__ float a_sh[8][32][kGatHeads];
  __shared__ int64_t src_sh[8][32];
  const bool unsorted = *ws.flags != 0;
  if (unsorted && blockIdx.x == 0 && threadIdx.x == 0) atomicOr(status, APT_FLAG_NOT_GROUPED);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t feat_dim = (int64_t)num_heads * head_dim;
  const int64_t nvec = feat_dim / VE;
  int64_t d = (int64_t)blockIdx.x * 8 + warp;
  const int64_t stride = (int64_t)gridDim.x * 8;
  for (; d < num_dst; d += stride) {
    const int64_t e0 = unsorted ? 0 : ws.range[d];
    const int64_t e1 = unsorted ? 0 : ws.range[d + 1];
    const int deg = (int)(e1 - e0);
    if (deg <= 32) {
      const bool has = lane < deg;
      const int64_t src = has ? row[e0 + lane] : 0;
      src_sh[warp][lane] = src;
#pragma unroll
      for (int h = 0; h < kGatHeads; ++h) {
        if (h < num_heads) {
          float sc = -INFINITY;
          if (has) {
            sc = Elem<T>::to_f(el[src * num_heads + h]) + Elem<T>::to_f(er[d * num_heads + h]);
            sc = sc > 0.f ? sc : sc * slope;
          }
          float m = sc;
#pragma unroll
          for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
          const float p = has ? expf(sc - m) : 0.f;
          float sum = p;
#pragma unroll
          for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
          const float a = sum > 0.f ? p / sum : 0.f;
          a_sh[warp][lane][h] = a;
          if (has && attn) attn[(e0 + lane) * num_heads + h] = Elem<T>::from_f(a);
        }
      }
      __syncwarp();
      for (int64_t c = lane; c < nvec; c += 32) {
        const int h = (int)((c * VE) / head_dim);
        float acc[VE];
#pragma unroll
        for (int t = 0; t < VE; ++t) acc[t] = 0.f;
#pragma unroll 4
        for (int j = 0; j < deg; ++j) {
          const float a = a_sh[warp][j][h];
          const Pack<T, VE> p = load_pack<T, VE>(ft + src_sh[warp][j] * feat_dim + c * VE);
#pragma unroll
          for (int t = 0; t < VE; ++t) acc[t] += a * Elem<T>::to_f(p.v[t]);
        }
        Pack<T, VE> o;
#pragma unroll
        for (int t = 0; t < VE; ++t) o.v[t] = Elem<T>::from_f(acc[t]);
        store_pack<T, VE>(out + d * feat_dim + c * VE, o);
      }
      __syncwarp();
      continue;
    }
    for (int64_t c = lane; c < nvec; c += 32) {
      const int h = (int)((c * VE) / head_dim);
      const float r = Elem<T>::to_f(er[d * num_heads + h]);
      float m = -INFINITY;
      for (int64_t e = e0; e < e1; ++e) {
        float sc = Elem<T>::to_f(el[row[e] * num_heads + h]) + r;
        sc = sc > 0.f ? sc : sc * slope;
        m = fmaxf(m, sc);
      }
      float denom = 0.f;
      for (int64_t e = e0; e < e1; ++e) {
        float sc = Elem<T>::to_f(el[row[e] * num_heads + h]) + r;
        sc = sc > 0.f ? sc : sc * slope;
        denom += expf(sc - m);
      }
      const float inv = denom > 0.f ? 1.f / denom : 0.f;
      float acc[VE];
#pragma unroll
      for (int t = 0; t < VE; ++t) acc[t] = 0.f;
      const bool writes_attn = attn != nullptr && (c * VE) % head_dim == 0;
      for (int64_t e = e0; e < e1; ++e) {
        const int64_t src = row[e];
        float sc = Elem<T>::to_f(el[src * num_heads + h]) + r;
        sc = sc > 0.f ? sc : sc * slope;
        const float a = expf(sc - m) * inv;
        if (writes_attn) attn[e * num_heads + h] = Elem<T>::from_f(a);
        const Pack<T, VE> p = load_pack<T, VE>(ft + src * feat_dim + c * VE);
#pragma unroll
        for (int t = 0; t < VE; ++t) acc[t] += a * Elem<T>::to_f(p.v[t]);
      }
      Pack<T, VE> o;
#pragma unroll
      for (int t = 0; t < VE; ++t) o.v[t] = Elem<T>::from_f(acc[t]);
      store_pack<T, VE>(out + d * feat_dim + c * VE, o);
    }
  }
}

template <typename T>
static int launch_gat(bool vec, const int64_t* row, const void* ft, const void* el, const void* er,
                      int num_heads, int64_t head_dim, float slope, int64_t num_dst, SpmmWs ws, void* out,
                      void* attn, int32_t* status, cudaStream_t s) {
  constexpr int VE = 16 / sizeof(T);
  const int64_t feat_dim = (int64_t)num_heads * head_dim;
  ProfScope prof("gat_rows", s);
  if (vec && feat_dim / VE > 16 && num_heads <= kGatHeads) {
    const int grid = wave_grid(ceil_div(num_dst, 8), 8);
    APT_LAUNCH((k_gat_rows_warp<T, VE>), grid, 256, 0, s, row, (const T*)ft, (const T*)el, (const T*)er, num_heads,
               head_dim, slope, num_dst, ws, (T*)out, (T*)attn, status);
  } else if (vec) {
    const int group = pow2_at_least_fwd(feat_dim / VE);
    const int grid = wave_grid(ceil_div(num_dst, 256 / group), 8);
    APT_LAUNCH((k_gat_rows<T, VE>), grid, 256, 0, s, row, (const T*)ft, (const T*)el, (const T*)er, num_heads,
               head_dim, slope, num_dst, ws, (T*)out, (T*)attn, group, status);
  } else {
    const int group = pow2_at_least_fwd(feat_dim);
    const int grid = wave_grid(ceil_div(num_dst, 256 / group), 8);
    APT_LAUNCH((k_gat_rows<T, 1>), grid, 256, 0, s, row, (const T*)ft, (const T*)el, (const T*)er, num_heads,
               head_dim, slope, num_dst, ws, (T*)out, (T*)attn, group, status);
  }
  return APT_OK;
}

// ---- backward of the fused GAT edge pipeline: the edge part ---------------------------
// Per destination row d and head h (s_e, a_e as in k_gat_rows, g = grad_out[d, h, :]):
//   dot_e = <g, ft[src_e, h, :]>;  t = sum_e a_e dot_e;
//   grad_s_e = a_e (dot_e - t) * (s_e > 0 ? 1 : slope);  grad_er[d, h] = sum_e grad_s_e
// attn[e, h] = a_e and grad_score[e, h] = grad_s_e go out per edge; the sums over the
// source side (grad_ft = sum a_e g, grad_el = sum grad_s_e) are SpMM calls in the
// reverse direction. The lanes of one head (lanes_per_head of them, a power of two
// inside the lane group) each hold a slice of g and of the ft row and meet in a
// butterfly of shuffles for the dot product.
template <typename T, int VE>
__global__ void __launch_bounds__(256)
k_gat_bwd_rows(const int64_t* __restrict__ row, const T* __restrict__ ft, const T* __restrict__ el,
               const T* __restrict__ er, const T* __restrict__ grad_out, int num_heads, int64_t head_dim,
               float slope, int64_t num_dst, SpmmWs ws, T* __restrict__ attn, T* __restrict__ grad_score,
               T* __restrict__ grad_er, int group, int lanes_per_head, int32_t* status,
               int64_t skip_up_to /* rows with at most this many edges belong to k_gat_bwd_warp */) {
  const bool unsorted = *ws.flags != 0;
  if (unsorted && blockIdx.x == 0 && threadIdx.x == 0) atomicOr(status, APT_FLAG_NOT_GROUPED);
  const int lane = threadIdx.x & 31;
  const int sub = lane % group;
  const unsigned gmask = group == 32 ? 0xffffffffu : (((1u << group) - 1u) << (lane - sub));
  const int64_t rows_per_block = blockDim.x / group;
  const int64_t feat_dim = (int64_t)num_heads * head_dim;
  const int64_t nvec = feat_dim / VE;
  int64_t d = (int64_t)blockIdx.x * rows_per_block + threadIdx.x / group;
  const int64_t stride = (int64_t)gridDim.x * rows_per_block;
  for (; d < num_dst; d += stride) {
    const int64_t e0 = unsorted ? 0 : ws.range[d];
    const int64_t e1 = unsorted ? 0 : ws.range[d + 1];
    if (e1 - e0 <= skip_up_to) continue;
    for (int64_t c0 = 0; c0 < nvec; c0 += group) {
      const int64_t c = c0 + sub;
      const bool live = c < nvec;
      const int h = live ? (int)((c * VE) / head_dim) : 0;
      const bool leader = live && (c * VE) % head_dim == 0;
      const float r = Elem<T>::to_f(er[d * num_heads + h]);
      float m = -INFINITY;
      for (int64_t e = e0; e < e1; ++e) {
        float s = Elem<T>::to_f(el[row[e] * num_heads + h]) + r;
        s = s > 0.f ? s : s * slope;
        m = fmaxf(m, s);
      }
      float denom = 0.f;
      for (int64_t e = e0; e < e1; ++e) {
        float s = Elem<T>::to_f(el[row[e] * num_heads + h]) + r;
        s = s > 0.f ? s : s * slope;
        denom += expf(s - m);
      }
      const float inv = denom > 0.f ? 1.f / denom : 0.f;
      float g[VE];
#pragma unroll
      for (int t = 0; t < VE; ++t) g[t] = 0.f;
      if (live) {
        const Pack<T, VE> p = load_pack<T, VE>(grad_out + d * feat_dim + c * VE);
#pragma unroll
        for (int t = 0; t < VE; ++t) g[t] = Elem<T>::to_f(p.v[t]);
      }
      // first walk: t = sum_e a_e dot_e; second walk: the per-edge results
      float tsum = 0.f, ger = 0.f;
      for (int pass = 0; pass < 2; ++pass) {
        for (int64_t e = e0; e < e1; ++e) {
          const int64_t src = row[e];
          const float raw = Elem<T>::to_f(el[src * num_heads + h]) + r;
          const float s = raw > 0.f ? raw : raw * slope;
          const float a = expf(s - m) * inv;
          float dot = 0.f;
          if (live) {
            const Pack<T, VE> p = load_pack<T, VE>(ft + src * feat_dim + c * VE);
#pragma unroll
            for (int t = 0; t < VE; ++t) dot += g[t] * Elem<T>::to_f(p.v[t]);
          }
          for (int o = lanes_per_head >> 1; o > 0; o >>= 1) dot += __shfl_xor_sync(gmask, dot, o, group);
          if (pass == 0) {
            tsum += a * dot;
          } else {
            const float gs = a * (dot - tsum) * (raw > 0.f ? 1.f : slope);
            ger += gs;
            if (leader) {
              attn[e * num_heads + h] = Elem<T>::from_f(a);
              grad_score[e * num_heads + h] = Elem<T>::from_f(gs);
            }
          }
        }
      }
      if (leader) grad_er[d * num_heads + h] = Elem<T>::from_f(ger);
    }
  }
}

// Wide rows with at most 32 edges (fixed-fanout blocks), one warp per destination: lane j
// scores edge j for all heads once, the lanes then walk the edges ONCE over ft (each lane its
// slice of grad_out and of the row, the lanes of a head meeting in a shuffle butterfly) and
// leave <grad_out, ft> per edge and head in shared memory, and lane j finishes edge j.
template <typename T, int VE>
__global__ void __launch_bounds__(256)
k_gat_bwd_warp(const int64_t* __restrict__ row, const T* __restrict__ ft, const T* __restrict__ el,
               const T* __restrict__ er, const T* __restrict__ grad_out, int num_heads, int64_t head_dim,
               float slope, int64_t num_dst, SpmmWs ws, T* __restrict__ attn, T* __restrict__ grad_score,
               T* __restrict__ grad_er, int lanes_per_head, int32_t* status) {
  __shared__ float a_sh[8][32][kGatHeads], fac_sh[8][32][kGatHeads], dot_sh[8][32][kGatHeads];
  __shared__ int64_t src_sh[8][32];
  const bool unsorted = *ws.flags != 0;
  if (unsorted && blockIdx.x == 0 && threadIdx.x == 0) atomicOr(status, APT_FLAG_NOT_GROUPED);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t feat_dim = (int64_t)num_heads * head_dim;
  const int64_t nvec = feat_dim / VE;
  int64_t d = (int64_t)blockIdx.x * 8 + warp;
  const int64_t stride = (int64_t)gridDim.x * 8;
  for (; d < num_dst; d += stride) {
    const int64_t e0 = unsorted ? 0 : ws.range[d];
    const int64_t e1 = unsorted ? 0 : ws.range[d + 1];
    const int deg = (int)(e1 - e0);
    if (deg > 32) continue;            // left to k_gat_bwd_rows
    const bool has = lane < deg;
    const int64_t src = has ? row[e0 + lane] : 0;
    src_sh[warp][lane] = src;
#pragma unroll
    for (int h = 0; h < kGatHeads; ++h) {
      if (h < num_heads) {
        float raw = 0.f, sc = -INFINITY;
        if (has) {
          raw = Elem<T>::to_f(el[src * num_heads + h]) + Elem<T>::to_f(er[d * num_heads + h]);
          sc = raw > 0.f ? raw : raw * slope;
        }
        float m = sc;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
        const float p = has ? expf(sc - m) : 0.f;
        float sum = p;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
        a_sh[warp][lane][h] = sum > 0.f ? p / sum : 0.f;
        fac_sh[warp][lane][h] = raw > 0.f ? 1.f : slope;
      }
    }
    __syncwarp();
    for (int64_t c0 = 0; c0 < nvec; c0 += 32) {
      const int64_t c = c0 + lane;
      const bool live = c < nvec;
      const int h = live ? (int)((c * VE) / head_dim) : 0;
      const bool leader = live && (c * VE) % head_dim == 0;
      float g[VE];
#pragma unroll
      for (int t = 0; t < VE; ++t) g[t] = 0.f;
      if (live) {
        const Pack<T, VE> p = load_pack<T, VE>(grad_out + d * feat_dim + c * VE);
#pragma unroll
        for (int t = 0; t < VE; ++t) g[t] = Elem<T>::to_f(p.v[t]);
      }
      for (int j = 0; j < deg; ++j) {
        float dot = 0.f;
        if (live) {
          const Pack<T, VE> p = load_pack<T, VE>(ft + src_sh[warp][j] * feat_dim + c * VE);
#pragma unroll
          for (int t = 0; t < VE; ++t) dot += g[t] * Elem<T>::to_f(p.v[t]);
        }
        for (int o = lanes_per_head >> 1; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
        if (leader) dot_sh[warp][j][h] = dot;
      }
    }
    __syncwarp();
#pragma unroll
    for (int h = 0; h < kGatHeads; ++h) {
      if (h < num_heads) {
        const float a = has ? a_sh[warp][lane][h] : 0.f;
        const float dot = has ? dot_sh[warp][lane][h] : 0.f;
        float t = a * dot;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
        const float gs = has ? a * (dot - t) * fac_sh[warp][lane][h] : 0.f;
        if (has) {
          attn[(e0 + lane) * num_heads + h] = Elem<T>::from_f(a);
          grad_score[(e0 + lane) * num_heads + h] = Elem<T>::from_f(gs);
        }
        float ger = gs;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) ger += __shfl_xor_sync(0xffffffffu, ger, o);
        if (lane == 0) grad_er[d * num_heads + h] = Elem<T>::from_f(ger);
      }
    }
    __syncwarp();
  }
}

// Any head width: one thread per (destination, head), everything in turn.
template <typename T>
__global__ void __launch_bounds__(256)
k_gat_bwd_generic(const int64_t* __restrict__ row, const T* __restrict__ ft, const T* __restrict__ el,
                  const T* __restrict__ er, const T* __restrict__ grad_out, int num_heads, int64_t head_dim,
                  float slope, int64_t num_dst, SpmmWs ws, T* __restrict__ attn, T* __restrict__ grad_score,
                  T* __restrict__ grad_er, int32_t* status) {
  const bool unsorted = *ws.flags != 0;
  if (unsorted && blockIdx.x == 0 && threadIdx.x == 0) atomicOr(status, APT_FLAG_NOT_GROUPED);
  const int64_t feat_dim = (int64_t)num_heads * head_dim;
  const int64_t total = num_dst * num_heads;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
    const int64_t d = i / num_heads;
    const int h = (int)(i - d * num_heads);
    const int64_t e0 = unsorted ? 0 : ws.range[d];
    const int64_t e1 = unsorted ? 0 : ws.range[d + 1];
    const float r = Elem<T>::to_f(er[d * num_heads + h]);
    float m = -INFINITY;
    for (int64_t e = e0; e < e1; ++e) {
      float s = Elem<T>::to_f(el[row[e] * num_heads + h]) + r;
      s = s > 0.f ? s : s * slope;
      m = fmaxf(m, s);
    }
    float denom = 0.f;
    for (int64_t e = e0; e < e1; ++e) {
      float s = Elem<T>::to_f(el[row[e] * num_heads + h]) + r;
      s = s > 0.f ? s : s * slope;
      denom += expf(s - m);
    }
    const float inv = denom > 0.f ? 1.f / denom : 0.f;
    const T* g = grad_out + d * feat_dim + (int64_t)h * head_dim;
    float tsum = 0.f, ger = 0.f;
    for (int pass = 0; pass < 2; ++pass) {
      for (int64_t e = e0; e < e1; ++e) {
        const int64_t src = row[e];
        const float raw = Elem<T>::to_f(el[src * num_heads + h]) + r;
        const float s = raw > 0.f ? raw : raw * slope;
        const float a = expf(s - m) * inv;
        const T* f = ft + src * feat_dim + (int64_t)h * head_dim;
        float dot = 0.f;
        for (int64_t k = 0; k < head_dim; ++k) dot += Elem<T>::to_f(g[k]) * Elem<T>::to_f(f[k]);
        if (pass == 0) {
          tsum += a * dot;
        } else {
          const float gs = a * (dot - tsum) * (raw > 0.f ? 1.f : slope);
          ger += gs;
          attn[e * num_heads + h] = Elem<T>::from_f(a);
          grad_score[e * num_heads + h] = Elem<T>::from_f(gs);
        }
      }
    }
    grad_er[d * num_heads + h] = Elem<T>::from_f(ger);
  }
}

template <typename T>
static int launch_gat_bwd(bool vec, const int64_t* row, const void* ft, const void* el, const void* er,
                          const void* grad_out, int num_heads, int64_t head_dim, float slope, int64_t num_dst,
                          SpmmWs ws, void* attn, void* grad_score, void* grad_er, int32_t* status, cudaStream_t s) {
  constexpr int VE = 16 / sizeof(T);
  const int64_t feat_dim = (int64_t)num_heads * head_dim;
  ProfScope prof("gat_bwd_rows", s);
  const int64_t lph = head_dim / VE;                   // lanes per head when rows are read as 16-byte vectors
  const bool pow2 = lph >= 1 && lph <= 32 && (lph & (lph - 1)) == 0;
  if (vec && pow2) {
    const int group = pow2_at_least_fwd(feat_dim / VE);
    if (group % lph == 0) {
      int64_t skip = -1;
      if (group == 32 && num_heads <= kGatHeads) {
        // rows of up to 32 edges: one warp per row; the kernel after it takes the longer rows
        const int grid_w = wave_grid(ceil_div(num_dst, 8), 8);
        APT_LAUNCH((k_gat_bwd_warp<T, VE>), grid_w, 256, 0, s, row, (const T*)ft, (const T*)el, (const T*)er,
                   (const T*)grad_out, num_heads, head_dim, slope, num_dst, ws, (T*)attn, (T*)grad_score,
                   (T*)grad_er, (int)lph, status);
        skip = 32;
      }
      const int grid = wave_grid(ceil_div(num_dst, 256 / group), 8);
      APT_LAUNCH((k_gat_bwd_rows<T, VE>), grid, 256, 0, s, row, (const T*)ft, (const T*)el, (const T*)er,
                 (const T*)grad_out, num_heads, head_dim, slope, num_dst, ws, (T*)attn, (T*)grad_score, (T*)grad_er,
                 group, (int)lph, status, skip);
      return APT_OK;
    }
  }
  const int grid = wave_grid(ceil_div(num_dst * num_heads, 256), 8);
  APT_LAUNCH((k_gat_bwd_generic<T>), grid, 256, 0, s, row, (const T*)ft, (const T*)el, (const T*)er,
             (const T*)grad_out, num_heads, head_dim, slope, num_dst, ws, (T*)attn, (T*)grad_score, (T*)grad_er, status);
  return APT_OK;
}

static int pow2_at_least(int64_t x) {
  int g = 1;
  while (g < x && g < 32) g <<= 1;
  return g;
}

constexpr int kLongWarps = 32;

// One block per long row: its kLongWarps warps take the row's edges in turn, each keeps
// its partial sums in fp32 registers, the partials meet in shared memory and the
// row is written once. Columns are covered 32 vectors at a time.
template <typename T, int VE, int OP>
__global__ void __launch_bounds__(kLongWarps * 32)
k_spmm_long(const int64_t* __restrict__ row, const T* __restrict__ in, const T* __restrict__ edata,
            int64_t edata_dim, int64_t feat_dim, SegTable st, SpmmWs ws, T* __restrict__ out) {
  __shared__ int64_t coo[kMaxSegments + 1], ioff[kMaxSegments + 1];
  __shared__ float part[kLongWarps][32][VE];
  for (int t = threadIdx.x; t <= st.nseg; t += blockDim.x) {
    coo[t] = st.coo_off[t];
    ioff[t] = OP == kCopyE ? 0 : st.in_off[t];
  }
  __syncthreads();
  const bool unsorted = ws.flags[0] != 0;
  const int num_long = ws.flags[2];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t nvec = feat_dim / VE;
  const int64_t per = feat_dim / edata_dim;
  for (int i = blockIdx.x; i < num_long; i += gridDim.x) {
    const int64_t d = ws.long_rows[i];
    const int64_t e0 = ws.range[d], e1 = ws.range[d + 1];
    for (int64_t c0 = 0; c0 < nvec; c0 += 32) {
      const int64_t c = c0 + lane;
      const int64_t ecol = (per > 1 && per % VE == 0) ? (c * VE) / per : -1;
      float acc[VE];
#pragma unroll
      for (int t = 0; t < VE; ++t) acc[t] = 0.f;
      // each warp takes every kLongWarps-th batch of 32 edges, resolved one per lane as in k_spmm_rows
      for (int64_t k0 = e0 + warp * 32; k0 < e1; k0 += kLongWarps * 32) {
        int my_e = 0;
        int64_t my_src = 0;
        if (k0 + lane < e1) {
          my_e = unsorted ? ws.order[k0 + lane] : (int)(k0 + lane);
          my_src = OP == kCopyE ? 0 : (ioff[st.nseg > 1 ? seg_of(coo, st.nseg, my_e) : 0] + row[my_e]) * feat_dim;
        }
        const int cnt = (int)min((int64_t)32, e1 - k0);
#pragma unroll 4
        for (int j = 0; j < cnt; ++j) {
          const int e = OP == kCopyU ? 0 : __shfl_sync(0xffffffffu, my_e, j);
          const int64_t src = __shfl_sync(0xffffffffu, my_src, j);
          if (c < nvec) edge_value<T, VE, OP>(acc, in, edata, src, e, feat_dim, edata_dim, per, c * VE, ecol);
        }
      }
#pragma unroll
      for (int t = 0; t < VE; ++t) part[warp][lane][t] = acc[t];
      __syncthreads();
      if (warp == 0 && c < nvec) {
        Pack<T, VE> o;
#pragma unroll
        for (int t = 0; t < VE; ++t) {
          float v = 0.f;
#pragma unroll
          for (int w = 0; w < kLongWarps; ++w) v += part[w][lane][t];
          o.v[t] = Elem<T>::from_f(v);
        }
        store_pack<T, VE>(out + d * feat_dim + c * VE, o);
      }
      __syncthreads();
    }
  }
}

template <typename T, int VE, int OP>
static int launch_spmm(const int64_t* row, const int64_t* col, int64_t E, const T* in,
                       const T* edata, int64_t edata_dim, int64_t feat_dim, SegTable st,
                       int64_t num_out_rows, SpmmWs ws, T* out, cudaStream_t s) {
  const int64_t nvec = feat_dim / VE;
  const int group = pow2_at_least(nvec);
  {
    ProfScope prof("spmm_rows", s);
    const int grid = wave_grid(ceil_div(num_out_rows, 256 / group), 8);
    APT_LAUNCH((k_spmm_rows<T, VE, OP>), grid, 256, 0, s, row, E, in, edata, edata_dim,
               feat_dim, st, num_out_rows, ws, out, group);
  }
  {
    ProfScope prof("spmm_long", s);
    const int grid = (int)std::min<int64_t>(E / kLongRow + 1, (int64_t)kNumSMs * 8);
    APT_LAUNCH((k_spmm_long<T, VE, OP>), grid, kLongWarps * 32, 0, s, row, in, edata, edata_dim, feat_dim, st, ws, out);
  }
  return APT_OK;
}

template <typename T, int VE>
static int dispatch_spmm_op(int op, const int64_t* row, const int64_t* col, int64_t E,
                            const T* in, const T* edata, int64_t edata_dim,
                            int64_t feat_dim, SegTable st, int64_t num_out_rows,
                            SpmmWs ws, T* out, cudaStream_t s) {
  switch (op) {
    case kCopyU: return launch_spmm<T, VE, kCopyU>(row, col, E, in, edata, edata_dim, feat_dim, st, num_out_rows, ws, out, s);
    case kCopyE: return launch_spmm<T, VE, kCopyE>(row, col, E, in, edata, edata_dim, feat_dim, st, num_out_rows, ws, out, s);
    case kUMulE: return launch_spmm<T, VE, kUMulE>(row, col, E, in, edata, edata_dim, feat_dim, st, num_out_rows, ws, out, s);
    default: return launch_spmm<T, VE, kUAddE>(row, col, E, in, edata, edata_dim, feat_dim, st, num_out_rows, ws, out, s);
  }
}

template <typename T>
static int dispatch_spmm(int op, bool vec, const int64_t* row, const int64_t* col, int64_t E,
                         const void* in, const void* edata, int64_t edata_dim,
                         int64_t feat_dim, SegTable st, int64_t num_out_rows, SpmmWs ws,
                         void* out, cudaStream_t s) {
  constexpr int VE = 16 / sizeof(T);
  if (vec)
    return dispatch_spmm_op<T, VE>(op, row, col, E, (const T*)in, (const T*)edata, edata_dim,
                                   feat_dim, st, num_out_rows, ws, (T*)out, s);
  return dispatch_spmm_op<T, 1>(op, row, col, E, (const T*)in, (const T*)edata, edata_dim,
                                feat_dim, st, num_out_rows, ws, (T*)out, s);
}

template <typename T, int VE>
static int launch_sddmm(int op, const int64_t* row, const int64_t* col, int64_t E,
                        const T* lhs, const T* rhs, int64_t feat_dim, SegTable st,
                        const int64_t* rhs_off, T* out, cudaStream_t s) {
  ProfScope prof("sddmm", s);
  const int grid = wave_grid(ceil_div(E * (feat_dim / VE), 256), 8);
  if (op == 0) {
    APT_LAUNCH((k_sddmm<T, VE, 0>), grid, 256, 0, s, row, col, E, lhs, rhs, feat_dim, st, rhs_off, out);
  } else {
    APT_LAUNCH((k_sddmm<T, VE, 1>), grid, 256, 0, s, row, col, E, lhs, rhs, feat_dim, st, rhs_off, out);
  }
  return APT_OK;
}

template <typename T>
static int dispatch_sddmm(int op, bool vec, const int64_t* row, const int64_t* col, int64_t E,
                          const void* lhs, const void* rhs, int64_t feat_dim, SegTable st,
                          const int64_t* rhs_off, void* out, cudaStream_t s) {
  constexpr int VE = 16 / sizeof(T);
  if (vec)
    return launch_sddmm<T, VE>(op, row, col, E, (const T*)lhs, (const T*)rhs, feat_dim, st, rhs_off, (T*)out, s);
  return launch_sddmm<T, 1>(op, row, col, E, (const T*)lhs, (const T*)rhs, feat_dim, st, rhs_off, (T*)out, s);
}

static size_t elem_size(int dtype) { return dtype == APT_F32 ? 4 : 2; }

}  // namespace apt

extern "C" size_t apt_spmm_workspace_bytes(int64_t num_out_rows, int64_t num_edges) {
  if (num_out_rows < 0 || num_edges < 0) return 0;
  return apt::spmm_layout(num_out_rows, num_edges, nullptr, nullptr);
}

extern "C" int apt_spmm_sum(int op, int dtype, const int64_t* coo_row, const int64_t* coo_col,
                            int64_t num_edges, const void* input, const void* edata,
                            int64_t edata_dim, int64_t feat_dim, const int64_t* coo_offset,
                            const int64_t* input_offset, const int64_t* output_offset,
                            int num_segments, int64_t num_out_rows, void* out,
                            void* workspace, size_t workspace_bytes, void* stream) {
  using namespace apt;
  APT_CHECK_ARG(op >= 0 && op <= 3, "apt_spmm_sum: op %d", op);
  APT_CHECK_ARG(dtype >= APT_F32 && dtype <= APT_F16, "apt_spmm_sum: dtype %d", dtype);
  APT_CHECK_ARG(num_edges >= 0 && feat_dim > 0 && num_out_rows >= 0, "apt_spmm_sum: bad sizes");
  APT_CHECK_ARG(num_segments >= 1 && num_segments <= kMaxSegments,
                "apt_spmm_sum: %d segments outside [1,%d]", num_segments, kMaxSegments);
  if (op == kCopyU) edata_dim = feat_dim;
  APT_CHECK_ARG(edata_dim > 0 && feat_dim % edata_dim == 0 && (op != kCopyE || edata_dim == feat_dim),
                "apt_spmm_sum: edata_dim %lld does not divide feat_dim %lld",
                (long long)edata_dim, (long long)feat_dim);
  cudaStream_t s = (cudaStream_t)stream;
  if (num_out_rows == 0) return APT_OK;
  const size_t esz = elem_size(dtype);
  APT_CHECK_ARG(out, "apt_spmm_sum: null output");
  if (num_edges == 0) {
    APT_CUDA(cudaMemsetAsync(out, 0, (size_t)num_out_rows * feat_dim * esz, s));
    return APT_OK;
  }
  APT_CHECK_ARG(coo_row && coo_col && coo_offset && output_offset && workspace &&
                    (op == kCopyE || (input && input_offset)) && (op == kCopyU || edata),
                "apt_spmm_sum: null pointer");
  APT_CHECK_ARG(((uintptr_t)workspace & 255) == 0, "apt_spmm_sum: workspace must be 256-byte aligned");
  APT_CHECK_ARG(num_edges < (int64_t)0x7fffffff, "apt_spmm_sum: too many edges");
  SpmmWs ws;
  const size_t need = spmm_layout(num_out_rows, num_edges, (char*)workspace, &ws);
  if (workspace_bytes < need) {
    set_error("apt_spmm_sum: workspace %zu < %zu bytes", workspace_bytes, need);
    return APT_ERR_CAPACITY;
  }
  SegTable st{coo_offset, input_offset, output_offset, num_segments};
  // edata is read as whole vectors only when it has one value per column.
  uint64_t bits = (uint64_t)(feat_dim * esz) | (uintptr_t)out;
  if (op != kCopyE) bits |= (uintptr_t)input;
  if (op != kCopyU && edata_dim == feat_dim) bits |= (uintptr_t)edata;
  const bool vec = (bits & 15) == 0;
  // flag word and the per-row counters of the counting sort (they follow each other) start at zero
  APT_CUDA(cudaMemsetAsync(ws.flags, 0, 256 + (size_t)num_out_rows * 4, s));
  {
    ProfScope prof("spmm_ranges", s);
    const int grid = wave_grid(ceil_div(num_edges, 256), 8);
    APT_LAUNCH(k_check_grouped, grid, 256, 0, s, coo_col, num_edges, st, num_out_rows, ws);
    APT_LAUNCH(k_edge_ranges, grid, 256, 0, s, coo_col, num_edges, st, num_out_rows, ws);
  }
  {
    // only do work when col was found not grouped by output row
    ProfScope prof("spmm_group", s);
    const int ge = wave_grid(ceil_div(num_edges, 256), 8);
    const int tiles = (int)ceil_div(num_out_rows, kDstTile);
    APT_LAUNCH(k_dst_hist, ge, 256, 0, s, coo_col, num_edges, st, num_out_rows, ws);
    APT_LAUNCH(k_dst_tile_sums, tiles, kDstTile, 0, s, num_out_rows, ws);
    APT_LAUNCH(k_dst_offsets, tiles, kDstTile, 0, s, num_out_rows, ws);
    APT_LAUNCH(k_dst_fill, ge, 256, 0, s, coo_col, num_edges, st, num_out_rows, ws);
  }
  switch (dtype) {
    case APT_F32:
      return dispatch_spmm<float>(op, vec, coo_row, coo_col, num_edges, input, edata, edata_dim,
                                  feat_dim, st, num_out_rows, ws, out, s);
    case APT_BF16:
      return dispatch_spmm<__nv_bfloat16>(op, vec, coo_row, coo_col, num_edges, input, edata,
                                          edata_dim, feat_dim, st, num_out_rows, ws, out, s);
    default:
      return dispatch_spmm<__half>(op, vec, coo_row, coo_col, num_edges, input, edata, edata_dim,
                                   feat_dim, st, num_out_rows, ws, out, s);
  }
}

extern "C" int apt_sddmm(int op, int dtype, const int64_t* coo_row, const int64_t* coo_col,
                         int64_t num_edges, const void* lhs, const void* rhs, int64_t feat_dim,
                         const int64_t* coo_offset, const int64_t* lhs_offset,
                         const int64_t* rhs_offset, int num_segments, void* out, void* stream) {
  using namespace apt;
  APT_CHECK_ARG(op == 0 || op == 1, "apt_sddmm: op %d", op);
  APT_CHECK_ARG(dtype >= APT_F32 && dtype <= APT_F16, "apt_sddmm: dtype %d", dtype);
  APT_CHECK_ARG(num_edges >= 0 && feat_dim > 0, "apt_sddmm: bad sizes");
  APT_CHECK_ARG(num_segments >= 1 && num_segments <= kMaxSegments,
                "apt_sddmm: %d segments outside [1,%d]", num_segments, kMaxSegments);
  if (num_edges == 0) return APT_OK;
  APT_CHECK_ARG(coo_row && coo_col && lhs && rhs && out && coo_offset && lhs_offset && rhs_offset,
                "apt_sddmm: null pointer");
  cudaStream_t s = (cudaStream_t)stream;
  const size_t esz = elem_size(dtype);
  SegTable st{coo_offset, lhs_offset, nullptr, num_segments};
  const uint64_t bits = (uint64_t)(feat_dim * esz) | (uintptr_t)lhs | (uintptr_t)rhs | (uintptr_t)out;
  const bool vec = (bits & 15) == 0;
  switch (dtype) {
    case APT_F32:
      return dispatch_sddmm<float>(op, vec, coo_row, coo_col, num_edges, lhs, rhs, feat_dim, st, rhs_offset, out, s);
    case APT_BF16:
      return dispatch_sddmm<__nv_bfloat16>(op, vec, coo_row, coo_col, num_edges, lhs, rhs, feat_dim, st, rhs_offset, out, s);
    default:
      return dispatch_sddmm<__half>(op, vec, coo_row, coo_col, num_edges, lhs, rhs, feat_dim, st, rhs_offset, out, s);
  }
}

extern "C" int apt_gat_edge_softmax_sum(int dtype, const int64_t* coo_row, const int64_t* coo_col,
                                        int64_t num_edges, const void* ft, const void* el, const void* er,
                                        int num_heads, int64_t head_dim, float negative_slope,
                                        int64_t num_dst, void* out, void* out_attn, void* workspace,
                                        size_t workspace_bytes, int32_t* status_word, void* stream) {
  using namespace apt;
  APT_CHECK_ARG(dtype >= APT_F32 && dtype <= APT_F16, "apt_gat_edge_softmax_sum: dtype %d", dtype);
  APT_CHECK_ARG(num_edges >= 0 && num_heads >= 1 && head_dim >= 1 && num_dst >= 0,
                "apt_gat_edge_softmax_sum: bad sizes");
  if (num_dst == 0) return APT_OK;
  const size_t esz = elem_size(dtype);
  const int64_t feat_dim = (int64_t)num_heads * head_dim;
  cudaStream_t s = (cudaStream_t)stream;
  APT_CHECK_ARG(out && status_word, "apt_gat_edge_softmax_sum: null output");
  if (num_edges == 0) {
    APT_CUDA(cudaMemsetAsync(out, 0, (size_t)num_dst * feat_dim * esz, s));
    return APT_OK;
  }
  APT_CHECK_ARG(coo_row && coo_col && ft && el && er && workspace, "apt_gat_edge_softmax_sum: null pointer");
  APT_CHECK_ARG(((uintptr_t)workspace & 255) == 0, "apt_gat_edge_softmax_sum: workspace must be 256-byte aligned");
  SpmmWs ws;
  const size_t need = spmm_layout(num_dst, 0, (char*)workspace, &ws);
  if (workspace_bytes < need) {
    set_error("apt_gat_edge_softmax_sum: workspace %zu < %zu bytes", workspace_bytes, need);
    return APT_ERR_CAPACITY;
  }
  APT_CUDA(cudaMemsetAsync(ws.flags, 0, 4, s));
  {
    ProfScope prof("spmm_ranges", s);
    const int grid = wave_grid(ceil_div(num_edges, 256), 8);
    APT_LAUNCH(k_edge_ranges_single, grid, 256, 0, s, coo_col, num_edges, num_dst, ws);
  }
  const int ve = 16 / (int)esz;
  const bool vec = (((uint64_t)(feat_dim * esz) | (uintptr_t)ft | (uintptr_t)out) & 15) == 0 && head_dim % ve == 0;
  switch (dtype) {
    case APT_F32:
      return launch_gat<float>(vec, coo_row, ft, el, er, num_heads, head_dim, negative_slope, num_dst, ws, out,
                               out_attn, status_word, s);
    case APT_BF16:
      return launch_gat<__nv_bfloat16>(vec, coo_row, ft, el, er, num_heads, head_dim, negative_slope, num_dst, ws,
                                       out, out_attn, status_word, s);
    default:
      return launch_gat<__half>(vec, coo_row, ft, el, er, num_heads, head_dim, negative_slope, num_dst, ws, out,
                                out_attn, status_word, s);
  }
}

extern "C" int apt_gat_edge_backward(int dtype, const int64_t* coo_row, const int64_t* coo_col, int64_t num_edges,
                                     const void* ft, const void* el, const void* er, const void* grad_out,
                                     int num_heads, int64_t head_dim, float negative_slope, int64_t num_dst,
                                     void* out_attn, void* out_grad_score, void* out_grad_er, void* workspace,
                                     size_t workspace_bytes, int32_t* status_word, void* stream) {
  using namespace apt;
  APT_CHECK_ARG(dtype >= APT_F32 && dtype <= APT_F16, "apt_gat_edge_backward: dtype %d", dtype);
  APT_CHECK_ARG(num_edges >= 0 && num_heads >= 1 && head_dim >= 1 && num_dst >= 0, "apt_gat_edge_backward: bad sizes");
  if (num_dst == 0) return APT_OK;
  const size_t esz = elem_size(dtype);
  const int64_t feat_dim = (int64_t)num_heads * head_dim;
  cudaStream_t s = (cudaStream_t)stream;
  APT_CHECK_ARG(out_grad_er && status_word, "apt_gat_edge_backward: null output");
  if (num_edges == 0) {
    APT_CUDA(cudaMemsetAsync(out_grad_er, 0, (size_t)num_dst * num_heads * esz, s));
    return APT_OK;
  }
  APT_CHECK_ARG(coo_row && coo_col && ft && el && er && grad_out && out_attn && out_grad_score && workspace,
                "apt_gat_edge_backward: null pointer");
  APT_CHECK_ARG(((uintptr_t)workspace & 255) == 0, "apt_gat_edge_backward: workspace must be 256-byte aligned");
  SpmmWs ws;
  const size_t need = spmm_layout(num_dst, 0, (char*)workspace, &ws);
  if (workspace_bytes < need) {
    set_error("apt_gat_edge_backward: workspace %zu < %zu bytes", workspace_bytes, need);
    return APT_ERR_CAPACITY;
  }
  APT_CUDA(cudaMemsetAsync(ws.flags, 0, 4, s));
  // edges that name no valid destination keep zeros
  APT_CUDA(cudaMemsetAsync(out_attn, 0, (size_t)num_edges * num_heads * esz, s));
  APT_CUDA(cudaMemsetAsync(out_grad_score, 0, (size_t)num_edges * num_heads * esz, s));
  {
    ProfScope prof("spmm_ranges", s);
    const int grid = wave_grid(ceil_div(num_edges, 256), 8);
    APT_LAUNCH(k_edge_ranges_single, grid, 256, 0, s, coo_col, num_edges, num_dst, ws);
  }
  const int ve = 16 / (int)esz;
  const bool vec = (((uint64_t)(feat_dim * esz) | (uintptr_t)ft | (uintptr_t)grad_out) & 15) == 0 && head_dim % ve == 0;
  switch (dtype) {
    case APT_F32:
      return launch_gat_bwd<float>(vec, coo_row, ft, el, er, grad_out, num_heads, head_dim, negative_slope, num_dst,
                                   ws, out_attn, out_grad_score, out_grad_er, status_word, s);
    case APT_BF16:
      return launch_gat_bwd<__nv_bfloat16>(vec, coo_row, ft, el, er, grad_out, num_heads, head_dim, negative_slope,
                                           num_dst, ws, out_attn, out_grad_score, out_grad_er, status_word, s);
    default:
      return launch_gat_bwd<__half>(vec, coo_row, ft, el, er, grad_out, num_heads, head_dim, negative_slope,
                                    num_dst, ws, out_attn, out_grad_score, out_grad_er, status_word, s);
  }
}
