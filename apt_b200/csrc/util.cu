// Setup utilities for the synthetic benchmark graphs: R-MAT edge generation,
// a radix sort of packed edge keys and standard-normal feature rows, all
// driven by the same counter-based Philox stream as the CPU oracle.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <cub/device/device_radix_sort.cuh>

#include "common.cuh"

namespace apt {

__global__ void __launch_bounds__(256)
k_rmat(uint32_t k0, uint32_t k1, int64_t first_edge, int64_t num_edges, int scale,
       int64_t num_nodes, float a, float ab, float abc, int64_t* __restrict__ out_src,
       int64_t* __restrict__ out_dst) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (; i < num_edges; i += stride) {
    const uint64_t e = (uint64_t)(first_edge + i);
    int64_t src = 0, dst = 0;
    // Each attempt consumes ceil(scale/4) Philox blocks: one 32-bit word per
    // level picks the quadrant. Attempts repeat (bounded) until both
    // endpoints are < num_nodes.
    for (uint32_t attempt = 0; attempt < 64; ++attempt) {
      src = 0;
      dst = 0;
      for (int lvl = 0; lvl < scale; lvl += 4) {
        const Philox4 p = philox4x32_10((uint32_t)e, (uint32_t)(e >> 32),
                                        (uint32_t)(lvl >> 2), attempt, k0, k1);
        for (int t = 0; t < 4 && lvl + t < scale; ++t) {
          const float u = (float)(p.w[t] >> 8) * (1.0f / 16777216.0f);
          const int sbit = u >= ab ? 1 : 0;
          const int dbit = (u >= a && u < ab) || u >= abc ? 1 : 0;
          src = (src << 1) | sbit;
          dst = (dst << 1) | dbit;
        }
      }
      if (src < num_nodes && dst < num_nodes) break;
      src %= num_nodes;
      dst %= num_nodes;
    }
    out_src[i] = src;
    out_dst[i] = dst;
  }
}

template <typename T>
__device__ __forceinline__ T cast_out(float x);
template <> __device__ __forceinline__ float cast_out<float>(float x) { return x; }
template <> __device__ __forceinline__ __nv_bfloat16 cast_out<__nv_bfloat16>(float x) { return __float2bfloat16_rn(x); }
template <> __device__ __forceinline__ __half cast_out<__half>(float x) { return __float2half_rn(x); }

// Four normals per Philox block (two Box-Muller pairs); element (row, col)
// uses block col>>2 of row's stream, word pair by col&3.
template <typename T>
__global__ void __launch_bounds__(256)
k_normal_rows(uint32_t k0, uint32_t k1, int64_t first_row, const int64_t* __restrict__ row_ids,
              int64_t num_rows, int64_t dim, T* __restrict__ out) {
  const int64_t quads = (dim + 3) / 4;
  const int64_t total = num_rows * quads;
  int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (; idx < total; idx += stride) {
    const int64_t r = idx / quads, q = idx - r * quads;
    const uint64_t row = (uint64_t)(row_ids ? row_ids[r] : first_row + r);
    const Philox4 p = philox4x32_10((uint32_t)row, (uint32_t)(row >> 32), (uint32_t)q, 0x6e6f726du, k0, k1);
    float z[4];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const float u1 = ((float)(p.w[2 * h] >> 8) + 1.0f) * (1.0f / 16777216.0f);  // (0,1]
      const float u2 = (float)(p.w[2 * h + 1] >> 8) * (1.0f / 16777216.0f);       // [0,1)
      const float rad = sqrtf(-2.0f * logf(u1));
      float sn, cs;
      sincospif(2.0f * u2, &sn, &cs);
      z[2 * h] = rad * cs;
      z[2 * h + 1] = rad * sn;
    }
    for (int t = 0; t < 4 && q * 4 + t < dim; ++t) out[r * dim + q * 4 + t] = cast_out<T>(z[t]);
  }
}

// Zipf-distributed ranks in [1, num_ranks]: rank k with probability proportional to the integral of
// x^-s over [k, k+1) (s > 1), drawn by inverting that integral at u in (0,1):
//     k = floor((1 + u ((N+1)^(1-s) - 1))^(1/(1-s))),   u = (53 random bits + 0.5) / 2^53.
// Draw i uses words 0 and 1 of Philox4x32-10 with counter (i, i >> 32, 0, "zipf").
__global__ void __launch_bounds__(256)
k_zipf_ranks(uint32_t k0, uint32_t k1, int64_t first_draw, int64_t num_draws, int64_t num_ranks, double s,
             int64_t* __restrict__ out) {
  const double e = 1.0 - s, span = pow((double)num_ranks + 1.0, e) - 1.0, inv = 1.0 / e;
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (; i < num_draws; i += stride) {
    const uint64_t d = (uint64_t)(first_draw + i);
    const Philox4 p = philox4x32_10((uint32_t)d, (uint32_t)(d >> 32), 0u, 0x7a697066u, k0, k1);
    const uint64_t bits = (((uint64_t)p.w[0] << 32) | p.w[1]) >> 11;
    const double u = ((double)bits + 0.5) * (1.0 / 9007199254740992.0);
    int64_t k = (int64_t)floor(pow(1.0 + u * span, inv));
    out[i] = k < 1 ? 1 : (k > num_ranks ? num_ranks : k);
  }
}

}  // namespace apt

extern "C" int apt_zipf_ranks(uint64_t seed, int64_t first_draw, int64_t num_draws, int64_t num_ranks, double s,
                              int64_t* out, void* stream) {
  using namespace apt;
  APT_CHECK_ARG(num_draws >= 0 && num_ranks >= 1 && s > 1.0, "apt_zipf_ranks: bad argument (s must exceed 1)");
  if (num_draws == 0) return APT_OK;
  APT_CHECK_ARG(out, "apt_zipf_ranks: null pointer");
  const int grid = wave_grid(ceil_div(num_draws, 256), 8);
  APT_LAUNCH(k_zipf_ranks, grid, 256, 0, (cudaStream_t)stream, (uint32_t)seed, (uint32_t)(seed >> 32), first_draw,
             num_draws, num_ranks, s, out);
  return APT_OK;
}

extern "C" int apt_rmat_edges(uint64_t seed, int64_t first_edge, int64_t num_edges, int scale,
                              int64_t num_nodes, float a, float b, float c, int64_t* out_src,
                              int64_t* out_dst, void* stream) {
  using namespace apt;
  APT_CHECK_ARG(num_edges >= 0 && scale >= 1 && scale <= 40 && num_nodes >= 1 &&
                    num_nodes <= ((int64_t)1 << scale),
                "apt_rmat_edges: bad sizes");
  if (num_edges == 0) return APT_OK;
  APT_CHECK_ARG(out_src && out_dst, "apt_rmat_edges: null pointer");
  cudaStream_t s = (cudaStream_t)stream;
  const int grid = wave_grid(ceil_div(num_edges, 256), 8);
  APT_LAUNCH(k_rmat, grid, 256, 0, s, (uint32_t)seed, (uint32_t)(seed >> 32), first_edge,
             num_edges, scale, num_nodes, a, a + b, a + b + c, out_src, out_dst);
  return APT_OK;
}

extern "C" size_t apt_sort_u64_temp_bytes(int64_t n) {
  size_t bytes = 0;
  if (n <= 0) return 256;
  cub::DeviceRadixSort::SortKeys(nullptr, bytes, (const uint64_t*)nullptr, (uint64_t*)nullptr, n, 0, 64);
  return bytes + 256;
}

extern "C" int apt_sort_u64(const uint64_t* keys_in, uint64_t* keys_out, int64_t n, void* temp,
                            size_t temp_bytes, int end_bit, void* stream) {
  using namespace apt;
  APT_CHECK_ARG(n >= 0 && end_bit >= 1 && end_bit <= 64, "apt_sort_u64: bad argument");
  if (n == 0) return APT_OK;
  APT_CHECK_ARG(keys_in && keys_out && temp, "apt_sort_u64: null pointer");
  APT_CUDA(cub::DeviceRadixSort::SortKeys(temp, temp_bytes, keys_in, keys_out, n, 0, end_bit,
                                          (cudaStream_t)stream));
  return APT_OK;
}

extern "C" int apt_normal_rows(uint64_t seed, int64_t first_row, const int64_t* row_ids,
                               int64_t num_rows, int64_t dim, int dtype, void* out, void* stream) {
  using namespace apt;
  APT_CHECK_ARG(num_rows >= 0 && dim >= 1, "apt_normal_rows: bad sizes");
  APT_CHECK_ARG(dtype >= APT_F32 && dtype <= APT_F16, "apt_normal_rows: dtype %d", dtype);
  if (num_rows == 0) return APT_OK;
  APT_CHECK_ARG(out, "apt_normal_rows: null pointer");
  cudaStream_t s = (cudaStream_t)stream;
  const uint32_t k0 = (uint32_t)seed, k1 = (uint32_t)(seed >> 32);
  const int grid = wave_grid(ceil_div(num_rows * ((dim + 3) / 4), 256), 8);
  switch (dtype) {
    case APT_F32: APT_LAUNCH(k_normal_rows<float>, grid, 256, 0, s, k0, k1, first_row, row_ids, num_rows, dim, (float*)out); break;
    case APT_BF16: APT_LAUNCH(k_normal_rows<__nv_bfloat16>, grid, 256, 0, s, k0, k1, first_row, row_ids, num_rows, dim, (__nv_bfloat16*)out); break;
    default: APT_LAUNCH(k_normal_rows<__half>, grid, 256, 0, s, k0, k1, first_row, row_ids, num_rows, dim, (__half*)out); break;
  }
  return APT_OK;
}
