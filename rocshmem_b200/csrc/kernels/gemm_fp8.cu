// Block-scaled e4m3 GEMMs (plain and grouped) on tcgen05 / TMEM. See gemm_fp8_core.cuh.
#include <cuda.h>
#include <cuda_bf16.h>

#include <algorithm>
#include <cstdlib>

#include "gemm_fp8_core.cuh"
#include "gemm_kernels.hpp"
#include "gemm_tmap.hpp"
#include "launch.cuh"

namespace rocshmem {
namespace kernels {

namespace {

struct PlainScheduler8 {
  int m, n, tiles_n, tiles;
  __device__ bool get(int iter, gemm::Tile &t) const {
    const int id = blockIdx.x + iter * gridDim.x;
    if (id >= tiles) return false;
    int mt, nt;
    gemm::raster(id, tiles / tiles_n, tiles_n, gemm::RASTER_GROUP, mt, nt);
    t.a_row = mt * gemm8::BM;
    t.b_row[0] = nt * gemm8::BN;
    t.b_row[1] = nt * gemm8::BN + gemm8::BN / 2;
    t.rows = min(gemm8::BM, m - t.a_row);
    t.cols = min(gemm8::BN, n - nt * gemm8::BN);
    t.c_row = t.a_row;
    t.c_col = nt * gemm8::BN;
    return true;
  }
  __device__ bool ready(const gemm::Tile &) const { return true; }
  __device__ void side_role() const {}
};

struct RowMajorEpilogue8 {
  __nv_bfloat16 *c;
  size_t ldc;
  __device__ __nv_bfloat16 *row_ptr(const gemm::Tile &t, int row) const {
    return c + static_cast<size_t>(t.c_row + row) * ldc + t.c_col;
  }
};

__global__ void __launch_bounds__(gemm8::THREADS, 1)
gemm_fp8_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                const float *a_scale, const float *b_scale, __nv_bfloat16 *c, int m, int n, int k) {
  extern __shared__ unsigned char smem_raw[];
  __shared__ gemm8::Shared sh;
  PlainScheduler8 sched;
  sched.m = m;
  sched.n = n;
  sched.tiles_n = (n + gemm8::BN - 1) / gemm8::BN;
  sched.tiles = ((m + gemm8::BM - 1) / gemm8::BM) * sched.tiles_n;
  RowMajorEpilogue8 epi{c, static_cast<size_t>(n)};
  gemm8::run<false, false>(&map_a, &map_b, a_scale, b_scale, k / gemm8::KB, sched, epi, smem_raw, sh);
}

constexpr int kMaxGroups8 = 256;

// Rows offsets[g] .. offsets[g + 1] of A use expert g's weight block B[g] ([n, k] rows g * n ...).
template <bool SWIGLU>
struct GroupedScheduler8 {
  const int *offsets;
  int groups, n, tiles_n;
  __device__ bool get(int iter, gemm::Tile &t) const {
    int id = blockIdx.x + iter * gridDim.x;
    for (int g = 0; g < groups; ++g) {
      const int lo = offsets[g], rows = offsets[g + 1] - lo;
      const int tiles_g = ((rows + gemm8::BM - 1) / gemm8::BM) * tiles_n;
      if (id < tiles_g) {
        int mt, nt;
        gemm::raster(id, tiles_g / tiles_n, tiles_n, gemm::RASTER_GROUP, mt, nt);
        t.a_row = lo + mt * gemm8::BM;
        t.rows = min(gemm8::BM, rows - mt * gemm8::BM);
        t.c_row = t.a_row;
        if (SWIGLU) {
          const int j0 = nt * (gemm8::BN / 2);
          t.b_row[0] = g * n + j0;
          t.b_row[1] = g * n + n / 2 + j0;
          t.cols = min(gemm8::BN / 2, n / 2 - j0);
          t.c_col = j0;
        } else {
          t.b_row[0] = g * n + nt * gemm8::BN;
          t.b_row[1] = t.b_row[0] + gemm8::BN / 2;
          t.cols = min(gemm8::BN, n - nt * gemm8::BN);
          t.c_col = nt * gemm8::BN;
        }
        return true;
      }
      id -= tiles_g;
    }
    return false;
  }
  __device__ bool ready(const gemm::Tile &) const { return true; }
  __device__ void side_role() const {}
};

template <bool SWIGLU>
__global__ void __launch_bounds__(gemm8::THREADS, 1)
grouped_gemm_fp8_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                        const float *a_scale, const float *b_scale, __nv_bfloat16 *c, const int *offsets,
                        int groups, int n, int k) {
  extern __shared__ unsigned char smem_raw[];
  __shared__ gemm8::Shared sh;
  __shared__ int s_offsets[kMaxGroups8 + 1];
  for (int i = threadIdx.x; i <= groups; i += blockDim.x) s_offsets[i] = offsets[i];
  __syncthreads();
  GroupedScheduler8<SWIGLU> sched;
  sched.offsets = s_offsets;
  sched.groups = groups;
  sched.n = n;
  sched.tiles_n = SWIGLU ? (n / 2 + gemm8::BN / 2 - 1) / (gemm8::BN / 2) : (n + gemm8::BN - 1) / gemm8::BN;
  RowMajorEpilogue8 epi{c, static_cast<size_t>(SWIGLU ? n / 2 : n)};
  gemm8::run<SWIGLU, false>(&map_a, &map_b, a_scale, b_scale, k / gemm8::KB, sched, epi, smem_raw, sh);
}

// Gate/up projection of a MoE layer whose output feeds the next block-scaled GEMM directly: silu(gate) * up is
// quantised to e4m3 with one scale per 128 columns in the epilogue (out_q [rows, n / 2], out_s [rows, n / 256]).
struct QuantEpilogue8 {
  unsigned char *q;
  float *s;
  size_t ldq, lds;
  __device__ __nv_bfloat16 *row_ptr(const gemm::Tile &, int) const { return nullptr; }
  __device__ unsigned char *q_row_ptr(const gemm::Tile &t, int row) const {
    return q + static_cast<size_t>(t.c_row + row) * ldq + t.c_col;
  }
  __device__ float *scale_ptr(const gemm::Tile &t, int row) const {
    return s + static_cast<size_t>(t.c_row + row) * lds + t.c_col / 128;
  }
};

template <bool A_GATHER>
__global__ void __launch_bounds__(A_GATHER ? gemm8::GATHER_THREADS : gemm8::THREADS, 1)
grouped_gemm_fp8_swiglu_quant_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                                     const float *a_scale, const float *b_scale, unsigned char *out_q, float *out_s,
                                     const int *offsets, int groups, int n, int k, gemm::GatherSrc src) {
  extern __shared__ unsigned char smem_raw[];
  __shared__ gemm8::Shared sh;
  __shared__ int s_offsets[kMaxGroups8 + 1];
  for (int i = threadIdx.x; i <= groups; i += blockDim.x) s_offsets[i] = offsets[i];
  __syncthreads();
  GroupedScheduler8<true> sched;
  sched.offsets = s_offsets;
  sched.groups = groups;
  sched.n = n;
  sched.tiles_n = (n / 2 + gemm8::BN / 2 - 1) / (gemm8::BN / 2);
  QuantEpilogue8 epi{out_q, out_s, static_cast<size_t>(n / 2), static_cast<size_t>(n / 256)};
  gemm8::run<true, false, false, true, A_GATHER>(&map_a, &map_b, a_scale, b_scale, k / gemm8::KB, sched, epi, smem_raw,
                                                 sh, &src);
}

// Down projection whose rows are scaled by their gate weight and added where they belong (see
// grouped_gemm_bf16_scatter_add).
struct ScatterAddEpilogue8 {
  __nv_bfloat16 *y;
  size_t ldc;
  const int *row_index;
  const float *weight;
  __device__ __nv_bfloat16 *row_ptr(const gemm::Tile &t, int row) const {
    return y + static_cast<size_t>(row_index[t.c_row + row]) * ldc + t.c_col;
  }
  __device__ float row_scale(const gemm::Tile &t, int row) const { return weight ? weight[t.c_row + row] : 1.0f; }
};

__global__ void __launch_bounds__(gemm8::THREADS, 1)
grouped_gemm_fp8_scatter_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                                const float *a_scale, const float *b_scale, __nv_bfloat16 *y, const int *offsets,
                                const int *row_index, const float *weight, int groups, int n, int k) {
  extern __shared__ unsigned char smem_raw[];
  __shared__ gemm8::Shared sh;
  __shared__ int s_offsets[kMaxGroups8 + 1];
  for (int i = threadIdx.x; i <= groups; i += blockDim.x) s_offsets[i] = offsets[i];
  __syncthreads();
  GroupedScheduler8<false> sched;
  sched.offsets = s_offsets;
  sched.groups = groups;
  sched.n = n;
  sched.tiles_n = (n + gemm8::BN - 1) / gemm8::BN;
  ScatterAddEpilogue8 epi{y, static_cast<size_t>(n), row_index, weight};
  gemm8::run<false, false, true, false>(&map_a, &map_b, a_scale, b_scale, k / gemm8::KB, sched, epi, smem_raw, sh);
}

template <typename K>
int prepare8(K kernel) {
  cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, gemm8::SMEM_BYTES);
  return e == cudaSuccess ? 0 : static_cast<int>(e);
}

}  // namespace

int fp8_error_count() {
  unsigned int v = 0;
  if (cudaMemcpyFromSymbol(&v, gemm::g_gemm_errors, sizeof(v)) != cudaSuccess) return -1;
  return static_cast<int>(v);
}

int gemm_fp8_blockscaled(const void *a_q, const float *a_scale, const void *b_q, const float *b_scale, void *c, int m,
                         int n, int k, void *stream) {
  // K blocks are consumed four at a time; B scale blocks cover 128 rows of B.
  if (m <= 0 || n <= 0 || k <= 0 || (k % 512) != 0 || (n % 128) != 0) return cudaErrorInvalidValue;
  CUtensorMap map_a, map_b;
  if (!encode_tmap_2d(&map_a, a_q, m, k, 1, gemm8::BM) || !encode_tmap_2d(&map_b, b_q, n, k, 1, gemm8::BN / 2)) return -1;
  const int tiles = ((m + gemm8::BM - 1) / gemm8::BM) * ((n + gemm8::BN - 1) / gemm8::BN);
  const int grid = std::min(tiles, device_sm_count());
  if (int rc = prepare8(gemm_fp8_kernel)) return rc;
  gemm_fp8_kernel<<<grid, gemm8::THREADS, gemm8::SMEM_BYTES, static_cast<cudaStream_t>(stream)>>>(
      map_a, map_b, a_scale, b_scale, static_cast<__nv_bfloat16 *>(c), m, n, k);
  return cudaGetLastError();
}

int grouped_gemm_fp8_blockscaled(const void *a_q, const float *a_scale, const void *b_q, const float *b_scale, void *c,
                                 const int *offsets, int groups, int max_rows, int n, int k, int swiglu,
                                 void *stream) {
  if (groups <= 0 || groups > kMaxGroups8 || max_rows <= 0 || n <= 0 || k <= 0 || (k % 512) != 0 || (n % 128) != 0) {
    return cudaErrorInvalidValue;
  }
  if (swiglu && (n % 256) != 0) return cudaErrorInvalidValue;  // gate and up halves are whole scale blocks
  CUtensorMap map_a, map_b;
  if (!encode_tmap_2d(&map_a, a_q, max_rows, k, 1, gemm8::BM) ||
      !encode_tmap_2d(&map_b, b_q, static_cast<uint64_t>(groups) * n, k, 1, gemm8::BN / 2)) {
    return -1;
  }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int grid = device_sm_count();
  auto launch = [&](auto kernel) -> int {
    if (int rc = prepare8(kernel)) return rc;
    kernel<<<grid, gemm8::THREADS, gemm8::SMEM_BYTES, s>>>(map_a, map_b, a_scale, b_scale,
                                                           static_cast<__nv_bfloat16 *>(c), offsets, groups, n, k);
    return cudaGetLastError();
  };
  return swiglu ? launch(grouped_gemm_fp8_kernel<true>) : launch(grouped_gemm_fp8_kernel<false>);
}

int grouped_gemm_fp8_swiglu_quant(const void *a_q, const float *a_scale, const int *row_index, const void *b_q,
                                   const float *b_scale, void *out_q, float *out_s, const int *offsets, int groups,
                                   int max_rows, int n, int k, void *stream) {
  if (groups <= 0 || groups > kMaxGroups8 || max_rows <= 0 || n <= 0 || k <= 0 || (k % 512) != 0 || (n % 256) != 0) {
    return cudaErrorInvalidValue;
  }
  if ((reinterpret_cast<uintptr_t>(out_q) & 15u) != 0 || (n / 2) % 16 != 0) return cudaErrorInvalidValue;
  CUtensorMap map_a, map_b;
  if (!encode_tmap_2d(&map_a, a_q, max_rows, k, 1, gemm8::BM) ||
      !encode_tmap_2d(&map_b, b_q, static_cast<uint64_t>(groups) * n, k, 1, gemm8::BN / 2)) {
    return -1;
  }
  gemm::GatherSrc src{row_index, static_cast<const unsigned char *>(a_q), static_cast<size_t>(k), a_scale, k / 128};
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (row_index != nullptr) {
    if (int rc = prepare8(grouped_gemm_fp8_swiglu_quant_kernel<true>)) return rc;
    grouped_gemm_fp8_swiglu_quant_kernel<true><<<device_sm_count(), gemm8::GATHER_THREADS, gemm8::SMEM_BYTES, s>>>(
        map_a, map_b, a_scale, b_scale, static_cast<unsigned char *>(out_q), out_s, offsets, groups, n, k, src);
  } else {
    if (int rc = prepare8(grouped_gemm_fp8_swiglu_quant_kernel<false>)) return rc;
    grouped_gemm_fp8_swiglu_quant_kernel<false><<<device_sm_count(), gemm8::THREADS, gemm8::SMEM_BYTES, s>>>(
        map_a, map_b, a_scale, b_scale, static_cast<unsigned char *>(out_q), out_s, offsets, groups, n, k, src);
  }
  return cudaGetLastError();
}

int grouped_gemm_fp8_scatter_add(const void *a_q, const float *a_scale, const void *b_q, const float *b_scale, void *y,
                                 const int *offsets, const int *row_index, const float *weights, int groups,
                                 int max_rows, int n, int k, void *stream) {
  if (groups <= 0 || groups > kMaxGroups8 || max_rows <= 0 || n <= 0 || k <= 0 || (k % 512) != 0 || (n % 128) != 0) {
    return cudaErrorInvalidValue;
  }
  if (row_index == nullptr || (reinterpret_cast<uintptr_t>(y) & 15u) != 0) return cudaErrorInvalidValue;
  CUtensorMap map_a, map_b;
  if (!encode_tmap_2d(&map_a, a_q, max_rows, k, 1, gemm8::BM) ||
      !encode_tmap_2d(&map_b, b_q, static_cast<uint64_t>(groups) * n, k, 1, gemm8::BN / 2)) {
    return -1;
  }
  if (int rc = prepare8(grouped_gemm_fp8_scatter_kernel)) return rc;
  grouped_gemm_fp8_scatter_kernel<<<device_sm_count(), gemm8::THREADS, gemm8::SMEM_BYTES,
                                    static_cast<cudaStream_t>(stream)>>>(
      map_a, map_b, a_scale, b_scale, static_cast<__nv_bfloat16 *>(y), offsets, row_index, weights, groups, n, k);
  return cudaGetLastError();
}

}  // namespace kernels
}  // namespace rocshmem
