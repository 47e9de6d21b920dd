// Plain and grouped bf16 GEMM on tcgen05 / TMEM (sm_100a). See gemm_core.cuh for the kernel structure.
#include <cuda.h>
#include <cuda_bf16.h>

#include <algorithm>
#include <cstdlib>

#include "../runtime/cuda_vmm_provider.hpp"
#include "gemm_core.cuh"
#include "gemm2_core.cuh"
#include "gemm_kernels.hpp"
#include "gemm_tmap.hpp"
#include "launch.cuh"

namespace rocshmem {
namespace kernels {

// ---- tensor maps -------------------------------------------------------------------------------------------

bool encode_tmap_2d(CUtensorMap *map, const void *base, uint64_t rows, uint64_t cols_elems, int elem_bytes,
                    uint32_t box_rows) {
  const CudaDriver &drv = CudaDriver::get();
  if (!drv.ok || drv.TensorMapEncodeTiled == nullptr) return false;
  cuuint64_t dims[2] = {cols_elems, rows};
  cuuint64_t strides[1] = {cols_elems * static_cast<uint64_t>(elem_bytes)};
  cuuint32_t box[2] = {static_cast<cuuint32_t>(gemm::SLAB_BYTES / elem_bytes), box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUtensorMapDataType dt = elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_UINT8;
  CUresult r = drv.TensorMapEncodeTiled(map, dt, 2, const_cast<void *>(base), dims, strides, box, estr,
                                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                        CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

namespace {

// ---- plain GEMM ------------------------------------------------------------------------------------------------
struct PlainScheduler {
  int m, n, tiles_n, tiles;
  __device__ bool get(int iter, gemm::Tile &t) const {
    const int id = blockIdx.x + iter * gridDim.x;
    if (id >= tiles) return false;
    int mt, nt;
    gemm::raster(id, tiles / tiles_n, tiles_n, gemm::RASTER_GROUP, mt, nt);
    t.a_row = mt * gemm::BM;
    t.b_row[0] = nt * gemm::BN;
    t.b_row[1] = nt * gemm::BN + gemm::BN / 2;
    t.rows = min(gemm::BM, m - t.a_row);
    t.cols = min(gemm::BN, n - nt * gemm::BN);
    t.c_row = t.a_row;
    t.c_col = nt * gemm::BN;
    return true;
  }
  __device__ bool ready(const gemm::Tile &) const { return true; }
  __device__ void side_role() const {}
};

struct RowMajorEpilogue {
  __nv_bfloat16 *c;
  size_t ldc;
  __device__ __nv_bfloat16 *row_ptr(const gemm::Tile &t, int row) const {
    return c + static_cast<size_t>(t.c_row + row) * ldc + t.c_col;
  }
};

__global__ void __launch_bounds__(gemm::THREADS, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                 __nv_bfloat16 *c, int m, int n, int k) {
  extern __shared__ unsigned char smem_raw[];
  __shared__ gemm::Shared sh;
  PlainScheduler sched;
  sched.m = m;
  sched.n = n;
  sched.tiles_n = (n + gemm::BN - 1) / gemm::BN;
  sched.tiles = ((m + gemm::BM - 1) / gemm::BM) * sched.tiles_n;
  RowMajorEpilogue epi{c, static_cast<size_t>(n)};
  gemm::run<false, false>(&map_a, &map_b, k * 2, sched, epi, smem_raw, sh);
}

// ---- plain GEMM, two CTAs per 256 x 256 tile ------------------------------------------------------------------
struct PairScheduler {
  int m, n, tiles_n, tiles;
  __device__ bool get(int iter, gemm::Tile &t) const {
    const int pairs = gridDim.x / 2;
    const int id = blockIdx.x / 2 + iter * pairs;
    if (id >= tiles) return false;
    int mt, nt;
    gemm::raster(id, tiles / tiles_n, tiles_n, gemm::RASTER_GROUP, mt, nt);
    t.a_row = mt * 2 * gemm2::BM;
    t.b_row[0] = nt * gemm2::BN;
    t.b_row[1] = nt * gemm2::BN + gemm2::BN / 2;
    t.rows = min(2 * gemm2::BM, m - t.a_row);
    t.cols = min(gemm2::BN, n - nt * gemm2::BN);
    t.c_row = t.a_row;
    t.c_col = nt * gemm2::BN;
    return true;
  }
  __device__ bool ready(const gemm::Tile &) const { return true; }
  __device__ void side_role() const {}
};

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(gemm2::THREADS, 1)
gemm_bf16_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                      __nv_bfloat16 *c, int m, int n, int k) {
  extern __shared__ unsigned char smem_raw[];
  __shared__ gemm2::Shared sh;
  PairScheduler sched;
  sched.m = m;
  sched.n = n;
  sched.tiles_n = (n + gemm2::BN - 1) / gemm2::BN;
  sched.tiles = ((m + 2 * gemm2::BM - 1) / (2 * gemm2::BM)) * sched.tiles_n;
  RowMajorEpilogue epi{c, static_cast<size_t>(n)};
  gemm2::run<false>(&map_a, &map_b, k * 2, sched, epi, smem_raw, sh);
}

// ---- grouped GEMM ------------------------------------------------------------------------------------------------
constexpr int kMaxGroups = 256;

template <bool SWIGLU>
struct GroupedScheduler {
  const int *offsets;  // shared-memory copy, groups + 1 entries
  int groups, n, tiles_n;
  __device__ bool get(int iter, gemm::Tile &t) const {
    int id = blockIdx.x + iter * gridDim.x;
    for (int g = 0; g < groups; ++g) {
      const int lo = offsets[g], rows = offsets[g + 1] - lo;
      const int tiles_g = ((rows + gemm::BM - 1) / gemm::BM) * tiles_n;
      if (id < tiles_g) {
        int mt, nt;
        gemm::raster(id, tiles_g / tiles_n, tiles_n, gemm::RASTER_GROUP, mt, nt);
        t.a_row = lo + mt * gemm::BM;
        t.rows = min(gemm::BM, rows - mt * gemm::BM);
        t.c_row = t.a_row;
        if (SWIGLU) {
          // 128 gate columns and the matching 128 up columns share one tile.
          const int j0 = nt * (gemm::BN / 2);
          t.b_row[0] = g * n + j0;
          t.b_row[1] = g * n + n / 2 + j0;
          t.cols = min(gemm::BN / 2, n / 2 - j0);
          t.c_col = j0;
        } else {
          t.b_row[0] = g * n + nt * gemm::BN;
          t.b_row[1] = t.b_row[0] + gemm::BN / 2;
          t.cols = min(gemm::BN, n - nt * gemm::BN);
          t.c_col = nt * gemm::BN;
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
__global__ void __launch_bounds__(gemm::THREADS, 1)
grouped_gemm_bf16_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                         __nv_bfloat16 *c, const int *offsets, int groups, int n, int k) {
  extern __shared__ unsigned char smem_raw[];
  __shared__ gemm::Shared sh;
  __shared__ int s_offsets[kMaxGroups + 1];
  for (int i = threadIdx.x; i <= groups; i += blockDim.x) s_offsets[i] = offsets[i];
  __syncthreads();
  GroupedScheduler<SWIGLU> sched;
  sched.offsets = s_offsets;
  sched.groups = groups;
  sched.n = n;
  sched.tiles_n = SWIGLU ? (n / 2 + gemm::BN / 2 - 1) / (gemm::BN / 2) : (n + gemm::BN - 1) / gemm::BN;
  RowMajorEpilogue epi{c, static_cast<size_t>(SWIGLU ? n / 2 : n)};
  gemm::run<false, SWIGLU>(&map_a, &map_b, k * 2, sched, epi, smem_raw, sh);
}

// Grouped GEMM whose A rows are gathered by index from the bf16 rows an expert-parallel dispatch delivered: position
// p of the grouped order reads source row row_index[p]. Replaces a separate gather pass over the activations.
template <bool SWIGLU>
__global__ void __launch_bounds__(gemm::GATHER_THREADS, 1)
grouped_gemm_bf16_gather_kernel(const __grid_constant__ CUtensorMap map_b, gemm::GatherSrc src, __nv_bfloat16 *c,
                                const int *offsets, int groups, int n, int k) {
  extern __shared__ unsigned char smem_raw[];
  __shared__ gemm::Shared sh;
  __shared__ int s_offsets[kMaxGroups + 1];
  for (int i = threadIdx.x; i <= groups; i += blockDim.x) s_offsets[i] = offsets[i];
  __syncthreads();
  GroupedScheduler<SWIGLU> sched;
  sched.offsets = s_offsets;
  sched.groups = groups;
  sched.n = n;
  sched.tiles_n = SWIGLU ? (n / 2 + gemm::BN / 2 - 1) / (gemm::BN / 2) : (n + gemm::BN - 1) / gemm::BN;
  RowMajorEpilogue epi{c, static_cast<size_t>(SWIGLU ? n / 2 : n)};
  gemm::run<false, SWIGLU, true>(&map_b, &map_b, k * 2, sched, epi, smem_raw, sh, &src);
}

// Rows of the grouped product are multiplied by a per-position weight and added to row row_index[p] of the
// destination: the gate-weighted sum over a token's local experts happens in the epilogue (packed bf16
// reductions in L2) instead of in a separate pass. The destination rows must be zero beforehand.
struct ScatterAddEpilogue {
  __nv_bfloat16 *y;
  size_t ldc;
  const int *row_index;
  const float *weight;
  __device__ __nv_bfloat16 *row_ptr(const gemm::Tile &t, int row) const {
    return y + static_cast<size_t>(row_index[t.c_row + row]) * ldc + t.c_col;
  }
  __device__ float row_scale(const gemm::Tile &t, int row) const { return weight ? weight[t.c_row + row] : 1.0f; }
};

__global__ void __launch_bounds__(gemm::THREADS, 1)
grouped_gemm_bf16_scatter_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                                 __nv_bfloat16 *y, const int *offsets, const int *row_index, const float *weight,
                                 int groups, int n, int k) {
  extern __shared__ unsigned char smem_raw[];
  __shared__ gemm::Shared sh;
  __shared__ int s_offsets[kMaxGroups + 1];
  for (int i = threadIdx.x; i <= groups; i += blockDim.x) s_offsets[i] = offsets[i];
  __syncthreads();
  GroupedScheduler<false> sched;
  sched.offsets = s_offsets;
  sched.groups = groups;
  sched.n = n;
  sched.tiles_n = (n + gemm::BN - 1) / gemm::BN;
  ScatterAddEpilogue epi{y, static_cast<size_t>(n), row_index, weight};
  gemm::run<false, false, false, true>(&map_a, &map_b, k * 2, sched, epi, smem_raw, sh);
}

template <typename K>
int prepare(K kernel) {
  // Kernels of different instantiations share one function-pointer type, so the attribute is set
  // on every call (it is a cheap host-side operation) rather than cached per type.
  cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, gemm::SMEM_BYTES);
  return e == cudaSuccess ? 0 : static_cast<int>(e);
}

}  // namespace

int fused_error_count();  // counter of the fused kernels' translation unit
int fp8_error_count();    // counter of the fp8 kernels' translation unit

int gemm_error_count() {
  unsigned int v = 0;
  if (cudaMemcpyFromSymbol(&v, gemm::g_gemm_errors, sizeof(v)) != cudaSuccess) return -1;
  const int fused = fused_error_count();
  const int fp8 = fp8_error_count();
  return static_cast<int>(v) + (fused > 0 ? fused : 0) + (fp8 > 0 ? fp8 : 0);
}

int gemm_bf16_pair(const void *a, const void *b, void *c, int m, int n, int k, void *stream) {
  if (m <= 0 || n <= 0 || k <= 0 || (k % 8) != 0) return cudaErrorInvalidValue;
  CUtensorMap map_a, map_b;
  if (!encode_tmap_2d(&map_a, a, m, k, 2, gemm2::BM) || !encode_tmap_2d(&map_b, b, n, k, 2, gemm2::BN / 2)) return -1;
  cudaError_t e = cudaFuncSetAttribute(gemm_bf16_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, gemm2::SMEM_BYTES);
  if (e != cudaSuccess) return static_cast<int>(e);
  const int tiles = ((m + 2 * gemm2::BM - 1) / (2 * gemm2::BM)) * ((n + gemm2::BN - 1) / gemm2::BN);
  const int pairs = std::max(1, std::min(tiles, device_sm_count() / 2));
  gemm_bf16_pair_kernel<<<2 * pairs, gemm2::THREADS, gemm2::SMEM_BYTES, static_cast<cudaStream_t>(stream)>>>(
      map_a, map_b, static_cast<__nv_bfloat16 *>(c), m, n, k);
  return cudaGetLastError();
}

int gemm_bf16_one_cta(const void *a, const void *b, void *c, int m, int n, int k, void *stream);

// More than one 128-row block: two CTAs per 256 x 256 tile (about 10 % faster, see gemm2_core.cuh), unless
// ROCSHMEM_GEMM_TWO_CTA=0 asks for the one-CTA kernel.
int gemm_bf16(const void *a, const void *b, void *c, int m, int n, int k, void *stream) {
  static const bool two_cta = [] {
    const char *e = std::getenv("ROCSHMEM_GEMM_TWO_CTA");
    return e == nullptr || e[0] != '0';
  }();
  if (two_cta && m > gemm::BM && device_sm_count() % 2 == 0) return gemm_bf16_pair(a, b, c, m, n, k, stream);
  return gemm_bf16_one_cta(a, b, c, m, n, k, stream);
}

int gemm_bf16_one_cta(const void *a, const void *b, void *c, int m, int n, int k, void *stream) {
  if (m <= 0 || n <= 0 || k <= 0 || (k % 8) != 0) return cudaErrorInvalidValue;
  CUtensorMap map_a, map_b;
  if (!encode_tmap_2d(&map_a, a, m, k, 2, gemm::BM) || !encode_tmap_2d(&map_b, b, n, k, 2, gemm::BN / 2)) return -1;
  if (int rc = prepare(gemm_bf16_kernel)) return rc;
  const int tiles = ((m + gemm::BM - 1) / gemm::BM) * ((n + gemm::BN - 1) / gemm::BN);
  const int grid = std::min(tiles, device_sm_count());
  gemm_bf16_kernel<<<grid, gemm::THREADS, gemm::SMEM_BYTES, static_cast<cudaStream_t>(stream)>>>(
      map_a, map_b, static_cast<__nv_bfloat16 *>(c), m, n, k);
  return cudaGetLastError();
}

int grouped_gemm_bf16(const void *a, const void *b, void *c, const int *offsets, int groups, int max_rows, int n,
                      int k, int swiglu, void *stream) {
  if (groups <= 0 || groups > kMaxGroups || max_rows <= 0 || n <= 0 || k <= 0 || (k % 8) != 0) return cudaErrorInvalidValue;
  if (swiglu && (n % 2) != 0) return cudaErrorInvalidValue;
  CUtensorMap map_a, map_b;
  if (!encode_tmap_2d(&map_a, a, max_rows, k, 2, gemm::BM) ||
      !encode_tmap_2d(&map_b, b, static_cast<uint64_t>(groups) * n, k, 2, gemm::BN / 2)) {
    return -1;
  }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  // The tile count depends on device-side offsets; every SM gets a CTA and idle ones exit at once.
  const int grid = device_sm_count();
  if (swiglu) {
    if (int rc = prepare(grouped_gemm_bf16_kernel<true>)) return rc;
    grouped_gemm_bf16_kernel<true><<<grid, gemm::THREADS, gemm::SMEM_BYTES, s>>>(
        map_a, map_b, static_cast<__nv_bfloat16 *>(c), offsets, groups, n, k);
  } else {
    if (int rc = prepare(grouped_gemm_bf16_kernel<false>)) return rc;
    grouped_gemm_bf16_kernel<false><<<grid, gemm::THREADS, gemm::SMEM_BYTES, s>>>(
        map_a, map_b, static_cast<__nv_bfloat16 *>(c), offsets, groups, n, k);
  }
  return cudaGetLastError();
}

int grouped_gemm_bf16_gathered(const void *a_rows, const int *row_index, const void *b, void *c, const int *offsets,
                               int groups, int n, int k, int swiglu, void *stream) {
  if (groups <= 0 || groups > kMaxGroups || n <= 0 || k <= 0 || (k % 64) != 0) return cudaErrorInvalidValue;
  if (swiglu && (n % 2) != 0) return cudaErrorInvalidValue;
  if (a_rows == nullptr || row_index == nullptr) return cudaErrorInvalidValue;
  CUtensorMap map_b;
  if (!encode_tmap_2d(&map_b, b, static_cast<uint64_t>(groups) * n, k, 2, gemm::BN / 2)) return -1;
  gemm::GatherSrc src{row_index, static_cast<const unsigned char *>(a_rows), static_cast<size_t>(k) * 2, nullptr, 0};
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int grid = device_sm_count();
  auto launch = [&](auto kernel) -> int {
    if (int rc = prepare(kernel)) return rc;
    kernel<<<grid, gemm::GATHER_THREADS, gemm::SMEM_BYTES, s>>>(map_b, src, static_cast<__nv_bfloat16 *>(c), offsets,
                                                                groups, n, k);
    return cudaGetLastError();
  };
  return swiglu ? launch(grouped_gemm_bf16_gather_kernel<true>) : launch(grouped_gemm_bf16_gather_kernel<false>);
}

int grouped_gemm_bf16_scatter_add(const void *a, const void *b, void *y, const int *offsets, const int *row_index,
                                  const float *weights, int groups, int max_rows, int n, int k, void *stream) {
  if (groups <= 0 || groups > kMaxGroups || max_rows <= 0 || n <= 0 || k <= 0 || (k % 8) != 0 || (n % 8) != 0) {
    return cudaErrorInvalidValue;
  }
  if (row_index == nullptr || (reinterpret_cast<uintptr_t>(y) & 15u) != 0) return cudaErrorInvalidValue;
  CUtensorMap map_a, map_b;
  if (!encode_tmap_2d(&map_a, a, max_rows, k, 2, gemm::BM) ||
      !encode_tmap_2d(&map_b, b, static_cast<uint64_t>(groups) * n, k, 2, gemm::BN / 2)) {
    return -1;
  }
  if (int rc = prepare(grouped_gemm_bf16_scatter_kernel)) return rc;
  grouped_gemm_bf16_scatter_kernel<<<device_sm_count(), gemm::THREADS, gemm::SMEM_BYTES,
                                     static_cast<cudaStream_t>(stream)>>>(
      map_a, map_b, static_cast<__nv_bfloat16 *>(y), offsets, row_index, weights, groups, n, k);
  return cudaGetLastError();
}

}  // namespace kernels
}  // namespace rocshmem
