// Python bindings of the tcgen05 GEMM kernels and the fused GEMM + collective kernels.
#include <pybind11/pybind11.h>

#include <stdexcept>
#include <string>

#include "gemm_kernels.hpp"

namespace py = pybind11;

namespace rocshmem {
namespace kernels {

namespace {
template <typename T>
T *P(uintptr_t v) { return reinterpret_cast<T *>(v); }
void check(int rc, const char *what) {
  if (rc == -1) throw std::runtime_error(std::string(what) + ": cannot encode tensor maps (driver entry point missing or bad shape)");
  if (rc != 0) throw std::runtime_error(std::string(what) + ": CUDA error " + std::to_string(rc));
}
}  // namespace

void bind_gemm(py::module_ &m) {
  m.def("gemm_bf16", [](uintptr_t a, uintptr_t b, uintptr_t c, int M, int N, int K, uintptr_t stream) {
    check(gemm_bf16(P<void>(a), P<void>(b), P<void>(c), M, N, K, P<void>(stream)), "gemm_bf16");
  });
  m.def("gemm_bf16_one_cta", [](uintptr_t a, uintptr_t b, uintptr_t c, int M, int N, int K, uintptr_t stream) {
    check(gemm_bf16_one_cta(P<void>(a), P<void>(b), P<void>(c), M, N, K, P<void>(stream)), "gemm_bf16_one_cta");
  });
  m.def("gemm_bf16_pair", [](uintptr_t a, uintptr_t b, uintptr_t c, int M, int N, int K, uintptr_t stream) {
    check(gemm_bf16_pair(P<void>(a), P<void>(b), P<void>(c), M, N, K, P<void>(stream)), "gemm_bf16_pair");
  });
  m.def("grouped_gemm_bf16", [](uintptr_t a, uintptr_t b, uintptr_t c, uintptr_t offsets, int groups, int max_rows,
                                int N, int K, int swiglu, uintptr_t stream) {
    check(grouped_gemm_bf16(P<void>(a), P<void>(b), P<void>(c), P<int>(offsets), groups, max_rows, N, K, swiglu,
                            P<void>(stream)), "grouped_gemm_bf16");
  });
  m.def("grouped_gemm_bf16_gathered", [](uintptr_t a_rows, uintptr_t row_index, uintptr_t b, uintptr_t c,
                                         uintptr_t offsets, int groups, int N, int K, int swiglu, uintptr_t stream) {
    check(grouped_gemm_bf16_gathered(P<void>(a_rows), P<int>(row_index), P<void>(b), P<void>(c), P<int>(offsets), groups,
                                     N, K, swiglu, P<void>(stream)), "grouped_gemm_bf16_gathered");
  });
  m.def("grouped_gemm_bf16_scatter_add", [](uintptr_t a, uintptr_t b, uintptr_t y, uintptr_t offsets,
                                            uintptr_t row_index, uintptr_t weights, int groups, int max_rows, int N,
                                            int K, uintptr_t stream) {
    check(grouped_gemm_bf16_scatter_add(P<void>(a), P<void>(b), P<void>(y), P<int>(offsets), P<int>(row_index),
                                        P<float>(weights), groups, max_rows, N, K, P<void>(stream)),
          "grouped_gemm_bf16_scatter_add");
  });
  m.def("grouped_gemm_fp8_swiglu_quant", [](uintptr_t a, uintptr_t a_s, uintptr_t row_index, uintptr_t b, uintptr_t b_s,
                                            uintptr_t out_q, uintptr_t out_s, uintptr_t offsets, int groups,
                                            int max_rows, int N, int K, uintptr_t stream) {
    check(grouped_gemm_fp8_swiglu_quant(P<void>(a), P<float>(a_s), P<int>(row_index), P<void>(b), P<float>(b_s),
                                        P<void>(out_q), P<float>(out_s), P<int>(offsets), groups, max_rows, N, K,
                                        P<void>(stream)), "grouped_gemm_fp8_swiglu_quant");
  });
  m.def("grouped_gemm_fp8_scatter_add", [](uintptr_t a, uintptr_t a_s, uintptr_t b, uintptr_t b_s, uintptr_t y,
                                           uintptr_t offsets, uintptr_t row_index, uintptr_t weights, int groups,
                                           int max_rows, int N, int K, uintptr_t stream) {
    check(grouped_gemm_fp8_scatter_add(P<void>(a), P<float>(a_s), P<void>(b), P<float>(b_s), P<void>(y),
                                       P<int>(offsets), P<int>(row_index), P<float>(weights), groups, max_rows, N, K,
                                       P<void>(stream)), "grouped_gemm_fp8_scatter_add");
  });
  m.def("gemm_error_count", [] { return gemm_error_count(); });
  m.def("gemm_fp8_blockscaled", [](uintptr_t a, uintptr_t a_s, uintptr_t b, uintptr_t b_s, uintptr_t c, int M, int N,
                                   int K, uintptr_t stream) {
    check(gemm_fp8_blockscaled(P<void>(a), P<float>(a_s), P<void>(b), P<float>(b_s), P<void>(c), M, N, K,
                               P<void>(stream)), "gemm_fp8_blockscaled");
  });
  m.def("grouped_gemm_fp8_blockscaled", [](uintptr_t a, uintptr_t a_s, uintptr_t b, uintptr_t b_s, uintptr_t c,
                                           uintptr_t offsets, int groups, int max_rows, int N, int K,
                                           int swiglu, uintptr_t stream) {
    check(grouped_gemm_fp8_blockscaled(P<void>(a), P<float>(a_s), P<void>(b), P<float>(b_s), P<void>(c),
                                       P<int>(offsets), groups, max_rows, N, K, swiglu, P<void>(stream)),
          "grouped_gemm_fp8_blockscaled");
  });
  m.def("ag_gemm_bf16", [](uintptr_t team, uintptr_t x, uintptr_t gathered, uintptr_t flags, uintptr_t b, uintptr_t c,
                           int m_shard, int N, int K, unsigned epoch, int swiglu, uintptr_t stream) {
    check(ag_gemm_bf16(reinterpret_cast<rocshmem_team_t>(team), P<void>(x), P<void>(gathered),
                       P<unsigned long long>(flags), P<void>(b), P<void>(c), m_shard, N, K, epoch, swiglu,
                       P<void>(stream)), "ag_gemm_bf16");
  });
  m.def("ag_gemm_fp8", [](uintptr_t team, uintptr_t x_q, uintptr_t x_s, uintptr_t gq, uintptr_t gs, uintptr_t flags,
                          uintptr_t b_q, uintptr_t b_s, uintptr_t c, int m_shard, int N, int K, unsigned epoch,
                          int swiglu, uintptr_t stream) {
    check(ag_gemm_fp8(reinterpret_cast<rocshmem_team_t>(team), P<void>(x_q), P<float>(x_s), P<void>(gq), P<float>(gs),
                      P<unsigned long long>(flags), P<void>(b_q), P<float>(b_s), P<void>(c), m_shard, N, K, epoch,
                      swiglu, P<void>(stream)), "ag_gemm_fp8");
  });
  m.def("gemm_rs_fp8", [](uintptr_t team, uintptr_t a_q, uintptr_t a_s, uintptr_t b_q, uintptr_t b_s,
                          uintptr_t staging, uintptr_t out, int m_shard, int N, int K, uintptr_t counter,
                          unsigned epoch, uintptr_t stream) {
    check(gemm_rs_fp8(reinterpret_cast<rocshmem_team_t>(team), P<void>(a_q), P<float>(a_s), P<void>(b_q), P<float>(b_s),
                      P<void>(staging), P<void>(out), m_shard, N, K, P<unsigned long long>(counter), epoch,
                      P<void>(stream)), "gemm_rs_fp8");
  });
  m.def("gemm_rs_bf16", [](uintptr_t team, uintptr_t a, uintptr_t b, uintptr_t staging, uintptr_t out, int m_shard,
                           int N, int K, uintptr_t counter, unsigned epoch, uintptr_t stream) {
    check(gemm_rs_bf16(reinterpret_cast<rocshmem_team_t>(team), P<void>(a), P<void>(b), P<void>(staging), P<void>(out),
                       m_shard, N, K, P<unsigned long long>(counter), epoch, P<void>(stream)), "gemm_rs_bf16");
  });
}

}  // namespace kernels
}  // namespace rocshmem
