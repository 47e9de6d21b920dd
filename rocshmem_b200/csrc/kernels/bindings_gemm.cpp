// Python bindings of the tcgen05 GEMM kernels and the fused GEMM + collective kernels.
#include <pybind11/pybind11.h>

namespace rocshmem {
namespace kernels {
void bind_gemm(pybind11::module_ &) {}
}  // namespace kernels
}  // namespace rocshmem
