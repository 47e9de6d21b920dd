// Python bindings of the MoE expert-parallel kernels.
#include <pybind11/pybind11.h>

namespace rocshmem {
namespace kernels {
void bind_ep(pybind11::module_ &) {}
}  // namespace kernels
}  // namespace rocshmem
