// Python bindings of the MoE expert-parallel kernels.
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include <stdexcept>
#include <string>

#include "ep_kernels.hpp"
#include "moe_kernels.hpp"

namespace py = pybind11;

namespace rocshmem {
namespace kernels {

namespace {
template <typename T>
T *P(uintptr_t v) { return reinterpret_cast<T *>(v); }

void check(int rc, const char *what) {
  if (rc != 0) throw std::runtime_error(std::string(what) + ": CUDA error " + std::to_string(rc));
}

struct EpHandle {
  EpConfig cfg{};
  EpBuffers buf{};
  uintptr_t team = 0;
  unsigned epoch = 0;
  unsigned long long combine_base = 0;  // dynamic mode: counter increments of all earlier combine calls
};
}  // namespace

void bind_ep(py::module_ &m) {
  py::class_<EpHandle>(m, "EpHandle")
      .def(py::init([](uintptr_t team, int num_experts, int top_k, int hidden, int max_tokens, int quantize,
                       int layout, int blocks, int dynamic, int expert_layout, int low_latency, py::dict ptrs) {
        EpHandle h;
        h.team = team;
        h.cfg = EpConfig{num_experts, top_k, hidden, max_tokens, quantize, layout, blocks, dynamic, expert_layout,
                         low_latency};
        auto get = [&ptrs](const char *k) -> uintptr_t {
          return ptrs.contains(k) ? ptrs[k].cast<uintptr_t>() : uintptr_t(0);
        };
        h.buf.recv_x = P<void>(get("recv_x"));
        h.buf.recv_scales = P<float>(get("recv_scales"));
        h.buf.recv_meta = P<int>(get("recv_meta"));
        h.buf.cnt_in = P<unsigned long long>(get("cnt_in"));
        h.buf.exp_in = P<unsigned long long>(get("exp_in"));
        h.buf.sent_slot = P<int>(get("sent_slot"));
        h.buf.tok_mask = P<unsigned long long>(get("tok_mask"));
        h.buf.blk_cnt = P<int>(get("blk_cnt"));
        h.buf.exp_cnt = P<int>(get("exp_cnt"));
        h.buf.grid_counter = P<unsigned long long>(get("grid_counter"));
        h.buf.phase_ns = P<unsigned long long>(get("phase_ns"));
        h.buf.recv_info = P<int>(get("recv_info"));
        h.buf.work_counter = P<unsigned long long>(get("work_counter"));
        h.buf.stage_meta = P<int>(get("stage_meta"));
        h.buf.item_tok = P<int>(get("item_tok"));
        h.buf.lay_offsets = P<int>(get("lay_offsets"));
        h.buf.lay_row = P<int>(get("lay_row"));
        h.buf.lay_k = P<int>(get("lay_k"));
        h.buf.lay_w = P<float>(get("lay_w"));
        return h;
      }))
      .def_readonly("epoch", &EpHandle::epoch)
      .def("dispatch", [](EpHandle &h, uintptr_t x, uintptr_t topk_idx, uintptr_t topk_w, int num_tokens,
                          uintptr_t stream) {
        h.epoch += 1;
        check(ep_dispatch(reinterpret_cast<rocshmem_team_t>(h.team), h.cfg, h.buf, P<void>(x), P<int>(topk_idx),
                          P<float>(topk_w), num_tokens, h.epoch, P<void>(stream)), "ep_dispatch");
      })
      .def("combine", [](EpHandle &h, uintptr_t y, uintptr_t out, uintptr_t topk_idx, uintptr_t topk_w,
                         int num_tokens, int weighted, uintptr_t stream) {
        check(ep_combine(reinterpret_cast<rocshmem_team_t>(h.team), h.cfg, h.buf, P<void>(y), P<void>(out),
                         P<int>(topk_idx), P<float>(topk_w), num_tokens, weighted, P<void>(stream), h.combine_base),
              "ep_combine");
        if (h.cfg.dynamic) h.combine_base += ep_combine_fetches(h.cfg, num_tokens);
      })
      .def("expert_layout", [](EpHandle &h, int n_ranks, uintptr_t offsets, uintptr_t row_index, uintptr_t pair_k,
                               uintptr_t cursor, uintptr_t stream) {
        check(ep_expert_layout(h.buf.recv_meta, h.buf.recv_info, n_ranks, h.cfg.max_tokens, h.cfg.layout,
                               h.cfg.num_experts / n_ranks, h.cfg.top_k, P<int>(offsets), P<int>(row_index),
                               P<int>(pair_k), P<int>(cursor), P<void>(stream)), "ep_expert_layout");
      });
  m.def("ep_default_blocks", [] { return ep_default_blocks(); });
  m.def("fp8_quantize_1x128", [](uintptr_t x, uintptr_t q, uintptr_t scales, size_t rows, int hidden, uintptr_t stream) {
    check(fp8_quantize_1x128(P<void>(x), P<void>(q), P<float>(scales), rows, hidden, P<void>(stream)), "fp8_quantize");
  });
  m.def("fp8_dequantize_1x128", [](uintptr_t q, uintptr_t scales, uintptr_t x, size_t rows, int hidden, uintptr_t stream) {
    check(fp8_dequantize_1x128(P<void>(q), P<float>(scales), P<void>(x), rows, hidden, P<void>(stream)), "fp8_dequantize");
  });
  m.def("moe_gather_rows", [](uintptr_t recv_x, uintptr_t scales, int fp8, uintptr_t offsets, int experts,
                              uintptr_t row_index, int hidden, uintptr_t out, uintptr_t stream) {
    check(moe_gather_rows(P<void>(recv_x), P<float>(scales), fp8, P<int>(offsets), experts, P<int>(row_index), hidden,
                          P<void>(out), P<void>(stream)), "moe_gather_rows");
  });
  m.def("moe_zero_rows", [](uintptr_t recv_info, int n_ranks, int hidden, uintptr_t y, uintptr_t stream) {
    check(moe_zero_rows(P<int>(recv_info), n_ranks, hidden, P<void>(y), P<void>(stream)), "moe_zero_rows");
  });
  m.attr("EP_META_WORDS") = EP_META_WORDS;
  m.attr("EP_WORK_WORDS") = EP_WORK_WORDS;
  m.attr("EP_MAX_RANKS") = EP_MAX_RANKS;
}

}  // namespace kernels
}  // namespace rocshmem
