// Python bindings (pybind11) of the runtime library. Pointers cross the boundary as integers; the
// Python layer wraps heap addresses into torch tensors.
#include <pybind11/functional.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include <cstring>

#include "kernels/kernels.hpp"
// Bindings of the MoE and GEMM kernels live beside those kernels' launchers.
namespace rocshmem { namespace kernels { void bind_ep(pybind11::module_ &m); void bind_gemm(pybind11::module_ &m); } }
#include "rocshmem/coalesce.h"
#include "rocshmem/rocshmem_debug.hpp"
#include "rocshmem/rocshmem_host.h"
#include "rocshmem/slab.h"
#include "runtime/allocator.hpp"
#include "runtime/bootstrap.hpp"
#include "runtime/config.hpp"
#include "runtime/host_ops.hpp"
#include "runtime/proxy.hpp"
#include "runtime/runtime.hpp"
#include "runtime/team.hpp"

namespace py = pybind11;
using namespace rocshmem;

namespace {

template <typename T>
T *ptr_of(uintptr_t v) { return reinterpret_cast<T *>(v); }
uintptr_t addr_of(const void *p) { return reinterpret_cast<uintptr_t>(p); }
rocshmem_team_t team_of(uintptr_t h) { return reinterpret_cast<rocshmem_team_t>(h); }

// The runtime, for calls that make no sense before init: an exception instead of a null dereference.
Runtime &live() {
  if (!Runtime::initialized()) throw std::runtime_error("rocshmem: library is not initialised");
  return Runtime::instance();
}
rocshmem_ctx_t ctx_of(uintptr_t c, uintptr_t t) { return rocshmem_ctx_t{ptr_of<void>(c), ptr_of<void>(t)}; }

void check_launch(int rc, const char *what) {
  if (rc != 0) throw std::runtime_error(std::string(what) + ": CUDA error " + std::to_string(rc));
}

std::map<std::string, std::string> to_overrides(const py::dict &d) {
  std::map<std::string, std::string> m;
  for (auto item : d) m[py::str(item.first)] = py::str(item.second);
  return m;
}

py::dict error_to_dict(const rocshmem_error_record &e) {
  py::dict d;
  d["count"] = e.count;
  d["kind"] = e.kind;
  d["pe"] = e.pe;
  d["where"] = e.where;
  d["addr"] = e.addr;
  d["expected"] = e.expected;
  d["observed"] = e.observed;
  return d;
}

}  // namespace

PYBIND11_MODULE(_C, m) {
  m.doc() = "rocshmem_b200 native runtime";

  // ---- lifecycle ----------------------------------------------------------------------------------
  m.def("init_with_store",
        [](int rank, int size, py::function put, py::function get, py::dict overrides, int n_local,
           int device, int timeout_ms) {
          auto put_fn = [put](const std::string &k, const std::string &v) {
            py::gil_scoped_acquire g;
            put(k, py::bytes(v));
          };
          auto get_fn = [get](const std::string &k, int ms) -> std::string {
            py::gil_scoped_acquire g;
            return py::cast<std::string>(get(k, ms));
          };
          auto bs = std::make_unique<CallbackBootstrap>(rank, size, put_fn, get_fn);
          bs->set_timeout_ms(timeout_ms);
          Config cfg = Config::from_env(to_overrides(overrides));
          Runtime::instance().init(std::move(bs), cfg, n_local, device);
          ROCSHMEM_TEAM_WORLD = Runtime::instance().team_world()->dev;
        },
        py::arg("rank"), py::arg("size"), py::arg("put"), py::arg("get"), py::arg("overrides"),
        py::arg("n_local") = 1, py::arg("device") = 0, py::arg("timeout_ms") = 120000);
  m.def("init_file",
        [](int rank, int size, const std::string &dir, py::dict overrides, int n_local, int device,
           int timeout_ms) {
          std::unique_ptr<Bootstrap> bs;
          if (size <= 1) bs = std::make_unique<LocalBootstrap>();
          else bs = std::make_unique<FileBootstrap>(dir, rank, size);
          bs->set_timeout_ms(timeout_ms);
          Config cfg = Config::from_env(to_overrides(overrides));
          py::gil_scoped_release rel;
          Runtime::instance().init(std::move(bs), cfg, n_local, device);
          ROCSHMEM_TEAM_WORLD = Runtime::instance().team_world()->dev;
        },
        py::arg("rank"), py::arg("size"), py::arg("dir"), py::arg("overrides"), py::arg("n_local") = 1,
        py::arg("device") = 0, py::arg("timeout_ms") = 120000);
  m.def("finalize", [] { host::finalize(); });
  m.def("is_initialized", [] { return Runtime::initialized(); });
  m.def("my_pe", [] { return host::my_pe(); });
  m.def("n_pes", [] { return host::n_pes(); });
  m.def("n_local", [] { return live().n_local(); });
  m.def("first_pe", [] { return live().first_pe(); });
  m.def("set_local_pe", [](int l) { rocshmemx_set_local_pe(l); });
  m.def("is_cuda", [] { return live().is_cuda(); });
  m.def("backend_name", [] { return std::string(live().mem().name()); });
  m.def("cuda_device_count", [] { return cuda_device_count(); });
  m.def("nvls_available", [] { return live().mc_base() != nullptr; });
  m.def("check_canaries", [] { return live().check_canaries(); });
  m.def("internal_guard_offsets", [] { return live().layout().guards; });
  m.def("dump_stats", [] { host::dump_stats(); });
  m.def("reset_stats", [] { host::reset_stats(); });
  m.def("device_stats", [](int local) { return live().read_stats(local); }, py::arg("local") = -1);
  m.def("host_stats", [] { return live().host_stats(); });
  m.def("get_error", [](int local) { return error_to_dict(live().read_error(local)); },
        py::arg("local") = -1);
  m.def("clear_error", [] { rocshmemx_clear_error(); });
  m.def("set_wait_timeout_ms", [](uint64_t ms) { rocshmemx_set_wait_timeout_ms(ms); });
  m.def("default_stream", [] { return addr_of(rocshmemx_default_stream()); });

  // ---- heap -------------------------------------------------------------------------------------------
  m.def("malloc", [](size_t bytes) { return addr_of(host::malloc(bytes)); });
  m.def("free", [](uintptr_t p) { host::free(ptr_of<void>(p)); });
  m.def("ptr", [](uintptr_t p, int pe) { return addr_of(host::ptr(ptr_of<void>(p), pe)); });
  m.def("heap_base", [](int pe) { return addr_of(live().heap_base(pe)); });
  m.def("heap_size", [] { return live().heap_size(); });
  m.def("heap_stride", [] { return live().stride(); });
  m.def("heap_used", [] { return live().heap_used(); });
  m.def("heap_avail", [] { return live().heap_avail(); });
  m.def("mc_base", [] { return addr_of(live().mc_base()); });
  m.def("heap_write", [](uintptr_t dst, py::bytes data) {
    std::string s = data;
    rocshmemx_heap_write(ptr_of<void>(dst), s.data(), s.size());
  });
  m.def("heap_read", [](uintptr_t src, size_t bytes) {
    std::string s(bytes, '\0');
    rocshmemx_heap_read(&s[0], ptr_of<void>(src), bytes);
    return py::bytes(s);
  });

  // ---- teams and contexts ----------------------------------------------------------------------------
  m.def("team_world", [] { return addr_of(ROCSHMEM_TEAM_WORLD); });
  m.def("team_split_strided", [](uintptr_t parent, int start, int stride, int size) {
    rocshmem_team_t out = nullptr;
    int rc = host::team_split_strided(team_of(parent), start, stride, size, nullptr, 0, &out);
    return py::make_tuple(rc, addr_of(out));
  });
  m.def("team_destroy", [](uintptr_t t) { host::team_destroy(team_of(t)); });
  m.def("team_n_pes", [](uintptr_t t) { return host::team_n_pes(team_of(t)); });
  m.def("team_my_pe", [](uintptr_t t) { return host::team_my_pe(team_of(t)); });
  m.def("team_translate_pe", [](uintptr_t s, int pe, uintptr_t d) {
    return host::team_translate_pe(team_of(s), pe, team_of(d));
  });
  m.def("team_sync", [](uintptr_t t) { return host::team_sync(team_of(t)); });
  m.def("num_user_teams", [] { return live().num_user_teams(); });
  m.def("ctx_create", [](int64_t options) {
    rocshmem_ctx_t c{nullptr, nullptr};
    int rc = host::ctx_create(options, &c);
    return py::make_tuple(rc, addr_of(c.ctx_opaque), addr_of(c.team_opaque));
  });
  m.def("team_create_ctx", [](uintptr_t team, int64_t options) {
    rocshmem_ctx_t c{nullptr, nullptr};
    int rc = host::team_create_ctx(team_of(team), options, &c);
    return py::make_tuple(rc, addr_of(c.ctx_opaque), addr_of(c.team_opaque));
  });
  m.def("ctx_destroy", [](uintptr_t c, uintptr_t t) { host::ctx_destroy(ctx_of(c, t)); });

  // ---- host RMA / AMO / sync ---------------------------------------------------------------------------
  m.def("putmem", [](uintptr_t dst, uintptr_t src, size_t n, int pe, uintptr_t c, uintptr_t t) {
    host::putmem(ctx_of(c, t), ptr_of<void>(dst), ptr_of<void>(src), n, pe);
  }, py::arg("dst"), py::arg("src"), py::arg("bytes"), py::arg("pe"), py::arg("ctx") = 0, py::arg("ctx_team") = 0);
  m.def("getmem", [](uintptr_t dst, uintptr_t src, size_t n, int pe, uintptr_t c, uintptr_t t) {
    host::getmem(ctx_of(c, t), ptr_of<void>(dst), ptr_of<void>(src), n, pe);
  }, py::arg("dst"), py::arg("src"), py::arg("bytes"), py::arg("pe"), py::arg("ctx") = 0, py::arg("ctx_team") = 0);
  m.def("putmem_nbi", [](uintptr_t dst, uintptr_t src, size_t n, int pe, uintptr_t c, uintptr_t t) {
    host::putmem_nbi(ctx_of(c, t), ptr_of<void>(dst), ptr_of<void>(src), n, pe);
  }, py::arg("dst"), py::arg("src"), py::arg("bytes"), py::arg("pe"), py::arg("ctx") = 0, py::arg("ctx_team") = 0);
  m.def("getmem_nbi", [](uintptr_t dst, uintptr_t src, size_t n, int pe, uintptr_t c, uintptr_t t) {
    host::getmem_nbi(ctx_of(c, t), ptr_of<void>(dst), ptr_of<void>(src), n, pe);
  }, py::arg("dst"), py::arg("src"), py::arg("bytes"), py::arg("pe"), py::arg("ctx") = 0, py::arg("ctx_team") = 0);
  m.def("p", [](uintptr_t dst, uint64_t bits, size_t elem, int pe) {
    host::p(rocshmem_ctx_t{nullptr, nullptr}, ptr_of<void>(dst), bits, elem, pe);
  });
  m.def("g", [](uintptr_t src, size_t elem, int pe) {
    return host::g(rocshmem_ctx_t{nullptr, nullptr}, ptr_of<void>(src), elem, pe);
  });
  m.def("amo", [](int op, int dtype, uintptr_t target, uint64_t value, uint64_t cond, int pe, uintptr_t c,
                  uintptr_t t) {
    return host::amo(ctx_of(c, t), op, dtype, ptr_of<void>(target), value, cond, pe);
  }, py::arg("op"), py::arg("dtype"), py::arg("target"), py::arg("value"), py::arg("cond"), py::arg("pe"),
     py::arg("ctx") = 0, py::arg("ctx_team") = 0);
  m.def("fence", [] { host::fence(rocshmem_ctx_t{nullptr, nullptr}); });
  m.def("quiet", [](uintptr_t c, uintptr_t t) { host::quiet(ctx_of(c, t)); }, py::arg("ctx") = 0,
        py::arg("ctx_team") = 0);
  m.def("barrier_all", [] { py::gil_scoped_release r; host::barrier_all(); });
  m.def("sync_all", [] { py::gil_scoped_release r; host::sync_all(); });
  m.def("wait_until", [](uintptr_t ivar, int dtype, int cmp, uint64_t value) {
    py::gil_scoped_release r;
    return host::wait_until(ptr_of<void>(ivar), dtype, cmp, value);
  });
  m.def("test", [](uintptr_t ivar, int dtype, int cmp, uint64_t value) {
    return host::test(ptr_of<void>(ivar), dtype, cmp, value);
  });
  m.def("wait_until_all", [](uintptr_t ivars, size_t n, std::vector<int> status, int dtype, int cmp,
                             std::vector<uint64_t> values, bool vector) {
    py::gil_scoped_release r;
    host::wait_until_all(ptr_of<void>(ivars), n, status.empty() ? nullptr : status.data(), dtype, cmp,
                         values.data(), vector);
  });
  m.def("wait_until_any", [](uintptr_t ivars, size_t n, std::vector<int> status, int dtype, int cmp,
                             std::vector<uint64_t> values, bool vector) {
    py::gil_scoped_release r;
    return host::wait_until_any(ptr_of<void>(ivars), n, status.empty() ? nullptr : status.data(), dtype,
                                cmp, values.data(), vector);
  });
  m.def("wait_until_some", [](uintptr_t ivars, size_t n, std::vector<int> status, int dtype, int cmp,
                              std::vector<uint64_t> values, bool vector) {
    std::vector<size_t> idx(n ? n : 1);
    size_t found;
    {
      py::gil_scoped_release r;
      found = host::wait_until_some(ptr_of<void>(ivars), n, idx.data(), status.empty() ? nullptr : status.data(),
                                    dtype, cmp, values.data(), vector);
    }
    idx.resize(found);
    return idx;
  });

  // ---- host collectives -----------------------------------------------------------------------------------
  m.def("broadcast", [](uintptr_t team, uintptr_t dst, uintptr_t src, size_t bytes, int root) {
    py::gil_scoped_release r;
    return host::broadcast(rocshmem_ctx_t{nullptr, nullptr}, team_of(team), ptr_of<void>(dst), ptr_of<void>(src), bytes, root);
  });
  m.def("reduce", [](uintptr_t team, uintptr_t dst, uintptr_t src, size_t n, int dtype, int op) {
    py::gil_scoped_release r;
    return host::reduce(rocshmem_ctx_t{nullptr, nullptr}, team_of(team), ptr_of<void>(dst), ptr_of<void>(src), n, dtype, op);
  });
  m.def("fcollect", [](uintptr_t team, uintptr_t dst, uintptr_t src, size_t bytes) {
    py::gil_scoped_release r;
    return host::fcollect(rocshmem_ctx_t{nullptr, nullptr}, team_of(team), ptr_of<void>(dst), ptr_of<void>(src), bytes);
  });
  m.def("alltoall", [](uintptr_t team, uintptr_t dst, uintptr_t src, size_t bytes) {
    py::gil_scoped_release r;
    return host::alltoall(rocshmem_ctx_t{nullptr, nullptr}, team_of(team), ptr_of<void>(dst), ptr_of<void>(src), bytes);
  });
  m.def("reduce_active_set", [](uintptr_t dst, uintptr_t src, size_t n, int dtype, int op, int start,
                                int log_stride, int size) {
    py::gil_scoped_release r;
    return host::reduce_active_set(rocshmem_ctx_t{nullptr, nullptr}, ptr_of<void>(dst), ptr_of<void>(src), n,
                                   dtype, op, start, log_stride, size);
  });

  // ---- stream-ordered library kernels ----------------------------------------------------------------------
  m.def("k_barrier", [](uintptr_t team, uintptr_t stream) {
    check_launch(kernels::coll_barrier(team_of(team), ptr_of<void>(stream)), "barrier");
  });
  m.def("k_allreduce", [](uintptr_t team, uintptr_t dst, uintptr_t src, size_t n, int dtype, int op, int algo,
                          uintptr_t stream) {
    check_launch(kernels::coll_allreduce(team_of(team), ptr_of<void>(dst), ptr_of<void>(src), n, dtype, op,
                                         algo, ptr_of<void>(stream)), "allreduce");
  });
  m.def("k_broadcast", [](uintptr_t team, uintptr_t dst, uintptr_t src, size_t bytes, int root,
                          uintptr_t stream, int flags) {
    check_launch(kernels::coll_broadcast(team_of(team), ptr_of<void>(dst), ptr_of<void>(src), bytes, root,
                                         ptr_of<void>(stream), flags), "broadcast");
  });
  m.def("k_fcollect", [](uintptr_t team, uintptr_t dst, uintptr_t src, size_t bytes, uintptr_t stream, int flags) {
    check_launch(kernels::coll_fcollect(team_of(team), ptr_of<void>(dst), ptr_of<void>(src), bytes,
                                        ptr_of<void>(stream), flags), "fcollect");
  });
  m.def("k_alltoall", [](uintptr_t team, uintptr_t dst, uintptr_t src, size_t bytes, uintptr_t stream, int flags) {
    check_launch(kernels::coll_alltoall(team_of(team), ptr_of<void>(dst), ptr_of<void>(src), bytes,
                                        ptr_of<void>(stream), flags), "alltoall");
  });
  m.def("coll_blocks_for", [](size_t bytes) { return kernels::coll_blocks_for(bytes); });
  kernels::bind_ep(m);
  kernels::bind_gemm(m);

  // ---- proxy -----------------------------------------------------------------------------------------------
  m.def("proxy_running", [] {
    Proxy *p = live().proxy();
    return p && p->running();
  });
  m.def("proxy_start", [] {
    // Test hook: start a proxy on any backend (the CPU backend exercises the ring protocol).
    static std::unique_ptr<Proxy> extra;
    if (!live().proxy()) {
      extra = std::make_unique<Proxy>(&live());
      extra->start();
      return addr_of(extra.get());
    }
    return addr_of(live().proxy());
  });
  m.def("proxy_stop", [](uintptr_t p) { ptr_of<Proxy>(p)->stop(); });
  m.def("proxy_submit", [](uintptr_t p, unsigned type, int pe, uintptr_t dst, uintptr_t src, uint64_t size,
                           uint64_t cond, unsigned op, unsigned dtype_size, bool blocking, uint64_t timeout_ms,
                           uint64_t team_slot) {
    rocshmem_proxy_cmd c;
    std::memset(&c, 0, sizeof(c));
    c.type = type;
    c.pe = pe;
    c.dst = dst;
    c.src = src;
    c.size = size;
    c.cond = cond;
    c.op = op;
    c.dtype_size = dtype_size;
    c.team_slot = team_slot;
    uint64_t fetched = 0;
    int rc;
    {
      py::gil_scoped_release r;
      rc = ptr_of<Proxy>(p)->submit(c, blocking, &fetched, timeout_ms);
    }
    return py::make_tuple(rc, fetched);
  }, py::arg("proxy"), py::arg("type"), py::arg("pe"), py::arg("dst"), py::arg("src"), py::arg("size"),
     py::arg("cond"), py::arg("op"), py::arg("dtype_size"), py::arg("blocking"), py::arg("timeout_ms"),
     py::arg("team_slot") = 0);
  m.def("team_slot", [](uintptr_t t) {
    HostTeam *ht = live().team_from_handle(team_of(t));
    return ht ? ht->slot : -1;
  });
  m.def("team_has_nvls", [](uintptr_t t) {
    HostTeam *ht = live().team_from_handle(team_of(t));
    return ht != nullptr && ht->mc_window != nullptr;
  });
  m.def("proxy_inject_drop", [](uintptr_t p, int n) { ptr_of<Proxy>(p)->inject_drop(n); });
  m.def("proxy_inject_delay_ms", [](uintptr_t p, int ms) { ptr_of<Proxy>(p)->inject_delay_ms(ms); });
  m.def("proxy_counts", [](uintptr_t p) {
    return py::make_tuple(ptr_of<Proxy>(p)->executed(), ptr_of<Proxy>(p)->dropped());
  });
  // ---- slab ---------------------------------------------------------------------------------------------------
  auto slab_of = [](uintptr_t base, uint64_t size) {
    rocshmemx_slab_t s{reinterpret_cast<char *>(base), size,
                       reinterpret_cast<unsigned long long *>(base + size)};
    return s;
  };
  m.def("slab_create", [](size_t bytes) {
    rocshmemx_slab_t s = rocshmemx_slab_create(bytes);
    return py::make_tuple(reinterpret_cast<uintptr_t>(s.base), static_cast<uint64_t>(s.size));
  });
  m.def("slab_destroy", [slab_of](uintptr_t base, uint64_t size) { rocshmemx_slab_destroy(slab_of(base, size)); });
  m.def("slab_reset", [slab_of](uintptr_t base, uint64_t size) { rocshmemx_slab_reset(slab_of(base, size)); });
  m.def("slab_used", [slab_of](uintptr_t base, uint64_t size) { return rocshmemx_slab_used(slab_of(base, size)); });
  m.def("slab_alloc_host", [slab_of](uintptr_t base, uint64_t size, size_t bytes, size_t align) {
    return reinterpret_cast<uintptr_t>(rocshmemx_slab_alloc_host(slab_of(base, size), bytes, align));
  });
  m.def("proxy_set_coalesce", [](uintptr_t p, bool on) { ptr_of<Proxy>(p)->set_coalesce(on); });
  m.def("proxy_merged", [](uintptr_t p) { return ptr_of<Proxy>(p)->merged(); });
  m.def("proxy_describe_command", [](uintptr_t p, unsigned i) { return ptr_of<Proxy>(p)->describe_command(i); });
  m.def("proxy_describe_completion", [](uintptr_t p, unsigned i) { return ptr_of<Proxy>(p)->describe_completion(i); });
  m.def("debug_print_ring", [](int first, int count) { live(); debug_print_ring(first, count); });
  // The lane-mask arithmetic of the warp coalescer, evaluated for every lane of one warp.
  m.def("coalesce_warp_plan", [](unsigned active, std::vector<std::tuple<int, uint64_t, uint64_t, uint64_t>> msgs) {
    if (msgs.size() != 32) throw std::invalid_argument("coalesce_warp_plan wants 32 lane messages");
    unsigned cont = 0;
    auto at = [&](int l) {
      coalesce::Msg m{std::get<0>(msgs[l]), std::get<1>(msgs[l]), std::get<2>(msgs[l]), std::get<3>(msgs[l])};
      return m;
    };
    for (int l = 0; l < 32; ++l) {
      if (!(active & (1u << l))) continue;
      int p = coalesce::previous_active(active, l);
      if (p >= 0 && coalesce::continues(at(p), at(l))) cont |= 1u << l;
    }
    std::vector<int> runs(32);
    for (int l = 0; l < 32; ++l) runs[l] = coalesce::run_length(active, cont, l);
    return runs;
  });
  m.def("coalesce_merge_runs", [](std::vector<std::tuple<int, uint64_t, uint64_t, uint64_t>> msgs) {
    std::vector<coalesce::Msg> m;
    for (auto &t : msgs) m.push_back({std::get<0>(t), std::get<1>(t), std::get<2>(t), std::get<3>(t)});
    size_t n = coalesce::merge_runs(m.data(), m.size());
    std::vector<std::tuple<int, uint64_t, uint64_t, uint64_t>> out;
    for (size_t i = 0; i < n; ++i) out.emplace_back(m[i].pe, m[i].dst, m[i].src, m[i].size);
    return out;
  });

  // ---- pieces exposed for unit tests ----------------------------------------------------------------------
  m.def("parse_size", [](const std::string &s) { return parse_size(s); });
  m.def("config_from_env", [](py::dict overrides) {
    Config c = Config::from_env(to_overrides(overrides));
    py::dict d;
    d["heap_size"] = c.heap_size;
    d["scratch_size"] = c.scratch_size;
    d["slab_size"] = c.slab_size;
    d["max_contexts"] = c.max_contexts;
    d["max_host_contexts"] = c.max_host_contexts;
    d["max_teams"] = c.max_teams;
    d["wait_timeout_ms"] = c.wait_timeout_ms;
    d["debug"] = c.debug;
    d["debug_checks"] = c.debug_checks;
    d["use_proxy"] = c.use_proxy;
    d["proxy_queue_size"] = c.proxy_queue_size;
    d["proxy_coalesce"] = c.proxy_coalesce;
    d["proxy_collectives"] = c.proxy_collectives;
    d["enable_nvls"] = c.enable_nvls;
    d["team_nvls"] = c.team_nvls;
    d["backend"] = c.backend;
    d["bootstrap_dir"] = c.bootstrap_dir;
    return d;
  });
  py::class_<Pow2Allocator>(m, "Pow2Allocator")
      .def(py::init<size_t, size_t>(), py::arg("size"), py::arg("alignment") = 128)
      .def("alloc", [](Pow2Allocator &a, size_t n) -> py::object {
        size_t off = a.alloc(n);
        if (off == Pow2Allocator::kNull) return py::none();
        return py::int_(off);
      })
      .def("free", &Pow2Allocator::free)
      .def("block_size", &Pow2Allocator::block_size)
      .def("used", &Pow2Allocator::used)
      .def("avail", &Pow2Allocator::avail)
      .def("managed", &Pow2Allocator::managed)
      .def("largest_free_block", &Pow2Allocator::largest_free_block)
      .def("bin_population", &Pow2Allocator::bin_population)
      .def("live_allocations", &Pow2Allocator::live_allocations);
  m.def("plan_split", [](int p_start, int p_stride, int p_size, int world, int start, int stride, int size) -> py::object {
    SplitPlan plan = plan_split(TeamTriplet{p_start, p_stride, p_size}, p_size, world, start, stride, size);
    if (!plan.ok) return py::none();
    return py::make_tuple(plan.world.pe_start, plan.world.stride, plan.world.size);
  });
  m.def("translate_pe", [](py::tuple src, int pe, py::tuple dst) {
    TeamTriplet s{src[0].cast<int>(), src[1].cast<int>(), src[2].cast<int>()};
    TeamTriplet d{dst[0].cast<int>(), dst[1].cast<int>(), dst[2].cast<int>()};
    return translate_pe(s, pe, d);
  });
  m.def("lowest_common_slot", [](std::vector<uint64_t> masks) { return TeamSlots::lowest_common(masks); });
  m.def("exchange_fds_file", [](const std::string &dir, int rank, int size, int fd, int timeout_ms) {
    FileBootstrap bs(dir, rank, size);
    bs.set_timeout_ms(timeout_ms);
    py::gil_scoped_release r;
    return exchange_fds(bs, "test", fd);
  });
  m.def("broadcast_fd_group_file", [](const std::string &dir, int rank, int size, std::vector<int> members, int fd,
                                      int timeout_ms) {
    FileBootstrap bs(dir, rank, size);
    bs.set_timeout_ms(timeout_ms);
    int my_index = -1;
    for (size_t i = 0; i < members.size(); ++i)
      if (members[i] == rank) my_index = static_cast<int>(i);
    if (my_index < 0) throw std::invalid_argument("broadcast_fd_group_file: the caller is not a member");
    py::gil_scoped_release r;
    return broadcast_fd_group(bs, "test-group", members, my_index, fd);
  });
  m.def("file_bootstrap_allgather", [](const std::string &dir, int rank, int size, py::bytes value, int timeout_ms) {
    FileBootstrap bs(dir, rank, size);
    bs.set_timeout_ms(timeout_ms);
    std::string in = value;
    std::string out(in.size() * size, '\0');
    {
      py::gil_scoped_release r;
      bs.allgather("t", in.data(), &out[0], in.size());
    }
    return py::bytes(out);
  });

  m.attr("NUM_STATS") = static_cast<int>(ROCSHMEM_NUM_STATS);
  m.attr("MAX_PES") = ROCSHMEM_MAX_PES;
  m.attr("ALIGNMENT") = static_cast<int>(ROCSHMEM_ALIGNMENT);
}
