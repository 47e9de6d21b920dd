#include "config.hpp"

#include <cctype>
#include <cerrno>
#include <cstdlib>
#include <stdexcept>

#include "rocshmem/rocshmem_common.h"

namespace rocshmem {

size_t parse_size(const std::string &text_in) {
  std::string text;
  for (char c : text_in) {
    if (!std::isspace(static_cast<unsigned char>(c))) text.push_back(c);
  }
  if (text.empty()) throw std::invalid_argument("empty size");
  unsigned shift = 0;
  char last = static_cast<char>(std::toupper(static_cast<unsigned char>(text.back())));
  if (last == 'B' && text.size() > 1) {  // allow "64MB" / "64MiB"
    text.pop_back();
    if (!text.empty() && (text.back() == 'i' || text.back() == 'I')) text.pop_back();
    if (text.empty()) throw std::invalid_argument("bad size '" + text_in + "'");
    last = static_cast<char>(std::toupper(static_cast<unsigned char>(text.back())));
  }
  switch (last) {
    case 'K': shift = 10; break;
    case 'M': shift = 20; break;
    case 'G': shift = 30; break;
    case 'T': shift = 40; break;
    default: break;
  }
  if (shift) text.pop_back();
  if (text.empty() || text[0] == '-') throw std::invalid_argument("bad size '" + text_in + "'");
  errno = 0;
  char *end = nullptr;
  unsigned long long v = std::strtoull(text.c_str(), &end, 0);
  if (errno != 0 || end == text.c_str() || *end != '\0') {
    throw std::invalid_argument("bad size '" + text_in + "'");
  }
  if (shift && (v >> (64 - shift)) != 0) throw std::invalid_argument("size overflows: " + text_in);
  return static_cast<size_t>(v << shift);
}

long parse_int(const std::string &text) {
  errno = 0;
  char *end = nullptr;
  long v = std::strtol(text.c_str(), &end, 0);
  while (end && *end && std::isspace(static_cast<unsigned char>(*end))) ++end;
  if (errno != 0 || end == text.c_str() || (end && *end != '\0')) {
    throw std::invalid_argument("bad integer '" + text + "'");
  }
  return v;
}

namespace {
bool lookup(const std::map<std::string, std::string> &ov, const char *key, std::string *out) {
  auto it = ov.find(key);
  if (it != ov.end()) {
    *out = it->second;
    return true;
  }
  const char *e = std::getenv(key);
  if (e && *e) {
    *out = e;
    return true;
  }
  return false;
}
}  // namespace

Config Config::from_env(const std::map<std::string, std::string> &ov) {
  Config c;
  std::string v;
  try {
    if (lookup(ov, "ROCSHMEM_HEAP_SIZE", &v)) c.heap_size = parse_size(v);
    if (lookup(ov, "ROCSHMEM_SCRATCH_SIZE", &v)) c.scratch_size = parse_size(v);
    if (lookup(ov, "ROCSHMEM_SLAB_SIZE", &v)) c.slab_size = parse_size(v);
    if (lookup(ov, "ROCSHMEM_MAX_NUM_CONTEXTS", &v)) c.max_contexts = static_cast<int>(parse_int(v));
    if (lookup(ov, "ROCSHMEM_MAX_NUM_HOST_CONTEXTS", &v))
      c.max_host_contexts = static_cast<int>(parse_int(v));
    if (lookup(ov, "ROCSHMEM_MAX_NUM_TEAMS", &v)) c.max_teams = static_cast<int>(parse_int(v));
    if (lookup(ov, "ROCSHMEM_WAIT_TIMEOUT_MS", &v))
      c.wait_timeout_ms = static_cast<uint64_t>(parse_int(v));
    if (lookup(ov, "ROCSHMEM_DEBUG", &v)) c.debug = static_cast<int>(parse_int(v));
    if (lookup(ov, "ROCSHMEM_DEBUG_CHECKS", &v)) c.debug_checks = static_cast<int>(parse_int(v));
    if (lookup(ov, "ROCSHMEM_USE_PROXY", &v)) c.use_proxy = static_cast<int>(parse_int(v));
    if (lookup(ov, "RO_NET_QUEUE_SIZE", &v)) c.proxy_queue_size = static_cast<int>(parse_int(v));
    if (lookup(ov, "RO_NET_CPU_QUEUE", &v)) c.proxy_on_cpu = static_cast<int>(parse_int(v));
    if (lookup(ov, "ROCSHMEM_PROXY_COLLECTIVES", &v)) c.proxy_collectives = static_cast<int>(parse_int(v)) != 0;
    if (lookup(ov, "ROCSHMEM_USE_WF_COAL", &v)) c.proxy_coalesce = static_cast<int>(parse_int(v)) != 0;
    if (lookup(ov, "ROCSHMEM_ENABLE_NVLS", &v)) c.enable_nvls = static_cast<int>(parse_int(v));
    if (lookup(ov, "ROCSHMEM_TEAM_NVLS", &v)) c.team_nvls = static_cast<int>(parse_int(v)) != 0;
    if (lookup(ov, "ROCSHMEM_BACKEND", &v)) c.backend = v;
    if (lookup(ov, "ROCSHMEM_BOOTSTRAP_DIR", &v)) c.bootstrap_dir = v;
  } catch (const std::invalid_argument &e) {
    throw std::invalid_argument(std::string("rocshmem config: ") + e.what());
  }
  c.validate();
  return c;
}

void Config::validate() const {
  auto fail = [](const std::string &m) { throw std::invalid_argument("rocshmem config: " + m); };
  if (heap_size < ROCSHMEM_ALIGNMENT) fail("ROCSHMEM_HEAP_SIZE must be at least 128 bytes");
  if (heap_size > (size_t(1) << 40)) fail("ROCSHMEM_HEAP_SIZE above 1 TiB");
  if (scratch_size < (size_t(1) << 16)) fail("ROCSHMEM_SCRATCH_SIZE must be at least 64 KiB");
  if (slab_size < 256) fail("ROCSHMEM_SLAB_SIZE must be at least 256 bytes");
  if (max_contexts < 1 || max_contexts > ROCSHMEM_CTX_SLOTS)
    fail("ROCSHMEM_MAX_NUM_CONTEXTS must be in [1, 4096]");
  if (max_host_contexts < 1 || max_host_contexts > 4096)
    fail("ROCSHMEM_MAX_NUM_HOST_CONTEXTS must be in [1, 4096]");
  if (max_teams < 1 || max_teams > ROCSHMEM_TEAM_SLOTS)
    fail("ROCSHMEM_MAX_NUM_TEAMS must be in [1, 64]");
  if (wait_timeout_ms == 0 || wait_timeout_ms > 3600000ull)
    fail("ROCSHMEM_WAIT_TIMEOUT_MS must be in [1, 3600000]; waits are always bounded");
  if (proxy_queue_size < 2 || (proxy_queue_size & (proxy_queue_size - 1)) != 0)
    fail("RO_NET_QUEUE_SIZE must be a power of two >= 2");
  if (backend != "auto" && backend != "cuda" && backend != "host")
    fail("ROCSHMEM_BACKEND must be auto, cuda or host");
}

}  // namespace rocshmem
