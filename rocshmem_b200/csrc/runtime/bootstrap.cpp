#include "bootstrap.hpp"

#include <fcntl.h>
#include <poll.h>
#include <sys/socket.h>
#include <sys/stat.h>
#include <sys/un.h>
#include <unistd.h>

#include <chrono>
#include <cstdio>
#include <cstring>
#include <fstream>
#include <random>
#include <sstream>
#include <thread>

namespace rocshmem {

namespace {
using Clock = std::chrono::steady_clock;

std::string hex_encode(const void *data, size_t n) {
  static const char *d = "0123456789abcdef";
  const unsigned char *p = static_cast<const unsigned char *>(data);
  std::string s(n * 2, '0');
  for (size_t i = 0; i < n; ++i) {
    s[2 * i] = d[p[i] >> 4];
    s[2 * i + 1] = d[p[i] & 15];
  }
  return s;
}

void hex_decode(const std::string &s, void *out, size_t n) {
  if (s.size() != 2 * n) throw BootstrapError("bootstrap: payload size mismatch");
  auto val = [](char c) -> int {
    if (c >= '0' && c <= '9') return c - '0';
    if (c >= 'a' && c <= 'f') return c - 'a' + 10;
    throw BootstrapError("bootstrap: bad payload character");
  };
  unsigned char *p = static_cast<unsigned char *>(out);
  for (size_t i = 0; i < n; ++i) p[i] = static_cast<unsigned char>(val(s[2 * i]) * 16 + val(s[2 * i + 1]));
}
}  // namespace

std::string Bootstrap::next_key(const std::string &tag) {
  uint64_t n = seq_[tag]++;
  return tag + "#" + std::to_string(n);
}

// Payloads are hex-encoded so that any store (including ones that treat values as text) carries
// them unchanged.
void Bootstrap::allgather(const std::string &tag, const void *in, void *out, size_t bytes) {
  std::vector<int> all(size_);
  for (int i = 0; i < size_; ++i) all[i] = i;
  allgather_group(tag, all, rank_, in, out, bytes);
}

void Bootstrap::allgather_group(const std::string &tag, const std::vector<int> &members,
                                int my_index, const void *in, void *out, size_t bytes) {
  if (my_index < 0 || my_index >= static_cast<int>(members.size()) || members[my_index] != rank_) {
    throw BootstrapError("bootstrap: caller is not at members[my_index]");
  }
  std::string key = next_key(tag);
  put(key + "/" + std::to_string(rank_), hex_encode(in, bytes));
  char *o = static_cast<char *>(out);
  for (size_t i = 0; i < members.size(); ++i) {
    if (static_cast<int>(i) == my_index) {
      std::memcpy(o + i * bytes, in, bytes);
      continue;
    }
    std::string v = get(key + "/" + std::to_string(members[i]), timeout_ms_);
    hex_decode(v, o + i * bytes, bytes);
  }
}

void Bootstrap::barrier(const std::string &tag) {
  char token = 1;
  std::vector<char> all(size_);
  allgather("barrier:" + tag, &token, all.data(), 1);
}

// ----------------------------------------------------------------------------------------------

void LocalBootstrap::put(const std::string &key, const std::string &value) { kv_[key] = value; }

std::string LocalBootstrap::get(const std::string &key, int) {
  auto it = kv_.find(key);
  if (it == kv_.end()) throw BootstrapError("bootstrap: key '" + key + "' was never set");
  return it->second;
}

// ----------------------------------------------------------------------------------------------

FileBootstrap::FileBootstrap(const std::string &dir, int rank, int size)
    : Bootstrap(rank, size), dir_(dir) {
  if (dir_.empty()) throw BootstrapError("FileBootstrap: empty directory");
  ::mkdir(dir_.c_str(), 0700);  // may already exist
  struct stat st;
  if (::stat(dir_.c_str(), &st) != 0 || !S_ISDIR(st.st_mode)) {
    throw BootstrapError("FileBootstrap: cannot use directory " + dir_);
  }
}

std::string FileBootstrap::path_for(const std::string &key) const {
  std::string name;
  for (char c : key) {
    bool ok = (c >= 'a' && c <= 'z') || (c >= 'A' && c <= 'Z') || (c >= '0' && c <= '9') ||
              c == '.' || c == '-' || c == '_';
    if (ok) {
      name.push_back(c);
    } else {
      char buf[8];
      std::snprintf(buf, sizeof(buf), "%%%02x", static_cast<unsigned char>(c));
      name += buf;
    }
  }
  return dir_ + "/" + name;
}

void FileBootstrap::put(const std::string &key, const std::string &value) {
  std::string final_path = path_for(key);
  std::string tmp = final_path + ".tmp." + std::to_string(::getpid());
  {
    std::ofstream f(tmp, std::ios::binary | std::ios::trunc);
    if (!f) throw BootstrapError("FileBootstrap: cannot write " + tmp);
    f.write(value.data(), static_cast<std::streamsize>(value.size()));
  }
  if (::rename(tmp.c_str(), final_path.c_str()) != 0) {
    throw BootstrapError("FileBootstrap: rename failed for " + final_path);
  }
}

std::string FileBootstrap::get(const std::string &key, int timeout_ms) {
  std::string path = path_for(key);
  auto deadline = Clock::now() + std::chrono::milliseconds(timeout_ms);
  int sleep_us = 50;
  for (;;) {
    std::ifstream f(path, std::ios::binary);
    if (f) {
      std::stringstream ss;
      ss << f.rdbuf();
      return ss.str();
    }
    if (Clock::now() > deadline) {
      throw BootstrapError("bootstrap: timed out after " + std::to_string(timeout_ms) +
                           " ms waiting for key '" + key + "' (a rank did not join?)");
    }
    std::this_thread::sleep_for(std::chrono::microseconds(sleep_us));
    if (sleep_us < 2000) sleep_us *= 2;
  }
}

// ----------------------------------------------------------------------------------------------
// File-descriptor exchange over abstract Unix datagram sockets.
// ----------------------------------------------------------------------------------------------

namespace {

socklen_t abstract_addr(const std::string &name, sockaddr_un *addr) {
  std::memset(addr, 0, sizeof(*addr));
  addr->sun_family = AF_UNIX;
  // sun_path[0] == 0 selects the abstract namespace; the name needs no file system entry.
  size_t n = name.size();
  if (n > sizeof(addr->sun_path) - 2) n = sizeof(addr->sun_path) - 2;
  std::memcpy(addr->sun_path + 1, name.data(), n);
  return static_cast<socklen_t>(offsetof(sockaddr_un, sun_path) + 1 + n);
}

// Returns false when the destination's queue is full (caller drains its own queue and retries).
bool send_fd(int sock, const sockaddr_un &to, socklen_t to_len, int src_rank, int fd) {
  msghdr msg;
  std::memset(&msg, 0, sizeof(msg));
  iovec iov;
  iov.iov_base = &src_rank;
  iov.iov_len = sizeof(src_rank);
  msg.msg_iov = &iov;
  msg.msg_iovlen = 1;
  msg.msg_name = const_cast<sockaddr_un *>(&to);
  msg.msg_namelen = to_len;
  alignas(cmsghdr) char ctrl[CMSG_SPACE(sizeof(int))];
  std::memset(ctrl, 0, sizeof(ctrl));
  msg.msg_control = ctrl;
  msg.msg_controllen = sizeof(ctrl);
  cmsghdr *c = CMSG_FIRSTHDR(&msg);
  c->cmsg_level = SOL_SOCKET;
  c->cmsg_type = SCM_RIGHTS;
  c->cmsg_len = CMSG_LEN(sizeof(int));
  std::memcpy(CMSG_DATA(c), &fd, sizeof(int));
  ssize_t r = ::sendmsg(sock, &msg, MSG_DONTWAIT);
  if (r == static_cast<ssize_t>(sizeof(src_rank))) return true;
  if (r < 0 && (errno == EINTR || errno == EAGAIN || errno == EWOULDBLOCK || errno == ENOBUFS)) {
    return false;
  }
  throw BootstrapError(std::string("exchange_fds: sendmsg failed: ") + std::strerror(errno));
}

bool recv_fd(int sock, int timeout_ms, int *src_rank, int *fd) {
  pollfd p;
  p.fd = sock;
  p.events = POLLIN;
  int pr = ::poll(&p, 1, timeout_ms);
  if (pr <= 0) return false;
  msghdr msg;
  std::memset(&msg, 0, sizeof(msg));
  iovec iov;
  iov.iov_base = src_rank;
  iov.iov_len = sizeof(*src_rank);
  msg.msg_iov = &iov;
  msg.msg_iovlen = 1;
  alignas(cmsghdr) char ctrl[CMSG_SPACE(sizeof(int))];
  msg.msg_control = ctrl;
  msg.msg_controllen = sizeof(ctrl);
  ssize_t r = ::recvmsg(sock, &msg, MSG_CMSG_CLOEXEC);
  if (r != static_cast<ssize_t>(sizeof(*src_rank))) return false;
  cmsghdr *c = CMSG_FIRSTHDR(&msg);
  if (!c || c->cmsg_level != SOL_SOCKET || c->cmsg_type != SCM_RIGHTS) return false;
  std::memcpy(fd, CMSG_DATA(c), sizeof(int));
  return true;
}

}  // namespace

std::vector<int> exchange_fds(Bootstrap &bs, const std::string &tag, int my_fd) {
  const int n = bs.size();
  const int me = bs.rank();
  std::vector<int> fds(n, -1);
  fds[me] = ::dup(my_fd);
  if (fds[me] < 0) throw BootstrapError("exchange_fds: dup failed");
  if (n == 1) return fds;

  // A job-unique socket-name prefix chosen by rank 0.
  uint64_t job[2] = {0, 0};
  if (me == 0) {
    std::random_device rd;
    job[0] = (static_cast<uint64_t>(rd()) << 32) ^ rd();
    job[1] = static_cast<uint64_t>(::getpid());
  }
  std::vector<uint64_t> jobs(2 * n);
  bs.allgather("fdx-job:" + tag, job, jobs.data(), sizeof(job));
  char prefix[96];
  std::snprintf(prefix, sizeof(prefix), "rocshmem_b200.%016llx.%llu.",
                static_cast<unsigned long long>(jobs[0]), static_cast<unsigned long long>(jobs[1]));

  int sock = ::socket(AF_UNIX, SOCK_DGRAM | SOCK_CLOEXEC, 0);
  if (sock < 0) throw BootstrapError("exchange_fds: socket() failed");
  sockaddr_un mine;
  socklen_t mine_len = abstract_addr(std::string(prefix) + tag + "." + std::to_string(me), &mine);
  if (::bind(sock, reinterpret_cast<sockaddr *>(&mine), mine_len) != 0) {
    ::close(sock);
    throw BootstrapError(std::string("exchange_fds: bind failed: ") + std::strerror(errno));
  }
  try {
    bs.barrier("fdx-bound:" + tag);  // every socket is bound before anybody sends
    // Sends and receives are interleaved: a datagram queue holds only a few messages, so a rank
    // whose send would block first drains what has already arrived for it.
    int next_send = 1, got = 0;
    auto deadline = Clock::now() + std::chrono::milliseconds(bs.timeout_ms());
    while (next_send < n || got < n - 1) {
      bool progressed = false;
      if (next_send < n) {
        int peer = (me + next_send) % n;
        sockaddr_un to;
        socklen_t to_len =
            abstract_addr(std::string(prefix) + tag + "." + std::to_string(peer), &to);
        if (send_fd(sock, to, to_len, me, my_fd)) {
          ++next_send;
          progressed = true;
        }
      }
      if (got < n - 1) {
        int src = -1, fd = -1;
        if (recv_fd(sock, next_send < n ? 0 : 50, &src, &fd)) {
          if (src < 0 || src >= n || fds[src] != -1) {
            if (fd >= 0) ::close(fd);
            throw BootstrapError("exchange_fds: unexpected sender");
          }
          fds[src] = fd;
          ++got;
          progressed = true;
        }
      }
      if (!progressed) {
        if (Clock::now() > deadline) {
          throw BootstrapError("exchange_fds: timed out waiting for a peer's descriptor");
        }
        std::this_thread::sleep_for(std::chrono::microseconds(200));
      }
    }
    bs.barrier("fdx-done:" + tag);
  } catch (...) {
    ::close(sock);
    for (int f : fds)
      if (f >= 0) ::close(f);
    throw;
  }
  ::close(sock);
  return fds;
}

int broadcast_fd_group(Bootstrap &bs, const std::string &tag, const std::vector<int> &members, int my_index,
                       int root_fd) {
  const int n = static_cast<int>(members.size());
  if (my_index == 0 && n == 1) return ::dup(root_fd);
  // Socket names start with a random word chosen by the sender, so two jobs on one host cannot meet.
  uint64_t job[2] = {0, 0};
  if (my_index == 0) {
    std::random_device rd;
    job[0] = (static_cast<uint64_t>(rd()) << 32) ^ rd();
    job[1] = static_cast<uint64_t>(::getpid());
  }
  std::vector<uint64_t> jobs(2 * size_t(n));
  bs.allgather_group("fdg-job:" + tag, members, my_index, job, jobs.data(), sizeof(job));
  char prefix[96];
  std::snprintf(prefix, sizeof(prefix), "rocshmem_b200.g.%016llx.%llu.", static_cast<unsigned long long>(jobs[0]),
                static_cast<unsigned long long>(jobs[1]));
  int sock = ::socket(AF_UNIX, SOCK_DGRAM | SOCK_CLOEXEC, 0);
  if (sock < 0) throw BootstrapError("broadcast_fd_group: socket() failed");
  int result = -1;
  try {
    sockaddr_un mine;
    socklen_t mine_len = abstract_addr(std::string(prefix) + std::to_string(my_index), &mine);
    if (::bind(sock, reinterpret_cast<sockaddr *>(&mine), mine_len) != 0) {
      throw BootstrapError(std::string("broadcast_fd_group: bind failed: ") + std::strerror(errno));
    }
    char one = 1;
    std::vector<char> all(static_cast<size_t>(n));
    bs.allgather_group("fdg-bound:" + tag, members, my_index, &one, all.data(), 1);  // receivers are bound
    auto deadline = Clock::now() + std::chrono::milliseconds(bs.timeout_ms());
    if (my_index == 0) {
      for (int i = 1; i < n; ++i) {
        sockaddr_un to;
        socklen_t to_len = abstract_addr(std::string(prefix) + std::to_string(i), &to);
        while (!send_fd(sock, to, to_len, 0, root_fd)) {
          if (Clock::now() > deadline) throw BootstrapError("broadcast_fd_group: timed out sending a descriptor");
          std::this_thread::sleep_for(std::chrono::microseconds(200));
        }
      }
      result = ::dup(root_fd);
      if (result < 0) throw BootstrapError("broadcast_fd_group: dup failed");
    } else {
      int src = -1;
      while (!recv_fd(sock, 50, &src, &result)) {
        if (Clock::now() > deadline) throw BootstrapError("broadcast_fd_group: timed out waiting for the descriptor");
      }
      if (src != 0) {
        if (result >= 0) ::close(result);
        result = -1;
        throw BootstrapError("broadcast_fd_group: unexpected sender");
      }
    }
  } catch (...) {
    ::close(sock);
    throw;
  }
  ::close(sock);
  return result;
}

}  // namespace rocshmem
