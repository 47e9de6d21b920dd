// Bootstrap: the out-of-band channel used while the runtime is being set up (exchange of heap
// handles, team-slot agreement, host barriers on the CPU backend).
//
// The reference uses MPI for all of this (rank/size, MPI_Allgather of IPC handles,
// MPI_Allreduce(BAND) for team slots, MPI_Barrier: src/ipc_policy.cpp:39-75,
// src/ipc/backend_ipc.cpp:167-233). Here the channel is a key-value store with blocking reads:
//   * CallbackBootstrap forwards to a torch.distributed store (TCPStore / FileStore / the store of
//     the default process group) supplied from Python;
//   * FileBootstrap is a native rendezvous through a directory for C++-only programs on one node;
//   * LocalBootstrap serves a single process.
// allgather / barrier / group variants are built on put/get in this file, and file descriptors
// (POSIX handles of cuMemCreate allocations, memfds of the CPU backend) travel between the processes
// over abstract-namespace Unix datagram sockets with SCM_RIGHTS.
//
// Every blocking read has a time-out and throws BootstrapError when it expires: a rank that never
// joins, or exits early, is reported on the host instead of hanging its peers.
#pragma once

#include <cstddef>
#include <cstdint>
#include <functional>
#include <map>
#include <mutex>
#include <stdexcept>
#include <string>
#include <vector>

namespace rocshmem {

class BootstrapError : public std::runtime_error {
 public:
  using std::runtime_error::runtime_error;
};

class Bootstrap {
 public:
  Bootstrap(int rank, int size) : rank_(rank), size_(size) {}
  virtual ~Bootstrap() = default;
  int rank() const { return rank_; }
  int size() const { return size_; }

  virtual void put(const std::string &key, const std::string &value) = 0;
  // Blocks until the key exists; throws BootstrapError after timeout_ms.
  virtual std::string get(const std::string &key, int timeout_ms) = 0;

  // Collectives over all ranks. `tag` must be used in the same order by every rank; an internal
  // per-tag sequence number makes repeated use safe.
  void allgather(const std::string &tag, const void *in, void *out, size_t bytes);
  void barrier(const std::string &tag);
  // Collectives over a subset (world ranks, identical order on every member). `my_index` is the
  // caller's position in `members`.
  void allgather_group(const std::string &tag, const std::vector<int> &members, int my_index,
                       const void *in, void *out, size_t bytes);

  int timeout_ms() const { return timeout_ms_; }
  void set_timeout_ms(int ms) { timeout_ms_ = ms; }

 protected:
  std::string next_key(const std::string &tag);
  int rank_;
  int size_;
  int timeout_ms_ = 120000;
  std::map<std::string, uint64_t> seq_;
};

class LocalBootstrap : public Bootstrap {
 public:
  LocalBootstrap() : Bootstrap(0, 1) {}
  void put(const std::string &key, const std::string &value) override;
  std::string get(const std::string &key, int timeout_ms) override;

 private:
  std::map<std::string, std::string> kv_;
};

// Rendezvous through files in a directory shared by the ranks of one node (for example under
// /dev/shm). put = write to a temporary name and rename; get = poll until the file exists.
class FileBootstrap : public Bootstrap {
 public:
  FileBootstrap(const std::string &dir, int rank, int size);
  void put(const std::string &key, const std::string &value) override;
  std::string get(const std::string &key, int timeout_ms) override;

 private:
  std::string path_for(const std::string &key) const;
  std::string dir_;
};

// Forwards to callables, e.g. the set/get of a torch.distributed store.
class CallbackBootstrap : public Bootstrap {
 public:
  using PutFn = std::function<void(const std::string &, const std::string &)>;
  using GetFn = std::function<std::string(const std::string &, int)>;
  CallbackBootstrap(int rank, int size, PutFn put, GetFn get)
      : Bootstrap(rank, size), put_(std::move(put)), get_(std::move(get)) {}
  void put(const std::string &key, const std::string &value) override { put_(key, value); }
  std::string get(const std::string &key, int timeout_ms) override { return get_(key, timeout_ms); }

 private:
  PutFn put_;
  GetFn get_;
};

// All-to-all exchange of one file descriptor per rank. Returns, for every rank r, a descriptor that
// refers to the same open file description as r's `my_fd` (the entry for the caller is a dup of
// my_fd). The caller owns and closes the returned descriptors.
std::vector<int> exchange_fds(Bootstrap &bs, const std::string &tag, int my_fd);

// One descriptor from the first process of `members` (world ranks, the same order on every member) to all the
// others. Collective over the members; `tag` must be unique per call. Returns a descriptor the caller owns: on
// the sender a dup of `root_fd`, elsewhere the received one. Throws BootstrapError on a time-out.
int broadcast_fd_group(Bootstrap &bs, const std::string &tag, const std::vector<int> &members, int my_index,
                       int root_fd);

}  // namespace rocshmem
