// Symmetric-heap allocator: power-of-two bins over an offset range.
//
// Behaviour kept from the reference's Pow2Bins/Binner/AddressRecord/Bin classes
// (src/memory/pow2_bins.hpp:90-319, src/memory/binner.hpp:109-231): 128-byte granularity, every
// request rounded up to a power of two, a request is served from the exact bin or by splitting the
// smallest larger block, size 0 and exhaustion return "null", and the heap (which need not be a
// power of two) is chopped greedily into the largest power-of-two chunks that fit. Because the
// algorithm is deterministic, PEs that issue the same call sequence obtain the same offsets with no
// communication, which is what makes rocshmem_malloc symmetric.
//
// Deliberate improvement: the reference never merges freed blocks (AddressRecord::combine is
// unused), so a heap fragments permanently. Here a freed block is merged with its buddy whenever the
// buddy is free too, up to the size of the top-level chunk it was cut from. The lowest-offset block
// of a bin is always handed out first, so determinism is preserved.
//
// The allocator works on offsets, not pointers: it never touches the memory it manages and is
// testable without a GPU.
#pragma once

#include <cstddef>
#include <cstdint>
#include <map>
#include <set>

namespace rocshmem {

class Pow2Allocator {
 public:
  static constexpr size_t kNull = ~size_t(0);

  // Manage [0, size). `alignment` must be a power of two; blocks are multiples of it.
  explicit Pow2Allocator(size_t size, size_t alignment = 128);

  // Offset of a block of at least `bytes` (rounded up to a power of two >= alignment),
  // or kNull when bytes == 0 or nothing fits.
  size_t alloc(size_t bytes);

  // Returns false (and changes nothing) when `offset` is not a live allocation.
  bool free(size_t offset);

  // Size actually reserved for a live allocation, 0 if unknown.
  size_t block_size(size_t offset) const;

  size_t size() const { return size_; }
  size_t alignment() const { return alignment_; }
  size_t used() const { return used_; }
  size_t avail() const { return managed_ - used_; }
  size_t managed() const { return managed_; }  // bytes covered by chunks (size minus tail < alignment)
  size_t live_allocations() const { return live_.size(); }
  // Largest request that could succeed right now.
  size_t largest_free_block() const;
  // Number of free blocks currently held in the bin of exactly `block` bytes.
  size_t bin_population(size_t block) const;

  static size_t round_up_pow2(size_t v);

 private:
  struct Live {
    size_t size;
    size_t chunk_base;
    size_t chunk_size;
  };
  struct FreeBlock {
    size_t chunk_base;
    size_t chunk_size;
  };

  size_t size_;
  size_t alignment_;
  size_t managed_ = 0;
  size_t used_ = 0;
  // bin size -> (offset -> origin chunk), offsets ordered so the lowest is taken first
  std::map<size_t, std::map<size_t, FreeBlock>> bins_;
  std::map<size_t, Live> live_;
};

}  // namespace rocshmem
