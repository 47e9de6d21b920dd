#include "allocator.hpp"

#include <stdexcept>

namespace rocshmem {

size_t Pow2Allocator::round_up_pow2(size_t v) {
  if (v <= 1) return 1;
  if (v > (size_t(1) << 63)) return 0;  // would overflow
  size_t p = 1;
  while (p < v) p <<= 1;
  return p;
}

Pow2Allocator::Pow2Allocator(size_t size, size_t alignment) : size_(size), alignment_(alignment) {
  if (alignment == 0 || (alignment & (alignment - 1)) != 0) {
    throw std::invalid_argument("Pow2Allocator: alignment must be a power of two");
  }
  // Chop [0, size) greedily into the largest power-of-two chunks, largest first. Every chunk
  // starts at a multiple of the alignment because all earlier chunks are multiples of it.
  size_t offset = 0;
  size_t remaining = size;
  while (remaining >= alignment_) {
    size_t chunk = size_t(1) << 63;
    while (chunk > remaining) chunk >>= 1;
    bins_[chunk][offset] = FreeBlock{offset, chunk};
    offset += chunk;
    remaining -= chunk;
    managed_ += chunk;
  }
}

size_t Pow2Allocator::alloc(size_t bytes) {
  if (bytes == 0) return kNull;
  size_t want = round_up_pow2(bytes);
  if (want == 0) return kNull;
  if (want < alignment_) want = alignment_;
  // Smallest non-empty bin that can serve the request.
  auto bin = bins_.lower_bound(want);
  while (bin != bins_.end() && bin->second.empty()) ++bin;
  if (bin == bins_.end()) return kNull;

  size_t have = bin->first;
  auto first = bin->second.begin();
  size_t offset = first->first;
  FreeBlock origin = first->second;
  bin->second.erase(first);
  // Split down: keep the low half, return the high half to its bin.
  while (have > want) {
    have >>= 1;
    bins_[have][offset + have] = origin;
  }
  live_[offset] = Live{want, origin.chunk_base, origin.chunk_size};
  used_ += want;
  return offset;
}

bool Pow2Allocator::free(size_t offset) {
  auto it = live_.find(offset);
  if (it == live_.end()) return false;
  Live rec = it->second;
  live_.erase(it);
  used_ -= rec.size;

  size_t size = rec.size;
  size_t off = offset;
  // Merge with the buddy while it is free, never beyond the top-level chunk.
  while (size < rec.chunk_size) {
    size_t rel = off - rec.chunk_base;
    size_t buddy = rec.chunk_base + (rel ^ size);
    auto bin = bins_.find(size);
    if (bin == bins_.end()) break;
    auto b = bin->second.find(buddy);
    if (b == bin->second.end()) break;
    bin->second.erase(b);
    if (buddy < off) off = buddy;
    size <<= 1;
  }
  bins_[size][off] = FreeBlock{rec.chunk_base, rec.chunk_size};
  return true;
}

size_t Pow2Allocator::block_size(size_t offset) const {
  auto it = live_.find(offset);
  return it == live_.end() ? 0 : it->second.size;
}

size_t Pow2Allocator::largest_free_block() const {
  for (auto it = bins_.rbegin(); it != bins_.rend(); ++it) {
    if (!it->second.empty()) return it->first;
  }
  return 0;
}

size_t Pow2Allocator::bin_population(size_t block) const {
  auto it = bins_.find(block);
  return it == bins_.end() ? 0 : it->second.size();
}

}  // namespace rocshmem
