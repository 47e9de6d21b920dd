#include "team.hpp"

namespace rocshmem {

SplitPlan plan_split(const TeamTriplet &parent_world, int parent_size, int world_size, int start,
                     int stride, int size) {
  SplitPlan plan;
  if (start < 0 || start >= parent_size || size < 1 || size > parent_size || stride < 1) {
    return plan;
  }
  TeamTriplet w;
  w.pe_start = parent_world.pe_in_world(start);
  w.stride = stride * parent_world.stride;
  w.size = size;
  // The reference compares the last member against num_pes with '>' and so admits a member equal
  // to num_pes (src/rocshmem.cpp:256-259); a PE index must be strictly below the world size.
  if (w.last_pe() >= world_size) return plan;
  // Every member must also be a member of the parent.
  TeamTriplet parent = parent_world;
  parent.size = parent_size;
  if (parent.pe_in_team(w.last_pe()) < 0) return plan;
  plan.ok = true;
  plan.world = w;
  return plan;
}

int translate_pe(const TeamTriplet &src, int src_pe, const TeamTriplet &dst) {
  if (src_pe < 0 || src_pe >= src.size) return -1;
  return dst.pe_in_team(src.pe_in_world(src_pe));
}

TeamSlots::TeamSlots(int max_teams) : max_(max_teams) {
  mask_ = (max_teams >= 64) ? ~uint64_t(0) : ((uint64_t(1) << max_teams) - 1);
}

int TeamSlots::lowest_common(const std::vector<uint64_t> &masks) {
  uint64_t all = ~uint64_t(0);
  for (uint64_t m : masks) all &= m;
  if (all == 0) return -1;
  return __builtin_ctzll(all);
}

bool TeamSlots::take(int slot) {
  if (slot < 0 || slot >= max_) return false;
  uint64_t bit = uint64_t(1) << slot;
  if (!(mask_ & bit)) return false;
  mask_ &= ~bit;
  return true;
}

void TeamSlots::release(int slot) {
  if (slot < 0 || slot >= max_) return;
  mask_ |= uint64_t(1) << slot;
}

int TeamSlots::in_use() const {
  uint64_t full = (max_ >= 64) ? ~uint64_t(0) : ((uint64_t(1) << max_) - 1);
  return __builtin_popcountll(full & ~mask_);
}

}  // namespace rocshmem
