// Team arithmetic: strided PE sets, world <-> team numbering, split validation, slot bitmask.
//
// Behaviour follows the reference's Team/TeamInfo (src/team.hpp:39-158, src/team.cpp:51-111) and the
// validation in rocshmem_team_split_strided (src/rocshmem.cpp:221-303). Pure host code; the device
// mirror of the result is rocshmem_team_dev.
#pragma once

#include <cstdint>
#include <vector>

namespace rocshmem {

struct TeamTriplet {
  int pe_start = 0;  // world numbering
  int stride = 1;
  int size = 0;

  int pe_in_world(int team_pe) const { return pe_start + stride * team_pe; }
  // Index of a world PE inside the set, -1 when it is not a member.
  int pe_in_team(int world_pe) const {
    if (world_pe < pe_start) return -1;
    int d = world_pe - pe_start;
    if (stride <= 0 || d % stride) return -1;
    int idx = d / stride;
    return idx < size ? idx : -1;
  }
  int last_pe() const { return pe_start + stride * (size - 1); }
};

// Result of validating a split request against the parent team.
struct SplitPlan {
  bool ok = false;      // false: the call returns -1 and creates nothing
  TeamTriplet world;    // the new team in world numbering
};

// (start, stride, size) are in the parent's numbering. The request is rejected when start or size
// fall outside the parent, stride < 1, or the last member would lie beyond the world.
SplitPlan plan_split(const TeamTriplet &parent_world, int parent_size, int world_size, int start,
                     int stride, int size);

// translate `src_pe` (numbering of `src`) into the numbering of `dst`; -1 when not a member of dst
// or src_pe is outside src.
int translate_pe(const TeamTriplet &src, int src_pe, const TeamTriplet &dst);

// Free-slot bookkeeping for the per-team sync pools. Bit i set = slot i free. Slot 0 belongs to
// TEAM_WORLD. All members of a new team AND their masks together and take the lowest common bit
// (reference: src/ipc/backend_ipc.cpp:197-233 does the same with MPI_Allreduce(BAND)).
class TeamSlots {
 public:
  explicit TeamSlots(int max_teams);
  uint64_t mask() const { return mask_; }
  static int lowest_common(const std::vector<uint64_t> &masks);
  bool take(int slot);
  void release(int slot);
  int in_use() const;
  int capacity() const { return max_; }

 private:
  int max_;
  uint64_t mask_;
};

}  // namespace rocshmem
