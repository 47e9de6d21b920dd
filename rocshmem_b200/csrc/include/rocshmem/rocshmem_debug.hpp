// Queue inspection for debugging (reference: include/rocshmem/rocshmem_debug.hpp:28-30, which dumps one send- or
// completion-queue entry of the NIC backend). The only queue here is the reverse-offload command ring, one per
// process: a command slot plays the role of a send-queue entry and its completion words that of a completion-queue
// entry. All functions print to stderr from the host and read the ring without taking part in its protocol.
#pragma once

namespace rocshmem {

// Prints `count` command slots starting at `first` (indices wrap around the ring): state, operation, PE, addresses,
// size, completion slot. Prints one line that says so when the process runs no proxy thread.
void debug_print_ring(int first, int count);

// Reference-compatible spellings. There is one ring per process, so the destination PE and the block only label the
// output; `index_wqe` selects the command slot, `cqe_index` the completion slot.
void debug_print_sq(int dest_pe, int src_wg, int index_wqe);
void debug_print_cq(int dest_pe, int src_wg, int cqe_index);

}  // namespace rocshmem
