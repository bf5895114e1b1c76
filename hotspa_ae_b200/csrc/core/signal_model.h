// Host model of the cross-GPU flag protocols: the same epoch / counter-set / double-buffer rules the kernels
// follow (csrc/runtime/symm.cu: symm_barrier_kernel; csrc/kernels/gemm_fused_comm.cu: ready flags of the
// all-gather mode, arrival counters of the reduce-scatter mode), run by CPU threads over std::atomic words
// with randomised delays.  Every wait is bounded; every read of "remote" data checks the tag the protocol
// promises.  It exists because these protocols cannot be raced on purpose on a shared GPU: a rule change
// (number of counter sets, number of staging buffers, who clears what and when) is tried here first.
// The parameters that the kernels fix (3 counter sets, 2 receive / staging buffers) are arguments so that the
// tests can show the model catching the broken variants.
#pragma once
#include <cstdint>

namespace hsb {

struct ModelResult {
  long checks = 0;       // tag / count comparisons made
  long violations = 0;   // comparisons that failed
  long timeouts = 0;     // bounded waits that gave up
};

// n ranks run `calls` barriers on one slot; epochs start at `first_epoch` and wrap.  A rank that leaves
// barrier k must observe that every rank entered barrier k.
ModelResult run_barrier_model(int n, int calls, uint32_t first_epoch, uint64_t seed);

// GEMM -> reduce-scatter arrivals: call e uses counter set e % counter_sets and receive buffer
// e % recv_buffers; at the start of call e a rank clears set (e + 2) % counter_sets of its own pad.
ModelResult run_reduce_scatter_model(int n, int calls, int counter_sets, int recv_buffers, int row_blocks,
                                     int parts, uint64_t seed);

// all-gather -> GEMM: call e stages into buffer e % stage_buffers, then publishes epoch e + 1 to every peer;
// a consumer waits for a peer's epoch before it pulls that peer's staged chunks.
ModelResult run_all_gather_model(int n, int calls, int stage_buffers, int chunks, uint64_t seed);

}  // namespace hsb
