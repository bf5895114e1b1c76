// Host-side planners: hot-switch reshard plans, pipeline schedules, sequence bucketing/packing,
// flat-arena layout.  Pure C++ (no CUDA) so they can be unit-tested anywhere.
//
// Reference counterparts (behaviour, not code): hetu/graph/switch_exec_graph.cc (ParamBlock /
// ParamSlice grid, sender-selection algorithms :388-566), hetu/graph/executable_graph.cc:934-1010
// (GPipe and pipedream-flush schedules), hotspa/llama_hot_switch.py:134-208 (bucket + first-fit).
#pragma once
#include <cstdint>
#include <string>
#include <vector>

#include "ds.h"

namespace hsb {

// One rectangular piece of one tensor that device `dst_rank` needs and device `src_rank` holds.
// Offsets are element offsets inside the *local shard* of the tensor on that device; rows are
// `src_ld` / `dst_ld` elements apart.  The executor adds the tensor's arena base on each side.
struct CopyDesc {
  int32_t tensor_id;
  int32_t src_rank;
  int32_t dst_rank;
  int64_t src_off;
  int64_t dst_off;
  int64_t rows;
  int64_t row_elems;
  int64_t src_ld;
  int64_t dst_ld;
};

enum SenderPolicy : int {
  SENDER_FCFS = 0,          // first owner in group order
  SENDER_ROUND_ROBIN = 1,   // rotate among owners per slice
  SENDER_GREEDY = 2,        // owner with the fewest bytes sent so far
  SENDER_BALANCED = 3,      // default: prefer local, then min(max(sent)), tie -> fewest distinct peers
};

struct TensorLayout {
  std::vector<int64_t> shape;   // global shape (1-D or 2-D; higher dims must be unsplit and are folded)
  DistributedStates ds;
  std::vector<int> group;       // global ranks, position = device index inside the DS
};

struct ReshardStats {
  std::vector<int64_t> sent_elems;   // per global rank
  std::vector<int64_t> recv_elems;
  int64_t local_elems = 0;
  int64_t remote_elems = 0;
};

// Explicit placement of one local shard: device `rank` stores the rectangle [r0, r1) x [c0, c1) of the
// (folded 2-D) global tensor, row-major with leading dimension c1 - c0.
struct Region { int rank; int64_t r0, r1, c0, c1; };

// Regions of a DS layout; `replica` >= 0 keeps, for every distinct shard, only the holder with that
// duplicate digit (modulo the duplicate count) so each shard appears exactly once.
std::vector<Region> regions_of(const TensorLayout& t, int replica = -1);

class ReshardPlanner {
 public:
  explicit ReshardPlanner(int world_size, int policy = SENDER_BALANCED);
  // General form: every dst region is assembled from the src regions that cover it.  With
  // `gather_all_owners` every owner of a cell contributes a descriptor (the executor sums them:
  // used for gradients whose replicas hold different partial sums); otherwise one owner is chosen.
  void add_tensor_regions(int tensor_id, const std::vector<Region>& src, const std::vector<Region>& dst,
                          bool gather_all_owners = false);
  // Adds the copies that realise src -> dst for one tensor.  Throws when a needed slice has no owner
  // or when partial (-2) states are involved (partial tensors must be reduced before a switch).
  void add_tensor(int tensor_id, const TensorLayout& src, const TensorLayout& dst);
  const std::vector<CopyDesc>& copies() const { return copies_; }
  std::vector<CopyDesc> copies_for_dst(int rank) const;
  std::vector<CopyDesc> copies_for_src(int rank) const;
  const ReshardStats& stats() const { return stats_; }

 private:
  int world_;
  int policy_;
  int rr_ = 0;
  std::vector<CopyDesc> copies_;
  ReshardStats stats_;
};

// Pipeline schedules.  A task is (is_forward, micro_batch).
struct PipeTask { bool forward; int micro_batch; };
std::vector<PipeTask> schedule_1f1b(int num_stages, int stage, int num_micro_batches);
std::vector<PipeTask> schedule_gpipe(int num_stages, int stage, int num_micro_batches);

// Bucketing + first-fit packing of variable-length sequences.
// bucket_bounds is descending, e.g. {32768, 16384, 4096, 0}: bucket i holds lengths in
// (bounds[i+1] + shift, bounds[i] + shift] and packs rows of capacity bounds[i] + shift (shift = 1
// when a row of n+1 tokens yields n input/label pairs).  Returns, per bucket, the packed rows
// (lists of sequence indices).
struct PackedBucket {
  int64_t max_len;
  int64_t min_len;
  std::vector<int> members;                 // sequence indices, longest first
  std::vector<std::vector<int>> rows;       // first-fit rows, each sums to <= max_len
};
std::vector<PackedBucket> bucket_and_pack(const std::vector<int64_t>& lengths,
                                          const std::vector<int64_t>& bucket_bounds, int64_t shift,
                                          bool drop_short);
// Split packed rows over dp ranks balancing tokens (longest-processing-time first).
std::vector<std::vector<int>> balance_rows(const std::vector<int64_t>& row_tokens, int dp);

// Descriptor table of the reshard kernel (csrc/runtime/symm.cu: reshard_kernel).
// Input: one rectangle per planned copy as addresses in this process (peer mappings resolved), in bytes.
// Output: the rectangles cut into work units of about `unit_bytes` (single-row rectangles by bytes, multi-row ones
// by rows, one descriptor per unit so that units can be interleaved), ordered round-robin over the source ranks
// starting with rank + 1, so that at any moment the ranks of a node pull from different peers.
//   descs     [n, 6] = src, dst, rows, row_bytes, src_ld_bytes, dst_ld_bytes   (ld = 0 for single-row units)
//   unit_rows [n]      rows per unit of the descriptor
//   prefix    [n + 1]  first unit index of every descriptor
struct RectBytes { int64_t src, dst, rows, row_bytes, src_ld, dst_ld; int src_rank; };
struct DescTable {
  std::vector<int64_t> descs;
  std::vector<int32_t> unit_rows, prefix;
};
DescTable build_reshard_descriptors(const std::vector<RectBytes>& rects, int64_t unit_bytes, int rank, int world);

// Flat arena: assigns aligned offsets to tensors in order; returns total size.
int64_t plan_arena(const std::vector<int64_t>& numels, int64_t align_elems, std::vector<int64_t>* offsets);

}  // namespace hsb
