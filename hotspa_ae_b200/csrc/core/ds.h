// Distributed-states (DS) algebra: how one tensor is laid out over a group of devices under one
// parallel strategy.
//
// A DS over `device_num` devices is a map  dim -> count  where dim >= 0 names a tensor dimension
// that is split `count` ways, dim == -1 is the number of duplicates and dim == -2 the number of
// partial (to-be-summed) copies.  `order` lists the dims whose count is > 1 from the slowest to
// the fastest varying digit of the device index (a mixed-radix number).
//
// Behavioural parity target: hetu/graph/distributed_states.{h,cc} of the reference
// (set_states / set_order / combine_states / combine_order / check_* / map_device_to_state_index /
// get_dup_group_index / get_devices_by_dim), and the comm-type table of
// hetu/graph/ops/Communication.cc:81-216.  This is an independent implementation.
#pragma once
#include <cstdint>
#include <map>
#include <string>
#include <utility>
#include <vector>

namespace hsb {

constexpr int kDup = -1;
constexpr int kPartial = -2;
constexpr int kNoHeteroDim = -3;

using StateMap = std::map<int, int>;

class DistributedStates {
 public:
  DistributedStates() = default;
  DistributedStates(int device_num, const StateMap& states, const std::vector<int>& order = {}, bool zero = false);

  int device_num() const { return device_num_; }
  const StateMap& states() const { return states_; }
  const std::vector<int>& order() const { return order_; }
  bool zero() const { return zero_; }
  void set_zero(bool z) { zero_ = z; }

  bool is_none() const { return device_num_ < 0; }
  bool is_valid() const;
  int get_dim(int dim) const;                       // count for `dim`, 1 when absent
  bool is_pure_duplicate() const { return device_num_ == get_dim(kDup); }
  bool check_equal(const DistributedStates& o) const;
  bool check_max_dim(int max_dim) const;

  // digit of every ordered dim for device `index` (position inside the placement group)
  StateMap map_device_to_state_index(int index) const;
  // mixed-radix index over the split (>= 0) dims only: dp rank for data, shard id for weights
  int get_dup_group_index(int index) const;
  // positions (into `group`) of the devices that differ from `index` only in the digit of `dim`
  std::vector<int> get_devices_by_dim(int dim, int index, const std::vector<int>& group) const;
  std::vector<int> get_loop_sizes() const;

  // merge the device digits of `src` dims into `dst` (used by the pattern checks below)
  static StateMap combine_states(const std::vector<int>& src, int dst, const StateMap& states);
  static std::vector<int> combine_order(const std::vector<int>& src, int dst, const std::vector<int>& order,
                                        bool* ok);
  bool check_combine(const DistributedStates& dst, const std::vector<int>& src_dims, int dst_dim) const;
  bool check_reduce_dim(const DistributedStates& dst, int dim) const;

  bool check_allreduce(const DistributedStates& dst) const;      // {-2} -> -1
  bool check_allgather(const DistributedStates& dst) const;      // split0 -> dup (inverse of scatter)
  bool check_reducescatter(const DistributedStates& dst) const;  // {-2} -> 0
  bool check_scatter(const DistributedStates& dst) const;        // {-1} -> 0
  bool check_broadcast(const DistributedStates& dst) const;
  bool check_reduce(const DistributedStates& dst) const;

  // local shard of a global shape on device `index`: per-dim (offset, size)
  std::vector<std::pair<int64_t, int64_t>> local_slice(const std::vector<int64_t>& global_shape, int index) const;
  std::vector<int64_t> local_shape(const std::vector<int64_t>& global_shape) const;

  std::string info() const;

 private:
  int device_num_ = -1;
  StateMap states_;
  std::vector<int> order_;
  bool zero_ = false;
};

// A list of DS, one per member of a heterogeneous replica set (size 1 = homogeneous).
class DistributedStatesUnion {
 public:
  DistributedStatesUnion() = default;
  DistributedStatesUnion(std::vector<DistributedStates> list, int hetero_dim = kNoHeteroDim)
      : list_(std::move(list)), hetero_dim_(hetero_dim) {}
  size_t size() const { return list_.size(); }
  bool is_hetero() const { return hetero_dim_ != kNoHeteroDim; }
  int hetero_dim() const { return hetero_dim_; }
  const std::vector<DistributedStates>& ds_list() const { return list_; }
  const DistributedStates& get(size_t i) const;
  // DS seen by the devices of member i: the hetero dim's count divided by the union size
  DistributedStates get_local(size_t i) const;
  bool check_equal(const DistributedStatesUnion& o) const;
  void add(const DistributedStates& ds) { list_.push_back(ds); }
  std::string info() const;

 private:
  std::vector<DistributedStates> list_;
  int hetero_dim_ = kNoHeteroDim;
};

enum CommType : uint32_t {
  COMM_UNUSED = 0,
  COMM_P2P = 1u << 0,
  COMM_SPLIT = 1u << 1,            // dup -> split: local slice, no traffic
  COMM_ALL_REDUCE = 1u << 2,
  COMM_ALL_GATHER = 1u << 3,
  COMM_REDUCE_SCATTER = 1u << 4,
  COMM_SCATTER = 1u << 5,
  COMM_BATCHED_SEND_RECV = 1u << 6,  // general repartition between different groups / layouts
  COMM_SPLIT_ALL_REDUCE = 1u << 7,   // heterogeneous variants
  COMM_SPLIT_REDUCE_SCATTER = 1u << 8,
  COMM_SPLIT_ALL_GATHER = 1u << 9,
  COMM_UNSUPPORTED = 1u << 31,
};

// Classify the resharding src -> dst for one union member.
uint32_t classify_comm(const DistributedStatesUnion& src, const std::vector<int>& src_group,
                       const DistributedStatesUnion& dst, const std::vector<int>& dst_group, size_t member = 0);
const char* comm_type_name(uint32_t t);

// Communication groups of the heterogeneous ("split") collectives for one rank.
// Member j of the union lives on ranks `groups[j]` with layout `local_ds[j]`; all members split the tensor on the same
// single dimension (possibly with different counts) and may duplicate it.  The tensor is cut into F = max split count
// micro-blocks; this rank holds `micro_blocks` consecutive ones, and for each of them `groups[i]` lists the rank groups
// (one holder per member, duplicates paired round-robin) this rank takes part in.
// Reference behaviour: hetu/graph/ops/Communication.cc:248-392.
struct SplitCommPlan {
  int split_dim = 0;
  int micro_blocks = 1;
  int first_micro_block = 0;
  std::vector<std::vector<std::vector<int>>> groups;
};
SplitCommPlan split_comm_groups(const std::vector<DistributedStates>& local_ds,
                                const std::vector<std::vector<int>>& groups, int rank);

// DS of `linear(a, b)` given the operand layouts (2-D, after resolving transposes):
// a is [m, k] with states {0: a_row, 1: a_col}, b is [k, n] with {0: b_row, 1: b_col}; needs a_col == b_row.
DistributedStates deduce_linear(const DistributedStates& a, const DistributedStates& b, bool trans_a, bool trans_b);

}  // namespace hsb
