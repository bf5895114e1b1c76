#include "ds.h"

#include <algorithm>
#include <sstream>
#include <stdexcept>

namespace hsb {

static void fail(const std::string& msg) { throw std::invalid_argument(msg); }

DistributedStates::DistributedStates(int device_num, const StateMap& states, const std::vector<int>& order, bool zero)
    : device_num_(device_num), zero_(zero) {
  if (device_num < 1) fail("DistributedStates: device_num must be >= 1");
  long prod = 1;
  for (const auto& kv : states) {
    if (kv.first < kPartial) fail("DistributedStates: dims below -2 are not valid");
    if (kv.second < 1) fail("DistributedStates: counts must be >= 1");
    if (kv.second > 1) {
      states_[kv.first] = kv.second;
      prod *= kv.second;
    }
  }
  if (!states_.count(kPartial)) states_[kPartial] = 1;
  if (!states_.count(kDup)) states_[kDup] = 1;
  if (prod != device_num) {
    std::ostringstream os;
    os << "DistributedStates: product of counts (" << prod << ") != device_num (" << device_num << ")";
    fail(os.str());
  }
  if (order.empty()) {
    for (const auto& kv : states_)
      if (kv.second > 1) order_.push_back(kv.first);  // std::map iterates in sorted order
  } else {
    for (const auto& kv : states_)
      if (kv.second > 1 && std::find(order.begin(), order.end(), kv.first) == order.end())
        fail("DistributedStates: order does not mention every dim whose count is > 1");
    for (int o : order) {
      auto it = states_.find(o);
      if (it != states_.end() && it->second > 1) {
        if (std::find(order_.begin(), order_.end(), o) != order_.end()) fail("DistributedStates: duplicate in order");
        order_.push_back(o);
      }
    }
  }
}

bool DistributedStates::is_valid() const {
  return device_num_ == 1 || (device_num_ > 1 && !states_.empty() && !order_.empty());
}

int DistributedStates::get_dim(int dim) const {
  auto it = states_.find(dim);
  return it == states_.end() ? 1 : it->second;
}

bool DistributedStates::check_equal(const DistributedStates& o) const {
  return device_num_ == o.device_num_ && states_ == o.states_ && order_ == o.order_;
}

bool DistributedStates::check_max_dim(int max_dim) const {
  for (const auto& kv : states_)
    if (kv.first >= max_dim) return false;
  return true;
}

StateMap DistributedStates::map_device_to_state_index(int index) const {
  StateMap out;
  for (auto it = order_.rbegin(); it != order_.rend(); ++it) {
    const int n = states_.at(*it);
    out[*it] = index % n;
    index /= n;
  }
  return out;
}

int DistributedStates::get_dup_group_index(int index) const {
  const StateMap digit = map_device_to_state_index(index);
  std::vector<int> dims;
  for (int o : order_)
    if (o >= 0) dims.push_back(o);
  std::sort(dims.begin(), dims.end());
  int idx = 0, radix = 1;
  for (auto it = dims.rbegin(); it != dims.rend(); ++it) {
    idx += digit.at(*it) * radix;
    radix *= get_dim(*it);
  }
  return idx;
}

std::vector<int> DistributedStates::get_devices_by_dim(int dim, int index, const std::vector<int>& group) const {
  auto pos = std::find(order_.begin(), order_.end(), dim);
  int interval = 1;
  if (pos != order_.end())
    for (auto it = pos + 1; it != order_.end(); ++it) interval *= states_.at(*it);
  const int macro = interval * get_dim(dim);
  const int start = index - index % macro + index % interval;
  std::vector<int> out;
  for (int i = start; i < start + macro; i += interval) {
    if (i < 0 || i >= static_cast<int>(group.size())) fail("get_devices_by_dim: group too small");
    out.push_back(group[i]);
  }
  return out;
}

std::vector<int> DistributedStates::get_loop_sizes() const {
  std::vector<int> sizes(order_.size(), 1);
  int acc = 1;
  for (int i = static_cast<int>(order_.size()) - 1; i >= 0; --i) {
    acc *= get_dim(order_[i]);
    sizes[i] = acc;
  }
  return sizes;
}

StateMap DistributedStates::combine_states(const std::vector<int>& src, int dst, const StateMap& in) {
  StateMap st = in;
  long value = 1;
  for (int s : src) {
    if (s == dst) fail("combine_states: src equals dst");
    if (s < 0) {
      value *= st.count(s) ? st[s] : 1;
      st[s] = 1;
    } else {
      auto it = st.find(s);
      if (it != st.end()) {
        value *= it->second;
        st.erase(it);
      }
      // tensor dims above the removed one slide down by one
      StateMap moved;
      for (const auto& kv : st) moved[(kv.first > s) ? kv.first - 1 : kv.first] = kv.second;
      st.swap(moved);
    }
  }
  int d = dst;
  if (d >= 0)
    for (int s : src)
      if (s >= 0 && dst > s) d -= 1;
  if (st.count(d)) st[d] *= static_cast<int>(value);
  else st[d] = static_cast<int>(value);
  // drop non-negative dims that ended up with count 1
  for (auto it = st.begin(); it != st.end();) {
    if (it->first >= 0 && it->second == 1) it = st.erase(it);
    else ++it;
  }
  return st;
}

std::vector<int> DistributedStates::combine_order(const std::vector<int>& src, int dst, const std::vector<int>& in,
                                                  bool* ok) {
  std::vector<int> order = in;
  *ok = true;
  std::vector<int> inds;
  auto collect = [&](int dim) {
    auto it = std::find(order.begin(), order.end(), dim);
    if (it != order.end()) inds.push_back(static_cast<int>(it - order.begin()));
  };
  for (int s : src) collect(s);
  collect(dst);
  std::sort(inds.begin(), inds.end());
  if (!inds.empty()) {
    for (size_t i = 1; i < inds.size(); ++i)
      if (inds[i] != inds[0] + static_cast<int>(i)) { *ok = false; return order; }  // digits must be adjacent
    for (int i = static_cast<int>(inds.size()) - 1; i >= 1; --i) order.erase(order.begin() + inds[i]);
    order[inds[0]] = dst;
    for (auto& o : order)
      if (o > 0)
        for (int s : src)
          if (s >= 0 && o > s) o -= 1;
  }
  return order;
}

bool DistributedStates::check_combine(const DistributedStates& dst, const std::vector<int>& src_dims,
                                      int dst_dim) const {
  bool ok = true;
  const StateMap st = combine_states(src_dims, dst_dim, states_);
  const std::vector<int> od = combine_order(src_dims, dst_dim, order_, &ok);
  if (!ok) return false;
  // compare ignoring count-1 entries of the non-negative dims (never stored) and keeping -1/-2
  StateMap want = dst.states_;
  return st == want && od == dst.order_;
}

bool DistributedStates::check_reduce_dim(const DistributedStates& dst, int dim) const {
  StateMap st = states_;
  if (dim < 0) st[dim] = 1;
  else st.erase(dim);
  std::vector<int> od = order_;
  auto it = std::find(od.begin(), od.end(), dim);
  if (it != od.end()) od.erase(it);
  return st == dst.states_ && od == dst.order_;
}

bool DistributedStates::check_allreduce(const DistributedStates& dst) const {
  return get_dim(kPartial) > 1 && check_combine(dst, {kPartial}, kDup);
}
bool DistributedStates::check_scatter(const DistributedStates& dst) const {
  return get_dim(kDup) > 1 && check_combine(dst, {kDup}, 0);
}
bool DistributedStates::check_allgather(const DistributedStates& dst) const {
  return get_dim(0) > 1 && dst.get_dim(kDup) > 1 && dst.check_combine(*this, {kDup}, 0);
}
bool DistributedStates::check_reducescatter(const DistributedStates& dst) const {
  return get_dim(kPartial) > 1 && check_combine(dst, {kPartial}, 0);
}
bool DistributedStates::check_broadcast(const DistributedStates& dst) const {
  return dst.get_dim(kDup) > 1 && dst.check_reduce_dim(*this, kDup);
}
bool DistributedStates::check_reduce(const DistributedStates& dst) const {
  return get_dim(kPartial) > 1 && check_reduce_dim(dst, kPartial);
}

std::vector<std::pair<int64_t, int64_t>> DistributedStates::local_slice(const std::vector<int64_t>& shape,
                                                                        int index) const {
  const StateMap digit = map_device_to_state_index(index);
  std::vector<std::pair<int64_t, int64_t>> out;
  for (size_t d = 0; d < shape.size(); ++d) {
    const int n = get_dim(static_cast<int>(d));
    if (shape[d] % n != 0) fail("local_slice: dimension not divisible by its split count");
    const int64_t sz = shape[d] / n;
    const auto it = digit.find(static_cast<int>(d));
    const int64_t k = it == digit.end() ? 0 : it->second;
    out.emplace_back(k * sz, sz);
  }
  return out;
}

std::vector<int64_t> DistributedStates::local_shape(const std::vector<int64_t>& shape) const {
  std::vector<int64_t> out(shape);
  for (size_t d = 0; d < shape.size(); ++d) {
    const int n = get_dim(static_cast<int>(d));
    if (shape[d] % n != 0) fail("local_shape: dimension not divisible by its split count");
    out[d] = shape[d] / n;
  }
  return out;
}

std::string DistributedStates::info() const {
  std::ostringstream os;
  os << "device_num=" << device_num_ << ", order=[";
  for (size_t i = 0; i < order_.size(); ++i) os << (i ? ", " : "") << order_[i];
  os << "], states={";
  bool first = true;
  for (const auto& kv : states_) {
    if (kv.second == 1) continue;
    os << (first ? "" : ", ") << kv.first << ": " << kv.second;
    first = false;
  }
  os << "}, zero=" << (zero_ ? "true" : "false");
  return os.str();
}

const DistributedStates& DistributedStatesUnion::get(size_t i) const {
  if (i >= list_.size()) fail("DistributedStatesUnion::get: index out of range");
  return list_[i];
}

DistributedStates DistributedStatesUnion::get_local(size_t i) const {
  const DistributedStates& ds = get(i);
  if (!is_hetero()) return ds;
  const int n = static_cast<int>(list_.size());
  StateMap st = ds.states();
  const int cur = ds.get_dim(hetero_dim_);
  if (cur % n != 0) fail("get_local: hetero dim count not divisible by the union size");
  st[hetero_dim_] = cur / n;
  std::vector<int> order = ds.order();
  if (cur / n == 1) order.erase(std::remove(order.begin(), order.end(), hetero_dim_), order.end());
  return DistributedStates(ds.device_num() / n, st, order, ds.zero());
}

bool DistributedStatesUnion::check_equal(const DistributedStatesUnion& o) const {
  if (hetero_dim_ != o.hetero_dim_ || list_.size() != o.list_.size()) return false;
  for (size_t i = 0; i < list_.size(); ++i)
    if (!list_[i].check_equal(o.list_[i])) return false;
  return true;
}

std::string DistributedStatesUnion::info() const {
  std::ostringstream os;
  os << "ds_list={";
  for (size_t i = 0; i < list_.size(); ++i) os << (i ? ", {" : "{") << list_[i].info() << "}";
  os << "}, hetero_dim=" << hetero_dim_;
  return os.str();
}

static uint32_t classify_pair(const DistributedStates& s, const DistributedStates& d, bool same_group) {
  if (s.check_equal(d)) return same_group ? COMM_UNUSED : COMM_P2P;
  if (same_group) {
    if (s.is_pure_duplicate()) return COMM_SPLIT;
    if (s.check_scatter(d)) return COMM_SCATTER;
    if (s.check_allreduce(d)) return COMM_ALL_REDUCE;
    if (s.check_allgather(d)) return COMM_ALL_GATHER;
    if (s.check_reducescatter(d)) return COMM_REDUCE_SCATTER;
    // any other same-group relayout with equal partial degree is a general repartition
    if (s.get_dim(kPartial) == d.get_dim(kPartial)) return COMM_BATCHED_SEND_RECV;
    return COMM_UNSUPPORTED;
  }
  if (s.get_dim(kPartial) == d.get_dim(kPartial)) return COMM_BATCHED_SEND_RECV;
  return COMM_UNSUPPORTED;
}

uint32_t classify_comm(const DistributedStatesUnion& src, const std::vector<int>& src_group,
                       const DistributedStatesUnion& dst, const std::vector<int>& dst_group, size_t member) {
  const bool same_group = src_group == dst_group;
  if (src.hetero_dim() == dst.hetero_dim()) {
    const size_t ms = std::min(member, src.size() - 1), md = std::min(member, dst.size() - 1);
    return classify_pair(src.get(ms), dst.get(md), same_group);
  }
  // differing hetero dims: split collectives over the union, plus an optional local pre-collective
  uint32_t t;
  if (src.hetero_dim() == kPartial && dst.hetero_dim() == kDup) t = COMM_SPLIT_ALL_REDUCE;
  else if (src.hetero_dim() == kPartial && dst.hetero_dim() == 0) t = COMM_SPLIT_REDUCE_SCATTER;
  else if (src.hetero_dim() == 0 && dst.hetero_dim() == kDup) t = COMM_SPLIT_ALL_GATHER;
  else return COMM_UNSUPPORTED;
  const size_t ms = std::min(member, src.size() - 1), md = std::min(member, dst.size() - 1);
  const DistributedStates ls = src.get_local(ms), ld = dst.get_local(md);
  if (!ls.check_equal(ld)) {
    const uint32_t local = classify_pair(ls, ld, true);
    if (local == COMM_UNSUPPORTED) return COMM_UNSUPPORTED;
    t |= local;
  }
  return t;
}

SplitCommPlan split_comm_groups(const std::vector<DistributedStates>& local_ds,
                                const std::vector<std::vector<int>>& groups, int rank) {
  if (local_ds.empty() || local_ds.size() != groups.size())
    throw std::invalid_argument("split_comm_groups: one device group per union member is required");
  const size_t members = local_ds.size();
  SplitCommPlan plan;
  int split_dim = kNoHeteroDim;
  int finest = 1;
  for (size_t j = 0; j < members; ++j) {
    int found = 0;
    for (const auto& kv : local_ds[j].states()) {
      if (kv.second == 1 || kv.first == kDup) continue;
      if (kv.first == kPartial) throw std::invalid_argument("split_comm_groups: a member's local layout is still partial");
      if (++found > 1) throw std::invalid_argument("split_comm_groups: members may split a single dimension only");
      if (split_dim == kNoHeteroDim) split_dim = kv.first;
      if (split_dim != kv.first) throw std::invalid_argument("split_comm_groups: members split different dimensions");
      finest = std::max(finest, kv.second);
    }
    if (local_ds[j].device_num() != static_cast<int>(groups[j].size()))
      throw std::invalid_argument("split_comm_groups: layout and device group sizes differ");
  }
  if (split_dim == kNoHeteroDim) split_dim = 0;
  plan.split_dim = split_dim;

  // holders[j][block][dup] = rank
  std::vector<std::vector<std::vector<int>>> holders(members);
  int my_member = -1, my_block = 0;
  for (size_t j = 0; j < members; ++j) {
    const int sj = local_ds[j].get_dim(split_dim), dj = local_ds[j].get_dim(kDup);
    if (finest % sj) throw std::invalid_argument("split_comm_groups: split counts must divide the finest one");
    holders[j].assign(sj, std::vector<int>(dj, -1));
    for (size_t i = 0; i < groups[j].size(); ++i) {
      const auto idx = local_ds[j].map_device_to_state_index(static_cast<int>(i));
      auto at = [&](int d) { auto it = idx.find(d); return it == idx.end() ? 0 : it->second; };
      holders[j][at(split_dim)][at(kDup)] = groups[j][i];
      if (groups[j][i] == rank) { my_member = static_cast<int>(j); my_block = at(split_dim); }
    }
  }
  if (my_member < 0) throw std::invalid_argument("split_comm_groups: rank is in no member of the union");
  const int per_block = finest / local_ds[my_member].get_dim(split_dim);
  plan.micro_blocks = per_block;
  plan.first_micro_block = my_block * per_block;
  for (int m = 0; m < per_block; ++m) {
    const int mb = plan.first_micro_block + m;
    size_t widest = 0;
    std::vector<const std::vector<int>*> who(members);
    for (size_t j = 0; j < members; ++j) {
      const int per = finest / local_ds[j].get_dim(split_dim);
      who[j] = &holders[j][mb / per];
      widest = std::max(widest, who[j]->size());
    }
    std::vector<std::vector<int>> mine;
    for (size_t k = 0; k < widest; ++k) {
      std::vector<int> g;
      bool has_me = false;
      for (size_t j = 0; j < members; ++j) {
        const int r = (*who[j])[k % who[j]->size()];
        g.push_back(r);
        has_me |= r == rank;
      }
      if (has_me) mine.push_back(std::move(g));
    }
    plan.groups.push_back(std::move(mine));
  }
  return plan;
}

const char* comm_type_name(uint32_t t) {
  switch (t) {
    case COMM_UNUSED: return "UNUSED";
    case COMM_P2P: return "P2P";
    case COMM_SPLIT: return "COMM_SPLIT";
    case COMM_ALL_REDUCE: return "ALL_REDUCE";
    case COMM_ALL_GATHER: return "ALL_GATHER";
    case COMM_REDUCE_SCATTER: return "REDUCE_SCATTER";
    case COMM_SCATTER: return "SCATTER";
    case COMM_BATCHED_SEND_RECV: return "BATCHED_ISEND_IRECV";
    case COMM_SPLIT_ALL_REDUCE: return "SPLIT_ALL_REDUCE";
    case COMM_SPLIT_REDUCE_SCATTER: return "SPLIT_REDUCE_SCATTER";
    case COMM_SPLIT_ALL_GATHER: return "SPLIT_ALL_GATHER";
    case COMM_UNSUPPORTED: return "UNSUPPORTED";
    default: return "COMPOSITE";
  }
}

DistributedStates deduce_linear(const DistributedStates& a, const DistributedStates& b, bool trans_a, bool trans_b) {
  // Resolve transposes to the math layout a:[m,k], b:[k,n].
  const int a_row = a.get_dim(trans_a ? 1 : 0), a_col = a.get_dim(trans_a ? 0 : 1);
  const int b_row = b.get_dim(trans_b ? 1 : 0), b_col = b.get_dim(trans_b ? 0 : 1);
  if (a.device_num() != b.device_num()) fail("deduce_linear: operands live on different device counts");
  if (a_col != b_row) fail("deduce_linear: contraction dim is split differently in the two operands");
  if (a.get_dim(kPartial) != 1 || b.get_dim(kPartial) != 1) fail("deduce_linear: partial operands are not supported");
  const int n = a.device_num();
  const int partial = a_col;
  const int used = partial * a_row * b_col;
  if (n % used != 0) fail("deduce_linear: layouts do not tile the device group");
  StateMap st{{kPartial, partial}, {kDup, n / used}, {0, a_row}, {1, b_col}};
  // Order: walk a's digits, mapping a's row dim -> 0, a's contraction dim -> -2, a's dup -> (b's col dim, 1)
  // when b splits its columns over exactly those devices, else -1.
  const int a_row_dim = trans_a ? 1 : 0, a_col_dim = trans_a ? 0 : 1;
  std::vector<int> order;
  auto push = [&](int d) {
    if (st[d] > 1 && std::find(order.begin(), order.end(), d) == order.end()) order.push_back(d);
  };
  for (int o : a.order()) {
    if (o == a_row_dim) push(0);
    else if (o == a_col_dim) push(kPartial);
    else if (o == kDup) {
      if (b_col > 1) push(1);
      if (st[kDup] > 1) push(kDup);
    }
  }
  push(kPartial); push(kDup); push(0); push(1);
  return DistributedStates(n, st, order, false);
}

}  // namespace hsb
