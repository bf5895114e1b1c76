#include "planner.h"

#include <map>

#include <algorithm>
#include <numeric>
#include <stdexcept>

namespace hsb {

static int64_t lcm64(int64_t a, int64_t b) { return a / std::gcd(a, b) * b; }

ReshardPlanner::ReshardPlanner(int world_size, int policy) : world_(world_size), policy_(policy) {
  stats_.sent_elems.assign(world_size, 0);
  stats_.recv_elems.assign(world_size, 0);
}

namespace {
struct Folded {
  int64_t R, C;      // folded global shape
  int sr, sc;        // split counts along rows / cols
  int row_dim, col_dim;  // which DS dims they came from (-100 = none)
};

Folded fold(const TensorLayout& t) {
  Folded f{1, 1, 1, 1, -100, -100};
  const auto& s = t.shape;
  if (s.empty()) return f;
  for (const auto& kv : t.ds.states())
    if (kv.first >= 2 && kv.second > 1) throw std::invalid_argument("reshard: only dims 0 and 1 may be split");
  if (s.size() == 1) {
    f.R = 1; f.C = s[0];
    f.sc = t.ds.get_dim(0); f.col_dim = 0;
  } else {
    f.R = s[0];
    f.C = 1;
    for (size_t d = 1; d < s.size(); ++d) f.C *= s[d];
    f.sr = t.ds.get_dim(0); f.row_dim = 0;
    f.sc = t.ds.get_dim(1); f.col_dim = 1;
  }
  if (f.R % f.sr || f.C % f.sc) throw std::invalid_argument("reshard: shape not divisible by split counts");
  return f;
}

int digit_of(const StateMap& m, int dim) {
  auto it = m.find(dim);
  return it == m.end() ? 0 : it->second;
}
}  // namespace

std::vector<Region> regions_of(const TensorLayout& t, int replica) {
  if (static_cast<int>(t.group.size()) != t.ds.device_num())
    throw std::invalid_argument("reshard: device group size does not match the DS device_num");
  const Folded f = fold(t);
  const int64_t lr = f.R / f.sr, lc = f.C / f.sc;
  const int ndup = t.ds.get_dim(kDup);
  std::vector<Region> out;
  for (int i = 0; i < t.ds.device_num(); ++i) {
    const StateMap dg = t.ds.map_device_to_state_index(i);
    if (replica >= 0 && digit_of(dg, kDup) != replica % ndup) continue;
    const int rd = f.row_dim == -100 ? 0 : digit_of(dg, f.row_dim);
    const int cd = f.col_dim == -100 ? 0 : digit_of(dg, f.col_dim);
    out.push_back({t.group[i], rd * lr, (rd + 1) * lr, cd * lc, (cd + 1) * lc});
  }
  return out;
}

void ReshardPlanner::add_tensor(int tensor_id, const TensorLayout& src, const TensorLayout& dst) {
  if (src.shape != dst.shape) throw std::invalid_argument("reshard: src and dst global shapes differ");
  if (src.ds.get_dim(kPartial) > 1 || dst.ds.get_dim(kPartial) > 1)
    throw std::invalid_argument("reshard: partial tensors cannot be switched; reduce them first");
  add_tensor_regions(tensor_id, regions_of(src), regions_of(dst), false);
}

void ReshardPlanner::add_tensor_regions(int tensor_id, const std::vector<Region>& src, const std::vector<Region>& dst,
                                        bool gather_all) {
  // cut lines of every region -> cells that no region boundary crosses
  std::vector<int64_t> rc, cc;
  for (const auto* v : {&src, &dst})
    for (const auto& g : *v) {
      if (g.r1 <= g.r0 || g.c1 <= g.c0) throw std::invalid_argument("reshard: empty region");
      if (g.rank < 0 || g.rank >= world_) throw std::invalid_argument("reshard: region rank outside the world");
      rc.push_back(g.r0); rc.push_back(g.r1); cc.push_back(g.c0); cc.push_back(g.c1);
    }
  std::sort(rc.begin(), rc.end()); rc.erase(std::unique(rc.begin(), rc.end()), rc.end());
  std::sort(cc.begin(), cc.end()); cc.erase(std::unique(cc.begin(), cc.end()), cc.end());

  for (const auto& dreg : dst) {
    const int dst_rank = dreg.rank;
    const int64_t dst_ld = dreg.c1 - dreg.c0;
    for (size_t ri = 0; ri + 1 < rc.size(); ++ri) {
      const int64_t r0 = rc[ri], r1 = rc[ri + 1];
      if (r0 < dreg.r0 || r1 > dreg.r1) continue;
      for (size_t ci = 0; ci + 1 < cc.size(); ++ci) {
        const int64_t c0 = cc[ci], c1 = cc[ci + 1];
        if (c0 < dreg.c0 || c1 > dreg.c1) continue;
        std::vector<const Region*> own;
        for (const auto& sreg : src)
          if (sreg.r0 <= r0 && r1 <= sreg.r1 && sreg.c0 <= c0 && c1 <= sreg.c1) own.push_back(&sreg);
        if (own.empty()) throw std::runtime_error("reshard: a needed slice has no owner (hot switch impossible)");
        std::vector<const Region*> chosen;
        if (gather_all) {
          chosen = own;
        } else {
          const Region* pick = nullptr;
          for (const auto* o : own)
            if (o->rank == dst_rank) { pick = o; break; }
          if (!pick) {
            switch (policy_) {
              case SENDER_FCFS: pick = own[0]; break;
              case SENDER_ROUND_ROBIN: pick = own[(rr_++) % own.size()]; break;
              case SENDER_GREEDY:
              case SENDER_BALANCED:
              default: {
                int64_t best = -1;
                const size_t start = policy_ == SENDER_BALANCED ? static_cast<size_t>(rr_++) % own.size() : 0;
                for (size_t k = 0; k < own.size(); ++k) {
                  const Region* o = own[(start + k) % own.size()];
                  const int64_t sent = stats_.sent_elems[o->rank];
                  if (best < 0 || sent < best) { best = sent; pick = o; }
                }
              }
            }
          }
          chosen.push_back(pick);
        }
        for (const Region* sreg : chosen) {
          CopyDesc d;
          d.tensor_id = tensor_id;
          d.src_rank = sreg->rank;
          d.dst_rank = dst_rank;
          d.rows = r1 - r0;
          d.row_elems = c1 - c0;
          d.src_ld = sreg->c1 - sreg->c0;
          d.dst_ld = dst_ld;
          d.src_off = (r0 - sreg->r0) * d.src_ld + (c0 - sreg->c0);
          d.dst_off = (r0 - dreg.r0) * dst_ld + (c0 - dreg.c0);
          const int64_t n = d.rows * d.row_elems;
          if (d.src_rank == dst_rank) stats_.local_elems += n;
          else {
            stats_.remote_elems += n;
            stats_.sent_elems[d.src_rank] += n;
            stats_.recv_elems[dst_rank] += n;
          }
          bool merged = false;
          // merge with an earlier descriptor of this tensor/pair that it extends downwards or sideways
          for (size_t k = copies_.size(); k-- > 0 && !merged;) {
            CopyDesc& p = copies_[k];
            if (p.tensor_id != d.tensor_id) break;
            if (p.src_rank != d.src_rank || p.dst_rank != d.dst_rank || p.src_ld != d.src_ld || p.dst_ld != d.dst_ld)
              continue;
            if (p.rows == d.rows && p.src_off + p.row_elems == d.src_off && p.dst_off + p.row_elems == d.dst_off) {
              p.row_elems += d.row_elems;
              merged = true;
            } else if (p.row_elems == d.row_elems && p.src_off + p.rows * p.src_ld == d.src_off &&
                       p.dst_off + p.rows * p.dst_ld == d.dst_off) {
              p.rows += d.rows;
              merged = true;
            }
          }
          if (!merged) copies_.push_back(d);
        }
      }
    }
  }
}

std::vector<CopyDesc> ReshardPlanner::copies_for_dst(int rank) const {
  std::vector<CopyDesc> out;
  for (const auto& c : copies_)
    if (c.dst_rank == rank) out.push_back(c);
  return out;
}
std::vector<CopyDesc> ReshardPlanner::copies_for_src(int rank) const {
  std::vector<CopyDesc> out;
  for (const auto& c : copies_)
    if (c.src_rank == rank) out.push_back(c);
  return out;
}

std::vector<PipeTask> schedule_1f1b(int num_stages, int stage, int nmb) {
  if (num_stages < 1 || stage < 0 || stage >= num_stages || nmb < 1)
    throw std::invalid_argument("schedule_1f1b: bad arguments");
  std::vector<PipeTask> tasks;
  const int warmup = std::min(num_stages - stage - 1, nmb);
  const int steady = nmb - warmup;
  int f = 0, b = 0;
  for (int i = 0; i < warmup; ++i) tasks.push_back({true, f++});
  for (int i = 0; i < steady; ++i) {
    tasks.push_back({true, f++});
    tasks.push_back({false, b++});
  }
  for (int i = 0; i < warmup; ++i) tasks.push_back({false, b++});
  return tasks;
}

std::vector<PipeTask> schedule_gpipe(int num_stages, int stage, int nmb) {
  if (num_stages < 1 || stage < 0 || stage >= num_stages || nmb < 1)
    throw std::invalid_argument("schedule_gpipe: bad arguments");
  std::vector<PipeTask> tasks;
  for (int i = 0; i < nmb; ++i) tasks.push_back({true, i});
  for (int i = 0; i < nmb; ++i) tasks.push_back({false, i});
  return tasks;
}

std::vector<PackedBucket> bucket_and_pack(const std::vector<int64_t>& lengths, const std::vector<int64_t>& bounds,
                                          int64_t extra, bool drop_short) {
  if (bounds.size() < 2) throw std::invalid_argument("bucket_and_pack: need at least two bounds");
  for (size_t i = 1; i < bounds.size(); ++i)
    if (bounds[i] >= bounds[i - 1]) throw std::invalid_argument("bucket_and_pack: bounds must be descending");
  std::vector<int> idx(lengths.size());
  std::iota(idx.begin(), idx.end(), 0);
  std::stable_sort(idx.begin(), idx.end(), [&](int a, int b) { return lengths[a] > lengths[b]; });
  std::vector<PackedBucket> out;
  for (size_t b = 0; b + 1 < bounds.size(); ++b) out.push_back({bounds[b], bounds[b + 1], {}, {}});
  for (int i : idx) {
    const int64_t len = lengths[i];
    bool placed = false;
    for (auto& bk : out) {
      if (len > bk.min_len + extra && len <= bk.max_len + extra) {
        bk.members.push_back(i);
        placed = true;
        break;
      }
    }
    if (!placed) {
      if (len > bounds.front() + extra) throw std::invalid_argument("bucket_and_pack: sequence longer than the largest bucket");
      if (!drop_short) out.back().members.push_back(i);
    }
  }
  for (auto& bk : out) {
    const int64_t cap = bk.max_len + extra;
    std::vector<char> used(bk.members.size(), 0);
    for (size_t i = 0; i < bk.members.size(); ++i) {
      if (used[i]) continue;
      used[i] = 1;
      std::vector<int> row{bk.members[i]};
      int64_t cur = lengths[bk.members[i]];
      for (size_t j = i + 1; j < bk.members.size(); ++j) {
        if (used[j]) continue;
        const int64_t l = lengths[bk.members[j]];
        if (cur + l <= cap) {
          row.push_back(bk.members[j]);
          cur += l;
          used[j] = 1;
        }
      }
      bk.rows.push_back(std::move(row));
    }
  }
  return out;
}

std::vector<std::vector<int>> balance_rows(const std::vector<int64_t>& row_tokens, int dp) {
  if (dp < 1) throw std::invalid_argument("balance_rows: dp must be >= 1");
  std::vector<int> idx(row_tokens.size());
  std::iota(idx.begin(), idx.end(), 0);
  std::stable_sort(idx.begin(), idx.end(), [&](int a, int b) { return row_tokens[a] > row_tokens[b]; });
  std::vector<std::vector<int>> out(dp);
  std::vector<int64_t> load(dp, 0);
  for (int i : idx) {
    int best = 0;
    for (int r = 1; r < dp; ++r)
      if (load[r] < load[best] || (load[r] == load[best] && out[r].size() < out[best].size())) best = r;
    out[best].push_back(i);
    load[best] += row_tokens[i];
  }
  return out;
}

DescTable build_reshard_descriptors(const std::vector<RectBytes>& rects, int64_t unit_bytes, int rank, int world) {
  if (unit_bytes <= 0 || world <= 0) throw std::invalid_argument("build_reshard_descriptors: bad unit or world size");
  struct Unit { int64_t src, dst, rows, row_bytes, src_ld, dst_ld; int32_t unit_rows; };
  std::map<int, std::vector<Unit>> by_src;
  for (const RectBytes& in : rects) {
    int64_t r = in.rows, rb = in.row_bytes, sld = in.src_ld, dld = in.dst_ld;
    if (r < 1 || rb < 1) throw std::invalid_argument("build_reshard_descriptors: empty rectangle");
    // full-width rectangles are one long row: fewer, larger units
    if (sld == rb && dld == rb) { rb *= r; sld = dld = rb; r = 1; }
    std::vector<Unit>& bucket = by_src[in.src_rank];
    if (r == 1 && rb > unit_bytes) {
      const int64_t chunks = (rb + unit_bytes - 1) / unit_bytes;
      for (int64_t k = 0; k < chunks; ++k) {
        const int64_t b0 = k * unit_bytes;
        bucket.push_back({in.src + b0, in.dst + b0, 1, std::min(unit_bytes, rb - b0), 0, 0, 1});
      }
    } else {
      const int64_t ur = std::max<int64_t>(1, unit_bytes / std::max<int64_t>(rb, 1));
      const int64_t units = (r + ur - 1) / ur;
      for (int64_t k = 0; k < units; ++k) {
        const int64_t r0 = k * ur;
        bucket.push_back({in.src + r0 * sld, in.dst + r0 * dld, std::min(ur, r - r0), rb, sld, dld,
                          static_cast<int32_t>(ur)});
      }
    }
  }
  std::vector<int> order;
  for (const auto& kv : by_src) order.push_back(kv.first);
  auto dist = [&](int q) { return ((q - rank - 1) % world + world) % world; };
  std::stable_sort(order.begin(), order.end(), [&](int a, int b) { return dist(a) < dist(b); });
  size_t left = 0;
  for (const auto& kv : by_src) left += kv.second.size();
  DescTable out;
  out.descs.reserve(left * 6);
  out.unit_rows.reserve(left);
  out.prefix.reserve(left + 1);
  out.prefix.push_back(0);
  std::map<int, size_t> cursor;
  while (left) {
    for (int q : order) {
      size_t& i = cursor[q];
      const std::vector<Unit>& b = by_src[q];
      if (i >= b.size()) continue;
      const Unit& u = b[i++];
      out.descs.insert(out.descs.end(), {u.src, u.dst, u.rows, u.row_bytes, u.src_ld, u.dst_ld});
      out.unit_rows.push_back(u.unit_rows);
      out.prefix.push_back(out.prefix.back() + static_cast<int32_t>((u.rows + u.unit_rows - 1) / u.unit_rows));
      --left;
    }
  }
  return out;
}

int64_t plan_arena(const std::vector<int64_t>& numels, int64_t align, std::vector<int64_t>* offsets) {
  if (align < 1) align = 1;
  int64_t off = 0;
  offsets->clear();
  for (int64_t n : numels) {
    off = (off + align - 1) / align * align;
    offsets->push_back(off);
    off += n;
  }
  return (off + align - 1) / align * align;
}

}  // namespace hsb
