// pybind11 surface of the host-side core (module `_hsb_core`).
#include <pybind11/numpy.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include "ds.h"
#include "nvml_profiler.h"
#include "planner.h"
#include "signal_model.h"
#include "symbol.h"

namespace py = pybind11;
using namespace hsb;

static IntSymbol to_symbol(const py::handle& h) {
  if (py::isinstance<IntSymbol>(h)) return h.cast<IntSymbol>();
  return IntSymbol(h.cast<int64_t>());
}

PYBIND11_MODULE(_hsb_core, m) {
  m.doc() = "hotspa_ae_b200 host core: distributed states, planners, symbolic ints, NVML reader";

  py::class_<DistributedStates>(m, "DistributedStates")
      .def(py::init<int, const StateMap&, const std::vector<int>&, bool>(), py::arg("device_num"), py::arg("states"),
           py::arg("order") = std::vector<int>{}, py::arg("zero") = false)
      .def_property_readonly("device_num", &DistributedStates::device_num)
      .def_property_readonly("states", &DistributedStates::states)
      .def_property_readonly("order", &DistributedStates::order)
      .def_property("zero", &DistributedStates::zero, &DistributedStates::set_zero)
      .def_property_readonly("is_pure_duplicate", &DistributedStates::is_pure_duplicate)
      .def("is_valid", &DistributedStates::is_valid)
      .def("get_dim", &DistributedStates::get_dim)
      .def("check_equal", &DistributedStates::check_equal)
      .def("check_max_dim", &DistributedStates::check_max_dim)
      .def("map_device_to_state_index", &DistributedStates::map_device_to_state_index)
      .def("map_to_local_data", &DistributedStates::map_device_to_state_index)
      .def("get_dup_group_index", &DistributedStates::get_dup_group_index)
      .def("get_devices_by_dim", &DistributedStates::get_devices_by_dim)
      .def("get_loop_sizes", &DistributedStates::get_loop_sizes)
      .def("check_allreduce", &DistributedStates::check_allreduce)
      .def("check_allgather", &DistributedStates::check_allgather)
      .def("check_reducescatter", &DistributedStates::check_reducescatter)
      .def("check_scatter", &DistributedStates::check_scatter)
      .def("check_broadcast", &DistributedStates::check_broadcast)
      .def("check_reduce", &DistributedStates::check_reduce)
      .def("check_combine", &DistributedStates::check_combine)
      .def("local_slice", &DistributedStates::local_slice)
      .def("local_shape", &DistributedStates::local_shape)
      .def("ds_info", &DistributedStates::info)
      .def("__repr__", [](const DistributedStates& d) { return "DistributedStates(" + d.info() + ")"; })
      .def("__eq__", &DistributedStates::check_equal)
      .def_static("combine_states", &DistributedStates::combine_states)
      .def_static("combine_order", [](const std::vector<int>& src, int dst, const std::vector<int>& order) {
        bool ok = true;
        auto out = DistributedStates::combine_order(src, dst, order, &ok);
        if (!ok) throw std::invalid_argument("combine_order: dims are not adjacent in the order");
        return out;
      });

  py::class_<DistributedStatesUnion>(m, "DistributedStatesUnion")
      .def(py::init<std::vector<DistributedStates>, int>(), py::arg("ds_list"), py::arg("hetero_dim") = kNoHeteroDim)
      .def_property_readonly("ds_list", &DistributedStatesUnion::ds_list)
      .def_property_readonly("hetero_dim", &DistributedStatesUnion::hetero_dim)
      .def("size", &DistributedStatesUnion::size)
      .def("__len__", &DistributedStatesUnion::size)
      .def("is_hetero", &DistributedStatesUnion::is_hetero)
      .def("get", &DistributedStatesUnion::get)
      .def("get_local", &DistributedStatesUnion::get_local)
      .def("check_equal", &DistributedStatesUnion::check_equal)
      .def("ds_union_info", &DistributedStatesUnion::info)
      .def("__repr__", [](const DistributedStatesUnion& d) { return "DistributedStatesUnion(" + d.info() + ")"; });

  m.def("classify_comm", &classify_comm, py::arg("src"), py::arg("src_group"), py::arg("dst"), py::arg("dst_group"),
        py::arg("member") = 0);
  m.def("comm_type_name", &comm_type_name);
  // host model of the cross-GPU flag protocols (threads + atomics); the GIL is released while the ranks run
  auto as_dict = [](const ModelResult& r) {
    py::dict d;
    d["checks"] = r.checks; d["violations"] = r.violations; d["timeouts"] = r.timeouts;
    return d;
  };
  m.def("run_barrier_model", [as_dict](int n, int calls, uint32_t first_epoch, uint64_t seed) {
    ModelResult r;
    { py::gil_scoped_release rel; r = run_barrier_model(n, calls, first_epoch, seed); }
    return as_dict(r);
  }, py::arg("n"), py::arg("calls"), py::arg("first_epoch") = 1u, py::arg("seed") = 0);
  m.def("run_reduce_scatter_model", [as_dict](int n, int calls, int counter_sets, int recv_buffers, int row_blocks,
                                              int parts, uint64_t seed) {
    ModelResult r;
    { py::gil_scoped_release rel;
      r = run_reduce_scatter_model(n, calls, counter_sets, recv_buffers, row_blocks, parts, seed); }
    return as_dict(r);
  }, py::arg("n"), py::arg("calls"), py::arg("counter_sets") = 3, py::arg("recv_buffers") = 2,
     py::arg("row_blocks") = 4, py::arg("parts") = 4, py::arg("seed") = 0);
  m.def("run_all_gather_model", [as_dict](int n, int calls, int stage_buffers, int chunks, uint64_t seed) {
    ModelResult r;
    { py::gil_scoped_release rel; r = run_all_gather_model(n, calls, stage_buffers, chunks, seed); }
    return as_dict(r);
  }, py::arg("n"), py::arg("calls"), py::arg("stage_buffers") = 2, py::arg("chunks") = 8, py::arg("seed") = 0);
  py::class_<SplitCommPlan>(m, "SplitCommPlan")
      .def_readonly("split_dim", &SplitCommPlan::split_dim)
      .def_readonly("micro_blocks", &SplitCommPlan::micro_blocks)
      .def_readonly("first_micro_block", &SplitCommPlan::first_micro_block)
      .def_readonly("groups", &SplitCommPlan::groups);
  m.def("split_comm_groups", &split_comm_groups, py::arg("local_ds"), py::arg("groups"), py::arg("rank"));
  m.def("deduce_linear", &deduce_linear);
  m.attr("COMM_UNUSED") = static_cast<uint32_t>(COMM_UNUSED);
  m.attr("COMM_P2P") = static_cast<uint32_t>(COMM_P2P);
  m.attr("COMM_SPLIT") = static_cast<uint32_t>(COMM_SPLIT);
  m.attr("COMM_ALL_REDUCE") = static_cast<uint32_t>(COMM_ALL_REDUCE);
  m.attr("COMM_ALL_GATHER") = static_cast<uint32_t>(COMM_ALL_GATHER);
  m.attr("COMM_REDUCE_SCATTER") = static_cast<uint32_t>(COMM_REDUCE_SCATTER);
  m.attr("COMM_SCATTER") = static_cast<uint32_t>(COMM_SCATTER);
  m.attr("COMM_BATCHED_SEND_RECV") = static_cast<uint32_t>(COMM_BATCHED_SEND_RECV);
  m.attr("COMM_SPLIT_ALL_REDUCE") = static_cast<uint32_t>(COMM_SPLIT_ALL_REDUCE);
  m.attr("COMM_SPLIT_REDUCE_SCATTER") = static_cast<uint32_t>(COMM_SPLIT_REDUCE_SCATTER);
  m.attr("COMM_SPLIT_ALL_GATHER") = static_cast<uint32_t>(COMM_SPLIT_ALL_GATHER);
  m.attr("COMM_UNSUPPORTED") = static_cast<uint32_t>(COMM_UNSUPPORTED);

  py::class_<CopyDesc>(m, "CopyDesc")
      .def_readonly("tensor_id", &CopyDesc::tensor_id)
      .def_readonly("src_rank", &CopyDesc::src_rank)
      .def_readonly("dst_rank", &CopyDesc::dst_rank)
      .def_readonly("src_off", &CopyDesc::src_off)
      .def_readonly("dst_off", &CopyDesc::dst_off)
      .def_readonly("rows", &CopyDesc::rows)
      .def_readonly("row_elems", &CopyDesc::row_elems)
      .def_readonly("src_ld", &CopyDesc::src_ld)
      .def_readonly("dst_ld", &CopyDesc::dst_ld)
      .def("as_tuple", [](const CopyDesc& c) {
        return py::make_tuple(c.tensor_id, c.src_rank, c.dst_rank, c.src_off, c.dst_off, c.rows, c.row_elems,
                              c.src_ld, c.dst_ld);
      });

  py::class_<ReshardStats>(m, "ReshardStats")
      .def_readonly("sent_elems", &ReshardStats::sent_elems)
      .def_readonly("recv_elems", &ReshardStats::recv_elems)
      .def_readonly("local_elems", &ReshardStats::local_elems)
      .def_readonly("remote_elems", &ReshardStats::remote_elems);

  py::class_<ReshardPlanner>(m, "ReshardPlanner")
      .def(py::init<int, int>(), py::arg("world_size"), py::arg("policy") = static_cast<int>(SENDER_BALANCED))
      .def("add_tensor",
           [](ReshardPlanner& p, int id, const std::vector<int64_t>& shape, const DistributedStates& sds,
              const std::vector<int>& sgroup, const DistributedStates& dds, const std::vector<int>& dgroup) {
             p.add_tensor(id, TensorLayout{shape, sds, sgroup}, TensorLayout{shape, dds, dgroup});
           })
      .def("add_tensor_regions",
           [](ReshardPlanner& p, int id, const std::vector<std::tuple<int, int64_t, int64_t, int64_t, int64_t>>& src,
              const std::vector<std::tuple<int, int64_t, int64_t, int64_t, int64_t>>& dst, bool gather_all) {
             std::vector<Region> s, d;
             for (const auto& t : src) s.push_back({std::get<0>(t), std::get<1>(t), std::get<2>(t), std::get<3>(t), std::get<4>(t)});
             for (const auto& t : dst) d.push_back({std::get<0>(t), std::get<1>(t), std::get<2>(t), std::get<3>(t), std::get<4>(t)});
             p.add_tensor_regions(id, s, d, gather_all);
           }, py::arg("tensor_id"), py::arg("src"), py::arg("dst"), py::arg("gather_all_owners") = false)
      .def("copies", &ReshardPlanner::copies)
      .def("copies_for_dst", &ReshardPlanner::copies_for_dst)
      .def("copies_for_src", &ReshardPlanner::copies_for_src)
      .def_property_readonly("stats", &ReshardPlanner::stats);
  m.def("regions_of", [](const std::vector<int64_t>& shape, const DistributedStates& ds, const std::vector<int>& group,
                         int replica) {
    std::vector<std::tuple<int, int64_t, int64_t, int64_t, int64_t>> out;
    for (const auto& r : regions_of(TensorLayout{shape, ds, group}, replica))
      out.emplace_back(r.rank, r.r0, r.r1, r.c0, r.c1);
    return out;
  }, py::arg("shape"), py::arg("ds"), py::arg("group"), py::arg("replica") = -1);
  m.attr("SENDER_FCFS") = static_cast<int>(SENDER_FCFS);
  m.attr("SENDER_ROUND_ROBIN") = static_cast<int>(SENDER_ROUND_ROBIN);
  m.attr("SENDER_GREEDY") = static_cast<int>(SENDER_GREEDY);
  m.attr("SENDER_BALANCED") = static_cast<int>(SENDER_BALANCED);

  auto tasks_to_py = [](const std::vector<PipeTask>& ts) {
    std::vector<std::pair<bool, int>> out;
    for (const auto& t : ts) out.emplace_back(t.forward, t.micro_batch);
    return out;
  };
  m.def("schedule_1f1b", [=](int stages, int stage, int nmb) { return tasks_to_py(schedule_1f1b(stages, stage, nmb)); });
  m.def("schedule_gpipe", [=](int stages, int stage, int nmb) { return tasks_to_py(schedule_gpipe(stages, stage, nmb)); });

  py::class_<PackedBucket>(m, "PackedBucket")
      .def_readonly("max_len", &PackedBucket::max_len)
      .def_readonly("min_len", &PackedBucket::min_len)
      .def_readonly("members", &PackedBucket::members)
      .def_readonly("rows", &PackedBucket::rows);
  m.def("bucket_and_pack", &bucket_and_pack, py::arg("lengths"), py::arg("bucket_bounds"), py::arg("shift") = 0,
        py::arg("drop_short") = false);
  m.def("balance_rows", &balance_rows);
  // rects: int64 [n, 7] = src, dst, rows, row_bytes, src_ld_bytes, dst_ld_bytes, src_rank
  m.def("build_reshard_descriptors", [](py::array_t<int64_t, py::array::c_style | py::array::forcecast> rects,
                                        int64_t unit_bytes, int rank, int world) {
    if (rects.ndim() != 2 || rects.shape(1) != 7) throw std::invalid_argument("rects must be [n, 7] int64");
    const auto r = rects.unchecked<2>();
    std::vector<RectBytes> in(static_cast<size_t>(r.shape(0)));
    for (py::ssize_t i = 0; i < r.shape(0); ++i)
      in[i] = {r(i, 0), r(i, 1), r(i, 2), r(i, 3), r(i, 4), r(i, 5), static_cast<int>(r(i, 6))};
    DescTable t;
    { py::gil_scoped_release rel; t = build_reshard_descriptors(in, unit_bytes, rank, world); }
    const py::ssize_t n = static_cast<py::ssize_t>(t.unit_rows.size());
    py::array_t<int64_t> descs({n, static_cast<py::ssize_t>(6)});
    std::copy(t.descs.begin(), t.descs.end(), descs.mutable_data());
    py::array_t<int32_t> unit_rows(n), prefix(n + 1);
    std::copy(t.unit_rows.begin(), t.unit_rows.end(), unit_rows.mutable_data());
    std::copy(t.prefix.begin(), t.prefix.end(), prefix.mutable_data());
    return py::make_tuple(descs, unit_rows, prefix);
  }, py::arg("rects"), py::arg("unit_bytes"), py::arg("rank"), py::arg("world"));
  m.def("plan_arena", [](const std::vector<int64_t>& numels, int64_t align) {
    std::vector<int64_t> offs;
    const int64_t total = plan_arena(numels, align, &offs);
    return py::make_tuple(offs, total);
  });

  py::class_<IntSymbol>(m, "IntSymbol")
      .def(py::init<>())
      .def(py::init<int64_t>())
      .def("set_data", &IntSymbol::set)
      .def("reset_data", &IntSymbol::set)
      .def_property("data", &IntSymbol::get, &IntSymbol::set)
      .def("get_data", &IntSymbol::get)
      .def("is_leaf", &IntSymbol::is_leaf)
      .def("is_instantiated", &IntSymbol::is_instantiated)
      .def("same", &IntSymbol::same)
      .def("__int__", &IntSymbol::get)
      .def("__index__", &IntSymbol::get)
      .def("__repr__", [](const IntSymbol& s) { return "IntSymbol" + s.repr(); })
      .def("__add__", [](const IntSymbol& a, py::handle b) { return IntSymbol::make(IntSymbol::ADD, a, to_symbol(b)); })
      .def("__radd__", [](const IntSymbol& a, py::handle b) { return IntSymbol::make(IntSymbol::ADD, to_symbol(b), a); })
      .def("__sub__", [](const IntSymbol& a, py::handle b) { return IntSymbol::make(IntSymbol::SUB, a, to_symbol(b)); })
      .def("__rsub__", [](const IntSymbol& a, py::handle b) { return IntSymbol::make(IntSymbol::SUB, to_symbol(b), a); })
      .def("__mul__", [](const IntSymbol& a, py::handle b) { return IntSymbol::make(IntSymbol::MUL, a, to_symbol(b)); })
      .def("__rmul__", [](const IntSymbol& a, py::handle b) { return IntSymbol::make(IntSymbol::MUL, to_symbol(b), a); })
      .def("__truediv__", [](const IntSymbol& a, py::handle b) { return IntSymbol::make(IntSymbol::DIV, a, to_symbol(b)); })
      .def("__floordiv__", [](const IntSymbol& a, py::handle b) { return IntSymbol::make(IntSymbol::DIV, a, to_symbol(b)); })
      .def("__rfloordiv__", [](const IntSymbol& a, py::handle b) { return IntSymbol::make(IntSymbol::DIV, to_symbol(b), a); })
      .def("__mod__", [](const IntSymbol& a, py::handle b) { return IntSymbol::make(IntSymbol::REM, a, to_symbol(b)); });

  py::class_<NvmlMemory>(m, "NvmlMemory")
      .def_readonly("ok", &NvmlMemory::ok)
      .def_readonly("total", &NvmlMemory::total)
      .def_readonly("used", &NvmlMemory::used)
      .def_readonly("free", &NvmlMemory::free);
  py::class_<NvlinkCounters>(m, "NvlinkCounters")
      .def_readonly("ok", &NvlinkCounters::ok)
      .def_readonly("tx_kib", &NvlinkCounters::tx_kib)
      .def_readonly("rx_kib", &NvlinkCounters::rx_kib);
  py::class_<NvmlProfiler>(m, "NvmlProfiler")
      .def(py::init<const std::string&>(), py::arg("lib_path") = "")
      .def("available", &NvmlProfiler::available)
      .def("device_count", &NvmlProfiler::device_count)
      .def("memory", &NvmlProfiler::memory)
      .def("nvlink", &NvmlProfiler::nvlink, py::arg("device"), py::arg("max_links") = 18);
}
