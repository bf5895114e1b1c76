#include "nvml_profiler.h"

#include <dlfcn.h>
#include <cstring>

namespace hsb {

namespace {
struct MemInfo { unsigned long long total, free, used; };
// Layout of nvmlFieldValue_t (public NVML header): fieldId, scopeId, timestamp, latencyUsec,
// valueType, nvmlReturn, value (8-byte union).
struct FieldValue {
  unsigned int fieldId;
  unsigned int scopeId;
  long long timestamp;
  long long latencyUsec;
  int valueType;
  int nvmlReturn;
  union { double d; unsigned int ui; unsigned long ul; unsigned long long ull; long long sll; } value;
};
constexpr unsigned int FI_NVLINK_TX_L0 = 138;  // NVML_FI_DEV_NVLINK_THROUGHPUT_DATA_TX (per link via scopeId)
constexpr unsigned int FI_NVLINK_RX_L0 = 139;  // NVML_FI_DEV_NVLINK_THROUGHPUT_DATA_RX
using fn_init_t = int (*)();
using fn_count_t = int (*)(unsigned int*);
using fn_handle_t = int (*)(unsigned int, void**);
using fn_mem_t = int (*)(void*, MemInfo*);
using fn_field_t = int (*)(void*, int, FieldValue*);
}  // namespace

NvmlProfiler::NvmlProfiler(const std::string& lib_path) {
  const char* path = lib_path.empty() ? "libnvidia-ml.so.1" : lib_path.c_str();
  handle_ = dlopen(path, RTLD_LAZY | RTLD_LOCAL);
  if (!handle_) return;
  auto init = reinterpret_cast<fn_init_t>(dlsym(handle_, "nvmlInit_v2"));
  fn_count_ = dlsym(handle_, "nvmlDeviceGetCount_v2");
  fn_handle_ = dlsym(handle_, "nvmlDeviceGetHandleByIndex_v2");
  fn_mem_ = dlsym(handle_, "nvmlDeviceGetMemoryInfo");
  fn_field_ = dlsym(handle_, "nvmlDeviceGetFieldValues");
  fn_shutdown_ = dlsym(handle_, "nvmlShutdown");
  if (!init || !fn_count_ || !fn_handle_ || !fn_mem_) return;
  ok_ = init() == 0;
}

NvmlProfiler::~NvmlProfiler() {
  if (handle_) {
    if (ok_ && fn_shutdown_) reinterpret_cast<fn_init_t>(fn_shutdown_)();
    dlclose(handle_);
  }
}

int NvmlProfiler::device_count() const {
  if (!ok_) return 0;
  unsigned int n = 0;
  if (reinterpret_cast<fn_count_t>(fn_count_)(&n) != 0) return 0;
  return static_cast<int>(n);
}

NvmlMemory NvmlProfiler::memory(int device) const {
  NvmlMemory out;
  if (!ok_) return out;
  void* dev = nullptr;
  if (reinterpret_cast<fn_handle_t>(fn_handle_)(static_cast<unsigned int>(device), &dev) != 0) return out;
  MemInfo mi{};
  if (reinterpret_cast<fn_mem_t>(fn_mem_)(dev, &mi) != 0) return out;
  out.ok = true;
  out.total = mi.total; out.used = mi.used; out.free = mi.free;
  return out;
}

NvlinkCounters NvmlProfiler::nvlink(int device, int max_links) const {
  NvlinkCounters out;
  if (!ok_ || !fn_field_) return out;
  void* dev = nullptr;
  if (reinterpret_cast<fn_handle_t>(fn_handle_)(static_cast<unsigned int>(device), &dev) != 0) return out;
  std::vector<FieldValue> fv(static_cast<size_t>(max_links) * 2);
  std::memset(fv.data(), 0, fv.size() * sizeof(FieldValue));
  for (int l = 0; l < max_links; ++l) {
    fv[2 * l].fieldId = FI_NVLINK_TX_L0; fv[2 * l].scopeId = static_cast<unsigned int>(l);
    fv[2 * l + 1].fieldId = FI_NVLINK_RX_L0; fv[2 * l + 1].scopeId = static_cast<unsigned int>(l);
  }
  if (reinterpret_cast<fn_field_t>(fn_field_)(dev, static_cast<int>(fv.size()), fv.data()) != 0) return out;
  for (int l = 0; l < max_links; ++l) {
    if (fv[2 * l].nvmlReturn != 0 || fv[2 * l + 1].nvmlReturn != 0) continue;
    out.tx_kib.push_back(fv[2 * l].value.ull);
    out.rx_kib.push_back(fv[2 * l + 1].value.ull);
  }
  out.ok = !out.tx_kib.empty();
  return out;
}

}  // namespace hsb
