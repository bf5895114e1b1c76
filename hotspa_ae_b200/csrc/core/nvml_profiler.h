// Thin runtime-loaded NVML reader: device memory (total/used) and per-link NVLink TX/RX byte
// counters, used by the hot-switch and memory profilers.  libnvidia-ml is opened with dlopen so
// the core library loads on machines without a driver; every call then reports "unavailable".
// Reference counterpart: hetu/graph/profiler.{h,cc} (CUDAProfiler).  Read-only: no setting is changed.
#pragma once
#include <cstdint>
#include <string>
#include <vector>

namespace hsb {

struct NvmlMemory { bool ok = false; uint64_t total = 0, used = 0, free = 0; };
struct NvlinkCounters { bool ok = false; std::vector<uint64_t> tx_kib, rx_kib; };

class NvmlProfiler {
 public:
  // `lib_path` empty -> "libnvidia-ml.so.1".  A test can point this at a fake library.
  explicit NvmlProfiler(const std::string& lib_path = "");
  ~NvmlProfiler();
  bool available() const { return ok_; }
  int device_count() const;
  NvmlMemory memory(int device) const;
  NvlinkCounters nvlink(int device, int max_links = 18) const;

 private:
  void* handle_ = nullptr;
  bool ok_ = false;
  void* fn_count_ = nullptr;
  void* fn_handle_ = nullptr;
  void* fn_mem_ = nullptr;
  void* fn_field_ = nullptr;
  void* fn_shutdown_ = nullptr;
};

}  // namespace hsb
