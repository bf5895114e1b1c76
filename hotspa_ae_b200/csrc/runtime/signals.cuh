// Cross-GPU flags over peer-mapped memory with bounded waits.
//
// A flag is a 32-bit word in a peer-visible buffer.  Writers publish data with st.release.sys /
// red.release.sys after the data; readers poll with ld.acquire.sys.  Flags carry epoch numbers so that
// buffers are reusable without clearing.  A wait that does not see its value within the caller's
// time limit records ST_TIMEOUT_PEER_FLAG in the status word and returns false; the kernel then
// skips its remaining work and exits, so the context stays usable and the host raises an error.
#pragma once
#include "common.cuh"

namespace hsb {

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_gpu(uint32_t* p, uint32_t v) {
  asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_gpu(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void red_add_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void red_add_release_gpu(uint32_t* p, uint32_t v) {
  asm volatile("red.release.gpu.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// Epoch comparison that survives wrap-around.
__device__ __forceinline__ bool epoch_reached(uint32_t seen, uint32_t want) {
  return static_cast<int32_t>(seen - want) >= 0;
}

// Spins until *flag >= want (system scope).  Returns false (and sets *status) on time-out.
__device__ __forceinline__ bool wait_flag_sys(const uint32_t* flag, uint32_t want, uint64_t limit_ns, int* status) {
  if (epoch_reached(ld_acquire_sys(flag), want)) return true;
  const uint64_t t0 = globaltimer_ns();
  uint32_t it = 0;
  while (!epoch_reached(ld_acquire_sys(flag), want)) {
    if (((++it) & 0x3f) == 0) {
      if (*reinterpret_cast<volatile int*>(status) != ST_OK) return false;
      if (globaltimer_ns() - t0 > limit_ns) {
        atomicCAS(status, ST_OK, ST_TIMEOUT_PEER_FLAG);
        return false;
      }
      __nanosleep(64);
    }
  }
  return true;
}
__device__ __forceinline__ bool wait_flag_gpu(const uint32_t* flag, uint32_t want, uint64_t limit_ns, int* status) {
  if (epoch_reached(ld_acquire_gpu(flag), want)) return true;
  const uint64_t t0 = globaltimer_ns();
  uint32_t it = 0;
  while (!epoch_reached(ld_acquire_gpu(flag), want)) {
    if (((++it) & 0x3f) == 0) {
      if (*reinterpret_cast<volatile int*>(status) != ST_OK) return false;
      if (globaltimer_ns() - t0 > limit_ns) {
        atomicCAS(status, ST_OK, ST_TIMEOUT_PEER_FLAG);
        return false;
      }
      __nanosleep(32);
    }
  }
  return true;
}

// 128-bit loads/stores that bypass L1 (peer memory is not kept coherent in L1).
__device__ __forceinline__ uint4 ld_peer_v4(const void* p) {
  uint4 v;
  asm volatile("ld.relaxed.sys.global.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p)
               : "memory");
  return v;
}
__device__ __forceinline__ void st_peer_v4(void* p, uint4 v) {
  asm volatile("st.relaxed.sys.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z),
               "r"(v.w)
               : "memory");
}

constexpr int SYMM_MAX_RANKS = 16;
// Pointers to the same buffer on every rank of a group, indexed by position in the group.
struct PeerPtrs {
  void* p[SYMM_MAX_RANKS];
};

}  // namespace hsb
