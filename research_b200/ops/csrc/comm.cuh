// Device-side primitives for kernels that talk to peer GPUs through mapped peer memory (NVLink):
// system-scope flag stores/loads and a *bounded* wait.  A wait that runs out records a status code and
// returns false; the kernel then skips the dependent work and exits, so the context stays usable.
// (The reference's vendored counterpart spins without a limit:
// third_party/ThunderKittens/include/ops/thread/util/sync.cuh:296-327.)
#pragma once
#include <stdint.h>

namespace b200comm {

enum CommError : int {
  ERR_PEER_READY = 21,   // a peer never announced its data for this epoch
  ERR_PEER_DONE = 22,    // a peer never finished reading / writing this rank's buffer
  ERR_LOCAL_FLAG = 23,   // a flag written by another CTA of the same kernel never arrived
};

constexpr int kMaxPeers = 8;
constexpr uint64_t kPeerWaitLimitNs = 2000000000ull;  // 2 s: the limit when the host configured none

// The status buffer that every kernel gets is four int32 words: [0] the first error code (0 = none), [1] unused,
// [2] the limit of a cross-GPU wait in milliseconds as configured by the host (0 = the 2 s default), [3] unused.
// The limit is read only on the slow path, after the first probes of a flag failed.
__device__ __forceinline__ uint64_t peer_wait_limit_ns(const int* status) {
  const int ms = reinterpret_cast<const volatile int*>(status)[2];
  return ms > 0 ? (uint64_t)ms * 1000000ull : kPeerWaitLimitNs;
}

// Layout of one rank's flag block (uint32 words) inside its symmetric arena.
//   ready[src]  written by rank src: "my buffer holds epoch e"
//   done[src]   written by rank src: "I finished using your buffer for epoch e"
struct FlagBlock {
  uint32_t ready[kMaxPeers];
  uint32_t done[kMaxPeers];
  uint32_t aux[48];
};

__device__ __forceinline__ uint64_t timer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
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
__device__ __forceinline__ void red_add_release_gpu(uint32_t* p, uint32_t v) {
  asm volatile("red.release.gpu.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// Epoch counters only grow, so "reached" is a signed distance test that survives wrap-around.
__device__ __forceinline__ bool reached(uint32_t seen, uint32_t want) { return (int32_t)(seen - want) >= 0; }

// Wait until *flag (written over NVLink by a peer) reaches `want`.
__device__ __forceinline__ bool wait_sys(const uint32_t* flag, uint32_t want, int* status, int code) {
  if (reached(ld_acquire_sys(flag), want)) return true;
  const uint64_t t0 = timer_ns();
  const uint64_t limit = peer_wait_limit_ns(status);
  while (true) {
#pragma unroll 1
    for (int i = 0; i < 64; ++i) {
      if (reached(ld_acquire_sys(flag), want)) return true;
      __nanosleep(200);
    }
    if (timer_ns() - t0 > limit) {
      atomicCAS(status, 0, code);
      return false;
    }
  }
}

// Same for a flag written by another CTA of this GPU.
__device__ __forceinline__ bool wait_gpu(const uint32_t* flag, uint32_t want, int* status, int code) {
  if (reached(ld_acquire_gpu(flag), want)) return true;
  const uint64_t t0 = timer_ns();
  const uint64_t limit = peer_wait_limit_ns(status);
  while (true) {
#pragma unroll 1
    for (int i = 0; i < 64; ++i) {
      if (reached(ld_acquire_gpu(flag), want)) return true;
      __nanosleep(100);
    }
    if (timer_ns() - t0 > limit) {
      atomicCAS(status, 0, code);
      return false;
    }
  }
}

}  // namespace b200comm
