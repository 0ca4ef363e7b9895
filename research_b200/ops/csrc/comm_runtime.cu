// Communication runtime for one node: device-memory arenas that every local rank can map (CUDA virtual
// memory management with POSIX file-descriptor handles), and the two pull collectives built on them.
//
//   b200c_vmm_alloc / import / free   one physical allocation per rank, exported as a descriptor that the
//                                     peers import and map read-write (the descriptor travels through the
//                                     unix-socket broker of the host library)
//   b200c_reduce_scatter_pull         out = scale * sum_r src_r  for the slice this rank owns, reading the
//                                     peers' fp32 gradient arenas over NVLink in a fixed rank order
//                                     (deterministic), with the sum of squares of the result for the
//                                     gradient norm folded into the same pass
//   b200c_all_gather_pull             every rank copies the peers' shards into its full buffer
//   b200c_mc_*                        NVLink multicast objects: one object spans the arenas of all ranks; a load
//                                     through its address returns the sum over the ranks' copies, reduced inside
//                                     the NVSwitch, and a store through it lands in every rank's copy
//   b200c_reduce_scatter_nvls         the reduce-scatter as multimem.ld_reduce loads (each rank reads its slice
//                                     once through the switch instead of one copy per peer)
//   b200c_all_gather_nvls             the all-gather as multimem.st stores of the rank's own shard
//
// Cross-GPU ordering uses per-rank flag blocks inside the arenas (comm.cuh): a kernel announces "my buffer
// holds epoch e" to every peer, waits (bounded) for the same from them before the first remote read, and
// its last CTA announces "done reading" and waits (bounded) until every peer has finished reading this
// rank's buffer, so the buffer may be overwritten as soon as the kernel has ended.
//
// Counterparts in the reference: third_party/ThunderKittens/include/types/system/vmm.cuh:15-93 (arena),
// ipc.cuh:59-139 (handle exchange), kernels/parallel/reduce_scatter/reduce_scatter.cu:8-55 and
// all_gather/all_gather.cu:8-51 (NVLS versions of the two collectives), include/types/system/vmm.cuh:95-172
// (multicast create / bind), include/common/multimem.cuh:26-134 (multimem PTX wrappers).
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include "comm.cuh"

using namespace b200comm;

namespace {

template <typename Fn>
Fn driver_fn(const char* name) {
  void* p = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint(name, &p, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess)
    return nullptr;
  return reinterpret_cast<Fn>(p);
}

struct Driver {
  CUresult (*getGranularity)(size_t*, const CUmemAllocationProp*, CUmemAllocationGranularity_flags) = nullptr;
  CUresult (*create)(CUmemGenericAllocationHandle*, size_t, const CUmemAllocationProp*, unsigned long long) = nullptr;
  CUresult (*release)(CUmemGenericAllocationHandle) = nullptr;
  CUresult (*reserve)(CUdeviceptr*, size_t, size_t, CUdeviceptr, unsigned long long) = nullptr;
  CUresult (*addressFree)(CUdeviceptr, size_t) = nullptr;
  CUresult (*map)(CUdeviceptr, size_t, size_t, CUmemGenericAllocationHandle, unsigned long long) = nullptr;
  CUresult (*unmap)(CUdeviceptr, size_t) = nullptr;
  CUresult (*setAccess)(CUdeviceptr, size_t, const CUmemAccessDesc*, size_t) = nullptr;
  CUresult (*exportHandle)(void*, CUmemGenericAllocationHandle, CUmemAllocationHandleType, unsigned long long) = nullptr;
  CUresult (*importHandle)(CUmemGenericAllocationHandle*, void*, CUmemAllocationHandleType) = nullptr;
  // NVLink multicast objects (NVSwitch); absent on drivers older than 12.1, then mc_ok stays false
  CUresult (*mcCreate)(CUmemGenericAllocationHandle*, const CUmulticastObjectProp*) = nullptr;
  CUresult (*mcAddDevice)(CUmemGenericAllocationHandle, CUdevice) = nullptr;
  CUresult (*mcBindAddr)(CUmemGenericAllocationHandle, size_t, CUdeviceptr, size_t, unsigned long long) = nullptr;
  CUresult (*mcUnbind)(CUmemGenericAllocationHandle, CUdevice, size_t, size_t) = nullptr;
  CUresult (*mcGranularity)(size_t*, const CUmulticastObjectProp*, CUmulticastGranularity_flags) = nullptr;
  bool ok = false;
  bool mc_ok = false;
};

const Driver& driver() {
  static Driver d;
  static bool tried = false;
  if (!tried) {
    tried = true;
    d.getGranularity = driver_fn<decltype(d.getGranularity)>("cuMemGetAllocationGranularity");
    d.create = driver_fn<decltype(d.create)>("cuMemCreate");
    d.release = driver_fn<decltype(d.release)>("cuMemRelease");
    d.reserve = driver_fn<decltype(d.reserve)>("cuMemAddressReserve");
    d.addressFree = driver_fn<decltype(d.addressFree)>("cuMemAddressFree");
    d.map = driver_fn<decltype(d.map)>("cuMemMap");
    d.unmap = driver_fn<decltype(d.unmap)>("cuMemUnmap");
    d.setAccess = driver_fn<decltype(d.setAccess)>("cuMemSetAccess");
    d.exportHandle = driver_fn<decltype(d.exportHandle)>("cuMemExportToShareableHandle");
    d.importHandle = driver_fn<decltype(d.importHandle)>("cuMemImportFromShareableHandle");
    d.mcCreate = driver_fn<decltype(d.mcCreate)>("cuMulticastCreate");
    d.mcAddDevice = driver_fn<decltype(d.mcAddDevice)>("cuMulticastAddDevice");
    d.mcBindAddr = driver_fn<decltype(d.mcBindAddr)>("cuMulticastBindAddr");
    d.mcUnbind = driver_fn<decltype(d.mcUnbind)>("cuMulticastUnbind");
    d.mcGranularity = driver_fn<decltype(d.mcGranularity)>("cuMulticastGetGranularity");
    d.mc_ok = d.mcCreate && d.mcAddDevice && d.mcBindAddr && d.mcUnbind && d.mcGranularity;
    d.ok = d.getGranularity && d.create && d.release && d.reserve && d.addressFree && d.map && d.unmap &&
           d.setAccess && d.exportHandle && d.importHandle;
  }
  return d;
}

typedef CUresult (*DeviceGetFn)(CUdevice*, int);
typedef CUresult (*DeviceGetAttributeFn)(int*, CUdevice_attribute, CUdevice);
CUresult no_device_get(CUdevice*, int) { return CUDA_ERROR_NOT_SUPPORTED; }
CUresult no_device_attr(int*, CUdevice_attribute, CUdevice) { return CUDA_ERROR_NOT_SUPPORTED; }
DeviceGetFn cuDeviceGetFn() {
  static DeviceGetFn fn = driver_fn<DeviceGetFn>("cuDeviceGet");
  return fn ? fn : no_device_get;
}
DeviceGetAttributeFn cuDeviceGetAttributeFn() {
  static DeviceGetAttributeFn fn = driver_fn<DeviceGetAttributeFn>("cuDeviceGetAttribute");
  return fn ? fn : no_device_attr;
}

CUmemAllocationProp arena_prop(int dev) {
  CUmemAllocationProp prop = {};
  prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
  prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  prop.location.id = dev;
  prop.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  return prop;
}

int map_rw(const Driver& d, CUmemGenericAllocationHandle h, size_t padded, int dev, void** out, size_t align = 0) {
  CUdeviceptr va = 0;
  if (d.reserve(&va, padded, align, 0, 0) != CUDA_SUCCESS) return -12;
  if (d.map(va, padded, 0, h, 0) != CUDA_SUCCESS) {
    d.addressFree(va, padded);
    return -13;
  }
  CUmemAccessDesc acc = {};
  acc.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  acc.location.id = dev;
  acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
  if (d.setAccess(va, padded, &acc, 1) != CUDA_SUCCESS) {
    d.unmap(va, padded);
    d.addressFree(va, padded);
    return -14;
  }
  *out = reinterpret_cast<void*>(va);
  return 0;
}

struct PeerPtrs {
  const void* src[kMaxPeers];
  FlagBlock* flags[kMaxPeers];
};

// Prologue shared by the pull kernels: announce, then wait for every peer's announcement.
__device__ __forceinline__ bool announce_and_wait_ready(const PeerPtrs& pp, int world, int rank, uint32_t epoch,
                                                        int* status, int* s_ok) {
  if (threadIdx.x == 0) *s_ok = 1;
  __syncthreads();
  if (blockIdx.x == 0 && threadIdx.x < world && (int)threadIdx.x != rank) {
    __threadfence_system();
    st_release_sys(&pp.flags[threadIdx.x]->ready[rank], epoch);
  }
  if (threadIdx.x < world && (int)threadIdx.x != rank) {
    if (!wait_sys(&pp.flags[rank]->ready[threadIdx.x], epoch, status, ERR_PEER_READY)) *s_ok = 0;
  }
  __syncthreads();
  return *s_ok != 0;
}

// Epilogue: the CTA that finishes last tells every peer that this rank is done reading, then waits until every
// peer is done reading this rank's buffer.  `counter` must be zero on entry and is left zero.
__device__ __forceinline__ void finish_and_wait_done(const PeerPtrs& pp, int world, int rank, uint32_t epoch,
                                                     uint32_t* counter, int* status) {
  __shared__ int s_last;
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    s_last = atomicAdd(counter, 1u) == gridDim.x - 1;
  }
  __syncthreads();
  if (!s_last) return;
  if (threadIdx.x < world && (int)threadIdx.x != rank) {
    __threadfence_system();  // orders the other CTAs' work (seen through the counter) before the flag store
    st_release_sys(&pp.flags[threadIdx.x]->done[rank], epoch);
    wait_sys(&pp.flags[rank]->done[threadIdx.x], epoch, status, ERR_PEER_DONE);
  }
  if (threadIdx.x == 0) *counter = 0u;
}

__global__ void __launch_bounds__(512)
reduce_scatter_pull_kernel(const PeerPtrs pp, float* __restrict__ out, long long n4, float scale,
                           float* __restrict__ sumsq, float* __restrict__ partials, uint32_t* counter, int world,
                           int rank, uint32_t epoch, int* status) {
  __shared__ int s_ok;
  __shared__ float s_red[16];
  const bool ok = announce_and_wait_ready(pp, world, rank, epoch, status, &s_ok);
  float ss = 0.f;
  if (ok) {
    float4* o4 = reinterpret_cast<float4*>(out);
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (long long)gridDim.x * blockDim.x) {
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int r = 0; r < kMaxPeers; ++r) {
        if (r < world) {
          const float4 v = reinterpret_cast<const float4*>(pp.src[r])[i];
          acc.x += v.x;
          acc.y += v.y;
          acc.z += v.z;
          acc.w += v.w;
        }
      }
      acc.x *= scale;
      acc.y *= scale;
      acc.z *= scale;
      acc.w *= scale;
      o4[i] = acc;
      ss += acc.x * acc.x + acc.y * acc.y + acc.z * acc.z + acc.w * acc.w;
    }
  }
  // deterministic sum of squares: per-CTA partials, added up in CTA order by the last CTA (below)
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, off);
  if ((threadIdx.x & 31) == 0) s_red[threadIdx.x >> 5] = ss;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
    for (int w = 0; w < (int)(blockDim.x >> 5); ++w) t += s_red[w];
    partials[blockIdx.x] = t;
  }
  __shared__ int s_last;
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    s_last = atomicAdd(counter, 1u) == gridDim.x - 1;
  }
  __syncthreads();
  if (!s_last) return;
  if (threadIdx.x == 0) {
    __threadfence();
    if (sumsq) {
      float t = 0.f;
      for (unsigned b = 0; b < gridDim.x; ++b) t += reinterpret_cast<volatile float*>(partials)[b];
      *sumsq += t;
    }
    *counter = 0u;
  }
  if (threadIdx.x < world && (int)threadIdx.x != rank) {
    st_release_sys(&pp.flags[threadIdx.x]->done[rank], epoch);
    wait_sys(&pp.flags[rank]->done[threadIdx.x], epoch, status, ERR_PEER_DONE);
  }
}

__global__ void __launch_bounds__(512)
all_gather_pull_kernel(const PeerPtrs pp, uint4* __restrict__ dst, long long n16_per_rank, uint32_t* counter,
                       int world, int rank, uint32_t epoch, int copy_self, int* status) {
  __shared__ int s_ok;
  const bool ok = announce_and_wait_ready(pp, world, rank, epoch, status, &s_ok);
  if (ok) {
    const long long total = n16_per_rank * world;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
      // start each rank at a different peer so that the pulls spread over the links
      const int r = (int)((i / n16_per_rank + rank + 1) % world);
      const long long j = i % n16_per_rank;
      if (r == rank && !copy_self) continue;
      dst[(long long)r * n16_per_rank + j] = reinterpret_cast<const uint4*>(pp.src[r])[j];
    }
  }
  finish_and_wait_done(pp, world, rank, epoch, counter, status);
}

// ---- multimem PTX wrappers (NVLink multicast addresses only) -----------------------------------------------
// Sum over every rank's copy of four consecutive floats, reduced in the switch.
__device__ __forceinline__ float4 multimem_ld_reduce_add_f32x4(const float* mc_addr) {
  float4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "l"(mc_addr)
               : "memory");
  return v;
}
// Store 16 bytes into every rank's copy.
__device__ __forceinline__ void multimem_st_b32x4(void* mc_addr, const uint4& v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc_addr), "f"(__uint_as_float(v.x)),
               "f"(__uint_as_float(v.y)), "f"(__uint_as_float(v.z)), "f"(__uint_as_float(v.w))
               : "memory");
}

// Tail of the reducing kernels: per-CTA partial sums of squares are added in CTA order by the CTA that finishes
// last (deterministic), which also runs the "done" handshake with the peers.
__device__ __forceinline__ void finish_reduce(const PeerPtrs& pp, float ss, float* sumsq, float* partials,
                                              uint32_t* counter, int world, int rank, uint32_t epoch, int* status) {
  __shared__ float s_red[16];
  __shared__ int s_last;
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, off);
  if ((threadIdx.x & 31) == 0) s_red[threadIdx.x >> 5] = ss;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
    for (int w = 0; w < (int)(blockDim.x >> 5); ++w) t += s_red[w];
    partials[blockIdx.x] = t;
    __threadfence();
    s_last = atomicAdd(counter, 1u) == gridDim.x - 1;
  }
  __syncthreads();
  if (!s_last) return;
  if (threadIdx.x == 0) {
    __threadfence();
    if (sumsq) {
      float t = 0.f;
      for (unsigned b = 0; b < gridDim.x; ++b) t += reinterpret_cast<volatile float*>(partials)[b];
      *sumsq += t;
    }
    *counter = 0u;
  }
  if (threadIdx.x < world && (int)threadIdx.x != rank) {
    st_release_sys(&pp.flags[threadIdx.x]->done[rank], epoch);
    wait_sys(&pp.flags[rank]->done[threadIdx.x], epoch, status, ERR_PEER_DONE);
  }
}

// out = scale * (sum over ranks of the slice at mc_src), one multimem.ld_reduce per 16 bytes.
__global__ void __launch_bounds__(512)
reduce_scatter_nvls_kernel(const PeerPtrs pp, const float* __restrict__ mc_src, float* __restrict__ out, long long n4,
                           float scale, float* __restrict__ sumsq, float* __restrict__ partials, uint32_t* counter,
                           int world, int rank, uint32_t epoch, int* status) {
  __shared__ int s_ok;
  const bool ok = announce_and_wait_ready(pp, world, rank, epoch, status, &s_ok);
  float ss = 0.f;
  if (ok) {
    float4* o4 = reinterpret_cast<float4*>(out);
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (long long)gridDim.x * blockDim.x) {
      float4 acc = multimem_ld_reduce_add_f32x4(mc_src + 4 * i);
      acc.x *= scale;
      acc.y *= scale;
      acc.z *= scale;
      acc.w *= scale;
      o4[i] = acc;
      ss += acc.x * acc.x + acc.y * acc.y + acc.z * acc.z + acc.w * acc.w;
    }
  }
  finish_reduce(pp, ss, sumsq, partials, counter, world, rank, epoch, status);
}

// Every rank stores its own shard through the multicast address: one store per 16 bytes reaches all ranks.
__global__ void __launch_bounds__(512)
all_gather_nvls_kernel(const PeerPtrs pp, const uint4* __restrict__ own, uint4* __restrict__ mc_dst, long long n16,
                       uint32_t* counter, int world, int rank, uint32_t epoch, int* status) {
  __shared__ int s_ok;
  // "ready" here means: the peer has reached this collective, so its buffer may be overwritten
  const bool ok = announce_and_wait_ready(pp, world, rank, epoch, status, &s_ok);
  if (ok) {
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n16; i += (long long)gridDim.x * blockDim.x)
      multimem_st_b32x4(mc_dst + i, own[i]);
  }
  __threadfence_system();  // this CTA's stores are performed at every rank before its count below
  // "done" here means: all of this rank's stores have landed; every rank leaves with every shard in place
  finish_and_wait_done(pp, world, rank, epoch, counter, status);
}

// Plain copies of up to a few dozen byte ranges in one launch (sources may be peers' arenas).  No flags: the caller
// orders the launch after whatever wrote the sources (a barrier over the ranks, stream order locally).
struct CopyPiece {
  const void* src;
  void* dst;
  long long bytes;
};
__global__ void __launch_bounds__(256) copy_pieces_kernel(const CopyPiece* __restrict__ pieces) {
  const CopyPiece pc = pieces[blockIdx.y];
  const long long n16 = pc.bytes >> 4;
  const uint4* s = reinterpret_cast<const uint4*>(pc.src);
  uint4* d = reinterpret_cast<uint4*>(pc.dst);
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n16; i += (long long)gridDim.x * blockDim.x)
    d[i] = s[i];
  if (blockIdx.x == 0) {   // the last bytes of a range whose length is not a multiple of 16
    const long long tail = pc.bytes & 15;
    if ((long long)threadIdx.x < tail)
      reinterpret_cast<uint8_t*>(pc.dst)[(n16 << 4) + threadIdx.x] =
          reinterpret_cast<const uint8_t*>(pc.src)[(n16 << 4) + threadIdx.x];
  }
}

// Barrier over the ranks of an arena: announce epoch, wait (bounded) for everybody else's announcement.
__global__ void peer_barrier_kernel(const PeerPtrs pp, int world, int rank, uint32_t epoch, int* status) {
  if (threadIdx.x < world && (int)threadIdx.x != rank) {
    __threadfence_system();
    st_release_sys(&pp.flags[threadIdx.x]->ready[rank], epoch);
    wait_sys(&pp.flags[rank]->ready[threadIdx.x], epoch, status, ERR_PEER_READY);
  }
}

// `max_ctas` > 0 caps the grid: a collective that runs beside compute kernels on another stream leaves them the
// rest of the machine (a few dozen CTAs keep the NVLink ports busy).
int grid_for_bytes(long long items, int block, int max_ctas = 0) {
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  long long b = (items + block - 1) / block;
  long long cap = (long long)sms * 2;
  if (max_ctas > 0 && max_ctas < cap) cap = max_ctas;
  if (b > cap) b = cap;
  return b < 1 ? 1 : (int)b;
}

}  // namespace

extern "C" {

// Allocates `bytes` (rounded up to the allocation granularity, returned in *padded) of device memory on the
// current device, mapped read-write, and exports it as a POSIX file descriptor in *fd (the caller closes it).
// `align` (0 = none, else a power of two): the size is also rounded up to it and the virtual address is aligned to
// it, which is what binding the arena to a multicast object asks for (b200c_mc_granularity).
int b200c_vmm_alloc(unsigned long long bytes, unsigned long long align, void** ptr, int* fd,
                    unsigned long long* padded) {
  const Driver& d = driver();
  if (!d.ok) return -3;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return -10;
  cudaFree(nullptr);  // make sure the primary context exists
  CUmemAllocationProp prop = arena_prop(dev);
  size_t gran = 0;
  if (d.getGranularity(&gran, &prop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED) != CUDA_SUCCESS || gran == 0) return -11;
  if (align > gran) {
    if (align % gran) return -2;
    gran = static_cast<size_t>(align);
  }
  const size_t size = (static_cast<size_t>(bytes) + gran - 1) / gran * gran;
  CUmemGenericAllocationHandle h;
  if (d.create(&h, size, &prop, 0) != CUDA_SUCCESS) return -15;
  int rc = map_rw(d, h, size, dev, ptr, gran);
  if (rc == 0) {
    int out_fd = -1;
    if (d.exportHandle(&out_fd, h, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0) != CUDA_SUCCESS) {
      d.unmap(reinterpret_cast<CUdeviceptr>(*ptr), size);
      d.addressFree(reinterpret_cast<CUdeviceptr>(*ptr), size);
      rc = -16;
    } else {
      *fd = out_fd;
      *padded = size;
    }
  }
  d.release(h);  // the mapping keeps the memory alive
  return rc;
}

// Maps a peer's allocation (descriptor received through the broker) read-write into this process.
int b200c_vmm_import(int fd, unsigned long long padded, void** ptr) {
  const Driver& d = driver();
  if (!d.ok) return -3;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return -10;
  cudaFree(nullptr);
  CUmemGenericAllocationHandle h;
  if (d.importHandle(&h, reinterpret_cast<void*>(static_cast<uintptr_t>(fd)), CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR) !=
      CUDA_SUCCESS)
    return -17;
  const int rc = map_rw(d, h, static_cast<size_t>(padded), dev, ptr);
  d.release(h);
  return rc;
}

int b200c_vmm_free(void* ptr, unsigned long long padded) {
  const Driver& d = driver();
  if (!d.ok) return -3;
  if (d.unmap(reinterpret_cast<CUdeviceptr>(ptr), static_cast<size_t>(padded)) != CUDA_SUCCESS) return -18;
  if (d.addressFree(reinterpret_cast<CUdeviceptr>(ptr), static_cast<size_t>(padded)) != CUDA_SUCCESS) return -19;
  return 0;
}

int b200c_flag_block_bytes() { return static_cast<int>(sizeof(FlagBlock)); }

// All ranks call this with the same epoch on the same channel; work queued before it on every rank's stream has
// completed (and its peer-memory writes are visible) when work queued after it starts.
int b200c_barrier(void* const* flags, int world, int rank, unsigned epoch, int* status, void* stream) {
  if (world < 1 || world > kMaxPeers || rank < 0 || rank >= world) return -2;
  PeerPtrs pp = {};
  for (int r = 0; r < world; ++r) {
    if (!flags[r]) return -1;
    pp.flags[r] = static_cast<FlagBlock*>(flags[r]);
  }
  peer_barrier_kernel<<<1, 32, 0, reinterpret_cast<cudaStream_t>(stream)>>>(pp, world, rank, epoch, status);
  return static_cast<int>(cudaGetLastError());
}

// src[r]: rank r's copy of the slice this rank owns (n fp32, n % 4 == 0, 16-byte aligned); flags[r]: rank r's
// flag block of this channel, as mapped here.  scratch: uint32 counter (zero) followed by >= 512 floats.
// n may be 0: the kernel then only takes part in the handshake (ranks may own slices of different sizes).
// max_ctas > 0 caps the grid (for launches that overlap compute kernels).
int b200c_reduce_scatter_pull(const void* const* src, void* out, long long n, float scale, void* sumsq,
                              void* const* flags, int world, int rank, unsigned epoch, int max_ctas, void* scratch,
                              int* status, void* stream) {
  if (world < 1 || world > kMaxPeers || rank < 0 || rank >= world || n < 0 || (n & 3)) return -2;
  PeerPtrs pp = {};
  for (int r = 0; r < world; ++r) {
    if ((reinterpret_cast<uintptr_t>(src[r]) & 15) || !flags[r]) return -1;
    pp.src[r] = src[r];
    pp.flags[r] = static_cast<FlagBlock*>(flags[r]);
  }
  if (reinterpret_cast<uintptr_t>(out) & 15) return -1;
  uint32_t* counter = static_cast<uint32_t*>(scratch);
  float* partials = reinterpret_cast<float*>(counter + 4);
  const int grid = grid_for_bytes(n / 4, 512, max_ctas);
  reduce_scatter_pull_kernel<<<grid, 512, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      pp, static_cast<float*>(out), n / 4, scale, static_cast<float*>(sumsq), partials, counter, world, rank, epoch,
      status);
  return static_cast<int>(cudaGetLastError());
}

// The same reduction through the multicast mapping: mc_src is the multicast address of the slice this rank owns.
int b200c_reduce_scatter_nvls(const void* mc_src, void* out, long long n, float scale, void* sumsq,
                              void* const* flags, int world, int rank, unsigned epoch, int max_ctas, void* scratch,
                              int* status, void* stream) {
  if (world < 1 || world > kMaxPeers || rank < 0 || rank >= world || n < 0 || (n & 3)) return -2;
  if (!mc_src || (reinterpret_cast<uintptr_t>(mc_src) & 15) || (reinterpret_cast<uintptr_t>(out) & 15)) return -1;
  PeerPtrs pp = {};
  for (int r = 0; r < world; ++r) {
    if (!flags[r]) return -1;
    pp.flags[r] = static_cast<FlagBlock*>(flags[r]);
  }
  uint32_t* counter = static_cast<uint32_t*>(scratch);
  float* partials = reinterpret_cast<float*>(counter + 4);
  const int grid = grid_for_bytes(n / 4, 512, max_ctas);
  reduce_scatter_nvls_kernel<<<grid, 512, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      pp, static_cast<const float*>(mc_src), static_cast<float*>(out), n / 4, scale, static_cast<float*>(sumsq),
      partials, counter, world, rank, epoch, status);
  return static_cast<int>(cudaGetLastError());
}

// own: this rank's shard (local address); mc_dst: the multicast address of the place of that shard in the full
// buffer.  When the kernel has ended, every rank's buffer holds every shard.
int b200c_all_gather_nvls(const void* own, void* mc_dst, long long bytes_per_rank, void* const* flags, int world,
                          int rank, unsigned epoch, void* scratch, int* status, void* stream) {
  if (world < 1 || world > kMaxPeers || rank < 0 || rank >= world || bytes_per_rank <= 0 || (bytes_per_rank & 15))
    return -2;
  if (!mc_dst || (reinterpret_cast<uintptr_t>(own) & 15) || (reinterpret_cast<uintptr_t>(mc_dst) & 15)) return -1;
  PeerPtrs pp = {};
  for (int r = 0; r < world; ++r) {
    if (!flags[r]) return -1;
    pp.flags[r] = static_cast<FlagBlock*>(flags[r]);
  }
  const long long n16 = bytes_per_rank / 16;
  const int grid = grid_for_bytes(n16, 512);
  all_gather_nvls_kernel<<<grid, 512, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      pp, static_cast<const uint4*>(own), static_cast<uint4*>(mc_dst), n16, static_cast<uint32_t*>(scratch), world,
      rank, epoch, status);
  return static_cast<int>(cudaGetLastError());
}

// table: device array of n_pieces {src, dst, bytes} records (16-byte aligned addresses).  Used to bring the weight
// shards of one layer from their owners' arenas into the local layer buffer.
int b200c_copy_pieces(const void* table, int n_pieces, int ctas_per_piece, void* stream) {
  if (!table || n_pieces <= 0 || n_pieces > 65535 || ctas_per_piece <= 0) return -2;
  copy_pieces_kernel<<<dim3(ctas_per_piece, n_pieces), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      static_cast<const CopyPiece*>(table));
  return static_cast<int>(cudaGetLastError());
}

// ---- NVLink multicast objects ---------------------------------------------------------------------------------
// 1 when the current device and the driver support multicast objects.
int b200c_mc_supported() {
  const Driver& d = driver();
  if (!d.ok || !d.mc_ok) return 0;
  int dev = 0, flag = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return 0;
  CUdevice cudev;
  if (cuDeviceGetFn()(&cudev, dev) != CUDA_SUCCESS) return 0;
  if (cuDeviceGetAttributeFn()(&flag, CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED, cudev) != CUDA_SUCCESS) return 0;
  return flag ? 1 : 0;
}

// Granularity (bytes) that sizes, offsets and addresses bound to a multicast object of `world` devices should be
// multiples of; 0 when multicast is unavailable.
unsigned long long b200c_mc_granularity(int world, unsigned long long bytes) {
  const Driver& d = driver();
  if (!d.mc_ok) return 0;
  CUmulticastObjectProp prop = {};
  prop.numDevices = static_cast<unsigned>(world);
  prop.size = static_cast<size_t>(bytes);
  prop.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  size_t gran = 0;
  if (d.mcGranularity(&gran, &prop, CU_MULTICAST_GRANULARITY_RECOMMENDED) != CUDA_SUCCESS) return 0;
  return gran;
}

// One rank creates the object (bytes = the arena size, a multiple of the granularity) and exports it as a file
// descriptor for the others; *handle is this process's reference.
int b200c_mc_create(unsigned long long bytes, int world, int* fd, unsigned long long* handle) {
  const Driver& d = driver();
  if (!d.ok || !d.mc_ok) return -3;
  cudaFree(nullptr);
  CUmulticastObjectProp prop = {};
  prop.numDevices = static_cast<unsigned>(world);
  prop.size = static_cast<size_t>(bytes);
  prop.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  CUmemGenericAllocationHandle h;
  CUresult r = d.mcCreate(&h, &prop);
  if (r != CUDA_SUCCESS) return -20 - 1000 * static_cast<int>(r);
  int out_fd = -1;
  if (d.exportHandle(&out_fd, h, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0) != CUDA_SUCCESS) {
    d.release(h);
    return -21;
  }
  *fd = out_fd;
  *handle = static_cast<unsigned long long>(h);
  return 0;
}

int b200c_mc_import(int fd, unsigned long long* handle) {
  const Driver& d = driver();
  if (!d.ok || !d.mc_ok) return -3;
  cudaFree(nullptr);
  CUmemGenericAllocationHandle h;
  if (d.importHandle(&h, reinterpret_cast<void*>(static_cast<uintptr_t>(fd)), CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR) !=
      CUDA_SUCCESS)
    return -22;
  *handle = static_cast<unsigned long long>(h);
  return 0;
}

// Every rank adds its device; binding may start only after all ranks have done so.
int b200c_mc_add_device(unsigned long long handle) {
  const Driver& d = driver();
  if (!d.mc_ok) return -3;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return -10;
  CUdevice cudev;
  if (cuDeviceGetFn()(&cudev, dev) != CUDA_SUCCESS) return -10;
  CUresult r = d.mcAddDevice(static_cast<CUmemGenericAllocationHandle>(handle), cudev);
  return r == CUDA_SUCCESS ? 0 : -23 - 1000 * static_cast<int>(r);
}

// Binds this rank's arena (local_ptr, bytes) at offset 0 of the object and maps the object read-write; *mc_ptr is
// the multicast address that corresponds to local_ptr.
int b200c_mc_bind_and_map(unsigned long long handle, void* local_ptr, unsigned long long bytes, void** mc_ptr) {
  const Driver& d = driver();
  if (!d.ok || !d.mc_ok) return -3;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return -10;
  const CUmemGenericAllocationHandle h = static_cast<CUmemGenericAllocationHandle>(handle);
  CUresult r = d.mcBindAddr(h, 0, reinterpret_cast<CUdeviceptr>(local_ptr), static_cast<size_t>(bytes), 0);
  if (r != CUDA_SUCCESS) return -24 - 1000 * static_cast<int>(r);
  const int rc = map_rw(d, h, static_cast<size_t>(bytes), dev, mc_ptr, 0);
  if (rc != 0) {
    CUdevice cudev;
    if (cuDeviceGetFn()(&cudev, dev) == CUDA_SUCCESS) d.mcUnbind(h, cudev, 0, static_cast<size_t>(bytes));
  }
  return rc;
}

// Unmaps the multicast address, unbinds this rank's memory and drops the reference.  Call it with no kernel in
// flight on any rank that still uses the mapping.
int b200c_mc_release(unsigned long long handle, void* mc_ptr, unsigned long long bytes) {
  const Driver& d = driver();
  if (!d.ok || !d.mc_ok) return -3;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return -10;
  const CUmemGenericAllocationHandle h = static_cast<CUmemGenericAllocationHandle>(handle);
  int rc = 0;
  if (mc_ptr) {
    if (d.unmap(reinterpret_cast<CUdeviceptr>(mc_ptr), static_cast<size_t>(bytes)) != CUDA_SUCCESS) rc = -18;
    if (d.addressFree(reinterpret_cast<CUdeviceptr>(mc_ptr), static_cast<size_t>(bytes)) != CUDA_SUCCESS) rc = -19;
    CUdevice cudev;
    if (cuDeviceGetFn()(&cudev, dev) == CUDA_SUCCESS &&
        d.mcUnbind(h, cudev, 0, static_cast<size_t>(bytes)) != CUDA_SUCCESS)
      rc = -25;
  }
  d.release(h);
  return rc;
}

// src[r]: rank r's shard (bytes_per_rank bytes, multiple of 16); dst: this rank's full buffer of world shards.
// copy_self = 0 when this rank's shard already sits at its place in dst.
int b200c_all_gather_pull(const void* const* src, void* dst, long long bytes_per_rank, void* const* flags, int world,
                          int rank, unsigned epoch, int copy_self, void* scratch, int* status, void* stream) {
  if (world < 1 || world > kMaxPeers || rank < 0 || rank >= world || bytes_per_rank <= 0 || (bytes_per_rank & 15))
    return -2;
  PeerPtrs pp = {};
  for (int r = 0; r < world; ++r) {
    if ((reinterpret_cast<uintptr_t>(src[r]) & 15) || !flags[r]) return -1;
    pp.src[r] = src[r];
    pp.flags[r] = static_cast<FlagBlock*>(flags[r]);
  }
  if (reinterpret_cast<uintptr_t>(dst) & 15) return -1;
  const long long n16 = bytes_per_rank / 16;
  const int grid = grid_for_bytes(n16 * world, 512);
  all_gather_pull_kernel<<<grid, 512, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      pp, static_cast<uint4*>(dst), n16, static_cast<uint32_t*>(scratch), world, rank, epoch, copy_self, status);
  return static_cast<int>(cudaGetLastError());
}

}  // extern "C"
