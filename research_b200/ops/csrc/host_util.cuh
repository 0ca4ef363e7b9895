// Host-side helpers shared by the launchers: tensor-map encoding through the driver entry point
// (no link-time dependency on libcuda), device attribute cache, error plumbing.
#pragma once
#include <stdlib.h>
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

namespace b200host {

// launcher return codes (negative = host-side rejection, positive = cudaError_t)
enum : int {
  RC_OK = 0,
  RC_BAD_ALIGNMENT = -1,
  RC_BAD_SHAPE = -2,
  RC_NO_DRIVER_ENTRY = -3,
  RC_TENSORMAP_FAILED = -4,
  RC_TOO_LARGE = -5,
  RC_SYMBOL_FAILED = -6,
};

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

inline int sm_count() {
  static int n[16] = {0};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 16) dev = 0;
  if (n[dev] == 0) cudaDeviceGetAttribute(&n[dev], cudaDevAttrMultiProcessorCount, dev);
  return n[dev];
}

// The opt-in to more than 48 KB of dynamic shared memory is an attribute of (function, device).  `done` is the
// caller's per-kernel table (one static table per template instantiation), indexed by the current device, so a
// process that drives several GPUs configures the kernel on each of them.  Devices beyond the table are
// configured on every launch.
constexpr int kMaxDevices = 64;
template <typename Kern>
inline int ensure_dynamic_smem(Kern* kern, int bytes, bool (&done)[kMaxDevices]) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return static_cast<int>(cudaGetLastError());
  const bool tracked = dev >= 0 && dev < kMaxDevices;
  if (tracked && done[dev]) return 0;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
  if (e != cudaSuccess) return static_cast<int>(e);
  if (tracked) done[dev] = true;
  return 0;
}

// RESEARCH_B200_PDL=0 turns programmatic dependent launch off for the kernels of a decode step that use it.
inline int pdl_enabled() {
  static const int on = [] {
    const char* v = getenv("RESEARCH_B200_PDL");
    return (v && v[0] == '0') ? 0 : 1;
  }();
  return on;
}

// Launch with programmatic dependent launch when `pdl` is set: the kernel may become resident while its predecessor
// in the stream is still running, and everything it reads or writes that the predecessor also touches must come
// after its `griddepcontrol.wait` (b200.cuh: pdl_wait), which returns when the predecessor has completed.  A
// predecessor lets this happen early by executing `griddepcontrol.launch_dependents` (pdl_launch_dependents) in
// every CTA; without it the dependent launch begins when the predecessor's last CTA has exited.
template <typename... KArgs, typename... Args>
inline cudaError_t launch_kernel(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                 bool pdl, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);
}

// Rank-3 row-major tensor [d2][d1][d0] (d0 innermost) with byte strides s1 (between d1 rows) and
// s2 (between d2 slabs); box {b0, b1, 1}; 128-byte swizzle; zero fill out of bounds.
inline int make_map_3d(CUtensorMap* out, CUtensorMapDataType dt, const void* base, uint64_t d0, uint64_t d1,
                       uint64_t d2, uint64_t s1_bytes, uint64_t s2_bytes, uint32_t b0, uint32_t b1,
                       CUtensorMapSwizzle swz = CU_TENSOR_MAP_SWIZZLE_128B) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return RC_NO_DRIVER_ENTRY;
  if ((reinterpret_cast<uintptr_t>(base) & 15) || (s1_bytes & 15) || (s2_bytes & 15)) return RC_BAD_ALIGNMENT;
  cuuint64_t dims[3] = {d0, d1, d2 ? d2 : 1};
  cuuint64_t strides[2] = {s1_bytes, s2_bytes ? s2_bytes : s1_bytes * d1};
  cuuint32_t box[3] = {b0, b1, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(out, dt, 3, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swz,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    fprintf(stderr,
            "research_b200: cuTensorMapEncodeTiled failed (%d) dims=(%llu,%llu,%llu) strides=(%llu,%llu) box=(%u,%u)\n",
            (int)r, (unsigned long long)dims[0], (unsigned long long)dims[1], (unsigned long long)dims[2],
            (unsigned long long)strides[0], (unsigned long long)strides[1], b0, b1);
    return RC_TENSORMAP_FAILED;
  }
  return RC_OK;
}

// Rank-4 tensor [d3][d2][d1][d0] with byte strides s1 <= s2 <= s3 (each a multiple of the one before,
// which is why attention orders its dims as head_dim, head, token, batch); box {b0, b1, b2, 1}.
inline int make_map_4d(CUtensorMap* out, CUtensorMapDataType dt, const void* base, uint64_t d0, uint64_t d1,
                       uint64_t d2, uint64_t d3, uint64_t s1_bytes, uint64_t s2_bytes, uint64_t s3_bytes, uint32_t b0,
                       uint32_t b1, uint32_t b2, CUtensorMapSwizzle swz = CU_TENSOR_MAP_SWIZZLE_128B) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return RC_NO_DRIVER_ENTRY;
  if ((reinterpret_cast<uintptr_t>(base) & 15) || (s1_bytes & 15) || (s2_bytes & 15) || (s3_bytes & 15))
    return RC_BAD_ALIGNMENT;
  cuuint64_t dims[4] = {d0, d1, d2, d3};
  cuuint64_t strides[3] = {s1_bytes, s2_bytes, s3_bytes};
  cuuint32_t box[4] = {b0, b1, b2, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = fn(out, dt, 4, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swz,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    fprintf(stderr,
            "research_b200: cuTensorMapEncodeTiled(4d) failed (%d) dims=(%llu,%llu,%llu,%llu) strides=(%llu,%llu,%llu)\n",
            (int)r, (unsigned long long)d0, (unsigned long long)d1, (unsigned long long)d2, (unsigned long long)d3,
            (unsigned long long)s1_bytes, (unsigned long long)s2_bytes, (unsigned long long)s3_bytes);
    return RC_TENSORMAP_FAILED;
  }
  return RC_OK;
}

}  // namespace b200host
