// Dion2's element-wise and selection stages for sm_100a (rules restated from the reference transform,
// src/jaxtitan/optim/dion2.py:34-125).  A parameter is a batch of `n` row-major fp32 matrices [rows, cols], `stride`
// elements apart (row ranges of a fused storage entry, or the experts of a stack).  One update touches each
// matrix twice, with a small selection kernel and the batched Polar-Express GEMMs in between:
//
//   1. accumulate: m <- m + clip * g; per slice (row or column, chosen by `axis`) the L1 norm of m and the sum of
//                  squares of bf16(m), as `splits` partial sums for column slices;
//   2. select:     every slice's rank by (norm descending, index ascending); the first k ranks are the selected
//                  slices: idx[b, rank], inv[b, slice] = rank or -1, sq_sel[b, rank];
//   3. gather:     stack[b] = bf16(selected slices) / (bf16(1.02 * bf16(||.||_F)) + eps), the dense bf16 input
//                  of the orthogonaliser, in rank order;
//   4. apply:      w <- w * decay - step * o on the selected slices (decay everywhere), m <- ef * m on the
//                  selected slices, compute copy <- bf16(w).
//
// Nothing here uses atomics or arrival order: the same inputs give the same bits.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace {

constexpr int kWarps = 8;
constexpr int kThreads = kWarps * 32;

__device__ __forceinline__ float bf16_round(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// ---- 1. accumulate + slice norms -------------------------------------------------------------------------
// Row slices: one warp per row.  grid = (ceil(rows / kWarps), n).
__global__ void dion2_accumulate_rows_kernel(const float* __restrict__ g_all, float* __restrict__ m_all,
                                             const float* __restrict__ clip, float* __restrict__ l1,
                                             float* __restrict__ sq, int rows, int cols, long long stride) {
  const int b = blockIdx.y;
  const int row = blockIdx.x * kWarps + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int lane = threadIdx.x & 31;
  const float c = clip ? clip[0] : 1.f;
  const float4* g = reinterpret_cast<const float4*>(g_all + b * stride + (long long)row * cols);
  float4* m = reinterpret_cast<float4*>(m_all + b * stride + (long long)row * cols);
  float a1 = 0.f, a2 = 0.f;
  for (int i = lane; i < (cols >> 2); i += 32) {
    const float4 gv = g[i];
    float4 mv = m[i];
    mv.x += c * gv.x; mv.y += c * gv.y; mv.z += c * gv.z; mv.w += c * gv.w;
    m[i] = mv;
    a1 += fabsf(mv.x) + fabsf(mv.y) + fabsf(mv.z) + fabsf(mv.w);
    const float r0 = bf16_round(mv.x), r1 = bf16_round(mv.y), r2 = bf16_round(mv.z), r3 = bf16_round(mv.w);
    a2 += r0 * r0 + r1 * r1 + r2 * r2 + r3 * r3;
  }
  a1 = warp_sum(a1);
  a2 = warp_sum(a2);
  if (lane == 0) {
    l1[(long long)b * rows + row] = a1;
    sq[(long long)b * rows + row] = a2;
  }
}

// Column slices: a block owns a strip of 128 columns and one of `splits` row ranges; its 8 warps take rows
// round-robin (512 contiguous bytes per row and warp).  grid = (ceil(cols / 128), n, splits); the partial sums
// land in l1 / sq [split, b, col].
__global__ void dion2_accumulate_cols_kernel(const float* __restrict__ g_all, float* __restrict__ m_all,
                                             const float* __restrict__ clip, float* __restrict__ l1,
                                             float* __restrict__ sq, int rows, int cols, long long stride,
                                             int rows_per_split, int n) {
  __shared__ float red1[kWarps][128];
  __shared__ float red2[kWarps][128];
  const int b = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int col = blockIdx.x * 128 + lane * 4;
  const int r_lo = blockIdx.z * rows_per_split;
  const int r_hi = min(rows, r_lo + rows_per_split);
  const float c = clip ? clip[0] : 1.f;
  float a1[4] = {0.f, 0.f, 0.f, 0.f}, a2[4] = {0.f, 0.f, 0.f, 0.f};
  if (col < cols) {
    const float* g = g_all + b * stride + col;
    float* m = m_all + b * stride + col;
    for (int r = r_lo + warp; r < r_hi; r += kWarps) {
      const float4 gv = *reinterpret_cast<const float4*>(g + (long long)r * cols);
      float4 mv = *reinterpret_cast<float4*>(m + (long long)r * cols);
      mv.x += c * gv.x; mv.y += c * gv.y; mv.z += c * gv.z; mv.w += c * gv.w;
      *reinterpret_cast<float4*>(m + (long long)r * cols) = mv;
      const float v[4] = {mv.x, mv.y, mv.z, mv.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        a1[j] += fabsf(v[j]);
        const float q = bf16_round(v[j]);
        a2[j] += q * q;
      }
    }
  }
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    red1[warp][lane * 4 + j] = a1[j];
    red2[warp][lane * 4 + j] = a2[j];
  }
  __syncthreads();
  if (threadIdx.x < 128) {
    const int cc = blockIdx.x * 128 + threadIdx.x;
    if (cc < cols) {
      float s1 = 0.f, s2 = 0.f;
#pragma unroll
      for (int w = 0; w < kWarps; ++w) {
        s1 += red1[w][threadIdx.x];
        s2 += red2[w][threadIdx.x];
      }
      const long long o = ((long long)blockIdx.z * n + b) * cols + cc;
      l1[o] = s1;
      sq[o] = s2;
    }
  }
}

// ---- 2. selection ------------------------------------------------------------------------------------------
// Rank by counting: slice i's rank is the number of slices that come before it in (norm descending, index
// ascending) order.  Every block holds the matrix's whole norm vector in shared memory and ranks 256 slices.
// grid = (ceil(dim / 256), n), dynamic shared memory = dim_pad floats (dim rounded up to 4).
__global__ void dion2_select_kernel(const float* __restrict__ l1, const float* __restrict__ sq, int splits, int n,
                                    int dim, int k, int* __restrict__ idx, int* __restrict__ inv,
                                    float* __restrict__ sq_sel) {
  extern __shared__ float vals[];
  const int b = blockIdx.y;
  const int dim_pad = (dim + 3) & ~3;
  for (int i = threadIdx.x; i < dim_pad; i += blockDim.x) {
    float v = -1.f;                                   // padding sorts after every real norm (norms are >= 0)
    if (i < dim) {
      v = 0.f;
      for (int s = 0; s < splits; ++s) v += l1[((long long)s * n + b) * dim + i];
      if (!(v == v)) v = 3.4e38f;                     // NaN: keep the order total so that ranks stay a permutation
    }
    vals[i] = v;
  }
  __syncthreads();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= dim) return;
  const float v = vals[i];
  int rank = 0;
  for (int j = 0; j < dim_pad; j += 4) {
    const float4 o = *reinterpret_cast<const float4*>(vals + j);
    rank += (o.x > v) || (o.x == v && j + 0 < i);
    rank += (o.y > v) || (o.y == v && j + 1 < i);
    rank += (o.z > v) || (o.z == v && j + 2 < i);
    rank += (o.w > v) || (o.w == v && j + 3 < i);
  }
  const bool chosen = rank < k;
  inv[(long long)b * dim + i] = chosen ? rank : -1;
  if (chosen) {
    idx[(long long)b * k + rank] = i;
    float s2 = 0.f;
    for (int s = 0; s < splits; ++s) s2 += sq[((long long)s * n + b) * dim + i];
    sq_sel[(long long)b * k + rank] = s2;
  }
}

// The divisor of matrix b, bit for bit what `x / (norm.to(bf16) * 1.02 + eps)` gives in bf16 arithmetic.
__device__ __forceinline__ float dion2_divisor(const float* __restrict__ sq_sel, int k, float eps, float* red) {
  float acc = 0.f;
  for (int i = threadIdx.x; i < k; i += blockDim.x) acc += sq_sel[i];
  acc = warp_sum(acc);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x < 32) {
    acc = threadIdx.x < (blockDim.x >> 5) ? red[threadIdx.x] : 0.f;
    acc = warp_sum(acc);
    if (threadIdx.x == 0) red[0] = bf16_round(bf16_round(bf16_round(sqrtf(acc)) * 1.02f) + eps);
  }
  __syncthreads();
  return red[0];
}

// ---- 3. gather -----------------------------------------------------------------------------------------------
// Row slices: stack[b, r, :] = m[b, idx[b, r], :] / d.  One warp per selected row; grid = (ceil(k / kWarps), n).
__global__ void dion2_gather_rows_kernel(const float* __restrict__ m_all, const int* __restrict__ idx,
                                         const float* __restrict__ sq_sel, __nv_bfloat16* __restrict__ stack,
                                         int cols, int k, long long stride, float eps) {
  __shared__ float red[32];
  const int b = blockIdx.y;
  const float d = dion2_divisor(sq_sel + (long long)b * k, k, eps, red);
  const int r = blockIdx.x * kWarps + (threadIdx.x >> 5);
  if (r >= k) return;
  const int lane = threadIdx.x & 31;
  const int src = idx[(long long)b * k + r];
  const float4* m = reinterpret_cast<const float4*>(m_all + b * stride + (long long)src * cols);
  uint2* out = reinterpret_cast<uint2*>(stack + ((long long)b * k + r) * cols);
  for (int i = lane; i < (cols >> 2); i += 32) {
    const float4 v = m[i];
    // bf16(m) first (the orthogonaliser's input is the bf16 cast), then the bf16 division
    __nv_bfloat162 lo = __floats2bfloat162_rn(bf16_round(v.x) / d, bf16_round(v.y) / d);
    __nv_bfloat162 hi = __floats2bfloat162_rn(bf16_round(v.z) / d, bf16_round(v.w) / d);
    uint2 p;
    p.x = *reinterpret_cast<uint32_t*>(&lo);
    p.y = *reinterpret_cast<uint32_t*>(&hi);
    out[i] = p;
  }
}

// Column slices: stack[b, r, c] = m[b, r, idx[b, c]] / d.  One warp per row; grid = (ceil(rows / kWarps), n).
__global__ void dion2_gather_cols_kernel(const float* __restrict__ m_all, const int* __restrict__ idx,
                                         const float* __restrict__ sq_sel, __nv_bfloat16* __restrict__ stack,
                                         int rows, int cols, int k, long long stride, float eps) {
  __shared__ float red[32];
  const int b = blockIdx.y;
  const float d = dion2_divisor(sq_sel + (long long)b * k, k, eps, red);
  const int r = blockIdx.x * kWarps + (threadIdx.x >> 5);
  if (r >= rows) return;
  const int lane = threadIdx.x & 31;
  const float* m = m_all + b * stride + (long long)r * cols;
  const int* id = idx + (long long)b * k;
  __nv_bfloat16* out = stack + ((long long)b * rows + r) * k;
  for (int c = lane; c < k; c += 32) out[c] = __float2bfloat16_rn(bf16_round(m[id[c]]) / d);
}

// ---- 4. apply --------------------------------------------------------------------------------------------------
// Row slices; one warp per row of w; grid = (ceil(rows / kWarps), n).
__global__ void dion2_apply_rows_kernel(float* __restrict__ w_all, float* __restrict__ m_all,
                                        const __nv_bfloat16* __restrict__ o_all, const int* __restrict__ inv,
                                        __nv_bfloat16* __restrict__ shadow_all, int rows, int cols, int k,
                                        long long stride, float decay, float step, float ef) {
  const int b = blockIdx.y;
  const int row = blockIdx.x * kWarps + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int lane = threadIdx.x & 31;
  const int p = inv[(long long)b * rows + row];
  if (p < 0 && decay == 1.f && shadow_all == nullptr) return;
  const long long base = b * stride + (long long)row * cols;
  float4* w = reinterpret_cast<float4*>(w_all + base);
  float4* m = reinterpret_cast<float4*>(m_all + base);
  const uint2* o = p >= 0 ? reinterpret_cast<const uint2*>(o_all + ((long long)b * k + p) * cols) : nullptr;
  uint2* sh = shadow_all ? reinterpret_cast<uint2*>(shadow_all + base) : nullptr;
  for (int i = lane; i < (cols >> 2); i += 32) {
    float4 wv = w[i];
    wv.x *= decay; wv.y *= decay; wv.z *= decay; wv.w *= decay;
    if (o) {
      const uint2 ov = o[i];
      const float2 o01 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&ov.x));
      const float2 o23 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&ov.y));
      wv.x -= step * o01.x; wv.y -= step * o01.y; wv.z -= step * o23.x; wv.w -= step * o23.y;
      float4 mv = m[i];
      mv.x *= ef; mv.y *= ef; mv.z *= ef; mv.w *= ef;
      m[i] = mv;
    }
    if (o || decay != 1.f) w[i] = wv;
    if (sh) {
      __nv_bfloat162 lo = __floats2bfloat162_rn(wv.x, wv.y);
      __nv_bfloat162 hi = __floats2bfloat162_rn(wv.z, wv.w);
      uint2 pk;
      pk.x = *reinterpret_cast<uint32_t*>(&lo);
      pk.y = *reinterpret_cast<uint32_t*>(&hi);
      sh[i] = pk;
    }
  }
}

// Column slices; one warp per row of w, o is [b, rows, k]; grid = (ceil(rows / kWarps), n).
__global__ void dion2_apply_cols_kernel(float* __restrict__ w_all, float* __restrict__ m_all,
                                        const __nv_bfloat16* __restrict__ o_all, const int* __restrict__ inv,
                                        __nv_bfloat16* __restrict__ shadow_all, int rows, int cols, int k,
                                        long long stride, float decay, float step, float ef) {
  const int b = blockIdx.y;
  const int row = blockIdx.x * kWarps + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int lane = threadIdx.x & 31;
  const long long base = b * stride + (long long)row * cols;
  float* w = w_all + base;
  float* m = m_all + base;
  const __nv_bfloat16* o = o_all + ((long long)b * rows + row) * k;
  const int4* pv = reinterpret_cast<const int4*>(inv + (long long)b * cols);
  uint2* sh = shadow_all ? reinterpret_cast<uint2*>(shadow_all + base) : nullptr;
  for (int i = lane; i < (cols >> 2); i += 32) {
    float4 wv = reinterpret_cast<float4*>(w)[i];
    const int4 p = pv[i];
    float wl[4] = {wv.x * decay, wv.y * decay, wv.z * decay, wv.w * decay};
    const int pl[4] = {p.x, p.y, p.z, p.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      if (pl[j] >= 0) {
        wl[j] -= step * __bfloat162float(o[pl[j]]);
        m[i * 4 + j] *= ef;
      }
    }
    wv = make_float4(wl[0], wl[1], wl[2], wl[3]);
    reinterpret_cast<float4*>(w)[i] = wv;
    if (sh) {
      __nv_bfloat162 lo = __floats2bfloat162_rn(wv.x, wv.y);
      __nv_bfloat162 hi = __floats2bfloat162_rn(wv.z, wv.w);
      uint2 pk;
      pk.x = *reinterpret_cast<uint32_t*>(&lo);
      pk.y = *reinterpret_cast<uint32_t*>(&hi);
      sh[i] = pk;
    }
  }
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

}  // namespace

// Every entry: 0 = launched; 2 = a size or alignment rule is not met (nothing launched); else the CUDA error.
// Rules: cols % 4 == 0, stride % 4 == 0, 16-byte aligned matrices, and for column slices cols % 4 == 0 for `inv`.

extern "C" int b200_dion2_accumulate(const void* g, void* m, const void* clip, void* l1, void* sq, int n, int rows,
                                     int cols, long long stride, int axis, int splits, void* stream) {
  if (n <= 0 || rows <= 0 || cols <= 0 || (cols & 3) || (stride & 3) || !aligned16(g) || !aligned16(m)) return 2;
  if (n > 65535 || splits < 1 || splits > 65535) return 2;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (axis == 0) {
    if (splits != 1) return 2;
    dim3 grid((rows + kWarps - 1) / kWarps, n);
    dion2_accumulate_rows_kernel<<<grid, kThreads, 0, s>>>(static_cast<const float*>(g), static_cast<float*>(m),
                                                         static_cast<const float*>(clip), static_cast<float*>(l1),
                                                         static_cast<float*>(sq), rows, cols, stride);
  } else {
    const int per = (rows + splits - 1) / splits;
    dim3 grid((cols + 127) / 128, n, splits);
    dion2_accumulate_cols_kernel<<<grid, kThreads, 0, s>>>(static_cast<const float*>(g), static_cast<float*>(m),
                                                         static_cast<const float*>(clip), static_cast<float*>(l1),
                                                         static_cast<float*>(sq), rows, cols, stride, per, n);
  }
  return static_cast<int>(cudaGetLastError());
}

extern "C" int b200_dion2_select(const void* l1, const void* sq, int splits, int n, int dim, int k, void* idx,
                                 void* inv, void* sq_sel, void* stream) {
  if (n <= 0 || n > 65535 || dim <= 0 || k <= 0 || k > dim || splits < 1) return 2;
  const size_t smem = static_cast<size_t>((dim + 3) & ~3) * sizeof(float);
  if (smem > 48 * 1024) return 2;                     // 12288 slices; larger matrices take the library path
  dim3 grid((dim + 255) / 256, n);
  dion2_select_kernel<<<grid, 256, smem, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const float*>(l1), static_cast<const float*>(sq), splits, n, dim, k, static_cast<int*>(idx),
      static_cast<int*>(inv), static_cast<float*>(sq_sel));
  return static_cast<int>(cudaGetLastError());
}

extern "C" int b200_dion2_gather(const void* m, const void* idx, const void* sq_sel, void* stack, int n, int rows,
                                 int cols, int k, long long stride, int axis, float eps, void* stream) {
  if (n <= 0 || n > 65535 || (cols & 3) || (stride & 3) || !aligned16(m) || !aligned16(stack)) return 2;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (axis == 0) {
    dim3 grid((k + kWarps - 1) / kWarps, n);
    dion2_gather_rows_kernel<<<grid, kThreads, 0, s>>>(static_cast<const float*>(m), static_cast<const int*>(idx),
                                                     static_cast<const float*>(sq_sel),
                                                     static_cast<__nv_bfloat16*>(stack), cols, k, stride, eps);
  } else {
    dim3 grid((rows + kWarps - 1) / kWarps, n);
    dion2_gather_cols_kernel<<<grid, kThreads, 0, s>>>(static_cast<const float*>(m), static_cast<const int*>(idx),
                                                     static_cast<const float*>(sq_sel),
                                                     static_cast<__nv_bfloat16*>(stack), rows, cols, k, stride, eps);
  }
  return static_cast<int>(cudaGetLastError());
}

extern "C" int b200_dion2_apply(void* w, void* m, const void* o, const void* inv, void* shadow, int n, int rows,
                                int cols, int k, long long stride, int axis, float decay, float step, float ef,
                                void* stream) {
  if (n <= 0 || n > 65535 || (cols & 3) || (stride & 3) || !aligned16(w) || !aligned16(m) || !aligned16(o)) return 2;
  if (shadow && (reinterpret_cast<uintptr_t>(shadow) & 7u)) return 2;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  dim3 grid((rows + kWarps - 1) / kWarps, n);
  if (axis == 0)
    dion2_apply_rows_kernel<<<grid, kThreads, 0, s>>>(static_cast<float*>(w), static_cast<float*>(m),
                                                    static_cast<const __nv_bfloat16*>(o),
                                                    static_cast<const int*>(inv),
                                                    static_cast<__nv_bfloat16*>(shadow), rows, cols, k, stride,
                                                    decay, step, ef);
  else
    dion2_apply_cols_kernel<<<grid, kThreads, 0, s>>>(static_cast<float*>(w), static_cast<float*>(m),
                                                    static_cast<const __nv_bfloat16*>(o),
                                                    static_cast<const int*>(inv),
                                                    static_cast<__nv_bfloat16*>(shadow), rows, cols, k, stride,
                                                    decay, step, ef);
  return static_cast<int>(cudaGetLastError());
}
