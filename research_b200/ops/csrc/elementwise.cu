// Bandwidth-bound kernels of the training step for sm_100a: RMSNorm (+ residual add), QK-RMSNorm
// fused with interleaved-pair RoPE, SwiGLU, embedding gather / scatter-add, masked cross-entropy
// with z-loss that leaves dlogits in place, flat-arena AdamW with bf16 shadow write, sum of squares.
// All use 128-bit global accesses; reductions are warp shuffles, fp32 throughout.
//
// Math restated from the reference: RMSNorm and its scale (models/components/norm.py:12-38), RoPE over
// even/odd pairs (models/components/position.py:9-39), QK-norm before RoPE
// (models/components/attention.py:112-126, 228-234), SwiGLU (models/components/ffn.py:13-51), masked CE in
// fp32 log-softmax (steps/eval.py:27-37), z-loss (steps/train.py:597-602), AdamW (optim/build.py:29-31).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "b200.cuh"
#include "host_util.cuh"

namespace {

constexpr int kWarpsPerBlock = 8;

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ void unpack8(const uint4& v, float (&f)[8]) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 t = __bfloat1622float2(h[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
  uint4 v;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  return v;
}
__device__ __forceinline__ void load8f(const float* p, float (&f)[8]) {
  float4 a = *reinterpret_cast<const float4*>(p);
  float4 b = *reinterpret_cast<const float4*>(p + 4);
  f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w;
  f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
}

// ------------------------------------------------------------------------------------------------
// RMSNorm forward: optionally res_out = x + delta first.  One warp per row, H % 8 == 0.
// ------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
rmsnorm_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ delta,
                   const float* __restrict__ w, __nv_bfloat16* __restrict__ res_out, __nv_bfloat16* __restrict__ y,
                   float* __restrict__ rstd_out, int rows, int H, float eps) {
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int nvec = H >> 3;
  for (long long row = (long long)blockIdx.x * kWarpsPerBlock + warp; row < rows;
       row += (long long)gridDim.x * kWarpsPerBlock) {
    const uint4* xr = reinterpret_cast<const uint4*>(x + row * H);
    const uint4* dr = delta ? reinterpret_cast<const uint4*>(delta + row * H) : nullptr;
    uint4* rr = res_out ? reinterpret_cast<uint4*>(res_out + row * H) : nullptr;
    float ss = 0.f;
    for (int v = lane; v < nvec; v += 32) {
      float f[8];
      unpack8(xr[v], f);
      if (dr) {
        float g[8];
        unpack8(dr[v], g);
#pragma unroll
        for (int i = 0; i < 8; ++i) f[i] += g[i];
        uint4 s = pack8(f);
        rr[v] = s;
        unpack8(s, f);  // normalise exactly what was stored
      }
#pragma unroll
      for (int i = 0; i < 8; ++i) ss += f[i] * f[i];
    }
    ss = warp_sum(ss);
    const float rstd = rsqrtf(ss / (float)H + eps);
    if (lane == 0 && rstd_out) rstd_out[row] = rstd;
    const uint4* src = dr ? reinterpret_cast<const uint4*>(res_out + row * H) : xr;
    uint4* yr = reinterpret_cast<uint4*>(y + row * H);
    for (int v = lane; v < nvec; v += 32) {
      float f[8], wv[8];
      unpack8(src[v], f);
      load8f(w + v * 8, wv);
#pragma unroll
      for (int i = 0; i < 8; ++i) f[i] = f[i] * rstd * wv[i];
      yr[v] = pack8(f);
    }
  }
}

// H == NV * 256: a warp keeps its whole row in registers, so every load of the row is in flight at once and the row
// is read from memory exactly once (the generic kernel above walks the row twice with one load in flight per lane).
template <int NV>
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
rmsnorm_fwd_reg_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ delta,
                       const float* __restrict__ w, __nv_bfloat16* __restrict__ res_out, __nv_bfloat16* __restrict__ y,
                       float* __restrict__ rstd_out, int rows, float eps) {
  constexpr int H = NV * 256;
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  for (long long row = (long long)blockIdx.x * kWarpsPerBlock + warp; row < rows;
       row += (long long)gridDim.x * kWarpsPerBlock) {
    const uint4* xr = reinterpret_cast<const uint4*>(x + row * H);
    uint4 raw[NV], draw[NV];
#pragma unroll
    for (int j = 0; j < NV; ++j) raw[j] = xr[lane + 32 * j];
    if (delta) {
      const uint4* dr = reinterpret_cast<const uint4*>(delta + row * H);
#pragma unroll
      for (int j = 0; j < NV; ++j) draw[j] = dr[lane + 32 * j];
    }
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < NV; ++j) {
      float f[8];
      unpack8(raw[j], f);
      if (delta) {
        float g[8];
        unpack8(draw[j], g);
#pragma unroll
        for (int i = 0; i < 8; ++i) f[i] += g[i];
        raw[j] = pack8(f);
        reinterpret_cast<uint4*>(res_out + row * H)[lane + 32 * j] = raw[j];
        unpack8(raw[j], f);  // normalise exactly what was stored
      }
#pragma unroll
      for (int i = 0; i < 8; ++i) ss += f[i] * f[i];
    }
    ss = warp_sum(ss);
    const float rstd = rsqrtf(ss / (float)H + eps);
    if (lane == 0 && rstd_out) rstd_out[row] = rstd;
    uint4* yr = reinterpret_cast<uint4*>(y + row * H);
#pragma unroll
    for (int j = 0; j < NV; ++j) {
      float f[8], wv[8];
      unpack8(raw[j], f);
      load8f(w + (lane + 32 * j) * 8, wv);
#pragma unroll
      for (int i = 0; i < 8; ++i) f[i] = f[i] * rstd * wv[i];
      yr[lane + 32 * j] = pack8(f);
    }
  }
}

// The same for a handful of rows (a decode step): one block per row, so that a row's loads are issued by 256 threads at
// once instead of one warp walking it.
__global__ void __launch_bounds__(256)
rmsnorm_fwd_row_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ delta,
                       const float* __restrict__ w, __nv_bfloat16* __restrict__ res_out, __nv_bfloat16* __restrict__ y,
                       float* __restrict__ rstd_out, int H, float eps) {
  __shared__ float part[8];
  b200::pdl_launch_dependents();   // no-ops unless launched as a dependent (decode steps)
  b200::pdl_wait();
  const long long row = blockIdx.x;
  const int nvec = H >> 3;
  const uint4* xr = reinterpret_cast<const uint4*>(x + row * H);
  const uint4* dr = delta ? reinterpret_cast<const uint4*>(delta + row * H) : nullptr;
  uint4* rr = res_out ? reinterpret_cast<uint4*>(res_out + row * H) : nullptr;
  float ss = 0.f;
  for (int v = threadIdx.x; v < nvec; v += 256) {
    float f[8];
    unpack8(xr[v], f);
    if (dr) {
      float g[8];
      unpack8(dr[v], g);
#pragma unroll
      for (int i = 0; i < 8; ++i) f[i] += g[i];
      uint4 s = pack8(f);
      rr[v] = s;
      unpack8(s, f);  // normalise exactly what was stored
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) ss += f[i] * f[i];
  }
  ss = warp_sum(ss);
  if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = ss;
  __syncthreads();
  float total = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) total += part[i];
  const float rstd = rsqrtf(total / (float)H + eps);
  if (threadIdx.x == 0 && rstd_out) rstd_out[row] = rstd;
  const uint4* src = dr ? reinterpret_cast<const uint4*>(res_out + row * H) : xr;
  uint4* yr = reinterpret_cast<uint4*>(y + row * H);
  for (int v = threadIdx.x; v < nvec; v += 256) {  // a thread re-reads only what it wrote itself
    float f[8], wv[8];
    unpack8(src[v], f);
    load8f(w + v * 8, wv);
#pragma unroll
    for (int i = 0; i < 8; ++i) f[i] = f[i] * rstd * wv[i];
    yr[v] = pack8(f);
  }
}

// Tail of a split-K GEMM for a handful of rows: the slices were reduce-added into an fp32 workspace that was zero
// before; this reads the sums, writes them as bf16 and puts the zeros back, so the workspace needs no separate
// fill before its next use.  n % 4 == 0.
__global__ void __launch_bounds__(256)
splitk_finish_kernel(float* __restrict__ ws, __nv_bfloat16* __restrict__ out, long long n4) {
  b200::pdl_launch_dependents();
  b200::pdl_wait();
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (long long)gridDim.x * blockDim.x) {
    const float4 v = reinterpret_cast<const float4*>(ws)[i];
    reinterpret_cast<float4*>(ws)[i] = make_float4(0.f, 0.f, 0.f, 0.f);
    __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
    uint2 packed;
    packed.x = *reinterpret_cast<uint32_t*>(&lo);
    packed.y = *reinterpret_cast<uint32_t*>(&hi);
    reinterpret_cast<uint2*>(out)[i] = packed;
  }
}

// RMSNorm backward.  dx = rstd * (dy*w - xhat * mean(dy*w*xhat)) (+ dres if given); dw += sum_rows dy*xhat
// NV > 0: H == NV * 256 and every lane keeps its dw partial sums in registers over all of its rows;
// NV == 0: any H % 8 == 0, partial sums go through shared-memory atomics.  Either way a block folds its
// partials in shared memory and issues one fp32 atomicAdd per column.
template <int NV>
__global__ void __launch_bounds__(kWarpsPerBlock * 32, (NV == 8 ? 2 : 1))
rmsnorm_bwd_kernel(const __nv_bfloat16* __restrict__ x, const float* __restrict__ w,
                   const float* __restrict__ rstd_in, const __nv_bfloat16* __restrict__ dy,
                   const __nv_bfloat16* __restrict__ dres, __nv_bfloat16* __restrict__ dx, float* __restrict__ dw,
                   int rows, int H) {
  extern __shared__ float dw_smem[];  // H floats
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int nvec = H >> 3;
  constexpr int NACC = NV > 0 ? NV : 1;
  float acc[NACC][8];
#pragma unroll
  for (int j = 0; j < NACC; ++j)
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[j][i] = 0.f;
  for (int i = threadIdx.x; i < H; i += blockDim.x) dw_smem[i] = 0.f;
  __syncthreads();
  for (long long row = (long long)blockIdx.x * kWarpsPerBlock + warp; row < rows;
       row += (long long)gridDim.x * kWarpsPerBlock) {
    const uint4* xr = reinterpret_cast<const uint4*>(x + row * H);
    const uint4* gr = reinterpret_cast<const uint4*>(dy + row * H);
    const float rstd = rstd_in[row];
    float dot = 0.f;
    // Up to H = 1024 the row of x and dy stays in registers (read once, all loads in flight: 0.61 of the copy
    // bandwidth against 0.45).  Above that the registers go to the dw partial sums; batching the loads of the first
    // pass there cost occupancy and measured slower (0.43 against 0.55 at H = 2048).
    constexpr bool kInRegs = NV > 0 && NV <= 4;
    constexpr int NRAW = kInRegs ? NV : 1;
    uint4 xraw[NRAW], graw[NRAW];
    if constexpr (kInRegs) {
#pragma unroll
      for (int j = 0; j < NV; ++j) {
        xraw[j] = xr[lane + 32 * j];
        graw[j] = gr[lane + 32 * j];
      }
#pragma unroll
      for (int j = 0; j < NV; ++j) {
        float f[8], g[8], wv[8];
        unpack8(xraw[j], f);
        unpack8(graw[j], g);
        load8f(w + (lane + 32 * j) * 8, wv);
#pragma unroll
        for (int i = 0; i < 8; ++i) dot += g[i] * wv[i] * f[i] * rstd;
      }
    } else if constexpr (NV == 8) {
#pragma unroll 4
      for (int j = 0; j < NV; ++j) {  // known trip count: four loads of x and of dy in flight per lane
        const int v = lane + 32 * j;
        float f[8], g[8], wv[8];
        unpack8(xr[v], f);
        unpack8(gr[v], g);
        load8f(w + v * 8, wv);
#pragma unroll
        for (int i = 0; i < 8; ++i) dot += g[i] * wv[i] * f[i] * rstd;
      }
    } else {
      for (int v = lane; v < nvec; v += 32) {
        float f[8], g[8], wv[8];
        unpack8(xr[v], f);
        unpack8(gr[v], g);
        load8f(w + v * 8, wv);
#pragma unroll
        for (int i = 0; i < 8; ++i) dot += g[i] * wv[i] * f[i] * rstd;
      }
    }
    dot = warp_sum(dot) / (float)H;
    const uint4* rr = dres ? reinterpret_cast<const uint4*>(dres + row * H) : nullptr;
    uint4* dxr = reinterpret_cast<uint4*>(dx + row * H);
    if constexpr (NV > 0) {
#pragma unroll
      for (int j = 0; j < NV; ++j) {
        const int v = lane + 32 * j;
        float f[8], g[8], wv[8], o[8];
        unpack8(kInRegs ? xraw[j < NRAW ? j : 0] : xr[v], f);
        unpack8(kInRegs ? graw[j < NRAW ? j : 0] : gr[v], g);
        load8f(w + v * 8, wv);
        float r[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        if (rr) unpack8(rr[v], r);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float xhat = f[i] * rstd;
          o[i] = rstd * (g[i] * wv[i] - xhat * dot) + r[i];
          acc[j][i] += g[i] * xhat;
        }
        dxr[v] = pack8(o);
      }
    } else {
      for (int v = lane; v < nvec; v += 32) {
        float f[8], g[8], wv[8], o[8];
        unpack8(xr[v], f);
        unpack8(gr[v], g);
        load8f(w + v * 8, wv);
        float r[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        if (rr) unpack8(rr[v], r);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float xhat = f[i] * rstd;
          o[i] = rstd * (g[i] * wv[i] - xhat * dot) + r[i];
          atomicAdd(&dw_smem[v * 8 + i], g[i] * xhat);
        }
        dxr[v] = pack8(o);
      }
    }
  }
  if constexpr (NV > 0) {
#pragma unroll
    for (int j = 0; j < NV; ++j)
#pragma unroll
      for (int i = 0; i < 8; ++i) atomicAdd(&dw_smem[(lane + 32 * j) * 8 + i], acc[j][i]);
  }
  __syncthreads();
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    const float v = dw_smem[i];
    if (v != 0.f) atomicAdd(&dw[i], v);
  }
}

// RMSNorm backward for wide rows (H = 8 * VEC * THREADS): a block walks rows, a thread owns 8 * VEC columns of every
// row, so the row of x and dy is read once into registers, the dw partial sums are 8 * VEC registers, and the loads
// of the block's next row are issued before the current row is reduced (one block-wide reduction of the dot product
// through shared memory per row, double buffered by parity), which keeps loads in flight all the time.
template <int VEC, int THREADS, int MINB>
__global__ void __launch_bounds__(THREADS, MINB)
rmsnorm_bwd_cols_kernel(const __nv_bfloat16* __restrict__ x, const float* __restrict__ w,
                        const float* __restrict__ rstd_in, const __nv_bfloat16* __restrict__ dy,
                        const __nv_bfloat16* __restrict__ dres, __nv_bfloat16* __restrict__ dx,
                        float* __restrict__ dw, int rows, int H) {
  __shared__ float red[2][32];
  const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
  constexpr int kWarps = THREADS / 32;
  const long long nvec = H >> 3;
  const float inv_h = 1.f / (float)H;
  float wv[VEC][8], acc[VEC][8];
#pragma unroll
  for (int v = 0; v < VEC; ++v) {
    load8f(w + (t + v * THREADS) * 8, wv[v]);
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[v][i] = 0.f;
  }
  const uint4 zero = make_uint4(0, 0, 0, 0);
  uint4 xc[VEC], gc[VEC], rc[VEC];
  float rs = 0.f;
  long long row = blockIdx.x;
  if (row < rows) {
#pragma unroll
    for (int v = 0; v < VEC; ++v) {
      xc[v] = reinterpret_cast<const uint4*>(x)[row * nvec + t + v * THREADS];
      gc[v] = reinterpret_cast<const uint4*>(dy)[row * nvec + t + v * THREADS];
      rc[v] = dres ? reinterpret_cast<const uint4*>(dres)[row * nvec + t + v * THREADS] : zero;
    }
    rs = rstd_in[row];
  }
  int parity = 0;
  for (; row < rows; row += gridDim.x, parity ^= 1) {
    uint4 xn[VEC], gn[VEC], rn[VEC];
    float rsn = 0.f;
    const long long next = row + gridDim.x;
    if (next < rows) {  // in flight while this row is reduced and written
#pragma unroll
      for (int v = 0; v < VEC; ++v) {
        xn[v] = reinterpret_cast<const uint4*>(x)[next * nvec + t + v * THREADS];
        gn[v] = reinterpret_cast<const uint4*>(dy)[next * nvec + t + v * THREADS];
        rn[v] = dres ? reinterpret_cast<const uint4*>(dres)[next * nvec + t + v * THREADS] : zero;
      }
      rsn = rstd_in[next];
    } else {
#pragma unroll
      for (int v = 0; v < VEC; ++v) xn[v] = gn[v] = rn[v] = zero;
    }
    float d = 0.f;
#pragma unroll
    for (int v = 0; v < VEC; ++v) {
      float f[8], g[8];
      unpack8(xc[v], f);
      unpack8(gc[v], g);
#pragma unroll
      for (int i = 0; i < 8; ++i) d += g[i] * wv[v][i] * f[i];
    }
    d = warp_sum(d * rs);
    if (lane == 0) red[parity][warp] = d;
    __syncthreads();
    const float dot = warp_sum(lane < kWarps ? red[parity][lane] : 0.f) * inv_h;
#pragma unroll
    for (int v = 0; v < VEC; ++v) {
      float f[8], g[8], r[8], o[8];
      unpack8(xc[v], f);
      unpack8(gc[v], g);
      unpack8(rc[v], r);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float xhat = f[i] * rs;
        o[i] = rs * (g[i] * wv[v][i] - xhat * dot) + r[i];
        acc[v][i] += g[i] * xhat;
      }
      reinterpret_cast<uint4*>(dx)[row * nvec + t + v * THREADS] = pack8(o);
    }
#pragma unroll
    for (int v = 0; v < VEC; ++v) {
      xc[v] = xn[v];
      gc[v] = gn[v];
      rc[v] = rn[v];
    }
    rs = rsn;
  }
#pragma unroll
  for (int v = 0; v < VEC; ++v)
#pragma unroll
    for (int i = 0; i < 8; ++i)
      if (acc[v][i] != 0.f) atomicAdd(&dw[(t + v * THREADS) * 8 + i], acc[v][i]);
}

// ------------------------------------------------------------------------------------------------
// QK-RMSNorm + RoPE (interleaved pairs) over the head dimension.  One warp handles one (token, head)
// vector of D elements (D % 8 == 0, D <= 256): lane l owns elements [8l, 8l+8) = 4 rotation pairs.
// in : [tokens, in_stride] with heads at column h*D;   out: [tokens, out_stride]
// w  : [D] fp32 norm scale or nullptr (no norm).  positions: [tokens] int32.  rope: 0 = skip rotation.
// Angle of pair i at position p: p * theta^(-2i/D).
// ------------------------------------------------------------------------------------------------
// sin and cos of an angle of any size: Cody-Waite reduction by 2*pi to [-pi, pi], then the special-function unit
__device__ __forceinline__ void sincos_reduced(float x, float* s, float* c) {
  const float k = rintf(x * 0.15915494309189535f);
  x = fmaf(k, -6.28318548202514648f, x);
  x = fmaf(k, 1.74845553e-7f, x);
  __sincosf(x, s, c);
}

// A head of D <= 256 elements is handled by `lph` lanes (a power of two, 8 elements per lane), so a warp works on
// 32 / lph heads at once; reductions stay inside the lane group.
__device__ __forceinline__ float group_sum(float v, int lph) {
  for (int off = lph >> 1; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
  return v;
}

__global__ void __launch_bounds__(kWarpsPerBlock * 32)
qknorm_rope_fwd_kernel(const __nv_bfloat16* __restrict__ in, long long in_stride, __nv_bfloat16* __restrict__ out,
                       long long out_stride, const float* __restrict__ w, const int* __restrict__ positions,
                       float* __restrict__ rstd_out, long long tokens, int heads, int D, float eps, float log2_theta,
                       int rope, int lph, const float* __restrict__ w2, int heads_first) {
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int hpw = 32 / lph;
  const int sub = lane / lph, l = lane % lph;
  const long long total = tokens * heads;
  const bool has_cols = l * 8 < D;
  // heads [0, heads_first) are scaled by w, the rest by w2 (query heads and key heads of a packed projection)
  float inv_freq[4], wv[8] = {1, 1, 1, 1, 1, 1, 1, 1}, wv2[8] = {1, 1, 1, 1, 1, 1, 1, 1};
#pragma unroll
  for (int i = 0; i < 4; ++i) inv_freq[i] = exp2f(-log2_theta * (2.f * (float)(l * 4 + i)) / (float)D);
  // the norm scales are weights (no predecessor writes them): they are read before the wait for the predecessor
  if (w && has_cols) load8f(w + l * 8, wv);
  if (w2 && has_cols) load8f(w2 + l * 8, wv2);
  b200::pdl_launch_dependents();   // no-ops unless launched as a dependent (decode steps)
  b200::pdl_wait();
  const long long groups = (total + hpw - 1) / hpw;
  for (long long gidx = (long long)blockIdx.x * kWarpsPerBlock + warp; gidx < groups;
       gidx += (long long)gridDim.x * kWarpsPerBlock) {
    const long long idx = gidx * hpw + sub;
    const bool active = has_cols && idx < total;
    const long long t = idx / heads;
    const int h = (int)(idx - t * heads);
    float f[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    if (active) unpack8(*reinterpret_cast<const uint4*>(in + t * in_stride + (long long)h * D + l * 8), f);
    if (w) {
      float ss = 0.f;
#pragma unroll
      for (int i = 0; i < 8; ++i) ss += f[i] * f[i];
      ss = group_sum(ss, lph);
      const float rstd = rsqrtf(ss / (float)D + eps);
      if (l == 0 && rstd_out && idx < total) rstd_out[idx] = rstd;
      const bool first = h < heads_first;
#pragma unroll
      for (int i = 0; i < 8; ++i) f[i] = f[i] * rstd * (first ? wv[i] : wv2[i]);
    }
    if (rope && active) {
      const float pos = (float)positions[t];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        float s, c;
        sincos_reduced(pos * inv_freq[i], &s, &c);
        const float a = f[2 * i], b = f[2 * i + 1];
        f[2 * i] = a * c - b * s;
        f[2 * i + 1] = a * s + b * c;
      }
    }
    if (active) *reinterpret_cast<uint4*>(out + t * out_stride + (long long)h * D + l * 8) = pack8(f);
  }
}

// backward of the above: grad wrt the pre-norm input, and dw (atomic fp32 adds, D columns)
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
qknorm_rope_bwd_kernel(const __nv_bfloat16* __restrict__ in, long long in_stride,
                       const __nv_bfloat16* __restrict__ dout, long long dout_stride,
                       __nv_bfloat16* __restrict__ din, long long din_stride, const float* __restrict__ w,
                       const int* __restrict__ positions, const float* __restrict__ rstd_in,
                       float* __restrict__ dw, long long tokens, int heads, int D, float log2_theta, int rope,
                       int lph, const float* __restrict__ w2, float* __restrict__ dw2, int heads_first) {
  __shared__ float dw_smem[512];
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int hpw = 32 / lph;
  const int sub = lane / lph, l = lane % lph;
  const long long total = tokens * heads;
  const bool has_cols = l * 8 < D;
  for (int i = threadIdx.x; i < 512; i += blockDim.x) dw_smem[i] = 0.f;
  __syncthreads();
  float inv_freq[4], wv[8] = {0, 0, 0, 0, 0, 0, 0, 0}, wv2[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#pragma unroll
  for (int i = 0; i < 4; ++i) inv_freq[i] = exp2f(-log2_theta * (2.f * (float)(l * 4 + i)) / (float)D);
  if (w && has_cols) load8f(w + l * 8, wv);
  if (w2 && has_cols) load8f(w2 + l * 8, wv2);
  float dw_acc[8] = {0, 0, 0, 0, 0, 0, 0, 0}, dw_acc2[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  const long long groups = (total + hpw - 1) / hpw;
  for (long long gidx = (long long)blockIdx.x * kWarpsPerBlock + warp; gidx < groups;
       gidx += (long long)gridDim.x * kWarpsPerBlock) {
    const long long idx = gidx * hpw + sub;
    const bool active = has_cols && idx < total;
    const long long t = idx / heads;
    const int h = (int)(idx - t * heads);
    float g[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    if (active) unpack8(*reinterpret_cast<const uint4*>(dout + t * dout_stride + (long long)h * D + l * 8), g);
    if (rope && active) {
      const float pos = (float)positions[t];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        float s, c;
        sincos_reduced(pos * inv_freq[i], &s, &c);
        const float a = g[2 * i], b = g[2 * i + 1];  // transpose of the rotation
        g[2 * i] = a * c + b * s;
        g[2 * i + 1] = -a * s + b * c;
      }
    }
    if (w) {
      float f[8] = {0, 0, 0, 0, 0, 0, 0, 0};
      if (active) unpack8(*reinterpret_cast<const uint4*>(in + t * in_stride + (long long)h * D + l * 8), f);
      const float rstd = idx < total ? rstd_in[idx] : 0.f;
      const bool first = h < heads_first;
      float dot = 0.f;
#pragma unroll
      for (int i = 0; i < 8; ++i) dot += g[i] * (first ? wv[i] : wv2[i]) * f[i] * rstd;
      dot = group_sum(dot, lph) / (float)D;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float xhat = f[i] * rstd;
        if (first) dw_acc[i] += g[i] * xhat; else dw_acc2[i] += g[i] * xhat;
        g[i] = rstd * (g[i] * (first ? wv[i] : wv2[i]) - xhat * dot);
      }
    }
    if (active) *reinterpret_cast<uint4*>(din + t * din_stride + (long long)h * D + l * 8) = pack8(g);
  }
  if (w && (dw || dw2)) {
    if (has_cols) {
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        atomicAdd(&dw_smem[l * 8 + i], dw_acc[i]);
        atomicAdd(&dw_smem[256 + l * 8 + i], dw_acc2[i]);
      }
    }
    __syncthreads();
    if (threadIdx.x < D) {
      if (dw) atomicAdd(&dw[threadIdx.x], dw_smem[threadIdx.x]);
      if (dw2) atomicAdd(&dw2[threadIdx.x], dw_smem[256 + threadIdx.x]);
    }
  }
}

// ------------------------------------------------------------------------------------------------
// SwiGLU on a fused [rows, 2*I] gate|up buffer: h = silu(g) * u.
// ------------------------------------------------------------------------------------------------
// sigmoid through the hardware tanh (one special-function op instead of an exponential and a reciprocal; 11 good
// bits, more than a bf16 result keeps): sigmoid(x) = 0.5 + 0.5 tanh(x / 2)
__device__ __forceinline__ float sigmoid_fast(float x) {
  float t;
  asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(0.5f * x));
  return fmaf(0.5f, t, 0.5f);
}

// Rows and vectors are walked with 32-bit arithmetic (the launchers check that rows * I / 8 fits); a 64-bit divide
// per thread and the two special-function ops per element used to make these kernels issue-bound.
__global__ void swiglu_fwd_kernel(const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ h, long long rows,
                                  int I) {
  const unsigned nvec = (unsigned)I >> 3;
  const unsigned total = (unsigned)rows * nvec;
  b200::pdl_launch_dependents();
  b200::pdl_wait();
  for (unsigned i = blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gridDim.x * blockDim.x) {
    const unsigned r = i / nvec;
    const unsigned v = i - r * nvec;
    const __nv_bfloat16* base = gu + (long long)r * 2 * I;
    float g[8], u[8], o[8];
    unpack8(*reinterpret_cast<const uint4*>(base + v * 8), g);
    unpack8(*reinterpret_cast<const uint4*>(base + I + v * 8), u);
#pragma unroll
    for (int k = 0; k < 8; ++k) o[k] = g[k] * sigmoid_fast(g[k]) * u[k];
    *reinterpret_cast<uint4*>(h + (long long)r * I + v * 8) = pack8(o);
  }
}
__global__ void swiglu_bwd_kernel(const __nv_bfloat16* __restrict__ gu, const __nv_bfloat16* __restrict__ dh,
                                  __nv_bfloat16* __restrict__ dgu, long long rows, int I) {
  const unsigned nvec = (unsigned)I >> 3;
  const unsigned total = (unsigned)rows * nvec;
  for (unsigned i = blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gridDim.x * blockDim.x) {
    const unsigned r = i / nvec;
    const unsigned v = i - r * nvec;
    const __nv_bfloat16* base = gu + (long long)r * 2 * I;
    float g[8], u[8], d[8], dg[8], du[8];
    unpack8(*reinterpret_cast<const uint4*>(base + v * 8), g);
    unpack8(*reinterpret_cast<const uint4*>(base + I + v * 8), u);
    unpack8(*reinterpret_cast<const uint4*>(dh + (long long)r * I + v * 8), d);
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const float sig = sigmoid_fast(g[k]);
      const float silu = g[k] * sig;
      du[k] = d[k] * silu;
      dg[k] = d[k] * u[k] * (sig + silu * (1.f - sig));
    }
    *reinterpret_cast<uint4*>(dgu + (long long)r * 2 * I + v * 8) = pack8(dg);
    *reinterpret_cast<uint4*>(dgu + (long long)r * 2 * I + I + v * 8) = pack8(du);
  }
}

// out = a * sigmoid(gate) (attention output gate) and its backward
__global__ void sigmoid_gate_fwd_kernel(const __nv_bfloat16* __restrict__ a, const __nv_bfloat16* __restrict__ gate,
                                        __nv_bfloat16* __restrict__ out, long long nvec) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += (long long)gridDim.x * blockDim.x) {
    float x[8], g[8];
    unpack8(reinterpret_cast<const uint4*>(a)[i], x);
    unpack8(reinterpret_cast<const uint4*>(gate)[i], g);
#pragma unroll
    for (int k = 0; k < 8; ++k) x[k] = x[k] * sigmoid_fast(g[k]);
    reinterpret_cast<uint4*>(out)[i] = pack8(x);
  }
}
__global__ void sigmoid_gate_bwd_kernel(const __nv_bfloat16* __restrict__ a, const __nv_bfloat16* __restrict__ gate,
                                        const __nv_bfloat16* __restrict__ dout, __nv_bfloat16* __restrict__ da,
                                        __nv_bfloat16* __restrict__ dgate, long long nvec) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += (long long)gridDim.x * blockDim.x) {
    float x[8], g[8], d[8], o1[8], o2[8];
    unpack8(reinterpret_cast<const uint4*>(a)[i], x);
    unpack8(reinterpret_cast<const uint4*>(gate)[i], g);
    unpack8(reinterpret_cast<const uint4*>(dout)[i], d);
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const float sig = sigmoid_fast(g[k]);
      o1[k] = d[k] * sig;
      o2[k] = d[k] * x[k] * sig * (1.f - sig);
    }
    reinterpret_cast<uint4*>(da)[i] = pack8(o1);
    reinterpret_cast<uint4*>(dgate)[i] = pack8(o2);
  }
}

// ------------------------------------------------------------------------------------------------
// Embedding gather (bf16 table) with optional scale, and scatter-add of gradients into fp32.
// ------------------------------------------------------------------------------------------------
__global__ void embedding_fwd_kernel(const int* __restrict__ ids, const __nv_bfloat16* __restrict__ table,
                                     __nv_bfloat16* __restrict__ out, long long tokens, int H, float scale) {
  const int nvec = H >> 3;
  const long long total = tokens * nvec;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long t = i / nvec;
    const int v = (int)(i - t * nvec);
    uint4 val = *reinterpret_cast<const uint4*>(table + (long long)ids[t] * H + v * 8);
    if (scale != 1.f) {
      float f[8];
      unpack8(val, f);
#pragma unroll
      for (int k = 0; k < 8; ++k) f[k] *= scale;
      val = pack8(f);
    }
    *reinterpret_cast<uint4*>(out + t * H + v * 8) = val;
  }
}
__global__ void embedding_bwd_kernel(const int* __restrict__ ids, const __nv_bfloat16* __restrict__ dout,
                                     float* __restrict__ dtable, long long tokens, int H, float scale) {
  const int nvec = H >> 3;
  const long long total = tokens * nvec;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long t = i / nvec;
    const int v = (int)(i - t * nvec);
    float f[8];
    unpack8(*reinterpret_cast<const uint4*>(dout + t * H + v * 8), f);
    float* dst = dtable + (long long)ids[t] * H + v * 8;
#pragma unroll
    for (int k = 0; k < 8; ++k) atomicAdd(dst + k, f[k] * scale);
  }
}

// ------------------------------------------------------------------------------------------------
// Masked cross-entropy + z-loss over one chunk of logits [rows, V] (bf16, row stride ld), in place:
//   loss_i = lse_i - logit_i[target_i];  z_i = lse_i^2            (only rows with mask != 0 count)
//   logits <- dlogits = grad_scale * mask_i * ((1 + 2 z_w lse_i) softmax - onehot)
// One block per row; three passes over the row (max, sum, write); the row stays in L1/L2.
// Sums are written per row (loss_row, z_row) so that the host-visible reduction is deterministic.
// vocab_offset/vocab_total support vocab-parallel logits: then max and sum come in precomputed
// (global_max / global_sum per row) and phase selects which pass runs.
// ------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(512)
ce_fwd_bwd_kernel(__nv_bfloat16* __restrict__ logits, long long ld, const int* __restrict__ targets,
                  const uint8_t* __restrict__ mask, float* __restrict__ loss_row, float* __restrict__ z_row,
                  float* __restrict__ lse_row, int V, float grad_scale, float z_weight, int write_grad) {
  __shared__ float red[32];
  const long long row = blockIdx.x;
  __nv_bfloat16* lr = logits + row * ld;
  const int nvec = V >> 3;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  const bool masked = mask[row] == 0;
  if (masked && !write_grad) {
    if (threadIdx.x == 0) { loss_row[row] = 0.f; z_row[row] = 0.f; if (lse_row) lse_row[row] = 0.f; }
    return;
  }
  if (masked) {  // zero gradient row, no loss
    const uint4 z = make_uint4(0, 0, 0, 0);
    for (int v = threadIdx.x; v < nvec; v += blockDim.x) reinterpret_cast<uint4*>(lr)[v] = z;
    for (int c = nvec * 8 + threadIdx.x; c < V; c += blockDim.x) lr[c] = __float2bfloat16(0.f);
    if (threadIdx.x == 0) { loss_row[row] = 0.f; z_row[row] = 0.f; if (lse_row) lse_row[row] = 0.f; }
    return;
  }
  // pass 1: max
  float m = -INFINITY;
  for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
    float f[8];
    unpack8(reinterpret_cast<const uint4*>(lr)[v], f);
#pragma unroll
    for (int k = 0; k < 8; ++k) m = fmaxf(m, f[k]);
  }
  for (int c = nvec * 8 + threadIdx.x; c < V; c += blockDim.x) m = fmaxf(m, __bfloat162float(lr[c]));
  m = warp_max(m);
  if (lane == 0) red[warp] = m;
  __syncthreads();
  m = (lane < nwarps) ? red[lane] : -INFINITY;
  m = warp_max(m);
  __syncthreads();
  // pass 2: sum exp
  float s = 0.f;
  for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
    float f[8];
    unpack8(reinterpret_cast<const uint4*>(lr)[v], f);
#pragma unroll
    for (int k = 0; k < 8; ++k) s += __expf(f[k] - m);
  }
  for (int c = nvec * 8 + threadIdx.x; c < V; c += blockDim.x) s += __expf(__bfloat162float(lr[c]) - m);
  s = warp_sum(s);
  if (lane == 0) red[warp] = s;
  __syncthreads();
  s = (lane < nwarps) ? red[lane] : 0.f;
  s = warp_sum(s);
  const float lse = m + logf(s);
  const int tgt = targets[row];
  const float tl = __bfloat162float(lr[tgt]);
  __syncthreads();  // everyone has read the target logit before it is overwritten
  if (threadIdx.x == 0) {
    loss_row[row] = lse - tl;
    z_row[row] = lse * lse;
    if (lse_row) lse_row[row] = lse;
  }
  if (!write_grad) return;
  // pass 3: gradient in place
  const float coef = grad_scale * (1.f + 2.f * z_weight * lse);
  const float inv_s = 1.f / s;
  for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
    float f[8];
    unpack8(reinterpret_cast<const uint4*>(lr)[v], f);
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      f[k] = coef * __expf(f[k] - m) * inv_s;
      if (v * 8 + k == tgt) f[k] -= grad_scale;
    }
    reinterpret_cast<uint4*>(lr)[v] = pack8(f);
  }
  for (int c = nvec * 8 + threadIdx.x; c < V; c += blockDim.x) {
    float g = coef * __expf(__bfloat162float(lr[c]) - m) * inv_s;
    if (c == tgt) g -= grad_scale;
    lr[c] = __float2bfloat16(g);
  }
}

// The same op with the row staged in shared memory: one bulk copy in, three passes over shared memory, one bulk
// copy out, so the logits cross the memory system once in each direction and two or three rows per SM overlap
// their phases.  V % 8 == 0 and 2 V bytes of dynamic shared memory; 16-byte aligned rows.
constexpr int kCeThreads = 512;
constexpr uint32_t kCeChunkBytes = 32768;
__global__ void __launch_bounds__(kCeThreads)
ce_fwd_bwd_staged_kernel(__nv_bfloat16* __restrict__ logits, long long ld, const int* __restrict__ targets,
                         const uint8_t* __restrict__ mask, float* __restrict__ loss_row, float* __restrict__ z_row,
                         float* __restrict__ lse_row, int V, float grad_scale, float z_weight, int write_grad,
                         int* __restrict__ status) {
  extern __shared__ __align__(128) unsigned char ce_row_smem[];
  __shared__ __align__(8) uint64_t bar;
  __shared__ float red[2][32];
  __shared__ int abort_flag;
  const long long row = blockIdx.x;
  __nv_bfloat16* grow = logits + row * ld;
  uint4* srow = reinterpret_cast<uint4*>(ce_row_smem);
  const int nvec = V >> 3;
  const uint32_t bytes = (uint32_t)V * 2u;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (mask[row] == 0) {
    if (write_grad) {
      const uint4 z = make_uint4(0, 0, 0, 0);
      for (int v = threadIdx.x; v < nvec; v += kCeThreads) reinterpret_cast<uint4*>(grow)[v] = z;
    }
    if (threadIdx.x == 0) { loss_row[row] = 0.f; z_row[row] = 0.f; if (lse_row) lse_row[row] = 0.f; }
    return;
  }
  if (threadIdx.x == 0) {
    abort_flag = 0;
    b200::mbar_init(&bar, 1);
    b200::mbar_fence_init();
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    b200::mbar_expect_tx(&bar, bytes);
    for (uint32_t off = 0; off < bytes; off += kCeChunkBytes)
      b200::bulk_g2s(ce_row_smem + off, reinterpret_cast<const unsigned char*>(grow) + off,
                     min(kCeChunkBytes, bytes - off), &bar);
  }
  const b200::AbortCtx ab{&abort_flag, status};
  const bool ok = b200::mbar_wait(&bar, 0, ab, b200::ERR_WAIT_FULL);
  if (!__syncthreads_and(ok)) {
    // the limit ran out (recorded in the status word): give the copies still in flight one more bounded wait so
    // that they do not land in shared memory of a CTA that has left, then leave without writing anything
    if (threadIdx.x == 0) {
      const uint64_t t0 = b200::globaltimer_ns();
      while (!b200::mbar_try_wait(&bar, 0) && b200::globaltimer_ns() - t0 < b200::kWaitLimitNs) {}
    }
    __syncthreads();
    return;
  }
  const int tgt = targets[row];
  const float tl = __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(ce_row_smem)[tgt]);
  // pass 1: the maximum, on packed pairs (no conversion to fp32: bf16 compares exactly)
  __nv_bfloat162 m2v = __float2bfloat162_rn(-INFINITY);
  for (int v = threadIdx.x; v < nvec; v += kCeThreads) {
    const uint4 q = srow[v];
    m2v = __hmax2(m2v, *reinterpret_cast<const __nv_bfloat162*>(&q.x));
    m2v = __hmax2(m2v, *reinterpret_cast<const __nv_bfloat162*>(&q.y));
    m2v = __hmax2(m2v, *reinterpret_cast<const __nv_bfloat162*>(&q.z));
    m2v = __hmax2(m2v, *reinterpret_cast<const __nv_bfloat162*>(&q.w));
  }
  float m = fmaxf(__low2float(m2v), __high2float(m2v));
  m = warp_max(m);
  if (lane == 0) red[0][warp] = m;
  __syncthreads();
  m = warp_max(red[0][lane & (kCeThreads / 32 - 1)]);
  constexpr float kLog2e = 1.4426950408889634f;
  const float m2 = m * kLog2e;
  float s = 0.f;
  for (int v = threadIdx.x; v < nvec; v += kCeThreads) {
    float f[8];
    unpack8(srow[v], f);
#pragma unroll
    for (int k = 0; k < 8; ++k) s += b200::ex2_approx(fmaf(f[k], kLog2e, -m2));
  }
  s = warp_sum(s);
  if (lane == 0) red[1][warp] = s;
  __syncthreads();
  s = warp_sum(lane < kCeThreads / 32 ? red[1][lane] : 0.f);
  const float lse = m + logf(s);
  if (threadIdx.x == 0) {
    loss_row[row] = lse - tl;
    z_row[row] = lse * lse;
    if (lse_row) lse_row[row] = lse;
  }
  if (!write_grad) return;
  const float coef = grad_scale * (1.f + 2.f * z_weight * lse) / s;
  for (int v = threadIdx.x; v < nvec; v += kCeThreads) {
    float f[8];
    unpack8(srow[v], f);
#pragma unroll
    for (int k = 0; k < 8; ++k) f[k] = coef * b200::ex2_approx(fmaf(f[k], kLog2e, -m2));
    const int off = tgt - v * 8;
    if (off >= 0 && off < 8) {
#pragma unroll
      for (int k = 0; k < 8; ++k)
        if (k == off) f[k] -= grad_scale;
    }
    srow[v] = pack8(f);
  }
  b200::fence_proxy_async_smem();      // the generic-proxy writes above are read by the bulk store below
  __syncthreads();
  if (threadIdx.x == 0) {
    for (uint32_t off = 0; off < bytes; off += kCeChunkBytes)
      b200::bulk_s2g(reinterpret_cast<unsigned char*>(grow) + off, ce_row_smem + off, min(kCeChunkBytes, bytes - off));
    b200::tma_commit_group();
    b200::tma_wait_group_read<0>();    // shared memory stays valid until the store has read it
  }
}

// ------------------------------------------------------------------------------------------------
// Flat-arena AdamW: p, m, v fp32 [n]; g bf16 or fp32 [n]; writes the bf16 shadow of p.
//   g' = g * gscale[0] (clip factor, device scalar; nullptr = 1)
//   m = b1 m + (1-b1) g';  v = b2 v + (1-b2) g'^2;  p -= lr * (mhat / (sqrt(vhat) + eps) + wd p)
// lr, bias corrections come from the host each step (schedule evaluated at the old step count).
// ------------------------------------------------------------------------------------------------
template <typename GT>
__global__ void adamw_kernel(float* __restrict__ p, float* __restrict__ m, float* __restrict__ v,
                             const GT* __restrict__ g, __nv_bfloat16* __restrict__ shadow,
                             const float* __restrict__ gscale, long long n, float lr, float b1, float b2, float eps,
                             float wd, float bc1, float bc2) {
  const float gs = gscale ? gscale[0] : 1.f;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    float gi;
    if constexpr (sizeof(GT) == 2)
      gi = __bfloat162float(g[i]) * gs;
    else
      gi = g[i] * gs;
    const float mi = b1 * m[i] + (1.f - b1) * gi;
    const float vi = b2 * v[i] + (1.f - b2) * gi * gi;
    m[i] = mi;
    v[i] = vi;
    const float mhat = mi / bc1;
    const float vhat = vi / bc2;
    float pi = p[i];
    pi -= lr * (mhat / (sqrtf(vhat) + eps) + wd * pi);
    p[i] = pi;
    if (shadow) shadow[i] = __float2bfloat16(pi);
  }
}

// Four elements per thread with 16-byte accesses (n % 4 == 0, 16-byte aligned arenas).
template <typename GT>
__global__ void __launch_bounds__(256)
adamw_vec4_kernel(float4* __restrict__ p, float4* __restrict__ m, float4* __restrict__ v, const GT* __restrict__ g,
                  __nv_bfloat16* __restrict__ shadow, const float* __restrict__ gscale, long long nvec, float lr,
                  float b1, float b2, float eps, float wd, float bc1, float bc2) {
  const float gs = gscale ? gscale[0] : 1.f;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec;
       i += (long long)gridDim.x * blockDim.x) {
    float gi[4];
    if constexpr (sizeof(GT) == 2) {
      const uint2 raw = reinterpret_cast<const uint2*>(g)[i];
      const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
      const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
      gi[0] = a.x; gi[1] = a.y; gi[2] = b.x; gi[3] = b.y;
    } else {
      const float4 raw = reinterpret_cast<const float4*>(g)[i];
      gi[0] = raw.x; gi[1] = raw.y; gi[2] = raw.z; gi[3] = raw.w;
    }
    const float4 m4 = m[i], v4 = v[i], p4 = p[i];
    float mi[4] = {m4.x, m4.y, m4.z, m4.w}, vi[4] = {v4.x, v4.y, v4.z, v4.w}, pi[4] = {p4.x, p4.y, p4.z, p4.w};
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float gk = gi[k] * gs;
      mi[k] = b1 * mi[k] + (1.f - b1) * gk;
      vi[k] = b2 * vi[k] + (1.f - b2) * gk * gk;
      const float mhat = mi[k] / bc1;
      const float vhat = vi[k] / bc2;
      pi[k] -= lr * (mhat / (sqrtf(vhat) + eps) + wd * pi[k]);
    }
    m[i] = make_float4(mi[0], mi[1], mi[2], mi[3]);
    v[i] = make_float4(vi[0], vi[1], vi[2], vi[3]);
    p[i] = make_float4(pi[0], pi[1], pi[2], pi[3]);
    if (shadow) {
      __nv_bfloat162 lo = __floats2bfloat162_rn(pi[0], pi[1]);
      __nv_bfloat162 hi = __floats2bfloat162_rn(pi[2], pi[3]);
      uint2 pk;
      pk.x = *reinterpret_cast<uint32_t*>(&lo);
      pk.y = *reinterpret_cast<uint32_t*>(&hi);
      reinterpret_cast<uint2*>(shadow)[i] = pk;
    }
  }
}

// sum of squares, two deterministic stages: per-block partials, then one block folds them
template <typename T>
__global__ void sumsq_partial_kernel(const T* __restrict__ x, long long n, float* __restrict__ partial) {
  __shared__ float red[32];
  float s = 0.f;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    float f;
    if constexpr (sizeof(T) == 2)
      f = __bfloat162float(x[i]);
    else
      f = x[i];
    s += f * f;
  }
  s = warp_sum(s);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = s;
  __syncthreads();
  if (threadIdx.x < 32) {
    s = threadIdx.x < (blockDim.x >> 5) ? red[threadIdx.x] : 0.f;
    s = warp_sum(s);
    if (threadIdx.x == 0) partial[blockIdx.x] = s;
  }
}
__global__ void sumsq_final_kernel(const float* __restrict__ partial, int nparts, float* __restrict__ out,
                                   int accumulate) {
  __shared__ float red[32];
  float s = 0.f;
  for (int i = threadIdx.x; i < nparts; i += blockDim.x) s += partial[i];
  s = warp_sum(s);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = s;
  __syncthreads();
  if (threadIdx.x < 32) {
    s = threadIdx.x < (blockDim.x >> 5) ? red[threadIdx.x] : 0.f;
    s = warp_sum(s);
    if (threadIdx.x == 0) out[0] = accumulate ? out[0] + s : s;
  }
}

// fp32 -> bf16 cast with scale (used for the bf16 shadow of Muon-updated weights and grad casts)
__global__ void cast_f32_bf16_kernel(const float* __restrict__ x, __nv_bfloat16* __restrict__ y, long long n,
                                     float scale) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
    y[i] = __float2bfloat16(x[i] * scale);
}

inline int grid_for(long long work_items, int block, int per_sm = 8) {
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  long long blocks = (work_items + block - 1) / block;
  long long cap = (long long)sms * per_sm;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  return (int)blocks;
}

}  // namespace

#define STREAM(s) reinterpret_cast<cudaStream_t>(s)
#define LAST_ERR() static_cast<int>(cudaGetLastError())

extern "C" int b200_rmsnorm_fwd(const void* x, const void* delta, const void* w, void* res_out, void* y, void* rstd,
                                int rows, int H, float eps, void* stream) {
  if (H % 8) return -2;
  if (rows > 0 && rows <= 512) {
    // few rows = a decode step: launched as a dependent so that it is resident when its predecessor ends
    return static_cast<int>(b200host::launch_kernel(
        rmsnorm_fwd_row_kernel, dim3(rows), dim3(256), 0, STREAM(stream), b200host::pdl_enabled() != 0,
        (const __nv_bfloat16*)x, (const __nv_bfloat16*)delta, (const float*)w, (__nv_bfloat16*)res_out,
        (__nv_bfloat16*)y, (float*)rstd, H, eps));
  }
  const int grid = grid_for((long long)rows, kWarpsPerBlock, 8);
#define RMS_FWD(NV)                                                                                         \
  rmsnorm_fwd_reg_kernel<NV><<<grid, kWarpsPerBlock * 32, 0, STREAM(stream)>>>(                             \
      (const __nv_bfloat16*)x, (const __nv_bfloat16*)delta, (const float*)w, (__nv_bfloat16*)res_out,       \
      (__nv_bfloat16*)y, (float*)rstd, rows, eps);                                                         \
  return LAST_ERR()
  switch (H) {
    case 1024: RMS_FWD(4);
    case 2048: RMS_FWD(8);
    case 4096: RMS_FWD(16);
    default: break;
  }
#undef RMS_FWD
  rmsnorm_fwd_kernel<<<grid, kWarpsPerBlock * 32, 0, STREAM(stream)>>>(
      (const __nv_bfloat16*)x, (const __nv_bfloat16*)delta, (const float*)w, (__nv_bfloat16*)res_out,
      (__nv_bfloat16*)y, (float*)rstd, rows, H, eps);
  return LAST_ERR();
}
extern "C" int b200_rmsnorm_bwd(const void* x, const void* w, const void* rstd, const void* dy, const void* dres,
                                void* dx, void* dw, int rows, int H, void* stream) {
  if (H % 8 || H * 4 > 48 * 1024) return -2;
  if (H == 4096 || H == 8192) {   // narrower rows: the warp-per-row kernel below measured faster
#define RMS_BWD_COLS(VEC, THREADS, MINB)                                                                        \
  rmsnorm_bwd_cols_kernel<VEC, THREADS, MINB><<<grid_for((long long)rows, 1, MINB), THREADS, 0, STREAM(stream)>>>( \
      (const __nv_bfloat16*)x, (const float*)w, (const float*)rstd, (const __nv_bfloat16*)dy,                   \
      (const __nv_bfloat16*)dres, (__nv_bfloat16*)dx, (float*)dw, rows, H)
    if (H == 4096) RMS_BWD_COLS(2, 256, 2);
    else RMS_BWD_COLS(2, 512, 1);
#undef RMS_BWD_COLS
    return LAST_ERR();
  }
  const int grid = grid_for((long long)rows, kWarpsPerBlock, 2);
#define RMS_BWD(NV)                                                                                     \
  rmsnorm_bwd_kernel<NV><<<grid, kWarpsPerBlock * 32, H * sizeof(float), STREAM(stream)>>>(              \
      (const __nv_bfloat16*)x, (const float*)w, (const float*)rstd, (const __nv_bfloat16*)dy,            \
      (const __nv_bfloat16*)dres, (__nv_bfloat16*)dx, (float*)dw, rows, H)
  switch (H) {
    case 256: RMS_BWD(1); break;
    case 512: RMS_BWD(2); break;
    case 1024: RMS_BWD(4); break;
    case 2048: RMS_BWD(8); break;
    case 4096: RMS_BWD(16); break;
    default: RMS_BWD(0); break;
  }
#undef RMS_BWD
  return LAST_ERR();
}
static int lanes_per_head(int D) {
  int lph = 1;
  while (lph * 8 < D) lph <<= 1;
  return lph;
}
extern "C" int b200_qknorm_rope_fwd(const void* in, long long in_stride, void* out, long long out_stride,
                                    const void* w, const void* positions, void* rstd, long long tokens, int heads,
                                    int D, float eps, float theta, int rope, void* stream) {
  if (D % 8 || D > 256) return -2;
  const int lph = lanes_per_head(D);
  const int grid = grid_for((tokens * heads + 32 / lph - 1) / (32 / lph), kWarpsPerBlock, 8);
  return static_cast<int>(b200host::launch_kernel(qknorm_rope_fwd_kernel, dim3(grid), dim3(kWarpsPerBlock * 32), 0,
                                                  STREAM(stream), tokens <= 512 && b200host::pdl_enabled() != 0,
      (const __nv_bfloat16*)in, in_stride, (__nv_bfloat16*)out, out_stride, (const float*)w, (const int*)positions,
      (float*)rstd, tokens, heads, D, eps, log2f(theta), rope, lph, nullptr, heads));
}
// Query and key heads of a packed projection in one launch: the first heads_q heads use wq, the next heads_k use wk
// (both or neither given); rstd is [tokens, heads_q + heads_k].
extern "C" int b200_qknorm_rope_fwd_qk(const void* in, long long in_stride, void* out, long long out_stride,
                                       const void* wq, const void* wk, const void* positions, void* rstd,
                                       long long tokens, int heads_q, int heads_k, int D, float eps, float theta,
                                       int rope, void* stream) {
  if (D % 8 || D > 256 || (wq == nullptr) != (wk == nullptr)) return -2;
  const int heads = heads_q + heads_k;
  const int lph = lanes_per_head(D);
  const int grid = grid_for((tokens * heads + 32 / lph - 1) / (32 / lph), kWarpsPerBlock, 8);
  return static_cast<int>(b200host::launch_kernel(qknorm_rope_fwd_kernel, dim3(grid), dim3(kWarpsPerBlock * 32), 0,
                                                  STREAM(stream), tokens <= 512 && b200host::pdl_enabled() != 0,
      (const __nv_bfloat16*)in, in_stride, (__nv_bfloat16*)out, out_stride, (const float*)wq, (const int*)positions,
      (float*)rstd, tokens, heads, D, eps, log2f(theta), rope, lph, (const float*)wk, heads_q));
}
extern "C" int b200_qknorm_rope_bwd(const void* in, long long in_stride, const void* dout, long long dout_stride,
                                    void* din, long long din_stride, const void* w, const void* positions,
                                    const void* rstd, void* dw, long long tokens, int heads, int D, float theta,
                                    int rope, void* stream) {
  if (D % 8 || D > 256) return -2;
  const int lph = lanes_per_head(D);
  const int grid = grid_for((tokens * heads + 32 / lph - 1) / (32 / lph), kWarpsPerBlock, 4);
  qknorm_rope_bwd_kernel<<<grid, kWarpsPerBlock * 32, 0, STREAM(stream)>>>(
      (const __nv_bfloat16*)in, in_stride, (const __nv_bfloat16*)dout, dout_stride, (__nv_bfloat16*)din, din_stride,
      (const float*)w, (const int*)positions, (const float*)rstd, (float*)dw, tokens, heads, D, log2f(theta), rope,
      lph, nullptr, nullptr, heads);
  return LAST_ERR();
}
extern "C" int b200_qknorm_rope_bwd_qk(const void* in, long long in_stride, const void* dout, long long dout_stride,
                                       void* din, long long din_stride, const void* wq, const void* wk,
                                       const void* positions, const void* rstd, void* dwq, void* dwk, long long tokens,
                                       int heads_q, int heads_k, int D, float theta, int rope, void* stream) {
  if (D % 8 || D > 256 || (wq == nullptr) != (wk == nullptr)) return -2;
  const int heads = heads_q + heads_k;
  const int lph = lanes_per_head(D);
  const int grid = grid_for((tokens * heads + 32 / lph - 1) / (32 / lph), kWarpsPerBlock, 4);
  qknorm_rope_bwd_kernel<<<grid, kWarpsPerBlock * 32, 0, STREAM(stream)>>>(
      (const __nv_bfloat16*)in, in_stride, (const __nv_bfloat16*)dout, dout_stride, (__nv_bfloat16*)din, din_stride,
      (const float*)wq, (const int*)positions, (const float*)rstd, (float*)dwq, tokens, heads, D, log2f(theta), rope,
      lph, (const float*)wk, (float*)dwk, heads_q);
  return LAST_ERR();
}
extern "C" int b200_swiglu_fwd(const void* gu, void* h, long long rows, int I, void* stream) {
  if (I % 8 || rows * (I / 8) >= (1LL << 32)) return -2;
  return static_cast<int>(b200host::launch_kernel(swiglu_fwd_kernel, dim3(grid_for(rows * (I / 8), 256)), dim3(256), 0,
                                                  STREAM(stream), rows <= 512 && b200host::pdl_enabled() != 0,
                                                  (const __nv_bfloat16*)gu, (__nv_bfloat16*)h, rows, I));
}
extern "C" int b200_swiglu_bwd(const void* gu, const void* dh, void* dgu, long long rows, int I, void* stream) {
  if (I % 8 || rows * (I / 8) >= (1LL << 32)) return -2;
  swiglu_bwd_kernel<<<grid_for(rows * (I / 8), 256), 256, 0, STREAM(stream)>>>(
      (const __nv_bfloat16*)gu, (const __nv_bfloat16*)dh, (__nv_bfloat16*)dgu, rows, I);
  return LAST_ERR();
}
extern "C" int b200_sigmoid_gate_fwd(const void* a, const void* gate, void* out, long long n, void* stream) {
  if (n % 8) return -2;
  sigmoid_gate_fwd_kernel<<<grid_for(n / 8, 256), 256, 0, STREAM(stream)>>>(
      (const __nv_bfloat16*)a, (const __nv_bfloat16*)gate, (__nv_bfloat16*)out, n / 8);
  return LAST_ERR();
}
extern "C" int b200_sigmoid_gate_bwd(const void* a, const void* gate, const void* dout, void* da, void* dgate,
                                     long long n, void* stream) {
  if (n % 8) return -2;
  sigmoid_gate_bwd_kernel<<<grid_for(n / 8, 256), 256, 0, STREAM(stream)>>>(
      (const __nv_bfloat16*)a, (const __nv_bfloat16*)gate, (const __nv_bfloat16*)dout, (__nv_bfloat16*)da,
      (__nv_bfloat16*)dgate, n / 8);
  return LAST_ERR();
}
extern "C" int b200_embedding_fwd(const void* ids, const void* table, void* out, long long tokens, int H,
                                  float scale, void* stream) {
  if (H % 8) return -2;
  embedding_fwd_kernel<<<grid_for(tokens * (H / 8), 256), 256, 0, STREAM(stream)>>>(
      (const int*)ids, (const __nv_bfloat16*)table, (__nv_bfloat16*)out, tokens, H, scale);
  return LAST_ERR();
}
extern "C" int b200_embedding_bwd(const void* ids, const void* dout, void* dtable, long long tokens, int H,
                                  float scale, void* stream) {
  if (H % 8) return -2;
  embedding_bwd_kernel<<<grid_for(tokens * (H / 8), 256), 256, 0, STREAM(stream)>>>(
      (const int*)ids, (const __nv_bfloat16*)dout, (float*)dtable, tokens, H, scale);
  return LAST_ERR();
}
extern "C" int b200_ce_fwd_bwd(void* logits, long long ld, const void* targets, const void* mask, void* loss_row,
                               void* z_row, void* lse_row, int rows, int V, float grad_scale, float z_weight,
                               int write_grad, void* status, void* stream) {
  if (rows <= 0) return 0;
  if (ld % 8) return -1;  // rows must stay 16-byte aligned for the vector path
  const size_t row_bytes = (size_t)V * 2;
  if (V % 8 == 0 && row_bytes <= 200 * 1024 && (reinterpret_cast<uintptr_t>(logits) & 15u) == 0 && status) {
    static bool configured[b200host::kMaxDevices] = {};
    if (int rc = b200host::ensure_dynamic_smem(ce_fwd_bwd_staged_kernel, 200 * 1024, configured)) return rc;
    ce_fwd_bwd_staged_kernel<<<rows, kCeThreads, row_bytes, STREAM(stream)>>>(
        (__nv_bfloat16*)logits, ld, (const int*)targets, (const uint8_t*)mask, (float*)loss_row, (float*)z_row,
        (float*)lse_row, V, grad_scale, z_weight, write_grad, (int*)status);
    return LAST_ERR();
  }
  ce_fwd_bwd_kernel<<<rows, 512, 0, STREAM(stream)>>>((__nv_bfloat16*)logits, ld, (const int*)targets,
                                                      (const uint8_t*)mask, (float*)loss_row, (float*)z_row,
                                                      (float*)lse_row, V, grad_scale, z_weight, write_grad);
  return LAST_ERR();
}
extern "C" int b200_adamw(void* p, void* m, void* v, const void* g, int g_is_bf16, void* shadow, const void* gscale,
                          long long n, float lr, float b1, float b2, float eps, float wd, float bc1, float bc2,
                          void* stream) {
  if (n <= 0) return 0;
  auto misaligned = [](const void* q, uintptr_t a) { return (reinterpret_cast<uintptr_t>(q) & (a - 1)) != 0; };
  if (n % 4 == 0 && !misaligned(p, 16) && !misaligned(m, 16) && !misaligned(v, 16) &&
      !misaligned(g, g_is_bf16 ? 8 : 16) && !misaligned(shadow, 8)) {
    const int vgrid = grid_for(n / 4, 256, 8);
    if (g_is_bf16)
      adamw_vec4_kernel<__nv_bfloat16><<<vgrid, 256, 0, STREAM(stream)>>>(
          (float4*)p, (float4*)m, (float4*)v, (const __nv_bfloat16*)g, (__nv_bfloat16*)shadow, (const float*)gscale,
          n / 4, lr, b1, b2, eps, wd, bc1, bc2);
    else
      adamw_vec4_kernel<float><<<vgrid, 256, 0, STREAM(stream)>>>((float4*)p, (float4*)m, (float4*)v, (const float*)g,
                                                                 (__nv_bfloat16*)shadow, (const float*)gscale, n / 4,
                                                                 lr, b1, b2, eps, wd, bc1, bc2);
    return LAST_ERR();
  }
  const int grid = grid_for(n, 256, 8);
  if (g_is_bf16)
    adamw_kernel<__nv_bfloat16><<<grid, 256, 0, STREAM(stream)>>>((float*)p, (float*)m, (float*)v,
                                                                   (const __nv_bfloat16*)g, (__nv_bfloat16*)shadow,
                                                                   (const float*)gscale, n, lr, b1, b2, eps, wd, bc1, bc2);
  else
    adamw_kernel<float><<<grid, 256, 0, STREAM(stream)>>>((float*)p, (float*)m, (float*)v, (const float*)g,
                                                           (__nv_bfloat16*)shadow, (const float*)gscale, n, lr, b1, b2,
                                                           eps, wd, bc1, bc2);
  return LAST_ERR();
}
// scratch: at least 1024 floats.  out[0] (+)= sum(x^2)
extern "C" int b200_sumsq(const void* x, int is_bf16, long long n, void* scratch, void* out, int accumulate,
                          void* stream) {
  int grid = grid_for(n, 512, 4);
  if (grid > 1024) grid = 1024;
  if (is_bf16)
    sumsq_partial_kernel<__nv_bfloat16><<<grid, 512, 0, STREAM(stream)>>>((const __nv_bfloat16*)x, n, (float*)scratch);
  else
    sumsq_partial_kernel<float><<<grid, 512, 0, STREAM(stream)>>>((const float*)x, n, (float*)scratch);
  sumsq_final_kernel<<<1, 256, 0, STREAM(stream)>>>((const float*)scratch, grid, (float*)out, accumulate);
  return LAST_ERR();
}
extern "C" int b200_cast_f32_bf16(const void* x, void* y, long long n, float scale, void* stream) {
  if (n <= 0) return 0;
  cast_f32_bf16_kernel<<<grid_for(n, 256, 8), 256, 0, STREAM(stream)>>>((const float*)x, (__nv_bfloat16*)y, n, scale);
  return LAST_ERR();
}

// ws: fp32 [n] holding split-K sums (zeroed again on return), out: bf16 [n]; n % 4 == 0, both 16-byte aligned.
extern "C" int b200_splitk_finish(void* ws, void* out, long long n, void* stream) {
  if (n <= 0 || n % 4) return -2;
  const long long n4 = n / 4;
  long long blocks = (n4 + 255) / 256;
  if (blocks > 148 * 8) blocks = 148 * 8;
  return static_cast<int>(b200host::launch_kernel(splitk_finish_kernel, dim3((int)blocks), dim3(256), 0, STREAM(stream),
                                                  b200host::pdl_enabled() != 0, (float*)ws, (__nv_bfloat16*)out, n4));
}
