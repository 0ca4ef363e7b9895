// Element-wise halves of the Muon update for sm_100a, written so that each logical matrix is touched twice:
//   1. momentum:  m <- beta m + (1 - beta) g';  u = (1 - beta) g' + beta m  (Nesterov),  g' = g * clip
//                 u is written as bf16 into a stacking buffer (input of the batched Newton-Schulz GEMMs) and
//                 sum(u^2) is accumulated for the Frobenius normalisation;
//   2. apply:     w <- w (1 - lr wd) - step * o;  compute copy (bf16) <- w
// Rules restated from the reference transform (src/jaxtitan/optim/muon.py:65-167).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace {

// blockIdx.y walks a batch of equal-size matrices: matrix b starts `stride` elements after matrix b-1 in g and m
// (they may be row slices of a fused parameter) and is written densely, `n` elements apart, into u; sumsq[b].
__global__ void muon_momentum_kernel(const float* __restrict__ g_all, float* __restrict__ m_all,
                                     __nv_bfloat16* __restrict__ u_all, float* __restrict__ sumsq_all,
                                     const float* __restrict__ clip, long long n, long long stride, int batch,
                                     float beta, int nesterov) {
  __shared__ float red[32];
  const float c = clip ? clip[0] : 1.f;
  const long long nvec = n >> 2;
  for (int b = blockIdx.y; b < batch; b += gridDim.y) {
  const float* g = g_all + b * stride;
  float* m = m_all + b * stride;
  __nv_bfloat16* u = u_all + b * n;
  float* sumsq = sumsq_all + b;
  float acc = 0.f;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec;
       i += (long long)gridDim.x * blockDim.x) {
    float4 gv = reinterpret_cast<const float4*>(g)[i];
    float4 mv = reinterpret_cast<float4*>(m)[i];
    float gs[4] = {gv.x * c, gv.y * c, gv.z * c, gv.w * c};
    float ms[4] = {mv.x, mv.y, mv.z, mv.w};
    float us[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      ms[k] = beta * ms[k] + (1.f - beta) * gs[k];
      us[k] = nesterov ? (1.f - beta) * gs[k] + beta * ms[k] : ms[k];
      acc += us[k] * us[k];
    }
    reinterpret_cast<float4*>(m)[i] = make_float4(ms[0], ms[1], ms[2], ms[3]);
    __nv_bfloat162 lo = __floats2bfloat162_rn(us[0], us[1]);
    __nv_bfloat162 hi = __floats2bfloat162_rn(us[2], us[3]);
    uint2 packed;
    packed.x = *reinterpret_cast<uint32_t*>(&lo);
    packed.y = *reinterpret_cast<uint32_t*>(&hi);
    reinterpret_cast<uint2*>(u)[i] = packed;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x < 32) {
    acc = threadIdx.x < (blockDim.x >> 5) ? red[threadIdx.x] : 0.f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if (threadIdx.x == 0) atomicAdd(sumsq, acc);
  }
  __syncthreads();
  }
}

__global__ void muon_apply_kernel(float* __restrict__ w_all, const __nv_bfloat16* __restrict__ o_all,
                                  __nv_bfloat16* __restrict__ shadow_all, long long n, long long stride, int batch,
                                  float decay, float step) {
  const long long nvec = n >> 2;
  for (int b = blockIdx.y; b < batch; b += gridDim.y) {
  float* w = w_all + b * stride;
  const __nv_bfloat16* o = o_all + b * n;
  __nv_bfloat16* shadow = shadow_all ? shadow_all + b * stride : nullptr;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec;
       i += (long long)gridDim.x * blockDim.x) {
    float4 wv = reinterpret_cast<float4*>(w)[i];
    const uint2 ov = reinterpret_cast<const uint2*>(o)[i];
    const float2 o01 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&ov.x));
    const float2 o23 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&ov.y));
    wv.x = wv.x * decay - step * o01.x;
    wv.y = wv.y * decay - step * o01.y;
    wv.z = wv.z * decay - step * o23.x;
    wv.w = wv.w * decay - step * o23.y;
    reinterpret_cast<float4*>(w)[i] = wv;
    if (shadow) {
      __nv_bfloat162 lo = __floats2bfloat162_rn(wv.x, wv.y);
      __nv_bfloat162 hi = __floats2bfloat162_rn(wv.z, wv.w);
      uint2 packed;
      packed.x = *reinterpret_cast<uint32_t*>(&lo);
      packed.y = *reinterpret_cast<uint32_t*>(&hi);
      reinterpret_cast<uint2*>(shadow)[i] = packed;
    }
  }
  }
}

// x[b] *= 1 / max(sqrt(sumsq[b]), eps) over a [batch, per] bf16 stack
__global__ void scale_by_inv_norm_kernel(__nv_bfloat16* __restrict__ x, const float* __restrict__ sumsq, long long per,
                                         int batch, float eps) {
  const long long nvec = per >> 3;
  for (int b = blockIdx.y; b < batch; b += gridDim.y) {
    const float inv = 1.f / fmaxf(sqrtf(sumsq[b]), eps);
    uint4* base = reinterpret_cast<uint4*>(x + (long long)b * per);
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec;
         i += (long long)gridDim.x * blockDim.x) {
      uint4 v = base[i];
      __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        float2 f = __bfloat1622float2(h[k]);
        h[k] = __floats2bfloat162_rn(f.x * inv, f.y * inv);
      }
      base[i] = v;
    }
  }
}

// p[b] = alpha * I + beta * a[b] for a stack of square bf16 matrices [batch, d, d]
__global__ void affine_identity_kernel(const __nv_bfloat16* __restrict__ a, __nv_bfloat16* __restrict__ p, int d,
                                       long long total, float alpha, float beta) {
  const long long per = (long long)d * d;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const long long r = i % per;
    const int row = (int)(r / d), col = (int)(r % d);
    p[i] = __float2bfloat16(beta * __bfloat162float(a[i]) + (row == col ? alpha : 0.f));
  }
}

// d a multiple of 8: one 16-byte chunk of a row per thread; the diagonal element of row r sits in chunk r / 8
__global__ void affine_identity_vec8_kernel(const uint4* __restrict__ a, uint4* __restrict__ p, int d,
                                            long long chunks, float alpha, float beta) {
  const unsigned cpr = (unsigned)d >> 3;                       // chunks per row
  const unsigned long long cpm = (unsigned long long)cpr * d;  // chunks per matrix
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < chunks;
       i += (long long)gridDim.x * blockDim.x) {
    const unsigned r = (unsigned)((unsigned long long)i % cpm);
    const unsigned row = r / cpr, ch = r - row * cpr;
    uint4 v = a[i];
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&v);
    const int diag = (row >> 3) == ch ? (int)(row & 7u) : -1;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      float2 f = __bfloat1622float2(h[k]);
      f.x = beta * f.x + (diag == 2 * k ? alpha : 0.f);
      f.y = beta * f.y + (diag == 2 * k + 1 ? alpha : 0.f);
      h[k] = __floats2bfloat162_rn(f.x, f.y);
    }
    p[i] = v;
  }
}

int blocks_for(long long items, int block, int per_sm) {
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  long long b = (items + block - 1) / block;
  const long long cap = (long long)sms * per_sm;
  if (b > cap) b = cap;
  return b < 1 ? 1 : (int)b;
}

}  // namespace

extern "C" int b200_muon_momentum(const void* g, void* m, void* u, void* sumsq, const void* clip, long long n,
                                  float beta, int nesterov, void* stream) {
  if (n <= 0 || (n & 3)) return -2;
  muon_momentum_kernel<<<blocks_for(n / 4, 256, 4), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      (const float*)g, (float*)m, (__nv_bfloat16*)u, (float*)sumsq, (const float*)clip, n, n, 1, beta, nesterov);
  return static_cast<int>(cudaGetLastError());
}
// `batch` matrices of `n` elements each, `stride` elements apart in g and m; u is [batch, n]; sumsq is [batch].
extern "C" int b200_muon_momentum_batched(const void* g, void* m, void* u, void* sumsq, const void* clip, long long n,
                                          long long stride, int batch, float beta, int nesterov, void* stream) {
  if (n <= 0 || (n & 3) || (stride & 3) || batch < 1) return -2;
  // about four waves of CTAs in total: many blocks per matrix for a single big matrix, few for a large batch
  const int by = batch > 65535 ? 65535 : batch;
  int bx = blocks_for(n / 4, 256, 4);
  const int per_matrix = (blocks_for(1LL << 40, 256, 4) + by - 1) / by;
  if (bx > per_matrix) bx = per_matrix;
  const dim3 grid(bx < 1 ? 1 : bx, by);
  muon_momentum_kernel<<<grid, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      (const float*)g, (float*)m, (__nv_bfloat16*)u, (float*)sumsq, (const float*)clip, n, stride, batch, beta,
      nesterov);
  return static_cast<int>(cudaGetLastError());
}
extern "C" int b200_muon_apply(void* w, const void* o, void* shadow, long long n, float decay, float step,
                               void* stream) {
  if (n <= 0 || (n & 3)) return -2;
  muon_apply_kernel<<<blocks_for(n / 4, 256, 4), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      (float*)w, (const __nv_bfloat16*)o, (__nv_bfloat16*)shadow, n, n, 1, decay, step);
  return static_cast<int>(cudaGetLastError());
}
// w and shadow: `batch` matrices `stride` elements apart; o is [batch, n].
extern "C" int b200_muon_apply_batched(void* w, const void* o, void* shadow, long long n, long long stride, int batch,
                                       float decay, float step, void* stream) {
  if (n <= 0 || (n & 3) || (stride & 3) || batch < 1) return -2;
  // about four waves of CTAs in total: many blocks per matrix for a single big matrix, few for a large batch
  const int by = batch > 65535 ? 65535 : batch;
  int bx = blocks_for(n / 4, 256, 4);
  const int per_matrix = (blocks_for(1LL << 40, 256, 4) + by - 1) / by;
  if (bx > per_matrix) bx = per_matrix;
  const dim3 grid(bx < 1 ? 1 : bx, by);
  muon_apply_kernel<<<grid, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      (float*)w, (const __nv_bfloat16*)o, (__nv_bfloat16*)shadow, n, stride, batch, decay, step);
  return static_cast<int>(cudaGetLastError());
}
extern "C" int b200_scale_by_inv_norm(void* x, const void* sumsq, long long per, int batch, float eps, void* stream) {
  if (per <= 0 || (per & 7) || batch <= 0) return -2;
  dim3 grid(blocks_for(per / 8, 256, 2), batch > 65535 ? 65535 : batch);
  scale_by_inv_norm_kernel<<<grid, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>((__nv_bfloat16*)x,
                                                                                   (const float*)sumsq, per, batch, eps);
  return static_cast<int>(cudaGetLastError());
}
extern "C" int b200_affine_identity(const void* a, void* p, int d, int batch, float alpha, float beta, void* stream) {
  const long long total = (long long)batch * d * d;
  if (total <= 0) return -2;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  const bool vec = (d % 8 == 0) && (reinterpret_cast<uintptr_t>(a) % 16 == 0) && (reinterpret_cast<uintptr_t>(p) % 16 == 0);
  if (vec)
    affine_identity_vec8_kernel<<<blocks_for(total / 8, 256, 8), 256, 0, s>>>((const uint4*)a, (uint4*)p, d, total / 8,
                                                                            alpha, beta);
  else
    affine_identity_kernel<<<blocks_for(total, 256, 8), 256, 0, s>>>((const __nv_bfloat16*)a, (__nv_bfloat16*)p, d,
                                                                     total, alpha, beta);
  return static_cast<int>(cudaGetLastError());
}
