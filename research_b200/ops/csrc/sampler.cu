// Next-token sampler for sm_100a: temperature, top-k threshold, categorical draw and log-probability in one kernel.
//
// One CTA per sequence.  The row of logits (bf16 or fp32, a few hundred KB, L2-resident) is read a handful of times:
//   1. radix select (4 passes of 8 bits over an order-preserving integer image of the floats) finds the k-th
//      largest value; everything >= it is kept, so ties at the threshold survive, as in the reference;
//   2. maximum and sum of exp((x - max) / T) over the kept values;
//   3. inverse-CDF draw in index order from a caller-provided uniform number: every thread owns a contiguous slice
//      of the vocabulary, a block scan finds the slice that contains the target mass, its owner walks the slice.
// top_k == 1 is an argmax (first index of the maximum) with log-probability 0.  Deterministic for a given uniform.
//
// Reference semantics: src/jaxtitan/infer/generation.py:225-242, 420-432 (logits / temperature, threshold top-k,
// categorical, log-probability under the filtered distribution).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math_constants.h>
#include <stdint.h>

namespace {

constexpr int kThreads = 1024;

__device__ __forceinline__ uint32_t ordered_bits(float x) {
  const uint32_t u = __float_as_uint(x);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);  // larger float <=> larger integer
}
__device__ __forceinline__ float from_ordered(uint32_t o) {
  const uint32_t u = (o & 0x80000000u) ? (o & 0x7fffffffu) : ~o;
  return __uint_as_float(u);
}

template <typename T>
__device__ __forceinline__ float load_logit(const T* row, int i);
template <>
__device__ __forceinline__ float load_logit<float>(const float* row, int i) { return row[i]; }
template <>
__device__ __forceinline__ float load_logit<__nv_bfloat16>(const __nv_bfloat16* row, int i) {
  return __bfloat162float(row[i]);
}

__device__ __forceinline__ float block_reduce(float v, bool is_max, float* scratch) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float t = __shfl_xor_sync(0xffffffffu, v, o);
    v = is_max ? fmaxf(v, t) : v + t;
  }
  __syncthreads();
  if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = v;
  __syncthreads();
  if (threadIdx.x < 32) {
    v = threadIdx.x < (kThreads >> 5) ? scratch[threadIdx.x] : (is_max ? -CUDART_INF_F : 0.f);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float t = __shfl_xor_sync(0xffffffffu, v, o);
      v = is_max ? fmaxf(v, t) : v + t;
    }
    if (threadIdx.x == 0) scratch[0] = v;
  }
  __syncthreads();
  const float out = scratch[0];
  __syncthreads();
  return out;
}

template <typename T>
__global__ void __launch_bounds__(kThreads)
sample_topk_kernel(const T* __restrict__ logits, long long ld, const float* __restrict__ uniform,
                   long long* __restrict__ token, float* __restrict__ logprob, int V, float inv_temp, int top_k) {
  __shared__ unsigned int hist[256];
  __shared__ float scratch[32];
  __shared__ float chunk_sum[kThreads];
  __shared__ unsigned int s_prefix, s_remaining;
  __shared__ int s_pick;
  const T* row = logits + (long long)blockIdx.x * ld;
  const int tid = threadIdx.x;

  // ---- threshold: k-th largest value (ordered integer image), or "keep everything"
  uint32_t thr_bits = 0u;
  if (top_k > 0 && top_k < V) {
    if (tid == 0) {
      s_prefix = 0u;
      s_remaining = (unsigned)top_k;
    }
    for (int pass = 0; pass < 4; ++pass) {
      const int shift = 24 - 8 * pass;
      if (tid < 256) hist[tid] = 0u;
      __syncthreads();
      const uint32_t prefix = s_prefix;
      const uint32_t mask = pass == 0 ? 0u : (0xffffffffu << (shift + 8));
      for (int i = tid; i < V; i += kThreads) {
        const uint32_t b = ordered_bits(load_logit<T>(row, i));
        if ((b & mask) == prefix) atomicAdd(&hist[(b >> shift) & 255u], 1u);
      }
      __syncthreads();
      if (tid == 0) {
        unsigned remaining = s_remaining;
        int bin = 255;
        for (; bin > 0; --bin) {
          if (hist[bin] >= remaining) break;
          remaining -= hist[bin];
        }
        s_prefix = prefix | ((uint32_t)bin << shift);
        s_remaining = remaining;
      }
      __syncthreads();
    }
    thr_bits = s_prefix;
  }
  const float thr = (top_k > 0 && top_k < V) ? from_ordered(thr_bits) : -CUDART_INF_F;

  // ---- maximum (always kept) and its first index
  float vmax = -CUDART_INF_F;
  for (int i = tid; i < V; i += kThreads) vmax = fmaxf(vmax, load_logit<T>(row, i));
  vmax = block_reduce(vmax, true, scratch);

  if (top_k == 1) {
    if (tid == 0) s_pick = V;
    __syncthreads();
    for (int i = tid; i < V; i += kThreads)
      if (load_logit<T>(row, i) == vmax) atomicMin(&s_pick, i);
    __syncthreads();
    if (tid == 0) {
      token[blockIdx.x] = s_pick;
      logprob[blockIdx.x] = 0.f;
    }
    return;
  }

  // ---- mass of every thread's contiguous slice
  const int per = (V + kThreads - 1) / kThreads;
  const int begin = min(tid * per, V), end = min(begin + per, V);
  float mine = 0.f;
  for (int i = begin; i < end; ++i) {
    const float x = load_logit<T>(row, i);
    if (x >= thr) mine += __expf((x - vmax) * inv_temp);
  }
  chunk_sum[tid] = mine;
  const float total = block_reduce(mine, false, scratch);

  // ---- inverse CDF in index order
  if (tid == 0) {
    float target = uniform[blockIdx.x] * total;
    if (!(target < total)) target = total * 0.99999994f;
    float run = 0.f;
    int owner = kThreads - 1;
    for (int t = 0; t < kThreads; ++t) {
      if (run + chunk_sum[t] > target) {
        owner = t;
        break;
      }
      run += chunk_sum[t];
    }
    const int b = min(owner * per, V), e = min(b + per, V);
    int pick = -1;
    float px = 0.f;
    for (int i = b; i < e; ++i) {
      const float x = load_logit<T>(row, i);
      if (x >= thr) {
        pick = i;  // the last kept index of the slice is the fall-back for rounding at the upper edge
        px = x;
        run += __expf((x - vmax) * inv_temp);
        if (run > target) break;
      }
    }
    if (pick < 0) {  // cannot happen while total > 0; keep the argmax rather than an invalid index
      for (int i = 0; i < V; ++i)
        if (load_logit<T>(row, i) == vmax) { pick = i; px = vmax; break; }
    }
    token[blockIdx.x] = pick;
    logprob[blockIdx.x] = (px - vmax) * inv_temp - __logf(total);
  }
}

}  // namespace

// logits: [B, V] rows `ld` elements apart, bf16 (is_bf16 = 1) or fp32.  uniform: fp32 [B] in [0, 1).
// token: int64 [B]; logprob: fp32 [B].  top_k <= 0 keeps the whole vocabulary.
extern "C" int b200_sample_topk(const void* logits, long long ld, int is_bf16, const void* uniform, void* token,
                                void* logprob, int B, int V, float temperature, int top_k, void* stream) {
  if (B <= 0 || V <= 0 || !(temperature > 0.f)) return -2;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  const float inv_temp = 1.f / temperature;
  if (is_bf16)
    sample_topk_kernel<__nv_bfloat16><<<B, kThreads, 0, s>>>((const __nv_bfloat16*)logits, ld, (const float*)uniform,
                                                            (long long*)token, (float*)logprob, V, inv_temp, top_k);
  else
    sample_topk_kernel<float><<<B, kThreads, 0, s>>>((const float*)logits, ld, (const float*)uniform,
                                                    (long long*)token, (float*)logprob, V, inv_temp, top_k);
  return static_cast<int>(cudaGetLastError());
}
