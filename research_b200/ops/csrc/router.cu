// Mixture-of-experts router math for sm_100a: everything after the router GEMM in one pass per direction, the
// per-layer load statistics, and the SMEBU bias update of all layers in one launch.
//
//   router_fwd    logits [T, E] (bf16 or fp32) -> scores = sigmoid or softmax (fp32), top-k of scores + bias (ties
//                 to the lower expert index, descending order), weights = unbiased scores of the picks, normalised
//                 over the picks for the sigmoid router, times route_scale.  One warp per token, an expert per
//                 lane and stride 32, k rounds of a warp arg-max: no sort, no [T, E] temporaries.
//   router_bwd    dlogits from dweights [T, k] and (optionally) dscores [T, E] (auxiliary losses), same warp layout.
//   router_stats  per-expert assignment counts and importance (sum of weights) with block-local shared-memory
//                 histograms, and the load summary (total, mean, min, max, max violation, entropy) written by the
//                 last block to finish.
//   smebu_update  violation -> tanh step -> mean-centre -> momentum -> bias, one block per MoE layer.
//
// Reference: src/jaxtitan/models/components/moe.py:98-147 (router), 794-840 (statistics);
// src/jaxtitan/steps/moe_balance.py:97-162 (SMEBU).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>

namespace {

constexpr int kMaxPerLane = 32;  // experts per lane: up to 1024 experts
constexpr unsigned kFull = 0xffffffffu;

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(kFull, v, o);
  return v;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(kFull, v, o));
  return v;
}

__device__ __forceinline__ float load_logit(const void* p, int is_bf16, long long i) {
  return is_bf16 ? __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i])
                 : reinterpret_cast<const float*>(p)[i];
}

// VPL = experts per lane (E <= 32 * VPL).
template <int VPL>
__global__ void __launch_bounds__(256)
router_fwd_kernel(const void* __restrict__ logits, int is_bf16, long long ld, const float* __restrict__ bias, int T,
                  int E, int k, int softmax, float route_scale, int* __restrict__ ids, float* __restrict__ weights,
                  float* __restrict__ scores) {
  const int lane = threadIdx.x & 31;
  const int warps = (gridDim.x * blockDim.x) >> 5;
  for (int t = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; t < T; t += warps) {
    float s[VPL], sel[VPL];
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
      const int e = lane + 32 * i;
      s[i] = e < E ? load_logit(logits, is_bf16, (long long)t * ld + e) : -INFINITY;
    }
    if (softmax) {
      float m = -INFINITY;
#pragma unroll
      for (int i = 0; i < VPL; ++i) m = fmaxf(m, s[i]);
      m = warp_max(m);
      float sum = 0.f;
#pragma unroll
      for (int i = 0; i < VPL; ++i) {
        s[i] = lane + 32 * i < E ? expf(s[i] - m) : 0.f;
        sum += s[i];
      }
      sum = warp_sum(sum);
      const float inv = 1.f / sum;
#pragma unroll
      for (int i = 0; i < VPL; ++i) s[i] *= inv;
    } else {
#pragma unroll
      for (int i = 0; i < VPL; ++i) s[i] = lane + 32 * i < E ? 1.f / (1.f + expf(-s[i])) : 0.f;
    }
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
      const int e = lane + 32 * i;
      if (e < E) {
        scores[(long long)t * E + e] = s[i];
        sel[i] = s[i] + bias[e];
      } else {
        sel[i] = -INFINITY;
      }
    }
    // k rounds of arg-max; lane j keeps the j-th pick
    unsigned taken = 0;  // bit i: my expert lane + 32 i is already picked
    int my_id = -1;
    float my_top = 0.f;
    for (int j = 0; j < k; ++j) {
      float best = -INFINITY;
      int best_e = 0x7fffffff;
#pragma unroll
      for (int i = 0; i < VPL; ++i) {
        const int e = lane + 32 * i;
        if (e < E && !((taken >> i) & 1u) && (sel[i] > best || best_e == 0x7fffffff)) {
          best = sel[i];
          best_e = e;
        }
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(kFull, best, o);
        const int oe = __shfl_xor_sync(kFull, best_e, o);
        if (oe != 0x7fffffff && (best_e == 0x7fffffff || ov > best || (ov == best && oe < best_e))) {
          best = ov;
          best_e = oe;
        }
      }
      // the owner marks the pick and publishes its unbiased score
      float top = 0.f;
      if ((best_e & 31) == lane) {
#pragma unroll
        for (int i = 0; i < VPL; ++i)
          if (i == (best_e >> 5)) {
            top = s[i];
            taken |= 1u << i;
          }
      }
      top = __shfl_sync(kFull, top, best_e & 31);
      if (lane == j) {
        my_id = best_e == 0x7fffffff ? -1 : best_e;  // no candidate left (NaN scores): an invalid assignment
        my_top = top;
      }
    }
    float w = my_top * route_scale;
    if (!softmax) {
      const float sum = warp_sum(lane < k ? my_top : 0.f) + 1e-20f;
      w = my_top / sum * route_scale;
    }
    if (lane < k) {
      ids[(long long)t * k + lane] = my_id;
      weights[(long long)t * k + lane] = w;
    }
  }
}

// dlogits from dweights [T, k] (may be null) and dscores [T, E] (may be null).
//   sigmoid: w_j = scale * top_j / (sum top + eps)   ->  dtop_j = scale * (dw_j - sum_i dw_i top_i / S) / S
//            dlogit_e = (dscores_e + sum_j [id_j = e] dtop_j) * s_e (1 - s_e)
//   softmax: w_j = scale * top_j                     ->  dtop_j = scale * dw_j
//            dlogit_e = s_e * (g_e - sum_e' s_e' g_e'),  g = dscores + scattered dtop
template <int VPL>
__global__ void __launch_bounds__(256)
router_bwd_kernel(const float* __restrict__ scores, const int* __restrict__ ids, const float* __restrict__ dweights,
                  const float* __restrict__ dscores, int T, int E, int k, int softmax, float route_scale,
                  void* __restrict__ dlogits, int out_bf16, long long ld) {
  const int lane = threadIdx.x & 31;
  const int warps = (gridDim.x * blockDim.x) >> 5;
  for (int t = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; t < T; t += warps) {
    float s[VPL], g[VPL];
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
      const int e = lane + 32 * i;
      s[i] = e < E ? scores[(long long)t * E + e] : 0.f;
      g[i] = (e < E && dscores) ? dscores[(long long)t * E + e] : 0.f;
    }
    int id = -1;
    float dtop = 0.f;
    if (dweights) {
      float top = 0.f, dw = 0.f;
      if (lane < k) {
        id = ids[(long long)t * k + lane];
        dw = dweights[(long long)t * k + lane];
        if (id >= 0 && id < E) top = scores[(long long)t * E + id]; else dw = 0.f;
      }
      if (softmax) {
        dtop = route_scale * dw;
      } else {
        const float S = warp_sum(top) + 1e-20f;
        const float dot = warp_sum(dw * top);
        dtop = route_scale * (dw - dot / S) / S;
      }
      for (int j = 0; j < k; ++j) {
        const int ej = __shfl_sync(kFull, id, j);
        const float dj = __shfl_sync(kFull, dtop, j);
#pragma unroll
        for (int i = 0; i < VPL; ++i)
          if (ej == lane + 32 * i) g[i] += dj;
      }
    }
    float dot = 0.f;
    if (softmax) {
#pragma unroll
      for (int i = 0; i < VPL; ++i) dot += s[i] * g[i];
      dot = warp_sum(dot);
    }
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
      const int e = lane + 32 * i;
      if (e < E) {
        const float d = softmax ? s[i] * (g[i] - dot) : g[i] * s[i] * (1.f - s[i]);
        if (out_bf16) reinterpret_cast<__nv_bfloat16*>(dlogits)[(long long)t * ld + e] = __float2bfloat16(d);
        else reinterpret_cast<float*>(dlogits)[(long long)t * ld + e] = d;
      }
    }
  }
}

constexpr int kStatChunk = 4096;    // assignments per block of the statistics pass
constexpr int kMaxExperts = 1024;

__device__ __forceinline__ float block_reduce(float v, float* scratch, int op) {  // op 0 sum, 1 max, 2 min
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float other = __shfl_xor_sync(kFull, v, o);
    v = op == 0 ? v + other : (op == 1 ? fmaxf(v, other) : fminf(v, other));
  }
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float r = scratch[0];
  for (int w = 1; w < nwarp; ++w) r = op == 0 ? r + scratch[w] : (op == 1 ? fmaxf(r, scratch[w]) : fminf(r, scratch[w]));
  return r;
}

// out (fp32, zeroed by the caller): counts[E] | importance[E] | summary[8] | block counter (as int).
// summary: total, mean, min, max, max violation, entropy of the load distribution.
__global__ void __launch_bounds__(256)
router_stats_kernel(const int* __restrict__ ids, const float* __restrict__ weights, int A, int E,
                    float* __restrict__ out) {
  __shared__ float s_cnt[kMaxExperts], s_imp[kMaxExperts];
  __shared__ float scratch[8];
  __shared__ int s_last;
  for (int e = threadIdx.x; e < E; e += blockDim.x) s_cnt[e] = 0.f, s_imp[e] = 0.f;
  __syncthreads();
  const int begin = blockIdx.x * kStatChunk, end = min(begin + kStatChunk, A);
  for (int a = begin + threadIdx.x; a < end; a += blockDim.x) {
    const int e = ids[a];
    if (e >= 0 && e < E) {
      atomicAdd(&s_cnt[e], 1.f);
      atomicAdd(&s_imp[e], weights[a]);
    }
  }
  __syncthreads();
  float* counts = out;
  float* importance = out + E;
  float* summary = out + 2 * E;
  int* counter = reinterpret_cast<int*>(out + 2 * E + 8);
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    if (s_cnt[e] != 0.f) atomicAdd(&counts[e], s_cnt[e]);   // whole numbers: exact in any order
    if (s_imp[e] != 0.f) atomicAdd(&importance[e], s_imp[e]);
  }
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) s_last = atomicAdd(counter, 1) == (int)gridDim.x - 1;
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  float sum = 0.f, mx = -INFINITY, mn = INFINITY;
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    const float c = __ldcg(&counts[e]);
    sum += c;
    mx = fmaxf(mx, c);
    mn = fminf(mn, c);
  }
  const float total = block_reduce(sum, scratch, 0);
  mx = block_reduce(mx, scratch, 1);
  mn = block_reduce(mn, scratch, 2);
  float ent = 0.f;
  const float denom = fmaxf(total, 1e-6f);
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    const float p = __ldcg(&counts[e]) / denom;
    if (p > 0.f) ent -= p * logf(p);
  }
  ent = block_reduce(ent, scratch, 0);
  if (threadIdx.x == 0) {
    const float mean = total / (float)E;
    summary[0] = total;
    summary[1] = mean;
    summary[2] = mn;
    summary[3] = mx;
    summary[4] = (mx - mean) / fmaxf(mean, 1e-6f);
    summary[5] = ent;
  }
}

struct LayerPtrs {
  float* bias;
  float* momentum;
};

// One block per MoE layer; counts [L, E] are the global assignment counts of the step.
__global__ void __launch_bounds__(256)
smebu_update_kernel(const float* __restrict__ counts, const LayerPtrs* __restrict__ layers, int E, float load_lr,
                    float clamp, float factor, float* __restrict__ sq_out) {
  __shared__ float scratch[8];
  const float* c = counts + (long long)blockIdx.x * E;
  float* bias = layers[blockIdx.x].bias;
  float* mom = layers[blockIdx.x].momentum;
  float sum = 0.f;
  for (int e = threadIdx.x; e < E; e += blockDim.x) sum += c[e];
  const float mean = block_reduce(sum, scratch, 0) / (float)E;
  const float inv = 1.f / fmaxf(mean, 1e-6f);
  float dsum = 0.f;
  for (int e = threadIdx.x; e < E; e += blockDim.x) dsum += load_lr * tanhf(clamp * (mean - c[e]) * inv);
  const float dmean = block_reduce(dsum, scratch, 0) / (float)E;
  float bsq = 0.f, msq = 0.f;
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    const float delta = load_lr * tanhf(clamp * (mean - c[e]) * inv) - dmean;
    const float m = factor * mom[e] + (1.f - factor) * delta;
    const float b = bias[e] + m;
    mom[e] = m;
    bias[e] = b;
    bsq += b * b;
    msq += m * m;
  }
  bsq = block_reduce(bsq, scratch, 0);
  msq = block_reduce(msq, scratch, 0);
  if (threadIdx.x == 0) {
    sq_out[2 * blockIdx.x] = bsq;
    sq_out[2 * blockIdx.x + 1] = msq;
  }
}

int grid_for_tokens(int T) {
  const int blocks = (T + 7) / 8;  // 8 warps per block, a token per warp
  return blocks < 148 * 8 ? (blocks > 0 ? blocks : 1) : 148 * 8;
}

}  // namespace

#define ROUTER_DISPATCH(VPL_CALL)                      \
  if (E <= 32) { VPL_CALL(1) }                         \
  else if (E <= 64) { VPL_CALL(2) }                    \
  else if (E <= 128) { VPL_CALL(4) }                   \
  else if (E <= 256) { VPL_CALL(8) }                   \
  else if (E <= 512) { VPL_CALL(16) }                  \
  else { VPL_CALL(32) }

extern "C" int b200_router_fwd(const void* logits, int is_bf16, long long ld, const float* bias, int T, int E, int k,
                               int softmax, float route_scale, int* ids, float* weights, float* scores,
                               cudaStream_t stream) {
  if (T <= 0) return 0;
  if (E <= 0 || E > 32 * kMaxPerLane || k <= 0 || k > 32 || k > E) return -1;
#define CALL(V)                                                                                                      \
  router_fwd_kernel<V><<<grid_for_tokens(T), 256, 0, stream>>>(logits, is_bf16, ld, bias, T, E, k, softmax,          \
                                                                 route_scale, ids, weights, scores);
  ROUTER_DISPATCH(CALL)
#undef CALL
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

extern "C" int b200_router_bwd(const float* scores, const int* ids, const float* dweights, const float* dscores, int T,
                               int E, int k, int softmax, float route_scale, void* dlogits, int out_bf16, long long ld,
                               cudaStream_t stream) {
  if (T <= 0) return 0;
  if (E <= 0 || E > 32 * kMaxPerLane || k <= 0 || k > 32 || k > E) return -1;
#define CALL(V)                                                                                                      \
  router_bwd_kernel<V><<<grid_for_tokens(T), 256, 0, stream>>>(scores, ids, dweights, dscores, T, E, k, softmax,     \
                                                                 route_scale, dlogits, out_bf16, ld);
  ROUTER_DISPATCH(CALL)
#undef CALL
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

// Floats the caller must zero for b200_router_stats: counts, importance, summary (8), counter.
extern "C" int b200_router_stats_floats(int E) { return 2 * E + 9; }

extern "C" int b200_router_stats(const int* ids, const float* weights, int A, int E, float* out, cudaStream_t stream) {
  if (E <= 0 || E > kMaxExperts || A <= 0) return -1;
  router_stats_kernel<<<(A + kStatChunk - 1) / kStatChunk, 256, 0, stream>>>(ids, weights, A, E, out);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

// layer_ptrs: device array of {bias, momentum} pointer pairs, one per layer; sq_out [layers, 2].
extern "C" int b200_smebu_update(const float* counts, const void* layer_ptrs, int layers, int E, float load_lr,
                                 float clamp, float factor, float* sq_out, cudaStream_t stream) {
  if (layers <= 0) return 0;
  if (E <= 0) return -1;
  smebu_update_kernel<<<layers, 256, 0, stream>>>(counts, reinterpret_cast<const LayerPtrs*>(layer_ptrs), E, load_lr,
                                                  clamp, factor, sq_out);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}
