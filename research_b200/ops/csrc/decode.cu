// Decode attention over a KV cache for sm_100a: one new query token per sequence, GQA, split-KV.
//
// The op is bandwidth bound (every cached K and V row is read once per step), so it runs on the SIMT pipes
// with 16-byte loads: a group of D/8 lanes owns one cache row at a time (8 bf16 per lane), a warp works on
// 32/(D/8) rows at once and keeps an online softmax state (m, l, acc[8]) per query head of the GQA group in
// registers, so K and V are read once for all G heads that share them.  The kv range of a sequence is cut
// into `splits` chunks across CTAs; a second small kernel merges the chunk results with their log-sum-exp
// weights.  Only rows in [lo[b], lengths[b]) are touched: nothing is read from unused pages.
//
// Oracle: softmax(q K^T / sqrt(D)) V in fp32 over the valid rows (reference decode path:
// infer/generation.py:302, models/components/attention.py:213-218, which attends over the whole padded
// cache with a mask).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math_constants.h>
#include <stdint.h>

#include "b200.cuh"
#include "host_util.cuh"

namespace {

constexpr int kWarps = 4;
constexpr float kLog2e = 1.4426950408889634f;

__device__ __forceinline__ float ex2f(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ void unpack8(const uint4& v, float* f) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 t = __bfloat1622float2(h[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}

struct DecodeParams {
  const __nv_bfloat16* q;  // [B, Hq, D]
  const __nv_bfloat16* k;  // [B, rows, Hkv, D] by strides
  const __nv_bfloat16* v;
  const int* lengths;      // [B]
  const int* lo;           // [B] or nullptr
  float* part_o;           // [B, Hq, splits, D]
  float* part_ml;          // [B, Hq, splits, 2]  (m in log2 units, l)
  long long k_row, k_batch, v_row, v_batch;  // element strides between rows (inside a page) and sequences
  long long k_head, v_head;                  // element stride between kv heads
  long long k_page, v_page;                  // element stride between pages
  int page_rows;                             // rows per page (a cache that is not paged passes all of them)
  int B, Hq, Hkv, splits;
  float scale_log2;
};

template <int D, int G>
__global__ void __launch_bounds__(kWarps * 32, (G <= 2 ? 6 : (G == 4 ? 4 : 2))) decode_attn_partial_kernel(const DecodeParams p) {
  constexpr int LPR = D / 8;      // lanes per cache row
  constexpr int RPW = 32 / LPR;   // rows per warp per step
  constexpr int GROUPS = kWarps * RPW;
  __shared__ float s_acc[GROUPS][G][D];
  __shared__ float s_ml[GROUPS][G][2];

  const int split = blockIdx.x, hkv = blockIdx.y, b = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int sub = lane / LPR, l = lane % LPR;
  const int grp = warp * RPW + sub;
  // lane groups run different numbers of rows, so shuffles name only the lanes of the own group
  const uint32_t gmask = LPR == 32 ? 0xffffffffu : (((1u << LPR) - 1u) << (sub * LPR));

  const int len = p.lengths[b];
  const int first = p.lo ? max(p.lo[b], 0) : 0;
  const int span = max(len - first, 0);
  int chunk = (span + p.splits - 1) / p.splits;
  chunk = (chunk + GROUPS - 1) / GROUPS * GROUPS;
  const int begin = first + split * chunk;
  const int end = min(begin + chunk, len);

  float q[G][8], acc[G][8], m[G], lsum[G];
#pragma unroll
  for (int g = 0; g < G; ++g) {
    const __nv_bfloat16* qp = p.q + ((long long)b * p.Hq + hkv * G + g) * D + l * 8;
    unpack8(*reinterpret_cast<const uint4*>(qp), q[g]);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      q[g][i] *= p.scale_log2;
      acc[g][i] = 0.f;
    }
    m[g] = -CUDART_INF_F;
    lsum[g] = 0.f;
  }
  const __nv_bfloat16* kb = p.k + b * p.k_batch + hkv * p.k_head + l * 8;
  const __nv_bfloat16* vb = p.v + b * p.v_batch + hkv * p.v_head + l * 8;
  const int page_rows = p.page_rows;

  // Software pipeline: the loads of the next UNROLL rows are in flight while the current ones are reduced.
  constexpr int UNROLL = 2;
  constexpr int STEP = GROUPS * UNROLL;
  uint4 kr[UNROLL], vr[UNROLL], kn[UNROLL], vn[UNROLL];
  auto fetch = [&](int r0, uint4 (&kd)[UNROLL], uint4 (&vd)[UNROLL]) {
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const int r = r0 + u * GROUPS;
      if (r < end) {
        const int pg = r / page_rows, in = r - pg * page_rows;
        kd[u] = __ldg(reinterpret_cast<const uint4*>(kb + pg * p.k_page + in * p.k_row));
        vd[u] = __ldg(reinterpret_cast<const uint4*>(vb + pg * p.v_page + in * p.v_row));
      }
    }
  };
  int r0 = begin + grp;
  fetch(r0, kr, vr);
  for (; r0 < end; r0 += STEP) {
    fetch(r0 + STEP, kn, vn);
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const int r = r0 + u * GROUPS;
      if (r < end) {  // uniform inside a lane group
        float kf[8], vf[8];
        unpack8(kr[u], kf);
        unpack8(vr[u], vf);
#pragma unroll
        for (int g = 0; g < G; ++g) {
          float s = 0.f;
#pragma unroll
          for (int i = 0; i < 8; ++i) s = fmaf(q[g][i], kf[i], s);
#pragma unroll
          for (int off = LPR >> 1; off > 0; off >>= 1) s += __shfl_xor_sync(gmask, s, off, LPR);
          const float m_new = fmaxf(m[g], s);
          const float alpha = ex2f(m[g] - m_new);
          const float pr = ex2f(s - m_new);
          m[g] = m_new;
          lsum[g] = lsum[g] * alpha + pr;
#pragma unroll
          for (int i = 0; i < 8; ++i) acc[g][i] = fmaf(acc[g][i], alpha, pr * vf[i]);
        }
      }
    }
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      kr[u] = kn[u];
      vr[u] = vn[u];
    }
  }
#pragma unroll
  for (int g = 0; g < G; ++g) {
#pragma unroll
    for (int i = 0; i < 8; ++i) s_acc[grp][g][l * 8 + i] = acc[g][i];
    if (l == 0) {
      s_ml[grp][g][0] = m[g];
      s_ml[grp][g][1] = lsum[g];
    }
  }
  __syncthreads();
  // merge the GROUPS partial states of this CTA: one thread per (g, d)
  for (int idx = threadIdx.x; idx < G * D; idx += kWarps * 32) {
    const int g = idx / D, d = idx % D;
    float mm = -CUDART_INF_F;
#pragma unroll
    for (int j = 0; j < GROUPS; ++j) mm = fmaxf(mm, s_ml[j][g][0]);
    float o = 0.f, ls = 0.f;
    if (mm > -CUDART_INF_F) {
#pragma unroll
      for (int j = 0; j < GROUPS; ++j) {
        const float w = ex2f(s_ml[j][g][0] - mm);
        o = fmaf(s_acc[j][g][d], w, o);
        ls = fmaf(s_ml[j][g][1], w, ls);
      }
    }
    const long long slot = ((long long)b * p.Hq + hkv * G + g) * p.splits + split;
    p.part_o[slot * D + d] = o;
    if (d == 0) {
      p.part_ml[slot * 2] = mm;
      p.part_ml[slot * 2 + 1] = ls;
    }
  }
}

// out[b,h,:] = sum_s w_s o_s / sum_s w_s l_s with w_s = 2^(m_s - max m); a row with no valid kv gives zeros
__global__ void decode_attn_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                         __nv_bfloat16* __restrict__ out, int splits, int D) {
  const long long bh = blockIdx.x;
  const int d = threadIdx.x;
  b200::pdl_launch_dependents();
  b200::pdl_wait();
  if (d >= D) return;
  float mm = -CUDART_INF_F;
  for (int s = 0; s < splits; ++s) mm = fmaxf(mm, part_ml[(bh * splits + s) * 2]);
  float o = 0.f, ls = 0.f;
  if (mm > -CUDART_INF_F) {
    for (int s = 0; s < splits; ++s) {
      const float w = ex2f(part_ml[(bh * splits + s) * 2] - mm);
      o = fmaf(part_o[(bh * splits + s) * D + d], w, o);
      ls = fmaf(part_ml[(bh * splits + s) * 2 + 1], w, ls);
    }
  }
  out[bh * D + d] = __float2bfloat16(ls > 0.f ? o / ls : 0.f);
}

// Cache append for one new token per sequence: row positions[b] of every kv head gets k_new / v_new.
// One thread per 8 elements; k_new / v_new are [B, Hkv, D] views with element strides between sequences.
__global__ void kv_append_kernel(const __nv_bfloat16* __restrict__ k_new, const __nv_bfloat16* __restrict__ v_new,
                                 long long kn_batch, long long vn_batch, __nv_bfloat16* __restrict__ k_cache,
                                 __nv_bfloat16* __restrict__ v_cache, const int* __restrict__ positions,
                                 long long c_batch, long long c_head, long long c_page, long long c_row, int page_rows,
                                 int B, int Hkv, int D) {
  const int per = D / 8;
  const int total = B * Hkv * per;
  b200::pdl_launch_dependents();
  b200::pdl_wait();
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gridDim.x * blockDim.x) {
    const int c = i % per, h = (i / per) % Hkv, b = i / (per * Hkv);
    const int r = positions[b];
    const int pg = r / page_rows, in = r - pg * page_rows;
    const long long dst = b * c_batch + h * c_head + pg * c_page + in * c_row + c * 8;
    *reinterpret_cast<uint4*>(k_cache + dst) = *reinterpret_cast<const uint4*>(k_new + b * kn_batch + h * D + c * 8);
    *reinterpret_cast<uint4*>(v_cache + dst) = *reinterpret_cast<const uint4*>(v_new + b * vn_batch + h * D + c * 8);
  }
}

template <int D>
int launch_partial(const DecodeParams& p, int G, cudaStream_t s) {
  const dim3 grid(p.splits, p.Hkv, p.B);
  switch (G) {
    case 1: decode_attn_partial_kernel<D, 1><<<grid, kWarps * 32, 0, s>>>(p); break;
    case 2: decode_attn_partial_kernel<D, 2><<<grid, kWarps * 32, 0, s>>>(p); break;
    case 4: decode_attn_partial_kernel<D, 4><<<grid, kWarps * 32, 0, s>>>(p); break;
    case 8: decode_attn_partial_kernel<D, 8><<<grid, kWarps * 32, 0, s>>>(p); break;
    default: return -2;
  }
  return static_cast<int>(cudaGetLastError());
}

// ---------------------------------------------------------------------------------------------------------------
// Head-major pages: the rows of one (page, kv head) are contiguous, so a tile of kTile rows of K (or V) is one
// contiguous block.  This variant streams such tiles into shared memory with bulk asynchronous copies
// (cp.async.bulk, completion on an mbarrier) through a ring of kStages slots, so that kStages tiles per CTA are in
// flight while the warps reduce the tile that has landed: the loads no longer wait for the arithmetic of the
// same thread, which is what held the register-resident kernel above at about half of the copy bandwidth.
// The arithmetic, the split-KV scheme and the merge are the same.
// ---------------------------------------------------------------------------------------------------------------
// Measured on B200 (32 x 2304 and 64 x 4096 cached rows, 16 / 8 heads of 128): tiles of 64 rows, 3 slots and 8 warps
// (two CTAs per SM) reach 0.72 / 0.83 of the copy bandwidth; 32-row tiles with 4 warps 0.54 / 0.61, 128-row tiles
// with 16 warps 0.65 / 0.76.
constexpr int kTile = 64;     // cache rows per tile
constexpr int kStages = 3;
constexpr int kPagedWarps = 8;
constexpr int ERR_DECODE_TILE = 31;  // status code: a tile never landed

struct PagedParams {
  const __nv_bfloat16* q;
  const __nv_bfloat16* k;
  const __nv_bfloat16* v;
  const int* lengths;
  const int* lo;
  float* part_o;
  float* part_ml;
  long long batch, head, page;  // element strides of the caches (K and V share them)
  int page_rows;
  int B, Hq, Hkv, splits;
  float scale_log2;
  int* status;
  long long q_batch;            // elements between the query rows of two sequences (heads are D apart)
};

__device__ __forceinline__ void bulk_load(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(b200::smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(src)), "r"(bytes), "r"(b200::smem_u32(bar))
               : "memory");
}

template <int D, int G, int TILE, int STAGES, int WARPS>
__global__ void __launch_bounds__(WARPS * 32) decode_attn_paged_kernel(const PagedParams p) {
  constexpr int LPR = D / 8;
  constexpr int RPW = 32 / LPR;
  constexpr int GROUPS = WARPS * RPW;
  constexpr int ROWS_PER_GROUP = TILE / GROUPS;
  constexpr uint32_t TILE_BYTES = TILE * D * 2;
  static_assert(TILE % GROUPS == 0, "a tile is a whole number of rows per lane group");
  extern __shared__ __align__(128) unsigned char smem[];
  __nv_bfloat16* ks = reinterpret_cast<__nv_bfloat16*>(smem);                           // [STAGES][TILE * D]
  __nv_bfloat16* vs = reinterpret_cast<__nv_bfloat16*>(smem + STAGES * TILE_BYTES);
  float* s_acc = reinterpret_cast<float*>(smem + 2 * STAGES * TILE_BYTES);             // [GROUPS][G][D]
  float* s_ml = s_acc + GROUPS * G * D;                                                 // [GROUPS][G][2]
  __shared__ uint64_t full[STAGES];
  __shared__ int abort_flag;

  const int split = blockIdx.x, hkv = blockIdx.y, b = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int sub = lane / LPR, l = lane % LPR;
  const int grp = warp * RPW + sub;
  const uint32_t gmask = LPR == 32 ? 0xffffffffu : (((1u << LPR) - 1u) << (sub * LPR));

  // launched as a programmatic dependent inside a decode step: resident early, everything in global memory (the
  // row just appended included) is read after the predecessor has completed
  b200::pdl_launch_dependents();
  b200::pdl_wait();
  const int len = p.lengths[b];
  const int first = p.lo ? max(p.lo[b], 0) : 0;
  const int tile_lo = first / TILE;
  const int tile_hi = len > first ? (len + TILE - 1) / TILE : tile_lo;
  const int per = (tile_hi - tile_lo + p.splits - 1) / p.splits;
  const int t_begin = tile_lo + split * per;
  const int n_tiles = max(min(t_begin + per, tile_hi) - t_begin, 0);

  if (threadIdx.x == 0) {
    abort_flag = 0;
    for (int s = 0; s < STAGES; ++s) b200::mbar_init(&full[s], 1);
    b200::mbar_fence_init();
  }
  __syncthreads();
  const b200::AbortCtx ab{&abort_flag, p.status};
  const __nv_bfloat16* kb = p.k + b * p.batch + hkv * p.head;
  const __nv_bfloat16* vb = p.v + b * p.batch + hkv * p.head;
  auto issue = [&](int i) {  // thread 0 only
    const int s = i % STAGES;
    const int r0 = (t_begin + i) * TILE;
    const int pg = r0 / p.page_rows, in = r0 - pg * p.page_rows;
    const long long off = pg * p.page + (long long)in * D;
    b200::mbar_expect_tx(&full[s], 2 * TILE_BYTES);
    bulk_load(ks + s * (TILE * D), kb + off, TILE_BYTES, &full[s]);
    bulk_load(vs + s * (TILE * D), vb + off, TILE_BYTES, &full[s]);
  };
  int issued = 0;
  if (threadIdx.x == 0)
    for (; issued < min(STAGES, n_tiles); ++issued) issue(issued);

  float q[G][8], acc[G][8], m[G], lsum[G];
#pragma unroll
  for (int g = 0; g < G; ++g) {
    const __nv_bfloat16* qp = p.q + (long long)b * p.q_batch + (long long)(hkv * G + g) * D + l * 8;
    unpack8(*reinterpret_cast<const uint4*>(qp), q[g]);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      q[g][i] *= p.scale_log2;
      acc[g][i] = 0.f;
    }
    m[g] = -CUDART_INF_F;
    lsum[g] = 0.f;
  }

  int done = 0;
  for (; done < n_tiles; ++done) {
    const int s = done % STAGES;
    // the verdict is made uniform over the CTA, so that either everybody reduces this tile or everybody leaves
    const bool landed = b200::mbar_wait(&full[s], (done / STAGES) & 1, ab, ERR_DECODE_TILE);
    if (!__syncthreads_and(landed)) break;
    const int r0 = (t_begin + done) * TILE;
    const __nv_bfloat16* kt = ks + s * (TILE * D) + l * 8;
    const __nv_bfloat16* vt = vs + s * (TILE * D) + l * 8;
    // Blocked online softmax: the scores of all rows of this lane group (and all heads of the GQA group) first, as
    // independent dot products and shuffle trees, then one running-maximum update and one rescale per tile.
    float sc[ROWS_PER_GROUP][G];
    bool valid[ROWS_PER_GROUP];
#pragma unroll
    for (int u = 0; u < ROWS_PER_GROUP; ++u) {
      const int j = grp + u * GROUPS;
      const int r = r0 + j;
      valid[u] = r >= first && r < len;  // uniform inside a lane group
      float kf[8];
      unpack8(*reinterpret_cast<const uint4*>(kt + j * D), kf);
#pragma unroll
      for (int g = 0; g < G; ++g) {
        float a = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) a = fmaf(q[g][i], kf[i], a);
        sc[u][g] = a;
      }
    }
#pragma unroll
    for (int off = LPR >> 1; off > 0; off >>= 1) {
#pragma unroll
      for (int u = 0; u < ROWS_PER_GROUP; ++u)
#pragma unroll
        for (int g = 0; g < G; ++g) sc[u][g] += __shfl_xor_sync(gmask, sc[u][g], off, LPR);
    }
    float pr[ROWS_PER_GROUP][G];
#pragma unroll
    for (int g = 0; g < G; ++g) {
      float m_new = m[g];
#pragma unroll
      for (int u = 0; u < ROWS_PER_GROUP; ++u) {
        sc[u][g] = valid[u] ? sc[u][g] : -CUDART_INF_F;  // rows outside the window (their bytes may be anything)
        m_new = fmaxf(m_new, sc[u][g]);
      }
      const float m_use = m_new == -CUDART_INF_F ? 0.f : m_new;  // nothing visible yet: keep the state at zero
      const float alpha = ex2f(m[g] - m_use);
      float psum = 0.f;
#pragma unroll
      for (int u = 0; u < ROWS_PER_GROUP; ++u) {
        pr[u][g] = ex2f(sc[u][g] - m_use);
        psum += pr[u][g];
      }
      m[g] = m_new;
      lsum[g] = lsum[g] * alpha + psum;
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[g][i] *= alpha;
    }
#pragma unroll
    for (int u = 0; u < ROWS_PER_GROUP; ++u) {
      if (valid[u]) {
        float vf[8];
        unpack8(*reinterpret_cast<const uint4*>(vt + (grp + u * GROUPS) * D), vf);
#pragma unroll
        for (int g = 0; g < G; ++g)
#pragma unroll
          for (int i = 0; i < 8; ++i) acc[g][i] = fmaf(pr[u][g], vf[i], acc[g][i]);
      }
    }
    __syncthreads();  // every warp is done with slot s
    if (threadIdx.x == 0 && issued < n_tiles && !abort_flag) issue(issued++);
  }
  if (done < n_tiles) {
    // a wait gave up: the copies already issued still target this CTA's shared memory, so thread 0 waits for them
    // (bounded again) before anybody leaves
    __syncthreads();
    if (threadIdx.x == 0) {
      for (int i = done; i < issued; ++i) {
        const uint64_t t0 = b200::globaltimer_ns();
        while (!b200::mbar_try_wait(&full[i % STAGES], (i / STAGES) & 1) &&
               b200::globaltimer_ns() - t0 < b200::kWaitLimitNs) {
        }
      }
    }
    __syncthreads();
    return;
  }
#pragma unroll
  for (int g = 0; g < G; ++g) {
#pragma unroll
    for (int i = 0; i < 8; ++i) s_acc[(grp * G + g) * D + l * 8 + i] = acc[g][i];
    if (l == 0) {
      s_ml[(grp * G + g) * 2] = m[g];
      s_ml[(grp * G + g) * 2 + 1] = lsum[g];
    }
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < G * D; idx += WARPS * 32) {
    const int g = idx / D, d = idx % D;
    float mm = -CUDART_INF_F;
#pragma unroll
    for (int j = 0; j < GROUPS; ++j) mm = fmaxf(mm, s_ml[(j * G + g) * 2]);
    float o = 0.f, ls = 0.f;
    if (mm > -CUDART_INF_F) {
#pragma unroll
      for (int j = 0; j < GROUPS; ++j) {
        const float w = ex2f(s_ml[(j * G + g) * 2] - mm);
        o = fmaf(s_acc[(j * G + g) * D + d], w, o);
        ls = fmaf(s_ml[(j * G + g) * 2 + 1], w, ls);
      }
    }
    const long long slot = ((long long)b * p.Hq + hkv * G + g) * p.splits + split;
    p.part_o[slot * D + d] = o;
    if (d == 0) {
      p.part_ml[slot * 2] = mm;
      p.part_ml[slot * 2 + 1] = ls;
    }
  }
}

template <int D, int G, int TILE, int STAGES, int WARPS>
constexpr int paged_smem_bytes() {
  return 2 * STAGES * TILE * D * 2 + (WARPS * (32 / (D / 8))) * G * (D + 2) * 4;
}

template <int D, int G, int TILE, int STAGES, int WARPS>
int launch_paged_cfg(const PagedParams& p, cudaStream_t s) {
  constexpr int bytes = paged_smem_bytes<D, G, TILE, STAGES, WARPS>();
  static bool configured[b200host::kMaxDevices] = {};  // per instantiation and device; the attribute is sticky
  if (b200host::ensure_dynamic_smem(decode_attn_paged_kernel<D, G, TILE, STAGES, WARPS>, bytes, configured) != 0)
    return -3;
  return static_cast<int>(b200host::launch_kernel(decode_attn_paged_kernel<D, G, TILE, STAGES, WARPS>,
                                                  dim3(p.splits, p.Hkv, p.B), dim3(WARPS * 32), bytes, s,
                                                  b200host::pdl_enabled() != 0, p));
}

template <int D, int G>
int launch_paged_one(const PagedParams& p, cudaStream_t s) {
  return launch_paged_cfg<D, G, kTile, kStages, kPagedWarps>(p, s);
}

template <int D>
int launch_paged(const PagedParams& p, int G, cudaStream_t s) {
  switch (G) {
    case 1: return launch_paged_one<D, 1>(p, s);
    case 2: return launch_paged_one<D, 2>(p, s);
    case 4: return launch_paged_one<D, 4>(p, s);
    case 8: return launch_paged_one<D, 8>(p, s);
    default: return -2;
  }
}

}  // namespace

// Number of kv splits: as many as fit in ONE wave of resident CTAs (a second, partly filled wave would leave most
// SMs idle for the time of a whole CTA), at least 256 rows each.
extern "C" int b200_decode_attn_splits(int B, int Hq, int Hkv, int max_rows) {
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int G = Hkv > 0 ? Hq / Hkv : 1;
  const int per_sm = G <= 2 ? 6 : (G == 4 ? 4 : 2);  // the kernels' launch bounds
  const int base = B * Hkv > 0 ? B * Hkv : 1;
  int splits = sms * per_sm / base;
  const int by_rows = (max_rows + 255) / 256;
  if (splits > by_rows) splits = by_rows;
  if (splits > 64) splits = 64;
  return splits < 1 ? 1 : splits;
}

// q, out: [B,Hq,D] bf16 contiguous.  k, v: caches addressed as base + b * batch + h * head + (r / page_rows) * page
// + (r % page_rows) * row (element strides), which covers both a dense [B, rows, Hkv, D] cache (page_rows = rows)
// and head-major pages [B, pages, Hkv, page_rows, D].  lengths: int32 [B] (rows valid per sequence), lo: int32 [B] or null (first visible row).
// part_o: fp32 [B*Hq*splits*D], part_ml: fp32 [B*Hq*splits*2] scratch.  Hq/Hkv must be 1, 2, 4 or 8; D is 64 or 128.
extern "C" int b200_decode_attn(const void* q, const void* k, const void* v, void* out, const void* lengths,
                                const void* lo, void* part_o, void* part_ml, int B, int Hq, int Hkv, int D,
                                long long k_row, long long k_batch, long long v_row, long long v_batch,
                                long long k_head, long long v_head, long long k_page, long long v_page, int page_rows,
                                float scale, int splits, void* stream) {
  if (B <= 0 || Hq <= 0 || Hkv <= 0 || Hq % Hkv || splits < 1 || page_rows < 1) return -2;
  if ((k_row % 8) || (k_batch % 8) || (v_row % 8) || (v_batch % 8) || (k_head % 8) || (v_head % 8) || (k_page % 8) ||
      (v_page % 8))
    return -1;  // 16-byte loads
  if ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v)) & 15) return -1;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  DecodeParams p{(const __nv_bfloat16*)q, (const __nv_bfloat16*)k, (const __nv_bfloat16*)v, (const int*)lengths,
                 (const int*)lo, (float*)part_o, (float*)part_ml, k_row, k_batch, v_row, v_batch, k_head, v_head, k_page,
                 v_page, page_rows, B, Hq, Hkv, splits, scale * kLog2e};
  int rc;
  if (D == 128) rc = launch_partial<128>(p, Hq / Hkv, s);
  else if (D == 64) rc = launch_partial<64>(p, Hq / Hkv, s);
  else return -2;
  if (rc) return rc;
  return static_cast<int>(b200host::launch_kernel(decode_attn_merge_kernel, dim3(B * Hq), dim3(D), 0, s,
                                                  b200host::pdl_enabled() != 0, (const float*)part_o,
                                                  (const float*)part_ml, (__nv_bfloat16*)out, splits, D));
}

// Append one token per sequence to head-major paged caches (see b200_decode_attn for the addressing).
extern "C" int b200_kv_append(const void* k_new, const void* v_new, long long kn_batch, long long vn_batch, void* k_cache,
                              void* v_cache, const void* positions, long long c_batch, long long c_head,
                              long long c_page, long long c_row, int page_rows, int B, int Hkv, int D, void* stream) {
  if (B <= 0 || Hkv <= 0 || D % 8 || page_rows < 1) return -2;
  if ((kn_batch % 8) || (vn_batch % 8) || (c_batch % 8) || (c_head % 8) || (c_page % 8) || (c_row % 8)) return -1;
  const int total = B * Hkv * (D / 8);
  return static_cast<int>(b200host::launch_kernel(
      kv_append_kernel, dim3((total + 255) / 256), dim3(256), 0, reinterpret_cast<cudaStream_t>(stream),
      b200host::pdl_enabled() != 0, (const __nv_bfloat16*)k_new, (const __nv_bfloat16*)v_new, kn_batch, vn_batch,
      (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache, (const int*)positions, c_batch, c_head, c_page, c_row, page_rows,
      B, Hkv, D));
}

// Splits for the tile-streaming kernel: one wave of resident CTAs (shared memory allows two per SM for GQA groups
// up to two, one otherwise), at least 256 rows each.
extern "C" int b200_decode_attn_paged_splits(int B, int Hq, int Hkv, int max_rows) {
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int G = Hkv > 0 ? Hq / Hkv : 1;
  const int per_sm = G <= 2 ? 2 : 1;  // by the shared memory of the tile ring and the merge scratch
  const int base = B * Hkv > 0 ? B * Hkv : 1;
  int splits = sms * per_sm / base;
  const int by_rows = (max_rows + 255) / 256;
  if (splits > by_rows) splits = by_rows;
  if (splits > 64) splits = 64;
  return splits < 1 ? 1 : splits;
}

// Decode attention over head-major pages [.., pages, Hkv, page_rows, D] whose rows are contiguous inside a
// (page, head) block: element strides `batch`, `head`, `page` (shared by K and V), page_rows a multiple of 64.
// Every page that holds a row below lengths[b] must be allocated in full (tiles of 64 rows are copied whole).
// Scratch and result as for b200_decode_attn; `status` is the device status word that bounded waits report to.
extern "C" int b200_decode_attn_paged(const void* q, const void* k, const void* v, void* out, const void* lengths,
                                      const void* lo, void* part_o, void* part_ml, int B, int Hq, int Hkv, int D,
                                      long long batch, long long head, long long page, int page_rows, float scale,
                                      int splits, long long q_batch, void* status, void* stream) {
  if (B <= 0 || Hq <= 0 || Hkv <= 0 || Hq % Hkv || splits < 1 || !status || q_batch < (long long)Hq * D || (q_batch % 8))
    return -2;
  if (page_rows < kTile || page_rows % kTile) return -2;  // a tile never straddles two pages
  if ((batch % 8) || (head % 8) || (page % 8)) return -1;  // 16-byte aligned bulk copies
  if ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v)) & 15) return -1;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  PagedParams p{(const __nv_bfloat16*)q, (const __nv_bfloat16*)k, (const __nv_bfloat16*)v, (const int*)lengths,
                (const int*)lo, (float*)part_o, (float*)part_ml, batch, head, page, page_rows, B, Hq, Hkv, splits,
                scale * kLog2e, (int*)status, q_batch};
  int rc;
  if (D == 128) rc = launch_paged<128>(p, Hq / Hkv, s);
  else if (D == 64) rc = launch_paged<64>(p, Hq / Hkv, s);
  else return -2;
  if (rc) return rc;
  return static_cast<int>(b200host::launch_kernel(decode_attn_merge_kernel, dim3(B * Hq), dim3(D), 0, s,
                                                  b200host::pdl_enabled() != 0, (const float*)part_o,
                                                  (const float*)part_ml, (__nv_bfloat16*)out, splits, D));
}
