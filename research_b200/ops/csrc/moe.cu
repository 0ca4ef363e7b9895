// Mixture-of-experts routing glue for sm_100a: everything between the router's top-k and the grouped expert GEMMs,
// and back, without a sort, a one-hot matrix or a host synchronisation.
//
//   rank      position of every (token, choice) assignment inside its expert in token order (the priority order
//             of capacity dropping), and the per-expert counts: a block histogram pass, then one warp per chunk
//             walks its chunk 32 assignments at a time with __match_any_sync
//   layout    per-expert kept rows (capacity), 128-row padded block starts, the tile -> expert table and the
//             per-expert contraction ranges that the grouped GEMMs take
//   dest/src  destination row of every kept assignment in the expert-major padded buffer and its inverse
//   gather    x_pad[r] = scale * x[token of row r] (zeros in padding rows): dispatch, and combine's backward
//   combine   y[t] = sum_j w[t,j] * y_pad[dest[t,j]]: combine, and dispatch's backward (w = 1)
//   combine_dw  dw[t,j] = <y_pad[dest[t,j]], dy[t]>
//
// With expert parallelism the same kernels address rows in peer arenas: `gather` runs on the sender and stores
// rows straight into the owning rank's buffer (row bases per destination rank), `combine` loads expert outputs
// from the owning rank's buffer.  Offsets between ranks come from an all-gather of the per-expert counts.
//
// Reference: src/jaxtitan/models/components/moe.py:538-696 (sort-based ragged all-to-all dispatcher),
// 198-316 (local dispatcher); vendored third_party/ThunderKittens/kernels/parallel/moe_dispatch_gemm (Hopper only).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace {

constexpr int kChunk = 2048;       // assignments per ranking chunk
constexpr int kMaxExperts = 1024;
constexpr int kMaxRanks = 8;

__global__ void __launch_bounds__(256) moe_hist_kernel(const int* __restrict__ expert_ids, int A, int E,
                                                       int* __restrict__ block_hist) {
  __shared__ int hist[kMaxExperts];
  for (int e = threadIdx.x; e < E; e += blockDim.x) hist[e] = 0;
  __syncthreads();
  const int begin = blockIdx.x * kChunk, end = min(begin + kChunk, A);
  for (int a = begin + threadIdx.x; a < end; a += blockDim.x) {
    const int e = expert_ids[a];
    if (e >= 0 && e < E) atomicAdd(&hist[e], 1);
  }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x) block_hist[blockIdx.x * E + e] = hist[e];
}

// One warp per chunk.  pos[a] = number of earlier assignments (in index order) with the same expert.
__global__ void __launch_bounds__(32) moe_rank_kernel(const int* __restrict__ expert_ids, int A, int E,
                                                      const int* __restrict__ block_hist, int* __restrict__ pos,
                                                      int* __restrict__ counts) {
  __shared__ int base[kMaxExperts];
  const int lane = threadIdx.x;
  const int nblk = gridDim.x;
  for (int e = lane; e < E; e += 32) {
    int before = 0, total = 0;
    for (int b = 0; b < nblk; ++b) {
      const int h = block_hist[b * E + e];
      if (b < (int)blockIdx.x) before += h;
      total += h;
    }
    base[e] = before;
    if (blockIdx.x == 0) counts[e] = total;
  }
  __syncwarp();
  const int begin = blockIdx.x * kChunk, end = min(begin + kChunk, A);
  for (int a0 = begin; a0 < end; a0 += 32) {
    const int a = a0 + lane;
    const bool valid = a < end;
    int e = valid ? expert_ids[a] : -1;
    if (e < 0 || e >= E) e = -1;
    const unsigned active = __ballot_sync(0xffffffffu, e >= 0);
    if (e >= 0) {
      const unsigned same = __match_any_sync(active, e);
      const int before = __popc(same & ((1u << lane) - 1u));
      const int b = base[e];
      pos[a] = b + before;
      __syncwarp(active);
      if (before == 0) base[e] = b + __popc(same);  // one writer per expert
    } else if (valid) {
      pos[a] = -1;
    }
    __syncwarp();
  }
}

// Single block.  kept[e] = min(counts[e], capacity); blocks padded to `pad` rows.
//   starts[e]      first row of expert e's block;  k_range[2e], [2e+1] = its padded row range
//   tile_group[t]  expert of 128-row tile t (or -1 past the last block)
__global__ void __launch_bounds__(256) moe_layout_kernel(const int* __restrict__ counts, int E, int capacity, int pad,
                                                         int tiles, int* __restrict__ starts,
                                                         int* __restrict__ k_range, int* __restrict__ tile_group,
                                                         int* __restrict__ kept_out) {
  __shared__ int s_start[kMaxExperts + 1];
  if (threadIdx.x == 0) {
    int cursor = 0;
    for (int e = 0; e < E; ++e) {
      const int c = counts[e];
      const int kept = capacity > 0 && c > capacity ? capacity : c;
      const int padded = (kept + pad - 1) / pad * pad;
      s_start[e] = cursor;
      starts[e] = cursor;
      k_range[2 * e] = cursor;
      k_range[2 * e + 1] = cursor + padded;
      if (kept_out) kept_out[e] = kept;
      cursor += padded;
    }
    s_start[E] = cursor;
  }
  __syncthreads();
  for (int t = threadIdx.x; t < tiles; t += blockDim.x) {
    const int row = t * 128;
    int g = -1;
    if (row < s_start[E]) {
      int lo = 0, hi = E;  // largest e with s_start[e] <= row
      while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (s_start[mid] <= row) lo = mid; else hi = mid;
      }
      g = lo;
    }
    tile_group[t] = g;
  }
}

// Zero the padding rows behind the real rows of every expert block (rows [starts[e] + counts[e], next multiple of
// 128)): the grouped GEMMs contract over whole padded blocks, so these rows must not hold stale data, while the
// real rows are about to be written by the senders.  One CTA per expert.
__global__ void __launch_bounds__(256) moe_zero_pad_kernel(__nv_bfloat16* __restrict__ buf, const int* __restrict__ starts,
                                                           const int* __restrict__ counts, int H) {
  const int e = blockIdx.x;
  const int first = starts[e] + counts[e];
  const int last = (first + 127) / 128 * 128;
  const long long n16 = (long long)(last - first) * H / 8;          // 16-byte units (H % 8 == 0)
  uint4* p = reinterpret_cast<uint4*>(buf + (long long)first * H);
  const uint4 z = make_uint4(0u, 0u, 0u, 0u);
  for (long long i = threadIdx.x; i < n16; i += blockDim.x) p[i] = z;
}

// dest[a] = starts[e] + pos[a] (+ row_base of the rank that owns e) for kept assignments, else -1; src[dest] = a.
// With expert parallelism experts_per_rank > 0: `starts` then holds, per global expert, the first row *for this
// sender* inside the owner's buffer, and dest encodes owner * rows_per_rank + row.
__global__ void moe_dest_kernel(const int* __restrict__ expert_ids, const int* __restrict__ pos,
                                const int* __restrict__ starts, int A, int E, int capacity, int experts_per_rank,
                                long long rows_per_rank, int* __restrict__ dest, int* __restrict__ src) {
  for (int a = blockIdx.x * blockDim.x + threadIdx.x; a < A; a += gridDim.x * blockDim.x) {
    const int e = expert_ids[a];
    const int p = pos[a];
    int d = -1;
    if (e >= 0 && e < E && p >= 0 && (capacity <= 0 || p < capacity)) {
      d = starts[e] + p;
      if (experts_per_rank > 0) d += (int)((e / experts_per_rank) * rows_per_rank);
      else if (src) src[d] = a;
    }
    dest[a] = d;
  }
}

struct RowBases {
  __nv_bfloat16* base[kMaxRanks];  // buffer of every rank (index 0 only without expert parallelism)
};

// Row-major copy, one warp per row of the padded buffer (local mode: src[] names the assignment, padding rows are
// zeroed) or per assignment (push mode: the row goes to dest[a] in the owner's buffer).
__global__ void __launch_bounds__(256)
moe_gather_kernel(const __nv_bfloat16* __restrict__ x, const float* __restrict__ scale, const int* __restrict__ src,
                  const int* __restrict__ dest, RowBases out, long long rows, int H, int k, long long rows_per_rank) {
  const int lane = threadIdx.x & 31;
  const long long warp = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const long long nwarps = (long long)gridDim.x * (blockDim.x >> 5);
  for (long long r = warp; r < rows; r += nwarps) {
    int a;
    __nv_bfloat16* dst;
    if (src) {  // local: r is a row of the padded buffer
      a = src[r];
      dst = out.base[0] + r * H;
    } else {    // push: r is an assignment
      a = (int)r;
      const int d = dest[a];
      if (d < 0) continue;
      const int owner = rows_per_rank > 0 ? (int)(d / rows_per_rank) : 0;
      dst = out.base[owner] + (d - owner * rows_per_rank) * H;
    }
    if (a < 0) {
      for (int c = lane * 8; c < H; c += 256) *reinterpret_cast<uint4*>(dst + c) = make_uint4(0, 0, 0, 0);
      continue;
    }
    const __nv_bfloat16* row = x + (long long)(a / k) * H;
    const float s = scale ? scale[a] : 1.f;
    for (int c = lane * 8; c < H; c += 256) {
      uint4 v = *reinterpret_cast<const uint4*>(row + c);
      if (scale) {
        __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          float2 f = __bfloat1622float2(h[i]);
          f.x *= s;
          f.y *= s;
          h[i] = __floats2bfloat162_rn(f.x, f.y);
        }
      }
      *reinterpret_cast<uint4*>(dst + c) = v;
    }
  }
}

struct RowSources {
  const __nv_bfloat16* base[kMaxRanks];
};

// y[t] = sum_j w[t,j] * pad[dest[t,j]]; one warp per token, fp32 accumulation.  H <= 8192.
// full occupancy (64 warps per SM): the kernel waits on scattered 16-byte loads, more warps hide more of them
__global__ void __launch_bounds__(256, 8)
moe_combine_kernel(RowSources pad, const float* __restrict__ w, const int* __restrict__ dest,
                   __nv_bfloat16* __restrict__ y, __nv_bfloat16* __restrict__ rows_out, long long T, int H, int k,
                   long long rows_per_rank) {
  const int lane = threadIdx.x & 31;
  const long long warp = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const long long nwarps = (long long)gridDim.x * (blockDim.x >> 5);
  for (long long t = warp; t < T; t += nwarps) {
    for (int c0 = 0; c0 < H; c0 += 256) {
      const int c = c0 + lane * 8;
      float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
      if (c < H) {
        for (int j = 0; j < k; ++j) {
          const int d = dest[t * k + j];
          if (d < 0) {
            if (rows_out) *reinterpret_cast<uint4*>(rows_out + (t * k + j) * H + c) = make_uint4(0, 0, 0, 0);
            continue;
          }
          const float wj = w ? w[t * k + j] : 1.f;
          const int owner = rows_per_rank > 0 ? (int)(d / rows_per_rank) : 0;
          const __nv_bfloat16* row = pad.base[owner] + (d - owner * rows_per_rank) * (long long)H;
          const uint4 v = *reinterpret_cast<const uint4*>(row + c);
          // optionally keep the unweighted row (the gradient of the routing weights needs it later)
          if (rows_out) *reinterpret_cast<uint4*>(rows_out + (t * k + j) * H + c) = v;
          const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const float2 f = __bfloat1622float2(h[i]);
            acc[2 * i] = fmaf(wj, f.x, acc[2 * i]);
            acc[2 * i + 1] = fmaf(wj, f.y, acc[2 * i + 1]);
          }
        }
        uint4 o;
        __nv_bfloat162* ho = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
        for (int i = 0; i < 4; ++i) ho[i] = __floats2bfloat162_rn(acc[2 * i], acc[2 * i + 1]);
        *reinterpret_cast<uint4*>(y + t * H + c) = o;
      }
    }
  }
}

// dw[a] = <pad[dest[a]], dy[a / k]>; one warp per assignment.
__global__ void __launch_bounds__(256)
moe_combine_dw_kernel(RowSources pad, const __nv_bfloat16* __restrict__ dy, const int* __restrict__ dest,
                      float* __restrict__ dw, long long A, int H, int k, long long rows_per_rank) {
  const int lane = threadIdx.x & 31;
  const long long warp = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const long long nwarps = (long long)gridDim.x * (blockDim.x >> 5);
  for (long long a = warp; a < A; a += nwarps) {
    const int d = dest[a];
    float acc = 0.f;
    if (d >= 0) {
      const int owner = rows_per_rank > 0 ? (int)(d / rows_per_rank) : 0;
      const __nv_bfloat16* row = pad.base[owner] + (d - owner * rows_per_rank) * (long long)H;
      const __nv_bfloat16* g = dy + (a / k) * H;
      for (int c = lane * 8; c < H; c += 256) {
        const uint4 v = *reinterpret_cast<const uint4*>(row + c);
        const uint4 u = *reinterpret_cast<const uint4*>(g + c);
        const __nv_bfloat162* hv = reinterpret_cast<const __nv_bfloat162*>(&v);
        const __nv_bfloat162* hu = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float2 f = __bfloat1622float2(hv[i]), q = __bfloat1622float2(hu[i]);
          acc += f.x * q.x + f.y * q.y;
        }
      }
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
    if (lane == 0) dw[a] = acc;
  }
}

int grid_rows(long long rows) {
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  long long b = (rows + 7) / 8;
  const long long cap = (long long)sms * 8;
  if (b > cap) b = cap;
  return b < 1 ? 1 : (int)b;
}

}  // namespace

extern "C" {

int b200_moe_chunks(int A) { return (A + kChunk - 1) / kChunk; }

// expert_ids: int32 [A] (assignment a = token * k + choice).  block_hist: int32 scratch [chunks * E].
// pos: int32 [A]; counts: int32 [E].
int b200_moe_rank(const void* expert_ids, int A, int E, void* block_hist, void* pos, void* counts, void* stream) {
  if (A <= 0 || E <= 0 || E > kMaxExperts) return -2;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  const int chunks = (A + kChunk - 1) / kChunk;
  moe_hist_kernel<<<chunks, 256, 0, s>>>((const int*)expert_ids, A, E, (int*)block_hist);
  moe_rank_kernel<<<chunks, 32, 0, s>>>((const int*)expert_ids, A, E, (const int*)block_hist, (int*)pos, (int*)counts);
  return static_cast<int>(cudaGetLastError());
}

// counts: int32 [E] -> starts [E], k_range [2E], tile_group [tiles], kept [E] (may be null).  capacity <= 0: none.
int b200_moe_layout(const void* counts, int E, int capacity, int pad, int tiles, void* starts, void* k_range,
                    void* tile_group, void* kept, void* stream) {
  if (E <= 0 || E > kMaxExperts || pad < 1 || tiles < 0) return -2;
  moe_layout_kernel<<<1, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>((const int*)counts, E, capacity, pad, tiles,
                                                                          (int*)starts, (int*)k_range,
                                                                          (int*)tile_group, (int*)kept);
  return static_cast<int>(cudaGetLastError());
}

// buf: [rows, H] bf16 expert-major buffer; starts / counts: int32 [E] first row and real row count of every block.
int b200_moe_zero_pad(void* buf, const void* starts, const void* counts, int E, int H, void* stream) {
  if (E <= 0 || E > kMaxExperts || H % 8) return -2;
  moe_zero_pad_kernel<<<E, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>((__nv_bfloat16*)buf, (const int*)starts,
                                                                            (const int*)counts, H);
  return static_cast<int>(cudaGetLastError());
}

// dest: int32 [A]; src: int32 [rows_pad] pre-filled with -1 (local mode) or null (push mode, experts_per_rank > 0).
int b200_moe_dest(const void* expert_ids, const void* pos, const void* starts, int A, int E, int capacity,
                  int experts_per_rank, long long rows_per_rank, void* dest, void* src, void* stream) {
  if (A <= 0 || E <= 0) return -2;
  moe_dest_kernel<<<(A + 255) / 256, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      (const int*)expert_ids, (const int*)pos, (const int*)starts, A, E, capacity, experts_per_rank, rows_per_rank,
      (int*)dest, (int*)src);
  return static_cast<int>(cudaGetLastError());
}

// Local mode (src != null): out[0] is the padded buffer [rows, H]; every row is written (zeros where src < 0).
// Push mode (src == null): rows = A assignments; row a goes to out[owner] at dest[a] - owner * rows_per_rank.
int b200_moe_gather(const void* x, const void* scale, const void* src, const void* dest, void* const* out, int n_out,
                    long long rows, int H, int k, long long rows_per_rank, void* stream) {
  if (rows <= 0 || H % 8 || k < 1 || n_out < 1 || n_out > kMaxRanks) return -2;
  RowBases rb = {};
  for (int i = 0; i < n_out; ++i) rb.base[i] = static_cast<__nv_bfloat16*>(out[i]);
  moe_gather_kernel<<<grid_rows(rows), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      (const __nv_bfloat16*)x, (const float*)scale, (const int*)src, (const int*)dest, rb, rows, H, k, rows_per_rank);
  return static_cast<int>(cudaGetLastError());
}

// rows_out (optional): bf16 [T * k, H]; row t*k+j receives the unweighted source row of assignment (t, j).
int b200_moe_combine(void* const* pad, int n_pad, const void* w, const void* dest, void* y, void* rows_out, long long T,
                     int H, int k, long long rows_per_rank, void* stream) {
  if (T <= 0 || H % 8 || k < 1 || n_pad < 1 || n_pad > kMaxRanks) return -2;
  RowSources rs = {};
  for (int i = 0; i < n_pad; ++i) rs.base[i] = static_cast<const __nv_bfloat16*>(pad[i]);
  moe_combine_kernel<<<grid_rows(T), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      rs, (const float*)w, (const int*)dest, (__nv_bfloat16*)y, (__nv_bfloat16*)rows_out, T, H, k, rows_per_rank);
  return static_cast<int>(cudaGetLastError());
}

int b200_moe_combine_dw(void* const* pad, int n_pad, const void* dy, const void* dest, void* dw, long long A, int H,
                        int k, long long rows_per_rank, void* stream) {
  if (A <= 0 || H % 8 || k < 1 || n_pad < 1 || n_pad > kMaxRanks) return -2;
  RowSources rs = {};
  for (int i = 0; i < n_pad; ++i) rs.base[i] = static_cast<const __nv_bfloat16*>(pad[i]);
  moe_combine_dw_kernel<<<grid_rows(A), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      rs, (const __nv_bfloat16*)dy, (const int*)dest, (float*)dw, A, H, k, rows_per_rank);
  return static_cast<int>(cudaGetLastError());
}

}  // extern "C"
