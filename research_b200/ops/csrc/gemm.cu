// bf16 GEMM for sm_100a: C[b] (+)= op(A[b]) * op(B[b]), fp32 accumulation in tensor memory.
//
// One persistent CTA per SM, 6 warps with fixed roles:
//   warp 0    TMA producer   : streams 128 x 64 (A) and BN x 64 (B) bf16 tiles into a 4-stage
//                              shared-memory ring (128-byte swizzle), one elected lane
//   warp 1    MMA issuer     : one lane issues tcgen05.mma (M=128, N=BN, K=16) into one of two
//                              TMEM accumulators and commits completion to mbarriers
//   warps 2-5 epilogue       : tcgen05.ld the finished accumulator (each warp owns its 32-lane
//                              TMEM quadrant = 32 output rows), convert, stage through swizzled
//                              shared memory and write with TMA (store, or reduce-add when
//                              accumulating into C); overlaps the next tile's main loop.
//
// Operand layouts (all row-major in global memory, leading strides multiples of 16 bytes):
//   a_mn = 0 : A stored [M][K]   (K contiguous, "K-major")      a_mn = 1 : A stored [K][M]
//   b_mn = 0 : B stored [N][K]   (the y = x W^T weight layout)  b_mn = 1 : B stored [K][N]
// which covers forward (NT), data-gradient (NN) and weight-gradient (TN) products without a
// transpose pass.  No cluster launch and no multicast loads: the same code runs on any number of
// GPUs.  The role this plays in the reference is XLA's cuBLAS dot; the hand-written comparator in
// its vendored tree is third_party/ThunderKittens/kernels/gemm/bf16_b200/bf16_b200_gemm.cu.
#include "b200.cuh"
#include "host_util.cuh"

using namespace b200;

namespace {

constexpr int BM = 128;
constexpr int BK = 64;
constexpr int STAGES = 4;
constexpr int A_TILE_BYTES = BM * BK * 2;
constexpr int EPI_WARPS = 4;
constexpr int STAGING_BYTES = 32 * 128;  // 32 rows x 128 bytes per epilogue warp buffer
constexpr int NUM_THREADS = 32 * (2 + EPI_WARPS);
constexpr int GROUP_M = 8;

template <int BN>
struct SmemLayout {
  static constexpr int B_TILE_BYTES = BN * BK * 2;
  static constexpr int STAGE_BYTES = A_TILE_BYTES + B_TILE_BYTES;
  static constexpr int STAGING_OFF = STAGES * STAGE_BYTES;
  static constexpr int BAR_OFF = STAGING_OFF + EPI_WARPS * 2 * STAGING_BYTES;
  static constexpr int TOTAL = BAR_OFF + 256;
};

struct GemmParams {
  int M, N, K, batch;
  int accumulate;
  int* status;
  // Grouped modes (both optional, device arrays):
  //  tile_group[m_tile]: batch index of the B operand for that 128-row tile of A/C (A and C are 2-D, rows of
  //                      each group padded to a multiple of 128); a negative entry skips the tile.
  //  k_range[2*b], k_range[2*b+1]: the K interval [begin, end) of batch b (multiples of 64), A and B are 2-D
  //                      and share the K axis (variable-length contraction, e.g. per-expert weight gradients).
  const int* tile_group;
  const int* k_range;
  // Split-K: the batch index selects a K slice of A and B, and every slice adds into the same C (z = 0).
  int c_shared;
  // Split-K with the finishing pass inside the kernel (fp32 C is a workspace that is zero between launches): the CTA
  // that adds the last slice of an output tile converts the tile's sums to bf16 into fin_out and clears the
  // workspace behind it.  fin_count: one zeroed counter per output tile, left zero.
  const float* fin_ws_ptr;
  __nv_bfloat16* fin_out;
  long long fin_ld_ws, fin_ld_out;
  unsigned int* fin_count;
  int fin_splits;
  // Programmatic dependent launch (skinny split-K products of a decode step): the weight tiles of the first stages
  // are requested before the wait for the predecessor, only the activation tiles and the output come after it.
  int pdl;
};

template <int BN, bool A_MN, bool B_MN, bool OUT_F32>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                 const __grid_constant__ CUtensorMap tmC, const GemmParams p) {
  using L = SmemLayout<BN>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));

  if (p.pdl) pdl_launch_dependents();   // the successor may take its place on the SMs; it waits for this grid itself

  uint64_t* full = reinterpret_cast<uint64_t*>(smem + L::BAR_OFF);
  uint64_t* empty = full + STAGES;
  uint64_t* tfull = empty + STAGES;
  uint64_t* tempty = tfull + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  volatile unsigned int* fin_prev = reinterpret_cast<volatile unsigned int*>(tmem_slot + 2);
  const AbortCtx ab{abort_flag, p.status};

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  const int tiles_m = (p.M + BM - 1) / BM;
  const int tiles_n = (p.N + BN - 1) / BN;
  const int per_batch = tiles_m * tiles_n;
  const int total_tiles = per_batch * p.batch;
  const int k_blocks = (p.K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tfull[a], 1);
      mbar_init(&tempty[a], EPI_WARPS);
    }
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 2 * BN);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // returns false when the tile has no work (skipped group tile or empty K interval)
  auto tile_extent = [&](int b, int m0, int& bB, int& zAC, int& kb_begin, int& kb_end) -> bool {
    bB = b;
    zAC = b;
    kb_begin = 0;
    kb_end = k_blocks;
    if (p.tile_group) {
      bB = p.tile_group[m0 / BM];
      zAC = 0;
      if (bB < 0) return false;
    }
    if (p.k_range) {
      kb_begin = p.k_range[2 * b] / BK;
      kb_end = (p.k_range[2 * b + 1] + BK - 1) / BK;
      if (kb_end <= kb_begin) return false;
    }
    return true;
  };
  auto tile_coords = [&](int t, int& b, int& m0, int& n0) {
    b = t / per_batch;
    const int r = t - b * per_batch;
    const int group_size = GROUP_M * tiles_n;
    const int g = r / group_size;
    const int first_m = g * GROUP_M;
    const int gm = min(GROUP_M, tiles_m - first_m);
    const int in_group = r - g * group_size;
    m0 = (first_m + in_group % gm) * BM;
    n0 = (in_group / gm) * BN;
  };

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      tma_prefetch_desc(&tmA);
      tma_prefetch_desc(&tmB);
      uint32_t it = 0;
      bool ok = true;
      auto load_b = [&](uint8_t* sB, uint64_t* bar, int kb, int n0, int zB) {
        if (!B_MN) {
          tma_load_3d(sB, &tmB, bar, kb * BK, n0, zB);
        } else {
#pragma unroll
          for (int j = 0; j < BN / 64; ++j) tma_load_3d(sB + j * 8192, &tmB, bar, n0 + j * 64, kb * BK, zB);
        }
      };
      // Dependent launch: B (the weights) does not depend on the predecessor, so the B tiles of the first tile's
      // first stages are on their way before this CTA waits for it; A follows after the wait.
      uint32_t b_ahead = 0;
      if (p.pdl) {
        if ((int)blockIdx.x < total_tiles) {
          int b, m0, n0, bB, zAC, kb0, kb1;
          tile_coords(blockIdx.x, b, m0, n0);
          if (tile_extent(b, m0, bB, zAC, kb0, kb1)) {
            const int zB = (p.k_range || p.c_shared) ? 0 : bB;
            const int k_off = p.c_shared ? b * k_blocks : 0;
            for (int kb = kb0 + k_off; kb < kb1 + k_off && b_ahead < (uint32_t)STAGES; ++kb, ++b_ahead) {
              uint8_t* sB = smem + b_ahead * L::STAGE_BYTES + A_TILE_BYTES;
              mbar_expect_tx(&full[b_ahead], L::STAGE_BYTES);
              load_b(sB, &full[b_ahead], kb, n0, zB);
            }
          }
        }
        pdl_wait();
      }
      for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
        int b, m0, n0, bB, zAC, kb0, kb1;
        tile_coords(t, b, m0, n0);
        if (!tile_extent(b, m0, bB, zAC, kb0, kb1)) continue;
        const int zA = (p.k_range || p.c_shared) ? 0 : zAC;
        const int zB = (p.k_range || p.c_shared) ? 0 : bB;
        const int k_off = p.c_shared ? b * k_blocks : 0;  // split-K: slice b of the full K axis
        for (int kb = kb0 + k_off; kb < kb1 + k_off; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          const bool b_requested = it < b_ahead;   // expect_tx and the B tile of this stage went out before the wait
          if (!b_requested && !mbar_wait(&empty[s], ph ^ 1, ab, ERR_WAIT_EMPTY)) { ok = false; break; }
          uint8_t* sA = smem + s * L::STAGE_BYTES;
          uint8_t* sB = sA + A_TILE_BYTES;
          if (!b_requested) mbar_expect_tx(&full[s], L::STAGE_BYTES);
          if (!A_MN) {
            tma_load_3d(sA, &tmA, &full[s], kb * BK, m0, zA);
          } else {
#pragma unroll
            for (int j = 0; j < BM / 64; ++j) tma_load_3d(sA + j * 8192, &tmA, &full[s], m0 + j * 64, kb * BK, zA);
          }
          if (!b_requested) load_b(sB, &full[s], kb, n0, zB);
        }
      }
      if (!ok) {
        // give copies already in flight time to land before the CTA's shared memory goes away
        const uint64_t t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_bf16(BM, BN, A_MN, B_MN);
      uint32_t it = 0;
      uint32_t tile_iter = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
        int b, m0, n0, bB, zAC, kb0, kb1;
        tile_coords(t, b, m0, n0);
        if (!tile_extent(b, m0, bB, zAC, kb0, kb1)) continue;
        const uint32_t acc = tile_iter & 1;
        const uint32_t acc_ph = (tile_iter >> 1) & 1;
        ++tile_iter;
        if (!mbar_wait(&tempty[acc], acc_ph ^ 1, ab, ERR_WAIT_TMEM_EMPTY)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait(&full[s], ph, ab, ERR_WAIT_FULL)) { ok = false; break; }
          tc_fence_after();
          const uint32_t a_base = smem_u32(smem + s * L::STAGE_BYTES);
          const uint32_t b_base = a_base + A_TILE_BYTES;
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            const uint64_t adesc = make_smem_desc_sw128(a_base + (A_MN ? k * 2048 : k * 32), A_MN ? 8192 : 16, 1024);
            const uint64_t bdesc = make_smem_desc_sw128(b_base + (B_MN ? k * 2048 : k * 32), B_MN ? 8192 : 16, 1024);
            tc_mma_ss(d_tmem, adesc, bdesc, idesc, (kb != kb0 || k != 0) ? 1u : 0u);
          }
          tc_commit(&empty[s]);  // stage reusable once these MMAs have read it
        }
        if (ok) tc_commit(&tfull[acc]);  // accumulator complete
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue
    const int q = warp & 3;  // TMEM lane quadrant this warp may access
    constexpr int COLS_PER_BOX = OUT_F32 ? 32 : 64;
    uint8_t* stage0 = smem + L::STAGING_OFF + (warp - 2) * 2 * STAGING_BYTES;
    uint32_t tile_iter = 0;
    uint32_t box_iter = 0;
    bool ok = true;
    if (p.pdl) pdl_wait();   // C (and the workspace behind it) belongs to the predecessor until it has completed
    for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
      int b, m0, n0, bB, zAC, kb0, kb1;
      tile_coords(t, b, m0, n0);
      if (!tile_extent(b, m0, bB, zAC, kb0, kb1)) continue;
      const uint32_t acc = tile_iter & 1;
      const uint32_t acc_ph = (tile_iter >> 1) & 1;
      ++tile_iter;
      if (!mbar_wait_warp(&tfull[acc], acc_ph, ab, ERR_WAIT_TMEM_FULL)) { ok = false; break; }
      tc_fence_after();
      const uint32_t t_row = tmem_base + acc * BN + (static_cast<uint32_t>(q * 32) << 16);
      const int row0 = m0 + q * 32;
#pragma unroll 1
      for (int j = 0; j < BN / COLS_PER_BOX; ++j) {
        const int col0 = n0 + j * COLS_PER_BOX;
        if (col0 >= p.N || row0 >= p.M) break;  // warp-uniform: nothing of this box is in range
        uint8_t* buf = stage0 + (box_iter & 1) * STAGING_BYTES;
        ++box_iter;
        if (lane == 0) tma_wait_group_read<1>();  // the store that last read this buffer is done
        __syncwarp();
        if (OUT_F32) {
          uint32_t r[32];
          tmem_ld_32x32b_x32(t_row + j * 32, r);
          tmem_ld_wait();
#pragma unroll
          for (int c = 0; c < 8; ++c)
            *reinterpret_cast<uint4*>(buf + sw128_offset(lane, c)) = make_uint4(r[4 * c], r[4 * c + 1], r[4 * c + 2], r[4 * c + 3]);
        } else {
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            uint32_t r[32];
            tmem_ld_32x32b_x32(t_row + j * 64 + h * 32, r);
            tmem_ld_wait();
#pragma unroll
            for (int c = 0; c < 4; ++c) {
              uint4 v;
              v.x = pack_bf16x2(__uint_as_float(r[8 * c + 0]), __uint_as_float(r[8 * c + 1]));
              v.y = pack_bf16x2(__uint_as_float(r[8 * c + 2]), __uint_as_float(r[8 * c + 3]));
              v.z = pack_bf16x2(__uint_as_float(r[8 * c + 4]), __uint_as_float(r[8 * c + 5]));
              v.w = pack_bf16x2(__uint_as_float(r[8 * c + 6]), __uint_as_float(r[8 * c + 7]));
              *reinterpret_cast<uint4*>(buf + sw128_offset(lane, h * 4 + c)) = v;
            }
          }
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
          const int zC = p.c_shared ? 0 : zAC;
          if (p.accumulate)
            tma_reduce_add_3d(&tmC, buf, col0, row0, zC);
          else
            tma_store_3d(&tmC, buf, col0, row0, zC);
          tma_commit_group();
        }
      }
      // every tcgen05.ld of this accumulator has completed: hand it back to the MMA issuer
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty[acc]);
      if (OUT_F32 && p.fin_out) {
        // split-K with the finishing pass fused: when this CTA's adds of the tile are in memory, count the slice;
        // the CTA that counts the last one converts the tile and clears the workspace
        float* ws = reinterpret_cast<float*>(const_cast<void*>(static_cast<const void*>(p.fin_ws_ptr)));
        if (lane == 0) {
          tma_wait_group<0>();
          fence_proxy_async_all();
          __threadfence();
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");   // the four epilogue warps
        const int tile_id = (m0 / BM) * ((p.N + BN - 1) / BN) + n0 / BN;
        if (warp == 2 && lane == 0) *fin_prev = atomicAdd(&p.fin_count[tile_id], 1u);
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (*fin_prev == (unsigned int)p.fin_splits - 1u) {
          __threadfence();
          const int tid = (int)threadIdx.x - 64;          // 0..127 among the epilogue threads
          const int rows = min(BM, p.M - m0);
          const int vec_per_row = min(BN, p.N - n0) >> 2;
          for (int i = tid; i < rows * vec_per_row; i += EPI_WARPS * 32) {
            const int r = i / vec_per_row, c = (i - r * vec_per_row) << 2;
            float4* src = reinterpret_cast<float4*>(ws + (long long)(m0 + r) * p.fin_ld_ws + n0 + c);
            const float4 v = __ldcg(src);
            uint2 o;
            o.x = pack_bf16x2(v.x, v.y);
            o.y = pack_bf16x2(v.z, v.w);
            *reinterpret_cast<uint2*>(p.fin_out + (long long)(m0 + r) * p.fin_ld_out + n0 + c) = o;
            __stcg(src, make_float4(0.f, 0.f, 0.f, 0.f));
          }
          if (tid == 0) p.fin_count[tile_id] = 0u;
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");   // fin_prev may be rewritten for the next tile
      }
    }
    if (lane == 0) tma_wait_group<0>();
  }

  // ------------------------------------------------------------------ teardown
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem_base, 2 * BN);
  }
}

template <int BN, bool A_MN, bool B_MN, bool OUT_F32>
int launch(const CUtensorMap& tmA, const CUtensorMap& tmB, const CUtensorMap& tmC, const GemmParams& p, int grid,
           cudaStream_t stream) {
  using L = SmemLayout<BN>;
  auto* kern = gemm_bf16_kernel<BN, A_MN, B_MN, OUT_F32>;
  constexpr int smem_bytes = L::TOTAL + 1024;
  static bool configured[b200host::kMaxDevices] = {};   // per kernel instantiation and device
  if (int rc = b200host::ensure_dynamic_smem(kern, smem_bytes, configured)) return rc;
  if (p.pdl) return static_cast<int>(b200host::launch_kernel(kern, dim3(grid), dim3(NUM_THREADS), smem_bytes, stream, true,
                                                             tmA, tmB, tmC, p));
  kern<<<grid, NUM_THREADS, smem_bytes, stream>>>(tmA, tmB, tmC, p);
  return static_cast<int>(cudaGetLastError());
}

template <int BN>
int dispatch(bool a_mn, bool b_mn, bool out_f32, const CUtensorMap& tmA, const CUtensorMap& tmB,
             const CUtensorMap& tmC, const GemmParams& p, int grid, cudaStream_t s) {
#define GEMM_CASE(A, B, F) \
  if (a_mn == A && b_mn == B && out_f32 == F) return launch<BN, A, B, F>(tmA, tmB, tmC, p, grid, s);
  GEMM_CASE(false, false, false)
  GEMM_CASE(false, false, true)
  GEMM_CASE(false, true, false)
  GEMM_CASE(false, true, true)
  GEMM_CASE(true, false, false)
  GEMM_CASE(true, false, true)
  GEMM_CASE(true, true, false)
  GEMM_CASE(true, true, true)
#undef GEMM_CASE
  return b200host::RC_BAD_SHAPE;
}

}  // namespace

// C[b] (+)= op(A[b]) op(B[b]) for b in [0, batch).  Leading strides (lda/ldb/ldc) and batch strides
// are in elements.  out_f32: C is fp32 (else bf16).  accumulate: add into C with TMA reduce-add.
// `status` is a device int the kernel sets non-zero if one of its bounded waits ran out.
static int gemm_impl(const void* A, const void* B, void* C, int M, int N, int K, int batch, int batch_a, int batch_b,
                     int batch_c, long long lda, long long ldb, long long ldc, long long stride_a, long long stride_b,
                     long long stride_c, int a_mn, int b_mn, int out_f32, int accumulate, int bn_hint,
                     const int* tile_group, const int* k_range, int* status, void* stream, int c_shared = 0,
                     void* fin_out = nullptr, long long fin_ld_out = 0, void* fin_count = nullptr, int pdl = 0);

extern "C" int b200_gemm_bf16(const void* A, const void* B, void* C, int M, int N, int K, int batch, long long lda,
                              long long ldb, long long ldc, long long stride_a, long long stride_b,
                              long long stride_c, int a_mn, int b_mn, int out_f32, int accumulate, int bn_hint,
                              int* status, void* stream) {
  return gemm_impl(A, B, C, M, N, K, batch, batch, batch, batch, lda, ldb, ldc, stride_a, stride_b, stride_c, a_mn,
                   b_mn, out_f32, accumulate, bn_hint, nullptr, nullptr, status, stream);
}

// Split-K product for skinny problems (few rows, e.g. one decode token per sequence): C[M,N] (fp32, zeroed by the
// caller) += A[:, slice] * B[:, slice]^T for `splits` equal K slices, one CTA tile per (N tile, slice), so that a
// weight matrix is streamed by many SMs at once.  K must be a multiple of 64 * splits.
extern "C" int b200_gemm_bf16_splitk(const void* A, const void* B, void* C, int M, int N, int K, int splits,
                                     long long lda, long long ldb, long long ldc, int* status, void* stream) {
  if (splits < 1 || K % (64 * splits)) return b200host::RC_BAD_SHAPE;
  const int kc = K / splits;
  return gemm_impl(A, B, C, M, N, kc, splits, 1, 1, 1, lda, ldb, ldc, 0, 0, 0, 0, 0, 1, 1, 0, nullptr, nullptr, status,
                   stream, 1, nullptr, 0, nullptr, b200host::pdl_enabled());
}

// The same with the finishing pass inside the kernel: `ws` is an fp32 [M, N] workspace (row stride ldws) that is zero
// on entry and zero again on exit, `out` receives the bf16 result (row stride ldo), `counters` holds one zeroed
// uint32 per 128 x BN output tile (left zero).  N, ldws and ldo must be multiples of 4.
extern "C" int b200_gemm_bf16_splitk_fused(const void* A, const void* B, void* ws, void* out, void* counters, int M,
                                           int N, int K, int splits, long long lda, long long ldb, long long ldws,
                                           long long ldo, int* status, void* stream) {
  if (splits < 1 || K % (64 * splits) || !out || !counters) return b200host::RC_BAD_SHAPE;
  const int kc = K / splits;
  return gemm_impl(A, B, ws, M, N, kc, splits, 1, 1, 1, lda, ldb, ldws, 0, 0, 0, 0, 0, 1, 1, 0, nullptr, nullptr,
                   status, stream, 1, out, ldo, counters, b200host::pdl_enabled());
}

// Split-K for any operand layout with an fp32 output that is accumulated into (weight gradients: the contraction
// runs over tokens and is long, the output has few tiles, and the partial sums are reduce-added anyway).
extern "C" int b200_gemm_bf16_splitk_acc(const void* A, const void* B, void* C, int M, int N, int K, int splits,
                                         long long lda, long long ldb, long long ldc, int a_mn, int b_mn, int* status,
                                         void* stream) {
  if (splits < 1 || K % (64 * splits)) return b200host::RC_BAD_SHAPE;
  const int kc = K / splits;
  return gemm_impl(A, B, C, M, N, kc, splits, 1, 1, 1, lda, ldb, ldc, 0, 0, 0, a_mn, b_mn, 1, 1, 0, nullptr, nullptr,
                   status, stream, 1);
}

// Grouped forward / data-gradient product: A [M_pad, K] and C [M_pad, N] are 2-D with every group's rows
// padded to a multiple of 128; B is [groups, ...]; tile_group[m_tile] names the group of each row tile.
extern "C" int b200_gemm_bf16_grouped_rows(const void* A, const void* B, void* C, int M_pad, int N, int K, int groups,
                                           long long lda, long long ldb, long long ldc, long long stride_b, int b_mn,
                                           int out_f32, int accumulate, const int* tile_group, int* status,
                                           void* stream) {
  return gemm_impl(A, B, C, M_pad, N, K, 1, 1, groups, 1, lda, ldb, ldc, 0, stride_b, 0, 0, b_mn, out_f32, accumulate,
                   0, tile_group, nullptr, status, stream);
}

// Grouped weight-gradient product: C[g] (+)= A[k0_g:k1_g, :M]^T B[k0_g:k1_g, :N]; A [K_total, M] and B [K_total, N]
// are 2-D and share the row (contraction) axis; k_range holds (k0, k1) per group, multiples of 64.
extern "C" int b200_gemm_bf16_grouped_k(const void* A, const void* B, void* C, int M, int N, int K_total, int groups,
                                        long long lda, long long ldb, long long ldc, long long stride_c, int out_f32,
                                        int accumulate, const int* k_range, int* status, void* stream) {
  return gemm_impl(A, B, C, M, N, K_total, groups, 1, 1, groups, lda, ldb, ldc, 0, 0, stride_c, 1, 1, out_f32,
                   accumulate, 0, nullptr, k_range, status, stream);
}

static int gemm_impl(const void* A, const void* B, void* C, int M, int N, int K, int batch, int batch_a, int batch_b,
                     int batch_c, long long lda, long long ldb, long long ldc, long long stride_a, long long stride_b,
                     long long stride_c, int a_mn, int b_mn, int out_f32, int accumulate, int bn_hint,
                     const int* tile_group, const int* k_range, int* status, void* stream, int c_shared, void* fin_out,
                     long long fin_ld_out, void* fin_count, int pdl) {
  using namespace b200host;
  if (M <= 0 || N <= 0 || K <= 0 || batch <= 0) return RC_BAD_SHAPE;
  const int BN = (bn_hint == 128 || bn_hint == 256) ? bn_hint : (N > 128 ? 256 : 128);
  CUtensorMap tmA, tmB, tmC;
  int rc;
  const CUtensorMapDataType bf = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  const int k_map = c_shared ? K * batch : K;  // split-K addresses slices through the K coordinate
  if (c_shared) batch_a = batch_b = batch_c = 1;
  if (!a_mn)
    rc = make_map_3d(&tmA, bf, A, k_map, M, batch_a, lda * 2, stride_a * 2, BK, BM);
  else
    rc = make_map_3d(&tmA, bf, A, M, k_map, batch_a, lda * 2, stride_a * 2, 64, BK);
  if (rc) return rc;
  if (!b_mn)
    rc = make_map_3d(&tmB, bf, B, k_map, N, batch_b, ldb * 2, stride_b * 2, BK, BN);
  else
    rc = make_map_3d(&tmB, bf, B, N, k_map, batch_b, ldb * 2, stride_b * 2, 64, BK);
  if (rc) return rc;
  if (out_f32)
    rc = make_map_3d(&tmC, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, C, N, M, batch_c, ldc * 4, stride_c * 4, 32, 32);
  else
    rc = make_map_3d(&tmC, bf, C, N, M, batch_c, ldc * 2, stride_c * 2, 64, 32);
  if (rc) return rc;

  GemmParams p{M, N, K, batch, accumulate, status, tile_group, k_range, c_shared};
  p.fin_ws_ptr = fin_out ? static_cast<const float*>(C) : nullptr;
  p.fin_out = static_cast<__nv_bfloat16*>(fin_out);
  p.fin_ld_ws = ldc;
  p.fin_ld_out = fin_ld_out;
  p.fin_count = static_cast<unsigned int*>(fin_count);
  p.fin_splits = batch;
  p.pdl = pdl;
  if (fin_out && (!c_shared || !out_f32 || !accumulate || !fin_count || (N & 3) || (ldc & 3) || (fin_ld_out & 3) ||
                  (reinterpret_cast<uintptr_t>(C) & 15) || (reinterpret_cast<uintptr_t>(fin_out) & 7)))
    return RC_BAD_SHAPE;
  const int tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN) * batch;
  const int grid = tiles < sm_count() ? tiles : sm_count();
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (BN == 256) return dispatch<256>(a_mn, b_mn, out_f32, tmA, tmB, tmC, p, grid, s);
  return dispatch<128>(a_mn, b_mn, out_f32, tmA, tmB, tmC, p, grid, s);
}
