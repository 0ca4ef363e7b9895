// Expert-parallel dispatch fused with the first grouped expert GEMM, for sm_100a and NVLink peer memory.
//
//   C[rows of expert e] = inbox[rows of e] * W[e]^T,   inbox[row] = x_{src rank}[src token]  (or zeros: padding)
//
// The owner of a set of experts holds an expert-major buffer of 128-row tiles (the "inbox").  Which token of which
// rank belongs in a row is told by a source list that the senders wrote into the owner's arena beforehand (8 bytes
// per row: epoch | rank | token).  The first few CTAs of the grid are transfer CTAs: four threads each run a ring of
// bulk copies that pull their quarter of a tile's rows from the senders' token buffers (plain loads from peer memory,
// no cluster multicast) into the local inbox; the thread that completes a tile publishes its flag.  The other
// CTAs are the persistent tcgen05 pipeline of the grouped GEMM; their TMA producer waits for a tile's flag before the
// first load of that tile, so the product starts on row blocks as they land and every remote byte crosses
// NVLink once.  The inbox is complete when the kernel has ended (the backward pass reads it again).
//
// All waits are bounded (b200.cuh, comm.cuh): one that runs out records a status code, the CTA stops issuing work,
// waits for its copies in flight, frees its tensor memory and returns.
//
// Reference counterparts: the dispatch CTAs / per-tile counters / gated GEMM CTAs of
// third_party/ThunderKittens/kernels/parallel/moe_dispatch_gemm/moe_dispatch_gemm_h100.cu:72-101, 147-183 (push
// model, unbounded waits); in the reference's own model code the dispatch is a ragged all-to-all followed by a
// grouped dot (models/components/moe.py:538-696).
#include "b200.cuh"
#include "comm.cuh"
#include "host_util.cuh"

using namespace b200;
using namespace b200comm;

namespace {

constexpr int BM = 128;
constexpr int BK = 64;
constexpr int STAGES = 4;
constexpr int A_TILE_BYTES = BM * BK * 2;
constexpr int EPI_WARPS = 4;
constexpr int STAGING_BYTES = 32 * 128;
constexpr int NUM_THREADS = 32 * (2 + EPI_WARPS);
constexpr int GROUP_M = 8;
// transfer CTAs: XFER_PIPES issuing threads, each with its own ring of XFER_BUFS chunks of at most XFER_CHUNK bytes
constexpr int XFER_PIPES = 4;
constexpr int XFER_BUFS = 8;
constexpr int XFER_LAG = XFER_BUFS - 2;
constexpr int XFER_CHUNK = 4096;
constexpr int XFER_RING_BYTES = XFER_PIPES * XFER_BUFS * XFER_CHUNK;
constexpr int XFER_ZERO_OFF = XFER_RING_BYTES;              // one chunk of zeros behind the rings
constexpr int ROWS_PER_PIPE = BM / XFER_PIPES;
constexpr int XFER_ENT_OFF = XFER_ZERO_OFF + XFER_CHUNK;    // the source entries of each pipe's rows of the tile
constexpr int XFER_BYTES = XFER_ENT_OFF + 2 * XFER_PIPES * ROWS_PER_PIPE * 8;   // two tiles' entries per pipe
constexpr int XFER_PUBLISH_DELAY = 2;                       // stores issued after a tile's last one before it is published
static_assert(ROWS_PER_PIPE == 32, "one source entry per lane of the transfer warp");

template <int BN>
struct SmemLayout {
  static constexpr int B_TILE_BYTES = BN * BK * 2;
  static constexpr int STAGE_BYTES = A_TILE_BYTES + B_TILE_BYTES;
  static constexpr int STAGING_OFF = STAGES * STAGE_BYTES;
  static constexpr int PIPE_END = STAGING_OFF + EPI_WARPS * 2 * STAGING_BYTES;
  static constexpr int BAR_OFF = PIPE_END > XFER_BYTES ? PIPE_END : XFER_BYTES;
  static constexpr int TOTAL = BAR_OFF + 512;
};

struct MoeGemmParams {
  int rows;                  // inbox rows, a multiple of 128
  int N, K;
  int world, rank;
  int n_xfer;                // transfer CTAs
  int tokens;                // rows of every rank's token buffer
  int chunk_bytes;           // bytes per bulk copy: divides 2 K, at most XFER_CHUNK, a multiple of 16
  uint32_t epoch;
  const int* tile_group;     // [rows / 128] expert of a tile, or -1 (no rows: nothing is copied or computed)
  const unsigned long long* sources;  // [rows] epoch << 32 | rank << 24 | token; another epoch = padding row
  const __nv_bfloat16* x[kMaxPeers];  // token buffers [tokens, K] of every rank as mapped here
  __nv_bfloat16* inbox;      // local [rows, K]
  uint32_t* row_flags;       // [rows / 128], hold an earlier epoch on entry
  uint32_t* tile_parts;      // [rows / 128], zero on entry, left zero
  int* status;
};

template <int BN>
__global__ void __launch_bounds__(NUM_THREADS, 1)
moe_dispatch_gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                         const __grid_constant__ CUtensorMap tmC, const MoeGemmParams p) {
  using L = SmemLayout<BN>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + L::BAR_OFF);
  uint64_t* empty = full + STAGES;
  uint64_t* tfull = empty + STAGES;
  uint64_t* tempty = tfull + 2;
  uint64_t* xbar = tempty + 2;  // barriers of the transfer rings
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(xbar + XFER_PIPES * XFER_BUFS);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const AbortCtx ab{abort_flag, p.status};

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const bool is_xfer = (int)blockIdx.x < p.n_xfer;   // lowest block indices: placed first
  const int n_compute = (int)gridDim.x - p.n_xfer;
  const int cta = (int)blockIdx.x - p.n_xfer;
  const int tiles_m = p.rows / BM;
  const int tiles_n = (p.N + BN - 1) / BN;
  const int total_tiles = tiles_m * tiles_n;
  const int k_blocks = p.K / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tfull[a], 1);
      mbar_init(&tempty[a], EPI_WARPS);
    }
    for (int i = 0; i < XFER_PIPES * XFER_BUFS; ++i) mbar_init(&xbar[i], 1);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (is_xfer) {
    // the chunk of zeros that padding rows are stored from
    for (int i = threadIdx.x; i < XFER_CHUNK / 16; i += NUM_THREADS)
      reinterpret_cast<uint4*>(smem + XFER_ZERO_OFF)[i] = make_uint4(0, 0, 0, 0);
    fence_proxy_async_smem();
  }
  if (warp == 1 && !is_xfer) {
    tmem_alloc(tmem_slot, 2 * BN);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = is_xfer ? 0u : *tmem_slot;

  auto tile_coords = [&](int t, int& mi, int& n0) {
    const int group_size = GROUP_M * tiles_n;
    const int g = t / group_size;
    const int first_m = g * GROUP_M;
    const int gm = min(GROUP_M, tiles_m - first_m);
    const int in_group = t - g * group_size;
    mi = first_m + in_group % gm;
    n0 = (in_group / gm) * BN;
  };

  if (is_xfer) {
    // ------------------------------------------------------------------ transfer CTA
    if (warp < XFER_PIPES) {
      // One pipe per warp.  The whole warp fetches the 32 source entries of its rows of a tile with one coalesced
      // load into shared memory (a dependent global load per row on the issuing thread would cost more than the
      // copy itself); lane 0 runs the ring of bulk copies.  The ring streams across tiles: the stores of a tile's
      // last rows are issued while the next tile's loads are already in flight, and the tile is published a few
      // stores later, once `cp.async.bulk.wait_group` says its stores have completed.
      uint8_t* ring = smem + warp * XFER_BUFS * XFER_CHUNK;
      const uint8_t* zeros = smem + XFER_ZERO_OFF;
      unsigned long long* ent_base =
          reinterpret_cast<unsigned long long*>(smem + XFER_ENT_OFF) + warp * 2 * ROWS_PER_PIPE;
      uint64_t* bar = xbar + warp * XFER_BUFS;
      const int chunks_per_row = p.K * 2 / p.chunk_bytes;
      const int items = ROWS_PER_PIPE * chunks_per_row;    // per tile and pipe (at least 32 > XFER_LAG)
      const long long row_bytes = (long long)p.K * 2;
      uint32_t phase = 0;                                   // bit b: parity of the next completion of ring buffer b
      bool ok = true;
      // where does row `i` of a tile's 32 rows of this pipe come from?  nullptr: a padding row
      auto source_of = [&](const unsigned long long* ent, int i) -> const uint8_t* {
        const unsigned long long e = ent[i];
        if ((uint32_t)(e >> 32) != p.epoch) return nullptr;
        const int src = (int)((e >> 24) & 0xffu), tok = (int)(e & 0xffffffu);
        if (src >= p.world || tok >= p.tokens) {            // not a row that exists: record it, store zeros
          atomicCAS(p.status, 0, ERR_BAD_ARG);
          return nullptr;
        }
        return reinterpret_cast<const uint8_t*>(p.x[src]) + (long long)tok * row_bytes;
      };
      // lane 0 only: store item j of tile `t` (entries `ent`) from its ring buffer (or from the zeros)
      auto store_item = [&](int t, const unsigned long long* ent, int j, long long g) -> bool {
        const int r = t * BM + warp * ROWS_PER_PIPE + j / chunks_per_row, c = j % chunks_per_row;
        const int buf = (int)(g % XFER_BUFS);
        uint8_t* dst = reinterpret_cast<uint8_t*>(p.inbox) + (long long)r * row_bytes + (long long)c * p.chunk_bytes;
        if (source_of(ent, j / chunks_per_row)) {
          if (!mbar_wait(&bar[buf], (phase >> buf) & 1u, ab, ERR_WAIT_FULL)) return false;
          phase ^= 1u << buf;
          bulk_s2g(dst, ring + buf * XFER_CHUNK, (uint32_t)p.chunk_bytes);
        } else {
          bulk_s2g(dst, zeros, (uint32_t)p.chunk_bytes);
        }
        tma_commit_group();
        return true;
      };
      auto publish = [&](int t) {
        fence_proxy_async_all();
        __threadfence();
        if (atomicAdd(&p.tile_parts[t], 1u) == (uint32_t)XFER_PIPES - 1u) {
          p.tile_parts[t] = 0u;
          __threadfence();
          st_release_gpu(&p.row_flags[t], p.epoch);
        }
      };
      long long g = 0;          // items issued so far by this pipe (ring position), all tiles
      int prev = -1;            // the tile whose last XFER_LAG stores are still to be issued, then to be published
      int k = 0;                // tiles handled by this pipe
      for (int t = (int)blockIdx.x; t < tiles_m && ok; t += p.n_xfer) {
        if (p.tile_group[t] < 0) continue;
        unsigned long long* ent = ent_base + (k & 1) * ROWS_PER_PIPE;
        const unsigned long long* ent_prev = ent_base + ((k & 1) ^ 1) * ROWS_PER_PIPE;
        __syncwarp();           // lane 0 is past the tile before the previous one, whose entries are overwritten now
        ent[lane] = p.sources[t * BM + warp * ROWS_PER_PIPE + lane];
        __syncwarp();
        if (lane == 0) {
          for (int i = 0; i < items && ok; ++i, ++g) {
            const int buf = (int)(g % XFER_BUFS);
            // the store that last read this ring buffer has finished reading it
            if (g >= XFER_BUFS) tma_wait_group_read<XFER_BUFS - XFER_LAG - 1>();
            const uint8_t* src = source_of(ent, i / chunks_per_row);
            if (src) {
              mbar_expect_tx(&bar[buf], (uint32_t)p.chunk_bytes);
              bulk_g2s(ring + buf * XFER_CHUNK, src + (long long)(i % chunks_per_row) * p.chunk_bytes,
                       (uint32_t)p.chunk_bytes, &bar[buf]);
            }
            // the store that lags XFER_LAG items behind: of this tile, or still of the previous one
            if (i >= XFER_LAG) {
              ok = store_item(t, ent, i - XFER_LAG, g - XFER_LAG);
            } else if (prev >= 0) {
              ok = store_item(prev, ent_prev, items - XFER_LAG + i, g - XFER_LAG);
            }
            if (ok && prev >= 0 && i == XFER_LAG - 1 + XFER_PUBLISH_DELAY) {
              tma_wait_group<XFER_PUBLISH_DELAY>();       // everything but the latest stores, so all of `prev`
              publish(prev);
              prev = -1;
            }
          }
          if (ok) prev = t;
        }
        ok = __shfl_sync(0xffffffffu, ok, 0);
        ++k;
      }
      if (lane == 0) {
        if (ok && prev >= 0) {
          // the last tile: its remaining stores, then everything is complete
          const unsigned long long* ent_last = ent_base + ((k - 1) & 1) * ROWS_PER_PIPE;
          for (int i = 0; i < XFER_LAG && ok; ++i, ++g) ok = store_item(prev, ent_last, items - XFER_LAG + i, g - XFER_LAG);
          tma_wait_group<0>();
          if (ok) publish(prev);
        }
        tma_wait_group<0>();
        if (!ok) {
          // give the loads still in flight time to land before shared memory is released
          const uint64_t t0 = globaltimer_ns();
          while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
        }
      }
    }
  } else if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      tma_prefetch_desc(&tmA);
      tma_prefetch_desc(&tmB);
      uint32_t it = 0;
      bool ok = true;
      for (int t = cta; t < total_tiles && ok; t += n_compute) {
        int mi, n0;
        tile_coords(t, mi, n0);
        const int g = p.tile_group[mi];
        if (g < 0) continue;
        if (!wait_gpu(&p.row_flags[mi], p.epoch, p.status, ERR_LOCAL_FLAG)) {
          *ab.flag = 1;
          ok = false;
          break;
        }
        fence_proxy_async_all();
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait(&empty[s], ph ^ 1, ab, ERR_WAIT_EMPTY)) { ok = false; break; }
          uint8_t* sA = smem + s * L::STAGE_BYTES;
          uint8_t* sB = sA + A_TILE_BYTES;
          mbar_expect_tx(&full[s], L::STAGE_BYTES);
          tma_load_3d(sA, &tmA, &full[s], kb * BK, mi * BM, 0);
          tma_load_3d(sB, &tmB, &full[s], kb * BK, n0, g);
        }
      }
      if (!ok) {
        const uint64_t t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_bf16(BM, BN, false, false);
      uint32_t it = 0, tile_iter = 0;
      bool ok = true;
      for (int t = cta; t < total_tiles && ok; t += n_compute) {
        int mi, n0;
        tile_coords(t, mi, n0);
        if (p.tile_group[mi] < 0) continue;
        const uint32_t acc = tile_iter & 1;
        const uint32_t acc_ph = (tile_iter >> 1) & 1;
        ++tile_iter;
        if (!mbar_wait(&tempty[acc], acc_ph ^ 1, ab, ERR_WAIT_TMEM_EMPTY)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait(&full[s], ph, ab, ERR_WAIT_FULL)) { ok = false; break; }
          tc_fence_after();
          const uint32_t a_base = smem_u32(smem + s * L::STAGE_BYTES);
          const uint32_t b_base = a_base + A_TILE_BYTES;
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            const uint64_t adesc = make_smem_desc_sw128(a_base + k * 32, 16, 1024);
            const uint64_t bdesc = make_smem_desc_sw128(b_base + k * 32, 16, 1024);
            tc_mma_ss(d_tmem, adesc, bdesc, idesc, (kb != 0 || k != 0) ? 1u : 0u);
          }
          tc_commit(&empty[s]);
        }
        if (ok) tc_commit(&tfull[acc]);
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue
    const int q = warp & 3;
    uint8_t* stage0 = smem + L::STAGING_OFF + (warp - 2) * 2 * STAGING_BYTES;
    uint32_t tile_iter = 0, box_iter = 0;
    bool ok = true;
    for (int t = cta; t < total_tiles && ok; t += n_compute) {
      int mi, n0;
      tile_coords(t, mi, n0);
      if (p.tile_group[mi] < 0) continue;
      const uint32_t acc = tile_iter & 1;
      const uint32_t acc_ph = (tile_iter >> 1) & 1;
      ++tile_iter;
      if (!mbar_wait_warp(&tfull[acc], acc_ph, ab, ERR_WAIT_TMEM_FULL)) { ok = false; break; }
      tc_fence_after();
      const uint32_t t_row = tmem_base + acc * BN + (static_cast<uint32_t>(q * 32) << 16);
      const int out_row = mi * BM + q * 32;
#pragma unroll 1
      for (int j = 0; j < BN / 64; ++j) {
        const int col0 = n0 + j * 64;
        if (col0 >= p.N) break;
        uint8_t* buf = stage0 + (box_iter & 1) * STAGING_BYTES;
        ++box_iter;
        if (lane == 0) tma_wait_group_read<1>();
        __syncwarp();
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
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
          tma_store_3d(&tmC, buf, col0, out_row, 0);
          tma_commit_group();
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty[acc]);
    }
    if (lane == 0) tma_wait_group<0>();
  }

  // ------------------------------------------------------------------ teardown
  tc_fence_before();
  __syncthreads();
  if (warp == 1 && !is_xfer) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem_base, 2 * BN);
  }
}

template <int BN>
int launch(const CUtensorMap& tmA, const CUtensorMap& tmB, const CUtensorMap& tmC, const MoeGemmParams& p, int grid,
           cudaStream_t stream) {
  using L = SmemLayout<BN>;
  auto* kern = moe_dispatch_gemm_kernel<BN>;
  constexpr int smem_bytes = L::TOTAL + 1024;
  static bool configured[b200host::kMaxDevices] = {};
  if (int rc = b200host::ensure_dynamic_smem(kern, smem_bytes, configured)) return rc;
  kern<<<grid, NUM_THREADS, smem_bytes, stream>>>(tmA, tmB, tmC, p);
  return static_cast<int>(cudaGetLastError());
}

struct ListPtrs {
  unsigned long long* p[kMaxPeers];
};
__global__ void moe_post_sources_entry(const int* __restrict__ dest, long long A, int top_k, long long rows_per_rank,
                                       int world, int rank, uint32_t epoch, const ListPtrs lists) {
  for (long long a = (long long)blockIdx.x * blockDim.x + threadIdx.x; a < A; a += (long long)gridDim.x * blockDim.x) {
    const int d = dest[a];
    if (d < 0) continue;
    const int owner = (int)(d / rows_per_rank);
    if (owner >= world) continue;
    const long long row = d - owner * rows_per_rank;
    const unsigned long long token = (unsigned long long)(a / top_k);
    lists.p[owner][row] = ((unsigned long long)epoch << 32) | ((unsigned long long)rank << 24) | token;
  }
}

}  // namespace

// Tell every owner where its inbox rows come from: for each kept assignment a of this rank (dest[a] = owner *
// rows_per_rank + row, or -1) store epoch | rank | token (a / top_k) into lists[owner][row] (8-byte stores into the
// owners' arenas).  Rows that nobody writes keep an older epoch and are read as padding.  tokens < 2^24, world <= 8.
extern "C" int b200_moe_post_sources(const void* dest, long long A, int top_k, long long rows_per_rank, int world,
                                     int rank, unsigned epoch, void* const* lists, void* stream) {
  if (A <= 0) return 0;
  if (world < 1 || world > kMaxPeers || rank < 0 || rank >= world || top_k <= 0 || rows_per_rank <= 0 ||
      A / top_k >= (1 << 24))
    return b200host::RC_BAD_SHAPE;
  ListPtrs lp = {};
  for (int r = 0; r < world; ++r) lp.p[r] = static_cast<unsigned long long*>(lists[r]);
  long long blocks = (A + 255) / 256;
  if (blocks > 1184) blocks = 1184;
  moe_post_sources_entry<<<(int)blocks, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      static_cast<const int*>(dest), A, top_k, rows_per_rank, world, rank, epoch, lp);
  return static_cast<int>(cudaGetLastError());
}

// C[rows, N] = inbox[rows, K] * W[group of the tile]^T with the inbox filled by this kernel's transfer CTAs from the
// ranks' token buffers x[r] ([tokens, K] bf16 as mapped here; every buffer and the source list are in place before
// the launch, e.g. behind a stream-ordered barrier).  W: [groups, N, K] bf16, `ldb` elements between its rows and
// `stride_b` between groups.  row_flags / tile_parts: rows / 128 uint32 each in local memory (flags hold earlier
// epochs, parts are zero).  K % 64 == 0, N % 64 == 0, rows % 128 == 0.
extern "C" int b200_moe_dispatch_gemm(const void* const* x, int tokens, const void* sources, void* inbox,
                                      const void* W, void* C, int rows, int N, int K, int groups, long long ldb,
                                      long long stride_b, const int* tile_group, int world, int rank, int n_xfer,
                                      void* row_flags, void* tile_parts, unsigned epoch, int* status, void* stream) {
  using namespace b200host;
  if (world < 1 || world > kMaxPeers || rank < 0 || rank >= world) return RC_BAD_SHAPE;
  if (rows <= 0 || rows % BM || N <= 0 || N % 64 || K <= 0 || K % BK || groups <= 0 || tokens <= 0 ||
      tokens >= (1 << 24))
    return RC_BAD_SHAPE;
  MoeGemmParams p = {};
  p.rows = rows;
  p.N = N;
  p.K = K;
  p.world = world;
  p.rank = rank;
  p.tokens = tokens;
  p.epoch = epoch;
  p.tile_group = tile_group;
  p.sources = static_cast<const unsigned long long*>(sources);
  for (int r = 0; r < world; ++r) {
    if (reinterpret_cast<uintptr_t>(x[r]) & 15u) return RC_BAD_ALIGNMENT;
    p.x[r] = static_cast<const __nv_bfloat16*>(x[r]);
  }
  if (reinterpret_cast<uintptr_t>(inbox) & 15u) return RC_BAD_ALIGNMENT;
  p.inbox = static_cast<__nv_bfloat16*>(inbox);
  p.row_flags = static_cast<uint32_t*>(row_flags);
  p.tile_parts = static_cast<uint32_t*>(tile_parts);
  p.status = status;
  // bytes per bulk copy: the largest power of two that divides a row, at most XFER_CHUNK (2 K is a multiple of 128)
  int chunk = XFER_CHUNK;
  while ((K * 2) % chunk) chunk >>= 1;
  if (chunk < 16) return RC_BAD_SHAPE;
  p.chunk_bytes = chunk;
  const int sms = sm_count();
  if (n_xfer <= 0) n_xfer = 16;
  if (n_xfer > sms / 4) n_xfer = sms / 4;
  p.n_xfer = n_xfer;
  const CUtensorMapDataType bf = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  const int BN = N > 128 ? 256 : 128;
  CUtensorMap tmA, tmB, tmC;
  int rc;
  if ((rc = make_map_3d(&tmA, bf, inbox, K, rows, 1, (uint64_t)K * 2, 0, BK, BM))) return rc;
  if ((rc = make_map_3d(&tmB, bf, W, K, N, groups, (uint64_t)ldb * 2, (uint64_t)stride_b * 2, BK, BN))) return rc;
  if ((rc = make_map_3d(&tmC, bf, C, N, rows, 1, (uint64_t)N * 2, 0, 64, 32))) return rc;
  const int tiles = (rows / BM) * ((N + BN - 1) / BN);
  const int compute = tiles < sms - n_xfer ? tiles : sms - n_xfer;
  const int grid = compute + n_xfer;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (BN == 256) return launch<256>(tmA, tmB, tmC, p, grid, s);
  return launch<128>(tmA, tmB, tmC, p, grid, s);
}
