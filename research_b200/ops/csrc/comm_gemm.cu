// Tensor-parallel GEMMs fused with their collective, for sm_100a and NVLink peer memory.
//
//   MODE_GATHER  (all-gather -> GEMM):  C = gather_rows(A_r) * op(B).  Every rank holds a row shard of A in its
//       symmetric arena.  The first few CTAs of the grid are transfer CTAs: four threads each run a pipeline
//       that pulls remote 8 KB boxes with TMA (plain loads from the peer's memory, no cluster multicast)
//       through a shared-memory ring into the local gathered buffer and publishes one flag per 128-row block.  The
//       compute CTAs are the usual persistent tcgen05 pipeline; they walk the row blocks in arrival order
//       (own rows first, read straight from the local shard, then rank+1, rank+2, ...) and their TMA producer
//       waits on a block's flag only before the first load of a tile that needs it.  The transfer therefore
//       overlaps the math tile by tile and every remote byte crosses NVLink once.
//   MODE_SCATTER (GEMM -> reduce-scatter):  C_r = sum over ranks of (A * op(B)) restricted to the rows rank r
//       owns.  The epilogue adds each finished 32 x 64 box into the owner's output buffer with a TMA
//       reduce-add (a store to peer memory); the row blocks are walked starting with the next rank's so that
//       the ranks hit different destinations at any time.  The owner zeroes its buffer before the launch.
//
// Rows are interleaved the way sequence parallelism lays them out: with `chunk_blocks` 128-row blocks per
// (batch, rank) stretch, block g of the full matrix belongs to rank (g / chunk_blocks) % world.
//
// Cross-GPU ordering (comm.cuh, all waits bounded): at start every rank tells its peers "my shard is in place"
// (gather) or "my output is zeroed" (scatter); a peer's data is touched only after that flag; at the end the
// last CTA tells the peers "done" and waits for theirs, so when the kernel has ended the shard may be
// overwritten (gather) and the output is complete (scatter).
//
// Reference counterparts: third_party/ThunderKittens/kernels/parallel/ag_gemm/ag_gemm_b200.cu:54-258 and
// gemm_rs/gemm_rs_b200.cu:48-198 (both use cluster-multicast loads and unbounded waits); in the reference's own
// model code these are XLA-inserted collectives around cuBLAS dots (models/execution.py:183-250).
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
constexpr int MODE_GATHER = 1;
constexpr int MODE_SCATTER = 2;
// transfer CTAs: XFER_PIPES issuing threads, each with its own ring of XFER_BUFS boxes of XFER_BOX_BYTES
constexpr int XFER_PIPES = 4;
constexpr int XFER_BUFS = 6;
constexpr int XFER_LAG = XFER_BUFS - 2;
constexpr int XFER_BOX_BYTES = 8192;
constexpr int XFER_RING_BYTES = XFER_PIPES * XFER_BUFS * XFER_BOX_BYTES;
constexpr int MAP_C = kMaxPeers;          // PeerMaps slots beyond the per-rank ones (gather mode)
constexpr int MAP_OWN = kMaxPeers + 1;    //   own shard, swizzled, for the producer
constexpr int MAP_FULL = kMaxPeers + 2;   //   gathered buffer, transfer geometry

template <int BN>
struct SmemLayout {
  static constexpr int B_TILE_BYTES = BN * BK * 2;
  static constexpr int STAGE_BYTES = A_TILE_BYTES + B_TILE_BYTES;
  static constexpr int STAGING_OFF = STAGES * STAGE_BYTES;
  static constexpr int PIPE_END = STAGING_OFF + EPI_WARPS * 2 * STAGING_BYTES;
  static constexpr int BAR_OFF = PIPE_END > XFER_RING_BYTES ? PIPE_END : XFER_RING_BYTES;
  static constexpr int TOTAL = BAR_OFF + 512;
};

struct PeerMaps {
  CUtensorMap m[kMaxPeers + 3];  // one per rank, then MAP_C / MAP_OWN / MAP_FULL
};

struct CommGemmParams {
  int M, N, K;               // full problem: M rows over all ranks
  int world, rank;
  int chunk_blocks;          // 128-row blocks per (batch, rank) stretch
  int blocks_per_rank;       // M / 128 / world
  int n_xfer;                // transfer CTAs (gather mode)
  int copy_own;              // transfer CTAs also copy this rank's own rows into the gathered buffer
  int xfer_cols, xfer_rows;  // box of the transfer maps: xfer_cols * xfer_rows * 2 == XFER_BOX_BYTES
  uint32_t epoch;
  uint32_t* row_flags;       // [M / 128] local flags, gather mode
  uint32_t* counter;         // zero on entry, left zero
  FlagBlock* flags[kMaxPeers];
  int* status;
};

// logical row block i (arrival order for this rank) -> owner rank, block inside the owner's shard, block of the
// full matrix
__device__ __forceinline__ void map_block(const CommGemmParams& p, int i, int first_step, int& owner, int& local,
                                          int& global) {
  const int s = i / p.blocks_per_rank;
  local = i - s * p.blocks_per_rank;
  owner = (p.rank + first_step + s) % p.world;
  const int b = local / p.chunk_blocks, j = local - b * p.chunk_blocks;
  global = (b * p.world + owner) * p.chunk_blocks + j;
}

template <int BN, bool B_MN, int MODE>
__global__ void __launch_bounds__(NUM_THREADS, 1)
comm_gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                 const __grid_constant__ PeerMaps peers, const CommGemmParams p) {
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
  // transfer CTAs take the lowest block indices so that they are placed first
  const int n_xfer = MODE == MODE_GATHER ? p.n_xfer : 0;
  const int n_compute = (int)gridDim.x - n_xfer;
  const bool is_xfer = (int)blockIdx.x < n_xfer;
  const int cta = (int)blockIdx.x - n_xfer;  // index among the compute CTAs
  const int tiles_m = p.M / BM;
  const int tiles_n = (p.N + BN - 1) / BN;
  const int total_tiles = tiles_m * tiles_n;
  const int k_blocks = p.K / BK;
  constexpr int kFirstStep = MODE == MODE_GATHER ? 0 : 1;

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
  // announce to the peers: shard in place (gather) / output zeroed (scatter)
  if (blockIdx.x == 0 && threadIdx.x < p.world && (int)threadIdx.x != p.rank) {
    __threadfence_system();
    st_release_sys(&p.flags[threadIdx.x]->ready[p.rank], p.epoch);
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
    mi = first_m + in_group % gm;  // logical row block
    n0 = (in_group / gm) * BN;
  };

  if (is_xfer) {
    // ------------------------------------------------------------------ transfer CTA (gather mode)
    if (lane == 0 && warp < XFER_PIPES) {
      // one pipeline per issuing thread: load a box from the owner's shard, store it into the gathered buffer
      const int pipe = (int)blockIdx.x * XFER_PIPES + warp;
      const int n_pipes = p.n_xfer * XFER_PIPES;
      uint8_t* ring = smem + warp * XFER_BUFS * XFER_BOX_BYTES;
      uint64_t* bar = xbar + warp * XFER_BUFS;
      const int remote_blocks = (p.world - 1) * p.blocks_per_rank;
      // this pipeline's blocks: remote logical indices blocks_per_rank + pipe, + n_pipes, ...; then own rows
      const int my_remote = remote_blocks > pipe ? (remote_blocks - pipe + n_pipes - 1) / n_pipes : 0;
      const int my_own =
          (p.copy_own && p.blocks_per_rank > pipe) ? (p.blocks_per_rank - pipe + n_pipes - 1) / n_pipes : 0;
      const int col_boxes = p.K / p.xfer_cols, row_boxes = BM / p.xfer_rows;
      const int boxes = col_boxes * row_boxes;  // per 128-row block
      const long long total = (long long)(my_remote + my_own) * boxes;
      auto locate = [&](long long i, int& owner, int& local, int& global, int& col, int& row, bool& last) {
        const int blk = (int)(i / boxes), bx = (int)(i % boxes);
        const int logical = blk < my_remote ? p.blocks_per_rank + pipe + blk * n_pipes : pipe + (blk - my_remote) * n_pipes;
        map_block(p, logical, 0, owner, local, global);
        col = (bx % col_boxes) * p.xfer_cols;
        row = (bx / col_boxes) * p.xfer_rows;
        last = bx == boxes - 1;
      };
      bool ok = true;
      uint32_t ready_mask = 1u << p.rank;
      for (long long i = 0; i < total + XFER_LAG && ok; ++i) {
        int owner, local, global, col, row;
        bool last;
        if (i < total) {
          locate(i, owner, local, global, col, row, last);
          if (!(ready_mask >> owner & 1u)) {
            if (!wait_sys(&p.flags[p.rank]->ready[owner], p.epoch, p.status, ERR_PEER_READY)) { ok = false; break; }
            ready_mask |= 1u << owner;
          }
          const int buf = (int)(i % XFER_BUFS);
          if (i >= XFER_BUFS) tma_wait_group_read<1>();  // the store that last read this buffer is done
          mbar_expect_tx(&bar[buf], XFER_BOX_BYTES);
          tma_load_3d(ring + buf * XFER_BOX_BYTES, &peers.m[owner], &bar[buf], col, local * BM + row, 0);
        }
        const long long j = i - XFER_LAG;
        if (j >= 0 && j < total) {
          locate(j, owner, local, global, col, row, last);
          const int buf = (int)(j % XFER_BUFS);
          if (!mbar_wait(&bar[buf], (uint32_t)(j / XFER_BUFS) & 1u, ab, ERR_WAIT_FULL)) { ok = false; break; }
          tma_store_3d(&peers.m[MAP_FULL], ring + buf * XFER_BOX_BYTES, col, global * BM + row, 0);
          tma_commit_group();
          if (last) {
            // the whole row block has been issued: wait until it is in memory, then publish it
            tma_wait_group<0>();
            fence_proxy_async_all();
            st_release_gpu(&p.row_flags[global], p.epoch);
          }
        }
      }
      tma_wait_group<0>();
      if (!ok) {
        const uint64_t t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
      }
      // last pipeline to finish: this rank has finished reading its peers' shards
      __threadfence();
      if (atomicAdd(p.counter, 1u) == (uint32_t)n_pipes - 1u) {
        *p.counter = 0u;
        for (int r = 0; r < p.world; ++r)
          if (r != p.rank) st_release_sys(&p.flags[r]->done[p.rank], p.epoch);
        for (int r = 0; r < p.world; ++r)
          if (r != p.rank) wait_sys(&p.flags[p.rank]->done[r], p.epoch, p.status, ERR_PEER_DONE);
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
        int mi, n0, owner, local, global;
        tile_coords(t, mi, n0);
        map_block(p, mi, kFirstStep, owner, local, global);
        const bool own_shard = MODE == MODE_GATHER && owner == p.rank;
        if (MODE == MODE_GATHER && !own_shard) {
          if (!wait_gpu(&p.row_flags[global], p.epoch, p.status, ERR_LOCAL_FLAG)) {
            *ab.flag = 1;
            ok = false;
            break;
          }
          fence_proxy_async_all();
        }
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait(&empty[s], ph ^ 1, ab, ERR_WAIT_EMPTY)) { ok = false; break; }
          uint8_t* sA = smem + s * L::STAGE_BYTES;
          uint8_t* sB = sA + A_TILE_BYTES;
          mbar_expect_tx(&full[s], L::STAGE_BYTES);
          if (own_shard)
            tma_load_3d(sA, &peers.m[MAP_OWN], &full[s], kb * BK, local * BM, 0);  // own rows: straight from the shard
          else
            tma_load_3d(sA, &tmA, &full[s], kb * BK, global * BM, 0);
          if (!B_MN) {
            tma_load_3d(sB, &tmB, &full[s], kb * BK, n0, 0);
          } else {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j) tma_load_3d(sB + j * 8192, &tmB, &full[s], n0 + j * 64, kb * BK, 0);
          }
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
      constexpr uint32_t idesc = make_idesc_bf16(BM, BN, false, B_MN);
      uint32_t it = 0, tile_iter = 0;
      bool ok = true;
      for (int t = cta; t < total_tiles && ok; t += n_compute) {
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
            const uint64_t bdesc = make_smem_desc_sw128(b_base + (B_MN ? k * 2048 : k * 32), B_MN ? 8192 : 16, 1024);
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
    uint32_t ready_mask = 1u << p.rank;
    bool ok = true;
    for (int t = cta; t < total_tiles && ok; t += n_compute) {
      int mi, n0, owner, local, global;
      tile_coords(t, mi, n0);
      map_block(p, mi, kFirstStep, owner, local, global);
      const uint32_t acc = tile_iter & 1;
      const uint32_t acc_ph = (tile_iter >> 1) & 1;
      ++tile_iter;
      if (!mbar_wait_warp(&tfull[acc], acc_ph, ab, ERR_WAIT_TMEM_FULL)) { ok = false; break; }
      tc_fence_after();
      if (MODE == MODE_SCATTER && !(ready_mask >> owner & 1u)) {
        // the owner has zeroed its output for this epoch
        bool got = true;
        if (lane == 0) got = wait_sys(&p.flags[p.rank]->ready[owner], p.epoch, p.status, ERR_PEER_READY);
        got = __shfl_sync(0xffffffffu, got, 0);
        if (!got) {
          if (lane == 0) *ab.flag = 1;
          ok = false;
          break;
        }
        ready_mask |= 1u << owner;
      }
      const uint32_t t_row = tmem_base + acc * BN + (static_cast<uint32_t>(q * 32) << 16);
      const int out_row = (MODE == MODE_GATHER ? global : local) * BM + q * 32;
      const CUtensorMap* out_map = MODE == MODE_GATHER ? &peers.m[MAP_C] : &peers.m[owner];
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
          if (MODE == MODE_SCATTER)
            tma_reduce_add_3d(out_map, buf, col0, out_row, 0);
          else
            tma_store_3d(out_map, buf, col0, out_row, 0);
          tma_commit_group();
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty[acc]);
    }
    if (lane == 0) {
      tma_wait_group<0>();
      if (MODE == MODE_SCATTER) {
        fence_proxy_async_all();
        __threadfence_system();
      }
    }
  }

  // ------------------------------------------------------------------ teardown
  tc_fence_before();
  __syncthreads();
  if (warp == 1 && !is_xfer) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem_base, 2 * BN);
  }
  if (MODE == MODE_SCATTER && threadIdx.x == 0) {
    // every reduce-add of this CTA has completed (each issuing lane waited for its groups above)
    __threadfence_system();
    if (atomicAdd(p.counter, 1u) == gridDim.x - 1u) {
      *p.counter = 0u;
      for (int r = 0; r < p.world; ++r)
        if (r != p.rank) st_release_sys(&p.flags[r]->done[p.rank], p.epoch);
      for (int r = 0; r < p.world; ++r)
        if (r != p.rank) wait_sys(&p.flags[p.rank]->done[r], p.epoch, p.status, ERR_PEER_DONE);
    }
  }
}

template <int BN, bool B_MN, int MODE>
int launch(const CUtensorMap& tmA, const CUtensorMap& tmB, const PeerMaps& peers, const CommGemmParams& p, int grid,
           cudaStream_t stream) {
  using L = SmemLayout<BN>;
  auto* kern = comm_gemm_kernel<BN, B_MN, MODE>;
  constexpr int smem_bytes = L::TOTAL + 1024;
  static bool configured[b200host::kMaxDevices] = {};   // per kernel instantiation and device
  if (int rc = b200host::ensure_dynamic_smem(kern, smem_bytes, configured)) return rc;
  kern<<<grid, NUM_THREADS, smem_bytes, stream>>>(tmA, tmB, peers, p);
  return static_cast<int>(cudaGetLastError());
}

int fill_common(CommGemmParams& p, int M, int N, int K, int world, int rank, int chunk_blocks, unsigned epoch,
                void* const* flags, void* counter, int* status) {
  using namespace b200host;
  if (world < 1 || world > kMaxPeers || rank < 0 || rank >= world) return RC_BAD_SHAPE;
  if (M <= 0 || N <= 0 || K <= 0 || M % (BM * world) || K % BK || N % 64) return RC_BAD_SHAPE;
  const int blocks_per_rank = M / BM / world;
  if (chunk_blocks <= 0 || blocks_per_rank % chunk_blocks) return RC_BAD_SHAPE;
  p.M = M;
  p.N = N;
  p.K = K;
  p.world = world;
  p.rank = rank;
  p.chunk_blocks = chunk_blocks;
  p.blocks_per_rank = blocks_per_rank;
  p.n_xfer = 0;
  p.xfer_cols = p.xfer_rows = 0;
  p.copy_own = 0;
  p.epoch = epoch;
  p.row_flags = nullptr;
  p.counter = static_cast<uint32_t*>(counter);
  for (int r = 0; r < kMaxPeers; ++r) p.flags[r] = r < world ? static_cast<FlagBlock*>(flags[r]) : nullptr;
  p.status = status;
  return 0;
}

}  // namespace

// C[M,N] = gather(A shards)[M,K] * op(B).  a_shards[r]: rank r's [M/world, K] bf16 shard as mapped here
// (a_shards[rank] is the local one); a_full: local [M,K] buffer the remote rows are gathered into (complete when
// the kernel has ended; own rows are copied too when copy_own is set, else they are the caller's job); B: [N,K] (b_mn = 0) or [K,N] (b_mn = 1); C: local [M,N] bf16.
// row_flags: M/128 uint32 in local memory (values from earlier epochs are fine); counter: one zeroed uint32.
extern "C" int b200_gemm_allgather(const void* const* a_shards, void* a_full, const void* B, void* C, int M, int N,
                                   int K, long long ldb, int b_mn, int world, int rank, int chunk_blocks, int n_xfer,
                                   int copy_own, void* row_flags, void* counter, void* const* flags, unsigned epoch, int* status,
                                   void* stream) {
  using namespace b200host;
  CommGemmParams p;
  int rc = fill_common(p, M, N, K, world, rank, chunk_blocks, epoch, flags, counter, status);
  if (rc) return rc;
  const int sms = sm_count();
  if (n_xfer <= 0) n_xfer = 16;
  if (n_xfer > sms / 4) n_xfer = sms / 4;
  p.n_xfer = n_xfer;
  p.copy_own = copy_own;
  p.row_flags = static_cast<uint32_t*>(row_flags);
  const CUtensorMapDataType bf = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  const int BN = N > 128 ? 256 : 128;
  CUtensorMap tmA, tmB;
  PeerMaps peers = {};
  // transfer boxes: rows as wide as the column count allows (up to 512 bytes), no swizzle
  p.xfer_cols = K % 256 == 0 ? 256 : (K % 128 == 0 ? 128 : 64);
  p.xfer_rows = XFER_BOX_BYTES / 2 / p.xfer_cols;
  if ((rc = make_map_3d(&tmA, bf, a_full, K, M, 1, (uint64_t)K * 2, 0, BK, BM))) return rc;
  for (int r = 0; r < world; ++r)
    if ((rc = make_map_3d(&peers.m[r], bf, a_shards[r], K, M / world, 1, (uint64_t)K * 2, 0, p.xfer_cols, p.xfer_rows,
                          CU_TENSOR_MAP_SWIZZLE_NONE)))
      return rc;
  if ((rc = make_map_3d(&peers.m[MAP_FULL], bf, a_full, K, M, 1, (uint64_t)K * 2, 0, p.xfer_cols, p.xfer_rows,
                        CU_TENSOR_MAP_SWIZZLE_NONE)))
    return rc;
  if ((rc = make_map_3d(&peers.m[MAP_OWN], bf, a_shards[rank], K, M / world, 1, (uint64_t)K * 2, 0, BK, BM))) return rc;
  if ((rc = make_map_3d(&peers.m[MAP_C], bf, C, N, M, 1, (uint64_t)N * 2, 0, 64, 32))) return rc;
  if (p.xfer_cols <= 0 || p.xfer_rows <= 0 || BM % p.xfer_rows || K % p.xfer_cols) return RC_BAD_SHAPE;
  if (!b_mn)
    rc = make_map_3d(&tmB, bf, B, K, N, 1, ldb * 2, 0, BK, BN);
  else
    rc = make_map_3d(&tmB, bf, B, N, K, 1, ldb * 2, 0, 64, BK);
  if (rc) return rc;
  const int tiles = (M / BM) * ((N + BN - 1) / BN);
  int compute = tiles < sms - n_xfer ? tiles : sms - n_xfer;
  const int grid = compute + n_xfer;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (BN == 256) return b_mn ? launch<256, true, MODE_GATHER>(tmA, tmB, peers, p, grid, s)
                             : launch<256, false, MODE_GATHER>(tmA, tmB, peers, p, grid, s);
  return b_mn ? launch<128, true, MODE_GATHER>(tmA, tmB, peers, p, grid, s)
              : launch<128, false, MODE_GATHER>(tmA, tmB, peers, p, grid, s);
}

// c_shards[r] += rows of (A[M,K] * op(B)) that rank r owns.  A: local [M,K] bf16; c_shards[r]: rank r's
// [M/world, N] bf16 output as mapped here, zeroed by its owner before that owner's launch.
extern "C" int b200_gemm_reducescatter(const void* A, const void* B, void* const* c_shards, int M, int N, int K,
                                       long long lda, long long ldb, int b_mn, int world, int rank, int chunk_blocks,
                                       void* counter, void* const* flags, unsigned epoch, int* status, void* stream) {
  using namespace b200host;
  CommGemmParams p;
  int rc = fill_common(p, M, N, K, world, rank, chunk_blocks, epoch, flags, counter, status);
  if (rc) return rc;
  const CUtensorMapDataType bf = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  const int BN = N > 128 ? 256 : 128;
  CUtensorMap tmA, tmB;
  PeerMaps peers = {};
  if ((rc = make_map_3d(&tmA, bf, A, K, M, 1, lda * 2, 0, BK, BM))) return rc;
  for (int r = 0; r < world; ++r)
    if ((rc = make_map_3d(&peers.m[r], bf, c_shards[r], N, M / world, 1, (uint64_t)N * 2, 0, 64, 32))) return rc;
  if (!b_mn)
    rc = make_map_3d(&tmB, bf, B, K, N, 1, ldb * 2, 0, BK, BN);
  else
    rc = make_map_3d(&tmB, bf, B, N, K, 1, ldb * 2, 0, 64, BK);
  if (rc) return rc;
  const int tiles = (M / BM) * ((N + BN - 1) / BN);
  const int sms = sm_count();
  const int grid = tiles < sms ? tiles : sms;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (BN == 256) return b_mn ? launch<256, true, MODE_SCATTER>(tmA, tmB, peers, p, grid, s)
                             : launch<256, false, MODE_SCATTER>(tmA, tmB, peers, p, grid, s);
  return b_mn ? launch<128, true, MODE_SCATTER>(tmA, tmB, peers, p, grid, s)
              : launch<128, false, MODE_SCATTER>(tmA, tmB, peers, p, grid, s);
}
