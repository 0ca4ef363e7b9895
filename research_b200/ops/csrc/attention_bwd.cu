// Flash attention backward for sm_100a (tcgen05 + TMEM + TMA): two kernels from one template.
//
//   dQ  kernel (DKV = false): a CTA keeps one 128-row query tile (Q_i, dO_i) resident and streams the
//        kv blocks:  S = Q K^T,  dP = dO V^T,  dS = P o (dP - delta),  dQ = scale * sum dS K.
//   dKV kernel (DKV = true) : a CTA keeps one 128-row kv tile (K_j, V_j) resident and streams the query
//        blocks of every query head that shares the kv head, working on transposed tiles so that the
//        thread-per-row math lines up with kv rows:
//        S^T = K Q^T,  dP^T = V dO^T,  dV = sum P^T dO,  dS^T = P^T o (dP^T - delta),  dK = scale * sum dS^T Q.
// Both recompute P from the saved log-sum-exp, so no atomics are needed and results are deterministic.
//
// Roles: warp 0 TMA producer (resident tiles once, streamed operands through a 4-slot ring), warp 1 MMA
// issuer, warps 2-9 element-wise stage: warp w owns TMEM lane quadrant w % 4 and one 64-column half of
// the 128 x 128 score tile, so two warps share each row.
//
// Software pipeline: the score MMA of block n+1 is issued as soon as the element-wise warps have copied
// S(n) out of tensor memory, so the tensor pipe works on block n+1 while block n's exponentials run.
// dS goes back to tensor memory as packed bf16 (in place over dP in the dKV kernel, where all 512 columns
// are taken) and is the A operand of the accumulate MMA straight from there; only P^T of the dKV kernel
// takes the trip through 128-byte swizzled shared memory.  The streamed operand is consumed a second time
// as an MN-major B operand from its ring slot (no transposed copy).  Per-query statistics of the dKV
// kernel (lse, delta of the streamed block) are staged through a small double-buffered shared array one
// block ahead.
//
// Masks as in the forward kernel: query row q sees kv positions [lo[q], q] (causal) or [lo[q], S).
// `hi` (int32 [B,Skv], non-decreasing) is the kv-side view: the last query position that can see kv k;
// the dKV kernel masks with it alone, so it must be given whenever `lo` is.
//
// Context parallelism (`ring.enabled`, see ring.cuh): K and V are the staging buffers in sequence order.  The dQ
// kernel carries the transfer CTAs that fill them and waits on a block's flag before it streams the block; the
// dKV kernel, which runs after it, finds everything staged and ADDS its dK / dV tiles into the accumulation
// buffer of the rank that owns those kv rows with TMA reduce-adds (bf16), own rows included, so that the
// contributions of all ranks and of both local query chunks meet in one buffer per owner.
//
// Oracle: autograd of softmax(QK^T * scale) V in fp32 (reference attention:
// models/components/attention.py:269-278).  The reference's only hand-written backward is Hopper wgmma
// (third_party/ThunderKittens/kernels/attention/mha_h100/mha_h100.cu:254-483).
#include <math_constants.h>

#include "b200.cuh"
#include "host_util.cuh"
#include "ring.cuh"

using namespace b200;

namespace {

constexpr int TILE = 128;
constexpr int RING = 4;
constexpr int EW_WARPS = 8;
constexpr int NUM_THREADS = 32 * (2 + EW_WARPS);
constexpr float kLog2e = 1.4426950408889634f;

template <int D>
struct BwdSmem {
  static constexpr int TILE_BYTES = TILE * D * 2;
  static constexpr int BUF_BYTES = TILE * TILE * 2;  // P^T staging (dKV), also the epilogue staging
  static constexpr int X_OFF = 0;                    // two resident tiles
  static constexpr int RING_OFF = X_OFF + 2 * TILE_BYTES;
  static constexpr int BUF_OFF = RING_OFF + RING * TILE_BYTES;
  static constexpr int STAT_OFF = BUF_OFF + BUF_BYTES;  // [2][lse2[128], delta[128]] fp32
  static constexpr int BAR_OFF = STAT_OFF + 2 * 2 * TILE * 4;
  static constexpr int TOTAL = BAR_OFF + 256;
};

struct BwdParams {
  int B, S, Skv, q_off, Hq, Hkv;  // S = query rows, Skv = kv rows, q_off = global position of query row 0
  int causal;
  float scale;
  const int* lo;       // [B,S] or nullptr (dQ kernel)
  const int* hi;       // [B,Skv] or nullptr (dKV kernel)
  const float* lse;    // [B,Hq,S]
  const float* delta;  // [B,Hq,S]
  int* status;
  b200ring::RingArgs ring;
};

// dK / dV accumulation buffers of every rank of the context group ([B, local rows, Hkv, D] bf16), as tensor maps.
struct OwnerMaps {
  CUtensorMap dk[b200comm::kMaxPeers];
  CUtensorMap dv[b200comm::kMaxPeers];
};

template <int D, bool DKV>
__global__ void __launch_bounds__(NUM_THREADS, 1)
attn_bwd_kernel(const __grid_constant__ CUtensorMap tmX1, const __grid_constant__ CUtensorMap tmX2,
                const __grid_constant__ CUtensorMap tmY1, const __grid_constant__ CUtensorMap tmY2,
                const __grid_constant__ CUtensorMap tmOut1, const __grid_constant__ CUtensorMap tmOut2,
                const __grid_constant__ OwnerMaps owners, const BwdParams p) {
  using L = BwdSmem<D>;
  constexpr int NBOX = D / 64;
  // The swizzled tiles need 1024-byte alignment and the budget has no room for a round-up, so the
  // alignment of the dynamic window is checked instead of assumed.
  extern __shared__ __align__(1024) uint8_t smem[];
  if (smem_u32(smem) & 1023u) {
    if (threadIdx.x == 0) atomicCAS(p.status, 0, ERR_BAD_ARG);
    return;
  }
  uint64_t* x_full = reinterpret_cast<uint64_t*>(smem + L::BAR_OFF);
  uint64_t* full = x_full + 1;
  uint64_t* empty = full + RING;
  uint64_t* s_full = empty + RING;     // S(n) is in tensor memory
  uint64_t* dp_full = s_full + 1;      // dP(n) is in tensor memory
  uint64_t* t1_free = dp_full + 1;     // S(n) has been copied out
  uint64_t* p_ready = t1_free + 1;     // P^T(n) is in shared memory (dKV)
  uint64_t* dv_done = p_ready + 1;     // the MMA that read P^T(n) has finished (dKV)
  uint64_t* ds_ready = dv_done + 1;    // dS(n) is in tensor memory
  uint64_t* acc_done = ds_ready + 1;   // every MMA has finished
  uint64_t* stat_ready = acc_done + 1; // statistics of block n are in shared memory (dKV)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(stat_ready + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const AbortCtx ab{abort_flag, p.status};

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int G = p.Hq / p.Hkv;
  const int q_tiles = (p.S + TILE - 1) / TILE;
  const int kv_tiles = (p.Skv + TILE - 1) / TILE;
  const int tiles = DKV ? kv_tiles : q_tiles;  // resident tiles per (batch, head)

  // ---- which resident tile, which stream range.  Tiles are handed out heaviest first over the whole
  //      grid (all heads of the longest tile, then the next), which balances the tail. ----------------
  int b, h_res, r0;            // batch, head of the resident tile, first row of the resident tile
  int blk_begin, blk_count;    // streamed block range (per query head for DKV)
  int n_total;                 // streamed blocks in total
  // context parallelism: the first CTAs of the dQ launch stage K/V instead of computing
  const int n_xfer = (!DKV && p.ring.enabled) ? p.ring.n_transfer : 0;
  const bool is_xfer = (int)blockIdx.x < n_xfer;
  {
    const int cta = is_xfer ? 0 : (int)blockIdx.x - n_xfer;
    const int nbh = p.B * (DKV ? p.Hkv : p.Hq);
    const int t_idx = cta / nbh;
    const int bh = cta % nbh;
    if (!DKV) {
      const int qt = tiles - 1 - t_idx;
      h_res = bh % p.Hq;
      b = bh / p.Hq;
      r0 = qt * TILE;
      blk_begin = p.lo ? p.lo[(long long)b * p.S + r0] / TILE : 0;
      int end = kv_tiles;
      if (p.causal) end = min(end, (p.q_off + min(r0 + TILE, p.S) - 1) / TILE + 1);
      blk_count = max(end - blk_begin, 0);
      n_total = blk_count;
    } else {
      const int kt = t_idx;
      h_res = bh % p.Hkv;
      b = bh / p.Hkv;
      r0 = kt * TILE;
      // query blocks are in local rows; a query row r sits at global position q_off + r
      blk_begin = p.causal ? max(0, (r0 - p.q_off) / TILE) : 0;
      int end = q_tiles;
      if (p.hi) {
        const int last_q = p.hi[(long long)b * p.Skv + min(r0 + TILE, p.Skv) - 1] - p.q_off;  // local row, may be < 0
        end = last_q < 0 ? 0 : min(end, last_q / TILE + 1);
      }
      blk_count = max(end - blk_begin, 0);
      n_total = blk_count * G;
    }
    if (is_xfer) blk_count = n_total = 0;
  }
  const int hkv = DKV ? h_res : h_res / G;

  if (threadIdx.x == 0) {
    mbar_init(x_full, 1);
    for (int s = 0; s < RING; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    mbar_init(s_full, 1);
    mbar_init(dp_full, 1);
    mbar_init(t1_free, EW_WARPS);
    mbar_init(p_ready, EW_WARPS);
    mbar_init(dv_done, 1);
    mbar_init(ds_ready, EW_WARPS);
    mbar_init(acc_done, 1);
    mbar_init(stat_ready, EW_WARPS);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tm_T1 = tmem_base, tm_T2 = tmem_base + 128, tm_A1 = tmem_base + 256, tm_A2 = tmem_base + 256 + D;
  // packed bf16 dS: warp half h writes 32 columns at tm_DS + 64 h.  The dKV kernel has no free columns
  // and overwrites the first half of each warp's own dP columns; the dQ kernel uses the unused quarter.
  const uint32_t tm_DS = DKV ? tm_T2 : tmem_base + 384;

  uint8_t* sX1 = smem + L::X_OFF;
  uint8_t* sX2 = sX1 + L::TILE_BYTES;
  uint8_t* sBuf = smem + L::BUF_OFF;

  if (is_xfer) {
    // ---------------------------------------------------------------- K/V transfer (context parallelism)
    // buffers and barriers of the copy pipelines sit in front of this kernel's statistics and barriers
    b200ring::transfer_cta<b200ring::pipes_for_window(L::STAT_OFF)>(p.ring, smem, ab);
  } else if (warp == 0) {
    // ---------------------------------------------------------------- TMA producer
    if (lane == 0 && n_total > 0) {
      tma_prefetch_desc(&tmX1);
      tma_prefetch_desc(&tmX2);
      tma_prefetch_desc(&tmY1);
      tma_prefetch_desc(&tmY2);
      mbar_expect_tx(x_full, 2 * L::TILE_BYTES);
      for (int bx = 0; bx < NBOX; ++bx) {
        tma_load_4d(sX1 + bx * 16384, &tmX1, x_full, bx * 64, h_res, r0, b);
        tma_load_4d(sX2 + bx * 16384, &tmX2, x_full, bx * 64, h_res, r0, b);
      }
      bool ok = true;
      for (int n = 0; n < n_total && ok; ++n) {
        const int g = DKV ? n / blk_count : 0;
        const int blk = blk_begin + (DKV ? n % blk_count : n);
        const int hy = DKV ? hkv * G + g : hkv;
        if (!DKV && p.ring.enabled && !b200ring::wait_block(p.ring, b, blk, p.status)) {
          *ab.flag = 1;   // the kv block never arrived: the other roles of this CTA stop waiting too
          ok = false;
          break;
        }
        for (int which = 0; which < 2; ++which) {
          const uint32_t item = 2 * n + which;
          const int slot = item % RING;
          if (!mbar_wait(&empty[slot], ((item / RING) & 1) ^ 1, ab, ERR_WAIT_EMPTY)) { ok = false; break; }
          mbar_expect_tx(&full[slot], L::TILE_BYTES);
          uint8_t* dst = smem + L::RING_OFF + slot * L::TILE_BYTES;
          for (int bx = 0; bx < NBOX; ++bx)
            tma_load_4d(dst + bx * 16384, which ? &tmY2 : &tmY1, &full[slot], bx * 64, hy, blk * TILE, b);
        }
      }
      if (!ok) {
        const uint64_t t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer
    if (lane == 0 && n_total > 0) {
      constexpr uint32_t idesc_t = make_idesc_bf16(TILE, TILE, false, false);  // X * Y^T, both K-major over D
      constexpr uint32_t idesc_a = make_idesc_bf16(TILE, D, false, true);      // K-major A * Y (MN-major)
      auto ybuf = [&](int item) -> const uint8_t* { return smem + L::RING_OFF + (item % RING) * L::TILE_BYTES; };
      auto ring_wait = [&](int item) { return mbar_wait(&full[item % RING], (item / RING) & 1, ab, ERR_WAIT_FULL); };
      // One descriptor per operand, built when the product is issued; the slice of an MMA instruction is that
      // descriptor plus a compile-time constant in its address field (units of 16 bytes), so nothing but an add
      // sits between two of the 64-clock instructions that this one thread issues.
      auto issue_t = [&](uint32_t d_tmem, const uint8_t* x, const uint8_t* y) {
        const uint64_t a0 = make_smem_desc_sw128(smem_u32(x), 16, 1024), b0 = make_smem_desc_sw128(smem_u32(y), 16, 1024);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint64_t off = (uint64_t)(((kk >> 2) * 16384 + (kk & 3) * 32) >> 4);
          tc_mma_ss(d_tmem, a0 + off, b0 + off, idesc_t, kk != 0 ? 1u : 0u);
        }
      };
      // A = P^T in shared memory
      auto issue_acc_ss = [&](uint32_t d_tmem, const uint8_t* y, bool accumulate) {
        const uint64_t a0 = make_smem_desc_sw128(smem_u32(sBuf), 16, 1024);
        const uint64_t b0 = make_smem_desc_sw128(smem_u32(y), 16384, 1024);
#pragma unroll
        for (int kk = 0; kk < TILE / 16; ++kk) {
          const uint64_t a_off = (uint64_t)(((kk >> 2) * 16384 + (kk & 3) * 32) >> 4);
          tc_mma_ss(d_tmem, a0 + a_off, b0 + (uint64_t)((kk * 2048) >> 4), idesc_a, (accumulate || kk != 0) ? 1u : 0u);
        }
      };
      // A = packed dS in tensor memory: 16 K-elements are 8 columns; the two 64-element halves sit 64 columns apart
      auto issue_acc_ts = [&](uint32_t d_tmem, const uint8_t* y, bool accumulate) {
        const uint64_t b0 = make_smem_desc_sw128(smem_u32(y), 16384, 1024);
#pragma unroll
        for (int kk = 0; kk < TILE / 16; ++kk) {
          tc_mma_ts(d_tmem, tm_DS + (kk >> 2) * 64 + (kk & 3) * 8, b0 + (uint64_t)((kk * 2048) >> 4), idesc_a,
                    (accumulate || kk != 0) ? 1u : 0u);
        }
      };
      bool ok = mbar_wait(x_full, 0, ab, ERR_WAIT_FULL);
      if (ok) ok = ring_wait(0);
      if (ok) {
        tc_fence_after();
        issue_t(tm_T1, sX1, ybuf(0));
        tc_commit(s_full);
        ok = ring_wait(1);
      }
      if (ok) {
        issue_t(tm_T2, sX2, ybuf(1));
        tc_commit(dp_full);
        if (!DKV) tc_commit(&empty[1]);  // V is only read by dP
      }
      for (int n = 0; n < n_total && ok; ++n) {
        const uint32_t ph = n & 1;
        const bool has_next = n + 1 < n_total;
        const int it_s = 2 * n + 2, it_p = 2 * n + 3;
        bool s_issued = !has_next;
        // S(n+1) ahead of everything else when its operands are already there
        if (has_next && mbar_try_wait(&full[it_s % RING], (it_s / RING) & 1) && mbar_try_wait(t1_free, ph)) {
          tc_fence_after();
          issue_t(tm_T1, sX1, ybuf(it_s));
          tc_commit(s_full);
          s_issued = true;
        }
        if (DKV) {
          if (!mbar_wait(p_ready, ph, ab, ERR_WAIT_P_READY)) { ok = false; break; }
          tc_fence_after();
          issue_acc_ss(tm_A2, ybuf(2 * n + 1), n > 0);  // dV += P^T dO
          tc_commit(dv_done);
          tc_commit(&empty[(2 * n + 1) % RING]);
        }
        if (!s_issued) {
          if (!ring_wait(it_s)) { ok = false; break; }
          if (!mbar_wait(t1_free, ph, ab, ERR_WAIT_TMEM_EMPTY)) { ok = false; break; }
          tc_fence_after();
          issue_t(tm_T1, sX1, ybuf(it_s));
          tc_commit(s_full);
        }
        if (!mbar_wait(ds_ready, ph, ab, ERR_WAIT_P_READY)) { ok = false; break; }
        tc_fence_after();
        issue_acc_ts(tm_A1, ybuf(2 * n), n > 0);  // dQ += dS K   or   dK += dS^T Q
        tc_commit(&empty[(2 * n) % RING]);
        if (has_next) {
          // after the accumulate MMA in issue order: in the dKV kernel dP(n+1) overwrites the dS it read
          if (!ring_wait(it_p)) { ok = false; break; }
          issue_t(tm_T2, sX2, ybuf(it_p));
          tc_commit(dp_full);
          if (!DKV) tc_commit(&empty[it_p % RING]);
        }
      }
      if (ok) tc_commit(acc_done);
    }
  } else {
    // ---------------------------------------------------------------- element-wise stage + epilogue
    const int quad = warp & 3;
    const int half = (warp - 2) >> 2;
    const int row = quad * 32 + lane;
    const int g_row = r0 + row;         // this thread's row: local query row (dQ) or kv position (dKV)
    const int q_pos = p.q_off + g_row;  // dQ only: global position of the query row
    const int t_ew = threadIdx.x - 64;  // 0..255 among the element-wise threads
    const uint32_t lane_sel = static_cast<uint32_t>(quad * 32) << 16;
    const float scale_log2 = p.scale * kLog2e;
    float* stats = reinterpret_cast<float*>(smem + L::STAT_OFF);
    float lse2_row = 0.f, delta_row = 0.f;
    int lo_row = 0;
    int q_min = 0, q_max = p.S - 1;  // dKV only: local query rows this kv row is visible to
    if (!DKV) {
      if (g_row < p.S) {
        const long long idx = ((long long)b * p.Hq + h_res) * p.S + g_row;
        lse2_row = p.lse[idx] * kLog2e;
        delta_row = p.delta[idx];
        if (p.lo) lo_row = p.lo[(long long)b * p.S + g_row];
      }
    } else {
      if (p.causal) q_min = max(0, g_row - p.q_off);
      if (p.hi && g_row < p.Skv) q_max = min(q_max, p.hi[(long long)b * p.Skv + g_row] - p.q_off);
    }
    // dKV: thread t < 128 fetches lse * log2(e) of query t of block n, thread t >= 128 its delta;
    // rows past the end get lse = +inf, which makes P exactly zero there.
    auto load_stat = [&](int n) -> float {
      const int g = n / blk_count;
      const int blk = blk_begin + n % blk_count;
      const int q = blk * TILE + (t_ew & 127);
      const long long idx = ((long long)b * p.Hq + hkv * G + g) * p.S + q;
      if (t_ew < 128) return q < p.S ? __ldg(p.lse + idx) * kLog2e : CUDART_INF_F;
      return q < p.S ? __ldg(p.delta + idx) : 0.f;
    };
    bool ok = n_total > 0;
    if (DKV && ok) {
      stats[t_ew] = load_stat(0);
      __syncwarp();
      if (lane == 0) mbar_arrive(stat_ready);
    }
    for (int n = 0; n < n_total && ok; ++n) {
      const uint32_t ph = n & 1;
      const int blk = blk_begin + (DKV ? n % blk_count : n);
      float stat_next = 0.f;
      if (DKV && n + 1 < n_total) stat_next = load_stat(n + 1);
      const float* st = stats + (n & 1) * 256 + half * 64;  // lse2 of this warp's 64 columns; delta 128 floats on
      if (DKV && !mbar_wait_warp(stat_ready, ph, ab, ERR_WAIT_S_READY)) { ok = false; break; }
      if (!mbar_wait_warp(s_full, ph, ab, ERR_WAIT_S_READY)) { ok = false; break; }
      tc_fence_after();
      float pv[64];
      {
        uint32_t ra[32], rb[32];
        tmem_ld_32x32b_x32(tm_T1 + lane_sel + half * 64, ra);
        tmem_ld_32x32b_x32(tm_T1 + lane_sel + half * 64 + 32, rb);
        tmem_ld_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(t1_free);
        if (!DKV) {
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            pv[i] = ex2_approx(fmaf(__uint_as_float(ra[i]), scale_log2, -lse2_row));
            pv[32 + i] = ex2_approx(fmaf(__uint_as_float(rb[i]), scale_log2, -lse2_row));
          }
        } else {
#pragma unroll
          for (int i4 = 0; i4 < 8; ++i4) {
            const float4 la = *reinterpret_cast<const float4*>(st + 4 * i4);
            const float4 lb = *reinterpret_cast<const float4*>(st + 32 + 4 * i4);
            pv[4 * i4 + 0] = ex2_approx(fmaf(__uint_as_float(ra[4 * i4 + 0]), scale_log2, -la.x));
            pv[4 * i4 + 1] = ex2_approx(fmaf(__uint_as_float(ra[4 * i4 + 1]), scale_log2, -la.y));
            pv[4 * i4 + 2] = ex2_approx(fmaf(__uint_as_float(ra[4 * i4 + 2]), scale_log2, -la.z));
            pv[4 * i4 + 3] = ex2_approx(fmaf(__uint_as_float(ra[4 * i4 + 3]), scale_log2, -la.w));
            pv[32 + 4 * i4 + 0] = ex2_approx(fmaf(__uint_as_float(rb[4 * i4 + 0]), scale_log2, -lb.x));
            pv[32 + 4 * i4 + 1] = ex2_approx(fmaf(__uint_as_float(rb[4 * i4 + 1]), scale_log2, -lb.y));
            pv[32 + 4 * i4 + 2] = ex2_approx(fmaf(__uint_as_float(rb[4 * i4 + 2]), scale_log2, -lb.z));
            pv[32 + 4 * i4 + 3] = ex2_approx(fmaf(__uint_as_float(rb[4 * i4 + 3]), scale_log2, -lb.w));
          }
        }
      }
      const int c0 = blk * TILE + half * 64;  // first column of this warp: kv position (dQ) or local query row (dKV)
      if (!DKV) {
        // rows = queries, columns = kv
        const int hi_col = g_row >= p.S ? -1 : (p.causal ? min(q_pos, p.Skv - 1) : p.Skv - 1);
        if (__any_sync(0xffffffffu, c0 + 63 > hi_col || c0 < lo_row)) {
#pragma unroll
          for (int i = 0; i < 64; ++i)
            if (c0 + i > hi_col || c0 + i < lo_row) pv[i] = 0.f;
        }
      } else {
        // rows = kv, columns = queries.  kv rows past Skv need no mask: they only reach output rows
        // that the store clips.
        if (__any_sync(0xffffffffu, c0 < q_min || c0 + 63 > q_max)) {
#pragma unroll
          for (int i = 0; i < 64; ++i)
            if (c0 + i < q_min || c0 + i > q_max) pv[i] = 0.f;
        }
        if (n > 0 && !mbar_wait_warp(dv_done, ph ^ 1, ab, ERR_WAIT_O_READY)) { ok = false; break; }
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          uint4 v;
          v.x = pack_bf16x2(pv[8 * k + 0], pv[8 * k + 1]);
          v.y = pack_bf16x2(pv[8 * k + 2], pv[8 * k + 3]);
          v.z = pack_bf16x2(pv[8 * k + 4], pv[8 * k + 5]);
          v.w = pack_bf16x2(pv[8 * k + 6], pv[8 * k + 7]);
          *reinterpret_cast<uint4*>(sBuf + half * 16384 + sw128_offset(row, k)) = v;
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(p_ready);
      }
      if (!mbar_wait_warp(dp_full, ph, ab, ERR_WAIT_S_READY)) { ok = false; break; }
      tc_fence_after();
      {
        uint32_t ra[32], rb[32], packed[32];
        tmem_ld_32x32b_x32(tm_T2 + lane_sel + half * 64, ra);
        tmem_ld_32x32b_x32(tm_T2 + lane_sel + half * 64 + 32, rb);
        tmem_ld_wait();
        if (!DKV) {
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            packed[i] = pack_bf16x2(pv[2 * i] * (__uint_as_float(ra[2 * i]) - delta_row),
                                    pv[2 * i + 1] * (__uint_as_float(ra[2 * i + 1]) - delta_row));
            packed[16 + i] = pack_bf16x2(pv[32 + 2 * i] * (__uint_as_float(rb[2 * i]) - delta_row),
                                         pv[32 + 2 * i + 1] * (__uint_as_float(rb[2 * i + 1]) - delta_row));
          }
        } else {
#pragma unroll
          for (int i4 = 0; i4 < 8; ++i4) {
            const float4 da = *reinterpret_cast<const float4*>(st + 128 + 4 * i4);
            const float4 db = *reinterpret_cast<const float4*>(st + 128 + 32 + 4 * i4);
            packed[2 * i4] = pack_bf16x2(pv[4 * i4] * (__uint_as_float(ra[4 * i4]) - da.x),
                                         pv[4 * i4 + 1] * (__uint_as_float(ra[4 * i4 + 1]) - da.y));
            packed[2 * i4 + 1] = pack_bf16x2(pv[4 * i4 + 2] * (__uint_as_float(ra[4 * i4 + 2]) - da.z),
                                             pv[4 * i4 + 3] * (__uint_as_float(ra[4 * i4 + 3]) - da.w));
            packed[16 + 2 * i4] = pack_bf16x2(pv[32 + 4 * i4] * (__uint_as_float(rb[4 * i4]) - db.x),
                                              pv[32 + 4 * i4 + 1] * (__uint_as_float(rb[4 * i4 + 1]) - db.y));
            packed[16 + 2 * i4 + 1] = pack_bf16x2(pv[32 + 4 * i4 + 2] * (__uint_as_float(rb[4 * i4 + 2]) - db.z),
                                                  pv[32 + 4 * i4 + 3] * (__uint_as_float(rb[4 * i4 + 3]) - db.w));
          }
        }
        tmem_st_32x32b_x32(tm_DS + lane_sel + half * 64, packed);
        tmem_st_wait();
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(ds_ready);
      if (DKV && n + 1 < n_total) {
        stats[((n + 1) & 1) * 256 + t_ew] = stat_next;
        __syncwarp();
        if (lane == 0) mbar_arrive(stat_ready);
      }
    }
    // ---- epilogue: accumulators -> bf16 -> global.  Warp (quad, half) owns rows quad*32.. and the
    //      64-column box `half` of the D columns (for D = 64 only half 0 has columns).  The softmax scale
    //      that dS left out is applied here (dQ and dK; dV has none).
    if (n_total > 0 && ok) ok = mbar_wait_warp(acc_done, 0, ab, ERR_WAIT_O_READY);
    // with per-owner accumulation a tile that no local query sees adds nothing; transfer CTAs compute nothing
    const bool skip_empty = is_xfer || (DKV && p.ring.enabled && n_total == 0);
    if ((n_total == 0 || ok) && half < NBOX && !skip_empty) {
      tc_fence_after();
      const int slab_row = r0 + quad * 32;
      uint8_t* slab = sBuf + half * 16384 + quad * 32 * 128;
      for (int which = 0; which < (DKV ? 2 : 1); ++which) {
        const uint32_t acc = (which == 0 ? tm_A1 : tm_A2) + lane_sel + half * 64;
        const float mul = which == 0 ? p.scale : 1.f;
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          uint32_t r[32];
          if (n_total > 0) {
            tmem_ld_32x32b_x32(acc + c * 32, r);
            tmem_ld_wait();
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) r[i] = 0u;
          }
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            uint4 v;
            v.x = pack_bf16x2(__uint_as_float(r[8 * k + 0]) * mul, __uint_as_float(r[8 * k + 1]) * mul);
            v.y = pack_bf16x2(__uint_as_float(r[8 * k + 2]) * mul, __uint_as_float(r[8 * k + 3]) * mul);
            v.z = pack_bf16x2(__uint_as_float(r[8 * k + 4]) * mul, __uint_as_float(r[8 * k + 5]) * mul);
            v.w = pack_bf16x2(__uint_as_float(r[8 * k + 6]) * mul, __uint_as_float(r[8 * k + 7]) * mul);
            *reinterpret_cast<uint4*>(slab + sw128_offset(lane, c * 4 + k)) = v;
          }
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0 && slab_row < (DKV ? p.Skv : p.S)) {
          if (DKV && p.ring.enabled) {
            // kv rows of the sequence -> the rank that owns them and the row in its buffer
            const int seg = slab_row / p.ring.seg_rows;
            const int owner = p.ring.seg_owner[seg];
            const int local = p.ring.seg_first_row[seg] + slab_row % p.ring.seg_rows;
            tma_reduce_add_4d(which == 0 ? &owners.dk[owner] : &owners.dv[owner], slab, half * 64, h_res, local, b);
          } else {
            tma_store_4d(which == 0 ? &tmOut1 : &tmOut2, slab, half * 64, h_res, slab_row, b);
          }
          tma_commit_group();
          tma_wait_group_read<0>();
        }
        __syncwarp();
      }
      if (lane == 0) {
        tma_wait_group<0>();
        if (DKV && p.ring.enabled) __threadfence_system();   // the adds have landed at their owners
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

// delta[b,h,s] = sum_d dO[b,s,h,d] * O[b,s,h,d]; D / 8 lanes per (b,s,h), so a warp covers 32 / (D / 8) heads at once
__global__ void attn_bwd_delta_kernel(const __nv_bfloat16* __restrict__ o, long long o_row, long long o_batch,
                                      const __nv_bfloat16* __restrict__ d_o, long long do_row, long long do_batch,
                                      float* __restrict__ delta, int B, int S, int H, int D) {
  const int lane = threadIdx.x & 31;
  const int lph = D >> 3;            // 8 or 16 lanes per head (D = 64 or 128)
  const int hpw = 32 / lph;
  const int sub = lane / lph, l = lane % lph;
  const long long total = (long long)B * S * H;
  const long long groups = (total + hpw - 1) / hpw;
  for (long long gidx = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); gidx < groups;
       gidx += (long long)gridDim.x * (blockDim.x >> 5)) {
    const long long idx = gidx * hpw + sub;
    float acc = 0.f;
    int h = 0, s = 0, b = 0;
    if (idx < total) {
      h = (int)(idx % H);
      const long long bs = idx / H;
      s = (int)(bs % S);
      b = (int)(bs / S);
      const __nv_bfloat16* po = o + b * o_batch + s * o_row + (long long)h * D + l * 8;
      const __nv_bfloat16* pd = d_o + b * do_batch + s * do_row + (long long)h * D + l * 8;
      const uint4 a = *reinterpret_cast<const uint4*>(po);
      const uint4 c = *reinterpret_cast<const uint4*>(pd);
      const __nv_bfloat162* ha = reinterpret_cast<const __nv_bfloat162*>(&a);
      const __nv_bfloat162* hc = reinterpret_cast<const __nv_bfloat162*>(&c);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 x = __bfloat1622float2(ha[i]), y = __bfloat1622float2(hc[i]);
        acc += x.x * y.x + x.y * y.y;
      }
    }
    for (int off = lph >> 1; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
    if (l == 0 && idx < total) delta[((long long)b * H + h) * S + s] = acc;
  }
}

template <int D, bool DKV>
int launch_bwd(const CUtensorMap& x1, const CUtensorMap& x2, const CUtensorMap& y1, const CUtensorMap& y2,
               const CUtensorMap& o1, const CUtensorMap& o2, const OwnerMaps& owners, const BwdParams& p,
               cudaStream_t stream) {
  using L = BwdSmem<D>;
  auto* kern = attn_bwd_kernel<D, DKV>;
  constexpr int smem_bytes = L::TOTAL;
  static bool configured[b200host::kMaxDevices] = {};   // per kernel instantiation and device
  if (int rc = b200host::ensure_dynamic_smem(kern, smem_bytes, configured)) return rc;
  const int tiles = ((DKV ? p.Skv : p.S) + TILE - 1) / TILE;
  const int grid = tiles * (DKV ? p.Hkv : p.Hq) * p.B + ((!DKV && p.ring.enabled) ? p.ring.n_transfer : 0);
  kern<<<grid, NUM_THREADS, smem_bytes, stream>>>(x1, x2, y1, y2, o1, o2, owners, p);
  return static_cast<int>(cudaGetLastError());
}

}  // namespace

// All tensors are [B,S,H,D] views (heads D apart, dense last dim) given by base pointer + element
// strides between tokens (`*_row`) and batches (`*_batch`), outputs included (so dq/dk/dv may be column
// ranges of one packed gradient buffer).  dq/dk/dv are written (not accumulated).
// delta: [B,Hq,S] fp32 scratch that this call fills.  lo / hi: int32 [B,S] or null.
static int attn_bwd_impl(const void* q, const void* k, const void* v, const void* o, const void* d_o, const void* lse,
                         void* delta, void* dq, void* dk, void* dv, const void* lo, const void* hi, int B, int S,
                         int Hq, int Hkv, int D, long long q_row, long long q_batch, long long k_row,
                         long long k_batch, long long v_row, long long v_batch, long long o_row, long long o_batch,
                         long long do_row, long long do_batch, long long dq_row, long long dq_batch, long long dk_row,
                         long long dk_batch, long long dv_row, long long dv_batch, float scale, int causal,
                         long long skv_and_qoff, const b200ring::RingHostArgs* ring, int* status, void* stream) {
  using namespace b200host;
  const int Skv = (skv_and_qoff & 0xffffffffLL) ? (int)(skv_and_qoff & 0xffffffffLL) : S;
  const int q_off = (int)(skv_and_qoff >> 32);
  if (q_off % 128 != 0 || q_off < 0) return RC_BAD_SHAPE;
  if (B <= 0 || S <= 0 || Hq <= 0 || Hkv <= 0 || Hq % Hkv) return RC_BAD_SHAPE;
  if (D != 128 && D != 64) return RC_BAD_SHAPE;
  if (lo != nullptr && hi == nullptr) return RC_BAD_SHAPE;  // the dKV kernel masks with the kv-side bound
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  const CUtensorMapDataType bf = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  const uint64_t hs = (uint64_t)D * 2;
  CUtensorMap tQ, tK, tV, tdO, tdQ, tdK, tdV;
  static const OwnerMaps no_owners = {};
  OwnerMaps owner_maps = {};
  int rc;
  BwdParams p{B, S, Skv, q_off, Hq, Hkv, causal, scale, (const int*)lo, (const int*)hi, (const float*)lse, (const float*)delta, status};
  if (ring) {
    // K and V are the staging buffers: dense [B, seq_len, Hkv, D]; dK / dV go to the owners' accumulation buffers
    if (k_row != (long long)Hkv * D || v_row != k_row || k_batch != (long long)ring->seq_len * k_row ||
        v_batch != k_batch || Skv > ring->seq_len || Skv % 128)
      return RC_BAD_SHAPE;
    if ((rc = b200ring::fill_ring_args(p.ring, *ring, const_cast<void*>(k), const_cast<void*>(v), B, Hkv, D))) return rc;
    const uint64_t row_b = (uint64_t)Hkv * D * 2, batch_b = (uint64_t)ring->local_rows * row_b;
    for (int r = 0; r < ring->world; ++r) {
      if (!ring->peer_dk[r] || !ring->peer_dv[r]) return RC_BAD_ALIGNMENT;
      if ((rc = make_map_4d(&owner_maps.dk[r], bf, ring->peer_dk[r], D, Hkv, ring->local_rows, B, hs, row_b, batch_b, 64,
                            1, 32)))
        return rc;
      if ((rc = make_map_4d(&owner_maps.dv[r], bf, ring->peer_dv[r], D, Hkv, ring->local_rows, B, hs, row_b, batch_b, 64,
                            1, 32)))
        return rc;
    }
  }
  {
    const long long rows = ((long long)B * S * Hq + (256 / D) - 1) / (256 / D);  // warps of work
    long long blocks = (rows + 7) / 8;
    if (blocks > 148 * 16) blocks = 148 * 16;
    attn_bwd_delta_kernel<<<(int)blocks, 256, 0, s>>>((const __nv_bfloat16*)o, o_row, o_batch,
                                                      (const __nv_bfloat16*)d_o, do_row, do_batch, (float*)delta, B, S,
                                                      Hq, D);
  }
  if ((rc = make_map_4d(&tQ, bf, q, D, Hq, S, B, hs, q_row * 2, q_batch * 2, 64, 1, 128))) return rc;
  if ((rc = make_map_4d(&tK, bf, k, D, Hkv, Skv, B, hs, k_row * 2, k_batch * 2, 64, 1, 128))) return rc;
  if ((rc = make_map_4d(&tV, bf, v, D, Hkv, Skv, B, hs, v_row * 2, v_batch * 2, 64, 1, 128))) return rc;
  if ((rc = make_map_4d(&tdO, bf, d_o, D, Hq, S, B, hs, do_row * 2, do_batch * 2, 64, 1, 128))) return rc;
  if ((rc = make_map_4d(&tdQ, bf, dq, D, Hq, S, B, hs, dq_row * 2, dq_batch * 2, 64, 1, 32))) return rc;
  if (!ring) {
    if ((rc = make_map_4d(&tdK, bf, dk, D, Hkv, Skv, B, hs, dk_row * 2, dk_batch * 2, 64, 1, 32))) return rc;
    if ((rc = make_map_4d(&tdV, bf, dv, D, Hkv, Skv, B, hs, dv_row * 2, dv_batch * 2, 64, 1, 32))) return rc;
  } else {
    tdK = tdQ;   // never stored through: the dKV kernel adds into the owners' buffers
    tdV = tdQ;
  }
  const OwnerMaps& om = ring ? owner_maps : no_owners;
  if (D == 128) {
    if ((rc = launch_bwd<128, false>(tQ, tdO, tK, tV, tdQ, tdQ, om, p, s))) return rc;
    return launch_bwd<128, true>(tK, tV, tQ, tdO, tdK, tdV, om, p, s);
  }
  if ((rc = launch_bwd<64, false>(tQ, tdO, tK, tV, tdQ, tdQ, om, p, s))) return rc;
  return launch_bwd<64, true>(tK, tV, tQ, tdO, tdK, tdV, om, p, s);
}

extern "C" int b200_attn_bwd(const void* q, const void* k, const void* v, const void* o, const void* d_o,
                             const void* lse, void* delta, void* dq, void* dk, void* dv, const void* lo,
                             const void* hi, int B, int S, int Hq, int Hkv, int D, long long q_row, long long q_batch,
                             long long k_row, long long k_batch, long long v_row, long long v_batch, long long o_row,
                             long long o_batch, long long do_row, long long do_batch, long long dq_row,
                             long long dq_batch, long long dk_row, long long dk_batch, long long dv_row,
                             long long dv_batch, float scale, int causal, long long skv_and_qoff, int* status,
                             void* stream) {
  return attn_bwd_impl(q, k, v, o, d_o, lse, delta, dq, dk, dv, lo, hi, B, S, Hq, Hkv, D, q_row, q_batch, k_row,
                       k_batch, v_row, v_batch, o_row, o_batch, do_row, do_batch, dq_row, dq_batch, dk_row, dk_batch,
                       dv_row, dv_batch, scale, causal, skv_and_qoff, nullptr, status, stream);
}

// The same for context parallelism (ring.cuh): k, v are this rank's staging buffers [B, seq_len, Hkv, D]; the dQ
// launch stages the blocks listed in `ring` while it runs; dK and dV are ADDED into the accumulation buffers of
// the ranks that own the kv rows (`ring->peer_dk / peer_dv`, zeroed by their owners before the launch).
extern "C" int b200_attn_bwd_ring(const void* q, const void* k, const void* v, const void* o, const void* d_o,
                                  const void* lse, void* delta, void* dq, const void* lo, const void* hi, int B, int S,
                                  int Hq, int Hkv, int D, long long q_row, long long q_batch, long long k_row,
                                  long long k_batch, long long o_row, long long o_batch, long long do_row,
                                  long long do_batch, long long dq_row, long long dq_batch, float scale, int causal,
                                  long long skv_and_qoff, const void* ring, int* status, void* stream) {
  if (!ring) return b200host::RC_BAD_SHAPE;
  return attn_bwd_impl(q, k, v, o, d_o, lse, delta, dq, nullptr, nullptr, lo, hi, B, S, Hq, Hkv, D, q_row, q_batch,
                       k_row, k_batch, k_row, k_batch, o_row, o_batch, do_row, do_batch, dq_row, dq_batch, 0, 0, 0, 0,
                       scale, causal, skv_and_qoff, static_cast<const b200ring::RingHostArgs*>(ring), status, stream);
}

// ---------------------------------------------------------------------------------------------------
// Allocation-free variant (see attention_bwd_noalloc.h): the delta scratch is a fixed array in the library
// image instead of a caller-allocated buffer.
// ---------------------------------------------------------------------------------------------------
#include "attention_bwd_noalloc.h"

static __device__ __align__(256) float g_attn_bwd_delta_scratch[B200_ATTN_NOALLOC_MAX_ROWS];

extern "C" int b200_attn_bwd_noalloc(const void* q, const void* k, const void* v, const void* o, const void* d_o,
                                     const void* lse, void* dq, void* dk, void* dv, const void* lo, const void* hi,
                                     int B, int S, int Hq, int Hkv, int D, long long q_row, long long q_batch,
                                     long long k_row, long long k_batch, long long v_row, long long v_batch,
                                     long long o_row, long long o_batch, long long do_row, long long do_batch,
                                     long long dq_row, long long dq_batch, long long dk_row, long long dk_batch,
                                     long long dv_row, long long dv_batch, float scale, int causal, int* status,
                                     void* stream) {
  if (B <= 0 || S <= 0 || Hq <= 0) return b200host::RC_BAD_SHAPE;
  const long long rows = (long long)B * Hq * S;
  if (rows > (long long)B200_ATTN_NOALLOC_MAX_ROWS) {
    fprintf(stderr,
            "b200_attn_bwd_noalloc: B*Hq*S = %lld exceeds the built-in scratch of %d rows; use b200_attn_bwd with a "
            "caller-provided delta buffer\n",
            rows, (int)B200_ATTN_NOALLOC_MAX_ROWS);
    return B200_ATTN_NOALLOC_TOO_LARGE;
  }
  // In host code the array's name is only a handle; the kernels need its device address, which differs per
  // device.  Looked up once per device (with that device current) and cached.
  static float* scratch_ptr[64] = {nullptr};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return B200_ATTN_NOALLOC_SYMBOL_FAILED;
  if (scratch_ptr[dev] == nullptr) {
    float* ptr = nullptr;
    const cudaError_t e = cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_attn_bwd_delta_scratch);
    if (e != cudaSuccess || ptr == nullptr) {
      fprintf(stderr, "b200_attn_bwd_noalloc: cudaGetSymbolAddress failed: %s\n", cudaGetErrorString(e));
      return B200_ATTN_NOALLOC_SYMBOL_FAILED;
    }
    scratch_ptr[dev] = ptr;
  }
  return b200_attn_bwd(q, k, v, o, d_o, lse, scratch_ptr[dev], dq, dk, dv, lo, hi, B, S, Hq, Hkv, D, q_row, q_batch,
                       k_row, k_batch, v_row, v_batch, o_row, o_batch, do_row, do_batch, dq_row, dq_batch, dk_row,
                       dk_batch, dv_row, dv_batch, scale, causal, 0LL, status, stream);
}
