// Flash attention backward for sm_100a (tcgen05 + TMEM + TMA): two kernels from one template.
//
//   dQ  kernel (DKV = false): a CTA keeps one 128-row query tile (Q_i, dO_i) resident and streams the
//        kv blocks:  S = Q K^T,  dP = dO V^T,  dS = P o (dP - delta) * scale,  dQ += dS K.
//   dKV kernel (DKV = true) : a CTA keeps one 128-row kv tile (K_j, V_j) resident and streams the query
//        blocks of every query head that shares the kv head, working on transposed tiles so that the
//        thread-per-row softmax math lines up with kv rows:
//        S^T = K Q^T,  dP^T = V dO^T,  P^T -> dV += P^T dO,  dS^T = P^T o (dP^T - delta) * scale -> dK += dS^T Q.
// Both recompute P from the saved log-sum-exp, so no atomics are needed and results are deterministic.
//
// Roles: warp 0 TMA producer (resident tiles once, stream operands through a 4-slot ring), warp 1 MMA
// issuer, warps 2-9 element-wise stage: warp w owns TMEM lane quadrant w % 4 and one 64-column half of
// the 128 x 128 score tile, so two warps share each row.  P / dS go to 128-byte swizzled shared memory as
// the K-major A operand of the accumulate MMAs; the streamed operand is consumed a second time as an
// MN-major B operand straight from its ring slot (no transposed copy).
//
// Masks as in the forward kernel: query row q sees kv positions [lo[q], q] (causal) or [lo[q], S).
// `hi` (int32 [B,S], non-decreasing) is the kv-side view: the last query position that can see kv k.
//
// Oracle: autograd of softmax(QK^T * scale) V in fp32 (reference attention:
// models/components/attention.py:269-278).  The reference's only hand-written backward is Hopper wgmma
// (third_party/ThunderKittens/kernels/attention/mha_h100/mha_h100.cu:254-483).
#include "b200.cuh"
#include "host_util.cuh"

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
  static constexpr int BUF_BYTES = TILE * TILE * 2;  // P / dS staging, also the epilogue staging
  static constexpr int X_OFF = 0;                    // two resident tiles
  static constexpr int RING_OFF = X_OFF + 2 * TILE_BYTES;
  static constexpr int BUF_OFF = RING_OFF + RING * TILE_BYTES;
  static constexpr int BAR_OFF = BUF_OFF + BUF_BYTES;
  static constexpr int TOTAL = BAR_OFF + 256;
};

struct BwdParams {
  int B, S, Skv, q_off, Hq, Hkv;  // S = query rows, Skv = kv rows, q_off = global position of query row 0
  int causal;
  float scale;
  const int* lo;       // [B,S] or nullptr
  const int* hi;       // [B,S] or nullptr (dKV kernel)
  const float* lse;    // [B,Hq,S]
  const float* delta;  // [B,Hq,S]
  int* status;
};

template <int D, bool DKV>
__global__ void __launch_bounds__(NUM_THREADS, 1)
attn_bwd_kernel(const __grid_constant__ CUtensorMap tmX1, const __grid_constant__ CUtensorMap tmX2,
                const __grid_constant__ CUtensorMap tmY1, const __grid_constant__ CUtensorMap tmY2,
                const __grid_constant__ CUtensorMap tmOut1, const __grid_constant__ CUtensorMap tmOut2,
                const BwdParams p) {
  using L = BwdSmem<D>;
  constexpr int NBOX = D / 64;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* x_full = reinterpret_cast<uint64_t*>(smem + L::BAR_OFF);
  uint64_t* full = x_full + 1;
  uint64_t* empty = full + RING;
  uint64_t* t_full = empty + RING;
  uint64_t* t_free = t_full + 1;
  uint64_t* p_ready = t_free + 1;
  uint64_t* dv_done = p_ready + 1;
  uint64_t* ds_ready = dv_done + 1;
  uint64_t* acc_done = ds_ready + 1;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_done + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const AbortCtx ab{abort_flag, p.status};

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int G = p.Hq / p.Hkv;
  const int q_tiles = (p.S + TILE - 1) / TILE;
  const int kv_tiles = (p.Skv + TILE - 1) / TILE;
  const int tiles = DKV ? kv_tiles : q_tiles;  // resident tiles per (batch, head)

  // ---- which resident tile, which stream range -------------------------------------------------
  int b, h_res, r0;            // batch, head of the resident tile, first row of the resident tile
  int blk_begin, blk_count;    // streamed block range (per query head for DKV)
  int n_total;                 // streamed blocks in total
  if (!DKV) {
    const int qt = tiles - 1 - (int)(blockIdx.x % tiles);  // heavy tiles first
    const int bh = blockIdx.x / tiles;
    h_res = bh % p.Hq;
    b = bh / p.Hq;
    r0 = qt * TILE;
    blk_begin = p.lo ? p.lo[(long long)b * p.S + r0] / TILE : 0;
    int end = kv_tiles;
    if (p.causal) end = min(end, (p.q_off + min(r0 + TILE, p.S) - 1) / TILE + 1);
    blk_count = max(end - blk_begin, 0);
    n_total = blk_count;
  } else {
    const int kt = (int)(blockIdx.x % tiles);  // early kv tiles have the most query blocks
    const int bh = blockIdx.x / tiles;
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
  const int hkv = DKV ? h_res : h_res / G;

  if (threadIdx.x == 0) {
    mbar_init(x_full, 1);
    for (int s = 0; s < RING; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    mbar_init(t_full, 1);
    mbar_init(t_free, EW_WARPS);
    mbar_init(p_ready, EW_WARPS);
    mbar_init(dv_done, 1);
    mbar_init(ds_ready, EW_WARPS);
    mbar_init(acc_done, 1);
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

  uint8_t* sX1 = smem + L::X_OFF;
  uint8_t* sX2 = sX1 + L::TILE_BYTES;
  uint8_t* sBuf = smem + L::BUF_OFF;

  if (warp == 0) {
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
      constexpr uint32_t idesc_a = make_idesc_bf16(TILE, D, false, true);      // buf (K-major) * Y (MN-major)
      auto issue_t = [&](uint32_t d_tmem, const uint8_t* x, const uint8_t* y) {
        const uint32_t a_base = smem_u32(x), b_base = smem_u32(y);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t off = (kk >> 2) * 16384 + (kk & 3) * 32;
          tc_mma_ss(d_tmem, make_smem_desc_sw128(a_base + off, 16, 1024), make_smem_desc_sw128(b_base + off, 16, 1024),
                    idesc_t, kk != 0 ? 1u : 0u);
        }
      };
      auto issue_acc = [&](uint32_t d_tmem, const uint8_t* y, bool accumulate) {
        const uint32_t a_base = smem_u32(sBuf), b_base = smem_u32(y);
#pragma unroll
        for (int kk = 0; kk < TILE / 16; ++kk) {
          const uint32_t a_off = (kk >> 2) * 16384 + (kk & 3) * 32;
          tc_mma_ss(d_tmem, make_smem_desc_sw128(a_base + a_off, 16, 1024),
                    make_smem_desc_sw128(b_base + kk * 2048, 16384, 1024), idesc_a, (accumulate || kk != 0) ? 1u : 0u);
        }
      };
      bool ok = mbar_wait(x_full, 0, ab, ERR_WAIT_FULL);
      for (int n = 0; n < n_total && ok; ++n) {
        const uint32_t ph = n & 1;
        const int s1 = (2 * n) % RING, s2 = (2 * n + 1) % RING;
        const uint32_t ring_ph = ((2 * n) / RING) & 1;
        const uint8_t* y1 = smem + L::RING_OFF + s1 * L::TILE_BYTES;
        const uint8_t* y2 = smem + L::RING_OFF + s2 * L::TILE_BYTES;
        if (!mbar_wait(&full[s1], ring_ph, ab, ERR_WAIT_FULL)) { ok = false; break; }
        if (!mbar_wait(&full[s2], ring_ph, ab, ERR_WAIT_FULL)) { ok = false; break; }
        if (n > 0 && !mbar_wait(t_free, ph ^ 1, ab, ERR_WAIT_TMEM_EMPTY)) { ok = false; break; }
        tc_fence_after();
        issue_t(tm_T1, sX1, y1);
        issue_t(tm_T2, sX2, y2);
        tc_commit(t_full);
        if (!DKV) {
          tc_commit(&empty[s2]);  // V is only read by dP
        } else {
          if (!mbar_wait(p_ready, ph, ab, ERR_WAIT_P_READY)) { ok = false; break; }
          tc_fence_after();
          issue_acc(tm_A2, y2, n > 0);  // dV += P^T dO
          tc_commit(dv_done);
          tc_commit(&empty[s2]);
        }
        if (!mbar_wait(ds_ready, ph, ab, ERR_WAIT_P_READY)) { ok = false; break; }
        tc_fence_after();
        issue_acc(tm_A1, y1, n > 0);  // dQ += dS K   or   dK += dS^T Q
        tc_commit(acc_done);
        tc_commit(&empty[s1]);
      }
    }
  } else {
    // ---------------------------------------------------------------- element-wise stage + epilogue
    const int quad = warp & 3;
    const int half = (warp - 2) >> 2;
    const int row = quad * 32 + lane;
    const int g_row = r0 + row;  // this thread's row: local query row (dQ) or kv position (dKV)
    const int q_pos = p.q_off + g_row;  // dQ only: global position of the query row
    const uint32_t lane_sel = static_cast<uint32_t>(quad * 32) << 16;
    const float scale_log2 = p.scale * kLog2e;
    float lse2_row = 0.f, delta_row = 0.f;
    int lo_row = 0;
    if (!DKV) {
      if (g_row < p.S) {
        const long long idx = ((long long)b * p.Hq + h_res) * p.S + g_row;
        lse2_row = p.lse[idx] * kLog2e;
        delta_row = p.delta[idx];
        if (p.lo) lo_row = p.lo[(long long)b * p.S + g_row];
      }
    }
    bool ok = n_total > 0;
    for (int n = 0; n < n_total && ok; ++n) {
      const uint32_t ph = n & 1;
      const int g = DKV ? n / blk_count : 0;
      const int blk = blk_begin + (DKV ? n % blk_count : n);
      const int c_base = blk * TILE + half * 64;  // global position of this warp's first column
      if (!mbar_wait_warp(t_full, ph, ab, ERR_WAIT_S_READY)) { ok = false; break; }
      tc_fence_after();
      if (!DKV) {
        // rows = queries, columns = kv
        const bool need_mask = (p.causal && blk * TILE + TILE - 1 > q_pos) || (blk * TILE < lo_row) ||
                               (blk * TILE + TILE > p.Skv) || (g_row >= p.S);
        const int hi_col = g_row >= p.S ? -1 : (p.causal ? min(q_pos, p.Skv - 1) : p.Skv - 1);
        if (n > 0 && !mbar_wait_warp(acc_done, ph ^ 1, ab, ERR_WAIT_O_READY)) { ok = false; break; }
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          uint32_t r1[32], r2[32];
          tmem_ld_32x32b_x32(tm_T1 + lane_sel + half * 64 + c * 32, r1);
          tmem_ld_32x32b_x32(tm_T2 + lane_sel + half * 64 + c * 32, r2);
          tmem_ld_wait();
          float ds[32];
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const float pr = exp2f(__uint_as_float(r1[i]) * scale_log2 - lse2_row);
            float v = pr * (__uint_as_float(r2[i]) - delta_row) * p.scale;
            if (need_mask) {
              const int col = c_base + c * 32 + i;
              if (col > hi_col || col < lo_row) v = 0.f;
            }
            ds[i] = v;
          }
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            uint4 v;
            v.x = pack_bf16x2(ds[8 * k + 0], ds[8 * k + 1]);
            v.y = pack_bf16x2(ds[8 * k + 2], ds[8 * k + 3]);
            v.z = pack_bf16x2(ds[8 * k + 4], ds[8 * k + 5]);
            v.w = pack_bf16x2(ds[8 * k + 6], ds[8 * k + 7]);
            *reinterpret_cast<uint4*>(sBuf + half * 16384 + sw128_offset(row, c * 4 + k)) = v;
          }
        }
        tc_fence_before();
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
          mbar_arrive(t_free);
          mbar_arrive(ds_ready);
        }
      } else {
        // rows = kv, columns = queries of head hq
        const int hq = hkv * G + g;
        const long long vec_base = ((long long)b * p.Hq + hq) * p.S;
        const int q_first = blk * TILE, q_last = min(blk * TILE + TILE, p.S) - 1;
        bool need_mask = (p.causal && p.q_off + q_first < r0 + TILE - 1) || (blk * TILE + TILE > p.S) ||
                         (r0 + TILE > p.Skv);
        if (p.lo) need_mask = need_mask || (p.lo[(long long)b * p.S + q_last] > r0);
        float pv[64];
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          uint32_t r1[32];
          tmem_ld_32x32b_x32(tm_T1 + lane_sel + half * 64 + c * 32, r1);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const int q = c_base + c * 32 + i;
            const float lse2 = q < p.S ? __ldg(p.lse + vec_base + q) * kLog2e : 0.f;
            float pr = exp2f(__uint_as_float(r1[i]) * scale_log2 - lse2);
            if (need_mask) {
              bool allowed = q < p.S && g_row < p.Skv && (!p.causal || p.q_off + q >= g_row);
              if (allowed && p.lo) allowed = g_row >= __ldg(p.lo + (long long)b * p.S + q);
              if (!allowed) pr = 0.f;
            }
            pv[c * 32 + i] = pr;
          }
        }
        if (n > 0 && !mbar_wait_warp(acc_done, ph ^ 1, ab, ERR_WAIT_O_READY)) { ok = false; break; }
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
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          uint32_t r2[32];
          tmem_ld_32x32b_x32(tm_T2 + lane_sel + half * 64 + c * 32, r2);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const int q = c_base + c * 32 + i;
            const float dl = q < p.S ? __ldg(p.delta + vec_base + q) : 0.f;
            pv[c * 32 + i] = pv[c * 32 + i] * (__uint_as_float(r2[i]) - dl) * p.scale;
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(t_free);
        if (!mbar_wait_warp(dv_done, ph, ab, ERR_WAIT_O_READY)) { ok = false; break; }
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
        if (lane == 0) mbar_arrive(ds_ready);
      }
    }
    // ---- epilogue: accumulators -> bf16 -> global.  Warp (quad, half) owns rows quad*32.. and the
    //      64-column box `half` of the D columns (for D = 64 only half 0 has columns).
    if (n_total > 0 && ok) ok = mbar_wait_warp(acc_done, (n_total - 1) & 1, ab, ERR_WAIT_O_READY);
    if ((n_total == 0 || ok) && half < NBOX) {
      tc_fence_after();
      const int slab_row = r0 + quad * 32;
      uint8_t* slab = sBuf + half * 16384 + quad * 32 * 128;
      for (int which = 0; which < (DKV ? 2 : 1); ++which) {
        const uint32_t acc = (which == 0 ? tm_A1 : tm_A2) + lane_sel + half * 64;
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
            v.x = pack_bf16x2(__uint_as_float(r[8 * k + 0]), __uint_as_float(r[8 * k + 1]));
            v.y = pack_bf16x2(__uint_as_float(r[8 * k + 2]), __uint_as_float(r[8 * k + 3]));
            v.z = pack_bf16x2(__uint_as_float(r[8 * k + 4]), __uint_as_float(r[8 * k + 5]));
            v.w = pack_bf16x2(__uint_as_float(r[8 * k + 6]), __uint_as_float(r[8 * k + 7]));
            *reinterpret_cast<uint4*>(slab + sw128_offset(lane, c * 4 + k)) = v;
          }
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0 && slab_row < (DKV ? p.Skv : p.S)) {
          tma_store_4d(which == 0 ? &tmOut1 : &tmOut2, slab, half * 64, h_res, slab_row, b);
          tma_commit_group();
          tma_wait_group_read<0>();
        }
        __syncwarp();
      }
      if (lane == 0) tma_wait_group<0>();
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

// delta[b,h,s] = sum_d dO[b,s,h,d] * O[b,s,h,d]; one warp per (b,s,h)
__global__ void attn_bwd_delta_kernel(const __nv_bfloat16* __restrict__ o, long long o_row, long long o_batch,
                                      const __nv_bfloat16* __restrict__ d_o, long long do_row, long long do_batch,
                                      float* __restrict__ delta, int B, int S, int H, int D) {
  const int lane = threadIdx.x & 31;
  const long long total = (long long)B * S * H;
  for (long long idx = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); idx < total;
       idx += (long long)gridDim.x * (blockDim.x >> 5)) {
    const int h = (int)(idx % H);
    const long long bs = idx / H;
    const int s = (int)(bs % S);
    const int b = (int)(bs / S);
    const __nv_bfloat16* po = o + b * o_batch + s * o_row + (long long)h * D;
    const __nv_bfloat16* pd = d_o + b * do_batch + s * do_row + (long long)h * D;
    float acc = 0.f;
    for (int d = lane * 8; d < D; d += 256) {
      const uint4 a = *reinterpret_cast<const uint4*>(po + d);
      const uint4 c = *reinterpret_cast<const uint4*>(pd + d);
      const __nv_bfloat162* ha = reinterpret_cast<const __nv_bfloat162*>(&a);
      const __nv_bfloat162* hc = reinterpret_cast<const __nv_bfloat162*>(&c);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 x = __bfloat1622float2(ha[i]), y = __bfloat1622float2(hc[i]);
        acc += x.x * y.x + x.y * y.y;
      }
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
    if (lane == 0) delta[((long long)b * H + h) * S + s] = acc;
  }
}

template <int D, bool DKV>
int launch_bwd(const CUtensorMap& x1, const CUtensorMap& x2, const CUtensorMap& y1, const CUtensorMap& y2,
               const CUtensorMap& o1, const CUtensorMap& o2, const BwdParams& p, cudaStream_t stream) {
  using L = BwdSmem<D>;
  auto* kern = attn_bwd_kernel<D, DKV>;
  constexpr int smem_bytes = L::TOTAL + 1024;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes);
    if (e != cudaSuccess) return static_cast<int>(e);
    configured = true;
  }
  const int tiles = ((DKV ? p.Skv : p.S) + TILE - 1) / TILE;
  const int grid = tiles * (DKV ? p.Hkv : p.Hq) * p.B;
  kern<<<grid, NUM_THREADS, smem_bytes, stream>>>(x1, x2, y1, y2, o1, o2, p);
  return static_cast<int>(cudaGetLastError());
}

}  // namespace

// All tensors are [B,S,H,D] views (heads D apart, dense last dim) given by base pointer + element
// strides between tokens (`*_row`) and batches (`*_batch`), outputs included (so dq/dk/dv may be column
// ranges of one packed gradient buffer).  dq/dk/dv are written (not accumulated).
// delta: [B,Hq,S] fp32 scratch that this call fills.  lo / hi: int32 [B,S] or null.
extern "C" int b200_attn_bwd(const void* q, const void* k, const void* v, const void* o, const void* d_o,
                             const void* lse, void* delta, void* dq, void* dk, void* dv, const void* lo,
                             const void* hi, int B, int S, int Hq, int Hkv, int D, long long q_row, long long q_batch,
                             long long k_row, long long k_batch, long long v_row, long long v_batch, long long o_row,
                             long long o_batch, long long do_row, long long do_batch, long long dq_row,
                             long long dq_batch, long long dk_row, long long dk_batch, long long dv_row,
                             long long dv_batch, float scale, int causal, long long skv_and_qoff, int* status,
                             void* stream) {
  using namespace b200host;
  const int Skv = (skv_and_qoff & 0xffffffffLL) ? (int)(skv_and_qoff & 0xffffffffLL) : S;
  const int q_off = (int)(skv_and_qoff >> 32);
  if (q_off % 128 != 0 || q_off < 0) return RC_BAD_SHAPE;
  if (B <= 0 || S <= 0 || Hq <= 0 || Hkv <= 0 || Hq % Hkv) return RC_BAD_SHAPE;
  if (D != 128 && D != 64) return RC_BAD_SHAPE;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  {
    const long long rows = (long long)B * S * Hq;
    long long blocks = (rows + 7) / 8;
    if (blocks > 148 * 16) blocks = 148 * 16;
    attn_bwd_delta_kernel<<<(int)blocks, 256, 0, s>>>((const __nv_bfloat16*)o, o_row, o_batch,
                                                      (const __nv_bfloat16*)d_o, do_row, do_batch, (float*)delta, B, S,
                                                      Hq, D);
  }
  const CUtensorMapDataType bf = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  const uint64_t hs = (uint64_t)D * 2;
  CUtensorMap tQ, tK, tV, tdO, tdQ, tdK, tdV;
  int rc;
  if ((rc = make_map_4d(&tQ, bf, q, D, Hq, S, B, hs, q_row * 2, q_batch * 2, 64, 1, 128))) return rc;
  if ((rc = make_map_4d(&tK, bf, k, D, Hkv, Skv, B, hs, k_row * 2, k_batch * 2, 64, 1, 128))) return rc;
  if ((rc = make_map_4d(&tV, bf, v, D, Hkv, Skv, B, hs, v_row * 2, v_batch * 2, 64, 1, 128))) return rc;
  if ((rc = make_map_4d(&tdO, bf, d_o, D, Hq, S, B, hs, do_row * 2, do_batch * 2, 64, 1, 128))) return rc;
  if ((rc = make_map_4d(&tdQ, bf, dq, D, Hq, S, B, hs, dq_row * 2, dq_batch * 2, 64, 1, 32))) return rc;
  if ((rc = make_map_4d(&tdK, bf, dk, D, Hkv, Skv, B, hs, dk_row * 2, dk_batch * 2, 64, 1, 32))) return rc;
  if ((rc = make_map_4d(&tdV, bf, dv, D, Hkv, Skv, B, hs, dv_row * 2, dv_batch * 2, 64, 1, 32))) return rc;
  BwdParams p{B, S, Skv, q_off, Hq, Hkv, causal, scale, (const int*)lo, (const int*)hi, (const float*)lse, (const float*)delta, status};
  if (D == 128) {
    if ((rc = launch_bwd<128, false>(tQ, tdO, tK, tV, tdQ, tdQ, p, s))) return rc;
    return launch_bwd<128, true>(tK, tV, tQ, tdO, tdK, tdV, p, s);
  }
  if ((rc = launch_bwd<64, false>(tQ, tdO, tK, tV, tdQ, tdQ, p, s))) return rc;
  return launch_bwd<64, true>(tK, tV, tQ, tdO, tdK, tdV, p, s);
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
