// Flash attention forward for sm_100a (tcgen05 + TMEM + TMA), bf16 in/out, fp32 softmax.
//
// One CTA owns 256 query rows of one (batch, head): two 128-row tiles that ping-pong through the
// tensor core so that the softmax of one tile overlaps the MMAs of the other.
//   warp 0      TMA producer: both Q tiles once, then K/V blocks of 128 rows through a 3-slot ring
//   warp 1      MMA issuer  : S_t = Q_t K^T (TMEM, 128 cols per tile), O_t += P_t V (TMEM, D cols)
//   warps 2-5   softmax of tile 0, warps 6-9 softmax of tile 1: one thread per query row reads its
//               row of S with tcgen05.ld, keeps the running max / sum, writes P (bf16) into 128-byte
//               swizzled shared memory for the second MMA, and rescales O in TMEM only when the
//               running max moved by more than 2^8 (so most blocks skip the rescale).
// Masks: every query row attends to kv positions in [lo[row], row] (causal) or [lo[row], S) (not
// causal); `lo` (int32 [B,S], non-decreasing along S, optional) encodes document starts and sliding
// windows, and whole kv blocks left of lo[first row] or right of the last row are skipped.
// GQA: query head h reads kv head h / (Hq / Hkv).  Writes O [B,S,Hq,D] and LSE [B,Hq,S] (natural log).
//
// Context parallelism (`ring.enabled`): K and V are the staging buffers of ring.cuh; the first `n_transfer` CTAs
// pull the rows from their owners while the others attend, and the TMA producer waits on a block's flag before it
// loads the block.
//
// Oracle: the reference's attention is softmax(QK^T / sqrt(D)) V with fp32 logits and probabilities
// cast to the compute dtype (models/components/attention.py:269-278); masks from
// models/components/masks.py:9-48.  Its vendored Blackwell comparator (other head dims, no backward, no
// document mask) is third_party/ThunderKittens/kernels/attention/bf16_b300_mha_causal/bf16_b300_mha_causal.cu.
#include "b200.cuh"
#include "host_util.cuh"
#include "ring.cuh"

using namespace b200;

namespace {

constexpr int NT = 2;          // query tiles per CTA
constexpr int TILE_M = 128;    // query rows per tile
constexpr int BLOCK_N = 128;   // kv rows per block
constexpr int KV_SLOTS = 3;
constexpr int NUM_THREADS = 32 * (2 + 4 * NT);
constexpr float kRescaleThreshold = 8.0f;  // log2 units

template <int D>
struct FwdSmem {
  static constexpr int TILE_D_BYTES = 128 * D * 2;    // Q tile, K block, V block
  static constexpr int P_BYTES = TILE_M * BLOCK_N * 2;
  static constexpr int Q_OFF = 0;
  static constexpr int P_OFF = Q_OFF + NT * TILE_D_BYTES;
  static constexpr int KV_OFF = P_OFF + NT * P_BYTES;
  static constexpr int BAR_OFF = KV_OFF + KV_SLOTS * TILE_D_BYTES;
  static constexpr int TOTAL = BAR_OFF + 256;
};

struct FwdParams {
  int B, S, Skv, q_off, Hq, Hkv;  // S = query rows; Skv = kv rows; q_off = global position of query row 0
  int causal;
  float scale_log2;  // softmax scale * log2(e)
  const int* lo;     // [B, S] or nullptr
  float* lse;        // [B, Hq, S]
  int* status;
  b200ring::RingArgs ring;
};

template <int D>
__global__ void __launch_bounds__(NUM_THREADS, 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmO, const FwdParams p) {
  using L = FwdSmem<D>;
  constexpr int NBOX = D / 64;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* q_full = reinterpret_cast<uint64_t*>(smem + L::BAR_OFF);
  uint64_t* kv_full = q_full + 1;
  uint64_t* kv_empty = kv_full + KV_SLOTS;
  uint64_t* s_full = kv_empty + KV_SLOTS;
  uint64_t* p_ready = s_full + NT;
  uint64_t* pv_done = p_ready + NT;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(pv_done + NT);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const AbortCtx ab{abort_flag, p.status};

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  // context parallelism: the first CTAs of the grid stage K/V instead of attending
  const int n_xfer = p.ring.enabled ? p.ring.n_transfer : 0;
  const bool is_xfer = (int)blockIdx.x < n_xfer;
  const int cta = is_xfer ? 0 : (int)blockIdx.x - n_xfer;
  // heavy (late) query tiles first: causal work grows with the tile index
  const int q_tiles = (p.S + NT * TILE_M - 1) / (NT * TILE_M);
  // ... over the whole grid (all heads of the longest tile, then the next), which balances the tail
  const int nbh = p.B * p.Hq;
  const int qt = q_tiles - 1 - (cta / nbh);
  const int bh = cta % nbh;
  const int h = bh % p.Hq;
  const int b = bh / p.Hq;
  const int hkv = h / (p.Hq / p.Hkv);
  const int q0 = qt * NT * TILE_M;

  // kv block range of this CTA (kv positions are global; query row r sits at global position q_off + r)
  int kv_begin = 0;
  if (p.lo) kv_begin = p.lo[(long long)b * p.S + q0] / BLOCK_N;
  int kv_end = (p.Skv + BLOCK_N - 1) / BLOCK_N;
  if (p.causal) kv_end = min(kv_end, (p.q_off + min(q0 + NT * TILE_M, p.S) - 1) / BLOCK_N + 1);
  const int n_blocks = is_xfer ? 0 : max(kv_end - kv_begin, 0);

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < KV_SLOTS; ++s) {
      mbar_init(&kv_full[s], 1);
      mbar_init(&kv_empty[s], 1);
    }
    for (int t = 0; t < NT; ++t) {
      mbar_init(&s_full[t], 1);
      mbar_init(&p_ready[t], 4);
      mbar_init(&pv_done[t], 1);
    }
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
  const uint32_t tmem_S = tmem_base;              // NT * 128 columns
  const uint32_t tmem_O = tmem_base + NT * 128;   // NT * D columns

  if (is_xfer) {
    // ---------------------------------------------------------------- K/V transfer (context parallelism)
    // buffers and barriers of the copy pipelines sit in front of this kernel's own barriers (L::BAR_OFF)
    b200ring::transfer_cta<b200ring::pipes_for_window(L::BAR_OFF)>(p.ring, smem, ab);
  } else if (warp == 0) {
    // ---------------------------------------------------------------- TMA producer
    if (lane == 0 && n_blocks > 0) {
      tma_prefetch_desc(&tmQ);
      tma_prefetch_desc(&tmK);
      tma_prefetch_desc(&tmV);
      mbar_expect_tx(q_full, NT * L::TILE_D_BYTES);
      for (int t = 0; t < NT; ++t)
        for (int bx = 0; bx < NBOX; ++bx)
          tma_load_4d(smem + L::Q_OFF + t * L::TILE_D_BYTES + bx * 16384, &tmQ, q_full, bx * 64, h, q0 + t * TILE_M, b);
      // item order: K0, then for each block j: K(j+1) if it exists, V(j)
      uint32_t item = 0;
      bool ok = true;
      auto load_block = [&](const CUtensorMap* tm, int j) {
        const int slot = item % KV_SLOTS;
        const uint32_t ph = (item / KV_SLOTS) & 1;
        if (!mbar_wait(&kv_empty[slot], ph ^ 1, ab, ERR_WAIT_EMPTY)) { ok = false; return; }
        if (p.ring.enabled && !b200ring::wait_block(p.ring, b, kv_begin + j, p.status)) {
          *ab.flag = 1;   // the block never arrived: the other roles of this CTA stop waiting too
          ok = false;
          return;
        }
        mbar_expect_tx(&kv_full[slot], L::TILE_D_BYTES);
        for (int bx = 0; bx < NBOX; ++bx)
          tma_load_4d(smem + L::KV_OFF + slot * L::TILE_D_BYTES + bx * 16384, tm, &kv_full[slot], bx * 64, hkv,
                      (kv_begin + j) * BLOCK_N, b);
        ++item;
      };
      load_block(&tmK, 0);
      for (int j = 0; j < n_blocks && ok; ++j) {
        if (j + 1 < n_blocks) load_block(&tmK, j + 1);
        if (ok) load_block(&tmV, j);
      }
      if (!ok) {
        const uint64_t t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer
    if (lane == 0 && n_blocks > 0) {
      constexpr uint32_t idesc_qk = make_idesc_bf16(TILE_M, BLOCK_N, false, false);
      constexpr uint32_t idesc_pv = make_idesc_bf16(TILE_M, D, false, true);
      bool ok = mbar_wait(q_full, 0, ab, ERR_WAIT_FULL);
      uint32_t item = 0;
      // Shared-memory descriptors are built once per operand; the slice of one MMA instruction is that descriptor
      // plus a compile-time constant in its address field (units of 16 bytes).  A tile product is D / 16 (or
      // BLOCK_N / 16) instructions of 64 clocks each and one thread issues them all, so next to nothing may sit
      // between two of them.
      uint64_t dq[NT], dp[NT], dk[KV_SLOTS], dv[KV_SLOTS];
#pragma unroll
      for (int t = 0; t < NT; ++t) {
        dq[t] = make_smem_desc_sw128(smem_u32(smem + L::Q_OFF + t * L::TILE_D_BYTES), 16, 1024);
        dp[t] = make_smem_desc_sw128(smem_u32(smem + L::P_OFF + t * L::P_BYTES), 16, 1024);
      }
#pragma unroll
      for (int sl = 0; sl < KV_SLOTS; ++sl) {
        const uint32_t kv_base = smem_u32(smem + L::KV_OFF + sl * L::TILE_D_BYTES);
        dk[sl] = make_smem_desc_sw128(kv_base, 16, 1024);
        dv[sl] = make_smem_desc_sw128(kv_base, 16384, 1024);
      }
      static_assert(KV_SLOTS == 3 && NT == 2, "slot and tile selects below are written out");
      auto issue_qk = [&](int t, int slot) {
        const uint64_t a0 = t == 0 ? dq[0] : dq[1], b0 = slot == 0 ? dk[0] : (slot == 1 ? dk[1] : dk[2]);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint64_t off = (uint64_t)(((kk >> 2) * 16384 + (kk & 3) * 32) >> 4);
          tc_mma_ss(tmem_S + t * 128, a0 + off, b0 + off, idesc_qk, kk != 0 ? 1u : 0u);
        }
        tc_commit(&s_full[t]);
      };
      auto issue_pv = [&](int t, int slot, bool accumulate) {
        const uint64_t a0 = t == 0 ? dp[0] : dp[1], b0 = slot == 0 ? dv[0] : (slot == 1 ? dv[1] : dv[2]);
#pragma unroll
        for (int kk = 0; kk < BLOCK_N / 16; ++kk) {
          const uint64_t a_off = (uint64_t)(((kk >> 2) * 16384 + (kk & 3) * 32) >> 4);
          const uint64_t b_off = (uint64_t)((kk * 2048) >> 4);
          tc_mma_ss(tmem_O + t * D, a0 + a_off, b0 + b_off, idesc_pv, (accumulate || kk != 0) ? 1u : 0u);
        }
        tc_commit(&pv_done[t]);
      };
      if (ok) {
        const int slot = item % KV_SLOTS;
        ok = mbar_wait(&kv_full[slot], (item / KV_SLOTS) & 1, ab, ERR_WAIT_FULL);
        if (ok) {
          tc_fence_after();
          for (int t = 0; t < NT; ++t) issue_qk(t, slot);
          tc_commit(&kv_empty[slot]);
          ++item;
        }
      }
      for (int j = 0; j < n_blocks && ok; ++j) {
        const bool has_next = j + 1 < n_blocks;
        const uint32_t k_item = item;
        const uint32_t v_item = item + (has_next ? 1 : 0);
        const int k_slot = k_item % KV_SLOTS, v_slot = v_item % KV_SLOTS;
        for (int t = 0; t < NT && ok; ++t) {
          if (!mbar_wait(&p_ready[t], j & 1, ab, ERR_WAIT_P_READY)) { ok = false; break; }
          tc_fence_after();
          if (has_next) {
            if (t == 0 && !mbar_wait(&kv_full[k_slot], (k_item / KV_SLOTS) & 1, ab, ERR_WAIT_FULL)) { ok = false; break; }
            tc_fence_after();
            issue_qk(t, k_slot);
            if (t == NT - 1) tc_commit(&kv_empty[k_slot]);
          }
          if (t == 0 && !mbar_wait(&kv_full[v_slot], (v_item / KV_SLOTS) & 1, ab, ERR_WAIT_FULL)) { ok = false; break; }
          tc_fence_after();
          issue_pv(t, v_slot, j > 0);
          if (t == NT - 1) tc_commit(&kv_empty[v_slot]);
        }
        item = v_item + 1;
      }
    }
  } else {
    // ---------------------------------------------------------------- softmax / correction / epilogue
    const int t = (warp - 2) >> 2;
    const int quad = warp & 3;
    const int row = quad * 32 + lane;
    const int q_row = q0 + t * TILE_M + row;       // local row (indexes lo / lse / O)
    const int q_pos = p.q_off + q_row;             // global position (compared with kv positions)
    const uint32_t lane_sel = static_cast<uint32_t>(quad * 32) << 16;
    const uint32_t tS = tmem_S + t * 128 + lane_sel;
    const uint32_t tO = tmem_O + t * D + lane_sel;
    uint8_t* sP = smem + L::P_OFF + t * L::P_BYTES;
    int lo_row = 0;
    if (p.lo) lo_row = p.lo[(long long)b * p.S + min(q_row, p.S - 1)];
    float m_ref = -1.0e30f;
    float l_sum = 0.f;
    bool ok = n_blocks > 0;
    for (int j = 0; j < n_blocks && ok; ++j) {
      const int kv0 = (kv_begin + j) * BLOCK_N;
      if (!mbar_wait_warp(&s_full[t], j & 1, ab, ERR_WAIT_S_READY)) { ok = false; break; }
      tc_fence_after();
      const bool need_mask = (p.causal && kv0 + BLOCK_N - 1 > q_pos) || (kv0 < lo_row) || (kv0 + BLOCK_N > p.Skv);
      const int hi = p.causal ? min(q_pos, p.Skv - 1) : p.Skv - 1;
      float sum = 0.f;
      // exponentials of 32 scores relative to m_ref, their sum, and P (bf16, 128-byte swizzle, K-major for the PV
      // MMA) into shared memory; returns the largest exponent argument seen (how far the row maximum moved)
      auto emit_chunk = [&](const uint32_t (&r)[32], int c) -> float {
        float e[32];
        float top = -INFINITY;
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          float v = __uint_as_float(r[i]) * p.scale_log2 - m_ref;
          if (need_mask) {
            const int col = kv0 + c * 32 + i;
            if (col > hi || col < lo_row) v = -INFINITY;
          }
          top = fmaxf(top, v);
          e[i] = ex2_approx(v);
          sum += e[i];
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          uint4 v;
          v.x = pack_bf16x2(e[8 * i + 0], e[8 * i + 1]);
          v.y = pack_bf16x2(e[8 * i + 2], e[8 * i + 3]);
          v.z = pack_bf16x2(e[8 * i + 4], e[8 * i + 5]);
          v.w = pack_bf16x2(e[8 * i + 6], e[8 * i + 7]);
          const int chunk = c * 4 + i;  // 16-byte chunk index along kv (16 per row)
          *reinterpret_cast<uint4*>(sP + (chunk >> 3) * 16384 + sw128_offset(row, chunk & 7)) = v;
        }
        return top;
      };
      // Fast path (every block but the first, unless a row maximum jumps): ONE pass over the scores with the
      // reference maximum of the previous blocks.  The lazy-rescale rule tolerates a maximum that is up to 2^8
      // above the reference, so the pass is kept when no row of the warp moved further; the loads of one chunk
      // are in flight while the previous chunk is worked on.
      bool done = false;
      if (j > 0) {
        if (!mbar_wait_warp(&pv_done[t], (j - 1) & 1, ab, ERR_WAIT_O_READY)) { ok = false; break; }   // P(j-1) consumed
        // all 128 scores of the row at once: the latency of the tensor-memory loads is paid once per block
        uint32_t ra[32], rb[32], rc[32], rd[32];
        tmem_ld_32x32b_x32(tS, ra);
        tmem_ld_32x32b_x32(tS + 32, rb);
        tmem_ld_32x32b_x32(tS + 64, rc);
        tmem_ld_32x32b_x32(tS + 96, rd);
        tmem_ld_wait();
        float top = emit_chunk(ra, 0);
        top = fmaxf(top, emit_chunk(rb, 1));
        top = fmaxf(top, emit_chunk(rc, 2));
        top = fmaxf(top, emit_chunk(rd, 3));
        done = !__any_sync(0xffffffffu, top > kRescaleThreshold);
        if (!done) sum = 0.f;   // a row maximum moved too far: redo the block with a new reference
      }
      if (!done) {
        // pass 1: block maximum of the scaled, masked scores
        float bm = -INFINITY;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t r[32];
          tmem_ld_32x32b_x32(tS + c * 32, r);
          tmem_ld_wait();
          if (need_mask) {
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              const int col = kv0 + c * 32 + i;
              const float v = (col > hi || col < lo_row) ? -INFINITY : __uint_as_float(r[i]);
              bm = fmaxf(bm, v);
            }
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) bm = fmaxf(bm, __uint_as_float(r[i]));
          }
        }
        bm *= p.scale_log2;  // scale > 0, so the maximum commutes with it
        const bool need = bm > m_ref + kRescaleThreshold;
        if (__any_sync(0xffffffffu, need)) {
          const float m_new = need ? bm : m_ref;
          const float alpha = ex2_approx(m_ref - m_new);
          if (j > 0) {
            // pv_done(j-1) was waited for above: O holds the sum over the blocks before this one
            tc_fence_after();
#pragma unroll
            for (int c = 0; c < D / 32; ++c) {
              uint32_t r[32];
              tmem_ld_32x32b_x32(tO + c * 32, r);
              tmem_ld_wait();
#pragma unroll
              for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
              tmem_st_32x32b_x32(tO + c * 32, r);
            }
            tmem_st_wait();
          }
          l_sum *= alpha;
          m_ref = m_new;
        }
        // pass 2: probabilities, row sum, P to shared memory
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t r[32];
          tmem_ld_32x32b_x32(tS + c * 32, r);
          tmem_ld_wait();
          emit_chunk(r, c);
        }
      }
      l_sum += sum;
      fence_proxy_async_smem();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_ready[t]);
    }
    if (ok) ok = mbar_wait_warp(&pv_done[t], (n_blocks - 1) & 1, ab, ERR_WAIT_O_READY);
    if (ok) {
      tc_fence_after();
      const float inv_l = l_sum > 0.f ? 1.f / l_sum : 0.f;
#pragma unroll
      for (int c = 0; c < D / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(tO + c * 32, r);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          uint4 v;
          v.x = pack_bf16x2(__uint_as_float(r[8 * i + 0]) * inv_l, __uint_as_float(r[8 * i + 1]) * inv_l);
          v.y = pack_bf16x2(__uint_as_float(r[8 * i + 2]) * inv_l, __uint_as_float(r[8 * i + 3]) * inv_l);
          v.z = pack_bf16x2(__uint_as_float(r[8 * i + 4]) * inv_l, __uint_as_float(r[8 * i + 5]) * inv_l);
          v.w = pack_bf16x2(__uint_as_float(r[8 * i + 6]) * inv_l, __uint_as_float(r[8 * i + 7]) * inv_l);
          *reinterpret_cast<uint4*>(sP + (c >> 1) * 16384 + sw128_offset(row, (c & 1) * 4 + i)) = v;
        }
      }
      fence_proxy_async_smem();
      __syncwarp();
      const int slab_row = q0 + t * TILE_M + quad * 32;
      if (lane == 0 && slab_row < p.S) {
        for (int bx = 0; bx < NBOX; ++bx)
          tma_store_4d(&tmO, sP + bx * 16384 + quad * 32 * 128, bx * 64, h, slab_row, b);
        tma_commit_group();
        tma_wait_group<0>();
      }
      if (q_row < p.S)
        p.lse[((long long)b * p.Hq + h) * p.S + q_row] =
            l_sum > 0.f ? m_ref * 0.6931471805599453f + logf(l_sum) : -INFINITY;
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

template <int D>
int launch_fwd(const CUtensorMap& tmQ, const CUtensorMap& tmK, const CUtensorMap& tmV, const CUtensorMap& tmO,
               const FwdParams& p, cudaStream_t stream) {
  using L = FwdSmem<D>;
  auto* kern = attn_fwd_kernel<D>;
  constexpr int smem_bytes = L::TOTAL + 1024;
  static bool configured[b200host::kMaxDevices] = {};   // per kernel instantiation and device
  if (int rc = b200host::ensure_dynamic_smem(kern, smem_bytes, configured)) return rc;
  const int q_tiles = (p.S + NT * TILE_M - 1) / (NT * TILE_M);
  const int grid = q_tiles * p.Hq * p.B + (p.ring.enabled ? p.ring.n_transfer : 0);
  kern<<<grid, NUM_THREADS, smem_bytes, stream>>>(tmQ, tmK, tmV, tmO, p);
  return static_cast<int>(cudaGetLastError());
}

}  // namespace

// q: [B,S,Hq,D] view with element strides (q_row = between tokens, q_batch = between batches; heads are D
// apart); k, v: [B,Skv,Hkv,D] likewise; o: [B,S,Hq,D]; lse: [B,Hq,S] fp32; lo: [B,S] int32 or null.
// skv_and_qoff packs the kv length and the global position of query row 0 for context-parallel callers
// (0 = same length as the queries, offset 0): low 32 bits Skv, high 32 bits q_off (a multiple of 128).
static int attn_fwd_impl(const void* q, const void* k, const void* v, void* o, void* lse, const void* lo, int B, int S,
                         int Hq, int Hkv, int D, long long q_row, long long q_batch, long long k_row,
                         long long k_batch, long long v_row, long long v_batch, long long o_row, long long o_batch,
                         float scale, int causal, long long skv_and_qoff, const b200ring::RingHostArgs* ring,
                         int* status, void* stream) {
  using namespace b200host;
  const int Skv = (skv_and_qoff & 0xffffffffLL) ? (int)(skv_and_qoff & 0xffffffffLL) : S;
  const int q_off = (int)(skv_and_qoff >> 32);
  if (q_off % 128 != 0 || q_off < 0) return RC_BAD_SHAPE;
  if (B <= 0 || S <= 0 || Hq <= 0 || Hkv <= 0 || Hq % Hkv) return RC_BAD_SHAPE;
  if (D != 128 && D != 64) return RC_BAD_SHAPE;
  const CUtensorMapDataType bf = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  CUtensorMap tmQ, tmK, tmV, tmO;
  int rc;
  if ((rc = make_map_4d(&tmQ, bf, q, D, Hq, S, B, (uint64_t)D * 2, q_row * 2, q_batch * 2, 64, 1, 128))) return rc;
  if ((rc = make_map_4d(&tmK, bf, k, D, Hkv, Skv, B, (uint64_t)D * 2, k_row * 2, k_batch * 2, 64, 1, 128))) return rc;
  if ((rc = make_map_4d(&tmV, bf, v, D, Hkv, Skv, B, (uint64_t)D * 2, v_row * 2, v_batch * 2, 64, 1, 128))) return rc;
  if ((rc = make_map_4d(&tmO, bf, o, D, Hq, S, B, (uint64_t)D * 2, o_row * 2, o_batch * 2, 64, 1, 32))) return rc;
  FwdParams p{B, S, Skv, q_off, Hq, Hkv, causal, scale * 1.4426950408889634f, (const int*)lo, (float*)lse, status};
  if (ring) {
    // K and V are the staging buffers: dense [B, seq_len, Hkv, D], filled by this launch's transfer CTAs
    if (k_row != (long long)Hkv * D || v_row != k_row || k_batch != (long long)ring->seq_len * k_row ||
        v_batch != k_batch || Skv > ring->seq_len)
      return RC_BAD_SHAPE;
    if ((rc = b200ring::fill_ring_args(p.ring, *ring, const_cast<void*>(k), const_cast<void*>(v), B, Hkv, D))) return rc;
  }
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (D == 128) return launch_fwd<128>(tmQ, tmK, tmV, tmO, p, s);
  return launch_fwd<64>(tmQ, tmK, tmV, tmO, p, s);
}

extern "C" int b200_attn_fwd(const void* q, const void* k, const void* v, void* o, void* lse, const void* lo, int B,
                             int S, int Hq, int Hkv, int D, long long q_row, long long q_batch, long long k_row,
                             long long k_batch, long long v_row, long long v_batch, long long o_row,
                             long long o_batch, float scale, int causal, long long skv_and_qoff, int* status,
                             void* stream) {
  return attn_fwd_impl(q, k, v, o, lse, lo, B, S, Hq, Hkv, D, q_row, q_batch, k_row, k_batch, v_row, v_batch, o_row,
                       o_batch, scale, causal, skv_and_qoff, nullptr, status, stream);
}

// The same with the K/V exchange of context parallelism inside the launch (ring.cuh): k, v are this rank's
// staging buffers [B, seq_len, Hkv, D]; `ring` says which blocks to pull from which rank's buffer.
extern "C" int b200_attn_fwd_ring(const void* q, const void* k, const void* v, void* o, void* lse, const void* lo,
                                  int B, int S, int Hq, int Hkv, int D, long long q_row, long long q_batch,
                                  long long k_row, long long k_batch, long long v_row, long long v_batch,
                                  long long o_row, long long o_batch, float scale, int causal,
                                  long long skv_and_qoff, const void* ring, int* status, void* stream) {
  if (!ring) return b200host::RC_BAD_SHAPE;
  return attn_fwd_impl(q, k, v, o, lse, lo, B, S, Hq, Hkv, D, q_row, q_batch, k_row, k_batch, v_row, v_batch, o_row,
                       o_batch, scale, causal, skv_and_qoff, static_cast<const b200ring::RingHostArgs*>(ring), status,
                       stream);
}
