// K/V exchange of context-parallel attention, done from inside the attention kernels.
//
// Every rank of the context group keeps its own K and V rows (local order) in a buffer of a symmetric arena.
// The first CTAs of an attention launch do no attention: they pull the K/V rows this rank's queries can see
// from the owners' buffers over NVLink (untiled bulk copies through shared memory, several pipelines per CTA,
// no multicast) into one local staging buffer in sequence order, and publish one flag per 128-row block.  The
// attention CTAs of the SAME launch load K/V blocks from the staging buffer with TMA and wait (bounded) on the
// block's flag before the first load, so attention on the blocks that have landed overlaps the transfer of the
// rest; nothing is gathered ahead of the kernel and only one staging buffer exists, whatever the layer count.
// In the backward pass the dK/dV kernel adds its tiles straight into the owners' gradient buffers with TMA
// reduce-adds (attention_bwd.cu).
//
// Cross-GPU protocol (flag blocks of comm.cuh): CTA 0 announces "my K/V for epoch e are in place"; a pipeline
// waits for the owner's announcement before its first read from that owner; the pipeline that finishes last
// tells every peer "done reading" and waits until every peer is done reading this rank's buffer, so the buffer
// may be rewritten as soon as the launch has ended.  Every wait is bounded and reports through the status word.
//
// Counterpart in the reference: third_party/ThunderKittens/kernels/parallel/ring_attn/ring_attn_h100.cu:77-215
// (communication CTAs forward K/V blocks to the next device while attention CTAs compute; unbounded waits).
#pragma once
#include "b200.cuh"
#include "comm.cuh"

namespace b200ring {

using namespace b200;
using namespace b200comm;

constexpr int kMaxPipes = 4;         // copy pipelines per transfer CTA at most, one elected thread each
constexpr int kBufs = 3;             // shared-memory buffers per pipeline
constexpr int kLag = 1;              // a chunk is stored kLag iterations after its load was issued
constexpr int kChunkBytes = 16384;   // bytes per bulk copy
constexpr int kPipeBytes = kBufs * kChunkBytes;

// Pipelines that fit into the first `window_bytes` of a kernel's dynamic shared memory (the part in front of the
// kernel's own barriers), leaving room for the pipelines' mbarriers behind the buffers.  The attention kernels
// size their window by head dimension, so head dimension 64 gets fewer pipelines than 128.
constexpr int pipes_for_window(int window_bytes) {
  const int fit = (window_bytes - kMaxPipes * kBufs * 8) / kPipeBytes;
  return fit > kMaxPipes ? kMaxPipes : fit;
}
constexpr int kMaxSegments = 16;     // 2 * kMaxPeers sequence segments (zig-zag split)

struct RingArgs {
  int enabled;             // 0: plain attention, everything below is ignored
  int world, rank;
  int n_transfer;          // leading CTAs of the grid that stage K/V (0: this launch finds everything staged)
  int n_units;             // 128-row blocks to stage in this launch
  int blocks_per_batch;    // sequence length / 128
  unsigned epoch;
  int row_bytes;           // Hkv * D * 2: one token of K (or V)
  long long src_batch_bytes;   // bytes between batches in the owners' buffers
  long long dst_batch_bytes;   // bytes between batches in the staging buffers
  const int4* units;       // {owner, first row in the owner's buffer, block index in the sequence, batch}
  const uint8_t* peer_k[kMaxPeers];
  const uint8_t* peer_v[kMaxPeers];
  uint8_t* stage_k;
  uint8_t* stage_v;
  uint32_t* block_flags;   // [batch][blocks_per_batch]: epoch at which the block was staged
  FlagBlock* flags[kMaxPeers];
  uint32_t* counter;       // zero on entry, left zero
  // backward only: where a 128-row block of the sequence lives at its owner
  int seg_rows;            // rows per sequence segment
  int seg_owner[kMaxSegments];
  int seg_first_row[kMaxSegments];   // first row of the segment in its owner's buffer
};

// Attention CTAs: K/V rows of sequence block `block` of batch `batch` are in the staging buffer.
__device__ __forceinline__ bool wait_block(const RingArgs& r, int batch, int block, int* status) {
  if (!wait_gpu(&r.block_flags[(long long)batch * r.blocks_per_batch + block], r.epoch, status, ERR_LOCAL_FLAG))
    return false;
  fence_proxy_async_all();   // the flag was read through the generic proxy, the rows are read by TMA
  return true;
}

// Body of a transfer CTA.  `smem`: PIPES * kPipeBytes of 128-byte aligned shared memory followed by PIPES * kBufs
// mbarriers, all of it unused by anything else in this CTA.  Called by every thread of the CTA.
template <int PIPES>
__device__ __forceinline__ void transfer_cta(const RingArgs& r, uint8_t* smem, const AbortCtx& ab) {
  static_assert(PIPES >= 1 && PIPES <= kMaxPipes, "the shared-memory window holds no copy pipeline");
  constexpr int kPipes = PIPES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + PIPES * kPipeBytes);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (blockIdx.x == 0 && (int)threadIdx.x < r.world && (int)threadIdx.x != r.rank) {
    __threadfence_system();
    st_release_sys(&r.flags[threadIdx.x]->ready[r.rank], r.epoch);
  }
  if (lane != 0 || warp >= kPipes) return;
  uint64_t* bar = bars + warp * kBufs;
  for (int i = 0; i < kBufs; ++i) mbar_init(&bar[i], 1);
  mbar_fence_init();
  uint8_t* ring = smem + warp * kBufs * kChunkBytes;
  const int pipe = (int)blockIdx.x * kPipes + warp;
  const int n_pipes = r.n_transfer * kPipes;
  const int unit_bytes = 128 * r.row_bytes;
  const int chunks_per_half = unit_bytes / kChunkBytes;      // K, then V
  const int chunks_per_unit = 2 * chunks_per_half;
  const int my_units = r.n_units > pipe ? (r.n_units - pipe + n_pipes - 1) / n_pipes : 0;
  const long long total = (long long)my_units * chunks_per_unit;
  auto locate = [&](long long i, const uint8_t*& src, uint8_t*& dst, int& owner, int& flag_index, bool& last) {
    const int4 d = r.units[pipe + (int)(i / chunks_per_unit) * n_pipes];
    const int c = (int)(i % chunks_per_unit);
    const bool is_v = c >= chunks_per_half;
    const long long off = (long long)(is_v ? c - chunks_per_half : c) * kChunkBytes;
    owner = d.x;
    src = (is_v ? r.peer_v[d.x] : r.peer_k[d.x]) + (long long)d.w * r.src_batch_bytes + (long long)d.y * r.row_bytes + off;
    dst = (is_v ? r.stage_v : r.stage_k) + (long long)d.w * r.dst_batch_bytes + (long long)d.z * unit_bytes + off;
    flag_index = d.w * r.blocks_per_batch + d.z;
    last = c == chunks_per_unit - 1;
  };
  bool ok = true;
  uint32_t ready_mask = 1u << r.rank;
  for (long long i = 0; i < total + kLag && ok; ++i) {
    const uint8_t* src;
    uint8_t* dst;
    int owner, flag_index;
    bool last;
    if (i < total) {
      locate(i, src, dst, owner, flag_index, last);
      if (!(ready_mask >> owner & 1u)) {
        if (!wait_sys(&r.flags[r.rank]->ready[owner], r.epoch, ab.status, ERR_PEER_READY)) { ok = false; break; }
        ready_mask |= 1u << owner;
      }
      const int buf = (int)(i % kBufs);
      if (i >= kBufs) tma_wait_group_read<kBufs - kLag - 1>();   // the store that last read this buffer is done
      mbar_expect_tx(&bar[buf], kChunkBytes);
      bulk_g2s(ring + buf * kChunkBytes, src, kChunkBytes, &bar[buf]);
    }
    const long long j = i - kLag;
    if (j >= 0 && j < total) {
      locate(j, src, dst, owner, flag_index, last);
      const int buf = (int)(j % kBufs);
      if (!mbar_wait(&bar[buf], (uint32_t)(j / kBufs) & 1u, ab, ERR_WAIT_FULL)) { ok = false; break; }
      bulk_s2g(dst, ring + buf * kChunkBytes, kChunkBytes);
      tma_commit_group();
      if (last) {
        tma_wait_group<0>();          // K and V rows of the block are in memory: publish the block
        fence_proxy_async_all();
        st_release_gpu(&r.block_flags[flag_index], r.epoch);
      }
    }
  }
  tma_wait_group<0>();
  if (!ok) {   // give copies in flight the time to land before the shared memory goes away
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
  }
  // the pipeline that finishes last: this rank has finished reading its peers' buffers
  __threadfence();
  if (atomicAdd(r.counter, 1u) == (uint32_t)n_pipes - 1u) {
    *r.counter = 0u;
    for (int p = 0; p < r.world; ++p)
      if (p != r.rank) st_release_sys(&r.flags[p]->done[r.rank], r.epoch);
    for (int p = 0; p < r.world; ++p)
      if (p != r.rank) wait_sys(&r.flags[r.rank]->done[p], r.epoch, ab.status, ERR_PEER_DONE);
  }
}

// What the host passes for a context-parallel launch (mirrored by a ctypes structure on the Python side).
struct RingHostArgs {
  int world, rank;
  int n_transfer, n_units;
  int seq_len;                 // rows of the whole sequence (= rows of the staging buffers per batch)
  int local_rows;              // rows per batch in every rank's K/V buffer
  unsigned epoch;
  int seg_rows;                // rows per sequence segment
  int seg_owner[kMaxSegments];
  int seg_first_row[kMaxSegments];
  const void* units;           // device int4[n_units]
  const void* peer_k[kMaxPeers];
  const void* peer_v[kMaxPeers];
  void* block_flags;           // device uint32[B * seq_len / 128]
  void* flags[kMaxPeers];      // every rank's flag block of the channel, as mapped here
  void* counter;               // device uint32, zero
  void* peer_dk[kMaxPeers];    // backward: every rank's dK / dV accumulation buffer [B, local_rows, Hkv, D] bf16
  void* peer_dv[kMaxPeers];
};

// Validates the host arguments and fills the device-side structure.  stage_k / stage_v: [B, seq_len, Hkv, D].
inline int fill_ring_args(RingArgs& r, const RingHostArgs& h, void* stage_k, void* stage_v, int B, int Hkv, int D) {
  if (h.world < 2 || h.world > kMaxPeers || h.rank < 0 || h.rank >= h.world) return -2;
  if (h.seq_len % 128 || h.local_rows % 128 || h.seg_rows <= 0 || h.seg_rows % 128) return -2;
  if (h.seq_len / h.seg_rows > kMaxSegments) return -2;
  const int row_bytes = Hkv * D * 2;
  if ((128 * row_bytes) % kChunkBytes) return -2;
  if (h.n_transfer < 0 || h.n_units < 0 || (h.n_units > 0 && (h.n_transfer <= 0 || !h.units))) return -2;
  if (!h.block_flags || !h.counter) return -1;
  r = RingArgs{};
  r.enabled = 1;
  r.world = h.world;
  r.rank = h.rank;
  r.n_transfer = h.n_units > 0 ? h.n_transfer : 0;
  r.n_units = h.n_units;
  r.blocks_per_batch = h.seq_len / 128;
  r.epoch = h.epoch;
  r.row_bytes = row_bytes;
  r.src_batch_bytes = (long long)h.local_rows * row_bytes;
  r.dst_batch_bytes = (long long)h.seq_len * row_bytes;
  r.units = static_cast<const int4*>(h.units);
  for (int p = 0; p < h.world; ++p) {
    if (!h.flags[p]) return -1;
    if (r.n_units > 0 && (!h.peer_k[p] || !h.peer_v[p])) return -1;
    if ((reinterpret_cast<uintptr_t>(h.peer_k[p]) | reinterpret_cast<uintptr_t>(h.peer_v[p])) & 15) return -1;
    r.peer_k[p] = static_cast<const uint8_t*>(h.peer_k[p]);
    r.peer_v[p] = static_cast<const uint8_t*>(h.peer_v[p]);
    r.flags[p] = static_cast<FlagBlock*>(h.flags[p]);
  }
  if ((reinterpret_cast<uintptr_t>(stage_k) | reinterpret_cast<uintptr_t>(stage_v)) & 15) return -1;
  r.stage_k = static_cast<uint8_t*>(stage_k);
  r.stage_v = static_cast<uint8_t*>(stage_v);
  r.block_flags = static_cast<uint32_t*>(h.block_flags);
  r.counter = static_cast<uint32_t*>(h.counter);
  r.seg_rows = h.seg_rows;
  for (int s = 0; s < kMaxSegments; ++s) {
    r.seg_owner[s] = h.seg_owner[s];
    r.seg_first_row[s] = h.seg_first_row[s];
  }
  (void)B;
  return 0;
}

}  // namespace b200ring
