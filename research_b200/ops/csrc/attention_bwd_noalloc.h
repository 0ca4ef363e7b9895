// Allocation-free entry point for the flash-attention backward pass.
//
// This declaration has no counterpart in the reference project: it exists for hosts that embed this
// library but are not allowed to allocate device memory themselves - for example a serving or training
// process whose memory was carved up front by a pool it does not own, a code path that runs while a
// stream is being recorded, or a plug-in loaded into a runtime that forbids cudaMalloc from callbacks.
//
// b200_attn_bwd needs one piece of scratch besides its inputs and outputs: delta[b, h, s] =
// sum_d dO * O, fp32, B * Hq * S values.  b200_attn_bwd_noalloc keeps that scratch in a fixed array that
// lives inside the library image on every GPU that loads it (B200_ATTN_NOALLOC_MAX_ROWS floats = 4 MiB,
// held until the process exits) and calls neither cudaMalloc / cudaFree nor any allocating library routine.
//
// Rules for callers:
//   * B * Hq * S must not exceed B200_ATTN_NOALLOC_MAX_ROWS; larger problems are rejected with
//     B200_ATTN_NOALLOC_TOO_LARGE (and a line on stderr) before anything is launched.
//   * The first call on each device looks up the array's device address (cudaGetSymbolAddress with that device
//     current) and caches it.  Make that first call outside of any stream capture, and do not let two threads
//     make the first call for the same device at the same time (the cache slot is written without a lock; both
//     would write the same value, but nothing orders the writes).
//   * All calls on one device share the one array.  The array keeps whatever the last call left in it; every
//     call overwrites the part it uses before reading it, so nothing has to be cleared - but two calls
//     that overlap in time on the same GPU (different streams, different threads) race on it.  Serialise them.
//   * Inputs, outputs and their strides are exactly those of b200_attn_bwd, minus the delta pointer.
#pragma once

#ifdef __cplusplus
extern "C" {
#endif

#define B200_ATTN_NOALLOC_MAX_ROWS (1 << 20)
#define B200_ATTN_NOALLOC_TOO_LARGE (-5)
#define B200_ATTN_NOALLOC_SYMBOL_FAILED (-6)

int b200_attn_bwd_noalloc(const void* q, const void* k, const void* v, const void* o, const void* d_o,
                          const void* lse, void* dq, void* dk, void* dv, const void* lo, const void* hi, int B,
                          int S, int Hq, int Hkv, int D, long long q_row, long long q_batch, long long k_row,
                          long long k_batch, long long v_row, long long v_batch, long long o_row, long long o_batch,
                          long long do_row, long long do_batch, long long dq_row, long long dq_batch,
                          long long dk_row, long long dk_batch, long long dv_row, long long dv_batch, float scale,
                          int causal, int* status, void* stream);

#ifdef __cplusplus
}
#endif
