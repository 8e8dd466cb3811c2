// An all-reduce entry point that never allocates.  It has no counterpart in the
// reference; it exists for callers that are not in a position to ask CUDA for
// memory at the moment they need a collective:
//   * a serving process whose framework took (nearly) all device memory for its own
//     pool at start-up, so that a later cudaMalloc of ring or staging space fails;
//   * a latency-critical step that must not run into the device-wide synchronisation
//     an allocation or a free implies.
// Such a caller cannot build a communicator (that allocates a heap per rank), but it
// can call this function: the scratch the kernel needs - barrier pads, an abort word,
// a status record and the staging area the ranks exchange data through - lives in a
// fixed array inside the library's device image.
//
// What it computes: the sum over `world` rank buffers that all live on the CURRENT
// device (the single-GPU emulation of a world: one cooperative launch whose block rows
// are the ranks), with the large-message peer-load/peer-store kernel.  outs[r] receives
// the sum for every r; ins[r] == outs[r] is allowed.
//
// Limits and rules
//   * world is 2, 4 or 8; nelems <= B200IPC_NOALLOC_MAX_ELEMS 16-bit elements per rank.
//     Larger requests are refused with return code 2 and a message on stderr.
//   * The array costs B200IPC_NOALLOC_SCRATCH_BYTES of device memory on every GPU that
//     loads the library, from load until the process exits.
//   * The first call on a device looks up the array's device address (a one-time,
//     per-device set-up inside this function).  Make that first call at start-up,
//     before any stream capture is begun on that device.
//   * All calls share the one array.  Every call re-clears the words that must start at
//     zero (stream-ordered, before its kernel), and the staging area simply keeps what
//     the previous call left.  Two calls that can overlap on the GPU (different streams
//     without an ordering between them) race on it: order them.
//   * Work is enqueued on `stream`; nothing is synchronised.  No cudaMalloc, cudaFree or
//     allocating library routine is called.
//
// dtype: 0 = fp16, 1 = bf16.  status_host may be null; otherwise 8 words are copied to it
// (stream-ordered, after the kernel): {code, rank, peer, cta, step, expected, seen, site},
// code 0 = fine, 1 = a bounded device-side wait ran out (2 s, or B200IPC_TIMEOUT_US microseconds when that
// environment variable is set), 2 = a rank stopped because another one had given up.  All emulated ranks
// share this one record.  A return value of 0 together with a non-zero code means that the kernel ended
// early: the contents of outs are then undefined.
//
// Returns 0 on success, 1 for a bad argument, 2 when nelems exceeds the maximum,
// 100 + cudaError_t when a CUDA call failed.
#pragma once

#include <stddef.h>
#include <stdint.h>

#define B200IPC_NOALLOC_MAX_ELEMS (256 * 1024)
#define B200IPC_NOALLOC_MAX_WORLD 8
#define B200IPC_NOALLOC_RANK_STRIDE (8192 + 2 * B200IPC_NOALLOC_MAX_ELEMS + 4096)
#define B200IPC_NOALLOC_SCRATCH_BYTES (B200IPC_NOALLOC_MAX_WORLD * B200IPC_NOALLOC_RANK_STRIDE)

#ifdef __cplusplus
extern "C" {
#endif

int b200ipc_allreduce_noalloc(const void* const* ins, void* const* outs, int world, size_t nelems, int dtype,
                              void* stream, uint32_t* status_host);

#ifdef __cplusplus
}
#endif
