// An entry point for callers that must not allocate device memory.
//
// This has no counterpart in jiamumuzhao/vllm-cpp; it exists for users of this
// library only.
//
// Who needs it.  Some programs that want split-KV decode attention cannot call
// cudaMalloc at the moment they need the kernel, or at all: code that runs inside
// a latency-critical serving loop where an allocation's implicit device
// synchronisation is not acceptable; a process whose device memory has been handed
// out in full to a pool it does not own; a plug-in loaded into a host application
// that forbids allocations from foreign code.  The ordinary entry point,
// vcb_attention_decode_mma, leaves the allocation of the merge scratch (partial
// outputs of the context splits) to its caller, which comes to the same problem.
//
// What it does.  vcb_attention_decode_mma_static runs the same kernels on the same
// inputs and outputs, but merges the splits through a fixed array that lives in the
// library's own device data segment.  It calls no cudaMalloc, no cudaFree and no
// library routine that allocates.
//
// The limit.  The array holds VCB_STATIC_SCRATCH_ROWS partial rows of up to
// VCB_STATIC_SCRATCH_DIM floats plus two statistics each, and one ticket counter per
// row (about 4.3 MB in all).  Every GPU
// on which the library is loaded carries it until the process exits.  A call needs
// n_list * nh * nsplit rows when nsplit > 1 (none when nsplit == 1); a call that
// needs more rows, or a head size above VCB_STATIC_SCRATCH_DIM, is refused with
// VCB_ERR_SCRATCH_TOO_SMALL and launches nothing.
//
// First call.  The first call on a device looks up the array's device address
// (cudaGetSymbolAddress, with that device current) and keeps it; make that first
// call before any stream capture begins.
//
// Sharing.  All calls on a device use the one array, and it keeps what the last call
// left in it.  The partial results need no clearing: every slot that the merge reads is
// written earlier in the same call.  The tickets by which the splits of a (request,
// kv head) find out who merges must start at zero; the entry point clears them on the
// caller's stream before each launch.  Two calls that overlap on the GPU (different
// streams) race on the array; run them on one stream or order them yourself.
//
// When the kernel cannot finish.  Every wait inside the kernel is bounded, and every page number it
// reads from a block table is checked against num_pages.  A wait that runs out ends the CTA's loop
// early; a page number outside [0, num_pages) is read as page 0.  Either way the call itself still
// returns 0 (it only launches) and `out` is wrong.  The kernel notes what happened in a word beside
// the array: vcb_attention_decode_mma_static_status waits for the device, hands the note back (0:
// nothing happened; 5: a wait for a cache tile ran out; 11: a page number outside the cache) and
// clears it.  Call it whenever a wrong result would matter, e.g. once every few hundred steps; it
// allocates nothing either.
#pragma once

#ifdef __cplusplus
extern "C" {
#endif

#define VCB_STATIC_SCRATCH_ROWS 8192
#define VCB_STATIC_SCRATCH_DIM 128
#define VCB_ERR_SCRATCH_TOO_SMALL 10003

// Arguments as vcb_attention_decode_mma, without the two scratch pointers:
//   q, out: [n_tokens, nh * d] bfloat16; cache: [pages][2][nkv][page][d] bfloat16;
//   q_start [n_reqs + 1], ctx_lens [n_reqs], block_table [n_reqs, bt_stride]: int32 on the device;
//   req_list: n_list request indices on the device, or null for 0..n_list-1;
//   nsplit: context splits per (request, kv head); page: slots per page, a multiple of 8;
//   num_pages: pages the cache holds; stream: a cudaStream_t.
// Returns 0, a cudaError_t value, or one of the VCB_ERR_* codes (10001 bad argument, 10002 a head
// size other than 64 or 128 or a page size that is no multiple of 8; nothing is launched then).
int vcb_attention_decode_mma_static(const void* q, const void* cache, void* out, const int* q_start,
                                    const int* ctx_lens, const int* block_table, int bt_stride,
                                    const int* req_list, int n_list, int nsplit, int nh, int nkv, int d,
                                    int page, int window, float scale, int num_pages, void* stream);

// *code = what the kernel noted since the last call of this function (see above); synchronises with the
// device.  Returns 0 or a cudaError_t value.
int vcb_attention_decode_mma_static_status(int* code);

#ifdef __cplusplus
}
#endif
