// lumen_attn_decode_noalloc: split-KV decode attention that allocates nothing.
//
// This entry point has no counterpart in the reference project; it is an addition of this
// library.
//
// Who it is for. Some programs that want to call this kernel cannot obtain device memory at
// the moment of the call, or ever: code that runs inside another framework's allocator
// callbacks or memory-pool bookkeeping, where a nested allocation would re-enter that
// allocator; plug-ins loaded into a host program whose memory budget is fixed at start-up and
// that must not grow it; real-time style serving loops that forbid cudaMalloc/cudaFree on the
// hot path because both can stall the whole device; and plain C or Rust callers that link this
// shared object without PyTorch and have no caching allocator to lean on. The ordinary entry
// point, lumen_attn_decode, asks its caller for two scratch buffers (the partial results of the
// segments a long sequence is cut into); this one keeps them in a fixed array that belongs to the library itself.
//
// What it does. Exactly what lumen_attn_decode does, with the same kernels: inputs and the
// output are the caller's (q, the paged K and V caches in the swizzled layout, the page table,
// each sequence's query position, out, and the int that reports a timed-out copy). The scratch
// is a file-scope `static __device__` array of LUMEN_DECODE_NOALLOC_MAX_FLOATS floats
// (16 MiB). It is part of the library's device image, so every GPU on which the library is
// loaded holds these 16 MiB from the first use of the library on that GPU until the process
// exits.
//
// Limits. max_segs is the number of 8-page segments the page table can hold, at least
// ceil(bt_stride / 8); more than 32 is never needed (a sequence of more than 256 pages is cut
// into 32 longer segments). The call needs B * nq * max_segs * (d + 2) floats. If that is more than
// the array holds, nothing is launched, a line that names the four numbers goes to stderr, and
// LUMEN_ERR_SCRATCH_TOO_SMALL is returned. (For 32 query heads of size 128: up to 126 sequences
// with page tables of 64 pages, i.e. 4,096 positions; 31 sequences with 256 pages.)
// Other return values are those of lumen_attn_decode (0 = launched, a cudaError_t, or
// LUMEN_ERR_UNSUPPORTED / LUMEN_ERR_BAD_ARGUMENT).
//
// First call on a device. The first call made while a given device is current looks up the
// array's address on that device (cudaGetSymbolAddress) and remembers it; that look-up may
// initialise the library's device image. Make this first call before any stream capture is
// begun on that device, and with the device current that the pointers belong to.
//
// Sharing. All calls on a device use the same array and it keeps what the last call left
// there. Nothing needs clearing between calls: each call overwrites every entry it later
// reads. But two calls whose kernels may run at the same time on one device (different
// streams, or different host threads without ordering) write the same memory and race; keep
// calls on one device in stream order. The function calls no cudaMalloc, cudaFree or any
// allocating library routine.
#pragma once
#include <cuda_runtime.h>

#define LUMEN_DECODE_NOALLOC_MAX_FLOATS (4u * 1024u * 1024u)
#define LUMEN_ERR_SCRATCH_TOO_SMALL 100004

extern "C" int lumen_attn_decode_noalloc(const void* q, const void* kcache, const void* vcache,
                                         const int* block_table, int bt_stride, const int* seq_pos,
                                         void* out, int B, int nq, int nkv, int d, int window,
                                         float scale, int max_segs, int* err, cudaStream_t stream);
