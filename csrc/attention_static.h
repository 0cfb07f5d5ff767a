// Allocation-free attention entry point.
//
// This entry point has no counterpart in the reference implementation. It exists for callers that are not
// allowed to allocate device memory at the moment they need attention: code running inside a memory-pool
// callback or under an allocator lock, a host that has handed all of its HBM to the KV cache and weight
// arenas up front, or an embedding application whose policy forbids cudaMalloc after start-up. Such a
// caller still owns its inputs and outputs, but has nowhere to put the split-K partial buffer that
// vg_attn_decode needs.
//
// vg_attn_decode_static is vg_attn_decode with that partial buffer taken from a fixed array that is part of
// the library image (VG_ATTN_STATIC_MAX_FLOATS floats = 16 MiB, resident on every GPU that loads the library
// until the process exits). Everything else - arguments, kernels, arithmetic, results - is identical.
//
// Rules of use:
//  * Size limit: N * nh * ns_grid * (hd + 2) must not exceed VG_ATTN_STATIC_MAX_FLOATS. A larger request is
//    refused with VG_ERR_STATIC_SCRATCH (-20) and a message on stderr; nothing is launched.
//  * `ns_grid` is the largest number of key splits a column may use (the models pass 32). A column of `len`
//    keys uses min(max(len / 64, 1), 32, ns_grid) splits, so a smaller `ns_grid` shrinks the buffer that is
//    needed and makes every split longer; it never drops keys. ns_grid < 1 is refused (-2).
//  * It calls no cudaMalloc / cudaFree and no allocating library routine.
//  * The first call on a device looks up the array's device address (cudaGetSymbolAddress, with the
//    stream's device current). Make that first call outside of any stream capture.
//  * The array is shared by every call on the device and keeps the previous call's contents. Nothing in it
//    has to start at zero: each launch writes every partial it later reads. Two calls whose kernels can run
//    at the same time on one GPU (different streams, no dependency between them) would overwrite each
//    other's partials - serialise them on one stream or with events.
//  * The device that owns `stream` must be the current device of the calling thread.
#pragma once
#include <cuda_runtime.h>

#define VG_ATTN_STATIC_MAX_FLOATS (4ll * 1024 * 1024)
#define VG_ERR_STATIC_SCRATCH (-20)

#ifdef __cplusplus
extern "C" {
#endif

// Same contract as vg_attn_decode (see api.h) without the `part` argument.
int vg_attn_decode_static(const void* q, const void* kc, const void* vc, const int* lens, const int* slots,
                          const int* base, const int* path, int path_ld, int N, int nh, int nkv, int hd, int max_seq,
                          int ns_grid, int direct, const void* gate, int ld_gate, void* out, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
