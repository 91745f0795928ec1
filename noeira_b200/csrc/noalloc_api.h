// Allocation-free entry point.  This has no counterpart in the reference code base.
//
// Who it is for: code that wants a bias-gradient style column sum but is not in a position to
// obtain device memory for the kernel's scratch — a plug-in running inside a host application that
// owns the allocator and hands out only the input and output buffers, a real-time control loop
// that must not enter the driver's allocation path (it can block for milliseconds), or a component
// that runs after the process has deliberately committed all device memory.  The regular entry
// point, nb_colsum_bf16, expects the caller to supply `nb_colsum_split(M) * N` floats of scratch for
// its per-slab partial sums; here that scratch is a fixed array compiled into the library.
//
// What it costs: the array (NB_COLSUM_NOALLOC_SCRATCH_FLOATS floats = 4 MiB) is part of the module
// image, so every GPU on which this library is loaded carries it until the process exits, whether or
// not the function is ever called.
//
// Limits and rules:
//   * nb_colsum_split(M) * N must not exceed NB_COLSUM_NOALLOC_SCRATCH_FLOATS, otherwise the call
//     returns NB_ERR_TOO_LARGE (10003) and launches nothing.  With the largest split (256 slabs,
//     reached from M = 16384 rows) that allows N up to 4096 columns; fewer rows allow more columns.
//   * The first call on each device looks up the device address of the array (cudaGetSymbolAddress,
//     with that device current) and caches it.  Make that first call outside any stream capture.
//   * The function itself calls no cudaMalloc / cudaFree and no allocating library routine.
//   * All calls on a device share the one array.  Nothing in it needs to start at zero — each call
//     overwrites every partial it later reads — but two calls that run concurrently on the same GPU
//     (different streams, or different host threads) race on it.  Serialise them on one stream.
//   * Inputs and outputs are still the caller's: x is bf16 [M, N] with row pitch ld (elements),
//     out is fp32 [N]; accumulate != 0 adds to out instead of overwriting it.
// Returns 0 on success, 10003 as above, 10001 for non-positive sizes, or a cudaError_t value.
#pragma once

#define NB_COLSUM_NOALLOC_SCRATCH_FLOATS (1 << 20)

#ifdef __cplusplus
extern "C" {
#endif
int nb_colsum_bf16_noalloc(const void* x, int M, int N, int ld, float* out, int accumulate, void* stream);
#ifdef __cplusplus
}
#endif
