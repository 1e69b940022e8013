// SSD chunk scan for callers that may not allocate device memory.
//
// This entry point has no counterpart in the reference implementation (which has neither a Mamba
// path nor a C interface); it exists for embedders of this library whose steady state forbids
// device allocation: an inference server that carves up the GPU once at start-up and then runs with
// the allocator locked, a real-time loop where cudaMalloc's implicit device synchronisation is not
// acceptable, or a plug-in that is handed input / output buffers by its host and has no allocator
// of its own to ask for the per-chunk state scratch that `bdh_ssd_chunk_scan` needs from its caller.
//
// Same computation and same input / output contract as `bdh_ssd_chunk_scan` (see bdh_kernels.h):
//     h_t = exp(loga_t) h_{t-1} + B_t (x) xw_t ;  y_t = C_t . h_t
//     xw [B,T,H,64], loga [B,T,H], Bm/Cm [B,T,128], h [B,H,128,64] in/out, y [B,T,H,64], fp32, T % 64 == 0
// but the per-chunk states and decays live in a fixed array inside the library instead of caller
// memory. Limits and rules:
//   * B * (T/64) * H must not exceed BDH_SSD_STATIC_MAX_CHUNK_HEADS (512); larger problems return
//     BDH_ERR_TOO_LARGE and print one line to stderr. The array occupies
//     512 * (128*64 + 1) * 4 bytes (about 16 MiB) on every GPU that loads the library, until exit.
//   * Nothing is allocated or freed: no cudaMalloc / cudaFree, no allocating library call.
//   * The first call on each device looks up the array's device address (cudaGetSymbolAddress, with
//     that device current) and remembers it. Make that first call outside of any stream capture.
//   * All calls share the one array and it keeps whatever the last call left in it. The kernels
//     overwrite every scratch element they later read, so nothing has to be cleared; but two calls
//     whose kernels overlap on the GPU (different streams, no dependency) race on it. Serialise them.
#pragma once
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

#define BDH_SSD_STATIC_MAX_CHUNK_HEADS 512

int bdh_ssd_chunk_scan_static(const float* xw, const float* loga, const float* Bm, const float* Cm, float* h,
                              float* y, int B, int T, int H, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
