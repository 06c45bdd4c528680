// Entry points of libvolta_kernels.so that never allocate.
//
// This header has no counterpart in the reference engine. It exists for callers that cannot call
// cudaMalloc (or any allocating library routine) at the moment they need a kernel: a server that sized
// one arena at start-up and guarantees that decoding allocates nothing, code embedded in another
// framework's memory pool, or a latency-bound loop for which the device-wide synchronisation of
// cudaMalloc / cudaFree is unacceptable.
#pragma once
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

// NVFP4 mat-vec for 1..16 activation rows on the prepacked decode layout, identical in arithmetic to
// ve_nvfp4_gemv_mma, with the split-K scratch held in device arrays built into the library instead of
// caller-provided buffers.
//
//   Wg  [N/16][K/64][32][4] 32-bit words, Sg [N/16][K/64][16][4] E4M3 bytes (quant/nvfp4.py: prepack_gv)
//   x   [M, K] bf16 with row pitch x_stride (elements); out [M, N] bf16 with pitch out_stride
//   residual: optional [M, N] bf16 added before rounding (nullptr for none)
//
// Limits: M <= 16, N % 16 == 0, K % 64 == 0, KS * N <= 32768 and N <= 65536. Anything larger returns
// cudaErrorInvalidValue and launches nothing. Calls cudaMalloc / cudaFree never; it issues one
// cudaMemsetAsync of the arrival counters (N/16 ints) when KS > 1, then the kernel.
//
// The first call on each device looks up the device addresses of the built-in arrays
// (cudaGetSymbolAddress) with that device current; make that first call before starting any stream
// capture. Host threads may make that first call concurrently (they resolve the same addresses and publish them
// together). Every GPU that loads the library keeps the arrays (2 MiB + 16 KiB) until the process exits.
//
// All calls on a device share the one scratch area and it keeps the previous call's contents: two calls
// that may overlap on the GPU (different streams without an ordering between them) race. Order them on
// one stream or with events.
//
// Returns 0 on success or a cudaError_t value.
int ve_nvfp4_gemv_mma_static(const void* Wg, const void* Sg, float gscale, const void* x, long x_stride,
                             void* out, long out_stride, const void* residual, long res_stride, int M, int N,
                             int K, int KS, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
