// NVFP4 mat-vec for decode and speculative-verify rows (M <= 16) with exact bf16 activations, built to
// stay HBM bound: no conversion instructions on the hot path.
//
// Weights are re-ordered at load time into the register order of mma.sync.m16n8k16 (see
// quant/nvfp4.py: prepack_gv): one 32-bit word per lane per 16 rows x 16 k block. A shift and a mask turn
// each pair of codes into a bf16x2 register whose value is code * 2^-126 (an E2M1 magnitude placed at
// bf16 bits [8:6] is exact, subnormal included); the activations' exponent is biased by +64 with one
// integer add, so products sit near 2^-62 and accumulate exactly in fp32; the factor 2^62 is folded into
// the tensor scale. One MMA covers exactly one 16-element scale block per row, so the E4M3 block scale
// (decoded with a shift and one multiply by 2^120) is applied to the MMA result.
//
// grid (N/16, KS): a CTA of 4 warps owns 16 output rows and 1/KS of K; warps interleave over 64-wide k
// groups (512 contiguous bytes per warp load). Warp partials are summed in warp order through shared
// memory; with KS > 1 the CTA partials go to a scratch buffer and the last CTA to arrive (per-row-block
// counter) sums them in split order, so results are deterministic and a row's value does not depend on how
// many rows are in the batch. The reference's counterpart is the skinny NVFP4 family
// (src/kernels/cuda/nvfp4/skinny_kernels.cu:14-310), which software-unpacks to FP16 for mma.m8n8k4.
#include <atomic>
#include "common.cuh"
#include "volta_noalloc.h"

namespace ve {

constexpr int kGvWarps = 4;

VE_DEVINL void mma_bf16_zero(float* d, const uint32_t* a, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
      : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "f"(0.f));
}
// E4M3 byte at bits [27:20] of `bits` -> float. (byte << 20) is the fp32 pattern of scale * 2^-120.
VE_DEVINL float scale_from_bits(uint32_t bits) {
  float r;
  asm("mul.rn.f32 %0, %1, %2;" : "=f"(r) : "f"(__uint_as_float(bits & 0x0FF00000u)), "f"(1.329227995784916e36f));
  return r;
}

template <int MT>  // MT = 1: up to 8 rows, 2: up to 16 rows
__global__ void __launch_bounds__(kGvWarps * 32)
nvfp4_gemv_mma_kernel(const uint4* __restrict__ Wg, const uint32_t* __restrict__ Sg, float alpha,
                      const __nv_bfloat16* __restrict__ x, long x_stride, __nv_bfloat16* __restrict__ out,
                      long out_stride, const __nv_bfloat16* __restrict__ residual, long res_stride, int M, int N,
                      int KG, int KS, float* __restrict__ ws, int* __restrict__ counters) {
  __shared__ float red[kGvWarps][16][8 * MT];
  __shared__ int s_last;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int rb = blockIdx.x, ks = blockIdx.y;
  const int per = (KG + KS - 1) / KS;
  const int kg_begin = ks * per, kg_end = min(KG, kg_begin + per);

  float acc[MT][4];
#pragma unroll
  for (int m = 0; m < MT; ++m) acc[m][0] = acc[m][1] = acc[m][2] = acc[m][3] = 0.f;

  const uint4* wrow = Wg + (size_t)rb * KG * 32 + lane;
  const uint32_t* srow = Sg + (size_t)rb * KG * 16;  // [kg][16 rows] words of 4 scale bytes
  const __nv_bfloat16* xr[MT];
  bool xok[MT];
#pragma unroll
  for (int m = 0; m < MT; ++m) {
    xok[m] = g + 8 * m < M;
    xr[m] = x + (long)(xok[m] ? g + 8 * m : 0) * x_stride + 4 * t;
  }

  int kg = kg_begin + warp;
  uint4 w = make_uint4(0, 0, 0, 0);
  uint32_t s0 = 0, s1 = 0;
  if (kg < kg_end) {
    w = __ldcs(wrow + (size_t)kg * 32);
    s0 = __ldg(srow + (size_t)kg * 16 + g);
    s1 = __ldg(srow + (size_t)kg * 16 + g + 8);
  }
  while (kg < kg_end) {
    const int nk = kg + kGvWarps;
    uint4 wn = make_uint4(0, 0, 0, 0);
    uint32_t s0n = 0, s1n = 0;
    if (nk < kg_end) {
      wn = __ldcs(wrow + (size_t)nk * 32);
      s0n = __ldg(srow + (size_t)nk * 16 + g);
      s1n = __ldg(srow + (size_t)nk * 16 + g + 8);
    }
    const uint32_t words[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
    for (int kb = 0; kb < 4; ++kb) {
      const uint32_t W = words[kb];
      uint32_t a[4];
      a[0] = ((W << 6) & 0x01C001C0u) | ((W << 3) & 0x80008000u);
      a[1] = ((W << 3) & 0x01C001C0u) | ((W << 2) & 0x80008000u);
      a[2] = (W & 0x01C001C0u) | ((W << 1) & 0x80008000u);
      a[3] = ((W >> 3) & 0x01C001C0u) | (W & 0x80008000u);
      const float sc0 = scale_from_bits(kb == 3 ? (s0 >> 4) : (s0 << (20 - 8 * kb)));
      const float sc1 = scale_from_bits(kb == 3 ? (s1 >> 4) : (s1 << (20 - 8 * kb)));
#pragma unroll
      for (int m = 0; m < MT; ++m) {
        uint2 xb = make_uint2(0u, 0u);
        if (xok[m]) xb = *reinterpret_cast<const uint2*>(xr[m] + (long)kg * 64 + kb * 16);
        float d[4];
        mma_bf16_zero(d, a, xb.x + 0x20002000u, xb.y + 0x20002000u);
        acc[m][0] = fmaf(sc0, d[0], acc[m][0]);
        acc[m][1] = fmaf(sc0, d[1], acc[m][1]);
        acc[m][2] = fmaf(sc1, d[2], acc[m][2]);
        acc[m][3] = fmaf(sc1, d[3], acc[m][3]);
      }
    }
    w = wn;
    s0 = s0n;
    s1 = s1n;
    kg = nk;
  }
  // warp partials -> shared, summed in warp order
#pragma unroll
  for (int m = 0; m < MT; ++m) {
    red[warp][g][m * 8 + 2 * t] = acc[m][0];
    red[warp][g][m * 8 + 2 * t + 1] = acc[m][1];
    red[warp][g + 8][m * 8 + 2 * t] = acc[m][2];
    red[warp][g + 8][m * 8 + 2 * t + 1] = acc[m][3];
  }
  __syncthreads();
  const int row = threadIdx.x >> 3, tk = threadIdx.x & 7;
  const int n = rb * 16 + row;
  float v[MT];
#pragma unroll
  for (int m = 0; m < MT; ++m) {
    float s = 0.f;
#pragma unroll
    for (int wv = 0; wv < kGvWarps; ++wv) s += red[wv][row][m * 8 + tk];
    v[m] = s;
  }
  if (KS > 1) {
#pragma unroll
    for (int m = 0; m < MT; ++m) ws[((size_t)ks * N + n) * (8 * MT) + m * 8 + tk] = v[m];
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
      const int prev = atomicAdd(&counters[rb], 1);
      s_last = (prev == KS - 1);
      if (s_last) counters[rb] = 0;
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
#pragma unroll
    for (int m = 0; m < MT; ++m) {
      float s = 0.f;
      for (int k2 = 0; k2 < KS; ++k2) s += __ldcg(ws + ((size_t)k2 * N + n) * (8 * MT) + m * 8 + tk);
      v[m] = s;
    }
  }
#pragma unroll
  for (int m = 0; m < MT; ++m) {
    const int tok = m * 8 + tk;
    if (tok < M && n < N) {
      float r = v[m] * alpha;
      if (residual) r += bf2f(residual[(long)tok * res_stride + n]);
      out[(long)tok * out_stride + n] = f2bf(r);
    }
  }
}

}  // namespace ve

using namespace ve;

extern "C" {

// Wg [N/16][K/64][32][4] words, Sg [N/16][K/64][16][4] bytes (prepack_gv). ws: fp32 scratch of at least
// KS * N * 16 floats when KS > 1; counters: N/16 zero-initialised ints (left zero on return).
int ve_nvfp4_gemv_mma(const void* Wg, const void* Sg, float gscale, const void* x, long x_stride, void* out,
                      long out_stride, const void* residual, long res_stride, int M, int N, int K, int KS, void* ws,
                      void* counters, cudaStream_t st) {
  if (M <= 0 || M > 16 || N % 16 || K % 64 || KS < 1) return cudaErrorInvalidValue;
  if (KS > 1 && (!ws || !counters)) return cudaErrorInvalidValue;
  const float alpha = gscale * 4.611686018427388e18f;  // 2^62
  dim3 grid(N / 16, KS);
  if (M <= 8)
    nvfp4_gemv_mma_kernel<1><<<grid, kGvWarps * 32, 0, st>>>(
        (const uint4*)Wg, (const uint32_t*)Sg, alpha, (const __nv_bfloat16*)x, x_stride, (__nv_bfloat16*)out,
        out_stride, (const __nv_bfloat16*)residual, res_stride, M, N, K / 64, KS, (float*)ws, (int*)counters);
  else
    nvfp4_gemv_mma_kernel<2><<<grid, kGvWarps * 32, 0, st>>>(
        (const uint4*)Wg, (const uint32_t*)Sg, alpha, (const __nv_bfloat16*)x, x_stride, (__nv_bfloat16*)out,
        out_stride, (const __nv_bfloat16*)residual, res_stride, M, N, K / 64, KS, (float*)ws, (int*)counters);
  VE_CHECK_LAUNCH();
}

}  // extern "C"

// ------------------------------------------------------------------------------------------------
// Allocation-free variant (declared in volta_noalloc.h; the reference has nothing like it).
//
// Some hosts of this library must not touch the CUDA allocator while they serve: an engine that took one
// arena at boot and promised "no allocation while decoding", a plugin living inside another runtime's
// memory pool, a latency-critical loop that cannot afford the device-wide synchronisation cudaMalloc and
// cudaFree imply. For them the split-K scratch of the mat-vec lives in the two file-scope device arrays
// below, which every GPU that loads this library holds until the process exits (2 MiB + 16 KiB).
// ------------------------------------------------------------------------------------------------
namespace ve {
constexpr int kStaticWsRows = 32768;      // limit on KS * N
constexpr int kStaticCounters = 4096;     // limit on N / 16
static __device__ __align__(256) float g_static_ws[(size_t)kStaticWsRows * 16];
static __device__ __align__(256) int g_static_counters[kStaticCounters];
constexpr int kMaxDevices = 64;
// device addresses of the arrays above, resolved per device. The pair is published through one atomic pointer so that a
// host thread that sees the entry sees both addresses (two threads making the first call on a device resolve the same
// values; whichever publishes last wins, harmlessly)
struct StaticAddrs { float* ws; int* cnt; };
static StaticAddrs g_addr_store[kMaxDevices];
static std::atomic<StaticAddrs*> g_addrs[kMaxDevices];
}  // namespace ve

extern "C" {

int ve_nvfp4_gemv_mma_static(const void* Wg, const void* Sg, float gscale, const void* x, long x_stride, void* out,
                             long out_stride, const void* residual, long res_stride, int M, int N, int K, int KS,
                             cudaStream_t st) {
  if (M <= 0 || M > 16 || N <= 0 || N % 16 || K <= 0 || K % 64 || KS < 1) return cudaErrorInvalidValue;
  // sizes beyond the built-in scratch are refused, never truncated
  if ((long)KS * N > kStaticWsRows || N / 16 > kStaticCounters) return cudaErrorInvalidValue;
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= kMaxDevices) return cudaErrorInvalidDevice;
  StaticAddrs* addrs = g_addrs[dev].load(std::memory_order_acquire);
  if (!addrs) {
    // In host code the array names are only handles; the kernel needs the addresses the current device
    // gave them. Resolved on the first call for each device.
    float* ws = nullptr;
    int* cnt = nullptr;
    e = cudaGetSymbolAddress((void**)&ws, g_static_ws);
    if (e != cudaSuccess) return (int)e;
    e = cudaGetSymbolAddress((void**)&cnt, g_static_counters);
    if (e != cudaSuccess) return (int)e;
    g_addr_store[dev] = StaticAddrs{ws, cnt};
    addrs = &g_addr_store[dev];
    g_addrs[dev].store(addrs, std::memory_order_release);
  }
  if (KS > 1) {
    // the arrival counters must read zero when the kernel starts; the partial sums need no clearing
    // because every slot that is read has been written by this call
    e = cudaMemsetAsync(addrs->cnt, 0, (size_t)(N / 16) * sizeof(int), st);
    if (e != cudaSuccess) return (int)e;
  }
  return ve_nvfp4_gemv_mma(Wg, Sg, gscale, x, x_stride, out, out_stride, residual, res_stride, M, N, K, KS,
                           addrs->ws, addrs->cnt, st);
}

}  // extern "C"
