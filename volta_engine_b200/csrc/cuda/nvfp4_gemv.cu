// NVFP4 weight x bf16 activation mat-vec for decode / verify rows (M <= 16).
//
//   out[m, n] = gscale * sum_k e2m1(Wp[n, k]) * e4m3(Ws[n, k/16]) * x[m, k]          (+ bias / residual)
//
// Checkpoint layout is consumed as is (compressed-tensors / modelopt): Wp [N, K/2] bytes with the even
// k in the low nibble, Ws [N, K/16] E4M3 bytes, one fp32 global scale
// (reference: src/loader/nvfp4.cpp:36-57, decode rule inc/engine/quant/fp4_fp8.h:14-40).
//
// Design: HBM-bound streaming kernel. One CTA (4 warps) owns R=4 output rows; its 128 threads stride over
// K, each streaming 16 B (32 weights) per row per iteration with evict-first loads (activations come
// through L1), and the four warp partials are summed through shared memory in warp order.
// FP4 decode is the hardware cvt.e2m1x2; partial sums per 16-element block are accumulated in fp32 with
// packed f32x2 FMAs and scaled once per block, so a row's result depends only on its own activations and
// a fixed summation order: the same bits for M = 1 and for a row inside a verify block.
#include "common.cuh"

namespace ve {

VE_DEVINL uint32_t cvt_e2m1x2_f16x2(uint32_t byte) {
  uint32_t r;
  asm("{ .reg .b8 t; cvt.u8.u32 t, %1; cvt.rn.f16x2.e2m1x2 %0, t; }" : "=r"(r) : "r"(byte));
  return r;
}
VE_DEVINL float e4m3_to_float(uint32_t b) {
  uint32_t r;
  asm("{ .reg .b16 t; cvt.u16.u32 t, %1; cvt.rn.f16x2.e4m3x2 %0, t; }" : "=r"(r) : "r"(b & 0xffu));
  return __half2float(__ushort_as_half((unsigned short)(r & 0xffffu)));
}
VE_DEVINL float2 ffma2(float2 a, float2 b, float2 c) {
  unsigned long long d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;"
      : "=l"(d)
      : "l"(*reinterpret_cast<unsigned long long*>(&a)), "l"(*reinterpret_cast<unsigned long long*>(&b)),
        "l"(*reinterpret_cast<unsigned long long*>(&c)));
  return *reinterpret_cast<float2*>(&d);
}

constexpr int kGemvRows = 4;    // output rows per warp
constexpr int kGemvWarps = 4;   // warps per CTA

template <int MR>
__global__ void __launch_bounds__(kGemvWarps * 32)
nvfp4_gemv_kernel(const uint8_t* __restrict__ Wp, const uint8_t* __restrict__ Ws, float gscale,
                  const __nv_bfloat16* __restrict__ x, long x_stride, __nv_bfloat16* __restrict__ out,
                  long out_stride, const __nv_bfloat16* __restrict__ residual, long res_stride, int M, int N, int K,
                  int m0) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int n0 = blockIdx.x * kGemvRows;
  __shared__ float part[kGemvWarps][kGemvRows][MR];
  grid_dep_launch();
  grid_dep_wait();
  const int kchunks = K >> 5;  // 32-element (16 B) chunks per row
  float acc[kGemvRows][MR];
#pragma unroll
  for (int r = 0; r < kGemvRows; ++r)
#pragma unroll
    for (int m = 0; m < MR; ++m) acc[r][m] = 0.f;

  const __nv_bfloat16* xr[MR];
#pragma unroll
  for (int m = 0; m < MR; ++m) xr[m] = x + (long)min(m0 + m, M - 1) * x_stride;

  for (int c = threadIdx.x; c < kchunks; c += kGemvWarps * 32) {
    uint4 w[kGemvRows];
    uint32_t sc[kGemvRows];
#pragma unroll
    for (int r = 0; r < kGemvRows; ++r) {
      const int n = min(n0 + r, N - 1);
      w[r] = __ldcs(reinterpret_cast<const uint4*>(Wp + (long)n * (K >> 1)) + c);
      sc[r] = __ldcs(reinterpret_cast<const unsigned short*>(Ws + (long)n * (K >> 4)) + c);
    }
#pragma unroll
    for (int blk = 0; blk < 2; ++blk) {
      float2 pb[kGemvRows][MR];
#pragma unroll
      for (int r = 0; r < kGemvRows; ++r)
#pragma unroll
        for (int m = 0; m < MR; ++m) pb[r][m] = make_float2(0.f, 0.f);
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        // 8 activations per row m: k = c*32 + blk*16 + half*8 .. +7
        float2 xv[MR][4];
#pragma unroll
        for (int m = 0; m < MR; ++m) {
          const uint4 t = *reinterpret_cast<const uint4*>(xr[m] + (long)c * 32 + blk * 16 + half * 8);
          const uint32_t u[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
          for (int j = 0; j < 4; ++j)
            xv[m][j] = make_float2(__uint_as_float(u[j] << 16), __uint_as_float(u[j] & 0xffff0000u));
        }
#pragma unroll
        for (int r = 0; r < kGemvRows; ++r) {
          const uint32_t word = blk == 0 ? (half == 0 ? w[r].x : w[r].y) : (half == 0 ? w[r].z : w[r].w);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const uint32_t h2 = cvt_e2m1x2_f16x2((word >> (8 * j)) & 0xffu);
            const float2 wf = __half22float2(*reinterpret_cast<const __half2*>(&h2));
#pragma unroll
            for (int m = 0; m < MR; ++m) pb[r][m] = ffma2(wf, xv[m][j], pb[r][m]);
          }
        }
      }
#pragma unroll
      for (int r = 0; r < kGemvRows; ++r) {
        const float s = e4m3_to_float(sc[r] >> (8 * blk));
#pragma unroll
        for (int m = 0; m < MR; ++m) acc[r][m] = fmaf(s, pb[r][m].x + pb[r][m].y, acc[r][m]);
      }
    }
  }
#pragma unroll
  for (int r = 0; r < kGemvRows; ++r)
#pragma unroll
    for (int m = 0; m < MR; ++m) {
      float v = acc[r][m];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
      if (lane == 0) part[warp][r][m] = v;
    }
  __syncthreads();
  if (threadIdx.x < kGemvRows * MR) {
    const int r = threadIdx.x / MR, m = threadIdx.x % MR;
    const int n = n0 + r;
    if (n < N && m0 + m < M) {
      float v = 0.f;
#pragma unroll
      for (int w = 0; w < kGemvWarps; ++w) v += part[w][r][m];
      v *= gscale;
      if (residual) v += bf2f(residual[(long)(m0 + m) * res_stride + n]);
      out[(long)(m0 + m) * out_stride + n] = f2bf(v);
    }
  }
}

// fp32-output variant for the LM head (logits stay fp32 for argmax / top-k / LSE).
template <int MR>
__global__ void __launch_bounds__(kGemvWarps * 32)
bf16_gemv_f32_kernel(const __nv_bfloat16* __restrict__ W, const __nv_bfloat16* __restrict__ x, long x_stride,
                     float* __restrict__ out, long out_stride, int M, int N, int K, int m0) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int n0 = blockIdx.x * kGemvRows;
  __shared__ float part[kGemvWarps][kGemvRows][MR];
  grid_dep_launch();
  grid_dep_wait();                   // x is the output of the kernel in front (this launch is a programmatic dependent)
  float acc[kGemvRows][MR];
#pragma unroll
  for (int r = 0; r < kGemvRows; ++r)
#pragma unroll
    for (int m = 0; m < MR; ++m) acc[r][m] = 0.f;
  const int kchunks = K >> 3;
  for (int c = threadIdx.x; c < kchunks; c += kGemvWarps * 32) {
    float2 xv[MR][4];
#pragma unroll
    for (int m = 0; m < MR; ++m) {
      const uint4 t = *reinterpret_cast<const uint4*>(x + (long)min(m0 + m, M - 1) * x_stride + (long)c * 8);
      const uint32_t u[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
      for (int j = 0; j < 4; ++j)
        xv[m][j] = make_float2(__uint_as_float(u[j] << 16), __uint_as_float(u[j] & 0xffff0000u));
    }
#pragma unroll
    for (int r = 0; r < kGemvRows; ++r) {
      const int n = min(n0 + r, N - 1);
      const uint4 t = __ldcs(reinterpret_cast<const uint4*>(W + (long)n * K) + c);
      const uint32_t u[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 wf = make_float2(__uint_as_float(u[j] << 16), __uint_as_float(u[j] & 0xffff0000u));
#pragma unroll
        for (int m = 0; m < MR; ++m) {
          acc[r][m] = fmaf(wf.x, xv[m][j].x, acc[r][m]);
          acc[r][m] = fmaf(wf.y, xv[m][j].y, acc[r][m]);
        }
      }
    }
  }
#pragma unroll
  for (int r = 0; r < kGemvRows; ++r)
#pragma unroll
    for (int m = 0; m < MR; ++m) {
      float v = acc[r][m];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
      if (lane == 0) part[warp][r][m] = v;
    }
  __syncthreads();
  if (threadIdx.x < kGemvRows * MR) {
    const int r = threadIdx.x / MR, m = threadIdx.x % MR;
    if (n0 + r < N && m0 + m < M) {
      float v = 0.f;
#pragma unroll
      for (int w = 0; w < kGemvWarps; ++w) v += part[w][r][m];
      out[(long)(m0 + m) * out_stride + n0 + r] = v;
    }
  }
}

}  // namespace ve

using namespace ve;

extern "C" {

// x [M, K] bf16 (row stride x_stride), out [M, N] bf16. residual (optional) is added in fp32 before rounding.
int ve_nvfp4_gemv(const void* Wp, const void* Ws, float gscale, const void* x, long x_stride, void* out,
                  long out_stride, const void* residual, long res_stride, int M, int N, int K, cudaStream_t st) {
  if (K % 32 || M <= 0 || N <= 0) return cudaErrorInvalidValue;
  const int blocks = (N + kGemvRows - 1) / kGemvRows;
  int m0 = 0;
  while (m0 < M) {
    const int left = M - m0;
#define VE_LAUNCH(MR)                                                                                            \
  nvfp4_gemv_kernel<MR><<<blocks, kGemvWarps * 32, 0, st>>>(                                                     \
      (const uint8_t*)Wp, (const uint8_t*)Ws, gscale, (const __nv_bfloat16*)x, x_stride, (__nv_bfloat16*)out,    \
      out_stride, (const __nv_bfloat16*)residual, res_stride, M, N, K, m0)
    if (left >= 4) {
      VE_LAUNCH(4);
      m0 += 4;
    } else if (left >= 2) {
      VE_LAUNCH(2);
      m0 += 2;
    } else {
      VE_LAUNCH(1);
      m0 += 1;
    }
#undef VE_LAUNCH
  }
  VE_CHECK_LAUNCH();
}

int ve_bf16_gemv_f32(const void* W, const void* x, long x_stride, void* out, long out_stride, int M, int N, int K,
                     cudaStream_t st) {
  if (K % 8 || M <= 0 || N <= 0) return cudaErrorInvalidValue;
  const int blocks = (N + kGemvRows - 1) / kGemvRows;
  int m0 = 0;
  while (m0 < M) {
    const int left = M - m0;
#define VE_LAUNCH(MR)                                                                                        \
  launch_pdl(bf16_gemv_f32_kernel<MR>, dim3(blocks), dim3(kGemvWarps * 32), 0, st, (const __nv_bfloat16*)W, \
             (const __nv_bfloat16*)x, x_stride, (float*)out, out_stride, M, N, K, m0)
    if (left >= 4) {
      VE_LAUNCH(4);
      m0 += 4;
    } else if (left >= 2) {
      VE_LAUNCH(2);
      m0 += 2;
    } else {
      VE_LAUNCH(1);
      m0 += 1;
    }
#undef VE_LAUNCH
  }
  VE_CHECK_LAUNCH();
}

}  // extern "C"
