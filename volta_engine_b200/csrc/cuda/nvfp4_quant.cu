// NVFP4 helpers: dequantise a weight matrix to bf16 (oracle / fallback path) and quantise activation rows
// to E2M1 codes + E4M3 block scales laid out for the block-scaled tensor-core GEMM.
// Rounding rules are the hardware cvt.rn.satfinite ones (round to nearest even, saturating), the same RNE
// tie rule the reference shares between host and device (inc/engine/quant/fp4_fp8.h:14-40).
#include "common.cuh"

namespace ve {

VE_DEVINL float e4m3_dec(uint32_t b) {
  uint32_t r;
  asm("{ .reg .b16 t; cvt.u16.u32 t, %1; cvt.rn.f16x2.e4m3x2 %0, t; }" : "=r"(r) : "r"(b & 0xffu));
  return __half2float(__ushort_as_half((unsigned short)(r & 0xffffu)));
}
VE_DEVINL uint32_t e4m3_enc(float v) {
  unsigned short r;
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(r) : "f"(0.f), "f"(v));
  return r & 0xffu;
}
// returns a byte: lo -> low nibble, hi -> high nibble
VE_DEVINL uint32_t e2m1x2_enc(float lo, float hi) {
  uint32_t r;
  asm("{ .reg .b8 t; cvt.rn.satfinite.e2m1x2.f32 t, %1, %2; cvt.u32.u8 %0, t; }" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}

__global__ void nvfp4_dequant_kernel(const uint8_t* __restrict__ Wp, const uint8_t* __restrict__ Ws, float gscale,
                                     __nv_bfloat16* __restrict__ out, long nblocks, int kblocks) {
  // one thread per 16-element block
  for (long b = blockIdx.x * (long)blockDim.x + threadIdx.x; b < nblocks; b += (long)gridDim.x * blockDim.x) {
    const float s = e4m3_dec(Ws[b]) * gscale;
    const uint2 w = *reinterpret_cast<const uint2*>(Wp + b * 8);
    const uint32_t words[2] = {w.x, w.y};
    __nv_bfloat16* o = out + b * 16;
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        uint32_t h2;
        const uint32_t byte = (words[i] >> (8 * j)) & 0xffu;
        asm("{ .reg .b8 t; cvt.u8.u32 t, %1; cvt.rn.f16x2.e2m1x2 %0, t; }" : "=r"(h2) : "r"(byte));
        const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&h2));
        o[i * 8 + j * 2] = f2bf(f.x * s);
        o[i * 8 + j * 2 + 1] = f2bf(f.y * s);
      }
  }
}

// Activation rows -> NVFP4. X [T, K] bf16 (pitch ldx). Xp [T, K/2]; scales either row-major [T, K/16]
// (blocked == 0) or in 512 B atoms [ceil(T/128)][K/64][512] (blocked == 1). inv_gscale multiplies x first.
__global__ void nvfp4_quant_rows_kernel(const __nv_bfloat16* __restrict__ X, long ldx, uint8_t* __restrict__ Xp,
                                        uint8_t* __restrict__ Xs, int T, int K, float inv_gscale, int blocked) {
  const int kb = K >> 4;
  const long total = (long)T * kb;
  for (long idx = blockIdx.x * (long)blockDim.x + threadIdx.x; idx < total; idx += (long)gridDim.x * blockDim.x) {
    const int r = (int)(idx / kb), b = (int)(idx % kb);
    const __nv_bfloat16* src = X + (long)r * ldx + b * 16;
    float v[16];
    const bf16x8 t0 = *reinterpret_cast<const bf16x8*>(src), t1 = *reinterpret_cast<const bf16x8*>(src + 8);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float2 f = __bfloat1622float2(t0.v[j]);
      v[2 * j] = f.x * inv_gscale;
      v[2 * j + 1] = f.y * inv_gscale;
      f = __bfloat1622float2(t1.v[j]);
      v[8 + 2 * j] = f.x * inv_gscale;
      v[8 + 2 * j + 1] = f.y * inv_gscale;
    }
    float amax = 0.f;
#pragma unroll
    for (int j = 0; j < 16; ++j) amax = fmaxf(amax, fabsf(v[j]));
    const uint32_t sb = e4m3_enc(amax * (1.f / 6.f));
    const float sd = e4m3_dec(sb);
    const float inv = sd > 0.f ? 1.f / sd : 0.f;
    uint32_t w[2] = {0u, 0u};
#pragma unroll
    for (int j = 0; j < 8; ++j) w[j >> 2] |= e2m1x2_enc(v[2 * j] * inv, v[2 * j + 1] * inv) << (8 * (j & 3));
    *reinterpret_cast<uint2*>(Xp + (long)r * (K >> 1) + b * 8) = make_uint2(w[0], w[1]);
    if (blocked) {
      const int tb = r >> 7, rr = r & 127, kg = b >> 2, j = b & 3;
      Xs[((long)tb * (K >> 6) + kg) * 512 + (rr & 31) * 16 + (rr >> 5) * 4 + j] = (uint8_t)sb;
    } else {
      Xs[(long)r * kb + b] = (uint8_t)sb;
    }
  }
}

}  // namespace ve

using namespace ve;

extern "C" {

int ve_nvfp4_dequant(const void* Wp, const void* Ws, float gscale, void* out, long N, int K, cudaStream_t st) {
  if (K % 16) return cudaErrorInvalidValue;
  const long nblocks = N * (K / 16);
  if (nblocks <= 0) return 0;
  const int blocks = (int)((nblocks + 255) / 256 < 148 * 16 ? (nblocks + 255) / 256 : 148 * 16);
  nvfp4_dequant_kernel<<<blocks, 256, 0, st>>>((const uint8_t*)Wp, (const uint8_t*)Ws, gscale, (__nv_bfloat16*)out,
                                               nblocks, K / 16);
  VE_CHECK_LAUNCH();
}

int ve_nvfp4_quant_rows(const void* X, long ldx, void* Xp, void* Xs, int T, int K, float inv_gscale, int blocked,
                        cudaStream_t st) {
  if (K % 64 || T <= 0) return cudaErrorInvalidValue;
  const long total = (long)T * (K / 16);
  const int blocks = (int)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
  nvfp4_quant_rows_kernel<<<blocks, 256, 0, st>>>((const __nv_bfloat16*)X, ldx, (uint8_t*)Xp, (uint8_t*)Xs, T, K,
                                                  inv_gscale, blocked);
  VE_CHECK_LAUNCH();
}

}  // extern "C"
