// Residual NVFP4 expansion of bf16 activations, shared by the decode linears.
//   x ~= sum_t 8^-t * q_t,   q_t = nvfp4( 8^t * (x - sum_{u<t} 8^-u q_u) )
// One 16-element block of a row becomes TERMS blocks of E2M1 codes with one E4M3 scale each (relative error 7e-4 at
// 3 terms, 5e-5 at 4: below bf16 rounding), which ride as extra columns of a block-scaled FP4 MMA.
#pragma once
#include "common.cuh"
#include <cuda_fp8.h>

namespace ve {

VE_DEVINL float dq_e4m3_dec(uint32_t b) {
  uint32_t r;
  asm("{ .reg .b16 t; cvt.u16.u32 t, %1; cvt.rn.f16x2.e4m3x2 %0, t; }" : "=r"(r) : "r"(b & 0xffu));
  return __half2float(__ushort_as_half((unsigned short)(r & 0xffffu)));
}
VE_DEVINL uint32_t dq_e4m3_enc(float v) {
  unsigned short r;
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(r) : "f"(0.f), "f"(v));
  return r & 0xffu;
}
VE_DEVINL uint32_t dq_e2m1x2_enc(float lo, float hi) {
  uint32_t r;
  asm("{ .reg .b8 t; cvt.rn.satfinite.e2m1x2.f32 t, %1, %2; cvt.u32.u8 %0, t; }" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}
VE_DEVINL float2 dq_e2m1x2_dec(uint32_t byte) {
  uint32_t r;
  asm("{ .reg .b8 t; cvt.u8.u32 t, %1; cvt.rn.f16x2.e2m1x2 %0, t; }" : "=r"(r) : "r"(byte));
  return __half22float2(*reinterpret_cast<const __half2*>(&r));
}

// x [M, K] bf16 (pitch ldx) -> Xp [M * TERMS, K/2] codes (virtual row m * TERMS + t) and scales in 512 B atoms
// [K/64][512] (atom byte (r%32)*16 + (r/32)*4 + j = scale of virtual row r, 16-block j of the 64-wide group).
// One 16-element block of a bf16 row -> TERMS residual NVFP4 blocks: 8 code bytes and one E4M3 scale per term.
VE_DEVINL void load16(const __nv_bfloat16* __restrict__ src, float* r) {
  const bf16x8 t0 = *reinterpret_cast<const bf16x8*>(src), t1 = *reinterpret_cast<const bf16x8*>(src + 8);
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    float2 f = __bfloat1622float2(t0.v[j]);
    r[2 * j] = f.x; r[2 * j + 1] = f.y;
    f = __bfloat1622float2(t1.v[j]);
    r[8 + 2 * j] = f.x; r[8 + 2 * j + 1] = f.y;
  }
}
VE_DEVINL float round_bf16(float x) { return bf2f(f2bf(x)); }

template <int TERMS>
VE_DEVINL void expand_block16(float* r, uint2* codes, uint32_t* scales) {
  float up = 1.f, down = 1.f;
#pragma unroll
  for (int t = 0; t < TERMS; ++t) {
    float amax = 0.f;
#pragma unroll
    for (int j = 0; j < 16; ++j) amax = fmaxf(amax, fabsf(r[j]));
    const uint32_t sb = dq_e4m3_enc(amax * up * (1.f / 6.f));
    const float sd = dq_e4m3_dec(sb);
    const float inv = sd > 0.f ? up / sd : 0.f;
    const float back = sd * down;
    uint32_t w[2] = {0u, 0u};
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const uint32_t byte = dq_e2m1x2_enc(r[2 * j] * inv, r[2 * j + 1] * inv);
      w[j >> 2] |= byte << (8 * (j & 3));
      const float2 d = dq_e2m1x2_dec(byte);
      r[2 * j] -= d.x * back;
      r[2 * j + 1] -= d.y * back;
    }
    codes[t] = make_uint2(w[0], w[1]);
    scales[t] = sb;
    up *= 8.f; down *= 0.125f;
  }
}

// The same expansion with a block shared by two lanes (lane parity = half of the block): r holds this lane's 8 values,
// codes[t] its 8 codes of term t; both lanes get the block's scale bytes. Bit-identical to expand_block16.
template <int TERMS>
VE_DEVINL void expand_half8(float* r, uint32_t* codes, uint32_t* scales) {
  float up = 1.f, down = 1.f;
#pragma unroll
  for (int t = 0; t < TERMS; ++t) {
    float amax = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) amax = fmaxf(amax, fabsf(r[j]));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
    const uint32_t sb = dq_e4m3_enc(amax * up * (1.f / 6.f));
    const float sd = dq_e4m3_dec(sb);
    const float inv = sd > 0.f ? up / sd : 0.f;
    const float back = sd * down;
    uint32_t w = 0u;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const uint32_t byte = dq_e2m1x2_enc(r[2 * j] * inv, r[2 * j + 1] * inv);
      w |= byte << (8 * j);
      const float2 d = dq_e2m1x2_dec(byte);
      r[2 * j] -= d.x * back;
      r[2 * j + 1] -= d.y * back;
    }
    codes[t] = w;
    scales[t] = sb;
    up *= 8.f; down *= 0.125f;
  }
}

}  // namespace ve
