// GGUF block formats: dequantisation fused into the mat-vec (decode / verify rows, M <= 16) and a plain
// dequantise-to-bf16 kernel that feeds the tcgen05 GEMM for prefill chunks.
//   Q8_0, Q4_0, Q4_1, Q5_0, Q5_1, IQ4_NL (32-value blocks), Q2_K, Q3_K, Q4_K, Q5_K, Q6_K, IQ4_XS and the codebook
//   formats IQ1_S, IQ1_M, IQ2_XXS, IQ2_XS, IQ2_S, IQ3_XXS, IQ3_S (256-value super-blocks), bf16 activations, fp32
//   accumulation.
// One warp per output row; a lane decodes 32 consecutive weights at a time straight from the packed row and
// multiplies them with the activations of every batch row, so the weights are read exactly once.
// Summation order per row is fixed (lane-strided chunks, then a butterfly), independent of M.
// Reference counterparts: src/kernels/cuda/gguf/gguf_linear.cu:38-160 (gemv on q8_1 activations) and the
// vendored dequantize kernels; block layouts as in quant/gguf.py.
#include "common.cuh"

namespace ve {

enum GgmlType { kQ4_0 = 2, kQ4_1 = 3, kQ5_0 = 6, kQ5_1 = 7, kQ8_0 = 8, kQ2_K = 10, kQ3_K = 11, kQ4_K = 12, kQ5_K = 13,
                kQ6_K = 14, kIQ2_XXS = 16, kIQ2_XS = 17, kIQ3_XXS = 18, kIQ1_S = 19, kIQ4_NL = 20, kIQ3_S = 21, kIQ2_S = 22,
                kIQ4_XS = 23, kIQ1_M = 29 };

// Codebook formats (IQ1 / IQ2 / IQ3): one table of grid vectors and sign bytes in device memory, uploaded once per device
// by the host (ve_gguf_set_iq_grids). Byte offsets of the parts, as in quant/gguf_iq.py:
//   0 sign bytes [128] | 128 iq2xxs [256][8] | 2176 iq2xs [512][8] | 6272 iq2s [1024][8] | 14464 iq3xxs [256][4]
//   | 15488 iq3s [512][4] | 17536 iq1s [2048][8] (int8)
__constant__ const uint8_t* kIqGrids;
constexpr int kOffSigns = 0, kOff2xxs = 128, kOff2xs = 2176, kOff2s = 6272, kOff3xxs = 14464, kOff3s = 15488, kOff1s = 17536;

// 8 grid bytes times a scale with the signs of `sb` (bit j set = element j negative)
VE_DEVINL void put8(const uint8_t* __restrict__ g, uint32_t sb, float db, float* w) {
  const uint2 v = *reinterpret_cast<const uint2*>(g);
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    w[j] = ((sb >> j) & 1 ? -db : db) * (float)((v.x >> (8 * j)) & 255);
    w[j + 4] = ((sb >> (j + 4)) & 1 ? -db : db) * (float)((v.y >> (8 * j)) & 255);
  }
}
VE_DEVINL void put4(const uint8_t* __restrict__ g, uint32_t sb, float db, float* w) {
  const uint32_t v = *reinterpret_cast<const uint32_t*>(g);
#pragma unroll
  for (int j = 0; j < 4; ++j) w[j] = ((sb >> j) & 1 ? -db : db) * (float)((v >> (8 * j)) & 255);
}
// 8 ternary grid values (int8) plus a shift, times a scale
VE_DEVINL void put8_shift(const uint8_t* __restrict__ g, float delta, float dl, float* w) {
  const uint2 v = *reinterpret_cast<const uint2*>(g);
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    w[j] = dl * ((float)(int8_t)((v.x >> (8 * j)) & 255) + delta);
    w[j + 4] = dl * ((float)(int8_t)((v.y >> (8 * j)) & 255) + delta);
  }
}

// the 16 non-uniform levels of the IQ4 formats
__constant__ int8_t kIq4Levels[16] = {-127, -104, -83, -65, -49, -35, -22, -10, 1, 13, 25, 38, 53, 69, 89, 113};

VE_DEVINL void scale_min_k4(const uint8_t* s, int sb, int& sc, int& mn) {
  if (sb < 4) { sc = s[sb] & 63; mn = s[sb + 4] & 63; }
  else { sc = (s[sb + 4] & 15) | ((s[sb - 4] >> 6) << 4); mn = (s[sb + 4] >> 4) | ((s[sb] >> 6) << 4); }
}

VE_DEVINL float h2f(const uint8_t* p) {
  return __half2float(__ushort_as_half((unsigned short)(p[0] | (p[1] << 8))));
}

// Decode the 32 weights of chunk `c` of a packed row into w[32].
template <int TYPE>
VE_DEVINL void decode32(const uint8_t* __restrict__ row, int c, float* w) {
  if (TYPE == kQ8_0) {
    const uint8_t* b = row + (size_t)c * 34;
    const float d = h2f(b);
#pragma unroll
    for (int j = 0; j < 32; ++j) w[j] = d * (float)(int8_t)b[2 + j];
  } else if (TYPE == kQ4_0) {
    const uint8_t* b = row + (size_t)c * 18;
    const float d = h2f(b);
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      w[j] = d * (float)((int)(b[2 + j] & 15) - 8);
      w[j + 16] = d * (float)((int)(b[2 + j] >> 4) - 8);
    }
  } else if (TYPE == kQ4_K) {
    const uint8_t* b = row + (size_t)(c >> 3) * 144;
    const int sb = c & 7;                       // sub-block 0..7
    const float d = h2f(b), dmin = h2f(b + 2);
    const uint8_t* s = b + 4;
    int sc, mn;
    scale_min_k4(s, sb, sc, mn);
    const float d1 = d * (float)sc, m1 = dmin * (float)mn;
    const uint8_t* q = b + 16 + (sb >> 1) * 32;
    const int shift = (sb & 1) * 4;
#pragma unroll
    for (int j = 0; j < 32; ++j) w[j] = d1 * (float)((q[j] >> shift) & 15) - m1;
  } else if (TYPE == kQ4_1) {
    const uint8_t* b = row + (size_t)c * 20;
    const float d = h2f(b), m = h2f(b + 2);
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      w[j] = fmaf(d, (float)(b[4 + j] & 15), m);
      w[j + 16] = fmaf(d, (float)(b[4 + j] >> 4), m);
    }
  } else if (TYPE == kQ5_0 || TYPE == kQ5_1) {
    const int hdr = TYPE == kQ5_0 ? 2 : 4;
    const uint8_t* b = row + (size_t)c * (TYPE == kQ5_0 ? 22 : 24);
    const float d = h2f(b), m = TYPE == kQ5_0 ? 0.f : h2f(b + 2);
    const uint32_t qh = b[hdr] | (b[hdr + 1] << 8) | (b[hdr + 2] << 16) | ((uint32_t)b[hdr + 3] << 24);
    const int off = TYPE == kQ5_0 ? 16 : 0;
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      const int q0 = (b[hdr + 4 + j] & 15) | (((qh >> j) & 1) << 4);
      const int q1 = (b[hdr + 4 + j] >> 4) | (((qh >> (j + 16)) & 1) << 4);
      w[j] = fmaf(d, (float)(q0 - off), m);
      w[j + 16] = fmaf(d, (float)(q1 - off), m);
    }
  } else if (TYPE == kIQ4_NL) {
    const uint8_t* b = row + (size_t)c * 18;
    const float d = h2f(b);
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      w[j] = d * (float)kIq4Levels[b[2 + j] & 15];
      w[j + 16] = d * (float)kIq4Levels[b[2 + j] >> 4];
    }
  } else if (TYPE == kIQ4_XS) {
    const uint8_t* b = row + (size_t)(c >> 3) * 136;
    const int ib = c & 7;
    const int sh = b[2] | (b[3] << 8);
    const int ls = ((b[4 + (ib >> 1)] >> (4 * (ib & 1))) & 15) | (((sh >> (2 * ib)) & 3) << 4);
    const float dl = h2f(b) * (float)(ls - 32);
    const uint8_t* q = b + 8 + ib * 16;
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      w[j] = dl * (float)kIq4Levels[q[j] & 15];
      w[j + 16] = dl * (float)kIq4Levels[q[j] >> 4];
    }
  } else if (TYPE == kIQ2_XXS) {
    const uint8_t* b = row + (size_t)(c >> 3) * 66;
    const uint8_t* q = b + 2 + (c & 7) * 8;
    const uint32_t aux = q[4] | (q[5] << 8) | (q[6] << 16) | ((uint32_t)q[7] << 24);
    const float db = h2f(b) * (0.5f + (float)(aux >> 28)) * 0.25f;
#pragma unroll
    for (int l = 0; l < 4; ++l)
      put8(kIqGrids + kOff2xxs + q[l] * 8, kIqGrids[kOffSigns + ((aux >> (7 * l)) & 127)], db, w + 8 * l);
  } else if (TYPE == kIQ2_XS) {
    const uint8_t* b = row + (size_t)(c >> 3) * 74;
    const int ib = c & 7;
    const uint8_t* q = b + 2 + ib * 8;
    const int sc = b[66 + ib];
    const float d = h2f(b);
#pragma unroll
    for (int l = 0; l < 4; ++l) {
      const int v = q[2 * l] | (q[2 * l + 1] << 8);
      const float db = d * (0.5f + (float)(l < 2 ? (sc & 15) : (sc >> 4))) * 0.25f;
      put8(kIqGrids + kOff2xs + (v & 511) * 8, kIqGrids[kOffSigns + (v >> 9)], db, w + 8 * l);
    }
  } else if (TYPE == kIQ2_S) {
    const uint8_t* b = row + (size_t)(c >> 3) * 82;
    const int ib = c & 7;
    const uint8_t* q = b + 2 + ib * 4;
    const uint8_t* sg = b + 34 + ib * 4;
    const int qh = b[66 + ib], sc = b[74 + ib];
    const float d = h2f(b);
#pragma unroll
    for (int l = 0; l < 4; ++l) {
      const float db = d * (0.5f + (float)(l < 2 ? (sc & 15) : (sc >> 4))) * 0.25f;
      put8(kIqGrids + kOff2s + (q[l] | ((qh << (8 - 2 * l)) & 0x300)) * 8, sg[l], db, w + 8 * l);
    }
  } else if (TYPE == kIQ3_XXS) {
    const uint8_t* b = row + (size_t)(c >> 3) * 98;
    const int ib = c & 7;
    const uint8_t* q = b + 2 + ib * 8;
    const uint8_t* a = b + 66 + ib * 4;
    const uint32_t aux = a[0] | (a[1] << 8) | (a[2] << 16) | ((uint32_t)a[3] << 24);
    const float db = h2f(b) * (0.5f + (float)(aux >> 28)) * 0.5f;
#pragma unroll
    for (int l = 0; l < 4; ++l) {
      const uint32_t sb = kIqGrids[kOffSigns + ((aux >> (7 * l)) & 127)];
      put4(kIqGrids + kOff3xxs + q[2 * l] * 4, sb, db, w + 8 * l);
      put4(kIqGrids + kOff3xxs + q[2 * l + 1] * 4, sb >> 4, db, w + 8 * l + 4);
    }
  } else if (TYPE == kIQ3_S) {
    const uint8_t* b = row + (size_t)(c >> 3) * 110;
    const int ib = c & 7;
    const uint8_t* q = b + 2 + ib * 8;
    const int qh = b[66 + ib];
    const uint8_t* sg = b + 74 + ib * 4;
    const int nib = (b[106 + (ib >> 1)] >> (4 * (ib & 1))) & 15;
    const float db = h2f(b) * (float)(1 + 2 * nib);
#pragma unroll
    for (int l = 0; l < 4; ++l) {
      put4(kIqGrids + kOff3s + (q[2 * l] | ((qh << (8 - 2 * l)) & 256)) * 4, sg[l], db, w + 8 * l);
      put4(kIqGrids + kOff3s + (q[2 * l + 1] | ((qh << (7 - 2 * l)) & 256)) * 4, sg[l] >> 4, db, w + 8 * l + 4);
    }
  } else if (TYPE == kIQ1_S) {
    const uint8_t* b = row + (size_t)(c >> 3) * 50;
    const int ib = c & 7;
    const uint8_t* q = b + 2 + ib * 4;
    const int qh = b[34 + 2 * ib] | (b[35 + 2 * ib] << 8);
    const float dl = h2f(b) * (float)(2 * ((qh >> 12) & 7) + 1);
    const float delta = (qh & 0x8000) ? -0.125f : 0.125f;
#pragma unroll
    for (int l = 0; l < 4; ++l)
      put8_shift(kIqGrids + kOff1s + (q[l] | (((qh >> (3 * l)) & 7) << 8)) * 8, delta, dl, w + 8 * l);
  } else if (TYPE == kIQ1_M) {
    const uint8_t* b = row + (size_t)(c >> 3) * 56;
    const int ib = c & 7;
    const uint8_t* q = b + ib * 4;
    const int q0 = b[32 + 2 * ib], q1 = b[33 + 2 * ib];
    const uint8_t* s8 = b + 48;
    const int s0 = s8[0] | (s8[1] << 8), s1 = s8[2] | (s8[3] << 8), s2 = s8[4] | (s8[5] << 8), s3 = s8[6] | (s8[7] << 8);
    const unsigned short bits = (unsigned short)((s0 >> 12) | ((s1 >> 8) & 0x00f0) | ((s2 >> 4) & 0x0f00) | (s3 & 0xf000));
    const float d = __half2float(__ushort_as_half(bits));
    const int sw = (ib >> 1) == 0 ? s0 : (ib >> 1) == 1 ? s1 : (ib >> 1) == 2 ? s2 : s3;
    const float dl1 = d * (float)(2 * ((sw >> (6 * (ib & 1))) & 7) + 1);
    const float dl2 = d * (float)(2 * ((sw >> (6 * (ib & 1) + 3)) & 7) + 1);
    put8_shift(kIqGrids + kOff1s + (q[0] | ((q0 << 8) & 0x700)) * 8, (q0 & 0x08) ? -0.125f : 0.125f, dl1, w);
    put8_shift(kIqGrids + kOff1s + (q[1] | ((q0 << 4) & 0x700)) * 8, (q0 & 0x80) ? -0.125f : 0.125f, dl1, w + 8);
    put8_shift(kIqGrids + kOff1s + (q[2] | ((q1 << 8) & 0x700)) * 8, (q1 & 0x08) ? -0.125f : 0.125f, dl2, w + 16);
    put8_shift(kIqGrids + kOff1s + (q[3] | ((q1 << 4) & 0x700)) * 8, (q1 & 0x80) ? -0.125f : 0.125f, dl2, w + 24);
  } else if (TYPE == kQ2_K) {
    const uint8_t* b = row + (size_t)(c >> 3) * 84;
    const int half = (c >> 2) & 1, sft = (c & 3) * 2;
    const float d = h2f(b + 80), dmin = h2f(b + 82);
    const uint8_t* q = b + 16 + half * 32;
#pragma unroll
    for (int part = 0; part < 2; ++part) {
      const int s = b[half * 8 + (c & 3) * 2 + part];
      const float dl = d * (float)(s & 15), ml = dmin * (float)(s >> 4);
#pragma unroll
      for (int l = 0; l < 16; ++l) w[part * 16 + l] = dl * (float)((q[part * 16 + l] >> sft) & 3) - ml;
    }
  } else if (TYPE == kQ3_K) {
    const uint8_t* b = row + (size_t)(c >> 3) * 110;
    const int half = (c >> 2) & 1, j4 = c & 3, sft = j4 * 2, bit = half * 4 + j4;
    const float d = h2f(b + 108);
    const uint8_t* hm = b;
    const uint8_t* q = b + 32 + half * 32;
    const uint8_t* s12 = b + 96;
#pragma unroll
    for (int part = 0; part < 2; ++part) {
      const int i = half * 8 + j4 * 2 + part;                 // scale index 0..15
      const int lo = i < 8 ? (s12[i] & 15) : (s12[i - 8] >> 4);
      const int hi = (s12[8 + (i & 3)] >> (2 * (i >> 2))) & 3;
      const float dl = d * (float)((lo | (hi << 4)) - 32);
#pragma unroll
      for (int l = 0; l < 16; ++l) {
        const int e = part * 16 + l;
        w[e] = dl * (float)((int)((q[e] >> sft) & 3) - (((hm[e] >> bit) & 1) ? 0 : 4));
      }
    }
  } else if (TYPE == kQ5_K) {
    const uint8_t* b = row + (size_t)(c >> 3) * 176;
    const int sb = c & 7;
    const float d = h2f(b), dmin = h2f(b + 2);
    int sc, mn;
    scale_min_k4(b + 4, sb, sc, mn);
    const float d1 = d * (float)sc, m1 = dmin * (float)mn;
    const uint8_t* qh = b + 16;
    const uint8_t* q = b + 48 + (sb >> 1) * 32;
    const int shift = (sb & 1) * 4;
#pragma unroll
    for (int j = 0; j < 32; ++j) w[j] = d1 * (float)(((q[j] >> shift) & 15) | (((qh[j] >> sb) & 1) << 4)) - m1;
  } else {  // Q6_K
    const uint8_t* b = row + (size_t)(c >> 3) * 210;
    const int sub = c & 7, half = sub >> 2, qtr = sub & 3;
    const uint8_t* ql = b + half * 64 + (qtr & 1) * 32;
    const uint8_t* qh = b + 128 + half * 32;
    const int8_t* sc = reinterpret_cast<const int8_t*>(b + 192) + half * 8 + qtr * 2;
    const float d = h2f(b + 208);
    const int lshift = (qtr >> 1) * 4, hshift = qtr * 2;
#pragma unroll
    for (int j = 0; j < 32; ++j) {
      const int q = (int)(((ql[j] >> lshift) & 15) | (((qh[j] >> hshift) & 3) << 4)) - 32;
      w[j] = d * (float)sc[j >> 4] * (float)q;
    }
  }
}

template <int TYPE>
__global__ void __launch_bounds__(256) gguf_gemv_kernel(const uint8_t* __restrict__ W, long row_bytes,
                                                        const __nv_bfloat16* __restrict__ x, long x_stride,
                                                        __nv_bfloat16* __restrict__ out, long out_stride,
                                                        float* __restrict__ out_f32, int M, int N, int K) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int n = blockIdx.x * 8 + warp;
  if (n >= N) return;
  const uint8_t* row = W + (size_t)n * row_bytes;
  float acc[16];
#pragma unroll
  for (int m = 0; m < 16; ++m) acc[m] = 0.f;
  const int chunks = K >> 5;
  for (int c = lane; c < chunks; c += 32) {
    float w[32];
    decode32<TYPE>(row, c, w);
#pragma unroll
    for (int m = 0; m < 16; ++m) {
      if (m >= M) break;
      const __nv_bfloat16* xr = x + (long)m * x_stride + (long)c * 32;
      float s = 0.f;
#pragma unroll
      for (int j = 0; j < 32; j += 8) {
        const bf16x8 t = *reinterpret_cast<const bf16x8*>(xr + j);
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const float2 f = __bfloat1622float2(t.v[u]);
          s = fmaf(w[j + 2 * u], f.x, s);
          s = fmaf(w[j + 2 * u + 1], f.y, s);
        }
      }
      acc[m] += s;
    }
  }
#pragma unroll
  for (int m = 0; m < 16; ++m) {
    if (m >= M) break;
    float v = warp_sum(acc[m]);
    if (lane == 0) {
      if (out_f32) out_f32[(long)m * out_stride + n] = v;
      else out[(long)m * out_stride + n] = f2bf(v);
    }
  }
}

// Routed experts stored as GGUF blocks (decode / verify rows): grid (output rows / 4 or / 8, routes), one warp per output
// row (FUSE: per gate / up pair, the gated activation applied before the store). W holds the experts of this rank back to
// back ([e_local][N][row_bytes]); route r reads activation row r / x_div and the expert ids[r] - e0; routes of experts
// that live elsewhere store zeros. The per-row sum runs in the order of the dense mat-vec (lane-strided 32-weight
// chunks, butterfly), so a route gives the same bits whatever else is in the batch.
template <int TYPE, int FUSE>
__global__ void __launch_bounds__(128) gguf_moe_gemv_kernel(const uint8_t* __restrict__ W, long row_bytes,
                                                            const int* __restrict__ ids, int e0, int e_local,
                                                            const __nv_bfloat16* __restrict__ x, long x_stride, int x_div,
                                                            __nv_bfloat16* __restrict__ out, long out_stride, int N, int K,
                                                            int act, float limit) {
  const int route = blockIdx.y;
  const int e = ids[route] - e0;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int half_n = N >> 1, n_out = FUSE ? half_n : N;
  const int r0 = blockIdx.x * 4 + warp;
  if (r0 >= n_out) return;
  if (e < 0 || e >= e_local) {
    if (lane == 0) out[(long)route * out_stride + r0] = f2bf(0.f);
    return;
  }
  const uint8_t* base = W + (size_t)e * N * row_bytes;
  const uint8_t* row0 = base + (size_t)r0 * row_bytes;
  const uint8_t* row1 = base + (size_t)(FUSE ? r0 + half_n : r0) * row_bytes;
  const __nv_bfloat16* xr = x + (long)(route / x_div) * x_stride;
  float acc0 = 0.f, acc1 = 0.f;
  const int chunks = K >> 5;
  for (int c = lane; c < chunks; c += 32) {
    float xv[32];
#pragma unroll
    for (int j = 0; j < 32; j += 8) {
      const bf16x8 t = *reinterpret_cast<const bf16x8*>(xr + (long)c * 32 + j);
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const float2 f = __bfloat1622float2(t.v[u]);
        xv[j + 2 * u] = f.x;
        xv[j + 2 * u + 1] = f.y;
      }
    }
    float w[32];
    decode32<TYPE>(row0, c, w);
    float s = 0.f;
#pragma unroll
    for (int j = 0; j < 32; ++j) s = fmaf(w[j], xv[j], s);
    acc0 += s;
    if (FUSE) {
      decode32<TYPE>(row1, c, w);
      s = 0.f;
#pragma unroll
      for (int j = 0; j < 32; ++j) s = fmaf(w[j], xv[j], s);
      acc1 += s;
    }
  }
  acc0 = warp_sum(acc0);
  if (FUSE) acc1 = warp_sum(acc1);
  if (lane != 0) return;
  if (FUSE) {
    // the unfused pair rounds both projections to bf16 before the activation: the same rounding points here
    float gate = bf2f(f2bf(acc0)), up = bf2f(f2bf(acc1));
    if (limit > 0.f) { gate = fminf(gate, limit); up = fminf(fmaxf(up, -limit), limit); }
    const float a = act ? 0.5f * gate * (1.f + tanhf(0.7978845608028654f * (gate + 0.044715f * gate * gate * gate)))
                        : gate / (1.f + __expf(-gate));
    out[(long)route * out_stride + r0] = f2bf(a * up);
  } else {
    out[(long)route * out_stride + r0] = f2bf(acc0);
  }
}

template <int TYPE>
__global__ void gguf_dequant_kernel(const uint8_t* __restrict__ W, long row_bytes, __nv_bfloat16* __restrict__ out,
                                    long N, int K) {
  const int chunks = K >> 5;
  const long total = N * chunks;
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < total; i += (long)gridDim.x * blockDim.x) {
    const long n = i / chunks;
    const int c = (int)(i % chunks);
    float w[32];
    decode32<TYPE>(W + (size_t)n * row_bytes, c, w);
    __nv_bfloat16* o = out + n * (long)K + (long)c * 32;
#pragma unroll
    for (int j = 0; j < 32; j += 2) *reinterpret_cast<__nv_bfloat162*>(o + j) = __floats2bfloat162_rn(w[j], w[j + 1]);
  }
}

}  // namespace ve

using namespace ve;

// which devices have had their grid table set (a codebook format launched without it would read through a null pointer)
static bool g_iq_ready[64];

static bool iq_type(int t) {
  return t == kIQ2_XXS || t == kIQ2_XS || t == kIQ2_S || t == kIQ3_XXS || t == kIQ3_S || t == kIQ1_S || t == kIQ1_M;
}
static bool iq_ready() {
  int dev = 0;
  return cudaGetDevice(&dev) == cudaSuccess && dev >= 0 && dev < 64 && g_iq_ready[dev];
}

extern "C" {

// `table`: device copy (on the current device, 16-byte aligned, 33920 bytes) of the grid file; it must outlive every launch.
int ve_gguf_set_iq_grids(const void* table) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= 64 || !table || ((uintptr_t)table & 15)) return cudaErrorInvalidValue;
  e = cudaMemcpyToSymbol(kIqGrids, &table, sizeof(table));
  if (e != cudaSuccess) return (int)e;
  g_iq_ready[dev] = true;
  return 0;
}

int ve_gguf_gemv(const void* W, int ggml_type, long row_bytes, const void* x, long x_stride, void* out, long out_stride,
                 int out_is_f32, int M, int N, int K, cudaStream_t st) {
  if (M <= 0 || M > 16 || N <= 0 || K % 32) return cudaErrorInvalidValue;
  if (ggml_type >= kQ2_K && ggml_type != kIQ4_NL && K % 256) return cudaErrorInvalidValue;
  if (iq_type(ggml_type) && !iq_ready()) return cudaErrorNotReady;
  const int blocks = (N + 7) / 8;
  __nv_bfloat16* ob = out_is_f32 ? nullptr : (__nv_bfloat16*)out;
  float* of = out_is_f32 ? (float*)out : nullptr;
#define VE_GG(T)                                                                                                  \
  gguf_gemv_kernel<T><<<blocks, 256, 0, st>>>((const uint8_t*)W, row_bytes, (const __nv_bfloat16*)x, x_stride, ob, \
                                              out_stride, of, M, N, K)
  switch (ggml_type) {
    case kQ8_0: VE_GG(kQ8_0); break;
    case kQ4_0: VE_GG(kQ4_0); break;
    case kQ4_K: VE_GG(kQ4_K); break;
    case kQ6_K: VE_GG(kQ6_K); break;
    case kQ4_1: VE_GG(kQ4_1); break;
    case kQ5_0: VE_GG(kQ5_0); break;
    case kQ5_1: VE_GG(kQ5_1); break;
    case kQ2_K: VE_GG(kQ2_K); break;
    case kQ3_K: VE_GG(kQ3_K); break;
    case kQ5_K: VE_GG(kQ5_K); break;
    case kIQ4_NL: VE_GG(kIQ4_NL); break;
    case kIQ4_XS: VE_GG(kIQ4_XS); break;
    case kIQ2_XXS: VE_GG(kIQ2_XXS); break;
    case kIQ2_XS: VE_GG(kIQ2_XS); break;
    case kIQ2_S: VE_GG(kIQ2_S); break;
    case kIQ3_XXS: VE_GG(kIQ3_XXS); break;
    case kIQ3_S: VE_GG(kIQ3_S); break;
    case kIQ1_S: VE_GG(kIQ1_S); break;
    case kIQ1_M: VE_GG(kIQ1_M); break;
    default: return cudaErrorInvalidValue;
  }
#undef VE_GG
  VE_CHECK_LAUNCH();
}

// Routed-expert mat-vec over GGUF blocks; see gguf_moe_gemv_kernel. fuse_act: W rows are [gate (N/2) | up (N/2)] and the
// output has N/2 columns act(gate) * up (act 0 SiLU, 1 tanh-GELU; limit > 0 clamps gate from above and up to +-limit).
int ve_gguf_moe_gemv(const void* W, int ggml_type, long row_bytes, const void* ids, int e0, int e_local, const void* x,
                     long x_stride, int x_div, void* out, long out_stride, int routes, int N, int K, int fuse_act, int act,
                     float limit, cudaStream_t st) {
  if (routes <= 0) return 0;
  if (N <= 0 || K % 32 || x_div <= 0 || (fuse_act && N % 2)) return cudaErrorInvalidValue;
  if (ggml_type >= kQ2_K && ggml_type != kIQ4_NL && K % 256) return cudaErrorInvalidValue;
  if (iq_type(ggml_type) && !iq_ready()) return cudaErrorNotReady;
  const int outs = fuse_act ? N / 2 : N;
  const dim3 grid((outs + 3) / 4, routes);
#define VE_GM(T)                                                                                                       \
  do {                                                                                                                 \
    if (fuse_act)                                                                                                      \
      gguf_moe_gemv_kernel<T, 1><<<grid, 128, 0, st>>>((const uint8_t*)W, row_bytes, (const int*)ids, e0, e_local,       \
                                                       (const __nv_bfloat16*)x, x_stride, x_div, (__nv_bfloat16*)out,    \
                                                       out_stride, N, K, act, limit);                                    \
    else                                                                                                               \
      gguf_moe_gemv_kernel<T, 0><<<grid, 128, 0, st>>>((const uint8_t*)W, row_bytes, (const int*)ids, e0, e_local,       \
                                                       (const __nv_bfloat16*)x, x_stride, x_div, (__nv_bfloat16*)out,    \
                                                       out_stride, N, K, act, limit);                                    \
  } while (0)
  switch (ggml_type) {
    case kQ8_0: VE_GM(kQ8_0); break;
    case kQ4_0: VE_GM(kQ4_0); break;
    case kQ4_K: VE_GM(kQ4_K); break;
    case kQ6_K: VE_GM(kQ6_K); break;
    case kQ4_1: VE_GM(kQ4_1); break;
    case kQ5_0: VE_GM(kQ5_0); break;
    case kQ5_1: VE_GM(kQ5_1); break;
    case kQ2_K: VE_GM(kQ2_K); break;
    case kQ3_K: VE_GM(kQ3_K); break;
    case kQ5_K: VE_GM(kQ5_K); break;
    case kIQ4_NL: VE_GM(kIQ4_NL); break;
    case kIQ4_XS: VE_GM(kIQ4_XS); break;
    case kIQ2_XXS: VE_GM(kIQ2_XXS); break;
    case kIQ2_XS: VE_GM(kIQ2_XS); break;
    case kIQ2_S: VE_GM(kIQ2_S); break;
    case kIQ3_XXS: VE_GM(kIQ3_XXS); break;
    case kIQ3_S: VE_GM(kIQ3_S); break;
    case kIQ1_S: VE_GM(kIQ1_S); break;
    case kIQ1_M: VE_GM(kIQ1_M); break;
    default: return cudaErrorInvalidValue;
  }
#undef VE_GM
  VE_CHECK_LAUNCH();
}

int ve_gguf_dequant(const void* W, int ggml_type, long row_bytes, void* out, long N, int K, cudaStream_t st) {
  if (N <= 0 || K % 32) return cudaErrorInvalidValue;
  if (ggml_type >= kQ2_K && ggml_type != kIQ4_NL && K % 256) return cudaErrorInvalidValue;
  if (iq_type(ggml_type) && !iq_ready()) return cudaErrorNotReady;
  const long total = N * (K / 32);
  const int blocks = (int)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
#define VE_GD(T) gguf_dequant_kernel<T><<<blocks, 256, 0, st>>>((const uint8_t*)W, row_bytes, (__nv_bfloat16*)out, N, K)
  switch (ggml_type) {
    case kQ8_0: VE_GD(kQ8_0); break;
    case kQ4_0: VE_GD(kQ4_0); break;
    case kQ4_K: VE_GD(kQ4_K); break;
    case kQ6_K: VE_GD(kQ6_K); break;
    case kQ4_1: VE_GD(kQ4_1); break;
    case kQ5_0: VE_GD(kQ5_0); break;
    case kQ5_1: VE_GD(kQ5_1); break;
    case kQ2_K: VE_GD(kQ2_K); break;
    case kQ3_K: VE_GD(kQ3_K); break;
    case kQ5_K: VE_GD(kQ5_K); break;
    case kIQ4_NL: VE_GD(kIQ4_NL); break;
    case kIQ4_XS: VE_GD(kIQ4_XS); break;
    case kIQ2_XXS: VE_GD(kIQ2_XXS); break;
    case kIQ2_XS: VE_GD(kIQ2_XS); break;
    case kIQ2_S: VE_GD(kIQ2_S); break;
    case kIQ3_XXS: VE_GD(kIQ3_XXS); break;
    case kIQ3_S: VE_GD(kIQ3_S); break;
    case kIQ1_S: VE_GD(kIQ1_S); break;
    case kIQ1_M: VE_GD(kIQ1_M); break;
    default: return cudaErrorInvalidValue;
  }
#undef VE_GD
  VE_CHECK_LAUNCH();
}

}  // extern "C"
