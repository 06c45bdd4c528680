// GGUF block formats: dequantisation fused into the mat-vec (decode / verify rows, M <= 16) and a plain
// dequantise-to-bf16 kernel that feeds the tcgen05 GEMM for prefill chunks.
//   Q8_0, Q4_0, Q4_1, Q5_0, Q5_1, IQ4_NL (32-value blocks) and Q2_K, Q3_K, Q4_K, Q5_K, Q6_K, IQ4_XS (256-value
//   super-blocks), bf16 activations, fp32 accumulation.
// One warp per output row; a lane decodes 32 consecutive weights at a time straight from the packed row and
// multiplies them with the activations of every batch row, so the weights are read exactly once.
// Summation order per row is fixed (lane-strided chunks, then a butterfly), independent of M.
// Reference counterparts: src/kernels/cuda/gguf/gguf_linear.cu:38-160 (gemv on q8_1 activations) and the
// vendored dequantize kernels; block layouts as in quant/gguf.py.
#include "common.cuh"

namespace ve {

enum GgmlType { kQ4_0 = 2, kQ4_1 = 3, kQ5_0 = 6, kQ5_1 = 7, kQ8_0 = 8, kQ2_K = 10, kQ3_K = 11, kQ4_K = 12, kQ5_K = 13,
                kQ6_K = 14, kIQ4_NL = 20, kIQ4_XS = 23 };

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

extern "C" {

int ve_gguf_gemv(const void* W, int ggml_type, long row_bytes, const void* x, long x_stride, void* out, long out_stride,
                 int out_is_f32, int M, int N, int K, cudaStream_t st) {
  if (M <= 0 || M > 16 || N <= 0 || K % 32) return cudaErrorInvalidValue;
  if (ggml_type >= kQ2_K && ggml_type != kIQ4_NL && K % 256) return cudaErrorInvalidValue;
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
    default: return cudaErrorInvalidValue;
  }
#undef VE_GG
  VE_CHECK_LAUNCH();
}

int ve_gguf_dequant(const void* W, int ggml_type, long row_bytes, void* out, long N, int K, cudaStream_t st) {
  if (N <= 0 || K % 32) return cudaErrorInvalidValue;
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
    default: return cudaErrorInvalidValue;
  }
#undef VE_GD
  VE_CHECK_LAUNCH();
}

}  // extern "C"
