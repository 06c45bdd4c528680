// Quantise-on-store for the scaled KV cache formats. The rotation kernel leaves rotated keys (and untouched values) in the
// fused qkv buffer; this kernel encodes one (row, kv head, K or V) per CTA into the paged byte pools and their scale pools.
//   I8   one byte per element, one fp16 scale per 64 elements (amax / 127)
//   Q4   4 bits per element (value + 8, low nibble = even element), one fp16 scale per 64 (amax / 7), after an orthonormal
//        64-point Walsh-Hadamard rotation of the 64 elements
//   FP4  E2M1 per element, one E4M3 scale byte per 16 elements (amax / 6)
// Format 2 = k8v4 (I8 keys, Q4 values), 3 = nvfp4 (FP4 both). A thread encodes one whole unit (64 or 16 elements).
// Reference: inc/engine/core/kv_format.h:9-18, src/backend/cuda/modules/kv_quant.cuh:166-246 (kv_store_unit, kv_fwht64).
#include "common.cuh"
#include <cuda_fp8.h>

namespace ve {

constexpr int kPageTokQ = 64;

VE_DEVINL void fwht64(float* v) {
#pragma unroll
  for (int h = 1; h < 64; h <<= 1) {
#pragma unroll
    for (int i = 0; i < 64; ++i) {
      if ((i & h) == 0) {
        const float a = v[i], b = v[i | h];
        v[i] = a + b;
        v[i | h] = a - b;
      }
    }
  }
#pragma unroll
  for (int i = 0; i < 64; ++i) v[i] *= 0.125f;
}

VE_DEVINL uint32_t e2m1_code(float x) {   // round to nearest (ties to even code), saturating at +-6
  const float a = fabsf(x);
  uint32_t c;
  if (a <= 0.25f) c = 0;
  else if (a < 0.75f) c = 1;
  else if (a <= 1.25f) c = 2;
  else if (a < 1.75f) c = 3;
  else if (a <= 2.5f) c = 4;
  else if (a < 3.5f) c = 5;
  else if (a <= 5.0f) c = 6;
  else c = 7;
  return c | (x < 0.f && c ? 8u : 0u);
}

// grid (rows, nkv, 2): z = 0 keys, 1 values. block 32: thread u encodes unit u.
__global__ void __launch_bounds__(32) kv_quant_store_kernel(const __nv_bfloat16* __restrict__ qkv, long q_stride,
                                                            const int* __restrict__ pos, const int* __restrict__ slot,
                                                            const int* __restrict__ page_table, int max_pages,
                                                            uint8_t* __restrict__ kpool, uint8_t* __restrict__ vpool,
                                                            uint8_t* __restrict__ kscale, uint8_t* __restrict__ vscale,
                                                            int nq, int nkv, int hd, int fmt) {
  grid_dep_wait();
  const int row = blockIdx.x, kvh = blockIdx.y, isv = blockIdx.z, u = threadIdx.x;
  const int s = slot ? slot[row] : 0;
  if (s < 0) return;
  const int p = pos[row];
  const int page = page_table[(long)s * max_pages + p / kPageTokQ];
  const long tok = ((long)page * nkv + kvh) * kPageTokQ + (p % kPageTokQ);
  const __nv_bfloat16* src = qkv + (long)row * q_stride + (long)(nq + (isv ? nkv : 0) + kvh) * hd;
  const int codec = fmt == 2 ? (isv ? 3 : 2) : 4;      // 2 I8, 3 Q4, 4 FP4
  uint8_t* data = isv ? vpool : kpool;
  uint8_t* sc = isv ? vscale : kscale;
  if (codec == 4) {
    if (u >= hd / 16) return;
    float v[16], amax = 0.f;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      v[i] = __bfloat162float(src[u * 16 + i]);
      amax = fmaxf(amax, fabsf(v[i]));
    }
    const __nv_fp8_storage_t sb = __nv_cvt_float_to_fp8(amax / 6.f, __NV_SATFINITE, __NV_E4M3);
    const float sf = __half2float(__half(__nv_cvt_fp8_to_halfraw(sb, __NV_E4M3)));
    const float inv = sf > 0.f ? 1.f / sf : 0.f;
    sc[tok * (hd / 16) + u] = (uint8_t)sb;
    uint8_t* d = data + tok * (hd / 2) + u * 8;
#pragma unroll
    for (int i = 0; i < 16; i += 2) d[i >> 1] = (uint8_t)(e2m1_code(v[i] * inv) | (e2m1_code(v[i + 1] * inv) << 4));
    return;
  }
  if (u >= hd / 64) return;
  float v[64], amax = 0.f;
#pragma unroll
  for (int i = 0; i < 64; ++i) v[i] = __bfloat162float(src[u * 64 + i]);
  if (codec == 3) fwht64(v);
#pragma unroll
  for (int i = 0; i < 64; ++i) amax = fmaxf(amax, fabsf(v[i]));
  const __half sh = __float2half_rn(amax / (codec == 2 ? 127.f : 7.f));
  const float sf = __half2float(sh);
  const float inv = sf > 0.f ? 1.f / sf : 0.f;
  reinterpret_cast<__half*>(sc)[tok * (hd / 64) + u] = sh;
  if (codec == 2) {
    int8_t* d = reinterpret_cast<int8_t*>(data) + tok * hd + u * 64;
#pragma unroll
    for (int i = 0; i < 64; ++i) d[i] = (int8_t)max(-127, min(127, __float2int_rn(v[i] * inv)));
  } else {
    uint8_t* d = data + tok * (hd / 2) + u * 32;
#pragma unroll
    for (int i = 0; i < 64; i += 2) {
      const int lo = max(-8, min(7, __float2int_rn(v[i] * inv))) + 8;
      const int hi = max(-8, min(7, __float2int_rn(v[i + 1] * inv))) + 8;
      d[i >> 1] = (uint8_t)(lo | (hi << 4));
    }
  }
}

}  // namespace ve

using namespace ve;

extern "C" {

int ve_kv_quant_store(const void* qkv, long q_stride, const void* pos, const void* slot, const void* page_table,
                      int max_pages, void* kpool, void* vpool, void* kscale, void* vscale, int rows, int nq, int nkv,
                      int hd, int fmt, cudaStream_t st) {
  if (rows <= 0) return 0;
  if ((fmt != 2 && fmt != 3) || hd % 64 || hd > 512) return cudaErrorInvalidValue;
  launch_pdl(kv_quant_store_kernel, dim3(rows, nkv, 2), dim3(32), 0, st, (const __nv_bfloat16*)qkv, q_stride, (const int*)pos,
             (const int*)slot, (const int*)page_table, max_pages, (uint8_t*)kpool, (uint8_t*)vpool, (uint8_t*)kscale,
             (uint8_t*)vscale, nq, nkv, hd, fmt);
  VE_CHECK_LAUNCH();
}

}  // extern "C"
