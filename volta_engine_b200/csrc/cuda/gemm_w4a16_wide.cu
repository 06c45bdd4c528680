// Prefill linear with NVFP4 weights and bf16 activations on 256 x 256 output tiles:
//   out[t, n] = alpha * sum_k W[n, k] * X[t, k],   W dequantised to bf16 inside the tile loader (exact products).
//
// Why a second W4A16 kernel: with one 128-feature tile per CTA every CTA pulls its own 256-token activation tile, 576
// bytes per k for 65 kFLOP, which at the tensor peak would need 12 TB/s from L2, and the 106 KB stages leave room for
// only two in flight, so the loop waits on TMA latency (0.33-0.43 of the measured bf16 peak). Here a CTA owns two
// 128-feature tiles that share one activation tile: 640 bytes per k for 131 kFLOP (205 FLOP/B), two accumulators of 256
// TMEM columns, 64-wide k steps of 74 KB so three stages fit, and the dequantising warps stay one stage ahead of the MMA.
// Warp roles (192 threads): warp 0 TMA producer, warp 1 TMEM owner + MMA issuer, warps 2..5 dequantise the two
// weight sub-tiles of each stage into swizzled bf16 and run the epilogue. Every wait is bounded.
// Reference kernel family this replaces: src/kernels/cuda/nvfp4/skinny_kernels.cu:531-558 (fused WMMA GEMM / dequant + HGEMM).
#include "common.cuh"
#include "tmap.h"

namespace ve {

struct WideParams {
  int N, T, K;
  float alpha;
  __nv_bfloat16* out;
  long ldo;
  const __nv_bfloat16* residual;
  long ldr;
  const uint8_t* sfa;     // [N/128][K/128][128][8] E4M3 scales
  int* status;
};

VE_DEVINL void w_e2m1x8_to_bf16x8(uint32_t w, uint32_t* o) {
  // table lookup on the byte-permute unit: bf16 patterns of {0, .5, 1, 1.5, 2, 3, 4, 6}
  const uint32_t mags = w & 0x77777777u, sg = (w >> 3) & 0x11111111u;
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const uint32_t sel = mags >> (16 * h), ssel = sg >> (16 * h);
    const uint32_t lo4 = __byte_perm(0xC0800000u, 0xC0804000u, sel);
    const uint32_t hi4 = __byte_perm(0x3F3F3F00u, 0x40404040u, sel) | __byte_perm(0x00008000u, 0u, ssel);
    o[2 * h] = __byte_perm(lo4, hi4, 0x5140);
    o[2 * h + 1] = __byte_perm(lo4, hi4, 0x7362);
  }
}
VE_DEVINL uint32_t w_e4m3_to_bf16x2_dup(uint32_t byte) {
  uint32_t r;
  asm("{ .reg .b16 t; cvt.u16.u32 t, %1; cvt.rn.f16x2.e4m3x2 %0, t; }" : "=r"(r) : "r"(byte | (byte << 8)));
  const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&r));
  const __nv_bfloat162 b = __floats2bfloat162_rn(f.x, f.y);
  return *reinterpret_cast<const uint32_t*>(&b);
}

constexpr int W_KT = 64, W_RAW = 128 * 32, W_DEQ = 128 * 128, W_B = 256 * 128, W_SF = 1024;
constexpr int W_STAGE = 2 * W_RAW + 2 * W_DEQ + W_B + 2 * W_SF;      // 75776
constexpr int W_STAGES = 3;
constexpr int W_SMEM = W_STAGES * W_STAGE + 1024;

__global__ void __launch_bounds__(192, 1)
gemm_w4a16_wide_kernel(const WideParams p, const __grid_constant__ CUtensorMap amap, const __grid_constant__ CUtensorMap bmap) {
  static_assert(W_STAGE % 1024 == 0, "stage must keep 1024 B alignment");
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  __shared__ uint64_t full[W_STAGES], empty[W_STAGES], deq[W_STAGES], acc_full;
  __shared__ uint32_t tmem_holder;
  __shared__ int s_fail;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n0 = blockIdx.x * 256, t0 = blockIdx.y * 256;
  const int nkt = p.K / W_KT;
  if (threadIdx.x == 0) {
    for (int s = 0; s < W_STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); mbar_init(&deq[s], 4); }
    mbar_init(&acc_full, 1);
    s_fail = 0;
    mbar_fence_init();
  }
  if (warp == 1) { tmem_alloc(&tmem_holder, 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_holder;
  auto stage_ptr = [&](int s) { return smem + (size_t)s * W_STAGE; };   // [RAW0][RAW1][DEQ0][DEQ1][B][SF0][SF1]
  constexpr int OFF_DEQ = 2 * W_RAW, OFF_B = OFF_DEQ + 2 * W_DEQ, OFF_SF = OFF_B + W_B;

  if (warp == 0) {
    if (elect_one()) {
      prefetch_tmap(&amap);
      prefetch_tmap(&bmap);
      for (int kt = 0; kt < nkt; ++kt) {
        const int s = kt % W_STAGES;
        if (!mbar_wait(&empty[s], ((kt / W_STAGES) & 1) ^ 1)) { atomicExch(&s_fail, 1); break; }
        uint8_t* st = stage_ptr(s);
        mbar_expect_tx(&full[s], 2 * W_RAW + W_B + 2 * W_SF);
        tma_load_2d(st, &amap, &full[s], kt * 32, n0);
        tma_load_2d(st + W_RAW, &amap, &full[s], kt * 32, n0 + 128);
        tma_load_2d(st + OFF_B, &bmap, &full[s], kt * W_KT, t0);
        const size_t blk = (size_t)(p.K / 128);
        bulk_load(st + OFF_SF, p.sfa + ((size_t)(blockIdx.x * 2) * blk + (kt >> 1)) * 1024, W_SF, &full[s]);
        bulk_load(st + OFF_SF + W_SF, p.sfa + ((size_t)(blockIdx.x * 2 + 1) * blk + (kt >> 1)) * 1024, W_SF, &full[s]);
      }
    }
  } else if (warp == 1) {
    if (elect_one()) {
      constexpr uint32_t idesc = make_idesc_f16(1, 1, 128, 256);
      bool ok = true;
      for (int kt = 0; kt < nkt && ok; ++kt) {
        const int s = kt % W_STAGES;
        ok = mbar_wait(&deq[s], (kt / W_STAGES) & 1);     // the dequantisers waited for the stage's bytes themselves
        if (!ok) break;
        tc_fence_after();
        uint8_t* st = stage_ptr(s);
        const uint64_t bd = make_desc_sw128(smem_u32(st + OFF_B));
#pragma unroll
        for (int sub = 0; sub < 2; ++sub) {
          const uint64_t ad = make_desc_sw128(smem_u32(st + OFF_DEQ + sub * W_DEQ));
#pragma unroll
          for (int kb = 0; kb < 4; ++kb)
            tc_mma_f16(tmem_base + sub * 256, ad + kb * 2, bd + kb * 2, idesc, (kt | kb) ? 1u : 0u);
        }
        tc_commit(&empty[s]);
      }
      if (!ok) atomicExch(&s_fail, 1);
      tc_commit(&acc_full);
    }
  } else {
    const int etid = (warp - 2) * 32 + lane;      // 0..127
    bool okd = true;
    for (int kt = 0; kt < nkt && okd; ++kt) {
      const int s = kt % W_STAGES;
      okd = mbar_wait(&full[s], (kt / W_STAGES) & 1);
      if (!okd) break;
      uint8_t* st = stage_ptr(s);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int q = etid + i * 128;               // 16 B chunk: sub-tile q/256, row (q%256)/2, 32 elements at (q%2)*32
        const int sub = q >> 8, row = (q & 255) >> 1, part = q & 1;
        const uint4 w = *reinterpret_cast<const uint4*>(st + sub * W_RAW + row * 32 + part * 16);
        const uint32_t words[4] = {w.x, w.y, w.z, w.w};
        const uint32_t s2 = *reinterpret_cast<const unsigned short*>(st + OFF_SF + sub * W_SF + row * 8 + (kt & 1) * 4 + part * 2);
        const uint32_t sca = w_e4m3_to_bf16x2_dup(s2 & 0xffu), scb = w_e4m3_to_bf16x2_dup(s2 >> 8);
        uint8_t* dq = st + OFF_DEQ + sub * W_DEQ + row * 128;
#pragma unroll
        for (int j = 0; j < 4; ++j) {               // 8 elements -> one 16 B chunk of bf16
          const uint32_t scale = j < 2 ? sca : scb;
          uint32_t o4[4];
          w_e2m1x8_to_bf16x8(words[j], o4);
#pragma unroll
          for (int b = 0; b < 4; ++b) {
            // code x scale has <= 6 significant bits: the bf16 product is exact
            const __nv_bfloat162 r = __hmul2(*reinterpret_cast<const __nv_bfloat162*>(&o4[b]),
                                             *reinterpret_cast<const __nv_bfloat162*>(&scale));
            o4[b] = *reinterpret_cast<const uint32_t*>(&r);
          }
          const int ch = part * 4 + j;                // 16 B chunk along the 64-wide k step
          *reinterpret_cast<uint4*>(dq + ((ch ^ (row & 7)) << 4)) = make_uint4(o4[0], o4[1], o4[2], o4[3]);
        }
      }
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(&deq[s]);
    }
    if (!okd) atomicExch(&s_fail, 1);
    // epilogue: TMEM lane = output feature, column = token; two accumulators
    const bool ok = mbar_wait(&acc_full, 0);
    if (!ok) atomicExch(&s_fail, 1);
    tc_fence_after();
    if (ok && !s_fail) {
      const int q = warp & 3;
#pragma unroll 1
      for (int sub = 0; sub < 2; ++sub) {
        const int n = n0 + sub * 128 + q * 32 + lane;
#pragma unroll 1
        for (int c0 = 0; c0 < 256; c0 += 16) {
          if (t0 + c0 >= p.T) break;
          uint32_t r[16];
          tmem_ld16(tmem_base + ((uint32_t)(q * 32) << 16) + sub * 256 + c0, r);
          tmem_ld_wait();
          if (n < p.N) {
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              const int t = t0 + c0 + j;
              if (t < p.T) {
                float v = __uint_as_float(r[j]) * p.alpha;
                if (p.residual) v += bf2f(p.residual[(long)t * p.ldr + n]);
                p.out[(long)t * p.ldo + n] = f2bf(v);
              }
            }
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem_base, 512); }
  if (threadIdx.x == 0 && s_fail && p.status) atomicExch(p.status, (int)kErrMbarTimeout);
}

}  // namespace ve

using namespace ve;

extern "C" {

// Wp [N, K/2] bytes, sfa [N/128][K/128][128][8], X [T, K] bf16 (pitch ldx). N % 256 == 0, K % 128 == 0.
int ve_gemm_w4a16_wide(const void* Wp, const void* sfa, const void* X, long ldx, void* out, long ldo, const void* residual,
                       long ldr, int T, int N, int K, float alpha, void* status, cudaStream_t st) {
  if (T <= 0 || N <= 0) return 0;
  if (N % 256 || K % 128) return cudaErrorInvalidValue;
  CUtensorMap amap, bmap;
  int rc = make_tmap_2d(&amap, Wp, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, N, K / 2, (uint64_t)K / 2, 128, 32, CU_TENSOR_MAP_SWIZZLE_NONE);
  if (rc) return rc;
  rc = make_tmap_2d(&bmap, X, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, T, K, (uint64_t)ldx * 2, 256, 64, CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc) return rc;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(gemm_w4a16_wide_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, W_SMEM);
    if (e != cudaSuccess) return (int)e;
    attr_set = true;
  }
  WideParams p{N, T, K, alpha, (__nv_bfloat16*)out, ldo, (const __nv_bfloat16*)residual, ldr, (const uint8_t*)sfa, (int*)status};
  dim3 grid(N / 256, (T + 255) / 256);
  gemm_w4a16_wide_kernel<<<grid, 192, W_SMEM, st>>>(p, amap, bmap);
  return (int)cudaGetLastError();
}

}  // extern "C"
