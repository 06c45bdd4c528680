// Tensor-core linear layers on tcgen05 / TMEM, fed by TMA:   out[t, n] = alpha * sum_k W[n, k] * X[t, k]
//
// The weight matrix is always the UMMA "A" operand (M = 128 output features per CTA, one TMEM lane per
// feature) and the activations are the "B" operand (N = BN tokens, 16..256), so the same kernel covers
// decode / verify blocks (BN = 16) and prefill chunks (BN = 256) and weights are streamed exactly once
// per token tile. Three operand modes:
//   MODE 0  bf16 weights x bf16 activations                         (kind::f16)
//   MODE 1  NVFP4 weights dequantised to bf16 in the tile loader x bf16 activations  (kind::f16, W4A16)
//   MODE 2  NVFP4 weights x NVFP4 activations, native block scaling  (kind::mxf4nvf4, UE4M3 per 16)
// NVFP4 = E2M1 codes (low nibble = even k) with one E4M3 scale per 16 elements and an fp32 tensor scale
// (reference decode rule: inc/engine/quant/fp4_fp8.h:14-40; reference kernels it replaces:
// src/kernels/cuda/nvfp4/skinny_kernels.cu:445-562 and src/kernels/cuda/gemm/gemm_f16.cu).
//
// Warp roles (192 threads): warp 0 = TMA producer, warp 1 = TMEM owner + MMA issuer, warps 2..5 =
// dequantisers during the main loop (MODE 1) and epilogue (TMEM -> registers -> global) at the end.
// Every mbarrier wait is bounded; on expiry the kernel records a status code and drains.
#include "common.cuh"
#include "tmap.h"

namespace ve {

struct GemmParams {
  int N, T, K;            // out features, tokens, reduction
  float alpha;            // tensor scale (weights' global scale x activations' global scale)
  __nv_bfloat16* out;     // [T, ldo]
  long ldo;
  const __nv_bfloat16* residual;  // optional [T, ldr]
  long ldr;
  float* out_f32;         // optional fp32 output instead of bf16 (LM head)
  const uint8_t* sfa;     // MODE 1: [N/128][K/128][128][8]; MODE 2: [N/128][K/64][512]
  const uint8_t* sfb;     // MODE 2: [ceil(T/128)][K/64][512]
  int* status;
  // Grouped (mixture-of-experts) form: weights of all experts stacked along N, activation rows sorted by
  // expert. tile_tab[tile] = {expert, first row, row count, 0}; blockIdx.y indexes tiles (count 0 = idle).
  const int* tile_tab;        // null for the plain GEMM
  int n_per_expert;           // rows of one expert inside the stacked weight
  const float* alpha_tab;     // per-expert tensor scale (null: alpha)
  int n_tiles;                // grid.y of the grouped form
};

template <int MODE>
struct GemmCfg {
  static constexpr int KT = MODE == 2 ? 256 : (MODE == 1 ? 128 : 64);  // K elements per stage
};

VE_DEVINL uint32_t e2m1x2_to_f16x2(uint32_t byte) {
  uint32_t r;
  asm("{ .reg .b8 t; cvt.u8.u32 t, %1; cvt.rn.f16x2.e2m1x2 %0, t; }" : "=r"(r) : "r"(byte));
  return r;
}
// Eight E2M1 codes (nibble i = element i) -> four bf16x2 words, by table lookup on the byte-permute unit instead of
// conversion instructions: the bf16 patterns of {0, .5, 1, 1.5, 2, 3, 4, 6} are 0x0000 3F00 3F80 3FC0 4000 4040 4080
// 40C0; prmt picks their low and high bytes with the codes' magnitudes as selector, a third lookup turns the sign
// bits into 0x80 bytes, and two more permutes interleave low and high bytes.
VE_DEVINL void e2m1x8_to_bf16x8(uint32_t w, uint32_t* o) {
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
VE_DEVINL uint32_t e4m3_to_bf16x2_dup(uint32_t byte) {  // both halves = the scale (exact: 3 mantissa bits)
  uint32_t r;
  asm("{ .reg .b16 t; cvt.u16.u32 t, %1; cvt.rn.f16x2.e4m3x2 %0, t; }" : "=r"(r) : "r"(byte | (byte << 8)));
  const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&r));
  const __nv_bfloat162 b = __floats2bfloat162_rn(f.x, f.y);
  return *reinterpret_cast<const uint32_t*>(&b);
}
VE_DEVINL uint32_t e4m3_to_f16x2_dup(uint32_t byte) {  // both halves = the scale
  uint32_t r;
  asm("{ .reg .b16 t; cvt.u16.u32 t, %1; cvt.rn.f16x2.e4m3x2 %0, t; }" : "=r"(r) : "r"(byte | (byte << 8)));
  return r;
}

template <int MODE, int BN, int STAGES>
__global__ void __launch_bounds__(192, 1)
gemm_kernel(const GemmParams p, const __grid_constant__ CUtensorMap amap, const __grid_constant__ CUtensorMap bmap) {
  constexpr int KT = GemmCfg<MODE>::KT;
  constexpr int A_RAW = MODE == 0 ? 128 * 128 : (MODE == 1 ? 128 * 64 : 128 * 128);  // bytes via TMA
  constexpr int A_DEQ = MODE == 1 ? 128 * 256 : 0;                                    // f16 tile, 2 sub-tiles
  constexpr int B_SUB = BN * 128;                                                     // one 128 B-wide sub-tile
  constexpr int B_NSUB = MODE == 1 ? 2 : 1;
  constexpr int B_BYTES = B_SUB * B_NSUB;
  constexpr int SFA_BYTES = MODE == 1 ? 1024 : (MODE == 2 ? 2048 : 0);
  constexpr int NB128 = (BN + 127) / 128;
  constexpr int SFB_BYTES = MODE == 2 ? 2048 * NB128 : 0;
  constexpr int STAGE_BYTES = A_RAW + A_DEQ + B_BYTES + SFA_BYTES + SFB_BYTES;
  constexpr int ACC_COLS = BN < 32 ? 32 : BN;
  constexpr int SF_COLS = MODE == 2 ? (16 + 16 * NB128) : 0;
  constexpr int TMEM_COLS = (ACC_COLS + SF_COLS) <= 32 ? 32 : (ACC_COLS + SF_COLS) <= 64 ? 64
                            : (ACC_COLS + SF_COLS) <= 128 ? 128 : (ACC_COLS + SF_COLS) <= 256 ? 256 : 512;
  static_assert(STAGE_BYTES % 1024 == 0, "stage must keep 1024 B alignment");

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  __shared__ uint64_t full[STAGES], empty[STAGES], deq[STAGES], acc_full;
  __shared__ uint32_t tmem_holder;
  __shared__ int s_fail;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n0 = blockIdx.x * 128;            // output feature of TMEM lane 0 (within the expert when grouped)
  int t0 = blockIdx.y * BN, t_end = p.T;      // token rows of this tile
  int a_row0 = n0;                            // first row of the weight tile in the (stacked) weight matrix
  size_t sf_tile = blockIdx.x;                // index of the 128-row scale tile
  float alpha = p.alpha;
  if (p.tile_tab) {
    const int4 tt = reinterpret_cast<const int4*>(p.tile_tab)[blockIdx.y];
    if (tt.z <= 0) return;                    // idle tile: uniform exit before any barrier or TMEM use
    t0 = tt.y;
    t_end = tt.y + tt.z;
    a_row0 = tt.x * p.n_per_expert + n0;
    sf_tile = (size_t)tt.x * (p.n_per_expert / 128) + blockIdx.x;
    if (p.alpha_tab) alpha = p.alpha_tab[tt.x];
  }
  const int nkt = p.K / KT;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
      mbar_init(&deq[s], 4);
    }
    mbar_init(&acc_full, 1);
    s_fail = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(&tmem_holder, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_holder;

  auto stage_ptr = [&](int s) { return smem + (size_t)s * STAGE_BYTES; };
  // layout inside a stage: [A_RAW][A_DEQ][B][SFA][SFB]

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (elect_one()) {
      prefetch_tmap(&amap);
      prefetch_tmap(&bmap);
      for (int kt = 0; kt < nkt; ++kt) {
        const int s = kt % STAGES;
        if (!mbar_wait(&empty[s], ((kt / STAGES) & 1) ^ 1)) {
          atomicExch(&s_fail, 1);
          break;
        }
        uint8_t* st = stage_ptr(s);
        mbar_expect_tx(&full[s], A_RAW + B_BYTES + SFA_BYTES + SFB_BYTES);
        if (MODE == 0) {
          tma_load_2d(st, &amap, &full[s], kt * 64, a_row0);
          tma_load_2d(st + A_RAW + A_DEQ, &bmap, &full[s], kt * 64, t0);
        } else if (MODE == 1) {
          tma_load_2d(st, &amap, &full[s], kt * 64, a_row0);  // 64 bytes = 128 fp4 per row, unswizzled
          tma_load_2d(st + A_RAW + A_DEQ, &bmap, &full[s], kt * 128, t0);
          tma_load_2d(st + A_RAW + A_DEQ + B_SUB, &bmap, &full[s], kt * 128 + 64, t0);
          bulk_load(st + A_RAW + A_DEQ + B_BYTES, p.sfa + (sf_tile * nkt + kt) * 1024, 1024, &full[s]);
        } else {
          tma_load_2d(st, &amap, &full[s], kt * 128, a_row0);  // 128 bytes = 256 fp4 per row
          tma_load_2d(st + A_RAW, &bmap, &full[s], kt * 128, t0);
          bulk_load(st + A_RAW + B_BYTES, p.sfa + (sf_tile * nkt + kt) * 2048, 2048, &full[s]);
#pragma unroll
          for (int b = 0; b < NB128; ++b)
            bulk_load(st + A_RAW + B_BYTES + SFA_BYTES + b * 2048,
                      p.sfb + ((size_t)(blockIdx.y * NB128 + b) * nkt + kt) * 2048, 2048, &full[s]);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (elect_one()) {
      constexpr uint32_t idesc = MODE == 0   ? make_idesc_f16(1, 1, 128, BN)
                                 : MODE == 1 ? make_idesc_f16(1, 1, 128, BN)
                                             : make_idesc_nvf4(128, BN);
      const uint32_t tmem_sfa = tmem_base + ACC_COLS, tmem_sfb = tmem_base + ACC_COLS + 16;
      bool ok = true;
      for (int kt = 0; kt < nkt && ok; ++kt) {
        const int s = kt % STAGES;
        const uint32_t par = (kt / STAGES) & 1;
        ok = mbar_wait(&full[s], par);
        if (ok && MODE == 1) ok = mbar_wait(&deq[s], par);
        if (!ok) break;
        tc_fence_after();
        uint8_t* st = stage_ptr(s);
        if (MODE == 2) {
          const uint32_t sfa_s = smem_u32(st + A_RAW + B_BYTES), sfb_s = sfa_s + SFA_BYTES;
#pragma unroll
          for (int kb = 0; kb < 4; ++kb) {
            tc_cp_sf(tmem_sfa + kb * 4, make_desc_sf(sfa_s + kb * 512));
#pragma unroll
            for (int b = 0; b < NB128; ++b)
              tc_cp_sf(tmem_sfb + kb * 4 * NB128 + b * 4, make_desc_sf(sfb_s + b * 2048 + kb * 512));
          }
          const uint64_t ad = make_desc_sw128(smem_u32(st)), bd = make_desc_sw128(smem_u32(st + A_RAW));
#pragma unroll
          for (int kb = 0; kb < 4; ++kb)
            tc_mma_nvf4(tmem_base, ad + kb * 2, bd + kb * 2, idesc, (kt | kb) ? 1u : 0u, tmem_sfa + kb * 4,
                        tmem_sfb + kb * 4 * NB128);
        } else {
          constexpr int NSUB = MODE == 1 ? 2 : 1;
          const uint32_t a_s = smem_u32(st + (MODE == 1 ? A_RAW : 0)), b_s = smem_u32(st + A_RAW + A_DEQ);
#pragma unroll
          for (int sub = 0; sub < NSUB; ++sub) {
            const uint64_t ad = make_desc_sw128(a_s + sub * 128 * 128), bd = make_desc_sw128(b_s + sub * B_SUB);
#pragma unroll
            for (int kb = 0; kb < 4; ++kb)
              tc_mma_f16(tmem_base, ad + kb * 2, bd + kb * 2, idesc, (kt | sub | kb) ? 1u : 0u);
          }
        }
        tc_commit(&empty[s]);
      }
      if (!ok) atomicExch(&s_fail, 1);
      tc_commit(&acc_full);
    }
  } else {
    // ------------------------------------------------------------------ dequantisers, then epilogue
    const int ew = warp - 2;        // 0..3
    const int etid = ew * 32 + lane;  // 0..127
    if (MODE == 1) {
      bool ok = true;
      for (int kt = 0; kt < nkt && ok; ++kt) {
        const int s = kt % STAGES;
        ok = mbar_wait(&full[s], (kt / STAGES) & 1);
        if (!ok) break;
        uint8_t* st = stage_ptr(s);
        const uint8_t* raw = st;
        const uint8_t* sc = st + A_RAW + A_DEQ + B_BYTES;
        uint8_t* dq = st + A_RAW;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int q = etid + i * 128;  // 16 B chunk of the raw tile: row q/4, 32 elements at (q%4)*32
          const int row = q >> 2, part = q & 3;
          const uint4 w = *reinterpret_cast<const uint4*>(raw + q * 16);
          const uint32_t words[4] = {w.x, w.y, w.z, w.w};
          const uint32_t s2 = *reinterpret_cast<const unsigned short*>(sc + row * 8 + part * 2);
          const uint32_t sca = e4m3_to_bf16x2_dup(s2 & 0xffu), scb = e4m3_to_bf16x2_dup(s2 >> 8);
#pragma unroll
          for (int j = 0; j < 4; ++j) {  // 8 elements -> one 16 B chunk of bf16
            const uint32_t scale = j < 2 ? sca : scb;
            uint32_t o4[4];
            e2m1x8_to_bf16x8(words[j], o4);
#pragma unroll
            for (int b = 0; b < 4; ++b) {
              // code x scale has <= 6 significant bits: the bf16 product is exact
              const __nv_bfloat162 r = __hmul2(*reinterpret_cast<const __nv_bfloat162*>(&o4[b]),
                                               *reinterpret_cast<const __nv_bfloat162*>(&scale));
              o4[b] = *reinterpret_cast<const uint32_t*>(&r);
            }
            const int chunk = part * 4 + j;  // 0..15 along K (8 elements each)
            const int sub = chunk >> 3, ch = chunk & 7;
            *reinterpret_cast<uint4*>(dq + sub * 128 * 128 + row * 128 + ((ch ^ (row & 7)) << 4)) =
                make_uint4(o4[0], o4[1], o4[2], o4[3]);
          }
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(&deq[s]);
      }
      if (!ok) atomicExch(&s_fail, 1);
    }
    // epilogue: TMEM lane = output feature, column = token
    const bool ok = mbar_wait(&acc_full, 0);
    if (!ok) atomicExch(&s_fail, 1);
    tc_fence_after();
    if (ok && !s_fail) {
      const int q = warp & 3;  // TMEM lane quarter this warp may touch
      const int n = n0 + q * 32 + lane;
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += 16) {
        uint32_t r[16];
        tmem_ld16(tmem_base + ((uint32_t)(q * 32) << 16) + c0, r);
        tmem_ld_wait();
        if (n < p.N) {
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const int t = t0 + c0 + j;
            if (t < t_end) {
              float v = __uint_as_float(r[j]) * alpha;
              if (p.residual) v += bf2f(p.residual[(long)t * p.ldr + n]);
              if (p.out_f32) p.out_f32[(long)t * p.ldo + n] = v;
              else p.out[(long)t * p.ldo + n] = f2bf(v);
            }
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
  if (threadIdx.x == 0 && s_fail && p.status) atomicExch(p.status, (int)kErrMbarTimeout);
}

template <int MODE, int BN, int STAGES>
static int launch_gemm(const GemmParams& p, const CUtensorMap& amap, const CUtensorMap& bmap, cudaStream_t st) {
  constexpr int KT = GemmCfg<MODE>::KT;
  constexpr int A_RAW = MODE == 0 ? 128 * 128 : (MODE == 1 ? 128 * 64 : 128 * 128);
  constexpr int A_DEQ = MODE == 1 ? 128 * 256 : 0;
  constexpr int B_BYTES = BN * 128 * (MODE == 1 ? 2 : 1);
  constexpr int SF = MODE == 1 ? 1024 : (MODE == 2 ? 2048 + 2048 * ((BN + 127) / 128) : 0);
  constexpr int smem = STAGES * (A_RAW + A_DEQ + B_BYTES + SF) + 1024;
  static_assert(smem <= 227 * 1024, "shared memory budget");
  if (p.K % KT) return (int)cudaErrorInvalidValue;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(gemm_kernel<MODE, BN, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return (int)e;
    attr_set = true;
  }
  dim3 grid((p.N + 127) / 128, p.tile_tab ? p.n_tiles : (p.T + BN - 1) / BN);
  gemm_kernel<MODE, BN, STAGES><<<grid, 192, smem, st>>>(p, amap, bmap);
  return (int)cudaGetLastError();
}

template <int MODE>
static int dispatch_gemm(const GemmParams& p, const CUtensorMap& amap, const CUtensorMap& bmap, int bn,
                         cudaStream_t st) {
  switch (bn) {
    case 16: return launch_gemm<MODE, 16, MODE == 1 ? 4 : 8>(p, amap, bmap, st);
    case 32: return launch_gemm<MODE, 32, MODE == 1 ? 4 : 8>(p, amap, bmap, st);
    case 64: return launch_gemm<MODE, 64, MODE == 1 ? 3 : 6>(p, amap, bmap, st);
    case 128: return launch_gemm<MODE, 128, MODE == 1 ? 3 : (MODE == 2 ? 5 : 6)>(p, amap, bmap, st);
    case 256: return launch_gemm<MODE, 256, MODE == 1 ? 2 : 4>(p, amap, bmap, st);
  }
  return (int)cudaErrorInvalidValue;
}

static int pick_bn(int T) { return T <= 16 ? 16 : T <= 32 ? 32 : T <= 64 ? 64 : T <= 128 ? 128 : 256; }

}  // namespace ve

using namespace ve;

extern "C" {

// bf16 weights W [N, K] (row pitch ldw elements), bf16 activations X [T, K] (pitch ldx).
int ve_gemm_bf16(const void* W, long ldw, const void* X, long ldx, void* out, long ldo, void* out_f32,
                 const void* residual, long ldr, int T, int N, int K, float alpha, void* status, cudaStream_t st) {
  if (T <= 0 || N <= 0) return 0;
  const int bn = pick_bn(T);
  CUtensorMap amap, bmap;
  int rc = make_tmap_2d(&amap, W, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, N, K, (uint64_t)ldw * 2, 128, 64,
                        CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc) return rc;
  rc = make_tmap_2d(&bmap, X, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, T, K, (uint64_t)ldx * 2, bn, 64,
                    CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc) return rc;
  GemmParams p{N, T, K, alpha, (__nv_bfloat16*)out, ldo, (const __nv_bfloat16*)residual, ldr, (float*)out_f32,
               nullptr, nullptr, (int*)status};
  return dispatch_gemm<0>(p, amap, bmap, bn, st);
}

// NVFP4 weights (Wp [N, K/2] bytes, blocked scales sfa [N/128][K/128][128][8]) x bf16 activations.
int ve_gemm_w4a16(const void* Wp, const void* sfa, const void* X, long ldx, void* out, long ldo, void* out_f32,
                  const void* residual, long ldr, int T, int N, int K, float alpha, void* status, cudaStream_t st) {
  if (T <= 0 || N <= 0) return 0;
  if (N % 128) return cudaErrorInvalidValue;
  const int bn = pick_bn(T);
  CUtensorMap amap, bmap;
  int rc = make_tmap_2d(&amap, Wp, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, N, K / 2, (uint64_t)K / 2, 128, 64,
                        CU_TENSOR_MAP_SWIZZLE_NONE);
  if (rc) return rc;
  rc = make_tmap_2d(&bmap, X, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, T, K, (uint64_t)ldx * 2, bn, 64,
                    CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc) return rc;
  GemmParams p{N, T, K, alpha, (__nv_bfloat16*)out, ldo, (const __nv_bfloat16*)residual, ldr, (float*)out_f32,
               (const uint8_t*)sfa, nullptr, (int*)status};
  return dispatch_gemm<1>(p, amap, bmap, bn, st);
}

// NVFP4 weights x NVFP4 activations. Scales of both operands in 512 B atoms:
//   sfa [N/128][K/64][512], sfb [ceil(T/128)][K/64][512]; atom byte (r%32)*16 + (r/32)*4 + j holds the
//   E4M3 scale of row r, 16-element block j of the 64-wide k group.
int ve_gemm_w4a4(const void* Wp, const void* sfa, const void* Xp, const void* sfb, void* out, long ldo,
                 void* out_f32, const void* residual, long ldr, int T, int N, int K, float alpha, void* status,
                 cudaStream_t st) {
  if (T <= 0 || N <= 0) return 0;
  if (N % 128) return cudaErrorInvalidValue;
  const int bn = pick_bn(T);
  CUtensorMap amap, bmap;
  int rc = make_tmap_2d(&amap, Wp, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, N, K / 2, (uint64_t)K / 2, 128, 128,
                        CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc) return rc;
  rc = make_tmap_2d(&bmap, Xp, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, T, K / 2, (uint64_t)K / 2, bn, 128,
                    CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc) return rc;
  GemmParams p{N, T, K, alpha, (__nv_bfloat16*)out, ldo, (const __nv_bfloat16*)residual, ldr, (float*)out_f32,
               (const uint8_t*)sfa, (const uint8_t*)sfb, (int*)status};
  return dispatch_gemm<2>(p, amap, bmap, bn, st);
}

// Grouped (mixture-of-experts) GEMMs. Weights of all experts are stacked along N ([E * N, K]); X holds the
// routed rows sorted by expert ([R, K]); tile_tab [n_tiles][4] ints = {expert, first row, rows, 0} with every
// tile covering at most `bn` rows of one expert (bn in {16, 32, 64, 128, 256}); out [R, N].
int ve_gemm_grouped_bf16(const void* W, long ldw, const void* X, long ldx, void* out, long ldo, int R, int E, int N,
                         int K, int bn, const void* tile_tab, int n_tiles, void* status, cudaStream_t st) {
  if (R <= 0 || n_tiles <= 0) return 0;
  CUtensorMap amap, bmap;
  int rc = make_tmap_2d(&amap, W, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)E * N, K, (uint64_t)ldw * 2, 128, 64,
                        CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc) return rc;
  rc = make_tmap_2d(&bmap, X, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, R, K, (uint64_t)ldx * 2, bn, 64,
                    CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc) return rc;
  GemmParams p{N, R, K, 1.f, (__nv_bfloat16*)out, ldo, nullptr, 0, nullptr, nullptr, nullptr, (int*)status,
               (const int*)tile_tab, N, nullptr, n_tiles};
  return dispatch_gemm<0>(p, amap, bmap, bn, st);
}

int ve_gemm_grouped_w4a16(const void* Wp, const void* sfa, const void* alpha_tab, const void* X, long ldx, void* out,
                          long ldo, int R, int E, int N, int K, int bn, const void* tile_tab, int n_tiles,
                          void* status, cudaStream_t st) {
  if (R <= 0 || n_tiles <= 0) return 0;
  if (N % 128) return cudaErrorInvalidValue;
  CUtensorMap amap, bmap;
  int rc = make_tmap_2d(&amap, Wp, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, (uint64_t)E * N, K / 2, (uint64_t)K / 2, 128, 64,
                        CU_TENSOR_MAP_SWIZZLE_NONE);
  if (rc) return rc;
  rc = make_tmap_2d(&bmap, X, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, R, K, (uint64_t)ldx * 2, bn, 64,
                    CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc) return rc;
  GemmParams p{N, R, K, 1.f, (__nv_bfloat16*)out, ldo, nullptr, 0, nullptr, (const uint8_t*)sfa, nullptr,
               (int*)status, (const int*)tile_tab, N, (const float*)alpha_tab, n_tiles};
  return dispatch_gemm<1>(p, amap, bmap, bn, st);
}

}  // extern "C"
