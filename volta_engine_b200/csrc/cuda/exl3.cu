// EXL3 (trellis-coded) weights: fused decode + mat-vec for decode / verify rows, 128-point Hadamard rotation,
// and a reconstruct-to-bf16 kernel that feeds the tcgen05 GEMM for prefill chunks.
//
// Format: codes uint16 [K/16, N/16, 16*bits]; one 16x16 tile is a cyclic stream of 256*bits bits (uint16 pairs
// = little-endian words, MSB first); position p = 8*lane + i owns the 16-bit window that starts at bit
// p*bits + bits - 16. In that order lane `lane` of a warp holds exactly the two B fragments of
// mma.m16n8k16 for the tile (k = 2t + (i&1) + 8*((i>>1)&1), n = g + 8*(i>>2), g = lane>>2, t = lane&3), so the
// decoded fp16 pairs go to the tensor core without any shuffle; the activations (<= 16 rows, fp16, already
// rotated) are the A operand, read through L1. One CTA owns 16 output columns, its 8 warps split K
// in a fixed order, and the cross-warp sum is a fixed tree: results do not depend on M or on the grid.
// Codebooks: 2 = MUL1 (x = w*0x83DCD12D, byte sum s, value = fma(1024+s, h(0x1eee), h(0xc931)) in fp16),
// 0 = 3INST (x = w*89226354+64248484), 1 = MCG (x = w*0xCBAC1FED), both y = (x & 0x8fff8fff) ^ 0x3b603b60,
// value = lo half + hi half.
// Reference counterparts: src/kernels/slang/ref_trellis.slang:1-130 (format statement),
// src/kernels/cuda/trellis/ (decode GEMV / GEMM), src/backend/cpu/linear_trellis.cpp:129-239.
#include "common.cuh"
#include <cuda_fp16.h>

namespace ve {

// Two windows -> packed half2 bits of the two decoded values (low half = first window).
template <int CB>
VE_DEVINL uint32_t exl3_decode2(uint32_t w0, uint32_t w1) {
  if (CB == 2) {
    const uint32_t h0 = __dp4a(w0 * 0x83DCD12Du, 0x01010101u, 0x6400u);   // fp16 bits of 1024 + s
    const uint32_t h1 = __dp4a(w1 * 0x83DCD12Du, 0x01010101u, 0x6400u);
    const uint32_t pk = __byte_perm(h0, h1, 0x5410);                       // low halves of h0, h1 (their high halves are 0)
    const __half2 a = __half2half2(__ushort_as_half((unsigned short)0x1eee));
    const __half2 b = __half2half2(__ushort_as_half((unsigned short)0xc931));
    const __half2 v = __hfma2(*reinterpret_cast<const __half2*>(&pk), a, b);
    return *reinterpret_cast<const uint32_t*>(&v);
  } else {
    uint32_t x0, x1;
    if (CB == 0) { x0 = w0 * 89226354u + 64248484u; x1 = w1 * 89226354u + 64248484u; }
    else { x0 = w0 * 0xCBAC1FEDu; x1 = w1 * 0xCBAC1FEDu; }
    x0 = (x0 & 0x8fff8fffu) ^ 0x3b603b60u;
    x1 = (x1 & 0x8fff8fffu) ^ 0x3b603b60u;
    const uint32_t lo = __byte_perm(x0, x1, 0x5410), hi = __byte_perm(x0, x1, 0x7632);
    const __half2 v = __hadd2(*reinterpret_cast<const __half2*>(&lo), *reinterpret_cast<const __half2*>(&hi));
    return *reinterpret_cast<const uint32_t*>(&v);
  }
}

// Words a lane needs from its tile and the bit offset of its first window inside them.
template <int BITS> struct Exl3Lane {
  static constexpr int NW = BITS <= 4 ? 2 : 3;
  int w0, off;
  VE_DEVINL explicit Exl3Lane(int lane) {
    const int total = 256 * BITS;
    const int s0 = (8 * lane * BITS + BITS - 16 + total) % total;
    w0 = s0 >> 5; off = s0 & 31;
  }
  VE_DEVINL void load(const uint32_t* __restrict__ tile, uint32_t* w) const {
#pragma unroll
    for (int j = 0; j < NW; ++j) { int idx = w0 + j; if (idx >= 8 * BITS) idx -= 8 * BITS; w[j] = __ldg(tile + idx); }
  }
  // The lane's 8 windows -> four packed half2 (B fragments b0,b1 of column block 0, then of block 1).
  template <int CB> VE_DEVINL void decode(const uint32_t* w, uint32_t* frag) const {
    uint32_t q[3];
    q[0] = __funnelshift_l(w[1], w[0], off);
    q[1] = __funnelshift_l(NW > 2 ? w[2] : 0u, w[1], off);
    q[2] = NW > 2 ? (w[2] << off) : 0u;
    uint32_t win[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int t = i * BITS, j = t >> 5, sh = t & 31;          // window i = bits [sh, sh + 16) below the top of q[j] : q[j + 1]
      if (sh <= 16) {
        win[i] = (q[j] >> (16 - sh)) & 0xffffu;                 // inside one word: a single bit-field extract
      } else {
        win[i] = __funnelshift_r(q[j + 1 > 2 ? 2 : j + 1], q[j], 48 - sh) & 0xffffu;
      }
    }
#pragma unroll
    for (int p = 0; p < 4; ++p) frag[p] = exl3_decode2<CB>(win[2 * p], win[2 * p + 1]);
  }
};

VE_DEVINL void mma_f16(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

constexpr int kExl3Warps = 8;

// x: fp16 [groups][M][K] rotated activations (read through L1: at most 16 x K halves, re-used by every warp);
// y: fp32 [groups][M][N]; group = blockIdx.y, its weights start at codes + expert[group] * expert_stride
// (expert == nullptr: one shared matrix). The column tiles of a group are split evenly over gridDim.x CTAs (the host
// sizes the grid to the number of CTAs that are resident at once, so every CTA gets the same work to within one tile
// and there is no partial last wave); a CTA walks its range in units of 4, 2 or 1 adjacent column tiles. In a unit every
// warp walks its share of K and reads NTW * 32 * BITS contiguous bytes per k-tile.
template <int BITS, int CB, int MH, int NTW>   // MH: 8 or 16 activation rows held by the A fragment
VE_DEVINL void exl3_gemv_unit(const uint32_t* __restrict__ base, size_t tstride, const __half* __restrict__ xlo,
                              const __half* __restrict__ xhi, bool row_lo, bool row_hi, float* __restrict__ y, float* red,
                              int M, int KT, int N, int nt0) {
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
  const int per = (KT + kExl3Warps - 1) / kExl3Warps;
  const int kt0 = warp * per, kt1 = min(KT, kt0 + per);
  const Exl3Lane<BITS> L(lane);
  constexpr int NW = Exl3Lane<BITS>::NW;
  base += (size_t)nt0 * (8 * BITS);
  float acc[NTW][2][4];
#pragma unroll
  for (int j = 0; j < NTW; ++j)
#pragma unroll
    for (int h = 0; h < 2; ++h)
#pragma unroll
      for (int i = 0; i < 4; ++i) acc[j][h][i] = 0.f;
  constexpr int UK = (NW == 2 ? 4 : 2) / NTW > 0 ? (NW == 2 ? 4 : 2) / NTW : 1;   // k-tiles per step of a warp
  // Two register buffers: the words of step i + 1 are requested before step i is decoded, so a warp's memory latency
  // overlaps its own arithmetic (the warps of a CTA run in lock-step and would otherwise all wait at the same time).
  uint32_t wn[UK][NTW][NW], an[UK][4];
  auto fetch = [&](int kt) {
#pragma unroll
    for (int u = 0; u < UK; ++u) {
      const int k = min(kt + u, kt1 - 1);                           // tail: re-read the last tile, its math is skipped
#pragma unroll
      for (int j = 0; j < NTW; ++j) L.load(base + (size_t)k * tstride + j * (8 * BITS), wn[u][j]);
      const int ko = k * 16;                                        // the A fragment of the same k-tile (L1 resident)
      an[u][0] = row_lo ? __ldg(reinterpret_cast<const uint32_t*>(xlo + ko)) : 0u;
      an[u][2] = row_lo ? __ldg(reinterpret_cast<const uint32_t*>(xlo + ko + 8)) : 0u;
      an[u][1] = row_hi ? __ldg(reinterpret_cast<const uint32_t*>(xhi + ko)) : 0u;
      an[u][3] = row_hi ? __ldg(reinterpret_cast<const uint32_t*>(xhi + ko + 8)) : 0u;
    }
  };
  if (kt0 < kt1) fetch(kt0);
  for (int kt = kt0; kt < kt1; kt += UK) {
    uint32_t w[UK][NTW][NW], a[UK][4];
#pragma unroll
    for (int u = 0; u < UK; ++u) {
#pragma unroll
      for (int j = 0; j < NTW; ++j)
#pragma unroll
        for (int i = 0; i < NW; ++i) w[u][j][i] = wn[u][j][i];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[u][i] = an[u][i];
    }
    if (kt + UK < kt1) fetch(kt + UK);
#pragma unroll
    for (int u = 0; u < UK; ++u) {
      if (kt + u < kt1) {
#pragma unroll
        for (int j = 0; j < NTW; ++j) {
          uint32_t f[4];
          L.template decode<CB>(w[u][j], f);
          mma_f16(acc[j][0], a[u], f[0], f[1]);
          mma_f16(acc[j][1], a[u], f[2], f[3]);
        }
      }
    }
  }
  // C fragment: c[0],c[1] -> row g, cols 2t,2t+1; c[2],c[3] -> row g+8.
  constexpr int W = 16 * NTW;
  __syncthreads();                                                  // the previous unit's sums have been read
  float* r = red + warp * 16 * W;
#pragma unroll
  for (int j = 0; j < NTW; ++j)
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int c = j * 16 + h * 8 + 2 * t;
      r[g * W + c] = acc[j][h][0]; r[g * W + c + 1] = acc[j][h][1];
      r[(g + 8) * W + c] = acc[j][h][2]; r[(g + 8) * W + c + 1] = acc[j][h][3];
    }
  __syncthreads();
  for (int i = tid; i < M * W; i += blockDim.x) {
    const int m = i / W, n = i % W;
    float s = 0.f;
#pragma unroll
    for (int wv = 0; wv < kExl3Warps; ++wv) s += red[wv * 16 * W + m * W + n];
    y[(size_t)m * N + nt0 * 16 + n] = s;
  }
}

template <int BITS, int CB, int MH>
__global__ void __launch_bounds__(kExl3Warps * 32, 2)
exl3_gemv_kernel(const uint16_t* __restrict__ codes, const __half* __restrict__ x, float* __restrict__ y,
                 int M, int K, int N, const int* __restrict__ expert, long expert_stride) {
  __shared__ float red[kExl3Warps * 256 * 4];                       // [warps][16 rows][16 * NTW cols], NTW <= 4
  const int grp = blockIdx.y;
  if (expert) { const int e = expert[grp]; if (e < 0) return; codes += (size_t)e * expert_stride; }
  x += (size_t)grp * M * K; y += (size_t)grp * M * N;
  const int lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const bool row_lo = g < M, row_hi = MH == 16 && g + 8 < M;
  const __half* xlo = x + (size_t)(row_lo ? g : 0) * K + 2 * t;
  const __half* xhi = x + (size_t)(row_hi ? g + 8 : 0) * K + 2 * t;
  const int KT = K >> 4, NT = N >> 4;
  const uint32_t* base = reinterpret_cast<const uint32_t*>(codes);
  const size_t tstride = (size_t)NT * (8 * BITS);
  int nt = (int)((long)NT * blockIdx.x / gridDim.x);
  const int nt_end = (int)((long)NT * (blockIdx.x + 1) / gridDim.x);
  while (nt < nt_end) {
    const int left = nt_end - nt;
    if (left >= 4) { exl3_gemv_unit<BITS, CB, MH, 4>(base, tstride, xlo, xhi, row_lo, row_hi, y, red, M, KT, N, nt); nt += 4; }
    else if (left >= 2) { exl3_gemv_unit<BITS, CB, MH, 2>(base, tstride, xlo, xhi, row_lo, row_hi, y, red, M, KT, N, nt); nt += 2; }
    else { exl3_gemv_unit<BITS, CB, MH, 1>(base, tstride, xlo, xhi, row_lo, row_hi, y, red, M, KT, N, nt); nt += 1; }
  }
}

// ------------------------------------------------------------------------------------------------ Hadamard
// dtype codes: 0 bf16, 1 fp32, 2 fp16.
template <int DT> VE_DEVINL void had_load4(const void* p, size_t i, float* v) {
  if (DT == 1) { const float4 f = *reinterpret_cast<const float4*>((const float*)p + i); v[0] = f.x; v[1] = f.y; v[2] = f.z; v[3] = f.w; }
  else if (DT == 0) {
    const uint2 u = *reinterpret_cast<const uint2*>((const __nv_bfloat16*)p + i);
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.y));
    v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
  } else {
    const uint2 u = *reinterpret_cast<const uint2*>((const __half*)p + i);
    const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&u.x));
    const float2 b = __half22float2(*reinterpret_cast<const __half2*>(&u.y));
    v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
  }
}
template <int DT> VE_DEVINL void had_store4(void* p, size_t i, const float* v) {
  if (DT == 1) *reinterpret_cast<float4*>((float*)p + i) = make_float4(v[0], v[1], v[2], v[3]);
  else if (DT == 0) {
    __nv_bfloat162 a = __floats2bfloat162_rn(v[0], v[1]), b = __floats2bfloat162_rn(v[2], v[3]);
    uint2 u; u.x = *reinterpret_cast<uint32_t*>(&a); u.y = *reinterpret_cast<uint32_t*>(&b);
    *reinterpret_cast<uint2*>((__nv_bfloat16*)p + i) = u;
  } else {
    __half2 a = __floats2half2_rn(v[0], v[1]), b = __floats2half2_rn(v[2], v[3]);
    uint2 u; u.x = *reinterpret_cast<uint32_t*>(&a); u.y = *reinterpret_cast<uint32_t*>(&b);
    *reinterpret_cast<uint2*>((__half*)p + i) = u;
  }
}

// In-warp 128-point Walsh-Hadamard transform (natural order, scaled by 1/sqrt(128)); lane holds elements 4l..4l+3.
VE_DEVINL void wht128(float* v, int lane) {
  float a = v[0] + v[1], b = v[0] - v[1], c = v[2] + v[3], d = v[2] - v[3];
  v[0] = a + c; v[1] = b + d; v[2] = a - c; v[3] = b - d;
#pragma unroll
  for (int m = 1; m < 32; m <<= 1) {
    const bool up = lane & m;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float o = __shfl_xor_sync(0xffffffffu, v[j], m);
      v[j] = up ? o - v[j] : v[j] + o;
    }
  }
  const float s = 0.08838834764831845f;
#pragma unroll
  for (int j = 0; j < 4; ++j) v[j] *= s;
}

struct HadArgs {
  const void* in; const void* in2; void* out;
  const __half* scale; const __half* scale2;
  const int* expert; long scale_stride;
  int rows, C, post, in_div, rows_per_group, act;
};

VE_DEVINL float act_apply(float x, int act) {
  if (act == 1) { const float t = tanhf(0.7978845608028654f * (x + 0.044715f * x * x * x)); return 0.5f * x * (1.f + t); }
  return x / (1.f + __expf(-x));
}

// One warp per 128-block. post == 0: out = had(in * scale); post == 1: out = had(in) * scale; with in2:
// out = act(had(in) * scale) * (had(in2) * scale2).
template <int DI, int DO>
__global__ void __launch_bounds__(256) had128_kernel(HadArgs a) {
  const int lane = threadIdx.x & 31;
  const int nb = a.C >> 7;
  const long total = (long)a.rows * nb;
  for (long blk = (long)blockIdx.x * 8 + (threadIdx.x >> 5); blk < total; blk += (long)gridDim.x * 8) {
    const int row = (int)(blk / nb), cb = (int)(blk % nb);
    const int col = cb * 128 + lane * 4;
    long soff = col;
    if (a.expert) {
      const int e = a.expert[row / a.rows_per_group];
      if (e < 0) continue;
      soff += (long)e * a.scale_stride;
    }
    float s[4] = {1.f, 1.f, 1.f, 1.f}, v[4];
    if (a.scale) had_load4<2>(a.scale, soff, s);
    had_load4<DI>(a.in, (size_t)(row / a.in_div) * a.C + col, v);
    if (!a.post) {
#pragma unroll
      for (int j = 0; j < 4; ++j) v[j] *= s[j];
    }
    wht128(v, lane);
    if (a.post) {
#pragma unroll
      for (int j = 0; j < 4; ++j) v[j] *= s[j];
    }
    if (a.in2) {
      float u[4], s2[4] = {1.f, 1.f, 1.f, 1.f};
      if (a.scale2) had_load4<2>(a.scale2, soff, s2);
      had_load4<DI>(a.in2, (size_t)(row / a.in_div) * a.C + col, u);
      wht128(u, lane);
#pragma unroll
      for (int j = 0; j < 4; ++j) v[j] = act_apply(v[j], a.act) * (u[j] * s2[j]);
    }
    had_store4<DO>(a.out, (size_t)row * a.C + col, v);
  }
}

// ------------------------------------------------------------------------------------------------ reconstruct
// codes -> bf16 [N][K] (output features major, K contiguous): the A operand layout of the tcgen05 GEMM.
// batch > 1: `batch` matrices back to back (the experts of a bank) -> [batch * N][K].
template <int BITS, int CB>
__global__ void __launch_bounds__(256) exl3_reconstruct_kernel(const uint16_t* __restrict__ codes,
                                                               __nv_bfloat16* __restrict__ out, int K, int N, int batch) {
  const int lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const int KT = K >> 4, NT = N >> 4;
  const Exl3Lane<BITS> L(lane);
  const long per = (long)KT * NT, total = per * batch;
  // consecutive warps walk kt for a fixed nt so that a CTA writes runs of 128 contiguous k per output row
  for (long gid = (long)blockIdx.x * 8 + (threadIdx.x >> 5); gid < total; gid += (long)gridDim.x * 8) {
    const long b = gid / per, id = gid % per;
    const int nt = (int)(id / KT), kt = (int)(id % KT);
    uint32_t w[3], f[4];
    L.load(reinterpret_cast<const uint32_t*>(codes) + ((size_t)b * per + (size_t)kt * NT + nt) * (8 * BITS), w);
    L.template decode<CB>(w, f);
#pragma unroll
    for (int p = 0; p < 4; ++p) {
      const float2 v = __half22float2(*reinterpret_cast<const __half2*>(&f[p]));
      const int n = nt * 16 + g + 8 * (p >> 1), k = kt * 16 + 2 * t + 8 * (p & 1);
      *reinterpret_cast<__nv_bfloat162*>(out + ((size_t)b * N + n) * K + k) = __floats2bfloat162_rn(v.x, v.y);
    }
  }
}

}  // namespace ve

using namespace ve;

// Grid: as many CTAs as are resident at once (occupancy x SMs), shared between the groups; never more than the column
// tiles of a group.
template <int BITS, int CB, int MH>
static int exl3_gemv_grid() {
  static int ctas = 0;
  if (!ctas) {
    int per_sm = 0, dev = 0, sms = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, exl3_gemv_kernel<BITS, CB, MH>, kExl3Warps * 32, 0) != cudaSuccess ||
        per_sm < 1)
      per_sm = 1;
    ctas = per_sm * sms;
  }
  return ctas;
}

template <int BITS, int CB>
static int exl3_gemv_launch(const void* codes, const void* x, void* y, int M, int K, int N, const int* expert,
                            long stride, int groups, cudaStream_t st) {
  const int NT = N / 16;
  if (M <= 8) {
    const int gx = max(1, min(NT, exl3_gemv_grid<BITS, CB, 8>() / groups));
    exl3_gemv_kernel<BITS, CB, 8><<<dim3(gx, groups), kExl3Warps * 32, 0, st>>>((const uint16_t*)codes, (const __half*)x,
                                                                                 (float*)y, M, K, N, expert, stride);
  } else {
    const int gx = max(1, min(NT, exl3_gemv_grid<BITS, CB, 16>() / groups));
    exl3_gemv_kernel<BITS, CB, 16><<<dim3(gx, groups), kExl3Warps * 32, 0, st>>>((const uint16_t*)codes, (const __half*)x,
                                                                                  (float*)y, M, K, N, expert, stride);
  }
  VE_CHECK_LAUNCH();
}

extern "C" {

int ve_exl3_gemv(const void* codes, const void* x, void* y, int M, int K, int N, int bits, int cb,
                 const void* expert, long expert_stride, int groups, cudaStream_t st) {
  if (M < 1 || M > 16 || K % 16 || N % 16 || groups < 1 || cb < 0 || cb > 2) return cudaErrorInvalidValue;
#define VE_EX(B)                                                                                             \
  case B:                                                                                                    \
    return cb == 2 ? exl3_gemv_launch<B, 2>(codes, x, y, M, K, N, (const int*)expert, expert_stride, groups, st) \
         : cb == 1 ? exl3_gemv_launch<B, 1>(codes, x, y, M, K, N, (const int*)expert, expert_stride, groups, st) \
                   : exl3_gemv_launch<B, 0>(codes, x, y, M, K, N, (const int*)expert, expert_stride, groups, st);
  switch (bits) {
    VE_EX(1) VE_EX(2) VE_EX(3) VE_EX(4) VE_EX(5) VE_EX(6) VE_EX(7) VE_EX(8)
    default: return cudaErrorInvalidValue;
  }
#undef VE_EX
}

static int exl3_reconstruct_n(const void* codes, void* out, int K, int N, int bits, int cb, int batch, cudaStream_t st);

int ve_exl3_reconstruct(const void* codes, void* out, int K, int N, int bits, int cb, cudaStream_t st) {
  return exl3_reconstruct_n(codes, out, K, N, bits, cb, 1, st);
}

// `batch` matrices back to back ([batch][K/16][N/16][16 * bits]) -> bf16 [batch * N][K]: the stacked A operand of the
// grouped GEMM for a slab of routed experts.
int ve_exl3_reconstruct_batch(const void* codes, void* out, int K, int N, int bits, int cb, int batch, cudaStream_t st) {
  return exl3_reconstruct_n(codes, out, K, N, bits, cb, batch, st);
}

}  // extern "C"

static int exl3_reconstruct_n(const void* codes, void* out, int K, int N, int bits, int cb, int batch, cudaStream_t st) {
  if (K % 16 || N % 16 || cb < 0 || cb > 2 || batch < 1) return cudaErrorInvalidValue;
  const long tiles = (long)(K / 16) * (N / 16) * batch;
  const int blocks = (int)((tiles + 7) / 8 < 148 * 8 ? (tiles + 7) / 8 : 148 * 8);
#define VE_RC(B)                                                                                                           \
  case B:                                                                                                                  \
    if (cb == 2) exl3_reconstruct_kernel<B, 2><<<blocks, 256, 0, st>>>((const uint16_t*)codes, (__nv_bfloat16*)out, K, N, batch); \
    else if (cb == 1) exl3_reconstruct_kernel<B, 1><<<blocks, 256, 0, st>>>((const uint16_t*)codes, (__nv_bfloat16*)out, K, N, batch); \
    else exl3_reconstruct_kernel<B, 0><<<blocks, 256, 0, st>>>((const uint16_t*)codes, (__nv_bfloat16*)out, K, N, batch);         \
    break;
  switch (bits) {
    VE_RC(1) VE_RC(2) VE_RC(3) VE_RC(4) VE_RC(5) VE_RC(6) VE_RC(7) VE_RC(8)
    default: return cudaErrorInvalidValue;
  }
#undef VE_RC
  VE_CHECK_LAUNCH();
}

extern "C" {

// dt codes: 0 bf16, 1 fp32, 2 fp16. Supported (in -> out): bf16->fp16, fp32->bf16, fp32->fp16, fp16->fp16, bf16->bf16.
int ve_had128(const void* in, const void* in2, void* out, const void* scale, const void* scale2, const void* expert,
              long scale_stride, int rows, int C, int post, int in_div, int rows_per_group, int act, int dt_in,
              int dt_out, cudaStream_t st) {
  if (rows < 1 || C % 128 || in_div < 1 || rows_per_group < 1) return cudaErrorInvalidValue;
  HadArgs a{in, in2, out, (const __half*)scale, (const __half*)scale2, (const int*)expert, scale_stride,
            rows, C, post, in_div, rows_per_group, act};
  const long blocks_needed = ((long)rows * (C / 128) + 7) / 8;
  const int blocks = (int)(blocks_needed < 148 * 8 ? blocks_needed : 148 * 8);
  if (dt_in == 0 && dt_out == 2) had128_kernel<0, 2><<<blocks, 256, 0, st>>>(a);
  else if (dt_in == 1 && dt_out == 0) had128_kernel<1, 0><<<blocks, 256, 0, st>>>(a);
  else if (dt_in == 1 && dt_out == 2) had128_kernel<1, 2><<<blocks, 256, 0, st>>>(a);
  else if (dt_in == 2 && dt_out == 2) had128_kernel<2, 2><<<blocks, 256, 0, st>>>(a);
  else if (dt_in == 0 && dt_out == 0) had128_kernel<0, 0><<<blocks, 256, 0, st>>>(a);
  else if (dt_in == 1 && dt_out == 1) had128_kernel<1, 1><<<blocks, 256, 0, st>>>(a);
  else return cudaErrorInvalidValue;
  VE_CHECK_LAUNCH();
}

}  // extern "C"
