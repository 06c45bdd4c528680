// DeepSeek-V4-style attention support kernels: cache writes on the model's quantisation grids, indexer preparation and
// selection, and the gather that turns a row's window entries, selected compressed entries and the per-head sink into a
// short virtual sequence of latent pages for the latent attention kernel (mla.cu), plus the output epilogue.
//
// Grids (inc/engine/modules/dsv4.h:12-30 in the reference names the same ones):
//   window row        512 E4M3 codes + 16 E8M0 exponents (one per 32 values)          528 bytes
//   compressed entry  256 bytes of E2M1 pairs (even dim low nibble) + 32 E4M3 scales   288 bytes
//   index key / query E2M1 x power-of-two per 32 values, stored as the bf16 value (exact)
//   attention output  E4M3 x power-of-two per 32 values, stored as the bf16 value (exact)
// Rotary embedding: adjacent pairs of the last 64 dims, angles from a table [pos][32] of (cos, sin).
#include "common.cuh"
#include <cuda_fp8.h>
#include <float.h>

namespace ve {

constexpr int kHD = 512, kRopeD = 64, kWindow = 128, kRing = 1024, kWinRow = 528, kCompRow = 288;
constexpr int kIdxDim = 128, kIdxHeads = 32, kSelTopk = 512, kLatRowD = 576, kKeysMax = kWindow + kSelTopk + 1;
constexpr int kPagesRow = (kKeysMax + 63) / 64, kGroupHeads = 8;

VE_DEVINL float bfr(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }

// 2^e = the smallest power of two >= v (v > 0, normal)
VE_DEVINL int pow2_ceil_exp(float v) {
  int e;
  const float m = frexpf(v, &e);   // v = m * 2^e, m in [0.5, 1)
  return m == 0.5f ? e - 1 : e;
}

VE_DEVINL uint8_t e4m3_enc(float v) { return (uint8_t)__nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E4M3); }
VE_DEVINL float e4m3_dec(uint8_t b) {
  const __half_raw h = __nv_cvt_fp8_to_halfraw((__nv_fp8_storage_t)b, __NV_E4M3);
  return __half2float(__half(h));
}

// nearest E2M1 magnitude code (0..7), ties to the even mantissa; sign in bit 3
VE_DEVINL uint32_t e2m1_enc(float x) {
  const float a = fabsf(x);
  uint32_t c = 0;
  c += a > 0.25f;
  c += a >= 0.75f;
  c += a > 1.25f;
  c += a >= 1.75f;
  c += a > 2.5f;
  c += a >= 3.5f;
  c += a > 5.0f;
  return c | (signbit(x) ? 8u : 0u);
}
VE_DEVINL float e2m1_dec(uint32_t c) {
  const float lut[8] = {0.f, 0.5f, 1.f, 1.5f, 2.f, 3.f, 4.f, 6.f};
  const float v = lut[c & 7];
  return (c & 8) ? -v : v;
}

VE_DEVINL void rope_pair_cs(float& a, float& b, const float* cs, bool inverse) {
  const float c = cs[0], s = inverse ? -cs[1] : cs[1];
  const float x = a * c - b * s, y = b * c + a * s;
  a = x;
  b = y;
}

// ------------------------------------------------------------------------------------------------ window ring
// grid rows, block 128: thread t owns dims 4t..4t+3.
__global__ void __launch_bounds__(128) dsv4_window_store_kernel(const __nv_bfloat16* __restrict__ kv, long kv_stride,
                                                                uint8_t* __restrict__ ring, const float* __restrict__ rope,
                                                                const int* __restrict__ slot, const int* __restrict__ pos,
                                                                int layer, long slot_stride,
                                                                const __nv_bfloat16* __restrict__ norm_w, float eps, float wbias) {
  __shared__ float red[33];
  grid_dep_launch();
  grid_dep_wait();
  const int r = blockIdx.x, t = threadIdx.x, d = 4 * t;
  const int sl = slot[r];
  if (sl < 0) return;
  const int p = pos[r];
  float v[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) v[j] = __bfloat162float(kv[(long)r * kv_stride + d + j]);
  if (norm_w) {   // the projection's RMSNorm, rounded to bf16 as the separate norm kernel stores it
    const float ss = block_sum(v[0] * v[0] + v[1] * v[1] + v[2] * v[2] + v[3] * v[3], red);
    const float inv = rsqrtf(ss / (float)kHD + eps);
#pragma unroll
    for (int j = 0; j < 4; ++j) v[j] = bfr(v[j] * inv * (__bfloat162float(norm_w[d + j]) + wbias));
  }
  if (d >= kHD - kRopeD) {
    const float* cs = rope + ((long)p * (kRopeD / 2) + (d - (kHD - kRopeD)) / 2) * 2;
    rope_pair_cs(v[0], v[1], cs, false);
    rope_pair_cs(v[2], v[3], cs + 2, false);
  }
  float amax = 0.f;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    v[j] = bfr(v[j]);
    amax = fmaxf(amax, fabsf(v[j]));
  }
#pragma unroll
  for (int o = 1; o < 8; o <<= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  const int e = pow2_ceil_exp(fmaxf(amax, 1e-4f) / 448.f);
  uint32_t word = 0;
#pragma unroll
  for (int j = 0; j < 4; ++j) word |= (uint32_t)e4m3_enc(fminf(fmaxf(ldexpf(v[j], -e), -448.f), 448.f)) << (8 * j);
  uint8_t* row = ring + (long)sl * slot_stride + ((long)layer * kRing + (p % kRing)) * kWinRow;
  *reinterpret_cast<uint32_t*>(row + d) = word;
  if ((t & 7) == 0) row[kHD + d / 32] = (uint8_t)(e + 127);
}

// ------------------------------------------------------------------------------------------------ compressor
// grid rows, block 128: the group ring keeps fp32 kv and score rows at pos % kRing.
__global__ void __launch_bounds__(128) dsv4_cring_store_kernel(const __nv_bfloat16* __restrict__ ckv, long ckv_stride,
                                                               const __nv_bfloat16* __restrict__ csc, long csc_stride,
                                                               float* __restrict__ ring_kv, float* __restrict__ ring_sc,
                                                               const int* __restrict__ slot, const int* __restrict__ pos,
                                                               long slot_stride) {
  grid_dep_launch();
  grid_dep_wait();
  const int r = blockIdx.x, sl = slot[r];
  if (sl < 0) return;
  const long at = (long)sl * slot_stride + (long)(pos[r] % kRing) * kHD;
  for (int d = threadIdx.x; d < kHD; d += 128) {
    ring_kv[at + d] = __bfloat162float(ckv[(long)r * ckv_stride + d]);
    ring_sc[at + d] = __bfloat162float(csc[(long)r * csc_stride + d]);
  }
}

// grid rows, block 128 (4 dims per thread). Rows that complete a group pool it, normalise, write the unrotated latent and
// the compressed entry (rope at the group's first position, NVFP4 grid).
__global__ void __launch_bounds__(128) dsv4_compress_kernel(const __nv_bfloat16* __restrict__ ckv, long ckv_stride,
                                                            const float* __restrict__ ring_kv, const float* __restrict__ ring_sc,
                                                            const __nv_bfloat16* __restrict__ norm_w,
                                                            __nv_bfloat16* __restrict__ latent_out, uint8_t* __restrict__ comp,
                                                            const float* __restrict__ rope, const int* __restrict__ slot,
                                                            const int* __restrict__ pos, long ring_slot_stride,
                                                            long comp_slot_stride, int ratio, float eps) {
  grid_dep_launch();
  grid_dep_wait();
  __shared__ float red[33];
  const int r = blockIdx.x, t = threadIdx.x, d = 4 * t;
  const int sl = slot[r];
  if (sl < 0) return;
  const int p = pos[r];
  if (p % ratio != ratio - 1) return;
  float v[4];
  if (ratio == 1) {
#pragma unroll
    for (int j = 0; j < 4; ++j) v[j] = __bfloat162float(ckv[(long)r * ckv_stride + d + j]);
  } else {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float mx = -FLT_MAX;
      for (int g = 0; g < ratio; ++g)
        mx = fmaxf(mx, ring_sc[(long)sl * ring_slot_stride + (long)((p - ratio + 1 + g) % kRing) * kHD + d + j]);
      float num = 0.f, den = 0.f;
      for (int g = 0; g < ratio; ++g) {
        const long at = (long)sl * ring_slot_stride + (long)((p - ratio + 1 + g) % kRing) * kHD + d + j;
        const float w = __expf(ring_sc[at] - mx);
        num += w * ring_kv[at];
        den += w;
      }
      v[j] = bfr(num / den);
    }
  }
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < 4; ++j) ss += v[j] * v[j];
  ss = block_sum(ss, red);
  const float rs = rsqrtf(ss / (float)kHD + eps);
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    v[j] = bfr(v[j] * rs * __bfloat162float(norm_w[d + j]));
    latent_out[(long)r * kHD + d + j] = __float2bfloat16_rn(v[j]);
  }
  const int p0 = p - ratio + 1;
  if (d >= kHD - kRopeD) {
    const float* cs = rope + ((long)p0 * (kRopeD / 2) + (d - (kHD - kRopeD)) / 2) * 2;
    rope_pair_cs(v[0], v[1], cs, false);
    rope_pair_cs(v[2], v[3], cs + 2, false);
  }
  float amax = 0.f;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    v[j] = bfr(v[j]);
    amax = fmaxf(amax, fabsf(v[j]));
  }
  amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
  amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
  const uint8_t s8 = e4m3_enc(fmaxf(amax, 6.f * 0.001953125f) / 6.f);
  const float s = e4m3_dec(s8);
  uint32_t half = 0;
#pragma unroll
  for (int j = 0; j < 4; ++j) half |= e2m1_enc(fminf(fmaxf(__fdiv_rn(v[j], s), -6.f), 6.f)) << (4 * j);
  uint8_t* ent = comp + (long)sl * comp_slot_stride + (long)(p / ratio) * kCompRow;
  *reinterpret_cast<uint16_t*>(ent + d / 2) = (uint16_t)half;
  if ((t & 3) == 0) ent[kHD / 2 + d / 16] = s8;
}

// ------------------------------------------------------------------------------------------------ index keys / queries
// One 128-wide vector per block (block 128, one dim per thread): optional RMSNorm, rope on the last 64 dims, MXFP4 value.
VE_DEVINL float idx_vector(float x, const __nv_bfloat16* norm_w, const float* cs_row, float eps, float* red) {
  const int t = threadIdx.x;
  if (norm_w) {
    const float ss = block_sum(x * x, red);
    x = bfr(x * rsqrtf(ss / (float)kIdxDim + eps) * __bfloat162float(norm_w[t]));
  }
  const float other = __shfl_xor_sync(0xffffffffu, x, 1);
  if (t >= kIdxDim - kRopeD) {
    const float* cs = cs_row + ((t - (kIdxDim - kRopeD)) / 2) * 2;
    x = (t & 1) ? (x * cs[0] + other * cs[1]) : (x * cs[0] - other * cs[1]);
  }
  x = bfr(x);
  const float amax = warp_max(fabsf(x));
  const int e = pow2_ceil_exp(fmaxf(amax, 6.f * 1.17549435e-38f) / 6.f);
  return ldexpf(e2m1_dec(e2m1_enc(fminf(fmaxf(ldexpf(x, -e), -6.f), 6.f))), e);
}

__global__ void __launch_bounds__(128) dsv4_index_key_kernel(const __nv_bfloat16* __restrict__ kraw, long kraw_stride,
                                                             const __nv_bfloat16* __restrict__ norm_w,
                                                             __nv_bfloat16* __restrict__ idxk, const float* __restrict__ rope,
                                                             const int* __restrict__ slot, const int* __restrict__ pos,
                                                             long slot_stride, int ratio, float eps) {
  grid_dep_launch();
  grid_dep_wait();
  __shared__ float red[33];
  const int r = blockIdx.x, sl = slot[r];
  if (sl < 0) return;
  const int p = pos[r];
  if (p % ratio != ratio - 1) return;
  const float x = __bfloat162float(kraw[(long)r * kraw_stride + threadIdx.x]);
  const float v = idx_vector(x, norm_w, rope + (long)(p - ratio + 1) * kRopeD, eps, red);
  idxk[(long)sl * slot_stride + (long)(p / ratio) * kIdxDim + threadIdx.x] = __float2bfloat16_rn(v);
}

// grid (rows, 32 heads)
__global__ void __launch_bounds__(128) dsv4_index_q_kernel(const __nv_bfloat16* __restrict__ q, long q_stride,
                                                           __nv_bfloat16* __restrict__ out, const float* __restrict__ rope,
                                                           const int* __restrict__ pos) {
  grid_dep_launch();
  grid_dep_wait();
  __shared__ float red[33];
  const int r = blockIdx.x, h = blockIdx.y;
  const float x = __bfloat162float(q[(long)r * q_stride + h * kIdxDim + threadIdx.x]);
  const float v = idx_vector(x, nullptr, rope + (long)pos[r] * kRopeD, 0.f, red);
  out[((long)r * kIdxHeads + h) * kIdxDim + threadIdx.x] = __float2bfloat16_rn(v);
}

// ------------------------------------------------------------------------------------------------ selection
VE_DEVINL uint32_t okey(float s) {
  const uint32_t b = __float_as_uint(s);
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

// Block-wide (1024 threads) radix threshold of the K-th largest key among n keys given by key(i): on return every thread
// holds (thr, need_eq): keys > thr are in, and the first need_eq keys == thr in index order.
template <typename KeyFn>
VE_DEVINL void radix_threshold(KeyFn key, int n, int K, uint32_t& thr, int& need_eq, int* hist, uint32_t* s_prefix, int* s_need) {
  const int tid = threadIdx.x;
  if (tid == 0) {
    *s_prefix = 0;
    *s_need = K;
  }
  for (int shift = 24; shift >= 0; shift -= 8) {
    if (tid < 256) hist[tid] = 0;
    __syncthreads();
    const uint32_t prefix = *s_prefix;
    const uint32_t himask = shift == 24 ? 0u : (0xffffffffu << (shift + 8));
    for (int i = tid; i < n; i += 1024) {
      const uint32_t k = key(i);
      if ((k & himask) == (prefix & himask)) atomicAdd(&hist[(k >> shift) & 255], 1);
    }
    __syncthreads();
    if (tid == 0) {
      int need = *s_need, b = 255;
      for (; b > 0; --b) {
        if (hist[b] >= need) break;
        need -= hist[b];
      }
      *s_prefix = prefix | ((uint32_t)b << shift);
      *s_need = need;
    }
    __syncthreads();
  }
  thr = *s_prefix;
  need_eq = *s_need;
}

// Exclusive prefix of a per-thread flag over the block in thread order (1024 threads); returns the prefix and adds the
// block total to *base (thread 0) after all threads have read it.
VE_DEVINL int block_prefix_flag(bool f, int* wcnt, int* woff, int* base, int& before) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const unsigned b = __ballot_sync(0xffffffffu, f);
  if (lane == 0) wcnt[warp] = __popc(b);
  __syncthreads();
  if (warp == 0) {
    const int v = wcnt[lane];
    int inc = v;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
      const int n = __shfl_up_sync(0xffffffffu, inc, off);
      if (lane >= off) inc += n;
    }
    woff[lane] = inc - v;
  }
  __syncthreads();
  before = *base + woff[warp] + __popc(b & ((1u << lane) - 1u));
  const int total = woff[31] + wcnt[31];
  __syncthreads();
  if (threadIdx.x == 0) *base += total;
  __syncthreads();
  return total;
}

// Level one of the two-level selection. grid rows, block 1024. cand [rows, stride] bytes: 1 for the `blocks` best blocks of
// `block` entries by their best score; the block holding the newest entry is always kept; all blocks when there are few.
__global__ void __launch_bounds__(1024) dsv4_candidates_kernel(const float* __restrict__ scores, long score_stride,
                                                               uint8_t* __restrict__ cand, long cand_stride,
                                                               const int* __restrict__ slot, const int* __restrict__ pos,
                                                               int ratio, int blocks, int block) {
  grid_dep_launch();
  grid_dep_wait();
  __shared__ int hist[256];
  __shared__ int wcnt[32], woff[32];
  __shared__ uint32_t s_prefix;
  __shared__ int s_need, s_base;
  const int r = blockIdx.x, tid = threadIdx.x;
  if (slot[r] < 0) return;
  const int n = (pos[r] + 1) / ratio;
  const int nb = (n + block - 1) / block;
  uint8_t* out = cand + (long)r * cand_stride;
  if (nb <= blocks) {
    for (int b = tid; b < nb; b += 1024) out[b] = 1;
    return;
  }
  const float* sc = scores + (long)r * score_stride;
  const int last = (n - 1) / block;
  auto key = [&](int b) -> uint32_t {
    if (b == last) return 0xffffffffu;
    float m = -FLT_MAX;
    for (int j = b * block; j < min(n, (b + 1) * block); ++j) m = fmaxf(m, sc[j]);
    return okey(m);
  };
  uint32_t thr;
  int need_eq;
  radix_threshold(key, nb, blocks, thr, need_eq, hist, &s_prefix, &s_need);
  if (tid == 0) s_base = 0;
  __syncthreads();
  for (int c0 = 0; c0 < nb; c0 += 1024) {
    const int b = c0 + tid;
    const uint32_t k = b < nb ? key(b) : 0u;
    const bool eq = b < nb && k == thr;
    int before;
    block_prefix_flag(eq, wcnt, woff, &s_base, before);
    if (b < nb) out[b] = (k > thr || (eq && before < need_eq)) ? 1 : 0;
  }
}

// grid rows, block 1024. sel [rows, 512] ascending positions of the best 512 entries among n = (pos + 1) / ratio (all of
// them when fewer compete); with cand, entries of unmarked blocks do not compete.
__global__ void __launch_bounds__(1024) dsv4_select_kernel(const float* __restrict__ scores, long score_stride,
                                                           const uint8_t* __restrict__ cand, long cand_stride, int cand_block,
                                                           int* __restrict__ sel, int* __restrict__ nsel,
                                                           const int* __restrict__ slot, const int* __restrict__ pos, int ratio) {
  grid_dep_launch();
  grid_dep_wait();
  __shared__ int hist[256];
  __shared__ int wcnt[32], woff[32];
  __shared__ uint32_t s_prefix;
  __shared__ int s_need, s_base, s_base2, s_valid;
  const int r = blockIdx.x, tid = threadIdx.x;
  if (slot[r] < 0) {
    if (tid == 0) nsel[r] = 0;
    return;
  }
  const int n = (pos[r] + 1) / ratio;
  const float* sc = scores + (long)r * score_stride;
  const uint8_t* cd = cand ? cand + (long)r * cand_stride : nullptr;
  int* out = sel + (long)r * kSelTopk;
  auto valid = [&](int i) -> bool { return !cd || cd[i / cand_block] != 0; };
  auto key = [&](int i) -> uint32_t { return valid(i) ? okey(sc[i]) : 0u; };
  if (tid == 0) s_valid = 0;
  __syncthreads();
  int mine = 0;
  for (int i = tid; i < n; i += 1024) mine += valid(i) ? 1 : 0;
  if (mine) atomicAdd(&s_valid, mine);
  __syncthreads();
  const int nvalid = s_valid;
  uint32_t thr = 0;
  int need_eq = 0;
  const bool all = nvalid <= kSelTopk;
  if (!all) radix_threshold(key, n, kSelTopk, thr, need_eq, hist, &s_prefix, &s_need);
  if (tid == 0) s_base = s_base2 = 0;
  __syncthreads();
  for (int c0 = 0; c0 < n; c0 += 1024) {
    const int i = c0 + tid;
    const bool in = i < n && valid(i);
    const uint32_t k = in ? okey(sc[i]) : 0u;
    bool take = in;
    if (!all) {
      const bool eq = in && k == thr;
      int before;
      block_prefix_flag(eq, wcnt, woff, &s_base, before);
      take = in && (k > thr || (eq && before < need_eq));
    }
    int at;
    block_prefix_flag(take, wcnt, woff, &s_base2, at);
    if (take && at < kSelTopk) out[at] = i;
  }
  if (tid == 0) nsel[r] = min(nvalid, kSelTopk);
}

// ------------------------------------------------------------------------------------------------ gather + q + output
// grid ((kKeysMax + 3) / 4, rows), block 256: 64 threads per key, 8 dims each. Key i of a row: window position lo + i for
// i < nwin, then the selected compressed entries, then the sink key (value 0, element 512 = 1).
__global__ void __launch_bounds__(256) dsv4_gather_kernel(const uint8_t* __restrict__ win, int layer, long win_slot_stride,
                                                          const uint8_t* __restrict__ comp, long comp_slot_stride,
                                                          const int* __restrict__ sel, const int* __restrict__ nsel,
                                                          const int* __restrict__ slot, const int* __restrict__ pos,
                                                          __nv_bfloat16* __restrict__ pages, int* __restrict__ nkeys,
                                                          int* __restrict__ v_pos, int* __restrict__ v_slot, int win_floor,
                                                          const int* __restrict__ key_end, int window,
                                                          const __nv_bfloat16* __restrict__ q, long q_stride,
                                                          __nv_bfloat16* __restrict__ q_abs, const float* __restrict__ sink,
                                                          const float* __restrict__ rope, int heads, float scale) {
  grid_dep_launch();
  grid_dep_wait();
  constexpr int kKeyBlocks = (kKeysMax + 3) / 4;
  if (blockIdx.x >= kKeyBlocks) {
    // the blocks past the keys prepare the row's queries (four heads per block, 64 threads each): rope on the last 64
    // dims, element 512 = sink / scale, the rest of the tail zero
    const int r = blockIdx.y, h = (blockIdx.x - kKeyBlocks) * 4 + (threadIdx.x >> 6), l = threadIdx.x & 63, d = 8 * l;
    if (h >= heads) return;
    const __nv_bfloat16* src = q + (long)r * q_stride + (long)h * kHD + d;
    __nv_bfloat16* dst = q_abs + ((long)r * heads + h) * kLatRowD;
    float v[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] = __bfloat162float(src[j]);
    if (d >= kHD - kRopeD) {
      const float* cs = rope + ((long)pos[r] * (kRopeD / 2) + (d - (kHD - kRopeD)) / 2) * 2;
#pragma unroll
      for (int j = 0; j < 4; ++j) rope_pair_cs(v[2 * j], v[2 * j + 1], cs + 2 * j, false);
    }
    __nv_bfloat16 o[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) o[j] = __float2bfloat16_rn(v[j]);
    *reinterpret_cast<uint4*>(dst + d) = *reinterpret_cast<const uint4*>(o);
    if (l < 8) {
      __nv_bfloat16 z[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) z[j] = __float2bfloat16_rn(0.f);
      if (l == 0) z[0] = __float2bfloat16_rn(sink[h] / scale);
      *reinterpret_cast<uint4*>(dst + kHD + 8 * l) = *reinterpret_cast<const uint4*>(z);
    }
    return;
  }
  const int r = blockIdx.y, i = blockIdx.x * 4 + (threadIdx.x >> 6), l = threadIdx.x & 63;
  const int sl = slot[r];
  if (sl < 0) {
    if (blockIdx.x == 0 && threadIdx.x == 0) {
      nkeys[r] = 1;
      v_pos[r] = 0;
      v_slot[r] = -1;
    }
    return;
  }
  // the newest ring position the row may read (its own position unless the caller widens it, as a drafter block does
  // whose rows all see the whole block) and how many positions back from there
  const int p = key_end ? key_end[r] : pos[r];
  const int lo = max(max(0, p - window + 1), win_floor);
  const int nwin = max(0, p + 1 - lo);
  const int ns = (comp && sel) ? nsel[r] : 0;
  const int total = nwin + ns + 1;
  if (blockIdx.x == 0 && threadIdx.x == 0) {   // the row's virtual sequence: slot r of the scratch table, last position total - 1
    nkeys[r] = total;
    v_pos[r] = total - 1;
    v_slot[r] = r;
  }
  if (i >= total) return;
  __nv_bfloat16* dst = pages + (((long)r * kPagesRow + i / 64) * 64 + i % 64) * kLatRowD;
  const int d = 8 * l;
  __nv_bfloat16 v[8];
  if (i < nwin) {
    const uint8_t* row = win + (long)sl * win_slot_stride + ((long)layer * kRing + ((lo + i) % kRing)) * kWinRow;
    const uint2 c = *reinterpret_cast<const uint2*>(row + d);
    const int e = (int)row[kHD + d / 32] - 127;
    const uint32_t w[2] = {c.x, c.y};
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] = __float2bfloat16_rn(ldexpf(e4m3_dec((uint8_t)(w[j / 4] >> (8 * (j % 4)))), e));
  } else if (i < nwin + ns) {
    const int t = sel[(long)r * kSelTopk + (i - nwin)];
    const uint8_t* ent = comp + (long)sl * comp_slot_stride + (long)t * kCompRow;
    const uint32_t c = *reinterpret_cast<const uint32_t*>(ent + d / 2);
    const float s = e4m3_dec(ent[kHD / 2 + d / 16]);
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] = __float2bfloat16_rn(e2m1_dec((c >> (4 * j)) & 15u) * s);
  } else {
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] = __float2bfloat16_rn(0.f);
  }
  *reinterpret_cast<uint4*>(dst + d) = *reinterpret_cast<const uint4*>(v);
  if (l < 8) {
    __nv_bfloat16 z[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) z[j] = __float2bfloat16_rn(0.f);
    if (l == 0 && i == total - 1) z[0] = __float2bfloat16_rn(1.f);
    *reinterpret_cast<uint4*>(dst + kHD + 8 * l) = *reinterpret_cast<const uint4*>(z);
  }
}

// grid (rows, heads), block 64 (8 dims each): rope on the last 64 dims, element 512 = sink / scale (so that the sink key,
// whose element 512 is 1, scores exactly the sink after the kernel's scaling), the rest of the tail zero.
__global__ void __launch_bounds__(64) dsv4_q_prep_kernel(const __nv_bfloat16* __restrict__ q, long q_stride,
                                                         __nv_bfloat16* __restrict__ q_abs, const float* __restrict__ sink,
                                                         const float* __restrict__ rope, const int* __restrict__ pos, int heads,
                                                         float scale) {
  grid_dep_launch();
  grid_dep_wait();
  const int r = blockIdx.x, h = blockIdx.y, l = threadIdx.x, d = 8 * l;
  const __nv_bfloat16* src = q + (long)r * q_stride + (long)h * kHD + d;
  __nv_bfloat16* dst = q_abs + ((long)r * heads + h) * kLatRowD;
  float v[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) v[j] = __bfloat162float(src[j]);
  if (d >= kHD - kRopeD) {
    const float* cs = rope + ((long)pos[r] * (kRopeD / 2) + (d - (kHD - kRopeD)) / 2) * 2;
#pragma unroll
    for (int j = 0; j < 4; ++j) rope_pair_cs(v[2 * j], v[2 * j + 1], cs + 2 * j, false);
  }
  __nv_bfloat16 o[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) o[j] = __float2bfloat16_rn(v[j]);
  *reinterpret_cast<uint4*>(dst + d) = *reinterpret_cast<const uint4*>(o);
  if (l < 8) {
    __nv_bfloat16 z[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) z[j] = __float2bfloat16_rn(0.f);
    if (l == 0) z[0] = __float2bfloat16_rn(sink[h] / scale);
    *reinterpret_cast<uint4*>(dst + kHD + 8 * l) = *reinterpret_cast<const uint4*>(z);
  }
}

// grid (rows, heads), block 128 (4 dims each): inverse rope, MXFP8 value grid, group-major output
// out[g][row][(h % 8) * 512 + d], g = h / 8.
__global__ void __launch_bounds__(128) dsv4_attn_out_kernel(const __nv_bfloat16* __restrict__ o_lat,
                                                            __nv_bfloat16* __restrict__ out, const float* __restrict__ rope,
                                                            const int* __restrict__ pos, const int* __restrict__ slot, int heads,
                                                            int rows) {
  grid_dep_launch();
  grid_dep_wait();
  const int r = blockIdx.x, h = blockIdx.y, t = threadIdx.x, d = 4 * t;
  if (slot[r] < 0) return;
  const __nv_bfloat16* src = o_lat + ((long)r * heads + h) * kHD + d;
  float v[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) v[j] = __bfloat162float(src[j]);
  if (d >= kHD - kRopeD) {
    const float* cs = rope + ((long)pos[r] * (kRopeD / 2) + (d - (kHD - kRopeD)) / 2) * 2;
    rope_pair_cs(v[0], v[1], cs, true);
    rope_pair_cs(v[2], v[3], cs + 2, true);
  }
  float amax = 0.f;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    v[j] = bfr(v[j]);
    amax = fmaxf(amax, fabsf(v[j]));
  }
#pragma unroll
  for (int o = 1; o < 8; o <<= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  const int e = pow2_ceil_exp(fmaxf(amax, 1e-4f) / 448.f);
  __nv_bfloat16* dst = out + ((long)(h / kGroupHeads) * rows + r) * (kGroupHeads * kHD) + (long)(h % kGroupHeads) * kHD + d;
#pragma unroll
  for (int j = 0; j < 4; ++j)
    dst[j] = __float2bfloat16_rn(ldexpf(e4m3_dec(e4m3_enc(fminf(fmaxf(ldexpf(v[j], -e), -448.f), 448.f))), e));
}

// ------------------------------------------------------------------------------------------------ grouped wo_a
// out[row][g * O + r] = sum_d o[g][row][d] * w[g][r][d] for decode rows (rows <= 16): one warp per (g, r) reads its weight
// row once and keeps one accumulator per row. grid (groups * O / 8), block 256. K = 8 heads * 512.
template <int RB>
__global__ void __launch_bounds__(256) dsv4_woa_kernel(const __nv_bfloat16* __restrict__ o, const __nv_bfloat16* __restrict__ w,
                                                       __nv_bfloat16* __restrict__ out, int groups, int O, int rows) {
  grid_dep_launch();
  grid_dep_wait();
  constexpr int KD = kGroupHeads * kHD;
  const int lane = threadIdx.x & 31, gr = blockIdx.x * 8 + (threadIdx.x >> 5);
  if (gr >= groups * O) return;
  const int g = gr / O;
  const __nv_bfloat16* wr = w + (long)gr * KD;
  float acc[RB];
#pragma unroll
  for (int n = 0; n < RB; ++n) acc[n] = 0.f;
  // four 16-byte weight loads in flight per lane before the first use (the weight stream is the only DRAM traffic)
  for (int d0 = lane * 8; d0 < KD; d0 += 1024) {
    uint4 wv[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) wv[u] = __ldg(reinterpret_cast<const uint4*>(wr + d0 + u * 256));
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const __nv_bfloat162* w2 = reinterpret_cast<const __nv_bfloat162*>(&wv[u]);
#pragma unroll
      for (int n = 0; n < RB; ++n) {
        if (n < rows) {
          const uint4 xv = *reinterpret_cast<const uint4*>(o + ((long)g * rows + n) * KD + d0 + u * 256);
          const __nv_bfloat162* x2 = reinterpret_cast<const __nv_bfloat162*>(&xv);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float2 a = __bfloat1622float2(w2[j]), b = __bfloat1622float2(x2[j]);
            acc[n] += a.x * b.x + a.y * b.y;
          }
        }
      }
    }
  }
#pragma unroll
  for (int n = 0; n < RB; ++n) {
    if (n < rows) {
      const float v = warp_sum(acc[n]);
      if (lane == 0) out[(long)n * groups * O + gr] = __float2bfloat16_rn(v);
    }
  }
}

// ------------------------------------------------------------------------------------------------ engram ids
// One block (rows <= 1024): every row records its token in the per-slot history, then hashes the last `ngram` tokens of its
// sequence into one table row per engram layer. Positions before the sequence start count as token 2 (the pad id).
__global__ void __launch_bounds__(1024) dsv4_engram_ids_kernel(const int* __restrict__ ids, const int* __restrict__ slot,
                                                               const int* __restrict__ pos, int* __restrict__ hist, long hist_stride,
                                                               int spare_slot, int* __restrict__ out, int tables, int table_rows,
                                                               int ngram, int rows) {
  grid_dep_launch();
  grid_dep_wait();
  const int r = threadIdx.x;
  int sl = 0, p = 0;
  if (r < rows) {
    sl = slot[r] < 0 ? spare_slot : slot[r];
    p = pos[r];
    hist[(long)sl * hist_stride + p] = ids[r];
  }
  __syncthreads();
  if (r >= rows) return;
  long long h = 0;
  for (int j = 0; j < ngram; ++j) {
    const long long t = p - j >= 0 ? (long long)hist[(long)sl * hist_stride + (p - j)] : 2ll;
    h = (h * 1000003ll + t * (2 * j + 1) + 12345ll) % 2147483647ll;
  }
  for (int i = 0; i < tables; ++i) out[(long)r * tables + i] = (int)((h * (2 * i + 3) + i) % table_rows);
}

// ------------------------------------------------------------------------------------------------ engram gate
// grid (rows, hc), block 256. kv [rows, (hc + 1) * H] = [key 0..hc-1 | value]; streams fp32 [rows, hc, H] in place.
__global__ void __launch_bounds__(256) dsv4_engram_gate_kernel(float* __restrict__ streams, const __nv_bfloat16* __restrict__ kv,
                                                               const float* __restrict__ w, const uint8_t* __restrict__ skip,
                                                               int H, int hc, float eps) {
  grid_dep_launch();
  grid_dep_wait();
  __shared__ float red[33];
  const int r = blockIdx.x, h = blockIdx.y;
  if (skip && skip[r]) return;
  float* s = streams + ((long)r * hc + h) * H;
  const __nv_bfloat16* key = kv + (long)r * (hc + 1) * H + (long)h * H;
  const __nv_bfloat16* val = kv + (long)r * (hc + 1) * H + (long)hc * H;
  const float* wh = w + (long)h * H;
  float ss = 0.f, kk = 0.f, dot = 0.f;
  for (int d = threadIdx.x; d < H; d += 256) {
    const float a = s[d], k = __bfloat162float(key[d]);
    ss += a * a;
    kk += k * k;
    dot += a * wh[d] * k;
  }
  ss = block_sum(ss, red);
  kk = block_sum(kk, red);
  dot = block_sum(dot, red);
  dot = dot * rsqrtf(ss / (float)H + eps) * rsqrtf(kk / (float)H + eps) * rsqrtf((float)H);
  const float z = copysignf(sqrtf(fmaxf(fabsf(dot), 1e-6f)), dot);
  const float gate = 1.f / (1.f + __expf(-z));
  for (int d = threadIdx.x; d < H; d += 256) s[d] += gate * __bfloat162float(val[d]);
}

}  // namespace ve

using namespace ve;

extern "C" {

int ve_dsv4_window_store(const void* kv, long kv_stride, void* ring, const void* rope, const void* slot, const void* pos, int layer,
                         long slot_stride, int rows, const void* norm_w, float eps, float wbias, cudaStream_t st) {
  if (rows <= 0) return 0;
  launch_pdl(dsv4_window_store_kernel, dim3(rows), dim3(128), 0, st, (const __nv_bfloat16*)kv, kv_stride, (uint8_t*)ring, (const float*)rope,
                                                 (const int*)slot, (const int*)pos, layer, slot_stride, (const __nv_bfloat16*)norm_w, eps, wbias);
  VE_CHECK_LAUNCH();
}

int ve_dsv4_cring_store(const void* ckv, long ckv_stride, const void* csc, long csc_stride, void* ring_kv, void* ring_sc,
                        const void* slot, const void* pos, long slot_stride, int rows, int unused, cudaStream_t st) {
  (void)unused;
  if (rows <= 0) return 0;
  launch_pdl(dsv4_cring_store_kernel, dim3(rows), dim3(128), 0, st, (const __nv_bfloat16*)ckv, ckv_stride, (const __nv_bfloat16*)csc, csc_stride,
                                                (float*)ring_kv, (float*)ring_sc, (const int*)slot, (const int*)pos, slot_stride);
  VE_CHECK_LAUNCH();
}

int ve_dsv4_compress(const void* ckv, long ckv_stride, const void* ring_kv, const void* ring_sc, const void* norm_w,
                     void* latent_out, void* comp, const void* rope, const void* slot, const void* pos, long ring_slot_stride,
                     long comp_slot_stride, int ratio, float eps, int rows, cudaStream_t st) {
  if (rows <= 0) return 0;
  if (ratio < 1 || (ratio > 1 && (!ring_kv || !ring_sc))) return cudaErrorInvalidValue;
  launch_pdl(dsv4_compress_kernel, dim3(rows), dim3(128), 0, st, (const __nv_bfloat16*)ckv, ckv_stride, (const float*)ring_kv, (const float*)ring_sc,
                                             (const __nv_bfloat16*)norm_w, (__nv_bfloat16*)latent_out, (uint8_t*)comp,
                                             (const float*)rope, (const int*)slot, (const int*)pos, ring_slot_stride,
                                             comp_slot_stride, ratio, eps);
  VE_CHECK_LAUNCH();
}

int ve_dsv4_index_key_store(const void* kraw, long kraw_stride, const void* norm_w, void* idxk, const void* rope, const void* slot,
                            const void* pos, const void* unused, long slot_stride, int ratio, float eps, int rows,
                            cudaStream_t st) {
  (void)unused;
  if (rows <= 0) return 0;
  launch_pdl(dsv4_index_key_kernel, dim3(rows), dim3(128), 0, st, (const __nv_bfloat16*)kraw, kraw_stride, (const __nv_bfloat16*)norm_w,
                                              (__nv_bfloat16*)idxk, (const float*)rope, (const int*)slot, (const int*)pos,
                                              slot_stride, ratio, eps);
  VE_CHECK_LAUNCH();
}

int ve_dsv4_index_q(const void* q, long q_stride, void* out, const void* rope, const void* pos, int rows, cudaStream_t st) {
  if (rows <= 0) return 0;
  launch_pdl(dsv4_index_q_kernel, dim3(rows, kIdxHeads), dim3(128), 0, st, (const __nv_bfloat16*)q, q_stride, (__nv_bfloat16*)out,
                                                             (const float*)rope, (const int*)pos);
  VE_CHECK_LAUNCH();
}

int ve_dsv4_candidates(const void* scores, long score_stride, void* cand, long cand_stride, const void* slot, const void* pos,
                       int ratio, int blocks, int block, int rows, cudaStream_t st) {
  if (rows <= 0) return 0;
  if (blocks < 1 || block < 1) return cudaErrorInvalidValue;
  launch_pdl(dsv4_candidates_kernel, dim3(rows), dim3(1024), 0, st, (const float*)scores, score_stride, (uint8_t*)cand, cand_stride, (const int*)slot,
                                                (const int*)pos, ratio, blocks, block);
  VE_CHECK_LAUNCH();
}

int ve_dsv4_select(const void* scores, long score_stride, const void* cand, long cand_stride, int cand_block, void* sel, void* nsel,
                   const void* slot, const void* pos, int ratio, int rows, cudaStream_t st) {
  if (rows <= 0) return 0;
  if (cand && cand_block < 1) return cudaErrorInvalidValue;
  launch_pdl(dsv4_select_kernel, dim3(rows), dim3(1024), 0, st, (const float*)scores, score_stride, (const uint8_t*)cand, cand_stride, cand_block,
                                            (int*)sel, (int*)nsel, (const int*)slot, (const int*)pos, ratio);
  VE_CHECK_LAUNCH();
}

int ve_dsv4_gather(const void* win, int layer, long win_slot_stride, const void* comp, long comp_slot_stride, const void* sel,
                   const void* nsel, const void* slot, const void* pos, void* pages, void* nkeys, void* v_pos, void* v_slot,
                   int win_floor, int rows, const void* key_end, int window, const void* q, long q_stride, void* q_abs,
                   const void* sink, const void* rope, int heads, float scale, cudaStream_t st) {
  if (rows <= 0) return 0;
  if (window < 1 || window + kSelTopk + 1 > kPagesRow * 64 || window > kRing) return cudaErrorInvalidValue;
  launch_pdl(dsv4_gather_kernel, dim3((kKeysMax + 3) / 4 + (q ? (heads + 3) / 4 : 0), rows), dim3(256), 0, st, (const uint8_t*)win, layer, win_slot_stride,
                                                                     (const uint8_t*)comp, comp_slot_stride, (const int*)sel,
                                                                     (const int*)nsel, (const int*)slot, (const int*)pos,
                                                                     (__nv_bfloat16*)pages, (int*)nkeys, (int*)v_pos,
                                                                     (int*)v_slot, win_floor, (const int*)key_end, window, (const __nv_bfloat16*)q, q_stride,
                                                                     (__nv_bfloat16*)q_abs, (const float*)sink, (const float*)rope, heads, scale);
  VE_CHECK_LAUNCH();
}

int ve_dsv4_q_prep(const void* q, long q_stride, void* q_abs, const void* sink, const void* rope, const void* pos, int heads,
                   float scale, int rows, cudaStream_t st) {
  if (rows <= 0) return 0;
  launch_pdl(dsv4_q_prep_kernel, dim3(rows, heads), dim3(64), 0, st, (const __nv_bfloat16*)q, q_stride, (__nv_bfloat16*)q_abs, (const float*)sink,
                                                       (const float*)rope, (const int*)pos, heads, scale);
  VE_CHECK_LAUNCH();
}

int ve_dsv4_attn_out(const void* o_lat, void* out, const void* rope, const void* pos, const void* slot, int heads, int rows,
                     cudaStream_t st) {
  if (rows <= 0) return 0;
  launch_pdl(dsv4_attn_out_kernel, dim3(rows, heads), dim3(128), 0, st, (const __nv_bfloat16*)o_lat, (__nv_bfloat16*)out, (const float*)rope,
                                                          (const int*)pos, (const int*)slot, heads, rows);
  VE_CHECK_LAUNCH();
}

int ve_dsv4_woa(const void* o, const void* w, void* out, int groups, int O, int rows, cudaStream_t st) {
  if (rows <= 0) return 0;
  if (rows > 16) return cudaErrorInvalidValue;
  const int grid = (groups * O + 7) / 8;
  const __nv_bfloat16 *op = (const __nv_bfloat16*)o, *wp = (const __nv_bfloat16*)w;
  if (rows <= 1) launch_pdl(dsv4_woa_kernel<1>, dim3(grid), dim3(256), 0, st, op, wp, (__nv_bfloat16*)out, groups, O, rows);
  else if (rows <= 4) launch_pdl(dsv4_woa_kernel<4>, dim3(grid), dim3(256), 0, st, op, wp, (__nv_bfloat16*)out, groups, O, rows);
  else launch_pdl(dsv4_woa_kernel<16>, dim3(grid), dim3(256), 0, st, op, wp, (__nv_bfloat16*)out, groups, O, rows);
  VE_CHECK_LAUNCH();
}

int ve_dsv4_engram_ids(const void* ids, const void* slot, const void* pos, void* hist, long hist_stride, int spare_slot, void* out,
                       int tables, int table_rows, int ngram, int rows, cudaStream_t st) {
  if (rows <= 0) return 0;
  if (rows > 1024 || tables < 1 || table_rows < 1) return cudaErrorInvalidValue;
  launch_pdl(dsv4_engram_ids_kernel, dim3(1), dim3(1024), 0, st, (const int*)ids, (const int*)slot, (const int*)pos, (int*)hist, hist_stride, spare_slot,
                                             (int*)out, tables, table_rows, ngram, rows);
  VE_CHECK_LAUNCH();
}

int ve_dsv4_engram_gate(void* streams, const void* kv, const void* w, const void* skip, int H, int hc, float eps, int rows,
                        cudaStream_t st) {
  if (rows <= 0) return 0;
  launch_pdl(dsv4_engram_gate_kernel, dim3(rows, hc), dim3(256), 0, st, (float*)streams, (const __nv_bfloat16*)kv, (const float*)w,
                                                          (const uint8_t*)skip, H, hc, eps);
  VE_CHECK_LAUNCH();
}

}  // extern "C"
