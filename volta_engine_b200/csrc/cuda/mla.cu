// Multi-head latent attention (MLA) with a decoupled RoPE key, in absorbed form over a paged latent cache.
//
// Cache row per token and layer: [c_kv (kv_lora = 512) | k_rope (64)] bf16 = 1152 bytes, shared by all heads.
// Per head h:  score = (q_nope[h] W_uk[h]) . c_kv + q_rope[h] . k_rope ;  out[h] = (softmax . c_kv) W_uv[h]^T.
// The reference implements the rope-free GLM variant (inc/engine/modules/mla.h:13-49,
// src/backend/cuda/modules/mla_latent.cu: absorb_q / latent_attn / expand_out / latent_reduce); the rope key and
// the 576-wide score are this engine's addition for DeepSeek-style checkpoints.
//
// Kernels: mla_rope_store (rotate q_rope / k_rope, write the latent row), mla_absorb_q (per-head 128 -> 512
// product), mla_decode (split-KV attention for decode / verify rows: 16 (token, head) rows per CTA, one page of
// 64 keys per step fetched by TMA into 128B-swizzled shared memory and used both as K and as V; the four warps
// split the keys for Q.K^T and the 512 latent columns for P.V), mla_expand_out (512 -> 128 per head).
// Split partials are merged by the shared attn_reduce kernel. Prefill chunks expand K/V per head and use the
// dense GQA kernel (see models/mla.py).
#include "common.cuh"
#include "tmap.h"
#include <float.h>

namespace ve {

constexpr int kLat = 512, kRope = 64, kLatRow = 576, kMlaPage = 64;

// grid (rows, heads + 1): blocks [0, heads) rotate q_rope of one head in place; block `heads` rotates k_rope and
// writes the latent row. q [rows, heads, q_dim] with the rope part at [q_dim - 64, q_dim). 32 threads per block.
__global__ void mla_rope_store_kernel(__nv_bfloat16* __restrict__ q, long q_stride, int q_dim, int heads,
                                      const __nv_bfloat16* __restrict__ ckv, long ckv_stride,
                                      const __nv_bfloat16* __restrict__ krope, long krope_stride,
                                      const int* __restrict__ pos, const int* __restrict__ slot,
                                      const int* __restrict__ page_table, int max_pages, __nv_bfloat16* __restrict__ pool,
                                      float theta, int interleaved) {
  const int row = blockIdx.x, h = blockIdx.y, i = threadIdx.x;   // i: rotation pair 0..31
  const int p = pos[row];
  const float inv_freq = exp2f(-log2f(theta) * (2.f * (float)i / (float)kRope));
  float sn, cs;
  sincosf((float)p * inv_freq, &sn, &cs);
  const int i0 = interleaved ? 2 * i : i, i1 = interleaved ? 2 * i + 1 : i + kRope / 2;
  if (h < heads) {
    __nv_bfloat16* v = q + (long)row * q_stride + (long)h * q_dim + (q_dim - kRope);
    const float a0 = bf2f(v[i0]), a1 = bf2f(v[i1]);
    // output always in half-split order so that q and k agree whatever the checkpoint's pairing
    v[i0] = f2bf(a0 * cs - a1 * sn);
    v[i1] = f2bf(a1 * cs + a0 * sn);
    return;
  }
  const int s = slot ? slot[row] : 0;
  if (s < 0) return;
  const int page = page_table[(long)s * max_pages + p / kMlaPage];
  __nv_bfloat16* dst = pool + ((long)page * kMlaPage + (p % kMlaPage)) * kLatRow;
  const __nv_bfloat16* kr = krope + (long)row * krope_stride;
  const float a0 = bf2f(kr[i0]), a1 = bf2f(kr[i1]);
  dst[kLat + i0] = f2bf(a0 * cs - a1 * sn);
  dst[kLat + i1] = f2bf(a1 * cs + a0 * sn);
  const __nv_bfloat16* c = ckv + (long)row * ckv_stride;
  for (int j = i * 16; j < i * 16 + 16; j += 8) *reinterpret_cast<bf16x8*>(dst + j) = *reinterpret_cast<const bf16x8*>(c + j);
}

// q_abs[row, h, 0:512] = q[row, h, 0:nope] @ W_uk[h] (nope x 512) ; q_abs[row, h, 512:576] = q_rope.
// grid (rows, heads), 128 threads: thread t owns 4 latent columns.
__global__ void mla_absorb_q_kernel(const __nv_bfloat16* __restrict__ q, long q_stride, int q_dim, int nope,
                                    const __nv_bfloat16* __restrict__ w_uk, __nv_bfloat16* __restrict__ q_abs, int heads) {
  __shared__ float qs[256];
  const int row = blockIdx.x, h = blockIdx.y;
  const __nv_bfloat16* qv = q + (long)row * q_stride + (long)h * q_dim;
  for (int i = threadIdx.x; i < nope; i += blockDim.x) qs[i] = bf2f(qv[i]);
  __syncthreads();
  const __nv_bfloat16* w = w_uk + (long)h * nope * kLat;
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
  const int c0 = threadIdx.x * 4;
#pragma unroll 8                                   // eight independent row loads in flight (the loop is latency-bound)
  for (int d = 0; d < nope; ++d) {
    const uint2 t = *reinterpret_cast<const uint2*>(w + (long)d * kLat + c0);
    const float qd = qs[d];
    acc[0] = fmaf(qd, __uint_as_float(t.x << 16), acc[0]);
    acc[1] = fmaf(qd, __uint_as_float(t.x & 0xffff0000u), acc[1]);
    acc[2] = fmaf(qd, __uint_as_float(t.y << 16), acc[2]);
    acc[3] = fmaf(qd, __uint_as_float(t.y & 0xffff0000u), acc[3]);
  }
  __nv_bfloat16* o = q_abs + ((long)row * heads + h) * kLatRow;
  *reinterpret_cast<__nv_bfloat162*>(o + c0) = __floats2bfloat162_rn(acc[0], acc[1]);
  *reinterpret_cast<__nv_bfloat162*>(o + c0 + 2) = __floats2bfloat162_rn(acc[2], acc[3]);
  if (threadIdx.x < kRope) o[kLat + threadIdx.x] = qv[q_dim - kRope + threadIdx.x];
}

// out[row, h, 0:vdim] = o_lat[row, h, 0:512] @ W_uv[h]^T  (W_uv [heads, vdim, 512]). grid (rows, heads), vdim threads.
__global__ void mla_expand_out_kernel(const __nv_bfloat16* __restrict__ o_lat, const __nv_bfloat16* __restrict__ w_uv,
                                      __nv_bfloat16* __restrict__ out, long out_stride, int heads, int vdim) {
  __shared__ float os[kLat];
  const int row = blockIdx.x, h = blockIdx.y;
  const __nv_bfloat16* o = o_lat + ((long)row * heads + h) * kLat;
  for (int i = threadIdx.x; i < kLat; i += blockDim.x) os[i] = bf2f(o[i]);
  __syncthreads();
  const int v = threadIdx.x;
  if (v >= vdim) return;
  const __nv_bfloat16* w = w_uv + ((long)h * vdim + v) * kLat;
  float acc = 0.f;
#pragma unroll 8
  for (int c = 0; c < kLat; c += 8) {
    const bf16x8 t = *reinterpret_cast<const bf16x8*>(w + c);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 f = __bfloat1622float2(t.v[j]);
      acc = fmaf(f.x, os[c + 2 * j], acc);
      acc = fmaf(f.y, os[c + 2 * j + 1], acc);
    }
  }
  out[(long)row * out_stride + (long)h * vdim + v] = f2bf(acc);
}

struct MlaParams {
  const __nv_bfloat16* q_abs;   // [rows, heads, 576]
  float* o_part;                // [rows, heads, nsplit, 512]
  float* lse_part;              // [rows, heads, nsplit]
  const int* pos;
  const int* slot;
  const int* page_table;
  int max_pages, heads, nsplit;
  float scale_log2;
  int* status;
};

VE_DEVINL void m_ldsm_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
VE_DEVINL void m_ldsm_x4_t(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
VE_DEVINL void m_mma(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

constexpr int kQPitch = kLatRow * 2 + 16;     // bytes per Q row in shared memory (padded against bank conflicts)
constexpr int kMlaTile = kMlaPage * kLatRow * 2;   // 73728 bytes: 9 sub-tiles of 64 keys x 128 B
constexpr int kSPitch = 68;                    // floats per row of the score exchange buffer

// grid (tokens * slabs_per_token, nsplit), 128 threads.
__global__ void __launch_bounds__(128) mla_decode_kernel(const MlaParams p, const __grid_constant__ CUtensorMap kmap) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* ktile[2] = {smem, smem + kMlaTile};
  uint8_t* qs = smem + 2 * kMlaTile;                         // 16 x kQPitch
  float* ss = reinterpret_cast<float*>(qs + 16 * kQPitch);   // 16 x kSPitch
  __shared__ uint64_t full[2];

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, t = lane & 3;
  const int slabs = (p.heads + 15) / 16;
  const int tok = blockIdx.x / slabs, head0 = (blockIdx.x % slabs) * 16, z = blockIdx.y;
  const int s = p.slot ? p.slot[tok] : 0;
  if (s < 0) return;
  const int ps = p.pos[tok];
  const int ntile_all = ps / kMlaPage + 1;
  const int tps = (ntile_all + p.nsplit - 1) / p.nsplit;
  const int kt_begin = z * tps, kt_end = min(ntile_all, kt_begin + tps);

  if (tid == 0) {
    mbar_init(&full[0], 1);
    mbar_init(&full[1], 1);
    mbar_fence_init();
  }
  // Q rows of this slab into shared memory (zero rows beyond the head count)
  for (int i = tid; i < 16 * (kLatRow / 8); i += 128) {
    const int r = i / (kLatRow / 8), c = (i % (kLatRow / 8)) * 8;
    bf16x8 v;
    if (head0 + r < p.heads) v = *reinterpret_cast<const bf16x8*>(p.q_abs + ((long)tok * p.heads + head0 + r) * kLatRow + c);
    else v.v[0] = v.v[1] = v.v[2] = v.v[3] = __floats2bfloat162_rn(0.f, 0.f);
    *reinterpret_cast<bf16x8*>(qs + r * kQPitch + c * 2) = v;
  }
  __syncthreads();
  auto issue = [&](int kt, int stage) {
    const int page = p.page_table[(long)s * p.max_pages + kt];
    mbar_expect_tx(&full[stage], kMlaTile);
#pragma unroll
    for (int c = 0; c < kLatRow / 64; ++c) tma_load_2d(ktile[stage] + c * 8192, &kmap, &full[stage], c * 64, page * kMlaPage);
  };
  if (tid == 0 && kt_begin < kt_end) issue(kt_begin, 0);

  float o[16][4];
#pragma unroll
  for (int i = 0; i < 16; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m_run[2] = {-FLT_MAX, -FLT_MAX}, l_run[2] = {0.f, 0.f};
  const uint32_t q_base = smem_u32(qs);
  bool failed = false;

  for (int kt = kt_begin; kt < kt_end; ++kt) {
    const int it = kt - kt_begin, stage = it & 1;
    const bool ok = mbar_wait(&full[stage], (it >> 1) & 1);
    if (!__syncthreads_and(ok)) { failed = true; break; }       // also: everyone is done with the other stage and ss
    if (tid == 0 && kt + 1 < kt_end) issue(kt + 1, stage ^ 1);
    const uint32_t kb = smem_u32(ktile[stage]);
    // ---- scores of this warp's 16 keys over the 576-wide row
    float sacc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll 4
    for (int kk = 0; kk < kLatRow / 16; ++kk) {
      uint32_t a[4];
      {
        const int mi = lane >> 3, rr = lane & 7;     // matrices: (rows 0-7,k lo) (rows 8-15,k lo) (rows 0-7,k hi) (rows 8-15,k hi)
        const int row = (mi & 1) * 8 + rr, col = kk * 16 + (mi >> 1) * 8;
        m_ldsm_x4(q_base + row * kQPitch + col * 2, a[0], a[1], a[2], a[3]);
      }
      const int c = (kk * 16) / 64, ci = ((kk * 16) % 64) / 8;
      const int mi = lane >> 3, rr = lane & 7;
      const int key = warp * 16 + (mi >> 1) * 8 + rr;
      const int ch = ci + (mi & 1);
      uint32_t b0, b1, b2, b3;
      m_ldsm_x4(kb + c * 8192 + key * 128 + ((ch ^ (key & 7)) << 4), b0, b1, b2, b3);
      m_mma(sacc[0], a, b0, b1);
      m_mma(sacc[1], a, b2, b3);
    }
#pragma unroll
    for (int nt = 0; nt < 2; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int row = g + (e >> 1) * 8, key_l = warp * 16 + nt * 8 + 2 * t + (e & 1);
        const int key = kt * kMlaPage + key_l;
        ss[row * kSPitch + key_l] = key <= ps ? sacc[nt][e] * p.scale_log2 : -FLT_MAX;
      }
    __syncthreads();
    // ---- every warp: softmax statistics of its two rows over all 64 keys, P fragments
    float sv[8][4];
    float mx[2] = {-FLT_MAX, -FLT_MAX};
#pragma unroll
    for (int nt = 0; nt < 8; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int h = e >> 1;
        const float v = ss[(g + h * 8) * kSPitch + nt * 8 + 2 * t + (e & 1)];
        sv[nt][e] = v;
        mx[h] = fmaxf(mx[h], v);
      }
    float corr[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
      mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
      const float m_new = fmaxf(m_run[h], mx[h]);
      corr[h] = (m_run[h] == -FLT_MAX) ? 0.f : exp2f(m_run[h] - m_new);
      m_run[h] = m_new;
      l_run[h] *= corr[h];
    }
    uint32_t pf[4][4];
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) {
      float pv[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int h = e >> 1;
        pv[e] = (sv[nt][e] == -FLT_MAX) ? 0.f : exp2f(sv[nt][e] - m_run[h]);
        l_run[h] += pv[e];
      }
      __nv_bfloat162 lo = __floats2bfloat162_rn(pv[0], pv[1]), hi = __floats2bfloat162_rn(pv[2], pv[3]);
      pf[nt >> 1][(nt & 1) * 2 + 0] = *reinterpret_cast<uint32_t*>(&lo);
      pf[nt >> 1][(nt & 1) * 2 + 1] = *reinterpret_cast<uint32_t*>(&hi);
    }
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      o[i][0] *= corr[0];
      o[i][1] *= corr[0];
      o[i][2] *= corr[1];
      o[i][3] *= corr[1];
    }
    // ---- O[:, warp*128 .. +128) += P . C   (the latent part of the same tile is V)
#pragma unroll
    for (int ks = 0; ks < 4; ++ks)
#pragma unroll
      for (int dp = 0; dp < 8; ++dp) {
        const int mi = lane >> 3, rr = lane & 7;
        const int key = ks * 16 + (mi & 1) * 8 + rr;
        const int d = warp * 128 + dp * 16 + (mi >> 1) * 8;
        const int c = d / 64, ch = (d % 64) / 8;
        uint32_t b0, b1, b2, b3;
        m_ldsm_x4_t(kb + c * 8192 + key * 128 + ((ch ^ (key & 7)) << 4), b0, b1, b2, b3);
        m_mma(o[2 * dp], pf[ks], b0, b1);
        m_mma(o[2 * dp + 1], pf[ks], b2, b3);
      }
  }
  if (failed) {
    if (tid == 0 && p.status) atomicExch(p.status, (int)kErrMbarTimeout);
    return;
  }
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 1);
    l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 2);
  }
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int head = head0 + g + h * 8;
    if (head >= p.heads) continue;
    const float inv = l_run[h] > 0.f ? 1.f / l_run[h] : 0.f;
    const long base = ((long)tok * p.heads + head) * p.nsplit + z;
    float* orow = p.o_part + base * kLat + warp * 128;
#pragma unroll
    for (int nt = 0; nt < 16; ++nt)
      *reinterpret_cast<float2*>(orow + nt * 8 + 2 * t) = make_float2(o[nt][2 * h] * inv, o[nt][2 * h + 1] * inv);
    if (warp == 0 && t == 0) p.lse_part[base] = l_run[h] > 0.f ? m_run[h] + log2f(l_run[h]) : -FLT_MAX;
  }
}

// Merge of split partials (same rule as the GQA reduce): grid rows*heads, 512 threads, output bf16 [rows, heads, 512].
__global__ void mla_reduce_kernel(const float* __restrict__ o_part, const float* __restrict__ lse_part,
                                  __nv_bfloat16* __restrict__ out, const int* __restrict__ slot, int heads, int nsplit) {
  const int row = blockIdx.x / heads, d = threadIdx.x;
  if (slot && slot[row] < 0) return;
  const long base = (long)blockIdx.x * nsplit;
  float mx = -FLT_MAX;
  for (int i = 0; i < nsplit; ++i) mx = fmaxf(mx, lse_part[base + i]);
  float acc = 0.f, wsum = 0.f;
  for (int i = 0; i < nsplit; ++i) {
    const float l = lse_part[base + i];
    const float w = (l == -FLT_MAX) ? 0.f : exp2f(l - mx);
    wsum += w;
    acc += w * o_part[(base + i) * kLat + d];
  }
  out[(long)blockIdx.x * kLat + d] = f2bf(wsum > 0.f ? acc / wsum : 0.f);
}

}  // namespace ve

using namespace ve;

extern "C" {

int ve_mla_rope_store(void* q, long q_stride, int q_dim, int heads, const void* ckv, long ckv_stride, const void* krope,
                      long krope_stride, const void* pos, const void* slot, const void* page_table, int max_pages,
                      void* pool, int rows, float theta, int interleaved, cudaStream_t st) {
  if (rows <= 0) return 0;
  dim3 grid(rows, heads + 1);
  mla_rope_store_kernel<<<grid, 32, 0, st>>>((__nv_bfloat16*)q, q_stride, q_dim, heads, (const __nv_bfloat16*)ckv, ckv_stride,
                                             (const __nv_bfloat16*)krope, krope_stride, (const int*)pos, (const int*)slot,
                                             (const int*)page_table, max_pages, (__nv_bfloat16*)pool, theta, interleaved);
  VE_CHECK_LAUNCH();
}

int ve_mla_absorb_q(const void* q, long q_stride, int q_dim, int nope, const void* w_uk, void* q_abs, int rows, int heads,
                    cudaStream_t st) {
  if (rows <= 0) return 0;
  if (nope > 256) return cudaErrorInvalidValue;
  dim3 grid(rows, heads);
  mla_absorb_q_kernel<<<grid, 128, 0, st>>>((const __nv_bfloat16*)q, q_stride, q_dim, nope, (const __nv_bfloat16*)w_uk,
                                            (__nv_bfloat16*)q_abs, heads);
  VE_CHECK_LAUNCH();
}

int ve_mla_expand_out(const void* o_lat, const void* w_uv, void* out, long out_stride, int rows, int heads, int vdim,
                      cudaStream_t st) {
  if (rows <= 0) return 0;
  if (vdim > 256) return cudaErrorInvalidValue;
  dim3 grid(rows, heads);
  mla_expand_out_kernel<<<grid, ((vdim + 31) / 32) * 32, 0, st>>>((const __nv_bfloat16*)o_lat, (const __nv_bfloat16*)w_uv,
                                                                  (__nv_bfloat16*)out, out_stride, heads, vdim);
  VE_CHECK_LAUNCH();
}

// q_abs [rows, heads, 576] -> o_lat [rows, heads, 512] bf16. Scratch: o_part rows*heads*nsplit*512 floats,
// lse_part rows*heads*nsplit floats.
int ve_mla_decode(const void* q_abs, void* o_lat, void* o_part, void* lse_part, const void* pos, const void* slot,
                  const void* page_table, int max_pages, void* pool, long pool_pages, int rows, int heads, int nsplit,
                  float scale, void* status, cudaStream_t st) {
  if (rows <= 0) return 0;
  MlaParams p;
  p.q_abs = (const __nv_bfloat16*)q_abs;
  p.o_part = (float*)o_part;
  p.lse_part = (float*)lse_part;
  p.pos = (const int*)pos;
  p.slot = (const int*)slot;
  p.page_table = (const int*)page_table;
  p.max_pages = max_pages;
  p.heads = heads;
  p.nsplit = nsplit;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.status = (int*)status;
  CUtensorMap kmap;
  int rc = make_tmap_2d(&kmap, pool, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)pool_pages * kMlaPage, kLatRow,
                        (uint64_t)kLatRow * 2, kMlaPage, 64, CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc) return rc;
  constexpr int smem = 2 * kMlaTile + 16 * kQPitch + 16 * kSPitch * 4 + 1024;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(mla_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return (int)e;
    attr_set = true;
  }
  const int slabs = (heads + 15) / 16;
  dim3 grid(rows * slabs, nsplit);
  mla_decode_kernel<<<grid, 128, smem, st>>>(p, kmap);
  rc = (int)cudaGetLastError();
  if (rc) return rc;
  mla_reduce_kernel<<<rows * heads, kLat, 0, st>>>((const float*)o_part, (const float*)lse_part, (__nv_bfloat16*)o_lat,
                                                   (const int*)slot, heads, nsplit);
  VE_CHECK_LAUNCH();
}

}  // extern "C"
