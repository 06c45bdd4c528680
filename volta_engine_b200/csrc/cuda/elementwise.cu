// Memory-bound row kernels: RMSNorm (plain / fused residual add / per-head), embedding gather,
// RoPE fused with the paged KV-cache store, SwiGLU / GELU-tanh gating, residual add, soft-cap.
// Math follows the reference definitions: inc/engine/modules/norm.h:9-31 (RMSNorm with a constant
// weight bias), inc/engine/backend/cuda/rope_math.cuh:9-27 (inv_freq = base^(-2i/rot_dim), NeoX or
// interleaved pairing, partial rotary), src/backend/cuda/modules/swiglu.cu:10-30 (clamped SwiGLU,
// GELU-tanh variant). All arithmetic is fp32; storage is bf16.
#include "common.cuh"
#include <cuda_fp8.h>

namespace ve {

// ------------------------------------------------------------------------------------------------
// RMSNorm. One CTA per row. Optional fused residual: res = res + x (+ x2); out = norm(res).
// `res` may be fp32 (res_f32 != 0) or bf16. x may be null when only normalising `res`.
// ------------------------------------------------------------------------------------------------
template <int VEC>
__global__ void __launch_bounds__(256) rmsnorm_kernel(const __nv_bfloat16* __restrict__ x, void* __restrict__ res,
                                                      int res_f32, const __nv_bfloat16* __restrict__ w,
                                                      __nv_bfloat16* __restrict__ out, int H, float eps,
                                                      float wbias, long x_stride, long out_stride) {
  __shared__ float red[33];
  extern __shared__ float rowbuf[];  // H floats
  grid_dep_wait();                   // inputs come from the kernel in front
  grid_dep_launch();                 // the kernel behind this one may be scheduled and set up now
  const long row = blockIdx.x;
  const __nv_bfloat16* xr = x ? x + row * x_stride : nullptr;
  float ss = 0.f;
  for (int i = threadIdx.x * VEC; i < H; i += blockDim.x * VEC) {
    float v[VEC];
#pragma unroll
    for (int j = 0; j < VEC; ++j) v[j] = 0.f;
    if (xr) {
      bf16x8 t = *reinterpret_cast<const bf16x8*>(xr + i);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float2 f = __bfloat1622float2(t.v[j]);
        v[2 * j] = f.x;
        v[2 * j + 1] = f.y;
      }
    }
    if (res) {
      if (res_f32) {
        float* rr = reinterpret_cast<float*>(res) + row * (long)H + i;
#pragma unroll
        for (int j = 0; j < VEC; ++j) {
          v[j] += rr[j];
          rr[j] = v[j];
        }
      } else {
        __nv_bfloat16* rr = reinterpret_cast<__nv_bfloat16*>(res) + row * (long)H + i;
        bf16x8 t = *reinterpret_cast<const bf16x8*>(rr);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          float2 f = __bfloat1622float2(t.v[j]);
          v[2 * j] += f.x;
          v[2 * j + 1] += f.y;
        }
        if (xr) {
          bf16x8 o;
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            o.v[j] = __floats2bfloat162_rn(v[2 * j], v[2 * j + 1]);
            // the residual stream is bf16: normalise what is stored so later readers agree
            float2 f = __bfloat1622float2(o.v[j]);
            v[2 * j] = f.x;
            v[2 * j + 1] = f.y;
          }
          *reinterpret_cast<bf16x8*>(rr) = o;
        }
      }
    }
#pragma unroll
    for (int j = 0; j < VEC; ++j) {
      ss += v[j] * v[j];
      rowbuf[i + j] = v[j];
    }
  }
  ss = block_sum(ss, red);
  const float inv = rsqrtf(ss / (float)H + eps);
  if (!out) return;
  __nv_bfloat16* orow = out + row * out_stride;
  for (int i = threadIdx.x * VEC; i < H; i += blockDim.x * VEC) {
    bf16x8 wv = *reinterpret_cast<const bf16x8*>(w + i);
    bf16x8 o;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float2 wf = __bfloat1622float2(wv.v[j]);
      o.v[j] = __floats2bfloat162_rn(rowbuf[i + 2 * j] * inv * (wf.x + wbias),
                                     rowbuf[i + 2 * j + 1] * inv * (wf.y + wbias));
    }
    *reinterpret_cast<bf16x8*>(orow + i) = o;
  }
}

// Per-head RMSNorm over head_dim (q/k norms): x [rows, heads, hd] in place. One warp per (row, head).
__global__ void rmsnorm_heads_kernel(__nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w, int rows,
                                     int heads, int hd, long row_stride, float eps, float wbias) {
  const int gw = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (gw >= rows * heads) return;
  const int r = gw / heads, h = gw % heads;
  __nv_bfloat16* p = x + r * row_stride + (long)h * hd;
  float ss = 0.f;
  for (int i = lane; i < hd; i += 32) {
    float v = bf2f(p[i]);
    ss += v * v;
  }
  ss = warp_sum(ss);
  const float inv = rsqrtf(ss / (float)hd + eps);
  for (int i = lane; i < hd; i += 32) p[i] = f2bf(bf2f(p[i]) * inv * (bf2f(w[i]) + wbias));
}

// ------------------------------------------------------------------------------------------------
// Embedding gather: out[r, :] = table[ids[r], :] * scale
// ------------------------------------------------------------------------------------------------
__global__ void embed_kernel(const int* __restrict__ ids, const __nv_bfloat16* __restrict__ table,
                             __nv_bfloat16* __restrict__ out, int H, int vocab, float scale) {
  grid_dep_wait();
  grid_dep_launch();
  const long row = blockIdx.x;
  int id = ids[row];
  id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);
  const __nv_bfloat16* src = table + (long)id * H;
  __nv_bfloat16* dst = out + row * (long)H;
  for (int i = threadIdx.x * 8; i < H; i += blockDim.x * 8) {
    bf16x8 t = *reinterpret_cast<const bf16x8*>(src + i);
    if (scale != 1.f) {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float2 f = __bfloat1622float2(t.v[j]);
        t.v[j] = __floats2bfloat162_rn(f.x * scale, f.y * scale);
      }
    }
    *reinterpret_cast<bf16x8*>(dst + i) = t;
  }
}

// ------------------------------------------------------------------------------------------------
// RoPE on q and k (in the fused qkv row) + store of k, v into the paged cache.
//   qkv   [rows, (nq + 2*nkv) * hd]
//   pos   [rows] int32, slot [rows] int32 (slot < 0: row is padding, nothing stored)
//   page_table [slots, max_pages] int32; K/V pools [pages, nkv, PAGE, hd]
// NeoX pairing (i, i + rot/2) or interleaved (2i, 2i+1); rot_dim <= hd.
// grid (rows, nq + nkv) ; block hd/2 threads (one rotation pair each), v copied by the k blocks.
// ------------------------------------------------------------------------------------------------
constexpr int kPage = 64;

__global__ void rope_store_kernel(__nv_bfloat16* __restrict__ qkv, const int* __restrict__ pos,
                                  const int* __restrict__ slot, const int* __restrict__ page_table, int max_pages,
                                  __nv_bfloat16* __restrict__ kpool, __nv_bfloat16* __restrict__ vpool, int nq,
                                  int nkv, int hd, int rot_dim, float theta, int interleaved, float pos_scale,
                                  int kv_fp8, const int* __restrict__ pos3, int sec0, int sec1) {
  grid_dep_wait();
  grid_dep_launch();
  const int row = blockIdx.x, head = blockIdx.y;
  const int p = pos[row];
  const int s = slot ? slot[row] : 0;
  const long row_off = (long)row * (nq + 2 * nkv) * hd;
  __nv_bfloat16* h = qkv + row_off + (long)head * hd;
  const int half = rot_dim >> 1;
  const int i = threadIdx.x;  // pair index, 0..hd/2-1
  float a0, a1;
  int i0, i1;
  if (i < half) {
    i0 = interleaved ? 2 * i : i;
    i1 = interleaved ? 2 * i + 1 : i + half;
  } else {  // not rotated: pass-through pair
    i0 = rot_dim + 2 * (i - half);
    i1 = i0 + 1;
  }
  a0 = bf2f(h[i0]);
  a1 = bf2f(h[i1]);
  if (i < half) {
    const float inv_freq = exp2f(-log2f(theta) * (2.f * (float)i / (float)rot_dim));
    float sn, cs;
    // multimodal rotary embedding: the pair's section picks the time / height / width position of the row
    const int pr = pos3 ? pos3[(i < sec0 ? 0 : (i < sec0 + sec1 ? 1 : 2)) * (long)gridDim.x + row] : p;
    sincosf((float)pr * pos_scale * inv_freq, &sn, &cs);
    const float r0 = a0 * cs - a1 * sn, r1 = a1 * cs + a0 * sn;
    a0 = r0;
    a1 = r1;
  }
  const __nv_bfloat16 b0 = f2bf(a0), b1 = f2bf(a1);
  if (head < nq) {
    h[i0] = b0;
    h[i1] = b1;
    return;
  }
  if (s < 0) return;
  const int kvh = head - nq;
  const int page = page_table[(long)s * max_pages + p / kPage];
  const long dst = (((long)page * nkv + kvh) * kPage + (p % kPage)) * hd;
  h[i0] = b0;
  h[i1] = b1;
  const __nv_bfloat16* v = qkv + row_off + (long)(nq + nkv + kvh) * hd;
  if (kv_fp8 == 2) return;   // scaled cache formats: the quantising store kernel reads the rotated keys from qkv
  if (kv_fp8) {   // E5M2 cache: one byte per element, rounded from the bf16 values
    uint8_t* k8 = reinterpret_cast<uint8_t*>(kpool);
    uint8_t* v8 = reinterpret_cast<uint8_t*>(vpool);
    k8[dst + i0] = (uint8_t)__nv_cvt_float_to_fp8(bf2f(b0), __NV_SATFINITE, __NV_E5M2);
    k8[dst + i1] = (uint8_t)__nv_cvt_float_to_fp8(bf2f(b1), __NV_SATFINITE, __NV_E5M2);
    v8[dst + 2 * i] = (uint8_t)__nv_cvt_float_to_fp8(bf2f(v[2 * i]), __NV_SATFINITE, __NV_E5M2);
    v8[dst + 2 * i + 1] = (uint8_t)__nv_cvt_float_to_fp8(bf2f(v[2 * i + 1]), __NV_SATFINITE, __NV_E5M2);
    return;
  }
  kpool[dst + i0] = b0;
  kpool[dst + i1] = b1;
  vpool[dst + 2 * i] = v[2 * i];
  vpool[dst + 2 * i + 1] = v[2 * i + 1];
}

// ------------------------------------------------------------------------------------------------
// Gated activations. gu [rows, 2*I] (gate first, then up) -> out [rows, I].
// act 0: silu(g)*u ; act 1: gelu_tanh(g)*u. limit > 0 clamps g <= limit and |u| <= limit.
// ------------------------------------------------------------------------------------------------
VE_DEVINL float act_silu(float g) { return g / (1.f + __expf(-g)); }
VE_DEVINL float act_gelu_tanh(float g) {
  const float k = 0.7978845608028654f;
  return 0.5f * g * (1.f + tanhf(k * (g + 0.044715f * g * g * g)));
}

__global__ void gated_act_kernel(const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ out, long rows,
                                 int I, int act, float limit, int interleave) {
  grid_dep_wait();
  grid_dep_launch();
  const long n8 = rows * (long)(I / 8);
  for (long idx = blockIdx.x * (long)blockDim.x + threadIdx.x; idx < n8; idx += (long)gridDim.x * blockDim.x) {
    const long r = idx / (I / 8);
    const int c = (int)(idx % (I / 8)) * 8;
    // interleave == 64: the row holds [64 gate | 64 up] per 128 columns (layout of the fused decode linear's weights)
    const long go = interleave ? (long)(c / 64) * 128 + (c % 64) : c;
    const long uo = interleave ? go + 64 : (long)I + c;
    bf16x8 g = *reinterpret_cast<const bf16x8*>(gu + r * 2L * I + go);
    bf16x8 u = *reinterpret_cast<const bf16x8*>(gu + r * 2L * I + uo);
    bf16x8 o;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float2 gf = __bfloat1622float2(g.v[j]), uf = __bfloat1622float2(u.v[j]);
      if (limit > 0.f) {
        gf.x = fminf(gf.x, limit);
        gf.y = fminf(gf.y, limit);
        uf.x = fminf(fmaxf(uf.x, -limit), limit);
        uf.y = fminf(fmaxf(uf.y, -limit), limit);
      }
      float ax = act ? act_gelu_tanh(gf.x) : act_silu(gf.x);
      float ay = act ? act_gelu_tanh(gf.y) : act_silu(gf.y);
      o.v[j] = __floats2bfloat162_rn(ax * uf.x, ay * uf.y);
    }
    *reinterpret_cast<bf16x8*>(out + r * (long)I + c) = o;
  }
}

__global__ void add_kernel(__nv_bfloat16* __restrict__ a, const __nv_bfloat16* __restrict__ b, long n8) {
  for (long idx = blockIdx.x * (long)blockDim.x + threadIdx.x; idx < n8; idx += (long)gridDim.x * blockDim.x) {
    bf16x8 x = reinterpret_cast<bf16x8*>(a)[idx], y = reinterpret_cast<const bf16x8*>(b)[idx];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float2 xf = __bfloat1622float2(x.v[j]), yf = __bfloat1622float2(y.v[j]);
      x.v[j] = __floats2bfloat162_rn(xf.x + yf.x, xf.y + yf.y);
    }
    reinterpret_cast<bf16x8*>(a)[idx] = x;
  }
}

__global__ void softcap_kernel(float* __restrict__ x, long n, float cap) {
  for (long idx = blockIdx.x * (long)blockDim.x + threadIdx.x; idx < n; idx += (long)gridDim.x * blockDim.x)
    x[idx] = cap * tanhf(x[idx] / cap);
}

}  // namespace ve

using namespace ve;

extern "C" {

int ve_rmsnorm(const void* x, void* res, int res_f32, const void* w, void* out, int rows, int H, float eps,
               float wbias, long x_stride, long out_stride, cudaStream_t st) {
  if (H % 8) return cudaErrorInvalidValue;
  if (rows <= 0) return 0;
  launch_pdl(rmsnorm_kernel<8>, dim3(rows), dim3(256), H * sizeof(float), st, (const __nv_bfloat16*)x, res, res_f32,
             (const __nv_bfloat16*)w, (__nv_bfloat16*)out, H, eps, wbias, x_stride ? x_stride : (long)H,
             out_stride ? out_stride : (long)H);
  VE_CHECK_LAUNCH();
}

int ve_rmsnorm_heads(void* x, const void* w, int rows, int heads, int hd, long row_stride, float eps, float wbias,
                     cudaStream_t st) {
  const int warps = rows * heads;
  if (warps <= 0) return 0;
  rmsnorm_heads_kernel<<<(warps + 7) / 8, 256, 0, st>>>((__nv_bfloat16*)x, (const __nv_bfloat16*)w, rows, heads, hd,
                                                        row_stride, eps, wbias);
  VE_CHECK_LAUNCH();
}

int ve_embed(const void* ids, const void* table, void* out, int rows, int H, int vocab, float scale,
             cudaStream_t st) {
  if (H % 8) return cudaErrorInvalidValue;
  if (rows <= 0) return 0;
  launch_pdl(embed_kernel, dim3(rows), dim3(128), 0, st, (const int*)ids, (const __nv_bfloat16*)table,
             (__nv_bfloat16*)out, H, vocab, scale);
  VE_CHECK_LAUNCH();
}

int ve_rope_store(void* qkv, const void* pos, const void* slot, const void* page_table, int max_pages, void* kpool,
                  void* vpool, int rows, int nq, int nkv, int hd, int rot_dim, float theta, int interleaved,
                  float pos_scale, int kv_fp8, const void* pos3, int sec0, int sec1, cudaStream_t st) {
  if (hd % 2 || rot_dim % 2 || rot_dim > hd || hd / 2 > 1024) return cudaErrorInvalidValue;
  if (rows <= 0) return 0;
  dim3 grid(rows, nq + nkv);
  launch_pdl(rope_store_kernel, grid, dim3(hd / 2), 0, st, (__nv_bfloat16*)qkv, (const int*)pos, (const int*)slot,
             (const int*)page_table, max_pages, (__nv_bfloat16*)kpool, (__nv_bfloat16*)vpool, nq, nkv, hd, rot_dim,
             theta, interleaved, pos_scale, kv_fp8, (const int*)pos3, sec0, sec1);
  VE_CHECK_LAUNCH();
}

int ve_gated_act(const void* gu, void* out, long rows, int I, int act, float limit, int interleave, cudaStream_t st) {
  if (I % 8 || (interleave && (interleave != 64 || I % 64))) return cudaErrorInvalidValue;
  if (rows <= 0) return 0;
  const long n8 = rows * (long)(I / 8);
  const int blocks = (int)((n8 + 255) / 256 < 148 * 8 ? (n8 + 255) / 256 : 148 * 8);
  launch_pdl(gated_act_kernel, dim3(blocks), dim3(256), 0, st, (const __nv_bfloat16*)gu, (__nv_bfloat16*)out, rows, I,
             act, limit, interleave);
  VE_CHECK_LAUNCH();
}

int ve_add(void* a, const void* b, long n, cudaStream_t st) {
  if (n % 8) return cudaErrorInvalidValue;
  if (n <= 0) return 0;
  const long n8 = n / 8;
  const int blocks = (int)((n8 + 255) / 256 < 148 * 8 ? (n8 + 255) / 256 : 148 * 8);
  add_kernel<<<blocks, 256, 0, st>>>((__nv_bfloat16*)a, (const __nv_bfloat16*)b, n8);
  VE_CHECK_LAUNCH();
}

int ve_softcap(void* x, long n, float cap, cudaStream_t st) {
  if (n <= 0) return 0;
  const int blocks = (int)((n + 255) / 256 < 148 * 8 ? (n + 255) / 256 : 148 * 8);
  softcap_kernel<<<blocks, 256, 0, st>>>((float*)x, n, cap);
  VE_CHECK_LAUNCH();
}

}  // extern "C"
