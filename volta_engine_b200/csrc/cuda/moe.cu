// Mixture-of-experts kernels: router selection, route-indexed NVFP4 mat-vecs for decode rows, deterministic
// combine, and the sort / tile-table / gather helpers that feed the grouped tcgen05 GEMM for prefill chunks.
//
// Router semantics (reference: src/backend/cuda/modules/moe.cu:297-384, inc/engine/modules/moe.h:80-96):
//   softmax form  top-k of the raw logits, weights = softmax over the chosen logits only;
//   sigmoid form  s = sigmoid(logit); choose top-k of s + bias; weights = s_k * scale / (sum of chosen s + 1e-9);
//   sqrt-softplus form (mode 2, inc/engine/modules/dsv4.h: route)  s = sqrt(softplus(logit)), otherwise as the sigmoid form;
//   ties go to the lowest expert index. Group-limited routing (DeepSeek-V3 style, absent from the reference):
//   experts are split into n_group groups, a group's score is the sum of its two best biased scores, only the
//   topk_group best groups stay eligible.
// Combine (reference: src/models/glm5_next.cpp:2232-2247): per row, routes are summed in route order with their
// weights, the shared expert is added with weight 1; expert-parallel ranks produce partial rows that the
// tensor-parallel all-reduce sums.
#include "common.cuh"
#include <float.h>

namespace ve {

struct RV {
  float v;
  int i;
};
VE_DEVINL RV rv_better(RV a, RV b) { return (b.v > a.v || (b.v == a.v && b.i < a.i)) ? b : a; }
VE_DEVINL RV block_best(RV a, RV* red) {
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nw = blockDim.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    RV b{__shfl_xor_sync(0xffffffffu, a.v, o), __shfl_xor_sync(0xffffffffu, a.i, o)};
    a = rv_better(a, b);
  }
  if (lane == 0) red[wid] = a;
  __syncthreads();
  if (wid == 0) {
    RV t = lane < nw ? red[lane] : RV{-FLT_MAX, 0x7fffffff};
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      RV b{__shfl_xor_sync(0xffffffffu, t.v, o), __shfl_xor_sync(0xffffffffu, t.i, o)};
      t = rv_better(t, b);
    }
    if (lane == 0) red[32] = t;
  }
  __syncthreads();
  RV r = red[32];
  __syncthreads();
  return r;
}

// One CTA (256 threads) per row. E <= 1024. score[] lives in shared memory.
__global__ void __launch_bounds__(256) router_select_kernel(const float* __restrict__ logits, long stride, int E, int topk,
                                                            int mode, const float* __restrict__ bias, float scale,
                                                            int n_group, int topk_group, int* __restrict__ ids,
                                                            float* __restrict__ weights, float* __restrict__ heat) {
  __shared__ float s_raw[1024], s_sel[1024];
  __shared__ float s_gscore[64];
  __shared__ RV red[33];
  __shared__ float s_w[32];
  __shared__ int s_id[32];
  const float* row = logits + blockIdx.x * stride;
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    // a row of NaN / inf logits (an overflowed hidden state) must still yield in-range expert ids: NaN counts as the
    // lowest score, infinities are clamped to the largest finite values
    float l = row[e];
    l = (l != l) ? -FLT_MAX : fminf(fmaxf(l, -FLT_MAX), FLT_MAX);
    // mode 2: sqrt(softplus(l)), softplus written so that large |l| neither overflows nor cancels
    const float s = mode == 1 ? 1.f / (1.f + __expf(-l)) : mode == 2 ? sqrtf(fmaxf(l, 0.f) + log1pf(__expf(-fabsf(l)))) : l;
    s_raw[e] = s;
    s_sel[e] = s + (bias ? bias[e] : 0.f);
  }
  __syncthreads();
  if (n_group > 1) {
    const int per = E / n_group;
    for (int g = threadIdx.x; g < n_group; g += blockDim.x) {   // sum of the two best scores of the group
      float b1 = -FLT_MAX, b2 = -FLT_MAX;
      for (int e = g * per; e < (g + 1) * per; ++e) {
        const float v = s_sel[e];
        if (v > b1) { b2 = b1; b1 = v; } else if (v > b2) b2 = v;
      }
      s_gscore[g] = b1 + b2;
    }
    __syncthreads();
    if (threadIdx.x == 0) {   // keep the topk_group best groups (ties -> lowest index); n_group is small
      bool keep[64];
      for (int g = 0; g < n_group; ++g) keep[g] = false;
      for (int k = 0; k < topk_group; ++k) {
        int best = -1;
        for (int g = 0; g < n_group; ++g)
          if (!keep[g] && (best < 0 || s_gscore[g] > s_gscore[best])) best = g;
        if (best >= 0) keep[best] = true;
      }
      for (int g = 0; g < n_group; ++g) s_gscore[g] = keep[g] ? 1.f : 0.f;
    }
    __syncthreads();
    for (int e = threadIdx.x; e < E; e += blockDim.x)
      if (s_gscore[e / per] == 0.f) s_sel[e] = -INFINITY;     // below every sanitised score: never picked
    __syncthreads();
  }
  for (int k = 0; k < topk; ++k) {
    RV a{-FLT_MAX, 0x7fffffff};
    for (int e = threadIdx.x; e < E; e += blockDim.x) a = rv_better(a, RV{s_sel[e], e});
    a = block_best(a, red);
    if (threadIdx.x == 0) {
      int pick = a.i;
      if (pick < 0 || pick >= E) {
        // nothing beat the sentinel (every remaining score is the lowest value): take the first expert not picked yet
        pick = 0;
        for (int e = 0; e < E; ++e) {
          bool used = false;
          for (int j = 0; j < k; ++j) used = used || s_id[j] == e;
          if (!used) { pick = e; break; }
        }
      }
      s_id[k] = pick;
      s_w[k] = s_raw[pick];
      s_sel[pick] = -INFINITY;                                  // taken (sanitised scores are >= -FLT_MAX)
    }
    __syncthreads();
  }
  if (threadIdx.x == 0) {
    if (mode == 0) {   // softmax over the chosen logits
      float m = -FLT_MAX, sum = 0.f;
      for (int k = 0; k < topk; ++k) m = fmaxf(m, s_w[k]);
      for (int k = 0; k < topk; ++k) { s_w[k] = __expf(s_w[k] - m); sum += s_w[k]; }
      for (int k = 0; k < topk; ++k) s_w[k] = sum > 0.f ? s_w[k] / sum * scale : scale / (float)topk;
    } else {
      float sum = 0.f;
      for (int k = 0; k < topk; ++k) sum += s_w[k];
      for (int k = 0; k < topk; ++k) s_w[k] = s_w[k] * scale / (sum + 1e-9f);
    }
    for (int k = 0; k < topk; ++k) {
      ids[blockIdx.x * topk + k] = s_id[k];
      weights[blockIdx.x * topk + k] = s_w[k];
      if (heat && s_id[k] >= 0 && s_id[k] < E) atomicAdd(&heat[s_id[k]], 1.f);      // routing histogram: monitor page and expert residency decisions
    }
  }
}

// ------------------------------------------------------------------------------------------------
// Route-indexed NVFP4 mat-vec (decode / verify rows). Stacked expert weights Wp [E_local, N, K/2],
// Ws [E_local, N, K/16], gs [E_local]. Route r uses expert ids[r] - e0 (skipped, output zero, when not local)
// and activation row r / x_div (x_div = topk for the first projection, 1 for the second).
// FUSE = 1: the weight holds gate rows [0, N/2) and up rows [N/2, N); output [routes, N/2] = act(gate) * up.
// grid (rows of output / 2, routes), 128 threads: the four warps split K, partials summed in warp order.
// ------------------------------------------------------------------------------------------------
VE_DEVINL uint32_t m_cvt_e2m1x2(uint32_t byte) {
  uint32_t r;
  asm("{ .reg .b8 t; cvt.u8.u32 t, %1; cvt.rn.f16x2.e2m1x2 %0, t; }" : "=r"(r) : "r"(byte));
  return r;
}
VE_DEVINL float m_e4m3(uint32_t b) {
  uint32_t r;
  asm("{ .reg .b16 t; cvt.u16.u32 t, %1; cvt.rn.f16x2.e4m3x2 %0, t; }" : "=r"(r) : "r"(b & 0xffu));
  return __half2float(__ushort_as_half((unsigned short)(r & 0xffffu)));
}

template <int FUSE>
__global__ void __launch_bounds__(128) nvfp4_moe_gemv_kernel(const uint8_t* __restrict__ Wp, const uint8_t* __restrict__ Ws,
                                                             const float* __restrict__ gs, const int* __restrict__ ids,
                                                             int e0, int e_local, const __nv_bfloat16* __restrict__ x,
                                                             long x_stride, int x_div, __nv_bfloat16* __restrict__ out,
                                                             long out_stride, int N, int K, int act, float limit) {
  const int route = blockIdx.y;
  const int e = ids[route] - e0;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int half_n = N >> 1;
  const int o0 = blockIdx.x * 2;   // first output column of this CTA
  __shared__ float part[4][4];
  if (e < 0 || e >= e_local) {
    if (threadIdx.x < 2) {
      const int o = o0 + threadIdx.x;
      if (o < (FUSE ? half_n : N)) out[(long)route * out_stride + o] = f2bf(0.f);
    }
    return;
  }
  // rows handled: FUSE: gate o0, o0+1 and up o0+half_n, o0+1+half_n ; else rows o0, o0+1
  int rows[4];
  const int nrows = FUSE ? 4 : 2;
  rows[0] = o0;
  rows[1] = o0 + 1;
  rows[2] = o0 + half_n;
  rows[3] = o0 + 1 + half_n;
  // Ws == nullptr: Wp is a device table of per-expert base pointers {packed, scales} (tiered residency: an entry may
  // point into device slots or into pinned host memory that the GPU reads in place)
  const uint8_t* wp = Ws ? Wp + (size_t)e * N * (K >> 1) : reinterpret_cast<const uint8_t* const*>(Wp)[2 * e];
  const uint8_t* ws = Ws ? Ws + (size_t)e * N * (K >> 4) : reinterpret_cast<const uint8_t* const*>(Wp)[2 * e + 1];
  const __nv_bfloat16* xr = x + (long)(route / x_div) * x_stride;
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
  const int kchunks = K >> 5;
  for (int c = threadIdx.x; c < kchunks; c += 128) {
    float xv[32];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const bf16x8 t = *reinterpret_cast<const bf16x8*>(xr + (long)c * 32 + j * 8);
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const float2 f = __bfloat1622float2(t.v[u]);
        xv[j * 8 + 2 * u] = f.x;
        xv[j * 8 + 2 * u + 1] = f.y;
      }
    }
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      if (r >= nrows) break;
      const int n = min(rows[r], N - 1);
      const uint4 w = __ldcs(reinterpret_cast<const uint4*>(wp + (size_t)n * (K >> 1)) + c);
      const uint32_t sc = __ldcs(reinterpret_cast<const unsigned short*>(ws + (size_t)n * (K >> 4)) + c);
      const uint32_t words[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
      for (int blk = 0; blk < 2; ++blk) {
        float s = 0.f;
#pragma unroll
        for (int hw = 0; hw < 2; ++hw) {
          const uint32_t word = words[blk * 2 + hw];
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const uint32_t h2 = m_cvt_e2m1x2((word >> (8 * j)) & 0xffu);
            const float2 wf = __half22float2(*reinterpret_cast<const __half2*>(&h2));
            s = fmaf(wf.x, xv[blk * 16 + hw * 8 + 2 * j], s);
            s = fmaf(wf.y, xv[blk * 16 + hw * 8 + 2 * j + 1], s);
          }
        }
        acc[r] = fmaf(m_e4m3(sc >> (8 * blk)), s, acc[r]);
      }
    }
  }
#pragma unroll
  for (int r = 0; r < 4; ++r) {
    const float v = warp_sum(acc[r]);
    if (lane == 0) part[warp][r] = v;
  }
  __syncthreads();
  if (threadIdx.x < 2) {
    const int o = o0 + threadIdx.x;
    const float g = gs[e];
    if (FUSE) {
      if (o < half_n) {
        float gate = (part[0][threadIdx.x] + part[1][threadIdx.x] + part[2][threadIdx.x] + part[3][threadIdx.x]) * g;
        float up = (part[0][2 + threadIdx.x] + part[1][2 + threadIdx.x] + part[2][2 + threadIdx.x] + part[3][2 + threadIdx.x]) * g;
        // the unfused pair rounds both projections to bf16 before the activation: keep the same bits
        gate = bf2f(f2bf(gate));
        up = bf2f(f2bf(up));
        if (limit > 0.f) { gate = fminf(gate, limit); up = fminf(fmaxf(up, -limit), limit); }
        const float a = act ? 0.5f * gate * (1.f + tanhf(0.7978845608028654f * (gate + 0.044715f * gate * gate * gate)))
                            : gate / (1.f + __expf(-gate));
        out[(long)route * out_stride + o] = f2bf(a * up);
      }
    } else if (o < N) {
      const float v = (part[0][threadIdx.x] + part[1][threadIdx.x] + part[2][threadIdx.x] + part[3][threadIdx.x]) * g;
      out[(long)route * out_stride + o] = f2bf(v);
    }
  }
}

// Warp-per-row form (K <= kMoeXMax): the route's activation row is staged once per CTA in shared memory (16-byte pieces
// stored piece-major so that consecutive lanes read consecutive pieces), every warp owns two weight rows (FUSE: gate row o and
// up row o + N/2; else rows 2w, 2w + 1 of the CTA's eight) and walks K with all 32 lanes, two 16-byte weight loads per row in
// flight; no cross-warp reduction. One CTA streams 8 weight rows instead of 2-4, which is what lets the weight stream,
// and not CTA turnover, set the time. grid (outs / (FUSE ? 4 : 8), routes), 128 threads.
constexpr int kMoeXMax = 8192;

VE_DEVINL float moe_chunk_dot(const uint4 w, const uint32_t sc, const float* xv) {
  const uint32_t words[4] = {w.x, w.y, w.z, w.w};
  float acc = 0.f;
#pragma unroll
  for (int blk = 0; blk < 2; ++blk) {
    float s = 0.f;
#pragma unroll
    for (int hw = 0; hw < 2; ++hw) {
      const uint32_t word = words[blk * 2 + hw];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const uint32_t h2 = m_cvt_e2m1x2((word >> (8 * j)) & 0xffu);
        const float2 wf = __half22float2(*reinterpret_cast<const __half2*>(&h2));
        s = fmaf(wf.x, xv[blk * 16 + hw * 8 + 2 * j], s);
        s = fmaf(wf.y, xv[blk * 16 + hw * 8 + 2 * j + 1], s);
      }
    }
    acc = fmaf(m_e4m3(sc >> (8 * blk)), s, acc);
  }
  return acc;
}

template <int FUSE>
__global__ void __launch_bounds__(128) nvfp4_moe_gemv_rows_kernel(const uint8_t* __restrict__ Wp, const uint8_t* __restrict__ Ws,
                                                                  const float* __restrict__ gs, const int* __restrict__ ids,
                                                                  int e0, int e_local, const __nv_bfloat16* __restrict__ x,
                                                                  long x_stride, int x_div, __nv_bfloat16* __restrict__ out,
                                                                  long out_stride, int N, int K, int act, float limit) {
  __shared__ __align__(16) __nv_bfloat16 xs[kMoeXMax];
  constexpr int OUTS = FUSE ? 4 : 8;
  const int route = blockIdx.y;
  const int e = ids[route] - e0;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int half_n = N >> 1, n_out = FUSE ? half_n : N;
  const int o_base = blockIdx.x * OUTS;
  if (e < 0 || e >= e_local) {
    if (threadIdx.x < OUTS && o_base + threadIdx.x < n_out) out[(long)route * out_stride + o_base + threadIdx.x] = f2bf(0.f);
    return;
  }
  const uint8_t* wp = Ws ? Wp + (size_t)e * N * (K >> 1) : reinterpret_cast<const uint8_t* const*>(Wp)[2 * e];
  const uint8_t* ws = Ws ? Ws + (size_t)e * N * (K >> 4) : reinterpret_cast<const uint8_t* const*>(Wp)[2 * e + 1];
  const __nv_bfloat16* xr = x + (long)(route / x_div) * x_stride;
  const int kchunks = K >> 5;
  // piece (j, c) = elements [32 c + 8 j, 32 c + 8 j + 8) of the row, stored at piece index j * kchunks + c
  for (int pc = threadIdx.x; pc < kchunks * 4; pc += 128) {
    const int c = pc >> 2, j = pc & 3;
    *reinterpret_cast<uint4*>(xs + ((long)j * kchunks + c) * 8) = *reinterpret_cast<const uint4*>(xr + (long)c * 32 + j * 8);
  }
  __syncthreads();
  const int r0 = FUSE ? o_base + warp : o_base + 2 * warp;
  const int r1 = FUSE ? r0 + half_n : r0 + 1;
  const int n0 = min(r0, N - 1), n1 = min(r1, N - 1);
  const uint4* w0 = reinterpret_cast<const uint4*>(wp + (size_t)n0 * (K >> 1));
  const uint4* w1 = reinterpret_cast<const uint4*>(wp + (size_t)n1 * (K >> 1));
  const unsigned short* s0 = reinterpret_cast<const unsigned short*>(ws + (size_t)n0 * (K >> 4));
  const unsigned short* s1 = reinterpret_cast<const unsigned short*>(ws + (size_t)n1 * (K >> 4));
  float acc0 = 0.f, acc1 = 0.f;
  for (int c = lane; c < kchunks; c += 64) {
    const int c2 = c + 32;
    const bool two = c2 < kchunks;
    // all weight loads of the two chunks first, then the arithmetic
    const uint4 a0 = __ldcs(w0 + c), a1 = __ldcs(w1 + c);
    const uint32_t sa0 = __ldcs(s0 + c), sa1 = __ldcs(s1 + c);
    uint4 b0 = make_uint4(0, 0, 0, 0), b1 = b0;
    uint32_t sb0 = 0, sb1 = 0;
    if (two) {
      b0 = __ldcs(w0 + c2);
      b1 = __ldcs(w1 + c2);
      sb0 = __ldcs(s0 + c2);
      sb1 = __ldcs(s1 + c2);
    }
    float xv[32];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const bf16x8 t = *reinterpret_cast<const bf16x8*>(xs + ((long)j * kchunks + c) * 8);
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const float2 f = __bfloat1622float2(t.v[u]);
        xv[j * 8 + 2 * u] = f.x;
        xv[j * 8 + 2 * u + 1] = f.y;
      }
    }
    acc0 += moe_chunk_dot(a0, sa0, xv);
    acc1 += moe_chunk_dot(a1, sa1, xv);
    if (two) {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const bf16x8 t = *reinterpret_cast<const bf16x8*>(xs + ((long)j * kchunks + c2) * 8);
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const float2 f = __bfloat1622float2(t.v[u]);
          xv[j * 8 + 2 * u] = f.x;
          xv[j * 8 + 2 * u + 1] = f.y;
        }
      }
      acc0 += moe_chunk_dot(b0, sb0, xv);
      acc1 += moe_chunk_dot(b1, sb1, xv);
    }
  }
  acc0 = warp_sum(acc0);
  acc1 = warp_sum(acc1);
  if (lane != 0) return;
  const float g = gs[e];
  if (FUSE) {
    if (r0 < half_n) {
      // the unfused pair rounds both projections to bf16 before the activation: keep the same rounding points
      float gate = bf2f(f2bf(acc0 * g)), up = bf2f(f2bf(acc1 * g));
      if (limit > 0.f) { gate = fminf(gate, limit); up = fminf(fmaxf(up, -limit), limit); }
      const float a = act ? 0.5f * gate * (1.f + tanhf(0.7978845608028654f * (gate + 0.044715f * gate * gate * gate)))
                          : gate / (1.f + __expf(-gate));
      out[(long)route * out_stride + r0] = f2bf(a * up);
    }
  } else {
    if (r0 < N) out[(long)route * out_stride + r0] = f2bf(acc0 * g);
    if (r1 < N) out[(long)route * out_stride + r1] = f2bf(acc1 * g);
  }
}

// y[t, :] = sum_k w[t, k] * d[row(t, k), :] (+ shared[t, :]); row(t,k) = inv ? inv[t*topk+k] : t*topk+k.
// Routes of non-local experts carry zero rows (decode) or are flagged by ids outside [e0, e0+e_local).
__global__ void moe_combine_kernel(const __nv_bfloat16* __restrict__ d, long d_stride, const float* __restrict__ w,
                                   const int* __restrict__ ids, const int* __restrict__ inv, int e0, int e_local,
                                   const __nv_bfloat16* __restrict__ shared, long sh_stride,
                                   const float* __restrict__ sh_gate, long sh_gate_stride,
                                   __nv_bfloat16* __restrict__ y, long y_stride, int topk, int H) {
  const int t = blockIdx.x;
  // optional sigmoid gate of the shared expert: its logit is one extra column of the router product
  const float sg = (shared && sh_gate) ? 1.f / (1.f + __expf(-sh_gate[(long)t * sh_gate_stride])) : 1.f;
  for (int c = threadIdx.x * 8; c < H; c += blockDim.x * 8) {
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
    for (int k = 0; k < topk; ++k) {
      const int r = t * topk + k;
      const int e = ids[r] - e0;
      if (e < 0 || e >= e_local) continue;
      const long src = inv ? inv[r] : r;
      const float wk = w[r];
      const bf16x8 v = *reinterpret_cast<const bf16x8*>(d + src * d_stride + c);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __bfloat1622float2(v.v[j]);
        acc[2 * j] = fmaf(wk, f.x, acc[2 * j]);
        acc[2 * j + 1] = fmaf(wk, f.y, acc[2 * j + 1]);
      }
    }
    if (shared) {
      const bf16x8 v = *reinterpret_cast<const bf16x8*>(shared + (long)t * sh_stride + c);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __bfloat1622float2(v.v[j]);
        acc[2 * j] = fmaf(sg, f.x, acc[2 * j]);
        acc[2 * j + 1] = fmaf(sg, f.y, acc[2 * j + 1]);
      }
    }
    bf16x8 o;
#pragma unroll
    for (int j = 0; j < 4; ++j) o.v[j] = __floats2bfloat162_rn(acc[2 * j], acc[2 * j + 1]);
    *reinterpret_cast<bf16x8*>(y + (long)t * y_stride + c) = o;
  }
}

// ------------------------------------------------------------------------------------------------
// Prefill helpers. One CTA of 1024 threads (routes <= ~64K, local experts <= 1024):
//   counts per local expert -> offsets -> position of every local route (inv[route], -1 when not local)
//   -> tile table of <= bn rows per tile for the grouped GEMM (unused tiles get count 0).
// Positions inside an expert are handed out by atomics; every route's result is independent of its
// position and the combine runs in route order, so the output does not depend on the order.
// ------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(1024) moe_sort_kernel(const int* __restrict__ ids, int routes, int e0, int e_local,
                                                        int bn, int* __restrict__ inv, int* __restrict__ sorted_route,
                                                        int* __restrict__ tile_tab, int max_tiles, int* __restrict__ totals) {
  __shared__ int cnt[1024], off[1025], fill[1024], tile0[1025];
  for (int e = threadIdx.x; e < e_local; e += blockDim.x) { cnt[e] = 0; fill[e] = 0; }
  __syncthreads();
  for (int r = threadIdx.x; r < routes; r += blockDim.x) {
    const int e = ids[r] - e0;
    if (e >= 0 && e < e_local) atomicAdd(&cnt[e], 1);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int a = 0, t = 0;
    for (int e = 0; e < e_local; ++e) {
      off[e] = a;
      tile0[e] = t;
      a += cnt[e];
      t += (cnt[e] + bn - 1) / bn;
    }
    off[e_local] = a;
    tile0[e_local] = t;
    totals[0] = a;   // local routes
    totals[1] = t;   // tiles in use
  }
  __syncthreads();
  for (int r = threadIdx.x; r < routes; r += blockDim.x) {
    const int e = ids[r] - e0;
    if (e >= 0 && e < e_local) {
      const int p = off[e] + atomicAdd(&fill[e], 1);
      inv[r] = p;
      sorted_route[p] = r;
    } else {
      inv[r] = -1;
    }
  }
  for (int e = threadIdx.x; e < e_local; e += blockDim.x) {
    const int nt = (cnt[e] + bn - 1) / bn;
    for (int j = 0; j < nt; ++j) {
      const int t = tile0[e] + j;
      if (t < max_tiles) {
        tile_tab[4 * t + 0] = e;
        tile_tab[4 * t + 1] = off[e] + j * bn;
        tile_tab[4 * t + 2] = min(bn, cnt[e] - j * bn);
        tile_tab[4 * t + 3] = 0;
      }
    }
  }
  __syncthreads();
  for (int t = tile0[e_local] + threadIdx.x; t < max_tiles; t += blockDim.x) {
    tile_tab[4 * t + 0] = 0;
    tile_tab[4 * t + 1] = 0;
    tile_tab[4 * t + 2] = 0;
    tile_tab[4 * t + 3] = 0;
  }
}

// xs[p, :] = x[sorted_route[p] / topk, :] for p < totals[0]
__global__ void moe_gather_kernel(const __nv_bfloat16* __restrict__ x, long x_stride, const int* __restrict__ sorted_route,
                                  const int* __restrict__ totals, int topk, __nv_bfloat16* __restrict__ xs, long xs_stride,
                                  int H, int max_rows) {
  const int p = blockIdx.x;
  if (p >= totals[0] || p >= max_rows) return;
  const __nv_bfloat16* src = x + (long)(sorted_route[p] / topk) * x_stride;
  for (int c = threadIdx.x * 8; c < H; c += blockDim.x * 8)
    *reinterpret_cast<bf16x8*>(xs + (long)p * xs_stride + c) = *reinterpret_cast<const bf16x8*>(src + c);
}

}  // namespace ve

using namespace ve;

extern "C" {

int ve_router_select(const void* logits, long stride, int rows, int E, int topk, int mode, const void* bias, float scale,
                     int n_group, int topk_group, void* ids, void* weights, void* heat, cudaStream_t st) {
  if (rows <= 0) return 0;
  if (E > 1024 || topk > 32 || topk < 1 || topk > E || n_group > 64 || (n_group > 1 && E % n_group)) return cudaErrorInvalidValue;
  if (n_group > 1 && (topk_group < 1 || topk_group > n_group || E / n_group < 2 || topk > topk_group * (E / n_group)))
    return cudaErrorInvalidValue;
  router_select_kernel<<<rows, 256, 0, st>>>((const float*)logits, stride, E, topk, mode, (const float*)bias, scale,
                                             n_group, topk_group, (int*)ids, (float*)weights, (float*)heat);
  VE_CHECK_LAUNCH();
}

int ve_nvfp4_moe_gemv(const void* Wp, const void* Ws, const void* gs, const void* ids, int e0, int e_local, const void* x,
                      long x_stride, int x_div, void* out, long out_stride, int routes, int N, int K, int fuse_act,
                      int act, float limit, cudaStream_t st) {
  if (routes <= 0) return 0;
  if (K % 32 || N % 2 || (fuse_act && N % 4)) return cudaErrorInvalidValue;
  const int outs = fuse_act ? N / 2 : N;
  if (K <= kMoeXMax) {
    if (fuse_act)
      nvfp4_moe_gemv_rows_kernel<1><<<dim3((outs + 3) / 4, routes), 128, 0, st>>>(
          (const uint8_t*)Wp, (const uint8_t*)Ws, (const float*)gs, (const int*)ids, e0, e_local, (const __nv_bfloat16*)x,
          x_stride, x_div, (__nv_bfloat16*)out, out_stride, N, K, act, limit);
    else
      nvfp4_moe_gemv_rows_kernel<0><<<dim3((outs + 7) / 8, routes), 128, 0, st>>>(
          (const uint8_t*)Wp, (const uint8_t*)Ws, (const float*)gs, (const int*)ids, e0, e_local, (const __nv_bfloat16*)x,
          x_stride, x_div, (__nv_bfloat16*)out, out_stride, N, K, act, limit);
    VE_CHECK_LAUNCH();
  }
  dim3 grid((outs + 1) / 2, routes);
  if (fuse_act)
    nvfp4_moe_gemv_kernel<1><<<grid, 128, 0, st>>>((const uint8_t*)Wp, (const uint8_t*)Ws, (const float*)gs, (const int*)ids,
                                                   e0, e_local, (const __nv_bfloat16*)x, x_stride, x_div,
                                                   (__nv_bfloat16*)out, out_stride, N, K, act, limit);
  else
    nvfp4_moe_gemv_kernel<0><<<grid, 128, 0, st>>>((const uint8_t*)Wp, (const uint8_t*)Ws, (const float*)gs, (const int*)ids,
                                                   e0, e_local, (const __nv_bfloat16*)x, x_stride, x_div,
                                                   (__nv_bfloat16*)out, out_stride, N, K, act, limit);
  VE_CHECK_LAUNCH();
}

int ve_moe_combine(const void* d, long d_stride, const void* w, const void* ids, const void* inv, int e0, int e_local,
                   const void* shared, long sh_stride, const void* sh_gate, long sh_gate_stride, void* y, long y_stride,
                   int rows, int topk, int H, cudaStream_t st) {
  if (rows <= 0) return 0;
  if (H % 8) return cudaErrorInvalidValue;
  moe_combine_kernel<<<rows, 256, 0, st>>>((const __nv_bfloat16*)d, d_stride, (const float*)w, (const int*)ids,
                                           (const int*)inv, e0, e_local, (const __nv_bfloat16*)shared, sh_stride,
                                           (const float*)sh_gate, sh_gate_stride, (__nv_bfloat16*)y, y_stride, topk, H);
  VE_CHECK_LAUNCH();
}

int ve_moe_sort(const void* ids, int routes, int e0, int e_local, int bn, void* inv, void* sorted_route, void* tile_tab,
                int max_tiles, void* totals, cudaStream_t st) {
  if (routes <= 0) return 0;
  if (e_local > 1024) return cudaErrorInvalidValue;
  moe_sort_kernel<<<1, 1024, 0, st>>>((const int*)ids, routes, e0, e_local, bn, (int*)inv, (int*)sorted_route,
                                      (int*)tile_tab, max_tiles, (int*)totals);
  VE_CHECK_LAUNCH();
}

int ve_moe_gather(const void* x, long x_stride, const void* sorted_route, const void* totals, int topk, void* xs,
                  long xs_stride, int H, int max_rows, cudaStream_t st) {
  if (max_rows <= 0) return 0;
  moe_gather_kernel<<<max_rows, 128, 0, st>>>((const __nv_bfloat16*)x, x_stride, (const int*)sorted_route,
                                              (const int*)totals, topk, (__nv_bfloat16*)xs, xs_stride, H, max_rows);
  VE_CHECK_LAUNCH();
}

}  // extern "C"
