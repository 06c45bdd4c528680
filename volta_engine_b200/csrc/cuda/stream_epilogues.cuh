// Row epilogues that follow the sum of a row-parallel projection, shared by the low-latency all-reduce kernel
// (which leaves the bf16-rounded sum of one row in shared memory) and by the single-GPU launch of the same step:
//   sandwich   resid = (resid + RMSNorm(y) * (w_post + b)) * scale ; out = RMSNorm(resid) * (w_next + b)
//              (reference: all_reduce_normed_add_kernel, src/comm/all_reduce_ipc.cu:404-522; residual fp32 or bf16)
//   gated      x[s] += post[s] * (y [+ gate * addend]) ; out[s] = RMSNorm(x[s]) * (1 + w[s])   for hc fp32 streams
//              (reference: all_reduce_gated_norm_kernel :524-667; GatedResidual::apply + stream_norm)
//   hc         x[h] = post[h] * y + sum_g comb[g][h] * x[g]   for 4 fp32 streams
//              (reference: all_reduce_hc_apply_kernel :669-768; HyperConnection::update)
// Every thread keeps the same column set through all passes of one row, so values written in one pass are re-read by
// their writer in the next without a barrier; the barriers inside block_sum order the rest.
#pragma once
#include "common.cuh"

namespace ve {

enum RowEpilogue { kEpiSandwich = 2, kEpiGated = 3, kEpiHc = 4 };

struct EpiArgs {
  float* xs;                        // fp32 residual [rows, H] (sandwich) or streams [rows, hc, H]
  __nv_bfloat16* res16;             // sandwich with a bf16 residual (xs == nullptr)
  const float* post;                // [rows, hc]
  const float* comb;                // [rows, 4, 4]
  const __nv_bfloat16* w;           // sandwich: post-norm weight [H]; gated: stream norm weights [hc, H]
  const __nv_bfloat16* w2;          // sandwich: weight of the next block's input norm [H]
  const __nv_bfloat16* addend;      // gated: optional [rows, H] added as gate[row] * addend before the stream update
  const float* addend_gate;         // [rows]
  __nv_bfloat16* out;               // sandwich [rows, H]; gated [rows, hc, H]
  float* outf;                      // gated: the normalised streams in fp32 [rows, hc, H] (input of the next mixer)
  float eps, wbias, scale;
  int hc, H;
};

VE_DEVINL float round_to_bf16(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }

// ybuf: H floats in shared memory holding the bf16-rounded row sum. red: >= 33 floats of shared memory.
template <int MODE>
VE_DEVINL void row_epilogue(const float* ybuf, int row, const EpiArgs& e, float* red) {
  const int tid = threadIdx.x, nt = blockDim.x, H = e.H;
  if (MODE == kEpiSandwich) {
    float ss = 0.f;
    for (int i = tid; i < H; i += nt) ss = fmaf(ybuf[i], ybuf[i], ss);
    ss = block_sum(ss, red);
    const float inv1 = rsqrtf(ss / (float)H + e.eps);
    float s2 = 0.f;
    if (e.xs) {
      float* r = e.xs + (long)row * H;
      for (int i = tid; i < H; i += nt) {
        const float t = round_to_bf16(ybuf[i] * inv1 * (__bfloat162float(e.w[i]) + e.wbias));
        const float v = (r[i] + t) * e.scale;
        r[i] = v;
        s2 = fmaf(v, v, s2);
      }
    } else {
      __nv_bfloat16* r = e.res16 + (long)row * H;
      for (int i = tid; i < H; i += nt) {
        const float t = round_to_bf16(ybuf[i] * inv1 * (__bfloat162float(e.w[i]) + e.wbias));
        const float v = round_to_bf16((__bfloat162float(r[i]) + t) * e.scale);
        r[i] = __float2bfloat16_rn(v);
        s2 = fmaf(v, v, s2);
      }
    }
    s2 = block_sum(s2, red);
    const float inv2 = rsqrtf(s2 / (float)H + e.eps);
    __nv_bfloat16* o = e.out + (long)row * H;
    for (int i = tid; i < H; i += nt) {
      const float v = e.xs ? e.xs[(long)row * H + i] : __bfloat162float(e.res16[(long)row * H + i]);
      o[i] = __float2bfloat16_rn(v * inv2 * (__bfloat162float(e.w2[i]) + e.wbias));
    }
  } else if (MODE == kEpiGated) {
    const float gate = e.addend ? e.addend_gate[row] : 0.f;
    for (int s = 0; s < e.hc; ++s) {
      float* x = e.xs + ((long)row * e.hc + s) * H;
      const float p = e.post[row * e.hc + s];
      float ss = 0.f;
      for (int i = tid; i < H; i += nt) {
        float y = ybuf[i];
        if (e.addend) y = round_to_bf16(fmaf(gate, __bfloat162float(e.addend[(long)row * H + i]), y));
        const float v = fmaf(p, y, x[i]);
        x[i] = v;
        ss = fmaf(v, v, ss);
      }
      ss = block_sum(ss, red);
      if (e.out || e.outf) {
        const float inv = rsqrtf(ss / (float)H + e.eps);
        const long ob = ((long)row * e.hc + s) * H;
        const __nv_bfloat16* ws = e.w + (long)s * H;
        for (int i = tid; i < H; i += nt) {
          const float nv = x[i] * inv * (1.f + __bfloat162float(ws[i]));
          if (e.outf) e.outf[ob + i] = nv;
          if (e.out) e.out[ob + i] = __float2bfloat16_rn(nv);
        }
      }
    }
  } else if (MODE == kEpiHc) {
    float* x = e.xs + (long)row * 4 * H;
    float post[4], comb[16];
#pragma unroll
    for (int h = 0; h < 4; ++h) post[h] = e.post[row * 4 + h];
#pragma unroll
    for (int i = 0; i < 16; ++i) comb[i] = e.comb[row * 16 + i];
    for (int i = tid; i < H; i += nt) {
      float xv[4];
#pragma unroll
      for (int g = 0; g < 4; ++g) xv[g] = x[(long)g * H + i];
      const float y = ybuf[i];
#pragma unroll
      for (int h = 0; h < 4; ++h) {
        float o = post[h] * y;
#pragma unroll
        for (int g = 0; g < 4; ++g) o = fmaf(comb[g * 4 + h], xv[g], o);
        x[(long)h * H + i] = o;
      }
    }
  }
}

}  // namespace ve
