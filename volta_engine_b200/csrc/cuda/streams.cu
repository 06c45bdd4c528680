// Multi-stream residual modules: fp32 residual streams [rows, hc, hidden] and the kernels that mix them.
//   Hyper-connections (4 streams; reference inc/engine/modules/mhc.h, arithmetic src/kernels/slang/mhc.slang):
//     collapse   24 mix logits = streams . fn^T, rms of the whole 4*D row, pre = sigmoid(.)+eps, post = 2*sigmoid(.),
//                comb = Sinkhorn(softmax rows), collapsed = sum_h pre[h] * stream[h]; optionally the RMSNorm of the
//                collapsed row and the lagged form (collapse with the previous step's pre) in the same launch.
//                One thread-block cluster of 8 CTAs per row: each CTA owns D/8 columns of all four streams, the 25
//                partial sums and the norm's sum of squares meet through distributed shared memory.
//     update     x[h] = post[h] * y + sum_g comb[g][h] * x[g]      (stream_epilogues.cuh, also fused into the all-reduce)
//     init / head mean
//   Gated residual (hc streams; reference inc/engine/modules/gated_residual.h:5-16, src/backend/cpu/gated_residual.cpp):
//     norm (+ deferred apply of the previous sublayer), low-rank gate t = silu(normed . down / hc),
//     post = 2 * sigmoid(normed . inject / hc), mixed = mean_s(sigmoid(up[s] . t) * normed[s]), shared-expert gate,
//     add_broadcast; apply and the per-stream norm are the gated epilogue.
//   N-gram embedding layer, device side (reference inc/engine/modules/ple.h:9-30, src/backend/cpu/ple.cpp):
//     gate_and_norm, conv_apply (causal dilated depthwise conv over chunk rows or the slot's ring), ring_update.
#include <cooperative_groups.h>

#include "common.cuh"
#include "stream_epilogues.cuh"

namespace cg = cooperative_groups;

namespace ve {

constexpr int kHcCluster = 8;
constexpr int kPleRing = 16;

VE_DEVINL float sigmoidf_(float x) { return 1.f / (1.f + __expf(-x)); }

// ------------------------------------------------------------------------------------------------ epilogues, local
template <int MODE>
__global__ void __launch_bounds__(1024) stream_epilogue_kernel(const __nv_bfloat16* __restrict__ y, long y_stride,
                                                               const EpiArgs e) {
  extern __shared__ float ybuf[];
  __shared__ float red[33];
  grid_dep_wait();
  const int row = blockIdx.x;
  for (int i = threadIdx.x; i < e.H; i += blockDim.x) ybuf[i] = __bfloat162float(y[(long)row * y_stride + i]);
  __syncthreads();
  row_epilogue<MODE>(ybuf, row, e, red);
  grid_dep_launch();
}

// in [rows, H] bf16 -> streams [rows, hc, H] fp32 (every stream a copy)
__global__ void init_streams_kernel(const __nv_bfloat16* __restrict__ in, float* __restrict__ xs, int H, int hc) {
  const int row = blockIdx.y;
  const int d = blockIdx.x * blockDim.x + threadIdx.x;
  if (d >= H) return;
  const float v = __bfloat162float(in[(long)row * H + d]);
  for (int s = 0; s < hc; ++s) xs[((long)row * hc + s) * H + d] = v;
}

// out[r, d] = bf16(mean_s streams[r, s, d])
__global__ void head_mean_kernel(const float* __restrict__ xs, __nv_bfloat16* __restrict__ out, int H, int hc) {
  const int row = blockIdx.y;
  const int d = blockIdx.x * blockDim.x + threadIdx.x;
  if (d >= H) return;
  float o = 0.f;
  for (int s = 0; s < hc; ++s) o += xs[((long)row * hc + s) * H + d];
  out[(long)row * H + d] = __float2bfloat16_rn(o / (float)hc);
}

// streams[r, s, :] = h[r * hc + s, :] + e[r, :]
__global__ void add_broadcast_kernel(const __nv_bfloat16* __restrict__ h, const __nv_bfloat16* __restrict__ e,
                                     float* __restrict__ xs, int H, int hc) {
  const int row = blockIdx.y;
  const int d = blockIdx.x * blockDim.x + threadIdx.x;
  if (d >= H) return;
  const float ev = __bfloat162float(e[(long)row * H + d]);
  for (int s = 0; s < hc; ++s) {
    const long o = ((long)row * hc + s) * H + d;
    xs[o] = __bfloat162float(h[o]) + ev;
  }
}

// ------------------------------------------------------------------------------------------------ hyper-connections
struct HcArgs {
  const float* streams;           // [rows, 4, D]
  const float* fn;                // [24, 4 * D]
  const float* base;              // [24]
  const float* scale;             // [3]
  const float* pre_in;            // lagged form: [rows, 4] used for the collapse instead of this step's pre
  const __nv_bfloat16* norm_w;    // optional RMSNorm of the collapsed row
  __nv_bfloat16* collapsed;       // [rows, D]
  float *post, *comb;             // [rows, 4], [rows, 16]
  float *inv_rms, *mix_logits, *pre;   // optional [rows], [rows, 24], [rows, 4]
  int D, iters;
  float hc_eps, rms_eps, norm_eps, norm_bias, post_scale;
};

__global__ void __cluster_dims__(kHcCluster, 1, 1) __launch_bounds__(256) hc_collapse_kernel(const HcArgs a) {
  cg::cluster_group cl = cg::this_cluster();
  __shared__ float wred[8][25];
  __shared__ float part[25];
  __shared__ float mixs[25];
  __shared__ float part2, red[33];
  const int c = (int)cl.block_rank(), row = blockIdx.y, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int D = a.D, cols = D / kHcCluster, c0 = c * cols;
  const long RL = 4L * D;
  const float* s = a.streams + (long)row * RL;
  float acc[25];
#pragma unroll
  for (int k = 0; k < 25; ++k) acc[k] = 0.f;
  for (int d = c0 + tid; d < c0 + cols; d += 256) {
#pragma unroll
    for (int h = 0; h < 4; ++h) {
      const float sv = s[(long)h * D + d];
      acc[24] = fmaf(sv, sv, acc[24]);
#pragma unroll
      for (int j = 0; j < 24; ++j) acc[j] = fmaf(sv, __ldg(a.fn + j * RL + (long)h * D + d), acc[j]);
    }
  }
#pragma unroll
  for (int k = 0; k < 25; ++k) {
    const float v = warp_sum(acc[k]);
    if (lane == 0) wred[warp][k] = v;
  }
  __syncthreads();
  if (tid < 25) {
    float v = 0.f;
    for (int w = 0; w < 8; ++w) v += wred[w][tid];
    part[tid] = v;
  }
  cl.sync();
  if (tid < 25) {
    float v = 0.f;
    for (int r = 0; r < kHcCluster; ++r) v += *cl.map_shared_rank(&part[tid], r);   // fixed order: same bits in every CTA
    mixs[tid] = v;
  }
  __syncthreads();
  const float rmr = rsqrtf(mixs[24] / (float)(4 * D) + a.rms_eps);
  float pre[4], use[4];
#pragma unroll
  for (int h = 0; h < 4; ++h) {
    pre[h] = sigmoidf_(fmaf(mixs[h] * rmr, a.scale[0], a.base[h])) + a.hc_eps;
    use[h] = a.pre_in ? a.pre_in[row * 4 + h] : pre[h];
  }
  if (c == 0 && tid == 0) {
    for (int h = 0; h < 4; ++h)
      a.post[row * 4 + h] = 2.f * sigmoidf_(fmaf(mixs[4 + h] * rmr, a.scale[1], a.base[4 + h])) * a.post_scale;
    float v[16];
    for (int i = 0; i < 16; ++i) v[i] = fmaf(mixs[8 + i] * rmr, a.scale[2], a.base[8 + i]);
    for (int r = 0; r < 4; ++r) {
      float m = v[r * 4];
      for (int b = 1; b < 4; ++b) m = fmaxf(m, v[r * 4 + b]);
      float sum = 0.f;
      for (int b = 0; b < 4; ++b) {
        v[r * 4 + b] = __expf(v[r * 4 + b] - m);
        sum += v[r * 4 + b];
      }
      for (int b = 0; b < 4; ++b) v[r * 4 + b] = v[r * 4 + b] / sum + a.hc_eps;
    }
    for (int it = 0; it < a.iters; ++it) {
      if (it > 0)
        for (int r = 0; r < 4; ++r) {
          float rs = 0.f;
          for (int b = 0; b < 4; ++b) rs += v[r * 4 + b];
          for (int b = 0; b < 4; ++b) v[r * 4 + b] = v[r * 4 + b] / (rs + a.hc_eps);
        }
      for (int b = 0; b < 4; ++b) {
        float cs = 0.f;
        for (int r = 0; r < 4; ++r) cs += v[r * 4 + b];
        for (int r = 0; r < 4; ++r) v[r * 4 + b] = v[r * 4 + b] / (cs + a.hc_eps);
      }
    }
    for (int i = 0; i < 16; ++i) a.comb[row * 16 + i] = v[i];
    if (a.inv_rms) a.inv_rms[row] = rmr;
    if (a.mix_logits)
      for (int k = 0; k < 24; ++k) a.mix_logits[row * 24 + k] = mixs[k];
    if (a.pre)
      for (int h = 0; h < 4; ++h) a.pre[row * 4 + h] = pre[h];
  }
  // collapse this CTA's columns (rounded to bf16, as the unfused collapse stores them)
  float ssn = 0.f;
  for (int d = c0 + tid; d < c0 + cols; d += 256) {
    float o = 0.f;
#pragma unroll
    for (int h = 0; h < 4; ++h) o = fmaf(use[h], s[(long)h * D + d], o);
    const __nv_bfloat16 ob = __float2bfloat16_rn(o);
    if (a.norm_w) {
      const float f = __bfloat162float(ob);
      ssn = fmaf(f, f, ssn);
    } else if (a.collapsed) {
      a.collapsed[(long)row * D + d] = ob;
    }
  }
  if (a.norm_w) {
    ssn = block_sum(ssn, red);
    if (tid == 0) part2 = ssn;
    cl.sync();
    float tot = 0.f;
    for (int r = 0; r < kHcCluster; ++r) tot += *cl.map_shared_rank(&part2, r);
    const float inv = rsqrtf(tot / (float)D + a.norm_eps);
    for (int d = c0 + tid; d < c0 + cols; d += 256) {
      float o = 0.f;
#pragma unroll
      for (int h = 0; h < 4; ++h) o = fmaf(use[h], s[(long)h * D + d], o);
      const float f = round_to_bf16(o);
      a.collapsed[(long)row * D + d] = __float2bfloat16_rn(f * inv * (__bfloat162float(a.norm_w[d]) + a.norm_bias));
    }
  }
  cl.sync();   // no CTA leaves while a peer may still read its shared memory
}

// ------------------------------------------------------------------------------------------------ gated residual
// grid rows * hc. x (+= prev_post * prev_y, stored) ; normed = x * inv_rms * (1 + w[s]) as fp32 and / or bf16 hi, lo.
__global__ void __launch_bounds__(256) gr_norm_kernel(float* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                                                      float* __restrict__ normed, __nv_bfloat16* __restrict__ hi,
                                                      __nv_bfloat16* __restrict__ lo, const float* __restrict__ prev_post,
                                                      const __nv_bfloat16* __restrict__ prev_y, int H, int hc, float eps) {
  __shared__ float red[33];
  grid_dep_wait();
  const int i = blockIdx.x, r = i / hc, s = i % hc;
  float* xr = x + (long)i * H;
  const float p = prev_y ? prev_post[i] : 0.f;
  float ss = 0.f;
  for (int d = threadIdx.x; d < H; d += blockDim.x) {
    float v = xr[d];
    if (prev_y) {
      v = fmaf(p, __bfloat162float(prev_y[(long)r * H + d]), v);
      xr[d] = v;
    }
    ss = fmaf(v, v, ss);
  }
  ss = block_sum(ss, red);
  const float inv = rsqrtf(ss / (float)H + eps);
  for (int d = threadIdx.x; d < H; d += blockDim.x) {
    const float nv = xr[d] * inv * (1.f + __bfloat162float(w[(long)s * H + d]));
    if (normed) normed[(long)i * H + d] = nv;
    if (hi) {
      const __nv_bfloat16 h = __float2bfloat16_rn(nv);
      hi[(long)i * H + d] = h;
      if (lo) lo[(long)i * H + d] = __float2bfloat16_rn(nv - __bfloat162float(h));
    }
  }
  grid_dep_launch();
}

// One warp per gate output j (j < rank: row j of down; else row j - rank of inject), up to 16 rows per pass.
// t[r, j] = silu(z / hc), post[r, s] = 2 * sigmoid(z / hc) with z = normed[r, :] . w_j.   grid (ceil(outs / 8), row tiles)
__global__ void __launch_bounds__(256) gr_gate_kernel(const float* __restrict__ normed, const __nv_bfloat16* __restrict__ down,
                                                      const __nv_bfloat16* __restrict__ inject, float* __restrict__ t,
                                                      float* __restrict__ post, int rows, int flat, int hc, int rank,
                                                      int outs) {
  grid_dep_wait();
  const int lane = threadIdx.x & 31, j = blockIdx.x * 8 + (threadIdx.x >> 5);
  if (j >= outs) return;
  const int r0 = blockIdx.y * 16, nr = min(16, rows - r0);
  const __nv_bfloat16* w = j < rank ? down + (long)j * flat : inject + (long)(j - rank) * flat;
  float acc[16];
#pragma unroll
  for (int m = 0; m < 16; ++m) acc[m] = 0.f;
  for (int k = lane * 2; k < flat; k += 64) {
    const float2 wf = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(w + k));
#pragma unroll
    for (int m = 0; m < 16; ++m) {
      if (m >= nr) break;
      const float2 nv = *reinterpret_cast<const float2*>(normed + (long)(r0 + m) * flat + k);
      acc[m] = fmaf(nv.x, wf.x, fmaf(nv.y, wf.y, acc[m]));
    }
  }
#pragma unroll
  for (int m = 0; m < 16; ++m) {
    if (m >= nr) break;
    const float z = warp_sum(acc[m]) / (float)hc;
    if (lane == 0) {
      if (j < rank) t[(long)(r0 + m) * rank + j] = z * sigmoidf_(z);
      else post[(long)(r0 + m) * hc + (j - rank)] = 2.f * sigmoidf_(z);
    }
  }
}

// mixed[r, d] = bf16(mean_s sigmoid(up[s * H + d, :] . t[r, :]) * normed[r, s, d]).  One warp per column d: eight lanes
// per stream (hc <= 4) share the rank-long dot product. grid (ceil(H / 8), row tiles of 16), t of the tile in shared memory.
__global__ void __launch_bounds__(256) gr_up_kernel(const float* __restrict__ normed, const float* __restrict__ t,
                                                    const __nv_bfloat16* __restrict__ up, __nv_bfloat16* __restrict__ mixed,
                                                    int rows, int H, int hc, int rank) {
  extern __shared__ float ts[];   // [16][rank]
  grid_dep_wait();
  const int r0 = blockIdx.y * 16, nr = min(16, rows - r0);
  for (int i = threadIdx.x; i < nr * rank; i += blockDim.x) ts[i] = t[(long)r0 * rank + i];
  __syncthreads();
  const int lane = threadIdx.x & 31, d = blockIdx.x * 8 + (threadIdx.x >> 5);
  if (d >= H) return;
  const int s = lane >> 3, sub = lane & 7, chunk = rank / 8;
  float acc[16];
#pragma unroll
  for (int m = 0; m < 16; ++m) acc[m] = 0.f;
  if (s < hc) {
    const __nv_bfloat16* u = up + ((long)s * H + d) * rank + sub * chunk;
    for (int k = 0; k < chunk; k += 2) {
      const float2 uf = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(u + k));
#pragma unroll
      for (int m = 0; m < 16; ++m) {
        if (m >= nr) break;
        const float* tr = ts + m * rank + sub * chunk + k;
        acc[m] = fmaf(tr[0], uf.x, fmaf(tr[1], uf.y, acc[m]));
      }
    }
  }
#pragma unroll
  for (int m = 0; m < 16; ++m) {
    if (m >= nr) break;
    float v = acc[m];
    v += __shfl_xor_sync(0xffffffffu, v, 1);
    v += __shfl_xor_sync(0xffffffffu, v, 2);
    v += __shfl_xor_sync(0xffffffffu, v, 4);
    float o = s < hc ? sigmoidf_(v) * normed[((long)(r0 + m) * hc + s) * H + d] : 0.f;
    o += __shfl_xor_sync(0xffffffffu, o, 8);
    o += __shfl_xor_sync(0xffffffffu, o, 16);
    if (lane == 0) mixed[(long)(r0 + m) * H + d] = __float2bfloat16_rn(o / (float)hc);
  }
}

// mixed = mean_s(sigmoid(u[r, s, d]) * normed[r, s, d]) for the GEMM form of the up projection
__global__ void gr_up_epilogue_kernel(const float* __restrict__ u, const float* __restrict__ normed,
                                      __nv_bfloat16* __restrict__ mixed, int H, int hc) {
  const int row = blockIdx.y;
  const int d = blockIdx.x * blockDim.x + threadIdx.x;
  if (d >= H) return;
  float o = 0.f;
  for (int s = 0; s < hc; ++s) {
    const long i = ((long)row * hc + s) * H + d;
    o = fmaf(sigmoidf_(u[i]), normed[i], o);
  }
  mixed[(long)row * H + d] = __float2bfloat16_rn(o / (float)hc);
}

// gate[r] = sigmoid(x[r] . w)
__global__ void __launch_bounds__(256) gr_shared_gate_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                                                             float* __restrict__ gate, int H) {
  __shared__ float red[33];
  grid_dep_wait();
  const int row = blockIdx.x;
  float acc = 0.f;
  for (int d = threadIdx.x; d < H; d += blockDim.x)
    acc = fmaf(__bfloat162float(x[(long)row * H + d]), __bfloat162float(w[d]), acc);
  acc = block_sum(acc, red);
  if (threadIdx.x == 0) gate[row] = sigmoidf_(acc);
}

// ------------------------------------------------------------------------------------------------ n-gram layer
// grid rows * hc: gate = dot(rmsnorm_k(key[r, s]), rmsnorm_q(streams[r, s])); sg = sigmoid(signed_sqrt(gate * scale));
// gated = sg * value[r] (fp32); normed = rmsnorm_c(gated) (bf16). All norm weights applied as 1 + w, grouped per stream.
__global__ void __launch_bounds__(256) ple_gate_kernel(const __nv_bfloat16* __restrict__ key, const __nv_bfloat16* __restrict__ value,
                                                       const float* __restrict__ xs, const __nv_bfloat16* __restrict__ nk,
                                                       const __nv_bfloat16* __restrict__ nq, const __nv_bfloat16* __restrict__ nc,
                                                       float* __restrict__ gated, __nv_bfloat16* __restrict__ normed, int H,
                                                       int hc, float eps, float gate_scale) {
  __shared__ float red[33];
  grid_dep_wait();
  const int i = blockIdx.x, r = i / hc, s = i % hc;
  const long base = (long)i * H;
  const __nv_bfloat16* k = key + base;
  const float* x = xs + base;
  const __nv_bfloat16* v = value + (long)r * H;
  float sk = 0.f, sq = 0.f, sv = 0.f;
  for (int d = threadIdx.x; d < H; d += blockDim.x) {
    const float kv = __bfloat162float(k[d]), vv = __bfloat162float(v[d]), xv = x[d];
    sk = fmaf(kv, kv, sk);
    sq = fmaf(xv, xv, sq);
    sv = fmaf(vv, vv, sv);
  }
  sk = block_sum(sk, red);
  sq = block_sum(sq, red);
  sv = block_sum(sv, red);
  const float ik = rsqrtf(sk / (float)H + eps), iq = rsqrtf(sq / (float)H + eps);
  float dot = 0.f;
  for (int d = threadIdx.x; d < H; d += blockDim.x)
    dot = fmaf(__bfloat162float(k[d]) * ik * (1.f + __bfloat162float(nk[(long)s * H + d])),
               x[d] * iq * (1.f + __bfloat162float(nq[(long)s * H + d])), dot);
  dot = block_sum(dot, red);
  const float g = dot * gate_scale;
  const float sign = g > 0.f ? 1.f : (g < 0.f ? -1.f : 0.f);
  const float sg = sigmoidf_(sign * sqrtf(fmaxf(fabsf(g), 1e-6f)));
  const float ig = rsqrtf(sg * sg * sv / (float)H + eps);
  for (int d = threadIdx.x; d < H; d += blockDim.x) {
    const float gv = sg * __bfloat162float(v[d]);
    gated[base + d] = gv;
    normed[base + d] = __float2bfloat16_rn(gv * ig * (1.f + __bfloat162float(nc[(long)s * H + d])));
  }
}

// streams += gated + silu(conv): taps at pos, pos - d, pos - 2d, pos - 3d (weight index 3, 2, 1, 0); a tap comes from this
// chunk's row r - k when that row is the same slot at that position, else from the slot's ring; zero below position 0.
__global__ void ple_conv_kernel(const __nv_bfloat16* __restrict__ normed, const __nv_bfloat16* __restrict__ conv_w,
                                const __nv_bfloat16* __restrict__ ring, const int* __restrict__ slot,
                                const int* __restrict__ pos, const float* __restrict__ gated, float* __restrict__ xs,
                                int rows, int channels, int dilation) {
  const int r = blockIdx.y;
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= channels) return;
  const int sl = slot[r], p = pos[r];
  if (sl < 0) return;
  float acc = 0.f;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int k = (3 - j) * dilation, sp = p - k;
    float xv = 0.f;
    if (sp >= 0) {
      const int rr = r - k;
      if (k == 0 || (rr >= 0 && slot[rr] == sl && pos[rr] == sp))
        xv = __bfloat162float(normed[(long)(k == 0 ? r : rr) * channels + c]);
      else
        xv = __bfloat162float(ring[((long)sl * kPleRing + (sp % kPleRing)) * channels + c]);
    }
    acc = fmaf(__bfloat162float(conv_w[(long)c * 4 + j]), xv, acc);
  }
  const long o = (long)r * channels + c;
  xs[o] += gated[o] + acc * sigmoidf_(acc);
}

__global__ void ple_ring_kernel(const __nv_bfloat16* __restrict__ normed, __nv_bfloat16* __restrict__ ring,
                                const int* __restrict__ slot, const int* __restrict__ pos, int channels) {
  const int r = blockIdx.y;
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= channels || slot[r] < 0) return;
  ring[((long)slot[r] * kPleRing + (pos[r] % kPleRing)) * channels + c] = normed[(long)r * channels + c];
}

}  // namespace ve

using namespace ve;

extern "C" {

// mode 2 sandwich, 3 gated streams, 4 hyper-connection update, applied to y [rows, H] bf16 (already summed over ranks)
int ve_stream_epilogue(int mode, const void* y, long y_stride, void* xs, void* res16, const void* post, const void* comb,
                       const void* w, const void* w2, const void* addend, const void* addend_gate, void* out, void* outf, int rows,
                       int H, int hc, float eps, float wbias, float scale, cudaStream_t st) {
  if (rows <= 0) return 0;
  EpiArgs e;
  e.xs = (float*)xs; e.res16 = (__nv_bfloat16*)res16; e.post = (const float*)post; e.comb = (const float*)comb;
  e.w = (const __nv_bfloat16*)w; e.w2 = (const __nv_bfloat16*)w2; e.addend = (const __nv_bfloat16*)addend;
  e.addend_gate = (const float*)addend_gate; e.out = (__nv_bfloat16*)out; e.outf = (float*)outf;
  e.eps = eps; e.wbias = wbias; e.scale = scale; e.hc = hc; e.H = H;
  int threads = ((H / 4 + 31) / 32) * 32;
  threads = threads > 1024 ? 1024 : (threads < 64 ? 64 : threads);
  const size_t smem = (size_t)H * sizeof(float);
  if (smem > 48 * 1024) return cudaErrorInvalidValue;
  switch (mode) {
    case kEpiSandwich:
      if ((!xs && !res16) || !w || !w2 || !out) return cudaErrorInvalidValue;
      launch_pdl(stream_epilogue_kernel<kEpiSandwich>, dim3(rows), dim3(threads), smem, st, (const __nv_bfloat16*)y, y_stride, e);
      break;
    case kEpiGated:
      if (!xs || !post || hc <= 0 || ((out || outf) && !w)) return cudaErrorInvalidValue;
      launch_pdl(stream_epilogue_kernel<kEpiGated>, dim3(rows), dim3(threads), smem, st, (const __nv_bfloat16*)y, y_stride, e);
      break;
    case kEpiHc:
      if (!xs || !post || !comb) return cudaErrorInvalidValue;
      launch_pdl(stream_epilogue_kernel<kEpiHc>, dim3(rows), dim3(threads), smem, st, (const __nv_bfloat16*)y, y_stride, e);
      break;
    default: return cudaErrorInvalidValue;
  }
  VE_CHECK_LAUNCH();
}

int ve_init_streams(const void* in, void* xs, int rows, int H, int hc, cudaStream_t st) {
  if (rows <= 0) return 0;
  init_streams_kernel<<<dim3((H + 255) / 256, rows), 256, 0, st>>>((const __nv_bfloat16*)in, (float*)xs, H, hc);
  VE_CHECK_LAUNCH();
}

int ve_head_mean(const void* xs, void* out, int rows, int H, int hc, cudaStream_t st) {
  if (rows <= 0) return 0;
  head_mean_kernel<<<dim3((H + 255) / 256, rows), 256, 0, st>>>((const float*)xs, (__nv_bfloat16*)out, H, hc);
  VE_CHECK_LAUNCH();
}

int ve_add_broadcast(const void* h, const void* e, void* xs, int rows, int H, int hc, cudaStream_t st) {
  if (rows <= 0) return 0;
  add_broadcast_kernel<<<dim3((H + 255) / 256, rows), 256, 0, st>>>((const __nv_bfloat16*)h, (const __nv_bfloat16*)e,
                                                                     (float*)xs, H, hc);
  VE_CHECK_LAUNCH();
}

int ve_hc_collapse(const void* streams, const void* fn, const void* base, const void* scale, const void* pre_in,
                   const void* norm_w, void* collapsed, void* post, void* comb, void* inv_rms, void* mix_logits, void* pre,
                   int rows, int D, int iters, float hc_eps, float rms_eps, float norm_eps, float norm_bias,
                   float post_scale, cudaStream_t st) {
  if (rows <= 0) return 0;
  if (D % kHcCluster || !post || !comb || iters < 1) return cudaErrorInvalidValue;
  HcArgs a;
  a.streams = (const float*)streams; a.fn = (const float*)fn; a.base = (const float*)base; a.scale = (const float*)scale;
  a.pre_in = (const float*)pre_in; a.norm_w = (const __nv_bfloat16*)norm_w; a.collapsed = (__nv_bfloat16*)collapsed;
  a.post = (float*)post; a.comb = (float*)comb; a.inv_rms = (float*)inv_rms; a.mix_logits = (float*)mix_logits;
  a.pre = (float*)pre; a.D = D; a.iters = iters; a.hc_eps = hc_eps; a.rms_eps = rms_eps; a.norm_eps = norm_eps;
  a.norm_bias = norm_bias; a.post_scale = post_scale;
  hc_collapse_kernel<<<dim3(kHcCluster, rows), 256, 0, st>>>(a);
  VE_CHECK_LAUNCH();
}

int ve_gr_norm(void* x, const void* w, void* normed, void* hi, void* lo, const void* prev_post, const void* prev_y,
               int rows, int H, int hc, float eps, cudaStream_t st) {
  if (rows <= 0) return 0;
  launch_pdl(gr_norm_kernel, dim3(rows * hc), dim3(256), 0, st, (float*)x, (const __nv_bfloat16*)w, (float*)normed,
             (__nv_bfloat16*)hi, (__nv_bfloat16*)lo, (const float*)prev_post, (const __nv_bfloat16*)prev_y, H, hc, eps);
  VE_CHECK_LAUNCH();
}

int ve_gr_gate(const void* normed, const void* down, const void* inject, void* t, void* post, int rows, int H, int hc,
               int rank, cudaStream_t st) {
  if (rows <= 0) return 0;
  const int flat = H * hc, outs = rank + (inject ? hc : 0);
  if (flat % 2) return cudaErrorInvalidValue;
  launch_pdl(gr_gate_kernel, dim3((outs + 7) / 8, (rows + 15) / 16), dim3(256), 0, st, (const float*)normed,
             (const __nv_bfloat16*)down, (const __nv_bfloat16*)inject, (float*)t, (float*)post, rows, flat, hc, rank, outs);
  VE_CHECK_LAUNCH();
}

int ve_gr_up(const void* normed, const void* t, const void* up, void* mixed, int rows, int H, int hc, int rank,
             cudaStream_t st) {
  if (rows <= 0) return 0;
  if (hc > 4 || rank % 16 || (size_t)16 * rank * sizeof(float) > 48 * 1024) return cudaErrorInvalidValue;
  launch_pdl(gr_up_kernel, dim3((H + 7) / 8, (rows + 15) / 16), dim3(256), (size_t)16 * rank * sizeof(float), st,
             (const float*)normed, (const float*)t, (const __nv_bfloat16*)up, (__nv_bfloat16*)mixed, rows, H, hc, rank);
  VE_CHECK_LAUNCH();
}

int ve_gr_up_epilogue(const void* u, const void* normed, void* mixed, int rows, int H, int hc, cudaStream_t st) {
  if (rows <= 0) return 0;
  gr_up_epilogue_kernel<<<dim3((H + 255) / 256, rows), 256, 0, st>>>((const float*)u, (const float*)normed,
                                                                      (__nv_bfloat16*)mixed, H, hc);
  VE_CHECK_LAUNCH();
}

int ve_gr_shared_gate(const void* x, const void* w, void* gate, int rows, int H, cudaStream_t st) {
  if (rows <= 0) return 0;
  launch_pdl(gr_shared_gate_kernel, dim3(rows), dim3(256), 0, st, (const __nv_bfloat16*)x, (const __nv_bfloat16*)w,
             (float*)gate, H);
  VE_CHECK_LAUNCH();
}

int ve_ple_gate(const void* key, const void* value, const void* xs, const void* nk, const void* nq, const void* nc,
                void* gated, void* normed, int rows, int H, int hc, float eps, float gate_scale, cudaStream_t st) {
  if (rows <= 0) return 0;
  launch_pdl(ple_gate_kernel, dim3(rows * hc), dim3(256), 0, st, (const __nv_bfloat16*)key, (const __nv_bfloat16*)value,
             (const float*)xs, (const __nv_bfloat16*)nk, (const __nv_bfloat16*)nq, (const __nv_bfloat16*)nc, (float*)gated,
             (__nv_bfloat16*)normed, H, hc, eps, gate_scale);
  VE_CHECK_LAUNCH();
}

int ve_ple_conv(const void* normed, const void* conv_w, const void* ring, const void* slot, const void* pos,
                const void* gated, void* xs, int rows, int channels, int dilation, cudaStream_t st) {
  if (rows <= 0) return 0;
  if (3 * dilation >= kPleRing) return cudaErrorInvalidValue;
  ple_conv_kernel<<<dim3((channels + 255) / 256, rows), 256, 0, st>>>(
      (const __nv_bfloat16*)normed, (const __nv_bfloat16*)conv_w, (const __nv_bfloat16*)ring, (const int*)slot,
      (const int*)pos, (const float*)gated, (float*)xs, rows, channels, dilation);
  VE_CHECK_LAUNCH();
}

int ve_ple_ring(const void* normed, void* ring, const void* slot, const void* pos, int rows, int channels,
                cudaStream_t st) {
  if (rows <= 0) return 0;
  ple_ring_kernel<<<dim3((channels + 255) / 256, rows), 256, 0, st>>>((const __nv_bfloat16*)normed, (__nv_bfloat16*)ring,
                                                                       (const int*)slot, (const int*)pos, channels);
  VE_CHECK_LAUNCH();
}

}  // extern "C"
