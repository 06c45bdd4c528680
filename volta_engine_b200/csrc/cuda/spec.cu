// Kernels of the block drafter and the sparse draft head.
//   publish_taps     row r of a target layer's output -> tap `tap` of its slot's position ring [slots, cap, taps_n * H]
//                    (slot and position read from device memory, so the launch replays inside a CUDA graph)
//   reduce_streams   fp32 streams [m, hc, H] -> one bf16 row per token (mean, or one chosen stream)
//   dynconv          grouped dynamic causal convolution inside a block: out[t, c] (+)= sum_k (base[k, c] + dyn[t, k, c / gs]) * x[t - k, c]
//   selector_walk    greedy chained walk over per-row candidate sets with a low-rank pairwise term
//   argmax_draft     out[0] = anchor, out[1 + i] = best candidate of block row 1 + i
//   sparse head      identity rows, column gather, scatter of subset logits into a full logits row
// Reference: src/spec/tap_ring.cu:12-54, inc/engine/spec/dflash.h:96-140 (dynconv, selector walk, argmax draft),
// inc/engine/modules/sparse_head.h:14-33.
#include "common.cuh"

namespace ve {

template <typename T>
__global__ void publish_taps_kernel(__nv_bfloat16* __restrict__ taps, const T* __restrict__ hidden, long h_stride,
                                    const int* __restrict__ slot, const int* __restrict__ pos, const int* __restrict__ owner,
                                    int tap, int H, int cap, long slot_stride, int taps_n) {
  grid_dep_wait();
  const int r = blockIdx.y;
  const int sl = slot ? slot[r] : 0, p = pos[r];
  if (sl < 0 || p < 0) return;
  if (owner && sl != *owner) return;
  __nv_bfloat16* dst = taps + (owner ? 0 : (long)sl * slot_stride) + ((long)(p % cap) * taps_n + tap) * H;
  const T* src = hidden + (long)r * h_stride;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < H; i += gridDim.x * blockDim.x)
    dst[i] = __float2bfloat16_rn((float)src[i]);
}

__global__ void reduce_streams_kernel(const float* __restrict__ xs, __nv_bfloat16* __restrict__ out, int H, int hc, int mode) {
  const int r = blockIdx.y;
  const float* in = xs + (long)r * hc * H;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < H; i += gridDim.x * blockDim.x) {
    float v = 0.f;
    if (mode == 0) {
      for (int s = 0; s < hc; ++s) v += in[(long)s * H + i];
      v /= (float)hc;
    } else {
      v = in[(long)(mode - 1) * H + i];
    }
    out[(long)r * H + i] = __float2bfloat16_rn(v);
  }
}

// x, out [T, C] fp32; dyn [T, taps, C / gs] bf16; base [taps, C] bf16. Rows before the block start read zero.
__global__ void dynconv_kernel(const float* __restrict__ x, const __nv_bfloat16* __restrict__ dyn,
                               const __nv_bfloat16* __restrict__ base, float* __restrict__ out, int T, int C, int taps, int gs,
                               int accumulate) {
  const int t = blockIdx.y;
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  const int G = C / gs;
  float acc = 0.f;
  for (int k = 0; k < taps; ++k) {
    if (t - k < 0) break;
    const float w = __bfloat162float(base[(long)k * C + c]) + __bfloat162float(dyn[((long)t * taps + k) * G + c / gs]);
    acc = fmaf(w, x[(long)(t - k) * C + c], acc);
  }
  float* o = out + (long)t * C + c;
  *o = accumulate ? *o + acc : acc;
}

// One CTA per sequence: chained greedy walk. score[c] = unary[i][c] + sum_r pred_cb[prev][r] * gate[i][r] * succ_cb[cand_c][r].
__global__ void __launch_bounds__(256) selector_walk_kernel(const float* __restrict__ unary, const int* __restrict__ cands,
                                                            const __nv_bfloat16* __restrict__ gate,
                                                            const __nv_bfloat16* __restrict__ pred_cb,
                                                            const __nv_bfloat16* __restrict__ succ_cb,
                                                            const int* __restrict__ anchor, int* __restrict__ out,
                                                            float* __restrict__ conf, int rows, int k, int rank) {
  extern __shared__ float sm[];
  float* ag = sm;            // [rank]
  float* scores = sm + rank; // [k]
  __shared__ int s_pred;
  const int b = blockIdx.x, t = threadIdx.x, warp = t >> 5, lane = t & 31;
  if (t == 0) {
    s_pred = anchor[b];
    out[(long)b * (rows + 1)] = s_pred;
    if (conf) conf[(long)b * (rows + 1)] = 1.f;
  }
  __syncthreads();
  for (int i = 0; i < rows; ++i) {
    const int pred = s_pred;
    const __nv_bfloat16* a = pred_cb + (long)pred * rank;
    const __nv_bfloat16* g = gate + ((long)b * rows + i) * rank;
    for (int r = t; r < rank; r += blockDim.x) ag[r] = __bfloat162float(a[r]) * __bfloat162float(g[r]);
    __syncthreads();
    const int* crow = cands + ((long)b * rows + i) * k;
    const float* urow = unary + ((long)b * rows + i) * k;
    for (int c = warp; c < k; c += blockDim.x / 32) {
      const __nv_bfloat16* s = succ_cb + (long)crow[c] * rank;
      float dot = 0.f;
      for (int r = lane; r < rank; r += 32) dot = fmaf(ag[r], __bfloat162float(s[r]), dot);
      dot = warp_sum(dot);
      if (lane == 0) scores[c] = urow[c] + dot;
    }
    __syncthreads();
    if (t == 0) {
      int best = 0;
      for (int c = 1; c < k; ++c)
        if (scores[c] > scores[best]) best = c;          // ties keep the earlier (higher-ranked) candidate
      s_pred = crow[best];
      out[(long)b * (rows + 1) + i + 1] = s_pred;
      if (conf) {
        float se = 0.f;
        for (int c = 0; c < k; ++c) se += __expf(scores[c] - scores[best]);
        conf[(long)b * (rows + 1) + i + 1] = 1.f / se;
      }
    }
    __syncthreads();
  }
}

__global__ void argmax_draft_kernel(const int* __restrict__ ix, int k, const int* __restrict__ anchor, int* __restrict__ out,
                                    int rows) {
  const int i = threadIdx.x;
  if (i == 0) out[0] = anchor[0];
  if (i < rows) out[1 + i] = ix[(long)(1 + i) * k];
}

// ident [rows, hidden]: rows [k0, k0 + rows) of the identity
__global__ void identity_rows_kernel(__nv_bfloat16* __restrict__ ident, int rows, int hidden, int k0) {
  const long i = blockIdx.x * (long)blockDim.x + threadIdx.x;
  if (i >= (long)rows * hidden) return;
  const int r = (int)(i / hidden), c = (int)(i % hidden);
  ident[i] = __float2bfloat16_rn(c == k0 + r ? 1.f : 0.f);
}

// w_sub[j, k0 + i] = chunk[i, cols[j]]
__global__ void sparse_gather_kernel(const __nv_bfloat16* __restrict__ chunk, long chunk_ld, int rows, int k0,
                                     const int* __restrict__ cols, int count, __nv_bfloat16* __restrict__ w_sub, int hidden) {
  const int j = blockIdx.x;
  if (j >= count) return;
  const int col = cols[j];
  for (int i = threadIdx.x; i < rows; i += blockDim.x) w_sub[(long)j * hidden + k0 + i] = chunk[(long)i * chunk_ld + col];
}

// logits[r, :] = lowest; logits[r, cols[j]] = sub[r, j]
__global__ void sparse_fill_kernel(__nv_bfloat16* __restrict__ logits, long ld, int width) {
  const int r = blockIdx.y;
  const __nv_bfloat16 lowest = __float2bfloat16_rn(-3.0e38f);
  for (int c = blockIdx.x * blockDim.x + threadIdx.x; c < width; c += gridDim.x * blockDim.x) logits[(long)r * ld + c] = lowest;
}
__global__ void sparse_scatter_kernel(const __nv_bfloat16* __restrict__ sub, int count, const int* __restrict__ cols,
                                      __nv_bfloat16* __restrict__ logits, long ld) {
  const int r = blockIdx.y;
  for (int j = blockIdx.x * blockDim.x + threadIdx.x; j < count; j += gridDim.x * blockDim.x)
    logits[(long)r * ld + cols[j]] = sub[(long)r * count + j];
}

}  // namespace ve

using namespace ve;

extern "C" {

// src_f32: hidden rows are fp32 (a model with an fp32 residual stream). owner != null: one ring, only rows of slot *owner publish.
int ve_publish_taps(void* taps, const void* hidden, long h_stride, int src_f32, const void* slot, const void* pos,
                    const void* owner, int m, int tap, int H, int cap, long slot_stride, int taps_n, cudaStream_t st) {
  if (m <= 0) return 0;
  if (tap < 0 || tap >= taps_n || cap <= 0) return cudaErrorInvalidValue;
  const dim3 grid((H + 1023) / 1024, m);
  if (src_f32)
    launch_pdl(publish_taps_kernel<float>, grid, dim3(256), 0, st, (__nv_bfloat16*)taps, (const float*)hidden, h_stride,
               (const int*)slot, (const int*)pos, (const int*)owner, tap, H, cap, slot_stride, taps_n);
  else
    launch_pdl(publish_taps_kernel<__nv_bfloat16>, grid, dim3(256), 0, st, (__nv_bfloat16*)taps, (const __nv_bfloat16*)hidden,
               h_stride, (const int*)slot, (const int*)pos, (const int*)owner, tap, H, cap, slot_stride, taps_n);
  VE_CHECK_LAUNCH();
}

int ve_reduce_streams(const void* xs, void* out, int m, int H, int hc, int mode, cudaStream_t st) {
  if (m <= 0) return 0;
  if (mode < 0 || mode > hc) return cudaErrorInvalidValue;
  reduce_streams_kernel<<<dim3((H + 1023) / 1024, m), 256, 0, st>>>((const float*)xs, (__nv_bfloat16*)out, H, hc, mode);
  VE_CHECK_LAUNCH();
}

int ve_dynconv(const void* x, const void* dyn, const void* base, void* out, int T, int C, int taps, int gs, int accumulate,
               cudaStream_t st) {
  if (T <= 0) return 0;
  if (C % gs) return cudaErrorInvalidValue;
  dynconv_kernel<<<dim3((C + 255) / 256, T), 256, 0, st>>>((const float*)x, (const __nv_bfloat16*)dyn,
                                                          (const __nv_bfloat16*)base, (float*)out, T, C, taps, gs, accumulate);
  VE_CHECK_LAUNCH();
}

int ve_selector_walk(const void* unary, const void* cands, const void* gate, const void* pred_cb, const void* succ_cb,
                     const void* anchor, void* out, void* conf, int bsz, int rows, int k, int rank, cudaStream_t st) {
  if (bsz <= 0 || rows <= 0) return 0;
  const size_t smem = (size_t)(rank + k) * sizeof(float);
  if (smem > 48 * 1024) return cudaErrorInvalidValue;
  selector_walk_kernel<<<bsz, 256, smem, st>>>((const float*)unary, (const int*)cands, (const __nv_bfloat16*)gate,
                                               (const __nv_bfloat16*)pred_cb, (const __nv_bfloat16*)succ_cb,
                                               (const int*)anchor, (int*)out, (float*)conf, rows, k, rank);
  VE_CHECK_LAUNCH();
}

int ve_argmax_draft(const void* ix, int k, const void* anchor, void* out, int rows, cudaStream_t st) {
  if (rows < 0 || rows > 31) return cudaErrorInvalidValue;
  argmax_draft_kernel<<<1, 32, 0, st>>>((const int*)ix, k, (const int*)anchor, (int*)out, rows);
  VE_CHECK_LAUNCH();
}

int ve_identity_rows(void* ident, int rows, int hidden, int k0, cudaStream_t st) {
  const long n = (long)rows * hidden;
  if (n <= 0) return 0;
  identity_rows_kernel<<<(int)((n + 255) / 256), 256, 0, st>>>((__nv_bfloat16*)ident, rows, hidden, k0);
  VE_CHECK_LAUNCH();
}

int ve_sparse_gather(const void* chunk, long chunk_ld, int rows, int k0, const void* cols, int count, void* w_sub, int hidden,
                     cudaStream_t st) {
  if (count <= 0 || rows <= 0) return 0;
  sparse_gather_kernel<<<count, 128, 0, st>>>((const __nv_bfloat16*)chunk, chunk_ld, rows, k0, (const int*)cols, count,
                                              (__nv_bfloat16*)w_sub, hidden);
  VE_CHECK_LAUNCH();
}

int ve_sparse_scatter(const void* sub, int count, const void* cols, void* logits, long ld, int width, int rows,
                      cudaStream_t st) {
  if (rows <= 0) return 0;
  sparse_fill_kernel<<<dim3(64, rows), 256, 0, st>>>((__nv_bfloat16*)logits, ld, width);
  if (count > 0)
    sparse_scatter_kernel<<<dim3((count + 255) / 256, rows), 256, 0, st>>>((const __nv_bfloat16*)sub, count, (const int*)cols,
                                                                           (__nv_bfloat16*)logits, ld);
  VE_CHECK_LAUNCH();
}

}  // extern "C"
