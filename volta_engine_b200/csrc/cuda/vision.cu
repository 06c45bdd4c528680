// Vision-tower pieces that the language-model kernels do not cover: LayerNorm with bias, bias + GELU, and the
// two-dimensional rotary embedding of patch queries / keys (half of the rotary pairs turn with the patch row,
// the other half with the patch column). Patch embedding, projections and MLPs run on the tcgen05 GEMM and the
// bidirectional attention on the paged attention kernel (key_end = last patch).
// Reference: inc/engine/modules/vision.h (patch-embed GEMM, LayerNorm / RMSNorm, qkv bias + 2-D rope, attention).
#include "common.cuh"

namespace ve {

// grid rows, block 256: y = (x - mean) / sqrt(var + eps) * w + b
__global__ void __launch_bounds__(256) layernorm_kernel(const __nv_bfloat16* __restrict__ x, long xs, const float* __restrict__ w,
                                                        const float* __restrict__ b, __nv_bfloat16* __restrict__ y, long ys,
                                                        int H, float eps) {
  __shared__ float red[33];
  const long r = blockIdx.x;
  float s = 0.f;
  for (int i = threadIdx.x; i < H; i += blockDim.x) s += bf2f(x[r * xs + i]);
  const float mean = block_sum(s, red) / H;
  float v = 0.f;
  for (int i = threadIdx.x; i < H; i += blockDim.x) { const float d = bf2f(x[r * xs + i]) - mean; v = fmaf(d, d, v); }
  const float inv = rsqrtf(block_sum(v, red) / H + eps);
  for (int i = threadIdx.x; i < H; i += blockDim.x)
    y[r * ys + i] = f2bf((bf2f(x[r * xs + i]) - mean) * inv * w[i] + (b ? b[i] : 0.f));
}

// x[r, c] = act(x[r, c] + bias[c]); act 0 none, 1 gelu (erf), 2 gelu (tanh), 3 silu
__global__ void bias_act_kernel(__nv_bfloat16* __restrict__ x, long xs, const float* __restrict__ bias, long rows, int cols, int act) {
  const long n = rows * cols;
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < n; i += (long)gridDim.x * blockDim.x) {
    const long r = i / cols;
    const int c = (int)(i % cols);
    float v = bf2f(x[r * xs + c]) + (bias ? bias[c] : 0.f);
    if (act == 1) v = 0.5f * v * (1.f + erff(v * 0.70710678118f));
    else if (act == 2) v = 0.5f * v * (1.f + tanhf(0.7978845608028654f * (v + 0.044715f * v * v * v)));
    else if (act == 3) v = v / (1.f + __expf(-v));
    x[r * xs + c] = f2bf(v);
  }
}

// qk [rows, heads*hd] in place. Pair i of a head (i < hd/2) is (x[i], x[i + hd/2]); pairs i < hd/4 turn with prow[r],
// the others with pcol[r], frequency theta^(-2 j / (hd/2)) with j the pair's index inside its half.
__global__ void rope2d_kernel(__nv_bfloat16* __restrict__ x, long xs, const int* __restrict__ prow, const int* __restrict__ pcol,
                              int heads, int hd, float theta) {
  const int r = blockIdx.x, h = blockIdx.y;
  const int half = hd / 2, quarter = hd / 4;
  for (int i = threadIdx.x; i < half; i += blockDim.x) {
    const int j = i < quarter ? i : i - quarter;
    const float pos = (float)(i < quarter ? prow[r] : pcol[r]);
    const float inv_freq = exp2f(-log2f(theta) * (2.f * (float)j / (float)half));
    float sn, cs;
    sincosf(pos * inv_freq, &sn, &cs);
    __nv_bfloat16* p = x + (long)r * xs + (long)h * hd;
    const float a = bf2f(p[i]), b = bf2f(p[i + half]);
    p[i] = f2bf(a * cs - b * sn);
    p[i + half] = f2bf(b * cs + a * sn);
  }
}

}  // namespace ve

using namespace ve;

extern "C" {

int ve_layernorm(const void* x, long xs, const void* w, const void* b, void* y, long ys, int rows, int H, float eps, cudaStream_t st) {
  if (rows <= 0) return 0;
  layernorm_kernel<<<rows, 256, 0, st>>>((const __nv_bfloat16*)x, xs, (const float*)w, (const float*)b, (__nv_bfloat16*)y, ys, H, eps);
  VE_CHECK_LAUNCH();
}
int ve_bias_act(void* x, long xs, const void* bias, long rows, int cols, int act, cudaStream_t st) {
  if (rows <= 0) return 0;
  const long n = rows * cols;
  const int blocks = (int)((n + 255) / 256 < 148 * 16 ? (n + 255) / 256 : 148 * 16);
  bias_act_kernel<<<blocks, 256, 0, st>>>((__nv_bfloat16*)x, xs, (const float*)bias, rows, cols, act);
  VE_CHECK_LAUNCH();
}
int ve_rope2d(void* x, long xs, const void* prow, const void* pcol, int rows, int heads, int hd, float theta, cudaStream_t st) {
  if (rows <= 0) return 0;
  if (hd % 4) return cudaErrorInvalidValue;
  rope2d_kernel<<<dim3(rows, heads), 64, 0, st>>>((__nv_bfloat16*)x, xs, (const int*)prow, (const int*)pcol, heads, hd, theta);
  VE_CHECK_LAUNCH();
}

}  // extern "C"
