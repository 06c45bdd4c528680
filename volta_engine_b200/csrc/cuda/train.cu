// Training primitives (fp32, row-major, caller's stream): the pieces the quantisation-tuning gradient passes are
// built from. Elementwise SwiGLU forward / backward (optionally with the clamp limit), row scaling, row-weighted
// squared error with gradient, Adam in three parameterisations (plain, log-scale s = s0 e^a, additive w = w0 + a),
// gathers / scatter-adds of routed rows, multiplicative parameters.
// Reference: inc/engine/train/grad.h:36-97, src/kernels/cuda/train/grad.cu.
#include "common.cuh"

namespace ve {

VE_DEVINL float sigm(float x) { return 1.f / (1.f + __expf(-x)); }

__global__ void swiglu_fwd_kernel(const float* g, const float* u, float* a, size_t n, float limit) {
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    float gv = g[i], uv = u[i];
    if (limit > 0.f) { gv = fminf(gv, limit); uv = fminf(fmaxf(uv, -limit), limit); }
    a[i] = gv * sigm(gv) * uv;
  }
}
__global__ void swiglu_bwd_kernel(const float* g, const float* u, const float* da, float* dg, float* du, size_t n, float limit) {
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    float gv = g[i], uv = u[i];
    bool g_live = true, u_live = true;
    if (limit > 0.f) {
      g_live = gv < limit; u_live = uv > -limit && uv < limit;
      gv = fminf(gv, limit); uv = fminf(fmaxf(uv, -limit), limit);
    }
    const float s = sigm(gv), act = gv * s;
    const float dact = s * (1.f + gv * (1.f - s));
    dg[i] = g_live ? da[i] * uv * dact : 0.f;
    du[i] = u_live ? da[i] * act : 0.f;
  }
}
__global__ void scale_rows_kernel(float* x, const float* s, int rows, int cols) {
  const size_t n = (size_t)rows * cols;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) x[i] *= s[i / cols];
}
// one block per row; partial[row] = w_r |y_r - t_r|^2 (t only: w_r |t_r|^2); dy = scale * 2 w_r (y - t)
__global__ void __launch_bounds__(256) sq_error_kernel(const float* y, const float* t, const float* w, int n, float* dy,
                                                       float scale, double* partial) {
  __shared__ float red[33];
  const int r = blockIdx.x;
  const float wr = w ? w[r] : 1.f;
  float acc = 0.f;
  for (int c = threadIdx.x; c < n; c += blockDim.x) {
    const float d = (y ? y[(size_t)r * n + c] : 0.f) - t[(size_t)r * n + c];
    acc = fmaf(d, d, acc);
    if (dy) dy[(size_t)r * n + c] = scale * 2.f * wr * d;
  }
  acc = block_sum(acc, red);
  if (threadIdx.x == 0) partial[r] = (double)acc * wr;
}
// mode 0: p -= step; mode 1: a -= step on d/da = s * g, s = s0 e^a; mode 2: a -= step, w = w0 + a
__global__ void adam_kernel(float* p, const float* base, float* derived, const float* g, float* m, float* v, size_t n,
                            float lr, float b1, float b2, float eps, float c1, float c2, float gscale, int mode) {
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    float gi = g[i] * gscale;
    if (mode == 1) gi *= derived[i];
    const float mi = b1 * m[i] + (1.f - b1) * gi, vi = b2 * v[i] + (1.f - b2) * gi * gi;
    m[i] = mi; v[i] = vi;
    const float pn = p[i] - lr * (mi / c1) / (sqrtf(vi / c2) + eps);
    p[i] = pn;
    if (mode == 1) derived[i] = base[i] * __expf(pn);
    else if (mode == 2) derived[i] = base[i] + pn;
  }
}
__global__ void gather_rows_kernel(const void* src, int half_src, const int* idx, const float* w, int n, int cols, float* dst) {
  const size_t total = (size_t)n * cols;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const int r = (int)(i / cols), c = (int)(i % cols);
    const size_t s = (size_t)idx[r] * cols + c;
    const float x = half_src ? __half2float(((const __half*)src)[s]) : ((const float*)src)[s];
    dst[i] = w ? x * w[r] : x;
  }
}
__global__ void scatter_add_rows_kernel(const float* src, const int* idx, const float* w, int n, int cols, float* dst) {
  const size_t total = (size_t)n * cols;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const int r = (int)(i / cols), c = (int)(i % cols);
    dst[(size_t)idx[r] * cols + c] += (w ? w[r] : 1.f) * src[i];
  }
}
__global__ void exp_scale_kernel(const float* base, const float* a, float* out, size_t n) {
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) out[i] = base[i] * __expf(a[i]);
}
__global__ void mul_kernel(const float* x, const float* y, float* out, size_t n) {
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) out[i] = x[i] * y[i];
}

static int blocks_for(size_t n) { const size_t b = (n + 255) / 256; return (int)(b < 148 * 16 ? (b ? b : 1) : 148 * 16); }

}  // namespace ve

using namespace ve;

extern "C" {

int ve_train_swiglu_fwd(const void* g, const void* u, void* a, long n, float limit, cudaStream_t st) {
  if (n <= 0) return 0;
  swiglu_fwd_kernel<<<blocks_for(n), 256, 0, st>>>((const float*)g, (const float*)u, (float*)a, (size_t)n, limit);
  VE_CHECK_LAUNCH();
}
int ve_train_swiglu_bwd(const void* g, const void* u, const void* da, void* dg, void* du, long n, float limit, cudaStream_t st) {
  if (n <= 0) return 0;
  swiglu_bwd_kernel<<<blocks_for(n), 256, 0, st>>>((const float*)g, (const float*)u, (const float*)da, (float*)dg, (float*)du, (size_t)n, limit);
  VE_CHECK_LAUNCH();
}
int ve_train_scale_rows(void* x, const void* s, int rows, int cols, cudaStream_t st) {
  if (rows <= 0) return 0;
  scale_rows_kernel<<<blocks_for((size_t)rows * cols), 256, 0, st>>>((float*)x, (const float*)s, rows, cols);
  VE_CHECK_LAUNCH();
}
int ve_train_sq_error(const void* y, const void* t, const void* w, int rows, int n, void* dy, float scale, void* partial, cudaStream_t st) {
  if (rows <= 0) return 0;
  sq_error_kernel<<<rows, 256, 0, st>>>((const float*)y, (const float*)t, (const float*)w, n, (float*)dy, scale, (double*)partial);
  VE_CHECK_LAUNCH();
}
int ve_train_adam(void* p, const void* base, void* derived, const void* g, void* m, void* v, long n, int step, float lr, float b1,
                  float b2, float eps, float gscale, int mode, cudaStream_t st) {
  if (n <= 0) return 0;
  if (step < 1 || mode < 0 || mode > 2) return cudaErrorInvalidValue;
  const float c1 = 1.f - powf(b1, (float)step), c2 = 1.f - powf(b2, (float)step);
  adam_kernel<<<blocks_for(n), 256, 0, st>>>((float*)p, (const float*)base, (float*)derived, (const float*)g, (float*)m, (float*)v,
                                             (size_t)n, lr, b1, b2, eps, c1, c2, gscale, mode);
  VE_CHECK_LAUNCH();
}
int ve_train_gather_rows(const void* src, int half_src, const void* idx, const void* w, int n, int cols, void* dst, cudaStream_t st) {
  if (n <= 0) return 0;
  gather_rows_kernel<<<blocks_for((size_t)n * cols), 256, 0, st>>>(src, half_src, (const int*)idx, (const float*)w, n, cols, (float*)dst);
  VE_CHECK_LAUNCH();
}
int ve_train_scatter_add_rows(const void* src, const void* idx, const void* w, int n, int cols, void* dst, cudaStream_t st) {
  if (n <= 0) return 0;
  scatter_add_rows_kernel<<<blocks_for((size_t)n * cols), 256, 0, st>>>((const float*)src, (const int*)idx, (const float*)w, n, cols, (float*)dst);
  VE_CHECK_LAUNCH();
}
int ve_train_exp_scale(const void* base, const void* a, void* out, long n, cudaStream_t st) {
  if (n <= 0) return 0;
  exp_scale_kernel<<<blocks_for(n), 256, 0, st>>>((const float*)base, (const float*)a, (float*)out, (size_t)n);
  VE_CHECK_LAUNCH();
}
int ve_train_mul(const void* x, const void* y, void* out, long n, cudaStream_t st) {
  if (n <= 0) return 0;
  mul_kernel<<<blocks_for(n), 256, 0, st>>>((const float*)x, (const float*)y, (float*)out, (size_t)n);
  VE_CHECK_LAUNCH();
}

}  // extern "C"
