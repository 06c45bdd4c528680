// Gated DeltaNet mixer (linear attention with a gated delta rule):
//   gdn_prepare    parallel over rows: causal short convolution + SiLU over the q|k|v channels (taps from earlier rows
//                  of the same slot in the batch, else from the slot's convolution state), L2 norm of q and k per head,
//                  q scale, decay exp(g) and beta per value head
//   gdn_recurrent  one CTA per (value head, slot): walks the slot's rows in order with the state column of every thread
//                  in registers:  S *= decay;  delta = (v - S^T k) * beta;  S += k (x) delta;  o = S^T q;
//                  stores the state, and (head 0) rolls the slot's convolution state forward
//   gdn_gated_norm y = rmsnorm(o) * w * silu(z)
// KDA (Kimi delta attention) is the same recurrence with one decay per key channel, S = diag(exp(g)) S, where
//   g = -5 sigmoid(exp(A_log[h]) (f + dt_bias)) and f is a low-rank projection of the input; its output gate is sigmoid(z)
//   (reference: src/backend/cpu/gdn_ref.cpp:32-57 kda_head_step, :94-127 project_kda_gates, :59-68 gate_norm_out).
// A row at position 0 starts its slot from zero state. fp32 state and arithmetic; the fused projection row is
// [q | k | v | z | b | a] in bf16. Reference: inc/engine/modules/gdn.h (project_gates, causal_conv1d_silu*,
// l2_norm_heads, recurrent_step[_rows], gated_rmsnorm).
#include "common.cuh"

namespace ve {

struct GdnArgs {
  const __nv_bfloat16* proj; long ld;
  const int* pos; const int* slot;
  float* conv_state;            // [slots][kc-1][C]
  float* rec_state;             // [slots][nv][dk][dv]
  const float* conv_w;          // [C][kc]
  const float* A_log; const float* dt_bias;
  float* u;                     // [rows][C]   conv + norm outputs
  float* gb;                    // [rows][2*nv] decay, beta
  float* o;                     // [rows][nv*dv]
  int rows, nk, nv, dk, dv, kc, slots;
  const float* kdec;            // KDA: [rows][nv * dk] per-key-channel decay exp(g); null = one decay per head (gb)
};

VE_DEVINL float siluf(float x) { return x / (1.f + __expf(-x)); }

// rows of the same slot directly in front of row i (at most lim)
VE_DEVINL int rows_before(const int* slot, const int* pos, int i, int lim) {
  int r = 0;
  while (r < lim && i - r - 1 >= 0 && slot[i - r - 1] == slot[i] && pos[i - r - 1] == pos[i] - r - 1) ++r;
  return r;
}

// grid (2*nk + nv + 1, rows), block = max(dk, dv) threads. Unit < nk: q head; < 2nk: k head; < 2nk+nv: v head; last: gates.
__global__ void gdn_prepare_kernel(const GdnArgs a) {
  __shared__ float red[33];
  grid_dep_launch();
  grid_dep_wait();
  const int unit = blockIdx.x, i = blockIdx.y, tid = threadIdx.x;
  const int s = a.slot[i];
  if (s < 0) return;
  const int C = 2 * a.nk * a.dk + a.nv * a.dv;
  if (unit == 2 * a.nk + a.nv) {
    if (tid < a.nv) {
      const __nv_bfloat16* row = a.proj + (long)i * a.ld + C + a.nv * a.dv;
      const float b = bf2f(row[tid]), av = bf2f(row[a.nv + tid]);
      const float x = av + a.dt_bias[tid];
      const float sp = x > 20.f ? x : log1pf(__expf(x));
      a.gb[(long)i * 2 * a.nv + tid] = __expf(-__expf(a.A_log[tid]) * sp);
      a.gb[(long)i * 2 * a.nv + a.nv + tid] = 1.f / (1.f + __expf(-b));
    }
    return;
  }
  const bool is_v = unit >= 2 * a.nk;
  const int width = is_v ? a.dv : a.dk;
  const int c0 = is_v ? 2 * a.nk * a.dk + (unit - 2 * a.nk) * a.dv : unit * a.dk;
  const int p = a.pos[i];
  const int r = rows_before(a.slot, a.pos, i, a.kc - 1);
  float val = 0.f;
  if (tid < width) {
    const int c = c0 + tid;
    float acc = 0.f;
    for (int d = 0; d < a.kc; ++d) {               // d = distance into the past of the tap
      if (p - d < 0) break;
      float x;
      if (d <= r) x = bf2f(a.proj[(long)(i - d) * a.ld + c]);
      else x = a.conv_state[((long)s * (a.kc - 1) + (a.kc - 1 - (d - r))) * C + c];
      acc += x * a.conv_w[(long)c * a.kc + (a.kc - 1 - d)];
    }
    val = siluf(acc);
  }
  if (!is_v) {
    const float ss = block_sum(val * val, red);
    const float inv = rsqrtf(ss + 1e-6f) * (unit < a.nk ? rsqrtf((float)a.dk) : 1.f);
    val *= inv;
  }
  if (tid < width) a.u[(long)i * C + c0 + tid] = val;
}

// grid (nv, slots), block dv threads; thread = one column of the head's state.
template <int DK>
__global__ void __launch_bounds__(256) gdn_recurrent_kernel(const GdnArgs a) {
  __shared__ float ks[DK], qs[DK], ds[DK];
  grid_dep_launch();
  grid_dep_wait();
  const int h = blockIdx.x, s = blockIdx.y, col = threadIdx.x;
  // rows of this slot (consecutive)
  int first = -1, count = 0;
  for (int i = 0; i < a.rows; ++i)
    if (a.slot[i] == s) { if (first < 0) first = i; ++count; }
  if (count == 0) return;
  const int C = 2 * a.nk * a.dk + a.nv * a.dv;
  const int kh = h / (a.nv / a.nk);
  const bool fresh = a.pos[first] == 0;
  float* st = a.rec_state + (((long)s * a.nv + h) * DK) * a.dv + col;
  float S[DK];
#pragma unroll
  for (int k = 0; k < DK; ++k) S[k] = fresh ? 0.f : st[(long)k * a.dv];
  for (int r = 0; r < count; ++r) {
    const int i = first + r;
    const float* ui = a.u + (long)i * C;
    const float decay = a.gb[(long)i * 2 * a.nv + h], beta = a.gb[(long)i * 2 * a.nv + a.nv + h];
    for (int t = col; t < DK; t += blockDim.x) {
      qs[t] = ui[kh * DK + t];
      ks[t] = ui[a.nk * DK + kh * DK + t];
      ds[t] = a.kdec ? a.kdec[((long)i * a.nv + h) * DK + t] : decay;
    }
    __syncthreads();
    const float v = ui[2 * a.nk * DK + h * a.dv + col];
    float mem = 0.f;
#pragma unroll
    for (int k = 0; k < DK; ++k) { S[k] *= ds[k]; mem = fmaf(S[k], ks[k], mem); }
    const float delta = (v - mem) * beta;
    float o = 0.f;
#pragma unroll
    for (int k = 0; k < DK; ++k) { S[k] = fmaf(ks[k], delta, S[k]); o = fmaf(S[k], qs[k], o); }
    a.o[(long)i * a.nv * a.dv + h * a.dv + col] = o;
    __syncthreads();
  }
#pragma unroll
  for (int k = 0; k < DK; ++k) st[(long)k * a.dv] = S[k];
  {
    // roll the convolution state: the newest kc-1 inputs of the slot, oldest first. The channels are dealt to the head
    // blocks of the slot (every channel is independent), so no block walks all of them alone.
    const int n1 = a.kc - 1;
    float* cs = a.conv_state + (long)s * n1 * C;
    for (int c = h * blockDim.x + col; c < C; c += gridDim.x * blockDim.x) {
      float old[8], nw[8];
      for (int t = 0; t < n1; ++t) old[t] = fresh ? 0.f : cs[(long)t * C + c];
      for (int t = 0; t < n1; ++t) {
        const int e = n1 - 1 - t;                    // distance from the last row
        if (e < count) nw[t] = bf2f(a.proj[(long)(first + count - 1 - e) * a.ld + c]);
        else nw[t] = old[n1 - 1 - (e - count)];
      }
      for (int t = 0; t < n1; ++t) cs[(long)t * C + c] = nw[t];
    }
  }
}

// grid (nv, rows), block dv threads.
template <bool SIGMOID>
__global__ void gdn_gated_norm_kernel(const float* __restrict__ o, const __nv_bfloat16* __restrict__ proj, long ld,
                                      const float* __restrict__ w, __nv_bfloat16* __restrict__ out, int nv, int dv,
                                      int z_off, float eps) {
  __shared__ float red[33];
  grid_dep_launch();
  grid_dep_wait();
  const int h = blockIdx.x, i = blockIdx.y, col = threadIdx.x;
  const float x = o[((long)i * nv + h) * dv + col];
  const float ss = block_sum(x * x, red);
  const float z = bf2f(proj[(long)i * ld + z_off + h * dv + col]);
  const float gate = SIGMOID ? 1.f / (1.f + __expf(-z)) : siluf(z);
  out[((long)i * nv + h) * dv + col] = f2bf(x * rsqrtf(ss / dv + eps) * w[col] * gate);
}

// KDA decay per key channel: kdec[row][j] = exp(-5 sigmoid(exp(A_log[j / dk]) (f[row][j] + dt_bias[j]))). grid (rows, channel chunks).
__global__ void kda_decay_kernel(const __nv_bfloat16* __restrict__ f, long ld, const float* __restrict__ A_log,
                                 const float* __restrict__ dt_bias, float* __restrict__ kdec, int channels, int dk) {
  grid_dep_launch();
  grid_dep_wait();
  const int i = blockIdx.x;
  for (int j = blockIdx.y * blockDim.x + threadIdx.x; j < channels; j += gridDim.y * blockDim.x) {
    const float x = __expf(A_log[j / dk]) * (bf2f(f[(long)i * ld + j]) + dt_bias[j]);
    kdec[(long)i * channels + j] = __expf(-5.f / (1.f + __expf(-x)));
  }
}

}  // namespace ve

using namespace ve;

extern "C" {

int ve_gdn_prepare(const void* proj, long ld, const void* pos, const void* slot, void* conv_state, const void* conv_w,
                   const void* A_log, const void* dt_bias, void* u, void* gb, int rows, int nk, int nv, int dk, int dv,
                   int kc, int slots, cudaStream_t st) {
  if (rows <= 0) return 0;
  if (kc < 2 || kc > 9 || dk > 256 || dv > 256 || nv % nk || nv > 256) return cudaErrorInvalidValue;
  GdnArgs a{(const __nv_bfloat16*)proj, ld, (const int*)pos, (const int*)slot, (float*)conv_state, nullptr,
            (const float*)conv_w, (const float*)A_log, (const float*)dt_bias, (float*)u, (float*)gb, nullptr,
            rows, nk, nv, dk, dv, kc, slots, nullptr};
  int threads = dk > dv ? dk : dv;
  if (threads < nv) threads = nv;
  threads = (threads + 31) / 32 * 32;
  launch_pdl(gdn_prepare_kernel, dim3(2 * nk + nv + 1, rows), dim3(threads), 0, st, a);
  VE_CHECK_LAUNCH();
}

int ve_gdn_recurrent(const void* proj, long ld, const void* pos, const void* slot, void* conv_state, void* rec_state,
                     const void* u, const void* gb, void* o, int rows, int nk, int nv, int dk, int dv, int kc, int slots,
                     cudaStream_t st) {
  if (rows <= 0) return 0;
  if (kc < 2 || kc > 9 || dv > 256 || dv % 32 || nv % nk) return cudaErrorInvalidValue;
  GdnArgs a{(const __nv_bfloat16*)proj, ld, (const int*)pos, (const int*)slot, (float*)conv_state, (float*)rec_state,
            nullptr, nullptr, nullptr, (float*)u, (float*)gb, (float*)o, rows, nk, nv, dk, dv, kc, slots, nullptr};
  if (dk == 128) launch_pdl(gdn_recurrent_kernel<128>, dim3(nv, slots), dim3(dv), 0, st, a);
  else if (dk == 64) launch_pdl(gdn_recurrent_kernel<64>, dim3(nv, slots), dim3(dv), 0, st, a);
  else return cudaErrorInvalidValue;
  VE_CHECK_LAUNCH();
}

// The recurrence with one decay per key channel (kdec [rows][nv * dk], already exponentiated).
int ve_kda_recurrent(const void* proj, long ld, const void* pos, const void* slot, void* conv_state, void* rec_state,
                     const void* u, const void* gb, void* o, const void* kdec, int rows, int nk, int nv, int dk, int dv, int kc,
                     int slots, cudaStream_t st) {
  if (rows <= 0) return 0;
  if (kc < 2 || kc > 9 || dv > 256 || dv % 32 || nv % nk || !kdec) return cudaErrorInvalidValue;
  GdnArgs a{(const __nv_bfloat16*)proj, ld, (const int*)pos, (const int*)slot, (float*)conv_state, (float*)rec_state,
            nullptr, nullptr, nullptr, (float*)u, (float*)gb, (float*)o, rows, nk, nv, dk, dv, kc, slots, (const float*)kdec};
  if (dk == 128) launch_pdl(gdn_recurrent_kernel<128>, dim3(nv, slots), dim3(dv), 0, st, a);
  else if (dk == 64) launch_pdl(gdn_recurrent_kernel<64>, dim3(nv, slots), dim3(dv), 0, st, a);
  else return cudaErrorInvalidValue;
  VE_CHECK_LAUNCH();
}

int ve_kda_decay(const void* f, long ld, const void* A_log, const void* dt_bias, void* kdec, int rows, int nv, int dk,
                 cudaStream_t st) {
  if (rows <= 0) return 0;
  const int chunks = (nv * dk + 1023) / 1024;          // 256 threads take four channels each
  launch_pdl(kda_decay_kernel, dim3(rows, chunks), dim3(256), 0, st, (const __nv_bfloat16*)f, ld, (const float*)A_log,
             (const float*)dt_bias, (float*)kdec, nv * dk, dk);
  VE_CHECK_LAUNCH();
}

int ve_gdn_gated_norm(const void* o, const void* proj, long ld, const void* w, void* out, int rows, int nv, int dv,
                      int conv_dim, int kc, float eps, cudaStream_t st) {
  if (rows <= 0) return 0;
  if (dv > 1024 || dv % 32) return cudaErrorInvalidValue;
  launch_pdl(gdn_gated_norm_kernel<false>, dim3(nv, rows), dim3(dv), 0, st, (const float*)o, (const __nv_bfloat16*)proj, ld,
             (const float*)w, (__nv_bfloat16*)out, nv, dv, conv_dim, eps);
  VE_CHECK_LAUNCH();
}

// y = rmsnorm(o) * w * sigmoid(z); z [rows, nv * dv] bf16 with row stride ld.
int ve_kda_gated_norm(const void* o, const void* z, long ld, const void* w, void* out, int rows, int nv, int dv, float eps,
                      cudaStream_t st) {
  if (rows <= 0) return 0;
  if (dv > 1024 || dv % 32) return cudaErrorInvalidValue;
  launch_pdl(gdn_gated_norm_kernel<true>, dim3(nv, rows), dim3(dv), 0, st, (const float*)o, (const __nv_bfloat16*)z, ld,
             (const float*)w, (__nv_bfloat16*)out, nv, dv, 0, eps);
  VE_CHECK_LAUNCH();
}

}  // extern "C"
