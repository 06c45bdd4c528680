// Runtime steering of the residual stream: per-slot control vectors and direction clamps applied after chosen
// layers, and a per-slot logit penalty on marker tokens.
//   add         x += strength * v
//   clamp       x -= max(x . v - ref, 0) * v
//   clamp_keep  the clamp, then x rescaled to the norm it had before (only when the clamp removed something)
// Device-resident tables indexed by the slot of each row keep the decode graphs valid; a slot without steering is
// not touched. Rows are covered by scope bits: prompt (pos < prompt_len), think (< think_end), answer (after).
// Reference: inc/engine/modules/steer.h:11-80 (kinds, scopes, table layout), src/backend/cuda/modules/steer.cu.
#include "common.cuh"

namespace ve {

constexpr int kSteerEntries = 4;
enum { kSteerOff = 0, kSteerAdd = 1, kSteerClamp = 2, kSteerClampKeep = 3 };

struct SteerCtl { int scope, prompt_len, think_end, penalty_n; float penalty; int pad[3]; };

// grid rows, block 256. hidden [rows, H] bf16; vec [slots][layers][4][H] fp32; par / kind [slots][layers][4].
__global__ void __launch_bounds__(256) steer_apply_kernel(__nv_bfloat16* __restrict__ hidden, long stride, const int* __restrict__ pos,
                                                          const int* __restrict__ slot, const SteerCtl* __restrict__ ctl,
                                                          const float* __restrict__ vec, const float* __restrict__ par,
                                                          const int* __restrict__ kind, int layers, int layer, int H) {
  __shared__ float red[33];
  grid_dep_launch();
  grid_dep_wait();
  const int row = blockIdx.x;
  const int s = slot ? slot[row] : 0;
  if (s < 0) return;
  const SteerCtl c = ctl[s];
  if (c.scope == 0) return;
  const int p = pos[row];
  const int bit = p < c.prompt_len ? 1 : (p < c.think_end ? 2 : 4);
  if (!(c.scope & bit)) return;
  const long e0 = ((long)s * layers + layer) * kSteerEntries;
  __nv_bfloat16* x = hidden + (long)row * stride;
  for (int e = 0; e < kSteerEntries; ++e) {
    const int k = kind[e0 + e];
    if (k == kSteerOff) continue;
    const float* v = vec + (e0 + e) * (long)H;
    const float pr = par[e0 + e];
    if (k == kSteerAdd) {
      for (int i = threadIdx.x; i < H; i += blockDim.x) x[i] = f2bf(bf2f(x[i]) + pr * v[i]);
      __syncthreads();
      continue;
    }
    float dot = 0.f, n0 = 0.f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) { const float xv = bf2f(x[i]); dot = fmaf(xv, v[i], dot); n0 = fmaf(xv, xv, n0); }
    dot = block_sum(dot, red);
    n0 = block_sum(n0, red);
    const float over = fmaxf(dot - pr, 0.f);
    if (over <= 0.f) continue;
    float n1 = 0.f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) { const float y = bf2f(x[i]) - over * v[i]; n1 = fmaf(y, y, n1); }
    n1 = block_sum(n1, red);
    const float scale = (k == kSteerClampKeep && n1 > 0.f) ? sqrtf(n0 / n1) : 1.f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) x[i] = f2bf((bf2f(x[i]) - over * v[i]) * scale);
    __syncthreads();
  }
}

// logits [rows, V] fp32 of this rank's vocabulary shard [id0, id0 + V): subtract the slot's penalty from its marker ids
// while the predicted token lies inside the reasoning block. grid rows, block 256.
__global__ void steer_penalize_kernel(float* __restrict__ logits, long stride, const int* __restrict__ pos,
                                      const int* __restrict__ slot, const SteerCtl* __restrict__ ctl,
                                      const int* __restrict__ ids, int max_ids, int id0, int V) {
  grid_dep_launch();
  grid_dep_wait();
  const int row = blockIdx.x;
  const int s = slot ? slot[row] : 0;
  if (s < 0) return;
  const SteerCtl c = ctl[s];
  if (c.penalty_n <= 0) return;
  const int p = pos[row] + 1;                       // position of the token being predicted
  if (p < c.prompt_len || p >= c.think_end) return;
  for (int i = threadIdx.x; i < c.penalty_n && i < max_ids; i += blockDim.x) {
    const int id = ids[(long)s * max_ids + i] - id0;
    if (id >= 0 && id < V) logits[(long)row * stride + id] -= c.penalty;
  }
}

}  // namespace ve

using namespace ve;

extern "C" {

int ve_steer_apply(void* hidden, long stride, const void* pos, const void* slot, const void* ctl, const void* vec,
                   const void* par, const void* kind, int rows, int layers, int layer, int H, cudaStream_t st) {
  if (rows <= 0) return 0;
  launch_pdl(steer_apply_kernel, dim3(rows), dim3(256), 0, st, (__nv_bfloat16*)hidden, stride, (const int*)pos,
             (const int*)slot, (const SteerCtl*)ctl, (const float*)vec, (const float*)par, (const int*)kind, layers, layer, H);
  VE_CHECK_LAUNCH();
}

int ve_steer_penalize(void* logits, long stride, const void* pos, const void* slot, const void* ctl, const void* ids,
                      int max_ids, int id0, int V, int rows, cudaStream_t st) {
  if (rows <= 0) return 0;
  launch_pdl(steer_penalize_kernel, dim3(rows), dim3(256), 0, st, (float*)logits, stride, (const int*)pos, (const int*)slot,
             (const SteerCtl*)ctl, (const int*)ids, max_ids, id0, V);
  VE_CHECK_LAUNCH();
}

}  // extern "C"
