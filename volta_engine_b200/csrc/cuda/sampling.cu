// Row-wise logits reductions for sampling on a vocabulary shard: argmax (ties -> lowest id), top-16
// candidates in descending order, log-sum-exp. These are what the host-side sampler merges across
// vocabulary shards (reference behaviour: inc/engine/runtime/sampling.h:9-15,82-110 and the shard merge
// in src/runtime/cluster.cpp:558-646; device kernels src/backend/cuda/modules/norm.cu batched_argmax*).
#include "common.cuh"
#include <float.h>

namespace ve {

struct ArgVal {
  float v;
  int i;
};
VE_DEVINL ArgVal better(ArgVal a, ArgVal b) { return (b.v > a.v || (b.v == a.v && b.i < a.i)) ? b : a; }

VE_DEVINL ArgVal block_argmax(ArgVal a, ArgVal* red) {
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nw = blockDim.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    ArgVal b;
    b.v = __shfl_xor_sync(0xffffffffu, a.v, o);
    b.i = __shfl_xor_sync(0xffffffffu, a.i, o);
    a = better(a, b);
  }
  if (lane == 0) red[wid] = a;
  __syncthreads();
  if (wid == 0) {
    ArgVal t = lane < nw ? red[lane] : ArgVal{-FLT_MAX, 0x7fffffff};
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      ArgVal b;
      b.v = __shfl_xor_sync(0xffffffffu, t.v, o);
      b.i = __shfl_xor_sync(0xffffffffu, t.i, o);
      t = better(t, b);
    }
    if (lane == 0) red[32] = t;
  }
  __syncthreads();
  ArgVal r = red[32];
  __syncthreads();
  return r;
}

// One CTA per row. Writes idx[row] (+ id_offset) and val[row].
__global__ void __launch_bounds__(1024) argmax_kernel(const float* __restrict__ logits, long stride, int V,
                                                      int id_offset, int* __restrict__ idx,
                                                      float* __restrict__ val) {
  __shared__ ArgVal red[33];
  const float* row = logits + blockIdx.x * stride;
  ArgVal a{-FLT_MAX, 0x7fffffff};
  for (int i = threadIdx.x; i < V; i += blockDim.x) a = better(a, ArgVal{row[i], i});
  a = block_argmax(a, red);
  if (threadIdx.x == 0) {
    idx[blockIdx.x] = a.i + id_offset;
    if (val) val[blockIdx.x] = a.v;
  }
}

// Two-stage argmax for wide vocabularies: grid (rows, NB) partial winners, then one small CTA per row.
__global__ void __launch_bounds__(256) argmax_part_kernel(const float* __restrict__ logits, long stride, int V,
                                                          float* __restrict__ pval, int* __restrict__ pidx) {
  __shared__ ArgVal red[33];
  grid_dep_launch();
  grid_dep_wait();
  const float* row = logits + blockIdx.x * stride;
  const int nb = gridDim.y, per = (V + nb - 1) / nb;
  const int lo = blockIdx.y * per, hi = min(V, lo + per);
  ArgVal a{-FLT_MAX, 0x7fffffff};
  for (int i = lo + threadIdx.x; i < hi; i += blockDim.x) a = better(a, ArgVal{row[i], i});
  a = block_argmax(a, red);
  if (threadIdx.x == 0) {
    pval[blockIdx.x * nb + blockIdx.y] = a.v;
    pidx[blockIdx.x * nb + blockIdx.y] = a.i;
  }
}
__global__ void __launch_bounds__(64) argmax_final_kernel(const float* __restrict__ pval, const int* __restrict__ pidx,
                                                          int nb, int id_offset, int* __restrict__ idx,
                                                          float* __restrict__ val) {
  grid_dep_launch();
  grid_dep_wait();
  __shared__ ArgVal red[33];
  ArgVal a{-FLT_MAX, 0x7fffffff};
  for (int i = threadIdx.x; i < nb; i += blockDim.x) a = better(a, ArgVal{pval[blockIdx.x * nb + i], pidx[blockIdx.x * nb + i]});
  a = block_argmax(a, red);
  if (threadIdx.x == 0) {
    idx[blockIdx.x] = a.i + id_offset;
    if (val) val[blockIdx.x] = a.v;
  }
}

// Top-K (K <= 16) by K rounds of block argmax with a "strictly after the previous pick" filter, so the
// logits are never modified: pick j is the best (value, id) pair ordered after pick j-1.
__global__ void __launch_bounds__(1024) topk_kernel(const float* __restrict__ logits, long stride, int V,
                                                    int id_offset, int K, int* __restrict__ ids,
                                                    float* __restrict__ vals, float* __restrict__ lse) {
  __shared__ ArgVal red[33];
  __shared__ float fred[33];
  const float* row = logits + blockIdx.x * stride;
  ArgVal prev{FLT_MAX, -1};
  float top = 0.f;
  for (int k = 0; k < K; ++k) {
    ArgVal a{-FLT_MAX, 0x7fffffff};
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
      const float v = row[i];
      const bool after = v < prev.v || (v == prev.v && i > prev.i);
      if (after) a = better(a, ArgVal{v, i});
    }
    a = block_argmax(a, red);
    if (k == 0) top = a.v;
    if (threadIdx.x == 0) {
      ids[blockIdx.x * K + k] = a.i == 0x7fffffff ? -1 : a.i + id_offset;
      vals[blockIdx.x * K + k] = a.v;
    }
    prev = a;
  }
  if (lse) {
    float s = 0.f;
    for (int i = threadIdx.x; i < V; i += blockDim.x) s += __expf(row[i] - top);
    s = block_sum(s, fred);
    if (threadIdx.x == 0) lse[blockIdx.x] = top + logf(s);
  }
}

}  // namespace ve

using namespace ve;

extern "C" {

int ve_argmax(const void* logits, long stride, int rows, int V, int id_offset, void* idx, void* val,
              cudaStream_t st) {
  if (rows <= 0) return 0;
  argmax_kernel<<<rows, 1024, 0, st>>>((const float*)logits, stride, V, id_offset, (int*)idx, (float*)val);
  VE_CHECK_LAUNCH();
}

// scratch: rows * nb floats + rows * nb ints
int ve_argmax2(const void* logits, long stride, int rows, int V, int id_offset, void* idx, void* val, void* pval,
               void* pidx, int nb, cudaStream_t st) {
  if (rows <= 0) return 0;
  dim3 grid(rows, nb);
  launch_pdl(argmax_part_kernel, grid, dim3(256), 0, st, (const float*)logits, stride, V, (float*)pval, (int*)pidx);
  launch_pdl(argmax_final_kernel, dim3(rows), dim3(64), 0, st, (const float*)pval, (const int*)pidx, nb, id_offset,
             (int*)idx, (float*)val);
  VE_CHECK_LAUNCH();
}

int ve_topk(const void* logits, long stride, int rows, int V, int id_offset, int K, void* ids, void* vals,
            void* lse, cudaStream_t st) {
  if (rows <= 0) return 0;
  if (K < 1 || K > 64) return cudaErrorInvalidValue;
  topk_kernel<<<rows, 1024, 0, st>>>((const float*)logits, stride, V, id_offset, K, (int*)ids, (float*)vals,
                                     (float*)lse);
  VE_CHECK_LAUNCH();
}

}  // extern "C"
