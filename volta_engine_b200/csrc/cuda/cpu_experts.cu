// GPU <-> CPU expert bridge: routes whose expert lives on the host are handed to a host service through a mailbox in pinned
// mapped memory and their weighted sum is added back after the device experts ran; both kernels read everything they need
// from device / mapped memory, so they replay inside CUDA graphs.
//   cpu_post      one CTA: takes the routes (row, expert, weight) of host-owned experts out of the route table (id := -1, so
//                 the device MoE kernels skip them), copies the rows' activations into the mailbox and publishes a request
//                 sequence number behind a system-scope fence
//   cpu_wait_add  one CTA: waits (bounded, status word on expiry) until the host has published the same sequence number,
//                 then adds the fp32 result rows to the layer output
// Mailbox layout (bytes): int64 header[8] = {req_seq, done_seq, layer, rows, nroutes, hidden, err, -}; routes at 64:
// kMaxRoutes x {int32 row, int32 expert, float weight, int32 -}; activations bf16 [16, hidden] at kOffX; results fp32
// [16, hidden] right after them.
// Reference: src/backend/cuda/modules/cpu_experts.cu:22-120 (cpu_post_kernel, cpu_wait_add_kernel),
// inc/engine/runtime/cpu_expert_service.h:13-60.
#include "common.cuh"

namespace ve {

constexpr int kMbRows = 16, kMaxRoutes = 512, kOffRoutes = 64, kOffX = kOffRoutes + kMaxRoutes * 16;

struct MbRoute { int row, expert; float weight; int pad; };

__global__ void __launch_bounds__(256) cpu_post_kernel(const __nv_bfloat16* __restrict__ x, long x_stride, int* __restrict__ ids,
                                                       const float* __restrict__ w, int rows, int topk, int hidden, int e0,
                                                       int e_local, const uint8_t* __restrict__ owner, uint8_t* mb,
                                                       unsigned long long* ctl, int layer) {
  __shared__ int s_pos[kMaxRoutes];
  __shared__ int s_total;
  grid_dep_wait();
  const int n = rows * topk, tid = threadIdx.x;
  for (int i = tid; i < n; i += blockDim.x) {
    const int e = ids[i] - e0;
    s_pos[i] = (e >= 0 && e < e_local && owner[e]) ? 1 : 0;
  }
  __syncthreads();
  if (tid == 0) {       // exclusive scan: mailbox order = route order
    int run = 0;
    for (int i = 0; i < n; ++i) {
      const int f = s_pos[i];
      s_pos[i] = f ? run : -1;
      run += f;
    }
    s_total = run;
  }
  __syncthreads();
  const int total = s_total;
  if (total == 0) {
    if (tid == 0) ctl[0] = 0;
    return;
  }
  MbRoute* routes = reinterpret_cast<MbRoute*>(mb + kOffRoutes);
  for (int i = tid; i < n; i += blockDim.x) {
    if (s_pos[i] < 0) continue;
    routes[s_pos[i]] = MbRoute{i / topk, ids[i], w[i], 0};
    ids[i] = -1;
  }
  __nv_bfloat16* mx = reinterpret_cast<__nv_bfloat16*>(mb + kOffX);
  for (int i = tid; i < rows * hidden; i += blockDim.x) mx[i] = x[(long)(i / hidden) * x_stride + i % hidden];
  __threadfence_system();
  __syncthreads();
  if (tid == 0) {
    long long* hdr = reinterpret_cast<long long*>(mb);
    hdr[2] = layer; hdr[3] = rows; hdr[4] = total; hdr[5] = hidden;
    const unsigned long long seq = ctl[1] + 1;
    ctl[1] = seq;
    ctl[0] = seq;
    __threadfence_system();
    *reinterpret_cast<volatile unsigned long long*>(hdr) = seq;
    __threadfence_system();
  }
}

__global__ void __launch_bounds__(256) cpu_wait_add_kernel(__nv_bfloat16* __restrict__ out, long out_stride, int rows, int hidden,
                                                           const uint8_t* mb, const unsigned long long* __restrict__ ctl,
                                                           unsigned long long budget_ns, int* status) {
  __shared__ int ok;
  grid_dep_wait();
  const unsigned long long seq = ctl[0];
  if (seq == 0) return;
  if (threadIdx.x == 0) {
    ok = 1;
    const volatile unsigned long long* done = reinterpret_cast<const volatile unsigned long long*>(mb) + 1;
    const uint64_t t0 = globaltimer_ns();
    while (*done < seq) {
      if (globaltimer_ns() - t0 > budget_ns) {
        ok = 0;
        if (status) atomicExch(status, (int)kErrPeerTimeout);
        break;
      }
      __nanosleep(200);
    }
  }
  __syncthreads();
  if (!ok) return;
  __threadfence_system();
  const float* mo = reinterpret_cast<const float*>(mb + kOffX + (size_t)kMbRows * hidden * 2);
  for (int i = threadIdx.x; i < rows * hidden; i += blockDim.x) {
    __nv_bfloat16* o = out + (long)(i / hidden) * out_stride + i % hidden;
    *o = __float2bfloat16_rn(__bfloat162float(*o) + __ldcv(mo + i));
  }
}

}  // namespace ve

using namespace ve;

extern "C" {

int ve_cpu_post(const void* x, long x_stride, void* ids, const void* w, int rows, int topk, int hidden, int e0, int e_local,
                const void* owner, void* mailbox, void* ctl, int layer, cudaStream_t st) {
  if (rows <= 0) return 0;
  if (rows > kMbRows || rows * topk > kMaxRoutes) return cudaErrorInvalidValue;
  launch_pdl(cpu_post_kernel, dim3(1), dim3(256), 0, st, (const __nv_bfloat16*)x, x_stride, (int*)ids, (const float*)w, rows,
             topk, hidden, e0, e_local, (const uint8_t*)owner, (uint8_t*)mailbox, (unsigned long long*)ctl, layer);
  VE_CHECK_LAUNCH();
}

int ve_cpu_wait_add(void* out, long out_stride, int rows, int hidden, const void* mailbox, const void* ctl,
                    unsigned long long budget_ns, void* status, cudaStream_t st) {
  if (rows <= 0) return 0;
  launch_pdl(cpu_wait_add_kernel, dim3(1), dim3(256), 0, st, (__nv_bfloat16*)out, out_stride, rows, hidden,
             (const uint8_t*)mailbox, (const unsigned long long*)ctl, budget_ns, (int*)status);
  VE_CHECK_LAUNCH();
}

int ve_cpu_mailbox_bytes(int hidden) { return kOffX + kMbRows * hidden * 2 + kMbRows * hidden * 4; }

}  // extern "C"
