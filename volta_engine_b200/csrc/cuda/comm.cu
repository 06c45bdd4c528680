// Tensor-parallel collectives over NVLink 5 / NVSwitch, written against peer-mapped symmetric memory.
// One process per GPU; every rank passes the same table of peer base pointers (and, when NVLS is
// available, the multicast alias of the same buffer).
//
// Forms (reference counterpart: src/comm/all_reduce_ipc.cu — LL push :65-134,365-402, fused
// all-reduce + residual + RMSNorm :136-298, staged pull :300-363, sequence protocol :14-51):
//   ll_allreduce      one-shot push for <= 16 rows: each 8 B of payload travels as a 16 B line
//                     {d0, seq, d1, seq}; the reader spins on its own memory until both tags match.
//                     mode 0: y = sum ; mode 1: residual += bf16(sum); out = RMSNorm(residual) * (w + b);
//                     modes 2-4: the sandwich-norm, gated-stream and hyper-connection epilogues of
//                     stream_epilogues.cuh applied to bf16(sum) in the same launch.
//   rs_norm_ag        two-shot for prefill chunks: every rank owns T/N rows; it pulls that slice from all
//                     peers (plain peer loads, or one multimem.ld_reduce through the switch), adds its
//                     residual shard, normalises, and pushes the normalised rows to every rank
//                     (peer stores or one multimem.st).
//   ll_argmax_merge   merges per-shard (value, id) pairs so every rank knows the global greedy token.
// Sums are taken in rank order 0..N-1 on every rank, so all ranks hold bit-identical results, and the
// fused forms round the reduced value to bf16 before the residual update, so fused == unfused bits.
// Sequence numbers live in device memory and are advanced by the kernels themselves (CUDA-graph replay
// safe). Every wait has a wall-clock budget; on expiry the kernel records kErrPeerTimeout in the status
// word and completes.
#include "common.cuh"
#include "stream_epilogues.cuh"

namespace ve {

constexpr int kMaxRanks = 8;
constexpr int kLLStages = 4;
constexpr int kLLMaxRows = 16;

struct CommArgs {
  uint8_t* peer[kMaxRanks];  // symmetric buffer base of every rank, as mapped into this process
  uint8_t* mc;               // multicast alias of the symmetric buffer (nullptr when NVLS is unavailable)
  int rank, size;
  uint32_t* seq;             // [4] device-resident counters: 0 = LL sequence, 1 = LL finished CTAs,
                             //                               2 = two-shot sequence, 3 = two-shot finished CTAs
  int* status;
  unsigned long long budget_ns;
  // byte offsets inside the symmetric buffer (identical on all ranks)
  size_t off_ll;     // LL staging: [stage][src][row][H/4 lines x 16 B]
  size_t ll_row_bytes;  // bytes reserved per (stage, src, row)
  size_t off_flags;  // barrier flags: [cta][src] u32
  size_t off_part;   // two-shot partial input  [T, H] bf16
  size_t off_xout;   // two-shot normalised out [T, H] bf16
};

VE_DEVINL void st_volatile_v4(void* p, uint4 v) {
  asm volatile("st.volatile.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
               : "memory");
}
VE_DEVINL uint4 ld_volatile_v4(const void* p) {
  uint4 v;
  asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p)
               : "memory");
  return v;
}

// Poll one LL line until both tags equal seq. Returns false on timeout, and at once when `gave_up` is already set: after
// the first wait of a launch (or of an earlier launch: the status word) ran out of time, every later wait is skipped, so a
// peer that left costs one wait budget, not one per line, source and replayed kernel.
VE_DEVINL bool ll_wait(const void* line, uint32_t seq, uint2& data, unsigned long long budget, volatile int* gave_up) {
  uint4 v = ld_volatile_v4(line);
  if (v.y == seq && v.w == seq) {
    data = make_uint2(v.x, v.z);
    return true;
  }
  if (*gave_up) return false;
  const uint64_t t0 = globaltimer_ns();
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 32; ++i) {
      v = ld_volatile_v4(line);
      if (v.y == seq && v.w == seq) {
        data = make_uint2(v.x, v.z);
        return true;
      }
    }
    if (*gave_up || globaltimer_ns() - t0 > budget) return false;
  }
}

VE_DEVINL uint32_t pack2(float lo, float hi) {
  __nv_bfloat162 t = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&t);
}

VE_DEVINL void acc_bf16x4(float* a, uint2 d) {
  a[0] += __uint_as_float(d.x << 16);
  a[1] += __uint_as_float(d.x & 0xffff0000u);
  a[2] += __uint_as_float(d.y << 16);
  a[3] += __uint_as_float(d.y & 0xffff0000u);
}

// grid = rows, block = 256..1024
template <int MODE>
__global__ void __launch_bounds__(1024) ll_allreduce_kernel(const CommArgs a, const __nv_bfloat16* __restrict__ partial,
                                                            long part_stride, __nv_bfloat16* __restrict__ residual,
                                                            const __nv_bfloat16* __restrict__ w,
                                                            __nv_bfloat16* __restrict__ out, long out_stride, int H,
                                                            float eps, float wbias, int pushed, const EpiArgs epi) {
  extern __shared__ float rowbuf[];  // H floats (MODE >= 1)
  __shared__ float red[33];
  __shared__ volatile int s_timeout;
  const int row = blockIdx.x, tid = threadIdx.x;
  grid_dep_launch();                 // the kernel behind this one may be scheduled and set up now
  const int lines = H >> 2;
  if (tid == 0) s_timeout = (a.status && *reinterpret_cast<volatile int*>(a.status) != 0) ? 1 : 0;
  __syncthreads();
  // partial / residual belong to the kernel in front, and the sequence number to the all-reduce before that one: both
  // are complete once the dependency wait returns (the kernel in front waited for that all-reduce itself)
  grid_dep_wait();
  const uint32_t seq = a.seq[0];
  const int stage = seq & (kLLStages - 1);
  const __nv_bfloat16* prow = partial + (long)row * part_stride;
  const size_t slot_me = a.off_ll + ((size_t)(stage * a.size + a.rank) * kLLMaxRows + row) * a.ll_row_bytes;
  // push (skipped when the kernel that produced ``partial`` already sent the lines from its epilogue)
  for (int l = tid; l < lines && !pushed; l += blockDim.x) {
    const uint2 d = *reinterpret_cast<const uint2*>(prow + l * 4);
    const uint4 pkt = make_uint4(d.x, seq, d.y, seq);
#pragma unroll
    for (int i = 1; i < kMaxRanks; ++i) {
      if (i >= a.size) break;
      const int peer = (a.rank + i) % a.size;
      st_volatile_v4(a.peer[peer] + slot_me + (size_t)l * 16, pkt);
    }
  }
  // gather + reduce in rank order. The lines of all sources are requested together and only the ones whose tags do not
  // match yet are asked for again: one round trip to L2 per poll, not one per source.
  float ss = 0.f;
  for (int l = tid; l < lines; l += blockDim.x) {
    uint4 v[kMaxRanks];
    const uint8_t* lp[kMaxRanks];
#pragma unroll
    for (int src = 0; src < kMaxRanks; ++src) {
      if (src >= a.size || src == a.rank) continue;
      lp[src] = a.peer[a.rank] + a.off_ll + ((size_t)(stage * a.size + src) * kLLMaxRows + row) * a.ll_row_bytes + (size_t)l * 16;
      v[src] = ld_volatile_v4(lp[src]);
    }
    bool all = false;
    uint64_t t0 = 0;
    while (!all) {
      all = true;
#pragma unroll
      for (int src = 0; src < kMaxRanks; ++src) {
        if (src >= a.size || src == a.rank) continue;
        if (v[src].y != seq || v[src].w != seq) {
          v[src] = ld_volatile_v4(lp[src]);
          all = all && v[src].y == seq && v[src].w == seq;
        }
      }
      if (all) break;
      if (s_timeout) break;
      if (t0 == 0) t0 = globaltimer_ns();
      else if (globaltimer_ns() - t0 > a.budget_ns) { s_timeout = 1; break; }
    }
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int src = 0; src < kMaxRanks; ++src) {
      if (src >= a.size) continue;
      uint2 d;
      if (src == a.rank) d = *reinterpret_cast<const uint2*>(prow + l * 4);
      else d = (v[src].y == seq && v[src].w == seq) ? make_uint2(v[src].x, v[src].z) : make_uint2(0u, 0u);
      acc_bf16x4(acc, d);
    }
    __nv_bfloat162 y01 = __floats2bfloat162_rn(acc[0], acc[1]), y23 = __floats2bfloat162_rn(acc[2], acc[3]);
    if (MODE == 0) {
      uint2 o;
      o.x = *reinterpret_cast<uint32_t*>(&y01);
      o.y = *reinterpret_cast<uint32_t*>(&y23);
      *reinterpret_cast<uint2*>(out + (long)row * out_stride + l * 4) = o;
    } else if (MODE >= 2) {
      const float2 f01 = __bfloat1622float2(y01), f23 = __bfloat1622float2(y23);
      rowbuf[l * 4 + 0] = f01.x;
      rowbuf[l * 4 + 1] = f01.y;
      rowbuf[l * 4 + 2] = f23.x;
      rowbuf[l * 4 + 3] = f23.y;
    } else {
      __nv_bfloat16* rr = residual + (long)row * H + l * 4;
      const uint2 rv = *reinterpret_cast<const uint2*>(rr);
      float r[4] = {0.f, 0.f, 0.f, 0.f};
      acc_bf16x4(r, rv);
      const float2 f01 = __bfloat1622float2(y01), f23 = __bfloat1622float2(y23);
      __nv_bfloat162 n01 = __floats2bfloat162_rn(f01.x + r[0], f01.y + r[1]);
      __nv_bfloat162 n23 = __floats2bfloat162_rn(f23.x + r[2], f23.y + r[3]);
      uint2 o;
      o.x = *reinterpret_cast<uint32_t*>(&n01);
      o.y = *reinterpret_cast<uint32_t*>(&n23);
      *reinterpret_cast<uint2*>(rr) = o;
      const float2 g01 = __bfloat1622float2(n01), g23 = __bfloat1622float2(n23);
      rowbuf[l * 4 + 0] = g01.x;
      rowbuf[l * 4 + 1] = g01.y;
      rowbuf[l * 4 + 2] = g23.x;
      rowbuf[l * 4 + 3] = g23.y;
      ss += g01.x * g01.x + g01.y * g01.y + g23.x * g23.x + g23.y * g23.y;
    }
  }
  if (MODE == 1) {
    ss = block_sum(ss, red);
    const float inv = rsqrtf(ss / (float)H + eps);
    for (int l = tid; l < lines; l += blockDim.x) {
      const uint2 wv = *reinterpret_cast<const uint2*>(w + l * 4);
      float wf[4] = {0.f, 0.f, 0.f, 0.f};
      acc_bf16x4(wf, wv);
      __nv_bfloat162 o01 = __floats2bfloat162_rn(rowbuf[l * 4] * inv * (wf[0] + wbias),
                                                 rowbuf[l * 4 + 1] * inv * (wf[1] + wbias));
      __nv_bfloat162 o23 = __floats2bfloat162_rn(rowbuf[l * 4 + 2] * inv * (wf[2] + wbias),
                                                 rowbuf[l * 4 + 3] * inv * (wf[3] + wbias));
      uint2 o;
      o.x = *reinterpret_cast<uint32_t*>(&o01);
      o.y = *reinterpret_cast<uint32_t*>(&o23);
      *reinterpret_cast<uint2*>(out + (long)row * out_stride + l * 4) = o;
    }
  }
  if (MODE >= 2) {
    __syncthreads();
    row_epilogue<MODE>(rowbuf, row, epi, red);
  }
  __syncthreads();
  if (tid == 0) {
    if (s_timeout && a.status) atomicExch(a.status, (int)kErrPeerTimeout);
    if (gridDim.x == 1) {
      a.seq[0] = seq + 1;               // one row: nothing to count (the next collective is a later kernel)
    } else {
      const uint32_t done = atomicAdd(&a.seq[1], 1u);
      if (done == gridDim.x - 1) {
        a.seq[1] = 0;
        __threadfence();
        a.seq[0] = seq + 1;
      }
    }
  }
}

// (value, id) merge: grid 1, block = 32 * rows? -> one thread per (row) ; rows <= 16
__global__ void ll_argmax_merge_kernel(const CommArgs a, const int* __restrict__ idx, const float* __restrict__ val,
                                       int* __restrict__ out_idx, int rows) {
  const int row = threadIdx.x;
  const uint32_t seq = a.seq[0];
  const int stage = seq & (kLLStages - 1);
  __shared__ volatile int s_gave_up;
  if (threadIdx.x == 0) s_gave_up = (a.status && *reinterpret_cast<volatile int*>(a.status) != 0) ? 1 : 0;
  __syncthreads();
  bool timeout = false;
  if (row < rows) {
    const uint4 pkt = make_uint4(__float_as_uint(val[row]), seq, (uint32_t)idx[row], seq);
    const size_t slot_me = a.off_ll + ((size_t)(stage * a.size + a.rank) * kLLMaxRows + row) * a.ll_row_bytes;
    for (int i = 1; i < a.size; ++i) st_volatile_v4(a.peer[(a.rank + i) % a.size] + slot_me, pkt);
    float best = val[row];
    int bi = idx[row];
    for (int src = 0; src < a.size; ++src) {
      if (src == a.rank) continue;
      const size_t slot = a.off_ll + ((size_t)(stage * a.size + src) * kLLMaxRows + row) * a.ll_row_bytes;
      uint2 d;
      if (!ll_wait(a.peer[a.rank] + slot, seq, d, a.budget_ns, &s_gave_up)) {
        timeout = true;
        s_gave_up = 1;
        continue;
      }
      const float v = __uint_as_float(d.x);
      const int id = (int)d.y;
      if (v > best || (v == best && id < bi)) {
        best = v;
        bi = id;
      }
    }
    out_idx[row] = bi;
  }
  if (timeout && a.status) atomicExch(a.status, (int)kErrPeerTimeout);
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    a.seq[0] = seq + 1;
  }
}

// ------------------------------------------------------------------------------------------------
// Cross-rank barrier for CTA `cta` (same grid on every rank). tag must increase monotonically.
// ------------------------------------------------------------------------------------------------
// A barrier that ran out of time (in this launch or, through the status word, an earlier one) makes the later ones
// return at once.
VE_DEVINL bool rank_barrier(const CommArgs& a, int cta, uint32_t tag) {
  __shared__ int ok_s;
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) ok_s = (a.status && *reinterpret_cast<volatile int*>(a.status) != 0) ? 0 : 1;
  __syncthreads();
  if (!ok_s) return false;
  if (threadIdx.x < a.size) {
    const int peer = threadIdx.x;
    uint32_t* theirs = reinterpret_cast<uint32_t*>(a.peer[peer] + a.off_flags) + (size_t)cta * kMaxRanks + a.rank;
    st_release_sys(theirs, tag);
    const uint32_t* mine = reinterpret_cast<const uint32_t*>(a.peer[a.rank] + a.off_flags) + (size_t)cta * kMaxRanks + peer;
    const uint64_t t0 = globaltimer_ns();
    while ((int32_t)(ld_acquire_sys(mine) - tag) < 0) {
      if (globaltimer_ns() - t0 > a.budget_ns) {
        ok_s = 0;
        break;
      }
    }
  }
  __syncthreads();
  return ok_s != 0;
}

VE_DEVINL uint4 multimem_ld_reduce_bf16x8(const void* mc_addr) {
  uint4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(mc_addr)
               : "memory");
  return v;
}
VE_DEVINL void multimem_st_v4(void* mc_addr, uint4 v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(mc_addr), "r"(v.x), "r"(v.y),
               "r"(v.z), "r"(v.w)
               : "memory");
}

// Two-shot reduce-scatter + residual + RMSNorm + all-gather. The partial [T, H] sits at off_part of every
// rank's symmetric buffer; rank r owns rows [r*Tl, (r+1)*Tl). res_shard [Tl, H] is local. The normalised
// rows land at off_xout of every rank. block = H/8 threads (one 16 B vector each), H <= 8192.
template <int NVLS>
__global__ void __launch_bounds__(1024) rs_norm_ag_kernel(const CommArgs a, __nv_bfloat16* __restrict__ res_shard,
                                                          const __nv_bfloat16* __restrict__ w, int T, int Tl, int H,
                                                          float eps, float wbias, int mode) {
  __shared__ float red[33];
  const uint32_t seq = a.seq[2];
  const int tid = threadIdx.x;
  bool ok = rank_barrier(a, blockIdx.x, 2 * seq + 1);
  const int row0 = a.rank * Tl;
  const bool active = tid * 8 < H;
  for (int lr = blockIdx.x; lr < Tl; lr += gridDim.x) {
    const int row = row0 + lr;
    if (row >= T) break;
    const size_t off = ((size_t)row * H + tid * 8) * 2;
    float v[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] = 0.f;
    if (active) {
      if (NVLS) {
        const uint4 s = multimem_ld_reduce_bf16x8(a.mc + a.off_part + off);
        acc_bf16x4(v, make_uint2(s.x, s.y));
        acc_bf16x4(v + 4, make_uint2(s.z, s.w));
      } else {
        for (int src = 0; src < a.size; ++src) {
          const uint4 s = *reinterpret_cast<const uint4*>(a.peer[src] + a.off_part + off);
          acc_bf16x4(v, make_uint2(s.x, s.y));
          acc_bf16x4(v + 4, make_uint2(s.z, s.w));
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] = bf2f(f2bf(v[j]));  // round the reduced value to bf16 first
      }
    }
    float ss = 0.f;
    uint4 o = make_uint4(0, 0, 0, 0);
    if (mode == 1) {
      if (active) {
        __nv_bfloat16* rr = res_shard + (size_t)lr * H + tid * 8;
        const uint4 rv = *reinterpret_cast<const uint4*>(rr);
        float r[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        acc_bf16x4(r, make_uint2(rv.x, rv.y));
        acc_bf16x4(r + 4, make_uint2(rv.z, rv.w));
        uint32_t nr[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          __nv_bfloat162 t = __floats2bfloat162_rn(v[2 * j] + r[2 * j], v[2 * j + 1] + r[2 * j + 1]);
          nr[j] = *reinterpret_cast<uint32_t*>(&t);
          const float2 f = __bfloat1622float2(t);
          v[2 * j] = f.x;
          v[2 * j + 1] = f.y;
          ss += f.x * f.x + f.y * f.y;
        }
        *reinterpret_cast<uint4*>(rr) = make_uint4(nr[0], nr[1], nr[2], nr[3]);
      }
      ss = block_sum(ss, red);
      const float inv = rsqrtf(ss / (float)H + eps);
      if (active) {
        const uint4 wv = *reinterpret_cast<const uint4*>(w + tid * 8);
        float wf[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        acc_bf16x4(wf, make_uint2(wv.x, wv.y));
        acc_bf16x4(wf + 4, make_uint2(wv.z, wv.w));
        uint32_t* op = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
        for (int j = 0; j < 4; ++j)
          op[j] = pack2(v[2 * j] * inv * (wf[2 * j] + wbias), v[2 * j + 1] * inv * (wf[2 * j + 1] + wbias));
      }
    } else if (active) {
      uint32_t* op = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
      for (int j = 0; j < 4; ++j) op[j] = pack2(v[2 * j], v[2 * j + 1]);
    }
    if (active) {
      if (NVLS) {
        multimem_st_v4(a.mc + a.off_xout + off, o);
      } else {
        for (int i = 0; i < a.size; ++i) {
          const int peer = (a.rank + i) % a.size;
          *reinterpret_cast<uint4*>(a.peer[peer] + a.off_xout + off) = o;
        }
      }
    }
  }
  if (!ok && tid == 0 && a.status) atomicExch(a.status, (int)kErrPeerTimeout);   // before the second barrier: it then returns at once
  __syncthreads();
  ok = rank_barrier(a, blockIdx.x, 2 * seq + 2) && ok;
  if (tid == 0) {
    if (!ok && a.status) atomicExch(a.status, (int)kErrPeerTimeout);
    __threadfence();
    const uint32_t done = atomicAdd(&a.seq[3], 1u);
    if (done == gridDim.x - 1) {
      a.seq[3] = 0;
      __threadfence();
      a.seq[2] = seq + 1;
    }
  }
}

// Test hook for the timeout path: waits (bounded by budget_ns) on a flag that nothing sets, records the
// status and returns. The context stays usable.
__global__ void wait_flag_kernel(const uint32_t* flag, uint32_t want, unsigned long long budget_ns, int* status) {
  if (*reinterpret_cast<volatile int*>(status) != 0) return;      // an earlier wait already gave up: do not wait again
  const uint64_t t0 = globaltimer_ns();
  while (ld_acquire_sys(flag) != want) {
    if (globaltimer_ns() - t0 > budget_ns) {
      atomicExch(status, (int)kErrPeerTimeout);
      return;
    }
  }
}

}  // namespace ve

using namespace ve;

extern "C" {

// args: pointer to a host CommArgs-compatible blob (see parallel/symm.py for the packing).
int ve_ll_allreduce(const void* args, int mode, const void* partial, long part_stride, void* residual, const void* w,
                    void* out, long out_stride, int rows, int H, float eps, float wbias, cudaStream_t st) {
  const CommArgs& a = *reinterpret_cast<const CommArgs*>(args);
  if (rows <= 0) return 0;
  if (rows > kLLMaxRows || H % 4 || (size_t)(H / 4) * 16 > a.ll_row_bytes) return cudaErrorInvalidValue;
  int threads = ((H / 4 + 31) / 32) * 32;
  threads = threads > 1024 ? 1024 : threads;
  const int pushed = (mode >> 1) & 1;      // bit 1: the producer of ``partial`` already sent this rank's lines
  // programmatic launch: set-up overlaps the linear in front, and the decode linear behind starts streaming its weights
  // while this kernel still waits for the peers' lines
  if ((mode & 1) == 0)
    launch_pdl(ll_allreduce_kernel<0>, dim3(rows), dim3(threads), 0, st, a, (const __nv_bfloat16*)partial, part_stride,
               (__nv_bfloat16*)nullptr, (const __nv_bfloat16*)nullptr, (__nv_bfloat16*)out, out_stride, H, eps, wbias, pushed,
               EpiArgs{});
  else
    launch_pdl(ll_allreduce_kernel<1>, dim3(rows), dim3(threads), H * sizeof(float), st, a, (const __nv_bfloat16*)partial,
               part_stride, (__nv_bfloat16*)residual, (const __nv_bfloat16*)w, (__nv_bfloat16*)out, out_stride, H, eps, wbias,
               pushed, EpiArgs{});
  VE_CHECK_LAUNCH();
}

// All-reduce of <= 16 decode rows with one of the stream epilogues (mode 2 sandwich, 3 gated streams, 4 hyper-connection)
// applied to the reduced row in the same launch.
int ve_ll_allreduce_epi(const void* args, int mode, int pushed, const void* partial, long part_stride, void* xs,
                        void* res16, const void* post, const void* comb, const void* w, const void* w2,
                        const void* addend, const void* addend_gate, void* out, void* outf, int rows, int H, int hc, float eps,
                        float wbias, float scale, cudaStream_t st) {
  const CommArgs& a = *reinterpret_cast<const CommArgs*>(args);
  if (rows <= 0) return 0;
  if (rows > kLLMaxRows || H % 4 || (size_t)(H / 4) * 16 > a.ll_row_bytes) return cudaErrorInvalidValue;
  EpiArgs e;
  e.xs = (float*)xs; e.res16 = (__nv_bfloat16*)res16; e.post = (const float*)post; e.comb = (const float*)comb;
  e.w = (const __nv_bfloat16*)w; e.w2 = (const __nv_bfloat16*)w2; e.addend = (const __nv_bfloat16*)addend;
  e.addend_gate = (const float*)addend_gate; e.out = (__nv_bfloat16*)out; e.outf = (float*)outf;
  e.eps = eps; e.wbias = wbias; e.scale = scale; e.hc = hc; e.H = H;
  int threads = ((H / 4 + 31) / 32) * 32;
  threads = threads > 1024 ? 1024 : threads;
  const size_t smem = (size_t)H * sizeof(float);
#define VE_LLE(M)                                                                                                     \
  launch_pdl(ll_allreduce_kernel<M>, dim3(rows), dim3(threads), smem, st, a, (const __nv_bfloat16*)partial, part_stride, \
             (__nv_bfloat16*)nullptr, (const __nv_bfloat16*)nullptr, (__nv_bfloat16*)nullptr, (long)0, H, eps, wbias,    \
             pushed, e)
  switch (mode) {
    case kEpiSandwich:
      if ((!xs && !res16) || !w || !w2 || !out) return cudaErrorInvalidValue;
      VE_LLE(kEpiSandwich);
      break;
    case kEpiGated:
      if (!xs || !post || hc <= 0 || ((out || outf) && !w)) return cudaErrorInvalidValue;
      VE_LLE(kEpiGated);
      break;
    case kEpiHc:
      if (!xs || !post || !comb) return cudaErrorInvalidValue;
      VE_LLE(kEpiHc);
      break;
    default: return cudaErrorInvalidValue;
  }
#undef VE_LLE
  VE_CHECK_LAUNCH();
}

int ve_ll_argmax_merge(const void* args, const void* idx, const void* val, void* out_idx, int rows, cudaStream_t st) {
  const CommArgs& a = *reinterpret_cast<const CommArgs*>(args);
  if (rows <= 0) return 0;
  if (rows > kLLMaxRows) return cudaErrorInvalidValue;
  ll_argmax_merge_kernel<<<1, 32, 0, st>>>(a, (const int*)idx, (const float*)val, (int*)out_idx, rows);
  VE_CHECK_LAUNCH();
}

// mode 0: xout = sum ; mode 1: res_shard += bf16(sum), xout = RMSNorm(res_shard) * (w + wbias).
int ve_rs_norm_ag(const void* args, void* res_shard, const void* w, int T, int Tl, int H, float eps, float wbias,
                  int mode, int use_nvls, int ctas, cudaStream_t st) {
  const CommArgs& a = *reinterpret_cast<const CommArgs*>(args);
  if (T <= 0) return 0;
  if (H % 8 || H / 8 > 1024) return cudaErrorInvalidValue;
  if (use_nvls && !a.mc) return cudaErrorInvalidValue;
  const int threads = ((H / 8 + 31) / 32) * 32;
  if (use_nvls)
    rs_norm_ag_kernel<1><<<ctas, threads, 0, st>>>(a, (__nv_bfloat16*)res_shard, (const __nv_bfloat16*)w, T, Tl, H, eps,
                                                   wbias, mode);
  else
    rs_norm_ag_kernel<0><<<ctas, threads, 0, st>>>(a, (__nv_bfloat16*)res_shard, (const __nv_bfloat16*)w, T, Tl, H, eps,
                                                   wbias, mode);
  VE_CHECK_LAUNCH();
}

int ve_wait_flag(const void* flag, unsigned int want, unsigned long long budget_ns, void* status, cudaStream_t st) {
  wait_flag_kernel<<<1, 1, 0, st>>>((const uint32_t*)flag, want, budget_ns, (int*)status);
  VE_CHECK_LAUNCH();
}

int ve_comm_args_size() { return (int)sizeof(CommArgs); }

}  // extern "C"
