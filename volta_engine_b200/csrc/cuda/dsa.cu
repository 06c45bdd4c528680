// Sparse-attention indexer with pooled keys (lightning indexer): which tokens of a long context a latent-attention
// row attends to.
//   per token : k = LayerNorm(Wk x) (128), gate = Wg x (128), w = Ww x (32); plane ring [k_norm | gate] per position
//   per pool  : key[d] = sum_j softmax_j(gate_j[d] + ape[j][d]) * k_j[d] over the 4 tokens of the pool (built by the row
//               that completes it)
//   per query : score[p] = (128 * 32)^-1/2 * sum_h w[h] * relu(q[h] . key[p]) over the complete pools p < (pos + 1) / 4
//               -- a [32 x 128] x [128 x pools] product on mma.sync tiles, keys streamed straight from global memory
//   select    : the 512 best pools by score (ties at the threshold in pool order): 4-pass radix threshold, then an ordered
//               compaction; expanded to token indices plus the raw tokens of the incomplete tail pool. A row whose context
//               holds at most 512 complete pools lists every position (dense).
//   gather    : the listed tokens' latent cache rows copied into scratch pages, so the absorbed latent-attention kernel
//               runs over a short virtual sequence.
// Reference: inc/engine/modules/dsa.h:11-54, src/backend/cpu/dsa_ref.cpp (score, select order), src/backend/cuda/modules/dsa.cu.
#include "common.cuh"

namespace ve {

constexpr int kDsaHeads = 32, kDsaDim = 128, kDsaPool = 4, kDsaTopk = 2048, kDsaSel = kDsaTopk / kDsaPool;
constexpr int kDsaKpad = 2112;                 // list entries per row: 2048 selected + 3 tail, padded to whole 64-token pages
constexpr int kDsaProj = kDsaDim + kDsaHeads + kDsaDim;   // fused projection [k | w | gate]
constexpr int kDsaPlane = 2 * kDsaDim, kDsaPlaneCap = 1024;
constexpr int kPageTok = 64;                  // tokens per cache page

// grid rows, block 128. proj [rows, 288] bf16.
__global__ void __launch_bounds__(128) dsa_prep_kernel(const __nv_bfloat16* __restrict__ proj, const __nv_bfloat16* __restrict__ ln_w,
                                                       const __nv_bfloat16* __restrict__ ln_b, __nv_bfloat16* __restrict__ plane,
                                                       float* __restrict__ w_out, const int* __restrict__ slot,
                                                       const int* __restrict__ pos, long plane_slot_stride) {
  __shared__ float red[33];
  const int r = blockIdx.x, d = threadIdx.x;
  const int sl = slot[r], p = pos[r];
  if (sl < 0) return;
  const __nv_bfloat16* pr = proj + (long)r * kDsaProj;
  const float v = __bfloat162float(pr[d]);
  const float mean = block_sum(v, red) / (float)kDsaDim;
  const float dv = v - mean;
  const float var = block_sum(dv * dv, red) / (float)kDsaDim;
  const float kn = dv * rsqrtf(var + 1e-6f) * __bfloat162float(ln_w[d]) + __bfloat162float(ln_b[d]);
  __nv_bfloat16* dst = plane + (long)sl * plane_slot_stride + (long)(p & (kDsaPlaneCap - 1)) * kDsaPlane;
  dst[d] = __float2bfloat16_rn(kn);
  dst[kDsaDim + d] = pr[kDsaDim + kDsaHeads + d];
  if (d < kDsaHeads) w_out[(long)r * kDsaHeads + d] = __bfloat162float(pr[kDsaDim + d]);
}

// grid rows, block 128: the row at position p with p % 4 == 3 builds pool p / 4
__global__ void __launch_bounds__(128) dsa_pool_kernel(const __nv_bfloat16* __restrict__ plane, __nv_bfloat16* __restrict__ pool_plane,
                                                       const __nv_bfloat16* __restrict__ ape, const int* __restrict__ slot,
                                                       const int* __restrict__ pos, long plane_slot_stride,
                                                       long pool_slot_stride) {
  const int r = blockIdx.x, d = threadIdx.x;
  const int sl = slot[r], p = pos[r];
  if (sl < 0 || (p & (kDsaPool - 1)) != kDsaPool - 1) return;
  const __nv_bfloat16* base = plane + (long)sl * plane_slot_stride;
  float k[kDsaPool], g[kDsaPool], mx = -1e30f;
#pragma unroll
  for (int j = 0; j < kDsaPool; ++j) {
    const __nv_bfloat16* src = base + (long)((p - (kDsaPool - 1) + j) & (kDsaPlaneCap - 1)) * kDsaPlane;
    k[j] = __bfloat162float(src[d]);
    g[j] = __bfloat162float(src[kDsaDim + d]) + __bfloat162float(ape[j * kDsaDim + d]);
    mx = fmaxf(mx, g[j]);
  }
  float sum = 0.f, acc = 0.f;
#pragma unroll
  for (int j = 0; j < kDsaPool; ++j) {
    const float e = __expf(g[j] - mx);
    sum += e;
    acc = fmaf(e, k[j], acc);
  }
  pool_plane[(long)sl * pool_slot_stride + (long)(p / kDsaPool) * kDsaDim + d] = __float2bfloat16_rn(acc / sum);
}

VE_DEVINL void mma_bf16_16816(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// grid (ceil(max_pools / 64), rows), block 256: each warp scores 8 pools. q_idx [rows, HEADS, 128] bf16, w [rows, HEADS]
// fp32 head weights (nullptr: every head counts 1, the block-sparse indexer's form). HEADS = 32 or 4 (rows of the 16-row
// tile beyond HEADS are zero).
template <int HEADS>
__global__ void __launch_bounds__(256) dsa_score_kernel(const __nv_bfloat16* __restrict__ q_idx, const float* __restrict__ w,
                                                        const __nv_bfloat16* __restrict__ pool_plane, float* __restrict__ scores,
                                                        long score_stride, const int* __restrict__ slot,
                                                        const int* __restrict__ pos, long pool_slot_stride, int div) {
  constexpr int LDQ = kDsaDim + 8;
  constexpr int MT = (HEADS + 15) / 16, HP = MT * 16;
  __shared__ __align__(16) __nv_bfloat16 sq[HP * LDQ];
  __shared__ float sw[HP];
  const int r = blockIdx.y, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int sl = slot[r];
  if (sl < 0) return;
  const int bound = (pos[r] + 1) / div;   // div: tokens per key entry (4 for the pooled indexers)
  if (blockIdx.x * 64 >= bound) return;
  for (int i = tid; i < HP * kDsaDim; i += 256) {
    const int h = i / kDsaDim;
    sq[h * LDQ + (i % kDsaDim)] = h < HEADS ? q_idx[(long)r * HEADS * kDsaDim + i] : __float2bfloat16_rn(0.f);
  }
  if (tid < HP) sw[tid] = tid < HEADS ? (w ? w[(long)r * HEADS + tid] : 1.f) : 0.f;
  __syncthreads();
  const int p0 = (blockIdx.x * 8 + warp) * 8;
  if (p0 >= bound) return;
  const int g = lane >> 2, t = lane & 3;
  const int pn = min(p0 + g, bound - 1);
  const __nv_bfloat16* key = pool_plane + (long)sl * pool_slot_stride + (long)pn * kDsaDim;
  float acc[MT][4];
#pragma unroll
  for (int mt = 0; mt < MT; ++mt) acc[mt][0] = acc[mt][1] = acc[mt][2] = acc[mt][3] = 0.f;
#pragma unroll
  for (int kk = 0; kk < kDsaDim / 16; ++kk) {
    const uint32_t b0 = *reinterpret_cast<const uint32_t*>(key + kk * 16 + 2 * t);
    const uint32_t b1 = *reinterpret_cast<const uint32_t*>(key + kk * 16 + 2 * t + 8);
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
      uint32_t a[4];
      const __nv_bfloat16* q0 = sq + (mt * 16 + g) * LDQ + kk * 16 + 2 * t;
      a[0] = *reinterpret_cast<const uint32_t*>(q0);
      a[1] = *reinterpret_cast<const uint32_t*>(q0 + 8 * LDQ);
      a[2] = *reinterpret_cast<const uint32_t*>(q0 + 8);
      a[3] = *reinterpret_cast<const uint32_t*>(q0 + 8 * LDQ + 8);
      mma_bf16_16816(acc[mt], a, b0, b1);
    }
  }
  // relu, head weight, sum over the 32 heads (rows of the two tiles), per pool column
  float c0 = 0.f, c1 = 0.f;
#pragma unroll
  for (int mt = 0; mt < MT; ++mt) {
    const float wa = sw[mt * 16 + g], wb = sw[mt * 16 + g + 8];
    c0 += fmaxf(acc[mt][0], 0.f) * wa + fmaxf(acc[mt][2], 0.f) * wb;
    c1 += fmaxf(acc[mt][1], 0.f) * wa + fmaxf(acc[mt][3], 0.f) * wb;
  }
#pragma unroll
  for (int off = 4; off < 32; off <<= 1) {
    c0 += __shfl_xor_sync(0xffffffffu, c0, off);
    c1 += __shfl_xor_sync(0xffffffffu, c1, off);
  }
  if (g == 0) {
    const float norm = w ? rsqrtf((float)(kDsaDim * HEADS)) : rsqrtf((float)kDsaDim);
    float* out = scores + (long)r * score_stride + p0 + 2 * t;
    if (p0 + 2 * t < bound) out[0] = c0 * norm;
    if (p0 + 2 * t + 1 < bound) out[1] = c1 * norm;
  }
}

VE_DEVINL uint32_t score_key(float s) {
  const uint32_t b = __float_as_uint(s);
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

// grid rows, block 1024. idx [rows, kDsaKpad], nkeys [rows].
__global__ void __launch_bounds__(1024) dsa_select_kernel(const float* __restrict__ scores, long score_stride,
                                                          int* __restrict__ idx, int* __restrict__ nkeys,
                                                          const int* __restrict__ slot, const int* __restrict__ pos) {
  __shared__ int hist[256];
  __shared__ int sel[kDsaSel];
  __shared__ int wcnt[2][32], woff[2][32];
  __shared__ uint32_t s_prefix;
  __shared__ int s_need, s_base[2];
  const int r = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  int* out = idx + (long)r * kDsaKpad;
  if (slot[r] < 0) {
    if (tid == 0) nkeys[r] = 0;
    return;
  }
  const int vis = pos[r] + 1, bound = vis / kDsaPool;
  if (bound <= kDsaSel) {   // dense: every position
    for (int i = tid; i < vis; i += 1024) out[i] = i;
    if (tid == 0) nkeys[r] = vis;
    return;
  }
  const float* sc = scores + (long)r * score_stride;
  if (tid == 0) {
    s_prefix = 0;
    s_need = kDsaSel;
  }
  // radix threshold: the key of the K-th best pool
  for (int shift = 24; shift >= 0; shift -= 8) {
    if (tid < 256) hist[tid] = 0;
    __syncthreads();
    const uint32_t prefix = s_prefix;
    const uint32_t himask = shift == 24 ? 0u : (0xffffffffu << (shift + 8));
    for (int p = tid; p < bound; p += 1024) {
      const uint32_t k = score_key(sc[p]);
      if ((k & himask) == (prefix & himask)) atomicAdd(&hist[(k >> shift) & 255], 1);
    }
    __syncthreads();
    if (tid == 0) {
      int need = s_need, b = 255;
      for (; b > 0; --b) {
        if (hist[b] >= need) break;
        need -= hist[b];
      }
      s_prefix = prefix | ((uint32_t)b << shift);
      s_need = need;
    }
    __syncthreads();
  }
  const uint32_t thr = s_prefix;
  const int need_eq = s_need, total_gt = kDsaSel - need_eq;
  if (tid == 0) s_base[0] = s_base[1] = 0;
  __syncthreads();
  // ordered compaction: strictly better pools in pool order, then the needed threshold ties in pool order
  for (int c0 = 0; c0 < bound; c0 += 1024) {
    const int p = c0 + tid;
    const uint32_t k = p < bound ? score_key(sc[p]) : 0u;
    const bool gt = p < bound && k > thr, eq = p < bound && k == thr;
    const unsigned bg = __ballot_sync(0xffffffffu, gt), be = __ballot_sync(0xffffffffu, eq);
    const unsigned below = (1u << lane) - 1u;
    if (lane == 0) {
      wcnt[0][warp] = __popc(bg);
      wcnt[1][warp] = __popc(be);
    }
    __syncthreads();
    if (warp < 2) {
      const int v = wcnt[warp][lane];
      int inc = v;
#pragma unroll
      for (int off = 1; off < 32; off <<= 1) {
        const int n = __shfl_up_sync(0xffffffffu, inc, off);
        if (lane >= off) inc += n;
      }
      woff[warp][lane] = inc - v;
    }
    __syncthreads();
    if (gt) sel[s_base[0] + woff[0][warp] + __popc(bg & below)] = p;
    if (eq) {
      const int at = s_base[1] + woff[1][warp] + __popc(be & below);
      if (at < need_eq) sel[total_gt + at] = p;
    }
    __syncthreads();
    if (tid == 0) {
      s_base[0] += woff[0][31] + wcnt[0][31];
      s_base[1] += woff[1][31] + wcnt[1][31];
    }
    __syncthreads();
  }
  for (int i = tid; i < kDsaTopk; i += 1024) out[i] = sel[i / kDsaPool] * kDsaPool + (i % kDsaPool);
  const int tail = vis % kDsaPool;
  if (tid < tail) out[kDsaTopk + tid] = vis - tail + tid;
  if (tid == 0) nkeys[r] = kDsaTopk + tail;
}

// Copy the listed tokens' cache rows into scratch pages: pool [pages, nkv, 64, row_elems], scratch [rows * pages_per_row,
// nkv, 64, row_elems]; entry i of row r lands in page r * pages_per_row + i / 64, token i % 64.
// grid (kDsaKpad / 4, rows, nkv), block 256 (64 threads per entry).
__global__ void __launch_bounds__(256) dsa_gather_kernel(const __nv_bfloat16* __restrict__ pool, const int* __restrict__ page_table,
                                                         int max_pages, const int* __restrict__ slot, const int* __restrict__ idx,
                                                         const int* __restrict__ nkeys, __nv_bfloat16* __restrict__ scratch,
                                                         int pages_per_row, int row_elems, int nkv) {
  const int r = blockIdx.y, i = blockIdx.x * 4 + (threadIdx.x >> 6), l = threadIdx.x & 63, kvh = blockIdx.z;
  const int sl = slot[r];
  if (sl < 0 || i >= nkeys[r]) return;
  const int tok = idx[(long)r * kDsaKpad + i];
  const int page = page_table[(long)sl * max_pages + tok / kPageTok];
  const uint4* src = reinterpret_cast<const uint4*>(pool + (((long)page * nkv + kvh) * kPageTok + tok % kPageTok) * row_elems);
  uint4* dst = reinterpret_cast<uint4*>(
      scratch + ((((long)r * pages_per_row + i / kPageTok) * nkv + kvh) * kPageTok + i % kPageTok) * row_elems);
  for (int c = l; c < row_elems / 8; c += 64) dst[c] = src[c];
}

// ------------------------------------------------------------------------------------------------ block-sparse indexer
// Variant with 4 indexer heads and unweighted pools (reference: inc/engine/modules/qsa.h:8-33):
//   per token : [q (4 x 128) | k (128)] = W x; q = rmsnorm(q) * (1 + w_q), rotated on its first rot dims at the row's position;
//               the raw k enters a ring of the last 1024 positions
//   per pool  : key = rope_at_pool_start(rmsnorm(mean of the pool's 4 raw keys) * (1 + w_k))
//   per query : score[p] = 128^-1/2 * sum_h relu(q[h] . key[p])       (dsa_score_kernel<4> without head weights)
constexpr int kQsaHeads = 4, kQsaProj = (kQsaHeads + 1) * kDsaDim, kQsaRing = 1024;

VE_DEVINL void rope_pair(float& a, float& b, int i, int rot, float theta, int pos) {
  const float inv = exp2f(-log2f(theta) * (2.f * (float)i / (float)rot));
  float sn, cs;
  sincosf((float)pos * inv, &sn, &cs);
  const float x = a * cs - b * sn, y = b * cs + a * sn;
  a = x;
  b = y;
}

// grid (rows, 5): blockIdx.y < 4 a query head, 4 the key. block 128 (one thread per dim; NeoX pairs (i, i + rot/2)).
__global__ void __launch_bounds__(128) qsa_prep_kernel(const __nv_bfloat16* __restrict__ qk, const __nv_bfloat16* __restrict__ q_norm_w,
                                                       __nv_bfloat16* __restrict__ q_out, __nv_bfloat16* __restrict__ ring,
                                                       const int* __restrict__ slot, const int* __restrict__ pos,
                                                       long ring_slot_stride, int rot, float theta, float eps) {
  __shared__ float red[33];
  __shared__ float v[kDsaDim];
  const int r = blockIdx.x, part = blockIdx.y, d = threadIdx.x;
  const int sl = slot[r], p = pos[r];
  if (sl < 0) return;
  const __nv_bfloat16 raw = qk[(long)r * kQsaProj + part * kDsaDim + d];
  if (part == kQsaHeads) {
    ring[(long)sl * ring_slot_stride + (long)(p & (kQsaRing - 1)) * kDsaDim + d] = raw;
    return;
  }
  const float x = __bfloat162float(raw);
  const float ss = block_sum(x * x, red);
  v[d] = x * rsqrtf(ss / (float)kDsaDim + eps) * (1.f + __bfloat162float(q_norm_w[d]));
  __syncthreads();
  const int half = rot / 2;
  if (d < half) {
    float a = v[d], b = v[d + half];
    rope_pair(a, b, d, rot, theta, p);
    v[d] = a;
    v[d + half] = b;
  }
  __syncthreads();
  q_out[((long)r * kQsaHeads + part) * kDsaDim + d] = __float2bfloat16_rn(v[d]);
}

// grid rows, block 128: the row at position p with p % 4 == 3 builds pool p / 4
__global__ void __launch_bounds__(128) qsa_pool_kernel(const __nv_bfloat16* __restrict__ ring, __nv_bfloat16* __restrict__ pool_plane,
                                                       const __nv_bfloat16* __restrict__ k_norm_w, const int* __restrict__ slot,
                                                       const int* __restrict__ pos, long ring_slot_stride, long pool_slot_stride,
                                                       int rot, float theta, float eps) {
  __shared__ float red[33];
  __shared__ float v[kDsaDim];
  const int r = blockIdx.x, d = threadIdx.x;
  const int sl = slot[r], p = pos[r];
  if (sl < 0 || (p & (kDsaPool - 1)) != kDsaPool - 1) return;
  float m = 0.f;
#pragma unroll
  for (int j = 0; j < kDsaPool; ++j)
    m += __bfloat162float(ring[(long)sl * ring_slot_stride + (long)((p - (kDsaPool - 1) + j) & (kQsaRing - 1)) * kDsaDim + d]);
  m *= 1.f / (float)kDsaPool;
  const float ss = block_sum(m * m, red);
  v[d] = m * rsqrtf(ss / (float)kDsaDim + eps) * (1.f + __bfloat162float(k_norm_w[d]));
  __syncthreads();
  const int half = rot / 2;
  if (d < half) {
    float a = v[d], b = v[d + half];
    rope_pair(a, b, d, rot, theta, p - (kDsaPool - 1));
    v[d] = a;
    v[d + half] = b;
  }
  __syncthreads();
  pool_plane[(long)sl * pool_slot_stride + (long)(p / kDsaPool) * kDsaDim + d] = __float2bfloat16_rn(v[d]);
}

}  // namespace ve

using namespace ve;

extern "C" {

int ve_dsa_prep(const void* proj, const void* ln_w, const void* ln_b, void* plane, void* w_out, const void* slot,
                const void* pos, long plane_slot_stride, int rows, cudaStream_t st) {
  if (rows <= 0) return 0;
  dsa_prep_kernel<<<rows, 128, 0, st>>>((const __nv_bfloat16*)proj, (const __nv_bfloat16*)ln_w, (const __nv_bfloat16*)ln_b,
                                        (__nv_bfloat16*)plane, (float*)w_out, (const int*)slot, (const int*)pos,
                                        plane_slot_stride);
  VE_CHECK_LAUNCH();
}

int ve_dsa_pool_update(const void* plane, void* pool_plane, const void* ape, const void* slot, const void* pos,
                       long plane_slot_stride, long pool_slot_stride, int rows, cudaStream_t st) {
  if (rows <= 0) return 0;
  dsa_pool_kernel<<<rows, 128, 0, st>>>((const __nv_bfloat16*)plane, (__nv_bfloat16*)pool_plane, (const __nv_bfloat16*)ape,
                                        (const int*)slot, (const int*)pos, plane_slot_stride, pool_slot_stride);
  VE_CHECK_LAUNCH();
}

// heads = 32 with head weights w (pooled-key indexer) or 4 with w == nullptr (block-sparse indexer)
static int dsa_score_launch(const void* q_idx, const void* w, const void* pool_plane, void* scores, long score_stride,
                            const void* slot, const void* pos, long pool_slot_stride, int rows, int max_pools, int heads, int div,
                            cudaStream_t st);

int ve_dsa_score(const void* q_idx, const void* w, const void* pool_plane, void* scores, long score_stride, const void* slot,
                 const void* pos, long pool_slot_stride, int rows, int max_pools, int heads, cudaStream_t st) {
  return dsa_score_launch(q_idx, w, pool_plane, scores, score_stride, slot, pos, pool_slot_stride, rows, max_pools, heads,
                          kDsaPool, st);
}

// The same score with one key entry per `div` tokens (1, 2, ...): entries below (pos + 1) / div are scored.
int ve_dsa_score_div(const void* q_idx, const void* w, const void* pool_plane, void* scores, long score_stride, const void* slot,
                     const void* pos, long pool_slot_stride, int rows, int max_pools, int heads, int div, cudaStream_t st) {
  if (div < 1) return cudaErrorInvalidValue;
  return dsa_score_launch(q_idx, w, pool_plane, scores, score_stride, slot, pos, pool_slot_stride, rows, max_pools, heads, div, st);
}

static int dsa_score_launch(const void* q_idx, const void* w, const void* pool_plane, void* scores, long score_stride,
                            const void* slot, const void* pos, long pool_slot_stride, int rows, int max_pools, int heads, int div,
                            cudaStream_t st) {
  if (rows <= 0 || max_pools <= 0) return 0;
  const dim3 grid((max_pools + 63) / 64, rows);
  if (heads == kDsaHeads)
    dsa_score_kernel<kDsaHeads><<<grid, 256, 0, st>>>((const __nv_bfloat16*)q_idx, (const float*)w,
                                                      (const __nv_bfloat16*)pool_plane, (float*)scores, score_stride,
                                                      (const int*)slot, (const int*)pos, pool_slot_stride, div);
  else if (heads == kQsaHeads)
    dsa_score_kernel<kQsaHeads><<<grid, 256, 0, st>>>((const __nv_bfloat16*)q_idx, (const float*)w,
                                                      (const __nv_bfloat16*)pool_plane, (float*)scores, score_stride,
                                                      (const int*)slot, (const int*)pos, pool_slot_stride, div);
  else
    return cudaErrorInvalidValue;
  VE_CHECK_LAUNCH();
}

int ve_qsa_prep(const void* qk, const void* q_norm_w, void* q_out, void* ring, const void* slot, const void* pos,
                long ring_slot_stride, int rot, float theta, float eps, int rows, cudaStream_t st) {
  if (rows <= 0) return 0;
  if (rot % 2 || rot > kDsaDim) return cudaErrorInvalidValue;
  qsa_prep_kernel<<<dim3(rows, kQsaHeads + 1), 128, 0, st>>>((const __nv_bfloat16*)qk, (const __nv_bfloat16*)q_norm_w,
                                                             (__nv_bfloat16*)q_out, (__nv_bfloat16*)ring, (const int*)slot,
                                                             (const int*)pos, ring_slot_stride, rot, theta, eps);
  VE_CHECK_LAUNCH();
}

int ve_qsa_pool_update(const void* ring, void* pool_plane, const void* k_norm_w, const void* slot, const void* pos,
                       long ring_slot_stride, long pool_slot_stride, int rot, float theta, float eps, int rows,
                       cudaStream_t st) {
  if (rows <= 0) return 0;
  qsa_pool_kernel<<<rows, 128, 0, st>>>((const __nv_bfloat16*)ring, (__nv_bfloat16*)pool_plane, (const __nv_bfloat16*)k_norm_w,
                                        (const int*)slot, (const int*)pos, ring_slot_stride, pool_slot_stride, rot, theta, eps);
  VE_CHECK_LAUNCH();
}

int ve_dsa_select(const void* scores, long score_stride, void* idx, void* nkeys, const void* slot, const void* pos, int rows,
                  cudaStream_t st) {
  if (rows <= 0) return 0;
  dsa_select_kernel<<<rows, 1024, 0, st>>>((const float*)scores, score_stride, (int*)idx, (int*)nkeys, (const int*)slot,
                                           (const int*)pos);
  VE_CHECK_LAUNCH();
}

int ve_dsa_gather(const void* pool, const void* page_table, int max_pages, const void* slot, const void* idx,
                  const void* nkeys, void* scratch, int pages_per_row, int row_elems, int nkv, int rows, cudaStream_t st) {
  if (rows <= 0) return 0;
  if (row_elems % 8 || pages_per_row * kPageTok < kDsaKpad || nkv < 1) return cudaErrorInvalidValue;
  dsa_gather_kernel<<<dim3(kDsaKpad / 4, rows, nkv), 256, 0, st>>>((const __nv_bfloat16*)pool, (const int*)page_table,
                                                                   max_pages, (const int*)slot, (const int*)idx,
                                                                   (const int*)nkeys, (__nv_bfloat16*)scratch, pages_per_row,
                                                                   row_elems, nkv);
  VE_CHECK_LAUNCH();
}

int ve_dsa_kpad() { return kDsaKpad; }

}  // extern "C"
