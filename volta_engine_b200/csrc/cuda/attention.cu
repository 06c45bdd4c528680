// Paged GQA attention for decode, speculative-verify blocks and chunked prefill in one kernel family.
//
// Semantics (reference: src/kernels/slang/ref_attention.slang:1-10,47-50,65-70 and
// inc/engine/modules/attention.h:40-57): causal softmax(q.k * scale) with a running fp32 maximum, optional
// sliding window counted back from the row position, optional per-row key_end for bidirectional image
// rows, optional sigmoid output gate. KV lives in a paged pool shared by all sequences:
//   K/V pool  [pages, kv_heads, 64 tokens, head_dim] bf16, page_table [slots, max_pages] int32.
//
// B200 design: a key tile is exactly one page, fetched by two (K, V) sets of TMA tiled loads into
// 128B-swizzled shared memory, double buffered on mbarriers; the G = q_heads / kv_heads query heads of a
// token share the CTA so K/V are read once per kv head. A query tile packs (token, head-in-group) pairs
// into 16-row MMA slabs (one per warp). Decode uses 1 warp per CTA and splits the key range over
// blockIdx.z with a grid that does not depend on the sequence position (CUDA-graph replay reads the
// positions from device memory); partial (o, lse) are merged by attn_reduce in split order.
// Tensor-core path here is mma.sync.m16n8k16 (bf16, fp32 accumulate).
#include "common.cuh"
#include "tmap.h"
#include <float.h>

namespace ve {

constexpr int kPageTok = 64;

struct AttnParams {
  const __nv_bfloat16* q;
  long q_stride;       // elements between rows of q
  __nv_bfloat16* out;  // [rows, nq*HD]
  long out_stride;
  const __nv_bfloat16* gate;  // optional [rows, nq*HD]
  long gate_stride;
  float* o_part;    // [rows, nq, nsplit, HD]
  float* lse_part;  // [rows, nq, nsplit]
  const int* pos;
  const int* slot;
  const int* key_end;     // optional
  const int* tile_first;  // optional (identity when null)
  const int* tile_count;
  const int* page_table;
  int max_pages;
  int nq, nkv, nsplit;
  float scale_log2;  // softmax scale * log2(e)
  int window;
  int* status;
  int nst;          // pipeline stages of the page loads (2 or 3)
  int early;               // 1: the prologue (descriptors, pages of earlier launches) runs ahead of the dependency wait
  const uint8_t* kscale;   // scaled cache formats: scale pools [pages, kv_heads, 64, scale bytes]
  const uint8_t* vscale;
  int* tickets;     // optional [tiles * nkv], zero between launches: the CTA that finishes a (tile, kv head) last merges
                    // the split partials itself (key-split kernel only), so no separate merge launch is needed
  // Tree verification (optional, per row): keys at cache positions >= tree_base[row] belong to the verify block, and
  // the row sees block key tree_base + j only when bit j of tree_mask[row] is set (its ancestors and itself); keys in
  // front of the block are seen as usual. Blocks hold at most 64 rows.
  const int* tree_base;
  const unsigned long long* tree_mask;
};

VE_DEVINL void ldsm_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}
VE_DEVINL void ldsm_x4_t(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}
VE_DEVINL void mma_bf16(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
VE_DEVINL uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 t = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&t);
}

VE_DEVINL uint32_t a_cvt_e2m1x2(uint32_t byte) {   // two E2M1 nibbles -> f16x2 (low nibble = first element)
  uint32_t r;
  asm("{ .reg .b8 t; cvt.u8.u32 t, %1; cvt.rn.f16x2.e2m1x2 %0, t; }" : "=r"(r) : "r"(byte));
  return r;
}
VE_DEVINL float a_e4m3(uint32_t b) {
  uint32_t r;
  asm("{ .reg .b16 t; cvt.u16.u32 t, %1; cvt.rn.f16x2.e4m3x2 %0, t; }" : "=r"(r) : "r"(b & 0xffu));
  return __half2float(__ushort_as_half((unsigned short)(r & 0xffffu)));
}
// 16 consecutive elements of one key, as bf16, to their place in the swizzled tile the tensor-core loads read
// (j = index of the 16-element group inside the row)
VE_DEVINL void put16(uint8_t* tile, int key, int j, const float* f) {
  uint32_t o[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) o[i] = pack_bf16(f[2 * i], f[2 * i + 1]);
  uint8_t* dst = tile + (j >> 2) * 8192 + key * 128;
  const int ch0 = (j & 3) * 2;
  *reinterpret_cast<uint4*>(dst + ((ch0 ^ (key & 7)) << 4)) = make_uint4(o[0], o[1], o[2], o[3]);
  *reinterpret_cast<uint4*>(dst + (((ch0 + 1) ^ (key & 7)) << 4)) = make_uint4(o[4], o[5], o[6], o[7]);
}

// KS (key-split, decode / verify tiles of <= 16 packed rows): all NW warps work on the same 16 rows and each takes
// its own 16-key slice of every 64-key page, so a page costs a quarter of the per-warp work; the warps' softmax
// states are merged through shared memory at the end.
// FMT: cache element format. 0 bf16 (pages land swizzled, ready for the tensor-core loads). 1 E5M2 bytes, 2 k8v4 (int8 keys
// and 4-bit Hadamard-rotated values with one fp16 scale per 64 elements), 3 nvfp4 (E2M1 with one E4M3 scale per 16):
// pages and their scales land in a staging buffer and the CTA expands them to bf16 tiles in the same layout, so the
// arithmetic is that of a bf16 cache whatever the storage (values of the rotated format are rotated back on the way).
template <int HD, int NW, bool KS, int FMT, bool TREE = false>
__global__ void __launch_bounds__(NW * 32) attn_kernel(const AttnParams p, const __grid_constant__ CUtensorMap kmap,
                                                       const __grid_constant__ CUtensorMap vmap) {
  // Everything up to grid_dep_wait() reads only what earlier steps left behind (row descriptors, page table, cache pages
  // that lie wholly before this launch's first row position), so it overlaps the kernels in front; the query rows and
  // the pages that hold this launch's own tokens are touched after the wait.
  grid_dep_launch();
  if (!p.early) grid_dep_wait();
  constexpr int TILE_BYTES = kPageTok * HD * 2;
  constexpr bool F8 = FMT != 0;       // staged formats
  constexpr int KB = FMT == 3 ? kPageTok * HD / 2 : kPageTok * HD;               // key bytes of one page
  constexpr int VB = FMT == 1 ? kPageTok * HD : kPageTok * HD / 2;               // value bytes of one page
  constexpr int SB = FMT == 2 ? kPageTok * (HD / 64) * 2 : (FMT == 3 ? kPageTok * (HD / 16) : 0);   // scale bytes (K, V alike)
  constexpr int STG = KB + VB + 2 * SB;                                          // one staging buffer
  constexpr int NCH = HD / 64;   // 128-byte column chunks per row
  constexpr int KSTEPS = HD / 16;
  constexpr int NT_O = HD / 8;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  __shared__ uint64_t full[3];
  const int nst = p.nst;

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int tile = blockIdx.x, kvh = blockIdx.y, z = blockIdx.z;
  const int G = p.nq / p.nkv;
  const int first = p.tile_first ? p.tile_first[tile] : tile;
  const int count = p.tile_count ? p.tile_count[tile] : 1;
  const int s = p.slot ? p.slot[first] : 0;
  if (count <= 0 || s < 0) return;

  // key range of the tile
  int lim_max = -1, pos_min = 0x7fffffff;
  for (int i = 0; i < count; ++i) {
    const int ps = p.pos[first + i];
    const int lm = p.key_end ? p.key_end[first + i] : ps;
    lim_max = max(lim_max, lm);
    pos_min = min(pos_min, ps);
  }
  const int kt_end_all = lim_max / kPageTok + 1;
  const int kt_begin_all = p.window > 0 ? max(0, pos_min - p.window + 1) / kPageTok : 0;
  const int ntile_all = kt_end_all - kt_begin_all;
  const int tps = (ntile_all + p.nsplit - 1) / p.nsplit;
  const int kt_begin = kt_begin_all + z * tps;
  const int kt_end = min(kt_end_all, kt_begin + tps);

  // this thread's two rows
  int r_tok[2], r_head[2], r_pos[2], r_lim[2], r_tb[2];
  unsigned long long r_tm[2];
  bool r_ok[2];
  constexpr bool tree = TREE;        // (a template parameter: the plain kernels keep their register count)
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int r = (KS ? 0 : warp * 16) + g + h * 8;
    r_ok[h] = r < count * G;
    const int rr = r_ok[h] ? r : 0;
    r_tok[h] = first + rr / G;
    r_head[h] = kvh * G + rr % G;
    r_pos[h] = p.pos[r_tok[h]];
    r_lim[h] = p.key_end ? p.key_end[r_tok[h]] : r_pos[h];
    r_tb[h] = tree ? p.tree_base[r_tok[h]] : 0x7fffffff;
    r_tm[h] = tree ? p.tree_mask[r_tok[h]] : ~0ull;
  }

  if (tid == 0) {
    mbar_init(&full[0], 1);
    mbar_init(&full[1], 1);
    mbar_init(&full[2], 1);
    mbar_fence_init();
  }
  __syncthreads();

  auto issue = [&](int kt, int stage) {
    const int page = p.page_table[(long)s * p.max_pages + kt];
    const int row = (page * p.nkv + kvh) * kPageTok;
    if (F8) {
      uint8_t* k8 = smem + stage * STG;
      mbar_expect_tx(&full[stage], STG);
      tma_load_2d(k8, &kmap, &full[stage], 0, row);
      tma_load_2d(k8 + KB, &vmap, &full[stage], 0, row);
      if (SB) {
        const size_t so = (size_t)(page * p.nkv + kvh) * SB;
        bulk_load(k8 + KB + VB, p.kscale + so, SB, &full[stage]);
        bulk_load(k8 + KB + VB + SB, p.vscale + so, SB, &full[stage]);
      }
      return;
    }
    uint8_t* kb = smem + stage * 2 * TILE_BYTES;
    uint8_t* vb = kb + TILE_BYTES;
    mbar_expect_tx(&full[stage], 2 * TILE_BYTES);
#pragma unroll
    for (int c = 0; c < NCH; ++c) {
      tma_load_2d(kb + c * 8192, &kmap, &full[stage], c * 64, row);
      tma_load_2d(vb + c * 8192, &vmap, &full[stage], c * 64, row);
    }
  };
  const int safe_end = pos_min / kPageTok;       // pages below hold tokens of earlier launches only
  int issued = 0;
  if (tid == 0)
    for (; issued < nst - 1 && kt_begin + issued < kt_end && kt_begin + issued < safe_end; ++issued)
      issue(kt_begin + issued, issued);
  grid_dep_wait();
  if (tid == 0)
    for (int i = issued; i < nst - 1 && kt_begin + i < kt_end; ++i) issue(kt_begin + i, i);

  // Q fragments straight from global memory
  uint32_t qf[KSTEPS][4];
#pragma unroll
  for (int kk = 0; kk < KSTEPS; ++kk) {
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const __nv_bfloat16* qr = p.q + (long)r_tok[h] * p.q_stride + (long)r_head[h] * HD + kk * 16 + 2 * t;
      qf[kk][h] = r_ok[h] ? *reinterpret_cast<const uint32_t*>(qr) : 0u;
      qf[kk][2 + h] = r_ok[h] ? *reinterpret_cast<const uint32_t*>(qr + 8) : 0u;
    }
  }

  float o[NT_O][4];
#pragma unroll
  for (int i = 0; i < NT_O; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m_run[2] = {-FLT_MAX, -FLT_MAX}, l_run[2] = {0.f, 0.f};

  const uint32_t smem_base = smem_u32(smem);
  bool failed = false;
  for (int kt = kt_begin; kt < kt_end; ++kt) {
    const int it = kt - kt_begin, stage = it % nst;
    const bool ok = mbar_wait(&full[stage], (it / nst) & 1);
    if (!__syncthreads_and(ok)) {
      failed = true;
      break;
    }
    // the stage of the previous iteration is free now (every warp passed the barrier above): refill it
    if (tid == 0 && kt + nst - 1 < kt_end) issue(kt + nst - 1, (it + nst - 1) % nst);
    if (F8) {
      // expand the page into the two bf16 tiles
      const uint8_t* st8 = smem + stage * STG;
      uint8_t* conv = smem + nst * STG;
      constexpr int G16 = HD / 16;                 // 16-element groups per key
      constexpr int CPT = kPageTok * G16;
      if (FMT == 1) {
        for (int idx = tid; idx < 2 * CPT; idx += NW * 32) {
          const int tile = idx / CPT, rem = idx % CPT;
          const int key = rem / G16, j = rem % G16;
          const uint4 raw = *reinterpret_cast<const uint4*>(st8 + tile * KB + key * HD + j * 16);
          const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
          float f[16];
#pragma unroll
          for (int q4 = 0; q4 < 4; ++q4) {
#pragma unroll
            for (int hh = 0; hh < 2; ++hh) {
              uint32_t h2;
              const unsigned short pair = (unsigned short)(w[q4] >> (16 * hh));
              asm("cvt.rn.f16x2.e5m2x2 %0, %1;" : "=r"(h2) : "h"(pair));
              const float2 v2 = __half22float2(*reinterpret_cast<const __half2*>(&h2));
              f[q4 * 4 + hh * 2] = v2.x;
              f[q4 * 4 + hh * 2 + 1] = v2.y;
            }
          }
          put16(conv + tile * TILE_BYTES, key, j, f);
        }
      } else if (FMT == 2) {
        const uint8_t* ksc = st8 + KB + VB;
        const uint8_t* vsc = ksc + SB;
        // keys: int8 x fp16 scale per 64
        for (int idx = tid; idx < CPT; idx += NW * 32) {
          const int key = idx / G16, j = idx % G16;
          const uint4 raw = *reinterpret_cast<const uint4*>(st8 + key * HD + j * 16);
          const float sc = __half2float(*reinterpret_cast<const __half*>(ksc + (key * (HD / 64) + (j >> 2)) * 2));
          const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
          float f[16];
#pragma unroll
          for (int i = 0; i < 16; ++i) f[i] = sc * (float)(int8_t)((w[i >> 2] >> (8 * (i & 3))) & 0xffu);
          put16(conv, key, j, f);
        }
        // values: 4-bit codes x fp16 scale per 64, rotated back by the 64-point Walsh-Hadamard transform
        for (int idx = tid; idx < kPageTok * (HD / 64); idx += NW * 32) {
          const int key = idx / (HD / 64), blk = idx % (HD / 64);
          const uint8_t* src = st8 + KB + key * (HD / 2) + blk * 32;
          const float sc = __half2float(*reinterpret_cast<const __half*>(vsc + (key * (HD / 64) + blk) * 2));
          float v[64];
#pragma unroll
          for (int q4 = 0; q4 < 2; ++q4) {
            const uint4 raw = *reinterpret_cast<const uint4*>(src + q4 * 16);
            const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              const uint32_t byte = (w[i >> 2] >> (8 * (i & 3))) & 0xffu;
              v[q4 * 32 + 2 * i] = sc * (float)((int)(byte & 15u) - 8);
              v[q4 * 32 + 2 * i + 1] = sc * (float)((int)(byte >> 4) - 8);
            }
          }
#pragma unroll
          for (int h = 1; h < 64; h <<= 1) {
#pragma unroll
            for (int i = 0; i < 64; ++i) {
              if ((i & h) == 0) {
                const float a = v[i], b = v[i | h];
                v[i] = a + b;
                v[i | h] = a - b;
              }
            }
          }
#pragma unroll
          for (int i = 0; i < 64; ++i) v[i] *= 0.125f;
#pragma unroll
          for (int q4 = 0; q4 < 4; ++q4) put16(conv + TILE_BYTES, key, blk * 4 + q4, v + q4 * 16);
        }
      } else {
        // E2M1 codes x E4M3 scale per 16, keys and values alike
        const uint8_t* sc0 = st8 + KB + VB;
        for (int idx = tid; idx < 2 * CPT; idx += NW * 32) {
          const int tile = idx / CPT, rem = idx % CPT;
          const int key = rem / G16, j = rem % G16;
          const uint2 raw = *reinterpret_cast<const uint2*>(st8 + tile * KB + key * (HD / 2) + j * 8);
          const float sc = a_e4m3(sc0[tile * SB + key * G16 + j]);
          const uint32_t w[2] = {raw.x, raw.y};
          float f[16];
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const uint32_t h2 = a_cvt_e2m1x2((w[i >> 2] >> (8 * (i & 3))) & 0xffu);
            const float2 v2 = __half22float2(*reinterpret_cast<const __half2*>(&h2));
            f[2 * i] = v2.x * sc;
            f[2 * i + 1] = v2.y * sc;
          }
          put16(conv + tile * TILE_BYTES, key, j, f);
        }
      }
      __syncthreads();
    }
    const uint32_t kb = F8 ? smem_base + nst * STG : smem_base + stage * 2 * TILE_BYTES, vb = kb + TILE_BYTES;

    // S = Q K^T  (16 rows x 64 keys per warp)
    constexpr int NP = KS ? 1 : 4;           // 16-key slices this warp scores per page
    const int key0 = KS ? warp * 16 : 0;     // first key of the warp's slice inside the page
    float sacc[2 * NP][4];
#pragma unroll
    for (int i = 0; i < 2 * NP; ++i) sacc[i][0] = sacc[i][1] = sacc[i][2] = sacc[i][3] = 0.f;
#pragma unroll
    for (int kk = 0; kk < KSTEPS; ++kk) {
      const int c = (kk * 16) / 64, ci = ((kk * 16) % 64) / 8;
#pragma unroll
      for (int np = 0; np < NP; ++np) {
        const int mi = lane >> 3, rr = lane & 7;
        const int key = key0 + np * 16 + (mi >> 1) * 8 + rr;
        const int ch = ci + (mi & 1);
        uint32_t b0, b1, b2, b3;
        ldsm_x4(kb + c * 8192 + key * 128 + ((ch ^ (key & 7)) << 4), b0, b1, b2, b3);
        mma_bf16(sacc[2 * np], qf[kk], b0, b1);
        mma_bf16(sacc[2 * np + 1], qf[kk], b2, b3);
      }
    }
    // mask + online softmax
    float mx[2] = {-FLT_MAX, -FLT_MAX};
#pragma unroll
    for (int nt = 0; nt < 2 * NP; ++nt) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int h = e >> 1;
        const int key = kt * kPageTok + key0 + nt * 8 + 2 * t + (e & 1);
        bool allow = r_ok[h] && key <= r_lim[h] && (p.window <= 0 || key > r_pos[h] - p.window);
        if (tree && key >= r_tb[h]) allow = allow && ((r_tm[h] >> ((key - r_tb[h]) & 63)) & 1ull) != 0ull;
        const float v = allow ? sacc[nt][e] * p.scale_log2 : -FLT_MAX;
        sacc[nt][e] = v;
        mx[h] = fmaxf(mx[h], v);
      }
    }
    float corr[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
      mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
      const float m_new = fmaxf(m_run[h], mx[h]);
      corr[h] = (m_run[h] == -FLT_MAX) ? 0.f : exp2f(m_run[h] - m_new);
      m_run[h] = m_new;
      l_run[h] *= corr[h];
    }
    uint32_t pf[NP][4];  // P as A fragments, one k-step of 16 keys per slice
#pragma unroll
    for (int nt = 0; nt < 2 * NP; ++nt) {
      float pv[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int h = e >> 1;
        pv[e] = (sacc[nt][e] == -FLT_MAX) ? 0.f : exp2f(sacc[nt][e] - m_run[h]);
        l_run[h] += pv[e];
      }
      const int ks = nt >> 1, hi = nt & 1;
      pf[ks][hi * 2 + 0] = pack_bf16(pv[0], pv[1]);
      pf[ks][hi * 2 + 1] = pack_bf16(pv[2], pv[3]);
    }
#pragma unroll
    for (int i = 0; i < NT_O; ++i) {
      o[i][0] *= corr[0];
      o[i][1] *= corr[0];
      o[i][2] *= corr[1];
      o[i][3] *= corr[1];
    }
    // O += P V
#pragma unroll
    for (int ks = 0; ks < NP; ++ks) {
#pragma unroll
      for (int dp = 0; dp < HD / 16; ++dp) {
        const int mi = lane >> 3, rr = lane & 7;
        const int key = key0 + ks * 16 + (mi & 1) * 8 + rr;
        const int d = dp * 16 + (mi >> 1) * 8;
        const int c = d / 64, ch = (d % 64) / 8;
        uint32_t b0, b1, b2, b3;
        ldsm_x4_t(vb + c * 8192 + key * 128 + ((ch ^ (key & 7)) << 4), b0, b1, b2, b3);
        mma_bf16(o[2 * dp], pf[ks], b0, b1);
        mma_bf16(o[2 * dp + 1], pf[ks], b2, b3);
      }
    }
  }
  if (failed) {
    if (tid == 0 && p.status) atomicExch(p.status, (int)kErrMbarTimeout);
    return;
  }

#pragma unroll
  for (int h = 0; h < 2; ++h) {
    l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 1);
    l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 2);
  }
  if (KS) {
    // merge the warps' (m, l, O) states; the page buffers are free now
    __syncthreads();
    float* ms = reinterpret_cast<float*>(smem);   // [NW][16]
    float* ls = ms + NW * 16;                       // [NW][16]
    float* os = ls + NW * 16;                       // [NW][16][HD]
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int row = g + h * 8;
      if (t == 0) { ms[warp * 16 + row] = m_run[h]; ls[warp * 16 + row] = l_run[h]; }
#pragma unroll
      for (int nt = 0; nt < NT_O; ++nt)
        *reinterpret_cast<float2*>(os + (size_t)(warp * 16 + row) * HD + nt * 8 + 2 * t) =
            make_float2(o[nt][2 * h], o[nt][2 * h + 1]);
    }
    __syncthreads();
    const int nrows = count * G;
    for (int idx = tid; idx < nrows * HD; idx += NW * 32) {
      const int row = idx / HD, d = idx % HD;
      float m = -FLT_MAX;
#pragma unroll
      for (int w = 0; w < NW; ++w) m = fmaxf(m, ms[w * 16 + row]);
      float acc = 0.f, l = 0.f;
#pragma unroll
      for (int w = 0; w < NW; ++w) {
        const float mw = ms[w * 16 + row];
        if (mw != -FLT_MAX) {
          const float c = exp2f(mw - m);
          acc += os[(size_t)(w * 16 + row) * HD + d] * c;
          l += ls[w * 16 + row] * c;
        }
      }
      const int tok = first + row / G, head = kvh * G + row % G;
      float v = l > 0.f ? acc / l : 0.f;
      if (p.nsplit == 1) {
        if (p.gate) v *= 1.f / (1.f + __expf(-bf2f(p.gate[(long)tok * p.gate_stride + (long)head * HD + d])));
        p.out[(long)tok * p.out_stride + (long)head * HD + d] = f2bf(v);
      } else {
        const long base = ((long)tok * p.nq + head) * p.nsplit + z;
        p.o_part[base * HD + d] = v;
        if (d == 0) p.lse_part[base] = l > 0.f ? m + log2f(l) : -FLT_MAX;
      }
    }
    if (p.nsplit > 1 && p.tickets) {
      __shared__ int s_last;
      __threadfence();
      __syncthreads();
      int* tk = p.tickets + (long)tile * p.nkv + kvh;
      if (tid == 0) s_last = atomicAdd(tk, 1) == p.nsplit - 1;
      __syncthreads();
      if (!s_last) return;
      __threadfence();
      // merge in split order (the same arithmetic as the stand-alone merge kernel)
      for (int idx = tid; idx < nrows * HD; idx += NW * 32) {
        const int row = idx / HD, d = idx % HD;
        const int tok = first + row / G, head = kvh * G + row % G;
        const long base = ((long)tok * p.nq + head) * p.nsplit;
        float mx = -FLT_MAX;
        for (int i = 0; i < p.nsplit; ++i) mx = fmaxf(mx, __ldcg(p.lse_part + base + i));
        float acc = 0.f, wsum = 0.f;
        for (int i = 0; i < p.nsplit; ++i) {
          const float l = __ldcg(p.lse_part + base + i);
          const float w = (l == -FLT_MAX) ? 0.f : exp2f(l - mx);
          wsum += w;
          acc += w * __ldcg(p.o_part + (base + i) * HD + d);
        }
        float v = wsum > 0.f ? acc / wsum : 0.f;
        if (p.gate) v *= 1.f / (1.f + __expf(-bf2f(p.gate[(long)tok * p.gate_stride + (long)head * HD + d])));
        p.out[(long)tok * p.out_stride + (long)head * HD + d] = f2bf(v);
      }
      if (tid == 0) *tk = 0;
    }
    return;
  }
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    if (!r_ok[h]) continue;
    const float inv = l_run[h] > 0.f ? 1.f / l_run[h] : 0.f;
    if (p.nsplit == 1) {
      __nv_bfloat16* orow = p.out + (long)r_tok[h] * p.out_stride + (long)r_head[h] * HD;
      const __nv_bfloat16* grow = p.gate ? p.gate + (long)r_tok[h] * p.gate_stride + (long)r_head[h] * HD : nullptr;
#pragma unroll
      for (int nt = 0; nt < NT_O; ++nt) {
        float a = o[nt][2 * h] * inv, b = o[nt][2 * h + 1] * inv;
        const int d = nt * 8 + 2 * t;
        if (grow) {
          a *= 1.f / (1.f + __expf(-bf2f(grow[d])));
          b *= 1.f / (1.f + __expf(-bf2f(grow[d + 1])));
        }
        *reinterpret_cast<uint32_t*>(orow + d) = pack_bf16(a, b);
      }
    } else {
      const long base = ((long)r_tok[h] * p.nq + r_head[h]) * p.nsplit + z;
      float* orow = p.o_part + base * HD;
#pragma unroll
      for (int nt = 0; nt < NT_O; ++nt) {
        const int d = nt * 8 + 2 * t;
        *reinterpret_cast<float2*>(orow + d) = make_float2(o[nt][2 * h] * inv, o[nt][2 * h + 1] * inv);
      }
      if (t == 0) p.lse_part[base] = l_run[h] > 0.f ? m_run[h] + log2f(l_run[h]) : -FLT_MAX;
    }
  }
}

// Merge split partials. grid (rows * nq), block (HD, kReduceGroups): the splits are dealt to kReduceGroups thread groups so
// that every load of a partial is in flight at once (one round trip for the log-sum-exps, one for the partial outputs)
// instead of one thread walking all splits; the groups' sums are combined through shared memory in group order, so the
// result does not depend on timing.
constexpr int kReduceGroups = 4;
constexpr int kReduceMaxSplit = 128;
__global__ void attn_reduce_kernel(const float* __restrict__ o_part, const float* __restrict__ lse_part,
                                   __nv_bfloat16* __restrict__ out, long out_stride,
                                   const __nv_bfloat16* __restrict__ gate, long gate_stride, const int* __restrict__ slot,
                                   int nq, int nsplit, int HD) {
  grid_dep_launch();
  grid_dep_wait();
  __shared__ float s_l[kReduceMaxSplit];
  __shared__ float s_acc[kReduceGroups][256];
  __shared__ float s_ws[kReduceGroups];
  const int row = blockIdx.x / nq, head = blockIdx.x % nq, d = threadIdx.x, sg = threadIdx.y;
  if (slot && slot[row] < 0) return;
  const long base = ((long)row * nq + head) * nsplit;
  const int tid = sg * HD + d;
  if (tid < nsplit) s_l[tid] = lse_part[base + tid];
  __syncthreads();
  float mx = -FLT_MAX;
  for (int i = 0; i < nsplit; ++i) mx = fmaxf(mx, s_l[i]);
  float acc = 0.f, wsum = 0.f;
#pragma unroll 8
  for (int i = sg; i < nsplit; i += kReduceGroups) {
    const float l = s_l[i];
    const float w = (l == -FLT_MAX) ? 0.f : exp2f(l - mx);
    wsum += w;
    acc += w * o_part[(base + i) * HD + d];
  }
  s_acc[sg][d] = acc;
  if (d == 0) s_ws[sg] = wsum;
  __syncthreads();
  if (sg != 0) return;
#pragma unroll
  for (int g = 1; g < kReduceGroups; ++g) {
    acc += s_acc[g][d];
    wsum += s_ws[g];
  }
  float v = wsum > 0.f ? acc / wsum : 0.f;
  if (gate) v *= 1.f / (1.f + __expf(-bf2f(gate[(long)row * gate_stride + (long)head * HD + d])));
  out[(long)row * out_stride + (long)head * HD + d] = f2bf(v);
}

}  // namespace ve
#include "attention_tc.cuh"
namespace ve {

template <int HD, int NW, bool KS, int FMT, bool TREE = false>
static int launch_attn(const AttnParams& p, const CUtensorMap& kmap, const CUtensorMap& vmap, int ntiles,
                       cudaStream_t st) {
  constexpr int TILE = kPageTok * HD * 2;
  constexpr int KB = FMT == 3 ? kPageTok * HD / 2 : kPageTok * HD, VB = FMT == 1 ? kPageTok * HD : kPageTok * HD / 2;
  constexpr int SB = FMT == 2 ? kPageTok * (HD / 64) * 2 : (FMT == 3 ? kPageTok * (HD / 16) : 0);
  const int smem = (FMT ? p.nst * (KB + VB + 2 * SB) + 2 * TILE : p.nst * 2 * TILE) + 1024;
  if (smem > 227 * 1024) return (int)cudaErrorInvalidValue;
  static int attr_smem = 0;
  if (smem > attr_smem) {
    cudaError_t e = cudaFuncSetAttribute(attn_kernel<HD, NW, KS, FMT, TREE>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return (int)e;
    attr_smem = smem;
  }
  dim3 grid(ntiles, p.nkv, p.nsplit);
  launch_pdl(attn_kernel<HD, NW, KS, FMT, TREE>, grid, dim3(NW * 32), smem, st, p, kmap, vmap);
  return (int)cudaGetLastError();
}

}  // namespace ve

using namespace ve;

extern "C" {

// warps: 1 (decode / verify: <= 16 packed rows per tile, one warp), 104 (same tiles, four warps that split the
// keys of every page), 4 (prefill: <= 64 packed rows, 16 per warp) or 8 (prefill on tcgen05: <= 128 packed rows per tile,
// bf16 cache, head_dim 128, one split).
int ve_attention(const void* q, long q_stride, void* out, long out_stride, const void* gate, long gate_stride,
                 void* o_part, void* lse_part, const void* pos, const void* slot, const void* key_end,
                 const void* tile_first, const void* tile_count, int ntiles, int rows, const void* page_table,
                 int max_pages, void* kpool, void* vpool, long pool_pages, int nq, int nkv, int hd, int nsplit,
                 float scale, int window, int warps, int kv_fp8, const void* kscale, const void* vscale, void* tickets,
                 const void* tree_base, const void* tree_mask, void* status, cudaStream_t st) {
  if (ntiles <= 0) return 0;
  if (nq % nkv || nsplit < 1 || nsplit > kReduceMaxSplit || kv_fp8 < 0 || kv_fp8 > 3) return cudaErrorInvalidValue;
  if (kv_fp8 >= 2 && ((hd != 128 && hd != 256) || warps == 1 || !kscale || !vscale)) return cudaErrorInvalidValue;
  AttnParams p;
  p.q = (const __nv_bfloat16*)q;
  p.q_stride = q_stride;
  p.out = (__nv_bfloat16*)out;
  p.out_stride = out_stride;
  p.gate = (const __nv_bfloat16*)gate;
  p.gate_stride = gate_stride;
  p.o_part = (float*)o_part;
  p.lse_part = (float*)lse_part;
  p.pos = (const int*)pos;
  p.slot = (const int*)slot;
  p.key_end = (const int*)key_end;
  p.tile_first = (const int*)tile_first;
  p.tile_count = (const int*)tile_count;
  p.page_table = (const int*)page_table;
  p.max_pages = max_pages;
  p.nq = nq;
  p.nkv = nkv;
  p.nsplit = nsplit;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.window = window;
  p.status = (int*)status;
  p.tickets = (warps == 104 && nsplit > 1) ? (int*)tickets : nullptr;
  {
    static int early = -1;
    if (early < 0) { const char* e = getenv("VOLTA_ATTN_EARLY"); early = (e && e[0] == '0') ? 0 : 1; }
    p.early = early;
  }
  p.kscale = (const uint8_t*)kscale;
  p.vscale = (const uint8_t*)vscale;
  p.tree_base = (const int*)tree_base;
  p.tree_mask = (const unsigned long long*)tree_mask;
  // tree rows: decode / verify tiles on a bf16 cache
  if ((tree_base != nullptr) != (tree_mask != nullptr) || (tree_base && (warps == 8 || warps == 4 || kv_fp8 != 0)))
    return cudaErrorInvalidValue;
  {
    static int stages = 0;      // VOLTA_ATTN_STAGES: page-load pipeline depth of the key-split decode kernel
    if (!stages) { const char* e = getenv("VOLTA_ATTN_STAGES"); stages = (e && e[0] == '2') ? 2 : 3; }   // 3: -8 % at 16K keys
    p.nst = (warps == 104 && hd <= 128) ? stages : 2;
  }
  if (warps == 8 && (hd != 128 || kv_fp8 != 0 || nsplit != 1 || ((uintptr_t)q & 15) || (q_stride & 7) ||
                     ((uintptr_t)out & 15) || (out_stride & 7) || ((uintptr_t)gate & 15) || (gate_stride & 7)))
    return cudaErrorInvalidValue;
  CUtensorMap kmap, vmap;
  const uint64_t total_rows = (uint64_t)pool_pages * nkv * kPageTok;
  int rc;
  if (kv_fp8) {   // byte caches: whole rows of the format's bytes per key, unswizzled staging tiles
    const int krow = kv_fp8 == 3 ? hd / 2 : hd, vrow = kv_fp8 == 1 ? hd : hd / 2;
    rc = make_tmap_2d(&kmap, kpool, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, total_rows, krow, (uint64_t)krow, kPageTok, krow,
                      CU_TENSOR_MAP_SWIZZLE_NONE);
    if (rc) return rc;
    rc = make_tmap_2d(&vmap, vpool, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, total_rows, vrow, (uint64_t)vrow, kPageTok, vrow,
                      CU_TENSOR_MAP_SWIZZLE_NONE);
  } else {
    rc = make_tmap_2d(&kmap, kpool, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, total_rows, hd, (uint64_t)hd * 2, kPageTok,
                      64, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc) return rc;
    rc = make_tmap_2d(&vmap, vpool, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, total_rows, hd, (uint64_t)hd * 2, kPageTok, 64,
                      CU_TENSOR_MAP_SWIZZLE_128B);
  }
  if (rc) return rc;
#define VE_ATTN2(HD_, F8_)                                                                  \
    rc = warps == 1     ? launch_attn<HD_, 1, false, F8_>(p, kmap, vmap, ntiles, st)        \
         : warps == 104 ? launch_attn<HD_, 4, true, F8_>(p, kmap, vmap, ntiles, st)         \
                        : launch_attn<HD_, 4, false, F8_>(p, kmap, vmap, ntiles, st);
#define VE_ATTNQ(HD_, F_)                                                                   \
    rc = warps == 104 ? launch_attn<HD_, 4, true, F_>(p, kmap, vmap, ntiles, st)            \
                      : launch_attn<HD_, 4, false, F_>(p, kmap, vmap, ntiles, st);
#define VE_ATTN(HD_)                                                             \
  if (hd == HD_) {                                                               \
    if (kv_fp8 == 1) { VE_ATTN2(HD_, 1) } else if (kv_fp8 == 0) { VE_ATTN2(HD_, 0) }            \
  } else
#define VE_ATTN_TREE(HD_)                                                                       \
    rc = warps == 1 ? launch_attn<HD_, 1, false, 0, true>(p, kmap, vmap, ntiles, st)            \
                    : launch_attn<HD_, 4, true, 0, true>(p, kmap, vmap, ntiles, st);
  if (tree_base) {
    if (hd == 64) { VE_ATTN_TREE(64) } else if (hd == 128) { VE_ATTN_TREE(128) } else if (hd == 256) { VE_ATTN_TREE(256) }
    else return cudaErrorInvalidValue;
  }
#undef VE_ATTN_TREE
  else if (warps == 8) { rc = launch_attn_tc<128>(p, kmap, vmap, ntiles, st); }
  else if (kv_fp8 == 2 && hd == 128) { VE_ATTNQ(128, 2) }
  else if (kv_fp8 == 2 && hd == 256) { VE_ATTNQ(256, 2) }
  else if (kv_fp8 == 3 && hd == 128) { VE_ATTNQ(128, 3) }
  else if (kv_fp8 == 3 && hd == 256) { VE_ATTNQ(256, 3) }
  else
  VE_ATTN(64) VE_ATTN(128) VE_ATTN(256) { return cudaErrorInvalidValue; }
#undef VE_ATTNQ
#undef VE_ATTN2
#undef VE_ATTN
  if (rc) return rc;
  if (nsplit > 1 && !p.tickets) {
  launch_pdl(attn_reduce_kernel, dim3(rows * nq), dim3(hd, kReduceGroups), 0, st, (const float*)o_part, (const float*)lse_part,
               (__nv_bfloat16*)out, out_stride, (const __nv_bfloat16*)gate, gate_stride, (const int*)slot, nq, nsplit, hd);
    rc = (int)cudaGetLastError();
  }
  return rc;
}

}  // extern "C"
