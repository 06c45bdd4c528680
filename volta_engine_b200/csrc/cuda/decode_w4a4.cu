// Decode / verify-row linear on the block-scaled FP4 tensor-core path with bf16-grade activations:
//   out[m, n] = alpha * sum_k W[n, k] * x[m, k],   W in NVFP4, x in bf16, M <= 16 rows.
//
// The weights stream through TMA into swizzled shared memory in their packed checkpoint form and are decoded by
// the tensor core itself (tcgen05.mma kind::mxf4nvf4, E4M3 scale per 16), so no ALU or conversion work is spent
// per weight and many 16 KB tiles are in flight per SM. kind::mxf4nvf4 wants FP4 on both sides; each activation
// row is therefore expanded into TERMS residual NVFP4 rows
//   x ~= sum_t 8^-t * q_t,   q_t = nvfp4( 8^t * (x - sum_{u<t} 8^-u q_u) )
// (relative error 7e-4 at 3 terms, 5e-5 at 4: below bf16 rounding) that ride as extra MMA columns for free; the
// epilogue folds the TERMS columns of a row back together. The expansion is done inside the kernel by the warps
// that are idle during the main loop, straight into the swizzled B operand of each pipeline stage. Weights are
// the UMMA A operand (128 features = TMEM lanes per CTA), the expanded rows the B operand (BN = 16 / 32 / 64).
// Small layers do not fill 148 SMs with one CTA per 128 features, so K is split over gridDim.y CTAs; partial
// sums go to an fp32 workspace and the CTA that arrives last (per-tile ticket) adds them in split order, which
// keeps the result independent of timing. Every wait is bounded and reports through the status word.
// Reference kernels this replaces: src/kernels/cuda/nvfp4/skinny_kernels.cu:445-562 (decode GEMV on mma.sync
// fragments with in-register decode).
#include "common.cuh"
#include <cuda_fp8.h>
#include "tmap.h"
#include "nvfp4_expand.cuh"

namespace ve {

// Stand-alone form of the expansion (tests): x [M, K] bf16 (pitch ldx) -> Xp [M * TERMS, K/2] codes (virtual row
// m * TERMS + t) and scales in 512 B atoms [K/64][512] (atom byte (r%32)*16 + (r/32)*4 + j = scale of virtual row r,
// 16-block j of the 64-wide group).
template <int TERMS>
__global__ void nvfp4_expand_rows_kernel(const __nv_bfloat16* __restrict__ X, long ldx, uint8_t* __restrict__ Xp,
                                         uint8_t* __restrict__ Xs, int M, int K) {
  const int kb = K >> 4;
  const int total = M * kb;
  for (int idx = blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += gridDim.x * blockDim.x) {
    const int m = idx / kb, b = idx % kb;
    float r[16];
    uint2 codes[TERMS];
    uint32_t sc[TERMS];
    load16(X + (long)m * ldx + b * 16, r);
    expand_block16<TERMS>(r, codes, sc);
#pragma unroll
    for (int t = 0; t < TERMS; ++t) {
      const int v = m * TERMS + t;
      *reinterpret_cast<uint2*>(Xp + (long)v * (K >> 1) + b * 8) = codes[t];
      Xs[(long)(b >> 2) * 512 + (v & 31) * 16 + (v >> 5) * 4 + (b & 3)] = (uint8_t)sc[t];
    }
  }
}

struct DecodeParams {
  int N, M, K;
  float alpha;
  const __nv_bfloat16* x; long ldx;   // activations [M, K]
  __nv_bfloat16* out; long ldo;
  const __nv_bfloat16* residual; long ldr;
  float* out_f32;
  const uint8_t* sfa;     // [N/128][K/64][512]
  float* ws;              // [N/128][KS][16][128] partial sums (KS > 1)
  int* tickets;           // [N/128], zero between launches
  int* status;
  int tpt;                // epilogue threads that build one activation tile (16, 32, 64 or 128)
  int act;                // 0: plain output. 1 / 2: gated activation (SiLU / tanh-GELU): every 128-row weight tile holds
                          // 64 gate rows followed by their 64 up rows, the output has N/2 columns act(gate) * up
  float act_limit;        // > 0: gate clamped from above, up clamped to +-limit
  // Optional fused pre-norm (M <= 4): the input of the product is RMSNorm(resid + delta) * (w + wbias), computed by the
  // producer warps while the weights stream; CTAs of tile 0 also write the updated residual (resid + delta, bf16) to
  // resid_out (a different buffer than resid: other CTAs still read the old one). x is not read in this mode.
  const __nv_bfloat16* pn_w;
  const __nv_bfloat16* pn_resid;
  const __nv_bfloat16* pn_delta;      // may be null (plain RMSNorm of resid)
  __nv_bfloat16* pn_resid_out;        // may be null when delta is null
  float pn_eps, pn_wbias;
  // Optional fused all-reduce send (tensor parallel decode): the CTA that holds a tile's final sums also writes them,
  // as low-latency lines {data, seq, data, seq}, into this rank's slot of every peer's staging area, so the
  // all-reduce kernel behind only has to wait, add and normalise. Null peers[0]: off.
  uint8_t* ll_peer[8];
  const uint32_t* ll_seq;
  int ll_rank, ll_size;
  size_t ll_off, ll_row_bytes;
  // Optional fused residual add + RMSNorm behind the product (one GPU, decode rows): every tile's final writer counts on a
  // launch-wide ticket; the CTA that arrives last reads the finished rows back, adds them to the residual stream (in place,
  // rounded to bf16 like the stand-alone kernel), and writes RMSNorm(residual) * (w + wbias) -- the next block's input --
  // so the norm costs no launch of its own. an_out null: off.
  // Optional fused rotary embedding + KV store (a stacked q | k | v projection with head_dim 128, so one weight tile is one
  // head): the tile's final writer rotates its q or k head at the row positions (NeoX pairs, partial rotary allowed) and
  // writes k / v rows straight into the paged cache (bf16 or E5M2), the same arithmetic and bits as the stand-alone
  // rotation kernel run on the rounded product. rp_pos null: off.
  const int* rp_pos;
  const int* rp_slot;
  const int* rp_table;
  int rp_max_pages;
  void* rp_kpool;
  void* rp_vpool;
  int rp_nq, rp_nkv, rp_rot, rp_fp8;
  float rp_theta;
  // Optional L2 prefetch for the kernel behind: while this kernel streams its own weights (marked evict-first), every CTA
  // asks for its share of [pf_ptr, pf_ptr + pf_bytes), the weights the next linear of the step will read, so that
  // kernel finds them in L2 instead of paying HBM latency at its start. pf_ptr null: off.
  const uint8_t* pf_ptr;
  size_t pf_bytes;
  const uint8_t* pf_ptr2;             // second range (the scale atoms)
  size_t pf_bytes2;
  int* an_ticket;
  __nv_bfloat16* an_resid;            // [M, N], pitch N
  const __nv_bfloat16* an_w;          // [N]
  __nv_bfloat16* an_out;              // [M, N], pitch N
  float an_eps, an_wbias;
};

// Warp roles (192 threads): warp 0 = TMA producer of weight tiles and their scale atoms; warp 1 = TMEM owner and
// MMA issuer; warps 2..5 = activation producers during the main loop (expand x into the B operand of each stage,
// straight into swizzled shared memory) and epilogue afterwards.
template <int BN, int TERMS, int STAGES>
__global__ void __launch_bounds__(192, 2)
decode_w4a4_kernel(const DecodeParams p, const __grid_constant__ CUtensorMap amap) {
  constexpr int A_BYTES = 128 * 128, B_BYTES = BN * 128, SF_BYTES = 2048;
  constexpr int STAGE_BYTES = A_BYTES + B_BYTES + 2 * SF_BYTES;
  constexpr int ACC_COLS = BN < 32 ? 32 : BN;
  constexpr int TMEM_COLS = ACC_COLS + 64 <= 64 ? 64 : 128;      // accumulator + two sets of scale columns
  constexpr int MROWS = BN / TERMS;
  static_assert(STAGE_BYTES % 1024 == 0, "stage must keep 1024 B alignment");

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  __shared__ uint64_t full[STAGES], empty[STAGES], acc_full;
  __shared__ uint32_t tmem_holder;
  __shared__ int s_fail, s_ticket;
  __shared__ float s_red[4];

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tile = blockIdx.x, n0 = tile * 128;
  const int KS = gridDim.y, ks = blockIdx.y;
  const int nkt_all = (p.K + 255) >> 8;           // a K that is a multiple of 128 only ends in a half tile (zero filled)
  const int kt0 = (int)((long)ks * nkt_all / KS), kt1 = (int)((long)(ks + 1) * nkt_all / KS);
  const int nkt = kt1 - kt0;
  const int nkg = nkt_all * 4;                    // scale atoms along K, padded to whole k-tiles
  const int tpt = p.tpt;

  auto stage_ptr = [&](int s) { return smem + (size_t)s * STAGE_BYTES; };   // [A][B][SFA][SFB]
  grid_dep_launch();                              // the kernel behind this one may be scheduled now
  if (threadIdx.x == 0) {
    // a stage is full after the TMA bytes (one arrive.expect_tx) and the tpt activation writers have arrived
    for (int s = 0; s < STAGES; ++s) { mbar_init(&full[s], 1 + tpt); mbar_init(&empty[s], 1); }
    mbar_init(&acc_full, 1);
    s_fail = 0;
    mbar_fence_init();
  }
  if (warp == 1) { tmem_alloc(&tmem_holder, TMEM_COLS); tmem_relinquish(); }
  if (warp >= 2) {
    // scales of the unused columns stay zero (their accumulator columns are never read)
    const int etid = threadIdx.x - 64;
    for (int s = 0; s < STAGES; ++s)
      *reinterpret_cast<uint4*>(stage_ptr(s) + A_BYTES + B_BYTES + SF_BYTES + etid * 16) = make_uint4(0, 0, 0, 0);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_holder;

  if (warp == 0) {
    if (elect_one()) {
      prefetch_tmap(&amap);
      const uint64_t pol = l2_policy_evict_first();
      // weights do not depend on the kernel in front: with a programmatic dependent launch they start streaming
      // while that kernel is still running
      for (int i = 0; i < nkt; ++i) {
        const int s = i % STAGES, kt = kt0 + i;
        if (!mbar_wait(&empty[s], ((i / STAGES) & 1) ^ 1)) { atomicExch(&s_fail, 1); break; }
        uint8_t* st = stage_ptr(s);
        mbar_expect_tx(&full[s], A_BYTES + SF_BYTES);
        tma_load_2d_hint(st, &amap, &full[s], kt * 128, n0, pol);
        if (p.pf_ptr && i == (nkt > STAGES ? STAGES : nkt - 1)) {
          // own pipeline is full: now ask for this CTA's share of the next kernel's weights (chunks of <= 64 KB)
          const size_t ctas = (size_t)gridDim.x * gridDim.y, me = (size_t)blockIdx.y * gridDim.x + blockIdx.x;
          for (int r = 0; r < 2; ++r) {
            const uint8_t* base = r ? p.pf_ptr2 : p.pf_ptr;
            const size_t total = r ? p.pf_bytes2 : p.pf_bytes;
            if (!base || !total) continue;
            const size_t per = ((total + ctas - 1) / ctas + 15) & ~(size_t)15;
            size_t lo = me * per;
            const size_t hi = lo + per < total ? lo + per : total;
            while (lo < hi) {
              const size_t n = hi - lo < 65536 ? (hi - lo) & ~(size_t)15 : 65536;
              if (!n) break;
              l2_prefetch(base + lo, (uint32_t)n);
              lo += n;
            }
          }
        }
        bulk_load(st + A_BYTES + B_BYTES, p.sfa + ((size_t)tile * nkg + kt * 4) * 512, SF_BYTES, &full[s]);
      }
    }
  } else if (warp == 1) {
    if (elect_one()) {
      constexpr uint32_t idesc = make_idesc_nvf4(128, BN);
      bool ok = true;
      for (int i = 0; i < nkt && ok; ++i) {
        const int s = i % STAGES;
        // the scale columns alternate between two sets: the copies of k-tile i + 1 then do not have to wait until the
        // MMAs of k-tile i have read theirs (a write-after-read chain through TMEM otherwise serialises the tiles)
        const uint32_t tmem_sfa = tmem_base + ACC_COLS + (i & 1) * 32, tmem_sfb = tmem_sfa + 16;
        ok = mbar_wait(&full[s], (i / STAGES) & 1);
        if (!ok) break;
        tc_fence_after();
        uint8_t* st = stage_ptr(s);
        const uint32_t sfa_s = smem_u32(st + A_BYTES + B_BYTES), sfb_s = sfa_s + SF_BYTES;
#pragma unroll
        for (int kb = 0; kb < 4; ++kb) {
          tc_cp_sf(tmem_sfa + kb * 4, make_desc_sf(sfa_s + kb * 512));
          tc_cp_sf(tmem_sfb + kb * 4, make_desc_sf(sfb_s + kb * 512));
        }
        const uint64_t ad = make_desc_sw128(smem_u32(st)), bd = make_desc_sw128(smem_u32(st + A_BYTES));
#pragma unroll
        for (int kb = 0; kb < 4; ++kb)
          tc_mma_nvf4(tmem_base, ad + kb * 2, bd + kb * 2, idesc, (i | kb) ? 1u : 0u, tmem_sfa + kb * 4, tmem_sfb + kb * 4);
        tc_commit(&empty[s]);
      }
      if (!ok) atomicExch(&s_fail, 1);
      tc_commit(&acc_full);
    }
  } else {
    const int etid = threadIdx.x - 64;           // 0..127
    grid_dep_wait();                             // x, residual and out belong to upstream kernels
    // ---- activation producer: groups of tpt threads own k-tiles g, g + ngroups, ...; inside a tile the 16 * M
    // blocks (row m, 16-block b) are dealt round-robin to the group's threads
    {
      // At most STAGES groups, and a count that divides STAGES: every stage is then always filled by the same
      // group, which meets the stage's phases in order (a parity wait cannot tell phases two apart).
      int ngroups = 128 / tpt;
      if (ngroups > STAGES) ngroups = STAGES;
      while (STAGES % ngroups) --ngroups;
      const int grp = etid / tpt, gt = etid % tpt;
      const int items = 16 * p.M;
      bool ok = true;
      float rs[4] = {0.f, 0.f, 0.f, 0.f};
      if (p.pn_w) {
        // row statistics over the whole row (every CTA needs them; 128 threads, fixed summation order)
        __shared__ float s_red[4][4];
        for (int m = 0; m < p.M; ++m) {
          float ss = 0.f;
          for (int i = etid * 16; i < p.K; i += 128 * 16) {
            float v[16], d[16];
            load16(p.pn_resid + (long)m * p.K + i, v);
            if (p.pn_delta) {
              load16(p.pn_delta + (long)m * p.K + i, d);
#pragma unroll
              for (int j = 0; j < 16; ++j) v[j] = round_bf16(v[j] + d[j]);
            }
#pragma unroll
            for (int j = 0; j < 16; ++j) ss = fmaf(v[j], v[j], ss);
          }
          ss = warp_sum(ss);
          if (lane == 0) s_red[warp - 2][m] = ss;
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
        for (int m = 0; m < p.M; ++m)
          rs[m] = rsqrtf((s_red[0][m] + s_red[1][m] + s_red[2][m] + s_red[3][m]) / (float)p.K + p.pn_eps);
      }
      for (int i = grp; i < nkt && ok && grp < ngroups; i += ngroups) {
        const int s = i % STAGES, kt = kt0 + i;
        ok = mbar_wait(&empty[s], ((i / STAGES) & 1) ^ 1);
        if (!ok) break;
        uint8_t* bt = stage_ptr(s) + A_BYTES;
        uint8_t* sf = bt + B_BYTES + SF_BYTES;
        for (int it = gt; it < items; it += tpt) {
          const int m = it >> 4, b = it & 15;
          uint2 codes[TERMS];
          uint32_t sc[TERMS];
          float r16[16];
          const int k0 = kt * 256 + b * 16;
          if (p.pn_w) {
            float d[16], w16[16];
            load16(p.pn_resid + (long)m * p.K + k0, r16);
            if (p.pn_delta) {
              load16(p.pn_delta + (long)m * p.K + k0, d);
#pragma unroll
              for (int j = 0; j < 16; ++j) r16[j] = round_bf16(r16[j] + d[j]);
              if (tile == 0 && p.pn_resid_out) {
                bf16x8 o0, o1;
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                  o0.v[j] = __floats2bfloat162_rn(r16[2 * j], r16[2 * j + 1]);
                  o1.v[j] = __floats2bfloat162_rn(r16[8 + 2 * j], r16[8 + 2 * j + 1]);
                }
                *reinterpret_cast<bf16x8*>(p.pn_resid_out + (long)m * p.K + k0) = o0;
                *reinterpret_cast<bf16x8*>(p.pn_resid_out + (long)m * p.K + k0 + 8) = o1;
              }
            }
            load16(p.pn_w + k0, w16);
            const float rm = m == 0 ? rs[0] : m == 1 ? rs[1] : m == 2 ? rs[2] : rs[3];
#pragma unroll
            for (int j = 0; j < 16; ++j) r16[j] = round_bf16(r16[j] * rm * (w16[j] + p.pn_wbias));
          } else if (k0 < p.K) {
            load16(p.x + (long)m * p.ldx + k0, r16);
          } else {
#pragma unroll
            for (int j = 0; j < 16; ++j) r16[j] = 0.f;   // beyond K: the half tile's weights are zero as well
          }
          expand_block16<TERMS>(r16, codes, sc);
#pragma unroll
          for (int t = 0; t < TERMS; ++t) {
            const int v = m * TERMS + t;
            *reinterpret_cast<uint2*>(bt + v * 128 + ((((b >> 1) ^ (v & 7))) << 4) + (b & 1) * 8) = codes[t];
            sf[(b >> 2) * 512 + (v & 31) * 16 + (v >> 5) * 4 + (b & 3)] = (uint8_t)sc[t];
          }
        }
        fence_proxy_async_smem();
        mbar_arrive(&full[s]);
      }
      if (!ok) atomicExch(&s_fail, 1);
    }
    // ---- epilogue: TMEM lane = output feature, column m * TERMS + t = term t of row m
    const int q = warp & 3;                      // TMEM lane quarter this warp may touch
    const int f = q * 32 + lane;                 // feature inside the tile
    const int n = n0 + f;
    const bool ok = nkt > 0 ? mbar_wait(&acc_full, 0) : true;
    if (!ok) atomicExch(&s_fail, 1);
    tc_fence_after();
    float acc[MROWS];
#pragma unroll
    for (int m = 0; m < MROWS; ++m) acc[m] = 0.f;
    if (ok && !s_fail && nkt > 0) {
#pragma unroll
      for (int c0 = 0; c0 < BN; c0 += 16) {
        uint32_t r[16];
        tmem_ld16(tmem_base + ((uint32_t)(q * 32) << 16) + c0, r);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 16; j += TERMS) {
          float v = 0.f, c = 1.f;
#pragma unroll
          for (int t = 0; t < TERMS; ++t) { v = fmaf(__uint_as_float(r[j + t]), c, v); c *= 0.125f; }
          acc[(c0 + j) / TERMS] = v;
        }
      }
    }
    bool write = true;
    if (KS > 1) {
      float* mine = p.ws + ((size_t)tile * KS + ks) * 16 * 128;
#pragma unroll
      for (int m = 0; m < MROWS; ++m)
        if (m < p.M) mine[m * 128 + f] = acc[m];
      __threadfence();
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (etid == 0) s_ticket = atomicAdd(p.tickets + tile, 1);
      asm volatile("bar.sync 1, 128;" ::: "memory");
      write = s_ticket == KS - 1;
      if (write) {
        __threadfence();
        const float* all = p.ws + (size_t)tile * KS * 16 * 128;
#pragma unroll
        for (int m = 0; m < MROWS; ++m) {
          if (m < p.M) {
            float s = 0.f;
            for (int k2 = 0; k2 < KS; ++k2) s += __ldcg(all + ((size_t)k2 * 16 + m) * 128 + f);
            acc[m] = s;
          }
        }
        if (etid == 0) p.tickets[tile] = 0;      // ready for the next launch
      }
    }
    if (p.act) {
      // gate and up of one feature sit in lanes f and f + 64 of the tile: meet through shared memory (the pipeline
      // stages are idle by now)
      float* sb = reinterpret_cast<float*>(smem);
      if (write) {
#pragma unroll
        for (int m = 0; m < MROWS; ++m)
          if (m < p.M) sb[m * 128 + f] = acc[m] * p.alpha;
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (write && f < 64 && !s_fail) {
        const int col = tile * 64 + f;
#pragma unroll
        for (int m = 0; m < MROWS; ++m) {
          if (m < p.M) {
            float g = sb[m * 128 + f], u = sb[m * 128 + 64 + f];
            if (p.act_limit > 0.f) { g = fminf(g, p.act_limit); u = fminf(fmaxf(u, -p.act_limit), p.act_limit); }
            const float a = p.act == 1 ? g / (1.f + __expf(-g))
                                       : 0.5f * g * (1.f + tanhf(0.7978845608028654f * (g + 0.044715f * g * g * g)));
            p.out[(long)m * p.ldo + col] = f2bf(a * u);
          }
        }
      }
    } else if (p.rp_pos) {
      // one tile = one head: stage the rounded product, then 64 threads rotate / store the pairs of every row
      float* sb = reinterpret_cast<float*>(smem);
      if (write) {
#pragma unroll
        for (int m = 0; m < MROWS; ++m)
          if (m < p.M) sb[m * 128 + f] = bf2f(f2bf(acc[m] * p.alpha));
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (write && f < 64 && !s_fail) {
        const int head = tile, half = p.rp_rot >> 1;
        const bool is_v = head >= p.rp_nq + p.rp_nkv, is_k = !is_v && head >= p.rp_nq;
        int i0, i1;
        if (is_v) { i0 = 2 * f; i1 = i0 + 1; }
        else if (f < half) { i0 = f; i1 = f + half; }
        else { i0 = p.rp_rot + 2 * (f - half); i1 = i0 + 1; }
        const float inv_freq = exp2f(-log2f(p.rp_theta) * (2.f * (float)f / (float)p.rp_rot));
#pragma unroll
        for (int m = 0; m < MROWS; ++m) {
          if (m < p.M) {
            float a0 = sb[m * 128 + i0], a1 = sb[m * 128 + i1];
            const int ps = p.rp_pos[m];
            const int sl = p.rp_slot ? p.rp_slot[m] : 0;
            if (!is_v && f < half && !(is_k && sl < 0)) {      // padding rows keep their key unrotated, like the rotation kernel
              float sn, cs;
              sincosf((float)ps * inv_freq, &sn, &cs);
              const float r0 = a0 * cs - a1 * sn, r1 = a1 * cs + a0 * sn;
              a0 = r0;
              a1 = r1;
            }
            const __nv_bfloat16 b0 = f2bf(a0), b1 = f2bf(a1);
            p.out[(long)m * p.ldo + n0 + i0] = b0;
            p.out[(long)m * p.ldo + n0 + i1] = b1;
            if ((is_k || is_v) && sl >= 0) {
              const int kvh = head - p.rp_nq - (is_v ? p.rp_nkv : 0);
              const int page = p.rp_table[(long)sl * p.rp_max_pages + ps / 64];
              const long dst = (((long)page * p.rp_nkv + kvh) * 64 + (ps % 64)) * 128;
              if (p.rp_fp8) {
                uint8_t* pool = reinterpret_cast<uint8_t*>(is_v ? p.rp_vpool : p.rp_kpool);
                pool[dst + i0] = (uint8_t)__nv_cvt_float_to_fp8(bf2f(b0), __NV_SATFINITE, __NV_E5M2);
                pool[dst + i1] = (uint8_t)__nv_cvt_float_to_fp8(bf2f(b1), __NV_SATFINITE, __NV_E5M2);
              } else {
                __nv_bfloat16* pool = reinterpret_cast<__nv_bfloat16*>(is_v ? p.rp_vpool : p.rp_kpool);
                pool[dst + i0] = b0;
                pool[dst + i1] = b1;
              }
            }
          }
        }
      }
    } else if (write && n < p.N && !s_fail) {
#pragma unroll
      for (int m = 0; m < MROWS; ++m) {
        if (m < p.M) {
          float v = acc[m] * p.alpha;
          if (p.residual) v += bf2f(p.residual[(long)m * p.ldr + n]);
          if (p.out_f32) p.out_f32[(long)m * p.ldo + n] = v;
          else p.out[(long)m * p.ldo + n] = f2bf(v);
          if (p.ll_seq) {
            // four neighbouring features make one 16-byte line; lane 4j sends it to every peer
            const uint32_t bits = (uint32_t)__bfloat16_as_ushort(f2bf(v));
            const uint32_t b1 = __shfl_down_sync(0xffffffffu, bits, 1), b2 = __shfl_down_sync(0xffffffffu, bits, 2),
                           b3 = __shfl_down_sync(0xffffffffu, bits, 3);
            if ((lane & 3) == 0) {
              const uint32_t seq = *p.ll_seq;
              const int stage = seq & 3;
              const size_t slot = p.ll_off + ((size_t)(stage * p.ll_size + p.ll_rank) * 16 + m) * p.ll_row_bytes +
                                  (size_t)(n >> 2) * 16;
              const uint4 pkt = make_uint4(bits | (b1 << 16), seq, b2 | (b3 << 16), seq);
              for (int i = 1; i < p.ll_size; ++i) {
                uint8_t* dst = p.ll_peer[(p.ll_rank + i) % p.ll_size] + slot;
                asm volatile("st.volatile.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(dst), "r"(pkt.x), "r"(pkt.y),
                             "r"(pkt.z), "r"(pkt.w) : "memory");
              }
            }
          }
        }
      }
    }
    if (p.an_out && write) {
      // the last tile to finish normalises the rows (write is uniform over the 128 epilogue threads)
      __threadfence();
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (etid == 0) s_ticket = atomicAdd(p.an_ticket, 1);
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (s_ticket == (int)gridDim.x - 1) {
        __threadfence();
        const int nv = p.N >> 3;                         // 8-element vectors per row
        for (int m = 0; m < p.M; ++m) {
          const uint4* orow = reinterpret_cast<const uint4*>(p.out + (long)m * p.ldo);
          uint4* rrow = reinterpret_cast<uint4*>(p.an_resid + (long)m * p.N);
          float ss = 0.f;
          for (int v = etid; v < nv; v += 128) {
            const uint4 o = __ldcg(orow + v), r = rrow[v];
            const uint32_t ow[4] = {o.x, o.y, o.z, o.w}, rw[4] = {r.x, r.y, r.z, r.w};
            uint32_t hw[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&ow[j]));
              const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&rw[j]));
              const __nv_bfloat162 h2 = __floats2bfloat162_rn(a.x + b.x, a.y + b.y);
              const float2 hf = __bfloat1622float2(h2);
              ss = fmaf(hf.x, hf.x, fmaf(hf.y, hf.y, ss));
              hw[j] = *reinterpret_cast<const uint32_t*>(&h2);
            }
            rrow[v] = make_uint4(hw[0], hw[1], hw[2], hw[3]);
          }
          ss = warp_sum(ss);
          if (lane == 0) s_red[q] = ss;
          asm volatile("bar.sync 1, 128;" ::: "memory");
          const float inv = rsqrtf((s_red[0] + s_red[1] + s_red[2] + s_red[3]) / (float)p.N + p.an_eps);
          const uint4* wrow = reinterpret_cast<const uint4*>(p.an_w);
          uint4* xrow = reinterpret_cast<uint4*>(p.an_out + (long)m * p.N);
          for (int v = etid; v < nv; v += 128) {
            const uint4 r = rrow[v], w4 = __ldg(wrow + v);
            const uint32_t rw[4] = {r.x, r.y, r.z, r.w}, ww[4] = {w4.x, w4.y, w4.z, w4.w};
            uint32_t xw[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const float2 h = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&rw[j]));
              const float2 g = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&ww[j]));
              const __nv_bfloat162 x2 = __floats2bfloat162_rn(h.x * inv * (g.x + p.an_wbias), h.y * inv * (g.y + p.an_wbias));
              xw[j] = *reinterpret_cast<const uint32_t*>(&x2);
            }
            xrow[v] = make_uint4(xw[0], xw[1], xw[2], xw[3]);
          }
          asm volatile("bar.sync 1, 128;" ::: "memory");
        }
        if (etid == 0) *p.an_ticket = 0;                 // ready for the next launch
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem_base, TMEM_COLS); }
  if (threadIdx.x == 0 && s_fail && p.status) atomicExch(p.status, (int)kErrMbarTimeout);
}

template <int BN, int TERMS, int STAGES>
static int launch_decode(const DecodeParams& p, const CUtensorMap& amap, int KS, int pdl, cudaStream_t st) {
  constexpr int smem = STAGES * (128 * 128 + BN * 128 + 4096) + 1024;
  static_assert(smem <= 113 * 1024, "two CTAs per SM");
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(decode_w4a4_kernel<BN, TERMS, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return (int)e;
    attr_set = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(p.N / 128, KS);
  cfg.blockDim = dim3(192);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = at;
  cfg.numAttrs = pdl ? 1 : 0;
  return (int)cudaLaunchKernelEx(&cfg, decode_w4a4_kernel<BN, TERMS, STAGES>, p, amap);
}

}  // namespace ve

using namespace ve;

extern "C" {

// Stand-alone form of the expansion the decode linear does in its producer warps (same arithmetic; used to test
// it). Xs must hold K/64 atoms of 512 B (zero-initialised once).
int ve_nvfp4_expand_rows(const void* X, long ldx, void* Xp, void* Xs, int M, int K, int terms, cudaStream_t st) {
  if (M < 1 || K % 64 || M * terms > 128) return cudaErrorInvalidValue;
  const int total = M * (K / 16);
  const int blocks = (total + 127) / 128;
  if (terms == 4) nvfp4_expand_rows_kernel<4><<<blocks, 128, 0, st>>>((const __nv_bfloat16*)X, ldx, (uint8_t*)Xp, (uint8_t*)Xs, M, K);
  else if (terms == 2) nvfp4_expand_rows_kernel<2><<<blocks, 128, 0, st>>>((const __nv_bfloat16*)X, ldx, (uint8_t*)Xp, (uint8_t*)Xs, M, K);
  else if (terms == 1) nvfp4_expand_rows_kernel<1><<<blocks, 128, 0, st>>>((const __nv_bfloat16*)X, ldx, (uint8_t*)Xp, (uint8_t*)Xs, M, K);
  else return cudaErrorInvalidValue;
  VE_CHECK_LAUNCH();
}

// Wp [N, K/2] codes, sfa [N/128][ceil(K/256)*4][512] (k-groups padded with zero scales to whole 256-wide tiles), X [M, K] bf16 (pitch ldx elements, rows 16-byte aligned).
// ws: fp32 [N/128][ks][16][128]; tickets: int [N/128] zeroed once; ks = K splits (>= 1).
// pdl != 0 launches with programmatic stream serialization: set-up and the first weight tiles overlap the kernel
// in front of it in the stream (the kernel waits for that kernel before it touches X, residual or out).
// The ranges the next ve_decode_w4a4 launch of this host thread asks the memory system to bring into L2 (consumed by that
// launch). Both pointers 16 B aligned; sizes are rounded down to multiples of 16 B.
static thread_local const void* g_pf_ptr = nullptr;
static thread_local size_t g_pf_bytes = 0;
static thread_local const void* g_pf_ptr2 = nullptr;
static thread_local size_t g_pf_bytes2 = 0;

int ve_decode_set_prefetch(const void* w, size_t bytes, const void* sf, size_t sf_bytes) {
  if (((uintptr_t)w & 15) || ((uintptr_t)sf & 15)) return cudaErrorMisalignedAddress;
  g_pf_ptr = w; g_pf_bytes = bytes & ~(size_t)15;
  g_pf_ptr2 = sf; g_pf_bytes2 = sf_bytes & ~(size_t)15;
  return 0;
}

int ve_decode_w4a4(const void* Wp, const void* sfa, const void* X, long ldx, void* out, long ldo, void* out_f32,
                   const void* residual, long ldr, int M, int N, int K, float alpha, int terms, int ks, int pdl, int act,
                   float act_limit, const void* pn_w, const void* pn_resid, const void* pn_delta, void* pn_resid_out,
                   float pn_eps, float pn_wbias, const void* comm_args, void* an_resid, const void* an_w, void* an_out,
                   float an_eps, float an_wbias, void* an_ticket, const void* rp_pos, const void* rp_slot,
                   const void* rp_table, int rp_max_pages, void* rp_kpool, void* rp_vpool, int rp_nq, int rp_nkv, int rp_rot,
                   float rp_theta, int rp_fp8, void* ws, void* tickets, void* status, cudaStream_t st) {
  if (rp_pos && (act || out_f32 || residual || comm_args || an_out || !out || !rp_table || !rp_kpool || !rp_vpool ||
                 N != (rp_nq + 2 * rp_nkv) * 128 || rp_rot < 2 || rp_rot > 128 || rp_rot % 2))
    return cudaErrorInvalidValue;
  if (act && (out_f32 || residual || !out)) return cudaErrorInvalidValue;
  if (an_out && (act || out_f32 || residual || comm_args || !out || !an_resid || !an_w || !an_ticket || ldo % 8 || N % 8))
    return cudaErrorInvalidValue;
  if (pn_w && (M > 4 || !pn_resid || K % 16 || (pn_delta && pn_resid_out == pn_resid))) return cudaErrorInvalidValue;
  if (M < 1 || N % 128 || K % 128 || (pn_w && K % 256) || ldx % 8 || (terms != 1 && terms != 2 && terms != 4) || M * terms > 64)
    return cudaErrorInvalidValue;
  if (ks < 1) ks = 1;
  if (ks > (K + 255) / 256) ks = (K + 255) / 256;
  if (ks > 1 && (!ws || !tickets)) return cudaErrorInvalidValue;
  const int cols = M * terms, bn = cols <= 16 ? 16 : cols <= 32 ? 32 : 64;
  CUtensorMap amap;
  int rc = make_tmap_2d(&amap, Wp, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, N, K / 2, (uint64_t)K / 2, 128, 128, CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc) return rc;
  int tpt = 16;
  while (tpt < 16 * M && tpt < 128) tpt <<= 1;
  DecodeParams p{N, M, K, alpha, (const __nv_bfloat16*)X, ldx, (__nv_bfloat16*)out, ldo, (const __nv_bfloat16*)residual, ldr,
                 (float*)out_f32, (const uint8_t*)sfa, (float*)ws, (int*)tickets, (int*)status, tpt, act, act_limit,
                 (const __nv_bfloat16*)pn_w, (const __nv_bfloat16*)pn_resid, (const __nv_bfloat16*)pn_delta,
                 (__nv_bfloat16*)pn_resid_out, pn_eps, pn_wbias};
  p.ll_seq = nullptr;
  for (int i = 0; i < 8; ++i) p.ll_peer[i] = nullptr;
  p.rp_pos = (const int*)rp_pos; p.rp_slot = (const int*)rp_slot; p.rp_table = (const int*)rp_table;
  p.rp_max_pages = rp_max_pages; p.rp_kpool = rp_kpool; p.rp_vpool = rp_vpool; p.rp_nq = rp_nq; p.rp_nkv = rp_nkv;
  p.rp_rot = rp_rot; p.rp_fp8 = rp_fp8; p.rp_theta = rp_theta;
  p.an_ticket = (int*)an_ticket; p.an_resid = (__nv_bfloat16*)an_resid; p.an_w = (const __nv_bfloat16*)an_w;
  p.an_out = (__nv_bfloat16*)an_out; p.an_eps = an_eps; p.an_wbias = an_wbias;
  p.pf_ptr = (const uint8_t*)g_pf_ptr; p.pf_bytes = g_pf_bytes; p.pf_ptr2 = (const uint8_t*)g_pf_ptr2; p.pf_bytes2 = g_pf_bytes2;
  g_pf_ptr = g_pf_ptr2 = nullptr; g_pf_bytes = g_pf_bytes2 = 0;
  if (comm_args) {
    // leading fields of ve::CommArgs (csrc/cuda/comm.cu): peer[8], mc, rank, size, seq, status, budget, off_ll, ll_row_bytes
    struct Lead { uint8_t* peer[8]; uint8_t* mc; int rank, size; uint32_t* seq; int* status; unsigned long long budget;
                  size_t off_ll, ll_row_bytes; };
    const Lead& a = *reinterpret_cast<const Lead*>(comm_args);
    if (act || out_f32 || residual || M > 16 || (size_t)N * 4 > a.ll_row_bytes) return cudaErrorInvalidValue;
    for (int i = 0; i < 8; ++i) p.ll_peer[i] = a.peer[i];
    p.ll_seq = a.seq; p.ll_rank = a.rank; p.ll_size = a.size; p.ll_off = a.off_ll; p.ll_row_bytes = a.ll_row_bytes;
  }
#define VE_DW(BN, T, S) return launch_decode<BN, T, S>(p, amap, ks, pdl, st)
  static int stages3 = -1;       // VOLTA_DW_STAGES=3: three pipeline stages (three CTAs per SM) for the one-row shapes
  if (stages3 < 0) { const char* e = getenv("VOLTA_DW_STAGES"); stages3 = (e && e[0] == '3') ? 1 : 0; }
  if (terms == 4) {
    if (bn == 16) { if (stages3) VE_DW(16, 4, 3); VE_DW(16, 4, 4); }
    if (bn == 32) VE_DW(32, 4, 4);
    VE_DW(64, 4, 3);
  }
  if (terms == 2) { if (bn == 16) VE_DW(16, 2, 4); if (bn == 32) VE_DW(32, 2, 4); VE_DW(64, 2, 3); }
  if (bn == 16) VE_DW(16, 1, 4);
  if (bn == 32) VE_DW(32, 1, 4);
  VE_DW(64, 1, 3);
#undef VE_DW
}

}  // extern "C"
