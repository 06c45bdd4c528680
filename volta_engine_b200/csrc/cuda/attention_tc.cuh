// Prefill attention on the fifth-generation tensor cores (tcgen05, accumulators in TMEM). Included by attention.cu.
//
// One CTA = one query tile of up to 128 packed rows ((token, head-in-group) pairs of one kv head, one TMEM lane per
// row) against the pages of its sequence, bf16 cache, head_dim 128, no key split. Per 64-key page:
//     S  = Q K^T      tcgen05.mma 128 x 64 x 128   (Q and the K page K-major in 128B-swizzled shared memory)
//     P  = exp2(S * scale - m)                      (softmax warps: tcgen05.ld of one row per thread, bf16 P written to
//                                                    shared memory in the K-major swizzled layout)
//     O += P V        tcgen05.mma 128 x 128 x 64   (V page as it lands from TMA: the MN-major operand form)
// Warp roles (320 threads): warp 0 streams pages by TMA (four stages), warp 1 issues the MMAs, warps 2..5 and 6..9 are two
// softmax groups of 128 threads (one row per thread each). The pages are dealt to two independent streams, even pages to
// the first group and odd pages to the second, each with its own S buffers (2 x 64 TMEM columns), its own running
// (reference maximum, row sum) and its own O accumulator (128 columns), so the exponentials of one stream run under the
// MMAs of the other and two warps per scheduler hide the TMEM-load and barrier latencies; the two partial results are
// merged like split-KV partials in the epilogue (both accumulators live in the same TMEM lanes, so a thread reads both).
// The reference maximum is only moved when a page raises it by more than 2^8 (then the O row is rescaled in TMEM by
// the thread that owns it); otherwise the old reference stays, probabilities are at most 2^8 and the final division by
// the row sum makes the result the same. The exponent is one FMA (score * scale - reference) and one ex2.approx.
// Every wait is bounded; on expiry the CTA records a status code, skips its stores and frees its TMEM.
// Semantics are those of attn_kernel (causal limit / key_end, sliding window, optional sigmoid gate); reference:
// src/kernels/slang/ref_attention.slang:1-10,47-50,65-70.
#pragma once

namespace ve {

VE_DEVINL void tmem_st32(uint32_t taddr, const uint32_t* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
        "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]),
        "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]),
        "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
VE_DEVINL void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// Descriptor of an MN-major operand stored with the 128-byte swizzle: 64 contiguous elements of the M / N extent per
// 128 B row, 8 rows (8 steps of K) per 1024 B atom; `lbo` = bytes to the next 64 elements of M / N, `sbo` = bytes to
// the next 8 steps of K.
VE_DEVINL uint64_t make_desc_sw128_mn(uint32_t saddr, uint32_t lbo, uint32_t sbo) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr & 0x3FFFF) >> 4);
  d |= (uint64_t)(lbo >> 4) << 16;
  d |= (uint64_t)(sbo >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}

constexpr int kTcRows = 128;        // query rows of a tile
constexpr int kTcThreads = 320;
constexpr float kTcLazyLog2 = 8.f;  // the reference maximum moves only when a page raises it by more than this

VE_DEVINL float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

template <int HD, int NST>
__global__ void __launch_bounds__(kTcThreads, 1) attn_prefill_tc_kernel(const AttnParams p, const __grid_constant__ CUtensorMap kmap,
                                                                        const __grid_constant__ CUtensorMap vmap) {
  static_assert(HD == 128, "the tcgen05 prefill kernel is written for head_dim 128");
  constexpr int TILE = kPageTok * HD * 2;       // one K or V page: 16 KB, two 64-column chunks of 8 KB
  constexpr int Q_BYTES = kTcRows * HD * 2;     // 32 KB, two 64-column chunks of 16 KB
  constexpr int P_BYTES = kTcRows * kPageTok * 2;
  // TMEM columns: S of stream t, buffer b at t * 128 + b * 64; O of stream t at 256 + t * 128
  constexpr uint32_t TMEM_COLS = 512, O_COL = 256;
  const float NEG_INF = __int_as_float(0xff800000);
  grid_dep_launch();
  grid_dep_wait();
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* q_s = smem;
  uint8_t* kv_s = smem + Q_BYTES;               // [NST][K page | V page]
  uint8_t* p_s = kv_s + NST * 2 * TILE;         // [2 streams][128 rows x 64 keys]
  __shared__ uint64_t full[NST], empty[NST], s_full[2][2], p_full[2], pv_done[2];
  __shared__ uint32_t tmem_holder;
  __shared__ int s_fail;

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  // later tiles of a sequence see more keys: they are started first so that the last wave holds the short ones
  const int tile = gridDim.x - 1 - blockIdx.x, kvh = blockIdx.y;
  const int G = p.nq / p.nkv;
  const int first = p.tile_first ? p.tile_first[tile] : tile;
  const int count = p.tile_count ? p.tile_count[tile] : 1;
  const int s = p.slot ? p.slot[first] : 0;
  if (count <= 0 || s < 0) return;              // uniform: before any barrier or TMEM use

  int lim_max = -1, pos_min = 0x7fffffff;
  for (int i = 0; i < count; ++i) {
    const int ps = p.pos[first + i];
    const int lm = p.key_end ? p.key_end[first + i] : ps;
    lim_max = max(lim_max, lm);
    pos_min = min(pos_min, ps);
  }
  const int kt_end = lim_max / kPageTok + 1;
  const int kt_begin = p.window > 0 ? max(0, pos_min - p.window + 1) / kPageTok : 0;
  const int n = kt_end - kt_begin;

  if (tid == 0) {
    for (int i = 0; i < NST; ++i) {
      mbar_init(&full[i], 1);
      mbar_init(&empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&s_full[i][0], 1);
      mbar_init(&s_full[i][1], 1);
      mbar_init(&p_full[i], 128);
      mbar_init(&pv_done[i], 1);
    }
    s_fail = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(&tmem_holder, TMEM_COLS);
    tmem_relinquish();
  }
  // a softmax thread owns one row of one stream: TMEM lane = 32 * (warp % 4) + lane, stream = (warp - 2) / 4
  const int r = (warp & 3) * 32 + lane;
  const int strm = warp >= 6 ? 1 : 0;
  const bool r_ok = warp >= 2 && r < count * G;
  const int rr = r_ok ? r : 0;
  const int r_tok = first + rr / G, r_head = kvh * G + rr % G;
  const int r_pos = p.pos[r_tok];
  const int r_lim = p.key_end ? p.key_end[r_tok] : r_pos;
  if (warp >= 2) {
    // each stream's threads bring in one 64-column half of their row of Q
    const uint4* src = reinterpret_cast<const uint4*>(p.q + (long)r_tok * p.q_stride + (long)r_head * HD) + strm * 8;
#pragma unroll
    for (int ch = 0; ch < 8; ++ch) {
      const uint4 v = r_ok ? src[ch] : make_uint4(0u, 0u, 0u, 0u);
      *reinterpret_cast<uint4*>(q_s + strm * (kTcRows * 128) + r * 128 + ((ch ^ (r & 7)) << 4)) = v;
    }
    fence_proxy_async_smem();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_holder;

  if (warp == 0) {
    // ------------------------------------------------------------------ page loads
    if (elect_one()) {
      prefetch_tmap(&kmap);
      prefetch_tmap(&vmap);
      for (int j = 0; j < n; ++j) {
        const int st = j % NST;
        if (j >= NST && !mbar_wait(&empty[st], ((j / NST) - 1) & 1)) {
          atomicExch(&s_fail, 1);
          break;
        }
        const int page = p.page_table[(long)s * p.max_pages + kt_begin + j];
        const int row = (page * p.nkv + kvh) * kPageTok;
        uint8_t* kb = kv_s + st * 2 * TILE;
        uint8_t* vb = kb + TILE;
        mbar_expect_tx(&full[st], 2 * TILE);
        tma_load_2d(kb, &kmap, &full[st], 0, row);
        tma_load_2d(kb + 8192, &kmap, &full[st], 64, row);
        tma_load_2d(vb, &vmap, &full[st], 0, row);
        tma_load_2d(vb + 8192, &vmap, &full[st], 64, row);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issue
    if (elect_one()) {
      constexpr uint32_t idesc_s = make_idesc_f16(1, 1, kTcRows, kPageTok);
      constexpr uint32_t idesc_pv = make_idesc_f16(1, 1, kTcRows, HD) | (1u << 16);      // B (the V page) is MN-major
      const uint32_t q_a = smem_u32(q_s), kv_a = smem_u32(kv_s), p_a = smem_u32(p_s);
      bool ok = true;
      // page j belongs to stream j & 1 and is that stream's page j >> 1
      auto issue_s = [&](int j) {
        const int st = j % NST, t = j & 1, b = (j >> 1) & 1;
        if (!mbar_wait(&full[st], (j / NST) & 1)) return false;
        tc_fence_after();
        const uint32_t kb = kv_a + st * 2 * TILE;
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk) {
          const int c = kk >> 2, off = (kk & 3) * 2;
          tc_mma_f16(tmem_base + t * 128 + b * kPageTok, make_desc_sw128(q_a + c * (kTcRows * 128)) + off,
                     make_desc_sw128(kb + c * 8192) + off, idesc_s, kk ? 1u : 0u);
        }
        tc_commit(&s_full[t][b]);
        return true;
      };
      ok = issue_s(0);
      if (ok && n > 1) ok = issue_s(1);
      for (int j = 0; j < n && ok; ++j) {
        // the S buffer page j + 2 lands in was read by the softmax of page j - 2, which ended before its P arrived
        if (j + 2 < n) ok = issue_s(j + 2);
        if (!ok) break;
        const int t = j & 1, i = j >> 1;
        ok = mbar_wait(&p_full[t], i & 1);
        if (!ok) break;
        tc_fence_after();
        const uint32_t vb = kv_a + (j % NST) * 2 * TILE + TILE;
#pragma unroll
        for (int ks = 0; ks < kPageTok / 16; ++ks)
          tc_mma_f16(tmem_base + O_COL + t * HD, make_desc_sw128(p_a + t * P_BYTES) + ks * 2,
                     make_desc_sw128_mn(vb + ks * 2048, 8192u, 1024u), idesc_pv, (i | ks) ? 1u : 0u);
        tc_commit(&pv_done[t]);
        tc_commit(&empty[j % NST]);
      }
      if (!ok) atomicExch(&s_fail, 1);
    }
  } else {
    // ------------------------------------------------------------------ softmax and correction of one stream
    const uint32_t t_lane = tmem_base + ((uint32_t)((warp & 3) * 32) << 16);
    const uint32_t o_col = O_COL + strm * HD;
    const int n_mine = (n - strm + 1) >> 1;
    float m_ref = NEG_INF, l0 = 0.f, l1 = 0.f;
    bool ok = true;
    uint8_t* prow = p_s + strm * P_BYTES + r * 128;
    for (int i = 0; i < n_mine; ++i) {
      const int b = i & 1, key0 = (kt_begin + 2 * i + strm) * kPageTok;
      ok = __all_sync(0xffffffffu, mbar_wait(&s_full[strm][b], (i >> 1) & 1));
      if (!ok) break;
      tc_fence_after();
      float sv[kPageTok];
      tmem_ld32(t_lane + strm * 128 + b * kPageTok, reinterpret_cast<uint32_t*>(sv));
      tmem_ld32(t_lane + strm * 128 + b * kPageTok + 32, reinterpret_cast<uint32_t*>(sv) + 32);
      tmem_ld_wait();
      if (!r_ok || key0 + kPageTok - 1 > r_lim || (p.window > 0 && key0 <= r_pos - p.window)) {
#pragma unroll
        for (int e = 0; e < kPageTok; ++e) {
          const int key = key0 + e;
          const bool allow = r_ok && key <= r_lim && (p.window <= 0 || key > r_pos - p.window);
          sv[e] = allow ? sv[e] : NEG_INF;
        }
      }
      float mx0 = sv[0], mx1 = sv[1], mx2 = sv[2], mx3 = sv[3];
#pragma unroll
      for (int e = 4; e < kPageTok; e += 4) {
        mx0 = fmaxf(mx0, sv[e]);
        mx1 = fmaxf(mx1, sv[e + 1]);
        mx2 = fmaxf(mx2, sv[e + 2]);
        mx3 = fmaxf(mx3, sv[e + 3]);
      }
      const float mx = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3)) * p.scale_log2;     // the scale is positive
      const bool grow = mx > m_ref + kTcLazyLog2;
      float alpha = 1.f;
      if (grow) {
        alpha = ex2_approx(m_ref - mx);          // 0 for the first keys a row sees
        m_ref = mx;
      }
      const bool fix = i > 0 && __any_sync(0xffffffffu, grow);
      // The stream's previous PV read the P buffer this page is about to overwrite and is the last writer of O: a row
      // correction waits for it now, otherwise the exponentials run first and only the stores of P wait.
      if (fix) {
        ok = __all_sync(0xffffffffu, mbar_wait(&pv_done[strm], (i - 1) & 1));
        if (!ok) break;
        tc_fence_after();
#pragma unroll 1
        for (int c0 = 0; c0 < HD; c0 += 32) {
          uint32_t ov[32];
          tmem_ld32(t_lane + o_col + c0, ov);
          tmem_ld_wait();
#pragma unroll
          for (int e = 0; e < 32; ++e) ov[e] = __float_as_uint(__uint_as_float(ov[e]) * alpha);
          tmem_st32(t_lane + o_col + c0, ov);
        }
        tmem_st_wait();
      }
      l0 *= alpha;
      l1 *= alpha;
      const float neg_m = m_ref == NEG_INF ? 0.f : -m_ref;
      uint32_t w[kPageTok / 2];
#pragma unroll
      for (int e = 0; e < kPageTok / 2; ++e) {
        const float p0 = ex2_approx(fmaf(sv[2 * e], p.scale_log2, neg_m));
        const float p1 = ex2_approx(fmaf(sv[2 * e + 1], p.scale_log2, neg_m));
        l0 += p0;
        l1 += p1;
        w[e] = pack_bf16(p0, p1);
      }
      if (i > 0 && !fix) {
        ok = __all_sync(0xffffffffu, mbar_wait(&pv_done[strm], (i - 1) & 1));
        if (!ok) break;
      }
#pragma unroll
      for (int ch = 0; ch < 8; ++ch)
        *reinterpret_cast<uint4*>(prow + ((ch ^ (r & 7)) << 4)) = make_uint4(w[4 * ch], w[4 * ch + 1], w[4 * ch + 2], w[4 * ch + 3]);
      fence_proxy_async_smem();
      tc_fence_before();
      mbar_arrive(&p_full[strm]);
    }
    if (n_mine > 0) ok = __all_sync(0xffffffffu, ok && mbar_wait(&pv_done[strm], (n_mine - 1) & 1));
    if (!ok) atomicExch(&s_fail, 1);
    // the stream's P buffer is free now (its last PV has completed): it carries (maximum, sum) to the merge
    reinterpret_cast<float*>(p_s + strm * P_BYTES)[r] = m_ref;
    reinterpret_cast<float*>(p_s + strm * P_BYTES)[kTcRows + r] = l0 + l1;
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (warp >= 2 && !s_fail) {
    // ------------------------------------------------------------------ merge of the two streams and output
    // stream 0's threads write columns 0..63 of their row, stream 1's threads columns 64..127
    const uint32_t t_lane = tmem_base + ((uint32_t)((warp & 3) * 32) << 16);
    const float* ml0 = reinterpret_cast<const float*>(p_s);
    const float* ml1 = reinterpret_cast<const float*>(p_s + P_BYTES);
    const float m0 = ml0[r], m1 = ml1[r];
    const float m = fmaxf(m0, m1);
    const float a0 = m == NEG_INF ? 0.f : ex2_approx(m0 - m), a1 = (m == NEG_INF || n < 2) ? 0.f : ex2_approx(m1 - m);
    const float l = ml0[kTcRows + r] * a0 + (n < 2 ? 0.f : ml1[kTcRows + r] * a1);
    const float inv = l > 0.f ? 1.f / l : 0.f;
    const float f0 = a0 * inv, f1 = a1 * inv;
    __nv_bfloat16* orow = p.out + (long)r_tok * p.out_stride + (long)r_head * HD;
    const __nv_bfloat16* grow_ = p.gate ? p.gate + (long)r_tok * p.gate_stride + (long)r_head * HD : nullptr;
#pragma unroll 1
    for (int c0 = strm * 64; c0 < strm * 64 + 64; c0 += 32) {
      uint32_t ov[32], ow[32];
      tmem_ld32(t_lane + O_COL + c0, ov);
      if (n > 1) tmem_ld32(t_lane + O_COL + HD + c0, ow);     // a one-page tile never wrote the second accumulator
      tmem_ld_wait();
      if (r_ok) {
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4) {
          uint32_t w[4];
          uint32_t gw[4] = {0u, 0u, 0u, 0u};
          if (grow_) {
            const uint4 g4 = *reinterpret_cast<const uint4*>(grow_ + c0 + q4 * 8);
            gw[0] = g4.x; gw[1] = g4.y; gw[2] = g4.z; gw[3] = g4.w;
          }
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            float a = __uint_as_float(ov[q4 * 8 + 2 * e]) * f0, c = __uint_as_float(ov[q4 * 8 + 2 * e + 1]) * f0;
            if (n > 1) {
              a = fmaf(__uint_as_float(ow[q4 * 8 + 2 * e]), f1, a);
              c = fmaf(__uint_as_float(ow[q4 * 8 + 2 * e + 1]), f1, c);
            }
            if (grow_) {
              const __nv_bfloat162 g2 = *reinterpret_cast<const __nv_bfloat162*>(&gw[e]);
              a *= 1.f / (1.f + __expf(-__low2float(g2)));
              c *= 1.f / (1.f + __expf(-__high2float(g2)));
            }
            w[e] = pack_bf16(a, c);
          }
          *reinterpret_cast<uint4*>(orow + c0 + q4 * 8) = make_uint4(w[0], w[1], w[2], w[3]);
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
  if (tid == 0 && s_fail && p.status) atomicExch(p.status, (int)kErrMbarTimeout);
}

template <int HD, int NST>
static int launch_attn_tc_n(const AttnParams& p, const CUtensorMap& kmap, const CUtensorMap& vmap, int ntiles, cudaStream_t st) {
  constexpr int smem = kTcRows * HD * 2 + NST * 2 * kPageTok * HD * 2 + 2 * kTcRows * kPageTok * 2 + 1024;
  static bool attr = false;
  if (!attr) {
    cudaError_t e = cudaFuncSetAttribute(attn_prefill_tc_kernel<HD, NST>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return (int)e;
    attr = true;
  }
  launch_pdl(attn_prefill_tc_kernel<HD, NST>, dim3(ntiles, p.nkv, 1), dim3(kTcThreads), smem, st, p, kmap, vmap);
  return (int)cudaGetLastError();
}

template <int HD>
static int launch_attn_tc(const AttnParams& p, const CUtensorMap& kmap, const CUtensorMap& vmap, int ntiles, cudaStream_t st) {
  return launch_attn_tc_n<HD, 4>(p, kmap, vmap, ntiles, st);      // a fifth stage measured the same (804 vs 803 TFLOP/s)
}

}  // namespace ve
