// One persistent kernel per decode step of the dense GQA decoder (<= 4 rows): every linear, the rotary embedding and
// KV store, paged attention with its split merge, the residual adds and RMSNorms, the tensor-parallel all-reduces and the
// LM head run as stages of a single launch, one CTA per SM.
//
// Why: a decode step of a 64-layer model is a chain of ~450 dependent kernels whose per-launch floor (TMEM allocation,
// barrier set-up, pipeline fill, drain) does not shrink with the weight shard, so the step sits far from the HBM byte
// floor on one GPU and does not scale over GPUs. Here the chain is a list of ops walked by every CTA:
//   * warp 0 streams weight tiles (TMA, packed NVFP4 + scale atoms) and KV pages into an 8-deep ring of shared-memory
//     stages. Weights do not depend on activations, so the stream runs ahead across op boundaries: the HBM pipe stays
//     busy while the other warps wait for a dependency.
//   * warp 1 issues tcgen05.mma kind::mxf4nvf4 (weights = A operand, 128 features per tile; activations expanded into
//     4 residual NVFP4 rows each = B operand, 16 columns) into two TMEM accumulators.
//   * warps 2-5 build the B operand of every unit (norm / activation / reductions fused into that step), run the
//     epilogues, the attention math (mma.sync m16n8k16 on swizzled pages) and the small finalise / merge stages.
// An op's (tile, k-tile) units are dealt to the CTAs in contiguous runs (tile-major), so all SMs stream every weight;
// a tile shared by several CTAs is summed in split order either by the consumer (partials) or by the CTA that arrives
// last on the tile's ticket, which keeps every result independent of timing. Stages are chained by per-op arrival
// counters in global memory (release / acquire at gpu scope); every wait is bounded and reports through the status word,
// and a status word that is already set makes every wait give up at once so the launch drains in microseconds.
// Tensor parallel: the CTA that finishes a tile of a row-parallel linear sends it as low-latency lines
// {data, seq, data, seq} into every peer's staging area (plain peer stores) and adds the peers' lines for the same
// tile in rank order, so the all-reduce has no launch and no barrier of its own.
// Reference hot path this replaces: src/models/gemma4.cpp:438-521 (graph of ~8 kernels per layer) with
// src/comm/all_reduce_ipc.cu:136-298 behind each row-parallel projection.
#include "common.cuh"
#include "nvfp4_expand.cuh"
#include "tmap.h"
#include <float.h>

namespace ve {

constexpr int DS_NS = 8;                                 // ring stages
constexpr int DS_A = 16384, DS_B = 2048, DS_SF = 2048;   // weight tile / B operand / one scale block
constexpr int DS_STAGE = DS_A + DS_B + 2 * DS_SF;        // 22528 B
constexpr int DS_SCR = 40960;                            // scratch: normalised-input row(s) or attention merge
constexpr int DS_MAXM = 4;
constexpr int DS_TERMS = 4;
constexpr int DS_LOOK = 4;                               // epilogues run this many units behind the B-operand fill
constexpr int DS_TMEM = 128;
constexpr int DS_SMEM = DS_NS * DS_STAGE + DS_SCR + 1024;

enum : int { OP_LINEAR = 0, OP_QKV_FIN = 1, OP_ATTN = 2, OP_MERGE = 3, OP_NORMOUT = 4 };
enum : int { IN_X = 0, IN_NORM = 1, IN_GATED = 2, IN_EMBED = 3 };
enum : int { OUT_PART = 0, OUT_LOGITS = 1, OUT_TICKET = 2 };

struct StepOp {
  int type, in_mode, out_mode, map;
  int N, K, upc, src;          // src: index of the op whose result this op reads
  float alpha;                 // tensor scale of this op's weights
  int ws_off;                  // float offset of this op's partial sums in the workspace
  int ms;                      // slots per tile in the workspace (>= most splits of a tile)
  int tk_off;                  // first ticket of this op (OUT_TICKET)
  int ncontrib;                // arrivals that complete this op
  int layer;
  int hpar;                    // IN_NORM: residual buffer read (the other one is written)
  int ypar;                    // OUT_TICKET: reduced-output buffer written
  int ar;                      // OUT_TICKET, tensor parallel: index of this all-reduce inside the step
  int flags;                   // 1: write the normalised input rows to xfinal
  const uint8_t* sfa;          // scale atoms [N/128][ceil(K/256)*4][512]
  const __nv_bfloat16* norm_w; // IN_NORM / IN_EMBED
};

struct StepParams {
  const StepOp* ops;
  const CUtensorMap* maps;     // weight maps, then K pool, then V pool
  uint32_t* cnt;               // [nops] arrival counters, zero between launches
  uint32_t* ctrl;              // [0] CTAs that finished
  int* tickets;
  float* ws;
  __nv_bfloat16* ybuf;         // [2][MAXM][H]
  __nv_bfloat16* hbuf;         // [2][MAXM][H]
  __nv_bfloat16* qbuf;         // [MAXM][nq * 128]
  __nv_bfloat16* attn_out;     // [MAXM][nq * 128]
  float* o_part;               // [MAXM][nq][S][128]
  float* lse_part;             // [MAXM][nq][S]
  __nv_bfloat16* xfinal;       // [MAXM][H]
  float* logits;
  const int* ids;
  const int* pos;
  const int* slot;
  const int* page_table;
  const __nv_bfloat16* embed;
  __nv_bfloat16* kpool;        // [layers][pages][nkv][64][128]
  __nv_bfloat16* vpool;
  int* status;
  uint8_t* peer[8];
  uint32_t* seq;
  unsigned long long off_ll, ll_row_bytes, budget_ns;
  long ldl, pool_layer_rows;
  int nops, kmap, vmap, M, H, nq, nkv, S, max_pages, vocab, rot, act, rank, size, n_ar, pad0;
  float eps, wbias, scale_log2, rope_theta, act_limit, embed_scale;
};

VE_DEVINL uint32_t ld_acquire_gpu(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
VE_DEVINL void fence_proxy_async_all() { asm volatile("fence.proxy.async;" ::: "memory"); }

// attention helpers (same fragments as attention.cu)
VE_DEVINL void ds_ldsm_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
VE_DEVINL void ds_ldsm_x4_t(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
VE_DEVINL void ds_mma_bf16(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
VE_DEVINL uint32_t ds_pack(float lo, float hi) {
  __nv_bfloat162 t = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&t);
}
VE_DEVINL void bar_compute() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

struct Ctx {
  const StepParams* p;
  uint8_t* smem;
  uint8_t* scratch;
  uint64_t *tfull, *bfull, *empty, *acc_full, *acc_empty;
  volatile int* s_fail;
  int cta, G;
  VE_DEVINL uint8_t* stage(int s) const { return smem + (size_t)s * DS_STAGE; }
  VE_DEVINL bool failed() const { return *s_fail != 0; }
  VE_DEVINL void fail() const { *s_fail = 1; }
  // bounded waits that give up at once after a failure anywhere in the CTA
  VE_DEVINL bool wait_bar(uint64_t* bar, uint32_t parity) const {
    if (failed()) return false;
    if (mbar_wait(bar, parity)) return true;
    fail();
    return false;
  }
  VE_DEVINL bool wait_cnt(const uint32_t* c, uint32_t target) const {
    if (failed()) return false;
    if ((int)(ld_acquire_gpu(c) - target) >= 0) return true;
    const uint64_t t0 = globaltimer_ns();
    for (;;) {
#pragma unroll 1
      for (int i = 0; i < 16; ++i)
        if ((int)(ld_acquire_gpu(c) - target) >= 0) return true;
      if (globaltimer_ns() - t0 > kWaitNs || failed()) { fail(); return false; }
    }
  }
};

VE_DEVINL int ds_kt(const StepOp& op) { return (op.K + 255) >> 8; }
VE_DEVINL void ds_run(const StepOp& op, int cta, int& u0, int& u1) {
  const int U = (op.N >> 7) * ds_kt(op);
  u0 = min(U, cta * op.upc);
  u1 = min(U, u0 + op.upc);
}
// CTAs that share tile t of op: first CTA and count
VE_DEVINL void ds_splits(const StepOp& op, int t, int& first, int& n) {
  const int KT = ds_kt(op);
  first = (t * KT) / op.upc;
  n = ((t + 1) * KT - 1) / op.upc - first + 1;
}

// key pages of attention item `it` of this step: rows x kv heads x S splits
struct AttnItem { int row, kvh, z, slot, pos, kt0, kt1; };
VE_DEVINL AttnItem ds_item(const StepParams& p, int it) {
  AttnItem a;
  a.row = it / (p.nkv * p.S);
  a.kvh = (it / p.S) % p.nkv;
  a.z = it % p.S;
  a.slot = p.slot ? p.slot[a.row] : 0;
  a.pos = p.pos[a.row];
  const int npages = a.slot >= 0 ? a.pos / 64 + 1 : 0;
  const int tps = (npages + p.S - 1) / p.S;
  a.kt0 = min(npages, a.z * tps);
  a.kt1 = min(npages, a.kt0 + tps);
  return a;
}
VE_DEVINL int ds_attn_tiles(const StepParams& p, int cta, int G) {
  const int items = p.M * p.nkv * p.S;
  int n = 0;
  for (int it = cta; it < items; it += G) {
    const AttnItem a = ds_item(p, it);
    n += 2 * (a.kt1 - a.kt0);
  }
  return n;
}

// ------------------------------------------------------------------------------------------------ loader (warp 0, lane 0)
VE_DEVINL void ds_loader(const Ctx& c) {
  const StepParams& p = *c.p;
  uint32_t r = 0;
  for (int oi = 0; oi < p.nops && !c.failed(); ++oi) {
    const StepOp& op = p.ops[oi];
    if (op.type == OP_LINEAR) {
      int u0, u1;
      ds_run(op, c.cta, u0, u1);
      const CUtensorMap* map = p.maps + op.map;
      const int KT = ds_kt(op), nkg = KT * 4;
      for (int u = u0; u < u1; ++u, ++r) {
        const int s = r % DS_NS;
        if (!c.wait_bar(&c.empty[s], ((r / DS_NS) & 1) ^ 1)) return;
        const int tile = u / KT, kt = u % KT;
        uint8_t* st = c.stage(s);
        mbar_expect_tx(&c.tfull[s], DS_A + DS_SF);
        tma_load_2d(st, map, &c.tfull[s], kt * 128, tile * 128);
        bulk_load(st + DS_A + DS_B, op.sfa + ((size_t)tile * nkg + kt * 4) * 512, DS_SF, &c.tfull[s]);
      }
    } else if (op.type == OP_ATTN) {
      const int items = p.M * p.nkv * p.S;
      int pos_min = 0x7fffffff;
      for (int m = 0; m < p.M; ++m)
        if (!p.slot || p.slot[m] >= 0) pos_min = min(pos_min, p.pos[m]);
      const int safe_end = pos_min / 64;        // pages below hold tokens of earlier steps only
      bool fresh = false;
      for (int it = c.cta; it < items; it += c.G) {
        const AttnItem a = ds_item(p, it);
        for (int kt = a.kt0; kt < a.kt1; ++kt) {
          if (kt >= safe_end && !fresh) {
            // this page receives the step's own keys: wait until the finalise stage has stored them
            if (!c.wait_cnt(p.cnt + op.src, p.ops[op.src].ncontrib)) return;
            fence_proxy_async_all();
            fresh = true;
          }
          const int page = p.page_table[(long)a.slot * p.max_pages + kt];
          const int row = (int)(op.layer * p.pool_layer_rows) + (page * p.nkv + a.kvh) * 64;
          for (int kv = 0; kv < 2; ++kv, ++r) {
            const int s = r % DS_NS;
            if (!c.wait_bar(&c.empty[s], ((r / DS_NS) & 1) ^ 1)) return;
            uint8_t* st = c.stage(s);
            const CUtensorMap* map = p.maps + (kv ? p.vmap : p.kmap);
            mbar_expect_tx(&c.tfull[s], DS_A);
            tma_load_2d(st, map, &c.tfull[s], 0, row);
            tma_load_2d(st + 8192, map, &c.tfull[s], 64, row);
          }
        }
      }
    }
  }
}

// ------------------------------------------------------------------------------------------------ MMA issuer (warp 1, lane 0)
VE_DEVINL void ds_mma(const Ctx& c, uint32_t tmem_base) {
  const StepParams& p = *c.p;
  constexpr uint32_t idesc = make_idesc_nvf4(128, 16);
  const uint32_t tmem_sfa = tmem_base + 64, tmem_sfb = tmem_base + 80;
  uint32_t r = 0, seg = 0;
  for (int oi = 0; oi < p.nops && !c.failed(); ++oi) {
    const StepOp& op = p.ops[oi];
    if (op.type == OP_ATTN) { r += ds_attn_tiles(p, c.cta, c.G); continue; }
    if (op.type != OP_LINEAR) continue;
    int u0, u1;
    ds_run(op, c.cta, u0, u1);
    const int KT = ds_kt(op);
    for (int u = u0; u < u1; ++u, ++r) {
      const int s = r % DS_NS, kt = u % KT;
      const uint32_t buf = seg & 1;
      const bool first = kt == 0 || u == u0;
      if (first && !c.wait_bar(&c.acc_empty[buf], ((seg >> 1) & 1) ^ 1)) return;
      if (!c.wait_bar(&c.tfull[s], (r / DS_NS) & 1)) return;
      if (!c.wait_bar(&c.bfull[s], (r / DS_NS) & 1)) return;
      tc_fence_after();
      uint8_t* st = c.stage(s);
      const uint32_t sfa_s = smem_u32(st + DS_A + DS_B), sfb_s = sfa_s + DS_SF;
#pragma unroll
      for (int kb = 0; kb < 4; ++kb) {
        tc_cp_sf(tmem_sfa + kb * 4, make_desc_sf(sfa_s + kb * 512));
        tc_cp_sf(tmem_sfb + kb * 4, make_desc_sf(sfb_s + kb * 512));
      }
      const uint64_t ad = make_desc_sw128(smem_u32(st)), bd = make_desc_sw128(smem_u32(st + DS_A));
#pragma unroll
      for (int kb = 0; kb < 4; ++kb)
        tc_mma_nvf4(tmem_base + buf * 32, ad + kb * 2, bd + kb * 2, idesc, (first && kb == 0) ? 0u : 1u,
                    tmem_sfa + kb * 4, tmem_sfb + kb * 4);
      tc_commit(&c.empty[s]);
      if (kt == KT - 1 || u == u1 - 1) { tc_commit(&c.acc_full[buf]); ++seg; }
    }
  }
}

// ------------------------------------------------------------------------------------------------ compute warps (2..5)
struct Cw {
  int ctid, cw, lane, q;       // thread 0..127, warp 0..3, lane, TMEM lane quarter
  float* s_rs;                 // [MAXM] row scales of the current normalised input
  float* s_red;                // [16]
  int* s_flag;
  int* s_ok;                   // [4] outcome of a wait / stop flag, published by thread 0 so that all 128 threads agree
  int nwait;                   // waits so far (same in every thread): picks the slot of s_ok
};

VE_DEVINL void ld8(const __nv_bfloat16* src, float* r) {
  const bf16x8 t = *reinterpret_cast<const bf16x8*>(src);
#pragma unroll
  for (int j = 0; j < 4; ++j) { const float2 f = __bfloat1622float2(t.v[j]); r[2 * j] = f.x; r[2 * j + 1] = f.y; }
}
VE_DEVINL void ld8_cg(const __nv_bfloat16* src, float* r) {
  const uint4 raw = __ldcg(reinterpret_cast<const uint4*>(src));
  const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w[j]));
    r[2 * j] = f.x; r[2 * j + 1] = f.y;
  }
}
VE_DEVINL uint4 pack8(const float* r) {
  return make_uint4(ds_pack(r[0], r[1]), ds_pack(r[2], r[3]), ds_pack(r[4], r[5]), ds_pack(r[6], r[7]));
}

// all 128 compute threads wait for `need` arrivals on the counter of op `oi`
// (the outcome goes through shared memory: threads that sampled the failure flag themselves could disagree and part ways
// in front of a named barrier)
VE_DEVINL bool cw_wait_op(const Ctx& c, Cw& w, int oi, uint32_t need) {
  const int slot = w.nwait++ & 1;
  if (w.ctid == 0) {
    w.s_ok[slot] = c.wait_cnt(c.p->cnt + oi, need) ? 1 : 0;
    __threadfence();
  }
  bar_compute();
  return w.s_ok[slot] != 0;
}
VE_DEVINL void cw_signal(const Ctx& c, const Cw& w, int oi) {
  __threadfence();
  bar_compute();
  if (w.ctid == 0) atomicAdd(c.p->cnt + oi, 1u);
}

// Input of a linear: what every unit's B-operand fill reads.
VE_DEVINL void cw_prologue(const Ctx& c, Cw& w, const StepOp& op) {
  const StepParams& p = *c.p;
  const int H = p.H;
  __nv_bfloat16* hrow = reinterpret_cast<__nv_bfloat16*>(c.scratch);
  if (op.in_mode == IN_X || op.in_mode == IN_GATED) {
    cw_wait_op(c, w, op.src, p.ops[op.src].ncontrib);
    return;
  }
  if (op.in_mode == IN_NORM) cw_wait_op(c, w, op.src, p.ops[op.src].ncontrib);
  const __nv_bfloat16* hin = p.hbuf + (size_t)op.hpar * DS_MAXM * H;
  __nv_bfloat16* hout = p.hbuf + (size_t)(op.hpar ^ 1) * DS_MAXM * H;
  const __nv_bfloat16* y = op.in_mode == IN_NORM ? p.ybuf + (size_t)p.ops[op.src].ypar * DS_MAXM * H : nullptr;
  for (int m = 0; m < p.M; ++m) {
    float ss = 0.f;
    int id = 0;
    if (op.in_mode == IN_EMBED) { id = p.ids[m]; id = id < 0 ? 0 : (id >= p.vocab ? p.vocab - 1 : id); }
    for (int i = w.ctid * 8; i < H; i += 1024) {
      float v[8];
      if (op.in_mode == IN_EMBED) {
        ld8(p.embed + (size_t)id * H + i, v);
        if (p.embed_scale != 1.f) {
#pragma unroll
          for (int j = 0; j < 8; ++j) v[j] = round_bf16(v[j] * p.embed_scale);
        }
      } else {
        float a[8];
        ld8_cg(hin + (size_t)m * H + i, v);
        ld8_cg(y + (size_t)m * H + i, a);
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] = round_bf16(v[j] + a[j]);
      }
      const uint4 o = pack8(v);
      *reinterpret_cast<uint4*>(hrow + (size_t)m * H + i) = o;
      if (c.cta == 0) *reinterpret_cast<uint4*>(hout + (size_t)m * H + i) = o;
#pragma unroll
      for (int j = 0; j < 8; ++j) ss = fmaf(v[j], v[j], ss);
    }
    ss = warp_sum(ss);
    if (w.lane == 0) w.s_red[w.cw * DS_MAXM + m] = ss;
  }
  bar_compute();
  if (w.ctid < p.M) {
    const int m = w.ctid;
    const float ss = w.s_red[m] + w.s_red[DS_MAXM + m] + w.s_red[2 * DS_MAXM + m] + w.s_red[3 * DS_MAXM + m];
    w.s_rs[m] = rsqrtf(ss / (float)H + p.eps);
  }
  bar_compute();
  if ((op.flags & 1) && c.cta == 0) {
    for (int m = 0; m < p.M; ++m) {
      const float rs = w.s_rs[m];
      for (int i = w.ctid * 8; i < H; i += 1024) {
        float v[8], g[8];
        ld8(hrow + (size_t)m * H + i, v);
        ld8(op.norm_w + i, g);
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] = v[j] * rs * (g[j] + p.wbias);
        *reinterpret_cast<uint4*>(p.xfinal + (size_t)m * H + i) = pack8(v);
      }
    }
  }
}

VE_DEVINL float ds_act(float g, float u, int act, float limit) {
  if (limit > 0.f) { g = fminf(g, limit); u = fminf(fmaxf(u, -limit), limit); }
  const float a = act == 1 ? g / (1.f + __expf(-g))
                           : 0.5f * g * (1.f + tanhf(0.7978845608028654f * (g + 0.044715f * g * g * g)));
  return a * u;
}

// B operand of unit u (ring index r): warp-wide, lane = (16-element block, half)
VE_DEVINL void cw_bfill(const Ctx& c, const Cw& w, const StepOp& op, int u, uint32_t r) {
  const StepParams& p = *c.p;
  const int s = r % DS_NS;
  int ok = 1;
  if (w.lane == 0) ok = c.wait_bar(&c.empty[s], ((r / DS_NS) & 1) ^ 1) ? 1 : 0;
  if (!__shfl_sync(0xffffffffu, ok, 0)) return;
  const int KT = ds_kt(op), kt = u % KT;
  const int b = w.lane >> 1, hf = w.lane & 1;
  const int k = kt * 256 + b * 16 + hf * 8;
  uint8_t* bt = c.stage(s) + DS_A;
  uint8_t* sf = bt + DS_B + DS_SF;
  const __nv_bfloat16* hrow = reinterpret_cast<const __nv_bfloat16*>(c.scratch);
  for (int m = 0; m < p.M; ++m) {
    float x[8];
    if (k >= op.K) {
#pragma unroll
      for (int j = 0; j < 8; ++j) x[j] = 0.f;
    } else if (op.in_mode == IN_X) {
      ld8_cg(p.attn_out + (size_t)m * op.K + k, x);
    } else if (op.in_mode == IN_GATED) {
      const StepOp& so = p.ops[op.src];
      const int t = k >> 6, f0 = k & 63;
      int first, n;
      ds_splits(so, t, first, n);
      float g[8], up[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) g[j] = up[j] = 0.f;
      for (int sp = 0; sp < n; ++sp) {
        const float* base = p.ws + so.ws_off + ((size_t)(t * so.ms + sp) * DS_MAXM + m) * 128 + f0;
        const float4 g0 = __ldcg(reinterpret_cast<const float4*>(base)), g1 = __ldcg(reinterpret_cast<const float4*>(base + 4));
        const float4 u0 = __ldcg(reinterpret_cast<const float4*>(base + 64)), u1 = __ldcg(reinterpret_cast<const float4*>(base + 68));
        g[0] += g0.x; g[1] += g0.y; g[2] += g0.z; g[3] += g0.w; g[4] += g1.x; g[5] += g1.y; g[6] += g1.z; g[7] += g1.w;
        up[0] += u0.x; up[1] += u0.y; up[2] += u0.z; up[3] += u0.w; up[4] += u1.x; up[5] += u1.y; up[6] += u1.z; up[7] += u1.w;
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) x[j] = round_bf16(ds_act(g[j] * so.alpha, up[j] * so.alpha, p.act, p.act_limit));
    } else {
      float g[8];
      ld8(hrow + (size_t)m * p.H + k, x);
      ld8(op.norm_w + k, g);
      const float rs = w.s_rs[m];
#pragma unroll
      for (int j = 0; j < 8; ++j) x[j] = round_bf16(x[j] * rs * (g[j] + p.wbias));
    }
    uint32_t codes[DS_TERMS], sc[DS_TERMS];
    expand_half8<DS_TERMS>(x, codes, sc);
#pragma unroll
    for (int t = 0; t < DS_TERMS; ++t) {
      const int v = m * DS_TERMS + t;
      *reinterpret_cast<uint32_t*>(bt + v * 128 + (((b >> 1) ^ (v & 7)) << 4) + (b & 1) * 8 + hf * 4) = codes[t];
      if (hf == 0) sf[(b >> 2) * 512 + (v & 31) * 16 + (v >> 5) * 4 + (b & 3)] = (uint8_t)sc[t];
    }
  }
  fence_proxy_async_smem();
  __syncwarp();
  if (w.lane == 0) mbar_arrive(&c.bfull[s]);
}

VE_DEVINL uint4 ds_ld_volatile_v4(const void* ptr) {
  uint4 v;
  asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(ptr)
               : "memory");
  return v;
}

// Epilogue of the segment that ends at unit j (tile t): TMEM lane = feature, column m * TERMS + term.
VE_DEVINL void cw_epilogue(const Ctx& c, const Cw& w, const StepOp& op, int oi, int j, uint32_t seg, uint32_t tmem_base) {
  const StepParams& p = *c.p;
  const int KT = ds_kt(op), t = j / KT;
  const uint32_t buf = seg & 1;
  const int f = w.q * 32 + w.lane, n = t * 128 + f;
  const bool ok = c.wait_bar(&c.acc_full[buf], (seg >> 1) & 1);
  tc_fence_after();
  float acc[DS_MAXM] = {0.f, 0.f, 0.f, 0.f};
  if (ok) {
    uint32_t r[16];
    tmem_ld16(tmem_base + ((uint32_t)(w.q * 32) << 16) + buf * 32, r);
    tmem_ld_wait();
#pragma unroll
    for (int m = 0; m < DS_MAXM; ++m) {
      float v = 0.f, s = 1.f;
#pragma unroll
      for (int tt = 0; tt < DS_TERMS; ++tt) { v = fmaf(__uint_as_float(r[m * DS_TERMS + tt]), s, v); s *= 0.125f; }
      acc[m] = v;
    }
  }
  tc_fence_before();
  bar_compute();
  if (w.ctid == 0) mbar_arrive(&c.acc_empty[buf]);
  int first, nsp;
  ds_splits(op, t, first, nsp);
  const int sp = c.cta - first;
  if (op.out_mode == OUT_LOGITS) {
    for (int m = 0; m < p.M; ++m) p.logits[(long)m * p.ldl + n] = acc[m] * op.alpha;
    return;
  }
  float* mine = p.ws + op.ws_off + ((size_t)(t * op.ms + sp) * DS_MAXM) * 128 + f;
  if (op.out_mode == OUT_PART) {
    for (int m = 0; m < p.M; ++m) mine[m * 128] = acc[m];
    return;
  }
  // OUT_TICKET: the CTA that arrives last on the tile adds the splits in order and publishes the rows
  bool last = true;
  if (nsp > 1) {
    for (int m = 0; m < p.M; ++m) mine[m * 128] = acc[m];
    __threadfence();
    bar_compute();
    if (w.ctid == 0) *w.s_flag = atomicAdd(p.tickets + op.tk_off + t, 1);
    bar_compute();
    last = *w.s_flag == nsp - 1;
    if (last) {
      __threadfence();
      const float* all = p.ws + op.ws_off + ((size_t)(t * op.ms) * DS_MAXM) * 128 + f;
      for (int m = 0; m < p.M; ++m) {
        float s = 0.f;
        for (int k2 = 0; k2 < nsp; ++k2) s += __ldcg(all + ((size_t)k2 * DS_MAXM + m) * 128);
        acc[m] = s;
      }
      if (w.ctid == 0) p.tickets[op.tk_off + t] = 0;
    }
  }
  if (!last) return;
  __nv_bfloat16* y = p.ybuf + (size_t)op.ypar * DS_MAXM * p.H;
  if (p.size > 1) {
    const uint32_t seq = p.seq[0] + (uint32_t)op.ar;
    const int stg = seq & 3;
    for (int m = 0; m < p.M; ++m) {
      const float mine_v = round_bf16(acc[m] * op.alpha);
      const uint32_t bits = (uint32_t)__bfloat16_as_ushort(f2bf(mine_v));
      const uint32_t b1 = __shfl_down_sync(0xffffffffu, bits, 1), b2 = __shfl_down_sync(0xffffffffu, bits, 2),
                     b3 = __shfl_down_sync(0xffffffffu, bits, 3);
      float tot[4] = {0.f, 0.f, 0.f, 0.f};
      if ((w.lane & 3) == 0) {
        const size_t line = (size_t)(n >> 2) * 16;
        const size_t slot_me = p.off_ll + ((size_t)(stg * p.size + p.rank) * 16 + m) * p.ll_row_bytes + line;
        const uint4 pkt = make_uint4(bits | (b1 << 16), seq, b2 | (b3 << 16), seq);
        for (int i = 1; i < p.size; ++i) {
          uint8_t* dst = p.peer[(p.rank + i) % p.size] + slot_me;
          asm volatile("st.volatile.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(dst), "r"(pkt.x), "r"(pkt.y), "r"(pkt.z),
                       "r"(pkt.w) : "memory");
        }
        for (int src = 0; src < p.size; ++src) {
          uint32_t d0 = pkt.x, d1 = pkt.z;
          if (src != p.rank) {
            const uint8_t* lp = p.peer[p.rank] + p.off_ll + ((size_t)(stg * p.size + src) * 16 + m) * p.ll_row_bytes + line;
            uint4 v = ds_ld_volatile_v4(lp);
            if (!(v.y == seq && v.w == seq) && !c.failed()) {
              const uint64_t t0 = globaltimer_ns();
              for (;;) {
                v = ds_ld_volatile_v4(lp);
                if (v.y == seq && v.w == seq) break;
                if (globaltimer_ns() - t0 > p.budget_ns || c.failed()) {
                  c.fail();
                  if (p.status) atomicExch(p.status, (int)kErrPeerTimeout);
                  break;
                }
              }
            }
            d0 = v.x; d1 = v.z;
          }
          tot[0] += __uint_as_float(d0 << 16);
          tot[1] += __uint_as_float(d0 & 0xffff0000u);
          tot[2] += __uint_as_float(d1 << 16);
          tot[3] += __uint_as_float(d1 & 0xffff0000u);
        }
        *reinterpret_cast<uint2*>(y + (size_t)m * p.H + n) = make_uint2(ds_pack(tot[0], tot[1]), ds_pack(tot[2], tot[3]));
      }
    }
  } else {
    for (int m = 0; m < p.M; ++m) y[(size_t)m * p.H + n] = f2bf(acc[m] * op.alpha);
  }
  cw_signal(c, w, oi);
}

// One head per CTA: split sum, rotary embedding, q to qbuf, k / v into the paged cache.
VE_DEVINL void cw_qkv_fin(const Ctx& c, Cw& w, const StepOp& op, int oi) {
  const StepParams& p = *c.p;
  const StepOp& so = p.ops[op.src];
  const int heads = p.nq + 2 * p.nkv;
  if (c.cta >= heads) return;
  if (!cw_wait_op(c, w, op.src, so.ncontrib)) return;
  float* sb = reinterpret_cast<float*>(c.scratch);
  const int f = w.ctid;
  for (int head = c.cta; head < heads; head += c.G) {
    int first, nsp;
    ds_splits(so, head, first, nsp);
    for (int m = 0; m < p.M; ++m) {
      float s = 0.f;
      for (int sp = 0; sp < nsp; ++sp) s += __ldcg(p.ws + so.ws_off + ((size_t)(head * so.ms + sp) * DS_MAXM + m) * 128 + f);
      sb[m * 128 + f] = round_bf16(s * so.alpha);
    }
    bar_compute();
    if (f < 64) {
      const int half = p.rot >> 1;
      const bool is_v = head >= p.nq + p.nkv, is_k = !is_v && head >= p.nq;
      int i0, i1;
      if (is_v) { i0 = 2 * f; i1 = i0 + 1; }
      else if (f < half) { i0 = f; i1 = f + half; }
      else { i0 = p.rot + 2 * (f - half); i1 = i0 + 1; }
      const float inv_freq = exp2f(-log2f(p.rope_theta) * (2.f * (float)f / (float)p.rot));
      for (int m = 0; m < p.M; ++m) {
        float a0 = sb[m * 128 + i0], a1 = sb[m * 128 + i1];
        const int ps = p.pos[m];
        const int sl = p.slot ? p.slot[m] : 0;
        if (!is_v && f < half && !(is_k && sl < 0)) {
          float sn, cs;
          sincosf((float)ps * inv_freq, &sn, &cs);
          const float r0 = a0 * cs - a1 * sn, r1 = a1 * cs + a0 * sn;
          a0 = r0;
          a1 = r1;
        }
        const __nv_bfloat16 b0 = f2bf(a0), b1 = f2bf(a1);
        if (!is_k && !is_v) {
          p.qbuf[(size_t)m * p.nq * 128 + head * 128 + i0] = b0;
          p.qbuf[(size_t)m * p.nq * 128 + head * 128 + i1] = b1;
        } else if (sl >= 0) {
          const int kvh = head - p.nq - (is_v ? p.nkv : 0);
          const int page = p.page_table[(long)sl * p.max_pages + ps / 64];
          const long dst = ((long)op.layer * p.pool_layer_rows + ((long)page * p.nkv + kvh) * 64 + (ps % 64)) * 128;
          __nv_bfloat16* pool = is_v ? p.vpool : p.kpool;
          pool[dst + i0] = b0;
          pool[dst + i1] = b1;
        }
      }
    }
    bar_compute();
  }
  fence_proxy_async_all();     // the cache rows are read back through TMA by other CTAs
  cw_signal(c, w, oi);
}

// Split-KV attention of this CTA's (row, kv head, split) items: each warp scores its own 16 keys of every page.
VE_DEVINL void cw_attn(const Ctx& c, Cw& w, const StepOp& op, int oi, uint32_t& r) {
  const StepParams& p = *c.p;
  const int items = p.M * p.nkv * p.S;
  if (c.cta >= items) return;
  if (!cw_wait_op(c, w, op.src, p.ops[op.src].ncontrib)) return;
  const int G = p.nq / p.nkv;
  const int lane = w.lane, g = lane >> 2, t4 = lane & 3;
  float* ms = reinterpret_cast<float*>(c.scratch);     // [4][16]
  float* ls = ms + 64;                                   // [4][16]
  float* os = ls + 64;                                   // [4][16][128]
  for (int it = c.cta; it < items; it += c.G) {
    const AttnItem a = ds_item(p, it);
    bool r_ok[2];
    int r_head[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int rr = g + h * 8;
      r_ok[h] = rr < G;
      r_head[h] = a.kvh * G + (r_ok[h] ? rr : 0);
    }
    uint32_t qf[8][4];
#pragma unroll
    for (int kk = 0; kk < 8; ++kk) {
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const __nv_bfloat16* qr = p.qbuf + (size_t)a.row * p.nq * 128 + (size_t)r_head[h] * 128 + kk * 16 + 2 * t4;
        qf[kk][h] = r_ok[h] ? __ldcg(reinterpret_cast<const uint32_t*>(qr)) : 0u;
        qf[kk][2 + h] = r_ok[h] ? __ldcg(reinterpret_cast<const uint32_t*>(qr + 8)) : 0u;
      }
    }
    float o[16][4];
#pragma unroll
    for (int i = 0; i < 16; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    float m_run[2] = {-FLT_MAX, -FLT_MAX}, l_run[2] = {0.f, 0.f};
    const int key0 = w.cw * 16;
    for (int kt = a.kt0; kt < a.kt1; ++kt) {
      // K page
      const int sk = r % DS_NS;
      const bool okk = c.wait_bar(&c.tfull[sk], (r / DS_NS) & 1);
      const uint32_t kb = smem_u32(c.stage(sk));
      float sacc[2][4];
#pragma unroll
      for (int i = 0; i < 2; ++i) sacc[i][0] = sacc[i][1] = sacc[i][2] = sacc[i][3] = 0.f;
      if (okk) {
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          const int cch = (kk * 16) / 64, ci = ((kk * 16) % 64) / 8;
          const int mi = lane >> 3, rr = lane & 7;
          const int key = key0 + (mi >> 1) * 8 + rr;
          const int ch = ci + (mi & 1);
          uint32_t b0, b1, b2, b3;
          ds_ldsm_x4(kb + cch * 8192 + key * 128 + ((ch ^ (key & 7)) << 4), b0, b1, b2, b3);
          ds_mma_bf16(sacc[0], qf[kk], b0, b1);
          ds_mma_bf16(sacc[1], qf[kk], b2, b3);
        }
      }
      bar_compute();
      if (w.ctid == 0) { mbar_arrive(&c.bfull[sk]); mbar_arrive(&c.empty[sk]); }   // (bfull keeps one phase per ring pass)
      ++r;
      float mx[2] = {-FLT_MAX, -FLT_MAX};
#pragma unroll
      for (int nt = 0; nt < 2; ++nt) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int h = e >> 1;
          const int key = kt * 64 + key0 + nt * 8 + 2 * t4 + (e & 1);
          const bool allow = r_ok[h] && key <= a.pos;
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
      uint32_t pf[4];
#pragma unroll
      for (int nt = 0; nt < 2; ++nt) {
        float pv[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int h = e >> 1;
          pv[e] = (sacc[nt][e] == -FLT_MAX) ? 0.f : exp2f(sacc[nt][e] - m_run[h]);
          l_run[h] += pv[e];
        }
        pf[nt * 2 + 0] = ds_pack(pv[0], pv[1]);
        pf[nt * 2 + 1] = ds_pack(pv[2], pv[3]);
      }
#pragma unroll
      for (int i = 0; i < 16; ++i) { o[i][0] *= corr[0]; o[i][1] *= corr[0]; o[i][2] *= corr[1]; o[i][3] *= corr[1]; }
      // V page
      const int sv = r % DS_NS;
      const bool okv = c.wait_bar(&c.tfull[sv], (r / DS_NS) & 1);
      const uint32_t vb = smem_u32(c.stage(sv));
      if (okv) {
#pragma unroll
        for (int dp = 0; dp < 8; ++dp) {
          const int mi = lane >> 3, rr = lane & 7;
          const int key = key0 + (mi & 1) * 8 + rr;
          const int d = dp * 16 + (mi >> 1) * 8;
          const int cch = d / 64, ch = (d % 64) / 8;
          uint32_t b0, b1, b2, b3;
          ds_ldsm_x4_t(vb + cch * 8192 + key * 128 + ((ch ^ (key & 7)) << 4), b0, b1, b2, b3);
          ds_mma_bf16(o[2 * dp], pf, b0, b1);
          ds_mma_bf16(o[2 * dp + 1], pf, b2, b3);
        }
      }
      bar_compute();
      if (w.ctid == 0) { mbar_arrive(&c.bfull[sv]); mbar_arrive(&c.empty[sv]); }
      ++r;
    }
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 1);
      l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 2);
    }
    // merge the four warps' states through the scratch area
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int row = g + h * 8;
      if (t4 == 0) { ms[w.cw * 16 + row] = m_run[h]; ls[w.cw * 16 + row] = l_run[h]; }
      if (row < G) {
#pragma unroll
        for (int nt = 0; nt < 16; ++nt)
          *reinterpret_cast<float2*>(os + (size_t)(w.cw * 16 + row) * 128 + nt * 8 + 2 * t4) =
              make_float2(o[nt][2 * h], o[nt][2 * h + 1]);
      }
    }
    bar_compute();
    for (int idx = w.ctid; idx < G * 128; idx += 128) {
      const int row = idx >> 7, d = idx & 127;
      float m = -FLT_MAX;
#pragma unroll
      for (int ww = 0; ww < 4; ++ww) m = fmaxf(m, ms[ww * 16 + row]);
      float acc = 0.f, l = 0.f;
#pragma unroll
      for (int ww = 0; ww < 4; ++ww) {
        const float mw = ms[ww * 16 + row];
        if (mw != -FLT_MAX) {
          const float cc = exp2f(mw - m);
          acc += os[(size_t)(ww * 16 + row) * 128 + d] * cc;
          l += ls[ww * 16 + row] * cc;
        }
      }
      const int head = a.kvh * G + row;
      const long base = ((long)a.row * p.nq + head) * p.S + a.z;
      p.o_part[base * 128 + d] = l > 0.f ? acc / l : 0.f;
      if (d == 0) p.lse_part[base] = l > 0.f ? m + log2f(l) : -FLT_MAX;
    }
    bar_compute();
  }
  cw_signal(c, w, oi);
}

// One (row, head) per CTA: merge the split partials in split order.
VE_DEVINL void cw_merge(const Ctx& c, Cw& w, const StepOp& op, int oi) {
  const StepParams& p = *c.p;
  const int items = p.M * p.nq;
  if (c.cta >= items) return;
  if (!cw_wait_op(c, w, op.src, p.ops[op.src].ncontrib)) return;
  const int d = w.ctid;
  for (int it = c.cta; it < items; it += c.G) {
    const int row = it / p.nq, head = it % p.nq;
    const long base = ((long)row * p.nq + head) * p.S;
    float mx = -FLT_MAX;
    for (int i = 0; i < p.S; ++i) mx = fmaxf(mx, __ldcg(p.lse_part + base + i));
    float acc = 0.f, wsum = 0.f;
    for (int i = 0; i < p.S; ++i) {
      const float l = __ldcg(p.lse_part + base + i);
      if (l == -FLT_MAX) continue;
      const float wt = exp2f(l - mx);
      wsum += wt;
      acc += wt * __ldcg(p.o_part + (base + i) * 128 + d);
    }
    p.attn_out[(size_t)row * p.nq * 128 + head * 128 + d] = f2bf(wsum > 0.f ? acc / wsum : 0.f);
  }
  cw_signal(c, w, oi);
}

VE_DEVINL void ds_compute(const Ctx& c, Cw& w, uint32_t tmem_base) {
  const StepParams& p = *c.p;
  uint32_t r = 0, seg = 0;
  for (int oi = 0; oi < p.nops; ++oi) {
    // stop after a failure, all 128 threads together
    if (w.ctid == 0) w.s_ok[2 + (oi & 1)] = c.failed() ? 1 : 0;
    bar_compute();
    if (w.s_ok[2 + (oi & 1)]) break;
    const StepOp& op = p.ops[oi];
    if (op.type == OP_QKV_FIN) { cw_qkv_fin(c, w, op, oi); continue; }
    if (op.type == OP_ATTN) { cw_attn(c, w, op, oi, r); continue; }
    if (op.type == OP_MERGE) { cw_merge(c, w, op, oi); continue; }
    if (op.type == OP_NORMOUT) {               // final residual add + norm when the LM head runs outside this kernel
      if (c.cta == 0) cw_prologue(c, w, op);
      continue;
    }
    int u0, u1;
    ds_run(op, c.cta, u0, u1);
    if (u0 >= u1) continue;
    cw_prologue(c, w, op);
    const int KT = ds_kt(op);
    for (int u = u0; u < u1; ++u, ++r) {
      if ((int)(r & 3) == w.cw) cw_bfill(c, w, op, u, r);
      const int j = u - DS_LOOK;
      if (j >= u0 && (j % KT == KT - 1)) cw_epilogue(c, w, op, oi, j, seg++, tmem_base);
    }
    for (int j = max(u0, u1 - DS_LOOK); j < u1; ++j)
      if (j % KT == KT - 1 || j == u1 - 1) cw_epilogue(c, w, op, oi, j, seg++, tmem_base);
    if (op.out_mode == OUT_PART) cw_signal(c, w, oi);
  }
}

__global__ void __launch_bounds__(192, 1) decode_step_kernel(const __grid_constant__ StepParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  __shared__ uint64_t tfull[DS_NS], bfull[DS_NS], empty[DS_NS], acc_full[2], acc_empty[2];
  __shared__ uint32_t tmem_holder;
  __shared__ int s_fail, s_flag, s_last, s_ok[4];
  __shared__ float s_rs[DS_MAXM], s_red[4 * DS_MAXM];

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int s = 0; s < DS_NS; ++s) { mbar_init(&tfull[s], 1); mbar_init(&bfull[s], 1); mbar_init(&empty[s], 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(&acc_full[b], 1); mbar_init(&acc_empty[b], 1); }
    // a status word left set by an earlier failure makes every wait of this launch give up at once
    s_fail = (p.status && *reinterpret_cast<volatile int*>(p.status) != 0) ? 1 : 0;
    mbar_fence_init();
  }
  if (warp == 1) { tmem_alloc(&tmem_holder, DS_TMEM); tmem_relinquish(); }
  if (warp >= 2) {
    // scale bytes of the B rows that no activation row uses stay zero
    const int ctid = threadIdx.x - 64;
    for (int s = 0; s < DS_NS; ++s)
      *reinterpret_cast<uint4*>(smem + (size_t)s * DS_STAGE + DS_A + DS_B + DS_SF + ctid * 16) = make_uint4(0, 0, 0, 0);
    fence_proxy_async_smem();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_holder;
  Ctx c{&p, smem, smem + (size_t)DS_NS * DS_STAGE, tfull, bfull, empty, acc_full, acc_empty, &s_fail,
        (int)blockIdx.x, (int)gridDim.x};
  if (warp == 0) {
    if (lane == 0) ds_loader(c);
  } else if (warp == 1) {
    if (lane == 0) ds_mma(c, tmem_base);
  } else {
    Cw w{(int)threadIdx.x - 64, warp - 2, lane, warp & 3, s_rs, s_red, &s_flag, s_ok, 0};
    ds_compute(c, w, tmem_base);
  }
  tc_fence_before();
  __syncthreads();
  if (s_fail && threadIdx.x == 0) {
    // after a failed wait copies of the loader may still be in flight: give each stage a short time to land
    for (int s = 0; s < DS_NS; ++s) {
      mbar_wait(&tfull[s], 0, 2000000ull);
      mbar_wait(&tfull[s], 1, 2000000ull);
    }
  }
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem_base, DS_TMEM); }
  if (threadIdx.x == 0) {
    if (s_fail && p.status) atomicCAS(p.status, 0, (int)kErrMbarTimeout);
    __threadfence();
    s_last = atomicAdd(p.ctrl, 1u) == gridDim.x - 1 ? 1 : 0;
  }
  __syncthreads();
  if (s_last) {
    // every CTA is done with the counters: leave them zero for the next launch and advance the line sequence
    for (int i = threadIdx.x; i < p.nops; i += blockDim.x) p.cnt[i] = 0;
    if (threadIdx.x == 0) {
      p.ctrl[0] = 0;
      if (p.size > 1) p.seq[0] = p.seq[0] + (uint32_t)p.n_ar;
      __threadfence();
    }
  }
}

}  // namespace ve

using namespace ve;

extern "C" {

int ve_decode_step_sizes(int* out) {
  out[0] = (int)sizeof(StepOp);
  out[1] = (int)sizeof(StepParams);
  out[2] = DS_SMEM;
  out[3] = DS_MAXM;
  return 0;
}

// 128-byte tensor map of a 2-D row-major tensor into host memory `out` (see tmap.h).
int ve_make_tmap_2d(void* out, const void* base, int dtype, int elem_bytes, long rows, long cols, long pitch_bytes,
                    int box_rows, int box_cols, int swizzle128) {
  return make_tmap_2d(reinterpret_cast<CUtensorMap*>(out), base,
                      dtype == 1 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_UINT8, elem_bytes,
                      (uint64_t)rows, (uint64_t)cols, (uint64_t)pitch_bytes, (uint32_t)box_rows, (uint32_t)box_cols,
                      swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE);
}

// params: host copy of StepParams. ctas: one per SM (all must be resident together: cooperative launch).
int ve_decode_step(const void* params, int ctas, int cooperative, cudaStream_t st) {
  const StepParams& p = *reinterpret_cast<const StepParams*>(params);
  if (p.M < 1 || p.M > DS_MAXM || p.H % 8 || (size_t)p.M * p.H * 2 > DS_SCR || p.nq % p.nkv || p.nq / p.nkv > 16 ||
      p.S < 1 || ctas < 1 || p.size < 1 || p.size > 8)
    return cudaErrorInvalidValue;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(decode_step_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, DS_SMEM);
    if (e != cudaSuccess) return (int)e;
    attr_set = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(ctas);
  cfg.blockDim = dim3(192);
  cfg.dynamicSmemBytes = DS_SMEM;
  cfg.stream = st;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeCooperative;
  at[0].val.cooperative = 1;
  cfg.attrs = at;
  cfg.numAttrs = cooperative ? 1 : 0;
  return (int)cudaLaunchKernelEx(&cfg, decode_step_kernel, p);
}

}  // extern "C"
