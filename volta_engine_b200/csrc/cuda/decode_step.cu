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

constexpr int DS_MAXNS = 10;                             // most ring stages (the count follows from the scratch a launch needs)
constexpr int DS_A = 16384, DS_SF = 2048;                // weight tile / its four scale atoms
constexpr int DS_STAGE = DS_A + DS_SF;                   // 18432 B: one unit as it lies in memory (or one K / V page)
constexpr int DS_SLOTS = 20;                             // operand cache: k-tiles of one op a CTA can hold
constexpr int DS_SFB = 256;                              // distance of the four scale atoms of a slot (16 rows used of 32)
constexpr int DS_SLOT = 2048 + 4 * DS_SFB;               // 16 operand rows x 128 B (swizzled) | scale atoms
constexpr int DS_CACHE = DS_SLOTS * DS_SLOT + 512;       // (the last atom is read 256 B past its slot)
constexpr int DS_MAXM = 4;
constexpr int DS_TERMS = 4;
constexpr int DS_TMEM = 256;                             // 2 issuers x 2 accumulators x 32 columns, scale columns from 128
constexpr int DS_SMEM = 226 * 1024;

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
  const uint8_t* wt;           // weight units [N/128][ceil(K/256)][18432]: the 128 x 128 B tile of packed codes as it sits
                               // in swizzled shared memory, followed by its four 512 B scale atoms
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
  unsigned long long* prof;    // optional [nops][4] timestamps (ns) of CTA prof_cta: op entered, input ready, units done, op left
  int* dbg;                    // [0] waits that gave up, then records {site, op, ring index / counter, cta, aux, -} from [8]
  uint8_t* peer[8];
  uint32_t* seq;
  unsigned long long off_ll, ll_row_bytes, budget_ns;
  long ldl, pool_layer_rows;
  int nops, kmap, vmap, M, H, nq, nkv, S, max_pages, vocab, rot, act, rank, size, n_ar, prof_cta, ns, scr;      // ns ring stages, scr scratch bytes
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
  uint8_t* smem;                 // ring stages
  uint8_t* cache;                // operand cache slots
  uint8_t* scratch;
  uint64_t *tfull, *cfull, *empty, *acc_full, *acc_empty;
  int ns;
  volatile int* s_fail;
  volatile uint32_t* attn_seq;   // attention ops this CTA's compute warps have finished
  volatile uint32_t* prog;       // [2] units each issuer has passed
  volatile uint32_t* kv_seq;     // attention items whose new keys / values this CTA has stored
  int cta, G;
  VE_DEVINL uint8_t* stage(int s) const { return smem + (size_t)s * DS_STAGE; }
  VE_DEVINL bool failed() const { return *s_fail != 0; }
  VE_DEVINL void fail() const { *s_fail = 1; }
  // bounded waits that give up at once after a failure anywhere in the CTA
  // the first wait of the launch that runs out of time leaves a record of where it was
  VE_DEVINL void record(int site, int oi, uint32_t r, int aux) const {
    if (!p->dbg) return;
    const int i = atomicAdd(p->dbg, 1);
    if (i < 1000) {
      int* d = p->dbg + 8 + 6 * i;
      d[0] = site; d[1] = oi; d[2] = (int)r; d[3] = cta; d[4] = aux;
    }
  }
  VE_DEVINL bool wait_bar(uint64_t* bar, uint32_t parity, int site = 0, int oi = -1, uint32_t r = 0) const {
    if (mbar_try_wait(bar, parity)) return true;      // the common case costs one instruction
    if (failed()) return false;
    if (mbar_wait(bar, parity)) return true;
    if ((threadIdx.x & 31) == 0) record(failed() ? site + 100 : site, oi, r, (int)parity);
    fail();
    return false;
  }
  VE_DEVINL bool wait_cnt(const uint32_t* c, uint32_t target, int site = 0, int oi = -1) const {
    if (failed()) return false;
    if ((int)(ld_acquire_gpu(c) - target) >= 0) return true;
    const uint64_t t0 = globaltimer_ns();
    for (;;) {
#pragma unroll 1
      for (int i = 0; i < 16; ++i)
        if ((int)(ld_acquire_gpu(c) - target) >= 0) return true;
      if (failed()) { record(site + 100, oi, ld_acquire_gpu(c), (int)target); return false; }
      if (globaltimer_ns() - t0 > kWaitNs) { record(site, oi, ld_acquire_gpu(c), (int)target); fail(); return false; }
    }
  }
};

VE_DEVINL int ds_kt(const StepOp& op) { return (op.K + 255) >> 8; }
VE_DEVINL void ds_run(const StepOp& op, int cta, int& u0, int& u1) {
  const int U = (op.N >> 7) * ds_kt(op);
  u0 = min(U, cta * op.upc);
  u1 = min(U, u0 + op.upc);
}
// Operand cache: the first min(KT, run length) units of a run touch distinct k-tiles; k-tile kt sits in slot
// (kt - first k-tile of the run) mod KT.
VE_DEVINL int ds_nslots(int KT, int u0, int u1) { return min(KT, u1 - u0); }
VE_DEVINL int ds_slot(int KT, int u0, int u) { return (u - u0) % KT; }
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
  uint32_t r = 0, nitems = 0;
  for (int oi = 0; oi < p.nops && !c.failed(); ++oi) {
    const StepOp& op = p.ops[oi];
    if (op.type == OP_LINEAR) {
      int u0, u1;
      ds_run(op, c.cta, u0, u1);
      // a CTA's run of units is one contiguous stretch of memory: pure sequential streaming
      const uint8_t* wt = op.wt;
      for (int u = u0; u < u1; ++u, ++r) {
        const int s = r % c.ns;
        if (!c.wait_bar(&c.empty[s], ((r / c.ns) & 1) ^ 1, 1, oi, r)) return;
        mbar_expect_tx(&c.tfull[s], DS_A + DS_SF);
        bulk_load(c.stage(s), wt + (size_t)u * (DS_A + DS_SF), DS_A + DS_SF, &c.tfull[s]);
      }
    } else if (op.type == OP_ATTN) {
      const int items = p.M * p.nkv * p.S;
      int pos_min = 0x7fffffff;
      for (int m = 0; m < p.M; ++m)
        if (!p.slot || p.slot[m] >= 0) pos_min = min(pos_min, p.pos[m]);
      const int safe_end = pos_min / 64;        // pages below hold tokens of earlier steps only
      for (int it = c.cta; it < items; it += c.G) {
        const AttnItem a = ds_item(p, it);
        ++nitems;
        bool fresh = false;
        for (int kt = a.kt0; kt < a.kt1; ++kt) {
          if (kt >= safe_end && !fresh) {
            // this page receives the step's own keys: the compute warps of this CTA store them (from the qkv partial
            // sums) before they start on the item, and say so through shared memory
            const uint64_t t0 = globaltimer_ns();
            while ((int)(*c.kv_seq - nitems) < 0) {
              if (c.failed()) return;
              if (globaltimer_ns() - t0 > kWaitNs) { c.record(2, oi, r, (int)nitems); c.fail(); return; }
            }
            fence_proxy_async_all();
            fresh = true;
          }
          const int page = p.page_table[(long)a.slot * p.max_pages + kt];
          const int row = (int)(op.layer * p.pool_layer_rows) + (page * p.nkv + a.kvh) * 64;
          for (int kv = 0; kv < 2; ++kv, ++r) {
            const int s = r % c.ns;
            if (!c.wait_bar(&c.empty[s], ((r / c.ns) & 1) ^ 1, 3, oi, r)) return;
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

// ------------------------------------------------------------------------------------------------ MMA issuers (warps 1 and 6, lane 0)
// Two issuer threads share the units of every run by unit parity, each with its own accumulators and scale columns: one
// thread's issue rate (about 65 cycles per tcgen05 instruction, thirteen of them per 18 KB unit) is half of what the weight
// stream needs. The epilogue adds the two accumulators in a fixed order, and the parity is that of the unit's index in
// the op, so the grouping of the sum does not depend on what ran before.
VE_DEVINL void ds_mma(const Ctx& c, uint32_t tmem_base, int which) {
  const StepParams& p = *c.p;
  constexpr uint32_t idesc = make_idesc_nvf4(128, 16);
  const uint32_t tmem_acc = tmem_base + which * 64;
  const uint32_t tmem_sfa = tmem_base + 128 + which * 32, tmem_sfb = tmem_sfa + 16;
  const uint32_t ring_s = smem_u32(c.smem), cache_s = smem_u32(c.cache);
  uint32_t r = 0, seg = 0, na = 0;
  uint32_t g = 0;               // units passed so far (same count in both issuers)
  uint32_t cpar = 0;            // phase parity of every cache slot's barrier (a slot is filled once per op that uses it)
  for (int oi = 0; oi < p.nops && !c.failed(); ++oi) {
    const StepOp& op = p.ops[oi];
    if (op.type == OP_ATTN) {
      // The issuers take no part in attention, but they must not run ahead of it: a parity wait cannot tell a stage's
      // phase from the one two ring passes earlier, so they wait here until the compute warps have used up the op's pages.
      if (c.cta < p.M * p.nkv * p.S) {
        ++na;
        const uint64_t t0 = globaltimer_ns();
        while ((int)(*c.attn_seq - na) < 0) {
          if (c.failed()) return;
          if (globaltimer_ns() - t0 > kWaitNs) { c.record(13, oi, r, (int)na); c.fail(); return; }
        }
      }
      r += ds_attn_tiles(p, c.cta, c.G);
      continue;
    }
    if (op.type != OP_LINEAR) continue;
    int u0, u1;
    ds_run(op, c.cta, u0, u1);
    if (u0 >= u1) continue;
    const int KT = ds_kt(op);
    const int nslots = ds_nslots(KT, u0, u1);
    int kt = u0 % KT, slot = 0;
    const uint32_t g0 = g;
    bool seg_start = true, issued = false;
    for (int u = u0; u < u1; ++u, ++r) {
      const uint32_t buf = seg & 1;
      if (seg_start) {
        // the epilogue warps have read this accumulator pair out (their tcgen05.ld is ordered before the arrive); an
        // issuer without a unit in the segment waits too, so that its arrival below cannot land in the phase before
        if (!c.wait_bar(&c.acc_empty[buf], ((seg >> 1) & 1) ^ 1, 10, oi, seg)) return;
        tc_fence_after();
        seg_start = false;
        issued = false;
      }
      if ((u & 1) == which) {
        // Stay close to the other issuer: it must have passed every unit of the ops before this one, and be within three
        // units inside it. An issuer without a unit in a stretch of ops would otherwise run ahead, and a parity wait
        // cannot tell a barrier's phase from the one two completions earlier: it would take a cache slot (or a ring
        // stage) that still holds the operand of an earlier op for its own.
        {
          const uint32_t need = max(g0, g >= 3u ? g - 3u : 0u);
          if ((int)(c.prog[which ^ 1] - need) < 0) {
            const uint64_t t0 = globaltimer_ns();
            while ((int)(c.prog[which ^ 1] - need) < 0) {
              if (c.failed()) return;
              if (globaltimer_ns() - t0 > kWaitNs) { c.record(14, oi, r, (int)g); c.fail(); return; }
            }
          }
        }
        const int s = r % c.ns;
        if (!c.wait_bar(&c.tfull[s], (r / c.ns) & 1, 11, oi, r)) return;
        if (!c.wait_bar(&c.cfull[slot], (cpar >> slot) & 1, 12, oi, slot)) return;
        const uint32_t st = ring_s + (uint32_t)s * DS_STAGE, bs = cache_s + (uint32_t)slot * DS_SLOT;
#pragma unroll
        for (int kb = 0; kb < 4; ++kb) {
          tc_cp_sf(tmem_sfa + kb * 4, make_desc_sf(st + DS_A + kb * 512));
          tc_cp_sf(tmem_sfb + kb * 4, make_desc_sf(bs + 2048 + kb * DS_SFB));
        }
        const uint64_t ad = make_desc_sw128(st), bd = make_desc_sw128(bs);
#pragma unroll
        for (int kb = 0; kb < 4; ++kb)
          tc_mma_nvf4(tmem_acc + buf * 32, ad + kb * 2, bd + kb * 2, idesc, (!issued && kb == 0) ? 0u : 1u,
                      tmem_sfa + kb * 4, tmem_sfb + kb * 4);
        tc_commit(&c.empty[s]);
        issued = true;
      }
      c.prog[which] = ++g;
      if (++slot == KT) slot = 0;
      if (++kt == KT || u == u1 - 1) {
        if (issued) tc_commit(&c.acc_full[buf]);
        else mbar_arrive(&c.acc_full[buf]);
        ++seg;
        kt = 0;
        seg_start = true;
      }
    }
    cpar ^= (nslots >= 32 ? 0xffffffffu : ((1u << nslots) - 1u));
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
VE_DEVINL void unpack8(uint4 raw, float* r) {
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
    w.s_ok[slot] = c.wait_cnt(c.p->cnt + oi, need, 20, oi) ? 1 : 0;
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
    // five 1024-element passes at a time, their loads issued together (one L2 round trip instead of five)
    for (int i0 = w.ctid * 8; i0 < H; i0 += 5 * 1024) {
      uint4 hv[5], yv[5];
#pragma unroll
      for (int q = 0; q < 5; ++q) {
        const int i = i0 + q * 1024;
        if (i < H) {
          if (op.in_mode == IN_EMBED) {
            hv[q] = *reinterpret_cast<const uint4*>(p.embed + (size_t)id * H + i);
          } else {
            hv[q] = __ldcg(reinterpret_cast<const uint4*>(hin + (size_t)m * H + i));
            yv[q] = __ldcg(reinterpret_cast<const uint4*>(y + (size_t)m * H + i));
          }
        }
      }
#pragma unroll
      for (int q = 0; q < 5; ++q) {
        const int i = i0 + q * 1024;
        if (i >= H) continue;
        float v[8];
        unpack8(hv[q], v);
        if (op.in_mode == IN_EMBED) {
          if (p.embed_scale != 1.f) {
#pragma unroll
            for (int j = 0; j < 8; ++j) v[j] = round_bf16(v[j] * p.embed_scale);
          }
        } else {
          float a[8];
          unpack8(yv[q], a);
#pragma unroll
          for (int j = 0; j < 8; ++j) v[j] = round_bf16(v[j] + a[j]);
        }
        const uint4 o = pack8(v);
        *reinterpret_cast<uint4*>(hrow + (size_t)m * H + i) = o;
        if (c.cta == 0) *reinterpret_cast<uint4*>(hout + (size_t)m * H + i) = o;
#pragma unroll
        for (int j = 0; j < 8; ++j) ss = fmaf(v[j], v[j], ss);
      }
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

// Eight consecutive input values of row m at column k of the op (zero beyond K): the fused part of every linear.
VE_DEVINL void cw_input8(const Ctx& c, const Cw& w, const StepOp& op, int m, int k, float* x) {
  const StepParams& p = *c.p;
  if (k >= op.K) {
#pragma unroll
    for (int j = 0; j < 8; ++j) x[j] = 0.f;
  } else if (op.in_mode == IN_X) {
    ld8_cg(p.attn_out + (size_t)m * op.K + k, x);
  } else if (op.in_mode == IN_GATED) {
    // act(gate) * up from the split partials of the gate / up tile that holds column k (64 gate rows, then their 64 up rows)
    const StepOp& so = p.ops[op.src];
    const int t = k >> 6, f0 = k & 63;
    int first, n;
    ds_splits(so, t, first, n);
    const float* base = p.ws + so.ws_off + ((size_t)(t * so.ms) * DS_MAXM + m) * 128 + f0;
    const size_t step = (size_t)DS_MAXM * 128;
    float g[8], up[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) g[j] = up[j] = 0.f;
    for (int sp = 0; sp < n; sp += 2) {
      // two splits per round, all eight loads in flight together
      const bool two = sp + 1 < n;
      const float* b0 = base + sp * step;
      const float* b1 = two ? b0 + step : b0;
      const float4 a0 = __ldcg(reinterpret_cast<const float4*>(b0)), a1 = __ldcg(reinterpret_cast<const float4*>(b0 + 4));
      const float4 a2 = __ldcg(reinterpret_cast<const float4*>(b0 + 64)), a3 = __ldcg(reinterpret_cast<const float4*>(b0 + 68));
      const float4 c0 = __ldcg(reinterpret_cast<const float4*>(b1)), c1 = __ldcg(reinterpret_cast<const float4*>(b1 + 4));
      const float4 c2 = __ldcg(reinterpret_cast<const float4*>(b1 + 64)), c3 = __ldcg(reinterpret_cast<const float4*>(b1 + 68));
      g[0] += a0.x; g[1] += a0.y; g[2] += a0.z; g[3] += a0.w; g[4] += a1.x; g[5] += a1.y; g[6] += a1.z; g[7] += a1.w;
      up[0] += a2.x; up[1] += a2.y; up[2] += a2.z; up[3] += a2.w; up[4] += a3.x; up[5] += a3.y; up[6] += a3.z; up[7] += a3.w;
      if (two) {
        g[0] += c0.x; g[1] += c0.y; g[2] += c0.z; g[3] += c0.w; g[4] += c1.x; g[5] += c1.y; g[6] += c1.z; g[7] += c1.w;
        up[0] += c2.x; up[1] += c2.y; up[2] += c2.z; up[3] += c2.w; up[4] += c3.x; up[5] += c3.y; up[6] += c3.z; up[7] += c3.w;
      }
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) x[j] = round_bf16(ds_act(g[j] * so.alpha, up[j] * so.alpha, p.act, p.act_limit));
  } else {
    float g[8];
    ld8(reinterpret_cast<const __nv_bfloat16*>(c.scratch) + (size_t)m * p.H + k, x);
    ld8(op.norm_w + k, g);
    const float rs = w.s_rs[m];
#pragma unroll
    for (int j = 0; j < 8; ++j) x[j] = round_bf16(x[j] * rs * (g[j] + p.wbias));
  }
}

// Operand of k-tile kt into cache slot `slot`: warp-wide, lane = (16-element block, half). The four compute warps take
// the slots of an op in turn; the issuers wait on the slot's barrier the first time a unit needs it.
VE_DEVINL void cw_fill_slot(const Ctx& c, const Cw& w, const StepOp& op, int kt, int slot) {
  const StepParams& p = *c.p;
  const int b = w.lane >> 1, hf = w.lane & 1;
  const int k = kt * 256 + b * 16 + hf * 8;
  uint8_t* bt = c.cache + (size_t)slot * DS_SLOT;
  uint8_t* sf = bt + 2048;
  for (int m = 0; m < p.M; ++m) {
    float x[8];
    cw_input8(c, w, op, m, k, x);
    uint32_t codes[DS_TERMS], sc[DS_TERMS];
    expand_half8<DS_TERMS>(x, codes, sc);
#pragma unroll
    for (int t = 0; t < DS_TERMS; ++t) {
      const int v = m * DS_TERMS + t;
      *reinterpret_cast<uint32_t*>(bt + v * 128 + (((b >> 1) ^ (v & 7)) << 4) + (b & 1) * 8 + hf * 4) = codes[t];
      if (hf == 0) sf[(b >> 2) * DS_SFB + v * 16 + (b & 3)] = (uint8_t)sc[t];
    }
  }
  fence_proxy_async_smem();
  __syncwarp();
  if (w.lane == 0) mbar_arrive(&c.cfull[slot]);
}

VE_DEVINL uint4 ds_ld_volatile_v4(const void* ptr) {
  uint4 v;
  asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(ptr)
               : "memory");
  return v;
}

// Epilogue of the segment that ends at unit j (tile t): TMEM lane = feature, column m * TERMS + term.
VE_DEVINL void cw_epilogue(const Ctx& c, const Cw& w, const StepOp& op, int oi, int u0, int j, uint32_t seg, uint32_t tmem_base) {
  const StepParams& p = *c.p;
  const int KT = ds_kt(op), t = j / KT;
  const uint32_t buf = seg & 1;
  const int f = w.q * 32 + w.lane, n = t * 128 + f;
  const bool ok = c.wait_bar(&c.acc_full[buf], (seg >> 1) & 1, 22, oi, seg);
  tc_fence_after();
  float acc[DS_MAXM] = {0.f, 0.f, 0.f, 0.f};
  if (ok) {
    // units of the segment alternate between the two issuers by unit parity; a one-unit segment has one accumulator
    const int js = max(u0, t * KT);
    const bool has0 = j > js || (j & 1) == 0, has1 = j > js || (j & 1) == 1;
#pragma unroll
    for (int who = 0; who < 2; ++who) {
      if (!(who ? has1 : has0)) continue;
      uint32_t r[16];
      tmem_ld16(tmem_base + ((uint32_t)(w.q * 32) << 16) + who * 64 + buf * 32, r);
      tmem_ld_wait();
#pragma unroll
      for (int m = 0; m < DS_MAXM; ++m) {
        float v = 0.f, s = 1.f;
#pragma unroll
        for (int tt = 0; tt < DS_TERMS; ++tt) { v = fmaf(__uint_as_float(r[m * DS_TERMS + tt]), s, v); s *= 0.125f; }
        acc[m] += v;
      }
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

// Split-KV attention of this CTA's (row, kv head, split) items.
VE_DEVINL void cw_attn(const Ctx& c, Cw& w, const StepOp& op, int oi, uint32_t& r) {
  const StepParams& p = *c.p;
  const int items = p.M * p.nkv * p.S;
  if (c.cta >= items) return;
  if (!cw_wait_op(c, w, op.src, p.ops[op.src].ncontrib)) return;
  const int G = p.nq / p.nkv;
  const int lane = w.lane, g = lane >> 2, t4 = lane & 3;
  float* ms = reinterpret_cast<float*>(c.scratch);     // [4][16]
  float* ls = ms + 64;                                   // [4][16]
  float* os = ls + 64;                                   // [4][G][128]
  __nv_bfloat16* qs = reinterpret_cast<__nv_bfloat16*>(os + 4 * G * 128);   // [G][128] rotated query heads of the item
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
    // Finalise the qkv projection for this item: the G query heads of its row (split sum, rounding, rotation) go to
    // shared memory; the key and value head of every row of the same sequence whose position lies in this item's pages
    // go into the paged cache (several CTAs may store the same row: same bits). 64 threads per head, one rotary pair each.
    {
      const StepOp& so = p.ops[op.src];
      const int f = w.ctid & 63, half = p.rot >> 1;
      const float inv_freq = exp2f(-log2f(p.rope_theta) * (2.f * (float)f / (float)p.rot));
      const int njobs = G + 2 * p.M;
      for (int job = w.ctid >> 6; job < njobs; job += 2) {
        const bool isq = job < G;
        const int m = isq ? a.row : (job - G) >> 1;
        const bool is_v = !isq && ((job - G) & 1);
        const int head = isq ? a.kvh * G + job : p.nq + (is_v ? p.nkv : 0) + a.kvh;
        const int ps = p.pos[m];
        const int sl = p.slot ? p.slot[m] : 0;
        if (!isq && (sl != a.slot || sl < 0 || ps / 64 < a.kt0 || ps / 64 >= a.kt1)) continue;
        int i0, i1;
        if (is_v) { i0 = 2 * f; i1 = i0 + 1; }
        else if (f < half) { i0 = f; i1 = f + half; }
        else { i0 = p.rot + 2 * (f - half); i1 = i0 + 1; }
        int first, nsp;
        ds_splits(so, head, first, nsp);
        const float* base = p.ws + so.ws_off + ((size_t)(head * so.ms) * DS_MAXM + m) * 128;
        float a0 = 0.f, a1 = 0.f;
        for (int sp = 0; sp < nsp; ++sp) {
          a0 += __ldcg(base + (size_t)sp * DS_MAXM * 128 + i0);
          a1 += __ldcg(base + (size_t)sp * DS_MAXM * 128 + i1);
        }
        a0 = round_bf16(a0 * so.alpha);
        a1 = round_bf16(a1 * so.alpha);
        if (!is_v && f < half) {
          float sn, cs;
          sincosf((float)ps * inv_freq, &sn, &cs);
          const float r0 = a0 * cs - a1 * sn, r1 = a1 * cs + a0 * sn;
          a0 = r0;
          a1 = r1;
        }
        const __nv_bfloat16 b0 = f2bf(a0), b1 = f2bf(a1);
        if (isq) {
          qs[job * 128 + i0] = b0;
          qs[job * 128 + i1] = b1;
        } else {
          const int page = p.page_table[(long)sl * p.max_pages + ps / 64];
          const long dst = ((long)op.layer * p.pool_layer_rows + ((long)page * p.nkv + a.kvh) * 64 + (ps % 64)) * 128;
          __nv_bfloat16* pool = is_v ? p.vpool : p.kpool;
          pool[dst + i0] = b0;
          pool[dst + i1] = b1;
        }
      }
      fence_proxy_async_all();       // the cache rows are read back through TMA by this CTA's loader
      __threadfence();
      bar_compute();
      if (w.ctid == 0) *c.kv_seq = *c.kv_seq + 1;
    }
    uint32_t qf[8][4];
#pragma unroll
    for (int kk = 0; kk < 8; ++kk) {
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const __nv_bfloat16* qr = qs + (r_ok[h] ? g + h * 8 : 0) * 128 + kk * 16 + 2 * t4;
        qf[kk][h] = r_ok[h] ? *reinterpret_cast<const uint32_t*>(qr) : 0u;
        qf[kk][2 + h] = r_ok[h] ? *reinterpret_cast<const uint32_t*>(qr + 8) : 0u;
      }
    }
    float o[16][4];
#pragma unroll
    for (int i = 0; i < 16; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    float m_run[2] = {-FLT_MAX, -FLT_MAX}, l_run[2] = {0.f, 0.f};
    // Each warp takes every fourth page of the item whole (16 query rows x 64 keys), so the page loop has no CTA-wide
    // barrier: four pages are in flight per CTA, one per warp, and a warp frees its two stages itself.
    const int npg = a.kt1 - a.kt0;
    for (int i = w.cw; i < npg; i += 4) {
      const int kt = a.kt0 + i;
      const uint32_t rk = r + 2 * i, rv = rk + 1;
      const int sk = rk % c.ns, sv = rv % c.ns;
      const bool okk = c.wait_bar(&c.tfull[sk], (rk / c.ns) & 1, 23, oi, rk);
      const uint32_t kb = smem_u32(c.stage(sk));
      float sacc[8][4];
#pragma unroll
      for (int j = 0; j < 8; ++j) sacc[j][0] = sacc[j][1] = sacc[j][2] = sacc[j][3] = 0.f;
      if (okk) {
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          const int cch = (kk * 16) / 64, ci = ((kk * 16) % 64) / 8;
#pragma unroll
          for (int np = 0; np < 4; ++np) {
            const int mi = lane >> 3, rr = lane & 7;
            const int key = np * 16 + (mi >> 1) * 8 + rr;
            const int ch = ci + (mi & 1);
            uint32_t b0, b1, b2, b3;
            ds_ldsm_x4(kb + cch * 8192 + key * 128 + ((ch ^ (key & 7)) << 4), b0, b1, b2, b3);
            ds_mma_bf16(sacc[2 * np], qf[kk], b0, b1);
            ds_mma_bf16(sacc[2 * np + 1], qf[kk], b2, b3);
          }
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&c.empty[sk]);
      float mx[2] = {-FLT_MAX, -FLT_MAX};
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int h = e >> 1;
          const int key = kt * 64 + nt * 8 + 2 * t4 + (e & 1);
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
      uint32_t pf[4][4];
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) {
        float pv[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int h = e >> 1;
          pv[e] = (sacc[nt][e] == -FLT_MAX) ? 0.f : exp2f(sacc[nt][e] - m_run[h]);
          l_run[h] += pv[e];
        }
        pf[nt >> 1][(nt & 1) * 2 + 0] = ds_pack(pv[0], pv[1]);
        pf[nt >> 1][(nt & 1) * 2 + 1] = ds_pack(pv[2], pv[3]);
      }
#pragma unroll
      for (int j = 0; j < 16; ++j) { o[j][0] *= corr[0]; o[j][1] *= corr[0]; o[j][2] *= corr[1]; o[j][3] *= corr[1]; }
      const bool okv = c.wait_bar(&c.tfull[sv], (rv / c.ns) & 1, 24, oi, rv);
      const uint32_t vb = smem_u32(c.stage(sv));
      if (okv) {
#pragma unroll
        for (int ks = 0; ks < 4; ++ks) {
#pragma unroll
          for (int dp = 0; dp < 8; ++dp) {
            const int mi = lane >> 3, rr = lane & 7;
            const int key = ks * 16 + (mi & 1) * 8 + rr;
            const int d = dp * 16 + (mi >> 1) * 8;
            const int cch = d / 64, ch = (d % 64) / 8;
            uint32_t b0, b1, b2, b3;
            ds_ldsm_x4_t(vb + cch * 8192 + key * 128 + ((ch ^ (key & 7)) << 4), b0, b1, b2, b3);
            ds_mma_bf16(o[2 * dp], pf[ks], b0, b1);
            ds_mma_bf16(o[2 * dp + 1], pf[ks], b2, b3);
          }
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&c.empty[sv]);
    }
    r += 2 * npg;
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
          *reinterpret_cast<float2*>(os + (size_t)(w.cw * G + row) * 128 + nt * 8 + 2 * t4) =
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
          acc += os[(size_t)(ww * G + row) * 128 + d] * cc;
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
  if (w.ctid == 0) { __threadfence_block(); *c.attn_seq = *c.attn_seq + 1; }
}

// One (row, head) per CTA: merge the split partials in split order. The split weights are computed once by the block
// (a thread per split) and shared; empty splits (sequence shorter than the split grid) cost one comparison.
VE_DEVINL void cw_merge(const Ctx& c, Cw& w, const StepOp& op, int oi) {
  const StepParams& p = *c.p;
  const int items = p.M * p.nq;
  if (c.cta >= items) return;
  if (!cw_wait_op(c, w, op.src, p.ops[op.src].ncontrib)) return;
  const int d = w.ctid;
  float* wts = reinterpret_cast<float*>(c.scratch);      // [S] weights, then [4] warp maxima / sums
  float* red = wts + ((p.S + 3) & ~3);
  for (int it = c.cta; it < items; it += c.G) {
    const int row = it / p.nq, head = it % p.nq;
    const long base = ((long)row * p.nq + head) * p.S;
    float mx = -FLT_MAX;
    for (int i = w.ctid; i < p.S; i += 128) {
      const float l = __ldcg(p.lse_part + base + i);
      wts[i] = l;
      mx = fmaxf(mx, l);
    }
    mx = warp_max(mx);
    if (w.lane == 0) red[w.cw] = mx;
    bar_compute();
    mx = fmaxf(fmaxf(red[0], red[1]), fmaxf(red[2], red[3]));
    bar_compute();
    for (int i = w.ctid; i < p.S; i += 128) {
      const float l = wts[i];
      wts[i] = (l == -FLT_MAX) ? 0.f : exp2f(l - mx);
    }
    bar_compute();
    float acc = 0.f, wsum = 0.f;
#pragma unroll 4
    for (int i = 0; i < p.S; ++i) {
      const float wt = wts[i];
      if (wt == 0.f) continue;
      wsum += wt;
      acc += wt * __ldcg(p.o_part + (base + i) * 128 + d);
    }
    p.attn_out[(size_t)row * p.nq * 128 + head * 128 + d] = f2bf(wsum > 0.f ? acc / wsum : 0.f);
    bar_compute();
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
    const bool prof = p.prof && c.cta == p.prof_cta && w.ctid == 0;
    if (prof) p.prof[oi * 4] = globaltimer_ns();
    if (op.type != OP_LINEAR && op.type != OP_NORMOUT) {
      if (op.type == OP_QKV_FIN) cw_qkv_fin(c, w, op, oi);
      else if (op.type == OP_ATTN) cw_attn(c, w, op, oi, r);
      else cw_merge(c, w, op, oi);
      if (prof) p.prof[oi * 4 + 3] = globaltimer_ns();
      continue;
    }
    if (op.type == OP_NORMOUT) {               // final residual add + norm when the LM head runs outside this kernel
      if (c.cta == 0) cw_prologue(c, w, op);
      continue;
    }
    int u0, u1;
    ds_run(op, c.cta, u0, u1);
    if (u0 >= u1) continue;
    cw_prologue(c, w, op);
    if (prof) p.prof[oi * 4 + 1] = globaltimer_ns();
    const int KT = ds_kt(op);
    // the operand of every k-tile of the run, once (the previous op's products have all been read: its last epilogue
    // waited for them), in the order the units need them
    const int nslots = ds_nslots(KT, u0, u1);
    for (int i = w.cw; i < nslots; i += 4) cw_fill_slot(c, w, op, (u0 + i) % KT, i);
    if (prof) p.prof[oi * 4 + 2] = globaltimer_ns();
    for (int j = u0; j < u1; ++j)
      if (j % KT == KT - 1 || j == u1 - 1) cw_epilogue(c, w, op, oi, u0, j, seg++, tmem_base);
    r += (uint32_t)(u1 - u0);
    if (op.out_mode == OUT_PART) cw_signal(c, w, oi);
    if (prof) p.prof[oi * 4 + 3] = globaltimer_ns();
  }
}

__global__ void __launch_bounds__(224, 1) decode_step_kernel(const __grid_constant__ StepParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  __shared__ uint64_t tfull[DS_MAXNS], empty[DS_MAXNS], cfull[DS_SLOTS], acc_full[2], acc_empty[2];
  __shared__ uint32_t tmem_holder;
  __shared__ int s_fail, s_flag, s_last, s_ok[4];
  __shared__ uint32_t s_attn_seq, s_prog[2], s_kv_seq;
  __shared__ float s_rs[DS_MAXM], s_red[4 * DS_MAXM];

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int s = 0; s < DS_MAXNS; ++s) { mbar_init(&tfull[s], 1); mbar_init(&empty[s], 1); }
    for (int s = 0; s < DS_SLOTS; ++s) mbar_init(&cfull[s], 1);
    for (int b = 0; b < 2; ++b) { mbar_init(&acc_full[b], 2); mbar_init(&acc_empty[b], 1); }
    // a status word left set by an earlier failure makes every wait of this launch give up at once
    s_fail = (p.status && *reinterpret_cast<volatile int*>(p.status) != 0) ? 1 : 0;
    s_attn_seq = 0;
    s_prog[0] = s_prog[1] = 0;
    s_kv_seq = 0;
    mbar_fence_init();
  }
  if (warp == 1) { tmem_alloc(&tmem_holder, DS_TMEM); tmem_relinquish(); }
  {
    // operand rows and scale bytes that no activation row uses stay zero for the whole launch (a stray scale byte in an
    // unused column costs the used columns their precision)
    uint8_t* cache0 = smem + (size_t)p.ns * DS_STAGE;
    for (int i = threadIdx.x * 16; i < DS_CACHE; i += blockDim.x * 16) *reinterpret_cast<uint4*>(cache0 + i) = make_uint4(0, 0, 0, 0);
    fence_proxy_async_smem();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_holder;
  // shared memory: ring stages | operand cache | scratch (row(s) of the normalised input, attention merge)
  Ctx c{&p, smem, smem + (size_t)p.ns * DS_STAGE, smem + (size_t)p.ns * DS_STAGE + DS_CACHE, tfull, cfull, empty, acc_full,
        acc_empty, p.ns, &s_fail, &s_attn_seq, s_prog, &s_kv_seq, (int)blockIdx.x, (int)gridDim.x};
  if (warp == 0) {
    if (lane == 0) ds_loader(c);
  } else if (warp == 1 || warp == 6) {
    if (lane == 0) ds_mma(c, tmem_base, warp == 1 ? 0 : 1);
  } else {
    Cw w{(int)threadIdx.x - 64, warp - 2, lane, warp & 3, s_rs, s_red, &s_flag, s_ok, 0};
    ds_compute(c, w, tmem_base);
  }
  tc_fence_before();
  __syncthreads();
  if (s_fail && threadIdx.x == 0) {
    // after a failed wait copies of the loader may still be in flight: give each stage a short time to land
    for (int s = 0; s < p.ns; ++s) {
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
  StepParams p = *reinterpret_cast<const StepParams*>(params);
  if (p.M < 1 || p.M > DS_MAXM || p.H % 8 || p.nkv < 1 || p.nq % p.nkv || p.nq / p.nkv > 16 || p.S < 1 || ctas < 1 ||
      p.size < 1 || p.size > 8)
    return cudaErrorInvalidValue;
  // scratch: the normalised-input rows of a linear, or the four warps' attention states; the ring takes what is left
  const int G = p.nq / p.nkv;
  const int need = max(max(p.M * p.H * 2, 512 + 4 * G * 128 * 4 + G * 256), (p.S + 8) * 4);
  p.scr = (need + 1023) / 1024 * 1024;
  p.ns = (DS_SMEM - 1024 - DS_CACHE - p.scr) / DS_STAGE;
  if (p.ns > DS_MAXNS) p.ns = DS_MAXNS;
  if (p.ns < 3) return cudaErrorInvalidValue;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(decode_step_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, DS_SMEM);
    if (e != cudaSuccess) return (int)e;
    attr_set = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(ctas);
  cfg.blockDim = dim3(224);
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
