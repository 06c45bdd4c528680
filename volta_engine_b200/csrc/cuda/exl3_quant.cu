// EXL3 quantiser: exact Viterbi trellis encoder on the device.
//
// A 16 x 16 tile is a cyclic stream of 256 * bits bits; position p owns the 16-bit window that ends at bit
// (p + 1) * bits, so consecutive windows overlap in 16 - bits bits: window s_p = ((s_{p-1} << bits) | new bits) & 0xffff.
// Encoding a tile = the window sequence that minimises sum_p (value(s_p) - target_p)^2 under that shift constraint,
// tail-biting (the stream is cyclic). The search is the one of the PyTorch statement (quant/exl3.py:
// viterbi_encode_tile): an open pass over the 65536-state trellis, then a second pass that starts from, and must return
// to, the state the first pass ended in; same arithmetic, same tie rules (lowest predecessor, lowest state).
//
// The recurrence is kept on the reduced table M_p[g] = min_j cost_p[(j << (16 - bits)) | g] (g = the low 16 - bits bits a
// successor keeps), since cost_{p+1}[s] = M_p[s >> bits] + (value(s) - t_{p+1})^2:
//     M_{p+1}[g'] = min_j  M_p[((j << (16 - bits)) | g') >> bits] + (value((j << (16 - bits)) | g') - t_{p+1})^2
// so a step touches all 65536 states but stores only 2^(16 - bits) costs (two buffers in shared memory: 32 KB at 4 bits,
// 128 KB at 2 bits) and one byte of back pointer per entry (global scratch, [255][2^(16 - bits)] per CTA). One CTA of
// 1024 threads encodes one tile at a time; the grid walks the tiles. bits = 1 does not fit shared memory and is left to
// the host statement.
// Reference counterpart: src/kernels/cuda/trellis/quant/exl3_quantize.cu:126-340, exl3_encode*.cu (Viterbi encoder).
#include "common.cuh"
#include <cuda_fp16.h>
#include <float.h>

namespace ve {

template <int CB>
VE_DEVINL float exl3_value(uint32_t w) {
  if (CB == 2) {
    const uint32_t h = __dp4a(w * 0x83DCD12Du, 0x01010101u, 0x6400u);          // fp16 bits of 1024 + byte sum
    const __half v = __hfma(__ushort_as_half((unsigned short)h), __ushort_as_half((unsigned short)0x1eee),
                            __ushort_as_half((unsigned short)0xc931));
    return __half2float(v);
  }
  uint32_t x = CB == 0 ? w * 89226354u + 64248484u : w * 0xCBAC1FEDu;
  x = (x & 0x8fff8fffu) ^ 0x3b603b60u;
  const __half v = __hadd(__ushort_as_half((unsigned short)(x & 0xffffu)), __ushort_as_half((unsigned short)(x >> 16)));
  return __half2float(v);
}

VE_DEVINL float sq_err(float v, float t) {
  const float d = __fsub_rn(v, t);
  return __fmul_rn(d, d);
}

// (cost, index) minimum over the block, ties to the lower index; result broadcast through shared memory.
VE_DEVINL void block_argmin(float& c, int& idx, float* s_c, int* s_i) {
#pragma unroll
  for (int m = 16; m; m >>= 1) {
    const float oc = __shfl_xor_sync(0xffffffffu, c, m);
    const int oi = __shfl_xor_sync(0xffffffffu, idx, m);
    if (oc < c || (oc == c && oi < idx)) { c = oc; idx = oi; }
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  if (lane == 0) { s_c[warp] = c; s_i[warp] = idx; }
  __syncthreads();
  if (warp == 0) {
    c = lane < nw ? s_c[lane] : FLT_MAX;
    idx = lane < nw ? s_i[lane] : 0x7fffffff;
#pragma unroll
    for (int m = 16; m; m >>= 1) {
      const float oc = __shfl_xor_sync(0xffffffffu, c, m);
      const int oi = __shfl_xor_sync(0xffffffffu, idx, m);
      if (oc < c || (oc == c && oi < idx)) { c = oc; idx = oi; }
    }
    if (lane == 0) { s_c[0] = c; s_i[0] = idx; }
  }
  __syncthreads();
  c = s_c[0];
  idx = s_i[0];
  __syncthreads();
}

template <int BITS, int CB>
__global__ void __launch_bounds__(1024) exl3_viterbi_kernel(const float* __restrict__ targets, int16_t* __restrict__ codes,
                                                            uint8_t* __restrict__ back_all, int tiles) {
  constexpr int G = 1 << (16 - BITS), B = 1 << BITS, LOW = 16 - BITS;
  extern __shared__ float smem_f[];
  float* Ma = smem_f;                      // [G]
  float* Mb = smem_f + G;                  // [G]
  __shared__ float s_t[256];
  __shared__ float s_c[32];
  __shared__ int s_i[32];
  __shared__ uint16_t s_path[256];
  uint8_t* back = back_all + (size_t)blockIdx.x * 255 * G;
  const float INF = __int_as_float(0x7f800000);

  for (int tile = blockIdx.x; tile < tiles; tile += gridDim.x) {
    for (int i = threadIdx.x; i < 256; i += blockDim.x) s_t[i] = targets[(size_t)tile * 256 + i];
    __syncthreads();
    int end_state = -1;
    for (int pass = 0; pass < 2; ++pass) {
      // position 0: open (every state allowed) or, in the closing pass, only the states whose upper 16 - bits bits are the
      // lower bits of the state the stream must return to
      const int hi = end_state & (G - 1);
      float* M = Ma;
      float* Mn = Mb;
      for (int g = threadIdx.x; g < G; g += blockDim.x) {
        float best = INF;
        int arg = 0;
        for (int j = 0; j < B; ++j) {
          const int s = (j << LOW) | g;
          float c = sq_err(exl3_value<CB>((uint32_t)s), s_t[0]);
          if (pass == 1 && (s >> BITS) != hi) c = INF;
          if (c < best) { best = c; arg = j; }
        }
        M[g] = best;
        back[g] = (uint8_t)arg;            // A_0
      }
      __syncthreads();
      for (int p = 1; p < 255; ++p) {
        const float t = s_t[p];
        uint8_t* bp = back + (size_t)p * G;
        for (int g = threadIdx.x; g < G; g += blockDim.x) {
          float best = INF;
          int arg = 0;
#pragma unroll 4
          for (int j = 0; j < B; ++j) {
            const int s = (j << LOW) | g;
            const float c = __fadd_rn(M[s >> BITS], sq_err(exl3_value<CB>((uint32_t)s), t));
            if (c < best) { best = c; arg = j; }
          }
          Mn[g] = best;
          bp[g] = (uint8_t)arg;            // A_p
        }
        __syncthreads();
        float* tmp = M; M = Mn; Mn = tmp;
      }
      // position 255: the full cost row c_255[s] = M_254[s >> bits] + err; its minimum (open pass) or the forced end
      int s_end;
      if (pass == 0) {
        float best = FLT_MAX;
        int arg = 0x7fffffff;
        for (int s = threadIdx.x; s < 65536; s += blockDim.x) {
          const float c = __fadd_rn(M[s >> BITS], sq_err(exl3_value<CB>((uint32_t)s), s_t[255]));
          if (c < best || (c == best && s < arg)) { best = c; arg = s; }
        }
        block_argmin(best, arg, s_c, s_i);
        s_end = arg;
        end_state = s_end;
      } else {
        const float forced = __fadd_rn(M[end_state >> BITS], sq_err(exl3_value<CB>((uint32_t)end_state), s_t[255]));
        if (forced < INF) {
          s_end = end_state;
          __syncthreads();
        } else {                           // (cannot happen for a consistent start set; mirrors the statement)
          float best = FLT_MAX;
          int arg = 0x7fffffff;
          for (int s = threadIdx.x; s < 65536; s += blockDim.x) {
            const float c = __fadd_rn(M[s >> BITS], sq_err(exl3_value<CB>((uint32_t)s), s_t[255]));
            if (c < best || (c == best && s < arg)) { best = c; arg = s; }
          }
          block_argmin(best, arg, s_c, s_i);
          s_end = arg;
        }
        // back-track: s_{p-1} = (A_{p-1}[s_p >> bits] << (16 - bits)) | (s_p >> bits)
        if (threadIdx.x == 0) {
          int s = s_end;
          s_path[255] = (uint16_t)s;
          for (int p = 254; p >= 0; --p) {
            const int g = s >> BITS;
            s = ((int)back[(size_t)p * G + g] << LOW) | g;
            s_path[p] = (uint16_t)s;
          }
        }
        __syncthreads();
      }
      __syncthreads();
    }
    // the stream: bits [p * bits, (p + 1) * bits) are the low bits of window p, most significant first; 32-bit words,
    // stored as two little-endian 16-bit halves (low half first)
    for (int wd = threadIdx.x; wd < 8 * BITS; wd += blockDim.x) {
      uint32_t word = 0;
      for (int b = 0; b < 32; ++b) {
        const int pos = wd * 32 + b;                       // bit index in the stream
        const int p = pos / BITS, k = pos % BITS;          // window p, k-th of its new bits (MSB first)
        const uint32_t bit = (s_path[p] >> (BITS - 1 - k)) & 1u;
        word |= bit << (31 - b);
      }
      codes[(size_t)tile * 16 * BITS + 2 * wd] = (int16_t)(word & 0xffffu);
      codes[(size_t)tile * 16 * BITS + 2 * wd + 1] = (int16_t)(word >> 16);
    }
    __syncthreads();
  }
}

}  // namespace ve

using namespace ve;

template <int BITS, int CB>
static int viterbi_launch(const void* targets, void* codes, void* back, int tiles, int ctas, cudaStream_t st) {
  const size_t smem = 2 * sizeof(float) * ((size_t)1 << (16 - BITS));
  cudaError_t e = cudaFuncSetAttribute(exl3_viterbi_kernel<BITS, CB>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return (int)e;
  exl3_viterbi_kernel<BITS, CB><<<ctas, 1024, smem, st>>>((const float*)targets, (int16_t*)codes, (uint8_t*)back, tiles);
  VE_CHECK_LAUNCH();
}

extern "C" {

// Bytes of back-pointer scratch one CTA needs at `bits`.
long ve_exl3_viterbi_scratch(int bits) { return bits < 2 || bits > 8 ? -1 : 255L * (1L << (16 - bits)); }

// targets fp32 [tiles][256] (stream-position order, in units of the codebook: unit variance), codes int16
// [tiles][16 * bits], back: ctas * ve_exl3_viterbi_scratch(bits) bytes. bits 2..8; cb 0 (3INST), 1 (MCG), 2 (MUL1).
int ve_exl3_viterbi(const void* targets, void* codes, void* back, int tiles, int bits, int cb, int ctas, cudaStream_t st) {
  if (tiles <= 0) return 0;
  if (bits < 2 || bits > 8 || cb < 0 || cb > 2 || ctas < 1 || !back) return cudaErrorInvalidValue;
#define VE_VT(B)                                                                              \
  case B:                                                                                     \
    return cb == 2 ? viterbi_launch<B, 2>(targets, codes, back, tiles, ctas, st)              \
         : cb == 1 ? viterbi_launch<B, 1>(targets, codes, back, tiles, ctas, st)              \
                   : viterbi_launch<B, 0>(targets, codes, back, tiles, ctas, st);
  switch (bits) {
    VE_VT(2) VE_VT(3) VE_VT(4) VE_VT(5) VE_VT(6) VE_VT(7) VE_VT(8)
    default: return cudaErrorInvalidValue;
  }
#undef VE_VT
}

}  // extern "C"
