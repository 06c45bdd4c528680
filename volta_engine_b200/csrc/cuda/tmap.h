// Host helper: build TMA tensor maps without linking libcuda (the driver entry point is resolved at run time).
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <string.h>

#include <memory>

namespace ve {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess) fn = (EncodeTiledFn)p;
  }
  return fn;
}

// A tensor map depends only on its arguments, and an engine encodes the same few hundred (one per weight, per KV pool
// and per activation buffer) again at every launch. Encoded maps are therefore kept in a direct-mapped table per
// host thread, keyed by all arguments: a launch costs one hash and one compare instead of a driver call.
struct TmapKey {
  const void* base;
  uint64_t rows, cols, pitch;
  uint32_t box_rows, box_cols;
  int dt, elem_bytes, swz, used;
};
struct TmapSlot {
  TmapKey key;
  CUtensorMap map;
};
constexpr int kTmapSlots = 2048;

inline TmapSlot* tmap_table() {
  static thread_local std::unique_ptr<TmapSlot[]> table;
  if (!table) {
    table.reset(new TmapSlot[kTmapSlots]);
    memset(table.get(), 0, sizeof(TmapSlot) * kTmapSlots);
  }
  return table.get();
}

// 2-D row-major tensor [rows, cols] of `elem_bytes`-wide elements, row pitch `pitch_bytes`.
// box = [box_rows, box_cols]; box_cols * elem_bytes must equal the swizzle span (128 B) when swizzled.
// Out-of-range elements read as zero. Returns 0 on success.
inline int make_tmap_2d(CUtensorMap* map, const void* base, CUtensorMapDataType dt, int elem_bytes, uint64_t rows,
                        uint64_t cols, uint64_t pitch_bytes, uint32_t box_rows, uint32_t box_cols,
                        CUtensorMapSwizzle swz) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return (int)cudaErrorNotSupported;
  if (((uintptr_t)base & 15) || (pitch_bytes & 15)) return (int)cudaErrorMisalignedAddress;
  TmapKey key;
  memset(&key, 0, sizeof(key));
  key.base = base, key.rows = rows, key.cols = cols, key.pitch = pitch_bytes;
  key.box_rows = box_rows, key.box_cols = box_cols, key.dt = (int)dt, key.elem_bytes = elem_bytes, key.swz = (int)swz, key.used = 1;
  uint64_t h = (uint64_t)(uintptr_t)base * 0x9E3779B97F4A7C15ull;
  h ^= (rows * 0xC2B2AE3D27D4EB4Full) ^ (cols << 17) ^ ((uint64_t)box_rows << 40) ^ ((uint64_t)box_cols << 52) ^ (uint64_t)swz;
  TmapSlot* slot = tmap_table() + ((h ^ (h >> 29)) & (kTmapSlots - 1));
  if (memcmp(&slot->key, &key, sizeof(key)) == 0) {
    memcpy(map, &slot->map, sizeof(CUtensorMap));
    return 0;
  }
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {pitch_bytes};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, dt, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swz,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return (int)cudaErrorInvalidValue;
  slot->key = key;
  memcpy(&slot->map, map, sizeof(CUtensorMap));
  return 0;
}

}  // namespace ve
