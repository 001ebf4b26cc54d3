// Mask access shared by the attention kernels: a (B,H,N,N) view given by element strides,
// the optional 64x64 tile summary, and per-row loaders that turn a run of mask entries into an
// additive bias in the base-2 logarithm domain (0 / -inf for boolean masks).
#pragma once
#include <cstdint>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include "../../include/jvpfa.h"

namespace jvpfa {

struct MaskView {
  const void* ptr;
  const uint8_t* summary;  // may be null
  int64_t s0, s1, s2, s3;  // element strides of (B,H,N,N)
  int kind;                // JVPFA_MASK_*
  int dtype;               // element type of an additive mask
  int n64;                 // number of 64-wide tiles along N
  int Hm;                  // number of distinct head planes in the summary
};

constexpr uint8_t kTileAnyKept = 1;     // some element of the tile takes part in attention
constexpr uint8_t kTileAnyMasked = 2;   // some element needs the mask: a boolean False, or an additive entry that is not zero

#if defined(__CUDACC__)
// Summary bits of the 64x64 tile (qt, kt) for batch b, head h; "mixed" when there is no summary.
__device__ __forceinline__ uint8_t mask_tile_bits(const MaskView& mv, int b, int h, int qt, int kt) {
  if (mv.kind == JVPFA_MASK_NONE) return kTileAnyKept;
  if (mv.summary == nullptr) return kTileAnyKept | kTileAnyMasked;
  const int bm = mv.s0 == 0 ? 0 : b;
  const int hm = mv.s1 == 0 ? 0 : h;
  return mv.summary[((static_cast<int64_t>(bm) * mv.Hm + hm) * mv.n64 + qt) * mv.n64 + kt];
}

__device__ __forceinline__ float mask_elem_as_float(const void* base, int64_t idx, int dtype) {
  if (dtype == JVPFA_F32) return static_cast<const float*>(base)[idx];
  if (dtype == JVPFA_BF16) return __bfloat162float(static_cast<const __nv_bfloat16*>(base)[idx]);
  return __half2float(static_cast<const __half*>(base)[idx]);
}

// bias[i] for entries (b, h, q, k0 + i*step_is_one), i in [0, CNT): 0 or -inf for a boolean mask,
// mask*log2e for an additive one. Entries with k >= N are excluded. Used with the q index fixed
// (a row of scores) -- `along_k == true` -- or with the k index fixed and q running (a row of
// transposed scores) -- `along_k == false`, in which case k0 is the fixed key index, q the first
// query index, and entries with q >= N are excluded.
template <int CNT>
__device__ __forceinline__ void mask_bias_run(float (&bias)[CNT], const MaskView& mv, int b, int h, int q, int k0, int N,
                                              bool along_k) {
  constexpr float kLog2e = 1.4426950408889634f;
  const float ninf = -INFINITY;
  const int64_t base = b * mv.s0 + h * mv.s1 + static_cast<int64_t>(q) * mv.s2 + static_cast<int64_t>(k0) * mv.s3;
  const int64_t step = along_k ? mv.s3 : mv.s2;
  const int first = along_k ? k0 : q;
  if (mv.kind == JVPFA_MASK_BOOL) {
    const uint8_t* mp = static_cast<const uint8_t*>(mv.ptr) + base;
    if (step == 1 && (reinterpret_cast<uintptr_t>(mp) & 15) == 0 && first + CNT <= N && (CNT % 16) == 0) {
#pragma unroll
      for (int c = 0; c < CNT / 16; ++c) {
        const uint4 v = *reinterpret_cast<const uint4*>(mp + 16 * c);
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int i = 0; i < 16; ++i) bias[16 * c + i] = ((w[i >> 2] >> (8 * (i & 3))) & 0xFFu) ? 0.0f : ninf;
      }
    } else {
#pragma unroll
      for (int i = 0; i < CNT; ++i) bias[i] = (first + i < N && mp[i * step]) ? 0.0f : ninf;
    }
  } else {
#pragma unroll
    for (int i = 0; i < CNT; ++i)
      bias[i] = (first + i < N) ? mask_elem_as_float(mv.ptr, base + i * step, mv.dtype) * kLog2e : ninf;
  }
}
#endif

}  // namespace jvpfa
