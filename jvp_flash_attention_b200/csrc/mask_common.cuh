// Mask access shared by the attention kernels: a (B,H,N,N) view given by element strides, the optional output of the
// summary pre-pass (per 64x64 tile: anything kept / anything excluded or biased; for boolean masks also the mask packed
// into bits in both orientations), and per-row loaders that turn a run of mask entries into an additive bias in the
// base-2 logarithm domain (0 / -inf for boolean masks).
//
// Layout of the summary buffer for a mask with P = Bm * Hm distinct planes, n64 = ceil(N / 64), n_pad = 64 n64:
//   tile flags   P * n64 * n64 bytes, rounded up to a multiple of 256
//   row bits     P * n64 * n_pad words of 64 bits: word [plane][key tile][query] holds the query's 64 entries of that key
//                tile (bit c = key 64 tile + c takes part); what a thread that owns a query row needs per tile
//   column bits  the same size: word [plane][query tile][key] holds the key's 64 entries of that query tile; what a
//                thread that owns a key row needs per tile
//   tile values  P * n64 * n64 floats (additive masks)
// Boolean masks: bit = the entry takes part; entries outside the sequence are zero bits. Additive masks (contiguous
// rows only): bit = the entry is +-0, and a tile all of whose other entries inside the sequence carry one and the same
// value c is flagged "two-valued" with c in the tile values -- the common additive masks (0 / -inf, 0 / a large negative
// constant) then cost one load per thread and tile like a boolean mask; every other tile is read element by element.
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
  const uint32_t* rowbits; // packed mask, query-major words (two 32-bit halves each); null if there is no summary
  const uint32_t* colbits; // packed mask, key-major words
  const float* tilevals;   // additive masks: the other value of a two-valued tile; null if there is none
  int n_pad;               // 64 * n64
};

inline size_t mask_tile_flag_bytes(size_t planes, size_t n64) { return (planes * n64 * n64 + 255) / 256 * 256; }
inline size_t mask_bit_bytes(size_t planes, size_t n64) { return planes * n64 * (64 * n64) * 8; }
inline size_t mask_tile_value_bytes(size_t planes, size_t n64) { return planes * n64 * n64 * sizeof(float); }

// The view the kernels work with, from the mask of a call and the summary buffer (or null) that came with it.
inline MaskView make_mask_view(const jvpfa_mask& mask, const uint8_t* summary, int B, int H, int N) {
  MaskView mv{};
  mv.ptr = mask.ptr;
  mv.summary = summary;
  mv.s0 = mask.stride[0]; mv.s1 = mask.stride[1]; mv.s2 = mask.stride[2]; mv.s3 = mask.stride[3];
  mv.kind = mask.kind;
  mv.dtype = mask.dtype;
  mv.n64 = (N + 63) / 64;
  mv.Hm = mask.stride[1] == 0 ? 1 : H;
  mv.n_pad = 64 * mv.n64;
  if (summary != nullptr && mask.kind != JVPFA_MASK_NONE) {
    const size_t planes = static_cast<size_t>(mask.stride[0] == 0 ? 1 : B) * mv.Hm;
    const uint8_t* bits = summary + mask_tile_flag_bytes(planes, mv.n64);
    mv.rowbits = reinterpret_cast<const uint32_t*>(bits);
    mv.colbits = reinterpret_cast<const uint32_t*>(bits + mask_bit_bytes(planes, mv.n64));
    if (mask.kind == JVPFA_MASK_ADDITIVE) mv.tilevals = reinterpret_cast<const float*>(bits + 2 * mask_bit_bytes(planes, mv.n64));
  }
  return mv;
}

constexpr uint8_t kTileAnyKept = 1;     // some element of the tile takes part in attention
constexpr uint8_t kTileAnyMasked = 2;   // some element needs the mask: a boolean False, or an additive entry that is not zero
constexpr uint8_t kTileTwoValued = 4;   // additive mask: every entry is +-0 or the tile's one other value (bit words + tile values)

#if defined(__CUDACC__)
// Summary bits of the 64x64 tile (qt, kt) for batch b, head h; "mixed" when there is no summary.
__device__ __forceinline__ uint8_t mask_tile_bits(const MaskView& mv, int b, int h, int qt, int kt) {
  if (mv.kind == JVPFA_MASK_NONE) return kTileAnyKept;
  if (mv.summary == nullptr) return kTileAnyKept | kTileAnyMasked;
  const int bm = mv.s0 == 0 ? 0 : b;
  const int hm = mv.s1 == 0 ? 0 : h;
  return mv.summary[((static_cast<int64_t>(bm) * mv.Hm + hm) * mv.n64 + qt) * mv.n64 + kt];
}

// The other value of the two-valued 64x64 tile (qt, kt) of an additive mask.
__device__ __forceinline__ float mask_tile_value(const MaskView& mv, int b, int h, int qt, int kt) {
  const int64_t plane = static_cast<int64_t>(mv.s0 == 0 ? 0 : b) * mv.Hm + (mv.s1 == 0 ? 0 : h);
  return __ldg(mv.tilevals + (plane * mv.n64 + qt) * mv.n64 + kt);
}

// 32 bits of the packed mask. Row form: query q against keys 64 tile + 32 half + i (bit i); column form: key k
// against queries 64 tile + 32 half + i.
__device__ __forceinline__ uint32_t mask_row_bits(const MaskView& mv, int b, int h, int q, int tile, int half) {
  const int64_t plane = static_cast<int64_t>(mv.s0 == 0 ? 0 : b) * mv.Hm + (mv.s1 == 0 ? 0 : h);
  return __ldg(mv.rowbits + ((plane * mv.n64 + tile) * mv.n_pad + q) * 2 + half);
}
__device__ __forceinline__ uint32_t mask_col_bits(const MaskView& mv, int b, int h, int tile, int k, int half) {
  const int64_t plane = static_cast<int64_t>(mv.s0 == 0 ? 0 : b) * mv.Hm + (mv.s1 == 0 ? 0 : h);
  return __ldg(mv.colbits + ((plane * mv.n64 + tile) * mv.n_pad + k) * 2 + half);
}

// How a thread applies the mask to its 32 scores of a tile, from the flags of its own 64x64 tile:
//   0 = nothing to do (the tile needs no mask), 1 = from the packed words (mask_apply_bits), 2 = element by element
__device__ __forceinline__ int mask_tile_mode(const MaskView& mv, uint8_t my_flags) {
  if (!(my_flags & kTileAnyMasked)) return 0;
  if (mv.rowbits == nullptr) return 2;
  if (mv.kind == JVPFA_MASK_BOOL || (my_flags & kTileTwoValued)) return 1;
  return 2;
}
// x2[i] = scores (2 i, 2 i + 1) in the log2 domain, mb = the thread's 32 bits (mask_row_bits / mask_col_bits), `other` =
// what a zero bit adds: -inf for a boolean mask, c log2(e) for a two-valued additive tile (whose zero bits outside the
// sequence are excluded by the caller's bound check, not here)
__device__ __forceinline__ void mask_apply_bits(float2 (&x2)[16], uint32_t mb, float other) {
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    if (!((mb >> (2 * i)) & 1u)) x2[i].x += other;
    if (!((mb >> (2 * i + 1)) & 1u)) x2[i].y += other;
  }
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
    const int es = mv.dtype == JVPFA_F32 ? 4 : 2;
    const uint8_t* mp = static_cast<const uint8_t*>(mv.ptr) + base * es;
    if (step == 1 && (reinterpret_cast<uintptr_t>(mp) & 15) == 0 && first + CNT <= N && (CNT % 8) == 0) {
      // a contiguous, aligned run: 16 bytes per load
      if (mv.dtype == JVPFA_F32) {
#pragma unroll
        for (int c = 0; c < CNT / 4; ++c) {
          const float4 v = *reinterpret_cast<const float4*>(mp + 16 * c);
          bias[4 * c] = v.x * kLog2e; bias[4 * c + 1] = v.y * kLog2e; bias[4 * c + 2] = v.z * kLog2e; bias[4 * c + 3] = v.w * kLog2e;
        }
      } else {
#pragma unroll
        for (int c = 0; c < CNT / 8; ++c) {
          const uint4 v = *reinterpret_cast<const uint4*>(mp + 16 * c);
          const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            float lo, hi;
            if (mv.dtype == JVPFA_BF16) {
              lo = __uint_as_float(w[i] << 16);
              hi = __uint_as_float(w[i] & 0xFFFF0000u);
            } else {
              const __half2 hh = *reinterpret_cast<const __half2*>(&w[i]);
              lo = __low2float(hh);
              hi = __high2float(hh);
            }
            bias[8 * c + 2 * i] = lo * kLog2e;
            bias[8 * c + 2 * i + 1] = hi * kLog2e;
          }
        }
      }
    } else {
#pragma unroll
      for (int i = 0; i < CNT; ++i)
        bias[i] = (first + i < N) ? mask_elem_as_float(mv.ptr, base + i * step, mv.dtype) * kLog2e : ninf;
    }
  }
}
#endif

}  // namespace jvpfa
