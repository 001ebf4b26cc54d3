// Dropout on the attention probabilities, regenerated wherever it is needed (forward and the three backward families)
// from a counter-based generator instead of being stored: Philox4x32-10 keyed by the 64-bit seed, counter
// (q >> 1, k >> 1, batch*head unit, 0); the four 32-bit outputs of one call belong to the 2 x 2 block of score elements
// (q, k) with index (q & 1) * 2 + (k & 1), and an element is kept when its number is >= p * 2^32. The reference only
// sketches dropout (jvp_flash_attention/jvp_attention.py:105-133, a Philox keep mask per tile) and refuses
// dropout_p != 0 (:2550).
#pragma once
#include <cstdint>

namespace jvpfa {

struct DropoutParams {
  uint32_t seed_lo, seed_hi;
  uint32_t threshold;   // keep when the element's 32-bit number is >= threshold
  float inv_keep;       // 1 / (1 - p)
};

inline DropoutParams make_dropout_params(float p, uint64_t seed) {
  DropoutParams d{};
  d.seed_lo = static_cast<uint32_t>(seed & 0xFFFFFFFFull);
  d.seed_hi = static_cast<uint32_t>(seed >> 32);
  const double t = static_cast<double>(p) * 4294967296.0 + 0.5;
  d.threshold = t >= 4294967295.0 ? 0xFFFFFFFFu : (t <= 0.0 ? 0u : static_cast<uint32_t>(t));
  d.inv_keep = p < 1.f ? 1.0f / (1.0f - p) : 0.f;
  return d;
}

#if defined(__CUDACC__)
__device__ __forceinline__ void philox4x32_10(uint32_t c0, uint32_t c1, uint32_t c2, uint32_t c3, uint32_t k0, uint32_t k1,
                                              uint32_t (&out)[4]) {
#pragma unroll
  for (int round = 0; round < 10; ++round) {
    const uint32_t hi0 = __umulhi(0xD2511F53u, c0), lo0 = 0xD2511F53u * c0;
    const uint32_t hi1 = __umulhi(0xCD9E8D57u, c2), lo1 = 0xCD9E8D57u * c2;
    c0 = hi1 ^ c1 ^ k0;
    c1 = lo1;
    c2 = hi0 ^ c3 ^ k1;
    c3 = lo0;
    k0 += 0x9E3779B9u;
    k1 += 0xBB67AE85u;
  }
  out[0] = c0; out[1] = c1; out[2] = c2; out[3] = c3;
}

// Keep bits of the 32 score elements (q, k0 .. k0 + 31), k0 even: bit i belongs to key k0 + i.
__device__ __forceinline__ uint32_t dropout_keep_along_k(const DropoutParams& d, int unit, int q, int k0) {
  uint32_t bits = 0;
  const int sel = (q & 1) * 2;
#pragma unroll
  for (int j = 0; j < 16; ++j) {
    uint32_t w[4];
    philox4x32_10(static_cast<uint32_t>(q >> 1), static_cast<uint32_t>((k0 >> 1) + j), static_cast<uint32_t>(unit), 0u,
                  d.seed_lo, d.seed_hi, w);
    const uint32_t a = sel ? w[2] : w[0], b = sel ? w[3] : w[1];
    bits |= (a >= d.threshold ? 1u : 0u) << (2 * j);
    bits |= (b >= d.threshold ? 1u : 0u) << (2 * j + 1);
  }
  return bits;
}

// Keep bits of the 32 score elements (q0 .. q0 + 31, k), q0 even: bit i belongs to query q0 + i.
__device__ __forceinline__ uint32_t dropout_keep_along_q(const DropoutParams& d, int unit, int q0, int k) {
  uint32_t bits = 0;
  const int sel = k & 1;
#pragma unroll
  for (int j = 0; j < 16; ++j) {
    uint32_t w[4];
    philox4x32_10(static_cast<uint32_t>((q0 >> 1) + j), static_cast<uint32_t>(k >> 1), static_cast<uint32_t>(unit), 0u,
                  d.seed_lo, d.seed_hi, w);
    const uint32_t a = sel ? w[1] : w[0], b = sel ? w[3] : w[2];
    bits |= (a >= d.threshold ? 1u : 0u) << (2 * j);
    bits |= (b >= d.threshold ? 1u : 0u) << (2 * j + 1);
  }
  return bits;
}

// The factors of score elements 2 i and 2 i + 1 of a thread's 32: 1 / (1 - p) where kept, 0 where dropped.
__device__ __forceinline__ float2 dropout_factors(uint32_t bits, int i, float inv_keep) {
  return make_float2((bits >> (2 * i)) & 1u ? inv_keep : 0.f, (bits >> (2 * i + 1)) & 1u ? inv_keep : 0.f);
}
#endif

}  // namespace jvpfa
