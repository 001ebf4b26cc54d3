// CUDA-core (fp32 FMA) kernels for the shapes the tensor-core kernels do not take: fp32 inputs
// (which must meet a 1e-4 tolerance that TF32 cannot) and head dimensions other than 64 / 128.
// Same mathematics and the same three-family split as the tensor-core kernels, 32x32 score tiles,
// all operands staged in shared memory as fp32, transposed ([d][row], row pitch 33) so that both
// the score products and the output products read shared memory without bank conflicts.
//
// Forward follows the reference's _attn_fwd / _attn_fwd_inner (jvp_flash_attention/jvp_attention.py:
// 673-1044, 136-347); backward follows _attn_bwd_dkdv / _attn_bwd_dq (:1426-1574, 1578-1718)
// extended with the tangent-output terms. Head dimension up to 256 (above 128 the backward streams its column-side
// tiles in two 128-wide chunks of the head dimension to stay inside shared memory).
#include <type_traits>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include "host_common.h"
#include "mask_common.cuh"

namespace jvpfa {
namespace {

constexpr int TB = 32;       // tile edge (rows and columns)
constexpr int PITCH = 33;    // padded pitch of transposed tiles
constexpr int NTHREADS = 256;
constexpr int kMaxD = 256;
constexpr int kChunkD = 128;   // widest slice of the head dimension the backward keeps of a column-side tile

enum { FAM_Q = 0, FAM_K = 1, FAM_V = 2 };

template <typename T> __device__ __forceinline__ float to_f(T x);
template <> __device__ __forceinline__ float to_f<float>(float x) { return x; }
template <> __device__ __forceinline__ float to_f<__half>(__half x) { return __half2float(x); }
template <> __device__ __forceinline__ float to_f<__nv_bfloat16>(__nv_bfloat16 x) { return __bfloat162float(x); }
template <typename T> __device__ __forceinline__ T from_f(float x);
template <> __device__ __forceinline__ float from_f<float>(float x) { return x; }
template <> __device__ __forceinline__ __half from_f<__half>(float x) { return __float2half_rn(x); }
template <> __device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float x) { return __float2bfloat16_rn(x); }

// dst[d * PITCH + r] = src[(row0 + r) * D + d] for r < TB (zero where row0 + r >= N)
// transposed tile: dst[d - d0][r] = src[row0 + r][d] for d in [d0, d0 + dn)
template <typename T>
__device__ __forceinline__ void load_tile_t(float* dst, const T* src, int row0, int N, int D, int d0, int dn) {
  for (int idx = threadIdx.x; idx < TB * dn; idx += NTHREADS) {
    const int r = idx / dn, d = idx - r * dn;
    const int row = row0 + r;
    dst[d * PITCH + r] = (row < N) ? to_f<T>(src[static_cast<size_t>(row) * D + d0 + d]) : 0.f;
  }
}
template <typename T>
__device__ __forceinline__ void load_tile_t(float* dst, const T* src, int row0, int N, int D) {
  load_tile_t<T>(dst, src, row0, N, D, 0, D);
}

struct GenParams {
  int H, N, D;
  int causal;
  float s;
  float c1;
  MaskView mv;
  const float4* stats;
  float out_scale;
  int dual;   // 0: primal-only backward, tangent tensors are absent
};

// score block of this thread: rows ty + 16 i, cols tx + 16 j (i, j < 2); acc[i][j] += sum_d A[d][row] B[d][col]
__device__ __forceinline__ void score_mac(float (&acc)[2][2], const float* At, const float* Bt, int D, int ty, int tx) {
#pragma unroll 4
  for (int d = 0; d < D; ++d) {
    const float a0 = At[d * PITCH + ty], a1 = At[d * PITCH + ty + 16];
    const float b0 = Bt[d * PITCH + tx], b1 = Bt[d * PITCH + tx + 16];
    acc[0][0] = fmaf(a0, b0, acc[0][0]);
    acc[0][1] = fmaf(a0, b1, acc[0][1]);
    acc[1][0] = fmaf(a1, b0, acc[1][0]);
    acc[1][1] = fmaf(a1, b1, acc[1][1]);
  }
}

// out block of this thread: rows ty + 16 i, d-columns tx + 16 j (j < D/16 rounded up);
// acc[i][j] += sum_c E[row][c] * Ct[dcol][c]
// Ct holds the head-dimension slice [16 J0, 16 (J0 + NJC)) of the tile, D is the full head dimension
template <int NJ, int J0 = 0, int NJC = NJ>
__device__ __forceinline__ void out_mac(float (&acc)[2][NJ], const float* E, const float* Ct, int D, int ty, int tx) {
#pragma unroll 2
  for (int c = 0; c < TB; ++c) {
    const float e0 = E[ty * PITCH + c], e1 = E[(ty + 16) * PITCH + c];
#pragma unroll
    for (int j = 0; j < NJC; ++j) {
      const int dc = tx + 16 * j;
      if (16 * J0 + dc < D) {
        const float v = Ct[dc * PITCH + c];
        acc[0][J0 + j] = fmaf(e0, v, acc[0][J0 + j]);
        acc[1][J0 + j] = fmaf(e1, v, acc[1][J0 + j]);
      }
    }
  }
}

__device__ __forceinline__ float half_warp_max(float x) {
#pragma unroll
  for (int off = 8; off > 0; off >>= 1) x = fmaxf(x, __shfl_xor_sync(0xFFFFFFFFu, x, off));
  return x;
}
__device__ __forceinline__ float half_warp_sum(float x) {
#pragma unroll
  for (int off = 8; off > 0; off >>= 1) x += __shfl_xor_sync(0xFFFFFFFFu, x, off);
  return x;
}

// additive bias (log2 domain) of score element (q, k): causal, bounds, mask
__device__ __forceinline__ float elem_bias(const GenParams& p, int b, int h, int q, int k, bool use_mask) {
  if (q >= p.N || k >= p.N) return -INFINITY;
  if (p.causal && k > q) return -INFINITY;
  if (use_mask) {
    const int64_t idx = b * p.mv.s0 + h * p.mv.s1 + static_cast<int64_t>(q) * p.mv.s2 + static_cast<int64_t>(k) * p.mv.s3;
    if (p.mv.kind == JVPFA_MASK_BOOL) return static_cast<const uint8_t*>(p.mv.ptr)[idx] ? 0.f : -INFINITY;
    return mask_elem_as_float(p.mv.ptr, idx, p.mv.dtype) * 1.4426950408889634f;
  }
  return 0.f;
}

__device__ __forceinline__ uint8_t tile32_bits(const MaskView& mv, int b, int h, int qt32, int kt32) {
  return mask_tile_bits(mv, b, h, qt32 >> 1, kt32 >> 1);
}

// ------------------------------------------------------------------------------------------- forward
template <typename T, int NJ, bool DUAL>
__global__ void __launch_bounds__(NTHREADS)
generic_fwd_kernel(const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v, const T* __restrict__ tq,
                   const T* __restrict__ tk, const T* __restrict__ tv, T* __restrict__ o, T* __restrict__ to,
                   float* __restrict__ lse2, float* __restrict__ mu_out, GenParams p) {
  extern __shared__ float sm[];
  const int D = p.D, N = p.N;
  const int tile = D * PITCH;
  float* Qt = sm;
  float* tQt = Qt + tile;
  float* Kt = tQt + tile;
  float* tKt = Kt + tile;
  float* Vt = tKt + tile;
  float* tVt = Vt + tile;
  float* Ps = tVt + tile;
  float* Ws = Ps + TB * PITCH;
  const int ty = threadIdx.x >> 4, tx = threadIdx.x & 15;
  const int qt = p.causal ? (gridDim.x - 1 - blockIdx.x) : blockIdx.x;
  const int bh = blockIdx.y, b = bh / p.H, h = bh % p.H;
  const size_t base = static_cast<size_t>(bh) * N * D;
  const int q0 = qt * TB;
  load_tile_t<T>(Qt, q + base, q0, N, D);
  if (DUAL) load_tile_t<T>(tQt, tq + base, q0, N, D);
  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f}, mu[2] = {0.f, 0.f};
  float accO[2][NJ], accT[2][NJ];
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int j = 0; j < NJ; ++j) { accO[i][j] = 0.f; accT[i][j] = 0.f; }
  int n_kt = (N + TB - 1) / TB;
  if (p.causal) n_kt = min(n_kt, qt + 1);
  for (int kt = 0; kt < n_kt; ++kt) {
    const uint8_t bits = p.mv.kind == JVPFA_MASK_NONE ? kTileAnyKept : tile32_bits(p.mv, b, h, qt, kt);
    if (!(bits & kTileAnyKept)) continue;
    const int k0 = kt * TB;
    __syncthreads();  // previous tile's products are done with the shared tiles
    load_tile_t<T>(Kt, k + base, k0, N, D);
    load_tile_t<T>(Vt, v + base, k0, N, D);
    if (DUAL) {
      load_tile_t<T>(tKt, tk + base, k0, N, D);
      load_tile_t<T>(tVt, tv + base, k0, N, D);
    }
    __syncthreads();
    float S[2][2] = {{0.f, 0.f}, {0.f, 0.f}}, tS[2][2] = {{0.f, 0.f}, {0.f, 0.f}};
    score_mac(S, Qt, Kt, D, ty, tx);
    if (DUAL) {
      score_mac(tS, tQt, Kt, D, ty, tx);
      score_mac(tS, Qt, tKt, D, ty, tx);
    }
    const bool use_mask = p.mv.kind != JVPFA_MASK_NONE && (bits & kTileAnyMasked);
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int qi = q0 + ty + 16 * i;
      float x[2];
#pragma unroll
      for (int j = 0; j < 2; ++j) x[j] = S[i][j] * p.c1 + elem_bias(p, b, h, qi, k0 + tx + 16 * j, use_mask);
      const float m_tile = half_warp_max(fmaxf(x[0], x[1]));
      const float m_new = fmaxf(m[i], m_tile);
      const float alpha = (m[i] == -INFINITY) ? 1.f : exp2f(m[i] - m_new);
      const float m_eff = (m_new == -INFINITY) ? 0.f : m_new;
      float ps = 0.f, ws = 0.f;
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const float pv = exp2f(x[j] - m_eff);
        const float wv = pv * (tS[i][j] * p.s);
        ps += pv;
        ws += wv;
        Ps[(ty + 16 * i) * PITCH + tx + 16 * j] = pv;
        Ws[(ty + 16 * i) * PITCH + tx + 16 * j] = wv;
      }
      l[i] = l[i] * alpha + half_warp_sum(ps);
      mu[i] = mu[i] * alpha + half_warp_sum(ws);
      m[i] = m_new;
#pragma unroll
      for (int j = 0; j < NJ; ++j) { accO[i][j] *= alpha; accT[i][j] *= alpha; }
    }
    __syncthreads();
    out_mac<NJ>(accO, Ps, Vt, D, ty, tx);
    if (DUAL) {
      out_mac<NJ>(accT, Ws, Vt, D, ty, tx);
      out_mac<NJ>(accT, Ps, tVt, D, ty, tx);
    }
  }
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int qi = q0 + ty + 16 * i;
    if (qi >= N) continue;
    const float linv = l[i] > 0.f ? 1.f / l[i] : 0.f;
    const float mul = mu[i] * linv;
#pragma unroll
    for (int j = 0; j < NJ; ++j) {
      const int dc = tx + 16 * j;
      if (dc < D) {
        const float ov = accO[i][j] * linv;
        o[base + static_cast<size_t>(qi) * D + dc] = from_f<T>(ov);
        if (DUAL) to[base + static_cast<size_t>(qi) * D + dc] = from_f<T>(accT[i][j] * linv - mul * ov);
      }
    }
    if (tx == 0) {
      lse2[static_cast<size_t>(bh) * N + qi] = l[i] > 0.f ? m[i] + log2f(l[i]) : -INFINITY;
      mu_out[static_cast<size_t>(bh) * N + qi] = mul;
    }
  }
}

// ------------------------------------------------------------------------------------------- backward
// stats[row] = (lse2, mu, Delta, a); one warp per row, any element type.
template <typename T>
__global__ void generic_preprocess_kernel(const T* __restrict__ o, const T* __restrict__ to, const T* __restrict__ go,
                                          const T* __restrict__ gto, const float* __restrict__ lse2,
                                          const float* __restrict__ mu, float4* __restrict__ stats, int64_t rows, int D) {
  const int64_t row = static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= rows) return;
  float s1 = 0.f, s2 = 0.f, s3 = 0.f;
  for (int d = lane; d < D; d += 32) {
    const size_t idx = static_cast<size_t>(row) * D + d;
    const float fo = to_f<T>(o[idx]), fto = gto ? to_f<T>(to[idx]) : 0.f, fgo = to_f<T>(go[idx]);
    const float fgto = gto ? to_f<T>(gto[idx]) : 0.f;
    s1 = fmaf(fgo, fo, s1);
    s2 = fmaf(fgto, fto, s2);
    s3 = fmaf(fgto, fo, s3);
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) {
    s1 += __shfl_xor_sync(0xFFFFFFFFu, s1, off);
    s2 += __shfl_xor_sync(0xFFFFFFFFu, s2, off);
    s3 += __shfl_xor_sync(0xFFFFFFFFu, s3, off);
  }
  if (lane == 0) {
    const float m = mu[row];
    stats[row] = make_float4(lse2[row], m, s1 + s2 - s3 * m, s3);
  }
}

// Row tile of 32 positions (queries for family Q, keys for K and V), streamed 32-wide column tiles.
//  family Q: R = Q, tQ, gO, gtO;  C = K, tK, V, tV   -> dQ, dtQ
//  family K: R = K, tK, V, tV;    C = Q, tQ, gO, gtO -> dK, dtK
//  family V: R = K, tK;           C = Q, tQ, gO, gtO -> dV, dtV
template <typename T, int NJ, int FAM>
__global__ void __launch_bounds__(NTHREADS)
generic_bwd_kernel(const T* __restrict__ r0p, const T* __restrict__ r1p, const T* __restrict__ r2p,
                   const T* __restrict__ r3p, const T* __restrict__ c0p, const T* __restrict__ c1p,
                   const T* __restrict__ c2p, const T* __restrict__ c3p, T* __restrict__ out0, T* __restrict__ out1,
                   GenParams p) {
  extern __shared__ float sm[];
  const int D = p.D, N = p.N;
  const int tile = D * PITCH;
  constexpr bool CHUNKED = NJ > kChunkD / 16;          // head dimension above 128: column-side tiles in two slices
  const int ctile = (CHUNKED ? kChunkD : D) * PITCH;
  float* R0 = sm;
  float* R1 = R0 + tile;
  float* R2 = R1 + tile;
  float* R3 = R2 + tile;
  float* C0 = R3 + tile;
  float* C1 = C0 + ctile;
  float* C2 = C1 + ctile;
  float* C3 = C2 + ctile;
  float* E0 = C3 + ctile;
  float* E1 = E0 + TB * PITCH;
  float4* st_s = reinterpret_cast<float4*>(E1 + TB * PITCH + 3);  // keep 16-byte alignment below
  st_s = reinterpret_cast<float4*>((reinterpret_cast<uintptr_t>(st_s) + 15) & ~uintptr_t(15));
  const int ty = threadIdx.x >> 4, tx = threadIdx.x & 15;
  const int rt = (p.causal && FAM == FAM_Q) ? (gridDim.x - 1 - blockIdx.x) : blockIdx.x;
  const int bh = blockIdx.y, b = bh / p.H, h = bh % p.H;
  const size_t base = static_cast<size_t>(bh) * N * D;
  const int r0 = rt * TB;
  load_tile_t<T>(R0, r0p + base, r0, N, D);
  const bool dual = p.dual != 0;
  if (dual) load_tile_t<T>(R1, r1p + base, r0, N, D);
  if (FAM != FAM_V) {
    load_tile_t<T>(R2, r2p + base, r0, N, D);
    if (dual) load_tile_t<T>(R3, r3p + base, r0, N, D);
  }
  float acc0[2][NJ], acc1[2][NJ];
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int j = 0; j < NJ; ++j) { acc0[i][j] = 0.f; acc1[i][j] = 0.f; }
  const int n_ct = (N + TB - 1) / TB;
  int j_begin = 0, j_end = n_ct;
  if (p.causal) {
    if (FAM == FAM_Q) j_end = min(n_ct, rt + 1);
    else j_begin = rt;
  }
  for (int ct = j_begin; ct < j_end; ++ct) {
    uint8_t bits = kTileAnyKept;
    if (p.mv.kind != JVPFA_MASK_NONE) bits = (FAM == FAM_Q) ? tile32_bits(p.mv, b, h, rt, ct) : tile32_bits(p.mv, b, h, ct, rt);
    if (!(bits & kTileAnyKept)) continue;
    const int c0 = ct * TB;
    // column-side tiles, head-dimension slice [d0, d0 + dn)
    auto load_c = [&](int d0, int dn) {
      load_tile_t<T>(C0, c0p + base, c0, N, D, d0, dn);
      if (dual) load_tile_t<T>(C1, c1p + base, c0, N, D, d0, dn);
      load_tile_t<T>(C2, c2p + base, c0, N, D, d0, dn);
      if (dual) load_tile_t<T>(C3, c3p + base, c0, N, D, d0, dn);
    };
    __syncthreads();
    load_c(0, CHUNKED ? kChunkD : D);
    // statistics of the query positions of this tile pair
    if (threadIdx.x < TB) {
      const int qpos = (FAM == FAM_Q ? r0 : c0) + threadIdx.x;
      float4 sv = make_float4(INFINITY, 0.f, 0.f, 0.f);
      if (qpos < N) {
        sv = p.stats[static_cast<size_t>(bh) * N + qpos];
        if (sv.x == -INFINITY) sv.x = INFINITY;
      }
      st_s[threadIdx.x] = sv;
    }
    __syncthreads();
    float T0[2][2] = {{0.f, 0.f}, {0.f, 0.f}}, T1[2][2] = {{0.f, 0.f}, {0.f, 0.f}};
    float T2[2][2] = {{0.f, 0.f}, {0.f, 0.f}}, T3[2][2] = {{0.f, 0.f}, {0.f, 0.f}};
    // score products over the head-dimension slice of length dn that starts at row-side offset ro (floats)
    auto scores = [&](int ro, int dn) {
      score_mac(T0, R0 + ro, C0, dn, ty, tx);
      if (dual) {
        score_mac(T1, R1 + ro, C0, dn, ty, tx);
        score_mac(T1, R0 + ro, C1, dn, ty, tx);
      }
      if (FAM != FAM_V) {
        score_mac(T2, R2 + ro, C2, dn, ty, tx);
        if (dual) {
          score_mac(T2, R3 + ro, C3, dn, ty, tx);
          if (FAM == FAM_Q) score_mac(T3, R3 + ro, C2, dn, ty, tx);
          else score_mac(T3, R2 + ro, C3, dn, ty, tx);
        }
      }
    };
    if constexpr (CHUNKED) {
      scores(0, kChunkD);
      __syncthreads();
      load_c(kChunkD, D - kChunkD);
      __syncthreads();
      scores(kChunkD * PITCH, D - kChunkD);
    } else {
      scores(0, D);
    }
    const bool use_mask = p.mv.kind != JVPFA_MASK_NONE && (bits & kTileAnyMasked);
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const int rr = ty + 16 * i, cc = tx + 16 * j;
        const int qpos = (FAM == FAM_Q) ? r0 + rr : c0 + cc;
        const int kpos = (FAM == FAM_Q) ? c0 + cc : r0 + rr;
        const float4 sq = st_s[(FAM == FAM_Q) ? rr : cc];
        const float P = exp2f(T0[i][j] * p.c1 + elem_bias(p, b, h, qpos, kpos, use_mask) - sq.x);
        const float ts = T1[i][j] * p.s;
        float v0, v1;
        if (FAM == FAM_V) {
          v0 = P;
          v1 = P * (ts - sq.y);
        } else {
          const float dp = T2[i][j] + T3[i][j] * (ts - sq.y) - sq.w * ts;
          v0 = P * (dp - sq.z);
          v1 = P * (T3[i][j] - sq.w);
        }
        E0[rr * PITCH + cc] = v0;
        E1[rr * PITCH + cc] = v1;
      }
    __syncthreads();
    // output products for the head-dimension columns [16 J0, 16 (J0 + NJC)) held in the column-side tiles
    auto outputs = [&](auto j0, auto njc) {
      constexpr int J0 = decltype(j0)::value, NJC = decltype(njc)::value;
      if (FAM == FAM_V) {
        out_mac<NJ, J0, NJC>(acc0, E0, C2, D, ty, tx);
        if (dual) {
          out_mac<NJ, J0, NJC>(acc0, E1, C3, D, ty, tx);
          out_mac<NJ, J0, NJC>(acc1, E0, C3, D, ty, tx);
        }
      } else {
        out_mac<NJ, J0, NJC>(acc0, E0, C0, D, ty, tx);
        if (dual) {
          out_mac<NJ, J0, NJC>(acc0, E1, C1, D, ty, tx);
          out_mac<NJ, J0, NJC>(acc1, E1, C0, D, ty, tx);
        }
      }
    };
    if constexpr (CHUNKED) {
      constexpr int JC = kChunkD / 16;
      outputs(std::integral_constant<int, JC>{}, std::integral_constant<int, NJ - JC>{});   // second slice is loaded
      __syncthreads();
      load_c(0, kChunkD);
      __syncthreads();
      outputs(std::integral_constant<int, 0>{}, std::integral_constant<int, JC>{});
    } else {
      outputs(std::integral_constant<int, 0>{}, std::integral_constant<int, NJ>{});
    }
  }
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int row = r0 + ty + 16 * i;
    if (row >= N) continue;
#pragma unroll
    for (int j = 0; j < NJ; ++j) {
      const int dc = tx + 16 * j;
      if (dc < D) {
        out0[base + static_cast<size_t>(row) * D + dc] = from_f<T>(acc0[i][j] * p.out_scale);
        if (dual) out1[base + static_cast<size_t>(row) * D + dc] = from_f<T>(acc1[i][j] * p.out_scale);
      }
    }
  }
}

GenParams make_params(int H, int N, int D, int causal, float s, const jvpfa_mask& mask, const uint8_t* summary) {
  GenParams p{};
  p.H = H; p.N = N; p.D = D; p.causal = causal; p.s = s; p.c1 = s * 1.4426950408889634f;
  p.mv.ptr = mask.ptr; p.mv.summary = summary;
  p.mv.s0 = mask.stride[0]; p.mv.s1 = mask.stride[1]; p.mv.s2 = mask.stride[2]; p.mv.s3 = mask.stride[3];
  p.mv.kind = mask.kind; p.mv.dtype = mask.dtype;
  p.mv.n64 = (N + 63) / 64;
  p.mv.Hm = mask.stride[1] == 0 ? 1 : H;
  p.out_scale = 1.f;
  return p;
}

template <typename T, int NJ>
int fwd_typed(const jvpfa_fwd_args& a, cudaStream_t stream) {
  GenParams p = make_params(a.H, a.N, a.D, a.causal, a.sm_scale, a.mask, a.mask_summary);
  const bool dual = a.tq != nullptr;
  const size_t smem = (6 * static_cast<size_t>(a.D) * PITCH + 2 * TB * PITCH) * sizeof(float);
  dim3 grid((a.N + TB - 1) / TB, a.B * a.H);
  auto launch = [&](auto kern) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)) != cudaSuccess)
      return JVPFA_ERR_LAUNCH;
    kern<<<grid, NTHREADS, smem, stream>>>(static_cast<const T*>(a.q), static_cast<const T*>(a.k),
                                           static_cast<const T*>(a.v), static_cast<const T*>(a.tq),
                                           static_cast<const T*>(a.tk), static_cast<const T*>(a.tv),
                                           static_cast<T*>(a.o), static_cast<T*>(a.to), a.lse2, a.mu, p);
    return cudaGetLastError() == cudaSuccess ? JVPFA_OK : JVPFA_ERR_LAUNCH;
  };
  return dual ? launch(generic_fwd_kernel<T, NJ, true>) : launch(generic_fwd_kernel<T, NJ, false>);
}

template <typename T>
int fwd_by_d(const jvpfa_fwd_args& a, cudaStream_t stream) {
  if (a.D <= 32) return fwd_typed<T, 2>(a, stream);
  if (a.D <= 64) return fwd_typed<T, 4>(a, stream);
  if (a.D <= 128) return fwd_typed<T, 8>(a, stream);
  return fwd_typed<T, 16>(a, stream);
}

template <typename T, int NJ, int FAM>
int bwd_family(const jvpfa_bwd_args& a, const float4* stats, cudaStream_t stream) {
  GenParams p = make_params(a.H, a.N, a.D, a.causal, a.sm_scale, a.mask, a.mask_summary);
  p.stats = stats;
  p.dual = a.tq != nullptr;
  const T *r[4], *c[4];
  T *o0, *o1;
  auto cp = [](const void* x) { return static_cast<const T*>(x); };
  if (FAM == FAM_Q) {
    r[0] = cp(a.q); r[1] = cp(a.tq); r[2] = cp(a.go); r[3] = cp(a.gto);
    c[0] = cp(a.k); c[1] = cp(a.tk); c[2] = cp(a.v); c[3] = cp(a.tv);
    o0 = static_cast<T*>(a.dq); o1 = static_cast<T*>(a.dtq); p.out_scale = a.sm_scale;
  } else if (FAM == FAM_K) {
    r[0] = cp(a.k); r[1] = cp(a.tk); r[2] = cp(a.v); r[3] = cp(a.tv);
    c[0] = cp(a.q); c[1] = cp(a.tq); c[2] = cp(a.go); c[3] = cp(a.gto);
    o0 = static_cast<T*>(a.dk); o1 = static_cast<T*>(a.dtk); p.out_scale = a.sm_scale;
  } else {
    r[0] = cp(a.k); r[1] = cp(a.tk); r[2] = cp(a.k); r[3] = cp(a.tk);
    c[0] = cp(a.q); c[1] = cp(a.tq); c[2] = cp(a.go); c[3] = cp(a.gto);
    o0 = static_cast<T*>(a.dv); o1 = static_cast<T*>(a.dtv); p.out_scale = 1.f;
  }
  const size_t cD = a.D > kChunkD ? kChunkD : a.D;   // column-side tiles hold at most 128 head-dimension columns
  const size_t smem = (4 * (static_cast<size_t>(a.D) + cD) * PITCH + 2 * TB * PITCH + 8) * sizeof(float) + TB * sizeof(float4) + 16;
  auto kern = generic_bwd_kernel<T, NJ, FAM>;
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)) != cudaSuccess)
    return JVPFA_ERR_LAUNCH;
  dim3 grid((a.N + TB - 1) / TB, a.B * a.H);
  kern<<<grid, NTHREADS, smem, stream>>>(r[0], r[1], r[2], r[3], c[0], c[1], c[2], c[3], o0, o1, p);
  return cudaGetLastError() == cudaSuccess ? JVPFA_OK : JVPFA_ERR_LAUNCH;
}

template <typename T, int NJ>
int bwd_typed(const jvpfa_bwd_args& a, cudaStream_t stream, const LaunchMarks& marks) {
  const int64_t rows = static_cast<int64_t>(a.B) * a.H * a.N;
  float4* stats = reinterpret_cast<float4*>(static_cast<uint8_t*>(a.workspace) + kStatusBytes);
  const unsigned blocks = static_cast<unsigned>((rows + 7) / 8);
  marks.mark(0);
  generic_preprocess_kernel<T><<<blocks, 256, 0, stream>>>(static_cast<const T*>(a.o), static_cast<const T*>(a.to),
                                                         static_cast<const T*>(a.go), static_cast<const T*>(a.gto),
                                                         a.lse2, a.mu, stats, rows, a.D);
  if (cudaGetLastError() != cudaSuccess) return JVPFA_ERR_LAUNCH;
  marks.mark(1);
  int rc = bwd_family<T, NJ, FAM_Q>(a, stats, stream);
  if (rc != JVPFA_OK) return rc;
  marks.mark(2);
  rc = bwd_family<T, NJ, FAM_K>(a, stats, stream);
  if (rc != JVPFA_OK) return rc;
  marks.mark(3);
  rc = bwd_family<T, NJ, FAM_V>(a, stats, stream);
  marks.mark(4);
  return rc;
}

template <typename T>
int bwd_by_d(const jvpfa_bwd_args& a, cudaStream_t stream, const LaunchMarks& marks) {
  if (a.D <= 32) return bwd_typed<T, 2>(a, stream, marks);
  if (a.D <= 64) return bwd_typed<T, 4>(a, stream, marks);
  if (a.D <= 128) return bwd_typed<T, 8>(a, stream, marks);
  return bwd_typed<T, 16>(a, stream, marks);
}

}  // namespace

int launch_fwd_generic(const jvpfa_fwd_args& a, cudaStream_t stream) {
  if (a.D > kMaxD) return JVPFA_ERR_UNSUPPORTED;
  switch (a.dtype) {
    case JVPFA_F32: return fwd_by_d<float>(a, stream);
    case JVPFA_F16: return fwd_by_d<__half>(a, stream);
    case JVPFA_BF16: return fwd_by_d<__nv_bfloat16>(a, stream);
    default: return JVPFA_ERR_UNSUPPORTED;
  }
}

size_t bwd_generic_workspace_bytes(const jvpfa_bwd_args& a) {
  return kStatusBytes + static_cast<size_t>(a.B) * a.H * a.N * sizeof(float4);
}

int launch_bwd_generic(const jvpfa_bwd_args& a, cudaStream_t stream, const LaunchMarks& marks) {
  if (a.D > kMaxD) return JVPFA_ERR_UNSUPPORTED;
  switch (a.dtype) {
    case JVPFA_F32: return bwd_by_d<float>(a, stream, marks);
    case JVPFA_F16: return bwd_by_d<__half>(a, stream, marks);
    case JVPFA_BF16: return bwd_by_d<__nv_bfloat16>(a, stream, marks);
    default: return JVPFA_ERR_UNSUPPORTED;
  }
}

}  // namespace jvpfa
