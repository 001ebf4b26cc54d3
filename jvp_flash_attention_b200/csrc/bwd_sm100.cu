// Dual (JVP) attention backward for sm_100a: gradients of sum(O*gO) + sum(tO*gtO) with respect to
// Q, K, V and the tangent inputs tQ, tK, tV, with tcgen05 MMAs accumulating in TMEM.
//
// Replaces the reference's _attn_bwd / _attn_bwd_causal (+ _attn_bwd_dkdv, _attn_bwd_dq)
// (jvp_flash_attention/jvp_attention.py:2019-2244, 1721-2016, 1426-1574, 1578-1718) and adds the
// gradient through the tangent output and the tangent-input gradients, which the reference does
// not compute (jvp_attention.py:3081, 3226).
//
// One kernel template, three output families. A CTA owns a "row" tile of 128 sequence positions
// whose operands stay in shared memory, and streams 64-wide "column" tiles of the other side:
//   family Q : rows = queries.  scores S, tS, X, A (q on TMEM lanes)    -> dQ, dtQ
//   family K : rows = keys.     transposed scores (k on TMEM lanes)      -> dK, dtK
//   family V : rows = keys.     transposed S, tS only                    -> dV, dtV
// with  S = Q K^T, tS = tQ K^T + Q tK^T, X = gO V^T + gtO tV^T, A = gtO V^T and per score element
//   P = exp2(c1 S + bias - lse2_q), ts = s tS, dtS = P (A - a_q),
//   dS = P (X + A (ts - mu_q) - a_q ts - Delta_q), tP = P (ts - mu_q);
//   dQ = s (dS K + dtS tK), dtQ = s dtS K, dK = s (dS^T Q + dtS^T tQ), dtK = s dtS^T Q,
//   dV = P^T gO + tP^T gtO, dtV = P^T gtO.
// The per-query statistics (lse2, mu, Delta, a) come packed as one float4 per query from the
// preprocess kernel. Family Q reads them per thread (thread = query row); families K and V stage
// the 64 statistics of the current query tile in shared memory and read them as broadcasts.
//
// Roles as in the forward kernel: warps 0-3 element-wise (thread r = TMEM lane r), warp 4 TMA
// producer, warp 5 MMA issuer. Column-side tiles flow through a ring of shared-memory slots in the
// order in which the MMA issuer releases them (tiles only the score MMAs read come first).
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include "host_common.h"
#include "mask_common.cuh"
#include "sm100_prims.cuh"

namespace jvpfa {
using namespace sm100;

namespace {

enum { FAM_Q = 0, FAM_K = 1, FAM_V = 2 };

struct BwdKParams {
  int H, N;
  int causal;
  float c1;  // sm_scale * log2(e)
  float s;   // sm_scale
  float out_scale;
  MaskView mv;
  const float4* stats;  // per (b,h,q): lse2, mu, Delta, a
  void* out0;
  void* out1;
  int* status;
  uint64_t budget_ns;
};

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

template <bool BF16>
__device__ __forceinline__ uint32_t pack2(float a, float b) {
  if constexpr (BF16) {
    __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
  } else {
    __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
  }
}

template <int D, int FAM>
struct BwdCfg {
  static constexpr int BR = 128;                         // rows per CTA
  static constexpr int BC = 64;                          // columns per streamed tile
  static constexpr int NR = (FAM == FAM_V) ? 2 : 4;      // resident row-side operand tiles
  static constexpr int NSLOT = (D == 128 && FAM != FAM_V) ? 6 : 8;
  static constexpr int TILE_R = BR * D * 2;
  static constexpr int TILE_C = BC * D * 2;
  static constexpr int TMEM_ACC0 = 0;
  static constexpr int TMEM_ACC1 = D;
  static constexpr int TMEM_T = 2 * D;                   // score tiles T0..T3, 64 columns each
  static constexpr int TMEM_COLS = 512;
  static constexpr size_t smem_bytes() { return NR * TILE_R + NSLOT * TILE_C + 2 * BC * 16 + (6 + 2 * NSLOT) * 8; }
};

// rmK: row-side tensor maps (box 128 rows); cmK: column-side tensor maps in ring (load) order.
//  family Q: rm = Q, tQ, gO, gtO;  cm = V, tV, K, tK
//  family K: rm = K, tK, V, tV;    cm = gO, gtO, Q, tQ
//  family V: rm = K, tK, (unused); cm = Q, tQ, gO, gtO
template <int D, int FAM, bool BF16>
__global__ void __launch_bounds__(192, 1)
bwd_sm100_kernel(const __grid_constant__ CUtensorMap rm0, const __grid_constant__ CUtensorMap rm1,
                 const __grid_constant__ CUtensorMap rm2, const __grid_constant__ CUtensorMap rm3,
                 const __grid_constant__ CUtensorMap cm0, const __grid_constant__ CUtensorMap cm1,
                 const __grid_constant__ CUtensorMap cm2, const __grid_constant__ CUtensorMap cm3,
                 const BwdKParams p) {
  using C = BwdCfg<D, FAM>;
  constexpr int NS = C::NSLOT;

  // Everything lives in dynamic shared memory so that the 128-byte-swizzled tiles can start at its
  // 1024-byte-aligned base without alignment slack: tiles, then statistics, then barriers.
  extern __shared__ __align__(1024) uint8_t smem[];
  auto sR = [&](int i) { return smem + i * C::TILE_R; };
  auto sSlot = [&](int k) { return smem + C::NR * C::TILE_R + k * C::TILE_C; };
  uint8_t* tail = smem + C::NR * C::TILE_R + NS * C::TILE_C;
  float4(*stats_s)[C::BC] = reinterpret_cast<float4(*)[C::BC]>(tail);
  uint64_t* bars = reinterpret_cast<uint64_t*>(tail + 2 * C::BC * sizeof(float4));
  uint64_t& r_full = bars[0];
  uint64_t& s_full = bars[1];
  uint64_t& p_full = bars[2];
  uint64_t& acc_final = bars[3];
  uint64_t* c_full = bars + 4;
  uint64_t* c_empty = bars + 4 + NS;
  uint32_t& tmem_base_s = *reinterpret_cast<uint32_t*>(bars + 4 + 2 * NS);
  int& poisoned = *reinterpret_cast<int*>(bars + 5 + 2 * NS);
  if ((smem_u32(smem) & 1023u) != 0u) {  // the swizzled layouts need this; never observed otherwise
    if (threadIdx.x == 0) atomicCAS(p.status, 0, WAIT_TIMEOUT_BASE + 99);
    return;
  }

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int n_rt = gridDim.x;
  // heavier tiles first under a causal mask: late query tiles, early key tiles
  const int rt = (p.causal && FAM == FAM_Q) ? (n_rt - 1 - static_cast<int>(blockIdx.x)) : blockIdx.x;
  const int bh = blockIdx.y;
  const int b = bh / p.H, h = bh % p.H;
  const int r0 = rt * C::BR;
  const int N = p.N;
  const int row_base = bh * N;
  const int n_ct = (N + C::BC - 1) / C::BC;
  int j_begin = 0, j_end = n_ct;
  if (p.causal) {
    if (FAM == FAM_Q) j_end = min(n_ct, (r0 + C::BR - 1) / C::BC + 1);
    else j_begin = r0 / C::BC;
  }

  const WaitCtx w{p.status, &poisoned, p.budget_ns};

  if (tid == 0) {
    poisoned = 0;
    mbar_init(&r_full, 1);
    for (int i = 0; i < NS; ++i) {
      mbar_init(&c_full[i], 1);
      mbar_init(&c_empty[i], 1);
    }
    mbar_init(&s_full, 1);
    mbar_init(&p_full, 128);
    mbar_init(&acc_final, 1);
    fence_mbar_init();
  }
  __syncthreads();
  if (warp == 5) {
    tmem_alloc(&tmem_base_s, C::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = tmem_base_s;

  // summary bits of column tile j against this row tile (64x64 summary entries are indexed [q][k])
  auto tile_bits = [&](int j) -> uint8_t {
    if (p.mv.kind == JVPFA_MASK_NONE) return kTileAnyKept;
    uint8_t bits;
    if (FAM == FAM_Q) {
      bits = mask_tile_bits(p.mv, b, h, 2 * rt, j);
      if (2 * rt + 1 < p.mv.n64) bits |= mask_tile_bits(p.mv, b, h, 2 * rt + 1, j);
    } else {
      bits = mask_tile_bits(p.mv, b, h, j, 2 * rt);
      if (2 * rt + 1 < p.mv.n64) bits |= mask_tile_bits(p.mv, b, h, j, 2 * rt + 1);
    }
    return bits;
  };

  if (warp == 4) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      mbar_arrive_expect_tx(&r_full, C::NR * C::TILE_R);
      tma_load_3d(sR(0), &rm0, &r_full, 0, row_base + r0, 0);
      tma_load_3d(sR(1), &rm1, &r_full, 0, row_base + r0, 0);
      if constexpr (C::NR == 4) {
        tma_load_3d(sR(2), &rm2, &r_full, 0, row_base + r0, 0);
        tma_load_3d(sR(3), &rm3, &r_full, 0, row_base + r0, 0);
      }
      const CUtensorMap* cms[4] = {&cm0, &cm1, &cm2, &cm3};
      int g = 0;
      for (int j = j_begin; j < j_end; ++j) {
        if (!(tile_bits(j) & kTileAnyKept)) continue;
        const int crow = row_base + j * C::BC;
#pragma unroll
        for (int e = 0; e < 4; ++e, ++g) {
          const int slot = g % NS;
          const uint32_t ph = (g / NS) & 1;
          mbar_wait(&c_empty[slot], ph ^ 1, w, 10 + e);
          mbar_arrive_expect_tx(&c_full[slot], C::TILE_C);
          tma_load_3d(sSlot(slot), cms[e], &c_full[slot], 0, crow, 0);
        }
      }
    }
    __syncwarp();
  } else if (warp == 5) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t FMT = BF16 ? FMT_BF16 : FMT_F16;
      const uint32_t idesc_sc = make_idesc(FMT, 128, C::BC, 0, 0);
      const uint32_t idesc_out = make_idesc(FMT, 128, D, 0, 1);
      const uint32_t T0 = tmem + C::TMEM_T, T1 = T0 + 64, T2 = T0 + 128, T3 = T0 + 192;
      const uint32_t E0 = (FAM == FAM_V) ? T0 : T2, E1 = (FAM == FAM_V) ? T1 : T3;

      // dst[128 x 64] (+)= R[128 x D] * Cc[64 x D]^T
      auto mma_nt = [&](uint32_t dst, const uint8_t* rtile, const uint8_t* ctile, uint32_t acc) {
        const uint32_t a = smem_u32(rtile), bb = smem_u32(ctile);
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint32_t oa = (k >> 2) * (C::BR * 128) + (k & 3) * 32;
          const uint32_t ob = (k >> 2) * (C::BC * 128) + (k & 3) * 32;
          umma_ss(dst, desc_kmajor_sw128(a + oa), desc_kmajor_sw128(bb + ob), idesc_sc, acc | (k > 0));
        }
      };
      // acc[128 x D] (+)= E[128 x 64] (TMEM, 16-bit) * Cc[64 x D]
      auto mma_out = [&](uint32_t accum, uint32_t e, const uint8_t* ctile, uint32_t acc) {
        const uint32_t bb = smem_u32(ctile);
#pragma unroll
        for (int k = 0; k < C::BC / 16; ++k)
          umma_ts(accum, e + k * 8, desc_mnmajor_sw128(bb + k * 2048, C::BC * 128), idesc_out, acc | (k > 0));
      };

      mbar_wait(&r_full, 0, w, 20);
      int it = 0;
      for (int j = j_begin; j < j_end; ++j) {
        if (!(tile_bits(j) & kTileAnyKept)) continue;
        int slot[4];
        uint32_t ph[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int g = 4 * it + e;
          slot[e] = g % NS;
          ph[e] = (g / NS) & 1;
        }
        const uint32_t acc0 = it > 0;
        if constexpr (FAM == FAM_V) {
          mbar_wait(&c_full[slot[0]], ph[0], w, 21);
          mbar_wait(&c_full[slot[1]], ph[1], w, 22);
          tc_fence_after_sync();
          mma_nt(T0, sR(0), sSlot(slot[0]), 0);  // S^T  = K Q^T
          mma_nt(T1, sR(1), sSlot(slot[0]), 0);  // tS^T = tK Q^T + K tQ^T
          mma_nt(T1, sR(0), sSlot(slot[1]), 1);
          umma_commit(&s_full);
          umma_commit(&c_empty[slot[0]]);
          umma_commit(&c_empty[slot[1]]);
          mbar_wait(&p_full, it & 1, w, 23);
          mbar_wait(&c_full[slot[2]], ph[2], w, 24);
          mbar_wait(&c_full[slot[3]], ph[3], w, 25);
          tc_fence_after_sync();
          mma_out(tmem + C::TMEM_ACC0, E0, sSlot(slot[2]), acc0);  // dV  += P^T gO + tP^T gtO
          mma_out(tmem + C::TMEM_ACC0, E1, sSlot(slot[3]), 1);
          mma_out(tmem + C::TMEM_ACC1, E0, sSlot(slot[3]), acc0);  // dtV += P^T gtO
          umma_commit(&c_empty[slot[2]]);
          umma_commit(&c_empty[slot[3]]);
        } else {
#pragma unroll
          for (int e = 0; e < 4; ++e) mbar_wait(&c_full[slot[e]], ph[e], w, 21 + e);
          tc_fence_after_sync();
          // ring positions: 0,1 = second operand pair (V,tV | gO,gtO), 2,3 = first pair (K,tK | Q,tQ)
          mma_nt(T0, sR(0), sSlot(slot[2]), 0);
          mma_nt(T1, sR(1), sSlot(slot[2]), 0);
          mma_nt(T1, sR(0), sSlot(slot[3]), 1);
          mma_nt(T2, sR(2), sSlot(slot[0]), 0);
          mma_nt(T2, sR(3), sSlot(slot[1]), 1);
          if constexpr (FAM == FAM_Q) mma_nt(T3, sR(3), sSlot(slot[0]), 0);  // A   = gtO V^T
          else mma_nt(T3, sR(2), sSlot(slot[1]), 0);                         // A^T = V gtO^T
          umma_commit(&s_full);
          umma_commit(&c_empty[slot[0]]);
          umma_commit(&c_empty[slot[1]]);
          mbar_wait(&p_full, it & 1, w, 26);
          tc_fence_after_sync();
          mma_out(tmem + C::TMEM_ACC0, E0, sSlot(slot[2]), acc0);
          mma_out(tmem + C::TMEM_ACC0, E1, sSlot(slot[3]), 1);
          mma_out(tmem + C::TMEM_ACC1, E1, sSlot(slot[2]), acc0);
          umma_commit(&c_empty[slot[2]]);
          umma_commit(&c_empty[slot[3]]);
        }
        ++it;
      }
      if (it > 0) umma_commit(&acc_final);
      else mbar_arrive(&acc_final);
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------------ element-wise + epilogue
    const int r = warp * 32 + lane;
    const int gr = r0 + r;             // global sequence index of this thread's row
    const int gr_c = min(gr, N - 1);
    const uint32_t lane_off = static_cast<uint32_t>(warp * 32) << 16;
    const uint32_t T0 = tmem + C::TMEM_T + lane_off, T1 = T0 + 64, T2 = T0 + 128, T3 = T0 + 192;
    const uint32_t E0 = (FAM == FAM_V) ? T0 : T2, E1 = (FAM == FAM_V) ? T1 : T3;
    float4 st_row = make_float4(0.f, 0.f, 0.f, 0.f);
    if (FAM == FAM_Q) {
      st_row = p.stats[static_cast<size_t>(row_base) + gr_c];
      if (st_row.x == -INFINITY) st_row.x = INFINITY;  // fully excluded query: P = 0
    }
    int it = 0;
    for (int j = j_begin; j < j_end; ++j) {
      const uint8_t bits = tile_bits(j);
      if (!(bits & kTileAnyKept)) continue;
      const int c0 = j * C::BC;
      if (FAM != FAM_Q) {
        if (r < C::BC) {
          float4 sv = make_float4(INFINITY, 0.f, 0.f, 0.f);
          if (c0 + r < N) {
            sv = p.stats[static_cast<size_t>(row_base) + c0 + r];
            if (sv.x == -INFINITY) sv.x = INFINITY;
          }
          stats_s[it & 1][r] = sv;
        }
        named_bar_sync(1, 128);
      }
      mbar_wait(&s_full, it & 1, w, 30);
      tc_fence_after_sync();
      const bool need_causal = p.causal && ((FAM == FAM_Q) ? (c0 + C::BC - 1 > r0) : (r0 + C::BR - 1 > c0));
      const bool need_bound = (FAM == FAM_Q) && (c0 + C::BC > N);
      const bool need_mask = p.mv.kind != JVPFA_MASK_NONE && (bits & kTileAnyMasked);
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t t0[16], t1[16], t2[16], t3[16];
        tmem_ld_x16(T0 + 16 * c, t0);
        tmem_ld_x16(T1 + 16 * c, t1);
        if constexpr (FAM != FAM_V) {
          tmem_ld_x16(T2 + 16 * c, t2);
          tmem_ld_x16(T3 + 16 * c, t3);
        }
        float bias[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) bias[i] = 0.f;
        if (need_mask) {
          if (FAM == FAM_Q) mask_bias_run<16>(bias, p.mv, b, h, gr_c, c0 + 16 * c, N, true);
          else mask_bias_run<16>(bias, p.mv, b, h, c0 + 16 * c, gr_c, N, false);
        }
        if (need_causal) {
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const int col = c0 + 16 * c + i;
            const bool ok = (FAM == FAM_Q) ? (col <= gr) : (gr <= col);
            if (!ok) bias[i] = -INFINITY;
          }
        }
        if (need_bound) {
#pragma unroll
          for (int i = 0; i < 16; ++i)
            if (c0 + 16 * c + i >= N) bias[i] = -INFINITY;
        }
        tmem_wait_ld();
        uint32_t e0[8], e1[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          float v0[2], v1[2];
#pragma unroll
          for (int u = 0; u < 2; ++u) {
            const int ii = 2 * i + u;
            float4 sq;
            if (FAM == FAM_Q) sq = st_row;
            else sq = stats_s[it & 1][16 * c + ii];
            const float P = fast_exp2(fmaf(__uint_as_float(t0[ii]), p.c1, bias[ii]) - sq.x);
            const float ts = __uint_as_float(t1[ii]) * p.s;
            if constexpr (FAM == FAM_V) {
              v0[u] = P;
              v1[u] = P * (ts - sq.y);
            } else {
              const float X = __uint_as_float(t2[ii]);
              const float A = __uint_as_float(t3[ii]);
              const float dp = X + A * (ts - sq.y) - sq.w * ts;
              v0[u] = P * (dp - sq.z);   // dS
              v1[u] = P * (A - sq.w);    // dtS
            }
          }
          e0[i] = pack2<BF16>(v0[0], v0[1]);
          e1[i] = pack2<BF16>(v1[0], v1[1]);
        }
        tmem_st_x8(E0 + 8 * c, e0);
        tmem_st_x8(E1 + 8 * c, e1);
      }
      tmem_wait_st();
      tc_fence_before_sync();
      mbar_arrive(&p_full);
      ++it;
    }
    // epilogue
    mbar_wait(&acc_final, 0, w, 31);
    tc_fence_after_sync();
    const size_t orow = (static_cast<size_t>(row_base) + gr) * D;
#pragma unroll
    for (int c = 0; c < D / 32; ++c) {
      uint32_t a0[32], a1[32];
      if (it > 0) {
        tmem_ld_x32(tmem + lane_off + C::TMEM_ACC0 + c * 32, a0);
        tmem_ld_x32(tmem + lane_off + C::TMEM_ACC1 + c * 32, a1);
        tmem_wait_ld();
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) { a0[i] = 0u; a1[i] = 0u; }
      }
      if (gr < N) {
        uint32_t q0[16], q1[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          q0[i] = pack2<BF16>(__uint_as_float(a0[2 * i]) * p.out_scale, __uint_as_float(a0[2 * i + 1]) * p.out_scale);
          q1[i] = pack2<BF16>(__uint_as_float(a1[2 * i]) * p.out_scale, __uint_as_float(a1[2 * i + 1]) * p.out_scale);
        }
        uint4* o0 = reinterpret_cast<uint4*>(static_cast<uint16_t*>(p.out0) + orow + c * 32);
        uint4* o1 = reinterpret_cast<uint4*>(static_cast<uint16_t*>(p.out1) + orow + c * 32);
#pragma unroll
        for (int v4 = 0; v4 < 4; ++v4) {
          o0[v4] = make_uint4(q0[4 * v4], q0[4 * v4 + 1], q0[4 * v4 + 2], q0[4 * v4 + 3]);
          o1[v4] = make_uint4(q1[4 * v4], q1[4 * v4 + 1], q1[4 * v4 + 2], q1[4 * v4 + 3]);
        }
      }
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 5) tmem_dealloc(tmem, C::TMEM_COLS);
}

// stats[row] = (lse2, mu, Delta, a) with a = rowsum(gtO o O), Delta = rowsum(gO o O) + rowsum(gtO o tO) - a mu.
// One warp per row; 16-bit inputs. Generalises the reference's _attn_bwd_preprocess
// (jvp_attention.py:1395-1422), which computes rowsum(O o dO) only.
template <bool BF16>
__global__ void bwd_preprocess_kernel(const uint16_t* __restrict__ o, const uint16_t* __restrict__ to,
                                      const uint16_t* __restrict__ go, const uint16_t* __restrict__ gto,
                                      const float* __restrict__ lse2, const float* __restrict__ mu,
                                      float4* __restrict__ stats, int64_t rows, int D) {
  const int64_t row = static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= rows) return;
  auto cvt = [](uint16_t x) -> float {
    if constexpr (BF16) return __uint_as_float(static_cast<uint32_t>(x) << 16);
    else return __half2float(__ushort_as_half(x));
  };
  float s_go_o = 0.f, s_gto_to = 0.f, s_gto_o = 0.f;
  for (int d = lane * 2; d < D; d += 64) {
    const size_t idx = static_cast<size_t>(row) * D + d;
    const uint32_t ov = *reinterpret_cast<const uint32_t*>(o + idx);
    const uint32_t tov = *reinterpret_cast<const uint32_t*>(to + idx);
    const uint32_t gov = *reinterpret_cast<const uint32_t*>(go + idx);
    const uint32_t gtov = gto ? *reinterpret_cast<const uint32_t*>(gto + idx) : 0u;
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      const float fo = cvt(static_cast<uint16_t>(ov >> (16 * u))), fto = cvt(static_cast<uint16_t>(tov >> (16 * u)));
      const float fgo = cvt(static_cast<uint16_t>(gov >> (16 * u))), fgto = cvt(static_cast<uint16_t>(gtov >> (16 * u)));
      s_go_o = fmaf(fgo, fo, s_go_o);
      s_gto_to = fmaf(fgto, fto, s_gto_to);
      s_gto_o = fmaf(fgto, fo, s_gto_o);
    }
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) {
    s_go_o += __shfl_xor_sync(0xFFFFFFFFu, s_go_o, off);
    s_gto_to += __shfl_xor_sync(0xFFFFFFFFu, s_gto_to, off);
    s_gto_o += __shfl_xor_sync(0xFFFFFFFFu, s_gto_o, off);
  }
  if (lane == 0) {
    const float m = mu[row];
    stats[row] = make_float4(lse2[row], m, s_go_o + s_gto_to - s_gto_o * m, s_gto_o);
  }
}

template <int D, int FAM, bool BF16>
int launch_family(const jvpfa_bwd_args& a, const float4* stats, cudaStream_t stream) {
  using C = BwdCfg<D, FAM>;
  const uint64_t rows = static_cast<uint64_t>(a.B) * a.H * a.N;
  const void* rsrc[4];
  const void* csrc[4];
  void *out0, *out1;
  float out_scale;
  if (FAM == FAM_Q) {
    rsrc[0] = a.q; rsrc[1] = a.tq; rsrc[2] = a.go; rsrc[3] = a.gto;
    csrc[0] = a.v; csrc[1] = a.tv; csrc[2] = a.k; csrc[3] = a.tk;
    out0 = a.dq; out1 = a.dtq; out_scale = a.sm_scale;
  } else if (FAM == FAM_K) {
    rsrc[0] = a.k; rsrc[1] = a.tk; rsrc[2] = a.v; rsrc[3] = a.tv;
    csrc[0] = a.go; csrc[1] = a.gto; csrc[2] = a.q; csrc[3] = a.tq;
    out0 = a.dk; out1 = a.dtk; out_scale = a.sm_scale;
  } else {
    rsrc[0] = a.k; rsrc[1] = a.tk; rsrc[2] = a.k; rsrc[3] = a.tk;
    csrc[0] = a.q; csrc[1] = a.tq; csrc[2] = a.go; csrc[3] = a.gto;
    out0 = a.dv; out1 = a.dtv; out_scale = 1.0f;
  }
  CUtensorMap rm[4], cm[4];
  for (int i = 0; i < 4; ++i) {
    if (!make_tile_map(&rm[i], rsrc[i], rows, D, C::BR, a.dtype)) return JVPFA_ERR_LAUNCH;
    if (!make_tile_map(&cm[i], csrc[i], rows, D, C::BC, a.dtype)) return JVPFA_ERR_LAUNCH;
  }
  BwdKParams p{};
  p.H = a.H; p.N = a.N; p.causal = a.causal;
  p.s = a.sm_scale;
  p.c1 = a.sm_scale * 1.4426950408889634f;
  p.out_scale = out_scale;
  p.mv.ptr = a.mask.ptr; p.mv.summary = a.mask_summary;
  p.mv.s0 = a.mask.stride[0]; p.mv.s1 = a.mask.stride[1]; p.mv.s2 = a.mask.stride[2]; p.mv.s3 = a.mask.stride[3];
  p.mv.kind = a.mask.kind; p.mv.dtype = a.mask.dtype;
  p.mv.n64 = (a.N + 63) / 64;
  p.mv.Hm = a.mask.stride[1] == 0 ? 1 : a.H;
  p.stats = stats;
  p.out0 = out0; p.out1 = out1;
  p.status = static_cast<int*>(a.workspace);
  p.budget_ns = wait_budget_ns();
  auto kern = bwd_sm100_kernel<D, FAM, BF16>;
  const size_t smem = C::smem_bytes();
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)) != cudaSuccess)
    return JVPFA_ERR_LAUNCH;
  dim3 grid((a.N + C::BR - 1) / C::BR, a.B * a.H);
  ScopedKernelTimer timer(FAM == FAM_Q ? KERNEL_BWD_Q : (FAM == FAM_K ? KERNEL_BWD_K : KERNEL_BWD_V), stream);
  kern<<<grid, 192, smem, stream>>>(rm[0], rm[1], rm[2], rm[3], cm[0], cm[1], cm[2], cm[3], p);
  return cudaGetLastError() == cudaSuccess ? JVPFA_OK : JVPFA_ERR_LAUNCH;
}

template <int D, bool BF16>
int launch_all(const jvpfa_bwd_args& a, cudaStream_t stream) {
  const int64_t rows = static_cast<int64_t>(a.B) * a.H * a.N;
  float4* stats = reinterpret_cast<float4*>(static_cast<uint8_t*>(a.workspace) + kStatusBytes);
  const int warps_per_block = 8;
  const unsigned blocks = static_cast<unsigned>((rows + warps_per_block - 1) / warps_per_block);
  {
  ScopedKernelTimer timer(KERNEL_BWD_PREPROCESS, stream);
  bwd_preprocess_kernel<BF16><<<blocks, warps_per_block * 32, 0, stream>>>(
      static_cast<const uint16_t*>(a.o), static_cast<const uint16_t*>(a.to), static_cast<const uint16_t*>(a.go),
      static_cast<const uint16_t*>(a.gto), a.lse2, a.mu, stats, rows, D);
  }
  if (cudaGetLastError() != cudaSuccess) return JVPFA_ERR_LAUNCH;
  int rc = launch_family<D, FAM_Q, BF16>(a, stats, stream);
  if (rc != JVPFA_OK) return rc;
  rc = launch_family<D, FAM_K, BF16>(a, stats, stream);
  if (rc != JVPFA_OK) return rc;
  return launch_family<D, FAM_V, BF16>(a, stats, stream);
}

}  // namespace

size_t bwd_sm100_workspace_bytes(const jvpfa_bwd_args& a) {
  return kStatusBytes + static_cast<size_t>(a.B) * a.H * a.N * sizeof(float4);
}

int launch_bwd_sm100(const jvpfa_bwd_args& a, cudaStream_t stream) {
  if (a.gto == nullptr) return JVPFA_ERR_BAD_ARG;  // the tensor-core path wants an explicit (possibly zero) gtO
  const bool bf = a.dtype == JVPFA_BF16;
  if (a.D == 64) return bf ? launch_all<64, true>(a, stream) : launch_all<64, false>(a, stream);
  return bf ? launch_all<128, true>(a, stream) : launch_all<128, false>(a, stream);
}

}  // namespace jvpfa
