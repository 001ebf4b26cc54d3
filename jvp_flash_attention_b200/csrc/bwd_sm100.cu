// Dual (JVP) attention backward for sm_100a: gradients of sum(O*gO) + sum(tO*gtO) with respect to
// Q, K, V and the tangent inputs tQ, tK, tV, with tcgen05 MMAs accumulating in TMEM.
//
// Replaces the reference's _attn_bwd / _attn_bwd_causal (+ _attn_bwd_dkdv, _attn_bwd_dq)
// (jvp_flash_attention/jvp_attention.py:2019-2244, 1721-2016, 1426-1574, 1578-1718) and adds the
// gradient through the tangent output and the tangent-input gradients, which the reference does
// not compute (jvp_attention.py:3081, 3226).
//
// One kernel template, one instantiation per output family. A CTA owns a "row" tile of 128 sequence positions
// whose operands stay in shared memory, and streams 64-wide "column" tiles of the other side:
//   family Q : rows = queries.  scores S, tS, X, A (q on TMEM lanes)    -> dQ, dtQ
//   family K : rows = keys.     transposed scores (k on TMEM lanes)      -> dK, dtK
//   family V : rows = keys.     transposed S, tS only                    -> dV, dtV
//   family KV: families K and V in one pass for head dimensions up to 64, where four accumulators and four score
//              tiles fit the 512 TMEM columns: 12 tile products where the two passes run 15
// with  S = Q K^T, tS = tQ K^T + Q tK^T, X = gO V^T + gtO tV^T, A = gtO V^T and per score element
//   P = exp2(c1 S + bias - lse2_q), ts = s tS, dtS = P (A - a_q),
//   dS = P (X + A (ts - mu_q) - a_q ts - Delta_q), tP = P (ts - mu_q);
//   dQ = s (dS K + dtS tK), dtQ = s dtS K, dK = s (dS^T Q + dtS^T tQ), dtK = s dtS^T Q,
//   dV = P^T gO + tP^T gtO, dtV = P^T gtO.
// The per-query statistics (lse2, mu, Delta, a) come packed as one float4 per query from the
// preprocess kernel. Family Q reads them per thread (thread = query row); families K and V stage
// the 64 statistics of the current query tile in shared memory and read them as broadcasts.
//
// Roles: warps 0-7 element-wise as two warpgroups that split the 64 columns of every score tile
// (thread = TMEM lane = one score row, 32 columns), warp 8 TMA producer, warps 9 and 10 MMA issuers (9: the
// score products S, tS; 10: the output products and X, A; two instruction streams keep the tensor pipe fed while
// one of them waits on a barrier). Column-side tiles flow through a ring of shared-memory slots in the order in
// which the issuers release them (tiles only the score MMAs read come first).
#include <type_traits>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include "host_common.h"
#include "dropout.cuh"
#include "mask_common.cuh"
#include "sm100_prims.cuh"

namespace jvpfa {
using namespace sm100;

namespace {

enum { FAM_Q = 0, FAM_K = 1, FAM_V = 2, FAM_KV = 3 };


struct BwdKParams {
  int H, N;
  int n_rt, n_units;   // row tiles per (batch, head) unit, number of units: the grid has n_rt * n_units blocks
  int unit_group;      // units per group of the block order
  int D;     // head dimension of the tensors (the kernel is compiled for it rounded up to 64 or 128)
  int causal;
  float c1;  // sm_scale * log2(e)
  float s;   // sm_scale
  float out_scale;
  MaskView mv;
  const float4* stats;  // per (b,h,q): lse2, mu, Delta, a
  void* out0;
  void* out1;
  void* out2;   // family KV: dV, dtV (written unscaled)
  void* out3;
  int* status;
  uint64_t budget_ns;
  DropoutParams drop;
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

// The residual of a pair after its bf16 rounding `hi`, as bf16 again (the lo part of the hi/lo split).
__device__ __forceinline__ uint32_t pack2_residual(float a, float b, uint32_t hi) {
  return pack2<true>(a - __uint_as_float(hi << 16), b - __uint_as_float(hi & 0xFFFF0000u));
}

// SPLIT: fp32 inputs on the tensor cores. The operands arrive as rows of 128 bf16 numbers [hi(64) | lo(64)] written by the
// split pre-pass, so the tiles have the geometry of the D = 128 kernel with the hi parts in slab 0 and the lo parts in
// slab 1; every product a b is accumulated as a_hi b_hi + a_lo b_hi + a_hi b_lo. Accumulators are 64 columns wide, the
// element-wise warps write hi and lo parts of their 16-bit operands, and the gradients are written as fp32.
template <int D, int FAM, bool SPLIT = false>
struct BwdCfg {
  static constexpr int BR = 128;                         // rows per CTA
  static constexpr int BC = 64;                          // columns per streamed tile
  static constexpr int NR = (FAM == FAM_V) ? 2 : 4;      // resident row-side operand tiles
  static constexpr int NA = 2;                           // buffers of the first column-side pair
  static constexpr bool KV = (FAM == FAM_KV);            // families K and V in one pass (head dimension <= 64)
  static constexpr int NB = (FAM == FAM_V || KV) ? 2 : 1;   // buffers of the second column-side pair
  static constexpr int TILE_R = BR * D * 2;
  static constexpr int PAIR = 2 * BC * D * 2;            // two stacked 64-row tiles = one 128-row operand
  static constexpr int SLAB = 128 * 128;                 // bytes of one 64-column slab of a 128-row tile
  static constexpr int HALF = BC * 128;                  // byte offset of the second tile inside a slab
  static constexpr int DV = SPLIT ? 64 : D;                 // columns of an accumulator
  static constexpr int NACC = KV ? 4 : 2;                // accumulators
  static constexpr int TMEM_ACC0 = 0;
  static constexpr int TMEM_ACC1 = DV;
  static constexpr int TMEM_ACC2 = 2 * DV;
  static constexpr int TMEM_T = NACC * DV;               // score tiles, 64 columns each
  static constexpr int EUP = 16;                         // family KV: columns from dS (dtS) to the P (tP) that shares its score tile
  static_assert(!KV || (D == 64 && !SPLIT), "four accumulators and four score tiles fit 512 TMEM columns only at 64");
  static constexpr int EBUF = SPLIT ? 128 : 64;             // family V: columns of one buffer of 16-bit P, tP (SPLIT: hi and lo parts)
  static constexpr int ELO = SPLIT ? (FAM == FAM_V ? 32 : 16) : 0;   // columns from the hi part of an operand to its lo part
  static constexpr int TMEM_COLS = 512;
  static constexpr int NBAR = 8 + 2 * NA + 2 * NB + 8;
  static constexpr size_t smem_bytes() { return NR * TILE_R + (NA + NB) * PAIR + 2 * BC * 16 + (NBAR + 2) * 8; }
};

// Tensor maps: rmK = row-side operands (box of 128 rows, all slabs); cmK = column-side operands (box of
// 64 rows, one 64-column slab), cm0/cm1 the first pair, cm2/cm3 the second pair:
//  family Q: rm = Q, tQ, gO, gtO;  first pair (K, tK),  second pair (V, tV)
//  family K: rm = K, tK, V, tV;    first pair (Q, tQ),  second pair (gO, gtO)
//  family V: rm = K, tK;           first pair (Q, tQ),  second pair (gO, gtO)
// The two tiles of a pair are stacked in shared memory as one 128-row operand, so that the score
// products against it run as N = 128 MMAs:
//  [S | R0 c1^T] = R0 [c0; c1]^T, then tS += R1 c0^T; and for families Q, K
//  Q: [A | gtO tV^T] = gtO [V; tV]^T, X += gO V^T;    K: [V gO^T | A^T] = V [gO; gtO]^T, X^T += tV gtO^T.
// Families Q and K keep one set of score tiles and overlap in two phases per tile: phase 1 reads S, tS
// (which frees them for the next tile's products), phase 2 reads X, A and writes the 16-bit dS, dtS operands;
// family V keeps one set of S, tS and two buffers of 16-bit P, tP. Family KV is family K whose element-wise threads
// also write tP and P, into the halves of the A and X tiles that the in-place dtS and dS leave unused, and whose output
// issuer adds the three products of family V.
// PAD: the tensors' head dimension is smaller than D (columns beyond it are zero-filled by TMA); the K steps and
// output columns that would only see zeros are then skipped at run time.
// DUAL = false: primal-only backward (no tangents, no gradient through a tangent output): S and X = gO V^T only,
// dS = P (X - Delta); dQ = s dS K, dK = s dS^T Q, dV = P^T gO. Tangent tiles are neither loaded nor multiplied.
// DROP: the forward applied dropout to the probabilities that multiply V, tV (dropout.cuh). The same keep pattern is
// regenerated here: it scales X and A (the gradients that arrive through V, tV) in families Q, K, and P, tP (the operands
// of dV, dtV) in family V; Delta and a come from the dropped-out O, tO and need no change.
template <int D, int FAM, bool BF16, bool PAD, bool DUAL, bool SPLIT = false, bool DROP = false>
__global__ void __launch_bounds__(352, 1)
bwd_sm100_kernel(const __grid_constant__ CUtensorMap rm0, const __grid_constant__ CUtensorMap rm1,
                 const __grid_constant__ CUtensorMap rm2, const __grid_constant__ CUtensorMap rm3,
                 const __grid_constant__ CUtensorMap cm0, const __grid_constant__ CUtensorMap cm1,
                 const __grid_constant__ CUtensorMap cm2, const __grid_constant__ CUtensorMap cm3,
                 const BwdKParams p) {
  using C = BwdCfg<D, FAM, SPLIT>;
  constexpr int NA = C::NA, NB = C::NB;
  constexpr int SLABS = D / 64;
  constexpr int DV = C::DV;
  static_assert(!SPLIT || (D == 128 && BF16 && !PAD), "the split-fp32 mode runs on the 128-column geometry in bf16");

  // Everything lives in dynamic shared memory so that the 128-byte-swizzled tiles can start at its
  // 1024-byte-aligned base without alignment slack: tiles, then statistics, then barriers.
  extern __shared__ __align__(1024) uint8_t smem[];
  auto sR = [&](int i) { return smem + i * C::TILE_R; };
  auto sA = [&](int k) { return smem + C::NR * C::TILE_R + k * C::PAIR; };
  auto sB = [&](int k) { return smem + C::NR * C::TILE_R + (NA + k) * C::PAIR; };
  uint8_t* tail = smem + C::NR * C::TILE_R + (NA + NB) * C::PAIR;
  // per-query statistics of the current column tile, negated, one array per field: [buffer][-lse2, -mu, -Delta, -a][column]
  float(*stats_s)[4][C::BC] = reinterpret_cast<float(*)[4][C::BC]>(tail);
  uint64_t* bars = reinterpret_cast<uint64_t*>(tail + 2 * C::BC * sizeof(float4));
  uint64_t& r_full = bars[0];       // row-side tiles 0, 1 (what the score products S, tS read) have landed
  uint64_t* st_full = bars + 1;   // [2] (family V uses both, Q/K only [0])
  uint64_t* p_full = bars + 3;    // [2]
  uint64_t& ph1_done = bars[5];
  uint64_t& xa_full = bars[6];
  uint64_t& acc_final = bars[7];
  uint64_t* a_full = bars + 8;
  uint64_t* a_empty = a_full + NA;
  uint64_t* b_full = a_empty + NA;
  uint64_t* b_empty = b_full + NB;
  uint64_t* e_free = b_empty + NB;   // [2] family V: the output products that read P, tP buffer b have completed
  uint64_t& a_ready = e_free[2];     // families Q, K: A of the current tile is complete (X still accumulating)
  uint64_t& pt_full = e_free[3];     // families Q, K: dtS of the current tile is in TMEM
  uint64_t& r23_full = e_free[4];    // families Q, K: row-side tiles 2, 3 (what the X, A products read) have landed
  uint64_t& sc_free = e_free[5];     // family V: all 256 element-wise threads hold S, tS in registers, the next tile's
                                     // score products may overwrite them
  uint64_t* pp_full = e_free + 6;    // [2] family V: P of buffer b is in TMEM
  uint32_t& tmem_base_s = *reinterpret_cast<uint32_t*>(bars + C::NBAR);
  int& poisoned = *reinterpret_cast<int*>(bars + C::NBAR + 1);
  if ((smem_u32(smem) & 1023u) != 0u) {  // the swizzled layouts need this; never observed otherwise
    if (threadIdx.x == 0) atomicCAS(p.status, 0, WAIT_TIMEOUT_BASE + 99);
    return;
  }

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int n_rt = p.n_rt;
  // heavier tiles first under a causal mask: late query tiles, early key tiles
  const BlockWork work = block_work(blockIdx.x, n_rt, p.n_units, p.unit_group, p.causal && FAM == FAM_Q);
  const int rt = work.tile;
  const int bh = work.unit;
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
    mbar_init(&r23_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&st_full[i], 1);
      mbar_init(&p_full[i], 256);
      mbar_init(&e_free[i], 1);
      mbar_init(&pp_full[i], 256);
    }
    mbar_init(&ph1_done, 256);
    mbar_init(&sc_free, 256);
    mbar_init(&xa_full, 1);
    mbar_init(&a_ready, 1);
    mbar_init(&pt_full, 256);
    mbar_init(&acc_final, 1);
    for (int i = 0; i < NA; ++i) {
      mbar_init(&a_full[i], 1);
      mbar_init(&a_empty[i], 1);
    }
    for (int i = 0; i < NB; ++i) {
      mbar_init(&b_full[i], 1);
      mbar_init(&b_empty[i], 1);
    }
    fence_mbar_init();
  }
  __syncthreads();
  if (warp == 9) {
    tmem_alloc(&tmem_base_s, C::TMEM_COLS);
    tmem_relinquish();
  }
  // the TMA producers need the barriers but not the TMEM address: they start loading while TMEM is being allocated
  const bool producer = (warp == 8);
  tc_fence_before_sync();
  if (!producer) named_bar_sync(2, 320);
  tc_fence_after_sync();
  const uint32_t tmem = producer ? 0u : tmem_base_s;

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
  // next column tile at or after j that takes part, or j_end
  auto next_active = [&](int j) {
    while (j < j_end && !(tile_bits(j) & kTileAnyKept)) ++j;
    return j;
  };

  if (warp == 8) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      // Order of the first loads: the row-side tiles of the score products, the first column pair, then the row-side
      // tiles of X, A and their first column pair -- the first score products start after 96 KB instead of 192 KB.
      mbar_arrive_expect_tx(&r_full, (DUAL ? 2 : 1) * C::TILE_R);
#pragma unroll
      for (int sl = 0; sl < SLABS; ++sl) {
        tma_load_tile(sR(0) + sl * C::SLAB, &rm0, &r_full, 64 * sl, r0, h, b);
        if constexpr (DUAL) tma_load_tile(sR(1) + sl * C::SLAB, &rm1, &r_full, 64 * sl, r0, h, b);
      }
      auto load_rows23 = [&]() {
        if constexpr (C::NR == 4) {
          mbar_arrive_expect_tx(&r23_full, (DUAL ? 2 : 1) * C::TILE_R);
#pragma unroll
          for (int sl = 0; sl < SLABS; ++sl) {
            tma_load_tile(sR(2) + sl * C::SLAB, &rm2, &r23_full, 64 * sl, r0, h, b);
            if constexpr (DUAL) tma_load_tile(sR(3) + sl * C::SLAB, &rm3, &r23_full, 64 * sl, r0, h, b);
          }
        }
      };
      int it = 0;
      for (int j = next_active(j_begin); j < j_end; j = next_active(j + 1), ++it) {
        const int crow = j * C::BC;   // first row of the column tile inside its (batch, head) unit
        {
          const int buf = it % NA;
          mbar_wait(&a_empty[buf], ((it / NA) & 1) ^ 1, w, 10);
          mbar_arrive_expect_tx(&a_full[buf], DUAL ? C::PAIR : C::PAIR / 2);
#pragma unroll
          for (int sl = 0; sl < SLABS; ++sl) {
            tma_load_tile(sA(buf) + sl * C::SLAB, &cm0, &a_full[buf], 64 * sl, crow, h, b);
            if constexpr (DUAL) tma_load_tile(sA(buf) + sl * C::SLAB + C::HALF, &cm1, &a_full[buf], 64 * sl, crow, h, b);
          }
        }
        if (it == 0) load_rows23();
        {
          const int buf = it % NB;
          mbar_wait(&b_empty[buf], ((it / NB) & 1) ^ 1, w, 11);
          mbar_arrive_expect_tx(&b_full[buf], DUAL ? C::PAIR : C::PAIR / 2);
#pragma unroll
          for (int sl = 0; sl < SLABS; ++sl) {
            tma_load_tile(sB(buf) + sl * C::SLAB, &cm2, &b_full[buf], 64 * sl, crow, h, b);
            if constexpr (DUAL) tma_load_tile(sB(buf) + sl * C::SLAB + C::HALF, &cm3, &b_full[buf], 64 * sl, crow, h, b);
          }
        }
      }
      if (it == 0) load_rows23();   // no column tile takes part: the loads still have to happen before the CTA ends
    }
    __syncwarp();
  } else if (warp >= 9) {
    // ------------------------------------------------------------------ MMA issuers: warp 9 the score products S, tS;
    // warp 10 the output products and X, A (two instruction streams keep the tensor pipe fed while one of them waits)
    {
      // all lanes run the loop so that addresses and descriptors stay warp-uniform; the elected lane issues
      const bool leader = elect_one_sync();
      const uint32_t lead = leader ? 1u : 0u;
      auto wait_all = [&](uint64_t* bar, uint32_t parity, int site) {
        mbar_wait(bar, parity, w, site);
        __syncwarp();
      };
      constexpr uint32_t FMT = BF16 ? FMT_BF16 : FMT_F16;
      const uint32_t idesc_64 = make_idesc(FMT, 128, 64, 0, 0);
      const uint32_t idesc_128 = make_idesc(FMT, 128, 128, 0, 0);
      const int dn = SPLIT ? 64 : (PAD ? ((p.D + 15) & ~15) : D);   // columns of the output products (head dimension rounded up)
      const int ksteps = dn / 16;                     // K steps of the score products that hold data
      const uint32_t idesc_out = make_idesc(FMT, 128, dn, 0, 1);
      const uint32_t TS0 = tmem + C::TMEM_T;

      // dst[128 x n] (+)= R[128 x D] * Cc[n x D]^T, Cc = n rows starting at `ctile` inside a pair buffer
      auto mma_nt = [&](uint32_t dst, const uint8_t* rtile, const uint8_t* ctile, uint32_t idesc, uint32_t acc) {
        // descriptors of the later K steps differ from the first only in the 16-byte-unit start address
        const uint64_t da = desc_kmajor_sw128(smem_u32(rtile)), db = desc_kmajor_sw128(smem_u32(ctile));
        if constexpr (SPLIT) {
          // hi hi + lo hi + hi lo: K steps 0-3 of slab 0 (hi) or slab 1 (lo) of the two operands
#pragma unroll
          for (int k = 0; k < 12; ++k) {
            const int a_slab = (k >> 2) == 1, b_slab = (k >> 2) == 2;
            const uint64_t oa = static_cast<uint64_t>((a_slab * C::SLAB + (k & 3) * 32) >> 4);
            const uint64_t ob = static_cast<uint64_t>((b_slab * C::SLAB + (k & 3) * 32) >> 4);
            umma_ss_pred(dst, da + oa, db + ob, idesc, acc | (k > 0), lead);
          }
        } else {
#pragma unroll
          for (int k = 0; k < D / 16; ++k) {
            const uint64_t o = static_cast<uint64_t>(((k >> 2) * C::SLAB + (k & 3) * 32) >> 4);
            if (!PAD || k < ksteps) umma_ss_pred(dst, da + o, db + o, idesc, acc | (k > 0), lead);
          }
        }
      };
      // acc[128 x D] (+)= E[128 x 64] (TMEM, 16-bit, two column groups of 16) * Cc[64 x D]
      auto mma_out = [&](uint32_t accum, uint32_t e, const uint8_t* ctile, uint32_t acc) {
        const uint64_t db = desc_mnmajor_sw128(smem_u32(ctile), C::SLAB);
#pragma unroll
        for (int k = 0; k < C::BC / 16; ++k) {
          const uint32_t ek = e + (FAM == FAM_V ? k * 8 : (k & 1) * 8 + (k >> 1) * 32);
          const uint64_t dk = db + static_cast<uint64_t>((k * 2048) >> 4);
          umma_ts_pred(accum, ek, dk, idesc_out, acc | (k > 0), lead);                                        // hi hi
          if constexpr (SPLIT) {
            umma_ts_pred(accum, ek + C::ELO, dk, idesc_out, 1, lead);                                         // lo hi
            umma_ts_pred(accum, ek, dk + static_cast<uint64_t>(C::SLAB >> 4), idesc_out, 1, lead);            // hi lo
          }
        }
      };
      // S, tS of tile i into score buffer sb
      auto issue_st = [&](int i, int sb) {
        const int buf = i % NA;
        wait_all(&a_full[buf], (i / NA) & 1, 20);
        // family V: the one score buffer is free once the element-wise threads hold S, tS of tile i - 1 in registers
        if constexpr (FAM == FAM_V) if (i >= 1) wait_all(&sc_free, (i - 1) & 1, 27);
        tc_fence_after_sync();
        const uint32_t T0 = TS0;
        if constexpr (DUAL) {
          mma_nt(T0, sR(0), sA(buf), idesc_128, 0);        // [S | R0 c1^T]
          mma_nt(T0 + 64, sR(1), sA(buf), idesc_64, 1);    // tS += R1 c0^T
        } else {
          mma_nt(T0, sR(0), sA(buf), idesc_64, 0);         // S
        }
        if (leader) umma_commit(&st_full[0]);
        if constexpr (FAM == FAM_V) if (leader) umma_commit(&a_empty[buf]);
        (void)sb;
      };
      // X, A of tile i (families Q, K)
      auto issue_xa = [&](int i) {
        const int buf = i % NB;
        wait_all(&b_full[buf], (i / NB) & 1, 21);
        tc_fence_after_sync();
        const uint32_t T2 = TS0 + 128;
        if constexpr (!DUAL) {
          mma_nt(FAM == FAM_Q ? T2 + 64 : T2, sR(2), sB(buf), idesc_64, 0);   // X = gO V^T (family K: its transpose)
        } else if constexpr (FAM == FAM_Q) {
          mma_nt(T2, sR(3), sB(buf), idesc_128, 0);               // [A | gtO tV^T]
          if (leader) umma_commit(&a_ready);
          mma_nt(T2 + 64, sR(2), sB(buf), idesc_64, 1);           // X += gO V^T
        } else {
          mma_nt(T2, sR(2), sB(buf), idesc_128, 0);               // [V gO^T | A^T]
          if (leader) umma_commit(&a_ready);
          mma_nt(T2, sR(3), sB(buf) + C::HALF, idesc_64, 1);      // X^T += tV gtO^T
        }
        if (leader) umma_commit(&xa_full);
        if constexpr (!C::KV) if (leader) umma_commit(&b_empty[buf]);   // family KV: gO, gtO are also operands of dV, dtV
      };

      if (warp == 9) wait_all(&r_full, 0, 22);
      else if constexpr (C::NR == 4) wait_all(&r23_full, 0, 37);
      int j = next_active(j_begin);
      int it = 0;
      if (warp == 9) {
        // ---- score issuer: S, tS of tile it + 1 as soon as the element-wise warps have read those of tile it
        if (j < j_end) issue_st(0, 0);
        for (; j < j_end; ++it) {
          const int jn = next_active(j + 1);
          if (jn < j_end) {
            if constexpr (FAM == FAM_V) {
              issue_st(it + 1, (it + 1) & 1);
            } else {
              wait_all(&ph1_done, it & 1, 25);
              issue_st(it + 1, 0);
            }
          }
          j = jn;
        }
      } else {
        // ---- output issuer
        if constexpr (FAM != FAM_V) if (j < j_end) issue_xa(0);
        for (; j < j_end; ++it) {
          const int jn = next_active(j + 1);
          const bool has_next = jn < j_end;
          if constexpr (FAM == FAM_V) {
            const int buf = it % NB;
            const uint32_t E0 = TS0 + 128 + (it & 1) * C::EBUF, E1 = E0 + C::EBUF / 2;   // 16-bit P, tP of this tile
            wait_all(&b_full[buf], (it / NB) & 1, 24);
            if constexpr (DUAL) {
              // P only needs S, which the first score chain completes: its two products run before tP exists
              wait_all(&pp_full[it & 1], (it >> 1) & 1, 29);
              tc_fence_after_sync();
              mma_out(tmem + C::TMEM_ACC0, E0, sB(buf), it > 0);             // dV  += P^T gO
              mma_out(tmem + C::TMEM_ACC1, E0, sB(buf) + C::HALF, it > 0);   // dtV += P^T gtO
            }
            wait_all(&p_full[it & 1], (it >> 1) & 1, 23);
            tc_fence_after_sync();
            if constexpr (DUAL) mma_out(tmem + C::TMEM_ACC0, E1, sB(buf) + C::HALF, 1);   // dV += tP^T gtO
            else mma_out(tmem + C::TMEM_ACC0, E0, sB(buf), it > 0);                         // dV += P^T gO
            if (leader) umma_commit(&b_empty[buf]);
            if (leader) umma_commit(&e_free[it & 1]);
          } else {
            const int buf = it % NA, bufb = it % NB;
            // dtS replaces A and dS replaces X in place (family Q: A first, X second; family K: X first, A second).
            // dtS only needs A, which the first X/A chain completes, so its two products run before dS exists.
            // Family KV: tP arrives with dtS (in the other half of the A tile), P with dS (in the X tile).
            const uint32_t E0 = (DUAL && FAM == FAM_Q) ? TS0 + 192 : TS0 + 128;   // dS
            const uint32_t E1 = (DUAL && FAM == FAM_Q) ? TS0 + 128 : TS0 + 192;   // dtS
            if constexpr (DUAL) {
              wait_all(&pt_full, it & 1, 28);
              tc_fence_after_sync();
              mma_out(tmem + C::TMEM_ACC0, E1, sA(buf) + C::HALF, it > 0);   // dtS c1
              mma_out(tmem + C::TMEM_ACC1, E1, sA(buf), it > 0);             // dtS c0
              if constexpr (C::KV) mma_out(tmem + C::TMEM_ACC2, E1 + C::EUP, sB(bufb) + C::HALF, it > 0);   // dV += tP^T gtO
            }
            wait_all(&p_full[0], it & 1, 26);
            tc_fence_after_sync();
            mma_out(tmem + C::TMEM_ACC0, E0, sA(buf), DUAL ? 1u : static_cast<uint32_t>(it > 0));   // dS c0
            if (leader) umma_commit(&a_empty[buf]);
            if constexpr (C::KV) {
              mma_out(tmem + C::TMEM_ACC2, E0 + C::EUP, sB(bufb), DUAL ? 1u : static_cast<uint32_t>(it > 0));   // dV += P^T gO
              if constexpr (DUAL) mma_out(tmem + C::TMEM_ACC2 + DV, E0 + C::EUP, sB(bufb) + C::HALF, it > 0);       // dtV += P^T gtO
              if (leader) umma_commit(&b_empty[bufb]);
            }
            if (has_next) issue_xa(it + 1);
          }
          j = jn;
        }
        if (it > 0) { if (leader) umma_commit(&acc_final); }
        else if (leader) mbar_arrive(&acc_final);
      }
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------------ element-wise + epilogue
    const int wg = warp >> 2;          // element-wise warpgroup: columns [32 wg, 32 wg + 32) of every tile
    const int r = (warp & 3) * 32 + lane;
    const int gr = r0 + r;             // global sequence index of this thread's row
    const int gr_c = min(gr, N - 1);
    const uint32_t lane_off = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const uint32_t TS0 = tmem + C::TMEM_T + lane_off;
    // negated statistics of this thread's query row (family Q): -lse2, -mu, -Delta, -a
    float4 nst = make_float4(0.f, 0.f, 0.f, 0.f);
    if (FAM == FAM_Q) {
      const float4 st = p.stats[static_cast<size_t>(row_base) + gr_c];
      nst = make_float4(-st.x, -st.y, -st.z, -st.w);
      if (st.x == -INFINITY) nst.x = -INFINITY;  // fully excluded query: P = 0
    }
    const float2 c1_2 = make_float2(p.c1, p.c1), s_2 = make_float2(p.s, p.s);
    int it = 0;
    // families K, V: the statistics of the next column tile are fetched one tile ahead (the load's latency
    // would otherwise stall all element-wise warps at the top of every tile)
    auto fetch_stats = [&](int j) -> float4 {
      // (nothing here may look at the loaded value: that would wait for the load on the spot)
      float4 sv = make_float4(INFINITY, 0.f, 0.f, 0.f);
      if (FAM != FAM_Q && tid < C::BC && j < j_end && j * C::BC + tid < N)
        sv = __ldg(&p.stats[static_cast<size_t>(row_base) + j * C::BC + tid]);
      return sv;
    };
    int j_next = next_active(j_begin);
    float4 sv_next = fetch_stats(j_next);
    for (int j = j_next; j < j_end; j = j_next, ++it) {
      const uint8_t bits = tile_bits(j);
      const int c0 = j * C::BC;
      const int cw = c0 + 32 * wg;   // first column of this thread
      j_next = next_active(j + 1);
      if (FAM != FAM_Q) {
        if (tid < C::BC) {
          const float4 sv = sv_next;
          stats_s[it & 1][0][tid] = (sv.x == -INFINITY) ? -INFINITY : -sv.x;   // fully excluded query: P = 0
          stats_s[it & 1][1][tid] = -sv.y;
          stats_s[it & 1][2][tid] = -sv.z;
          stats_s[it & 1][3][tid] = -sv.w;
        }
        named_bar_sync(1, 256);
        sv_next = fetch_stats(j_next);
      }
      // pair of negated statistics for columns (2 i, 2 i + 1) of this thread
      auto stat2 = [&](int field, int i) -> float2 {
        if (FAM == FAM_Q) {
          const float v = field == 0 ? nst.x : (field == 1 ? nst.y : (field == 2 ? nst.z : nst.w));
          return make_float2(v, v);
        }
        return *reinterpret_cast<const float2*>(&stats_s[it & 1][field][32 * wg + 2 * i]);
      };
      const int sb = (FAM == FAM_V) ? (it & 1) : 0;   // family V: P, tP buffer of this tile
      const uint32_t T0 = TS0 + 32 * wg, T1 = T0 + 64;
      const uint32_t EV0 = TS0 + 128 + sb * C::EBUF + 16 * wg, EV1 = EV0 + C::EBUF / 2;   // family V: this thread's 16 columns of P, tP
      // dropout pattern of this thread's 32 score elements: its row is a query in family Q, a key in families K and V
      uint32_t keep_bits = 0xFFFFFFFFu;
      if constexpr (DROP)
        keep_bits = (FAM == FAM_Q) ? dropout_keep_along_k(p.drop, bh, gr, cw) : dropout_keep_along_q(p.drop, bh, cw, gr);
      auto keep2 = [&](int ip) -> float2 { return dropout_factors(keep_bits, ip, p.drop.inv_keep); };
      // family V, dual: P goes back to TMEM first (its two output products start while tP is computed)
      constexpr bool SPLIT_P = (FAM == FAM_V) && DUAL;
      // families Q, K: the upper 16 of a thread's 32 score columns take the lo parts (split mode) or P, tP (family KV)
      constexpr bool UPPER_USED = SPLIT || C::KV;
      mbar_wait(&st_full[0], it & 1, w, 30);
      tc_fence_after_sync();
      // ---- phase 1: P and ts of this thread's 32 columns (packed fp32x2 arithmetic: the element-wise
      // warps share their schedulers with the MMA-issuing warp, so every instruction saved here counts)
      float2 P2[16], ts2[16];
      {
        uint32_t a0[32], a1[32];
        tmem_ld_x32(T0, a0);
        if constexpr (DUAL) tmem_ld_x32(T1, a1);
        tmem_wait_ld();
        if constexpr (FAM != FAM_V) {
          tc_fence_before_sync();
          mbar_arrive(&ph1_done);   // S, tS are in registers: the next tile's products may overwrite them
        } else {
          tc_fence_before_sync();
          mbar_arrive(&sc_free);    // likewise: family V keeps one score buffer and two buffers of 16-bit P, tP
        }
        const bool need_causal = p.causal && ((FAM == FAM_Q) ? (c0 + C::BC - 1 > r0) : (r0 + C::BR - 1 > c0));
        const bool need_bound = (FAM == FAM_Q) && (c0 + C::BC > N);
        const bool need_mask = p.mv.kind != JVPFA_MASK_NONE && (bits & kTileAnyMasked);
        float2 x2[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          x2[i] = __ffma2_rn(make_float2(__uint_as_float(a0[2 * i]), __uint_as_float(a0[2 * i + 1])), c1_2, stat2(0, i));
          if constexpr (DUAL) ts2[i] = __fmul2_rn(make_float2(__uint_as_float(a1[2 * i]), __uint_as_float(a1[2 * i + 1])), s_2);
        }
        // The mask as this thread sees it: the flags of its own 64x64 tile (query tile, key tile). Packed by the summary
        // pre-pass (a boolean mask, or a two-valued tile of an additive one), this thread's 32 entries of the tile are
        // one word: its query row against the tile's keys in family Q, its key row against the tile's queries in the
        // other families. Anything else is read element by element below.
        const int my_qt = (FAM == FAM_Q) ? (gr_c >> 6) : j, my_kt = (FAM == FAM_Q) ? j : (gr_c >> 6);
        int mask_mode = 0;
        if (need_mask) mask_mode = mask_tile_mode(p.mv, mask_tile_bits(p.mv, b, h, my_qt, my_kt));
        if (mask_mode == 1) {
          const float other = p.mv.kind == JVPFA_MASK_BOOL ? -INFINITY : mask_tile_value(p.mv, b, h, my_qt, my_kt) * 1.4426950408889634f;
          mask_apply_bits(x2, (FAM == FAM_Q) ? mask_row_bits(p.mv, b, h, gr_c, j, wg) : mask_col_bits(p.mv, b, h, j, gr_c, wg), other);
        }
        const bool mask_elems = mask_mode == 2;
        // (keys past the end of the sequence: zero bits of a boolean mask already exclude them)
        if (need_causal || (need_bound && !(mask_mode == 1 && p.mv.kind == JVPFA_MASK_BOOL)) || mask_elems) {
#pragma unroll
          for (int hch = 0; hch < 2; ++hch) {
            float bias[16];
#pragma unroll
            for (int i = 0; i < 16; ++i) bias[i] = 0.f;
            if (mask_elems) {
              if (FAM == FAM_Q) mask_bias_run<16>(bias, p.mv, b, h, gr_c, cw + 16 * hch, N, true);
              else mask_bias_run<16>(bias, p.mv, b, h, cw + 16 * hch, gr_c, N, false);
            }
            if (need_causal) {
#pragma unroll
              for (int i = 0; i < 16; ++i) {
                const int col = cw + 16 * hch + i;
                const bool ok = (FAM == FAM_Q) ? (col <= gr) : (gr <= col);
                if (!ok) bias[i] = -INFINITY;
              }
            }
            if (need_bound) {
#pragma unroll
              for (int i = 0; i < 16; ++i)
                if (cw + 16 * hch + i >= N) bias[i] = -INFINITY;
            }
#pragma unroll
            for (int i = 0; i < 8; ++i)
              x2[8 * hch + i] = __fadd2_rn(x2[8 * hch + i], make_float2(bias[2 * i], bias[2 * i + 1]));
          }
        }
#pragma unroll
        for (int i = 0; i < 16; ++i) P2[i] = make_float2(fast_exp2(x2[i].x), fast_exp2(x2[i].y));
      }
      // family KV: P as the 16-bit operand of dV, dtV (dropped out; dS, dtS use the P before dropout)
      auto pack_p = [&](int ip) -> uint32_t {
        float2 pk = P2[ip];
        if constexpr (DROP) pk = __fmul2_rn(pk, keep2(ip));
        return pack2<BF16>(pk.x, pk.y);
      };
      if constexpr (SPLIT_P) {
        // P into this tile's 16-bit buffer (which the output products of tile it - 2 read), then tP = P (ts - mu)
        if (it >= 2) {
          mbar_wait(&e_free[sb], ((it >> 1) - 1) & 1, w, 35);
          tc_fence_after_sync();
        }
        {
          uint32_t e0[16];
          if constexpr (DROP) {
#pragma unroll
            for (int i = 0; i < 16; ++i) P2[i] = __fmul2_rn(P2[i], keep2(i));   // from here on P is only an operand of dV, dtV
          }
#pragma unroll
          for (int i = 0; i < 16; ++i) e0[i] = pack2<BF16>(P2[i].x, P2[i].y);
          tmem_st_x16(EV0, e0);
          if constexpr (SPLIT) {
            uint32_t l0[16];
#pragma unroll
            for (int i = 0; i < 16; ++i) l0[i] = pack2_residual(P2[i].x, P2[i].y, e0[i]);
            tmem_st_x16(EV0 + C::ELO, l0);
          }
        }
        tmem_wait_st();
        tc_fence_before_sync();
        mbar_arrive(&pp_full[sb]);
        uint32_t e1[16], l1[16];
#pragma unroll
        for (int ip = 0; ip < 16; ++ip) {
          const float2 tp = __fmul2_rn(P2[ip], __fadd2_rn(ts2[ip], stat2(1, ip)));
          e1[ip] = pack2<BF16>(tp.x, tp.y);
          if constexpr (SPLIT) l1[ip] = pack2_residual(tp.x, tp.y, e1[ip]);
        }
        tmem_st_x16(EV1, e1);
        if constexpr (SPLIT) tmem_st_x16(EV1 + C::ELO, l1);
      } else if constexpr (FAM == FAM_V) {
        // P (and tP = P (ts - mu)) into this tile's 16-bit buffer, which the output products of tile it - 2 read
        if (it >= 2) {
          mbar_wait(&e_free[sb], ((it >> 1) - 1) & 1, w, 35);
          tc_fence_after_sync();
        }
#pragma unroll
        for (int hch = 0; hch < 2; ++hch) {
          uint32_t e0[8], e1[8], l0[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const int ip = 8 * hch + i;
            if constexpr (DROP) P2[ip] = __fmul2_rn(P2[ip], keep2(ip));
            e0[i] = pack2<BF16>(P2[ip].x, P2[ip].y);
            if constexpr (SPLIT) l0[i] = pack2_residual(P2[ip].x, P2[ip].y, e0[i]);
            if constexpr (DUAL) {
              const float2 tp = __fmul2_rn(P2[ip], __fadd2_rn(ts2[ip], stat2(1, ip)));
              e1[i] = pack2<BF16>(tp.x, tp.y);
            }
          }
          tmem_st_x8(EV0 + 8 * hch, e0);
          if constexpr (SPLIT) tmem_st_x8(EV0 + C::ELO + 8 * hch, l0);
          if constexpr (DUAL) tmem_st_x8(EV1 + 8 * hch, e1);
        }
      } else {
        // ---- phase 2: X, A -> dS = P (X - Delta + ts (A - a) - mu A), dtS = P (A - a); both replace their
        // source in place in this thread's own columns
        const uint32_t T2 = TS0 + 128 + 32 * wg, T3 = T2 + 64;
        if constexpr (DUAL) {
          const uint32_t TA = (FAM == FAM_Q) ? T2 : T3, TX = (FAM == FAM_Q) ? T3 : T2;
          // phase 2a, as soon as A is complete: dtS, and everything of dS that does not need X (kept in ts2)
          mbar_wait(&a_ready, it & 1, w, 33);
          tc_fence_after_sync();
          // (split mode: the lo parts go into the upper half of this thread's 32 columns, so all of them are read first;
          // family KV puts tP there)
          uint32_t ar[2][16];
          if constexpr (UPPER_USED) {
            tmem_ld_x16(TA, ar[0]);
            tmem_ld_x16(TA + 16, ar[1]);
            tmem_wait_ld();
          }
#pragma unroll
          for (int hch = 0; hch < 2; ++hch) {
            if constexpr (!UPPER_USED) {
              tmem_ld_x16(TA + 16 * hch, ar[hch]);
              tmem_wait_ld();
            }
            uint32_t e1[8], l1[8], u1[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const int ip = 8 * hch + i;
              float2 A = make_float2(__uint_as_float(ar[hch][2 * i]), __uint_as_float(ar[hch][2 * i + 1]));
              if constexpr (DROP) A = __fmul2_rn(A, keep2(ip));
              if constexpr (C::KV) {   // tP = P (ts - mu), the operand of dV += tP^T gtO (dropped out like P)
                float2 tp = __fmul2_rn(P2[ip], __fadd2_rn(ts2[ip], stat2(1, ip)));
                if constexpr (DROP) tp = __fmul2_rn(tp, keep2(ip));
                u1[i] = pack2<BF16>(tp.x, tp.y);
              }
              const float2 d = __fadd2_rn(A, stat2(3, ip));                       // A - a
              float2 t = __ffma2_rn(ts2[ip], d, stat2(2, ip));                    // ts (A - a) - Delta
              ts2[ip] = __ffma2_rn(stat2(1, ip), A, t);                           // - mu A
              const float2 dts = __fmul2_rn(P2[ip], d);
              e1[i] = pack2<BF16>(dts.x, dts.y);
              if constexpr (SPLIT) l1[i] = pack2_residual(dts.x, dts.y, e1[i]);
            }
            tmem_st_x8(TA + 8 * hch, e1);
            if constexpr (SPLIT) tmem_st_x8(TA + C::ELO + 8 * hch, l1);
            if constexpr (C::KV) tmem_st_x8(TA + C::EUP + 8 * hch, u1);
          }
          tmem_wait_st();
          tc_fence_before_sync();
          mbar_arrive(&pt_full);
          // phase 2b, when X is complete
          mbar_wait(&xa_full, it & 1, w, 31);
          tc_fence_after_sync();
          uint32_t xr[2][16];
          if constexpr (UPPER_USED) {
            tmem_ld_x16(TX, xr[0]);
            tmem_ld_x16(TX + 16, xr[1]);
            tmem_wait_ld();
          }
#pragma unroll
          for (int hch = 0; hch < 2; ++hch) {
            if constexpr (!UPPER_USED) {
              tmem_ld_x16(TX + 16 * hch, xr[hch]);
              tmem_wait_ld();
            }
            uint32_t e0[8], l0[8], u0[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const int ip = 8 * hch + i;
              float2 X = make_float2(__uint_as_float(xr[hch][2 * i]), __uint_as_float(xr[hch][2 * i + 1]));
              if constexpr (DROP) X = __fmul2_rn(X, keep2(ip));
              const float2 ds = __fmul2_rn(P2[ip], __fadd2_rn(X, ts2[ip]));
              e0[i] = pack2<BF16>(ds.x, ds.y);
              if constexpr (SPLIT) l0[i] = pack2_residual(ds.x, ds.y, e0[i]);
              if constexpr (C::KV) u0[i] = pack_p(ip);
            }
            tmem_st_x8(TX + 8 * hch, e0);
            if constexpr (SPLIT) tmem_st_x8(TX + C::ELO + 8 * hch, l0);
            if constexpr (C::KV) tmem_st_x8(TX + C::EUP + 8 * hch, u0);
          }
        } else {
          mbar_wait(&xa_full, it & 1, w, 31);
          tc_fence_after_sync();
          const uint32_t TX = (FAM == FAM_Q) ? T3 : T2;
          uint32_t xr[2][16];
          if constexpr (UPPER_USED) {
            tmem_ld_x16(TX, xr[0]);
            tmem_ld_x16(TX + 16, xr[1]);
            tmem_wait_ld();
          }
#pragma unroll
          for (int hch = 0; hch < 2; ++hch) {
            if constexpr (!UPPER_USED) {
              tmem_ld_x16(TX + 16 * hch, xr[hch]);
              tmem_wait_ld();
            }
            uint32_t e0[8], l0[8], u0[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const int ip = 8 * hch + i;
              float2 X = make_float2(__uint_as_float(xr[hch][2 * i]), __uint_as_float(xr[hch][2 * i + 1]));
              if constexpr (DROP) X = __fmul2_rn(X, keep2(ip));
              const float2 ds = __fmul2_rn(P2[ip], __fadd2_rn(X, stat2(2, ip)));  // P (X - Delta)
              e0[i] = pack2<BF16>(ds.x, ds.y);
              if constexpr (SPLIT) l0[i] = pack2_residual(ds.x, ds.y, e0[i]);
              if constexpr (C::KV) u0[i] = pack_p(ip);
            }
            tmem_st_x8(T2 + 8 * hch, e0);
            if constexpr (SPLIT) tmem_st_x8(T2 + C::ELO + 8 * hch, l0);
            if constexpr (C::KV) tmem_st_x8(T2 + C::EUP + 8 * hch, u0);
          }
        }
      }
      tmem_wait_st();
      tc_fence_before_sync();
      mbar_arrive(&p_full[sb]);
    }
    // epilogue
    mbar_wait(&acc_final, 0, w, 32);
    tc_fence_after_sync();
    // Each warpgroup writes half of the head dimension; the rows go through this warp's patch of shared memory (the
    // first row-side tile is no longer needed: every product has completed) so that the global stores are row segments.
    if (it == 0) {   // nothing was multiplied: the row-side loads may still be in flight
      mbar_wait(&r_full, 0, w, 36);
      if constexpr (C::NR == 4) mbar_wait(&r23_full, 0, w, 38);
    }
    if constexpr (SPLIT) {
      // fp32 outputs: this warpgroup's 32 columns are 128 bytes per row
      uint8_t* patch = sR(0) + warp * (32 * 128);
      uint32_t q0[2][16], q1[2][16];
      {
        uint32_t a0[32], a1[32];
        if (it > 0) {
          tmem_ld_x32(tmem + lane_off + C::TMEM_ACC0 + wg * 32, a0);
          if constexpr (DUAL) tmem_ld_x32(tmem + lane_off + C::TMEM_ACC1 + wg * 32, a1);
          tmem_wait_ld();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) { a0[i] = 0u; a1[i] = 0u; }
        }
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          q0[i >> 4][i & 15] = __float_as_uint(__uint_as_float(a0[i]) * p.out_scale);
          if constexpr (DUAL) q1[i >> 4][i & 15] = __float_as_uint(__uint_as_float(a1[i]) * p.out_scale);
        }
      }
      const int col0 = wg * 32;
      const int wrow0 = r0 + (warp & 3) * 32;
      const size_t goff = (static_cast<size_t>(row_base) + wrow0) * p.D + col0;      // in fp32 elements
      const int rows = N - wrow0, cols16 = 2 * (p.D - col0);                          // columns in 16-bit units
      store_rows_via_smem<2>(patch, q0, reinterpret_cast<uint16_t*>(static_cast<float*>(p.out0) + goff),
                             2 * static_cast<size_t>(p.D), rows, cols16, lane);
      if constexpr (DUAL)
        store_rows_via_smem<2>(patch, q1, reinterpret_cast<uint16_t*>(static_cast<float*>(p.out1) + goff),
                               2 * static_cast<size_t>(p.D), rows, cols16, lane);
    } else {
      constexpr int CH = D / 64;
      uint8_t* patch = sR(0) + warp * (32 * CH * 64);
      const int col0 = wg * (D / 2);
      const int wrow0 = r0 + (warp & 3) * 32;
      const size_t goff = (static_cast<size_t>(row_base) + wrow0) * p.D + col0;
      const int rows = N - wrow0, cols = p.D - col0;
      // one pair of accumulators (an output and its tangent counterpart) at a time; family KV has two pairs
#pragma unroll
      for (int g = 0; g < C::NACC / 2; ++g) {
        const uint32_t acc = tmem + lane_off + (g == 0 ? C::TMEM_ACC0 : C::TMEM_ACC2);
        const float scale = (g == 0) ? p.out_scale : 1.0f;
        void* const o0 = (g == 0) ? p.out0 : p.out2;
        void* const o1 = (g == 0) ? p.out1 : p.out3;
        uint32_t q0[CH][16], q1[CH][16];
#pragma unroll
        for (int cc = 0; cc < CH; ++cc) {
          const int c = wg * CH + cc;
          uint32_t a0[32], a1[32];
          if (it > 0) {
            tmem_ld_x32(acc + c * 32, a0);
            if constexpr (DUAL) tmem_ld_x32(acc + DV + c * 32, a1);
            tmem_wait_ld();
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) { a0[i] = 0u; a1[i] = 0u; }
          }
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            q0[cc][i] = pack2<BF16>(__uint_as_float(a0[2 * i]) * scale, __uint_as_float(a0[2 * i + 1]) * scale);
            if constexpr (DUAL)
              q1[cc][i] = pack2<BF16>(__uint_as_float(a1[2 * i]) * scale, __uint_as_float(a1[2 * i + 1]) * scale);
          }
        }
        store_rows_via_smem<CH>(patch, q0, static_cast<uint16_t*>(o0) + goff, p.D, rows, cols, lane);
        if constexpr (DUAL) store_rows_via_smem<CH>(patch, q1, static_cast<uint16_t*>(o1) + goff, p.D, rows, cols, lane);
      }
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 9) tmem_dealloc(tmem, C::TMEM_COLS);
}

// Where the rows of the upstream gradients start: go and gto may be strided views, o and to are contiguous.
struct GradLayout {
  int H, N;
  TensorView go, gto;
  __host__ __device__ int64_t offset(int64_t row, const TensorView& v) const {
    if (v.sh == v.sn * N && v.sb == v.sh * H) return row * v.sn;   // rows evenly spaced (the contiguous case)
    const int64_t n = row % N, bh = row / N;
    return (bh / H) * v.sb + (bh % H) * v.sh + n * v.sn;
  }
};

// stats[row] = (lse2, mu, Delta, a) with a = rowsum(gtO o O), Delta = rowsum(gO o O) + rowsum(gtO o tO) - a mu.
// Half a warp per row; 16-bit inputs. Generalises the reference's _attn_bwd_preprocess
// (jvp_attention.py:1395-1422), which computes rowsum(O o dO) only.
template <bool BF16>
__global__ void bwd_preprocess_kernel(const uint16_t* __restrict__ o, const uint16_t* __restrict__ to,
                                      const uint16_t* __restrict__ go, const uint16_t* __restrict__ gto,
                                      const float* __restrict__ lse2, const float* __restrict__ mu,
                                      float4* __restrict__ stats, int64_t rows, int D, const GradLayout gl) {
  // half a warp per row, 16 bytes per lane and tensor in flight
  const int lane = threadIdx.x & 31, l16 = lane & 15;
  const int64_t row = (static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5)) * 2 + (lane >> 4);
  const bool live = row < rows;
  const int64_t go_row = live ? gl.offset(row, gl.go) : 0, gto_row = live ? gl.offset(row, gl.gto) : 0;
  auto lo = [](uint32_t x) -> float {
    if constexpr (BF16) return __uint_as_float(x << 16);
    else return __half2float(__ushort_as_half(static_cast<uint16_t>(x & 0xFFFFu)));
  };
  auto hi = [](uint32_t x) -> float {
    if constexpr (BF16) return __uint_as_float(x & 0xFFFF0000u);
    else return __half2float(__ushort_as_half(static_cast<uint16_t>(x >> 16)));
  };
  float s_go_o = 0.f, s_gto_to = 0.f, s_gto_o = 0.f;
  if (live) {
    for (int d = l16 * 8; d < D; d += 128) {
      const size_t idx = static_cast<size_t>(row) * D + d;
      const uint4 z = make_uint4(0u, 0u, 0u, 0u);
      const uint4 ov = *reinterpret_cast<const uint4*>(o + idx);
      const uint4 gov = *reinterpret_cast<const uint4*>(go + go_row + d);
      const uint4 tov = gto ? *reinterpret_cast<const uint4*>(to + idx) : z;
      const uint4 gtov = gto ? *reinterpret_cast<const uint4*>(gto + gto_row + d) : z;
      const uint32_t a0[4] = {ov.x, ov.y, ov.z, ov.w}, a1[4] = {tov.x, tov.y, tov.z, tov.w};
      const uint32_t a2[4] = {gov.x, gov.y, gov.z, gov.w}, a3[4] = {gtov.x, gtov.y, gtov.z, gtov.w};
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        s_go_o = fmaf(lo(a2[u]), lo(a0[u]), s_go_o);     s_go_o = fmaf(hi(a2[u]), hi(a0[u]), s_go_o);
        s_gto_to = fmaf(lo(a3[u]), lo(a1[u]), s_gto_to); s_gto_to = fmaf(hi(a3[u]), hi(a1[u]), s_gto_to);
        s_gto_o = fmaf(lo(a3[u]), lo(a0[u]), s_gto_o);   s_gto_o = fmaf(hi(a3[u]), hi(a0[u]), s_gto_o);
      }
    }
  }
#pragma unroll
  for (int off = 8; off > 0; off >>= 1) {
    s_go_o += __shfl_xor_sync(0xFFFFFFFFu, s_go_o, off);
    s_gto_to += __shfl_xor_sync(0xFFFFFFFFu, s_gto_to, off);
    s_gto_o += __shfl_xor_sync(0xFFFFFFFFu, s_gto_o, off);
  }
  if (l16 == 0 && live) {
    const float m = mu[row];
    stats[row] = make_float4(lse2[row], m, s_go_o + s_gto_to - s_gto_o * m, s_gto_o);
  }
}

// The same statistics from fp32 tensors (head dimension <= 64): half a warp per row, one float4 per lane and tensor.
__global__ void bwd_preprocess_f32_kernel(const float* __restrict__ o, const float* __restrict__ to,
                                          const float* __restrict__ go, const float* __restrict__ gto,
                                          const float* __restrict__ lse2, const float* __restrict__ mu,
                                          float4* __restrict__ stats, int64_t rows, int D, const GradLayout gl) {
  const int lane = threadIdx.x & 31, l16 = lane & 15;
  const int64_t row = (static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5)) * 2 + (lane >> 4);
  const bool live = row < rows;
  const int64_t go_row = live ? gl.offset(row, gl.go) : 0, gto_row = live ? gl.offset(row, gl.gto) : 0;
  float s_go_o = 0.f, s_gto_to = 0.f, s_gto_o = 0.f;
  if (live && l16 * 4 < D) {
    const size_t idx = static_cast<size_t>(row) * D + l16 * 4;
    const float4 z = make_float4(0.f, 0.f, 0.f, 0.f);
    const float4 ov = *reinterpret_cast<const float4*>(o + idx);
    const float4 gov = *reinterpret_cast<const float4*>(go + go_row + l16 * 4);
    const float4 tov = gto ? *reinterpret_cast<const float4*>(to + idx) : z;
    const float4 gtov = gto ? *reinterpret_cast<const float4*>(gto + gto_row + l16 * 4) : z;
    s_go_o = gov.x * ov.x + gov.y * ov.y + gov.z * ov.z + gov.w * ov.w;
    s_gto_to = gtov.x * tov.x + gtov.y * tov.y + gtov.z * tov.z + gtov.w * tov.w;
    s_gto_o = gtov.x * ov.x + gtov.y * ov.y + gtov.z * ov.z + gtov.w * ov.w;
  }
#pragma unroll
  for (int off = 8; off > 0; off >>= 1) {
    s_go_o += __shfl_xor_sync(0xFFFFFFFFu, s_go_o, off);
    s_gto_to += __shfl_xor_sync(0xFFFFFFFFu, s_gto_to, off);
    s_gto_o += __shfl_xor_sync(0xFFFFFFFFu, s_gto_o, off);
  }
  if (l16 == 0 && live) {
    const float m = mu[row];
    stats[row] = make_float4(lse2[row], m, s_go_o + s_gto_to - s_gto_o * m, s_gto_o);
  }
}

// `a` holds the operands the tensor maps are built on: in the split-fp32 mode (SPLIT) the bf16 hi/lo tensors of the
// pre-pass with 128 columns, and `real_D` is the head dimension of the outputs.
template <int D, int FAM, bool BF16, bool PAD, bool DUAL, bool SPLIT = false, bool DROP = false>
int launch_family(const jvpfa_bwd_args& a, const float4* stats, cudaStream_t stream, int real_D = 0) {
  using C = BwdCfg<D, FAM, SPLIT>;
  const TensorView vq = make_view(a.q, a.q_strides, a.H, a.N, a.D), vk = make_view(a.k, a.k_strides, a.H, a.N, a.D),
                   vv = make_view(a.v, a.v_strides, a.H, a.N, a.D), vtq = make_view(a.tq, a.tq_strides, a.H, a.N, a.D),
                   vtk = make_view(a.tk, a.tk_strides, a.H, a.N, a.D), vtv = make_view(a.tv, a.tv_strides, a.H, a.N, a.D),
                   vgo = make_view(a.go, a.go_strides, a.H, a.N, a.D), vgto = make_view(a.gto, a.gto_strides, a.H, a.N, a.D);
  TensorView rsrc[4];
  TensorView csrc[4];
  void *out0, *out1, *out2 = nullptr, *out3 = nullptr;
  float out_scale;
  if (FAM == FAM_Q) {
    rsrc[0] = vq; rsrc[1] = vtq; rsrc[2] = vgo; rsrc[3] = vgto;
    csrc[0] = vk; csrc[1] = vtk; csrc[2] = vv; csrc[3] = vtv;
    out0 = a.dq; out1 = a.dtq; out_scale = a.sm_scale;
  } else if (FAM == FAM_K || FAM == FAM_KV) {
    rsrc[0] = vk; rsrc[1] = vtk; rsrc[2] = vv; rsrc[3] = vtv;
    csrc[0] = vq; csrc[1] = vtq; csrc[2] = vgo; csrc[3] = vgto;
    out0 = a.dk; out1 = a.dtk; out_scale = a.sm_scale;
    if (FAM == FAM_KV) { out2 = a.dv; out3 = a.dtv; }
  } else {
    rsrc[0] = vk; rsrc[1] = vtk; rsrc[2] = vk; rsrc[3] = vtk;
    csrc[0] = vq; csrc[1] = vtq; csrc[2] = vgo; csrc[3] = vgto;
    out0 = a.dv; out1 = a.dtv; out_scale = 1.0f;
  }
  if (!DUAL) {  // tensors that do not exist in the primal-only call: alias the maps to existing ones, they are never used
    rsrc[1] = rsrc[0]; rsrc[3] = rsrc[2];
    csrc[1] = csrc[0]; csrc[3] = csrc[2];
  }
  CUtensorMap rm[4], cm[4];
  for (int i = 0; i < 4; ++i) {
    if (!make_tile_map(&rm[i], rsrc[i], a.B, a.H, a.N, a.D, C::BR, a.dtype)) return JVPFA_ERR_LAUNCH;
    if (!make_tile_map(&cm[i], csrc[i], a.B, a.H, a.N, a.D, C::BC, a.dtype)) return JVPFA_ERR_LAUNCH;
  }
  BwdKParams p{};
  p.H = a.H; p.N = a.N; p.D = SPLIT ? real_D : a.D; p.causal = a.causal;
  p.s = a.sm_scale;
  p.c1 = a.sm_scale * 1.4426950408889634f;
  p.out_scale = out_scale;
  p.mv = make_mask_view(a.mask, a.mask_summary, a.B, a.H, a.N);
  p.stats = stats;
  p.out0 = out0; p.out1 = out1; p.out2 = out2; p.out3 = out3;
  p.status = static_cast<int*>(a.workspace);
  p.budget_ns = wait_budget_ns();
  p.drop = make_dropout_params(a.dropout_p, a.dropout_seed);
  auto kern = bwd_sm100_kernel<D, FAM, BF16, PAD, DUAL, SPLIT, DROP>;
  const size_t smem = C::smem_bytes();
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)) != cudaSuccess)
    return JVPFA_ERR_LAUNCH;
  p.n_rt = (a.N + C::BR - 1) / C::BR;
  p.n_units = a.B * a.H;
  p.unit_group = unit_group_size(p.n_units);
  dim3 grid(static_cast<unsigned>(p.n_rt) * static_cast<unsigned>(p.n_units));
  kern<<<grid, 352, smem, stream>>>(rm[0], rm[1], rm[2], rm[3], cm[0], cm[1], cm[2], cm[3], p);
  return cudaGetLastError() == cudaSuccess ? JVPFA_OK : JVPFA_ERR_LAUNCH;
}

template <int D, bool BF16>
int launch_all(const jvpfa_bwd_args& a, cudaStream_t stream, const LaunchMarks& marks) {
  const int64_t rows = static_cast<int64_t>(a.B) * a.H * a.N;
  float4* stats = reinterpret_cast<float4*>(static_cast<uint8_t*>(a.workspace) + kStatusBytes);
  const int warps_per_block = 8;   // two rows per warp
  const unsigned blocks = static_cast<unsigned>((rows + 2 * warps_per_block - 1) / (2 * warps_per_block));
  marks.mark(0);
  const GradLayout gl{a.H, a.N, make_view(a.go, a.go_strides, a.H, a.N, a.D), make_view(a.gto, a.gto_strides, a.H, a.N, a.D)};
  bwd_preprocess_kernel<BF16><<<blocks, warps_per_block * 32, 0, stream>>>(
      static_cast<const uint16_t*>(a.o), static_cast<const uint16_t*>(a.to), static_cast<const uint16_t*>(a.go),
      static_cast<const uint16_t*>(a.gto), a.lse2, a.mu, stats, rows, a.D, gl);
  if (cudaGetLastError() != cudaSuccess) return JVPFA_ERR_LAUNCH;
  auto three = [&](auto pad, auto dual, auto drop) {
    constexpr bool P = decltype(pad)::value, DU = decltype(dual)::value, DR = decltype(drop)::value;
    marks.mark(1);
    int rc = launch_family<D, FAM_Q, BF16, P, DU, false, DR>(a, stats, stream);
    if (rc != JVPFA_OK) return rc;
    marks.mark(2);
    if constexpr (D == 64) {   // the key-side gradients in one pass
      rc = launch_family<D, FAM_KV, BF16, P, DU, false, DR>(a, stats, stream);
      marks.mark(3);
    } else {
      rc = launch_family<D, FAM_K, BF16, P, DU, false, DR>(a, stats, stream);
      if (rc != JVPFA_OK) return rc;
      marks.mark(3);
      rc = launch_family<D, FAM_V, BF16, P, DU, false, DR>(a, stats, stream);
    }
    marks.mark(4);
    return rc;
  };
  const bool dual = a.tq != nullptr;
  if (a.dropout_p > 0.f) {
    if (a.D == D) return dual ? three(std::false_type{}, std::true_type{}, std::true_type{}) : three(std::false_type{}, std::false_type{}, std::true_type{});
    return dual ? three(std::true_type{}, std::true_type{}, std::true_type{}) : three(std::true_type{}, std::false_type{}, std::true_type{});
  }
  if (a.D == D) return dual ? three(std::false_type{}, std::true_type{}, std::false_type{}) : three(std::false_type{}, std::false_type{}, std::false_type{});
  return dual ? three(std::true_type{}, std::true_type{}, std::false_type{}) : three(std::true_type{}, std::false_type{}, std::false_type{});
}

// fp32 inputs: statistics from the fp32 tensors, split pre-pass of the eight (primal-only: four) MMA operands into the
// workspace, then the three family kernels in their split mode on the split tensors. Workspace: status block, statistics,
// split tensors.
template <bool DUAL, bool DROP>
int launch_split(const jvpfa_bwd_args& a, cudaStream_t stream, const LaunchMarks& marks) {
  const int64_t rows = static_cast<int64_t>(a.B) * a.H * a.N;
  uint8_t* ws = static_cast<uint8_t*>(a.workspace);
  float4* stats = reinterpret_cast<float4*>(ws + kStatusBytes);
  uint8_t* base = ws + kStatusBytes + align_up(static_cast<size_t>(rows) * sizeof(float4), 256);
  const int n_t = DUAL ? 8 : 4;
  const void* src[8] = {a.q, a.k, a.v, a.go, a.tq, a.tk, a.tv, a.gto};
  uint16_t* dst[8];
  for (int i = 0; i < n_t; ++i) dst[i] = reinterpret_cast<uint16_t*>(base + static_cast<size_t>(i) * rows * kSplitRowBytes);
  marks.mark(0);
  const int warps_per_block = 8;   // two rows per warp
  const unsigned blocks = static_cast<unsigned>((rows + 2 * warps_per_block - 1) / (2 * warps_per_block));
  const GradLayout gl{a.H, a.N, make_view(a.go, a.go_strides, a.H, a.N, a.D), make_view(a.gto, a.gto_strides, a.H, a.N, a.D)};
  bwd_preprocess_f32_kernel<<<blocks, warps_per_block * 32, 0, stream>>>(
      static_cast<const float*>(a.o), static_cast<const float*>(a.to), static_cast<const float*>(a.go),
      static_cast<const float*>(a.gto), a.lse2, a.mu, stats, rows, a.D, gl);
  if (cudaGetLastError() != cudaSuccess) return JVPFA_ERR_LAUNCH;
  const jvpfa_strides* sst[8] = {&a.q_strides, &a.k_strides, &a.v_strides, &a.go_strides,
                                 &a.tq_strides, &a.tk_strides, &a.tv_strides, &a.gto_strides};
  TensorView views[8];
  for (int i = 0; i < n_t; ++i) views[i] = make_view(src[i], *sst[i], a.H, a.N, a.D);
  int rc = launch_split_fp32(views, dst, n_t, a.B, a.H, a.N, a.D, stream);
  if (rc != JVPFA_OK) return rc;
  jvpfa_bwd_args m = a;      // what the tensor maps are built on: the contiguous split tensors
  m.D = 128;
  m.dtype = JVPFA_BF16;
  const jvpfa_strides none{0, 0, 0};
  m.q_strides = m.k_strides = m.v_strides = m.tq_strides = m.tk_strides = m.tv_strides = m.go_strides = m.gto_strides = none;
  m.q = dst[0]; m.k = dst[1]; m.v = dst[2]; m.go = dst[3];
  if (DUAL) { m.tq = dst[4]; m.tk = dst[5]; m.tv = dst[6]; m.gto = dst[7]; }
  marks.mark(1);
  rc = launch_family<128, FAM_Q, true, false, DUAL, true, DROP>(m, stats, stream, a.D);
  if (rc != JVPFA_OK) return rc;
  marks.mark(2);
  rc = launch_family<128, FAM_K, true, false, DUAL, true, DROP>(m, stats, stream, a.D);
  if (rc != JVPFA_OK) return rc;
  marks.mark(3);
  rc = launch_family<128, FAM_V, true, false, DUAL, true, DROP>(m, stats, stream, a.D);
  marks.mark(4);
  return rc;
}

}  // namespace

size_t bwd_sm100_split_workspace_bytes(const jvpfa_bwd_args& a) {
  const size_t rows = static_cast<size_t>(a.B) * a.H * a.N;
  return kStatusBytes + align_up(rows * sizeof(float4), 256) + (a.tq != nullptr ? 8 : 4) * rows * kSplitRowBytes;
}

int launch_bwd_sm100_split(const jvpfa_bwd_args& a, cudaStream_t stream, const LaunchMarks& marks) {
  if (a.dropout_p > 0.f)
    return a.tq != nullptr ? launch_split<true, true>(a, stream, marks) : launch_split<false, true>(a, stream, marks);
  return a.tq != nullptr ? launch_split<true, false>(a, stream, marks) : launch_split<false, false>(a, stream, marks);
}

size_t bwd_sm100_workspace_bytes(const jvpfa_bwd_args& a) {
  return kStatusBytes + static_cast<size_t>(a.B) * a.H * a.N * sizeof(float4);
}

int launch_bwd_sm100(const jvpfa_bwd_args& a, cudaStream_t stream, const LaunchMarks& marks) {
  const bool bf = a.dtype == JVPFA_BF16;
  if (sm100_padded_dim(a.D) == 64) return bf ? launch_all<64, true>(a, stream, marks) : launch_all<64, false>(a, stream, marks);
  return bf ? launch_all<128, true>(a, stream, marks) : launch_all<128, false>(a, stream, marks);
}

}  // namespace jvpfa
