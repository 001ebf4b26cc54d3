// Dual (JVP) attention forward for sm_100a: O = softmax(s QK^T + mask) V and its tangent tO in one
// pass, with tcgen05 MMAs accumulating in TMEM and K/tK/V/tV tiles staged by TMA.
//
// Replaces the reference's _attn_fwd_tma / _attn_fwd_inner_tma (jvp_flash_attention/jvp_attention.py:
// 1100-1392, 350-559). Per (128-row query tile, batch*head) one CTA of 12 warps:
//   warps 0-7  two softmax warpgroups that split the 64 columns of every score tile: thread r of a
//              warpgroup owns score row r (TMEM lane r) and 32 columns; keeps m, l, mu in registers, turns the
//              score tile S and tangent-score tile tS into 16-bit P and W = P o (s tS) written back to TMEM;
//              the two halves of a row exchange their maxima (and, at the end, their sums) through shared memory
//   warp 8     TMA producer of Q, tQ and the stacked [K; tK] pairs (one lane)
//   warp 11    TMA producer of the V, tV tiles (one lane)
//   warp 9     issues the score products (lane 0); owns the TMEM allocation
//   warp 10    issues the output products (lane 0). tcgen05.mma issue blocks once three to four instructions are
//              queued, so one issuing thread idles the tensor pipe during each of its barrier waits and commits;
//              two instruction streams keep it fed.
// Per 64-column key tile: [S | Q tK^T] = Q [K; tK]^T as one N = 128 product against the stacked pair, then
// tS += tQ K^T (operands in shared memory), then O += P V, T += W V + P tV (P, W read from TMEM; V, tV as
// MN-major shared-memory operands). Epilogue: O/l, tO = T/l - (mu/l) O/l, lse2 = m + log2 l, mu/l.
// TMEM columns: O [0,D), T [D,2D), one score buffer (S 64 | tS 64), then two buffers of 16-bit (P 32 | W 32). The score
// buffer is released as soon as every softmax thread holds its part of S, tS in registers, so that the next tile's
// score products are queued behind the running output products instead of waiting for them to complete.
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


struct FwdKParams {
  int H, N;
  int n_qt, n_units;   // query tiles per (batch, head) unit, number of units: the grid has n_qt * n_units blocks
  int unit_group;      // units per group of the block order
  int D;       // head dimension of the tensors (the kernel is compiled for it rounded up to 64 or 128)
  int causal;
  float c1;      // sm_scale * log2(e)
  float s;       // sm_scale
  float thresh;  // lazy-rescale threshold in the log2 domain
  MaskView mv;
  void* o;
  void* to;
  float* lse2;
  float* mu;
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

__device__ __forceinline__ uint32_t pack2_residual(float a, float b, uint32_t hi) {
  return pack2<true>(a - __uint_as_float(hi << 16), b - __uint_as_float(hi & 0xFFFF0000u));
}

// SPLIT: fp32 inputs on the tensor cores. A pre-pass splits every fp32 operand x into two bf16 numbers hi + lo (x - hi - lo
// is below 2^-18 |x|) and writes them side by side as one 128-column row [hi(64) | lo(64)], so the tiles have the
// shared-memory geometry of the D = 128 kernel with the hi part in slab 0 and the lo part in slab 1; every product a b is
// then accumulated in fp32 as a_hi b_hi + a_lo b_hi + a_hi b_lo (what is left out is of the order 2^-18 |a||b|; an fp16 lo
// part would carry three more bits, but one product cannot take an fp16 operand against a bf16 one). The accumulators are 64
// columns wide, P and W = P o (s tS) go back to TMEM as hi and lo parts, and the outputs are written as fp32.
template <int D, bool SPLIT = false>
struct FwdCfg {
  static constexpr int BM = 128;
  static constexpr int BN = 64;
  static constexpr int STAGES = (D == 64) ? 4 : 2;
  static constexpr int TILE_Q = BM * D * 2;
  static constexpr int TILE_V = BN * D * 2;
  static constexpr int PAIR_K = 2 * BN * D * 2;  // K and tK stacked as one 128-row operand
  static constexpr int SLAB = 128 * 128;          // bytes of one 64-column slab of a 128-row tile
  static constexpr int HALF = BN * 128;           // byte offset of tK inside a slab of the pair
  static constexpr int STAGE = PAIR_K + 2 * TILE_V;
  static constexpr int DV = SPLIT ? 64 : D;      // columns of the O and T accumulators
  static constexpr int TMEM_O = 0;
  static constexpr int TMEM_T = DV;
  static constexpr int TMEM_S = 2 * DV;       // S 64 columns, tS 64 columns further (one buffer)
  static constexpr int TMEM_P = 2 * DV + 128; // 16-bit P (32 columns) and W (32 columns further), buffer b at + PBUF b;
  static constexpr int PBUF = SPLIT ? 128 : 64;  // SPLIT: P hi, P lo, W hi, W lo, 32 columns each
  static constexpr int TMEM_COLS = 512;
  static constexpr int NBAR = 4 + 4 * STAGES + 4 + 2;
  static constexpr size_t smem_bytes() { return 2 * TILE_Q + STAGES * STAGE + 2 * 2 * 128 * 4 + (NBAR + 2) * 8; }
};

// Warps 0-7: two softmax warpgroups that split the 64 columns of every score tile (thread = TMEM lane =
// one score row, 32 columns; the row maximum and the final row sums are exchanged through shared
// memory); warps 8, 11: TMA producers (one lane each: Q and K pairs / V tiles); warps 9, 10: MMA issuers (one lane each: scores / outputs), warp 9 owns the
// TMEM allocation.
// PAD: the tensors' head dimension is smaller than D (columns beyond it are zero-filled by TMA); the K steps and
// output columns that would only see zeros are then skipped at run time.
// DROP: dropout on the attention probabilities (dropout.cuh): P and W reach TMEM dropped out and rescaled, the row sums l
// and mu are those of the probabilities before dropout.
template <int D, bool DUAL, bool BF16, bool PAD, bool SPLIT = false, bool DROP = false>
__global__ void __launch_bounds__(384, 1)
fwd_sm100_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmTQ,
                 const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmTK,
                 const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmTV,
                 const FwdKParams p) {
  using C = FwdCfg<D, SPLIT>;
  constexpr int ST = C::STAGES;
  constexpr int SLABS = D / 64;
  constexpr int DV = C::DV;
  static_assert(!SPLIT || (D == 128 && BF16 && !PAD), "the split-fp32 mode runs on the 128-column geometry in bf16");

  extern __shared__ __align__(1024) uint8_t smem[];
  uint8_t* sQ = smem;
  uint8_t* sTQ = sQ + C::TILE_Q;
  auto sK = [&](int st) { return smem + 2 * C::TILE_Q + st * C::STAGE; };   // [K; tK] pair
  auto sV = [&](int st) { return sK(st) + C::PAIR_K; };
  auto sTV = [&](int st) { return sV(st) + C::TILE_V; };
  uint8_t* tail = smem + 2 * C::TILE_Q + ST * C::STAGE;
  float(*xch)[2][128] = reinterpret_cast<float(*)[2][128]>(tail);          // [parity][warpgroup][row]
  uint64_t* bars = reinterpret_cast<uint64_t*>(tail + 2 * 2 * 128 * 4);
  uint64_t& q_full = bars[0];
  uint64_t& o_done = bars[1];
  uint64_t& o_final = bars[2];
  uint64_t& s_full = bars[4];        // S, tS of the current tile are complete
  uint64_t& s_free = bars[5];        // all 256 softmax threads have S, tS in registers: the next tile's products may overwrite them
  uint64_t* p_full = bars + 6;       // [2]
  uint64_t* k_full = bars + 8;
  uint64_t* v_full = k_full + ST;
  uint64_t* k_empty = v_full + ST;
  uint64_t* v_empty = k_empty + ST;
  uint64_t* p_free = v_empty + ST;   // [2]: the PV products that read P, W buffer b have completed
  uint32_t& tmem_base_s = *reinterpret_cast<uint32_t*>(bars + C::NBAR);
  int& poisoned = *reinterpret_cast<int*>(bars + C::NBAR + 1);
  if ((smem_u32(smem) & 1023u) != 0u) {  // the swizzled layouts need this; never observed otherwise
    if (threadIdx.x == 0) atomicCAS(p.status, 0, WAIT_TIMEOUT_BASE + 99);
    return;
  }

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const BlockWork work = block_work(blockIdx.x, p.n_qt, p.n_units, p.unit_group, p.causal != 0);   // heavy query tiles first
  const int qt = work.tile;
  const int bh = work.unit;
  const int b = bh / p.H, h = bh % p.H;
  const int q0 = qt * C::BM;
  const int N = p.N;
  const int row_base = bh * N;
  int n_kt = (N + C::BN - 1) / C::BN;
  if (p.causal) n_kt = min(n_kt, (q0 + C::BM - 1) / C::BN + 1);

  const WaitCtx w{p.status, &poisoned, p.budget_ns};

  if (tid == 0) {
    poisoned = 0;
    mbar_init(&q_full, 1);
    for (int i = 0; i < ST; ++i) {
      mbar_init(&k_full[i], 1);
      mbar_init(&v_full[i], 1);
      mbar_init(&k_empty[i], 1);
      mbar_init(&v_empty[i], 1);
    }
    mbar_init(&s_full, 1);
    mbar_init(&s_free, 256);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&p_full[i], 256);
      mbar_init(&p_free[i], 1);
    }
    mbar_init(&o_done, 1);
    mbar_init(&o_final, 1);
    fence_mbar_init();
  }
  __syncthreads();
  if (warp == 9) {
    tmem_alloc(&tmem_base_s, C::TMEM_COLS);
    tmem_relinquish();
  }
  // the TMA producers need the barriers but not the TMEM address: they start loading while TMEM is being allocated
  const bool producer = (warp == 8 || warp == 11);
  tc_fence_before_sync();
  if (!producer) named_bar_sync(2, 320);
  tc_fence_after_sync();
  const uint32_t tmem = producer ? 0u : tmem_base_s;

  // Key tile j takes part unless the mask summary says that nothing in it is kept.
  auto tile_bits = [&](int j) -> uint8_t {
    if (p.mv.kind == JVPFA_MASK_NONE) return kTileAnyKept;
    uint8_t bits = mask_tile_bits(p.mv, b, h, 2 * qt, j);
    if (2 * qt + 1 < p.mv.n64) bits |= mask_tile_bits(p.mv, b, h, 2 * qt + 1, j);
    return bits;
  };

  if (warp == 11) {
    // ------------------------------------------------------------------ TMA producer of the V, tV tiles (a warp of
    // its own: V slots free up a tile later than K slots, one producer waiting for them would hold the K loads back)
    if (lane == 0) {
      int it = 0;
      for (int j = 0; j < n_kt; ++j) {
        if (!(tile_bits(j) & kTileAnyKept)) continue;
        const int st = it % ST;
        const uint32_t ph = (it / ST) & 1;
        const int krow = j * C::BN;   // first key row of the tile inside its (batch, head) unit
        mbar_wait(&v_empty[st], ph ^ 1, w, 11);
        mbar_arrive_expect_tx(&v_full[st], (DUAL ? 2 : 1) * C::TILE_V);
        if constexpr (!PAD && SLABS > 1) {
          // the slabs of a V tile are consecutive in shared memory: one box per tensor through the 3-D map
          tma_load_slabs(sV(st), &tmV, &v_full[st], krow, h, b);
          if constexpr (DUAL) tma_load_slabs(sTV(st), &tmTV, &v_full[st], krow, h, b);
        } else {
#pragma unroll
          for (int sl = 0; sl < SLABS; ++sl) {
            tma_load_tile(sV(st) + sl * C::HALF, &tmV, &v_full[st], 64 * sl, krow, h, b);
            if constexpr (DUAL) tma_load_tile(sTV(st) + sl * C::HALF, &tmTV, &v_full[st], 64 * sl, krow, h, b);
          }
        }
        ++it;
      }
    }
    __syncwarp();
  } else if (warp == 8) {
    // ------------------------------------------------------------------ TMA producer of Q, tQ and the [K; tK] pairs
    if (lane == 0) {
      tma_prefetch_desc(&tmQ);
      tma_prefetch_desc(&tmK);
      tma_prefetch_desc(&tmV);
      mbar_arrive_expect_tx(&q_full, (DUAL ? 2 : 1) * C::TILE_Q);
#pragma unroll
      for (int sl = 0; sl < SLABS; ++sl) {
        tma_load_tile(sQ + sl * C::SLAB, &tmQ, &q_full, 64 * sl, q0, h, b);
        if constexpr (DUAL) tma_load_tile(sTQ + sl * C::SLAB, &tmTQ, &q_full, 64 * sl, q0, h, b);
      }
      int it = 0;
      for (int j = 0; j < n_kt; ++j) {
        if (!(tile_bits(j) & kTileAnyKept)) continue;
        const int st = it % ST;
        const uint32_t ph = (it / ST) & 1;
        const int krow = j * C::BN;   // first key row of the tile inside its (batch, head) unit
        mbar_wait(&k_empty[st], ph ^ 1, w, 10);
        mbar_arrive_expect_tx(&k_full[st], (DUAL ? 2 : 1) * C::TILE_V);
#pragma unroll
        for (int sl = 0; sl < SLABS; ++sl) {
          tma_load_tile(sK(st) + sl * C::SLAB, &tmK, &k_full[st], 64 * sl, krow, h, b);
          if constexpr (DUAL) tma_load_tile(sK(st) + sl * C::SLAB + C::HALF, &tmTK, &k_full[st], 64 * sl, krow, h, b);
        }
        ++it;
      }
    }
    __syncwarp();
  } else if (warp >= 9) {
    // ------------------------------------------------------------------ MMA issuers: warp 9 scores, warp 10 outputs
    // all lanes run the loops (waits included) so that the warp stays converged; the elected lane issues
    const bool leader = elect_one_sync();
    auto wait_all = [&](uint64_t* bar, uint32_t parity, int site) {
      mbar_wait(bar, parity, w, site);
      __syncwarp();
    };
    {
    constexpr uint32_t FMT = BF16 ? FMT_BF16 : FMT_F16;
    const uint32_t idesc_64 = make_idesc(FMT, 128, 64, 0, 0);
    const uint32_t idesc_128 = make_idesc(FMT, 128, 128, 0, 0);
    const int dn = SPLIT ? 64 : (PAD ? ((p.D + 15) & ~15) : D);   // columns of the output products (head dimension rounded up to the MMA granularity)
    const int ksteps = dn / 16;                            // K steps of the score products that hold data
    const uint32_t idesc_pv = make_idesc(FMT, 128, dn, 0, 1);
    const uint64_t dQ = desc_kmajor_sw128(smem_u32(sQ)), dTQ = desc_kmajor_sw128(smem_u32(sTQ));

    auto issue_qk = [&](int it) {
      const int st = it % ST;
      const uint32_t ph = (it / ST) & 1;
      const uint32_t S_t = tmem + C::TMEM_S;
      wait_all(&k_full[st], ph, 20);
      if (it >= 1) wait_all(&s_free, (it - 1) & 1, 24);
      tc_fence_after_sync();
      const uint64_t dK = desc_kmajor_sw128(smem_u32(sK(st)));
      if (leader) {
        if constexpr (SPLIT) {
          // hi hi + lo hi + hi lo: K steps 0-3 of the left (a) and right (b) operand's slab 0 (hi) or slab 1 (lo)
#pragma unroll
          for (int k = 0; k < 12; ++k) {
            const int a_slab = (k >> 2) == 1, b_slab = (k >> 2) == 2;
            const uint64_t oa = static_cast<uint64_t>((a_slab * C::SLAB + (k & 3) * 32) >> 4);
            const uint64_t ob = static_cast<uint64_t>((b_slab * C::SLAB + (k & 3) * 32) >> 4);
            umma_ss(S_t, dQ + oa, dK + ob, DUAL ? idesc_128 : idesc_64, k > 0);                        // [S | Q tK^T]
          }
          if constexpr (DUAL) {
#pragma unroll
            for (int k = 0; k < 12; ++k) {
              const int a_slab = (k >> 2) == 1, b_slab = (k >> 2) == 2;
              const uint64_t oa = static_cast<uint64_t>((a_slab * C::SLAB + (k & 3) * 32) >> 4);
              const uint64_t ob = static_cast<uint64_t>((b_slab * C::SLAB + (k & 3) * 32) >> 4);
              umma_ss(S_t + 64, dTQ + oa, dK + ob, idesc_64, 1);                                        // tS += tQ K^T
            }
          }
        } else {
#pragma unroll
          for (int k = 0; k < D / 16; ++k) {
            const uint64_t o = static_cast<uint64_t>(((k >> 2) * C::SLAB + (k & 3) * 32) >> 4);
            if (!PAD || k < ksteps) umma_ss(S_t, dQ + o, dK + o, DUAL ? idesc_128 : idesc_64, k > 0);   // [S | Q tK^T]
          }
          if constexpr (DUAL) {
#pragma unroll
            for (int k = 0; k < D / 16; ++k) {
              const uint64_t o = static_cast<uint64_t>(((k >> 2) * C::SLAB + (k & 3) * 32) >> 4);
              if (!PAD || k < ksteps) umma_ss(S_t + 64, dTQ + o, dK + o, idesc_64, 1);                    // tS += tQ K^T
            }
          }
        }
        umma_commit(&s_full);
        umma_commit(&k_empty[st]);
      }
    };
    auto issue_pv = [&](int it, bool last) {
      const int st = it % ST;
      const uint32_t ph = (it / ST) & 1;
      const uint32_t P_t = tmem + C::TMEM_P + (it & 1) * C::PBUF;
      const uint32_t W_t = P_t + (SPLIT ? 64 : 32);
      wait_all(&p_full[it & 1], (it >> 1) & 1, 21);
      wait_all(&v_full[st], ph, 22);
      tc_fence_after_sync();
      const uint64_t dV0 = desc_mnmajor_sw128(smem_u32(sV(st)), C::BN * 128);
      const uint64_t dTV0 = desc_mnmajor_sw128(smem_u32(sTV(st)), C::BN * 128);
      const uint32_t acc0 = it > 0;
      if (leader) {
#pragma unroll
        for (int k = 0; k < C::BN / 16; ++k) {
          const uint64_t ok = static_cast<uint64_t>((k * 2048) >> 4);
          const uint32_t eo = k * 8;
          if constexpr (SPLIT) {
            // the lo part of an operand in TMEM sits 32 columns after its hi part, the lo slab of V, tV one slab further
            const uint64_t lo = static_cast<uint64_t>(C::HALF >> 4);
            // acc += e_hi c_hi + e_lo c_hi + e_hi c_lo
            auto three = [&](uint32_t accum, uint32_t e, uint64_t c, uint32_t first_acc) {
              umma_ts(accum, e, c, idesc_pv, first_acc);
              umma_ts(accum, e + 32, c, idesc_pv, 1);
              umma_ts(accum, e, c + lo, idesc_pv, 1);
            };
            three(tmem + C::TMEM_O, P_t + eo, dV0 + ok, acc0 | (k > 0));
            if constexpr (DUAL) {
              three(tmem + C::TMEM_T, W_t + eo, dV0 + ok, acc0 | (k > 0));
              three(tmem + C::TMEM_T, P_t + eo, dTV0 + ok, 1);
            }
          } else {
            umma_ts(tmem + C::TMEM_O, P_t + eo, dV0 + ok, idesc_pv, acc0 | (k > 0));
            if constexpr (DUAL) {
              umma_ts(tmem + C::TMEM_T, W_t + eo, dV0 + ok, idesc_pv, acc0 | (k > 0));
              umma_ts(tmem + C::TMEM_T, P_t + eo, dTV0 + ok, idesc_pv, 1);
            }
          }
        }
        umma_commit(&v_empty[st]);
        umma_commit(&p_free[it & 1]);
        umma_commit(&o_done);
        if (last) umma_commit(&o_final);
      }
    };

    int it = 0;
    if (warp == 9) {
      wait_all(&q_full, 0, 23);
      for (int j = 0; j < n_kt; ++j) {
        if (!(tile_bits(j) & kTileAnyKept)) continue;
        issue_qk(it);
        ++it;
      }
    } else {
      for (int j = 0; j < n_kt; ++j) {
        if (!(tile_bits(j) & kTileAnyKept)) continue;
        if (it > 0) issue_pv(it - 1, false);
        ++it;
      }
      if (it > 0) issue_pv(it - 1, true);
    }
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------------ softmax, correction, epilogue
    const int wg = warp >> 2;
    const int r = (warp & 3) * 32 + lane;
    const int qi = q0 + r;
    const int qi_c = min(qi, N - 1);
    const uint32_t lane_off = static_cast<uint32_t>((warp & 3) * 32) << 16;
    float m_used = -INFINITY;
    float2 l2 = make_float2(0.f, 0.f), mu2 = make_float2(0.f, 0.f);   // partial row sums over this thread's columns
    const float2 c1_2 = make_float2(p.c1, p.c1), s_2 = make_float2(p.s, p.s);
    int it = 0;
    for (int j = 0; j < n_kt; ++j) {
      const uint8_t bits = tile_bits(j);
      if (!(bits & kTileAnyKept)) continue;
      const uint32_t S_t = tmem + C::TMEM_S + lane_off + 32 * wg;
      const uint32_t tS_t = S_t + 64;
      const uint32_t P_t = tmem + C::TMEM_P + (it & 1) * C::PBUF + lane_off + 16 * wg;   // this thread's 16 columns of P
      const uint32_t W_t = P_t + (SPLIT ? 64 : 32);
      mbar_wait(&s_full, it & 1, w, 30);
      tc_fence_after_sync();
      // scores of this thread's 32 columns in the log2 domain, two per register pair (packed fp32x2
      // arithmetic: the softmax warps share their schedulers with the MMA-issuing warp)
      float2 x2[16];
      uint32_t ts[32];
      {
        uint32_t r0[32];
        tmem_ld_x32(S_t, r0);
        if constexpr (DUAL) tmem_ld_x32(tS_t, ts);
        tmem_wait_ld();
        // S and tS are in registers: the next tile's score products may overwrite them
        tc_fence_before_sync();
        mbar_arrive(&s_free);
#pragma unroll
        for (int i = 0; i < 16; ++i)
          x2[i] = __fmul2_rn(make_float2(__uint_as_float(r0[2 * i]), __uint_as_float(r0[2 * i + 1])), c1_2);
      }
      const int k0 = j * C::BN + 32 * wg;   // first key of this thread's columns
      const bool need_causal = p.causal && j * C::BN + C::BN - 1 > q0;
      const bool need_bound = j * C::BN + C::BN > N;
      const bool need_mask = p.mv.kind != JVPFA_MASK_NONE && (bits & kTileAnyMasked);
      // The mask as this thread sees it: the flags of its own 64x64 tile (the two 64-row halves of the query tile may
      // differ). Packed by the summary pre-pass (a boolean mask, or a two-valued tile of an additive one), this row's 32
      // entries of the tile are one word; anything else is read element by element below.
      int mask_mode = 0;
      if (need_mask) mask_mode = mask_tile_mode(p.mv, mask_tile_bits(p.mv, b, h, qi_c >> 6, j));
      if (mask_mode == 1) {
        const float other = p.mv.kind == JVPFA_MASK_BOOL ? -INFINITY : mask_tile_value(p.mv, b, h, qi_c >> 6, j) * 1.4426950408889634f;
        mask_apply_bits(x2, mask_row_bits(p.mv, b, h, qi_c, j, wg), other);
      }
      const bool mask_elems = mask_mode == 2;
      // (keys past the end of the sequence: zero bits of a boolean mask already exclude them)
      if (need_causal || (need_bound && !(mask_mode == 1 && p.mv.kind == JVPFA_MASK_BOOL)) || mask_elems) {
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          float bias[16];
#pragma unroll
          for (int i = 0; i < 16; ++i) bias[i] = 0.f;
          if (mask_elems) mask_bias_run<16>(bias, p.mv, b, h, qi_c, k0 + 16 * c, N, true);
          if (need_causal) {
#pragma unroll
            for (int i = 0; i < 16; ++i)
              if (k0 + 16 * c + i > qi) bias[i] = -INFINITY;
          }
          if (need_bound) {
#pragma unroll
            for (int i = 0; i < 16; ++i)
              if (k0 + 16 * c + i >= N) bias[i] = -INFINITY;
          }
#pragma unroll
          for (int i = 0; i < 8; ++i) x2[8 * c + i] = __fadd2_rn(x2[8 * c + i], make_float2(bias[2 * i], bias[2 * i + 1]));
        }
      }
      float m_tile = fmaxf(x2[0].x, x2[0].y);
#pragma unroll
      for (int i = 1; i < 16; ++i) m_tile = fmaxf(m_tile, fmaxf(x2[i].x, x2[i].y));
      // row maximum over both warpgroups: the two warps that share these 32 rows meet on a barrier of their own
      xch[it & 1][wg][r] = m_tile;
      named_bar_sync(3 + (warp & 3), 64);
      m_tile = fmaxf(m_tile, xch[it & 1][wg ^ 1][r]);
      const float m_new = fmaxf(m_used, m_tile);
      const bool need = m_new > m_used + p.thresh;
      if (__any_sync(0xFFFFFFFFu, need)) {   // same rows, same values in both warpgroups: same decision
        const float alpha = (m_used == -INFINITY) ? 1.0f : fast_exp2(m_used - m_new);
        if (it > 0) {
          mbar_wait(&o_done, (it - 1) & 1, w, 31);
          tc_fence_after_sync();
          // warpgroup 0 rescales O, warpgroup 1 rescales T
          if (DUAL || wg == 0) {
            const uint32_t base = tmem + lane_off + (wg == 0 ? C::TMEM_O : C::TMEM_T);
#pragma unroll
            for (int c = 0; c < DV / 32; ++c) {
              uint32_t a[32];
              tmem_ld_x32(base + c * 32, a);
              tmem_wait_ld();
#pragma unroll
              for (int i = 0; i < 32; ++i) a[i] = __float_as_uint(__uint_as_float(a[i]) * alpha);
              tmem_st_x32(base + c * 32, a);
            }
          }
        }
        l2.x *= alpha; l2.y *= alpha;
        mu2.x *= alpha; mu2.y *= alpha;
        m_used = m_new;
      }
      const float m_eff = (m_used == -INFINITY) ? 0.f : m_used;
      const float2 nm2 = make_float2(-m_eff, -m_eff);
      uint32_t keep_bits = 0xFFFFFFFFu;
      if constexpr (DROP) keep_bits = dropout_keep_along_k(p.drop, bh, qi, k0);
      {
        // the PV products of tile it - 2 read this P, W buffer
        if (it >= 2) {
          mbar_wait(&p_free[it & 1], ((it >> 1) - 1) & 1, w, 33);
          tc_fence_after_sync();
        }
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          uint32_t pk[8], wk[8], pkl[8], wkl[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const int ip = 8 * c + i;
            const float2 e = __fadd2_rn(x2[ip], nm2);
            const float2 pp = make_float2(fast_exp2(e.x), fast_exp2(e.y));
            l2 = __fadd2_rn(l2, pp);
            float2 keep2 = make_float2(1.f, 1.f);
            if constexpr (DROP) keep2 = dropout_factors(keep_bits, ip, p.drop.inv_keep);
            const float2 pd = DROP ? __fmul2_rn(pp, keep2) : pp;     // what multiplies V, tV
            pk[i] = pack2<BF16>(pd.x, pd.y);
            if constexpr (SPLIT) pkl[i] = pack2_residual(pd.x, pd.y, pk[i]);
            if constexpr (DUAL) {
              const float2 tsv = __fmul2_rn(make_float2(__uint_as_float(ts[2 * ip]), __uint_as_float(ts[2 * ip + 1])), s_2);
              const float2 ww = __fmul2_rn(pp, tsv);
              mu2 = __fadd2_rn(mu2, ww);
              const float2 wd = DROP ? __fmul2_rn(ww, keep2) : ww;
              wk[i] = pack2<BF16>(wd.x, wd.y);
              if constexpr (SPLIT) wkl[i] = pack2_residual(wd.x, wd.y, wk[i]);
            }
          }
          tmem_st_x8(P_t + 8 * c, pk);
          if constexpr (SPLIT) tmem_st_x8(P_t + 32 + 8 * c, pkl);
          if constexpr (DUAL) {
            tmem_st_x8(W_t + 8 * c, wk);
            if constexpr (SPLIT) tmem_st_x8(W_t + 32 + 8 * c, wkl);
          }
        }
      }
      tmem_wait_st();
      tc_fence_before_sync();
      mbar_arrive(&p_full[it & 1]);
      ++it;
    }
    // epilogue: total row sums over both warpgroups, then each warpgroup writes half of the head dimension.
    // o_done flips once per key tile and a parity wait is only meaningful within one phase of the
    // barrier, so the end of the last accumulation has a barrier of its own.
    float l = l2.x + l2.y, mu = mu2.x + mu2.y;
    named_bar_sync(3 + (warp & 3), 64);
    xch[0][wg][r] = l;
    xch[1][wg][r] = mu;
    named_bar_sync(3 + (warp & 3), 64);
    l += xch[0][wg ^ 1][r];
    mu += xch[1][wg ^ 1][r];
    if (it > 0) {
      mbar_wait(&o_final, 0, w, 32);
      tc_fence_after_sync();
    }
    const float linv = (l > 0.f) ? 1.0f / l : 0.f;
    const float mul = mu * linv;
    // Each warpgroup writes half of the head dimension; the rows go through this warp's patch of shared memory (the Q
    // tile is no longer needed: every product that reads it has completed) so that the global stores are row segments.
    if (it == 0) mbar_wait(&q_full, 0, w, 34);   // nothing was multiplied: the Q load itself may still be in flight
    if constexpr (SPLIT) {
      // fp32 outputs: this warpgroup's 32 columns are 128 bytes per row
      uint8_t* patch = sQ + warp * (32 * 128);
      uint32_t po[2][16], pt[2][16];
      {
        uint32_t ov[32], tv[32];
        if (it > 0) {
          tmem_ld_x32(tmem + lane_off + C::TMEM_O + wg * 32, ov);
          if constexpr (DUAL) tmem_ld_x32(tmem + lane_off + C::TMEM_T + wg * 32, tv);
          tmem_wait_ld();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) { ov[i] = 0u; tv[i] = 0u; }
        }
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const float o = __uint_as_float(ov[i]) * linv;
          po[i >> 4][i & 15] = __float_as_uint(o);
          if constexpr (DUAL) pt[i >> 4][i & 15] = __float_as_uint(__uint_as_float(tv[i]) * linv - mul * o);
        }
      }
      const int col0 = wg * 32;
      const int wrow0 = q0 + (warp & 3) * 32;
      const size_t goff = (static_cast<size_t>(row_base) + wrow0) * p.D + col0;      // in fp32 elements
      const int rows = N - wrow0, cols16 = 2 * (p.D - col0);                          // columns in 16-bit units
      store_rows_via_smem<2>(patch, po, reinterpret_cast<uint16_t*>(static_cast<float*>(p.o) + goff), 2 * static_cast<size_t>(p.D),
                             rows, cols16, lane);
      if constexpr (DUAL)
        store_rows_via_smem<2>(patch, pt, reinterpret_cast<uint16_t*>(static_cast<float*>(p.to) + goff),
                               2 * static_cast<size_t>(p.D), rows, cols16, lane);
    } else {
      constexpr int CH = D / 64;
      uint8_t* patch = sQ + warp * (32 * CH * 64);
      uint32_t po[CH][16], pt[CH][16];
#pragma unroll
      for (int cc = 0; cc < CH; ++cc) {
        const int c = wg * CH + cc;
        uint32_t ov[32], tv[32];
        if (it > 0) {
          tmem_ld_x32(tmem + lane_off + C::TMEM_O + c * 32, ov);
          if constexpr (DUAL) tmem_ld_x32(tmem + lane_off + C::TMEM_T + c * 32, tv);
          tmem_wait_ld();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) { ov[i] = 0u; tv[i] = 0u; }
        }
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const float o0 = __uint_as_float(ov[2 * i]) * linv, o1 = __uint_as_float(ov[2 * i + 1]) * linv;
          po[cc][i] = pack2<BF16>(o0, o1);
          if constexpr (DUAL) {
            const float t0 = __uint_as_float(tv[2 * i]) * linv - mul * o0;
            const float t1 = __uint_as_float(tv[2 * i + 1]) * linv - mul * o1;
            pt[cc][i] = pack2<BF16>(t0, t1);
          }
        }
      }
      const int col0 = wg * (D / 2);                                   // first column of this warpgroup
      const int wrow0 = q0 + (warp & 3) * 32;                          // first row of this warp
      const size_t goff = (static_cast<size_t>(row_base) + wrow0) * p.D + col0;
      const int rows = N - wrow0, cols = p.D - col0;
      store_rows_via_smem<CH>(patch, po, static_cast<uint16_t*>(p.o) + goff, p.D, rows, cols, lane);
      if constexpr (DUAL) store_rows_via_smem<CH>(patch, pt, static_cast<uint16_t*>(p.to) + goff, p.D, rows, cols, lane);
    }
    if (qi < N && wg == 0) {
      p.lse2[static_cast<size_t>(row_base) + qi] = (l > 0.f) ? m_used + log2f(l) : -INFINITY;
      p.mu[static_cast<size_t>(row_base) + qi] = mul;
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 9) tmem_dealloc(tmem, C::TMEM_COLS);
}

template <int D, bool DUAL, bool BF16, bool PAD, bool DROP = false>
int launch_one(const jvpfa_fwd_args& a, cudaStream_t stream) {
  using C = FwdCfg<D>;
  CUtensorMap mQ, mTQ, mK, mTK, mV, mTV;
  auto tile = [&](CUtensorMap* m, const void* ptr, const jvpfa_strides& st, int box_rows) {
    return make_tile_map(m, make_view(ptr, st, a.H, a.N, a.D), a.B, a.H, a.N, a.D, box_rows, a.dtype);
  };
  auto vmap = [&](CUtensorMap* m, const void* ptr, const jvpfa_strides& st) {
    return (!PAD && D > 64) ? make_slab_map(m, make_view(ptr, st, a.H, a.N, a.D), a.B, a.H, a.N, a.D, C::BN, a.dtype)
                            : tile(m, ptr, st, C::BN);
  };
  bool ok = tile(&mQ, a.q, a.q_strides, C::BM) && tile(&mK, a.k, a.k_strides, C::BN) && vmap(&mV, a.v, a.v_strides);
  if (DUAL) {
    ok = ok && tile(&mTQ, a.tq, a.tq_strides, C::BM) && tile(&mTK, a.tk, a.tk_strides, C::BN) && vmap(&mTV, a.tv, a.tv_strides);
  } else {
    mTQ = mQ; mTK = mK; mTV = mV;
  }
  if (!ok) return JVPFA_ERR_LAUNCH;
  FwdKParams p{};
  p.H = a.H; p.N = a.N; p.D = a.D; p.causal = a.causal;
  p.s = a.sm_scale;
  p.c1 = a.sm_scale * 1.4426950408889634f;
  p.thresh = BF16 ? 8.0f : 6.0f;
  p.mv = make_mask_view(a.mask, a.mask_summary, a.B, a.H, a.N);
  p.o = a.o; p.to = a.to; p.lse2 = a.lse2; p.mu = a.mu;
  p.status = static_cast<int*>(a.workspace);
  p.budget_ns = wait_budget_ns();
  p.drop = make_dropout_params(a.dropout_p, a.dropout_seed);
  auto kern = fwd_sm100_kernel<D, DUAL, BF16, PAD, false, DROP>;
  const size_t smem = C::smem_bytes();
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)) != cudaSuccess)
    return JVPFA_ERR_LAUNCH;
  p.n_qt = (a.N + C::BM - 1) / C::BM;
  p.n_units = a.B * a.H;
  p.unit_group = unit_group_size(p.n_units);
  dim3 grid(static_cast<unsigned>(p.n_qt) * static_cast<unsigned>(p.n_units));
  kern<<<grid, 384, smem, stream>>>(mQ, mTQ, mK, mTK, mV, mTV, p);
  return cudaGetLastError() == cudaSuccess ? JVPFA_OK : JVPFA_ERR_LAUNCH;
}

// fp32 inputs: split pre-pass into the workspace, then the 128-column kernel in its split mode on the split tensors.
template <bool DUAL, bool DROP>
int launch_split(const jvpfa_fwd_args& a, cudaStream_t stream) {
  using C = FwdCfg<128, true>;
  const int64_t rows = static_cast<int64_t>(a.B) * a.H * a.N;
  const int n_t = DUAL ? 6 : 3;
  const void* src[6] = {a.q, a.k, a.v, a.tq, a.tk, a.tv};
  uint16_t* dst[6];
  uint8_t* base = static_cast<uint8_t*>(a.workspace) + kStatusBytes;
  for (int i = 0; i < n_t; ++i) dst[i] = reinterpret_cast<uint16_t*>(base + static_cast<size_t>(i) * rows * kSplitRowBytes);
  const jvpfa_strides* sst[6] = {&a.q_strides, &a.k_strides, &a.v_strides, &a.tq_strides, &a.tk_strides, &a.tv_strides};
  TensorView views[6];
  for (int i = 0; i < n_t; ++i) views[i] = make_view(src[i], *sst[i], a.H, a.N, a.D);
  int rc = launch_split_fp32(views, dst, n_t, a.B, a.H, a.N, a.D, stream);
  if (rc != JVPFA_OK) return rc;
  CUtensorMap mQ, mTQ, mK, mTK, mV, mTV;
  const jvpfa_strides none{0, 0, 0};
  auto tile = [&](CUtensorMap* m, const void* ptr, int box_rows) {
    return make_tile_map(m, make_view(ptr, none, a.H, a.N, 128), a.B, a.H, a.N, 128, box_rows, JVPFA_BF16);
  };
  auto slab = [&](CUtensorMap* m, const void* ptr) {
    return make_slab_map(m, make_view(ptr, none, a.H, a.N, 128), a.B, a.H, a.N, 128, C::BN, JVPFA_BF16);
  };
  bool ok = tile(&mQ, dst[0], C::BM) && tile(&mK, dst[1], C::BN) && slab(&mV, dst[2]);
  if (DUAL) {
    ok = ok && tile(&mTQ, dst[3], C::BM) && tile(&mTK, dst[4], C::BN) && slab(&mTV, dst[5]);
  } else {
    mTQ = mQ; mTK = mK; mTV = mV;
  }
  if (!ok) return JVPFA_ERR_LAUNCH;
  FwdKParams p{};
  p.H = a.H; p.N = a.N; p.D = a.D; p.causal = a.causal;
  p.s = a.sm_scale;
  p.c1 = a.sm_scale * 1.4426950408889634f;
  p.thresh = 8.0f;
  p.mv = make_mask_view(a.mask, a.mask_summary, a.B, a.H, a.N);
  p.o = a.o; p.to = a.to; p.lse2 = a.lse2; p.mu = a.mu;
  p.status = static_cast<int*>(a.workspace);
  p.budget_ns = wait_budget_ns();
  p.drop = make_dropout_params(a.dropout_p, a.dropout_seed);
  auto kern = fwd_sm100_kernel<128, DUAL, true, false, true, DROP>;
  const size_t smem = C::smem_bytes();
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)) != cudaSuccess)
    return JVPFA_ERR_LAUNCH;
  p.n_qt = (a.N + C::BM - 1) / C::BM;
  p.n_units = a.B * a.H;
  p.unit_group = unit_group_size(p.n_units);
  dim3 grid(static_cast<unsigned>(p.n_qt) * static_cast<unsigned>(p.n_units));
  kern<<<grid, 384, smem, stream>>>(mQ, mTQ, mK, mTK, mV, mTV, p);
  return cudaGetLastError() == cudaSuccess ? JVPFA_OK : JVPFA_ERR_LAUNCH;
}

}  // namespace

bool sm100_split_path_supported(int dtype, int D, int N) {
  return dtype == JVPFA_F32 && D >= 8 && D <= 64 && (D % 8) == 0 && N >= 1;
}

size_t fwd_sm100_split_workspace_bytes(const jvpfa_fwd_args& a) {
  const size_t rows = static_cast<size_t>(a.B) * a.H * a.N;
  return kStatusBytes + (a.tq != nullptr ? 6 : 3) * rows * kSplitRowBytes;
}

int launch_fwd_sm100_split(const jvpfa_fwd_args& a, cudaStream_t stream) {
  if (a.dropout_p > 0.f) return a.tq != nullptr ? launch_split<true, true>(a, stream) : launch_split<false, true>(a, stream);
  return a.tq != nullptr ? launch_split<true, false>(a, stream) : launch_split<false, false>(a, stream);
}

bool sm100_path_supported(int dtype, int D, int N) {
  // head dimensions other than 64 / 128 run on the next wider kernel with zero-filled columns
  return (dtype == JVPFA_BF16 || dtype == JVPFA_F16) && D >= 8 && D <= 128 && (D % 8) == 0 && N >= 1;
}

namespace {
template <int D, bool PAD>
int launch_by_mode(const jvpfa_fwd_args& a, cudaStream_t stream) {
  const bool dual = a.tq != nullptr;
  const bool bf = a.dtype == JVPFA_BF16;
  if (a.dropout_p > 0.f) {
    if (dual) return bf ? launch_one<D, true, true, PAD, true>(a, stream) : launch_one<D, true, false, PAD, true>(a, stream);
    return bf ? launch_one<D, false, true, PAD, true>(a, stream) : launch_one<D, false, false, PAD, true>(a, stream);
  }
  if (dual) return bf ? launch_one<D, true, true, PAD>(a, stream) : launch_one<D, true, false, PAD>(a, stream);
  return bf ? launch_one<D, false, true, PAD>(a, stream) : launch_one<D, false, false, PAD>(a, stream);
}
}  // namespace

int launch_fwd_sm100(const jvpfa_fwd_args& a, cudaStream_t stream) {
  if (sm100_padded_dim(a.D) == 64) return a.D == 64 ? launch_by_mode<64, false>(a, stream) : launch_by_mode<64, true>(a, stream);
  return a.D == 128 ? launch_by_mode<128, false>(a, stream) : launch_by_mode<128, true>(a, stream);
}

}  // namespace jvpfa
