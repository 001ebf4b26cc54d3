// Blackwell (sm_100a) device primitives used by the tensor-core attention kernels:
// mbarrier with bounded waits, TMA tile loads, TMEM allocation, tcgen05 MMA / commit /
// TMEM load-store, and the shared-memory / instruction descriptor encodings.
//
// Every wait is bounded: a waiter that runs out of time records a code in a global status word
// and sets a CTA-wide "poisoned" flag, after which all further waits in that CTA give up after a
// few polls, so that the kernel always runs to its end and frees its TMEM.
#pragma once
#include <cstdint>
#include <cuda.h>
#include <cuda_runtime.h>

namespace jvpfa {
namespace sm100 {

// ---------------------------------------------------------------------------------------------
// addresses
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ uint64_t global_timer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

// ---------------------------------------------------------------------------------------------
// mbarrier
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_mbar_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("{\n\t.reg .b64 st;\n\tmbarrier.arrive.shared::cta.b64 st, [%0];\n\t}" ::"r"(smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("{\n\t.reg .b64 st;\n\tmbarrier.arrive.expect_tx.shared::cta.b64 st, [%0], %1;\n\t}" ::"r"(
                   smem_u32(bar)),
               "r"(bytes)
               : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}

// Status codes written to the global status word when a wait gives up.
enum : int { WAIT_OK = 0, WAIT_TIMEOUT_BASE = 100 };

struct WaitCtx {
  int* status;              // global status word (0 = fine)
  volatile int* poisoned;   // CTA-wide flag in shared memory
  uint64_t budget_ns;       // time a single wait may take before it gives up
};

// Waits for the phase with the given parity to complete. Returns false if it gave up.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, const WaitCtx& w, int site) {
  if (mbar_try_wait(bar, parity)) return true;
  const bool poisoned = (*w.poisoned != 0);
  uint64_t t0 = 0;
  uint32_t polls = 0;
  while (true) {
    if (mbar_try_wait(bar, parity)) return true;
    ++polls;
    if (poisoned) {
      if (polls > 64u) return false;
      continue;
    }
    if ((polls & 255u) == 0u) {
      const uint64_t now = global_timer_ns();
      if (t0 == 0) t0 = now;
      if (now - t0 > w.budget_ns || *w.poisoned != 0) {
        *w.poisoned = 1;
        atomicCAS(w.status, 0, WAIT_TIMEOUT_BASE + site);
        return false;
      }
    }
  }
}

// ---------------------------------------------------------------------------------------------
// TMA (tiled bulk tensor loads into this CTA's shared memory, completion on an mbarrier)
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* tmap) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(tmap)) : "memory");
}
// One 64-column slab of `box rows` rows of a (D, N, H, B) tensor map, starting at (column c, row n) of unit (h, b).
__device__ __forceinline__ void tma_load_tile(void* dst, const CUtensorMap* tmap, uint64_t* bar, int c, int n, int h,
                                              int b) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cta.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5}], [%6];" ::
          "r"(smem_u32(dst)),
      "l"(reinterpret_cast<uint64_t>(tmap)), "r"(c), "r"(n), "r"(h), "r"(b), "r"(smem_u32(bar))
      : "memory");
}
// All slabs of `box rows` rows of a (64, N, D / 64, H, B) tensor map, starting at row n of unit (h, b).
__device__ __forceinline__ void tma_load_slabs(void* dst, const CUtensorMap* tmap, uint64_t* bar, int n, int h, int b) {
  asm volatile(
      "cp.async.bulk.tensor.5d.shared::cta.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5, %6}], [%7];" ::
          "r"(smem_u32(dst)),
      "l"(reinterpret_cast<uint64_t>(tmap)), "r"(0), "r"(n), "r"(0), "r"(h), "r"(b), "r"(smem_u32(bar))
      : "memory");
}

// ---------------------------------------------------------------------------------------------
// TMEM allocation (warp-collective; one warp of the CTA owns alloc and dealloc)
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_dst, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_dst)),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}

__device__ __forceinline__ void tc_fence_before_sync() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after_sync() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// ---------------------------------------------------------------------------------------------
// descriptors
// ---------------------------------------------------------------------------------------------
// Shared-memory matrix descriptor (64 bit): start address, leading/stride byte offsets in 16-byte
// units, descriptor version 1 (bits 46-47), swizzle mode in bits 61-63 (2 = 128-byte swizzle).
__host__ __device__ __forceinline__ uint64_t make_smem_desc(uint32_t smem_addr, uint32_t lbo_bytes,
                                                            uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4);
  d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3FFFu) << 16;
  d |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3FFFu) << 32;
  d |= static_cast<uint64_t>(1) << 46;  // descriptor version for sm_100
  d |= static_cast<uint64_t>(2) << 61;  // 128-byte swizzle
  return d;
}

// A K-major operand tile whose rows are 128 bytes (64 two-byte elements) wide, rows packed at
// 128-byte pitch in 8-row swizzle atoms of 1024 bytes: stride offset = 1024, leading offset unused.
__device__ __forceinline__ uint64_t desc_kmajor_sw128(uint32_t smem_addr) {
  return make_smem_desc(smem_addr, 16, 1024);
}
// An MN-major operand (the MN index is contiguous in memory, 64 elements = 128 bytes per row of
// the K index): 8 K-rows form a 1024-byte atom (stride offset), the next group of 64 MN elements
// starts `mn_group_bytes` further on (leading offset).
__device__ __forceinline__ uint64_t desc_mnmajor_sw128(uint32_t smem_addr, uint32_t mn_group_bytes) {
  return make_smem_desc(smem_addr, mn_group_bytes, 1024);
}

enum : uint32_t { FMT_F16 = 0, FMT_BF16 = 1 };

// Instruction descriptor for kind::f16 with fp32 accumulation (both operands in the same 16-bit format: the hardware
// does not take an fp16 operand against a bf16 one).
__host__ __device__ __forceinline__ uint32_t make_idesc(uint32_t ab_fmt, uint32_t M, uint32_t N, uint32_t a_mn_major,
                                                        uint32_t b_mn_major) {
  uint32_t d = 0;
  d |= 1u << 4;                 // accumulator format: fp32
  d |= (ab_fmt & 7u) << 7;      // A format
  d |= (ab_fmt & 7u) << 10;     // B format
  d |= (a_mn_major & 1u) << 15;
  d |= (b_mn_major & 1u) << 16;
  d |= ((N >> 3) & 0x3Fu) << 17;
  d |= ((M >> 4) & 0x1Fu) << 24;
  return d;
}

// One lane of the (converged) warp. The lane that issues tcgen05.mma has to be chosen this way: with the
// predicate of elect.sync the compiler keeps descriptors and addresses in uniform registers and one thread issues an
// instruction every 10-12 cycles; behind `lane == 0` the same code needs 45-48 cycles per instruction (measured with
// N = 16 instructions that leave the tensor pipe idle), which is slower than the pipe executes N <= 64 shapes and
// leaves no slack for N = 128.
__device__ __forceinline__ bool elect_one_sync() {
  uint32_t pred;
  asm volatile(
      "{\n\t.reg .pred P;\n\t"
      "elect.sync _|P, 0xFFFFFFFF;\n\t"
      "selp.b32 %0, 1, 0, P;\n\t}"
      : "=r"(pred));
  return pred != 0;
}

// ---------------------------------------------------------------------------------------------
// MMA issue (one thread), commit to an mbarrier
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void umma_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                        uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                        uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}" ::"r"(d_tmem),
      "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Whole-warp forms: every lane executes the instruction, only the lane with `issue` != 0 performs it, so the code
// around a group of MMAs needs no branch.
__device__ __forceinline__ void umma_ss_pred(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                             uint32_t accumulate, uint32_t issue) {
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "setp.ne.b32 q, %5, 0;\n\t"
      "@q tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(issue)
      : "memory");
}
__device__ __forceinline__ void umma_ts_pred(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                             uint32_t accumulate, uint32_t issue) {
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "setp.ne.b32 q, %5, 0;\n\t"
      "@q tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}" ::"r"(d_tmem),
      "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(issue)
      : "memory");
}
// Arrives once on the barrier when all MMAs issued so far by this thread have completed.
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}

// ---------------------------------------------------------------------------------------------
// TMEM <-> registers, shape 32x32b: thread t of the warp touches lane (quadrant base + t),
// N consecutive 32-bit columns starting at the column in taddr.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void tmem_ld_x32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
      "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_x16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_st_x32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
      "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
      "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]),
      "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]),
      "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void tmem_st_x16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
      "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}

__device__ __forceinline__ void tmem_st_x8(uint32_t taddr, const uint32_t (&r)[8]) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"r"(taddr), "r"(r[0]),
               "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7])
               : "memory");
}
// Named barrier among a subset of the CTA's threads.
__device__ __forceinline__ void named_bar_sync(uint32_t id, uint32_t nthreads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}

// ---------------------------------------------------------------------------------------------
// Order of the CTAs of a launch. The hardware hands out blocks in increasing blockIdx.x, one whenever an SM has
// room, which is a dynamic longest-first schedule if heavy blocks come first. Under a causal mask the cost of a
// (row tile, batch*head unit) block depends on the row tile, so inside a group of `unit_group` units all units' heaviest
// tiles come first, then the next heaviest, and so on (a unit-by-unit order leaves a tail of heavy blocks of the last
// unit, which shows once a GPU holds only a few units); groups follow one another so that the key/value (or query-side)
// tensors the running blocks stream stay a working set of that many units in L2.
// ---------------------------------------------------------------------------------------------
struct BlockWork {
  int tile;   // row tile of the block
  int unit;   // batch * head unit
};
// `descending`: the heaviest row tile is the last one (queries under a causal mask), else the first.
__device__ __forceinline__ BlockWork block_work(int block, int n_tiles, int n_units, int unit_group, bool descending) {
  const int per_group = unit_group * n_tiles;
  const int g = block / per_group;
  const int rem = block - g * per_group;
  const int u0 = g * unit_group;
  const int gs = min(unit_group, n_units - u0);
  const int ti = rem / gs;
  BlockWork w;
  w.tile = descending ? n_tiles - 1 - ti : ti;
  w.unit = u0 + (rem - ti * gs);
  return w;
}

// ---------------------------------------------------------------------------------------------
// Epilogue stores. After a 32x32b TMEM load every lane of a warp holds one output row; written as they are, one
// 16-byte store instruction touches 32 different 128-byte lines and the kernel spends thousands of cycles in the
// store unit. The rows go through a per-warp shared-memory patch instead, so that each store instruction writes
// whole row segments: CH * 4 consecutive lanes cover one row's CH * 64 bytes.
//
//   patch   this warp's 32 x (CH * 64) bytes of shared memory (16-byte aligned)
//   packed  this lane's row: CH chunks of 32 sixteen-bit values, two per register
//   dst     address of the first of the warp's 32 rows at this warp's first column; rows `pitch` elements apart
//   rows    how many of the 32 rows exist (rows past the end of the sequence are not written)
//   cols    how many of the CH * 32 columns exist (a multiple of 8; columns past the head dimension are not written)
// ---------------------------------------------------------------------------------------------
template <int CH>
__device__ __forceinline__ void store_rows_via_smem(uint8_t* patch, const uint32_t (&packed)[CH][16], uint16_t* dst,
                                                    size_t pitch, int rows, int cols, int lane) {
  constexpr int ROWB = CH * 64;   // bytes per row in the patch
  constexpr int LPR = CH * 4;     // lanes (16-byte pieces) per row
  constexpr int RPP = 32 / LPR;   // rows per store instruction
  auto swz = [](int row) { return CH == 1 ? ((row >> 1) & 3) : (row & (LPR - 1)); };
  __syncwarp();
#pragma unroll
  for (int c = 0; c < CH; ++c)
#pragma unroll
    for (int v = 0; v < 4; ++v) {
      const int pc = c * 4 + v;
      *reinterpret_cast<uint4*>(patch + lane * ROWB + ((pc ^ swz(lane)) << 4)) =
          make_uint4(packed[c][4 * v], packed[c][4 * v + 1], packed[c][4 * v + 2], packed[c][4 * v + 3]);
    }
  __syncwarp();
  const int pc = lane % LPR;
#pragma unroll
  for (int i = 0; i < LPR; ++i) {
    const int row = i * RPP + lane / LPR;
    const uint4 val = *reinterpret_cast<const uint4*>(patch + row * ROWB + ((pc ^ swz(row)) << 4));
    if (row < rows && pc * 8 < cols) *reinterpret_cast<uint4*>(dst + row * pitch + pc * 8) = val;
  }
}

}  // namespace sm100
}  // namespace jvpfa
