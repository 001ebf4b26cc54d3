// C ABI of libjvpfa.so: argument validation, kernel-family selection by shape, the mask-summary
// pre-pass, status read-back. See include/jvpfa.h for the contract of each entry point.
#include <cstdlib>
#include <cstring>
#include <mutex>
#include "host_common.h"
#include "mask_common.cuh"
#include "sm100_prims.cuh"

namespace jvpfa {

TensorMapEncodeFn tensor_map_encoder() {
  static TensorMapEncodeFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPointByVersion("cuTensorMapEncodeTiled", &p, 12000, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<TensorMapEncodeFn>(p);
  });
  return fn;
}

bool make_tile_map(CUtensorMap* out, const TensorView& v, int B, int H, int N, int D, int box_rows, int dtype) {
  TensorMapEncodeFn enc = tensor_map_encoder();
  if (enc == nullptr || v.ptr == nullptr) return false;
  const cuuint64_t dims[4] = {static_cast<cuuint64_t>(D), static_cast<cuuint64_t>(N), static_cast<cuuint64_t>(H),
                              static_cast<cuuint64_t>(B)};
  // a dimension of extent 1 may come with any stride (a broadcast view has 0): TMA wants a multiple of 16 bytes
  auto bytes = [](int64_t elems, cuuint64_t extent) { return extent == 1 ? cuuint64_t{16} : static_cast<cuuint64_t>(elems) * 2; };
  const cuuint64_t strides[3] = {bytes(v.sn, dims[1]), bytes(v.sh, dims[2]), bytes(v.sb, dims[3])};
  const cuuint32_t box[4] = {64, static_cast<cuuint32_t>(box_rows), 1, 1};
  const cuuint32_t estr[4] = {1, 1, 1, 1};
  const CUtensorMapDataType dt = dtype == JVPFA_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  return enc(out, dt, 4, const_cast<void*>(v.ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
             CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

bool make_slab_map(CUtensorMap* out, const TensorView& v, int B, int H, int N, int D, int box_rows, int dtype) {
  TensorMapEncodeFn enc = tensor_map_encoder();
  if (enc == nullptr || v.ptr == nullptr || D % 64 != 0) return false;
  const cuuint64_t dims[5] = {64, static_cast<cuuint64_t>(N), static_cast<cuuint64_t>(D / 64), static_cast<cuuint64_t>(H),
                              static_cast<cuuint64_t>(B)};
  auto bytes = [](int64_t elems, cuuint64_t extent) { return extent == 1 ? cuuint64_t{16} : static_cast<cuuint64_t>(elems) * 2; };
  const cuuint64_t strides[4] = {bytes(v.sn, dims[1]), 128, bytes(v.sh, dims[3]), bytes(v.sb, dims[4])};
  const cuuint32_t box[5] = {64, static_cast<cuuint32_t>(box_rows), static_cast<cuuint32_t>(D / 64), 1, 1};
  const cuuint32_t estr[5] = {1, 1, 1, 1, 1};
  const CUtensorMapDataType dt = dtype == JVPFA_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  return enc(out, dt, 5, const_cast<void*>(v.ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
             CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

int unit_group_size(int n_units) {
  // Measured on the causal headline shape: with 16 or 32 units on a GPU groups of 4, 8 and 16 units are 9-15 % faster
  // than unit-by-unit order and equal among themselves; with 128 units all group sizes are within noise of one another.
  // 4 keeps the working set that the running blocks stream (4 MB per unit at N = 4096, D = 128) far below the L2 size.
  return n_units < 4 ? (n_units < 1 ? 1 : n_units) : 4;
}

uint64_t wait_budget_ns() {
  static uint64_t ns = [] {
    const char* e = std::getenv("JVPFA_WAIT_BUDGET_MS");
    const long ms = e ? std::atol(e) : 4000;
    return static_cast<uint64_t>(ms > 0 ? ms : 4000) * 1000000ull;
  }();
  return ns;
}

namespace {

// Summary pre-pass. One CTA per (mask plane, band of 64 queries). The band is walked in chunks of 256 bytes per row
// (256 boolean entries, 128 16-bit or 64 fp32 ones): the chunk goes through shared memory (16-byte loads when the rows are
// contiguous and aligned, element-wise loads for any other layout), then thread t owns column t of the chunk and
// walks down its 64 queries. That gives, per chunk: the key-major 64-bit word of every column, the query-major 32-bit
// half-words of every row (one warp ballot per row), and the "anything kept" / "anything excluded or biased" flags of
// the 64x64 tiles the chunk touches. Entries outside the sequence count as not kept and set no flag. The bit words
// are written for boolean masks only.
constexpr int kSummaryRowBytes = 256;
__global__ void __launch_bounds__(256)
mask_summary_kernel(MaskView mv, int N, uint8_t* flags, uint32_t* rowbits, uint64_t* colbits, int vec_ok) {
  const int band = blockIdx.x;
  const int plane = blockIdx.y;
  const int bm = plane / mv.Hm, hm = plane % mv.Hm;
  extern __shared__ __align__(16) uint8_t sm[];
  uint8_t* tile = sm;                                                    // [64][256 bytes]
  uint32_t* tflags = reinterpret_cast<uint32_t*>(sm + 64 * kSummaryRowBytes);   // n64 words
  for (int i = threadIdx.x; i < mv.n64; i += blockDim.x) tflags[i] = 0;
  const int es = mv.kind == JVPFA_MASK_BOOL ? 1 : (mv.dtype == JVPFA_F32 ? 4 : 2);
  const int cc = kSummaryRowBytes / es;   // columns per chunk
  const int64_t plane_off = bm * mv.s0 + hm * mv.s1;
  const uint8_t* base = static_cast<const uint8_t*>(mv.ptr);
  const int t = threadIdx.x, lane = t & 31;
  const int q0 = band * 64;
  for (int k0 = 0; k0 < mv.n_pad; k0 += cc) {
    __syncthreads();   // the previous chunk has been consumed (and, the first time, the flags are cleared)
    // ---- load the chunk: rows q0 .. q0 + 63, columns k0 .. k0 + cc - 1, zero where outside the sequence
    if (vec_ok) {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int r = (t >> 4) + 16 * i, piece = t & 15;
        const int q = q0 + r, kf = k0 + piece * (16 / es);      // first column of this 16-byte piece
        uint4 v = make_uint4(0u, 0u, 0u, 0u);
        if (q < N && kf + 16 / es <= N) {
          v = *reinterpret_cast<const uint4*>(base + (plane_off + static_cast<int64_t>(q) * mv.s2 + kf) * es);
        } else if (q < N && kf < N) {                           // the piece straddles the end of the row
          uint8_t tmp[16] = {0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0};
          const uint8_t* src = base + (plane_off + static_cast<int64_t>(q) * mv.s2 + kf) * es;
          for (int j = 0; j < (N - kf) * es; ++j) tmp[j] = src[j];
          v = *reinterpret_cast<const uint4*>(tmp);
        }
        *reinterpret_cast<uint4*>(tile + r * kSummaryRowBytes + piece * 16) = v;
      }
    } else {
      for (int e = t; e < 64 * cc; e += 256) {
        const int r = e / cc, c = e - r * cc;
        const int q = q0 + r, k = k0 + c;
        const bool in = q < N && k < N;
        const int64_t idx = plane_off + static_cast<int64_t>(q) * mv.s2 + static_cast<int64_t>(k) * mv.s3;
        if (es == 1) tile[r * kSummaryRowBytes + c] = in ? base[idx] : 0;
        else if (es == 2) reinterpret_cast<uint16_t*>(tile)[r * (kSummaryRowBytes / 2) + c] = in ? reinterpret_cast<const uint16_t*>(base)[idx] : 0;
        else reinterpret_cast<uint32_t*>(tile)[r * (kSummaryRowBytes / 4) + c] = in ? reinterpret_cast<const uint32_t*>(base)[idx] : 0u;
      }
    }
    __syncthreads();
    // ---- thread t owns column k0 + t
    if (t < cc && k0 + t < mv.n_pad) {   // (whole warps: cc and n_pad are multiples of 32)
      const int k = k0 + t;
      uint64_t word = 0;
      bool any_masked = false;
      uint32_t mine0 = 0, mine1 = 0;   // ballots of rows lane and lane + 32
#pragma unroll 8
      for (int r = 0; r < 64; ++r) {
        const bool in = (q0 + r < N) && (k < N);
        bool kept, masked;
        if (mv.kind == JVPFA_MASK_BOOL) {
          kept = tile[r * kSummaryRowBytes + t] != 0;
          masked = !kept;
        } else {
          const float m = mask_elem_as_float(tile, r * cc + t, mv.dtype);
          kept = m != -INFINITY;
          masked = m != 0.f;
        }
        kept = kept && in;
        any_masked |= masked && in;
        word |= static_cast<uint64_t>(kept) << r;
        const uint32_t ballot = __ballot_sync(0xFFFFFFFFu, kept);
        if ((r & 31) == lane) { if (r < 32) mine0 = ballot; else mine1 = ballot; }
      }
      const int kt = k >> 6, half = (k >> 5) & 1;   // the same for the whole warp
      if (mv.kind == JVPFA_MASK_BOOL) {
        colbits[(static_cast<int64_t>(plane) * mv.n64 + band) * mv.n_pad + k] = word;
        uint32_t* rb = rowbits + ((static_cast<int64_t>(plane) * mv.n64 + kt) * mv.n_pad + q0) * 2 + half;
        rb[2 * lane] = mine0;
        rb[2 * (lane + 32)] = mine1;
      }
      const uint32_t fl = (__any_sync(0xFFFFFFFFu, word != 0) ? kTileAnyKept : 0u) | (__any_sync(0xFFFFFFFFu, any_masked) ? kTileAnyMasked : 0u);
      if (lane == 0 && fl) atomicOr(&tflags[kt], fl);
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < mv.n64; i += blockDim.x)
    flags[(static_cast<int64_t>(plane) * mv.n64 + band) * mv.n64 + i] = static_cast<uint8_t>(tflags[i]);
}

// The same for a boolean mask whose rows are contiguous and 16-byte aligned, without the detour through shared
// memory: a warp takes a key tile, its lanes the band's queries (two passes of 32), one half-tile of 32 keys after the
// other. A lane loads its query's 32 bytes, turns them into 32 bits (that is the query-major half-word), and 32 ballots
// transpose the warp's 32 x 32 bits into the key-major words. blockIdx.z of gridDim.z takes every gridDim.z-th key tile
// (more blocks in flight: the kernel lives on memory latency).
__global__ void __launch_bounds__(256)
mask_summary_bool_kernel(MaskView mv, int N, uint8_t* flags, uint32_t* rowbits, uint64_t* colbits) {
  const int band = blockIdx.x;
  const int plane = blockIdx.y;
  const int bm = plane / mv.Hm, hm = plane % mv.Hm;
  const uint8_t* base = static_cast<const uint8_t*>(mv.ptr) + bm * mv.s0 + hm * mv.s1;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int q0 = band * 64;
  // 4 bytes that are zero / non-zero -> 4 bits
  auto bits4 = [](uint32_t w) -> uint32_t { return (((__vcmpne4(w, 0u) & 0x01010101u) * 0x01020408u) >> 24) & 0xFu; };
  for (int kt = blockIdx.z + gridDim.z * warp; kt < mv.n64; kt += gridDim.z * 8) {
    // all four loads of the tile first (two half-tiles x two passes of queries), so that they are in flight together
    uint32_t w[2][2][8];
    uint32_t valid4[2][2];
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int k0 = kt * 64 + half * 32;
#pragma unroll
      for (int pass = 0; pass < 2; ++pass) {
        const int q = q0 + 32 * pass + lane;
        const uint32_t valid = (q < N && k0 < N) ? (N - k0 >= 32 ? 0xFFFFFFFFu : ((1u << (N - k0)) - 1u)) : 0u;
        valid4[half][pass] = valid;
#pragma unroll
        for (int i = 0; i < 8; ++i) w[half][pass][i] = 0;
        if (valid) {
          const uint8_t* src = base + static_cast<int64_t>(q) * mv.s2 + k0;
          if (valid == 0xFFFFFFFFu) {
            const uint4 a = *reinterpret_cast<const uint4*>(src), c = *reinterpret_cast<const uint4*>(src + 16);
            w[half][pass][0] = a.x; w[half][pass][1] = a.y; w[half][pass][2] = a.z; w[half][pass][3] = a.w;
            w[half][pass][4] = c.x; w[half][pass][5] = c.y; w[half][pass][6] = c.z; w[half][pass][7] = c.w;
          } else {
#pragma unroll
            for (int i = 0; i < 8; ++i)
              for (int j = 0; j < 4; ++j)
                if (k0 + 4 * i + j < N) w[half][pass][i] |= static_cast<uint32_t>(src[4 * i + j]) << (8 * j);
          }
        }
      }
    }
    uint32_t kept_any = 0, masked_any = 0;
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int k0 = kt * 64 + half * 32;
      uint32_t col_lo = 0, col_hi = 0;   // lane c: the key-major word of key k0 + c
#pragma unroll
      for (int pass = 0; pass < 2; ++pass) {
        const int q = q0 + 32 * pass + lane;
        const uint32_t valid = valid4[half][pass];
        uint32_t bits = 0;
#pragma unroll
        for (int i = 0; i < 8; ++i) bits |= bits4(w[half][pass][i]) << (4 * i);
        bits &= valid;
        rowbits[((static_cast<int64_t>(plane) * mv.n64 + kt) * mv.n_pad + q) * 2 + half] = bits;
        kept_any |= bits;
        masked_any |= ~bits & valid;
#pragma unroll
        for (int c = 0; c < 32; ++c) {
          const uint32_t ballot = __ballot_sync(0xFFFFFFFFu, ((bits >> c) & 1u) != 0u);
          if (c == lane) { if (pass == 0) col_lo = ballot; else col_hi = ballot; }
        }
      }
      colbits[(static_cast<int64_t>(plane) * mv.n64 + band) * mv.n_pad + k0 + lane] = (static_cast<uint64_t>(col_hi) << 32) | col_lo;
    }
    const bool any_kept = __any_sync(0xFFFFFFFFu, kept_any != 0u);
    const bool any_masked = __any_sync(0xFFFFFFFFu, masked_any != 0u);
    if (lane == 0)
      flags[(static_cast<int64_t>(plane) * mv.n64 + band) * mv.n64 + kt] =
          static_cast<uint8_t>((any_kept ? kTileAnyKept : 0) | (any_masked ? kTileAnyMasked : 0));
  }
}

// Additive mask whose rows are contiguous and 16-byte aligned, same scheme as the boolean kernel: a warp takes a key
// tile, its lanes the band's queries. Bit = the entry is +-0. Per 64x64 tile: "kept" (anything but -inf), "needs the mask"
// (anything but +-0), and "two-valued": all entries that are not +-0 carry the same bit pattern, which goes into the tile
// values as a float. ES = bytes per element.
template <int ES>
__global__ void __launch_bounds__(256)
mask_summary_additive_kernel(MaskView mv, int N, uint8_t* flags, uint32_t* rowbits, uint64_t* colbits, float* tilevals) {
  const int band = blockIdx.x;
  const int plane = blockIdx.y;
  const int bm = plane / mv.Hm, hm = plane % mv.Hm;
  const uint8_t* base = static_cast<const uint8_t*>(mv.ptr) + (bm * mv.s0 + hm * mv.s1) * ES;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int q0 = band * 64;
  constexpr int WORDS = 32 * ES / 4;   // 32-bit words of a query's 32 entries
  const uint32_t ninf = ES == 4 ? 0xFF800000u : (mv.dtype == JVPFA_BF16 ? 0xFF80u : 0xFC00u);
  const uint32_t absmask = ES == 4 ? 0x7FFFFFFFu : 0x7FFFu;
  for (int kt = blockIdx.z + gridDim.z * warp; kt < mv.n64; kt += gridDim.z * 8) {
    bool kept_any = false, masked_any = false, has = false, multi = false;
    uint32_t val = 0;
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int k0 = kt * 64 + half * 32;
      uint32_t w[2][WORDS];
      int cnt[2];   // entries of this lane's run that lie inside the sequence
#pragma unroll
      for (int pass = 0; pass < 2; ++pass) {
        const int q = q0 + 32 * pass + lane;
        cnt[pass] = (q < N && k0 < N) ? min(32, N - k0) : 0;
#pragma unroll
        for (int i = 0; i < WORDS; ++i) w[pass][i] = 0;
        const uint8_t* src = base + (static_cast<int64_t>(q) * mv.s2 + k0) * ES;
        if (cnt[pass] == 32) {
#pragma unroll
          for (int i = 0; i < WORDS / 4; ++i) {
            const uint4 v = *reinterpret_cast<const uint4*>(src + 16 * i);
            w[pass][4 * i] = v.x; w[pass][4 * i + 1] = v.y; w[pass][4 * i + 2] = v.z; w[pass][4 * i + 3] = v.w;
          }
        } else if (cnt[pass] > 0) {
#pragma unroll
          for (int i = 0; i < WORDS; ++i)
            for (int j = 0; j < 4; ++j)
              if (4 * i + j < cnt[pass] * ES) w[pass][i] |= static_cast<uint32_t>(src[4 * i + j]) << (8 * j);
        }
      }
      uint32_t col_lo = 0, col_hi = 0;
#pragma unroll
      for (int pass = 0; pass < 2; ++pass) {
        const int q = q0 + 32 * pass + lane;
        uint32_t bits = 0;
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const uint32_t e = ES == 4 ? w[pass][i] : ((w[pass][i >> 1] >> (16 * (i & 1))) & 0xFFFFu);
          const bool in = i < cnt[pass];
          const bool zero = (e & absmask) == 0u;
          bits |= (in && zero ? 1u : 0u) << i;
          kept_any |= in && e != ninf;
          const bool nz = in && !zero;
          masked_any |= nz;
          multi |= nz && has && e != val;
          val = (nz && !has) ? e : val;
          has |= nz;
        }
        rowbits[((static_cast<int64_t>(plane) * mv.n64 + kt) * mv.n_pad + q) * 2 + half] = bits;
#pragma unroll
        for (int c = 0; c < 32; ++c) {
          const uint32_t ballot = __ballot_sync(0xFFFFFFFFu, ((bits >> c) & 1u) != 0u);
          if (c == lane) { if (pass == 0) col_lo = ballot; else col_hi = ballot; }
        }
      }
      colbits[(static_cast<int64_t>(plane) * mv.n64 + band) * mv.n_pad + k0 + lane] = (static_cast<uint64_t>(col_hi) << 32) | col_lo;
    }
    const bool any_kept = __any_sync(0xFFFFFFFFu, kept_any);
    const bool any_masked = __any_sync(0xFFFFFFFFu, masked_any);
    const bool any_multi = __any_sync(0xFFFFFFFFu, multi);
    const uint32_t has_b = __ballot_sync(0xFFFFFFFFu, has);
    const uint32_t v0 = __shfl_sync(0xFFFFFFFFu, val, has_b ? __ffs(has_b) - 1 : 0);
    const bool same = __all_sync(0xFFFFFFFFu, !has || val == v0);
    if (lane == 0) {
      const bool two = !any_multi && same;
      const int64_t t = (static_cast<int64_t>(plane) * mv.n64 + band) * mv.n64 + kt;
      flags[t] = static_cast<uint8_t>((any_kept ? kTileAnyKept : 0) | (any_masked ? kTileAnyMasked : 0) | (two ? kTileTwoValued : 0));
      float c = 0.f;
      if (has_b) {
        if (ES == 4) c = __uint_as_float(v0);
        else if (mv.dtype == JVPFA_BF16) c = __uint_as_float(v0 << 16);
        else c = __half2float(__ushort_as_half(static_cast<unsigned short>(v0)));
      }
      tilevals[t] = c;
    }
  }
}

// Self-test of the failure-detection path: one thread waits on an mbarrier that nothing ever arrives on. The wait
// runs out of its budget, records WAIT_TIMEOUT_BASE + 77 in the status word and marks the CTA as poisoned; a second
// wait then gives up after a few polls. The kernel returns normally. out: [0], [1] = results of the two waits
// (0 = gave up), [2], [3] = their durations in microseconds.
__global__ void selftest_timeout_kernel(int* status, uint64_t budget_ns, int* out) {
  __shared__ uint64_t bar;
  __shared__ int poisoned;
  if (threadIdx.x == 0) {
    poisoned = 0;
    sm100::mbar_init(&bar, 1);
    sm100::fence_mbar_init();
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    const sm100::WaitCtx w{status, &poisoned, budget_ns};
    const uint64_t t0 = sm100::global_timer_ns();
    const bool first = sm100::mbar_wait(&bar, 0, w, 77);
    const uint64_t t1 = sm100::global_timer_ns();
    const bool second = sm100::mbar_wait(&bar, 0, w, 78);
    const uint64_t t2 = sm100::global_timer_ns();
    out[0] = first ? 1 : 0;
    out[1] = second ? 1 : 0;
    out[2] = static_cast<int>((t1 - t0) / 1000);
    out[3] = static_cast<int>((t2 - t1) / 1000);
  }
}

// Average SM clock over a stretch of time: one thread reads the SM's cycle counter and the global nanosecond timer,
// sleeps until `duration_ns` have passed (bounded: at most one second), and reads both again. Launched on a stream of
// its own it sits beside whatever else runs on that SM and reports the clock that work actually got.
__global__ void sm_clock_probe_kernel(uint64_t duration_ns, float* mhz_out) {
  if (threadIdx.x != 0) return;
  const uint64_t t0 = sm100::global_timer_ns();
  const long long c0 = clock64();
  uint64_t t1 = t0;
  for (int i = 0; i < 2000000 && t1 - t0 < duration_ns; ++i) {
    __nanosleep(1000);
    t1 = sm100::global_timer_ns();
  }
  const long long c1 = clock64();
  *mhz_out = t1 > t0 ? static_cast<float>(static_cast<double>(c1 - c0) * 1e3 / static_cast<double>(t1 - t0)) : 0.f;
}

int check_common(int B, int H, int N, int D, int dtype, int causal, const jvpfa_mask& mask, const void* ws, size_t ws_bytes,
                 size_t ws_need) {
  if (B <= 0 || H <= 0 || N <= 0 || D <= 0) return JVPFA_ERR_BAD_ARG;
  if (dtype != JVPFA_F16 && dtype != JVPFA_BF16 && dtype != JVPFA_F32) return JVPFA_ERR_UNSUPPORTED;
  if (causal && mask.kind != JVPFA_MASK_NONE) return JVPFA_ERR_CAUSAL_MASK;
  if (mask.kind != JVPFA_MASK_NONE) {
    if (mask.ptr == nullptr) return JVPFA_ERR_BAD_ARG;
    if (mask.kind != JVPFA_MASK_BOOL && mask.kind != JVPFA_MASK_ADDITIVE) return JVPFA_ERR_BAD_ARG;
    if (mask.kind == JVPFA_MASK_ADDITIVE && mask.dtype != JVPFA_F16 && mask.dtype != JVPFA_BF16 && mask.dtype != JVPFA_F32)
      return JVPFA_ERR_UNSUPPORTED;
  }
  if (ws == nullptr || ws_bytes < ws_need) return JVPFA_ERR_WORKSPACE;
  if (static_cast<uint64_t>(B) * H * N >= (1ull << 31)) return JVPFA_ERR_UNSUPPORTED;
  return JVPFA_OK;
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

// Input layouts: the tensor-core paths read strided views in place when TMA (16-bit inputs) or the split pre-pass
// (fp32 inputs) can address them; the CUDA-core kernels take contiguous tensors only.
int check_layouts(const void* const* ptrs, const jvpfa_strides* const* strides, int n, int B, int H, int N, int D, int dtype) {
  const bool tensor_cores = sm100_path_supported(dtype, D, N) || sm100_split_path_supported(dtype, D, N);
  const int elem = dtype == JVPFA_F32 ? 4 : 2;
  for (int i = 0; i < n; ++i) {
    if (ptrs[i] == nullptr || is_contiguous(*strides[i], H, N, D)) continue;
    if (!tensor_cores) return JVPFA_ERR_UNSUPPORTED;
    const TensorView v = make_view(ptrs[i], *strides[i], H, N, D);
    const bool ok = (v.sb * elem) % 16 == 0 && (v.sh * elem) % 16 == 0 && (v.sn * elem) % 16 == 0 && v.sn > 0 &&
                    (v.sh > 0 || H == 1) && (v.sb > 0 || B == 1);
    if (!ok) return JVPFA_ERR_UNSUPPORTED;
  }
  return JVPFA_OK;
}

}  // namespace
}  // namespace jvpfa

using namespace jvpfa;

extern "C" {

int jvpfa_version(void) { return 200; }

const char* jvpfa_error_string(int status) {
  switch (status) {
    case JVPFA_OK: return "ok";
    case JVPFA_ERR_BAD_ARG: return "bad argument (null pointer, non-positive size or misaligned pointer)";
    case JVPFA_ERR_UNSUPPORTED: return "unsupported shape or dtype";
    case JVPFA_ERR_CAUSAL_MASK: return "causal attention does not support an attention mask";
    case JVPFA_ERR_WORKSPACE: return "workspace missing or too small";
    case JVPFA_ERR_LAUNCH: return "CUDA launch or tensor-map encoding failed";
    case JVPFA_ERR_DEVICE_TIMEOUT: return "a bounded device-side wait gave up";
    case JVPFA_ERR_NO_ALLOC_LIMIT: return "problem exceeds the fixed scratch of the allocation-free entry point";
    default: return "unknown status";
  }
}

size_t jvpfa_fwd_workspace_bytes(const jvpfa_fwd_args* a) {
  if (a != nullptr && sm100_split_path_supported(a->dtype, a->D, a->N)) return fwd_sm100_split_workspace_bytes(*a);
  return kStatusBytes;
}

size_t jvpfa_bwd_workspace_bytes(const jvpfa_bwd_args* a) {
  if (a == nullptr) return kStatusBytes;
  if (sm100_path_supported(a->dtype, a->D, a->N)) return bwd_sm100_workspace_bytes(*a);
  if (sm100_split_path_supported(a->dtype, a->D, a->N)) return bwd_sm100_split_workspace_bytes(*a);
  return bwd_generic_workspace_bytes(*a);
}

size_t jvpfa_mask_summary_bytes(int32_t Bm, int32_t Hm, int32_t N) {
  const size_t n64 = (static_cast<size_t>(N) + 63) / 64;
  const size_t planes = static_cast<size_t>(Bm) * Hm;
  return mask_tile_flag_bytes(planes, n64) + 2 * mask_bit_bytes(planes, n64) + mask_tile_value_bytes(planes, n64);
}

int jvpfa_mask_summary(const jvpfa_mask* mask, int32_t B, int32_t H, int32_t N, uint8_t* summary, void* stream) {
  if (mask == nullptr || summary == nullptr || mask->ptr == nullptr || B <= 0 || H <= 0 || N <= 0) return JVPFA_ERR_BAD_ARG;
  if (mask->kind != JVPFA_MASK_BOOL && mask->kind != JVPFA_MASK_ADDITIVE) return JVPFA_ERR_BAD_ARG;
  if ((reinterpret_cast<uintptr_t>(summary) & 15) != 0) return JVPFA_ERR_BAD_ARG;
  const MaskView mv = make_mask_view(*mask, nullptr, B, H, N);
  const int Bm = mask->stride[0] == 0 ? 1 : B;
  const size_t planes = static_cast<size_t>(Bm) * mv.Hm;
  uint8_t* bits = summary + mask_tile_flag_bytes(planes, mv.n64);
  // 16-byte loads need rows that are contiguous, and every row start on a 16-byte boundary
  const int es = mask->kind == JVPFA_MASK_BOOL ? 1 : (mask->dtype == JVPFA_F32 ? 4 : 2);
  auto mult16 = [&](int64_t stride) { return (stride * es) % 16 == 0; };
  const int vec_ok = mv.s3 == 1 && (reinterpret_cast<uintptr_t>(mask->ptr) & 15) == 0 && mult16(mv.s2) &&
                     (mv.s0 == 0 || mult16(mv.s0)) && (mv.s1 == 0 || mult16(mv.s1));
  dim3 grid(mv.n64, static_cast<unsigned>(planes));
  if (vec_ok && mask->kind == JVPFA_MASK_BOOL) {
    grid.z = mv.n64 >= 16 ? 4 : (mv.n64 >= 4 ? 2 : 1);
    mask_summary_bool_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        mv, N, summary, reinterpret_cast<uint32_t*>(bits), reinterpret_cast<uint64_t*>(bits + mask_bit_bytes(planes, mv.n64)));
    return cudaGetLastError() == cudaSuccess ? JVPFA_OK : JVPFA_ERR_LAUNCH;
  }
  if (vec_ok && mask->kind == JVPFA_MASK_ADDITIVE) {
    grid.z = mv.n64 >= 16 ? 4 : (mv.n64 >= 4 ? 2 : 1);
    uint32_t* rb = reinterpret_cast<uint32_t*>(bits);
    uint64_t* cb = reinterpret_cast<uint64_t*>(bits + mask_bit_bytes(planes, mv.n64));
    float* tv = reinterpret_cast<float*>(bits + 2 * mask_bit_bytes(planes, mv.n64));
    if (es == 4) mask_summary_additive_kernel<4><<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(mv, N, summary, rb, cb, tv);
    else mask_summary_additive_kernel<2><<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(mv, N, summary, rb, cb, tv);
    return cudaGetLastError() == cudaSuccess ? JVPFA_OK : JVPFA_ERR_LAUNCH;
  }
  const size_t smem = 64 * kSummaryRowBytes + mv.n64 * sizeof(uint32_t);
  mask_summary_kernel<<<grid, 256, smem, static_cast<cudaStream_t>(stream)>>>(
      mv, N, summary, reinterpret_cast<uint32_t*>(bits), reinterpret_cast<uint64_t*>(bits + mask_bit_bytes(planes, mv.n64)), vec_ok);
  return cudaGetLastError() == cudaSuccess ? JVPFA_OK : JVPFA_ERR_LAUNCH;
}

int jvpfa_fwd(const jvpfa_fwd_args* a, void* stream) {
  if (a == nullptr) return JVPFA_ERR_BAD_ARG;
  int rc = check_common(a->B, a->H, a->N, a->D, a->dtype, a->causal, a->mask, a->workspace, a->workspace_bytes, kStatusBytes);
  if (rc != JVPFA_OK) return rc;
  if (!a->q || !a->k || !a->v || !a->o || !a->lse2 || !a->mu) return JVPFA_ERR_BAD_ARG;
  const bool dual = a->tq != nullptr;
  if (dual && (!a->tk || !a->tv || !a->to)) return JVPFA_ERR_BAD_ARG;
  if (!dual && (a->tk || a->tv)) return JVPFA_ERR_BAD_ARG;
  if (!aligned16(a->q) || !aligned16(a->k) || !aligned16(a->v) || !aligned16(a->o) ||
      (dual && (!aligned16(a->tq) || !aligned16(a->tk) || !aligned16(a->tv) || !aligned16(a->to))))
    return JVPFA_ERR_BAD_ARG;
  {
    const void* ptrs[6] = {a->q, a->k, a->v, a->tq, a->tk, a->tv};
    const jvpfa_strides* st[6] = {&a->q_strides, &a->k_strides, &a->v_strides, &a->tq_strides, &a->tk_strides, &a->tv_strides};
    rc = check_layouts(ptrs, st, dual ? 6 : 3, a->B, a->H, a->N, a->D, a->dtype);
    if (rc != JVPFA_OK) return rc;
  }
  if (!(a->dropout_p >= 0.f && a->dropout_p < 1.f)) return JVPFA_ERR_BAD_ARG;
  // dropout exists in the tensor-core kernels only
  if (a->dropout_p > 0.f && !sm100_path_supported(a->dtype, a->D, a->N) &&
      !(sm100_split_path_supported(a->dtype, a->D, a->N) && a->workspace_bytes >= fwd_sm100_split_workspace_bytes(*a)))
    return JVPFA_ERR_UNSUPPORTED;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (sm100_path_supported(a->dtype, a->D, a->N)) return launch_fwd_sm100(*a, s);
  // fp32: the tensor-core path when the workspace has room for the split operands, else the CUDA-core kernels
  if (sm100_split_path_supported(a->dtype, a->D, a->N) && a->workspace_bytes >= fwd_sm100_split_workspace_bytes(*a))
    return launch_fwd_sm100_split(*a, s);
  {
    const jvpfa_strides* st[6] = {&a->q_strides, &a->k_strides, &a->v_strides, &a->tq_strides, &a->tk_strides, &a->tv_strides};
    for (int i = 0; i < (dual ? 6 : 3); ++i)
      if (!is_contiguous(*st[i], a->H, a->N, a->D)) return JVPFA_ERR_UNSUPPORTED;
  }
  return launch_fwd_generic(*a, s);
}

namespace {
int bwd_checked(const jvpfa_bwd_args* a, void* stream, void* const* events) {
  if (a == nullptr) return JVPFA_ERR_BAD_ARG;
  // smallest workspace any path takes: the status block and one float4 of statistics per row
  int rc = check_common(a->B, a->H, a->N, a->D, a->dtype, a->causal, a->mask, a->workspace, a->workspace_bytes,
                        sm100_path_supported(a->dtype, a->D, a->N) ? bwd_sm100_workspace_bytes(*a) : bwd_generic_workspace_bytes(*a));
  if (rc != JVPFA_OK) return rc;
  if (!a->q || !a->k || !a->v || !a->o || !a->lse2 || !a->mu || !a->go || !a->dq || !a->dk || !a->dv) return JVPFA_ERR_BAD_ARG;
  const bool dual = a->tq != nullptr;   // tq == NULL: primal-only backward, the tangent-side pointers are ignored
  if (dual && (!a->tk || !a->tv || !a->to || !a->gto || !a->dtq || !a->dtk || !a->dtv)) return JVPFA_ERR_BAD_ARG;
  const void* ptrs[] = {a->q, a->k, a->v, a->o, a->go, a->dq, a->dk, a->dv};
  for (const void* p : ptrs)
    if (!aligned16(p)) return JVPFA_ERR_BAD_ARG;
  if (dual) {
    const void* tptrs[] = {a->tq, a->tk, a->tv, a->to, a->gto, a->dtq, a->dtk, a->dtv};
    for (const void* p : tptrs)
      if (!aligned16(p)) return JVPFA_ERR_BAD_ARG;
  }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  // Primal-only call: the tangent-side pointers are documented as ignored, so the kernels never see them (the
  // preprocess kernels decide by gto whether the tangent terms enter Delta).
  jvpfa_bwd_args eff = *a;
  if (!dual) {
    eff.tk = eff.tv = eff.to = eff.gto = nullptr;
    eff.dtq = eff.dtk = eff.dtv = nullptr;
  }
  {
    const void* ptrs[8] = {eff.q, eff.k, eff.v, eff.go, eff.tq, eff.tk, eff.tv, eff.gto};
    const jvpfa_strides* st[8] = {&eff.q_strides, &eff.k_strides, &eff.v_strides, &eff.go_strides,
                                  &eff.tq_strides, &eff.tk_strides, &eff.tv_strides, &eff.gto_strides};
    rc = check_layouts(ptrs, st, dual ? 8 : 4, eff.B, eff.H, eff.N, eff.D, eff.dtype);
    if (rc != JVPFA_OK) return rc;
  }
  if (!(eff.dropout_p >= 0.f && eff.dropout_p < 1.f)) return JVPFA_ERR_BAD_ARG;
  // dropout exists in the tensor-core kernels only
  if (eff.dropout_p > 0.f && !sm100_path_supported(eff.dtype, eff.D, eff.N) &&
      !(sm100_split_path_supported(eff.dtype, eff.D, eff.N) && eff.workspace_bytes >= bwd_sm100_split_workspace_bytes(eff)))
    return JVPFA_ERR_UNSUPPORTED;
  LaunchMarks marks;
  marks.events = events;
  marks.stream = s;
  if (sm100_path_supported(eff.dtype, eff.D, eff.N)) return launch_bwd_sm100(eff, s, marks);
  // fp32: the tensor-core path when the workspace has room for the split operands, else the CUDA-core kernels
  if (sm100_split_path_supported(eff.dtype, eff.D, eff.N) && eff.workspace_bytes >= bwd_sm100_split_workspace_bytes(eff))
    return launch_bwd_sm100_split(eff, s, marks);
  {
    const jvpfa_strides* st[8] = {&eff.q_strides, &eff.k_strides, &eff.v_strides, &eff.go_strides,
                                  &eff.tq_strides, &eff.tk_strides, &eff.tv_strides, &eff.gto_strides};
    for (int i = 0; i < (dual ? 8 : 4); ++i)
      if (!is_contiguous(*st[i], eff.H, eff.N, eff.D)) return JVPFA_ERR_UNSUPPORTED;
  }
  return launch_bwd_generic(eff, s, marks);
}
}  // namespace

int jvpfa_bwd(const jvpfa_bwd_args* a, void* stream) { return bwd_checked(a, stream, nullptr); }

int jvpfa_bwd_marked(const jvpfa_bwd_args* a, void* stream, void* const* events, int32_t n_events) {
  if (events == nullptr || n_events != 5) return JVPFA_ERR_BAD_ARG;
  for (int i = 0; i < 5; ++i)
    if (events[i] == nullptr) return JVPFA_ERR_BAD_ARG;
  return bwd_checked(a, stream, events);
}

int jvpfa_sm_clock_probe(float* mhz_out, int32_t duration_us, void* stream) {
  if (mhz_out == nullptr || duration_us <= 0 || duration_us > 1000000) return JVPFA_ERR_BAD_ARG;
  sm_clock_probe_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<uint64_t>(duration_us) * 1000ull, mhz_out);
  return cudaGetLastError() == cudaSuccess ? JVPFA_OK : JVPFA_ERR_LAUNCH;
}

int jvpfa_selftest_timeout(void* workspace, int32_t budget_us, int32_t* out4, void* stream) {
  if (workspace == nullptr || out4 == nullptr || budget_us <= 0 || budget_us > 1000000) return JVPFA_ERR_BAD_ARG;
  selftest_timeout_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<int*>(workspace), static_cast<uint64_t>(budget_us) * 1000ull, out4);
  return cudaGetLastError() == cudaSuccess ? JVPFA_OK : JVPFA_ERR_LAUNCH;
}

int jvpfa_read_status(void* workspace, void* stream, int32_t* detail) {
  if (workspace == nullptr) return JVPFA_ERR_BAD_ARG;
  int32_t word = 0;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (cudaMemcpyAsync(&word, workspace, 4, cudaMemcpyDeviceToHost, s) != cudaSuccess) return JVPFA_ERR_LAUNCH;
  if (cudaStreamSynchronize(s) != cudaSuccess) return JVPFA_ERR_LAUNCH;
  if (detail) *detail = word;
  if (word != 0) {
    cudaMemsetAsync(workspace, 0, 4, s);
    return JVPFA_ERR_DEVICE_TIMEOUT;
  }
  return JVPFA_OK;
}

}  // extern "C"
