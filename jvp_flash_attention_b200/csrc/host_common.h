// Host-side helpers shared by the launchers: TMA tensor-map encoding through the driver entry
// point (the library does not link libcuda), the device status word, small utilities.
#pragma once
#include <cstdint>
#include <cstdio>
#include <cuda.h>
#include <cuda_runtime.h>
#include "../../include/jvpfa.h"

namespace jvpfa {

typedef CUresult (*TensorMapEncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                      const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                      CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

TensorMapEncodeFn tensor_map_encoder();

// A (rows x D) row-major matrix of 16-bit elements, D a multiple of 8, as a 2-D tensor map with a box of
// (64 columns, box_rows rows): one TMA copy per 64-column slab lands in shared memory as [box_rows][64
// elements] in the 128-byte-swizzled layout the MMA descriptors expect; columns at or beyond D read as
// zero, which is how head dimensions that are not 64 or 128 ride on the 64- and 128-wide kernels.
// Returns false if the driver rejects the encoding.
bool make_tile_map(CUtensorMap* out, const void* base, uint64_t rows, int D, int box_rows, int dtype);

// The same matrix (D a multiple of 64) as a 3-D map (64, rows, D / 64): one box of (64, box_rows, D / 64) lands as
// D / 64 consecutive 128-byte-swizzled slabs of [box_rows][64]. One large box instead of one box per slab: the TMA
// unit of an SM delivers 43 B/clk in 32 KB boxes, 36 in 16 KB boxes and 29 in 8 KB boxes (measured).
bool make_slab_map(CUtensorMap* out, const void* base, uint64_t rows, int D, int box_rows, int dtype);

// Wait budget of a single device-side mbarrier wait, in nanoseconds (JVPFA_WAIT_BUDGET_MS, default 4000 ms).
uint64_t wait_budget_ns();

inline size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

// Workspace layout shared by forward and backward: [0,256) status word + padding, then per-call scratch.
constexpr size_t kStatusBytes = 256;

// Optional caller-owned events of jvpfa_bwd_marked: mark(i) records event i on the stream when events were given.
struct LaunchMarks {
  void* const* events = nullptr;
  cudaStream_t stream = nullptr;
  void mark(int i) const {
    if (events != nullptr) cudaEventRecord(static_cast<cudaEvent_t>(events[i]), stream);
  }
};

// fp32 inputs on the tensor cores (head dimension <= 64, a multiple of 8): every operand is split into bf16 hi + lo parts
// by a pre-pass into the workspace and every product runs as three bf16 products accumulated in fp32.
constexpr int kSplitMaxTensors = 8;
constexpr size_t kSplitRowBytes = 256;   // one split row: 64 hi + 64 lo bf16 numbers
int launch_split_fp32(const void* const* src, uint16_t* const* dst, int n_tensors, int64_t rows, int D, cudaStream_t stream);
bool sm100_split_path_supported(int dtype, int D, int N);
size_t fwd_sm100_split_workspace_bytes(const jvpfa_fwd_args& a);
size_t bwd_sm100_split_workspace_bytes(const jvpfa_bwd_args& a);
int launch_fwd_sm100_split(const jvpfa_fwd_args& a, cudaStream_t stream);
int launch_bwd_sm100_split(const jvpfa_bwd_args& a, cudaStream_t stream, const LaunchMarks& marks);

int launch_fwd_sm100(const jvpfa_fwd_args& a, cudaStream_t stream);
int launch_bwd_sm100(const jvpfa_bwd_args& a, cudaStream_t stream, const LaunchMarks& marks);
size_t bwd_sm100_workspace_bytes(const jvpfa_bwd_args& a);
bool sm100_path_supported(int dtype, int D, int N);
inline int sm100_padded_dim(int D) { return D <= 64 ? 64 : 128; }

int launch_fwd_generic(const jvpfa_fwd_args& a, cudaStream_t stream);
int launch_bwd_generic(const jvpfa_bwd_args& a, cudaStream_t stream, const LaunchMarks& marks);
size_t bwd_generic_workspace_bytes(const jvpfa_bwd_args& a);

}  // namespace jvpfa
