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

// A (B,H,N,D) input of 16-bit elements given by element strides along B, H, N (D contiguous).
struct TensorView {
  const void* ptr;
  int64_t sb, sh, sn;
};
// The view of a tensor with the ABI's strides; all-zero strides mean the contiguous layout.
inline TensorView make_view(const void* ptr, const jvpfa_strides& st, int H, int N, int D) {
  if (st.b == 0 && st.h == 0 && st.n == 0) return TensorView{ptr, static_cast<int64_t>(H) * N * D, static_cast<int64_t>(N) * D, D};
  return TensorView{ptr, st.b, st.h, st.n};
}
inline bool is_contiguous(const jvpfa_strides& st, int H, int N, int D) {
  return (st.b == 0 && st.h == 0 && st.n == 0) ||
         (st.n == D && st.h == static_cast<int64_t>(N) * D && st.b == static_cast<int64_t>(H) * N * D);
}
// TMA can read the view in place: base and every stride a multiple of 16 bytes.
inline bool view_tma_compatible(const TensorView& v, int elem_bytes) {
  return (reinterpret_cast<uintptr_t>(v.ptr) & 15) == 0 && (v.sb * elem_bytes) % 16 == 0 && (v.sh * elem_bytes) % 16 == 0 &&
         (v.sn * elem_bytes) % 16 == 0 && v.sb >= 0 && v.sh >= 0 && v.sn > 0;
}

// The view as a 4-D tensor map (D, N, H, B) with a box of (64 columns, box_rows rows, 1, 1): one TMA copy per
// 64-column slab lands in shared memory as [box_rows][64 elements] in the 128-byte-swizzled layout the MMA descriptors
// expect; columns at or beyond D and rows at or beyond N read as zero, which is how head dimensions that are not 64 or
// 128 ride on the 64- and 128-wide kernels and how ragged sequence lengths stay inside their (batch, head) unit.
// Returns false if the driver rejects the encoding.
bool make_tile_map(CUtensorMap* out, const TensorView& v, int B, int H, int N, int D, int box_rows, int dtype);

// The same view (D a multiple of 64) as a 5-D map (64, N, D / 64, H, B): one box of (64, box_rows, D / 64, 1, 1) lands as
// D / 64 consecutive 128-byte-swizzled slabs of [box_rows][64]. One large box instead of one box per slab: the TMA
// unit of an SM delivers 43 B/clk in 32 KB boxes, 36 in 16 KB boxes and 29 in 8 KB boxes (measured).
bool make_slab_map(CUtensorMap* out, const TensorView& v, int B, int H, int N, int D, int box_rows, int dtype);

// Units per group of the block order (see block_work in sm100_prims.cuh).
int unit_group_size(int n_units);

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
int launch_split_fp32(const TensorView* src, uint16_t* const* dst, int n_tensors, int B, int H, int N, int D, cudaStream_t stream);
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
