// Pre-pass of the fp32 tensor-core path: every fp32 row of up to 64 columns becomes one row of 128 bf16 numbers
// [hi(64) | lo(64)], hi = x rounded to bf16, lo = x - hi rounded to bf16, so that x = hi + lo + r with |r| <= 2^-18 |x|
// (bf16 keeps the range of fp32, so nothing overflows or is flushed); columns at or beyond the head dimension are zero. The
// tensor-core kernels then see tiles with the shared-memory geometry of a 128-column 16-bit tensor whose first slab
// holds the hi parts and whose second slab holds the lo parts. HBM-bound: 4 D bytes read and 256 bytes written per row.
#include <cuda_bf16.h>
#include "host_common.h"

namespace jvpfa {
namespace {

struct SplitArgs {
  TensorView src[kSplitMaxTensors];   // fp32 sources, possibly strided views (strides in elements)
  uint16_t* dst[kSplitMaxTensors];
  int H, N;
};

__device__ __forceinline__ void split2(float a, float b, uint32_t& hi, uint32_t& lo) {
  const __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  hi = *reinterpret_cast<const uint32_t*>(&h);
  const __nv_bfloat162 l = __floats2bfloat162_rn(a - __uint_as_float(hi << 16), b - __uint_as_float(hi & 0xFFFF0000u));
  lo = *reinterpret_cast<const uint32_t*>(&l);
}

// One thread per group of 8 columns of one row; blockIdx.y selects the tensor.
__global__ void split_fp32_kernel(const SplitArgs a, int64_t rows, int D) {
  const int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  const int64_t row = idx >> 3;
  const int g = static_cast<int>(idx & 7);
  if (row >= rows) return;
  uint32_t hi[4] = {0u, 0u, 0u, 0u}, lo[4] = {0u, 0u, 0u, 0u};
  if (g * 8 < D) {
    const TensorView& v = a.src[blockIdx.y];
    const int64_t n = row % a.N, bh = row / a.N;
    const float4* s = reinterpret_cast<const float4*>(static_cast<const float*>(v.ptr) + (bh / a.H) * v.sb + (bh % a.H) * v.sh +
                                                      n * v.sn + g * 8);
    const float4 x = s[0], y = s[1];
    split2(x.x, x.y, hi[0], lo[0]);
    split2(x.z, x.w, hi[1], lo[1]);
    split2(y.x, y.y, hi[2], lo[2]);
    split2(y.z, y.w, hi[3], lo[3]);
  }
  uint16_t* d = a.dst[blockIdx.y] + row * 128 + g * 8;
  *reinterpret_cast<uint4*>(d) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
  *reinterpret_cast<uint4*>(d + 64) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
}

}  // namespace

int launch_split_fp32(const TensorView* src, uint16_t* const* dst, int n_tensors, int B, int H, int N, int D,
                      cudaStream_t stream) {
  if (n_tensors <= 0 || n_tensors > kSplitMaxTensors || D <= 0 || D > 64 || (D % 8) != 0) return JVPFA_ERR_BAD_ARG;
  SplitArgs a{};
  a.H = H;
  a.N = N;
  const int64_t rows = static_cast<int64_t>(B) * H * N;
  for (int i = 0; i < n_tensors; ++i) {
    a.src[i] = src[i];
    a.dst[i] = dst[i];
  }
  const int64_t threads = rows * 8;
  dim3 grid(static_cast<unsigned>((threads + 255) / 256), n_tensors);
  split_fp32_kernel<<<grid, 256, 0, stream>>>(a, rows, D);
  return cudaGetLastError() == cudaSuccess ? JVPFA_OK : JVPFA_ERR_LAUNCH;
}

}  // namespace jvpfa
