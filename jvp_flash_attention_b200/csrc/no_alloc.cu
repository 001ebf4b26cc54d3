// jvpfa_bwd_noalloc: the dual backward for callers that must not, or cannot, allocate device memory.
//
// Who that is: a plug-in that runs inside a serving or training process whose own memory pool has
// already claimed nearly all of the GPU's memory (a cudaMalloc from the plug-in would fail, and the
// pool gives the plug-in no allocation hook), and code on a latency-critical path, where
// cudaMalloc / cudaFree are off limits because they synchronise the whole device. Such a caller can
// still pass its input and output tensors, but has nowhere to get the backward's scratch from (the
// device status word and one float4 of per-row statistics per query row). This entry point keeps
// that scratch in a fixed array that is part of the library image, so the call itself allocates
// nothing: no cudaMalloc, no cudaFree, no allocating library routine. (With CUDA's lazy module loading the
// driver sets the image's 4 MiB array up when the first call on a device asks for its address; a caller whose
// pool is about to take the rest of the GPU's memory makes that first call before the pool grows, or runs
// with CUDA_MODULE_LOADING=EAGER.)
#include <mutex>
#include "host_common.h"

namespace {

constexpr int64_t kNoAllocMaxRows = JVPFA_NO_ALLOC_MAX_ROWS;
constexpr size_t kNoAllocBytes = jvpfa::kStatusBytes + static_cast<size_t>(kNoAllocMaxRows) * 16;

// The scratch itself. Every GPU that loads the library holds these 4 MiB + 256 B until the process
// exits. In host code this name is only a stand-in for the symbol, never a device address: host code
// asks the runtime for the address (below) and hands that to the kernels.
static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoAllocBytes];

constexpr int kMaxDevices = 64;
std::mutex g_setup_mutex;
void* g_scratch_addr[kMaxDevices] = {};

// Device address of the scratch on the current device; looked up once per device, with that device current.
int scratch_address(void** out) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return JVPFA_ERR_LAUNCH;
  std::lock_guard<std::mutex> guard(g_setup_mutex);
  if (g_scratch_addr[dev] == nullptr) {
    void* ptr = nullptr;
    if (cudaGetSymbolAddress(&ptr, g_noalloc_scratch) != cudaSuccess || ptr == nullptr) {
      (void)cudaGetLastError();   // do not leave the failed look-up behind as this thread's sticky error
      return JVPFA_ERR_LAUNCH;
    }
    g_scratch_addr[dev] = ptr;
  }
  *out = g_scratch_addr[dev];
  return JVPFA_OK;
}

}  // namespace

extern "C" int jvpfa_bwd_noalloc(const jvpfa_bwd_args* args, int32_t* status_word_out, void* stream) {
  if (args == nullptr) return JVPFA_ERR_BAD_ARG;
  if (args->B <= 0 || args->H <= 0 || args->N <= 0) return JVPFA_ERR_BAD_ARG;
  const int64_t rows = static_cast<int64_t>(args->B) * args->H * args->N;
  if (rows > kNoAllocMaxRows) return JVPFA_ERR_NO_ALLOC_LIMIT;
  void* scratch = nullptr;
  int rc = scratch_address(&scratch);
  if (rc != JVPFA_OK) return rc;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  // The array keeps whatever the previous call left. Only the status word has to start at zero (the
  // kernels record the first wait that gave up with a compare-and-swap against 0); the statistics are
  // rewritten in full for the rows of this call before anything reads them.
  if (cudaMemsetAsync(scratch, 0, jvpfa::kStatusBytes, s) != cudaSuccess) return JVPFA_ERR_LAUNCH;
  jvpfa_bwd_args with_scratch = *args;
  with_scratch.workspace = scratch;
  // exactly what the status word and the statistics take: fp32 inputs therefore run on the CUDA-core kernels here
  // (their tensor-core path would want room for split operands that this fixed array does not have)
  with_scratch.workspace_bytes = jvpfa::kStatusBytes + static_cast<size_t>(rows) * 16;
  rc = jvpfa_bwd(&with_scratch, stream);
  if (rc != JVPFA_OK) return rc;
  if (status_word_out != nullptr &&
      cudaMemcpyAsync(status_word_out, scratch, sizeof(int32_t), cudaMemcpyDeviceToDevice, s) != cudaSuccess)
    return JVPFA_ERR_LAUNCH;
  return JVPFA_OK;
}
