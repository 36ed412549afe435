// Single translation unit of libvexact_b200.so: every kernel family plus the
// C-ABI entry points declared in include/vexact_b200.h.
#include "norm.cuh"
#include "softmax.cuh"
#include "kv.cuh"
#include "gemm.cuh"
#include "attn.cuh"
#include "attn_tc.cuh"
#include "moe.cuh"
#include "noalloc.cuh"
#include "step.cuh"
#include "sample.cuh"

// Copies the device status word ({code, detail, block, spare}) to host memory and clears it.
// Synchronises the stream: call it outside graph capture, after the work of interest.
extern "C" int b200_status_read(int* host_out4, void* stream) {
  using namespace b200;
  if (!host_out4) return B200_ERR_ARG;
  cudaStream_t st = (cudaStream_t)stream;
  if (cudaMemcpyFromSymbolAsync(host_out4, g_status, sizeof(int) * 4, 0, cudaMemcpyDeviceToHost, st) != cudaSuccess)
    return B200_ERR_LAUNCH;
  if (cudaStreamSynchronize(st) != cudaSuccess) return B200_ERR_LAUNCH;
  const int zero[4] = {0, 0, 0, 0};
  if (cudaMemcpyToSymbolAsync(g_status, zero, sizeof(zero), 0, cudaMemcpyHostToDevice, st) != cudaSuccess)
    return B200_ERR_LAUNCH;
  if (cudaStreamSynchronize(st) != cudaSuccess) return B200_ERR_LAUNCH;
  return B200_OK;
}

extern "C" int b200_abi_version(void) { return 1; }
