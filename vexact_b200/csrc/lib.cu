// Single translation unit of libvexact_b200.so: every kernel family plus the
// C-ABI entry points declared in include/vexact_b200.h.
#include "norm.cuh"
#include "softmax.cuh"
#include "kv.cuh"
#include "gemm.cuh"
#include "attn.cuh"
#include "attn_tc.cuh"
#include "attn_rows.cuh"
#include "attn_bwd_mma.cuh"
#include "moe.cuh"
#include "noalloc.cuh"
#include "step.cuh"
#include "sample.cuh"

// Self-test of the bounded wait every kernel here relies on: one CTA waits, with a limit of
// `limit_us` microseconds, on an mbarrier that nothing ever completes.  The wait must give up, record
// B200_STATUS_WAIT_EXPIRED with detail 999 in the status word and let the kernel return; out_flag[0] is
// set to 1 when the wait returned "expired" and to 2 if it (impossibly) saw the barrier complete.
namespace b200 {
__global__ void wait_expiry_selftest_kernel(unsigned long long limit_ns, int* out_flag) {
  __shared__ uint64_t bar;
  __shared__ int abort_mem;
  pdl_trigger();
  pdl_wait();  // launched through launch_k like every kernel here: wait before touching global memory
  if (threadIdx.x == 0) {
    abort_mem = 0;
    ptx::mbar_init(ptx::smem_u32(&bar), 1);
    ptx::fence_barrier_init();
    const bool done = ptx::mbar_wait(ptx::smem_u32(&bar), 0, &abort_mem, 999, limit_ns);
    *out_flag = done ? 2 : 1;
  }
}
}  // namespace b200

extern "C" int b200_selftest_wait_expiry(int limit_us, int* out_flag_device, void* stream) {
  using namespace b200;
  if (!out_flag_device || limit_us <= 0 || limit_us > 1000000) return B200_ERR_ARG;
  launch_k(wait_expiry_selftest_kernel, dim3(1), dim3(32), 0, (cudaStream_t)stream,
           (unsigned long long)limit_us * 1000ull, out_flag_device);
  return launch_status();
}

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

// Bumped whenever an exported signature changes.
extern "C" int b200_abi_version(void) { return 4; }

// Hash of the sources and compiler flags this binary was built from (set by the build script);
// the loader compares it with the sources beside it and refuses a stale library.
#ifndef B200_SOURCE_HASH
#define B200_SOURCE_HASH "unknown"
#endif
extern "C" const char* b200_source_hash(void) { return B200_SOURCE_HASH; }
