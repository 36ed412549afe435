// Shared device/host helpers for the sm_100a rollout-forward kernels.
//
// Conventions used by every kernel in this directory:
//   * every entry point launches on the caller's stream, allocates nothing and
//     never synchronises, so it can be captured into a CUDA graph;
//   * every reduction uses one fixed tree that depends only on the row length,
//     never on the number of rows, so a row's result is bitwise independent of
//     the batch it is computed in;
//   * every spin-wait is bounded: on expiry the kernel writes a code into the
//     device status word (see b200_status_read) and returns.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdlib.h>

#include <atomic>

#define B200_OK 0
#define B200_ERR_ARG (-1)
#define B200_ERR_SHAPE (-2)
#define B200_ERR_LAUNCH (-3)
#define B200_ERR_DRIVER (-4)

// Codes a kernel may leave in the device status word.
#define B200_STATUS_OK 0
#define B200_STATUS_WAIT_EXPIRED 1
#define B200_STATUS_BAD_INDEX 2

namespace b200 {

// Device status word: [0] = first non-zero code seen, [1] = detail (barrier id
// or offending index), [2] = block id, [3] = spare.
__device__ int g_status[4];  // one copy: all kernels are built as a single translation unit

__device__ __forceinline__ void report_status(int code, int detail) {
  if (atomicCAS(&g_status[0], 0, code) == 0) {
    g_status[1] = detail;
    g_status[2] = (int)blockIdx.x;
  }
}

__device__ __forceinline__ float bf2f(__nv_bfloat16 v) { return __bfloat162float(v); }
__device__ __forceinline__ __nv_bfloat16 f2bf(float v) { return __float2bfloat16_rn(v); }
// Round an fp32 value to bf16 precision and keep it in fp32 (models a bf16
// tensor being materialised between two torch ops).
__device__ __forceinline__ float round_bf(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }

__device__ __forceinline__ uint32_t pack_bf2(float lo, float hi) {
  __nv_bfloat162 t = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&t);
}
__device__ __forceinline__ void unpack_bf2(uint32_t v, float& lo, float& hi) {
  __nv_bfloat162 t = *reinterpret_cast<__nv_bfloat162*>(&v);
  lo = __low2float(t);
  hi = __high2float(t);
}

// Fixed butterfly reductions over a full warp.
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Block-wide sum with a fixed order: warp butterflies, then warp 0 folds the
// per-warp partials with another butterfly.  `scratch` holds 32 floats.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nwarps = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float t = (lane < nwarps) ? scratch[lane] : 0.f;
  t = warp_sum(t);
  return t;
}
__device__ __forceinline__ float block_max(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nwarps = (blockDim.x + 31) >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float t = (lane < nwarps) ? scratch[lane] : -INFINITY;
  t = warp_max(t);
  return t;
}

__device__ __forceinline__ uint64_t global_timer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

// Programmatic dependent launch.  Kernels of the per-layer chain are launched with the
// programmatic-stream-serialization attribute: a kernel may start (and run its prologue) while
// its predecessor drains, and touches global memory only after pdl_wait(), which returns once
// the predecessor has completed and its writes are visible.  pdl_trigger() lets the successor
// begin launching; every CTA calls it first thing, so a successor can become resident only
// when every CTA of this kernel has started.  Without the attribute both are no-ops.
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// Programmatic dependent launch (B200_PDL): 0 = off, 1 = every kernel, 3 = only kernels without dynamic
// shared memory, i.e. the short row / routing / permutation kernels, which can be resident beside a
// finishing GEMM or attention CTA and then start the moment it is done; 2 (default) = those plus the dense
// GEMMs, which request their first weight tiles before they wait.  Every kernel waits
// (griddepcontrol.wait) before it touches what its predecessor wrote.  Measured inside the captured
// decode step: mode 3 is worth 2.5 % on the small dense models and neutral on the 30B-A3B shape;
// mode 1 costs the latter 0.4 %.
inline int pdl_mode() {
  static const int mode = []() {
    const char* v = getenv("B200_PDL");
    return v ? atoi(v) : 2;
  }();
  return mode;
}

template <typename... KArgs, typename... Args>
inline void launch_k_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, bool pdl,
                         Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl ? 1 : 0;
  cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

template <typename... KArgs, typename... Args>
inline void launch_k(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  const int mode = pdl_mode();
  cfg.numAttrs = (mode == 1 || (mode >= 2 && smem == 0)) ? 1 : 0;
  cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// Facts and one-time settings that belong to a device, not to the process: a process that drives
// several GPUs gets each of them looked up / set once, with that device current.
constexpr int B200_MAX_DEVICES = 64;

struct PerDeviceFlags {
  std::atomic<int> v[B200_MAX_DEVICES];  // static storage: zero-initialised
};

inline int current_device_index() {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= B200_MAX_DEVICES) return -1;
  return dev;
}

// Raises a kernel's dynamic shared-memory limit once per device (the attribute is per device).
template <typename KernelT>
inline int set_max_dyn_smem_once(PerDeviceFlags& done, KernelT kernel, int bytes) {
  const int dev = current_device_index();
  if (dev < 0) return B200_ERR_LAUNCH;
  if (done.v[dev].load(std::memory_order_acquire) == 0) {
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes) != cudaSuccess)
      return B200_ERR_LAUNCH;
    done.v[dev].store(1, std::memory_order_release);
  }
  return B200_OK;
}

// SM count of the current device (cached per device).
inline int sm_count() {
  static PerDeviceFlags cache;
  const int dev = current_device_index();
  if (dev < 0) return 148;
  int n = cache.v[dev].load(std::memory_order_acquire);
  if (n == 0) {
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cache.v[dev].store(n, std::memory_order_release);
  }
  return n;
}

inline int launch_status() {
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? B200_OK : B200_ERR_LAUNCH;
}

}  // namespace b200
