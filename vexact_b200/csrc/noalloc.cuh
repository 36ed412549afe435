// Grouped GEMM for callers that cannot allocate device memory.
//
// b200_moe_grouped_gemm needs a small table in global memory that says which rows of which
// expert each token tile covers.  Its usual caller gets that table from b200_moe_permute into
// memory it allocated with torch.  Some callers have no allocator to ask: a C or C++ host that
// owns its buffers statically, code running while a stream capture is open on another thread
// (cudaMalloc is not permitted to it), or a service whose memory budget is fixed at start-up.
// For them this file offers one entry point that takes what quack's varlen GEMM takes
// (expert-sorted rows plus cu_seqlens) and keeps the tile table in a fixed array that is part
// of the library image.
//
// The array, its one-time address lookup and the entry point live together in this file (all
// kernels of the library are one translation unit, so the symbol below has exactly one copy).
//   * Every GPU that loads the library holds the array (about 64 KiB) until the process exits.
//   * Host code must not pass `g_noalloc_tiles` to a kernel: on the host that name is only a
//     handle.  The device address is fetched once per device with cudaGetSymbolAddress, with
//     that device current, and that pointer is what kernels receive.
//   * All calls share the array and it keeps the previous call's contents.  Each call rewrites
//     the tile count and every tile entry it will read before the GEMM reads them (both
//     kernels are on the caller's stream, in order).  Two calls that overlap on the GPU (on
//     different streams) race on the array: serialise them.
//   * The looked-up address is cached per device for the life of the process.  cudaDeviceReset()
//     destroys the context the address belongs to: after a reset the cached value is stale and
//     this entry point must not be used again in that process.
//   * cu_seqlens comes from the caller, so it is checked on the device: a group whose bounds are
//     not 0 <= cu_seqlens[g] <= cu_seqlens[g+1] <= x_rows is clipped to the valid rows (dropped
//     when it is decreasing) and B200_STATUS_BAD_INDEX with the group id is left in the status
//     word; no tile ever names a row outside [0, x_rows).
#pragma once
#include <atomic>

#include "gemm.cuh"

namespace b200 {

constexpr int NOALLOC_MAX_TILES = 4095;   // token tiles one call may need
constexpr int NOALLOC_MAX_GROUPS = 1024;  // experts
constexpr int NOALLOC_MAX_DEVICES = 64;

// entry 0 = {tile count, 0, 0, 0}; entries 1.. = {group, first_row, n_rows, 0}
static __device__ __align__(256) int4 g_noalloc_tiles[NOALLOC_MAX_TILES + 1];

// Device address of the array on the current device (looked up once per device).
// Host threads may race on the first call: every racer looks up the same value, the slot is atomic.
inline int noalloc_tiles_ptr(int4** out) {
  static std::atomic<int4*> ptrs[NOALLOC_MAX_DEVICES];
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= NOALLOC_MAX_DEVICES) return B200_ERR_LAUNCH;
  int4* cached = ptrs[dev].load(std::memory_order_acquire);
  if (cached == nullptr) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_noalloc_tiles) != cudaSuccess || p == nullptr) return B200_ERR_LAUNCH;
    cached = static_cast<int4*>(p);
    ptrs[dev].store(cached, std::memory_order_release);
  }
  *out = cached;
  return B200_OK;
}

// One CTA: tiles of at most `tile_rows` consecutive rows per group, in group order.
__global__ void __launch_bounds__(1024)
tiles_from_cu_seqlens_kernel(const int* __restrict__ cu_seqlens, int num_groups, int tile_rows,
                             int4* __restrict__ table /* entry 0 = count */, int max_tiles, int x_rows) {
  __shared__ int first_tile[NOALLOC_MAX_GROUPS + 1];
  const int g = threadIdx.x;
  int rows = 0, r0 = 0;
  if (g < num_groups) {
    const int lo = cu_seqlens[g], hi = cu_seqlens[g + 1];
    if (lo < 0 || hi < lo || hi > x_rows) report_status(B200_STATUS_BAD_INDEX, g);
    r0 = min(max(lo, 0), x_rows);
    rows = hi < lo ? 0 : min(max(hi, r0), x_rows) - r0;  // a decreasing group is dropped, an overrun clipped
  }
  const int tiles = (rows + tile_rows - 1) / tile_rows;
  first_tile[g] = tiles;
  __syncthreads();
  if (g == 0) {  // exclusive scan; at most 1024 small integers
    int run = 0;
    for (int i = 0; i < num_groups; ++i) {
      const int t = first_tile[i];
      first_tile[i] = run;
      run += t;
    }
    first_tile[num_groups] = run;
    table[0] = make_int4(min(run, max_tiles), 0, 0, 0);
  }
  __syncthreads();
  if (g < num_groups) {
    const int t0 = first_tile[g];
    for (int j = 0; j < tiles; ++j)
      if (t0 + j < max_tiles)
        table[1 + t0 + j] = make_int4(g, r0 + j * tile_rows, min(tile_rows, rows - j * tile_rows), 0);
  }
}

}  // namespace b200

// Same arithmetic and the same GEMM kernel as b200_moe_grouped_gemm (modes 0 and 1), for rows
// already sorted by group, with the tile table kept in the library's fixed device array.
//   x [x_rows, K] bf16, w [num_groups, n_out | 2*n_out, K] bf16, cu_seqlens [num_groups + 1] int32
//   (device memory: rows of group g are cu_seqlens[g] .. cu_seqlens[g+1]), out [x_rows, n_out] bf16.
// Limits: num_groups <= 1024 and num_groups + x_rows / 64 <= 4095 token tiles; beyond them the
// call returns -2 and launches nothing.  It calls no cudaMalloc / cudaFree.  The first call on a
// device looks up the array's device address; make that call before any stream capture begins.
extern "C" int b200_moe_grouped_gemm_noalloc(const void* x, const void* w, const void* row_scale, void* out,
                                             const void* cu_seqlens, long long x_rows, int num_groups,
                                             int n_out, int K, long long out_row_stride, int mode,
                                             void* stream) {
  using namespace b200;
  if (!x || !w || !out || !cu_seqlens || x_rows < 0 || num_groups <= 0 || n_out <= 0 || K <= 0 ||
      (mode != 0 && mode != 1))
    return B200_ERR_ARG;
  constexpr int kTileRows = 64;
  if (num_groups > NOALLOC_MAX_GROUPS) return B200_ERR_SHAPE;
  const long long bound = (long long)num_groups + x_rows / kTileRows;
  if (bound > NOALLOC_MAX_TILES) return B200_ERR_SHAPE;
  if (x_rows == 0) return B200_OK;
  int4* table = nullptr;
  int rc = noalloc_tiles_ptr(&table);
  if (rc) return rc;
  cudaStream_t st = (cudaStream_t)stream;
  if (x_rows > 0x7fffffffLL) return B200_ERR_SHAPE;
  tiles_from_cu_seqlens_kernel<<<1, 1024, 0, st>>>((const int*)cu_seqlens, num_groups, kTileRows, table,
                                                   NOALLOC_MAX_TILES, (int)x_rows);
  rc = launch_status();
  if (rc) return rc;
  return b200_moe_grouped_gemm(x, w, row_scale, out, table + 1, table, x_rows, num_groups, n_out, K,
                               out_row_stride, (int)bound, kTileRows, mode, stream);
}
