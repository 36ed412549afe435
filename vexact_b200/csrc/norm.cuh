// RMSNorm and last-dim mean: HBM-bound row kernels.
//
// Replaces vexact/batch_invariant_ops/batch_invariant_ops.py:638-688
// (_rms_norm_kernel, single rounding), :337-382 (mean_kernel) and the HF eager
// RMSNorm formula (transformers Qwen3RMSNorm: round x*rsqrt(var+eps) to the
// input dtype, then multiply by the weight), which is what the reference hits
// for Qwen3/Qwen2/Qwen3-MoE through its aten::mean.dim override.
//
// Layout: x is [rows, n] with an element stride between rows; the row itself is
// contiguous.  One CTA of 128 threads owns one row when n > 1024, one warp owns
// one row otherwise.  Each thread reads 16-byte vectors at a fixed stride and
// keeps them in registers, so the row is read from HBM exactly once.  The sum of
// squares is accumulated per thread in element order, then folded with the fixed
// butterfly in common.cuh: the order depends on n only, never on `rows`.
#pragma once
#include "common.cuh"

namespace b200 {

enum { RMS_SINGLE_ROUND = 0, RMS_HF_DOUBLE_ROUND = 1 };

__device__ __forceinline__ float rms_scale(float sumsq, int n, float eps, int mode) {
  const float var = sumsq / (float)n;
  // mode 0 mirrors `1.0 / tl.sqrt(sum_sq / n_cols + eps)`; mode 1 mirrors torch.rsqrt.
  return mode == RMS_SINGLE_ROUND ? 1.0f / sqrtf(var + eps) : rsqrtf(var + eps);
}

__device__ __forceinline__ float rms_apply(float x, float inv, float w, int mode) {
  if (mode == RMS_SINGLE_ROUND) return x * inv * w;  // caller rounds once
  return w * round_bf(x * inv);                       // HF: bf16(x*inv) then * weight
}

// MAXV = number of 16-byte vectors a thread may cache (n <= MAXV * 8 * THREADS).
template <int THREADS, int MAXV, bool ADD_RESIDUAL>
__device__ __forceinline__ void rmsnorm_row(const __nv_bfloat16* __restrict__ x,
                                            const __nv_bfloat16* __restrict__ res,
                                            const __nv_bfloat16* __restrict__ w,
                                            __nv_bfloat16* __restrict__ out,
                                            __nv_bfloat16* __restrict__ sum_out, int n, float eps,
                                            int mode, int tid, float* scratch) {
  const int nvec = n >> 3;
  uint4 cache[MAXV];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < MAXV; ++i) {
    const int v = tid + i * THREADS;
    if (v < nvec) {
      uint4 a = reinterpret_cast<const uint4*>(x)[v];
      if (ADD_RESIDUAL) {
        // hidden = residual + x, rounded to bf16 exactly like the bf16 tensor add in the model.
        const uint4 r = reinterpret_cast<const uint4*>(res)[v];
        uint32_t* ap = reinterpret_cast<uint32_t*>(&a);
        const uint32_t* rp = reinterpret_cast<const uint32_t*>(&r);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          float a0, a1, r0, r1;
          unpack_bf2(ap[j], a0, a1);
          unpack_bf2(rp[j], r0, r1);
          ap[j] = pack_bf2(r0 + a0, r1 + a1);
        }
        reinterpret_cast<uint4*>(sum_out)[v] = a;
      }
      cache[i] = a;
      const uint32_t* ap = reinterpret_cast<const uint32_t*>(&a);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float a0, a1;
        unpack_bf2(ap[j], a0, a1);
        ss += a0 * a0;
        ss += a1 * a1;
      }
    }
  }
  float tot;
  if (THREADS == 32) {
    tot = warp_sum(ss);
  } else {
    tot = block_sum(ss, scratch);
  }
  const float inv = rms_scale(tot, n, eps, mode);
#pragma unroll
  for (int i = 0; i < MAXV; ++i) {
    const int v = tid + i * THREADS;
    if (v < nvec) {
      const uint4 a = cache[i];
      const uint4 ww = reinterpret_cast<const uint4*>(w)[v];
      const uint32_t* ap = reinterpret_cast<const uint32_t*>(&a);
      const uint32_t* wp = reinterpret_cast<const uint32_t*>(&ww);
      uint4 o;
      uint32_t* op = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float a0, a1, w0, w1;
        unpack_bf2(ap[j], a0, a1);
        unpack_bf2(wp[j], w0, w1);
        op[j] = pack_bf2(rms_apply(a0, inv, w0, mode), rms_apply(a1, inv, w1, mode));
      }
      reinterpret_cast<uint4*>(out)[v] = o;
    }
  }
}

// CTA-per-row variant: 128 threads, up to 8 cached vectors per thread (n <= 8192).
template <bool ADD_RESIDUAL>
__global__ void __launch_bounds__(128)
rmsnorm_cta_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ res,
                   const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ out,
                   __nv_bfloat16* __restrict__ sum_out, long long x_stride, long long res_stride,
                   long long out_stride, long long sum_stride, int n, float eps, int mode) {
  pdl_trigger();
  pdl_wait();
  __shared__ float scratch[32];
  const long long row = blockIdx.x;
  rmsnorm_row<128, 8, ADD_RESIDUAL>(x + row * x_stride, ADD_RESIDUAL ? res + row * res_stride : nullptr, w,
                                    out + row * out_stride,
                                    ADD_RESIDUAL ? sum_out + row * sum_stride : nullptr, n, eps, mode,
                                    threadIdx.x, scratch);
}

// Warp-per-row variant for short rows (n <= 1024), 8 rows per CTA.
template <bool ADD_RESIDUAL>
__global__ void __launch_bounds__(256)
rmsnorm_warp_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ res,
                    const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ out,
                    __nv_bfloat16* __restrict__ sum_out, long long x_stride, long long res_stride,
                    long long out_stride, long long sum_stride, long long rows, int n, float eps,
                    int mode) {
  pdl_trigger();
  pdl_wait();
  const long long row = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (row >= rows) return;
  rmsnorm_row<32, 4, ADD_RESIDUAL>(x + row * x_stride, ADD_RESIDUAL ? res + row * res_stride : nullptr, w,
                                   out + row * out_stride,
                                   ADD_RESIDUAL ? sum_out + row * sum_stride : nullptr, n, eps, mode,
                                   threadIdx.x & 31, nullptr);
}

// Generic (any n, any alignment) fallback: one CTA per row, scalar loads, two passes.
__global__ void __launch_bounds__(128)
rmsnorm_generic_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ res,
                       const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ out,
                       __nv_bfloat16* __restrict__ sum_out, long long x_stride, long long res_stride,
                       long long out_stride, long long sum_stride, int n, float eps, int mode) {
  pdl_trigger();
  pdl_wait();
  __shared__ float scratch[32];
  const long long row = blockIdx.x;
  const __nv_bfloat16* xr = x + row * x_stride;
  const __nv_bfloat16* rr = res ? res + row * res_stride : nullptr;
  __nv_bfloat16* sr = sum_out ? sum_out + row * sum_stride : nullptr;
  float ss = 0.f;
  for (int i = threadIdx.x; i < n; i += 128) {
    float a = bf2f(xr[i]);
    if (rr) {
      a = round_bf(bf2f(rr[i]) + a);
      sr[i] = f2bf(a);
    }
    ss += a * a;
  }
  const float tot = block_sum(ss, scratch);
  const float inv = rms_scale(tot, n, eps, mode);
  for (int i = threadIdx.x; i < n; i += 128) {
    const float a = rr ? bf2f(sr[i]) : bf2f(xr[i]);
    out[row * out_stride + i] = f2bf(rms_apply(a, inv, bf2f(w[i]), mode));
  }
}

// Mean over the last dim, fp32 in / fp32 out (the HF RMSNorm variance).  One warp per row.
template <typename T>
__global__ void __launch_bounds__(256)
mean_lastdim_kernel(const T* __restrict__ x, T* __restrict__ out, long long rows, int n,
                    long long x_stride) {
  pdl_trigger();
  pdl_wait();
  const long long row = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int lane = threadIdx.x & 31;
  const T* xr = x + row * x_stride;
  float acc = 0.f;
  for (int i = lane; i < n; i += 32) acc += (float)xr[i];
  acc = warp_sum(acc);
  if (lane == 0) out[row] = (T)(acc / (float)n);
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

}  // namespace b200

extern "C" int b200_rmsnorm(const void* x, const void* weight, void* out, long long rows, int n,
                            long long x_row_stride, long long out_row_stride, float eps, int mode,
                            void* stream) {
  using namespace b200;
  if (!x || !weight || !out || rows < 0 || n <= 0 || (mode != 0 && mode != 1)) return B200_ERR_ARG;
  if (rows == 0) return B200_OK;
  auto X = (const __nv_bfloat16*)x;
  auto W = (const __nv_bfloat16*)weight;
  auto O = (__nv_bfloat16*)out;
  cudaStream_t st = (cudaStream_t)stream;
  const bool vec = (n % 8 == 0) && aligned16(x) && aligned16(weight) && aligned16(out) &&
                   (x_row_stride % 8 == 0) && (out_row_stride % 8 == 0);
  if (vec && n <= 1024) {
    launch_k(rmsnorm_warp_kernel<false>, dim3((unsigned)((rows + 7) / 8)), dim3(256), 0, st, 
        X, nullptr, W, O, nullptr, x_row_stride, 0, out_row_stride, 0, rows, n, eps, mode);
  } else if (vec && n <= 8192) {
    launch_k(rmsnorm_cta_kernel<false>, dim3((unsigned)rows), dim3(128), 0, st, X, nullptr, W, O, nullptr, x_row_stride, 0,
                                                               out_row_stride, 0, n, eps, mode);
  } else {
    launch_k(rmsnorm_generic_kernel, dim3((unsigned)rows), dim3(128), 0, st, X, nullptr, W, O, nullptr, x_row_stride, 0,
                                                            out_row_stride, 0, n, eps, mode);
  }
  return launch_status();
}

extern "C" int b200_add_rmsnorm(const void* x, const void* residual, const void* weight, void* sum_out,
                                void* out, long long rows, int n, float eps, int mode, void* stream) {
  using namespace b200;
  if (!x || !residual || !weight || !out || !sum_out || rows < 0 || n <= 0 || (mode != 0 && mode != 1))
    return B200_ERR_ARG;
  if (rows == 0) return B200_OK;
  auto X = (const __nv_bfloat16*)x;
  auto R = (const __nv_bfloat16*)residual;
  auto W = (const __nv_bfloat16*)weight;
  auto O = (__nv_bfloat16*)out;
  auto S = (__nv_bfloat16*)sum_out;
  cudaStream_t st = (cudaStream_t)stream;
  const bool vec = (n % 8 == 0) && aligned16(x) && aligned16(residual) && aligned16(weight) &&
                   aligned16(out) && aligned16(sum_out);
  if (vec && n <= 1024) {
    launch_k(rmsnorm_warp_kernel<true>, dim3((unsigned)((rows + 7) / 8)), dim3(256), 0, st, X, R, W, O, S, n, n, n, n, rows, n,
                                                                          eps, mode);
  } else if (vec && n <= 8192) {
    launch_k(rmsnorm_cta_kernel<true>, dim3((unsigned)rows), dim3(128), 0, st, X, R, W, O, S, n, n, n, n, n, eps, mode);
  } else {
    launch_k(rmsnorm_generic_kernel, dim3((unsigned)rows), dim3(128), 0, st, X, R, W, O, S, n, n, n, n, n, eps, mode);
  }
  return launch_status();
}

extern "C" int b200_mean_lastdim(const void* x, void* out, long long rows, int n, long long x_row_stride,
                                 int dtype /*0 = f32, 1 = bf16*/, void* stream) {
  using namespace b200;
  if (!x || !out || rows < 0 || n <= 0) return B200_ERR_ARG;
  if (rows == 0) return B200_OK;
  cudaStream_t st = (cudaStream_t)stream;
  const unsigned grid = (unsigned)((rows + 7) / 8);
  if (dtype == 0) {
    launch_k(mean_lastdim_kernel<float>, dim3(grid), dim3(256), 0, st, (const float*)x, (float*)out, rows, n, x_row_stride);
  } else if (dtype == 1) {
    launch_k(mean_lastdim_kernel<__nv_bfloat16>, dim3(grid), dim3(256), 0, st, (const __nv_bfloat16*)x, (__nv_bfloat16*)out, rows, n, x_row_stride);
  } else {
    return B200_ERR_ARG;
  }
  return launch_status();
}

// ------------------------------------------------------------------ RMSNorm backward (training-side twin)
// Follows BatchInvariantRMSNormFunction.backward (vexact/batch_invariant_ops/batch_invariant_ops.py:701-725):
//   inv = rsqrt(mean(x^2) + eps); normed = x * inv; d = g * w
//   grad_x = inv * (d - normed * mean(d * normed))                       (per row: batch invariant)
//   grad_w = sum over rows of g * normed                                 (fixed order: see below)
// grad_w is reduced in two fixed stages, 64 consecutive rows per partial and then the partials in ascending
// order, so the result depends on the row count only (the reference's torch .sum(0) leaves its order to
// the library).
namespace b200 {

constexpr int RMSB_ROWS_PER_PARTIAL = 64;

__global__ void __launch_bounds__(256)
rmsnorm_bwd_row_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                       const __nv_bfloat16* __restrict__ g, __nv_bfloat16* __restrict__ gx,
                       float* __restrict__ inv_out, int n, float eps) {
  pdl_trigger();
  pdl_wait();
  __shared__ float scratch[32];
  const long long row = blockIdx.x;
  const __nv_bfloat16* xr = x + row * n;
  const __nv_bfloat16* gr = g + row * n;
  float ss = 0.f;
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const float v = bf2f(xr[i]);
    ss = fmaf(v, v, ss);
  }
  const float inv = rsqrtf(block_sum(ss, scratch) / (float)n + eps);
  float dot = 0.f;
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const float d = bf2f(gr[i]) * bf2f(w[i]);
    dot = fmaf(d, bf2f(xr[i]) * inv, dot);
  }
  const float c = block_sum(dot, scratch) / (float)n;
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const float normed = bf2f(xr[i]) * inv;
    const float d = bf2f(gr[i]) * bf2f(w[i]);
    gx[row * n + i] = f2bf(inv * (d - normed * c));
  }
  if (threadIdx.x == 0) inv_out[row] = inv;
}

// partial[blk][col] = sum over the block's rows (ascending) of g * x * inv
__global__ void __launch_bounds__(256)
rmsnorm_bwd_wpartial_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ g,
                            const float* __restrict__ inv, float* __restrict__ partial, long long rows, int n) {
  pdl_trigger();
  pdl_wait();
  const int col = blockIdx.x * blockDim.x + threadIdx.x;
  if (col >= n) return;
  const long long r0 = (long long)blockIdx.y * RMSB_ROWS_PER_PARTIAL;
  const long long r1 = r0 + RMSB_ROWS_PER_PARTIAL < rows ? r0 + RMSB_ROWS_PER_PARTIAL : rows;
  float acc = 0.f;
  for (long long r = r0; r < r1; ++r) acc += bf2f(g[r * n + col]) * (bf2f(x[r * n + col]) * inv[r]);
  partial[(long long)blockIdx.y * n + col] = acc;
}

__global__ void __launch_bounds__(256)
rmsnorm_bwd_wfinal_kernel(const float* __restrict__ partial, __nv_bfloat16* __restrict__ gw, int nparts, int n) {
  pdl_trigger();
  pdl_wait();
  const int col = blockIdx.x * blockDim.x + threadIdx.x;
  if (col >= n) return;
  float acc = 0.f;
  for (int b = 0; b < nparts; ++b) acc += partial[(long long)b * n + col];
  gw[col] = f2bf(acc);
}

}  // namespace b200

// x, grad_out, grad_in [rows, n] bf16 contiguous; weight, grad_weight [n] bf16.
// scratch: fp32, rows + ceil(rows / 64) * n elements (inverse norms, then the grad_weight partials).
extern "C" int b200_rmsnorm_backward(const void* x, const void* weight, const void* grad_out, void* grad_in,
                                     void* grad_weight, void* scratch_f32, long long rows, int n, float eps,
                                     void* stream) {
  using namespace b200;
  if (!x || !weight || !grad_out || !grad_in || !grad_weight || !scratch_f32 || rows < 0 || n <= 0) return B200_ERR_ARG;
  if (rows == 0) return B200_OK;
  if (rows > 0x7fffffffLL) return B200_ERR_SHAPE;
  cudaStream_t st = (cudaStream_t)stream;
  float* inv = (float*)scratch_f32;
  float* partial = inv + rows;
  const int nparts = (int)((rows + RMSB_ROWS_PER_PARTIAL - 1) / RMSB_ROWS_PER_PARTIAL);
  launch_k(rmsnorm_bwd_row_kernel, dim3((unsigned)rows), dim3(256), 0, st, (const __nv_bfloat16*)x,
           (const __nv_bfloat16*)weight, (const __nv_bfloat16*)grad_out, (__nv_bfloat16*)grad_in, inv, n, eps);
  launch_k(rmsnorm_bwd_wpartial_kernel, dim3((unsigned)((n + 255) / 256), (unsigned)nparts), dim3(256), 0, st,
           (const __nv_bfloat16*)x, (const __nv_bfloat16*)grad_out, (const float*)inv, partial, rows, n);
  launch_k(rmsnorm_bwd_wfinal_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, st, (const float*)partial,
           (__nv_bfloat16*)grad_weight, nparts, n);
  return launch_status();
}
