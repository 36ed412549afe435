// Row log-softmax and per-token log-probability: HBM-bound row kernels.
//
// Replaces vexact/batch_invariant_ops/batch_invariant_ops.py:232-331
// (_log_softmax_kernel / log_softmax: max pass, sum-exp pass, write pass) and
// vexact/batch_invariant_ops/standalone_logprobs.py:28-55, whose arithmetic is
// flash-attn's Triton cross-entropy forward (logprob = x[label] - logsumexp(x)).
//
// One CTA of 1024 threads owns one row.  Each thread walks 16-byte vectors at a
// fixed stride keeping a private (max, sum exp(x - max)) pair; pairs are merged
// with a fixed butterfly inside each warp and a second butterfly over the 32
// warp results.  The merge order is a function of the row length only.
#pragma once
#include "common.cuh"

namespace b200 {

struct MaxSum {
  float m, s;
};

__device__ __forceinline__ MaxSum ms_merge(MaxSum a, MaxSum b) {
  const float m = fmaxf(a.m, b.m);
  MaxSum r;
  r.m = m;
  // exp(-inf - finite) = 0; the (m == -inf) guard keeps empty partials NaN free.
  const float ea = (a.m == -INFINITY) ? 0.f : expf(a.m - m);
  const float eb = (b.m == -INFINITY) ? 0.f : expf(b.m - m);
  r.s = a.s * ea + b.s * eb;
  return r;
}

__device__ __forceinline__ void ms_push(MaxSum& a, float x) {
  if (x > a.m) {
    a.s = (a.m == -INFINITY) ? 0.f : a.s * expf(a.m - x);
    a.m = x;
    a.s += 1.0f;
  } else if (x > -INFINITY) {
    a.s += expf(x - a.m);
  }
}

// Vector form: one rescale per vector, then the exps in element order.
template <int VEC>
__device__ __forceinline__ void ms_push_vec(MaxSum& a, const float* x) {
  float vm = x[0];
#pragma unroll
  for (int j = 1; j < VEC; ++j) vm = fmaxf(vm, x[j]);
  if (vm > a.m) {
    a.s = (a.m == -INFINITY) ? 0.f : a.s * expf(a.m - vm);
    a.m = vm;
  }
  if (a.m > -INFINITY) {
#pragma unroll
    for (int j = 0; j < VEC; ++j) a.s += expf(x[j] - a.m);
  }
}

__device__ __forceinline__ MaxSum ms_block_reduce(MaxSum v, float* sm, float* ss) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nwarps = blockDim.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    MaxSum t;
    t.m = __shfl_xor_sync(0xffffffffu, v.m, o);
    t.s = __shfl_xor_sync(0xffffffffu, v.s, o);
    // Merge in lane order so both partners compute the same bits.
    v = (lane & o) ? ms_merge(t, v) : ms_merge(v, t);
  }
  __syncthreads();
  if (lane == 0) {
    sm[warp] = v.m;
    ss[warp] = v.s;
  }
  __syncthreads();
  MaxSum t;
  t.m = lane < nwarps ? sm[lane] : -INFINITY;
  t.s = lane < nwarps ? ss[lane] : 0.f;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    MaxSum u;
    u.m = __shfl_xor_sync(0xffffffffu, t.m, o);
    u.s = __shfl_xor_sync(0xffffffffu, t.s, o);
    t = (lane & o) ? ms_merge(u, t) : ms_merge(t, u);
  }
  return t;
}

template <typename T>
struct RowLoader;

template <>
struct RowLoader<float> {
  static constexpr int VEC = 4;
  static __device__ __forceinline__ void load(const float* p, float* v) {
    const float4 t = *reinterpret_cast<const float4*>(p);
    v[0] = t.x, v[1] = t.y, v[2] = t.z, v[3] = t.w;
  }
};
template <>
struct RowLoader<__nv_bfloat16> {
  static constexpr int VEC = 8;
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, float* v) {
    const uint4 t = *reinterpret_cast<const uint4*>(p);
    const uint32_t* tp = reinterpret_cast<const uint32_t*>(&t);
#pragma unroll
    for (int j = 0; j < 4; ++j) unpack_bf2(tp[j], v[2 * j], v[2 * j + 1]);
  }
};

// Streams one row and returns its (max, sum exp) pair.  `vec_ok` is a launch-wide
// property (base pointer 16-byte aligned and row stride a multiple of the vector
// width), so every row of a launch, and the same row in any other batch, walks
// its elements in the same order.
template <typename T>
__device__ __forceinline__ MaxSum row_max_sum(const T* __restrict__ row, int n, bool vec_ok, float* sm,
                                              float* ss) {
  constexpr int VEC = RowLoader<T>::VEC;
  MaxSum acc;
  acc.m = -INFINITY;
  acc.s = 0.f;
  const int nvec = vec_ok ? n / VEC : 0;
  for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
    float x[VEC];
    RowLoader<T>::load(row + (size_t)v * VEC, x);
    ms_push_vec<VEC>(acc, x);
  }
  for (int i = nvec * VEC + threadIdx.x; i < n; i += blockDim.x) ms_push(acc, (float)row[i]);
  return ms_block_reduce(acc, sm, ss);
}

__global__ void __launch_bounds__(1024)
log_softmax_f32_kernel(const float* __restrict__ x, float* __restrict__ out, int n, long long x_stride,
                       long long out_stride, bool vec) {
  pdl_trigger();
  pdl_wait();
  __shared__ float sm[32], ss[32];
  const float* row = x + (long long)blockIdx.x * x_stride;
  float* orow = out + (long long)blockIdx.x * out_stride;
  const MaxSum r = row_max_sum<float>(row, n, vec, sm, ss);
  const float lse = logf(r.s);
  // out = x - max - log(sum), in that order, as the reference kernel's third pass.
  if (vec) {
    const int nvec = n >> 2;
    for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
      float4 t = reinterpret_cast<const float4*>(row)[v];
      t.x = t.x - r.m - lse;
      t.y = t.y - r.m - lse;
      t.z = t.z - r.m - lse;
      t.w = t.w - r.m - lse;
      reinterpret_cast<float4*>(orow)[v] = t;
    }
    for (int i = (nvec << 2) + threadIdx.x; i < n; i += blockDim.x) orow[i] = row[i] - r.m - lse;
  } else {
    for (int i = threadIdx.x; i < n; i += blockDim.x) orow[i] = row[i] - r.m - lse;
  }
}

template <typename T>
__global__ void __launch_bounds__(1024)
gather_logprob_kernel(const T* __restrict__ x, const long long* __restrict__ labels,
                      float* __restrict__ out, int n, long long x_stride, long long ignore_index,
                      bool vec) {
  pdl_trigger();
  pdl_wait();
  __shared__ float sm[32], ss[32];
  const T* row = x + (long long)blockIdx.x * x_stride;
  const long long label = labels[blockIdx.x];
  const MaxSum r = row_max_sum<T>(row, n, vec, sm, ss);
  if (threadIdx.x == 0) {
    float lp = 0.f;  // ignored labels produce a zero loss in the reference kernel
    if (label != ignore_index && label >= 0 && label < n) {
      const float lse = logf(r.s) + r.m;
      lp = (float)row[label] - lse;
    }
    out[blockIdx.x] = lp;
  }
}

// Gradient of gather_logprob_kernel with respect to the logits (flash-attn's cross-entropy backward with the sign
// of a log-probability, flash_attn/ops/triton/cross_entropy.py): dx[i] = g * ((i == label) - exp(x[i] - lse)),
// a zero row for an ignored label.  The (max, sum) walk is the forward's, so lse has the forward's bits.
template <typename T>
__global__ void __launch_bounds__(1024)
gather_logprob_backward_kernel(const T* __restrict__ x, const long long* __restrict__ labels,
                               const float* __restrict__ grad_out, T* __restrict__ dx, int n, long long x_stride,
                               long long dx_stride, long long ignore_index, bool vec) {
  pdl_trigger();
  pdl_wait();
  __shared__ float sm[32], ss[32];
  const T* row = x + (long long)blockIdx.x * x_stride;
  T* drow = dx + (long long)blockIdx.x * dx_stride;
  const long long label = labels[blockIdx.x];
  const MaxSum r = row_max_sum<T>(row, n, vec, sm, ss);
  const bool live = label != ignore_index && label >= 0 && label < n;
  const float lse = logf(r.s) + r.m, g = live ? grad_out[blockIdx.x] : 0.f;
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const float xi = (float)row[i];      // read before the write: dx may be x itself (inplace_backward)
    drow[i] = (T)(live ? g * ((i == label ? 1.f : 0.f) - expf(xi - lse)) : 0.f);
  }
}

// Greedy token and its log-probability in one pass over a row of logits: argmax (lowest index on
// ties, as torch.argmax) and logprob = max - logsumexp = -log(sum exp(x - max)).  Replaces the
// torch.argmax + cross-entropy pair of Inferencer._select_tokens (inferencer.py:393-449) for greedy
// decoding; the log-probability has the same bits as gather_logprob_kernel given the same label.
template <typename T>
__global__ void __launch_bounds__(1024)
greedy_logprob_kernel(const T* __restrict__ x, long long* __restrict__ tokens, float* __restrict__ logprobs,
                      int n, long long x_stride, bool vec) {
  pdl_trigger();
  pdl_wait();
  __shared__ float sm[32], ss[32];
  __shared__ int si[32];
  const T* row = x + (long long)blockIdx.x * x_stride;
  // One pass: the (max, sum) walk of row_max_sum, element for element, plus this thread's first
  // index of its own maximum (a thread's indices ascend, so `>` keeps the lowest one).
  constexpr int VEC = RowLoader<T>::VEC;
  MaxSum acc;
  acc.m = -INFINITY;
  acc.s = 0.f;
  float bm = -INFINITY;
  int bi = 0x7fffffff;
  const int nvec = vec ? n / VEC : 0;
  for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
    float xv[VEC];
    RowLoader<T>::load(row + (size_t)v * VEC, xv);
    ms_push_vec<VEC>(acc, xv);
#pragma unroll
    for (int j = 0; j < VEC; ++j)
      if (xv[j] > bm) {
        bm = xv[j];
        bi = v * VEC + j;
      }
  }
  for (int i = nvec * VEC + threadIdx.x; i < n; i += blockDim.x) {
    const float xi = (float)row[i];
    ms_push(acc, xi);
    if (xi > bm) {
      bm = xi;
      bi = i;
    }
  }
  const MaxSum r = ms_block_reduce(acc, sm, ss);
  int best = (bm == r.m) ? bi : 0x7fffffff;  // lowest index holding the row maximum
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) best = min(best, __shfl_xor_sync(0xffffffffu, best, o));
  __syncthreads();
  if (lane == 0) si[warp] = best;
  __syncthreads();
  if (warp == 0) {
    int b = lane < (int)(blockDim.x >> 5) ? si[lane] : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) b = min(b, __shfl_xor_sync(0xffffffffu, b, o));
    if (lane == 0) {
      if (b == 0x7fffffff) b = 0;  // a row without any value above -inf
      tokens[blockIdx.x] = b;
      const float lse = logf(r.s) + r.m;
      logprobs[blockIdx.x] = (float)row[b] - lse;
    }
  }
}

}  // namespace b200

extern "C" int b200_log_softmax_f32(const void* x, void* out, long long rows, int n, long long x_row_stride,
                                    long long out_row_stride, void* stream) {
  using namespace b200;
  if (!x || !out || rows < 0 || n <= 0) return B200_ERR_ARG;
  if (rows == 0) return B200_OK;
  const bool vec = ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(out)) & 15) == 0 &&
                   x_row_stride % 4 == 0 && out_row_stride % 4 == 0;
  launch_k(log_softmax_f32_kernel, dim3((unsigned)rows), dim3(1024), 0, (cudaStream_t)stream, 
      (const float*)x, (float*)out, n, x_row_stride, out_row_stride, vec);
  return launch_status();
}

extern "C" int b200_gather_logprob(const void* logits, const void* labels, void* out, long long rows, int n,
                                   long long row_stride, int dtype /*0 = f32, 1 = bf16*/,
                                   long long ignore_index, void* stream) {
  using namespace b200;
  if (!logits || !labels || !out || rows < 0 || n <= 0) return B200_ERR_ARG;
  if (rows == 0) return B200_OK;
  cudaStream_t st = (cudaStream_t)stream;
  const bool aligned = (reinterpret_cast<uintptr_t>(logits) & 15) == 0;
  if (dtype == 0) {
    launch_k(gather_logprob_kernel<float>, dim3((unsigned)rows), dim3(1024), 0, st, 
        (const float*)logits, (const long long*)labels, (float*)out, n, row_stride, ignore_index,
        aligned && row_stride % 4 == 0);
  } else if (dtype == 1) {
    launch_k(gather_logprob_kernel<__nv_bfloat16>, dim3((unsigned)rows), dim3(1024), 0, st, 
        (const __nv_bfloat16*)logits, (const long long*)labels, (float*)out, n, row_stride, ignore_index,
        aligned && row_stride % 8 == 0);
  } else {
    return B200_ERR_ARG;
  }
  return launch_status();
}

// d logprob / d logits for b200_gather_logprob: dlogits[r, i] = grad_out[r] * ((i == label[r]) - softmax(logits[r])[i])
// in the logits' dtype; dlogits may alias logits (rows are processed after their statistics are known).
extern "C" int b200_gather_logprob_backward(const void* logits, const void* labels, const void* grad_out_f32,
                                            void* dlogits, long long rows, int n, long long row_stride,
                                            long long d_row_stride, int dtype /*0 = f32, 1 = bf16*/,
                                            long long ignore_index, void* stream) {
  using namespace b200;
  if (!logits || !labels || !grad_out_f32 || !dlogits || rows < 0 || n <= 0) return B200_ERR_ARG;
  if (rows == 0) return B200_OK;
  cudaStream_t st = (cudaStream_t)stream;
  const bool aligned = (reinterpret_cast<uintptr_t>(logits) & 15) == 0;
  if (dtype == 0)
    launch_k(gather_logprob_backward_kernel<float>, dim3((unsigned)rows), dim3(1024), 0, st, (const float*)logits,
             (const long long*)labels, (const float*)grad_out_f32, (float*)dlogits, n, row_stride, d_row_stride,
             ignore_index, aligned && row_stride % 4 == 0);
  else if (dtype == 1)
    launch_k(gather_logprob_backward_kernel<__nv_bfloat16>, dim3((unsigned)rows), dim3(1024), 0, st,
             (const __nv_bfloat16*)logits, (const long long*)labels, (const float*)grad_out_f32,
             (__nv_bfloat16*)dlogits, n, row_stride, d_row_stride, ignore_index, aligned && row_stride % 8 == 0);
  else
    return B200_ERR_ARG;
  return launch_status();
}

extern "C" int b200_greedy_logprob(const void* logits, void* tokens_i64, void* logprobs_f32, long long rows, int n,
                                   long long row_stride, int dtype /*0 = f32, 1 = bf16*/, void* stream) {
  using namespace b200;
  if (!logits || !tokens_i64 || !logprobs_f32 || rows < 0 || n <= 0) return B200_ERR_ARG;
  if (rows == 0) return B200_OK;
  cudaStream_t st = (cudaStream_t)stream;
  const bool aligned = (reinterpret_cast<uintptr_t>(logits) & 15) == 0;
  if (dtype == 0)
    launch_k(greedy_logprob_kernel<float>, dim3((unsigned)rows), dim3(1024), 0, st, (const float*)logits,
             (long long*)tokens_i64, (float*)logprobs_f32, n, row_stride, aligned && row_stride % 4 == 0);
  else if (dtype == 1)
    launch_k(greedy_logprob_kernel<__nv_bfloat16>, dim3((unsigned)rows), dim3(1024), 0, st,
             (const __nv_bfloat16*)logits, (long long*)tokens_i64, (float*)logprobs_f32, n, row_stride,
             aligned && row_stride % 8 == 0);
  else
    return B200_ERR_ARG;
  return launch_status();
}
