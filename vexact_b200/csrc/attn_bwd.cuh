// Backward of the packed (non-paged) causal varlen attention: dq, dk, dv.
//
// Follows vexact/batch_invariant_ops/triton_invariant_attention.py:194-431 (_varlen_attn_bwd_dq_kernel,
// _varlen_attn_bwd_dkv_kernel): per sequence, query i of q_len sits at absolute position i + (kv_len - q_len)
// and sees the keys up to that position;
//   p  = exp(scale * q.k - lse)            delta = sum_d out * dout
//   dv = sum_i bf16(p)^T dout              ds = p * (dout.v - delta) * scale
//   dq = sum_j bf16(ds) k                  dk = sum_i bf16(ds)^T q      (a KV head sums over its query heads)
// with fp32 accumulation and the reference's rounding points (p and ds become bf16 before their products).
// The reference's forward saves the log-sum-exp; this library's forward kernels do not, so the first kernel
// recomputes it (one more pass over the keys) and leaves lse and delta in caller-provided scratch for the second.
//
// This file holds the plain form: 32 x 32 tiles staged in shared memory as fp32, fp32 FMAs on the CUDA cores,
// every sum in a fixed order (key blocks ascending for dq; query heads, then query blocks ascending for dk / dv)
// and no atomics, so gradients are deterministic and a sequence's gradients do not depend on the batch.  It is
// what B200_ATTN_BWD_SIMT=1 runs and what the tensor-core form (attn_bwd_mma.cuh, the default) is checked against.
#pragma once
#include "common.cuh"

namespace b200 {

constexpr int AB_T = 32;          // queries per tile = keys per tile
constexpr int AB_THREADS = 256;   // thread (ty, tx) = (tid / 16, tid % 16)

struct AttnBwdParams {
  const __nv_bfloat16 *q, *k, *v, *out, *dout;   // [total_q, hq, DK], [total_k, hkv, DK], [total_k, hkv, DV], [total_q, hq, DV] x 2
  __nv_bfloat16 *dq, *dk, *dv;
  float *lse, *delta;                            // scratch [total_q, hq]
  const int *cu_q, *cu_k;                        // [num_seqs + 1]
  int hq, hkv;
  long long total_q, total_k;
  float scale;
};

// rows x D bf16 values (row r at src + r * row_stride) -> fp32 tile dst[32][D + 1]; rows past `valid` are zeros.
template <int D>
__device__ __forceinline__ void ab_load_tile(float* dst, const __nv_bfloat16* src, long long row_stride, int valid) {
  for (int e = threadIdx.x; e < AB_T * D / 2; e += AB_THREADS) {
    const int r = e / (D / 2), c = (e % (D / 2)) * 2;
    float a = 0.f, b = 0.f;
    if (r < valid) unpack_bf2(*reinterpret_cast<const uint32_t*>(src + (long long)r * row_stride + c), a, b);
    dst[r * (D + 1) + c] = a;
    dst[r * (D + 1) + c + 1] = b;
  }
}

// s[a][b] = A[i0 + a, :] . B[j0 + b, :] over D columns of two [32][D + 1] tiles.
template <int D>
__device__ __forceinline__ void ab_dot2x2(const float* A, const float* B, int i0, int j0, float (&s)[2][2]) {
  s[0][0] = s[0][1] = s[1][0] = s[1][1] = 0.f;
  const float* a0 = A + i0 * (D + 1);
  const float* b0 = B + j0 * (D + 1);
#pragma unroll 8
  for (int d = 0; d < D; ++d) {
    const float x0 = a0[d], x1 = a0[D + 1 + d], y0 = b0[d], y1 = b0[D + 1 + d];
    s[0][0] = fmaf(x0, y0, s[0][0]);
    s[0][1] = fmaf(x0, y1, s[0][1]);
    s[1][0] = fmaf(x1, y0, s[1][0]);
    s[1][1] = fmaf(x1, y1, s[1][1]);
  }
}

// Reduction over the 16 threads that share a ty (lanes of one half-warp).
__device__ __forceinline__ float ab_max16(float v) {
#pragma unroll
  for (int o = 8; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float ab_sum16(float v) {
#pragma unroll
  for (int o = 8; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ __forceinline__ bool ab_bounds(const AttnBwdParams& p, int seq, int& q0, int& q_len, int& k0, int& kv_len) {
  q0 = p.cu_q[seq];
  k0 = p.cu_k[seq];
  const int q1 = p.cu_q[seq + 1], k1 = p.cu_k[seq + 1];
  q_len = q1 - q0;
  kv_len = k1 - k0;
  if (q0 < 0 || k0 < 0 || q_len < 0 || kv_len < 0 || q1 > p.total_q || k1 > p.total_k) {
    if (threadIdx.x == 0 && blockIdx.x == 0 && blockIdx.y == 0) report_status(B200_STATUS_BAD_INDEX, seq);
    return false;
  }
  return true;
}

// Grid (query tiles, query heads, sequences).  Writes lse, delta and dq of its 32 queries.
template <int DK, int DV>
__global__ void __launch_bounds__(AB_THREADS) attn_bwd_dq_kernel(const AttnBwdParams p) {
  pdl_trigger();
  pdl_wait();
  extern __shared__ float ab_smem[];
  float* sQ = ab_smem;                      // [32][DK + 1]
  float* sK = sQ + AB_T * (DK + 1);         // [32][DK + 1]
  float* sV = sK + AB_T * (DK + 1);         // [32][DV + 1]
  float* sDO = sV + AB_T * (DV + 1);        // [32][DV + 1]
  float* sDS = sDO + AB_T * (DV + 1);       // [32][33]
  float* sDelta = sDS + AB_T * (AB_T + 1);  // [32]
  const int seq = blockIdx.z, h = blockIdx.y, m0 = blockIdx.x * AB_T;
  int q0, q_len, k0, kv_len;
  if (!ab_bounds(p, seq, q0, q_len, k0, kv_len)) return;
  if (blockIdx.x == gridDim.x - 1 && q_len > (int)gridDim.x * AB_T && threadIdx.x == 0 && h == 0)
    report_status(B200_STATUS_BAD_INDEX, seq);          // more queries than the grid was sized for
  if (m0 >= q_len) return;
  const int rows = min(AB_T, q_len - m0);
  const int kvh = h / (p.hq / p.hkv);
  const int shift = kv_len - q_len;                     // query i sees keys j <= i + shift
  const int tid = threadIdx.x, ty = tid >> 4, tx = tid & 15, i0 = 2 * ty, j0 = 2 * tx;
  const long long qrow = (long long)p.hq * DK, orow = (long long)p.hq * DV;
  const long long krow = (long long)p.hkv * DK, vrow = (long long)p.hkv * DV;
  const __nv_bfloat16* qb = p.q + ((long long)(q0 + m0) * p.hq + h) * DK;
  const __nv_bfloat16* dob = p.dout + ((long long)(q0 + m0) * p.hq + h) * DV;
  const __nv_bfloat16* ob = p.out + ((long long)(q0 + m0) * p.hq + h) * DV;
  ab_load_tile<DK>(sQ, qb, qrow, rows);
  ab_load_tile<DV>(sDO, dob, orow, rows);
  {   // delta: warp w takes rows 4w .. 4w + 3
    const int warp = tid >> 5, lane = tid & 31;
    for (int r = warp * 4; r < warp * 4 + 4; ++r) {
      float acc = 0.f;
      if (r < rows)
        for (int d = lane; d < DV; d += 32) acc += bf2f(ob[(long long)r * orow + d]) * bf2f(dob[(long long)r * orow + d]);
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
      if (lane == 0) sDelta[r] = acc;
    }
  }
  __syncthreads();
  const int n_end = min(kv_len, m0 + rows + shift);     // keys any query of this tile can see
  // ---- pass 1: log-sum-exp of the scaled scores of every row
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
  for (int n0 = 0; n0 < n_end; n0 += AB_T) {
    ab_load_tile<DK>(sK, p.k + ((long long)(k0 + n0) * p.hkv + kvh) * DK, krow, min(AB_T, kv_len - n0));
    __syncthreads();
    float s[2][2];
    ab_dot2x2<DK>(sQ, sK, i0, j0, s);
#pragma unroll
    for (int a = 0; a < 2; ++a) {
      const int i = m0 + i0 + a;
      float bm = -INFINITY;
#pragma unroll
      for (int b = 0; b < 2; ++b) {
        const int j = n0 + j0 + b;
        s[a][b] = (i0 + a < rows && j < kv_len && j <= i + shift) ? s[a][b] * p.scale : -INFINITY;
        bm = fmaxf(bm, s[a][b]);
      }
      bm = ab_max16(bm);
      const float m_new = fmaxf(m_run[a], bm);
      float part = 0.f;
      if (m_new != -INFINITY) {
#pragma unroll
        for (int b = 0; b < 2; ++b) part += s[a][b] == -INFINITY ? 0.f : expf(s[a][b] - m_new);
      }
      part = ab_sum16(part);
      if (m_new != -INFINITY) {
        l_run[a] = (m_run[a] == -INFINITY ? 0.f : l_run[a] * expf(m_run[a] - m_new)) + part;
        m_run[a] = m_new;
      }
    }
    __syncthreads();
  }
  float lse[2], delta[2];
#pragma unroll
  for (int a = 0; a < 2; ++a) {
    lse[a] = l_run[a] > 0.f ? m_run[a] + logf(l_run[a]) : INFINITY;   // a row that sees no key: p = exp(-inf) = 0
    delta[a] = sDelta[i0 + a];
    if (tx == 0 && i0 + a < rows) {
      const long long at = (long long)(q0 + m0 + i0 + a) * p.hq + h;
      p.lse[at] = lse[a];
      p.delta[at] = delta[a];
    }
  }
  // ---- pass 2: dq
  float acc[2][DK / 16];
#pragma unroll
  for (int a = 0; a < 2; ++a)
#pragma unroll
    for (int c = 0; c < DK / 16; ++c) acc[a][c] = 0.f;
  for (int n0 = 0; n0 < n_end; n0 += AB_T) {
    const int kvalid = min(AB_T, kv_len - n0);
    ab_load_tile<DK>(sK, p.k + ((long long)(k0 + n0) * p.hkv + kvh) * DK, krow, kvalid);
    ab_load_tile<DV>(sV, p.v + ((long long)(k0 + n0) * p.hkv + kvh) * DV, vrow, kvalid);
    __syncthreads();
    float s[2][2], dp[2][2];
    ab_dot2x2<DK>(sQ, sK, i0, j0, s);
    ab_dot2x2<DV>(sDO, sV, i0, j0, dp);
#pragma unroll
    for (int a = 0; a < 2; ++a) {
      const int i = m0 + i0 + a;
#pragma unroll
      for (int b = 0; b < 2; ++b) {
        const int j = n0 + j0 + b;
        const bool on = i0 + a < rows && j < kv_len && j <= i + shift;
        const float pr = on ? expf(s[a][b] * p.scale - lse[a]) : 0.f;
        sDS[(i0 + a) * (AB_T + 1) + j0 + b] = round_bf(pr * (dp[a][b] - delta[a]) * p.scale);
      }
    }
    __syncthreads();
    for (int j = 0; j < AB_T; ++j) {
      const float d0 = sDS[i0 * (AB_T + 1) + j], d1 = sDS[(i0 + 1) * (AB_T + 1) + j];
#pragma unroll
      for (int c = 0; c < DK / 16; ++c) {
        const float kv = sK[j * (DK + 1) + tx + 16 * c];
        acc[0][c] = fmaf(d0, kv, acc[0][c]);
        acc[1][c] = fmaf(d1, kv, acc[1][c]);
      }
    }
    __syncthreads();
  }
#pragma unroll
  for (int a = 0; a < 2; ++a) {
    if (i0 + a >= rows) continue;
    __nv_bfloat16* dst = p.dq + ((long long)(q0 + m0 + i0 + a) * p.hq + h) * DK;
#pragma unroll
    for (int c = 0; c < DK / 16; ++c) dst[tx + 16 * c] = f2bf(acc[a][c]);
  }
}

// Grid (key tiles, KV heads, sequences).  Writes dk and dv of its 32 keys; reads lse and delta.
template <int DK, int DV>
__global__ void __launch_bounds__(AB_THREADS) attn_bwd_dkv_kernel(const AttnBwdParams p) {
  pdl_trigger();
  pdl_wait();
  extern __shared__ float ab_smem[];
  float* sQ = ab_smem;                      // [32][DK + 1]
  float* sK = sQ + AB_T * (DK + 1);
  float* sV = sK + AB_T * (DK + 1);         // [32][DV + 1]
  float* sDO = sV + AB_T * (DV + 1);
  float* sP = sDO + AB_T * (DV + 1);        // [32 queries][33]
  float* sDS = sP + AB_T * (AB_T + 1);
  float* sL = sDS + AB_T * (AB_T + 1);      // [32]
  float* sD = sL + AB_T;                    // [32]
  const int seq = blockIdx.z, kvh = blockIdx.y, n0 = blockIdx.x * AB_T;
  int q0, q_len, k0, kv_len;
  if (!ab_bounds(p, seq, q0, q_len, k0, kv_len)) return;
  if (blockIdx.x == gridDim.x - 1 && kv_len > (int)gridDim.x * AB_T && threadIdx.x == 0 && kvh == 0)
    report_status(B200_STATUS_BAD_INDEX, seq);          // more keys than the grid was sized for
  if (n0 >= kv_len) return;
  const int kvalid = min(AB_T, kv_len - n0);
  const int group = p.hq / p.hkv;
  const int shift = kv_len - q_len;
  const int tid = threadIdx.x, ty = tid >> 4, tx = tid & 15, i0 = 2 * ty, j0 = 2 * tx;
  const long long qrow = (long long)p.hq * DK, orow = (long long)p.hq * DV;
  const long long krow = (long long)p.hkv * DK, vrow = (long long)p.hkv * DV;
  ab_load_tile<DK>(sK, p.k + ((long long)(k0 + n0) * p.hkv + kvh) * DK, krow, kvalid);
  ab_load_tile<DV>(sV, p.v + ((long long)(k0 + n0) * p.hkv + kvh) * DV, vrow, kvalid);
  float adk[2][DK / 16], adv[2][DV / 16];               // key rows 2 ty, 2 ty + 1; columns tx + 16 c
#pragma unroll
  for (int a = 0; a < 2; ++a) {
#pragma unroll
    for (int c = 0; c < DK / 16; ++c) adk[a][c] = 0.f;
#pragma unroll
    for (int c = 0; c < DV / 16; ++c) adv[a][c] = 0.f;
  }
  const int i_first = max(0, n0 - shift);               // first query that sees key n0
  for (int g = 0; g < group; ++g) {
    const int h = kvh * group + g;
    for (int m0 = (i_first / AB_T) * AB_T; m0 < q_len; m0 += AB_T) {
      const int rows = min(AB_T, q_len - m0);
      __syncthreads();                                  // the previous tile's products are done
      ab_load_tile<DK>(sQ, p.q + ((long long)(q0 + m0) * p.hq + h) * DK, qrow, rows);
      ab_load_tile<DV>(sDO, p.dout + ((long long)(q0 + m0) * p.hq + h) * DV, orow, rows);
      if (tid < AB_T) {
        const long long at = (long long)(q0 + m0 + tid) * p.hq + h;
        sL[tid] = tid < rows ? p.lse[at] : INFINITY;
        sD[tid] = tid < rows ? p.delta[at] : 0.f;
      }
      __syncthreads();
      float s[2][2], dp[2][2];
      ab_dot2x2<DK>(sQ, sK, i0, j0, s);
      ab_dot2x2<DV>(sDO, sV, i0, j0, dp);
#pragma unroll
      for (int a = 0; a < 2; ++a) {
        const int i = m0 + i0 + a;
#pragma unroll
        for (int b = 0; b < 2; ++b) {
          const int j = n0 + j0 + b;
          const bool on = i0 + a < rows && j0 + b < kvalid && j <= i + shift;
          const float pr = on ? expf(s[a][b] * p.scale - sL[i0 + a]) : 0.f;
          sP[(i0 + a) * (AB_T + 1) + j0 + b] = round_bf(pr);
          sDS[(i0 + a) * (AB_T + 1) + j0 + b] = round_bf(pr * (dp[a][b] - sD[i0 + a]) * p.scale);
        }
      }
      __syncthreads();
      for (int i = 0; i < AB_T; ++i) {                  // this thread's two keys are tile columns 2 ty, 2 ty + 1
        const float p0 = sP[i * (AB_T + 1) + i0], p1 = sP[i * (AB_T + 1) + i0 + 1];
        const float d0 = sDS[i * (AB_T + 1) + i0], d1 = sDS[i * (AB_T + 1) + i0 + 1];
#pragma unroll
        for (int c = 0; c < DV / 16; ++c) {
          const float x = sDO[i * (DV + 1) + tx + 16 * c];
          adv[0][c] = fmaf(p0, x, adv[0][c]);
          adv[1][c] = fmaf(p1, x, adv[1][c]);
        }
#pragma unroll
        for (int c = 0; c < DK / 16; ++c) {
          const float x = sQ[i * (DK + 1) + tx + 16 * c];
          adk[0][c] = fmaf(d0, x, adk[0][c]);
          adk[1][c] = fmaf(d1, x, adk[1][c]);
        }
      }
    }
  }
#pragma unroll
  for (int a = 0; a < 2; ++a) {
    if (i0 + a >= kvalid) continue;
    __nv_bfloat16* dkp = p.dk + ((long long)(k0 + n0 + i0 + a) * p.hkv + kvh) * DK;
    __nv_bfloat16* dvp = p.dv + ((long long)(k0 + n0 + i0 + a) * p.hkv + kvh) * DV;
#pragma unroll
    for (int c = 0; c < DK / 16; ++c) dkp[tx + 16 * c] = f2bf(adk[a][c]);
#pragma unroll
    for (int c = 0; c < DV / 16; ++c) dvp[tx + 16 * c] = f2bf(adv[a][c]);
  }
}

template <int DK, int DV>
inline int attn_bwd_launch(const AttnBwdParams& p, int num_seqs, int max_seqlen_q, int max_seqlen_k, cudaStream_t st) {
  const int smem_dq = (2 * AB_T * (DK + 1) + 2 * AB_T * (DV + 1) + AB_T * (AB_T + 1) + AB_T) * (int)sizeof(float);
  const int smem_dkv = (2 * AB_T * (DK + 1) + 2 * AB_T * (DV + 1) + 2 * AB_T * (AB_T + 1) + 2 * AB_T) * (int)sizeof(float);
  static PerDeviceFlags set_dq, set_dkv;
  if (int rc = set_max_dyn_smem_once(set_dq, attn_bwd_dq_kernel<DK, DV>, smem_dq)) return rc;
  if (int rc = set_max_dyn_smem_once(set_dkv, attn_bwd_dkv_kernel<DK, DV>, smem_dkv)) return rc;
  const unsigned qt = (unsigned)((max_seqlen_q + AB_T - 1) / AB_T), kt = (unsigned)((max_seqlen_k + AB_T - 1) / AB_T);
  launch_k(attn_bwd_dq_kernel<DK, DV>, dim3(qt, (unsigned)p.hq, (unsigned)num_seqs), dim3(AB_THREADS), (size_t)smem_dq,
           st, p);
  if (int rc = launch_status()) return rc;
  launch_k(attn_bwd_dkv_kernel<DK, DV>, dim3(kt, (unsigned)p.hkv, (unsigned)num_seqs), dim3(AB_THREADS),
           (size_t)smem_dkv, st, p);
  return launch_status();
}

}  // namespace b200
