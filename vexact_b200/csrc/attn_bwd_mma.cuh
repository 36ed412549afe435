// The backward of attn_bwd.cuh on the tensor cores (mma.sync m16n8k16, bf16 x bf16 -> fp32): the same two kernels,
// the same arithmetic (p = exp(scale * q.k - lse), ds = p * (dout.v - delta) * scale, p and ds rounded to bf16 before
// their products, fp32 accumulation), tiles staged in shared memory as bf16 and read with ldmatrix.
//
//   dq kernel:  a CTA owns 64 queries of one head (16 per warp) and walks the keys 64 at a time:
//               S = Q K^T and dP = dO V^T with K / V rows as the n operand, then dQ += bf16(dS) K with K read
//               through a transposing ldmatrix.  A first walk over the keys gives the log-sum-exp.
//   dkv kernel: a CTA owns 64 keys of one KV head (16 per warp) and walks its query heads and their queries 32 at a
//               time with the roles swapped: S^T = K Q^T, dP^T = V dO^T, dV += bf16(P^T) dO, dK += bf16(dS^T) Q.
//
// Every sum runs in a fixed order (key tiles ascending; heads, then query tiles ascending) with the instruction's
// own order inside a 16-wide step, no atomics: deterministic, and independent of the batch.
#pragma once
#include "attn.cuh"       // ldmatrix_x4, ldmatrix_x4_trans, mma_bf16_16816
#include "attn_bwd.cuh"   // AttnBwdParams, ab_bounds
#include "gemm.cuh"       // env_int

namespace b200 {

constexpr int ABM_THREADS = 128;   // 4 warps
constexpr int ABM_PAD = 8;         // bf16 elements of padding per tile row: ldmatrix rows land in distinct banks

// rows x D bf16 (row r at src + r * row_stride) -> tile dst[R][D + 8]; rows past `valid` are zeros.
template <int D, int R>
__device__ __forceinline__ void abm_load(__nv_bfloat16* dst, const __nv_bfloat16* src, long long row_stride, int valid) {
  constexpr int VPR = D / 8;
  for (int e = threadIdx.x; e < R * VPR; e += ABM_THREADS) {
    const int r = e / VPR, c = (e % VPR) * 8;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (r < valid) v = *reinterpret_cast<const uint4*>(src + (long long)r * row_stride + c);
    *reinterpret_cast<uint4*>(dst + r * (D + ABM_PAD) + c) = v;
  }
}

// A fragment: rows r0 .. r0 + 15, columns k0 .. k0 + 15 of a [rows][ld] tile.
__device__ __forceinline__ void abm_frag_a(uint32_t base, int ld, int r0, int k0, int lane, uint32_t (&a)[4]) {
  ldmatrix_x4(base + (uint32_t)((r0 + (lane & 15)) * ld + k0 + (lane >> 4) * 8) * 2, a[0], a[1], a[2], a[3]);
}
// B fragments of two n8 tiles whose n index is the tile's ROW (rows n0 .. n0 + 15), k = columns k0 .. k0 + 15.
// b[0], b[1] belong to rows n0 .. n0 + 7, b[2], b[3] to rows n0 + 8 .. n0 + 15.
__device__ __forceinline__ void abm_frag_b_rows(uint32_t base, int ld, int n0, int k0, int lane, uint32_t (&b)[4]) {
  ldmatrix_x4(base + (uint32_t)((n0 + (lane & 7) + (lane >> 4) * 8) * ld + k0 + ((lane >> 3) & 1) * 8) * 2, b[0], b[1],
              b[2], b[3]);
}
// B fragments of two n8 tiles whose n index is the tile's COLUMN (columns n0 .. n0 + 15), k = rows k0 .. k0 + 15.
__device__ __forceinline__ void abm_frag_b_cols(uint32_t base, int ld, int k0, int n0, int lane, uint32_t (&b)[4]) {
  ldmatrix_x4_trans(base + (uint32_t)((k0 + (lane & 7) + ((lane >> 3) & 1) * 8) * ld + n0 + (lane >> 4) * 8) * 2, b[0],
                    b[1], b[2], b[3]);
}

__device__ __forceinline__ float abm_quad_max(float v) {
  v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 1));
  return fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 2));
}
__device__ __forceinline__ float abm_quad_sum(float v) {
  v += __shfl_xor_sync(0xffffffffu, v, 1);
  return v + __shfl_xor_sync(0xffffffffu, v, 2);
}

// acc[NT][4] (16 rows x NT * 8 columns) = X[r0 .. r0 + 15, 0 .. D) . Y[0 .. NT * 8, 0 .. D)^T.
template <int D, int NT>
__device__ __forceinline__ void abm_rows_dot(uint32_t x_base, uint32_t y_base, int r0, int lane, float (&acc)[NT][4]) {
#pragma unroll
  for (int j = 0; j < NT; ++j)
#pragma unroll
    for (int e = 0; e < 4; ++e) acc[j][e] = 0.f;
#pragma unroll
  for (int kk = 0; kk < D / 16; ++kk) {
    uint32_t a[4];
    abm_frag_a(x_base, D + ABM_PAD, r0, kk * 16, lane, a);
#pragma unroll
    for (int jp = 0; jp < NT / 2; ++jp) {
      uint32_t b[4];
      abm_frag_b_rows(y_base, D + ABM_PAD, jp * 16, kk * 16, lane, b);
      mma_bf16_16816(acc[2 * jp], a[0], a[1], a[2], a[3], b[0], b[1]);
      mma_bf16_16816(acc[2 * jp + 1], a[0], a[1], a[2], a[3], b[2], b[3]);
    }
  }
}

// out[D / 8][4] (16 rows x D columns) += W[16 rows x KS * 16] . Y[0 .. KS * 16, 0 .. D), W given as A fragments.
template <int D, int KS>
__device__ __forceinline__ void abm_accumulate(uint32_t y_base, int lane, const uint32_t (&w)[KS][4], float (&out)[D / 8][4]) {
#pragma unroll
  for (int np = 0; np < D / 16; ++np)
#pragma unroll
    for (int ks = 0; ks < KS; ++ks) {
      uint32_t b[4];
      abm_frag_b_cols(y_base, D + ABM_PAD, ks * 16, np * 16, lane, b);
      mma_bf16_16816(out[2 * np], w[ks][0], w[ks][1], w[ks][2], w[ks][3], b[0], b[1]);
      mma_bf16_16816(out[2 * np + 1], w[ks][0], w[ks][1], w[ks][2], w[ks][3], b[2], b[3]);
    }
}

// Grid (query tiles of 64, query heads, sequences).  Writes lse, delta and dq of its queries.
template <int DK, int DV>
__global__ void __launch_bounds__(ABM_THREADS) attn_bwd_dq_mma_kernel(const AttnBwdParams p) {
  pdl_trigger();
  pdl_wait();
  extern __shared__ __align__(16) unsigned char abm_smem[];
  __nv_bfloat16* sQ = reinterpret_cast<__nv_bfloat16*>(abm_smem);   // [64][DK + 8]
  __nv_bfloat16* sDO = sQ + 64 * (DK + ABM_PAD);                      // [64][DV + 8]
  __nv_bfloat16* sK = sDO + 64 * (DV + ABM_PAD);                      // [64][DK + 8]
  __nv_bfloat16* sV = sK + 64 * (DK + ABM_PAD);                       // [64][DV + 8]
  float* sDelta = reinterpret_cast<float*>(sV + 64 * (DV + ABM_PAD)); // [64]
  const int seq = blockIdx.z, h = blockIdx.y, m0 = blockIdx.x * 64;
  int q0, q_len, k0, kv_len;
  if (!ab_bounds(p, seq, q0, q_len, k0, kv_len)) return;
  if (blockIdx.x == gridDim.x - 1 && q_len > (int)gridDim.x * 64 && threadIdx.x == 0 && h == 0)
    report_status(B200_STATUS_BAD_INDEX, seq);
  if (m0 >= q_len) return;
  const int rows = min(64, q_len - m0);
  const int kvh = h / (p.hq / p.hkv);
  const int shift = kv_len - q_len;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, gid = lane >> 2, tig = lane & 3;
  const long long qrow = (long long)p.hq * DK, orow = (long long)p.hq * DV;
  const long long krow = (long long)p.hkv * DK, vrow = (long long)p.hkv * DV;
  const __nv_bfloat16* dob = p.dout + ((long long)(q0 + m0) * p.hq + h) * DV;
  const __nv_bfloat16* ob = p.out + ((long long)(q0 + m0) * p.hq + h) * DV;
  abm_load<DK, 64>(sQ, p.q + ((long long)(q0 + m0) * p.hq + h) * DK, qrow, rows);
  abm_load<DV, 64>(sDO, dob, orow, rows);
  for (int r = warp * 16; r < warp * 16 + 16; ++r) {     // delta of the warp's own 16 rows
    float acc = 0.f;
    if (r < rows)
      for (int d = lane; d < DV; d += 32) acc += bf2f(ob[(long long)r * orow + d]) * bf2f(dob[(long long)r * orow + d]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if (lane == 0) sDelta[r] = acc;
  }
  __syncthreads();
  const uint32_t q_base = (uint32_t)__cvta_generic_to_shared(sQ), do_base = (uint32_t)__cvta_generic_to_shared(sDO);
  const uint32_t k_base = (uint32_t)__cvta_generic_to_shared(sK), v_base = (uint32_t)__cvta_generic_to_shared(sV);
  const int wq = warp * 16;
  const int row_of[2] = {wq + gid, wq + gid + 8};         // the two tile rows this thread's fragments cover
  const int n_end = min(kv_len, m0 + rows + shift);
  // scores of one 64-key tile, scaled and masked (-inf where the query does not see the key)
  auto scores = [&](int n0, float (&s)[8][4]) {
    abm_rows_dot<DK, 8>(q_base, k_base, wq, lane, s);
#pragma unroll
    for (int j = 0; j < 8; ++j)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int r = row_of[e >> 1], key = n0 + j * 8 + 2 * tig + (e & 1);
        s[j][e] = (r < rows && key < kv_len && key <= m0 + r + shift) ? s[j][e] * p.scale : -INFINITY;
      }
  };
  // ---- pass 1: log-sum-exp per row
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
  for (int n0 = 0; n0 < n_end; n0 += 64) {
    __syncthreads();
    abm_load<DK, 64>(sK, p.k + ((long long)(k0 + n0) * p.hkv + kvh) * DK, krow, min(64, kv_len - n0));
    __syncthreads();
    float s[8][4];
    scores(n0, s);
#pragma unroll
    for (int a = 0; a < 2; ++a) {
      float bm = -INFINITY;
#pragma unroll
      for (int j = 0; j < 8; ++j) bm = fmaxf(bm, fmaxf(s[j][2 * a], s[j][2 * a + 1]));
      bm = abm_quad_max(bm);
      const float m_new = fmaxf(m_run[a], bm);
      float part = 0.f;
      if (m_new != -INFINITY) {
#pragma unroll
        for (int j = 0; j < 8; ++j)
#pragma unroll
          for (int e = 0; e < 2; ++e) part += s[j][2 * a + e] == -INFINITY ? 0.f : expf(s[j][2 * a + e] - m_new);
      }
      part = abm_quad_sum(part);
      if (m_new != -INFINITY) {
        l_run[a] = (m_run[a] == -INFINITY ? 0.f : l_run[a] * expf(m_run[a] - m_new)) + part;
        m_run[a] = m_new;
      }
    }
  }
  float lse[2], delta[2];
#pragma unroll
  for (int a = 0; a < 2; ++a) {
    lse[a] = l_run[a] > 0.f ? m_run[a] + logf(l_run[a]) : INFINITY;
    delta[a] = sDelta[row_of[a]];
    if (tig == 0 && row_of[a] < rows) {
      const long long at = (long long)(q0 + m0 + row_of[a]) * p.hq + h;
      p.lse[at] = lse[a];
      p.delta[at] = delta[a];
    }
  }
  // ---- pass 2: dq
  float acc[DK / 8][4];
#pragma unroll
  for (int j = 0; j < DK / 8; ++j)
#pragma unroll
    for (int e = 0; e < 4; ++e) acc[j][e] = 0.f;
  for (int n0 = 0; n0 < n_end; n0 += 64) {
    const int kvalid = min(64, kv_len - n0);
    __syncthreads();
    abm_load<DK, 64>(sK, p.k + ((long long)(k0 + n0) * p.hkv + kvh) * DK, krow, kvalid);
    abm_load<DV, 64>(sV, p.v + ((long long)(k0 + n0) * p.hkv + kvh) * DV, vrow, kvalid);
    __syncthreads();
    float s[8][4], dp[8][4];
    scores(n0, s);
    abm_rows_dot<DV, 8>(do_base, v_base, wq, lane, dp);
    uint32_t ds[4][4];                                     // bf16 dS as A fragments, one per 16 keys
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float d[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float pr = s[j][e] == -INFINITY ? 0.f : expf(s[j][e] - lse[e >> 1]);
        d[e] = pr * (dp[j][e] - delta[e >> 1]) * p.scale;
      }
      ds[j >> 1][(j & 1) * 2] = pack_bf2(d[0], d[1]);       // rows gid
      ds[j >> 1][(j & 1) * 2 + 1] = pack_bf2(d[2], d[3]);   // rows gid + 8
    }
    abm_accumulate<DK, 4>(k_base, lane, ds, acc);
  }
#pragma unroll
  for (int a = 0; a < 2; ++a) {
    if (row_of[a] >= rows) continue;
    __nv_bfloat16* dst = p.dq + ((long long)(q0 + m0 + row_of[a]) * p.hq + h) * DK;
#pragma unroll
    for (int j = 0; j < DK / 8; ++j)
      *reinterpret_cast<uint32_t*>(dst + j * 8 + 2 * tig) = pack_bf2(acc[j][2 * a], acc[j][2 * a + 1]);
  }
}

// Grid (key tiles of 64, KV heads, sequences).  Writes dk and dv of its keys; reads lse and delta.
template <int DK, int DV>
__global__ void __launch_bounds__(ABM_THREADS) attn_bwd_dkv_mma_kernel(const AttnBwdParams p) {
  pdl_trigger();
  pdl_wait();
  extern __shared__ __align__(16) unsigned char abm_smem[];
  __nv_bfloat16* sK = reinterpret_cast<__nv_bfloat16*>(abm_smem);   // [64][DK + 8]
  __nv_bfloat16* sV = sK + 64 * (DK + ABM_PAD);                       // [64][DV + 8]
  __nv_bfloat16* sQ = sV + 64 * (DV + ABM_PAD);                       // [32][DK + 8]
  __nv_bfloat16* sDO = sQ + 32 * (DK + ABM_PAD);                      // [32][DV + 8]
  float* sL = reinterpret_cast<float*>(sDO + 32 * (DV + ABM_PAD));    // [32]
  float* sD = sL + 32;                                                // [32]
  const int seq = blockIdx.z, kvh = blockIdx.y, n0 = blockIdx.x * 64;
  int q0, q_len, k0, kv_len;
  if (!ab_bounds(p, seq, q0, q_len, k0, kv_len)) return;
  if (blockIdx.x == gridDim.x - 1 && kv_len > (int)gridDim.x * 64 && threadIdx.x == 0 && kvh == 0)
    report_status(B200_STATUS_BAD_INDEX, seq);
  if (n0 >= kv_len) return;
  const int kvalid = min(64, kv_len - n0);
  const int group = p.hq / p.hkv;
  const int shift = kv_len - q_len;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, gid = lane >> 2, tig = lane & 3;
  const long long qrow = (long long)p.hq * DK, orow = (long long)p.hq * DV;
  const long long krow = (long long)p.hkv * DK, vrow = (long long)p.hkv * DV;
  abm_load<DK, 64>(sK, p.k + ((long long)(k0 + n0) * p.hkv + kvh) * DK, krow, kvalid);
  abm_load<DV, 64>(sV, p.v + ((long long)(k0 + n0) * p.hkv + kvh) * DV, vrow, kvalid);
  const uint32_t q_base = (uint32_t)__cvta_generic_to_shared(sQ), do_base = (uint32_t)__cvta_generic_to_shared(sDO);
  const uint32_t k_base = (uint32_t)__cvta_generic_to_shared(sK), v_base = (uint32_t)__cvta_generic_to_shared(sV);
  const int wk = warp * 16;
  const int key_of[2] = {wk + gid, wk + gid + 8};         // tile-local keys of this thread's fragment rows
  float adk[DK / 8][4], adv[DV / 8][4];
#pragma unroll
  for (int j = 0; j < DK / 8; ++j)
#pragma unroll
    for (int e = 0; e < 4; ++e) adk[j][e] = 0.f;
#pragma unroll
  for (int j = 0; j < DV / 8; ++j)
#pragma unroll
    for (int e = 0; e < 4; ++e) adv[j][e] = 0.f;
  const int i_first = max(0, n0 - shift);
  for (int g = 0; g < group; ++g) {
    const int h = kvh * group + g;
    for (int m0 = (i_first / 32) * 32; m0 < q_len; m0 += 32) {
      const int rows = min(32, q_len - m0);
      __syncthreads();
      abm_load<DK, 32>(sQ, p.q + ((long long)(q0 + m0) * p.hq + h) * DK, qrow, rows);
      abm_load<DV, 32>(sDO, p.dout + ((long long)(q0 + m0) * p.hq + h) * DV, orow, rows);
      if (tid < 32) {
        const long long at = (long long)(q0 + m0 + tid) * p.hq + h;
        sL[tid] = tid < rows ? p.lse[at] : INFINITY;
        sD[tid] = tid < rows ? p.delta[at] : 0.f;
      }
      __syncthreads();
      float st[4][4], dpt[4][4];                           // [keys of this warp] x [32 queries]
      abm_rows_dot<DK, 4>(k_base, q_base, wk, lane, st);
      abm_rows_dot<DV, 4>(v_base, do_base, wk, lane, dpt);
      uint32_t pa[2][4], dsa[2][4];                        // bf16 P^T and dS^T as A fragments, one per 16 queries
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float pr[4], d[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int key = key_of[e >> 1], col = j * 8 + 2 * tig + (e & 1);
          const bool on = col < rows && key < kvalid && n0 + key <= m0 + col + shift;
          pr[e] = on ? expf(st[j][e] * p.scale - sL[col]) : 0.f;
          d[e] = pr[e] * (dpt[j][e] - sD[col]) * p.scale;
        }
        pa[j >> 1][(j & 1) * 2] = pack_bf2(pr[0], pr[1]);
        pa[j >> 1][(j & 1) * 2 + 1] = pack_bf2(pr[2], pr[3]);
        dsa[j >> 1][(j & 1) * 2] = pack_bf2(d[0], d[1]);
        dsa[j >> 1][(j & 1) * 2 + 1] = pack_bf2(d[2], d[3]);
      }
      abm_accumulate<DV, 2>(do_base, lane, pa, adv);
      abm_accumulate<DK, 2>(q_base, lane, dsa, adk);
    }
  }
#pragma unroll
  for (int a = 0; a < 2; ++a) {
    if (key_of[a] >= kvalid) continue;
    __nv_bfloat16* dkp = p.dk + ((long long)(k0 + n0 + key_of[a]) * p.hkv + kvh) * DK;
    __nv_bfloat16* dvp = p.dv + ((long long)(k0 + n0 + key_of[a]) * p.hkv + kvh) * DV;
#pragma unroll
    for (int j = 0; j < DK / 8; ++j)
      *reinterpret_cast<uint32_t*>(dkp + j * 8 + 2 * tig) = pack_bf2(adk[j][2 * a], adk[j][2 * a + 1]);
#pragma unroll
    for (int j = 0; j < DV / 8; ++j)
      *reinterpret_cast<uint32_t*>(dvp + j * 8 + 2 * tig) = pack_bf2(adv[j][2 * a], adv[j][2 * a + 1]);
  }
}

template <int DK, int DV>
inline int attn_bwd_mma_launch(const AttnBwdParams& p, int num_seqs, int max_seqlen_q, int max_seqlen_k,
                               cudaStream_t st) {
  const int smem_dq = (2 * 64 * (DK + ABM_PAD) + 2 * 64 * (DV + ABM_PAD)) * 2 + 64 * (int)sizeof(float);
  const int smem_dkv = (96 * (DK + ABM_PAD) + 96 * (DV + ABM_PAD)) * 2 + 64 * (int)sizeof(float);
  static PerDeviceFlags set_dq, set_dkv;
  if (int rc = set_max_dyn_smem_once(set_dq, attn_bwd_dq_mma_kernel<DK, DV>, smem_dq)) return rc;
  if (int rc = set_max_dyn_smem_once(set_dkv, attn_bwd_dkv_mma_kernel<DK, DV>, smem_dkv)) return rc;
  const unsigned qt = (unsigned)((max_seqlen_q + 63) / 64), kt = (unsigned)((max_seqlen_k + 63) / 64);
  launch_k(attn_bwd_dq_mma_kernel<DK, DV>, dim3(qt, (unsigned)p.hq, (unsigned)num_seqs), dim3(ABM_THREADS),
           (size_t)smem_dq, st, p);
  if (int rc = launch_status()) return rc;
  launch_k(attn_bwd_dkv_mma_kernel<DK, DV>, dim3(kt, (unsigned)p.hkv, (unsigned)num_seqs), dim3(ABM_THREADS),
           (size_t)smem_dkv, st, p);
  return launch_status();
}

}  // namespace b200

// dq, dk, dv of packed causal varlen attention (triton_invariant_attention.py:194-431).  All tensors bf16 and
// contiguous: q / dq [total_q, hq, dk_dim], k / dk [total_k, hkv, dk_dim], v / dv [total_k, hkv, dv_dim], out /
// dout [total_q, hq, dv_dim]; cu_seqlens_q / _k [num_seqs + 1] int32; lse / delta: fp32 scratch [total_q, hq].
// (dk_dim, dv_dim) one of (64, 64), (128, 128), (192, 128).  Keys or queries of no sequence keep what dq / dk / dv
// held (pass zero-filled tensors).  Sequences longer than max_seqlen_q / max_seqlen_k are reported (status code 2).
extern "C" int b200_varlen_attn_backward(const void* q, const void* k, const void* v, const void* out, const void* dout,
                                         const void* cu_seqlens_q, const void* cu_seqlens_k, void* dq, void* dk,
                                         void* dv, void* lse_scratch_f32, void* delta_scratch_f32, int num_seqs,
                                         int max_seqlen_q, int max_seqlen_k, long long total_q, long long total_k,
                                         int num_q_heads, int num_kv_heads, int dk_dim, int dv_dim,
                                         float softmax_scale, void* stream) {
  using namespace b200;
  if (!q || !k || !v || !out || !dout || !cu_seqlens_q || !cu_seqlens_k || !dq || !dk || !dv || !lse_scratch_f32 ||
      !delta_scratch_f32 || num_seqs < 0 || max_seqlen_q < 0 || max_seqlen_k < 0 || total_q < 0 || total_k < 0 ||
      num_q_heads <= 0 || num_kv_heads <= 0)
    return B200_ERR_ARG;
  if (num_q_heads % num_kv_heads != 0 || num_seqs > 65535 || num_q_heads > 65535) return B200_ERR_SHAPE;
  if (total_q > 0x7fffffffLL || total_k > 0x7fffffffLL) return B200_ERR_SHAPE;
  if (num_seqs == 0 || max_seqlen_q == 0 || max_seqlen_k == 0) return B200_OK;
  AttnBwdParams p{(const __nv_bfloat16*)q, (const __nv_bfloat16*)k, (const __nv_bfloat16*)v,
                  (const __nv_bfloat16*)out, (const __nv_bfloat16*)dout, (__nv_bfloat16*)dq, (__nv_bfloat16*)dk,
                  (__nv_bfloat16*)dv, (float*)lse_scratch_f32, (float*)delta_scratch_f32, (const int*)cu_seqlens_q,
                  (const int*)cu_seqlens_k, num_q_heads, num_kv_heads, total_q, total_k, softmax_scale};
  cudaStream_t st = (cudaStream_t)stream;
  static const int simt = env_int("B200_ATTN_BWD_SIMT", 0);     // development knob: the CUDA-core kernels
  if (simt) {
    if (dk_dim == 64 && dv_dim == 64) return attn_bwd_launch<64, 64>(p, num_seqs, max_seqlen_q, max_seqlen_k, st);
    if (dk_dim == 128 && dv_dim == 128) return attn_bwd_launch<128, 128>(p, num_seqs, max_seqlen_q, max_seqlen_k, st);
    if (dk_dim == 192 && dv_dim == 128) return attn_bwd_launch<192, 128>(p, num_seqs, max_seqlen_q, max_seqlen_k, st);
    return B200_ERR_SHAPE;
  }
  if (dk_dim == 64 && dv_dim == 64) return attn_bwd_mma_launch<64, 64>(p, num_seqs, max_seqlen_q, max_seqlen_k, st);
  if (dk_dim == 128 && dv_dim == 128) return attn_bwd_mma_launch<128, 128>(p, num_seqs, max_seqlen_q, max_seqlen_k, st);
  if (dk_dim == 192 && dv_dim == 128) return attn_bwd_mma_launch<192, 128>(p, num_seqs, max_seqlen_q, max_seqlen_k, st);
  return B200_ERR_SHAPE;
}
