// Token sampling over a row of logits: temperature, top-k, top-p, exponential-noise arg-max, and the
// chosen token's log-probability, one CTA per row.
//
// Follows the reference's Sampler.batch_sample_token (vexact/inferencer/sampler.py:32-87) with the
// sort-based apply_top_k_top_p (:148-186) and _random_sample (:120-146): x = fp32(logits) / T; keep
// x >= k-th largest; in ascending order mask the prefix whose cumulative softmax mass is <= 1 - p;
// token = argmax softmax(masked x) / q with q ~ Exp(1) supplied by the caller (one draw of
// torch's exponential_(), as the reference makes).  The log-probability is the one
// logprobs_from_logits_flash_attn gives for that token on the raw logits (same bits as
// gather_logprob_kernel).
//
// No sort: thresholds come from three-level radix histograms over an order-preserving 32-bit key
// (counts for top-k, 2^-40 fixed-point probability mass for top-p), so every step is integer-exact
// and deterministic, and a row's result does not depend on the batch.  Where the reference's
// cumulative sum crosses 1 - p inside a run of equal values it masks part of the run (which
// part is its sort's business); this kernel keeps the whole run.
#pragma once
#include "softmax.cuh"

namespace b200 {

constexpr int SMP_THREADS = 1024;
constexpr int SMP_BINS = 2048;

__device__ __forceinline__ uint32_t smp_key(float x) {  // monotone: a < b  <=>  key(a) < key(b)
  const uint32_t u = __float_as_uint(x);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

struct SampleParams {
  const void* logits;
  const float* q;
  long long* tokens;
  float* logprobs;
  int n;
  long long row_stride, q_stride;
  float temperature, top_p;
  int top_k;
  bool vec;
  float* masked_out;       // MASK form: fp32 [rows, n], the scaled logits with everything cut by top-k / top-p at -inf
  long long out_stride;
};

// Digit layout of the three radix levels: bits 31..21, 20..10, 9..0.
__device__ __forceinline__ int smp_shift(int level) { return level == 0 ? 21 : (level == 1 ? 10 : 0); }
__device__ __forceinline__ int smp_bins(int level) { return level == 2 ? 1024 : 2048; }

// MASK = true stops after the two thresholds and writes the masked logits (the reference's apply_top_k_top_p as
// an operator of its own, sampler.py:146-186) instead of drawing a token.
template <typename T, bool MASK = false>
__global__ void __launch_bounds__(SMP_THREADS) sample_token_kernel(const SampleParams p) {
  pdl_trigger();
  pdl_wait();
  __shared__ float sm[32], ss[32];
  __shared__ int si[32];
  __shared__ unsigned hist[SMP_BINS];
  __shared__ unsigned long long mass[SMP_BINS];
  __shared__ unsigned s_pick[2];                // chosen bin, count above it
  __shared__ unsigned long long s_cum;          // mass below the chosen bin
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int n = p.n;
  const T* row = reinterpret_cast<const T*>(p.logits) + (long long)blockIdx.x * p.row_stride;
  const float* qrow = MASK ? nullptr : p.q + (long long)blockIdx.x * p.q_stride;
  const bool has_temp = p.temperature != 1.0f;
  auto scaled = [&](int i) {
    const float x = (float)row[i];
    return has_temp ? __fdiv_rn(x, p.temperature) : x;
  };

  // raw (max, sum exp): the walk of gather_logprob_kernel, for the log-probability
  const MaxSum raw = row_max_sum<T>(row, n, p.vec, sm, ss);
  __syncthreads();
  const float m_t = has_temp ? __fdiv_rn(raw.m, p.temperature) : raw.m;  // division is monotone

  // ---- top-k: key of the k-th largest scaled logit
  uint32_t key_k = 0;  // keep key >= key_k
  if (p.top_k > 0 && p.top_k < n) {
    uint32_t prefix = 0, prefix_mask = 0;
    unsigned remaining = (unsigned)p.top_k;
    for (int level = 0; level < 3; ++level) {
      const int shift = smp_shift(level), nb = smp_bins(level);
      for (int b = tid; b < SMP_BINS; b += SMP_THREADS) hist[b] = 0;
      __syncthreads();
      for (int base = 0; base < n; base += SMP_THREADS) {
        const int i = base + tid;
        unsigned bin = 0xffffffffu;
        if (i < n) {
          const uint32_t key = smp_key(scaled(i));
          if ((key & prefix_mask) == prefix) bin = (key >> shift) & (nb - 1);
        }
        const unsigned peers = __match_any_sync(0xffffffffu, bin);
        if (bin != 0xffffffffu && lane == __ffs(peers) - 1) atomicAdd(&hist[bin], (unsigned)__popc(peers));
      }
      __syncthreads();
      if (warp == 0) {  // from the top: first bin where the running count reaches `remaining`
        const int per = nb / 32;
        const int hi = nb - 1 - lane * per;  // lane 0 owns the highest bins
        unsigned mine = 0;
        for (int j = 0; j < per; ++j) mine += hist[hi - j];
        unsigned incl = mine;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
          const unsigned t = __shfl_up_sync(0xffffffffu, incl, o);
          if (lane >= o) incl += t;
        }
        const unsigned excl = incl - mine;
        if (excl < remaining && remaining <= incl) {
          unsigned run = excl;
          for (int j = 0; j < per; ++j) {
            const unsigned c = hist[hi - j];
            if (run + c >= remaining) {
              s_pick[0] = (unsigned)(hi - j);
              s_pick[1] = run;
              break;
            }
            run += c;
          }
        }
      }
      __syncthreads();
      prefix |= s_pick[0] << shift;
      prefix_mask |= (uint32_t)(nb - 1) << shift;
      remaining -= s_pick[1];
      __syncthreads();
    }
    key_k = prefix;
  }

  // ---- top-p: lowest key that survives the ascending cumulative-mass cut
  uint32_t key_p = 0;  // keep key >= key_p
  if (p.top_p < 1.0f) {
    // normaliser over what top-k kept (fixed tree)
    float z = 0.f;
    for (int i = tid; i < n; i += SMP_THREADS) {
      const float y = scaled(i);
      if (smp_key(y) >= key_k) z += expf(y - m_t);
    }
    z = warp_sum(z);
    if (lane == 0) ss[warp] = z;
    __syncthreads();
    z = warp_sum(lane < SMP_THREADS / 32 ? ss[lane] : 0.f);
    z = __shfl_sync(0xffffffffu, z, 0);
    __syncthreads();
    const float cut = 1.0f - p.top_p;  // fp32, as the reference's `1 - p`
    const unsigned long long target = (unsigned long long)((double)cut * 1099511627776.0);  // 2^40
    uint32_t prefix = 0, prefix_mask = 0;
    unsigned long long cum = 0;  // mass of the kept-by-top-k keys below the current prefix
    for (int level = 0; level < 3; ++level) {
      const int shift = smp_shift(level), nb = smp_bins(level);
      for (int b = tid; b < SMP_BINS; b += SMP_THREADS) mass[b] = 0ull;
      __syncthreads();
      for (int base = 0; base < n; base += SMP_THREADS) {
        const int i = base + tid;
        unsigned bin = 0xffffffffu;
        unsigned long long w = 0;
        if (i < n) {
          const float y = scaled(i);
          const uint32_t key = smp_key(y);
          if (key >= key_k && (key & prefix_mask) == prefix) {
            bin = (key >> shift) & (nb - 1);
            w = (unsigned long long)((double)(expf(y - m_t) / z) * 1099511627776.0);
          }
        }
        const unsigned peers = __match_any_sync(0xffffffffu, bin);
        const unsigned lo = __reduce_add_sync(peers, (unsigned)(w & 0xfffffull));
        const unsigned hi = __reduce_add_sync(peers, (unsigned)(w >> 20));
        if (bin != 0xffffffffu && lane == __ffs(peers) - 1)
          atomicAdd(&mass[bin], ((unsigned long long)hi << 20) + lo);
      }
      __syncthreads();
      if (warp == 0) {  // ascending: first bin whose inclusive mass exceeds the target
        const int per = nb / 32;
        const int lo_bin = lane * per;
        unsigned long long mine = 0;
        for (int j = 0; j < per; ++j) mine += mass[lo_bin + j];
        unsigned long long incl = mine;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
          const unsigned long long t = __shfl_up_sync(0xffffffffu, incl, o);
          if (lane >= o) incl += t;
        }
        const unsigned long long excl = incl - mine;
        const unsigned long long total = __shfl_sync(0xffffffffu, incl, 31);
        bool found = false;
        if (cum + excl <= target && cum + incl > target) {
          unsigned long long run = cum + excl;
          for (int j = 0; j < per; ++j) {
            const unsigned long long c = mass[lo_bin + j];
            if (run + c > target) {
              s_pick[0] = (unsigned)(lo_bin + j);
              s_cum = run;
              found = true;
              break;
            }
            run += c;
          }
        }
        // rounding of the fixed-point masses can leave the total at or below the target: keep the top bin
        if (!__any_sync(0xffffffffu, found) && lane == 31) {
          int b = nb - 1;
          while (b > 0 && mass[b] == 0ull) --b;
          s_pick[0] = (unsigned)b;
          s_cum = cum + total - mass[b];
        }
      }
      __syncthreads();
      prefix |= s_pick[0] << shift;
      prefix_mask |= (uint32_t)(nb - 1) << shift;
      cum = s_cum;
      __syncthreads();
    }
    key_p = prefix;
  }
  const uint32_t key_min = key_k > key_p ? key_k : key_p;

  if constexpr (MASK) {
    float* orow = p.masked_out + (long long)blockIdx.x * p.out_stride;
    for (int i = tid; i < n; i += SMP_THREADS) {
      const float y = scaled(i);
      orow[i] = smp_key(y) >= key_min ? y : -INFINITY;
    }
    return;
  }

  // ---- argmax of exp(y - max) / q over the kept tokens (lowest index on ties)
  float best = -INFINITY;
  int best_i = 0x7fffffff;
  auto consider = [&](float x, float qv, int i) {  // a thread's indices ascend: `>` keeps its lowest
    const float y = has_temp ? __fdiv_rn(x, p.temperature) : x;
    if (smp_key(y) >= key_min) {
      const float r = __fdiv_rn(expf(y - m_t), qv);
      if (r > best) {
        best = r;
        best_i = i;
      }
    }
  };
  constexpr int VEC = RowLoader<T>::VEC;
  const bool qvec = p.vec && (reinterpret_cast<uintptr_t>(qrow) & 15) == 0;
  const int nvec = qvec ? n / VEC : 0;
  for (int v = tid; v < nvec; v += SMP_THREADS) {
    float xv[VEC], qv[VEC];
    RowLoader<T>::load(row + (size_t)v * VEC, xv);
#pragma unroll
    for (int j = 0; j < VEC; j += 4) RowLoader<float>::load(qrow + (size_t)v * VEC + j, qv + j);
#pragma unroll
    for (int j = 0; j < VEC; ++j) consider(xv[j], qv[j], v * VEC + j);
  }
  for (int i = nvec * VEC + tid; i < n; i += SMP_THREADS) consider((float)row[i], qrow[i], i);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ob = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
    if (ob > best || (ob == best && oi < best_i)) {
      best = ob;
      best_i = oi;
    }
  }
  if (lane == 0) {
    sm[warp] = best;
    si[warp] = best_i;
  }
  __syncthreads();
  if (warp == 0) {
    best = lane < SMP_THREADS / 32 ? sm[lane] : -INFINITY;
    best_i = lane < SMP_THREADS / 32 ? si[lane] : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
      if (ob > best || (ob == best && oi < best_i)) {
        best = ob;
        best_i = oi;
      }
    }
    if (lane == 0) {
      if (best_i == 0x7fffffff) best_i = 0;
      p.tokens[blockIdx.x] = best_i;
      p.logprobs[blockIdx.x] = (float)row[best_i] - (logf(raw.s) + raw.m);
    }
  }
}

}  // namespace b200

extern "C" int b200_greedy_logprob(const void* logits, void* tokens_i64, void* logprobs_f32, long long rows, int n,
                                   long long row_stride, int dtype, void* stream);

extern "C" int b200_sample_token(const void* logits, const void* noise_q_f32, void* tokens_i64, void* logprobs_f32,
                                 long long rows, int n, long long row_stride, long long q_row_stride, int dtype,
                                 float temperature, int top_k, float top_p, void* stream) {
  using namespace b200;
  if (!logits || !tokens_i64 || !logprobs_f32 || rows < 0 || n <= 0) return B200_ERR_ARG;
  // the reference samples only when temperature > 0 and top_p > 0 (sampler.py:55); else arg-max
  if (!noise_q_f32 || !(temperature > 0.f) || !(top_p > 0.f))
    return b200_greedy_logprob(logits, tokens_i64, logprobs_f32, rows, n, row_stride, dtype, stream);
  if (rows == 0) return B200_OK;
  if (dtype != 0 && dtype != 1) return B200_ERR_ARG;
  const bool aligned = (reinterpret_cast<uintptr_t>(logits) & 15) == 0;
  SampleParams p{logits, (const float*)noise_q_f32, (long long*)tokens_i64, (float*)logprobs_f32, n, row_stride,
                 q_row_stride, temperature, top_p, top_k, aligned && row_stride % (dtype == 0 ? 4 : 8) == 0, nullptr, 0};
  cudaStream_t st = (cudaStream_t)stream;
  if (dtype == 0)
    launch_k(sample_token_kernel<float>, dim3((unsigned)rows), dim3(SMP_THREADS), 0, st, p);
  else
    launch_k(sample_token_kernel<__nv_bfloat16>, dim3((unsigned)rows), dim3(SMP_THREADS), 0, st, p);
  return launch_status();
}

// The masking step alone: out[r, i] = x[r, i] / temperature where the token survives top-k and top-p, -inf
// elsewhere (fp32 [rows, n]); the thresholds are the ones b200_sample_token uses.  top_k <= 0 and top_p >= 1
// switch the respective cut off.
extern "C" int b200_apply_top_k_top_p(const void* logits, void* out_f32, long long rows, int n, long long row_stride,
                                      long long out_row_stride, int dtype, float temperature, int top_k, float top_p,
                                      void* stream) {
  using namespace b200;
  if (!logits || !out_f32 || rows < 0 || n <= 0 || !(temperature > 0.f) || (dtype != 0 && dtype != 1))
    return B200_ERR_ARG;
  if (rows == 0) return B200_OK;
  const bool aligned = (reinterpret_cast<uintptr_t>(logits) & 15) == 0;
  SampleParams p{logits, nullptr, nullptr, nullptr, n, row_stride, 0, temperature, top_p, top_k,
                 aligned && row_stride % (dtype == 0 ? 4 : 8) == 0, (float*)out_f32, out_row_stride};
  cudaStream_t st = (cudaStream_t)stream;
  if (dtype == 0)
    launch_k(sample_token_kernel<float, true>, dim3((unsigned)rows), dim3(SMP_THREADS), 0, st, p);
  else
    launch_k(sample_token_kernel<__nv_bfloat16, true>, dim3((unsigned)rows), dim3(SMP_THREADS), 0, st, p);
  return launch_status();
}

// ------------------------------------------------------------------ per-request seeded noise
// Seeded sampling (vexact/inferencer/sampler.py:57-63, 90-118) keys the random stream of a request by its
// seed and by the absolute position of the token being sampled, so a request draws the same token whatever
// batch it sits in.  The reference delegates this to vLLM's Gumbel kernel; here the Exp(1) noise the
// sampling kernel consumes (token = argmax softmax / q) is generated with Philox4x32-10 (Salmon et al.,
// "Parallel random numbers: as easy as 1, 2, 3", SC'11): key = the 64-bit seed, counter = (column / 4,
// position low, position high, 0), four uniforms per counter, u = (x + 0.5) * 2^-32, q = -ln(u).  It is the
// same construction, not the same stream: tokens differ from vLLM's for a given seed.
namespace b200 {

__device__ __forceinline__ void philox4x32_10(uint32_t c0, uint32_t c1, uint32_t c2, uint32_t c3, uint32_t k0,
                                              uint32_t k1, uint32_t (&out)[4]) {
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    const uint32_t hi0 = __umulhi(0xD2511F53u, c0), lo0 = 0xD2511F53u * c0;
    const uint32_t hi1 = __umulhi(0xCD9E8D57u, c2), lo1 = 0xCD9E8D57u * c2;
    const uint32_t n0 = hi1 ^ c1 ^ k0, n1 = lo1, n2 = hi0 ^ c3 ^ k1, n3 = lo0;
    c0 = n0, c1 = n1, c2 = n2, c3 = n3;
    k0 += 0x9E3779B9u;
    k1 += 0xBB67AE85u;
  }
  out[0] = c0, out[1] = c1, out[2] = c2, out[3] = c3;
}

__global__ void __launch_bounds__(256)
seeded_exponential_kernel(float* __restrict__ q, const long long* __restrict__ seeds,
                          const long long* __restrict__ positions, int n, long long q_stride) {
  pdl_trigger();
  pdl_wait();
  const long long row = blockIdx.y;
  const unsigned long long seed = (unsigned long long)seeds[row], pos = (unsigned long long)positions[row];
  const int quad = blockIdx.x * blockDim.x + threadIdx.x;   // columns 4 quad .. 4 quad + 3
  if (quad * 4 >= n) return;
  uint32_t x[4];
  philox4x32_10((uint32_t)quad, (uint32_t)pos, (uint32_t)(pos >> 32), 0u, (uint32_t)seed, (uint32_t)(seed >> 32), x);
  float* dst = q + row * q_stride + (long long)quad * 4;
#pragma unroll
  for (int i = 0; i < 4; ++i)
    if (quad * 4 + i < n) dst[i] = -logf(((float)x[i] + 0.5f) * 2.3283064365386963e-10f);
}

}  // namespace b200

extern "C" int b200_seeded_exponential(void* noise_q_f32, const void* seeds_i64, const void* positions_i64,
                                       long long rows, int n, long long q_row_stride, void* stream) {
  using namespace b200;
  if (!noise_q_f32 || !seeds_i64 || !positions_i64 || rows < 0 || n <= 0) return B200_ERR_ARG;
  if (rows == 0) return B200_OK;
  if (rows > 65535) return B200_ERR_SHAPE;
  const int quads = (n + 3) / 4;
  launch_k(seeded_exponential_kernel, dim3((unsigned)((quads + 255) / 256), (unsigned)rows), dim3(256), 0,
           (cudaStream_t)stream, (float*)noise_q_f32, (const long long*)seeds_i64, (const long long*)positions_i64, n,
           q_row_stride);
  return launch_status();
}
