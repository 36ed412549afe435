// MoE routing, token permutation and the fixed-order top-k reduction.
// Integer parts are bit-exact; the floating-point parts round where the
// reference's torch ops materialise tensors.
//
// Replaces
//   vexact/models/qwen3_moe/modeling_qwen3_moe.py:128-134   softmax -> topk -> renorm -> cast
//   vexact/models/deepseek_v3/modeling_deepseek_v3.py:185-208 sigmoid + bias, group-limited top-k
//   vexact/batch_invariant_ops/fused_moe.py:268-292          _build_moe_indices (stable argsort by
//       expert, inverse permutation, histogram, cumulative sum)
//   vexact/batch_invariant_ops/group_gemm/kernel/moe.py:28-78, 255-335 (histogram, scatter)
//   vexact/batch_invariant_ops/group_gemm/kernel/moe.py:86-160 (moe_gather: fp32 sum over the k
//       expert rows of a token in k order, then one cast)
//   vexact/batch_invariant_ops/fused_moe.py:325-336           silu * up * routing weight
//
// Top-k ties are broken towards the lower expert index; selected experts are
// returned in descending weight order (what torch.topk(sorted=True) returns).
#pragma once
#include "common.cuh"
#include "norm.cuh"

namespace b200 {

constexpr int MOE_MAX_EXPERTS = 256;
constexpr int MOE_MAX_TOPK = 16;

// Softmax -> top-k -> renorm of one token's logits by one warp.  Each lane owns experts lane,
// lane + 32, ... (up to 8).
template <typename TIn>
__device__ __forceinline__ void route_softmax_topk_token(const TIn* __restrict__ row, long long tok,
                                                         __nv_bfloat16* __restrict__ w_bf16,
                                                         float* __restrict__ w_f32, int* __restrict__ idx_i32,
                                                         long long* __restrict__ idx_i64, int E, int topk,
                                                         int renorm, int lane) {
  constexpr int PER = MOE_MAX_EXPERTS / 32;
  float v[PER];
  float mx = -INFINITY;
#pragma unroll
  for (int i = 0; i < PER; ++i) {
    const int e = lane + 32 * i;
    v[i] = e < E ? (float)row[e] : -INFINITY;
    mx = fmaxf(mx, v[i]);
  }
  mx = warp_max(mx);
  float sum = 0.f;
#pragma unroll
  for (int i = 0; i < PER; ++i) {
    const int e = lane + 32 * i;
    v[i] = e < E ? expf(v[i] - mx) : 0.f;
    sum += v[i];
  }
  sum = warp_sum(sum);
#pragma unroll
  for (int i = 0; i < PER; ++i) {
    v[i] = v[i] / sum;  // softmax probabilities (fp32)
    // A row of NaN logits (a padded token of a captured batch: its hidden state is never defined) must
    // still select experts inside [0, E): NaN compares false with everything, so it counts as 0 here.
    if (!(v[i] == v[i])) v[i] = 0.f;
  }

  float sel_w[MOE_MAX_TOPK];
  int sel_e[MOE_MAX_TOPK];
  for (int k = 0; k < topk; ++k) {
    // lane-local best (lowest index on ties), then a butterfly with the same tie rule
    float bv = -1.f;
    int be = 0x7fffffff;
#pragma unroll
    for (int i = 0; i < PER; ++i) {
      const int e = lane + 32 * i;
      if (e < E && (v[i] > bv)) {
        bv = v[i];
        be = e;
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oe = __shfl_xor_sync(0xffffffffu, be, o);
      if (ov > bv || (ov == bv && oe < be)) {
        bv = ov;
        be = oe;
      }
    }
    if (be < 0 || be >= E) be = 0;  // unreachable for topk <= E
    sel_w[k] = bv;
    sel_e[k] = be;
    if ((be & 31) == lane) {
#pragma unroll
      for (int i = 0; i < PER; ++i)
        if (lane + 32 * i == be) v[i] = -2.f;  // remove from the candidate set
    }
  }
  if (lane == 0) {
    float denom = 1.f;
    if (renorm) {
      denom = 0.f;
      for (int k = 0; k < topk; ++k) denom += sel_w[k];
    }
    for (int k = 0; k < topk; ++k) {
      const float w = renorm ? sel_w[k] / denom : sel_w[k];
      if (w_bf16) w_bf16[tok * topk + k] = f2bf(w);
      if (w_f32) w_f32[tok * topk + k] = w;
      if (idx_i32) idx_i32[tok * topk + k] = sel_e[k];
      if (idx_i64) idx_i64[tok * topk + k] = sel_e[k];
    }
  }
}

// One warp per token.
template <typename TIn>
__global__ void __launch_bounds__(256)
moe_route_softmax_topk_kernel(const TIn* __restrict__ logits, long long row_stride,
                              __nv_bfloat16* __restrict__ w_bf16, float* __restrict__ w_f32,
                              int* __restrict__ idx_i32, long long* __restrict__ idx_i64, long long T, int E,
                              int topk, int renorm) {
  pdl_trigger();
  pdl_wait();
  const long long tok = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (tok >= T) return;
  route_softmax_topk_token<TIn>(logits + tok * row_stride, tok, w_bf16, w_f32, idx_i32, idx_i64, E, topk, renorm,
                                threadIdx.x & 31);
}

// DeepSeek-V3 routing.  One warp per token; E <= 256.
//   s = sigmoid(logit); c = s + bias; group score = sum of the group's top-2 c;
//   keep the top `topk_group` groups, zero the rest (masked_fill 0.0), top-k over c;
//   weights = s[selected] (/ (sum + 1e-20) if renorm) * scale.
// torch.topk(sorted=False) leaves the order of the selected experts unspecified; this kernel
// returns them in descending choice-score order, ties to the lower index.
__global__ void __launch_bounds__(256)
moe_route_sigmoid_group_topk_kernel(const float* __restrict__ logits, long long row_stride,
                                    const float* __restrict__ bias, float* __restrict__ w_out,
                                    int* __restrict__ idx_i32, long long* __restrict__ idx_i64, long long T,
                                    int E, int n_group, int topk_group, int topk, int renorm, float scale) {
  pdl_trigger();
  pdl_wait();
  __shared__ float s_sig[8][MOE_MAX_EXPERTS];
  __shared__ float s_choice[8][MOE_MAX_EXPERTS];
  __shared__ float s_gscore[8][32];
  const int wib = threadIdx.x >> 5;
  const long long tok = (long long)blockIdx.x * 8 + wib;
  if (tok >= T) return;
  const int lane = threadIdx.x & 31;
  const float* row = logits + tok * row_stride;
  float* sig = s_sig[wib];
  float* choice = s_choice[wib];
  for (int e = lane; e < E; e += 32) {
    float s = 1.0f / (1.0f + expf(-row[e]));
    // NaN logits (a padded token of a captured batch) count as score 0, so that the selection below
    // always finds candidates inside [0, E)
    if (!(s == s)) s = 0.f;
    float c = s + (bias ? bias[e] : 0.f);
    if (!(c == c)) c = 0.f;
    sig[e] = s;
    choice[e] = c;
  }
  __syncwarp();
  const int gsize = E / n_group;
  for (int gidx = lane; gidx < n_group; gidx += 32) {
    float t1 = -INFINITY, t2 = -INFINITY;
    for (int j = 0; j < gsize; ++j) {
      const float c = choice[gidx * gsize + j];
      if (c > t1) {
        t2 = t1;
        t1 = c;
      } else if (c > t2) {
        t2 = c;
      }
    }
    s_gscore[wib][gidx] = t1 + t2;
  }
  __syncwarp();
  // Select the top groups (lane 0, n_group <= 32), then mask the others to 0.0.
  unsigned keep = 0;
  if (lane == 0) {
    for (int r = 0; r < topk_group; ++r) {
      float bv = -INFINITY;
      int bg = -1;
      for (int gi = 0; gi < n_group; ++gi)
        if (!((keep >> gi) & 1u) && s_gscore[wib][gi] > bv) {
          bv = s_gscore[wib][gi];
          bg = gi;
        }
      if (bg >= 0) keep |= 1u << bg;
    }
  }
  keep = __shfl_sync(0xffffffffu, keep, 0);
  for (int e = lane; e < E; e += 32)
    if (!((keep >> (e / gsize)) & 1u)) choice[e] = 0.0f;
  __syncwarp();
  float sel_w[MOE_MAX_TOPK];
  int sel_e[MOE_MAX_TOPK];
  for (int k = 0; k < topk; ++k) {
    float bv = -INFINITY;
    int be = 0x7fffffff;
    for (int e = lane; e < E; e += 32) {
      const float c = choice[e];
      if (c > bv) {
        bv = c;
        be = e;
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oe = __shfl_xor_sync(0xffffffffu, be, o);
      if (ov > bv || (ov == bv && oe < be)) {
        bv = ov;
        be = oe;
      }
    }
    if (be < 0 || be >= E) be = 0;  // unreachable for topk <= E; keeps the shared-memory accesses in range regardless
    sel_e[k] = be;
    sel_w[k] = sig[be];
    __syncwarp();
    if (lane == 0) choice[be] = -INFINITY;
    __syncwarp();
  }
  if (lane == 0) {
    float denom = 1.f;
    if (renorm) {
      denom = 0.f;
      for (int k = 0; k < topk; ++k) denom += sel_w[k];
      denom += 1e-20f;
    }
    for (int k = 0; k < topk; ++k) {
      float w = renorm ? sel_w[k] / denom : sel_w[k];
      w = w * scale;
      w_out[tok * topk + k] = w;
      if (idx_i32) idx_i32[tok * topk + k] = sel_e[k];
      if (idx_i64) idx_i64[tok * topk + k] = sel_e[k];
    }
  }
}

// Index build: one CTA of 1024 threads.  For flat index f = t * topk + k (the order
// expert_index.flatten() has) computes its position in the stable sort by expert:
//   scatter_index[f] = cu_seqlens[e_f] + #{f' < f : e_f' == e_f}
// plus cu_seqlens[E + 1] and the token-tile table of the grouped GEMM (tiles of at most
// `tile_rows` consecutive rows of one expert).
//
// Warp w owns the contiguous segment [w * seg, (w + 1) * seg) of the flat array and walks it 32
// entries at a time: __match_any_sync groups equal experts, the lowest lane of a group bumps the
// warp's private per-expert counter, so every entry learns its rank among the warp's earlier
// entries of the same expert.  A per-expert scan over the 32 warps and a scan over the experts
// turn those ranks into global positions.  All of it is integer arithmetic: bit-exact.
template <typename TIdx>
__global__ void __launch_bounds__(1024)
moe_index_kernel(const TIdx* __restrict__ experts, long long n, int E, int tile_rows,
                 int* __restrict__ scatter_index, int* __restrict__ cu_seqlens, int4* __restrict__ tile_table,
                 int* __restrict__ tile_count, int max_tiles, int topk, int* __restrict__ gather_index,
                 const __nv_bfloat16* __restrict__ weights, __nv_bfloat16* __restrict__ row_scale) {
  pdl_trigger();
  pdl_wait();
  __shared__ int cnt[32][MOE_MAX_EXPERTS];  // per-warp counts, then per-warp exclusive offsets
  __shared__ int base[MOE_MAX_EXPERTS];     // expert totals, then exclusive prefix (cu_seqlens)
  __shared__ int tbase[MOE_MAX_EXPERTS];    // first tile index of each expert
  __shared__ int wsum[32];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  for (int i = tid; i < 32 * MOE_MAX_EXPERTS; i += 1024) (&cnt[0][0])[i] = 0;
  __syncthreads();
  const long long seg = ((n + 31) / 32 + 31) / 32 * 32;  // entries per warp, a multiple of 32
  const long long w0 = warp * seg;
  // pass 1: rank of every entry among the warp's earlier entries of the same expert
  for (long long o = 0; o < seg; o += 32) {
    const long long i = w0 + o + lane;
    int e = -1;
    if (i < n) {
      const long long ev = (long long)experts[i];
      if (ev >= 0 && ev < E)
        e = (int)ev;
      else
        report_status(B200_STATUS_BAD_INDEX, (int)ev);
    }
    const unsigned mask = __match_any_sync(0xffffffffu, e);
    const int rank = __popc(mask & ((1u << lane) - 1u));
    const int leader = __ffs(mask) - 1;
    int old = 0;
    if (rank == 0 && e >= 0) {
      old = cnt[warp][e];
      cnt[warp][e] = old + __popc(mask);
    }
    old = __shfl_sync(0xffffffffu, old, leader);
    if (i < n) scatter_index[i] = e >= 0 ? old + rank : -1;
    __syncwarp();
  }
  __syncthreads();
  // per expert: exclusive scan over the warps, total into base[]
  if (tid < E) {
    int run = 0;
#pragma unroll 8
    for (int w = 0; w < 32; ++w) {
      const int c = cnt[w][tid];
      cnt[w][tid] = run;
      run += c;
    }
    base[tid] = run;
  }
  __syncthreads();
  // exclusive scans over the experts (rows and tiles), 256 threads = 8 warps
  if (tid < MOE_MAX_EXPERTS) {
    const int rows = tid < E ? base[tid] : 0;
    const int tiles = (rows + tile_rows - 1) / tile_rows;
    int r = rows, t = tiles;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int r2 = __shfl_up_sync(0xffffffffu, r, o);
      const int t2 = __shfl_up_sync(0xffffffffu, t, o);
      if (lane >= o) {
        r += r2;
        t += t2;
      }
    }
    if (lane == 31) {
      wsum[warp] = r;
      wsum[8 + warp] = t;
    }
    // (only warps 0..7 reach here; named barrier over their 256 threads)
    asm volatile("bar.sync 2, 256;" ::: "memory");
    int roff = 0, toff = 0;
    for (int w = 0; w < warp; ++w) {
      roff += wsum[w];
      toff += wsum[8 + w];
    }
    const int rexcl = roff + r - rows;
    const int texcl = toff + t - tiles;
    asm volatile("bar.sync 2, 256;" ::: "memory");
    if (tid < E) {
      base[tid] = rexcl;
      tbase[tid] = texcl;
      cu_seqlens[tid] = rexcl;
      for (int j = 0; j < tiles; ++j)
        if (texcl + j < max_tiles)
          tile_table[texcl + j] = make_int4(tid, rexcl + j * tile_rows, min(tile_rows, rows - j * tile_rows), 0);
      if (tid == E - 1) {
        cu_seqlens[E] = rexcl + rows;
        *tile_count = min(texcl + tiles, max_tiles);
      }
    }
  }
  __syncthreads();
  // pass 2: local rank -> global position
  for (long long o = 0; o < seg; o += 32) {
    const long long i = w0 + o + lane;
    if (i < n) {
      const long long ev = (long long)experts[i];
      if (ev >= 0 && ev < E) {
        const int pos = scatter_index[i] + base[(int)ev] + cnt[warp][(int)ev];
        scatter_index[i] = pos;
        // the inverse map for a GEMM that gathers its rows (sorted row -> token), and the routing weight
        // of each sorted row, so that no permuted copy of the activations has to be made
        if (gather_index) gather_index[pos] = (int)(i / topk);
        if (row_scale) row_scale[pos] = weights[i];
      }
    }
  }
}

// Row scatter: x_perm[scatter_index[f]] = x[f / topk]; row_scale[scatter_index[f]] = weights[f].
__global__ void __launch_bounds__(128)
moe_scatter_rows_kernel(const __nv_bfloat16* __restrict__ x, long long x_stride,
                        const __nv_bfloat16* __restrict__ weights, const int* __restrict__ scatter_index,
                        __nv_bfloat16* __restrict__ x_perm, __nv_bfloat16* __restrict__ row_scale, int H,
                        int topk) {
  pdl_trigger();
  pdl_wait();
  const long long f = blockIdx.x;
  const int pos = scatter_index[f];
  if (pos < 0) return;
  const __nv_bfloat16* src = x + (f / topk) * x_stride;
  __nv_bfloat16* dst = x_perm + (long long)pos * H;
  for (int i = threadIdx.x; i < (H >> 3); i += 128)
    reinterpret_cast<uint4*>(dst)[i] = reinterpret_cast<const uint4*>(src)[i];
  if (threadIdx.x == 0 && row_scale && weights) row_scale[pos] = weights[f];
}

// Sum of a token's top-k expert rows (16-byte vector v of each) in k order, fp32.  For topk <= 8 the k row
// positions are read first and the k row loads are issued together, so the chain is two memory latencies
// instead of 2k; the additions run in k order either way (same bits).
__device__ __forceinline__ void moe_topk_row_sum(const __nv_bfloat16* __restrict__ y,
                                                 const int* __restrict__ scatter_index, long long t, int topk,
                                                 int H, int v, float (&acc)[8]) {
#pragma unroll
  for (int j = 0; j < 8; ++j) acc[j] = 0.f;
  if (topk <= 8) {
    int pos[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) pos[k] = k < topk ? scatter_index[t * topk + k] : -1;
    uint4 r[8];
#pragma unroll
    for (int k = 0; k < 8; ++k)
      r[k] = pos[k] >= 0 ? reinterpret_cast<const uint4*>(y + (long long)pos[k] * H)[v] : make_uint4(0, 0, 0, 0);
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      if (pos[k] < 0) continue;
      const uint32_t* rp = reinterpret_cast<const uint32_t*>(&r[k]);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float a, b;
        unpack_bf2(rp[j], a, b);
        acc[2 * j] += a;
        acc[2 * j + 1] += b;
      }
    }
    return;
  }
  for (int k = 0; k < topk; ++k) {
    const int pos = scatter_index[t * topk + k];
    if (pos < 0) continue;
    const uint4 r = reinterpret_cast<const uint4*>(y + (long long)pos * H)[v];
    const uint32_t* rp = reinterpret_cast<const uint32_t*>(&r);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float a, b;
      unpack_bf2(rp[j], a, b);
      acc[2 * j] += a;
      acc[2 * j + 1] += b;
    }
  }
}

// The top-k sum below followed, in the same launch, by the residual add and the RMSNorm that the next
// decoder layer starts with:  m = bf16(sum_k y[...]) (+ addend);  s = bf16(residual + m);
// out = rmsnorm(s) * w.  Same arithmetic, element for element, as moe_unpermute_reduce_kernel followed
// by rmsnorm_cta_kernel<true> (the sum of squares is accumulated and reduced in that kernel's order).
__global__ void __launch_bounds__(128)
moe_unpermute_add_rmsnorm_kernel(const __nv_bfloat16* __restrict__ y, const int* __restrict__ scatter_index,
                                 const __nv_bfloat16* __restrict__ addend, const __nv_bfloat16* __restrict__ res,
                                 const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ sum_out,
                                 __nv_bfloat16* __restrict__ out, int H, int topk, float eps, int mode) {
  pdl_trigger();
  pdl_wait();
  __shared__ float scratch[32];
  constexpr int MAXV = 8, THREADS = 128;
  const long long t = blockIdx.x;
  const int nvec = H >> 3;
  uint4 cache[MAXV];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < MAXV; ++i) {
    const int v = threadIdx.x + i * THREADS;
    if (v < nvec) {
      float acc[8];
      moe_topk_row_sum(y, scatter_index, t, topk, H, v, acc);
      if (addend) {
        const uint4 r = reinterpret_cast<const uint4*>(addend + t * H)[v];
        const uint32_t* rp = reinterpret_cast<const uint32_t*>(&r);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          float a, b;
          unpack_bf2(rp[j], a, b);
          acc[2 * j] = round_bf(acc[2 * j]) + a;
          acc[2 * j + 1] = round_bf(acc[2 * j + 1]) + b;
        }
      }
      // m = bf16(acc); s = bf16(residual + m)
      const uint4 r = reinterpret_cast<const uint4*>(res + t * H)[v];
      const uint32_t* rp = reinterpret_cast<const uint32_t*>(&r);
      uint4 a;
      uint32_t* ap = reinterpret_cast<uint32_t*>(&a);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float r0, r1;
        unpack_bf2(rp[j], r0, r1);
        ap[j] = pack_bf2(r0 + round_bf(acc[2 * j]), r1 + round_bf(acc[2 * j + 1]));
      }
      reinterpret_cast<uint4*>(sum_out + t * H)[v] = a;
      cache[i] = a;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float a0, a1;
        unpack_bf2(ap[j], a0, a1);
        ss += a0 * a0;
        ss += a1 * a1;
      }
    }
  }
  const float tot = block_sum(ss, scratch);
  const float inv = rms_scale(tot, H, eps, mode);
#pragma unroll
  for (int i = 0; i < MAXV; ++i) {
    const int v = threadIdx.x + i * THREADS;
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
      reinterpret_cast<uint4*>(out + t * H)[v] = o;
    }
  }
}

// out[t] = bf16( sum_k fp32(y[scatter_index[t, k]]) ), k ascending; optionally followed by
// out[t] = bf16(fp32(out[t]) + fp32(addend[t])) (shared-expert or residual add as a separate bf16 op).
__global__ void __launch_bounds__(256)
moe_unpermute_reduce_kernel(const __nv_bfloat16* __restrict__ y, const int* __restrict__ scatter_index,
                            const __nv_bfloat16* __restrict__ addend, __nv_bfloat16* __restrict__ out, int H,
                            int topk) {
  pdl_trigger();
  pdl_wait();
  const long long t = blockIdx.x;
  for (int v = threadIdx.x; v < (H >> 3); v += 256) {
    float acc[8];
    moe_topk_row_sum(y, scatter_index, t, topk, H, v, acc);
    if (addend) {
      const uint4 r = reinterpret_cast<const uint4*>(addend + t * H)[v];
      const uint32_t* rp = reinterpret_cast<const uint32_t*>(&r);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float a, b;
        unpack_bf2(rp[j], a, b);
        acc[2 * j] = round_bf(acc[2 * j]) + a;
        acc[2 * j + 1] = round_bf(acc[2 * j + 1]) + b;
      }
    }
    uint4 o;
    uint32_t* op = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
    for (int j = 0; j < 4; ++j) op[j] = pack_bf2(acc[2 * j], acc[2 * j + 1]);
    reinterpret_cast<uint4*>(out + t * H)[v] = o;
  }
}

// The two row permutations as operators of their own, over an index array the caller supplies
// (group_gemm/kernel/moe.py:304 moe_scatter, :131 moe_gather).  Unlike the kernels above, which only ever see
// indices this library built, these check every index against the row count: a bad one is skipped and
// reported through the status word (B200_STATUS_BAD_INDEX), where the reference has a device assert.
// Rows are moved as 16-byte vectors, so the scatter serves any 2-byte element type.
__global__ void __launch_bounds__(128)
moe_scatter_checked_kernel(const uint4* __restrict__ x, long long x_stride_v, const int* __restrict__ index,
                           long long index_stride_t, long long index_stride_k, uint4* __restrict__ out,
                           long long out_rows, int hv, int topk) {
  pdl_trigger();
  pdl_wait();
  const long long f = blockIdx.x;
  const long long t = f / topk;
  const int pos = index[t * index_stride_t + (f - t * topk) * index_stride_k];
  if (pos < 0 || pos >= out_rows) {
    if (threadIdx.x == 0) report_status(B200_STATUS_BAD_INDEX, (int)f);
    return;
  }
  const uint4* src = x + t * x_stride_v;
  uint4* dst = out + (long long)pos * hv;
  for (int i = threadIdx.x; i < hv; i += 128) dst[i] = src[i];
}

// out[t] = bf16( sum_k fp32(x[index[t, k]]) ), k ascending.
__global__ void __launch_bounds__(256)
moe_gather_checked_kernel(const __nv_bfloat16* __restrict__ x, long long x_rows, const int* __restrict__ index,
                          long long index_stride_t, long long index_stride_k, __nv_bfloat16* __restrict__ out,
                          int H, int topk) {
  pdl_trigger();
  pdl_wait();
  const long long t = blockIdx.x;
  for (int v = threadIdx.x; v < (H >> 3); v += 256) {
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
    for (int k = 0; k < topk; ++k) {
      const int pos = index[t * index_stride_t + k * index_stride_k];
      if (pos < 0 || pos >= x_rows) {
        if (v == 0) report_status(B200_STATUS_BAD_INDEX, (int)(t * topk + k));
        continue;
      }
      const uint4 r = reinterpret_cast<const uint4*>(x + (long long)pos * H)[v];
      const uint32_t* rp = reinterpret_cast<const uint32_t*>(&r);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float a, b;
        unpack_bf2(rp[j], a, b);
        acc[2 * j] += a;
        acc[2 * j + 1] += b;
      }
    }
    uint4 o;
    uint32_t* op = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
    for (int j = 0; j < 4; ++j) op[j] = pack_bf2(acc[2 * j], acc[2 * j + 1]);
    reinterpret_cast<uint4*>(out + t * H)[v] = o;
  }
}

// Weight gradient of a grouped GEMM, the contraction running over each group's own rows ("ragged K"):
//   c[g, m, n] = sum over rows r of group g, ascending, of a[r, m] * b[r, n]      (fp32 fmaf chain, one rounding)
// (group_gemm/kernel/group_gemm.py:255-400 group_gemm_same_mn with transpose_a).  A training-side operator kept
// simple: one CTA per 64 x 64 tile of one group's output, rows staged 16 at a time through shared memory, fp32
// FMAs on the CUDA cores.  With ~rows/groups rows per group the work is a few GFLOP and the kernel is bound by
// writing c (groups * M * N * 2 bytes); an empty group gets zeros.  A group whose bounds leave [0, rows] or
// decrease is clipped and reported through the status word.
constexpr int WG_TILE = 64, WG_ROWS = 16;
__global__ void __launch_bounds__(256)
moe_wgrad_kernel(const __nv_bfloat16* __restrict__ a, const __nv_bfloat16* __restrict__ b,
                 __nv_bfloat16* __restrict__ c, const int* __restrict__ cu_seqlens, long long rows, int M, int N) {
  pdl_trigger();
  pdl_wait();
  __shared__ float sa[WG_ROWS][WG_TILE], sb[WG_ROWS][WG_TILE];
  const int g = blockIdx.z, m0 = blockIdx.y * WG_TILE, n0 = blockIdx.x * WG_TILE;
  long long r0 = cu_seqlens[g], r1 = cu_seqlens[g + 1];
  if (r0 < 0 || r1 > rows || r1 < r0) {
    if (threadIdx.x == 0 && blockIdx.x == 0 && blockIdx.y == 0) report_status(B200_STATUS_BAD_INDEX, g);
    r0 = r0 < 0 ? 0 : (r0 > rows ? rows : r0);
    r1 = r1 > rows ? rows : r1;
    if (r1 < r0) r1 = r0;
  }
  const int tid = threadIdx.x, ty = tid >> 4, tx = tid & 15;
  const int lr = tid >> 4, lc = (tid & 15) * 4;       // this thread stages row lr, columns lc..lc+3 of both tiles
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
  for (long long r = r0; r < r1; r += WG_ROWS) {
    const long long row = r + lr;
    float va[4] = {0.f, 0.f, 0.f, 0.f}, vb[4] = {0.f, 0.f, 0.f, 0.f};
    if (row < r1) {
      if (m0 + lc < M) {            // M and N are multiples of 4: a group of four columns is inside or outside
        const uint2 q = *reinterpret_cast<const uint2*>(a + row * M + m0 + lc);
        unpack_bf2(q.x, va[0], va[1]);
        unpack_bf2(q.y, va[2], va[3]);
      }
      if (n0 + lc < N) {
        const uint2 q = *reinterpret_cast<const uint2*>(b + row * N + n0 + lc);
        unpack_bf2(q.x, vb[0], vb[1]);
        unpack_bf2(q.y, vb[2], vb[3]);
      }
    }
    __syncthreads();                // the previous chunk has been consumed
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      sa[lr][lc + j] = va[j];
      sb[lr][lc + j] = vb[j];
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < WG_ROWS; ++k) {
      float xa[4], xb[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) xa[i] = sa[k][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) xb[j] = sb[k][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(xa[i], xb[j], acc[i][j]);
    }
  }
  __nv_bfloat16* cg = c + (long long)g * M * N;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int m = m0 + ty * 4 + i, n = n0 + tx * 4;
    if (m < M && n < N) {
      uint2 o;
      o.x = pack_bf2(acc[i][0], acc[i][1]);
      o.y = pack_bf2(acc[i][2], acc[i][3]);
      *reinterpret_cast<uint2*>(cg + (long long)m * N + n) = o;
    }
  }
}

// The same weight gradient on the tensor cores (mma.sync m16n8k16, bf16 x bf16 -> fp32): one CTA per 128 x 128
// tile of one group's output, eight warps of 64 x 32 each, the group's rows staged 32 at a time as bf16 and read
// with transposing ldmatrix (both operands have the contraction as their row dimension).  Products are exact,
// the sum runs over 16-row steps in ascending order with the instruction's own order inside a step: deterministic,
// and within fp32 rounding of the CUDA-core kernel above.  M and N multiples of 8, 16-byte aligned pointers.
constexpr int WGM_TILE = 128, WGM_ROWS = 32, WGM_LD = WGM_TILE + 8;   // padded row: ldmatrix rows 272 bytes apart
__global__ void __launch_bounds__(256)
moe_wgrad_mma_kernel(const __nv_bfloat16* __restrict__ a, const __nv_bfloat16* __restrict__ b,
                     __nv_bfloat16* __restrict__ c, const int* __restrict__ cu_seqlens, long long rows, int M, int N) {
  pdl_trigger();
  pdl_wait();
  __shared__ __align__(16) __nv_bfloat16 sa[WGM_ROWS][WGM_LD], sb[WGM_ROWS][WGM_LD];
  const int g = blockIdx.z, m0 = blockIdx.y * WGM_TILE, n0 = blockIdx.x * WGM_TILE;
  long long r0 = cu_seqlens[g], r1 = cu_seqlens[g + 1];
  if (r0 < 0 || r1 > rows || r1 < r0) {
    if (threadIdx.x == 0 && blockIdx.x == 0 && blockIdx.y == 0) report_status(B200_STATUS_BAD_INDEX, g);
    r0 = r0 < 0 ? 0 : (r0 > rows ? rows : r0);
    r1 = r1 > rows ? rows : r1;
    if (r1 < r0) r1 = r0;
  }
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int wm = (warp >> 2) * 64, wn = (warp & 3) * 32;        // this warp's 64 x 32 corner inside the tile
  float acc[4][4][4];                                            // [m16 tile][n8 tile][fragment]
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
      for (int e = 0; e < 4; ++e) acc[i][j][e] = 0.f;
  const uint32_t sa_base = (uint32_t)__cvta_generic_to_shared(&sa[0][0]);
  const uint32_t sb_base = (uint32_t)__cvta_generic_to_shared(&sb[0][0]);
  for (long long r = r0; r < r1; r += WGM_ROWS) {
    __syncthreads();                                             // the previous chunk has been consumed
#pragma unroll
    for (int it = 0; it < 2; ++it) {                             // 32 rows x 16 vectors of 8 columns per operand
      const int e = tid + it * 256, lr = e >> 4, lc = (e & 15) * 8;
      uint4 va = make_uint4(0, 0, 0, 0), vb = make_uint4(0, 0, 0, 0);
      if (r + lr < r1) {
        if (m0 + lc < M) va = *reinterpret_cast<const uint4*>(a + (r + lr) * M + m0 + lc);
        if (n0 + lc < N) vb = *reinterpret_cast<const uint4*>(b + (r + lr) * N + n0 + lc);
      }
      *reinterpret_cast<uint4*>(&sa[lr][lc]) = va;
      *reinterpret_cast<uint4*>(&sb[lr][lc]) = vb;
    }
    __syncthreads();
#pragma unroll
    for (int kk0 = 0; kk0 < WGM_ROWS; kk0 += 16) {
      uint32_t bf[4][2];
#pragma unroll
      for (int jp = 0; jp < 2; ++jp) {                           // two n8 tiles per ldmatrix
        const int row = kk0 + (lane & 7) + ((lane >> 3) & 1) * 8, col = wn + jp * 16 + (lane >> 4) * 8;
        ldmatrix_x4_trans(sb_base + (uint32_t)(row * WGM_LD + col) * 2, bf[2 * jp][0], bf[2 * jp][1],
                          bf[2 * jp + 1][0], bf[2 * jp + 1][1]);
      }
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int row = kk0 + (lane & 7) + (lane >> 4) * 8, col = wm + i * 16 + ((lane >> 3) & 1) * 8;
        uint32_t a0, a1, a2, a3;
        ldmatrix_x4_trans(sa_base + (uint32_t)(row * WGM_LD + col) * 2, a0, a1, a2, a3);
#pragma unroll
        for (int j = 0; j < 4; ++j) mma_bf16_16816(acc[i][j], a0, a1, a2, a3, bf[j][0], bf[j][1]);
      }
    }
  }
  __nv_bfloat16* cg = c + (long long)g * M * N;
  const int gid = lane >> 2, tig = lane & 3;
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + wn + j * 8 + 2 * tig;
      if (n >= N) continue;
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        const int m = m0 + wm + i * 16 + gid + half * 8;
        if (m < M)
          *reinterpret_cast<uint32_t*>(cg + (long long)m * N + n) = pack_bf2(acc[i][j][2 * half], acc[i][j][2 * half + 1]);
      }
    }
}

// out[g, c, r] = x[g, r, c] for 2-byte elements: 64 x 64 tiles through shared memory, 16-byte loads and stores.
// R and C multiples of 8.  (The dgrad grouped GEMM reads the expert weights with the other dimension contiguous.)
__global__ void __launch_bounds__(256)
transpose_last2_kernel(const uint16_t* __restrict__ x, uint16_t* __restrict__ out, int R, int C) {
  pdl_trigger();
  pdl_wait();
  __shared__ __align__(16) uint16_t t[64][72];
  const long long base = (long long)blockIdx.z * R * C;
  const int r0 = blockIdx.y * 64, c0 = blockIdx.x * 64, tid = threadIdx.x;
#pragma unroll
  for (int it = 0; it < 2; ++it) {
    const int e = tid + it * 256, lr = e >> 3, lc = (e & 7) * 8;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (r0 + lr < R && c0 + lc < C) v = *reinterpret_cast<const uint4*>(x + base + (long long)(r0 + lr) * C + c0 + lc);
    *reinterpret_cast<uint4*>(&t[lr][lc]) = v;
  }
  __syncthreads();
#pragma unroll
  for (int it = 0; it < 2; ++it) {
    const int e = tid + it * 256, oc = e >> 3, orr = (e & 7) * 8;     // output row oc (a source column), 8 source rows
    if (c0 + oc < C && r0 + orr < R) {
      uint16_t w[8];
#pragma unroll
      for (int k = 0; k < 8; ++k) w[k] = t[orr + k][oc];
      uint4 v;
      v.x = w[0] | ((uint32_t)w[1] << 16);
      v.y = w[2] | ((uint32_t)w[3] << 16);
      v.z = w[4] | ((uint32_t)w[5] << 16);
      v.w = w[6] | ((uint32_t)w[7] << 16);
      *reinterpret_cast<uint4*>(out + base + (long long)(c0 + oc) * R + r0 + orr) = v;
    }
  }
}

// h = bf16(bf16(bf16(silu(g)) * u) * s): the unfused tail of fc1 for split gate / up weights.
__global__ void __launch_bounds__(256)
swiglu_scale_kernel(const __nv_bfloat16* __restrict__ gate, const __nv_bfloat16* __restrict__ up,
                    const __nv_bfloat16* __restrict__ row_scale, __nv_bfloat16* __restrict__ out, long long rows,
                    int I, long long in_stride) {
  pdl_trigger();
  pdl_wait();
  const long long i = (long long)blockIdx.x * 256 + threadIdx.x;
  if (i >= rows * I) return;
  const long long r = i / I;
  const long long src = r * in_stride + (i - r * I);
  const float g = bf2f(gate[src]);
  const float u = bf2f(up[src]);
  const float sg = round_bf(g / (1.0f + expf(-g)));
  float h = round_bf(sg * u);
  if (row_scale) h = round_bf(h * bf2f(row_scale[r]));
  out[i] = f2bf(h);
}

}  // namespace b200

extern "C" int b200_moe_route_softmax_topk(const void* logits, int logits_dtype /*0 = f32, 1 = bf16*/,
                                           long long row_stride, void* weights_bf16, void* weights_f32,
                                           void* experts_i32, void* experts_i64, long long T, int E, int topk,
                                           int renorm, void* stream) {
  using namespace b200;
  if (!logits || T < 0 || E <= 0 || topk <= 0 || (!experts_i32 && !experts_i64) || (!weights_bf16 && !weights_f32))
    return B200_ERR_ARG;
  if (E > MOE_MAX_EXPERTS || topk > MOE_MAX_TOPK || topk > E) return B200_ERR_SHAPE;
  if (T == 0) return B200_OK;
  cudaStream_t st = (cudaStream_t)stream;
  const unsigned grid = (unsigned)((T + 7) / 8);
  if (logits_dtype == 0)
    launch_k(moe_route_softmax_topk_kernel<float>, dim3(grid), dim3(256), 0, st, 
        (const float*)logits, row_stride, (__nv_bfloat16*)weights_bf16, (float*)weights_f32, (int*)experts_i32,
        (long long*)experts_i64, T, E, topk, renorm);
  else if (logits_dtype == 1)
    launch_k(moe_route_softmax_topk_kernel<__nv_bfloat16>, dim3(grid), dim3(256), 0, st, 
        (const __nv_bfloat16*)logits, row_stride, (__nv_bfloat16*)weights_bf16, (float*)weights_f32,
        (int*)experts_i32, (long long*)experts_i64, T, E, topk, renorm);
  else
    return B200_ERR_ARG;
  return launch_status();
}

// ------------------------------------------------------------------ routing + plan in two launches
// The decode chain route -> index -> scatter is three dependent launches of which the middle one (a stable
// counting sort on one CTA) exists only to give every sorted row a position.  Which position a row gets
// inside its expert's group changes no result: a GEMM row's value does not depend on where the row sits, and
// the top-k sum finds its rows through scatter_index.  So the routing kernel hands out ranks itself (one
// atomicAdd per selected expert: counts[e]++), the last of its CTAs to finish (a ticket counter, nobody waits
// for anybody) turns the counts into cu_seqlens and the token-tile table and clears the counters for the next
// call, and the scatter kernel places row f at cu_seqlens[e] + rank[f].  The order of rows within an expert
// therefore varies from run to run; every output bit is the same.  b200_moe_permute keeps the stable order
// (it is what reproduces the reference's index arrays).
namespace b200 {

template <typename TIn>
__global__ void __launch_bounds__(256)
moe_route_plan_kernel(const TIn* __restrict__ logits, long long row_stride, __nv_bfloat16* __restrict__ w_bf16,
                      long long* __restrict__ idx_i64, int* __restrict__ rank_out, int* __restrict__ counters,
                      int* __restrict__ cu_seqlens, int4* __restrict__ tile_table, int* __restrict__ tile_count,
                      long long T, int E, int topk, int renorm, int tile_rows, int max_tiles) {
  pdl_trigger();
  pdl_wait();
  __shared__ int s_last;
  __shared__ int s_scan[2][8];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const long long tok = (long long)blockIdx.x * 8 + warp;
  if (tok < T) {
    route_softmax_topk_token<TIn>(logits + tok * row_stride, tok, w_bf16, nullptr, nullptr, idx_i64, E, topk, renorm,
                                  lane);
    __syncwarp();
    // the expert ids were just written by lane 0: lane k takes entry k's rank in its expert's group
    if (lane < topk) {
      const int e = (int)idx_i64[tok * topk + lane];
      rank_out[tok * topk + lane] = atomicAdd(&counters[e], 1);
    }
  }
  // counters[MOE_MAX_EXPERTS] is the ticket: the CTA that draws the last one sees every count
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) s_last = atomicAdd(&counters[MOE_MAX_EXPERTS], 1) == (int)gridDim.x - 1;
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  // 256 threads, one expert each (E <= MOE_MAX_EXPERTS = 256): exclusive scans of rows and tiles
  const int e = threadIdx.x;
  const int rows = e < E ? __ldcg(&counters[e]) : 0;
  const int tiles = (rows + tile_rows - 1) / tile_rows;
  int r = rows, t = tiles;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int r2 = __shfl_up_sync(0xffffffffu, r, o);
    const int t2 = __shfl_up_sync(0xffffffffu, t, o);
    if (lane >= o) {
      r += r2;
      t += t2;
    }
  }
  if (lane == 31) {
    s_scan[0][warp] = r;
    s_scan[1][warp] = t;
  }
  __syncthreads();
  int roff = 0, toff = 0;
  for (int w = 0; w < warp; ++w) {
    roff += s_scan[0][w];
    toff += s_scan[1][w];
  }
  const int rexcl = roff + r - rows, texcl = toff + t - tiles;
  if (e < E) {
    cu_seqlens[e] = rexcl;
    for (int j = 0; j < tiles; ++j)
      if (texcl + j < max_tiles)
        tile_table[texcl + j] = make_int4(e, rexcl + j * tile_rows, min(tile_rows, rows - j * tile_rows), 0);
    if (e == E - 1) {
      cu_seqlens[E] = rexcl + rows;
      *tile_count = min(texcl + tiles, max_tiles);
    }
    counters[e] = 0;   // ready for the next call
  }
  if (threadIdx.x == 0) counters[MOE_MAX_EXPERTS] = 0;
}

// Row f = (token f / topk, choice f % topk) goes to sorted row cu_seqlens[expert] + rank[f].
__global__ void __launch_bounds__(128)
moe_scatter_ranked_kernel(const __nv_bfloat16* __restrict__ x, long long x_stride,
                          const long long* __restrict__ experts, const __nv_bfloat16* __restrict__ weights,
                          const int* __restrict__ rank, const int* __restrict__ cu_seqlens,
                          int* __restrict__ scatter_index, __nv_bfloat16* __restrict__ x_perm,
                          __nv_bfloat16* __restrict__ row_scale, int H, int topk, int E, long long n) {
  pdl_trigger();
  pdl_wait();
  const long long f = blockIdx.x;
  const long long e = experts[f];
  if (e < 0 || e >= E) {
    if (threadIdx.x == 0) {
      report_status(B200_STATUS_BAD_INDEX, (int)e);
      scatter_index[f] = -1;
    }
    return;
  }
  const long long pos = (long long)cu_seqlens[e] + rank[f];
  if (pos < 0 || pos >= n) {   // counters that were not clean when the routing kernel ran
    if (threadIdx.x == 0) {
      report_status(B200_STATUS_BAD_INDEX, (int)pos);
      scatter_index[f] = -1;
    }
    return;
  }
  const __nv_bfloat16* src = x + (f / topk) * x_stride;
  __nv_bfloat16* dst = x_perm + pos * H;
  for (int i = threadIdx.x; i < (H >> 3); i += 128)
    reinterpret_cast<uint4*>(dst)[i] = reinterpret_cast<const uint4*>(src)[i];
  if (threadIdx.x == 0) {
    scatter_index[f] = (int)pos;
    if (row_scale && weights) row_scale[pos] = weights[f];
  }
}

}  // namespace b200

// Qwen3-MoE routing (modeling_qwen3_moe.py:128-134) that also plans the permutation: weights_bf16 [T, topk],
// experts_i64 [T, topk] as b200_moe_route_softmax_topk writes them, plus rank [T*topk] i32 (the row's place
// inside its expert's group), cu_seqlens [E+1], tile_table / tile_count as b200_moe_permute writes them.
// counters: E_max + 1 = 257 int32, zero before the first call; every call leaves them zero again.  Calls that
// share a counters array must not overlap on the GPU.
extern "C" int b200_moe_route_plan_softmax_topk(const void* logits, int logits_dtype /*0 = f32, 1 = bf16*/,
                                                long long row_stride, void* weights_bf16, void* experts_i64,
                                                void* rank_i32, void* counters_i32, void* cu_seqlens,
                                                void* tile_table, void* tile_count, long long T, int E, int topk,
                                                int renorm, int tile_rows, int max_tiles, void* stream) {
  using namespace b200;
  if (!logits || !weights_bf16 || !experts_i64 || !rank_i32 || !counters_i32 || !cu_seqlens || !tile_table ||
      !tile_count || T <= 0 || E <= 0 || topk <= 0 || tile_rows <= 0 || max_tiles <= 0)
    return B200_ERR_ARG;
  if (E > MOE_MAX_EXPERTS || topk > MOE_MAX_TOPK || topk > E || topk > 32) return B200_ERR_SHAPE;
  cudaStream_t st = (cudaStream_t)stream;
  const unsigned grid = (unsigned)((T + 7) / 8);
  if (logits_dtype == 0)
    launch_k(moe_route_plan_kernel<float>, dim3(grid), dim3(256), 0, st, (const float*)logits, row_stride,
             (__nv_bfloat16*)weights_bf16, (long long*)experts_i64, (int*)rank_i32, (int*)counters_i32,
             (int*)cu_seqlens, (int4*)tile_table, (int*)tile_count, T, E, topk, renorm, tile_rows, max_tiles);
  else if (logits_dtype == 1)
    launch_k(moe_route_plan_kernel<__nv_bfloat16>, dim3(grid), dim3(256), 0, st, (const __nv_bfloat16*)logits,
             row_stride, (__nv_bfloat16*)weights_bf16, (long long*)experts_i64, (int*)rank_i32, (int*)counters_i32,
             (int*)cu_seqlens, (int4*)tile_table, (int*)tile_count, T, E, topk, renorm, tile_rows, max_tiles);
  else
    return B200_ERR_ARG;
  return launch_status();
}

// The permuted copy for a plan made by b200_moe_route_plan_softmax_topk: x_perm, row_scale and scatter_index.
extern "C" int b200_moe_scatter_ranked(const void* x, long long x_row_stride, const void* experts_i64,
                                       const void* weights_bf16, const void* rank_i32, const void* cu_seqlens,
                                       void* scatter_index, void* x_perm, void* row_scale, long long T, int topk,
                                       int E, int H, void* stream) {
  using namespace b200;
  if (!x || !experts_i64 || !rank_i32 || !cu_seqlens || !scatter_index || !x_perm || T < 0 || topk <= 0 || E <= 0 ||
      H <= 0 || (row_scale && !weights_bf16))
    return B200_ERR_ARG;
  if (H % 8 != 0 || x_row_stride % 8 != 0) return B200_ERR_SHAPE;
  const long long n = T * topk;
  if (n == 0) return B200_OK;
  if (n > 0x7fffffffLL) return B200_ERR_SHAPE;
  launch_k(moe_scatter_ranked_kernel, dim3((unsigned)n), dim3(128), 0, (cudaStream_t)stream, (const __nv_bfloat16*)x,
           x_row_stride, (const long long*)experts_i64, (const __nv_bfloat16*)weights_bf16, (const int*)rank_i32,
           (const int*)cu_seqlens, (int*)scatter_index, (__nv_bfloat16*)x_perm, (__nv_bfloat16*)row_scale, H, topk, E, n);
  return launch_status();
}

extern "C" int b200_moe_route_sigmoid_group_topk(const void* logits_f32, long long row_stride,
                                                 const void* bias_f32, void* weights_f32, void* experts_i32,
                                                 void* experts_i64, long long T, int E, int n_group,
                                                 int topk_group, int topk, int renorm, float scale,
                                                 void* stream) {
  using namespace b200;
  if (!logits_f32 || !weights_f32 || (!experts_i32 && !experts_i64) || T < 0 || E <= 0 || n_group <= 0 ||
      topk_group <= 0 || topk <= 0)
    return B200_ERR_ARG;
  if (E > MOE_MAX_EXPERTS || topk > MOE_MAX_TOPK || n_group > 32 || E % n_group != 0 || topk_group > n_group ||
      E / n_group < 2)
    return B200_ERR_SHAPE;
  if (T == 0) return B200_OK;
  launch_k(moe_route_sigmoid_group_topk_kernel, dim3((unsigned)((T + 7) / 8)), dim3(256), 0, (cudaStream_t)stream, 
      (const float*)logits_f32, row_stride, (const float*)bias_f32, (float*)weights_f32, (int*)experts_i32,
      (long long*)experts_i64, T, E, n_group, topk_group, topk, renorm, scale);
  return launch_status();
}

// Builds the permutation (scatter_index, cu_seqlens, tile table) and moves the rows.
//   experts [T, topk] (int32 or int64), weights [T, topk] bf16 (may be null), x [T, H] bf16
//   -> scatter_index [T * topk] i32, cu_seqlens [E + 1] i32, x_perm [T * topk, H] bf16,
//      row_scale [T * topk] bf16 (if weights), tile_table [max_tiles] int4, tile_count [1] i32.
extern "C" int b200_moe_permute(const void* experts, int experts_dtype /*0 = i32, 1 = i64*/,
                                const void* weights_bf16, const void* x, long long x_row_stride,
                                void* scatter_index, void* cu_seqlens, void* x_perm, void* row_scale,
                                void* tile_table, void* tile_count, long long T, int topk, int E, int H,
                                int tile_rows, int max_tiles, void* stream) {
  using namespace b200;
  if (!experts || !scatter_index || !cu_seqlens || !tile_table || !tile_count || T < 0 || topk <= 0 || E <= 0 ||
      H <= 0 || tile_rows <= 0 || max_tiles <= 0)
    return B200_ERR_ARG;
  if (E > MOE_MAX_EXPERTS || H % 8 != 0 || x_row_stride % 8 != 0) return B200_ERR_SHAPE;
  cudaStream_t st = (cudaStream_t)stream;
  const long long n = T * topk;
  if (experts_dtype == 0)
    launch_k(moe_index_kernel<int>, dim3(1), dim3(1024), 0, st, (const int*)experts, n, E, tile_rows, (int*)scatter_index,
             (int*)cu_seqlens, (int4*)tile_table, (int*)tile_count, max_tiles, 1, (int*)nullptr,
             (const __nv_bfloat16*)nullptr, (__nv_bfloat16*)nullptr);
  else if (experts_dtype == 1)
    launch_k(moe_index_kernel<long long>, dim3(1), dim3(1024), 0, st, (const long long*)experts, n, E, tile_rows,
             (int*)scatter_index, (int*)cu_seqlens, (int4*)tile_table, (int*)tile_count, max_tiles, 1,
             (int*)nullptr, (const __nv_bfloat16*)nullptr, (__nv_bfloat16*)nullptr);
  else
    return B200_ERR_ARG;
  int rc = launch_status();
  if (rc || n == 0 || !x || !x_perm) return rc;
  launch_k(moe_scatter_rows_kernel, dim3((unsigned)n), dim3(128), 0, st, (const __nv_bfloat16*)x, x_row_stride,
                                                       (const __nv_bfloat16*)weights_bf16,
                                                       (const int*)scatter_index, (__nv_bfloat16*)x_perm,
                                                       (__nv_bfloat16*)row_scale, H, topk);
  return launch_status();
}

// b200_moe_permute without the permuted copy: the index arrays, plus gather_index [T * topk] i32 (sorted row
// -> token, the reference's `A_idx = order // topk`, fused_moe.py:285) and row_scale (routing weight per sorted
// row) for b200_moe_grouped_gemm_gather.  One launch.
extern "C" int b200_moe_permute_index(const void* experts, int experts_dtype /*0 = i32, 1 = i64*/,
                                      const void* weights_bf16, void* scatter_index, void* cu_seqlens,
                                      void* gather_index, void* row_scale, void* tile_table, void* tile_count,
                                      long long T, int topk, int E, int tile_rows, int max_tiles, void* stream) {
  using namespace b200;
  if (!experts || !scatter_index || !cu_seqlens || !gather_index || !tile_table || !tile_count || T < 0 ||
      topk <= 0 || E <= 0 || tile_rows <= 0 || max_tiles <= 0 || (row_scale && !weights_bf16))
    return B200_ERR_ARG;
  if (E > MOE_MAX_EXPERTS) return B200_ERR_SHAPE;
  cudaStream_t st = (cudaStream_t)stream;
  const long long n = T * topk;
  if (experts_dtype == 0)
    launch_k(moe_index_kernel<int>, dim3(1), dim3(1024), 0, st, (const int*)experts, n, E, tile_rows,
             (int*)scatter_index, (int*)cu_seqlens, (int4*)tile_table, (int*)tile_count, max_tiles, topk,
             (int*)gather_index, (const __nv_bfloat16*)weights_bf16, (__nv_bfloat16*)row_scale);
  else if (experts_dtype == 1)
    launch_k(moe_index_kernel<long long>, dim3(1), dim3(1024), 0, st, (const long long*)experts, n, E, tile_rows,
             (int*)scatter_index, (int*)cu_seqlens, (int4*)tile_table, (int*)tile_count, max_tiles, topk,
             (int*)gather_index, (const __nv_bfloat16*)weights_bf16, (__nv_bfloat16*)row_scale);
  else
    return B200_ERR_ARG;
  return launch_status();
}

extern "C" int b200_moe_unpermute_reduce(const void* y, const void* scatter_index, const void* addend,
                                         void* out, long long T, int topk, int H, void* stream) {
  using namespace b200;
  if (!y || !scatter_index || !out || T < 0 || topk <= 0 || H <= 0) return B200_ERR_ARG;
  if (H % 8 != 0) return B200_ERR_SHAPE;
  if (T == 0) return B200_OK;
  launch_k(moe_unpermute_reduce_kernel, dim3((unsigned)T), dim3(256), 0, (cudaStream_t)stream, 
      (const __nv_bfloat16*)y, (const int*)scatter_index, (const __nv_bfloat16*)addend, (__nv_bfloat16*)out, H,
      topk);
  return launch_status();
}

// out[index[t, k]] = x[t] for every (t, k): rows of a 2-byte element type, H a multiple of 8, x rows
// x_row_stride elements apart (a multiple of 8), out [out_rows, H] contiguous, index [T, topk] i32 with the
// given element strides.  An index outside [0, out_rows) is skipped and reported through the status word.
extern "C" int b200_moe_scatter(const void* x, long long x_row_stride, const void* index_i32,
                                long long index_stride_t, long long index_stride_k, void* out, long long out_rows,
                                long long T, int topk, int H, void* stream) {
  using namespace b200;
  if (!x || !index_i32 || !out || T < 0 || topk <= 0 || H <= 0 || out_rows < 0) return B200_ERR_ARG;
  if (H % 8 != 0 || x_row_stride % 8 != 0 || T * topk > 0x7fffffffLL) return B200_ERR_SHAPE;
  if (T == 0) return B200_OK;
  launch_k(moe_scatter_checked_kernel, dim3((unsigned)(T * topk)), dim3(128), 0, (cudaStream_t)stream,
           (const uint4*)x, x_row_stride / 8, (const int*)index_i32, index_stride_t, index_stride_k, (uint4*)out,
           out_rows, H / 8, topk);
  return launch_status();
}

// out[t] = bf16(sum over k, ascending, of fp32(x[index[t, k]])): x [x_rows, H] bf16 contiguous, out [T, H].
// An index outside [0, x_rows) contributes nothing and is reported through the status word.
extern "C" int b200_moe_gather(const void* x, long long x_rows, const void* index_i32, long long index_stride_t,
                               long long index_stride_k, void* out, long long T, int topk, int H, void* stream) {
  using namespace b200;
  if (!x || !index_i32 || !out || T < 0 || topk <= 0 || H <= 0 || x_rows < 0) return B200_ERR_ARG;
  if (H % 8 != 0 || T > 0x7fffffffLL) return B200_ERR_SHAPE;
  if (T == 0) return B200_OK;
  launch_k(moe_gather_checked_kernel, dim3((unsigned)T), dim3(256), 0, (cudaStream_t)stream,
           (const __nv_bfloat16*)x, x_rows, (const int*)index_i32, index_stride_t, index_stride_k,
           (__nv_bfloat16*)out, H, topk);
  return launch_status();
}

// out[g, c, r] = x[g, r, c]: x [G, R, C], out [G, C, R], contiguous, 2-byte elements, R and C multiples of 8,
// 16-byte aligned pointers.
extern "C" int b200_transpose_last2(const void* x, void* out, int G, int R, int C, void* stream) {
  using namespace b200;
  if (!x || !out || G <= 0 || R <= 0 || C <= 0) return B200_ERR_ARG;
  if (R % 8 != 0 || C % 8 != 0 || G > 65535 || (R + 63) / 64 > 65535 ||
      ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(out)) & 15) != 0)
    return B200_ERR_SHAPE;
  launch_k(transpose_last2_kernel, dim3((unsigned)((C + 63) / 64), (unsigned)((R + 63) / 64), (unsigned)G), dim3(256), 0,
           (cudaStream_t)stream, (const uint16_t*)x, (uint16_t*)out, R, C);
  return launch_status();
}

// c[g] = a[rows of g]^T @ b[rows of g]: a [rows, M], b [rows, N], c [G, M, N] bf16 contiguous, cu_seqlens
// [G + 1] i32 (rows of group g are [cu[g], cu[g + 1])).  M and N multiples of 4, 8-byte aligned pointers.
extern "C" int b200_moe_grouped_wgrad(const void* a, const void* b, void* c, const void* cu_seqlens, long long rows,
                                      int num_groups, int M, int N, void* stream) {
  using namespace b200;
  if (!a || !b || !c || !cu_seqlens || rows < 0 || num_groups <= 0 || M <= 0 || N <= 0) return B200_ERR_ARG;
  if (M % 4 != 0 || N % 4 != 0 || num_groups > 65535 || (M + WG_TILE - 1) / WG_TILE > 65535) return B200_ERR_SHAPE;
  static const int simt = env_int("B200_WGRAD_SIMT", 0);        // development knob: the CUDA-core kernel
  const bool vec16 = M % 8 == 0 && N % 8 == 0 &&
                     ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b)) & 15) == 0 &&
                     (reinterpret_cast<uintptr_t>(c) & 3) == 0;
  if (vec16 && !simt) {
    launch_k(moe_wgrad_mma_kernel, dim3((unsigned)((N + WGM_TILE - 1) / WGM_TILE),
                                        (unsigned)((M + WGM_TILE - 1) / WGM_TILE), (unsigned)num_groups),
             dim3(256), 0, (cudaStream_t)stream, (const __nv_bfloat16*)a, (const __nv_bfloat16*)b,
             (__nv_bfloat16*)c, (const int*)cu_seqlens, rows, M, N);
    return launch_status();
  }
  launch_k(moe_wgrad_kernel, dim3((unsigned)((N + WG_TILE - 1) / WG_TILE), (unsigned)((M + WG_TILE - 1) / WG_TILE),
                                  (unsigned)num_groups),
           dim3(256), 0, (cudaStream_t)stream, (const __nv_bfloat16*)a, (const __nv_bfloat16*)b, (__nv_bfloat16*)c,
           (const int*)cu_seqlens, rows, M, N);
  return launch_status();
}

// b200_moe_unpermute_reduce + b200_add_rmsnorm in one launch: sum_out = residual + moe output (the new
// residual stream), out = rmsnorm(sum_out) * weight.  H a multiple of 8 in 1032..8192.
extern "C" int b200_moe_unpermute_add_rmsnorm(const void* y, const void* scatter_index, const void* addend,
                                              const void* residual, const void* weight, void* sum_out, void* out,
                                              long long T, int topk, int H, float eps, int mode, void* stream) {
  using namespace b200;
  if (!y || !scatter_index || !residual || !weight || !sum_out || !out || T < 0 || topk <= 0 || H <= 0 ||
      (mode != 0 && mode != 1))
    return B200_ERR_ARG;
  // rows of up to 1024 elements go through the warp-per-row norm kernel, whose reduction tree differs
  if (H % 8 != 0 || H > 8192 || H <= 1024) return B200_ERR_SHAPE;
  if (((reinterpret_cast<uintptr_t>(y) | reinterpret_cast<uintptr_t>(residual) | reinterpret_cast<uintptr_t>(weight) |
        reinterpret_cast<uintptr_t>(sum_out) | reinterpret_cast<uintptr_t>(out) |
        reinterpret_cast<uintptr_t>(addend)) & 15) != 0)
    return B200_ERR_ARG;
  if (T == 0) return B200_OK;
  launch_k(moe_unpermute_add_rmsnorm_kernel, dim3((unsigned)T), dim3(128), 0, (cudaStream_t)stream,
           (const __nv_bfloat16*)y, (const int*)scatter_index, (const __nv_bfloat16*)addend,
           (const __nv_bfloat16*)residual, (const __nv_bfloat16*)weight, (__nv_bfloat16*)sum_out, (__nv_bfloat16*)out,
           H, topk, eps, mode);
  return launch_status();
}

extern "C" int b200_swiglu_scale_strided(const void* gate, const void* up, const void* row_scale, void* out,
                                         long long rows, int I, long long in_row_stride, void* stream) {
  using namespace b200;
  if (!gate || !up || !out || rows < 0 || I <= 0 || in_row_stride < I) return B200_ERR_ARG;
  if (rows == 0) return B200_OK;
  const long long n = rows * I;
  launch_k(swiglu_scale_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, (cudaStream_t)stream,
           (const __nv_bfloat16*)gate, (const __nv_bfloat16*)up, (const __nv_bfloat16*)row_scale, (__nv_bfloat16*)out,
           rows, I, in_row_stride);
  return launch_status();
}

extern "C" int b200_swiglu_scale(const void* gate, const void* up, const void* row_scale, void* out,
                                 long long rows, int I, void* stream) {
  return b200_swiglu_scale_strided(gate, up, row_scale, out, rows, I, I, stream);
}
