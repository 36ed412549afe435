// Paged KV-cache store, and the fused q/k-RMSNorm + RoPE + store used by the
// decoder-stack runner.  Pure copies and elementwise math: HBM-bound.
//
// b200_kv_store replaces vexact/batch_invariant_ops/kv_cache_context.py:260-314
// (_store_cache_kernel launched twice by store_kvcache): token i's [heads*dim]
// row goes to flat slot slot_mapping[i] of a cache laid out
// [blocks, page, heads, dim]; slot -1 is skipped.  K and V go in one launch and
// may have different head dims (MLA: 192 / 128).
//
// b200_qknorm_rope_store fuses what the HF Qwen3 / Qwen2 attention module does
// between the QKV projection and the attention call: per-head RMSNorm of q and k
// (HF formula, optional), rotary embedding with HF's rounding points
// (q*cos and rotate_half(q)*sin are each rounded to bf16, then added and rounded),
// and the store of k and v into the paged cache.
#pragma once
#include "common.cuh"

namespace b200 {

__global__ void __launch_bounds__(128)
kv_store_kernel(const __nv_bfloat16* __restrict__ k, const __nv_bfloat16* __restrict__ v,
                __nv_bfloat16* __restrict__ k_cache, __nv_bfloat16* __restrict__ v_cache,
                const int* __restrict__ slot_mapping, long long k_tok_stride, long long v_tok_stride,
                int k_row, int v_row, long long num_slots) {
  pdl_trigger();
  pdl_wait();
  const long long tok = blockIdx.x;
  const long long slot = slot_mapping[tok];
  if (slot < 0) return;
  if (slot >= num_slots) {
    report_status(B200_STATUS_BAD_INDEX, (int)slot);
    return;
  }
  const __nv_bfloat16* ks = k + tok * k_tok_stride;
  const __nv_bfloat16* vs = v + tok * v_tok_stride;
  __nv_bfloat16* kd = k_cache + slot * k_row;
  __nv_bfloat16* vd = v_cache + slot * v_row;
  const bool vec = ((reinterpret_cast<uintptr_t>(ks) | reinterpret_cast<uintptr_t>(vs) |
                     reinterpret_cast<uintptr_t>(kd) | reinterpret_cast<uintptr_t>(vd)) & 15) == 0 &&
                   (k_row % 8 == 0) && (v_row % 8 == 0);
  if (vec) {
    for (int i = threadIdx.x; i < (k_row >> 3); i += 128)
      reinterpret_cast<uint4*>(kd)[i] = reinterpret_cast<const uint4*>(ks)[i];
    for (int i = threadIdx.x; i < (v_row >> 3); i += 128)
      reinterpret_cast<uint4*>(vd)[i] = reinterpret_cast<const uint4*>(vs)[i];
  } else {
    for (int i = threadIdx.x; i < k_row; i += 128) kd[i] = ks[i];
    for (int i = threadIdx.x; i < v_row; i += 128) vd[i] = vs[i];
  }
}

// One CTA per token, eight warps taking its heads in turn (head h of the fused qkv row: q heads, then k heads,
// then v heads).  head_dim is 128: each lane owns 4 consecutive elements; rotate_half pairs element j with
// j +- 64, i.e. lane l with lane l ^ 16.  The token's 64 (cos, sin) pairs are computed once, by the CTA, while
// every warp's head slices are already on their way from memory.
__global__ void __launch_bounds__(256)
qknorm_rope_store_kernel(const __nv_bfloat16* __restrict__ qkv, long long qkv_stride,
                         const long long* __restrict__ positions, const int* __restrict__ slot_mapping,
                         const __nv_bfloat16* __restrict__ q_norm_w, const __nv_bfloat16* __restrict__ k_norm_w,
                         const float* __restrict__ inv_freq, __nv_bfloat16* __restrict__ q_out,
                         __nv_bfloat16* __restrict__ k_cache, __nv_bfloat16* __restrict__ v_cache,
                         int num_q_heads, int num_kv_heads, long long num_tokens, long long num_slots,
                         float eps) {
  pdl_trigger();
  pdl_wait();
  constexpr int D = 128, MAXH = 8;   // heads per warp held in registers at a time
  const int heads_total = num_q_heads + 2 * num_kv_heads;
  __shared__ float s_cos[64], s_sin[64];
  const long long tok = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const __nv_bfloat16* row = qkv + tok * qkv_stride;
  const long long slot = slot_mapping[tok];
  for (int h0 = 0; h0 < heads_total; h0 += 8 * MAXH) {
    // this warp's heads of the chunk: h0 + warp, h0 + warp + 8, ...; all their slices are requested first
    uint2 raw[MAXH];
#pragma unroll
    for (int i = 0; i < MAXH; ++i) {
      const int head = h0 + warp + 8 * i;
      raw[i] = head < heads_total ? *reinterpret_cast<const uint2*>(row + (long long)head * D + lane * 4)
                                  : make_uint2(0u, 0u);
    }
    if (h0 == 0) {
      if (threadIdx.x < 64) {
        const float ang = (float)positions[tok] * inv_freq[threadIdx.x];
        s_cos[threadIdx.x] = round_bf(cosf(ang));
        s_sin[threadIdx.x] = round_bf(sinf(ang));
      }
      __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < MAXH; ++i) {
      const int head = h0 + warp + 8 * i;
      if (head >= heads_total) break;
      const bool is_q = head < num_q_heads;
      const bool is_k = !is_q && head < num_q_heads + num_kv_heads;
      if (!is_q) {
        if (slot < 0) continue;  // padded token: nothing to cache
        if (slot >= num_slots) {
          if (lane == 0) report_status(B200_STATUS_BAD_INDEX, (int)slot);
          continue;
        }
      }
      if (!is_q && !is_k) {  // V: plain copy into the cache
        const int kvh = head - num_q_heads - num_kv_heads;
        *reinterpret_cast<uint2*>(v_cache + (slot * num_kv_heads + kvh) * D + lane * 4) = raw[i];
        continue;
      }
      float x[4];
      unpack_bf2(raw[i].x, x[0], x[1]);
      unpack_bf2(raw[i].y, x[2], x[3]);
      const __nv_bfloat16* nw = is_q ? q_norm_w : k_norm_w;
      if (nw != nullptr) {
        float ss = 0.f;
#pragma unroll
        for (int j = 0; j < 4; ++j) ss += x[j] * x[j];
        ss = warp_sum(ss);
        const float inv = rsqrtf(ss / (float)D + eps);
        const uint2 wr = *reinterpret_cast<const uint2*>(nw + lane * 4);
        float w[4];
        unpack_bf2(wr.x, w[0], w[1]);
        unpack_bf2(wr.y, w[2], w[3]);
#pragma unroll
        for (int j = 0; j < 4; ++j) x[j] = round_bf(w[j] * round_bf(x[j] * inv));
      }
      // RoPE.  cos/sin are bf16 tensors in the HF model: emb = cat(freqs, freqs),
      // freqs[j] = position * inv_freq[j] in fp32, cos = bf16(cos(emb)).
      float partner[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) partner[j] = __shfl_xor_sync(0xffffffffu, x[j], 16);
      const bool upper = lane >= 16;  // elements 64..127
      float y[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int fi = (lane & 15) * 4 + j;  // frequency index in [0, 64)
        const float rot = upper ? partner[j] : -partner[j];  // rotate_half: cat(-x2, x1)
        y[j] = round_bf(round_bf(x[j] * s_cos[fi]) + round_bf(rot * s_sin[fi]));
      }
      uint2 o;
      o.x = pack_bf2(y[0], y[1]);
      o.y = pack_bf2(y[2], y[3]);
      if (is_q) {
        *reinterpret_cast<uint2*>(q_out + (tok * num_q_heads + head) * D + lane * 4) = o;
      } else {
        const int kvh = head - num_q_heads;
        *reinterpret_cast<uint2*>(k_cache + (slot * num_kv_heads + kvh) * D + lane * 4) = o;
      }
    }
  }
}

// Multi-head latent attention (DeepSeek-V3 / Moonlight): what deepseek_v3_attention_forward
// (vexact/models/deepseek_v3/modeling_deepseek_v3.py:225-283) does between its projections and the
// attention call.  One warp per (token, head):
//   q  [T, heads, nope + rope]  : nope part copied, rope part rotated        -> q_out [T, heads, nope + rope]
//   kvb[T, heads, nope + dv]    : k_nope | value (output of kv_b_proj)
//   kr [T, rope]                : the shared rotary key (last columns of kv_a_proj_with_mqa)
//   K cache row = cat(k_nope[h], rot(kr)) (the rotated shared key is repeated for every head, as the
//   reference's k_rot.expand does), V cache row = value[h].
// Rotary embedding is HF's apply_rotary_pos_emb_interleave: pairs (x[2j], x[2j+1]) are first
// de-interleaved to (first half, second half), then rotate_half is applied with bf16 cos/sin and bf16
// products, and the result stays in the de-interleaved order.  rope dim is 64: lane j owns pair j.
__global__ void __launch_bounds__(256)
mla_rope_store_kernel(const __nv_bfloat16* __restrict__ q, long long q_stride,
                      const __nv_bfloat16* __restrict__ kvb, long long kvb_stride,
                      const __nv_bfloat16* __restrict__ kr, long long kr_stride,
                      const long long* __restrict__ positions, const int* __restrict__ slot_mapping,
                      const float* __restrict__ inv_freq, __nv_bfloat16* __restrict__ q_out,
                      __nv_bfloat16* __restrict__ k_cache, __nv_bfloat16* __restrict__ v_cache, int heads,
                      int nope, int dv, long long num_tokens, long long num_slots) {
  pdl_trigger();
  pdl_wait();
  constexpr int ROPE = 64;
  const long long wid = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (wid >= num_tokens * heads) return;
  const int lane = threadIdx.x & 31;
  const long long tok = wid / heads;
  const int head = (int)(wid % heads);
  const int dq = nope + ROPE;
  const float pos = (float)positions[tok];
  const float ang = pos * inv_freq[lane];
  const float c = round_bf(cosf(ang)), sn = round_bf(sinf(ang));
  auto rotate = [&](uint32_t pair, float& first, float& second) {
    float xe, xo;  // x[2j], x[2j+1]
    unpack_bf2(pair, xe, xo);
    first = round_bf(round_bf(xe * c) + round_bf(-xo * sn));   // (q*cos) + (rotate_half(q)*sin), first half
    second = round_bf(round_bf(xo * c) + round_bf(xe * sn));   // second half
  };
  // ---- query
  const __nv_bfloat16* qs = q + tok * q_stride + (long long)head * dq;
  __nv_bfloat16* qd = q_out + (tok * heads + head) * dq;
  for (int i = lane; i < (nope >> 1); i += 32)
    reinterpret_cast<uint32_t*>(qd)[i] = reinterpret_cast<const uint32_t*>(qs)[i];
  {
    float f, s2;
    rotate(reinterpret_cast<const uint32_t*>(qs + nope)[lane], f, s2);
    qd[nope + lane] = f2bf(f);
    qd[nope + 32 + lane] = f2bf(s2);
  }
  // ---- key / value into the paged caches
  const long long slot = slot_mapping[tok];
  if (slot < 0) return;
  if (slot >= num_slots) {
    if (lane == 0) report_status(B200_STATUS_BAD_INDEX, (int)slot);
    return;
  }
  const __nv_bfloat16* ks = kvb + tok * kvb_stride + (long long)head * (nope + dv);
  __nv_bfloat16* kd = k_cache + (slot * heads + head) * dq;
  __nv_bfloat16* vd = v_cache + (slot * heads + head) * dv;
  for (int i = lane; i < (nope >> 1); i += 32)
    reinterpret_cast<uint32_t*>(kd)[i] = reinterpret_cast<const uint32_t*>(ks)[i];
  for (int i = lane; i < (dv >> 1); i += 32)
    reinterpret_cast<uint32_t*>(vd)[i] = reinterpret_cast<const uint32_t*>(ks + nope)[i];
  {
    float f, s2;
    rotate(reinterpret_cast<const uint32_t*>(kr + tok * kr_stride)[lane], f, s2);
    kd[nope + lane] = f2bf(f);
    kd[nope + 32 + lane] = f2bf(s2);
  }
}

}  // namespace b200

extern "C" int b200_kv_store(const void* key, const void* value, void* k_cache, void* v_cache,
                             const void* slot_mapping, long long num_tokens, int num_kv_heads, int k_head_dim,
                             int v_head_dim, long long k_token_stride, long long v_token_stride,
                             long long num_slots, void* stream) {
  using namespace b200;
  if (!key || !value || !k_cache || !v_cache || !slot_mapping || num_tokens < 0 || num_kv_heads <= 0 ||
      k_head_dim <= 0 || v_head_dim <= 0 || num_slots < 0)
    return B200_ERR_ARG;
  if (num_tokens == 0) return B200_OK;
  launch_k(kv_store_kernel, dim3((unsigned)num_tokens), dim3(128), 0, (cudaStream_t)stream, 
      (const __nv_bfloat16*)key, (const __nv_bfloat16*)value, (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache,
      (const int*)slot_mapping, k_token_stride, v_token_stride, num_kv_heads * k_head_dim,
      num_kv_heads * v_head_dim, num_slots);
  return launch_status();
}

extern "C" int b200_qknorm_rope_store(const void* qkv, long long qkv_token_stride, const void* positions,
                                      const void* slot_mapping, const void* q_norm_weight,
                                      const void* k_norm_weight, const void* inv_freq, void* q_out,
                                      void* k_cache, void* v_cache, long long num_tokens, int num_q_heads,
                                      int num_kv_heads, int head_dim, long long num_slots, float eps,
                                      void* stream) {
  using namespace b200;
  if (!qkv || !positions || !slot_mapping || !inv_freq || !q_out || !k_cache || !v_cache || num_tokens < 0 ||
      num_q_heads <= 0 || num_kv_heads <= 0)
    return B200_ERR_ARG;
  if (head_dim != 128) return B200_ERR_SHAPE;
  if ((q_norm_weight == nullptr) != (k_norm_weight == nullptr)) return B200_ERR_ARG;
  if (qkv_token_stride % 4 != 0 || (reinterpret_cast<uintptr_t>(qkv) & 7) != 0) return B200_ERR_ARG;
  if (num_tokens == 0) return B200_OK;
  if (num_tokens > 0x7fffffffLL) return B200_ERR_SHAPE;
  launch_k(qknorm_rope_store_kernel, dim3((unsigned)num_tokens), dim3(256), 0, (cudaStream_t)stream, 
      (const __nv_bfloat16*)qkv, qkv_token_stride, (const long long*)positions, (const int*)slot_mapping,
      (const __nv_bfloat16*)q_norm_weight, (const __nv_bfloat16*)k_norm_weight, (const float*)inv_freq,
      (__nv_bfloat16*)q_out, (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache, num_q_heads, num_kv_heads,
      num_tokens, num_slots, eps);
  return launch_status();
}

extern "C" int b200_mla_rope_store(const void* q, long long q_token_stride, const void* kvb,
                                   long long kvb_token_stride, const void* k_rot, long long k_rot_token_stride,
                                   const void* positions, const void* slot_mapping, const void* inv_freq,
                                   void* q_out, void* k_cache, void* v_cache, long long num_tokens, int num_heads,
                                   int qk_nope_dim, int qk_rope_dim, int v_dim, long long num_slots,
                                   void* stream) {
  using namespace b200;
  if (!q || !kvb || !k_rot || !positions || !slot_mapping || !inv_freq || !q_out || !k_cache || !v_cache ||
      num_tokens < 0 || num_heads <= 0)
    return B200_ERR_ARG;
  if (qk_rope_dim != 64 || qk_nope_dim % 2 || v_dim % 2 || qk_nope_dim <= 0 || v_dim <= 0) return B200_ERR_SHAPE;
  if (q_token_stride % 2 || kvb_token_stride % 2 || k_rot_token_stride % 2 ||
      ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(kvb) | reinterpret_cast<uintptr_t>(k_rot)) & 3))
    return B200_ERR_ARG;
  if (num_tokens == 0) return B200_OK;
  const long long warps = num_tokens * num_heads;
  launch_k(mla_rope_store_kernel, dim3((unsigned)((warps + 7) / 8)), dim3(256), 0, (cudaStream_t)stream,
           (const __nv_bfloat16*)q, q_token_stride, (const __nv_bfloat16*)kvb, kvb_token_stride,
           (const __nv_bfloat16*)k_rot, k_rot_token_stride, (const long long*)positions,
           (const int*)slot_mapping, (const float*)inv_freq, (__nv_bfloat16*)q_out, (__nv_bfloat16*)k_cache,
           (__nv_bfloat16*)v_cache, num_heads, qk_nope_dim, v_dim, num_tokens, num_slots);
  return launch_status();
}
