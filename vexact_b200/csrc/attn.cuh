// Causal paged-KV attention forward (decode, chunked prefill and full prefill in
// one kernel).
//
// Replaces vexact/batch_invariant_ops/triton_invariant_attention.py:434-603
// (_paged_attn_fwd_block_kernel) and the FA3/FA4 calls of
// vexact/batch_invariant_ops/flash_attention.py:142-178 (num_splits = 1).
//
// Work unit.  One warp (= one CTA) owns up to 8 "columns" of one KV head, a
// column being one (query position, query head) pair: for a GQA group of G <= 8
// heads a CTA covers floor(8 / G) consecutive query positions of one sequence,
// so a decode step of Qwen3-30B-A3B (G = 8) fills the tile with one token.  The
// CTA streams that sequence's K and V pages once, 64 keys per stage, through a
// ring of shared-memory stages written by TMA (4-D tensor map over the cache
// [blocks, page, kv_heads, dim], one box per page and 64-element half of the
// head dim, 128-byte swizzle, so the tiles are bank-conflict free for ldmatrix).
//
// Orientation.  S^T[key, col] = K[key, :] . Q[col, :] and
// O^T[d, col] = sum_key V[key, d] * P^T[key, col]: keys (then d) sit on the MMA M
// axis and the 8 columns on the N axis, so no MMA row is wasted on padding in
// decode.  P^T is re-laid out from accumulator to B-operand form with movmatrix.
//
// Invariance.  Every column walks the keys from 0 upward in fixed 64-key blocks
// with one online-softmax update per block (base-2, scale folded in, P rounded
// to bf16 before the PV product and before the row sum, as the reference does);
// masked keys contribute exactly 0 and leave max / sum / accumulator bitwise
// unchanged, so a token's result does not depend on how many other tokens share
// the tile, on its slot in the tile, or on whether it arrives as decode, as a
// prefill chunk or in a full prefill.  There is no split over KV.
//
// Algorithmic bytes per launch: sum over sequences of ctx * kv_heads * (Dk + Dv) * 2
// (each K/V element once) + Q read + O write: the roofline is HBM bandwidth.
#pragma once
#include <cuda.h>

#include "ptx.cuh"
#include "tmap.cuh"

namespace b200 {

constexpr int ATT_BN = 64;  // keys per stage

struct AttnParams {
  const __nv_bfloat16* q;  // [total_q, num_q_heads, DK]
  __nv_bfloat16* out;      // [total_q, num_q_heads, DV]
  long long q_tok_stride, q_head_stride, o_tok_stride, o_head_stride;
  const int* cu_seqlens_q;  // [num_seqs + 1]
  const int* seqused_k;     // [num_seqs]
  const int* page_table;    // [num_seqs, page_table_stride]
  long long page_table_stride;
  int max_pages;  // page-table columns
  int page_size;
  int box_tokens;  // tokens per TMA box = min(page_size, ATT_BN)
  int num_q_heads, num_kv_heads, group;
  int pos_per_tile;  // query positions per CTA = 8 / min(group, 8)
  int head_chunks;   // ceil(group / 8)
  float qk_scale;    // softmax_scale * log2(e)
  int num_blocks;    // cache blocks
  // tcgen05 kernel (persistent CTAs): tile grid dims and total
  int tc_q_tiles, tc_hy, tc_tiles;
  int tc_slots;          // tile positions walked: tc_tiles rounded up to whole rounds of the grid
  int num_seqs;
  const int* seq_order;  // [num_seqs] sequence of each slot (longest first), or null
  int max_seqlen_q;      // the caller's bound on queries per sequence: it sized the tile grid
  int q_tma;             // rows-on-lanes kernel: the query tile comes by TMA (a 3-D box over [token, head, dim])
  int o_tma;             // rows-on-lanes kernel: a warp's 32 output rows leave by one asynchronous TMA store
  int scalar_out;        // development knob B200_ATTN_OUT_SCALAR=1: 2-byte output stores in the keys-on-lanes kernel
};

__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2,
                                            uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2,
                                                  uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}
__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t v) {
  uint32_t r;
  asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(r) : "r"(v));
  return r;
}
__device__ __forceinline__ void mma_bf16_16816(float* c, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                               uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
      "{%0, %1, %2, %3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Byte offset of (row, 16-byte chunk) inside a [rows][64 x bf16] tile stored with the 128-byte swizzle.
__device__ __forceinline__ uint32_t sw128(int row, int chunk) {
  return (uint32_t)(row * 128 + ((chunk ^ (row & 7)) << 4));
}

template <int DK, int DV, int STAGES>
__global__ void __launch_bounds__(32)
paged_attn_kernel(const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v,
                  const AttnParams p) {
  constexpr int KH = DK / 64, VH = DV / 64;  // 64-wide halves of the head dims
  constexpr int K_BYTES = ATT_BN * DK * 2, V_BYTES = ATT_BN * DV * 2;
  constexpr int STAGE_BYTES = K_BYTES + V_BYTES;
  extern __shared__ uint8_t smem_raw[];
  __shared__ uint64_t full_bar_mem[STAGES];
  __shared__ int abort_mem;
  volatile int* abort_flag = &abort_mem;
  const uint32_t tile_base = (ptx::smem_u32(smem_raw) + 1023) & ~1023u;
  uint8_t* tile_ptr = smem_raw + (tile_base - ptx::smem_u32(smem_raw));

  pdl_trigger();
  pdl_wait();
  const int lane = threadIdx.x;
  const int g = lane >> 2, t = lane & 3;
  // KV heads vary fastest in launch order, so the CTAs that walk the same sequence's pages (one
  // per KV head) run at the same time and share DRAM pages and 256-byte L2 sectors.
  const int seq = blockIdx.z;
  const int kvh = blockIdx.y / p.head_chunks;
  const int hchunk = blockIdx.y % p.head_chunks;
  const int heads_here = min(8, p.group - hchunk * 8);  // query heads of this KV head covered by the CTA

  const int q_start = p.cu_seqlens_q[seq];
  const int q_len = p.cu_seqlens_q[seq + 1] - q_start;
  const int kv_len = p.seqused_k[seq];
  const int tile_pos0 = blockIdx.x * p.pos_per_tile;  // first query index (within the sequence) of this tile
  if (q_len > p.max_seqlen_q || (q_len > 0 && kv_len < q_len)) {
    // more queries than the grid was sized for, or fewer keys than queries: the tail rows would be
    // skipped silently / the first query's absolute position would be negative.  Flag it, compute nothing.
    if (lane == 0) report_status(B200_STATUS_BAD_INDEX, seq);
    return;
  }
  if (q_len <= 0 || kv_len <= 0 || tile_pos0 >= q_len) return;
  const int q_abs0 = kv_len - q_len;  // absolute position of the sequence's first query

  // Column c (0..7) -> (position index pi, head index hi).  Unused columns copy column 0's
  // position with a zero query so that all their arithmetic stays finite.
  auto col_valid = [&](int c) {
    const int pi = c / heads_here;
    return pi < p.pos_per_tile && tile_pos0 + pi < q_len;
  };
  auto col_qidx = [&](int c) { return tile_pos0 + (col_valid(c) ? c / heads_here : 0); };
  auto col_head = [&](int c) { return kvh * p.group + hchunk * 8 + (c % heads_here); };

  int last_q = tile_pos0 + p.pos_per_tile - 1;
  if (last_q > q_len - 1) last_q = q_len - 1;
  const int max_pos = q_abs0 + last_q;
  const int nblk = max_pos / ATT_BN + 1;

  if (lane == 0) {
    *abort_flag = 0;
    for (int s = 0; s < STAGES; ++s) ptx::mbar_init(ptx::smem_u32(&full_bar_mem[s]), 1);
    ptx::fence_barrier_init();
    ptx::prefetch_tensormap(&tm_k);
    ptx::prefetch_tensormap(&tm_v);
  }
  __syncwarp();

  const int boxes_per_blk = ATT_BN / p.box_tokens;
  const int* ptab = p.page_table + (long long)seq * p.page_table_stride;
  const int valid_pages = (kv_len + p.page_size - 1) / p.page_size;

  auto issue_block = [&](int blk) {
    // Warp-collective.  Lane b looks up the page of box b and issues its copies, so the page-table
    // reads of one block overlap.  Every box is always issued so the byte count is constant; boxes
    // wholly beyond the sequence use an out-of-range block coordinate and are zero-filled by TMA.
    const int s = blk % STAGES;
    const uint32_t bar = ptx::smem_u32(&full_bar_mem[s]);
    const uint32_t sk = tile_base + (uint32_t)s * STAGE_BYTES;
    const uint32_t sv = sk + K_BYTES;
    ptx::fence_proxy_async_smem();  // this lane's reads of the stage come before the refill
    __syncwarp();
    if (lane == 0) ptx::mbar_expect_tx(bar, STAGE_BYTES);
    __syncwarp();
    if (lane < boxes_per_blk) {
      const int b = lane;
      const int tok = blk * ATT_BN + b * p.box_tokens;
      const int lpage = tok / p.page_size;
      const int in_page = tok - lpage * p.page_size;
      int phys = -1;
      if (lpage < valid_pages && lpage < p.max_pages) phys = ptab[lpage];
      if (phys < 0 || phys >= p.num_blocks) phys = -1;
      const uint32_t row_off = (uint32_t)(b * p.box_tokens) * 128;
#pragma unroll
      for (int h = 0; h < KH; ++h)
        ptx::tma_load_4d(sk + h * (ATT_BN * 128) + row_off, &tm_k, bar, h * 64, kvh, in_page, phys,
                         ptx::kEvictFirst);
#pragma unroll
      for (int h = 0; h < VH; ++h)
        ptx::tma_load_4d(sv + h * (ATT_BN * 128) + row_off, &tm_v, bar, h * 64, kvh, in_page, phys,
                         ptx::kEvictFirst);
    }
  };

  for (int b = 0; b < STAGES && b < nblk; ++b) issue_block(b);

  // Q^T as the B operand of S^T = K Q^T: column g, d = kk*16 + 2t (+8).
  uint32_t qb[DK / 16][2];
  {
    const bool v = col_valid(g);
    const __nv_bfloat16* qrow =
        p.q + (long long)(q_start + col_qidx(g)) * p.q_tok_stride + (long long)col_head(g) * p.q_head_stride;
#pragma unroll
    for (int kk = 0; kk < DK / 16; ++kk) {
      qb[kk][0] = v ? *reinterpret_cast<const uint32_t*>(qrow + kk * 16 + 2 * t) : 0u;
      qb[kk][1] = v ? *reinterpret_cast<const uint32_t*>(qrow + kk * 16 + 8 + 2 * t) : 0u;
    }
  }
  // This thread's two columns (2t, 2t+1): absolute query positions for the causal mask.
  int cpos[2];
#pragma unroll
  for (int j = 0; j < 2; ++j) cpos[j] = q_abs0 + col_qidx(2 * t + j);

  float o[DV / 16][4];
#pragma unroll
  for (int i = 0; i < DV / 16; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};

  bool ok = true;
  for (int blk = 0; blk < nblk; ++blk) {
    const int s = blk % STAGES;
    ok = ptx::mbar_wait(ptx::smem_u32(&full_bar_mem[s]), (blk / STAGES) & 1, abort_flag, 500 + s);
    ok = __all_sync(0xffffffffu, ok);
    if (!ok) break;
    const uint32_t sk = tile_base + (uint32_t)s * STAGE_BYTES;
    const uint32_t sv = sk + K_BYTES;
    const int key0 = blk * ATT_BN;

    // Keys at or beyond kv_len may hold anything (stale or never written): their scores are masked
    // below, and their V rows are cleared here so that 0 * V stays 0.
    if (key0 + ATT_BN > kv_len) {
      const int first_bad = kv_len - key0;
      uint8_t* vt = tile_ptr + (size_t)s * STAGE_BYTES + K_BYTES;
      for (int r = first_bad; r < ATT_BN; ++r)
#pragma unroll
        for (int h = 0; h < VH; ++h)
          reinterpret_cast<uint32_t*>(vt + h * (ATT_BN * 128) + r * 128)[lane] = 0u;
      __syncwarp();
    }

    // ---- S^T = K Q^T : 4 m-tiles of 16 keys, DK/16 k-steps.
    float sc[ATT_BN / 16][4];
#pragma unroll
    for (int mt = 0; mt < ATT_BN / 16; ++mt) {
      sc[mt][0] = sc[mt][1] = sc[mt][2] = sc[mt][3] = 0.f;
#pragma unroll
      for (int kk = 0; kk < DK / 16; ++kk) {
        const int mi = lane >> 3;
        const int key = mt * 16 + (mi & 1) * 8 + (lane & 7);
        const int chunk = kk * 2 + (mi >> 1);
        uint32_t a0, a1, a2, a3;
        ldmatrix_x4(sk + (chunk >> 3) * (ATT_BN * 128) + sw128(key, chunk & 7), a0, a1, a2, a3);
        mma_bf16_16816(sc[mt], a0, a1, a2, a3, qb[kk][0], qb[kk][1]);
      }
    }

    // ---- online softmax per column (thread owns columns 2t, 2t+1; keys g and g+8 of each m-tile).
    float alpha[2];
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      float mx = -INFINITY;
#pragma unroll
      for (int mt = 0; mt < ATT_BN / 16; ++mt) {
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
          const int key = key0 + mt * 16 + g + hh * 8;
          float v = sc[mt][hh * 2 + j] * p.qk_scale;
          if (key > cpos[j]) v = -INFINITY;
          sc[mt][hh * 2 + j] = v;
          mx = fmaxf(mx, v);
        }
      }
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 4));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 8));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 16));
      const float m_new = fmaxf(m_run[j], mx);  // finite from block 0 on: key 0 is never masked
      alpha[j] = exp2f(m_run[j] - m_new);       // exp2(-inf) = 0 on the first block
      float sum = 0.f;
#pragma unroll
      for (int mt = 0; mt < ATT_BN / 16; ++mt) {
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
          const float pv = round_bf(exp2f(sc[mt][hh * 2 + j] - m_new));
          sc[mt][hh * 2 + j] = pv;
          sum += pv;
        }
      }
      sum += __shfl_xor_sync(0xffffffffu, sum, 4);
      sum += __shfl_xor_sync(0xffffffffu, sum, 8);
      sum += __shfl_xor_sync(0xffffffffu, sum, 16);
      l_run[j] = l_run[j] * alpha[j] + sum;
      m_run[j] = m_new;
    }
#pragma unroll
    for (int i = 0; i < DV / 16; ++i) {
      o[i][0] *= alpha[0];
      o[i][1] *= alpha[1];
      o[i][2] *= alpha[0];
      o[i][3] *= alpha[1];
    }

    // ---- P^T as B operand: per 16-key step, b0 = keys 2t..2t+1 (of the low 8), b1 = of the high 8.
    uint32_t pb[ATT_BN / 16][2];
#pragma unroll
    for (int mt = 0; mt < ATT_BN / 16; ++mt) {
      pb[mt][0] = movmatrix_trans(pack_bf2(sc[mt][0], sc[mt][1]));
      pb[mt][1] = movmatrix_trans(pack_bf2(sc[mt][2], sc[mt][3]));
    }

    // ---- O^T += V^T P^T : DV/16 m-tiles of d, 4 k-steps of 16 keys.
#pragma unroll
    for (int dm = 0; dm < DV / 16; ++dm) {
#pragma unroll
      for (int kk = 0; kk < ATT_BN / 16; ++kk) {
        const int mi = lane >> 3;
        const int key = kk * 16 + (mi >> 1) * 8 + (lane & 7);
        const int chunk = dm * 2 + (mi & 1);
        uint32_t a0, a1, a2, a3;
        ldmatrix_x4_trans(sv + (chunk >> 3) * (ATT_BN * 128) + sw128(key, chunk & 7), a0, a1, a2, a3);
        mma_bf16_16816(o[dm], a0, a1, a2, a3, pb[kk][0], pb[kk][1]);
      }
    }

    // Refill this stage for block blk + STAGES.  All reads of the stage are complete (their
    // results were consumed by the MMAs above); order them before the async-proxy write.
    __syncwarp();
    if (blk + STAGES < nblk) issue_block(blk + STAGES);
  }

  if (ok) {
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const int c = 2 * t + j;
      if (!col_valid(c)) continue;
      const float inv = 1.0f / l_run[j];
      __nv_bfloat16* orow = p.out + (long long)(q_start + col_qidx(c)) * p.o_tok_stride +
                            (long long)col_head(c) * p.o_head_stride;
#pragma unroll
      for (int dm = 0; dm < DV / 16; ++dm) {
        orow[dm * 16 + g] = f2bf(o[dm][j] * inv);
        orow[dm * 16 + g + 8] = f2bf(o[dm][2 + j] * inv);
      }
    }
  } else if (lane == 0) {
    // Aborted: leave time for TMA copies still in flight to land in this CTA's shared memory.
    const uint64_t t0 = global_timer_ns();
    while (global_timer_ns() - t0 < 200000ull) {
    }
  }
}

// 4-D map over a cache [blocks, page, heads, dim] (strides in elements); box = 64 x 1 x box_tokens x 1.
inline int make_tmap_cache(CUtensorMap* m, const void* base, int num_blocks, int page, int heads, int dim,
                           long long block_stride, long long page_stride, long long head_stride,
                           int box_tokens) {
  EncodeTiledFn enc = tensor_map_encoder();
  if (!enc) return B200_ERR_DRIVER;
  if ((reinterpret_cast<uintptr_t>(base) & 15) || (block_stride * 2) % 16 || (page_stride * 2) % 16 ||
      (head_stride * 2) % 16)
    return B200_ERR_ARG;
  cuuint64_t dims[4] = {(cuuint64_t)dim, (cuuint64_t)heads, (cuuint64_t)page, (cuuint64_t)num_blocks};
  cuuint64_t strides[3] = {(cuuint64_t)head_stride * 2, (cuuint64_t)page_stride * 2,
                           (cuuint64_t)block_stride * 2};
  cuuint32_t box[4] = {64, 1, (cuuint32_t)box_tokens, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = enc(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? B200_OK : B200_ERR_DRIVER;
}

template <int DK, int DV, int STAGES>
inline int attn_launch(const CUtensorMap& tk, const CUtensorMap& tv, const AttnParams& p, dim3 grid,
                       cudaStream_t st) {
  constexpr int smem = STAGES * ATT_BN * (DK + DV) * 2 + 1024;
  static PerDeviceFlags attr_set;
  if (int rc = set_max_dyn_smem_once(attr_set, paged_attn_kernel<DK, DV, STAGES>, smem)) return rc;
  launch_k(paged_attn_kernel<DK, DV, STAGES>, grid, dim3(32), (size_t)smem, st, tk, tv, p);
  return launch_status();
}

// Which attention kernel runs: the tcgen05 kernel (attn_tc.cuh) for the head dims it covers, unless
// B200_ATTN=simt asks for this file's mma.sync kernel (kept as the fallback for other head dims and as
// a cross-check).  The choice never depends on the batch.
inline bool attn_use_tensor_memory() {
  static const bool on = []() {
    const char* v = getenv("B200_ATTN");
    return !(v && v[0] == 's');
  }();
  return on;
}
int attn_tc_dispatch(const CUtensorMap& tk, const CUtensorMap& tv, const AttnParams& p, dim3 grid, int dk, int nc,
                     cudaStream_t st);
int attn_rows_dispatch(const CUtensorMap& tk, const CUtensorMap& tv, const CUtensorMap& tq, const CUtensorMap& to,
                       const AttnParams& p, cudaStream_t st);

// Queries as a 3-D tensor [tokens][heads][dim] with a box of {64 dims, box_heads, box_tokens}: the box's rows
// land in shared memory in (token, head) order, 128 bytes each, 128-byte swizzle, which is the row order of a
// rows-on-lanes tile.  Tokens past the end read as zeros.
inline int make_tmap_q(CUtensorMap* m, const void* q, long long tokens, int heads, int dim, long long tok_stride,
                       long long head_stride, int box_heads, int box_tokens, bool swizzle = true) {
  EncodeTiledFn enc = tensor_map_encoder();
  if (!enc) return B200_ERR_DRIVER;
  if ((reinterpret_cast<uintptr_t>(q) & 15) || (tok_stride * 2) % 16 || (head_stride * 2) % 16 || box_heads <= 0 ||
      box_heads > 256 || box_tokens <= 0 || box_tokens > 256 || tokens <= 0)
    return B200_ERR_ARG;
  cuuint64_t dims[3] = {(cuuint64_t)dim, (cuuint64_t)heads, (cuuint64_t)tokens};
  cuuint64_t strides[2] = {(cuuint64_t)head_stride * 2, (cuuint64_t)tok_stride * 2};
  cuuint32_t box[3] = {64u, (cuuint32_t)box_heads, (cuuint32_t)box_tokens};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = enc(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(q), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? B200_OK : B200_ERR_DRIVER;
}
// Prefill tiles of head dim 128: rows-on-lanes kernel unless B200_ATTN_PREFILL=cols.
// (Read at every call, so that a test can run both kernels in one process and compare their bits.)
inline bool attn_prefill_rows() {
  const char* v = getenv("B200_ATTN_PREFILL");
  return !(v && v[0] == 'c');
}

}  // namespace b200

// Causal attention of packed queries against a paged KV cache.
//   q   [total_q, num_q_heads, dk]   (strides in elements; innermost contiguous)
//   k_cache / v_cache [num_blocks, page_size, num_kv_heads, dk | dv]
//   cu_seqlens_q [num_seqs + 1], seqused_k [num_seqs], page_table [num_seqs, max_pages]  (int32)
//   out [total_q, num_q_heads, dv]
// Sequence i's queries are its last (cu[i+1] - cu[i]) positions of seqused_k[i] cached tokens.
// max_seqlen_q bounds the per-sequence query count (it sizes the grid).
extern "C" int b200_paged_attn_fwd_ordered(const void* q, const void* k_cache, const void* v_cache, void* out,
                                           const void* cu_seqlens_q, const void* seqused_k, const void* page_table,
                                           int num_seqs, int max_seqlen_q, int num_q_heads, int num_kv_heads,
                                           int dk, int dv, int num_blocks, int page_size, int max_pages,
                                           long long page_table_stride, long long q_tok_stride,
                                           long long q_head_stride, long long o_tok_stride, long long o_head_stride,
                                           long long kc_block_stride, long long kc_page_stride,
                                           long long kc_head_stride, long long vc_block_stride,
                                           long long vc_page_stride, long long vc_head_stride, float softmax_scale,
                                           const void* seq_order, long long total_q, void* stream);

extern "C" int b200_paged_attn_fwd(const void* q, const void* k_cache, const void* v_cache, void* out,
                                   const void* cu_seqlens_q, const void* seqused_k, const void* page_table,
                                   int num_seqs, int max_seqlen_q, int num_q_heads, int num_kv_heads, int dk,
                                   int dv, int num_blocks, int page_size, int max_pages,
                                   long long page_table_stride, long long q_tok_stride, long long q_head_stride,
                                   long long o_tok_stride, long long o_head_stride, long long kc_block_stride,
                                   long long kc_page_stride, long long kc_head_stride, long long vc_block_stride,
                                   long long vc_page_stride, long long vc_head_stride, float softmax_scale,
                                   void* stream) {
  return b200_paged_attn_fwd_ordered(q, k_cache, v_cache, out, cu_seqlens_q, seqused_k, page_table, num_seqs,
                                     max_seqlen_q, num_q_heads, num_kv_heads, dk, dv, num_blocks, page_size,
                                     max_pages, page_table_stride, q_tok_stride, q_head_stride, o_tok_stride,
                                     o_head_stride, kc_block_stride, kc_page_stride, kc_head_stride,
                                     vc_block_stride, vc_page_stride, vc_head_stride, softmax_scale, nullptr, 0, stream);
}

// Same, with an optional processing order: seq_order[i] (int32, a permutation of 0..num_seqs-1, e.g.
// sequences by descending context length) is the sequence the i-th group of tiles belongs to.  The
// order changes which CTA computes a sequence and when, never a result.  The mma.sync kernel ignores it.
extern "C" int b200_paged_attn_fwd_ordered(const void* q, const void* k_cache, const void* v_cache, void* out,
                                           const void* cu_seqlens_q, const void* seqused_k, const void* page_table,
                                           int num_seqs, int max_seqlen_q, int num_q_heads, int num_kv_heads,
                                           int dk, int dv, int num_blocks, int page_size, int max_pages,
                                           long long page_table_stride, long long q_tok_stride,
                                           long long q_head_stride, long long o_tok_stride, long long o_head_stride,
                                           long long kc_block_stride, long long kc_page_stride,
                                           long long kc_head_stride, long long vc_block_stride,
                                           long long vc_page_stride, long long vc_head_stride, float softmax_scale,
                                           const void* seq_order, long long total_q, void* stream) {
  using namespace b200;
  if (!q || !k_cache || !v_cache || !out || !cu_seqlens_q || !seqused_k || !page_table || num_seqs < 0 ||
      max_seqlen_q < 0 || num_q_heads <= 0 || num_kv_heads <= 0 || num_blocks <= 0 || page_size <= 0 ||
      max_pages <= 0)
    return B200_ERR_ARG;
  if (num_q_heads % num_kv_heads != 0) return B200_ERR_ARG;
  const int group = num_q_heads / num_kv_heads;
  if (group > 8 && group % 8 != 0) return B200_ERR_SHAPE;
  if (page_size % 8 != 0) return B200_ERR_SHAPE;
  if (page_size < ATT_BN ? (ATT_BN % page_size != 0) : (page_size % ATT_BN != 0)) return B200_ERR_SHAPE;
  if (q_tok_stride % 2 || q_head_stride % 2 || (reinterpret_cast<uintptr_t>(q) & 3)) return B200_ERR_ARG;
  if (num_seqs == 0 || max_seqlen_q == 0) return B200_OK;
  AttnParams p{};
  p.q = (const __nv_bfloat16*)q;
  p.out = (__nv_bfloat16*)out;
  p.q_tok_stride = q_tok_stride;
  p.q_head_stride = q_head_stride;
  p.o_tok_stride = o_tok_stride;
  p.o_head_stride = o_head_stride;
  p.cu_seqlens_q = (const int*)cu_seqlens_q;
  p.seqused_k = (const int*)seqused_k;
  p.page_table = (const int*)page_table;
  p.page_table_stride = page_table_stride;
  p.max_pages = max_pages;
  p.page_size = page_size;
  p.box_tokens = page_size < ATT_BN ? page_size : ATT_BN;
  p.num_q_heads = num_q_heads;
  p.num_kv_heads = num_kv_heads;
  p.group = group;
  p.pos_per_tile = group >= 8 ? 1 : 8 / group;
  p.head_chunks = (group + 7) / 8;
  p.qk_scale = softmax_scale * 1.44269504f;
  p.num_blocks = num_blocks;
  CUtensorMap tk, tv;
  int rc = make_tmap_cache(&tk, k_cache, num_blocks, page_size, num_kv_heads, dk, kc_block_stride,
                           kc_page_stride, kc_head_stride, p.box_tokens);
  if (rc) return rc;
  rc = make_tmap_cache(&tv, v_cache, num_blocks, page_size, num_kv_heads, dv, vc_block_stride, vc_page_stride,
                       vc_head_stride, p.box_tokens);
  if (rc) return rc;
  cudaStream_t st = (cudaStream_t)stream;
  p.max_seqlen_q = max_seqlen_q;
  {
    const char* v = getenv("B200_ATTN_OUT_SCALAR");
    p.scalar_out = (v && v[0] == '1') ? 1 : 0;
  }
  if (num_seqs > 65535 || num_kv_heads * p.head_chunks > 65535) return B200_ERR_SHAPE;
  const int hh = group < 8 ? group : 8;
  if (attn_use_tensor_memory() && dv == 128 && (dk == 128 || dk == 192) && q_tok_stride % 8 == 0 &&
      q_head_stride % 8 == 0 && (reinterpret_cast<uintptr_t>(q) & 15) == 0) {
    // tcgen05 kernels.  A decode step (one query per sequence) uses the narrow keys-on-lanes tile (16
    // columns); steps with longer query runs use 128-row tiles with a row per thread (attn_rows.cuh) for
    // head dim 128 and the 32-column keys-on-lanes tile for the 192 / 128 dims.  B200_ATTN_PREFILL=cols
    // keeps the 64-column keys-on-lanes tile for head dim 128 (the same bits, for cross-checks).
    const bool rows = max_seqlen_q > 1 && dk == 128 && attn_prefill_rows();
    const int nc = max_seqlen_q == 1 ? 16 : (dk == 128 ? (rows ? 128 : 64) : 32);
    p.pos_per_tile = nc / hh;
    dim3 grid((unsigned)((max_seqlen_q + p.pos_per_tile - 1) / p.pos_per_tile),
              (unsigned)(num_kv_heads * p.head_chunks), (unsigned)num_seqs);
    p.tc_q_tiles = (int)grid.x;
    p.tc_hy = (int)grid.y;
    if ((long long)grid.x * grid.y * grid.z > 0x7fffffffll) return B200_ERR_SHAPE;
    p.tc_tiles = (int)(grid.x * grid.y * grid.z);
    {
      const int ctas = p.tc_tiles < sm_count() ? p.tc_tiles : sm_count();  // = the launch's grid
      if (ctas > 0) p.tc_slots = (p.tc_tiles + ctas - 1) / ctas * ctas;
    }
    p.num_seqs = num_seqs;
    p.seq_order = (const int*)seq_order;
    if (rows) {
      // The query tile by TMA when every tile of a KV head has the same (heads, positions) shape, i.e. the
      // group is at most 8 heads or a multiple of 8, and the head stride is at least a head (a box row must
      // not run into the next head); otherwise the loader warp copies the rows itself.
      CUtensorMap tq = tk;
      const int hh_const = group < 8 ? group : 8;
      const char* qenv = getenv("B200_ATTN_Q_TMA");
      p.q_tma = 0;
      if (!(qenv && qenv[0] == '0') && (group <= 8 || group % 8 == 0) && q_head_stride >= dk &&
          total_q > 0 &&
          make_tmap_q(&tq, q, total_q, num_q_heads, dk, q_tok_stride, q_head_stride, hh_const, p.pos_per_tile) == B200_OK)
        p.q_tma = 1;
      // The output the same way round: each softmax warp owns 32 consecutive tile rows = 32 / heads whole
      // positions (when the head count per tile divides 32), i.e. one box of {64 dims, heads, 32 / heads positions}
      // of out [token, head, dim], stored from 128-byte-swizzled shared memory.
      CUtensorMap to = tk;
      const char* oenv = getenv("B200_ATTN_O_TMA");
      p.o_tma = 0;
      if (!(oenv && oenv[0] == '0') && (group <= 8 || group % 8 == 0) && 32 % hh_const == 0 && o_head_stride >= dv &&
          total_q > 0 &&
          make_tmap_q(&to, out, total_q, num_q_heads, dv, o_tok_stride, o_head_stride, hh_const, 32 / hh_const, true) ==
              B200_OK)
        p.o_tma = 1;
      return attn_rows_dispatch(tk, tv, tq, to, p, st);
    }
    return attn_tc_dispatch(tk, tv, p, grid, dk, nc, st);
  }
  const int q_tiles = (max_seqlen_q + p.pos_per_tile - 1) / p.pos_per_tile;
  dim3 grid((unsigned)q_tiles, (unsigned)(num_kv_heads * p.head_chunks), (unsigned)num_seqs);
  if (dk == 128 && dv == 128) return attn_launch<128, 128, 3>(tk, tv, p, grid, st);
  if (dk == 192 && dv == 128) return attn_launch<192, 128, 2>(tk, tv, p, grid, st);
  if (dk == 64 && dv == 64) return attn_launch<64, 64, 3>(tk, tv, p, grid, st);
  return B200_ERR_SHAPE;
}
