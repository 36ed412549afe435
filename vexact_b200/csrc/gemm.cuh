// Weight-streaming bf16 GEMM on tcgen05 tensor cores with TMA-staged tiles.
// One kernel serves the dense projections (aten::mm / aten::addmm) and the
// fused-MoE grouped GEMMs.
//
// Replaces vexact/batch_invariant_ops/batch_invariant_ops.py:54-229
// (matmul_kernel_persistent / matmul_persistent: fp32 accumulation, sequential K
// loop, no split-K, bias added in fp32 before the cast) and the grouped GEMMs of
// vexact/batch_invariant_ops/fused_moe.py:319-339 (quack gemm with cu_seqlens_m)
// / group_gemm/kernel/group_gemm.py:65-250 (group_gemm_same_nk).
//
// Orientation.  out[t, n] = sum_k X[t, k] * W[n, k] with W = nn.Linear.weight
// ([N, K], K contiguous) and X = activations ([T, K], K contiguous).  The weight
// rows sit on the UMMA M axis (always 128 rows per instruction) and the tokens on
// the UMMA N axis, so decode batches stream each weight tile from HBM exactly
// once and a one-token batch costs a 16-column instruction, not a 128-row one.
//
// Batch invariance.  A token's dot products are always computed by M=128, K=16
// instructions walking K from 0 upward in 64-element stages with fp32
// accumulation in tensor memory; there is no split-K and nothing depends on how
// many tokens share the tile or where in the tile the token sits.
//
// Pipeline.  Persistent CTAs (one per SM) walk a static round-robin tile list.
// Warp 0 issues TMA loads into a ring of shared-memory stages, warp 1 issues
// tcgen05.mma into one of two tensor-memory accumulators, warps 2-5 drain the
// other accumulator (tcgen05.ld), apply the epilogue and store.  All waits are
// bounded (ptx::mbar_wait).
//
// Algorithmic bytes per launch: 2*(N*K + T*K + T*N); the weight term dominates
// for decode shapes, so the roofline is HBM bandwidth.
#pragma once
#include <stdlib.h>
#include <cuda.h>  // CUtensorMap and enums only: the encoder is looked up at run time, libcuda is not linked

#include "ptx.cuh"
#include "tmap.cuh"

namespace b200 {

constexpr int GEMM_BK = 64;             // K elements per stage = one 128-byte swizzle row
constexpr int GEMM_WTILE = 128;         // weight rows per tile = UMMA M
constexpr int GEMM_WBYTES = GEMM_WTILE * GEMM_BK * 2;
constexpr int GEMM_THREADS = 192;       // producer warp, MMA warp, 4 epilogue warps
constexpr int GEMM_MAX_STAGES = 12;
constexpr int GEMM_SMEM_BUDGET = 227 * 1024;
constexpr int GEMM_EXCH_PAD = 8;  // the SwiGLU exchange buffer holds xrows_max + 8 bf16 per feature row

struct GemmParams {
  int n_w;               // output features per group (plain: N; SwiGLU: intermediate size I)
  int k;                 // reduction length
  int w_tiles;           // weight tiles per group
  int w_rows_per_group;  // rows of the 2-D weight view per group (plain: N; SwiGLU: 2*I)
  int up_offset;         // SwiGLU: row offset of the "up" half inside a group (= I)
  // Token tiling.  Dense: tiles are computed from (t_rows, rows_per_tile).  Grouped:
  // tile_table[i] = {group, first_row, n_rows, 0}, *tile_count entries are valid.
  int t_rows;
  int rows_per_tile;
  int dense_t_tiles;
  const int4* tile_table;
  // Grouped GEMM over rows that were never permuted: row r of a tile is x[gather_idx[row0 + r]] (null: x is
  // already in tile order).  The activation tensor map then has a one-row box and the producer warp fetches
  // four rows per TMA gather.
  const int* gather_idx;
  int fp16;             // plain dense mode: operands, bias and 16-bit output are fp16 instead of bf16
  int scalar_epilogue;  // development knob B200_GEMM_EPI_SCALAR=1: 2-byte stores in the plain epilogue
  const int* tile_count;
  int xbox;       // rows per activation TMA box (multiple of 16)
  int xrows_max;  // largest token count of any tile (multiple of xbox, <= 256)
  int stages;
  int katoms;     // 64-element K atoms per pipeline stage (1, 2 or 4)
  int tmem_cols;  // power of two >= 2 * xrows_max
  // Epilogue.
  void* out;
  long long ldo;
  int out_f32;
  const __nv_bfloat16* bias;       // [n_w] or null (plain mode)
  const __nv_bfloat16* row_scale;  // [rows] or null (SwiGLU mode: routing weight of each permuted row)
  float4* head_part;               // head mode: [t_rows, w_tiles] per-tile {max, sum exp(x - max), argmax, 0}
  uint64_t w_policy;
};

// Epilogue modes of gemm_ws_kernel.
constexpr int GEMM_PLAIN = 0;   // out = acc (+ bias)
constexpr int GEMM_SWIGLU = 1;  // gate / up rows stacked on M, out = silu(gate) * up * row_scale
constexpr int GEMM_HEAD = 2;    // lm_head: no logits are stored; per (token, weight tile) the maximum, the sum of
                                // exp(x - max) and the arg-max of the tile's 128 bf16-rounded logits
constexpr float kLog2e = 1.4426950408889634f;

// 2^x on the special-function unit (relative error below 2^-22; results below the normal range flush to zero).
__device__ __forceinline__ float gemm_ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Development aid (off unless the library is compiled with -DB200_GEMM_TRACE): every CTA writes %globaltimer
// stamps of its milestones; b200_debug_gemm_trace copies them out.
#ifdef B200_GEMM_TRACE
__device__ unsigned long long g_gemm_trace[256][8];
#define GEMM_STAMP(ev)                                                              \
  do {                                                                              \
    if (blockIdx.x < 256) g_gemm_trace[blockIdx.x][ev] = global_timer_ns();         \
  } while (0)
#else
#define GEMM_STAMP(ev) \
  do {                 \
  } while (0)
#endif

struct GemmTile {
  int group, row0, n, wt;
};

__device__ __forceinline__ bool gemm_tile(const GemmParams& p, int t_tiles, long long linear, GemmTile& t) {
  if (linear >= (long long)t_tiles * p.w_tiles) return false;
  t.wt = (int)(linear / t_tiles);
  const int tt = (int)(linear % t_tiles);
  if (p.tile_table) {
    const int4 e = p.tile_table[tt];
    t.group = e.x;
    t.row0 = e.y;
    t.n = e.z;
  } else {
    t.group = 0;
    t.row0 = tt * p.rows_per_tile;
    t.n = min(p.rows_per_tile, p.t_rows - t.row0);
  }
  return true;
}

template <int MODE>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_ws_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_x,
               const GemmParams p) {
  constexpr bool SWIGLU = MODE == GEMM_SWIGLU;
  constexpr bool HEAD = MODE == GEMM_HEAD;
  extern __shared__ uint8_t smem_raw[];
  if (threadIdx.x == 0) GEMM_STAMP(0);   // CTA started
  // Control block, then 1024-byte aligned stages (the 128-byte swizzle repeats every 1024 B).
  // bars[0..S) full, [S..2S) empty, [2S..2S+2) tmem_full, [2S+2..2S+4) tmem_empty
  const int S = p.stages;
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem_raw + (2 * GEMM_MAX_STAGES + 4) * 8);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem_raw + (2 * GEMM_MAX_STAGES + 4) * 8 + 8);
  const uint32_t smem_base = ptx::smem_u32(smem_raw);
  const uint32_t stage_base = (smem_base + 256 + 1023) & ~1023u;
  const int atom_bytes = GEMM_WBYTES + p.xrows_max * (GEMM_BK * 2);
  const int KA = p.katoms;
  const int stage_bytes = atom_bytes * KA;
  __nv_bfloat16* exch =
      reinterpret_cast<__nv_bfloat16*>(smem_raw + (stage_base - smem_base) + (size_t)S * stage_bytes);

  const int exch_pitch = p.xrows_max + GEMM_EXCH_PAD;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  auto full_bar = [&](int s) { return smem_base + 8u * s; };
  auto empty_bar = [&](int s) { return smem_base + 8u * (S + s); };
  auto tfull_bar = [&](int b) { return smem_base + 8u * (2 * S + b); };
  auto tempty_bar = [&](int b) { return smem_base + 8u * (2 * S + 2 + b); };

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int s = 0; s < S; ++s) {
      ptx::mbar_init(full_bar(s), 1);
      ptx::mbar_init(empty_bar(s), 1);
    }
    for (int b = 0; b < 2; ++b) {
      ptx::mbar_init(tfull_bar(b), 1);
      ptx::mbar_init(tempty_bar(b), 128);
    }
    ptx::fence_barrier_init();
    ptx::prefetch_tensormap(&tm_w);
    ptx::prefetch_tensormap(&tm_x);
  }
  if (warp == 1) {
    ptx::tmem_alloc(ptx::smem_u32(tmem_slot), (uint32_t)p.tmem_cols);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  pdl_trigger();
  if (threadIdx.x == 0) GEMM_STAMP(1);   // set-up done
  const int num_kb = (p.k + GEMM_BK * KA - 1) / (GEMM_BK * KA);  // K beyond the tensor reads as zero
  // Everything above is set-up.  What the previous kernel wrote (activations, the tile table) is read only
  // after pdl_wait().  The weights are not its output: with a static tiling (no tile table) the producer
  // requests its first ring of weight tiles before it waits, so that under programmatic dependent launch
  // their HBM latency runs alongside the predecessor's tail.
  int prefetched = 0;
  if (warp == 0 && !SWIGLU && !p.tile_table && !p.gather_idx) {
    GemmTile t;
    if (gemm_tile(p, p.dense_t_tiles, blockIdx.x, t)) {   // the same for every lane
      prefetched = num_kb < S ? num_kb : S;
      if (ptx::elect_one()) {
        const int nbox = (t.n + p.xbox - 1) / p.xbox;
        const uint32_t tx = GEMM_WBYTES + (uint32_t)nbox * p.xbox * (GEMM_BK * 2);
        const int wrow = t.wt * GEMM_WTILE;
        for (int kb = 0; kb < prefetched; ++kb) {
          ptx::mbar_expect_tx(full_bar(kb), tx * KA);
          for (int a = 0; a < KA; ++a)
            ptx::tma_load_2d(stage_base + (uint32_t)kb * stage_bytes + (uint32_t)a * atom_bytes, &tm_w, full_bar(kb),
                             (kb * KA + a) * GEMM_BK, wrow, p.w_policy);
        }
      }
    }
  }
  pdl_wait();
  const int t_tiles = p.tile_table ? *p.tile_count : p.dense_t_tiles;

  if (warp == 0 && p.gather_idx) {
    // ------------------------------------------------------------ TMA producer, gathered activation rows
    // The whole warp runs the loop: lane 0 arms the barrier and loads the weights, lane l fetches rows
    // 4l .. 4l+3 of the tile by index.  Rows past the tile's end repeat its first row (their columns are
    // never stored); rows past the last group of four keep whatever the stage held.
    const int lane = threadIdx.x & 31;
    uint32_t ph = 0;
    int s = 0;
    bool ok = true;
    for (long long lin = blockIdx.x; ok; lin += gridDim.x) {
      GemmTile t;
      if (!gemm_tile(p, t_tiles, lin, t)) break;
      const int ngrp = (t.n + 3) >> 2;
      int ri[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int r = 4 * lane + j;
        int v = lane < ngrp ? p.gather_idx[t.row0 + (r < t.n ? r : 0)] : 0;
        if (v < 0 || v >= p.t_rows) {
          report_status(B200_STATUS_BAD_INDEX, v);
          v = 0;
        }
        ri[j] = v;
      }
      const uint32_t tx = GEMM_WBYTES + (uint32_t)ngrp * 4 * (GEMM_BK * 2);
      const int wrow = t.group * p.w_rows_per_group + t.wt * (SWIGLU ? 64 : GEMM_WTILE);
      for (int kb = 0; kb < num_kb; ++kb, s = (s + 1 == S ? 0 : s + 1), ph ^= (s == 0)) {
        if (!ptx::mbar_wait_warp(empty_bar(s), ph ^ 1, abort_flag, 100 + s)) {
          ok = false;
          break;
        }
        if (lane == 0) ptx::mbar_expect_tx(full_bar(s), tx * KA);
        __syncwarp();   // the barrier is armed before any lane's copy can complete on it
        for (int a = 0; a < KA; ++a) {
          const uint32_t sw = stage_base + (uint32_t)s * stage_bytes + (uint32_t)a * atom_bytes;
          const uint32_t sx = sw + GEMM_WBYTES;
          const int kcol = (kb * KA + a) * GEMM_BK;
          if (lane == 0) {
            if (SWIGLU) {
              ptx::tma_load_2d(sw, &tm_w, full_bar(s), kcol, wrow, p.w_policy);
              ptx::tma_load_2d(sw + 64 * GEMM_BK * 2, &tm_w, full_bar(s), kcol, wrow + p.up_offset, p.w_policy);
            } else {
              ptx::tma_load_2d(sw, &tm_w, full_bar(s), kcol, wrow, p.w_policy);
            }
          }
          if (lane < ngrp)
            ptx::tma_gather4_2d(sx + (uint32_t)lane * 4 * (GEMM_BK * 2), &tm_x, full_bar(s), kcol, ri[0], ri[1],
                                ri[2], ri[3], ptx::kEvictLast);
        }
      }
    }
  } else if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (ptx::elect_one()) {
      uint32_t it = 0;   // running stage counter across tiles
      int s = 0;         // ring slot of `it`
      uint32_t ph = 0;   // parity of the slot's current use
      bool ok = true;
      for (long long lin = blockIdx.x; ok; lin += gridDim.x) {
        GemmTile t;
        if (!gemm_tile(p, t_tiles, lin, t)) break;
        const int nbox = (t.n + p.xbox - 1) / p.xbox;
        const uint32_t tx = GEMM_WBYTES + (uint32_t)nbox * p.xbox * (GEMM_BK * 2);
        const int wrow = t.group * p.w_rows_per_group + t.wt * (SWIGLU ? 64 : GEMM_WTILE);
        for (int kb = 0; kb < num_kb; ++kb, ++it, s = (s + 1 == S ? 0 : s + 1), ph ^= (s == 0)) {
          // the first tile's first `prefetched` stages were armed, and their weights requested, before pdl_wait
          const bool early = it < (uint32_t)prefetched;
          if (!early) {
            if (!ptx::mbar_wait(empty_bar(s), ph ^ 1, abort_flag, 100 + s)) {
              ok = false;
              break;
            }
            ptx::mbar_expect_tx(full_bar(s), tx * KA);
          }
          for (int a = 0; a < KA; ++a) {
            const uint32_t sw = stage_base + (uint32_t)s * stage_bytes + (uint32_t)a * atom_bytes;
            const uint32_t sx = sw + GEMM_WBYTES;
            const int kcol = (kb * KA + a) * GEMM_BK;
            if (early) {
            } else if (SWIGLU) {
              ptx::tma_load_2d(sw, &tm_w, full_bar(s), kcol, wrow, p.w_policy);
              ptx::tma_load_2d(sw + 64 * GEMM_BK * 2, &tm_w, full_bar(s), kcol, wrow + p.up_offset, p.w_policy);
            } else {
              ptx::tma_load_2d(sw, &tm_w, full_bar(s), kcol, wrow, p.w_policy);
            }
            for (int b = 0; b < nbox; ++b)
              ptx::tma_load_2d(sx + (uint32_t)b * p.xbox * (GEMM_BK * 2), &tm_x, full_bar(s), kcol,
                               t.row0 + b * p.xbox, ptx::kEvictLast);
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (ptx::elect_one()) {
      uint32_t it = 0, tile_it = 0, ph = 0;
      int s = 0;
      bool ok = true;
      for (long long lin = blockIdx.x; ok; lin += gridDim.x, ++tile_it) {
        GemmTile t;
        if (!gemm_tile(p, t_tiles, lin, t)) break;
        const int buf = tile_it & 1;
        const int nbox = (t.n + p.xbox - 1) / p.xbox;
        const uint32_t idesc = p.fp16 ? ptx::umma_idesc_f16_m128((uint32_t)(nbox * p.xbox))
                                      : ptx::umma_idesc_bf16_m128((uint32_t)(nbox * p.xbox));
        if (!ptx::mbar_wait(tempty_bar(buf), ((tile_it >> 1) & 1) ^ 1, abort_flag, 200 + buf)) break;
        ptx::tc_fence_after();
        const uint32_t d_tmem = tmem_base + (uint32_t)(buf * p.xrows_max);
        const uint64_t desc_hi = ptx::umma_desc_k_sw128(0) & 0xFFFFFFFF00000000ull;
        for (int kb = 0; kb < num_kb; ++kb, ++it, s = (s + 1 == S ? 0 : s + 1), ph ^= (s == 0)) {
          if (!ptx::mbar_wait(full_bar(s), ph, abort_flag, 300 + s)) {
            ok = false;
            break;
          }
          ptx::tc_fence_after();
          if (it == 0) GEMM_STAMP(2);    // first stage landed
          for (int a = 0; a < KA; ++a) {
            const uint32_t sw = stage_base + (uint32_t)s * stage_bytes + (uint32_t)a * atom_bytes;
            // descriptors differ only in the start-address field: +2 (32 bytes) per 16-element K step
            const uint64_t da = desc_hi | (uint64_t)(((sw & 0x3FFFFu) >> 4) | (1u << 16));
            const uint64_t db = desc_hi | (uint64_t)((((sw + GEMM_WBYTES) & 0x3FFFFu) >> 4) | (1u << 16));
            ptx::umma_bf16(d_tmem, da, db, idesc, (kb | a) != 0 ? 1u : 0u);
#pragma unroll
            for (int kk = 1; kk < GEMM_BK / 16; ++kk) ptx::umma_bf16_acc(d_tmem, da + 2 * kk, db + 2 * kk, idesc);
          }
          ptx::umma_commit(empty_bar(s));  // stage is free once these MMAs have read it
        }
        if (ok) ptx::umma_commit(tfull_bar(buf));
        GEMM_STAMP(3);                   // last MMA of the tile issued
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (warps 2..5)
    const int q = warp & 3;              // tensor-memory lane quadrant this warp may read
    uint32_t tile_it = 0;
    for (long long lin = blockIdx.x;; lin += gridDim.x, ++tile_it) {
      GemmTile t;
      if (!gemm_tile(p, t_tiles, lin, t)) break;
      const int buf = tile_it & 1;
      const bool ready = ptx::mbar_wait(tfull_bar(buf), (tile_it >> 1) & 1, abort_flag, 400 + buf);
      if (SWIGLU || HEAD) {
        // The four epilogue warps meet at named barriers below, so they must leave together: a wait
        // that gave up has raised the abort flag before its warp arrives here, and everyone reads
        // the flag after this barrier.
        ptx::named_barrier_sync(1, 128);
        if (*abort_flag) break;
      } else if (!__all_sync(0xffffffffu, ready)) {
        break;
      }
      ptx::tc_fence_after();
      if (threadIdx.x == 64) GEMM_STAMP(4);   // accumulator complete
      const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(buf * p.xrows_max);
      const int ncol = ((t.n + 15) / 16) * 16;
      if (HEAD) {
        // Thread = vocabulary row f of the tile; columns = tokens.  Per 16 columns: every logit is rounded
        // to bf16 (the logits tensor the reference materialises is bf16), then per column the warp's
        // maximum (redux.sync), sum of exp(x - max) (a halving butterfly: 16 shuffles for 16 columns, the
        // same tree for every column) and lowest row holding the maximum.  The four warps' partials meet
        // in shared memory in row order.  Nothing here depends on how many tokens share the tile.
        const int f = t.wt * GEMM_WTILE + q * 32 + lane;
        const bool fvalid = f < p.n_w;
        float* hs_m = reinterpret_cast<float*>(exch);           // [4][xrows_max]
        float* hs_s = hs_m + 4 * p.xrows_max;
        int* hs_i = reinterpret_cast<int*>(hs_s + 4 * p.xrows_max);
        const int mycol = ((lane >> 4) & 1) * 8 + ((lane >> 3) & 1) * 4 + ((lane >> 2) & 1) * 2 + ((lane >> 1) & 1);
        for (int c0 = 0; c0 < ncol; c0 += 16) {
          uint32_t r[16];
          ptx::tmem_ld16(taddr + c0, r);
          ptx::tmem_ld_wait();
          float v[16], e[16];
          float my_m = -INFINITY;
          int my_i = 0;
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            v[j] = fvalid ? round_bf(__uint_as_float(r[j])) : -INFINITY;
            float m;
            asm volatile("redux.sync.max.f32 %0, %1, 0xffffffff;" : "=f"(m) : "f"(v[j]));
            const unsigned hit = __ballot_sync(0xffffffffu, v[j] == m);
            e[j] = v[j] == -INFINITY ? 0.f : gemm_ex2((v[j] - m) * kLog2e);
            if (j == mycol) {
              my_m = m;
              my_i = __ffs(hit) - 1;
            }
          }
          // sum over the 32 rows of each of the 16 columns
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const bool up = lane & 16;
            const float got = __shfl_xor_sync(0xffffffffu, up ? e[i] : e[i + 8], 16);
            e[i] = (up ? e[i + 8] : e[i]) + got;
          }
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const bool up = lane & 8;
            const float got = __shfl_xor_sync(0xffffffffu, up ? e[i] : e[i + 4], 8);
            e[i] = (up ? e[i + 4] : e[i]) + got;
          }
#pragma unroll
          for (int i = 0; i < 2; ++i) {
            const bool up = lane & 4;
            const float got = __shfl_xor_sync(0xffffffffu, up ? e[i] : e[i + 2], 4);
            e[i] = (up ? e[i + 2] : e[i]) + got;
          }
          {
            const bool up = lane & 2;
            const float got = __shfl_xor_sync(0xffffffffu, up ? e[0] : e[1], 2);
            e[0] = (up ? e[1] : e[0]) + got;
          }
          e[0] += __shfl_xor_sync(0xffffffffu, e[0], 1);
          if ((lane & 1) == 0) {
            const int c = c0 + mycol;
            hs_m[q * p.xrows_max + c] = my_m;
            hs_s[q * p.xrows_max + c] = e[0];
            hs_i[q * p.xrows_max + c] = t.wt * GEMM_WTILE + q * 32 + my_i;
          }
        }
        ptx::named_barrier_sync(1, 128);
        for (int c = q * 32 + lane; c < t.n; c += 128) {
          float m = -INFINITY;
#pragma unroll
          for (int w = 0; w < 4; ++w) m = fmaxf(m, hs_m[w * p.xrows_max + c]);
          float sum = 0.f;
          int idx = 0x7fffffff;
#pragma unroll
          for (int w = 0; w < 4; ++w) {   // rows ascend with w: the first warp holding the maximum has the lowest row
            const float mw = hs_m[w * p.xrows_max + c];
            if (mw != -INFINITY) sum += hs_s[w * p.xrows_max + c] * gemm_ex2((mw - m) * kLog2e);
            if (mw == m && idx == 0x7fffffff) idx = hs_i[w * p.xrows_max + c];
          }
          p.head_part[(long long)(t.row0 + c) * p.w_tiles + t.wt] = make_float4(m, sum, __int_as_float(idx), 0.f);
        }
        ptx::named_barrier_sync(1, 128);  // the partial arrays are reused by the next tile
      } else if (!SWIGLU) {
        const int f = t.wt * GEMM_WTILE + q * 32 + lane;
        const bool fvalid = f < p.n_w;
        const float bias = !(p.bias && fvalid) ? 0.f
                           : p.fp16     ? __half2float(reinterpret_cast<const __half*>(p.bias)[f])
                                        : bf2f(p.bias[f]);
        // rounds to the 16-bit output type (bf16, or fp16 for fp16 operands) and returns the bits
        auto cvt16 = [&](float v) -> unsigned short {
          if (p.fp16) return __half_as_ushort(__float2half_rn(v));
          return __bfloat16_as_ushort(f2bf(v));
        };
        // bf16 output whose rows allow 16-byte stores: each warp turns its 32 features x 16 tokens around in
        // shared memory, so that a lane stores eight consecutive features of one token (16 bytes) and one
        // instruction covers eight token rows, instead of one 2-byte store per (feature, token).
        const bool vec_out = !p.scalar_epilogue && !p.out_f32 && (p.ldo & 7) == 0 && (p.n_w & 7) == 0 &&
                             (reinterpret_cast<uintptr_t>(p.out) & 15) == 0;
        if (vec_out) {
          __nv_bfloat16* stg = exch + q * (16 * 32);      // [16 tokens][32 features] per warp
          const int part = lane & 3, rsub = lane >> 2;
          const int f8 = t.wt * GEMM_WTILE + q * 32 + part * 8;
          for (int c0 = 0; c0 < ncol; c0 += 16) {
            uint32_t r[16];
            ptx::tmem_ld16(taddr + c0, r);
            ptx::tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 16; ++j)
              reinterpret_cast<unsigned short*>(stg)[j * 32 + lane] = cvt16(__uint_as_float(r[j]) + bias);
            __syncwarp();
#pragma unroll
            for (int h = 0; h < 2; ++h) {
              const int row = h * 8 + rsub, c = c0 + row;
              const uint4 v = *reinterpret_cast<const uint4*>(stg + row * 32 + part * 8);
              if (c < t.n && f8 < p.n_w)
                *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(p.out) + (long long)(t.row0 + c) * p.ldo + f8) = v;
            }
            __syncwarp();
          }
        } else
        for (int c0 = 0; c0 < ncol; c0 += 16) {
          uint32_t r[16];
          ptx::tmem_ld16(taddr + c0, r);
          ptx::tmem_ld_wait();
          if (fvalid) {
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              const int c = c0 + j;
              if (c < t.n) {
                const float v = __uint_as_float(r[j]) + bias;
                const long long o = (long long)(t.row0 + c) * p.ldo + f;
                if (p.out_f32)
                  reinterpret_cast<float*>(p.out)[o] = v;
                else
                  reinterpret_cast<unsigned short*>(p.out)[o] = cvt16(v);
              }
            }
          }
        }
      } else {
        // Lanes 0..63 hold the gate rows, lanes 64..127 the up rows of the same 64 features.
        const int fi = (q & 1) * 32 + lane;
        if (q >= 2) {
          for (int c0 = 0; c0 < ncol; c0 += 16) {
            uint32_t r[16];
            ptx::tmem_ld16(taddr + c0, r);
            ptx::tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 16; ++j) exch[fi * exch_pitch + c0 + j] = f2bf(__uint_as_float(r[j]));
          }
        }
        ptx::named_barrier_sync(1, 128);
        if (q < 2) {
          const int f = t.wt * 64 + fi;
          const bool fvalid = f < p.n_w;
          for (int c0 = 0; c0 < ncol; c0 += 16) {
            uint32_t r[16];
            ptx::tmem_ld16(taddr + c0, r);
            ptx::tmem_ld_wait();
            if (fvalid) {
#pragma unroll
              for (int j = 0; j < 16; ++j) {
                const int c = c0 + j;
                if (c < t.n) {
                  // Rounding points of fused_moe.py:319-336: each GEMM output, silu(), the
                  // gate*up product and the routing-weight product are bf16 tensors.
                  const float g = round_bf(__uint_as_float(r[j]));
                  const float u = bf2f(exch[fi * exch_pitch + c]);
                  const float sg = round_bf(g / (1.0f + expf(-g)));
                  float h = round_bf(sg * u);
                  if (p.row_scale) h = round_bf(h * bf2f(p.row_scale[t.row0 + c]));
                  reinterpret_cast<__nv_bfloat16*>(p.out)[(long long)(t.row0 + c) * p.ldo + f] = f2bf(h);
                }
              }
            }
          }
        }
        ptx::named_barrier_sync(1, 128);  // exchange buffer is reused by the next tile
      }
      ptx::tc_fence_before();
      ptx::mbar_arrive(tempty_bar(buf));
      if (threadIdx.x == 64) GEMM_STAMP(5);   // tile stored
    }
  }

  // Teardown.  On an aborted run give in-flight TMA copies time to land before the CTA exits.
  __syncthreads();
  if (*abort_flag) {
    const uint64_t t0 = global_timer_ns();
    while (global_timer_ns() - t0 < 200000ull) {
    }
  }
  ptx::tc_fence_after();
  if (warp == 1) {
    __syncwarp();
    ptx::tmem_dealloc(tmem_base, (uint32_t)p.tmem_cols);
  }
}

// ------------------------------------------------------------------ host side

// 2-D bf16 tensor [rows, cols] with `row_stride` elements between rows; box = 64 cols x box_rows,
// 128-byte swizzle.  Out-of-range elements read as zero.
inline int make_tmap_2d(CUtensorMap* m, const void* base, uint64_t rows, uint64_t cols, uint64_t row_stride,
                        uint32_t box_rows, bool fp16 = false) {
  EncodeTiledFn enc = tensor_map_encoder();
  if (!enc) return B200_ERR_DRIVER;
  if ((reinterpret_cast<uintptr_t>(base) & 15) || (row_stride * 2) % 16 || box_rows == 0 || box_rows > 256)
    return B200_ERR_ARG;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {row_stride * 2};
  cuuint32_t box[2] = {(cuuint32_t)GEMM_BK, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(m, fp16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2,
                   const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? B200_OK : B200_ERR_DRIVER;
}

inline int round_up(int v, int m) { return (v + m - 1) / m * m; }

// Development knobs (unset in normal use): B200_GEMM_XBOX = rows per activation box of the grouped
// GEMM (16, 32 or 64), B200_GEMM_STAGES = cap on pipeline stages.
inline int env_int(const char* name, int dflt) {
  const char* v = getenv(name);
  return v ? atoi(v) : dflt;
}

template <int MODE>
inline int gemm_launch(const CUtensorMap& tw, const CUtensorMap& tx, GemmParams& p, long long max_tiles,
                       cudaStream_t st) {
  constexpr bool SWIGLU = MODE == GEMM_SWIGLU;
  static PerDeviceFlags attr_set;
  if (int rc = set_max_dyn_smem_once(attr_set, gemm_ws_kernel<MODE>, GEMM_SMEM_BUDGET)) return rc;
  const int atom_bytes = GEMM_WBYTES + p.xrows_max * GEMM_BK * 2;
  // epilogue scratch after the stages: the SwiGLU exchange buffer, or the head mode's per-warp partials
  const int exch_bytes_pre = SWIGLU ? 64 * (p.xrows_max + GEMM_EXCH_PAD) * 2
                                    : (MODE == GEMM_HEAD ? 3 * 4 * p.xrows_max * 4 : 4 * 16 * 32 * 2);
  // K atoms per stage: fewer, larger stages cut the per-stage barrier round trips; keep >= 3 stages.
  static const int ka_env = env_int("B200_GEMM_KATOMS", 2);
  int ka = (ka_env == 1 || ka_env == 2 || ka_env == 4) ? ka_env : 2;
  while (ka > 1 && ((GEMM_SMEM_BUDGET - 256 - 1024 - exch_bytes_pre) / (atom_bytes * ka) < 3 ||
                    (p.k + GEMM_BK - 1) / GEMM_BK < ka))
    ka >>= 1;
  p.katoms = ka;
  static const int epi_scalar = env_int("B200_GEMM_EPI_SCALAR", 0);
  p.scalar_epilogue = epi_scalar;
  const int stage_bytes = atom_bytes * ka;
  const int exch_bytes = exch_bytes_pre;
  int stages = (GEMM_SMEM_BUDGET - 256 - 1024 - exch_bytes) / stage_bytes;
  if (stages > GEMM_MAX_STAGES) stages = GEMM_MAX_STAGES;
  {
    static const int cap = env_int("B200_GEMM_STAGES", GEMM_MAX_STAGES);
    if (stages > cap) stages = cap;
  }
  if (stages < 2) return B200_ERR_SHAPE;
  p.stages = stages;
  int cols = 32;
  while (cols < 2 * p.xrows_max) cols <<= 1;
  if (cols > 512) return B200_ERR_SHAPE;
  p.tmem_cols = cols;
  const size_t smem = 256 + 1024 + (size_t)stages * stage_bytes + exch_bytes;
  long long grid = max_tiles < sm_count() ? max_tiles : sm_count();
  if (grid <= 0) return B200_OK;
  // A dense GEMM (static tiling) may start under its predecessor's tail: it prefetches weights before it waits.
  launch_k_pdl(gemm_ws_kernel<MODE>, dim3((unsigned)grid), dim3(GEMM_THREADS), smem, st,
               pdl_mode() == 1 || (pdl_mode() == 2 && !p.tile_table), tw, tx, p);
  return launch_status();
}

}  // namespace b200

namespace b200 {
// fp32 GEMM for the DeepSeek-V3 router (modeling_deepseek_v3.py:97-100 runs F.linear in fp32):
// one warp per output element, lanes stride over K, fixed butterfly.  Exact fp32 FMA arithmetic
// (the reference's Triton path feeds tl.dot fp32 operands, i.e. TF32 inputs).
// TIn = float, or __nv_bfloat16 operands widened to fp32 on the fly: the same arithmetic as converting the
// tensors first (x.float() @ w.float().T), without the two conversion kernels and their copies.
template <typename TIn>
__global__ void __launch_bounds__(256)
gemm_f32_kernel(const TIn* __restrict__ x, const TIn* __restrict__ w, const float* __restrict__ bias,
                float* __restrict__ out, long long T, int N, int K, long long x_stride, long long w_stride,
                long long out_stride) {
  pdl_trigger();
  pdl_wait();
  const long long wid = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (wid >= T * N) return;
  const int lane = threadIdx.x & 31;
  const long long t = wid / N;
  const int n = (int)(wid % N);
  const TIn* xr = x + t * x_stride;
  const TIn* wr = w + (long long)n * w_stride;
  float acc = 0.f;
  for (int k = lane; k < K; k += 32) acc = fmaf((float)xr[k], (float)wr[k], acc);
  acc = warp_sum(acc);
  if (lane == 0) out[t * out_stride + n] = acc + (bias ? bias[n] : 0.f);
}
}  // namespace b200

extern "C" int b200_gemm_f32(const void* x, const void* w, const void* bias, void* out, long long T, int N,
                             int K, long long x_row_stride, long long w_row_stride, long long out_row_stride,
                             void* stream) {
  using namespace b200;
  if (!x || !w || !out || T < 0 || N <= 0 || K <= 0) return B200_ERR_ARG;
  if (T == 0) return B200_OK;
  const long long warps = T * N;
  launch_k(gemm_f32_kernel<float>, dim3((unsigned)((warps + 7) / 8)), dim3(256), 0, (cudaStream_t)stream,
           (const float*)x, (const float*)w, (const float*)bias, (float*)out, T, N, K, x_row_stride, w_row_stride,
           out_row_stride);
  return launch_status();
}

// The DeepSeek-V3 router on bf16 tensors: out_f32[T, N] = float(x) @ float(w)^T, bit-identical to
// b200_gemm_f32 on x.float() and w.float() (what PatchDeepseekV3TopkRouter.forward computes,
// modeling_deepseek_v3.py:97-100) without materialising the fp32 copies every step.
extern "C" int b200_gemm_f32_from_bf16(const void* x, const void* w, void* out, long long T, int N, int K,
                                       long long x_row_stride, long long w_row_stride, long long out_row_stride,
                                       void* stream) {
  using namespace b200;
  if (!x || !w || !out || T < 0 || N <= 0 || K <= 0) return B200_ERR_ARG;
  if (T == 0) return B200_OK;
  const long long warps = T * N;
  launch_k(gemm_f32_kernel<__nv_bfloat16>, dim3((unsigned)((warps + 7) / 8)), dim3(256), 0, (cudaStream_t)stream,
           (const __nv_bfloat16*)x, (const __nv_bfloat16*)w, (const float*)nullptr, (float*)out, T, N, K,
           x_row_stride, w_row_stride, out_row_stride);
  return launch_status();
}

// out[T, N] = x[T, K] @ w[N, K]^T (+ bias[N], added in fp32 before the cast).
// x rows are `x_row_stride` elements apart, w rows `w_row_stride`, out rows `out_row_stride`.
namespace b200 {
inline int gemm_dense_16bit(const void* x, const void* w, const void* bias, void* out, long long T, int N, int K,
                            long long x_row_stride, long long w_row_stride, long long out_row_stride, int out_dtype,
                            bool fp16, void* stream) {
  if (!x || !w || !out || T < 0 || N <= 0 || K <= 0 || (out_dtype != 0 && out_dtype != 1)) return B200_ERR_ARG;
  if (K % 8 != 0 || x_row_stride % 8 != 0 || w_row_stride % 8 != 0) return B200_ERR_SHAPE;
  if (T == 0) return B200_OK;
  if (T > 0x7fffffffLL) return B200_ERR_SHAPE;
  GemmParams p{};
  p.n_w = N;
  p.k = K;
  p.w_tiles = (N + GEMM_WTILE - 1) / GEMM_WTILE;
  p.w_rows_per_group = N;
  p.up_offset = 0;
  p.t_rows = (int)T;
  // Token tiling.  A token's result does not depend on the tile it lands in (tokens are independent
  // UMMA columns), so the tile width is chosen for speed only.  Every tile streams K/64 stages of
  // (16 KiB of weights + 128 B per token) into shared memory and the persistent CTAs work through
  // the tiles in rounds, so the cost of a tiling is rounds x bytes per stage; take the cheapest.
  {
    const int sms = sm_count();
    const int min_tiles = (int)((T + 255) / 256);
    const int max_tiles = (int)((T + 15) / 16);
    long long best_cost = -1;
    for (int tt = min_tiles; tt <= max_tiles; ++tt) {
      const int rows = round_up((int)((T + tt - 1) / tt), 16);
      const int tiles_t = (int)((T + rows - 1) / rows);
      const long long rounds = ((long long)tiles_t * p.w_tiles + sms - 1) / sms;
      const long long cost = rounds * (GEMM_WBYTES + rows * GEMM_BK * 2);
      if (best_cost < 0 || cost < best_cost) {
        best_cost = cost;
        p.rows_per_tile = rows;
        p.dense_t_tiles = tiles_t;
      }
    }
  }
  p.tile_table = nullptr;
  p.tile_count = nullptr;
  p.xbox = p.rows_per_tile;
  p.xrows_max = p.rows_per_tile;
  p.out = out;
  p.ldo = out_row_stride;
  p.out_f32 = out_dtype;
  p.bias = (const __nv_bfloat16*)bias;
  p.row_scale = nullptr;
  p.w_policy = p.dense_t_tiles == 1 ? ptx::kEvictFirst : ptx::kEvictNormal;
  p.fp16 = fp16 ? 1 : 0;
  CUtensorMap tw, tx;
  int rc = make_tmap_2d(&tw, w, (uint64_t)N, (uint64_t)K, (uint64_t)w_row_stride, GEMM_WTILE, fp16);
  if (rc) return rc;
  rc = make_tmap_2d(&tx, x, (uint64_t)T, (uint64_t)K, (uint64_t)x_row_stride, (uint32_t)p.xbox, fp16);
  if (rc) return rc;
  return gemm_launch<GEMM_PLAIN>(tw, tx, p, (long long)p.w_tiles * p.dense_t_tiles, (cudaStream_t)stream);
}
}  // namespace b200

extern "C" int b200_gemm_bf16(const void* x, const void* w, const void* bias, void* out, long long T, int N,
                              int K, long long x_row_stride, long long w_row_stride, long long out_row_stride,
                              int out_dtype /*0 = bf16, 1 = f32*/, void* stream) {
  return b200::gemm_dense_16bit(x, w, bias, out, T, N, K, x_row_stride, w_row_stride, out_row_stride, out_dtype, false,
                                stream);
}

// The same GEMM on fp16 tensors (the reference's matmul_persistent serves bf16, fp16 and fp32,
// batch_invariant_ops.py:181-189): fp32 accumulation in the same K order, bias added in fp32, one rounding to fp16.
extern "C" int b200_gemm_f16(const void* x, const void* w, const void* bias, void* out, long long T, int N, int K,
                             long long x_row_stride, long long w_row_stride, long long out_row_stride,
                             int out_dtype /*0 = f16, 1 = f32*/, void* stream) {
  return b200::gemm_dense_16bit(x, w, bias, out, T, N, K, x_row_stride, w_row_stride, out_row_stride, out_dtype, true,
                                stream);
}

namespace b200 {
// Second half of the fused lm_head -> greedy token + log-probability: one warp per token folds the
// token's per-tile {max, sum exp(x - max), argmax} partials in a fixed order (lane l takes tiles l, l + 32,
// ... in ascending order, then a butterfly over the lanes), so the result depends on the vocabulary size
// alone.  token = lowest index holding the row maximum; logprob = max - logsumexp = -ln(sum exp(x - max)).
struct HeadAcc {
  float m, s;
  int i;
};
__device__ __forceinline__ HeadAcc head_join(const HeadAcc& a, const HeadAcc& b) {
  HeadAcc r;
  r.m = fmaxf(a.m, b.m);
  const float sa = a.m == -INFINITY ? 0.f : a.s * gemm_ex2((a.m - r.m) * kLog2e);
  const float sb = b.m == -INFINITY ? 0.f : b.s * gemm_ex2((b.m - r.m) * kLog2e);
  r.s = sa + sb;
  r.i = a.m == b.m ? min(a.i, b.i) : (a.m > b.m ? a.i : b.i);
  return r;
}
__global__ void __launch_bounds__(256)
lm_head_combine_kernel(const float4* __restrict__ part, int w_tiles, long long T, long long* __restrict__ tokens,
                       float* __restrict__ logprobs) {
  pdl_trigger();
  pdl_wait();
  const long long tkn = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (tkn >= T) return;
  const int lane = threadIdx.x & 31;
  HeadAcc acc = {-INFINITY, 0.f, 0x7fffffff};
  for (int w = lane; w < w_tiles; w += 32) {
    const float4 v = part[tkn * w_tiles + w];
    acc = head_join(acc, HeadAcc{v.x, v.y, __float_as_int(v.z)});
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    HeadAcc other;
    other.m = __shfl_xor_sync(0xffffffffu, acc.m, o);
    other.s = __shfl_xor_sync(0xffffffffu, acc.s, o);
    other.i = __shfl_xor_sync(0xffffffffu, acc.i, o);
    acc = head_join(acc, other);
  }
  if (lane == 0) {
    tokens[tkn] = acc.i == 0x7fffffff ? 0 : acc.i;
    logprobs[tkn] = -logf(acc.s);
  }
}
}  // namespace b200

// Fused lm_head -> greedy token + its log-probability without materialising the [T, V] logits
// (vexact/inferencer/inferencer.py:393-449 for greedy requests that want scores but not logits):
// the lm_head GEMM's epilogue reduces each 128-row weight tile to {max, sum exp, argmax} per token
// (bf16-rounded logits, as the reference's logits tensor holds them) into `partials`
// ([T, ceil(V / 128)] float4, caller-provided scratch), and a second kernel folds them per token.
extern "C" int b200_lm_head_greedy(const void* x, const void* w, void* partials, void* tokens_i64,
                                   void* logprobs_f32, long long T, int V, int K, long long x_row_stride,
                                   long long w_row_stride, void* stream) {
  using namespace b200;
  if (!x || !w || !partials || !tokens_i64 || !logprobs_f32 || T < 0 || V <= 0 || K <= 0) return B200_ERR_ARG;
  if (K % 8 != 0 || x_row_stride % 8 != 0 || w_row_stride % 8 != 0) return B200_ERR_SHAPE;
  if (T == 0) return B200_OK;
  if (T > 0x7fffffffLL) return B200_ERR_SHAPE;
  GemmParams p{};
  p.n_w = V;
  p.k = K;
  p.w_tiles = (V + GEMM_WTILE - 1) / GEMM_WTILE;
  p.w_rows_per_group = V;
  p.t_rows = (int)T;
  {   // token tiling: the dense GEMM's cost model (a token's arithmetic does not depend on its tile)
    const int sms = sm_count();
    const int min_tiles = (int)((T + 255) / 256), max_tiles = (int)((T + 15) / 16);
    long long best_cost = -1;
    for (int tt = min_tiles; tt <= max_tiles; ++tt) {
      const int rows = round_up((int)((T + tt - 1) / tt), 16);
      const int tiles_t = (int)((T + rows - 1) / rows);
      const long long rounds = ((long long)tiles_t * p.w_tiles + sms - 1) / sms;
      const long long cost = rounds * (GEMM_WBYTES + rows * GEMM_BK * 2);
      if (best_cost < 0 || cost < best_cost) {
        best_cost = cost;
        p.rows_per_tile = rows;
        p.dense_t_tiles = tiles_t;
      }
    }
  }
  p.xbox = p.rows_per_tile;
  p.xrows_max = p.rows_per_tile;
  p.head_part = (float4*)partials;
  p.w_policy = p.dense_t_tiles == 1 ? ptx::kEvictFirst : ptx::kEvictNormal;
  CUtensorMap tw, tx;
  int rc = make_tmap_2d(&tw, w, (uint64_t)V, (uint64_t)K, (uint64_t)w_row_stride, GEMM_WTILE);
  if (rc) return rc;
  rc = make_tmap_2d(&tx, x, (uint64_t)T, (uint64_t)K, (uint64_t)x_row_stride, (uint32_t)p.xbox);
  if (rc) return rc;
  rc = gemm_launch<GEMM_HEAD>(tw, tx, p, (long long)p.w_tiles * p.dense_t_tiles, (cudaStream_t)stream);
  if (rc) return rc;
  launch_k(lm_head_combine_kernel, dim3((unsigned)((T + 7) / 8)), dim3(256), 0, (cudaStream_t)stream,
           (const float4*)partials, p.w_tiles, T, (long long*)tokens_i64, (float*)logprobs_f32);
  return launch_status();
}

// Grouped GEMM over expert-sorted rows.
//   mode 0: out[r, n] = x[r, :] . w[g(r), n, :]                      (w: [G, N, K])
//   mode 1: out[r, i] = silu(x . w[g, i, :]) * (x . w[g, I + i, :]) * row_scale[r]   (w: [G, 2I, K], n_out = I)
// tile_table / tile_count come from b200_moe_permute: every tile lies inside one group.
namespace b200 {
// gather_index == nullptr: x holds the expert-sorted rows ([x_rows, K], contiguous).  Otherwise x is the
// unpermuted [x_rows, K] matrix with rows x_row_stride apart and sorted row r is x[gather_index[r]].
inline int moe_grouped_gemm_impl(const void* x, long long x_rows, long long x_row_stride, const void* gather_index,
                                 const void* w, const void* row_scale, void* out, const void* tile_table,
                                 const void* tile_count, int num_groups, int n_out, int K, long long out_row_stride,
                                 int max_tiles, int tile_rows_max, int mode, void* stream) {
  if (!x || !w || !out || !tile_table || !tile_count || x_rows < 0 || num_groups <= 0 || n_out <= 0 || K <= 0 ||
      max_tiles < 0 || (mode != 0 && mode != 1))
    return B200_ERR_ARG;
  if (K % 8 != 0 || tile_rows_max % 16 != 0 || tile_rows_max <= 0 || tile_rows_max > 256) return B200_ERR_SHAPE;
  if (gather_index && (tile_rows_max > 128 || x_row_stride % 8 != 0 || x_rows > 0x7fffffffLL)) return B200_ERR_SHAPE;
  if (x_rows == 0 || max_tiles == 0) return B200_OK;
  GemmParams p{};
  p.n_w = n_out;
  p.k = K;
  p.w_tiles = mode == 1 ? (n_out + 63) / 64 : (n_out + GEMM_WTILE - 1) / GEMM_WTILE;
  p.w_rows_per_group = mode == 1 ? 2 * n_out : n_out;
  p.up_offset = mode == 1 ? n_out : 0;
  p.t_rows = (int)x_rows;
  p.rows_per_tile = 0;
  p.dense_t_tiles = 0;
  p.tile_table = (const int4*)tile_table;
  p.tile_count = (const int*)tile_count;
  p.gather_idx = (const int*)gather_index;
  // One activation box per stage when the tile height allows it (fewer TMA issues per stage).
  static const int xbox_env = env_int("B200_GEMM_XBOX", 64);
  p.xbox = (xbox_env == 16 || xbox_env == 32 || xbox_env == 64) && tile_rows_max % xbox_env == 0 ? xbox_env : 16;
  p.xrows_max = tile_rows_max;
  p.out = out;
  p.ldo = out_row_stride;
  p.out_f32 = 0;
  p.bias = nullptr;
  p.row_scale = (const __nv_bfloat16*)row_scale;
  p.w_policy = ptx::kEvictFirst;
  CUtensorMap tw, tx;
  int rc = make_tmap_2d(&tw, w, (uint64_t)num_groups * p.w_rows_per_group, (uint64_t)K, (uint64_t)K,
                        mode == 1 ? 64 : GEMM_WTILE);
  if (rc) return rc;
  rc = gather_index ? make_tmap_2d(&tx, x, (uint64_t)x_rows, (uint64_t)K, (uint64_t)x_row_stride, 1u)
                    : make_tmap_2d(&tx, x, (uint64_t)x_rows, (uint64_t)K, (uint64_t)K, (uint32_t)p.xbox);
  if (rc) return rc;
  const long long tiles = (long long)max_tiles * p.w_tiles;
  if (mode == 1) return gemm_launch<GEMM_SWIGLU>(tw, tx, p, tiles, (cudaStream_t)stream);
  return gemm_launch<GEMM_PLAIN>(tw, tx, p, tiles, (cudaStream_t)stream);
}
}  // namespace b200

extern "C" int b200_moe_grouped_gemm(const void* x, const void* w, const void* row_scale, void* out,
                                     const void* tile_table, const void* tile_count, long long x_rows,
                                     int num_groups, int n_out, int K, long long out_row_stride,
                                     int max_tiles, int tile_rows_max, int mode, void* stream) {
  return b200::moe_grouped_gemm_impl(x, x_rows, K, nullptr, w, row_scale, out, tile_table, tile_count, num_groups,
                                     n_out, K, out_row_stride, max_tiles, tile_rows_max, mode, stream);
}

// The same GEMM reading its activation rows where they lie: x is the unpermuted [T, K] matrix and sorted row r
// of the tile table is x[gather_index[r]] (quack's `A_idx`, fused_moe.py:319-322).  No permuted copy of the
// activations is made; the result is the same bits as b200_moe_grouped_gemm on the permuted copy.
// gather_index [sorted rows] i32 comes from b200_moe_permute_index.  tile_rows_max <= 128.
extern "C" int b200_moe_grouped_gemm_gather(const void* x, long long T, long long x_row_stride,
                                            const void* gather_index, const void* w, const void* row_scale,
                                            void* out, const void* tile_table, const void* tile_count,
                                            int num_groups, int n_out, int K, long long out_row_stride,
                                            int max_tiles, int tile_rows_max, int mode, void* stream) {
  if (!gather_index) return B200_ERR_ARG;
  return b200::moe_grouped_gemm_impl(x, T, x_row_stride, gather_index, w, row_scale, out, tile_table, tile_count,
                                     num_groups, n_out, K, out_row_stride, max_tiles, tile_rows_max, mode, stream);
}

#ifdef B200_GEMM_TRACE
extern "C" int b200_debug_gemm_trace(long long* host_out /* [256][8] */) {
  cudaDeviceSynchronize();
  const size_t bytes = sizeof(unsigned long long) * 256 * 8;
  if (cudaMemcpyFromSymbol(host_out, b200::g_gemm_trace, bytes) != cudaSuccess) return -1;
  void* dev = nullptr;
  if (cudaGetSymbolAddress(&dev, b200::g_gemm_trace) != cudaSuccess) return -1;
  return cudaMemset(dev, 0, bytes) == cudaSuccess ? 0 : -1;   // the next launch starts from a clean slate
}
#endif
