// Causal paged-KV attention on tcgen05 tensor cores (decode, chunked prefill, full prefill).
//
// Same interface, work split and invariance rules as attn.cuh; what changes is where the two
// contractions run.  A tile is NC "columns" (a column = one (query position, query head) pair of one
// KV head of one sequence); its keys are walked in blocks of 128:
//
//   S^T[key, col] = K[key, :] . Q[col, :]      UMMA M = 128 keys, N = NC, K = head dim   -> TMEM
//   softmax over keys, per column               256 compute threads
//   O^T[d, col]   = V[key, d]^T . P^T[key, col] UMMA M = 128 (d), N = NC, K = 128 keys    -> TMEM
//
// K and V pages arrive by TMA (4-D tensor map over the cache, one box per 16-token page and 64-wide
// half of the head dim, 128-byte swizzle), which is exactly the canonical UMMA layout: K is consumed
// K-major, V MN-major (its contraction dim, the keys, is the row dim), no transposes anywhere.
//
// The kernel is persistent: one CTA per SM takes tiles round-robin, and every role keeps a running
// block counter over its tiles, so the K and V rings, the two S buffers in tensor memory and the two
// Q buffers carry on from one tile into the next without draining.
//
// Warp roles (12 warps): 0 = K producer and 10 = V producer (TMA + page-table look-ups, one block
// ahead), 1 = UMMA issuer and TMEM owner (QK^T runs one block ahead of PV), 11 = Q loader (one tile
// ahead), 2..9 = compute.  A compute thread is TMEM lane tl - key tl of the block when it reads S^T,
// value dim tl when it reads O^T - for half of the columns (the two warps of a lane quadrant split
// the column groups of four): two warps per scheduler hide each other's latencies.  Per block it
// publishes its warp's per-column maximum (redux.sync), takes the new running maximum, writes
// p = 2^(s - m) as bf16 into the P^T tile, adds the block's p over its warp's 32 keys (a butterfly, xor
// 16 / 8 / 4 / 2 / 1) into that key group's running row sum (l_g = l_g * alpha + s_g) and folds the previous
// block's O^T into its fp32 accumulators; the four group sums of a row meet at the end of the tile as
// (l_0 + l_1) + (l_2 + l_3).  attn_rows.cuh performs the same operations with a row per thread.
//
// Invariance: a column's arithmetic (block order, rescale, bf16 rounding of P before the PV product
// and before the row sum, the row-sum tree) does not depend on NC, on the other columns or on the
// batch; masked keys contribute exact zeros.  All waits are bounded.
#pragma once
#include <cuda.h>

#include "attn.cuh"

namespace b200 {

constexpr int ATC_BN = 128;       // keys per block
constexpr int ATC_THREADS = 384;  // K producer, MMA, 8 compute warps, V producer, Q loader

// Shared-memory descriptor for an MN-major bf16 operand stored as [k rows][64 mn elements] tiles with
// the 128-byte swizzle: 8 k rows are 1024 B apart (stride byte offset), consecutive 64-element MN
// groups are `mn_group_bytes` apart (leading byte offset).
__device__ __forceinline__ uint64_t umma_desc_mn_sw128(uint32_t smem_addr, uint32_t mn_group_bytes) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);
  d |= (uint64_t)((mn_group_bytes >> 4) & 0x3FFFu) << 16;
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}

// bf16 x bf16 -> fp32, M = 128; a_mn selects an MN-major A operand.
__device__ __forceinline__ uint32_t umma_idesc_bf16(uint32_t n, bool a_mn) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((a_mn ? 1u : 0u) << 15) | ((n >> 3) << 17) | ((128u >> 4) << 24);
}

// 2^x for x <= 0 on the special-function unit (results below the normal range flush to zero).
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Sums N per-lane values over the 32 lanes of a warp for N columns at once: at each butterfly step a lane
// keeps half of its columns and hands the other half to its partner, so N columns cost N - 1 + (5 - log2 N)
// shuffles instead of 5 N.  Every column is added in the plain butterfly order (xor 16, 8, 4, 2, 1).  On
// return e[0] holds the sum of column `halving_col<N>(lane)`.
template <int N>
__device__ __forceinline__ int halving_col(int lane) {
  int col = 0, cnt = N;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    if (cnt > 1) {
      cnt >>= 1;
      if (lane & o) col += cnt;
    }
  }
  return col;
}
template <int N>
__device__ __forceinline__ void halving_warp_sum(float (&e)[N], int lane) {
  int cnt = N;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    if (cnt > 1) {
      cnt >>= 1;
      const bool up = lane & o;
#pragma unroll
      for (int i = 0; i < N / 2; ++i) {
        if (i < cnt) {
          const float got = __shfl_xor_sync(0xffffffffu, up ? e[i] : e[i + cnt], o);
          e[i] = (up ? e[i + cnt] : e[i]) + got;
        }
      }
    } else {
      e[0] += __shfl_xor_sync(0xffffffffu, e[0], o);
    }
  }
}

// One unit of work: NC columns of one (sequence, KV head[, head chunk]) pair.
struct AtcTile {
  int seq, kvh, hchunk, heads_here, pos_per_tile, q_start, q_len, kv_len, tile_pos0, q_abs0, nblk;
  bool valid;
};

// The three words of a tile's description that live in global memory.
struct AtcRaw {
  int q_start, q_end, kv_len, seq, eff;
};

// Tiles are numbered with the KV head fastest, then the sequence slot, then the query tile from the LAST
// tile of a sequence down to the first: under the causal mask a later query tile walks more key blocks,
// so the numbering runs from the most expensive tiles to the cheapest and the round-by-round dealing below
// hands every CTA a similar total.  Slot i is sequence seq_order[i] when the caller gives an order
// (longest contexts first), else sequence i.
// The persistent CTAs take the tiles round by round, every other round in reverse ("snake"): with a
// longest-first order the CTAs' totals then differ by about one tile however ragged the batch is.
// Position `lin` of a CTA's walk (blockIdx.x + round * gridDim.x) maps to tile `eff`, or to none in the
// last, partly filled round.
__device__ __forceinline__ int atc_eff(const AttnParams& p, int lin) {
  const int G = (int)gridDim.x;
  const int round = lin / G, pos = lin - round * G;
  const int eff = round * G + ((round & 1) ? G - 1 - pos : pos);
  return eff < p.tc_tiles ? eff : -1;
}

__device__ __forceinline__ AtcRaw atc_raw(const AttnParams& p, int lin) {
  AtcRaw r = {0, 0, 0, 0, -1};
  r.eff = atc_eff(p, lin);
  if (r.eff < 0) return r;
  const int slot = (r.eff % (p.tc_hy * p.num_seqs)) / p.tc_hy;
  r.seq = p.seq_order ? p.seq_order[slot] : slot;
  if (r.seq < 0 || r.seq >= p.num_seqs) {  // a bad order entry: skip the tile, flag it
    report_status(B200_STATUS_BAD_INDEX, r.seq);
    r.eff = -1;
    return r;
  }
  r.q_start = p.cu_seqlens_q[r.seq];
  r.q_end = p.cu_seqlens_q[r.seq + 1];
  r.kv_len = p.seqused_k[r.seq];
  const int q_len = r.q_end - r.q_start;
  if (q_len > p.max_seqlen_q || (q_len > 0 && r.kv_len < q_len)) {
    // more queries than the tile grid covers, or fewer keys than queries: skip the tile, flag the sequence
    report_status(B200_STATUS_BAD_INDEX, r.seq);
    r.eff = -1;
  }
  return r;
}

template <int NC>
__device__ __forceinline__ void atc_make(const AttnParams& p, int lin, const AtcRaw& r, AtcTile& t) {
  const int eff = r.eff < 0 ? 0 : r.eff;
  const int x = p.tc_q_tiles - 1 - eff / (p.tc_hy * p.num_seqs);
  const int y = eff % p.tc_hy;
  t.seq = r.seq;
  t.kvh = y / p.head_chunks;
  t.hchunk = y % p.head_chunks;
  t.heads_here = min(8, p.group - t.hchunk * 8);
  t.pos_per_tile = NC / t.heads_here;
  t.q_start = r.q_start;
  t.q_len = r.q_end - r.q_start;
  t.kv_len = r.kv_len;
  t.tile_pos0 = x * t.pos_per_tile;
  t.valid = r.eff >= 0 && t.q_len > 0 && t.kv_len > 0 && t.tile_pos0 < t.q_len;
  t.q_abs0 = t.kv_len - t.q_len;
  int last_q = t.tile_pos0 + t.pos_per_tile - 1;
  if (last_q > t.q_len - 1) last_q = t.q_len - 1;
  t.nblk = t.valid ? (t.q_abs0 + last_q) / ATC_BN + 1 : 0;
}

template <int NC>
__device__ __forceinline__ void atc_tile(const AttnParams& p, int lin, AtcTile& t) {
  atc_make<NC>(p, lin, atc_raw(p, lin), t);
}


// First valid tile at or after lin in this CTA's round-robin sequence, or -1.
template <int NC>
__device__ __forceinline__ int atc_next_tile(const AttnParams& p, int lin, AtcTile& t) {
  for (; lin < p.tc_slots; lin += (int)gridDim.x) {
    atc_tile<NC>(p, lin, t);
    if (t.valid) return lin;
  }
  return -1;
}

template <int DK, int DV, int NC, int KST, int VST>
__global__ void __launch_bounds__(ATC_THREADS, 1)
paged_attn_tc_kernel(const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v,
                     const AttnParams p) {
  static_assert(DV == 128, "the PV product puts the value dim on the 128 UMMA rows");
  constexpr int KH = DK / 64, VH = DV / 64;
  constexpr int K_BYTES = ATC_BN * DK * 2, V_BYTES = ATC_BN * DV * 2;
  constexpr int KV_BYTES = KST * K_BYTES + VST * V_BYTES;  // a ring of K blocks, then a ring of V blocks
  constexpr int Q_BYTES = KH * NC * 128;      // KH halves of [NC rows][128 B]; two such buffers
  constexpr int TMEM_COLS = (3 * NC <= 32) ? 32 : (3 * NC <= 64) ? 64 : (3 * NC <= 128) ? 128 : 256;

  extern __shared__ uint8_t smem_raw[];
  __shared__ uint64_t bars[2 * KST + 2 * VST + 12];
  __shared__ int abort_mem;
  __shared__ uint32_t tmem_slot;
  __shared__ __align__(16) int s_cpos[NC];          // absolute query position of each column
  __shared__ __align__(16) float s_wmax[2][NC][4];  // per-warp column maxima of a block (by block parity)
  __shared__ __align__(16) float s_m[2][NC];        // running maxima after a block (by block parity)
  __shared__ __align__(16) float s_alpha[2][NC];    // rescale factors of a block (by block parity)
  __shared__ __align__(16) float s_lred[NC][4];     // per-warp row sums at the end of a tile
  volatile int* abort_flag = &abort_mem;

  const uint32_t raw = ptx::smem_u32(smem_raw);
  const uint32_t base = (raw + 1023) & ~1023u;
  uint8_t* base_ptr = smem_raw + (base - raw);
  const uint32_t v_ring = base + KST * K_BYTES;
  const uint32_t q_smem = base + KV_BYTES;
  const uint32_t p_smem = q_smem + 2 * Q_BYTES;
  uint8_t* q_ptr = base_ptr + KV_BYTES;
  uint8_t* p_ptr = q_ptr + 2 * Q_BYTES;

  auto bar = [&](int i) { return ptx::smem_u32(&bars[i]); };
  constexpr int NB = 2 * KST + 2 * VST;
  auto kfull_bar = [&](int s) { return bar(s); };
  auto kempty_bar = [&](int s) { return bar(KST + s); };
  auto vfull_bar = [&](int s) { return bar(2 * KST + s); };
  auto vempty_bar = [&](int s) { return bar(2 * KST + VST + s); };
  auto sfull_bar = [&](int b) { return bar(NB + b); };
  auto sfree_bar = [&](int b) { return bar(NB + 2 + b); };
  const uint32_t pready_bar = bar(NB + 4), ofull_bar = bar(NB + 5), ofree_bar = bar(NB + 6);
  auto qfull_bar = [&](int b) { return bar(NB + 7 + b); };
  auto qfree_bar = [&](int b) { return bar(NB + 9 + b); };

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int s = 0; s < KST; ++s) {
      ptx::mbar_init(kfull_bar(s), 1);
      ptx::mbar_init(kempty_bar(s), 1);
    }
    for (int s = 0; s < VST; ++s) {
      ptx::mbar_init(vfull_bar(s), 1);
      ptx::mbar_init(vempty_bar(s), 1);
    }
    for (int b = 0; b < 2; ++b) {
      ptx::mbar_init(sfull_bar(b), 1);
      ptx::mbar_init(sfree_bar(b), 8);  // one arrival per compute warp
      ptx::mbar_init(qfull_bar(b), 1);
      ptx::mbar_init(qfree_bar(b), 1);
    }
    ptx::mbar_init(pready_bar, 8);
    ptx::mbar_init(ofull_bar, 1);
    ptx::mbar_init(ofree_bar, 8);
    ptx::fence_barrier_init();
    ptx::prefetch_tensormap(&tm_k);
    ptx::prefetch_tensormap(&tm_v);
  }
  if (warp == 1) {
    ptx::tmem_alloc(ptx::smem_u32(&tmem_slot), TMEM_COLS);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem_base = tmem_slot;
  const uint32_t tm_s0 = tmem_base, tm_o = tmem_base + 2 * NC;
  pdl_trigger();
  pdl_wait();  // set-up above; the previous kernel's outputs are read from here on

  if (warp == 0 || warp == 10) {
    // ------------------------------------------------------------------ TMA producers (whole warps):
    // warp 0 streams K blocks, warp 6 streams V blocks, each through its own ring, so K runs ahead as
    // soon as a QK^T has consumed its block and V as soon as a PV product has; both run ahead across
    // tile boundaries.
    const bool is_k = warp == 0;
    const int nst = is_k ? KST : VST, halves = is_k ? KH : VH;
    const uint32_t blk_bytes = is_k ? K_BYTES : V_BYTES;
    const uint32_t ring = is_k ? base : v_ring;
    const CUtensorMap* tm = is_k ? &tm_k : &tm_v;
    const int boxes = ATC_BN / p.box_tokens;
    uint32_t g = 0;  // running block counter over this CTA's tiles
    bool ok = true;
    for (int lin = blockIdx.x; lin < p.tc_slots && ok; lin += (int)gridDim.x) {
      AtcTile t;
      atc_tile<NC>(p, lin, t);
      if (!t.valid) continue;
      const int* ptab = p.page_table + (long long)t.seq * p.page_table_stride;
      const int valid_pages = (t.kv_len + p.page_size - 1) / p.page_size;
      // lane b's page of block j; read one block ahead so that the look-up is over when the slot frees
      auto page_of = [&](int j, int b, int& in_page) {
        const int tok = j * ATC_BN + b * p.box_tokens;
        const int lpage = tok / p.page_size;
        in_page = tok - lpage * p.page_size;
        int phys = -1;
        if (lpage < valid_pages && lpage < p.max_pages) phys = ptab[lpage];
        if (phys < 0 || phys >= p.num_blocks) phys = -1;  // out-of-range block: TMA fills zeros
        return phys;
      };
      int in_page_next = 0;
      int phys_next = lane < boxes ? page_of(0, lane, in_page_next) : -1;
      for (int j = 0; j < t.nblk && ok; ++j, ++g) {
        const int phys0 = phys_next, in_page0 = in_page_next;
        if (j + 1 < t.nblk && lane < boxes) phys_next = page_of(j + 1, lane, in_page_next);
        const int s = g % nst;
        const uint32_t fb = is_k ? kfull_bar(s) : vfull_bar(s);
        bool w = true;
        if (lane == 0)
          w = ptx::mbar_wait(is_k ? kempty_bar(s) : vempty_bar(s), ((g / nst) & 1) ^ 1, abort_flag, 600 + s);
        ok = __all_sync(0xffffffffu, w);
        if (!ok) break;
        const uint32_t dst = ring + (uint32_t)s * blk_bytes;
        if (lane == 0) ptx::mbar_expect_tx(fb, blk_bytes);
        __syncwarp();
        for (int b = lane; b < boxes; b += 32) {
          int in_page = in_page0;
          const int phys = b == lane ? phys0 : page_of(j, b, in_page);
          const uint32_t row_off = (uint32_t)(b * p.box_tokens) * 128;
          for (int h = 0; h < halves; ++h)
            ptx::tma_load_4d(dst + h * (ATC_BN * 128) + row_off, tm, fb, h * 64, t.kvh, in_page, phys,
                             ptx::kEvictFirst);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ UMMA issuer
    if (ptx::elect_one()) {
      const uint32_t idesc_s = umma_idesc_bf16(NC, false), idesc_o = umma_idesc_bf16(NC, true);
      const uint64_t hi_k = ptx::umma_desc_k_sw128(0) & 0xFFFFFFFF00000000ull;
      auto kdesc = [&](uint32_t addr) { return hi_k | (uint64_t)(((addr & 0x3FFFFu) >> 4) | (1u << 16)); };
      AtcTile t;
      int lin = atc_next_tile<NC>(p, blockIdx.x, t);  // tile of the next QK^T to issue
      uint32_t gs = 0, gp = 0, tile_it = 0;                 // next QK^T block, next PV block, tile counter
      int j = 0;                                            // block of that tile
      AtcRaw raw_next = {0, 0, 0, 0, -1};
      auto issue_next_s = [&]() {  // S^T of global block gs into S buffer gs & 1
        const int qb = tile_it & 1;
        if (j == 0) {
          // the next tile's description: loads only, used when this tile's last QK^T has been issued
          if (lin + (int)gridDim.x < p.tc_slots) raw_next = atc_raw(p, lin + (int)gridDim.x);
          if (!ptx::mbar_wait(qfull_bar(qb), (tile_it >> 1) & 1, abort_flag, 605 + qb)) return false;
        }
        const int s = gs % KST, b = gs & 1;
        if (!ptx::mbar_wait(kfull_bar(s), (gs / KST) & 1, abort_flag, 610 + s)) return false;
        if (!ptx::mbar_wait(sfree_bar(b), ((gs >> 1) & 1) ^ 1, abort_flag, 620 + b)) return false;
        ptx::tc_fence_after();
        const uint32_t sk = base + (uint32_t)s * K_BYTES, qs = q_smem + qb * Q_BYTES;
#pragma unroll
        for (int kk = 0; kk < DK / 16; ++kk) {
          const uint64_t da = kdesc(sk + (kk >> 2) * (ATC_BN * 128) + (kk & 3) * 32);
          const uint64_t db = kdesc(qs + (kk >> 2) * (NC * 128) + (kk & 3) * 32);
          ptx::umma_bf16(tm_s0 + b * NC, da, db, idesc_s, kk != 0 ? 1u : 0u);
        }
        ptx::umma_commit(sfull_bar(b));
        ptx::umma_commit(kempty_bar(s));  // the K block is free once this QK^T has read it
        ++gs;
        if (++j == t.nblk) {
          ptx::umma_commit(qfree_bar(qb));  // every QK^T of this tile has been issued: Q buffer reusable
          j = 0;
          ++tile_it;
          const int cand = lin + (int)gridDim.x;
          lin = -1;
          if (cand < p.tc_slots) {
            atc_make<NC>(p, cand, raw_next, t);
            lin = t.valid ? cand : atc_next_tile<NC>(p, cand + (int)gridDim.x, t);
          }
        }
        return true;
      };
      // QK^T runs one block ahead of the PV product (two S buffers in tensor memory), also from one
      // tile into the next; the PV product depends on the block number alone.
      bool ok = lin >= 0 && issue_next_s();
      while (ok && gp < gs) {
        if (lin >= 0 && !issue_next_s()) break;
        const uint32_t g = gp;
        const int s = g % VST;
        if (!ptx::mbar_wait(pready_bar, g & 1, abort_flag, 630)) break;
        if (!ptx::mbar_wait(ofree_bar, (g & 1) ^ 1, abort_flag, 631)) break;
        if (!ptx::mbar_wait(vfull_bar(s), (g / VST) & 1, abort_flag, 615 + s)) break;
        ptx::tc_fence_after();
        const uint32_t sv = v_ring + (uint32_t)s * V_BYTES;
#pragma unroll
        for (int kk = 0; kk < ATC_BN / 16; ++kk) {
          // A = V^T: 16 keys per step are 16 rows of 128 B; the second 64-wide d half is ATC_BN*128 B on
          const uint64_t da = umma_desc_mn_sw128(sv + kk * 16 * 128, ATC_BN * 128);
          const uint64_t db = kdesc(p_smem + (kk >> 2) * (NC * 128) + (kk & 3) * 32);
          ptx::umma_bf16(tm_o, da, db, idesc_o, kk != 0 ? 1u : 0u);
        }
        ptx::umma_commit(ofull_bar);
        ptx::umma_commit(vempty_bar(s));
        ++gp;
      }
    }
  } else if (warp == 11) {
    // ------------------------------------------------------------------ Q loader (whole warp): the
    // tile's query rows go to shared memory in the K-major swizzled layout (B operand of S^T = K Q^T),
    // one tile ahead of the tile being computed (two Q buffers).
    AtcTile t;
    uint32_t tile_it = 0;
    for (int lin = atc_next_tile<NC>(p, blockIdx.x, t); lin >= 0;
         lin = atc_next_tile<NC>(p, lin + (int)gridDim.x, t), ++tile_it) {
      const int qb = tile_it & 1;
      bool w = true;
      if (lane == 0) w = ptx::mbar_wait(qfree_bar(qb), ((tile_it >> 1) & 1) ^ 1, abort_flag, 660 + qb);
      if (!__all_sync(0xffffffffu, w)) break;
      uint8_t* qd = q_ptr + qb * Q_BYTES;
#pragma unroll 4
      for (int i = lane; i < NC * (DK / 8); i += 32) {
        const int c = i / (DK / 8), ch = i % (DK / 8);  // column, 16-byte chunk of its row
        const int pi = c / t.heads_here;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (pi < t.pos_per_tile && t.tile_pos0 + pi < t.q_len) {
          const int head = t.kvh * p.group + t.hchunk * 8 + (c % t.heads_here);
          const __nv_bfloat16* qrow = p.q + (long long)(t.q_start + t.tile_pos0 + pi) * p.q_tok_stride +
                                      (long long)head * p.q_head_stride;
          v = *reinterpret_cast<const uint4*>(qrow + ch * 8);
        }
        *reinterpret_cast<uint4*>(qd + (ch >> 3) * (NC * 128) + sw128(c, ch & 7)) = v;
      }
      ptx::fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(qfull_bar(qb));
    }
  } else {
    // ------------------------------------------------------------------ compute threads (warps 2..9)
    // A thread is TMEM lane `tl` (key tl of the block for S^T, value dim tl for O^T) for half of the
    // tile's columns: columns come in groups of four and the two warps of a lane quadrant take the even
    // and the odd groups.  Per block:
    //   A  read my key's scores, scale and mask them, publish the warp's per-column maximum
    //   B  running maximum and rescale factor alpha (one thread per column; with few columns every
    //      thread does it for itself in phase C and the barrier goes away)
    //   C  p = 2^(s - m) rounded to bf16 -> P^T tile and my per-key share of the row sum;
    //      o = (o + O^T of the previous block) * alpha
    // The row sum stays split over the 128 key lanes until the tile ends.
    constexpr int NCT = 256;           // compute threads
    constexpr int NG = NC / 8;         // column groups per thread
    constexpr int NCL = NC / 2;        // columns per thread
    constexpr int CHG = 2;             // groups handled per pass (bounds the registers in flight)
    constexpr bool LOCAL_M = NC <= 16;
    // The running maximum never goes below this, so a column whose keys are all masked so far (only
    // possible for a query placed before the cached context) needs no -inf special cases: its
    // probabilities and rescale factors come out as exact zeros.
    constexpr float kMinMax = -3.0e38f;
    const int ct = threadIdx.x - 64;   // 0..255
    const int q4 = warp & 3;           // TMEM lane quadrant of this warp
    const int hsel = (warp - 2) >> 2;  // 0: even column groups, 1: odd ones
    const int tl = q4 * 32 + lane;     // TMEM lane
    const uint32_t lane_addr = (uint32_t)(q4 * 32) << 16;
    auto gcol = [&](int lg) { return (2 * lg + hsel) * 4; };  // first column of my group lg
    const int mycol = halving_col<NCL>(lane);                 // the local column whose row sum I end up holding
    // my key's 2-byte slot in row c of the P^T tile (K-major, 128-byte swizzle) is
    // p_mine + c*128 + ((p_ch ^ (c&7)) << 4); for column i of my group lg that is p_slot[i] + lg*1024
    uint8_t* p_mine = p_ptr + (tl >> 6) * (NC * 128) + (tl & 7) * 2;
    const int p_ch = (tl & 63) >> 3;
    uint8_t* p_slot[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) p_slot[i] = p_mine + (hsel * 4 + i) * 128 + ((p_ch ^ (hsel * 4 + i)) << 4);
    uint32_t g0 = 0;
    AtcTile t, tn;
    int lin = atc_next_tile<NC>(p, blockIdx.x, t);
    while (lin >= 0) {
      // the next tile's description is read now (loads only, nothing waits for them) so that it is at
      // hand when the tile starts
      const int cand = lin + (int)gridDim.x;
      const bool have_cand = cand < p.tc_slots;
      AtcRaw raw_next = {0, 0, 0, 0, -1};
      if (have_cand) raw_next = atc_raw(p, cand);
      // columns at or beyond ncv are padding: their scores are never looked at and whatever their P^T
      // rows hold only reaches O^T columns that are not stored
      const int npos = min(t.pos_per_tile, t.q_len - t.tile_pos0);
      const int ncv = npos * t.heads_here;
      // Narrow (decode) tiles skip their padding groups; wide tiles work on them too, which keeps the
      // column groups in one straight run of instructions (padding only occurs in a sequence's last tile).
      auto live = [&](int gc) { return NC > 16 || gc < ncv; };
      bool go;
      for (int c = ct; c < NC; c += NCT) {
        const int pi = c / t.heads_here;
        s_cpos[c] = t.q_abs0 + t.tile_pos0 + (pi < npos ? pi : 0);
      }
      ptx::named_barrier_sync(3, NCT);
      if (*abort_flag) break;

      float o_acc[NCL];
      float l_w = 0.f;   // running row sum of my warp's 32 keys for local column `mycol`
      float m_run[LOCAL_M ? NCL : 1];
#pragma unroll
      for (int c = 0; c < NCL; ++c) {
        o_acc[c] = 0.f;
        if constexpr (LOCAL_M) m_run[c] = -INFINITY;
      }
      // scale and causal mask of four raw scores of my key, columns gc..gc+3
      auto finish_scores = [&](const uint32_t (&r)[4], int gc, int key, float (&v)[4]) {
        const int4 cp = *reinterpret_cast<const int4*>(&s_cpos[gc]);
        const int cpv[4] = {cp.x, cp.y, cp.z, cp.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float sc = __uint_as_float(r[i]) * p.qk_scale;
          v[i] = key > cpv[i] ? -INFINITY : sc;
        }
      };
      for (int j = 0; j < t.nblk; ++j) {
        const uint32_t g = g0 + j;
        const int b = g & 1, s = g % VST;
        const int key0 = j * ATC_BN;
        const int key = key0 + tl;
        float sv[NC == 16 ? NCL : 1];  // with few columns the scores are kept from phase A to phase C
        // A wait that gives up raises the CTA's abort flag before its thread reaches the next named
        // barrier; every thread still arrives at every barrier and all leave the loops together after it.
        go = __all_sync(0xffffffffu, ptx::mbar_wait(sfull_bar(b), (g >> 1) & 1, abort_flag, 640 + b));
        if (go) {
          ptx::tc_fence_after();
          // (A) per-column maximum over this warp's 32 keys
#pragma unroll
          for (int ch0 = 0; ch0 < NG; ch0 += CHG) {
            uint32_t rs[CHG][4];
#pragma unroll
            for (int k = 0; k < CHG; ++k)
              if (live(gcol(ch0 + k))) ptx::tmem_ld4(tm_s0 + b * NC + lane_addr + gcol(ch0 + k), rs[k]);
            ptx::tmem_ld_wait();
#pragma unroll
            for (int k = 0; k < CHG; ++k) {
              const int gc = gcol(ch0 + k);
              if (live(gc)) {
                float v[4];
                finish_scores(rs[k], gc, key, v);
                float mine = -INFINITY;
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                  float w;
                  asm volatile("redux.sync.max.f32 %0, %1, 0xffffffff;" : "=f"(w) : "f"(v[i]));
                  if ((lane & 3) == i) mine = w;
                  if constexpr (NC == 16) sv[(ch0 + k) * 4 + i] = v[i];
                }
                if (lane < 4) s_wmax[b][gc + lane][q4] = mine;
              }
            }
          }
          // keys at or beyond kv_len may hold anything: clear their V rows so that 0 * V stays 0
          if (key0 + ATC_BN > t.kv_len &&
              __all_sync(0xffffffffu, ptx::mbar_wait(vfull_bar(s), (g / VST) & 1, abort_flag, 645))) {
            uint8_t* vt = base_ptr + (size_t)KST * K_BYTES + (size_t)s * V_BYTES;
            for (int r = t.kv_len - key0 + (ct >> 5); r < ATC_BN; r += NCT / 32)
#pragma unroll
              for (int h = 0; h < VH; ++h) reinterpret_cast<uint32_t*>(vt + h * (ATC_BN * 128) + r * 128)[lane] = 0u;
          }
        }
        ptx::named_barrier_sync(3, NCT);
        if (*abort_flag) break;
        // (B) running maximum and rescale factor, one thread per column
        if constexpr (!LOCAL_M) {
          for (int c = ct; c < NC; c += NCT) {
            const float4 w = *reinterpret_cast<const float4*>(s_wmax[b][c]);
            const float m_old = j == 0 ? -INFINITY : s_m[b ^ 1][c];
            const float m_new = fmaxf(fmaxf(m_old, kMinMax), fmaxf(fmaxf(w.x, w.y), fmaxf(w.z, w.w)));
            s_m[b][c] = m_new;
            s_alpha[b][c] = fast_exp2(m_old - m_new);
          }
          ptx::named_barrier_sync(3, NCT);
          if (*abort_flag) break;
        }
        // (C) the previous block's PV product has been running meanwhile; once it is over its O^T can be
        //     folded in and the P^T tile it read can be rewritten
        go = true;
        if (j > 0) go = __all_sync(0xffffffffu, ptx::mbar_wait(ofull_bar, (g - 1) & 1, abort_flag, 650));
        if (go) {
          ptx::tc_fence_after();
          float pfl[NCL];       // this block's bf16-rounded p of my key, per local column
          float a_mine = 0.f;   // alpha of local column `mycol`
#pragma unroll
          for (int c = 0; c < NCL; ++c) pfl[c] = 0.f;
#pragma unroll
          for (int ch0 = 0; ch0 < NG; ch0 += CHG) {
            uint32_t rc[CHG][4], ro[CHG][4];
#pragma unroll
            for (int k = 0; k < CHG; ++k) {
              const int gc = gcol(ch0 + k);
              if (live(gc)) {
                if constexpr (NC != 16) ptx::tmem_ld4(tm_s0 + b * NC + lane_addr + gc, rc[k]);
                // (block 0 reads whatever the buffer holds and drops it below: no branch in this run)
                ptx::tmem_ld4(tm_o + lane_addr + gc, ro[k]);
              }
            }
            ptx::tmem_ld_wait();
            // Loads first, stores last: the compiler cannot tell that the P^T stores leave the shared
            // arrays read here alone, so interleaving them would serialise the columns.
            float v[CHG][4], mv[CHG][4], av[CHG][4];
#pragma unroll
            for (int k = 0; k < CHG; ++k) {
              const int gc = gcol(ch0 + k);
              if (live(gc)) {
                if constexpr (NC == 16) {
#pragma unroll
                  for (int i = 0; i < 4; ++i) v[k][i] = sv[(ch0 + k) * 4 + i];
                } else {
                  finish_scores(rc[k], gc, key, v[k]);
                }
                if constexpr (LOCAL_M) {
#pragma unroll
                  for (int i = 0; i < 4; ++i) {
                    const float4 w = *reinterpret_cast<const float4*>(s_wmax[b][gc + i]);
                    mv[k][i] = fmaxf(fmaxf(m_run[(ch0 + k) * 4 + i], kMinMax), fmaxf(fmaxf(w.x, w.y), fmaxf(w.z, w.w)));
                  }
                } else {
                  const float4 m4 = *reinterpret_cast<const float4*>(&s_m[b][gc]);
                  const float4 a4 = *reinterpret_cast<const float4*>(&s_alpha[b][gc]);
                  mv[k][0] = m4.x, mv[k][1] = m4.y, mv[k][2] = m4.z, mv[k][3] = m4.w;
                  av[k][0] = a4.x, av[k][1] = a4.y, av[k][2] = a4.z, av[k][3] = a4.w;
                }
              }
            }
            __nv_bfloat16 pb[CHG][4];
#pragma unroll
            for (int k = 0; k < CHG; ++k) {
              if (live(gcol(ch0 + k))) {
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                  const int lc = (ch0 + k) * 4 + i;
                  if constexpr (LOCAL_M) {
                    av[k][i] = fast_exp2(m_run[lc] - mv[k][i]);
                    m_run[lc] = mv[k][i];
                  }
                  pb[k][i] = f2bf(fast_exp2(v[k][i] - mv[k][i]));
                  pfl[lc] = bf2f(pb[k][i]);
                  if (lc == mycol) a_mine = av[k][i];
                  // (the first block finds o = 0 and no O^T yet: the product below is 0 either way)
                  o_acc[lc] += j > 0 ? __uint_as_float(ro[k][i]) : 0.f;
                  o_acc[lc] *= av[k][i];
                }
              }
            }
#pragma unroll
            for (int k = 0; k < CHG; ++k) {
              const int gc = gcol(ch0 + k);
              if (live(gc)) {
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                  *reinterpret_cast<__nv_bfloat16*>(p_slot[i] + (ch0 + k) * 1024) = pb[k][i];
                }
              }
            }
          }
          // the block's p summed over my warp's 32 keys, every column in butterfly order
          halving_warp_sum<NCL>(pfl, lane);
          l_w = l_w * a_mine + pfl[0];
          // every thread orders its own tensor-memory reads and shared-memory writes, then one lane
          // per warp arrives (256 arrivals on one barrier word would serialise)
          ptx::tc_fence_before();
          ptx::fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            ptx::mbar_arrive(sfree_bar(b));  // this S buffer may be overwritten two blocks on
            if (j > 0) ptx::mbar_arrive(ofree_bar);
            ptx::mbar_arrive(pready_bar);
          }
        }
      }
      go = !*abort_flag;
      if (go) go = __all_sync(0xffffffffu, ptx::mbar_wait(ofull_bar, (g0 + t.nblk - 1) & 1, abort_flag, 651));
      if (go) {
        ptx::tc_fence_after();
#pragma unroll
        for (int ch0 = 0; ch0 < NG; ch0 += CHG) {
          uint32_t ro[CHG][4];
#pragma unroll
          for (int k = 0; k < CHG; ++k)
            if (live(gcol(ch0 + k))) ptx::tmem_ld4(tm_o + lane_addr + gcol(ch0 + k), ro[k]);
          ptx::tmem_ld_wait();
#pragma unroll
          for (int k = 0; k < CHG; ++k)
            if (live(gcol(ch0 + k))) {
#pragma unroll
              for (int i = 0; i < 4; ++i) o_acc[(ch0 + k) * 4 + i] += __uint_as_float(ro[k][i]);
            }
        }
        ptx::tc_fence_before();
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(ofree_bar);
        // row sums: each warp publishes its key group's sum of every column it holds; the four groups
        // are added as (l_0 + l_1) + (l_2 + l_3) below
        s_lred[gcol(mycol >> 2) + (mycol & 3)][q4] = l_w;
      }
      ptx::named_barrier_sync(3, NCT);
      if (*abort_flag) break;  // uniform over the compute threads: read after a common barrier
      // Output.  A thread holds one value-dim element of NC / 2 columns; stored as they are that is one 2-byte
      // store per column.  Each warp turns 8 columns x its 32 dims around in shared memory instead (its 512-byte
      // slice of the P^T tile, which nothing reads between the tile's last PV product and the barrier that
      // opens the next tile), so that a lane stores 16 bytes and one instruction writes all 8 columns.
      const bool vec_out = !p.scalar_out && ((reinterpret_cast<uintptr_t>(p.out) | (uintptr_t)(p.o_tok_stride * 2) |
                             (uintptr_t)(p.o_head_stride * 2)) & 15) == 0;
      if (vec_out) {
        __nv_bfloat16* stg = reinterpret_cast<__nv_bfloat16*>(p_ptr) + (warp - 2) * 256;
#pragma unroll
        for (int g8 = 0; g8 < NCL / 8; ++g8) {
#pragma unroll
          for (int k = 0; k < 8; ++k) {
            const int lc = g8 * 8 + k;
            const int c = ((lc >> 2) << 3) + hsel * 4 + (lc & 3);
            float v = 0.f;
            if (c < ncv) {
              const float4 l4 = *reinterpret_cast<const float4*>(s_lred[c]);
              const float l = (l4.x + l4.y) + (l4.z + l4.w);
              v = o_acc[lc] * (1.0f / l);
            }
            stg[k * 32 + lane] = f2bf(v);
          }
          __syncwarp();
          {
            const int k = lane >> 2, part = lane & 3;
            const int lc = g8 * 8 + k;
            const int c = ((lc >> 2) << 3) + hsel * 4 + (lc & 3);
            if (c < ncv) {
              const int pi = c / t.heads_here, h = c - pi * t.heads_here;
              __nv_bfloat16* orow = p.out + (long long)(t.q_start + t.tile_pos0 + pi) * p.o_tok_stride +
                                    (long long)(t.kvh * p.group + t.hchunk * 8 + h) * p.o_head_stride;
              *reinterpret_cast<uint4*>(orow + q4 * 32 + part * 8) =
                  *reinterpret_cast<const uint4*>(stg + k * 32 + part * 8);
            }
          }
          __syncwarp();
        }
      } else {
        int pi = 0, h = 0;  // column c = position pi of the tile, head h of this KV head's chunk
#pragma unroll
        for (int c = 0; c < NC; ++c) {
          if (((c >> 2) & 1) == hsel && c < ncv) {
            const int lc = ((c >> 3) << 2) + (c & 3);
            const float4 l4 = *reinterpret_cast<const float4*>(s_lred[c]);
            const float l = (l4.x + l4.y) + (l4.z + l4.w);
            __nv_bfloat16* orow = p.out + (long long)(t.q_start + t.tile_pos0 + pi) * p.o_tok_stride +
                                  (long long)(t.kvh * p.group + t.hchunk * 8 + h) * p.o_head_stride;
            orow[tl] = f2bf(o_acc[lc] * (1.0f / l));
          }
          if (++h == t.heads_here) {
            h = 0;
            ++pi;
          }
        }
      }
      g0 += t.nblk;
      lin = -1;
      if (have_cand) {
        atc_make<NC>(p, cand, raw_next, tn);
        lin = tn.valid ? cand : atc_next_tile<NC>(p, cand + (int)gridDim.x, tn);
      }
      t = tn;
    }
  }

  __syncthreads();
  if (*abort_flag) {
    const uint64_t t0 = global_timer_ns();
    while (global_timer_ns() - t0 < 200000ull) {
    }
  }
  ptx::tc_fence_after();
  if (warp == 1) {
    __syncwarp();
    ptx::tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

template <int DK, int DV, int NC, int KST, int VST>
inline int attn_tc_launch(const CUtensorMap& tk, const CUtensorMap& tv, const AttnParams& p, dim3 grid,
                          cudaStream_t st) {
  constexpr int smem = ATC_BN * (KST * DK + VST * DV) * 2 + 2 * (DK / 64) * NC * 128 + 2 * NC * 128 + 1024;
  static_assert(smem <= 227 * 1024, "shared memory budget");
  static PerDeviceFlags attr_set;
  if (int rc = set_max_dyn_smem_once(attr_set, paged_attn_tc_kernel<DK, DV, NC, KST, VST>, smem)) return rc;
  const int nctas = p.tc_tiles < sm_count() ? p.tc_tiles : sm_count();
  (void)grid;
  launch_k(paged_attn_tc_kernel<DK, DV, NC, KST, VST>, dim3((unsigned)nctas), dim3(ATC_THREADS), (size_t)smem, st, tk,
           tv, p);
  return launch_status();
}

inline int attn_tc_dispatch(const CUtensorMap& tk, const CUtensorMap& tv, const AttnParams& p, dim3 grid, int dk,
                            int nc, cudaStream_t st) {
  if (dk == 128 && nc == 16) return attn_tc_launch<128, 128, 16, 3, 3>(tk, tv, p, grid, st);
  if (dk == 128 && nc == 64) return attn_tc_launch<128, 128, 64, 2, 2>(tk, tv, p, grid, st);
  if (dk == 192 && nc == 16) return attn_tc_launch<192, 128, 16, 2, 3>(tk, tv, p, grid, st);
  if (dk == 192 && nc == 32) return attn_tc_launch<192, 128, 32, 2, 2>(tk, tv, p, grid, st);
  return B200_ERR_SHAPE;
}

}  // namespace b200

