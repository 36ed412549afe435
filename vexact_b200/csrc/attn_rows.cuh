// Causal paged-KV attention for prefill / chunked-prefill tiles on tcgen05: query rows on the TMEM lanes.
//
// attn_tc.cuh puts the KEYS of a block on the 128 tensor-memory lanes (S^T = K Q^T), which suits decode
// (few query columns, the KV stream is the bound) but makes the softmax of a wide tile expensive: the
// column maximum is a cross-lane reduction per score and P^T is stored two bytes at a time.  Here a tile
// is 128 ROWS, a row being one (query position, query head) pair of one KV head of one sequence, and two
// threads own a whole row:
//
//   S[row, key]  = Q[row, :] . K[key, :]      UMMA M = 128 rows, N = 128 keys, K = head dim     -> TMEM
//   softmax      two threads per row, 64 keys each in registers: one exchange (the half-row maxima) per block
//   O[row, d]    = P[row, key] . V[key, d]    UMMA M = 128 rows, N = 128 (d), K = 128 keys      -> TMEM
//
// K pages arrive by TMA and are consumed K-major as the B operand of the first product; V pages are
// consumed as they lie (MN-major B operand of the second).  P is written to shared memory as the K-major
// A operand, sixteen bytes at a time.
//
// The arithmetic of a row is, operation for operation, the arithmetic attn_tc.cuh performs for the same
// (position, head) as a column: blocks of 128 keys from key 0 upward, v = s * scale, running maximum with
// the same floor, p = bf16(2^(v - m)), the row sum kept as four 32-key group sums each added in the
// butterfly order (k, k + 16), (.., + 8), (.., + 4), (.., + 2), (.., + 1) with l_g = l_g * alpha + s_g per
// block and l = (l_0 + l_1) + (l_2 + l_3) at the end, O folded block by block as o = (o + O_prev) * alpha.
// A token therefore gets the same bits from a decode step, a chunk and a full prefill.
//
// Warps (12): 0 K producer, 1 UMMA issuer + TMEM owner, 2 V producer, 3 Q loader, 4-11 compute: a row is
// shared by two threads (warps w and w + 4 of a lane quadrant), each taking 64 of the block's 128 keys for
// the softmax and 64 of the 128 value dims for o, the fold and the final store.
// Persistent CTAs, running block counters across tiles, every wait bounded, as in attn_tc.cuh.
#pragma once
#include "attn_tc.cuh"

namespace b200 {

// Development aid (off unless the library is compiled with -DB200_ATTN_TRACE): CTA 0 writes clock64() stamps
// of its roles' per-block events into g_attn_trace[role][block][event].
#ifdef B200_ATTN_TRACE
__device__ long long g_attn_trace[4][64][8];
#define ATR_STAMP(role, blk, ev)                                                          \
  do {                                                                                      \
    if (blockIdx.x == 0 && (threadIdx.x & 31) == 0 && (blk) < 64) g_attn_trace[role][blk][ev] = clock64(); \
  } while (0)
#else
#define ATR_STAMP(role, blk, ev) \
  do {                           \
  } while (0)
#endif

constexpr int ATR_ROWS = 128;      // rows per tile = UMMA M
constexpr int ATR_THREADS = 384;

// bf16 x bf16 -> fp32, M = 128, A K-major, B K-major or MN-major.
__device__ __forceinline__ uint32_t umma_idesc_bf16_b(uint32_t n, bool b_mn) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((b_mn ? 1u : 0u) << 16) | ((n >> 3) << 17) | ((128u >> 4) << 24);
}

// 32 lanes x 32 consecutive 32-bit columns.
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}

// Sum of 32 values in the butterfly order of a warp reduction (xor 16, 8, 4, 2, 1), done by one thread.
__device__ __forceinline__ float butterfly_order_sum32(const float (&p)[32]) {
  float a[16], b[8], c[4];
#pragma unroll
  for (int i = 0; i < 16; ++i) a[i] = p[i] + p[i + 16];
#pragma unroll
  for (int i = 0; i < 8; ++i) b[i] = a[i] + a[i + 8];
#pragma unroll
  for (int i = 0; i < 4; ++i) c[i] = b[i] + b[i + 4];
  return (c[0] + c[2]) + (c[1] + c[3]);
}

template <int DK>
__global__ void __launch_bounds__(ATR_THREADS, 1)
paged_attn_rows_kernel(const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v,
                       const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_out,
                       const AttnParams p) {
  constexpr int DV = 128, NC = ATR_ROWS, KST = 2, VST = 2;
  constexpr int KH = DK / 64, VH = DV / 64;
  constexpr int K_BYTES = ATC_BN * DK * 2, V_BYTES = ATC_BN * DV * 2;
  constexpr int KV_BYTES = KST * K_BYTES + VST * V_BYTES;
  constexpr int Q_BYTES = KH * NC * 128;   // KH halves of [128 rows][128 B]; two such buffers
  constexpr int P_BYTES = 2 * NC * 128;    // two 64-key halves of [128 rows][128 B]
  constexpr int TMEM_COLS = 512;           // S0, S1 (128 each), O (128)

  // All shared memory is dynamic (the tiles take 224 of the 227 KB): the 1024-byte aligned tiles first,
  // then the small arrays.  The launcher asks for the tiles + small arrays + what the alignment may cost.
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = ptx::smem_u32(smem_raw);
  const uint32_t base = (raw + 1023) & ~1023u;
  uint8_t* base_ptr = smem_raw + (base - raw);
  const uint32_t v_ring = base + KST * K_BYTES;
  const uint32_t q_smem = base + KV_BYTES;
  const uint32_t p_smem = q_smem + 2 * Q_BYTES;
  uint8_t* q_ptr = base_ptr + KV_BYTES;
  uint8_t* p_ptr = q_ptr + 2 * Q_BYTES;
  uint8_t* small = p_ptr + P_BYTES;
  {
    uint32_t granted;
    asm volatile("mov.u32 %0, %%dynamic_smem_size;" : "=r"(granted));
    if ((base - raw) + KV_BYTES + 2 * Q_BYTES + P_BYTES + 256 + 4 * NC * 4 + 16 > granted) {
      // the aligned layout does not fit what the launch granted (only possible if something else put
      // static shared memory in front of the dynamic region): every thread leaves before any set-up
      if (threadIdx.x == 0) report_status(B200_STATUS_BAD_INDEX, -(int)(base - raw));
      return;
    }
  }
  uint64_t* bars = reinterpret_cast<uint64_t*>(small);                       // 2*KST + 2*VST + 15 barriers (< 256 bytes)
  float (*s_hmax)[2][NC] = reinterpret_cast<float (*)[2][NC]>(small + 256);   // [block parity][half][row] half-row maxima
  uint32_t* tmem_slot_p = reinterpret_cast<uint32_t*>(small + 256 + 4 * NC * 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(small + 256 + 4 * NC * 4 + 8);

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
  auto pair_bar = [&](int q) { return bar(NB + 11 + q); };   // the two compute warps of lane quadrant q meet here

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
      ptx::mbar_init(sfree_bar(b), 8);   // one arrival per compute warp
      ptx::mbar_init(qfull_bar(b), 1);
      ptx::mbar_init(qfree_bar(b), 1);
    }
    for (int q = 0; q < 4; ++q) ptx::mbar_init(pair_bar(q), 2);
    ptx::mbar_init(pready_bar, 8);       // compute warps
    ptx::mbar_init(ofull_bar, 1);
    ptx::mbar_init(ofree_bar, 8);
    ptx::fence_barrier_init();
    ptx::prefetch_tensormap(&tm_k);
    ptx::prefetch_tensormap(&tm_v);
    if (p.q_tma) ptx::prefetch_tensormap(&tm_q);
    if (p.o_tma) ptx::prefetch_tensormap(&tm_out);
  }
  if (warp == 1) {
    ptx::tmem_alloc(ptx::smem_u32(tmem_slot_p), TMEM_COLS);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem_base = *tmem_slot_p;
  const uint32_t tm_s0 = tmem_base, tm_o = tmem_base + 2 * ATC_BN;
  pdl_trigger();
  pdl_wait();

  if (warp == 0 || warp == 2) {
    // ------------------------------------------------------------------ TMA producers (whole warps):
    // warp 0 streams K blocks, warp 2 V blocks, each through its own ring, one block ahead and across
    // tile boundaries (same scheme as attn_tc.cuh).
    const bool is_k = warp == 0;
    const int nst = is_k ? KST : VST, halves = is_k ? KH : VH;
    const uint32_t blk_bytes = is_k ? K_BYTES : V_BYTES;
    const uint32_t ring = is_k ? base : v_ring;
    const CUtensorMap* tm = is_k ? &tm_k : &tm_v;
    const int boxes = ATC_BN / p.box_tokens;
    uint32_t g = 0;
    bool ok = true;
    for (int lin = blockIdx.x; lin < p.tc_slots && ok; lin += (int)gridDim.x) {
      AtcTile t;
      atc_tile<NC>(p, lin, t);
      if (!t.valid) continue;
      const int* ptab = p.page_table + (long long)t.seq * p.page_table_stride;
      const int valid_pages = (t.kv_len + p.page_size - 1) / p.page_size;
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
          w = ptx::mbar_wait(is_k ? kempty_bar(s) : vempty_bar(s), ((g / nst) & 1) ^ 1, abort_flag, 700 + s);
        ok = __all_sync(0xffffffffu, w);
        if (!ok) break;
        const uint32_t dst = ring + (uint32_t)s * blk_bytes;
        ATR_STAMP(3, g, is_k ? 0 : 2);   // ring slot free seen
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
      const uint32_t idesc_s = umma_idesc_bf16_b(ATC_BN, false), idesc_o = umma_idesc_bf16_b(DV, true);
      const uint64_t hi_k = ptx::umma_desc_k_sw128(0) & 0xFFFFFFFF00000000ull;
      auto kdesc = [&](uint32_t addr) { return hi_k | (uint64_t)(((addr & 0x3FFFFu) >> 4) | (1u << 16)); };
      AtcTile t;
      int lin = atc_next_tile<NC>(p, blockIdx.x, t);   // tile of the next QK^T to issue
      uint32_t gs = 0, gp = 0, tile_it = 0;             // next QK^T block, next PV block, tile counter
      int j = 0;
      auto issue_next_s = [&]() {   // S of global block gs into S buffer gs & 1
        const int qb = tile_it & 1;
        if (j == 0 && !ptx::mbar_wait(qfull_bar(qb), (tile_it >> 1) & 1, abort_flag, 705 + qb)) return false;
        const int s = gs % KST, b = gs & 1;
        if (!ptx::mbar_wait(kfull_bar(s), (gs / KST) & 1, abort_flag, 710 + s)) return false;
        if (!ptx::mbar_wait(sfree_bar(b), ((gs >> 1) & 1) ^ 1, abort_flag, 720 + b)) return false;
        ptx::tc_fence_after();
        const uint32_t sk = base + (uint32_t)s * K_BYTES, qs = q_smem + qb * Q_BYTES;
#pragma unroll
        for (int kk = 0; kk < DK / 16; ++kk) {
          const uint64_t da = kdesc(qs + (kk >> 2) * (NC * 128) + (kk & 3) * 32);       // A = Q rows
          const uint64_t db = kdesc(sk + (kk >> 2) * (ATC_BN * 128) + (kk & 3) * 32);   // B = keys
          ptx::umma_bf16(tm_s0 + b * ATC_BN, da, db, idesc_s, kk != 0 ? 1u : 0u);
        }
        ptx::umma_commit(sfull_bar(b));
        ptx::umma_commit(kempty_bar(s));
        ATR_STAMP(0, gs, 0);   // QK issued
        ++gs;
        if (++j == t.nblk) {
          ptx::umma_commit(qfree_bar(qb));
          j = 0;
          ++tile_it;
          lin = atc_next_tile<NC>(p, lin + (int)gridDim.x, t);
        }
        return true;
      };
      bool ok = lin >= 0 && issue_next_s();
      while (ok && gp < gs) {
        if (lin >= 0 && !issue_next_s()) break;
        const uint32_t g = gp;
        const int s = g % VST;
        if (!ptx::mbar_wait(pready_bar, g & 1, abort_flag, 730)) break;
        ATR_STAMP(0, g, 1);    // P ready seen
        if (!ptx::mbar_wait(ofree_bar, (g & 1) ^ 1, abort_flag, 731)) break;
        ATR_STAMP(0, g, 2);    // O free seen
        if (!ptx::mbar_wait(vfull_bar(s), (g / VST) & 1, abort_flag, 715 + s)) break;
        ATR_STAMP(0, g, 3);    // V full seen
        ptx::tc_fence_after();
        const uint32_t sv = v_ring + (uint32_t)s * V_BYTES;
#pragma unroll
        for (int kk = 0; kk < ATC_BN / 16; ++kk) {
          const uint64_t da = kdesc(p_smem + (kk >> 2) * (NC * 128) + (kk & 3) * 32);    // A = P rows, K = keys
          // B = V as it lies: 16 keys per step are 16 rows of 128 B; the other 64-wide d half is ATC_BN*128 B on
          const uint64_t db = umma_desc_mn_sw128(sv + kk * 16 * 128, ATC_BN * 128);
          ptx::umma_bf16(tm_o, da, db, idesc_o, kk != 0 ? 1u : 0u);
        }
        ptx::umma_commit(ofull_bar);
        ptx::umma_commit(vempty_bar(s));
        ATR_STAMP(0, g, 4);    // PV issued
        ++gp;
      }
    }
  } else if (warp == 3) {
    // ------------------------------------------------------------------ Q loader (whole warp), one tile ahead
    AtcTile t;
    uint32_t tile_it = 0;
    for (int lin = atc_next_tile<NC>(p, blockIdx.x, t); lin >= 0;
         lin = atc_next_tile<NC>(p, lin + (int)gridDim.x, t), ++tile_it) {
      const int qb = tile_it & 1;
      bool w = true;
      if (lane == 0) w = ptx::mbar_wait(qfree_bar(qb), ((tile_it >> 1) & 1) ^ 1, abort_flag, 760 + qb);
      if (!__all_sync(0xffffffffu, w)) break;
      uint8_t* qd = q_ptr + qb * Q_BYTES;
      if (p.q_tma) {
        // One box per 64-dim half: {64 dims, heads of this KV head's chunk, positions of the tile}; its rows
        // arrive in (position, head) order, 128 bytes each, swizzled, i.e. as the tile's rows.  Positions past
        // the last query token read as zeros; positions past this sequence's queries are other sequences'
        // rows, whose results are never stored.
        if (lane == 0) {
          const int rows = t.heads_here * t.pos_per_tile;
          ptx::mbar_expect_tx(qfull_bar(qb), (uint32_t)(rows * 128 * (DK / 64)));
#pragma unroll
          for (int h = 0; h < DK / 64; ++h)
            ptx::tma_load_3d(q_smem + qb * Q_BYTES + h * (NC * 128), &tm_q, qfull_bar(qb), h * 64,
                             t.kvh * p.group + t.hchunk * 8, t.q_start + t.tile_pos0, ptx::kEvictLast);
        }
        __syncwarp();
        continue;
      }
#pragma unroll 8
      for (int i = lane; i < NC * (DK / 8); i += 32) {
        const int c = i / (DK / 8), ch = i % (DK / 8);   // row, 16-byte chunk of its head vector
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
    // ------------------------------------------------------------------ compute (warps 4..11)
    // Thread = (row, half): TMEM lane `row` for keys [64 half, 64 half + 64) of every block and for value
    // dims [64 half, 64 half + 64) of O.  The two threads of a row (warps w and w + 4 of a lane quadrant)
    // meet once per block to join their half-row maxima.  Per block:
    //   S half row -> registers, v = s * scale (+ causal mask), half-row maximum      (one TMEM round trip)
    //   join maxima with the partner -> m, alpha
    //   fold the previous block's O into o: o = (o + O_prev) * alpha                  (frees O for the next PV)
    //   p = bf16(2^(v - m)) -> P tile; two 32-key group sums in butterfly order, l_g = l_g * alpha + s_g
    constexpr float kMinMax = -3.0e38f;   // floor of the running maximum (as in attn_tc.cuh)
    const int q4 = warp & 3, half = (warp - 4) >> 2;
    const int row = q4 * 32 + lane;
    const uint32_t lane_addr = (uint32_t)(q4 * 32) << 16;
    const uint32_t o_addr = tm_o + lane_addr + half * 64;
    uint8_t* p_half = p_ptr + half * (NC * 128);   // my 64 keys are one 64-key half of the P tile
    uint32_t g0 = 0, pair_phase = 0;
    // Meeting point of a row's two threads: a bounded mbarrier wait like every other wait here (a bar.sync
    // would strand one warp if its partner left on an abort).
    auto pair_sync = [&]() {
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(pair_bar(q4));
      const bool ok = ptx::mbar_wait_warp(pair_bar(q4), pair_phase & 1, abort_flag, 780 + q4);
      ++pair_phase;
      return ok;
    };
    AtcTile t, tn;
    bool alive = true;
    bool store_pending = false;   // an asynchronous output store of this warp still reads its slice of the P tile
    int lin = atc_next_tile<NC>(p, blockIdx.x, t);
    while (lin >= 0 && alive) {
      // the next tile's description is requested now (loads only) so that it is at hand when this tile ends
      const int cand = lin + (int)gridDim.x;
      const bool have_cand = cand < p.tc_slots;
      AtcRaw raw_next = {0, 0, 0, 0, -1};
      if (have_cand) raw_next = atc_raw(p, cand);
      const int npos = min(t.pos_per_tile, t.q_len - t.tile_pos0);
      const int pi = row / t.heads_here, hd = row - pi * t.heads_here;
      const int cpos = t.q_abs0 + t.tile_pos0 + (pi < npos ? pi : 0);   // padding rows borrow position 0's mask
      float m_run = -INFINITY, l_a = 0.f, l_b = 0.f;   // l of my two key groups (2 half, 2 half + 1)
      float o[64];
#pragma unroll
      for (int i = 0; i < 64; ++i) o[i] = 0.f;
      for (int j = 0; j < t.nblk; ++j) {
        const uint32_t g = g0 + j;
        const int b = g & 1, s = g % VST;
        const int key0 = j * ATC_BN + half * 64;          // first key of my half of the block
        const bool masked = key0 + 63 > cpos;
        if (!ptx::mbar_wait_warp(sfull_bar(b), (g >> 1) & 1, abort_flag, 740 + b)) {
          alive = false;
          break;
        }
        ptx::tc_fence_after();
        if (warp == 4) ATR_STAMP(1, g, 0);   // S full seen
        if (store_pending) {   // (uniform over the warp) the previous tile's output has left shared memory by now
          if (lane == 0) ptx::bulk_wait_read0();
          __syncwarp();
          store_pending = false;
        }
        float v[64];
        {
          uint32_t r0[32], r1[32];
          tmem_ld32(tm_s0 + b * ATC_BN + lane_addr + half * 64, r0);
          tmem_ld32(tm_s0 + b * ATC_BN + lane_addr + half * 64 + 32, r1);
          ptx::tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            v[i] = __uint_as_float(r0[i]) * p.qk_scale;
            v[32 + i] = __uint_as_float(r1[i]) * p.qk_scale;
          }
        }
        if (masked) {
#pragma unroll
          for (int i = 0; i < 64; ++i)
            if (key0 + i > cpos) v[i] = -INFINITY;
        }
        float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
        for (int i = 0; i < 64; ++i) mx4[i & 3] = fmaxf(mx4[i & 3], v[i]);
        const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
        s_hmax[b][half][row] = mx;
        if (!pair_sync()) {
          alive = false;
          break;
        }
        const float m_new = fmaxf(fmaxf(m_run, kMinMax), fmaxf(mx, s_hmax[b][half ^ 1][row]));
        const float alpha = fast_exp2(m_run - m_new);
        m_run = m_new;
        if (warp == 4) ATR_STAMP(1, g, 1);   // maxima joined
        // fold the previous block's O (its PV product has also finished reading the P tile by then)
        if (j > 0) {
          if (!ptx::mbar_wait_warp(ofull_bar, (g - 1) & 1, abort_flag, 750)) {
            alive = false;
            break;
          }
          ptx::tc_fence_after();
#pragma unroll
          for (int c = 0; c < 2; ++c) {   // two 16-column loads in flight per wait
            uint32_t r0[16], r1[16];
            ptx::tmem_ld16(o_addr + c * 32, r0);
            ptx::tmem_ld16(o_addr + c * 32 + 16, r1);
            ptx::tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              o[c * 32 + i] = (o[c * 32 + i] + __uint_as_float(r0[i])) * alpha;
              o[c * 32 + 16 + i] = (o[c * 32 + 16 + i] + __uint_as_float(r1[i])) * alpha;
            }
          }
          ptx::tc_fence_before();
          __syncwarp();
          if (lane == 0) ptx::mbar_arrive(ofree_bar);
        }
        if (warp == 4) ATR_STAMP(1, g, 2);   // folded
        // p = bf16(2^(v - m)), group sums in butterfly order, P half row -> shared memory
        float sa, sb;
        {
          float pf[32];
          uint32_t pk[16];
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            const __nv_bfloat162 b2 = __floats2bfloat162_rn(fast_exp2(v[i] - m_new), fast_exp2(v[i + 1] - m_new));
            pf[i] = __low2float(b2);
            pf[i + 1] = __high2float(b2);
            pk[i >> 1] = *reinterpret_cast<const uint32_t*>(&b2);
          }
          sa = butterfly_order_sum32(pf);
#pragma unroll
          for (int q = 0; q < 4; ++q)
            *reinterpret_cast<uint4*>(p_half + sw128(row, q)) = make_uint4(pk[q * 4], pk[q * 4 + 1], pk[q * 4 + 2], pk[q * 4 + 3]);
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            const __nv_bfloat162 b2 =
                __floats2bfloat162_rn(fast_exp2(v[32 + i] - m_new), fast_exp2(v[32 + i + 1] - m_new));
            pf[i] = __low2float(b2);
            pf[i + 1] = __high2float(b2);
            pk[i >> 1] = *reinterpret_cast<const uint32_t*>(&b2);
          }
          sb = butterfly_order_sum32(pf);
#pragma unroll
          for (int q = 0; q < 4; ++q)
            *reinterpret_cast<uint4*>(p_half + sw128(row, 4 + q)) = make_uint4(pk[q * 4], pk[q * 4 + 1], pk[q * 4 + 2], pk[q * 4 + 3]);
        }
        l_a = l_a * alpha + sa;
        l_b = l_b * alpha + sb;
        // keys at or beyond kv_len may hold anything: clear their V rows so that 0 * V stays 0
        if (j * ATC_BN + ATC_BN > t.kv_len) {
          if (!ptx::mbar_wait_warp(vfull_bar(s), (g / VST) & 1, abort_flag, 745)) {
            alive = false;
            break;
          }
          uint8_t* vt = base_ptr + (size_t)KST * K_BYTES + (size_t)s * V_BYTES;
          for (int r = t.kv_len - j * ATC_BN + (warp - 4); r < ATC_BN; r += 8)
#pragma unroll
            for (int h = 0; h < VH; ++h) reinterpret_cast<uint32_t*>(vt + h * (ATC_BN * 128) + r * 128)[lane] = 0u;
        }
        ptx::tc_fence_before();
        ptx::fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
          ptx::mbar_arrive(sfree_bar(b));
          ptx::mbar_arrive(pready_bar);
        }
        if (warp == 4) ATR_STAMP(1, g, 3);   // P published
      }
      if (!alive) break;
      // tile end: the last block's O, the row sum, the store
      if (!ptx::mbar_wait_warp(ofull_bar, (g0 + t.nblk - 1) & 1, abort_flag, 751)) break;
      ptx::tc_fence_after();
      if (warp == 4) ATR_STAMP(2, g0 + t.nblk - 1, 0);   // last O complete
      {
        uint32_t r0[32], r1[32];
        tmem_ld32(o_addr, r0);
        tmem_ld32(o_addr + 32, r1);
        ptx::tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          o[i] += __uint_as_float(r0[i]);
          o[32 + i] += __uint_as_float(r1[i]);
        }
      }
      ptx::tc_fence_before();
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(ofree_bar);
      if (warp == 4) ATR_STAMP(2, g0 + t.nblk - 1, 1);   // O read
      // The half-row sums meet in the maxima buffer of the tile's last block: both threads of every row read
      // it before that block's P was published, and the next tile's first block uses the other buffer.
      float (*s_lh)[NC] = s_hmax[(g0 + t.nblk - 1) & 1];
      s_lh[half][row] = l_a + l_b;             // (l_0 + l_1) from half 0, (l_2 + l_3) from half 1
      if (!pair_sync()) break;
      if (warp == 4) ATR_STAMP(2, g0 + t.nblk - 1, 2);   // row sums joined
      {
        // Output.  A thread holds 64 value dims of one row (128 bytes); stored from there, one warp instruction
        // would touch 32 rows' lines with 16 bytes each.  The warp first lays its 32 half rows down in its own
        // 4 KB of the P tile (idle from the tile's last PV product until this warp's next P write; swizzled), then eight
        // lanes store one row's 128 bytes, four rows per instruction.
        const float inv = 1.0f / (s_lh[0][row] + s_lh[1][row]);
        const float inv_heads = 1.0f / (float)t.heads_here;
        const bool vec = ((reinterpret_cast<uintptr_t>(p.out) | (uintptr_t)(p.o_tok_stride * 2) |
                           (uintptr_t)(p.o_head_stride * 2)) & 15) == 0;
        if (vec) {
#pragma unroll
          for (int q = 0; q < 8; ++q)   // 128-byte rows, 16-byte chunks swizzled by row: no bank conflicts
            *reinterpret_cast<uint4*>(p_half + sw128(row, q)) = make_uint4(pack_bf2(o[q * 8] * inv, o[q * 8 + 1] * inv), pack_bf2(o[q * 8 + 2] * inv, o[q * 8 + 3] * inv),
                                 pack_bf2(o[q * 8 + 4] * inv, o[q * 8 + 5] * inv), pack_bf2(o[q * 8 + 6] * inv, o[q * 8 + 7] * inv));
          const int ppw = 32 / t.heads_here;   // whole positions in this warp's 32 rows (if heads divide 32)
          if (p.o_tma && ppw * t.heads_here == 32 && (q4 + 1) * ppw <= npos) {
            // every row of the warp is a real query: one asynchronous store of the warp's box
            ptx::fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) {
              ptx::tma_store_3d(&tm_out, ptx::smem_u32(p_half + q4 * 32 * 128), half * 64,
                                t.kvh * p.group + t.hchunk * 8, t.q_start + t.tile_pos0 + q4 * ppw);
              ptx::bulk_commit();
            }
            store_pending = true;
          } else {
          __syncwarp();
#pragma unroll
          for (int it = 0; it < 8; ++it) {
            const int r = q4 * 32 + it * 4 + (lane >> 3);          // tile row whose chunk (lane & 7) I store
            // r / heads_here without an integer division: exact for r < 128 and at most 8 heads
            const int rpi = (int)(((float)r + 0.5f) * inv_heads), rhd = r - rpi * t.heads_here;
            if (rpi < npos) {
              const uint4 v = *reinterpret_cast<const uint4*>(p_half + sw128(r, lane & 7));
              __nv_bfloat16* orow = p.out + (long long)(t.q_start + t.tile_pos0 + rpi) * p.o_tok_stride +
                                    (long long)(t.kvh * p.group + t.hchunk * 8 + rhd) * p.o_head_stride + half * 64;
              reinterpret_cast<uint4*>(orow)[lane & 7] = v;
            }
          }
          __syncwarp();
          }
        } else if (pi < npos) {
          __nv_bfloat16* orow = p.out + (long long)(t.q_start + t.tile_pos0 + pi) * p.o_tok_stride +
                                (long long)(t.kvh * p.group + t.hchunk * 8 + hd) * p.o_head_stride + half * 64;
#pragma unroll
          for (int i = 0; i < 64; ++i) orow[i] = f2bf(o[i] * inv);
        }
      }
      if (warp == 4) ATR_STAMP(2, g0 + t.nblk - 1, 3);   // tile stored
      g0 += t.nblk;
      lin = -1;
      if (have_cand) {
        atc_make<NC>(p, cand, raw_next, tn);
        lin = tn.valid ? cand : atc_next_tile<NC>(p, cand + (int)gridDim.x, tn);
      }
      t = tn;
    }
    if (lane == 0) ptx::bulk_wait0();   // this warp's output stores are complete before the CTA may leave
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

template <int DK>
inline int attn_rows_launch(const CUtensorMap& tk, const CUtensorMap& tv, const CUtensorMap& tq, const CUtensorMap& to,
                            const AttnParams& p, cudaStream_t st) {
  // tiles (K ring, V ring, two Q buffers, P) + small arrays (barriers, alpha, l, TMEM slot, abort flag) + alignment
  constexpr int tiles = ATC_BN * (2 * DK + 2 * 128) * 2 + 2 * (DK / 64) * ATR_ROWS * 128 + 2 * ATR_ROWS * 128;
  constexpr int small = 256 + 4 * ATR_ROWS * 4 + 16;
  constexpr int smem = (tiles + small + 1023 <= 227 * 1024) ? tiles + small + 1023 : 227 * 1024;
  static_assert(tiles + small <= 227 * 1024, "shared memory budget");
  static PerDeviceFlags attr_set;
  if (int rc = set_max_dyn_smem_once(attr_set, paged_attn_rows_kernel<DK>, smem)) return rc;
  const int nctas = p.tc_tiles < sm_count() ? p.tc_tiles : sm_count();
  launch_k(paged_attn_rows_kernel<DK>, dim3((unsigned)nctas), dim3(ATR_THREADS), (size_t)smem, st, tk, tv, tq, to, p);
  return launch_status();
}

inline int attn_rows_dispatch(const CUtensorMap& tk, const CUtensorMap& tv, const CUtensorMap& tq, const CUtensorMap& to,
                              const AttnParams& p, cudaStream_t st) {
  return attn_rows_launch<128>(tk, tv, tq, to, p, st);
}

}  // namespace b200

#ifdef B200_ATTN_TRACE
extern "C" int b200_debug_read_trace(long long* host_out /* [4][64][8] */) {
  return cudaMemcpyFromSymbol(host_out, b200::g_attn_trace, sizeof(long long) * 4 * 64 * 8) == cudaSuccess ? 0 : -3;
}
#endif
