// One scheduler step's input buffers, built on the device from per-request counters.
//
// Replaces the per-token host loops of the reference's Inferencer._prepare_gen_ctx
// (vexact/inferencer/inferencer.py:193-291: slot mapping, context lens, block tables,
// query_start_loc, input / position ids) and the fills and copies of
// _prepare_input_buffers_from_gen_ctx (:293-349) that pad them to the captured graph's shape.
// All of it is integer work and bit-exact.
//
// One launch: every CTA rebuilds the (short) prefix sum of tokens_this_step in shared memory,
// then the grid strides over the padded token range (a token finds its request by binary search
// in the prefix sums) and over the padded block-table rows; CTA 0 writes the per-request arrays.
#pragma once
#include "common.cuh"

namespace b200 {

constexpr int STEP_MAX_SEQS = 8192;
constexpr int STEP_THREADS = 256;

struct StepParams {
  const int* num_computed;     // [num_seqs]
  const int* tokens_this_step; // [num_seqs]
  const int* block_tables_in;  // [num_seqs, max_blocks]
  const long long* prefill_ids;
  const int* prefill_offset;   // [num_seqs], -1 = decode
  const long long* last_tokens;
  int num_seqs, graph_num_seqs, capture_tokens, max_blocks, page_size;
  long long* input_ids;
  long long* position_ids;
  int* slot_mapping;
  int* context_lens;
  int* query_start_loc;
  int* block_tables_out;
  int* step_info;
};

__global__ void __launch_bounds__(STEP_THREADS) prepare_step_kernel(const StepParams p) {
  pdl_trigger();
  pdl_wait();
  extern __shared__ int s_qsl[];  // [num_seqs + 1] exclusive prefix sums of tokens_this_step
  __shared__ int s_part[STEP_THREADS];
  __shared__ int s_max[STEP_THREADS];
  const int tid = threadIdx.x;
  // prefix sum: each thread owns a contiguous slice of the requests
  const int per = (p.num_seqs + STEP_THREADS - 1) / STEP_THREADS;
  const int lo = min(tid * per, p.num_seqs), hi = min(lo + per, p.num_seqs);
  int sum = 0, mx = 0;
  for (int i = lo; i < hi; ++i) {
    const int n = p.tokens_this_step[i];
    sum += n;
    mx = max(mx, n);
  }
  s_part[tid] = sum;
  s_max[tid] = mx;
  __syncthreads();
  for (int off = 1; off < STEP_THREADS; off <<= 1) {  // inclusive scan of the slice sums
    const int v = tid >= off ? s_part[tid - off] : 0;
    const int m = tid >= off ? s_max[tid - off] : 0;
    __syncthreads();
    s_part[tid] += v;
    s_max[tid] = max(s_max[tid], m);
    __syncthreads();
  }
  int run = tid > 0 ? s_part[tid - 1] : 0;
  for (int i = lo; i < hi; ++i) {
    s_qsl[i] = run;
    run += p.tokens_this_step[i];
  }
  const int total = s_part[STEP_THREADS - 1];
  if (tid == 0) s_qsl[p.num_seqs] = total;
  __syncthreads();

  if (blockIdx.x == 0) {  // per-request arrays, padded request rows
    for (int i = tid; i < p.graph_num_seqs; i += STEP_THREADS) p.context_lens[i] = i < p.num_seqs ? p.num_computed[i] : 0;
    for (int i = tid; i <= p.graph_num_seqs; i += STEP_THREADS) p.query_start_loc[i] = i <= p.num_seqs ? s_qsl[i] : total;
    if (tid == 0) {
      p.step_info[0] = total;
      p.step_info[1] = s_max[STEP_THREADS - 1];
      if (total > p.capture_tokens) report_status(B200_STATUS_BAD_INDEX, total);
    }
  }

  const int stride = gridDim.x * STEP_THREADS;
  const int first = blockIdx.x * STEP_THREADS + tid;
  // token-level buffers
  for (int t = first; t < p.capture_tokens; t += stride) {
    int slot = -1;
    long long id = 0, pos = 0;
    if (t < total) {
      int a = 0, b = p.num_seqs;  // last request with s_qsl[i] <= t (zero-length requests are skipped)
      while (b - a > 1) {
        const int mid = (a + b) >> 1;
        if (s_qsl[mid] <= t) a = mid; else b = mid;
      }
      const int k = t - s_qsl[a];
      const int n = s_qsl[a + 1] - s_qsl[a];
      const int start = p.num_computed[a] - n;
      pos = start + k;
      const int blk = (int)(pos / p.page_size);
      const int block_id = blk < p.max_blocks ? p.block_tables_in[(long long)a * p.max_blocks + blk] : -1;
      if (start < 0 || block_id < 0) {
        report_status(B200_STATUS_BAD_INDEX, a);
      } else {
        slot = block_id * p.page_size + (int)(pos - (long long)blk * p.page_size);
      }
      const int off = p.prefill_offset ? p.prefill_offset[a] : -1;
      id = off >= 0 ? p.prefill_ids[off + k] : (p.last_tokens ? p.last_tokens[a] : 0);
    }
    p.slot_mapping[t] = slot;
    p.input_ids[t] = id;
    p.position_ids[t] = pos;
  }
  // block tables: the requests' rows, then zero rows up to the captured request count
  const long long cells = (long long)p.graph_num_seqs * p.max_blocks;
  const long long live = (long long)p.num_seqs * p.max_blocks;
  for (long long e = first; e < cells; e += stride) p.block_tables_out[e] = e < live ? p.block_tables_in[e] : 0;
}

}  // namespace b200

extern "C" int b200_prepare_step(const int* num_computed_tokens, const int* tokens_this_step, const int* block_tables_in,
                                 const long long* prefill_ids, const int* prefill_offset, const long long* last_tokens,
                                 int num_seqs, int graph_num_seqs, int capture_tokens, int max_blocks, int page_size,
                                 long long* input_ids, long long* position_ids, int* slot_mapping, int* context_lens,
                                 int* query_start_loc, int* block_tables_out, int* step_info, void* stream) {
  using namespace b200;
  if (!num_computed_tokens || !tokens_this_step || !block_tables_in || !input_ids || !position_ids || !slot_mapping ||
      !context_lens || !query_start_loc || !block_tables_out || !step_info)
    return B200_ERR_ARG;
  if (num_seqs < 0 || graph_num_seqs < num_seqs || capture_tokens < 0 || max_blocks <= 0 || page_size <= 0)
    return B200_ERR_ARG;
  if (num_seqs > STEP_MAX_SEQS) return B200_ERR_SHAPE;
  if (prefill_offset && !prefill_ids) return B200_ERR_ARG;
  StepParams p{num_computed_tokens, tokens_this_step, block_tables_in, prefill_ids, prefill_offset, last_tokens,
               num_seqs, graph_num_seqs, capture_tokens, max_blocks, page_size, input_ids, position_ids, slot_mapping,
               context_lens, query_start_loc, block_tables_out, step_info};
  const long long work = (long long)graph_num_seqs * max_blocks > capture_tokens ? (long long)graph_num_seqs * max_blocks
                                                                                  : capture_tokens;
  long long ctas = (work + STEP_THREADS * 4 - 1) / (STEP_THREADS * 4);
  if (ctas < 1) ctas = 1;
  if (ctas > 4 * sm_count()) ctas = 4 * sm_count();
  launch_k(prepare_step_kernel, dim3((unsigned)ctas), dim3(STEP_THREADS), (size_t)(num_seqs + 1) * sizeof(int),
           (cudaStream_t)stream, p);
  return launch_status();
}

// ------------------------------------------------------------------ row gathers of the stage runner
// Two gathers of [rows, H] bf16 rows that the reference leaves to torch indexing kernels: the embedding
// lookup (HF nn.Embedding on input_ids) and the pick of each sequence's last token before the final norm and
// lm_head (vexact/inferencer/inferencer.py:403-404: hidden[query_start_loc[1:] - 1]).
namespace b200 {

// mode 0: src row = ids[t] (int64).  mode 1: src row = max(query_start_loc[t + 1] - 1, 0) (int32 offsets).
// A row index outside [0, src_rows) is reported and reads row 0.
__global__ void __launch_bounds__(256)
gather_rows_kernel(const __nv_bfloat16* __restrict__ src, long long src_stride, long long src_rows,
                   const long long* __restrict__ ids, const int* __restrict__ query_start_loc,
                   __nv_bfloat16* __restrict__ out, int H) {
  pdl_trigger();
  pdl_wait();
  const long long t = blockIdx.x;
  long long r = ids ? ids[t] : (long long)query_start_loc[t + 1] - 1;
  if (!ids && r < 0) r = 0;   // a zero-length (padding) sequence: any row will do, its result is not used
  if (r < 0 || r >= src_rows) {
    if (threadIdx.x == 0) report_status(B200_STATUS_BAD_INDEX, (int)r);
    r = 0;
  }
  const uint4* s = reinterpret_cast<const uint4*>(src + r * src_stride);
  uint4* d = reinterpret_cast<uint4*>(out + t * (long long)H);
  for (int i = threadIdx.x; i < (H >> 3); i += 256) d[i] = s[i];
}

}  // namespace b200

// out[t, :] = src[ids[t], :] (ids int64) or, with ids == NULL, src[max(query_start_loc[t + 1] - 1, 0), :].
// src rows are src_row_stride elements apart; out is [T, H] contiguous; H a multiple of 8; 16-byte aligned rows.
extern "C" int b200_gather_rows(const void* src, long long src_rows, long long src_row_stride, const void* ids_i64,
                                const void* query_start_loc_i32, void* out, long long T, int H, void* stream) {
  using namespace b200;
  if (!src || !out || (!ids_i64 && !query_start_loc_i32) || src_rows <= 0 || T < 0 || H <= 0) return B200_ERR_ARG;
  if (H % 8 != 0 || src_row_stride % 8 != 0 || (reinterpret_cast<uintptr_t>(src) & 15) ||
      (reinterpret_cast<uintptr_t>(out) & 15))
    return B200_ERR_SHAPE;
  if (T == 0) return B200_OK;
  if (T > 0x7fffffffLL) return B200_ERR_SHAPE;
  launch_k(gather_rows_kernel, dim3((unsigned)T), dim3(256), 0, (cudaStream_t)stream, (const __nv_bfloat16*)src,
           src_row_stride, src_rows, (const long long*)ids_i64, (const int*)query_start_loc_i32, (__nv_bfloat16*)out, H);
  return launch_status();
}
