// Device-side bookkeeping of the batched greedy decode loop, so that sequences can finish -- end-of-sequence token or
// their own generation limit -- without the host touching the batch between steps.
//
// The reference's executor rebuilds the live batch on the host after every token: read the logits back, argmax, drop
// finished sequences, re-derive the per-type index lists, upload them (tvm/llama_auto_batcher/llama_exec_graph.py:
// 94-100, 102-141).  Here the batch of a fused decode node is ordered once (mlora_bucket_sort: rows without adapter
// first, then by adapter) and then only ever shrinks, so each step starts with a STABLE COMPACTION of the live
// sequences into the first rows of a fixed-size step (which keeps the adapter order) and ends with the finish test.
// A step captured in a CUDA graph for B rows serves any number of live sequences <= B: the rows beyond them are padding
// (no adapter, position -1: the attention kernel neither stores nor reads anything for them).
#include "common.cuh"

namespace mlora {
namespace {

constexpr int kStepThreads = 1024;

// One CTA.  live[b] != 0: sequence b (in the node's sorted order) still generates.
__global__ void __launch_bounds__(kStepThreads) decode_step_begin_kernel(
    const int32_t* __restrict__ live, const int32_t* __restrict__ seq_slot, const int32_t* __restrict__ adapter_slot,
    const int32_t* __restrict__ last_tok, int n_seq, int n_rows, int32_t* __restrict__ seq_lens,
    int32_t* __restrict__ row_src, int32_t* __restrict__ row_slot, int32_t* __restrict__ row_pos,
    int32_t* __restrict__ row_adapter, int32_t* __restrict__ row_tok, int32_t* __restrict__ n_live_out) {
  __shared__ int warp_cnt[kStepThreads / 32];
  __shared__ int base;
  pdl_launch_dependents();
  pdl_wait();
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  if (tid == 0) base = 0;
  __syncthreads();
  for (int b0 = 0; b0 < n_seq; b0 += kStepThreads) {
    const int b = b0 + tid;
    const bool on = b < n_seq && live[b] != 0;
    const unsigned m = __ballot_sync(0xffffffffu, on);
    if (lane == 0) warp_cnt[warp] = __popc(m);
    __syncthreads();
    int before = base;
    for (int w = 0; w < warp; ++w) before += warp_cnt[w];
    const int i = before + __popc(m & ((1u << lane) - 1));  // row of this sequence: live sequences keep their order
    if (on && i < n_rows) {
      const int s = seq_slot[b];
      const int p = seq_lens[s];
      seq_lens[s] = p + 1;  // one row per sequence: no two threads share s
      row_src[i] = b;
      row_slot[i] = s;
      row_pos[i] = p;
      row_adapter[i] = adapter_slot[b];
      row_tok[i] = last_tok[b];
    }
    __syncthreads();
    if (tid == 0) {
      int c = 0;
      for (int w = 0; w < kStepThreads / 32; ++w) c += warp_cnt[w];
      base += c;
    }
    __syncthreads();
  }
  const int n_live = base;
  for (int i = n_live + tid; i < n_rows; i += kStepThreads) {  // padding rows
    row_src[i] = -1;
    row_slot[i] = 0;
    row_pos[i] = -1;
    row_adapter[i] = -1;
    row_tok[i] = 0;
  }
  if (tid == 0) *n_live_out = n_live < n_rows ? n_live : n_rows;
}

// One thread per row: record the row's new token, then decide whether its sequence goes on.
__global__ void decode_step_end_kernel(const int32_t* __restrict__ row_src, const int32_t* __restrict__ next_tok,
                                       int n_rows, int32_t* __restrict__ live, int32_t* __restrict__ last_tok,
                                       int32_t* __restrict__ gen_count, const int32_t* __restrict__ max_gen,
                                       int32_t* __restrict__ out_tokens, int64_t ld_out, int32_t eos_id,
                                       int32_t* __restrict__ n_live_io) {
  pdl_launch_dependents();
  pdl_wait();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n_rows) return;
  const int b = row_src[i];
  if (b < 0) return;
  const int tok = next_tok[i];
  const int n = gen_count[b];
  if (n < ld_out) out_tokens[(size_t)b * ld_out + n] = tok;
  gen_count[b] = n + 1;
  last_tok[b] = tok;
  if (tok == eos_id || n + 1 >= max_gen[b] || n + 1 >= ld_out) {
    live[b] = 0;
    atomicSub(n_live_io, 1);
  }
}

}  // namespace
}  // namespace mlora

using namespace mlora;

extern "C" int mlora_decode_step_begin(const int32_t* d_live, const int32_t* d_seq_slot, const int32_t* d_adapter_slot,
                                       const int32_t* d_last_tok, int32_t n_seq, int32_t n_rows, int32_t* d_seq_lens,
                                       int32_t* d_row_src, int32_t* d_row_slot, int32_t* d_row_pos,
                                       int32_t* d_row_adapter, int32_t* d_row_tok, int32_t* d_n_live, void* stream) {
  MLORA_REQUIRE(n_seq >= 0 && n_rows >= 0, "decode_step_begin: bad sizes n_seq=%d n_rows=%d", n_seq, n_rows);
  MLORA_REQUIRE(d_live && d_seq_slot && d_adapter_slot && d_last_tok && d_seq_lens && d_row_src && d_row_slot &&
                    d_row_pos && d_row_adapter && d_row_tok && d_n_live,
                "decode_step_begin: null pointer");
  if (n_rows == 0) return MLORA_OK;
  launch_pdl(decode_step_begin_kernel, 1, kStepThreads, 0, (cudaStream_t)stream, d_live, d_seq_slot, d_adapter_slot,
             d_last_tok, n_seq, n_rows, d_seq_lens, d_row_src, d_row_slot, d_row_pos, d_row_adapter, d_row_tok, d_n_live);
  count_launch();
  MLORA_CHECK_LAUNCH("decode_step_begin_kernel");
  return MLORA_OK;
}

extern "C" int mlora_decode_step_end(const int32_t* d_row_src, const int32_t* d_next_tok, int32_t n_rows, int32_t* d_live,
                                     int32_t* d_last_tok, int32_t* d_gen_count, const int32_t* d_max_gen,
                                     int32_t* d_out_tokens, int64_t ld_out, int32_t eos_id, int32_t* d_n_live,
                                     void* stream) {
  MLORA_REQUIRE(n_rows >= 0 && ld_out > 0, "decode_step_end: bad sizes n_rows=%d ld_out=%lld", n_rows, (long long)ld_out);
  MLORA_REQUIRE(d_row_src && d_next_tok && d_live && d_last_tok && d_gen_count && d_max_gen && d_out_tokens && d_n_live,
                "decode_step_end: null pointer");
  if (n_rows == 0) return MLORA_OK;
  launch_pdl(decode_step_end_kernel, (n_rows + 127) / 128, 128, 0, (cudaStream_t)stream, d_row_src, d_next_tok, n_rows,
             d_live, d_last_tok, d_gen_count, d_max_gen, d_out_tokens, ld_out, eos_id, d_n_live);
  count_launch();
  MLORA_CHECK_LAUNCH("decode_step_end_kernel");
  return MLORA_OK;
}
