/* libmlora: C ABI of the B200 (sm_100a) multi-LoRA decode path.
 *
 * Every pointer named `d_*` or documented as "device" is a CUDA device pointer
 * owned by the caller; nothing is allocated or freed by the library.  Every
 * call is asynchronous on `stream` (a cudaStream_t passed as void*), returns
 * 0 on success and a negative MLORA_E* code when the arguments are rejected
 * on the host (mlora_last_error() then holds a message).  bf16 tensors are
 * row-major with 16-byte aligned rows.  Process-wide state is limited to: a launch counter, the
 * thread-local message behind mlora_last_error(), per-device "attribute already set" marks of the
 * kernels, and the 16 MiB device array of mlora_paged_attention_static (documented there).
 *
 * The citations name the interface of the reference project
 * (llm-db/tensor-program-optimization-with-auto-batching) that each entry
 * point stands in for, by path inside that project.
 */
#ifndef MLORA_H_
#define MLORA_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define MLORA_OK 0
#define MLORA_EINVAL (-1) /* argument rejected on the host */
#define MLORA_ECUDA (-2)  /* a CUDA runtime call or launch failed */
#define MLORA_ESIZE (-3)  /* workspace too small / size beyond a stated limit */

/* flags of mlora_linear */
#define MLORA_OUT_F32 1     /* y is float32 (lm_head logits) instead of bf16 */
#define MLORA_SILU_MUL 2    /* W holds gate/up rows interleaved in blocks of 8 (rows 16j..16j+7 = gate
                               rows 8j.., rows 16j+8..16j+15 = up rows 8j..); y[t, c] = silu(g)*u, y has
                               out/2 columns */
#define MLORA_FORCE_SIMT 4  /* use the CUDA-core warp-per-row kernel whatever the shape */
#define MLORA_W_PACKED 8    /* d_W is the tiled layout written by mlora_pack_weight */
#define MLORA_B_PACKED 16   /* d_B_all is the tiled layout written by mlora_pack_lora_b */
#define MLORA_LORA_PER_ROW 64 /* the batch has many distinct adapters per token tile (e.g. every request its own):
                               run the base projection, then add the expand with a kernel laid out by (row, output
                               feature) that streams each row's B_all[slot] up to the adapter's own rank, instead of
                               one masked tensor-core stage per distinct adapter.  bf16 outputs are rounded twice
                               (projection, then sum).  With MLORA_SILU_MUL the projection leaves fp32 pre-activations
                               of the gate / up rows in the tail of d_work, and the expand kernel adds the adapters and
                               applies silu(gate)*up: d_work must then hold mlora_linear_workspace_flags(T, in, out,
                               flags) bytes (the flag is ignored, i.e. the tensor-core stages run, when it holds less) */
#define MLORA_B_SPLIT 128   /* with MLORA_LORA_PER_ROW: d_B_all is the rank-compact "split" layout -- every adapter stored
                               as rank/8 slices [out, 8] bf16 laid one after the other (the split-to-the-minimum-rank
                               strategy of tvm/lora_only/case_study/multiple_ranks.py:98-151 as a data layout: slices of
                               one adapter are summed) -- and d_ranks holds 2*n_adapters ints: the ranks (multiples of
                               8), then the index of each adapter's first slice.  The expand then reads exactly
                               rank * out * 2 bytes per row, in whole 16-byte units per output feature, whatever the
                               widest rank of the stack is */
#define MLORA_SHARE_LORA_KERNEL 32 /* hint for a call WITHOUT LoRA operands that sits between calls with them
                               (gate/up/down when only q/k/v/o carry adapters): run the kernel variant the LoRA
                               calls use, so one code footprint stays hot in the instruction caches for the whole
                               step; results are identical either way */

int mlora_version(void);
const char* mlora_last_error(void);
/* Number of kernels this library has launched in this process (for benchmarks' launch counts). */
uint64_t mlora_launch_count(void);

/* ---- (d) request -> adapter bucketing --------------------------------------------------------
 * Stable counting sort of n rows by key (has_adapter, tid, wid), rows without adapter
 * (tid < 0) first.  Replaces LlamaSeqInfo.order_seqs and the per-type position / weight-id
 * lists of LlamaSeqInfo.get_decode_method (tvm/llama_auto_batcher/llama_seq_info.py:61-75,
 * 77-104), which the reference recomputes on the host for every token step
 * (tvm/llama_auto_batcher/llama_exec_graph.py:106,114), and the np.sort of adapter ids in
 * huggingface/generation/gen_lora.py:78.
 *   d_tids  [n] int32 or NULL (NULL = every row with wid >= 0 is type 0, wid < 0 = no adapter)
 *   d_wids  [n] int32, 0 <= wid < n_wids for rows that have an adapter
 *   by_type_only != 0: key is (has_adapter, tid) only (get_decode_method's grouping: positions
 *                      stay ascending inside a type)
 * outputs (device):
 *   d_perm        [n]   perm[i] = index in the input of the row that lands at sorted position i
 *   d_sorted_tid  [n], d_sorted_wid [n]   tid / wid of the row at sorted position i (NULL to skip)
 *   d_seg_offsets [n_keys+1], d_seg_tid [n_keys], d_seg_wid [n_keys]: compacted runs of equal key
 *                 (only the first *n_seg entries are written, plus seg_offsets[n_seg] = n)
 *   d_counts      [n_types+2]: counts[0] = n_seg, counts[1] = rows without adapter,
 *                 counts[2+t] = rows of type t
 * n_keys = 1 + n_types * n_wids (or n_types+1 when by_type_only), at most 8192.  d_work needs
 * mlora_bucket_sort_workspace(n, n_types, n_wids) bytes (0 when n <= 1024). */
size_t mlora_bucket_sort_workspace(int32_t n, int32_t n_types, int32_t n_wids);
int mlora_bucket_sort(const int32_t* d_tids, const int32_t* d_wids, int32_t n, int32_t n_types,
                      int32_t n_wids, int32_t by_type_only, int32_t* d_perm, int32_t* d_sorted_tid,
                      int32_t* d_sorted_wid, int32_t* d_seg_offsets, int32_t* d_seg_tid,
                      int32_t* d_seg_wid, int32_t* d_counts, void* d_work, size_t work_bytes,
                      void* stream);

/* ---- (a) LoRA shrink: u[t, m*r_max + j] = sum_k x[t,k] * A_all[slot[t], m*r_max + j, k] --------
 * First half of the "take_matmul" pair (tvm/custom/fuse_take_matmul.py:78-111; Lora.forward
 * synthesised at tvm/llama_auto_batcher/compile_tvm.py:106-112) and of the two bmm's of
 * GatherBMMLinear.forward (huggingface/custom_peft/lora_gatherbmm_linear_layer.py:16-19).
 *   d_x [T, in] bf16 (row stride ldx elements); d_A_all [N, n_mod*r_max, in] bf16;
 *   d_ranks [N] int32 (rank of each adapter slot, <= r_max; rows of A_all at or beyond the rank
 *   must be zero: the kernels multiply them rather than look the rank up, except that the decode-size
 *   kernel skips rows beyond the first 16 of a module that lie beyond the adapter's rank);
 *   d_slots [T] int32 (adapter slot of each row; < 0 or >= n_adapters = none -> u row is zero);
 *   d_u [T, n_mod*r_max] float32.  n_mod modules share the input (q,k,v or gate,up).
 * T < 256: one warp per (row, rank index) on CUDA cores.  T >= 256 (prefill) with n_mod*r_max <= 256:
 * a segmented grouped GEMM on the tensor cores (tcgen05, TMA fed): one CTA per 128 rows, one
 * accumulator per distinct adapter among them, rows pick their adapter's columns on the way out
 * (the segmented "take_matmul" of tvm/custom/fuse_take_matmul.py:78-111 without the sort: rows of
 * one request are contiguous already).  Should one of that kernel's bounded waits expire, the
 * affected rows of d_u are NaN. */
int mlora_lora_shrink(const void* d_x, int64_t ldx, const void* d_A_all, const int32_t* d_ranks,
                      const int32_t* d_slots, int32_t n_adapters, int32_t T, int32_t in, int32_t r_max,
                      int32_t n_mod, float* d_u, void* stream);

/* ---- (a)+(b) base projection with the LoRA expand fused into the output write ----------------
 *   y[t, o] = sum_k x[t,k] W[o,k]  +  scale[s] * sum_j u[t, m(o)*r_max + j] * B_all[s, o, j]
 * with s = slot[t] (skipped when s < 0 or d_u == NULL) and m(o) the module that owns output row o
 * (mod_offsets[m] <= o < mod_offsets[m+1]).  With MLORA_SILU_MUL (n_mod = 2: gate, up) B_all is
 * [N, out, 2*r_max]: a gate row holds its B in columns [0, r_max) and zeros in [r_max, 2*r_max), an up
 * row the other way round, so that one dot product against u = [u_gate | u_up] serves both.
 * Padding of A_all / B_all beyond an adapter's rank must be zero.
 * Stands in for base_layer(x) + bmm(bmm(x, A), B*scaling)
 * (huggingface/custom_peft/lora_gatherbmm_linear_layer.py:15-20) and for nn.Linear followed by
 * "q += q_ft_proj(h, wids)" (tvm/llama_auto_batcher/compile_tvm.py:126-134, 142-155; the
 * write_tensor_part scatter of tvm/custom/write_tensor_part.py is subsumed because rows are
 * addressed directly).
 *   d_x [T,in] bf16; d_W [out,in] bf16; d_y [T, out or out/2] bf16 (or f32 with MLORA_OUT_F32),
 *   row stride ldy elements; d_B_all [N, out, r_max] bf16, r_max a multiple of 8; d_scales [N] float32;
 *   h_mod_offsets: HOST array of n_mod+1 ints (NULL when n_mod == 1), n_mod <= 8.
 *   d_work / work_bytes: scratch for split-K partial sums of the tensor-core kernel,
 *   mlora_linear_workspace(T, in, out) bytes (may be NULL/0: then the CUDA-core kernel runs).  The
 *   buffer must be zero-filled once before its first use (arrival counters; they reset themselves)
 *   and may be shared by calls of any shape on one stream; concurrent calls need separate buffers.
 *   Its first int32 is a status word: non-zero after a kernel gave up a bounded wait -- bit 0 (1) weight
 *   producer waiting for a free ring slot, 1 (2) MMA issuer waiting for operands, 2 (4) output warps
 *   waiting for an accumulator, 3 (8) MMA issuer waiting for a free accumulator, 4 (16) token-tile
 *   producer waiting for a free slot, 5 (32) LoRA operand builder waiting for the operand cache, 6 (64)
 *   MMA issuer waiting for the operand cache, 7 (128) finishing CTA waiting for the partial sums of a
 *   split tile.  The output of that call is then undefined, and because late contributors of a split
 *   tile may still bump its arrival counter afterwards, the whole buffer must be zero-filled again
 *   before its next use (the word is sticky: the caller clears it). */
size_t mlora_linear_workspace(int32_t T, int32_t in, int32_t out);
/* Introspection, host side only (no device work): how the tensor-core kernel deals a projection of this shape to its CTAs.
 * h_plan12 (HOST, 12 int32): [0] token rows per tile, [1] CTAs, [2] row tiles (128 outputs), [3] token tiles, [4] k-blocks
 * (64 of in), [5] k-block steps per CTA, [6] token tiles per group (0: contiguous ranges of k-blocks over all tiles, split
 * tiles handed over between CTAs -- decode sizes), [7] lanes (> 0: CTA c serves token tile c mod [6] of every group and the
 * row tiles c / [6] + s * [7], s = 0 .. [8] - 1; 0 with [6] > 0: contiguous chunks of [8] tiles per group), [8] steps per
 * group, [9] groups, [10] chunk length in the last, narrower group (chunk form), [11] 0. */
int mlora_linear_plan(int32_t T, int32_t in, int32_t out, int32_t* h_plan12);
/* The same for a call with these flags: more than mlora_linear_workspace only for MLORA_SILU_MUL | MLORA_LORA_PER_ROW. */
size_t mlora_linear_workspace_flags(int32_t T, int32_t in, int32_t out, int32_t flags);
/* Weight pre-packing (load time).  Rewrites W [out,in] bf16 as tiles [ceil(out/128)][ceil(in/64)] of
 * 128 rows x 64 columns, each tile 16 KB contiguous and already in the 128-byte-swizzled K-major
 * layout the tensor cores read from shared memory (zero padded), so that the projection kernel
 * fetches a whole pipeline stage with one contiguous bulk copy instead of 128 row requests.
 * The reference transposes / stacks weights once at load as well
 * (tvm/llama_auto_batcher/compile_tvm.py:287-320).  Pass the result to mlora_linear with
 * MLORA_W_PACKED (tensor-core kernel only). */
/* The same for an adapter stack: B_all [N, out, r_max] (r_max 16, 32, 64 or 128; for an interleaved
 * gate/up stack pass the doubled pitch) -> tiles [slot][row tile][64-wide rank slice] of 128 rows,
 * pre-swizzled, so each LoRA stage of the tensor-core expand is one bulk copy.  Pass the result to
 * mlora_linear with MLORA_B_PACKED (needs tile-aligned module boundaries). */
size_t mlora_packed_lora_b_bytes(int32_t n_adapters, int32_t out, int32_t r_max);
int mlora_pack_lora_b(const void* d_B_all, int32_t n_adapters, int32_t out, int32_t r_max, void* d_Bp,
                      void* stream);
size_t mlora_packed_weight_bytes(int32_t out, int32_t in);
int mlora_pack_weight(const void* d_W, int32_t out, int32_t in, void* d_Wp, void* stream);
int mlora_linear(const void* d_x, int64_t ldx, const void* d_W, void* d_y, int64_t ldy, int32_t T,
                 int32_t in, int32_t out, const float* d_u, const void* d_B_all,
                 const int32_t* d_ranks, const float* d_scales, const int32_t* d_slots,
                 int32_t n_adapters, int32_t r_max, int32_t n_mod, const int32_t* h_mod_offsets,
                 int32_t flags, void* d_work, size_t work_bytes, void* stream);
/* mlora_linear with the residual add + RMSNorm that sits between two decoder projections folded into their epilogues
 * (T <= 32, tensor-core kernel only: d_work required).  The reference runs these as separate modules: o_proj, residual
 * add, post_attention_layernorm, gate/up (huggingface LlamaDecoderLayer as wrapped by
 * huggingface/custom_peft/wrap_model.py; tvm/llama_auto_batcher/llama_for_causal_lm.py:96-112).  RMSNorm is
 * h = x * w / rms(x); the factor 1/rms(x) of a row commutes with the next linear map, so
 *   producer (d_res != NULL): d_res[t, o] (fp32, pitch ld_res) += y[t, o];  d_y[t, o] = bf16(d_res[t, o] * d_norm_w[o]);
 *       d_sumsq_out[(o / 128) * 32 + t] = sum over that block of 128 outputs of d_res[t, o]^2   (ceil(out/128) * 32 floats);
 *   consumer (d_sumsq_in != NULL): every output row t is multiplied by
 *       rsqrt(sum_{j < n_sumsq_in} d_sumsq_in[j * 32 + t] / norm_dim + eps) before the activation (SiLU*up) and the store.
 * A call may be both.  Sums are taken in a fixed order (deterministic).  Not with MLORA_LORA_PER_ROW / MLORA_FORCE_SIMT;
 * the producer form not with MLORA_SILU_MUL / MLORA_OUT_F32.  Rounding differs from norm-then-project (bf16(x*w) * 1/rms in
 * fp32 instead of bf16(x*w/rms)); both are within the path's bf16 tolerance. */
int mlora_linear_norm(const void* d_x, int64_t ldx, const void* d_W, void* d_y, int64_t ldy, int32_t T, int32_t in,
                      int32_t out, const float* d_u, const void* d_B_all, const int32_t* d_ranks,
                      const float* d_scales, const int32_t* d_slots, int32_t n_adapters, int32_t r_max, int32_t n_mod,
                      const int32_t* h_mod_offsets, int32_t flags, void* d_work, size_t work_bytes, float* d_res,
                      int64_t ld_res, const void* d_norm_w, float* d_sumsq_out, const float* d_sumsq_in,
                      int32_t n_sumsq_in, float eps, int32_t norm_dim, void* stream);
/* mlora_lora_shrink + mlora_linear as ONE call, i.e. the whole of
 * base_layer(x) + bmm(bmm(x, A), B*scaling) (huggingface/custom_peft/lora_gatherbmm_linear_layer.py:15-20).
 * d_A_all as for mlora_lora_shrink; d_u [T, n_mod*r_max] float32 is scratch the call writes before it
 * reads it.  It issues the shrink kernel and the projection kernel back to back on `stream` (a single
 * kernel that computed the shrink in the projection's idle output warps and published it with a
 * grid-wide counter was measured slower than this pair under programmatic dependent launch, and is
 * not kept). */
int mlora_lora_linear(const void* d_x, int64_t ldx, const void* d_W, void* d_y, int64_t ldy, int32_t T,
                      int32_t in, int32_t out, const void* d_A_all, float* d_u, const void* d_B_all,
                      const int32_t* d_ranks, const float* d_scales, const int32_t* d_slots,
                      int32_t n_adapters, int32_t r_max, int32_t n_mod, const int32_t* h_mod_offsets,
                      int32_t flags, void* d_work, size_t work_bytes, void* stream);

/* ---- a chain of decode-size projections in ONE persistent launch ------------------------------------
 * Everything between two attention calls of the decoder layer
 * (tvm/llama_auto_batcher/llama_for_causal_lm.py:71-84; the reference runs a whole step as one VM
 * function, tvm/llama_auto_batcher/llama_exec_graph.py:126) as up to MLORA_CHAIN_MAX_PHASES phases:
 *   phase = [res += delta; x = RMSNorm(res) * norm_w]  ->  [u = A_all[slot] . x]  ->  y = x Wp^T (+ expand of u)
 * where both bracketed row operations are optional.  Phase i+1 reads what phase i wrote (d_x of phase
 * i+1 = d_y of phase i, or d_delta of phase i+1 = d_y of phase i when it has a norm); the kernel orders
 * them with grid-wide barriers instead of kernel boundaries and keeps streaming weights across them.
 * Results are bit-identical to the same sequence of mlora_residual_rmsnorm / mlora_lora_shrink /
 * mlora_linear calls (same tile split, same reduction orders).
 *   d_x [T,in] bf16 (row stride ldx; written by the norm when d_res != NULL, then ldx == in, in <= 8192)
 *   d_Wp: mlora_pack_weight layout.  d_y [T, out or out/2] bf16 (f32 with MLORA_OUT_F32), rows 16-byte multiples
 *   flags: MLORA_OUT_F32 | MLORA_SILU_MUL only
 *   d_res fp32 [T,in] in/out or NULL (no norm); d_delta bf16 [T,in] or NULL; d_norm_w bf16 [in]
 *   d_Bp: mlora_pack_lora_b layout or NULL (no adapters on this phase); then d_A_all [N, n_mod*r_max, in],
 *   d_u [T, n_mod*r_max] float32 (written by the shrink, read by the expand), mod_offsets as for mlora_linear
 *   (n_mod <= 4, tile-aligned modules; ignored with MLORA_SILU_MUL, whose stack is the interleaved one)
 * T <= 32 (decode batches).  d_slots / d_ranks / d_scales as for mlora_linear, shared by all phases.
 * d_work: the scratch of mlora_linear (largest mlora_linear_workspace of the phases), zero-filled once; the
 * status word is shared too, with bit 8 (256) = a grid barrier wait expired.  All CTAs of the launch must be
 * co-resident: nothing else may occupy the device's SMs for the duration (a wait that cannot be satisfied
 * expires and sets the status word; it does not hang). */
#define MLORA_CHAIN_MAX_PHASES 6
typedef struct mlora_chain_phase {
  const void* d_x;
  int64_t ldx;
  const void* d_Wp;
  void* d_y;
  int64_t ldy;
  int32_t in, out, flags;
  float eps;
  float* d_res;
  const void* d_delta;
  const void* d_norm_w;
  const void* d_A_all;
  float* d_u;
  const void* d_Bp;
  int32_t r_max, n_mod;
  int32_t mod_offsets[5];
} mlora_chain_phase;
int mlora_decode_chain(const mlora_chain_phase* phases, int32_t n_phases, int32_t T, const int32_t* d_slots,
                       const int32_t* d_ranks, const float* d_scales, int32_t n_adapters, void* d_work,
                       size_t work_bytes, void* stream);

/* ---- (b) fused residual add + RMSNorm ----------------------------------------------------------
 *   res[t,:] += delta[t,:] (skipped when d_delta == NULL);  out[t,:] = res * rsqrt(mean(res^2)+eps) * w
 * nn.RMSNorm + the "hidden_states += ..." of LlamaDecoderLayer.forward
 * (tvm/llama_auto_batcher/llama_for_causal_lm.py:76-84,93).
 *   d_delta [T,H] bf16 or NULL; d_res [T,H] float32 in/out; d_w [H] bf16; d_out [T,H] bf16. */
int mlora_residual_rmsnorm(const void* d_delta, float* d_res, const void* d_w, float eps,
                           void* d_out, int32_t T, int32_t H, void* stream);

/* The same with the LoRA shrink of the projection that reads the normalised row fused in:
 *   res_out = res_in + delta;  out = RMSNorm(res_out) * w;  u[t, j] = A_all[slot[t], j, :] . out[t, :]
 * (out as rounded to bf16, i.e. exactly what mlora_lora_shrink would read).  One launch instead of two for
 * "input_layernorm -> q/k/v adapters" (llama_for_causal_lm.py:76-84 followed by compile_tvm.py:126-134).
 * Several CTAs share a row and re-read the old residual while one of them writes the new one, so the
 * residual moves from d_res_in to a DIFFERENT buffer d_res_out.  H <= 8192; d_A_all [N, r_tot, H] with
 * zero rows beyond each adapter's rank (all r_tot rows are read and multiplied: for stacks whose adapters are
 * much narrower than the pitch the two separate calls read less); d_u [T, r_tot] float32. */
int mlora_residual_rmsnorm_shrink(const void* d_delta, const float* d_res_in, float* d_res_out, const void* d_w,
                                  float eps, void* d_out, int32_t T, int32_t H, const void* d_A_all,
                                  const int32_t* d_slots, int32_t n_adapters, int32_t r_tot, float* d_u,
                                  void* stream);

/* ---- embedding gather: res[t,:] = float(E[ids[t], :]) ------------------------------------------
 * vm["embed"](input_ids, params) (tvm/llama_auto_batcher/llama_for_causal_lm.py:121-122).
 * Optionally also writes the gathered rows as bf16 to d_out_bf16 (the reference's return value). */
int mlora_embed(const int32_t* d_ids, const void* d_E, int32_t T, int32_t H, int32_t vocab,
                float* d_res, void* d_out_bf16, void* stream);

/* ---- greedy token: tok[t] = first index of the row maximum -------------------------------------
 * Replaces logits.numpy() + np.argmax per row (tvm/llama_auto_batcher/llama_exec_graph.py:92,134-137). */
int mlora_argmax(const float* d_logits, int64_t ld, int32_t T, int32_t V, int32_t* d_tok,
                 void* stream);

/* ---- (c) paged KV cache -------------------------------------------------------------------------
 * Cache layout per layer: K pages [n_pages, Hkv, page_size, D] bf16 and V pages of the same shape.
 * Block table [n_slots, max_pages] int32 (page ids of a sequence in order); d_seq_lens [n_slots]
 * int32 = tokens already stored.  Rows of a step carry d_row_slot[t] (cache slot of the row's
 * sequence) and d_row_pos[t] (position of the row's token in its sequence).
 * Together these stand in for paged_kv_cache.attention_with_fused_qkv(layer, qkv, n_q)
 * (tvm/llama_auto_batcher/llama_for_causal_lm.py:55-64) on a cache made by create_paged_kv_cache
 * (:148-174: rope INLINE, scale 1, rotary_dim = head_dim, no sliding window).
 *
 * mlora_kv_append_rope: rotates q and k of every row (rotate-half pairing), writes q back in
 * place into d_qkv and stores rotated k and v into the pages (prefill path).
 *   d_qkv [T, (Hq+2*Hkv)*D] bf16, row stride ld elements. */
int mlora_kv_append_rope(void* d_qkv, int64_t ld, void* d_k_pages, void* d_v_pages,
                         const int32_t* d_block_table, int32_t max_pages, const int32_t* d_row_slot,
                         const int32_t* d_row_pos, int32_t T, int32_t Hq, int32_t Hkv, int32_t D,
                         int32_t page_size, float rope_theta, void* stream);

/* mlora_paged_attention: out[t, h*D..] = softmax(q_t k^T / sqrt(D)) v over tokens 0..pos_t of the
 * row's sequence, gathered through the block table.
 *   fused_append != 0 (decode, one row per sequence): q and the row's new k are rotated here, the
 *     new k/v are stored into the pages at position pos_t, and d_qkv is left untouched.
 *   fused_append == 0: d_qkv already holds rotated q and the pages already hold tokens 0..pos_t
 *     (after mlora_kv_append_rope).
 *   n_splits > 1 splits every row's context over n_splits CTAs; needs d_work of
 *   mlora_paged_attention_workspace(T, Hq, D, n_splits) bytes.  n_splits <= 0 lets the library pick. */
size_t mlora_paged_attention_workspace(int32_t T, int32_t Hq, int32_t D, int32_t n_splits);
int mlora_paged_attention(const void* d_qkv, int64_t ld, void* d_k_pages, void* d_v_pages,
                          const int32_t* d_block_table, int32_t max_pages,
                          const int32_t* d_row_slot, const int32_t* d_row_pos, int32_t T, int32_t Hq,
                          int32_t Hkv, int32_t D, int32_t page_size, float rope_theta,
                          int32_t fused_append, void* d_out, int64_t ld_out, int32_t n_splits,
                          void* d_work, size_t work_bytes, void* stream);

/* mlora_prefill_attention: causal attention for prompt rows on the tensor cores, after mlora_kv_append_rope has
 * rotated q in place and stored the rows' k / v -- the ragged prefill path of attention_with_fused_qkv
 * (tvm/llama_auto_batcher/llama_for_causal_lm.py:55-64; prefill call llama_exec_graph.py:75-85).  The rows are given as
 * tiles: d_tiles [n_tiles][4] int32 = (cache slot, index of the tile's first row in d_qkv / d_out, rows <= 128,
 * position of that first row in its sequence); the rows of a tile are consecutive rows of ONE sequence at consecutive
 * positions.  Same result as mlora_paged_attention(fused_append = 0) on those rows (different summation order).
 * head_dim 128 and page size 16 only; n_pages_total = pages in d_k_pages / d_v_pages; T = rows of d_qkv.
 * d_status (optional, device int32): set to 1 if a bounded wait expired (the affected rows are then zeros). */
int mlora_prefill_attention(const void* d_qkv, int64_t ld, const void* d_k_pages, const void* d_v_pages,
                            int32_t n_pages_total, const int32_t* d_block_table, int32_t max_pages,
                            const int32_t* d_tiles, int32_t n_tiles, int32_t Hq, int32_t Hkv, int32_t D,
                            int32_t page_size, int32_t T, void* d_out, int64_t ld_out, int32_t* d_status, void* stream);

/* Split count the library picks for n_splits <= 0 (1 = every (row, head) is one CTA, no merge kernel). */
uint32_t mlora_paged_attention_splits(int32_t T, int32_t Hq, int32_t max_pages);

/* mlora_paged_attention_shrink: attention as above AND, in the same launch, the LoRA shrink of the projection that
 * reads its output -- o_proj's half of "q += ft_proj(h, wids)" (tvm/llama_auto_batcher/compile_tvm.py:126-134 applied
 * to the output projection; huggingface/custom_peft/lora_gatherbmm_linear_layer.py:16-19):
 *   d_u[t, j] = sum_c A_all[slot[t], j, c] * out[t, c]      (out as rounded to bf16; rows without adapter give 0)
 * Every (row, head) CTA adds its head's share to per-head partial sums; the last head of a row to finish adds them in
 * head order.  d_A_all [N, r_max, Hq*D] bf16 (rows at or beyond an adapter's rank zero), d_u [T, r_max] float32.
 * Only where the library runs one CTA per (row, head) (mlora_paged_attention_splits(...) == 1); otherwise the call
 * is refused and the caller runs mlora_paged_attention + mlora_lora_shrink.  d_shrink_work:
 * mlora_paged_attention_shrink_workspace(T, Hq, r_max) bytes, zero-filled once before first use (arrival counters,
 * they reset themselves), not shared with concurrent calls.  Sums in a different order than mlora_lora_shrink. */
size_t mlora_paged_attention_shrink_workspace(int32_t T, int32_t Hq, int32_t r_max);
int mlora_paged_attention_shrink(const void* d_qkv, int64_t ld, void* d_k_pages, void* d_v_pages,
                                 const int32_t* d_block_table, int32_t max_pages, const int32_t* d_row_slot,
                                 const int32_t* d_row_pos, int32_t T, int32_t Hq, int32_t Hkv, int32_t D,
                                 int32_t page_size, float rope_theta, int32_t fused_append, void* d_out,
                                 int64_t ld_out, const void* d_A_all, const int32_t* d_ranks, const int32_t* d_slots,
                                 int32_t n_adapters, int32_t r_max, float* d_u, void* d_shrink_work,
                                 size_t shrink_work_bytes, void* stream);

/* mlora_paged_attention_static: the same operation for callers that must not allocate.
 * (No counterpart in the reference project; added for embedders of this library.)
 * Some hosts of this code hand out all device memory themselves at start-up -- a serving runtime
 * with a fixed arena, or a plugin loaded into a process whose allocator belongs to someone else --
 * and their request path may not call cudaMalloc (it can stall the whole device, and the memory may
 * simply all be spoken for).  For them the split-KV partial results go into a 16 MiB array that is
 * part of the library image (mlora_paged_attention_static_max_bytes()); each GPU that loads the
 * library holds that array until the process ends.  The call allocates and frees nothing.
 *  - The first call on each device looks up the array's device address (one cudaGetSymbolAddress, with
 *    that device current) and remembers it; make that first call before any stream capture starts.
 *  - Arguments are validated first (MLORA_EINVAL).  n_splits > 1 whose partials (T * Hq * n_splits * (D+2) * 4
 *    bytes) exceed the array is rejected with MLORA_ESIZE; n_splits <= 0 picks a split count, and every count
 *    the library picks by itself fits.
 *  - The array that is used is the one of the CURRENT device (cudaGetDevice) at the time of the call: `stream`
 *    must belong to that device.
 *  - All calls on a device share the one array, and it keeps whatever the previous call left in it.
 *    Nothing in it needs clearing between calls (every partial is written before it is read), but two
 *    calls that overlap on the GPU (different streams) would overwrite each other: serialise them.
 * Arguments as mlora_paged_attention, without d_work / work_bytes. */
size_t mlora_paged_attention_static_max_bytes(void);
int mlora_paged_attention_static(const void* d_qkv, int64_t ld, void* d_k_pages, void* d_v_pages,
                                 const int32_t* d_block_table, int32_t max_pages,
                                 const int32_t* d_row_slot, const int32_t* d_row_pos, int32_t T,
                                 int32_t Hq, int32_t Hkv, int32_t D, int32_t page_size,
                                 float rope_theta, int32_t fused_append, void* d_out, int64_t ld_out,
                                 int32_t n_splits, void* stream);

/* ---- decode-step bookkeeping on the device (keeps a whole step inside one CUDA graph) ----------
 * For each live row b: slot = d_row_slot[b]; d_row_pos[b] = d_seq_lens[slot]; d_seq_lens[slot] += 1.
 * What kv_state_begin_forward(kv, seq_ids, [1]*B) does on the host in the reference
 * (tvm/llama_auto_batcher/llama_exec_graph.py:121-125).  Pages must already be reserved. */
int mlora_kv_begin_decode(const int32_t* d_row_slot, int32_t* d_seq_lens, int32_t* d_row_pos,
                          int32_t B, void* stream);

/* ---- tensor parallelism: the exchange after a row-parallel projection, over peer memory ---------------
 * (The reference is single-device; this is the Megatron-style split of the same decoder layer,
 * tvm/llama_auto_batcher/llama_for_causal_lm.py:71-84: o and down produce partial sums on every rank.)
 * One process per GPU.  mlora_tp_create allocates this rank's arena (device memory, once, at set-up);
 * mlora_tp_export writes its 64-byte CUDA IPC handle, which the ranks exchange by any means;
 * mlora_tp_connect maps a peer's arena.  Then, on every rank, in the same order:
 *   mlora_tp_allreduce_rmsnorm:  s = sum over ranks of d_partial (bf16 [T,H], summed in rank order in fp32,
 *     rounded to bf16);  d_res != NULL: res += s, d_out = RMSNorm(res) * w (what all-reduce followed by
 *     mlora_residual_rmsnorm gives);  d_res == NULL: d_out = s (a plain all-reduce; d_out may be d_partial).
 * ONE kernel per rank: it stores its rows into the peers' arenas over NVLink, sets a per-row flag there, waits
 * (bounded) for the peers' rows to land in its own arena, and reduces locally.  T <= 512 and <= T_max, H <= 8192.
 * Beyond four ranks (or with MLORA_TP_TWO_STEP=1 in the environment at mlora_tp_create; =0 forces the form above) the
 * kernel works in two steps: row t is reduced by rank t mod world, which receives that row from every peer and stores
 * the rounded sum into every peer's arena; same result bits, 2 (world-1)/world of the partial result leaves a rank
 * instead of world-1 times it.  All ranks of a group must use the same form.
 * The calls of the ranks must pair up one to one; a rank whose peer's rows do not arrive within the spin limit
 * (mlora_tp_set_spin_limit polls of ~100 ns; default 2^22) sets bit g (rank g missing) in its status word
 * (mlora_tp_status), produces garbage for that exchange and returns -- it does not hang.  After such a failure
 * all ranks call mlora_tp_reset between two host-side barriers.  Peers must stay alive (and must not destroy
 * their arena) while any rank may still launch an exchange. */
size_t mlora_tp_arena_bytes(int32_t T_max, int32_t H);
int mlora_tp_create(int32_t rank, int32_t world, int32_t T_max, int32_t H, void** ctx_out);
int mlora_tp_export(void* ctx, void* handle_out64);
int mlora_tp_connect(void* ctx, int32_t peer_rank, const void* handle64);
int mlora_tp_set_spin_limit(void* ctx, uint32_t polls);
int mlora_tp_status(void* ctx, int32_t* status_out);
int mlora_tp_reset(void* ctx);
int mlora_tp_destroy(void* ctx);
int mlora_tp_allreduce_rmsnorm(void* ctx, const void* d_partial, float* d_res, const void* d_w, float eps,
                               void* d_out, int32_t T, int32_t H, void* stream);

/* ---- the batched greedy loop with sequences that finish, without the host in between --------------
 * The reference's executor reads the logits back after every token, takes the argmax on the host, drops
 * finished sequences (end-of-sequence token or the sequence's own max_gen_len) and rebuilds the index lists of
 * the live batch (tvm/llama_auto_batcher/llama_exec_graph.py:94-100, 102-141).  These two calls keep that state
 * on the device.  The sequences of a fused decode node are held in the order of mlora_bucket_sort (rows without
 * adapter first, then by adapter); per sequence b: d_live[b], d_seq_slot[b] (KV cache slot), d_adapter_slot[b],
 * d_last_tok[b], d_gen_count[b], d_max_gen[b], d_out_tokens[b, 0..ld_out).
 *
 * mlora_decode_step_begin: stable compaction of the live sequences into rows 0..n_live-1 of a step of n_rows rows
 * (the adapter order survives); for each: d_row_src = b, d_row_slot, d_row_pos = seq_lens[slot]++ (what
 * kv_state_begin_forward(kv, seq_ids, [1]*B) does), d_row_adapter, d_row_tok.  Rows n_live..n_rows-1 become
 * padding: no adapter, position -1 (mlora_paged_attention stores and reads nothing for them), token 0.
 * *d_n_live = n_live.  n_rows must be >= the number of live sequences.
 *
 * mlora_decode_step_end: for every live row i: the new token d_next_tok[i] is appended to d_out_tokens[b,
 * gen_count[b]++] and becomes d_last_tok[b]; the sequence stops (d_live[b] = 0, *d_n_live decremented) when the
 * token equals eos_id (pass -1 for none) or gen_count reaches d_max_gen[b] (or ld_out). */
int mlora_decode_step_begin(const int32_t* d_live, const int32_t* d_seq_slot, const int32_t* d_adapter_slot,
                            const int32_t* d_last_tok, int32_t n_seq, int32_t n_rows, int32_t* d_seq_lens,
                            int32_t* d_row_src, int32_t* d_row_slot, int32_t* d_row_pos, int32_t* d_row_adapter,
                            int32_t* d_row_tok, int32_t* d_n_live, void* stream);
int mlora_decode_step_end(const int32_t* d_row_src, const int32_t* d_next_tok, int32_t n_rows, int32_t* d_live,
                          int32_t* d_last_tok, int32_t* d_gen_count, const int32_t* d_max_gen,
                          int32_t* d_out_tokens, int64_t ld_out, int32_t eos_id, int32_t* d_n_live, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* MLORA_H_ */
