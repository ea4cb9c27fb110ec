/*
 * moe_b200.h - C ABI of libmoe_b200.so: the sm_100a implementation of the
 * `moe_fused_linear` hot path of transformers-qwen3-moe-fused.
 *
 * Conventions shared by every entry point
 *   - Every pointer except `stream` is a DEVICE pointer owned by the caller.  The
 *     library never allocates, frees or retains device memory.
 *   - `stream` is a cudaStream_t passed as void*; work is enqueued on it and the call
 *     returns without synchronising.  `m_sizes` is only ever read on the device.
 *   - Return value: 0 = success; < 0 = argument error, nothing was launched
 *     (see MOE_ERR_*); > 0 = a cudaError_t reported by the runtime.
 *   - dtype codes: MOE_F32 / MOE_BF16 / MOE_F16 for floating point tensors,
 *     MOE_I32 / MOE_I64 for integer tensors.
 *   - All tensors are dense row-major ("contiguous" in torch terms).
 *
 * The comment on each function names the reference interface it stands in for
 * (path inside the reference project : lines).
 */
#ifndef MOE_B200_H_
#define MOE_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum { MOE_F32 = 0, MOE_BF16 = 1, MOE_F16 = 2, MOE_I32 = 3, MOE_I64 = 4 };

enum {
  MOE_OK = 0,
  MOE_ERR_DTYPE = -1,      /* unsupported dtype code or dtype combination        */
  MOE_ERR_SHAPE = -2,      /* negative / inconsistent / unsupported extent       */
  MOE_ERR_NULL = -3,       /* a required pointer is NULL                         */
  MOE_ERR_WORKSPACE = -4,  /* workspace missing or smaller than the query said   */
  MOE_ERR_UNSUPPORTED = -5,/* valid request that this build has no kernel for    */
  MOE_ERR_ALIGN = -6,      /* pointer or pitch not aligned as the kernel needs   */
  MOE_ERR_DEVICE = -7      /* device is not sm_100 or a driver entry is missing  */
};

/* Which kernel family a grouped GEMM call may use.
 * AUTO:      tcgen05 when the shape and dtype are eligible, SIMT otherwise.
 * SIMT:      CUDA-core kernel (any shape, fp32 math for fp32 inputs).
 * TC:        tcgen05 kernel (CTA-pair form where there is one) or MOE_ERR_UNSUPPORTED.
 * TC_SINGLE: tcgen05 kernel, single-CTA form, or MOE_ERR_UNSUPPORTED. */
enum { MOE_PATH_AUTO = 0, MOE_PATH_SIMT = 1, MOE_PATH_TC = 2, MOE_PATH_TC_SINGLE = 3 };

/* Library build version (monotonic integer). */
int moe_b200_version(void);

/* Human readable text for a status returned by any function below. */
const char* moe_status_string(int status);

/* Set / get the kernel family used by the grouped GEMM entry points (process wide,
 * MOE_PATH_*; default AUTO).  Returns the previous value.
 * For tests and measurements only (they compare the kernel families on the same inputs):
 * the setting is one word shared by every thread and stream of the process and is read when
 * a call is issued, so production code leaves it at AUTO, where the selection depends on
 * dtype, extents and alignment of the call alone. */
int moe_set_gemm_path(int path);
int moe_get_gemm_path(void);

/* ---------------------------------------------------------------------------------
 * Stable sort of rows by expert id.
 * Replaces qwen3_moe_fused/kernels/indexing.py:48-65 (get_expert_counts_and_idx) and,
 * with idx/inv_idx NULL, :18-23 (get_expert_counts).
 *   s        (M,)  expert id per row, s_dtype = MOE_I32 or MOE_I64, values in [0,E)
 *   counts   (E,)  int32  rows per expert
 *   inv_idx  (M,)  int32  inv_idx[j] = original row at sorted position j (gather index)
 *   idx      (M,)  int32  idx[b]     = sorted position of original row b
 * Ties keep their original order (identical to a stable argsort).
 * ws must hold moe_sort_workspace_bytes(M, E) bytes; its contents are scratch.
 * ------------------------------------------------------------------------------- */
size_t moe_sort_workspace_bytes(int64_t M, int E);
int moe_sort_by_expert(const void* s, int s_dtype, int64_t M, int E,
                       int32_t* counts, int32_t* inv_idx, int32_t* idx,
                       void* ws, size_t ws_bytes, void* stream);

/* moe_sort_by_expert without a workspace argument, for callers that cannot allocate device
 * memory where they call it (no cudaMalloc allowed there, or no allocator at all): the scratch
 * is a fixed array of moe_sort_static_capacity_bytes() (256 KB) inside the library's device
 * image.  Same inputs, outputs and results as moe_sort_by_expert.
 *   - Sizes whose scratch need (moe_sort_workspace_bytes(M, E)) exceeds the capacity are
 *     rejected with MOE_ERR_WORKSPACE and nothing is launched.
 *   - The call itself allocates nothing.  The first call on each device looks up the array's
 *     device address (with that device current); make that first call before any stream capture.
 *   - All calls on a device share the one array: two calls whose kernels can overlap on the GPU
 *     (different streams, no dependency between them) race.  Calls on one stream are safe; the
 *     array keeps the last call's contents and nothing in it needs clearing between calls.
 * This entry point has no counterpart in the reference. */
size_t moe_sort_static_capacity_bytes(void);
int moe_sort_by_expert_static(const void* s, int s_dtype, int64_t M, int E,
                              int32_t* counts, int32_t* inv_idx, int32_t* idx, void* stream);

/* Begin/end row of every expert in an already sorted id vector.
 * Replaces qwen3_moe_fused/kernels/indexing.py:7-14 (get_batch_begins_ends).
 *   begins_ends (E,2) int32: [e,0] = #rows with id < e, [e,1] = #rows with id <= e */
int moe_batch_begins_ends(const void* s_sorted, int s_dtype, int64_t M, int E,
                          int32_t* begins_ends, void* stream);

/* ---------------------------------------------------------------------------------
 * Grouped GEMMs.  Rows of x / y are sorted by expert; expert e owns m_sizes[e]
 * consecutive rows (m_sizes_dtype MOE_I32 or MOE_I64, sum = M, zeros allowed).
 * Accumulation is fp32; the result is rounded once to dtype_out.
 * ws/ws_bytes: device scratch of moe_grouped_gemm_workspace_bytes() bytes, 128-byte aligned,
 *   owned by the caller.  A small launch ahead of each GEMM writes per-expert tensor maps and a
 *   work-item counter into it, so one workspace serves one GEMM at a time: calls issued on one
 *   stream may share it, calls on different streams need one each.  Forward and dX also accept
 *   NULL/0 and then run a slower form (no per-expert maps, fixed tile order); dW on the
 *   tensor-core path and the fused / gathered / scattered forms return MOE_ERR_WORKSPACE.
 * ------------------------------------------------------------------------------- */
size_t moe_grouped_gemm_workspace_bytes(int which /*0 fwd, 1 dx, 2 dw*/, int64_t M, int N, int K, int E);

/* y[m,n] = sum_k w[e(m),n,k] * x[m,k];  x (M,K), w (E,N,K), y (M,N).
 * Replaces qwen3_moe_fused/grouped_gemm/forward.py:116-160 (grouped_gemm_forward). */
int moe_grouped_gemm_fwd(const void* x, const void* w, const void* m_sizes, int m_sizes_dtype,
                         void* y, int64_t M, int N, int K, int E, int dtype_in, int dtype_out,
                         void* ws, size_t ws_bytes, void* stream);

/* y[m,n] = sum_k w[e(m),k,n] * x[m,k];  x (M,K), w (E,K,N), y (M,N)  (this is dX).
 * Replaces qwen3_moe_fused/grouped_gemm/forward_transposed.py:107-151
 * (grouped_gemm_forward_transposed). */
int moe_grouped_gemm_dx(const void* x, const void* w, const void* m_sizes, int m_sizes_dtype,
                        void* y, int64_t M, int N, int K, int E, int dtype_in, int dtype_out,
                        void* ws, size_t ws_bytes, void* stream);

/* w[e,n,k] = sum_{m in group e} y[m,n] * x[m,k];  x (M,K), y (M,N), w (E,N,K).
 * Experts without rows get zeros.
 * Replaces qwen3_moe_fused/grouped_gemm/backward_dw.py:92-134 (grouped_gemm_backward_dw). */
int moe_grouped_gemm_dw(const void* x, const void* y, const void* m_sizes, int m_sizes_dtype,
                        void* w, int64_t M, int N, int K, int E, int dtype_in, int dtype_out,
                        void* ws, size_t ws_bytes, void* stream);

/* Gate projection, up projection and SiLU-mul of the expert MLP in one kernel:
 *   h[m,i] = T(T(silu(e)) * g),  e = T(sum_k w_gate[e(m),i,k] x[m,k]),  g = T(sum_k w_up[e(m),i,k] x[m,k])
 * with T = dtype: bit-identical to moe_grouped_gemm_fwd twice followed by moe_silu_mul_fwd, without
 * writing or re-reading the two projections.  x (M,K), w_gate / w_up (E,I,K), h (M,I).
 * Replaces qwen3_moe_fused/modular_qwen3_moe_fused.py:105-108 (inference; the projections are
 * not kept for a backward pass).  Tensor-core CTA-pair kernel only: bf16/fp16, workspace
 * required; MOE_ERR_UNSUPPORTED otherwise. */
int moe_gate_up_silu_fwd(const void* x, const void* w_gate, const void* w_up, const void* m_sizes,
                         int m_sizes_dtype, void* h, int64_t M, int I, int K, int E, int dtype,
                         void* ws, size_t ws_bytes, void* stream);

/* moe_gate_up_silu_fwd and moe_grouped_gemm_fwd with the token rows gathered inside the kernel's
 * token load: sorted row r (r < M, grouped by m_sizes as usual) is row row_index[r] / index_div of x,
 * which has x_rows rows (row_index: DEVICE int32 array of M entries).  Passing the sort's gather index
 * and k = index_div feeds the expert GEMMs straight from the (T, hidden) token tensor, without
 * materialising the expanded, sorted copy (qwen3_moe_fused/modular_qwen3_moe_fused.py:95-103 builds that
 * copy with expand + reshape + index).  The result is bit-identical to gathering first.  Rows are fetched
 * with TMA tile::gather4 loads.  Tensor-core CTA-pair kernels only: bf16/fp16, N (I) >= 192 for the plain
 * forward, workspace required; MOE_ERR_UNSUPPORTED / MOE_ERR_WORKSPACE otherwise. */
int moe_gate_up_silu_fwd_gather(const void* x, int64_t x_rows, const int32_t* row_index, int index_div,
                                const void* w_gate, const void* w_up, const void* m_sizes,
                                int m_sizes_dtype, void* h, int64_t M, int I, int K, int E, int dtype,
                                void* ws, size_t ws_bytes, void* stream);
int moe_grouped_gemm_fwd_gather(const void* x, int64_t x_rows, const int32_t* row_index, int index_div,
                                const void* w, const void* m_sizes, int m_sizes_dtype, void* y,
                                int64_t M, int N, int K, int E, int dtype_in, int dtype_out,
                                void* ws, size_t ws_bytes, void* stream);

/* Forward with an NF4 weight decoded inside the kernel:
 *   w[e,n,k] = code[nibble(e,n,k)] * absmax[(e*N*K + n*K + k) / blocksize], rounded to
 *   dtype_in, then as moe_grouped_gemm_fwd.  packed: E*N*K/2 bytes, element 2j in the
 *   HIGH nibble of byte j and element 2j+1 in the low nibble; code: 16 fp32;
 *   absmax: E*N*K/blocksize fp32 (already un-nested); blocksize a power of two.
 * Replaces qwen3_moe_fused/grouped_gemm/forward_4bit.py:135-208 (grouped_gemm_forward_4bit). */
int moe_grouped_gemm_fwd_nf4(const void* x, const uint8_t* packed, const float* code,
                             const float* absmax, int blocksize,
                             const void* m_sizes, int m_sizes_dtype, void* y,
                             int64_t M, int N, int K, int E, int dtype_in, int dtype_out,
                             void* ws, size_t ws_bytes, void* stream);

/* dX through an NF4 weight decoded inside the kernel:
 *   y[m,n] = sum_k w[e(m),k,n] * x[m,k],  w = the NF4 tensor of logical shape (E,K,N)
 *   (K = the layer's out_features, N = its in_features), decoded as in
 *   moe_grouped_gemm_fwd_nf4.  x (M,K), y (M,N).
 * The reference has no fused form: its backward decodes the whole weight first
 * (qwen3_moe_fused/kernels/fast_lora.py:57-63,128; quantize/layer.py:17-22).
 * Tensor-core CTA-pair kernel only: bf16/fp16, blocksize >= 64, N % 64 == 0, K % 64 == 0,
 * N >= 192; MOE_ERR_UNSUPPORTED otherwise (decode with moe_nf4_dequant and call
 * moe_grouped_gemm_dx instead). */
int moe_grouped_gemm_dx_nf4(const void* x, const uint8_t* packed, const float* code,
                            const float* absmax, int blocksize, const void* m_sizes,
                            int m_sizes_dtype, void* y, int64_t M, int N, int K, int E,
                            int dtype_in, int dtype_out, void* ws, size_t ws_bytes, void* stream);

/* fp32 absmax from a double-quantised ("nested") one: out[i] = code2[q[i]] * absmax2[i /
 * blocksize2] + offset[0] (offset may be NULL = 0), product and sum each rounded to fp32.
 * q: n bytes; code2: 256 fp32 levels; absmax2: fp32 per blocksize2 (a power of two) entries.
 * Replaces the dequantize_blockwise + offset step at
 * qwen3_moe_fused/grouped_gemm/forward_4bit.py:149-153 (a bitsandbytes call there). */
int moe_absmax_unnest(const uint8_t* q, const float* code2, const float* absmax2, int blocksize2,
                      const float* offset, float* out, int64_t n, void* stream);

/* Stand-alone NF4 decode of n_elems weights (same format as above) to dtype_out.
 * Stands in for the bitsandbytes dequantize_4bit call at
 * qwen3_moe_fused/quantize/layer.py:21 and qwen3_moe_fused/kernels/fast_lora.py:62. */
int moe_nf4_dequant(const uint8_t* packed, const float* code, const float* absmax, int blocksize,
                    void* out, int64_t n_elems, int dtype_out, void* stream);

/* ---------------------------------------------------------------------------------
 * SiLU-mul.  Replaces qwen3_moe_fused/kernels/silu_mul.py:114-161.
 *   fwd:         h = dtype(silu_f32(e)) * g
 *   bwd:         de, dg from dh, e, g
 *   bwd_inplace: (dh, e, g) overwritten by (h, de, dg)
 * ------------------------------------------------------------------------------- */
int moe_silu_mul_fwd(const void* e, const void* g, void* h, int64_t n, int dtype, void* stream);
int moe_silu_mul_bwd(const void* dh, const void* e, const void* g, void* de, void* dg,
                     int64_t n, int dtype, void* stream);
int moe_silu_mul_bwd_inplace(void* dh, void* e, void* g, int64_t n, int dtype, void* stream);

/* ---------------------------------------------------------------------------------
 * Router: softmax over E logits in fp32, top-k (value descending, ties by ascending
 * expert id), optional renormalisation, weights rounded to dtype_w.
 * Replaces qwen3_moe_fused/modular_qwen3_moe_fused.py:87-93.
 *   logits (T,E) dtype_logits; weights (T,k) dtype_w; experts (T,k) int64
 * ------------------------------------------------------------------------------- */
int moe_router_softmax_topk(const void* logits, int dtype_logits, int64_t T, int E, int k,
                            int norm_topk, void* weights, int dtype_w, int64_t* experts,
                            void* stream);

/* out[j,:] = hidden[sort_idx[j] / k, :]   (expand by k then gather, in one pass).
 * Replaces qwen3_moe_fused/modular_qwen3_moe_fused.py:95-103. */
int moe_gather_rows(const void* hidden, const int32_t* sort_idx, int k, void* out,
                    int64_t rows, int H, int dtype, void* stream);

/* The same rows as moe_gather_rows, written token by token through the inverse index:
 * out[inv_sort_idx[t*k + j], :] = hidden[t, :] for j < k.  Every token row is read once.
 * Replaces qwen3_moe_fused/modular_qwen3_moe_fused.py:95-103. */
int moe_expand_rows(const void* hidden, const int32_t* inv_sort_idx, int k, void* out,
                    int64_t tokens, int H, int dtype, void* stream);

/* out[t,:] = sum_j weights[t,j] * y[inv_sort_idx[t*k+j], :]  with the reference's
 * rounding (product and sum in fp32, one rounding to dtype).
 * Replaces qwen3_moe_fused/modular_qwen3_moe_fused.py:112-115. */
int moe_combine(const void* y, const int32_t* inv_sort_idx, const void* weights, void* out,
                int64_t T, int k, int H, int dtype, void* stream);

/* ---------------------------------------------------------------------------------
 * Expert parallelism over peer memory.  The reference has no multi-GPU path
 * (README.md:26 lists it as open); these entry points have no counterpart there.
 * A "group" is the run of rows that one source rank sent for one local expert.
 * ------------------------------------------------------------------------------- */

/* Rows sorted by expert (m_sizes[e] rows each, M in total, row_bytes each) are copied to
 * one destination per expert: row i of expert e goes to dst_ptrs[e] + i * row_bytes.
 * dst_limit (DEVICE array of E int32, may be NULL = no limits): a negative entry leaves the
 * expert's rows where they are (not part of this push); otherwise rows with i >= dst_limit[e]
 * would overrun the receiver's buffer: they are NOT written and, when `dropped` is given,
 * counted there (DEVICE int32, incremented once per dropped row; the caller clears and reads
 * it: a non-zero count means the receiver's results for those rows are missing).
 * dst_ptrs is a DEVICE array of E 64-bit addresses, 16-byte aligned, in this GPU's memory or
 * in a peer GPU's memory mapped into this process; the stores are plain global stores.  The
 * call neither waits for nor signals the receiver.  Rows are visited starting with expert
 * first_expert and wrapping around (ranks that start at different experts do not all write
 * to the same destination at once).  With src_index (M int32, may be NULL) sorted row r is
 * read from row src_index[r] / src_div of `rows`: passing the sort's gather index and k
 * pushes token rows without expanding them first.  max_ctas <= 0 picks a grid from the SM
 * count. */
int moe_ep_push_rows(const void* rows, int64_t M, int64_t row_bytes, const void* m_sizes,
                     int m_sizes_dtype, int E, const uint64_t* dst_ptrs,
                     const int32_t* dst_limit, int first_expert, const int32_t* src_index,
                     int src_div, int max_ctas, int32_t* dropped, void* stream);

/* Token-deduplicated dispatch: a token whose k experts live on r distinct ranks is sent r times,
 * not k times.  Step 1, bookkeeping (one launch): selected holds T * k expert ids (token-major,
 * int32/int64); expert e lives on rank e / (E / world).  pos[t * world + d] (DEVICE int32) = number of
 * earlier tokens of this rank that also have an expert on rank d, or -1 if token t has none there;
 * n_tokens[d] = tokens with an expert on d (what the ranks exchange to lay out their token buffers). */
int moe_ep_token_positions(const void* selected, int sel_dtype, int64_t T, int k, int E, int world,
                           int32_t* pos, int32_t* n_tokens, void* stream);

/* Step 2: tokens (T rows of row_bytes) are copied to slot pos[t * world + d] + slot_base[d] of rank
 * d's token buffer (dst_ptrs[d], DEVICE array of `world` addresses; slot_base: DEVICE int32 per rank,
 * NULL = zeros: where this rank's tokens start on rank d) wherever pos is not negative.  Slots >=
 * slot_limit would overrun the receiver: not written, counted in `dropped` (may be NULL).
 * Destinations are visited starting with first_rank. */
int moe_ep_push_tokens(const void* tokens, int64_t T, int64_t row_bytes, const int32_t* pos,
                       const int32_t* slot_base, int world, int first_rank, const uint64_t* dst_ptrs,
                       int slot_limit, int max_ctas, int32_t* dropped, void* stream);

/* Step 3: for every expanded row r (sorted by expert, m_sizes[e] rows per expert, M in total;
 * sort_idx[r] / k is its token) the slot of its token on the rank that owns its expert is stored as
 * one int32 at dst_ptrs[e] + 4 i, i = position of r among the rows of e: the same addressing as
 * moe_ep_push_rows with 4-byte rows.  dst_limit / dropped as there.  The owner reads its rows as
 * tokens[index[row]]. */
int moe_ep_push_index(const int32_t* pos, const int32_t* slot_base, int world, const int32_t* sort_idx,
                      int k, int64_t M, const void* m_sizes, int m_sizes_dtype, int E,
                      const uint64_t* dst_ptrs, const int32_t* dst_limit, int32_t* dropped, void* stream);

/* Owner's side of the token-deduplicated dispatch: out[r] = tokens[index[r]] for r < min(*n_rows,
 * max_rows); n_rows is a DEVICE int64 (the received row count of moe_ep_plan), so the call needs no
 * host read.  An index outside [0, token_rows) reads row 0. */
int moe_ep_expand_rows(const void* tokens, int64_t token_rows, int64_t row_bytes, const int32_t* index,
                       const int64_t* n_rows, int64_t max_rows, void* out, void* stream);

/* Row bookkeeping of one routing decision for the exchange above, in one launch.
 * counts (world, E) int32 on the device: rows of every rank per global expert (expert e lives on
 * rank e / (E / world)).  The plan covers local experts lo..hi-1 of every rank (0, E / world for
 * all).  Outputs, all on the device: send_row[E] (first row, in the owner's buffer, of this
 * rank's rows of expert e; 0 outside the range), send_ok[E] (1 inside the range), and for the
 * G = (hi - lo) * world groups this rank receives, ordered (local expert, slot j) with slot j
 * holding the rows of source rank (rank + 1 + j) % world: group_sizes[G], weight_index[G]
 * (local expert minus lo), group_src[G], return_row[G] (first row of the group in its source
 * rank's sorted order); local_m_sizes[hi - lo]; recv_rows[1]. */
int moe_ep_plan(const int32_t* counts, int world, int rank, int E, int lo, int hi,
                int64_t* send_row, int32_t* send_ok, int32_t* group_sizes, int32_t* weight_index,
                int64_t* group_src, int64_t* return_row, int32_t* local_m_sizes,
                int64_t* recv_rows, void* stream);

/* moe_grouped_gemm_fwd / moe_grouped_gemm_dx over G groups where group g multiplies by
 * weight slice weight_index[g] (NULL: slice g) of n_weights, and its output rows are
 * written from the address out_ptrs[g] on (DEVICE array of G 64-bit addresses, 16-byte
 * aligned, local or peer memory) instead of into one contiguous y: the epilogue's TMA
 * stores go straight to the rank that owns the tokens.  out_template is any 16-byte
 * aligned buffer of at least one output row (only its address seeds the tensor maps).
 * Tensor-core CTA-pair kernels only: bf16/fp16 in and out, N >= 192, workspace required;
 * MOE_ERR_UNSUPPORTED otherwise. */
int moe_grouped_gemm_fwd_scattered(const void* x, const void* w, const void* group_sizes,
                                   int group_sizes_dtype, const int32_t* weight_index,
                                   int n_weights, const uint64_t* out_ptrs, void* out_template,
                                   int64_t M, int N, int K, int G, int dtype_in, int dtype_out,
                                   void* ws, size_t ws_bytes, void* stream);
int moe_grouped_gemm_dx_scattered(const void* x, const void* w, const void* group_sizes,
                                  int group_sizes_dtype, const int32_t* weight_index,
                                  int n_weights, const uint64_t* out_ptrs, void* out_template,
                                  int64_t M, int N, int K, int G, int dtype_in, int dtype_out,
                                  void* ws, size_t ws_bytes, void* stream);

/* Diagnostics.  Every wait inside the tensor-core kernels is bounded; a wait that gave up
 * records (reason << 16 | CTA index) in a device-side word.  This call copies that word to
 * *flag_out (0 = no wait was ever abandoned) and optionally clears it.  It synchronises
 * the device, so it is meant for tests and post-mortems, not for the hot path.
 * No counterpart in the reference. */
int moe_debug_read_error(int* flag_out, int clear);

/* Diagnostic counter: how many times, since the library was loaded, a role of a tensor-core kernel
 * found the barrier of the tile ring complete before the tile id of its round was visible in shared
 * memory and had to wait for it (harmless, but worth knowing).  Synchronises the device.
 * No counterpart in the reference. */
int moe_debug_read_late_values(int* out);

/* Text describing the most recent host-side set-up failure on the calling thread (for
 * instance the driver's answer to a tensor-map encode), "" if there was none.
 * No counterpart in the reference. */
const char* moe_debug_last_detail(void);

#ifdef __cplusplus
}
#endif
#endif /* MOE_B200_H_ */
