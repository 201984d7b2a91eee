/* C ABI of libfvsdpa.so: the Wan DiT self-attention hot path for NVIDIA B200
 * (sm_100a).  Plain pointers and sizes only; every pointer that is not marked
 * "host" is a CUDA device pointer of the current device; `stream` is a
 * cudaStream_t / CUstream passed as void*.
 *
 * Each entry point names the reference interface (zaitrarrio/fastvideo-rs,
 * path inside that repository) it stands in for.
 *
 * Return convention (the reference's tri-state, rt/sdpa_rule.rs:441-454 and
 * rt/attn_dc.rs:225-237): FV_RAN (0) the kernel was launched, FV_DECLINED (1)
 * the call is outside what this library runs (caller falls to its next route
 * step; nothing was launched), negative = hard error, text in
 * fv_last_error().  Launches are asynchronous on `stream`; nothing here
 * synchronises except the functions that say so.  The caller owns every
 * buffer.  There is no CPU fallback: on a machine without an sm_100 device
 * every compute entry returns FV_ERR_NO_DEVICE.
 */
#ifndef FV_SDPA_H
#define FV_SDPA_H
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define FV_API __attribute__((visibility("default")))
#else
#define FV_API
#endif

#define FV_RAN 0
#define FV_DECLINED 1
#define FV_ERR_INVALID (-1)   /* bad argument (null pointer, negative size, misaligned pointer) */
#define FV_ERR_CUDA (-2)      /* a CUDA call failed */
#define FV_ERR_NO_DEVICE (-3) /* no sm_100 device is current */
#define FV_ERR_DEVICE_STATUS (-4) /* a kernel reported a bounded wait that ran out */
#define FV_ERR_NCCL (-5)

#define FV_MASK_NONE 0
#define FV_MASK_BLOCK_CAUSAL 1

#define FV_NORM_ACROSS_HEADS 0
#define FV_NORM_PER_HEAD 1

#define FV_MAX_SEGMENTS 16

/* Text of the calling thread's last error ("" if none).  Host pointer, valid until the next call. */
FV_API const char* fv_last_error(void);

/* Library version string (host pointer). */
FV_API const char* fv_version(void);

/* Reads and clears the current device's kernel status word.  Synchronises `stream`.
 * Returns FV_RAN when every kernel finished its waits, FV_ERR_DEVICE_STATUS when one
 * gave up (code in *code_out: 100 + role), FV_ERR_CUDA on a CUDA error.
 * The word is part of the library's module image (a file-scope __device__ array, zero at load): every
 * kernel of the library reports there, the two-pass call on built-in scratch included, and neither this
 * call nor any launch allocates for it. */
FV_API int fv_device_status(void* stream, int* code_out);

/* One line naming the kernel the calling thread's last successful call launched, with its launch shape
 * ("" before the first).  The first launch of each kind of kernel in a process also prints that line on
 * stderr (FV_LOG=0 silences it) -- the counterpart of the reference's log-once lines
 * (crates/fastvideo-cudarc/src/rt/attn.rs:306-310, rt/ops.rs:1385-1401). */
FV_API const char* fv_last_kernel(void);

/* The calling thread's NEXT attention launch (fv_sdpa_*, fv_sp_forward_bf16's passes are set by the handle itself)
 * leaves `sms` SMs without a CTA.  The attention kernel is persistent and a CTA of it fills an SM: a collective whose
 * copy kernels should run BESIDE the launch (an NCCL all-gather of the next keys under the pass over the local ones)
 * otherwise waits for the launch to end, or makes part of its CTAs start late.  0 .. 128; one launch only. */
FV_API int fv_hint_spare_sms(int sms);

/* Failure-path self-test: launches ONE CTA of one warp that waits, with a budget of `cycles` clock cycles
 * (1e3 .. 2e9), on a barrier nobody arrives at.  The wait runs out, the kernel records status 109 and
 * returns normally; the next fv_device_status then answers FV_ERR_DEVICE_STATUS.  Nothing traps and the
 * context stays usable: this is how a host checks its handling of a kernel that gave up.  No counterpart
 * in the reference (its debug build traps instead, crates/fastvideo-cudarc/src/rt/attn_dc.cu:89-105). */
FV_API int fv_selftest_wait_timeout(void* stream, long long cycles);

/* ---- dense / block-causal SDPA -------------------------------------------------
 * Replaces rt::attn_dc::dense_fwd (crates/fastvideo-cudarc/src/rt/attn_dc.rs:213-273)
 * and rt::attn::device_mma_sdpa_causal (crates/fastvideo-cudarc/src/rt/attn.rs:647-730),
 * the kernels rt::sdpa::sdpa (rt/sdpa.rs:141-164) reaches on a B200.
 *
 * q [bh, sq, 128], k and v [bh, sk, 128]: bf16, contiguous, 16-byte aligned.
 * out [bh, sq, 128]: bf16 when out_is_bf16 != 0, else f32.
 * scale: softmax scale (> 0), e.g. 1/sqrt(128).
 * mask_mode FV_MASK_BLOCK_CAUSAL: query row i (global index q_row0 + i) sees key j iff
 *   (tk <= tq && (window == 0 || tq - tk < window)) || tk < sink, t = index / block_tokens
 *   (rt/attn.rs:448-453).  Rows that see no key give zeros.
 * Declines: d != 128, bh/sq/sk == 0, sq or sk > INT32_MAX / 2.
 */
FV_API int fv_sdpa_dense_bf16(void* stream, const void* q, const void* k, const void* v, void* out, int out_is_bf16,
                       int bh, int sq, int sk, int d, float scale, int mask_mode, int block_tokens, int window,
                       int sink, int q_row0);

/* fv_sdpa_dense_bf16 with the head merge folded into the output store: q, k, v as above with bh = batch * heads
 * (head index fastest), out [batch, sq, heads * 128] -- the layout merge_heads produces
 * (crates/fastvideo-cudarc/src/rt/kernels/core.cu:430-443, rt/ops.rs:2373-2385) and the output projection reads, so
 * WanAttention::attend (crates/fastvideo-cudarc/src/wan/transformer.rs:180-192) needs no merge launch.
 * Same values as fv_sdpa_dense_bf16, bit for bit, in another order. */
FV_API int fv_sdpa_dense_merged_bf16(void* stream, const void* q, const void* k, const void* v, void* out,
                                     int out_is_bf16, int batch, int heads, int sq, int sk, int d, float scale,
                                     int mask_mode, int block_tokens, int window, int sink, int q_row0);

/* ---- split-KV: a short query block against a long key window ----------------------
 * The shape of Plan::kv_window (crates/fastvideo-cudarc/src/rt/sdpa.rs:122-133, :300-326): the causal Wan caller
 * (crates/fastvideo-cudarc/src/wan/transformer.rs:250-313, wan/causal.rs) attends one block of frames (e.g. 4 680
 * rows) to the cached window (up to 32 760 keys), unmasked.  Such a launch fills the GPU a non-integer number of
 * times; cutting each head's keys into `splits` equal ranges that run side by side and merging the parts by their
 * log-sum-exp evens that out.  Same result as fv_sdpa_dense_bf16 up to f32 rounding of the merge.
 *
 * fv_sdpa_splitkv_choose: the number of ranges (1 = do not split, else 2..8, always a divisor of sk) a cost model
 *   picks for this shape on a GPU with sm_count SMs.
 * fv_sdpa_splitkv_workspace_bytes: bytes of caller-owned device workspace for `splits` ranges (0 for bad arguments).
 * fv_sdpa_splitkv_bf16: q [bh, sq, 128], k and v [bh, sk, 128] bf16; out [bh, sq, 128], or with out_heads = h > 0
 *   the merged-heads layout [bh / h, sq, h * 128]; bf16 or f32.  splits in 2..8 with sk % splits == 0 (else an
 *   error).  Launches the attention kernel once over bh * splits planes and one merge kernel; nothing synchronises.
 */
FV_API int fv_sdpa_splitkv_choose(int bh, int sq, int sk, int sm_count);
FV_API size_t fv_sdpa_splitkv_workspace_bytes(int bh, int sq, int splits);
FV_API int fv_sdpa_splitkv_bf16(void* stream, const void* q, const void* k, const void* v, void* out, int out_is_bf16,
                                int bh, int sq, int sk, int d, float scale, int splits, int out_heads, void* workspace,
                                size_t workspace_bytes);

/* The general form behind fv_sdpa_dense_bf16, used by the sequence-parallel path.
 * K and V are `nseg` segments (nseg <= FV_MAX_SEGMENTS), segment s holding seg_len[s]
 * keys whose global indices start at seg_start[s]; segment s of head h starts at element
 * ((s * bh + h) * seg_rows) * 128 of k / v (seg_rows >= every seg_len; rows between
 * seg_len[s] and seg_rows must hold finite values, e.g. zeros).
 * lse_out (optional, f32 [bh, sq]): log2-domain log-sum-exp of each row, -inf for a row
 *   that saw no key.
 * prev_o / prev_lse (optional, both or neither; f32 [bh, sq, 128] and [bh, sq]): the
 *   normalised result and lse of an earlier call over a disjoint key set; the output is
 *   then the exact softmax over the union of both key sets.
 * seg_len / seg_start are host pointers. */
FV_API int fv_sdpa_segments_bf16(void* stream, const void* q, const void* k, const void* v, void* out, int out_is_bf16,
                          int bh, int sq, int nseg, const int* seg_len, const int* seg_start, int seg_rows,
                          float scale, int mask_mode, int block_tokens, int window, int sink, int q_row0,
                          float* lse_out, const float* prev_o, const float* prev_lse);

/* fv_sdpa_segments_bf16 for a query shard made of TWO runs of the sequence: rows [0, q_split) have global
 * indices q_row0 + i, rows [q_split, sq) have q_row1 + (i - q_split) (q_split = 0: one run).  This is the
 * shard a rank holds under a zig-zag split of a causally masked sequence (an early and a late piece, so
 * that every rank sees about the same number of keys).  The reference shards contiguously only
 * (crates/fastvideo-cudarc/src/rt/sp.rs:16-28) and does not shard its block-causal route at all
 * (rt/sdpa_rule.rs:523-532). */
FV_API int fv_sdpa_segments_runs_bf16(void* stream, const void* q, const void* k, const void* v, void* out,
                                      int out_is_bf16, int bh, int sq, int nseg, const int* seg_len,
                                      const int* seg_start, int seg_rows, float scale, int mask_mode,
                                      int block_tokens, int window, int sink, int q_row0, int q_split, int q_row1,
                                      float* lse_out, const float* prev_o, const float* prev_lse);

/* Two-pass attention without any allocation -- no counterpart in the reference.
 *
 * For hosts that may not allocate device memory where they call attention: a serving loop with a fixed
 * memory budget, a real-time thread that must not take the allocator's device-wide synchronisation, a
 * runtime whose buffers all come from a pool sized at start-up.  The other entry points need scratch from
 * somewhere (the pass-1 result of a two-pass evaluation is a caller buffer; the split-KV parts are a caller
 * workspace).  This one computes the same thing as fv_sdpa_segments_bf16
 * called twice -- pass 1 over the local keys (k_local / v_local: one segment of local_len keys starting at
 * global index local_start, local_rows rows per head in memory), pass 2 over the gathered segments
 * (k_all / v_all as in fv_sdpa_segments_bf16; give the local segment length 0 there) merging pass 1 -- and
 * keeps the pass-1 result (f32 [bh, sq, 128] + [bh, sq]) in a fixed array inside the library.  A bounded wait
 * that runs out inside it is reported through fv_device_status like any other.  It calls no cudaMalloc, cudaFree or other allocating routine.
 *   Limit: bh * sq <= 65 024 rows (the array is about 32 MiB per GPU, held until the process exits);
 *     larger calls return FV_ERR_INVALID with the numbers in fv_last_error().
 *   remote_ready_event: optional cudaEvent_t; pass 2 waits for it on `stream` (record it after the K/V
 *     all-gather on the communication stream), so pass 1 overlaps the exchange.
 *   The first call on each device looks up the array's device address (cudaGetSymbolAddress, with that
 *     device current); make that first call before any stream capture.
 *   Every call uses the same array: nothing in it has to start at zero (pass 1 writes every row that pass 2
 *     reads), the pass-1 area is simply overwritten.  Calls that overlap on one GPU (two streams, two threads) race on it -- serialise them.
 *   Dense only (no mask). */
FV_API int fv_sdpa_two_pass_noalloc_bf16(void* stream, const void* q, const void* k_local, const void* v_local,
                                         int local_len, int local_start, int local_rows, const void* k_all,
                                         const void* v_all, int nseg, const int* seg_len, const int* seg_start,
                                         int seg_rows, void* out, int out_is_bf16, int bh, int sq, float scale,
                                         void* remote_ready_event);

/* ---- Wan q/k prologue -------------------------------------------------------------
 * Replaces the two CudaTensor::qk_norm_rope_bhsd launches and the split_heads_bhsd launch of
 * WanAttention::forward_self (crates/fastvideo-cudarc/src/wan/transformer.rs:163-178,287-289;
 * rt/fused.rs:193-330; host twin rt/ops.rs:2304-2371) by one pass.
 *
 * proj [batch, seq, width] bf16: the (fused) projection; q, k and v occupy columns
 *   [col_x, col_x + heads*128) of each row.  wq, wk f32 [heads*128]: RMSNorm weights.
 * cosv, sinv f32 [seq, 128] (both or neither; null = no rotation): the 3-D RoPE tables
 *   of fv_wan_rope_tables.  eps: RMSNorm epsilon (1e-6 for Wan).
 * norm_scope FV_NORM_ACROSS_HEADS: mean(x^2) over all heads*128 values of the row (Wan);
 *   FV_NORM_PER_HEAD: over one head's 128 values.
 * q_out, k_out, v_out [batch*heads, seq, 128] bf16; any may be null to skip it.
 * Declines: d != 128, heads > 64, empty sizes. */
FV_API int fv_wan_qk_prep_bf16(void* stream, const void* proj, int width, int col_q, int col_k, int col_v,
                               const float* wq, const float* wk, const float* cosv, const float* sinv, int batch,
                               int seq, int heads, int d, float eps, int norm_scope, void* q_out, void* k_out,
                               void* v_out);

/* 3-D RoPE tables on the host: wan_rope_at (crates/fastvideo-cudarc/src/wan/transformer.rs:447-544).
 * (ppf, pph, ppw): the token grid in patches; rows are tokens frame-major then height then width,
 * each row [t | h | w] with h = w = 2*(d/6) and t = d - h - w (44/42/42 at d = 128).
 * cos_host, sin_host: host arrays [ppf*pph*ppw, d] f32.  No GPU needed. */
FV_API int fv_wan_rope_tables(int ppf, int pph, int ppw, int d, double theta, int start_frame, float* cos_host,
                              float* sin_host);

/* ---- video sparse attention (VSA) ------------------------------------------------------
 * rt::vsa (crates/fastvideo-cudarc/src/rt/vsa.rs): TilePlan (:39-109), topk_for (:34-37),
 * vsa_attention_device (:358-470) with its launchers (rt/ops.rs:811-923,1074-1383,1554-1619;
 * rt/attn_dc.rs:275-604); arithmetic of the host twin vsa_attention_host (rt/vsa.rs:116-262). */

/* ---- the causal K/V cache's device work (Self-Forcing inference) ---------------------------------------
 * fv_wan_qk_prep_cache_bf16 is fv_wan_qk_prep_bf16 whose K and V land in the cache: k_cache / v_cache are
 * [batch * heads, cache_rows, 128] bf16 and token s of the block is written at row cache_row0 + s (q_out stays
 * [batch * heads, seq, 128]).  It replaces the prologue plus the two copy_tokens launches with which the
 * reference appends a block to its cache (crates/fastvideo-cudarc/src/wan/causal.rs:194-236,541-628; caller
 * wan/transformer.rs:290-313).  Errors: block does not fit the cache.
 *
 * fv_wan_rope_bhsd rotates n rows of every plane with Wan's interleaved-pair RoPE: source rows
 * [src_row0, src_row0 + n) of planes of src_plane_rows rows, table rows 0 .. n-1 (cos, sin f32 [n, 128], each
 * value twice), destination rows [dst_row0, dst_row0 + n) of planes of dst_plane_rows rows; source and
 * destination bf16 or f32 each; negate_sin rotates back.  One launch in place of rope_bhsd_f32 + quantize_bf16 +
 * copy_tokens of KvRope::RebasedSink (wan/causal.rs:246-275,734-812): un-roped copy of the sink = (cache K bf16,
 * own tables, negate_sin = 1) -> f32 buffer; re-roped sink = (that buffer, the target frames' tables) -> cache K rows
 * [0, sink).  Arithmetic of the host twin apply_rotary_bshd (rt/ops.rs:1903-1933): products and sums rounded
 * separately, one rounding to bf16.  Source and destination may be the same rows.  Declines: empty sizes. */
FV_API int fv_wan_qk_prep_cache_bf16(void* stream, const void* proj, int width, int col_q, int col_k, int col_v,
                                     const float* wq, const float* wk, const float* cosv, const float* sinv, int batch,
                                     int seq, int heads, int d, float eps, int norm_scope, void* q_out, void* k_cache,
                                     void* v_cache, int cache_rows, int cache_row0);
FV_API int fv_wan_rope_bhsd(void* stream, const void* src, int src_is_bf16, int src_plane_rows, int src_row0,
                            const float* cosv, const float* sinv, int negate_sin, int planes, int n, void* dst,
                            int dst_is_bf16, int dst_plane_rows, int dst_row0);

/* The cache's host arithmetic and its roll.
 * fv_kv_plan is KvSpec::plan (crates/fastvideo-cudarc/src/wan/causal.rs:289-336): for a block of n tokens that starts
 * at token current_start of the rollout and a cache in state (global_end, local_end_prev) it gives the rows the
 * block is written to [local_start, local_end), the rows dropped after the sink first (evicted) and the first row
 * the block's queries read (window_start); the reference's errors (a global window asked for more frames than it
 * keeps, a block before the cache start, a write past the cache) are FV_ERR_INVALID with the reference's text.
 * fv_kv_roll moves rows [sink + evicted, local_end_prev) of every plane of a [planes, cache_rows, 128] cache
 * (elem_bytes 2 or 4) down to row sink, in chunks that do not overlap (shift_tokens_down, causal.rs:236-249).
 * fv_sdpa_window_bf16 is Plan::kv_window over such a cache (rt/sdpa.rs:122-133,300-326; wan/transformer.rs:290-313):
 * unmasked attention of q [bh, sq, 128] over rows [window_start, window_start + window_len) of k_cache / v_cache
 * [bh, cache_rows, 128] bf16, read in place (no narrow + copy); out_heads as in fv_sdpa_dense_merged_bf16 (0: BHSD). */
typedef struct fv_kv_spec {
    int frame_tokens;   /* tokens per latent frame */
    int capacity;       /* rows of a cache plane */
    int sink;           /* rows kept at the head when the cache rolls */
    int max_attention;  /* keys a block reads, back from its end */
    int rolling;        /* 1: local_attn_size given, the cache rolls; 0: a clip longer than the window is an error */
} fv_kv_spec;
typedef struct fv_kv_move {
    long long evicted, local_start, local_end, window_start;
} fv_kv_move;
FV_API int fv_kv_plan(const fv_kv_spec* spec, long long global_end, long long local_end_prev, long long current_start,
                      long long n, fv_kv_move* out);
FV_API int fv_kv_roll(void* stream, void* cache, int elem_bytes, int planes, int cache_rows, int sink, int evicted,
                      int local_end_prev);
FV_API int fv_sdpa_window_bf16(void* stream, const void* q, const void* k_cache, const void* v_cache, void* out,
                               int out_is_bf16, int bh, int sq, int cache_rows, int window_start, int window_len, int d,
                               float scale, int out_heads);

/* ---- operand rounding for f32-stored activations ------------------------------------------------
 * The reference rounds q, k, v to bf16 before its attention kernels under bf16 activations and rounds the
 * result again (act16_operands and the tail of dense, crates/fastvideo-cudarc/src/rt/sdpa.rs:167-181,184-214:
 * three cast launches before, one after).  A host whose tensors are f32 enters here:
 * fv_act16_operands rounds all three operands (RNE) in ONE launch into caller-provided bf16 buffers
 * (q_count and kv_count are value counts; k and v have kv_count each); the attention entries then run on
 * those; fv_act16_widen widens a bf16 result back to f32 storage, so the values the host sees are the
 * bf16-rounded ones the reference returns.  Pointers 16-byte aligned.  Declines: empty sizes. */
FV_API int fv_act16_operands(void* stream, const float* q, const float* k, const float* v, long long q_count,
                             long long kv_count, void* q16, void* k16, void* v16);
FV_API int fv_act16_widen(void* stream, const void* src16, long long count, float* dst);

/* ---- the block glue either side of self-attention (bf16 activations) ---------------------------------
 * e: the block's AdaLN table, f32 [batch, e_rows, dim] (6 rows in Wan: shift/scale/gate of attention and FFN);
 * hidden rows are [batch * seq, dim] bf16, dim a multiple of 8, at most 6 144.  Both are one pass over HBM: a
 * row is read once and kept in registers for both LayerNorm statistics.
 *
 * fv_wan_ln_adaln_bf16 replaces CudaTensor::ln_adaln_e under bf16 activations
 *   (crates/fastvideo-cudarc/src/rt/fused.rs:20-70 -> rt/act16.rs:253-275, kernel rt/kernels/act16.cu:184-209;
 *   the call before attention, wan/transformer.rs:949-953):
 *   out = bf16( (x - mean) * rsqrt(var + eps) * (1 + e[b, scale_slot]) + e[b, shift_slot] ), f32 statistics.
 * fv_wan_self_residual_norm_bf16 replaces wan::fuse::self_residual_norm (crates/fastvideo-cudarc/src/wan/fuse.rs:
 *   108-166, kernel wan/kernels/block.cu:54-78 with res_mode 0 / ln_mode 0; the call after attention,
 *   wan/transformer.rs:959-971): s = hidden + attn * e[b, gate_slot] in f32 (product and sum rounded separately);
 *   hidden_out = bf16(s); normed_out = bf16( LN(s) * norm_w + norm_b ) with the statistics of the UNROUNDED s
 *   (FastVideo's rounding points).  norm_w, norm_b f32 [dim].
 * Declines: dim not a multiple of 8 or above 6 144, empty sizes. */
FV_API int fv_wan_ln_adaln_bf16(void* stream, const void* x, const float* e, int scale_slot, int shift_slot, int batch,
                                int seq, int dim, int e_rows, float eps, void* out);
FV_API int fv_wan_self_residual_norm_bf16(void* stream, const void* hidden, const void* attn, const float* e, int gate_slot,
                                          const float* norm_w, const float* norm_b, int batch, int seq, int dim, int e_rows,
                                          float eps, void* hidden_out, void* normed_out);

/* topk_for: clamp(ceil((1 - sparsity) * num_tiles), 1, num_tiles). */
FV_API int fv_vsa_topk_for(double sparsity, int num_tiles);

/* TilePlan::new for a (T, H, W) grid of patch tokens: 4x4x4 cubes of 64 slots, partial cubes at the
 * edges.  The plan is a host object; its tables are uploaded to the current device on first use. */
FV_API int fv_vsa_plan_create(int gt, int gh, int gw, void** plan_out);
FV_API int fv_vsa_plan_destroy(void* plan);
/* num_tiles, seq = T*H*W, padded = num_tiles*64, tiles = cubes along (T, H, W); any may be null. */
FV_API int fv_vsa_plan_info(void* plan, int* num_tiles, int* seq, int* padded, int tiles[3]);
/* Host copies: slot_src [padded] (-1 = padding), token_slot [seq], block_sizes [num_tiles]; any may be null. */
FV_API int fv_vsa_plan_host(void* plan, int32_t* slot_src, uint32_t* token_slot, uint32_t* block_sizes);
/* Uploads the plan's tables to the current device now (otherwise the first forward does). */
FV_API int fv_vsa_plan_upload(void* plan);
/* Bytes of caller-owned device workspace fv_vsa_forward_bf16 needs for (bh, topk); 0 on bad arguments. */
FV_API size_t fv_vsa_workspace_bytes(void* plan, int bh, int topk);

/* One VSA attention call.  q, k, v [bh, seq, 128] bf16 (q, k already normed and rotated); gate
 * [bh, seq, 128] bf16 or null (= ones): out = coarse * gate + fine, the reference's LINEAR gate
 * (rt/vsa.rs:252-256) -- a caller that wants a sigmoid gate applies it to the gate tensor first.
 * out [bh, seq, 128] bf16 or f32.  topk is clamped to [1, num_tiles].  workspace: device memory of at
 * least fv_vsa_workspace_bytes, 256-byte aligned, private to this call until it completes.
 * Optional device outputs for checks: selected_out u32 [bh, num_tiles, topk] (ASCENDING tile index;
 * the same set the reference's host picks, which emits by descending score), scores_out f32
 * [bh, num_tiles, num_tiles] (bit-identical to the host twin), coarse_out f32 [bh, num_tiles, 128].
 * Declines: more than 4096 tiles, shared memory of the fine kernel beyond the device limit. */
FV_API int fv_vsa_forward_bf16(void* stream, void* plan, const void* q, const void* k, const void* v,
                               const void* gate, int bh, int topk, float scale, void* out, int out_is_bf16,
                               void* workspace, size_t workspace_bytes, uint32_t* selected_out, float* scores_out,
                               float* coarse_out);

/* ---- the kernel-selection plugin ------------------------------------------------------
 * rt::sdpa_rule (crates/fastvideo-cudarc/src/rt/sdpa_rule.rs) as C: the Probe trait
 * (:321-350) becomes plain data, the enums keep their order, and one kernel is added:
 * FV_KERNEL_B200, this library's sm_100a kernel (seam value "b200"; the `auto` pick where
 * b200_loaded is set).  All functions are pure and run without a GPU. */
#define FV_BACKEND_DENSE 0
#define FV_BACKEND_CUBLAS 1
#define FV_BACKEND_FLASH 2
#define FV_BACKEND_HOST 3
#define FV_BACKEND_SPARSE 4

#define FV_KERNEL_V1 0
#define FV_KERNEL_V2 1
#define FV_KERNEL_V3 2
#define FV_KERNEL_V3S 3
#define FV_KERNEL_CUDNN 4
#define FV_KERNEL_DC 5
#define FV_KERNEL_B200 6

#define FV_STEP_RETIRED 0
#define FV_STEP_FLASH_F32 1
#define FV_STEP_SAGE 2
#define FV_STEP_MMA 3
#define FV_STEP_CUBLAS 4
#define FV_STEP_COMPOSED 5

#define FV_MMA_FIXED 0
#define FV_MMA_RULE 1
#define FV_MMA_TIMED 2

typedef struct fv_probe {
    int backend;            /* FASTVIDEO_SDPA, FV_BACKEND_* */
    int sp_world;           /* FASTVIDEO_SP_WORLD, >= 1 */
    int mma_default;        /* a bf16 tensor-core device is expected */
    int has_sage;           /* SageAttention2 on */
    int sage_min_seq;
    int fp8_dense;
    int causal_flash;       /* FASTVIDEO_WAN_CAUSAL_FLASH */
    char kernel_choice[32]; /* FASTVIDEO_FLASH_KERNEL / [kernels] dense_attention, lower case */
    int has_sm;             /* a device is present */
    int sm_major;
    int sms;
    int dc_loaded;          /* the reference's attn_dc module is loaded */
    int b200_loaded;        /* this library is loaded on a compute-capability 10.x device */
    int auto_timed;         /* FASTVIDEO_SDPA_AUTO=timed */
    int cudnn_has_plan;
} fv_probe;

typedef struct fv_step {
    int kind;     /* FV_STEP_* */
    int out_bf16; /* Sage, Mma */
    int retired;  /* Retired: the FV_BACKEND_* that was asked for */
} fv_step;

/* The settings and the current device as a probe (reads the FASTVIDEO_* variables each call;
 * without a device has_sm = 0, mma_default = 0, b200_loaded = 0).  Never fails. */
FV_API void fv_probe_live(fv_probe* out);
/* Defaults of a B200 with this library loaded and no variable set. */
FV_API void fv_probe_default(fv_probe* out);

FV_API int fv_rule_parse_backend(const char* v);
FV_API int fv_rule_parse_auto_timed(const char* v);
/* -1 when v is not a fixed kernel of the H3-VAE override (auto, dc, b200, anything else) */
FV_API int fv_rule_parse_kernel_override(const char* v);
FV_API int fv_rule_flash_v2_fills(size_t sq, size_t bh, size_t sms);
/* 0 = cuDNN, 1 = flash_mma_fwd2 */
FV_API int fv_rule_pick(int sm_major, size_t sq, size_t sk, size_t d);
/* dims_ok[0] is set when k == [b, h, sk, d] of q and v == k (Shape::of) */
FV_API void fv_rule_shape_of(const size_t q[4], const size_t k[4], const size_t v[4], size_t* sq, size_t* sk,
                             int* dims_ok);
/* Writes the route (at most 5 steps) and returns its length. */
FV_API int fv_rule_dense_route(const size_t q[4], const size_t k[4], const size_t v[4], int masked, int out_bf16,
                               const fv_probe* p, fv_step steps[8]);
FV_API int fv_rule_flash_kernel_for(size_t sq, size_t bh, size_t sms, const fv_probe* p);
/* Returns FV_MMA_*; *kernel gets the FV_KERNEL_* of Fixed and Rule, *sm_major that of Rule. */
FV_API int fv_rule_mma_kernel(const size_t q[4], const size_t k[4], const size_t v[4], int out_bf16,
                              const fv_probe* p, int* kernel, int* sm_major);
FV_API int fv_rule_fp8_first(const fv_probe* p);
FV_API int fv_rule_block_causal_first(const fv_probe* p);
FV_API int fv_rule_vdn_window_first(const fv_probe* p);
FV_API int fv_rule_kv_window_flash(int flash /* -1 unset */, const fv_probe* p);
FV_API int fv_rule_mma_sdpa_supported(size_t b, size_t h, size_t sq, size_t sk, size_t d, int sm_major);

/* ---- the one attention entry ----------------------------------------------------------
 * rt::sdpa::sdpa(q, k, v, &Plan) (crates/fastvideo-cudarc/src/rt/sdpa.rs:27-164) for bf16
 * BHSD operands on the device.  The plan says what the call computes; which kernel runs is
 * fv_rule_*'s choice from `probe` (null = fv_probe_live).  FV_RAN: this library's kernel ran
 * and `out` ([b, h, sq, d], bf16 when out_is_bf16 else f32) is being written on `stream`.
 * FV_DECLINED: the chosen step is not this library's (cuBLAS, composed, another kernel, an
 * additive mask, a head dim other than 128 ...): nothing was launched and the caller runs that
 * step itself.  Errors: rank / shape mismatch ("sdpa expects BHSD"), a retired backend. */
#define FV_PLAN_DENSE 0        /* Plan::dense / Plan::masked (mask may be set) */
#define FV_PLAN_COMPOSED 1     /* Plan::composed: never ours */
#define FV_PLAN_BLOCK_CAUSAL 2 /* Plan::block_causal */
#define FV_PLAN_VDN_WINDOW 3   /* Plan::vdn_window: never ours */
#define FV_PLAN_KV_WINDOW 4    /* Plan::kv_window / kv_window_with */

typedef struct fv_plan {
    int kind;
    int has_scale;    /* 0: scale = 1/sqrt(d) */
    float scale;
    int has_mask;     /* Dense / Composed: an additive [.., sq, sk] mask is present */
    int fp8_first;
    int block_tokens; /* BlockCausal */
    int window;
    int sink;
    int kv_flash;     /* KvWindow: -1 unset, 0, 1 */
} fv_plan;

FV_API int fv_sdpa(void* stream, const void* q, const void* k, const void* v, const size_t q_shape[4],
                   const size_t k_shape[4], const size_t v_shape[4], const fv_plan* plan, const fv_probe* probe,
                   void* out, int out_is_bf16);

/* fv_sdpa with a caller-owned device workspace.  fv_sdpa_ws_bytes gives the size this shape can use (0: none --
 * the call is then fv_sdpa).  With at least that many bytes, an unmasked plan (Plan::kv_window above all: a block of
 * frames against the cached window, crates/fastvideo-cudarc/src/wan/transformer.rs:250-313) whose grid would fill
 * the SMs a ragged number of times runs as fv_sdpa_splitkv_bf16.  A null or smaller workspace is not an error: the
 * call runs unsplit. */
FV_API size_t fv_sdpa_ws_bytes(const size_t q_shape[4], const size_t k_shape[4], const fv_plan* plan,
                               const fv_probe* probe);
FV_API int fv_sdpa_ws(void* stream, const void* q, const void* k, const void* v, const size_t q_shape[4],
                      const size_t k_shape[4], const size_t v_shape[4], const fv_plan* plan, const fv_probe* probe,
                      void* out, int out_is_bf16, void* workspace, size_t workspace_bytes);

/* ---- sequence-parallel split ------------------------------------------------------------
 * sp::shard_ranges (crates/fastvideo-cudarc/src/rt/sp.rs:16-28): contiguous shards, the
 * remainder going to the low ranks.  start and len are host arrays of `world` ints. */
FV_API void fv_shard_ranges(int seq, int world, int* start, int* len);

/* ---- sequence-parallel attention, one handle per rank ---------------------------------------
 * Replaces dispatch_sharded_multi_gpu (crates/fastvideo-cudarc/src/rt/sdpa.rs:354-410: K/V replicated on
 * every rank, outputs gathered through the host) by: contiguous token shards of q, k, v on every rank
 * (fv_shard_ranges), ONE exchange per call -- an NCCL all-gather of the bf16 K and V shards into this rank's
 * own HBM on a high-priority stream of the handle -- overlapped with attention over the local keys, then a
 * second pass over the other ranks' keys that merges the first by log-sum-exp.  The output stays sharded.
 * One rank per GPU (a process or a thread with that GPU current).  NCCL is looked up at run time
 * (libnccl.so.2); without it the calls that need it return FV_ERR_NCCL.
 *
 * fv_sp_unique_id: 128 bytes (an ncclUniqueId) that rank 0 makes and hands to every rank by the host's own
 *   means.  Host pointer.
 * fv_sp_create: collective over the `world` ranks (ncclCommInitRank), world <= FV_MAX_SEGMENTS; allocates the
 *   handle's buffers on the current device (gathered K/V: 2 * world * bh * seg_rows * 256 bytes; the first
 *   pass' f32 result; a zero-padded copy of the shard when shards are uneven).  groups <= 0: the heads are
 *   exchanged in 2 groups from 8 ranks on, else 1 (the second pass of a group starts when that group has
 *   arrived).  world == 1 needs neither an id nor NCCL.  unique_id: host pointer.
 * fv_sp_info: this rank's first token, its shard length, the longest shard, the head groups.
 * fv_sp_forward_bf16: q, k, v [bh, len, 128] bf16 shards of this rank, out [bh, len, 128] bf16 or f32.
 *   mask_mode FV_MASK_BLOCK_CAUSAL applies the mask of fv_sdpa_dense_bf16 over GLOBAL token indices; shards no
 *   row of this rank can see are left out of the second pass.  An error return from one rank alone (a null
 *   operand, a handle used on another device) happens before that rank joins the exchange: the other ranks'
 *   gathers then never complete, so treat it as fatal for the communicator (destroy the handles).  Asynchronous on `stream` (on return `stream`
 *   is ordered after the exchange, so k and v may be rewritten by later work on it); calls on one handle must
 *   be issued in the same order on every rank and from one stream at a time.  A rank without rows (more ranks
 *   than tokens) still calls: it takes part in the exchange and computes nothing (its operands may be null).
 * fv_sp_destroy: frees the handle (synchronise the streams that used it first).
 */
/* The segment lengths fv_sp_forward_bf16 gives its second pass on `rank` (host arithmetic only, no device needed):
 * lens_out[r] (host, `world` ints) = the shard length of rank r if some row of `rank` can see one of its keys under
 * the mask, else 0; 0 for `rank` itself. */
FV_API int fv_sp_second_pass_lens(int seq, int world, int rank, int mask_mode, int block_tokens, int window, int sink,
                                  int* lens_out);
FV_API int fv_sp_unique_id(void* id_out_128_bytes);
FV_API int fv_sp_create(const void* unique_id, int world, int rank, int seq, int bh, int groups, void** sp_out);
/* fv_sp_create with an explicit rendezvous deadline: a rank that waits longer than timeout_seconds for the
 * others gives the communicator up (ncclCommAbort) and returns FV_ERR_NCCL instead of blocking for ever;
 * timeout_seconds <= 0 uses NCCL's own blocking rendezvous.  fv_sp_create uses FV_SP_INIT_TIMEOUT_S (default
 * 120).  After the rendezvous the ranks compare (seq, bh, groups, world): a rank created with other numbers
 * makes every rank return FV_ERR_INVALID here, not hang in the first exchange.  The reference has no
 * rendezvous at all (its ranks are threads of one process, crates/fastvideo-cudarc/src/rt/sdpa.rs:371-410). */
FV_API int fv_sp_create_timeout(const void* unique_id, int world, int rank, int seq, int bh, int groups,
                                double timeout_seconds, void** sp_out);
FV_API int fv_sp_info(void* sp, int* start, int* len, int* seg_rows, int* groups);
FV_API int fv_sp_forward_bf16(void* sp, void* stream, const void* q, const void* k, const void* v, void* out,
                              int out_is_bf16, float scale, int mask_mode, int block_tokens, int window, int sink);
FV_API int fv_sp_destroy(void* sp);

#ifdef __cplusplus
}
#endif
#endif /* FV_SDPA_H */
