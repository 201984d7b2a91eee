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

#define FV_MAX_SEGMENTS 8

/* Text of the calling thread's last error ("" if none).  Host pointer, valid until the next call. */
FV_API const char* fv_last_error(void);

/* Library version string (host pointer). */
FV_API const char* fv_version(void);

/* Reads and clears the current device's kernel status word.  Synchronises `stream`.
 * Returns FV_RAN when every kernel finished its waits, FV_ERR_DEVICE_STATUS when one
 * gave up (code in *code_out: 100 + role), FV_ERR_CUDA on a CUDA error. */
FV_API int fv_device_status(void* stream, int* code_out);

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

#ifdef __cplusplus
}
#endif
#endif /* FV_SDPA_H */
