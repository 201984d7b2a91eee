// Host-side runtime shared by the entry points: thread-local error text,
// device capability check, the per-device kernel status word, and the
// cuTensorMapEncodeTiled entry obtained from the driver at run time (the
// library links against cudart only).
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdarg.h>
#include "../../include/fv_sdpa.h"

namespace fvrt {

int fail(int code, const char* fmt, ...);   // sets the error text, returns code
void clear_error();
// FV_RAN when the current device is sm_100 / sm_103; else FV_ERR_NO_DEVICE (text set).
int require_sm100(int* device_out);
// Device pointer of the current device's status word.  The word lives in a file-scope __device__
// array of the library (zero when the module loads), so asking for it never allocates.
int status_word(int device, int** ptr_out);
// Number of SMs of `device` (cached).
int sm_count(int device, int* out);
// SMs the calling thread asked its next attention launch to leave free (fv_hint_spare_sms); cleared by the call.
int take_spare_sms();
// One line on stderr the first time `key` (a small integer per kernel kind) is seen in this
// process, like the reference's rt::log::info_once one-liners that name the kernel a call ran
// (crates/fastvideo-cudarc/src/rt/attn.rs:306-310).  FV_LOG=0 silences them.  The text of the last
// line of each thread is also kept for fv_last_kernel().
enum LogKey { kLogDense = 0, kLogCausal, kLogSplitKv, kLogPrep, kLogVsa, kLogSp, kLogGlue, kLogKeys };
void ran(LogKey key, const char* fmt, ...);

// 4-D bf16 tensor map, dims innermost first, strides in bytes for dims 1..3,
// box (64, box_rows, 1, 1), 128-byte swizzle, out-of-range reads as zero.
int encode_map4(CUtensorMap* map, const void* base, const uint64_t dims[4], const uint64_t strides[3],
                uint32_t box_rows);
// The same through a small per-process cache keyed by (base, dims, strides, box_rows): a denoising
// loop calls with the same buffers every step, and the reference re-encodes three maps per call
// (crates/fastvideo-cudarc/src/rt/attn_dc.rs:242-246).
int encode_map4_cached(CUtensorMap* map, const void* base, const uint64_t dims[4], const uint64_t strides[3],
                       uint32_t box_rows);

#define FV_CUDA(expr)                                                                           \
    do {                                                                                        \
        cudaError_t e__ = (expr);                                                               \
        if (e__ != cudaSuccess) return fvrt::fail(FV_ERR_CUDA, "%s: %s", #expr, cudaGetErrorString(e__)); \
    } while (0)

}  // namespace fvrt
