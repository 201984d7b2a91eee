// Entry kernels and host launcher of the head-dim-128 SDPA forward.
#include "sdpa_fwd.cuh"
#include "sdpa_fwd64.cuh"
#include "fv_runtime.h"
#include <math.h>
#include <stdlib.h>
#include <mutex>

namespace fvsdpa {

constexpr int kStages = 4;

// One entry per softmax variant (see sdpa_body); FV_SDPA_VARIANT picks one at run time for A/B timing,
// kDefaultVariant otherwise.
template <int VAR, bool MASKED, bool SPLITP = false>
__global__ void __launch_bounds__(kThreads, 1)
fv_sdpa_fwd_d128(const __grid_constant__ CUtensorMap tq, const __grid_constant__ CUtensorMap tk,
                 const __grid_constant__ CUtensorMap tv, const __grid_constant__ Params p) {
#if defined(__CUDA_ARCH_FEAT_SM100_ALL) || defined(__CUDA_ARCH_FEAT_SM103_ALL)
    extern __shared__ __align__(1024) unsigned char fv_smem[];
    sdpa_body<kStages, VAR, MASKED, SPLITP>(&tq, &tk, &tv, p, fv_smem);
#endif
}

// The double-buffered-S schedule (sdpa_fwd64.cuh); variants 100 + VAR.
template <int VAR, bool MASKED>
__global__ void __launch_bounds__(kThreads, 1)
fv_sdpa_fwd64_d128(const __grid_constant__ CUtensorMap tq, const __grid_constant__ CUtensorMap tk,
                   const __grid_constant__ CUtensorMap tv, const __grid_constant__ Params p) {
#if defined(__CUDA_ARCH_FEAT_SM100_ALL) || defined(__CUDA_ARCH_FEAT_SM103_ALL)
    extern __shared__ __align__(1024) unsigned char fv_smem[];
    sdpa_body64<kStages, VAR, MASKED>(&tq, &tk, &tv, p, fv_smem);
#endif
}

// 213 = softmax mix 13 (packed f32x2 arithmetic + a quarter of the exponentials of unmasked tiles on the FMA pipe +
// three-input max) with P handed over in two halves: the fastest of the mixes measured
// on B200 (A/B with FV_SDPA_VARIANT and the native checker's --bench mode).
constexpr int kDefaultVariant = 213;
typedef void (*KernelFn)(const CUtensorMap, const CUtensorMap, const CUtensorMap, const Params);
static KernelFn kernel_for(int var, bool masked) {
    switch (var) {
        case 213: return masked ? fv_sdpa_fwd_d128<13, true, true> : fv_sdpa_fwd_d128<13, false, true>;  // 13 + split P
        case 200: return masked ? fv_sdpa_fwd_d128<0, true, true> : fv_sdpa_fwd_d128<0, false, true>;     // 0 + split P
        case 100: return masked ? fv_sdpa_fwd64_d128<0, true> : fv_sdpa_fwd64_d128<0, false>;
        case 101: return masked ? fv_sdpa_fwd64_d128<1, true> : fv_sdpa_fwd64_d128<1, false>;
        case 1: return masked ? fv_sdpa_fwd_d128<1, true> : fv_sdpa_fwd_d128<1, false>;
        case 3: return masked ? fv_sdpa_fwd_d128<3, true> : fv_sdpa_fwd_d128<3, false>;
        case 5: return masked ? fv_sdpa_fwd_d128<5, true> : fv_sdpa_fwd_d128<5, false>;
        case 8: return masked ? fv_sdpa_fwd_d128<8, true> : fv_sdpa_fwd_d128<8, false>;
        case 9: return masked ? fv_sdpa_fwd_d128<9, true> : fv_sdpa_fwd_d128<9, false>;
        case 11: return masked ? fv_sdpa_fwd_d128<11, true> : fv_sdpa_fwd_d128<11, false>;
        case 13: return masked ? fv_sdpa_fwd_d128<13, true> : fv_sdpa_fwd_d128<13, false>;
        case 2: return masked ? fv_sdpa_fwd_d128<2, true> : fv_sdpa_fwd_d128<2, false>;
        case 64: return masked ? fv_sdpa_fwd_d128<64, true> : fv_sdpa_fwd_d128<64, false>;
        case 128: return masked ? fv_sdpa_fwd_d128<128, true> : fv_sdpa_fwd_d128<128, false>;
        case 256: return masked ? fv_sdpa_fwd_d128<256, true> : fv_sdpa_fwd_d128<256, false>;
        case 448: return masked ? fv_sdpa_fwd_d128<448, true> : fv_sdpa_fwd_d128<448, false>;
        case 960: return masked ? fv_sdpa_fwd_d128<960, true> : fv_sdpa_fwd_d128<960, false>;
        case 1472: return masked ? fv_sdpa_fwd_d128<1472, true> : fv_sdpa_fwd_d128<1472, false>;
        case 1984: return masked ? fv_sdpa_fwd_d128<1984, true> : fv_sdpa_fwd_d128<1984, false>;
        case 4032: return masked ? fv_sdpa_fwd_d128<4032, true> : fv_sdpa_fwd_d128<4032, false>;
        case 6080: return masked ? fv_sdpa_fwd_d128<6080, true> : fv_sdpa_fwd_d128<6080, false>;
        case 10176: return masked ? fv_sdpa_fwd_d128<10176, true> : fv_sdpa_fwd_d128<10176, false>;
        case 4: return masked ? fv_sdpa_fwd_d128<4, true> : fv_sdpa_fwd_d128<4, false>;
        case 12: return masked ? fv_sdpa_fwd_d128<12, true> : fv_sdpa_fwd_d128<12, false>;
        case 7: return masked ? fv_sdpa_fwd_d128<7, true> : fv_sdpa_fwd_d128<7, false>;
        case 32: return masked ? fv_sdpa_fwd_d128<32, true> : fv_sdpa_fwd_d128<32, false>;
        case 16: return masked ? fv_sdpa_fwd_d128<16, true> : fv_sdpa_fwd_d128<16, false>;
        case 24: return masked ? fv_sdpa_fwd_d128<24, true> : fv_sdpa_fwd_d128<24, false>;
        case 10: return masked ? fv_sdpa_fwd_d128<10, true> : fv_sdpa_fwd_d128<10, false>;
        default: return masked ? fv_sdpa_fwd_d128<0, true> : fv_sdpa_fwd_d128<0, false>;
    }
}
static int chosen_variant() {
    static int v = -1;
    if (v < 0) {
        const char* e = getenv("FV_SDPA_VARIANT");
        v = e ? atoi(e) : kDefaultVariant;
        if (v < 0 || v > 16383) v = kDefaultVariant;
    }
    return v;
}

static int launch(cudaStream_t stream, const void* q, const void* k, const void* v, void* out, int out_is_bf16, int bh,
                  int sq, int nseg, const int* seg_len, const int* seg_start, int seg_rows, float scale, int mask_mode,
                  int block_tokens, int window, int sink, int q_row0, float* lse_out, const float* prev_o,
                  const float* prev_lse, int* status_in = nullptr, int out_heads = 0) {
    int dev;
    int rc = fvrt::require_sm100(&dev);
    if (rc != FV_RAN) return rc;
    if (!q || !k || !v || !out) return fvrt::fail(FV_ERR_INVALID, "sdpa: null operand");
    if (((uintptr_t)q | (uintptr_t)k | (uintptr_t)v | (uintptr_t)out) & 15)
        return fvrt::fail(FV_ERR_INVALID, "sdpa: operands must be 16-byte aligned");
    if ((prev_o == nullptr) != (prev_lse == nullptr))
        return fvrt::fail(FV_ERR_INVALID, "sdpa: prev_o and prev_lse go together");
    if (prev_o && ((uintptr_t)prev_o & 15)) return fvrt::fail(FV_ERR_INVALID, "sdpa: prev_o must be 16-byte aligned");
    if (!(scale > 0.f) || !isfinite(scale)) return fvrt::fail(FV_ERR_INVALID, "sdpa: scale must be positive and finite");
    if (mask_mode != FV_MASK_NONE && mask_mode != FV_MASK_BLOCK_CAUSAL)
        return fvrt::fail(FV_ERR_INVALID, "sdpa: unknown mask mode %d", mask_mode);
    if (mask_mode == FV_MASK_BLOCK_CAUSAL && (block_tokens < 1 || window < 0 || sink < 0 || q_row0 < 0))
        return fvrt::fail(FV_ERR_INVALID, "sdpa: block-causal needs block_tokens >= 1, window, sink, q_row0 >= 0");
    if (nseg < 1 || nseg > kMaxSeg) return fvrt::fail(FV_ERR_INVALID, "sdpa: 1..%d K/V segments", kMaxSeg);

    Params p{};
    p.out = out;
    p.lse_out = lse_out;
    p.prev_o = prev_o;
    p.prev_lse = prev_lse;
    p.out_is_bf16 = out_is_bf16 ? 1 : 0;
    p.out_heads = out_heads;
    p.bh = bh;
    p.sq = sq;
    p.nqb = (sq + kRowsPerCta - 1) / kRowsPerCta;
    p.sl2 = scale * 1.4426950408889634f;
    p.nseg = nseg;
    long long total = 0;
    for (int s = 0; s < nseg; s++) {
        if (seg_len[s] < 0 || seg_len[s] > seg_rows || seg_start[s] < 0)
            return fvrt::fail(FV_ERR_INVALID, "sdpa: segment %d has length %d (rows %d), start %d", s, seg_len[s], seg_rows,
                              seg_start[s]);
        p.seg_len[s] = seg_len[s];
        p.seg_start[s] = seg_start[s];
        total += seg_len[s];
        if ((long long)seg_start[s] + seg_len[s] > 0x3fffffffll) return FV_DECLINED;
    }
    if (total == 0) return FV_DECLINED;
    p.mask_mode = mask_mode;
    p.block_tokens = block_tokens;
    p.window = window;
    p.sink = sink;
    p.q_row0 = q_row0;
    p.heavy_first = mask_mode == FV_MASK_BLOCK_CAUSAL;
    if (status_in) {
        p.status = status_in;
    } else {
        rc = fvrt::status_word(dev, &p.status);
        if (rc != FV_RAN) return rc;
    }

    const long long grid = (long long)p.nqb * bh;
    if (grid > 0x7fffffffll) return FV_DECLINED;

    CUtensorMap tq, tk, tv;
    {
        const uint64_t dq[4] = {128, (uint64_t)sq, (uint64_t)bh, 1};
        const uint64_t sqb[3] = {256, (uint64_t)sq * 256, (uint64_t)sq * 256 * bh};
        rc = fvrt::encode_map4(&tq, q, dq, sqb, 128);
        if (rc != FV_RAN) return rc;
        const uint64_t dk[4] = {128, (uint64_t)seg_rows, (uint64_t)bh, (uint64_t)nseg};
        const uint64_t skb[3] = {256, (uint64_t)seg_rows * 256, (uint64_t)seg_rows * 256 * bh};
        rc = fvrt::encode_map4(&tk, k, dk, skb, 128);
        if (rc != FV_RAN) return rc;
        rc = fvrt::encode_map4(&tv, v, dk, skb, 128);
        if (rc != FV_RAN) return rc;
    }

    static bool attr_set[8][16384][2] = {};
    constexpr uint32_t smem = smem_bytes<kStages>();
    const int var = chosen_variant();
    const bool masked = mask_mode != FV_MASK_NONE;
    const KernelFn fn = kernel_for(var, masked);
    {
        static std::mutex attr_mu;
        std::lock_guard<std::mutex> attr_lock(attr_mu);
        if (!attr_set[dev & 7][var][masked]) {
            FV_CUDA(cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
            attr_set[dev & 7][var][masked] = true;
        }
    }
    fn<<<(unsigned)grid, kThreads, smem, stream>>>(tq, tk, tv, p);
    FV_CUDA(cudaGetLastError());
    return FV_RAN;
}

// ---- built-in scratch for callers that cannot allocate ---------------------------------------------
// 256 bytes of status block, then the pass-1 result of the two-pass evaluation: kNoAllocMaxRows rows of
// 128 f32 and one f32 log-sum-exp per row.  Held by every GPU that loads the library until the process
// exits (about 32 MiB).
constexpr long long kNoAllocMaxRows = 65024;
constexpr size_t kNoAllocFloats = 64 + (size_t)kNoAllocMaxRows * (kD + 1);
static __device__ __align__(256) float fv_noalloc_scratch[kNoAllocFloats];
// In host code the array's name is only a stand-in: the device address comes from the runtime, once per
// device, with that device current.
static float* g_noalloc_ptr[64] = {};

static int noalloc_base(int dev, float** out) {
    if (!g_noalloc_ptr[dev]) {
        float* ptr = nullptr;
        cudaError_t e = cudaGetSymbolAddress((void**)&ptr, fv_noalloc_scratch);
        if (e != cudaSuccess || !ptr)
            return fvrt::fail(FV_ERR_CUDA, "cudaGetSymbolAddress(fv_noalloc_scratch) on device %d: %s", dev,
                              cudaGetErrorString(e));
        g_noalloc_ptr[dev] = ptr;
    }
    *out = g_noalloc_ptr[dev];
    return FV_RAN;
}

static int two_pass_noalloc(cudaStream_t stream, const void* q, const void* k_local, const void* v_local, int local_len,
                            int local_start, int local_rows, const void* k_all, const void* v_all, int nseg,
                            const int* seg_len, const int* seg_start, int seg_rows, void* out, int out_is_bf16, int bh,
                            int sq, float scale, cudaEvent_t remote_ready) {
    int dev;
    int rc = fvrt::require_sm100(&dev);
    if (rc != FV_RAN) return rc;
    const long long rows = (long long)bh * sq;
    if (rows > kNoAllocMaxRows)
        return fvrt::fail(FV_ERR_INVALID,
                          "sdpa two-pass (no allocation): bh*sq = %lld rows, the built-in scratch holds %lld; use "
                          "fv_sdpa_segments_bf16 with buffers of your own for larger calls", rows, kNoAllocMaxRows);
    float* base;
    rc = noalloc_base(dev, &base);
    if (rc != FV_RAN) return rc;
    int* status = reinterpret_cast<int*>(base);
    float* o1 = base + 64;
    float* lse1 = o1 + (size_t)kNoAllocMaxRows * kD;
    // The scratch keeps what the previous call left: the status word has to start at zero.
    FV_CUDA(cudaMemsetAsync(status, 0, 256, stream));
    rc = launch(stream, q, k_local, v_local, o1, 0, bh, sq, 1, &local_len, &local_start, local_rows, scale, FV_MASK_NONE,
                0, 0, 0, 0, lse1, nullptr, nullptr, status);
    if (rc != FV_RAN) return rc;
    if (remote_ready) FV_CUDA(cudaStreamWaitEvent(stream, remote_ready, 0));
    return launch(stream, q, k_all, v_all, out, out_is_bf16, bh, sq, nseg, seg_len, seg_start, seg_rows, scale,
                  FV_MASK_NONE, 0, 0, 0, 0, nullptr, o1, lse1, status);
}

}  // namespace fvsdpa

extern "C" int fv_sdpa_two_pass_noalloc_bf16(void* stream, const void* q, const void* k_local, const void* v_local,
                                             int local_len, int local_start, int local_rows, const void* k_all,
                                             const void* v_all, int nseg, const int* seg_len, const int* seg_start,
                                             int seg_rows, void* out, int out_is_bf16, int bh, int sq, float scale,
                                             void* remote_ready_event) {
    fvrt::clear_error();
    if (bh <= 0 || sq <= 0 || nseg <= 0 || seg_rows <= 0 || local_rows <= 0) return FV_DECLINED;
    if (!seg_len || !seg_start) return fvrt::fail(FV_ERR_INVALID, "sdpa: null segment table");
    return fvsdpa::two_pass_noalloc((cudaStream_t)stream, q, k_local, v_local, local_len, local_start, local_rows, k_all,
                                    v_all, nseg, seg_len, seg_start, seg_rows, out, out_is_bf16, bh, sq, scale,
                                    (cudaEvent_t)remote_ready_event);
}

extern "C" int fv_sdpa_segments_bf16(void* stream, const void* q, const void* k, const void* v, void* out,
                                     int out_is_bf16, int bh, int sq, int nseg, const int* seg_len,
                                     const int* seg_start, int seg_rows, float scale, int mask_mode, int block_tokens,
                                     int window, int sink, int q_row0, float* lse_out, const float* prev_o,
                                     const float* prev_lse) {
    fvrt::clear_error();
    if (bh <= 0 || sq <= 0 || nseg <= 0 || seg_rows <= 0) return FV_DECLINED;
    if (sq > 0x3fffffff || seg_rows > 0x3fffffff) return FV_DECLINED;
    if (!seg_len || !seg_start) return fvrt::fail(FV_ERR_INVALID, "sdpa: null segment table");
    return fvsdpa::launch((cudaStream_t)stream, q, k, v, out, out_is_bf16, bh, sq, nseg, seg_len, seg_start, seg_rows,
                          scale, mask_mode, block_tokens, window, sink, q_row0, lse_out, prev_o, prev_lse);
}

extern "C" int fv_sdpa_dense_bf16(void* stream, const void* q, const void* k, const void* v, void* out, int out_is_bf16,
                                  int bh, int sq, int sk, int d, float scale, int mask_mode, int block_tokens,
                                  int window, int sink, int q_row0) {
    fvrt::clear_error();
    if (d != 128 || bh <= 0 || sq <= 0 || sk <= 0) return FV_DECLINED;
    if (sq > 0x3fffffff || sk > 0x3fffffff) return FV_DECLINED;
    const int len = sk, start = 0;
    return fvsdpa::launch((cudaStream_t)stream, q, k, v, out, out_is_bf16, bh, sq, 1, &len, &start, sk, scale, mask_mode,
                          block_tokens, window, sink, q_row0, nullptr, nullptr, nullptr);
}

extern "C" int fv_sdpa_dense_merged_bf16(void* stream, const void* q, const void* k, const void* v, void* out,
                                         int out_is_bf16, int batch, int heads, int sq, int sk, int d, float scale,
                                         int mask_mode, int block_tokens, int window, int sink, int q_row0) {
    fvrt::clear_error();
    if (d != 128 || batch <= 0 || heads <= 0 || sq <= 0 || sk <= 0) return FV_DECLINED;
    if (sq > 0x3fffffff || sk > 0x3fffffff || (long long)batch * heads > 0x7fffffffll) return FV_DECLINED;
    const int len = sk, start = 0;
    return fvsdpa::launch((cudaStream_t)stream, q, k, v, out, out_is_bf16, batch * heads, sq, 1, &len, &start, sk, scale,
                          mask_mode, block_tokens, window, sink, q_row0, nullptr, nullptr, nullptr, nullptr, heads);
}
