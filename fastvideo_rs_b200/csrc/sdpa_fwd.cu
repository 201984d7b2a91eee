// Entry kernels and host launcher of the head-dim-128 SDPA forward.
#include "sdpa_fwd.cuh"
#include "sdpa_fwd64.cuh"
#include "fv_runtime.h"
#include <cuda_bf16.h>
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
                  const float* prev_lse, int* status_in = nullptr, int out_heads = 0, int q_div = 1) {
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
    if (q_div < 1 || bh % q_div != 0) return fvrt::fail(FV_ERR_INVALID, "sdpa: %d planes do not split by %d", bh, q_div);

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
    p.q_div = q_div;
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
        const uint64_t qplanes = (uint64_t)(bh / q_div);
        const uint64_t dq[4] = {128, (uint64_t)sq, qplanes, 1};
        const uint64_t sqb[3] = {256, (uint64_t)sq * 256, (uint64_t)sq * 256 * qplanes};
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
    if (q_div > 1 && (var == 100 || var == 101)) return FV_DECLINED;  // the 64-key schedule has no split-KV form
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


// ---- split-KV: few query rows against a long key window ----------------------------------------------
// A block of 4 680 queries over a 32 760-key window fills 148 SMs 1.54 times: the second wave runs
// half empty.  Each head's keys are cut into `splits` equal ranges that run as planes of their own
// (k and v are only viewed as [bh * splits, sk / splits, 128]; q is read through q_div), every plane
// leaves a normalised f32 result and its log-sum-exp in the workspace, and one HBM-bound kernel merges
// them.  The merge is the two-pass formula of the epilogue applied to `splits` parts at once.
constexpr int kMaxSplits = 8;

template <int OUT16>
__global__ void __launch_bounds__(256)
fv_splitkv_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_lse, void* __restrict__ out,
                        int bh, int sq, int splits, int out_heads) {
    const long long row = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);  // one warp per (plane, query row)
    if (row >= (long long)bh * sq) return;
    const int lane = threadIdx.x & 31;
    const int h = (int)(row / sq), r = (int)(row % sq);
    float lse[kMaxSplits];
    float M = __int_as_float(0xff800000);
#pragma unroll
    for (int s = 0; s < kMaxSplits; s++) {
        lse[s] = s < splits ? part_lse[((size_t)h * splits + s) * sq + r] : __int_as_float(0xff800000);
        M = fmaxf(M, lse[s]);
    }
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    if (M != __int_as_float(0xff800000)) {
        float den = 0.f;
#pragma unroll
        for (int s = 0; s < kMaxSplits; s++) {
            lse[s] = s < splits ? exp2f(lse[s] - M) : 0.f;  // now the weight of part s
            den += lse[s];
        }
        const float inv = 1.f / den;
#pragma unroll
        for (int s = 0; s < kMaxSplits; s++) {
            if (s >= splits) break;
            const float w = lse[s] * inv;
            const float4 t = reinterpret_cast<const float4*>(part_o + (((size_t)h * splits + s) * sq + r) * kD)[lane];
            acc.x = fmaf(t.x, w, acc.x);
            acc.y = fmaf(t.y, w, acc.y);
            acc.z = fmaf(t.z, w, acc.z);
            acc.w = fmaf(t.w, w, acc.w);
        }
    }
    size_t ooff = (size_t)row * kD;
    if (out_heads > 0) ooff = (((size_t)(h / out_heads) * sq + r) * out_heads + h % out_heads) * kD;
    if (OUT16) {
        const __nv_bfloat162 lo = __floats2bfloat162_rn(acc.x, acc.y), hi = __floats2bfloat162_rn(acc.z, acc.w);
        reinterpret_cast<uint2*>(reinterpret_cast<unsigned short*>(out) + ooff)[lane] =
            make_uint2(*reinterpret_cast<const uint32_t*>(&lo), *reinterpret_cast<const uint32_t*>(&hi));
    } else {
        reinterpret_cast<float4*>(reinterpret_cast<float*>(out) + ooff)[lane] = acc;
    }
}

static size_t splitkv_bytes(long long bh, long long sq, int splits) {
    return (size_t)bh * splits * sq * (kD + 1) * sizeof(float);
}

// Estimated duration in microseconds of `splits` ranges on `sms` SMs: equal CTAs run in whole waves, a
// 256 x 128 tile step takes about 2 us, a CTA pays about 3 steps of fill and drain (4 with the f32
// store of a part), the merge moves (splits + 1) x the output at about 5 TB/s.
static double splitkv_cost(long long bh, long long sq, long long sk, int splits, int sms) {
    const long long nqb = (sq + kRowsPerCta - 1) / kRowsPerCta;
    const long long waves = (nqb * bh * splits + sms - 1) / sms;
    const long long tiles = (sk / splits + kBN - 1) / kBN;
    double us = (double)waves * (double)(tiles + (splits > 1 ? 4 : 3)) * 2.0;
    if (splits > 1) us += 3.0 + (double)bh * sq * kD * 4.0 * (splits + 1) / 5.0e6;
    return us;
}

static int splitkv_choose(long long bh, long long sq, long long sk, int sms) {
    if (bh <= 0 || sq <= 0 || sk <= 0 || sms <= 0) return 1;
    int best = 1;
    double best_us = splitkv_cost(bh, sq, sk, 1, sms);
    for (int s = 2; s <= kMaxSplits; s++) {
        if (sk % s != 0 || sk / s < 4 * kBN || bh * s > 0x7fffffffll) continue;
        const double us = splitkv_cost(bh, sq, sk, s, sms);
        if (us < 0.93 * best_us) {  // a split has to pay for itself by more than the model's error (a few per cent)
            best = s;
            best_us = us;
        }
    }
    return best;
}

static int splitkv(cudaStream_t stream, const void* q, const void* k, const void* v, void* out, int out_is_bf16, int bh,
                   int sq, int sk, float scale, int splits, int out_heads, void* workspace, size_t workspace_bytes) {
    if (splits < 2 || splits > kMaxSplits) return fvrt::fail(FV_ERR_INVALID, "split-KV: 2..%d splits", kMaxSplits);
    if (sk % splits != 0) return fvrt::fail(FV_ERR_INVALID, "split-KV: %d keys do not divide into %d ranges", sk, splits);
    if ((long long)bh * splits > 0x7fffffffll) return FV_DECLINED;
    if (out_heads < 0 || (out_heads > 0 && bh % out_heads != 0))
        return fvrt::fail(FV_ERR_INVALID, "split-KV: %d planes are not whole batches of %d heads", bh, out_heads);
    const size_t need = splitkv_bytes(bh, sq, splits);
    if (!workspace || workspace_bytes < need)
        return fvrt::fail(FV_ERR_INVALID, "split-KV: workspace of %zu bytes, %zu needed", workspace_bytes, need);
    if (((uintptr_t)workspace | (uintptr_t)out) & 15) return fvrt::fail(FV_ERR_INVALID, "split-KV: buffers must be 16-byte aligned");
    float* part_o = static_cast<float*>(workspace);
    float* part_lse = part_o + (size_t)bh * splits * sq * kD;
    const int len = sk / splits, start = 0;
    // The key index only matters under a mask; split-KV is unmasked, so every range may start at 0.
    int rc = launch(stream, q, k, v, part_o, 0, bh * splits, sq, 1, &len, &start, len, scale, FV_MASK_NONE, 0, 0, 0, 0,
                    part_lse, nullptr, nullptr, nullptr, 0, splits);
    if (rc != FV_RAN) return rc;
    const long long rows = (long long)bh * sq;
    const unsigned grid = (unsigned)((rows + 7) / 8);
    if (out_is_bf16)
        fv_splitkv_merge_kernel<1><<<grid, 256, 0, stream>>>(part_o, part_lse, out, bh, sq, splits, out_heads);
    else
        fv_splitkv_merge_kernel<0><<<grid, 256, 0, stream>>>(part_o, part_lse, out, bh, sq, splits, out_heads);
    FV_CUDA(cudaGetLastError());
    return FV_RAN;
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

extern "C" int fv_sdpa_splitkv_choose(int bh, int sq, int sk, int sm_count) {
    return fvsdpa::splitkv_choose(bh, sq, sk, sm_count);
}

extern "C" size_t fv_sdpa_splitkv_workspace_bytes(int bh, int sq, int splits) {
    if (bh <= 0 || sq <= 0 || splits < 2 || splits > fvsdpa::kMaxSplits) return 0;
    return fvsdpa::splitkv_bytes(bh, sq, splits);
}

extern "C" int fv_sdpa_splitkv_bf16(void* stream, const void* q, const void* k, const void* v, void* out,
                                    int out_is_bf16, int bh, int sq, int sk, int d, float scale, int splits,
                                    int out_heads, void* workspace, size_t workspace_bytes) {
    fvrt::clear_error();
    if (d != 128 || bh <= 0 || sq <= 0 || sk <= 0) return FV_DECLINED;
    if (sq > 0x3fffffff || sk > 0x3fffffff) return FV_DECLINED;
    return fvsdpa::splitkv((cudaStream_t)stream, q, k, v, out, out_is_bf16, bh, sq, sk, scale, splits, out_heads,
                           workspace, workspace_bytes);
}
