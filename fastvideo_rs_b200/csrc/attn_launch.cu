// Kernels, host launcher and C entries of the head-dim-128 attention forward (attn_fwd.cuh):
// the dense / block-causal / segmented call, the two-pass call on built-in scratch, and split-KV.
#include "attn_fwd.cuh"
#include "fv_runtime.h"
#include <cuda_bf16.h>
#include <math.h>
#include <stdlib.h>
#include <mutex>

namespace fvattn {

template <bool MASKED>
__global__ void __launch_bounds__(kThreads, 1)
fv_attn_fwd_d128(const __grid_constant__ CUtensorMap mq, const __grid_constant__ CUtensorMap mk,
                 const __grid_constant__ CUtensorMap mv, const __grid_constant__ Job jb) {
#if defined(__CUDA_ARCH_FEAT_SM100_ALL) || defined(__CUDA_ARCH_FEAT_SM103_ALL)
    extern __shared__ __align__(1024) unsigned char fv_smem[];
    attn_persistent<MASKED>(&mq, &mk, &mv, jb, fv_smem);
#endif
}

// Waits on a barrier nobody arrives at, with a budget of `cycles`: the bounded-wait failure path on
// its own (status word written, abort flag raised, normal return).
__global__ void fv_wait_probe_kernel(int* status, long long cycles) {
#if defined(__CUDA_ARCH_FEAT_SM100_ALL) || defined(__CUDA_ARCH_FEAT_SM103_ALL)
    __shared__ __align__(8) unsigned long long bar;
    __shared__ int abort_flag;
    const uint32_t b = fvp::smem_u32(&bar);
    if (threadIdx.x == 0) {
        fvp::mbar_init(b, 1);
        abort_flag = 0;
        fvp::mbar_init_fence();
    }
    __syncthreads();
    const fvp::WaitCtl ctl{&abort_flag, status, 9, cycles};
    fvp::mbar_wait(b, 0, ctl);
#endif
}

typedef void (*KernelFn)(const CUtensorMap, const CUtensorMap, const CUtensorMap, const Job);

struct LaunchArgs {
    const void *q, *k, *v;
    void* out;
    int out_is_bf16 = 1, planes = 0, sq = 0, nseg = 1;
    const int *seg_len = nullptr, *seg_start = nullptr;
    int seg_rows = 0;
    int kv_plane_rows = 0;  // rows between two planes of k / v when they are windows of longer planes (0: seg_rows)
    float scale = 0.f;
    int mask_mode = FV_MASK_NONE, block_tokens = 0, window = 0, sink = 0, q_row0 = 0;
    float* lse_out = nullptr;
    const float *prev_o = nullptr, *prev_lse = nullptr;
    int out_heads = 0, q_div = 1;
    int q_split = 0, q_row1 = 0;
};

#ifdef FV_ATT_TRACE
static unsigned long long* g_fv_trace = nullptr;
static int g_fv_trace_steps = 0;
extern "C" __attribute__((visibility("default"))) void fv_debug_set_trace(unsigned long long* dev_buf, int steps) {
    g_fv_trace = dev_buf;
    g_fv_trace_steps = steps;
}
#endif

static int launch(cudaStream_t stream, const LaunchArgs& a) {
    int dev;
    int rc = fvrt::require_sm100(&dev);
    if (rc != FV_RAN) return rc;
    if (!a.q || !a.k || !a.v || !a.out) return fvrt::fail(FV_ERR_INVALID, "sdpa: null operand");
    if (((uintptr_t)a.q | (uintptr_t)a.k | (uintptr_t)a.v | (uintptr_t)a.out) & 15)
        return fvrt::fail(FV_ERR_INVALID, "sdpa: operands must be 16-byte aligned");
    if ((a.prev_o == nullptr) != (a.prev_lse == nullptr))
        return fvrt::fail(FV_ERR_INVALID, "sdpa: prev_o and prev_lse go together");
    if (a.prev_o && ((uintptr_t)a.prev_o & 15)) return fvrt::fail(FV_ERR_INVALID, "sdpa: prev_o must be 16-byte aligned");
    if (!(a.scale > 0.f) || !isfinite(a.scale)) return fvrt::fail(FV_ERR_INVALID, "sdpa: scale must be positive and finite");
    if (a.mask_mode != FV_MASK_NONE && a.mask_mode != FV_MASK_BLOCK_CAUSAL)
        return fvrt::fail(FV_ERR_INVALID, "sdpa: unknown mask mode %d", a.mask_mode);
    if (a.mask_mode == FV_MASK_BLOCK_CAUSAL && (a.block_tokens < 1 || a.window < 0 || a.sink < 0 || a.q_row0 < 0))
        return fvrt::fail(FV_ERR_INVALID, "sdpa: block-causal needs block_tokens >= 1, window, sink, q_row0 >= 0");
    if (a.q_split < 0 || a.q_split >= a.sq || a.q_row1 < 0)
        return fvrt::fail(FV_ERR_INVALID, "sdpa: second row run starts at row %d of %d, global index %d", a.q_split, a.sq, a.q_row1);
    if (a.nseg < 1 || a.nseg > kMaxSeg) return fvrt::fail(FV_ERR_INVALID, "sdpa: 1..%d K/V segments", kMaxSeg);
    if (a.q_div < 1 || a.planes % a.q_div != 0)
        return fvrt::fail(FV_ERR_INVALID, "sdpa: %d planes do not split by %d", a.planes, a.q_div);

    Job jb{};
    jb.out = a.out;
    jb.lse_out = a.lse_out;
    jb.prev_o = a.prev_o;
    jb.prev_lse = a.prev_lse;
    jb.out_is_bf16 = a.out_is_bf16 ? 1 : 0;
    jb.out_heads = a.out_heads;
    jb.planes = a.planes;
    jb.sq = a.sq;
    jb.q_blocks = (a.sq + kItemRows - 1) / kItemRows;
    jb.sl2 = a.scale * 1.4426950408889634f;
    jb.nseg = a.nseg;
    long long total = 0;
    for (int s = 0; s < a.nseg; s++) {
        if (a.seg_len[s] < 0 || a.seg_len[s] > a.seg_rows || a.seg_start[s] < 0)
            return fvrt::fail(FV_ERR_INVALID, "sdpa: segment %d has length %d (rows %d), start %d", s, a.seg_len[s],
                              a.seg_rows, a.seg_start[s]);
        jb.seg_len[s] = a.seg_len[s];
        jb.seg_start[s] = a.seg_start[s];
        total += a.seg_len[s];
        if ((long long)a.seg_start[s] + a.seg_len[s] > 0x3fffffffll) return FV_DECLINED;
    }
    if (total == 0) return FV_DECLINED;
    const bool masked = a.mask_mode != FV_MASK_NONE;
    jb.block_tokens = a.block_tokens;
    jb.window = a.window;
    jb.sink = a.sink;
    jb.q_row0 = a.q_row0;
    jb.q_split = a.q_split;
    jb.q_row1 = a.q_row1;
    jb.heavy_first = masked ? 1 : 0;
    jb.q_div = a.q_div;
    jb.wait_cycles = FV_WAIT_CYCLES;
#ifdef FV_ATT_TRACE
    jb.trace = g_fv_trace;
    jb.trace_steps = g_fv_trace_steps;
#endif
    rc = fvrt::status_word(dev, &jb.status);
    if (rc != FV_RAN) return rc;
    const long long items = (long long)jb.q_blocks * a.planes;
    if (items > 0x7fffffffll) return FV_DECLINED;
    jb.items = (int)items;

    CUtensorMap mq, mk, mv;
    {
        const uint64_t qplanes = (uint64_t)(a.planes / a.q_div);
        const uint64_t dq[4] = {128, (uint64_t)a.sq, qplanes, 1};
        const uint64_t sqb[3] = {256, (uint64_t)a.sq * 256, (uint64_t)a.sq * 256 * qplanes};
        rc = fvrt::encode_map4_cached(&mq, a.q, dq, sqb, 128);
        if (rc != FV_RAN) return rc;
        // (a window of a longer plane: the map's row extent stays the window, so rows past it read as zeros and
        // nothing beyond the last plane's window is touched; only the plane stride is the longer plane's)
        const uint64_t plane_rows = (uint64_t)(a.kv_plane_rows > 0 ? a.kv_plane_rows : a.seg_rows);
        const uint64_t dk[4] = {128, (uint64_t)a.seg_rows, (uint64_t)a.planes, (uint64_t)a.nseg};
        const uint64_t skb[3] = {256, plane_rows * 256, plane_rows * 256 * a.planes};
        rc = fvrt::encode_map4_cached(&mk, a.k, dk, skb, 128);
        if (rc != FV_RAN) return rc;
        rc = fvrt::encode_map4_cached(&mv, a.v, dk, skb, 128);
        if (rc != FV_RAN) return rc;
    }

    const KernelFn fn = masked ? fv_attn_fwd_d128<true> : fv_attn_fwd_d128<false>;
    {
        static bool attr_set[64][2] = {};
        static std::mutex attr_mu;
        std::lock_guard<std::mutex> attr_lock(attr_mu);
        if (!attr_set[dev][masked]) {
            FV_CUDA(cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)Smem::total));
            attr_set[dev][masked] = true;
        }
    }
    int sms = 0;
    rc = fvrt::sm_count(dev, &sms);
    if (rc != FV_RAN) return rc;
    // A persistent CTA holds its SM for the whole launch (168 registers x 384 threads are the SM's register file): a
    // caller that runs a collective's copy kernels beside this launch asks for some SMs to stay free.
    const int spare = fvrt::take_spare_sms();
    if (spare > 0 && sms - spare >= 16) sms -= spare;
    const unsigned grid = (unsigned)(items < sms ? items : sms);
    fn<<<grid, kThreads, Smem::total, stream>>>(mq, mk, mv, jb);
    FV_CUDA(cudaGetLastError());
    fvrt::ran(masked ? fvrt::kLogCausal : fvrt::kLogDense,
              "sdpa: fv_attn_fwd_d128<%s> (sm_100a tcgen05, persistent, %u CTAs x %d threads) planes=%d sq=%d keys=%lld", masked ? "block-causal" : "dense",
              grid, kThreads, a.planes, a.sq, total);
    return FV_RAN;
}

// ---- built-in scratch for callers that cannot allocate ---------------------------------------------
// The pass-1 result of the two-pass evaluation: kNoAllocMaxRows rows of 128 f32 and one f32
// log-sum-exp per row.  Held by every GPU that loads the library until the process exits (about 32 MiB).
constexpr long long kNoAllocMaxRows = 65024;
constexpr size_t kNoAllocFloats = 64 + (size_t)kNoAllocMaxRows * (kD + 1);
static __device__ __align__(256) float fv_noalloc_scratch[kNoAllocFloats];
// In host code the array's name is only a stand-in: the device address comes from the runtime, once per
// device, with that device current.
static float* g_noalloc_ptr[64] = {};
static std::mutex g_noalloc_mu;

static int noalloc_base(int dev, float** out) {
    std::lock_guard<std::mutex> lk(g_noalloc_mu);
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
    // Nothing in the scratch has to start at zero: pass 1 writes every row of o1 / lse1 that pass 2 reads.
    // Bounded-wait failures go to the library's one status word (fv_device_status), itself part of the
    // module image.
    float* o1 = base + 64;
    float* lse1 = o1 + (size_t)kNoAllocMaxRows * kD;
    LaunchArgs p1;
    p1.q = q; p1.k = k_local; p1.v = v_local; p1.out = o1; p1.out_is_bf16 = 0; p1.planes = bh; p1.sq = sq;
    p1.nseg = 1; p1.seg_len = &local_len; p1.seg_start = &local_start; p1.seg_rows = local_rows; p1.scale = scale;
    p1.lse_out = lse1;
    rc = launch(stream, p1);
    if (rc != FV_RAN) return rc;
    if (remote_ready) FV_CUDA(cudaStreamWaitEvent(stream, remote_ready, 0));
    LaunchArgs p2;
    p2.q = q; p2.k = k_all; p2.v = v_all; p2.out = out; p2.out_is_bf16 = out_is_bf16; p2.planes = bh; p2.sq = sq;
    p2.nseg = nseg; p2.seg_len = seg_len; p2.seg_start = seg_start; p2.seg_rows = seg_rows; p2.scale = scale;
    p2.prev_o = o1; p2.prev_lse = lse1;
    return launch(stream, p2);
}

// ---- split-KV: few query rows against a long key window ----------------------------------------------
// A block of 4 680 queries over a 32 760-key window is 19 x 12 = 228 work items on 148 SMs: the second
// round runs half empty.  Each head's keys are cut into `splits` equal ranges that run as planes of
// their own (k and v are only viewed as [bh * splits, sk / splits, 128]; q is read through q_div), every
// plane leaves a normalised f32 result and its log-sum-exp in the workspace, and one HBM-bound kernel
// merges them.  The merge is the two-pass formula of the attention epilogue applied to `splits` parts.
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

// Estimated duration in microseconds of `splits` ranges on `sms` SMs: equal work items run in whole
// rounds, a 256 x 128 tile step takes about 2 us, an item pays about 3 steps of fill and drain (4 with
// the f32 store of a part), the merge moves (splits + 1) x the output at about 5 TB/s.
static double splitkv_cost(long long bh, long long sq, long long sk, int splits, int sms) {
    const long long nqb = (sq + kItemRows - 1) / kItemRows;
    const long long waves = (nqb * bh * splits + sms - 1) / sms;
    const long long tiles = (sk / splits + kKeyTile - 1) / kKeyTile;
    double us = (double)waves * (double)(tiles + (splits > 1 ? 4 : 3)) * 2.0;
    if (splits > 1) us += 3.0 + (double)bh * sq * kD * 4.0 * (splits + 1) / 5.0e6;
    return us;
}

static int splitkv_choose(long long bh, long long sq, long long sk, int sms) {
    if (bh <= 0 || sq <= 0 || sk <= 0 || sms <= 0) return 1;
    int best = 1;
    double best_us = splitkv_cost(bh, sq, sk, 1, sms);
    for (int s = 2; s <= kMaxSplits; s++) {
        if (sk % s != 0 || sk / s < 4 * kKeyTile || bh * s > 0x7fffffffll) continue;
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
    LaunchArgs a;
    a.q = q; a.k = k; a.v = v; a.out = part_o; a.out_is_bf16 = 0; a.planes = bh * splits; a.sq = sq;
    a.nseg = 1; a.seg_len = &len; a.seg_start = &start; a.seg_rows = len; a.scale = scale;
    a.lse_out = part_lse; a.q_div = splits;
    int rc = launch(stream, a);
    if (rc != FV_RAN) return rc;
    const long long rows = (long long)bh * sq;
    const unsigned grid = (unsigned)((rows + 7) / 8);
    if (out_is_bf16)
        fv_splitkv_merge_kernel<1><<<grid, 256, 0, stream>>>(part_o, part_lse, out, bh, sq, splits, out_heads);
    else
        fv_splitkv_merge_kernel<0><<<grid, 256, 0, stream>>>(part_o, part_lse, out, bh, sq, splits, out_heads);
    FV_CUDA(cudaGetLastError());
    fvrt::ran(fvrt::kLogSplitKv, "sdpa: split-KV, %d key ranges of %d + fv_splitkv_merge_kernel", splits, len);
    return FV_RAN;
}

}  // namespace fvattn

extern "C" int fv_sdpa_two_pass_noalloc_bf16(void* stream, const void* q, const void* k_local, const void* v_local,
                                             int local_len, int local_start, int local_rows, const void* k_all,
                                             const void* v_all, int nseg, const int* seg_len, const int* seg_start,
                                             int seg_rows, void* out, int out_is_bf16, int bh, int sq, float scale,
                                             void* remote_ready_event) {
    fvrt::clear_error();
    if (bh <= 0 || sq <= 0 || nseg <= 0 || seg_rows <= 0 || local_rows <= 0) return FV_DECLINED;
    if (!seg_len || !seg_start) return fvrt::fail(FV_ERR_INVALID, "sdpa: null segment table");
    return fvattn::two_pass_noalloc((cudaStream_t)stream, q, k_local, v_local, local_len, local_start, local_rows, k_all,
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
    fvattn::LaunchArgs a;
    a.q = q; a.k = k; a.v = v; a.out = out; a.out_is_bf16 = out_is_bf16; a.planes = bh; a.sq = sq;
    a.nseg = nseg; a.seg_len = seg_len; a.seg_start = seg_start; a.seg_rows = seg_rows; a.scale = scale;
    a.mask_mode = mask_mode; a.block_tokens = block_tokens; a.window = window; a.sink = sink; a.q_row0 = q_row0;
    a.lse_out = lse_out; a.prev_o = prev_o; a.prev_lse = prev_lse;
    return fvattn::launch((cudaStream_t)stream, a);
}

extern "C" int fv_sdpa_segments_runs_bf16(void* stream, const void* q, const void* k, const void* v, void* out,
                                          int out_is_bf16, int bh, int sq, int nseg, const int* seg_len,
                                          const int* seg_start, int seg_rows, float scale, int mask_mode,
                                          int block_tokens, int window, int sink, int q_row0, int q_split, int q_row1,
                                          float* lse_out, const float* prev_o, const float* prev_lse) {
    fvrt::clear_error();
    if (bh <= 0 || sq <= 0 || nseg <= 0 || seg_rows <= 0) return FV_DECLINED;
    if (sq > 0x3fffffff || seg_rows > 0x3fffffff) return FV_DECLINED;
    if (!seg_len || !seg_start) return fvrt::fail(FV_ERR_INVALID, "sdpa: null segment table");
    fvattn::LaunchArgs a;
    a.q = q; a.k = k; a.v = v; a.out = out; a.out_is_bf16 = out_is_bf16; a.planes = bh; a.sq = sq;
    a.nseg = nseg; a.seg_len = seg_len; a.seg_start = seg_start; a.seg_rows = seg_rows; a.scale = scale;
    a.mask_mode = mask_mode; a.block_tokens = block_tokens; a.window = window; a.sink = sink; a.q_row0 = q_row0;
    a.q_split = q_split; a.q_row1 = q_row1;
    a.lse_out = lse_out; a.prev_o = prev_o; a.prev_lse = prev_lse;
    return fvattn::launch((cudaStream_t)stream, a);
}

static int dense_call(void* stream, const void* q, const void* k, const void* v, void* out, int out_is_bf16, int planes,
                      int sq, int sk, float scale, int mask_mode, int block_tokens, int window, int sink, int q_row0,
                      int out_heads) {
    const int len = sk, start = 0;
    fvattn::LaunchArgs a;
    a.q = q; a.k = k; a.v = v; a.out = out; a.out_is_bf16 = out_is_bf16; a.planes = planes; a.sq = sq;
    a.nseg = 1; a.seg_len = &len; a.seg_start = &start; a.seg_rows = sk; a.scale = scale;
    a.mask_mode = mask_mode; a.block_tokens = block_tokens; a.window = window; a.sink = sink; a.q_row0 = q_row0;
    a.out_heads = out_heads;
    return fvattn::launch((cudaStream_t)stream, a);
}

extern "C" int fv_sdpa_dense_bf16(void* stream, const void* q, const void* k, const void* v, void* out, int out_is_bf16,
                                  int bh, int sq, int sk, int d, float scale, int mask_mode, int block_tokens,
                                  int window, int sink, int q_row0) {
    fvrt::clear_error();
    if (d != 128 || bh <= 0 || sq <= 0 || sk <= 0) return FV_DECLINED;
    if (sq > 0x3fffffff || sk > 0x3fffffff) return FV_DECLINED;
    return dense_call(stream, q, k, v, out, out_is_bf16, bh, sq, sk, scale, mask_mode, block_tokens, window, sink, q_row0, 0);
}

extern "C" int fv_sdpa_window_bf16(void* stream, const void* q, const void* k_cache, const void* v_cache, void* out,
                                   int out_is_bf16, int bh, int sq, int cache_rows, int window_start, int window_len, int d,
                                   float scale, int out_heads) {
    fvrt::clear_error();
    if (d != 128 || bh <= 0 || sq <= 0 || window_len <= 0) return FV_DECLINED;
    if (sq > 0x3fffffff || cache_rows > 0x3fffffff) return FV_DECLINED;
    if (window_start < 0 || (long long)window_start + window_len > cache_rows)
        return fvrt::fail(FV_ERR_INVALID, "sdpa window: rows [%d, %d) outside a cache of %d rows", window_start,
                          window_start + window_len, cache_rows);
    if (out_heads < 0 || (out_heads > 0 && bh % out_heads != 0)) return fvrt::fail(FV_ERR_INVALID, "sdpa window: out_heads %d", out_heads);
    if (!k_cache || !v_cache) return fvrt::fail(FV_ERR_INVALID, "sdpa: null operand");
    const int len = window_len, start = 0;
    fvattn::LaunchArgs a;
    a.q = q;
    a.k = static_cast<const unsigned short*>(k_cache) + (size_t)window_start * 128;
    a.v = static_cast<const unsigned short*>(v_cache) + (size_t)window_start * 128;
    a.out = out; a.out_is_bf16 = out_is_bf16; a.planes = bh; a.sq = sq;
    a.nseg = 1; a.seg_len = &len; a.seg_start = &start; a.seg_rows = window_len; a.kv_plane_rows = cache_rows; a.scale = scale;
    a.out_heads = out_heads;
    return fvattn::launch((cudaStream_t)stream, a);
}

extern "C" int fv_sdpa_dense_merged_bf16(void* stream, const void* q, const void* k, const void* v, void* out,
                                         int out_is_bf16, int batch, int heads, int sq, int sk, int d, float scale,
                                         int mask_mode, int block_tokens, int window, int sink, int q_row0) {
    fvrt::clear_error();
    if (d != 128 || batch <= 0 || heads <= 0 || sq <= 0 || sk <= 0) return FV_DECLINED;
    if (sq > 0x3fffffff || sk > 0x3fffffff || (long long)batch * heads > 0x7fffffffll) return FV_DECLINED;
    return dense_call(stream, q, k, v, out, out_is_bf16, batch * heads, sq, sk, scale, mask_mode, block_tokens, window, sink,
                      q_row0, heads);
}

extern "C" int fv_sdpa_splitkv_choose(int bh, int sq, int sk, int sm_count) {
    return fvattn::splitkv_choose(bh, sq, sk, sm_count);
}

extern "C" size_t fv_sdpa_splitkv_workspace_bytes(int bh, int sq, int splits) {
    if (bh <= 0 || sq <= 0 || splits < 2 || splits > fvattn::kMaxSplits) return 0;
    return fvattn::splitkv_bytes(bh, sq, splits);
}

extern "C" int fv_sdpa_splitkv_bf16(void* stream, const void* q, const void* k, const void* v, void* out,
                                    int out_is_bf16, int bh, int sq, int sk, int d, float scale, int splits,
                                    int out_heads, void* workspace, size_t workspace_bytes) {
    fvrt::clear_error();
    if (d != 128 || bh <= 0 || sq <= 0 || sk <= 0) return FV_DECLINED;
    if (sq > 0x3fffffff || sk > 0x3fffffff) return FV_DECLINED;
    return fvattn::splitkv((cudaStream_t)stream, q, k, v, out, out_is_bf16, bh, sq, sk, scale, splits, out_heads,
                           workspace, workspace_bytes);
}

extern "C" int fv_selftest_wait_timeout(void* stream, long long cycles) {
    fvrt::clear_error();
    int dev;
    int rc = fvrt::require_sm100(&dev);
    if (rc != FV_RAN) return rc;
    if (cycles < 1000 || cycles > 2000000000ll) return fvrt::fail(FV_ERR_INVALID, "selftest: 1e3 .. 2e9 cycles");
    int* status;
    rc = fvrt::status_word(dev, &status);
    if (rc != FV_RAN) return rc;
    fvattn::fv_wait_probe_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(status, cycles);
    FV_CUDA(cudaGetLastError());
    return FV_RAN;
}
