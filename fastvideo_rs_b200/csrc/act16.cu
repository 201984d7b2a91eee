// Operand rounding for callers whose activations are stored as f32: the reference rounds q, k and v to
// bf16 before the attention kernels under bf16 activations and rounds the result again
// (act16_operands and the tail of dense, crates/fastvideo-cudarc/src/rt/sdpa.rs:167-181,184-214; three
// cast_f32_bf16 launches and one more after, rt/ops.rs cast_f32_bf16_device / cast_bf16_f32_device).
//
// Here the three roundings are ONE launch (a persistent grid walks q, then k, then v as one index
// space of 8-value groups: 32 bytes read, 16 written per thread step), and the widening of the bf16
// result to the caller's f32 storage is a second one.  Both are pure HBM streams.
#include "fv_runtime.h"
#include <stdint.h>

namespace fvact {

constexpr int kThreads = 256;

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    uint32_t r;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
}

struct Three {
    const float* src[3];
    void* dst[3];
    long long groups[3];  // whole groups of 8 values
    long long count[3];   // values
};

__global__ void __launch_bounds__(kThreads) round3_kernel(Three t) {
    const long long stride = (long long)gridDim.x * kThreads;
    const long long first = (long long)blockIdx.x * kThreads + threadIdx.x;
#pragma unroll
    for (int a = 0; a < 3; ++a) {
        const float4* __restrict__ s = reinterpret_cast<const float4*>(t.src[a]);
        uint4* __restrict__ d = reinterpret_cast<uint4*>(t.dst[a]);
        for (long long g = first; g < t.groups[a]; g += stride) {
            const float4 lo = __ldcs(s + 2 * g), hi = __ldcs(s + 2 * g + 1);
            uint4 o;
            o.x = pack_bf16(lo.x, lo.y);
            o.y = pack_bf16(lo.z, lo.w);
            o.z = pack_bf16(hi.x, hi.y);
            o.w = pack_bf16(hi.z, hi.w);
            d[g] = o;
        }
        // ragged tail (fewer than 8 values), one thread
        if (first == 0) {
            unsigned short* d16 = reinterpret_cast<unsigned short*>(t.dst[a]);
            for (long long i = t.groups[a] * 8; i < t.count[a]; ++i)
                d16[i] = (unsigned short)(pack_bf16(t.src[a][i], 0.f) & 0xffffu);
        }
    }
}

__global__ void __launch_bounds__(kThreads) widen_kernel(const uint4* __restrict__ src, float4* __restrict__ dst, long long groups,
                                                         long long count) {
    const long long stride = (long long)gridDim.x * kThreads;
    const long long first = (long long)blockIdx.x * kThreads + threadIdx.x;
    for (long long g = first; g < groups; g += stride) {
        const uint4 u = __ldcs(src + g);
        float4 lo, hi;
        lo.x = __uint_as_float(u.x << 16); lo.y = __uint_as_float(u.x & 0xffff0000u);
        lo.z = __uint_as_float(u.y << 16); lo.w = __uint_as_float(u.y & 0xffff0000u);
        hi.x = __uint_as_float(u.z << 16); hi.y = __uint_as_float(u.z & 0xffff0000u);
        hi.z = __uint_as_float(u.w << 16); hi.w = __uint_as_float(u.w & 0xffff0000u);
        __stcs(dst + 2 * g, lo);
        __stcs(dst + 2 * g + 1, hi);
    }
    if (first == 0) {
        const unsigned short* s16 = reinterpret_cast<const unsigned short*>(src);
        float* d32 = reinterpret_cast<float*>(dst);
        for (long long i = groups * 8; i < count; ++i) d32[i] = __uint_as_float((uint32_t)s16[i] << 16);
    }
}

int grid_for(long long groups) {
    int dev = 0, sms = 148;
    if (cudaGetDevice(&dev) == cudaSuccess) fvrt::sm_count(dev, &sms);
    long long want = (groups + kThreads - 1) / kThreads;
    long long cap = (long long)sms * 8;
    return (int)(want < 1 ? 1 : (want < cap ? want : cap));
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

}  // namespace fvact

extern "C" int fv_act16_operands(void* stream, const float* q, const float* k, const float* v, long long q_count,
                                 long long kv_count, void* q16, void* k16, void* v16) {
    fvrt::clear_error();
    int dev;
    int rc = fvrt::require_sm100(&dev);
    if (rc != FV_RAN) return rc;
    if (q_count <= 0 || kv_count <= 0) return FV_DECLINED;
    if (!q || !k || !v || !q16 || !k16 || !v16) return fvrt::fail(FV_ERR_INVALID, "act16_operands: null pointer");
    if (!fvact::aligned16(q) || !fvact::aligned16(k) || !fvact::aligned16(v) || !fvact::aligned16(q16) || !fvact::aligned16(k16) ||
        !fvact::aligned16(v16))
        return fvrt::fail(FV_ERR_INVALID, "act16_operands: pointers must be 16-byte aligned");
    fvact::Three t;
    t.src[0] = q; t.src[1] = k; t.src[2] = v;
    t.dst[0] = q16; t.dst[1] = k16; t.dst[2] = v16;
    t.count[0] = q_count; t.count[1] = t.count[2] = kv_count;
    for (int a = 0; a < 3; ++a) t.groups[a] = t.count[a] / 8;
    const long long most = t.groups[0] > t.groups[1] ? t.groups[0] : t.groups[1];
    fvact::round3_kernel<<<fvact::grid_for(most), fvact::kThreads, 0, (cudaStream_t)stream>>>(t);
    FV_CUDA(cudaGetLastError());
    return FV_RAN;
}

extern "C" int fv_act16_widen(void* stream, const void* src16, long long count, float* dst) {
    fvrt::clear_error();
    int dev;
    int rc = fvrt::require_sm100(&dev);
    if (rc != FV_RAN) return rc;
    if (count <= 0) return FV_DECLINED;
    if (!src16 || !dst) return fvrt::fail(FV_ERR_INVALID, "act16_widen: null pointer");
    if (!fvact::aligned16(src16) || !fvact::aligned16(dst)) return fvrt::fail(FV_ERR_INVALID, "act16_widen: pointers must be 16-byte aligned");
    const long long groups = count / 8;
    fvact::widen_kernel<<<fvact::grid_for(groups), fvact::kThreads, 0, (cudaStream_t)stream>>>(
        reinterpret_cast<const uint4*>(src16), reinterpret_cast<float4*>(dst), groups, count);
    FV_CUDA(cudaGetLastError());
    return FV_RAN;
}
