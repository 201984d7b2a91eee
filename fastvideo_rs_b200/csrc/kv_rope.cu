// Wan's interleaved-pair RoPE over rows of BHSD tensors, source and destination each a window of rows
// inside planes of their own length: the operation the causal K/V cache of the reference runs when it
// re-ropes its sink keys (KvRope::RebasedSink, crates/fastvideo-cudarc/src/wan/causal.rs:62-76,734-812;
// rope_bhsd_f32, :246-263 -> apply_rotary_bshd, rt/ops.rs:1903-1933 / :2625-2650), where it is
// rope_bhsd_f32 + quantize_bf16 + copy_tokens (three launches and two temporaries) per layer and block.
//
// Here it is one pass: row t of every plane is read at src_row0 + t, rotated with table row t
// (o_even = x0 cos - x1 sin, o_odd = x0 sin + x1 cos; products and sums rounded separately like the host
// twin; sin may be negated to rotate back, which is how the un-roped copy of the sink is taken) and
// written at dst_row0 + t, in f32 or rounded once to bf16.  HBM-bound: a thread moves 8 values.
#include "fv_runtime.h"
#include <stdint.h>

namespace fvkv {

constexpr int kD = 128;
constexpr int kThreads = 256;

struct Args {
    const void* src;
    void* dst;
    const float* cosv;
    const float* sinv;
    long long chunks;  // planes * n * 16
    int n, src_rows, src_row0, dst_rows, dst_row0;
    float sin_sign;
};

__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
    uint32_t r;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
}

template <bool SRC16, bool DST16>
__global__ void __launch_bounds__(kThreads) fv_wan_rope_bhsd_kernel(const Args a) {
    const long long stride = (long long)gridDim.x * kThreads;
    for (long long c = (long long)blockIdx.x * kThreads + threadIdx.x; c < a.chunks; c += stride) {
        const int part = (int)(c & 15);
        const long long rowi = c >> 4;
        const int t = (int)(rowi % a.n);
        const long long plane = rowi / a.n;
        const size_t si = ((size_t)plane * a.src_rows + a.src_row0 + t) * kD + 8 * part;
        const size_t di = ((size_t)plane * a.dst_rows + a.dst_row0 + t) * kD + 8 * part;
        float x[8];
        if (SRC16) {
            const uint4 u = *reinterpret_cast<const uint4*>(static_cast<const unsigned short*>(a.src) + si);
            const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
            for (int i = 0; i < 4; i++) {
                x[2 * i] = __uint_as_float(w[i] << 16);
                x[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
            }
        } else {
            const float4* sp = reinterpret_cast<const float4*>(static_cast<const float*>(a.src) + si);
            const float4 lo = sp[0], hi = sp[1];
            x[0] = lo.x; x[1] = lo.y; x[2] = lo.z; x[3] = lo.w; x[4] = hi.x; x[5] = hi.y; x[6] = hi.z; x[7] = hi.w;
        }
        const float4* cp = reinterpret_cast<const float4*>(a.cosv + (size_t)t * kD + 8 * part);
        const float4* np = reinterpret_cast<const float4*>(a.sinv + (size_t)t * kD + 8 * part);
        const float4 c0 = __ldg(cp), c1 = __ldg(cp + 1), s0 = __ldg(np), s1 = __ldg(np + 1);
        // (the tables hold every value twice; both factors of a pair are read at its even index like the host twin)
        const float cs[4] = {c0.x, c0.z, c1.x, c1.z};
        const float sn[4] = {s0.x * a.sin_sign, s0.z * a.sin_sign, s1.x * a.sin_sign, s1.z * a.sin_sign};
        float o[8];
#pragma unroll
        for (int i = 0; i < 4; i++) {
            o[2 * i] = __fsub_rn(__fmul_rn(x[2 * i], cs[i]), __fmul_rn(x[2 * i + 1], sn[i]));
            o[2 * i + 1] = __fadd_rn(__fmul_rn(x[2 * i], sn[i]), __fmul_rn(x[2 * i + 1], cs[i]));
        }
        if (DST16) {
            *reinterpret_cast<uint4*>(static_cast<unsigned short*>(a.dst) + di) =
                make_uint4(pack2(o[0], o[1]), pack2(o[2], o[3]), pack2(o[4], o[5]), pack2(o[6], o[7]));
        } else {
            float4* dp = reinterpret_cast<float4*>(static_cast<float*>(a.dst) + di);
            dp[0] = make_float4(o[0], o[1], o[2], o[3]);
            dp[1] = make_float4(o[4], o[5], o[6], o[7]);
        }
    }
}

}  // namespace fvkv

extern "C" int fv_wan_rope_bhsd(void* stream, const void* src, int src_is_bf16, int src_plane_rows, int src_row0,
                                const float* cosv, const float* sinv, int negate_sin, int planes, int n, void* dst,
                                int dst_is_bf16, int dst_plane_rows, int dst_row0) {
    fvrt::clear_error();
    if (planes <= 0 || n <= 0) return FV_DECLINED;
    int dev;
    int rc = fvrt::require_sm100(&dev);
    if (rc != FV_RAN) return rc;
    if (!src || !dst || !cosv || !sinv) return fvrt::fail(FV_ERR_INVALID, "rope_bhsd: null operand");
    if (((uintptr_t)src | (uintptr_t)dst | (uintptr_t)cosv | (uintptr_t)sinv) & 15)
        return fvrt::fail(FV_ERR_INVALID, "rope_bhsd: operands must be 16-byte aligned");
    if (src_row0 < 0 || dst_row0 < 0 || (long long)src_row0 + n > src_plane_rows || (long long)dst_row0 + n > dst_plane_rows)
        return fvrt::fail(FV_ERR_INVALID, "rope_bhsd: %d rows at %d / %d do not fit planes of %d / %d rows", n, src_row0, dst_row0,
                          src_plane_rows, dst_plane_rows);
    fvkv::Args a{};
    a.src = src;
    a.dst = dst;
    a.cosv = cosv;
    a.sinv = sinv;
    a.chunks = (long long)planes * n * 16;
    a.n = n;
    a.src_rows = src_plane_rows;
    a.src_row0 = src_row0;
    a.dst_rows = dst_plane_rows;
    a.dst_row0 = dst_row0;
    a.sin_sign = negate_sin ? -1.f : 1.f;
    int sms = 0;
    rc = fvrt::sm_count(dev, &sms);
    if (rc != FV_RAN) return rc;
    long long want = (a.chunks + fvkv::kThreads - 1) / fvkv::kThreads;
    const unsigned grid = (unsigned)(want < (long long)sms * 8 ? want : (long long)sms * 8);
    cudaStream_t st = (cudaStream_t)stream;
    if (src_is_bf16 && dst_is_bf16) fvkv::fv_wan_rope_bhsd_kernel<true, true><<<grid, fvkv::kThreads, 0, st>>>(a);
    else if (src_is_bf16) fvkv::fv_wan_rope_bhsd_kernel<true, false><<<grid, fvkv::kThreads, 0, st>>>(a);
    else if (dst_is_bf16) fvkv::fv_wan_rope_bhsd_kernel<false, true><<<grid, fvkv::kThreads, 0, st>>>(a);
    else fvkv::fv_wan_rope_bhsd_kernel<false, false><<<grid, fvkv::kThreads, 0, st>>>(a);
    FV_CUDA(cudaGetLastError());
    return FV_RAN;
}

// ---- the cache's pointer arithmetic and its roll ----------------------------------------------------------
// KvSpec::plan (crates/fastvideo-cudarc/src/wan/causal.rs:289-336): where a block of n tokens that starts at
// token current_start of the rollout goes in a cache whose state is (global_end, local_end_prev).
extern "C" int fv_kv_plan(const fv_kv_spec* spec, long long global_end, long long local_end_prev, long long current_start,
                          long long n, fv_kv_move* out) {
    fvrt::clear_error();
    if (!spec || !out) return fvrt::fail(FV_ERR_INVALID, "kv plan: null argument");
    if (global_end < 0 || local_end_prev < 0 || current_start < 0 || n < 0 || spec->capacity < 0 || spec->max_attention < 0)
        return fvrt::fail(FV_ERR_INVALID, "kv plan: negative argument");
    const long long current_end = current_start + n;
    if (!spec->rolling && current_end > spec->max_attention)
        return fvrt::fail(FV_ERR_INVALID,
                          "causal Wan local_attn_size=-1 keeps a %lld-frame KV window; got current_end=%lld tokens with "
                          "frame_seqlen=%d (set local_attn_size for longer rollouts)",
                          (long long)spec->max_attention / (spec->frame_tokens > 0 ? spec->frame_tokens : 1), current_end,
                          spec->frame_tokens);
    if (current_end < global_end && current_end + local_end_prev < global_end)
        return fvrt::fail(FV_ERR_INVALID, "causal kv: block before the cache start");
    const long long advance = current_end > global_end ? current_end - global_end : 0;
    const long long evicted =
        (spec->rolling && current_end > global_end && n + local_end_prev > spec->capacity) ? n + local_end_prev - spec->capacity : 0;
    const long long back = global_end > current_end ? global_end - current_end : 0;
    long long local_end = local_end_prev + advance;
    if (local_end < back || local_end - back < evicted) return fvrt::fail(FV_ERR_INVALID, "causal kv: pointer underflow");
    local_end = local_end - back - evicted;
    if (local_end < n) return fvrt::fail(FV_ERR_INVALID, "causal kv: block longer than the cache");
    const long long cap = spec->capacity > n ? spec->capacity : n;
    if (local_end > cap) return fvrt::fail(FV_ERR_INVALID, "causal kv: write end %lld past the cache (%d tokens)", local_end, spec->capacity);
    out->evicted = evicted;
    out->local_start = local_end - n;
    out->local_end = local_end;
    out->window_start = local_end > spec->max_attention ? local_end - spec->max_attention : 0;
    return FV_RAN;
}

// The roll of a full cache (causal.rs:560-585 / update_static): rows [sink + evicted, local_end_prev) of every plane
// move down to row sink.  Source and destination overlap when more rows move than are evicted, so the move goes
// in chunks no longer than the shift (shift_tokens_down, causal.rs:236-249), each one strided 2-D copy over all
// planes on the caller's stream.
extern "C" int fv_kv_roll(void* stream, void* cache, int elem_bytes, int planes, int cache_rows, int sink, int evicted,
                          int local_end_prev) {
    fvrt::clear_error();
    if (planes <= 0 || evicted <= 0) return FV_DECLINED;
    if (!cache) return fvrt::fail(FV_ERR_INVALID, "kv roll: null cache");
    if ((elem_bytes != 2 && elem_bytes != 4) || sink < 0 || local_end_prev > cache_rows || sink + evicted > local_end_prev)
        return fvrt::fail(FV_ERR_INVALID, "kv roll: sink %d + evicted %d against %d cached rows of %d", sink, evicted, local_end_prev,
                          cache_rows);
    const size_t row = (size_t)fvkv::kD * elem_bytes, pitch = (size_t)cache_rows * row;
    unsigned char* base = static_cast<unsigned char*>(cache);
    int from = sink + evicted, to = sink, left = local_end_prev - from;
    while (left > 0) {
        const int n = left < evicted ? left : evicted;
        FV_CUDA(cudaMemcpy2DAsync(base + (size_t)to * row, pitch, base + (size_t)from * row, pitch, (size_t)n * row, planes,
                                  cudaMemcpyDeviceToDevice, (cudaStream_t)stream));
        from += n;
        to += n;
        left -= n;
    }
    return FV_RAN;
}
