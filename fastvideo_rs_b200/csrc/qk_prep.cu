// Wan q/k prologue: RMSNorm (statistic over the whole heads*d projection row, or per head),
// weight, interleaved-pair 3-D RoPE, head split to BHSD bf16 -- one pass over the fused QKV
// projection, V's head split riding along.  HBM-bound: reads each projection element once,
// writes each output element once.
//
// Replaces the two qk_norm_rope_bhsd launches and the split_heads_bhsd launch of
// WanAttention::forward_self (crates/fastvideo-cudarc/src/wan/transformer.rs:163-178,287-289;
// kernels crates/fastvideo-cudarc/src/rt/kernels/core.cu:368-428).  Arithmetic follows the f32
// host twin crates/fastvideo-cudarc/src/rt/ops.rs:2304-2350: inv = 1/sqrt(mean(x^2) + eps),
// y = (x*inv)*w, even = y0*cos[s,even] - y1*sin[s,even+1], odd = y0*sin[s,even+1] + y1*cos[s,even],
// every product and sum rounded separately (no fused multiply-add), then one rounding to bf16.
// Only the sum of squares differs: fused multiply-adds in a tree instead of a sequential sum of rounded squares.
#include "fv_runtime.h"
#include <cuda_bf16.h>
#include <math.h>
#include <stdlib.h>
#include <string.h>
#include <vector>

namespace fvprep {

constexpr int kD = 128;

struct Params {
    const __nv_bfloat16* proj;  // [batch, seq, width]
    const float* wq;            // [heads*128]
    const float* wk;
    const float* cosv;          // [seq, 128] or null (no rotation)
    const float* sinv;
    __nv_bfloat16* q_out;       // [batch*heads, seq, 128] (null: skip q)
    __nv_bfloat16* k_out;
    __nv_bfloat16* v_out;       // null: skip v
    int batch, seq, heads, width, col_q, col_k, col_v;
    float eps;
    int per_head;
    int kv_rows, kv_row0;       // k_out / v_out planes have kv_rows token rows and token s lands in row kv_row0 + s
                                // (kv_rows = seq, kv_row0 = 0: plain BHSD; otherwise the tail of a K/V cache)
};

__device__ __forceinline__ void unpack8(const uint4& u, float (&f)[8]) {
    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int i = 0; i < 4; i++) {
        f[2 * i] = __uint_as_float(w[i] << 16);
        f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
}
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
    uint32_t r;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
}

// Sum of the squares of 8 values on top of `acc` (fused multiply-adds: one rounding per term).
__device__ __forceinline__ float sumsq8(const float (&x)[8], float acc) {
#pragma unroll
    for (int i = 0; i < 8; i++) acc = fmaf(x[i], x[i], acc);
    return acc;
}
// Butterfly over `span` lanes (16: the threads of one head, 32: the warp); every lane ends with the sum.
__device__ __forceinline__ void lanes_sum(float& a, float& c, int span) {
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        if (o < span) {
            a += __shfl_xor_sync(0xffffffffu, a, o);
            c += __shfl_xor_sync(0xffffffffu, c, o);
        }
    }
}
// Row totals from the per-warp partial sums rb[0..nwarps) and rb[nwarps..2*nwarps): lane l takes warp l's
// partials and the warp runs one more butterfly, so every thread gets the same bits in 2 loads.
__device__ __forceinline__ void warps_sum(const float* rb, int nwarps, int lane, float& a, float& c) {
    a = lane < nwarps ? rb[lane] : 0.f;
    c = lane < nwarps ? rb[nwarps + lane] : 0.f;
    lanes_sum(a, c, 32);
}

// One CTA per token row (b, s); thread t owns elements 8t..8t+7 of the heads*128 row, i.e.
// 8 consecutive dims of head (8t)/128.  blockDim.x = heads*16.
template <int MAXT, int MINB>
__global__ void __launch_bounds__(MAXT, MINB) fv_wan_qk_prep_kernel(const Params p) {
    extern __shared__ float red[];  // [2][nwarps]
    const int row = blockIdx.x;     // b*seq + s
    const int b = row / p.seq, s = row % p.seq;
    const int t = threadIdx.x, lane = t & 31, warp = t >> 5, nwarps = blockDim.x >> 5;
    // The block is rounded up to whole warps; threads past the row take part in the reductions only.
    const bool act = t < p.heads * 16;
    const int h = act ? (8 * t) / kD : 0, pd = act ? (8 * t) % kD : 0;
    const __nv_bfloat16* src = p.proj + (size_t)row * p.width;
    const size_t dst = (((size_t)b * p.heads + h) * p.seq + s) * kD + pd;
    const size_t dst_kv = (((size_t)b * p.heads + h) * p.kv_rows + p.kv_row0 + s) * kD + pd;

    if (p.v_out && act) {
        const uint4 v = *reinterpret_cast<const uint4*>(src + p.col_v + 8 * t);
        *reinterpret_cast<uint4*>(p.v_out + dst_kv) = v;
    }
    // Everything the row needs is requested before the reduction, so the kernel pays one memory round trip, not three:
    // rope factors (cos at the even index, sin at the odd one of each pair; the tables repeat each value twice) and weights.
    float cs[4] = {1.f, 1.f, 1.f, 1.f}, sn[4] = {0.f, 0.f, 0.f, 0.f};
    float wqv[8], wkv[8];
    if (act) {
        if (p.cosv) {
            const float4* cp = reinterpret_cast<const float4*>(p.cosv + (size_t)s * kD + pd);
            const float4* sp = reinterpret_cast<const float4*>(p.sinv + (size_t)s * kD + pd);
            const float4 c0 = __ldg(cp), c1 = __ldg(cp + 1), s0 = __ldg(sp), s1 = __ldg(sp + 1);
            cs[0] = c0.x; cs[1] = c0.z; cs[2] = c1.x; cs[3] = c1.z;
            sn[0] = s0.y; sn[1] = s0.w; sn[2] = s1.y; sn[3] = s1.w;
        }
        if (p.q_out) {
            const float4 w0 = __ldg(reinterpret_cast<const float4*>(p.wq + 8 * t)), w1 = __ldg(reinterpret_cast<const float4*>(p.wq + 8 * t + 4));
            wqv[0] = w0.x; wqv[1] = w0.y; wqv[2] = w0.z; wqv[3] = w0.w; wqv[4] = w1.x; wqv[5] = w1.y; wqv[6] = w1.z; wqv[7] = w1.w;
        }
        if (p.k_out) {
            const float4 w0 = __ldg(reinterpret_cast<const float4*>(p.wk + 8 * t)), w1 = __ldg(reinterpret_cast<const float4*>(p.wk + 8 * t + 4));
            wkv[0] = w0.x; wkv[1] = w0.y; wkv[2] = w0.z; wkv[3] = w0.w; wkv[4] = w1.x; wkv[5] = w1.y; wkv[6] = w1.z; wkv[7] = w1.w;
        }
    }
    float xq[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f}, xk[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    float sq = 0.f, sk = 0.f;
    if (p.q_out && act) {
        unpack8(*reinterpret_cast<const uint4*>(src + p.col_q + 8 * t), xq);
        sq = sumsq8(xq, sq);
    }
    if (p.k_out && act) {
        unpack8(*reinterpret_cast<const uint4*>(src + p.col_k + 8 * t), xk);
        sk = sumsq8(xk, sk);
    }
    // Sum of squares: over the 16 threads of a head (per_head) or over the whole row.
    lanes_sum(sq, sk, p.per_head ? 16 : 32);
    float denom = (float)kD;
    if (!p.per_head) {
        if (lane == 0) {
            red[warp] = sq;
            red[nwarps + warp] = sk;
        }
        __syncthreads();
        warps_sum(red, nwarps, lane, sq, sk);
        denom = (float)(p.heads * kD);
    }
    if (!act) return;
    auto finish = [&](const float (&x)[8], float ss, const float (&wv)[8], __nv_bfloat16* out, size_t dst) {
        const float ms = __fdiv_rn(ss, denom);
        const float inv = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(ms, p.eps)));
        float y[8];
#pragma unroll
        for (int i = 0; i < 8; i++) y[i] = __fmul_rn(__fmul_rn(x[i], inv), wv[i]);
        float o[8];
        if (p.cosv) {
#pragma unroll
            for (int i = 0; i < 8; i += 2) {
                const float c = cs[i >> 1], sv = sn[i >> 1];
                o[i] = __fsub_rn(__fmul_rn(y[i], c), __fmul_rn(y[i + 1], sv));
                o[i + 1] = __fadd_rn(__fmul_rn(y[i], sv), __fmul_rn(y[i + 1], c));
            }
        } else {
#pragma unroll
            for (int i = 0; i < 8; i++) o[i] = y[i];
        }
        *reinterpret_cast<uint4*>(out + dst) =
            make_uint4(pack2(o[0], o[1]), pack2(o[2], o[3]), pack2(o[4], o[5]), pack2(o[6], o[7]));
    };
    if (p.q_out) finish(xq, sq, wqv, p.q_out, dst);
    if (p.k_out) finish(xk, sk, wkv, p.k_out, dst_kv);
}


// ---- the same arithmetic with a group of warps per row, rows held in registers ------------------------
// A group of G warps (G = 1, 2 or 4 by row width) owns a row; thread g of the group holds the 8-value
// chunks g, g + 32 G, g + 64 G, ... of q and of k as packed bf16 (J chunks each, 16-byte loads, all issued
// before anything is used; v's chunks are requested first and stored as they arrive).  Groups are
// independent: the only synchronisation is one named barrier among the G warps of a group per row, for the
// exchange of the per-warp partial sums.  Several groups per CTA and several CTAs per SM keep enough rows
// in flight to cover the memory latency without a staging ring, a copy unit or a wait that could run out.
// The reduction tree is the row kernel's, bit for bit: chunk c is that kernel's thread c, so warp gw of the
// group holds, in its iteration j, exactly the 32 partials of that kernel's warp gw + G j in the same lanes;
// the butterflies and the exchange through red[] are the same.
template <int J, int G, int NG, int MINB>
__global__ void __launch_bounds__(32 * G * NG, MINB) fv_wan_qk_prep_group_kernel(const Params p, long long rows) {
    __shared__ float red[2][NG][2][32];
    const int t = threadIdx.x, lane = t & 31;
    const int grp = t / (32 * G), g = t % (32 * G), gw = g >> 5;
    const int chunks = p.heads * 16, nwarps = (chunks + 31) >> 5;
    const int pd = 8 * (g & 15);  // (8 c) % 128 is the same for every chunk of a thread: 32 G is a multiple of 16
    const float denom = p.per_head ? (float)kD : (float)(p.heads * kD);
    const int span = p.per_head ? 16 : 32;
    const long long stride = (long long)gridDim.x * NG;
    int it = 0;
    for (long long row = (long long)blockIdx.x * NG + grp; row < rows; row += stride, it ^= 1) {
        const int b = (int)(row / p.seq), s = (int)(row % p.seq);
        const __nv_bfloat16* src = p.proj + (size_t)row * p.width;
        uint4 vq[J], vk[J];
        if (p.v_out) {
            uint4 vv[J];
#pragma unroll
            for (int j = 0; j < J; j++) {
                const int c = g + 32 * G * j;
                if (c < chunks) vv[j] = __ldcs(reinterpret_cast<const uint4*>(src + p.col_v + 8 * c));
            }
#pragma unroll
            for (int j = 0; j < J; j++) {
                const int c = g + 32 * G * j;
                vq[j] = make_uint4(0u, 0u, 0u, 0u);
                if (p.q_out && c < chunks) vq[j] = __ldcs(reinterpret_cast<const uint4*>(src + p.col_q + 8 * c));
            }
#pragma unroll
            for (int j = 0; j < J; j++) {
                const int c = g + 32 * G * j;
                vk[j] = make_uint4(0u, 0u, 0u, 0u);
                if (p.k_out && c < chunks) vk[j] = __ldcs(reinterpret_cast<const uint4*>(src + p.col_k + 8 * c));
            }
#pragma unroll
            for (int j = 0; j < J; j++) {
                const int c = g + 32 * G * j;
                if (c < chunks)
                    *reinterpret_cast<uint4*>(p.v_out + (((size_t)b * p.heads + (c >> 4)) * p.kv_rows + p.kv_row0 + s) * kD + pd) = vv[j];
            }
        } else {
#pragma unroll
            for (int j = 0; j < J; j++) {
                const int c = g + 32 * G * j;
                vq[j] = vk[j] = make_uint4(0u, 0u, 0u, 0u);
                if (p.q_out && c < chunks) vq[j] = __ldcs(reinterpret_cast<const uint4*>(src + p.col_q + 8 * c));
                if (p.k_out && c < chunks) vk[j] = __ldcs(reinterpret_cast<const uint4*>(src + p.col_k + 8 * c));
            }
        }
        float cs[4] = {1.f, 1.f, 1.f, 1.f}, sn[4] = {0.f, 0.f, 0.f, 0.f};
        if (p.cosv) {
            const float4* cp = reinterpret_cast<const float4*>(p.cosv + (size_t)s * kD + pd);
            const float4* sp = reinterpret_cast<const float4*>(p.sinv + (size_t)s * kD + pd);
            const float4 c0 = __ldg(cp), c1 = __ldg(cp + 1), s0 = __ldg(sp), s1 = __ldg(sp + 1);
            cs[0] = c0.x; cs[1] = c0.z; cs[2] = c1.x; cs[3] = c1.z;
            sn[0] = s0.y; sn[1] = s0.w; sn[2] = s1.y; sn[3] = s1.w;
        }
        // per-chunk sums of squares, then the row kernel's butterflies warp by warp
        float sq[J], sk[J];
#pragma unroll
        for (int j = 0; j < J; j++) {
            float x[8];
            unpack8(vq[j], x);
            sq[j] = sumsq8(x, 0.f);
            unpack8(vk[j], x);
            sk[j] = sumsq8(x, 0.f);
        }
#pragma unroll
        for (int j = 0; j < J; j++) lanes_sum(sq[j], sk[j], span);
        float tq = 0.f, tk = 0.f;
        if (!p.per_head) {
            float* rb = &red[it][grp][0][0];
            if (lane == 0) {
#pragma unroll
                for (int j = 0; j < J; j++) {
                    const int w = gw + G * j;
                    if (w < 32) {
                        rb[w] = sq[j];
                        rb[32 + w] = sk[j];
                    }
                }
            }
            if (G == 1) __syncwarp();
            else asm volatile("bar.sync %0, %1;" ::"r"(1 + grp), "r"(32 * G) : "memory");
            tq = lane < nwarps ? rb[lane] : 0.f;
            tk = lane < nwarps ? rb[32 + lane] : 0.f;
            lanes_sum(tq, tk, 32);
        }
#pragma unroll
        for (int j = 0; j < J; j++) {
            const int c = g + 32 * G * j;
            if (c >= chunks) continue;
            const size_t plane = (size_t)b * p.heads + (c >> 4);
            const size_t dst_q = (plane * p.seq + s) * kD + pd, dst_kv = (plane * p.kv_rows + p.kv_row0 + s) * kD + pd;
            auto finish = [&](const uint4& raw, float ss, const float* wsrc, __nv_bfloat16* out, size_t dst) {
                float x[8];
                unpack8(raw, x);
                const float4 w0 = __ldg(reinterpret_cast<const float4*>(wsrc + 8 * c)), w1 = __ldg(reinterpret_cast<const float4*>(wsrc + 8 * c + 4));
                const float wv[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
                const float ms = __fdiv_rn(ss, denom);
                const float inv = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(ms, p.eps)));
                float y[8], o[8];
#pragma unroll
                for (int i = 0; i < 8; i++) y[i] = __fmul_rn(__fmul_rn(x[i], inv), wv[i]);
                if (p.cosv) {
#pragma unroll
                    for (int i = 0; i < 8; i += 2) {
                        const float cc = cs[i >> 1], sv = sn[i >> 1];
                        o[i] = __fsub_rn(__fmul_rn(y[i], cc), __fmul_rn(y[i + 1], sv));
                        o[i + 1] = __fadd_rn(__fmul_rn(y[i], sv), __fmul_rn(y[i + 1], cc));
                    }
                } else {
#pragma unroll
                    for (int i = 0; i < 8; i++) o[i] = y[i];
                }
                *reinterpret_cast<uint4*>(out + dst) =
                    make_uint4(pack2(o[0], o[1]), pack2(o[2], o[3]), pack2(o[4], o[5]), pack2(o[6], o[7]));
            };
            if (p.q_out) finish(vq[j], p.per_head ? sq[j] : tq, p.wq, p.q_out, dst_q);
            if (p.k_out) finish(vk[j], p.per_head ? sk[j] : tk, p.wk, p.k_out, dst_kv);
        }
    }
}

template <int G, int NG>
int launch_group(const Params& p, long long rows, int j_need, int sms, cudaStream_t stream) {
    auto go = [&](auto kern, int per_sm) -> int {
        long long grid = (long long)sms * per_sm;
        const long long need = (rows + NG - 1) / NG;
        if (grid > need) grid = need;
        kern<<<(unsigned)grid, 32 * G * NG, 0, stream>>>(p, rows);
        FV_CUDA(cudaGetLastError());
        return FV_RAN;
    };
    switch (j_need) {
        case 1: return go(fv_wan_qk_prep_group_kernel<1, G, NG, 4>, 4);
        case 2: return go(fv_wan_qk_prep_group_kernel<2, G, NG, 4>, 4);
        case 3: return go(fv_wan_qk_prep_group_kernel<3, G, NG, 2>, 2);
        case 4: return go(fv_wan_qk_prep_group_kernel<4, G, NG, 2>, 2);
        default: return go(fv_wan_qk_prep_group_kernel<5, G, NG, 2>, 2);
    }
}

}  // namespace fvprep

static int qk_prep_impl(void* stream, const void* proj, int width, int col_q, int col_k, int col_v, const float* wq,
                        const float* wk, const float* cosv, const float* sinv, int batch, int seq, int heads, int d, float eps,
                        int norm_scope, void* q_out, void* k_out, void* v_out, int kv_rows, int kv_row0);

extern "C" int fv_wan_qk_prep_bf16(void* stream, const void* proj, int width, int col_q, int col_k, int col_v,
                                   const float* wq, const float* wk, const float* cosv, const float* sinv, int batch,
                                   int seq, int heads, int d, float eps, int norm_scope, void* q_out, void* k_out,
                                   void* v_out) {
    return qk_prep_impl(stream, proj, width, col_q, col_k, col_v, wq, wk, cosv, sinv, batch, seq, heads, d, eps, norm_scope, q_out,
                        k_out, v_out, seq, 0);
}

extern "C" int fv_wan_qk_prep_cache_bf16(void* stream, const void* proj, int width, int col_q, int col_k, int col_v,
                                         const float* wq, const float* wk, const float* cosv, const float* sinv, int batch,
                                         int seq, int heads, int d, float eps, int norm_scope, void* q_out, void* k_cache,
                                         void* v_cache, int cache_rows, int cache_row0) {
    if (cache_rows <= 0 || cache_row0 < 0 || (long long)cache_row0 + seq > cache_rows) {
        fvrt::clear_error();
        return fvrt::fail(FV_ERR_INVALID, "qk_prep: %d tokens at row %d do not fit a cache of %d rows", seq, cache_row0, cache_rows);
    }
    return qk_prep_impl(stream, proj, width, col_q, col_k, col_v, wq, wk, cosv, sinv, batch, seq, heads, d, eps, norm_scope, q_out,
                        k_cache, v_cache, cache_rows, cache_row0);
}

static int qk_prep_impl(void* stream, const void* proj, int width, int col_q, int col_k, int col_v, const float* wq,
                        const float* wk, const float* cosv, const float* sinv, int batch, int seq, int heads, int d, float eps,
                        int norm_scope, void* q_out, void* k_out, void* v_out, int kv_rows, int kv_row0) {
    fvrt::clear_error();
    if (d != 128 || batch <= 0 || seq <= 0 || heads <= 0 || heads > 64) return FV_DECLINED;
    if ((long long)batch * seq > 0x7fffffffll) return FV_DECLINED;
    int dev;
    int rc = fvrt::require_sm100(&dev);
    if (rc != FV_RAN) return rc;
    if (!proj || (!q_out && !k_out && !v_out)) return fvrt::fail(FV_ERR_INVALID, "qk_prep: null operand");
    if ((q_out && !wq) || (k_out && !wk)) return fvrt::fail(FV_ERR_INVALID, "qk_prep: missing norm weight");
    if ((cosv == nullptr) != (sinv == nullptr)) return fvrt::fail(FV_ERR_INVALID, "qk_prep: cos and sin go together");
    if (norm_scope != FV_NORM_ACROSS_HEADS && norm_scope != FV_NORM_PER_HEAD)
        return fvrt::fail(FV_ERR_INVALID, "qk_prep: unknown norm scope %d", norm_scope);
    const int dim = heads * d;
    auto bad_col = [&](int c) { return c < 0 || (c & 7) || c + dim > width; };
    if ((width & 7) || (q_out && bad_col(col_q)) || (k_out && bad_col(col_k)) || (v_out && bad_col(col_v)))
        return fvrt::fail(FV_ERR_INVALID, "qk_prep: columns must be multiples of 8 inside the row (width %d)", width);
    const uintptr_t al = (uintptr_t)proj | (uintptr_t)q_out | (uintptr_t)k_out | (uintptr_t)v_out | (uintptr_t)wq |
                         (uintptr_t)wk | (uintptr_t)cosv | (uintptr_t)sinv;
    if (al & 15) return fvrt::fail(FV_ERR_INVALID, "qk_prep: pointers must be 16-byte aligned");
    fvprep::Params p{};
    p.proj = (const __nv_bfloat16*)proj;
    p.wq = wq;
    p.wk = wk;
    p.cosv = cosv;
    p.sinv = sinv;
    p.q_out = (__nv_bfloat16*)q_out;
    p.k_out = (__nv_bfloat16*)k_out;
    p.v_out = (__nv_bfloat16*)v_out;
    p.batch = batch;
    p.seq = seq;
    p.heads = heads;
    p.width = width;
    p.col_q = col_q;
    p.col_k = col_k;
    p.col_v = col_v;
    p.eps = eps;
    p.per_head = norm_scope == FV_NORM_PER_HEAD;
    p.kv_rows = kv_rows;
    p.kv_row0 = kv_row0;
    const int threads = (heads * 16 + 31) & ~31;
    const char* which = getenv("FV_PREP_KERNEL");  // "row": the one-CTA-per-row kernel (A/B timing and the bit-equality test)
    if (!which || which[0] != 'r') {
        int sms = 0;
        rc = fvrt::sm_count(dev, &sms);
        if (rc != FV_RAN) return rc;
        const long long rows = (long long)batch * seq;
        const int chunks = heads * 16;
        // warps per row: 8 above 40 heads, 4 above 16, 2 above 8, else 1; chunks per thread follow (at most 5)
        const int G = heads > 40 ? 8 : (heads > 16 ? 4 : (heads > 8 ? 2 : 1));
        if (G == 8) rc = fvprep::launch_group<8, 1>(p, rows, (chunks + 255) / 256, sms, (cudaStream_t)stream);
        else if (G == 4) rc = fvprep::launch_group<4, 2>(p, rows, (chunks + 127) / 128, sms, (cudaStream_t)stream);
        else if (G == 2) rc = fvprep::launch_group<2, 4>(p, rows, (chunks + 63) / 64, sms, (cudaStream_t)stream);
        else rc = fvprep::launch_group<1, 8>(p, rows, (chunks + 31) / 32, sms, (cudaStream_t)stream);
        if (rc == FV_RAN)
            fvrt::ran(fvrt::kLogPrep, "qk_prep: fv_wan_qk_prep_group_kernel (%d warps per row, rows in registers) %lld rows x %d heads", G, rows, heads);
        return rc;
    }
    const size_t smem = 2 * (threads / 32 + 1) * sizeof(float);
    // up to 40 heads: 640-thread blocks, two per SM (register cap 51); beyond: one block of up to 1024 threads
    if (threads <= 640)
        fvprep::fv_wan_qk_prep_kernel<640, 2><<<(unsigned)(batch * seq), threads, smem, (cudaStream_t)stream>>>(p);
    else
        fvprep::fv_wan_qk_prep_kernel<1024, 1><<<(unsigned)(batch * seq), threads, smem, (cudaStream_t)stream>>>(p);
    FV_CUDA(cudaGetLastError());
    return FV_RAN;
}

// 3-D RoPE tables of Wan on the host: wan_rope_at / rotary_1d,
// crates/fastvideo-cudarc/src/wan/transformer.rs:447-463,490-544.  freq = 1/theta^(2i/dim) in f64
// narrowed to f32, angle = position (f32) * freq in f32, cosf / sinf, each value twice
// (interleaved pairs); row = [t | h | w] with h = w = 2*(d/6), t = d - h - w.
extern "C" int fv_wan_rope_tables(int ppf, int pph, int ppw, int d, double theta, int start_frame, float* cos_host,
                                  float* sin_host) {
    fvrt::clear_error();
    if (ppf <= 0 || pph <= 0 || ppw <= 0 || d <= 0 || (d & 1) || start_frame < 0 || !cos_host || !sin_host)
        return fvrt::fail(FV_ERR_INVALID, "rope tables: bad grid (%d, %d, %d) or head dim %d", ppf, pph, ppw, d);
    const int h_dim = 2 * (d / 6), w_dim = h_dim, t_dim = d - h_dim - w_dim;
    auto axis = [&](int dim, int n, std::vector<float>& c, std::vector<float>& s) {
        c.assign((size_t)n * dim, 0.f);
        s.assign((size_t)n * dim, 0.f);
        for (int i = 0; i < dim / 2; i++) {
            const float freq = (float)(1.0 / pow(theta, 2.0 * (double)i / (double)dim));
            for (int pos = 0; pos < n; pos++) {
                const float arg = (float)pos * freq;
                const float cv = cosf(arg), sv = sinf(arg);
                c[(size_t)pos * dim + 2 * i] = c[(size_t)pos * dim + 2 * i + 1] = cv;
                s[(size_t)pos * dim + 2 * i] = s[(size_t)pos * dim + 2 * i + 1] = sv;
            }
        }
    };
    std::vector<float> ct, st, ch, sh, cw, sw;
    axis(t_dim, start_frame + ppf, ct, st);
    axis(h_dim, pph, ch, sh);
    axis(w_dim, ppw, cw, sw);
    size_t o = 0;
    for (int ft = start_frame; ft < start_frame + ppf; ft++)
        for (int fh = 0; fh < pph; fh++)
            for (int fw = 0; fw < ppw; fw++) {
                memcpy(cos_host + o, &ct[(size_t)ft * t_dim], sizeof(float) * t_dim);
                memcpy(sin_host + o, &st[(size_t)ft * t_dim], sizeof(float) * t_dim);
                o += t_dim;
                memcpy(cos_host + o, &ch[(size_t)fh * h_dim], sizeof(float) * h_dim);
                memcpy(sin_host + o, &sh[(size_t)fh * h_dim], sizeof(float) * h_dim);
                o += h_dim;
                memcpy(cos_host + o, &cw[(size_t)fw * w_dim], sizeof(float) * w_dim);
                memcpy(sin_host + o, &sw[(size_t)fw * w_dim], sizeof(float) * w_dim);
                o += w_dim;
            }
    return FV_RAN;
}
