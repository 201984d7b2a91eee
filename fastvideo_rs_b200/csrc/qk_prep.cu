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
#include "fv_ptx.cuh"
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

    if (p.v_out && act) {
        const uint4 v = *reinterpret_cast<const uint4*>(src + p.col_v + 8 * t);
        *reinterpret_cast<uint4*>(p.v_out + dst) = v;
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
    auto finish = [&](const float (&x)[8], float ss, const float (&wv)[8], __nv_bfloat16* out) {
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
    if (p.q_out) finish(xq, sq, wqv, p.q_out);
    if (p.k_out) finish(xk, sk, wkv, p.k_out);
}


// ---- the same arithmetic behind a ring of staged rows -----------------------------------------------
// One CTA per row pays the whole DRAM round trip once per row with nothing else in flight.  Here a
// CTA is persistent: it walks rows blockIdx.x, + gridDim.x, ... and keeps `stages` of them in flight
// as bulk copies (q, k, v column ranges of the projection row and the row's cos / sin) into a ring
// in shared memory, each stage completing on an mbarrier.  The block reduction's barrier doubles as
// "every thread has read its part of the stage", after which one thread refills it.  The norm
// weights stay in registers for the CTA's lifetime.  Values and rounding are those of the kernel
// above, bit for bit (same reduction tree).
struct RingGeom {
    int stages;
    uint32_t off_k, off_v, off_cos, off_sin;  // byte offsets inside a stage (q at 0)
    uint32_t stage_bytes;
    long long rows;                            // batch * seq
    int* status;
};

template <int MAXT, int MINB>
__global__ void __launch_bounds__(MAXT, MINB) fv_wan_qk_prep_ring_kernel(const Params p, const RingGeom g) {
    using namespace fvp;
    extern __shared__ __align__(128) unsigned char ring_smem[];
    const int t = threadIdx.x, lane = t & 31, warp = t >> 5, nwarps = blockDim.x >> 5;
    const bool act = t < p.heads * 16;
    const int h = act ? (8 * t) / kD : 0, pd = act ? (8 * t) % kD : 0;
    const uint32_t dimB = (uint32_t)p.heads * kD * 2u;
    const uint32_t base = smem_u32(ring_smem);
    const uint32_t bars = base + (uint32_t)g.stages * g.stage_bytes;
    unsigned char* tail = ring_smem + (size_t)g.stages * g.stage_bytes + 8 * g.stages;
    float* red = reinterpret_cast<float*>(tail);                       // [2][2 * nwarps]
    volatile int* abort_ptr = reinterpret_cast<volatile int*>(tail + 16 * nwarps);

    if (t == 0) {
        for (int s = 0; s < g.stages; s++) mbar_init(bars + 8 * s, 1);
        *abort_ptr = (*(volatile int*)g.status != FV_ST_OK) ? 1 : 0;
        mbar_init_fence();
    }
    __syncthreads();
    if (*abort_ptr) return;  // CTA-uniform
    const WaitCtl ctl{abort_ptr, g.status, 7};

    uint32_t row_bytes = 0;
    if (p.q_out) row_bytes += dimB;
    if (p.k_out) row_bytes += dimB;
    if (p.v_out) row_bytes += dimB;
    if (p.cosv) row_bytes += 2u * kD * 4u;
    auto issue = [&](long long row, int srow, int s) {  // one thread; srow = row % seq
        const uint32_t dst = base + (uint32_t)s * g.stage_bytes, bar = bars + 8 * s;
        const __nv_bfloat16* src = p.proj + (size_t)row * p.width;
        mbar_expect_tx(bar, row_bytes);
        if (p.q_out) bulk_load(dst, src + p.col_q, dimB, bar);
        if (p.k_out) bulk_load(dst + g.off_k, src + p.col_k, dimB, bar);
        if (p.v_out) bulk_load(dst + g.off_v, src + p.col_v, dimB, bar);
        if (p.cosv) {
            const size_t sidx = (size_t)srow * kD;
            bulk_load(dst + g.off_cos, p.cosv + sidx, kD * 4u, bar);
            bulk_load(dst + g.off_sin, p.sinv + sidx, kD * 4u, bar);
        }
    };
    // Row indices advance by gridDim.x; (batch, position) follow by subtraction, the ring slot and its
    // phase by counting: no division inside the loop.
    const int step = (int)gridDim.x;
    auto advance = [&](int& b, int& srow) {
        srow += step;
        while (srow >= p.seq) {
            srow -= p.seq;
            b++;
        }
    };
    long long issued = 0;                    // rows of this CTA handed to the copy unit (thread 0 only)
    long long nrow = (long long)blockIdx.x;  // next row to hand over, its batch and position, its slot
    int nb = (int)(blockIdx.x / (unsigned)p.seq), nsrow = (int)(blockIdx.x % (unsigned)p.seq), nslot = 0;
    if (t == 0) {
        for (; nslot < g.stages && nrow < g.rows; nslot++) {
            issue(nrow, nsrow, nslot);
            issued++;
            nrow += step;
            advance(nb, nsrow);
        }
    }

    float wqv[8], wkv[8];
#pragma unroll
    for (int i = 0; i < 8; i++) wqv[i] = wkv[i] = 0.f;
    if (act && p.q_out) {
        const float4 w0 = __ldg(reinterpret_cast<const float4*>(p.wq + 8 * t)), w1 = __ldg(reinterpret_cast<const float4*>(p.wq + 8 * t + 4));
        wqv[0] = w0.x; wqv[1] = w0.y; wqv[2] = w0.z; wqv[3] = w0.w; wqv[4] = w1.x; wqv[5] = w1.y; wqv[6] = w1.z; wqv[7] = w1.w;
    }
    if (act && p.k_out) {
        const float4 w0 = __ldg(reinterpret_cast<const float4*>(p.wk + 8 * t)), w1 = __ldg(reinterpret_cast<const float4*>(p.wk + 8 * t + 4));
        wkv[0] = w0.x; wkv[1] = w0.y; wkv[2] = w0.z; wkv[3] = w0.w; wkv[4] = w1.x; wkv[5] = w1.y; wkv[6] = w1.z; wkv[7] = w1.w;
    }
    const float denom = p.per_head ? (float)kD : (float)(p.heads * kD);
    const int span = p.per_head ? 16 : 32;

    long long i = 0;
    bool failed = false;
    int b = (int)(blockIdx.x / (unsigned)p.seq), srow = (int)(blockIdx.x % (unsigned)p.seq);
    int s = 0;
    uint32_t ph = 0;
    for (long long row = (long long)blockIdx.x; row < g.rows; row += step, i++) {  // CTA-uniform trip count
        const bool ok = mbar_wait(bars + 8 * s, ph, ctl);
        const unsigned char* st = ring_smem + (size_t)s * g.stage_bytes;
        float xq[8], xk[8];
#pragma unroll
        for (int j = 0; j < 8; j++) xq[j] = xk[j] = 0.f;
        float cs[4] = {1.f, 1.f, 1.f, 1.f}, sn[4] = {0.f, 0.f, 0.f, 0.f};
        uint4 vv = make_uint4(0u, 0u, 0u, 0u);
        float sq = 0.f, sk = 0.f;
        if (ok && act) {
            if (p.q_out) {
                unpack8(*reinterpret_cast<const uint4*>(st + 16 * t), xq);
                sq = sumsq8(xq, sq);
            }
            if (p.k_out) {
                unpack8(*reinterpret_cast<const uint4*>(st + g.off_k + 16 * t), xk);
                sk = sumsq8(xk, sk);
            }
            if (p.v_out) vv = *reinterpret_cast<const uint4*>(st + g.off_v + 16 * t);
            if (p.cosv) {
                const float4* cp = reinterpret_cast<const float4*>(st + g.off_cos + 4 * pd);
                const float4* sp = reinterpret_cast<const float4*>(st + g.off_sin + 4 * pd);
                const float4 c0 = cp[0], c1 = cp[1], s0 = sp[0], s1 = sp[1];
                cs[0] = c0.x; cs[1] = c0.z; cs[2] = c1.x; cs[3] = c1.z;
                sn[0] = s0.y; sn[1] = s0.w; sn[2] = s1.y; sn[3] = s1.w;
            }
        }
        lanes_sum(sq, sk, span);
        float* rb = red + (i & 1) * 2 * nwarps;
        if (lane == 0) {
            rb[warp] = sq;
            rb[nwarps + warp] = sk;
        }
        // One barrier per row: the reduction's, the verdict on the wait, and the release of stage s.
        if (!__syncthreads_and(ok ? 1 : 0)) {
            failed = true;
            break;  // CTA-uniform
        }
        if (t == 0 && nrow < g.rows) {  // the slot just read is the next one to fill
            issue(nrow, nsrow, s);
            issued++;
            nrow += step;
            advance(nb, nsrow);
        }
        if (!p.per_head) warps_sum(rb, nwarps, lane, sq, sk);
        const size_t dst = (((size_t)b * p.heads + h) * p.seq + srow) * kD + pd;
        advance(b, srow);
        if (++s == g.stages) {
            s = 0;
            ph ^= 1u;
        }
        if (!act) continue;
        if (p.v_out) *reinterpret_cast<uint4*>(p.v_out + dst) = vv;
        auto finish = [&](const float (&x)[8], float ss, const float (&wv)[8], __nv_bfloat16* out) {
            const float ms = __fdiv_rn(ss, denom);
            const float inv = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(ms, p.eps)));
            float y[8];
#pragma unroll
            for (int j = 0; j < 8; j++) y[j] = __fmul_rn(__fmul_rn(x[j], inv), wv[j]);
            float o[8];
            if (p.cosv) {
#pragma unroll
                for (int j = 0; j < 8; j += 2) {
                    const float c = cs[j >> 1], sv = sn[j >> 1];
                    o[j] = __fsub_rn(__fmul_rn(y[j], c), __fmul_rn(y[j + 1], sv));
                    o[j + 1] = __fadd_rn(__fmul_rn(y[j], sv), __fmul_rn(y[j + 1], c));
                }
            } else {
#pragma unroll
                for (int j = 0; j < 8; j++) o[j] = y[j];
            }
            *reinterpret_cast<uint4*>(out + dst) =
                make_uint4(pack2(o[0], o[1]), pack2(o[2], o[3]), pack2(o[4], o[5]), pack2(o[6], o[7]));
        };
        if (p.q_out) finish(xq, sq, wqv, p.q_out);
        if (p.k_out) finish(xk, sk, wkv, p.k_out);
    }
    // A wait ran out: copies already handed to the copy unit must land before the ring goes away.
    if (failed && t == 0) {
        for (long long j = i; j < issued; j++)
            if (!mbar_drain(bars + 8 * (uint32_t)(j % g.stages), (uint32_t)((j / g.stages) & 1))) break;
    }
}

}  // namespace fvprep

extern "C" int fv_wan_qk_prep_bf16(void* stream, const void* proj, int width, int col_q, int col_k, int col_v,
                                   const float* wq, const float* wk, const float* cosv, const float* sinv, int batch,
                                   int seq, int heads, int d, float eps, int norm_scope, void* q_out, void* k_out,
                                   void* v_out) {
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
    const int threads = (heads * 16 + 31) & ~31;
    const char* which = getenv("FV_PREP_KERNEL");  // "row": the one-CTA-per-row kernel (A/B timing)
    if (!(which && which[0] == 'r')) {
        // ring geometry: stage = q | k | v | cos | sin; as many stages as fit, several CTAs per SM for narrow rows
        const uint32_t dimB = (uint32_t)dim * 2u;
        fvprep::RingGeom g{};
        g.off_k = dimB;
        g.off_v = 2 * dimB;
        g.off_cos = 3 * dimB;
        g.off_sin = 3 * dimB + 512;
        g.stage_bytes = 3 * dimB + 1024;
        g.rows = (long long)batch * seq;
        rc = fvrt::status_word(dev, &g.status);
        if (rc != FV_RAN) return rc;
        const int ctas_per_sm = threads <= 256 ? 4 : (threads <= 320 ? 2 : 1);
        const uint32_t budget = (200u / (uint32_t)ctas_per_sm) * 1024u;
        g.stages = (int)(budget / g.stage_bytes);
        if (g.stages > 8) g.stages = 8;
        if (g.stages < 2) g.stages = 2;
        const size_t extra = 8 * (size_t)g.stages + 16 * (size_t)(threads / 32) + 16;
        const size_t smem_ring = (size_t)g.stages * g.stage_bytes + extra;
        int sms = 0;
        FV_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
        long long grid = (long long)sms * ctas_per_sm;
        if (grid > g.rows) grid = g.rows;
        auto run = [&](auto kern) -> int {
            FV_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_ring));
            kern<<<(unsigned)grid, threads, smem_ring, (cudaStream_t)stream>>>(p, g);
            FV_CUDA(cudaGetLastError());
            return FV_RAN;
        };
        if (threads <= 256) return run(fvprep::fv_wan_qk_prep_ring_kernel<256, 4>);
        if (threads <= 640) return run(fvprep::fv_wan_qk_prep_ring_kernel<640, 1>);
        return run(fvprep::fv_wan_qk_prep_ring_kernel<1024, 1>);
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
