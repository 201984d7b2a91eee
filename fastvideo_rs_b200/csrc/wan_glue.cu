// The two HBM-bound passes either side of Wan self-attention, under bf16 activations:
//
//   before   ln_adaln_e: unaffine LayerNorm of the hidden row, then the AdaLN modulation
//            y = LN(x) * (1 + e[b, scale]) + e[b, shift], one rounding to bf16
//            (crates/fastvideo-cudarc/src/rt/kernels/act16.cu:184-209, caller wan/transformer.rs:949-953)
//   after    self_residual_norm: hidden' = h + attn * e[b, gate] in f32 (product and sum rounded
//            separately), stored rounded to bf16; LayerNorm with f32 affine over the UNROUNDED sum,
//            one rounding (wan_res_ln with res_mode 0 / ln_mode 0,
//            crates/fastvideo-cudarc/src/wan/kernels/block.cu:17-78; caller wan/transformer.rs:959-971,
//            host twin wan/fuse.rs:108-166)
//
// The reference runs one CTA per row with strided loops that read the row three times (mean, variance,
// output).  Here a row is read ONCE: a group of G warps (G = 1, 2 or 4 by row width) holds it in
// registers as 16-byte vectors, every lane issuing all its loads before the first reduction, and the
// two statistics are reduced by warp shuffles plus one shared-memory exchange between the G warps.
// CTAs are persistent (a few per SM) and walk the rows with the grid's stride.
// Per row of `dim` values: ln_adaln reads 2 dim bytes and writes 2 dim; self_residual_norm reads 4 dim and
// writes 4 dim; the AdaLN rows and the affine (f32, 3 rows per batch element) stay in L2.
#include "fv_runtime.h"
#include <cuda_bf16.h>
#include <stdint.h>

namespace fvglue {

constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;
constexpr int kVec = 6;  // 16-byte vectors (8 bf16) a lane holds at most: dim <= 8 * 32 * 6 * G

__device__ __forceinline__ float bf_lo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf_hi(uint32_t w) { return __uint_as_float(w & 0xffff0000u); }
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    uint32_t r;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
}
__device__ __forceinline__ void unpack8(const uint4& u, float (&f)[8]) {
    f[0] = bf_lo(u.x); f[1] = bf_hi(u.x); f[2] = bf_lo(u.y); f[3] = bf_hi(u.y);
    f[4] = bf_lo(u.z); f[5] = bf_hi(u.z); f[6] = bf_lo(u.w); f[7] = bf_hi(u.w);
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
    return make_uint4(pack_bf16(f[0], f[1]), pack_bf16(f[2], f[3]), pack_bf16(f[4], f[5]), pack_bf16(f[6], f[7]));
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// Sum over the G warps of a row group.  `slot` is one of two shared arrays (alternating, so that a warp that
// is already at the next reduction cannot overwrite a partial another warp still has to read).
template <int G>
__device__ __forceinline__ float group_sum(float v, float* slot, int warp) {
    v = warp_sum(v);
    if (G == 1) return v;
    if ((threadIdx.x & 31) == 0) slot[warp] = v;
    __syncthreads();
    float t = 0.f;
    const int g0 = warp / G * G;
#pragma unroll
    for (int i = 0; i < G; i++) t += slot[g0 + i];
    return t;
}

struct Geo {
    int rows, seq, dim, e_rows, nvec;  // nvec = dim / 8
};

// MODE 0: ln_adaln_e.  MODE 1: self_residual_norm.
template <int G, int MODE>
__global__ void __launch_bounds__(kThreads, MODE == 0 ? 3 : 2)
fv_wan_glue_kernel(const uint4* __restrict__ x, const uint4* __restrict__ a, const float* __restrict__ e, int slot0, int slot1,
                   const float* __restrict__ w, const float* __restrict__ b, uint4* __restrict__ out0, uint4* __restrict__ out1,
                   Geo g, float eps) {
    __shared__ float red[4][kWarps];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int rows_per_cta = kWarps / G;
    const int sub = warp % G;  // this warp's part of the row
    const float inv_dim = 1.0f / (float)g.dim;
    int it = 0;
    const long stride = (long)gridDim.x * rows_per_cta;
    // The x vectors of a row (MODE 0: requested one row ahead, so that a row's loads are in flight while the
    // row before it goes through its two reductions; MODE 1 has twice the loads per row and does without).
    auto load_x = [&](long row0, uint4 (&dst)[kVec]) -> int {
        const long row = row0 + warp / G;
        int n = 0;
        if (row < g.rows) {
            const long base = row * (long)g.nvec;
#pragma unroll
            for (int i = 0; i < kVec; i++) {
                const int vec = (i * G + sub) * 32 + lane;
                if (vec < g.nvec) {
                    dst[i] = x[base + vec];
                    n = i + 1;
                }
            }
        }
        return n;
    };
    uint4 xr[kVec], nx[kVec];
    int cnt = 0, ncnt = 0;
    if (MODE == 0 && (long)blockIdx.x * rows_per_cta < g.rows) ncnt = load_x((long)blockIdx.x * rows_per_cta, nx);
    for (long row0 = (long)blockIdx.x * rows_per_cta; row0 < g.rows; row0 += stride, it++) {
        const long row = row0 + warp / G;
        const bool live = row < g.rows;  // (a dead warp still takes part in the CTA's barriers)
        const long base = (live ? row : 0) * (long)g.nvec;
        const long tb = (live ? row / g.seq : 0) * (long)g.e_rows;
        float v[MODE == 0 ? 1 : kVec][8];  // MODE 1 keeps the unrounded sums; MODE 0 unpacks xr again in every pass
        uint4 ar[kVec];
        auto vals = [&](int i, float (&f)[8]) {
            if (MODE == 0) {
                unpack8(xr[i], f);
            } else {
#pragma unroll
                for (int c = 0; c < 8; c++) f[c] = v[MODE == 0 ? 0 : i][c];
            }
        };
        if (MODE == 0) {
            cnt = ncnt;
#pragma unroll
            for (int i = 0; i < kVec; i++) xr[i] = nx[i];
            ncnt = row0 + stride < g.rows ? load_x(row0 + stride, nx) : 0;
        } else {
            cnt = load_x(row0, xr);
#pragma unroll
            for (int i = 0; i < kVec; i++) {
                const int vec = (i * G + sub) * 32 + lane;
                if (i < cnt) ar[i] = a[base + vec];
            }
        }
        float s = 0.f;
#pragma unroll
        for (int i = 0; i < kVec; i++) {
            if (i < cnt) {
                float f[8];
                unpack8(xr[i], f);
                if (MODE == 1) {
                    const int vec = (i * G + sub) * 32 + lane;
                    float av[8];
                    unpack8(ar[i], av);
                    const float4* gp = reinterpret_cast<const float4*>(e + (tb + slot0) * (long)g.dim + (long)vec * 8);
                    const float4 g0 = gp[0], g1 = gp[1];
                    const float gg[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
#pragma unroll
                    for (int c = 0; c < 8; c++) f[c] = v[MODE == 0 ? 0 : i][c] = __fadd_rn(f[c], __fmul_rn(av[c], gg[c]));
                    out0[base + vec] = pack8(f);  // the new hidden state, rounded
                }
#pragma unroll
                for (int c = 0; c < 8; c++) s += f[c];
            }
        }
        const float mean = group_sum<G>(s, red[(it & 1) * 2], warp) * inv_dim;
        float q = 0.f;
#pragma unroll
        for (int i = 0; i < kVec; i++) {
            if (i < cnt) {
                float f[8];
                vals(i, f);
#pragma unroll
                for (int c = 0; c < 8; c++) {
                    const float d = f[c] - mean;
                    q = fmaf(d, d, q);
                }
            }
        }
        const float inv = rsqrtf(group_sum<G>(q, red[(it & 1) * 2 + 1], warp) * inv_dim + eps);
#pragma unroll
        for (int i = 0; i < kVec; i++) {
            if (i < cnt) {
                const int vec = (i * G + sub) * 32 + lane;
                float y[8], f[8];
                vals(i, f);
                if (MODE == 0) {
                    const float4* sp = reinterpret_cast<const float4*>(e + (tb + slot0) * (long)g.dim + (long)vec * 8);
                    const float4* hp = reinterpret_cast<const float4*>(e + (tb + slot1) * (long)g.dim + (long)vec * 8);
                    const float4 s0 = sp[0], s1 = sp[1], h0 = hp[0], h1 = hp[1];
                    const float sc[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
                    const float sh[8] = {h0.x, h0.y, h0.z, h0.w, h1.x, h1.y, h1.z, h1.w};
#pragma unroll
                    for (int c = 0; c < 8; c++) y[c] = ((f[c] - mean) * inv) * (1.0f + sc[c]) + sh[c];
                    out0[base + vec] = pack8(y);
                } else {
                    const float4* wp = reinterpret_cast<const float4*>(w + (long)vec * 8);
                    const float4* bp = reinterpret_cast<const float4*>(b + (long)vec * 8);
                    const float4 w0 = wp[0], w1 = wp[1], b0 = bp[0], b1 = bp[1];
                    const float ww[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
                    const float bb[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
#pragma unroll
                    for (int c = 0; c < 8; c++)
                        y[c] = __fadd_rn(__fmul_rn(__fmul_rn(__fsub_rn(f[c], mean), inv), ww[c]), bb[c]);
                    out1[base + vec] = pack8(y);
                }
            }
        }
    }
}

template <int MODE>
static int launch(cudaStream_t stream, const void* x, const void* a, const float* e, int slot0, int slot1, const float* w,
                  const float* b, void* out0, void* out1, int batch, int seq, int dim, int e_rows, float eps) {
    int dev;
    int rc = fvrt::require_sm100(&dev);
    if (rc != FV_RAN) return rc;
    const char* what = MODE == 0 ? "ln_adaln" : "self_residual_norm";
    if (!x || !e || !out0 || (MODE == 1 && (!a || !w || !b || !out1))) return fvrt::fail(FV_ERR_INVALID, "%s: null operand", what);
    if (slot0 < 0 || slot0 >= e_rows || (MODE == 0 && (slot1 < 0 || slot1 >= e_rows)))
        return fvrt::fail(FV_ERR_INVALID, "%s: slot outside the %d rows of the AdaLN table", what, e_rows);
    if (((uintptr_t)x | (uintptr_t)a | (uintptr_t)e | (uintptr_t)w | (uintptr_t)b | (uintptr_t)out0 | (uintptr_t)out1) & 15)
        return fvrt::fail(FV_ERR_INVALID, "%s: operands must be 16-byte aligned", what);
    if (!(eps >= 0.f)) return fvrt::fail(FV_ERR_INVALID, "%s: eps must not be negative", what);
    if (dim % 8 != 0 || dim > 8 * 32 * kVec * 4) return FV_DECLINED;  // rows of up to 6 144 values, whole 16-byte vectors
    const long long rows = (long long)batch * seq;
    if (rows > 0x7fffffffll) return FV_DECLINED;
    Geo g{(int)rows, seq, dim, e_rows, dim / 8};
    const int G = dim <= 8 * 32 * kVec ? 1 : (dim <= 8 * 32 * kVec * 2 ? 2 : 4);
    int sms = 0;
    rc = fvrt::sm_count(dev, &sms);
    if (rc != FV_RAN) return rc;
    const long long want = (rows + kWarps / G - 1) / (kWarps / G);
    const unsigned grid = (unsigned)(want < (long long)sms * 6 ? want : (long long)sms * 6);
    const uint4 *xv = static_cast<const uint4*>(x), *av = static_cast<const uint4*>(a);
    uint4 *o0 = static_cast<uint4*>(out0), *o1 = static_cast<uint4*>(out1);
    if (G == 1) fv_wan_glue_kernel<1, MODE><<<grid, kThreads, 0, stream>>>(xv, av, e, slot0, slot1, w, b, o0, o1, g, eps);
    else if (G == 2) fv_wan_glue_kernel<2, MODE><<<grid, kThreads, 0, stream>>>(xv, av, e, slot0, slot1, w, b, o0, o1, g, eps);
    else fv_wan_glue_kernel<4, MODE><<<grid, kThreads, 0, stream>>>(xv, av, e, slot0, slot1, w, b, o0, o1, g, eps);
    FV_CUDA(cudaGetLastError());
    fvrt::ran(fvrt::kLogGlue, "wan glue: fv_wan_glue_kernel<%d, %s> %u CTAs, %lld rows of %d", G, what, grid, rows, dim);
    return FV_RAN;
}

}  // namespace fvglue

extern "C" int fv_wan_ln_adaln_bf16(void* stream, const void* x, const float* e, int scale_slot, int shift_slot, int batch,
                                    int seq, int dim, int e_rows, float eps, void* out) {
    fvrt::clear_error();
    if (batch <= 0 || seq <= 0 || dim <= 0 || e_rows <= 0) return FV_DECLINED;
    return fvglue::launch<0>((cudaStream_t)stream, x, nullptr, e, scale_slot, shift_slot, nullptr, nullptr, out, nullptr, batch,
                             seq, dim, e_rows, eps);
}

extern "C" int fv_wan_self_residual_norm_bf16(void* stream, const void* hidden, const void* attn, const float* e, int gate_slot,
                                              const float* norm_w, const float* norm_b, int batch, int seq, int dim, int e_rows,
                                              float eps, void* hidden_out, void* normed_out) {
    fvrt::clear_error();
    if (batch <= 0 || seq <= 0 || dim <= 0 || e_rows <= 0) return FV_DECLINED;
    return fvglue::launch<1>((cudaStream_t)stream, hidden, attn, e, gate_slot, 0, norm_w, norm_b, hidden_out, normed_out, batch,
                             seq, dim, e_rows, eps);
}
