// Driver for the REFERENCE's own attention kernels (the incumbent this repository is measured against and
// checked against): it #includes the reference's CUDA sources from $FV_REFERENCE_ROOT at build time --
// nothing of the reference is copied into this repository -- and launches, with the reference's own
// geometry,
//   dc100   fa_dc100_fwd_d128          crates/fastvideo-cudarc/src/rt/attn_dc.cu:480-488,
//                                      launch: rt/attn_dc.rs:213-273 (grid (ceil(sq/256), bh) x 384, DC100_SMEM(4))
//   v2      flash_mma_fwd2_d128        rt/kernels/attn2.cu:607-621, launch: rt/attn.rs:378-395
//   causal  flash_mma_fwd2_causal_d128 rt/kernels/attn2.cu:626-633, launch: rt/attn.rs:689-699
// on tensors the caller supplies as raw bf16 files (so the same seeded inputs go through this repository's
// kernels, the reference's kernels and the CPU oracle), writes the bf16 output, and times the launch with
// CUDA events.
//
//   incumbent_driver <dc100|v2|causal> <bh> <sq> <sk> [--mask bt,win,sink] [--in q.bin k.bin v.bin]
//                    [--out out.bin] [--bench iterations]
// Without --in the operands are N(0,1)-like values from a fixed LCG (timing only).  One JSON line on stdout.
#include <algorithm>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>
#include <cuda.h>
#include <cuda_runtime.h>

#include "crates/fastvideo-cudarc/src/rt/kernels/core.cu"
#include "crates/fastvideo-cudarc/src/rt/kernels/sol.cu"
#include "crates/fastvideo-cudarc/src/rt/kernels/attn2.cu"
#include "crates/fastvideo-cudarc/src/rt/kernels/attn3.cu"
#include "crates/fastvideo-cudarc/src/rt/kernels/moe.cu"
#include "crates/fastvideo-cudarc/src/rt/kernels/nvfp4.cu"
#include "crates/fastvideo-cudarc/src/ltx2/kernels/dit.cu"
#include "crates/fastvideo-cudarc/src/rt/kernels/act16.cu"
#include "crates/fastvideo-cudarc/src/h3/kernels/block_ops.cu"
#include "crates/fastvideo-cudarc/src/h3/kernels/video_vae.cu"
#include "crates/fastvideo-cudarc/src/ltx2/kernels/video_vae.cu"
#include "crates/fastvideo-cudarc/src/rt/kernels/dit_fusions.cu"
#include "crates/fastvideo-cudarc/src/wan/kernels/block.cu"
#include "crates/fastvideo-cudarc/src/rt/kernels/lora_fuse.cu"
#include "crates/fastvideo-cudarc/src/rt/attn_dc.cu"

#define CK(x)                                                                                     \
    do {                                                                                          \
        cudaError_t e_ = (x);                                                                     \
        if (e_ != cudaSuccess) {                                                                  \
            printf("{\"fatal\": \"%s:%d %s\"}\n", __FILE__, __LINE__, cudaGetErrorString(e_));   \
            return 3;                                                                             \
        }                                                                                         \
    } while (0)

typedef CUresult (*EncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                             const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                             CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// The 3-D map the reference encodes for its dc kernels (rt/attn_dc.rs:128-148): (d, s, bh), box 64 x 128 x 1,
// 128-byte swizzle, rows past s read as zero.
static bool encode3(DcTensorMap* out, const void* ptr, int s, int bh) {
    static EncodeFn fn = nullptr;
    if (!fn) {
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", (void**)&fn, cudaEnableDefault, &q) != cudaSuccess || !fn) return false;
    }
    CUtensorMap m;
    cuuint64_t dims[3] = {128, (cuuint64_t)s, (cuuint64_t)bh};
    cuuint64_t strides[2] = {256, (cuuint64_t)s * 256};
    cuuint32_t box[3] = {64, 128, 1}, es[3] = {1, 1, 1};
    if (fn(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, (void*)ptr, dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
           CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return false;
    memcpy(out, &m, sizeof(m));
    return true;
}

static unsigned short host_bf16(float x) {
    unsigned int u;
    memcpy(&u, &x, 4);
    u += 0x7FFFu + ((u >> 16) & 1u);
    return (unsigned short)(u >> 16);
}

static bool read_file(const char* path, std::vector<unsigned short>& v) {
    FILE* f = fopen(path, "rb");
    if (!f) return false;
    const size_t got = fread(v.data(), 2, v.size(), f);
    fclose(f);
    return got == v.size();
}

int main(int argc, char** argv) {
    if (argc < 5) {
        printf("{\"fatal\": \"usage: incumbent_driver <dc100|v2|causal> bh sq sk [--mask bt,win,sink] [--in q k v] [--out o] [--bench n]\"}\n");
        return 2;
    }
    const std::string kern = argv[1];
    const int bh = atoi(argv[2]), sq = atoi(argv[3]), sk = atoi(argv[4]);
    int bt = 0, win = 0, sink = 0, iters = 0;
    const char *fq = nullptr, *fk = nullptr, *fv = nullptr, *fo = nullptr;
    for (int i = 5; i < argc; i++) {
        if (!strcmp(argv[i], "--mask") && i + 1 < argc) sscanf(argv[++i], "%d,%d,%d", &bt, &win, &sink);
        else if (!strcmp(argv[i], "--in") && i + 3 < argc) { fq = argv[++i]; fk = argv[++i]; fv = argv[++i]; }
        else if (!strcmp(argv[i], "--out") && i + 1 < argc) fo = argv[++i];
        else if (!strcmp(argv[i], "--bench") && i + 1 < argc) iters = atoi(argv[++i]);
    }
    if (bh < 1 || sq < 1 || sk < 1 || bh > 65535 || (kern == "causal" && bt < 1)) {
        printf("{\"fatal\": \"bad shape\"}\n");
        return 2;
    }
    const size_t nq = (size_t)bh * sq * 128, nk = (size_t)bh * sk * 128;
    std::vector<unsigned short> hq(nq), hk(nk), hv(nk);
    if (fq) {
        if (!read_file(fq, hq) || !read_file(fk, hk) || !read_file(fv, hv)) {
            printf("{\"fatal\": \"cannot read the operand files\"}\n");
            return 2;
        }
    } else {
        unsigned long long s = 0x9E3779B97F4A7C15ull;
        auto rnd = [&]() {
            float a = 0.f;
            for (int i = 0; i < 4; i++) {
                s = s * 6364136223846793005ull + 1442695040888963407ull;
                a += (float)((s >> 40) & 0xFFFFFF) / 16777216.0f - 0.5f;
            }
            return a * 1.7320508f;
        };
        std::vector<unsigned short> table(1u << 20);
        for (auto& x : table) x = host_bf16(rnd());
        for (auto* vec : {&hq, &hk, &hv})
            for (auto& x : *vec) {
                s = s * 6364136223846793005ull + 1442695040888963407ull;
                x = table[(s >> 40) & ((1u << 20) - 1)];
            }
    }
    unsigned short *dq, *dk, *dv, *dout;
    float* dummy;
    CK(cudaMalloc(&dq, nq * 2));
    CK(cudaMalloc(&dk, nk * 2));
    CK(cudaMalloc(&dv, nk * 2));
    CK(cudaMalloc(&dout, nq * 2));
    CK(cudaMalloc(&dummy, 256));
    CK(cudaMemcpy(dq, hq.data(), nq * 2, cudaMemcpyHostToDevice));
    CK(cudaMemcpy(dk, hk.data(), nk * 2, cudaMemcpyHostToDevice));
    CK(cudaMemcpy(dv, hv.data(), nk * 2, cudaMemcpyHostToDevice));
    CK(cudaMemset(dout, 0xff, nq * 2));
    const float sl2 = (1.0f / sqrtf(128.f)) * 1.4426950408889634f;  // scale * log2 e (rt/attn.rs:303-304)
    DcTensorMap tq, tk, tv;
    if (kern == "dc100") {
        if (!encode3(&tq, dq, sq, bh) || !encode3(&tk, dk, sk, bh) || !encode3(&tv, dv, sk, bh)) {
            printf("{\"fatal\": \"cuTensorMapEncodeTiled\"}\n");
            return 3;
        }
        CK(cudaFuncSetAttribute(fa_dc100_fwd_d128, cudaFuncAttributeMaxDynamicSharedMemorySize, DC100_SMEM(4)));
    } else if (kern == "v2") {
        CK(cudaFuncSetAttribute(flash_mma_fwd2_d128, cudaFuncAttributeMaxDynamicSharedMemorySize, 4 * 64 * 128 * 2));
    } else if (kern == "causal") {
        CK(cudaFuncSetAttribute(flash_mma_fwd2_causal_d128, cudaFuncAttributeMaxDynamicSharedMemorySize, 4 * 64 * 128 * 2));
    } else {
        printf("{\"fatal\": \"unknown kernel\"}\n");
        return 2;
    }
    auto launch = [&]() {
        if (kern == "dc100") {
            dim3 grid((sq + 255) / 256, bh);
            fa_dc100_fwd_d128<<<grid, 384, DC100_SMEM(4)>>>(tq, tk, tv, dummy, dout, 1, sq, sk, sl2);
        } else if (kern == "v2") {
            dim3 grid((sq + 127) / 128, bh);
            flash_mma_fwd2_d128<<<grid, 256, 4 * 64 * 128 * 2>>>(dq, dk, dv, dummy, dout, 1, sq, sk, sl2);
        } else {
            dim3 grid((sq + 127) / 128, bh);
            flash_mma_fwd2_causal_d128<<<grid, 256, 4 * 64 * 128 * 2>>>(dq, dk, dv, dummy, dout, 1, sq, sk, sl2, bt, win, sink);
        }
    };
    launch();
    CK(cudaGetLastError());
    CK(cudaDeviceSynchronize());
    double ms = 0;
    if (iters > 0) {
        cudaEvent_t e0, e1;
        CK(cudaEventCreate(&e0));
        CK(cudaEventCreate(&e1));
        std::vector<float> t;
        for (int i = 0; i < iters + 2; i++) {
            CK(cudaEventRecord(e0));
            launch();
            CK(cudaEventRecord(e1));
            CK(cudaEventSynchronize(e1));
            float x;
            CK(cudaEventElapsedTime(&x, e0, e1));
            if (i >= 2) t.push_back(x);
        }
        std::sort(t.begin(), t.end());
        ms = t[t.size() / 2];
    }
    if (fo) {
        std::vector<unsigned short> ho(nq);
        CK(cudaMemcpy(ho.data(), dout, nq * 2, cudaMemcpyDeviceToHost));
        FILE* f = fopen(fo, "wb");
        if (!f || fwrite(ho.data(), 2, nq, f) != nq) {
            printf("{\"fatal\": \"cannot write the output file\"}\n");
            return 2;
        }
        fclose(f);
    }
    double vis = (double)sq * sk;
    if (kern == "causal") {
        vis = 0;
        for (int i = 0; i < sq; i++) {
            const long long tqb = i / bt;
            long long hi = std::min<long long>(sk, (tqb + 1) * bt), lo = win > 0 ? std::max<long long>(0, tqb - win + 1) * bt : 0;
            long long snk = std::min<long long>(std::min<long long>(sk, (long long)sink * bt), lo);
            vis += (double)(hi - lo) + (double)snk;
        }
    }
    printf("{\"kernel\": \"%s\", \"bh\": %d, \"sq\": %d, \"sk\": %d, \"mask\": [%d, %d, %d], \"ms\": %.4f, \"tflops\": %.1f}\n", kern.c_str(), bh,
           sq, sk, bt, win, sink, ms, ms > 0 ? 4.0 * bh * vis * 128 / (ms * 1e-3) / 1e12 : 0.0);
    return 0;
}
