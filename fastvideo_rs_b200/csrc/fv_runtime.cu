#include "fv_runtime.h"
#include <mutex>
#include <stdio.h>
#include <string.h>
#include <stdlib.h>

namespace fvrt {

static thread_local char g_err[512] = "";

int fail(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
    return code;
}
void clear_error() { g_err[0] = 0; }

static const int kMaxDev = 64;
static std::mutex g_mu;
static int g_sm[kMaxDev];      // 0 = not probed, else major*10+minor
static int g_sms[kMaxDev];     // 0 = not probed, else the number of SMs
static int* g_status[kMaxDev];
// The kernels' status word (and room to spare): part of the module image, zero at load, one instance
// per device that loads the library.  Host code only ever uses its address, taken once per device.
static __device__ __align__(256) int fv_status_block[64];

int require_sm100(int* device_out) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess || dev < 0 || dev >= kMaxDev) {
        cudaGetLastError();
        return fail(FV_ERR_NO_DEVICE, "no CUDA device is current (%s); this library has no CPU path",
                    e == cudaSuccess ? "bad index" : cudaGetErrorString(e));
    }
    int sm;
    {
        std::lock_guard<std::mutex> lk(g_mu);
        sm = g_sm[dev];
    }
    if (sm == 0) {
        int major = 0, minor = 0;
        FV_CUDA(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev));
        FV_CUDA(cudaDeviceGetAttribute(&minor, cudaDevAttrComputeCapabilityMinor, dev));
        sm = major * 10 + minor;
        std::lock_guard<std::mutex> lk(g_mu);
        g_sm[dev] = sm;
    }
    if (sm != 100 && sm != 103)
        return fail(FV_ERR_NO_DEVICE, "device %d is sm_%d; these kernels are built for sm_100a only", dev, sm);
    if (device_out) *device_out = dev;
    return FV_RAN;
}

int status_word(int device, int** ptr_out) {
    std::lock_guard<std::mutex> lk(g_mu);
    if (!g_status[device]) {
        int* p = nullptr;
        cudaError_t e = cudaGetSymbolAddress((void**)&p, fv_status_block);  // `device` is current (require_sm100)
        if (e != cudaSuccess || !p)
            return fail(FV_ERR_CUDA, "cudaGetSymbolAddress(status block) on device %d: %s", device, cudaGetErrorString(e));
        g_status[device] = p;
    }
    *ptr_out = g_status[device];
    return FV_RAN;
}

int sm_count(int device, int* out) {
    std::lock_guard<std::mutex> lk(g_mu);
    if (!g_sms[device]) {
        int n = 0;
        FV_CUDA(cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, device));
        g_sms[device] = n > 0 ? n : 1;
    }
    *out = g_sms[device];
    return FV_RAN;
}

// SMs the calling thread's NEXT attention launch leaves free (fv_hint_spare_sms); read and cleared by that launch.
static thread_local int g_spare_sms = 0;
int take_spare_sms() {
    const int n = g_spare_sms;
    g_spare_sms = 0;
    return n;
}

static thread_local char g_last_kernel[256] = "";
static bool g_logged[kLogKeys];

void ran(LogKey key, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_last_kernel, sizeof(g_last_kernel), fmt, ap);
    va_end(ap);
    bool first;
    {
        std::lock_guard<std::mutex> lk(g_mu);
        first = !g_logged[key];
        g_logged[key] = true;
    }
    if (first) {
        const char* e = getenv("FV_LOG");
        if (!e || strcmp(e, "0") != 0) fprintf(stderr, "fvsdpa: %s\n", g_last_kernel);
    }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn g_encode = nullptr;

int encode_map4(CUtensorMap* map, const void* base, const uint64_t dims[4], const uint64_t strides[3],
                uint32_t box_rows) {
    if (!g_encode) {
        std::lock_guard<std::mutex> lk(g_mu);
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult qres;
        FV_CUDA(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres));
        if (!fn || qres != cudaDriverEntryPointSuccess)
            return fail(FV_ERR_CUDA, "the driver does not export cuTensorMapEncodeTiled");
        g_encode = (EncodeTiledFn)fn;
    }
    cuuint64_t d[4] = {dims[0], dims[1], dims[2], dims[3]};
    cuuint64_t s[3] = {strides[0], strides[1], strides[2]};
    cuuint32_t box[4] = {64, box_rows, 1, 1};
    cuuint32_t es[4] = {1, 1, 1, 1};
    CUresult r = g_encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), d, s, box, es,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS)
        return fail(FV_ERR_CUDA, "cuTensorMapEncodeTiled failed (%d): dims %llu,%llu,%llu,%llu strides %llu,%llu,%llu", (int)r,
                    (unsigned long long)d[0], (unsigned long long)d[1], (unsigned long long)d[2], (unsigned long long)d[3],
                    (unsigned long long)s[0], (unsigned long long)s[1], (unsigned long long)s[2]);
    return FV_RAN;
}

struct MapKey {
    const void* base;
    uint64_t dims[4], strides[3];
    uint32_t box_rows;
};
static const int kMapSlots = 32;
static MapKey g_map_key[kMapSlots];
static CUtensorMap g_map_val[kMapSlots];
static int g_map_used = 0, g_map_next = 0;

int encode_map4_cached(CUtensorMap* map, const void* base, const uint64_t dims[4], const uint64_t strides[3],
                       uint32_t box_rows) {
    MapKey k;
    memset(&k, 0, sizeof(k));
    k.base = base;
    for (int i = 0; i < 4; i++) k.dims[i] = dims[i];
    for (int i = 0; i < 3; i++) k.strides[i] = strides[i];
    k.box_rows = box_rows;
    {
        std::lock_guard<std::mutex> lk(g_mu);
        for (int i = 0; i < g_map_used; i++)
            if (memcmp(&g_map_key[i], &k, sizeof(k)) == 0) {
                *map = g_map_val[i];
                return FV_RAN;
            }
    }
    const int rc = encode_map4(map, base, dims, strides, box_rows);
    if (rc != FV_RAN) return rc;
    std::lock_guard<std::mutex> lk(g_mu);
    const int slot = g_map_used < kMapSlots ? g_map_used++ : (g_map_next++ % kMapSlots);
    g_map_key[slot] = k;
    g_map_val[slot] = *map;
    return FV_RAN;
}

}  // namespace fvrt

extern "C" const char* fv_last_kernel(void) { return fvrt::g_last_kernel; }

extern "C" int fv_hint_spare_sms(int sms) {
    fvrt::clear_error();
    if (sms < 0 || sms > 128) return fvrt::fail(FV_ERR_INVALID, "spare SMs: %d (0 .. 128)", sms);
    fvrt::g_spare_sms = sms;
    return FV_RAN;
}
extern "C" const char* fv_last_error(void) { return fvrt::g_err; }
extern "C" const char* fv_version(void) { return "fvsdpa 0.1 (sm_100a)"; }

extern "C" int fv_device_status(void* stream, int* code_out) {
    fvrt::clear_error();
    int dev;
    int rc = fvrt::require_sm100(&dev);
    if (rc != FV_RAN) return rc;
    int* w;
    rc = fvrt::status_word(dev, &w);
    if (rc != FV_RAN) return rc;
    int code = 0;
    FV_CUDA(cudaMemcpyAsync(&code, w, sizeof(int), cudaMemcpyDeviceToHost, (cudaStream_t)stream));
    FV_CUDA(cudaStreamSynchronize((cudaStream_t)stream));
    if (code_out) *code_out = code;
    if (code != 0) {
        FV_CUDA(cudaMemsetAsync(w, 0, sizeof(int), (cudaStream_t)stream));
        FV_CUDA(cudaStreamSynchronize((cudaStream_t)stream));
        return fvrt::fail(FV_ERR_DEVICE_STATUS, "a kernel gave up a bounded wait (status %d: role %d)", code, code - 100);
    }
    return FV_RAN;
}
