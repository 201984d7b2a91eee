#include "sdpa_rule.h"
#include <limits.h>

namespace fvrule {

Shape Shape::of(const size_t q[4], const size_t k[4], const size_t v[4]) {
    Shape s{};
    s.sq = q[2];
    s.sk = k[2];
    // k == [b, h, sk, d] of q, and v == k
    const bool k_ok = k[0] == q[0] && k[1] == q[1] && k[3] == q[3];
    const bool v_ok = v[0] == k[0] && v[1] == k[1] && v[2] == k[2] && v[3] == k[3];
    s.has_dims = k_ok && v_ok;
    if (s.has_dims) s.dims = Dims{q[0], q[1], q[2], k[2], q[3]};
    return s;
}

Backend parse_backend(const std::string& v) {
    if (v == "cublas") return Backend::Cublas;
    if (v == "flash") return Backend::Flash;
    if (v == "host") return Backend::Host;
    if (v == "sparse") return Backend::Sparse;
    return Backend::Dense;
}

static std::string trim(const std::string& v) {
    size_t a = 0, b = v.size();
    while (a < b && (v[a] == ' ' || v[a] == '\t' || v[a] == '\n' || v[a] == '\r')) a++;
    while (b > a && (v[b - 1] == ' ' || v[b - 1] == '\t' || v[b - 1] == '\n' || v[b - 1] == '\r')) b--;
    return v.substr(a, b - a);
}

AutoMode parse_auto_mode(const std::string& v) { return trim(v) == "timed" ? AutoMode::Timed : AutoMode::Rule; }

bool parse_kernel_override(const std::string& v, FlashKernel* out) {
    static const struct { const char* n; FlashKernel k; } tab[] = {
        {"v1", FlashKernel::V1}, {"v2", FlashKernel::V2}, {"v3", FlashKernel::V3},
        {"v3s", FlashKernel::V3s}, {"cudnn", FlashKernel::Cudnn}};
    for (const auto& e : tab)
        if (v == e.n) {
            *out = e.k;
            return true;
        }
    return false;
}

const char* flash_kernel_name(FlashKernel k) {
    switch (k) {
        case FlashKernel::V1: return "v1";
        case FlashKernel::V2: return "v2";
        case FlashKernel::V3: return "v3";
        case FlashKernel::V3s: return "v3s";
        case FlashKernel::Cudnn: return "cudnn";
        case FlashKernel::Dc: return "dc";
        case FlashKernel::B200: return "b200";
    }
    return "?";
}

static size_t div_ceil(size_t a, size_t b) { return a / b + (a % b ? 1 : 0); }
static size_t sat_mul(size_t a, size_t b) {
    if (a != 0 && b > SIZE_MAX / a) return SIZE_MAX;
    return a * b;
}

bool flash_v2_fills(size_t sq, size_t bh, size_t sms) {
    return sat_mul(div_ceil(sq, 2 * MMA_TILE), bh) >= 16 * (sms < 1 ? 1 : sms);
}

bool cudnn_default(int sm_major) { return sm_major == 12; }

// The one measured row (sm_12x, d = 128): cuDNN for self-attention-sized keys 24 576..=128 000.
DensePick pick(int sm_major, size_t sq, size_t sk, size_t d) {
    if (sm_major == 12 && d == 128 && sq >= 24576 && sk >= 24576 && sk <= 128000) return DensePick::Cudnn;
    return DensePick::V2;
}

std::vector<Step> dense_route(const Shape& shape, bool masked, bool out_bf16, const Probe& p) {
    std::vector<Step> route;
    if (!masked) {
        if (p.backend == Backend::Host || p.backend == Backend::Sparse)
            return {Step{StepKind::Retired, 0, p.backend}};
        if (p.backend == Backend::Flash) route.push_back(Step{StepKind::FlashF32, 0, Backend::Dense});
        if (p.backend != Backend::Cublas && p.mma_default) {
            if (p.has_sage && shape.sq >= p.sage_min_seq && shape.sk >= p.sage_min_seq)
                route.push_back(Step{StepKind::Sage, out_bf16 ? 1 : 0, Backend::Dense});
            route.push_back(Step{StepKind::Mma, out_bf16 ? 1 : 0, Backend::Dense});
        }
        route.push_back(Step{StepKind::Cublas, 0, Backend::Dense});
    }
    route.push_back(Step{StepKind::Composed, 0, Backend::Dense});
    return route;
}

FlashKernel flash_kernel_for(size_t sq, size_t bh, size_t sms, const Probe& p) {
    const std::string& c = p.kernel_choice;
    if (c == "v1") return FlashKernel::V1;
    if (c == "v2") return FlashKernel::V2;
    if (c == "v3") return FlashKernel::V3;
    if (c == "v3s") return FlashKernel::V3s;
    if (c == "cudnn") return FlashKernel::Cudnn;
    if (c == "dc") return FlashKernel::Dc;
    if (c == "b200") return FlashKernel::B200;
    if (p.b200_loaded) return FlashKernel::B200;
    if (p.dc_loaded) return FlashKernel::Dc;
    if (flash_v2_fills(sq, bh, sms)) return FlashKernel::V2;
    return FlashKernel::V1;
}

MmaKernel mma_kernel(const Shape& shape, bool out_bf16, const Probe& p) {
    if (!shape.has_dims || !p.has_sm) return MmaKernel{MmaKind::Fixed, flash_kernel_for(SIZE_MAX, 1, 1, p), 0};
    const Dims& d = shape.dims;
    const FlashKernel k = flash_kernel_for(d.sq, d.b * d.h, p.sms, p);
    if (k == FlashKernel::V2 && out_bf16 && cudnn_default(p.sm_major) && p.kernel_choice == "auto") {
        if (p.auto_mode == AutoMode::Timed) return MmaKernel{MmaKind::Timed, FlashKernel::V2, 0};
        FlashKernel kernel = FlashKernel::V2;
        if (pick(p.sm_major, d.sq, d.sk, d.d) == DensePick::Cudnn && p.cudnn_has_plan) kernel = FlashKernel::Cudnn;
        return MmaKernel{MmaKind::Rule, kernel, p.sm_major};
    }
    return MmaKernel{MmaKind::Fixed, k, 0};
}

bool fp8_first(const Probe& p) { return p.fp8_dense; }
bool block_causal_first(const Probe& p) { return p.causal_flash && p.sp_world == 1 && p.mma_default; }
bool vdn_window_first(const Probe& p) { return p.sp_world == 1 && p.mma_default; }
bool kv_window_flash(int flash, const Probe& p) { return flash < 0 ? p.causal_flash : flash != 0; }

bool mma_sdpa_supported(size_t b, size_t h, size_t sq, size_t sk, size_t d, int sm_major) {
    const size_t bh = b * h;
    return sm_major >= 8 && (d == 64 || d == 128) && sq > 0 && sk > 0 && bh >= 1 && bh <= 65535 &&
           sq <= (size_t)INT_MAX && sk <= (size_t)INT_MAX;
}

}  // namespace fvrule
