// The kernel chooser of the dense-attention entry, as a pure function of a probe.
//
// Mirrors crates/fastvideo-cudarc/src/rt/sdpa_rule.rs (enums :50-67, :197-205, :259-280, :395-411,
// :456-466; Probe :321-350; Shape/Dims :352-393; dense_route :416-439; flash_kernel_for :476-490;
// mma_kernel :495-515; pick/RULES :69-133; the route predicates :517-538) with one added kernel,
// FlashKernel::B200: this library's sm_100a kernel.  `auto` picks it on a compute-capability
// 10.x device where the library is loaded, ahead of the reference's own attn_dc kernel; the seam
// value "b200" (FASTVIDEO_FLASH_KERNEL / [kernels] dense_attention) fixes it.  Every other choice
// is unchanged, so a probe without the library loaded gives the reference's answers.
#pragma once
#include <stddef.h>
#include <stdint.h>
#include <string>
#include <vector>

namespace fvrule {

enum class Backend : int { Dense = 0, Cublas = 1, Flash = 2, Host = 3, Sparse = 4 };
enum class FlashKernel : int { V1 = 0, V2 = 1, V3 = 2, V3s = 3, Cudnn = 4, Dc = 5, B200 = 6 };
enum class AutoMode : int { Rule = 0, Timed = 1 };
enum class DensePick : int { Cudnn = 0, V2 = 1 };

// One step of a dense route.  Sage / Mma carry the output type.
enum class StepKind : int { Retired = 0, FlashF32 = 1, Sage = 2, Mma = 3, Cublas = 4, Composed = 5 };
struct Step {
    StepKind kind;
    int out_bf16;      // Sage, Mma
    Backend retired;   // Retired
    bool operator==(const Step& o) const { return kind == o.kind && out_bf16 == o.out_bf16 && retired == o.retired; }
};

enum class MmaKind : int { Fixed = 0, Rule = 1, Timed = 2 };
struct MmaKernel {
    MmaKind kind;
    FlashKernel kernel;  // Fixed, Rule
    int sm_major;        // Rule
};

// What the chooser reads (the reference's Probe trait as plain data, plus b200_loaded).
struct Probe {
    Backend backend = Backend::Dense;
    size_t sp_world = 1;
    bool mma_default = true;
    bool has_sage = false;
    size_t sage_min_seq = 0;
    bool fp8_dense = false;
    bool causal_flash = true;
    std::string kernel_choice = "auto";  // lower-cased, not trimmed
    bool has_sm = true;
    int sm_major = 10;
    size_t sms = 148;
    bool dc_loaded = false;
    bool b200_loaded = false;
    AutoMode auto_mode = AutoMode::Rule;
    bool cudnn_has_plan = false;  // answer for every shape asked
};

struct Dims {
    size_t b, h, sq, sk, d;
};
struct Shape {
    size_t sq, sk;
    bool has_dims;
    Dims dims;
    // From the operands' shapes (each rank 4).
    static Shape of(const size_t q[4], const size_t k[4], const size_t v[4]);
};

Backend parse_backend(const std::string& v);
AutoMode parse_auto_mode(const std::string& v);
// h3_vae override parse: returns false for "auto" and anything else that is not a fixed kernel.
bool parse_kernel_override(const std::string& v, FlashKernel* out);
const char* flash_kernel_name(FlashKernel k);

constexpr size_t MMA_TILE = 64;
bool flash_v2_fills(size_t sq, size_t bh, size_t sms);
bool cudnn_default(int sm_major);
DensePick pick(int sm_major, size_t sq, size_t sk, size_t d);

std::vector<Step> dense_route(const Shape& shape, bool masked, bool out_bf16, const Probe& p);
FlashKernel flash_kernel_for(size_t sq, size_t bh, size_t sms, const Probe& p);
MmaKernel mma_kernel(const Shape& shape, bool out_bf16, const Probe& p);
bool fp8_first(const Probe& p);
bool block_causal_first(const Probe& p);
bool vdn_window_first(const Probe& p);
bool kv_window_flash(int flash /* -1 = unset, 0, 1 */, const Probe& p);

// mma_sdpa_supported, crates/fastvideo-cudarc/src/rt/attn.rs:107-128
bool mma_sdpa_supported(size_t b, size_t h, size_t sq, size_t sk, size_t d, int sm_major);

}  // namespace fvrule
