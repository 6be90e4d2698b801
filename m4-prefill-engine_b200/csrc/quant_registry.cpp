// QuantRegistry implementation: the eight built-in descriptors of the reference
// (src/router/quant_registry.mm:60-172, same names, sizes and kernel-name strings) and kernel-name
// resolution for the CUDA launchers.  Two planar MLX layouts are registered as well, so that the layer coordinator
// can bind them: the group-32 planes of the reference's layer benchmarks under the kernel names of its unified
// pipelines (unified_multi_scale_kernels.metal: gemm_mma_mlx_4bit_64x64, qkv_head_gemm_mma_mlx_4bit_64x64), and
// the group-64 extension layout.  Their struct_size is the bytes one block occupies over all three planes.
#include "../../include/quant_registry.h"

#include <cstring>
#include <iostream>

namespace b200_llm {

QuantRegistry& QuantRegistry::instance() {
    static QuantRegistry inst;
    return inst;
}

QuantRegistry::QuantRegistry() { register_builtin_codecs(); }

void QuantRegistry::register_codec(const QuantCodecDescriptor& desc) {
    auto old = registry_.find(desc.format);
    if (old != registry_.end()) name_to_format_.erase(old->second.name);
    registry_[desc.format] = desc;
    name_to_format_[desc.name] = desc.format;
}

const QuantCodecDescriptor* QuantRegistry::get(QuantFormat format) const {
    auto it = registry_.find(format);
    return it == registry_.end() ? nullptr : &it->second;
}

const QuantCodecDescriptor* QuantRegistry::get_by_name(const std::string& name) const {
    auto it = name_to_format_.find(name);
    return it == name_to_format_.end() ? nullptr : get(it->second);
}

std::vector<QuantFormat> QuantRegistry::available_formats() const {
    std::vector<QuantFormat> out;
    out.reserve(registry_.size());
    for (const auto& kv : registry_) out.push_back(kv.first);
    return out;
}

bool QuantRegistry::has_format(QuantFormat format) const { return registry_.count(format) != 0; }

size_t QuantRegistry::compute_weight_bytes(QuantFormat format, size_t num_elements) const {
    const QuantCodecDescriptor* d = get(format);
    if (!d) {
        std::cerr << "[QuantRegistry] Unknown format: " << (int)format << std::endl;
        return 0;
    }
    return (num_elements + d->block_size - 1) / d->block_size * d->struct_size;
}

KernelBinding QuantRegistry::resolve_kernel(const std::string& kernel_name) const {
    KernelBinding b;
    for (const auto& kv : registry_) {
        const QuantCodecDescriptor& d = kv.second;
        if (kernel_name == d.gemm_kernel_name) { b.valid = true; b.format = d.format; b.layout = LAYOUT_STANDARD; }
        else if (kernel_name == d.head_gemm_kernel_name) { b.valid = true; b.format = d.format; b.layout = LAYOUT_DIRECT_HEAD; }
        else continue;
        // Q8_0 is a KV-cache format: the reference registers kernel names for it but ships no such
        // kernel (src/router/quant_registry.mm:153-154); the same holds here.
        b.implemented = d.format != QUANT_Q8_0 && d.format != QUANT_CUSTOM;
        return b;
    }
    return b;
}

void QuantRegistry::register_builtin_codecs() {
    struct Row { QuantFormat f; const char* name; const char* desc; uint32_t bs; size_t ss; double bpw; const char* stem; bool tc; };
    const Row rows[] = {
        {QUANT_Q4_0, "Q4_0", "32-element symmetric 4-bit blocks, fp16 scale", 32, sizeof(block_q4_0), 4.50, "q4_0", true},
        {QUANT_MLX_4BIT, "MLX_4BIT", "32-element affine 4-bit blocks, fp16 scale and bias", 32, sizeof(block_mlx_4bit), 5.00, "mlx_4bit", true},
        {QUANT_Q4_K, "Q4_K", "256-element super-blocks of 8x32, 6-bit sub-scales and minimums", 256, sizeof(block_q4_K), 4.50, "q4_k", true},
        {QUANT_TERNARY_1_58, "TERNARY_1_58", "32-element ternary {-1,0,+1} blocks, fp16 scale", 32, sizeof(block_ternary_1_58), 3.00, "ternary_1_58", true},
        {QUANT_VAR_RATE_AFFINE, "VAR_RATE_AFFINE", "256-element mixed 3/4/5-bit affine super-blocks", 256, sizeof(block_var_rate_affine), 5.00, "var_rate_affine", true},
        {QUANT_EXL3, "EXL3", "256-element codebook super-blocks with residual correction", 256, sizeof(block_exl3), 4.50, "exl3", true},
        {QUANT_Q8_0, "Q8_0", "32-element symmetric 8-bit blocks (KV cache)", 32, sizeof(block_q8_0), 8.50, "q8_0", false},
        {QUANT_PRISM_Q2_0, "PRISM_Q2_0", "128-element 2-bit ternary blocks, fp16 scale", 128, sizeof(block_prism_q2_0), 2.125, "prism_q2_0", true},
    };
    for (const Row& r : rows) {
        QuantCodecDescriptor d;
        d.format = r.f; d.name = r.name; d.description = r.desc; d.block_size = r.bs; d.struct_size = r.ss;
        d.bits_per_weight = r.bpw;
        d.gemm_kernel_name = std::string("quant_router_gemm_") + r.stem + "_64x64";
        d.head_gemm_kernel_name = std::string("quant_router_head_gemm_") + r.stem + "_64x64";
        d.quantize_fn = nullptr; d.dequantize_fn = nullptr;
        d.tensor_core_codec = r.tc;
        register_codec(d);
    }
    QuantCodecDescriptor p;
    p.format = QUANT_MLX_4BIT_PLANAR; p.name = "MLX_4BIT_PLANAR";
    p.description = "32-element affine 4-bit blocks in three planes: nibbles, fp16 scales, fp16 biases";
    p.block_size = 32; p.struct_size = 20; p.bits_per_weight = 5.0;
    p.gemm_kernel_name = "gemm_mma_mlx_4bit_64x64"; p.head_gemm_kernel_name = "qkv_head_gemm_mma_mlx_4bit_64x64";
    p.quantize_fn = nullptr; p.dequantize_fn = nullptr; p.tensor_core_codec = true;
    register_codec(p);
    p.format = QUANT_MLX_4BIT_G64; p.name = "MLX_4BIT_G64";
    p.description = "64-element affine 4-bit groups, sequential nibbles, in three planes";
    p.block_size = 64; p.struct_size = 36; p.bits_per_weight = 4.5;
    p.gemm_kernel_name = "quant_router_gemm_mlx_4bit_g64_64x64"; p.head_gemm_kernel_name = "quant_router_head_gemm_mlx_4bit_g64_64x64";
    register_codec(p);
}

}  // namespace b200_llm

using b200_llm::QuantRegistry;

static void copy_str(const std::string& s, char* out, size_t cap) {
    if (!out || cap == 0) return;
    size_t n = s.size() < cap - 1 ? s.size() : cap - 1;
    memcpy(out, s.data(), n);
    out[n] = 0;
}

extern "C" {

int b200_registry_count(void) { return (int)QuantRegistry::instance().available_formats().size(); }

int b200_registry_format_at(int index) {
    auto f = QuantRegistry::instance().available_formats();
    return (index < 0 || index >= (int)f.size()) ? -1 : (int)f[index];
}

int b200_registry_describe(int format, char* name_out, size_t name_cap, uint32_t* block_size, size_t* struct_size,
                           double* bits_per_weight, char* gemm_kernel_out, size_t gemm_cap, char* head_kernel_out, size_t head_cap) {
    const auto* d = QuantRegistry::instance().get((QuantFormat)format);
    if (!d) return 0;
    copy_str(d->name, name_out, name_cap);
    if (block_size) *block_size = d->block_size;
    if (struct_size) *struct_size = d->struct_size;
    if (bits_per_weight) *bits_per_weight = d->bits_per_weight;
    copy_str(d->gemm_kernel_name, gemm_kernel_out, gemm_cap);
    copy_str(d->head_gemm_kernel_name, head_kernel_out, head_cap);
    return 1;
}

size_t b200_registry_weight_bytes(int format, size_t num_elements) {
    return QuantRegistry::instance().compute_weight_bytes((QuantFormat)format, num_elements);
}

int b200_registry_format_by_name(const char* name) {
    const auto* d = name ? QuantRegistry::instance().get_by_name(name) : nullptr;
    return d ? (int)d->format : -1;
}

int b200_registry_resolve_kernel(const char* kernel_name, int* format, int* layout, int* implemented) {
    if (!kernel_name) return 0;
    b200_llm::KernelBinding b = QuantRegistry::instance().resolve_kernel(kernel_name);
    if (!b.valid) return 0;
    if (format) *format = (int)b.format;
    if (layout) *layout = (int)b.layout;
    if (implemented) *implemented = b.implemented ? 1 : 0;
    return 1;
}

int b200_registry_register(int format, const char* name, uint32_t block_size, size_t struct_size, double bits_per_weight,
                           const char* gemm_kernel, const char* head_kernel) {
    b200_llm::QuantCodecDescriptor d;
    d.format = (QuantFormat)format; d.name = name ? name : ""; d.description = "registered at run time";
    d.block_size = block_size; d.struct_size = struct_size; d.bits_per_weight = bits_per_weight;
    d.gemm_kernel_name = gemm_kernel ? gemm_kernel : ""; d.head_gemm_kernel_name = head_kernel ? head_kernel : "";
    QuantRegistry::instance().register_codec(d);
    return 0;
}

}  // extern "C"
