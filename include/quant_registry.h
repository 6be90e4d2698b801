// Format-descriptor -> kernel dispatch registry.
//
// Same surface as the reference's src/router/quant_registry.h:14-65: a process-wide singleton
// mapping QuantFormat to a QuantCodecDescriptor {name, block_size, struct_size, bits_per_weight,
// gemm_kernel_name, head_gemm_kernel_name, quantize_fn, dequantize_fn}, lookup by enum or name,
// byte sizing, dynamic registration through REGISTER_QUANT_CODEC.  The kernel-name strings of the
// reference are kept as lookup keys; resolve_kernel() turns one into the (format, layout) pair the
// CUDA launcher takes, which is how the layer coordinator binds its projections
// (models/transformer_layer.mm:38-47 does the same through Metal pipeline names).
#pragma once
#ifdef __cplusplus
#include <cstddef>
#include <cstdint>
#include <functional>
#include <map>
#include <string>
#include <vector>

#include "quant_router.h"

namespace b200_llm {

struct QuantCodecDescriptor {
    QuantFormat format;
    std::string name;
    std::string description;
    uint32_t block_size;
    size_t struct_size;
    double bits_per_weight;
    std::string gemm_kernel_name;
    std::string head_gemm_kernel_name;
    std::function<void(const void* src, void* dst, size_t count)> quantize_fn;
    std::function<void(const void* src, float* dst, size_t count)> dequantize_fn;
    // true when the format has a TMA + tcgen05 codec (otherwise the CUDA-core kernel serves it)
    bool tensor_core_codec = false;
};

struct KernelBinding {      // what a kernel name resolves to
    bool valid = false;
    QuantFormat format = QUANT_Q4_0;
    LayoutMode layout = LAYOUT_STANDARD;
    bool implemented = false;   // a launcher exists for this (format, layout)
};

class QuantRegistry {
public:
    static QuantRegistry& instance();
    void register_codec(const QuantCodecDescriptor& desc);
    const QuantCodecDescriptor* get(QuantFormat format) const;
    const QuantCodecDescriptor* get_by_name(const std::string& name) const;
    std::vector<QuantFormat> available_formats() const;
    size_t compute_weight_bytes(QuantFormat format, size_t num_elements) const;
    bool has_format(QuantFormat format) const;
    KernelBinding resolve_kernel(const std::string& kernel_name) const;

private:
    QuantRegistry();
    void register_builtin_codecs();
    std::map<QuantFormat, QuantCodecDescriptor> registry_;
    std::map<std::string, QuantFormat> name_to_format_;
};

struct CodecRegistrationHelper {
    explicit CodecRegistrationHelper(const QuantCodecDescriptor& desc) { QuantRegistry::instance().register_codec(desc); }
};

#define B200_CONCAT_INNER(a, b) a##b
#define B200_CONCAT(a, b) B200_CONCAT_INNER(a, b)
#define REGISTER_QUANT_CODEC(...) \
    static ::b200_llm::CodecRegistrationHelper B200_CONCAT(_codec_reg_, __LINE__)(__VA_ARGS__);

}  // namespace b200_llm

namespace metal_llm = b200_llm;   // the reference's namespace name, for code written against it

// C view of the registry for bindings and tests.

#else   /* C callers see the C entry points below only */
#include <stddef.h>
#include <stdint.h>
#endif

#ifdef __cplusplus
extern "C" {
#endif
int b200_registry_count(void);
int b200_registry_format_at(int index);
int b200_registry_describe(int format, char* name_out, size_t name_cap, uint32_t* block_size, size_t* struct_size,
                           double* bits_per_weight, char* gemm_kernel_out, size_t gemm_cap, char* head_kernel_out,
                           size_t head_cap);
size_t b200_registry_weight_bytes(int format, size_t num_elements);
int b200_registry_format_by_name(const char* name);
/* returns 1 and fills format/layout/implemented when the kernel name is known, else 0 */
int b200_registry_resolve_kernel(const char* kernel_name, int* format, int* layout, int* implemented);
/* registers (or replaces) a descriptor at run time; returns 0 */
int b200_registry_register(int format, const char* name, uint32_t block_size, size_t struct_size, double bits_per_weight,
                           const char* gemm_kernel, const char* head_kernel);
#ifdef __cplusplus
}
#endif
