// Quantization format descriptors for the B200 prefill path.
//
// Binary-compatible with the reference's `quant_router.h:14-136` (format ids, layout
// modes, packed block structs, per-format metadata and byte sizing).  The structs are
// never dereferenced on the device through these types -- the CUDA codecs address raw
// bytes -- but hosts, tests and the CPU oracle use them to build and size buffers.
//
// Two descriptor extensions that the reference does not have are declared at the end
// (MLX group-64 sequential layout and ternary with one scale per row); they use format
// ids >= 100 so ids 0..7 keep their reference meaning.
#pragma once
#include <cstddef>
#include <cstdint>

#if defined(__CUDACC__)
#include <cuda_fp16.h>
typedef __half qr_half;
#else
typedef _Float16 qr_half;
#endif

// ---- format ids (reference quant_router.h:14-23) ---------------------------------
enum QuantFormat : int {
    QUANT_Q4_0            = 0,   // 18 B / 32:  half d; u8 qs[16]
    QUANT_MLX_4BIT        = 1,   // 20 B / 32:  half d; half bias; u8 qs[16]
    QUANT_Q4_K            = 2,   // 144 B / 256
    QUANT_TERNARY_1_58    = 3,   // 12 B / 32:  half d; half pad; u32 qs[2]
    QUANT_VAR_RATE_AFFINE = 4,   // 160 B / 256
    QUANT_EXL3            = 5,   // 144 B / 256
    QUANT_Q8_0            = 6,   // 34 B / 32 (KV cache only)
    QUANT_PRISM_Q2_0      = 7,   // 34 B / 128
    // extensions (no counterpart in the reference)
    QUANT_MLX_4BIT_G64    = 100, // planar: u32 qs[N][K/8] | half scales[N][K/64] | half biases[N][K/64]
    QUANT_TERNARY_ROW     = 101, // planar: u32 qs[N][K/16] | half row_scale[N]
    QUANT_MLX_4BIT_PLANAR = 102, // planar, group 32 (unified_multi_scale_kernels.metal:17-31, packer bench_all_scales.mm:62-95):
                                 // u8 qs[N*K/32][16] | half scales[N*K/32] | half biases[N*K/32], each plane 16-byte aligned;
                                 // byte j of a block: low nibble = element j, high nibble = element j + 16
    QUANT_CUSTOM          = 99
};

// ---- output layouts (reference quant_router.h:25-28) ------------------------------
enum LayoutMode : int {
    LAYOUT_STANDARD    = 0,  // Y[m][n]
    LAYOUT_DIRECT_HEAD = 1   // Y[h][m][d] with n = h*D + d
};

#pragma pack(push, 1)
struct block_q4_0            { qr_half d; uint8_t qs[16]; };
struct block_mlx_4bit        { qr_half d; qr_half bias; uint8_t qs[16]; };
struct block_q4_K            { qr_half d; qr_half dmin; uint8_t scales[12]; uint8_t qs[128]; };
struct block_ternary_1_58    { qr_half d; qr_half _pad; uint32_t qs[2]; };
struct block_var_rate_affine { qr_half d; qr_half bias; uint8_t scales[8]; uint8_t biases[8];
                               uint8_t modes[8]; uint8_t _pad[4]; uint8_t qs[128]; };
struct block_exl3            { qr_half d; qr_half bias; uint8_t scales[8]; uint8_t residuals[8];
                               int8_t codebook[16]; uint8_t _pad[12]; uint8_t qs[96]; };
struct block_q8_0            { qr_half d; int8_t qs[32]; };
struct block_prism_q2_0      { qr_half d; uint8_t qs[32]; };
#pragma pack(pop)

static_assert(sizeof(block_q4_0) == 18, "Q4_0 block is 18 bytes");
static_assert(sizeof(block_mlx_4bit) == 20, "MLX block is 20 bytes");
static_assert(sizeof(block_q4_K) == 144, "Q4_K super-block is 144 bytes");
static_assert(sizeof(block_ternary_1_58) == 12, "ternary block is 12 bytes");
static_assert(sizeof(block_var_rate_affine) == 160, "var-rate super-block is 160 bytes");
static_assert(sizeof(block_exl3) == 144, "EXL3 super-block is 144 bytes");
static_assert(sizeof(block_q8_0) == 34, "Q8_0 block is 34 bytes");
static_assert(sizeof(block_prism_q2_0) == 34, "Prism Q2_0 block is 34 bytes");

// ---- metadata (reference quant_router.h:101-136) -----------------------------------
struct QuantFormatInfo {
    QuantFormat format;
    const char* name;
    const char* description;
    uint32_t block_size;     // elements per block / super-block
    uint32_t block_bytes;    // bytes per block struct
    double bits_per_weight;
};

inline QuantFormatInfo get_quant_info(QuantFormat fmt) {
    switch (fmt) {
        case QUANT_Q4_0:            return {fmt, "Q4_0", "32-elem symmetric 4-bit block, fp16 scale", 32, 18, 4.50};
        case QUANT_MLX_4BIT:        return {fmt, "MLX_4BIT", "32-elem affine 4-bit block, fp16 scale + bias", 32, 20, 5.00};
        case QUANT_Q4_K:            return {fmt, "Q4_K", "256-elem super-block, 6-bit sub-scales and mins", 256, 144, 4.50};
        case QUANT_TERNARY_1_58:    return {fmt, "TERNARY_1_58", "32-elem ternary block, fp16 scale", 32, 12, 3.00};
        case QUANT_VAR_RATE_AFFINE: return {fmt, "VAR_RATE_AFFINE", "256-elem mixed 3/4/5-bit affine super-block", 256, 160, 5.00};
        case QUANT_EXL3:            return {fmt, "EXL3", "256-elem codebook super-block with residual correction", 256, 144, 4.50};
        case QUANT_Q8_0:            return {fmt, "Q8_0", "32-elem symmetric 8-bit block, fp16 scale", 32, 34, 8.50};
        case QUANT_PRISM_Q2_0:      return {fmt, "PRISM_Q2_0", "128-elem 2-bit ternary block, fp16 scale", 128, 34, 2.125};
        default: break;
    }
    return {QUANT_Q4_0, "UNKNOWN", "Unknown format", 32, 0, 0.0};
}

inline size_t compute_quant_weight_bytes(QuantFormat fmt, size_t total_elements) {
    QuantFormatInfo info = get_quant_info(fmt);
    size_t num_blocks = (total_elements + info.block_size - 1) / info.block_size;
    return num_blocks * info.block_bytes;
}

// Byte size of a [N][K] weight matrix; covers the two planar extension layouts too.
inline size_t compute_quant_matrix_bytes(QuantFormat fmt, size_t K, size_t N) {
    if (fmt == QUANT_MLX_4BIT_G64) return N * (K / 8) * 4 + 2 * N * (K / 64) * 2;
    if (fmt == QUANT_TERNARY_ROW)  return N * (K / 16) * 4 + N * 2;
    if (fmt == QUANT_MLX_4BIT_PLANAR) {          // the reference's mlx_4bit_buffer_size(): planes padded to 16 bytes
        const size_t blocks = N * (K / 32), scales_off = (blocks * 16 + 15) & ~(size_t)15;
        return ((scales_off + blocks * 2 + 15) & ~(size_t)15) + blocks * 2;
    }
    QuantFormatInfo info = get_quant_info(fmt);
    if (info.block_bytes == 0) return 0;
    return N * (K / info.block_size) * (size_t)info.block_bytes;
}
