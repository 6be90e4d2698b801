// Host build of the device unpackers (csrc/codecs.cuh) for CPU-only tests: runs the per-row,
// per-256-chunk, per-64-sub-tile unpack exactly as a dequant thread of the GEMM kernel does and
// returns the fp16 bit patterns in natural [N][K] order.
#include <cstdint>
#include <cstring>
#include "../m4-prefill-engine_b200/csrc/codecs.cuh"

template <int FMT>
static void run(const uint8_t* W, uint16_t* out, uint32_t N, uint32_t K) {
    constexpr int RB = cdc::Codec<FMT>::ROW_BYTES;
    constexpr int CH = cdc::Codec<FMT>::CHUNK;                  // K elements per packed stage
    const size_t row_bytes = (size_t)(K / CH) * RB;
    const uint8_t* plane2 = W + (size_t)N * row_bytes;          // metadata planes of the planar layouts
    for (uint32_t n = 0; n < N; n++)
        for (uint32_t kc = 0; kc < K / CH; kc++) {
            uint32_t r[RB / 4];
            std::memcpy(r, W + n * row_bytes + (size_t)kc * RB, RB);
            constexpr int MW = cdc::Codec<FMT>::META_WORDS > 0 ? cdc::Codec<FMT>::META_WORDS : 4;
            uint32_t meta[MW] = {};
            if (cdc::Codec<FMT>::META_WORDS != 0) {             // MW scales then MW biases of this chunk (one per 256 / MW elements)
                const size_t groups = (size_t)(K / 256) * MW, at = ((size_t)n * groups + (size_t)kc * MW) * 2;
                std::memcpy(meta, plane2 + at, MW * 2);
                std::memcpy(meta + MW / 2, plane2 + (size_t)N * groups * 2 + at, MW * 2);
            }
            for (int s = 0; s < CH / 64; s++) {
                uint32_t o[32];
                cdc::Codec<FMT>::dequant64(r, s, o, meta);
                std::memcpy(out + (size_t)n * K + kc * CH + s * 64, o, 128);
            }
        }
}

extern "C" int codec_host_dequant(int fmt, const uint8_t* W, uint16_t* out, uint32_t N, uint32_t K) {
    switch (fmt) {
        case QUANT_Q4_0: run<QUANT_Q4_0>(W, out, N, K); return 0;
        case QUANT_MLX_4BIT: run<QUANT_MLX_4BIT>(W, out, N, K); return 0;
        case QUANT_Q4_K: run<QUANT_Q4_K>(W, out, N, K); return 0;
        case QUANT_TERNARY_1_58: run<QUANT_TERNARY_1_58>(W, out, N, K); return 0;
        case QUANT_VAR_RATE_AFFINE: run<QUANT_VAR_RATE_AFFINE>(W, out, N, K); return 0;
        case QUANT_EXL3: run<QUANT_EXL3>(W, out, N, K); return 0;
        case QUANT_PRISM_Q2_0: run<QUANT_PRISM_Q2_0>(W, out, N, K); return 0;
        case QUANT_MLX_4BIT_G64: run<QUANT_MLX_4BIT_G64>(W, out, N, K); return 0;
        case QUANT_MLX_4BIT_PLANAR: run<QUANT_MLX_4BIT_PLANAR>(W, out, N, K); return 0;
        case QUANT_TERNARY_ROW: run<QUANT_TERNARY_ROW>(W, out, N, K); return 0;   // integers code-1: the row scale is applied later
        default: return -3;
    }
}
