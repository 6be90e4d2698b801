// Host build of the device unpackers (csrc/codecs.cuh) for CPU-only tests: runs the per-row,
// per-256-chunk, per-64-sub-tile unpack exactly as a dequant thread of the GEMM kernel does and
// returns the fp16 bit patterns in natural [N][K] order.
#include <cstdint>
#include <cstring>
#include "../m4-prefill-engine_b200/csrc/codecs.cuh"

template <int FMT>
static void run(const uint8_t* W, uint16_t* out, uint32_t N, uint32_t K) {
    constexpr int RB = cdc::Codec<FMT>::ROW_BYTES;
    const size_t row_bytes = (size_t)(K / 256) * RB;
    for (uint32_t n = 0; n < N; n++)
        for (uint32_t kc = 0; kc < K / 256; kc++) {
            uint32_t r[RB / 4];
            std::memcpy(r, W + n * row_bytes + (size_t)kc * RB, RB);
            for (int s = 0; s < 4; s++) {
                uint32_t o[32];
                cdc::Codec<FMT>::dequant64(r, s, o);
                std::memcpy(out + (size_t)n * K + kc * 256 + s * 64, o, 128);
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
        default: return -3;
    }
}
