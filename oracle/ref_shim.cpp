// CHECKER ONLY -- C entry points over the reference's own CPU verifier sources.
//
// This file contains no reference code.  oracle/build.py pipes the reference sources, where
// they lie in the reference checkout, through two mechanical text substitutions (the
// Grand-Central-Dispatch `dispatch_apply(n, queue, ^(size_t i){ ... });` loops become OpenMP
// `for` loops; `__fp16` becomes `_Float16`) into a temporary directory, and this file includes
// the results by the names below.  Loop bodies are untouched, so the arithmetic is the
// reference's.  The only output is oracle/_ref/libm4ref.so (git-ignored).
//
//   REF_GOLD_H    <- tests/e2e/cpu_gold_reference.h            (7 GEMM golds, attention, swiglu)
//   REF_GEN_INC   <- tests/e2e/test_common.h, generator section (seeded LCG generators)
//   REF_BRICK3    <- brick3_swiglu_bench.mm, generator + fused SwiGLU gold section
//   REF_BRICK4    <- brick4_attn_bench.mm, Q8_0 quantiser + attention gold section
//   REF_LAYER     <- bench_8b_engine.mm, generator + layer gold section
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <string>
#include <vector>

#include REF_GOLD_H   // pulls in the reference's quant_router.h (block structs)

namespace refgen {
#include REF_GEN_INC
}
namespace brick3 {
#include REF_BRICK3
}
namespace brick4 {
#include REF_BRICK4
}
namespace layer8b {
#include REF_LAYER
}

#ifdef _OPENMP
#include <omp.h>
#endif

extern "C" {

// OpenMP team size used by the rewritten dispatch_apply loops: set it (n > 0) and report what a parallel region gets.
int ref_set_threads(int n) {
    int got = 1;
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#pragma omp parallel
    {
#pragma omp single
        got = omp_get_num_threads();
    }
#endif
    return got;
}

int ref_gemm(int format, const _Float16* A, const void* W, _Float16* C, uint32_t M, uint32_t N, uint32_t K,
             int direct_head, uint32_t H, uint32_t D) {
    bool dh = direct_head != 0;
    switch (format) {
        case 0: cpu_gold_reference_q4_0(A, (const block_q4_0*)W, C, M, N, K, dh, H, D); return 0;
        case 1: cpu_gold_reference_mlx_4bit(A, (const block_mlx_4bit*)W, C, M, N, K, dh, H, D); return 0;
        case 2: cpu_gold_reference_q4_k(A, (const block_q4_K*)W, C, M, N, K, dh, H, D); return 0;
        case 3: cpu_gold_reference_ternary_1_58(A, (const block_ternary_1_58*)W, C, M, N, K, dh, H, D); return 0;
        case 4: cpu_gold_reference_var_rate_affine(A, (const block_var_rate_affine*)W, C, M, N, K, dh, H, D); return 0;
        case 5: cpu_gold_reference_exl3(A, (const block_exl3*)W, C, M, N, K, dh, H, D); return 0;
        case 7: cpu_gold_reference_prism_q2_0(A, (const block_prism_q2_0*)W, C, M, N, K, dh, H, D); return 0;
        default: return -3;
    }
}

void ref_attention(const _Float16* Q, const _Float16* K, const _Float16* V, _Float16* O, uint32_t H, uint32_t M,
                   uint32_t D, float scale) {
    cpu_gold_reference_attention(Q, K, V, O, H, M, D, scale);
}

void ref_swiglu_elementwise(const _Float16* g, const _Float16* u, _Float16* o, uint32_t count) {
    cpu_gold_reference_swiglu(g, u, o, count);
}

uint32_t ref_gen_activations(uint32_t state, _Float16* data, size_t count) {
    refgen::prng_seed(state);
    refgen::generate_activations(data, count);
    return refgen::g_prng_state;
}

uint32_t ref_gen_weights(uint32_t state, int format, void* out, size_t num_blocks) {
    refgen::prng_seed(state);
    switch (format) {
        case 0: refgen::generate_q4_0_weights((block_q4_0*)out, num_blocks); break;
        case 1: refgen::generate_mlx_4bit_weights((block_mlx_4bit*)out, num_blocks); break;
        case 2: refgen::generate_q4_k_weights((block_q4_K*)out, num_blocks); break;
        case 3: refgen::generate_ternary_1_58_weights((block_ternary_1_58*)out, num_blocks); break;
        case 4: refgen::generate_var_rate_affine_weights((block_var_rate_affine*)out, num_blocks); break;
        case 5: refgen::generate_exl3_weights((block_exl3*)out, num_blocks); break;
        case 7: refgen::generate_prism_q2_0_weights((block_prism_q2_0*)out, num_blocks); break;
        default: break;
    }
    return refgen::g_prng_state;
}

void ref_brick3_swiglu(uint32_t seed, _Float16* A, void* Wg, void* Wu, _Float16* Out, uint32_t M, uint32_t F, uint32_t K,
                       int generate) {
    if (generate) {
        brick3::prng_state = seed;
        brick3::generate_activations(A, (size_t)M * K);
        brick3::generate_q4_0_weights((block_q4_0*)Wg, (size_t)F * (K / 32));
        brick3::generate_q4_0_weights((block_q4_0*)Wu, (size_t)F * (K / 32));
    }
    brick3::cpu_gold_reference_swiglu(A, (const block_q4_0*)Wg, (const block_q4_0*)Wu, Out, M, F, K);
}

void ref_quantize_q8_0(const _Float16* src, void* dst, size_t n) { brick4::quantize_to_q8_0(src, (block_q8_0*)dst, n); }
void ref_dequantize_q8_0(const void* src, _Float16* dst, size_t n) { brick4::dequantize_q8_0((const block_q8_0*)src, dst, n); }
void ref_brick4_attention(const _Float16* Q, const _Float16* K, const _Float16* V, _Float16* O, uint32_t H, uint32_t M,
                          uint32_t D, float scale) {
    brick4::cpu_gold_reference_causal_attention(Q, K, V, O, H, M, D, scale);
}

uint32_t ref_layer_gen_q4_0(uint32_t state, void* out, size_t num_blocks, float scale_factor) {
    layer8b::prng_state = state;
    layer8b::generate_q4_0_weights((block_q4_0*)out, num_blocks, scale_factor);
    return layer8b::prng_state;
}

void ref_layer(const _Float16* X, const void* Wq, const void* Wk, const void* Wv, const void* Wo, const void* Wg,
               const void* Wu, const void* Wd, _Float16* Y, uint32_t M, uint32_t K, uint32_t H, uint32_t D,
               uint32_t F, float attn_scale) {
    layer8b::cpu_reference_prefill_layer(X, (const block_q4_0*)Wq, (const block_q4_0*)Wk, (const block_q4_0*)Wv,
                                         (const block_q4_0*)Wo, (const block_q4_0*)Wg, (const block_q4_0*)Wu,
                                         (const block_q4_0*)Wd, Y, M, K, H, D, F, attn_scale, nullptr);
}

}  // extern "C"
