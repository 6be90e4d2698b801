// CPU ORACLE -- TEST INFRASTRUCTURE ONLY.
//
// A plain C++17/OpenMP restatement of the reference's double-precision CPU verifier for
// the prefill hot path.  It is the checker for the CUDA kernels and the timed CPU
// baseline; nothing in the product path may call it.
//
// Pinning: every function below is checked in tests/ against (a) the known-answer tests
// of the reference (tests/e2e/test_tier1_feature_coverage.mm), (b) the reference's own
// header compiled as oracle/_ref (bit-exact on seeded inputs) and (c) the committed
// fixtures in tests/golden/.  RMSNorm, RoPE and grouped-query attention have no CPU
// counterpart in the reference (they exist only as calls into a third-party array
// library there), so those three are "restated, parity unpinned".
//
// Each function cites the reference file:line it follows.  Accumulation order follows
// the reference so results agree bit-for-bit with its verifier, but the code is
// organised differently: a weight row is first expanded to (k index, double weight)
// pairs in the reference's visiting order, then dotted with each activation row.

#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <vector>
#ifdef _OPENMP
#include <omp.h>
#endif

#include "../include/quant_router.h"

typedef _Float16 f16;

namespace {

// ------------------------------------------------------------------------------------
// Row expansion: w[j], kidx[j] for j in the reference's accumulation order.
// ------------------------------------------------------------------------------------

// 3-bit stream: 8 values per 3 bytes, LSB first (tests/e2e/cpu_gold_reference.h:238-251).
inline void unpack3(const uint8_t* p, uint8_t q[8]) {
    uint32_t v = (uint32_t)p[0] | ((uint32_t)p[1] << 8) | ((uint32_t)p[2] << 16);
    for (int i = 0; i < 8; i++) q[i] = (v >> (3 * i)) & 7u;
}
// 5-bit stream: 8 values per 5 bytes, LSB first (tests/e2e/cpu_gold_reference.h:262-275).
inline void unpack5(const uint8_t* p, uint8_t q[8]) {
    uint64_t v = 0;
    for (int i = 0; i < 5; i++) v |= (uint64_t)p[i] << (8 * i);
    for (int i = 0; i < 8; i++) q[i] = (uint8_t)((v >> (5 * i)) & 31u);
}

// Q4_0: tests/e2e/cpu_gold_reference.h:33-43.  Visiting order per block: i, i+16 interleaved.
void expand_q4_0(const uint8_t* row, uint32_t K, double* w, uint32_t* kidx) {
    const block_q4_0* b = (const block_q4_0*)row;
    size_t j = 0;
    for (uint32_t blk = 0; blk < K / 32; blk++) {
        double d = (double)b[blk].d;
        for (int i = 0; i < 16; i++) {
            uint8_t byte = b[blk].qs[i];
            w[j] = (double)((int)(byte & 0x0F) - 8) * d; kidx[j++] = blk * 32 + i;
            w[j] = (double)((int)(byte >> 4) - 8) * d;   kidx[j++] = blk * 32 + i + 16;
        }
    }
}

// MLX 4-bit AoS: tests/e2e/cpu_gold_reference.h:73-86.
void expand_mlx(const uint8_t* row, uint32_t K, double* w, uint32_t* kidx) {
    const block_mlx_4bit* b = (const block_mlx_4bit*)row;
    size_t j = 0;
    for (uint32_t blk = 0; blk < K / 32; blk++) {
        double d = (double)b[blk].d, bias = (double)b[blk].bias;
        for (int i = 0; i < 16; i++) {
            uint8_t byte = b[blk].qs[i];
            w[j] = (double)(int)(byte & 0x0F) * d + bias; kidx[j++] = blk * 32 + i;
            w[j] = (double)(int)(byte >> 4) * d + bias;   kidx[j++] = blk * 32 + i + 16;
        }
    }
}

// Q4_K: tests/e2e/cpu_gold_reference.h:116-146 (the reference's own 12-byte scale packing).
void expand_q4_k(const uint8_t* row, uint32_t K, double* w, uint32_t* kidx) {
    const block_q4_K* b = (const block_q4_K*)row;
    size_t j = 0;
    for (uint32_t sb = 0; sb < K / 256; sb++) {
        const block_q4_K& blk = b[sb];
        double d = (double)blk.d, dmin = (double)blk.dmin;
        uint8_t sc[8], mn[8];
        for (int t = 0; t < 4; t++) {
            sc[t]     = blk.scales[t] & 0x3F;
            sc[t + 4] = blk.scales[t + 4] & 0x3F;
            mn[t]     = (blk.scales[t + 8] & 0x0F) | ((blk.scales[t] >> 6) << 4);
            mn[t + 4] = ((blk.scales[t + 8] >> 4) & 0x0F) | ((blk.scales[t + 4] >> 6) << 4);
        }
        for (int s = 0; s < 8; s++) {
            double d_sub = d * (double)sc[s];
            double m_sub = dmin * (double)mn[s];
            uint32_t kb = sb * 256 + s * 32;
            for (int i = 0; i < 16; i++) {
                uint8_t byte = blk.qs[s * 16 + i];
                w[j] = (double)(int)(byte & 0x0F) * d_sub - m_sub; kidx[j++] = kb + i;
                w[j] = (double)(int)(byte >> 4) * d_sub - m_sub;   kidx[j++] = kb + i + 16;
            }
        }
    }
}

// Ternary, 32-element blocks: tests/e2e/cpu_gold_reference.h:176-189 (code 3 gives +2*d here).
void expand_ternary(const uint8_t* row, uint32_t K, double* w, uint32_t* kidx) {
    const block_ternary_1_58* b = (const block_ternary_1_58*)row;
    size_t j = 0;
    for (uint32_t blk = 0; blk < K / 32; blk++) {
        double d = (double)b[blk].d;
        for (int u = 0; u < 2; u++) {
            uint32_t q = b[blk].qs[u];
            for (int t = 0; t < 16; t++) {
                int c = (int)((q >> (t * 2)) & 3u) - 1;
                w[j] = (double)c * d; kidx[j++] = blk * 32 + u * 16 + t;
            }
        }
    }
}

// Variable-rate affine: tests/e2e/cpu_gold_reference.h:214-311.
void expand_var_rate(const uint8_t* row, uint32_t K, double* w, uint32_t* kidx) {
    static const uint32_t sub_off[8] = {0, 12, 24, 40, 56, 72, 88, 108};
    const block_var_rate_affine* b = (const block_var_rate_affine*)row;
    size_t j = 0;
    for (uint32_t sb = 0; sb < K / 256; sb++) {
        const block_var_rate_affine& blk = b[sb];
        double d = (double)blk.d, bias = (double)blk.bias;
        for (int s = 0; s < 8; s++) {
            double sub_scale = d * (double)blk.scales[s] * 0.0625;
            double sub_bias = bias + d * ((double)blk.biases[s] - 128.0) * 0.0625;
            uint8_t mode = blk.modes[s];
            uint8_t bits = mode & 7u, perm = (mode >> 3) & 3u;
            const uint8_t* p = blk.qs + sub_off[s];
            double uw[32];
            if (bits == 3) {
                for (int g = 0; g < 4; g++) {
                    uint8_t q[8]; unpack3(p + g * 3, q);
                    for (int i = 0; i < 8; i++) uw[g * 8 + i] = ((double)q[i] - 4.0) * sub_scale + sub_bias;
                }
            } else if (bits == 5) {
                for (int g = 0; g < 4; g++) {
                    uint8_t q[8]; unpack5(p + g * 5, q);
                    for (int i = 0; i < 8; i++) uw[g * 8 + i] = ((double)q[i] - 16.0) * sub_scale + sub_bias;
                }
            } else {
                for (int i = 0; i < 16; i++) {
                    uw[i]      = ((double)(p[i] & 0x0F) - 8.0) * sub_scale + sub_bias;
                    uw[16 + i] = ((double)(p[i] >> 4) - 8.0) * sub_scale + sub_bias;
                }
            }
            uint32_t kb = sb * 256 + s * 32;
            for (int t = 0; t < 32; t++) {
                uint32_t dst = t;
                if (perm == 1) dst = ((t & 1) << 4) | (t >> 1);
                else if (perm == 2) dst = 31 - t;
                w[j] = uw[t]; kidx[j++] = kb + dst;
            }
        }
    }
}

// EXL3-style codebook: tests/e2e/cpu_gold_reference.h:342-389.
void expand_exl3(const uint8_t* row, uint32_t K, double* w, uint32_t* kidx) {
    const block_exl3* b = (const block_exl3*)row;
    size_t j = 0;
    for (uint32_t sb = 0; sb < K / 256; sb++) {
        const block_exl3& blk = b[sb];
        double d = (double)blk.d, bias = (double)blk.bias;
        for (int s = 0; s < 8; s++) {
            double sub_scale = d * (double)blk.scales[s] * 0.015625;
            double sub_res = d * ((double)blk.residuals[s] - 128.0) * 0.0078125;
            const uint8_t* p = blk.qs + s * 12;
            uint32_t kb = sb * 256 + s * 32;
            for (int g = 0; g < 4; g++) {
                uint8_t q[8]; unpack3(p + g * 3, q);
                for (int i = 0; i < 8; i++) {
                    double c_base = (double)blk.codebook[q[i]];
                    double c_res = (double)blk.codebook[q[i] + 8];
                    w[j] = bias + sub_scale * c_base + sub_res * c_res;
                    kidx[j++] = kb + g * 8 + i;
                }
            }
        }
    }
}

// Prism Q2_0, 128-element blocks: tests/e2e/cpu_gold_reference.h:416-429.
void expand_prism(const uint8_t* row, uint32_t K, double* w, uint32_t* kidx) {
    const block_prism_q2_0* b = (const block_prism_q2_0*)row;
    size_t j = 0;
    for (uint32_t blk = 0; blk < K / 128; blk++) {
        double d = (double)b[blk].d;
        for (int byte = 0; byte < 32; byte++) {
            uint8_t v = b[blk].qs[byte];
            for (int t = 0; t < 4; t++) {
                int c = (int)((v >> (t * 2)) & 3u) - 1;
                w[j] = (double)c * d; kidx[j++] = blk * 128 + byte * 4 + t;
            }
        }
    }
}

// Extension layouts (no reference gold; restatements of the MLX / ternary golds above with
// a different grouping).  The whole matrix is one buffer: planes follow one another.
//   MLX g64 : u32 qs[N][K/8] | f16 scale[N][K/64] | f16 bias[N][K/64]; nibble t of word i is k=8i+t.
//   ternary row-scale : u32 qs[N][K/16] | f16 row_scale[N]; code t of word i is k=16i+t.
void expand_mlx_g64(const uint8_t* base, uint32_t n, uint32_t N, uint32_t K, double* w, uint32_t* kidx) {
    const uint32_t* qs = (const uint32_t*)base + (size_t)n * (K / 8);
    const f16* scales = (const f16*)(base + (size_t)N * (K / 8) * 4) + (size_t)n * (K / 64);
    const f16* biases = (const f16*)(base + (size_t)N * (K / 8) * 4 + (size_t)N * (K / 64) * 2) + (size_t)n * (K / 64);
    for (uint32_t k = 0; k < K; k++) {
        uint32_t q = (qs[k / 8] >> (4 * (k % 8))) & 15u;
        w[k] = (double)(int)q * (double)scales[k / 64] + (double)biases[k / 64];
        kidx[k] = k;
    }
}
//   MLX planar g32 (the layout of the reference's layer benchmarks, unified_multi_scale_kernels.metal:17-31 and
//   bench_all_scales.mm:62-95; values as the AoS gold cpu_gold_reference.h:55-95): u8 qs[blocks][16] | f16 scale[blocks]
//   | f16 bias[blocks], planes padded to 16 bytes, block = n*(K/32) + k/32, byte j: low nibble = element j, high j+16.
void expand_mlx_planar(const uint8_t* base, uint32_t n, uint32_t N, uint32_t K, double* w, uint32_t* kidx) {
    const size_t blocks = (size_t)N * (K / 32);
    const size_t scales_off = (blocks * 16 + 15) & ~(size_t)15, biases_off = (scales_off + blocks * 2 + 15) & ~(size_t)15;
    const f16* scales = (const f16*)(base + scales_off);
    const f16* biases = (const f16*)(base + biases_off);
    for (uint32_t k = 0; k < K; k++) {
        const size_t blk = (size_t)n * (K / 32) + k / 32;
        const uint8_t byte = base[blk * 16 + (k % 16)];
        const int q = (k % 32) < 16 ? (byte & 15) : (byte >> 4);
        w[k] = (double)q * (double)scales[blk] + (double)biases[blk];
        kidx[k] = k;
    }
}
void expand_ternary_row(const uint8_t* base, uint32_t n, uint32_t N, uint32_t K, double* w, uint32_t* kidx) {
    const uint32_t* qs = (const uint32_t*)base + (size_t)n * (K / 16);
    const f16* rs = (const f16*)(base + (size_t)N * (K / 16) * 4);
    double d = (double)rs[n];
    for (uint32_t k = 0; k < K; k++) {
        int c = (int)((qs[k / 16] >> (2 * (k % 16))) & 3u) - 1;
        w[k] = (double)c * d; kidx[k] = k;
    }
}

bool expand_row(int format, const uint8_t* W, uint32_t n, uint32_t N, uint32_t K, double* w, uint32_t* kidx) {
    if (format == QUANT_MLX_4BIT_G64) { expand_mlx_g64(W, n, N, K, w, kidx); return true; }
    if (format == QUANT_TERNARY_ROW)  { expand_ternary_row(W, n, N, K, w, kidx); return true; }
    if (format == QUANT_MLX_4BIT_PLANAR) { expand_mlx_planar(W, n, N, K, w, kidx); return true; }
    QuantFormatInfo info = get_quant_info((QuantFormat)format);
    const uint8_t* row = W + (size_t)n * (K / info.block_size) * info.block_bytes;
    switch (format) {
        case QUANT_Q4_0: expand_q4_0(row, K, w, kidx); return true;
        case QUANT_MLX_4BIT: expand_mlx(row, K, w, kidx); return true;
        case QUANT_Q4_K: expand_q4_k(row, K, w, kidx); return true;
        case QUANT_TERNARY_1_58: expand_ternary(row, K, w, kidx); return true;
        case QUANT_VAR_RATE_AFFINE: expand_var_rate(row, K, w, kidx); return true;
        case QUANT_EXL3: expand_exl3(row, K, w, kidx); return true;
        case QUANT_PRISM_Q2_0: expand_prism(row, K, w, kidx); return true;
        default: return false;
    }
}

inline bool format_ok(int format, uint32_t K) {
    if (format == QUANT_MLX_4BIT_G64) return K % 64 == 0;
    if (format == QUANT_TERNARY_ROW) return K % 16 == 0;
    if (format == QUANT_MLX_4BIT_PLANAR) return K % 32 == 0;
    if (format < 0 || format > 7 || format == QUANT_Q8_0) return false;
    return K % get_quant_info((QuantFormat)format).block_size == 0;
}

// LCG shared by every reference generator (tests/e2e/test_common.h:259-266).
struct Lcg {
    uint32_t s;
    uint32_t next() { s = s * 1664525u + 1013904223u; return s; }
    float u() { return (float)next() / (float)0xFFFFFFFF; }
    float uniform(float lo, float hi) { float t = u(); return lo + t * (hi - lo); }
};

inline uint8_t nibble_byte(Lcg& g) {       // tests/e2e/test_common.h:283-285
    uint8_t low = (uint8_t)g.uniform(0.0f, 16.0f);
    uint8_t high = (uint8_t)g.uniform(0.0f, 16.0f);
    return (uint8_t)((high << 4) | (low & 0x0F));
}
inline void pack3(Lcg& g, uint8_t* out) {  // tests/e2e/test_common.h:362-367
    uint8_t q[8];
    for (int i = 0; i < 8; i++) q[i] = (uint8_t)g.uniform(0.0f, 8.0f) & 7u;
    out[0] = q[0] | (q[1] << 3) | ((q[2] & 3) << 6);
    out[1] = (q[2] >> 2) | (q[3] << 1) | (q[4] << 4) | ((q[5] & 1) << 7);
    out[2] = (q[5] >> 1) | (q[6] << 2) | (q[7] << 5);
}

}  // namespace

extern "C" {

// ------------------------------------------------------------------------------------
// GEMM gold: C = fp16( sum_k A[m,k] * dequant(W)[n,k] ) in double
// (tests/e2e/cpu_gold_reference.h:15-440; identical copies in bench_universal_router.mm:199-583).
// Returns 0, or -3 for an unknown format / -4 for a K the format cannot tile.
// ------------------------------------------------------------------------------------
int orc_gemm(int format, const f16* A, const uint8_t* W, f16* C, uint32_t M, uint32_t N, uint32_t K,
             int direct_head, uint32_t H, uint32_t D) {
    if (!format_ok(format, K)) return (format >= 0 && (format <= 7 || format >= 100) && format != QUANT_Q8_0) ? -4 : -3;
    std::vector<double> Ad((size_t)M * K);
    for (size_t i = 0; i < (size_t)M * K; i++) Ad[i] = (double)A[i];
#pragma omp parallel
    {
        std::vector<double> w(K);
        std::vector<uint32_t> kidx(K);
#pragma omp for schedule(dynamic, 4)
        for (int64_t n = 0; n < (int64_t)N; n++) {
            expand_row(format, W, (uint32_t)n, N, K, w.data(), kidx.data());
            for (uint32_t m = 0; m < M; m++) {
                const double* a = Ad.data() + (size_t)m * K;
                double acc = 0.0;
                for (uint32_t j = 0; j < K; j++) acc += a[kidx[j]] * w[j];
                size_t o = (direct_head && H > 0 && D > 0)
                               ? ((size_t)(n / D) * M + m) * D + (n % D)
                               : (size_t)m * N + n;
                C[o] = (f16)acc;
            }
        }
    }
    return 0;
}

// Same contraction, double output (no fp16 rounding) -- used for ulp-aware tolerances.
int orc_gemm_f64(int format, const f16* A, const uint8_t* W, double* C, uint32_t M, uint32_t N, uint32_t K) {
    if (!format_ok(format, K)) return -4;
    std::vector<double> Ad((size_t)M * K);
    for (size_t i = 0; i < (size_t)M * K; i++) Ad[i] = (double)A[i];
#pragma omp parallel
    {
        std::vector<double> w(K);
        std::vector<uint32_t> kidx(K);
#pragma omp for schedule(dynamic, 4)
        for (int64_t n = 0; n < (int64_t)N; n++) {
            expand_row(format, W, (uint32_t)n, N, K, w.data(), kidx.data());
            for (uint32_t m = 0; m < M; m++) {
                const double* a = Ad.data() + (size_t)m * K;
                double acc = 0.0;
                for (uint32_t j = 0; j < K; j++) acc += a[kidx[j]] * w[j];
                C[(size_t)m * N + n] = acc;
            }
        }
    }
    return 0;
}

// Dequantise a whole matrix to double [N][K] in natural k order (bit-exact unpack checks).
int orc_dequant_matrix(int format, const uint8_t* W, double* out, uint32_t N, uint32_t K) {
    if (!format_ok(format, K)) return -4;
    std::vector<double> w(K);
    std::vector<uint32_t> kidx(K);
    for (uint32_t n = 0; n < N; n++) {
        expand_row(format, W, n, N, K, w.data(), kidx.data());
        for (uint32_t j = 0; j < K; j++) out[(size_t)n * K + kidx[j]] = w[j];
    }
    return 0;
}

// ------------------------------------------------------------------------------------
// Fused SwiGLU gold: Out = fp16( silu(A.Wg^T) * (A.Wu^T) ), double through the activation
// (brick3_swiglu_bench.mm:49-99; the reference is Q4_0 only, here any format).
// ------------------------------------------------------------------------------------
int orc_swiglu_fused(int format, const f16* A, const uint8_t* Wg, const uint8_t* Wu, f16* Out,
                     uint32_t M, uint32_t F, uint32_t K) {
    if (!format_ok(format, K)) return -4;
    std::vector<double> Ad((size_t)M * K);
    for (size_t i = 0; i < (size_t)M * K; i++) Ad[i] = (double)A[i];
#pragma omp parallel
    {
        std::vector<double> wg(K), wu(K);
        std::vector<uint32_t> kidx(K), kidx2(K);
#pragma omp for schedule(dynamic, 4)
        for (int64_t n = 0; n < (int64_t)F; n++) {
            expand_row(format, Wg, (uint32_t)n, F, K, wg.data(), kidx.data());
            expand_row(format, Wu, (uint32_t)n, F, K, wu.data(), kidx2.data());
            for (uint32_t m = 0; m < M; m++) {
                const double* a = Ad.data() + (size_t)m * K;
                double g = 0.0, u = 0.0;
                for (uint32_t j = 0; j < K; j++) { g += a[kidx[j]] * wg[j]; u += a[kidx[j]] * wu[j]; }
                double silu = g / (1.0 + std::exp(-g));
                Out[(size_t)m * F + n] = (f16)(silu * u);
            }
        }
    }
    return 0;
}

// Elementwise SwiGLU in fp32 on fp16 inputs (tests/e2e/cpu_gold_reference.h:499-511).
void orc_swiglu_elementwise(const f16* gate, const f16* up, f16* out, uint32_t count) {
    for (uint32_t i = 0; i < count; i++) {
        float g = (float)gate[i], u = (float)up[i];
        float s = g / (1.0f + std::exp(-g));
        out[i] = (f16)(s * u);
    }
}

// ------------------------------------------------------------------------------------
// Q8_0 KV compression (brick4_attn_bench.mm:37-65; device twin unified_8b_kernels.metal:118-145):
// d32 = amax/127 in fp32, stored d = fp16(d32); q = clamp(round_half_away(x * (1/d32)), -128, 127).
// ------------------------------------------------------------------------------------
void orc_quantize_q8_0(const f16* src, block_q8_0* dst, size_t num_elements) {
    size_t nb = num_elements / 32;
    for (size_t b = 0; b < nb; b++) {
        const f16* s = src + b * 32;
        float amax = 0.0f;
        for (int i = 0; i < 32; i++) amax = std::max(amax, std::fabs((float)s[i]));
        float d = amax / 127.0f;
        dst[b].d = (f16)d;
        float id = (d > 0.0f) ? (1.0f / d) : 0.0f;
        for (int i = 0; i < 32; i++) {
            int q = (int)std::round((float)s[i] * id);
            dst[b].qs[i] = (int8_t)std::max(-128, std::min(127, q));
        }
    }
}
void orc_dequantize_q8_0(const block_q8_0* src, f16* dst, size_t num_elements) {
    size_t nb = num_elements / 32;
    for (size_t b = 0; b < nb; b++) {
        float d = (float)src[b].d;
        for (int i = 0; i < 32; i++) dst[b * 32 + i] = (f16)((float)src[b].qs[i] * d);
    }
}

// ------------------------------------------------------------------------------------
// Causal attention gold in double (brick4_attn_bench.mm:70-119; tests/e2e/cpu_gold_reference.h:443-496).
// Q [Hq,M,D]; K,V [Hkv,Mkv,D] fp16; query row i sits at absolute position pos0+i and attends
// keys 0..pos0+i.  Hq == Hkv, pos0 == 0, Mkv == M is the reference case; Hkv < Hq maps
// query head h to kv head h / (Hq/Hkv) (grouped-query attention: restated, unpinned).
// out_tokens_major != 0 writes O[m][h*D+d] instead of O[h][m][d].
// ------------------------------------------------------------------------------------
void orc_attention(const f16* Q, const f16* K, const f16* V, f16* O, uint32_t Hq, uint32_t Hkv, uint32_t M,
                   uint32_t Mkv, uint32_t D, float scale, uint32_t pos0, int out_tokens_major) {
    uint32_t group = Hq / Hkv;
#pragma omp parallel for schedule(dynamic, 1) collapse(2)
    for (int64_t h = 0; h < (int64_t)Hq; h++) {
        for (int64_t i = 0; i < (int64_t)M; i++) {
            const f16* q = Q + ((size_t)h * M + i) * D;
            const f16* kh = K + (size_t)(h / group) * Mkv * D;
            const f16* vh = V + (size_t)(h / group) * Mkv * D;
            uint32_t last = std::min<uint32_t>(pos0 + (uint32_t)i, Mkv - 1);
            std::vector<double> sc(last + 1);
            double mx = -1e30;
            for (uint32_t j = 0; j <= last; j++) {
                double dot = 0.0;
                for (uint32_t d = 0; d < D; d++) dot += (double)q[d] * (double)kh[(size_t)j * D + d];
                double s = dot * (double)scale;
                sc[j] = s;
                if (s > mx) mx = s;
            }
            double sum = 0.0;
            for (uint32_t j = 0; j <= last; j++) { sc[j] = std::exp(sc[j] - mx); sum += sc[j]; }
            double inv = (sum > 0.0) ? 1.0 / sum : 0.0;
            for (uint32_t d = 0; d < D; d++) {
                double acc = 0.0;
                for (uint32_t j = 0; j <= last; j++) acc += (sc[j] * inv) * (double)vh[(size_t)j * D + d];
                size_t o = out_tokens_major ? ((size_t)i * Hq + h) * D + d : ((size_t)h * M + i) * D + d;
                O[o] = (f16)acc;
            }
        }
    }
}

// ------------------------------------------------------------------------------------
// RMSNorm (src/engine/model.py:39-45): fp32 mean square, x*rsqrt(var+eps) rounded to fp16,
// then times the fp16 weight (rounded to fp16 again).  Restated in double for the sums.
// ------------------------------------------------------------------------------------
void orc_rmsnorm(const f16* X, const f16* weight, f16* Y, uint32_t M, uint32_t K, float eps) {
    for (uint32_t m = 0; m < M; m++) {
        double ss = 0.0;
        for (uint32_t k = 0; k < K; k++) { double v = (double)X[(size_t)m * K + k]; ss += v * v; }
        double r = 1.0 / std::sqrt(ss / (double)K + (double)eps);
        for (uint32_t k = 0; k < K; k++) {
            f16 normed = (f16)((double)X[(size_t)m * K + k] * r);
            Y[(size_t)m * K + k] = (f16)((float)normed * (float)weight[k]);
        }
    }
}

// ------------------------------------------------------------------------------------
// Rotary embedding, non-interleaved ("rotate-half") form selected by traditional=False in
// src/engine/model.py:112-116: element i pairs with i+D/2, angle = pos * theta^(-2i/D).
// X is [H][M][D]; positions start at pos0.  In place, double trig.
// ------------------------------------------------------------------------------------
void orc_rope(f16* X, uint32_t H, uint32_t M, uint32_t D, float theta, uint32_t pos0) {
    uint32_t half = D / 2;
    for (uint32_t h = 0; h < H; h++)
        for (uint32_t m = 0; m < M; m++) {
            f16* x = X + ((size_t)h * M + m) * D;
            for (uint32_t i = 0; i < half; i++) {
                double inv_freq = std::pow((double)theta, -2.0 * (double)i / (double)D);
                double ang = (double)(pos0 + m) * inv_freq;
                double c = std::cos(ang), s = std::sin(ang);
                double a = (double)x[i], b = (double)x[i + half];
                x[i] = (f16)(a * c - b * s);
                x[i + half] = (f16)(b * c + a * s);
            }
        }
}

// ------------------------------------------------------------------------------------
// Layer gold, composed from the golds above with the reference's rounding points
// (bench_8b_engine.mm:74-225: X_mid = fp16(X + O), S = fp16(silu(g)*u), X_out = fp16(X_mid + down);
// attention output rounded to fp16 before the O projection).  Accumulators are double where
// the reference uses float.  Switches add what only the reference's Python block has:
// rms_eps > 0 enables the two RMSNorms (norm weights norm1/norm2, fp16 [K]); rope_theta > 0
// enables RoPE on Q and K; Hkv < H is grouped-query attention; kv_q8 != 0 round-trips K and V
// through Q8_0 before attention.  W_q is [H*D][K], W_k/W_v are [Hkv*D][K], W_o is [K][H*D].
// ------------------------------------------------------------------------------------
int orc_layer(int format, const f16* X_in, const uint8_t* Wq, const uint8_t* Wk, const uint8_t* Wv,
              const uint8_t* Wo, const uint8_t* Wg, const uint8_t* Wu, const uint8_t* Wd, f16* X_out,
              uint32_t M, uint32_t K, uint32_t H, uint32_t Hkv, uint32_t D, uint32_t F, float attn_scale,
              float rms_eps, const f16* norm1, const f16* norm2, float rope_theta, int kv_q8) {
    size_t MK = (size_t)M * K;
    uint32_t QD = H * D, KD = Hkv * D;
    std::vector<f16> xn(MK), q((size_t)M * QD), k((size_t)M * KD), v((size_t)M * KD);
    const f16* x_attn = X_in;
    if (rms_eps > 0.0f) { orc_rmsnorm(X_in, norm1, xn.data(), M, K, rms_eps); x_attn = xn.data(); }
    // head-major projections (the reference rounds Q,K,V to fp16 on its device path: the
    // direct-head GEMM writes fp16)
    int rc = orc_gemm(format, x_attn, Wq, q.data(), M, QD, K, 1, H, D);
    if (rc) return rc;
    orc_gemm(format, x_attn, Wk, k.data(), M, KD, K, 1, Hkv, D);
    orc_gemm(format, x_attn, Wv, v.data(), M, KD, K, 1, Hkv, D);
    if (rope_theta > 0.0f) { orc_rope(q.data(), H, M, D, rope_theta, 0); orc_rope(k.data(), Hkv, M, D, rope_theta, 0); }
    if (kv_q8) {
        std::vector<block_q8_0> blk((size_t)M * KD / 32);
        orc_quantize_q8_0(k.data(), blk.data(), (size_t)M * KD); orc_dequantize_q8_0(blk.data(), k.data(), (size_t)M * KD);
        orc_quantize_q8_0(v.data(), blk.data(), (size_t)M * KD); orc_dequantize_q8_0(blk.data(), v.data(), (size_t)M * KD);
    }
    std::vector<f16> attn((size_t)M * QD);
    orc_attention(q.data(), k.data(), v.data(), attn.data(), H, Hkv, M, M, D, attn_scale, 0, 1);
    std::vector<double> proj(MK);
    orc_gemm_f64(format, attn.data(), Wo, proj.data(), M, K, QD);
    std::vector<f16> x_mid(MK);
    for (size_t i = 0; i < MK; i++) x_mid[i] = (f16)((double)X_in[i] + proj[i]);
    const f16* x_mlp = x_mid.data();
    if (rms_eps > 0.0f) { orc_rmsnorm(x_mid.data(), norm2, xn.data(), M, K, rms_eps); x_mlp = xn.data(); }
    std::vector<f16> act((size_t)M * F);
    orc_swiglu_fused(format, x_mlp, Wg, Wu, act.data(), M, F, K);
    orc_gemm_f64(format, act.data(), Wd, proj.data(), M, K, F);
    for (size_t i = 0; i < MK; i++) X_out[i] = (f16)((double)x_mid[i] + proj[i]);
    return 0;
}

// ------------------------------------------------------------------------------------
// Seeded generators, family "tests": tests/e2e/test_common.h:253-427 (one LCG state that
// the caller threads through: pass the state in, get the advanced state back).
// ------------------------------------------------------------------------------------
uint32_t orc_gen_activations(uint32_t state, f16* data, size_t count) {   // test_common.h:269-276
    Lcg g{state};
    for (size_t i = 0; i < count; i++) {
        float u1 = std::max(1e-6f, (float)g.next() / 4294967295.0f);
        float u2 = (float)g.next() / 4294967295.0f;
        float z0 = std::sqrt(-2.0f * std::log(u1)) * std::cos(2.0f * 3.14159265f * u2);
        data[i] = (f16)(z0 * 0.35f);
    }
    return g.s;
}

uint32_t orc_gen_weights(uint32_t state, int format, uint8_t* out, size_t num_blocks) {
    Lcg g{state};
    switch (format) {
        case QUANT_Q4_0: {                                   // test_common.h:279-288
            block_q4_0* b = (block_q4_0*)out;
            for (size_t i = 0; i < num_blocks; i++) {
                b[i].d = (f16)g.uniform(0.002f, 0.04f);
                for (int t = 0; t < 16; t++) b[i].qs[t] = nibble_byte(g);
            }
            break;
        }
        case QUANT_MLX_4BIT: {                               // test_common.h:290-300
            block_mlx_4bit* b = (block_mlx_4bit*)out;
            for (size_t i = 0; i < num_blocks; i++) {
                b[i].d = (f16)g.uniform(0.001f, 0.03f);
                b[i].bias = (f16)g.uniform(-0.05f, 0.05f);
                for (int t = 0; t < 16; t++) b[i].qs[t] = nibble_byte(g);
            }
            break;
        }
        case QUANT_Q4_K: {                                   // test_common.h:302-325
            block_q4_K* b = (block_q4_K*)out;
            for (size_t i = 0; i < num_blocks; i++) {
                b[i].d = (f16)g.uniform(0.0002f, 0.002f);
                b[i].dmin = (f16)g.uniform(0.0001f, 0.001f);
                uint8_t sc[8], mn[8];
                for (int t = 0; t < 8; t++) { sc[t] = (uint8_t)g.uniform(1.0f, 63.0f); mn[t] = (uint8_t)g.uniform(0.0f, 63.0f); }
                for (int t = 0; t < 4; t++) {
                    b[i].scales[t]     = (sc[t] & 0x3F) | ((mn[t] >> 4) << 6);
                    b[i].scales[t + 4] = (sc[t + 4] & 0x3F) | ((mn[t + 4] >> 4) << 6);
                    b[i].scales[t + 8] = (mn[t] & 0x0F) | ((mn[t + 4] & 0x0F) << 4);
                }
                for (int t = 0; t < 128; t++) b[i].qs[t] = nibble_byte(g);
            }
            break;
        }
        case QUANT_TERNARY_1_58: {                           // test_common.h:327-341
            block_ternary_1_58* b = (block_ternary_1_58*)out;
            for (size_t i = 0; i < num_blocks; i++) {
                b[i].d = (f16)g.uniform(0.01f, 0.05f);
                b[i]._pad = (f16)0;
                for (int u = 0; u < 2; u++) {
                    uint32_t val = 0;
                    for (int t = 0; t < 16; t++) {
                        int c = (int)g.uniform(0.0f, 3.0f);
                        if (c > 2) c = 2;
                        val |= (uint32_t)c << (t * 2);
                    }
                    b[i].qs[u] = val;
                }
            }
            break;
        }
        case QUANT_VAR_RATE_AFFINE: {                        // test_common.h:343-388
            static const uint32_t sub_off[8] = {0, 12, 24, 40, 56, 72, 88, 108};
            static const uint8_t sub_bits[8] = {3, 3, 4, 4, 4, 4, 5, 5};
            block_var_rate_affine* b = (block_var_rate_affine*)out;
            for (size_t i = 0; i < num_blocks; i++) {
                b[i].d = (f16)g.uniform(0.0004f, 0.004f);
                b[i].bias = (f16)g.uniform(-0.005f, 0.01f);
                std::memset(b[i]._pad, 0, 4);
                for (int s = 0; s < 8; s++) {
                    b[i].scales[s] = (uint8_t)g.uniform(10.0f, 210.0f);
                    b[i].biases[s] = (uint8_t)g.uniform(0.0f, 255.0f);
                    b[i].modes[s] = (uint8_t)(((s % 3) << 3) | sub_bits[s]);
                    uint8_t* p = b[i].qs + sub_off[s];
                    if (sub_bits[s] == 3) {
                        for (int gi = 0; gi < 4; gi++) pack3(g, p + gi * 3);
                    } else if (sub_bits[s] == 5) {
                        for (int gi = 0; gi < 4; gi++) {
                            uint8_t q[8];
                            for (int t = 0; t < 8; t++) q[t] = (uint8_t)g.uniform(0.0f, 32.0f) & 31u;
                            uint64_t v = 0;
                            for (int t = 0; t < 8; t++) v |= (uint64_t)q[t] << (5 * t);
                            for (int t = 0; t < 5; t++) p[gi * 5 + t] = (uint8_t)(v >> (8 * t));
                        }
                    } else {
                        for (int t = 0; t < 16; t++) p[t] = nibble_byte(g);
                    }
                }
            }
            break;
        }
        case QUANT_EXL3: {                                   // test_common.h:390-413
            block_exl3* b = (block_exl3*)out;
            for (size_t i = 0; i < num_blocks; i++) {
                b[i].d = (f16)g.uniform(0.0003f, 0.003f);
                b[i].bias = (f16)g.uniform(-0.004f, 0.008f);
                std::memset(b[i]._pad, 0, 12);
                for (int t = 0; t < 16; t++) b[i].codebook[t] = (int8_t)g.uniform(-8.0f, 7.0f);
                for (int s = 0; s < 8; s++) {
                    b[i].scales[s] = (uint8_t)g.uniform(15.0f, 220.0f);
                    b[i].residuals[s] = (uint8_t)g.uniform(0.0f, 255.0f);
                    for (int gi = 0; gi < 4; gi++) pack3(g, b[i].qs + s * 12 + gi * 3);
                }
            }
            break;
        }
        case QUANT_PRISM_Q2_0: {                             // test_common.h:415-427
            block_prism_q2_0* b = (block_prism_q2_0*)out;
            for (size_t i = 0; i < num_blocks; i++) {
                b[i].d = (f16)g.uniform(0.01f, 0.05f);
                for (int t = 0; t < 32; t++) {
                    uint8_t val = 0;
                    for (int c = 0; c < 4; c++) val |= (uint8_t)((g.next() % 4) << (c * 2));
                    b[i].qs[t] = val;
                }
            }
            break;
        }
        default: break;
    }
    return g.s;
}

// Brick-3 inputs: X = u*2-1, Q4_0 d = u*0.04+0.002 (brick3_swiglu_bench.mm:23-44).
uint32_t orc_gen_brick3_activations(uint32_t state, f16* data, size_t count) {
    Lcg g{state};
    for (size_t i = 0; i < count; i++) data[i] = (f16)(g.u() * 2.0f - 1.0f);
    return g.s;
}
// Q4_0 with d = u*range + offset; nibbles as (uint8)(u*16): the generator of the benches
// (bench_universal_router.mm:38-47 uses range 0.04, offset 0.002; bench_8b_engine.mm:44-53 uses
// range 0.003, offset 0.0003).
uint32_t orc_gen_q4_0_affine_scale(uint32_t state, uint8_t* out, size_t num_blocks, float range, float offset) {
    Lcg g{state};
    block_q4_0* b = (block_q4_0*)out;
    for (size_t i = 0; i < num_blocks; i++) {
        b[i].d = (f16)(g.u() * range + offset);
        for (int t = 0; t < 16; t++) {
            uint8_t low = (uint8_t)(g.u() * 16.0f);
            uint8_t high = (uint8_t)(g.u() * 16.0f);
            b[i].qs[t] = (uint8_t)((high << 4) | (low & 0x0F));
        }
    }
    return g.s;
}

int orc_num_threads(void);
// Sets the OpenMP team size of later calls (n <= 0: leave as is) and returns the size a parallel region then gets.
// Launchers such as torchrun export OMP_NUM_THREADS=1 to their children; a caller that wants every host core says so here.
int orc_set_num_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#endif
    return orc_num_threads();
}

int orc_num_threads(void) {
    int n = 1;
#ifdef _OPENMP
#pragma omp parallel
    {
#pragma omp single
        n = omp_get_num_threads();
    }
#endif
    return n;
}

}  // extern "C"
