// Per-format unpackers: packed weight bytes (held in registers) -> fp16 pairs.
//
// One thread owns one weight row.  For every K chunk (`CHUNK` elements: 256, or 1024 for the
// 34-byte Prism blocks, whose rows are a 16-byte multiple only every 1024 elements) it holds the
// row's packed bytes (`ROW_BYTES`, a multiple of 16 for every format) in registers `r[]` and
// produces, for each 64-element sub-tile `s` of the chunk, 32 words `out[i]` = fp16 pair
// (k = 2i, 2i+1).  All loops unroll so that register indices are compile-time constants.
//
// Arithmetic follows the reference's device unpackers (quant_router_kernels.metal:111-436): the
// integer code is turned into an exact fp16 value and one fused fp16 multiply-add applies the
// scale (and bias / minimum), so each weight is rounded once, exactly as `fma(half4(q), d, off)`
// does there.  Integer -> fp16 uses the mantissa trick: 0x6400|q is the fp16 number 1024+q and
// 0x5400|(q<<4) is 64+q, so a nibble never needs a convert instruction.
//
// The same code compiles for the host (tests/codec_host_shim.cpp, built with g++ by
// tests/test_host_cpu.py) with `prmt` and the fp16 pair arithmetic emulated, which lets the unpack
// logic be checked bit-for-bit against the CPU oracle without a GPU.
#pragma once
#include <cstdint>
#include "../../include/quant_router.h"

#if defined(__CUDACC__)
#include <cuda_fp16.h>
#define CDC_HD __host__ __device__ __forceinline__
#else
#define CDC_HD inline
#endif

namespace cdc {

// ---- primitive helpers -------------------------------------------------------------------
CDC_HD uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
#if defined(__CUDA_ARCH__)
    return __byte_perm(a, b, sel);
#else
    uint64_t src = (uint64_t)a | ((uint64_t)b << 32);
    uint32_t out = 0;
    for (int i = 0; i < 4; i++) {
        uint32_t n = (sel >> (4 * i)) & 7u;
        out |= (uint32_t)((src >> (8 * n)) & 0xFF) << (8 * i);
    }
    return out;
#endif
}

#if !defined(__CUDA_ARCH__)
inline _Float16 bits2h(uint16_t b) { _Float16 h; __builtin_memcpy(&h, &b, 2); return h; }
inline uint16_t h2bits(_Float16 h) { uint16_t b; __builtin_memcpy(&b, &h, 2); return b; }
inline uint32_t pack2(_Float16 lo, _Float16 hi) { return (uint32_t)h2bits(lo) | ((uint32_t)h2bits(hi) << 16); }
#endif

// fp16x2 arithmetic on raw 32-bit words (each result rounded once, like the hardware)
CDC_HD uint32_t h2sub(uint32_t a, uint32_t b) {
#if defined(__CUDA_ARCH__)
    __half2 r = __hsub2(*reinterpret_cast<__half2*>(&a), *reinterpret_cast<__half2*>(&b));
    return *reinterpret_cast<uint32_t*>(&r);
#else
    return pack2((_Float16)((double)bits2h(a & 0xFFFF) - (double)bits2h(b & 0xFFFF)),
                 (_Float16)((double)bits2h(a >> 16) - (double)bits2h(b >> 16)));
#endif
}
CDC_HD uint32_t h2mul(uint32_t a, uint32_t b) {
#if defined(__CUDA_ARCH__)
    __half2 r = __hmul2(*reinterpret_cast<__half2*>(&a), *reinterpret_cast<__half2*>(&b));
    return *reinterpret_cast<uint32_t*>(&r);
#else
    return pack2((_Float16)((double)bits2h(a & 0xFFFF) * (double)bits2h(b & 0xFFFF)),
                 (_Float16)((double)bits2h(a >> 16) * (double)bits2h(b >> 16)));
#endif
}
CDC_HD uint32_t h2fma(uint32_t a, uint32_t b, uint32_t c) {
#if defined(__CUDA_ARCH__)
    __half2 r = __hfma2(*reinterpret_cast<__half2*>(&a), *reinterpret_cast<__half2*>(&b), *reinterpret_cast<__half2*>(&c));
    return *reinterpret_cast<uint32_t*>(&r);
#else
    return pack2((_Float16)((double)bits2h(a & 0xFFFF) * (double)bits2h(b & 0xFFFF) + (double)bits2h(c & 0xFFFF)),
                 (_Float16)((double)bits2h(a >> 16) * (double)bits2h(b >> 16) + (double)bits2h(c >> 16)));
#endif
}
CDC_HD float h_lo_to_float(uint32_t w) {
#if defined(__CUDA_ARCH__)
    return __half2float(__ushort_as_half((unsigned short)(w & 0xFFFF)));
#else
    return (float)bits2h(w & 0xFFFF);
#endif
}
CDC_HD float h_hi_to_float(uint32_t w) { return h_lo_to_float(w >> 16); }
CDC_HD uint32_t float_to_h(float f) {  // fp16 bits in the low half
#if defined(__CUDA_ARCH__)
    return (uint32_t)__half_as_ushort(__float2half_rn(f));
#else
    return (uint32_t)h2bits((_Float16)f);
#endif
}
CDC_HD uint32_t dup16(uint32_t h) { return (h & 0xFFFFu) | (h << 16); }

// 16-bit field at (even) byte offset `o` of the register file, copied into both halves
CDC_HD uint32_t bcast16(const uint32_t* r, int o) {
    return (o & 2) ? prmt(r[o >> 2], 0u, 0x3232u) : prmt(r[o >> 2], 0u, 0x1010u);
}
// bytes o, o+1 (o even) -> byte o in bits 0-7, byte o+1 in bits 16-23
CDC_HD uint32_t spread_pair(const uint32_t* r, int o) {
    return (o & 2) ? prmt(r[o >> 2], 0u, 0x4342u) : prmt(r[o >> 2], 0u, 0x4140u);
}
CDC_HD uint32_t byte_at(const uint32_t* r, int o) { return (r[o >> 2] >> (8 * (o & 3))) & 0xFFu; }

constexpr uint32_t H2_1024 = 0x64006400u, H2_64 = 0x54005400u;
constexpr uint32_t H2_1032 = 0x64086408u, H2_72 = 0x54805480u;   // 1024+8, 64+8
constexpr uint32_t H2_1025 = 0x64016401u;

// two bytes spread by spread_pair -> (1024 + low nibbles) and (64 + high nibbles)
CDC_HD void nib_pairs(uint32_t sp, uint32_t& lo, uint32_t& hi) {
    lo = (sp & 0x000F000Fu) | H2_1024;
    hi = (sp & 0x00F000F0u) | H2_64;
}

// Traits every codec may override: META_WORDS 32-bit words of per-chunk metadata that live outside the packed
// row (fetched from global memory by the unpack thread), ROW_SCALE when the weights are unpacked to exact small
// integers and one fp16 scale per output row is applied to the fp32 accumulator instead.
// HDR_WORDS / sub_lo / sub_hi describe which 32-bit words of the packed row dequant64(r, s, ...) reads: the
// header words [0, HDR_WORDS) plus the words [sub_lo(s), sub_hi(s)).  The unpack thread loads only those.
struct CodecDefaults {
    static constexpr int CHUNK = 256;     // K elements per packed stage (ROW_BYTES bytes of a row)
    static constexpr int TMA_ELEM_BYTES = 1;   // element size of the TMA map over the packed bytes (a box side holds at most 256 elements)
    static constexpr int HDR_WORDS = 0;
    static constexpr int META_WORDS = 0;
    static constexpr bool ROW_SCALE = false;
    static constexpr bool RAW_SWIZZLE_128 = false;   // packed tile staged with the 128-byte swizzle (ROW_BYTES == 128 only)
};

template <int FMT> struct Codec;

// ---- Q4_0: 18 B / 32 (quant_router_kernels.metal:111-146) ---------------------------------
template <> struct Codec<QUANT_Q4_0> : CodecDefaults {
    static constexpr int ROW_BYTES = 144;   // 8 blocks per 256 elements
    static constexpr int GROUPS = 3;      // unpack warp groups per matrix in the projection kernel
    CDC_HD static constexpr int sub_lo(int s) { return 9 * s; }
    CDC_HD static constexpr int sub_hi(int s) { return 9 * s + 9; }
    CDC_HD static void dequant64(const uint32_t* r, int s, uint32_t* out, const uint32_t* = nullptr) {
#pragma unroll
        for (int bi = 0; bi < 2; bi++) {
            const int o = 18 * (2 * s + bi);
            const uint32_t d2 = bcast16(r, o);
#pragma unroll
            for (int p = 0; p < 8; p++) {
                uint32_t lo, hi;
                nib_pairs(spread_pair(r, o + 2 + 2 * p), lo, hi);
                out[16 * bi + p] = h2mul(h2sub(lo, H2_1032), d2);       // elements 2p, 2p+1
                out[16 * bi + 8 + p] = h2mul(h2sub(hi, H2_72), d2);     // elements 16+2p, 17+2p
            }
        }
    }
};

// ---- MLX 4-bit affine, 20 B / 32 (quant_router_kernels.metal:149-185) -----------------------
template <> struct Codec<QUANT_MLX_4BIT> : CodecDefaults {
    static constexpr int ROW_BYTES = 160;
    static constexpr int GROUPS = 3;      // unpack warp groups per matrix in the projection kernel
    CDC_HD static constexpr int sub_lo(int s) { return 10 * s; }
    CDC_HD static constexpr int sub_hi(int s) { return 10 * s + 10; }
    CDC_HD static void dequant64(const uint32_t* r, int s, uint32_t* out, const uint32_t* = nullptr) {
#pragma unroll
        for (int bi = 0; bi < 2; bi++) {
            const int o = 20 * (2 * s + bi);
            const uint32_t d2 = bcast16(r, o), b2 = bcast16(r, o + 2);
#pragma unroll
            for (int p = 0; p < 8; p++) {
                uint32_t lo, hi;
                nib_pairs(spread_pair(r, o + 4 + 2 * p), lo, hi);
                out[16 * bi + p] = h2fma(h2sub(lo, H2_1024), d2, b2);
                out[16 * bi + 8 + p] = h2fma(h2sub(hi, H2_64), d2, b2);
            }
        }
    }
};

// ---- Q4_K, 144 B / 256 (quant_router_kernels.metal:188-238; gold cpu_gold_reference.h:116-146) --
template <> struct Codec<QUANT_Q4_K> : CodecDefaults {
    static constexpr int ROW_BYTES = 144;
    static constexpr int GROUPS = 3;      // unpack warp groups per matrix in the projection kernel
    static constexpr int HDR_WORDS = 4;   // d, dmin, 12 bytes of 6-bit scales / minimums
    CDC_HD static constexpr int sub_lo(int s) { return 4 + 8 * s; }
    CDC_HD static constexpr int sub_hi(int s) { return 12 + 8 * s; }
    CDC_HD static void dequant64(const uint32_t* r, int s, uint32_t* out, const uint32_t* = nullptr) {
        const uint32_t d_dmin = r[0];   // (d, dmin) as an fp16 pair
#pragma unroll
        for (int bi = 0; bi < 2; bi++) {
            const int j = 2 * s + bi;
            const uint32_t sj = byte_at(r, 4 + j);
            uint32_t sc = sj & 63u, mn;
            if (j < 4) mn = (byte_at(r, 4 + j + 8) & 15u) | ((sj >> 6) << 4);
            else       mn = (byte_at(r, 4 + j + 4) >> 4) | ((sj >> 6) << 4);
            // (sc, mn) as exact fp16.  q*sc <= 945 is exact in fp16, so w = fma(q*sc, d, -m_sub) rounds the
            // product once (tighter than the reference's fp16 d*sc, which rounds the sub-scale first);
            // m_sub = dmin*mn is rounded once as in the reference.
            const uint32_t scm = h2sub((sc | (mn << 16)) | H2_1024, H2_1024);
            const uint32_t sc2 = prmt(scm, 0u, 0x1010u);
            const uint32_t negm2 = prmt(h2mul(scm, d_dmin), 0u, 0x3232u) ^ 0x80008000u;
            const uint32_t d2 = prmt(d_dmin, 0u, 0x1010u);
#pragma unroll
            for (int p = 0; p < 8; p++) {
                uint32_t lo, hi;
                nib_pairs(spread_pair(r, 16 + 16 * j + 2 * p), lo, hi);
                out[16 * bi + p] = h2fma(h2mul(h2sub(lo, H2_1024), sc2), d2, negm2);
                out[16 * bi + 8 + p] = h2fma(h2mul(h2sub(hi, H2_64), sc2), d2, negm2);
            }
        }
    }
};

// ---- ternary, 12 B / 32 (gold cpu_gold_reference.h:176-189: value = (code-1)*d, code 3 -> +2d) --
template <> struct Codec<QUANT_TERNARY_1_58> : CodecDefaults {
    static constexpr int ROW_BYTES = 96;
    static constexpr int GROUPS = 3;      // unpack warp groups per matrix in the projection kernel
    CDC_HD static constexpr int sub_lo(int s) { return 6 * s; }
    CDC_HD static constexpr int sub_hi(int s) { return 6 * s + 6; }
    CDC_HD static void dequant64(const uint32_t* r, int s, uint32_t* out, const uint32_t* = nullptr) {
#pragma unroll
        for (int bi = 0; bi < 2; bi++) {
            const int w = 3 * (2 * s + bi);
            const uint32_t d2 = prmt(r[w], 0u, 0x1010u);
#pragma unroll
            for (int u = 0; u < 2; u++) {
                const uint32_t q = r[w + 1 + u];
#pragma unroll
                for (int i = 0; i < 8; i++) {
                    uint32_t t = q >> (4 * i);
                    uint32_t x = (t & 3u) | ((t << 14) & 0x30000u) | H2_1024;
                    out[16 * bi + 8 * u + i] = h2mul(h2sub(x, H2_1025), d2);
                }
            }
        }
    }
};

// ---- EXL3-style codebook, 144 B / 256 (quant_router_kernels.metal:368-411; gold :342-389) ---------
template <> struct Codec<QUANT_EXL3> : CodecDefaults {
    static constexpr int ROW_BYTES = 144;
    static constexpr int GROUPS = 3;      // unpack warp groups per matrix in the projection kernel
    static constexpr int HDR_WORDS = 9;   // d, bias, sub-scales, residual scales, two 8-entry codebooks
    CDC_HD static constexpr int sub_lo(int s) { return 12 + 6 * s; }
    CDC_HD static constexpr int sub_hi(int s) { return 18 + 6 * s; }
    CDC_HD static void dequant64(const uint32_t* r, int s, uint32_t* out, const uint32_t* = nullptr) {
        const float d = h_lo_to_float(r[0]), bias = h_hi_to_float(r[0]);
#pragma unroll
        for (int bi = 0; bi < 2; bi++) {
            const int j = 2 * s + bi;
            const float sub_scale = d * (float)byte_at(r, 4 + j) * 0.015625f;
            const float sub_res = d * ((float)byte_at(r, 12 + j) - 128.0f) * 0.0078125f;
            uint32_t L[4];
#pragma unroll
            for (int e = 0; e < 4; e++) {
                float c0 = (float)(int8_t)byte_at(r, 20 + 2 * e), r0 = (float)(int8_t)byte_at(r, 28 + 2 * e);
                float c1 = (float)(int8_t)byte_at(r, 21 + 2 * e), r1 = (float)(int8_t)byte_at(r, 29 + 2 * e);
                L[e] = float_to_h(bias + sub_scale * c0 + sub_res * r0) |
                       (float_to_h(bias + sub_scale * c1 + sub_res * r1) << 16);
            }
            const int w = 12 + 3 * j;
            const uint32_t w0 = r[w], w1 = r[w + 1], w2 = r[w + 2];
            const uint32_t v[4] = {w0 & 0xFFFFFFu, ((w0 >> 24) | (w1 << 8)) & 0xFFFFFFu,
                                   ((w1 >> 16) | (w2 << 16)) & 0xFFFFFFu, w2 >> 8};
            // The eight table entries as two byte tables (low bytes, high bytes): one byte permute then looks up four
            // 3-bit codes at once (its selector nibbles are the codes), two more interleave the bytes back into fp16 pairs.
            const uint32_t lo_a = prmt(L[0], L[1], 0x6420u), lo_b = prmt(L[2], L[3], 0x6420u);
            const uint32_t hi_a = prmt(L[0], L[1], 0x7531u), hi_b = prmt(L[2], L[3], 0x7531u);
#pragma unroll
            for (int g = 0; g < 4; g++) {
                // eight 3-bit codes -> eight nibbles: 12-bit halves apart, then 6-bit pairs, then single codes
                uint32_t x = (v[g] & 0xFFFu) | ((v[g] & 0xFFF000u) << 4);
                x = (x & 0x003F003Fu) | ((x & 0x0FC00FC0u) << 2);
                x = (x & 0x07070707u) | ((x & 0x38383838u) << 1);
#pragma unroll
                for (int h = 0; h < 2; h++) {
                    const uint32_t sel = h ? (x >> 16) : x;           // codes 4h .. 4h + 3
                    const uint32_t lo4 = prmt(lo_a, lo_b, sel), hi4 = prmt(hi_a, hi_b, sel);
                    out[16 * bi + 4 * g + 2 * h] = prmt(lo4, hi4, 0x5140u);
                    out[16 * bi + 4 * g + 2 * h + 1] = prmt(lo4, hi4, 0x7362u);
                }
            }
        }
    }
};

// ---- variable-rate affine, 160 B / 256 (quant_router_kernels.metal:265-365; gold :214-311) ---------
template <> struct Codec<QUANT_VAR_RATE_AFFINE> : CodecDefaults {
    static constexpr int ROW_BYTES = 160;
    static constexpr int GROUPS = 3;      // unpack warp groups per matrix in the projection kernel (fits 96 registers without spilling: 111-120 us against 134-140 us with two)
    static constexpr int HDR_WORDS = 7;   // d, bias, sub-scales, sub-biases, mode bytes
    // payload runs start at bytes 32 + {0,12,24,40,56,72,88,108}; any run may be read as five words
    CDC_HD static constexpr int sub_lo(int s) { return s == 0 ? 8 : (s == 1 ? 14 : (s == 2 ? 22 : 30)); }
    CDC_HD static constexpr int sub_hi(int s) { return s == 0 ? 16 : (s == 1 ? 23 : (s == 2 ? 31 : 40)); }
    CDC_HD static void dequant64(const uint32_t* r, int s, uint32_t* out, const uint32_t* = nullptr) {
        const float d = h_lo_to_float(r[0]), bias = h_hi_to_float(r[0]);
#pragma unroll
        for (int bi = 0; bi < 2; bi++) {
            const int j = 2 * s + bi;
            const int offs[8] = {0, 12, 24, 40, 56, 72, 88, 108};
            const int w = 8 + offs[j] / 4;
            const uint32_t sc2 = dup16(float_to_h(d * (float)byte_at(r, 4 + j) * 0.0625f));
            const uint32_t bs2 = dup16(float_to_h(bias + d * ((float)byte_at(r, 12 + j) - 128.0f) * 0.0625f));
            const uint32_t mode = byte_at(r, 20 + j);
            const uint32_t bits = mode & 7u, perm = (mode >> 3) & 3u;
            uint32_t pk[16];   // source-order pairs (2i, 2i+1)
            if (bits == 3u) {
                const uint32_t w0 = r[w], w1 = r[w + 1], w2 = r[w + 2];
                const uint32_t v[4] = {w0 & 0xFFFFFFu, ((w0 >> 24) | (w1 << 8)) & 0xFFFFFFu,
                                       ((w1 >> 16) | (w2 << 16)) & 0xFFFFFFu, w2 >> 8};
#pragma unroll
                for (int g = 0; g < 4; g++)
#pragma unroll
                    for (int i = 0; i < 4; i++) {
                        uint32_t t = v[g] >> (6 * i);
                        uint32_t x = (t & 7u) | ((t << 13) & 0x70000u) | H2_1024;
                        pk[4 * g + i] = h2fma(h2sub(x, 0x64046404u), sc2, bs2);      // q - 4
                    }
            } else if (bits == 5u) {
#pragma unroll
                for (int g = 0; g < 4; g++) {
                    // 40-bit group g starts at bit 40g of the 20-byte run = bit 8g of word g
                    const uint32_t a = r[w + g], b = r[w + g + 1];
                    const uint64_t v = (g == 0) ? ((uint64_t)a | ((uint64_t)(b & 0xFFu) << 32))
                                                : (((((uint64_t)b << 32) | a) >> (8 * g)) & 0xFFFFFFFFFFull);
#pragma unroll
                    for (int i = 0; i < 4; i++) {
                        uint32_t t = (uint32_t)(v >> (10 * i));
                        uint32_t x = (t & 31u) | ((t << 11) & 0x1F0000u) | H2_1024;
                        pk[4 * g + i] = h2fma(h2sub(x, 0x64106410u), sc2, bs2);      // q - 16
                    }
                }
            } else {
#pragma unroll
                for (int p = 0; p < 8; p++) {
                    uint32_t lo, hi;
                    nib_pairs(spread_pair(r, 4 * w + 2 * p), lo, hi);
                    pk[p] = h2fma(h2sub(lo, H2_1032), sc2, bs2);
                    pk[8 + p] = h2fma(h2sub(hi, H2_72), sc2, bs2);
                }
            }
            // destination permutation: 0 identity; 1 even sources first, then odd; 2 reversed.  Branches, not selects: the
            // rows of a warp usually share the mode byte, and even when they do not, the three arms together cost less than
            // computing all three results for every output.
            if (perm == 1u) {
#pragma unroll
                for (int i = 0; i < 8; i++) {
                    out[16 * bi + i] = prmt(pk[2 * i], pk[2 * i + 1], 0x5410u);
                    out[16 * bi + 8 + i] = prmt(pk[2 * i], pk[2 * i + 1], 0x7632u);
                }
            } else if (perm == 2u) {
#pragma unroll
                for (int i = 0; i < 16; i++) out[16 * bi + i] = prmt(pk[15 - i], 0u, 0x1032u);
            } else {
#pragma unroll
                for (int i = 0; i < 16; i++) out[16 * bi + i] = pk[i];
            }
        }
    }
};

// ---- MLX 4-bit, group 64, sequential nibbles, planar (extension layout 100) --------------------------
// Packed row: u32 words of 8 nibbles, nibble t of word i is k = 8i + t; 128 bytes per 256 elements.  Per 64
// elements one fp16 scale and one fp16 bias in two planes behind the nibble plane; meta[0..1] hold the four
// scales of the chunk, meta[2..3] the four biases.  w = q*s + b, one fused fp16 multiply-add.
template <> struct Codec<QUANT_MLX_4BIT_G64> : CodecDefaults {
    static constexpr int ROW_BYTES = 128;
    static constexpr int GROUPS = 3;
    CDC_HD static constexpr int sub_lo(int s) { return 8 * s; }
    CDC_HD static constexpr int sub_hi(int s) { return 8 * s + 8; }
    static constexpr int META_WORDS = 4;
    static constexpr bool RAW_SWIZZLE_128 = true;
    CDC_HD static void dequant64(const uint32_t* r, int s, uint32_t* out, const uint32_t* meta) {
        const uint32_t d2 = bcast16(meta, 2 * s), b2 = bcast16(meta + 2, 2 * s);
#pragma unroll
        for (int i = 0; i < 8; i++) {
            const uint32_t w = r[8 * s + i], w8 = w >> 8;
            // nibble pairs (n0,n4) (n1,n5) (n2,n6) (n3,n7) as (1024+n) or (64+n) halves, then back to k order
            const uint32_t a04 = h2fma(h2sub((w & 0x000F000Fu) | H2_1024, H2_1024), d2, b2);
            const uint32_t a15 = h2fma(h2sub((w & 0x00F000F0u) | H2_64, H2_64), d2, b2);
            const uint32_t a26 = h2fma(h2sub((w8 & 0x000F000Fu) | H2_1024, H2_1024), d2, b2);
            const uint32_t a37 = h2fma(h2sub((w8 & 0x00F000F0u) | H2_64, H2_64), d2, b2);
            out[4 * i + 0] = prmt(a04, a15, 0x5410u);
            out[4 * i + 1] = prmt(a26, a37, 0x5410u);
            out[4 * i + 2] = prmt(a04, a15, 0x7632u);
            out[4 * i + 3] = prmt(a26, a37, 0x7632u);
        }
    }
};

// ---- MLX 4-bit, group 32, planar (unified_multi_scale_kernels.metal:17-79; layout id 102) ----------------
// The reference's layer benchmarks keep MLX weights as three planes: 16 nibble bytes per block of 32 (byte j: low
// nibble = element j, high nibble = element j + 16, as in the 20-byte block), then one fp16 scale per block, then
// one fp16 bias per block.  Packed row: 128 bytes per 256 elements; meta[0..3] hold the chunk's eight scales,
// meta[4..7] its eight biases.  w = q*s + b, one fused fp16 multiply-add.
template <> struct Codec<QUANT_MLX_4BIT_PLANAR> : CodecDefaults {
    static constexpr int ROW_BYTES = 128;
    static constexpr int GROUPS = 3;
    CDC_HD static constexpr int sub_lo(int s) { return 8 * s; }
    CDC_HD static constexpr int sub_hi(int s) { return 8 * s + 8; }
    static constexpr int META_WORDS = 8;
    static constexpr bool RAW_SWIZZLE_128 = true;
    CDC_HD static void dequant64(const uint32_t* r, int s, uint32_t* out, const uint32_t* meta) {
#pragma unroll
        for (int bi = 0; bi < 2; bi++) {
            const int b = 2 * s + bi;
            const uint32_t d2 = bcast16(meta, 2 * b), b2 = bcast16(meta + 4, 2 * b);
#pragma unroll
            for (int p = 0; p < 8; p++) {
                uint32_t lo, hi;
                nib_pairs(spread_pair(r, 16 * b + 2 * p), lo, hi);
                out[16 * bi + p] = h2fma(h2sub(lo, H2_1024), d2, b2);
                out[16 * bi + 8 + p] = h2fma(h2sub(hi, H2_64), d2, b2);
            }
        }
    }
};

// ---- ternary with one scale per output row, planar (extension layout 101) -------------------------------
// Packed row: u32 words of 16 two-bit codes, code t of word i is k = 16i + t; 64 bytes per 256 elements.  The
// weights go to the tensor core as the exact integers code - 1; the row's fp16 scale multiplies the fp32
// accumulator in the epilogue, so the result is rounded once.
template <> struct Codec<QUANT_TERNARY_ROW> : CodecDefaults {
    static constexpr int ROW_BYTES = 64;
    static constexpr int GROUPS = 3;
    CDC_HD static constexpr int sub_lo(int s) { return 4 * s; }
    CDC_HD static constexpr int sub_hi(int s) { return 4 * s + 4; }
    static constexpr bool ROW_SCALE = true;
    CDC_HD static void dequant64(const uint32_t* r, int s, uint32_t* out, const uint32_t* = nullptr) {
#pragma unroll
        for (int wi = 0; wi < 4; wi++) {
            const uint32_t q = r[4 * s + wi];
#pragma unroll
            for (int i = 0; i < 8; i++) {
                const uint32_t t = q >> (4 * i);
                const uint32_t x = (t & 3u) | ((t << 14) & 0x30000u) | H2_1024;
                out[8 * wi + i] = h2sub(x, H2_1025);
            }
        }
    }
};

// ---- Prism Q2_0, 34 B / 128 (quant_router_kernels.metal:414-436; gold cpu_gold_reference.h:402-440) ------------
// Block = fp16 d + 32 bytes of 2-bit codes, element 4b+j = (qs[b] >> 2j) & 3, value = (code - 1) * d (code 3 gives
// +2d, as in the reference on both its paths).  34-byte blocks make a row a 16-byte multiple only every 8 blocks,
// so the packed stage of this format is 1024 elements = 272 bytes and holds 16 sub-tiles.  Sub-tile s lies in block
// b = s / 2: its 16 code bytes start at byte 34b + 2 + 16 (s % 2), which is 2 (mod 4) for even b: those are read as
// five words and shifted by 16 bits.  (code - 1) * d is exact in fp16, so the weights carry no rounding at all.
template <> struct Codec<QUANT_PRISM_Q2_0> : CodecDefaults {
    static constexpr int CHUNK = 1024;
    static constexpr int ROW_BYTES = 272;
    static constexpr int TMA_ELEM_BYTES = 2;   // 272 bytes per box row exceed 256 one-byte elements: the map counts 16-bit words
    static constexpr int GROUPS = 3;
    CDC_HD static constexpr int d_byte(int s) { return 34 * (s / 2); }
    CDC_HD static constexpr int code_byte(int s) { return 34 * (s / 2) + 2 + 16 * (s % 2); }
    CDC_HD static constexpr int sub_lo(int s) { return d_byte(s) / 4; }
    CDC_HD static constexpr int sub_hi(int s) { return (code_byte(s) + 16 + 3) / 4; }
    CDC_HD static void dequant64(const uint32_t* r, int s, uint32_t* out, const uint32_t* = nullptr) {
        const uint32_t d2 = bcast16(r, d_byte(s));
        const int c0 = code_byte(s), w0 = c0 / 4;
#pragma unroll
        for (int wi = 0; wi < 4; wi++) {
            // 16 codes of elements 16wi .. 16wi+15 of the sub-tile
            const uint32_t q = (c0 & 2) ? prmt(r[w0 + wi], r[w0 + wi + 1], 0x5432u) : r[w0 + wi];
#pragma unroll
            for (int i = 0; i < 8; i++) {
                const uint32_t t = q >> (4 * i);
                const uint32_t x = (t & 3u) | ((t << 14) & 0x30000u) | H2_1024;
                out[8 * wi + i] = h2mul(h2sub(x, H2_1025), d2);
            }
        }
    }
};

}  // namespace cdc
