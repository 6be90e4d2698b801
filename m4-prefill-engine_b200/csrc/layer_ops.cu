// RMSNorm, rotary embedding and the fp32 residual add used by the decoder layer.
//
// The reference has these only in its Python block (src/engine/model.py:39-45 RMSNorm in its own
// code; :112-116 rotary embedding through a third-party array library, non-interleaved form), so
// the CPU oracle for them is a restatement (oracle/oracle.cpp: orc_rmsnorm, orc_rope).
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <mutex>

#include "../../include/b200_bridge.h"
#include "bridge_state.cuh"
#include "layer_ops.cuh"

namespace lops {

// one CTA of 256 threads per row; each thread walks 8-element vectors
__global__ void __launch_bounds__(256) rmsnorm_kernel(const __half* __restrict__ X, const __half* __restrict__ W,
                                                      __half* __restrict__ Y, uint32_t K, float eps) {
    const __half* x = X + (size_t)blockIdx.x * K;
    __half* y = Y + (size_t)blockIdx.x * K;
    float ss = 0.0f;
    const bool vec = (K % 8 == 0) && ((((uintptr_t)x | (uintptr_t)y | (uintptr_t)W) & 15u) == 0);
    if (vec) {
        for (uint32_t i = threadIdx.x; i < K / 8; i += blockDim.x) {
            uint4 v = reinterpret_cast<const uint4*>(x)[i];
            const __half2* h = reinterpret_cast<const __half2*>(&v);
#pragma unroll
            for (int j = 0; j < 4; j++) { float2 f = __half22float2(h[j]); ss += f.x * f.x + f.y * f.y; }
        }
    } else {
        for (uint32_t i = threadIdx.x; i < K; i += blockDim.x) { float f = __half2float(x[i]); ss += f * f; }
    }
    __shared__ float red[8];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    float tot = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; i++) tot += red[i];
    const float r = 1.0f / sqrtf(tot / (float)K + eps);
    if (vec) {
        for (uint32_t i = threadIdx.x; i < K / 8; i += blockDim.x) {
            uint4 v = reinterpret_cast<const uint4*>(x)[i], w = reinterpret_cast<const uint4*>(W)[i], o;
            const __half2* h = reinterpret_cast<const __half2*>(&v);
            const __half2* wh = reinterpret_cast<const __half2*>(&w);
            __half2* oh = reinterpret_cast<__half2*>(&o);
#pragma unroll
            for (int j = 0; j < 4; j++) {
                float2 f = __half22float2(h[j]), g = __half22float2(wh[j]);
                __half2 n = __floats2half2_rn(f.x * r, f.y * r);          // rounded to fp16 first, as the reference does
                float2 nf = __half22float2(n);
                oh[j] = __floats2half2_rn(nf.x * g.x, nf.y * g.y);
            }
            reinterpret_cast<uint4*>(y)[i] = o;
        }
    } else {
        for (uint32_t i = threadIdx.x; i < K; i += blockDim.x) {
            __half n = __float2half_rn(__half2float(x[i]) * r);
            y[i] = __float2half_rn(__half2float(n) * __half2float(W[i]));
        }
    }
}

__global__ void rope_kernel(__half* __restrict__ X, uint32_t M, uint32_t D, float log2_theta, uint32_t pos0, size_t total_pairs) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total_pairs) return;
    const uint32_t half = D / 2;
    const uint32_t j = (uint32_t)(i % half);
    const size_t row = i / half;                 // h*M + m
    const uint32_t m = (uint32_t)(row % M);
    const float inv_freq = exp2f(-2.0f * (float)j / (float)D * log2_theta);
    const float ang = (float)(pos0 + m) * inv_freq;
    float s, c;
    sincosf(ang, &s, &c);
    __half* x = X + row * D;
    const float a = __half2float(x[j]), b = __half2float(x[j + half]);
    x[j] = __float2half_rn(__fmaf_rn(a, c, -__fmul_rn(b, s)));
    x[j + half] = __float2half_rn(__fmaf_rn(b, c, __fmul_rn(a, s)));
}

// (cos, sin) of every (position, frequency) of a launch, for the projection epilogue that applies the rotation itself:
// table[m][j] = sincos((pos0 + m) * theta^(-2j/D)), the very expression of the kernels above, so a fused rotation and a
// separate one agree bit for bit.
__global__ void rope_table_kernel(float2* __restrict__ table, uint32_t M, uint32_t D, float log2_theta, uint32_t pos0) {
    const uint32_t half = D / 2;
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (size_t)M * half) return;
    const uint32_t m = (uint32_t)(i / half), j = (uint32_t)(i % half);
    float s, c;
    sincosf((float)(pos0 + m) * exp2f(-2.0f * (float)j / (float)D * log2_theta), &s, &c);
    table[i] = make_float2(c, s);
}

// Rotate-half RoPE for D % 4 == 0: one thread owns two adjacent frequencies of one token and walks all heads, so
// the sine and cosine (the expensive part) are computed once per token and frequency instead of once per head, and
// every access is a 4-byte pair.  Element arithmetic is that of rope_kernel.
__global__ void rope_heads_kernel(__half* __restrict__ X, uint32_t H, uint32_t M, uint32_t D, float log2_theta, uint32_t pos0) {
    const uint32_t half = D / 2, per_tok = half / 2;
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (size_t)M * per_tok) return;
    const uint32_t m = (uint32_t)(i / per_tok), j = 2u * (uint32_t)(i % per_tok);
    float s0, c0, s1, c1;
    sincosf((float)(pos0 + m) * exp2f(-2.0f * (float)j / (float)D * log2_theta), &s0, &c0);
    sincosf((float)(pos0 + m) * exp2f(-2.0f * (float)(j + 1) / (float)D * log2_theta), &s1, &c1);
    __half* x = X + (size_t)m * D + j;
    const size_t head_stride = (size_t)M * D;
    // heads in batches of four: all loads of a batch are issued before its first store (the stores would
    // otherwise order every later load behind them, one memory round trip per head)
    for (uint32_t h0 = 0; h0 < H; h0 += 4, x += 4 * head_stride) {
        __half2 lo[4], hi[4];
#pragma unroll
        for (int u = 0; u < 4; u++)
            if (h0 + u < H) {
                lo[u] = *reinterpret_cast<const __half2*>(x + u * head_stride);
                hi[u] = *reinterpret_cast<const __half2*>(x + u * head_stride + half);
            }
#pragma unroll
        for (int u = 0; u < 4; u++)
            if (h0 + u < H) {
                const float a0 = __low2float(lo[u]), a1 = __high2float(lo[u]), b0 = __low2float(hi[u]), b1 = __high2float(hi[u]);
                // (multiply-adds spelled out so that every kernel that rotates rounds alike)
                *reinterpret_cast<__half2*>(x + u * head_stride) =
                    __halves2half2(__float2half_rn(__fmaf_rn(a0, c0, -__fmul_rn(b0, s0))), __float2half_rn(__fmaf_rn(a1, c1, -__fmul_rn(b1, s1))));
                *reinterpret_cast<__half2*>(x + u * head_stride + half) =
                    __halves2half2(__float2half_rn(__fmaf_rn(b0, c0, __fmul_rn(a0, s0))), __float2half_rn(__fmaf_rn(b1, c1, __fmul_rn(a1, s1))));
            }
    }
}

__global__ void add_residual_f32_kernel(const __half* __restrict__ A, const float* __restrict__ B, __half* __restrict__ Y, size_t n) {
    const size_t i = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * 4;
    if (i + 3 < n) {
        const float4 b = *reinterpret_cast<const float4*>(B + i);
        const __half2 a0 = *reinterpret_cast<const __half2*>(A + i), a1 = *reinterpret_cast<const __half2*>(A + i + 2);
        *reinterpret_cast<__half2*>(Y + i) = __floats2half2_rn(__low2float(a0) + b.x, __high2float(a0) + b.y);
        *reinterpret_cast<__half2*>(Y + i + 2) = __floats2half2_rn(__low2float(a1) + b.z, __high2float(a1) + b.w);
    } else {
        for (size_t k = i; k < n; k++) Y[k] = __float2half_rn(__half2float(A[k]) + B[k]);
    }
}

// Y = fp16(A + B), eight elements per thread (16-byte accesses; the launcher checks alignment and n % 8)
__global__ void add_residual_f16_kernel(const __half* __restrict__ A, const __half* __restrict__ B, __half* __restrict__ Y, size_t n8) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n8) return;
    const uint4 a = reinterpret_cast<const uint4*>(A)[i], b = reinterpret_cast<const uint4*>(B)[i];
    uint4 o;
    const __half2* ah = reinterpret_cast<const __half2*>(&a);
    const __half2* bh = reinterpret_cast<const __half2*>(&b);
    __half2* oh = reinterpret_cast<__half2*>(&o);
#pragma unroll
    for (int j = 0; j < 4; j++) {
        const float2 fa = __half22float2(ah[j]), fb = __half22float2(bh[j]);
        oh[j] = __floats2half2_rn(fa.x + fb.x, fa.y + fb.y);
    }
    reinterpret_cast<uint4*>(Y)[i] = o;
}

// Residual add fused into the normalisation that follows it: S = fp16(A + B) (the block's output, kept for the next
// residual), Y = rmsnorm(S) * W.  One CTA of 256 threads per row; a thread reads back only the vectors it wrote itself,
// and the barrier of the row reduction separates every read of A from the first write of Y, so Y may alias A.
// Rows must be 16-byte aligned with K a multiple of 8 (checked by the launcher).
__global__ void __launch_bounds__(256) rmsnorm_add_kernel(const __half* A, const __half* __restrict__ B,
                                                          const __half* __restrict__ W, __half* __restrict__ S, __half* Y,
                                                          uint32_t K, float eps) {
    const size_t row = (size_t)blockIdx.x * K;
    float ss = 0.0f;
    for (uint32_t i = threadIdx.x; i < K / 8; i += blockDim.x) {
        const uint4 a = reinterpret_cast<const uint4*>(A + row)[i], b = reinterpret_cast<const uint4*>(B + row)[i];
        uint4 o;
        const __half2* ah = reinterpret_cast<const __half2*>(&a);
        const __half2* bh = reinterpret_cast<const __half2*>(&b);
        __half2* oh = reinterpret_cast<__half2*>(&o);
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const float2 fa = __half22float2(ah[j]), fb = __half22float2(bh[j]);
            oh[j] = __floats2half2_rn(fa.x + fb.x, fa.y + fb.y);
            const float2 f = __half22float2(oh[j]);
            ss += f.x * f.x + f.y * f.y;
        }
        reinterpret_cast<uint4*>(S + row)[i] = o;
    }
    __shared__ float red[8];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    float tot = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; i++) tot += red[i];
    const float r = 1.0f / sqrtf(tot / (float)K + eps);
    for (uint32_t i = threadIdx.x; i < K / 8; i += blockDim.x) {
        const uint4 v = reinterpret_cast<const uint4*>(S + row)[i], w = reinterpret_cast<const uint4*>(W)[i];
        uint4 o;
        const __half2* h = reinterpret_cast<const __half2*>(&v);
        const __half2* wh = reinterpret_cast<const __half2*>(&w);
        __half2* oh = reinterpret_cast<__half2*>(&o);
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const float2 f = __half22float2(h[j]), g = __half22float2(wh[j]);
            const __half2 n = __floats2half2_rn(f.x * r, f.y * r);            // rounded to fp16 first, as in rmsnorm_kernel
            const float2 nf = __half22float2(n);
            oh[j] = __floats2half2_rn(nf.x * g.x, nf.y * g.y);
        }
        reinterpret_cast<uint4*>(Y + row)[i] = o;
    }
}

cudaError_t rmsnorm(const void* X, const void* weight, void* Y, uint32_t M, uint32_t K, float eps, cudaStream_t s) {
    rmsnorm_kernel<<<M, 256, 0, s>>>((const __half*)X, (const __half*)weight, (__half*)Y, K, eps);
    return cudaGetLastError();
}
cudaError_t rmsnorm_add(const void* A, const void* B, const void* weight, void* S, void* Y, uint32_t M, uint32_t K, float eps,
                        cudaStream_t s) {
    if (K % 8 != 0 || ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B) | reinterpret_cast<uintptr_t>(weight) |
                        reinterpret_cast<uintptr_t>(S) | reinterpret_cast<uintptr_t>(Y)) & 15u))
        return cudaErrorInvalidValue;
    rmsnorm_add_kernel<<<M, 256, 0, s>>>((const __half*)A, (const __half*)B, (const __half*)weight, (__half*)S, (__half*)Y, K, eps);
    return cudaGetLastError();
}
cudaError_t rope(void* X, uint32_t H, uint32_t M, uint32_t D, float theta, uint32_t pos0, cudaStream_t s) {
    if (D % 4 == 0 && (reinterpret_cast<uintptr_t>(X) & 3u) == 0) {
        const size_t threads = (size_t)M * (D / 4);
        rope_heads_kernel<<<(unsigned)((threads + 127) / 128), 128, 0, s>>>((__half*)X, H, M, D, log2f(theta), pos0);
        return cudaGetLastError();
    }
    const size_t pairs = (size_t)H * M * (D / 2);
    rope_kernel<<<(unsigned)((pairs + 255) / 256), 256, 0, s>>>((__half*)X, M, D, log2f(theta), pos0, pairs);
    return cudaGetLastError();
}
// Everything between the Q/K/V projections and attention in one pass: rotary embedding on Q and K (in place for Q),
// K and V compressed to Q8_0 records.  One warp per token walks that token's rows of all heads: a row of D = 128 fp16 is
// 8 bytes per lane, the rotation partner (i +- D/2) sits 16 lanes away, the 32 values of a Q8_0 record are those of 8
// neighbouring lanes, and the token's (cos, sin) values are read from the table once and reused for every head.
// Arithmetic is that of rope_heads_kernel and of attn::quantize_q8_0_kernel, bit for bit.
__global__ void __launch_bounds__(128) kv_post_d128_kernel(__half* __restrict__ Q, const __half* __restrict__ Kin, const __half* __restrict__ Vin,
                                                           uint8_t* __restrict__ Kq, uint8_t* __restrict__ Vq, __half* __restrict__ Kout,
                                                           __half* __restrict__ Vout, const float2* __restrict__ table, uint32_t Hq, uint32_t Hkv,
                                                           uint32_t M, int rope, int q8, int dq) {
    constexpr uint32_t D = 128, HALF = 64;
    const uint32_t m = blockIdx.x * 4u + (threadIdx.x >> 5), lane = threadIdx.x & 31u;
    if (m >= M) return;
    const bool upper = lane >= 16u;
    float2 cs[4];
    if (rope) {
        const float4* t4 = reinterpret_cast<const float4*>(table + (size_t)m * HALF + (lane & 15u) * 4u);
        const float4 a = __ldg(t4), b = __ldg(t4 + 1);
        cs[0] = make_float2(a.x, a.y); cs[1] = make_float2(a.z, a.w); cs[2] = make_float2(b.x, b.y); cs[3] = make_float2(b.z, b.w);
    }
    auto rotate = [&](uint2 w) {
        uint2 pw;
        pw.x = __shfl_xor_sync(0xffffffffu, w.x, 16); pw.y = __shfl_xor_sync(0xffffffffu, w.y, 16);
        const float2 x01 = __half22float2(*reinterpret_cast<const __half2*>(&w.x)), x23 = __half22float2(*reinterpret_cast<const __half2*>(&w.y));
        const float2 y01 = __half22float2(*reinterpret_cast<const __half2*>(&pw.x)), y23 = __half22float2(*reinterpret_cast<const __half2*>(&pw.y));
        const float x[4] = {x01.x, x01.y, x23.x, x23.y}, y[4] = {y01.x, y01.y, y23.x, y23.y};
        float r[4];
#pragma unroll
        for (int e = 0; e < 4; e++)      // lower half: a*c - b*s with (a, b) = (x, y); upper half: b*c + a*s with (a, b) = (y, x)
            r[e] = upper ? __fmaf_rn(x[e], cs[e].x, __fmul_rn(y[e], cs[e].y)) : __fmaf_rn(x[e], cs[e].x, -__fmul_rn(y[e], cs[e].y));
        const __half2 h01 = __floats2half2_rn(r[0], r[1]), h23 = __floats2half2_rn(r[2], r[3]);
        uint2 o;
        o.x = *reinterpret_cast<const uint32_t*>(&h01); o.y = *reinterpret_cast<const uint32_t*>(&h23);
        return o;
    };
    // rec_row: the four records of this (head, token) row; dq_row (optional): the row's values as the cache will give them
    // back, fp16(q * fp16(d)) -- what attention over the Q8_0 cache multiplies with
    auto quantise = [&](uint2 w, uint8_t* rec_row, __half* dq_row) {
        const float2 f01 = __half22float2(*reinterpret_cast<const __half2*>(&w.x)), f23 = __half22float2(*reinterpret_cast<const __half2*>(&w.y));
        const float v[4] = {f01.x, f01.y, f23.x, f23.y};
        float amax = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 4));
        const float d = __fdiv_rn(amax, 127.0f);
        const float id = d > 0.0f ? __fdiv_rn(1.0f, d) : 0.0f;
        uint16_t* o = reinterpret_cast<uint16_t*>(rec_row + (lane >> 3) * 34u);
        const __half dh = __float2half_rn(d);
        if ((lane & 7u) == 0u) o[0] = __half_as_ushort(dh);
        uint32_t back[2];
#pragma unroll
        for (int e = 0; e < 2; e++) {
            int q0 = (int)roundf(__fmul_rn(v[2 * e], id)), q1 = (int)roundf(__fmul_rn(v[2 * e + 1], id));
            q0 = max(-128, min(127, q0)); q1 = max(-128, min(127, q1));
            o[1 + (lane & 7u) * 2u + e] = (uint16_t)((uint32_t)(uint8_t)(int8_t)q0 | ((uint32_t)(uint8_t)(int8_t)q1 << 8));
            back[e] = (uint32_t)__half_as_ushort(__hmul(__int2half_rn(q0), dh)) | ((uint32_t)__half_as_ushort(__hmul(__int2half_rn(q1), dh)) << 16);
        }
        if (dq_row) *reinterpret_cast<uint2*>(dq_row + lane * 4u) = make_uint2(back[0], back[1]);
    };
    if (rope) {
        // heads in batches of four: the loads of a batch are issued before its first store
        for (uint32_t h0 = 0; h0 < Hq; h0 += 4) {
            uint2 w[4];
#pragma unroll
            for (int u = 0; u < 4; u++)
                if (h0 + u < Hq) w[u] = *reinterpret_cast<const uint2*>(Q + ((size_t)(h0 + u) * M + m) * D + lane * 4u);
#pragma unroll
            for (int u = 0; u < 4; u++)
                if (h0 + u < Hq) *reinterpret_cast<uint2*>(Q + ((size_t)(h0 + u) * M + m) * D + lane * 4u) = rotate(w[u]);
        }
    }
    for (uint32_t h = 0; h < Hkv; h++) {
        const size_t row = ((size_t)h * M + m);
        uint2 k = *reinterpret_cast<const uint2*>(Kin + row * D + lane * 4u);
        const uint2 v = *reinterpret_cast<const uint2*>(Vin + row * D + lane * 4u);
        if (rope) k = rotate(k);
        if (q8) {
            quantise(k, Kq + row * (D / 32u) * 34u, dq ? Kout + row * D : nullptr);
            quantise(v, Vq + row * (D / 32u) * 34u, dq ? Vout + row * D : nullptr);
        } else if (rope) {
            *reinterpret_cast<uint2*>(Kout + row * D + lane * 4u) = k;
        }
    }
}

cudaError_t kv_post(void* Q, void* K, void* V, void* Kq, void* Vq, const void* rope_table, uint32_t Hq, uint32_t Hkv,
                    uint32_t M, uint32_t D, bool rope, bool q8, bool dequant_in_place, cudaStream_t s) {
    if (D != 128 || (rope && !rope_table) || (q8 && (!Kq || !Vq))) return cudaErrorInvalidValue;
    if (((reinterpret_cast<uintptr_t>(Q) | reinterpret_cast<uintptr_t>(K) | reinterpret_cast<uintptr_t>(V)) & 7u) ||
        (reinterpret_cast<uintptr_t>(rope_table) & 15u))
        return cudaErrorInvalidValue;
    kv_post_d128_kernel<<<(M + 3) / 4, 128, 0, s>>>((__half*)Q, (const __half*)K, (const __half*)V, (uint8_t*)Kq, (uint8_t*)Vq, (__half*)K,
                                                   (__half*)V, (const float2*)rope_table, Hq, Hkv, M, rope ? 1 : 0, q8 ? 1 : 0,
                                                   (q8 && dequant_in_place) ? 1 : 0);
    return cudaGetLastError();
}

cudaError_t build_rope_table(void* table, uint32_t M, uint32_t D, float theta, uint32_t pos0, cudaStream_t s) {
    const size_t n = (size_t)M * (D / 2);
    rope_table_kernel<<<(unsigned)((n + 255) / 256), 256, 0, s>>>((float2*)table, M, D, log2f(theta), pos0);
    return cudaGetLastError();
}
cudaError_t add_residual_f32(const void* A, const float* B, void* Y, size_t n, cudaStream_t s) {
    const size_t threads = (n + 3) / 4;
    add_residual_f32_kernel<<<(unsigned)((threads + 255) / 256), 256, 0, s>>>((const __half*)A, B, (__half*)Y, n);
    return cudaGetLastError();
}

cudaError_t add_residual_f16(const void* A, const void* B, void* Y, size_t n, cudaStream_t s) {
    if (n % 8 != 0 || ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B) | reinterpret_cast<uintptr_t>(Y)) & 15u))
        return cudaErrorInvalidValue;
    const size_t n8 = n / 8;
    add_residual_f16_kernel<<<(unsigned)((n8 + 255) / 256), 256, 0, s>>>((const __half*)A, (const __half*)B, (__half*)Y, n8);
    return cudaGetLastError();
}

}  // namespace lops

using namespace bridge;

extern "C" {

int b200_bridge_rmsnorm(void* X, void* weight, void* Y, uint32_t M, uint32_t K, float eps) {
    std::lock_guard<std::mutex> lock(g.mu);
    if (!g.initialized) return -1;
    if (!X || !weight || !Y) return -2;
    if (M == 0 || K == 0) return -4;
    int rc = 0;
    const size_t bytes = (size_t)M * K * 2;
    const void* x = resolve_in(X, bytes, g.stage_x, false, &rc);
    if (rc) return rc;
    const void* w = resolve_in(weight, (size_t)K * 2, g.stage_aux0, false, &rc);
    if (rc) return rc;
    void* host_dst = nullptr;
    void* y = resolve_out(Y, bytes, g.stage_y, &host_dst, &rc);
    if (rc) return rc;
    if (lops::rmsnorm(x, w, y, M, K, eps, g.stream) != cudaSuccess) return -6;
    g.launches++;
    if (host_dst && copy_back(host_dst, y, bytes) != 0) return -5;
    return 0;
}

/* In-place rotary embedding on X [H][M][D] (device or host pointer). */
int b200_bridge_rope(void* X, uint32_t H, uint32_t M, uint32_t D, float theta, uint32_t pos0) {
    std::lock_guard<std::mutex> lock(g.mu);
    if (!g.initialized) return -1;
    if (!X) return -2;
    if (H == 0 || M == 0 || D == 0 || (D % 2) != 0 || theta <= 0.0f) return -4;
    const size_t bytes = (size_t)H * M * D * 2;
    if (is_device_ptr(X)) {
        if (lops::rope(X, H, M, D, theta, pos0, g.stream) != cudaSuccess) return -6;
        g.launches++;
        return 0;
    }
    int rc = 0;
    void* x = const_cast<void*>(resolve_in(X, bytes, g.stage_x, false, &rc));
    if (rc) return rc;
    if (lops::rope(x, H, M, D, theta, pos0, g.stream) != cudaSuccess) return -6;
    g.launches++;
    return copy_back(X, x, bytes);
}

}  // extern "C"
