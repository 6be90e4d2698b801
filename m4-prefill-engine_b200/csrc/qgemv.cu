// Single-token projection on CUDA cores: the decode-like end of the path (m4_bridge_dispatch_gemv, and
// m4_bridge_dispatch_gemm with M = 1; reference: gemv_q4_0 and friends, quant_router_kernels.metal:930-1144).
// With one token the projection is a stream over the packed weights (9.4 MB at the 8B shape) with a few
// multiply-adds per weight: HBM-bound byte work that gains nothing from the tensor core (its 128-row tiles spend
// 16 dependent unpack-and-MMA steps per CTA on latency).  Here one lane owns one 256-element chunk of one weight
// row: it loads the chunk's packed bytes (the codecs' ROW_BYTES, 16-byte loads), unpacks them with the same
// register-level codecs as the tensor-core kernel (bit-identical fp16 weights), multiplies with the activations kept
// as fp32 in shared memory (chunk stride 257 words: conflict-free) and accumulates in fp32; the lanes of a row are
// reduced with shuffles.  The kernel is written for M tokens (every weight is unpacked once and used M times), but
// measured on B200 it only beats the tensor-core path at M = 1 (8.3 us against 12.6 us at K = N = 4096; 12.6 us at
// M = 2, 16.5 us at M = 3: fp32 multiply-adds on CUDA cores), so only M = 1 is dispatched here.
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdint>

#include "codecs.cuh"
#include "qgemm.cuh"

namespace qg {

namespace {

constexpr int GV_THREADS = 256;
constexpr int GV_MAX_M = 8;
constexpr int XSTRIDE = 257;                 // fp32 words per 256-element activation chunk in shared memory

struct GvParams {
    const __half* X; const uint8_t* W; __half* Y;
    uint32_t M, N, K, chunks;                // chunks = K / 256
    uint32_t rows_per_warp, lanes_per_row;   // chunks < 32: 32 / chunks rows per warp; else 1 row, 32 lanes
    const uint8_t* meta;                     // planar layouts: scale / bias planes behind the packed plane
    const __half* row_scale;                 // per-row scale (integer-valued codecs)
};

template <int FMT, int M>
__global__ void __launch_bounds__(GV_THREADS) qgemv_kernel(const GvParams p) {
    using Cd = cdc::Codec<FMT>;
    constexpr int RB = Cd::ROW_BYTES;
    extern __shared__ float sx[];            // [M][chunks][XSTRIDE]
    const uint32_t tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    for (uint32_t i = tid; i < M * p.K; i += GV_THREADS) {
        const uint32_t m = i / p.K, k = i % p.K;
        sx[(size_t)m * p.chunks * XSTRIDE + (k >> 8) * XSTRIDE + (k & 255u)] = __half2float(p.X[(size_t)m * p.K + k]);
    }
    __syncthreads();
    const uint32_t warps_total = gridDim.x * (GV_THREADS / 32), gw = blockIdx.x * (GV_THREADS / 32) + warp;
    const uint32_t sub = lane / p.lanes_per_row, l = lane % p.lanes_per_row;       // row within the warp's group, lane within the row
    const size_t row_bytes = (size_t)p.chunks * RB;
    for (uint32_t n0 = gw * p.rows_per_warp; n0 < p.N; n0 += warps_total * p.rows_per_warp) {
        const uint32_t n = n0 + sub;
        float acc[M];
#pragma unroll
        for (int m = 0; m < M; m++) acc[m] = 0.0f;
        if (n < p.N) {
            for (uint32_t c = l; c < p.chunks; c += p.lanes_per_row) {
                uint32_t r[RB / 4];
                const uint4* src = reinterpret_cast<const uint4*>(p.W + (size_t)n * row_bytes + (size_t)c * RB);
#pragma unroll
                for (int i = 0; i < RB / 16; i++) {
                    const uint4 v = __ldg(src + i);
                    r[4 * i] = v.x; r[4 * i + 1] = v.y; r[4 * i + 2] = v.z; r[4 * i + 3] = v.w;
                }
                constexpr int MW = Cd::META_WORDS > 0 ? Cd::META_WORDS : 4;
                uint32_t meta[MW] = {};
                if (Cd::META_WORDS != 0) {           // one scale and one bias per 64 (4 words) or 32 (8 words) elements, two planes
                    const uint32_t groups = (p.K / 256) * MW;
                    const uint8_t* mp = p.meta + ((size_t)n * groups + (size_t)c * MW) * 2;
                    const uint8_t* bp = mp + (size_t)p.N * groups * 2;
                    if (MW == 4) {
                        const uint2 sc = __ldg(reinterpret_cast<const uint2*>(mp));
                        const uint2 bi = __ldg(reinterpret_cast<const uint2*>(bp));
                        meta[0] = sc.x; meta[1] = sc.y; meta[2] = bi.x; meta[3] = bi.y;
                    } else {
                        const uint4 sc = __ldg(reinterpret_cast<const uint4*>(mp));
                        const uint4 bi = __ldg(reinterpret_cast<const uint4*>(bp));
                        meta[0] = sc.x; meta[1] = sc.y; meta[2] = sc.z; meta[3] = sc.w;
                        meta[MW - 4] = bi.x; meta[MW - 3] = bi.y; meta[MW - 2] = bi.z; meta[MW - 1] = bi.w;
                    }
                }
                const float* xc = sx + (size_t)c * XSTRIDE;
#pragma unroll
                for (int s = 0; s < 4; s++) {
                    uint32_t o[32];
                    Cd::dequant64(r, s, o, meta);
#pragma unroll
                    for (int i = 0; i < 32; i++) {
                        const float2 w = __half22float2(*reinterpret_cast<const __half2*>(&o[i]));
#pragma unroll
                        for (int m = 0; m < M; m++) {
                            const float* xm = xc + (size_t)m * p.chunks * XSTRIDE + s * 64 + 2 * i;
                            acc[m] = fmaf(w.x, xm[0], acc[m]);
                            acc[m] = fmaf(w.y, xm[1], acc[m]);
                        }
                    }
                }
            }
        }
        // lanes of one row: lanes_per_row is a power of two and rows are lane-aligned groups
#pragma unroll
        for (int m = 0; m < M; m++)
            for (uint32_t off = p.lanes_per_row >> 1; off > 0; off >>= 1) acc[m] += __shfl_xor_sync(0xffffffffu, acc[m], off);
        if (l == 0 && n < p.N) {
            const float rs = Cd::ROW_SCALE ? __half2float(p.row_scale[n]) : 1.0f;
#pragma unroll
            for (int m = 0; m < M; m++) p.Y[(size_t)m * p.N + n] = __float2half_rn(Cd::ROW_SCALE ? acc[m] * rs : acc[m]);
        }
    }
}

int g_gv_sms = 0;

template <int FMT, int M>
cudaError_t launch_gemv_m(const GemmArgs& a, cudaStream_t stream) {
    using Cd = cdc::Codec<FMT>;
    GvParams p;
    p.X = (const __half*)a.X; p.W = (const uint8_t*)a.W0; p.Y = (__half*)a.Y;
    p.M = a.M; p.N = a.N; p.K = a.K; p.chunks = a.K / 256;
    if (p.chunks >= 32) { p.rows_per_warp = 1; p.lanes_per_row = 32; }
    else { uint32_t lp = 1; while (lp < p.chunks) lp <<= 1; p.lanes_per_row = lp; p.rows_per_warp = 32 / lp; }
    const size_t plane = (size_t)a.N * p.chunks * Cd::ROW_BYTES;
    p.meta = (const uint8_t*)a.W0 + plane;
    p.row_scale = (const __half*)p.meta;
    const size_t smem = (size_t)M * p.chunks * XSTRIDE * sizeof(float);
    static bool attr = false;
    if (!attr) {
        cudaError_t e = cudaFuncSetAttribute(qgemv_kernel<FMT, M>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        if (e != cudaSuccess) return e;
        attr = true;
    }
    if (!g_gv_sms) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&g_gv_sms, cudaDevAttrMultiProcessorCount, dev);
        if (g_gv_sms <= 0) g_gv_sms = 148;
    }
    // as many CTAs as fit per SM given the activation copy each keeps in shared memory, but no more warps than rows
    uint32_t per_sm = smem ? (uint32_t)((220 * 1024) / (smem + 1024)) : 8u;
    per_sm = per_sm < 1u ? 1u : (per_sm > 8u ? 8u : per_sm);
    uint32_t grid = (uint32_t)g_gv_sms * per_sm;
    const uint32_t need = (a.N + p.rows_per_warp * (GV_THREADS / 32) - 1) / (p.rows_per_warp * (GV_THREADS / 32));
    if (grid > need) grid = need;
    qgemv_kernel<FMT, M><<<grid, GV_THREADS, smem, stream>>>(p);
    return cudaGetLastError();
}

template <int FMT>
cudaError_t launch_gemv_fmt(const GemmArgs& a, cudaStream_t s) {
    return a.M == 1 ? launch_gemv_m<FMT, 1>(a, s) : cudaErrorInvalidValue;
}

}  // namespace

bool gemv_path_ok(const GemmArgs& a) {
    if (a.force_generic || a.M != 1 || a.W1 || a.residual || a.partial_out || a.layout != 0 || a.scatter.world || a.n_extra) return false;
    if (a.K == 0 || a.K % 256 != 0 || a.N == 0) return false;
    if (((uintptr_t)a.W0 & 15u) || ((uintptr_t)a.X & 1u)) return false;
    if ((size_t)a.M * (a.K / 256) * XSTRIDE * sizeof(float) > 200 * 1024) return false;
    switch (a.format) {
        case QUANT_Q4_0: case QUANT_MLX_4BIT: case QUANT_Q4_K: case QUANT_TERNARY_1_58: case QUANT_VAR_RATE_AFFINE: case QUANT_EXL3:
        case QUANT_MLX_4BIT_G64: case QUANT_TERNARY_ROW: case QUANT_MLX_4BIT_PLANAR: return true;
        default: return false;
    }
}

cudaError_t launch_gemv(const GemmArgs& a, cudaStream_t s) {
    switch (a.format) {
        case QUANT_Q4_0: return launch_gemv_fmt<QUANT_Q4_0>(a, s);
        case QUANT_MLX_4BIT: return launch_gemv_fmt<QUANT_MLX_4BIT>(a, s);
        case QUANT_Q4_K: return launch_gemv_fmt<QUANT_Q4_K>(a, s);
        case QUANT_TERNARY_1_58: return launch_gemv_fmt<QUANT_TERNARY_1_58>(a, s);
        case QUANT_VAR_RATE_AFFINE: return launch_gemv_fmt<QUANT_VAR_RATE_AFFINE>(a, s);
        case QUANT_EXL3: return launch_gemv_fmt<QUANT_EXL3>(a, s);
        case QUANT_MLX_4BIT_G64: return launch_gemv_fmt<QUANT_MLX_4BIT_G64>(a, s);
        case QUANT_MLX_4BIT_PLANAR: return launch_gemv_fmt<QUANT_MLX_4BIT_PLANAR>(a, s);
        case QUANT_TERNARY_ROW: return launch_gemv_fmt<QUANT_TERNARY_ROW>(a, s);
        default: return cudaErrorInvalidValue;
    }
}

}  // namespace qg
