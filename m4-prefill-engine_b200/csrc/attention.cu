// Causal flash attention over a Q8_0-compressed KV cache, and the Q8_0 compressor itself.
//
// Replaces flash_attn_mma_64x64_q8_0_d{64,128} (brick4_attn_kernels.metal:573-911),
// flash_attn_q8_0_causal_d128 (unified_8b_kernels.metal:857-998) and quantize_kv_to_q8_0
// (unified_8b_kernels.metal:118-145; host twin brick4_attn_bench.mm:37-55).
//
//   Q  [Hq][M][D] fp16        K,V [Hkv][Mkv][D/32] block_q8_0 (34 B: fp16 d, int8 qs[32])
//   O  [Hq][M][D] or [M][Hq*D] fp16
//   query row i sits at position pos0 + i and attends keys 0 .. pos0 + i; query head h reads
//   kv head h / (Hq/Hkv) (Hq == Hkv is the reference's case).
//
// One CTA = 64 query rows of one head, 4 warps x 16 rows.  Per 64-key step: the packed K and V
// bytes of the next step stream in with cp.async while this step's bytes are unpacked to fp16
// (value = fp16(q * d), the same rounding as the reference's dequantize_q8_0), S = Q.K^T and
// O += P.V run on the warp-level tensor-core MMA with fp32 accumulators, and the online softmax
// keeps its running max / sum per row in fp32 with quad shuffles.  Unlike the reference kernel
// (S and O in half, brick4_attn_kernels.metal:631,700) both accumulators stay in fp32.
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdint>
#include <mutex>

#include "../../include/b200_bridge.h"
#include "../../include/quant_router.h"
#include "bridge_state.cuh"
#include "layer_ops.cuh"

namespace attn {

constexpr int BQ = 64, BK = 64, THREADS = 128;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void cp_async16(void* dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t (&r)[4], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_h2(float lo, float hi) {
    __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&h);
}

struct Params {
    const __half* Q; const uint8_t* K; const uint8_t* V; __half* O;
    uint32_t Hq, Hkv, M, Mkv, pos0;
    float scale_log2e;
    int out_tokens_major, kv_fp16;
};

// D: head dim (64 or 128).  Shared layout: Q, K, V fp16 tiles with a 16-byte row pad (ldmatrix
// conflict-free), then two stages of packed K and V bytes.
template <int D>
__global__ void __launch_bounds__(THREADS) attn_q8kv_kernel(const Params p) {
    constexpr int LD = D + 8;                     // fp16 elements per padded row
    constexpr int ROW_RAW = (D / 32) * 34;        // packed bytes per key row
    constexpr int RAW_TILE = BK * ROW_RAW;        // contiguous: keys of one head follow one another
    constexpr int RAW_TILE_PAD = ((RAW_TILE + 15) & ~15) + 16;   // + one 16-byte phase
    extern __shared__ __align__(16) uint8_t smem[];
    __half* sQ = reinterpret_cast<__half*>(smem);
    __half* sK = sQ + BQ * LD;
    __half* sV = sK + BK * LD;
    uint8_t* sRaw = reinterpret_cast<uint8_t*>(sV + BK * LD);   // [2 stages][K,V][RAW_TILE_PAD]

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t4 = lane & 3;
    const uint32_t qt = gridDim.x - 1 - blockIdx.x;            // longest (latest) query tiles first
    const uint32_t h = blockIdx.y, hk = h / (p.Hq / p.Hkv);
    const uint32_t q0 = qt * BQ;
    const uint32_t last_pos = min(p.pos0 + min(q0 + BQ, p.M) - 1, p.Mkv - 1);   // last key any row of the tile may see
    const uint32_t n_ktiles = last_pos / BK + 1;

    // ---- stage the Q tile (rows past M are zero) ----
    for (int i = tid; i < BQ * (D / 8); i += THREADS) {
        const int r = i / (D / 8), c = i % (D / 8);
        uint4 v = make_uint4(0, 0, 0, 0);
        if (q0 + r < p.M) v = *reinterpret_cast<const uint4*>(p.Q + ((size_t)h * p.M + q0 + r) * D + c * 8);
        *reinterpret_cast<uint4*>(sQ + r * LD + c * 8) = v;
    }

    const size_t kv_row_bytes = p.kv_fp16 ? (size_t)D * 2 : (size_t)ROW_RAW;
    const uint8_t* Kh = p.K + (size_t)hk * p.Mkv * kv_row_bytes;
    const uint8_t* Vh = p.V + (size_t)hk * p.Mkv * kv_row_bytes;

    // issue the async copy of key tile `kt` into raw stage `st` (Q8_0), or straight into sK/sV (fp16 KV)
    auto issue = [&](uint32_t kt, int st) {
        const uint32_t k0 = kt * BK;
        const uint32_t rows = min((uint32_t)BK, p.Mkv - k0);
        if (p.kv_fp16) {
            for (int i = tid; i < BK * (D / 8); i += THREADS) {
                const int r = i / (D / 8), c = i % (D / 8);
                if ((uint32_t)r < rows) {
                    cp_async16(sK + r * LD + c * 8, Kh + ((size_t)(k0 + r) * D + c * 8) * 2);
                    cp_async16(sV + r * LD + c * 8, Vh + ((size_t)(k0 + r) * D + c * 8) * 2);
                }
            }
        } else {
            // Rows of one head are contiguous but only 2-byte aligned as a run (34-byte blocks), so copy
            // the 16-byte-aligned middle with cp.async and the ragged head and tail with 2-byte loads; the
            // shared-memory copy keeps the source's phase within 16 bytes (unpack() reads from +phase).
            const uint32_t bytes = rows * ROW_RAW;
#pragma unroll
            for (int which = 0; which < 2; which++) {
                const uint8_t* src = (which ? Vh : Kh) + (size_t)k0 * ROW_RAW;
                const uint32_t ph = (uint32_t)((uintptr_t)src & 15u);
                uint8_t* dst = sRaw + (size_t)(st * 2 + which) * RAW_TILE_PAD + ph;
                const uint32_t head = min(bytes, (16u - ph) & 15u);
                const uint32_t chunks = (bytes - head) / 16;
                for (uint32_t i = tid * 2; i < head; i += THREADS * 2)
                    *reinterpret_cast<uint16_t*>(dst + i) = *reinterpret_cast<const uint16_t*>(src + i);
                for (uint32_t i = tid; i < chunks; i += THREADS) cp_async16(dst + head + i * 16, src + head + i * 16);
                for (uint32_t i = head + chunks * 16 + tid * 2; i < bytes; i += THREADS * 2)
                    *reinterpret_cast<uint16_t*>(dst + i) = *reinterpret_cast<const uint16_t*>(src + i);
            }
        }
        cp_async_commit();
    };

    // unpack raw stage `st` into sK / sV: one thread per (row, 32-block), value = fp16(q * d)
    auto unpack = [&](uint32_t kt, int st) {
        const uint32_t k0 = kt * BK;
        const uint32_t rows = min((uint32_t)BK, p.Mkv - k0);
        const uint8_t* kraw = sRaw + (size_t)(st * 2 + 0) * RAW_TILE_PAD + ((uintptr_t)(Kh + (size_t)k0 * ROW_RAW) & 15u);
        const uint8_t* vraw = sRaw + (size_t)(st * 2 + 1) * RAW_TILE_PAD + ((uintptr_t)(Vh + (size_t)k0 * ROW_RAW) & 15u);
        for (int i = tid; i < 2 * BK * (D / 32); i += THREADS) {
            const int which = i / (BK * (D / 32));
            const int j = i % (BK * (D / 32));
            const int r = j / (D / 32), b = j % (D / 32);
            __half* dst = (which ? sV : sK) + r * LD + b * 32;
            if ((uint32_t)r < rows) {
                const uint8_t* blk = (which ? vraw : kraw) + (size_t)r * ROW_RAW + b * 34;
                const float d = __half2float(*reinterpret_cast<const __half*>(blk));
                const uint16_t* q16 = reinterpret_cast<const uint16_t*>(blk + 2);
#pragma unroll
                for (int e = 0; e < 16; e++) {
                    const uint16_t two = q16[e];
                    const float a = (float)(int8_t)(two & 0xFF) * d, c = (float)(int8_t)(two >> 8) * d;
                    *reinterpret_cast<__half2*>(dst + 2 * e) = __floats2half2_rn(a, c);
                }
            } else {
#pragma unroll
                for (int e = 0; e < 16; e++) *reinterpret_cast<uint32_t*>(dst + 2 * e) = 0u;
            }
        }
    };

    issue(0, 0);
    __syncthreads();    // Q tile visible

    // Q fragments for this warp's 16 rows
    uint32_t qf[D / 16][4];
#pragma unroll
    for (int kk = 0; kk < D / 16; kk++)
        ldsm_x4(qf[kk], sQ + (warp * 16 + (lane & 15)) * LD + kk * 16 + (lane >> 4) * 8);

    float o[D / 8][4];
#pragma unroll
    for (int i = 0; i < D / 8; i++) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f; }
    float m_run[2] = {-1e30f, -1e30f}, l_run[2] = {0.0f, 0.0f};
    const uint32_t row_pos[2] = {p.pos0 + q0 + warp * 16 + g, p.pos0 + q0 + warp * 16 + g + 8};

    for (uint32_t kt = 0; kt < n_ktiles; kt++) {
        const int st = kt & 1;
        cp_async_wait<0>();
        __syncthreads();                       // tile kt landed; everyone is done reading sK/sV of tile kt-1
        if (!p.kv_fp16) {
            if (kt + 1 < n_ktiles) issue(kt + 1, st ^ 1);
            unpack(kt, st);
            __syncthreads();
        }
        const uint32_t k0 = kt * BK;
        // warps whose rows all sit before this key tile have nothing to add
        const bool active = k0 <= p.pos0 + q0 + warp * 16 + 15;
        if (active) {
            float s[BK / 8][4];
#pragma unroll
            for (int i = 0; i < BK / 8; i++) { s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.0f; }
#pragma unroll
            for (int kk = 0; kk < D / 16; kk++) {
#pragma unroll
                for (int nt = 0; nt < BK / 16; nt++) {
                    uint32_t b[4];
                    ldsm_x4(b, sK + (nt * 16 + (lane >> 4) * 8 + (lane & 7)) * LD + kk * 16 + ((lane >> 3) & 1) * 8);
                    mma16816(s[2 * nt], qf[kk], b[0], b[1]);
                    mma16816(s[2 * nt + 1], qf[kk], b[2], b[3]);
                }
            }
            // scale, causal mask, running max
            float mx[2] = {m_run[0], m_run[1]};
#pragma unroll
            for (int nt = 0; nt < BK / 8; nt++)
#pragma unroll
                for (int e = 0; e < 4; e++) {
                    const uint32_t key = k0 + nt * 8 + t4 * 2 + (e & 1);
                    const int rr = e >> 1;
                    float v = s[nt][e] * p.scale_log2e;
                    if (key > row_pos[rr] || key >= p.Mkv) v = -1e30f;
                    s[nt][e] = v;
                    mx[rr] = fmaxf(mx[rr], v);
                }
#pragma unroll
            for (int rr = 0; rr < 2; rr++) {
                mx[rr] = fmaxf(mx[rr], __shfl_xor_sync(0xffffffffu, mx[rr], 1));
                mx[rr] = fmaxf(mx[rr], __shfl_xor_sync(0xffffffffu, mx[rr], 2));
            }
            float corr[2], rs[2] = {0.0f, 0.0f};
#pragma unroll
            for (int rr = 0; rr < 2; rr++) { corr[rr] = exp2f(m_run[rr] - mx[rr]); m_run[rr] = mx[rr]; }
            uint32_t pf[BK / 16][4];
#pragma unroll
            for (int nt = 0; nt < BK / 8; nt++) {
                float e0 = exp2f(s[nt][0] - mx[0]), e1 = exp2f(s[nt][1] - mx[0]);
                float e2 = exp2f(s[nt][2] - mx[1]), e3 = exp2f(s[nt][3] - mx[1]);
                // masked entries: exp2(-1e30 - m) underflows to 0 for any finite m; rows that have seen no
                // key yet keep m = -1e30 and would give exp2(0) = 1, so force those to 0
                if (s[nt][0] <= -1e30f) e0 = 0.0f;
                if (s[nt][1] <= -1e30f) e1 = 0.0f;
                if (s[nt][2] <= -1e30f) e2 = 0.0f;
                if (s[nt][3] <= -1e30f) e3 = 0.0f;
                rs[0] += e0 + e1; rs[1] += e2 + e3;
                pf[nt >> 1][(nt & 1) * 2 + 0] = pack_h2(e0, e1);
                pf[nt >> 1][(nt & 1) * 2 + 1] = pack_h2(e2, e3);
            }
#pragma unroll
            for (int rr = 0; rr < 2; rr++) l_run[rr] = l_run[rr] * corr[rr] + rs[rr];
#pragma unroll
            for (int i = 0; i < D / 8; i++) { o[i][0] *= corr[0]; o[i][1] *= corr[0]; o[i][2] *= corr[1]; o[i][3] *= corr[1]; }
            // O += P . V
#pragma unroll
            for (int kk = 0; kk < BK / 16; kk++) {
#pragma unroll
                for (int dt = 0; dt < D / 16; dt++) {
                    uint32_t b[4];
                    ldsm_x4_t(b, sV + (kk * 16 + ((lane >> 3) & 1) * 8 + (lane & 7)) * LD + dt * 16 + (lane >> 4) * 8);
                    mma16816(o[2 * dt], pf[kk], b[0], b[1]);
                    mma16816(o[2 * dt + 1], pf[kk], b[2], b[3]);
                }
            }
        }
        if (p.kv_fp16) {
            __syncthreads();                   // all reads of sK/sV done before the next tile overwrites them
            if (kt + 1 < n_ktiles) issue(kt + 1, 0);
        }
    }
    cp_async_wait<0>();

    // ---- finalise: divide by the row sums (quad-reduced) and write ----
#pragma unroll
    for (int rr = 0; rr < 2; rr++) {
        l_run[rr] += __shfl_xor_sync(0xffffffffu, l_run[rr], 1);
        l_run[rr] += __shfl_xor_sync(0xffffffffu, l_run[rr], 2);
    }
    const float inv[2] = {l_run[0] > 0.0f ? 1.0f / l_run[0] : 0.0f, l_run[1] > 0.0f ? 1.0f / l_run[1] : 0.0f};
#pragma unroll
    for (int rr = 0; rr < 2; rr++) {
        const uint32_t row = q0 + warp * 16 + g + rr * 8;
        if (row >= p.M) continue;
        __half* dst = p.out_tokens_major ? p.O + ((size_t)row * p.Hq + h) * D : p.O + ((size_t)h * p.M + row) * D;
#pragma unroll
        for (int i = 0; i < D / 8; i++)
            *reinterpret_cast<uint32_t*>(dst + i * 8 + t4 * 2) = pack_h2(o[i][rr * 2] * inv[rr], o[i][rr * 2 + 1] * inv[rr]);
    }
}

// ---------------------------------------------------------------------------------------------
// Grouped-head variant: one CTA = one kv head x a block of query positions x all G = Hq/Hkv query
// heads that share that kv head (128 rows: 8 warps x 16 rows; each warp holds 16 consecutive
// positions of one head).  A K/V tile is fetched and unpacked once for all G heads, int8 -> fp16
// goes through the mantissa trick (no convert instructions: 0x6400 | (q ^ 0x80) is the fp16 number
// 1024 + 128 + q), and the unpacked tiles are double-buffered so the unpack of key tile j+1
// overlaps the MMAs of tile j across warps.
// ---------------------------------------------------------------------------------------------
constexpr int GQ_ROWS = 128, GQ_THREADS = 256;

template <int D, int G>
__global__ void __launch_bounds__(GQ_THREADS) attn_gqa_kernel(const Params p) {
    constexpr int LD = D + 8;
    constexpr int BP = GQ_ROWS / G;               // query positions per CTA
    constexpr int ROW_RAW = (D / 32) * 34;
    constexpr int RAW_TILE = BK * ROW_RAW;
    constexpr int RAW_TILE_PAD = ((RAW_TILE + 15) & ~15) + 16;
    constexpr int WPH = BP / 16;                  // warps per head
    extern __shared__ __align__(16) uint8_t smem[];
    __half* sQ = reinterpret_cast<__half*>(smem);
    __half* sKV = sQ + GQ_ROWS * LD;              // [2 buffers][K, V][BK][LD]
    uint8_t* sRaw = reinterpret_cast<uint8_t*>(sKV + 4 * BK * LD);   // [2 stages][K, V][RAW_TILE_PAD]

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t4 = lane & 3;
    const uint32_t pb = gridDim.x - 1 - blockIdx.x;             // latest position blocks (longest) first
    const uint32_t hk = blockIdx.y;
    const uint32_t p0 = pb * BP;
    const uint32_t last_pos = min(p.pos0 + min(p0 + BP, p.M) - 1, p.Mkv - 1);
    const uint32_t n_ktiles = last_pos / BK + 1;

    // ---- stage Q: row r = head (r / BP), position p0 + r % BP ----
    for (int i = tid; i < GQ_ROWS * (D / 8); i += GQ_THREADS) {
        const int r = i / (D / 8), c = i % (D / 8);
        const uint32_t h = hk * G + r / BP, pos = p0 + r % BP;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (pos < p.M) v = *reinterpret_cast<const uint4*>(p.Q + ((size_t)h * p.M + pos) * D + c * 8);
        *reinterpret_cast<uint4*>(sQ + r * LD + c * 8) = v;
    }
    const size_t kv_row_bytes = p.kv_fp16 ? (size_t)D * 2 : (size_t)ROW_RAW;
    const uint8_t* Kh = p.K + (size_t)hk * p.Mkv * kv_row_bytes;
    const uint8_t* Vh = p.V + (size_t)hk * p.Mkv * kv_row_bytes;

    // async copy of key tile kt: packed bytes into raw stage kt&1, or fp16 rows straight into buffer kt&1
    auto issue = [&](uint32_t kt) {
        const uint32_t k0 = kt * BK, rows = min((uint32_t)BK, p.Mkv - k0);
        const int st = kt & 1;
        if (p.kv_fp16) {
            __half* bK = sKV + (size_t)(st * 2 + 0) * BK * LD;
            __half* bV = sKV + (size_t)(st * 2 + 1) * BK * LD;
            for (int i = tid; i < BK * (D / 8); i += GQ_THREADS) {
                const int r = i / (D / 8), c = i % (D / 8);
                if ((uint32_t)r < rows) {
                    cp_async16(bK + r * LD + c * 8, Kh + ((size_t)(k0 + r) * D + c * 8) * 2);
                    cp_async16(bV + r * LD + c * 8, Vh + ((size_t)(k0 + r) * D + c * 8) * 2);
                } else {
                    *reinterpret_cast<uint4*>(bK + r * LD + c * 8) = make_uint4(0, 0, 0, 0);
                    *reinterpret_cast<uint4*>(bV + r * LD + c * 8) = make_uint4(0, 0, 0, 0);
                }
            }
        } else {
            const uint32_t bytes = rows * ROW_RAW;
#pragma unroll
            for (int which = 0; which < 2; which++) {
                const uint8_t* src = (which ? Vh : Kh) + (size_t)k0 * ROW_RAW;
                const uint32_t ph = (uint32_t)((uintptr_t)src & 15u);
                uint8_t* dst = sRaw + (size_t)(st * 2 + which) * RAW_TILE_PAD + ph;
                const uint32_t head = min(bytes, (16u - ph) & 15u);
                const uint32_t chunks = (bytes - head) / 16;
                for (uint32_t i = tid * 2; i < head; i += GQ_THREADS * 2)
                    *reinterpret_cast<uint16_t*>(dst + i) = *reinterpret_cast<const uint16_t*>(src + i);
                for (uint32_t i = tid; i < chunks; i += GQ_THREADS) cp_async16(dst + head + i * 16, src + head + i * 16);
                for (uint32_t i = head + chunks * 16 + tid * 2; i < bytes; i += GQ_THREADS * 2)
                    *reinterpret_cast<uint16_t*>(dst + i) = *reinterpret_cast<const uint16_t*>(src + i);
            }
        }
        cp_async_commit();
    };

    // raw stage kt&1 -> fp16 buffer kt&1; one thread per (row, 32-block); value = fp16(q * d) rounded once
    auto unpack = [&](uint32_t kt) {
        const uint32_t k0 = kt * BK, rows = min((uint32_t)BK, p.Mkv - k0);
        const int st = kt & 1;
        const uint8_t* kraw = sRaw + (size_t)(st * 2 + 0) * RAW_TILE_PAD + ((uintptr_t)(Kh + (size_t)k0 * ROW_RAW) & 15u);
        const uint8_t* vraw = sRaw + (size_t)(st * 2 + 1) * RAW_TILE_PAD + ((uintptr_t)(Vh + (size_t)k0 * ROW_RAW) & 15u);
        for (int i = tid; i < 2 * BK * (D / 32); i += GQ_THREADS) {
            const int which = i / (BK * (D / 32));
            const int j = i % (BK * (D / 32));
            const int r = j / (D / 32), b = j % (D / 32);
            __half* dst = sKV + (size_t)(st * 2 + which) * BK * LD + r * LD + b * 32;
            if ((uint32_t)r < rows) {
                const uint8_t* blk = (which ? vraw : kraw) + (size_t)r * ROW_RAW + b * 34;
                const uint16_t* q16 = reinterpret_cast<const uint16_t*>(blk);
                const uint32_t dd = q16[0];
                const uint32_t d2 = dd | (dd << 16);
#pragma unroll
                for (int e = 0; e < 4; e++) {
                    uint32_t o[4];
#pragma unroll
                    for (int f = 0; f < 4; f++) {
                        const uint32_t two = q16[1 + e * 4 + f];
                        // bytes (b0, b1) -> lanes (bits 0-7, bits 16-23); flip the sign bit: unsigned q + 128
                        const uint32_t x = (__byte_perm(two, 0u, 0x4140u) ^ 0x00800080u) | 0x64006400u;
                        const __half2 qh = __hsub2(*reinterpret_cast<const __half2*>(&x), __half2half2(__float2half(1152.0f)));
                        const __half2 w = __hmul2(qh, *reinterpret_cast<const __half2*>(&d2));
                        o[f] = *reinterpret_cast<const uint32_t*>(&w);
                    }
                    *reinterpret_cast<uint4*>(dst + e * 8) = make_uint4(o[0], o[1], o[2], o[3]);
                }
            } else {
#pragma unroll
                for (int e = 0; e < 4; e++) *reinterpret_cast<uint4*>(dst + e * 8) = make_uint4(0, 0, 0, 0);
            }
        }
    };

    issue(0);
    if (n_ktiles > 1 && !p.kv_fp16) { /* second tile is issued inside the loop, after the first unpack */ }
    cp_async_wait<0>();
    __syncthreads();                               // Q tile and key tile 0 are in shared memory
    if (!p.kv_fp16) unpack(0);

    const uint32_t head = hk * G + warp / WPH;
    const uint32_t wpos = p0 + (warp % WPH) * 16;   // first query position of this warp
    uint32_t qf[D / 16][4];
#pragma unroll
    for (int kk = 0; kk < D / 16; kk++)
        ldsm_x4(qf[kk], sQ + (warp * 16 + (lane & 15)) * LD + kk * 16 + (lane >> 4) * 8);
    float o[D / 8][4];
#pragma unroll
    for (int i = 0; i < D / 8; i++) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f; }
    float m_run[2] = {-1e30f, -1e30f}, l_run[2] = {0.0f, 0.0f};
    const uint32_t row_pos[2] = {p.pos0 + wpos + g, p.pos0 + wpos + g + 8};

    if (n_ktiles > 1) issue(1);
    for (uint32_t kt = 0; kt < n_ktiles; kt++) {
        // tile kt is unpacked (or landed, fp16 KV) in buffer kt&1 once every thread passes this barrier;
        // the packed bytes of tile kt+1 are waited for first
        cp_async_wait<0>();
        __syncthreads();
        if (kt + 1 < n_ktiles && !p.kv_fp16) unpack(kt + 1);            // raw stage (kt+1)&1 -> buffer (kt+1)&1
        const __half* sK = sKV + (size_t)((kt & 1) * 2 + 0) * BK * LD;
        const __half* sV = sKV + (size_t)((kt & 1) * 2 + 1) * BK * LD;
        const uint32_t k0 = kt * BK;
        if (k0 <= p.pos0 + wpos + 15) {
            float s[BK / 8][4];
#pragma unroll
            for (int i = 0; i < BK / 8; i++) { s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.0f; }
#pragma unroll
            for (int kk = 0; kk < D / 16; kk++) {
#pragma unroll
                for (int nt = 0; nt < BK / 16; nt++) {
                    uint32_t b[4];
                    ldsm_x4(b, sK + (nt * 16 + (lane >> 4) * 8 + (lane & 7)) * LD + kk * 16 + ((lane >> 3) & 1) * 8);
                    mma16816(s[2 * nt], qf[kk], b[0], b[1]);
                    mma16816(s[2 * nt + 1], qf[kk], b[2], b[3]);
                }
            }
            float mx[2] = {m_run[0], m_run[1]};
#pragma unroll
            for (int nt = 0; nt < BK / 8; nt++)
#pragma unroll
                for (int e = 0; e < 4; e++) {
                    const uint32_t key = k0 + nt * 8 + t4 * 2 + (e & 1);
                    const int rr = e >> 1;
                    float v = s[nt][e] * p.scale_log2e;
                    if (key > row_pos[rr] || key >= p.Mkv) v = -1e30f;
                    s[nt][e] = v;
                    mx[rr] = fmaxf(mx[rr], v);
                }
#pragma unroll
            for (int rr = 0; rr < 2; rr++) {
                mx[rr] = fmaxf(mx[rr], __shfl_xor_sync(0xffffffffu, mx[rr], 1));
                mx[rr] = fmaxf(mx[rr], __shfl_xor_sync(0xffffffffu, mx[rr], 2));
            }
            float corr[2], rs[2] = {0.0f, 0.0f};
#pragma unroll
            for (int rr = 0; rr < 2; rr++) { corr[rr] = exp2f(m_run[rr] - mx[rr]); m_run[rr] = mx[rr]; }
            uint32_t pf[BK / 16][4];
#pragma unroll
            for (int nt = 0; nt < BK / 8; nt++) {
                float e0 = exp2f(s[nt][0] - mx[0]), e1 = exp2f(s[nt][1] - mx[0]);
                float e2 = exp2f(s[nt][2] - mx[1]), e3 = exp2f(s[nt][3] - mx[1]);
                if (s[nt][0] <= -1e30f) e0 = 0.0f;
                if (s[nt][1] <= -1e30f) e1 = 0.0f;
                if (s[nt][2] <= -1e30f) e2 = 0.0f;
                if (s[nt][3] <= -1e30f) e3 = 0.0f;
                rs[0] += e0 + e1; rs[1] += e2 + e3;
                pf[nt >> 1][(nt & 1) * 2 + 0] = pack_h2(e0, e1);
                pf[nt >> 1][(nt & 1) * 2 + 1] = pack_h2(e2, e3);
            }
#pragma unroll
            for (int rr = 0; rr < 2; rr++) l_run[rr] = l_run[rr] * corr[rr] + rs[rr];
#pragma unroll
            for (int i = 0; i < D / 8; i++) { o[i][0] *= corr[0]; o[i][1] *= corr[0]; o[i][2] *= corr[1]; o[i][3] *= corr[1]; }
#pragma unroll
            for (int kk = 0; kk < BK / 16; kk++) {
#pragma unroll
                for (int dt = 0; dt < D / 16; dt++) {
                    uint32_t b[4];
                    ldsm_x4_t(b, sV + (kk * 16 + ((lane >> 3) & 1) * 8 + (lane & 7)) * LD + dt * 16 + (lane >> 4) * 8);
                    mma16816(o[2 * dt], pf[kk], b[0], b[1]);
                    mma16816(o[2 * dt + 1], pf[kk], b[2], b[3]);
                }
            }
        }
        // The copy of tile kt+2 reuses raw stage kt&1 (unpacked before this iteration's barrier) or, for
        // fp16 KV, buffer kt&1 -- which this iteration's MMAs still read, hence the barrier in that case.
        if (kt + 2 < n_ktiles) {
            if (p.kv_fp16) __syncthreads();
            issue(kt + 2);
        }
    }
    cp_async_wait<0>();

#pragma unroll
    for (int rr = 0; rr < 2; rr++) {
        l_run[rr] += __shfl_xor_sync(0xffffffffu, l_run[rr], 1);
        l_run[rr] += __shfl_xor_sync(0xffffffffu, l_run[rr], 2);
    }
    const float inv[2] = {l_run[0] > 0.0f ? 1.0f / l_run[0] : 0.0f, l_run[1] > 0.0f ? 1.0f / l_run[1] : 0.0f};
#pragma unroll
    for (int rr = 0; rr < 2; rr++) {
        const uint32_t pos = wpos + g + rr * 8;
        if (pos >= p.M) continue;
        __half* dst = p.out_tokens_major ? p.O + ((size_t)pos * p.Hq + head) * D : p.O + ((size_t)head * p.M + pos) * D;
#pragma unroll
        for (int i = 0; i < D / 8; i++)
            *reinterpret_cast<uint32_t*>(dst + i * 8 + t4 * 2) = pack_h2(o[i][rr * 2] * inv[rr], o[i][rr * 2 + 1] * inv[rr]);
    }
}

template <int D> size_t gqa_smem_bytes() {
    constexpr int LD = D + 8;
    constexpr int RAW_TILE_PAD = (((BK * (D / 32) * 34) + 15) & ~15) + 16;
    return (size_t)(GQ_ROWS + 4 * BK) * LD * 2 + 4 * (size_t)RAW_TILE_PAD;
}

template <int D, int G> cudaError_t launch_gqa(const Params& p, cudaStream_t stream) {
    constexpr int BP = GQ_ROWS / G;
    dim3 grid((p.M + BP - 1) / BP, p.Hkv);
    cudaFuncSetAttribute(attn_gqa_kernel<D, G>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)gqa_smem_bytes<D>());
    attn_gqa_kernel<D, G><<<grid, GQ_THREADS, gqa_smem_bytes<D>(), stream>>>(p);
    return cudaGetLastError();
}

// Q8_0 compression, one thread per 32-value block.  Bit-exact with the reference: the scale is
// amax/127 in fp32, stored rounded to fp16, while the quantisation step uses the reciprocal of
// the *unrounded* fp32 scale; rounding is half away from zero; codes are clamped to [-128, 127].
// A CTA's 128 blocks (4352 output bytes, a multiple of 16) are assembled in shared memory and written
// back with 16-byte stores; inputs are read with 16-byte loads.
constexpr int QZ_THREADS = 128;
__global__ void __launch_bounds__(QZ_THREADS) quantize_q8_0_kernel(const __half* __restrict__ src, uint8_t* __restrict__ dst, size_t nblocks) {
    __shared__ __align__(16) uint8_t stage[QZ_THREADS * 34];
    const size_t b0 = (size_t)blockIdx.x * QZ_THREADS;
    const size_t b = b0 + threadIdx.x;
    const bool vec_in = (reinterpret_cast<uintptr_t>(src) & 15u) == 0;
    if (b < nblocks) {
        const __half* s = src + b * 32;
        float v[32], amax = 0.0f;
        if (vec_in) {
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const uint4 w = reinterpret_cast<const uint4*>(s)[i];
                const uint32_t ws[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
                for (int k = 0; k < 4; k++) {
                    const __half2 h = *reinterpret_cast<const __half2*>(&ws[k]);
                    v[8 * i + 2 * k] = __low2float(h); v[8 * i + 2 * k + 1] = __high2float(h);
                }
            }
        } else {
#pragma unroll
            for (int i = 0; i < 32; i++) v[i] = __half2float(s[i]);
        }
#pragma unroll
        for (int i = 0; i < 32; i++) amax = fmaxf(amax, fabsf(v[i]));
        const float d = __fdiv_rn(amax, 127.0f);
        const float id = d > 0.0f ? __fdiv_rn(1.0f, d) : 0.0f;
        uint16_t* o = reinterpret_cast<uint16_t*>(stage + threadIdx.x * 34);      // 34 is even: 2-byte aligned
        o[0] = __half_as_ushort(__float2half_rn(d));
#pragma unroll
        for (int i = 0; i < 16; i++) {
            int q0 = (int)roundf(__fmul_rn(v[2 * i], id)), q1 = (int)roundf(__fmul_rn(v[2 * i + 1], id));
            q0 = max(-128, min(127, q0)); q1 = max(-128, min(127, q1));
            o[1 + i] = (uint16_t)((uint32_t)(uint8_t)(int8_t)q0 | ((uint32_t)(uint8_t)(int8_t)q1 << 8));
        }
    }
    __syncthreads();
    const size_t nb_here = nblocks - b0 < (size_t)QZ_THREADS ? nblocks - b0 : (size_t)QZ_THREADS;
    const size_t bytes = nb_here * 34;
    uint8_t* out = dst + b0 * 34;
    if ((reinterpret_cast<uintptr_t>(out) & 15u) == 0) {
        for (size_t i = threadIdx.x; i < bytes / 16; i += QZ_THREADS)
            reinterpret_cast<uint4*>(out)[i] = reinterpret_cast<const uint4*>(stage)[i];
        for (size_t i = (bytes / 16) * 16 + threadIdx.x; i < bytes; i += QZ_THREADS) out[i] = stage[i];
    } else {
        for (size_t i = threadIdx.x; i < bytes / 2; i += QZ_THREADS)
            reinterpret_cast<uint16_t*>(out)[i] = reinterpret_cast<const uint16_t*>(stage)[i];
    }
}

__global__ void dequantize_q8_0_kernel(const uint8_t* __restrict__ src, __half* __restrict__ dst, size_t nblocks) {
    const size_t b = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (b >= nblocks) return;
    const uint8_t* blk = src + b * 34;
    const float d = __half2float(*reinterpret_cast<const __half*>(blk));
#pragma unroll
    for (int i = 0; i < 32; i++) dst[b * 32 + i] = __float2half_rn((float)(int8_t)blk[2 + i] * d);
}

template <int D> size_t smem_bytes() {
    constexpr int LD = D + 8;
    constexpr int RAW_TILE_PAD = (((BK * (D / 32) * 34) + 15) & ~15) + 16;
    return (size_t)(BQ + 2 * BK) * LD * 2 + 4 * (size_t)RAW_TILE_PAD;
}

cudaError_t launch_attention(const Params& p, uint32_t D, cudaStream_t stream) {
    // grouped-head kernel when the group size divides its 128-row tile into whole warps
    const uint32_t G = p.Hq / p.Hkv;
    if (D == 128) {
        if (G == 1) return launch_gqa<128, 1>(p, stream);
        if (G == 2) return launch_gqa<128, 2>(p, stream);
        if (G == 4) return launch_gqa<128, 4>(p, stream);
        if (G == 8) return launch_gqa<128, 8>(p, stream);
    } else if (D == 64) {
        if (G == 1) return launch_gqa<64, 1>(p, stream);
        if (G == 2) return launch_gqa<64, 2>(p, stream);
        if (G == 4) return launch_gqa<64, 4>(p, stream);
        if (G == 8) return launch_gqa<64, 8>(p, stream);
    }
    dim3 grid((p.M + BQ - 1) / BQ, p.Hq);
    if (D == 128) {
        cudaFuncSetAttribute(attn_q8kv_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_bytes<128>());
        attn_q8kv_kernel<128><<<grid, THREADS, smem_bytes<128>(), stream>>>(p);
    } else if (D == 64) {
        cudaFuncSetAttribute(attn_q8kv_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_bytes<64>());
        attn_q8kv_kernel<64><<<grid, THREADS, smem_bytes<64>(), stream>>>(p);
    } else {
        return cudaErrorInvalidValue;
    }
    return cudaGetLastError();
}

cudaError_t launch_quantize(const void* src, void* dst, size_t n_elements, cudaStream_t stream) {
    const size_t nb = n_elements / 32;
    if (nb == 0) return cudaSuccess;
    quantize_q8_0_kernel<<<(unsigned)((nb + QZ_THREADS - 1) / QZ_THREADS), QZ_THREADS, 0, stream>>>((const __half*)src, (uint8_t*)dst, nb);
    return cudaGetLastError();
}

cudaError_t launch_dequantize(const void* src, void* dst, size_t n_elements, cudaStream_t stream) {
    const size_t nb = n_elements / 32;
    if (nb == 0) return cudaSuccess;
    dequantize_q8_0_kernel<<<(unsigned)((nb + 127) / 128), 128, 0, stream>>>((const uint8_t*)src, (__half*)dst, nb);
    return cudaGetLastError();
}

cudaError_t launch_attention_simple(const void* Q, const void* K, const void* V, void* O, uint32_t Hq, uint32_t Hkv,
                                    uint32_t M, uint32_t Mkv, uint32_t D, float scale, uint32_t pos0, int out_tokens_major,
                                    int kv_fp16, cudaStream_t stream) {
    Params p;
    p.Q = (const __half*)Q; p.K = (const uint8_t*)K; p.V = (const uint8_t*)V; p.O = (__half*)O;
    p.Hq = Hq; p.Hkv = Hkv; p.M = M; p.Mkv = Mkv; p.pos0 = pos0;
    p.scale_log2e = scale * 1.4426950408889634f;
    p.out_tokens_major = out_tokens_major; p.kv_fp16 = kv_fp16;
    return launch_attention(p, D, stream);
}

}  // namespace attn

using namespace bridge;

extern "C" {

/* Compress fp16 values to Q8_0 (n_elements % 32 == 0): src fp16, dst 34 bytes per 32 values. */
int b200_bridge_quantize_kv_q8_0(void* src, size_t src_bytes, void* dst, size_t dst_bytes, size_t n_elements) {
    std::lock_guard<std::mutex> lock(g.mu);
    if (!g.initialized) return -1;
    if (!src || !dst || ((uintptr_t)src % 2) != 0) return -2;
    if (n_elements == 0 || n_elements % 32 != 0) return -4;
    const size_t out_bytes = n_elements / 32 * 34;
    if (src_bytes < n_elements * 2 || dst_bytes < out_bytes) return -2;
    int rc = 0;
    const void* s = resolve_in(src, n_elements * 2, g.stage_x, false, &rc);
    if (rc) return rc;
    void* host_dst = nullptr;
    void* d = resolve_out(dst, out_bytes, g.stage_y, &host_dst, &rc);
    if (rc) return rc;
    if (attn::launch_quantize(s, d, n_elements, g.stream) != cudaSuccess) return -6;
    g.launches++;
    if (host_dst && copy_back(host_dst, d, out_bytes) != 0) return -5;
    return 0;
}

int b200_bridge_dequantize_q8_0(void* src, size_t src_bytes, void* dst, size_t dst_bytes, size_t n_elements) {
    std::lock_guard<std::mutex> lock(g.mu);
    if (!g.initialized) return -1;
    if (!src || !dst || ((uintptr_t)dst % 2) != 0) return -2;
    if (n_elements == 0 || n_elements % 32 != 0) return -4;
    const size_t in_bytes = n_elements / 32 * 34;
    if (src_bytes < in_bytes || dst_bytes < n_elements * 2) return -2;
    int rc = 0;
    const void* s = resolve_in(src, in_bytes, g.stage_x, false, &rc);
    if (rc) return rc;
    void* host_dst = nullptr;
    void* d = resolve_out(dst, n_elements * 2, g.stage_y, &host_dst, &rc);
    if (rc) return rc;
    if (attn::launch_dequantize(s, d, n_elements, g.stream) != cudaSuccess) return -6;
    g.launches++;
    if (host_dst && copy_back(host_dst, d, n_elements * 2) != 0) return -5;
    return 0;
}

/* Causal attention.  Q [Hq][M][D] fp16; K, V [Hkv][Mkv][D/32] Q8_0 blocks (or fp16 [Hkv][Mkv][D] when
 * kv_fp16 != 0); O [Hq][M][D], or [M][Hq*D] when out_tokens_major != 0.  D is 64 or 128; Hq % Hkv == 0. */
int b200_bridge_dispatch_attention_q8kv(void* Q, void* K, void* V, void* O, uint32_t Hq, uint32_t Hkv, uint32_t M, uint32_t Mkv,
                                        uint32_t D, float scale, uint32_t pos0, int out_tokens_major, int kv_fp16) {
    std::lock_guard<std::mutex> lock(g.mu);
    if (!g.initialized) return -1;
    if (!Q || !K || !V || !O) return -2;
    if (Hq == 0 || Hkv == 0 || M == 0 || Mkv == 0 || (D != 64 && D != 128) || Hq % Hkv != 0) return -4;
    if (((uintptr_t)Q % 16) != 0 || ((uintptr_t)O % 4) != 0) return -2;
    const size_t q_bytes = (size_t)Hq * M * D * 2;
    const size_t kv_bytes = kv_fp16 ? (size_t)Hkv * Mkv * D * 2 : (size_t)Hkv * Mkv * (D / 32) * 34;
    int rc = 0;
    attn::Params p;
    p.Q = (const __half*)resolve_in(Q, q_bytes, g.stage_x, false, &rc);
    if (rc) return rc;
    p.K = (const uint8_t*)resolve_in(K, kv_bytes, g.stage_aux0, false, &rc);
    if (rc) return rc;
    p.V = (const uint8_t*)resolve_in(V, kv_bytes, g.stage_aux1, false, &rc);
    if (rc) return rc;
    if (((uintptr_t)p.K % 2) != 0 || ((uintptr_t)p.V % 2) != 0) return -2;
    if (kv_fp16 && ((((uintptr_t)p.K | (uintptr_t)p.V) % 16) != 0)) return -2;
    void* host_dst = nullptr;
    p.O = (__half*)resolve_out(O, q_bytes, g.stage_y, &host_dst, &rc);
    if (rc) return rc;
    p.Hq = Hq; p.Hkv = Hkv; p.M = M; p.Mkv = Mkv; p.pos0 = pos0;
    p.scale_log2e = scale * 1.4426950408889634f;
    p.out_tokens_major = out_tokens_major; p.kv_fp16 = kv_fp16;
    if (attn::launch_attention(p, D, g.stream) != cudaSuccess) { set_error("attention launch failed"); return -6; }
    g.launches++;
    if (host_dst && copy_back(host_dst, p.O, q_bytes) != 0) return -5;
    return 0;
}

}  // extern "C"
