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
#include "ptx.cuh"

namespace attn {

int g_force_legacy = 0;      // testing hook: 1 routes head-dim-128 attention to the warp-level MMA kernels; 2 and 3 to the
                             // tensor-memory kernel that unpacks Q8_0 tiles itself, with V transposed in shared memory
                             // (K-major B operand) or in its natural form (MN-major)

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
    int v_mode = 0;    // tensor-memory kernel: 0 V as an MN-major B operand (unpacked like K), 1 V transposed in shared memory
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

// ---------------------------------------------------------------------------------------------
// Tensor-memory variant (head dim 128, Q8_0 cache): the two contractions of a 128-key step run as
// tcgen05.mma with their accumulators in tensor memory.
//
//   CTA = one kv head x 128/G query positions x the G query heads sharing it (128 rows = UMMA M).
//   Shared memory holds four fp16 operand tiles in the 128-byte-swizzled K-major layout of the
//   projection kernel (two 64-column atoms each): Q [row][d], K [key][d], V^T [d][key], P [row][key],
//   plus two stages of packed K/V bytes fetched with cp.async.  Per key tile:
//     all threads     unpack K (16-byte stores) and V (transposed: 2-byte stores, a warp writes 32
//                     consecutive keys of one d, i.e. 64 contiguous bytes)
//     one thread      S = Q.K^T        : 8 MMAs 128x128x16 -> tensor-memory columns 0..127
//     warps 0-3       thread = query row = tensor-memory lane: scale, causal mask, running max and
//                     sum in registers (no shuffles: a thread owns its whole row), P = exp2(s - m) to
//                     shared memory as fp16, O *= exp2(m_old - m_new) in tensor memory, skipped while
//                     no row of the warp raised its maximum
//     one thread      O += P.V         : 8 MMAs 128x128x16 -> tensor-memory columns 128..255
//   The phases of one tile are separated by CTA barriers and two mbarriers the MMAs commit to.
//   Every mbarrier wait is bounded; on expiry the CTA stops issuing work and leaves.
// ---------------------------------------------------------------------------------------------
constexpr int TC_ROWS = 128, TC_BK = 128, TC_WORKERS = 256, TC_THREADS = TC_WORKERS + 32, TC_D = 128;   // 8 worker warps + the MMA issuer

// Development aid: with -DATTN_TRACE thread 0 of CTA (0,0) accumulates clock64() deltas per phase of the key-tile loop.
#ifdef ATTN_TRACE
__device__ unsigned long long g_attn_trace[8];
#define ATR_DECL unsigned long long atr_t = clock64(), atr_acc[8] = {0, 0, 0, 0, 0, 0, 0, 0}
#define ATR(i) do { const unsigned long long n_ = clock64(); atr_acc[i] += n_ - atr_t; atr_t = n_; } while (0)
#define ATR_FLUSH() do { if (threadIdx.x == 0 && blockIdx.x == 0 && blockIdx.y == 0) for (int i_ = 0; i_ < 8; i_++) g_attn_trace[i_] = atr_acc[i_]; } while (0)
#else
#define ATR_DECL do { } while (0)
#define ATR(i) do { } while (0)
#define ATR_FLUSH() do { } while (0)
#endif
constexpr int TC_ATOM = 128 * 128;                       // bytes of one [128 rows][64 fp16] atom
constexpr int TC_TILE = 2 * TC_ATOM;                     // one operand tile
constexpr int TC_ROW_RAW = (TC_D / 32) * 34;             // packed bytes of one key
constexpr int TC_RAW_TILE = TC_BK * TC_ROW_RAW;
constexpr int TC_RAW_PAD = ((TC_RAW_TILE + 15) & ~15) + 16;
constexpr size_t TC_SMEM = 1024 + 4 * (size_t)TC_TILE + 4 * (size_t)TC_RAW_PAD + 64 + 2 * 2 * 128 * 4;

__device__ __forceinline__ float ex2(float x) {        // 2^x, one MUFU instruction; ex2(-inf) = 0
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// 2^x for x <= 8 without the special-function unit: x = n + f with n the nearest integer (read off the low mantissa bits of
// x + 1.5 * 2^23) and |f| <= 1/2, 2^f as a degree-5 polynomial (relative error 3e-6, far below the fp16 rounding of the
// probabilities it produces), n added to the exponent field.  Inputs below -120 (masked scores are -inf) give 2^-120.
__device__ __forceinline__ float ex2_poly(float x) {
    x = fmaxf(x, -120.0f);
    const float r = x + 12582912.0f;
    const float f = x - (r - 12582912.0f);
    float p = 1.3333558146e-3f;
    p = fmaf(p, f, 9.6181291076e-3f);
    p = fmaf(p, f, 5.5504108665e-2f);
    p = fmaf(p, f, 2.4022650696e-1f);
    p = fmaf(p, f, 6.9314718056e-1f);
    p = fmaf(p, f, 1.0f);
    return __int_as_float(__float_as_int(p) + (__float_as_int(r) << 23));
}

// byte offset of fp16 element (row, col) inside a K-major swizzled tile of two 64-column atoms
__device__ __forceinline__ uint32_t tc_off(uint32_t row, uint32_t col) {
    return (col >> 6) * TC_ATOM + (row >> 3) * 1024u + (row & 7u) * 128u + ((((col & 63u) >> 3) ^ (row & 7u)) << 4) + (col & 7u) * 2u;
}

template <int G>
__global__ void __launch_bounds__(TC_THREADS, 1) attn_tc_kernel(const Params p, int* err) {
    constexpr int BP = TC_ROWS / G;                      // query positions per CTA
    extern __shared__ uint8_t smem_raw_[];
    uint8_t* base = smem_raw_ + ((1024u - (ptx::smem_u32(smem_raw_) & 1023u)) & 1023u);
    uint8_t* sQ = base;
    uint8_t* sK = sQ + TC_TILE;
    uint8_t* sVt = sK + TC_TILE;
    uint8_t* sP = sVt + TC_TILE;
    uint8_t* sRaw = sP + TC_TILE;                        // [2 stages][K, V][TC_RAW_PAD]
    uint64_t* bar_s = reinterpret_cast<uint64_t*>(sRaw + 4 * TC_RAW_PAD);
    uint64_t* bar_o = bar_s + 1;
    uint64_t* bar_raw = bar_o + 1;                       // [2] packed K/V bytes of a stage landed (bulk copies)
    uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(bar_raw + 2);
    volatile uint32_t* abort_flag = tmem_holder + 1;
    float* xch = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(bar_s) + 64);   // [2 parities][2 halves][128 rows]

    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t pb = gridDim.x - 1 - blockIdx.x;      // latest position blocks (longest) first
    const uint32_t hk = blockIdx.y;
    const uint32_t p0 = pb * BP;
    const uint32_t last_pos = min(p.pos0 + min(p0 + BP, p.M) - 1, p.Mkv - 1);
    const uint32_t n_ktiles = last_pos / TC_BK + 1;

    // (initialised by the thread that later issues the first bulk copy onto bar_raw, before any CTA barrier)
    if (tid == TC_WORKERS) {
        ptx::mbar_init(bar_s, 1); ptx::mbar_init(bar_o, 1); ptx::mbar_init(&bar_raw[0], 1); ptx::mbar_init(&bar_raw[1], 1);
        *abort_flag = 0u;
        ptx::fence_barrier_init();
    }
    __syncwarp();
    // Warp 8 issues every MMA and every bulk copy and does nothing else: the issuing thread is held while the
    // tensor pipe works through its MMAs, which would otherwise delay a worker warp's share of the unpacking.
    const bool worker = warp < 8u;
    if (warp == 8) { ptx::tmem_alloc(tmem_holder, 256); ptx::tmem_relinquish(); }

    const uint8_t* Kh = p.K + (size_t)hk * p.Mkv * TC_ROW_RAW;
    const uint8_t* Vh = p.V + (size_t)hk * p.Mkv * TC_ROW_RAW;

    // async copy of the packed bytes of key tile kt into raw stage kt & 1.  Global addresses are only 2-byte
    // aligned in general: the 16-byte phase of the source (the same for every tile of a head, a tile being 17408
    // bytes) is kept in shared memory, the ragged ends (< 16 bytes each) go through registers.
    const uint32_t phK = (uint32_t)((uintptr_t)Kh & 15u), phV = (uint32_t)((uintptr_t)Vh & 15u);
    const uint8_t* const k_end = p.K + (size_t)p.Hkv * p.Mkv * TC_ROW_RAW;
    const uint8_t* const v_end = p.V + (size_t)p.Hkv * p.Mkv * TC_ROW_RAW;
    // A tile goes as two bulk copies issued by one thread when the 16-byte-aligned span around it stays inside
    // the K and V buffers (always, except possibly at the very first and very last bytes of a buffer); otherwise
    // every thread copies 16-byte pieces with cp.async and the ragged ends through registers.
    auto bulk_ok = [&](uint32_t kt) {
        const uint32_t k0 = kt * TC_BK, bytes = min((uint32_t)TC_BK, p.Mkv - k0) * TC_ROW_RAW;
        const uint8_t* ks = Kh + (size_t)k0 * TC_ROW_RAW - phK;
        const uint8_t* vs = Vh + (size_t)k0 * TC_ROW_RAW - phV;
        return ks >= p.K && vs >= p.V && ks + ((phK + bytes + 15u) & ~15u) <= k_end && vs + ((phV + bytes + 15u) & ~15u) <= v_end;
    };
    auto issue = [&](uint32_t kt) {
        const uint32_t k0 = kt * TC_BK, rows = min((uint32_t)TC_BK, p.Mkv - k0);
        const uint32_t bytes = rows * TC_ROW_RAW;
        if (bulk_ok(kt)) {
            if (tid == TC_WORKERS) {
                const uint32_t nk = (phK + bytes + 15u) & ~15u, nv = (phV + bytes + 15u) & ~15u;
                ptx::mbar_arrive_expect_tx(&bar_raw[kt & 1u], nk + nv);
                ptx::bulk_load_1d(sRaw + ((kt & 1u) * 2 + 0) * TC_RAW_PAD, Kh + (size_t)k0 * TC_ROW_RAW - phK, nk, &bar_raw[kt & 1u]);
                ptx::bulk_load_1d(sRaw + ((kt & 1u) * 2 + 1) * TC_RAW_PAD, Vh + (size_t)k0 * TC_ROW_RAW - phV, nv, &bar_raw[kt & 1u]);
            }
            return;
        }
#pragma unroll
        for (int which = 0; which < 2; which++) {
            const uint32_t ph = which ? phV : phK;
            const uint8_t* src = (which ? Vh : Kh) + (size_t)k0 * TC_ROW_RAW;
            uint8_t* dst = sRaw + ((kt & 1u) * 2 + which) * TC_RAW_PAD + ph;
            const uint32_t head = min(bytes, (16u - ph) & 15u);
            const uint32_t chunks = (bytes - head) >> 4, tail0 = head + (chunks << 4);
            if (tid * 2u < head) *reinterpret_cast<uint16_t*>(dst + tid * 2u) = *reinterpret_cast<const uint16_t*>(src + tid * 2u);
            for (uint32_t i = tid; i < chunks; i += TC_THREADS) cp_async16(dst + head + (i << 4), src + head + (i << 4));
            if (tail0 + tid * 2u < bytes)
                *reinterpret_cast<uint16_t*>(dst + tail0 + tid * 2u) = *reinterpret_cast<const uint16_t*>(src + tail0 + tid * 2u);
        }
        cp_async_commit();
    };
    // packed bytes of tile kt have landed (a CTA barrier must follow before other threads' copies are read)
    uint32_t raw_phase = 0;                               // bit s: parity of the next bulk completion of stage s
    auto wait_raw = [&](uint32_t kt) {
        if (bulk_ok(kt)) {
            const uint32_t st = kt & 1u;
            ptx::mbar_wait<32>(&bar_raw[st], (raw_phase >> st) & 1u, abort_flag, err, 204);
            raw_phase ^= 1u << st;
        } else {
            cp_async_wait<0>();
        }
    };

    // raw stage kt & 1 -> sK (row-major keys) or sVt (transposed), one matrix per call, by all 256 threads: thread
    // t takes dims [64 h, 64 h + 64) of key r (r = t % 128, h = t / 128), 68 packed bytes read as 17 words when the
    // row is 4-byte aligned (it is whenever the cache base is), values = fp16(q * d) rounded once as the reference's
    // dequantize_q8_0.  K goes out as 16-byte stores, V^T as 2-byte stores (a warp writes 32 consecutive keys of
    // one d: 64 contiguous bytes, no bank conflict).
    auto unpack = [&](uint32_t kt, const uint32_t which) {
        const uint32_t k0 = kt * TC_BK, rows = min((uint32_t)TC_BK, p.Mkv - k0);
        const uint32_t r = tid & 127u, h = tid >> 7;
        const uint8_t* rawp = sRaw + (size_t)((kt & 1u) * 2 + which) * TC_RAW_PAD +
                              (which ? phV : phK) + r * TC_ROW_RAW + h * 68u;
        const __half2 off = __half2half2(__float2half(1152.0f));
        uint8_t* vt[8];
        const bool transposed = which && p.v_mode != 0;
        if (transposed) {
            const uint32_t cr = (r & 63u) >> 3;
            uint8_t* vb = sVt + (r >> 6) * TC_ATOM + h * 8u * 1024u + (r & 7u) * 2u;     // dims 64 h ..: 8 row groups further
#pragma unroll
            for (int x = 0; x < 8; x++) vt[x] = vb + x * 128 + ((cr ^ (uint32_t)x) << 4);
        }
        uint32_t q[17];                                    // two blocks: 68 bytes
        if (r < rows) {
            if ((ptx::smem_u32(rawp) & 3u) == 0u) {
#pragma unroll
                for (int i = 0; i < 17; i++) q[i] = reinterpret_cast<const uint32_t*>(rawp)[i];
            } else {
#pragma unroll
                for (int i = 0; i < 17; i++) {
                    const uint16_t* hp = reinterpret_cast<const uint16_t*>(rawp) + 2 * i;
                    q[i] = (uint32_t)hp[0] | ((uint32_t)hp[1] << 16);
                }
            }
        }
#pragma unroll
        for (int b = 0; b < 2; b++) {                      // block b of this half: bytes [34 b, 34 b + 34)
            uint32_t w[16];
            if (r < rows) {
                // 16-bit field f of the block sits at byte 34 b + 2 f: half (17 b + f) & 1 of word (17 b + f) / 2
                const uint32_t dw = q[(17 * b) >> 1];
                const uint32_t dd = ((17 * b) & 1) ? (dw >> 16) : (dw & 0xFFFFu);
                const uint32_t d2 = dd | (dd << 16);
#pragma unroll
                for (int f = 0; f < 16; f++) {
                    const int hidx = 17 * b + 1 + f;       // index of the 16-bit field holding codes 2f, 2f+1
                    const uint32_t word = q[hidx >> 1];
                    // bytes (b0, b1) -> (bits 0-7, bits 16-23); flip the sign bit: unsigned q + 128; 0x6400 | x = 1024 + x
                    const uint32_t sp = (hidx & 1) ? __byte_perm(word, 0u, 0x4342u) : __byte_perm(word, 0u, 0x4140u);
                    const uint32_t x = (sp ^ 0x00800080u) | 0x64006400u;
                    const __half2 qh = __hsub2(*reinterpret_cast<const __half2*>(&x), off);
                    const __half2 v = __hmul2(qh, *reinterpret_cast<const __half2*>(&d2));
                    w[f] = *reinterpret_cast<const uint32_t*>(&v);
                }
            } else {
#pragma unroll
                for (int f = 0; f < 16; f++) w[f] = 0u;    // absent keys: zero (P is zero there, 0 * garbage is not)
            }
            if (!transposed) {
                // row r, 16-byte chunks 4 b .. 4 b + 3 of atom h: (rowbase | xr << 4) ^ (c << 4) = rowbase + ((c ^ xr) << 4)
                uint8_t* rowb = (which ? sVt : sK) + h * TC_ATOM + (r >> 3) * 1024u + (r & 7u) * 128u + ((r & 7u) << 4);
#pragma unroll
                for (int e = 0; e < 4; e++)
                    *reinterpret_cast<uint4*>(rowb + (((b * 4 + e) << 4) ^ ((r & 7u) << 4)) - ((r & 7u) << 4)) =
                        make_uint4(w[4 * e], w[4 * e + 1], w[4 * e + 2], w[4 * e + 3]);
            } else {
                // element (d, key r) of V^T: vt[d & 7] + (d >> 3) * 1024 with the eight swizzled row starts vt[]
                // computed once per call, so every store is base register + immediate
#pragma unroll
                for (int f = 0; f < 16; f++) {
                    const int d = b * 32 + 2 * f;          // within this thread's 64 dims
                    *reinterpret_cast<uint16_t*>(vt[d & 7] + (d >> 3) * 1024) = (uint16_t)(w[f] & 0xFFFFu);
                    *reinterpret_cast<uint16_t*>(vt[(d + 1) & 7] + ((d + 1) >> 3) * 1024) = (uint16_t)(w[f] >> 16);
                }
            }
        }
    };

    issue(0);                                              // the first packed tile travels while Q is staged
    // ---- stage Q: row r = head (r / BP), position p0 + r % BP ----
    for (uint32_t i = tid; i < TC_ROWS * (TC_D / 8); i += TC_THREADS) {
        const uint32_t r = i / (TC_D / 8), c = i % (TC_D / 8);
        const uint32_t h = hk * G + r / BP, pos = p0 + r % BP;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (pos < p.M) v = *reinterpret_cast<const uint4*>(p.Q + ((size_t)h * p.M + pos) * TC_D + c * 8);
        *reinterpret_cast<uint4*>(sQ + tc_off(r, c * 8)) = v;
    }
    ptx::tc_fence_before_sync();
    __syncthreads();
    ptx::tc_fence_after_sync();
    const uint32_t tmem = *tmem_holder;
    const uint32_t tS = tmem, tO = tmem + 128u;
    const uint32_t idesc = ptx::umma_idesc_f16(128, 128);
    const uint64_t desc_hi = ptx::umma_desc_k_sw128(0u);
    auto desc = [&](const uint8_t* tile, int atom, int kk) {
        return desc_hi | (uint64_t)((((ptx::smem_u32(tile) + atom * TC_ATOM) & 0x3FFFFu) >> 4) + 2 * kk);
    };
    // V as the B operand of O += P.V in its natural [key][d] form: MN-major (d contiguous), 128-byte swizzle.  The 64
    // d of an atom row are the contiguous run, the second atom (d 64..127) lies TC_ATOM bytes further (leading byte
    // offset), groups of eight keys are 1024 bytes apart (stride byte offset); 16 keys further = 2048 bytes.
    const uint32_t idesc_pv = p.v_mode == 0 ? (idesc | (1u << 16)) : idesc;
    const uint64_t vdesc_hi = ((uint64_t)(TC_ATOM >> 4) << 16) | ((uint64_t)(1024 >> 4) << 32) | ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
    auto desc_v = [&](int atom, int kk) {
        if (p.v_mode != 0) return desc(sVt, atom, kk);
        return vdesc_hi | (uint64_t)(((ptx::smem_u32(sVt) + (uint32_t)(atom * 4 + kk) * 2048u) & 0x3FFFFu) >> 4);
    };

    // Two threads per query row: thread t and t + 128 (warps w and w + 4 address the same tensor-memory lanes)
    // own columns [0, 64) and [64, 128) of the row's scores and outputs.  They share the running maximum (one
    // float exchanged through shared memory per tile) and keep partial sums that meet only in the epilogue.
    const uint32_t row = tid & 127u, half_id = tid >> 7, c_base = half_id * 64u;
    const uint32_t head = hk * G + row / BP, pos = p0 + row % BP;
    const uint32_t row_pos = p.pos0 + pos;
    float m_run = -1e30f, l_run = 0.0f;
    const uint32_t lane_addr = ((warp & 3u) * 32u) << 16;
    bool ok = true;

    // Schedule of one key tile: the S MMAs run while V is unpacked, the PV MMAs while the next tile's K is unpacked.
    //   sK  : written by unpack K(kt) during PV(kt-1), read by S(kt)
    //   sVt : written by unpack V(kt) during S(kt) (after PV(kt-1) has completed), read by PV(kt)
    //   sP / O in tensor memory : written by the softmax of tile kt after PV(kt-1) has completed
    wait_raw(0);
    __syncthreads();                                       // packed bytes of tile 0 visible to every thread
    if (worker) unpack(0, 0);
    if (n_ktiles > 1) issue(1);
    ATR_DECL;
    for (uint32_t kt = 0; kt < n_ktiles; kt++) {
        const uint32_t ph = kt & 1u;
        ptx::fence_proxy_async_smem();                     // this thread's part of sK(kt)
        __syncthreads();
        ATR(0);
        if (*abort_flag) break;
        if (warp == 8) {
            ptx::tc_fence_after_sync();
            if (ptx::elect_one()) {
#pragma unroll
                for (int a = 0; a < 2; a++)
#pragma unroll
                    for (int kk = 0; kk < 4; kk++)
                        ptx::umma_f16_ss(tS, desc(sQ, a, kk), desc(sK, a, kk), idesc, (uint32_t)(a | kk) != 0u);
                ptx::umma_commit(bar_s);
            }
            __syncwarp();
        }
        // PV(kt-1) must be done before sVt, sP and O are touched again (a failed wait sets the abort flag, which
        // is tested after the next CTA barrier)
        if (kt > 0) ptx::mbar_wait<32>(bar_o, ph ^ 1u, abort_flag, err, 202);
        if (worker) unpack(kt, 1);
        ATR(1);
        if (worker) {
            ok = __all_sync(0xffffffffu, ptx::mbar_wait<32>(bar_s, ph, abort_flag, err, 201));
            ATR(2);
            // (a failed wait has set the abort flag; the code below still runs so that the pair barrier and the
            // warp-collective tensor-memory accesses stay matched, its results are discarded after the CTA barrier)
            ptx::tc_fence_after_sync();
            const uint32_t k0 = kt * TC_BK;
            // tiles entirely at or below every row's position (and inside the cache) need no mask
            const bool full = (k0 + TC_BK - 1 <= p.pos0 + p0) && (k0 + TC_BK <= p.Mkv);
            float sc[64];
#pragma unroll
            for (int c0 = 0; c0 < 64; c0 += 16) {
                uint32_t v[16];
                ptx::tmem_ld_x16(tS + lane_addr + c_base + c0, v);
#pragma unroll
                for (int j = 0; j < 16; j++) sc[c0 + j] = __uint_as_float(v[j]);
            }
            ptx::tmem_ld_wait();
            float mx = -1e30f;
            if (full) {
#pragma unroll
                for (int j = 0; j < 64; j++) mx = fmaxf(mx, sc[j]);
            } else {
#pragma unroll
                for (int j = 0; j < 64; j++) {
                    const uint32_t key = k0 + c_base + j;
                    if (key > row_pos || key >= p.Mkv) sc[j] = -INFINITY;
                    mx = fmaxf(mx, sc[j]);
                }
            }
            mx = mx * p.scale_log2e;                        // the scale is positive: max and scaling commute
            float* xm = xch + ph * 256u;
            xm[half_id * 128u + row] = mx;
            ptx::bar_sync(1 + (int)(warp & 3u), 64);        // this warp and its partner
            mx = fmaxf(fmaxf(mx, xm[(half_id ^ 1u) * 128u + row]), m_run);
            const float corr = ex2(m_run - mx);
            m_run = mx;
            ATR(3);
            float rs = 0.0f;
#pragma unroll
            for (int c0 = 0; c0 < 64; c0 += 16) {
                uint32_t pk[8];
#pragma unroll
                for (int j = 0; j < 16; j += 2) {
                    // masked scores are -inf: fma gives -inf, ex2 gives 0
                    const float e0 = ex2(fmaf(sc[c0 + j], p.scale_log2e, -mx));
                    const float e1 = ex2(fmaf(sc[c0 + j + 1], p.scale_log2e, -mx));
                    rs += e0 + e1;
                    pk[j >> 1] = pack_h2(e0, e1);
                }
                *reinterpret_cast<uint4*>(sP + tc_off(row, c_base + c0)) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
                *reinterpret_cast<uint4*>(sP + tc_off(row, c_base + c0 + 8)) = make_uint4(pk[4], pk[5], pk[6], pk[7]);
            }
            l_run = l_run * corr + rs;
            ATR(4);
            // O *= corr on this thread's 64 columns, skipped while no row of this warp raised its maximum
            if (kt > 0 && __any_sync(0xffffffffu, corr != 1.0f)) {
#pragma unroll
                for (int c0 = 0; c0 < 64; c0 += 16) {
                    uint32_t v[16];
                    ptx::tmem_ld_x16(tO + lane_addr + c_base + c0, v);
                    ptx::tmem_ld_wait();
#pragma unroll
                    for (int j = 0; j < 16; j++) v[j] = __float_as_uint(__uint_as_float(v[j]) * corr);
                    ptx::tmem_st_x16(tO + lane_addr + c_base + c0, v);
                }
                ptx::tmem_st_wait();
            }
            ptx::fence_proxy_async_smem();
            ATR(5);
            ptx::tc_fence_before_sync();
        }
        __syncthreads();
        ATR(6);
        if (*abort_flag) break;
        if (warp == 8) {
            ptx::tc_fence_after_sync();
            if (ptx::elect_one()) {
#pragma unroll
                for (int a = 0; a < 2; a++)
#pragma unroll
                    for (int kk = 0; kk < 4; kk++)
                        ptx::umma_f16_ss(tO, desc(sP, a, kk), desc_v(a, kk), idesc_pv, (kt | (uint32_t)(a | kk)) != 0u);
                ptx::umma_commit(bar_o);
            }
            __syncwarp();
        }
        if (kt + 1 < n_ktiles) {
            // Bulk copies complete on an mbarrier that every thread waits on itself, and raw stage kt & 1 was last read
            // (V of tile kt) before the barrier above: no further CTA barrier, so the workers start on the next K tile
            // while warp 8 is still held issuing the PV MMAs.  The cp.async path needs every thread's copies to be visible.
            wait_raw(kt + 1);
            if (!bulk_ok(kt + 1)) __syncthreads();
            ATR(0);
            if (kt + 2 < n_ktiles) issue(kt + 2);
            ATR(6);
            if (worker) unpack(kt + 1, 0);                 // sK is free: S(kt) completed before this tile's softmax
        }
        ATR(7);
    }
    // the last PV
    ptx::mbar_wait<32>(bar_o, (n_ktiles - 1u) & 1u, abort_flag, err, 203);
    __syncthreads();
    ATR_FLUSH();
    cp_async_wait<0>();

    if (worker) xch[half_id * 128u + row] = l_run;         // (the loop's last use of this buffer is behind a CTA barrier)
    __syncthreads();
    if (worker && !*abort_flag) {
        // (the tensor-memory loads are warp-collective: every lane takes part, only the stores depend on the row)
        ptx::tc_fence_after_sync();
        const bool row_ok = pos < p.M;
        const float l_tot = l_run + xch[(half_id ^ 1u) * 128u + row];
        const float inv = l_tot > 0.0f ? 1.0f / l_tot : 0.0f;
        __half* dst = (p.out_tokens_major ? p.O + ((size_t)pos * p.Hq + head) * TC_D : p.O + ((size_t)head * p.M + pos) * TC_D) + c_base;
#pragma unroll
        for (int c0 = 0; c0 < 64; c0 += 16) {
            uint32_t v[16];
            ptx::tmem_ld_x16(tO + lane_addr + c_base + c0, v);
            ptx::tmem_ld_wait();
            uint32_t pk[8];
#pragma unroll
            for (int j = 0; j < 16; j += 2) pk[j >> 1] = pack_h2(__uint_as_float(v[j]) * inv, __uint_as_float(v[j + 1]) * inv);
            if (row_ok) {
                *reinterpret_cast<uint4*>(dst + c0) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
                *reinterpret_cast<uint4*>(dst + c0 + 8) = make_uint4(pk[4], pk[5], pk[6], pk[7]);
            }
        }
    }
    ptx::tc_fence_before_sync();
    __syncthreads();
    if (warp == 8) { ptx::tc_fence_after_sync(); ptx::tmem_dealloc(tmem, 256); }
}

template <int G> cudaError_t launch_tc(const Params& p, cudaStream_t stream) {
    constexpr int BP = TC_ROWS / G;
    dim3 grid((p.M + BP - 1) / BP, p.Hkv);
    static bool attr_set = false;
    if (!attr_set) {
        cudaError_t e = cudaFuncSetAttribute(attn_tc_kernel<G>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)TC_SMEM);
        if (e != cudaSuccess) return e;
        attr_set = true;
    }
    attn_tc_kernel<G><<<grid, TC_THREADS, TC_SMEM, stream>>>(p, bridge::g.err_word);
    return cudaGetLastError();
}


// ---------------------------------------------------------------------------------------------
// Tensor-memory variant fed by TMA (head dim 128): K and V arrive as fp16 [Hkv][Mkv][128] -- an fp16 cache as it is, a
// Q8_0 cache dequantised once per call by dequant_q8_0_rows_kernel below (value = fp16(q * d), the rounding of the
// reference's dequantize_q8_0), instead of once per 128-position query block inside the attention kernel, where
// unpacking took half of every key tile's time.  TMA writes the tiles straight into the 128-byte-swizzled operand
// layout; V is used in its natural [key][d] form as an MN-major B operand.
//
//   shared memory   Q, P (32 KB each), two stages each of K and V (4 x 32 KB)
//   tensor memory   S in two buffers (columns 0..127, 128..255), O (256..383)
//   warp 8          one thread issues every TMA load and every MMA:
//                     S(kt+1) = Q.K(kt+1)^T is issued while the workers are busy with the softmax of tile kt,
//                     O += P(kt).V(kt) right after the CTA barrier that ends that softmax
//   warps 0-7       softmax of tile kt as in the kernel above (two threads per query row): S(kt) from tensor memory,
//                   running maximum, then -- once PV(kt-1) has completed -- P to shared memory and the rescaling of O
//   One CTA barrier per key tile.  Every mbarrier wait is bounded.
//
//   Buffer reuse      S buffer b: written by S(kt), kt & 1 == b, issued after the barrier of tile kt-1, by which the
//                     workers have read S(kt-2) out of it.  K stage: the issuing thread waits for S(kt) itself during
//                     tile kt and requests K(kt+2) then, a whole tile before it is needed.  V stage and P:
//                     freed by the completion of PV(kt), which the workers (before writing P(kt+1)) and the issuing
//                     thread (before requesting V(kt+2)) wait for during tile kt+1.
// ---------------------------------------------------------------------------------------------
constexpr size_t T2_SMEM = 1024 + 6 * (size_t)TC_TILE + 128 + 2 * 2 * 128 * 4;

template <int G>
__global__ void __launch_bounds__(TC_THREADS, 1)
attn_tma_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
                const Params p, int* err) {
    constexpr int BP = TC_ROWS / G;                      // query positions per CTA
    extern __shared__ uint8_t smem_raw_[];
    ATR_DECL;
    uint8_t* base = smem_raw_ + ((1024u - (ptx::smem_u32(smem_raw_) & 1023u)) & 1023u);
    uint8_t* sQ = base;
    uint8_t* sP = sQ + TC_TILE;
    uint8_t* sK = sP + TC_TILE;                          // [2 stages]
    uint8_t* sV = sK + 2 * TC_TILE;                      // [2 stages]
    uint64_t* bar_s = reinterpret_cast<uint64_t*>(sV + 2 * TC_TILE);   // [2] S(kt) complete in buffer kt & 1
    uint64_t* bar_o = bar_s + 2;                         // PV(kt) complete
    uint64_t* k_full = bar_o + 1;                        // [2] K(kt) landed in stage kt & 1
    uint64_t* v_full = k_full + 2;                       // [2]
    uint64_t* q_full = v_full + 2;                       // the query tile landed
    uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(q_full + 1);
    volatile uint32_t* abort_flag = tmem_holder + 1;
    float* xch = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(bar_s) + 128);   // [2 parities][2 halves][128 rows]

    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    // CTAs start in the order of their linear index (x fastest): kv heads along x, position blocks along y, latest block
    // (most key tiles) first, so the long CTAs of every head start before any short one and the short ones fill the tail
    const uint32_t pb = gridDim.y - 1 - blockIdx.y;
    const uint32_t hk = blockIdx.x;
    const uint32_t p0 = pb * BP;
    const uint32_t last_pos = min(p.pos0 + min(p0 + BP, p.M) - 1, p.Mkv - 1);
    const uint32_t n_ktiles = last_pos / TC_BK + 1;
    const bool worker = warp < 8u;

    auto load_tile = [&](const CUtensorMap* map, uint8_t* stage_base, uint64_t* bar, uint32_t kt) {   // one thread
        uint8_t* dst = stage_base + (kt & 1u) * TC_TILE;
        ptx::mbar_arrive_expect_tx(&bar[kt & 1u], TC_TILE);
        ptx::tma_load_3d(dst, map, &bar[kt & 1u], 0, (int)(kt * TC_BK), (int)hk);             // d 0..63
        ptx::tma_load_3d(dst + TC_ATOM, map, &bar[kt & 1u], 64, (int)(kt * TC_BK), (int)hk);  // d 64..127
    };
    if (tid == TC_WORKERS) {
        for (int i = 0; i < 2; i++) { ptx::mbar_init(&bar_s[i], 1); ptx::mbar_init(&k_full[i], 1); ptx::mbar_init(&v_full[i], 1); }
        ptx::mbar_init(bar_o, 1); ptx::mbar_init(q_full, 1);
        *abort_flag = 0u;
        ptx::fence_barrier_init();
        // Q: row r = head hk * G + r / BP, position p0 + r % BP: a box of BP positions x G heads per 64 d, which lands as the
        // 128 rows of an atom in exactly that order; positions past M read as zero
        ptx::mbar_arrive_expect_tx(q_full, TC_TILE);
        ptx::tma_load_3d(sQ, &tmQ, q_full, 0, (int)p0, (int)(hk * G));
        ptx::tma_load_3d(sQ + TC_ATOM, &tmQ, q_full, 64, (int)p0, (int)(hk * G));
        load_tile(&tmK, sK, k_full, 0); load_tile(&tmV, sV, v_full, 0);
        if (n_ktiles > 1) { load_tile(&tmK, sK, k_full, 1); load_tile(&tmV, sV, v_full, 1); }
    }
    __syncwarp();
    if (warp == 8) { ptx::tmem_alloc(tmem_holder, 512); ptx::tmem_relinquish(); }

    ptx::tc_fence_before_sync();
    __syncthreads();
    ptx::tc_fence_after_sync();
    const uint32_t tmem = *tmem_holder;
    const uint32_t tO = tmem + 256u;
    const uint32_t idesc = ptx::umma_idesc_f16(128, 128);
    const uint32_t idesc_pv = idesc | (1u << 16);         // B (= V) MN-major
    const uint64_t desc_hi = ptx::umma_desc_k_sw128(0u);
    auto desc = [&](const uint8_t* tile, int atom, int kk) {
        return desc_hi | (uint64_t)((((ptx::smem_u32(tile) + atom * TC_ATOM) & 0x3FFFFu) >> 4) + 2 * kk);
    };
    // V [key][d]: the 64 d of an atom row are the contiguous run, the second atom lies TC_ATOM bytes further (leading
    // byte offset), groups of eight keys are 1024 bytes apart (stride byte offset); 16 keys further = 2048 bytes
    const uint64_t vdesc_hi = ((uint64_t)(TC_ATOM >> 4) << 16) | ((uint64_t)(1024 >> 4) << 32) | ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
    auto desc_v = [&](const uint8_t* tile, int step) {   // step: 16 keys
        return vdesc_hi | (uint64_t)(((ptx::smem_u32(tile) + (uint32_t)step * 2048u) & 0x3FFFFu) >> 4);
    };
    auto issue_s = [&](uint32_t kt) {                     // one thread
        const uint8_t* kt_tile = sK + (kt & 1u) * TC_TILE;
#pragma unroll
        for (int a = 0; a < 2; a++)
#pragma unroll
            for (int kk = 0; kk < 4; kk++)
                ptx::umma_f16_ss(tmem + (kt & 1u) * 128u, desc(sQ, a, kk), desc(kt_tile, a, kk), idesc, (uint32_t)(a | kk) != 0u);
        ptx::umma_commit(&bar_s[kt & 1u]);
    };

    const uint32_t row = tid & 127u, half_id = tid >> 7, c_base = half_id * 64u;
    const uint32_t head = hk * G + row / BP, pos = p0 + row % BP;
    const uint32_t row_pos = p.pos0 + pos;
    float m_run = -1e30f, l_run = 0.0f;
    const uint32_t lane_addr = ((warp & 3u) * 32u) << 16;

    if (warp == 8) {
        const bool ok = __all_sync(0xffffffffu, ptx::mbar_wait(q_full, 0u, abort_flag, err, 210) &&
                                                    ptx::mbar_wait(&k_full[0], 0u, abort_flag, err, 211));
        ptx::tc_fence_after_sync();
        if (ok && ptx::elect_one()) issue_s(0);
        __syncwarp();
    }
    ATR(7);                                                // prologue
    for (uint32_t kt = 0; kt < n_ktiles; kt++) {
        const uint32_t st = kt & 1u, use = (kt >> 1) & 1u;     // stage / S buffer and the parity of this use of it
        if (warp == 8) {
            bool ok = true;
            if (kt + 1 < n_ktiles) {
                ok = __all_sync(0xffffffffu, ptx::mbar_wait(&k_full[st ^ 1u], ((kt + 1) >> 1) & 1u, abort_flag, err, 211));
                ptx::tc_fence_after_sync();
                if (ok && ptx::elect_one()) issue_s(kt + 1);
                __syncwarp();
            }
            if (ok && kt + 2 < n_ktiles) {
                // K stage kt & 1 is free once S(kt) has completed: request K(kt+2) now, a whole tile before S(kt+2) is issued
                ok = __all_sync(0xffffffffu, ptx::mbar_wait<32>(&bar_s[st], use, abort_flag, err, 217));
                if (ok && lane == 0) load_tile(&tmK, sK, k_full, kt + 2);
                __syncwarp();
            }
            if (ok && kt > 0 && kt + 1 < n_ktiles) {
                // V stage (kt + 1) & 1 was read by PV(kt - 1)
                ok = __all_sync(0xffffffffu, ptx::mbar_wait<32>(bar_o, (kt - 1) & 1u, abort_flag, err, 212));
                if (ok && lane == 0) load_tile(&tmV, sV, v_full, kt + 1);
                __syncwarp();
            }
        } else {
            bool ok = __all_sync(0xffffffffu, ptx::mbar_wait<32>(&bar_s[st], use, abort_flag, err, 213));
            // (a failed wait has set the abort flag; the code below still runs so that the pair barrier and the
            // warp-collective tensor-memory accesses stay matched, its results are discarded after the CTA barrier)
            ptx::tc_fence_after_sync();
            ATR(0);
            const uint32_t k0 = kt * TC_BK;
            const bool full = (k0 + TC_BK - 1 <= p.pos0 + p0) && (k0 + TC_BK <= p.Mkv);
            float sc[64];
#pragma unroll
            for (int c0 = 0; c0 < 64; c0 += 16) {
                uint32_t v[16];
                ptx::tmem_ld_x16(tmem + st * 128u + lane_addr + c_base + c0, v);
#pragma unroll
                for (int j = 0; j < 16; j++) sc[c0 + j] = __uint_as_float(v[j]);
            }
            ptx::tmem_ld_wait();
            float mx = -1e30f;
            if (full) {
#pragma unroll
                for (int j = 0; j < 64; j++) mx = fmaxf(mx, sc[j]);
            } else {
#pragma unroll
                for (int j = 0; j < 64; j++) {
                    const uint32_t key = k0 + c_base + j;
                    if (key > row_pos || key >= p.Mkv) sc[j] = -INFINITY;
                    mx = fmaxf(mx, sc[j]);
                }
            }
            mx = mx * p.scale_log2e;                        // the scale is positive: max and scaling commute
            float* xm = xch + st * 256u;
            xm[half_id * 128u + row] = mx;
            ptx::bar_sync(1 + (int)(warp & 3u), 64);        // this warp and its partner
            mx = fmaxf(fmaxf(mx, xm[(half_id ^ 1u) * 128u + row]), m_run);
            // The reference maximum of a row moves only when the tile's maximum exceeds it by more than 2^8: probabilities
            // are then 2^(s - m_run) <= 256 instead of <= 1, which fp16 P and the fp32 sums hold just as well, the final
            // division by the row sum removes the common factor, and O has to be rescaled in tensor memory only when that
            // happens (after the first tile: hardly ever) instead of whenever any of a warp's 32 rows sees a new maximum
            // (almost every tile).  Both threads of a row take the same decision (same m_run, same mx).
            float corr = 1.0f;
            if (mx > m_run + 8.0f) { corr = ex2(m_run - mx); m_run = mx; }
            ATR(1);
            uint32_t pk[32];
            float rs = 0.0f;
#pragma unroll
            for (int j = 0; j < 64; j += 2) {
                // masked scores are -inf: fma gives -inf, ex2 gives 0.  One exponential in four is evaluated as a polynomial
                // on the FMA pipe: the SM's 16 ex2 per clock bound this loop (one in two made it issue-bound: 70 us against 62).
                const float x0 = fmaf(sc[j], p.scale_log2e, -m_run), x1 = fmaf(sc[j + 1], p.scale_log2e, -m_run);
                const float e0 = ex2(x0);
                const float e1 = (j & 2) ? ex2_poly(x1) : ex2(x1);
                rs += e0 + e1;
                pk[j >> 1] = pack_h2(e0, e1);
            }
            l_run = l_run * corr + rs;
            ATR(2);
            // P and O belong to PV(kt-1) until it has completed
            if (kt > 0) ok = __all_sync(0xffffffffu, ptx::mbar_wait<32>(bar_o, (kt - 1) & 1u, abort_flag, err, 214)) && ok;
            ptx::tc_fence_after_sync();
            ATR(3);
#pragma unroll
            for (int c0 = 0; c0 < 64; c0 += 8)
                *reinterpret_cast<uint4*>(sP + tc_off(row, c_base + c0)) = make_uint4(pk[c0 / 2], pk[c0 / 2 + 1], pk[c0 / 2 + 2], pk[c0 / 2 + 3]);
            ATR(4);
            // O *= corr on this thread's 64 columns, skipped while no row of this warp raised its maximum
            if (kt > 0 && __any_sync(0xffffffffu, corr != 1.0f)) {
#pragma unroll
                for (int c0 = 0; c0 < 64; c0 += 16) {
                    uint32_t v[16];
                    ptx::tmem_ld_x16(tO + lane_addr + c_base + c0, v);
                    ptx::tmem_ld_wait();
#pragma unroll
                    for (int j = 0; j < 16; j++) v[j] = __float_as_uint(__uint_as_float(v[j]) * corr);
                    ptx::tmem_st_x16(tO + lane_addr + c_base + c0, v);
                }
                ptx::tmem_st_wait();
            }
            ptx::fence_proxy_async_smem();
            ptx::tc_fence_before_sync();
            ATR(5);
        }
        __syncthreads();
        ATR(6);
        if (*abort_flag) break;
        if (warp == 8) {
            const bool ok = __all_sync(0xffffffffu, ptx::mbar_wait(&v_full[st], use, abort_flag, err, 215));
            ptx::tc_fence_after_sync();
            if (ok && ptx::elect_one()) {
                const uint8_t* v_tile = sV + st * TC_TILE;
#pragma unroll
                for (int a = 0; a < 2; a++)
#pragma unroll
                    for (int kk = 0; kk < 4; kk++)
                        ptx::umma_f16_ss(tO, desc(sP, a, kk), desc_v(v_tile, a * 4 + kk), idesc_pv, (kt | (uint32_t)(a | kk)) != 0u);
                ptx::umma_commit(bar_o);
            }
            __syncwarp();
        }
    }
    // the last PV
    if (!*abort_flag) ptx::mbar_wait<32>(bar_o, (n_ktiles - 1u) & 1u, abort_flag, err, 216);
    __syncthreads();
    ATR_FLUSH();

    if (worker) xch[half_id * 128u + row] = l_run;         // (the loop's last use of this buffer is behind a CTA barrier)
    __syncthreads();
    const bool bad = *abort_flag != 0u;
    if (worker && !bad) {
        // (the tensor-memory loads are warp-collective: every lane takes part, only the stores depend on the row)
        ptx::tc_fence_after_sync();
        const bool row_ok = pos < p.M;
        const float l_tot = l_run + xch[(half_id ^ 1u) * 128u + row];
        const float inv = l_tot > 0.0f ? 1.0f / l_tot : 0.0f;
        __half* dst = (p.out_tokens_major ? p.O + ((size_t)pos * p.Hq + head) * TC_D : p.O + ((size_t)head * p.M + pos) * TC_D) + c_base;
#pragma unroll
        for (int c0 = 0; c0 < 64; c0 += 16) {
            uint32_t v[16];
            ptx::tmem_ld_x16(tO + lane_addr + c_base + c0, v);
            ptx::tmem_ld_wait();
            uint32_t pk[8];
#pragma unroll
            for (int j = 0; j < 16; j += 2) pk[j >> 1] = pack_h2(__uint_as_float(v[j]) * inv, __uint_as_float(v[j + 1]) * inv);
            if (row_ok) {
                *reinterpret_cast<uint4*>(dst + c0) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
                *reinterpret_cast<uint4*>(dst + c0 + 8) = make_uint4(pk[4], pk[5], pk[6], pk[7]);
            }
        }
    }
    ptx::tc_fence_before_sync();
    __syncthreads();
    if (bad) {      // let loads that are still in flight land before the CTA gives its shared memory back
        const long long t0 = clock64();
        while (clock64() - t0 < 4000000LL) { }
        __syncthreads();
    }
    if (warp == 8) { ptx::tc_fence_after_sync(); ptx::tmem_dealloc(tmem, 512); }
}

// Q8_0 rows of head dim 128 (four 34-byte blocks, 2-byte aligned) -> fp16, one warp per key: lane l takes codes
// 4 (l % 8) .. + 3 of block l / 8 and writes 8 bytes, a warp one 256-byte row.  value = fp16(q * d), one rounding.
__global__ void __launch_bounds__(256) dequant_q8_0_rows_kernel(const uint8_t* __restrict__ K, const uint8_t* __restrict__ V,
                                                               __half* __restrict__ out, size_t rows) {
    const size_t w = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const uint32_t lane = threadIdx.x & 31u;
    if (w >= 2 * rows) return;
    const uint8_t* blk = (w < rows ? K + w * TC_ROW_RAW : V + (w - rows) * TC_ROW_RAW) + (lane >> 3) * 34u;
    const __half d = *reinterpret_cast<const __half*>(blk);
    const uint16_t* cp = reinterpret_cast<const uint16_t*>(blk + 2u + 4u * (lane & 7u));
    const uint32_t c = (uint32_t)cp[0] | ((uint32_t)cp[1] << 16);
    __half v[4];
#pragma unroll
    for (int i = 0; i < 4; i++) v[i] = __hmul(__int2half_rn((int)(int8_t)(c >> (8 * i))), d);
    uint2 o;
    o.x = (uint32_t)__half_as_ushort(v[0]) | ((uint32_t)__half_as_ushort(v[1]) << 16);
    o.y = (uint32_t)__half_as_ushort(v[2]) | ((uint32_t)__half_as_ushort(v[3]) << 16);
    *reinterpret_cast<uint2*>(out + w * TC_D + lane * 4u) = o;
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = [] {
        void* f = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess)
            f = nullptr;
        return (EncodeTiledFn)f;
    }();
    return fn;
}
// fp16 [heads][rows][128] as a 3-D map, boxes of box_heads x box_rows x 64 d with the 128-byte swizzle (box_heads * box_rows
// == 128: one atom); rows past the end read as zero
static bool make_kv_map(CUtensorMap* m, const void* ptr, uint32_t heads, uint32_t rows, uint32_t box_rows, uint32_t box_heads) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return false;
    cuuint64_t dims[3] = {TC_D, rows, heads};
    cuuint64_t strides[2] = {TC_D * 2, (cuuint64_t)rows * TC_D * 2};
    cuuint32_t box[3] = {64, box_rows, box_heads};
    cuuint32_t estr[3] = {1, 1, 1};
    return fn(m, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
              CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

int g_last_launches = 1;     // kernels the last launch_attention call enqueued

template <int G> cudaError_t launch_tma(const Params& p, cudaStream_t stream) {
    constexpr int BP = TC_ROWS / G;
    const __half *Kf = reinterpret_cast<const __half*>(p.K), *Vf = reinterpret_cast<const __half*>(p.V);
    g_last_launches = 1;
    if (!p.kv_fp16) {
        // the Q8_0 cache is dequantised once per call into a scratch block that grows with the longest context seen
        const size_t rows = (size_t)p.Hkv * p.Mkv;
        if (!bridge::g.kv_fp16.ensure(2 * rows * TC_D * sizeof(__half))) return cudaErrorMemoryAllocation;
        __half* scratch = static_cast<__half*>(bridge::g.kv_fp16.p);
        const size_t threads = 2 * rows * 32;
        dequant_q8_0_rows_kernel<<<(unsigned)((threads + 255) / 256), 256, 0, stream>>>(p.K, p.V, scratch, rows);
        cudaError_t e = cudaGetLastError();
        if (e != cudaSuccess) return e;
        Kf = scratch; Vf = scratch + rows * TC_D;
        g_last_launches = 2;
    }
    CUtensorMap tmQ, tmK, tmV;
    if (!make_kv_map(&tmK, Kf, p.Hkv, p.Mkv, TC_BK, 1) || !make_kv_map(&tmV, Vf, p.Hkv, p.Mkv, TC_BK, 1) ||
        !make_kv_map(&tmQ, p.Q, p.Hq, p.M, BP, G))
        return cudaErrorInvalidValue;
    dim3 grid(p.Hkv, (p.M + BP - 1) / BP);
    static bool attr_set = false;
    if (!attr_set) {
        cudaError_t e = cudaFuncSetAttribute(attn_tma_kernel<G>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)T2_SMEM);
        if (e != cudaSuccess) return e;
        attr_set = true;
    }
    attn_tma_kernel<G><<<grid, TC_THREADS, T2_SMEM, stream>>>(tmQ, tmK, tmV, p, bridge::g.err_word);
    return cudaGetLastError();
}

template <int D> size_t smem_bytes() {
    constexpr int LD = D + 8;
    constexpr int RAW_TILE_PAD = (((BK * (D / 32) * 34) + 15) & ~15) + 16;
    return (size_t)(BQ + 2 * BK) * LD * 2 + 4 * (size_t)RAW_TILE_PAD;
}

cudaError_t launch_attention(const Params& p, uint32_t D, cudaStream_t stream) {
    // grouped-head kernel when the group size divides its 128-row tile into whole warps
    const uint32_t G = p.Hq / p.Hkv;
    g_last_launches = 1;
    // tensor-memory kernels: head dim 128, every row of a lone pointer 16-byte aligned for the Q loads.  Default: K and V
    // as fp16 through TMA (a Q8_0 cache is dequantised once per call first; an fp16 cache needs 16-byte alignment).
    const bool tc_ok = D == 128 && ((uintptr_t)p.Q & 15u) == 0 && ((uintptr_t)p.O & 15u) == 0;
    if (tc_ok && g_force_legacy == 0 && (!p.kv_fp16 || (((uintptr_t)p.K | (uintptr_t)p.V) & 15u) == 0) && encode_fn() != nullptr) {
        if (G == 1) return launch_tma<1>(p, stream);
        if (G == 2) return launch_tma<2>(p, stream);
        if (G == 4) return launch_tma<4>(p, stream);
        if (G == 8) return launch_tma<8>(p, stream);
    }
    // the kernel that unpacks the Q8_0 tiles itself (hooks 2 and 3)
    if (tc_ok && !p.kv_fp16 && g_force_legacy != 1) {
        Params q = p;
        q.v_mode = g_force_legacy == 2 ? 1 : 0;
        if (G == 1) return launch_tc<1>(q, stream);
        if (G == 2) return launch_tc<2>(q, stream);
        if (G == 4) return launch_tc<4>(q, stream);
        if (G == 8) return launch_tc<8>(q, stream);
    }
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

int last_attention_launches() { return g_last_launches; }

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

void b200_bridge_force_legacy_attention(int on) { attn::g_force_legacy = on; }
int b200_bridge_attention_launches(void) { return attn::g_last_launches; }
#ifdef ATTN_TRACE
void b200_bridge_debug_attn_trace(unsigned long long* out) { cudaMemcpyFromSymbol(out, attn::g_attn_trace, 64); }
#endif

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
    g.launches += (uint64_t)attn::g_last_launches;
    if (host_dst && copy_back(host_dst, p.O, q_bytes) != 0) return -5;
    return 0;
}

}  // extern "C"
