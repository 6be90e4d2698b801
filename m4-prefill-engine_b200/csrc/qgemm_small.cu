// Few-token projection: Y[m][n] = sum_k X[m][k] * dequant(W)[n][k] for token counts where one launch has too few
// output tiles to fill the GPU (the decode-like shapes M = 33 / 128 / 129 of the router sweep,
// bench_universal_router.mm:764-773, and every projection of a short prefill).  HBM-bound: the packed weights are
// read once, so what matters is how fast an SM turns packed bytes into MMA operands.
//
// Differences from the persistent kernel in qgemm.cu, all aimed at that:
//   * the unpacked weights never touch shared memory: a thread owns one weight row = one tensor-memory lane, unpacks 64
//     elements to 32 registers of fp16 pairs and writes them with one tcgen05.st into a ring of A-operand stages in
//     tensor memory; the MMA takes A from tensor memory (tcgen05.mma [d], [a], b-desc) and only the activations from
//     shared memory.  That removes the 16 KB store + 16 KB operand read per 64-element step that bound the other kernel;
//   * small CTAs (4 unpack warps = the 4 lane quadrants, a copy warp, an MMA warp; <= 100 KB of shared memory, 256
//     tensor-memory columns) so that two CTAs share an SM and one's copies and unpacking overlap the other's;
//   * one work item per CTA: K is split up to eight ways, the splits of a tile form a thread-block cluster, and the
//     partial tiles meet in distributed shared memory (each CTA of the cluster sums one slice of the token columns in
//     split order -- deterministic -- and writes fp16 Y): no scratch buffer in global memory, no counters.
//
// Every mbarrier wait is bounded (ptx::mbar_wait).  The two cluster barriers are hardware barriers: every thread of
// every CTA reaches them on every path, including after a wait has given up.
#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstring>
#include <mutex>
#include <utility>

#include "codecs.cuh"
#include "ptx.cuh"
#include "qgemm.cuh"

namespace qg {
namespace small {

constexpr int W_TILE = 128;          // weight rows per tile = UMMA M = tensor-memory lanes
constexpr int KSTEP = 64;            // K elements per MMA group (4 MMAs of K = 16) and per A stage
constexpr int A_STAGES = 4;          // ring of unpacked-weight stages in tensor memory, 32 columns each
constexpr int A_COLS = KSTEP / 2;    // fp16 pairs: 32 columns per stage
constexpr int ACC_COL = A_STAGES * A_COLS;   // accumulator behind the A ring (columns 128 ..)
constexpr int TMEM_COLS = 256;
constexpr int RAW_STAGES = 2, B_STAGES = 4;
constexpr int THREADS = 192;         // warps 0-3 unpack + epilogue, warp 4 copies, warp 5 issues MMAs
constexpr int MAX_T = 128;

struct Params {
    uint32_t M, N, K, T;
    uint32_t n_tok_tiles, n_w_tiles, k_splits, kchunks;      // kchunks: packed chunks per split
    __half* Y;
    const __half* residual;
    uint32_t layout, D;
    int* err;
    const uint8_t* meta0;
    const __half* row_scale0;
};

__device__ __forceinline__ void tmem_st_x32(uint32_t taddr, const uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
          "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]),
          "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]),
          "r"(r[30]), "r"(r[31])
        : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem desc]: fp16 operands, fp32 accumulate, A rows = tensor-memory lanes, K packed two per column
__device__ __forceinline__ void umma_f16_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(tmem_d), "r"(tmem_a), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ uint32_t cluster_ctarank() { uint32_t r; asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r)); return r; }
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// address of `local` (a shared-memory address of this CTA) in the shared memory of CTA `rank` of the cluster
__device__ __forceinline__ uint32_t map_to_rank(uint32_t local, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local), "r"(rank));
    return r;
}
__device__ __forceinline__ void st_cluster_f32(uint32_t addr, float v) {
    asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(addr), "f"(v) : "memory");
}

template <int W, int HI>
__device__ __forceinline__ void ld_words(const uint8_t* rowp, uint32_t* r) {
    if constexpr (W < HI) {
        if constexpr (W % 4 == 0 && W + 4 <= HI) {
            const uint4 v = *reinterpret_cast<const uint4*>(rowp + W * 4);
            r[W] = v.x; r[W + 1] = v.y; r[W + 2] = v.z; r[W + 3] = v.w;
            ld_words<W + 4, HI>(rowp, r);
        } else if constexpr (W % 2 == 0 && W + 2 <= HI) {
            const uint2 v = *reinterpret_cast<const uint2*>(rowp + W * 4);
            r[W] = v.x; r[W + 1] = v.y;
            ld_words<W + 2, HI>(rowp, r);
        } else {
            r[W] = *reinterpret_cast<const uint32_t*>(rowp + W * 4);
            ld_words<W + 1, HI>(rowp, r);
        }
    }
}
template <int S> struct IntC { static constexpr int value = S; };
template <class F, int... S>
__device__ __forceinline__ void for_each_sub(F& f, std::integer_sequence<int, S...>) { (f(IntC<S>{}), ...); }

template <int FMT>
__global__ void __launch_bounds__(THREADS, 2)
qgemm_small_kernel(const __grid_constant__ CUtensorMap tmX, const __grid_constant__ CUtensorMap tmW, const Params p) {
    using Cd = cdc::Codec<FMT>;
    constexpr int ROW_BYTES = Cd::ROW_BYTES;
    constexpr int RAW_TILE_BYTES = ROW_BYTES * W_TILE;
    constexpr int SUBS = Cd::CHUNK / KSTEP;
    static_assert(!Cd::RAW_SWIZZLE_128 && Cd::META_WORDS == 0, "planar layouts with side planes stay on the persistent kernel");

    extern __shared__ uint8_t smem_dyn[];
    const uint32_t pad = (1024u - (ptx::smem_u32(smem_dyn) & 1023u)) & 1023u;
    uint8_t* sB = smem_dyn + pad;                                   // [B_STAGES][T rows of 128 bytes], 128-byte swizzle
    const uint32_t b_stage_bytes = p.T * 128u;
    uint8_t* sRaw = sB + B_STAGES * b_stage_bytes;                  // [RAW_STAGES][128 rows][ROW_BYTES]
    uint64_t* bars = reinterpret_cast<uint64_t*>(sRaw + RAW_STAGES * RAW_TILE_BYTES);
    uint64_t* raw_full = bars;
    uint64_t* raw_empty = raw_full + RAW_STAGES;
    uint64_t* a_full = raw_empty + RAW_STAGES;
    uint64_t* a_empty = a_full + A_STAGES;
    uint64_t* b_full = a_empty + A_STAGES;
    uint64_t* b_empty = b_full + B_STAGES;
    uint64_t* acc_full = b_empty + B_STAGES;
    uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(acc_full + 1);
    volatile uint32_t* abort_flag = tmem_holder + 1;
    // after the main loop the activation and packed rings are idle: the cluster's partial tiles land there
    float* recv = reinterpret_cast<float*>(sB);                     // [k_splits][T / k_splits token columns][128 features]

    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t ks = blockIdx.x % p.k_splits;                    // == rank inside the cluster
    const uint32_t tile = blockIdx.x / p.k_splits;
    const uint32_t wt = tile % p.n_w_tiles, tt = tile / p.n_w_tiles;
    const uint32_t ksteps = p.kchunks * (uint32_t)SUBS;

    if (threadIdx.x == 0) {
        for (int i = 0; i < RAW_STAGES; i++) { ptx::mbar_init(&raw_full[i], 1); ptx::mbar_init(&raw_empty[i], 4); }
        for (int i = 0; i < A_STAGES; i++) { ptx::mbar_init(&a_full[i], 4); ptx::mbar_init(&a_empty[i], 1); }
        for (int i = 0; i < B_STAGES; i++) { ptx::mbar_init(&b_full[i], 1); ptx::mbar_init(&b_empty[i], 1); }
        ptx::mbar_init(acc_full, 1);
        *abort_flag = 0u;
        ptx::fence_barrier_init();
    }
    if (warp == 5) { ptx::tmem_alloc(tmem_holder, TMEM_COLS); ptx::tmem_relinquish(); }
    ptx::tc_fence_before_sync();
    __syncthreads();
    ptx::tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_holder;

    if (warp == 4) {
        // ---------------- copies: packed weight chunks and activation tiles, interleaved in consumption order ----------------
        if (lane == 0) { ptx::prefetch_tensormap(&tmW); ptx::prefetch_tensormap(&tmX); }
        uint32_t rs = 0, rph = 0, bs = 0, bph = 0;
        bool ok = true;
        for (uint32_t kc = 0; ok && kc < p.kchunks; kc++) {
            ok = __all_sync(0xffffffffu, ptx::mbar_wait<32>(&raw_empty[rs], rph ^ 1u, abort_flag, p.err, 111));
            if (!ok) break;
            if (lane == 0) {
                ptx::mbar_arrive_expect_tx(&raw_full[rs], RAW_TILE_BYTES);
                ptx::tma_load_2d(sRaw + rs * RAW_TILE_BYTES, &tmW, &raw_full[rs],
                                 (int)((ks * p.kchunks + kc) * (ROW_BYTES / Cd::TMA_ELEM_BYTES)), (int)(wt * W_TILE));
            }
            __syncwarp();
            if (++rs == RAW_STAGES) { rs = 0; rph ^= 1u; }
            for (uint32_t s = 0; ok && s < (uint32_t)SUBS; s++) {
                ok = __all_sync(0xffffffffu, ptx::mbar_wait<32>(&b_empty[bs], bph ^ 1u, abort_flag, p.err, 112));
                if (!ok) break;
                if (lane == 0) {
                    ptx::mbar_arrive_expect_tx(&b_full[bs], b_stage_bytes);
                    ptx::tma_load_2d(sB + bs * b_stage_bytes, &tmX, &b_full[bs],
                                     (int)((ks * p.kchunks + kc) * Cd::CHUNK + s * KSTEP), (int)(tt * p.T));
                }
                __syncwarp();
                if (++bs == B_STAGES) { bs = 0; bph ^= 1u; }
            }
        }
    } else if (warp == 5) {
        // ---------------- MMA issuer ----------------
        const uint32_t idesc = ptx::umma_idesc_f16(W_TILE, p.T);
        const uint64_t desc_hi = ptx::umma_desc_k_sw128(0u);
        const uint32_t b_lo0 = (ptx::smem_u32(sB) & 0x3FFFFu) >> 4;
        uint32_t as = 0, aph = 0, bs = 0, bph = 0;
        bool ok = true;
        for (uint32_t st = 0; st < ksteps; st++) {
            ok = __all_sync(0xffffffffu, ptx::mbar_wait(&a_full[as], aph, abort_flag, p.err, 113) &&
                                             ptx::mbar_wait(&b_full[bs], bph, abort_flag, p.err, 114));
            if (!ok) break;
            ptx::tc_fence_after_sync();
            if (ptx::elect_one()) {
                const uint64_t bdesc = desc_hi | (uint64_t)(b_lo0 + bs * (b_stage_bytes >> 4));
                const uint32_t acol = tmem_base + as * A_COLS;
#pragma unroll
                for (int kk = 0; kk < KSTEP / 16; kk++)
                    umma_f16_ts(tmem_base + ACC_COL, acol + kk * 8, bdesc + 2 * kk, idesc, (st | (uint32_t)kk) != 0u);
                ptx::umma_commit(&a_empty[as]);
                ptx::umma_commit(&b_empty[bs]);
            }
            __syncwarp();
            if (++as == A_STAGES) { as = 0; aph ^= 1u; }
            if (++bs == B_STAGES) { bs = 0; bph ^= 1u; }
        }
        if (ok && ptx::elect_one()) ptx::umma_commit(acc_full);
        __syncwarp();
    } else {
        // ---------------- unpack: packed bytes -> registers -> tensor memory (A operand) ----------------
        const uint32_t row = warp * 32u + lane;                     // weight row of the tile = tensor-memory lane
        const uint32_t lane_base = (warp * 32u) << 16;
        uint32_t rs = 0, rph = 0, as = 0, aph = 0;
        bool ok = true;
        for (uint32_t kc = 0; ok && kc < p.kchunks; kc++) {
            ok = __all_sync(0xffffffffu, ptx::mbar_wait<32>(&raw_full[rs], rph, abort_flag, p.err, 115));
            if (!ok) break;
            uint32_t r[ROW_BYTES / 4];
            const uint8_t* rowp = sRaw + rs * RAW_TILE_BYTES + row * ROW_BYTES;
            ld_words<0, Cd::HDR_WORDS>(rowp, r);
            auto sub_tile = [&](auto S) {
                constexpr int s = decltype(S)::value;
                uint32_t o[32];
                ld_words<Cd::sub_lo(s), Cd::sub_hi(s)>(rowp, r);
                Cd::dequant64(r, s, o, nullptr);
                ok = __all_sync(0xffffffffu, ok && ptx::mbar_wait<32>(&a_empty[as], aph ^ 1u, abort_flag, p.err, 116));
                if (ok) {
                    ptx::tc_fence_after_sync();                      // the MMAs that read this stage have completed
                    tmem_st_x32(tmem_base + lane_base + as * A_COLS, o);
                    ptx::tmem_st_wait();
                    ptx::tc_fence_before_sync();
                    __syncwarp();
                    if (lane == 0) ptx::mbar_arrive(&a_full[as]);
                }
                if (++as == A_STAGES) { as = 0; aph ^= 1u; }
            };
            for_each_sub(sub_tile, std::make_integer_sequence<int, SUBS>{});
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(&raw_empty[rs]);         // after the stores that consumed every loaded register
            if (++rs == RAW_STAGES) { rs = 0; rph ^= 1u; }
        }
    }

    // ---------------- partial tiles meet in the cluster's shared memory ----------------
    // (1) every CTA of the cluster has finished its main loop: its rings may be overwritten
    if (warp < 4) {
        // the accumulator is complete once every MMA has; a failed wait sets the abort flag, the barriers are still reached
        ptx::mbar_wait<64>(acc_full, 0u, abort_flag, p.err, 117);
    }
    __syncthreads();
    const bool bad = *abort_flag != 0u;
    cluster_sync_all();
    const uint32_t cols = p.T / p.k_splits;                         // token columns each CTA of the cluster finishes
    if (warp < 4 && !bad) {
        ptx::tc_fence_after_sync();
        const uint32_t f = warp * 32u + lane;                       // feature row of the tile
        const uint32_t n = wt * W_TILE + f;
        float rsc = 1.0f;
        if (Cd::ROW_SCALE) rsc = n < p.N ? __half2float(p.row_scale0[n]) : 0.0f;
        const uint32_t taddr = tmem_base + ((warp * 32u) << 16) + ACC_COL;
        const uint32_t my_slot = ptx::smem_u32(recv) + (ks * cols * W_TILE + f) * 4u;     // [ks][col][f] in the owner's buffer
        for (uint32_t c0 = 0; c0 < p.T; c0 += 16) {
            uint32_t v[16];
            ptx::tmem_ld_x16(taddr + c0, v);
            ptx::tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 16; j++) {
                const uint32_t c = c0 + j, owner = c / cols, cl = c - owner * cols;
                const float x = Cd::ROW_SCALE ? __uint_as_float(v[j]) * rsc : __uint_as_float(v[j]);
                st_cluster_f32(map_to_rank(my_slot + cl * W_TILE * 4u, owner), x);
            }
        }
    }
    // (2) every partial value has landed
    cluster_sync_all();
    if (!bad) {
        // this CTA's token columns [ks * cols, (ks + 1) * cols): sum over the splits in split order, write fp16
        const uint32_t tok0 = tt * p.T + ks * cols;
        for (uint32_t i = threadIdx.x; i < cols * (W_TILE / 2); i += THREADS) {
            const uint32_t cl = i / (W_TILE / 2), f = (i % (W_TILE / 2)) * 2u;
            const uint32_t tok = tok0 + cl, n = wt * W_TILE + f;
            if (tok >= p.M || n >= p.N) continue;
            float a0 = 0.0f, a1 = 0.0f;
            for (uint32_t s = 0; s < p.k_splits; s++) {
                const float2 v = *reinterpret_cast<const float2*>(recv + (s * cols + cl) * W_TILE + f);
                a0 += v.x; a1 += v.y;
            }
            const bool pair = n + 1u < p.N;
            if (p.layout == 1) {
                const size_t o = ((size_t)(n / p.D) * p.M + tok) * p.D + (n % p.D);          // D is even: the pair stays in one head
                if (pair) *reinterpret_cast<__half2*>(p.Y + o) = __floats2half2_rn(a0, a1);
                else p.Y[o] = __float2half_rn(a0);
            } else {
                const size_t o = (size_t)tok * p.N + n;
                if (p.residual) { a0 += __half2float(p.residual[o]); if (pair) a1 += __half2float(p.residual[o + 1]); }
                if (pair && (p.N % 2u == 0u)) *reinterpret_cast<__half2*>(p.Y + o) = __floats2half2_rn(a0, a1);
                else { p.Y[o] = __float2half_rn(a0); if (pair) p.Y[o + 1] = __float2half_rn(a1); }
            }
        }
    }
    // ---------------- teardown ----------------
    ptx::tc_fence_before_sync();
    __syncthreads();
    if (bad) {      // let copies that are still in flight land before the CTA gives its shared memory back
        const long long t0 = clock64();
        while (clock64() - t0 < 4000000LL) { }
        __syncthreads();
    }
    if (warp == 5) { ptx::tc_fence_after_sync(); ptx::tmem_dealloc(tmem_base, TMEM_COLS); }
    // no CTA of the cluster leaves while another may still read its shared memory (all reads precede this point)
    cluster_sync_all();
}

// ---------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------
namespace {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = [] {
        void* f = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess)
            f = nullptr;
        return (EncodeTiledFn)f;
    }();
    return fn;
}
bool make_map(CUtensorMap* m, CUtensorMapDataType dt, const void* ptr, uint64_t inner, uint64_t outer, uint64_t row_bytes,
              uint32_t box_inner, uint32_t box_outer, CUtensorMapSwizzle sw) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return false;
    cuuint64_t dims[2] = {inner, outer};
    cuuint64_t strides[1] = {row_bytes};
    cuuint32_t box[2] = {box_inner, box_outer};
    cuuint32_t estr[2] = {1, 1};
    return fn(m, dt, 2, const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, sw,
              CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

struct Plan { uint32_t T, n_tok_tiles, n_w_tiles, k_splits, kchunks; size_t smem; };

template <int FMT> size_t smem_bytes(uint32_t T) {
    return 1024 + (size_t)B_STAGES * T * 128 + (size_t)RAW_STAGES * cdc::Codec<FMT>::ROW_BYTES * W_TILE + 256;
}

int g_sms = 0;
int sms() {
    if (!g_sms) { int dev = 0; cudaGetDevice(&dev); cudaDeviceGetAttribute(&g_sms, cudaDevAttrMultiProcessorCount, dev); if (g_sms <= 0) g_sms = 148; }
    return g_sms;
}

template <int FMT> bool make_plan(const GemmArgs& a, Plan& pl) {
    using Cd = cdc::Codec<FMT>;
    pl.n_tok_tiles = (a.M + MAX_T - 1) / MAX_T;
    const uint32_t per = (a.M + pl.n_tok_tiles - 1) / pl.n_tok_tiles;
    pl.T = (per + 15u) & ~15u;
    pl.n_w_tiles = (a.N + W_TILE - 1) / W_TILE;
    const uint32_t chunks = a.K / Cd::CHUNK;
    const uint32_t tiles = pl.n_tok_tiles * pl.n_w_tiles;
    // split K while all CTAs still fit on the GPU at two per SM, every split keeps a whole chunk, and the token columns
    // divide evenly among the CTAs of a cluster
    pl.k_splits = 1;
    for (uint32_t s = 2; s <= 8; s *= 2) {
        if (tiles * s > 2u * (uint32_t)sms() || chunks % s != 0 || pl.T % s != 0) break;
        pl.k_splits = s;
    }
    pl.kchunks = chunks / pl.k_splits;
    pl.smem = smem_bytes<FMT>(pl.T);
    // the cluster's receive buffer ([T][128] floats) lies over the activation and packed rings
    const size_t rings = (size_t)B_STAGES * pl.T * 128 + (size_t)RAW_STAGES * Cd::ROW_BYTES * W_TILE;
    return (size_t)pl.T * W_TILE * 4 <= rings && tiles * pl.k_splits <= 65535u * 8u;
}

template <int FMT> cudaError_t launch_fmt(const GemmArgs& a, int* err, cudaStream_t stream) {
    using Cd = cdc::Codec<FMT>;
    Plan pl;
    if (!make_plan<FMT>(a, pl)) return cudaErrorInvalidValue;
    const uint64_t w_row_bytes = (uint64_t)(a.K / Cd::CHUNK) * Cd::ROW_BYTES;
    CUtensorMap tmX, tmW;
    if (!make_map(&tmX, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, a.X, a.K, a.M, (uint64_t)a.K * 2, KSTEP, pl.T, CU_TENSOR_MAP_SWIZZLE_128B))
        return cudaErrorInvalidValue;
    constexpr int EB = Cd::TMA_ELEM_BYTES;
    if (!make_map(&tmW, EB == 2 ? CU_TENSOR_MAP_DATA_TYPE_UINT16 : CU_TENSOR_MAP_DATA_TYPE_UINT8, a.W0, w_row_bytes / EB, a.N, w_row_bytes,
                  Cd::ROW_BYTES / EB, W_TILE, CU_TENSOR_MAP_SWIZZLE_NONE))
        return cudaErrorInvalidValue;
    Params p;
    p.M = a.M; p.N = a.N; p.K = a.K; p.T = pl.T;
    p.n_tok_tiles = pl.n_tok_tiles; p.n_w_tiles = pl.n_w_tiles; p.k_splits = pl.k_splits; p.kchunks = pl.kchunks;
    p.Y = (__half*)a.Y; p.residual = (const __half*)a.residual; p.layout = (uint32_t)a.layout; p.D = a.D ? a.D : 2;
    p.err = err;
    p.meta0 = (const uint8_t*)a.W0 + (size_t)a.N * w_row_bytes;
    p.row_scale0 = (const __half*)p.meta0;
    static uint64_t attr_mask = 0;
    static std::mutex mu;
    {
        int dev = 0;
        cudaGetDevice(&dev);
        std::lock_guard<std::mutex> lock(mu);
        if (!(dev >= 0 && dev < 64 && ((attr_mask >> dev) & 1u))) {
            cudaError_t e = cudaFuncSetAttribute(qgemm_small_kernel<FMT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_bytes<FMT>(MAX_T));
            if (e != cudaSuccess) return e;
            if (dev >= 0 && dev < 64) attr_mask |= 1ull << dev;
        }
    }
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    cfg.gridDim = dim3(pl.n_tok_tiles * pl.n_w_tiles * pl.k_splits);
    cfg.blockDim = dim3(THREADS);
    cfg.dynamicSmemBytes = pl.smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = pl.k_splits; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr; cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, qgemm_small_kernel<FMT>, tmX, tmW, p);
}

bool g_enabled = true;

}  // namespace
}  // namespace small

void set_small_kernel_enabled(bool on) { small::g_enabled = on; }

bool small_path_ok(const GemmArgs& a) {
    if (!small::g_enabled || a.force_generic) return false;
    if (a.W1 || a.partial_out || a.scatter.world || a.n_extra || a.post[0] || a.post[1] || a.post[2]) return false;
    if (a.M == 0 || a.N == 0 || a.K == 0) return false;
    if (((uintptr_t)a.X & 15u) || ((uintptr_t)a.W0 & 15u) || ((uintptr_t)a.Y & 3u)) return false;
    if (a.residual && (a.layout != 0 || ((uintptr_t)a.residual & 1u))) return false;
    if (a.layout == 1 && (a.D == 0 || a.D % 2u != 0u)) return false;
    uint32_t chunk = 256;
    switch (a.format) {
        case QUANT_Q4_0: case QUANT_MLX_4BIT: case QUANT_Q4_K: case QUANT_TERNARY_1_58: case QUANT_VAR_RATE_AFFINE: case QUANT_EXL3:
        case QUANT_TERNARY_ROW: break;
        case QUANT_PRISM_Q2_0: chunk = 1024; break;
        default: return false;          // the planar group-64 layout reads side planes per chunk: persistent kernel
    }
    if (a.K % chunk != 0) return false;
    // worthwhile where the persistent kernel would leave SMs idle: fewer output tiles (at its tile height) than SMs
    const uint32_t big_tiles = ((a.M + 255u) / 256u) * ((a.N + 127u) / 128u);
    int dev = 0, n_sm = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n_sm, cudaDevAttrMultiProcessorCount, dev);
    return a.M <= 256u && big_tiles < (uint32_t)n_sm;
}

cudaError_t launch_small(const GemmArgs& a, int* err, cudaStream_t stream) {
    switch (a.format) {
        case QUANT_Q4_0: return small::launch_fmt<QUANT_Q4_0>(a, err, stream);
        case QUANT_MLX_4BIT: return small::launch_fmt<QUANT_MLX_4BIT>(a, err, stream);
        case QUANT_Q4_K: return small::launch_fmt<QUANT_Q4_K>(a, err, stream);
        case QUANT_TERNARY_1_58: return small::launch_fmt<QUANT_TERNARY_1_58>(a, err, stream);
        case QUANT_VAR_RATE_AFFINE: return small::launch_fmt<QUANT_VAR_RATE_AFFINE>(a, err, stream);
        case QUANT_EXL3: return small::launch_fmt<QUANT_EXL3>(a, err, stream);
        case QUANT_TERNARY_ROW: return small::launch_fmt<QUANT_TERNARY_ROW>(a, err, stream);
        case QUANT_PRISM_Q2_0: return small::launch_fmt<QUANT_PRISM_Q2_0>(a, err, stream);
        default: return cudaErrorInvalidValue;
    }
}

}  // namespace qg
