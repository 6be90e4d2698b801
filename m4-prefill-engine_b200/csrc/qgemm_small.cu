// Few-token projection: Y[m][n] = sum_k X[m][k] * dequant(W)[n][k] for up to 128 tokens where one launch has too few
// output tiles to fill the GPU (the decode-like shapes M = 33 / 127 / 128 of the router sweep,
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
//   * one work item per CTA: K is split up to eight ways and the splits of a tile form a thread-block cluster.  Every CTA
//     writes its partial tile to a scratch buffer (which stays in L2), one cluster barrier later each CTA of the cluster
//     sums one slice of the token columns in split order -- deterministic -- and writes fp16 Y: no counters, no CTA that
//     has to add everything alone.  (Passing the partial tiles through distributed shared memory instead measured
//     slower: remote shared-memory stores ran at about 10 bytes per clock per SM.)
//
// Every mbarrier wait is bounded (ptx::mbar_wait).  The cluster barrier is a hardware barrier: every thread of every
// CTA reaches it on every path, including after a wait has given up.
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
constexpr int UNPACK_WARPS = 4;      // one per lane quadrant (a second group of four measured slower: 2080 against 550 cycles per sub-tile)
constexpr int THREADS = (UNPACK_WARPS + 2) * 32;    // warps 0-3 unpack + epilogue, warp 4 copies, warp 5 issues MMAs
constexpr int COPY_WARP = UNPACK_WARPS, MMA_WARP = UNPACK_WARPS + 1;
constexpr int MAX_T = 128;

// Development aid: with -DQS_TRACE the first CTA records clock64() stamps at its synchronisation points into a device
// array that b200_debug_small_trace copies out.  Compiled out otherwise.
#ifdef QS_TRACE
__device__ unsigned long long g_qs_trace[8][64];
#define QST(role, slot) do { if (blockIdx.x == QS_TRACE && (slot) < 64) g_qs_trace[role][slot] = clock64(); } while (0)
#else
#define QST(role, slot) do { } while (0)
#endif

struct Params {
    uint32_t M, N, K, T;
    uint32_t n_tok_tiles, n_w_tiles, k_splits, kchunks;      // kchunks: packed chunks per split
    __half* Y;
    const __half* residual;
    uint32_t layout, D;
    int* err;
    float* scratch;              // [k_splits][tiles][T][128] partial tiles (k_splits > 1)
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
// words [W, HI) of a packed row; SW: the row was staged with the 128-byte TMA swizzle (16-byte chunk index ^ row % 8, the
// planar layouts' 128-byte rows) and is read in whole chunks
template <int W, int HI, bool SW = false>
__device__ __forceinline__ void ld_words(const uint8_t* rowp, uint32_t* r, uint32_t xr = 0u) {
    if constexpr (W < HI) {
        if constexpr (W % 4 == 0 && W + 4 <= HI) {
            const uint4 v = *reinterpret_cast<const uint4*>(rowp + (SW ? ((uint32_t)(W / 4) ^ xr) << 4 : (uint32_t)W * 4u));
            r[W] = v.x; r[W + 1] = v.y; r[W + 2] = v.z; r[W + 3] = v.w;
            ld_words<W + 4, HI, SW>(rowp, r, xr);
        } else if constexpr (W % 2 == 0 && W + 2 <= HI) {
            static_assert(!SW, "swizzled rows are read in 16-byte chunks");
            const uint2 v = *reinterpret_cast<const uint2*>(rowp + W * 4);
            r[W] = v.x; r[W + 1] = v.y;
            ld_words<W + 2, HI, SW>(rowp, r, xr);
        } else {
            static_assert(!SW, "swizzled rows are read in 16-byte chunks");
            r[W] = *reinterpret_cast<const uint32_t*>(rowp + W * 4);
            ld_words<W + 1, HI, SW>(rowp, r, xr);
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
    constexpr bool SW = Cd::RAW_SWIZZLE_128;
    constexpr int MW = Cd::META_WORDS > 0 ? Cd::META_WORDS : 4;      // scale / bias words per chunk of the planar layouts

    extern __shared__ uint8_t smem_dyn[];
    ptx::launch_dependents();     // the next kernel in the stream may set itself up while this grid runs
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


    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t ks = blockIdx.x % p.k_splits;                    // == rank inside the cluster
    const uint32_t tile = blockIdx.x / p.k_splits;
    const uint32_t wt = tile % p.n_w_tiles, tt = tile / p.n_w_tiles;
    const uint32_t ksteps = p.kchunks * (uint32_t)SUBS;

    if (threadIdx.x == 0) {
        for (int i = 0; i < RAW_STAGES; i++) { ptx::mbar_init(&raw_full[i], 1); ptx::mbar_init(&raw_empty[i], UNPACK_WARPS); }
        for (int i = 0; i < A_STAGES; i++) { ptx::mbar_init(&a_full[i], 4); ptx::mbar_init(&a_empty[i], 1); }
        for (int i = 0; i < B_STAGES; i++) { ptx::mbar_init(&b_full[i], 1); ptx::mbar_init(&b_empty[i], 1); }
        ptx::mbar_init(acc_full, 1);
        *abort_flag = 0u;
        ptx::fence_barrier_init();
    }
    if (threadIdx.x == 0) QST(0, 0);
    if (warp == MMA_WARP) { ptx::tmem_alloc(tmem_holder, TMEM_COLS); ptx::tmem_relinquish(); }
    ptx::tc_fence_before_sync();
    __syncthreads();
    if (threadIdx.x == 0) QST(0, 1);
    ptx::tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_holder;
    // everything above touched only this CTA's shared and tensor memory; global memory is first touched below
    ptx::grid_dependency_wait();
    if (threadIdx.x == 0) QST(0, 2);

    if (warp == COPY_WARP) {
        // ---------------- copies: packed weight chunks run ahead of the activation tiles ----------------
        // (the packed bytes are what the launch waits for: every chunk that has a free stage is requested before the
        // activation tiles of the chunk in front of it)
        if (lane == 0) { ptx::prefetch_tensormap(&tmW); ptx::prefetch_tensormap(&tmX); }
        uint32_t rs = 0, rph = 0, bs = 0, bph = 0, raw_next = 0;
        bool ok = true;
        auto issue_raw = [&](bool block) {       // request chunk raw_next if its stage is free (block: wait for it)
            if (raw_next >= p.kchunks) return;
            bool free_now = ptx::mbar_try_wait(&raw_empty[rs], rph ^ 1u);
            if (!free_now && block) free_now = ptx::mbar_wait<32>(&raw_empty[rs], rph ^ 1u, abort_flag, p.err, 111);
            free_now = __all_sync(0xffffffffu, free_now);
            if (!free_now) { if (block) ok = false; return; }
            if (lane == 0) {
                QST(1, raw_next);
                ptx::mbar_arrive_expect_tx(&raw_full[rs], RAW_TILE_BYTES);
                ptx::tma_load_2d(sRaw + rs * RAW_TILE_BYTES, &tmW, &raw_full[rs],
                                 (int)((ks * p.kchunks + raw_next) * (ROW_BYTES / Cd::TMA_ELEM_BYTES)), (int)(wt * W_TILE));
            }
            __syncwarp();
            raw_next++;
            if (++rs == RAW_STAGES) { rs = 0; rph ^= 1u; }
        };
        for (int i = 0; i < RAW_STAGES; i++) issue_raw(false);
        for (uint32_t kc = 0; ok && kc < p.kchunks; kc++) {
            if (raw_next <= kc) issue_raw(true);              // the chunk these activation tiles belong to must be on its way
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
                issue_raw(false);                             // a packed stage may have been released meanwhile
            }
        }
    } else if (warp == MMA_WARP) {
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
            if (lane == 0) QST(2, st);
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
        const uint32_t quad = warp & 3u;                            // lane quadrant
        const uint32_t row = quad * 32u + lane;                     // weight row of the tile = tensor-memory lane
        const uint32_t lane_base = (quad * 32u) << 16;
        uint32_t rs = 0, rph = 0;
        bool ok = true;
        for (uint32_t kc = 0; ok && kc < p.kchunks; kc++) {
            // planar layouts: this chunk's scales and biases come straight from their planes in global memory, requested
            // before the wait for the packed bytes
            uint32_t meta[MW] = {};
            if (Cd::META_WORDS != 0) {
                const uint32_t n = wt * W_TILE + row;
                if (n < p.N) {
                    const uint32_t groups = (p.K / 256u) * MW;
                    const uint8_t* mp = p.meta0 + ((size_t)n * groups + (size_t)(ks * p.kchunks + kc) * MW) * 2;
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
            }
            ok = __all_sync(0xffffffffu, ptx::mbar_wait<32>(&raw_full[rs], rph, abort_flag, p.err, 115));
            if (!ok) break;
            if (threadIdx.x == 0) QST(3, kc);
            uint32_t r[ROW_BYTES / 4];
            const uint8_t* rowp = sRaw + rs * RAW_TILE_BYTES + row * ROW_BYTES;
            const uint32_t xr = row & 7u;
            ld_words<0, Cd::HDR_WORDS, SW>(rowp, r, xr);
            auto sub_tile = [&](auto S) {
                constexpr int s = decltype(S)::value;
                // step of this CTA, its stage of the A ring and the parity of that stage's use
                const uint32_t step = kc * (uint32_t)SUBS + (uint32_t)s, as = step % A_STAGES, aph = (step / A_STAGES) & 1u;
                uint32_t o[32];
                ld_words<Cd::sub_lo(s), Cd::sub_hi(s), SW>(rowp, r, xr);
                Cd::dequant64(r, s, o, meta);
                ok = __all_sync(0xffffffffu, ok && ptx::mbar_wait<32>(&a_empty[as], aph ^ 1u, abort_flag, p.err, 116));
                if (ok) {
                    ptx::tc_fence_after_sync();                      // the MMAs that read this stage have completed
                    tmem_st_x32(tmem_base + lane_base + as * A_COLS, o);
                    ptx::tmem_st_wait();
                    ptx::tc_fence_before_sync();
                    __syncwarp();
                    if (lane == 0) ptx::mbar_arrive(&a_full[as]);
                    if (threadIdx.x == 0) QST(4, step);
                }
            };
            for_each_sub(sub_tile, std::make_integer_sequence<int, SUBS>{});
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(&raw_empty[rs]);         // after the stores that consumed every loaded register
            if (++rs == RAW_STAGES) { rs = 0; rph ^= 1u; }
        }
    }

    // ---------------- partial tiles meet in the scratch buffer, the cluster shares out the sums ----------------
    if (warp < 4) {
        // the accumulator is complete once every MMA has; a failed wait sets the abort flag, the barrier is still reached
        ptx::mbar_wait<64>(acc_full, 0u, abort_flag, p.err, 117);
    }
    __syncthreads();
    if (threadIdx.x == 0) QST(0, 3);
    const bool bad = *abort_flag != 0u;
    const uint32_t n_tiles = p.n_w_tiles * p.n_tok_tiles;
    const size_t tile_floats = (size_t)p.T * W_TILE;
    if (warp < 4 && !bad) {
        ptx::tc_fence_after_sync();
        const uint32_t f = warp * 32u + lane;                       // feature row of the tile
        const uint32_t n = wt * W_TILE + f;
        float rsc = 1.0f;
        if (Cd::ROW_SCALE) rsc = n < p.N ? __half2float(p.row_scale0[n]) : 0.0f;
        const uint32_t taddr = tmem_base + ((warp * 32u) << 16) + ACC_COL;
        if (p.k_splits > 1u) {
            // [split][tile][token column][feature]: a warp's store covers 32 consecutive features of one column
            float* dst = p.scratch + ((size_t)ks * n_tiles + tile) * tile_floats + f;
            for (uint32_t c0 = 0; c0 < p.T; c0 += 16) {
                uint32_t v[16];
                ptx::tmem_ld_x16(taddr + c0, v);
                ptx::tmem_ld_wait();
#pragma unroll
                for (int j = 0; j < 16; j++)
                    __stcg(dst + (size_t)(c0 + j) * W_TILE, Cd::ROW_SCALE ? __uint_as_float(v[j]) * rsc : __uint_as_float(v[j]));
            }
        } else {
            // no split: this CTA's accumulator is the result
            const uint32_t tok0 = tt * p.T;
            for (uint32_t c0 = 0; c0 < p.T; c0 += 16) {
                uint32_t v[16];
                ptx::tmem_ld_x16(taddr + c0, v);
                ptx::tmem_ld_wait();
                if (n >= p.N) continue;
#pragma unroll
                for (int j = 0; j < 16; j++) {
                    const uint32_t tok = tok0 + c0 + j;
                    if (tok >= p.M) break;
                    float a = Cd::ROW_SCALE ? __uint_as_float(v[j]) * rsc : __uint_as_float(v[j]);
                    const size_t o = p.layout == 1 ? ((size_t)(n / p.D) * p.M + tok) * p.D + (n % p.D) : (size_t)tok * p.N + n;
                    if (p.residual) a += __half2float(p.residual[o]);
                    p.Y[o] = __float2half_rn(a);
                }
            }
        }
    }
    if (threadIdx.x == 0) QST(0, 5);
    // every partial tile of the cluster is written (release / acquire at cluster scope covers the global stores)
    cluster_sync_all();
    if (threadIdx.x == 0) QST(0, 6);
    if (!bad && p.k_splits > 1u) {
        // this CTA's token columns [ks * cols, (ks + 1) * cols): sum over the splits in split order, write fp16
        const uint32_t cols = p.T / p.k_splits;
        const float* base = p.scratch + (size_t)tile * tile_floats + (size_t)(ks * cols) * W_TILE;
        const size_t split_stride = (size_t)n_tiles * tile_floats;
        const uint32_t tok0 = tt * p.T + ks * cols;
        for (uint32_t i = threadIdx.x; i < cols * (W_TILE / 4); i += THREADS) {
            const uint32_t cl = i / (W_TILE / 4), f = (i % (W_TILE / 4)) * 4u;
            const uint32_t tok = tok0 + cl, n = wt * W_TILE + f;
            if (tok >= p.M || n >= p.N) continue;
            float4 acc = __ldcg(reinterpret_cast<const float4*>(base + (size_t)cl * W_TILE + f));
            for (uint32_t s = 1; s < p.k_splits; s++) {
                const float4 v = __ldcg(reinterpret_cast<const float4*>(base + s * split_stride + (size_t)cl * W_TILE + f));
                acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
            }
            float a[4] = {acc.x, acc.y, acc.z, acc.w};
#pragma unroll
            for (int e = 0; e < 4; e++) {
                if (n + e >= p.N) break;
                const size_t o = p.layout == 1 ? ((size_t)((n + e) / p.D) * p.M + tok) * p.D + ((n + e) % p.D) : (size_t)tok * p.N + n + e;
                if (p.residual) a[e] += __half2float(p.residual[o]);
                p.Y[o] = __float2half_rn(a[e]);
            }
        }
    }
    // ---------------- teardown ----------------
    if (threadIdx.x == 0) QST(0, 7);
    ptx::tc_fence_before_sync();
    __syncthreads();
    if (bad) {      // let copies that are still in flight land before the CTA gives its shared memory back
        const long long t0 = clock64();
        while (clock64() - t0 < 4000000LL) { }
        __syncthreads();
    }
    if (warp == MMA_WARP) { ptx::tc_fence_after_sync(); ptx::tmem_dealloc(tmem_base, TMEM_COLS); }
    if (threadIdx.x == 0) QST(0, 8);
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

// alignment slack + activation ring + packed ring + barrier block
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
    // at least 80 KB, so that no more than two CTAs share an SM: each holds 256 of the SM's 512 tensor-memory columns, and a
    // third CTA would sit in tcgen05.alloc until one of the others leaves
    pl.smem = smem_bytes<FMT>(pl.T);
    if (pl.smem < 80 * 1024) pl.smem = 80 * 1024;
    return tiles * pl.k_splits <= 65535u * 8u;
}

template <int FMT> size_t scratch_floats_fmt(const GemmArgs& a) {
    Plan pl;
    if (!make_plan<FMT>(a, pl) || pl.k_splits <= 1) return 0;
    return (size_t)pl.k_splits * pl.n_tok_tiles * pl.n_w_tiles * pl.T * W_TILE;
}

template <int FMT> cudaError_t launch_fmt(const GemmArgs& a, const Workspace& ws, cudaStream_t stream) {
    using Cd = cdc::Codec<FMT>;
    Plan pl;
    if (!make_plan<FMT>(a, pl)) return cudaErrorInvalidValue;
    if (pl.k_splits > 1 && (!ws.partial || ws.partial_floats < (size_t)pl.k_splits * pl.n_tok_tiles * pl.n_w_tiles * pl.T * W_TILE))
        return cudaErrorInvalidValue;
    const uint64_t w_row_bytes = (uint64_t)(a.K / Cd::CHUNK) * Cd::ROW_BYTES;
    CUtensorMap tmX, tmW;
    if (!make_map(&tmX, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, a.X, a.K, a.M, (uint64_t)a.K * 2, KSTEP, pl.T, CU_TENSOR_MAP_SWIZZLE_128B))
        return cudaErrorInvalidValue;
    constexpr int EB = Cd::TMA_ELEM_BYTES;
    if (!make_map(&tmW, EB == 2 ? CU_TENSOR_MAP_DATA_TYPE_UINT16 : CU_TENSOR_MAP_DATA_TYPE_UINT8, a.W0, w_row_bytes / EB, a.N, w_row_bytes,
                  Cd::ROW_BYTES / EB, W_TILE, Cd::RAW_SWIZZLE_128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE))
        return cudaErrorInvalidValue;
    Params p;
    p.M = a.M; p.N = a.N; p.K = a.K; p.T = pl.T;
    p.n_tok_tiles = pl.n_tok_tiles; p.n_w_tiles = pl.n_w_tiles; p.k_splits = pl.k_splits; p.kchunks = pl.kchunks;
    p.Y = (__half*)a.Y; p.residual = (const __half*)a.residual; p.layout = (uint32_t)a.layout; p.D = a.D ? a.D : 2;
    p.err = ws.err; p.scratch = ws.partial;
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
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = pl.k_splits; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;      // prologue may overlap the previous kernel's tail
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr; cfg.numAttrs = 2;
    return cudaLaunchKernelEx(&cfg, qgemm_small_kernel<FMT>, tmX, tmW, p);
}

int g_mode = 1;

}  // namespace
}  // namespace small

void set_small_kernel_enabled(int mode) { small::g_mode = mode; }

#ifdef QS_TRACE
extern "C" int b200_debug_small_trace(unsigned long long* out) {
    return cudaMemcpyFromSymbol(out, small::g_qs_trace, sizeof(small::g_qs_trace)) == cudaSuccess ? 0 : -1;
}
#endif

bool small_path_ok(const GemmArgs& a) {
    if (small::g_mode == 0 || a.force_generic) return false;
    if (a.W1 || a.partial_out || a.scatter.world || a.n_extra || a.post[0] || a.post[1] || a.post[2]) return false;
    if (a.M == 0 || a.N == 0 || a.K == 0) return false;
    if (((uintptr_t)a.X & 15u) || ((uintptr_t)a.W0 & 15u) || ((uintptr_t)a.Y & 3u)) return false;
    if (a.residual && (a.layout != 0 || ((uintptr_t)a.residual & 1u))) return false;
    if (a.layout == 1 && (a.D == 0 || a.D % 2u != 0u)) return false;
    uint32_t chunk = 256;
    switch (a.format) {
        case QUANT_Q4_0: case QUANT_MLX_4BIT: case QUANT_Q4_K: case QUANT_TERNARY_1_58: case QUANT_VAR_RATE_AFFINE: case QUANT_EXL3:
        case QUANT_TERNARY_ROW: case QUANT_MLX_4BIT_G64: case QUANT_MLX_4BIT_PLANAR: break;
        case QUANT_PRISM_Q2_0: chunk = 1024; break;
        default: return false;
    }
    if (a.K % chunk != 0) return false;
    // worthwhile where the persistent kernel would leave SMs idle: fewer output tiles (at its tile height) than SMs
    const uint32_t big_tiles = ((a.M + 255u) / 256u) * ((a.N + 127u) / 128u);
    int dev = 0, n_sm = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n_sm, cudaDevAttrMultiProcessorCount, dev);
    // (one token tile of up to 128 tokens: with two, every weight tile would be unpacked twice)
    if (small::g_mode == 2) return true;
    return a.M <= (uint32_t)small::MAX_T && big_tiles < (uint32_t)n_sm;
}

#define QG_SMALL_DISPATCH(EXPR)                                                            \
    switch (a.format) {                                                                    \
        case QUANT_Q4_0: { constexpr int F = QUANT_Q4_0; return EXPR; }                    \
        case QUANT_MLX_4BIT: { constexpr int F = QUANT_MLX_4BIT; return EXPR; }            \
        case QUANT_Q4_K: { constexpr int F = QUANT_Q4_K; return EXPR; }                    \
        case QUANT_TERNARY_1_58: { constexpr int F = QUANT_TERNARY_1_58; return EXPR; }    \
        case QUANT_VAR_RATE_AFFINE: { constexpr int F = QUANT_VAR_RATE_AFFINE; return EXPR; } \
        case QUANT_EXL3: { constexpr int F = QUANT_EXL3; return EXPR; }                    \
        case QUANT_TERNARY_ROW: { constexpr int F = QUANT_TERNARY_ROW; return EXPR; }      \
        case QUANT_MLX_4BIT_G64: { constexpr int F = QUANT_MLX_4BIT_G64; return EXPR; }    \
        case QUANT_MLX_4BIT_PLANAR: { constexpr int F = QUANT_MLX_4BIT_PLANAR; return EXPR; } \
        case QUANT_PRISM_Q2_0: { constexpr int F = QUANT_PRISM_Q2_0; return EXPR; }        \
        default: break;                                                                    \
    }

cudaError_t launch_small(const GemmArgs& a, const Workspace& ws, cudaStream_t stream) {
    QG_SMALL_DISPATCH(small::launch_fmt<F>(a, ws, stream))
    return cudaErrorInvalidValue;
}

size_t small_scratch_floats(const GemmArgs& a) {
    QG_SMALL_DISPATCH(small::scratch_floats_fmt<F>(a))
    return 0;
}

}  // namespace qg
