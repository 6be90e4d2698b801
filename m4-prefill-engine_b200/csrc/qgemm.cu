// Dequant-fused projection GEMM and dual gate/up SwiGLU for sm_100a.
//
//   Y[m][n] = sum_k X[m][k] * dequant(W)[n][k]
//   Y[m][n] = silu(X.Wg^T)[m][n] * (X.Wu^T)[m][n]         (SwiGLU: tiles of 64 gate rows + their 64 up rows)
//
// Replaces the reference's 64x64 simdgroup-matrix engine and its 14 entry points
// (quant_router_kernels.metal:442-927) and the Brick-3 fused SwiGLU
// (brick3_swiglu_kernels.metal:428-965) with one warp-specialised, persistent kernel:
//
//   * operands are swapped: the 128 weight rows of a tile are the UMMA "M" side, up to 256
//     tokens are the "N" side, so one unpacked weight tile feeds a 128 x T x 16 MMA;
//   * one warp streams packed weight bytes with TMA (2-D map over the raw byte matrix, one box =
//     128 rows x the bytes of 256 K-elements, ring of 2-6 stages sized from the shared memory left
//     over); one warp streams fp16 activations with TMA into 128-byte-swizzled K-major tiles; one
//     warp issues tcgen05.mma (fp16 x fp16 -> fp32 in tensor memory); 8-12 unpack warps turn packed
//     bytes into the swizzled fp16 K-major layout the MMA reads; the last 4 warps drain tensor
//     memory and write fp16.  Weight and activation tiles of one 64-element K step share a 3-deep
//     operand ring with one full/empty mbarrier pair per stage;
//   * a SwiGLU tile is 64 rows of the gate matrix plus the same 64 rows of the up matrix (two TMA
//     boxes into one packed stage), so unpacking, MMA shape and tile width are those of the plain
//     projection; the epilogue pairs each gate lane with its up lane through shared memory;
//   * two accumulator buffers in tensor memory overlap a tile's epilogue with the next tile;
//   * for few tokens the K range is split across CTAs; partial tiles meet in a scratch buffer
//     and the last CTA of a tile adds them in split order (deterministic) and writes Y.
//
// Every mbarrier wait is bounded (ptx::mbar_wait): on expiry the CTA records a code in the
// error word, stops issuing work, lets outstanding copies land, frees tensor memory and exits.
#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <unordered_map>
#include <utility>

#include "codecs.cuh"
#include "ptx.cuh"
#include "qgemm.cuh"

namespace qg {

// Development aid: with -DQG_TRACE one CTA records clock64() stamps at its synchronisation points
// (role, step, tag) into a device array that a host harness reads back.  Compiled out otherwise.
#ifdef QG_TRACE
#ifndef QG_TRACE_CTA
#define QG_TRACE_CTA 0
#endif
__device__ unsigned long long g_trace[8][256][4];
__device__ unsigned long long g_cta_ns[256][4];     // per CTA: entry, after set-up, before teardown, exit (globaltimer ns)
__device__ __forceinline__ unsigned long long gtimer() { unsigned long long t; asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t)); return t; }
#define QCTA(tag) do { if (threadIdx.x == 0 && blockIdx.x < 256u) g_cta_ns[blockIdx.x][tag] = gtimer(); } while (0)
#define QTR_(role, step, tag) do { if (blockIdx.x == QG_TRACE_CTA && (step) < 256u) g_trace[role][step][tag] = clock64(); } while (0)
#define QTRC(role, step, tag) QTR_(role, step, tag)            /* coarse: once per tile */
#if QG_TRACE >= 2
#define QTR(role, step, tag) QTR_(role, step, tag)             /* fine: once per 64-element step */
#else
#define QTR(role, step, tag) do { } while (0)
#endif
#else
#define QTR(role, step, tag) do { } while (0)
#define QTRC(role, step, tag) do { } while (0)
#define QCTA(tag) do { } while (0)
#endif

constexpr int W_TILE = 128;     // weight rows per tile = UMMA M
constexpr int KSTEP = 64;       // fp16 elements per 128-byte swizzled row
constexpr int KCHUNK = 256;     // K elements per packed-weight stage (cdc::Codec<FMT>::CHUNK; 1024 for the Prism blocks)
constexpr int MAX_RAW_STAGES = 6;   // packed-weight ring depth is chosen per launch from the shared memory left over
constexpr int SMEM_BYTES = 226 * 1024;  // dynamic shared memory of every launch
constexpr int STAGES = 3;       // ring of unpacked weight tiles (one 64-element K step each)
constexpr int MAX_B_STAGES = 4;  // ring of activation tiles: deeper, so a tile is requested three steps before its MMA
constexpr int MAX_A_STAGES = 6, PAIR_MAX_B_STAGES = 6;   // CTA-pair launches: deeper rings of smaller stages (see qgemm_kernel)
constexpr int A_TILE_BYTES = W_TILE * 128;
constexpr int TMEM_COLS = 512;
constexpr int ACC_STRIDE = 256; // tensor-memory columns per accumulator buffer

constexpr int XCHG_BYTES = 2 * 128 * 32;   // epilogue exchange area: two buffers of 16 tokens x 128 features of fp16 (row-wise
                                           // epilogue), or of 8 floats per epilogue thread (SwiGLU)
constexpr int XCHG_BYTES_F32 = XCHG_BYTES;       // fp32 staging turns over 8 tokens at a time: the same two 4 KB buffers
constexpr int GATE_ROWS = W_TILE / 2;      // SwiGLU tile: 64 gate rows on TMEM lanes 0..63, their 64 up rows on lanes 64..127

template <int FMT> struct Cfg {
    // Unpack warp groups.  With G == STAGES group g owns operand stage g (it unpacks every step with
    // step % STAGES == g); with G < STAGES group g takes the sub-tiles s with s % G == g.  G must not exceed
    // STAGES: the parity wait on a stage's "empty" barrier is only unambiguous if the waiting group is never
    // two phases ahead, which holds when its own previous wait already implied the phase before.
    static constexpr int DQ_GROUPS = cdc::Codec<FMT>::GROUPS;
    static_assert(DQ_GROUPS >= 1 && DQ_GROUPS <= STAGES, "unpack groups are bounded by the operand ring depth");
    static constexpr int CHUNK = cdc::Codec<FMT>::CHUNK;          // K elements per packed stage
    static constexpr int SUBS = CHUNK / KSTEP;                    // 64-element sub-tiles (MMA steps) per packed stage
    static_assert(STAGES == 3 && SUBS % STAGES == 1, "the unpack loop's ownership counter relies on SUBS = 1 (mod STAGES)");
    static constexpr int DQ_THREADS = 128 * DQ_GROUPS;   // arrivals that release a packed stage
    static constexpr int FILL_THREADS = 128;             // arrivals that publish an unpacked stage
    // Warp placement.  A warp's scheduler is warp % 4.  The MMA-issuing thread is back-pressured by the tensor
    // pipe with next to no queueing, so every cycle one of its few instructions waits for an issue slot is idle
    // tensor time: measured on B200, three ALU-busy warps on its scheduler stretch a 64-element step from about
    // 575 to 700 cycles, the same warps on the other schedulers cost nothing.  Scheduler 2 therefore hosts only
    // the light warps (MMA issuer = warp 2, packed-weight producer = warp 6, activation producer = warp 10, idle
    // warps behind them, and the one epilogue warp that must sit there for its TMEM lane quadrant); the unpack
    // warps take the ids with warp % 4 != 2, three per group of four ids.
    static constexpr int DQ_WARPS = DQ_THREADS / 32;
    static constexpr int QUADS = (DQ_WARPS + 2) / 3 < 3 ? 3 : (DQ_WARPS + 2) / 3;
    static constexpr int EPI_WARP0 = 4 * QUADS;
    static constexpr int THREADS = (EPI_WARP0 + 4) * 32;
};

struct Params {
    uint32_t M, N, K;
    uint32_t T;                  // tokens per tile (multiple of 16)
    uint32_t n_tok_tiles, n_w_tiles, k_splits, kchunks;   // kchunks: 256-element chunks per split
    uint32_t raw_stages, b_stage_bytes, b_stages;         // ring depth of packed weights; bytes of one activation stage (T*128); activation ring depth
    uint32_t a_stages;                                    // ring depth of unpacked weight tiles (STAGES; more for CTA pairs)
    __half* Y;
    const __half* residual;
    float* partial_out;
    uint32_t layout, H, D;
    float* ws_partial;
    uint32_t* ws_counters;
    int* err;
    // planar layouts: per-64 scale plane followed by the bias plane (meta), or one fp16 scale per row
    // grouped launch: weight tiles [0, grp_tiles[0]) belong to matrix 0 (W0 -> Y), the next grp_tiles[1] to matrix 1, ...
    uint32_t groups, grp_tiles[3], grp_N[3];
    __half* grp_Y[3];
    GemmArgs::Scatter scatter;   // fused reduce-scatter of fp32 partial sums to peer ranks (world == 0: off)
    GemmArgs::WaitRows wait_rows; // activations other ranks are still writing (flags == nullptr: off)
    uint32_t tt_shift;           // rotation of the token-tile order (fused reduce-scatter only, else 0)
    uint32_t tiles_per_owner;    // output tiles whose token rows belong to one rank (fused reduce-scatter only)
    uint32_t swiglu;             // 1: tiles are 64 gate rows (matrix 0) + their 64 up rows (matrix 1); output = silu(g) * u
    uint32_t row_epi;            // 1: outputs leave through the row-wise epilogue (16-byte stores of whole token rows)
    // per matrix of a (grouped) head-major launch: POST_ROPE rotates each head's pairs (i, i + D/2) with the table's
    // cosines and sines of the token's position; POST_Q8 writes block_q8_0 records [head][token][D/32] instead of fp16
    uint32_t grp_post[3];
    const float2* rope_table;    // [M][D/2] (cos, sin), row = token index of this launch
    uint32_t kv_tokens, kv_pos0; // POST_Q8 records go to [head][kv_tokens][D/32], this launch's token t at index kv_pos0 + t
    const uint8_t* meta0;
    const uint8_t* meta1;
    const __half* row_scale0;
    const __half* row_scale1;
};

// Packed-weight stages that fit beside the operand ring for a given activation-tile height.
template <int FMT> inline long raw_stages_fit(uint32_t T, long xchg_bytes, uint32_t b_stages, uint32_t a_stages = STAGES) {
    const long avail = (long)SMEM_BYTES - 1024 /*alignment slack*/ - 512 /*barriers*/ - xchg_bytes -
                       (long)a_stages * A_TILE_BYTES - (long)b_stages * T * 128;
    return avail / ((long)cdc::Codec<FMT>::ROW_BYTES * W_TILE);
}
// Activation ring depth: four stages when two packed-weight stages still fit beside them, else three.
template <int FMT> inline uint32_t b_stages_for(uint32_t T, long xchg_bytes) {
    return raw_stages_fit<FMT>(T, xchg_bytes, MAX_B_STAGES) >= 2 ? MAX_B_STAGES : STAGES;
}
template <int FMT> inline uint32_t raw_stages_for(uint32_t T, long xchg_bytes) {
    const long n = raw_stages_fit<FMT>(T, xchg_bytes, b_stages_for<FMT>(T, xchg_bytes));
    // (every codec fits at least one stage beside three activation stages of 256 tokens and the largest exchange area;
    // with a single stage the copy of the next chunk cannot overlap the unpacking, which only the 272-byte rows reach)
    return (uint32_t)(n < 1 ? 1 : (n > MAX_RAW_STAGES ? MAX_RAW_STAGES : n));
}
static_assert(SMEM_BYTES - 1024 - 512 - XCHG_BYTES_F32 - STAGES * A_TILE_BYTES - STAGES * 256 * 128 >= 272 * W_TILE,
              "one packed stage of the widest codec must fit in the tightest configuration");

// Loads the words [W, HI) of a packed row from shared memory into r[] with the widest aligned loads.  SW: the row
// was staged with the 128-byte TMA swizzle (16-byte chunk index ^ row % 8); such rows are read in whole chunks.
template <int W, int HI, bool SW>
__device__ __forceinline__ void ld_words(const uint8_t* rowp, uint32_t xr, uint32_t* r) {
    if constexpr (W < HI) {
        if constexpr (W % 4 == 0 && W + 4 <= HI) {
            const uint4 v = *reinterpret_cast<const uint4*>(rowp + (SW ? ((uint32_t)(W / 4) ^ xr) << 4 : (uint32_t)W * 4u));
            r[W] = v.x; r[W + 1] = v.y; r[W + 2] = v.z; r[W + 3] = v.w;
            ld_words<W + 4, HI, SW>(rowp, xr, r);
        } else if constexpr (W % 2 == 0 && W + 2 <= HI) {
            static_assert(!SW, "swizzled rows are read in 16-byte chunks");
            const uint2 v = *reinterpret_cast<const uint2*>(rowp + W * 4);
            r[W] = v.x; r[W + 1] = v.y;
            ld_words<W + 2, HI, SW>(rowp, xr, r);
        } else {
            static_assert(!SW, "swizzled rows are read in 16-byte chunks");
            r[W] = *reinterpret_cast<const uint32_t*>(rowp + W * 4);
            ld_words<W + 1, HI, SW>(rowp, xr, r);
        }
    }
}
template <int S> struct IntC { static constexpr int value = S; };
// calls f(IntC<0>{}), f(IntC<1>{}), ... in order: the sub-tiles of one packed stage, each with a compile-time index
template <class F, int... S>
__device__ __forceinline__ void for_each_sub(F& f, std::integer_sequence<int, S...>) { (f(IntC<S>{}), ...); }

struct Tile { uint32_t wt, tt, ks, id; };
__device__ __forceinline__ Tile decode_tile(uint32_t idx, const Params& p) {
    Tile t;
    t.ks = idx % p.k_splits;
    uint32_t rest = idx / p.k_splits;
    t.wt = rest % p.n_w_tiles;
    t.tt = rest / p.n_w_tiles;
    // fused reduce-scatter: rank r starts with the token rows of owner r + 1 and ends with its own, so that at any
    // time the ranks send to different owners (all ranks walking the owners in the same order would converge on one
    // owner's NVLink port at a time) and the last, local tiles overlap the tail of the remote transfers
    if (p.tt_shift) { t.tt += p.tt_shift; if (t.tt >= p.n_tok_tiles) t.tt -= p.n_tok_tiles; }
    t.id = t.tt * p.n_w_tiles + t.wt;
    return t;
}

// element (tok, n) of an output of width N_out (p.N, or the width of one matrix of a grouped launch)
__device__ __forceinline__ size_t out_index(const Params& p, uint32_t tok, uint32_t n, uint32_t N_out) {
    if (p.layout == 1) return ((size_t)(n / p.D) * p.M + tok) * p.D + (n % p.D);
    return (size_t)tok * N_out + n;
}
__device__ __forceinline__ size_t out_index(const Params& p, uint32_t tok, uint32_t n) { return out_index(p, tok, n, p.N); }

__device__ __forceinline__ float silu_mul(float g, float u) { return __fdividef(g, 1.0f + __expf(-g)) * u; }

// Adds the S partial tiles of output tile t (fp32 [S][tiles][T][128] scratch) and writes the result the way the
// launch asked for: fp16 Y (either layout, optional residual) or fp32 partial_out.  Thread i of n handles float4
// column groups i, i + n, ... of the tile's valid token rows, U of them per round.
template <int S>
__device__ __forceinline__ void splitk_fixup(const Params& p, const Tile& t, uint32_t tid, uint32_t nthreads) {
    constexpr int U = 16 / S;
    const uint32_t tok0 = t.tt * p.T;
    const uint32_t valid = tok0 < p.M ? min(p.T, p.M - tok0) : 0u;
    const uint32_t total4 = valid * (W_TILE / 4);
    const size_t split_stride = (size_t)(p.n_w_tiles * p.n_tok_tiles) * p.T * W_TILE;
    const float4* base = reinterpret_cast<const float4*>(p.ws_partial + (size_t)t.id * p.T * W_TILE);
    // grouped launch: the matrix this tile belongs to decides the output buffer and its width
    uint32_t wt_l = t.wt, Ng = p.N;
    __half* Yg = p.Y;
    if (p.groups > 1u) {
        uint32_t gi = 0;
        if (wt_l >= p.grp_tiles[0]) { wt_l -= p.grp_tiles[0]; gi = 1; if (wt_l >= p.grp_tiles[1]) { wt_l -= p.grp_tiles[1]; gi = 2; } }
        Ng = p.grp_N[gi]; Yg = p.grp_Y[gi];
    }
    const bool vec_ok = (p.layout == 1) ? (p.D % 4u == 0u) : (Ng % 4u == 0u);
    for (uint32_t i0 = tid; i0 < total4; i0 += nthreads * U) {
        float4 v[U][S];
#pragma unroll
        for (int u = 0; u < U; u++) {
            const uint32_t i = i0 + u * nthreads;
#pragma unroll
            for (int sp = 0; sp < S; sp++)
                v[u][sp] = i < total4 ? __ldcg(base + sp * (split_stride / 4) + i) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
#pragma unroll
        for (int u = 0; u < U; u++) {
            const uint32_t i = i0 + u * nthreads;
            if (i >= total4) continue;
            float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int sp = 0; sp < S; sp++) { acc[0] += v[u][sp].x; acc[1] += v[u][sp].y; acc[2] += v[u][sp].z; acc[3] += v[u][sp].w; }
            const uint32_t tok = tok0 + (i >> 5), n0 = wt_l * W_TILE + (i & 31u) * 4u;
            if (n0 >= Ng) continue;
            if (p.partial_out) {
                float* dst = p.partial_out + (size_t)tok * Ng + n0;
                if (vec_ok && n0 + 3u < Ng) *reinterpret_cast<float4*>(dst) = make_float4(acc[0], acc[1], acc[2], acc[3]);
                else
                    for (uint32_t e = 0; e < 4u && n0 + e < Ng; e++) dst[e] = acc[e];
            } else if (vec_ok && n0 + 3u < Ng) {
                const size_t o = out_index(p, tok, n0, Ng);        // n0 % 4 == 0: the four outputs are contiguous
                if (p.residual) {
                    const uint2 r = *reinterpret_cast<const uint2*>(p.residual + o);
                    const __half2 r01 = *reinterpret_cast<const __half2*>(&r.x), r23 = *reinterpret_cast<const __half2*>(&r.y);
                    acc[0] += __low2float(r01); acc[1] += __high2float(r01); acc[2] += __low2float(r23); acc[3] += __high2float(r23);
                }
                const __half2 h01 = __halves2half2(__float2half_rn(acc[0]), __float2half_rn(acc[1]));
                const __half2 h23 = __halves2half2(__float2half_rn(acc[2]), __float2half_rn(acc[3]));
                uint2 w;
                w.x = *reinterpret_cast<const uint32_t*>(&h01); w.y = *reinterpret_cast<const uint32_t*>(&h23);
                *reinterpret_cast<uint2*>(Yg + o) = w;
            } else {
                for (uint32_t e = 0; e < 4u && n0 + e < Ng; e++) {
                    const size_t o = out_index(p, tok, n0 + e, Ng);
                    Yg[o] = __float2half_rn(p.residual ? acc[e] + __half2float(p.residual[o]) : acc[e]);
                }
            }
        }
    }
}

// Row-wise epilogue of one output tile.  The accumulator comes out of tensor memory with one thread per feature (16
// token columns at a time); written out like that, a warp's store covers 32 features of one token (64 bytes of fp16) and
// a residual would be read with strided 2-byte loads.  Instead each batch of 16 tokens x 128 features is turned over
// through shared memory: the feature-owning threads deposit their values, and after one barrier among the 128 epilogue
// threads each thread moves 16-byte chunks of whole token rows -- a warp's store covers two full 256-byte rows of fp16 (or
// one 512-byte row of fp32 partial sums), which is what both HBM and NVLink want, and a residual is read the same way.
// Two buffers alternate, so one barrier per batch suffices (a buffer is rewritten only after the barrier of the batch in
// between, which every thread reaches after its reads of that buffer).
//   KIND 0: fp16 to Y            KIND 1: fp16(acc + residual) to Y
//   KIND 2: fp32 partial sums    KIND 3: fp16 partial sums          (both to `partial`, standard layout of width p.N)
// Q8_0 record of the 32 values held by four neighbouring lanes (8 each, fp16 pairs in w): fp32 amax / 127 as the scale
// (stored rounded to fp16), codes from the reciprocal of the unrounded scale, rounded half away from zero and clamped --
// the arithmetic of attn::quantize_q8_0_kernel, i.e. of the reference's quantize_kv_to_q8_0 (unified_8b_kernels.metal:118-145).
// `blk` is the record (34 bytes, 2-byte aligned), `part` this lane's quarter of it.  All 32 lanes call (shuffles).
__device__ __forceinline__ void store_q8_quarter(const uint4& w, uint8_t* blk, uint32_t part, bool write) {
    const __half2* h = reinterpret_cast<const __half2*>(&w);
    float v[8], amax = 0.0f;
#pragma unroll
    for (int e = 0; e < 4; e++) { const float2 f = __half22float2(h[e]); v[2 * e] = f.x; v[2 * e + 1] = f.y; }
#pragma unroll
    for (int e = 0; e < 8; e++) amax = fmaxf(amax, fabsf(v[e]));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
    const float d = __fdiv_rn(amax, 127.0f);
    const float id = d > 0.0f ? __fdiv_rn(1.0f, d) : 0.0f;
    if (!write) return;
    uint16_t* o = reinterpret_cast<uint16_t*>(blk);
    if (part == 0u) o[0] = __half_as_ushort(__float2half_rn(d));
#pragma unroll
    for (int e = 0; e < 4; e++) {
        int q0 = (int)roundf(__fmul_rn(v[2 * e], id)), q1 = (int)roundf(__fmul_rn(v[2 * e + 1], id));
        q0 = max(-128, min(127, q0)); q1 = max(-128, min(127, q1));
        o[1 + part * 4u + e] = (uint16_t)((uint32_t)(uint8_t)(int8_t)q0 | ((uint32_t)(uint8_t)(int8_t)q1 << 8));
    }
}

constexpr uint32_t POST_ROPE = 1u, POST_Q8 = 2u;

template <int KIND>
__device__ __forceinline__ void row_epilogue(const Params& p, uint8_t* stage, uint32_t& batch_ctr, uint32_t taddr, uint32_t et,
                                             uint32_t tok0, uint32_t valid, float rsc, bool row_scale, uint32_t n_tile0, uint32_t Ng,
                                             __half* Yg, void* partial) {
    constexpr bool F32 = KIND == 1 || KIND == 2;    // staged as fp32 (the residual is added before the one fp16 rounding)
    constexpr int CH = F32 ? 4 : 8;                 // elements per 16-byte chunk of the staging buffer
    constexpr int CPR = W_TILE / CH;                // chunks per token row of the tile
    constexpr int ROWS = 128 / CPR;                 // token rows the 128 threads cover per pass
    constexpr int TOK = F32 ? 8 : 16;               // token rows turned over per barrier: one buffer is 4 KB either way, so the
                                                    // exchange area stays at 8 KB and the operand rings keep their depth
    constexpr int PASSES = TOK / ROWS;
    constexpr int BUF = TOK * W_TILE * (F32 ? 4 : 2);
    static_assert(2 * BUF <= XCHG_BYTES, "two staging buffers fit the exchange area");
    const uint32_t chunk = et % CPR, jrow = et / CPR;
    const uint32_t n = n_tile0 + chunk * CH;
    const bool n_ok = n < Ng;
    size_t col_base, tok_stride;
    if (KIND >= 2) { col_base = n; tok_stride = p.N; }
    else if (p.layout == 1) { col_base = (size_t)(n / p.D) * p.M * p.D + (n % p.D); tok_stride = p.D; }
    else { col_base = n; tok_stride = Ng; }
    col_base += (size_t)tok0 * tok_stride;
    for (uint32_t c0 = 0; c0 < p.T; c0 += 16) {
        uint2 res[16 / ROWS];
        if (KIND == 1) {             // requested before the accumulator is read: the latency hides behind the turn-over
#pragma unroll
            for (int h = 0; h < 16 / ROWS; h++) {
                const uint32_t tok = c0 + jrow + h * ROWS;
                res[h] = (n_ok && tok < valid) ? __ldg(reinterpret_cast<const uint2*>(p.residual + col_base + (size_t)tok * tok_stride))
                                               : make_uint2(0u, 0u);
            }
        }
        uint32_t v[16];
        ptx::tmem_ld_x16(taddr + c0, v);
        ptx::tmem_ld_wait();
#pragma unroll
        for (int part = 0; part < 16 / TOK; part++, batch_ctr++) {
            uint8_t* buf = stage + (batch_ctr & 1u) * BUF;
            if (F32) {
                float* b = reinterpret_cast<float*>(buf) + et;
#pragma unroll
                for (int j = 0; j < TOK; j++) {
                    const float f = __uint_as_float(v[part * TOK + j]);
                    b[j * W_TILE] = row_scale ? f * rsc : f;
                }
            } else {
                __half* b = reinterpret_cast<__half*>(buf) + et;
#pragma unroll
                for (int j = 0; j < TOK; j++) {
                    const float f = __uint_as_float(v[part * TOK + j]);
                    b[j * W_TILE] = __float2half_rn(row_scale ? f * rsc : f);
                }
            }
            ptx::bar_sync(2, 128);
#pragma unroll
            for (int h = 0; h < PASSES; h++) {
                const uint32_t j = jrow + h * ROWS, tok = c0 + part * TOK + j;
                if (!n_ok || tok >= valid) continue;
                const uint4 w = reinterpret_cast<const uint4*>(buf)[j * CPR + chunk];
                if (KIND == 2) {
                    *reinterpret_cast<uint4*>(reinterpret_cast<float*>(partial) + col_base + (size_t)tok * tok_stride) = w;
                } else if (KIND == 3) {
                    *reinterpret_cast<uint4*>(reinterpret_cast<__half*>(partial) + col_base + (size_t)tok * tok_stride) = w;
                } else if (KIND == 1) {
                    const uint2 rs = res[part * PASSES + h];
                    const __half2 r01 = *reinterpret_cast<const __half2*>(&rs.x), r23 = *reinterpret_cast<const __half2*>(&rs.y);
                    const __half2 h01 = __floats2half2_rn(__uint_as_float(w.x) + __low2float(r01), __uint_as_float(w.y) + __high2float(r01));
                    const __half2 h23 = __floats2half2_rn(__uint_as_float(w.z) + __low2float(r23), __uint_as_float(w.w) + __high2float(r23));
                    uint2 o;
                    o.x = *reinterpret_cast<const uint32_t*>(&h01); o.y = *reinterpret_cast<const uint32_t*>(&h23);
                    *reinterpret_cast<uint2*>(Yg + col_base + (size_t)tok * tok_stride) = o;
                } else {
                    *reinterpret_cast<uint4*>(Yg + col_base + (size_t)tok * tok_stride) = w;
                }
            }
        }
    }
}

// KIND 0 with the K/V-cache post-operations of a head-major projection fused in: the staged fp16 row (exactly what the
// plain epilogue would have written) is rotated (POST_ROPE) and / or compressed to Q8_0 (POST_Q8) by the row-moving
// threads.  A thread's 8 features lie in one half of one head; their rotation partners are the chunk D/16 away in the
// same staged row, and the 32 values of a Q8_0 record are those of four neighbouring lanes.
__device__ __forceinline__ void row_epilogue_kv(const Params& p, uint8_t* stage, uint32_t& batch_ctr, uint32_t taddr, uint32_t et,
                                                uint32_t tok0, uint32_t valid, uint32_t n_tile0, uint32_t Ng, __half* Yg, uint32_t post) {
    constexpr int CPR = W_TILE / 8, ROWS = 128 / CPR, PASSES = 16 / ROWS, BUF = 16 * W_TILE * 2;
    const uint32_t chunk = et % CPR, jrow = et / CPR;
    const uint32_t n = n_tile0 + chunk * 8u;
    const bool n_ok = n < Ng;
    const uint32_t half_d = p.D / 2u, head = n / p.D, f = n % p.D;          // f: first of the 8 features inside its head
    const bool upper = f >= half_d;
    const uint32_t partner = chunk ^ (half_d / 8u);
    const size_t col_base = ((size_t)head * p.M + tok0) * p.D + f;          // fp16 output [head][token][D]
    for (uint32_t c0 = 0; c0 < p.T; c0 += 16, batch_ctr++) {
        uint8_t* buf = stage + (batch_ctr & 1u) * BUF;
        uint32_t v[16];
        ptx::tmem_ld_x16(taddr + c0, v);
        ptx::tmem_ld_wait();
        __half* b = reinterpret_cast<__half*>(buf) + et;
#pragma unroll
        for (int j = 0; j < 16; j++) b[j * W_TILE] = __float2half_rn(__uint_as_float(v[j]));
        ptx::bar_sync(2, 128);
#pragma unroll
        for (int h = 0; h < PASSES; h++) {
            const uint32_t j = jrow + h * ROWS, tok = c0 + j;
            const bool ok = n_ok && tok < valid;
            uint4 w = reinterpret_cast<const uint4*>(buf)[j * CPR + chunk];
            if (post & POST_ROPE) {
                const uint4 pw = reinterpret_cast<const uint4*>(buf)[j * CPR + partner];
                const uint32_t trow = ok ? tok0 + tok : 0u;
                const float4* tab = reinterpret_cast<const float4*>(p.rope_table + (size_t)trow * half_d + (f % half_d));
                const __half2* hx = reinterpret_cast<const __half2*>(&w);
                const __half2* hy = reinterpret_cast<const __half2*>(&pw);
                uint4 o;
                __half2* ho = reinterpret_cast<__half2*>(&o);
#pragma unroll
                for (int e = 0; e < 4; e++) {
                    const float4 cs = __ldg(tab + e);                       // (cos, sin) of two neighbouring frequencies
                    const float2 x = __half22float2(hx[e]), y = __half22float2(hy[e]);
                    // lower half: a*c - b*s with (a, b) = (x, y); upper half: b*c + a*s with (a, b) = (y, x)
                    const float r0 = upper ? __fmaf_rn(x.x, cs.x, __fmul_rn(y.x, cs.y)) : __fmaf_rn(x.x, cs.x, -__fmul_rn(y.x, cs.y));
                    const float r1 = upper ? __fmaf_rn(x.y, cs.z, __fmul_rn(y.y, cs.w)) : __fmaf_rn(x.y, cs.z, -__fmul_rn(y.y, cs.w));
                    ho[e] = __floats2half2_rn(r0, r1);
                }
                w = o;
            }
            if (post & POST_Q8) {
                // record (head, token, f / 32): 34 bytes each, [head][token][D/32]
                uint8_t* blk = reinterpret_cast<uint8_t*>(Yg) + (((size_t)head * p.kv_tokens + p.kv_pos0 + (ok ? tok0 + tok : 0u)) * (p.D / 32u) + f / 32u) * 34u;
                store_q8_quarter(w, blk, chunk & 3u, ok);
            } else if (ok) {
                *reinterpret_cast<uint4*>(Yg + col_base + (size_t)tok * p.D) = w;
            }
        }
    }
}

// RESID: the launch adds a residual in the epilogue (its prefetch ring costs registers the plain launch should not pay for)
// PAIR: the launch runs as clusters of two CTAs whose tensor cores work on one 256-row MMA (cta_group::2).  CTA r of a
// pair unpacks its own weight tile (rows of tile 2 i + r) into its own shared memory and loads tokens 128 r .. 128 r + 127
// of the 256-token tile; the even CTA's MMA warp issues 256 x 256 x 16 MMAs that read A from both CTAs and each half of B
// from the CTA that holds it, and every CTA finds the accumulator of its own 128 rows in its own tensor memory, so the
// epilogue is that of the single-CTA kernel.  Per SM and 64-element step the MMAs then read 32 KB of shared memory instead
// of 48 KB and TMA writes 16 KB instead of 32 KB -- with one CTA per MMA the shared-memory pipe, not the tensor pipe, bounds
// the step (measured: tensor-core operand reads plus unpack stores and loads keep it busy 98 % of the active cycles).
//   "full" barriers of the operand rings and the accumulator's "empty" barriers live in the even CTA: the odd CTA's unpack
//   and epilogue warps arrive there remotely, and a relay warp forwards the completion of the odd CTA's activation loads;
//   "empty" / accumulator-"full" arrivals are tcgen05.commit multicasts to the barrier at the same offset in both CTAs.
template <int FMT, bool RESID, bool PAIR>
__global__ void __launch_bounds__(Cfg<FMT>::THREADS, 1)
qgemm_kernel(const __grid_constant__ CUtensorMap tmX, const __grid_constant__ CUtensorMap tmW0,
             const __grid_constant__ CUtensorMap tmW1, const __grid_constant__ CUtensorMap tmW2, const Params p) {
    using C = Cfg<FMT>;
    using Cd = cdc::Codec<FMT>;
    static_assert(!PAIR || (C::EPI_WARP0 > 14 && C::DQ_WARPS == 12), "the pair kernel uses the idle warp 14 as its relay");
    constexpr int ROW_BYTES = Cd::ROW_BYTES;
    constexpr int RAW_TILE_BYTES = ROW_BYTES * W_TILE;

    extern __shared__ uint8_t smem_dyn[];
    ptx::launch_dependents();     // the next projection in the stream may set itself up on SMs this grid leaves idle
    QCTA(0);
    const uint32_t pad = (1024u - (ptx::smem_u32(smem_dyn) & 1023u)) & 1023u;
    uint8_t* sB = smem_dyn + pad;
    uint8_t* sA = sB + p.b_stages * p.b_stage_bytes;
    uint8_t* sRaw = sA + p.a_stages * A_TILE_BYTES;
    uint64_t* bars = reinterpret_cast<uint64_t*>(sRaw + p.raw_stages * RAW_TILE_BYTES);
    uint64_t* raw_full = bars;
    uint64_t* raw_empty = raw_full + MAX_RAW_STAGES;
    // Two operand rings with their own full/empty pairs.  The activation ring is one stage deeper than the
    // unpacked-weight ring: an activation tile comes from L2 / HBM and has to be requested about three steps
    // before its MMA for the load latency to stay off the critical path when the inputs are not L2-resident
    // (with a shared three-deep ring the request could only go out two steps ahead).
    uint64_t* a_full = raw_empty + MAX_RAW_STAGES;      // unpacked weight tile published (one arrival per unpack warp)
    uint64_t* a_empty = a_full + MAX_A_STAGES;          // ... consumed (one tcgen05.commit)
    uint64_t* b_full = a_empty + MAX_A_STAGES;          // activation tile landed (producer's arrival + TMA byte count)
    uint64_t* b_empty = b_full + PAIR_MAX_B_STAGES;     // ... consumed (one tcgen05.commit)
    uint64_t* tm_full = b_empty + PAIR_MAX_B_STAGES;
    uint64_t* tm_empty = tm_full + 2;
    uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(tm_empty + 2);
    volatile uint32_t* abort_flag = tmem_holder + 1;
    volatile uint32_t* last_flag = tmem_holder + 2;
    float4* xchg = reinterpret_cast<float4*>(reinterpret_cast<uint8_t*>(bars) + 512);   // epilogue exchange area (16-byte aligned)

    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t pair_rank = PAIR ? ptx::cluster_ctarank() : 0u;     // 0: the CTA whose MMA warp issues for the pair
    // work items: output tiles (x K splits), or for a pair launch pairs of weight tiles that share a token tile
    const uint32_t total_tiles = PAIR ? (p.n_w_tiles / 2u) * p.n_tok_tiles : p.n_w_tiles * p.n_tok_tiles * p.k_splits;
    const uint32_t first_tile = PAIR ? (blockIdx.x >> 1) : blockIdx.x, tile_stride = PAIR ? (gridDim.x >> 1) : gridDim.x;
    auto tile_of = [&](uint32_t idx) {
        if (!PAIR) return decode_tile(idx, p);
        Tile t;
        const uint32_t n_wp = p.n_w_tiles / 2u;
        t.ks = 0u; t.wt = 2u * (idx % n_wp) + pair_rank; t.tt = idx / n_wp;
        if (p.tt_shift) { t.tt += p.tt_shift; if (t.tt >= p.n_tok_tiles) t.tt -= p.n_tok_tiles; }
        t.id = t.tt * p.n_w_tiles + t.wt;
        return t;
    };
    const uint32_t ksteps = p.kchunks * (uint32_t)C::SUBS;
    const uint32_t b_rows = PAIR ? p.T / 2u : p.T;                      // token rows of the activation tile this CTA loads

    if (threadIdx.x == 0) {
        // pair launch: the even CTA's "full" barriers also count the odd CTA's arrivals (unpack warps, relay, epilogue warps)
        const uint32_t both = (PAIR && pair_rank == 0u) ? 2u : 1u;
        for (int i = 0; i < MAX_RAW_STAGES; i++) { ptx::mbar_init(&raw_full[i], 1); ptx::mbar_init(&raw_empty[i], C::DQ_THREADS / 32); }
        for (int i = 0; i < MAX_A_STAGES; i++) { ptx::mbar_init(&a_full[i], both * (C::FILL_THREADS / 32)); ptx::mbar_init(&a_empty[i], 1); }
        for (int i = 0; i < PAIR_MAX_B_STAGES; i++) { ptx::mbar_init(&b_full[i], both); ptx::mbar_init(&b_empty[i], 1); }
        for (int i = 0; i < 2; i++) { ptx::mbar_init(&tm_full[i], 1); ptx::mbar_init(&tm_empty[i], both * 4u); }
        *abort_flag = 0u;
        *last_flag = 0u;
        ptx::fence_barrier_init();
    }
    if (warp == 2) {
        if (PAIR) { ptx::tmem_alloc_pair(tmem_holder, TMEM_COLS); ptx::tmem_relinquish_pair(); }
        else { ptx::tmem_alloc(tmem_holder, TMEM_COLS); ptx::tmem_relinquish(); }
    }
    ptx::tc_fence_before_sync();
    __syncthreads();
    if (PAIR) ptx::cluster_sync_all();        // both CTAs' barriers are initialised before either arrives on the other's
    ptx::tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_holder;
    // Everything above touched only this CTA's shared and tensor memory; global memory (inputs another kernel may
    // still be writing, the split-K scratch the previous launch may still be using) is first touched below.
    ptx::grid_dependency_wait();
    if (threadIdx.x == 0) QTRC(7, 0u, 0);
    QCTA(1);

    const uint32_t wq = warp & 3u, wg = warp >> 2;
    const bool pre_epi = warp < (uint32_t)C::EPI_WARP0;
    // unpack warp index among the ids with warp % 4 != 2 (meaningless for the others)
    const uint32_t uw = wg * 3u + (wq == 3u ? 2u : wq);
    if (pre_epi && wq == 2u && wg == 1u) {
        // ---------------- packed-weight producer ----------------
        // The whole warp walks the loop (only lane 0 issues): a lone lane looping while its 31 siblings
        // already sit at the final barrier gets scheduled far less often than a converged warp.
        if (lane == 0) {
            ptx::prefetch_tensormap(&tmW0);
            if (p.swiglu || p.groups > 1u) ptx::prefetch_tensormap(&tmW1);
            if (p.groups > 2u) ptx::prefetch_tensormap(&tmW2);
        }
        uint32_t rs = 0, rph = 0, wtr = 0;
        (void)wtr;
        bool ok = true;
        for (uint32_t idx = first_tile; ok && idx < total_tiles; idx += tile_stride) {
            const Tile t = tile_of(idx);
            for (uint32_t kc = 0; kc < p.kchunks; kc++) {
                ok = __all_sync(0xffffffffu, ptx::mbar_wait<64>(&raw_empty[rs], rph ^ 1u, abort_flag, p.err, 101));
                if (!ok) break;
                if (lane == 0) {
                    QTR(0, wtr, 0);
                    ptx::mbar_arrive_expect_tx(&raw_full[rs], RAW_TILE_BYTES);
                    const int x = (int)((t.ks * p.kchunks + kc) * (ROW_BYTES / Cd::TMA_ELEM_BYTES));    // in elements of the map
                    if (p.swiglu) {     // the maps of a SwiGLU launch have 64-row boxes: gate rows, then the same rows of up
                        const int y = (int)(t.wt * GATE_ROWS);
                        ptx::tma_load_2d(sRaw + rs * RAW_TILE_BYTES, &tmW0, &raw_full[rs], x, y);
                        ptx::tma_load_2d(sRaw + rs * RAW_TILE_BYTES + GATE_ROWS * ROW_BYTES, &tmW1, &raw_full[rs], x, y);
                    } else if (p.groups > 1u) {
                        // grouped launch: this weight tile belongs to one of up to three matrices
                        uint32_t wl = t.wt;
                        const CUtensorMap* tm = &tmW0;
                        if (wl >= p.grp_tiles[0]) { wl -= p.grp_tiles[0]; tm = &tmW1; if (wl >= p.grp_tiles[1]) { wl -= p.grp_tiles[1]; tm = &tmW2; } }
                        ptx::tma_load_2d(sRaw + rs * RAW_TILE_BYTES, tm, &raw_full[rs], x, (int)(wl * W_TILE));
                    } else {
                        ptx::tma_load_2d(sRaw + rs * RAW_TILE_BYTES, &tmW0, &raw_full[rs], x, (int)(t.wt * W_TILE));
                    }
                    QTR(0, wtr, 1); wtr++;
                }
                __syncwarp();
                if (++rs == p.raw_stages) { rs = 0; rph ^= 1u; }
            }
        }
    } else if (pre_epi && wq == 2u && wg == 2u) {
        // ---------------- activation producer ----------------
        if (lane == 0) ptx::prefetch_tensormap(&tmX);
        uint32_t bs = 0, bph = 0, xtr = 0;
        (void)xtr;
        bool ok = true;
        uint32_t rows_seen = 0;               // bit o: owner o's rows are known to be there
        for (uint32_t idx = first_tile; ok && idx < total_tiles; idx += tile_stride) {
            const Tile t = tile_of(idx);
            const uint32_t k0 = t.ks * p.kchunks * (uint32_t)C::CHUNK;
            if (p.wait_rows.flags) {
                // rows this CTA is about to load: wait until their owners have written them (system-scope acquire, then the
                // proxy fence that orders the TMA reads behind it)
                const uint32_t r0 = t.tt * p.T + pair_rank * b_rows, r1 = min(r0 + b_rows, p.M) - 1u;
                for (uint32_t o = r0 / p.wait_rows.rows; ok && o <= r1 / p.wait_rows.rows; o++) {
                    if ((rows_seen >> o) & 1u) continue;
                    const long long t0 = clock64();
                    for (;;) {
                        uint32_t v;
                        asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p.wait_rows.flags + o) : "memory");
                        if ((int32_t)(v - p.wait_rows.epoch) >= 0) break;
                        if (*abort_flag || clock64() - t0 > p.wait_rows.limit_cycles) {
                            *abort_flag = 1u;
                            if (p.err) atomicCAS(p.err, 0, 110);
                            ok = false;
                            break;
                        }
                        __nanosleep(100);
                    }
                    rows_seen |= 1u << o;
                }
                asm volatile("fence.proxy.async.global;" ::: "memory");
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
            }
            for (uint32_t ks = 0; ks < ksteps; ks++) {
                ok = __all_sync(0xffffffffu, ptx::mbar_wait<32>(&b_empty[bs], bph ^ 1u, abort_flag, p.err, 102));
                if (!ok) break;
                if (lane == 0) {
                    QTR(1, xtr, 0);
                    ptx::mbar_arrive_expect_tx(&b_full[bs], b_rows * 128u);
                    ptx::tma_load_2d(sB + bs * p.b_stage_bytes, &tmX, &b_full[bs], (int)(k0 + ks * KSTEP), (int)(t.tt * p.T + pair_rank * b_rows));
                    QTR(1, xtr, 1); xtr++;
                }
                __syncwarp();
                if (++bs == p.b_stages) { bs = 0; bph ^= 1u; }
            }
        }
    } else if (PAIR && pair_rank == 1u && warp == 14u) {
        // ---------------- relay (odd CTA): activation tile landed here -> one arrival on the even CTA's barrier ----------------
        uint32_t bs = 0, bph = 0;
        bool ok = true;
        for (uint32_t idx = first_tile; ok && idx < total_tiles; idx += tile_stride) {
            for (uint32_t ks = 0; ks < ksteps; ks++) {
                ok = __all_sync(0xffffffffu, ptx::mbar_wait(&b_full[bs], bph, abort_flag, p.err, 109));
                if (!ok) break;
                if (lane == 0) ptx::mbar_arrive_cluster(&b_full[bs], 0u);
                __syncwarp();
                if (++bs == p.b_stages) { bs = 0; bph ^= 1u; }
            }
        }
    } else if (warp == 2 && (!PAIR || pair_rank == 0u)) {
        // ---------------- MMA issuer ----------------
        const uint32_t idesc = ptx::umma_idesc_f16(PAIR ? 2 * W_TILE : W_TILE, p.T);
        // operand descriptors differ between stages only in the 14-bit start-address field
        const uint64_t desc_hi = ptx::umma_desc_k_sw128(0u);
        const uint32_t a_lo0 = (ptx::smem_u32(sA) & 0x3FFFFu) >> 4, b_lo0 = (ptx::smem_u32(sB) & 0x3FFFFu) >> 4;
        uint32_t st = 0, sph = 0, bst = 0, bsph = 0, it = 0, mtr = 0;
        (void)mtr;
        bool ok = true;
        for (uint32_t idx = first_tile; ok && idx < total_tiles; idx += tile_stride, it++) {
            const uint32_t buf = it & 1u;
            ok = __all_sync(0xffffffffu, PAIR ? ptx::mbar_wait_cluster(&tm_empty[buf], ((it >> 1) & 1u) ^ 1u, abort_flag, p.err, 103)
                                                   : ptx::mbar_wait(&tm_empty[buf], ((it >> 1) & 1u) ^ 1u, abort_flag, p.err, 103));
            if (!ok) break;
            ptx::tc_fence_after_sync();
            if (lane == 0) QTRC(2, 200u + it, 0);
            for (uint32_t ks = 0; ks < ksteps; ks++) {
                if (lane == 0) QTR(2, mtr, 0);
                // (no tcgen05 fence here: the stage was written by TMA and by generic stores that were
                // followed by fence.proxy.async; the mbarrier acquire orders them before the MMA's reads)
                // (the vote keeps the warp converged for elect.sync even if a wait gives up)
                if (PAIR) ok = __all_sync(0xffffffffu, ptx::mbar_wait_cluster(&a_full[st], sph, abort_flag, p.err, 104) &&
                                                           ptx::mbar_wait_cluster(&b_full[bst], bsph, abort_flag, p.err, 105));
                else ok = __all_sync(0xffffffffu, ptx::mbar_wait(&a_full[st], sph, abort_flag, p.err, 104) &&
                                                      ptx::mbar_wait(&b_full[bst], bsph, abort_flag, p.err, 105));
                if (!ok) break;
                if (ptx::elect_one()) {
                    QTR(2, mtr, 2);
                    const uint64_t bdesc = desc_hi | (uint64_t)(b_lo0 + bst * (p.b_stage_bytes >> 4));
                    const uint64_t adesc = desc_hi | (uint64_t)(a_lo0 + st * (A_TILE_BYTES >> 4));
                    const uint32_t dcol = tmem_base + buf * ACC_STRIDE;
                    if (PAIR) {
#pragma unroll
                        for (int kk = 0; kk < KSTEP / 16; kk++)
                            ptx::umma_pair_f16_ss(dcol, adesc + 2 * kk, bdesc + 2 * kk, idesc, (ks | (uint32_t)kk) != 0u);
                        ptx::umma_pair_commit(&a_empty[st]);
                        ptx::umma_pair_commit(&b_empty[bst]);
                    } else {
#pragma unroll
                        for (int kk = 0; kk < KSTEP / 16; kk++)
                            ptx::umma_f16_ss(dcol, adesc + 2 * kk, bdesc + 2 * kk, idesc, (ks | (uint32_t)kk) != 0u);
                        ptx::umma_commit(&a_empty[st]);
                        ptx::umma_commit(&b_empty[bst]);
                    }
                    QTR(2, mtr, 3); mtr++;
                }
                __syncwarp();
                if (++st == p.a_stages) { st = 0; sph ^= 1u; }
                if (++bst == p.b_stages) { bst = 0; bsph ^= 1u; }
            }
            if (ok && ptx::elect_one()) {      // same lane as the MMAs
                if (PAIR) ptx::umma_pair_commit(&tm_full[buf]); else ptx::umma_commit(&tm_full[buf]);
                QTRC(2, 200u + it, 1);
            }
            __syncwarp();
        }
    } else if (pre_epi && wq != 2u && uw < (uint32_t)C::DQ_WARPS) {
        // ---------------- unpack warps: packed bytes -> swizzled fp16 K-major tile ----------------
        constexpr int G = C::DQ_GROUPS;
        const uint32_t dq = uw * 32u + lane;                  // 0 .. DQ_THREADS-1
        const uint32_t grp = dq >> 7;                         // sub-tile phase this warp group unpacks
        const uint32_t row = dq & 127;                        // weight row inside the tile
        // which matrix the row comes from, and its row there (SwiGLU tiles hold 64 rows of each)
        const uint32_t mat = p.swiglu ? (row >> 6) : 0u;
        const uint32_t mrow_in_tile = p.swiglu ? (row & 63u) : row;
        const uint32_t row_off = (row >> 3) * 1024 + (row & 7) * 128, xr = row & 7;
        uint32_t rs = 0, rph = 0, kn = 0;                     // kn: running 64-element step of this CTA
        uint32_t km = 0, own_ph = 0;                          // (kn / 4) % STAGES; phase of the group's next operand stage
        uint32_t own_st = grp;                                // ... and that stage: the group's steps g, g + 3, ... use stages (g + 3 j) % a_stages
        bool ok = true;
        for (uint32_t idx = first_tile; ok && idx < total_tiles; idx += tile_stride) {
            const Tile t = tile_of(idx);
            // META_WORDS / 2 words of scales and as many of biases per chunk: one group per 64 elements (4 words)
            // or per 32 elements (8 words); the bias plane follows the scale plane
            constexpr int MW = Cd::META_WORDS > 0 ? Cd::META_WORDS : 4;
            uint32_t meta_next[MW] = {};
            auto load_meta = [&](uint32_t kc, uint32_t (&m)[MW]) {
                const uint32_t n = t.wt * (p.swiglu ? GATE_ROWS : W_TILE) + mrow_in_tile;
                if (n < p.N) {
                    const uint32_t groups = (p.K / 256) * MW;
                    const uint8_t* mp = (mat == 0 ? p.meta0 : p.meta1) + ((size_t)n * groups + (size_t)(t.ks * p.kchunks + kc) * MW) * 2;
                    const uint8_t* bp = mp + (size_t)p.N * groups * 2;
                    if (MW == 4) {
                        const uint2 sc = __ldg(reinterpret_cast<const uint2*>(mp));
                        const uint2 bi = __ldg(reinterpret_cast<const uint2*>(bp));
                        m[0] = sc.x; m[1] = sc.y; m[2] = bi.x; m[3] = bi.y;
                    } else {
                        const uint4 sc = __ldg(reinterpret_cast<const uint4*>(mp));
                        const uint4 bi = __ldg(reinterpret_cast<const uint4*>(bp));
                        m[0] = sc.x; m[1] = sc.y; m[2] = sc.z; m[3] = sc.w;
                        m[MW - 4] = bi.x; m[MW - 3] = bi.y; m[MW - 2] = bi.z; m[MW - 1] = bi.w;
                    }
                }
            };
            (void)load_meta; (void)meta_next;
            for (uint32_t kc = 0; ok && kc < p.kchunks; kc++) {
                // scales and biases kept outside the packed rows come straight from global memory, one chunk
                // ahead of their use so the latency hides behind the unpacking of the current chunk
                uint32_t meta[MW] = {};
                if (Cd::META_WORDS != 0) {
                    if (kc == 0) load_meta(0u, meta_next);
#pragma unroll
                    for (int i = 0; i < MW; i++) meta[i] = meta_next[i];
                    if (kc + 1 < p.kchunks) load_meta(kc + 1, meta_next);
                }
                ok = __all_sync(0xffffffffu, ptx::mbar_wait<32>(&raw_full[rs], rph, abort_flag, p.err, 106));
                if (!ok) break;
                if (row == 0) QTR(3, (kn >> 2) * 2 + grp, 0);
                // Only the words a sub-tile needs are loaded, right before it is unpacked: a group handles one or
                // two of a chunk's four sub-tiles, and short-lived inputs leave the registers to the 32 outputs.
                uint32_t r[ROW_BYTES / 4];
                const uint8_t* rowp = sRaw + rs * RAW_TILE_BYTES + row * ROW_BYTES;
                constexpr bool SW = Cd::RAW_SWIZZLE_128;
                ld_words<0, Cd::HDR_WORDS, SW>(rowp, xr, r);
                auto sub_tile = [&](auto S) {
                    constexpr int s = decltype(S)::value;
                    // owner of this 64-element step: with G == STAGES the group that owns operand stage
                    // (step % STAGES); the chunk counter km = (kn / SUBS) % 3 stands in for kn % 3 (SUBS = 1 mod 3)
                    uint32_t own = (G == STAGES) ? km + (uint32_t)(s % STAGES) : (uint32_t)(s % G);
                    if (G == STAGES && own >= (uint32_t)STAGES) own -= (uint32_t)STAGES;
                    if (own == grp) {
                        uint32_t o[32];
                        ld_words<Cd::sub_lo(s), Cd::sub_hi(s), SW>(rowp, xr, r);
                        Cd::dequant64(r, s, o, meta);
                        if (row == 0) QTR(4 + grp, kn + s, 0);
                        uint32_t as, aph;
                        if (G == STAGES) {      // three stages: always the group's own; deeper rings (CTA pairs): every third stage in turn
                            as = own_st; aph = own_ph;
                            own_st += (uint32_t)STAGES;
                            if (own_st >= p.a_stages) { own_st -= p.a_stages; own_ph ^= 1u; }
                        }
                        else { const uint32_t step = kn + s; as = step % STAGES; aph = (step / STAGES) & 1u; }
                        ok = __all_sync(0xffffffffu, ok && ptx::mbar_wait<32>(&a_empty[as], aph ^ 1u, abort_flag, p.err, 107));
                        if (row == 0) QTR(4 + grp, kn + s, 1);
                        if (ok) {
                            uint8_t* dst = sA + as * A_TILE_BYTES + row_off;
#pragma unroll
                            for (int c = 0; c < 8; c++)
                                *reinterpret_cast<uint4*>(dst + ((c ^ xr) << 4)) = make_uint4(o[4 * c], o[4 * c + 1], o[4 * c + 2], o[4 * c + 3]);
                            ptx::fence_proxy_async_smem();
                            __syncwarp();                      // every lane's stores are fenced; one arrival per warp
                            if (lane == 0) { if (PAIR && pair_rank == 1u) ptx::mbar_arrive_cluster(&a_full[as], 0u); else ptx::mbar_arrive(&a_full[as]); }
                            if (row == 0) QTR(4 + grp, kn + s, 2);
                        }
                    }
                };
                for_each_sub(sub_tile, std::make_integer_sequence<int, C::SUBS>{});
                km = (km == (uint32_t)STAGES - 1u) ? 0u : km + 1u;
                kn += (uint32_t)C::SUBS;
                // Release the packed stage only now: the stores above consumed every register loaded
                // from it, so the loads have certainly returned.  (An arrive issued right after the
                // loads let the next TMA write overtake reads that were still in flight.)
                __syncwarp();
                if (lane == 0) ptx::mbar_arrive(&raw_empty[rs]);
                if (row == 0) QTR(3, ((kn >> 2) - 1) * 2 + grp, 3);
                if (++rs == p.raw_stages) { rs = 0; rph ^= 1u; }
            }
        }
    } else if (warp >= (uint32_t)C::EPI_WARP0) {
        // ---------------- epilogue: tensor memory -> fp16 (or fp32 partials) ----------------
        const uint32_t q = warp - C::EPI_WARP0;               // == warp % 4: the TMEM lane quadrant
        const uint32_t et = threadIdx.x - C::EPI_WARP0 * 32;  // 0..127
        uint32_t it = 0, xb_i = 0;
        // Fused reduce-scatter: every epilogue warp counts the tiles it has stored per owning rank (eight counters per warp
        // in shared memory).  After its last tile the warp fences its peer stores at system scope once -- a system-scope
        // fence under full store traffic costs several microseconds, so there is one per warp and launch, not one per
        // owner -- and adds its counts to the rank-wide counters; the warp that completes an owner's count (tiles x 4
        // epilogue warps) raises this rank's arrival flag on that owner.  Counting per warp needs no barrier among the
        // epilogue warps, so a warp that gave up on a wait cannot strand the others.
        uint32_t* sc_cnt = reinterpret_cast<uint32_t*>(bars) + 96 + q * 8;      // bytes 384..511 of the barrier block
        if (p.scatter.world && lane < 8u) sc_cnt[lane] = 0u;
        __syncwarp();
        bool sc_ok = true;
        auto scatter_flush = [&]() {
            __threadfence_system();
            __syncwarp();
            if (lane < p.scatter.world) {
                const uint32_t c = sc_cnt[lane];
                if (c) {
                    const uint32_t old = atomicAdd(p.scatter.done_counter + 4 + lane, c);
                    if (old + c == 4u * p.tiles_per_owner) {
                        p.scatter.done_counter[4 + lane] = 0u;
                        __threadfence_system();
                        asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p.scatter.flags[lane] + p.scatter.rank), "r"(p.scatter.epoch) : "memory");
                    }
                }
            }
            __syncwarp();
        };
        for (uint32_t idx = first_tile; idx < total_tiles; idx += tile_stride, it++) {
            const Tile t = tile_of(idx);
            const uint32_t buf = it & 1u;
            if (p.residual && p.k_splits == 1u) {
                // The epilogue warps idle through the tile's main loop: use that time to pull the residual tile
                // (T rows of 256 bytes) into L2, so the loads below wait for an L2 hit rather than for HBM.
                const uint32_t rows = t.tt * p.T < p.M ? min(p.T, p.M - t.tt * p.T) : 0u;
                const uint32_t n0 = t.wt * W_TILE;
                for (uint32_t r = et; r < rows; r += 128u) {
                    const char* line = reinterpret_cast<const char*>(p.residual + (size_t)(t.tt * p.T + r) * p.N + n0);
                    if (n0 < p.N) asm volatile("prefetch.global.L2 [%0];" ::"l"(line));
                    if (n0 + 64u < p.N) asm volatile("prefetch.global.L2 [%0];" ::"l"(line + 128));
                }
            }
            if (!ptx::mbar_wait<256>(&tm_full[buf], (it >> 1) & 1u, abort_flag, p.err, 108)) { sc_ok = false; break; }
            if (et == 0) QTRC(6, it, 0);
            ptx::tc_fence_after_sync();
            // grouped launch: the matrix this tile belongs to decides the output buffer and its width
            uint32_t wt_l = t.wt, Ng = p.N, grp_post = p.grp_post[0];
            __half* Yg = p.Y;
            if (p.groups > 1u) {
                uint32_t gi = 0;
                if (wt_l >= p.grp_tiles[0]) { wt_l -= p.grp_tiles[0]; gi = 1; if (wt_l >= p.grp_tiles[1]) { wt_l -= p.grp_tiles[1]; gi = 2; } }
                Ng = p.grp_N[gi]; Yg = p.grp_Y[gi]; grp_post = p.grp_post[gi];
            }
            const uint32_t n = wt_l * W_TILE + q * 32 + lane;
            const bool n_ok = n < Ng;
            // output element (tok, n) lives at out_base + tok * out_stride in either layout; the head split
            // (a division by a run-time D) is done once per tile here, never per element
            const size_t out_stride = (p.layout == 1) ? (size_t)p.D : (size_t)Ng;
            const size_t out_base = (p.layout == 1) ? ((size_t)(n / p.D) * p.M * p.D + (n % p.D)) : (size_t)n;
            const uint32_t taddr = tmem_base + ((q * 32u) << 16) + buf * ACC_STRIDE;
            const uint32_t tok0 = t.tt * p.T;
            float* ws = p.ws_partial + ((size_t)t.ks * (p.n_w_tiles * p.n_tok_tiles) + t.id) * p.T * W_TILE;
            // The destination kind is fixed per launch; branching on it once per tile (not per element) keeps
            // the inner loops to a convert, an address add and a store.
            const uint32_t valid = tok0 < p.M ? min(p.T, p.M - tok0) : 0u;     // token columns of this tile that exist
            // fused reduce-scatter: this tile's token rows belong to one rank; its fp32 sums go to that rank's
            // receive buffer (slot = this rank) over NVLink, tile by tile, while other tiles are still being computed
            float* partial_dst = p.partial_out;
            if (p.scatter.world) {
                const uint32_t owner = tok0 / p.scatter.rows;
                // slot `rank` of the owner's buffer, offset so that (tok * N + n) addresses this tile's rows; in elements of the
                // partial type (fp16 partials: the same arithmetic in halves, hence the division by two of the float pointer offset)
                const ptrdiff_t off = ((ptrdiff_t)p.scatter.rank - (ptrdiff_t)owner) * (ptrdiff_t)p.scatter.rows * (ptrdiff_t)p.N;
                partial_dst = p.scatter.fp16 ? reinterpret_cast<float*>(reinterpret_cast<__half*>(p.scatter.recv[owner]) + off)
                                             : p.scatter.recv[owner] + off;
                if (lane == 0) sc_cnt[owner]++;
            }
            const int mode = p.k_splits > 1 ? 0 : (partial_dst ? 1 : ((RESID && p.residual) ? 2 : 3));
            // integer-valued codecs: the row's scale multiplies the fp32 accumulator (before SiLU, before split-K sums)
            float rsc0 = 1.0f;
            if (Cd::ROW_SCALE && !p.swiglu) rsc0 = n_ok ? __half2float(p.row_scale0[n]) : 0.0f;
            if (p.row_epi) {
                // row-wise epilogue (everything but SwiGLU tiles, split-K partial tiles and outputs that cannot take 16-byte stores)
                uint8_t* stage = reinterpret_cast<uint8_t*>(xchg);
                if (mode == 1) {
                    if (p.scatter.world && p.scatter.fp16) row_epilogue<3>(p, stage, xb_i, taddr, et, tok0, valid, rsc0, Cd::ROW_SCALE, wt_l * W_TILE, Ng, Yg, partial_dst);
                    else row_epilogue<2>(p, stage, xb_i, taddr, et, tok0, valid, rsc0, Cd::ROW_SCALE, wt_l * W_TILE, Ng, Yg, partial_dst);
                } else if (mode == 2) {
                    row_epilogue<1>(p, stage, xb_i, taddr, et, tok0, valid, rsc0, Cd::ROW_SCALE, wt_l * W_TILE, Ng, Yg, nullptr);
                } else if (grp_post) {
                    row_epilogue_kv(p, stage, xb_i, taddr, et, tok0, valid, wt_l * W_TILE, Ng, Yg, grp_post);
                } else {
                    row_epilogue<0>(p, stage, xb_i, taddr, et, tok0, valid, rsc0, Cd::ROW_SCALE, wt_l * W_TILE, Ng, Yg, nullptr);
                }
            } else if (p.swiglu) {
                // SwiGLU tile: lanes 0..63 (warps 0,1) hold the gate projection of 64 features, lanes 64..127
                // (warps 2,3) the up projection of the same features.  Thread et and thread et ^ 64 own the two
                // halves of one feature: per batch of 16 token columns they swap 8 values through shared memory,
                // the gate thread finishes columns 0..7, the up thread columns 8..15.
                const uint32_t nf = t.wt * GATE_ROWS + (q & 1u) * 32u + lane;
                const bool nf_ok = nf < p.N;
                const bool up_side = q >= 2u;
                float rsc = 1.0f;
                if (Cd::ROW_SCALE) rsc = nf_ok ? __half2float((up_side ? p.row_scale1 : p.row_scale0)[nf]) : 0.0f;
                __half* dstb = p.Y + nf + (size_t)(tok0 + (up_side ? 8u : 0u)) * p.N;
                const uint32_t vlim = valid > (up_side ? 8u : 0u) ? valid - (up_side ? 8u : 0u) : 0u;   // columns left from this thread's first
                for (uint32_t c0 = 0; c0 < p.T; c0 += 16, xb_i++) {
                    uint32_t v[16];
                    ptx::tmem_ld_x16(taddr + c0, v);
                    ptx::tmem_ld_wait();
                    float f[16];
#pragma unroll
                    for (int j = 0; j < 16; j++) f[j] = Cd::ROW_SCALE ? __uint_as_float(v[j]) * rsc : __uint_as_float(v[j]);
                    float4* xb = xchg + (xb_i & 1u) * 256u;
                    // send the half the partner finishes: gate values of columns 8..15, up values of columns 0..7
                    xb[et] = up_side ? make_float4(f[0], f[1], f[2], f[3]) : make_float4(f[8], f[9], f[10], f[11]);
                    xb[128 + et] = up_side ? make_float4(f[4], f[5], f[6], f[7]) : make_float4(f[12], f[13], f[14], f[15]);
                    ptx::bar_sync(2, 128);
                    const float4 r0 = xb[et ^ 64u], r1 = xb[128 + (et ^ 64u)];
                    const float rv[8] = {r0.x, r0.y, r0.z, r0.w, r1.x, r1.y, r1.z, r1.w};
                    float o8[8];
#pragma unroll
                    for (int j = 0; j < 8; j++) o8[j] = up_side ? silu_mul(rv[j], f[8 + j]) : silu_mul(f[j], rv[j]);
                    if (nf_ok && c0 < vlim) {
                        const uint32_t lim = vlim - c0;
                        __half* dst = dstb + (size_t)c0 * p.N;
                        if (lim >= 8u) {
#pragma unroll
                            for (int j = 0; j < 8; j++) dst[(size_t)j * p.N] = __float2half_rn(o8[j]);
                        } else {
#pragma unroll
                            for (int j = 0; j < 8; j++) if ((uint32_t)j < lim) dst[(size_t)j * p.N] = __float2half_rn(o8[j]);
                        }
                    }
                }
            } else {
            // Residual epilogue: the residual values of a batch (16 strided 2-byte loads per thread) are requested
            // two batches ahead, all 16 at once and with no store in between (Y may alias the residual, so the
            // compiler would otherwise order every load behind the previous store and pay one memory latency per
            // element); 32 loads in flight per thread, on top of the L2 prefetch issued while the tile was computed.
            __half ring[RESID ? 2 : 1][16];
            auto load_residual = [&](uint32_t c0, __half (&dst)[16]) {
                if (RESID && mode == 2 && n_ok && c0 < valid) {
                    const uint32_t lim = valid - c0;
                    const __half* src = p.residual + out_base + (size_t)(tok0 + c0) * out_stride;
#pragma unroll
                    for (int j = 0; j < 16; j++) dst[j] = (uint32_t)j < lim ? __ldg(src + j * out_stride) : __half(0.0f);
                }
            };
#pragma unroll
            for (int u = 0; u < (RESID ? 2 : 0); u++) load_residual(16u * u, ring[u]);
            auto process_batch = [&](const uint32_t c0, const __half (&res)[16]) {
                uint32_t v[16];
                if (et == 0 && it == 0) QTR(7, 1 + c0 / 16, 0);
                ptx::tmem_ld_x16(taddr + c0, v);
                ptx::tmem_ld_wait();
                if (et == 0 && it == 0) QTR(7, 1 + c0 / 16, 1);
                float f[16];
#pragma unroll
                for (int j = 0; j < 16; j++) {
                    f[j] = __uint_as_float(v[j]);
                    if (Cd::ROW_SCALE) f[j] *= rsc0;
                }
                if (mode == 0) {
                    float* dst = ws + (size_t)c0 * W_TILE + q * 32 + lane;
#pragma unroll
                    for (int j = 0; j < 16; j++) dst[(size_t)j * W_TILE] = f[j];
                } else if (n_ok && c0 < valid) {
                    const uint32_t lim = valid - c0;                            // >= 1 columns of this batch exist
                    if (mode == 1) {
                        float* dst = partial_dst + (size_t)(tok0 + c0) * p.N + n;
#pragma unroll
                        for (int j = 0; j < 16; j++) if ((uint32_t)j < lim) dst[(size_t)j * p.N] = f[j];
                    } else if (RESID && mode == 2) {
                        const size_t o = out_base + (size_t)(tok0 + c0) * out_stride;
#pragma unroll
                        for (int j = 0; j < 16; j++)
                            if ((uint32_t)j < lim) p.Y[o + j * out_stride] = __float2half_rn(f[j] + __half2float(res[j]));
                    } else {
                        __half* dst = Yg + out_base + (size_t)(tok0 + c0) * out_stride;
                        if (lim >= 16u) {                                       // whole batch exists: no per-store predicate
#pragma unroll
                            for (int j = 0; j < 16; j++) dst[j * out_stride] = __float2half_rn(f[j]);
                        } else {
#pragma unroll
                            for (int j = 0; j < 16; j++) if ((uint32_t)j < lim) dst[j * out_stride] = __float2half_rn(f[j]);
                        }
                    }
                }
            };
            for (uint32_t c00 = 0; c00 < p.T; c00 += 32) {
#pragma unroll
                for (int u = 0; u < 2; u++) {
                    const uint32_t c0 = c00 + 16u * u;
                    if (c0 < p.T) {
                        __half res[16];
                        if (RESID) {
#pragma unroll
                            for (int j = 0; j < 16; j++) res[j] = ring[u][j];
                            load_residual(c0 + 32u, ring[u]);
                        }
                        process_batch(c0, res);
                    }
                }
            }
            }
            ptx::tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) { if (PAIR && pair_rank == 1u) ptx::mbar_arrive_cluster(&tm_empty[buf], 0u); else ptx::mbar_arrive(&tm_empty[buf]); }
            if (et == 0) QTRC(6, it, 1);
            if (p.k_splits > 1) {
                // count this partial tile in; the CTA that completes the count adds the partial tiles after the
                // role loops have ended (every CTA of a split launch owns exactly one work item)
                __threadfence();
                ptx::bar_sync(1, 128);
                if (et == 0) {
                    const uint32_t old = atomicAdd(&p.ws_counters[t.id], 1u);
                    *last_flag = (old == p.k_splits - 1u) ? 1u : 0u;
                }
            }
        }
        if (p.scatter.world && sc_ok) scatter_flush();
    }

    // ---------------- teardown ----------------
    ptx::tc_fence_before_sync();
    __syncthreads();
    if (threadIdx.x == 0) QTRC(7, 0u, 1);
    QCTA(2);
    if (*abort_flag) {
        // let copies that are still in flight land before the CTA gives its shared memory back
        const long long t0 = clock64();
        while (clock64() - t0 < 4000000LL) { }
        __syncthreads();
    }
    // pair launch: neither CTA may leave (or free tensor memory) while the other's MMAs, commits or arrivals can still
    // reach it; every thread of both CTAs gets here on every path, also after a wait has given up
    if (PAIR) ptx::cluster_sync_all();
    if (warp == 2) {
        ptx::tc_fence_after_sync();
        if (PAIR) ptx::tmem_dealloc_pair(tmem_base, TMEM_COLS); else ptx::tmem_dealloc(tmem_base, TMEM_COLS);
    }
    if (p.k_splits > 1 && *last_flag && !*abort_flag) {
        // Split-K fix-up by the whole CTA: the partial tiles of this output tile are complete (this CTA's arrival
        // completed the count), every warp is idle by now, and 16 float4 loads per thread keep enough bytes in
        // flight to cover the L2 latency in one or two rounds.  The sum runs in split order, so the result does not
        // depend on which CTA arrived last.
        __threadfence();
        const Tile t = decode_tile(blockIdx.x, p);
        switch (p.k_splits) {
            case 2: splitk_fixup<2>(p, t, threadIdx.x, C::THREADS); break;
            case 4: splitk_fixup<4>(p, t, threadIdx.x, C::THREADS); break;
            default: splitk_fixup<8>(p, t, threadIdx.x, C::THREADS); break;
        }
        if (threadIdx.x == 0) p.ws_counters[t.id] = 0u;
    }
    QCTA(3);
}

// ---------------------------------------------------------------------------------------------
// CUDA-core fallback for shapes the TMA path cannot take (K not a multiple of 256, rows or
// pointers not 16-byte aligned, formats without a tensor-core codec).  One thread per output,
// fp32 accumulation, weights unpacked per element in fp32 following the CPU gold's formulas.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ float ldh(const uint8_t* p) {
    return __half2float(__ushort_as_half((unsigned short)(p[0] | (p[1] << 8))));
}
__device__ __forceinline__ uint32_t bits3(const uint8_t* p, int i) {   // i-th 3-bit value of a 3-byte group run
    const uint8_t* g = p + (i >> 3) * 3;
    uint32_t v = g[0] | (g[1] << 8) | (g[2] << 16);
    return (v >> (3 * (i & 7))) & 7u;
}
__device__ float generic_weight(int fmt, const uint8_t* W, uint32_t n, uint32_t k, uint32_t N, uint32_t K) {
    switch (fmt) {
        case QUANT_Q4_0: {
            const uint8_t* b = W + ((size_t)n * (K / 32) + k / 32) * 18;
            uint32_t i = k % 32; uint8_t byte = b[2 + (i & 15)];
            int q = (i < 16) ? (byte & 15) : (byte >> 4);
            return (float)(q - 8) * ldh(b);
        }
        case QUANT_MLX_4BIT: {
            const uint8_t* b = W + ((size_t)n * (K / 32) + k / 32) * 20;
            uint32_t i = k % 32; uint8_t byte = b[4 + (i & 15)];
            int q = (i < 16) ? (byte & 15) : (byte >> 4);
            return (float)q * ldh(b) + ldh(b + 2);
        }
        case QUANT_Q4_K: {
            const uint8_t* b = W + ((size_t)n * (K / 256) + k / 256) * 144;
            uint32_t j = (k % 256) / 32, i = k % 32;
            const uint8_t* sc = b + 4;
            uint32_t s6 = sc[j] & 63u;
            uint32_t m6 = (j < 4) ? ((sc[j + 8] & 15u) | ((sc[j] >> 6) << 4)) : ((sc[j + 4] >> 4) | ((sc[j] >> 6) << 4));
            uint8_t byte = b[16 + 16 * j + (i & 15)];
            int q = (i < 16) ? (byte & 15) : (byte >> 4);
            return (float)q * (ldh(b) * (float)s6) - ldh(b + 2) * (float)m6;
        }
        case QUANT_TERNARY_1_58: {
            const uint8_t* b = W + ((size_t)n * (K / 32) + k / 32) * 12;
            uint32_t i = k % 32;
            uint32_t word = b[4 + 4 * (i / 16)] | (b[5 + 4 * (i / 16)] << 8) | (b[6 + 4 * (i / 16)] << 16) | ((uint32_t)b[7 + 4 * (i / 16)] << 24);
            int c = (int)((word >> (2 * (i % 16))) & 3u) - 1;
            return (float)c * ldh(b);
        }
        case QUANT_PRISM_Q2_0: {
            const uint8_t* b = W + ((size_t)n * (K / 128) + k / 128) * 34;
            uint32_t i = k % 128;
            int c = (int)((b[2 + i / 4] >> (2 * (i % 4))) & 3u) - 1;
            return (float)c * ldh(b);
        }
        case QUANT_EXL3: {
            const uint8_t* b = W + ((size_t)n * (K / 256) + k / 256) * 144;
            uint32_t j = (k % 256) / 32, i = k % 32;
            float d = ldh(b), bias = ldh(b + 2);
            float sub_scale = d * (float)b[4 + j] * 0.015625f, sub_res = d * ((float)b[12 + j] - 128.0f) * 0.0078125f;
            uint32_t q = bits3(b + 48 + 12 * j, (int)i);
            return bias + sub_scale * (float)(int8_t)b[20 + q] + sub_res * (float)(int8_t)b[28 + q];
        }
        case QUANT_VAR_RATE_AFFINE: {
            const uint8_t* b = W + ((size_t)n * (K / 256) + k / 256) * 160;
            const int offs[8] = {0, 12, 24, 40, 56, 72, 88, 108};
            uint32_t j = (k % 256) / 32, dst = k % 32;
            float d = ldh(b), bias = ldh(b + 2);
            float sub_scale = d * (float)b[4 + j] * 0.0625f, sub_bias = bias + d * ((float)b[12 + j] - 128.0f) * 0.0625f;
            uint32_t mode = b[20 + j], bits = mode & 7u, perm = (mode >> 3) & 3u;
            // invert the destination permutation: which source element lands on k?
            uint32_t src = dst;
            if (perm == 1u) src = (dst < 16) ? 2 * dst : 2 * (dst - 16) + 1;
            else if (perm == 2u) src = 31 - dst;
            const uint8_t* pq = b + 32 + offs[j];
            float qv;
            if (bits == 3u) qv = (float)bits3(pq, (int)src) - 4.0f;
            else if (bits == 5u) {
                const uint8_t* g = pq + (src >> 3) * 5;
                uint64_t v = 0;
                for (int t = 0; t < 5; t++) v |= (uint64_t)g[t] << (8 * t);
                qv = (float)((v >> (5 * (src & 7))) & 31u) - 16.0f;
            } else {
                uint8_t byte = pq[src & 15];
                qv = (float)((src < 16) ? (byte & 15) : (byte >> 4)) - 8.0f;
            }
            return qv * sub_scale + sub_bias;
        }
        case QUANT_MLX_4BIT_G64: {
            const uint32_t* qs = reinterpret_cast<const uint32_t*>(W) + (size_t)n * (K / 8);
            const __half* sc = reinterpret_cast<const __half*>(W + (size_t)N * (K / 8) * 4) + (size_t)n * (K / 64);
            const __half* bi = sc + (size_t)N * (K / 64);
            uint32_t q = (qs[k / 8] >> (4 * (k % 8))) & 15u;
            return (float)q * __half2float(sc[k / 64]) + __half2float(bi[k / 64]);
        }
        case QUANT_MLX_4BIT_PLANAR: {
            const size_t blocks = (size_t)N * (K / 32), blk = (size_t)n * (K / 32) + k / 32;
            const size_t scales_off = (blocks * 16 + 15) & ~(size_t)15, biases_off = (scales_off + blocks * 2 + 15) & ~(size_t)15;
            const uint8_t byte = W[blk * 16 + (k % 16)];
            const uint32_t q = ((k % 32) < 16) ? (byte & 15u) : (byte >> 4);
            return (float)q * __half2float(reinterpret_cast<const __half*>(W + scales_off)[blk]) +
                   __half2float(reinterpret_cast<const __half*>(W + biases_off)[blk]);
        }
        case QUANT_TERNARY_ROW: {
            const uint32_t* qs = reinterpret_cast<const uint32_t*>(W) + (size_t)n * (K / 16);
            const __half* rs = reinterpret_cast<const __half*>(W + (size_t)N * (K / 16) * 4);
            int c = (int)((qs[k / 16] >> (2 * (k % 16))) & 3u) - 1;
            return (float)c * __half2float(rs[n]);
        }
        default: return 0.0f;
    }
}

__global__ void qgemm_generic_kernel(int fmt, const __half* X, const uint8_t* W0, const uint8_t* W1, Params p) {
    const uint32_t n = blockIdx.x * blockDim.x + threadIdx.x;
    const uint32_t tok = blockIdx.y * blockDim.y + threadIdx.y;
    if (n >= p.N || tok >= p.M) return;
    const __half* x = X + (size_t)tok * p.K;
    float acc = 0.0f, acc2 = 0.0f;
    for (uint32_t k = 0; k < p.K; k++) {
        const float a = __half2float(x[k]);
        acc += a * generic_weight(fmt, W0, n, k, p.N, p.K);
        if (W1) acc2 += a * generic_weight(fmt, W1, n, k, p.N, p.K);
    }
    if (W1) acc = acc / (1.0f + expf(-acc)) * acc2;
    if (p.partial_out) { p.partial_out[(size_t)tok * p.N + n] = acc; return; }
    const size_t o = out_index(p, tok, n);
    if (p.residual) acc += __half2float(p.residual[o]);
    p.Y[o] = __float2half_rn(acc);
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
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess)
            f = nullptr;
        return (EncodeTiledFn)f;
    }();
    return fn;
}

bool make_map_2d(CUtensorMap* m, CUtensorMapDataType dt, size_t elem, const void* ptr, uint64_t inner, uint64_t outer,
                 uint64_t row_bytes, uint32_t box_inner, uint32_t box_outer, CUtensorMapSwizzle sw) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return false;
    cuuint64_t dims[2] = {inner, outer};
    cuuint64_t strides[1] = {row_bytes};
    cuuint32_t box[2] = {box_inner, box_outer};
    cuuint32_t estr[2] = {1, 1};
    (void)elem;
    return fn(m, dt, 2, const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, sw,
              CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// bytes of one row of one packed stage (CHUNK elements), 0 for formats without a tensor-core codec
int row_bytes_256(int fmt) {
    switch (fmt) {
        case QUANT_PRISM_Q2_0: return 272;       // 8 blocks of 34 bytes per 1024 elements
        case QUANT_Q4_0: return 144;
        case QUANT_MLX_4BIT: return 160;
        case QUANT_Q4_K: return 144;
        case QUANT_TERNARY_1_58: return 96;
        case QUANT_VAR_RATE_AFFINE: return 160;
        case QUANT_EXL3: return 144;
        case QUANT_MLX_4BIT_G64: return 128;     // nibble plane only; scales and biases sit in planes behind it
        case QUANT_MLX_4BIT_PLANAR: return 128;  // nibble plane only; one scale and one bias per 32 elements in planes behind it
        case QUANT_TERNARY_ROW: return 64;       // 2-bit plane only; one fp16 scale per row behind it
        default: return 0;
    }
}

uint32_t chunk_elems(int fmt) { return fmt == QUANT_PRISM_Q2_0 ? 1024u : (uint32_t)KCHUNK; }

int g_sm_count = 0;
int sm_count() {
    if (!g_sm_count) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&g_sm_count, cudaDevAttrMultiProcessorCount, dev);
        if (g_sm_count <= 0) g_sm_count = 148;
    }
    return g_sm_count;
}

struct Plan { uint32_t T, n_tok_tiles, n_w_tiles, k_splits, kchunks; };

Plan make_plan(const GemmArgs& a) {
    const uint32_t tok_max = 256u;
    Plan pl;
    pl.n_tok_tiles = (a.M + tok_max - 1) / tok_max;
    uint32_t per = (a.M + pl.n_tok_tiles - 1) / pl.n_tok_tiles;
    pl.T = (per + 15u) & ~15u;
    const uint32_t rows_per_tile = a.W1 ? GATE_ROWS : W_TILE;    // output features per tile
    pl.n_w_tiles = (a.N + rows_per_tile - 1) / rows_per_tile;
    for (uint32_t e = 0; e < a.n_extra && e < 2u; e++) pl.n_w_tiles += (a.N_extra[e] + W_TILE - 1) / W_TILE;   // grouped launch
    const uint32_t chunks = a.K / chunk_elems(a.format);
    pl.k_splits = 1;
    if (!a.W1 && !a.scatter.world) {       // (the fused reduce-scatter epilogue writes whole tiles: no K split)
        // split K while the grid would leave most SMs idle and every split keeps >= 2 chunks
        const uint32_t tiles = pl.n_tok_tiles * pl.n_w_tiles;
        const uint32_t sms = (uint32_t)sm_count();
        for (uint32_t s = 2; s <= 8; s *= 2) {
            if (tiles * s > sms || chunks % s != 0 || chunks / s < 2) break;
            pl.k_splits = s;
        }
        if (pl.n_tok_tiles * pl.n_w_tiles > 4096) pl.k_splits = 1;
    }
    pl.kchunks = chunks / pl.k_splits;
    return pl;
}

// CTA pairs need the idle warp 14 as their relay: a codec with three unpack groups (twelve unpack warps) has it -- every
// codec as of now; one with two groups would stay on one CTA per MMA.
template <int FMT> constexpr bool pair_capable() { return Cfg<FMT>::DQ_WARPS == 12 && Cfg<FMT>::EPI_WARP0 > 14; }

// The dynamic shared-memory attribute is per device: set once for every device a launch (or prepare_device) sees.
template <int FMT>
cudaError_t set_kernel_attributes() {
    static uint64_t done_mask = 0;          // bit d: set on device d
    static std::mutex mu;
    int dev = 0;
    cudaGetDevice(&dev);
    std::lock_guard<std::mutex> lock(mu);
    if (dev >= 0 && dev < 64 && (done_mask >> dev) & 1u) return cudaSuccess;
    cudaError_t e = cudaFuncSetAttribute(qgemm_kernel<FMT, false, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(qgemm_kernel<FMT, true, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    if constexpr (pair_capable<FMT>()) {
        if (e == cudaSuccess) e = cudaFuncSetAttribute(qgemm_kernel<FMT, false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(qgemm_kernel<FMT, true, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    }
    if (e == cudaSuccess && dev >= 0 && dev < 64) done_mask |= 1ull << dev;
    return e;
}

bool g_pair_enabled = true;      // testing hook: off keeps every launch on one CTA per MMA
bool pair_swiglu() { static const char* e = getenv("B200_PAIR_SWIGLU"); return !(e && e[0] == '0'); }   // tuning aid: B200_PAIR_SWIGLU=0 keeps SwiGLU launches on one CTA per MMA
int g_last_pair = 0;             // CTA pairs of the last launch (0: it ran with one CTA per MMA)

// Clusters of two CTAs (one CTA per SM) that can be resident at once: the pair launch's grid.  Asked of the runtime once
// per format; half the SM count where the query fails.
template <int FMT> int max_pairs() {
    static int n = 0;
    if (n == 0) {
        if constexpr (pair_capable<FMT>()) {
            cudaLaunchConfig_t cfg;
            memset(&cfg, 0, sizeof(cfg));
            cfg.gridDim = dim3(2 * (unsigned)sm_count()); cfg.blockDim = dim3(Cfg<FMT>::THREADS); cfg.dynamicSmemBytes = SMEM_BYTES;
            cudaLaunchAttribute at[1];
            at[0].id = cudaLaunchAttributeClusterDimension;
            at[0].val.clusterDim.x = 2; at[0].val.clusterDim.y = 1; at[0].val.clusterDim.z = 1;
            cfg.attrs = at; cfg.numAttrs = 1;
            int c = 0;
            if (cudaOccupancyMaxActiveClusters(&c, qgemm_kernel<FMT, false, true>, &cfg) == cudaSuccess && c > 0) n = c;
            else { cudaGetLastError(); n = sm_count() / 2; }
        } else n = sm_count() / 2;
        if (n > sm_count() / 2) n = sm_count() / 2;
        if (n < 1) n = 1;
    }
    return n;
}

template <int FMT>
cudaError_t launch_fast(const GemmArgs& a, const Workspace& ws, cudaStream_t stream) {
    using C = Cfg<FMT>;
    const Plan pl = make_plan(a);
    const int rb = cdc::Codec<FMT>::ROW_BYTES;
    const uint64_t w_row_bytes = (uint64_t)(a.K / C::CHUNK) * rb;
    // CTA pairs (cta_group::2): token tiles that halve into whole 16-row groups, no K split, weight tiles in pairs.
    // (SwiGLU launches included: 352-372 us against 380-392 us at the 8B shape, the layer 0.75 ms against 0.80 ms.)
    const bool pair = pair_capable<FMT>() && g_pair_enabled && pl.k_splits == 1 && pl.T >= 128u && pl.T % 32u == 0u && pl.n_w_tiles % 2u == 0u && (!a.W1 || pair_swiglu());
    const uint32_t t_cta = pair ? pl.T / 2u : pl.T;             // token rows of the activation tile one CTA loads
    g_last_pair = pair ? 1 : 0;
    CUtensorMap tmX, tmW0, tmW1, tmW2;
    if (!make_map_2d(&tmX, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, a.X, a.K, a.M, (uint64_t)a.K * 2, KSTEP, t_cta,
                     CU_TENSOR_MAP_SWIZZLE_128B))
        return cudaErrorInvalidValue;
    const CUtensorMapSwizzle wsw = cdc::Codec<FMT>::RAW_SWIZZLE_128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE;
    const uint32_t box_rows = a.W1 ? GATE_ROWS : W_TILE;
    constexpr int EB = cdc::Codec<FMT>::TMA_ELEM_BYTES;
    const CUtensorMapDataType wdt = EB == 2 ? CU_TENSOR_MAP_DATA_TYPE_UINT16 : CU_TENSOR_MAP_DATA_TYPE_UINT8;
    if (!make_map_2d(&tmW0, wdt, EB, a.W0, w_row_bytes / EB, a.N, w_row_bytes, rb / EB, box_rows, wsw))
        return cudaErrorInvalidValue;
    // second / third map: the up matrix of a SwiGLU launch, or the extra matrices of a grouped launch
    const bool grouped = a.n_extra > 0;
    if (grouped && (a.n_extra > 2 || a.W1 || a.residual || a.partial_out || a.scatter.world ||
                    cdc::Codec<FMT>::META_WORDS != 0 || cdc::Codec<FMT>::ROW_SCALE))
        return cudaErrorInvalidValue;
    const void* w1 = a.W1 ? a.W1 : (grouped ? a.W_extra[0] : a.W0);
    const uint32_t n1 = grouped ? a.N_extra[0] : a.N;
    const void* w2 = a.n_extra > 1 ? a.W_extra[1] : a.W0;
    const uint32_t n2 = a.n_extra > 1 ? a.N_extra[1] : a.N;
    if (!make_map_2d(&tmW1, wdt, EB, w1, w_row_bytes / EB, n1, w_row_bytes, rb / EB, box_rows, wsw))
        return cudaErrorInvalidValue;
    if (!make_map_2d(&tmW2, wdt, EB, w2, w_row_bytes / EB, n2, w_row_bytes, rb / EB, box_rows, wsw))
        return cudaErrorInvalidValue;

    Params p;
    p.M = a.M; p.N = a.N; p.K = a.K;
    p.T = pl.T; p.n_tok_tiles = pl.n_tok_tiles; p.n_w_tiles = pl.n_w_tiles; p.k_splits = pl.k_splits; p.kchunks = pl.kchunks;
    p.swiglu = a.W1 ? 1u : 0u;
    // Row-wise epilogue: wherever every output row can take 16-byte stores (and, with a residual, 8-byte loads).  SwiGLU
    // tiles and split-K partial tiles have their own paths.
    const bool partial_f32 = (a.partial_out != nullptr) || (a.scatter.world && !a.scatter.fp16);
    bool row_ok = !a.W1 && pl.k_splits == 1;
    auto aligned16 = [](const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15u) == 0; };
    if (row_ok) {
        if (a.partial_out) row_ok = aligned16(a.partial_out) && a.N % 4u == 0u;
        else if (a.scatter.world) {
            row_ok = a.N % 8u == 0u;
            for (uint32_t o = 0; o < a.scatter.world; o++) row_ok = row_ok && aligned16(a.scatter.recv[o]);
        } else {
            row_ok = aligned16(a.Y) && a.N % 8u == 0u && (a.layout != 1 || (a.D % 8u == 0u));
            if (a.residual) row_ok = row_ok && (reinterpret_cast<uintptr_t>(a.residual) & 7u) == 0;
            for (uint32_t e = 0; e < a.n_extra && e < 2u; e++) row_ok = row_ok && aligned16(a.Y_extra[e]) && a.N_extra[e] % 8u == 0u;
        }
    }
    if (a.scatter.world && a.scatter.fp16 && !row_ok) return cudaErrorInvalidValue;     // fp16 partial sums exist on the row-wise epilogue only
    // K/V-cache post-operations: head-major fp16 row epilogue only, whole heads per 128-row tile, Q8_0 records of 32
    const bool any_post = (a.post[0] | a.post[1] | a.post[2]) != 0u;
    if (any_post) {
        if (!row_ok || a.layout != 1 || a.residual || a.partial_out || a.scatter.world || cdc::Codec<FMT>::ROW_SCALE ||
            (a.D != 64u && a.D != 128u) || a.N % a.D != 0u)
            return cudaErrorInvalidValue;
        for (uint32_t e = 0; e < a.n_extra && e < 2u; e++) if (a.N_extra[e] % a.D != 0u) return cudaErrorInvalidValue;
        if (((a.post[0] | a.post[1] | a.post[2]) & POST_ROPE) && (!a.rope_table || (reinterpret_cast<uintptr_t>(a.rope_table) & 15u))) return cudaErrorInvalidValue;
    }
    p.rope_table = reinterpret_cast<const float2*>(a.rope_table);
    p.kv_tokens = a.kv_tokens ? a.kv_tokens : a.M; p.kv_pos0 = a.kv_pos0;
    if (any_post && (uint64_t)p.kv_pos0 + a.M > p.kv_tokens) return cudaErrorInvalidValue;
    for (int gi = 0; gi < 3; gi++) p.grp_post[gi] = (uint32_t)gi <= a.n_extra ? a.post[gi] : 0u;
    p.row_epi = row_ok ? 1u : 0u;
    const long xchg_bytes = a.W1 ? XCHG_BYTES : (row_ok ? ((partial_f32 || a.residual) ? XCHG_BYTES_F32 : XCHG_BYTES) : 0);
    p.b_stage_bytes = t_cta * 128u;
    p.a_stages = STAGES;
    if (pair) {
        // A stage is handed over between the two CTAs of a pair (remote arrival, multicast commit), which adds latency to
        // every turn of a ring, and an activation stage is only 16 KB: deeper rings, as far as two packed stages still fit
        // beside them.  Measured at the 8B shapes (Q4_0, M = 2048): 6 activation + 4 weight stages 54.0 / 171 us
        // (K = 4096 / 14336), 6 + 5: 54.9 / 183, 4 + 4: 55.1 / 178, 4 + 3: 55.6 / 190; one CTA per MMA: 59.5 / 194.
        static const uint32_t choices[][2] = {{6, 4}, {5, 4}, {4, 4}, {4, 3}};
        p.b_stages = 4; p.a_stages = 3;
        for (const auto& c : choices)
            if (raw_stages_fit<FMT>(t_cta, xchg_bytes, c[0], c[1]) >= 2) { p.b_stages = c[0]; p.a_stages = c[1]; break; }
        // tuning aid: B200_PAIR_STAGES="<activation stages>,<weight stages>" overrides the choice where it fits
        static const char* ov = getenv("B200_PAIR_STAGES");
        if (ov) {
            unsigned ob = 0, oa = 0;
            if (sscanf(ov, "%u,%u", &ob, &oa) == 2 && ob >= 2 && ob <= (unsigned)PAIR_MAX_B_STAGES && oa >= 3 && oa <= (unsigned)MAX_A_STAGES &&
                raw_stages_fit<FMT>(t_cta, xchg_bytes, ob, oa) >= 1) { p.b_stages = ob; p.a_stages = oa; }
        }
        long n = raw_stages_fit<FMT>(t_cta, xchg_bytes, p.b_stages, p.a_stages);
        p.raw_stages = (uint32_t)(n < 1 ? 1 : (n > MAX_RAW_STAGES ? MAX_RAW_STAGES : n));
        if (raw_stages_fit<FMT>(t_cta, xchg_bytes, p.b_stages, p.a_stages) < 1) return cudaErrorInvalidValue;
    } else {
        p.raw_stages = raw_stages_for<FMT>(t_cta, xchg_bytes);
        p.b_stages = b_stages_for<FMT>(t_cta, xchg_bytes);
    }
    p.Y = (__half*)a.Y; p.residual = (const __half*)a.residual; p.partial_out = a.partial_out;
    p.scatter = a.scatter;
    p.wait_rows = a.wait_rows;
    if (a.wait_rows.flags && (pl.k_splits != 1 || a.wait_rows.rows == 0 || a.M > 32u * a.wait_rows.rows)) return cudaErrorInvalidValue;
    p.groups = 1u + a.n_extra;
    p.grp_tiles[0] = (a.N + W_TILE - 1) / W_TILE; p.grp_N[0] = a.N; p.grp_Y[0] = (__half*)a.Y;
    for (uint32_t e = 0; e < 2u; e++) {
        const bool on = e < a.n_extra;
        p.grp_tiles[1 + e] = on ? (a.N_extra[e] + W_TILE - 1) / W_TILE : 0u;
        p.grp_N[1 + e] = on ? a.N_extra[e] : 0u; p.grp_Y[1 + e] = on ? (__half*)a.Y_extra[e] : nullptr;
    }
    if (a.scatter.world && (pl.k_splits != 1 || a.W1 || a.scatter.rows % pl.T != 0 || a.scatter.rows * a.scatter.world != a.M)) return cudaErrorInvalidValue;
    p.tt_shift = 0; p.tiles_per_owner = 0;
    if (a.scatter.world) {
        p.tiles_per_owner = pl.n_w_tiles * (a.scatter.rows / pl.T);
        p.tt_shift = ((a.scatter.rank + 1u) % a.scatter.world) * (a.scatter.rows / pl.T);
    }
    p.layout = (uint32_t)a.layout; p.H = a.H; p.D = a.D ? a.D : 1;
    p.ws_partial = ws.partial; p.ws_counters = ws.counters; p.err = ws.err;
    // planar layouts: everything behind the N x (K/256 * ROW_BYTES) plane of packed values
    const size_t plane = (size_t)a.N * w_row_bytes;
    p.meta0 = (const uint8_t*)a.W0 + plane;
    p.meta1 = a.W1 ? (const uint8_t*)a.W1 + plane : p.meta0;
    p.row_scale0 = (const __half*)p.meta0;
    p.row_scale1 = (const __half*)p.meta1;
    if (pl.k_splits > 1) {
        const size_t need = (size_t)pl.k_splits * pl.n_tok_tiles * pl.n_w_tiles * pl.T * W_TILE;
        if (!ws.partial || !ws.counters || ws.partial_floats < need) return cudaErrorInvalidValue;
    }

    constexpr size_t smem = SMEM_BYTES;
    { cudaError_t e = set_kernel_attributes<FMT>(); if (e != cudaSuccess) return e; }
    const uint32_t total = pl.n_tok_tiles * pl.n_w_tiles * pl.k_splits;
    const uint32_t grid = total < (uint32_t)sm_count() ? total : (uint32_t)sm_count();
    // Programmatic stream serialization: this grid's CTAs may be placed (and run their prologue up to
    // griddepcontrol.wait) while the previous kernel in the stream drains, which hides the launch latency between
    // back-to-back projections.  Stream order is unchanged: nothing is read or written before that wait.
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    cfg.gridDim = dim3(grid); cfg.blockDim = dim3(C::THREADS); cfg.dynamicSmemBytes = smem; cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr; cfg.numAttrs = 1;
    if constexpr (pair_capable<FMT>()) {
        if (pair) {
            // one cluster of two CTAs per pair of SMs; a pair walks pairs of weight tiles that share a token tile
            const uint32_t pair_tiles = (pl.n_w_tiles / 2u) * pl.n_tok_tiles;
            const uint32_t pairs = pair_tiles < (uint32_t)max_pairs<FMT>() ? pair_tiles : (uint32_t)max_pairs<FMT>();
            cfg.gridDim = dim3(2u * pairs);
            g_last_pair = (int)pairs;
            attr[1].id = cudaLaunchAttributeClusterDimension;
            attr[1].val.clusterDim.x = 2; attr[1].val.clusterDim.y = 1; attr[1].val.clusterDim.z = 1;
            cfg.numAttrs = 2;
            if (a.residual) return cudaLaunchKernelEx(&cfg, qgemm_kernel<FMT, true, true>, tmX, tmW0, tmW1, tmW2, p);
            return cudaLaunchKernelEx(&cfg, qgemm_kernel<FMT, false, true>, tmX, tmW0, tmW1, tmW2, p);
        }
    }
    // (the split-K fix-up adds the residual outside the epilogue loop: only unsplit residual launches need the RESID build)
    if (a.residual && pl.k_splits == 1) return cudaLaunchKernelEx(&cfg, qgemm_kernel<FMT, true, false>, tmX, tmW0, tmW1, tmW2, p);
    return cudaLaunchKernelEx(&cfg, qgemm_kernel<FMT, false, false>, tmX, tmW0, tmW1, tmW2, p);
}

cudaError_t dispatch_fast(const GemmArgs& a, const Workspace& ws, cudaStream_t s) {
    switch (a.format) {
        case QUANT_Q4_0: return launch_fast<QUANT_Q4_0>(a, ws, s);
        case QUANT_MLX_4BIT: return launch_fast<QUANT_MLX_4BIT>(a, ws, s);
        case QUANT_Q4_K: return launch_fast<QUANT_Q4_K>(a, ws, s);
        case QUANT_TERNARY_1_58: return launch_fast<QUANT_TERNARY_1_58>(a, ws, s);
        case QUANT_VAR_RATE_AFFINE: return launch_fast<QUANT_VAR_RATE_AFFINE>(a, ws, s);
        case QUANT_EXL3: return launch_fast<QUANT_EXL3>(a, ws, s);
        case QUANT_MLX_4BIT_G64: return launch_fast<QUANT_MLX_4BIT_G64>(a, ws, s);
        case QUANT_MLX_4BIT_PLANAR: return launch_fast<QUANT_MLX_4BIT_PLANAR>(a, ws, s);
        case QUANT_TERNARY_ROW: return launch_fast<QUANT_TERNARY_ROW>(a, ws, s);
        case QUANT_PRISM_Q2_0: return launch_fast<QUANT_PRISM_Q2_0>(a, ws, s);
        default: return cudaErrorInvalidValue;
    }
}

thread_local int g_last_launches = 0;

}  // namespace

cudaError_t prepare_device() {
    cudaError_t e = set_kernel_attributes<QUANT_Q4_0>();
    if (e == cudaSuccess) e = set_kernel_attributes<QUANT_MLX_4BIT>();
    if (e == cudaSuccess) e = set_kernel_attributes<QUANT_Q4_K>();
    if (e == cudaSuccess) e = set_kernel_attributes<QUANT_TERNARY_1_58>();
    if (e == cudaSuccess) e = set_kernel_attributes<QUANT_VAR_RATE_AFFINE>();
    if (e == cudaSuccess) e = set_kernel_attributes<QUANT_EXL3>();
    if (e == cudaSuccess) e = set_kernel_attributes<QUANT_MLX_4BIT_G64>();
    if (e == cudaSuccess) e = set_kernel_attributes<QUANT_MLX_4BIT_PLANAR>();
    if (e == cudaSuccess) e = set_kernel_attributes<QUANT_TERNARY_ROW>();
    if (e == cudaSuccess) e = set_kernel_attributes<QUANT_PRISM_Q2_0>();
    return e;
}

bool fast_path_ok(const GemmArgs& a) {
    if (a.force_generic) return false;
    if (row_bytes_256(a.format) == 0) return false;
    if (a.K == 0 || a.K % chunk_elems(a.format) != 0) return false;
    if (((uintptr_t)a.X & 15u) || ((uintptr_t)a.W0 & 15u) || (a.W1 && ((uintptr_t)a.W1 & 15u))) return false;
    for (uint32_t e = 0; e < a.n_extra && e < 2u; e++)
        if (!a.W_extra[e] || ((uintptr_t)a.W_extra[e] & 15u) || !a.Y_extra[e] || a.N_extra[e] == 0) return false;
    if (a.M == 0 || a.N == 0) return false;
    return encode_fn() != nullptr;
}

size_t workspace_floats(const GemmArgs& a) {
    if (gemv_path_ok(a)) return 0;
    if (small_path_ok(a)) return small_scratch_floats(a);
    if (!fast_path_ok(a)) return 0;
    const Plan pl = make_plan(a);
    if (pl.k_splits <= 1) return 0;
    return (size_t)pl.k_splits * pl.n_tok_tiles * pl.n_w_tiles * pl.T * W_TILE;
}

cudaError_t launch(const GemmArgs& a, const Workspace& ws, cudaStream_t stream) {
    g_last_launches = 1;
    if (a.wait_rows.flags) return fast_path_ok(a) ? dispatch_fast(a, ws, stream) : cudaErrorInvalidValue;   // only the persistent kernel waits for rows
    if (gemv_path_ok(a)) return launch_gemv(a, stream);
    if (small_path_ok(a)) return launch_small(a, ws, stream);
    if (fast_path_ok(a)) return dispatch_fast(a, ws, stream);
    if (a.scatter.world || a.n_extra) return cudaErrorInvalidValue;   // fused reduce-scatter and grouped launches exist on the tensor-core path only
    Params p;
    memset(&p, 0, sizeof(p));
    p.M = a.M; p.N = a.N; p.K = a.K;
    p.Y = (__half*)a.Y; p.residual = (const __half*)a.residual; p.partial_out = a.partial_out;
    p.layout = (uint32_t)a.layout; p.H = a.H; p.D = a.D ? a.D : 1;
    dim3 block(32, 8), grid((a.N + 31) / 32, (a.M + 7) / 8);
    qgemm_generic_kernel<<<grid, block, 0, stream>>>(a.format, (const __half*)a.X, (const uint8_t*)a.W0, (const uint8_t*)a.W1, p);
    return cudaGetLastError();
}

int last_launch_count() { return g_last_launches; }
void set_pair_kernel_enabled(bool on) { g_pair_enabled = on; }
int last_launch_pairs() { return g_last_pair; }

}  // namespace qg
