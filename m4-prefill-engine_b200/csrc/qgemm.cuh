// Host-side interface of the dequant-fused projection kernels (internal to the library; the
// public surface is include/b200_bridge.h).
#pragma once
#include <cuda_runtime.h>
#include <cstddef>
#include <cstdint>

namespace qg {

struct GemmArgs {
    int format;               // QuantFormat id
    const void* X;            // [M][K] fp16, device
    const void* W0;           // packed weights [N][K/blk] (gate matrix for SwiGLU)
    const void* W1;           // up matrix for SwiGLU, else nullptr
    void* Y;                  // fp16 out: [M][N], or [H][M][D] when layout == 1
    uint32_t M, N, K;
    int layout;               // LayoutMode
    uint32_t H, D;            // direct-head split of N
    const void* residual;     // optional fp16 [M][N] added in the epilogue (standard layout only)
    float* partial_out;       // optional fp32 [M][N]: write raw accumulators instead of fp16 Y
    int force_generic;        // testing hook: use the CUDA-core fallback kernel
    // Grouped launch: up to two more projections of the same X (same K, format, layout and D) run in the same
    // grid, their weight tiles queued behind those of W0.  n_extra == 0: off.  Plain fp16 outputs only.
    uint32_t n_extra;
    const void* W_extra[2];
    void* Y_extra[2];
    uint32_t N_extra[2];
    // K/V-cache post-operations fused into the epilogue of a head-major launch (layout 1, D 64 or 128, no K split; else the
    // launch is refused): post[i] for matrix i (0 = W0, 1.. = W_extra) is a bit set of 1 = rotary embedding with
    // rope_table[token][D/2] = (cos, sin) of that token's position, 2 = write block_q8_0 records [head][token][D/32] to Y
    // instead of fp16.  The results are bit-identical to the plain projection followed by lops::rope and attn::launch_quantize.
    uint32_t post[3];
    const void* rope_table;
    uint32_t kv_tokens, kv_pos0;     // Q8_0 records go to [head][kv_tokens][D/32] at token index kv_pos0 + t (kv_tokens == 0: M, offset 0)
    // Tensor-parallel reduce-scatter fused into the epilogue (row-split projections): instead of one local fp32
    // [M][N] buffer, token rows [o * rows, (o + 1) * rows) go to rank o's receive buffer, slot `rank`, through
    // peer-mapped pointers.  Rank r works through the owners in the order r + 1, r + 2, ..., r (its own rows last);
    // when all tiles of owner o are stored and fenced at system scope, flag `rank` in rank o's flag array is raised
    // to `epoch`.  world == 0: off.
    struct Scatter {
        uint32_t world, rank, rows;      // rows = M / world token rows owned by each rank (a multiple of the token tile)
        float* recv[8];                  // recv[o]: rank o's buffer, fp32 [world][rows][N]
        uint32_t* flags[8];              // flags[o]: rank o's arrival flags, one word per source rank
        uint32_t epoch;
        uint32_t fp16;                   // != 0: partial sums travel as fp16 (recv[o] then holds fp16 [world][rows][N]), else fp32
        uint32_t* done_counter;          // 16 device-local words, zero between launches (words 4..11: one tile counter per owner)
    } scatter;
    // Activations that other ranks are still writing (the rows an owner-side reduction broadcasts): token rows
    // [o * rows, (o + 1) * rows) may be read once flags[o] has reached `epoch`.  The warp that loads a token tile polls the
    // flags of the owners the tile covers first (bounded; error code 110), so the launch needs no separate wait kernel in
    // front of it and starts on the rows that are already there.  flags == nullptr: off.  Persistent kernel, no K split.
    struct WaitRows {
        const uint32_t* flags;           // this rank's "rows written" flags, one word per owner
        uint32_t rows, epoch;
        long long limit_cycles;          // give up after this many clock64 ticks
    } wait_rows;
};

struct Workspace {            // split-K scratch, owned by the caller
    float* partial = nullptr; // >= partial_floats
    size_t partial_floats = 0;
    uint32_t* counters = nullptr;  // >= 4096 zero-initialised words; the kernel leaves them zero
    int* err = nullptr;       // device error word (0 = ok)
};

// Sets the dynamic shared-memory attribute of every kernel instantiation on the current device (which also loads the
// module image there).  Called once per device at initialisation; launches repeat it only for a device they have not seen.
cudaError_t prepare_device();
// True if (format, shape, pointers) can take the TMA + tcgen05 path.
bool fast_path_ok(const GemmArgs& a);
// Floats of split-K scratch the launch will use (0 when it does not split).
size_t workspace_floats(const GemmArgs& a);
// Enqueue on `stream`.  Returns cudaSuccess or the launch error.
// Single-token path on CUDA cores (qgemv.cu): M == 1, plain standard-layout output, K % 256 == 0.
bool gemv_path_ok(const GemmArgs& a);
cudaError_t launch_gemv(const GemmArgs& a, cudaStream_t stream);
cudaError_t launch(const GemmArgs& a, const Workspace& ws, cudaStream_t stream);
// Few-token path (qgemm_small.cu): weights unpacked straight into tensor memory, K split across a thread-block cluster whose
// CTAs share out the sum of the partial tiles.  Taken for M <= 128 where the persistent kernel would leave SMs idle.
bool small_path_ok(const GemmArgs& a);
size_t small_scratch_floats(const GemmArgs& a);
cudaError_t launch_small(const GemmArgs& a, const Workspace& ws, cudaStream_t stream);
void set_small_kernel_enabled(int mode);     // testing hook: 0 routes those shapes to the persistent kernel again, 1 default,
                                             // 2 takes every shape the kernel can compute (any number of token tiles)
// Number of kernels the last launch() enqueued (1, or 2 with the generic tail) -- for launch accounting.
int last_launch_count();
void set_pair_kernel_enabled(bool on);        // testing hook: off keeps every launch of the persistent kernel on one CTA per MMA
int last_launch_pairs();                      // CTA pairs (cta_group::2) of the last persistent-kernel launch, 0 if it ran without

}  // namespace qg
