/* C ABI of libb200_bridge.so -- the drop-in boundary for the prefill hot path.
 *
 * The first eight entry points keep the names, signatures, error codes and ownership rules of
 * the reference's bridge (core/bridge/m4_mlx_bridge.h:23-106; validation order of
 * core/bridge/m4_mlx_bridge.mm:194-230), so the reference's ctypes wrapper
 * (core/bridge/m4_bridge.py:58-101) binds to this library unchanged.  What differs is where the
 * buffers may live: every pointer may be a CUDA device pointer (used in place, zero-copy) or a
 * host pointer (pinned or pageable; staged to the device inside the call, result copied back on
 * the bridge stream).  Work is enqueued on one internal CUDA stream and the call returns at once;
 * m4_bridge_synchronize() waits for everything enqueued so far.  The caller keeps all buffers
 * alive until then.  The library never frees or retains caller memory.
 *
 * Error codes (core/bridge/m4_mlx_bridge.h:49-56):
 *    0 ok; -1 not initialised; -2 null pointer, X/Y not 2-byte aligned, or a buffer too small;
 *   -3 format outside 0..5; -4 a dimension is 0, K % 32 != 0, or K % 256 != 0 for the
 *   super-block formats 2, 4, 5; -5 device staging allocation failed; -6 kernel launch failed.
 *
 * The b200_bridge_* entry points are extensions for the rest of the hot path (head-major
 * output, fused SwiGLU, Q8_0 KV compression, causal attention over a Q8_0 cache, the decoder
 * layer).  They follow the same pointer and error conventions.
 */
#ifndef B200_BRIDGE_H
#define B200_BRIDGE_H

#include <stdbool.h>
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* core/bridge/m4_mlx_bridge.h:23 -- acquire the device and the stream.  The path argument named a
 * shader library in the reference; kernels are compiled into this library, so it is ignored. */
bool m4_bridge_init(const char* ignored_path);

/* core/bridge/m4_mlx_bridge.h:33 -- bytes of a [N][K] weight matrix in `format` (0..5), 0 if invalid. */
size_t m4_bridge_get_expected_weight_bytes(int format, uint32_t K, uint32_t N);

/* core/bridge/m4_mlx_bridge.h:57 -- Y[M][N] = X[M][K] . dequant(W[N][K])^T, fp16 in/out, fp32 accumulate. */
int m4_bridge_dispatch_gemm(void* X_ptr, size_t X_bytes, void* W_ptr, size_t W_bytes, void* Y_ptr, size_t Y_bytes,
                            int format, uint32_t M, uint32_t K, uint32_t N);

/* core/bridge/m4_mlx_bridge.h:78 -- the same with M = 1 (core/bridge/m4_mlx_bridge.mm:293-302). */
int m4_bridge_dispatch_gemv(void* x_ptr, size_t x_bytes, void* W_ptr, size_t W_bytes, void* y_ptr, size_t y_bytes,
                            int format, uint32_t K, uint32_t N);

/* core/bridge/m4_mlx_bridge.h:88 -- wait for all enqueued work. */
void m4_bridge_synchronize(void);

/* core/bridge/m4_mlx_bridge.h:94 -- memory footprint in MB; here: device memory in use on the bridge's GPU. */
double m4_bridge_get_uma_footprint_mb(void);

/* core/bridge/m4_mlx_bridge.h:99 */
bool m4_bridge_is_initialized(void);

/* core/bridge/m4_mlx_bridge.h:104 -- wait, free staging and scratch memory, forget registered weights. */
void m4_bridge_shutdown(void);

/* ------------------------------------------------------------------------------------------ */
/* Extensions                                                                                 */
/* ------------------------------------------------------------------------------------------ */

/* Formats accepted by the *_ex entry points in addition to 0..5:
 *   7   PRISM_Q2_0 (quant_router.h:93-96)
 *   100 MLX 4-bit, group 64, sequential nibbles, planar: u32 qs[N][K/8] | f16 scale[N][K/64] | f16 bias[N][K/64]
 *   101 ternary, 16 codes per u32, one fp16 scale per row, planar: u32 qs[N][K/16] | f16 scale[N]          */
size_t b200_bridge_weight_bytes(int format, uint32_t K, uint32_t N);

/* GEMM with the reference's LayoutMode (quant_router.h:25-28; the direct-head entry points of
 * quant_router_kernels.metal:754-927): layout 1 writes Y[h][m][d], n = h*D + d, N == H*D.
 * `residual` (may be NULL) is an fp16 [M][N] matrix added to the fp32 accumulator before the
 * single fp16 rounding (the X + O_proj and X_mid + down steps of bench_8b_engine.mm:188-191,215-217);
 * standard layout only. */
int b200_bridge_dispatch_gemm_ex(void* X_ptr, size_t X_bytes, void* W_ptr, size_t W_bytes, void* Y_ptr, size_t Y_bytes,
                                 int format, uint32_t M, uint32_t K, uint32_t N, int layout, uint32_t H, uint32_t D,
                                 void* residual_ptr, size_t residual_bytes);

/* Fused gate/up SwiGLU, Out[M][F] = silu(X.Wg^T) * (X.Wu^T) with the activation on the fp32
 * accumulators (brick3_swiglu_kernels.metal:428-698; gold brick3_swiglu_bench.mm:49-99). */
int b200_bridge_dispatch_swiglu(void* X_ptr, size_t X_bytes, void* Wg_ptr, void* Wu_ptr, size_t W_bytes_each, void* Out_ptr,
                                size_t Out_bytes, int format, uint32_t M, uint32_t K, uint32_t F);

/* Q8_0 KV compression of n_elements fp16 values (n_elements % 32 == 0): 34 bytes out per 32 values,
 * bit-exact with quantize_kv_to_q8_0 (unified_8b_kernels.metal:118-145) and quantize_to_q8_0
 * (brick4_attn_bench.mm:37-55); and its inverse, dequantize_q8_0 (brick4_attn_bench.mm:57-65). */
int b200_bridge_quantize_kv_q8_0(void* src_f16, size_t src_bytes, void* dst_q8, size_t dst_bytes, size_t n_elements);
int b200_bridge_dequantize_q8_0(void* src_q8, size_t src_bytes, void* dst_f16, size_t dst_bytes, size_t n_elements);

/* Causal flash attention over a Q8_0 KV cache (flash_attn_mma_64x64_q8_0_d{64,128},
 * brick4_attn_kernels.metal:573-911; token-major output as flash_attn_q8_0_causal_d128,
 * unified_8b_kernels.metal:857-998).  Q [Hq][M][D] fp16; K, V [Hkv][Mkv][D/32] Q8_0 blocks, or fp16
 * [Hkv][Mkv][D] when kv_fp16 != 0 (the fp16 twin, brick4_attn_kernels.metal:243-522); O [Hq][M][D], or
 * [M][Hq*D] when out_tokens_major != 0.  Query row i is at position pos0 + i and sees keys 0..pos0+i;
 * query head h reads kv head h / (Hq/Hkv).  D is 64 or 128. */
int b200_bridge_dispatch_attention_q8kv(void* Q, void* K, void* V, void* O, uint32_t Hq, uint32_t Hkv, uint32_t M,
                                        uint32_t Mkv, uint32_t D, float scale, uint32_t pos0, int out_tokens_major,
                                        int kv_fp16);

/* RMSNorm as the reference's block applies it (src/engine/model.py:39-45): fp32 mean square,
 * x * rsqrt(var + eps) rounded to fp16, then times the fp16 weight.  X, Y [M][K]; weight [K]. */
int b200_bridge_rmsnorm(void* X, void* weight, void* Y, uint32_t M, uint32_t K, float eps);

/* Rotary embedding in place on X [H][M][D], non-interleaved pairing (i, i + D/2), angle
 * (pos0 + m) * theta^(-2i/D) (src/engine/model.py:112-116 with traditional = False). */
int b200_bridge_rope(void* X, uint32_t H, uint32_t M, uint32_t D, float theta, uint32_t pos0);

/* No counterpart in the reference.  m4_bridge_dispatch_gemm for callers that must not allocate device
 * memory at run time (hosts whose own pool owns the rest of the GPU, latency-critical loops that cannot
 * take the implicit synchronisation of cudaMalloc): same arguments, same result, but device pointers
 * only, and the split-K scratch lives in a 12 MiB device array inside the library image (held by every
 * GPU that loads the library until exit) instead of being allocated on demand.  Never calls cudaMalloc
 * or cudaFree.  Returns -7 (message in b200_bridge_last_error_string) when the shape needs more than
 * 3 Mi floats of scratch, -2 for host pointers.  m4_bridge_init makes the array and the kernels resident on the
 * bridge's GPU, so initialise the bridge at start-up, before the host application reserves the rest of the GPU's
 * memory and before any stream capture.  All calls share the one array (tile
 * counters are cleared on the stream before each launch), so calls that overlap on the GPU would race. */
int b200_bridge_gemm_scratch_static(void* X_ptr, size_t X_bytes, void* W_ptr, size_t W_bytes, void* Y_ptr, size_t Y_bytes,
                                    int format, uint32_t M, uint32_t K, uint32_t N);

/* Upload a host weight buffer once; later dispatches that pass the same host pointer and size
 * use the device copy instead of staging it again.  Returns 0, -2 or -5. */
int b200_bridge_register_weights(const void* host_ptr, size_t bytes);
int b200_bridge_unregister_weights(const void* host_ptr);

/* 0 if no kernel has reported a fault since init; otherwise the first code reported: a bounded wait ran out inside a
 * projection kernel (101..110; 109 the CTA-pair relay, 110 rows another rank had not written), the few-token projection
 * kernel (111..117), an attention kernel (201..204, 210..217) or the peer exchange (301, 302); 401: a token id outside the
 * embedding table. */
int b200_bridge_device_error(void);
const char* b200_bridge_last_error_string(void);

/* Kernels enqueued by this library since init (launch accounting for benchmarks). */
uint64_t b200_bridge_kernel_launches(void);

/* The internal stream as a cudaStream_t, for callers that want to order their own work or
 * time with CUDA events on it. */
void* b200_bridge_stream(void);

/* Testing hook: non-zero routes every GEMM through the CUDA-core fallback kernel. */
/* Clears the device error word after the caller has read it with b200_bridge_device_error (waits for the streams),
 * together with the split-K tile counters, which a launch that gave up on a bounded wait leaves part-way. */
int b200_bridge_clear_device_error(void);
/* Testing hook: writes `value` into split-K tile counter `index` (what an aborted split-K launch leaves behind). */
int b200_bridge_debug_set_tile_counter(uint32_t index, uint32_t value);
void b200_bridge_force_generic(int on);
/* Testing hook: 0 routes few-token projections (M <= 128 with fewer output tiles than SMs) to the persistent kernel
 * instead of the cluster kernel that is their default; 1 restores the default; 2 sends every shape the cluster kernel can
 * compute to it, whatever the token count (one CTA per 128 x 128 output tile, two CTAs per SM). */
void b200_bridge_enable_small_kernel(int on);
/* Testing hook: 0 keeps the persistent projection kernel on one CTA per MMA; != 0 restores the default, CTA pairs
 * (tcgen05 cta_group::2: one 256-row MMA over two SMs) wherever a launch has token tiles of 128 to 256 rows (a multiple of
 * 32), no K split and an even number of weight tiles.  b200_bridge_last_launch_pair returns the number of CTA pairs of the last such launch (0: none). */
void b200_bridge_enable_pair_kernel(int on);
int b200_bridge_last_launch_pair(void);
/* Up to three projections of the same activations in one launch (the Q, K and V projections of a layer): Y[i] =
 * X . W[i]^T with W[i] packed [N[i]][K/blk] in `format`, outputs in `layout` (LAYOUT_DIRECT_HEAD: [N[i]/D][M][D]).
 * Device pointers only, K % 256 == 0, formats 0..5; returns -4 where a grouped launch is not available (the caller then
 * dispatches the projections one by one).  Few-token launches split K as a single projection would.  Results are
 * bit-identical to separate dispatches that run the same split.  No counterpart in the reference. */
int b200_bridge_dispatch_gemm_grouped(const void* X, const void* const* W, void* const* Y, const uint32_t* N, uint32_t count,
                                      int format, uint32_t M, uint32_t K, int layout, uint32_t D);
/* Q, K and V projections of one block in one launch with the K/V-cache work fused into the epilogue: head-major outputs
 * (the reference's LAYOUT_DIRECT_HEAD scatter, quant_router_kernels.metal:570-575), rotary embedding on Q and K at
 * positions pos0 .. pos0+M-1 (rope_theta > 0; src/engine/model.py:218-226) and, with kv_q8_0 != 0, K and V written straight
 * into a Q8_0 cache (quantize_kv_to_q8_0, unified_8b_kernels.metal:118-145; cache update of src/engine/modules.py:628-729):
 * Kc / Vc are then block_q8_0 [Hkv][kv_tokens][D/32] and this call fills tokens pos0 .. pos0+M-1 of every head (kv_tokens
 * == 0 means M).  Without kv_q8_0, Kc / Vc are fp16 [Hkv][M][D].  Q is fp16 [Hq][M][D].  Device pointers, formats 0..5,
 * D 64 or 128, K % 256 == 0.  Bit-identical to the projections followed by b200_bridge_rope and
 * b200_bridge_quantize_kv_q8_0.  Returns -4 where the fused launch is not available (few tokens: the planner splits K). */
int b200_bridge_dispatch_qkv_fused(const void* X, const void* Wq, const void* Wk, const void* Wv, void* Q, void* Kc, void* Vc, int format,
                                   uint32_t M, uint32_t K, uint32_t Hq, uint32_t Hkv, uint32_t D, float rope_theta, uint32_t pos0,
                                   int kv_q8_0, uint32_t kv_tokens);
/* Testing hook, so that the attention kernels can be compared on the same inputs: 1 routes head-dim-128 attention to the
 * warp-level MMA kernels; 2 and 3 to the tensor-memory kernel that unpacks the Q8_0 tiles itself (2: V transposed in shared
 * memory, 3: V in its natural form); 0 restores the default (Q8_0 cache dequantised once per call, tiles through TMA). */
void b200_bridge_force_legacy_attention(int on);
/* Kernels the last attention dispatch enqueued (2 when a Q8_0 cache was dequantised first). */
int b200_bridge_attention_launches(void);

#ifdef __cplusplus
}
#endif
#endif /* B200_BRIDGE_H */
