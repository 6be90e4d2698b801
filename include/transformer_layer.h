// Decoder-layer API.
//
// Same shape as the reference's models/transformer_layer.h:12-69: a config struct, a coordinator
// whose constructor allocates the intermediates, initialize_pipelines() that binds the projection
// kernels through the registry's kernel names, and forward() that only *enqueues* the layer (the
// caller synchronises), taking X_in, the seven weight buffers and X_out.  Metal objects become
// CUDA ones: device -> device ordinal, queue / command buffer -> cudaStream_t, MTLBuffer ->
// device pointer.
//
// Semantics follow the reference's CPU layer (bench_8b_engine.mm:74-225): QKV head-major
// projections, causal attention, O projection with X_mid = fp16(X + O), fused SwiGLU, down
// projection with X_out = fp16(X_mid + down).  The extra config fields default to that behaviour
// (multi-head attention, no normalisation, no rotary embedding, fp16 KV, one GPU) and add what the
// reference's Python block has (src/engine/model.py:181-270): RMSNorm, grouped-query attention,
// rotary embedding; plus the Q8_0 KV cache of its benches and tensor parallelism.
#pragma once
#ifdef __cplusplus
#include <cstddef>
#include <cstdint>

#include "quant_registry.h"

typedef struct CUstream_st* cudaStream_t;
namespace peer { struct Exchange; }

namespace b200_llm {

struct TransformerLayerConfig {
    uint32_t M = 128;            // tokens
    uint32_t K = 2048;           // hidden size
    uint32_t H = 32;             // query heads (of the whole model, before tensor-parallel split)
    uint32_t D = 64;             // head size
    uint32_t N_mlp = 8192;       // MLP width (whole model)
    float attn_scale = 0.125f;
    QuantFormat weight_format = QUANT_Q4_0;
    // ---- additions (defaults reproduce the reference layer) ----
    uint32_t num_kv_heads = 0;   // 0 = H (multi-head attention)
    float rms_eps = 0.0f;        // > 0 enables RMSNorm before attention and before the MLP
    float rope_theta = 0.0f;     // > 0 enables rotary embedding on Q and K
    bool kv_q8_0 = false;        // compress K and V to Q8_0 before attention
    uint32_t tp_size = 1;        // tensor-parallel ranks; weights passed to forward() are this rank's shards
};

// Sum-reduce `count` fp32 values in place across the tensor-parallel group, ordered on `stream`.
typedef void (*AllReduceFn)(void* ctx, float* buf, size_t count, cudaStream_t stream);

class TransformerLayerCoordinator {
public:
    TransformerLayerCoordinator(int device, cudaStream_t stream, const TransformerLayerConfig& config);
    ~TransformerLayerCoordinator();
    TransformerLayerCoordinator(const TransformerLayerCoordinator&) = delete;
    TransformerLayerCoordinator& operator=(const TransformerLayerCoordinator&) = delete;

    // Resolve the registry's kernel names for config.weight_format.  `library` is ignored (kernels are
    // compiled in).  False if the format has no projection kernel or allocation failed.
    bool initialize_pipelines(const void* library = nullptr);

    // fp16 [K] RMSNorm weights (device pointers); required when rms_eps > 0.
    void set_norm_weights(const void* attn_norm, const void* mlp_norm);
    // required when tp_size > 1 (unless the peer exchange below is set)
    void set_allreduce(AllReduceFn fn, void* ctx);
    // Tensor-parallel reduction fused into the row-split projections: their epilogue scatters fp32 partial rows
    // straight into the owning rank's receive buffer over NVLink, the owner adds them and the residual and writes
    // the fp16 rows into every rank's result buffer.  All pointers are mapped into this process (peer / IPC
    // mappings for the other ranks): recv[o] fp32 [world][M/world][K], out0[o] / out1[o] fp16 [M][K] (result of the
    // O and down projections), flags[o] 16 zero-initialised words.  Needs M / world to be a multiple of 256.
    bool set_peer_exchange(uint32_t rank, uint32_t world, void* const* recv, void* const* out0, void* const* out1,
                           void* const* flags);
    // The same exchange shared with other layers (b200_peer_exchange_create): epoch, flags and counters belong to the
    // buffers, so the layers of a model take turns on one set of buffers.  With RMSNorm enabled the owner of a row
    // normalises it before sending it out, i.e. the residual stream is sharded by rows between the two reductions.
    bool attach_peer_exchange(peer::Exchange* shared);

    // Per-launch timing: with profiling on, forward() records a CUDA event after every launch; profile() returns, for
    // the last forward, up to `cap` (label, microseconds) pairs in launch order (the caller synchronises first).
    void set_profiling(bool on);
    // Rotary embedding and Q8_0 K/V compression in the epilogue of the grouped Q/K/V projection (taken where that launch
    // runs without a K split) instead of one pass over Q, K and V behind the projection (the default, which measures
    // faster).  The results are bit-identical either way.
    void set_fused_kv_epilogue(bool on);
    size_t profile(const char** labels, float* us, size_t cap) const;

    // Enqueue one layer on `stream`.  All pointers are device pointers.  Weight shapes for rank r of
    // tp_size: W_q [H/tp*D][K], W_k/W_v [Hkv/tp*D][K], W_o [K][H/tp*D], W_gate/W_up [N_mlp/tp][K],
    // W_down [K][N_mlp/tp], each in weight_format with rows contiguous along the input dimension.
    void forward(cudaStream_t stream, const void* X_in, const void* W_q, const void* W_k, const void* W_v,
                 const void* W_o, const void* W_gate, const void* W_up, const void* W_down, void* X_out);

    const TransformerLayerConfig& config() const { return config_; }
    int last_status() const { return status_; }           // 0, or the first error of the last forward()
    uint32_t kernels_per_forward() const { return launches_; }

private:
    struct Impl;
    Impl* impl_;
    TransformerLayerConfig config_;
    int device_;
    int status_ = 0;
    uint32_t launches_ = 0;
};

}  // namespace b200_llm

#else   /* C callers see the C entry points below only */
#include <stddef.h>
#include <stdint.h>
#endif

#ifdef __cplusplus
extern "C" {
#endif
typedef struct {
    uint32_t M, K, H, D, N_mlp;
    float attn_scale;
    int weight_format;
    uint32_t num_kv_heads;
    float rms_eps;
    float rope_theta;
    int kv_q8_0;
    uint32_t tp_size;
} b200_layer_config;

/* Create on the bridge's device and stream (m4_bridge_init first).  NULL on failure. */
void* b200_layer_create(const b200_layer_config* cfg);
void b200_layer_destroy(void* layer);
int b200_layer_set_norm_weights(void* layer, const void* attn_norm, const void* mlp_norm);
/* fn(ctx, device fp32 buffer, count): called from forward() on the calling thread, between
 * enqueued kernels; it must order its work on the bridge stream (b200_bridge_stream()). */
int b200_layer_set_allreduce(void* layer, void (*fn)(void* ctx, void* buf, size_t count), void* ctx);
/* X_in / X_out may be host or device pointers; weights must be device pointers or host buffers
 * registered with b200_bridge_register_weights.  Returns 0 or a bridge error code. */
int b200_layer_forward(void* layer, const void* X_in, const void* W_q, const void* W_k, const void* W_v,
                       const void* W_o, const void* W_gate, const void* W_up, const void* W_down, void* X_out);
uint32_t b200_layer_kernels_per_forward(void* layer);

/* ---- tensor-parallel exchange over peer memory (no counterpart in the reference, which is single-device) ---- */
/* Device memory that other processes of the node can map: allocates `bytes` (zero-filled) and writes a 64-byte
 * handle to pass to the peers; the peers map it with b200_peer_open.  Return 0 or -5. */
int b200_peer_alloc(size_t bytes, void** ptr, unsigned char* handle64);
int b200_peer_open(const unsigned char* handle64, void** ptr);
int b200_peer_close(void* ptr);
int b200_peer_free(void* ptr);
/* See TransformerLayerCoordinator::set_peer_exchange; arrays of `world` pointers indexed by rank. */
int b200_layer_set_peer_exchange(void* layer, uint32_t rank, uint32_t world, void* const* recv, void* const* out0,
                                 void* const* out1, void* const* flags);
/* One exchange for several layers (the layers of a model run one after the other on the same buffers): create it from
 * the same pointer arrays, attach it to each layer, destroy it after the layers.  NULL / -4 on bad arguments.
 * partial_fp16 != 0: the partial sums of a row-split projection cross NVLink as fp16 instead of fp32 (half the bytes; each
 * rank's partial is rounded to fp16 once before the owner adds them in fp32); every rank of a group must pass the same value. */
void* b200_peer_exchange_create(uint32_t rank, uint32_t world, void* const* recv, void* const* out0, void* const* out1,
                                void* const* flags, int partial_fp16);
void b200_peer_exchange_destroy(void* exchange);
int b200_layer_attach_peer_exchange(void* layer, void* exchange);
/* Per-launch timing of the next forward calls (CUDA events between launches); b200_layer_profile waits for the stream
 * and writes up to `cap` labels (label_bytes each, NUL-terminated) and durations in microseconds; returns the count. */
int b200_layer_set_profiling(void* layer, int on);
int b200_layer_set_fused_kv_epilogue(void* layer, int on);
int b200_layer_profile(void* layer, char* labels, size_t label_bytes, float* us, size_t cap);
/* The three steps on their own (device pointers): partial sums of Y = X.W^T scattered to the owners' receive
 * buffers; the owner's reduction + residual + broadcast into out[]; the wait for every rank's rows. */
int b200_peer_gemm_scatter(const void* X, const void* W, int format, uint32_t M, uint32_t K, uint32_t N, uint32_t rank,
                           uint32_t world, void* const* recv, void* const* flags, uint32_t epoch);
int b200_peer_reduce_broadcast(uint32_t rank, uint32_t world, void* const* recv, void* const* out, void* const* flags,
                               uint32_t epoch, const void* residual, uint32_t M, uint32_t K);
int b200_peer_wait_rows(uint32_t rank, uint32_t world, void* const* flags, uint32_t epoch);
/* The owner's reduction with the normalisation that follows it fused in: this rank's rows of fp16(residual + sum) go to
 * the local buffer `keep` ([M][K]), rmsnorm(those rows) * norm_w (fp16 [K]) to every rank's out[]. */
int b200_peer_reduce_norm_broadcast(uint32_t rank, uint32_t world, void* const* recv, void* const* out, void* const* flags,
                                    uint32_t epoch, const void* residual, uint32_t M, uint32_t K, const void* norm_w, float eps,
                                    void* keep);
/* Bound of the exchange's flag waits in milliseconds (0 restores the default of about ten seconds).  A wait that runs
 * out sets device error 301 (arrival flags) or 302 (result rows) and the kernel returns; later waits return at once
 * until the error word is cleared. */
void b200_peer_set_wait_limit_ms(unsigned ms);
/* Partial-sum type of the three primitive entry points above: 0 fp32 (default), != 0 fp16 (the receive buffers then hold
 * fp16 [world][M / world][N]). */
void b200_peer_set_partial_fp16(int on);
#ifdef __cplusplus
}
#endif
