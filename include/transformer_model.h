// Multi-layer model loop over the decoder layer: token embedding, L decoder layers, final RMSNorm, lm_head.
//
// Shape of the reference's TransformerModel (src/engine/model.py:273-368): an fp16 embedding table gathered by
// token id (out-of-range ids are an error, model.py:60-63), num_layers TransformerBlocks run one after the other on
// the hidden state, a final RMSNorm, and the lm_head projection to vocab_size logits through the same quantised
// Linear as every other projection.  Here all layers share one TransformerLayerCoordinator (one set of intermediates
// for the whole model; per-layer state is nine weight pointers), the hidden state ping-pongs between two buffers,
// and the whole prefill is enqueued on one stream without a host synchronisation between layers.
//
// forward() is the stateless prefill of the reference's use_cache = False path (model.py:224-229: rotary positions
// from 0, keys and values of this call only).  Tensor parallel: the layers' weights are this rank's shards as for
// TransformerLayerCoordinator::forward, lm_head holds this rank's rows of the vocabulary (logits come out column-
// split, no collective), the embedding table is replicated.
#pragma once
#ifdef __cplusplus
#include <cstddef>
#include <cstdint>

#include "transformer_layer.h"

namespace b200_llm {

struct TransformerModelConfig {
    TransformerLayerConfig layer;      // M = tokens per prefill call; K, H, D, N_mlp, format, GQA, eps, theta, KV format, tp
    uint32_t num_layers = 4;
    uint32_t vocab_size = 1024;
};

struct LayerWeights {                  // device pointers; shapes as for TransformerLayerCoordinator::forward
    const void *w_q = nullptr, *w_k = nullptr, *w_v = nullptr, *w_o = nullptr, *w_gate = nullptr, *w_up = nullptr, *w_down = nullptr;
    const void *attn_norm = nullptr, *mlp_norm = nullptr;     // fp16 [K]; required when rms_eps > 0
};

class TransformerModel {
public:
    TransformerModel(int device, cudaStream_t stream, const TransformerModelConfig& config);
    ~TransformerModel();
    TransformerModel(const TransformerModel&) = delete;
    TransformerModel& operator=(const TransformerModel&) = delete;

    bool initialize();                                        // allocates the hidden-state buffers and the shared layer coordinator
    void set_embedding(const void* table_f16);                // [vocab_size][K] fp16
    bool set_layer(uint32_t index, const LayerWeights& w);
    // final_norm: fp16 [K] (required when rms_eps > 0); lm_head: packed [vocab_rows][K/blk] in the layers' weight format
    // (vocab_rows = vocab_size, or this rank's share of it)
    bool set_head(const void* final_norm, const void* lm_head, uint32_t vocab_rows);
    bool attach_peer_exchange(peer::Exchange* shared);        // tensor parallel with the fused exchange (else set_allreduce on layer())

    // Enqueue the prefill of config.layer.M tokens.  tokens: int32 device pointer.  logits: fp16 [M][vocab_rows] or
    // nullptr (skip the head); hidden: fp16 [M][K] copy of the last layer's output, or nullptr.  Returns 0 or a bridge
    // error code; a token id outside [0, vocab_size) sets device error 401 (its row is gathered as zeros).
    int forward(cudaStream_t stream, const int32_t* tokens, void* logits, void* hidden);

    TransformerLayerCoordinator* layer() { return layer_; }
    const TransformerModelConfig& config() const { return config_; }
    uint32_t kernels_per_forward() const { return launches_; }
    uint32_t vocab_rows() const;                              // rows of the lm_head given to set_head (0 before)

private:
    struct Impl;
    Impl* impl_;
    TransformerLayerCoordinator* layer_ = nullptr;
    TransformerModelConfig config_;
    int device_;
    uint32_t launches_ = 0;
};

}  // namespace b200_llm

#else   /* C callers see the C entry points below only */
#include <stddef.h>
#include <stdint.h>
#include "transformer_layer.h"
#endif

#ifdef __cplusplus
extern "C" {
#endif
typedef struct {
    b200_layer_config layer;
    uint32_t num_layers, vocab_size;
} b200_model_config;

/* No counterpart in the reference's C ABI (its model loop is Python, src/engine/model.py:273-368); these entry points put
 * that loop behind the same library.  Create on the bridge's device and stream (m4_bridge_init first). */
void* b200_model_create(const b200_model_config* cfg);
void b200_model_destroy(void* model);
/* Weights: device pointers, or host buffers registered with b200_bridge_register_weights.  0, -2 (null / unknown
 * pointer) or -4 (index out of range). */
int b200_model_set_embedding(void* model, const void* table_f16);
int b200_model_set_layer(void* model, uint32_t index, const void* w_q, const void* w_k, const void* w_v, const void* w_o,
                         const void* w_gate, const void* w_up, const void* w_down, const void* attn_norm, const void* mlp_norm);
int b200_model_set_head(void* model, const void* final_norm, const void* lm_head, uint32_t vocab_rows);
int b200_model_attach_peer_exchange(void* model, void* exchange);
/* fn as for b200_layer_set_allreduce (tensor parallel without the fused exchange). */
int b200_model_set_allreduce(void* model, void (*fn)(void* ctx, void* buf, size_t count), void* ctx);
/* tokens: n_tokens int32 ids, host or device pointer, n_tokens == layer.M.  Host ids are checked before anything is
 * enqueued: -8 if one lies outside [0, vocab_size) (the reference raises IndexError, src/engine/model.py:60-63).
 * logits (fp16 [M][vocab_rows]) and hidden (fp16 [M][K]) may be host or device pointers or NULL. */
int b200_model_forward(void* model, const int32_t* tokens, uint32_t n_tokens, void* logits, void* hidden);
uint32_t b200_model_kernels_per_forward(void* model);
#ifdef __cplusplus
}
#endif
