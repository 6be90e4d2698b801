// TransformerModel: embedding gather, L decoder layers on one shared coordinator, final RMSNorm, lm_head
// (reference: src/engine/model.py:273-368 for the shape of the loop, :48-63 for the embedding's bounds rule).
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstring>
#include <mutex>
#include <string>
#include <vector>

#include "../../include/b200_bridge.h"
#include "../../include/transformer_model.h"
#include "bridge_state.cuh"
#include "layer_ops.cuh"
#include "peer_reduce.cuh"
#include "qgemm.cuh"

namespace b200_llm {

namespace {
// One CTA per token: copies the token's row of the table (16-byte accesses when rows are 16-byte multiples).  An id
// outside the table reports code 401 through the error word and yields a zero row, so nothing reads out of bounds.
__global__ void __launch_bounds__(128) embedding_gather_kernel(const __half* __restrict__ table, const int32_t* __restrict__ tokens,
                                                               __half* __restrict__ out, uint32_t K, uint32_t vocab, int* err) {
    const int32_t id = tokens[blockIdx.x];
    const bool ok = id >= 0 && (uint32_t)id < vocab;
    if (!ok && threadIdx.x == 0 && err) atomicCAS(err, 0, 401);
    __half* dst = out + (size_t)blockIdx.x * K;
    const __half* src = table + (size_t)(ok ? id : 0) * K;
    if (K % 8 == 0 && ((((uintptr_t)table | (uintptr_t)out) & 15u) == 0)) {
        for (uint32_t i = threadIdx.x; i < K / 8; i += blockDim.x)
            reinterpret_cast<uint4*>(dst)[i] = ok ? reinterpret_cast<const uint4*>(src)[i] : make_uint4(0u, 0u, 0u, 0u);
    } else {
        for (uint32_t i = threadIdx.x; i < K; i += blockDim.x) dst[i] = ok ? src[i] : __half(0.0f);
    }
}
}  // namespace

struct TransformerModel::Impl {
    void *h0 = nullptr, *h1 = nullptr, *xn = nullptr;
    const void* embedding = nullptr;
    const void *final_norm = nullptr, *lm_head = nullptr;
    uint32_t vocab_rows = 0;
    std::vector<LayerWeights> layers;
    peer::Exchange* px = nullptr;
    float* ws = nullptr;             // split-K scratch of the head projection
    size_t ws_floats = 0;
    uint32_t* counters = nullptr;
    int* err = nullptr;
    KernelBinding head_binding;
    cudaStream_t stream = nullptr;
    bool ready = false;
};

TransformerModel::TransformerModel(int device, cudaStream_t stream, const TransformerModelConfig& config)
    : impl_(new Impl), config_(config), device_(device) {
    impl_->stream = stream;
    impl_->layers.resize(config.num_layers);
}

TransformerModel::~TransformerModel() {
    delete layer_;
    void* bufs[] = {impl_->h0, impl_->h1, impl_->xn, impl_->ws, impl_->counters};
    for (void* b : bufs) if (b) cudaFree(b);
    delete impl_;
}

bool TransformerModel::initialize() {
    const TransformerLayerConfig& c = config_.layer;
    if (config_.num_layers == 0 || config_.vocab_size == 0) return false;
    cudaSetDevice(device_);
    layer_ = new TransformerLayerCoordinator(device_, impl_->stream, c);
    if (!layer_->initialize_pipelines(nullptr)) return false;
    const QuantCodecDescriptor* d = QuantRegistry::instance().get(c.weight_format);
    if (!d) return false;
    impl_->head_binding = QuantRegistry::instance().resolve_kernel(d->gemm_kernel_name);
    if (!impl_->head_binding.valid || !impl_->head_binding.implemented) return false;
    const size_t MK = (size_t)c.M * c.K * 2;
    if (cudaMalloc(&impl_->h0, MK) != cudaSuccess || cudaMalloc(&impl_->h1, MK) != cudaSuccess || cudaMalloc(&impl_->xn, MK) != cudaSuccess ||
        cudaMalloc((void**)&impl_->counters, 4096 * 4 + 64) != cudaSuccess) { cudaGetLastError(); return false; }
    cudaMemset(impl_->counters, 0, 4096 * 4 + 64);
    impl_->err = bridge::g.err_word ? bridge::g.err_word : reinterpret_cast<int*>(impl_->counters + 4096);
    impl_->ready = true;
    return true;
}

void TransformerModel::set_embedding(const void* table) { impl_->embedding = table; }

bool TransformerModel::set_layer(uint32_t index, const LayerWeights& w) {
    if (index >= config_.num_layers) return false;
    impl_->layers[index] = w;
    return true;
}

bool TransformerModel::set_head(const void* final_norm, const void* lm_head, uint32_t vocab_rows) {
    if (!lm_head || vocab_rows == 0 || vocab_rows > config_.vocab_size) return false;
    const TransformerLayerConfig& c = config_.layer;
    // split-K scratch for the head projection at this width (few-token prefills split K)
    qg::GemmArgs a; memset(&a, 0, sizeof(a));
    a.format = c.weight_format; a.M = c.M; a.N = vocab_rows; a.K = c.K;
    a.X = (const void*)16; a.W0 = (const void*)16; a.Y = (void*)16;     // alignment probes only
    const size_t need = qg::workspace_floats(a);
    if (need > impl_->ws_floats) {
        if (impl_->ws) { cudaStreamSynchronize(impl_->stream); cudaFree(impl_->ws); impl_->ws = nullptr; impl_->ws_floats = 0; }
        if (cudaMalloc((void**)&impl_->ws, need * 4) != cudaSuccess) { cudaGetLastError(); return false; }
        impl_->ws_floats = need;
    }
    impl_->final_norm = final_norm; impl_->lm_head = lm_head; impl_->vocab_rows = vocab_rows;
    return true;
}

uint32_t TransformerModel::vocab_rows() const { return impl_->vocab_rows; }

bool TransformerModel::attach_peer_exchange(peer::Exchange* shared) {
    if (!layer_ || !layer_->attach_peer_exchange(shared)) return false;
    impl_->px = shared;
    return true;
}

int TransformerModel::forward(cudaStream_t stream, const int32_t* tokens, void* logits, void* hidden) {
    Impl& im = *impl_;
    const TransformerLayerConfig& c = config_.layer;
    launches_ = 0;
    if (!im.ready) return -1;
    if (!tokens || !im.embedding) return -2;
    if (logits && !im.lm_head) return -2;
    if (c.rms_eps > 0.0f && logits && !im.final_norm) return -2;
    for (const LayerWeights& w : im.layers) {
        if (!w.w_q || !w.w_k || !w.w_v || !w.w_o || !w.w_gate || !w.w_up || !w.w_down) return -2;
        if (c.rms_eps > 0.0f && (!w.attn_norm || !w.mlp_norm)) return -2;
    }
    // With the fused exchange the hidden state lives in this rank's copy of the exchange's second result buffer: every
    // layer reads its input there and the owners' reductions write the layer's output there (no copy between layers;
    // a rank's reads of a layer's input are all enqueued before the projection whose arrival the writers wait for).
    void* cur = im.px ? im.px->out[1][im.px->rank] : im.h0;
    void* nxt = im.px ? cur : im.h1;
    embedding_gather_kernel<<<c.M, 128, 0, stream>>>((const __half*)im.embedding, tokens, (__half*)cur, c.K, config_.vocab_size, im.err);
    if (cudaGetLastError() != cudaSuccess) return -6;
    launches_++;
    for (const LayerWeights& w : im.layers) {
        if (c.rms_eps > 0.0f) layer_->set_norm_weights(w.attn_norm, w.mlp_norm);
        layer_->forward(stream, cur, w.w_q, w.w_k, w.w_v, w.w_o, w.w_gate, w.w_up, w.w_down, nxt);
        if (layer_->last_status()) return layer_->last_status();
        launches_ += layer_->kernels_per_forward();
        void* t = cur; cur = nxt; nxt = t;
    }
    if (hidden) {
        if (cudaMemcpyAsync(hidden, cur, (size_t)c.M * c.K * 2, cudaMemcpyDeviceToDevice, stream) != cudaSuccess) { cudaGetLastError(); return -6; }
    }
    if (logits) {
        const void* x = cur;
        if (c.rms_eps > 0.0f) {
            if (lops::rmsnorm(cur, im.final_norm, im.xn, c.M, c.K, c.rms_eps, stream) != cudaSuccess) return -6;
            launches_++;
            x = im.xn;
        }
        qg::GemmArgs a; memset(&a, 0, sizeof(a));
        a.format = im.head_binding.format; a.X = x; a.W0 = im.lm_head; a.Y = logits; a.M = c.M; a.N = im.vocab_rows; a.K = c.K;
        a.layout = im.head_binding.layout;
        qg::Workspace ws;
        ws.partial = im.ws; ws.partial_floats = im.ws_floats; ws.counters = im.counters; ws.err = im.err;
        if (qg::launch(a, ws, stream) != cudaSuccess) { cudaGetLastError(); return -6; }
        launches_ += (uint32_t)qg::last_launch_count();
    }
    return 0;
}

}  // namespace b200_llm

// ---------------------------------------------------------------------------------------------
// C ABI
// ---------------------------------------------------------------------------------------------
using namespace bridge;
using b200_llm::TransformerModel;

namespace {
struct ModelHandle {
    TransformerModel* model = nullptr;
    void (*py_fn)(void*, void*, size_t) = nullptr;
    void* py_ctx = nullptr;
    DevBuf stage_tokens, stage_logits, stage_hidden;
};
void model_allreduce_trampoline(void* ctx, float* buf, size_t count, cudaStream_t) {
    ModelHandle* h = (ModelHandle*)ctx;
    h->py_fn(h->py_ctx, buf, count);
}
// device pointer as is, registered host buffer -> its device copy, anything else -> nullptr
const void* resident(const void* p) {
    if (!p) return nullptr;
    if (is_device_ptr(p)) return p;
    auto it = g.registered.find(p);
    return it == g.registered.end() ? nullptr : it->second.dev;
}
}  // namespace

extern "C" {

void* b200_model_create(const b200_model_config* cfg) {
    std::lock_guard<std::mutex> lock(g.mu);
    if (!g.initialized || !cfg) return nullptr;
    b200_llm::TransformerModelConfig mc;
    b200_llm::TransformerLayerConfig& c = mc.layer;
    const b200_layer_config& l = cfg->layer;
    c.M = l.M; c.K = l.K; c.H = l.H; c.D = l.D; c.N_mlp = l.N_mlp; c.attn_scale = l.attn_scale;
    c.weight_format = (QuantFormat)l.weight_format; c.num_kv_heads = l.num_kv_heads; c.rms_eps = l.rms_eps;
    c.rope_theta = l.rope_theta; c.kv_q8_0 = l.kv_q8_0 != 0; c.tp_size = l.tp_size ? l.tp_size : 1;
    mc.num_layers = cfg->num_layers; mc.vocab_size = cfg->vocab_size;
    ModelHandle* h = new ModelHandle;
    h->model = new TransformerModel(g.device, g.stream, mc);
    if (!h->model->initialize()) {
        set_error("model: initialisation failed (format without a projection kernel, bad shape, or out of device memory)");
        delete h->model; delete h;
        return nullptr;
    }
    return h;
}

void b200_model_destroy(void* model) {
    if (!model) return;
    std::lock_guard<std::mutex> lock(g.mu);
    ModelHandle* h = (ModelHandle*)model;
    if (g.initialized) cudaStreamSynchronize(g.stream);
    h->stage_tokens.release(); h->stage_logits.release(); h->stage_hidden.release();
    delete h->model;
    delete h;
}

int b200_model_set_embedding(void* model, const void* table) {
    std::lock_guard<std::mutex> lock(g.mu);
    if (!model) return -2;
    const void* t = resident(table);
    if (!t) return -2;
    ((ModelHandle*)model)->model->set_embedding(t);
    return 0;
}

int b200_model_set_layer(void* model, uint32_t index, const void* w_q, const void* w_k, const void* w_v, const void* w_o,
                         const void* w_gate, const void* w_up, const void* w_down, const void* attn_norm, const void* mlp_norm) {
    std::lock_guard<std::mutex> lock(g.mu);
    if (!model) return -2;
    b200_llm::LayerWeights w;
    w.w_q = resident(w_q); w.w_k = resident(w_k); w.w_v = resident(w_v); w.w_o = resident(w_o);
    w.w_gate = resident(w_gate); w.w_up = resident(w_up); w.w_down = resident(w_down);
    w.attn_norm = resident(attn_norm); w.mlp_norm = resident(mlp_norm);
    if (!w.w_q || !w.w_k || !w.w_v || !w.w_o || !w.w_gate || !w.w_up || !w.w_down) return -2;
    if ((attn_norm && !w.attn_norm) || (mlp_norm && !w.mlp_norm)) return -2;
    return ((ModelHandle*)model)->model->set_layer(index, w) ? 0 : -4;
}

int b200_model_set_head(void* model, const void* final_norm, const void* lm_head, uint32_t vocab_rows) {
    std::lock_guard<std::mutex> lock(g.mu);
    if (!model) return -2;
    const void* n = resident(final_norm);
    const void* w = resident(lm_head);
    if (!w || (final_norm && !n)) return -2;
    return ((ModelHandle*)model)->model->set_head(n, w, vocab_rows) ? 0 : -4;
}

int b200_model_attach_peer_exchange(void* model, void* exchange) {
    std::lock_guard<std::mutex> lock(g.mu);
    if (!g.initialized) return -1;
    if (!model || !exchange) return -2;
    return ((ModelHandle*)model)->model->attach_peer_exchange((peer::Exchange*)exchange) ? 0 : -4;
}

int b200_model_set_allreduce(void* model, void (*fn)(void*, void*, size_t), void* ctx) {
    if (!model || !fn) return -2;
    ModelHandle* h = (ModelHandle*)model;
    h->py_fn = fn; h->py_ctx = ctx;
    h->model->layer()->set_allreduce(model_allreduce_trampoline, h);
    return 0;
}

int b200_model_forward(void* model, const int32_t* tokens, uint32_t n_tokens, void* logits, void* hidden) {
    std::lock_guard<std::mutex> lock(g.mu);
    if (!g.initialized) return -1;
    if (!model || !tokens) return -2;
    ModelHandle* h = (ModelHandle*)model;
    const auto& mc = h->model->config();
    const auto& c = mc.layer;
    if (n_tokens != c.M) return -4;
    const int32_t* tok_dev = tokens;
    if (!is_device_ptr(tokens)) {
        for (uint32_t i = 0; i < n_tokens; i++)
            if (tokens[i] < 0 || (uint32_t)tokens[i] >= mc.vocab_size) {
                set_error("token id " + std::to_string(tokens[i]) + " at position " + std::to_string(i) + " is outside the vocabulary [0, " +
                          std::to_string(mc.vocab_size) + ")");
                return -8;
            }
        int rc = 0;
        tok_dev = (const int32_t*)resolve_in(tokens, (size_t)n_tokens * 4, h->stage_tokens, false, &rc);
        if (rc) return rc;
    }
    int rc = 0;
    void *logits_host = nullptr, *hidden_host = nullptr, *lg = nullptr, *hd = nullptr;
    const size_t logit_bytes = (size_t)c.M * h->model->vocab_rows() * 2, hid_bytes = (size_t)c.M * c.K * 2;
    if (logits && h->model->vocab_rows() == 0) return -2;
    if (logits) { lg = resolve_out(logits, logit_bytes, h->stage_logits, &logits_host, &rc); if (rc) return rc; }
    if (hidden) { hd = resolve_out(hidden, hid_bytes, h->stage_hidden, &hidden_host, &rc); if (rc) return rc; }
    rc = h->model->forward(g.stream, tok_dev, lg, hd);
    if (rc) return rc;
    g.launches += h->model->kernels_per_forward();
    if (hidden_host && copy_back(hidden_host, hd, hid_bytes) != 0) return -5;
    if (logits_host && copy_back(logits_host, lg, logit_bytes) != 0) return -5;
    return 0;
}

uint32_t b200_model_kernels_per_forward(void* model) { return model ? ((ModelHandle*)model)->model->kernels_per_forward() : 0; }

}  // extern "C"
