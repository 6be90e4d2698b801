// TransformerLayerCoordinator: composition of the hot-path kernels into one decoder layer
// (reference: models/transformer_layer.mm:7-218 for the shape of the class,
// bench_8b_engine.mm:74-225 for what the layer computes and where it rounds to fp16).
#include <cuda_runtime.h>

#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <string>
#include <vector>

#include "../../include/b200_bridge.h"
#include "../../include/transformer_layer.h"
#include "bridge_state.cuh"
#include "layer_ops.cuh"
#include "peer_reduce.cuh"
#include "qgemm.cuh"

namespace b200_llm {

struct TransformerLayerCoordinator::Impl {
    // intermediates (device)
    void *xn = nullptr, *q = nullptr, *k = nullptr, *v = nullptr, *kq = nullptr, *vq = nullptr;
    void *attn = nullptr, *x_mid = nullptr, *act = nullptr;
    void* rope_table = nullptr;      // (cos, sin) [M][D/2] of positions 0..M-1 for the fused rotation in the Q/K/V epilogue
    float* partial = nullptr;        // tensor-parallel partial sums [M][K]
    float* ws = nullptr;             // split-K scratch
    size_t ws_floats = 0;
    uint32_t* counters = nullptr;
    int* err = nullptr;
    const void *norm1 = nullptr, *norm2 = nullptr;
    AllReduceFn allreduce = nullptr;
    void* allreduce_ctx = nullptr;
    KernelBinding gemm_binding, head_binding;
    peer::Exchange own_px;           // exchange attached with set_peer_exchange (buffers of this layer alone)
    peer::Exchange* px = nullptr;    // the exchange in use: &own_px, or one shared by the layers of a model (nullptr: none)
    bool bound = false;
    cudaStream_t stream = nullptr;
    // per-launch timing of one forward (profile_forward): an event after every launch
    bool fuse_kv = false;            // rotary embedding and Q8_0 K/V in the Q/K/V projection's epilogue (where that launch allows it)
                                     // instead of one launch behind it; same bits, and measured slower: the work lands on the
                                     // epilogue warps, which share issue slots with the unpack and MMA warps
    bool profiling = false;
    std::vector<cudaEvent_t> events;
    std::vector<std::string> labels;
    size_t n_marks = 0;
};

static bool dev_alloc(void** p, size_t bytes) {
    if (cudaMalloc(p, bytes ? bytes : 16) != cudaSuccess) { cudaGetLastError(); *p = nullptr; return false; }
    return true;
}

TransformerLayerCoordinator::TransformerLayerCoordinator(int device, cudaStream_t stream, const TransformerLayerConfig& config)
    : impl_(new Impl), config_(config), device_(device) {
    if (config_.num_kv_heads == 0) config_.num_kv_heads = config_.H;
    if (config_.tp_size == 0) config_.tp_size = 1;
    impl_->stream = stream;
}

TransformerLayerCoordinator::~TransformerLayerCoordinator() {
    void* bufs[] = {impl_->xn, impl_->q, impl_->k, impl_->v, impl_->kq, impl_->vq, impl_->attn, impl_->x_mid, impl_->act,
                    impl_->partial, impl_->ws, impl_->counters, impl_->own_px.done_counter, impl_->rope_table};
    for (void* b : bufs) if (b) cudaFree(b);
    for (cudaEvent_t e : impl_->events) cudaEventDestroy(e);
    delete impl_;
}

bool TransformerLayerCoordinator::initialize_pipelines(const void*) {
    const TransformerLayerConfig& c = config_;
    const QuantCodecDescriptor* d = QuantRegistry::instance().get(c.weight_format);
    if (!d) { status_ = -3; return false; }
    impl_->gemm_binding = QuantRegistry::instance().resolve_kernel(d->gemm_kernel_name);
    impl_->head_binding = QuantRegistry::instance().resolve_kernel(d->head_gemm_kernel_name);
    if (!impl_->gemm_binding.valid || !impl_->gemm_binding.implemented || !impl_->head_binding.valid ||
        !impl_->head_binding.implemented) { status_ = -3; return false; }
    if (c.M == 0 || c.K == 0 || c.H == 0 || c.D == 0 || c.N_mlp == 0) { status_ = -4; return false; }
    if (c.H % c.tp_size || c.num_kv_heads % c.tp_size || c.N_mlp % c.tp_size || c.H % c.num_kv_heads) { status_ = -4; return false; }
    if (c.D != 64 && c.D != 128) { status_ = -4; return false; }
    const uint32_t hq = c.H / c.tp_size, hkv = c.num_kv_heads / c.tp_size, f = c.N_mlp / c.tp_size;
    if (d->block_size && ((c.K % d->block_size) || ((hq * c.D) % d->block_size) || (f % d->block_size))) { status_ = -4; return false; }
    cudaSetDevice(device_);
    const size_t MK = (size_t)c.M * c.K * 2;
    bool ok = dev_alloc(&impl_->xn, MK) && dev_alloc(&impl_->x_mid, MK) &&
              dev_alloc(&impl_->q, (size_t)c.M * hq * c.D * 2) && dev_alloc(&impl_->k, (size_t)c.M * hkv * c.D * 2) &&
              dev_alloc(&impl_->v, (size_t)c.M * hkv * c.D * 2) && dev_alloc(&impl_->attn, (size_t)c.M * hq * c.D * 2) &&
              dev_alloc(&impl_->act, (size_t)c.M * f * 2);
    if (ok && c.kv_q8_0) {
        const size_t qb = (size_t)c.M * hkv * c.D / 32 * 34;
        ok = dev_alloc(&impl_->kq, qb) && dev_alloc(&impl_->vq, qb);
    }
    if (ok && c.tp_size > 1) ok = dev_alloc((void**)&impl_->partial, (size_t)c.M * c.K * 4);
    if (ok && c.rope_theta > 0.0f) {
        ok = dev_alloc(&impl_->rope_table, (size_t)c.M * (c.D / 2) * 8) &&
             lops::build_rope_table(impl_->rope_table, c.M, c.D, c.rope_theta, 0, impl_->stream) == cudaSuccess;
    }
    // split-K scratch: sized for the largest projection of this layer (tokens <= 256 per tile)
    if (ok) {
        size_t need = 0;
        const uint32_t ns[4] = {hq * c.D, hkv * c.D, c.K, f};
        const uint32_t ks[4] = {c.K, c.K, hq * c.D, c.K};
        for (int i = 0; i < 4; i++) {
            qg::GemmArgs a; memset(&a, 0, sizeof(a));
            a.format = c.weight_format; a.M = c.M; a.N = ns[i]; a.K = ks[i];
            a.X = (const void*)16; a.W0 = (const void*)16; a.Y = (void*)16;   // alignment probes only
            size_t w = qg::workspace_floats(a);
            if (w > need) need = w;
        }
        {   // the grouped Q + K + V launch
            qg::GemmArgs a; memset(&a, 0, sizeof(a));
            a.format = c.weight_format; a.M = c.M; a.N = hq * c.D; a.K = c.K; a.layout = LAYOUT_DIRECT_HEAD; a.H = hq; a.D = c.D;
            a.X = (const void*)16; a.W0 = (const void*)16; a.Y = (void*)16;
            a.n_extra = 2; a.W_extra[0] = a.W_extra[1] = (const void*)16; a.Y_extra[0] = a.Y_extra[1] = (void*)16;
            a.N_extra[0] = a.N_extra[1] = hkv * c.D;
            const size_t w = qg::workspace_floats(a);
            if (w > need) need = w;
        }
        { qg::GemmArgs a; memset(&a, 0, sizeof(a)); a.format = c.weight_format; a.M = c.M; a.N = c.K; a.K = f;
          a.X = (const void*)16; a.W0 = (const void*)16; a.Y = (void*)16; size_t w = qg::workspace_floats(a); if (w > need) need = w; }
        impl_->ws_floats = need;
        if (need) ok = dev_alloc((void**)&impl_->ws, need * 4);
        if (ok) ok = dev_alloc((void**)&impl_->counters, 4096 * 4 + 64);
        if (ok) {
            cudaMemset(impl_->counters, 0, 4096 * 4 + 64);
            impl_->err = reinterpret_cast<int*>(impl_->counters + 4096);
        }
    }
    if (!ok) { status_ = -5; return false; }
    impl_->bound = true;
    status_ = 0;
    return true;
}

void TransformerLayerCoordinator::set_norm_weights(const void* a, const void* m) { impl_->norm1 = a; impl_->norm2 = m; }
void TransformerLayerCoordinator::set_allreduce(AllReduceFn fn, void* ctx) { impl_->allreduce = fn; impl_->allreduce_ctx = ctx; }

bool TransformerLayerCoordinator::set_peer_exchange(uint32_t rank, uint32_t world, void* const* recv, void* const* out0,
                                                    void* const* out1, void* const* flags) {
    const TransformerLayerConfig& c = config_;
    if (world != c.tp_size || world < 2 || world > 8 || rank >= world || c.M % world != 0 || (c.M / world) % 256 != 0) return false;
    peer::Exchange& x = impl_->own_px;
    if (!x.done_counter) {
        if (!dev_alloc((void**)&x.done_counter, 64)) return false;
        cudaMemset(x.done_counter, 0, 64);
    }
    for (uint32_t o = 0; o < world; o++) {
        if (!recv[o] || !out0[o] || !out1[o] || !flags[o]) return false;
        x.recv[o] = (float*)recv[o]; x.out[0][o] = out0[o]; x.out[1][o] = out1[o]; x.flags[o] = (uint32_t*)flags[o];
    }
    x.rank = rank; x.world = world;
    // The epoch belongs to the buffers, not to the layer: flags only grow, and buffers that have been used before
    // (by this layer or another one) hold the last epoch of that use.  An idle exchange has the same value in every
    // flag word of every rank, so this rank's own word tells where to continue.
    uint32_t seen = 0;
    cudaStreamSynchronize(impl_->stream);
    if (cudaMemcpy(&seen, x.flags[rank] + rank, sizeof(uint32_t), cudaMemcpyDeviceToHost) != cudaSuccess) { cudaGetLastError(); return false; }
    x.epoch = seen;
    impl_->px = &x;
    return true;
}

bool TransformerLayerCoordinator::attach_peer_exchange(peer::Exchange* shared) {
    const TransformerLayerConfig& c = config_;
    if (!shared || shared->world != c.tp_size || shared->world < 2 || c.M % shared->world != 0 || (c.M / shared->world) % 256 != 0 ||
        !shared->done_counter)
        return false;
    impl_->px = shared;       // epoch, flags and counters live with the buffers: any number of layers may take turns on them
    return true;
}

void TransformerLayerCoordinator::set_profiling(bool on) { impl_->profiling = on; }
void TransformerLayerCoordinator::set_fused_kv_epilogue(bool on) { impl_->fuse_kv = on; }

size_t TransformerLayerCoordinator::profile(const char** labels, float* us, size_t cap) const {
    const Impl& im = *impl_;
    if (im.n_marks < 2) return 0;
    size_t n = 0;
    for (size_t i = 1; i < im.n_marks && n < cap; i++, n++) {
        float ms = 0.0f;
        if (cudaEventElapsedTime(&ms, im.events[i - 1], im.events[i]) != cudaSuccess) { cudaGetLastError(); ms = -1.0f; }
        us[n] = ms * 1000.0f;
        labels[n] = im.labels[i].c_str();
    }
    return n;
}

void TransformerLayerCoordinator::forward(cudaStream_t stream, const void* X_in, const void* W_q, const void* W_k,
                                          const void* W_v, const void* W_o, const void* W_gate, const void* W_up,
                                          const void* W_down, void* X_out) {
    const TransformerLayerConfig& c = config_;
    Impl& im = *impl_;
    launches_ = 0;
    if (!im.bound) { status_ = -1; return; }
    if (!X_in || !W_q || !W_k || !W_v || !W_o || !W_gate || !W_up || !W_down || !X_out) { status_ = -2; return; }
    if (c.rms_eps > 0.0f && (!im.norm1 || !im.norm2)) { status_ = -2; return; }
    if (c.tp_size > 1 && !im.allreduce && !im.px) { status_ = -2; return; }
    status_ = 0;
    const uint32_t hq = c.H / c.tp_size, hkv = c.num_kv_heads / c.tp_size, f = c.N_mlp / c.tp_size;
    qg::Workspace ws;
    ws.partial = im.ws; ws.partial_floats = im.ws_floats; ws.counters = im.counters; ws.err = im.err;

    auto gemm = [&](const KernelBinding& kb, const void* X, const void* W0, const void* W1, void* Y, uint32_t N, uint32_t K,
                    uint32_t H, const void* residual, float* partial_out) {
        if (status_) return;
        qg::GemmArgs a; memset(&a, 0, sizeof(a));
        a.format = kb.format; a.X = X; a.W0 = W0; a.W1 = W1; a.Y = Y; a.M = c.M; a.N = N; a.K = K;
        a.layout = kb.layout; a.H = H; a.D = c.D; a.residual = residual; a.partial_out = partial_out;
        if (qg::launch(a, ws, stream) != cudaSuccess) { status_ = -6; return; }
        launches_ += (uint32_t)qg::last_launch_count();
    };
    auto check = [&](cudaError_t e) { if (e != cudaSuccess && !status_) status_ = -6; else launches_++; };
    // profiling: an event after every step; label i names what ran between event i-1 and event i
    im.n_marks = 0;
    auto mark = [&](const char* what) {
        if (!im.profiling) return;
        if (im.n_marks == im.events.size()) {
            cudaEvent_t e = nullptr;
            if (cudaEventCreate(&e) != cudaSuccess) { cudaGetLastError(); return; }
            im.events.push_back(e); im.labels.emplace_back();
        }
        im.labels[im.n_marks] = what;
        cudaEventRecord(im.events[im.n_marks++], stream);
    };
    mark("start");

    // 1. attention block
    const void* x_attn = X_in;
    if (c.rms_eps > 0.0f) { check(lops::rmsnorm(X_in, im.norm1, im.xn, c.M, c.K, c.rms_eps, stream)); x_attn = im.xn; mark("rmsnorm 1"); }
    // Q, K and V read the same activations: one grouped launch (their weight tiles share the persistent grid, so
    // the two narrow projections do not each leave most SMs idle); separate launches where that is not available
    // Where the grouped launch runs without a K split, its epilogue also rotates Q and K (rotary embedding) and writes K
    // and V as Q8_0 records, which removes four launches and a round trip of Q, K and V through memory.
    bool qkv_done = false, kv_fused = false;
    for (int attempt = im.fuse_kv ? 0 : 1; attempt < 2 && !qkv_done && !status_; attempt++) {
        const bool fuse = attempt == 0 && (c.rope_theta > 0.0f || c.kv_q8_0);
        if (attempt == 0 && !fuse) continue;
        qg::GemmArgs a; memset(&a, 0, sizeof(a));
        a.format = im.head_binding.format; a.X = x_attn; a.W0 = W_q; a.Y = im.q; a.M = c.M; a.N = hq * c.D; a.K = c.K;
        a.layout = im.head_binding.layout; a.H = hq; a.D = c.D;
        a.n_extra = 2; a.W_extra[0] = W_k; a.W_extra[1] = W_v; a.Y_extra[0] = im.k; a.Y_extra[1] = im.v;
        a.N_extra[0] = a.N_extra[1] = hkv * c.D;
        if (fuse) {
            const uint32_t rope = c.rope_theta > 0.0f ? 1u : 0u, q8 = c.kv_q8_0 ? 2u : 0u;
            a.post[0] = rope; a.post[1] = rope | q8; a.post[2] = q8;
            a.rope_table = im.rope_table;
            if (q8) { a.Y_extra[0] = im.kq; a.Y_extra[1] = im.vq; }
        }
        if (qg::launch(a, ws, stream) == cudaSuccess) {
            qkv_done = true; kv_fused = fuse;
            launches_ += (uint32_t)qg::last_launch_count();
            mark(fuse ? "q+k+v projections (grouped) with rope and q8_0 kv in the epilogue" : "q+k+v projections (grouped)");
        } else cudaGetLastError();
    }
    if (!qkv_done) {
        gemm(im.head_binding, x_attn, W_q, nullptr, im.q, hq * c.D, c.K, hq, nullptr, nullptr);
        gemm(im.head_binding, x_attn, W_k, nullptr, im.k, hkv * c.D, c.K, hkv, nullptr, nullptr);
        gemm(im.head_binding, x_attn, W_v, nullptr, im.v, hkv * c.D, c.K, hkv, nullptr, nullptr);
        mark("q, k, v projections (3 launches)");
    }
    const void *kk = im.k, *vv = im.v;
    bool kv_as_fp16 = !c.kv_q8_0;
    if (kv_fused) {
        if (c.kv_q8_0) { kk = im.kq; vv = im.vq; }
    } else if ((c.rope_theta > 0.0f || c.kv_q8_0) &&
               lops::kv_post(im.q, im.k, im.v, im.kq, im.vq, im.rope_table, hq, hkv, c.M, c.D, c.rope_theta > 0.0f, c.kv_q8_0, true, stream) == cudaSuccess) {
        // one pass over Q, K and V: rotary embedding, the Q8_0 records, and K and V overwritten by the values the records
        // give back, so that attention over this cache gets its operands as fp16 tiles without unpacking them again
        launches_++;
        kv_as_fp16 = true;
        mark("rope q, k + quantize k, v (one launch)");
    } else {
        cudaGetLastError();
        if (c.rope_theta > 0.0f) {
            check(lops::rope(im.q, hq, c.M, c.D, c.rope_theta, 0, stream));
            check(lops::rope(im.k, hkv, c.M, c.D, c.rope_theta, 0, stream));
            mark("rope q, k");
        }
        if (c.kv_q8_0) {
            check(attn::launch_quantize(im.k, im.kq, (size_t)hkv * c.M * c.D, stream));
            check(attn::launch_quantize(im.v, im.vq, (size_t)hkv * c.M * c.D, stream));
            kk = im.kq; vv = im.vq;
            mark("quantize k, v to q8_0");
        }
    }
    check(attn::launch_attention_simple(im.q, kk, vv, im.attn, hq, hkv, c.M, c.M, c.D, c.attn_scale, 0, 1, kv_as_fp16 ? 1 : 0, stream));
    launches_ += (uint32_t)(attn::last_attention_launches() - 1);
    mark("attention");
    // 2. O projection + first residual
    const void* x_mid = im.x_mid;
    // row-split projection with the reduction fused in: scatter in the epilogue, owner reduces and broadcasts
    // `norm_w` != nullptr: the owner normalises its rows before writing them to every rank and keeps the plain rows
    // (the next block's residual) in `keep`.
    // `defer_wait`: the kernel that consumes the broadcast rows waits for them itself, tile by tile (the gate/up projection's
    // activation loads), instead of a wait kernel in front of it
    auto reduced_gemm = [&](const void* X, const void* W, uint32_t Kin, const void* residual, int which_out, const void* norm_w,
                            void* keep, const char* what, bool defer_wait) {
        if (status_) return;
        peer::Exchange& x = *im.px;
        x.epoch++;
        qg::GemmArgs a; memset(&a, 0, sizeof(a));
        a.format = im.gemm_binding.format; a.X = X; a.W0 = W; a.M = c.M; a.N = c.K; a.K = Kin; a.layout = im.gemm_binding.layout;
        a.scatter.world = x.world; a.scatter.rank = x.rank; a.scatter.rows = c.M / x.world; a.scatter.epoch = x.epoch;
        a.scatter.done_counter = x.done_counter; a.scatter.fp16 = x.partial_fp16 ? 1u : 0u;
        for (uint32_t o = 0; o < x.world; o++) { a.scatter.recv[o] = x.recv[o]; a.scatter.flags[o] = x.flags[o]; }
        if (qg::launch(a, ws, stream) != cudaSuccess) { status_ = -6; return; }
        launches_ += (uint32_t)qg::last_launch_count();
        mark(what);
        check(peer::reduce_broadcast(x, which_out, residual, c.M, c.K, im.err, stream, norm_w, c.rms_eps, keep));
        mark(norm_w ? "owner: sum + residual + rmsnorm -> all ranks" : "owner: sum + residual -> all ranks");
        if (defer_wait) return;
        check(peer::wait_rows(x, im.err, stream));
        mark("wait for all ranks' rows");
    };
    // One GPU with a normalisation after the attention block: the O projection writes its plain fp16 output and the
    // residual add rides on the RMSNorm kernel that has to read that output anyway (the projection's residual epilogue
    // costs about 20 us per launch at M=2048; the extra operand of the normalisation about 3 us).  The block output is
    // fp16(fp16(attn * Wo) + x), the rounding of an unfused add.
    const bool fuse_add_norm = c.tp_size == 1 && c.rms_eps > 0.0f && c.K % 8u == 0u && (reinterpret_cast<uintptr_t>(X_in) & 15u) == 0;
    // fused exchange with a normalisation behind it: the residual stream stays sharded by rows between the two
    // reductions (x_mid holds this rank's rows only) and the rows every rank receives are already normalised
    const bool px_norm = im.px && c.rms_eps > 0.0f && c.K % 1024u == 0u && c.K <= 8192u;
    if (fuse_add_norm) {
        gemm(im.gemm_binding, im.attn, W_o, nullptr, im.xn, c.K, hq * c.D, 0, nullptr, nullptr);
        mark("o projection");
    } else if (c.tp_size == 1) {
        gemm(im.gemm_binding, im.attn, W_o, nullptr, im.x_mid, c.K, hq * c.D, 0, X_in, nullptr);
        mark("o projection + residual");
    } else if (im.px) {
        reduced_gemm(im.attn, W_o, hq * c.D, X_in, 0, px_norm ? im.norm2 : nullptr, px_norm ? im.x_mid : nullptr,
                     "o projection, partial rows scattered to their owners", /*defer_wait=*/px_norm);
        if (!px_norm) x_mid = im.px->out[0][im.px->rank];
    } else {
        gemm(im.gemm_binding, im.attn, W_o, nullptr, nullptr, c.K, hq * c.D, 0, nullptr, im.partial);
        if (!status_) im.allreduce(im.allreduce_ctx, im.partial, (size_t)c.M * c.K, stream);
        check(lops::add_residual_f32(X_in, im.partial, im.x_mid, (size_t)c.M * c.K, stream));
        mark("o projection + all-reduce + residual");
    }
    // 3. MLP
    const void* x_mlp = x_mid;
    if (fuse_add_norm) { check(lops::rmsnorm_add(im.xn, X_in, im.norm2, im.x_mid, im.xn, c.M, c.K, c.rms_eps, stream)); x_mlp = im.xn; mark("residual + rmsnorm 2"); }
    else if (px_norm) x_mlp = im.px->out[0][im.px->rank];
    else if (c.rms_eps > 0.0f) { check(lops::rmsnorm(x_mid, im.norm2, im.xn, c.M, c.K, c.rms_eps, stream)); x_mlp = im.xn; mark("rmsnorm 2"); }
    bool mlp_done = false;
    if (px_norm && !status_) {
        // the normalised rows are still arriving from their owners: the projection waits for each token tile's rows itself
        peer::Exchange& x = *im.px;
        qg::GemmArgs a; memset(&a, 0, sizeof(a));
        a.format = im.gemm_binding.format; a.X = x_mlp; a.W0 = W_gate; a.W1 = W_up; a.Y = im.act; a.M = c.M; a.N = f; a.K = c.K;
        a.layout = im.gemm_binding.layout; a.D = c.D;
        a.wait_rows.flags = x.flags[x.rank] + 8; a.wait_rows.rows = c.M / x.world; a.wait_rows.epoch = x.epoch;
        a.wait_rows.limit_cycles = peer::wait_limit_cycles();
        if (qg::launch(a, ws, stream) == cudaSuccess) {
            launches_ += (uint32_t)qg::last_launch_count();
            mlp_done = true;
        } else {
            cudaGetLastError();
            check(peer::wait_rows(x, im.err, stream));
            mark("wait for all ranks' rows");
        }
    }
    if (!mlp_done) gemm(im.gemm_binding, x_mlp, W_gate, W_up, im.act, f, c.K, 0, nullptr, nullptr);
    mark("gate/up SwiGLU");
    // The MLP block's residual rides in the down projection's epilogue (row-wise: the residual row is read with the same
    // 16-byte-granular accesses the output row is written with).  B200_LAYER_SPLIT_ADD=1 selects the older arrangement, a
    // plain projection followed by a 16-byte-wide add kernel, for comparison.
    static const bool split_add_env = [] { const char* e = getenv("B200_LAYER_SPLIT_ADD"); return e && e[0] == '1'; }();
    const bool split_add = split_add_env && fuse_add_norm && ((size_t)c.M * c.K) % 8u == 0u && (reinterpret_cast<uintptr_t>(X_out) & 15u) == 0;
    if (split_add) {
        gemm(im.gemm_binding, im.act, W_down, nullptr, im.xn, c.K, f, 0, nullptr, nullptr);
        mark("down projection");
        check(lops::add_residual_f16(im.x_mid, im.xn, X_out, (size_t)c.M * c.K, stream));
        mark("residual add");
    } else if (c.tp_size == 1) {
        gemm(im.gemm_binding, im.act, W_down, nullptr, X_out, c.K, f, 0, im.x_mid, nullptr);
        mark("down projection + residual");
    } else if (im.px) {
        // (x_mid: this rank's rows are all the owner's reduction reads)
        reduced_gemm(im.act, W_down, f, x_mid, 1, nullptr, nullptr, "down projection, partial rows scattered to their owners", false);
        // the result sits in this rank's copy of the second result buffer; a caller that hands that very buffer in as
        // X_out (the layers of a model do) needs no copy
        if (!status_ && X_out != im.px->out[1][im.px->rank]) {
            check(cudaMemcpyAsync(X_out, im.px->out[1][im.px->rank], (size_t)c.M * c.K * 2, cudaMemcpyDeviceToDevice, stream));
            mark("copy result out of the exchange buffer");
        }
    } else {
        gemm(im.gemm_binding, im.act, W_down, nullptr, nullptr, c.K, f, 0, nullptr, im.partial);
        if (!status_) im.allreduce(im.allreduce_ctx, im.partial, (size_t)c.M * c.K, stream);
        check(lops::add_residual_f32(im.x_mid, im.partial, X_out, (size_t)c.M * c.K, stream));
        mark("down projection + all-reduce + residual");
    }
}

}  // namespace b200_llm

// ---------------------------------------------------------------------------------------------
// C ABI
// ---------------------------------------------------------------------------------------------
using namespace bridge;
using b200_llm::TransformerLayerCoordinator;

namespace {
struct LayerHandle {
    TransformerLayerCoordinator* layer;
    void (*py_fn)(void*, void*, size_t) = nullptr;
    void* py_ctx = nullptr;
    DevBuf stage_in, stage_out;
};
void allreduce_trampoline(void* ctx, float* buf, size_t count, cudaStream_t) {
    LayerHandle* h = (LayerHandle*)ctx;
    h->py_fn(h->py_ctx, buf, count);
}
}  // namespace

extern "C" {

void* b200_layer_create(const b200_layer_config* cfg) {
    std::lock_guard<std::mutex> lock(g.mu);
    if (!g.initialized || !cfg) return nullptr;
    b200_llm::TransformerLayerConfig c;
    c.M = cfg->M; c.K = cfg->K; c.H = cfg->H; c.D = cfg->D; c.N_mlp = cfg->N_mlp; c.attn_scale = cfg->attn_scale;
    c.weight_format = (QuantFormat)cfg->weight_format; c.num_kv_heads = cfg->num_kv_heads; c.rms_eps = cfg->rms_eps;
    c.rope_theta = cfg->rope_theta; c.kv_q8_0 = cfg->kv_q8_0 != 0; c.tp_size = cfg->tp_size ? cfg->tp_size : 1;
    LayerHandle* h = new LayerHandle;
    h->layer = new TransformerLayerCoordinator(g.device, g.stream, c);
    if (!h->layer->initialize_pipelines(nullptr)) {
        set_error("layer: initialize_pipelines failed with status " + std::to_string(h->layer->last_status()));
        delete h->layer; delete h;
        return nullptr;
    }
    return h;
}

void b200_layer_destroy(void* layer) {
    if (!layer) return;
    std::lock_guard<std::mutex> lock(g.mu);
    LayerHandle* h = (LayerHandle*)layer;
    if (g.initialized) cudaStreamSynchronize(g.stream);
    h->stage_in.release(); h->stage_out.release();
    delete h->layer;
    delete h;
}

int b200_layer_set_norm_weights(void* layer, const void* a, const void* m) {
    if (!layer || !a || !m) return -2;
    ((LayerHandle*)layer)->layer->set_norm_weights(a, m);
    return 0;
}

int b200_layer_set_allreduce(void* layer, void (*fn)(void*, void*, size_t), void* ctx) {
    if (!layer || !fn) return -2;
    LayerHandle* h = (LayerHandle*)layer;
    h->py_fn = fn; h->py_ctx = ctx;
    h->layer->set_allreduce(allreduce_trampoline, h);
    return 0;
}

int b200_layer_forward(void* layer, const void* X_in, const void* W_q, const void* W_k, const void* W_v, const void* W_o,
                       const void* W_gate, const void* W_up, const void* W_down, void* X_out) {
    std::lock_guard<std::mutex> lock(g.mu);
    if (!g.initialized) return -1;
    if (!layer || !X_in || !X_out) return -2;
    LayerHandle* h = (LayerHandle*)layer;
    const auto& c = h->layer->config();
    const size_t bytes = (size_t)c.M * c.K * 2;
    int rc = 0;
    const void* x = resolve_in(X_in, bytes, h->stage_in, false, &rc);
    if (rc) return rc;
    void* host_dst = nullptr;
    void* y = resolve_out(X_out, bytes, h->stage_out, &host_dst, &rc);
    if (rc) return rc;
    const void* w[7] = {W_q, W_k, W_v, W_o, W_gate, W_up, W_down};
    for (int i = 0; i < 7; i++) {
        if (!w[i]) return -2;
        if (!is_device_ptr(w[i])) {
            auto it = g.registered.find(w[i]);
            if (it == g.registered.end()) { set_error("layer weights must be device pointers or registered host buffers"); return -2; }
            w[i] = it->second.dev;
        }
    }
    h->layer->forward(g.stream, x, w[0], w[1], w[2], w[3], w[4], w[5], w[6], y);
    if (h->layer->last_status()) return h->layer->last_status();
    g.launches += h->layer->kernels_per_forward();
    if (host_dst && copy_back(host_dst, y, bytes) != 0) return -5;
    return 0;
}

uint32_t b200_layer_kernels_per_forward(void* layer) { return layer ? ((LayerHandle*)layer)->layer->kernels_per_forward() : 0; }

int b200_layer_set_peer_exchange(void* layer, uint32_t rank, uint32_t world, void* const* recv, void* const* out0,
                                 void* const* out1, void* const* flags) {
    std::lock_guard<std::mutex> lock(g.mu);
    if (!g.initialized) return -1;
    if (!layer || !recv || !out0 || !out1 || !flags) return -2;
    return ((LayerHandle*)layer)->layer->set_peer_exchange(rank, world, recv, out0, out1, flags) ? 0 : -4;
}

void* b200_peer_exchange_create(uint32_t rank, uint32_t world, void* const* recv, void* const* out0, void* const* out1,
                                void* const* flags, int partial_fp16) {
    std::lock_guard<std::mutex> lock(g.mu);
    if (!g.initialized || !recv || !out0 || !out1 || !flags || world < 2 || world > 8 || rank >= world) return nullptr;
    peer::Exchange* x = new peer::Exchange;
    for (uint32_t o = 0; o < world; o++) {
        if (!recv[o] || !out0[o] || !out1[o] || !flags[o]) { delete x; return nullptr; }
        x->recv[o] = (float*)recv[o]; x->out[0][o] = out0[o]; x->out[1][o] = out1[o]; x->flags[o] = (uint32_t*)flags[o];
    }
    x->rank = rank; x->world = world; x->partial_fp16 = partial_fp16 != 0;
    if (cudaMalloc((void**)&x->done_counter, 64) != cudaSuccess) { cudaGetLastError(); delete x; return nullptr; }
    cudaMemset(x->done_counter, 0, 64);
    uint32_t seen = 0;                         // buffers that were used before continue from their last epoch
    cudaStreamSynchronize(g.stream);
    if (cudaMemcpy(&seen, x->flags[rank] + rank, sizeof(uint32_t), cudaMemcpyDeviceToHost) != cudaSuccess) {
        cudaGetLastError(); cudaFree(x->done_counter); delete x; return nullptr;
    }
    x->epoch = seen;
    return x;
}

void b200_peer_exchange_destroy(void* exchange) {
    if (!exchange) return;
    std::lock_guard<std::mutex> lock(g.mu);
    peer::Exchange* x = (peer::Exchange*)exchange;
    if (g.initialized) cudaStreamSynchronize(g.stream);
    if (x->done_counter) cudaFree(x->done_counter);
    delete x;
}

int b200_layer_attach_peer_exchange(void* layer, void* exchange) {
    std::lock_guard<std::mutex> lock(g.mu);
    if (!g.initialized) return -1;
    if (!layer || !exchange) return -2;
    return ((LayerHandle*)layer)->layer->attach_peer_exchange((peer::Exchange*)exchange) ? 0 : -4;
}

int b200_layer_set_fused_kv_epilogue(void* layer, int on) {
    if (!layer) return -2;
    ((LayerHandle*)layer)->layer->set_fused_kv_epilogue(on != 0);
    return 0;
}

int b200_layer_set_profiling(void* layer, int on) {
    if (!layer) return -2;
    ((LayerHandle*)layer)->layer->set_profiling(on != 0);
    return 0;
}

int b200_layer_profile(void* layer, char* labels, size_t label_bytes, float* us, size_t cap) {
    std::lock_guard<std::mutex> lock(g.mu);
    if (!g.initialized) return -1;
    if (!layer || !labels || !us || label_bytes == 0) return -2;
    cudaStreamSynchronize(g.stream);
    std::vector<const char*> names(cap);
    const size_t n = ((LayerHandle*)layer)->layer->profile(names.data(), us, cap);
    for (size_t i = 0; i < n; i++) {
        strncpy(labels + i * label_bytes, names[i], label_bytes - 1);
        labels[i * label_bytes + label_bytes - 1] = 0;
    }
    return (int)n;
}

int b200_peer_alloc(size_t bytes, void** ptr, unsigned char* handle64) {
    std::lock_guard<std::mutex> lock(g.mu);
    if (!g.initialized) return -1;
    if (!ptr || !handle64 || bytes == 0) return -2;
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "the handle travels as 64 bytes");
    void* p = nullptr;
    if (cudaMalloc(&p, bytes) != cudaSuccess) { cudaGetLastError(); return -5; }
    cudaIpcMemHandle_t h;
    if (cudaMemset(p, 0, bytes) != cudaSuccess || cudaIpcGetMemHandle(&h, p) != cudaSuccess) {
        set_error(std::string("b200_peer_alloc: ") + cudaGetErrorString(cudaGetLastError()));
        cudaFree(p);
        return -5;
    }
    memcpy(handle64, &h, 64);
    *ptr = p;
    return 0;
}

int b200_peer_open(const unsigned char* handle64, void** ptr) {
    std::lock_guard<std::mutex> lock(g.mu);
    if (!g.initialized) return -1;
    if (!handle64 || !ptr) return -2;
    cudaIpcMemHandle_t h;
    memcpy(&h, handle64, 64);
    cudaError_t e = cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess);
    if (e != cudaSuccess) { set_error(std::string("cudaIpcOpenMemHandle: ") + cudaGetErrorString(e)); cudaGetLastError(); return -5; }
    return 0;
}

int b200_peer_close(void* ptr) { return ptr && cudaIpcCloseMemHandle(ptr) == cudaSuccess ? 0 : -2; }
int b200_peer_free(void* ptr) { return ptr && cudaFree(ptr) == cudaSuccess ? 0 : -2; }

namespace {
uint32_t* g_peer_counter = nullptr;      // counter words for the primitive entry points below
bool g_peer_partial_fp16 = false;        // partial-sum type of the primitive entry points (b200_peer_set_partial_fp16)
bool peer_counter_ready() {
    if (g_peer_counter) return true;
    if (cudaMalloc((void**)&g_peer_counter, 64) != cudaSuccess) { cudaGetLastError(); g_peer_counter = nullptr; return false; }
    cudaMemsetAsync(g_peer_counter, 0, 64, g.stream);
    return true;
}
}  // namespace

int b200_peer_gemm_scatter(const void* X, const void* W, int format, uint32_t M, uint32_t K, uint32_t N, uint32_t rank,
                           uint32_t world, void* const* recv, void* const* flags, uint32_t epoch) {
    std::lock_guard<std::mutex> lock(g.mu);
    if (!g.initialized) return -1;
    if (!X || !W || !recv || !flags || world < 1 || world > 8 || rank >= world) return -2;
    if (M == 0 || K == 0 || N == 0 || M % world != 0) return -4;
    if (!peer_counter_ready()) return -5;
    qg::GemmArgs a; memset(&a, 0, sizeof(a));
    a.format = format; a.X = X; a.W0 = W; a.M = M; a.N = N; a.K = K; a.layout = LAYOUT_STANDARD;
    a.scatter.world = world; a.scatter.rank = rank; a.scatter.rows = M / world; a.scatter.epoch = epoch;
    a.scatter.done_counter = g_peer_counter; a.scatter.fp16 = g_peer_partial_fp16 ? 1u : 0u;
    for (uint32_t o = 0; o < world; o++) { a.scatter.recv[o] = (float*)recv[o]; a.scatter.flags[o] = (uint32_t*)flags[o]; }
    qg::Workspace ws;
    ws.partial = (float*)g.ws_partial.p; ws.partial_floats = g.ws_partial.cap / sizeof(float); ws.counters = g.counters; ws.err = g.err_word;
    cudaError_t e = qg::launch(a, ws, g.stream);
    if (e != cudaSuccess) { set_error(std::string("gemm_scatter launch failed: ") + cudaGetErrorString(e)); return e == cudaErrorInvalidValue ? -4 : -6; }
    g.launches += (uint64_t)qg::last_launch_count();
    return 0;
}

int b200_peer_reduce_broadcast(uint32_t rank, uint32_t world, void* const* recv, void* const* out, void* const* flags,
                               uint32_t epoch, const void* residual, uint32_t M, uint32_t K) {
    std::lock_guard<std::mutex> lock(g.mu);
    if (!g.initialized) return -1;
    if (!recv || !out || !flags || !residual || world < 1 || world > 8 || rank >= world) return -2;
    if (!peer_counter_ready()) return -5;
    peer::Exchange x;
    x.world = world; x.rank = rank; x.epoch = epoch; x.done_counter = g_peer_counter; x.partial_fp16 = g_peer_partial_fp16;
    for (uint32_t o = 0; o < world; o++) { x.recv[o] = (float*)recv[o]; x.out[0][o] = out[o]; x.flags[o] = (uint32_t*)flags[o]; }
    if (peer::reduce_broadcast(x, 0, residual, M, K, g.err_word, g.stream) != cudaSuccess) { cudaGetLastError(); return -4; }
    g.launches++;
    return 0;
}

int b200_peer_reduce_norm_broadcast(uint32_t rank, uint32_t world, void* const* recv, void* const* out, void* const* flags,
                                    uint32_t epoch, const void* residual, uint32_t M, uint32_t K, const void* norm_w, float eps,
                                    void* keep) {
    std::lock_guard<std::mutex> lock(g.mu);
    if (!g.initialized) return -1;
    if (!recv || !out || !flags || !residual || !norm_w || !keep || world < 1 || world > 8 || rank >= world) return -2;
    if (!peer_counter_ready()) return -5;
    peer::Exchange x;
    x.world = world; x.rank = rank; x.epoch = epoch; x.done_counter = g_peer_counter; x.partial_fp16 = g_peer_partial_fp16;
    for (uint32_t o = 0; o < world; o++) { x.recv[o] = (float*)recv[o]; x.out[0][o] = out[o]; x.flags[o] = (uint32_t*)flags[o]; }
    if (peer::reduce_broadcast(x, 0, residual, M, K, g.err_word, g.stream, norm_w, eps, keep) != cudaSuccess) { cudaGetLastError(); return -4; }
    g.launches++;
    return 0;
}

void b200_peer_set_wait_limit_ms(unsigned ms) { peer::set_wait_limit_ms(ms); }
void b200_peer_set_partial_fp16(int on) { g_peer_partial_fp16 = on != 0; }

int b200_peer_wait_rows(uint32_t rank, uint32_t world, void* const* flags, uint32_t epoch) {
    std::lock_guard<std::mutex> lock(g.mu);
    if (!g.initialized) return -1;
    if (!flags || world < 1 || world > 8 || rank >= world) return -2;
    peer::Exchange x;
    x.world = world; x.rank = rank; x.epoch = epoch;
    for (uint32_t o = 0; o < world; o++) x.flags[o] = (uint32_t*)flags[o];
    if (peer::wait_rows(x, g.err_word, g.stream) != cudaSuccess) { cudaGetLastError(); return -6; }
    g.launches++;
    return 0;
}

}  // extern "C"
