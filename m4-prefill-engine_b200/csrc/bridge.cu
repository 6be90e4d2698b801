// C ABI of the bridge (include/b200_bridge.h): argument validation in the reference's order
// (core/bridge/m4_mlx_bridge.mm:194-230), host/device pointer resolution, staging, and dispatch
// onto the kernels.  One compute stream plus two copy streams for host buffers; a mutex guards all state, as in the reference
// (core/bridge/m4_mlx_bridge.mm:20,84,284-287).
#include <cuda_runtime.h>

#include <atomic>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <string>
#include <unordered_map>

#include "../../include/b200_bridge.h"
#include "../../include/quant_router.h"
#include "bridge_state.cuh"
#include "layer_ops.cuh"
#include "qgemm.cuh"

namespace bridge {

State g;

bool DevBuf::ensure(size_t n) {
    if (n <= cap) return true;
    if (p) cudaFree(p);        // implicit device sync: nothing in flight still uses the old block
    p = nullptr; cap = 0;
    size_t want = n + n / 4;
    if (cudaMalloc(&p, want) != cudaSuccess) { cudaGetLastError(); p = nullptr; return false; }
    cap = want;
    return true;
}
void DevBuf::release() { if (p) cudaFree(p); p = nullptr; cap = 0; }

void set_error(const std::string& s) { g.last_error = s; }

bool is_device_ptr(const void* ptr) {
    cudaPointerAttributes at;
    if (cudaPointerGetAttributes(&at, ptr) != cudaSuccess) { cudaGetLastError(); return false; }
    return at.type == cudaMemoryTypeDevice || at.type == cudaMemoryTypeManaged;
}

// Device address for an input buffer: the pointer itself when it is device memory, the
// registered device copy when it is a registered host weight buffer, else a staged copy.
const void* resolve_in(const void* ptr, size_t bytes, DevBuf& stage, bool weights, int* rc) {
    if (is_device_ptr(ptr)) return ptr;
    if (weights) {
        auto it = g.registered.find(ptr);
        if (it != g.registered.end() && it->second.bytes >= bytes) return it->second.dev;
    }
    // a projection's copy back may still be writing the host buffer this call reads
    for (StageSlot& sl : g.slots)
        if (sl.out_pending) cudaStreamWaitEvent(g.stream, sl.ev_out, 0);
    if (!stage.ensure(bytes)) { *rc = -5; return nullptr; }
    if (cudaMemcpyAsync(stage.p, ptr, bytes, cudaMemcpyHostToDevice, g.stream) != cudaSuccess) {
        cudaGetLastError(); *rc = -5; return nullptr;
    }
    g.h2d_bytes += bytes;
    return stage.p;
}

// Device address to write an output into; `*host_dst` is set when a copy back is needed.
void* resolve_out(void* ptr, size_t bytes, DevBuf& stage, void** host_dst, int* rc) {
    *host_dst = nullptr;
    if (is_device_ptr(ptr)) return ptr;
    if (!stage.ensure(bytes)) { *rc = -5; return nullptr; }
    *host_dst = ptr;
    return stage.p;
}

int copy_back(void* host_dst, const void* dev_src, size_t bytes) {
    if (cudaMemcpyAsync(host_dst, dev_src, bytes, cudaMemcpyDeviceToHost, g.stream) != cudaSuccess) { cudaGetLastError(); return -5; }
    g.d2h_bytes += bytes;
    cudaEventRecord(g.ev_main_d2h, g.stream);
    g.main_d2h_pending = true;
    g.main_d2h_seq = ++g.dispatch_seq;
    return 0;
}

namespace {

inline bool overlaps(const void* a, size_t an, const char* b, size_t bn) {
    const char* ac = static_cast<const char*>(a);
    return b && ac < b + bn && b < ac + an;
}

// Host input of a pipelined projection call: staged on the copy-in stream into the slot's buffer.
const void* stage_in(const void* ptr, size_t bytes, StageSlot& sl, DevBuf& buf, bool weights, bool* staged, int* rc) {
    if (is_device_ptr(ptr)) return ptr;
    if (weights) {
        auto it = g.registered.find(ptr);
        if (it != g.registered.end() && it->second.bytes >= bytes) return it->second.dev;
    }
    // ordering through host memory: an earlier call's result may still be on its way into this buffer
    for (StageSlot& o : g.slots)
        if (o.out_pending && overlaps(ptr, bytes, o.out_ptr, o.out_bytes)) cudaStreamWaitEvent(g.stream_in, o.ev_out, 0);
    if (!*staged) {     // first upload of this call: the slot's buffers must be free, earlier host results complete
        if (sl.used) cudaStreamWaitEvent(g.stream_in, sl.ev_kernel, 0);
        if (g.main_d2h_pending) cudaStreamWaitEvent(g.stream_in, g.ev_main_d2h, 0);
    }
    if (!buf.ensure(bytes)) { *rc = -5; return nullptr; }
    if (cudaMemcpyAsync(buf.p, ptr, bytes, cudaMemcpyHostToDevice, g.stream_in) != cudaSuccess) { cudaGetLastError(); *rc = -5; return nullptr; }
    g.h2d_bytes += bytes;
    *staged = true;
    return buf.p;
}

}  // namespace

bool ensure_workspace(size_t floats) {
    if (floats == 0) return true;
    if (!g.ws_partial.ensure(floats * sizeof(float))) return false;
    return true;
}

int validate_gemm(const void* X, size_t Xb, const void* W, size_t Wb, const void* Y, size_t Yb, int format, bool extended,
                  uint32_t M, uint32_t K, uint32_t N) {
    if (!g.initialized) return -1;
    if (!X || !W || !Y) return -2;
    if (((uintptr_t)X % 2 != 0) || ((uintptr_t)Y % 2 != 0)) return -2;
    const bool base_fmt = format >= 0 && format < 6;
    const bool ext_fmt = extended && (format == QUANT_PRISM_Q2_0 || format == QUANT_MLX_4BIT_G64 || format == QUANT_TERNARY_ROW ||
                                     format == QUANT_MLX_4BIT_PLANAR);
    if (!base_fmt && !ext_fmt) return -3;
    if (M == 0 || K == 0 || N == 0) return -4;
    if ((K % 32) != 0) return -4;
    if ((format == 2 || format == 4 || format == 5) && (K % 256) != 0) return -4;
    if (format == QUANT_PRISM_Q2_0 && (K % 128) != 0) return -4;
    if (format == QUANT_MLX_4BIT_G64 && (K % 64) != 0) return -4;
    const size_t min_x = (size_t)M * K * 2, min_y = (size_t)M * N * 2;
    const size_t min_w = compute_quant_matrix_bytes((QuantFormat)format, K, N);
    if (Xb < min_x || Yb < min_y || Wb < min_w) return -2;
    return 0;
}

int run_gemm(void* X, size_t Xb, void* W0, void* W1, size_t Wb, void* Y, size_t Yb, int format, uint32_t M, uint32_t K,
             uint32_t N, int layout, uint32_t H, uint32_t D, void* residual) {
    int rc = 0;
    const size_t x_bytes = (size_t)M * K * 2, y_bytes = (size_t)M * N * 2;
    const size_t w_bytes = compute_quant_matrix_bytes((QuantFormat)format, K, N);
    qg::GemmArgs a;
    memset(&a, 0, sizeof(a));
    a.format = format;
    // Host buffers go through one of two staging sets, uploads on the copy-in stream, the download on the
    // copy-out stream; consecutive calls alternate sets, so call i+1 uploads while call i computes and downloads.
    // The slot's buffers are reused two calls later: its uploads wait for the kernel that last read them, its
    // kernel waits for the download that last read its output buffer.
    StageSlot& sl = g.slots[g.slot_seq & 1u];
    bool staged_in = false;
    a.X = stage_in(X, x_bytes, sl, sl.x, false, &staged_in, &rc);
    if (rc) return rc;
    a.W0 = stage_in(W0, w_bytes, sl, sl.w0, true, &staged_in, &rc);
    if (rc) return rc;
    if (W1) { a.W1 = stage_in(W1, w_bytes, sl, sl.w1, true, &staged_in, &rc); if (rc) return rc; }
    if (residual) { a.residual = stage_in(residual, y_bytes, sl, sl.res, false, &staged_in, &rc); if (rc) return rc; }
    void* host_dst = nullptr;
    if (is_device_ptr(Y)) {
        a.Y = Y;
    } else {
        if (!sl.y.ensure(y_bytes)) return -5;
        a.Y = sl.y.p;
        host_dst = Y;
    }
    a.M = M; a.N = N; a.K = K; a.layout = layout; a.H = H; a.D = D;
    a.force_generic = g.force_generic;
    (void)Xb; (void)Wb; (void)Yb;
    if (!ensure_workspace(qg::workspace_floats(a))) return -5;
    if (staged_in) {
        cudaEventRecord(sl.ev_in, g.stream_in);
        cudaStreamWaitEvent(g.stream, sl.ev_in, 0);
    }
    if (host_dst && sl.out_pending) cudaStreamWaitEvent(g.stream, sl.ev_out, 0);
    qg::Workspace ws;
    ws.partial = (float*)g.ws_partial.p; ws.partial_floats = g.ws_partial.cap / sizeof(float);
    ws.counters = g.counters; ws.err = g.err_word;
    cudaError_t e = qg::launch(a, ws, g.stream);
    if (e != cudaSuccess) { set_error(std::string("kernel launch failed: ") + cudaGetErrorString(e)); return -6; }
    g.launches += (uint64_t)qg::last_launch_count();
    if (staged_in || host_dst) {
        cudaEventRecord(sl.ev_kernel, g.stream);
        sl.used = true;
        g.slot_seq++;
    }
    if (host_dst) {
        cudaStreamWaitEvent(g.stream_out, sl.ev_kernel, 0);
        if (cudaMemcpyAsync(host_dst, a.Y, y_bytes, cudaMemcpyDeviceToHost, g.stream_out) != cudaSuccess) { cudaGetLastError(); return -5; }
        cudaEventRecord(sl.ev_out, g.stream_out);
        sl.out_pending = true; sl.out_ptr = static_cast<const char*>(host_dst); sl.out_bytes = y_bytes;
        sl.out_seq = ++g.dispatch_seq;
        g.d2h_bytes += y_bytes;
    }
    return 0;
}

// Everything the bridge has enqueued, on all three streams (caller holds no lock-protected references).
cudaError_t sync_all_streams(cudaStream_t main, cudaStream_t in, cudaStream_t out) {
    cudaError_t e = cudaStreamSynchronize(in);
    cudaError_t e2 = cudaStreamSynchronize(main);
    cudaError_t e3 = cudaStreamSynchronize(out);
    return e != cudaSuccess ? e : (e2 != cudaSuccess ? e2 : e3);
}

}  // namespace bridge

using namespace bridge;

extern "C" {

bool m4_bridge_init(const char*) {
    std::lock_guard<std::mutex> lock(g.mu);
    if (g.initialized) return true;
    int ndev = 0;
    if (cudaGetDeviceCount(&ndev) != cudaSuccess || ndev == 0) {
        cudaGetLastError();
        set_error("no CUDA device: this library has no CPU path");
        return false;
    }
    cudaGetDevice(&g.device);
    cudaDeviceProp prop;
    cudaGetDeviceProperties(&prop, g.device);
    if (prop.major != 10) {
        set_error("kernels are built for sm_100a only; found sm_" + std::to_string(prop.major) + std::to_string(prop.minor));
        return false;
    }
    if (cudaStreamCreateWithFlags(&g.stream, cudaStreamNonBlocking) != cudaSuccess ||
        cudaStreamCreateWithFlags(&g.stream_in, cudaStreamNonBlocking) != cudaSuccess ||
        cudaStreamCreateWithFlags(&g.stream_out, cudaStreamNonBlocking) != cudaSuccess) { cudaGetLastError(); return false; }
    bool ev_ok = cudaEventCreateWithFlags(&g.ev_main_d2h, cudaEventDisableTiming) == cudaSuccess;
    for (StageSlot& sl : g.slots) {
        ev_ok = ev_ok && cudaEventCreateWithFlags(&sl.ev_in, cudaEventDisableTiming) == cudaSuccess &&
                cudaEventCreateWithFlags(&sl.ev_kernel, cudaEventDisableTiming) == cudaSuccess &&
                cudaEventCreateWithFlags(&sl.ev_out, cudaEventDisableTiming) == cudaSuccess;
        sl.used = false; sl.out_pending = false; sl.out_ptr = nullptr; sl.out_bytes = 0;
    }
    if (!ev_ok) { cudaGetLastError(); return false; }
    g.slot_seq = 0; g.main_d2h_pending = false;
    if (cudaMalloc(&g.counters, 4096 * sizeof(uint32_t) + 64) != cudaSuccess) { cudaGetLastError(); return false; }
    cudaMemsetAsync(g.counters, 0, 4096 * sizeof(uint32_t) + 64, g.stream);
    g.err_word = reinterpret_cast<int*>(g.counters + 4096);
    cudaStreamSynchronize(g.stream);
    // everything that makes the driver load code or reserve memory happens here, not in a later dispatch: the kernels'
    // shared-memory attributes (which load the module image) and the static scratch array of the allocation-free entry point
    if (qg::prepare_device() != cudaSuccess) { cudaGetLastError(); set_error("setting kernel attributes failed"); return false; }
    static_scratch_prepare(g.device);
    g.launches = 0; g.h2d_bytes = 0; g.d2h_bytes = 0; g.dispatch_seq = 0;
    g.initialized = true;
    return true;
}

size_t m4_bridge_get_expected_weight_bytes(int format, uint32_t K, uint32_t N) {
    if (format < 0 || format >= 6) return 0;
    return compute_quant_matrix_bytes((QuantFormat)format, K, N);
}

size_t b200_bridge_weight_bytes(int format, uint32_t K, uint32_t N) {
    if (!((format >= 0 && format < 6) || format == QUANT_PRISM_Q2_0 || format == QUANT_MLX_4BIT_G64 || format == QUANT_TERNARY_ROW ||
          format == QUANT_MLX_4BIT_PLANAR))
        return 0;
    return compute_quant_matrix_bytes((QuantFormat)format, K, N);
}

int m4_bridge_dispatch_gemm(void* X, size_t Xb, void* W, size_t Wb, void* Y, size_t Yb, int format, uint32_t M, uint32_t K,
                            uint32_t N) {
    std::lock_guard<std::mutex> lock(g.mu);
    int rc = validate_gemm(X, Xb, W, Wb, Y, Yb, format, false, M, K, N);
    if (rc) return rc;
    return run_gemm(X, Xb, W, nullptr, Wb, Y, Yb, format, M, K, N, LAYOUT_STANDARD, 0, 0, nullptr);
}

int m4_bridge_dispatch_gemv(void* x, size_t xb, void* W, size_t Wb, void* y, size_t yb, int format, uint32_t K, uint32_t N) {
    return m4_bridge_dispatch_gemm(x, xb, W, Wb, y, yb, format, 1, K, N);
}

int b200_bridge_dispatch_gemm_ex(void* X, size_t Xb, void* W, size_t Wb, void* Y, size_t Yb, int format, uint32_t M, uint32_t K,
                                 uint32_t N, int layout, uint32_t H, uint32_t D, void* residual, size_t residual_bytes) {
    std::lock_guard<std::mutex> lock(g.mu);
    int rc = validate_gemm(X, Xb, W, Wb, Y, Yb, format, true, M, K, N);
    if (rc) return rc;
    if (layout != LAYOUT_STANDARD && layout != LAYOUT_DIRECT_HEAD) return -4;
    if (layout == LAYOUT_DIRECT_HEAD && (H == 0 || D == 0 || (uint64_t)H * D != N)) return -4;
    if (residual) {
        if (layout != LAYOUT_STANDARD) return -4;
        if (((uintptr_t)residual % 2) != 0 || residual_bytes < (size_t)M * N * 2) return -2;
    }
    return run_gemm(X, Xb, W, nullptr, Wb, Y, Yb, format, M, K, N, layout, H, D, residual);
}

int b200_bridge_dispatch_swiglu(void* X, size_t Xb, void* Wg, void* Wu, size_t Wb, void* Out, size_t Ob, int format, uint32_t M,
                                uint32_t K, uint32_t F) {
    std::lock_guard<std::mutex> lock(g.mu);
    if (g.initialized && !Wu) return -2;
    int rc = validate_gemm(X, Xb, Wg, Wb, Out, Ob, format, true, M, K, F);
    if (rc) return rc;
    return run_gemm(X, Xb, Wg, Wu, Wb, Out, Ob, format, M, K, F, LAYOUT_STANDARD, 0, 0, nullptr);
}

int b200_bridge_dispatch_gemm_grouped(const void* X, const void* const* W, void* const* Y, const uint32_t* N, uint32_t count,
                                      int format, uint32_t M, uint32_t K, int layout, uint32_t D) {
    std::lock_guard<std::mutex> lock(g.mu);
    if (!g.initialized) return -1;
    if (!X || !W || !Y || !N || count < 1 || count > 3) return -2;
    if (format < 0 || format >= 6) return -3;
    if (M == 0 || K == 0 || (K % 256) != 0) return -4;
    if (layout != LAYOUT_STANDARD && layout != LAYOUT_DIRECT_HEAD) return -4;
    for (uint32_t i = 0; i < count; i++) {
        if (!W[i] || !Y[i] || !is_device_ptr(W[i]) || !is_device_ptr(Y[i])) return -2;
        if (N[i] == 0 || (layout == LAYOUT_DIRECT_HEAD && (D == 0 || N[i] % D != 0))) return -4;
    }
    if (!is_device_ptr(X)) return -2;
    qg::GemmArgs a;
    memset(&a, 0, sizeof(a));
    a.format = format; a.X = X; a.W0 = W[0]; a.Y = Y[0]; a.M = M; a.N = N[0]; a.K = K; a.layout = layout; a.D = D;
    a.H = layout == LAYOUT_DIRECT_HEAD ? N[0] / D : 0;
    a.n_extra = count - 1;
    for (uint32_t i = 1; i < count; i++) { a.W_extra[i - 1] = W[i]; a.Y_extra[i - 1] = Y[i]; a.N_extra[i - 1] = N[i]; }
    a.force_generic = g.force_generic;
    if (!ensure_workspace(qg::workspace_floats(a))) return -5;      // few-token grouped launches split K
    qg::Workspace ws;
    ws.partial = (float*)g.ws_partial.p; ws.partial_floats = g.ws_partial.cap / sizeof(float);
    ws.counters = g.counters; ws.err = g.err_word;
    cudaError_t e = qg::launch(a, ws, g.stream);
    if (e == cudaErrorInvalidValue) { cudaGetLastError(); return -4; }
    if (e != cudaSuccess) { set_error(std::string("kernel launch failed: ") + cudaGetErrorString(e)); return -6; }
    g.launches += (uint64_t)qg::last_launch_count();
    return 0;
}

int b200_bridge_dispatch_qkv_fused(const void* X, const void* Wq, const void* Wk, const void* Wv, void* Q, void* Kc, void* Vc, int format,
                                   uint32_t M, uint32_t K, uint32_t Hq, uint32_t Hkv, uint32_t D, float rope_theta, uint32_t pos0,
                                   int kv_q8_0, uint32_t kv_tokens) {
    std::lock_guard<std::mutex> lock(g.mu);
    if (!g.initialized) return -1;
    if (!X || !Wq || !Wk || !Wv || !Q || !Kc || !Vc) return -2;
    const void* ptrs[7] = {X, Wq, Wk, Wv, Q, Kc, Vc};
    for (const void* q : ptrs) if (!is_device_ptr(q)) return -2;
    if (format < 0 || format >= 6) return -3;
    if (M == 0 || K == 0 || Hq == 0 || Hkv == 0 || (D != 64 && D != 128) || K % 256 != 0 || Hq % Hkv != 0) return -4;
    if (kv_tokens == 0) kv_tokens = M;
    if (kv_q8_0 ? ((uint64_t)pos0 + M > kv_tokens) : (pos0 != 0 && kv_tokens != M)) return -4;
    if (!kv_q8_0 && kv_tokens != M) return -4;                 // fp16 K/V come out as [Hkv][M][D] of this call only
    qg::GemmArgs a;
    memset(&a, 0, sizeof(a));
    a.format = format; a.X = X; a.W0 = Wq; a.Y = Q; a.M = M; a.N = Hq * D; a.K = K; a.layout = LAYOUT_DIRECT_HEAD; a.H = Hq; a.D = D;
    a.n_extra = 2; a.W_extra[0] = Wk; a.W_extra[1] = Wv; a.Y_extra[0] = Kc; a.Y_extra[1] = Vc; a.N_extra[0] = a.N_extra[1] = Hkv * D;
    const uint32_t rope = rope_theta > 0.0f ? 1u : 0u, q8 = kv_q8_0 ? 2u : 0u;
    a.post[0] = rope; a.post[1] = rope | q8; a.post[2] = q8;
    a.kv_tokens = kv_tokens; a.kv_pos0 = kv_q8_0 ? pos0 : 0u;
    if (rope) {
        // (cos, sin) of positions pos0 .. pos0 + M - 1, rebuilt only when the request changes
        if (g.rope_M != M || g.rope_D != D || g.rope_theta != rope_theta || g.rope_pos0 != pos0 || !g.rope_table.p) {
            cudaStreamSynchronize(g.stream);                  // the table may still be in use by the previous launch
            if (!g.rope_table.ensure((size_t)M * (D / 2) * 8)) return -5;
            if (lops::build_rope_table(g.rope_table.p, M, D, rope_theta, pos0, g.stream) != cudaSuccess) { cudaGetLastError(); return -6; }
            g.rope_M = M; g.rope_D = D; g.rope_theta = rope_theta; g.rope_pos0 = pos0;
            g.launches++;
        }
        a.rope_table = g.rope_table.p;
    }
    if (!a.post[0] && !a.post[1] && !a.post[2]) {}            // nothing to fuse: a plain grouped launch
    if (!ensure_workspace(qg::workspace_floats(a))) return -5;
    qg::Workspace ws;
    ws.partial = (float*)g.ws_partial.p; ws.partial_floats = g.ws_partial.cap / sizeof(float);
    ws.counters = g.counters; ws.err = g.err_word;
    cudaError_t e = qg::launch(a, ws, g.stream);
    if (e == cudaErrorInvalidValue) { cudaGetLastError(); return -4; }
    if (e != cudaSuccess) { set_error(std::string("kernel launch failed: ") + cudaGetErrorString(e)); return -6; }
    g.launches += (uint64_t)qg::last_launch_count();
    return 0;
}

int b200_bridge_register_weights(const void* host_ptr, size_t bytes) {
    std::lock_guard<std::mutex> lock(g.mu);
    if (!g.initialized) return -1;
    if (!host_ptr || bytes == 0) return -2;
    if (is_device_ptr(host_ptr)) return 0;     // already resident
    auto it = g.registered.find(host_ptr);
    if (it != g.registered.end()) { cudaFree(it->second.dev); g.registered.erase(it); }
    void* dev = nullptr;
    if (cudaMalloc(&dev, bytes) != cudaSuccess) { cudaGetLastError(); return -5; }
    if (cudaMemcpyAsync(dev, host_ptr, bytes, cudaMemcpyHostToDevice, g.stream) != cudaSuccess) { cudaGetLastError(); cudaFree(dev); return -5; }
    cudaStreamSynchronize(g.stream);
    g.registered[host_ptr] = Registered{dev, bytes};
    return 0;
}

int b200_bridge_unregister_weights(const void* host_ptr) {
    std::lock_guard<std::mutex> lock(g.mu);
    auto it = g.registered.find(host_ptr);
    if (it == g.registered.end()) return -2;
    sync_all_streams(g.stream, g.stream_in, g.stream_out);
    cudaFree(it->second.dev);
    g.registered.erase(it);
    return 0;
}

void m4_bridge_synchronize(void) {
    // The lock is not held while waiting (dispatches from other threads may go on), so the "copy pending" marks may
    // only be cleared for copies that were already enqueued when the wait began: their events are recorded under the
    // lock before the wait and queried afterwards.  A copy enqueued by another thread in between keeps its mark.
    cudaStream_t s, si, so;
    uint64_t seq_before;
    {
        std::lock_guard<std::mutex> lock(g.mu);
        if (!g.initialized) return;
        s = g.stream; si = g.stream_in; so = g.stream_out;
        seq_before = g.dispatch_seq;
    }
    cudaError_t e = sync_all_streams(s, si, so);
    {
        std::lock_guard<std::mutex> lock(g.mu);
        if (g.initialized) {
            for (StageSlot& sl : g.slots)
                if (sl.out_pending && (sl.out_seq <= seq_before || cudaEventQuery(sl.ev_out) == cudaSuccess)) {
                    sl.out_pending = false; sl.out_ptr = nullptr; sl.out_bytes = 0;
                }
            if (g.main_d2h_pending && (g.main_d2h_seq <= seq_before || cudaEventQuery(g.ev_main_d2h) == cudaSuccess))
                g.main_d2h_pending = false;
            cudaGetLastError();     // cudaErrorNotReady from a query is not an error
        }
    }
    if (e != cudaSuccess) {
        std::lock_guard<std::mutex> lock(g.mu);
        set_error(std::string("stream error: ") + cudaGetErrorString(e));
        fprintf(stderr, "[b200_bridge] %s\n", g.last_error.c_str());
    }
}

double m4_bridge_get_uma_footprint_mb(void) {
    size_t free_b = 0, total_b = 0;
    if (cudaMemGetInfo(&free_b, &total_b) != cudaSuccess) { cudaGetLastError(); return 0.0; }
    return (double)(total_b - free_b) / (1024.0 * 1024.0);
}

bool m4_bridge_is_initialized(void) {
    std::lock_guard<std::mutex> lock(g.mu);
    return g.initialized;
}

void m4_bridge_shutdown(void) {
    std::lock_guard<std::mutex> lock(g.mu);
    if (!g.initialized) return;
    sync_all_streams(g.stream, g.stream_in, g.stream_out);
    for (StageSlot& sl : g.slots) {
        sl.x.release(); sl.w0.release(); sl.w1.release(); sl.res.release(); sl.y.release();
        cudaEventDestroy(sl.ev_in); cudaEventDestroy(sl.ev_kernel); cudaEventDestroy(sl.ev_out);
        sl.ev_in = sl.ev_kernel = sl.ev_out = nullptr; sl.used = false; sl.out_pending = false;
    }
    cudaEventDestroy(g.ev_main_d2h); g.ev_main_d2h = nullptr;
    cudaStreamDestroy(g.stream_in); cudaStreamDestroy(g.stream_out); g.stream_in = g.stream_out = nullptr;
    g.stage_x.release(); g.stage_w0.release(); g.stage_w1.release(); g.stage_y.release(); g.stage_res.release();
    g.stage_aux0.release(); g.stage_aux1.release(); g.stage_aux2.release();
    g.ws_partial.release();
    g.rope_table.release(); g.rope_M = g.rope_D = 0;
    g.kv_fp16.release();
    for (auto& kv : g.registered) cudaFree(kv.second.dev);
    g.registered.clear();
    cudaFree(g.counters); g.counters = nullptr; g.err_word = nullptr;
    cudaStreamDestroy(g.stream); g.stream = nullptr;
    static_scratch_forget();
    g.initialized = false;
}

int b200_bridge_device_error(void) {
    std::lock_guard<std::mutex> lock(g.mu);
    if (!g.initialized) return -1;
    int v = 0;
    cudaStreamSynchronize(g.stream);
    cudaMemcpy(&v, g.err_word, sizeof(int), cudaMemcpyDeviceToHost);
    return v;
}

int b200_bridge_clear_device_error(void) {
    std::lock_guard<std::mutex> lock(g.mu);
    if (!g.initialized) return -1;
    sync_all_streams(g.stream, g.stream_in, g.stream_out);
    // A split-K launch that gave up on a bounded wait leaves its tile counters part-way: the counters and the error
    // word are one block and are cleared together, so the next split-K launch starts from zero again.
    return cudaMemset(g.counters, 0, 4096 * sizeof(uint32_t) + 64) == cudaSuccess ? 0 : -6;
}

/* Testing hook: writes `value` into split-K tile counter `index` (what an aborted split-K launch leaves behind). */
int b200_bridge_debug_set_tile_counter(uint32_t index, uint32_t value) {
    std::lock_guard<std::mutex> lock(g.mu);
    if (!g.initialized) return -1;
    if (index >= 4096) return -2;
    cudaStreamSynchronize(g.stream);
    return cudaMemcpy(g.counters + index, &value, sizeof(uint32_t), cudaMemcpyHostToDevice) == cudaSuccess ? 0 : -6;
}

const char* b200_bridge_last_error_string(void) { return g.last_error.c_str(); }
uint64_t b200_bridge_kernel_launches(void) { return g.launches; }
void* b200_bridge_stream(void) { return (void*)g.stream; }
void b200_bridge_force_generic(int on) { g.force_generic = on; }
void b200_bridge_enable_small_kernel(int on) { qg::set_small_kernel_enabled(on); }
void b200_bridge_enable_pair_kernel(int on) { qg::set_pair_kernel_enabled(on != 0); }
int b200_bridge_last_launch_pair(void) { return qg::last_launch_pairs(); }

}  // extern "C"
