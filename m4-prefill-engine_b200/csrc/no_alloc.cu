// b200_bridge_gemm_scratch_static: the few-token projection GEMM with its split-K scratch in a
// fixed device array that is part of the library image, for callers that must not allocate.
//
// Who needs this.  Some hosts give a plug-in no room to allocate device memory once they are
// running: the host application's own pool already owns the rest of the GPU's memory, so a
// cudaMalloc made inside the library can fail (or succeed only by stalling the host while the
// driver synchronises the device), and latency-critical serving loops forbid that implicit
// synchronisation outright.  The regular entry points grow their split-K scratch (and their
// staging buffers for host pointers) on demand with cudaMalloc; this one never calls cudaMalloc,
// cudaFree or any allocating library routine.  It therefore takes device pointers only, and its
// scratch is the array below, which every GPU that loads the library holds until the process
// exits.
//
// Limits and rules.
//   * The split-K scratch a launch needs (k_splits x tiles x tokens-per-tile x 128 floats) must fit
//     B200_STATIC_SCRATCH_FLOATS; larger requests are refused with -7 and a message, nothing runs.
//   * m4_bridge_init looks up the array's device address (cudaGetSymbolAddress, with the bridge's
//     device current) and sets the kernels' shared-memory attributes, so the module image and the
//     array are resident on the GPU before the host application reserves the rest of its memory:
//     initialise the bridge first.  A first call on another device does the same look-up itself;
//     make it at start-up too, and before any stream capture begins.  m4_bridge_shutdown forgets
//     the cached addresses.
//   * All calls share the one array.  It keeps whatever the previous call left in it; the tile
//     counters, which must start at zero, are cleared on the stream before every launch.  Two calls
//     that overlap on the GPU (different streams, threads or processes sharing the device context)
//     would race on it: issue them one after the other, as the bridge's single stream does.
#include <cuda_runtime.h>

#include <cstring>
#include <mutex>
#include <string>

#include "../../include/b200_bridge.h"
#include "../../include/quant_router.h"
#include "bridge_state.cuh"
#include "qgemm.cuh"

#define B200_STATIC_SCRATCH_FLOATS (3u * 1024u * 1024u)      /* 12 MiB of partial sums */
#define B200_STATIC_COUNTERS 4096u

namespace {

struct StaticScratch {
    float partial[B200_STATIC_SCRATCH_FLOATS];
    uint32_t counters[B200_STATIC_COUNTERS];
};

// Device memory reserved in the library image.  In host code this name is only a handle for
// cudaGetSymbolAddress -- it is not a device address and must never be handed to a kernel.
static __device__ __align__(256) StaticScratch g_static_scratch;

constexpr int MAX_DEVICES = 64;
StaticScratch* g_scratch_addr[MAX_DEVICES] = {nullptr};   // per device, filled on first use
std::mutex g_scratch_mu;

// Device address of the scratch array on the current device (looked up once per device).
cudaError_t scratch_address(int device, StaticScratch** out) {
    std::lock_guard<std::mutex> lock(g_scratch_mu);
    if (device < 0 || device >= MAX_DEVICES) return cudaErrorInvalidDevice;
    if (!g_scratch_addr[device]) {
        void* p = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&p, g_static_scratch);
        if (e != cudaSuccess) return e;
        g_scratch_addr[device] = static_cast<StaticScratch*>(p);
    }
    *out = g_scratch_addr[device];
    return cudaSuccess;
}

}  // namespace

namespace bridge {
// Called by m4_bridge_init (device current): materialises the module image with its scratch array on the GPU and
// caches the array's address, so that no later call of the entry point below makes the driver reserve memory.
bool static_scratch_prepare(int device) {
    StaticScratch* sc = nullptr;
    if (scratch_address(device, &sc) != cudaSuccess) { cudaGetLastError(); return false; }
    return true;
}
// Called by m4_bridge_shutdown: addresses looked up under a context that may be torn down are not kept.
void static_scratch_forget() {
    std::lock_guard<std::mutex> lock(g_scratch_mu);
    for (int i = 0; i < MAX_DEVICES; i++) g_scratch_addr[i] = nullptr;
}
}  // namespace bridge

using namespace bridge;

extern "C" {

int b200_bridge_gemm_scratch_static(void* X, size_t X_bytes, void* W, size_t W_bytes, void* Y, size_t Y_bytes, int format,
                                    uint32_t M, uint32_t K, uint32_t N) {
    std::lock_guard<std::mutex> lock(g.mu);
    if (!g.initialized) return -1;
    if (!X || !W || !Y) return -2;
    if (((uintptr_t)X % 2 != 0) || ((uintptr_t)Y % 2 != 0)) return -2;
    if (format < 0 || format >= 6) return -3;
    if (M == 0 || K == 0 || N == 0 || (K % 32) != 0) return -4;
    if ((format == 2 || format == 4 || format == 5) && (K % 256) != 0) return -4;
    const size_t min_w = compute_quant_matrix_bytes((QuantFormat)format, K, N);
    if (X_bytes < (size_t)M * K * 2 || Y_bytes < (size_t)M * N * 2 || W_bytes < min_w) return -2;
    if (!is_device_ptr(X) || !is_device_ptr(W) || !is_device_ptr(Y)) {
        set_error("b200_bridge_gemm_scratch_static takes device pointers only: staging a host buffer would need an allocation");
        return -2;
    }
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev != g.device) {
        set_error("b200_bridge_gemm_scratch_static: the bridge's device must be the current device");
        return -2;
    }
    qg::GemmArgs a;
    memset(&a, 0, sizeof(a));
    a.format = format; a.X = X; a.W0 = W; a.Y = Y; a.M = M; a.N = N; a.K = K; a.layout = LAYOUT_STANDARD;
    const size_t need = qg::workspace_floats(a);
    if (need > (size_t)B200_STATIC_SCRATCH_FLOATS) {
        set_error("b200_bridge_gemm_scratch_static: this shape needs " + std::to_string(need) +
                  " floats of split-K scratch, the static array holds " + std::to_string(B200_STATIC_SCRATCH_FLOATS));
        return -7;
    }
    StaticScratch* sc = nullptr;
    cudaError_t e = scratch_address(dev, &sc);
    if (e != cudaSuccess) {
        set_error(std::string("cudaGetSymbolAddress failed: ") + cudaGetErrorString(e));
        return -5;
    }
    // the counters must be zero when the kernel starts; the partial sums need no clearing (every
    // element that is read was written by this launch)
    if (cudaMemsetAsync(sc->counters, 0, sizeof(sc->counters), g.stream) != cudaSuccess) { cudaGetLastError(); return -6; }
    qg::Workspace ws;
    ws.partial = sc->partial; ws.partial_floats = B200_STATIC_SCRATCH_FLOATS; ws.counters = sc->counters; ws.err = g.err_word;
    e = qg::launch(a, ws, g.stream);
    if (e != cudaSuccess) { set_error(std::string("kernel launch failed: ") + cudaGetErrorString(e)); return -6; }
    g.launches += (uint64_t)qg::last_launch_count();
    return 0;
}

}  // extern "C"
