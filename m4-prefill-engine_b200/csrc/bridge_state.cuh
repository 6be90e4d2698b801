// Process-wide state of the bridge, shared by the translation units that implement the C ABI.
#pragma once
#include <cuda_runtime.h>

#include <cstdint>
#include <mutex>
#include <string>
#include <unordered_map>

namespace bridge {

struct DevBuf {                 // grow-only device block
    void* p = nullptr;
    size_t cap = 0;
    bool ensure(size_t n);
    void release();
};

struct Registered { void* dev; size_t bytes; };

// One of two staging sets of the projection entry points.  A call that is handed host buffers copies its
// inputs on the copy-in stream, runs its kernel on the main stream and copies its result back on the copy-out
// stream, so the upload of call i+1 and the download of call i overlap (they use different copy engines).
struct StageSlot {
    DevBuf x, w0, w1, res, y;
    cudaEvent_t ev_in = nullptr, ev_kernel = nullptr, ev_out = nullptr;
    bool used = false;               // ev_kernel has been recorded at least once
    bool out_pending = false;        // a copy back from y has been enqueued since the last synchronize
    const char* out_ptr = nullptr;   // host range that copy writes
    size_t out_bytes = 0;
    uint64_t out_seq = 0;            // State::dispatch_seq when that copy was enqueued
};

struct State {
    std::mutex mu;
    bool initialized = false;
    int device = 0;
    cudaStream_t stream = nullptr;       // kernels (and the staging copies of everything but the projections)
    cudaStream_t stream_in = nullptr;    // host -> device copies of the projection entry points
    cudaStream_t stream_out = nullptr;   // device -> host copies of the projection entry points
    StageSlot slots[2];
    uint64_t slot_seq = 0;
    cudaEvent_t ev_main_d2h = nullptr;   // last copy back issued on the main stream by another entry point
    bool main_d2h_pending = false;
    uint64_t main_d2h_seq = 0;
    uint64_t dispatch_seq = 0;           // counts device -> host copies enqueued; synchronize clears marks up to its snapshot
    DevBuf stage_x, stage_w0, stage_w1, stage_y, stage_res, stage_aux0, stage_aux1, stage_aux2;
    DevBuf ws_partial;          // split-K partial tiles
    DevBuf kv_fp16;             // K and V of the last Q8_0 attention call, dequantised once per call (attention.cu)
    DevBuf rope_table;          // (cos, sin) table of the last fused Q/K/V dispatch, and the request it was built for
    uint32_t rope_M = 0, rope_D = 0, rope_pos0 = 0;
    float rope_theta = 0.0f;
    uint32_t* counters = nullptr;  // 4096 tile counters (kept zero between launches) + error word
    int* err_word = nullptr;
    std::unordered_map<const void*, Registered> registered;
    std::string last_error;
    uint64_t launches = 0, h2d_bytes = 0, d2h_bytes = 0;
    int force_generic = 0;
};

extern State g;

void set_error(const std::string& s);
bool is_device_ptr(const void* ptr);
const void* resolve_in(const void* ptr, size_t bytes, DevBuf& stage, bool weights, int* rc);
void* resolve_out(void* ptr, size_t bytes, DevBuf& stage, void** host_dst, int* rc);
// Device -> host copy of a staged result on the main stream (entry points other than the projections).
int copy_back(void* host_dst, const void* dev_src, size_t bytes);
// Static split-K scratch of the allocation-free entry point (no_alloc.cu): made resident at init, forgotten at shutdown.
bool static_scratch_prepare(int device);
void static_scratch_forget();

}  // namespace bridge
