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

struct State {
    std::mutex mu;
    bool initialized = false;
    int device = 0;
    cudaStream_t stream = nullptr;
    DevBuf stage_x, stage_w0, stage_w1, stage_y, stage_res, stage_aux0, stage_aux1, stage_aux2;
    DevBuf ws_partial;          // split-K partial tiles
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

}  // namespace bridge
