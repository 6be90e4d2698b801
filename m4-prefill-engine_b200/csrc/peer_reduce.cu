// Reduce + residual + broadcast over peer memory (NVLink), the consumer side of the fused reduce-scatter in the
// projection epilogue.  Data moves with plain peer stores; ranks signal each other with release stores to flag
// words and wait with acquire loads, every wait bounded (about ten seconds) and reported through the error word.
#include "peer_reduce.cuh"

#include <cuda_fp16.h>

namespace peer {

namespace {

// About ten seconds: ranks reach their first exchange with the skew of their first kernel loads, which can be a
// large fraction of a second; a rank that never arrives still ends the wait.
constexpr long long DEFAULT_WAIT_LIMIT_CYCLES = 20000000000LL;
long long g_wait_limit_cycles = DEFAULT_WAIT_LIMIT_CYCLES;      // host copy, passed to every launch

__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// true when flags[0 .. world) have all reached epoch; gives up after WAIT_LIMIT_CYCLES
__device__ bool wait_flags(const uint32_t* flags, uint32_t world, uint32_t epoch, int* err, int code, long long limit) {
    // once any wait of this process has given up, later ones do not wait again (the host reads the error word and
    // stops using the exchange; without this a broken group would cost ten seconds per kernel)
    if (err && *reinterpret_cast<volatile int*>(err) != 0) return false;
    const long long t0 = clock64();
    for (uint32_t s = 0; s < world; s++) {
        while ((int32_t)(ld_acquire_sys(flags + s) - epoch) < 0) {
            if (clock64() - t0 > limit) {
                if (err) atomicCAS(err, 0, code);
                return false;
            }
            __nanosleep(200);
        }
    }
    return true;
}

struct ReduceParams {
    uint32_t world, rank, rows, K, epoch;
    const float* recv;            // this rank's receive buffer [world][rows][K]
    const __half* residual;       // [M][K], this rank's rows are read
    __half* out[8];
    uint32_t* flags[8];
    const uint32_t* my_flags;
    uint32_t* done_counter;
    int* err;
    long long wait_limit;
};

__global__ void __launch_bounds__(256) reduce_broadcast_kernel(const ReduceParams p) {
    __shared__ uint32_t ok_s;
    if (threadIdx.x == 0) ok_s = wait_flags(p.my_flags, p.world, p.epoch, p.err, 301, p.wait_limit) ? 1u : 0u;
    __syncthreads();
    if (ok_s) {
        const size_t n4 = (size_t)p.rows * p.K / 4;               // K % 4 == 0 (K is a multiple of 32)
        const size_t src_stride4 = n4;
        const float4* recv4 = reinterpret_cast<const float4*>(p.recv);
        const size_t row0 = (size_t)p.rank * p.rows * p.K;          // first element of this rank's rows in [M][K]
        for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (size_t)gridDim.x * blockDim.x) {
            float4 acc = __ldcg(recv4 + i);
            for (uint32_t s = 1; s < p.world; s++) {
                const float4 v = __ldcg(recv4 + s * src_stride4 + i);
                acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
            }
            const uint2 r = *reinterpret_cast<const uint2*>(p.residual + row0 + i * 4);
            const __half2 r01 = *reinterpret_cast<const __half2*>(&r.x), r23 = *reinterpret_cast<const __half2*>(&r.y);
            const __half2 h01 = __floats2half2_rn(acc.x + __low2float(r01), acc.y + __high2float(r01));
            const __half2 h23 = __floats2half2_rn(acc.z + __low2float(r23), acc.w + __high2float(r23));
            uint2 w;
            w.x = *reinterpret_cast<const uint32_t*>(&h01); w.y = *reinterpret_cast<const uint32_t*>(&h23);
            for (uint32_t o = 0; o < p.world; o++) *reinterpret_cast<uint2*>(p.out[o] + row0 + i * 4) = w;
        }
    }
    // the CTA that completes the count tells every rank that this rank's rows are written (peer stores fenced first)
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {
        const uint32_t old = atomicAdd(p.done_counter, 1u);
        if (old == gridDim.x - 1u) {
            *p.done_counter = 0u;
            __threadfence_system();
            for (uint32_t o = 0; o < p.world; o++) st_release_sys(p.flags[o] + 8 + p.rank, p.epoch);
        }
    }
}

__global__ void wait_rows_kernel(const uint32_t* my_flags, uint32_t world, uint32_t epoch, int* err, long long limit) {
    if (threadIdx.x == 0) wait_flags(my_flags + 8, world, epoch, err, 302, limit);
}

}  // namespace

cudaError_t reduce_broadcast(const Exchange& x, int which_out, const void* residual, uint32_t M, uint32_t K, int* err,
                             cudaStream_t stream) {
    if (x.world == 0 || x.world > 8 || M % x.world != 0 || K % 4 != 0) return cudaErrorInvalidValue;
    ReduceParams p;
    p.world = x.world; p.rank = x.rank; p.rows = M / x.world; p.K = K; p.epoch = x.epoch;
    p.recv = x.recv[x.rank];
    p.residual = (const __half*)residual;
    for (uint32_t o = 0; o < 8; o++) { p.out[o] = (__half*)x.out[which_out][o]; p.flags[o] = x.flags[o]; }
    p.my_flags = x.flags[x.rank];
    p.done_counter = x.done_counter + 1;
    p.err = err;
    p.wait_limit = g_wait_limit_cycles;
    int dev = 0, sms = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    reduce_broadcast_kernel<<<sms * 4, 256, 0, stream>>>(p);
    return cudaGetLastError();
}

cudaError_t wait_rows(const Exchange& x, int* err, cudaStream_t stream) {
    wait_rows_kernel<<<1, 32, 0, stream>>>(x.flags[x.rank], x.world, x.epoch, err, g_wait_limit_cycles);
    return cudaGetLastError();
}

void set_wait_limit_ms(unsigned ms) { g_wait_limit_cycles = ms ? (long long)ms * 2000000LL : DEFAULT_WAIT_LIMIT_CYCLES; }

}  // namespace peer
