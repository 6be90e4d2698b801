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

// True when flags[0 .. world) have all reached epoch; gives up after `limit` cycles.  Called by every lane of one warp:
// lane s polls flag s, so the `world` round trips to the flag words overlap instead of following one another, and one
// acquire fence at system scope after the last poll orders the data reads behind all of them.
__device__ bool wait_flags(const uint32_t* flags, uint32_t world, uint32_t epoch, int* err, int code, long long limit) {
    // once any wait of this process has given up, later ones do not wait again (the host reads the error word and
    // stops using the exchange; without this a broken group would cost ten seconds per kernel)
    if (err && *reinterpret_cast<volatile int*>(err) != 0) return false;
    const uint32_t lane = threadIdx.x & 31u;
    const long long t0 = clock64();
    bool mine = lane >= world;
    for (;;) {
        if (!mine) {
            uint32_t v;
            asm volatile("ld.relaxed.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(flags + lane) : "memory");
            mine = (int32_t)(v - epoch) >= 0;
        }
        if (__all_sync(0xffffffffu, mine)) break;
        if (__any_sync(0xffffffffu, clock64() - t0 > limit)) {
            if (lane == 0 && err) atomicCAS(err, 0, code);
            return false;
        }
        __nanosleep(100);
    }
    asm volatile("fence.acq_rel.sys;" ::: "memory");
    return true;
}

// four consecutive partial sums (group index i4) of a receive buffer that holds fp32 or fp16 values
template <bool H>
__device__ __forceinline__ float4 ld_partial4(const void* base, size_t i4) {
    if (H) {
        const uint2 u = __ldcg(reinterpret_cast<const uint2*>(base) + i4);
        const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&u.x)), b = __half22float2(*reinterpret_cast<const __half2*>(&u.y));
        return make_float4(a.x, a.y, b.x, b.y);
    }
    return __ldcg(reinterpret_cast<const float4*>(base) + i4);
}

struct ReduceParams {
    uint32_t world, rank, rows, K, epoch;
    const void* recv;             // this rank's receive buffer [world][rows][K], fp32 or fp16
    const __half* residual;       // [M][K], this rank's rows are read
    const __half* norm_w;         // [K] RMSNorm weights: the rows written to every rank are normalised (nullptr: plain sum)
    __half* keep;                 // [M][K] local buffer that receives this rank's un-normalised rows (required with norm_w)
    float eps;
    __half* out[8];
    uint32_t* flags[8];
    const uint32_t* my_flags;
    uint32_t* done_counter;
    int* err;
    long long wait_limit;
};

template <bool H>
__global__ void __launch_bounds__(256) reduce_broadcast_kernel(const ReduceParams p) {
    __shared__ uint32_t ok_s;
    if (threadIdx.x < 32) {
        const bool ok = wait_flags(p.my_flags, p.world, p.epoch, p.err, 301, p.wait_limit);
        if (threadIdx.x == 0) ok_s = ok ? 1u : 0u;
    }
    __syncthreads();
    if (ok_s) {
        constexpr int U = 4;                                       // float4 groups in flight per thread and source
        const size_t n4 = (size_t)p.rows * p.K / 4;               // K % 4 == 0 (K is a multiple of 32)
        const size_t src_stride4 = n4;
        const size_t row0 = (size_t)p.rank * p.rows * p.K;          // first element of this rank's rows in [M][K]
        const size_t step = (size_t)gridDim.x * blockDim.x;
        for (size_t i0 = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i0 < n4; i0 += step * U) {
            float4 acc[U];
            uint2 rs[U];
#pragma unroll
            for (int u = 0; u < U; u++) {
                const size_t i = i0 + u * step;
                if (i < n4) { acc[u] = ld_partial4<H>(p.recv, i); rs[u] = *reinterpret_cast<const uint2*>(p.residual + row0 + i * 4); }
            }
            for (uint32_t s = 1; s < p.world; s++) {
                float4 t[U];
#pragma unroll
                for (int u = 0; u < U; u++) { const size_t i = i0 + u * step; if (i < n4) t[u] = ld_partial4<H>(p.recv, s * src_stride4 + i); }
#pragma unroll
                for (int u = 0; u < U; u++) { acc[u].x += t[u].x; acc[u].y += t[u].y; acc[u].z += t[u].z; acc[u].w += t[u].w; }
            }
#pragma unroll
            for (int u = 0; u < U; u++) {
                const size_t i = i0 + u * step;
                if (i >= n4) continue;
                const __half2 r01 = *reinterpret_cast<const __half2*>(&rs[u].x), r23 = *reinterpret_cast<const __half2*>(&rs[u].y);
                const __half2 h01 = __floats2half2_rn(acc[u].x + __low2float(r01), acc[u].y + __high2float(r01));
                const __half2 h23 = __floats2half2_rn(acc[u].z + __low2float(r23), acc[u].w + __high2float(r23));
                uint2 w;
                w.x = *reinterpret_cast<const uint32_t*>(&h01); w.y = *reinterpret_cast<const uint32_t*>(&h23);
                for (uint32_t o = 0; o < p.world; o++) *reinterpret_cast<uint2*>(p.out[o] + row0 + i * 4) = w;
            }
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

// The same reduction for a row-sharded residual stream: one CTA per owned row computes s = fp16(residual + sum of the
// partial rows), keeps it in the local `keep` buffer (the residual of the block after this one), and writes
// rmsnorm(s) * w into every rank's copy of the output, so the normalisation runs once per row on its owner instead of
// on every rank for all rows.  Arithmetic of the normalisation as in lops::rmsnorm_add_kernel.
// V = float4 groups per thread (K = 1024 * V): a thread issues all of its loads (V per source rank, the residual and
// the norm weights) before the first use, and the row's sums stay in registers between the two passes.
template <int V, bool H>
__global__ void __launch_bounds__(256) reduce_norm_broadcast_kernel(const ReduceParams p) {
    __shared__ uint32_t ok_s;
    __shared__ float red[8];
    if (threadIdx.x < 32) {
        const bool ok = wait_flags(p.my_flags, p.world, p.epoch, p.err, 301, p.wait_limit);
        if (threadIdx.x == 0) ok_s = ok ? 1u : 0u;
    }
    __syncthreads();
    if (ok_s) {
        const uint32_t K4 = p.K / 4;
        const size_t src_stride4 = (size_t)p.rows * K4;
        for (uint32_t r = blockIdx.x; r < p.rows; r += gridDim.x) {
            const size_t row_el = ((size_t)p.rank * p.rows + r) * p.K;      // first element of the row in [M][K]
            float4 acc[V];
            uint2 rs[V], wv[V];
#pragma unroll
            for (int v = 0; v < V; v++) {
                const uint32_t i = threadIdx.x + v * 256;
                acc[v] = ld_partial4<H>(p.recv, (size_t)r * K4 + i);
                rs[v] = *reinterpret_cast<const uint2*>(p.residual + row_el + i * 4);
                wv[v] = __ldg(reinterpret_cast<const uint2*>(p.norm_w + i * 4));
            }
            for (uint32_t s = 1; s < p.world; s++) {
                float4 t[V];
#pragma unroll
                for (int v = 0; v < V; v++) t[v] = ld_partial4<H>(p.recv, s * src_stride4 + (size_t)r * K4 + threadIdx.x + v * 256);
#pragma unroll
                for (int v = 0; v < V; v++) { acc[v].x += t[v].x; acc[v].y += t[v].y; acc[v].z += t[v].z; acc[v].w += t[v].w; }
            }
            float ss = 0.0f;
            __half2 h[V][2];
#pragma unroll
            for (int v = 0; v < V; v++) {
                const __half2 r01 = *reinterpret_cast<const __half2*>(&rs[v].x), r23 = *reinterpret_cast<const __half2*>(&rs[v].y);
                h[v][0] = __floats2half2_rn(acc[v].x + __low2float(r01), acc[v].y + __high2float(r01));
                h[v][1] = __floats2half2_rn(acc[v].z + __low2float(r23), acc[v].w + __high2float(r23));
                const float2 f01 = __half22float2(h[v][0]), f23 = __half22float2(h[v][1]);
                ss += f01.x * f01.x + f01.y * f01.y + f23.x * f23.x + f23.y * f23.y;
                uint2 w;
                w.x = *reinterpret_cast<const uint32_t*>(&h[v][0]); w.y = *reinterpret_cast<const uint32_t*>(&h[v][1]);
                *reinterpret_cast<uint2*>(p.keep + row_el + (threadIdx.x + v * 256) * 4) = w;
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
            __syncthreads();                      // the previous row's readers of red[] are done
            if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
            __syncthreads();
            float tot = 0.0f;
#pragma unroll
            for (int i = 0; i < 8; i++) tot += red[i];
            const float rn = 1.0f / sqrtf(tot / (float)p.K + p.eps);
#pragma unroll
            for (int v = 0; v < V; v++) {
                const __half2* wh = reinterpret_cast<const __half2*>(&wv[v]);
                uint2 o;
                __half2* oh = reinterpret_cast<__half2*>(&o);
#pragma unroll
                for (int j = 0; j < 2; j++) {
                    const float2 f = __half22float2(h[v][j]), g = __half22float2(wh[j]);
                    const __half2 n = __floats2half2_rn(f.x * rn, f.y * rn);          // rounded to fp16 first, as the reference does
                    const float2 nf = __half22float2(n);
                    oh[j] = __floats2half2_rn(nf.x * g.x, nf.y * g.y);
                }
                for (uint32_t d = 0; d < p.world; d++) *reinterpret_cast<uint2*>(p.out[d] + row_el + (threadIdx.x + v * 256) * 4) = o;
            }
        }
    }
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
    wait_flags(my_flags + 8, world, epoch, err, 302, limit);      // one warp
}

}  // namespace

cudaError_t reduce_broadcast(const Exchange& x, int which_out, const void* residual, uint32_t M, uint32_t K, int* err,
                             cudaStream_t stream, const void* norm_w, float eps, void* keep) {
    if (x.world == 0 || x.world > 8 || M % x.world != 0 || K % 4 != 0) return cudaErrorInvalidValue;
    if (norm_w && (!keep || eps <= 0.0f || K % 1024 != 0 || K > 8192)) return cudaErrorInvalidValue;
    ReduceParams p;
    p.norm_w = (const __half*)norm_w; p.keep = (__half*)keep; p.eps = eps;
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
    if (norm_w) {
        const uint32_t rows = M / x.world;
        const uint32_t grid = rows < (uint32_t)sms * 8u ? rows : (uint32_t)sms * 8u;
#define LAUNCH_NORM(V) do { if (x.partial_fp16) reduce_norm_broadcast_kernel<V, true><<<grid, 256, 0, stream>>>(p); \
                            else reduce_norm_broadcast_kernel<V, false><<<grid, 256, 0, stream>>>(p); } while (0)
        switch (K / 1024) {
            case 1: LAUNCH_NORM(1); break;
            case 2: LAUNCH_NORM(2); break;
            case 3: LAUNCH_NORM(3); break;
            case 4: LAUNCH_NORM(4); break;
            case 5: LAUNCH_NORM(5); break;
            case 6: LAUNCH_NORM(6); break;
            case 7: LAUNCH_NORM(7); break;
            default: LAUNCH_NORM(8); break;
        }
#undef LAUNCH_NORM
    } else if (x.partial_fp16) {
        reduce_broadcast_kernel<true><<<sms * 4, 256, 0, stream>>>(p);
    } else {
        reduce_broadcast_kernel<false><<<sms * 4, 256, 0, stream>>>(p);
    }
    return cudaGetLastError();
}

cudaError_t wait_rows(const Exchange& x, int* err, cudaStream_t stream) {
    wait_rows_kernel<<<1, 32, 0, stream>>>(x.flags[x.rank], x.world, x.epoch, err, g_wait_limit_cycles);
    return cudaGetLastError();
}

long long wait_limit_cycles() { return g_wait_limit_cycles; }
void set_wait_limit_ms(unsigned ms) { g_wait_limit_cycles = ms ? (long long)ms * 2000000LL : DEFAULT_WAIT_LIMIT_CYCLES; }

}  // namespace peer
