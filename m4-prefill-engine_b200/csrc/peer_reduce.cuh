// Second half of the tensor-parallel all-reduce that the row-split projections start in their epilogue
// (qg::GemmArgs::Scatter): sum the partial rows this rank owns, add the residual, and write the fp16 result into
// every rank's copy of the output.
#pragma once
#include <cuda_runtime.h>
#include <cstdint>

namespace peer {

struct Exchange {
    uint32_t world = 0, rank = 0;
    float* recv[8] = {};          // recv[o]: rank o's receive buffer, fp32 [world][M / world][K]  (peer-mapped)
    void* out[2][8] = {};         // out[b][o]: rank o's copy of result buffer b, fp16 [M][K]      (peer-mapped)
    uint32_t* flags[8] = {};      // flags[o]: rank o's flag words: [0..7] partial sums arrived, [8..15] result rows written
    uint32_t* done_counter = nullptr;   // two device-local words, zero between launches
    uint32_t epoch = 0;           // raised once per reduced projection; flags only ever grow
};

// Rows [rank * rows, (rank + 1) * rows) of  residual + sum over sources  -> fp16, written to out[o] of every rank o;
// waits (bounded) for all sources' arrival flags first and raises this rank's "rows written" flag on every rank last.
cudaError_t reduce_broadcast(const Exchange& x, int which_out, const void* residual, uint32_t M, uint32_t K, int* err,
                             cudaStream_t stream);
// Returns once every rank's rows of the current epoch are in this rank's out buffer (bounded wait).
cudaError_t wait_rows(const Exchange& x, int* err, cudaStream_t stream);

// Bound of the flag waits in milliseconds at about 2 GHz (0 = the default of ten seconds).
void set_wait_limit_ms(unsigned ms);

}  // namespace peer
