// Second half of the tensor-parallel all-reduce that the row-split projections start in their epilogue
// (qg::GemmArgs::Scatter): sum the partial rows this rank owns, add the residual, and write the fp16 result into
// every rank's copy of the output.
#pragma once
#include <cuda_runtime.h>
#include <cstdint>

namespace peer {

struct Exchange {
    uint32_t world = 0, rank = 0;
    float* recv[8] = {};          // recv[o]: rank o's receive buffer, fp32 (or fp16) [world][M / world][K]  (peer-mapped)
    void* out[2][8] = {};         // out[b][o]: rank o's copy of result buffer b, fp16 [M][K]      (peer-mapped)
    uint32_t* flags[8] = {};      // flags[o]: rank o's flag words: [0..7] partial sums arrived, [8..15] result rows written
    uint32_t* done_counter = nullptr;   // 16 device-local words, zero between launches (1: reduction kernel, 4..11: projection epilogue)
    uint32_t epoch = 0;           // raised once per reduced projection; flags only ever grow
    bool partial_fp16 = false;    // partial sums travel (and sit in recv[]) as fp16 instead of fp32: half the NVLink bytes, one
                                  // extra fp16 rounding per rank and output before the fp32 sum
};

// Rows [rank * rows, (rank + 1) * rows) of  residual + sum over sources  -> fp16, written to out[o] of every rank o;
// waits (bounded) for all sources' arrival flags first and raises this rank's "rows written" flag on every rank last.
// With `norm_w` (fp16 [K]) the rows written to every rank are rmsnorm(residual + sum) * norm_w, and the un-normalised
// fp16 rows stay in the local buffer `keep` ([M][K], only this rank's rows are written): the residual stream is then
// sharded by rows between the two reductions of a layer and the normalisation runs once per row, on its owner.
cudaError_t reduce_broadcast(const Exchange& x, int which_out, const void* residual, uint32_t M, uint32_t K, int* err,
                             cudaStream_t stream, const void* norm_w = nullptr, float eps = 0.0f, void* keep = nullptr);
// Returns once every rank's rows of the current epoch are in this rank's out buffer (bounded wait).
cudaError_t wait_rows(const Exchange& x, int* err, cudaStream_t stream);

// Bound of the flag waits in milliseconds at about 2 GHz (0 = the default of ten seconds).
void set_wait_limit_ms(unsigned ms);
long long wait_limit_cycles();       // the bound of every flag wait, in clock64 ticks

}  // namespace peer
