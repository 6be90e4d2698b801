// Small per-layer kernels around the GEMMs and the attention kernel (internal interface).
#pragma once
#include <cuda_runtime.h>
#include <cstddef>
#include <cstdint>

namespace lops {
// Y[m][:] = fp16( fp16(x * rsqrt(mean(x^2) + eps)) * w ), sums in fp32.
cudaError_t rmsnorm(const void* X, const void* weight, void* Y, uint32_t M, uint32_t K, float eps, cudaStream_t s);
// S = fp16(A + B), Y = rmsnorm(S) * weight; Y may alias A; 16-byte aligned rows (else cudaErrorInvalidValue)
cudaError_t rmsnorm_add(const void* A, const void* B, const void* weight, void* S, void* Y, uint32_t M, uint32_t K, float eps,
                        cudaStream_t s);
// Rotate-half rotary embedding in place on X [H][M][D]; positions pos0 .. pos0+M-1.
cudaError_t rope(void* X, uint32_t H, uint32_t M, uint32_t D, float theta, uint32_t pos0, cudaStream_t s);
// table[m][j] = (cos, sin) of (pos0 + m) * theta^(-2j/D), float2 [M][D/2]: the rotation operand of the fused projection epilogue.
cudaError_t build_rope_table(void* table, uint32_t M, uint32_t D, float theta, uint32_t pos0, cudaStream_t s);
// One launch for everything between the Q/K/V projections and attention (head size 128): rotary embedding on Q [Hq][M][D] and
// K [Hkv][M][D] in place (rope), K and V compressed to Q8_0 records [Hkv][M][D/32] (q8).  Bit-identical to rope() on Q and K
// followed by attn::launch_quantize on K and V.  With dequant_in_place (and q8) K and V are overwritten by what the records
// give back, fp16(q * d): the operands of attention over this Q8_0 cache, ready for it as fp16 tiles.
// cudaErrorInvalidValue for other head sizes or misaligned buffers.
cudaError_t kv_post(void* Q, void* K, void* V, void* Kq, void* Vq, const void* rope_table, uint32_t Hq, uint32_t Hkv,
                    uint32_t M, uint32_t D, bool rope, bool q8, bool dequant_in_place, cudaStream_t s);
// Y = fp16(float(A) + B) elementwise, A fp16, B fp32 (residual add after an fp32 all-reduce).
cudaError_t add_residual_f32(const void* A_f16, const float* B_f32, void* Y_f16, size_t n, cudaStream_t s);
// Y = fp16(A + B), all fp16; n % 8 == 0 and 16-byte aligned pointers (else cudaErrorInvalidValue)
cudaError_t add_residual_f16(const void* A, const void* B, void* Y, size_t n, cudaStream_t s);
}  // namespace lops

namespace attn {
struct Params;
cudaError_t launch_quantize(const void* src, void* dst, size_t n_elements, cudaStream_t stream);
cudaError_t launch_dequantize(const void* src, void* dst, size_t n_elements, cudaStream_t stream);
// thin wrapper so other translation units need not see attn::Params
int last_attention_launches();     // kernels the last launch_attention_simple call enqueued (2 when a Q8_0 cache was dequantised first)
cudaError_t launch_attention_simple(const void* Q, const void* K, const void* V, void* O, uint32_t Hq, uint32_t Hkv,
                                    uint32_t M, uint32_t Mkv, uint32_t D, float scale, uint32_t pos0, int out_tokens_major,
                                    int kv_fp16, cudaStream_t stream);
}  // namespace attn
