// Launchers of the quantisation kernels (NVFP4 / FP8 block-scaled quantise, dequantise, GEMM, GEMV).
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace tb {

// x bf16 [M,K] -> q E4M3 [M,K], scales fp32 [M, ceil(K/128)] (x ~= q * scale).
void launch_fp8_quantize_act(const __nv_bfloat16* x, uint8_t* q, float* scales, int M, int K, cudaStream_t s);

// C[M,N] bf16 = (xq * xs) @ (wq * ws)^T with xs per 1x128 segment and ws per 128x128 block. `status` (optional)
// receives a non-zero code if a bounded wait inside the kernel expired.
void launch_fp8_block_gemm(const uint8_t* xq, const float* xs, const uint8_t* wq, const float* ws, __nv_bfloat16* C,
                           int M, int N, int K, int* status, cudaStream_t s);

// NVFP4: two E2M1 codes per byte (low nibble first), one E4M3 scale per 16 elements, one fp32 tensor scale.
void launch_nvfp4_quantize(const void* w, bool w_is_bf16, long long rows, long long K, bool hadamard, uint8_t* packed,
                           uint8_t* scales_e4m3, float* tscale, unsigned int* amax_scratch, cudaStream_t s);
void launch_nvfp4_dequant(const uint8_t* packed, const void* scales, bool scale_bf16, const float* tscale, long long rows,
                          long long K, __nv_bfloat16* out, cudaStream_t s);
void launch_nvfp4_gemv(const __nv_bfloat16* x, const uint8_t* packed, const void* scales, bool scale_bf16,
                       const float* tscale, __nv_bfloat16* y, int M, int N, int K, cudaStream_t s);
void launch_fwht16(const __nv_bfloat16* x, __nv_bfloat16* out, long long n, cudaStream_t s);

// Block-scaled NVFP4 GEMM (nvfp4_gemm.cu). Scales travel in a blocked layout: per 128 rows and 64 elements of K,
// 512 bytes ordered (row % 32) * 16 + (row / 32) * 4 + (k / 16) % 4; blocks stored [row block][nvfp4_sf_kblocks(K)].
int nvfp4_sf_kblocks(int K);
// x bf16 [M, K] (row pitch ld) -> packed E2M1 [M, K / 2] + unsigned E4M3 block scales (blocked layout, buffer pre-zeroed).
void launch_nvfp4_quantize_act(const __nv_bfloat16* x, long long ld, int M, int K, bool hadamard, uint8_t* packed,
                               uint8_t* sf_blocked, cudaStream_t s);
// Row-major E4M3 scales [R, K / 16] -> blocked layout (buffer pre-zeroed).
void launch_nvfp4_block_scales(const uint8_t* scales, int R, int K, uint8_t* out, cudaStream_t s);
// C[M, N] bf16 = alpha * (A .* SFA) (B .* SFB)^T on tcgen05 kind::mxf4nvf4 (K % 32 == 0, N % 8 == 0). tile_n: 0 = choose,
// 128 = double-buffered 128 x 128 tiles, 256 = 128 x 256 tiles with one accumulator.
// bias (bf16 [N], may be null) is added after alpha; gelu applies tanh-GELU after the bias.
void launch_nvfp4_gemm(const uint8_t* a_packed, const uint8_t* sfa, const uint8_t* b_packed, const uint8_t* sfb,
                       __nv_bfloat16* C, int M, int N, int K, float alpha, const __nv_bfloat16* bias, bool gelu, int* status,
                       int tile_n, cudaStream_t s);

// MXFP8: E4M3 values with one power-of-two (UE8M0) scale per 32 elements of K, scales in the blocked layout of the
// block-scaled GEMM (512 bytes per 128 rows x 128 elements of K; buffer pre-zeroed).
int mxfp8_sf_kblocks(int K);
void launch_mxfp8_quantize(const __nv_bfloat16* x, long long ld, int R, int K, uint8_t* q, uint8_t* sf_blocked, cudaStream_t s);
// C[M, N] bf16 = alpha * (A .* SFA) (B .* SFB)^T on tcgen05 kind::mxf8f6f4.block_scale (K % 32 == 0, N % 8 == 0).
void launch_mxfp8_gemm(const uint8_t* a, const uint8_t* sfa, const uint8_t* b, const uint8_t* sfb, __nv_bfloat16* C, int M,
                       int N, int K, float alpha, const __nv_bfloat16* bias, bool gelu, int* status, int tile_n, cudaStream_t s);

// GGML / GGUF block formats (F32, F16, BF16, Q4_0, Q4_1, Q5_0, Q8_0, Q4_K, Q5_K, Q6_K) decoded on the device:
// to bf16, or straight into NVFP4 (optional 16-point Hadamard rotation) without a bf16 copy of the tensor.
void launch_ggml_dequant(const uint8_t* raw, int type, long long n, __nv_bfloat16* out, cudaStream_t s);
void launch_ggml_to_nvfp4(const uint8_t* raw, int type, long long rows, long long K, bool hadamard, uint8_t* packed,
                          uint8_t* scales_e4m3, float* tscale, unsigned int* amax_scratch, cudaStream_t s);

}  // namespace tb
