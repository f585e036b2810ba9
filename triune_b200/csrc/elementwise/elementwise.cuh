// Launchers of the bandwidth-bound kernels (normalisation, feature map, loss, MoE data movement,
// optimizer updates, quantisation helpers). All pointers are device pointers; all launches are
// asynchronous on the given stream.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace tb {

// y = rmsnorm(x [+ res]) * w ; if res != null also writes sum_out = x + res. d % 8 == 0, d <= 2048.
void launch_rmsnorm_fwd(const __nv_bfloat16* x, const __nv_bfloat16* res, const __nv_bfloat16* w, __nv_bfloat16* y,
                        __nv_bfloat16* sum_out, float* rstd, int rows, int d, float eps, cudaStream_t s);
// dx = d(rmsnorm)/dx * dy [+ dres]; dw (fp32, pre-zeroed or accumulating) += sum_rows dy * xhat.
void launch_rmsnorm_bwd(const __nv_bfloat16* x, const __nv_bfloat16* w, const __nv_bfloat16* dy, const float* rstd,
                        const __nv_bfloat16* dres, __nv_bfloat16* dx, float* dw, int rows, int d, cudaStream_t s);

// out[n] (+)= sum over rows of x[m, n] (bf16 in, fp32 out); `partial` holds colsum_parts(M, N) x N floats.
int colsum_parts(int M, int N);
void launch_colsum(const __nv_bfloat16* x, long long ld, int M, int N, float* partial, int parts, float* out,
                   bool accumulate, cudaStream_t s);

void launch_qk_prep_fwd(const __nv_bfloat16* in, long long in_ld, int k_col_offset, __nv_bfloat16* out, const float* cs,
                        const float* sn, long long tokens, int T, int H, int D, cudaStream_t s);
void launch_qk_prep_bwd(const __nv_bfloat16* in, long long in_ld, int k_col_offset, const __nv_bfloat16* dout,
                        __nv_bfloat16* d_in, long long d_in_ld, const float* cs, const float* sn, long long tokens,
                        int T, int H, int D, cudaStream_t s);

// Row-wise cross entropy over bf16 logits [rows, V] (row stride ld). Writes per-row loss (0 for ignored
// rows) and, when grad_scale != 0, overwrites the logits with grad_scale * (softmax - onehot).
// With grad_dst (a [rows, V] bf16 buffer of the same row stride) the gradient goes there and the logits stay intact.
void launch_ce_fwd_bwd(__nv_bfloat16* logits, long long ld, const long long* targets, float* row_loss, int rows, int V,
                       long long ignore_index, float grad_scale, cudaStream_t s, __nv_bfloat16* grad_dst = nullptr);

// out = silu(gate) * up over rows of `width` bf16 (width % 8 == 0); every operand has its own row pitch.
void launch_swiglu_fwd(const __nv_bfloat16* gate, long long ld_g, const __nv_bfloat16* up, long long ld_u,
                       __nv_bfloat16* out, long long ld_o, long long rows, int width, cudaStream_t s);
// d(gate) = dh * up * silu'(gate), d(up) = dh * silu(gate).
void launch_swiglu_bwd(const __nv_bfloat16* gate, long long ld_g, const __nv_bfloat16* up, long long ld_u,
                       const __nv_bfloat16* dh, long long ld_d, __nv_bfloat16* dgate, long long ld_dg,
                       __nv_bfloat16* dup, long long ld_du, long long rows, int width, cudaStream_t s);
// Half-split rotary embedding of x [rows = B*T, H, D] with cos/sin [T, D/2] fp32; `transpose` applies the inverse
// rotation (the gradient). D % 16 == 0.
void launch_rope(const __nv_bfloat16* x, long long ld_x, __nv_bfloat16* y, long long ld_y, const float* cs,
                 const float* sn, long long rows, int T, int H, int D, bool transpose, cudaStream_t s);
// Embedding gradient: grad[ids[n], :] += dy[n, :] (fp32 [V, width], 16-byte aligned rows; width % 4 == 0).
void launch_embedding_bwd(const __nv_bfloat16* dy, long long ld, const long long* ids, float* grad, long long tokens,
                          int width, long long V, cudaStream_t s);

// dst[r] = scale[r] * src[row_src[r]] (zero row when row_src[r] < 0). Rows of `width` bf16 (width % 8 == 0).
void launch_gather_rows(__nv_bfloat16* dst, const __nv_bfloat16* src, const int* row_src, const float* row_scale,
                        int dst_rows, int width, int src_rows, cudaStream_t s);
// out[t] = sum_j w[t,j] * src[pos[t,j]] (+ add_scale * add[t]); pos < 0 skips the term. w may be null (=1).
// An index >= src_rows is skipped and recorded (see index_error_word), never followed.
void launch_combine_rows(__nv_bfloat16* out, const __nv_bfloat16* src, const int* pos, const float* w,
                         const __nv_bfloat16* add, float add_scale, int tokens, int k, int width, int src_rows,
                         cudaStream_t s);
// {kernel id (1 gather_rows, 2 combine_rows; 0 = none), row, offending index, limit} of the first out-of-table index
// seen since the last clear. Synchronises.
void index_error_word(int out[4], bool clear);
// dots[t,j] = <a[t], b[pos[t,j]]> (0 when pos < 0).
void launch_row_dots(float* dots, const __nv_bfloat16* a, const __nv_bfloat16* b, const int* pos, int tokens, int k,
                     int width, cudaStream_t s);

// Fused AdamW over a flat shard: fp32 master p, moments m, v; grads bf16 or fp32; writes bf16 copy.
// grad_scale is read from device memory (clip coefficient) when grad_scale_ptr != null.
void launch_adamw_flat(float* master, float* m, float* v, const void* grad, bool grad_is_f32, __nv_bfloat16* param_bf16,
                       long long n, float lr, float beta1, float beta2, float eps, float weight_decay,
                       float bias_corr1, float bias_corr2, const float* grad_scale_ptr, float grad_scale,
                       const float* hyper, cudaStream_t s);
// `hyper` (optional, device fp32[8]) overrides host scalars so a captured CUDA graph follows the schedule:
//   [0] lr  [1] adam 1-beta1^t  [2] adam 1-beta2^t  [3] muon lr  [4] expert lr  [5] core 1-beta1^t  [6] core 1-beta2^t
//   [7] 1 - expert_lr * expert_wd
// sum of squares of a flat buffer accumulated into out[0] (fp32 atomic per block).
void launch_sumsq(const void* x, bool is_f32, long long n, float* out, cudaStream_t s);

// Muon momentum: M = beta*M + G; U = nesterov ? G + beta*M : M (bf16 out for the polar iteration).
void launch_muon_momentum(float* mom, const void* grad, bool grad_is_f32, __nv_bfloat16* u_out, long long n, float beta,
                          bool nesterov, const float* grad_scale_ptr, cudaStream_t s);
// W_master = W_master * (1 - lr*wd) - lr*scale*O ; also refresh bf16 copy.
void launch_muon_apply(float* master, const __nv_bfloat16* o, __nv_bfloat16* param_bf16, long long n, float lr,
                       float wd, float scale, const float* hyper, cudaStream_t s);
// Newton-Schulz set-up for `batch` matrices X [m, n] (m <= n, n % 8 == 0, contiguous): Y = X / safe with
// safe = max(1.15 sigma_max estimate, ||X||_F / sqrt(m), 0.7 ||X||_F); sigma from a four-step power iteration.
// `scratch`: fp32 [2 * batch * n + 2 * batch] (two iterate buffers, ||X||_F^2 and sigma^2 per matrix). n <= 12288.
void launch_ns_prepare(const __nv_bfloat16* X, __nv_bfloat16* Y, int batch, int m, int n, float eps, float* scratch,
                       cudaStream_t s);
// X = a*X + Y (bf16, elementwise) used by the Newton-Schulz blend when not fused in a GEMM epilogue.
void launch_axpby_bf16(__nv_bfloat16* x, const __nv_bfloat16* y, float a, float b, long long n, cudaStream_t s);

// Batched triangular AdamW on [nmat, r1, r1] cores (fp32 state), optional upper-triangular mask.
void launch_triangular_adamw(const float* S, float* m, float* v, float* delta, int nmat, int r1, float beta1,
                             float beta2, float eps, float bias_corr1, float bias_corr2, bool triu, const float* hyper,
                             cudaStream_t s);
// P = momentum*P + steer*(G-P)
void launch_steer_update(float* P, const float* G, long long n, float momentum, float steer, cudaStream_t s);

// 3-way tier router: tiers[r] from logits[r,3]; all_reflex flag (int) set to 0 if any row is not tier 0.
void launch_route_tiers(const float* logits, int* tiers, int* all_reflex, int rows, float threshold, cudaStream_t s);
// |act| binned into num_bins, max-normalised, ABGR-packed colours.
void launch_neuron_heatmap(const float* act, long long n, int num_bins, float* bin_scratch, uint32_t* rgba,
                           cudaStream_t s);
// act [rows,width] fp32 + tiers -> RGBA8 [rows,width].
void launch_tier_render(const float* act, const int* tiers, uint32_t* rgba, int rows, int width, cudaStream_t s);

// MoE routing: top-k + mixing weights + sort keys + per-(expert, slot) counts; gradient of the weights; and the
// dispatch plan from the sorted keys (see moe_route.cu).
void launch_moe_route_topk(const float* logits, const float* bias, const float* temperature, float temp_value, int N, int E, int K,
                           long long* idx, float* w, void* keys, bool keys32, int* counts, cudaStream_t s);
void launch_moe_route_bwd(const float* logits, const float* temperature, float temp_value, const long long* idx, const float* w,
                          const float* dw, int N, int E, int K, float* dlogits, cudaStream_t s);
void launch_moe_plan_sorted(const void* sorted_keys, bool keys32, const long long* order, const int* counts, int A, int E, int K, int cap,
                            int R, int* pos, unsigned char* keep, int* row_src, int* tile_group, int* group_offsets,
                            long long* accepted, cudaStream_t s);

}  // namespace tb
