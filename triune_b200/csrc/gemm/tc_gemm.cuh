// Interface of the bf16 tcgen05 GEMM family (dense / batched / grouped-by-rows / grouped-by-reduction).
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace tb {

enum GemmMode : int {
  GEMM_DENSE = 0,      // C[b] = A[b] * B[b]^T, b in [0, batch)
  GEMM_GROUPED_M = 1,  // rows of A are grouped (padded to 128); tile_group[m_tile] selects B[g] and bias[g]
  GEMM_GROUPED_K = 2,  // C[g] = sum over rows in [group_offsets[g], group_offsets[g+1]) (weight gradients)
};

enum GemmFlags : int {
  GF_OUT_F32 = 1,     // C is fp32 (default bf16)
  GF_ACCUMULATE = 2,  // C += result
  GF_GELU = 4,        // C = gelu_tanh(result + bias); gelu_tanh'(result + bias) optionally saved to aux_out
  GF_DGELU = 8,       // C = result * aux_in (aux_in = the derivative rows saved by GF_GELU)
  GF_PAIRED_GROUPS = 16,  // GEMM_GROUPED_M: every group's rows are padded to 256, so tile_group[2i] == tile_group[2i+1]
  // SwiGLU over a fused gate/up weight B = [gate rows (n_split) ; up rows (n_split)], dense mode, K-major operands:
  GF_SWIGLU = 32,   // C [M, N = n_split] = silu(A gate^T) * (A up^T); aux_out [M, 2 N] optionally receives both pre-activations
  GF_ADDAUX = 128,  // C = alpha * A B^T + beta * aux_in (aux_in: bf16, C's layout; bf16 output, no bias)
  GF_DSWIGLU = 64,  // acc = A B^T [M, N = n_split] is d(hidden); aux_in [M, 2 N] holds gate | up; C [M, 2 N] = d(gate) | d(up)
};

// Operand layouts. "K-major": the reduction index is contiguous (x[M,K] row-major, w[N,K] row-major).
// "MN-major": the non-reduction index is contiguous (x stored [K,M] row-major). Both feed the tensor
// core directly from 128B-swizzled shared memory; no transposes are materialised.
struct GemmArgs {
  const __nv_bfloat16* A;
  const __nv_bfloat16* B;
  void* C;
  int M, N, K;
  long long lda, ldb, ldc;             // leading dimensions in elements
  long long strideA, strideB, strideC; // batch strides in elements (0 = shared)
  int batch;
  bool a_mn_major, b_mn_major;
  int mode;
  int flags;
  float alpha;
  const __nv_bfloat16* bias;  // [batch or groups][N] or null
  long long bias_stride;
  const __nv_bfloat16* aux_in;  // same layout as C (bf16), for GF_DGELU
  __nv_bfloat16* aux_out;       // same layout as C (bf16), activation derivative from GF_GELU
  const float* row_scale;       // [M] or null
  const int* tile_group;        // GEMM_GROUPED_M: [ceil(M/128)], -1 marks an unused tile
  const int* group_offsets;     // GEMM_GROUPED_K: [batch+1], multiples of 64
  // GEMM_GROUPED_K, optional: [runs][2] = (first row, number of 64-row blocks) of the row runs to reduce over. With it
  // group_offsets[g] .. group_offsets[g+1] index RUNS instead of rows, so a group may skip rows that hold nothing
  // (segments of a fixed-capacity buffer that are only partly filled). First rows must be multiples of 64.
  const int* k_runs;
  int* status;                  // optional device status word (see KernelStatus)
  int n_split;                  // GF_SWIGLU / GF_DSWIGLU: FFN hidden width (N); 0 otherwise
  float beta;                   // GF_ADDAUX: weight of aux_in
};

// Launches on `stream`. Throws std::runtime_error on invalid arguments.
void launch_tc_gemm(const GemmArgs& args, cudaStream_t stream);

// CTA-pair (tcgen05 cta_group::2) variant for dense products with long reductions; returns false, launching
// nothing, when the shape does not suit it. launch_tc_gemm tries it first.
bool launch_tc_gemm_pair(const GemmArgs& args, cudaStream_t stream);
long long tc_gemm_pair_launch_count();
// Developer aid: sixteen int64 counters (device memory) that one epilogue warp per CTA adds its phase times to; null disables.
void tc_gemm_set_debug_buffer(long long* counters);  // launches taken by the CTA-pair kernel so far in this process

}  // namespace tb
