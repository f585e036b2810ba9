// Launchers of the gated-linear-attention kernels (head_dim 64, chunk 64, bf16 in, fp32 state).
//
// The sequence is processed in three phases, forward and backward alike:
//   1. per chunk, in parallel:   local state contribution (K~^T V, or Q~^T dO going backward)
//   2. per (batch, head):        inter-chunk recurrence over the chunk states (elementwise scan)
//   3. per chunk, in parallel:   outputs (or input gradients) from the chunk-start state + intra-chunk scores
// Every matrix product runs as tcgen05.mma (M=64) on TMA-fed, 128B-swizzled shared-memory tiles with the
// accumulators in TMEM. Per-dimension decays are kept exact by referencing each 16-token sub-chunk of keys
// to its own first row, so every exponent stays within [-80, 80] given the per-token clamp g >= -5.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace tb {

constexpr float GLA_MIN_LOG_DECAY = -5.0f;

// A [B*T rows] x [64 cols] bf16 slice of a wider row-major matrix: element (row, c) = ptr[row*ld + col0 + h*64 + c].
struct GlaMat {
  const void* ptr;
  long long ld;
  int col0;
};

struct GlaDims {
  int B, T, H;
  bool gate_logits;  // g holds raw logits (log-sigmoid applied in-kernel) instead of log decays
};

// mode 0: kv[bh,c] = (k * exp(b_last - b))^T v and decay[bh,c] = exp(b_last);  mode 1: kv = (q * exp(b))^T dO.
void launch_gla_chunk_outer(int mode, GlaMat X, GlaMat Y, GlaMat G, float* out_kv, float* out_decay, GlaDims d,
                            int* status, cudaStream_t s);
// forward: states[c] = S before chunk c, S <- decay[c] * S + kv[c];  reverse: states[c] = dS after chunk c.
void launch_gla_scan(const float* kv, const float* decay, const float* init, __nv_bfloat16* states, float* final_state,
                     int BH, int NT, bool reverse, cudaStream_t s);
void launch_gla_fwd_out(GlaMat Q, GlaMat K, GlaMat V, GlaMat G, const __nv_bfloat16* states, GlaMat O, GlaDims d,
                        int* status, cudaStream_t s);
void launch_gla_bwd_main(GlaMat Q, GlaMat K, GlaMat V, GlaMat G, GlaMat dO, const __nv_bfloat16* states,
                         const __nv_bfloat16* dstates, GlaMat dQ, GlaMat dK, GlaMat dV, float* dgl_local,
                         float* chunk_tot, GlaDims d, int* status, cudaStream_t s);
// end_term (optional, fp32 [B*H, 64]): rowsum(dS_T * S_T), the gate gradient that reaches every token through a
// differentiated final state.
void launch_gla_dg_finalize(const float* dgl_local, const float* chunk_tot, GlaMat G, GlaMat dG, GlaDims d,
                            cudaStream_t s, const float* end_term = nullptr);
// Developer aid: eight int64 counters (device memory) receiving the backward kernel's phase clocks; null disables.
void gla_set_debug_buffer(long long* counters);
// One decode step for B*H heads: state [BH,64,64] fp32 in place; q,k,v,g rows of 64 bf16; out bf16.
void launch_gla_decode_step(GlaMat Q, GlaMat K, GlaMat V, GlaMat G, float* state, GlaMat O, int B, int H,
                            bool gate_logits, cudaStream_t s);
// Gated DeltaNet token recurrence over T tokens (T = 1: one decode step) for B*H heads of dimension D (64 or 128):
// state [BH,D,D] fp32 in place; beta: null (1), fp32 [B*T,H] (beta_mode 1) or fp32 [B*T,H*D] (beta_mode 2).
void launch_gdn_recurrent(const GlaMat& Q, const GlaMat& K, const GlaMat& V, const GlaMat& G, const float* beta,
                          int beta_mode, float* state, const GlaMat& O, int B, int T, int H, int D, bool gate_logits,
                          float scale, cudaStream_t s);

// ---- Gated DeltaNet, chunk-parallel training path (gdn_chunk_kernels.cu) ----
struct GdnDims {
  int B, T, H, D;    // T a multiple of 64, D = 64 or 128 (keys and values)
  bool gate_logits;
};
// Per-chunk tensors produced by the forward pass and kept for the backward pass. nchunks = B * H * T / 64.
struct GdnScratch {
  __nv_bfloat16* U0;      // [nchunks, 64, D]   T (beta V)
  __nv_bfloat16* W;       // [nchunks, 64, D]   T (beta Kbar)
  __nv_bfloat16* Tm;      // [nchunks, 64, 64]  (I + L)^-1
  __nv_bfloat16* Kend;    // [nchunks, 64, D]   k e^{b_C - b}
  float* decay;           // [nchunks, D]       e^{b_C}
  float* Lraw;            // [nchunks, 64, 64]  strict decayed key-key scores (null: not kept)
  __nv_bfloat16* U;       // [nchunks, 64, D]   effective values
  __nv_bfloat16* states;  // [nchunks, D, D]    state before each chunk
  float* fin;             // [B * H, D, D]      state after the last token
};
struct GdnBwdScratch {
  float* G1;              // [nchunks, 64, D]
  float* H1;              // [nchunks, D, D]
  __nv_bfloat16* dU;      // [nchunks, 64, D]
  __nv_bfloat16* dSend;   // [nchunks, D, D]    gradient of the state after each chunk
  float* dS0;             // [B * H, D, D]      gradient of the initial state
  float* dq1;             // [nchunks, 64, D]
  float* dkw1;            // [nchunks, 64, D]
  float* dkr1;            // [nchunks, 64, D]
  __nv_bfloat16* dW;      // [nchunks, 64, D]
  __nv_bfloat16* dLraw;   // [nchunks, 64, 64]
  float* dbeta;           // [B * T, H] (null without beta)
  float* dgl_local;       // [B * T, H * D]     in-chunk part of the gate gradient
  float* chunk_tot;       // [B * H * D / 64, T / 64, 64] chunk totals (the layout gla_dg_finalize reads with H * D / 64 heads)
};
// out = scale * GatedDeltaNet(q, k, v, g, beta); beta fp32 [B*T, H] or null; init fp32 [B*H, D, D] or null.
void launch_gdn_chunk_fwd(const GlaMat& Q, const GlaMat& K, const GlaMat& V, const GlaMat& G, const float* beta,
                          const float* init, const GlaMat& O, const GdnScratch& w, const GdnDims& d, float scale,
                          int* status, cudaStream_t s);
// Writes dq, dk, dv and fills dbeta, dS0, dgl_local, chunk_tot; the gate gradient is completed by
// launch_gla_dg_finalize with H * D / 64 heads. dfin: gradient of the final state (fp32 [B*H, D, D]) or null.
void launch_gdn_chunk_bwd(const GlaMat& Q, const GlaMat& K, const GlaMat& V, const GlaMat& G, const GlaMat& dO,
                          const float* beta, const float* dfin, const GlaMat& dQ, const GlaMat& dK, const GlaMat& dV,
                          const GdnScratch& w, const GdnBwdScratch& x, const GdnDims& d, float scale, int* status,
                          cudaStream_t s);

}  // namespace tb
