// Gated DeltaNet, exact token recurrence in one kernel (inference / prefill / decode; no gradient).
//
//   v_pred = S_{t-1}^T k_t            u_t = v_t - v_pred
//   S_t    = diag(exp(g_t)) S_{t-1} + (beta_t * k_t) u_t^T          (g <= 0 per key dimension; beta per token and
//   o_t    = scale * S_t^T q_t                                        head, per key dimension, or absent = 1)
//
// One CTA per (batch, head). The dk x dv state lives in registers for the whole sequence: thread (part, c) owns
// rows [part*RP, part*RP + RP) of column c, so the two contractions of a token (k^T S and q^T S) are RP fused
// multiply-adds per thread plus a sum of the NPART partials through shared memory. Tokens are staged in blocks of 16
// through a double-buffered shared-memory ring with 16-byte loads, so global latency is paid once per block and
// overlaps the arithmetic of the previous block. A delta rule couples all key dimensions of a head (k^T S), so unlike
// plain GLA it cannot be split into 64-wide slices; the kernel is templated on the head dimension instead.
//
// Replaces the reference's per-token Python loop (triune/kernels/fast_gla.py:781-836) and its single-token decode.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <stdexcept>
#include <string>

#include "gla.cuh"

namespace tb {

namespace {


__device__ __forceinline__ float gdn_log_decay(float x, bool logits) {
  const float g = logits ? (fminf(x, 0.f) - log1pf(__expf(-fabsf(x)))) : fminf(x, 0.f);
  return fmaxf(g, GLA_MIN_LOG_DECAY);
}

// D: head dimension (keys and values). THREADS = D * NPART. GDN_TB: tokens per staged block.
template <int D, int NPART, int GDN_TB>
__global__ void __launch_bounds__(D* NPART) gdn_recurrent_kernel(
    const __nv_bfloat16* __restrict__ q, long long q_ld, int qcol, const __nv_bfloat16* __restrict__ k, long long k_ld,
    int kcol, const __nv_bfloat16* __restrict__ v, long long v_ld, int vcol, const __nv_bfloat16* __restrict__ g,
    long long g_ld, int gcol, const float* __restrict__ beta, int beta_mode /*0 none, 1 [B*T,H], 2 [B*T,H*D]*/,
    float* __restrict__ state /*[B*H, D, D] in/out*/, __nv_bfloat16* __restrict__ out, long long o_ld, int ocol, int T,
    int H, int logits, float scale) {
  constexpr int RP = D / NPART;          // state rows per thread
  constexpr int VEC = D / 8;             // 16-byte vectors per token and tensor
  __shared__ __align__(16) __nv_bfloat16 sIn[2][GDN_TB][4][D];  // q, k, v, g of a token block
  __shared__ float sBeta[2][GDN_TB][D];                         // beta per key dimension (mode 2) or [.][0] (mode 1)
  __shared__ float sK[D], sQ[D], sDec[D];                       // current token: beta*k, q, exp(g) in fp32
  __shared__ float sKraw[D];
  __shared__ float sPart[2][NPART][D];

  const int tid = threadIdx.x, c = tid % D, part = tid / D;
  const int bh = blockIdx.x, h = bh % H, b = bh / H;
  const long long row0 = (long long)b * T;

  float S[RP];
  {
    const float* sp = state + ((long long)bh * D + part * RP) * D + c;
#pragma unroll
    for (int r = 0; r < RP; ++r) S[r] = sp[(long long)r * D];
  }

  auto stage = [&](int blk, int buf) {
    const int t0 = blk * GDN_TB;
    for (int i = tid; i < GDN_TB * 4 * VEC; i += D * NPART) {
      const int tt = i / (4 * VEC), rem = i % (4 * VEC), which = rem / VEC, vec = rem % VEC;
      const int t = t0 + tt;
      if (t < T) {
        const __nv_bfloat16* src = which == 0   ? q + (row0 + t) * q_ld + qcol
                                   : which == 1 ? k + (row0 + t) * k_ld + kcol
                                   : which == 2 ? v + (row0 + t) * v_ld + vcol
                                                : g + (row0 + t) * g_ld + gcol;
        // asynchronous 16-byte copy: the block lands while the previous one is being computed
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(
                         (uint32_t)__cvta_generic_to_shared(&sIn[buf][tt][which][vec * 8])),
                     "l"(src + h * D + vec * 8)
                     : "memory");
      } else {
        *reinterpret_cast<uint4*>(&sIn[buf][tt][which][vec * 8]) = make_uint4(0u, 0u, 0u, 0u);
      }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
    if (beta_mode == 2) {
      for (int i = tid; i < GDN_TB * D; i += D * NPART) {
        const int tt = i / D, d = i % D, t = t0 + tt;
        sBeta[buf][tt][d] = t < T ? beta[((row0 + t) * H + h) * D + d] : 0.f;
      }
    } else if (beta_mode == 1) {
      if (tid < GDN_TB) sBeta[buf][tid][0] = (t0 + tid) < T ? beta[(row0 + t0 + tid) * H + h] : 0.f;
    }
  };

  const int nblk = (T + GDN_TB - 1) / GDN_TB;
  stage(0, 0);
  asm volatile("cp.async.wait_group 0;" ::: "memory");
  __syncthreads();
  for (int blk = 0; blk < nblk; ++blk) {
    const int buf = blk & 1;
    if (blk + 1 < nblk) stage(blk + 1, buf ^ 1);  // lands in the other buffer while this block is computed
    const int tcount = min(GDN_TB, T - blk * GDN_TB);
    for (int tt = 0; tt < tcount; ++tt) {
      // token operands in fp32: one thread per key dimension
      if (tid < D) {
        const float kk = __bfloat162float(sIn[buf][tt][1][tid]);
        const float bt = beta_mode == 0 ? 1.f : (beta_mode == 1 ? sBeta[buf][tt][0] : sBeta[buf][tt][tid]);
        sKraw[tid] = kk;
        sK[tid] = bt * kk;
        sQ[tid] = __bfloat162float(sIn[buf][tt][0][tid]);
        sDec[tid] = __expf(gdn_log_decay(__bfloat162float(sIn[buf][tt][3][tid]), logits != 0));
      }
      __syncthreads();
      float acc = 0.f;
#pragma unroll
      for (int r = 0; r < RP; ++r) acc += sKraw[part * RP + r] * S[r];
      sPart[0][part][c] = acc;
      __syncthreads();
      float vp = 0.f;
#pragma unroll
      for (int pp = 0; pp < NPART; ++pp) vp += sPart[0][pp][c];
      const float u = __bfloat162float(sIn[buf][tt][2][c]) - vp;
      float oacc = 0.f;
#pragma unroll
      for (int r = 0; r < RP; ++r) {
        const int d = part * RP + r;
        S[r] = sDec[d] * S[r] + sK[d] * u;
        oacc += sQ[d] * S[r];
      }
      sPart[1][part][c] = oacc;
      __syncthreads();
      if (part == 0) {
        float o = 0.f;
#pragma unroll
        for (int pp = 0; pp < NPART; ++pp) o += sPart[1][pp][c];
        out[(row0 + blk * GDN_TB + tt) * o_ld + ocol + h * D + c] = __float2bfloat16(o * scale);
      }
      // the next token's operand pass rewrites sK.. only after every thread passed the barrier above, and sPart[0] is
      // rewritten only after the next operand barrier: no further barrier needed here
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncthreads();  // block boundary: the staged next block is complete and this buffer may be overwritten
  }
  {
    float* sp = state + ((long long)bh * D + part * RP) * D + c;
#pragma unroll
    for (int r = 0; r < RP; ++r) sp[(long long)r * D] = S[r];
  }
}

}  // namespace

void launch_gdn_recurrent(const GlaMat& Q, const GlaMat& K, const GlaMat& V, const GlaMat& G, const float* beta,
                          int beta_mode, float* state, const GlaMat& O, int B, int T, int H, int D, bool logits,
                          float scale, cudaStream_t s) {
  if (B <= 0 || T <= 0) return;
  auto p = [](const GlaMat& m) { return reinterpret_cast<const __nv_bfloat16*>(m.ptr); };
  auto po = reinterpret_cast<__nv_bfloat16*>(const_cast<void*>(O.ptr));
  if (D == 64)
    gdn_recurrent_kernel<64, 4, 16><<<B * H, 256, 0, s>>>(p(Q), Q.ld, Q.col0, p(K), K.ld, K.col0, p(V), V.ld, V.col0, p(G),
                                                      G.ld, G.col0, beta, beta_mode, state, po, O.ld, O.col0, T, H,
                                                      logits ? 1 : 0, scale);
  else if (D == 128)
    gdn_recurrent_kernel<128, 4, 8><<<B * H, 512, 0, s>>>(p(Q), Q.ld, Q.col0, p(K), K.ld, K.col0, p(V), V.ld, V.col0, p(G),
                                                       G.ld, G.col0, beta, beta_mode, state, po, O.ld, O.col0, T, H,
                                                       logits ? 1 : 0, scale);
  else
    throw std::runtime_error("gdn_recurrent: head dimension must be 64 or 128");
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) throw std::runtime_error(std::string("gdn_recurrent launch failed: ") + cudaGetErrorString(e));
}

}  // namespace tb
