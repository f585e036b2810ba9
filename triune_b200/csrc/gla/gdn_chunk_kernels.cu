// Chunk-parallel Gated DeltaNet for training (forward and backward), head_dim 64 or 128, chunk 64.
//
// Recurrence per (batch, head), g <= 0 a per-key-dimension log decay, beta a per-token write strength:
//   u_t = beta_t (v_t - S_{t-1}^T k_t),   S_t = diag(e^{g_t}) S_{t-1} + k_t u_t^T,   o_t = S_t^T q_t.
// Inside a chunk (b = inclusive cumsum of g, bp = exclusive, b_C = last row):
//   Kbar = k e^{bp}   Qbar = q e^{b}   Kend = k e^{b_C - b}
//   Lraw[t,s] = sum_d k_td k_sd e^{bp_td - b_sd} (s < t)    L = diag(beta) Lraw    T = (I + L)^-1
//   A[t,s]    = sum_d q_td k_sd e^{b_td - b_sd}  (s <= t)
//   F1  U0 = T (beta V), W = T (beta Kbar)                     per chunk, tcgen05
//   F2  U = U0 - W S,  S' = diag(e^{b_C}) S + Kend^T U         sequential over chunks, fp32 CUDA cores, dv-sliced
//   F3  O = A U + Qbar S                                        per chunk, tcgen05
//   B1  G1 = A^T dO, H1 = Qbar^T dO                             per chunk, tcgen05
//   B2  dU = G1 + Kend dS',  dS = H1 + e^{b_C} dS' - W^T dU     reverse sequential (same kernel as F2)
//   B3a dQbar = dO S^T, dKend = U dS'^T, dW = -dU S^T           per chunk, tcgen05
//   B3b dVb = T^T dU, dKb = T^T dW, dL = -strict(dVb U0^T + dKb W^T), dv, dbeta, dLraw = beta dL
//   B3c dA = mask(dO U^T); dq, dk from dA and dLraw through the sub-chunk factorisation; gate-gradient terms
// The decayed scores only factor into matrix products around a reference row; as in the GLA kernels every 16-token
// sub-chunk j of keys is referenced to r_j = b at the row before it:
//   K~[s] = k_s e^{r_j(s) - b_s} (exponent in [0, 80]),  Q~(j)[t] = q_t e^{b_t - r_j},  K^(j)[t] = k_t e^{bp_t - r_j}
//   (both <= 0 exponents, zero rows for t < 16 j), A[:, 16j:16j+16] = Q~(j) K~_j^T,  Lraw[:, 16j:16j+16] = K^(j) K~_j^T.
// Gate gradient: everything depends on g only through q e^{B}, the write key k e^{-B} and the read key k e^{B_{t-1}}
// (B = cumulative log decay of the whole sequence), so dL/dB_t = q dq - k dk_w + (k dk_r)_{t+1} and dg is its suffix sum;
// B3c emits the in-chunk suffix sums and chunk totals that gla_dg_finalize completes.
//
// Replaces the reference's Python chunk loop and Triton forward (triune/kernels/fast_gla.py:382-550, 781-836).
#include <cuda.h>

#include <stdexcept>
#include <string>

#include "../common/per_device.h"
#include "../common/ptx.cuh"
#include "../common/tma_desc.h"
#include "gla.cuh"
#include "gla_tiles.cuh"

namespace tb {

namespace {

constexpr int C = 64;            // chunk length
constexpr int GDN_THREADS = 256;
constexpr int LP = 68;           // row pitch (floats) of 64 x 64 fp32 scratch matrices

struct GBars {
  uint64_t tma;
  uint64_t mma[4];
  uint32_t tmem_slot;
  int failed;
};

__device__ __forceinline__ uint8_t* aligned_smem(uint8_t* raw) {
  const uint32_t a = smem_u32(raw);
  return raw + (((a + 1023u) & ~1023u) - a);
}

__device__ __forceinline__ void cta_setup(GBars* bars, int nmma, uint32_t tmem_cols) {
  if (threadIdx.x == 0) {
    mbar_init(&bars->tma, 1);
    for (int i = 0; i < nmma; ++i) mbar_init(&bars->mma[i], 1);
    bars->failed = 0;
    mbar_fence_init();
  }
  if ((threadIdx.x >> 5) == 0) {
    tmem_alloc(&bars->tmem_slot, tmem_cols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
}

__device__ __forceinline__ void cta_teardown(GBars* bars, uint32_t tmem, uint32_t tmem_cols, int* status) {
  tc_fence_before_sync();
  __syncthreads();
  if (bars->failed != 0 && threadIdx.x == 0 && status != nullptr) atomicCAS(status, 0, bars->failed);
  if ((threadIdx.x >> 5) == 0) {
    tc_fence_after_sync();
    tmem_dealloc(tmem, tmem_cols);
  }
}

// All threads: wait for the input tiles; false (and the failure recorded) when the wait ran out.
__device__ __forceinline__ bool wait_inputs(GBars* bars) {
  if (!mbar_wait(&bars->tma, 0)) bars->failed = ST_TIMEOUT_FULL;
  __syncthreads();
  return bars->failed == 0;
}
// All threads: wait for the MMAs committed to barrier i (each barrier is used once per CTA).
__device__ __forceinline__ bool wait_mma(GBars* bars, int i) {
  const bool ok = __all_sync(0xffffffffu, mbar_wait(&bars->mma[i], 0));
  if (ok)
    tc_fence_after_sync();
  else if ((threadIdx.x & 31) == 0)
    bars->failed = ST_TIMEOUT_TMEM;
  return ok;
}
// Phase boundary: shared-memory writes of this phase become visible to the tensor core / every thread.
__device__ __forceinline__ bool phase_sync(GBars* bars) {
  fence_proxy_async_smem();
  tc_fence_before_sync();
  __syncthreads();
  return bars->failed == 0;
}

// bmat[t][d] (fp32, row pitch D + 4) = inclusive cumulative clamped log decay of the gate tiles (D / 64 tiles side by side).
template <int D>
__device__ __forceinline__ void cumsum_d(const uint8_t* sG, float* bmat, bool logits) {
  constexpr int PARTS = GDN_THREADS / D, LEN = C / PARTS, BST = D + 4;
  __shared__ float totals[GDN_THREADS];
  const int tid = threadIdx.x, d = tid % D, part = tid / D;
  const uint8_t* tile = sG + (d >> 6) * TILE;
  const int dc = d & 63;
  float c[LEN];
  float run = 0.f;
#pragma unroll
  for (int i = 0; i < LEN; ++i) {
    const int r = part * LEN + i;
    const __nv_bfloat16 x = *reinterpret_cast<const __nv_bfloat16*>(tile + sw_off(r, dc >> 3) + (dc & 7) * 2);
    run += log_decay(__bfloat162float(x), logits);
    c[i] = run;
  }
  totals[part * D + d] = run;
  __syncthreads();
  float base = 0.f;
  for (int pp = 0; pp < part; ++pp) base += totals[pp * D + d];
#pragma unroll
  for (int i = 0; i < LEN; ++i) bmat[(part * LEN + i) * BST + d] = base + c[i];
  __syncthreads();
}

// ftab[(i * 4 + j) * D + d] = e^{r_i - r_j} for j <= i (1 on the diagonal, 0 above), r_0 = 0, r_i = b[16 i - 1].
template <int D>
__device__ __forceinline__ void factor_tables_d(const float* bmat, float* ftab) {
  constexpr int BST = D + 4;
  for (int idx = threadIdx.x; idx < 16 * D; idx += GDN_THREADS) {
    const int d = idx % D, ij = idx / D, i = ij >> 2, j = ij & 3;
    float f = 0.f;
    if (j <= i) {
      const float ri = i == 0 ? 0.f : bmat[(16 * i - 1) * BST + d];
      const float rj = j == 0 ? 0.f : bmat[(16 * j - 1) * BST + d];
      f = j == i ? 1.f : __expf(ri - rj);
    }
    ftab[idx] = f;
  }
  __syncthreads();
}

// Rows of the cumulative decay around one row: b_t, bp_t = b_{t-1} (0 for t = 0), r_i (0 for i = 0), for 8 dims.
template <int D>
__device__ __forceinline__ void decay_rows(const float* bmat, int row, int col8, float (&bt)[8], float (&bp)[8],
                                           float (&ri)[8]) {
  constexpr int BST = D + 4;
  ld8(bmat + row * BST + col8, bt);
  if (row == 0) {
#pragma unroll
    for (int e = 0; e < 8; ++e) bp[e] = 0.f;
  } else {
    ld8(bmat + (row - 1) * BST + col8, bp);
  }
  const int i = row >> 4;
  if (i == 0) {
#pragma unroll
    for (int e = 0; e < 8; ++e) ri[e] = 0.f;
  } else {
    ld8(bmat + (16 * i - 1) * BST + col8, ri);
  }
}

// Score operands of a chunk. From q and k tiles (D / 64 tiles side by side each):
//   aj[j] (D / 64 tiles each): X~(j)[t] = x_t e^{c_t - r_j} for j <= i(t), zero rows otherwise, with c = b (queries) or
//                              c = bp (keys in their row role: USE_BP)
//   sKt: K~[s] = k_s e^{r_i(s) - b_s}
// x may be q (F3, B1, B3c) or k (F1, B3c); sX == nullptr skips the row-side tiles, sKsrc == nullptr skips K~.
template <int D, bool USE_BP>
__device__ __forceinline__ void build_row_operands(const uint8_t* sX, uint8_t* const (&aj)[4], const float* bmat,
                                                   const float* ftab) {
  constexpr int CH = D / 8;
  for (int idx = threadIdx.x; idx < C * CH; idx += GDN_THREADS) {
    const int row = idx / CH, ch = idx % CH, half = ch >> 3, cc = ch & 7;
    const uint32_t off = half * TILE + sw_off(row, cc);
    float x[8], bt[8], bp[8], ri[8], xe[8], o[8];
    unpack8(*reinterpret_cast<const uint4*>(sX + off), x);
    decay_rows<D>(bmat, row, ch * 8, bt, bp, ri);
    const int i = row >> 4;
#pragma unroll
    for (int e = 0; e < 8; ++e) xe[e] = x[e] * __expf((USE_BP ? bp[e] : bt[e]) - ri[e]);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      if (j < i) {
        float f[8];
        ld8(ftab + (i * 4 + j) * D + ch * 8, f);
#pragma unroll
        for (int e = 0; e < 8; ++e) o[e] = xe[e] * f[e];
      } else if (j == i) {
#pragma unroll
        for (int e = 0; e < 8; ++e) o[e] = xe[e];
      } else {
#pragma unroll
        for (int e = 0; e < 8; ++e) o[e] = 0.f;
      }
      *reinterpret_cast<uint4*>(aj[j] + off) = pack8(o);
    }
  }
}
template <int D>
__device__ __forceinline__ void build_key_operand(const uint8_t* sK, uint8_t* sKt, const float* bmat) {
  constexpr int CH = D / 8;
  for (int idx = threadIdx.x; idx < C * CH; idx += GDN_THREADS) {
    const int row = idx / CH, ch = idx % CH, half = ch >> 3, cc = ch & 7;
    const uint32_t off = half * TILE + sw_off(row, cc);
    float k[8], bt[8], bp[8], ri[8], o[8];
    unpack8(*reinterpret_cast<const uint4*>(sK + off), k);
    decay_rows<D>(bmat, row, ch * 8, bt, bp, ri);
#pragma unroll
    for (int e = 0; e < 8; ++e) o[e] = k[e] * __expf(ri[e] - bt[e]);
    *reinterpret_cast<uint4*>(sKt + off) = pack8(o);
  }
}

// Score MMAs: acc[:, 16j:16j+16] = X~(j) K~_j^T reduced over D (one thread issues).
template <int D>
__device__ __forceinline__ void issue_scores(uint32_t tmem_col, const uint32_t (&aj)[4], uint32_t kt_addr) {
  constexpr int NH = D / 64;
  constexpr uint32_t idesc = make_idesc(64, 16, 1, 1, 0, 0);
#pragma unroll
  for (int j = 0; j < 4; ++j) {
#pragma unroll
    for (int h = 0; h < NH; ++h) {
#pragma unroll
      for (int k = 0; k < 4; ++k)
        umma_bf16(tmem_col + 16 * j, desc_k(aj[j] + h * TILE, k), desc_k(kt_addr + h * TILE + j * 2048, k), idesc,
                  (h > 0 || k > 0) ? 1u : 0u);
    }
  }
}

// Row / column ownership of an M = 64 accumulator with NC columns among the eight warps: TMEM lane quarter
// (warp & 3) holds rows 16 q .. 16 q + 15 in its lanes 0..15; the two warps of a quarter split the columns.
struct Acc64 {
  int quarter, chalf, row;
  bool active;
  __device__ __forceinline__ Acc64() {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    quarter = warp & 3;
    chalf = warp >> 2;
    row = quarter * 16 + (lane & 15);
    active = lane < 16;
  }
};

__device__ __forceinline__ void store8_bf16(__nv_bfloat16* dst, const float* v) {
  float o[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) o[e] = v[e];
  *reinterpret_cast<uint4*>(dst) = pack8(o);
}

// ------------------------------------------------------------------------------------------------
// F1: per chunk  U0 = T (beta V), W = T (beta Kbar), T = (I + diag(beta) Lraw)^-1; also Kend and e^{b_C}.
// ------------------------------------------------------------------------------------------------
template <int D>
struct WyCfg {
  static constexpr int NH = D / 64;
  static constexpr int TILES = 4 * NH /*K V G Kt*/ + 4 * NH /*K^(j), later beta V | beta Kbar*/ + 1 /*T*/;
  static constexpr int BMAT = C * (D + 4) * 4;
  static constexpr int SMEM = TILES * TILE + BMAT + 16 * D * 4 + C * LP * 4 + 1024 + 256;
  static constexpr int TMEM_COLS = D == 128 ? 512 : 256;  // 64 score columns + 2 D
};

template <int D>
__global__ void __launch_bounds__(GDN_THREADS) gdn_wy_kernel(
    const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
    const __grid_constant__ CUtensorMap tmG, int kcol, int vcol, int gcol, const float* __restrict__ beta,
    __nv_bfloat16* __restrict__ U0_out, __nv_bfloat16* __restrict__ W_out, __nv_bfloat16* __restrict__ T_out,
    __nv_bfloat16* __restrict__ Kend_out, float* __restrict__ decay_out, float* __restrict__ Lraw_out, int T, int H,
    int logits, int* status) {
  using Cfg = WyCfg<D>;
  constexpr int NH = Cfg::NH, BST = D + 4, CH = D / 8;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = aligned_smem(smem_raw);
  uint8_t* sK = smem;
  uint8_t* sV = sK + NH * TILE;
  uint8_t* sG = sV + NH * TILE;
  uint8_t* sKt = sG + NH * TILE;
  uint8_t* sR = sKt + NH * TILE;   // 4 * NH tiles: K^(1) K^(0) K^(2) K^(3); later [beta V | beta Kbar] in the first 2 * NH
  uint8_t* sT = sR + 4 * NH * TILE;
  float* bmat = reinterpret_cast<float*>(sT + TILE);
  float* ftab = bmat + C * BST;
  float* Lm = ftab + 16 * D;
  GBars* bars = reinterpret_cast<GBars*>(Lm + C * LP);
  const int tid = threadIdx.x;
  const int NT = T / C;
  const int cidx = blockIdx.x, chunk = cidx % NT, bh = cidx / NT, h = bh % H, b = bh / H;
  const int row0 = b * T + chunk * C;

  cta_setup(bars, 2, Cfg::TMEM_COLS);
  const uint32_t tmem = bars->tmem_slot;
  if (tid == 0) {
    mbar_expect_tx(&bars->tma, 3 * NH * TILE);
#pragma unroll
    for (int n = 0; n < NH; ++n) {
      tma_load_3d(sK + n * TILE, &tmK, &bars->tma, kcol + h * D + n * 64, row0, 0);
      tma_load_3d(sV + n * TILE, &tmV, &bars->tma, vcol + h * D + n * 64, row0, 0);
      tma_load_3d(sG + n * TILE, &tmG, &bars->tma, gcol + h * D + n * 64, row0, 0);
    }
  }
  bool ok = wait_inputs(bars);
  const Acc64 me;
  // K^(j) lives at tile block perm(j): K^(0) = Kbar sits second so that [beta V | beta Kbar] can later be formed in
  // the first 2 * NH tiles with Kbar scaled in place.
  uint8_t* const kh[4] = {sR + 1 * NH * TILE, sR + 0 * NH * TILE, sR + 2 * NH * TILE, sR + 3 * NH * TILE};
  if (ok) {
    cumsum_d<D>(sG, bmat, logits != 0);
    factor_tables_d<D>(bmat, ftab);
    build_row_operands<D, true>(sK, kh, bmat, ftab);
    build_key_operand<D>(sK, sKt, bmat);
    // Kend[s] = K~[s] e^{b_C - r_i(s)} and e^{b_C}: inputs of the state pass
    for (int idx = tid; idx < C * CH; idx += GDN_THREADS) {
      const int row = idx / CH, ch = idx % CH, half = ch >> 3, cc = ch & 7;
      float kt[8], bl[8], bt[8], bp[8], ri[8], o[8];
      unpack8(*reinterpret_cast<const uint4*>(sK + half * TILE + sw_off(row, cc)), kt);
      decay_rows<D>(bmat, row, ch * 8, bt, bp, ri);
      ld8(bmat + 63 * BST + ch * 8, bl);
#pragma unroll
      for (int e = 0; e < 8; ++e) o[e] = kt[e] * __expf(bl[e] - bt[e]);
      *reinterpret_cast<uint4*>(Kend_out + ((long long)cidx * C + row) * D + ch * 8) = pack8(o);
    }
    if (tid < D) decay_out[(long long)cidx * D + tid] = __expf(bmat[63 * BST + tid]);
  }
  ok = phase_sync(bars);
  if (ok) {
    if (tid == 0) {
      tc_fence_after_sync();
      const uint32_t aj[4] = {smem_u32(kh[0]), smem_u32(kh[1]), smem_u32(kh[2]), smem_u32(kh[3])};
      issue_scores<D>(tmem, aj, smem_u32(sKt));
      umma_commit(&bars->mma[0]);
    }
    ok = wait_mma(bars, 0);
    if (ok) {
      // L = diag(beta) strict(Lraw) into shared memory (fp32); the raw scores go out for the backward pass
      float v[32];
      load_acc_cols<32>(tmem, me.chalf * 32, me.quarter, v);
      if (me.active) {
        const float bt = beta != nullptr ? beta[(long long)(row0 + me.row) * H + h] : 1.f;
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const int s = me.chalf * 32 + i;
          const float raw = s < me.row ? v[i] : 0.f;
          Lm[me.row * LP + s] = bt * raw;
          if (Lraw_out != nullptr) Lraw_out[((long long)cidx * C + me.row) * C + s] = raw;
        }
      }
      // right-hand sides [beta V | beta Kbar] over the K^(j) tiles (the score MMAs have completed)
      for (int idx = tid; idx < C * CH; idx += GDN_THREADS) {
        const int row = idx / CH, ch = idx % CH, half = ch >> 3, cc = ch & 7;
        const uint32_t off = half * TILE + sw_off(row, cc);
        const float bt = beta != nullptr ? beta[(long long)(row0 + row) * H + h] : 1.f;
        float x[8];
        unpack8(*reinterpret_cast<const uint4*>(sV + off), x);
#pragma unroll
        for (int e = 0; e < 8; ++e) x[e] *= bt;
        *reinterpret_cast<uint4*>(sR + off) = pack8(x);
        uint4* pk = reinterpret_cast<uint4*>(sR + NH * TILE + off);
        unpack8(*pk, x);
#pragma unroll
        for (int e = 0; e < 8; ++e) x[e] *= bt;
        *pk = pack8(x);
      }
    }
  }
  ok = phase_sync(bars);
  if (ok) {
    // T = (I + L)^-1 by forward substitution: thread c owns column c, row i = e_i - L[i, :i] T[:i, c].
    if (tid < C) {
      float t[C];
#pragma unroll
      for (int i = 0; i < C; ++i) {
        float acc = (i == tid) ? 1.f : 0.f;
#pragma unroll
        for (int j = 0; j < i; j += 4) {
          const float4 l = *reinterpret_cast<const float4*>(Lm + i * LP + j);
          acc -= l.x * t[j];
          if (j + 1 < i) acc -= l.y * t[j + 1];
          if (j + 2 < i) acc -= l.z * t[j + 2];
          if (j + 3 < i) acc -= l.w * t[j + 3];
        }
        t[i] = acc;
      }
#pragma unroll
      for (int i = 0; i < C; ++i)
        *reinterpret_cast<__nv_bfloat16*>(sT + sw_off(i, tid >> 3) + (tid & 7) * 2) = __float2bfloat16(t[i]);
    }
  }
  ok = phase_sync(bars);
  if (ok) {
    if (tid == 0) {
      tc_fence_after_sync();
      constexpr uint32_t id = make_idesc(64, 2 * D, 1, 1, 0, 1);
      const uint32_t aT = smem_u32(sT), aR = smem_u32(sR);
#pragma unroll
      for (int k = 0; k < 4; ++k) umma_bf16(tmem + 64, desc_k(aT, k), desc_mn(aR, k), id, k > 0 ? 1u : 0u);
      umma_commit(&bars->mma[1]);
    }
    // T goes out (bf16, row-major) while the tensor core works
    for (int idx = tid; idx < C * 8; idx += GDN_THREADS) {
      const int row = idx >> 3, ch = idx & 7;
      *reinterpret_cast<uint4*>(T_out + ((long long)cidx * C + row) * C + ch * 8) =
          *reinterpret_cast<const uint4*>(sT + sw_off(row, ch));
    }
    ok = wait_mma(bars, 1);
    if (ok) {
      // accumulator columns [64, 64 + D) = U0, [64 + D, 64 + 2 D) = W; each thread row takes D / 2 columns of both
#pragma unroll 1
      for (int which = 0; which < 2; ++which) {
        __nv_bfloat16* dst = (which == 0 ? U0_out : W_out) + ((long long)cidx * C + me.row) * D;
#pragma unroll 1
        for (int c0 = me.chalf * (D / 2); c0 < (me.chalf + 1) * (D / 2); c0 += 32) {
          float v[32];
          load_acc_cols<32>(tmem, 64 + which * D + c0, me.quarter, v);
          if (me.active) {
#pragma unroll
            for (int c8 = 0; c8 < 4; ++c8) store8_bf16(dst + c0 + c8 * 8, v + c8 * 8);
          }
        }
      }
    }
  }
  cta_teardown(bars, tmem, Cfg::TMEM_COLS, status);
}

// ------------------------------------------------------------------------------------------------
// F2 / B2: the sequential pass over the chunks of one (batch, head), split over slices of 32 state columns.
//   forward:  U  = U0 - W S,        S <- e^{b_C} S + Kend^T U          (X1 = W,    X2 = Kend)
//   reverse:  dU = G1 + Kend dS,    dS <- H1 + e^{b_C} dS - W^T dU     (X1 = Kend, X2 = W)
// fp32 arithmetic on CUDA cores (the products are 64 x D x 32 per chunk and strictly sequential); the operand tiles
// of the next chunk are fetched with cp.async while the current one is processed.
// ------------------------------------------------------------------------------------------------
constexpr int DVS = 32;  // state columns per CTA

__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gsrc) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(smem_dst)), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

template <int D>
struct StateCfg {
  static constexpr int XP = D + 8;                     // row pitch (bf16) of the operand tiles
  static constexpr int X_BYTES = C * XP * 2;
  static constexpr int ADD_BYTES = C * DVS * 4;        // the [64, 32] addend slice (bf16 forward, fp32 reverse)
  static constexpr int SP = DVS + 4;                   // row pitch (floats) of the state slice, the product and its partial
  static constexpr int SMEM = 2 * (2 * X_BYTES + ADD_BYTES) + D * SP * 4 + 2 * C * SP * 4 + 1024 + 256;
  // update ownership: thread = (group of 4 state rows, CC consecutive columns)
  static constexpr int CC = D * DVS / GDN_THREADS / 4;  // 4 (D = 128) or 2 (D = 64)
  static constexpr int TPR = DVS / CC;                  // threads per row group
};

// Register tiling. Both products are bound by shared-memory bandwidth unless a thread reuses what it loads: a thread
// owns a 4 x 4 (product 1) or 4 x CC (product 2) block of outputs, so one 16-byte load of state (or product) values
// and one load of operand values feed 16 multiply-adds. Product 1 splits its reduction over the key dimension between
// the two halves of the block and adds the partial sums through shared memory.
template <int D, bool REV>
__global__ void __launch_bounds__(GDN_THREADS) gdn_state_kernel(
    const __nv_bfloat16* __restrict__ X1, const __nv_bfloat16* __restrict__ X2, const void* __restrict__ add1,
    const float* __restrict__ add2, const float* __restrict__ decay, const float* __restrict__ init,
    __nv_bfloat16* __restrict__ out1, __nv_bfloat16* __restrict__ states, float* __restrict__ fin, int NT) {
  using Cfg = StateCfg<D>;
  constexpr int XP = Cfg::XP, SP = Cfg::SP, CC = Cfg::CC, TPR = Cfg::TPR;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = aligned_smem(smem_raw);
  uint8_t* stage[2] = {smem, smem + 2 * Cfg::X_BYTES + Cfg::ADD_BYTES};
  float* sS = reinterpret_cast<float*>(smem + 2 * (2 * Cfg::X_BYTES + Cfg::ADD_BYTES));
  float* sP = sS + D * SP;      // product 1 (U or dU), fp32
  float* sRed = sP + C * SP;    // partial sums of product 1 from the upper half of the block
  const int tid = threadIdx.x;
  const int slices = D / DVS, bh = blockIdx.x / slices, slice = blockIdx.x % slices;
  const int col0 = slice * DVS;

  auto prefetch = [&](int i, int buf) {
    const int c = REV ? NT - 1 - i : i;
    const long long cidx = (long long)bh * NT + c;
    __nv_bfloat16* d1 = reinterpret_cast<__nv_bfloat16*>(stage[buf]);
    __nv_bfloat16* d2 = reinterpret_cast<__nv_bfloat16*>(stage[buf] + Cfg::X_BYTES);
    uint8_t* da = stage[buf] + 2 * Cfg::X_BYTES;
    const __nv_bfloat16* s1 = X1 + cidx * C * D;
    const __nv_bfloat16* s2 = X2 + cidx * C * D;
    for (int idx = tid; idx < C * (D / 8); idx += GDN_THREADS) {
      const int r = idx / (D / 8), v = idx % (D / 8);
      cp_async16(d1 + r * XP + v * 8, s1 + r * D + v * 8);
      cp_async16(d2 + r * XP + v * 8, s2 + r * D + v * 8);
    }
    if (REV) {
      const float* sa = reinterpret_cast<const float*>(add1) + cidx * C * D + col0;
      for (int idx = tid; idx < C * (DVS / 4); idx += GDN_THREADS) {
        const int r = idx / (DVS / 4), v = idx % (DVS / 4);
        cp_async16(da + (r * DVS + v * 4) * 4, sa + r * D + v * 4);
      }
    } else {
      const __nv_bfloat16* sa = reinterpret_cast<const __nv_bfloat16*>(add1) + cidx * C * D + col0;
      for (int idx = tid; idx < C * (DVS / 8); idx += GDN_THREADS) {
        const int r = idx / (DVS / 8), v = idx % (DVS / 8);
        cp_async16(da + (r * DVS + v * 8) * 2, sa + r * D + v * 8);
      }
    }
    cp_async_commit();
  };

  // state slice in registers: thread (row group sg, column group sc) holds S[4 sg .. 4 sg + 3][col0 + CC sc .. + CC)
  const int sg = tid / TPR, sc = tid % TPR;
  const int sd0 = sg * 4, scol = sc * CC;
  float S[4][CC];
#pragma unroll
  for (int r = 0; r < 4; ++r)
#pragma unroll
    for (int e = 0; e < CC; ++e)
      S[r][e] = init != nullptr ? init[((long long)bh * D + sd0 + r) * D + col0 + scol + e] : 0.f;
  // product 1 ownership: reduction half kh, rows 4 pg .. 4 pg + 3, columns 4 pc .. 4 pc + 3
  const int kh = tid >> 7, pg = (tid & 127) >> 3, pc = tid & 7;

  if (NT > 0) prefetch(0, 0);
  for (int i = 0; i < NT; ++i) {
    const int buf = i & 1;
    const int c = REV ? NT - 1 - i : i;
    const long long cidx = (long long)bh * NT + c;
    // state before this chunk goes out (bf16) and into shared memory (fp32) for the first product
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      __nv_bfloat16* so = states + (cidx * D + sd0 + r) * D + col0 + scol;
      if (CC == 4) {
        *reinterpret_cast<uint2*>(so) = make_uint2(pack_bf16x2(S[r][0], S[r][1]), pack_bf16x2(S[r][2 % CC], S[r][3 % CC]));
        *reinterpret_cast<float4*>(sS + (sd0 + r) * SP + scol) = make_float4(S[r][0], S[r][1], S[r][2 % CC], S[r][3 % CC]);
      } else {
        *reinterpret_cast<uint32_t*>(so) = pack_bf16x2(S[r][0], S[r][1]);
        *reinterpret_cast<float2*>(sS + (sd0 + r) * SP + scol) = make_float2(S[r][0], S[r][1]);
      }
    }
    // addends of the update, fetched early
    float dec[4], a2[4][CC];
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      dec[r] = decay[cidx * D + sd0 + r];
#pragma unroll
      for (int e = 0; e < CC; ++e) a2[r][e] = 0.f;
      if (REV) {
        const float* ap = add2 + (cidx * D + sd0 + r) * D + col0 + scol;
        if (CC == 4) {
          const float4 t = *reinterpret_cast<const float4*>(ap);
          a2[r][0] = t.x; a2[r][1] = t.y; a2[r][2 % CC] = t.z; a2[r][3 % CC] = t.w;
        } else {
          const float2 t = *reinterpret_cast<const float2*>(ap);
          a2[r][0] = t.x; a2[r][1] = t.y;
        }
      }
    }
    cp_async_wait<0>();
    __syncthreads();  // tiles of this chunk and the state slice are visible; the other stage is free
    if (i + 1 < NT) prefetch(i + 1, buf ^ 1);
    const __nv_bfloat16* x1 = reinterpret_cast<const __nv_bfloat16*>(stage[buf]);
    const __nv_bfloat16* x2 = reinterpret_cast<const __nv_bfloat16*>(stage[buf] + Cfg::X_BYTES);
    const uint8_t* ad = stage[buf] + 2 * Cfg::X_BYTES;
    // ---- product 1: P[r][cols] = add1[r][cols] -/+ X1[r][:] S[:, cols]; each block half reduces half of the key dims
    float acc[4][4];
#pragma unroll
    for (int r = 0; r < 4; ++r)
#pragma unroll
      for (int e = 0; e < 4; ++e) acc[r][e] = 0.f;
#pragma unroll 2
    for (int d8 = kh * (D / 16); d8 < (kh + 1) * (D / 16); ++d8) {
      float xw[4][8];
#pragma unroll
      for (int r = 0; r < 4; ++r) unpack8(*reinterpret_cast<const uint4*>(x1 + (pg * 4 + r) * XP + d8 * 8), xw[r]);
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const float4 s4 = *reinterpret_cast<const float4*>(sS + (d8 * 8 + e) * SP + pc * 4);
#pragma unroll
        for (int r = 0; r < 4; ++r) {
          acc[r][0] += xw[r][e] * s4.x; acc[r][1] += xw[r][e] * s4.y;
          acc[r][2] += xw[r][e] * s4.z; acc[r][3] += xw[r][e] * s4.w;
        }
      }
    }
    if (kh == 1) {
#pragma unroll
      for (int r = 0; r < 4; ++r)
        *reinterpret_cast<float4*>(sRed + (pg * 4 + r) * SP + pc * 4) = make_float4(acc[r][0], acc[r][1], acc[r][2], acc[r][3]);
    }
    __syncthreads();
    if (kh == 0) {
#pragma unroll
      for (int r = 0; r < 4; ++r) {
        const int row = pg * 4 + r;
        const float4 o = *reinterpret_cast<const float4*>(sRed + row * SP + pc * 4);
        float v[4] = {acc[r][0] + o.x, acc[r][1] + o.y, acc[r][2] + o.z, acc[r][3] + o.w};
        if (REV) {
          const float4 b = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(ad) + row * DVS + pc * 4);
          v[0] = b.x + v[0]; v[1] = b.y + v[1]; v[2] = b.z + v[2]; v[3] = b.w + v[3];
        } else {
          const uint2 raw = *reinterpret_cast<const uint2*>(reinterpret_cast<const __nv_bfloat16*>(ad) + row * DVS + pc * 4);
          float b0, b1, b2, b3;
          unpack_f2(bf16x2_to_f2(raw.x), b0, b1);
          unpack_f2(bf16x2_to_f2(raw.y), b2, b3);
          v[0] = b0 - v[0]; v[1] = b1 - v[1]; v[2] = b2 - v[2]; v[3] = b3 - v[3];
        }
        *reinterpret_cast<float4*>(sP + row * SP + pc * 4) = make_float4(v[0], v[1], v[2], v[3]);
        *reinterpret_cast<uint2*>(out1 + (cidx * C + row) * D + col0 + pc * 4) =
            make_uint2(pack_bf16x2(v[0], v[1]), pack_bf16x2(v[2], v[3]));
      }
    }
    __syncthreads();
    // ---- product 2: S[d][cols] = e^{b_C}[d] S + add2 +/- sum_t X2[t][d] P[t][cols]
    {
      float up[4][CC];
#pragma unroll
      for (int r = 0; r < 4; ++r)
#pragma unroll
        for (int e = 0; e < CC; ++e) up[r][e] = 0.f;
#pragma unroll 4
      for (int t = 0; t < C; ++t) {
        const uint2 xr = *reinterpret_cast<const uint2*>(x2 + t * XP + sd0);
        float xv[4];
        unpack_f2(bf16x2_to_f2(xr.x), xv[0], xv[1]);
        unpack_f2(bf16x2_to_f2(xr.y), xv[2], xv[3]);
        float pv[CC];
        if (CC == 4) {
          const float4 p = *reinterpret_cast<const float4*>(sP + t * SP + scol);
          pv[0] = p.x; pv[1] = p.y; pv[2 % CC] = p.z; pv[3 % CC] = p.w;
        } else {
          const float2 p = *reinterpret_cast<const float2*>(sP + t * SP + scol);
          pv[0] = p.x; pv[1] = p.y;
        }
#pragma unroll
        for (int r = 0; r < 4; ++r)
#pragma unroll
          for (int e = 0; e < CC; ++e) up[r][e] += xv[r] * pv[e];
      }
#pragma unroll
      for (int r = 0; r < 4; ++r)
#pragma unroll
        for (int e = 0; e < CC; ++e) S[r][e] = dec[r] * S[r][e] + a2[r][e] + (REV ? -up[r][e] : up[r][e]);
    }
    // the next iteration's barrier orders these reads of sP / stage[buf] against their next writes
  }
  cp_async_wait<0>();
#pragma unroll
  for (int r = 0; r < 4; ++r)
#pragma unroll
    for (int e = 0; e < CC; ++e) fin[((long long)bh * D + sd0 + r) * D + col0 + scol + e] = S[r][e];
}

// ------------------------------------------------------------------------------------------------
// F3: O = scale * (mask(P) U + Q~(0) S),  P[:, 16j:16j+16] = Q~(j) K~_j^T
// B1: G1 = mask(P)^T dO,  H1 = Q~(0)^T dO       (MODE_B1)
// ------------------------------------------------------------------------------------------------
template <int D, bool B1>
struct OutCfg {
  static constexpr int NH = D / 64;
  // Q K G | Y (U or dO) | S (forward only) | Q~(0..2) | K~ | P ; Q~(3) takes over the gate tiles
  static constexpr int TILES = 3 * NH + NH + (B1 ? 0 : NH * NH) + 3 * NH + NH + 1;
  static constexpr int BMAT = C * (D + 4) * 4;
  static constexpr int SMEM = TILES * TILE + BMAT + 16 * D * 4 + 1024 + 256;
  static constexpr int TMEM_COLS = B1 ? (D == 128 ? 512 : 256) : 256;
};

template <int D, bool B1>
__global__ void __launch_bounds__(GDN_THREADS) gdn_scores_kernel(
    const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
    const __grid_constant__ CUtensorMap tmG, const __grid_constant__ CUtensorMap tmY,
    const __grid_constant__ CUtensorMap tmS, int qcol, int kcol, int gcol, int ycol, int y_is_chunked,
    __nv_bfloat16* __restrict__ out, long long out_ld, int ocol, float scale, float* __restrict__ G1_out,
    float* __restrict__ H1_out, int T, int H, int logits, int* status) {
  using Cfg = OutCfg<D, B1>;
  constexpr int NH = Cfg::NH, BST = D + 4;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = aligned_smem(smem_raw);
  uint8_t* sQ = smem;
  uint8_t* sK = sQ + NH * TILE;
  uint8_t* sG = sK + NH * TILE;
  uint8_t* sY = sG + NH * TILE;
  uint8_t* sS = sY + NH * TILE;
  uint8_t* sA = sS + (B1 ? 0 : NH * NH) * TILE;  // Q~(0), Q~(1), Q~(2)
  uint8_t* sKt = sA + 3 * NH * TILE;
  uint8_t* sP = sKt + NH * TILE;
  float* bmat = reinterpret_cast<float*>(sP + TILE);
  float* ftab = bmat + C * BST;
  GBars* bars = reinterpret_cast<GBars*>(ftab + 16 * D);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int NT = T / C;
  const int cidx = blockIdx.x, chunk = cidx % NT, bh = cidx / NT, h = bh % H, b = bh / H;
  const int row0 = b * T + chunk * C;

  cta_setup(bars, 2, Cfg::TMEM_COLS);
  const uint32_t tmem = bars->tmem_slot;
  if (tid == 0) {
    mbar_expect_tx(&bars->tma, (4 * NH + (B1 ? 0 : NH * NH)) * TILE);
#pragma unroll
    for (int n = 0; n < NH; ++n) {
      tma_load_3d(sQ + n * TILE, &tmQ, &bars->tma, qcol + h * D + n * 64, row0, 0);
      tma_load_3d(sK + n * TILE, &tmK, &bars->tma, kcol + h * D + n * 64, row0, 0);
      tma_load_3d(sG + n * TILE, &tmG, &bars->tma, gcol + h * D + n * 64, row0, 0);
      if (y_is_chunked)
        tma_load_3d(sY + n * TILE, &tmY, &bars->tma, n * 64, cidx * C, 0);
      else
        tma_load_3d(sY + n * TILE, &tmY, &bars->tma, ycol + h * D + n * 64, row0, 0);
    }
    if (!B1) {
#pragma unroll
      for (int hh = 0; hh < NH; ++hh)
#pragma unroll
        for (int n = 0; n < NH; ++n)
          tma_load_3d(sS + (hh * NH + n) * TILE, &tmS, &bars->tma, n * 64, cidx * D + hh * 64, 0);
    }
  }
  bool ok = wait_inputs(bars);
  const Acc64 me;
  uint8_t* const qj[4] = {sA, sA + NH * TILE, sA + 2 * NH * TILE, sG};  // Q~(3) overwrites the gate tiles
  constexpr int COL_P = 0, COL_O = 64, COL_H = 64 + D;
  if (ok) {
    cumsum_d<D>(sG, bmat, logits != 0);
    factor_tables_d<D>(bmat, ftab);
    build_row_operands<D, false>(sQ, qj, bmat, ftab);
    build_key_operand<D>(sK, sKt, bmat);
  }
  ok = phase_sync(bars);
  if (ok) {
    if (tid == 0) {
      tc_fence_after_sync();
      const uint32_t aj[4] = {smem_u32(qj[0]), smem_u32(qj[1]), smem_u32(qj[2]), smem_u32(qj[3])};
      issue_scores<D>(tmem + COL_P, aj, smem_u32(sKt));
      if (B1) {
        // H1[dk, dv] = Q~(0)^T dO: M = D rows (key dims), reduction over the 64 tokens
        constexpr uint32_t id = make_idesc(D, D, 1, 1, 1, 1);
        const uint32_t a0 = smem_u32(qj[0]), ay = smem_u32(sY);
#pragma unroll
        for (int k = 0; k < 4; ++k) umma_bf16(tmem + COL_H, desc_mn(a0, k), desc_mn(ay, k), id, k > 0 ? 1u : 0u);
      } else {
        // Q~(0) S: reduction over the D key dims, S consumed as [dk rows][dv contiguous]
        constexpr uint32_t id = make_idesc(64, D, 1, 1, 0, 1);
        const uint32_t a0 = smem_u32(qj[0]), as = smem_u32(sS);
#pragma unroll
        for (int hh = 0; hh < NH; ++hh)
#pragma unroll
          for (int k = 0; k < 4; ++k)
            umma_bf16(tmem + COL_O, desc_k(a0 + hh * TILE, k), desc_mn(as + hh * NH * TILE, k), id,
                      (hh > 0 || k > 0) ? 1u : 0u);
      }
      umma_commit(&bars->mma[0]);
    }
    ok = wait_mma(bars, 0);
    if (ok) {
      float v[32];
      load_acc_cols<32>(tmem, COL_P + me.chalf * 32, me.quarter, v);
      if (me.active) store_row_cols<32>(sP, me.row, me.chalf * 32, v, me.row);  // causal mask, diagonal kept
    }
  }
  ok = phase_sync(bars);
  if (ok) {
    if (tid == 0) {
      tc_fence_after_sync();
      const uint32_t ap = smem_u32(sP), ay = smem_u32(sY);
      if (B1) {
        constexpr uint32_t id = make_idesc(64, D, 1, 1, 1, 1);  // G1 = P^T dO
#pragma unroll
        for (int k = 0; k < 4; ++k) umma_bf16(tmem + COL_O, desc_mn(ap, k), desc_mn(ay, k), id, k > 0 ? 1u : 0u);
      } else {
        constexpr uint32_t id = make_idesc(64, D, 1, 1, 0, 1);  // O += P U
#pragma unroll
        for (int k = 0; k < 4; ++k) umma_bf16(tmem + COL_O, desc_k(ap, k), desc_mn(ay, k), id, 1u);
      }
      umma_commit(&bars->mma[1]);
    }
    ok = wait_mma(bars, 1);
    if (ok) {
#pragma unroll 1
      for (int c0 = me.chalf * (D / 2); c0 < (me.chalf + 1) * (D / 2); c0 += 32) {
        float v[32];
        load_acc_cols<32>(tmem, COL_O + c0, me.quarter, v);
        if (me.active) {
          if (B1) {
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] *= scale;  // the output scale enters the backward pass here
            float* dst = G1_out + ((long long)cidx * C + me.row) * D + c0;
#pragma unroll
            for (int c4 = 0; c4 < 8; ++c4)
              *reinterpret_cast<float4*>(dst + c4 * 4) = make_float4(v[c4 * 4], v[c4 * 4 + 1], v[c4 * 4 + 2], v[c4 * 4 + 3]);
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] *= scale;
            __nv_bfloat16* dst = out + (long long)(row0 + me.row) * out_ld + ocol + h * D + c0;
#pragma unroll
            for (int c8 = 0; c8 < 4; ++c8) store8_bf16(dst + c8 * 8, v + c8 * 8);
          }
        }
      }
      if (B1) {
        // H1: M = D accumulator rows. D = 128: lane = row, two warps per lane quarter split the columns;
        // D = 64: the M = 64 layout.
        if (D == 128) {
          const int hrow = (warp & 3) * 32 + lane;
          float* dst = H1_out + ((long long)cidx * D + hrow) * D;
#pragma unroll 1
          for (int c0 = (warp >> 2) * 64; c0 < (warp >> 2) * 64 + 64; c0 += 32) {
            uint32_t r[32];
            tmem_ld_32x32b_x32(tmem + ((uint32_t)((warp & 3) * 32) << 16) + COL_H + c0, r);
            tmem_ld_wait();
#pragma unroll
            for (int c4 = 0; c4 < 8; ++c4)
              *reinterpret_cast<float4*>(dst + c0 + c4 * 4) =
                  make_float4(scale * __uint_as_float(r[c4 * 4]), scale * __uint_as_float(r[c4 * 4 + 1]),
                              scale * __uint_as_float(r[c4 * 4 + 2]), scale * __uint_as_float(r[c4 * 4 + 3]));
          }
        } else {
          float v[32];
          load_acc_cols<32>(tmem, COL_H + me.chalf * 32, me.quarter, v);
          if (me.active) {
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] *= scale;
            float* dst = H1_out + ((long long)cidx * D + me.row) * D + me.chalf * 32;
#pragma unroll
            for (int c4 = 0; c4 < 8; ++c4)
              *reinterpret_cast<float4*>(dst + c4 * 4) = make_float4(v[c4 * 4], v[c4 * 4 + 1], v[c4 * 4 + 2], v[c4 * 4 + 3]);
          }
        }
      }
    }
  }
  cta_teardown(bars, tmem, Cfg::TMEM_COLS, status);
}

// ------------------------------------------------------------------------------------------------
// B3a: dq1 = e^{b} (dO S^T),  dkw1 = e^{b_C - b} (U dS'^T),  dW = -(dU S^T)
// ------------------------------------------------------------------------------------------------
template <int D>
struct B3aCfg {
  static constexpr int NH = D / 64;
  static constexpr int TILES = 4 * NH /*dO U dU G*/ + 2 * NH * NH /*S, dS' as [dv half][D rows x 64]*/;
  static constexpr int BMAT = C * (D + 4) * 4;
  static constexpr int SMEM = TILES * TILE + BMAT + 1024 + 256;
  static constexpr int TMEM_COLS = D == 128 ? 512 : 256;
};

template <int D>
__global__ void __launch_bounds__(GDN_THREADS) gdn_bwd_state_terms_kernel(
    const __grid_constant__ CUtensorMap tmdO, const __grid_constant__ CUtensorMap tmU,
    const __grid_constant__ CUtensorMap tmdU, const __grid_constant__ CUtensorMap tmG,
    const __grid_constant__ CUtensorMap tmS, const __grid_constant__ CUtensorMap tmdS, int docol, int gcol,
    float* __restrict__ dq1, float* __restrict__ dkw1, __nv_bfloat16* __restrict__ dW, float scale, int T, int H,
    int logits, int* status) {
  using Cfg = B3aCfg<D>;
  constexpr int NH = Cfg::NH, BST = D + 4, SB = NH * TILE;  // one dv half of a state: D rows x 128 bytes
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = aligned_smem(smem_raw);
  uint8_t* sdO = smem;
  uint8_t* sU = sdO + NH * TILE;
  uint8_t* sdU = sU + NH * TILE;
  uint8_t* sG = sdU + NH * TILE;
  uint8_t* sS = sG + NH * TILE;
  uint8_t* sdS = sS + NH * SB;
  float* bmat = reinterpret_cast<float*>(sdS + NH * SB);
  GBars* bars = reinterpret_cast<GBars*>(bmat + C * BST);
  const int tid = threadIdx.x;
  const int NT = T / C;
  const int cidx = blockIdx.x, chunk = cidx % NT, bh = cidx / NT, h = bh % H, b = bh / H;
  const int row0 = b * T + chunk * C;

  cta_setup(bars, 1, Cfg::TMEM_COLS);
  const uint32_t tmem = bars->tmem_slot;
  if (tid == 0) {
    mbar_expect_tx(&bars->tma, (4 * NH + 2 * NH * NH) * TILE);
#pragma unroll
    for (int n = 0; n < NH; ++n) {
      tma_load_3d(sdO + n * TILE, &tmdO, &bars->tma, docol + h * D + n * 64, row0, 0);
      tma_load_3d(sU + n * TILE, &tmU, &bars->tma, n * 64, cidx * C, 0);
      tma_load_3d(sdU + n * TILE, &tmdU, &bars->tma, n * 64, cidx * C, 0);
      tma_load_3d(sG + n * TILE, &tmG, &bars->tma, gcol + h * D + n * 64, row0, 0);
      // states as K-major B operands: [dv half n][D key rows][64 value columns]
      tma_load_3d(sS + n * SB, &tmS, &bars->tma, n * 64, cidx * D, 0);
      tma_load_3d(sdS + n * SB, &tmdS, &bars->tma, n * 64, cidx * D, 0);
    }
  }
  bool ok = wait_inputs(bars);
  const Acc64 me;
  if (ok) {
    if (tid == 0) {
      tc_fence_after_sync();
      constexpr uint32_t id = make_idesc(64, D, 1, 1, 0, 0);
      const uint32_t ado = smem_u32(sdO), au = smem_u32(sU), adu = smem_u32(sdU), as = smem_u32(sS), ads = smem_u32(sdS);
#pragma unroll
      for (int n = 0; n < NH; ++n)
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const uint32_t acc = (n > 0 || k > 0) ? 1u : 0u;
          umma_bf16(tmem + 0, desc_k(ado + n * TILE, k), desc_k(as + n * SB, k), id, acc);       // dO S^T
          umma_bf16(tmem + D, desc_k(au + n * TILE, k), desc_k(ads + n * SB, k), id, acc);        // U dS'^T
          umma_bf16(tmem + 2 * D, desc_k(adu + n * TILE, k), desc_k(as + n * SB, k), id, acc);    // dU S^T
        }
      umma_commit(&bars->mma[0]);
    }
    cumsum_d<D>(sG, bmat, logits != 0);
    ok = wait_mma(bars, 0);
    if (ok) {
#pragma unroll 1
      for (int c0 = me.chalf * (D / 2); c0 < (me.chalf + 1) * (D / 2); c0 += 32) {
        float v[32], bt[32], bl[32];
        if (me.active) {
          ld_row<32>(bmat + me.row * BST + c0, bt);
          ld_row<32>(bmat + 63 * BST + c0, bl);
        }
        const long long o = ((long long)cidx * C + me.row) * D + c0;
        load_acc_cols<32>(tmem, 0 + c0, me.quarter, v);
        if (me.active) {
#pragma unroll
          for (int c4 = 0; c4 < 8; ++c4)
            *reinterpret_cast<float4*>(dq1 + o + c4 * 4) =
                make_float4(scale * v[c4 * 4] * __expf(bt[c4 * 4]), scale * v[c4 * 4 + 1] * __expf(bt[c4 * 4 + 1]),
                            scale * v[c4 * 4 + 2] * __expf(bt[c4 * 4 + 2]), scale * v[c4 * 4 + 3] * __expf(bt[c4 * 4 + 3]));
        }
        load_acc_cols<32>(tmem, D + c0, me.quarter, v);
        if (me.active) {
#pragma unroll
          for (int c4 = 0; c4 < 8; ++c4)
            *reinterpret_cast<float4*>(dkw1 + o + c4 * 4) =
                make_float4(v[c4 * 4] * __expf(bl[c4 * 4] - bt[c4 * 4]), v[c4 * 4 + 1] * __expf(bl[c4 * 4 + 1] - bt[c4 * 4 + 1]),
                            v[c4 * 4 + 2] * __expf(bl[c4 * 4 + 2] - bt[c4 * 4 + 2]),
                            v[c4 * 4 + 3] * __expf(bl[c4 * 4 + 3] - bt[c4 * 4 + 3]));
        }
        load_acc_cols<32>(tmem, 2 * D + c0, me.quarter, v);
        if (me.active) {
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = -v[i];
#pragma unroll
          for (int c8 = 0; c8 < 4; ++c8) store8_bf16(dW + o + c8 * 8, v + c8 * 8);
        }
      }
    }
  }
  cta_teardown(bars, tmem, Cfg::TMEM_COLS, status);
}

// ------------------------------------------------------------------------------------------------
// B3b: through the UT transform. [dVb | dKb] = T^T [dU | dW];  dL = -strict(dVb U0^T + dKb W^T);
//      dv = beta dVb;  dkr1 = beta e^{bp} dKb;  dbeta = <dVb, V> + <dKb, Kbar> + <dL, Lraw>;  dLraw = beta dL
// ------------------------------------------------------------------------------------------------
template <int D>
struct B3bCfg {
  static constexpr int NH = D / 64;
  static constexpr int TILES = 1 /*T*/ + 2 * NH /*dU dW*/ + 2 * NH /*U0 W*/ + 3 * NH /*V K G*/ + 2 * NH /*dVb dKb*/;
  static constexpr int BMAT = C * (D + 4) * 4;
  static constexpr int SMEM = TILES * TILE + BMAT + C * 4 + 1024 + 256;
  static constexpr int TMEM_COLS = D == 128 ? 512 : 256;  // 2 D + 64
};

template <int D>
__global__ void __launch_bounds__(GDN_THREADS) gdn_bwd_wy_kernel(
    const __grid_constant__ CUtensorMap tmT, const __grid_constant__ CUtensorMap tmdU,
    const __grid_constant__ CUtensorMap tmdW, const __grid_constant__ CUtensorMap tmU0,
    const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmV,
    const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmG, int vcol, int kcol, int gcol,
    const float* __restrict__ beta, const float* __restrict__ Lraw, __nv_bfloat16* __restrict__ dv, long long dv_ld,
    int dvcol, float* __restrict__ dkr1, float* __restrict__ dbeta, __nv_bfloat16* __restrict__ dLraw, int T, int H,
    int logits, int* status) {
  using Cfg = B3bCfg<D>;
  constexpr int NH = Cfg::NH, BST = D + 4;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = aligned_smem(smem_raw);
  uint8_t* sT = smem;
  uint8_t* sdUW = sT + TILE;            // [dU | dW]: 2 * NH tiles, one MN-major B operand of width 2 D
  uint8_t* sU0 = sdUW + 2 * NH * TILE;
  uint8_t* sW = sU0 + NH * TILE;
  uint8_t* sV = sW + NH * TILE;
  uint8_t* sK = sV + NH * TILE;
  uint8_t* sG = sK + NH * TILE;
  uint8_t* sdVb = sG + NH * TILE;
  uint8_t* sdKb = sdVb + NH * TILE;
  float* bmat = reinterpret_cast<float*>(sdKb + NH * TILE);
  float* dbs = bmat + C * BST;  // per-row dbeta partial sums
  GBars* bars = reinterpret_cast<GBars*>(dbs + C);
  const int tid = threadIdx.x;
  const int NT = T / C;
  const int cidx = blockIdx.x, chunk = cidx % NT, bh = cidx / NT, h = bh % H, b = bh / H;
  const int row0 = b * T + chunk * C;

  cta_setup(bars, 2, Cfg::TMEM_COLS);
  const uint32_t tmem = bars->tmem_slot;
  if (tid == 0) {
    mbar_expect_tx(&bars->tma, (1 + 7 * NH) * TILE);
    tma_load_3d(sT, &tmT, &bars->tma, 0, cidx * C, 0);
#pragma unroll
    for (int n = 0; n < NH; ++n) {
      tma_load_3d(sdUW + n * TILE, &tmdU, &bars->tma, n * 64, cidx * C, 0);
      tma_load_3d(sdUW + (NH + n) * TILE, &tmdW, &bars->tma, n * 64, cidx * C, 0);
      tma_load_3d(sU0 + n * TILE, &tmU0, &bars->tma, n * 64, cidx * C, 0);
      tma_load_3d(sW + n * TILE, &tmW, &bars->tma, n * 64, cidx * C, 0);
      tma_load_3d(sV + n * TILE, &tmV, &bars->tma, vcol + h * D + n * 64, row0, 0);
      tma_load_3d(sK + n * TILE, &tmK, &bars->tma, kcol + h * D + n * 64, row0, 0);
      tma_load_3d(sG + n * TILE, &tmG, &bars->tma, gcol + h * D + n * 64, row0, 0);
    }
  }
  bool ok = wait_inputs(bars);
  const Acc64 me;
  if (ok) {
    if (tid == 0) {
      tc_fence_after_sync();
      constexpr uint32_t id = make_idesc(64, 2 * D, 1, 1, 1, 1);  // T^T [dU | dW]: T read with its columns as M
      const uint32_t at = smem_u32(sT), ab = smem_u32(sdUW);
#pragma unroll
      for (int k = 0; k < 4; ++k) umma_bf16(tmem, desc_mn(at, k), desc_mn(ab, k), id, k > 0 ? 1u : 0u);
      umma_commit(&bars->mma[0]);
    }
    if (tid < C) dbs[tid] = 0.f;
    cumsum_d<D>(sG, bmat, logits != 0);
    ok = wait_mma(bars, 0);
    if (ok) {
      // warps 0-3 (chalf 0) own the dVb row, warps 4-7 (chalf 1) the dKb row of their token s = me.row
      const float bt = (me.active && beta != nullptr) ? beta[(long long)(row0 + me.row) * H + h] : 1.f;
      float part = 0.f;
#pragma unroll 1
      for (int c0 = 0; c0 < D; c0 += 32) {
        float v[32];
        load_acc_cols<32>(tmem, me.chalf * D + c0, me.quarter, v);
        if (me.active) {
          const int half = c0 >> 6, cin = c0 & 63;
          if (me.chalf == 0) {
            // dv = beta dVb, <dVb, V>
            float o[32];
#pragma unroll
            for (int c8 = 0; c8 < 4; ++c8) {
              float x[8];
              unpack8(*reinterpret_cast<const uint4*>(sV + half * TILE + sw_off(me.row, (cin >> 3) + c8)), x);
#pragma unroll
              for (int e = 0; e < 8; ++e) {
                part += v[c8 * 8 + e] * x[e];
                o[c8 * 8 + e] = bt * v[c8 * 8 + e];
              }
            }
            __nv_bfloat16* dst = dv + (long long)(row0 + me.row) * dv_ld + dvcol + h * D + c0;
#pragma unroll
            for (int c8 = 0; c8 < 4; ++c8) store8_bf16(dst + c8 * 8, o + c8 * 8);
            store_row_cols<32>(sdVb + half * TILE, me.row, cin, v, 1 << 30);
          } else {
            // dkr1 = beta e^{bp} dKb, <dKb, Kbar>
            float bp[32];
            if (me.row == 0) {
#pragma unroll
              for (int i = 0; i < 32; ++i) bp[i] = 0.f;
            } else {
              ld_row<32>(bmat + (me.row - 1) * BST + c0, bp);
            }
            float o[32];
#pragma unroll
            for (int c8 = 0; c8 < 4; ++c8) {
              float x[8];
              unpack8(*reinterpret_cast<const uint4*>(sK + half * TILE + sw_off(me.row, (cin >> 3) + c8)), x);
#pragma unroll
              for (int e = 0; e < 8; ++e) {
                const float ebp = __expf(bp[c8 * 8 + e]);
                part += v[c8 * 8 + e] * x[e] * ebp;
                o[c8 * 8 + e] = bt * ebp * v[c8 * 8 + e];
              }
            }
            float* dst = dkr1 + ((long long)cidx * C + me.row) * D + c0;
#pragma unroll
            for (int c4 = 0; c4 < 8; ++c4)
              *reinterpret_cast<float4*>(dst + c4 * 4) = make_float4(o[c4 * 4], o[c4 * 4 + 1], o[c4 * 4 + 2], o[c4 * 4 + 3]);
            store_row_cols<32>(sdKb + half * TILE, me.row, cin, v, 1 << 30);
          }
        }
      }
      if (me.active) atomicAdd(&dbs[me.row], part);
    }
  }
  ok = phase_sync(bars);
  if (ok) {
    if (tid == 0) {
      tc_fence_after_sync();
      constexpr uint32_t id = make_idesc(64, 64, 1, 1, 0, 0);
      const uint32_t av = smem_u32(sdVb), ak = smem_u32(sdKb), au0 = smem_u32(sU0), aw = smem_u32(sW);
#pragma unroll
      for (int n = 0; n < NH; ++n)
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          umma_bf16(tmem + 2 * D, desc_k(av + n * TILE, k), desc_k(au0 + n * TILE, k), id, (n > 0 || k > 0) ? 1u : 0u);
        }
#pragma unroll
      for (int n = 0; n < NH; ++n)
#pragma unroll
        for (int k = 0; k < 4; ++k) umma_bf16(tmem + 2 * D, desc_k(ak + n * TILE, k), desc_k(aw + n * TILE, k), id, 1u);
      umma_commit(&bars->mma[1]);
    }
    ok = wait_mma(bars, 1);
    if (ok) {
      float v[32];
      load_acc_cols<32>(tmem, 2 * D + me.chalf * 32, me.quarter, v);
      if (me.active) {
        const float bt = beta != nullptr ? beta[(long long)(row0 + me.row) * H + h] : 1.f;
        const float* lr = Lraw + ((long long)cidx * C + me.row) * C + me.chalf * 32;
        float part = 0.f, o[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const int s = me.chalf * 32 + i;
          const float dl = s < me.row ? -v[i] : 0.f;
          if (beta != nullptr) part += dl * lr[i];
          o[i] = bt * dl;
        }
        __nv_bfloat16* dst = dLraw + ((long long)cidx * C + me.row) * C + me.chalf * 32;
#pragma unroll
        for (int c8 = 0; c8 < 4; ++c8) store8_bf16(dst + c8 * 8, o + c8 * 8);
        atomicAdd(&dbs[me.row], part);
      }
    }
  }
  __syncthreads();
  if (ok && dbeta != nullptr && tid < C) dbeta[(long long)(row0 + tid) * H + h] = dbs[tid];
  cta_teardown(bars, tmem, Cfg::TMEM_COLS, status);
}

// ------------------------------------------------------------------------------------------------
// B3c: per chunk and per 64-wide slice of the key dimension. dA = mask(dO U^T) and dLraw (from B3b) are pushed
// through the score factorisation:
//   dq   = dq1  + sum_{j<=i} e^{b_t  - r_j} (dA_j    K~_j)[t]
//   dk_r = dkr1 + sum_{j<=i} e^{bp_t - r_j} (dLraw_j K~_j)[t]
//   dk_w = dkw1 + e^{r_i(s) - b_s} (dA^T Q~(i) + dLraw^T K^(i))[s]
// and dk = dk_w + dk_r;  gate terms E1 = q dq - k dk_w, E2 = k dk_r.
// ------------------------------------------------------------------------------------------------
struct B3cCfg {
  // Q K G | dO U (2 * NH) | dLraw dA | Q~(0..3) K~ K^(0..3)
  static constexpr int tiles(int NH) { return 3 + 2 * NH + 2 + 9; }
  static constexpr int smem(int NH) { return tiles(NH) * TILE + 4 * C * LP * 4 + 16 * 64 * 4 + 1024 + 256; }
};

template <int NH>
__global__ void __launch_bounds__(GDN_THREADS) gdn_bwd_scores_kernel(
    const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
    const __grid_constant__ CUtensorMap tmG, const __grid_constant__ CUtensorMap tmdO,
    const __grid_constant__ CUtensorMap tmU, const __grid_constant__ CUtensorMap tmdL, int qcol, int kcol, int gcol,
    int docol, const float* __restrict__ dq1, const float* __restrict__ dkw1, const float* __restrict__ dkr1,
    __nv_bfloat16* __restrict__ dq, long long dq_ld, int dqcol, __nv_bfloat16* __restrict__ dk, long long dk_ld,
    int dkcol, float* __restrict__ dgl_local, float* __restrict__ chunk_tot, float scale, int T, int H, int logits,
    int* status) {
  constexpr int D = NH * 64, DH = 64, BST = DH + 4;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = aligned_smem(smem_raw);
  uint8_t* sQ = smem;
  uint8_t* sK = sQ + TILE;
  uint8_t* sG = sK + TILE;
  uint8_t* sdO = sG + TILE;
  uint8_t* sU = sdO + NH * TILE;
  uint8_t* sdL = sU + NH * TILE;
  uint8_t* sdA = sdL + TILE;
  uint8_t* sA = sdA + TILE;        // Q~(0..3)
  uint8_t* sKt = sA + 4 * TILE;
  uint8_t* sKh = sKt + TILE;       // K^(0..3)
  float* bmat = reinterpret_cast<float*>(sKh + 4 * TILE);
  float* e1 = bmat + C * LP;       // q dq - k dk_w  (+ E2 before the suffix sums)
  float* e2 = e1 + C * LP;         // k dk_r
  float* dkr = e2 + C * LP;        // dk_r itself
  float* ftab = dkr + C * LP;
  GBars* bars = reinterpret_cast<GBars*>(ftab + 16 * 64);
  static_assert(BST == LP, "the 64-wide decay matrix uses the common 68-float pitch");
  const int tid = threadIdx.x;
  const int NT = T / C;
  const int dh = blockIdx.x % NH, cidx = blockIdx.x / NH;
  const int chunk = cidx % NT, bh = cidx / NT, h = bh % H, b = bh / H;
  const int row0 = b * T + chunk * C;
  const int dcol = h * D + dh * DH;  // first column of this slice inside a [rows, H * D] matrix

  cta_setup(bars, 3, 512);
  const uint32_t tmem = bars->tmem_slot;
  if (tid == 0) {
    mbar_expect_tx(&bars->tma, (4 + 2 * NH) * TILE);
    tma_load_3d(sQ, &tmQ, &bars->tma, qcol + dcol, row0, 0);
    tma_load_3d(sK, &tmK, &bars->tma, kcol + dcol, row0, 0);
    tma_load_3d(sG, &tmG, &bars->tma, gcol + dcol, row0, 0);
    tma_load_3d(sdL, &tmdL, &bars->tma, 0, cidx * C, 0);
#pragma unroll
    for (int n = 0; n < NH; ++n) {
      tma_load_3d(sdO + n * TILE, &tmdO, &bars->tma, docol + h * D + n * 64, row0, 0);
      tma_load_3d(sU + n * TILE, &tmU, &bars->tma, n * 64, cidx * C, 0);
    }
  }
  bool ok = wait_inputs(bars);
  const Acc64 me;
  uint8_t* const qj[4] = {sA, sA + TILE, sA + 2 * TILE, sA + 3 * TILE};
  uint8_t* const kj[4] = {sKh, sKh + TILE, sKh + 2 * TILE, sKh + 3 * TILE};
  if (ok) {
    if (tid == 0) {
      // dA = dO U^T needs no decay: start it right away
      tc_fence_after_sync();
      constexpr uint32_t id = make_idesc(64, 64, 1, 1, 0, 0);
      const uint32_t ado = smem_u32(sdO), au = smem_u32(sU);
#pragma unroll
      for (int n = 0; n < NH; ++n)
#pragma unroll
        for (int k = 0; k < 4; ++k)
          umma_bf16(tmem, desc_k(ado + n * TILE, k), desc_k(au + n * TILE, k), id, (n > 0 || k > 0) ? 1u : 0u);
      umma_commit(&bars->mma[0]);
    }
    cumsum_d<64>(sG, bmat, logits != 0);
    factor_tables_d<64>(bmat, ftab);
    build_row_operands<64, false>(sQ, qj, bmat, ftab);
    build_row_operands<64, true>(sK, kj, bmat, ftab);
    build_key_operand<64>(sK, sKt, bmat);
    ok = wait_mma(bars, 0);
    if (ok) {
      float v[32];
      load_acc_cols<32>(tmem, me.chalf * 32, me.quarter, v);
      if (me.active) {
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] *= scale;
        store_row_cols<32>(sdA, me.row, me.chalf * 32, v, me.row);
      }
    }
  }
  ok = phase_sync(bars);
  // e^{c_t - r_i} for this thread's row and its 32 columns: c = b (queries) and c = bp (keys in their row role)
  const int c0 = me.chalf * 32;
  const int irow = me.row >> 4;
  if (ok) {
    if (tid == 0) {
      tc_fence_after_sync();
      constexpr uint32_t id = make_idesc(64, 64, 1, 1, 0, 1);
      const uint32_t ada = smem_u32(sdA), adl = smem_u32(sdL), akt = smem_u32(sKt);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        umma_bf16(tmem + 64 * j, desc_k(ada, j), desc_mn(akt, j), id, 0u);        // dA_j K~_j
        umma_bf16(tmem + 256 + 64 * j, desc_k(adl, j), desc_mn(akt, j), id, 0u);  // dLraw_j K~_j
      }
      umma_commit(&bars->mma[1]);
    }
    float eb[32], ep[32];
    if (me.active) {
      float bt[32], bp[32], ri[32];
      ld_row<32>(bmat + me.row * BST + c0, bt);
      if (me.row == 0) {
#pragma unroll
        for (int i = 0; i < 32; ++i) bp[i] = 0.f;
      } else {
        ld_row<32>(bmat + (me.row - 1) * BST + c0, bp);
      }
      if (irow == 0) {
#pragma unroll
        for (int i = 0; i < 32; ++i) ri[i] = 0.f;
      } else {
        ld_row<32>(bmat + (16 * irow - 1) * BST + c0, ri);
      }
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        eb[i] = __expf(bt[i] - ri[i]);
        ep[i] = __expf(bp[i] - ri[i]);
      }
    }
    ok = wait_mma(bars, 1);
    if (ok) {
      float accq[32], accr[32];
#pragma unroll
      for (int i = 0; i < 32; ++i) accq[i] = accr[i] = 0.f;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float vq[32], vr[32];
        load_acc_cols<32>(tmem, 64 * j + c0, me.quarter, vq);        // warp-collective: every lane executes the loads
        load_acc_cols<32>(tmem, 256 + 64 * j + c0, me.quarter, vr);
        if (me.active && j <= irow) {
          float f[32];
          ld_row<32>(ftab + (irow * 4 + j) * 64 + c0, f);
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            accq[i] += vq[i] * f[i];
            accr[i] += vr[i] * f[i];
          }
        }
      }
      if (me.active) {
        const long long o = ((long long)cidx * C + me.row) * D + dh * DH + c0;
        float a1[32], a2[32];
        ld_row<32>(dq1 + o, a1);
        ld_row<32>(dkr1 + o, a2);
        float qv[32], kv[32];
#pragma unroll
        for (int c8 = 0; c8 < 4; ++c8) {
          float x[8];
          unpack8(*reinterpret_cast<const uint4*>(sQ + sw_off(me.row, c0 / 8 + c8)), x);
#pragma unroll
          for (int e = 0; e < 8; ++e) qv[c8 * 8 + e] = x[e];
          unpack8(*reinterpret_cast<const uint4*>(sK + sw_off(me.row, c0 / 8 + c8)), x);
#pragma unroll
          for (int e = 0; e < 8; ++e) kv[c8 * 8 + e] = x[e];
        }
        float dqv[32], dkrv[32], t1[32], t2[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          dqv[i] = a1[i] + eb[i] * accq[i];
          dkrv[i] = a2[i] + ep[i] * accr[i];
          t1[i] = qv[i] * dqv[i];
          t2[i] = kv[i] * dkrv[i];
        }
        __nv_bfloat16* dst = dq + (long long)(row0 + me.row) * dq_ld + dqcol + dcol + c0;
#pragma unroll
        for (int c8 = 0; c8 < 4; ++c8) store8_bf16(dst + c8 * 8, dqv + c8 * 8);
#pragma unroll
        for (int c4 = 0; c4 < 8; ++c4) {
          *reinterpret_cast<float4*>(e1 + me.row * LP + c0 + c4 * 4) = make_float4(t1[c4 * 4], t1[c4 * 4 + 1], t1[c4 * 4 + 2], t1[c4 * 4 + 3]);
          *reinterpret_cast<float4*>(e2 + me.row * LP + c0 + c4 * 4) = make_float4(t2[c4 * 4], t2[c4 * 4 + 1], t2[c4 * 4 + 2], t2[c4 * 4 + 3]);
          *reinterpret_cast<float4*>(dkr + me.row * LP + c0 + c4 * 4) =
              make_float4(dkrv[c4 * 4], dkrv[c4 * 4 + 1], dkrv[c4 * 4 + 2], dkrv[c4 * 4 + 3]);
        }
      }
    }
  }
  ok = phase_sync(bars);
  if (ok) {
    if (tid == 0) {
      tc_fence_after_sync();
      constexpr uint32_t id = make_idesc(64, 64, 1, 1, 1, 1);
      const uint32_t ada = smem_u32(sdA), adl = smem_u32(sdL);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          umma_bf16(tmem + 64 * j, desc_mn(ada, k), desc_mn(smem_u32(qj[j]), k), id, k > 0 ? 1u : 0u);        // dA^T Q~(j)
          umma_bf16(tmem + 256 + 64 * j, desc_mn(adl, k), desc_mn(smem_u32(kj[j]), k), id, k > 0 ? 1u : 0u);  // dLraw^T K^(j)
        }
      }
      umma_commit(&bars->mma[2]);
    }
    // e^{r_i - b_s} for this thread's row
    float ek[32];
    if (me.active) {
      float bt[32], ri[32];
      ld_row<32>(bmat + me.row * BST + c0, bt);
      if (irow == 0) {
#pragma unroll
        for (int i = 0; i < 32; ++i) ri[i] = 0.f;
      } else {
        ld_row<32>(bmat + (16 * irow - 1) * BST + c0, ri);
      }
#pragma unroll
      for (int i = 0; i < 32; ++i) ek[i] = __expf(ri[i] - bt[i]);
    }
    ok = wait_mma(bars, 2);
    if (ok) {
      // rows of sub-chunk i live in accumulator i (= this warp's lane quarter)
      float va[32], vl[32];
      load_acc_cols<32>(tmem, 64 * me.quarter + c0, me.quarter, va);
      load_acc_cols<32>(tmem, 256 + 64 * me.quarter + c0, me.quarter, vl);
      if (me.active) {
        const long long o = ((long long)cidx * C + me.row) * D + dh * DH + c0;
        float a1[32], r[32], t1[32], kv[32], dkv[32];
        ld_row<32>(dkw1 + o, a1);
        ld_row<32>(dkr + me.row * LP + c0, r);
        ld_row<32>(e1 + me.row * LP + c0, t1);
#pragma unroll
        for (int c8 = 0; c8 < 4; ++c8) {
          float x[8];
          unpack8(*reinterpret_cast<const uint4*>(sK + sw_off(me.row, c0 / 8 + c8)), x);
#pragma unroll
          for (int e = 0; e < 8; ++e) kv[c8 * 8 + e] = x[e];
        }
        float t2[32];
        ld_row<32>(e2 + me.row * LP + c0, t2);
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const float dkw = a1[i] + ek[i] * (va[i] + vl[i]);
          dkv[i] = dkw + r[i];
          t1[i] = t1[i] - kv[i] * dkw + t2[i];  // E1 + E2: what the suffix sums run over
        }
        __nv_bfloat16* dst = dk + (long long)(row0 + me.row) * dk_ld + dkcol + dcol + c0;
#pragma unroll
        for (int c8 = 0; c8 < 4; ++c8) store8_bf16(dst + c8 * 8, dkv + c8 * 8);
#pragma unroll
        for (int c4 = 0; c4 < 8; ++c4)
          *reinterpret_cast<float4*>(e1 + me.row * LP + c0 + c4 * 4) = make_float4(t1[c4 * 4], t1[c4 * 4 + 1], t1[c4 * 4 + 2], t1[c4 * 4 + 3]);
      }
    }
  }
  __syncthreads();
  ok = bars->failed == 0;
  if (ok) {
    // dgl_local[t] = sum_{tau >= t} (E1 + E2)[tau] - E2[t] inside the chunk; chunk_tot = sum over the chunk
    constexpr int NPARTS = GDN_THREADS / 64, PR = C / NPARTS;
    const int d = tid & 63, part = tid >> 6;
    float acc = 0.f;
    for (int t = PR * part + PR - 1; t >= PR * part; --t) {
      acc += e1[t * LP + d];
      e1[t * LP + d] = acc;
    }
    __syncthreads();
    float base = 0.f;
    for (int pp = part + 1; pp < NPARTS; ++pp) base += e1[(PR * pp) * LP + d];
    float* dst = dgl_local + (long long)row0 * (H * D) + dcol + d;
    for (int t = PR * part; t < PR * part + PR; ++t) dst[(long long)t * (H * D)] = e1[t * LP + d] + base - e2[t * LP + d];
    if (part == 0) chunk_tot[(((long long)bh * NH + dh) * NT + chunk) * 64 + d] = e1[d] + base;
  }
  cta_teardown(bars, tmem, 512, status);
}

// ------------------------------------------------------------------------------------------------ host side
CUtensorMap user_map(const GlaMat& m, long long rows) {
  return make_tmap_3d(m.ptr, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)m.ld, (uint64_t)rows, 1, (uint64_t)m.ld * 2ull,
                      (uint64_t)m.ld * 2ull * (uint64_t)rows, 64, 64);
}
// [rows, width] contiguous bf16 scratch; box 64 columns x box_rows rows
CUtensorMap scratch_map(const void* p, long long rows, int width, int box_rows) {
  return make_tmap_3d(p, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)width, (uint64_t)rows, 1, (uint64_t)width * 2ull,
                      (uint64_t)width * 2ull * (uint64_t)rows, 64, (uint32_t)box_rows);
}

void check(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) throw std::runtime_error(std::string(what) + " launch failed: " + cudaGetErrorString(e));
}
template <typename K>
void smem_attr(K kern, int bytes) {
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
  if (e != cudaSuccess) throw std::runtime_error(std::string("cannot set shared memory size: ") + cudaGetErrorString(e));
}
void check_dims(const GdnDims& d) {
  if (d.T <= 0 || d.T % C != 0) throw std::runtime_error("gdn chunk kernels need T to be a positive multiple of 64");
  if (d.D != 64 && d.D != 128) throw std::runtime_error("gdn chunk kernels support head_dim 64 and 128");
}

template <int D>
void fwd_impl(const GlaMat& Q, const GlaMat& K, const GlaMat& V, const GlaMat& G, const float* beta, const float* init,
              const GlaMat& O, const GdnScratch& w, const GdnDims& d, float scale, int* status, cudaStream_t s) {
  const long long rows = (long long)d.B * d.T;
  const int NT = d.T / C, BH = d.B * d.H, nchunks = BH * NT;
  CUtensorMap tk = user_map(K, rows), tv = user_map(V, rows), tg = user_map(G, rows), tq = user_map(Q, rows);
  {
    auto kern = gdn_wy_kernel<D>;
    static PerDeviceOnce once;
    if (once.first_use()) smem_attr(kern, WyCfg<D>::SMEM);
    kern<<<nchunks, GDN_THREADS, WyCfg<D>::SMEM, s>>>(tk, tv, tg, K.col0, V.col0, G.col0, beta, w.U0, w.W, w.Tm, w.Kend,
                                                      w.decay, w.Lraw, d.T, d.H, d.gate_logits ? 1 : 0, status);
    check("gdn_wy");
  }
  {
    auto kern = gdn_state_kernel<D, false>;
    static PerDeviceOnce once;
    if (once.first_use()) smem_attr(kern, StateCfg<D>::SMEM);
    kern<<<BH * (D / DVS), GDN_THREADS, StateCfg<D>::SMEM, s>>>(w.W, w.Kend, w.U0, nullptr, w.decay, init, w.U, w.states,
                                                               w.fin, NT);
    check("gdn_state_fwd");
  }
  {
    auto kern = gdn_scores_kernel<D, false>;
    static PerDeviceOnce once;
    if (once.first_use()) smem_attr(kern, OutCfg<D, false>::SMEM);
    CUtensorMap tu = scratch_map(w.U, (long long)nchunks * C, D, 64), ts = scratch_map(w.states, (long long)nchunks * D, D, 64);
    kern<<<nchunks, GDN_THREADS, OutCfg<D, false>::SMEM, s>>>(
        tq, tk, tg, tu, ts, Q.col0, K.col0, G.col0, 0, 1, reinterpret_cast<__nv_bfloat16*>(const_cast<void*>(O.ptr)), O.ld,
        O.col0, scale, nullptr, nullptr, d.T, d.H, d.gate_logits ? 1 : 0, status);
    check("gdn_out");
  }
}

template <int D>
void bwd_impl(const GlaMat& Q, const GlaMat& K, const GlaMat& V, const GlaMat& G, const GlaMat& dO, const float* beta,
              const float* dfin, const GlaMat& dQ, const GlaMat& dK, const GlaMat& dV, const GdnScratch& w,
              const GdnBwdScratch& x, const GdnDims& d, float scale, int* status, cudaStream_t s) {
  constexpr int NH = D / 64;
  const long long rows = (long long)d.B * d.T;
  const int NT = d.T / C, BH = d.B * d.H, nchunks = BH * NT;
  const long long crow = (long long)nchunks * C, srow = (long long)nchunks * D;
  CUtensorMap tq = user_map(Q, rows), tk = user_map(K, rows), tv = user_map(V, rows), tg = user_map(G, rows),
              tdo = user_map(dO, rows);
  CUtensorMap tu = scratch_map(w.U, crow, D, 64), tu0 = scratch_map(w.U0, crow, D, 64), tw = scratch_map(w.W, crow, D, 64),
              tt = scratch_map(w.Tm, crow, C, 64), tdu = scratch_map(x.dU, crow, D, 64),
              tdw = scratch_map(x.dW, crow, D, 64), tdl = scratch_map(x.dLraw, crow, C, 64);
  // states as K-major B operands: boxes of D rows x 64 columns
  CUtensorMap tsk = scratch_map(w.states, srow, D, D), tdsk = scratch_map(x.dSend, srow, D, D);
  const int lg = d.gate_logits ? 1 : 0;
  {
    auto kern = gdn_scores_kernel<D, true>;
    static PerDeviceOnce once;
    if (once.first_use()) smem_attr(kern, OutCfg<D, true>::SMEM);
    kern<<<nchunks, GDN_THREADS, OutCfg<D, true>::SMEM, s>>>(tq, tk, tg, tdo, tdo, Q.col0, K.col0, G.col0, dO.col0, 0,
                                                             nullptr, 0, 0, scale, x.G1, x.H1, d.T, d.H, lg, status);
    check("gdn_bwd_local");
  }
  {
    auto kern = gdn_state_kernel<D, true>;
    static PerDeviceOnce once;
    if (once.first_use()) smem_attr(kern, StateCfg<D>::SMEM);
    kern<<<BH * (D / DVS), GDN_THREADS, StateCfg<D>::SMEM, s>>>(w.Kend, w.W, x.G1, x.H1, w.decay, dfin, x.dU, x.dSend,
                                                               x.dS0, NT);
    check("gdn_state_bwd");
  }
  {
    auto kern = gdn_bwd_state_terms_kernel<D>;
    static PerDeviceOnce once;
    if (once.first_use()) smem_attr(kern, B3aCfg<D>::SMEM);
    kern<<<nchunks, GDN_THREADS, B3aCfg<D>::SMEM, s>>>(tdo, tu, tdu, tg, tsk, tdsk, dO.col0, G.col0, x.dq1, x.dkw1, x.dW,
                                                       scale, d.T, d.H, lg, status);
    check("gdn_bwd_state_terms");
  }
  {
    auto kern = gdn_bwd_wy_kernel<D>;
    static PerDeviceOnce once;
    if (once.first_use()) smem_attr(kern, B3bCfg<D>::SMEM);
    kern<<<nchunks, GDN_THREADS, B3bCfg<D>::SMEM, s>>>(
        tt, tdu, tdw, tu0, tw, tv, tk, tg, V.col0, K.col0, G.col0, beta, w.Lraw,
        reinterpret_cast<__nv_bfloat16*>(const_cast<void*>(dV.ptr)), dV.ld, dV.col0, x.dkr1, x.dbeta, x.dLraw, d.T, d.H, lg,
        status);
    check("gdn_bwd_wy");
  }
  {
    auto kern = gdn_bwd_scores_kernel<NH>;
    static PerDeviceOnce once;
    if (once.first_use()) smem_attr(kern, B3cCfg::smem(NH));
    kern<<<nchunks * NH, GDN_THREADS, B3cCfg::smem(NH), s>>>(
        tq, tk, tg, tdo, tu, tdl, Q.col0, K.col0, G.col0, dO.col0, x.dq1, x.dkw1, x.dkr1,
        reinterpret_cast<__nv_bfloat16*>(const_cast<void*>(dQ.ptr)), dQ.ld, dQ.col0,
        reinterpret_cast<__nv_bfloat16*>(const_cast<void*>(dK.ptr)), dK.ld, dK.col0, x.dgl_local, x.chunk_tot, scale, d.T,
        d.H, lg, status);
    check("gdn_bwd_scores");
  }
}

}  // namespace

void launch_gdn_chunk_fwd(const GlaMat& Q, const GlaMat& K, const GlaMat& V, const GlaMat& G, const float* beta,
                          const float* init, const GlaMat& O, const GdnScratch& w, const GdnDims& d, float scale,
                          int* status, cudaStream_t s) {
  check_dims(d);
  if (d.D == 128) fwd_impl<128>(Q, K, V, G, beta, init, O, w, d, scale, status, s);
  else fwd_impl<64>(Q, K, V, G, beta, init, O, w, d, scale, status, s);
}

void launch_gdn_chunk_bwd(const GlaMat& Q, const GlaMat& K, const GlaMat& V, const GlaMat& G, const GlaMat& dO,
                          const float* beta, const float* dfin, const GlaMat& dQ, const GlaMat& dK, const GlaMat& dV,
                          const GdnScratch& w, const GdnBwdScratch& x, const GdnDims& d, float scale, int* status,
                          cudaStream_t s) {
  check_dims(d);
  if (d.D == 128) bwd_impl<128>(Q, K, V, G, dO, beta, dfin, dQ, dK, dV, w, x, d, scale, status, s);
  else bwd_impl<64>(Q, K, V, G, dO, beta, dfin, dQ, dK, dV, w, x, d, scale, status, s);
}

}  // namespace tb
