// Chunked gated linear attention on tcgen05 tensor cores (head_dim 64, chunk 64).
//
// Recurrence (per batch, head): S_t = diag(exp(g_t)) S_{t-1} + k_t v_t^T, o_t = q_t^T S_t, with g <= 0 a
// per-key-dimension log decay. With b = cumsum(g) inside a chunk:
//   o_t = (q_t * e^{b_t})^T S_0 + sum_{s<=t} [ sum_d q_td k_sd e^{b_td - b_sd} ] v_s
//   S_C = diag(e^{b_C}) S_0 + sum_s (k_s * e^{b_C - b_s}) v_s^T
// The score term has a per-dimension weight, so it only factors into a matrix product around a reference
// row. Keys are referenced per 16-token sub-chunk j to r_j = b at the row before the sub-chunk:
//   K~[s]    = k_s * e^{r_j - b_s}      (s in sub-chunk j; exponent in [0, 80])
//   Q~(j)[t] = q_t * e^{b_t - r_j}      (t >= 16 j; exponent <= 0)
// and P[:, 16j:16j+16] = Q~(j) K~_j^T is one MMA (M=64, N=16, K=64) per sub-chunk.
//
// Replaces the reference's Triton chunk kernel and scan (triune/kernels/fast_gla.py:33-380, 569-689).
#include "gla.cuh"

#include <cuda.h>

#include <stdexcept>
#include <string>

#include "../common/per_device.h"
#include "../common/ptx.cuh"
#include "../common/tma_desc.h"
#include "gla_tiles.cuh"

namespace tb {

namespace {

constexpr int C = 64;             // chunk length (tokens)
constexpr int D = 64;             // head dim (keys and values)
constexpr int GLA_THREADS = 128;
// Row pitch (floats) of the fp32 scratch matrices in shared memory (cumulative log decay, gate-gradient terms).
// Rows stay 16-byte aligned and consecutive rows start one 16-byte bank group apart, so float4 accesses with one
// row per lane are conflict-free (a pitch of 64 puts every row on the same banks: 16-way conflicts).
constexpr int BST = 68;
constexpr int BMAT_BYTES = C * BST * 4;

// Fills bmat[t][d] (fp32, 64x64) with the inclusive cumulative log decay of the gate tile, for a block of NTHR =
// 64 * P threads (P in {2,4,8}). Thread (part, d) scans its 64/P tokens of column d in registers (independent
// shared-memory reads, no round trip per token), publishes the part's total, and after ONE barrier adds the totals of
// the earlier parts while writing its rows. (The previous form scanned in place in shared memory: 64/P dependent
// load-add-store round trips twice, up to 2.5 K clocks in the 128-thread kernel.)
template <int NTHR>
__device__ __forceinline__ void build_cumsum(const uint8_t* g_tile, float* bmat, bool logits) {
  constexpr int PARTS = NTHR / 64, LEN = C / PARTS;
  __shared__ float totals[PARTS * 64];
  const int tid = threadIdx.x, d = tid & 63, part = tid >> 6;
  float c[LEN];
  float run = 0.f;
#pragma unroll
  for (int i = 0; i < LEN; ++i) {
    const int r = part * LEN + i;
    const __nv_bfloat16 x = *reinterpret_cast<const __nv_bfloat16*>(g_tile + sw_off(r, d >> 3) + (d & 7) * 2);
    run += log_decay(__bfloat162float(x), logits);
    c[i] = run;
  }
  totals[part * 64 + d] = run;
  __syncthreads();
  float base = 0.f;
  for (int pp = 0; pp < part; ++pp) base += totals[pp * 64 + d];
#pragma unroll
  for (int i = 0; i < LEN; ++i) bmat[(part * LEN + i) * BST + d] = base + c[i];
  __syncthreads();
}

struct Bars {
  uint64_t tma;
  uint64_t mma[3];
  uint32_t tmem_slot;
  int failed;
};

// ------------------------------------------------------------------------------------------------
// Phase 1 (and its backward twin): out[bh, c] = (X * e^{w})^T Y  (64x64 fp32), w = b_last - b or b.
// ------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(GLA_THREADS) gla_chunk_outer_kernel(const __grid_constant__ CUtensorMap tmX,
                                                                      const __grid_constant__ CUtensorMap tmY,
                                                                      const __grid_constant__ CUtensorMap tmG,
                                                                      int xcol, int ycol, int gcol, int mode,
                                                                      float* __restrict__ out_kv,
                                                                      float* __restrict__ out_decay, int T, int H,
                                                                      int logits, int* status) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  uint8_t* smem = smem_raw + (((raw + 1023u) & ~1023u) - raw);
  uint8_t* sX = smem;
  uint8_t* sY = smem + TILE;
  uint8_t* sG = smem + 2 * TILE;
  float* bmat = reinterpret_cast<float*>(smem + 3 * TILE);
  Bars* bars = reinterpret_cast<Bars*>(smem + 3 * TILE + BMAT_BYTES);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int NT = T / C;
  const int chunk = blockIdx.x % NT, bh = blockIdx.x / NT, h = bh % H, b = bh / H;
  const int row0 = b * T + chunk * C;

  if (tid == 0) {
    mbar_init(&bars->tma, 1);
    mbar_init(&bars->mma[0], 1);
    bars->failed = 0;
    mbar_fence_init();
  }
  if (warp == 0) {
    tmem_alloc(&bars->tmem_slot, 64);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = bars->tmem_slot;
  if (tid == 0) {
    mbar_expect_tx(&bars->tma, 3 * TILE);
    tma_load_3d(sX, &tmX, &bars->tma, xcol + h * D, row0, 0);
    tma_load_3d(sY, &tmY, &bars->tma, ycol + h * D, row0, 0);
    tma_load_3d(sG, &tmG, &bars->tma, gcol + h * D, row0, 0);
  }
  bool ok = mbar_wait(&bars->tma, 0);
  if (!ok) bars->failed = ST_TIMEOUT_FULL;
  __syncthreads();
  ok = bars->failed == 0;
  if (ok) {
    build_cumsum<GLA_THREADS>(sG, bmat, logits != 0);
    for (int idx = tid; idx < 512; idx += blockDim.x) {
      const int row = idx >> 3, ch = idx & 7;
      uint4* px = reinterpret_cast<uint4*>(sX + sw_off(row, ch));
      float f[8], bt[8], bl[8];
      unpack8(*px, f);
      ld8(bmat + row * BST + ch * 8, bt);
      ld8(bmat + 63 * BST + ch * 8, bl);
#pragma unroll
      for (int i = 0; i < 8; ++i) f[i] *= __expf(mode == 0 ? (bl[i] - bt[i]) : bt[i]);
      *px = pack8(f);
    }
    fence_proxy_async_smem();
    __syncthreads();
    if (tid == 0) {
      tc_fence_after_sync();
      constexpr uint32_t idesc = make_idesc(64, 64, 1, 1, 1, 1);
      const uint32_t ax = smem_u32(sX), ay = smem_u32(sY);
#pragma unroll
      for (int k = 0; k < 4; ++k) umma_bf16(tmem, desc_mn(ax, k), desc_mn(ay, k), idesc, k > 0);
      umma_commit(&bars->mma[0]);
    }
    ok = mbar_wait(&bars->mma[0], 0);
    ok = __all_sync(0xffffffffu, ok);
    if (ok) {
      tc_fence_after_sync();
      float* dst = out_kv + ((long long)blockIdx.x * D + (warp * 16 + (lane & 15))) * D;
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(tmem + ((uint32_t)(warp * 32) << 16) + half * 32, r);
        tmem_ld_wait();
        if (lane < 16) {
#pragma unroll
          for (int i = 0; i < 32; i += 4)
            *reinterpret_cast<float4*>(dst + half * 32 + i) =
                make_float4(__uint_as_float(r[i]), __uint_as_float(r[i + 1]), __uint_as_float(r[i + 2]),
                            __uint_as_float(r[i + 3]));
        }
      }
      if (mode == 0 && out_decay != nullptr && tid < D) out_decay[(long long)blockIdx.x * D + tid] = __expf(bmat[63 * BST + tid]);
    } else if (lane == 0) {
      bars->failed = ST_TIMEOUT_TMEM;
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (bars->failed != 0 && tid == 0 && status != nullptr) atomicCAS(status, 0, bars->failed);
  if (warp == 0) {
    tc_fence_after_sync();
    tmem_dealloc(tmem, 64);
  }
}

// ------------------------------------------------------------------------------------------------
// Phase 2: inter-chunk scan, one thread per state element, sequential over chunks.
// ------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) gla_scan_kernel(const float* __restrict__ kv, const float* __restrict__ decay,
                                                       const float* __restrict__ init,
                                                       __nv_bfloat16* __restrict__ states,
                                                       float* __restrict__ final_state, int NT, int reverse) {
  const int bh = blockIdx.x / 16;
  const int e = (blockIdx.x % 16) * 256 + threadIdx.x;  // element of the 64x64 state
  const int dk = e >> 6;
  float s = init ? init[(long long)bh * 4096 + e] : 0.f;
  for (int i = 0; i < NT; ++i) {
    const int c = reverse ? NT - 1 - i : i;
    const long long blk = (long long)bh * NT + c;
    states[blk * 4096 + e] = __float2bfloat16(s);
    s = decay[blk * 64 + dk] * s + kv[blk * 4096 + e];
  }
  if (final_state) final_state[(long long)bh * 4096 + e] = s;
}

// ------------------------------------------------------------------------------------------------
// Shared operand construction for phase 3 (forward) and the main backward kernel.
//   sQ -> sA[0..3]: Q~(j)[t] = q_t e^{b_t - r_j} for t >= 16 j (zero rows above), r_0 = 0, r_j = b[16j-1]
//   sK -> sKt:      K~[s]    = k_s e^{r_j(s) - b_s}
// ------------------------------------------------------------------------------------------------
// Factor tables of a chunk. With r_0 = 0 and r_j = b[16j-1] (the cumulative log decay just before sub-chunk j) and
// b_C = b[63]:
//   ftab[i][j][d] = e^{r_i - r_j}  for j <= i (<= 1; zero elsewhere)      gl[i][d] = e^{b_C - r_i}  (<= 1)
// Every exponential of the form e^{b_t - r_j} then costs one multiply on top of e^{b_t - r_i} (i = sub-chunk of t),
// which a thread computes once per element: the special-function unit was a quarter of the backward kernel's time.
constexpr int FTAB_FLOATS = 4 * 4 * D;
constexpr int GL_FLOATS = 4 * D;

__device__ __forceinline__ void build_factor_tables(const float* bmat, float* ftab, float* gl) {
  for (int idx = threadIdx.x; idx < FTAB_FLOATS; idx += blockDim.x) {
    const int i = idx >> 8, j = (idx >> 6) & 3, d = idx & 63;
    float f = 0.f;
    if (j <= i) {
      const float ri = i == 0 ? 0.f : bmat[(16 * i - 1) * BST + d];
      const float rj = j == 0 ? 0.f : bmat[(16 * j - 1) * BST + d];
      f = j == i ? 1.f : __expf(ri - rj);
    }
    ftab[idx] = f;
  }
  if (gl != nullptr) {
    for (int idx = threadIdx.x; idx < GL_FLOATS; idx += blockDim.x) {
      const int i = idx >> 6, d = idx & 63;
      const float ri = i == 0 ? 0.f : bmat[(16 * i - 1) * BST + d];
      gl[idx] = __expf(bmat[63 * BST + d] - ri);
    }
  }
  __syncthreads();
}

__device__ __forceinline__ void build_score_operands(const uint8_t* sQ, const uint8_t* sK, uint8_t* sA, uint8_t* sKt,
                                                     uint8_t* sKe, const float* bmat, const float* ftab,
                                                     const float* gl) {
  for (int idx = threadIdx.x; idx < 512; idx += blockDim.x) {
    const int row = idx >> 3, ch = idx & 7;
    const uint32_t off = sw_off(row, ch);
    float q[8], k[8], bt[8], rj[8];
    unpack8(*reinterpret_cast<const uint4*>(sQ + off), q);
    unpack8(*reinterpret_cast<const uint4*>(sK + off), k);
    ld8(bmat + row * BST + ch * 8, bt);
    const int jrow = row >> 4;
    if (jrow == 0) {
#pragma unroll
      for (int i = 0; i < 8; ++i) rj[i] = 0.f;
    } else {
      ld8(bmat + (16 * jrow - 1) * BST + ch * 8, rj);
    }
    float qe[8], o[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) qe[i] = q[i] * __expf(bt[i] - rj[i]);  // q_t e^{b_t - r_jrow}
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      if (j < jrow) {
        float f[8];
        ld8(ftab + (jrow * 4 + j) * D + ch * 8, f);
#pragma unroll
        for (int i = 0; i < 8; ++i) o[i] = qe[i] * f[i];
      } else if (j == jrow) {
#pragma unroll
        for (int i = 0; i < 8; ++i) o[i] = qe[i];
      } else {
#pragma unroll
        for (int i = 0; i < 8; ++i) o[i] = 0.f;
      }
      *reinterpret_cast<uint4*>(sA + j * TILE + off) = pack8(o);
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) o[i] = k[i] * __expf(rj[i] - bt[i]);  // K~: k_s e^{r_j(s) - b_s}
    *reinterpret_cast<uint4*>(sKt + off) = pack8(o);
    if (sKe != nullptr) {  // K_end[s] = k_s e^{b_C - b_s} = K~[s] e^{b_C - r_j(s)}
      float g8[8];
      ld8(gl + jrow * D + ch * 8, g8);
#pragma unroll
      for (int i = 0; i < 8; ++i) o[i] *= g8[i];
      *reinterpret_cast<uint4*>(sKe + off) = pack8(o);
    }
  }
}

// Issue the score MMAs P[:, 16j:16j+16] = Q~(j) K~_j^T into TMEM columns [p_col, p_col+64).
__device__ __forceinline__ void issue_score_mmas(uint32_t tmem, uint32_t p_col, uint32_t a_addr, uint32_t kt_addr) {
  constexpr uint32_t idesc = make_idesc(64, 16, 1, 1, 0, 0);
#pragma unroll
  for (int j = 0; j < 4; ++j) {
#pragma unroll
    for (int k = 0; k < 4; ++k)
      umma_bf16(tmem + p_col + 16 * j, desc_k(a_addr + j * TILE, k), desc_k(kt_addr + j * 2048, k), idesc, k > 0);
  }
}

// ------------------------------------------------------------------------------------------------
// Phase 3 forward: o = Q~(0) S_c + mask(P) V
// ------------------------------------------------------------------------------------------------
constexpr int FWD_SMEM = 5 * TILE + BMAT_BYTES + FTAB_FLOATS * 4 + 4 * TILE + TILE + TILE + 1024 + 256;

constexpr int FWD_THREADS = 256;

__global__ void __launch_bounds__(FWD_THREADS) gla_fwd_out_kernel(const __grid_constant__ CUtensorMap tmQ,
                                                                  const __grid_constant__ CUtensorMap tmK,
                                                                  const __grid_constant__ CUtensorMap tmV,
                                                                  const __grid_constant__ CUtensorMap tmG,
                                                                  const __grid_constant__ CUtensorMap tmS, int qcol,
                                                                  int kcol, int vcol, int gcol,
                                                                  __nv_bfloat16* __restrict__ out, long long out_ld,
                                                                  int ocol, int T, int H, int logits, int* status) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  uint8_t* smem = smem_raw + (((raw + 1023u) & ~1023u) - raw);
  uint8_t* sQ = smem;
  uint8_t* sK = smem + TILE;
  uint8_t* sV = smem + 2 * TILE;
  uint8_t* sG = smem + 3 * TILE;
  uint8_t* sS = smem + 4 * TILE;
  uint8_t* sA = smem + 5 * TILE;       // 4 tiles
  uint8_t* sKt = smem + 9 * TILE;
  uint8_t* sP = smem + 10 * TILE;
  float* bmat = reinterpret_cast<float*>(smem + 11 * TILE);
  float* ftab = bmat + C * BST;
  Bars* bars = reinterpret_cast<Bars*>(smem + 11 * TILE + BMAT_BYTES + FTAB_FLOATS * 4);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int NT = T / C;
  const int chunk = blockIdx.x % NT, bh = blockIdx.x / NT, h = bh % H, b = bh / H;
  const int row0 = b * T + chunk * C;

  if (tid == 0) {
    mbar_init(&bars->tma, 1);
    mbar_init(&bars->mma[0], 1);
    mbar_init(&bars->mma[1], 1);
    bars->failed = 0;
    mbar_fence_init();
  }
  if (warp == 0) {
    tmem_alloc(&bars->tmem_slot, 128);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = bars->tmem_slot;
  if (tid == 0) {
    mbar_expect_tx(&bars->tma, 5 * TILE);
    tma_load_3d(sQ, &tmQ, &bars->tma, qcol + h * D, row0, 0);
    tma_load_3d(sK, &tmK, &bars->tma, kcol + h * D, row0, 0);
    tma_load_3d(sV, &tmV, &bars->tma, vcol + h * D, row0, 0);
    tma_load_3d(sG, &tmG, &bars->tma, gcol + h * D, row0, 0);
    tma_load_3d(sS, &tmS, &bars->tma, 0, blockIdx.x * D, 0);
  }
  bool ok = mbar_wait(&bars->tma, 0);
  if (!ok) bars->failed = ST_TIMEOUT_FULL;
  __syncthreads();
  ok = bars->failed == 0;
  // eight warps: TMEM lane quarter (warp & 3) x 32-column half (warp >> 2) of every 64-column accumulator
  const int quarter = warp & 3, c0 = (warp >> 2) * 32;
  const int row = quarter * 16 + (lane & 15);
  if (ok) {
    build_cumsum<FWD_THREADS>(sG, bmat, logits != 0);
    build_factor_tables(bmat, ftab, nullptr);
    build_score_operands(sQ, sK, sA, sKt, nullptr, bmat, ftab, nullptr);
    fence_proxy_async_smem();
    __syncthreads();
    if (tid == 0) {
      tc_fence_after_sync();
      issue_score_mmas(tmem, 0, smem_u32(sA), smem_u32(sKt));
      constexpr uint32_t id_qs = make_idesc(64, 64, 1, 1, 0, 1);
      const uint32_t a0 = smem_u32(sA), ss = smem_u32(sS);
#pragma unroll
      for (int k = 0; k < 4; ++k) umma_bf16(tmem + 64, desc_k(a0, k), desc_mn(ss, k), id_qs, k > 0);
      umma_commit(&bars->mma[0]);
    }
    ok = __all_sync(0xffffffffu, mbar_wait(&bars->mma[0], 0));
    if (ok) {
      tc_fence_after_sync();
      float v[32];
      load_acc_cols<32>(tmem, c0, quarter, v);
      if (lane < 16) store_row_cols<32>(sP, row, c0, v, row);
      fence_proxy_async_smem();
      tc_fence_before_sync();
    } else if (lane == 0) {
      bars->failed = ST_TIMEOUT_TMEM;
    }
    __syncthreads();
    ok = bars->failed == 0;
    if (ok) {
      if (tid == 0) {
        tc_fence_after_sync();
        constexpr uint32_t id_pv = make_idesc(64, 64, 1, 1, 0, 1);
        const uint32_t ap = smem_u32(sP), av = smem_u32(sV);
#pragma unroll
        for (int k = 0; k < 4; ++k) umma_bf16(tmem + 64, desc_k(ap, k), desc_mn(av, k), id_pv, 1u);
        umma_commit(&bars->mma[1]);
      }
      ok = __all_sync(0xffffffffu, mbar_wait(&bars->mma[1], 0));
      if (ok) {
        tc_fence_after_sync();
        float v[32];
        load_acc_cols<32>(tmem, 64 + c0, quarter, v);
        if (lane < 16) {
          __nv_bfloat16* dst = out + (long long)(row0 + row) * out_ld + ocol + h * D + c0;
#pragma unroll
          for (int ch = 0; ch < 4; ++ch) {
            float o[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) o[i] = v[ch * 8 + i];
            *reinterpret_cast<uint4*>(dst + ch * 8) = pack8(o);
          }
        }
      } else if (lane == 0) {
        bars->failed = ST_TIMEOUT_TMEM;
      }
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (bars->failed != 0 && tid == 0 && status != nullptr) atomicCAS(status, 0, bars->failed);
  if (warp == 0) {
    tc_fence_after_sync();
    tmem_dealloc(tmem, 128);
  }
}

// ------------------------------------------------------------------------------------------------
// Main backward kernel (per chunk): dq, dk, dv and the in-chunk part of the gate gradient.
//   dP = mask(dO V^T)
//   dv = P^T dO + K_end dS_end          K_end[s] = k_s e^{b_C - b_s}
//   dq = e^{b_t} (dO S_c^T) + sum_j e^{b_t - r_j} (dP_j K~_j)
//   dk = e^{b_C - b_s} (V dS_end^T) + e^{r_j(s) - b_s} (dP^T Q~(j(s)))
//   dg_t = sum_{tau >= t} (q dq - k dk)   (suffix over the whole sequence; chunk suffix added by dg_finalize)
// ------------------------------------------------------------------------------------------------
constexpr int BWD_TILES = 2 * 7 + 4 + 4;  // 2 x (Q K V G dO S dS) | A0..3 | Kt Kend P dP
constexpr int BWD_SMEM = BWD_TILES * TILE + 2 * BMAT_BYTES + (FTAB_FLOATS + GL_FLOATS) * 4 + 1024 + 256;

constexpr int BWD_THREADS = 512;

struct BwdBars {
  uint64_t tma[2];  // input tiles of the two buffers
  uint64_t mma[3];
  uint32_t tmem_slot;
  int failed;
};

__global__ void __launch_bounds__(BWD_THREADS) gla_bwd_main_kernel(
    const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
    const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmG,
    const __grid_constant__ CUtensorMap tmdO, const __grid_constant__ CUtensorMap tmS,
    const __grid_constant__ CUtensorMap tmdS, int qcol, int kcol, int vcol, int gcol, int docol,
    __nv_bfloat16* __restrict__ dq, long long dq_ld, int dqcol, __nv_bfloat16* __restrict__ dk, long long dk_ld,
    int dkcol, __nv_bfloat16* __restrict__ dv, long long dv_ld, int dvcol, float* __restrict__ dgl_local,
    float* __restrict__ chunk_tot, int T, int H, int logits, int nchunks, int* status, long long* dbg) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  uint8_t* smem = smem_raw + (((raw + 1023u) & ~1023u) - raw);
  // optional phase timers (developer aid): thread 0 adds the clocks spent up to each mark to dbg[i]
  const bool timed = dbg != nullptr && threadIdx.x == 0;
  long long tmark = timed ? clock64() : 0;
  auto mark = [&](int i) {
    if (timed) {
      const long long now = clock64();
      atomicAdd(reinterpret_cast<unsigned long long*>(dbg + i), (unsigned long long)(now - tmark));
      tmark = now;
    }
  };
  uint8_t* sIn = smem;              // 2 buffers x 7 input tiles (Q K V G dO S dS)
  uint8_t* sA = smem + 14 * TILE;   // 4 tiles
  uint8_t* sKt = smem + 18 * TILE;
  uint8_t* sKe = smem + 19 * TILE;
  uint8_t* sP = smem + 20 * TILE;
  uint8_t* sdP = smem + 21 * TILE;
  float* bmat = reinterpret_cast<float*>(smem + BWD_TILES * TILE);
  float* dmat = bmat + C * BST;
  float* ftab = dmat + C * BST;
  float* gl = ftab + FTAB_FLOATS;
  BwdBars* bars = reinterpret_cast<BwdBars*>(smem + BWD_TILES * TILE + 2 * BMAT_BYTES + (FTAB_FLOATS + GL_FLOATS) * 4);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int NT = T / C;

  if (tid == 0) {
    mbar_init(&bars->tma[0], 1);
    mbar_init(&bars->tma[1], 1);
    for (int i = 0; i < 3; ++i) mbar_init(&bars->mma[i], 1);
    bars->failed = 0;
    mbar_fence_init();
  }
  if (warp == 0) {
    tmem_alloc(&bars->tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = bars->tmem_slot;
  mark(0);  // barrier init + TMEM allocation
  // The CTA is persistent: it walks the chunks blockIdx.x, blockIdx.x + gridDim.x, ... and loads the input tiles of
  // the next chunk into the other buffer while it works on the current one, so neither the load latency nor the
  // per-CTA set-up (TMEM allocation, barrier init, block scheduling) is paid per chunk.
  auto issue_loads = [&](int cidx, int buf) {
    const int ch_ = cidx % NT, bh_ = cidx / NT, h_ = bh_ % H, r0_ = (bh_ / H) * T + ch_ * C;
    uint8_t* dst = sIn + buf * 7 * TILE;
    uint64_t* bar = &bars->tma[buf];
    mbar_expect_tx(bar, 7 * TILE);
    tma_load_3d(dst, &tmQ, bar, qcol + h_ * D, r0_, 0);
    tma_load_3d(dst + TILE, &tmK, bar, kcol + h_ * D, r0_, 0);
    tma_load_3d(dst + 2 * TILE, &tmV, bar, vcol + h_ * D, r0_, 0);
    tma_load_3d(dst + 3 * TILE, &tmG, bar, gcol + h_ * D, r0_, 0);
    tma_load_3d(dst + 4 * TILE, &tmdO, bar, docol + h_ * D, r0_, 0);
    tma_load_3d(dst + 5 * TILE, &tmS, bar, 0, cidx * D, 0);
    tma_load_3d(dst + 6 * TILE, &tmdS, bar, 0, cidx * D, 0);
  };
  if (tid == 0 && (int)blockIdx.x < nchunks) issue_loads(blockIdx.x, 0);
  int it = 0;
  int pend_buf = -1;        // thread 0: buffer with a prefetch in flight (waited for, bounded, if the loop is left early)
  uint32_t pend_par = 0;
  for (int cidx = blockIdx.x; cidx < nchunks; cidx += gridDim.x, ++it) {
  const int buf = it & 1;
  const uint32_t par = (uint32_t)(it & 1);  // parity of the once-per-chunk MMA barriers
  const int chunk = cidx % NT, bh = cidx / NT, h = bh % H, b = bh / H;
  const int row0 = b * T + chunk * C;
  uint8_t* sQ = sIn + buf * 7 * TILE;
  uint8_t* sK = sQ + TILE;
  uint8_t* sV = sQ + 2 * TILE;
  uint8_t* sG = sQ + 3 * TILE;
  uint8_t* sdO = sQ + 4 * TILE;
  uint8_t* sS = sQ + 5 * TILE;
  uint8_t* sdS = sQ + 6 * TILE;
  if (tid == 0 && cidx + (int)gridDim.x < nchunks) {
    fence_proxy_async_smem();  // the other buffer was last read through the generic proxy (previous chunk)
    issue_loads(cidx + gridDim.x, buf ^ 1);
    pend_buf = buf ^ 1;
    pend_par = (uint32_t)(((it + 1) >> 1) & 1);
  } else {
    pend_buf = -1;
  }
  bool ok = mbar_wait(&bars->tma[buf], (uint32_t)((it >> 1) & 1));
  if (!ok) bars->failed = ST_TIMEOUT_FULL;
  __syncthreads();
  mark(1);  // input tiles
  ok = bars->failed == 0;
  constexpr int CPW = 64 / (BWD_THREADS / 128);      // accumulator columns per warp (16 warps: 16)
  const int quarter = warp & 3, c0 = (warp >> 2) * CPW;  // TMEM lane quarter / first column of this warp
  const int row = quarter * 16 + (lane & 15);        // accumulator row owned by this thread when lane < 16
  if (ok) {
    build_cumsum<BWD_THREADS>(sG, bmat, logits != 0);
    build_factor_tables(bmat, ftab, gl);
    build_score_operands(sQ, sK, sA, sKt, sKe, bmat, ftab, gl);  // also K_end[s] = k_s e^{b_C - b_s}
    fence_proxy_async_smem();
    __syncthreads();
    mark(2);  // cumulative decay and operand tiles
    // ---- stage 1: P (cols 0..63) and dP = dO V^T (cols 64..127)
    if (tid == 0) {
      tc_fence_after_sync();
      issue_score_mmas(tmem, 0, smem_u32(sA), smem_u32(sKt));
      constexpr uint32_t id = make_idesc(64, 64, 1, 1, 0, 0);
      const uint32_t a = smem_u32(sdO), bb = smem_u32(sV);
#pragma unroll
      for (int k = 0; k < 4; ++k) umma_bf16(tmem + 64, desc_k(a, k), desc_k(bb, k), id, k > 0);
      umma_commit(&bars->mma[0]);
    }
    ok = __all_sync(0xffffffffu, mbar_wait(&bars->mma[0], par));
    if (ok) {
      tc_fence_after_sync();
      float v[CPW];
      load_acc_cols<CPW>(tmem, 0 + c0, quarter, v);
      if (lane < 16) store_row_cols<CPW>(sP, row, c0, v, row);
      load_acc_cols<CPW>(tmem, 64 + c0, quarter, v);
      if (lane < 16) store_row_cols<CPW>(sdP, row, c0, v, row);
      fence_proxy_async_smem();
      tc_fence_before_sync();
    } else if (lane == 0) {
      bars->failed = ST_TIMEOUT_TMEM;
    }
    __syncthreads();
    ok = bars->failed == 0;
  }
  mark(3);  // stage 1
  if (ok) {
    // ---- stage 2: dv (128..191), R1 = dO S^T (192..255), T_j = dP_j K~_j (256+64j)
    if (tid == 0) {
      tc_fence_after_sync();
      constexpr uint32_t id_mm = make_idesc(64, 64, 1, 1, 1, 1);
      constexpr uint32_t id_kk = make_idesc(64, 64, 1, 1, 0, 0);
      constexpr uint32_t id_km = make_idesc(64, 64, 1, 1, 0, 1);
      const uint32_t aP = smem_u32(sP), adO = smem_u32(sdO), aKe = smem_u32(sKe), adS = smem_u32(sdS);
      const uint32_t aS = smem_u32(sS), adP = smem_u32(sdP), aKt = smem_u32(sKt);
#pragma unroll
      for (int k = 0; k < 4; ++k) umma_bf16(tmem + 128, desc_mn(aP, k), desc_mn(adO, k), id_mm, k > 0);
#pragma unroll
      for (int k = 0; k < 4; ++k) umma_bf16(tmem + 128, desc_k(aKe, k), desc_mn(adS, k), id_km, 1u);
#pragma unroll
      for (int k = 0; k < 4; ++k) umma_bf16(tmem + 192, desc_k(adO, k), desc_k(aS, k), id_kk, k > 0);
#pragma unroll
      for (int j = 0; j < 4; ++j)
        umma_bf16(tmem + 256 + 64 * j, desc_k(adP, j), desc_mn(aKt, j), id_km, 0u);
      umma_commit(&bars->mma[1]);
    }
    // e^{b_t - r_i} for this thread's row (i = its sub-chunk) and columns: the only exponentials of this stage; the
    // shared-memory reads and the special-function work overlap the MMAs
    const int jrow = row >> 4;
    float e0[CPW];
    {
      float bt[CPW], rj[CPW];
      ld_row<CPW>(bmat + row * BST + c0, bt);
      if (jrow == 0) {
#pragma unroll
        for (int d = 0; d < CPW; ++d) rj[d] = 0.f;
      } else {
        ld_row<CPW>(bmat + (16 * jrow - 1) * BST + c0, rj);
      }
#pragma unroll
      for (int d = 0; d < CPW; ++d) e0[d] = __expf(bt[d] - rj[d]);
    }
    ok = __all_sync(0xffffffffu, mbar_wait(&bars->mma[1], par));
    if (ok) {
      tc_fence_after_sync();
      float v[CPW];
      // dv
      load_acc_cols<CPW>(tmem, 128 + c0, quarter, v);
      if (lane < 16) {
        __nv_bfloat16* dst = dv + (long long)(row0 + row) * dv_ld + dvcol + h * D + c0;
#pragma unroll
        for (int ch = 0; ch < CPW / 8; ++ch) {
          float o[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) o[i] = v[ch * 8 + i];
          *reinterpret_cast<uint4*>(dst + ch * 8) = pack8(o);
        }
      }
      // dq = e^{b_t} R1 + sum_{j <= i} e^{b_t - r_j} T_j, with e^{b_t - r_j} = e0 * ftab[i][j] (r_0 = 0 covers R1)
      float acc[CPW];
      load_acc_cols<CPW>(tmem, 192 + c0, quarter, v);
#pragma unroll
      for (int d = 0; d < CPW; ++d) acc[d] = v[d];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        load_acc_cols<CPW>(tmem, 256 + 64 * j + c0, quarter, v);  // warp-collective: every lane executes the load
        if (j <= jrow) {
          float f[CPW];
          ld_row<CPW>(ftab + (jrow * 4 + j) * D + c0, f);
          if (j == 0) {
#pragma unroll
            for (int d = 0; d < CPW; ++d) acc[d] = (acc[d] + v[d]) * (e0[d] * f[d]);
          } else {
#pragma unroll
            for (int d = 0; d < CPW; ++d) acc[d] += v[d] * (e0[d] * f[d]);
          }
        }
      }
      if (lane < 16) {
        __nv_bfloat16* dst = dq + (long long)(row0 + row) * dq_ld + dqcol + h * D + c0;
#pragma unroll
        for (int ch = 0; ch < CPW / 8; ++ch) {
          float o[8], q[8], qd[8];
          unpack8(*reinterpret_cast<const uint4*>(sQ + sw_off(row, c0 / 8 + ch)), q);
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            o[i] = acc[ch * 8 + i];
            qd[i] = q[i] * o[i];
          }
          st8(dmat + row * BST + c0 + ch * 8, qd);
          *reinterpret_cast<uint4*>(dst + ch * 8) = pack8(o);
        }
      }
      tc_fence_before_sync();
    } else if (lane == 0) {
      bars->failed = ST_TIMEOUT_TMEM;
    }
    __syncthreads();
    ok = bars->failed == 0;
  }
  mark(4);  // stage 2
  if (ok) {
    // ---- stage 3: R2 = V dS^T (192..255), U_j = dP^T Q~(j) (256+64j)
    if (tid == 0) {
      tc_fence_after_sync();
      constexpr uint32_t id_kk = make_idesc(64, 64, 1, 1, 0, 0);
      constexpr uint32_t id_mm = make_idesc(64, 64, 1, 1, 1, 1);
      const uint32_t aV = smem_u32(sV), adS = smem_u32(sdS), adP = smem_u32(sdP), aA = smem_u32(sA);
#pragma unroll
      for (int k = 0; k < 4; ++k) umma_bf16(tmem + 192, desc_k(aV, k), desc_k(adS, k), id_kk, k > 0);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
#pragma unroll
        for (int k = 0; k < 4; ++k)
          umma_bf16(tmem + 256 + 64 * j, desc_mn(adP, k), desc_mn(aA + j * TILE, k), id_mm, k > 0);
      }
      umma_commit(&bars->mma[2]);
    }
    // dk = e^{b_C - b_s} R2 + e^{r_q - b_s} U_q with q the sub-chunk of s; e^{b_C - b_s} = e^{r_q - b_s} gl[q]
    float x0[CPW], gq[CPW];
    {
      float bt[CPW], br[CPW];
      ld_row<CPW>(bmat + row * BST + c0, bt);
      if (quarter > 0) {
        ld_row<CPW>(bmat + (16 * quarter - 1) * BST + c0, br);
      } else {
#pragma unroll
        for (int d = 0; d < CPW; ++d) br[d] = 0.f;
      }
#pragma unroll
      for (int d = 0; d < CPW; ++d) x0[d] = __expf(br[d] - bt[d]);
      ld_row<CPW>(gl + quarter * D + c0, gq);
    }
    ok = __all_sync(0xffffffffu, mbar_wait(&bars->mma[2], par));
    if (ok) {
      tc_fence_after_sync();
      float v[CPW], acc[CPW];
      load_acc_cols<CPW>(tmem, 192 + c0, quarter, v);
#pragma unroll
      for (int d = 0; d < CPW; ++d) acc[d] = v[d] * gq[d];
      load_acc_cols<CPW>(tmem, 256 + 64 * quarter + c0, quarter, v);  // rows of sub-chunk j = quarter live in accumulator j
#pragma unroll
      for (int d = 0; d < CPW; ++d) acc[d] = (acc[d] + v[d]) * x0[d];
      if (lane < 16) {
        __nv_bfloat16* dst = dk + (long long)(row0 + row) * dk_ld + dkcol + h * D + c0;
#pragma unroll
        for (int ch = 0; ch < CPW / 8; ++ch) {
          float o[8], k[8], qd[8];
          unpack8(*reinterpret_cast<const uint4*>(sK + sw_off(row, c0 / 8 + ch)), k);
          ld8(dmat + row * BST + c0 + ch * 8, qd);
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            o[i] = acc[ch * 8 + i];
            qd[i] -= k[i] * o[i];
          }
          st8(dmat + row * BST + c0 + ch * 8, qd);
          *reinterpret_cast<uint4*>(dst + ch * 8) = pack8(o);
        }
      }
    } else if (lane == 0) {
      bars->failed = ST_TIMEOUT_TMEM;
    }
    __syncthreads();
    ok = bars->failed == 0;
  }
  mark(5);  // stage 3
  if (ok) {
    // in-chunk suffix sum of (q dq - k dk) per key dimension: parts of PR rows in parallel, then the totals of the
    // later parts (left in their first rows) are added on the way out
    constexpr int NPARTS = BWD_THREADS / 64, PR = C / NPARTS;
    const int d = tid & 63, part = tid >> 6;
    float acc = 0.f;
    for (int t = PR * part + PR - 1; t >= PR * part; --t) {
      acc += dmat[t * BST + d];
      dmat[t * BST + d] = acc;
    }
    __syncthreads();
    float base = 0.f;
    for (int pp = part + 1; pp < NPARTS; ++pp) base += dmat[(PR * pp) * BST + d];
    float* dst = dgl_local + (long long)row0 * (H * D) + h * D + d;
    for (int t = PR * part; t < PR * part + PR; ++t) dst[(long long)t * (H * D)] = dmat[t * BST + d] + base;
    if (part == 0) chunk_tot[(long long)cidx * D + d] = dmat[d] + base;
  }
  mark(6);  // suffix sums
  if (timed) atomicAdd(reinterpret_cast<unsigned long long*>(dbg + 7), 1ull);
  // chunk boundary: every read of this chunk's tiles, scratch matrices and accumulators is done before the next
  // chunk rewrites them
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  if (bars->failed != 0) break;
  }  // chunk loop
  if (bars->failed != 0 && tid == 0 && pend_buf >= 0) (void)mbar_wait(&bars->tma[pend_buf], pend_par);
  tc_fence_before_sync();
  __syncthreads();
  if (bars->failed != 0 && tid == 0 && status != nullptr) atomicCAS(status, 0, bars->failed);
  if (warp == 0) {
    tc_fence_after_sync();
    tmem_dealloc(tmem, 512);
  }
}

// dg[t] = (local suffix + totals of later chunks) * d(log decay)/d(gate input)
__global__ void __launch_bounds__(256) gla_dg_finalize_kernel(const float* __restrict__ dgl_local,
                                                              const float* __restrict__ chunk_tot,
                                                              const __nv_bfloat16* __restrict__ g, long long g_ld,
                                                              int gcol, __nv_bfloat16* __restrict__ dg, long long dg_ld,
                                                              int dgcol, int T, int H, int logits,
                                                              const float* __restrict__ end_term) {
  __shared__ float carry[D];
  const int NT = T / C;
  const int chunk = blockIdx.x % NT, bh = blockIdx.x / NT, h = bh % H, b = bh / H;
  if (threadIdx.x < D) {
    // end_term[bh][d] = sum_v dS_T[d][v] S_T[d][v]: the final state depends on every log decay of the sequence
    float acc = end_term != nullptr ? end_term[(long long)bh * D + threadIdx.x] : 0.f;
    for (int c = chunk + 1; c < NT; ++c) acc += chunk_tot[((long long)bh * NT + c) * D + threadIdx.x];
    carry[threadIdx.x] = acc;
  }
  __syncthreads();
  const long long row0 = (long long)b * T + chunk * C;
  for (int i = threadIdx.x; i < C * D; i += blockDim.x) {
    const int t = i >> 6, d = i & 63;
    const float x = __bfloat162float(g[(row0 + t) * g_ld + gcol + h * D + d]);
    const float raw = logits ? (fminf(x, 0.f) - log1pf(__expf(-fabsf(x)))) : x;
    float deriv;
    if (logits)
      deriv = (raw >= GLA_MIN_LOG_DECAY) ? 1.f / (1.f + __expf(x)) : 0.f;  // d logsigmoid = sigmoid(-x)
    else
      deriv = (x <= 0.f && x >= GLA_MIN_LOG_DECAY) ? 1.f : 0.f;
    const float val = (dgl_local[(row0 + t) * (H * D) + h * D + d] + carry[d]) * deriv;
    dg[(row0 + t) * dg_ld + dgcol + h * D + d] = __float2bfloat16(val);
  }
}

// ------------------------------------------------------------------------------------------------
// Decode step: S <- diag(e^{g}) S + k v^T ; o = q^T S. One CTA per (batch, head), 64x64 state in fp32.
// ------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) gla_decode_step_kernel(const __nv_bfloat16* __restrict__ q, long long q_ld, int qcol,
                                                              const __nv_bfloat16* __restrict__ k, long long k_ld, int kcol,
                                                              const __nv_bfloat16* __restrict__ v, long long v_ld, int vcol,
                                                              const __nv_bfloat16* __restrict__ g, long long g_ld, int gcol,
                                                              float* __restrict__ state, __nv_bfloat16* __restrict__ o,
                                                              long long o_ld, int ocol, int H, int logits) {
  __shared__ float sq[D], sk[D], sv[D], sd[D], part[4][D];
  const int bh = blockIdx.x, h = bh % H, b = bh / H;
  const int tid = threadIdx.x;
  if (tid < D) {
    sq[tid] = __bfloat162float(q[b * q_ld + qcol + h * D + tid]);
    sk[tid] = __bfloat162float(k[b * k_ld + kcol + h * D + tid]);
    sv[tid] = __bfloat162float(v[b * v_ld + vcol + h * D + tid]);
    sd[tid] = __expf(log_decay(__bfloat162float(g[b * g_ld + gcol + h * D + tid]), logits != 0));
  }
  __syncthreads();
  const int dv = tid & 63, quarter = tid >> 6;
  float* S = state + (long long)bh * D * D;
  float acc = 0.f;
#pragma unroll 4
  for (int i = quarter * 16; i < quarter * 16 + 16; ++i) {
    const float s = sd[i] * S[i * D + dv] + sk[i] * sv[dv];
    S[i * D + dv] = s;
    acc += sq[i] * s;
  }
  part[quarter][dv] = acc;
  __syncthreads();
  if (tid < D) o[b * o_ld + ocol + h * D + tid] = __float2bfloat16(part[0][tid] + part[1][tid] + part[2][tid] + part[3][tid]);
}

CUtensorMap tile_map(const GlaMat& m, long long rows, int width_cols) {
  // dims: {cols of the wide matrix, rows}; box {64, 64}
  return make_tmap_3d(m.ptr, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)width_cols, (uint64_t)rows, 1,
                      (uint64_t)m.ld * 2ull, (uint64_t)m.ld * 2ull * (uint64_t)rows, 64, 64);
}

void check_launch(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) throw std::runtime_error(std::string(what) + " launch failed: " + cudaGetErrorString(e));
}

template <typename K>
void set_smem(K kern, int bytes) {
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
  if (e != cudaSuccess) throw std::runtime_error(std::string("cannot set shared memory size: ") + cudaGetErrorString(e));
}

void check_dims(const GlaDims& d) {
  if (d.T % C != 0 || d.T <= 0) throw std::runtime_error("gla kernels need T to be a positive multiple of 64");
}

}  // namespace

void launch_gla_chunk_outer(int mode, GlaMat X, GlaMat Y, GlaMat G, float* out_kv, float* out_decay, GlaDims d,
                            int* status, cudaStream_t s) {
  check_dims(d);
  const long long rows = (long long)d.B * d.T;
  const int width = (int)X.ld;
  CUtensorMap tx = tile_map(X, rows, (int)X.ld), ty = tile_map(Y, rows, (int)Y.ld), tg = tile_map(G, rows, (int)G.ld);
  (void)width;
  constexpr int SMEM = 3 * TILE + BMAT_BYTES + 1024 + 256;
  static PerDeviceOnce cfg;  // the attribute is per device
  if (cfg.first_use()) set_smem(gla_chunk_outer_kernel, SMEM);
  const int grid = d.B * d.H * (d.T / C);
  gla_chunk_outer_kernel<<<grid, GLA_THREADS, SMEM, s>>>(tx, ty, tg, X.col0, Y.col0, G.col0, mode, out_kv, out_decay, d.T,
                                                         d.H, d.gate_logits ? 1 : 0, status);
  check_launch("gla_chunk_outer");
}

void launch_gla_scan(const float* kv, const float* decay, const float* init, __nv_bfloat16* states, float* final_state,
                     int BH, int NT, bool reverse, cudaStream_t s) {
  gla_scan_kernel<<<BH * 16, 256, 0, s>>>(kv, decay, init, states, final_state, NT, reverse ? 1 : 0);
  check_launch("gla_scan");
}

void launch_gla_fwd_out(GlaMat Q, GlaMat K, GlaMat V, GlaMat G, const __nv_bfloat16* states, GlaMat O, GlaDims d,
                        int* status, cudaStream_t s) {
  check_dims(d);
  const long long rows = (long long)d.B * d.T;
  const long long srows = (long long)d.B * d.H * (d.T / C) * D;
  CUtensorMap tq = tile_map(Q, rows, (int)Q.ld), tk = tile_map(K, rows, (int)K.ld), tv = tile_map(V, rows, (int)V.ld),
              tg = tile_map(G, rows, (int)G.ld);
  GlaMat S{states, D, 0};
  CUtensorMap ts = tile_map(S, srows, D);
  static PerDeviceOnce cfg;  // the attribute is per device
  if (cfg.first_use()) set_smem(gla_fwd_out_kernel, FWD_SMEM);
  const int grid = d.B * d.H * (d.T / C);
  gla_fwd_out_kernel<<<grid, FWD_THREADS, FWD_SMEM, s>>>(tq, tk, tv, tg, ts, Q.col0, K.col0, V.col0, G.col0,
                                                         reinterpret_cast<__nv_bfloat16*>(const_cast<void*>(O.ptr)), O.ld,
                                                         O.col0, d.T, d.H, d.gate_logits ? 1 : 0, status);
  check_launch("gla_fwd_out");
}

static long long* g_gla_dbg = nullptr;
void gla_set_debug_buffer(long long* p) { g_gla_dbg = p; }

void launch_gla_bwd_main(GlaMat Q, GlaMat K, GlaMat V, GlaMat G, GlaMat dO, const __nv_bfloat16* states,
                         const __nv_bfloat16* dstates, GlaMat dQ, GlaMat dK, GlaMat dV, float* dgl_local,
                         float* chunk_tot, GlaDims d, int* status, cudaStream_t s) {
  check_dims(d);
  const long long rows = (long long)d.B * d.T;
  const long long srows = (long long)d.B * d.H * (d.T / C) * D;
  CUtensorMap tq = tile_map(Q, rows, (int)Q.ld), tk = tile_map(K, rows, (int)K.ld), tv = tile_map(V, rows, (int)V.ld),
              tg = tile_map(G, rows, (int)G.ld), tdo = tile_map(dO, rows, (int)dO.ld);
  GlaMat S{states, D, 0}, dS{dstates, D, 0};
  CUtensorMap ts = tile_map(S, srows, D), tds = tile_map(dS, srows, D);
  static PerDeviceOnce cfg;  // the attribute is per device
  if (cfg.first_use()) set_smem(gla_bwd_main_kernel, BWD_SMEM);
  const int nchunks = d.B * d.H * (d.T / C);
  static int sms = 0;
  if (sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (sms <= 0) sms = 148;
  }
  const int grid = nchunks < sms ? nchunks : sms;  // one persistent CTA per SM
  gla_bwd_main_kernel<<<grid, BWD_THREADS, BWD_SMEM, s>>>(
      tq, tk, tv, tg, tdo, ts, tds, Q.col0, K.col0, V.col0, G.col0, dO.col0,
      reinterpret_cast<__nv_bfloat16*>(const_cast<void*>(dQ.ptr)), dQ.ld, dQ.col0,
      reinterpret_cast<__nv_bfloat16*>(const_cast<void*>(dK.ptr)), dK.ld, dK.col0,
      reinterpret_cast<__nv_bfloat16*>(const_cast<void*>(dV.ptr)), dV.ld, dV.col0, dgl_local, chunk_tot, d.T, d.H,
      d.gate_logits ? 1 : 0, nchunks, status, g_gla_dbg);
  check_launch("gla_bwd_main");
}

void launch_gla_dg_finalize(const float* dgl_local, const float* chunk_tot, GlaMat G, GlaMat dG, GlaDims d,
                            cudaStream_t s, const float* end_term) {
  check_dims(d);
  const int grid = d.B * d.H * (d.T / C);
  gla_dg_finalize_kernel<<<grid, 256, 0, s>>>(dgl_local, chunk_tot, reinterpret_cast<const __nv_bfloat16*>(G.ptr), G.ld,
                                              G.col0, reinterpret_cast<__nv_bfloat16*>(const_cast<void*>(dG.ptr)), dG.ld,
                                              dG.col0, d.T, d.H, d.gate_logits ? 1 : 0, end_term);
  check_launch("gla_dg_finalize");
}

void launch_gla_decode_step(GlaMat Q, GlaMat K, GlaMat V, GlaMat G, float* state, GlaMat O, int B, int H,
                            bool gate_logits, cudaStream_t s) {
  auto p = [](const GlaMat& m) { return reinterpret_cast<const __nv_bfloat16*>(m.ptr); };
  gla_decode_step_kernel<<<B * H, 256, 0, s>>>(p(Q), Q.ld, Q.col0, p(K), K.ld, K.col0, p(V), V.ld, V.col0, p(G), G.ld,
                                               G.col0, state, reinterpret_cast<__nv_bfloat16*>(const_cast<void*>(O.ptr)),
                                               O.ld, O.col0, H, gate_logits ? 1 : 0);
  check_launch("gla_decode_step");
}

}  // namespace tb
