// Shared pieces of the tcgen05 GEMM kernels (single-CTA and CTA-pair variants): tile bookkeeping and the epilogue.
#pragma once

#include <cuda.h>

#include "../common/ptx.cuh"
#include "tc_gemm.cuh"

namespace tb {

namespace {

constexpr int BM = 128;
constexpr int BK = 64;
constexpr int GEMM_THREADS = 320;  // warp 0 TMA, warp 1 MMA, warps 2..9 epilogue
constexpr int EPI_TILE = 32 * 128;  // one staged output tile: 32 rows x 128 bytes

template <int BN>
struct GemmCfg {
  static constexpr int A_BYTES = BM * BK * 2;
  static constexpr int B_BYTES = BN * BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGES = (BN == 256) ? 4 : (BN == 192 ? 4 : (BN == 128 ? 6 : 8));
  static constexpr int TMEM_COLS = (BN == 192) ? 512 : 2 * BN;  // power of two >= 2 * BN
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 8 * 4096 /*epilogue staging: 8 warps x 1 tile*/ + 1024 /*alignment slack*/ + 256;
};

struct KParams {
  int M, N, K;
  int mode, flags, batch;
  int num_m, num_n;
  long long ldc, strideC;
  int a_batched, b_batched;
  float alpha;
  void* C;
  const __nv_bfloat16* bias;
  long long bias_stride;
  const __nv_bfloat16* aux_in;
  __nv_bfloat16* aux_out;
  const float* row_scale;
  const int* tile_group;
  const int* group_offsets;
  const int* k_runs;    // grouped-K over a run list: (first row, 64-row blocks) pairs; group_offsets then index runs
  int* status;
  long long* dbg;       // optional phase timers (clock ticks summed over one warp's chunks), null in normal runs
  int total_tiles;
  int group_m;          // tile order: blocks of group_m row tiles x all column tiles (see raster)
  int splits;           // split-K factor (dense mode, fp32 accumulate only)
  int iters_per_split;  // K iterations (of 64) handled by one split
  int n_split;          // SwiGLU epilogues: column offset of the "up" half (= FFN hidden width)
  float beta;           // EPI_ADDAUX: weight of the added rows
};

struct Tile {
  int m0, n0, ba, bb, g, k_begin, k_iters;
  int k_end;  // run-list mode: k_begin .. k_end are the group's runs, k_iters the blocks in them
  bool valid;
};

// Grouped-K over a run list: 64-row blocks in runs [r0, r1) (a negative count reads as an empty run).
__device__ __forceinline__ int run_list_blocks(const int* __restrict__ runs, int r0, int r1) {
  int s = 0;
  for (int r = r0; r < r1; ++r) {
    const int n = runs[2 * r + 1];
    s += n > 0 ? n : 0;
  }
  return s;
}
// The producer's walk over a group's runs: `run` starts at Tile::k_begin with left = 0; returns the first row of the
// next block. Called exactly Tile::k_iters times, so a non-empty run is always ahead.
__device__ __forceinline__ int run_list_next(const int* __restrict__ runs, int& run, int run_end, int& left, int& kpos) {
  while (left <= 0 && run < run_end) {
    kpos = runs[2 * run];
    left = runs[2 * run + 1];
    ++run;
  }
  const int k0 = kpos;
  kpos += 64;
  --left;
  return k0;
}

// Tile order. The CTAs of one wave should share as many operand tiles as possible: the tiles are walked in blocks
// of group_m row tiles x all num_n column tiles, row tile fastest inside a block, and group_m * num_n is about the
// number of SMs. A block's A tiles are then read from DRAM once (every column tile of the block uses them while they
// are in L2) instead of once per column tile, which matters as soon as A plus the output outgrow L2.
__device__ __forceinline__ void raster(int r, int num_m, int num_n, int group_m, int& m_idx, int& n_idx) {
  const int per_block = group_m * num_n;
  const int blk = r / per_block, within = r % per_block;
  const int m_first = blk * group_m;
  const int gm = (num_m - m_first) < group_m ? (num_m - m_first) : group_m;
  m_idx = m_first + within % gm;
  n_idx = within / gm;
}
__host__ inline int raster_group_m(int num_m, int num_n, int ctas) {
  int g = ctas / (num_n < 1 ? 1 : num_n);
  if (g < 1) g = 1;
  return g > num_m ? num_m : g;
}

__device__ __forceinline__ Tile decode_tile(const KParams& p, int t) {
  Tile tl;
  tl.valid = true;
  if (p.mode == GEMM_GROUPED_M) {
    int m_idx, n_idx;
    raster(t, p.num_m, p.num_n, p.group_m, m_idx, n_idx);
    int g = p.tile_group[m_idx];
    tl.valid = g >= 0;
    tl.g = g < 0 ? 0 : g;
    tl.m0 = m_idx * BM;
    tl.n0 = n_idx;  // scaled by BN by the caller
    tl.ba = 0;
    tl.bb = tl.g;
    tl.k_begin = 0;
    tl.k_iters = (p.K + BK - 1) / BK;
  } else {
    int per_b = p.num_m * p.num_n;
    int split = 0;
    if (p.splits > 1) {
      const int base = per_b * p.batch;
      split = t / base;
      t = t % base;
    }
    int b = t / per_b, r = t % per_b;
    int m_idx, n_idx;
    raster(r, p.num_m, p.num_n, p.group_m, m_idx, n_idx);
    tl.m0 = m_idx * BM;
    tl.n0 = n_idx;
    tl.g = b;
    if (p.mode == GEMM_GROUPED_K) {
      tl.ba = 0;
      tl.bb = 0;
      int k0 = p.group_offsets[b], k1 = p.group_offsets[b + 1];
      tl.k_begin = k0;
      tl.k_end = k1;
      tl.k_iters = p.k_runs ? run_list_blocks(p.k_runs, k0, k1) : (k1 - k0 + BK - 1) / BK;
    } else {
      tl.ba = p.a_batched ? b : 0;
      tl.bb = p.b_batched ? b : 0;
      const int total_iters = (p.K + BK - 1) / BK;
      if (p.splits > 1) {
        tl.k_begin = split * p.iters_per_split * BK;
        const int left = total_iters - split * p.iters_per_split;
        tl.k_iters = left < p.iters_per_split ? (left < 0 ? 0 : left) : p.iters_per_split;
      } else {
        tl.k_begin = 0;
        tl.k_iters = total_iters;
      }
    }
  }
  return tl;
}

__device__ __forceinline__ void report(const KParams& p, int code) {
  if (p.status != nullptr) atomicCAS(p.status, 0, code);
}

// Epilogue kinds (compile-time, so the plain stores do not carry the activation code's registers):
//   EPI_PLAIN      alpha, bias, row scale, bf16 output (store or reduce-add)
//   EPI_PLAIN_F32  the same with an fp32 output (weight-gradient accumulation, split-K)
//   EPI_GELU       bias, tanh-GELU, bf16 output; optionally GELU'(pre-activation) as a second bf16 output
//   EPI_MULAUX     output = alpha * acc * aux_in (the backward of EPI_GELU: aux_in holds GELU')
//   EPI_SWIGLU     accumulator columns [0, n/2) hold gate, [n/2, n) hold up pre-activations of the SAME output columns
//                  (the producer loads the two row blocks of the fused gate/up weight side by side); output =
//                  silu(gate) * up, and optionally both pre-activations go out as bf16 (aux_out, [M, 2 * n_split])
//   EPI_DSWIGLU    acc = d(hidden); reads gate/up from aux_in and writes d(gate), d(up) into C ([M, 2 * n_split])
//   EPI_ADDAUX     output = alpha * acc + beta * aux_in (bf16 rows of C's layout): the blends of the Newton-Schulz
//                  iteration (b A + c A A, a X + B X) without separate elementwise passes
enum { EPI_PLAIN = 0, EPI_PLAIN_F32 = 1, EPI_GELU = 2, EPI_MULAUX = 3, EPI_SWIGLU = 4, EPI_DSWIGLU = 5, EPI_ADDAUX = 6 };

// One accumulator tile (128 rows x n_cols fp32 in TMEM at tmem_acc) through the epilogue EPI and out to global
// memory. Called by the eight epilogue warps of a CTA: a warp can only read the TMEM lanes of its quarter
// (warp % 4), so two warps share every quarter and take alternate column chunks (col_half 0 / 1). Per chunk (64 bytes
// of output per row: 32 bf16 or 16 fp32 columns) a warp reads the accumulator, applies the epilogue in packed f32x2
// arithmetic, writes its 32 rows into one of its two 64B-swizzled staging buffers and one lane hands the buffer to TMA
// (plain store, or reduce-add for accumulate / split-K). The buffers alternate, and a buffer is reused once the store
// issued two chunks earlier has read it, so a warp never waits for the store it has just issued: with one buffer per
// warp that wait (about a microsecond per chunk) made short reductions epilogue-bound. Ragged M/N edges are clipped
// by the tensor map. m_base is the first output row of this CTA's 128 rows, n0 the first output column of the tile;
// `buf` carries the buffer choice from tile to tile.
constexpr int EPI_BUF = 32 * 64;  // one staging buffer: 32 rows x 64 bytes

__device__ __forceinline__ uint8_t* epi_claim(uint8_t* my_stage, uint32_t& buf, int lane) {
  if (lane == 0) tma_store_wait_read<1>();
  __syncwarp();
  uint8_t* st = my_stage + buf * EPI_BUF;
  buf ^= 1u;
  return st;
}
// 16-byte unit j of row `lane` in a 64B-swizzled buffer
__device__ __forceinline__ uint32_t epi_off(int lane, int j) { return lane * 64 + ((j ^ ((lane >> 1) & 3)) << 4); }

template <int EPI>
__device__ __forceinline__ void epilogue_tile(const KParams& p, const Tile& tl, const CUtensorMap* tmC,
                                              const CUtensorMap* tmAux, uint32_t tmem_acc, int n_cols, int n0,
                                              int m_base, int lane_base, int col_half, int lane, uint8_t* my_stage,
                                              uint32_t& buf) {
  constexpr bool out_f32 = (EPI == EPI_PLAIN_F32);
  constexpr int CW = out_f32 ? 16 : 32;  // columns per staged chunk (64 bytes)
  constexpr int NP = CW / 2;             // packed fp32 pairs per lane and chunk
  const bool reduce_add = ((p.flags & GF_ACCUMULATE) != 0) || p.splits > 1;
  const uint64_t alpha2 = pack_f2(p.alpha, p.alpha);
  const int gm = m_base + lane_base + lane;
  const bool row_ok = gm < p.M;
  const int out_batch = (p.mode == GEMM_GROUPED_M) ? 0 : tl.g;
  const long long c_off = (long long)out_batch * p.strideC + (long long)gm * p.ldc;
  const __nv_bfloat16* bias = p.bias ? p.bias + (long long)tl.g * p.bias_stride : nullptr;
#pragma unroll 1
  for (int c = col_half * CW; c < n_cols; c += 2 * CW) {
    if (n0 + c >= p.N) break;
    const bool timed = p.dbg != nullptr && lane == 0 && lane_base == 0 && col_half == 0;
    long long tk0 = 0, tk1 = 0, tk2 = 0, tk3 = 0;
    if (timed) tk0 = clock64();
    uint64_t v[NP];
    // Multiplier rows (the activation derivative saved by the forward pass): issue the loads first so their
    // latency hides behind the TMEM read.
    uint4 auxv[4];
    if constexpr (EPI == EPI_MULAUX || EPI == EPI_ADDAUX) {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int gn = n0 + c + j * 8;
        auxv[j] = (row_ok && gn < p.N) ? *reinterpret_cast<const uint4*>(p.aux_in + c_off + gn)
                                       : make_uint4(0u, 0u, 0u, 0u);
      }
    }
    if (tl.k_iters > 0) {
      const uint32_t taddr = tmem_acc + ((uint32_t)lane_base << 16) + c;
      if constexpr (out_f32) {
        uint32_t r[16];
        tmem_ld_32x32b_x16(taddr, r);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < NP; ++i) v[i] = pack_f2(__uint_as_float(r[2 * i]), __uint_as_float(r[2 * i + 1]));
      } else {
        uint32_t r[32];
        tmem_ld_32x32b_x32(taddr, r);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < NP; ++i) v[i] = pack_f2(__uint_as_float(r[2 * i]), __uint_as_float(r[2 * i + 1]));
      }
    } else {
#pragma unroll
      for (int i = 0; i < NP; ++i) v[i] = 0ull;
    }
    if (timed) tk1 = clock64();
    // alpha and bias: one packed fma per pair
    if (bias) {
#pragma unroll
      for (int j = 0; j < NP / 4; ++j) {
        const int gn = n0 + c + j * 8;
        if (gn < p.N) {
          const uint4 bv = *reinterpret_cast<const uint4*>(bias + gn);
          v[j * 4 + 0] = fma2(v[j * 4 + 0], alpha2, bf16x2_to_f2(bv.x));
          v[j * 4 + 1] = fma2(v[j * 4 + 1], alpha2, bf16x2_to_f2(bv.y));
          v[j * 4 + 2] = fma2(v[j * 4 + 2], alpha2, bf16x2_to_f2(bv.z));
          v[j * 4 + 3] = fma2(v[j * 4 + 3], alpha2, bf16x2_to_f2(bv.w));
        }
      }
    } else if (p.alpha != 1.0f) {
#pragma unroll
      for (int i = 0; i < NP; ++i) v[i] = mul2(v[i], alpha2);
    }
    uint8_t* st;
    if constexpr (EPI == EPI_PLAIN_F32) {
      if (p.row_scale) {
        const float rs = row_ok ? p.row_scale[gm] : 1.0f;
        const uint64_t rs2 = pack_f2(rs, rs);
#pragma unroll
        for (int i = 0; i < NP; ++i) v[i] = mul2(v[i], rs2);
      }
      st = epi_claim(my_stage, buf, lane);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float4 o;
        unpack_f2(v[j * 2], o.x, o.y);
        unpack_f2(v[j * 2 + 1], o.z, o.w);
        *reinterpret_cast<float4*>(st + epi_off(lane, j)) = o;
      }
    } else {
      uint32_t q[16];  // the chunk as bf16 pairs
      if constexpr (EPI == EPI_GELU) {
        // gelu(x) = h + h t with h = x / 2, t = tanh(k0 (x + k1 x^3)); its derivative
        // (1 + t) / 2 + h (1 - t^2) k0 (1 + 3 k1 x^2) reuses t and goes out as a second bf16 tile, so the
        // backward GEMM's epilogue is a single multiply.
        const uint64_t C0 = pack_f2(0.7978845608028654f, 0.7978845608028654f);
        const uint64_t C1 = pack_f2(0.0356774081363001f, 0.0356774081363001f);
        const uint64_t NC0 = pack_f2(-0.7978845608028654f, -0.7978845608028654f);
        const uint64_t NC3 = pack_f2(-0.1070322244089003f, -0.1070322244089003f);
        const uint64_t HALF = pack_f2(0.5f, 0.5f);
        const uint64_t NEG1 = pack_f2(-1.0f, -1.0f);
        if (p.aux_out) {
          uint32_t dq[16];
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const uint64_t x = v[i % NP];
            const uint64_t x2 = mul2(x, x);
            const uint64_t tt = tanh2(mul2(x, fma2(x2, C1, C0)));
            const uint64_t h = mul2(x, HALF);
            q[i] = f2_to_bf16x2(fma2(h, tt, h));
            const uint64_t sgm = fma2(tt, HALF, HALF);
            const uint64_t nq = fma2(tt, tt, NEG1);   // -(1 - t^2)
            const uint64_t ndu = fma2(x2, NC3, NC0);  // -k0 (1 + 3 k1 x^2)
            dq[i] = f2_to_bf16x2(fma2(mul2(h, nq), ndu, sgm));
          }
          uint8_t* sd = epi_claim(my_stage, buf, lane);
#pragma unroll
          for (int j = 0; j < 4; ++j)
            *reinterpret_cast<uint4*>(sd + epi_off(lane, j)) =
                make_uint4(dq[j * 4 + 0], dq[j * 4 + 1], dq[j * 4 + 2], dq[j * 4 + 3]);
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            tma_store_3d(tmAux, sd, n0 + c, m_base + lane_base, out_batch);
            tma_store_commit();
          }
        } else {
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const uint64_t x = v[i % NP];
            const uint64_t tt = tanh2(mul2(x, fma2(mul2(x, x), C1, C0)));
            const uint64_t h = mul2(x, HALF);
            q[i] = f2_to_bf16x2(fma2(h, tt, h));
          }
        }
      } else if constexpr (EPI == EPI_MULAUX) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          q[j * 4 + 0] = f2_to_bf16x2(mul2(v[(j * 4 + 0) % NP], bf16x2_to_f2(auxv[j].x)));
          q[j * 4 + 1] = f2_to_bf16x2(mul2(v[(j * 4 + 1) % NP], bf16x2_to_f2(auxv[j].y)));
          q[j * 4 + 2] = f2_to_bf16x2(mul2(v[(j * 4 + 2) % NP], bf16x2_to_f2(auxv[j].z)));
          q[j * 4 + 3] = f2_to_bf16x2(mul2(v[(j * 4 + 3) % NP], bf16x2_to_f2(auxv[j].w)));
        }
      } else if constexpr (EPI == EPI_ADDAUX) {
        const uint64_t beta2 = pack_f2(p.beta, p.beta);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          q[j * 4 + 0] = f2_to_bf16x2(fma2(bf16x2_to_f2(auxv[j].x), beta2, v[(j * 4 + 0) % NP]));
          q[j * 4 + 1] = f2_to_bf16x2(fma2(bf16x2_to_f2(auxv[j].y), beta2, v[(j * 4 + 1) % NP]));
          q[j * 4 + 2] = f2_to_bf16x2(fma2(bf16x2_to_f2(auxv[j].z), beta2, v[(j * 4 + 2) % NP]));
          q[j * 4 + 3] = f2_to_bf16x2(fma2(bf16x2_to_f2(auxv[j].w), beta2, v[(j * 4 + 3) % NP]));
        }
      } else {
        if (p.row_scale) {
          const float rs = row_ok ? p.row_scale[gm] : 1.0f;
          const uint64_t rs2 = pack_f2(rs, rs);
#pragma unroll
          for (int i = 0; i < 16; ++i) q[i] = f2_to_bf16x2(mul2(v[i % NP], rs2));
        } else {
#pragma unroll
          for (int i = 0; i < 16; ++i) q[i] = f2_to_bf16x2(v[i % NP]);
        }
      }
      if (timed) tk2 = clock64();
      st = epi_claim(my_stage, buf, lane);
      if (timed) tk3 = clock64();
#pragma unroll
      for (int j = 0; j < 4; ++j)
        *reinterpret_cast<uint4*>(st + epi_off(lane, j)) =
            make_uint4(q[j * 4 + 0], q[j * 4 + 1], q[j * 4 + 2], q[j * 4 + 3]);
    }
    fence_proxy_async_smem();
    __syncwarp();
    if (timed) {
      const long long tk4 = clock64();
      atomicAdd(reinterpret_cast<unsigned long long*>(p.dbg + 0), (unsigned long long)(tk1 - tk0));  // TMEM read
      atomicAdd(reinterpret_cast<unsigned long long*>(p.dbg + 1), (unsigned long long)(tk2 - tk1));  // arithmetic
      atomicAdd(reinterpret_cast<unsigned long long*>(p.dbg + 2), (unsigned long long)(tk3 - tk2));  // buffer claim
      atomicAdd(reinterpret_cast<unsigned long long*>(p.dbg + 3), (unsigned long long)(tk4 - tk3));  // staging writes + fence
      atomicAdd(reinterpret_cast<unsigned long long*>(p.dbg + 4), 1ull);                              // chunks
    }
    if (lane == 0) {
      if (reduce_add)
        tma_reduce_add_3d(tmC, st, n0 + c, m_base + lane_base, out_batch);
      else
        tma_store_3d(tmC, st, n0 + c, m_base + lane_base, out_batch);
      tma_store_commit();
    }
    if (timed) atomicAdd(reinterpret_cast<unsigned long long*>(p.dbg + 7), (unsigned long long)(clock64() - tk0));  // whole chunk
  }
}

// Stage one 32-row x 32-column bf16 chunk (16 packed pairs per lane) and hand it to TMA.
__device__ __forceinline__ void epi_store_chunk(const CUtensorMap* tm, const uint32_t (&q)[16], int col, int row,
                                                int batch, int lane, uint8_t* my_stage, uint32_t& buf) {
  uint8_t* st = epi_claim(my_stage, buf, lane);
#pragma unroll
  for (int j = 0; j < 4; ++j)
    *reinterpret_cast<uint4*>(st + epi_off(lane, j)) = make_uint4(q[j * 4 + 0], q[j * 4 + 1], q[j * 4 + 2], q[j * 4 + 3]);
  fence_proxy_async_smem();
  __syncwarp();
  if (lane == 0) {
    tma_store_3d(tm, st, col, row, batch);
    tma_store_commit();
  }
}

__device__ __forceinline__ float sigmoid_f(float x) { return __fdividef(1.0f, 1.0f + __expf(-x)); }

// SwiGLU forward epilogue: n_cols accumulator columns = [gate (n_cols/2) | up (n_cols/2)] of output columns
// [n0, n0 + n_cols/2). Same warp roles and staging as epilogue_tile.
__device__ __forceinline__ void epilogue_tile_swiglu(const KParams& p, const Tile& tl, const CUtensorMap* tmC,
                                                     const CUtensorMap* tmAux, uint32_t tmem_acc, int n_cols, int n0,
                                                     int m_base, int lane_base, int col_half, int lane,
                                                     uint8_t* my_stage, uint32_t& buf) {
  const int half = n_cols >> 1;
#pragma unroll 1
  for (int c = col_half * 32; c < half; c += 64) {
    if (n0 + c >= p.N) break;
    uint32_t rg[32], ru[32];
    if (tl.k_iters > 0) {
      const uint32_t taddr = tmem_acc + ((uint32_t)lane_base << 16) + c;
      tmem_ld_32x32b_x32(taddr, rg);
      tmem_ld_32x32b_x32(taddr + half, ru);
      tmem_ld_wait();
    } else {
#pragma unroll
      for (int i = 0; i < 32; ++i) rg[i] = ru[i] = 0u;
    }
    uint32_t q[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const float g0 = __uint_as_float(rg[2 * i]), g1 = __uint_as_float(rg[2 * i + 1]);
      const float u0 = __uint_as_float(ru[2 * i]), u1 = __uint_as_float(ru[2 * i + 1]);
      q[i] = pack_bf16x2(g0 * sigmoid_f(g0) * u0, g1 * sigmoid_f(g1) * u1);
    }
    epi_store_chunk(tmC, q, n0 + c, m_base + lane_base, 0, lane, my_stage, buf);
    if (p.aux_out) {
#pragma unroll
      for (int i = 0; i < 16; ++i) q[i] = pack_bf16x2(__uint_as_float(rg[2 * i]), __uint_as_float(rg[2 * i + 1]));
      epi_store_chunk(tmAux, q, n0 + c, m_base + lane_base, 0, lane, my_stage, buf);
#pragma unroll
      for (int i = 0; i < 16; ++i) q[i] = pack_bf16x2(__uint_as_float(ru[2 * i]), __uint_as_float(ru[2 * i + 1]));
      epi_store_chunk(tmAux, q, p.n_split + n0 + c, m_base + lane_base, 0, lane, my_stage, buf);
    }
  }
}

// SwiGLU backward epilogue: acc = d(hidden) for output columns [n0, n0 + n_cols); with g, u read from aux_in
// ([M, 2 * n_split], row pitch ldc) it writes d(gate) = dh * u * silu'(g) and d(up) = dh * silu(g) into C
// ([M, 2 * n_split]) at columns n0.. and n_split + n0...
__device__ __forceinline__ void epilogue_tile_dswiglu(const KParams& p, const Tile& tl, const CUtensorMap* tmC,
                                                      uint32_t tmem_acc, int n_cols, int n0, int m_base, int lane_base,
                                                      int col_half, int lane, uint8_t* my_stage, uint32_t& buf) {
  const int gm = m_base + lane_base + lane;
  const bool row_ok = gm < p.M;
  const long long c_off = (long long)gm * p.ldc;
#pragma unroll 1
  for (int c = col_half * 32; c < n_cols; c += 64) {
    if (n0 + c >= p.N) break;
    uint4 gv[4], uv[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int gn = n0 + c + j * 8;
      const bool ok = row_ok && gn < p.N;
      gv[j] = ok ? *reinterpret_cast<const uint4*>(p.aux_in + c_off + gn) : make_uint4(0u, 0u, 0u, 0u);
      uv[j] = ok ? *reinterpret_cast<const uint4*>(p.aux_in + c_off + p.n_split + gn) : make_uint4(0u, 0u, 0u, 0u);
    }
    uint32_t r[32];
    if (tl.k_iters > 0) {
      tmem_ld_32x32b_x32(tmem_acc + ((uint32_t)lane_base << 16) + c, r);
      tmem_ld_wait();
    } else {
#pragma unroll
      for (int i = 0; i < 32; ++i) r[i] = 0u;
    }
    uint32_t qg[16], qu[16];
    const uint32_t* gp = reinterpret_cast<const uint32_t*>(gv);
    const uint32_t* up = reinterpret_cast<const uint32_t*>(uv);
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      float g0, g1, u0, u1;
      unpack_f2(bf16x2_to_f2(gp[i]), g0, g1);
      unpack_f2(bf16x2_to_f2(up[i]), u0, u1);
      const float d0 = __uint_as_float(r[2 * i]) * p.alpha, d1 = __uint_as_float(r[2 * i + 1]) * p.alpha;
      const float s0 = sigmoid_f(g0), s1 = sigmoid_f(g1);
      qg[i] = pack_bf16x2(d0 * u0 * s0 * (1.0f + g0 * (1.0f - s0)), d1 * u1 * s1 * (1.0f + g1 * (1.0f - s1)));
      qu[i] = pack_bf16x2(d0 * g0 * s0, d1 * g1 * s1);
    }
    epi_store_chunk(tmC, qg, n0 + c, m_base + lane_base, 0, lane, my_stage, buf);
    epi_store_chunk(tmC, qu, p.n_split + n0 + c, m_base + lane_base, 0, lane, my_stage, buf);
  }
}

// One call site for every epilogue kind.
template <int EPI>
__device__ __forceinline__ void run_epilogue(const KParams& p, const Tile& tl, const CUtensorMap* tmC,
                                             const CUtensorMap* tmAux, uint32_t tmem_acc, int n_cols, int n0, int m_base,
                                             int lane_base, int col_half, int lane, uint8_t* my_stage, uint32_t& buf) {
  if constexpr (EPI == EPI_SWIGLU)
    epilogue_tile_swiglu(p, tl, tmC, tmAux, tmem_acc, n_cols, n0, m_base, lane_base, col_half, lane, my_stage, buf);
  else if constexpr (EPI == EPI_DSWIGLU)
    epilogue_tile_dswiglu(p, tl, tmC, tmem_acc, n_cols, n0, m_base, lane_base, col_half, lane, my_stage, buf);
  else
    epilogue_tile<EPI>(p, tl, tmC, tmAux, tmem_acc, n_cols, n0, m_base, lane_base, col_half, lane, my_stage, buf);
}

}  // namespace

}  // namespace tb
