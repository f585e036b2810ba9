// bf16 GEMM on the 5th-generation tensor cores: C = alpha * A * B^T (+ epilogue).
//
// One persistent CTA per SM, 320 threads, three roles:
//   warp 0    TMA producer: cp.async.bulk.tensor tiles of A (128 x 64) and B (BN x 64) into a ring of
//             128B-swizzled shared-memory stages, completion signalled on mbarriers;
//   warp 1    MMA issuer: one thread issues tcgen05.mma (M=128, N=BN, K=16) reading the stages through
//             shared-memory descriptors and accumulating into TMEM; tcgen05.commit releases a stage
//             back to the producer and, after the last K step, publishes the accumulator;
//   warps 2-9 epilogue: tcgen05.ld the fp32 accumulator (lane == output row), apply the epilogue in packed
//             f32x2 arithmetic (bias, GELU plus its derivative, multiply by saved rows, row scale), stage the
//             converted rows in shared memory and hand them to TMA (store or reduce-add).
// The accumulator is double-buffered in TMEM (2 x BN columns) so the epilogue of tile i overlaps the
// main loop of tile i+1. No cluster multicast is used; every CTA loads its own tiles.
//
// Replaces the reference's library GEMM call sites (torch.matmul / bmm / addmm in
// triune/model/attention.py:537-572, triune/model/moe.py:385-437, triune/kernels/fast_muon.py:15-161).
#include "tc_gemm.cuh"

#include <cuda.h>

#include <cstdlib>
#include <stdexcept>
#include <string>

#include "../common/ptx.cuh"
#include "../common/tma_desc.h"

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
  int* status;
  int total_tiles;
  int splits;           // split-K factor (dense mode, fp32 accumulate only)
  int iters_per_split;  // K iterations (of 64) handled by one split
};

struct Tile {
  int m0, n0, ba, bb, g, k_begin, k_iters;
  bool valid;
};

__device__ __forceinline__ Tile decode_tile(const KParams& p, int t) {
  Tile tl;
  tl.valid = true;
  if (p.mode == GEMM_GROUPED_M) {
    int m_idx = t % p.num_m, n_idx = t / p.num_m;
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
    tl.m0 = (r % p.num_m) * BM;
    tl.n0 = r / p.num_m;
    tl.g = b;
    if (p.mode == GEMM_GROUPED_K) {
      tl.ba = 0;
      tl.bb = 0;
      int k0 = p.group_offsets[b], k1 = p.group_offsets[b + 1];
      tl.k_begin = k0;
      tl.k_iters = (k1 - k0 + BK - 1) / BK;
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
enum { EPI_PLAIN = 0, EPI_PLAIN_F32 = 1, EPI_GELU = 2, EPI_MULAUX = 3 };

template <int BN, bool A_MN, bool B_MN, int EPI>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
    tc_gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                   const __grid_constant__ CUtensorMap tmC, const __grid_constant__ CUtensorMap tmAux, const KParams p) {
  using Cfg = GemmCfg<BN>;
  constexpr int STAGES = Cfg::STAGES;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  uint8_t* smem = smem_raw + (((raw + 1023u) & ~1023u) - raw);
  uint8_t* smemA = smem;
  uint8_t* smemB = smem + STAGES * Cfg::A_BYTES;
  uint8_t* smem_epi = smem + STAGES * Cfg::STAGE_BYTES;  // 8 warps x 1 staging tile
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem_epi + 8 * EPI_TILE);
  uint64_t* full = bars;                    // [STAGES] TMA -> MMA
  uint64_t* empty = bars + STAGES;          // [STAGES] MMA -> TMA
  uint64_t* acc_full = bars + 2 * STAGES;   // [2] MMA -> epilogue
  uint64_t* acc_empty = acc_full + 2;       // [2] epilogue -> MMA
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&acc_full[a], 1);
      mbar_init(&acc_empty[a], 8);
    }
    mbar_fence_init();
    prefetch_tmap(&tmA);
    prefetch_tmap(&tmB);
    prefetch_tmap(&tmC);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, Cfg::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      int issued = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < p.total_tiles && ok; t += gridDim.x) {
        Tile tl = decode_tile(p, t);
        if (!tl.valid) continue;
        const int n0 = tl.n0 * BN;
        for (int it = 0; it < tl.k_iters; ++it) {
          if (!mbar_wait(&empty[stage], phase ^ 1)) {
            report(p, ST_TIMEOUT_EMPTY);
            ok = false;
            break;
          }
          mbar_expect_tx(&full[stage], Cfg::STAGE_BYTES);
          const int k0 = tl.k_begin + it * BK;
          uint8_t* a_dst = smemA + stage * Cfg::A_BYTES;
          uint8_t* b_dst = smemB + stage * Cfg::B_BYTES;
          if (A_MN) {
#pragma unroll
            for (int j = 0; j < BM / 64; ++j)
              tma_load_3d(a_dst + j * (BK * 128), &tmA, &full[stage], tl.m0 + 64 * j, k0, tl.ba);
          } else {
            tma_load_3d(a_dst, &tmA, &full[stage], k0, tl.m0, tl.ba);
          }
          if (B_MN) {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j)
              tma_load_3d(b_dst + j * (BK * 128), &tmB, &full[stage], n0 + 64 * j, k0, tl.bb);
          } else {
            tma_load_3d(b_dst, &tmB, &full[stage], k0, n0, tl.bb);
          }
          ++issued;
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
      if (!ok) {
        // Give loads that are still in flight a bounded chance to land before the CTA retires.
        int pending = issued < STAGES ? issued : STAGES;
        int s = stage;
        uint32_t ph = phase;
        for (int i = 0; i < pending; ++i) {
          if (--s < 0) {
            s = STAGES - 1;
            ph ^= 1;
          }
          (void)mbar_wait(&full[s], ph);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc(BM, BN, 1, 1, A_MN ? 1 : 0, B_MN ? 1 : 0);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < p.total_tiles && ok; t += gridDim.x) {
        Tile tl = decode_tile(p, t);
        if (!tl.valid) continue;
        if (!mbar_wait(&acc_empty[acc], acc_phase ^ 1)) {
          report(p, ST_TIMEOUT_TMEM);
          break;
        }
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int it = 0; it < tl.k_iters; ++it) {
          if (!mbar_wait(&full[stage], phase)) {
            report(p, ST_TIMEOUT_FULL);
            ok = false;
            break;
          }
          tc_fence_after_sync();
          const uint32_t a_addr = smem_u32(smemA + stage * Cfg::A_BYTES);
          const uint32_t b_addr = smem_u32(smemB + stage * Cfg::B_BYTES);
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            const uint64_t adesc = A_MN ? make_smem_desc(a_addr + k * 2048, BK * 128, 1024)
                                        : make_smem_desc(a_addr + k * 32, 16, 1024);
            const uint64_t bdesc = B_MN ? make_smem_desc(b_addr + k * 2048, BK * 128, 1024)
                                        : make_smem_desc(b_addr + k * 32, 16, 1024);
            umma_bf16(d_tmem, adesc, bdesc, idesc, (it > 0 || k > 0) ? 1u : 0u);
          }
          umma_commit(&empty[stage]);
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (!ok) break;
        if (tl.k_iters > 0)
          umma_commit(&acc_full[acc]);
        else
          mbar_arrive(&acc_full[acc]);  // empty reduction: the epilogue substitutes zeros
        if (++acc == 2) {
          acc = 0;
          acc_phase ^= 1;
        }
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (warps 2..5)
    // Each warp owns 32 accumulator rows. Per column chunk (128 bytes of output: 64 bf16 or 32 fp32) it reads the
    // fp32 accumulator from TMEM, applies the epilogue, writes the rows into a private 128B-swizzled staging tile
    // and one lane hands the tile to TMA (plain store, or reduce-add for accumulate / split-K): global writes are
    // full 128-byte lines regardless of the row pitch, and ragged M/N edges are clipped by the tensor map.
    // Eight epilogue warps: a warp can only read the TMEM lanes of its quarter (warp % 4), so two warps share every
    // quarter and take alternate column chunks. Short reductions (K = 384) make the epilogue the longer phase of a
    // tile; halving it is worth more than a deeper load ring.
    const int lane_base = (warp & 3) * 32;
    const int col_half = (warp - 2) >> 2;
    uint8_t* my_stage = smem_epi + (warp - 2) * EPI_TILE;  // one staging tile per warp (a second one costs a load stage and measured slower)
    int acc = 0;
    uint32_t acc_phase = 0;
    constexpr bool out_f32 = (EPI == EPI_PLAIN_F32);
    constexpr int CW = out_f32 ? 32 : 64;  // columns per staged chunk (128 bytes)
    constexpr int NP = CW / 2;             // packed fp32 pairs per lane and chunk
    const bool reduce_add = ((p.flags & GF_ACCUMULATE) != 0) || p.splits > 1;
    const uint64_t alpha2 = pack_f2(p.alpha, p.alpha);
    for (int t = blockIdx.x; t < p.total_tiles; t += gridDim.x) {
      Tile tl = decode_tile(p, t);
      if (!tl.valid) continue;
      bool ok = mbar_wait(&acc_full[acc], acc_phase);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) {
        if (lane == 0) report(p, ST_TIMEOUT_TMEM);
        break;
      }
      tc_fence_after_sync();
      const int n0 = tl.n0 * BN;
      const int gm = tl.m0 + lane_base + lane;
      const bool row_ok = gm < p.M;
      const int out_batch = (p.mode == GEMM_GROUPED_M) ? 0 : tl.g;
      const long long c_off = (long long)out_batch * p.strideC + (long long)gm * p.ldc;
      const __nv_bfloat16* bias = p.bias ? p.bias + (long long)tl.g * p.bias_stride : nullptr;
#pragma unroll 1
      for (int c = col_half * CW; c < BN; c += 2 * CW) {
        if (n0 + c >= p.N) break;
        uint64_t v[NP];
        // Multiplier rows (the activation derivative saved by the forward pass): issue the loads first so their
        // latency hides behind the TMEM reads.
        uint4 auxv[8];
        if constexpr (EPI == EPI_MULAUX) {
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const int gn = n0 + c + j * 8;
            auxv[j] = (row_ok && gn < p.N) ? *reinterpret_cast<const uint4*>(p.aux_in + c_off + gn)
                                           : make_uint4(0u, 0u, 0u, 0u);
          }
        }
        if (tl.k_iters > 0) {
          uint32_t r0[32], r1[32];
          const uint32_t taddr = tmem_base + ((uint32_t)lane_base << 16) + acc * BN + c;
          tmem_ld_32x32b_x32(taddr, r0);
          if (!out_f32) tmem_ld_32x32b_x32(taddr + 32, r1);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 16; ++i) v[i] = pack_f2(__uint_as_float(r0[2 * i]), __uint_as_float(r0[2 * i + 1]));
          if (!out_f32) {
#pragma unroll
            for (int i = 0; i < 16; ++i)
              v[(NP - 16) + i] = pack_f2(__uint_as_float(r1[2 * i]), __uint_as_float(r1[2 * i + 1]));
          }
        } else {
#pragma unroll
          for (int i = 0; i < NP; ++i) v[i] = 0ull;
        }
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
        uint8_t* st = my_stage;
        if constexpr (EPI == EPI_PLAIN_F32) {
          if (p.row_scale) {
            const float rs = row_ok ? p.row_scale[gm] : 1.0f;
            const uint64_t rs2 = pack_f2(rs, rs);
#pragma unroll
            for (int i = 0; i < NP; ++i) v[i] = mul2(v[i], rs2);
          }
          if (lane == 0) tma_store_wait_read<0>();
          __syncwarp();
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            float4 o;
            unpack_f2(v[(j * 2) % NP], o.x, o.y);
            unpack_f2(v[(j * 2 + 1) % NP], o.z, o.w);
            *reinterpret_cast<float4*>(st + lane * 128 + ((j ^ (lane & 7)) << 4)) = o;
          }
        } else {
          uint32_t q[32];  // the chunk as bf16 pairs
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
              uint32_t dq[32];
#pragma unroll
              for (int i = 0; i < 32; ++i) {
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
              if (lane == 0) tma_store_wait_read<0>();
              __syncwarp();
#pragma unroll
              for (int j = 0; j < 8; ++j)
                *reinterpret_cast<uint4*>(st + lane * 128 + ((j ^ (lane & 7)) << 4)) =
                    make_uint4(dq[j * 4 + 0], dq[j * 4 + 1], dq[j * 4 + 2], dq[j * 4 + 3]);
              fence_proxy_async_smem();
              __syncwarp();
              if (lane == 0) {
                tma_store_3d(&tmAux, st, n0 + c, tl.m0 + lane_base, out_batch);
                tma_store_commit();
              }
            } else {
#pragma unroll
              for (int i = 0; i < 32; ++i) {
                const uint64_t x = v[i % NP];
                const uint64_t tt = tanh2(mul2(x, fma2(mul2(x, x), C1, C0)));
                const uint64_t h = mul2(x, HALF);
                q[i] = f2_to_bf16x2(fma2(h, tt, h));
              }
            }
          } else if constexpr (EPI == EPI_MULAUX) {
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              q[j * 4 + 0] = f2_to_bf16x2(mul2(v[(j * 4 + 0) % NP], bf16x2_to_f2(auxv[j].x)));
              q[j * 4 + 1] = f2_to_bf16x2(mul2(v[(j * 4 + 1) % NP], bf16x2_to_f2(auxv[j].y)));
              q[j * 4 + 2] = f2_to_bf16x2(mul2(v[(j * 4 + 2) % NP], bf16x2_to_f2(auxv[j].z)));
              q[j * 4 + 3] = f2_to_bf16x2(mul2(v[(j * 4 + 3) % NP], bf16x2_to_f2(auxv[j].w)));
            }
          } else {
            if (p.row_scale) {
              const float rs = row_ok ? p.row_scale[gm] : 1.0f;
              const uint64_t rs2 = pack_f2(rs, rs);
#pragma unroll
              for (int i = 0; i < 32; ++i) q[i] = f2_to_bf16x2(mul2(v[i % NP], rs2));
            } else {
#pragma unroll
              for (int i = 0; i < 32; ++i) q[i] = f2_to_bf16x2(v[i % NP]);
            }
          }
          if (lane == 0) tma_store_wait_read<0>();
          __syncwarp();
#pragma unroll
          for (int j = 0; j < 8; ++j)
            *reinterpret_cast<uint4*>(st + lane * 128 + ((j ^ (lane & 7)) << 4)) =
                make_uint4(q[j * 4 + 0], q[j * 4 + 1], q[j * 4 + 2], q[j * 4 + 3]);
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
          if (reduce_add)
            tma_reduce_add_3d(&tmC, st, n0 + c, tl.m0 + lane_base, out_batch);
          else
            tma_store_3d(&tmC, st, n0 + c, tl.m0 + lane_base, out_batch);
          tma_store_commit();
        }
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[acc]);
      if (++acc == 2) {
        acc = 0;
        acc_phase ^= 1;
      }
    }
    if (lane == 0) tma_store_wait<0>();  // staged tiles must be fully written before the CTA retires
    __syncwarp();
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
  }
}

template <int BN, bool A_MN, bool B_MN, int EPI>
void launch_variant(const CUtensorMap& tmA, const CUtensorMap& tmB, const CUtensorMap& tmC, const CUtensorMap& tmAux,
                    const KParams& kp, int grid, cudaStream_t stream) {
  auto kern = tc_gemm_kernel<BN, A_MN, B_MN, EPI>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, GemmCfg<BN>::SMEM_BYTES);
    if (e != cudaSuccess) throw std::runtime_error(std::string("tc_gemm: cannot set shared memory size: ") + cudaGetErrorString(e));
    configured = true;
  }
  kern<<<grid, GEMM_THREADS, GemmCfg<BN>::SMEM_BYTES, stream>>>(tmA, tmB, tmC, tmAux, kp);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) throw std::runtime_error(std::string("tc_gemm launch failed: ") + cudaGetErrorString(e));
}

template <int BN, bool A_MN, bool B_MN>
void dispatch_epi(int epi, const CUtensorMap& tmA, const CUtensorMap& tmB, const CUtensorMap& tmC,
                  const CUtensorMap& tmAux, const KParams& kp, int grid, cudaStream_t s) {
  if (epi == EPI_PLAIN) return launch_variant<BN, A_MN, B_MN, EPI_PLAIN>(tmA, tmB, tmC, tmAux, kp, grid, s);
  if (epi == EPI_PLAIN_F32) return launch_variant<BN, A_MN, B_MN, EPI_PLAIN_F32>(tmA, tmB, tmC, tmAux, kp, grid, s);
  if constexpr (!A_MN) {  // the activation epilogues follow row-major activations
    if (epi == EPI_GELU) return launch_variant<BN, A_MN, B_MN, EPI_GELU>(tmA, tmB, tmC, tmAux, kp, grid, s);
    if (epi == EPI_MULAUX) return launch_variant<BN, A_MN, B_MN, EPI_MULAUX>(tmA, tmB, tmC, tmAux, kp, grid, s);
  }
  throw std::runtime_error("tc_gemm: activation epilogues need a K-major A operand");
}

template <int BN>
void dispatch_major(bool a_mn, bool b_mn, int epi, const CUtensorMap& tmA, const CUtensorMap& tmB, const CUtensorMap& tmC,
                    const CUtensorMap& tmAux, const KParams& kp, int grid, cudaStream_t s) {
  if (!a_mn && !b_mn) dispatch_epi<BN, false, false>(epi, tmA, tmB, tmC, tmAux, kp, grid, s);
  else if (!a_mn && b_mn) dispatch_epi<BN, false, true>(epi, tmA, tmB, tmC, tmAux, kp, grid, s);
  else if (a_mn && !b_mn) dispatch_epi<BN, true, false>(epi, tmA, tmB, tmC, tmAux, kp, grid, s);
  else dispatch_epi<BN, true, true>(epi, tmA, tmB, tmC, tmAux, kp, grid, s);
}

int sm_count() {
  static int n = 0;
  if (n == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    if (n <= 0) n = 148;
  }
  return n;
}

}  // namespace

void launch_tc_gemm(const GemmArgs& a, cudaStream_t stream) {
  if (a.M <= 0 || a.N <= 0) return;
  if (a.N % 8 != 0) throw std::runtime_error("tc_gemm: N must be a multiple of 8");
  if (a.ldc % 8 != 0) throw std::runtime_error("tc_gemm: ldc must be a multiple of 8");
  if (a.lda % 8 != 0 || a.ldb % 8 != 0) throw std::runtime_error("tc_gemm: lda/ldb must be multiples of 8");
  if (a.mode != GEMM_GROUPED_K && a.K <= 0) throw std::runtime_error("tc_gemm: K must be positive");
  if (a.mode == GEMM_GROUPED_M && a.tile_group == nullptr) throw std::runtime_error("tc_gemm: tile_group missing");
  if ((a.flags & GF_OUT_F32) && (a.flags & (GF_GELU | GF_DGELU)))
    throw std::runtime_error("tc_gemm: activation epilogues write bf16 outputs");
  if ((a.flags & (GF_GELU | GF_DGELU)) && a.row_scale != nullptr)
    throw std::runtime_error("tc_gemm: activation epilogues take no row scale");
  if ((a.flags & GF_GELU) && (a.flags & GF_DGELU)) throw std::runtime_error("tc_gemm: one activation epilogue at a time");
  if ((a.flags & GF_DGELU) && a.aux_in == nullptr) throw std::runtime_error("tc_gemm: multiplier rows missing");
  if ((reinterpret_cast<uintptr_t>(a.C) & 15) != 0) throw std::runtime_error("tc_gemm: C must be 16-byte aligned");
  if (a.mode == GEMM_GROUPED_K && (a.group_offsets == nullptr || !a.a_mn_major || !a.b_mn_major))
    throw std::runtime_error("tc_gemm: grouped-K needs group_offsets and MN-major operands");

  // widest tile that divides N: the tensor core is most efficient at N = 256, then 192 (e.g. N = 384), then 128
  int BN = (a.N >= 256 && a.N % 256 == 0) ? 256 : ((a.N >= 192 && a.N % 192 == 0) ? 192 : (a.N > 64 ? 128 : 64));
  {
    static const int forced = [] {
      const char* e = std::getenv("TRIUNE_GEMM_BN");  // experiments only: force the tile width
      return e ? std::atoi(e) : 0;
    }();
    if (forced == 64 || forced == 128 || forced == 192 || forced == 256) BN = forced;
  }
  KParams kp;
  kp.M = a.M; kp.N = a.N; kp.K = a.K;
  kp.mode = a.mode; kp.flags = a.flags; kp.batch = a.batch < 1 ? 1 : a.batch;
  kp.num_m = (a.M + BM - 1) / BM;
  kp.num_n = (a.N + BN - 1) / BN;
  kp.ldc = a.ldc; kp.strideC = a.strideC;
  kp.a_batched = a.strideA != 0; kp.b_batched = a.strideB != 0;
  kp.alpha = a.alpha;
  kp.C = a.C; kp.bias = a.bias; kp.bias_stride = a.bias_stride;
  kp.aux_in = a.aux_in; kp.aux_out = a.aux_out; kp.row_scale = a.row_scale;
  kp.tile_group = a.tile_group; kp.group_offsets = a.group_offsets; kp.status = a.status;
  kp.total_tiles = kp.num_m * kp.num_n * (a.mode == GEMM_GROUPED_M ? 1 : kp.batch);
  kp.splits = 1;
  kp.iters_per_split = 0;
  // Split-K: weight gradients reduce over tens of thousands of tokens into a handful of output tiles; spread the
  // reduction over idle SMs. Only when the output is an fp32 accumulator (partials are added with red.add).
  if (a.mode == GEMM_DENSE && (kp.flags & GF_OUT_F32) && (kp.flags & GF_ACCUMULATE) && a.bias == nullptr &&
      a.row_scale == nullptr && !(kp.flags & (GF_GELU | GF_DGELU))) {
    const int total_iters = (a.K + BK - 1) / BK;
    const int sms = sm_count();
    if (kp.total_tiles * 2 <= sms && total_iters >= 16) {
      int splits = sms / kp.total_tiles;
      const int max_splits = total_iters / 8;
      if (splits > max_splits) splits = max_splits;
      if (splits > 1) {
        kp.iters_per_split = (total_iters + splits - 1) / splits;
        kp.splits = (total_iters + kp.iters_per_split - 1) / kp.iters_per_split;
        kp.total_tiles *= kp.splits;
      }
    }
  }

  // Tensor maps. dims are {contiguous, rows, batch}.
  const uint64_t a_rows_total = (a.mode == GEMM_GROUPED_K) ? (uint64_t)a.K : 0;  // K = total rows for grouped-K
  CUtensorMap tmA, tmB;
  const uint64_t nbA = kp.a_batched ? (uint64_t)kp.batch : 1, nbB = (a.mode == GEMM_GROUPED_M || kp.b_batched) ? (uint64_t)kp.batch : 1;
  const uint64_t sA = (kp.a_batched ? (uint64_t)a.strideA : (uint64_t)a.lda) * 2ull;
  const uint64_t sB = ((a.mode == GEMM_GROUPED_M || kp.b_batched) ? (uint64_t)a.strideB : (uint64_t)a.ldb) * 2ull;
  if (a.a_mn_major) {
    const uint64_t krows = (a.mode == GEMM_GROUPED_K) ? a_rows_total : (uint64_t)a.K;
    tmA = make_tmap_3d(a.A, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)a.M, krows, nbA, (uint64_t)a.lda * 2ull, sA, 64, BK);
  } else {
    tmA = make_tmap_3d(a.A, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)a.K, (uint64_t)a.M, nbA, (uint64_t)a.lda * 2ull, sA, BK, BM);
  }
  if (a.b_mn_major) {
    const uint64_t krows = (a.mode == GEMM_GROUPED_K) ? a_rows_total : (uint64_t)a.K;
    tmB = make_tmap_3d(a.B, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)a.N, krows, nbB, (uint64_t)a.ldb * 2ull, sB, 64, BK);
  } else {
    tmB = make_tmap_3d(a.B, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)a.K, (uint64_t)a.N, nbB, (uint64_t)a.ldb * 2ull, sB, BK, (uint32_t)BN);
  }
  // output maps: rows of 128 bytes (64 bf16 / 32 fp32) x 32 rows, one box per epilogue warp and column chunk
  const bool c_f32 = (kp.flags & GF_OUT_F32) != 0;
  const int c_elem = c_f32 ? 4 : 2;
  const uint64_t c_batches = (a.mode == GEMM_GROUPED_M) ? 1 : (uint64_t)kp.batch;
  const uint64_t c_bstride = (c_batches > 1 ? (uint64_t)a.strideC : (uint64_t)a.ldc * (uint64_t)a.M) * c_elem;
  CUtensorMap tmC = make_tmap_3d(a.C, c_f32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, c_elem,
                                 (uint64_t)a.N, (uint64_t)a.M, c_batches, (uint64_t)a.ldc * c_elem, c_bstride,
                                 c_f32 ? 32 : 64, 32);
  CUtensorMap tmAux = tmC;
  if (a.aux_out != nullptr)
    tmAux = make_tmap_3d(a.aux_out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)a.N, (uint64_t)a.M, c_batches,
                         (uint64_t)a.ldc * 2ull, (c_batches > 1 ? (uint64_t)a.strideC : (uint64_t)a.ldc * (uint64_t)a.M) * 2ull, 64, 32);
  const int grid = kp.total_tiles < sm_count() ? kp.total_tiles : sm_count();
  const int epi = (kp.flags & GF_GELU) ? EPI_GELU : ((kp.flags & GF_DGELU) ? EPI_MULAUX : (c_f32 ? EPI_PLAIN_F32 : EPI_PLAIN));
  if (BN == 256) dispatch_major<256>(a.a_mn_major, a.b_mn_major, epi, tmA, tmB, tmC, tmAux, kp, grid, stream);
  else if (BN == 192) dispatch_major<192>(a.a_mn_major, a.b_mn_major, epi, tmA, tmB, tmC, tmAux, kp, grid, stream);
  else if (BN == 128) dispatch_major<128>(a.a_mn_major, a.b_mn_major, epi, tmA, tmB, tmC, tmAux, kp, grid, stream);
  else dispatch_major<64>(a.a_mn_major, a.b_mn_major, epi, tmA, tmB, tmC, tmAux, kp, grid, stream);
}

}  // namespace tb
