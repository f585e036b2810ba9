// Block-scaled GEMMs on the 5th-generation tensor cores: C[M, N] (bf16) = alpha * (A .* SFA) (B .* SFB)^T, the scales
// applied by the tensor core itself (`tcgen05.mma ... .block_scale` reads them from TMEM, where `tcgen05.cp` places
// them from shared memory), so no operand is ever decoded to bf16:
//
//   NVFP4  A, B packed E2M1 (two codes per byte, K contiguous), one unsigned E4M3 scale per 16 elements of K;
//          `kind::mxf4nvf4.block16`, 64 elements of K per instruction (four times the bf16 work per issue slot).
//   MXFP8  A, B E4M3, one power-of-two (UE8M0) scale per 32 elements of K; `kind::mxf8f6f4`, 32 elements of K per
//          instruction (twice the bf16 work per issue slot). Replaces the promotion of every 128-deep K block out
//          of TMEM that fp32 block scales need.
//
// Scale layout (global and shared memory alike): per block of 128 rows and per FOUR scale groups along K (64 elements
// for NVFP4, 128 for MXFP8), 512 bytes ordered
//   byte = (row % 32) * 16 + (row / 32) * 4 + (group % 4)
// i.e. 32 "rows" of 16 bytes; one `tcgen05.cp.32x128b.warpx4` copies such a block into 4 TMEM columns (replicated over
// the four lane quarters), where lane r % 32 holds in column (r / 32) the four scales of row r. NVFP4 consumes all four
// per instruction; MXFP8 one, chosen by the scale-id fields of the instruction descriptor. Blocks are stored
// [row block][k block], so the scales of one 128-row operand tile for one stage are contiguous: one bulk copy.
//
// Structure as the bf16 GEMM (gemm/tc_gemm.cu): persistent CTAs; warp 0 producer (TMA tiles of A and B, bulk copies of
// the scale blocks), warp 1 one-thread issuer (scale copies, MMAs, commits), warps 2-9 epilogue out of TMEM through the
// shared epilogue (alpha, bf16, TMA store). Two tile shapes: 128 x 128 with a double-buffered accumulator (the
// epilogue of tile i under the MMAs of tile i + 1; short reductions), and 128 x 256 with ONE accumulator (512 TMEM
// columns hold two such accumulators but then no scales): a stage then carries 48 KB for 512 clocks of tensor work
// instead of 32 KB for 256, which is what an operand-load-bound kernel needs, at the price of an exposed epilogue
// (a few per cent once K >= 2048). All waits are bounded.
//
// Replaces the reference's FP4 linear, which decodes the weights and calls a bf16 GEMM
// (triune/kernels/fast_nvfp4.py:243-342, 455-535), and its FP8 linear (triune/kernels/fast_fp8.py:28-106).
#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>

#include <stdexcept>
#include <string>

#include "../common/per_device.h"
#include "../common/ptx.cuh"
#include "../common/tma_desc.h"
#include "../gemm/tc_gemm_impl.cuh"
#include "quant.cuh"

namespace tb {

int nvfp4_sf_kblocks(int K) { return ((K + 255) / 256) * 4; }  // 512-byte blocks per 128 rows: whole stages of 256 elements
int mxfp8_sf_kblocks(int K) { return (K + 127) / 128; }        // one block per stage of 128 elements

namespace {

constexpr int FBM = 128;
constexpr int FBK_BYTES = 128;           // bytes of K per row and stage: 256 E2M1 or 128 E4M3 elements
constexpr int F_KB = 4;                  // MMAs per stage (32 bytes of K each)
constexpr int FA_BYTES = FBM * FBK_BYTES;
constexpr int F_TMEM_COLS = 512;

template <int BN, bool FP8>
struct BSCfg {
  static constexpr int STAGES = BN == 128 ? 4 : 3;
  static constexpr int ACC_BUFS = BN == 128 ? 2 : 1;
  static constexpr int B_BYTES = BN * FBK_BYTES;
  static constexpr int SF_BLOCKS = FP8 ? 1 : F_KB;           // 512-byte scale blocks per 128 rows and stage
  static constexpr int SFA_BYTES = SF_BLOCKS * 512;
  static constexpr int SFB_BYTES = (BN / 128) * SF_BLOCKS * 512;
  static constexpr int STAGE_BYTES = FA_BYTES + B_BYTES + SFA_BYTES + SFB_BYTES;
  static constexpr int SMEM = STAGES * STAGE_BYTES + 8 * EPI_TILE + 1024 + 256;
  static constexpr int COL_SFA = ACC_BUFS * BN;              // 256 either way
  static constexpr int COL_SFB = COL_SFA + 4 * SF_BLOCKS;
  static_assert(COL_SFB + 4 * SF_BLOCKS * (BN / 128) <= F_TMEM_COLS, "TMEM budget");
  static_assert(SMEM <= 227 * 1024, "shared memory budget");
};

__device__ __forceinline__ void bulk_load(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   smem_u32(smem_dst)),
               "l"(gsrc), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}
// Descriptor of a 32 x 16-byte block in shared memory without swizzle: 8-row groups are 128 bytes apart.
__device__ __forceinline__ uint64_t sf_desc(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3FFFF) >> 4);
  d |= (uint64_t)(16 >> 4) << 16;    // leading byte offset (one 16-byte column only)
  d |= (uint64_t)(128 >> 4) << 32;   // stride between 8-row groups
  d |= (uint64_t)1 << 46;            // descriptor version
  return d;                          // swizzle mode 0
}
__device__ __forceinline__ void tmem_cp_32x128b(uint32_t taddr, uint64_t desc) {
  asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(desc) : "memory");
}
// Instruction descriptor of the block-scaled kinds: [4,6) B scale id, [7,10) A format, [10,13) B format, [15] / [16]
// majors (K only), [17,23) N >> 3, [23] scale format (0 = UE4M3, 1 = UE8M0), [24,29) M >> 4, [29,31) A scale id,
// [31] K size (0 = 64 for the 4-bit kind, 32 for the 8-bit kind). Formats: E2M1 = 1 under kind::mxf4nvf4, E4M3 = 0
// under kind::mxf8f6f4. The scale ids pick the byte of the 32-bit TMEM scale column (one scale per instruction).
__host__ __device__ constexpr uint32_t make_idesc_nvfp4(uint32_t M, uint32_t N) {
  return (1u << 7) | (1u << 10) | ((N >> 3) << 17) | ((M >> 4) << 24);
}
__host__ __device__ constexpr uint32_t make_idesc_mxfp8(uint32_t M, uint32_t N, uint32_t sf_id) {
  return (sf_id << 4) | ((N >> 3) << 17) | (1u << 23) | ((M >> 4) << 24) | (sf_id << 29);
}
__device__ __forceinline__ void umma_nvfp4(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t tsfa,
                                           uint32_t tsfb, uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.block16 [%0], %1, %2, %3, [%5], [%6], p;\n\t"
      "}\n" ::"r"(tmem_d),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(tsfa), "r"(tsfb)
      : "memory");
}
__device__ __forceinline__ void umma_mxfp8(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t tsfa,
                                           uint32_t tsfb, uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale.scale_vec::1X [%0], %1, %2, %3, [%5], [%6], p;\n\t"
      "}\n" ::"r"(tmem_d),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(tsfa), "r"(tsfb)
      : "memory");
}

template <int BN, bool FP8, int EPI>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
    block_scaled_gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                             const __grid_constant__ CUtensorMap tmC, const uint8_t* __restrict__ sfa,
                             const uint8_t* __restrict__ sfb, const KParams p, int k_stages, int sf_kblocks) {
  using Cfg = BSCfg<BN, FP8>;
  constexpr int F_STAGES = Cfg::STAGES, FB_BYTES = Cfg::B_BYTES, ACC = Cfg::ACC_BUFS, SFB_ = Cfg::SF_BLOCKS;
  constexpr int F_STAGE_BYTES = Cfg::STAGE_BYTES, F_COL_SFA = Cfg::COL_SFA, F_COL_SFB = Cfg::COL_SFB;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  uint8_t* smem = smem_raw + (((raw + 1023u) & ~1023u) - raw);
  uint8_t* smemA = smem;
  uint8_t* smemB = smemA + F_STAGES * FA_BYTES;
  uint8_t* smemSFA = smemB + F_STAGES * FB_BYTES;
  uint8_t* smemSFB = smemSFA + F_STAGES * Cfg::SFA_BYTES;
  uint8_t* smem_epi = smemSFB + F_STAGES * Cfg::SFB_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem_epi + 8 * EPI_TILE);
  uint64_t* full = bars;
  uint64_t* empty = bars + F_STAGES;
  uint64_t* acc_full = bars + 2 * F_STAGES;
  uint64_t* acc_empty = acc_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  static_assert(ACC <= 2, "two accumulator barriers are laid out");
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < F_STAGES; ++s) {
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
    tmem_alloc(tmem_slot, F_TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0, issued = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < p.total_tiles && ok; t += gridDim.x) {
        int m_idx, n_idx;
        raster(t, p.num_m, p.num_n, p.group_m, m_idx, n_idx);
        for (int it = 0; it < k_stages; ++it) {
          if (!mbar_wait(&empty[stage], phase ^ 1)) {
            report(p, ST_TIMEOUT_EMPTY);
            ok = false;
            break;
          }
          mbar_expect_tx(&full[stage], F_STAGE_BYTES);
          tma_load_3d(smemA + stage * FA_BYTES, &tmA, &full[stage], it * FBK_BYTES, m_idx * FBM, 0);
          tma_load_3d(smemB + stage * FB_BYTES, &tmB, &full[stage], it * FBK_BYTES, n_idx * BN, 0);
          bulk_load(smemSFA + stage * Cfg::SFA_BYTES, sfa + ((long long)m_idx * sf_kblocks + it * SFB_) * 512,
                    Cfg::SFA_BYTES, &full[stage]);
#pragma unroll
          for (int h = 0; h < BN / 128; ++h)  // scale rows of the tile's 128-row halves (row blocks are sf_kblocks apart)
            bulk_load(smemSFB + stage * Cfg::SFB_BYTES + h * Cfg::SFA_BYTES,
                      sfb + ((long long)(n_idx * (BN / 128) + h) * sf_kblocks + it * SFB_) * 512, Cfg::SFA_BYTES,
                      &full[stage]);
          ++issued;
          if (++stage == F_STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
      if (!ok) {
        int pending = issued < F_STAGES ? issued : F_STAGES, s = stage;
        uint32_t ph = phase;
        for (int i = 0; i < pending; ++i) {
          if (--s < 0) {
            s = F_STAGES - 1;
            ph ^= 1;
          }
          (void)mbar_wait(&full[s], ph);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      int stage = 0, acc = 0;
      uint32_t phase = 0, acc_phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < p.total_tiles && ok; t += gridDim.x) {
        if (!mbar_wait(&acc_empty[acc], acc_phase ^ 1)) {
          report(p, ST_TIMEOUT_TMEM);
          break;
        }
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int it = 0; it < k_stages; ++it) {
          if (!mbar_wait(&full[stage], phase)) {
            report(p, ST_TIMEOUT_FULL);
            ok = false;
            break;
          }
          tc_fence_after_sync();
          const uint32_t a_addr = smem_u32(smemA + stage * FA_BYTES), b_addr = smem_u32(smemB + stage * FB_BYTES);
          const uint32_t sa = smem_u32(smemSFA + stage * Cfg::SFA_BYTES), sb = smem_u32(smemSFB + stage * Cfg::SFB_BYTES);
#pragma unroll
          for (int j = 0; j < SFB_; ++j) tmem_cp_32x128b(tmem_base + F_COL_SFA + 4 * j, sf_desc(sa + j * 512));
#pragma unroll
          for (int h = 0; h < BN / 128; ++h)
#pragma unroll
            for (int j = 0; j < SFB_; ++j)
              tmem_cp_32x128b(tmem_base + F_COL_SFB + 4 * (j * (BN / 128) + h), sf_desc(sb + (h * SFB_ + j) * 512));
#pragma unroll
          for (int kb = 0; kb < F_KB; ++kb) {
            const uint64_t ad = make_smem_desc(a_addr + kb * 32, 16, 1024), bd = make_smem_desc(b_addr + kb * 32, 16, 1024);
            const uint32_t accum = (it > 0 || kb > 0) ? 1u : 0u;
            if constexpr (FP8) {
              // the four scales of a stage share one TMEM column per 32 rows; the instruction takes byte kb of it
              umma_mxfp8(d_tmem, ad, bd, make_idesc_mxfp8(FBM, BN, kb), tmem_base + F_COL_SFA, tmem_base + F_COL_SFB, accum);
            } else {
              // N = 256: the two 128-row halves of B hold their scales for k block kb in columns 4 * (h * 4 + kb); the
              // instruction reads 8 consecutive columns from its scale address, so the halves are interleaved per kb
              umma_nvfp4(d_tmem, ad, bd, make_idesc_nvfp4(FBM, BN), tmem_base + F_COL_SFA + 4 * kb,
                         tmem_base + F_COL_SFB + 4 * kb * (BN / 128), accum);
            }
          }
          umma_commit(&empty[stage]);
          if (++stage == F_STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (!ok) break;
        umma_commit(&acc_full[acc]);
        if (++acc == ACC) {
          acc = 0;
          acc_phase ^= 1;
        }
      }
    }
  } else {
    const int lane_base = (warp & 3) * 32, col_half = (warp - 2) >> 2;
    uint8_t* my_stage = smem_epi + (warp - 2) * EPI_TILE;
    int acc = 0;
    uint32_t acc_phase = 0, buf = 0;
    for (int t = blockIdx.x; t < p.total_tiles; t += gridDim.x) {
      int m_idx, n_idx;
      raster(t, p.num_m, p.num_n, p.group_m, m_idx, n_idx);
      Tile tl;
      tl.valid = true;
      tl.m0 = m_idx * FBM;
      tl.n0 = n_idx;
      tl.ba = tl.bb = tl.g = 0;
      tl.k_begin = 0;
      tl.k_iters = k_stages;
      bool ok = mbar_wait(&acc_full[acc], acc_phase);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) {
        if (lane == 0) report(p, ST_TIMEOUT_TMEM);
        break;
      }
      tc_fence_after_sync();
      epilogue_tile<EPI>(p, tl, &tmC, &tmC, tmem_base + acc * BN, BN, n_idx * BN, tl.m0, lane_base, col_half, lane, my_stage, buf);
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[acc]);
      if (++acc == ACC) {
        acc = 0;
        acc_phase ^= 1;
      }
    }
    if (lane == 0) tma_store_wait<0>();
    __syncwarp();
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, F_TMEM_COLS);
  }
}

// Activation quantiser: x bf16 [M, K] -> packed E2M1 [M, K / 2] and unsigned E4M3 block scales in the blocked layout
// the GEMM loads. One thread per 16 elements; `hadamard` applies the 16-point Walsh-Hadamard rotation first (weights
// quantised with the same rotation then see x H (W H)^T = x W^T).
// Two floats -> one byte of E2M1 codes (round to nearest even, saturating), `lo` in the low nibble.
__device__ __forceinline__ uint32_t e2m1x2(float lo, float hi) {
  uint32_t r;
  asm("{\n\t"
      ".reg .b8 t;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 t, %1, %2;\n\t"
      "cvt.u32.u8 %0, t;\n\t"
      "}" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}
__device__ __forceinline__ uint32_t e2m1_code_f(float x) {
  // nearest representable magnitude of {0, .5, 1, 1.5, 2, 3, 4, 6}, ties to the even code
  const float a = fabsf(x);
  uint32_t c = a <= 0.25f ? 0u : a < 0.75f ? 1u : a <= 1.25f ? 2u : a < 1.75f ? 3u : a <= 2.5f ? 4u : a < 3.5f ? 5u : a <= 5.0f ? 6u : 7u;
  return c | (x < 0.f ? 8u : 0u);
}
__device__ __forceinline__ void fwht16_rot(float (&v)[16]) {
#pragma unroll
  for (int h = 1; h < 16; h <<= 1) {
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      if ((i & h) == 0) {
        const float a = v[i], b = v[i + h];
        v[i] = a + b;
        v[i + h] = a - b;
      }
    }
  }
#pragma unroll
  for (int i = 0; i < 16; ++i) v[i] *= 0.25f;
}

// One CTA pass covers ONE 512-byte scale block: 128 rows x 4 scale groups (64 elements of K). Thread pair (row, group)
// = (item / 4, item % 4): four neighbouring threads read 128 contiguous bytes of a row and write 32 contiguous bytes of
// codes; the block's scales are collected in shared memory in the blocked order and leave as one coalesced 512-byte
// store (written byte by byte from the threads they would be 4-byte fragments of 32-byte sectors).
__global__ void __launch_bounds__(256) nvfp4_quantize_act_kernel(const __nv_bfloat16* __restrict__ x, long long ld, int M,
                                                                 int K, int sf_kblocks, int hadamard,
                                                                 uint8_t* __restrict__ packed, uint8_t* __restrict__ sf) {
  __shared__ __align__(16) uint8_t s_sf[512];
  const int rb = blockIdx.x;
  const int groups = K >> 4;          // scale groups per row
  const int kblocks = (groups + 3) >> 2;
  for (int kb = blockIdx.y; kb < kblocks; kb += gridDim.y) {
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int item = threadIdx.x + h * 256;
      const int ri = item >> 2, g = item & 3;
      const int r = rb * 128 + ri, b = kb * 4 + g;
      uint8_t scb = 0;
      if (r < M && b < groups) {
        const uint4* src = reinterpret_cast<const uint4*>(x + (long long)r * ld + b * 16);
        const uint4 u0 = src[0], u1 = src[1];
        float v[16];
        const __nv_bfloat162* p0 = reinterpret_cast<const __nv_bfloat162*>(&u0);
        const __nv_bfloat162* p1 = reinterpret_cast<const __nv_bfloat162*>(&u1);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 f0 = __bfloat1622float2(p0[j]), f1 = __bfloat1622float2(p1[j]);
          v[2 * j] = f0.x; v[2 * j + 1] = f0.y;
          v[8 + 2 * j] = f1.x; v[8 + 2 * j + 1] = f1.y;
        }
        if (hadamard) fwht16_rot(v);
        float amax = 0.f;
#pragma unroll
        for (int j = 0; j < 16; ++j) amax = fmaxf(amax, fabsf(v[j]));
        // scale = amax / 6 rounded to E4M3 (at least the smallest subnormal, so a block of zeros keeps a finite scale)
        const __nv_fp8_storage_t sc = __nv_cvt_float_to_fp8(fminf(fmaxf(amax * (1.0f / 6.0f), 0.001953125f), 448.0f), __NV_SATFINITE, __NV_E4M3);
        const __half_raw hr = __nv_cvt_fp8_to_halfraw(sc, __NV_E4M3);
        const float inv = 1.0f / __half2float(*reinterpret_cast<const __half*>(&hr));
        uint32_t lo = 0, hi = 0;
#pragma unroll
        for (int j = 0; j < 4; ++j) lo |= e2m1x2(v[2 * j] * inv, v[2 * j + 1] * inv) << (8 * j);
#pragma unroll
        for (int j = 0; j < 4; ++j) hi |= e2m1x2(v[8 + 2 * j] * inv, v[9 + 2 * j] * inv) << (8 * j);
        *reinterpret_cast<uint2*>(packed + (long long)r * (K >> 1) + b * 8) = make_uint2(lo, hi);
        scb = (uint8_t)sc;
      }
      s_sf[(ri & 31) * 16 + (ri >> 5) * 4 + g] = scb;
    }
    __syncthreads();
    if (threadIdx.x < 32)
      reinterpret_cast<uint4*>(sf + ((long long)rb * sf_kblocks + kb) * 512)[threadIdx.x] = reinterpret_cast<const uint4*>(s_sf)[threadIdx.x];
    __syncthreads();
  }
}

// Row-major E4M3 scales [R, K / 16] -> the blocked layout (weights, once at conversion time).
__global__ void __launch_bounds__(256) nvfp4_block_scales_kernel(const uint8_t* __restrict__ s, int R, int kb16,
                                                                 int sf_kblocks, uint8_t* __restrict__ out) {
  const long long total = (long long)R * kb16;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int r = (int)(i / kb16), b = (int)(i % kb16);
    const int rb = r >> 7, ri = r & 127;
    out[((long long)rb * sf_kblocks + (b >> 2)) * 512 + (ri & 31) * 16 + (ri >> 5) * 4 + (b & 3)] = s[i];
  }
}

// MXFP8 quantiser: x bf16 [R, K] -> E4M3 [R, K] and one power-of-two (UE8M0) scale per 32 elements in the blocked
// layout (used for activations at run time and for weights at conversion time). The scale is the smallest power of
// two that brings the block's largest magnitude under the E4M3 maximum (448); E4M3 is a floating format, so a
// power-of-two scale costs no relative precision against amax / 448.
__global__ void __launch_bounds__(256) mxfp8_quantize_kernel(const __nv_bfloat16* __restrict__ x, long long ld, int R, int K,
                                                             int sf_kblocks, uint8_t* __restrict__ q, uint8_t* __restrict__ sf) {
  // same tiling as the NVFP4 quantiser: one pass = one 512-byte scale block = 128 rows x 4 groups of 32 elements
  __shared__ __align__(16) uint8_t s_sf[512];
  const int rb = blockIdx.x;
  const int groups = K >> 5;
  const int kblocks = (groups + 3) >> 2;
  for (int kb = blockIdx.y; kb < kblocks; kb += gridDim.y) {
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int item = threadIdx.x + h * 256;
      const int ri = item >> 2, g = item & 3;
      const int r = rb * 128 + ri, b = kb * 4 + g;
      uint8_t scb = 0;
      if (r < R && b < groups) {
        const uint4* src = reinterpret_cast<const uint4*>(x + (long long)r * ld + b * 32);
        uint4 u[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) u[j] = src[j];
        float v[32];
        float amax = 0.f;
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const float2 f = __bfloat1622float2(reinterpret_cast<const __nv_bfloat162*>(u)[j]);
          v[2 * j] = f.x;
          v[2 * j + 1] = f.y;
          amax = fmaxf(amax, fmaxf(fabsf(f.x), fabsf(f.y)));
        }
        // e = ceil(log2(amax / 448)) in integer arithmetic: amax = m * 2^ea with m in [1, 2) and 448 = 1.75 * 2^8, so
        // amax <= 448 * 2^e  <=>  e >= ea - 8 + (m > 1.75)
        int e = -127;
        if (amax > 0.f) {
          const uint32_t bits = __float_as_uint(amax);
          e = (int)((bits >> 23) & 0xFF) - 127 - 8 + ((bits & 0x7FFFFF) > 0x600000 ? 1 : 0);
          e = e < -127 ? -127 : (e > 127 ? 127 : e);
        }
        // 2^-e: the exponent field 127 - e is a normal number for e in [-127, 126]; e = 127 needs the denormal 2^-127
        const float mul = e == 127 ? 5.877471754111438e-39f : __uint_as_float((uint32_t)(127 - e) << 23);
        uint32_t w[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const uint32_t p0 = __nv_cvt_float2_to_fp8x2(make_float2(v[4 * j] * mul, v[4 * j + 1] * mul), __NV_SATFINITE, __NV_E4M3);
          const uint32_t p1 = __nv_cvt_float2_to_fp8x2(make_float2(v[4 * j + 2] * mul, v[4 * j + 3] * mul), __NV_SATFINITE, __NV_E4M3);
          w[j] = p0 | (p1 << 16);
        }
        uint4* dst = reinterpret_cast<uint4*>(q + (long long)r * K + b * 32);
        dst[0] = make_uint4(w[0], w[1], w[2], w[3]);
        dst[1] = make_uint4(w[4], w[5], w[6], w[7]);
        scb = (uint8_t)(e + 127);
      }
      s_sf[(ri & 31) * 16 + (ri >> 5) * 4 + g] = scb;
    }
    __syncthreads();
    if (threadIdx.x < 32)
      reinterpret_cast<uint4*>(sf + ((long long)rb * sf_kblocks + kb) * 512)[threadIdx.x] = reinterpret_cast<const uint4*>(s_sf)[threadIdx.x];
    __syncthreads();
  }
}

int sm_count_f() {
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

// grid: one CTA row per 128 rows, and as many CTAs along K as fill the GPU a few times over (each loops over k blocks)
static dim3 quant_grid(int rows, int kblocks) {
  const int rbs = (rows + 127) / 128;
  int ky = (148 * 8 + rbs - 1) / rbs;
  ky = ky < 1 ? 1 : (ky > kblocks ? kblocks : ky);
  return dim3((unsigned)rbs, (unsigned)ky, 1);
}

void launch_nvfp4_quantize_act(const __nv_bfloat16* x, long long ld, int M, int K, bool hadamard, uint8_t* packed,
                               uint8_t* sf_blocked, cudaStream_t s) {
  if (M <= 0) return;
  const int kblocks = ((K >> 4) + 3) / 4;
  nvfp4_quantize_act_kernel<<<quant_grid(M, kblocks), 256, 0, s>>>(x, ld, M, K, nvfp4_sf_kblocks(K), hadamard ? 1 : 0, packed, sf_blocked);
}

void launch_nvfp4_block_scales(const uint8_t* scales, int R, int K, uint8_t* out, cudaStream_t s) {
  if (R <= 0) return;
  const long long total = (long long)R * (K >> 4);
  long long blocks = (total + 255) / 256;
  if (blocks > 148ll * 16) blocks = 148ll * 16;
  nvfp4_block_scales_kernel<<<(int)blocks, 256, 0, s>>>(scales, R, K >> 4, nvfp4_sf_kblocks(K), out);
}

namespace {

template <int BN, bool FP8, int EPI>
void launch_block_scaled(const uint8_t* a, const uint8_t* sfa, const uint8_t* b, const uint8_t* sfb, __nv_bfloat16* C, int M,
                         int N, int K, float alpha, const __nv_bfloat16* bias, int* status, cudaStream_t s) {
  using Cfg = BSCfg<BN, FP8>;
  const int row_bytes = FP8 ? K : K / 2;
  KParams kp{};
  kp.M = M; kp.N = N; kp.K = K;
  kp.mode = GEMM_DENSE; kp.flags = 0; kp.batch = 1;
  kp.num_m = (M + FBM - 1) / FBM;
  kp.num_n = (N + BN - 1) / BN;
  kp.ldc = N; kp.strideC = 0;
  kp.alpha = alpha;
  kp.C = C;
  kp.bias = bias;  // bf16 [N], added after alpha (before the activation)
  kp.status = status;
  kp.total_tiles = kp.num_m * kp.num_n;
  kp.splits = 1;
  kp.group_m = raster_group_m(kp.num_m, kp.num_n, sm_count_f());
  const int k_stages = (row_bytes + FBK_BYTES - 1) / FBK_BYTES;
  const int sf_kblocks = FP8 ? mxfp8_sf_kblocks(K) : nvfp4_sf_kblocks(K);
  CUtensorMap tmA = make_tmap_3d(a, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, (uint64_t)row_bytes, (uint64_t)M, 1, (uint64_t)row_bytes,
                                 (uint64_t)row_bytes * (uint64_t)M, FBK_BYTES, FBM);
  CUtensorMap tmB = make_tmap_3d(b, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, (uint64_t)row_bytes, (uint64_t)N, 1, (uint64_t)row_bytes,
                                 (uint64_t)row_bytes * (uint64_t)N, FBK_BYTES, BN);
  CUtensorMap tmC = make_tmap_3d(C, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)N, (uint64_t)M, 1, (uint64_t)N * 2ull,
                                 (uint64_t)N * 2ull * (uint64_t)M, 32, 32);
  static PerDeviceOnce once;
  if (once.first_use()) {
    cudaError_t e = cudaFuncSetAttribute(block_scaled_gemm_kernel<BN, FP8, EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM);
    if (e != cudaSuccess) throw std::runtime_error(std::string("block_scaled_gemm: cannot set shared memory size: ") + cudaGetErrorString(e));
  }
  const int grid = kp.total_tiles < sm_count_f() ? kp.total_tiles : sm_count_f();
  block_scaled_gemm_kernel<BN, FP8, EPI><<<grid, GEMM_THREADS, Cfg::SMEM, s>>>(tmA, tmB, tmC, sfa, sfb, kp, k_stages, sf_kblocks);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) throw std::runtime_error(std::string("block_scaled_gemm launch failed: ") + cudaGetErrorString(e));
}

// The wide tile pays once the reduction is long enough to hide its exposed epilogue and there are enough tiles to fill
// the GPU; `tile_n` forces a shape (0 = choose).
bool wide_tile(int M, int N, int K_bytes, int tile_n) {
  if (tile_n == 128) return false;
  if (tile_n == 256) return true;
  const long long tiles256 = (long long)((M + 127) / 128) * ((N + 255) / 256);
  return K_bytes >= 1024 && N >= 256 && tiles256 >= sm_count_f();
}

}  // namespace

template <bool FP8>
void dispatch_block_scaled(const uint8_t* a, const uint8_t* sfa, const uint8_t* b, const uint8_t* sfb, __nv_bfloat16* C, int M,
                           int N, int K, int k_bytes, float alpha, const __nv_bfloat16* bias, bool gelu, int* status, int tile_n,
                           cudaStream_t s) {
  const bool wide = wide_tile(M, N, k_bytes, tile_n);
  if (gelu) {
    if (wide) launch_block_scaled<256, FP8, EPI_GELU>(a, sfa, b, sfb, C, M, N, K, alpha, bias, status, s);
    else launch_block_scaled<128, FP8, EPI_GELU>(a, sfa, b, sfb, C, M, N, K, alpha, bias, status, s);
  } else {
    if (wide) launch_block_scaled<256, FP8, EPI_PLAIN>(a, sfa, b, sfb, C, M, N, K, alpha, bias, status, s);
    else launch_block_scaled<128, FP8, EPI_PLAIN>(a, sfa, b, sfb, C, M, N, K, alpha, bias, status, s);
  }
}

void launch_nvfp4_gemm(const uint8_t* a_packed, const uint8_t* sfa, const uint8_t* b_packed, const uint8_t* sfb,
                       __nv_bfloat16* C, int M, int N, int K, float alpha, const __nv_bfloat16* bias, bool gelu, int* status,
                       int tile_n, cudaStream_t s) {
  if (M <= 0 || N <= 0) return;
  if (K % 32 != 0) throw std::runtime_error("nvfp4_gemm: K must be a multiple of 32 (16-byte rows of packed codes)");
  if (N % 8 != 0) throw std::runtime_error("nvfp4_gemm: N must be a multiple of 8");
  dispatch_block_scaled<false>(a_packed, sfa, b_packed, sfb, C, M, N, K, K / 2, alpha, bias, gelu, status, tile_n, s);
}

void launch_mxfp8_quantize(const __nv_bfloat16* x, long long ld, int R, int K, uint8_t* q, uint8_t* sf_blocked, cudaStream_t s) {
  if (R <= 0) return;
  if (K % 32 != 0) throw std::runtime_error("mxfp8_quantize: K must be a multiple of 32");
  const int kblocks = ((K >> 5) + 3) / 4;
  mxfp8_quantize_kernel<<<quant_grid(R, kblocks), 256, 0, s>>>(x, ld, R, K, mxfp8_sf_kblocks(K), q, sf_blocked);
}

void launch_mxfp8_gemm(const uint8_t* a, const uint8_t* sfa, const uint8_t* b, const uint8_t* sfb, __nv_bfloat16* C, int M,
                       int N, int K, float alpha, const __nv_bfloat16* bias, bool gelu, int* status, int tile_n, cudaStream_t s) {
  if (M <= 0 || N <= 0) return;
  if (K % 32 != 0) throw std::runtime_error("mxfp8_gemm: K must be a multiple of 32");
  if (N % 8 != 0) throw std::runtime_error("mxfp8_gemm: N must be a multiple of 8");
  dispatch_block_scaled<true>(a, sfa, b, sfb, C, M, N, K, K, alpha, bias, gelu, status, tile_n, s);
}

}  // namespace tb
