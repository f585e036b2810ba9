// Block-scaled NVFP4 GEMM on the 5th-generation tensor cores: C[M, N] (bf16) = alpha * (A .* SFA) (B .* SFB)^T with A, B
// packed E2M1 (two codes per byte, K contiguous) and one unsigned E4M3 scale per 16 elements of K. The scales are
// applied by the tensor core itself: `tcgen05.mma.kind::mxf4nvf4.block_scale` reads them from TMEM, where
// `tcgen05.cp` places them from shared memory, so no operand is ever decoded to bf16 and the K = 64 instruction does
// four times the work of a bf16 instruction per issue slot.
//
// Scale layout (global and shared memory alike): per block of 128 rows and per 64 elements of K, 512 bytes ordered
//   byte = (row % 32) * 16 + (row / 32) * 4 + (k / 16) % 4
// i.e. 32 "rows" of 16 bytes; one `tcgen05.cp.32x128b.warpx4` copies such a block into 4 TMEM columns (replicated over
// the four lane quarters), where lane r holds in column (r / 32) the four scales of row r. Blocks are stored
// [row block][k block], so the scales of a 128 x 256 stage are 2 KB contiguous and travel as one bulk copy.
//
// Structure as the bf16 GEMM (gemm/tc_gemm.cu): persistent CTAs; warp 0 producer (TMA tiles of A and B, bulk copies of
// the scale blocks), warp 1 one-thread issuer (scale copies, MMAs, commits), warps 2-9 epilogue out of a double-buffered
// TMEM accumulator through the shared epilogue (alpha, bf16, TMA store). All waits are bounded.
//
// Replaces the reference's FP4 linear, which decodes the weights and calls a bf16 GEMM
// (triune/kernels/fast_nvfp4.py:243-342, 455-535).
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

namespace {

constexpr int FBM = 128, FBN = 128;
constexpr int FBK_BYTES = 128;           // 256 E2M1 elements of K per stage
constexpr int F_KB = 4;                  // MMAs (64 elements of K each) per stage
constexpr int F_STAGES = 4;
constexpr int FA_BYTES = FBM * FBK_BYTES, FB_BYTES = FBN * FBK_BYTES;
constexpr int FSF_BYTES = F_KB * 512;    // scale blocks of one 128-row operand tile for one stage
constexpr int F_STAGE_BYTES = FA_BYTES + FB_BYTES + 2 * FSF_BYTES;
constexpr int F_SMEM = F_STAGES * F_STAGE_BYTES + 8 * EPI_TILE + 1024 + 256;
constexpr int F_TMEM_COLS = 512;         // 2 x 128 accumulator columns + 32 scale columns
constexpr int F_COL_SFA = 256, F_COL_SFB = 256 + 4 * F_KB;

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
// Instruction descriptor of the block-scaled kinds: [4,6) B scale id, [7,10) A format, [10,13) B format (E2M1 = 1 for
// kind::mxf4nvf4), [15] / [16] majors (K only), [17,23) N >> 3, [23] scale format (0 = UE4M3), [24,29) M >> 4,
// [29,31) A scale id, [31] K size (0 = 64).
__host__ __device__ constexpr uint32_t make_idesc_nvfp4(uint32_t M, uint32_t N) {
  return (1u << 7) | (1u << 10) | ((N >> 3) << 17) | ((M >> 4) << 24);
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

__global__ void __launch_bounds__(GEMM_THREADS, 1)
    nvfp4_gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                      const __grid_constant__ CUtensorMap tmC, const uint8_t* __restrict__ sfa,
                      const uint8_t* __restrict__ sfb, const KParams p, int k_stages, int sf_kblocks) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  uint8_t* smem = smem_raw + (((raw + 1023u) & ~1023u) - raw);
  uint8_t* smemA = smem;
  uint8_t* smemB = smemA + F_STAGES * FA_BYTES;
  uint8_t* smemSFA = smemB + F_STAGES * FB_BYTES;
  uint8_t* smemSFB = smemSFA + F_STAGES * FSF_BYTES;
  uint8_t* smem_epi = smemSFB + F_STAGES * FSF_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem_epi + 8 * EPI_TILE);
  uint64_t* full = bars;
  uint64_t* empty = bars + F_STAGES;
  uint64_t* acc_full = bars + 2 * F_STAGES;
  uint64_t* acc_empty = acc_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
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
          tma_load_3d(smemB + stage * FB_BYTES, &tmB, &full[stage], it * FBK_BYTES, n_idx * FBN, 0);
          bulk_load(smemSFA + stage * FSF_BYTES, sfa + ((long long)m_idx * sf_kblocks + it * F_KB) * 512, FSF_BYTES,
                    &full[stage]);
          bulk_load(smemSFB + stage * FSF_BYTES, sfb + ((long long)n_idx * sf_kblocks + it * F_KB) * 512, FSF_BYTES,
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
      constexpr uint32_t idesc = make_idesc_nvfp4(FBM, FBN);
      int stage = 0, acc = 0;
      uint32_t phase = 0, acc_phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < p.total_tiles && ok; t += gridDim.x) {
        if (!mbar_wait(&acc_empty[acc], acc_phase ^ 1)) {
          report(p, ST_TIMEOUT_TMEM);
          break;
        }
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * FBN;
        for (int it = 0; it < k_stages; ++it) {
          if (!mbar_wait(&full[stage], phase)) {
            report(p, ST_TIMEOUT_FULL);
            ok = false;
            break;
          }
          tc_fence_after_sync();
          const uint32_t a_addr = smem_u32(smemA + stage * FA_BYTES), b_addr = smem_u32(smemB + stage * FB_BYTES);
          const uint32_t sa = smem_u32(smemSFA + stage * FSF_BYTES), sb = smem_u32(smemSFB + stage * FSF_BYTES);
#pragma unroll
          for (int kb = 0; kb < F_KB; ++kb) {
            tmem_cp_32x128b(tmem_base + F_COL_SFA + 4 * kb, sf_desc(sa + kb * 512));
            tmem_cp_32x128b(tmem_base + F_COL_SFB + 4 * kb, sf_desc(sb + kb * 512));
          }
#pragma unroll
          for (int kb = 0; kb < F_KB; ++kb)
            umma_nvfp4(d_tmem, make_smem_desc(a_addr + kb * 32, 16, 1024), make_smem_desc(b_addr + kb * 32, 16, 1024), idesc,
                       tmem_base + F_COL_SFA + 4 * kb, tmem_base + F_COL_SFB + 4 * kb, (it > 0 || kb > 0) ? 1u : 0u);
          umma_commit(&empty[stage]);
          if (++stage == F_STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (!ok) break;
        umma_commit(&acc_full[acc]);
        if (++acc == 2) {
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
      epilogue_tile<EPI_PLAIN>(p, tl, &tmC, &tmC, tmem_base + acc * FBN, FBN, n_idx * FBN, tl.m0, lane_base, col_half, lane,
                               my_stage, buf);
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[acc]);
      if (++acc == 2) {
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

__global__ void __launch_bounds__(256) nvfp4_quantize_act_kernel(const __nv_bfloat16* __restrict__ x, long long ld, int M,
                                                                 int K, int sf_kblocks, int hadamard,
                                                                 uint8_t* __restrict__ packed, uint8_t* __restrict__ sf) {
  const int kb16 = K >> 4;
  const long long total = (long long)M * kb16;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int r = (int)(i / kb16), b = (int)(i % kb16);
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
    for (int j = 0; j < 8; ++j) lo |= e2m1_code_f(v[j] * inv) << (4 * j);
#pragma unroll
    for (int j = 0; j < 8; ++j) hi |= e2m1_code_f(v[8 + j] * inv) << (4 * j);
    *reinterpret_cast<uint2*>(packed + (long long)r * (K >> 1) + b * 8) = make_uint2(lo, hi);
    const int rb = r >> 7, ri = r & 127;
    sf[((long long)rb * sf_kblocks + (b >> 2)) * 512 + (ri & 31) * 16 + (ri >> 5) * 4 + (b & 3)] = (uint8_t)sc;
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

int nvfp4_sf_kblocks(int K) { return ((K + 255) / 256) * 4; }

void launch_nvfp4_quantize_act(const __nv_bfloat16* x, long long ld, int M, int K, bool hadamard, uint8_t* packed,
                               uint8_t* sf_blocked, cudaStream_t s) {
  if (M <= 0) return;
  const long long total = (long long)M * (K >> 4);
  long long blocks = (total + 255) / 256;
  if (blocks > 148ll * 16) blocks = 148ll * 16;
  nvfp4_quantize_act_kernel<<<(int)blocks, 256, 0, s>>>(x, ld, M, K, nvfp4_sf_kblocks(K), hadamard ? 1 : 0, packed, sf_blocked);
}

void launch_nvfp4_block_scales(const uint8_t* scales, int R, int K, uint8_t* out, cudaStream_t s) {
  if (R <= 0) return;
  const long long total = (long long)R * (K >> 4);
  long long blocks = (total + 255) / 256;
  if (blocks > 148ll * 16) blocks = 148ll * 16;
  nvfp4_block_scales_kernel<<<(int)blocks, 256, 0, s>>>(scales, R, K >> 4, nvfp4_sf_kblocks(K), out);
}

void launch_nvfp4_gemm(const uint8_t* a_packed, const uint8_t* sfa, const uint8_t* b_packed, const uint8_t* sfb,
                       __nv_bfloat16* C, int M, int N, int K, float alpha, int* status, cudaStream_t s) {
  if (M <= 0 || N <= 0) return;
  if (K % 32 != 0) throw std::runtime_error("nvfp4_gemm: K must be a multiple of 32 (16-byte rows of packed codes)");
  if (N % 8 != 0) throw std::runtime_error("nvfp4_gemm: N must be a multiple of 8");
  KParams kp{};
  kp.M = M; kp.N = N; kp.K = K;
  kp.mode = GEMM_DENSE; kp.flags = 0; kp.batch = 1;
  kp.num_m = (M + FBM - 1) / FBM;
  kp.num_n = (N + FBN - 1) / FBN;
  kp.ldc = N; kp.strideC = 0;
  kp.alpha = alpha;
  kp.C = C;
  kp.status = status;
  kp.total_tiles = kp.num_m * kp.num_n;
  kp.splits = 1;
  kp.group_m = raster_group_m(kp.num_m, kp.num_n, sm_count_f());
  const int k_stages = (K / 2 + FBK_BYTES - 1) / FBK_BYTES;
  CUtensorMap tmA = make_tmap_3d(a_packed, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, (uint64_t)K / 2, (uint64_t)M, 1, (uint64_t)K / 2,
                                 (uint64_t)K / 2 * (uint64_t)M, FBK_BYTES, FBM);
  CUtensorMap tmB = make_tmap_3d(b_packed, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, (uint64_t)K / 2, (uint64_t)N, 1, (uint64_t)K / 2,
                                 (uint64_t)K / 2 * (uint64_t)N, FBK_BYTES, FBN);
  CUtensorMap tmC = make_tmap_3d(C, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)N, (uint64_t)M, 1, (uint64_t)N * 2ull,
                                 (uint64_t)N * 2ull * (uint64_t)M, 32, 32);
  static PerDeviceOnce once;
  if (once.first_use()) {
    cudaError_t e = cudaFuncSetAttribute(nvfp4_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, F_SMEM);
    if (e != cudaSuccess) throw std::runtime_error(std::string("nvfp4_gemm: cannot set shared memory size: ") + cudaGetErrorString(e));
  }
  const int grid = kp.total_tiles < sm_count_f() ? kp.total_tiles : sm_count_f();
  nvfp4_gemm_kernel<<<grid, GEMM_THREADS, F_SMEM, s>>>(tmA, tmB, tmC, sfa, sfb, kp, k_stages, nvfp4_sf_kblocks(K));
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) throw std::runtime_error(std::string("nvfp4_gemm launch failed: ") + cudaGetErrorString(e));
}

}  // namespace tb
