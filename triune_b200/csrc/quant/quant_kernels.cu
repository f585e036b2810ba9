// Quantised serving kernels for sm_100a.
//
//  * fp8_quantize_act_kernel   bf16 [M,K] -> E4M3 [M,K] + one fp32 scale per 1x128 row segment.
//  * fp8_block_gemm_kernel     C[M,N] = sum_kb xs[m,kb] * ws[n/128,kb] * (Xq[m,kb] . Wq[n,kb]); persistent,
//                              warp-specialised: TMA producer, one-thread tcgen05 `kind::f8f6f4` issuer, 8 epilogue
//                              warps. Every 128-deep K block is multiplied into its own TMEM buffer (two buffers
//                              alternate) and promoted into fp32 registers with the product of its two scales, so
//                              the tensor core never sees a scale and the accumulation across blocks is fp32.
//  * nvfp4_* kernels           E2M1 codes (two per byte) + one E4M3 (or bf16) scale per 16 elements + fp32 tensor
//                              scale: quantise (optional folded 16-point Hadamard rotation), dequantise to bf16, and a
//                              small-M GEMV that streams the packed weights once (decode path, bandwidth-bound).
//
// Every mbarrier wait is bounded; on expiry a status word is written and the CTA frees its TMEM and returns.
#include <cuda_fp8.h>

#include <stdexcept>
#include <string>

#include "../common/per_device.h"
#include "../common/ptx.cuh"
#include "../common/tma_desc.h"
#include "quant.cuh"

namespace tb {
namespace {

constexpr int QBM = 128, QBN = 128, QBK = 128;  // one stage = one 128x128 scale block of each operand
constexpr int QSTAGES = 4;
constexpr int QA_BYTES = QBM * QBK, QB_BYTES = QBN * QBK, QSTAGE_BYTES = QA_BYTES + QB_BYTES;
constexpr int Q_THREADS = 320;  // warp 0 TMA, warp 1 MMA + TMEM owner, warps 2..9 epilogue
constexpr int Q_SMEM = QSTAGES * QSTAGE_BYTES + 1024 + 256;

__device__ __forceinline__ uint8_t to_e4m3(float x) {
  return (uint8_t)__nv_cvt_float_to_fp8(x, __NV_SATFINITE, __NV_E4M3);
}
__device__ __forceinline__ float from_e4m3(uint8_t b) {
  __half_raw h = __nv_cvt_fp8_to_halfraw((__nv_fp8_storage_t)b, __NV_E4M3);
  return __half2float(*reinterpret_cast<__half*>(&h));
}

// ---------------------------------------------------------------------------------------------------------
// Activation quantiser: one warp per 1x128 segment, 4 elements per lane.
// ---------------------------------------------------------------------------------------------------------
__global__ void fp8_quantize_act_kernel(const __nv_bfloat16* __restrict__ x, uint8_t* __restrict__ q,
                                        float* __restrict__ scales, int M, int K, int KB) {
  const long long seg = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (seg >= (long long)M * KB) return;
  const int lane = threadIdx.x & 31;
  const int row = (int)(seg / KB), kb = (int)(seg % KB);
  const int k = kb * 128 + lane * 4;
  float v[4] = {0.f, 0.f, 0.f, 0.f};
  if (k + 3 < K) {
    const uint2 raw = *reinterpret_cast<const uint2*>(x + (long long)row * K + k);
    const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&raw.x);
    const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
    v[0] = __low2float(a); v[1] = __high2float(a); v[2] = __low2float(b); v[3] = __high2float(b);
  } else {
    for (int i = 0; i < 4; ++i)
      if (k + i < K) v[i] = __bfloat162float(x[(long long)row * K + k + i]);
  }
  float amax = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  const float scale = fmaxf(amax, 1e-12f) / 448.0f;
  const float inv = 1.0f / scale;
  if (lane == 0) scales[seg] = scale;
  if (k + 3 < K) {
    uint32_t packed = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) packed |= (uint32_t)to_e4m3(v[i] * inv) << (8 * i);
    *reinterpret_cast<uint32_t*>(q + (long long)row * K + k) = packed;
  } else {
    for (int i = 0; i < 4; ++i)
      if (k + i < K) q[(long long)row * K + k + i] = to_e4m3(v[i] * inv);
  }
}

// ---------------------------------------------------------------------------------------------------------
// Block-scaled FP8 GEMM
// ---------------------------------------------------------------------------------------------------------
struct Fp8Params {
  int M, N, K, KB;      // KB = ceil(K / 128)
  int num_m, num_n;
  const float* xs;      // [M, KB]
  const float* ws;      // [ceil(N/128), KB]
  __nv_bfloat16* C;     // [M, N]
  int* status;
};

__global__ void __launch_bounds__(Q_THREADS, 1)
    fp8_block_gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                          const Fp8Params p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  uint8_t* smem = smem_raw + (((raw + 1023u) & ~1023u) - raw);
  uint8_t* smemA = smem;
  uint8_t* smemB = smem + QSTAGES * QA_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + QSTAGES * QSTAGE_BYTES);
  uint64_t* full = bars;
  uint64_t* empty = bars + QSTAGES;
  uint64_t* acc_full = bars + 2 * QSTAGES;
  uint64_t* acc_empty = acc_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int s = 0; s < QSTAGES; ++s) {
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
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 256);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  const int total_tiles = p.num_m * p.num_n;

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0, issued = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
        const int m0 = (t / p.num_n) * QBM, n0 = (t % p.num_n) * QBN;
        for (int kb = 0; kb < p.KB; ++kb) {
          if (!mbar_wait(&empty[stage], phase ^ 1)) {
            if (p.status) atomicExch(p.status, 1);
            ok = false;
            break;
          }
          mbar_expect_tx(&full[stage], QSTAGE_BYTES);
          tma_load_3d(smemA + stage * QA_BYTES, &tmA, &full[stage], kb * QBK, m0, 0);
          tma_load_3d(smemB + stage * QB_BYTES, &tmB, &full[stage], kb * QBK, n0, 0);
          ++issued;
          if (++stage == QSTAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
      if (!ok) {
        int pending = issued < QSTAGES ? issued : QSTAGES, s = stage;
        uint32_t ph = phase;
        for (int i = 0; i < pending; ++i) {
          if (--s < 0) {
            s = QSTAGES - 1;
            ph ^= 1;
          }
          (void)mbar_wait(&full[s], ph);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc(QBM, QBN, 0, 0, 0, 0);  // E4M3 x E4M3 -> fp32, both K-major
      int stage = 0, acc = 0;
      uint32_t phase = 0, acc_phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
        for (int kb = 0; kb < p.KB; ++kb) {
          if (!mbar_wait(&acc_empty[acc], acc_phase ^ 1) || !mbar_wait(&full[stage], phase)) {
            if (p.status) atomicExch(p.status, 2);
            ok = false;
            break;
          }
          tc_fence_after_sync();
          const uint32_t a_addr = smem_u32(smemA + stage * QA_BYTES);
          const uint32_t b_addr = smem_u32(smemB + stage * QB_BYTES);
          const uint32_t d_tmem = tmem_base + acc * QBN;
#pragma unroll
          for (int k = 0; k < QBK / 32; ++k)
            umma_fp8(d_tmem, make_smem_desc(a_addr + k * 32, 16, 1024), make_smem_desc(b_addr + k * 32, 16, 1024), idesc,
                     k > 0 ? 1u : 0u);
          umma_commit(&empty[stage]);
          umma_commit(&acc_full[acc]);
          if (++stage == QSTAGES) {
            stage = 0;
            phase ^= 1;
          }
          if (++acc == 2) {
            acc = 0;
            acc_phase ^= 1;
          }
        }
      }
    }
  } else {
    // Epilogue warp e = warp - 2: TMEM lane quarter (warp % 4), column half e / 4; one output row per thread,
    // 64 fp32 running sums in registers.
    const int e = warp - 2;
    const int lane_base = (warp & 3) * 32;
    const int col_base = (e >> 2) * 64;
    int acc = 0;
    uint32_t acc_phase = 0;
    bool alive = true;
    for (int t = blockIdx.x; t < total_tiles && alive; t += gridDim.x) {
      const int m0 = (t / p.num_n) * QBM, nb = t % p.num_n, n0 = nb * QBN;
      const int gm = m0 + lane_base + lane;
      const bool row_ok = gm < p.M;
      float sum[64];
#pragma unroll
      for (int i = 0; i < 64; ++i) sum[i] = 0.f;
      for (int kb = 0; kb < p.KB; ++kb) {
        bool ok = mbar_wait(&acc_full[acc], acc_phase);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) {
          if (lane == 0 && p.status) atomicExch(p.status, 3);
          alive = false;
          break;
        }
        tc_fence_after_sync();
        const float s = (row_ok ? p.xs[(long long)gm * p.KB + kb] : 0.f) * p.ws[(long long)nb * p.KB + kb];
        const uint32_t taddr = tmem_base + ((uint32_t)lane_base << 16) + acc * QBN + col_base;
        uint32_t r[32];
        tmem_ld_32x32b_x32(taddr, r);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) sum[i] = fmaf(s, __uint_as_float(r[i]), sum[i]);
        tmem_ld_32x32b_x32(taddr + 32, r);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) sum[32 + i] = fmaf(s, __uint_as_float(r[i]), sum[32 + i]);
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(&acc_empty[acc]);
        if (++acc == 2) {
          acc = 0;
          acc_phase ^= 1;
        }
      }
      if (!alive) break;
      if (row_ok) {
        __nv_bfloat16* crow = p.C + (long long)gm * p.N + n0 + col_base;
#pragma unroll
        for (int g = 0; g < 8; ++g) {
          if (n0 + col_base + g * 8 < p.N) {
            uint4 o;
            o.x = pack_bf16x2(sum[g * 8 + 0], sum[g * 8 + 1]);
            o.y = pack_bf16x2(sum[g * 8 + 2], sum[g * 8 + 3]);
            o.z = pack_bf16x2(sum[g * 8 + 4], sum[g * 8 + 5]);
            o.w = pack_bf16x2(sum[g * 8 + 6], sum[g * 8 + 7]);
            *reinterpret_cast<uint4*>(crow + g * 8) = o;
          }
        }
      }
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 256);
  }
}

// ---------------------------------------------------------------------------------------------------------
// NVFP4
// ---------------------------------------------------------------------------------------------------------
__device__ __forceinline__ void fwht16_inplace(float (&v)[16]) {
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

__device__ __forceinline__ float e2m1_value(uint32_t code) {
  // magnitudes 0, .5, 1, 1.5, 2, 3, 4, 6 packed as halves of the value times two in a 32-bit table: 0,1,2,3,4,6,8,12
  const uint32_t m = code & 7u;
  const float mag = (float)((0xC8643210u >> (4 * m)) & 0xFu) * 0.5f;
  return (code & 8u) ? -mag : mag;
}

__device__ __forceinline__ uint32_t e2m1_code(float x) {
  const float a = fabsf(x);
  uint32_t idx = (a > 0.25f) + (a > 0.75f) + (a > 1.25f) + (a > 1.75f) + (a > 2.5f) + (a > 3.5f) + (a > 5.0f);
  return idx | (x < 0.f ? 8u : 0u);
}

template <typename T>
__device__ __forceinline__ void load16(const T* src, float (&v)[16]);
template <>
__device__ __forceinline__ void load16<__nv_bfloat16>(const __nv_bfloat16* src, float (&v)[16]) {
  const uint4 a = reinterpret_cast<const uint4*>(src)[0], b = reinterpret_cast<const uint4*>(src)[1];
  const uint32_t w[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    v[2 * i] = __uint_as_float(w[i] << 16);
    v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
  }
}
template <>
__device__ __forceinline__ void load16<float>(const float* src, float (&v)[16]) {
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float4 f = reinterpret_cast<const float4*>(src)[i];
    v[4 * i] = f.x; v[4 * i + 1] = f.y; v[4 * i + 2] = f.z; v[4 * i + 3] = f.w;
  }
}

// ---------------------------------------------------------------------------------------------------------
// GGML block formats (GGUF files): random-access decode of element i of a block.
// ---------------------------------------------------------------------------------------------------------
enum GgmlType : int { GGML_F32 = 0, GGML_F16 = 1, GGML_Q4_0 = 2, GGML_Q4_1 = 3, GGML_Q5_0 = 6, GGML_Q8_0 = 8, GGML_Q4_K = 12,
                      GGML_Q5_K = 13, GGML_Q6_K = 14, GGML_BF16 = 30 };

__host__ __device__ inline int ggml_block_elems(int t) {
  return (t == GGML_Q4_K || t == GGML_Q5_K || t == GGML_Q6_K) ? 256 : ((t == GGML_F32 || t == GGML_F16 || t == GGML_BF16) ? 1 : 32);
}
__host__ __device__ inline int ggml_block_bytes(int t) {
  switch (t) {
    case GGML_F32: return 4;
    case GGML_F16: case GGML_BF16: return 2;
    case GGML_Q4_0: return 18;
    case GGML_Q4_1: return 20;
    case GGML_Q5_0: return 22;
    case GGML_Q8_0: return 34;
    case GGML_Q4_K: return 144;
    case GGML_Q5_K: return 176;
    case GGML_Q6_K: return 210;
    default: return 0;
  }
}

__device__ __forceinline__ float ld_half(const uint8_t* p) {  // blocks are only 2-byte aligned
  const unsigned short h = (unsigned short)p[0] | ((unsigned short)p[1] << 8);
  return __half2float(__ushort_as_half(h));
}

__device__ __forceinline__ void k4_scale_min(const uint8_t* q, int j, float& sc, float& mn) {
  if (j < 4) {
    sc = (float)(q[j] & 63);
    mn = (float)(q[j + 4] & 63);
  } else {
    sc = (float)((q[j + 4] & 0xF) | ((q[j - 4] >> 6) << 4));
    mn = (float)((q[j + 4] >> 4) | ((q[j] >> 6) << 4));
  }
}

__device__ __forceinline__ float ggml_elem(const uint8_t* blk, int type, int i) {
  switch (type) {
    case GGML_F32: return *reinterpret_cast<const float*>(blk);
    case GGML_F16: return ld_half(blk);
    case GGML_BF16: return __uint_as_float(((unsigned int)blk[0] | ((unsigned int)blk[1] << 8)) << 16);
    case GGML_Q4_0: {
      const uint8_t* qs = blk + 2;
      const int q = i < 16 ? (qs[i] & 0xF) : (qs[i - 16] >> 4);
      return ld_half(blk) * (float)(q - 8);
    }
    case GGML_Q4_1: {
      const uint8_t* qs = blk + 4;
      const int q = i < 16 ? (qs[i] & 0xF) : (qs[i - 16] >> 4);
      return ld_half(blk) * (float)q + ld_half(blk + 2);
    }
    case GGML_Q5_0: {
      const unsigned int qh = (unsigned int)blk[2] | ((unsigned int)blk[3] << 8) | ((unsigned int)blk[4] << 16) | ((unsigned int)blk[5] << 24);
      const uint8_t* qs = blk + 6;
      const int lo = i < 16 ? (qs[i] & 0xF) : (qs[i - 16] >> 4);
      return ld_half(blk) * (float)((lo | (int)(((qh >> i) & 1u) << 4)) - 16);
    }
    case GGML_Q8_0: return ld_half(blk) * (float)reinterpret_cast<const int8_t*>(blk + 2)[i];
    case GGML_Q4_K:
    case GGML_Q5_K: {
      const float d = ld_half(blk), dmin = ld_half(blk + 2);
      const uint8_t* scales = blk + 4;
      const int g = i >> 6, half = (i >> 5) & 1, l = i & 31;
      float sc, mn;
      k4_scale_min(scales, 2 * g + half, sc, mn);
      int q;
      if (type == GGML_Q4_K) {
        const uint8_t b = blk[16 + 32 * g + l];
        q = half ? (b >> 4) : (b & 0xF);
      } else {
        const uint8_t hb = blk[16 + l];
        const uint8_t b = blk[48 + 32 * g + l];
        q = (half ? (b >> 4) : (b & 0xF)) + (((hb >> (2 * g + half)) & 1) << 4);
      }
      return d * sc * (float)q - dmin * mn;
    }
    case GGML_Q6_K: {
      const int n = i >> 7, r = i & 127, quarter = r >> 5, l = r & 31;
      const uint8_t* ql = blk + 64 * n;
      const uint8_t* qh = blk + 128 + 32 * n;
      const int8_t* sc = reinterpret_cast<const int8_t*>(blk + 192) + 8 * n;
      const float d = ld_half(blk + 208);
      const uint8_t lo = (quarter & 1) ? ql[l + 32] : ql[l];
      const int q = ((quarter < 2 ? (lo & 0xF) : (lo >> 4)) | (((qh[l] >> (2 * quarter)) & 3) << 4)) - 32;
      return d * (float)sc[(l >> 4) + 2 * quarter] * (float)q;
    }
    default: return 0.f;
  }
}

// Sources of 16 consecutive values for the NVFP4 quantiser: plain arrays or GGML blocks decoded on the fly.
template <typename T>
struct ArraySrc {
  const T* p;
  __device__ __forceinline__ void load(long long b, float (&v)[16]) const { load16<T>(p + b * 16, v); }
};
struct GgmlSrc {
  const uint8_t* raw;
  int type, elems, bytes;
  __device__ __forceinline__ void load(long long b, float (&v)[16]) const {
    const long long e0 = b * 16;
    const uint8_t* blk = raw + (e0 / elems) * bytes;
    const int i0 = (int)(e0 % elems);
    if (elems == 1) {
#pragma unroll
      for (int i = 0; i < 16; ++i) v[i] = ggml_elem(raw + (e0 + i) * bytes, type, 0);
    } else {
#pragma unroll
      for (int i = 0; i < 16; ++i) v[i] = ggml_elem(blk, type, i0 + i);  // 16 divides 32 and 256: never crosses a block
    }
  }
};

__global__ void ggml_dequant_kernel(GgmlSrc src, long long n, __nv_bfloat16* __restrict__ out) {
  for (long long g = (long long)blockIdx.x * blockDim.x + threadIdx.x; g * 8 < n; g += (long long)gridDim.x * blockDim.x) {
    const long long e0 = g * 8;
    float v[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const long long e = e0 + i;
      v[i] = e < n ? ggml_elem(src.raw + (e / src.elems) * src.bytes, src.type, (int)(e % src.elems)) : 0.f;
    }
    if (e0 + 8 <= n) {
      *reinterpret_cast<uint4*>(out + e0) = make_uint4(pack_bf16x2(v[0], v[1]), pack_bf16x2(v[2], v[3]), pack_bf16x2(v[4], v[5]),
                                                      pack_bf16x2(v[6], v[7]));
    } else {
      for (int i = 0; e0 + i < n; ++i) out[e0 + i] = __float2bfloat16(v[i]);
    }
  }
}

// pass 1: global max of |x| (after the optional rotation), as the bit pattern of a non-negative float
template <typename Src>
__global__ void nvfp4_amax_kernel(Src w, long long nblocks, int hadamard, unsigned int* gmax_bits) {
  float m = 0.f;
  for (long long b = (long long)blockIdx.x * blockDim.x + threadIdx.x; b < nblocks; b += (long long)gridDim.x * blockDim.x) {
    float v[16];
    w.load(b, v);
    if (hadamard) fwht16_inplace(v);
#pragma unroll
    for (int i = 0; i < 16; ++i) m = fmaxf(m, fabsf(v[i]));
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
  if ((threadIdx.x & 31) == 0) atomicMax(gmax_bits, __float_as_uint(m));
}

// pass 2: codes + block scales
template <typename Src>
__global__ void nvfp4_quantize_kernel(Src w, long long nblocks, int hadamard,
                                      const unsigned int* __restrict__ gmax_bits, uint8_t* __restrict__ packed,
                                      uint8_t* __restrict__ scales, float* __restrict__ tscale_out) {
  const float tscale = fmaxf(__uint_as_float(*gmax_bits) / (6.0f * 448.0f), 1e-12f);
  if (blockIdx.x == 0 && threadIdx.x == 0) *tscale_out = tscale;
  for (long long b = (long long)blockIdx.x * blockDim.x + threadIdx.x; b < nblocks; b += (long long)gridDim.x * blockDim.x) {
    float v[16];
    w.load(b, v);
    if (hadamard) fwht16_inplace(v);
    float amax = 0.f;
#pragma unroll
    for (int i = 0; i < 16; ++i) amax = fmaxf(amax, fabsf(v[i]));
    const float sc_f = fminf(fmaxf(amax / 6.0f / tscale, 0.001953125f), 448.0f);
    const uint8_t sc = to_e4m3(sc_f);
    scales[b] = sc;
    const float inv = 1.0f / (from_e4m3(sc) * tscale);
    uint32_t lo = 0, hi = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) lo |= e2m1_code(v[i] * inv) << (4 * i);
#pragma unroll
    for (int i = 0; i < 8; ++i) hi |= e2m1_code(v[8 + i] * inv) << (4 * i);
    *reinterpret_cast<uint2*>(packed + b * 8) = make_uint2(lo, hi);
  }
}

__device__ __forceinline__ float load_scale(const void* scales, long long b, int scale_bf16) {
  if (scale_bf16) return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(scales)[b]);
  return from_e4m3(reinterpret_cast<const uint8_t*>(scales)[b]);
}

__global__ void nvfp4_dequant_kernel(const uint8_t* __restrict__ packed, const void* __restrict__ scales, int scale_bf16,
                                     const float* __restrict__ tscale, long long nblocks, __nv_bfloat16* __restrict__ out) {
  const float ts = *tscale;
  for (long long b = (long long)blockIdx.x * blockDim.x + threadIdx.x; b < nblocks; b += (long long)gridDim.x * blockDim.x) {
    const uint2 c = *reinterpret_cast<const uint2*>(packed + b * 8);
    const float eff = load_scale(scales, b, scale_bf16) * ts;
    uint32_t o[8];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      o[i] = pack_bf16x2(e2m1_value(c.x >> (8 * i)) * eff, e2m1_value(c.x >> (8 * i + 4)) * eff);
      o[4 + i] = pack_bf16x2(e2m1_value(c.y >> (8 * i)) * eff, e2m1_value(c.y >> (8 * i + 4)) * eff);
    }
    uint4* dst = reinterpret_cast<uint4*>(out + b * 16);
    dst[0] = make_uint4(o[0], o[1], o[2], o[3]);
    dst[1] = make_uint4(o[4], o[5], o[6], o[7]);
  }
}

// y[m, n] = sum_k x[m, k] * W[n, k] for m < M <= 8. One warp per output column n; lanes stride over the 16-element
// blocks of the row, so each packed byte is read exactly once from HBM.
constexpr int GEMV_MAX_M = 8;
__global__ void nvfp4_gemv_kernel(const __nv_bfloat16* __restrict__ x, const uint8_t* __restrict__ packed,
                                  const void* __restrict__ scales, int scale_bf16, const float* __restrict__ tscale,
                                  __nv_bfloat16* __restrict__ y, int M, int N, int K) {
  const int n = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (n >= N) return;
  const int lane = threadIdx.x & 31;
  const int kblocks = K >> 4;
  float acc[GEMV_MAX_M];
#pragma unroll
  for (int m = 0; m < GEMV_MAX_M; ++m) acc[m] = 0.f;
  for (int kb = lane; kb < kblocks; kb += 32) {
    const long long b = (long long)n * kblocks + kb;
    const uint2 c = *reinterpret_cast<const uint2*>(packed + b * 8);
    const float sc = load_scale(scales, b, scale_bf16);
    float wv[16];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      wv[2 * i] = e2m1_value(c.x >> (8 * i));
      wv[2 * i + 1] = e2m1_value(c.x >> (8 * i + 4));
      wv[8 + 2 * i] = e2m1_value(c.y >> (8 * i));
      wv[8 + 2 * i + 1] = e2m1_value(c.y >> (8 * i + 4));
    }
#pragma unroll
    for (int m = 0; m < GEMV_MAX_M; ++m) {
      if (m < M) {
        float xv[16];
        load16<__nv_bfloat16>(x + (long long)m * K + kb * 16, xv);
        float d = 0.f;
#pragma unroll
        for (int i = 0; i < 16; ++i) d = fmaf(xv[i], wv[i], d);
        acc[m] = fmaf(d, sc, acc[m]);
      }
    }
  }
  const float ts = *tscale;
#pragma unroll
  for (int m = 0; m < GEMV_MAX_M; ++m) {
    float a = acc[m];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) a += __shfl_xor_sync(0xffffffffu, a, o);
    if (lane == 0 && m < M) y[(long long)m * N + n] = __float2bfloat16(a * ts);
  }
}

__global__ void fwht16_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ out, long long nblocks) {
  for (long long b = (long long)blockIdx.x * blockDim.x + threadIdx.x; b < nblocks; b += (long long)gridDim.x * blockDim.x) {
    float v[16];
    load16<__nv_bfloat16>(x + b * 16, v);
    fwht16_inplace(v);
    uint32_t o[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) o[i] = pack_bf16x2(v[2 * i], v[2 * i + 1]);
    uint4* dst = reinterpret_cast<uint4*>(out + b * 16);
    dst[0] = make_uint4(o[0], o[1], o[2], o[3]);
    dst[1] = make_uint4(o[4], o[5], o[6], o[7]);
  }
}

inline int grid_for(long long work, int per_block) {
  long long g = (work + per_block - 1) / per_block;
  if (g < 1) g = 1;
  if (g > 148 * 16) g = 148 * 16;
  return (int)g;
}
inline void check_launch(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) throw std::runtime_error(std::string(what) + " launch failed: " + cudaGetErrorString(e));
}

}  // namespace

void launch_fp8_quantize_act(const __nv_bfloat16* x, uint8_t* q, float* scales, int M, int K, cudaStream_t s) {
  if (M <= 0 || K <= 0) return;
  if (K % 4 != 0) throw std::runtime_error("fp8_quantize_act: K must be a multiple of 4");
  const int KB = (K + 127) / 128;
  const long long segs = (long long)M * KB;
  fp8_quantize_act_kernel<<<(unsigned)((segs + 7) / 8), 256, 0, s>>>(x, q, scales, M, K, KB);
  check_launch("fp8_quantize_act");
}

void launch_fp8_block_gemm(const uint8_t* xq, const float* xs, const uint8_t* wq, const float* ws, __nv_bfloat16* C,
                           int M, int N, int K, int* status, cudaStream_t s) {
  if (M <= 0 || N <= 0) return;
  if (K <= 0 || K % 16 != 0) throw std::runtime_error("fp8_block_gemm: K must be a positive multiple of 16");
  if (N % 8 != 0) throw std::runtime_error("fp8_block_gemm: N must be a multiple of 8");
  Fp8Params p;
  p.M = M; p.N = N; p.K = K; p.KB = (K + 127) / 128;
  p.num_m = (M + QBM - 1) / QBM; p.num_n = (N + QBN - 1) / QBN;
  p.xs = xs; p.ws = ws; p.C = C; p.status = status;
  CUtensorMap tmA = make_tmap_3d(xq, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, (uint64_t)K, (uint64_t)M, 1, (uint64_t)K,
                                 (uint64_t)K * (uint64_t)M, QBK, QBM);
  CUtensorMap tmB = make_tmap_3d(wq, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, (uint64_t)K, (uint64_t)N, 1, (uint64_t)K,
                                 (uint64_t)K * (uint64_t)N, QBK, QBN);
  static PerDeviceOnce configured;  // the attribute is per device
  if (configured.first_use()) {
    cudaError_t e = cudaFuncSetAttribute(fp8_block_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Q_SMEM);
    if (e != cudaSuccess) throw std::runtime_error(std::string("fp8_block_gemm: ") + cudaGetErrorString(e));
  }
  int sms = 0, dev = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (sms <= 0) sms = 148;
  const int tiles = p.num_m * p.num_n;
  fp8_block_gemm_kernel<<<tiles < sms ? tiles : sms, Q_THREADS, Q_SMEM, s>>>(tmA, tmB, p);
  check_launch("fp8_block_gemm");
}

void launch_nvfp4_quantize(const void* w, bool w_is_bf16, long long rows, long long K, bool hadamard, uint8_t* packed,
                           uint8_t* scales_e4m3, float* tscale, unsigned int* amax_scratch, cudaStream_t s) {
  if (K % 16 != 0) throw std::runtime_error("nvfp4_quantize: K must be a multiple of 16");
  const long long nblocks = rows * (K / 16);
  if (nblocks <= 0) return;
  cudaMemsetAsync(amax_scratch, 0, sizeof(unsigned int), s);
  const int g = grid_for(nblocks, 256);
  if (w_is_bf16) {
    ArraySrc<__nv_bfloat16> src{(const __nv_bfloat16*)w};
    nvfp4_amax_kernel<<<g, 256, 0, s>>>(src, nblocks, (int)hadamard, amax_scratch);
    nvfp4_quantize_kernel<<<g, 256, 0, s>>>(src, nblocks, (int)hadamard, amax_scratch, packed, scales_e4m3, tscale);
  } else {
    ArraySrc<float> src{(const float*)w};
    nvfp4_amax_kernel<<<g, 256, 0, s>>>(src, nblocks, (int)hadamard, amax_scratch);
    nvfp4_quantize_kernel<<<g, 256, 0, s>>>(src, nblocks, (int)hadamard, amax_scratch, packed, scales_e4m3, tscale);
  }
  check_launch("nvfp4_quantize");
}

static GgmlSrc make_ggml_src(const uint8_t* raw, int type, long long n) {
  const int be = ggml_block_elems(type), bb = ggml_block_bytes(type);
  if (bb == 0) throw std::runtime_error("ggml: unsupported tensor type " + std::to_string(type));
  if (n % be != 0) throw std::runtime_error("ggml: element count is not a multiple of the block size");
  return GgmlSrc{raw, type, be, bb};
}

void launch_ggml_dequant(const uint8_t* raw, int type, long long n, __nv_bfloat16* out, cudaStream_t s) {
  if (n <= 0) return;
  ggml_dequant_kernel<<<grid_for((n + 7) / 8, 256), 256, 0, s>>>(make_ggml_src(raw, type, n), n, out);
  check_launch("ggml_dequant");
}

void launch_ggml_to_nvfp4(const uint8_t* raw, int type, long long rows, long long K, bool hadamard, uint8_t* packed,
                          uint8_t* scales_e4m3, float* tscale, unsigned int* amax_scratch, cudaStream_t s) {
  if (K % 16 != 0) throw std::runtime_error("ggml_to_nvfp4: K must be a multiple of 16");
  const long long nblocks = rows * (K / 16);
  if (nblocks <= 0) return;
  GgmlSrc src = make_ggml_src(raw, type, rows * K);
  cudaMemsetAsync(amax_scratch, 0, sizeof(unsigned int), s);
  const int g = grid_for(nblocks, 256);
  nvfp4_amax_kernel<<<g, 256, 0, s>>>(src, nblocks, (int)hadamard, amax_scratch);
  nvfp4_quantize_kernel<<<g, 256, 0, s>>>(src, nblocks, (int)hadamard, amax_scratch, packed, scales_e4m3, tscale);
  check_launch("ggml_to_nvfp4");
}

void launch_nvfp4_dequant(const uint8_t* packed, const void* scales, bool scale_bf16, const float* tscale, long long rows,
                          long long K, __nv_bfloat16* out, cudaStream_t s) {
  const long long nblocks = rows * (K / 16);
  if (nblocks <= 0) return;
  nvfp4_dequant_kernel<<<grid_for(nblocks, 256), 256, 0, s>>>(packed, scales, scale_bf16, tscale, nblocks, out);
  check_launch("nvfp4_dequant");
}

void launch_nvfp4_gemv(const __nv_bfloat16* x, const uint8_t* packed, const void* scales, bool scale_bf16,
                       const float* tscale, __nv_bfloat16* y, int M, int N, int K, cudaStream_t s) {
  if (M < 1 || M > GEMV_MAX_M) throw std::runtime_error("nvfp4_gemv: 1 <= M <= 8");
  if (K % 16 != 0) throw std::runtime_error("nvfp4_gemv: K must be a multiple of 16");
  nvfp4_gemv_kernel<<<(N + 7) / 8, 256, 0, s>>>(x, packed, scales, scale_bf16, tscale, y, M, N, K);
  check_launch("nvfp4_gemv");
}

void launch_fwht16(const __nv_bfloat16* x, __nv_bfloat16* out, long long n, cudaStream_t s) {
  if (n % 16 != 0) throw std::runtime_error("fwht16: element count must be a multiple of 16");
  if (n == 0) return;
  fwht16_kernel<<<grid_for(n / 16, 256), 256, 0, s>>>(x, out, n / 16);
  check_launch("fwht16");
}

}  // namespace tb
