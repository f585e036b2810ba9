// Shared-memory tile helpers of the chunked linear-attention kernels (GLA and Gated DeltaNet): 64 x 64 bf16 tiles with
// 128-byte rows in the 128B-swizzled layout that TMA writes and tcgen05 reads, their operand descriptors, conversions
// between packed bf16 and fp32, and the clamped log decay.
#pragma once
#include <cuda_bf16.h>
#include <stdint.h>

#include "../common/ptx.cuh"
#include "gla.cuh"

namespace tb {

namespace {

constexpr int TILE = 64 * 128;  // bytes of one 64x64 bf16 tile (128-byte rows)

__device__ __forceinline__ void ld8(const float* p, float (&f)[8]) {
  const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
  f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w;
  f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
}
__device__ __forceinline__ void st8(float* p, const float (&f)[8]) {
  *reinterpret_cast<float4*>(p) = make_float4(f[0], f[1], f[2], f[3]);
  *reinterpret_cast<float4*>(p + 4) = make_float4(f[4], f[5], f[6], f[7]);
}

__device__ __forceinline__ uint32_t sw_off(int row, int chunk) { return row * 128 + ((chunk ^ (row & 7)) << 4); }

__device__ __forceinline__ float log_decay(float x, bool logits) {
  // log(1 + e) with e in (0, 1]: the fast logarithm's absolute error (1e-7) is far below the bf16 spacing of the gate
  float g = logits ? (fminf(x, 0.f) - __logf(1.0f + __expf(-fabsf(x)))) : fminf(x, 0.f);
  return fmaxf(g, GLA_MIN_LOG_DECAY);
}

__device__ __forceinline__ void unpack8(const uint4& u, float (&f)[8]) {
  const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 t = __bfloat1622float2(p[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
  uint4 u;
  u.x = pack_bf16x2(f[0], f[1]);
  u.y = pack_bf16x2(f[2], f[3]);
  u.z = pack_bf16x2(f[4], f[5]);
  u.w = pack_bf16x2(f[6], f[7]);
  return u;
}

// K-major operand view of a tile (rows = M/N index, cols = reduction): step k advances 32 bytes.
__device__ __forceinline__ uint64_t desc_k(uint32_t tile_addr, int kstep) {
  return make_smem_desc(tile_addr + kstep * 32, 16, 1024);
}
// MN-major operand view (rows = reduction index, cols = M/N index): step k advances 16 rows.
__device__ __forceinline__ uint64_t desc_mn(uint32_t tile_addr, int kstep) {
  return make_smem_desc(tile_addr + kstep * 2048, TILE, 1024);
}

// N-column slice (N = 16 or 32) of an accumulator row: TMEM lane quarter `quarter`, columns [col, col + N).
template <int N>
__device__ __forceinline__ void load_acc_cols(uint32_t tmem, uint32_t col, int quarter, float (&v)[N]) {
  uint32_t r[N];
  if constexpr (N == 32) tmem_ld_32x32b_x32(tmem + ((uint32_t)(quarter * 32) << 16) + col, r);
  else tmem_ld_32x32b_x16(tmem + ((uint32_t)(quarter * 32) << 16) + col, r);
  tmem_ld_wait();
#pragma unroll
  for (int i = 0; i < N; ++i) v[i] = __uint_as_float(r[i]);
}
// Writes columns [c0, c0 + N) of a row as bf16 into a swizzled tile; columns > limit are zeroed (causal mask).
template <int N>
__device__ __forceinline__ void store_row_cols(uint8_t* tile, int row, int c0, const float (&v)[N], int limit) {
#pragma unroll
  for (int c8 = 0; c8 < N / 8; ++c8) {
    const int ch = c0 / 8 + c8;
    float o[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) o[i] = (ch * 8 + i <= limit) ? v[c8 * 8 + i] : 0.f;
    *reinterpret_cast<uint4*>(tile + sw_off(row, ch)) = pack8(o);
  }
}
template <int N>
__device__ __forceinline__ void ld_row(const float* p, float (&f)[N]) {
#pragma unroll
  for (int i = 0; i < N / 4; ++i) {
    const float4 t = *reinterpret_cast<const float4*>(p + 4 * i);
    f[4 * i] = t.x; f[4 * i + 1] = t.y; f[4 * i + 2] = t.z; f[4 * i + 3] = t.w;
  }
}
}  // namespace

}  // namespace tb
