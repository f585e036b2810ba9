// Bandwidth-bound row kernels: RMSNorm (+ residual add) forward/backward and the GLA q/k feature
// map (ELU+1 -> L2 normalise -> half-split RoPE) forward/backward. One warp owns one row (RMSNorm) or
// one (token, head) vector (feature map); all global traffic is 16-byte (RMSNorm) or 4-byte-pair
// coalesced (feature map) and every tensor is touched exactly once per pass.
//
// Reference semantics: triune/kernels/fast_rmsnorm.py:181-335 (norm, fused add-norm),
// triune/model/attention.py:14-80 and :509-531 (feature map + RoPE).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../common/ptx.cuh"
#include "elementwise.cuh"

namespace tb {

namespace {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// Each lane holds up to MAXV 8-element vectors of its row (d <= 32*8*MAXV).
constexpr int MAXV = 8;

template <bool HAS_RES>
__global__ void __launch_bounds__(256) rmsnorm_fwd_kernel(const __nv_bfloat16* __restrict__ x,
                                                          const __nv_bfloat16* __restrict__ res,
                                                          const __nv_bfloat16* __restrict__ w,
                                                          __nv_bfloat16* __restrict__ y,
                                                          __nv_bfloat16* __restrict__ sum_out,
                                                          float* __restrict__ rstd, int rows, int d, float eps) {
  const int warps_per_block = blockDim.x >> 5;
  const int lane = threadIdx.x & 31;
  const int nvec = d >> 3;
  for (long long row = (long long)blockIdx.x * warps_per_block + (threadIdx.x >> 5); row < rows;
       row += (long long)gridDim.x * warps_per_block) {
    const uint4* xr = reinterpret_cast<const uint4*>(x + row * d);
    const uint4* rr = HAS_RES ? reinterpret_cast<const uint4*>(res + row * d) : nullptr;
    float vals[MAXV][8];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < MAXV; ++i) {
      const int v = lane + i * 32;
      if (v < nvec) {
        uint4 xv = xr[v];
        const __nv_bfloat162* x2 = reinterpret_cast<const __nv_bfloat162*>(&xv);
        if (HAS_RES) {
          uint4 rv = rr[v];
          const __nv_bfloat162* r2 = reinterpret_cast<const __nv_bfloat162*>(&rv);
          uint4 sv;
          uint32_t* s32 = reinterpret_cast<uint32_t*>(&sv);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            float2 a = __bfloat1622float2(x2[j]), b = __bfloat1622float2(r2[j]);
            s32[j] = pack_bf16x2(a.x + b.x, a.y + b.y);
            float2 s = __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&s32[j]));
            vals[i][2 * j] = s.x;
            vals[i][2 * j + 1] = s.y;
          }
          reinterpret_cast<uint4*>(sum_out + row * d)[v] = sv;
        } else {
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            float2 a = __bfloat1622float2(x2[j]);
            vals[i][2 * j] = a.x;
            vals[i][2 * j + 1] = a.y;
          }
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) ss += vals[i][j] * vals[i][j];
      }
    }
    ss = warp_sum(ss);
    const float inv = rsqrtf(ss / (float)d + eps);
    if (lane == 0 && rstd) rstd[row] = inv;
#pragma unroll
    for (int i = 0; i < MAXV; ++i) {
      const int v = lane + i * 32;
      if (v < nvec) {
        uint4 wv = reinterpret_cast<const uint4*>(w)[v];
        const __nv_bfloat162* w2 = reinterpret_cast<const __nv_bfloat162*>(&wv);
        uint4 ov;
        uint32_t* o32 = reinterpret_cast<uint32_t*>(&ov);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          float2 wf = __bfloat1622float2(w2[j]);
          o32[j] = pack_bf16x2(vals[i][2 * j] * inv * wf.x, vals[i][2 * j + 1] * inv * wf.y);
        }
        reinterpret_cast<uint4*>(y + row * d)[v] = ov;
      }
    }
  }
}

// dx = rstd * (w*dy - xhat * mean(w*dy*xhat)) [+ dres_in]; dw += sum_rows dy * xhat (fp32 atomics,
// one atomic per column per block after an in-block reduction).
template <bool HAS_DRES>
__global__ void __launch_bounds__(256) rmsnorm_bwd_kernel(const __nv_bfloat16* __restrict__ x,
                                                          const __nv_bfloat16* __restrict__ w,
                                                          const __nv_bfloat16* __restrict__ dy,
                                                          const float* __restrict__ rstd,
                                                          const __nv_bfloat16* __restrict__ dres,
                                                          __nv_bfloat16* __restrict__ dx, float* __restrict__ dw,
                                                          int rows, int d) {
  extern __shared__ float dw_smem[];  // [d]
  const int warps_per_block = blockDim.x >> 5;
  const int lane = threadIdx.x & 31;
  const int nvec = d >> 3;
  for (int i = threadIdx.x; i < d; i += blockDim.x) dw_smem[i] = 0.f;
  __syncthreads();
  float dwacc[MAXV][8];
#pragma unroll
  for (int i = 0; i < MAXV; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) dwacc[i][j] = 0.f;

  for (long long row = (long long)blockIdx.x * warps_per_block + (threadIdx.x >> 5); row < rows;
       row += (long long)gridDim.x * warps_per_block) {
    const float inv = rstd[row];
    float xh[MAXV][8], wdy[MAXV][8];
    float dot = 0.f;
#pragma unroll
    for (int i = 0; i < MAXV; ++i) {
      const int v = lane + i * 32;
      if (v < nvec) {
        uint4 xv = reinterpret_cast<const uint4*>(x + row * d)[v];
        uint4 gv = reinterpret_cast<const uint4*>(dy + row * d)[v];
        uint4 wv = reinterpret_cast<const uint4*>(w)[v];
        const __nv_bfloat162* x2 = reinterpret_cast<const __nv_bfloat162*>(&xv);
        const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&gv);
        const __nv_bfloat162* w2 = reinterpret_cast<const __nv_bfloat162*>(&wv);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          float2 xf = __bfloat1622float2(x2[j]), gf = __bfloat1622float2(g2[j]), wf = __bfloat1622float2(w2[j]);
          xh[i][2 * j] = xf.x * inv;
          xh[i][2 * j + 1] = xf.y * inv;
          wdy[i][2 * j] = gf.x * wf.x;
          wdy[i][2 * j + 1] = gf.y * wf.y;
          dwacc[i][2 * j] += gf.x * xh[i][2 * j];
          dwacc[i][2 * j + 1] += gf.y * xh[i][2 * j + 1];
          dot += wdy[i][2 * j] * xh[i][2 * j] + wdy[i][2 * j + 1] * xh[i][2 * j + 1];
        }
      }
    }
    dot = warp_sum(dot) / (float)d;
#pragma unroll
    for (int i = 0; i < MAXV; ++i) {
      const int v = lane + i * 32;
      if (v < nvec) {
        float o[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = inv * (wdy[i][j] - xh[i][j] * dot);
        if (HAS_DRES) {
          uint4 rv = reinterpret_cast<const uint4*>(dres + row * d)[v];
          const __nv_bfloat162* r2 = reinterpret_cast<const __nv_bfloat162*>(&rv);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            float2 rf = __bfloat1622float2(r2[j]);
            o[2 * j] += rf.x;
            o[2 * j + 1] += rf.y;
          }
        }
        uint4 ov;
        ov.x = pack_bf16x2(o[0], o[1]);
        ov.y = pack_bf16x2(o[2], o[3]);
        ov.z = pack_bf16x2(o[4], o[5]);
        ov.w = pack_bf16x2(o[6], o[7]);
        reinterpret_cast<uint4*>(dx + row * d)[v] = ov;
      }
    }
  }
#pragma unroll
  for (int i = 0; i < MAXV; ++i) {
    const int v = lane + i * 32;
    if (v < nvec) {
#pragma unroll
      for (int j = 0; j < 8; ++j) atomicAdd(&dw_smem[v * 8 + j], dwacc[i][j]);
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < d; i += blockDim.x) atomicAdd(&dw[i], dw_smem[i]);
}

// ---------------------------------------------------------------- q/k feature map + RoPE
// in: rows of width in_ld holding q at column 0 and k at column HD_total (both [H, D]); one warp per
// (token, head, q-or-k). out: [tokens, 2, H, D] contiguous. cos/sin: [T, D/2] fp32, token t uses
// position (t % T) (tokens are laid out [B, T]).
template <int D>
__global__ void __launch_bounds__(256) qk_prep_fwd_kernel(const __nv_bfloat16* __restrict__ in, long long in_ld,
                                                          int k_col_offset, __nv_bfloat16* __restrict__ out,
                                                          const float* __restrict__ cs, const float* __restrict__ sn,
                                                          long long tokens, int T, int H) {
  constexpr int PAIRS = D / 64;  // pairs (i, i + D/2) handled per lane
  const int lane = threadIdx.x & 31;
  const long long total = tokens * 2 * H;
  for (long long idx = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); idx < total;
       idx += (long long)gridDim.x * (blockDim.x >> 5)) {
    const int h = idx % H;
    const int which = (idx / H) % 2;
    const long long tok = idx / (2 * H);
    const __nv_bfloat16* src = in + tok * in_ld + (which ? k_col_offset : 0) + h * D;
    float f0[PAIRS], f1[PAIRS];
    float ss = 0.f;
#pragma unroll
    for (int p = 0; p < PAIRS; ++p) {
      const int i = lane + p * 32;
      float a = __bfloat162float(src[i]), b = __bfloat162float(src[i + D / 2]);
      a = a > 0.f ? a + 1.f : __expf(a);
      b = b > 0.f ? b + 1.f : __expf(b);
      f0[p] = a;
      f1[p] = b;
      ss += a * a + b * b;
    }
    ss = warp_sum(ss);
    const float inv = 1.0f / fmaxf(sqrtf(ss), 1e-6f);
    __nv_bfloat16* dst = out + ((tok * 2 + which) * H + h) * D;
    const int pos = (int)(tok % T);
#pragma unroll
    for (int p = 0; p < PAIRS; ++p) {
      const int i = lane + p * 32;
      float c = 1.f, s = 0.f;
      if (cs) {
        c = cs[(long long)pos * (D / 2) + i];
        s = sn[(long long)pos * (D / 2) + i];
      }
      const float a = f0[p] * inv, b = f1[p] * inv;
      dst[i] = __float2bfloat16(a * c - b * s);
      dst[i + D / 2] = __float2bfloat16(b * c + a * s);
    }
  }
}

// Backward: recompute f and n from the raw input, undo the rotation on the incoming gradient, then
// d f = (dn - n (n . dn)) / |f| and d raw = d f * (raw > 0 ? 1 : f). Writes into d_in at the same
// column layout as `in` (q at 0, k at k_col_offset).
template <int D>
__global__ void __launch_bounds__(256) qk_prep_bwd_kernel(const __nv_bfloat16* __restrict__ in, long long in_ld,
                                                          int k_col_offset, const __nv_bfloat16* __restrict__ dout,
                                                          __nv_bfloat16* __restrict__ d_in, long long d_in_ld,
                                                          const float* __restrict__ cs, const float* __restrict__ sn,
                                                          long long tokens, int T, int H) {
  constexpr int PAIRS = D / 64;
  const int lane = threadIdx.x & 31;
  const long long total = tokens * 2 * H;
  for (long long idx = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); idx < total;
       idx += (long long)gridDim.x * (blockDim.x >> 5)) {
    const int h = idx % H;
    const int which = (idx / H) % 2;
    const long long tok = idx / (2 * H);
    const __nv_bfloat16* src = in + tok * in_ld + (which ? k_col_offset : 0) + h * D;
    const __nv_bfloat16* g = dout + ((tok * 2 + which) * H + h) * D;
    float raw0[PAIRS], raw1[PAIRS], f0[PAIRS], f1[PAIRS], dn0[PAIRS], dn1[PAIRS];
    float ss = 0.f;
    const int pos = (int)(tok % T);
#pragma unroll
    for (int p = 0; p < PAIRS; ++p) {
      const int i = lane + p * 32;
      raw0[p] = __bfloat162float(src[i]);
      raw1[p] = __bfloat162float(src[i + D / 2]);
      f0[p] = raw0[p] > 0.f ? raw0[p] + 1.f : __expf(raw0[p]);
      f1[p] = raw1[p] > 0.f ? raw1[p] + 1.f : __expf(raw1[p]);
      ss += f0[p] * f0[p] + f1[p] * f1[p];
      float c = 1.f, s = 0.f;
      if (cs) {
        c = cs[(long long)pos * (D / 2) + i];
        s = sn[(long long)pos * (D / 2) + i];
      }
      const float ga = __bfloat162float(g[i]), gb = __bfloat162float(g[i + D / 2]);
      dn0[p] = ga * c + gb * s;   // transpose of the rotation
      dn1[p] = gb * c - ga * s;
    }
    ss = warp_sum(ss);
    const float nrm = fmaxf(sqrtf(ss), 1e-6f);
    const float inv = 1.0f / nrm;
    float dot = 0.f;
#pragma unroll
    for (int p = 0; p < PAIRS; ++p) dot += f0[p] * inv * dn0[p] + f1[p] * inv * dn1[p];
    dot = warp_sum(dot);
    __nv_bfloat16* dst = d_in + tok * d_in_ld + (which ? k_col_offset : 0) + h * D;
#pragma unroll
    for (int p = 0; p < PAIRS; ++p) {
      const int i = lane + p * 32;
      const float df0 = (dn0[p] - f0[p] * inv * dot) * inv;
      const float df1 = (dn1[p] - f1[p] * inv * dot) * inv;
      dst[i] = __float2bfloat16(df0 * (raw0[p] > 0.f ? 1.f : f0[p]));
      dst[i + D / 2] = __float2bfloat16(df1 * (raw1[p] > 0.f ? 1.f : f1[p]));
    }
  }
}

inline int row_grid(long long work_items, int per_block) {
  long long b = (work_items + per_block - 1) / per_block;
  const long long cap = 148ll * 8;
  return (int)(b < 1 ? 1 : (b > cap ? cap : b));
}

}  // namespace

void launch_rmsnorm_fwd(const __nv_bfloat16* x, const __nv_bfloat16* res, const __nv_bfloat16* w, __nv_bfloat16* y,
                        __nv_bfloat16* sum_out, float* rstd, int rows, int d, float eps, cudaStream_t s) {
  if (rows == 0) return;
  const int grid = row_grid(rows, 8);
  if (res)
    rmsnorm_fwd_kernel<true><<<grid, 256, 0, s>>>(x, res, w, y, sum_out, rstd, rows, d, eps);
  else
    rmsnorm_fwd_kernel<false><<<grid, 256, 0, s>>>(x, nullptr, w, y, nullptr, rstd, rows, d, eps);
}

void launch_rmsnorm_bwd(const __nv_bfloat16* x, const __nv_bfloat16* w, const __nv_bfloat16* dy, const float* rstd,
                        const __nv_bfloat16* dres, __nv_bfloat16* dx, float* dw, int rows, int d, cudaStream_t s) {
  if (rows == 0) return;
  long long b = ((long long)rows + 8 * 16 - 1) / (8 * 16);  // >=16 rows per warp so the dw atomics amortise
  const int grid = (int)(b < 1 ? 1 : (b > 148 * 4 ? 148 * 4 : b));
  if (dres)
    rmsnorm_bwd_kernel<true><<<grid, 256, d * sizeof(float), s>>>(x, w, dy, rstd, dres, dx, dw, rows, d);
  else
    rmsnorm_bwd_kernel<false><<<grid, 256, d * sizeof(float), s>>>(x, w, dy, rstd, nullptr, dx, dw, rows, d);
}

void launch_qk_prep_fwd(const __nv_bfloat16* in, long long in_ld, int k_col_offset, __nv_bfloat16* out, const float* cs,
                        const float* sn, long long tokens, int T, int H, int D, cudaStream_t s) {
  if (tokens == 0) return;
  const int grid = row_grid(tokens * 2 * H, 8);
  if (D == 64)
    qk_prep_fwd_kernel<64><<<grid, 256, 0, s>>>(in, in_ld, k_col_offset, out, cs, sn, tokens, T, H);
  else
    qk_prep_fwd_kernel<128><<<grid, 256, 0, s>>>(in, in_ld, k_col_offset, out, cs, sn, tokens, T, H);
}

void launch_qk_prep_bwd(const __nv_bfloat16* in, long long in_ld, int k_col_offset, const __nv_bfloat16* dout,
                        __nv_bfloat16* d_in, long long d_in_ld, const float* cs, const float* sn, long long tokens,
                        int T, int H, int D, cudaStream_t s) {
  if (tokens == 0) return;
  const int grid = row_grid(tokens * 2 * H, 8);
  if (D == 64)
    qk_prep_bwd_kernel<64><<<grid, 256, 0, s>>>(in, in_ld, k_col_offset, dout, d_in, d_in_ld, cs, sn, tokens, T, H);
  else
    qk_prep_bwd_kernel<128><<<grid, 256, 0, s>>>(in, in_ld, k_col_offset, dout, d_in, d_in_ld, cs, sn, tokens, T, H);
}

}  // namespace tb
