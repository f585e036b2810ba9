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

// Each lane holds up to MAXV 8-element vectors of its row (d <= 32*8*MAXV); MAXV is a template parameter so
// narrow models do not pay registers for wide ones.

template <bool HAS_RES, int MAXV>
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
template <bool HAS_DRES, int MAXV>
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
// in: rows of width in_ld holding q at column 0 and k at column k_col_offset (both [H, D]). One vector = one
// (token, head, q-or-k) row of D elements, handled by D/8 lanes with one 16-byte load each; the rotation
// partner of element i (i + D/2) lives in lane ^ (D/16). out: [tokens, 2, H, D] contiguous. cos/sin: [T, D/2]
// fp32, token t uses position (t % T) (tokens are laid out [B, T]).
template <int D>
struct PrepGeom {
  static constexpr int LPV = D / 8;        // lanes per vector
  static constexpr int VPW = 32 / LPV;     // vectors per warp
};

template <int LPV>
__device__ __forceinline__ float group_sum(float v) {
#pragma unroll
  for (int o = LPV / 2; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ __forceinline__ void load8(const __nv_bfloat16* p, float (&f)[8]) {
  uint4 u = *reinterpret_cast<const uint4*>(p);
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 t = __bfloat1622float2(h[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}
__device__ __forceinline__ void store8(__nv_bfloat16* p, const float (&f)[8]) {
  uint4 u;
  u.x = pack_bf16x2(f[0], f[1]);
  u.y = pack_bf16x2(f[2], f[3]);
  u.z = pack_bf16x2(f[4], f[5]);
  u.w = pack_bf16x2(f[6], f[7]);
  *reinterpret_cast<uint4*>(p) = u;
}

template <int D>
__global__ void __launch_bounds__(256) qk_prep_fwd_kernel(const __nv_bfloat16* __restrict__ in, long long in_ld,
                                                          int k_col_offset, __nv_bfloat16* __restrict__ out,
                                                          const float* __restrict__ cs, const float* __restrict__ sn,
                                                          long long tokens, int T, int H) {
  constexpr int LPV = PrepGeom<D>::LPV, VPW = PrepGeom<D>::VPW;
  const int lane = threadIdx.x & 31, sub = lane % LPV, vin = lane / LPV;
  const long long total = tokens * 2 * H;
  const long long warps = (long long)gridDim.x * (blockDim.x >> 5);
  for (long long base = ((long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5)) * VPW; base < total;
       base += warps * VPW) {
    const long long idx = base + vin;
    const bool live = idx < total;
    const long long cidx = live ? idx : total - 1;
    const int h = cidx % H;
    const int which = (cidx / H) % 2;
    const long long tok = cidx / (2 * H);
    float f[8];
    load8(in + tok * in_ld + (which ? k_col_offset : 0) + h * D + sub * 8, f);
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      f[i] = f[i] > 0.f ? f[i] + 1.f : __expf(f[i]);
      ss += f[i] * f[i];
    }
    ss = group_sum<LPV>(ss);
    const float inv = 1.0f / fmaxf(sqrtf(ss), 1e-6f);
    float o[8];
    const bool upper = sub >= LPV / 2;
    const int pos = (int)(tok % T);
    const int ci = (sub % (LPV / 2)) * 8;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float mine = f[i] * inv;
      const float other = __shfl_xor_sync(0xffffffffu, mine, LPV / 2);
      float c = 1.f, s = 0.f;
      if (cs) {
        c = cs[(long long)pos * (D / 2) + ci + i];
        s = sn[(long long)pos * (D / 2) + ci + i];
      }
      o[i] = upper ? (mine * c + other * s) : (mine * c - other * s);
    }
    if (live) store8(out + ((tok * 2 + which) * H + h) * D + sub * 8, o);
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
  constexpr int LPV = PrepGeom<D>::LPV, VPW = PrepGeom<D>::VPW;
  const int lane = threadIdx.x & 31, sub = lane % LPV, vin = lane / LPV;
  const long long total = tokens * 2 * H;
  const long long warps = (long long)gridDim.x * (blockDim.x >> 5);
  for (long long base = ((long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5)) * VPW; base < total;
       base += warps * VPW) {
    const long long idx = base + vin;
    const bool live = idx < total;
    const long long cidx = live ? idx : total - 1;
    const int h = cidx % H;
    const int which = (cidx / H) % 2;
    const long long tok = cidx / (2 * H);
    float raw[8], f[8], g[8], dn[8];
    load8(in + tok * in_ld + (which ? k_col_offset : 0) + h * D + sub * 8, raw);
    load8(dout + ((tok * 2 + which) * H + h) * D + sub * 8, g);
    float ss = 0.f;
    const bool upper = sub >= LPV / 2;
    const int pos = (int)(tok % T);
    const int ci = (sub % (LPV / 2)) * 8;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      f[i] = raw[i] > 0.f ? raw[i] + 1.f : __expf(raw[i]);
      ss += f[i] * f[i];
      const float other = __shfl_xor_sync(0xffffffffu, g[i], LPV / 2);
      float c = 1.f, s = 0.f;
      if (cs) {
        c = cs[(long long)pos * (D / 2) + ci + i];
        s = sn[(long long)pos * (D / 2) + ci + i];
      }
      // transpose of the rotation: lower half gets g*c + g_partner*s, upper half g*c - g_partner*s
      dn[i] = upper ? (g[i] * c - other * s) : (g[i] * c + other * s);
    }
    ss = group_sum<LPV>(ss);
    const float inv = 1.0f / fmaxf(sqrtf(ss), 1e-6f);
    float dot = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) dot += f[i] * inv * dn[i];
    dot = group_sum<LPV>(dot);
    float o[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float df = (dn[i] - f[i] * inv * dot) * inv;
      o[i] = df * (raw[i] > 0.f ? 1.f : f[i]);
    }
    if (live) store8(d_in + tok * d_in_ld + (which ? k_col_offset : 0) + h * D + sub * 8, o);
  }
}

inline int row_grid(long long work_items, int per_block) {
  long long b = (work_items + per_block - 1) / per_block;
  const long long cap = 148ll * 16;
  return (int)(b < 1 ? 1 : (b > cap ? cap : b));
}


template <int MAXV>
void rmsnorm_fwd_dispatch(const __nv_bfloat16* x, const __nv_bfloat16* res, const __nv_bfloat16* w, __nv_bfloat16* y,
                          __nv_bfloat16* sum_out, float* rstd, int rows, int d, float eps, int grid, cudaStream_t s) {
  if (res)
    rmsnorm_fwd_kernel<true, MAXV><<<grid, 256, 0, s>>>(x, res, w, y, sum_out, rstd, rows, d, eps);
  else
    rmsnorm_fwd_kernel<false, MAXV><<<grid, 256, 0, s>>>(x, nullptr, w, y, nullptr, rstd, rows, d, eps);
}

template <int MAXV>
void rmsnorm_bwd_dispatch(const __nv_bfloat16* x, const __nv_bfloat16* w, const __nv_bfloat16* dy, const float* rstd,
                          const __nv_bfloat16* dres, __nv_bfloat16* dx, float* dw, int rows, int d, int grid,
                          cudaStream_t s) {
  if (dres)
    rmsnorm_bwd_kernel<true, MAXV><<<grid, 256, d * sizeof(float), s>>>(x, w, dy, rstd, dres, dx, dw, rows, d);
  else
    rmsnorm_bwd_kernel<false, MAXV><<<grid, 256, d * sizeof(float), s>>>(x, w, dy, rstd, nullptr, dx, dw, rows, d);
}

}  // namespace

void launch_rmsnorm_fwd(const __nv_bfloat16* x, const __nv_bfloat16* res, const __nv_bfloat16* w, __nv_bfloat16* y,
                        __nv_bfloat16* sum_out, float* rstd, int rows, int d, float eps, cudaStream_t s) {
  if (rows == 0) return;
  const int grid = row_grid(rows, 8);
  if (d <= 512) rmsnorm_fwd_dispatch<2>(x, res, w, y, sum_out, rstd, rows, d, eps, grid, s);
  else if (d <= 1024) rmsnorm_fwd_dispatch<4>(x, res, w, y, sum_out, rstd, rows, d, eps, grid, s);
  else rmsnorm_fwd_dispatch<8>(x, res, w, y, sum_out, rstd, rows, d, eps, grid, s);
}

void launch_rmsnorm_bwd(const __nv_bfloat16* x, const __nv_bfloat16* w, const __nv_bfloat16* dy, const float* rstd,
                        const __nv_bfloat16* dres, __nv_bfloat16* dx, float* dw, int rows, int d, cudaStream_t s) {
  if (rows == 0) return;
  // few, fat blocks: every block ends with d global atomics into dw, so the block count bounds the contention
  long long b = ((long long)rows + 8 * 8 - 1) / (8 * 8);
  const int grid = (int)(b < 1 ? 1 : (b > 148 * 3 ? 148 * 3 : b));
  if (d <= 512) rmsnorm_bwd_dispatch<2>(x, w, dy, rstd, dres, dx, dw, rows, d, grid, s);
  else if (d <= 1024) rmsnorm_bwd_dispatch<4>(x, w, dy, rstd, dres, dx, dw, rows, d, grid, s);
  else rmsnorm_bwd_dispatch<8>(x, w, dy, rstd, dres, dx, dw, rows, d, grid, s);
}

void launch_qk_prep_fwd(const __nv_bfloat16* in, long long in_ld, int k_col_offset, __nv_bfloat16* out, const float* cs,
                        const float* sn, long long tokens, int T, int H, int D, cudaStream_t s) {
  if (tokens == 0) return;
  const int grid = row_grid(tokens * 2 * H, 8 * (256 / D));
  if (D == 64)
    qk_prep_fwd_kernel<64><<<grid, 256, 0, s>>>(in, in_ld, k_col_offset, out, cs, sn, tokens, T, H);
  else
    qk_prep_fwd_kernel<128><<<grid, 256, 0, s>>>(in, in_ld, k_col_offset, out, cs, sn, tokens, T, H);
}

void launch_qk_prep_bwd(const __nv_bfloat16* in, long long in_ld, int k_col_offset, const __nv_bfloat16* dout,
                        __nv_bfloat16* d_in, long long d_in_ld, const float* cs, const float* sn, long long tokens,
                        int T, int H, int D, cudaStream_t s) {
  if (tokens == 0) return;
  const int grid = row_grid(tokens * 2 * H, 8 * (256 / D));
  if (D == 64)
    qk_prep_bwd_kernel<64><<<grid, 256, 0, s>>>(in, in_ld, k_col_offset, dout, d_in, d_in_ld, cs, sn, tokens, T, H);
  else
    qk_prep_bwd_kernel<128><<<grid, 256, 0, s>>>(in, in_ld, k_col_offset, dout, d_in, d_in_ld, cs, sn, tokens, T, H);
}


// ------------------------------------------------------------------------------------------------
// Column sums of a bf16 matrix (bias gradients): out[n] (+)= sum_m x[m, n].
// Phase 1: a block owns a 256-column slab and every gridDim.y-th group of 8 rows; a warp reads 512 contiguous bytes
// of one row per step, a thread keeps 8 fp32 sums, the block's 8 warps are combined through shared memory and one
// partial row is written per block. Phase 2 adds the partial rows in a fixed order, so results are reproducible.
// ------------------------------------------------------------------------------------------------
namespace {

__global__ void __launch_bounds__(256) colsum_partial_kernel(const __nv_bfloat16* __restrict__ x, long long ld, int M,
                                                             int N, float* __restrict__ partial) {
  __shared__ float red[8][256];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int col = blockIdx.x * 256 + lane * 8;
  float acc[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) acc[i] = 0.f;
  if (col < N) {
    for (int m = blockIdx.y * 8 + warp; m < M; m += gridDim.y * 8) {
      const uint4 u = *reinterpret_cast<const uint4*>(x + (long long)m * ld + col);
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 f = __bfloat1622float2(h[i]);
        acc[2 * i] += f.x;
        acc[2 * i + 1] += f.y;
      }
    }
  }
#pragma unroll
  for (int i = 0; i < 8; ++i) red[warp][lane * 8 + i] = acc[i];
  __syncthreads();
  const int c = blockIdx.x * 256 + threadIdx.x;
  if (c < N) {
    float s = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) s += red[w][threadIdx.x];
    partial[(long long)blockIdx.y * N + c] = s;
  }
}

__global__ void colsum_finalize_kernel(const float* __restrict__ partial, int parts, int N, float* __restrict__ out,
                                       int accumulate) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= N) return;
  float s = 0.f;
  for (int p = 0; p < parts; ++p) s += partial[(long long)p * N + c];
  out[c] = accumulate ? out[c] + s : s;
}

}  // namespace

int colsum_parts(int M, int N) {
  const int slabs = (N + 255) / 256;
  int parts = (148 * 4 + slabs - 1) / slabs;
  const int max_parts = (M + 63) / 64;  // at least 8 rows per warp
  if (parts > max_parts) parts = max_parts;
  return parts < 1 ? 1 : parts;
}

void launch_colsum(const __nv_bfloat16* x, long long ld, int M, int N, float* partial, int parts, float* out,
                   bool accumulate, cudaStream_t s) {
  dim3 grid((N + 255) / 256, parts);
  colsum_partial_kernel<<<grid, 256, 0, s>>>(x, ld, M, N, partial);
  colsum_finalize_kernel<<<(N + 255) / 256, 256, 0, s>>>(partial, parts, N, out, accumulate ? 1 : 0);
}

}  // namespace tb
