// Cross-entropy with in-place gradient, MoE row movement (gather / weighted combine / row dots), flat
// optimizer updates (AdamW, Muon momentum and apply, triangular AdamW core, steer update) and the
// small routing / visualisation kernels of the native engine.
//
// Reference semantics: triune/kernels/fast_cross_entropy.py:20-220 (CE, in-place chunk gradient),
// triune/model/moe.py:385-437 (capacity gather, weighted index_add), triune/kernels/fast_triangular.py:23-88,
// csrc/kernels/muon.cu:26-99, csrc/kernels/centroid_steer.cu:48-114, csrc/kernels/router.cu:24-82,
// csrc/engine/engine.cpp:314-414 of the reference project.
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <stdexcept>
#include <string>
#include <float.h>
#include <stdint.h>

#include "../common/per_device.h"
#include "../common/ptx.cuh"
#include "elementwise.cuh"

namespace tb {

namespace {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

template <int THREADS>
__device__ __forceinline__ float block_sum(float v, float* red) {
  v = warp_sum(v);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  float t = ((threadIdx.x & 31) < THREADS / 32) ? red[threadIdx.x & 31] : 0.f;
  t = warp_sum(t);
  return __shfl_sync(0xffffffffu, t, 0);
}
template <int THREADS>
__device__ __forceinline__ float block_max(float v, float* red) {
  v = warp_max(v);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  float t = ((threadIdx.x & 31) < THREADS / 32) ? red[threadIdx.x & 31] : -FLT_MAX;
  t = warp_max(t);
  return __shfl_sync(0xffffffffu, t, 0);
}

// One block per row. Pass 1: online max / sum-exp over 16-byte vectors; pass 2 (second read hits L2):
// write grad_scale * (softmax - onehot) in place.
constexpr int CE_THREADS = 256;
__global__ void __launch_bounds__(CE_THREADS) ce_fwd_bwd_kernel(__nv_bfloat16* __restrict__ logits, long long ld,
                                                                const long long* __restrict__ targets,
                                                                float* __restrict__ row_loss, int V,
                                                                long long ignore_index, float grad_scale,
                                                                __nv_bfloat16* grad_dst) {
  __shared__ float red[CE_THREADS / 32];
  const long long row = blockIdx.x;
  __nv_bfloat16* lp = logits + row * ld;
  // gradient destination: the logits themselves (in place) unless a separate [rows, V] buffer of the same pitch is given
  __nv_bfloat16* gp = grad_dst != nullptr ? grad_dst + row * ld : lp;
  uint4* gv = reinterpret_cast<uint4*>(gp);
  const long long tgt = targets[row];
  const int nvec = V >> 3;
  uint4* lv = reinterpret_cast<uint4*>(lp);
  if (tgt == ignore_index) {
    if (threadIdx.x == 0) row_loss[row] = 0.f;
    if (grad_scale != 0.f) {
      for (int v = threadIdx.x; v < nvec; v += CE_THREADS) gv[v] = make_uint4(0, 0, 0, 0);
      for (int i = nvec * 8 + threadIdx.x; i < V; i += CE_THREADS) gp[i] = __float2bfloat16(0.f);
    }
    return;
  }
  float mx = -FLT_MAX, sm = 0.f;
  for (int v = threadIdx.x; v < nvec; v += CE_THREADS) {
    uint4 x = lv[v];
    const __nv_bfloat162* x2 = reinterpret_cast<const __nv_bfloat162*>(&x);
    float f[8];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float2 t = __bfloat1622float2(x2[j]);
      f[2 * j] = t.x;
      f[2 * j + 1] = t.y;
    }
    float lm = f[0];
#pragma unroll
    for (int j = 1; j < 8; ++j) lm = fmaxf(lm, f[j]);
    if (lm > mx) {
      sm *= __expf(mx - lm);
      mx = lm;
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) sm += __expf(f[j] - mx);
  }
  for (int i = nvec * 8 + threadIdx.x; i < V; i += CE_THREADS) {
    float f = __bfloat162float(lp[i]);
    if (f > mx) {
      sm *= __expf(mx - f);
      mx = f;
    }
    sm += __expf(f - mx);
  }
  const float gmx = block_max<CE_THREADS>(mx, red);
  sm *= __expf(mx - gmx);
  const float gsm = block_sum<CE_THREADS>(sm, red);
  const float lse = gmx + logf(gsm);
  if (threadIdx.x == 0) row_loss[row] = lse - __bfloat162float(lp[tgt]);
  if (grad_scale == 0.f) return;
  __syncthreads();  // the target logit above is read before anyone overwrites it
  const float inv = grad_scale / gsm;
  for (int v = threadIdx.x; v < nvec; v += CE_THREADS) {
    uint4 x = lv[v];
    const __nv_bfloat162* x2 = reinterpret_cast<const __nv_bfloat162*>(&x);
    float f[8];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float2 t = __bfloat1622float2(x2[j]);
      f[2 * j] = __expf(t.x - gmx) * inv;
      f[2 * j + 1] = __expf(t.y - gmx) * inv;
    }
    const long long base = (long long)v * 8;
    if (tgt >= base && tgt < base + 8) f[tgt - base] -= grad_scale;
    uint4 o;
    o.x = pack_bf16x2(f[0], f[1]);
    o.y = pack_bf16x2(f[2], f[3]);
    o.z = pack_bf16x2(f[4], f[5]);
    o.w = pack_bf16x2(f[6], f[7]);
    gv[v] = o;
  }
  for (int i = nvec * 8 + threadIdx.x; i < V; i += CE_THREADS) {
    float f = __expf(__bfloat162float(lp[i]) - gmx) * inv;
    if (i == tgt) f -= grad_scale;
    gp[i] = __float2bfloat16(f);
  }
}

// ---------------------------------------------------------------- index checks of the row-movement kernels
// An index that leaves its table (a corrupted dispatch plan) is neither followed nor trapped on: the access is
// skipped and the first offender is recorded here as {kernel id, row, index, limit}; the host reads it with
// index_error_word() (a device-to-host copy, so only tests and debugging runs do).
__device__ int g_index_error[4] = {0, 0, 0, 0};
__device__ __forceinline__ void record_index_error(int kernel_id, int row, int index, int limit) {
  if (atomicCAS(&g_index_error[0], 0, kernel_id) == 0) {
    g_index_error[1] = row;
    g_index_error[2] = index;
    g_index_error[3] = limit;
  }
}

// ---------------------------------------------------------------- MoE row movement
__global__ void __launch_bounds__(256) gather_rows_kernel(__nv_bfloat16* __restrict__ dst,
                                                          const __nv_bfloat16* __restrict__ src,
                                                          const int* __restrict__ row_src,
                                                          const float* __restrict__ row_scale, int dst_rows,
                                                          int width, int src_rows) {
  const int nvec = width >> 3;
  const long long total = (long long)dst_rows * nvec;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int r = (int)(i / nvec), v = (int)(i % nvec);
    const int s = row_src[r];
    uint4 o = make_uint4(0, 0, 0, 0);
    if (s >= src_rows) {
      if (v == 0) record_index_error(1, r, s, src_rows);
    } else if (s >= 0) {
      o = reinterpret_cast<const uint4*>(src + (long long)s * width)[v];
      if (row_scale) {
        const float sc = row_scale[r];
        __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          float2 f = __bfloat1622float2(o2[j]);
          o2[j] = __floats2bfloat162_rn(f.x * sc, f.y * sc);
        }
      }
    }
    reinterpret_cast<uint4*>(dst + (long long)r * width)[v] = o;
  }
}

__global__ void __launch_bounds__(256) combine_rows_kernel(__nv_bfloat16* __restrict__ out,
                                                           const __nv_bfloat16* __restrict__ src,
                                                           const int* __restrict__ pos, const float* __restrict__ w,
                                                           const __nv_bfloat16* __restrict__ add, float add_scale,
                                                           int tokens, int k, int width, int src_rows) {
  const int nvec = width >> 3;
  const long long total = (long long)tokens * nvec;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int t = (int)(i / nvec), v = (int)(i % nvec);
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
    if (add) {
      uint4 a = reinterpret_cast<const uint4*>(add + (long long)t * width)[v];
      const __nv_bfloat162* a2 = reinterpret_cast<const __nv_bfloat162*>(&a);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float2 f = __bfloat1622float2(a2[j]);
        acc[2 * j] = f.x * add_scale;
        acc[2 * j + 1] = f.y * add_scale;
      }
    }
    for (int j = 0; j < k; ++j) {
      const int p = pos[(long long)t * k + j];
      if (p < 0) continue;
      if (p >= src_rows) {
        if (v == 0) record_index_error(2, t, p, src_rows);
        continue;
      }
      const float wt = w ? w[(long long)t * k + j] : 1.f;
      uint4 x = reinterpret_cast<const uint4*>(src + (long long)p * width)[v];
      const __nv_bfloat162* x2 = reinterpret_cast<const __nv_bfloat162*>(&x);
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        float2 f = __bfloat1622float2(x2[q]);
        acc[2 * q] += wt * f.x;
        acc[2 * q + 1] += wt * f.y;
      }
    }
    uint4 o;
    o.x = pack_bf16x2(acc[0], acc[1]);
    o.y = pack_bf16x2(acc[2], acc[3]);
    o.z = pack_bf16x2(acc[4], acc[5]);
    o.w = pack_bf16x2(acc[6], acc[7]);
    reinterpret_cast<uint4*>(out + (long long)t * width)[v] = o;
  }
}

// one warp per (token, slot)
__global__ void __launch_bounds__(256) row_dots_kernel(float* __restrict__ dots, const __nv_bfloat16* __restrict__ a,
                                                       const __nv_bfloat16* __restrict__ b,
                                                       const int* __restrict__ pos, int tokens, int k, int width) {
  const int lane = threadIdx.x & 31;
  const int nvec = width >> 3;
  const long long total = (long long)tokens * k;
  for (long long i = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); i < total;
       i += (long long)gridDim.x * (blockDim.x >> 5)) {
    const long long t = i / k;
    const int p = pos[i];
    float acc = 0.f;
    if (p >= 0) {
      for (int v = lane; v < nvec; v += 32) {
        uint4 x = reinterpret_cast<const uint4*>(a + t * width)[v];
        uint4 y = reinterpret_cast<const uint4*>(b + (long long)p * width)[v];
        const __nv_bfloat162* x2 = reinterpret_cast<const __nv_bfloat162*>(&x);
        const __nv_bfloat162* y2 = reinterpret_cast<const __nv_bfloat162*>(&y);
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          float2 f = __bfloat1622float2(x2[q]), g = __bfloat1622float2(y2[q]);
          acc += f.x * g.x + f.y * g.y;
        }
      }
    }
    acc = warp_sum(acc);
    if (lane == 0) dots[i] = acc;
  }
}

// ---------------------------------------------------------------- optimizer updates
template <bool GRAD_F32>
__global__ void __launch_bounds__(256) adamw_flat_kernel(float* __restrict__ master, float* __restrict__ m,
                                                         float* __restrict__ v, const void* __restrict__ grad,
                                                         __nv_bfloat16* __restrict__ pb, long long n, float lr,
                                                         float beta1, float beta2, float eps, float wd, float bc1,
                                                         float bc2, const float* __restrict__ gsp, float gs,
                                                         const float* __restrict__ hyper) {
  const float scale = gsp ? (*gsp) * gs : gs;
  if (hyper) {  // device-resident hyper-parameters (CUDA-graph replay): lr, bias corrections
    lr = hyper[0];
    bc1 = hyper[1];
    bc2 = hyper[2];
  }
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    float g = GRAD_F32 ? reinterpret_cast<const float*>(grad)[i]
                       : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(grad)[i]);
    g *= scale;
    float mi = beta1 * m[i] + (1.f - beta1) * g;
    float vi = beta2 * v[i] + (1.f - beta2) * g * g;
    m[i] = mi;
    v[i] = vi;
    float p = master[i];
    p = p * (1.f - lr * wd) - lr * (mi / bc1) / (sqrtf(vi / bc2) + eps);
    master[i] = p;
    if (pb) pb[i] = __float2bfloat16(p);
  }
}

template <bool IS_F32>
__global__ void __launch_bounds__(256) sumsq_kernel(const void* __restrict__ x, long long n, float* __restrict__ out) {
  __shared__ float red[8];
  float acc = 0.f;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    float f = IS_F32 ? reinterpret_cast<const float*>(x)[i]
                     : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(x)[i]);
    acc += f * f;
  }
  acc = block_sum<256>(acc, red);
  if (threadIdx.x == 0) atomicAdd(out, acc);
}

template <bool GRAD_F32>
__global__ void __launch_bounds__(256) muon_momentum_kernel(float* __restrict__ mom, const void* __restrict__ grad,
                                                            __nv_bfloat16* __restrict__ u, long long n, float beta,
                                                            bool nesterov, const float* __restrict__ gsp) {
  const float scale = gsp ? *gsp : 1.f;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    float g = GRAD_F32 ? reinterpret_cast<const float*>(grad)[i]
                       : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(grad)[i]);
    g *= scale;
    // lerp form of the reference: M <- beta*M + (1-beta)*G ; U = nesterov ? lerp(G, M, beta) : M
    float mi = beta * mom[i] + (1.f - beta) * g;
    mom[i] = mi;
    float ui = nesterov ? (g * (1.f - beta) + mi * beta) : mi;
    u[i] = __float2bfloat16(ui);
  }
}

__global__ void __launch_bounds__(256) muon_apply_kernel(float* __restrict__ master,
                                                         const __nv_bfloat16* __restrict__ o,
                                                         __nv_bfloat16* __restrict__ pb, long long n, float lr, float wd,
                                                         float scale, const float* __restrict__ hyper) {
  if (hyper) lr = hyper[3];
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    float p = master[i] * (1.f - lr * wd) - lr * scale * __bfloat162float(o[i]);
    master[i] = p;
    if (pb) pb[i] = __float2bfloat16(p);
  }
}

__global__ void __launch_bounds__(256) axpby_bf16_kernel(__nv_bfloat16* __restrict__ x,
                                                         const __nv_bfloat16* __restrict__ y, float a, float b,
                                                         long long n) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
    x[i] = __float2bfloat16(a * __bfloat162float(x[i]) + b * __bfloat162float(y[i]));
}

// Newton-Schulz set-up for a stack of matrices X [K, m, n] (m <= n, bf16, rows contiguous): Frobenius norm, a four-step
// power iteration for the largest singular value (v <- X^T X v from the constant start vector, the deterministic
// estimate of triune/kernels/fast_muon.py:15-91), and Y = X / max(1.15 sigma, ||X||_F / sqrt(m), 0.7 ||X||_F) so that the
// quintic iteration starts inside its basin. Replaces nine fp32 library products and three reductions per shape group.
//
// Every matrix is split by rows over several CTAs, and one launch is one power-iteration step done in ONE pass over X:
// a CTA stages 8 rows in shared memory, its warps form u_r = x_r . v for those rows, then every thread adds u_r x_r into
// the columns it owns (registers), so X^T (X v) needs no second read. The partial X^T u of a CTA goes to the next
// vector with fp32 atomics; the next launch normalises it while loading. (One CTA per matrix, the first form of this
// kernel, read a 1536 x 6144 matrix ten times at the bandwidth of one SM: 7 ms per call on the 1.5 B-class models.)
constexpr int NSP_THREADS = 256;
constexpr int NSP_ROWS = 8;  // rows per shared-memory tile = warps per CTA
__global__ void __launch_bounds__(NSP_THREADS) ns_power_step_kernel(const __nv_bfloat16* __restrict__ X,
                                                                    const float* __restrict__ v_in, float* __restrict__ v_out,
                                                                    float* __restrict__ fro2, float* __restrict__ sigma2, int m,
                                                                    int n, int rows_per_cta, float eps) {
  extern __shared__ __align__(16) uint8_t nsp_raw[];
  float* v = reinterpret_cast<float*>(nsp_raw);                                   // [n]
  __nv_bfloat16* tile = reinterpret_cast<__nv_bfloat16*>(nsp_raw + (size_t)n * 4);  // [NSP_ROWS][n]
  __shared__ float red[NSP_THREADS / 32];
  __shared__ float u[NSP_ROWS];
  const int k = blockIdx.y;
  const __nv_bfloat16* x = X + (long long)k * m * n;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nvec = n >> 3;
  // the iterate, normalised here (the previous launch left it as a sum of partial products)
  if (v_in) {
    float s2 = 0.f;
    for (int c = tid; c < n; c += NSP_THREADS) {
      const float t = v_in[(long long)k * n + c];
      v[c] = t;
      s2 += t * t;
    }
    const float inv = 1.f / fmaxf(sqrtf(block_sum<NSP_THREADS>(s2, red)), eps);
    for (int c = tid; c < n; c += NSP_THREADS) v[c] *= inv;
  } else {
    const float v0 = rsqrtf((float)n);
    for (int c = tid; c < n; c += NSP_THREADS) v[c] = v0;
  }
  __syncthreads();
  constexpr int MAXV = 6;  // column vectors (8 columns each) per thread: n <= 6 * 8 * 256 = 12288
  float acc[MAXV][8];
#pragma unroll
  for (int q = 0; q < MAXV; ++q)
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[q][j] = 0.f;
  float ss = 0.f, su = 0.f;
  const int r_begin = blockIdx.x * rows_per_cta;
  const int r_end = min(m, r_begin + rows_per_cta);
  for (int r0 = r_begin; r0 < r_end; r0 += NSP_ROWS) {
    const int rows = min(NSP_ROWS, r_end - r0);
    for (int i = tid; i < rows * nvec; i += NSP_THREADS)
      reinterpret_cast<uint4*>(tile)[i] = reinterpret_cast<const uint4*>(x + (long long)r0 * n)[i];
    __syncthreads();
    if (warp < rows) {
      const uint4* row = reinterpret_cast<const uint4*>(tile + (size_t)warp * n);
      float a = 0.f, sq = 0.f;
      for (int c8 = lane; c8 < nvec; c8 += 32) {
        const uint4 w4 = row[c8];
        const __nv_bfloat162* p2 = reinterpret_cast<const __nv_bfloat162*>(&w4);
        const float* vp = v + c8 * 8;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 f = __bfloat1622float2(p2[j]);
          a += f.x * vp[2 * j] + f.y * vp[2 * j + 1];
          sq += f.x * f.x + f.y * f.y;
        }
      }
      a = warp_sum(a);
      sq = warp_sum(sq);
      if (lane == 0) {
        u[warp] = a;
        ss += sq;
        su += a * a;
      }
    }
    __syncthreads();
#pragma unroll
    for (int q = 0; q < MAXV; ++q) {
      const int c8 = tid + q * NSP_THREADS;
      if (c8 < nvec) {
        for (int r = 0; r < rows; ++r) {
          const uint4 w4 = reinterpret_cast<const uint4*>(tile + (size_t)r * n)[c8];
          const __nv_bfloat162* p2 = reinterpret_cast<const __nv_bfloat162*>(&w4);
          const float ur = u[r];
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float2 f = __bfloat1622float2(p2[j]);
            acc[q][2 * j] += f.x * ur;
            acc[q][2 * j + 1] += f.y * ur;
          }
        }
      }
    }
    __syncthreads();
  }
  if (v_out) {
#pragma unroll
    for (int q = 0; q < MAXV; ++q) {
      const int c8 = tid + q * NSP_THREADS;
      if (c8 < nvec) {
        float* dst = v_out + (long long)k * n + c8 * 8;
#pragma unroll
        for (int j = 0; j < 8; ++j) atomicAdd(dst + j, acc[q][j]);
      }
    }
  }
  if (lane == 0) {
    if (fro2) atomicAdd(fro2 + k, ss);
    if (sigma2) atomicAdd(sigma2 + k, su);
  }
}

__global__ void __launch_bounds__(256) ns_scale_kernel(const __nv_bfloat16* __restrict__ X, __nv_bfloat16* __restrict__ Y,
                                                       const float* __restrict__ fro2, const float* __restrict__ sigma2,
                                                       long long per_matrix_vec, long long total_vec, int m, float eps) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total_vec; i += (long long)gridDim.x * blockDim.x) {
    const int k = (int)(i / per_matrix_vec);
    const float fro = fmaxf(sqrtf(fro2[k]), eps), sigma = sqrtf(sigma2[k]);
    const float sc = 1.f / fmaxf(fmaxf(1.15f * sigma, fro * rsqrtf((float)m)), 0.7f * fro);
    uint4 w4 = reinterpret_cast<const uint4*>(X)[i];
    __nv_bfloat162* p2 = reinterpret_cast<__nv_bfloat162*>(&w4);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 f = __bfloat1622float2(p2[j]);
      p2[j] = __floats2bfloat162_rn(f.x * sc, f.y * sc);
    }
    reinterpret_cast<uint4*>(Y)[i] = w4;
  }
}

__global__ void __launch_bounds__(256) triangular_adamw_kernel(const float* __restrict__ S, float* __restrict__ m,
                                                               float* __restrict__ v, float* __restrict__ delta,
                                                               long long total, int r1, float beta1, float beta2,
                                                               float eps, float bc1, float bc2, bool triu,
                                                               const float* __restrict__ hyper) {
  if (hyper) {
    bc1 = hyper[5];
    bc2 = hyper[6];
  }
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int within = (int)(i % ((long long)r1 * r1));
    const int row = within / r1, col = within % r1;
    const bool keep = !triu || row <= col;
    const float s = keep ? S[i] : 0.f;
    float mi = beta1 * m[i] + (1.f - beta1) * s;
    float vi = beta2 * v[i] + (1.f - beta2) * s * s;
    m[i] = mi;
    v[i] = vi;
    delta[i] = keep ? (mi / bc1) / (sqrtf(vi / bc2) + eps) : 0.f;
  }
}

__global__ void __launch_bounds__(256) steer_update_kernel(float* __restrict__ P, const float* __restrict__ G,
                                                           long long n, float momentum, float steer) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const float p = P[i];
    P[i] = momentum * p + steer * (G[i] - p);
  }
}

// ---------------------------------------------------------------- routing tiers / rendering
__global__ void __launch_bounds__(256) route_tiers_kernel(const float* __restrict__ logits, int* __restrict__ tiers,
                                                          int* __restrict__ all_reflex, int rows, float threshold) {
  const int r = blockIdx.x * blockDim.x + threadIdx.x;
  bool not_reflex = false;
  if (r < rows) {
    const float a = logits[3 * r], b = logits[3 * r + 1], c = logits[3 * r + 2];
    const float mx = fmaxf(a, fmaxf(b, c));
    const float ea = __expf(a - mx), eb = __expf(b - mx), ec = __expf(c - mx);
    const float inv = 1.f / (ea + eb + ec);
    const int tier = (ea * inv >= threshold) ? 0 : (eb >= ec ? 1 : 2);
    tiers[r] = tier;
    not_reflex = tier != 0;
  }
  const unsigned any = __ballot_sync(0xffffffffu, not_reflex);
  if ((threadIdx.x & 31) == 0 && any != 0u && all_reflex) atomicExch(all_reflex, 0);
}

__global__ void __launch_bounds__(256) heatmap_bins_kernel(const float* __restrict__ act, long long n, int num_bins,
                                                           float* __restrict__ bins) {
  __shared__ float red[8];
  const int b = blockIdx.x;
  const long long per = n / num_bins > 0 ? n / num_bins : 1;
  const long long s = (long long)b * per;
  long long e = (b == num_bins - 1) ? n : s + per;
  if (e > n) e = n;
  float acc = 0.f;
  for (long long i = s + threadIdx.x; i < e; i += blockDim.x) acc += fabsf(act[i]);
  acc = block_sum<256>(acc, red);
  if (threadIdx.x == 0) bins[b] = e > s ? acc / (float)(e - s) : 0.f;
}

__global__ void __launch_bounds__(256) heatmap_colour_kernel(const float* __restrict__ bins, int num_bins,
                                                             uint32_t* __restrict__ rgba) {
  __shared__ float red[8];
  float mx = 0.f;
  for (int i = threadIdx.x; i < num_bins; i += blockDim.x) mx = fmaxf(mx, bins[i]);
  mx = block_max<256>(mx, red);
  mx = fmaxf(mx, 1e-12f);
  for (int i = threadIdx.x; i < num_bins; i += blockDim.x) {
    const float vn = bins[i] / mx;
    const uint32_t r = (uint32_t)(fminf(1.f, 1.4f * vn) * 249.f);
    const uint32_t g = (uint32_t)(vn * vn * 115.f);
    const uint32_t b = (uint32_t)((1.f - 0.7f * vn) * 60.f);
    rgba[i] = (255u << 24) | (b << 16) | (g << 8) | r;
  }
}

__global__ void __launch_bounds__(256) tier_render_kernel(const float* __restrict__ act, const int* __restrict__ tiers,
                                                          uint32_t* __restrict__ rgba, int rows, int width) {
  const long long total = (long long)rows * width;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int r = (int)(i / width);
    const int t = tiers[r];
    const float cr = t == 0 ? 16.f : (t == 1 ? 245.f : 139.f);
    const float cg = t == 0 ? 185.f : (t == 1 ? 158.f : 92.f);
    const float cb = t == 0 ? 129.f : (t == 1 ? 11.f : 246.f);
    const float inten = fminf(1.f, fabsf(act[i]));
    const uint32_t R = (uint32_t)(cr * inten), G = (uint32_t)(cg * inten), B = (uint32_t)(cb * inten);
    rgba[i] = (255u << 24) | (B << 16) | (G << 8) | R;
  }
}

inline int flat_grid(long long n, int threads = 256) {
  long long b = (n + threads - 1) / threads;
  const long long cap = 148ll * 16;
  return (int)(b < 1 ? 1 : (b > cap ? cap : b));
}

}  // namespace

void launch_ce_fwd_bwd(__nv_bfloat16* logits, long long ld, const long long* targets, float* row_loss, int rows, int V,
                       long long ignore_index, float grad_scale, cudaStream_t s, __nv_bfloat16* grad_dst) {
  if (rows == 0) return;
  ce_fwd_bwd_kernel<<<rows, CE_THREADS, 0, s>>>(logits, ld, targets, row_loss, V, ignore_index, grad_scale, grad_dst);
}

void launch_gather_rows(__nv_bfloat16* dst, const __nv_bfloat16* src, const int* row_src, const float* row_scale,
                        int dst_rows, int width, int src_rows, cudaStream_t s) {
  if (dst_rows == 0) return;
  gather_rows_kernel<<<flat_grid((long long)dst_rows * (width >> 3)), 256, 0, s>>>(dst, src, row_src, row_scale,
                                                                                    dst_rows, width, src_rows);
}

void launch_combine_rows(__nv_bfloat16* out, const __nv_bfloat16* src, const int* pos, const float* w,
                         const __nv_bfloat16* add, float add_scale, int tokens, int k, int width, int src_rows,
                         cudaStream_t s) {
  if (tokens == 0) return;
  combine_rows_kernel<<<flat_grid((long long)tokens * (width >> 3)), 256, 0, s>>>(out, src, pos, w, add, add_scale,
                                                                                   tokens, k, width, src_rows);
}

void index_error_word(int out[4], bool clear) {
  cudaMemcpyFromSymbol(out, g_index_error, sizeof(int) * 4);
  if (clear) {
    const int zero[4] = {0, 0, 0, 0};
    cudaMemcpyToSymbol(g_index_error, zero, sizeof(zero));
  }
}

void launch_row_dots(float* dots, const __nv_bfloat16* a, const __nv_bfloat16* b, const int* pos, int tokens, int k,
                     int width, cudaStream_t s) {
  if (tokens == 0) return;
  row_dots_kernel<<<flat_grid((long long)tokens * k * 32), 256, 0, s>>>(dots, a, b, pos, tokens, k, width);
}

void launch_adamw_flat(float* master, float* m, float* v, const void* grad, bool grad_is_f32, __nv_bfloat16* param_bf16,
                       long long n, float lr, float beta1, float beta2, float eps, float weight_decay,
                       float bias_corr1, float bias_corr2, const float* grad_scale_ptr, float grad_scale,
                       const float* hyper, cudaStream_t s) {
  if (n == 0) return;
  if (grad_is_f32)
    adamw_flat_kernel<true><<<flat_grid(n), 256, 0, s>>>(master, m, v, grad, param_bf16, n, lr, beta1, beta2, eps,
                                                         weight_decay, bias_corr1, bias_corr2, grad_scale_ptr,
                                                         grad_scale, hyper);
  else
    adamw_flat_kernel<false><<<flat_grid(n), 256, 0, s>>>(master, m, v, grad, param_bf16, n, lr, beta1, beta2, eps,
                                                          weight_decay, bias_corr1, bias_corr2, grad_scale_ptr,
                                                          grad_scale, hyper);
}

void launch_sumsq(const void* x, bool is_f32, long long n, float* out, cudaStream_t s) {
  if (n == 0) return;
  if (is_f32)
    sumsq_kernel<true><<<flat_grid(n), 256, 0, s>>>(x, n, out);
  else
    sumsq_kernel<false><<<flat_grid(n), 256, 0, s>>>(x, n, out);
}

void launch_muon_momentum(float* mom, const void* grad, bool grad_is_f32, __nv_bfloat16* u_out, long long n, float beta,
                          bool nesterov, const float* grad_scale_ptr, cudaStream_t s) {
  if (n == 0) return;
  if (grad_is_f32)
    muon_momentum_kernel<true><<<flat_grid(n), 256, 0, s>>>(mom, grad, u_out, n, beta, nesterov, grad_scale_ptr);
  else
    muon_momentum_kernel<false><<<flat_grid(n), 256, 0, s>>>(mom, grad, u_out, n, beta, nesterov, grad_scale_ptr);
}

void launch_muon_apply(float* master, const __nv_bfloat16* o, __nv_bfloat16* param_bf16, long long n, float lr,
                       float wd, float scale, const float* hyper, cudaStream_t s) {
  if (n == 0) return;
  muon_apply_kernel<<<flat_grid(n), 256, 0, s>>>(master, o, param_bf16, n, lr, wd, scale, hyper);
}

void launch_ns_prepare(const __nv_bfloat16* X, __nv_bfloat16* Y, int batch, int m, int n, float eps, float* scratch,
                       cudaStream_t s) {
  // scratch: fp32 [2 * batch * n + 2 * batch]: two iterate buffers, then ||X||_F^2 and sigma^2 per matrix
  if (batch <= 0) return;
  if (n > 6 * 8 * NSP_THREADS || (size_t)n * 20 > 226 * 1024) throw std::runtime_error("ns_prepare: n <= 11568");
  const size_t smem = (size_t)n * 4 + (size_t)NSP_ROWS * n * 2;
  constexpr int kMaxDyn = 226 * 1024;  // the kernel also has a few static words; 227 KB is the limit for both together
  if (smem > (size_t)kMaxDyn) throw std::runtime_error("ns_prepare: the iterate and an 8-row tile do not fit shared memory");
  static PerDeviceOnce once;
  if (once.first_use()) {
    cudaError_t e = cudaFuncSetAttribute(ns_power_step_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kMaxDyn);
    if (e != cudaSuccess) throw std::runtime_error(std::string("ns_prepare: cannot set shared memory size: ") + cudaGetErrorString(e));
  }
  float* va = scratch;
  float* vb = scratch + (size_t)batch * n;
  float* fro2 = scratch + 2 * (size_t)batch * n;
  float* sigma2 = fro2 + batch;
  // rows per CTA: enough CTAs to fill the GPU a few times over, whole 8-row tiles
  int splits = (148 * 4 + batch - 1) / batch;
  int rows_per_cta = (m + splits - 1) / splits;
  rows_per_cta = (rows_per_cta + NSP_ROWS - 1) / NSP_ROWS * NSP_ROWS;
  splits = (m + rows_per_cta - 1) / rows_per_cta;
  const dim3 grid((unsigned)splits, (unsigned)batch, 1);
  cudaMemsetAsync(fro2, 0, sizeof(float) * 2 * batch, s);
  const float* vin = nullptr;
  for (int it = 0; it < 5; ++it) {
    float* vout = (it & 1) ? vb : va;
    const bool last = it == 4;
    if (!last) cudaMemsetAsync(vout, 0, sizeof(float) * (size_t)batch * n, s);
    ns_power_step_kernel<<<grid, NSP_THREADS, smem, s>>>(X, vin, last ? nullptr : vout, it == 0 ? fro2 : nullptr,
                                                         last ? sigma2 : nullptr, m, n, rows_per_cta, eps);
    vin = vout;
  }
  const long long per = (long long)m * (n >> 3), total = per * batch;
  ns_scale_kernel<<<flat_grid(total), 256, 0, s>>>(X, Y, fro2, sigma2, per, total, m, eps);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) throw std::runtime_error(std::string("ns_prepare launch failed: ") + cudaGetErrorString(e));
}

void launch_axpby_bf16(__nv_bfloat16* x, const __nv_bfloat16* y, float a, float b, long long n, cudaStream_t s) {
  if (n == 0) return;
  axpby_bf16_kernel<<<flat_grid(n), 256, 0, s>>>(x, y, a, b, n);
}

void launch_triangular_adamw(const float* S, float* m, float* v, float* delta, int nmat, int r1, float beta1,
                             float beta2, float eps, float bias_corr1, float bias_corr2, bool triu, const float* hyper,
                             cudaStream_t s) {
  const long long total = (long long)nmat * r1 * r1;
  if (total == 0) return;
  triangular_adamw_kernel<<<flat_grid(total), 256, 0, s>>>(S, m, v, delta, total, r1, beta1, beta2, eps, bias_corr1,
                                                           bias_corr2, triu, hyper);
}

void launch_steer_update(float* P, const float* G, long long n, float momentum, float steer, cudaStream_t s) {
  if (n == 0) return;
  steer_update_kernel<<<flat_grid(n), 256, 0, s>>>(P, G, n, momentum, steer);
}

void launch_route_tiers(const float* logits, int* tiers, int* all_reflex, int rows, float threshold, cudaStream_t s) {
  if (rows == 0) return;
  route_tiers_kernel<<<(rows + 255) / 256, 256, 0, s>>>(logits, tiers, all_reflex, rows, threshold);
}

void launch_neuron_heatmap(const float* act, long long n, int num_bins, float* bin_scratch, uint32_t* rgba,
                           cudaStream_t s) {
  if (num_bins == 0) return;
  heatmap_bins_kernel<<<num_bins, 256, 0, s>>>(act, n, num_bins, bin_scratch);
  heatmap_colour_kernel<<<1, 256, 0, s>>>(bin_scratch, num_bins, rgba);
}

void launch_tier_render(const float* act, const int* tiers, uint32_t* rgba, int rows, int width, cudaStream_t s) {
  if (rows == 0) return;
  tier_render_kernel<<<flat_grid((long long)rows * width), 256, 0, s>>>(act, tiers, rgba, rows, width);
}

}  // namespace tb
