// Stand-alone bandwidth-bound operators: SwiGLU forward / backward, rotary embedding (forward and, with the sine
// negated, backward), and the embedding gradient as a scatter-add into the fp32 gradient arena.
//
// Inside the FFN the SwiGLU arithmetic is an epilogue of the tcgen05 GEMM (gemm/tc_gemm_impl.cuh); these kernels serve
// callers that hold gate and up as separate tensors, the softmax-attention mixer (RoPE outside the GLA feature map)
// and the token embedding. Reference semantics: triune/kernels/fast_swiglu.py:19-45, csrc/kernels/swiglu.cu:14-47,
// triune/kernels/fast_rope.py:16-80 of the reference project.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../common/ptx.cuh"
#include "elementwise.cuh"

namespace tb {

namespace {

__device__ __forceinline__ void unpack8f(const uint4& u, float (&f)[8]) {
  const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 t = __bfloat1622float2(p[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}
__device__ __forceinline__ uint4 pack8f(const float (&f)[8]) {
  uint4 u;
  u.x = pack_bf16x2(f[0], f[1]);
  u.y = pack_bf16x2(f[2], f[3]);
  u.z = pack_bf16x2(f[4], f[5]);
  u.w = pack_bf16x2(f[6], f[7]);
  return u;
}
__device__ __forceinline__ float sigmoidf_fast(float x) { return __fdividef(1.0f, 1.0f + __expf(-x)); }

inline int flat_blocks(long long work, int threads) {
  long long b = (work + threads - 1) / threads;
  const long long cap = 148ll * 16;
  return (int)(b < 1 ? 1 : (b > cap ? cap : b));
}

// out[r, c] = silu(gate[r, c]) * up[r, c]; rows of `width` bf16 (width % 8 == 0) with independent row pitches, so
// gate and up may be the two halves of one fused projection output.
__global__ void __launch_bounds__(256) swiglu_fwd_kernel(const __nv_bfloat16* __restrict__ gate, long long ld_g,
                                                         const __nv_bfloat16* __restrict__ up, long long ld_u,
                                                         __nv_bfloat16* __restrict__ out, long long ld_o, long long rows,
                                                         int width) {
  const int nvec = width >> 3;
  const long long total = rows * nvec;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / nvec;
    const int v = (int)(i % nvec);
    float g[8], u[8], o[8];
    unpack8f(reinterpret_cast<const uint4*>(gate + r * ld_g)[v], g);
    unpack8f(reinterpret_cast<const uint4*>(up + r * ld_u)[v], u);
#pragma unroll
    for (int j = 0; j < 8; ++j) o[j] = g[j] * sigmoidf_fast(g[j]) * u[j];
    reinterpret_cast<uint4*>(out + r * ld_o)[v] = pack8f(o);
  }
}

// d(gate) = dh * up * silu'(gate), d(up) = dh * silu(gate), silu'(g) = s (1 + g (1 - s)), s = sigmoid(g).
__global__ void __launch_bounds__(256) swiglu_bwd_kernel(const __nv_bfloat16* __restrict__ gate, long long ld_g,
                                                         const __nv_bfloat16* __restrict__ up, long long ld_u,
                                                         const __nv_bfloat16* __restrict__ dh, long long ld_d,
                                                         __nv_bfloat16* __restrict__ dgate, long long ld_dg,
                                                         __nv_bfloat16* __restrict__ dup, long long ld_du, long long rows,
                                                         int width) {
  const int nvec = width >> 3;
  const long long total = rows * nvec;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / nvec;
    const int v = (int)(i % nvec);
    float g[8], u[8], d[8], og[8], ou[8];
    unpack8f(reinterpret_cast<const uint4*>(gate + r * ld_g)[v], g);
    unpack8f(reinterpret_cast<const uint4*>(up + r * ld_u)[v], u);
    unpack8f(reinterpret_cast<const uint4*>(dh + r * ld_d)[v], d);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float s = sigmoidf_fast(g[j]);
      og[j] = d[j] * u[j] * s * (1.0f + g[j] * (1.0f - s));
      ou[j] = d[j] * g[j] * s;
    }
    reinterpret_cast<uint4*>(dgate + r * ld_dg)[v] = pack8f(og);
    reinterpret_cast<uint4*>(dup + r * ld_du)[v] = pack8f(ou);
  }
}

// Half-split rotary embedding over x [rows = B*T, H, D] (row pitch ld, heads contiguous): for every pair
// (x1, x2) = (x[..., j], x[..., j + D/2]):  y1 = x1 c - sign * x2 s,  y2 = x2 c + sign * x1 s  with c, s from
// cos/sin [T, D/2] (fp32) at position (row % T). sign = +1 rotates, sign = -1 is the transpose (the gradient).
__global__ void __launch_bounds__(256) rope_kernel(const __nv_bfloat16* __restrict__ x, long long ld_x,
                                                   __nv_bfloat16* __restrict__ y, long long ld_y,
                                                   const float* __restrict__ cs, const float* __restrict__ sn,
                                                   long long rows, int T, int H, int D, float sign) {
  const int half = D >> 1, hv = half >> 3;  // 16-byte vectors per half head
  const long long total = rows * H * hv;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int v = (int)(i % hv);
    const long long rh = i / hv;
    const int h = (int)(rh % H);
    const long long r = rh / H;
    const int t = (int)(r % T);
    const __nv_bfloat16* xp = x + r * ld_x + (long long)h * D + v * 8;
    __nv_bfloat16* yp = y + r * ld_y + (long long)h * D + v * 8;
    float a[8], b[8], oa[8], ob[8];
    unpack8f(*reinterpret_cast<const uint4*>(xp), a);
    unpack8f(*reinterpret_cast<const uint4*>(xp + half), b);
    const float* cp = cs + (long long)t * half + v * 8;
    const float* sp = sn + (long long)t * half + v * 8;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float c = cp[j], s = sign * sp[j];
      oa[j] = a[j] * c - b[j] * s;
      ob[j] = b[j] * c + a[j] * s;
    }
    *reinterpret_cast<uint4*>(yp) = pack8f(oa);
    *reinterpret_cast<uint4*>(yp + half) = pack8f(ob);
  }
}

// grad[ids[n], :] += dy[n, :] for every token n (fp32 accumulation with vector reductions; tokens with an id
// outside [0, V) are skipped). width % 4 == 0.
__global__ void __launch_bounds__(256) embedding_bwd_kernel(const __nv_bfloat16* __restrict__ dy, long long ld,
                                                            const long long* __restrict__ ids, float* __restrict__ grad,
                                                            long long tokens, int width, long long V) {
  const int nvec = width >> 2;
  const long long total = tokens * nvec;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long n = i / nvec;
    const int v = (int)(i % nvec);
    const long long id = ids[n];
    if (id < 0 || id >= V) continue;
    const uint2 raw = *reinterpret_cast<const uint2*>(dy + n * ld + v * 4);
    const float2 lo = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
    const float2 hi = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
    float* dst = grad + id * width + v * 4;
    asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst), "f"(lo.x), "f"(lo.y), "f"(hi.x), "f"(hi.y)
                 : "memory");
  }
}

}  // namespace

void launch_swiglu_fwd(const __nv_bfloat16* gate, long long ld_g, const __nv_bfloat16* up, long long ld_u,
                       __nv_bfloat16* out, long long ld_o, long long rows, int width, cudaStream_t s) {
  if (rows <= 0 || width <= 0) return;
  swiglu_fwd_kernel<<<flat_blocks(rows * (width >> 3), 256), 256, 0, s>>>(gate, ld_g, up, ld_u, out, ld_o, rows, width);
}

void launch_swiglu_bwd(const __nv_bfloat16* gate, long long ld_g, const __nv_bfloat16* up, long long ld_u,
                       const __nv_bfloat16* dh, long long ld_d, __nv_bfloat16* dgate, long long ld_dg,
                       __nv_bfloat16* dup, long long ld_du, long long rows, int width, cudaStream_t s) {
  if (rows <= 0 || width <= 0) return;
  swiglu_bwd_kernel<<<flat_blocks(rows * (width >> 3), 256), 256, 0, s>>>(gate, ld_g, up, ld_u, dh, ld_d, dgate, ld_dg,
                                                                          dup, ld_du, rows, width);
}

void launch_rope(const __nv_bfloat16* x, long long ld_x, __nv_bfloat16* y, long long ld_y, const float* cs,
                 const float* sn, long long rows, int T, int H, int D, bool transpose, cudaStream_t s) {
  if (rows <= 0) return;
  rope_kernel<<<flat_blocks(rows * H * (D >> 4), 256), 256, 0, s>>>(x, ld_x, y, ld_y, cs, sn, rows, T, H, D,
                                                                    transpose ? -1.0f : 1.0f);
}

void launch_embedding_bwd(const __nv_bfloat16* dy, long long ld, const long long* ids, float* grad, long long tokens,
                          int width, long long V, cudaStream_t s) {
  if (tokens <= 0) return;
  embedding_bwd_kernel<<<flat_blocks(tokens * (width >> 2), 256), 256, 0, s>>>(dy, ld, ids, grad, tokens, width, V);
}

}  // namespace tb
