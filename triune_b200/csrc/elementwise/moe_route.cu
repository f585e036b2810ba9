// Mixture-of-experts routing and dispatch planning without a host round trip.
//
//   moe_route_topk     per token: softmax(logits / T), top-k on the biased logits, mixing weights from the unbiased
//                      probabilities renormalised over the selection; also emits one 64-bit sort key per assignment
//                      (expert | k-slot | descending weight) and per-(expert, slot) counts.
//   moe_route_bwd      gradient of the mixing weights with respect to the logits (probabilities are recomputed).
//   moe_plan_sorted    after ONE stable sort of the keys: capacity admission (per (slot, expert) the `cap` largest
//                      weights, ties to the lower token index) and the expert-major row of every accepted assignment,
//                      the source token of every buffer row, the expert of every 128-row tile and the padded expert
//                      offsets, all in closed form from the sorted position and the counts.
//
// Replaces the top-k / softmax / capacity / permutation chain of triune/model/moe.py:198-215 and :385-410, which in a
// PyTorch composition costs five sorts and a dozen scatter / cumsum launches per layer.
#include <cuda_runtime.h>
#include <stdint.h>

#include <stdexcept>
#include <string>

#include "elementwise.cuh"

namespace tb {
namespace {

constexpr int MAX_E = 64, MAX_K = 4;

// Sort keys: ascending key order = expert, then slot, then DEScending weight (weights are positive, so bit order = value
// order). Up to 32 experts the key fits 31 bits (5 + 2 + the top 24 bits of the weight: sign, exponent, 15 mantissa
// bits), which halves the passes and the bytes of the radix sort; weights closer than 2^-15 relative then count as
// ties and go to the lower token index like exact ties.
template <typename KeyT>
__device__ __forceinline__ KeyT make_route_key(int e, int j, float w) {
  if constexpr (sizeof(KeyT) == 4)
    return (KeyT)(((uint32_t)e << 26) | ((uint32_t)j << 24) | (0xFFFFFFu - (__float_as_uint(w) >> 8)));
  else
    return ((long long)e << 36) | ((long long)j << 32) | (long long)(0xFFFFFFFFu - __float_as_uint(w));
}
template <typename KeyT>
__device__ __forceinline__ void split_route_key(KeyT key, int& e, int& j) {
  if constexpr (sizeof(KeyT) == 4) {
    e = (int)((uint32_t)key >> 26);
    j = (int)(((uint32_t)key >> 24) & 3u);
  } else {
    e = (int)(key >> 36);
    j = (int)((key >> 32) & 0xF);
  }
}

template <typename KeyT>
__global__ void __launch_bounds__(256) moe_route_topk_kernel(const float* __restrict__ logits, const float* __restrict__ bias,
                                                             const float* __restrict__ temperature, float temp_value, int N, int E,
                                                             int K, long long* __restrict__ idx, float* __restrict__ w,
                                                             KeyT* __restrict__ keys, int* __restrict__ counts /*[E][K]*/) {
  __shared__ int hist[MAX_E * MAX_K];
  for (int i = threadIdx.x; i < E * K; i += blockDim.x) hist[i] = 0;
  __syncthreads();
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t < N) {
    const float inv_t = 1.0f / (temperature ? *temperature : temp_value);
    float l[MAX_E];
    float mx = -INFINITY;
    const float* row = logits + (long long)t * E;
#pragma unroll 8
    for (int e = 0; e < E; ++e) {
      l[e] = row[e];
      mx = fmaxf(mx, l[e] * inv_t);
    }
    float denom = 0.f;
    for (int e = 0; e < E; ++e) denom += __expf(l[e] * inv_t - mx);
    int sel[MAX_K];
    float pw[MAX_K];
    float psum = 0.f;
    unsigned long long taken = 0ull;
    for (int j = 0; j < K; ++j) {
      int best = 0;
      float bv = -INFINITY;
      for (int e = 0; e < E; ++e) {
        const float v = l[e] + bias[e];
        if (!((taken >> e) & 1ull) && v > bv) {  // strict >: ties go to the lower expert index, like torch.topk
          bv = v;
          best = e;
        }
      }
      taken |= 1ull << best;
      sel[j] = best;
      pw[j] = __expf(l[best] * inv_t - mx) / denom;
      psum += pw[j];
    }
    const float norm = K > 1 ? 1.0f / (psum + 1e-20f) : 1.0f;
    for (int j = 0; j < K; ++j) {
      const float wj = pw[j] * norm;
      idx[(long long)t * K + j] = sel[j];
      w[(long long)t * K + j] = wj;
      keys[(long long)t * K + j] = make_route_key<KeyT>(sel[j], j, wj);
      atomicAdd(&hist[sel[j] * K + j], 1);
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < E * K; i += blockDim.x)
    if (hist[i]) atomicAdd(&counts[i], hist[i]);
}

__global__ void __launch_bounds__(256) moe_route_bwd_kernel(const float* __restrict__ logits, const float* __restrict__ temperature,
                                                            float temp_value, const long long* __restrict__ idx,
                                                            const float* __restrict__ w, const float* __restrict__ dw, int N, int E,
                                                            int K, float* __restrict__ dlogits) {
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= N) return;
  const float inv_t = 1.0f / (temperature ? *temperature : temp_value);
  const float* row = logits + (long long)t * E;
  float p[MAX_E];
  float mx = -INFINITY;
  for (int e = 0; e < E; ++e) mx = fmaxf(mx, row[e] * inv_t);
  float denom = 0.f;
  for (int e = 0; e < E; ++e) {
    p[e] = __expf(row[e] * inv_t - mx);
    denom += p[e];
  }
  const float inv_d = 1.0f / denom;
  // w_j = p_j / S over the selection: dL/dp_j = (dw_j - sum_i dw_i w_i) / S, zero outside the selection
  float S = 0.f, dot = 0.f;
  for (int j = 0; j < K; ++j) {
    S += p[idx[(long long)t * K + j]] * inv_d;
    dot += dw[(long long)t * K + j] * w[(long long)t * K + j];
  }
  float g[MAX_K];
  float pg = 0.f;
  for (int j = 0; j < K; ++j) {
    g[j] = K > 1 ? (dw[(long long)t * K + j] - dot) / (S + 1e-20f) : dw[(long long)t * K + j];
    pg += p[idx[(long long)t * K + j]] * inv_d * g[j];
  }
  float* out = dlogits + (long long)t * E;
  for (int e = 0; e < E; ++e) out[e] = -inv_t * p[e] * inv_d * pg;
  for (int j = 0; j < K; ++j) {
    const int e = (int)idx[(long long)t * K + j];
    out[e] += inv_t * p[e] * inv_d * g[j];
  }
}

// One thread per SORTED assignment.
template <typename KeyT>
__global__ void __launch_bounds__(256) moe_plan_sorted_kernel(const KeyT* __restrict__ sorted_keys,
                                                              const long long* __restrict__ order, const int* __restrict__ counts,
                                                              int A, int E, int K, int cap, int R, int* __restrict__ pos,
                                                              unsigned char* __restrict__ keep, int* __restrict__ row_src,
                                                              int* __restrict__ tile_group, int* __restrict__ group_offsets,
                                                              long long* __restrict__ accepted /*[E]*/) {
  __shared__ int seg_start[MAX_E * MAX_K];   // first sorted index of (expert, slot)
  __shared__ int seg_base[MAX_E * MAX_K];    // first buffer row of (expert, slot)
  __shared__ int exp_pad_start[MAX_E + 1];   // padded row offset of each expert
  if (threadIdx.x == 0) {
    int run = 0, rows = 0;
    for (int e = 0; e < E; ++e) {
      exp_pad_start[e] = rows;
      int acc = 0;
      for (int j = 0; j < K; ++j) {
        const int c = counts[e * K + j];
        seg_start[e * K + j] = run;
        seg_base[e * K + j] = rows + acc;
        run += c;
        acc += c < cap ? c : cap;
      }
      rows += (acc + 255) / 256 * 256;  // whole pairs of 128-row tiles: the CTA-pair GEMM needs one expert per pair
      if (blockIdx.x == 0) accepted[e] = acc;
    }
    exp_pad_start[E] = rows;
  }
  __syncthreads();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < A) {
    int e, j;
    split_route_key<KeyT>(sorted_keys[i], e, j);
    const int a = (int)order[i];
    const int rank = i - seg_start[e * K + j];
    const bool ok = rank < cap;
    keep[a] = ok ? 1 : 0;
    const int row = seg_base[e * K + j] + rank;
    pos[a] = ok ? row : -1;
    if (ok) row_src[row] = a / K;
  }
  // tile table and offsets: one pass by the first threads of the grid
  const int tiles = R / 128;
  for (int tix = blockIdx.x * blockDim.x + threadIdx.x; tix < tiles; tix += gridDim.x * blockDim.x) {
    const int r0 = tix * 128;
    int g = -1;
    for (int e = 0; e < E; ++e)
      if (r0 >= exp_pad_start[e] && r0 < exp_pad_start[e + 1]) g = e;
    tile_group[tix] = g;
  }
  if (blockIdx.x == 0)
    for (int e = threadIdx.x; e <= E; e += blockDim.x) group_offsets[e] = exp_pad_start[e];
}

void check(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) throw std::runtime_error(std::string(what) + " launch failed: " + cudaGetErrorString(e));
}

}  // namespace

void launch_moe_route_topk(const float* logits, const float* bias, const float* temperature, float temp_value, int N, int E, int K,
                           long long* idx, float* w, void* keys, bool keys32, int* counts, cudaStream_t s) {
  if (E > MAX_E || K > MAX_K || K > E) throw std::runtime_error("moe_route_topk: at most 64 experts and top-4");
  cudaMemsetAsync(counts, 0, sizeof(int) * E * K, s);
  if (N <= 0) return;
  if (keys32) {
    if (E > 32) throw std::runtime_error("moe_route_topk: 32-bit sort keys hold at most 32 experts");
    moe_route_topk_kernel<int><<<(N + 255) / 256, 256, 0, s>>>(logits, bias, temperature, temp_value, N, E, K, idx, w, (int*)keys, counts);
  } else {
    moe_route_topk_kernel<long long><<<(N + 255) / 256, 256, 0, s>>>(logits, bias, temperature, temp_value, N, E, K, idx, w,
                                                                    (long long*)keys, counts);
  }
  check("moe_route_topk");
}

void launch_moe_route_bwd(const float* logits, const float* temperature, float temp_value, const long long* idx, const float* w,
                          const float* dw, int N, int E, int K, float* dlogits, cudaStream_t s) {
  if (N <= 0) return;
  moe_route_bwd_kernel<<<(N + 255) / 256, 256, 0, s>>>(logits, temperature, temp_value, idx, w, dw, N, E, K, dlogits);
  check("moe_route_bwd");
}

void launch_moe_plan_sorted(const void* sorted_keys, bool keys32, const long long* order, const int* counts, int A, int E, int K, int cap,
                            int R, int* pos, unsigned char* keep, int* row_src, int* tile_group, int* group_offsets,
                            long long* accepted, cudaStream_t s) {
  if (E > MAX_E || K > MAX_K) throw std::runtime_error("moe_plan_sorted: at most 64 experts and top-4");
  cudaMemsetAsync(row_src, 0xFF, sizeof(int) * (size_t)R, s);  // -1 = padding row
  if (keys32)
    moe_plan_sorted_kernel<int><<<(A + 255) / 256, 256, 0, s>>>((const int*)sorted_keys, order, counts, A, E, K, cap, R, pos, keep, row_src,
                                                                tile_group, group_offsets, accepted);
  else
    moe_plan_sorted_kernel<long long><<<(A + 255) / 256, 256, 0, s>>>((const long long*)sorted_keys, order, counts, A, E, K, cap, R, pos,
                                                                      keep, row_src, tile_group, group_offsets, accepted);
  check("moe_plan_sorted");
}

}  // namespace tb
