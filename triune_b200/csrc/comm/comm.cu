// Fused data-parallel step over NVLink: gradient reduce-scatter (peer loads or NVLS multimem.ld_reduce)
// + 1/world scale + grad-norm partials, then AdamW on the owned shard with the new bf16 parameters stored
// straight into every peer (peer stores or multimem.st): reduce-scatter, update and all-gather without NCCL.
//
// Replaces the reference's DDP all-reduce + clip_grad_norm_ + fused AdamW (triune/trainer/distributed.py:142-156,
// triune/trainer/engine.py:426-430).
#include "comm.cuh"

#include <stdexcept>
#include <string>

#include "../common/ptx.cuh"

namespace tb {

namespace {

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ float4 ld_peer_f4(const float* p) {
  float4 v;
  asm volatile("ld.volatile.global.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p));
  return v;
}
__device__ __forceinline__ float4 multimem_ld_reduce_f4(const float* mc) {
  float4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "l"(mc)
               : "memory");
  return v;
}
__device__ __forceinline__ void multimem_st_16B(void* mc, uint4 v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc), "f"(__uint_as_float(v.x)),
               "f"(__uint_as_float(v.y)), "f"(__uint_as_float(v.z)), "f"(__uint_as_float(v.w))
               : "memory");
}

__device__ __forceinline__ uint32_t* pad_of(const PeerTable& pt, int peer) {
  return reinterpret_cast<uint32_t*>(pt.signals[peer]);
}
__device__ __forceinline__ int slot(int channel, int src) { return channel * COMM_MAX_RANKS + src; }

// Bounded wait for `epoch` on (channel, src) of the LOCAL pad.
__device__ __forceinline__ bool wait_flag(const PeerTable& pt, int channel, int src, uint32_t epoch,
                                          unsigned long long limit_ns) {
  const uint32_t* p = pad_of(pt, pt.rank) + slot(channel, src);
  const unsigned long long t0 = globaltimer_ns();
  while (true) {
    if ((int)(ld_acquire_sys(p) - epoch) >= 0) return true;
    if (globaltimer_ns() - t0 > limit_ns) return false;
    __nanosleep(64);
  }
}

// Thread `threadIdx.x < world` waits for its peer; result combined over the CTA. All threads must call.
__device__ __forceinline__ bool cta_wait_all(const PeerTable& pt, int channel, uint32_t epoch, int* status,
                                             unsigned long long limit_ns = WAIT_LIMIT_NS) {
  __shared__ int ok_flag;
  if (threadIdx.x == 0) ok_flag = 1;
  __syncthreads();
  if (threadIdx.x < pt.world) {
    if (!wait_flag(pt, channel, threadIdx.x, epoch, limit_ns)) {
      ok_flag = 0;
      if (status) atomicCAS(status, 0, ST_TIMEOUT_PEER);
    }
  }
  __syncthreads();
  return ok_flag != 0;
}

__device__ __forceinline__ void signal_all(const PeerTable& pt, int channel, uint32_t epoch) {
  // caller guarantees prior writes are complete device-wide; make them visible system-wide first
  __threadfence_system();
  if (threadIdx.x < pt.world) st_release_sys(pad_of(pt, threadIdx.x) + slot(channel, pt.rank), epoch);
}

__device__ __forceinline__ float block_sum_256(float v, float* red) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  float t = (threadIdx.x & 31) < 8 ? red[threadIdx.x & 31] : 0.f;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
  return __shfl_sync(0xffffffffu, t, 0);
}

// ---------------------------------------------------------------- phase 1: reduce-scatter + norm partial
__global__ void __launch_bounds__(256) dp_reduce_scatter_kernel(PeerTable pt, long long grad_off, long long norm_off,
                                                                RangeList ranges, uint32_t epoch,
                                                                const uint32_t* __restrict__ epoch_dev, int use_multimem,
                                                                unsigned int* block_counter, int* status) {
  __shared__ float red[8];
  __shared__ int last_block;
  if (epoch_dev) epoch = *epoch_dev;  // device-resident epoch: the launch can be replayed from a CUDA graph
  // announce that this rank's gradients are final, then wait until every peer said the same
  if (blockIdx.x == 0) signal_all(pt, CH_GRADS_READY, epoch);
  const bool ok = cta_wait_all(pt, CH_GRADS_READY, epoch, status);
  float* local_grad = reinterpret_cast<float*>(pt.bufs[pt.rank] + grad_off);
  float* norm = reinterpret_cast<float*>(pt.bufs[pt.rank] + norm_off);  // [world] partials + [world] accumulator
  float ss = 0.f;
  if (ok) {
    const float inv = 1.0f / (float)pt.world;
    // A peer load takes a few microseconds to come back over NVLink; one 16-byte load per thread keeps about 1 MB in
    // flight, a fraction of the link's bandwidth-delay product. Each thread therefore owns U strided vectors per pass
    // and issues all of their loads (per peer) before the first add.
    constexpr int U = 4;
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (int r = 0; r < ranges.count; ++r) {
      const long long b4 = ranges.r[r].begin >> 2, e4 = ranges.r[r].end >> 2;
      for (long long i0 = b4 + (long long)blockIdx.x * blockDim.x + threadIdx.x; i0 < e4; i0 += stride * U) {
        float4 acc[U];
        if (use_multimem) {
#pragma unroll
          for (int u = 0; u < U; ++u) {
            const long long i = i0 + u * stride;
            acc[u] = i < e4 ? multimem_ld_reduce_f4(reinterpret_cast<const float*>(pt.multicast + grad_off) + i * 4)
                            : make_float4(0.f, 0.f, 0.f, 0.f);
          }
        } else {
#pragma unroll
          for (int u = 0; u < U; ++u) acc[u] = make_float4(0.f, 0.f, 0.f, 0.f);
          for (int p = 0; p < pt.world; ++p) {
            const int peer = (pt.rank + p) % pt.world;  // stagger so ranks do not all hit the same peer first
            const float* src = reinterpret_cast<const float*>(pt.bufs[peer] + grad_off);
            float4 v[U];
#pragma unroll
            for (int u = 0; u < U; ++u) {
              const long long i = i0 + u * stride;
              v[u] = i < e4 ? ld_peer_f4(src + i * 4) : make_float4(0.f, 0.f, 0.f, 0.f);
            }
#pragma unroll
            for (int u = 0; u < U; ++u) {
              acc[u].x += v[u].x; acc[u].y += v[u].y; acc[u].z += v[u].z; acc[u].w += v[u].w;
            }
          }
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const long long i = i0 + u * stride;
          if (i < e4) {
            float4 a = acc[u];
            a.x *= inv; a.y *= inv; a.z *= inv; a.w *= inv;
            reinterpret_cast<float4*>(local_grad)[i] = a;
            ss += a.x * a.x + a.y * a.y + a.z * a.z + a.w * a.w;
          }
        }
      }
    }
  }
  ss = block_sum_256(ss, red);
  if (threadIdx.x == 0) {
    atomicAdd(&norm[pt.world], ss);
    __threadfence();
    last_block = (atomicAdd(block_counter, 1u) == gridDim.x - 1) ? 1 : 0;
  }
  __syncthreads();
  if (last_block) {
    // every CTA of this rank is done reading peers: publish the partial and raise the flag
    if (threadIdx.x < pt.world) {
      const float total = *reinterpret_cast<volatile float*>(&norm[pt.world]);
      float* peer_norm = reinterpret_cast<float*>(pt.bufs[threadIdx.x] + norm_off);
      asm volatile("st.relaxed.sys.global.f32 [%0], %1;" ::"l"(peer_norm + pt.rank), "f"(total) : "memory");
    }
    __syncthreads();
    signal_all(pt, CH_NORM_PARTIAL, epoch);
    if (threadIdx.x == 0) {
      norm[pt.world] = 0.f;
      *block_counter = 0u;
    }
  }
}

// ---------------------------------------------------------------- phase 2: AdamW on the shard + all-gather
__global__ void __launch_bounds__(256) dp_adamw_allgather_kernel(PeerTable pt, long long grad_off, long long norm_off,
                                                                 long long param_off, ElemRange owned,
                                                                 long long state_base, float* __restrict__ master,
                                                                 float* __restrict__ m, float* __restrict__ v, float lr,
                                                                 float beta1, float beta2, float eps, float wd, float bc1,
                                                                 float bc2, float max_norm, float* clip_out,
                                                                 float* norm_out, uint32_t epoch,
                                                                 const uint32_t* __restrict__ epoch_dev,
                                                                 const float* __restrict__ hyper, int use_multimem,
                                                                 int* status) {
  if (epoch_dev) epoch = *epoch_dev;
  if (hyper) {  // [0] lr, [1] 1 - beta1^t, [2] 1 - beta2^t of this step, written by the host before the launch
    lr = hyper[0];
    bc1 = hyper[1];
    bc2 = hyper[2];
  }
  const bool ok = cta_wait_all(pt, CH_NORM_PARTIAL, epoch, status);
  if (!ok) return;
  const float* norm = reinterpret_cast<const float*>(pt.bufs[pt.rank] + norm_off);
  float tot = 0.f;
  for (int p = 0; p < pt.world; ++p) tot += *reinterpret_cast<const volatile float*>(&norm[p]);
  const float gnorm = sqrtf(tot);
  const float coef = max_norm > 0.f ? fminf(1.f, max_norm / (gnorm + 1e-6f)) : 1.f;
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    if (clip_out) *clip_out = coef;
    if (norm_out) *norm_out = gnorm;
  }
  const float* grad = reinterpret_cast<const float*>(pt.bufs[pt.rank] + grad_off);
  const long long b8 = owned.begin >> 3, e8 = owned.end >> 3;
  for (long long i = b8 + (long long)blockIdx.x * blockDim.x + threadIdx.x; i < e8; i += (long long)gridDim.x * blockDim.x) {
    float p8[8];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const long long e = i * 8 + h * 4, s = e - state_base;
      float4 g = *reinterpret_cast<const float4*>(grad + e);
      float4 pm = *reinterpret_cast<float4*>(master + s), mm = *reinterpret_cast<float4*>(m + s),
             vv = *reinterpret_cast<float4*>(v + s);
      float gg[4] = {g.x * coef, g.y * coef, g.z * coef, g.w * coef};
      float pp[4] = {pm.x, pm.y, pm.z, pm.w}, m4[4] = {mm.x, mm.y, mm.z, mm.w}, v4[4] = {vv.x, vv.y, vv.z, vv.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        m4[j] = beta1 * m4[j] + (1.f - beta1) * gg[j];
        v4[j] = beta2 * v4[j] + (1.f - beta2) * gg[j] * gg[j];
        pp[j] = pp[j] * (1.f - lr * wd) - lr * (m4[j] / bc1) / (sqrtf(v4[j] / bc2) + eps);
        p8[h * 4 + j] = pp[j];
      }
      *reinterpret_cast<float4*>(master + s) = make_float4(pp[0], pp[1], pp[2], pp[3]);
      *reinterpret_cast<float4*>(m + s) = make_float4(m4[0], m4[1], m4[2], m4[3]);
      *reinterpret_cast<float4*>(v + s) = make_float4(v4[0], v4[1], v4[2], v4[3]);
    }
    uint4 out;
    out.x = pack_bf16x2(p8[0], p8[1]);
    out.y = pack_bf16x2(p8[2], p8[3]);
    out.z = pack_bf16x2(p8[4], p8[5]);
    out.w = pack_bf16x2(p8[6], p8[7]);
    if (use_multimem) {
      multimem_st_16B(reinterpret_cast<uint8_t*>(pt.multicast + param_off) + i * 16, out);
    } else {
      for (int p = 0; p < pt.world; ++p) {
        const int peer = (pt.rank + p) % pt.world;
        *reinterpret_cast<uint4*>(reinterpret_cast<uint8_t*>(pt.bufs[peer] + param_off) + i * 16) = out;
      }
    }
  }
}

__global__ void __launch_bounds__(256) dp_broadcast_ranges_kernel(PeerTable pt, long long param_off, RangeList ranges,
                                                                  int use_multimem) {
  const uint8_t* local = reinterpret_cast<const uint8_t*>(pt.bufs[pt.rank] + param_off);
  for (int r = 0; r < ranges.count; ++r) {
    const long long b8 = ranges.r[r].begin >> 3, e8 = ranges.r[r].end >> 3;
    for (long long i = b8 + (long long)blockIdx.x * blockDim.x + threadIdx.x; i < e8;
         i += (long long)gridDim.x * blockDim.x) {
      const uint4 val = *reinterpret_cast<const uint4*>(local + i * 16);
      if (use_multimem) {
        multimem_st_16B(reinterpret_cast<uint8_t*>(pt.multicast + param_off) + i * 16, val);
      } else {
        for (int p = 1; p < pt.world; ++p) {
          const int peer = (pt.rank + p) % pt.world;
          *reinterpret_cast<uint4*>(reinterpret_cast<uint8_t*>(pt.bufs[peer] + param_off) + i * 16) = val;
        }
      }
    }
  }
}

__global__ void __launch_bounds__(32) comm_barrier_kernel(PeerTable pt, int channel, uint32_t epoch,
                                                          const uint32_t* __restrict__ epoch_dev, int* status) {
  if (epoch_dev) epoch = *epoch_dev;
  signal_all(pt, channel, epoch);
  (void)cta_wait_all(pt, channel, epoch, status);
}

__global__ void __launch_bounds__(32) comm_wait_only_kernel(PeerTable pt, int channel, uint32_t epoch,
                                                            unsigned long long limit_ns, int* status) {
  (void)cta_wait_all(pt, channel, epoch, status, limit_ns);
}

__global__ void __launch_bounds__(256) metric_allreduce_kernel(PeerTable pt, long long metric_off,
                                                               const float* __restrict__ local, float* __restrict__ out,
                                                               int n, int channel, uint32_t epoch,
                                                               const uint32_t* __restrict__ epoch_dev, int* status) {
  if (epoch_dev) epoch = *epoch_dev;  // device-resident epoch: the launch can be replayed from a CUDA graph
  // slot layout in each rank's buffer: [world][n]
  for (int i = threadIdx.x; i < n * pt.world; i += blockDim.x) {
    const int peer = i / n, j = i % n;
    float* dst = reinterpret_cast<float*>(pt.bufs[peer] + metric_off) + (long long)pt.rank * n + j;
    asm volatile("st.relaxed.sys.global.f32 [%0], %1;" ::"l"(dst), "f"(local[j]) : "memory");
  }
  __syncthreads();
  signal_all(pt, channel, epoch);
  if (!cta_wait_all(pt, channel, epoch, status)) return;
  const float* mine = reinterpret_cast<const float*>(pt.bufs[pt.rank] + metric_off);
  for (int j = threadIdx.x; j < n; j += blockDim.x) {
    float s = 0.f;
    for (int p = 0; p < pt.world; ++p) s += *reinterpret_cast<const volatile float*>(&mine[(long long)p * n + j]);
    out[j] = s;
  }
}

void check(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) throw std::runtime_error(std::string(what) + " launch failed: " + cudaGetErrorString(e));
}

int comm_grid() { return 148 * 2; }

}  // namespace

void launch_dp_reduce_scatter(PeerTable pt, long long grad_off, long long norm_off, RangeList ranges, uint32_t epoch,
                              const uint32_t* epoch_dev, bool use_multimem, unsigned int* block_counter, int* status, cudaStream_t s) {
  if (pt.world > COMM_MAX_RANKS) throw std::runtime_error("too many ranks for the signal pad layout");
  dp_reduce_scatter_kernel<<<comm_grid(), 256, 0, s>>>(pt, grad_off, norm_off, ranges, epoch, epoch_dev,
                                                       use_multimem ? 1 : 0, block_counter, status);
  check("dp_reduce_scatter");
}

void launch_dp_adamw_allgather(PeerTable pt, long long grad_off, long long norm_off, long long param_off,
                               ElemRange owned, long long state_base, float* master, float* m, float* v, float lr,
                               float beta1, float beta2, float eps, float wd, float bc1, float bc2, float max_norm,
                               float* clip_out, float* norm_out, uint32_t epoch, const uint32_t* epoch_dev,
                               const float* hyper, bool use_multimem, int* status, cudaStream_t s) {
  dp_adamw_allgather_kernel<<<comm_grid(), 256, 0, s>>>(pt, grad_off, norm_off, param_off, owned, state_base, master, m,
                                                        v, lr, beta1, beta2, eps, wd, bc1, bc2, max_norm, clip_out,
                                                        norm_out, epoch, epoch_dev, hyper, use_multimem ? 1 : 0, status);
  check("dp_adamw_allgather");
}

void launch_dp_broadcast_ranges(PeerTable pt, long long param_off, RangeList ranges, bool use_multimem,
                                cudaStream_t s) {
  if (ranges.count == 0) return;
  dp_broadcast_ranges_kernel<<<comm_grid(), 256, 0, s>>>(pt, param_off, ranges, use_multimem ? 1 : 0);
  check("dp_broadcast_ranges");
}

void launch_comm_barrier(PeerTable pt, int channel, uint32_t epoch, const uint32_t* epoch_dev, int* status,
                         cudaStream_t s) {
  comm_barrier_kernel<<<1, 32, 0, s>>>(pt, channel, epoch, epoch_dev, status);
  check("comm_barrier");
}

void launch_comm_wait_only(PeerTable pt, int channel, uint32_t epoch, unsigned long long limit_ns, int* status,
                           cudaStream_t s) {
  comm_wait_only_kernel<<<1, 32, 0, s>>>(pt, channel, epoch, limit_ns, status);
  check("comm_wait_only");
}

void launch_metric_allreduce(PeerTable pt, long long metric_off, const float* local, float* out, int n, int channel,
                             uint32_t epoch, const uint32_t* epoch_dev, int* status, cudaStream_t s) {
  metric_allreduce_kernel<<<1, 256, 0, s>>>(pt, metric_off, local, out, n, channel, epoch, epoch_dev, status);
  check("metric_allreduce");
}

}  // namespace tb
