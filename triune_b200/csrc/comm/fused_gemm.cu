// tcgen05 GEMMs fused with their collective over NVLink peer memory (no NCCL, no cluster multicast).
//
//   FG_REDUCE_SCATTER   row-parallel linear: C_partial = A[M, K/tp] * B^T is never materialised; every 128-row output
//                       tile goes straight from the epilogue to the rank that owns those rows with a TMA reduce-add
//                       into that rank's buffer (tensor maps of all peers' buffers come as a device table). Tiles are
//                       visited starting with the next rank's rows so the NVLink traffic is spread over the whole
//                       main loop.
//   FG_ALL_GATHER       column-parallel linear over sequence-sharded activations: four extra "fetch" warps per CTA
//                       pull the remote row shards of A chunk by chunk (128 rows) over NVLink into the local copy of
//                       the gathered buffer and publish a per-chunk flag; the TMA producer waits (bounded) for the
//                       flag of a chunk before loading tiles of it. Tiles of the local shard come first, so the
//                       tensor cores start at once and every remote byte crosses NVLink exactly once.
//   FG_SCATTER_ROWS     expert-parallel combine: grouped-by-rows expert GEMM whose epilogue adds the expert bias,
//                       applies the routing weight and stores every output row into the token owner's receive
//                       buffer (row_dst table: destination rank and slot), the reverse all-to-all.
//
// Structure as in the plain GEMM: persistent CTAs, warp 0 TMA producer, warp 1 single-thread MMA issuer, warps 2-5
// epilogue, accumulators double-buffered in TMEM. A is K-major; B is K-major (forward) or MN-major (data gradient).
// Every wait is bounded; on expiry the status word is set and the CTA drains and frees its TMEM.
#include <cuda.h>

#include <stdexcept>
#include <string>

#include "../common/per_device.h"
#include "../common/ptx.cuh"
#include "../common/tma_desc.h"
#include "fused_gemm.cuh"

namespace tb {
namespace {

constexpr int BM = 128, BK = 64;
constexpr int EPI_TILE = 32 * 128;
constexpr unsigned long long FLAG_WAIT_NS = 2000000000ull;
constexpr int FETCH_PARTS = 4;  // a 128-row chunk is fetched as four 32-row parts, each with its own flag

template <int BN>
struct Cfg {
  static constexpr int A_BYTES = BM * BK * 2, B_BYTES = BN * BK * 2, STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGES = BN == 256 ? 4 : 6;
  static constexpr int TMEM_COLS = 2 * BN;
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 8 * EPI_TILE + 1024 + 256;
};

struct FParams {
  int M, N, K, mode, out_f32;
  int num_m, num_n, total_tiles, m_rotate;
  // reduce-scatter
  const CUtensorMap* c_maps;
  int rows_per_dest;
  // all-gather
  const uint64_t* peer_bufs;
  long long a_off;  // byte offset of the gathered A buffer inside every rank's symmetric buffer
  int rows_per_src, rank, world;
  uint32_t* chunk_flags;
  uint32_t epoch;
  // scatter rows
  const int* tile_group;
  const int* row_dst;
  int slots_per_rank;
  long long out_off, out_ld;
  const __nv_bfloat16* bias;
  long long bias_stride;
  const float* row_scale;
  int gelu;
  int* status;
};

struct FTile {
  int m_idx, n_idx, g;
  bool valid;
};

__device__ __forceinline__ FTile decode(const FParams& p, int t) {
  FTile tl;
  tl.valid = true;
  tl.g = 0;
  if (p.mode == FG_ALL_GATHER) {  // m-major: all column tiles of one 128-row chunk are adjacent
    tl.m_idx = (t / p.num_n + p.m_rotate) % p.num_m;
    tl.n_idx = t % p.num_n;
  } else if (p.mode == FG_REDUCE_SCATTER) {
    tl.m_idx = (t % p.num_m + p.m_rotate) % p.num_m;
    tl.n_idx = t / p.num_m;
  } else {
    tl.m_idx = t % p.num_m;
    tl.n_idx = t / p.num_m;
    const int g = p.tile_group[tl.m_idx];
    tl.valid = g >= 0;
    tl.g = g < 0 ? 0 : g;
  }
  return tl;
}

__device__ __forceinline__ void report(const FParams& p, int code) {
  if (p.status) atomicCAS(p.status, 0, code);
}
__device__ __forceinline__ uint32_t ld_acquire_gpu(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_gpu(uint32_t* p, uint32_t v) {
  asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint4 ld_peer_16B(const void* p) {
  uint4 v;
  asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}

template <int BN, bool B_MN, int MODE>
__global__ void __launch_bounds__(MODE == FG_ALL_GATHER ? 320 : 192, 1)
    fused_gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                      const __grid_constant__ CUtensorMap tmC, const FParams p) {
  using C = Cfg<BN>;
  constexpr int STAGES = C::STAGES;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  uint8_t* smem = smem_raw + (((raw + 1023u) & ~1023u) - raw);
  uint8_t* smemA = smem;
  uint8_t* smemB = smem + STAGES * C::A_BYTES;
  uint8_t* smem_epi = smem + STAGES * C::STAGE_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem_epi + 8 * EPI_TILE);
  uint64_t* full = bars;
  uint64_t* empty = bars + STAGES;
  uint64_t* acc_full = bars + 2 * STAGES;
  uint64_t* acc_empty = acc_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int k_iters = (p.K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&acc_full[a], 1);
      mbar_init(&acc_empty[a], 4);
    }
    mbar_fence_init();
    prefetch_tmap(&tmA);
    prefetch_tmap(&tmB);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, C::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ---------------------------------------------------------------- TMA producer
    if (lane == 0) {
      int stage = 0, issued = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < p.total_tiles && ok; t += gridDim.x) {
        const FTile tl = decode(p, t);
        if (!tl.valid) continue;
        const int m0 = tl.m_idx * BM, n0 = tl.n_idx * BN;
        if (MODE == FG_ALL_GATHER && (m0 / p.rows_per_src) != p.rank) {
          // rows of a remote shard: wait until the fetch warps of some CTA have landed this chunk locally
          const unsigned long long t0 = globaltimer_ns();
          for (int part = 0; part < FETCH_PARTS && ok; ++part) {
            while ((int)(ld_acquire_gpu(p.chunk_flags + tl.m_idx * FETCH_PARTS + part) - p.epoch) < 0) {
              if (globaltimer_ns() - t0 > FLAG_WAIT_NS) {
                report(p, 5);
                ok = false;
                break;
              }
              __nanosleep(128);
            }
          }
          if (!ok) break;
          asm volatile("fence.proxy.async;" ::: "memory");  // generic-proxy stores of the fetch warps -> TMA reads
        }
        for (int it = 0; it < k_iters; ++it) {
          if (!mbar_wait(&empty[stage], phase ^ 1)) {
            report(p, 1);
            ok = false;
            break;
          }
          mbar_expect_tx(&full[stage], C::STAGE_BYTES);
          const int k0 = it * BK;
          tma_load_3d(smemA + stage * C::A_BYTES, &tmA, &full[stage], k0, m0, 0);
          uint8_t* b_dst = smemB + stage * C::B_BYTES;
          if (B_MN) {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j) tma_load_3d(b_dst + j * (BK * 128), &tmB, &full[stage], n0 + 64 * j, k0, tl.g);
          } else {
            tma_load_3d(b_dst, &tmB, &full[stage], k0, n0, tl.g);
          }
          ++issued;
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
      if (!ok) {
        int pending = issued < STAGES ? issued : STAGES, s = stage;
        uint32_t ph = phase;
        for (int i = 0; i < pending; ++i) {
          if (--s < 0) {
            s = STAGES - 1;
            ph ^= 1;
          }
          (void)mbar_wait(&full[s], ph);
        }
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc(BM, BN, 1, 1, 0, B_MN ? 1 : 0);
      int stage = 0, acc = 0;
      uint32_t phase = 0, acc_phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < p.total_tiles && ok; t += gridDim.x) {
        const FTile tl = decode(p, t);
        if (!tl.valid) continue;
        if (!mbar_wait(&acc_empty[acc], acc_phase ^ 1)) {
          report(p, 2);
          break;
        }
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int it = 0; it < k_iters; ++it) {
          if (!mbar_wait(&full[stage], phase)) {
            report(p, 3);
            ok = false;
            break;
          }
          tc_fence_after_sync();
          const uint32_t a_addr = smem_u32(smemA + stage * C::A_BYTES);
          const uint32_t b_addr = smem_u32(smemB + stage * C::B_BYTES);
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            const uint64_t adesc = make_smem_desc(a_addr + k * 32, 16, 1024);
            const uint64_t bdesc = B_MN ? make_smem_desc(b_addr + k * 2048, BK * 128, 1024) : make_smem_desc(b_addr + k * 32, 16, 1024);
            umma_bf16(d_tmem, adesc, bdesc, idesc, (it > 0 || k > 0) ? 1u : 0u);
          }
          umma_commit(&empty[stage]);
          if (++stage == STAGES) {
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
  } else if (warp < 6) {
    // ---------------------------------------------------------------- epilogue
    const int lane_base = (warp & 3) * 32;
    uint8_t* my_stage = smem_epi + (warp & 3) * (2 * EPI_TILE);
    int buf = 0, acc = 0;
    uint32_t acc_phase = 0;
    const bool out_f32 = p.out_f32 != 0;
    const int CW = (MODE != FG_SCATTER_ROWS && out_f32) ? 32 : 64;
    for (int t = blockIdx.x; t < p.total_tiles; t += gridDim.x) {
      const FTile tl = decode(p, t);
      if (!tl.valid) continue;
      bool ok = mbar_wait(&acc_full[acc], acc_phase);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) {
        if (lane == 0) report(p, 4);
        break;
      }
      tc_fence_after_sync();
      const int m0 = tl.m_idx * BM, n0 = tl.n_idx * BN;
      const int gm = m0 + lane_base + lane;
      // destination of this warp's 32 rows
      const CUtensorMap* tm = &tmC;
      int row_coord = m0 + lane_base;
      if (MODE == FG_REDUCE_SCATTER) {
        tm = p.c_maps + (m0 / p.rows_per_dest);
        row_coord = (m0 % p.rows_per_dest) + lane_base;
      }
      uint8_t* dst_row = nullptr;
      float rs = 1.f;
      if (MODE == FG_SCATTER_ROWS) {
        const int d = gm < p.M ? p.row_dst[gm] : -1;
        if (d >= 0) {
          const int drank = d / p.slots_per_rank, dslot = d % p.slots_per_rank;
          dst_row = reinterpret_cast<uint8_t*>(p.peer_bufs[drank]) + p.out_off + (long long)dslot * p.out_ld * 2;
          if (p.row_scale) rs = p.row_scale[gm];
        }
      }
      const __nv_bfloat16* bias = (MODE == FG_SCATTER_ROWS && p.bias) ? p.bias + (long long)tl.g * p.bias_stride : nullptr;
#pragma unroll 1
      for (int c = 0; c < BN; c += CW) {
        if (n0 + c >= p.N) break;
        float v[64];
        uint32_t r[32];
        tmem_ld_32x32b_x32(tmem_base + ((uint32_t)lane_base << 16) + acc * BN + c, r);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
        if (CW == 64) {
          tmem_ld_32x32b_x32(tmem_base + ((uint32_t)lane_base << 16) + acc * BN + c + 32, r);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) v[32 + i] = __uint_as_float(r[i]);
        }
        if (MODE == FG_SCATTER_ROWS) {
          if (dst_row != nullptr) {
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              const int gn = n0 + c + j * 8;
              if (gn < p.N) {
                float b8[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
                if (bias) {
                  const uint4 bv = *reinterpret_cast<const uint4*>(bias + gn);
                  const __nv_bfloat162* b2 = reinterpret_cast<const __nv_bfloat162*>(&bv);
#pragma unroll
                  for (int i = 0; i < 4; ++i) {
                    const float2 f = __bfloat1622float2(b2[i]);
                    b8[2 * i] = f.x;
                    b8[2 * i + 1] = f.y;
                  }
                }
                uint4 o;
                o.x = pack_bf16x2((v[j * 8 + 0] + b8[0]) * rs, (v[j * 8 + 1] + b8[1]) * rs);
                o.y = pack_bf16x2((v[j * 8 + 2] + b8[2]) * rs, (v[j * 8 + 3] + b8[3]) * rs);
                o.z = pack_bf16x2((v[j * 8 + 4] + b8[4]) * rs, (v[j * 8 + 5] + b8[5]) * rs);
                o.w = pack_bf16x2((v[j * 8 + 6] + b8[6]) * rs, (v[j * 8 + 7] + b8[7]) * rs);
                *reinterpret_cast<uint4*>(dst_row + (long long)gn * 2) = o;  // peer store over NVLink (or local)
              }
            }
          }
          continue;
        }
        if (lane == 0) tma_store_wait_read<1>();
        __syncwarp();
        uint8_t* st = my_stage + buf * EPI_TILE;
        if (out_f32) {
#pragma unroll
          for (int j = 0; j < 8; ++j)
            *reinterpret_cast<float4*>(st + lane * 128 + ((j ^ (lane & 7)) << 4)) =
                make_float4(v[j * 4 + 0], v[j * 4 + 1], v[j * 4 + 2], v[j * 4 + 3]);
        } else {
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            uint4 o;
            o.x = pack_bf16x2(v[j * 8 + 0], v[j * 8 + 1]);
            o.y = pack_bf16x2(v[j * 8 + 2], v[j * 8 + 3]);
            o.z = pack_bf16x2(v[j * 8 + 4], v[j * 8 + 5]);
            o.w = pack_bf16x2(v[j * 8 + 6], v[j * 8 + 7]);
            *reinterpret_cast<uint4*>(st + lane * 128 + ((j ^ (lane & 7)) << 4)) = o;
          }
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
          if (MODE == FG_REDUCE_SCATTER)
            tma_reduce_add_3d(tm, st, n0 + c, row_coord, 0);  // adds into the owner's buffer, local or peer
          else
            tma_store_3d(tm, st, n0 + c, row_coord, 0);
          tma_store_commit();
        }
        buf ^= 1;
      }
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
  } else if (MODE == FG_ALL_GATHER) {
    // ---------------------------------------------------------------- fetch warps (6..9): remote shards -> local buffer
    const int ft = threadIdx.x - 192;                      // 0..127
    const long long row_bytes = (long long)p.K * 2;         // gathered A is [M, K] bf16, dense
    const long long part_bytes = row_bytes * (BM / FETCH_PARTS);
    uint8_t* local = reinterpret_cast<uint8_t*>(p.peer_bufs[p.rank]) + p.a_off;
    // Work item = a quarter of a 128-row chunk (32 rows), visited in the order in which the tiles need the chunks, so
    // one chunk is pulled by four CTAs at once and the first remote chunks land early.
    const int items = p.num_m * FETCH_PARTS;
    for (int i = blockIdx.x; i < items; i += gridDim.x) {
      const int chunk = (i / FETCH_PARTS + p.m_rotate) % p.num_m, part = i % FETCH_PARTS;
      const int src = (chunk * BM) / p.rows_per_src;
      if (src == p.rank) continue;
      const long long off = ((long long)chunk * FETCH_PARTS + part) * part_bytes;
      const uint8_t* remote = reinterpret_cast<const uint8_t*>(p.peer_bufs[src]) + p.a_off + off;
      uint8_t* dst = local + off;
      const long long n16 = part_bytes >> 4;
      long long j = ft;
      for (; j + 7 * 128 < n16; j += 8 * 128) {  // eight 16-byte loads in flight per thread
        uint4 v[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) v[u] = ld_peer_16B(remote + ((j + u * 128) << 4));
#pragma unroll
        for (int u = 0; u < 8; ++u) *reinterpret_cast<uint4*>(dst + ((j + u * 128) << 4)) = v[u];
      }
      for (; j < n16; j += 128) *reinterpret_cast<uint4*>(dst + (j << 4)) = ld_peer_16B(remote + (j << 4));
      __threadfence();
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (ft == 0) st_release_gpu(p.chunk_flags + chunk * FETCH_PARTS + part, p.epoch);
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, C::TMEM_COLS);
  }
}

int sm_count() {
  static int n = 0;
  if (n == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    if (n <= 0) n = 148;
  }
  return n;
}

template <int BN, bool B_MN, int MODE>
void launch(const CUtensorMap& tmA, const CUtensorMap& tmB, const CUtensorMap& tmC, const FParams& p, cudaStream_t s) {
  auto kern = fused_gemm_kernel<BN, B_MN, MODE>;
  static PerDeviceOnce configured;  // the attribute is per device
  if (configured.first_use()) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg<BN>::SMEM_BYTES);
    if (e != cudaSuccess) throw std::runtime_error(std::string("fused_gemm: ") + cudaGetErrorString(e));
  }
  const int grid = p.total_tiles < sm_count() ? p.total_tiles : sm_count();
  kern<<<grid, MODE == FG_ALL_GATHER ? 320 : 192, Cfg<BN>::SMEM_BYTES, s>>>(tmA, tmB, tmC, p);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) throw std::runtime_error(std::string("fused_gemm launch failed: ") + cudaGetErrorString(e));
}

template <int MODE>
void dispatch(int BN, bool b_mn, const CUtensorMap& tmA, const CUtensorMap& tmB, const CUtensorMap& tmC, const FParams& p,
              cudaStream_t s) {
  if (BN == 256) {
    if (b_mn) launch<256, true, MODE>(tmA, tmB, tmC, p, s);
    else launch<256, false, MODE>(tmA, tmB, tmC, p, s);
  } else {
    if (b_mn) launch<128, true, MODE>(tmA, tmB, tmC, p, s);
    else launch<128, false, MODE>(tmA, tmB, tmC, p, s);
  }
}

}  // namespace

void build_peer_c_maps(const uint64_t* peer_base_ptrs, int world, long long byte_offset, int rows, int N, long long ldc,
                       bool f32, void* host_out /* world * sizeof(CUtensorMap) */) {
  CUtensorMap* out = reinterpret_cast<CUtensorMap*>(host_out);
  const int es = f32 ? 4 : 2;
  for (int r = 0; r < world; ++r)
    out[r] = make_tmap_3d(reinterpret_cast<const void*>(peer_base_ptrs[r] + byte_offset),
                          f32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, es, (uint64_t)N, (uint64_t)rows, 1,
                          (uint64_t)ldc * es, (uint64_t)ldc * es * (uint64_t)rows, f32 ? 32 : 64, 32);
}

void launch_fused_gemm(const FusedGemmArgs& a, cudaStream_t stream) {
  if (a.M <= 0 || a.N <= 0 || a.K <= 0) return;
  if (a.N % 8 || a.K % 8 || a.lda % 8 || a.ldb % 8) throw std::runtime_error("fused_gemm: N, K, lda, ldb must be multiples of 8");
  FParams p{};
  p.M = a.M; p.N = a.N; p.K = a.K; p.mode = a.mode; p.out_f32 = a.out_f32 ? 1 : 0;
  const int BN = (a.N % 256 == 0) ? 256 : 128;
  p.num_m = (a.M + BM - 1) / BM;
  p.num_n = (a.N + BN - 1) / BN;
  p.total_tiles = p.num_m * p.num_n;
  p.status = a.status;
  p.peer_bufs = a.peer_bufs; p.rank = a.rank; p.world = a.world;
  CUtensorMap tmC{};
  int groups = 1;
  if (a.mode == FG_REDUCE_SCATTER) {
    if (a.c_maps == nullptr || a.rows_per_dest <= 0 || a.rows_per_dest % BM || a.M != a.rows_per_dest * a.world)
      throw std::runtime_error("fused_gemm reduce-scatter: M must be world * rows_per_dest with rows_per_dest a multiple of 128");
    p.c_maps = reinterpret_cast<const CUtensorMap*>(a.c_maps);
    p.rows_per_dest = a.rows_per_dest;
    p.m_rotate = ((a.rank + 1) % a.world) * (a.rows_per_dest / BM);
  } else if (a.mode == FG_ALL_GATHER) {
    if (a.rows_per_src <= 0 || a.rows_per_src % BM || a.M != a.rows_per_src * a.world || a.lda != a.K || a.chunk_flags == nullptr)
      throw std::runtime_error("fused_gemm all-gather: M = world * rows_per_src (multiple of 128), dense A, chunk flags required");
    p.rows_per_src = a.rows_per_src; p.a_off = a.a_off; p.chunk_flags = a.chunk_flags; p.epoch = a.epoch;
    p.m_rotate = a.rank * (a.rows_per_src / BM);
    if ((reinterpret_cast<uintptr_t>(a.C) & 15) || a.ldc % 8) throw std::runtime_error("fused_gemm: C alignment");
    tmC = make_tmap_3d(a.C, a.out_f32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, a.out_f32 ? 4 : 2,
                       (uint64_t)a.N, (uint64_t)a.M, 1, (uint64_t)a.ldc * (a.out_f32 ? 4 : 2),
                       (uint64_t)a.ldc * (a.out_f32 ? 4 : 2) * (uint64_t)a.M, a.out_f32 ? 32 : 64, 32);
  } else if (a.mode == FG_SCATTER_ROWS) {
    if (a.tile_group == nullptr || a.row_dst == nullptr || a.slots_per_rank <= 0 || a.out_ld % 8)
      throw std::runtime_error("fused_gemm scatter: tile_group, row_dst, slots_per_rank and an 8-aligned out_ld are required");
    p.tile_group = a.tile_group; p.row_dst = a.row_dst; p.slots_per_rank = a.slots_per_rank;
    p.out_off = a.out_off; p.out_ld = a.out_ld; p.bias = a.bias; p.bias_stride = a.bias_stride; p.row_scale = a.row_scale;
    groups = a.groups < 1 ? 1 : a.groups;
  } else {
    throw std::runtime_error("fused_gemm: unknown mode");
  }
  CUtensorMap tmA = make_tmap_3d(a.A, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)a.K, (uint64_t)a.M, 1, (uint64_t)a.lda * 2ull,
                                 (uint64_t)a.lda * 2ull * (uint64_t)a.M, BK, BM);
  CUtensorMap tmB;
  if (a.b_mn_major)
    tmB = make_tmap_3d(a.B, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)a.N, (uint64_t)a.K, (uint64_t)groups, (uint64_t)a.ldb * 2ull,
                       (uint64_t)a.strideB * 2ull, 64, BK);
  else
    tmB = make_tmap_3d(a.B, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)a.K, (uint64_t)a.N, (uint64_t)groups, (uint64_t)a.ldb * 2ull,
                       (uint64_t)a.strideB * 2ull, BK, (uint32_t)BN);
  if (a.mode == FG_REDUCE_SCATTER) dispatch<FG_REDUCE_SCATTER>(BN, a.b_mn_major, tmA, tmB, tmC, p, stream);
  else if (a.mode == FG_ALL_GATHER) dispatch<FG_ALL_GATHER>(BN, a.b_mn_major, tmA, tmB, tmC, p, stream);
  else dispatch<FG_SCATTER_ROWS>(BN, a.b_mn_major, tmA, tmB, tmC, p, stream);
}

}  // namespace tb
