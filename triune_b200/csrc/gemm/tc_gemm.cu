// bf16 GEMM on the 5th-generation tensor cores: C = alpha * A * B^T (+ epilogue).
//
// One persistent CTA per SM, 320 threads, three roles:
//   warp 0    TMA producer: cp.async.bulk.tensor tiles of A (128 x 64) and B (BN x 64) into a ring of
//             128B-swizzled shared-memory stages, completion signalled on mbarriers;
//   warp 1    MMA issuer: one thread issues tcgen05.mma (M=128, N=BN, K=16) reading the stages through
//             shared-memory descriptors and accumulating into TMEM; tcgen05.commit releases a stage
//             back to the producer and, after the last K step, publishes the accumulator;
//   warps 2-9 epilogue: tcgen05.ld the fp32 accumulator (lane == output row), apply the epilogue in packed
//             f32x2 arithmetic (bias, GELU plus its derivative, multiply by saved rows, row scale), stage the
//             converted rows in shared memory and hand them to TMA (store or reduce-add).
// The accumulator is double-buffered in TMEM (2 x BN columns) so the epilogue of tile i overlaps the
// main loop of tile i+1. No cluster multicast is used; every CTA loads its own tiles.
//
// Replaces the reference's library GEMM call sites (torch.matmul / bmm / addmm in
// triune/model/attention.py:537-572, triune/model/moe.py:385-437, triune/kernels/fast_muon.py:15-161).
#include "tc_gemm.cuh"

#include <cuda.h>

#include <cstdlib>
#include <stdexcept>
#include <string>

#include "../common/per_device.h"
#include "../common/ptx.cuh"
#include "../common/tma_desc.h"
#include "tc_gemm_impl.cuh"

namespace tb {

namespace {

template <int BN, bool A_MN, bool B_MN, int EPI>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
    tc_gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                   const __grid_constant__ CUtensorMap tmC, const __grid_constant__ CUtensorMap tmAux, const KParams p) {
  using Cfg = GemmCfg<BN>;
  constexpr int STAGES = Cfg::STAGES;
  constexpr int NOUT = (EPI == EPI_SWIGLU) ? BN / 2 : BN;  // output columns per tile (SwiGLU: gate | up side by side)
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  uint8_t* smem = smem_raw + (((raw + 1023u) & ~1023u) - raw);
  uint8_t* smemA = smem;
  uint8_t* smemB = smem + STAGES * Cfg::A_BYTES;
  uint8_t* smem_epi = smem + STAGES * Cfg::STAGE_BYTES;  // 8 warps x 1 staging tile
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem_epi + 8 * EPI_TILE);
  uint64_t* full = bars;                    // [STAGES] TMA -> MMA
  uint64_t* empty = bars + STAGES;          // [STAGES] MMA -> TMA
  uint64_t* acc_full = bars + 2 * STAGES;   // [2] MMA -> epilogue
  uint64_t* acc_empty = acc_full + 2;       // [2] epilogue -> MMA
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
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
    tmem_alloc(tmem_slot, Cfg::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  const long long t_begin = (p.dbg != nullptr && threadIdx.x == 128) ? clock64() : 0;
  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      int issued = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < p.total_tiles && ok; t += gridDim.x) {
        Tile tl = decode_tile(p, t);
        if (!tl.valid) continue;
        const int n0 = tl.n0 * NOUT;
        int run = tl.k_begin, run_left = 0, run_pos = 0;  // run-list walk (grouped-K with k_runs)
        for (int it = 0; it < tl.k_iters; ++it) {
          if (!mbar_wait(&empty[stage], phase ^ 1)) {
            report(p, ST_TIMEOUT_EMPTY);
            ok = false;
            break;
          }
          mbar_expect_tx(&full[stage], Cfg::STAGE_BYTES);
          const int k0 = p.k_runs ? run_list_next(p.k_runs, run, tl.k_end, run_left, run_pos) : tl.k_begin + it * BK;
          uint8_t* a_dst = smemA + stage * Cfg::A_BYTES;
          uint8_t* b_dst = smemB + stage * Cfg::B_BYTES;
          if (A_MN) {
#pragma unroll
            for (int j = 0; j < BM / 64; ++j)
              tma_load_3d(a_dst + j * (BK * 128), &tmA, &full[stage], tl.m0 + 64 * j, k0, tl.ba);
          } else {
            tma_load_3d(a_dst, &tmA, &full[stage], k0, tl.m0, tl.ba);
          }
          if constexpr (EPI == EPI_SWIGLU) {
            // gate rows [n0, n0 + BN/2) and up rows [n_split + n0, ...) of the fused weight, side by side in the tile
            tma_load_3d(b_dst, &tmB, &full[stage], k0, n0, tl.bb);
            tma_load_3d(b_dst + (BN / 2) * 128, &tmB, &full[stage], k0, p.n_split + n0, tl.bb);
          } else if (B_MN) {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j)
              tma_load_3d(b_dst + j * (BK * 128), &tmB, &full[stage], n0 + 64 * j, k0, tl.bb);
          } else {
            tma_load_3d(b_dst, &tmB, &full[stage], k0, n0, tl.bb);
          }
          ++issued;
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
      if (!ok) {
        // Give loads that are still in flight a bounded chance to land before the CTA retires.
        int pending = issued < STAGES ? issued : STAGES;
        int s = stage;
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
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc(BM, BN, 1, 1, A_MN ? 1 : 0, B_MN ? 1 : 0);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < p.total_tiles && ok; t += gridDim.x) {
        Tile tl = decode_tile(p, t);
        if (!tl.valid) continue;
        if (!mbar_wait(&acc_empty[acc], acc_phase ^ 1)) {
          report(p, ST_TIMEOUT_TMEM);
          break;
        }
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int it = 0; it < tl.k_iters; ++it) {
          if (!mbar_wait(&full[stage], phase)) {
            report(p, ST_TIMEOUT_FULL);
            ok = false;
            break;
          }
          tc_fence_after_sync();
          const uint32_t a_addr = smem_u32(smemA + stage * Cfg::A_BYTES);
          const uint32_t b_addr = smem_u32(smemB + stage * Cfg::B_BYTES);
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            const uint64_t adesc = A_MN ? make_smem_desc(a_addr + k * 2048, BK * 128, 1024)
                                        : make_smem_desc(a_addr + k * 32, 16, 1024);
            const uint64_t bdesc = B_MN ? make_smem_desc(b_addr + k * 2048, BK * 128, 1024)
                                        : make_smem_desc(b_addr + k * 32, 16, 1024);
            umma_bf16(d_tmem, adesc, bdesc, idesc, (it > 0 || k > 0) ? 1u : 0u);
          }
          umma_commit(&empty[stage]);
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (!ok) break;
        if (tl.k_iters > 0)
          umma_commit(&acc_full[acc]);
        else
          mbar_arrive(&acc_full[acc]);  // empty reduction: the epilogue substitutes zeros
        if (++acc == 2) {
          acc = 0;
          acc_phase ^= 1;
        }
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (warps 2..9)
    // Short reductions (K = 384) make the epilogue the longer phase of a tile; eight warps halve it, which is worth
    // more than a deeper load ring.
    const int lane_base = (warp & 3) * 32;
    const int col_half = (warp - 2) >> 2;
    uint8_t* my_stage = smem_epi + (warp - 2) * EPI_TILE;  // one staging tile per warp (a second one costs a load stage and measured slower)
    int acc = 0;
    uint32_t acc_phase = 0, buf = 0;
    for (int t = blockIdx.x; t < p.total_tiles; t += gridDim.x) {
      Tile tl = decode_tile(p, t);
      if (!tl.valid) continue;
      const bool timed = p.dbg != nullptr && lane == 0 && warp == 2;
      const long long tw0 = timed ? clock64() : 0;
      bool ok = mbar_wait(&acc_full[acc], acc_phase);
      ok = __all_sync(0xffffffffu, ok);
      if (timed) {
        atomicAdd(reinterpret_cast<unsigned long long*>(p.dbg + 5), (unsigned long long)(clock64() - tw0));  // wait for MMA
        atomicAdd(reinterpret_cast<unsigned long long*>(p.dbg + 6), 1ull);                                    // tiles
      }
      if (!ok) {
        if (lane == 0) report(p, ST_TIMEOUT_TMEM);
        break;
      }
      tc_fence_after_sync();
      run_epilogue<EPI>(p, tl, &tmC, &tmAux, tmem_base + acc * BN, BN, tl.n0 * NOUT, tl.m0, lane_base, col_half, lane,
                        my_stage, buf);
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[acc]);
      if (++acc == 2) {
        acc = 0;
        acc_phase ^= 1;
      }
    }
    const long long t_drain = (p.dbg != nullptr && threadIdx.x == 128) ? clock64() : 0;
    if (lane == 0) tma_store_wait<0>();  // staged tiles must be fully written before the CTA retires
    __syncwarp();
    if (p.dbg != nullptr && threadIdx.x == 128) {
      const long long now = clock64();
      atomicAdd(reinterpret_cast<unsigned long long*>(p.dbg + 8), (unsigned long long)(now - t_begin));  // role lifetime
      atomicAdd(reinterpret_cast<unsigned long long*>(p.dbg + 9), (unsigned long long)(now - t_drain));  // final drain
      atomicAdd(reinterpret_cast<unsigned long long*>(p.dbg + 10), 1ull);
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
  }
}

template <int BN, bool A_MN, bool B_MN, int EPI>
void launch_variant(const CUtensorMap& tmA, const CUtensorMap& tmB, const CUtensorMap& tmC, const CUtensorMap& tmAux,
                    const KParams& kp, int grid, cudaStream_t stream) {
  auto kern = tc_gemm_kernel<BN, A_MN, B_MN, EPI>;
  static PerDeviceOnce configured;  // the attribute is per device
  if (configured.first_use()) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, GemmCfg<BN>::SMEM_BYTES);
    if (e != cudaSuccess) throw std::runtime_error(std::string("tc_gemm: cannot set shared memory size: ") + cudaGetErrorString(e));
  }
  kern<<<grid, GEMM_THREADS, GemmCfg<BN>::SMEM_BYTES, stream>>>(tmA, tmB, tmC, tmAux, kp);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) throw std::runtime_error(std::string("tc_gemm launch failed: ") + cudaGetErrorString(e));
}

template <int BN, bool A_MN, bool B_MN>
void dispatch_epi(int epi, const CUtensorMap& tmA, const CUtensorMap& tmB, const CUtensorMap& tmC,
                  const CUtensorMap& tmAux, const KParams& kp, int grid, cudaStream_t s) {
  if (epi == EPI_PLAIN) return launch_variant<BN, A_MN, B_MN, EPI_PLAIN>(tmA, tmB, tmC, tmAux, kp, grid, s);
  if (epi == EPI_PLAIN_F32) return launch_variant<BN, A_MN, B_MN, EPI_PLAIN_F32>(tmA, tmB, tmC, tmAux, kp, grid, s);
  if constexpr (!A_MN) {  // the activation epilogues follow row-major activations
    if (epi == EPI_GELU) return launch_variant<BN, A_MN, B_MN, EPI_GELU>(tmA, tmB, tmC, tmAux, kp, grid, s);
    if (epi == EPI_MULAUX) return launch_variant<BN, A_MN, B_MN, EPI_MULAUX>(tmA, tmB, tmC, tmAux, kp, grid, s);
    if (epi == EPI_DSWIGLU) return launch_variant<BN, A_MN, B_MN, EPI_DSWIGLU>(tmA, tmB, tmC, tmAux, kp, grid, s);
    if (epi == EPI_ADDAUX) return launch_variant<BN, A_MN, B_MN, EPI_ADDAUX>(tmA, tmB, tmC, tmAux, kp, grid, s);
    if constexpr (!B_MN) {
      if (epi == EPI_SWIGLU) return launch_variant<BN, A_MN, B_MN, EPI_SWIGLU>(tmA, tmB, tmC, tmAux, kp, grid, s);
    }
  }
  throw std::runtime_error("tc_gemm: activation epilogues need a K-major A operand");
}

template <int BN>
void dispatch_major(bool a_mn, bool b_mn, int epi, const CUtensorMap& tmA, const CUtensorMap& tmB, const CUtensorMap& tmC,
                    const CUtensorMap& tmAux, const KParams& kp, int grid, cudaStream_t s) {
  if (!a_mn && !b_mn) dispatch_epi<BN, false, false>(epi, tmA, tmB, tmC, tmAux, kp, grid, s);
  else if (!a_mn && b_mn) dispatch_epi<BN, false, true>(epi, tmA, tmB, tmC, tmAux, kp, grid, s);
  else if (a_mn && !b_mn) dispatch_epi<BN, true, false>(epi, tmA, tmB, tmC, tmAux, kp, grid, s);
  else dispatch_epi<BN, true, true>(epi, tmA, tmB, tmC, tmAux, kp, grid, s);
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

}  // namespace

static long long* g_gemm_dbg = nullptr;
void tc_gemm_set_debug_buffer(long long* p) { g_gemm_dbg = p; }

void launch_tc_gemm(const GemmArgs& a, cudaStream_t stream) {
  if (a.M <= 0 || a.N <= 0) return;
  if (a.N % 8 != 0) throw std::runtime_error("tc_gemm: N must be a multiple of 8");
  if (a.ldc % 8 != 0) throw std::runtime_error("tc_gemm: ldc must be a multiple of 8");
  if (a.lda % 8 != 0 || a.ldb % 8 != 0) throw std::runtime_error("tc_gemm: lda/ldb must be multiples of 8");
  if (a.mode != GEMM_GROUPED_K && a.K <= 0) throw std::runtime_error("tc_gemm: K must be positive");
  if (a.mode == GEMM_GROUPED_M && a.tile_group == nullptr) throw std::runtime_error("tc_gemm: tile_group missing");
  if ((a.flags & GF_OUT_F32) && (a.flags & (GF_GELU | GF_DGELU)))
    throw std::runtime_error("tc_gemm: activation epilogues write bf16 outputs");
  if ((a.flags & (GF_GELU | GF_DGELU)) && a.row_scale != nullptr)
    throw std::runtime_error("tc_gemm: activation epilogues take no row scale");
  if ((a.flags & GF_GELU) && (a.flags & GF_DGELU)) throw std::runtime_error("tc_gemm: one activation epilogue at a time");
  if ((a.flags & GF_DGELU) && a.aux_in == nullptr) throw std::runtime_error("tc_gemm: multiplier rows missing");
  if ((reinterpret_cast<uintptr_t>(a.C) & 15) != 0) throw std::runtime_error("tc_gemm: C must be 16-byte aligned");
  if (a.mode == GEMM_GROUPED_K && (a.group_offsets == nullptr || !a.a_mn_major || !a.b_mn_major))
    throw std::runtime_error("tc_gemm: grouped-K needs group_offsets and MN-major operands");
  const bool addaux = (a.flags & GF_ADDAUX) != 0;
  if (addaux && (a.aux_in == nullptr || a.a_mn_major || a.bias != nullptr || a.row_scale != nullptr ||
                 (a.flags & (GF_OUT_F32 | GF_ACCUMULATE | GF_GELU | GF_DGELU | GF_SWIGLU | GF_DSWIGLU))))
    throw std::runtime_error("tc_gemm: the add-rows epilogue takes K-major A, bf16 output, rows to add, nothing else");
  const bool swiglu = (a.flags & GF_SWIGLU) != 0, dswiglu = (a.flags & GF_DSWIGLU) != 0;
  if (swiglu || dswiglu) {
    if (a.mode != GEMM_DENSE || a.batch > 1 || a.a_mn_major || (a.flags & (GF_OUT_F32 | GF_ACCUMULATE | GF_GELU | GF_DGELU)) ||
        a.bias != nullptr || a.row_scale != nullptr || (swiglu && dswiglu))
      throw std::runtime_error("tc_gemm: the SwiGLU epilogues take dense K-major activations, bf16 output, no bias");
    if (a.n_split != a.N || a.N % 32 != 0) throw std::runtime_error("tc_gemm: SwiGLU needs N == n_split, a multiple of 32");
    if (swiglu && a.b_mn_major) throw std::runtime_error("tc_gemm: the fused gate/up weight must be K-major");
    if (dswiglu && a.aux_in == nullptr) throw std::runtime_error("tc_gemm: gate/up rows missing");
  }

  {
    static const bool pairs = [] {
      const char* e = std::getenv("TRIUNE_GEMM_PAIR");  // "0" keeps every product on the one-CTA kernel
      return !(e && e[0] == '0');
    }();
    if (pairs && launch_tc_gemm_pair(a, stream)) return;
  }

  // widest tile that divides N: the tensor core is most efficient at N = 256, then 192 (e.g. N = 384), then 128
  int BN = (a.N >= 256 && a.N % 256 == 0) ? 256 : ((a.N >= 192 && a.N % 192 == 0) ? 192 : (a.N > 64 ? 128 : 64));
  {
    static const int forced = [] {
      const char* e = std::getenv("TRIUNE_GEMM_BN");  // experiments only: force the tile width
      return e ? std::atoi(e) : 0;
    }();
    if (forced == 64 || forced == 128 || forced == 192 || forced == 256) BN = forced;
  }
  // SwiGLU forward: a tile of BN accumulator columns yields BN / 2 output columns
  if (swiglu) BN = (a.N % 128 == 0) ? 256 : ((a.N % 64 == 0) ? 128 : 64);
  const int n_out = swiglu ? BN / 2 : BN;
  KParams kp;
  kp.M = a.M; kp.N = a.N; kp.K = a.K;
  kp.mode = a.mode; kp.flags = a.flags; kp.batch = a.batch < 1 ? 1 : a.batch;
  kp.num_m = (a.M + BM - 1) / BM;
  kp.num_n = (a.N + n_out - 1) / n_out;
  kp.n_split = a.n_split;
  kp.beta = a.beta;
  kp.ldc = a.ldc; kp.strideC = a.strideC;
  kp.a_batched = a.strideA != 0; kp.b_batched = a.strideB != 0;
  kp.alpha = a.alpha;
  kp.C = a.C; kp.bias = a.bias; kp.bias_stride = a.bias_stride;
  kp.aux_in = a.aux_in; kp.aux_out = a.aux_out; kp.row_scale = a.row_scale;
  kp.tile_group = a.tile_group; kp.group_offsets = a.group_offsets; kp.status = a.status;
  kp.k_runs = a.mode == GEMM_GROUPED_K ? a.k_runs : nullptr;
  kp.dbg = g_gemm_dbg;
  kp.total_tiles = kp.num_m * kp.num_n * (a.mode == GEMM_GROUPED_M ? 1 : kp.batch);
  kp.splits = 1;
  kp.iters_per_split = 0;
  kp.group_m = raster_group_m(kp.num_m, kp.num_n, sm_count());
  // Split-K: weight gradients reduce over tens of thousands of tokens into a handful of output tiles; spread the
  // reduction over idle SMs. Only when the output is an fp32 accumulator (partials are added with red.add).
  if (a.mode == GEMM_DENSE && (kp.flags & GF_OUT_F32) && (kp.flags & GF_ACCUMULATE) && a.bias == nullptr &&
      a.row_scale == nullptr && !(kp.flags & (GF_GELU | GF_DGELU))) {
    const int total_iters = (a.K + BK - 1) / BK;
    const int sms = sm_count();
    if (kp.total_tiles * 2 <= sms && total_iters >= 16) {
      int splits = sms / kp.total_tiles;
      int max_splits = total_iters / 8;
      static const int split_cap = [] {
        const char* e = std::getenv("TRIUNE_GEMM_MAX_SPLITS");  // tuning knob: upper bound of the split-K factor
        return e ? std::atoi(e) : 0;
      }();
      if (split_cap > 0 && max_splits > split_cap) max_splits = split_cap;
      if (splits > max_splits) splits = max_splits;
      if (splits > 1) {
        kp.iters_per_split = (total_iters + splits - 1) / splits;
        kp.splits = (total_iters + kp.iters_per_split - 1) / kp.iters_per_split;
        kp.total_tiles *= kp.splits;
      }
    }
  }

  // Tensor maps. dims are {contiguous, rows, batch}.
  const uint64_t a_rows_total = (a.mode == GEMM_GROUPED_K) ? (uint64_t)a.K : 0;  // K = total rows for grouped-K
  CUtensorMap tmA, tmB;
  const uint64_t nbA = kp.a_batched ? (uint64_t)kp.batch : 1, nbB = (a.mode == GEMM_GROUPED_M || kp.b_batched) ? (uint64_t)kp.batch : 1;
  const uint64_t sA = (kp.a_batched ? (uint64_t)a.strideA : (uint64_t)a.lda) * 2ull;
  const uint64_t sB = ((a.mode == GEMM_GROUPED_M || kp.b_batched) ? (uint64_t)a.strideB : (uint64_t)a.ldb) * 2ull;
  if (a.a_mn_major) {
    const uint64_t krows = (a.mode == GEMM_GROUPED_K) ? a_rows_total : (uint64_t)a.K;
    tmA = make_tmap_3d(a.A, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)a.M, krows, nbA, (uint64_t)a.lda * 2ull, sA, 64, BK);
  } else {
    tmA = make_tmap_3d(a.A, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)a.K, (uint64_t)a.M, nbA, (uint64_t)a.lda * 2ull, sA, BK, BM);
  }
  if (a.b_mn_major) {
    const uint64_t krows = (a.mode == GEMM_GROUPED_K) ? a_rows_total : (uint64_t)a.K;
    tmB = make_tmap_3d(a.B, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)a.N, krows, nbB, (uint64_t)a.ldb * 2ull, sB, 64, BK);
  } else {
    // SwiGLU forward: B is the fused [2 N, K] weight, fetched as two boxes of BN / 2 rows
    tmB = make_tmap_3d(a.B, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)a.K, (uint64_t)(swiglu ? 2 * a.N : a.N), nbB,
                       (uint64_t)a.ldb * 2ull, sB, BK, (uint32_t)n_out);
  }
  // output maps: rows of 64 bytes (32 bf16 / 16 fp32) x 32 rows, one box per epilogue warp and column chunk
  const bool c_f32 = (kp.flags & GF_OUT_F32) != 0;
  const int c_elem = c_f32 ? 4 : 2;
  const uint64_t c_batches = (a.mode == GEMM_GROUPED_M) ? 1 : (uint64_t)kp.batch;
  const uint64_t c_bstride = (c_batches > 1 ? (uint64_t)a.strideC : (uint64_t)a.ldc * (uint64_t)a.M) * c_elem;
  const uint64_t c_cols = dswiglu ? 2ull * (uint64_t)a.N : (uint64_t)a.N;  // d(gate) | d(up)
  CUtensorMap tmC = make_tmap_3d(a.C, c_f32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, c_elem,
                                 c_cols, (uint64_t)a.M, c_batches, (uint64_t)a.ldc * c_elem, c_bstride,
                                 c_f32 ? 16 : 32, 32);
  CUtensorMap tmAux = tmC;
  if (swiglu && a.aux_out != nullptr)  // gate | up pre-activations, [M, 2 N] contiguous
    tmAux = make_tmap_3d(a.aux_out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, 2ull * (uint64_t)a.N, (uint64_t)a.M, 1,
                         4ull * (uint64_t)a.N, 4ull * (uint64_t)a.N * (uint64_t)a.M, 32, 32);
  else if (a.aux_out != nullptr)
    tmAux = make_tmap_3d(a.aux_out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)a.N, (uint64_t)a.M, c_batches,
                         (uint64_t)a.ldc * 2ull, (c_batches > 1 ? (uint64_t)a.strideC : (uint64_t)a.ldc * (uint64_t)a.M) * 2ull, 32, 32);
  const int grid = kp.total_tiles < sm_count() ? kp.total_tiles : sm_count();
  const int epi = addaux ? EPI_ADDAUX : swiglu ? EPI_SWIGLU
                  : (dswiglu ? EPI_DSWIGLU
                     : ((kp.flags & GF_GELU) ? EPI_GELU : ((kp.flags & GF_DGELU) ? EPI_MULAUX : (c_f32 ? EPI_PLAIN_F32 : EPI_PLAIN))));
  if (BN == 256) dispatch_major<256>(a.a_mn_major, a.b_mn_major, epi, tmA, tmB, tmC, tmAux, kp, grid, stream);
  else if (BN == 192) dispatch_major<192>(a.a_mn_major, a.b_mn_major, epi, tmA, tmB, tmC, tmAux, kp, grid, stream);
  else if (BN == 128) dispatch_major<128>(a.a_mn_major, a.b_mn_major, epi, tmA, tmB, tmC, tmAux, kp, grid, stream);
  else dispatch_major<64>(a.a_mn_major, a.b_mn_major, epi, tmA, tmB, tmC, tmAux, kp, grid, stream);
}

}  // namespace tb
