// bf16 GEMM on CTA pairs (tcgen05 cta_group::2): C = alpha * A * B^T (+ epilogue), 256-row tiles.
//
// An SM can take 64 bytes per clock from L2. A single CTA computing a 128 x 256 tile needs 48 KB per 64-deep K step
// (768 clocks of loads) for 512 clocks of tensor work, so the one-CTA kernel is bound by its loads at about two
// thirds of the tensor rate; narrower outputs (N = 384) are worse. Pairing two CTAs of a cluster on one 256-row tile
// halves the B traffic of each: every CTA loads its own 128 rows of A and only HALF of the B tile, and the MMA issued
// by the even CTA runs on both tensor cores, each reading both halves of B through the cluster's shared memory.
//
//   NCFG = 256   pair tile 256 x 256; per CTA and K step 16 KB of A + 16 KB of B = 512 clocks of loads for 512 clocks
//                of tensor work; the accumulator (256 TMEM columns) is double-buffered so the epilogue of one tile
//                overlaps the main loop of the next;
//   NCFG = 384   pair tile 256 x 384 as two MMAs per K step (N = 256 and N = 128) that share A; 16 KB + 24 KB of
//                loads for 768 clocks of tensor work; 384 TMEM columns, single-buffered. This is the shape of every
//                product whose output is as wide as the model (d = 384): input gradients and weight gradients.
//
// Roles per CTA: warp 0 TMA producer (both CTAs), warp 1 MMA issuer (even CTA only; the odd CTA's warp 1 only takes
// part in the TMEM allocation), warps 2-9 epilogue (both CTAs, each on its own 128 accumulator rows). Completion of a
// stage's loads from both CTAs is counted on the even CTA's barrier; tcgen05.commit releases a stage, and publishes
// an accumulator, in both CTAs at once. Loads carry no cluster multicast. Every wait is bounded.
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

template <int NCFG>
struct PairCfg {
  static constexpr int A_BYTES = BM * BK * 2;            // this CTA's 128 rows of A
  static constexpr int B_BOXES = NCFG / 128;             // 64-row (or 64-column) boxes in this CTA's half of B
  static constexpr int B_BYTES = B_BOXES * 64 * BK * 2;  // half of the B tile
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGES = (NCFG == 256) ? 6 : 4;
  static constexpr int NACC = (NCFG == 256) ? 2 : 1;  // accumulator buffers in the 512 TMEM columns
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 8 * 4096 + 1024 + 256;
};

__device__ __forceinline__ Tile decode_pair_tile(const KParams& p, int t, int num_mp) {
  Tile tl;
  tl.valid = true;
  const int per_split = num_mp * p.num_n;
  const int split = t / per_split, r = t % per_split;  // grouped-K: `split` is the group
  int m_idx, n_idx;
  raster(r, num_mp, p.num_n, p.group_m, m_idx, n_idx);
  tl.m0 = m_idx * (2 * BM);
  tl.n0 = n_idx;
  tl.g = 0;
  tl.ba = 0;
  tl.bb = 0;
  const int total_iters = (p.K + BK - 1) / BK;
  if (p.mode == GEMM_GROUPED_M) {  // rows grouped by expert, groups padded to whole pairs: B and bias follow the group
    const int g = p.tile_group[2 * m_idx];
    tl.valid = g >= 0;
    tl.g = g < 0 ? 0 : g;
    tl.bb = tl.g;
    tl.k_begin = 0;
    tl.k_iters = total_iters;
  } else if (p.mode == GEMM_GROUPED_K) {
    tl.g = split;
    const int k0 = p.group_offsets[split], k1 = p.group_offsets[split + 1];
    tl.k_begin = k0;
    tl.k_end = k1;
    tl.k_iters = p.k_runs ? run_list_blocks(p.k_runs, k0, k1) : (k1 - k0 + BK - 1) / BK;
  } else if (p.splits > 1) {
    tl.k_begin = split * p.iters_per_split * BK;
    const int left = total_iters - split * p.iters_per_split;
    tl.k_iters = left < p.iters_per_split ? (left < 0 ? 0 : left) : p.iters_per_split;
  } else {
    tl.k_begin = 0;
    tl.k_iters = total_iters;
  }
  return tl;
}

template <int NCFG, bool A_MN, bool B_MN, int EPI>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
    tc_gemm_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                        const __grid_constant__ CUtensorMap tmC, const __grid_constant__ CUtensorMap tmAux,
                        const KParams p, const int num_mp, const int pair_tiles) {
  using Cfg = PairCfg<NCFG>;
  constexpr int STAGES = Cfg::STAGES;
  constexpr int NACC = Cfg::NACC;
  constexpr int NOUT = (EPI == EPI_SWIGLU) ? NCFG / 2 : NCFG;  // output columns per pair tile
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  uint8_t* smem = smem_raw + (((raw + 1023u) & ~1023u) - raw);
  uint8_t* smemA = smem;
  uint8_t* smemB = smem + STAGES * Cfg::A_BYTES;
  uint8_t* smem_epi = smem + STAGES * Cfg::STAGE_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem_epi + 8 * EPI_TILE);
  uint64_t* full = bars;                    // [STAGES] loads of both CTAs -> MMA (used in the even CTA)
  uint64_t* empty = bars + STAGES;          // [STAGES] MMA -> this CTA's producer
  uint64_t* acc_full = bars + 2 * STAGES;   // [2] MMA -> this CTA's epilogue
  uint64_t* acc_empty = acc_full + 2;       // [2] epilogues of both CTAs -> MMA (used in the even CTA)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();  // 0 = even CTA (issues the MMAs), 1 = odd CTA
  const int cluster_id = blockIdx.x >> 1, num_clusters = gridDim.x >> 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&acc_full[a], 1);
      mbar_init(&acc_empty[a], 16);  // eight epilogue warps in each of the two CTAs
    }
    mbar_fence_init();
    prefetch_tmap(&tmA);
    prefetch_tmap(&tmB);
    prefetch_tmap(&tmC);
  }
  if (warp == 1) {
    tmem_alloc_pair(tmem_slot, 512);
    tmem_relinquish_pair();
  }
  tc_fence_before_sync();
  cluster_sync_all();  // both CTAs' barriers are initialised before either signals the other
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer (both CTAs)
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      int issued = 0;
      bool ok = true;
      for (int t = cluster_id; t < pair_tiles && ok; t += num_clusters) {
        const Tile tl = decode_pair_tile(p, t, num_mp);
        if (!tl.valid) continue;
        const int n0 = tl.n0 * NOUT;
        const int m0 = tl.m0 + (int)rank * BM;
        int run = tl.k_begin, run_left = 0, run_pos = 0;  // run-list walk (grouped-K with k_runs)
        for (int it = 0; it < tl.k_iters; ++it) {
          if (!mbar_wait(&empty[stage], phase ^ 1)) {
            report(p, ST_TIMEOUT_EMPTY);
            ok = false;
            break;
          }
          if (rank == 0) mbar_expect_tx(&full[stage], 2 * Cfg::STAGE_BYTES);
          const uint32_t bar = mapa_shared(smem_u32(&full[stage]), 0);
          const int k0 = p.k_runs ? run_list_next(p.k_runs, run, tl.k_end, run_left, run_pos) : tl.k_begin + it * BK;
          uint8_t* a_dst = smemA + stage * Cfg::A_BYTES;
          uint8_t* b_dst = smemB + stage * Cfg::B_BYTES;
          if (A_MN) {
#pragma unroll
            for (int j = 0; j < BM / 64; ++j) tma_load_3d_pair(a_dst + j * (BK * 128), &tmA, bar, m0 + 64 * j, k0, 0);
          } else {
            tma_load_3d_pair(a_dst, &tmA, bar, k0, m0, 0);
          }
#pragma unroll
          for (int j = 0; j < Cfg::B_BOXES; ++j) {
            // this CTA's half of B: boxes 0,1 belong to the N = 256 MMA, box 2 (NCFG = 384) to the N = 128 MMA
            // SwiGLU forward: the even CTA holds the 128 gate rows, the odd CTA the 128 up rows of the same outputs
            const int nb = (EPI == EPI_SWIGLU) ? ((rank == 0 ? n0 : p.n_split + n0) + 64 * j)
                           : ((j < 2) ? (n0 + 128 * (int)rank + 64 * j) : (n0 + 256 + 64 * (int)rank));
            if (B_MN)
              tma_load_3d_pair(b_dst + j * (BK * 128), &tmB, bar, nb, k0, tl.bb);
            else
              tma_load_3d_pair(b_dst + j * (64 * 128), &tmB, bar, k0, nb, tl.bb);
          }
          ++issued;
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
      if (!ok && rank == 0) {
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
    // ------------------------------------------------------------ MMA issuer (even CTA only)
    if (lane == 0 && rank == 0) {
      constexpr uint32_t idesc_main = make_idesc(2 * BM, 256, 1, 1, A_MN ? 1 : 0, B_MN ? 1 : 0);
      constexpr uint32_t idesc_tail = make_idesc(2 * BM, 128, 1, 1, A_MN ? 1 : 0, B_MN ? 1 : 0);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int t = cluster_id; t < pair_tiles && ok; t += num_clusters) {
        const Tile tl = decode_pair_tile(p, t, num_mp);
        if (!tl.valid) continue;
        if (!mbar_wait(&acc_empty[acc], acc_phase ^ 1)) {
          report(p, ST_TIMEOUT_TMEM);
          break;
        }
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * 256;
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
            umma_bf16_pair(d_tmem, adesc, bdesc, idesc_main, (it > 0 || k > 0) ? 1u : 0u);
            if (NCFG == 384) {
              const uint32_t b2 = b_addr + 2 * (64 * 128);  // third box: this CTA's 64 of the last 128 columns
              const uint64_t bdesc2 = B_MN ? make_smem_desc(b2 + k * 2048, BK * 128, 1024)
                                           : make_smem_desc(b2 + k * 32, 16, 1024);
              umma_bf16_pair(d_tmem + 256, adesc, bdesc2, idesc_tail, (it > 0 || k > 0) ? 1u : 0u);
            }
          }
          umma_commit_pair(&empty[stage], 3);  // frees the stage in both CTAs
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (!ok) break;
        if (tl.k_iters > 0) {
          umma_commit_pair(&acc_full[acc], 3);
        } else {  // empty reduction: both epilogues substitute zeros
          mbar_arrive(&acc_full[acc]);
          mbar_arrive_cluster(mapa_shared(smem_u32(&acc_full[acc]), 1));
        }
        if (++acc == NACC) {
          acc = 0;
          acc_phase ^= 1;
        }
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (warps 2..9, both CTAs)
    const int lane_base = (warp & 3) * 32;
    const int col_half = (warp - 2) >> 2;
    uint8_t* my_stage = smem_epi + (warp - 2) * EPI_TILE;
    int acc = 0;
    uint32_t acc_phase = 0, buf = 0;
    for (int t = cluster_id; t < pair_tiles; t += num_clusters) {
      const Tile tl = decode_pair_tile(p, t, num_mp);
      if (!tl.valid) continue;
      bool ok = mbar_wait(&acc_full[acc], acc_phase);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) {
        if (lane == 0) report(p, ST_TIMEOUT_TMEM);
        break;
      }
      tc_fence_after_sync();
      run_epilogue<EPI>(p, tl, &tmC, &tmAux, tmem_base + acc * 256, NCFG, tl.n0 * NOUT, tl.m0 + (int)rank * BM,
                        lane_base, col_half, lane, my_stage, buf);
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) {
        if (rank == 0)
          mbar_arrive(&acc_empty[acc]);
        else
          mbar_arrive_cluster(mapa_shared(smem_u32(&acc_empty[acc]), 0));
      }
      if (++acc == NACC) {
        acc = 0;
        acc_phase ^= 1;
      }
    }
    if (lane == 0) tma_store_wait<0>();  // staged tiles must be fully written before the CTA retires
    __syncwarp();
  }

  // Neither CTA may retire, or free the shared TMEM allocation, while the other can still read its shared memory,
  // signal its barriers or read its accumulator rows.
  tc_fence_before_sync();
  cluster_sync_all();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc_pair(tmem_base, 512);
  }
}

template <int NCFG, bool A_MN, bool B_MN, int EPI>
void launch_pair_variant(const CUtensorMap& tmA, const CUtensorMap& tmB, const CUtensorMap& tmC,
                         const CUtensorMap& tmAux, const KParams& kp, int num_mp, int pair_tiles, int clusters,
                         cudaStream_t stream) {
  auto kern = tc_gemm_pair_kernel<NCFG, A_MN, B_MN, EPI>;
  static PerDeviceOnce configured;  // the attribute is per device
  if (configured.first_use()) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, PairCfg<NCFG>::SMEM_BYTES);
    if (e != cudaSuccess)
      throw std::runtime_error(std::string("tc_gemm_pair: cannot set shared memory size: ") + cudaGetErrorString(e));
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * clusters, 1, 1);
  cfg.blockDim = dim3(GEMM_THREADS, 1, 1);
  cfg.dynamicSmemBytes = PairCfg<NCFG>::SMEM_BYTES;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, kern, tmA, tmB, tmC, tmAux, kp, num_mp, pair_tiles);
  if (e != cudaSuccess) throw std::runtime_error(std::string("tc_gemm_pair launch failed: ") + cudaGetErrorString(e));
}

template <int NCFG, bool A_MN, bool B_MN>
void dispatch_pair_epi(int epi, const CUtensorMap& tmA, const CUtensorMap& tmB, const CUtensorMap& tmC,
                       const CUtensorMap& tmAux, const KParams& kp, int num_mp, int pair_tiles, int clusters,
                       cudaStream_t s) {
  if constexpr (NCFG == 256 && !A_MN) {
    if (epi == EPI_DSWIGLU)
      return launch_pair_variant<NCFG, A_MN, B_MN, EPI_DSWIGLU>(tmA, tmB, tmC, tmAux, kp, num_mp, pair_tiles, clusters, s);
    if constexpr (!B_MN) {
      if (epi == EPI_SWIGLU)
        return launch_pair_variant<NCFG, A_MN, B_MN, EPI_SWIGLU>(tmA, tmB, tmC, tmAux, kp, num_mp, pair_tiles, clusters, s);
    }
  }
  if (epi == EPI_SWIGLU || epi == EPI_DSWIGLU) throw std::runtime_error("tc_gemm_pair: unsupported SwiGLU variant");
  if (epi == EPI_PLAIN_F32)
    launch_pair_variant<NCFG, A_MN, B_MN, EPI_PLAIN_F32>(tmA, tmB, tmC, tmAux, kp, num_mp, pair_tiles, clusters, s);
  else
    launch_pair_variant<NCFG, A_MN, B_MN, EPI_PLAIN>(tmA, tmB, tmC, tmAux, kp, num_mp, pair_tiles, clusters, s);
}

template <int NCFG>
void dispatch_pair_major(bool a_mn, bool b_mn, int epi, const CUtensorMap& tmA, const CUtensorMap& tmB,
                         const CUtensorMap& tmC, const CUtensorMap& tmAux, const KParams& kp, int num_mp,
                         int pair_tiles, int clusters, cudaStream_t s) {
  if (!a_mn && !b_mn) dispatch_pair_epi<NCFG, false, false>(epi, tmA, tmB, tmC, tmAux, kp, num_mp, pair_tiles, clusters, s);
  else if (!a_mn && b_mn) dispatch_pair_epi<NCFG, false, true>(epi, tmA, tmB, tmC, tmAux, kp, num_mp, pair_tiles, clusters, s);
  else if (a_mn && !b_mn) dispatch_pair_epi<NCFG, true, false>(epi, tmA, tmB, tmC, tmAux, kp, num_mp, pair_tiles, clusters, s);
  else dispatch_pair_epi<NCFG, true, true>(epi, tmA, tmB, tmC, tmAux, kp, num_mp, pair_tiles, clusters, s);
}

long long g_pair_launches = 0;

int pair_sm_count() {
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

// Runs the product on CTA pairs when the shape suits them; returns false (nothing launched) otherwise.
bool launch_tc_gemm_pair(const GemmArgs& a, cudaStream_t stream) {
  const bool grouped_k = a.mode == GEMM_GROUPED_K;
  const bool grouped_m = a.mode == GEMM_GROUPED_M;
  const int groups = grouped_k ? (a.batch < 1 ? 1 : a.batch) : 1;
  if (grouped_k) {
    if (a.group_offsets == nullptr || !a.a_mn_major || !a.b_mn_major) return false;
  } else if (grouped_m) {
    if (!(a.flags & GF_PAIRED_GROUPS) || a.tile_group == nullptr || a.strideA != 0 || (a.M % (2 * BM)) != 0) return false;
  } else if (a.mode != GEMM_DENSE || a.batch > 1 || a.strideA != 0 || a.strideB != 0) {
    return false;
  }
  if (a.flags & (GF_GELU | GF_DGELU | GF_ADDAUX)) return false;
  if (a.M < 2 * BM) return false;
  const int num_m_tiles = (a.M + BM - 1) / BM;
  if ((num_m_tiles & 1) && num_m_tiles < 9) return false;  // an odd tile leaves half a pair idle: too costly when few
  const long long k_each = (long long)a.K / groups;       // grouped-K: K is the total over the groups
  static const long long min_k = [] {
    const char* e = std::getenv("TRIUNE_GEMM_PAIR_MIN_K");  // tuning knob: shortest reduction handed to CTA pairs
    return e ? std::atoll(e) : 768ll;
  }();
  const bool swiglu = (a.flags & GF_SWIGLU) != 0, dswiglu = (a.flags & GF_DSWIGLU) != 0;
  int ncfg = 0;
  if (swiglu) {
    // 256 accumulator columns = 128 gate + 128 up columns of 128 outputs
    if (a.N % 128 == 0 && k_each >= min_k && !a.a_mn_major && !a.b_mn_major) ncfg = 256;
  } else if (dswiglu) {
    if (a.N % 256 == 0 && k_each >= min_k && !a.a_mn_major) ncfg = 256;
  } else if (a.N % 384 == 0 && k_each >= (min_k < 1024 ? 1024 : min_k)) ncfg = 384;  // single-buffered: long reductions only
  else if (a.N % 256 == 0 && k_each >= min_k) ncfg = 256;
  if (ncfg == 0) return false;
  const int n_out = swiglu ? ncfg / 2 : ncfg;

  KParams kp;
  kp.M = a.M; kp.N = a.N; kp.K = a.K;
  kp.mode = a.mode; kp.flags = a.flags; kp.batch = groups;
  kp.num_m = (a.M + BM - 1) / BM;
  kp.num_n = a.N / n_out;
  kp.n_split = a.n_split;
  kp.beta = 0.f;
  kp.ldc = a.ldc; kp.strideC = a.strideC;
  kp.a_batched = 0; kp.b_batched = 0;
  kp.alpha = a.alpha;
  kp.C = a.C; kp.bias = a.bias; kp.bias_stride = a.bias_stride;
  kp.aux_in = a.aux_in; kp.aux_out = a.aux_out; kp.row_scale = a.row_scale;
  kp.tile_group = a.tile_group; kp.group_offsets = a.group_offsets; kp.status = a.status;
  kp.k_runs = grouped_k ? a.k_runs : nullptr;
  kp.dbg = nullptr;
  kp.splits = 1;
  kp.iters_per_split = 0;
  const int num_mp = (kp.num_m + 1) / 2;
  kp.group_m = raster_group_m(num_mp, kp.num_n, pair_sm_count() / 2);
  int pair_tiles = num_mp * kp.num_n * groups;
  const int max_clusters = pair_sm_count() / 2;
  // Split-K exactly as in the one-CTA kernel: only into an fp32 accumulator, when the tiles leave most SMs idle.
  if (!grouped_k && !grouped_m && (kp.flags & GF_OUT_F32) && (kp.flags & GF_ACCUMULATE) && a.bias == nullptr && a.row_scale == nullptr) {
    const int total_iters = (a.K + BK - 1) / BK;
    if (pair_tiles * 2 <= max_clusters && total_iters >= 16) {
      int splits = max_clusters / pair_tiles;
      const int max_splits = total_iters / 8;
      if (splits > max_splits) splits = max_splits;
      if (splits > 1) {
        kp.iters_per_split = (total_iters + splits - 1) / splits;
        kp.splits = (total_iters + kp.iters_per_split - 1) / kp.iters_per_split;
        pair_tiles *= kp.splits;
      }
    }
  }
  kp.total_tiles = pair_tiles;

  CUtensorMap tmA, tmB;
  const uint64_t nbB = grouped_m ? (uint64_t)(a.batch < 1 ? 1 : a.batch) : 1;  // grouped-M: one B matrix per group
  const uint64_t sB = (grouped_m ? (uint64_t)a.strideB : (uint64_t)a.ldb) * 2ull;
  if (a.a_mn_major)
    tmA = make_tmap_3d(a.A, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)a.M, (uint64_t)a.K, 1, (uint64_t)a.lda * 2ull,
                       (uint64_t)a.lda * 2ull, 64, BK);
  else
    tmA = make_tmap_3d(a.A, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)a.K, (uint64_t)a.M, 1, (uint64_t)a.lda * 2ull,
                       (uint64_t)a.lda * 2ull, BK, BM);
  if (a.b_mn_major)
    tmB = make_tmap_3d(a.B, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)a.N, (uint64_t)a.K, nbB, (uint64_t)a.ldb * 2ull,
                       sB, 64, BK);
  else
    tmB = make_tmap_3d(a.B, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)a.K, (uint64_t)(swiglu ? 2 * a.N : a.N), nbB,
                       (uint64_t)a.ldb * 2ull, sB, BK, 64);
  const bool c_f32 = (kp.flags & GF_OUT_F32) != 0;
  const int c_elem = c_f32 ? 4 : 2;
  const uint64_t c_bstride = (groups > 1 ? (uint64_t)a.strideC : (uint64_t)a.ldc * (uint64_t)a.M) * c_elem;
  CUtensorMap tmC = make_tmap_3d(a.C, c_f32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, c_elem,
                                 dswiglu ? 2ull * (uint64_t)a.N : (uint64_t)a.N, (uint64_t)a.M, (uint64_t)groups,
                                 (uint64_t)a.ldc * c_elem, c_bstride, c_f32 ? 16 : 32, 32);
  CUtensorMap tmAux = tmC;
  if (swiglu && a.aux_out != nullptr)  // gate | up pre-activations, [M, 2 N] contiguous
    tmAux = make_tmap_3d(a.aux_out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, 2ull * (uint64_t)a.N, (uint64_t)a.M, 1,
                         4ull * (uint64_t)a.N, 4ull * (uint64_t)a.N * (uint64_t)a.M, 32, 32);
  const int clusters = pair_tiles < max_clusters ? pair_tiles : max_clusters;
  const int epi = swiglu ? EPI_SWIGLU : (dswiglu ? EPI_DSWIGLU : (c_f32 ? EPI_PLAIN_F32 : EPI_PLAIN));
  if (ncfg == 256)
    dispatch_pair_major<256>(a.a_mn_major, a.b_mn_major, epi, tmA, tmB, tmC, tmAux, kp, num_mp, pair_tiles, clusters, stream);
  else
    dispatch_pair_major<384>(a.a_mn_major, a.b_mn_major, epi, tmA, tmB, tmC, tmAux, kp, num_mp, pair_tiles, clusters, stream);
  ++g_pair_launches;
  return true;
}

long long tc_gemm_pair_launch_count() { return g_pair_launches; }

}  // namespace tb
