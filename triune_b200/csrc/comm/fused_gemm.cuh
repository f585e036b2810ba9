// GEMMs fused with a collective over NVLink peer memory, and the expert-parallel dispatch kernels around them.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace tb {

enum FusedGemmMode : int {
  FG_REDUCE_SCATTER = 0,  // C rows are owned by ranks; partial tiles are TMA reduce-added into the owner's buffer
  FG_ALL_GATHER = 1,      // A rows are sharded over ranks; remote shards are fetched chunk by chunk while the GEMM runs
  FG_SCATTER_ROWS = 2,    // grouped-by-rows GEMM whose output rows are stored into per-row destinations on peers
};

struct FusedGemmArgs {
  int mode;
  const __nv_bfloat16* A;  // [M, K] K-major (all-gather: the LOCAL copy of the gathered buffer)
  const __nv_bfloat16* B;  // [N, K] K-major, or [K, N] when b_mn_major; scatter mode: [groups][...]
  int M, N, K;
  long long lda, ldb, strideB;
  bool b_mn_major, out_f32;
  int groups;
  int rank, world;
  const uint64_t* peer_bufs;  // device array [world] of the peers' symmetric buffer base addresses
  // reduce-scatter
  const void* c_maps;  // device array [world] of tensor maps over the owners' output buffers (build_peer_c_maps)
  int rows_per_dest;
  // all-gather
  void* C;
  long long ldc;
  long long a_off;
  int rows_per_src;
  uint32_t* chunk_flags;  // [4 * M / 128] local flags (one per 32-row part), monotonically increasing epochs
  uint32_t epoch;
  // scatter rows
  const int* tile_group;  // [ceil(M/128)] expert of each row tile, -1 = skip
  const int* row_dst;     // [M] destination rank * slots_per_rank + slot, -1 = drop the row
  int slots_per_rank;
  long long out_off, out_ld;  // byte offset of the receive buffer in the symmetric buffer; its row pitch in elements
  const __nv_bfloat16* bias;
  long long bias_stride;
  const float* row_scale;
  int* status;
};

void launch_fused_gemm(const FusedGemmArgs& a, cudaStream_t stream);

// Fills `host_out` (world * 128 bytes) with tensor maps over rows x N output buffers that live at `byte_offset` inside
// every peer's symmetric buffer; copy it to the device and pass it as c_maps.
void build_peer_c_maps(const uint64_t* peer_base_ptrs, int world, long long byte_offset, int rows, int N, long long ldc, bool f32,
                       void* host_out);

// Expert-parallel dispatch. For assignment a = (token t, choice k) with expert e = idx[a] (or -1): destination rank
// e / experts_per_rank, segment (e % experts_per_rank, source rank), position pos[a] inside the segment (< cap or the
// assignment is dropped). Copies row t of x into the destination's input buffer and records the return slot
// (source rank * slots_per_rank + a) in the destination's row_dst table; publishes this rank's per-expert counts.
void launch_ep_dispatch(const __nv_bfloat16* x, int d, const int* idx, const int* pos, int n_assign, int top_k, int experts_per_rank,
                        int cap, int rank, int world, const uint64_t* peer_bufs, long long in_off, long long dst_off,
                        long long cnt_off, const int* counts, int num_experts, int slots_per_rank, cudaStream_t s);

// On the expert owner, after the dispatch barrier: builds tile_group for the grouped GEMM from the received counts and
// invalidates (row_dst = -1) the rows of every segment beyond its count.
void launch_ep_build_tiles(const int* counts_all /* [world][experts_per_rank] */, int experts_per_rank, int world, int cap,
                           int* tile_group, int* row_dst, cudaStream_t s);

// Zeroes the rows of an expert-major buffer [experts_per_rank][world][cap][d] beyond each segment's count.
void launch_ep_zero_invalid_rows(__nv_bfloat16* buf, int d, const int* counts_all, int experts_per_rank, int world, int cap,
                                 cudaStream_t s);

}  // namespace tb
