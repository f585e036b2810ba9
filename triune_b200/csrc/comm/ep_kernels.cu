// Expert-parallel all-to-all dispatch over NVLink peer stores (no NCCL), and the tile-list builder of the expert owner.
//
// Layout on every rank (all inside its symmetric buffer):
//   input buffer   [experts_per_rank][world][cap] rows of d bf16: segment (e, src) holds the tokens rank `src` routed
//                  to local expert e; cap is a multiple of 128 so every GEMM row tile belongs to one segment;
//   row_dst table  one int per input row: where the expert output of that row goes back (rank * slots + slot);
//   counts table   [world][experts_per_rank]: how many rows of each segment are valid this step.
#include <stdexcept>
#include <string>

#include "../common/ptx.cuh"
#include "fused_gemm.cuh"

namespace tb {
namespace {

__global__ void __launch_bounds__(256) ep_dispatch_kernel(const __nv_bfloat16* __restrict__ x, int d, const int* __restrict__ idx,
                                                          const int* __restrict__ pos, int n_assign, int top_k,
                                                          int experts_per_rank, int cap, int rank, int world,
                                                          const uint64_t* __restrict__ peer_bufs, long long in_off,
                                                          long long dst_off, long long cnt_off, const int* __restrict__ counts,
                                                          int num_experts, int slots_per_rank) {
  const int lanes_per_row = d / 8;  // 16-byte vectors per row
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  const int nwarps = (gridDim.x * blockDim.x) >> 5;
  for (int a = warp; a < n_assign; a += nwarps) {
    const int e = idx[a];
    const int ps = pos[a];
    if (e < 0 || ps < 0 || ps >= cap) continue;  // dropped by capacity
    const int dst = e / experts_per_rank, el = e % experts_per_rank;
    const long long row = ((long long)el * world + rank) * cap + ps;
    uint8_t* base = reinterpret_cast<uint8_t*>(peer_bufs[dst]);
    const uint4* src = reinterpret_cast<const uint4*>(x + (long long)(a / top_k) * d);
    uint4* out = reinterpret_cast<uint4*>(base + in_off + row * d * 2);
    for (int j = lane; j < lanes_per_row; j += 32) out[j] = src[j];
    if (lane == 0) reinterpret_cast<int*>(base + dst_off)[row] = rank * slots_per_rank + a;
  }
  // counts: thread i of block 0 publishes count[e = i] to the owner of expert i
  if (blockIdx.x == 0) {
    for (int e = threadIdx.x; e < num_experts; e += blockDim.x) {
      const int dst = e / experts_per_rank, el = e % experts_per_rank;
      int c = counts[e];
      if (c > cap) c = cap;
      reinterpret_cast<int*>(reinterpret_cast<uint8_t*>(peer_bufs[dst]) + cnt_off)[rank * experts_per_rank + el] = c;
    }
  }
}

__global__ void __launch_bounds__(256) ep_build_tiles_kernel(const int* __restrict__ counts_all, int experts_per_rank, int world,
                                                             int cap, int* __restrict__ tile_group, int* __restrict__ row_dst) {
  const int tiles_per_seg = cap / 128;
  const int nseg = experts_per_rank * world;
  const long long total_rows = (long long)nseg * cap;
  for (long long r = (long long)blockIdx.x * blockDim.x + threadIdx.x; r < total_rows; r += (long long)gridDim.x * blockDim.x) {
    const int seg = (int)(r / cap), p = (int)(r % cap);
    const int el = seg / world, src = seg % world;
    const int cnt = counts_all[src * experts_per_rank + el];
    if (p >= cnt) row_dst[r] = -1;
    if ((p & 127) == 0) tile_group[seg * tiles_per_seg + (p >> 7)] = (p < cnt) ? el : -1;
  }
}

// Zero every row of the expert-major buffer that holds no token this step (position >= count of its segment), so
// the weight-gradient GEMMs can run over whole expert ranges. One warp per row.
__global__ void __launch_bounds__(256) ep_zero_invalid_rows_kernel(__nv_bfloat16* __restrict__ buf, int d,
                                                                   const int* __restrict__ counts_all, int experts_per_rank,
                                                                   int world, int cap) {
  const long long total_rows = (long long)experts_per_rank * world * cap;
  const int lane = threadIdx.x & 31;
  const long long warp = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const long long nwarps = ((long long)gridDim.x * blockDim.x) >> 5;
  for (long long r = warp; r < total_rows; r += nwarps) {
    const int seg = (int)(r / cap), p = (int)(r % cap);
    if (p < counts_all[(seg % world) * experts_per_rank + seg / world]) continue;
    uint4* row = reinterpret_cast<uint4*>(buf + r * d);
    for (int j = lane; j < d / 8; j += 32) row[j] = make_uint4(0u, 0u, 0u, 0u);
  }
}

}  // namespace

void launch_ep_zero_invalid_rows(__nv_bfloat16* buf, int d, const int* counts_all, int experts_per_rank, int world, int cap,
                                 cudaStream_t s) {
  if (d % 8 != 0) throw std::runtime_error("ep_zero_invalid_rows: d must be a multiple of 8");
  ep_zero_invalid_rows_kernel<<<148 * 8, 256, 0, s>>>(buf, d, counts_all, experts_per_rank, world, cap);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) throw std::runtime_error(std::string("ep_zero_invalid_rows launch failed: ") + cudaGetErrorString(e));
}

void launch_ep_dispatch(const __nv_bfloat16* x, int d, const int* idx, const int* pos, int n_assign, int top_k, int experts_per_rank,
                        int cap, int rank, int world, const uint64_t* peer_bufs, long long in_off, long long dst_off,
                        long long cnt_off, const int* counts, int num_experts, int slots_per_rank, cudaStream_t s) {
  if (d % 8 != 0) throw std::runtime_error("ep_dispatch: d must be a multiple of 8");
  if (cap % 128 != 0) throw std::runtime_error("ep_dispatch: per-source capacity must be a multiple of 128");
  if (n_assign <= 0) return;
  int blocks = (n_assign + 7) / 8;
  if (blocks > 148 * 8) blocks = 148 * 8;
  ep_dispatch_kernel<<<blocks, 256, 0, s>>>(x, d, idx, pos, n_assign, top_k, experts_per_rank, cap, rank, world, peer_bufs, in_off,
                                            dst_off, cnt_off, counts, num_experts, slots_per_rank);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) throw std::runtime_error(std::string("ep_dispatch launch failed: ") + cudaGetErrorString(e));
}

void launch_ep_build_tiles(const int* counts_all, int experts_per_rank, int world, int cap, int* tile_group, int* row_dst,
                           cudaStream_t s) {
  const long long rows = (long long)experts_per_rank * world * cap;
  int blocks = (int)((rows + 255) / 256);
  if (blocks > 148 * 8) blocks = 148 * 8;
  ep_build_tiles_kernel<<<blocks, 256, 0, s>>>(counts_all, experts_per_rank, world, cap, tile_group, row_dst);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) throw std::runtime_error(std::string("ep_build_tiles launch failed: ") + cudaGetErrorString(e));
}

}  // namespace tb
