// In-kernel NVLink collectives over symmetric memory: peer load/store, NVLS multimem reduce/broadcast,
// epoch-counted flags with bounded waits. No NCCL on these paths.
//
// Every rank owns one symmetric buffer mapped by all peers (peer base pointers come as a device array) and one
// signal pad of 32-bit epoch counters. Flag slot (channel c, source rank s) of a pad is word c*MAX_RANKS + s.
// A notification is a st.release.sys of the current epoch into the peer's pad; a wait is a bounded
// ld.acquire.sys spin on the local pad that gives up after WAIT_LIMIT_NS and sets the status word.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace tb {

constexpr int COMM_MAX_RANKS = 16;

enum CommChannel : int {
  CH_GRADS_READY = 0,   // backward finished, gradients may be read by peers
  CH_NORM_PARTIAL = 1,  // reduced-shard sum of squares published (also: this rank finished reading peers)
  CH_PARAMS_DONE = 2,   // updated parameters written into every peer
  CH_USER0 = 3,
  CH_USER1 = 4,
  CH_USER2 = 5,
  CH_USER3 = 6,
};

struct PeerTable {
  int rank;
  int world;
  const uint64_t* bufs;     // [world] device pointers to the peers' symmetric data buffers
  const uint64_t* signals;  // [world] device pointers to the peers' signal pads
  uint64_t multicast;       // NVLS multicast address of the data buffer (0 = unavailable)
};

struct ElemRange {
  long long begin, end;  // element offsets into the flat buffers
};

// Owned ranges of this rank (AdamW shard, owned Muon matrices, owned experts): at most 64 pieces.
struct RangeList {
  int count;
  ElemRange r[64];
};

// Phase 1 of the fused data-parallel step. For every owned range: g = (1/world) * sum_p grad_p (peer loads or
// multimem.ld_reduce), written in place into the local gradient buffer; accumulates the sum of squares of the
// reduced values; the last CTA publishes that partial to every peer (slot [rank] of their norm array) and raises
// CH_NORM_PARTIAL. grad_off / norm_off are byte offsets of the gradient arena and of the fp32[world] norm array
// inside the symmetric buffer.
void launch_dp_reduce_scatter(PeerTable pt, long long grad_off, long long norm_off, RangeList ranges, uint32_t epoch,
                              const uint32_t* epoch_dev, bool use_multimem, unsigned int* block_counter, int* status, cudaStream_t s);

// Phase 2 for the AdamW tier: waits for all norm partials, derives the clip coefficient (written to clip_out),
// applies AdamW to the owned range and stores the new bf16 parameters into EVERY rank's parameter arena.
void launch_dp_adamw_allgather(PeerTable pt, long long grad_off, long long norm_off, long long param_off,
                               ElemRange owned, long long state_base, float* master, float* m, float* v, float lr,
                               float beta1, float beta2, float eps, float wd, float bc1, float bc2, float max_norm,
                               float* clip_out, float* norm_out, uint32_t epoch, const uint32_t* epoch_dev,
                               const float* hyper, bool use_multimem, int* status, cudaStream_t s);

// Broadcast locally updated bf16 parameter ranges to every peer (plain peer stores or multimem.st).
void launch_dp_broadcast_ranges(PeerTable pt, long long param_off, RangeList ranges, bool use_multimem,
                                cudaStream_t s);

// All ranks: raise `channel` on every peer, then wait until every peer raised it (bounded). One CTA.
void launch_comm_barrier(PeerTable pt, int channel, uint32_t epoch, const uint32_t* epoch_dev, int* status,
                         cudaStream_t s);

// Scalar metrics all-reduce (sum) piggy-backed on the signal protocol: each rank stores its `n` floats into slot
// [rank] of every peer's metric array, barriers, and sums. out[n] on every rank.
void launch_metric_allreduce(PeerTable pt, long long metric_off, const float* local, float* out, int n, int channel,
                             uint32_t epoch, const uint32_t* epoch_dev, int* status, cudaStream_t s);

// A wait that is expected to expire (used by failure-detection tests): waits on a channel nobody raises with a
// short limit and reports ST_TIMEOUT_PEER through status; the context stays usable.
void launch_comm_wait_only(PeerTable pt, int channel, uint32_t epoch, unsigned long long limit_ns, int* status,
                           cudaStream_t s);

}  // namespace tb
