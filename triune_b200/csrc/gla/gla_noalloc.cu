// Allocation-free variant of the GLA forward: same kernels as the torch entry point (gla_fwd), with the scratch
// they need taken from a file-scope device array instead of the caller's allocator. See gla_noalloc.h.
#include "gla_noalloc.h"

#include <stdint.h>

#include "gla.cuh"

namespace {

constexpr unsigned long long kMaxChunks = TRIUNE_NOALLOC_MAX_CHUNKS;
constexpr unsigned long long kKvBytes = kMaxChunks * 64ull * 64ull * 4ull;      // fp32 chunk contributions
constexpr unsigned long long kDecayBytes = kMaxChunks * 64ull * 4ull;           // fp32 chunk decays
constexpr unsigned long long kStatesBytes = kMaxChunks * 64ull * 64ull * 2ull;  // bf16 chunk-start states
constexpr unsigned long long kStatusBytes = 256ull;
constexpr unsigned long long kScratchBytes = kKvBytes + kDecayBytes + kStatesBytes + kStatusBytes;

// In host code this name is only a handle for cudaGetSymbolAddress; it is not a device pointer.
static __device__ __align__(256) unsigned char g_gla_scratch[kScratchBytes];

constexpr int kMaxDevices = 64;
unsigned char* g_scratch_ptr[kMaxDevices] = {nullptr};

// Device address of the scratch array on the current device (resolved once per device).
unsigned char* scratch_for_current_device(int* err) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
    *err = -3;
    return nullptr;
  }
  if (g_scratch_ptr[dev] == nullptr) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_gla_scratch) != cudaSuccess || p == nullptr) {
      *err = -3;
      return nullptr;
    }
    g_scratch_ptr[dev] = static_cast<unsigned char*>(p);
  }
  return g_scratch_ptr[dev];
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

}  // namespace

extern "C" unsigned long long triune_gla_noalloc_scratch_bytes(void) { return kScratchBytes; }

extern "C" int triune_gla_forward_noalloc(const void* q, const void* k, const void* v, const void* g, void* out,
                                          float* final_state, const float* init_state, int B, int T, int H,
                                          int gate_logits, int* status_out, cudaStream_t stream) {
  if (!q || !k || !v || !g || !out || !final_state || B <= 0 || H <= 0 || T <= 0 || (T % 64) != 0) return -1;
  if (!aligned16(q) || !aligned16(k) || !aligned16(v) || !aligned16(g) || !aligned16(out)) return -1;
  const unsigned long long chunks = (unsigned long long)B * H * (T / 64);
  if (chunks > kMaxChunks) return -2;  // the built-in scratch is sized for TRIUNE_NOALLOC_MAX_CHUNKS chunks
  int err = 0;
  unsigned char* base = scratch_for_current_device(&err);
  if (!base) return err;
  float* kv = reinterpret_cast<float*>(base);
  float* decay = reinterpret_cast<float*>(base + kKvBytes);
  __nv_bfloat16* states = reinterpret_cast<__nv_bfloat16*>(base + kKvBytes + kDecayBytes);
  int* status = reinterpret_cast<int*>(base + kKvBytes + kDecayBytes + kStatesBytes);
  // The status word must start at zero; everything else in the scratch is fully rewritten for the chunks in use.
  if (cudaMemsetAsync(status, 0, sizeof(int), stream) != cudaSuccess) return -3;
  const long long ld = (long long)H * 64;
  tb::GlaMat Q{q, ld, 0}, K{k, ld, 0}, V{v, ld, 0}, G{g, ld, 0}, O{out, ld, 0};
  tb::GlaDims d{B, T, H, gate_logits != 0};
  try {
    tb::launch_gla_chunk_outer(0, K, V, G, kv, decay, d, status, stream);
    tb::launch_gla_scan(kv, decay, init_state, states, final_state, B * H, T / 64, false, stream);
    tb::launch_gla_fwd_out(Q, K, V, G, states, O, d, status, stream);
  } catch (...) {
    return -3;
  }
  if (status_out != nullptr &&
      cudaMemcpyAsync(status_out, status, sizeof(int), cudaMemcpyDeviceToHost, stream) != cudaSuccess)
    return -3;
  return 0;
}
