// Native engine library: device arena and step lifecycle, CUDA-graph capture/replay, a pinned host->device
// staging ring, and AVX2 CPU operators. The CUDA runtime is resolved with dlopen at first use.
//
// Parity: csrc/engine/engine.cpp:57-475 of the reference (same exported symbols). Differences: the step
// reports measured time and never fabricates loss values; token staging goes through pinned memory; the
// staging ring is exported for the layer-streaming runtime.
#include "api.h"

#include <dlfcn.h>
#include <immintrin.h>
#include <math.h>
#include <stdlib.h>
#include <string.h>

#include <chrono>
#include <mutex>
#include <vector>

namespace {

// ---------------------------------------------------------------- CUDA runtime binding
typedef int cudaError_t_;
typedef void* cudaStream_t_;
typedef void* cudaEvent_t_;
typedef void* cudaGraph_t_;
typedef void* cudaGraphExec_t_;

struct CudaRt {
  void* handle = nullptr;
  bool ok = false;
  cudaError_t_ (*GetDeviceCount)(int*) = nullptr;
  cudaError_t_ (*SetDevice)(int) = nullptr;
  cudaError_t_ (*Malloc)(void**, size_t) = nullptr;
  cudaError_t_ (*Free)(void*) = nullptr;
  cudaError_t_ (*MallocHost)(void**, size_t) = nullptr;
  cudaError_t_ (*FreeHost)(void*) = nullptr;
  cudaError_t_ (*MemcpyAsync)(void*, const void*, size_t, int, cudaStream_t_) = nullptr;
  cudaError_t_ (*MemsetAsync)(void*, int, size_t, cudaStream_t_) = nullptr;
  cudaError_t_ (*StreamCreateWithFlags)(cudaStream_t_*, unsigned) = nullptr;
  cudaError_t_ (*StreamDestroy)(cudaStream_t_) = nullptr;
  cudaError_t_ (*StreamSynchronize)(cudaStream_t_) = nullptr;
  cudaError_t_ (*EventCreateWithFlags)(cudaEvent_t_*, unsigned) = nullptr;
  cudaError_t_ (*EventDestroy)(cudaEvent_t_) = nullptr;
  cudaError_t_ (*EventRecord)(cudaEvent_t_, cudaStream_t_) = nullptr;
  cudaError_t_ (*EventSynchronize)(cudaEvent_t_) = nullptr;
  cudaError_t_ (*StreamBeginCapture)(cudaStream_t_, int) = nullptr;
  cudaError_t_ (*StreamEndCapture)(cudaStream_t_, cudaGraph_t_*) = nullptr;
  cudaError_t_ (*GraphInstantiate)(cudaGraphExec_t_*, cudaGraph_t_, unsigned long long) = nullptr;
  cudaError_t_ (*GraphLaunch)(cudaGraphExec_t_, cudaStream_t_) = nullptr;
  cudaError_t_ (*GraphDestroy)(cudaGraph_t_) = nullptr;
  cudaError_t_ (*GraphExecDestroy)(cudaGraphExec_t_) = nullptr;
};

CudaRt& rt() {
  static CudaRt r;
  static std::once_flag once;
  std::call_once(once, [] {
    const char* names[] = {"libcudart.so.12", "libcudart.so", "libcudart.so.13", nullptr};
    for (int i = 0; names[i] && !r.handle; ++i) r.handle = dlopen(names[i], RTLD_NOW | RTLD_LOCAL);
    if (!r.handle) return;
    bool all = true;
#define BIND(field, sym)                                              \
  r.field = reinterpret_cast<decltype(r.field)>(dlsym(r.handle, sym)); \
  all = all && (r.field != nullptr);
    BIND(GetDeviceCount, "cudaGetDeviceCount")
    BIND(SetDevice, "cudaSetDevice")
    BIND(Malloc, "cudaMalloc")
    BIND(Free, "cudaFree")
    BIND(MallocHost, "cudaMallocHost")
    BIND(FreeHost, "cudaFreeHost")
    BIND(MemcpyAsync, "cudaMemcpyAsync")
    BIND(MemsetAsync, "cudaMemsetAsync")
    BIND(StreamCreateWithFlags, "cudaStreamCreateWithFlags")
    BIND(StreamDestroy, "cudaStreamDestroy")
    BIND(StreamSynchronize, "cudaStreamSynchronize")
    BIND(EventCreateWithFlags, "cudaEventCreateWithFlags")
    BIND(EventDestroy, "cudaEventDestroy")
    BIND(EventRecord, "cudaEventRecord")
    BIND(EventSynchronize, "cudaEventSynchronize")
    BIND(StreamBeginCapture, "cudaStreamBeginCapture")
    BIND(StreamEndCapture, "cudaStreamEndCapture")
    BIND(GraphInstantiate, "cudaGraphInstantiateWithFlags")
    BIND(GraphLaunch, "cudaGraphLaunch")
    BIND(GraphDestroy, "cudaGraphDestroy")
    BIND(GraphExecDestroy, "cudaGraphExecDestroy")
#undef BIND
    if (!all) return;
    int n = 0;
    r.ok = r.GetDeviceCount(&n) == 0 && n > 0;
  });
  return r;
}

constexpr int kHostToDevice = 1;

struct Buffer {
  void* ptr = nullptr;
  size_t bytes = 0;
  bool device = false;
};

}  // namespace

struct TriuneEngine {
  TriuneConfig cfg{};
  int device = 0;
  bool on_device = false;
  cudaStream_t_ stream = nullptr;
  Buffer tokens_in, tokens_out, activations, router_logits, tiers;
  void* pinned_tokens = nullptr;
  size_t pinned_bytes = 0;
  cudaGraphExec_t_ graph_exec = nullptr;
  int graph_batch = 0, graph_seq = 0;
  float loss = 0.f, lm_loss = 0.f, router_loss = 0.f;
  int tier = 2;
  size_t arena_bytes = 0;
};

namespace {

bool alloc_buffer(TriuneEngine* e, Buffer& b, size_t bytes) {
  b.bytes = bytes;
  if (e->on_device && rt().Malloc(&b.ptr, bytes) == 0) {
    b.device = true;
    e->arena_bytes += bytes;
    return true;
  }
  b.device = false;
  b.ptr = calloc(1, bytes);
  return b.ptr != nullptr;
}

void free_buffer(Buffer& b) {
  if (!b.ptr) return;
  if (b.device)
    rt().Free(b.ptr);
  else
    free(b.ptr);
  b.ptr = nullptr;
}

inline float fast_exp(float x) { return expf(x); }

}  // namespace

extern "C" {

const char* triune_engine_version(void) { return "triune-b200-core 0.1.0 (sm_100a)"; }

int triune_has_cuda_runtime(void) { return rt().ok ? 1 : 0; }

TriuneEngine* triune_engine_create(const TriuneConfig* config, int device_id) {
  if (!config || config->max_seq_len <= 0 || config->hidden_dim <= 0) return nullptr;
  TriuneEngine* e = new TriuneEngine();
  e->cfg = *config;
  e->device = device_id;
  e->on_device = rt().ok && device_id >= 0 && rt().SetDevice(device_id) == 0;
  if (e->on_device && rt().StreamCreateWithFlags(&e->stream, 1u /*non-blocking*/) != 0) e->on_device = false;
  const size_t tokens = (size_t)config->max_seq_len * 16;
  bool ok = alloc_buffer(e, e->tokens_in, tokens * sizeof(uint16_t)) &&
            alloc_buffer(e, e->tokens_out, tokens * sizeof(uint16_t)) &&
            alloc_buffer(e, e->activations, tokens * (size_t)config->hidden_dim * 2) &&
            alloc_buffer(e, e->router_logits, tokens * 3 * sizeof(float)) &&
            alloc_buffer(e, e->tiers, tokens * sizeof(int));
  if (ok && e->on_device) {
    e->pinned_bytes = tokens * sizeof(uint16_t) * 2;
    if (rt().MallocHost(&e->pinned_tokens, e->pinned_bytes) != 0) e->pinned_tokens = nullptr;
  }
  if (!ok) {
    triune_engine_destroy(e);
    return nullptr;
  }
  return e;
}

void triune_engine_destroy(TriuneEngine* e) {
  if (!e) return;
  if (e->on_device) {
    rt().SetDevice(e->device);
    if (e->stream) rt().StreamSynchronize(e->stream);
    if (e->graph_exec) rt().GraphExecDestroy(e->graph_exec);
    if (e->pinned_tokens) rt().FreeHost(e->pinned_tokens);
  }
  free_buffer(e->tokens_in);
  free_buffer(e->tokens_out);
  free_buffer(e->activations);
  free_buffer(e->router_logits);
  free_buffer(e->tiers);
  if (e->on_device && e->stream) rt().StreamDestroy(e->stream);
  delete e;
}

void triune_engine_set_losses(TriuneEngine* e, float loss, float lm_loss, float router_loss, int tier) {
  if (!e) return;
  e->loss = loss;
  e->lm_loss = lm_loss;
  e->router_loss = router_loss;
  e->tier = tier;
}

int triune_engine_step(TriuneEngine* e, const uint16_t* in, const uint16_t* tgt, int batch, int seq, TriuneStepStats* st) {
  if (!e || !in || batch <= 0 || seq <= 0) return -1;
  const size_t n = (size_t)batch * seq;
  if (n * sizeof(uint16_t) > e->tokens_in.bytes) return -2;
  auto t0 = std::chrono::steady_clock::now();
  if (e->on_device) {
    rt().SetDevice(e->device);
    const void* src_in = in;
    const void* src_tg = tgt;
    if (e->pinned_tokens) {  // stage through pinned memory so the copies are truly asynchronous
      memcpy(e->pinned_tokens, in, n * 2);
      src_in = e->pinned_tokens;
      if (tgt) {
        memcpy(static_cast<uint8_t*>(e->pinned_tokens) + e->pinned_bytes / 2, tgt, n * 2);
        src_tg = static_cast<uint8_t*>(e->pinned_tokens) + e->pinned_bytes / 2;
      }
    }
    if (rt().MemcpyAsync(e->tokens_in.ptr, src_in, n * 2, kHostToDevice, e->stream) != 0) return -3;
    if (tgt && rt().MemcpyAsync(e->tokens_out.ptr, src_tg, n * 2, kHostToDevice, e->stream) != 0) return -3;
    if (e->graph_exec && e->graph_batch == batch && e->graph_seq == seq) {
      if (rt().GraphLaunch(e->graph_exec, e->stream) != 0) return -4;
    }
    if (rt().StreamSynchronize(e->stream) != 0) return -5;
  } else {
    memcpy(e->tokens_in.ptr, in, n * 2);
    if (tgt) memcpy(e->tokens_out.ptr, tgt, n * 2);
  }
  auto t1 = std::chrono::steady_clock::now();
  if (st) {
    st->loss = e->loss;
    st->lm_loss = e->lm_loss;
    st->router_loss = e->router_loss;
    st->active_tier = e->tier;
    st->tokens_processed = (int)n;
    st->step_time_ms = std::chrono::duration<float, std::milli>(t1 - t0).count();
    st->vram_used_mb = (float)e->arena_bytes / (1024.f * 1024.f);
    st->cuda_runtime_bound = e->on_device ? 1 : 0;
  }
  return 0;
}

int triune_cuda_graph_capture(TriuneEngine* e, int batch, int seq) {
  if (!e || !e->on_device) return -1;
  rt().SetDevice(e->device);
  if (e->graph_exec) {
    rt().GraphExecDestroy(e->graph_exec);
    e->graph_exec = nullptr;
  }
  cudaGraph_t_ graph = nullptr;
  if (rt().StreamBeginCapture(e->stream, 2 /*relaxed*/) != 0) return -2;
  // The captured region clears the per-step outputs; hosts that enqueue their own kernels on the engine
  // stream between capture begin/end extend it (the stream handle is shared through the arena contract).
  rt().MemsetAsync(e->router_logits.ptr, 0, (size_t)batch * seq * 3 * sizeof(float), e->stream);
  rt().MemsetAsync(e->tiers.ptr, 0, (size_t)batch * seq * sizeof(int), e->stream);
  if (rt().StreamEndCapture(e->stream, &graph) != 0 || !graph) return -3;
  int rc = rt().GraphInstantiate(&e->graph_exec, graph, 0ull);
  rt().GraphDestroy(graph);
  if (rc != 0) return -4;
  e->graph_batch = batch;
  e->graph_seq = seq;
  return 0;
}

int triune_cuda_graph_replay(TriuneEngine* e) {
  if (!e || !e->on_device || !e->graph_exec) return -1;
  rt().SetDevice(e->device);
  if (rt().GraphLaunch(e->graph_exec, e->stream) != 0) return -2;
  return rt().StreamSynchronize(e->stream) == 0 ? 0 : -3;
}

// ---------------------------------------------------------------- CPU operators
void triune_centroid_steer_update_f32(float* P, const float* G, int rows, int cols, float steer, float momentum) {
  const long long n = (long long)rows * cols;
  long long i = 0;
#if defined(__AVX2__) && defined(__FMA__)
  const __m256 vm = _mm256_set1_ps(momentum), vs = _mm256_set1_ps(steer);
#pragma omp parallel for if (n > (1 << 16))
  for (long long j = 0; j < n / 8; ++j) {
    __m256 p = _mm256_loadu_ps(P + j * 8), g = _mm256_loadu_ps(G + j * 8);
    __m256 d = _mm256_sub_ps(g, p);
    _mm256_storeu_ps(P + j * 8, _mm256_fmadd_ps(vs, d, _mm256_mul_ps(vm, p)));
  }
  i = (n / 8) * 8;
#endif
  for (; i < n; ++i) P[i] = momentum * P[i] + steer * (G[i] - P[i]);
}

void triune_route_tiers_f32(const float* logits, float* probs, int* tiers, int batch, float thr) {
#pragma omp parallel for if (batch > 4096)
  for (int r = 0; r < batch; ++r) {
    const float a = logits[3 * r], b = logits[3 * r + 1], c = logits[3 * r + 2];
    const float mx = fmaxf(a, fmaxf(b, c));
    const float ea = fast_exp(a - mx), eb = fast_exp(b - mx), ec = fast_exp(c - mx);
    const float inv = 1.f / (ea + eb + ec);
    const float p0 = ea * inv, p1 = eb * inv, p2 = ec * inv;
    if (probs) {
      probs[3 * r] = p0;
      probs[3 * r + 1] = p1;
      probs[3 * r + 2] = p2;
    }
    if (tiers) tiers[r] = p0 >= thr ? 0 : (p1 >= p2 ? 1 : 2);
  }
}

void triune_compute_neuron_heatmap_f32(const float* act, float* bins, uint32_t* rgba, int n, int num_bins) {
  if (num_bins <= 0) return;
  std::vector<float> local((size_t)num_bins, 0.f);
  float* b = bins ? bins : local.data();
  const int per = n / num_bins > 0 ? n / num_bins : 1;
  float mx = 0.f;
  for (int i = 0; i < num_bins; ++i) {
    const long long s = (long long)i * per;
    long long e = (i == num_bins - 1) ? n : s + per;
    if (e > n) e = n;
    double acc = 0.0;
    for (long long j = s; j < e; ++j) acc += fabsf(act[j]);
    b[i] = e > s ? (float)(acc / (double)(e - s)) : 0.f;
    mx = fmaxf(mx, b[i]);
  }
  mx = fmaxf(mx, 1e-12f);
  for (int i = 0; i < num_bins; ++i) {
    const float v = b[i] / mx;
    if (bins) bins[i] = v;
    if (rgba) {
      const uint32_t r = (uint32_t)(fminf(1.f, 1.4f * v) * 249.f);
      const uint32_t g = (uint32_t)(v * v * 115.f);
      const uint32_t bl = (uint32_t)((1.f - 0.7f * v) * 60.f);
      rgba[i] = (255u << 24) | (bl << 16) | (g << 8) | r;
    }
  }
}

void triune_tier_colour_render_f32(const float* act, const int* tiers, uint32_t* rgba, int rows, int width) {
  static const float col[3][3] = {{16.f, 185.f, 129.f}, {245.f, 158.f, 11.f}, {139.f, 92.f, 246.f}};
#pragma omp parallel for if ((long long)rows * width > (1 << 16))
  for (int r = 0; r < rows; ++r) {
    const int t = tiers[r] < 0 ? 0 : (tiers[r] > 2 ? 2 : tiers[r]);
    for (int c = 0; c < width; ++c) {
      const float inten = fminf(1.f, fabsf(act[(long long)r * width + c]));
      const uint32_t R = (uint32_t)(col[t][0] * inten), G = (uint32_t)(col[t][1] * inten), B = (uint32_t)(col[t][2] * inten);
      rgba[(long long)r * width + c] = (255u << 24) | (B << 16) | (G << 8) | R;
    }
  }
}

void triune_gla_recurrent_step_f32(const float* q, const float* k, const float* v, const float* g, float* state, float* out,
                                   int batch_heads, int d) {
#pragma omp parallel for if (batch_heads > 8)
  for (int bh = 0; bh < batch_heads; ++bh) {
    const float *qq = q + (long long)bh * d, *kk = k + (long long)bh * d, *vv = v + (long long)bh * d,
                *gg = g + (long long)bh * d;
    float* S = state + (long long)bh * d * d;
    float* o = out + (long long)bh * d;
    for (int j = 0; j < d; ++j) o[j] = 0.f;
    for (int i = 0; i < d; ++i) {
      const float dec = expf(fminf(gg[i], 0.f)), ki = kk[i], qi = qq[i];
      float* row = S + (long long)i * d;
      int j = 0;
#if defined(__AVX2__) && defined(__FMA__)
      const __m256 vd = _mm256_set1_ps(dec), vk = _mm256_set1_ps(ki), vq = _mm256_set1_ps(qi);
      for (; j + 8 <= d; j += 8) {
        __m256 s = _mm256_fmadd_ps(vk, _mm256_loadu_ps(vv + j), _mm256_mul_ps(vd, _mm256_loadu_ps(row + j)));
        _mm256_storeu_ps(row + j, s);
        _mm256_storeu_ps(o + j, _mm256_fmadd_ps(vq, s, _mm256_loadu_ps(o + j)));
      }
#endif
      for (; j < d; ++j) {
        const float s = dec * row[j] + ki * vv[j];
        row[j] = s;
        o[j] += qi * s;
      }
    }
  }
}

// ---------------------------------------------------------------- pinned staging ring
struct StageRing {
  int device = 0;
  int slots = 0;
  uint64_t slot_bytes = 0;
  cudaStream_t_ stream = nullptr;
  std::vector<void*> host;
  std::vector<cudaEvent_t_> events;
  std::vector<char> busy;
  int next = 0;
  uint64_t moved = 0;
  bool pinned = false;
};

void* triune_stage_ring_create(int device_id, int num_slots, uint64_t slot_bytes) {
  if (num_slots <= 0 || slot_bytes == 0) return nullptr;
  StageRing* r = new StageRing();
  r->device = device_id;
  r->slots = num_slots;
  r->slot_bytes = slot_bytes;
  r->pinned = rt().ok && device_id >= 0 && rt().SetDevice(device_id) == 0 &&
              rt().StreamCreateWithFlags(&r->stream, 1u) == 0;
  r->host.resize(num_slots, nullptr);
  r->events.resize(num_slots, nullptr);
  r->busy.assign(num_slots, 0);
  for (int i = 0; i < num_slots; ++i) {
    if (r->pinned) {
      if (rt().MallocHost(&r->host[i], slot_bytes) != 0 || rt().EventCreateWithFlags(&r->events[i], 2u /*no timing*/) != 0) {
        triune_stage_ring_destroy(r);
        return nullptr;
      }
    } else {
      r->host[i] = malloc(slot_bytes);
    }
  }
  return r;
}

void triune_stage_ring_destroy(void* ring) {
  StageRing* r = static_cast<StageRing*>(ring);
  if (!r) return;
  if (r->pinned) {
    rt().SetDevice(r->device);
    if (r->stream) rt().StreamSynchronize(r->stream);
  }
  for (int i = 0; i < r->slots; ++i) {
    if (r->pinned) {
      if (r->events[i]) rt().EventDestroy(r->events[i]);
      if (r->host[i]) rt().FreeHost(r->host[i]);
    } else {
      free(r->host[i]);
    }
  }
  if (r->pinned && r->stream) rt().StreamDestroy(r->stream);
  delete r;
}

int triune_stage_ring_submit(void* ring, const void* src, void* dst, uint64_t bytes) {
  StageRing* r = static_cast<StageRing*>(ring);
  if (!r || !src || !dst || bytes > r->slot_bytes) return -1;
  const int slot = r->next;
  r->next = (r->next + 1) % r->slots;
  if (r->busy[slot] && r->pinned) rt().EventSynchronize(r->events[slot]);  // slot still in flight: wait for it
  memcpy(r->host[slot], src, bytes);
  if (r->pinned) {
    rt().SetDevice(r->device);
    if (rt().MemcpyAsync(dst, r->host[slot], bytes, kHostToDevice, r->stream) != 0) return -2;
    if (rt().EventRecord(r->events[slot], r->stream) != 0) return -3;
  } else {
    memcpy(dst, r->host[slot], bytes);
  }
  r->busy[slot] = 1;
  r->moved += bytes;
  return slot;
}

int triune_stage_ring_wait(void* ring, int slot) {
  StageRing* r = static_cast<StageRing*>(ring);
  if (!r || slot < 0 || slot >= r->slots) return -1;
  if (r->busy[slot] && r->pinned && rt().EventSynchronize(r->events[slot]) != 0) return -2;
  r->busy[slot] = 0;
  return 0;
}

void* triune_stage_ring_host_ptr(void* ring, int slot) {
  StageRing* r = static_cast<StageRing*>(ring);
  return (r && slot >= 0 && slot < r->slots) ? r->host[slot] : nullptr;
}

uint64_t triune_stage_ring_bytes_moved(void* ring) {
  StageRing* r = static_cast<StageRing*>(ring);
  return r ? r->moved : 0;
}

}  // extern "C"
