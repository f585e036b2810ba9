/* C ABI of the native engine library (libtriune_core.so).
 *
 * Symbol names, argument order and struct layouts follow the reference's csrc/engine/api.h:20-103 so hosts
 * written against it (ctypes, P/Invoke) keep working. The CUDA runtime is bound at run time with dlopen, so
 * the library also loads on machines without a GPU; there every device feature degrades to host memory.
 */
#ifndef TRIUNE_B200_ENGINE_API_H
#define TRIUNE_B200_ENGINE_API_H

#include <stdint.h>

#if defined(_WIN32)
#define TRIUNE_API __declspec(dllexport)
#else
#define TRIUNE_API __attribute__((visibility("default")))
#endif

#ifdef __cplusplus
extern "C" {
#endif

typedef struct TriuneEngine TriuneEngine;

typedef struct {
  int vocab_size;
  int hidden_dim;
  int num_layers;
  int num_heads;
  int head_dim;
  int num_experts;
  int top_k;
  int max_seq_len;
  float reflex_threshold;
} TriuneConfig;

typedef struct {
  float loss;             /* last values given to triune_engine_set_losses (the engine does not invent losses) */
  float lm_loss;
  float router_loss;
  int active_tier;        /* 0 Reflex, 1 Limbic, 2 Cortex */
  int tokens_processed;
  float step_time_ms;     /* measured: host->device staging + graph replay + stream sync */
  float vram_used_mb;     /* bytes held by the engine arena */
  int cuda_runtime_bound; /* 1 when libcudart was found and a device is usable */
} TriuneStepStats;

/* 1. lifecycle */
TRIUNE_API TriuneEngine* triune_engine_create(const TriuneConfig* config, int device_id);
TRIUNE_API void triune_engine_destroy(TriuneEngine* engine);
TRIUNE_API const char* triune_engine_version(void);
TRIUNE_API int triune_has_cuda_runtime(void);

/* 2. step: stage token ids to the device through the pinned ring, replay the captured graph (if any), sync */
TRIUNE_API int triune_engine_step(TriuneEngine* engine, const uint16_t* input_tokens, const uint16_t* target_tokens,
                                  int batch_size, int seq_len, TriuneStepStats* out_stats);

/* 3. CUDA graph capture / replay on the engine stream */
TRIUNE_API int triune_cuda_graph_capture(TriuneEngine* engine, int batch_size, int seq_len);
TRIUNE_API int triune_cuda_graph_replay(TriuneEngine* engine);

/* 4. CPU operator entry points (fp32, contiguous) */
TRIUNE_API void triune_centroid_steer_update_f32(float* P, const float* Grad_proj, int rows, int cols, float steer_scale,
                                                 float momentum);
TRIUNE_API void triune_route_tiers_f32(const float* logits, float* probs_out, int* selected_tiers_out, int batch_size,
                                       float reflex_threshold);
TRIUNE_API void triune_compute_neuron_heatmap_f32(const float* activations, float* bins_out, uint32_t* rgba_out,
                                                  int num_elements, int num_bins);
TRIUNE_API void triune_gla_recurrent_step_f32(const float* q, const float* k, const float* v, const float* g, float* state,
                                              float* out, int batch_heads, int head_dim);

/* 5. additions of this library */
TRIUNE_API void triune_engine_set_losses(TriuneEngine* engine, float loss, float lm_loss, float router_loss, int tier);
/* tier colour image (Reflex #10B981, Limbic #F59E0B, Cortex #8B5CF6, scaled by clamp(|act|,0,1)); ABGR packed */
TRIUNE_API void triune_tier_colour_render_f32(const float* activations, const int* tiers, uint32_t* rgba_out, int rows,
                                              int width);
/* pinned host -> device staging ring (cudaMemcpyAsync on a side stream, one event per slot) */
TRIUNE_API void* triune_stage_ring_create(int device_id, int num_slots, uint64_t slot_bytes);
TRIUNE_API void triune_stage_ring_destroy(void* ring);
/* copy src (host) into slot's pinned buffer and start the async copy to dst_device; returns slot index or <0 */
TRIUNE_API int triune_stage_ring_submit(void* ring, const void* src_host, void* dst_device, uint64_t bytes);
/* block the calling thread until the slot's copy has landed; returns 0 on success */
TRIUNE_API int triune_stage_ring_wait(void* ring, int slot);
TRIUNE_API void* triune_stage_ring_host_ptr(void* ring, int slot);
TRIUNE_API uint64_t triune_stage_ring_bytes_moved(void* ring);

#ifdef __cplusplus
}
#endif
#endif
