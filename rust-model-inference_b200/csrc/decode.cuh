// Launchers of the decode-step kernels (decode.cu), used by the session code (qwen3.cu).
#pragma once
#include "common.cuh"

struct decode_dims {
  size_t batch, capacity;
  size_t n_embd, n_layer, n_head, n_head_kv, hd, n_ff, vocab;
  float eps;
};

int32_t launch_embed(rmi_ctx* ctx, const rmi_weight* emb, const uint32_t* prompts, size_t n_prompt, const uint32_t* gen,
                     size_t n_gen, const int* d_step, float* x, size_t batch);
int32_t launch_rmsnorm_quant(rmi_ctx* ctx, float* x, const float* add, const float* weight, size_t n, float eps,
                             uint8_t* q8, float* scales, size_t batch);
int32_t launch_qk_norm_rope_kv(rmi_ctx* ctx, const decode_dims& d, const float* qkv, const float* q_norm,
                               const float* k_norm, const float* rope, const int* d_step, uint16_t* q16,
                               uint16_t* k_cache, uint16_t* v_cache, size_t layer, float* q32 = nullptr,
                               float* k32_cache = nullptr, float* v32_cache = nullptr);
size_t attention_smem_bytes(const decode_dims& d);
int32_t launch_attention(rmi_ctx* ctx, const decode_dims& d, const uint16_t* q16, uint16_t* k_cache,
                         uint16_t* v_cache, const int* d_step, size_t layer, float* attn_out, uint8_t* q8,
                         float* scales, const float* qkv = nullptr, const float* q_norm = nullptr,
                         const float* k_norm = nullptr, const float* rope = nullptr);
bool attention_seq_shape_ok(const decode_dims& d);
bool attention_seq_eligible(const decode_dims& d);
size_t attention_seq_smem_bytes(const decode_dims& d, bool global_scores);
size_t attention_seq_scratch_bytes(const decode_dims& d);
// score_scratch: null = score rows in shared memory; else attention_seq_scratch_bytes(d) bytes of device memory
int32_t launch_attention_seq(rmi_ctx* ctx, const decode_dims& d, const uint16_t* q16, const uint16_t* k_cache,
                             const uint16_t* v_cache, const int* d_step, size_t layer, float* attn_out, uint8_t* q8,
                             float* scales, void* score_scratch);
// shared memory per CTA of the attention kernel a CLI forward variant (RMI_FORWARD_APP_*) uses
size_t cli_attention_smem_bytes(const decode_dims& d, int forward);
int32_t launch_attention_online(rmi_ctx* ctx, const decode_dims& d, const float* q32, const uint16_t* k_cache,
                                const uint16_t* v_cache, const int* d_step, size_t layer, float* attn_out, uint8_t* q8,
                                float* scales);
int32_t launch_attention_f32kv(rmi_ctx* ctx, const decode_dims& d, const float* q32, const float* k_cache,
                               const float* v_cache, const int* d_step, size_t layer, float* attn_out, uint8_t* q8,
                               float* scales, bool sequential_pv = false);
int32_t launch_attention_scores_f16kv(rmi_ctx* ctx, const decode_dims& d, const float* q32, const uint16_t* k_cache,
                                      const uint16_t* v_cache, const int* d_step, size_t layer, float* attn_out,
                                      uint8_t* q8, float* scales);
size_t argmax_scratch_floats(size_t batch);
int32_t launch_argmax(rmi_ctx* ctx, const float* logits, size_t vocab, const int* d_step, size_t n_prompt, uint32_t* gen,
                      size_t n_gen, int* flag, size_t batch, float* part_v, uint32_t* part_i, bool last_index = false);
int32_t launch_step_inc(rmi_ctx* ctx, int* d_step);

// prefill.cu: batched prompt processing (rows r = b_local * P + p for sequences b0.. and positions p < P)
bool prefill_supported(const rmi_ctx* ctx, const decode_dims& d, size_t P);
int32_t launch_embed_rows(rmi_ctx* ctx, const rmi_weight* emb, const uint32_t* prompts, size_t n_prompt, size_t P, size_t b0,
                          size_t rows, float* x);
int32_t launch_rmsnorm_rows(rmi_ctx* ctx, float* x, const float* add, const float* weight, size_t n, float eps, float* out,
                            size_t rows);
int32_t launch_qk_norm_rope_kv_rows(rmi_ctx* ctx, const decode_dims& d, const float* qkv, const float* q_norm,
                                    const float* k_norm, const float* rope, size_t P, size_t b0, size_t rows, uint16_t* q16,
                                    uint16_t* k_cache, uint16_t* v_cache, size_t layer);
int32_t launch_attention_prefill(rmi_ctx* ctx, const decode_dims& d, const uint16_t* q16, const uint16_t* k_cache,
                                 const uint16_t* v_cache, size_t layer, size_t P, size_t b0, size_t n_seq, float* attn_out);
int32_t launch_set_step(rmi_ctx* ctx, int* d_step, int value);
