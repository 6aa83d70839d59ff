/*
 * rmi_oracle.h -- CPU restatement of the quantized-matmul hot path of
 * rust-model-inference (Rust), written in plain C.
 *
 * TEST INFRASTRUCTURE ONLY.  This library is the checker the CUDA path is compared
 * against and the timed CPU baseline; it is never linked into, loaded by, or called
 * from the product library.
 *
 * Parity status: PINNED.  Every function is checked against the known-answer vectors
 * the reference's own tests hold for this path (tests/test_oracle_golden.py lists each
 * vector with the reference test it comes from).  The reference itself (Rust, crates
 * not vendored) cannot be compiled where this was written, so no reference binary is
 * used.  Three spots stay unpinned at bit level because the reference has no x86
 * fixture for them: exp() inside softmax/SiLU (platform libm), the plain-loop
 * dot_f16 used by attention, and the legacy f32-input matmul_q8_0 (no test of the
 * reference calls it; its two restatements are pinned on data where both orders
 * must give the exact integer result).
 *
 * Each function cites the reference file:line (paths relative to the reference
 * project root) it restates.
 */
#ifndef RMI_ORACLE_H
#define RMI_ORACLE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Which of the reference's three instruction-set variants is being restated.
 * They differ in rounding/accumulation order and are not bit-identical to each other. */
enum {
  ORC_SEM_AVX2 = 0,   /* x86_64 production path  */
  ORC_SEM_NEON = 1,   /* aarch64 production path */
  ORC_SEM_SCALAR = 2, /* portable fallback; also `--features parity-trace` quantizer */
  /* Not a variant of the reference: the x86 quantizer (src/ops/quant/q8_0.rs:176-230) followed by
   * whole-block accumulation sum = fma(f32(dot32), wd*xs, sum) (the order of neon.rs:59-70).  It
   * states what the device's tensor-core GEMM computes for an x86 host (exact int32 block sums,
   * one f32 chain per output); its f32 results are within 1e-5 of ORC_SEM_AVX2, not bit-equal.
   * Accepted by the Q8_0 quantizer, matmul and FFN entry points only. */
  ORC_SEM_AVX2_BLOCK = 3
};

/* How exp() is evaluated inside softmax / SiLU. The reference calls the platform libm.
 * ORC_EXP_LIBM: expf() of this host's libm (what the reference would do on this host).
 * ORC_EXP_CR:   (float)exp((double)x), i.e. the correctly rounded f32 exponential
 *               (up to double rounding with probability ~2^-28). Deterministic across
 *               hosts and devices; the CUDA path implements this one. */
enum { ORC_EXP_LIBM = 0, ORC_EXP_CR = 1 };

void orc_set_exp_mode(int mode);
int orc_get_exp_mode(void);
float orc_expf(float x);

/* src/ops/float.rs:177-207 (IEEE binary16 <-> binary32, round to nearest even) */
uint16_t orc_f32_to_f16(float v);
float orc_f16_to_f32(uint16_t bits);
void orc_f32_slice_to_f16(const float* src, uint16_t* dst, size_t n);
/* src/ops/quant/mod.rs:13-22 (table-free f16 decode used by the K-quant code) */
float orc_f16_from_bytes(const uint8_t* data, size_t len, size_t byte_idx);

/* src/ops/quant/q8_0.rs:3-24 (dispatch), :49-71 scalar, :176-230 AVX2, :75-165 NEON */
void orc_quantize_q8_0(const float* input, size_t n, uint8_t* q8, float* scales, int sem);

/* src/ops/kernel/q8_0/scalar.rs:31-58, avx2.rs:53-174, neon.rs:49-73.
 * output has row_end-row_start elements (dispatch.rs:27-36). */
void orc_matmul_q8_0_range(const uint8_t* weight, const uint8_t* input_q8,
                           const float* input_scales, float* output, size_t n_in,
                           size_t row_start, size_t row_end, int sem);
/* Same arithmetic through hand-written AVX2 intrinsics (4-row tile); only built on
 * x86 with AVX2+FMA+F16C. Returns 0 when unavailable. Bit-identical to
 * orc_matmul_q8_0_range(..., ORC_SEM_AVX2). Used for the timed CPU baseline. */
int orc_matmul_q8_0_range_avx2_fast(const uint8_t* weight, const uint8_t* input_q8,
                                    const float* input_scales, float* output, size_t n_in,
                                    size_t row_start, size_t row_end);
int orc_quantize_q8_0_avx2_fast(const float* input, size_t n, uint8_t* q8, float* scales);
int orc_has_avx2_fast(void);

/* src/ops/kernel/q8_0/parallel.rs:102-139: writes output[my_start..my_end] of the
 * full-length output. */
void orc_matmul_q8_0_parallel_rows(const uint8_t* weight, const uint8_t* input_q8,
                                   const float* input_scales, float* output, size_t n_in,
                                   size_t n_out, size_t ith, size_t nth, int sem);
/* Exact int32 dot of every 32-block: sums[(row-row_start)*blocks + b]. */
void orc_q8_0_block_sums(const uint8_t* weight, const uint8_t* input_q8, int32_t* sums,
                         size_t n_in, size_t row_start, size_t row_end);
/* src/ops/kernel/q8_0/scalar.rs:3-29 (f32 input, no activation quantization) */
void orc_matmul_q8_0_fallback_range(const uint8_t* weight, const float* input, float* output,
                                    size_t n_in, size_t row_start, size_t row_end);
/* src/ops/kernel/q8_0/avx2.rs:180-217 (f32 input, two 8-lane accumulators) */
void orc_matmul_q8_0_avx2_range(const uint8_t* weight, const float* input, float* output,
                                size_t n_in, size_t row_start, size_t row_end);
/* src/ops/kernel/q8_0/parallel.rs:317-341: ops::matmul_q8_0 = AVX2 kernel on x86 (ORC_SEM_AVX2), scalar elsewhere */
void orc_matmul_q8_0_f32(const uint8_t* weight, const float* input, float* output, size_t n_in, size_t n_out,
                         int sem);
/* src/ops/kernel/trait_.rs:57-109: Kernel::forward / forward_batched for Q8Kernel:
 * per token: quantize the row, then the GEMV. n_tokens rows. */
void orc_q8_forward_batched(const uint8_t* weight, const float* input, float* output,
                            size_t n_tokens, size_t n_in, size_t n_out, int sem, int threads);

/* src/ops/quant/fuse.rs:25-40: byte concatenation along rows. Returns rows, or 0 when the
 * two row strides differ (the reference returns None). out must hold a_len+b_len. */
size_t orc_fuse_vstack(const uint8_t* a, size_t a_len, size_t a_rows, const uint8_t* b,
                       size_t b_len, size_t b_rows, uint8_t* out);

/* src/ops/activation/mod.rs:137-151: up[i] *= g / (1 + exp(-g)) */
void orc_silu_mul_inplace(const float* gate, float* up, size_t n);
/* src/models/qwen3.rs:981-1046 for M tokens: quantize, gate, up, silu*mul, quantize, down.
 * x [M,n_embd] -> out [M,n_embd]. act (optional, may be NULL) receives the [M,n_ff]
 * SwiGLU activations before re-quantization. */
void orc_ffn_swiglu_q8_0(const uint8_t* w_gate, const uint8_t* w_up, const uint8_t* w_down,
                         const float* x, float* out, float* act, size_t m, size_t n_embd,
                         size_t n_ff, int sem, int threads);

/* src/ops/quant/mod.rs:36-40 */
typedef struct {
  float d;
  int8_t qs[256];
  int16_t bsums[16];
} orc_block_q8k;
/* src/ops/quant/mod.rs:82-122 (scalar), :142-200 (AVX2). sem: ORC_SEM_AVX2 or SCALAR. */
void orc_quantize_row_q8_k(const float* x, size_t n, orc_block_q8k* out, int sem);
/* src/ops/quant/mod.rs:210-289 (scalar), :701-799 (AVX2). nb super-blocks. */
float orc_vec_dot_q4k_q8k(const uint8_t* q4k, size_t q4k_len, const orc_block_q8k* q8k,
                          size_t nb, int sem);
/* exact integer parts of one super-block dot: sumi_scaled = sum_j sc_j * sum q4*q8,
 * sumi_mins = sum_j bsums_j * min_{j/2}. */
void orc_q4k_q8k_block_ints(const uint8_t* q4k_block, const orc_block_q8k* q8k,
                            int32_t* sumi_scaled, int32_t* sumi_mins);
/* src/ops/quant/mod.rs:456-490, :492-508 */
void orc_dequantize_row_q4_k(const uint8_t* bytes, size_t bytes_len, float* output, size_t n);
void orc_dequantize_q4_k_weight(const uint8_t* bytes, size_t bytes_len, size_t n_rows,
                                size_t n_cols, float* output);
/* ---- Q4_0 (18-byte blocks: f16 d | 16 nibble bytes; value l = low nibble of byte l, value 16+l = high nibble)
 * src/ops/kernel/q4_0/scalar.rs:13-53; the AVX2 kernel (q4_0/avx2.rs:25-108) is bit-identical by contract:
 * exact int32 block dot of (nibble - 8) with the Q8_0 activation, sum += (f32(dot) * d) * scale in block order. */
void orc_q4_0_forward_prequantized(const uint8_t* weight, const uint8_t* input_q8, const float* input_scales,
                                   float* output, size_t n_in, size_t n_out, size_t ith, size_t nth);

/* ---- Q6_K (210-byte super-blocks: ql[128] | qh[64] | scales i8[16] | f16 d) ----
 * src/ops/quant/mod.rs:530-569: w = (d * sc) * q, q in [-32, 31]. */
void orc_dequantize_row_q6_k(const uint8_t* bytes, size_t bytes_len, float* output, size_t n);
/* src/ops/quant/mod.rs:640-692 (scalar), :964-1064 (AVX2). nb super-blocks. */
float orc_vec_dot_q6k_q8k(const uint8_t* q6k, size_t q6k_len, const orc_block_q8k* q8k, size_t nb, int sem);
/* the eight exact int32 lane sums of one super-block as the AVX2 kernel forms them (after the -32 offset term) */
void orc_q6k_q8k_block_lanes(const uint8_t* q6k_block, const orc_block_q8k* q8k, int32_t lanes[8]);
/* src/ops/kernel/q6_k.rs:44-80 (Q8_K activation, vec_dot per row, (ith, nth) partition) */
void orc_q6k_forward_prepared(const uint8_t* weight, size_t weight_len, const float* input_f32, float* output,
                              size_t n_in, size_t n_out, size_t ith, size_t nth, int sem);
/* src/ops/kernel/q6_k.rs:83-115 (Q8_0 activation dequantized, row dequantized, sequential f32 dot) */
void orc_q6k_forward_prequantized(const uint8_t* weight, size_t weight_len, const uint8_t* input_q8,
                                  const float* input_scales, float* output, size_t n_in, size_t n_out,
                                  size_t ith, size_t nth);

/* src/core/model.rs:65-85: dequantize the whole matrix, then sequential f32 dot per row. */
void orc_q4k_forward_dequant(const uint8_t* weight, size_t weight_len, size_t out_features,
                             size_t in_features, const float* input, float* output,
                             float* scratch, size_t scratch_len);
/* src/ops/kernel/q4_k.rs:56-93 (Q8_K activation, vec_dot per row) */
void orc_q4k_forward_prepared(const uint8_t* weight, size_t weight_len, const float* input_f32,
                              float* output, size_t n_in, size_t n_out, size_t ith, size_t nth,
                              int sem);
/* src/ops/kernel/q4_k.rs:20-54 (Q8_0 activation dequantized, row dequantized, f32 dot) */
void orc_q4k_forward_prequantized(const uint8_t* weight, size_t weight_len,
                                  const uint8_t* input_q8, const float* input_scales,
                                  float* output, size_t n_in, size_t n_out, size_t ith,
                                  size_t nth);

/* src/ops/norm.rs:3-11, :13-19 */
void orc_rms_norm(const float* input, const float* weight, float* output, size_t n, float eps);
void orc_rms_norm_inplace(float* x, const float* weight, size_t n, float eps);
/* src/ops/rope.rs:21-37 */
void orc_rope_neox(float* x, size_t len, size_t pos, size_t head_dim, float freq_base);
/* The cos/sin pairs rope_neox uses at `pos`: table[2*i]=cos, table[2*i+1]=sin, i<head_dim/2 */
void orc_rope_table(size_t pos, size_t head_dim, float freq_base, float* table);
/* src/ops/attention.rs:28-38 (x86 path) */
void orc_softmax(float* x, size_t n);
/* src/ops/dot.rs:99-119 (x86 path: f64 accumulation of f32 products) */
float orc_dot_f16(const uint16_t* a, const uint16_t* b, size_t n);
/* src/ops/embedding.rs:12-22 */
void orc_embedding_lookup_q8_0(const uint8_t* weight, uint32_t token, size_t n_embd, float* out);
/* src/ops/embedding.rs:24-38: ((nibble as f32) - 8.0) * d */
void orc_embedding_lookup_q4_0(const uint8_t* weight, uint32_t token, size_t n_embd, float* out);
/* src/ops/embedding.rs:40-47: dequantize_row_q6_k of the token's row */
void orc_embedding_lookup_q6_k(const uint8_t* weight, uint32_t token, size_t n_embd, float* out);
/* src/models/qwen3.rs:172-191: first maximal index; returns -1 on empty or non-finite. */
int64_t orc_greedy_token(const float* logits, size_t n);

/* src/models/qwen3.rs:20-35, :224-236 */
typedef struct {
  size_t n_embd, n_layer, n_head, n_head_kv, head_dim, n_ff, vocab;
  float eps, freq_base;
} orc_qwen3_config;
typedef struct {
  const float* attn_norm;
  const float* ffn_norm;
  const float* q_norm;
  const float* k_norm;
  const uint8_t* wq;
  const uint8_t* wk;
  const uint8_t* wv;
  const uint8_t* wo;
  const uint8_t* w_gate;
  const uint8_t* w_up;
  const uint8_t* w_down;
} orc_qwen3_layer;
typedef struct {
  orc_qwen3_config cfg;
  const orc_qwen3_layer* layers;
  const float* output_norm;
  const uint8_t* token_embd; /* Q8_0 [vocab, n_embd] */
  const uint8_t* output;     /* Q8_0 [vocab, n_embd]; == token_embd when tied */
} orc_qwen3_model;

/* src/models/qwen3.rs:440-550 + :581-1158: greedy generation with an F16 KV cache.
 * Feeds the prompt one token at a time, then generates n_gen tokens (EOS stop disabled
 * because the synthetic vocabulary has no tokenizer). Returns the number of tokens
 * written to out_tokens, or -1 on non-finite logits.
 * trace (optional): receives the hidden state x after the last layer of every step,
 * [steps, n_embd]. logits_last (optional): logits of the final step, [vocab]. */
int64_t orc_qwen3_generate(const orc_qwen3_model* model, const uint32_t* prompt, size_t n_prompt,
                           size_t n_gen, uint32_t* out_tokens, int sem, int threads,
                           float* trace, float* logits_last);

/* The CLI's copy of the same forward (src/app/text.rs:257-648, F16 KV cache): f32 query against the f16 keys
 * (dot_f16_f32), online soft-max with a running maximum that starts at 0, vec_mad_f16_f32 / vec_scale_f32 on
 * the output row, and the last maximal index as the greedy token (:664-670).  Same arguments as above. */
int64_t orc_qwen3_generate_cli(const orc_qwen3_model* model, const uint32_t* prompt, size_t n_prompt,
                               size_t n_gen, uint32_t* out_tokens, int sem, int threads,
                               float* trace, float* logits_last);
int64_t orc_qwen3_generate_cli_f32kv(const orc_qwen3_model* model, const uint32_t* prompt, size_t n_prompt,
                                     size_t n_gen, uint32_t* out_tokens, int sem, int threads, float* trace,
                                     float* logits_last);
int64_t orc_qwen3_generate_logits_tool(const orc_qwen3_model* model, const uint32_t* prompt, size_t n_prompt,
                                       size_t n_gen, uint32_t* out_tokens, int sem, int threads, float* trace,
                                       float* logits_last, int kv_f32);
float orc_dot_f32(const float* a, const float* b, size_t n, int sem);
float orc_dot_f16_f32(const float* a, const uint16_t* b, size_t n, int sem);
void orc_vec_mad_f16_f32(float* y, const uint16_t* x, float v, size_t n, int sem);
int64_t orc_greedy_token_last(const float* logits, size_t n);

#ifdef __cplusplus
}
#endif
#endif
