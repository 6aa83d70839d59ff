/*
 * rmi_cuda.h -- C ABI of librmi_cuda.so: the quantized-matmul hot path of
 * rust-model-inference on NVIDIA B200 (sm_100a).
 *
 * Every entry point replaces (or is bound by) one interface of the reference; the
 * comment above each declaration names it as path:line inside the reference project.
 * All functions return an rmi_status (0 = ok).  After a non-zero return
 * rmi_last_error() holds a message for the calling thread.  There is no CPU fallback:
 * when no CUDA device is usable rmi_init fails and nothing else can be called.
 *
 * Pointer conventions: plain names are HOST pointers (the call copies in and out and
 * returns after the result is in the host buffer).  Entry points ending in _dev take
 * DEVICE pointers, enqueue on the context's stream and return without synchronising.
 *
 * Threading: a context may be used from several host threads; calls are serialised on
 * one stream.  The reference invokes its kernels from every pool thread with
 * (ith, nth) (src/ops/kernel/trait_.rs:15-31); here the caller passes the row range
 * [row_begin, row_end) that (ith, nth) selects, and only that range of `output` is
 * written, exactly as src/ops/kernel/q8_0/parallel.rs:124-139 does.
 */
#ifndef RMI_CUDA_H
#define RMI_CUDA_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct rmi_ctx rmi_ctx;
typedef struct rmi_weight rmi_weight;
typedef struct rmi_gguf rmi_gguf;
typedef struct rmi_qwen3 rmi_qwen3;
typedef struct rmi_session rmi_session;

typedef enum {
  RMI_OK = 0,
  RMI_ERR_BAD_HANDLE = 1,  /* null / foreign handle */
  RMI_ERR_BAD_SHAPE = 2,   /* n_in % 32 != 0 (Q8_0), % 256 != 0 (Q4_K), short buffer, bad row range */
  RMI_ERR_OOM = 3,         /* device or host allocation failed */
  RMI_ERR_CUDA = 4,        /* a CUDA call failed; message has the CUDA error string */
  RMI_ERR_TIMEOUT = 5,     /* a bounded device-side wait gave up (kernel returned cleanly) */
  RMI_ERR_UNSUPPORTED = 6, /* ggml type / semantics / size not handled by this path */
  RMI_ERR_IO = 7,          /* file open / mmap failed */
  RMI_ERR_FORMAT = 8,      /* malformed GGUF or model metadata */
  RMI_ERR_NONFINITE = 9    /* "Cannot sample non-finite logits" (src/models/qwen3.rs:172-191) */
} rmi_status;

/* ggml type ids as in src/core/tensor.rs:15-35 */
enum { RMI_GGML_F32 = 0, RMI_GGML_F16 = 1, RMI_GGML_Q4_0 = 2, RMI_GGML_Q8_0 = 8, RMI_GGML_Q4_K = 12, RMI_GGML_Q6_K = 14 };

/* The reference has three instruction-set variants of this path whose f32 results are not
 * bit-identical to each other (docs/OPTIMIZATION.md:330-332).  The device reproduces the
 * chosen one bit for bit:
 *   AVX2   src/ops/quant/q8_0.rs:176-230 + src/ops/kernel/q8_0/avx2.rs:53-174
 *   NEON   src/ops/quant/q8_0.rs:75-165  + src/ops/kernel/q8_0/neon.rs:49-73
 *   SCALAR src/ops/quant/q8_0.rs:49-71   + src/ops/kernel/q8_0/scalar.rs:31-58
 * Calls of up to 32 activation rows (decode) run memory-bound GEMV kernels and are bit-exact
 * under all three settings.  Calls of more than 32 rows (prefill) run the tcgen05 int8 GEMM:
 * one MMA per 32-block gives the exact int32 block sum, and the epilogue accumulates
 * sum = fma(f32(dot), wd*xs, sum) per block -- bit for bit the NEON order, and with a separate
 * multiply and add the SCALAR order.  The AVX2 variant accumulates eight partial sums per block
 * (avx2.rs:96-153), an order the tensor core cannot deliver.  For it the GEMM keeps the AVX2
 * quantizer (activation bytes and scale bits are those of q8_0.rs:176-230) and the exact block
 * sums, and accumulates whole blocks: each matmul's f32 output is within 1e-5 (max |a-b| /
 * max |ref|) of the eight-lane order on the same quantized input.  rmi_set_prefill_exact(ctx, 1)
 * keeps AVX2 calls of every size on the bit-exact CUDA-core kernels instead (slower).
 * Element-wise steps (rms_norm, rope, softmax, SiLU) follow the reference's portable x86 code
 * under all three settings; exp() is the correctly rounded f32 exponential. */
typedef enum { RMI_SEM_AVX2 = 0, RMI_SEM_NEON = 1, RMI_SEM_SCALAR = 2 } rmi_semantics;

/* ---- context ------------------------------------------------------------------------
 * Replaces VulkanContext::new / Drop (src/vulkan.rs:31-59, :713-725) and the lazy global
 * in src/ops/float.rs:44-58.  Init failure is an error, never a CPU fallback. */
int32_t rmi_init(int32_t device, rmi_ctx** out);
int32_t rmi_destroy(rmi_ctx* ctx);
const char* rmi_last_error(void);
int32_t rmi_set_semantics(rmi_ctx* ctx, int32_t sem);
int32_t rmi_get_semantics(rmi_ctx* ctx, int32_t* sem);
/* AVX2 semantics only (see above): on != 0 keeps calls of more than 32 rows on the CUDA-core kernels
 * that reproduce matmul_q8_0_vs_q8_0_avx2 (src/ops/kernel/q8_0/avx2.rs:53-174) bit for bit; the
 * default (0) runs them on the tensor cores. */
int32_t rmi_set_prefill_exact(rmi_ctx* ctx, int32_t on);
/* Use an existing cudaStream_t (e.g. the framework's current stream); NULL restores the
 * context's own stream. */
int32_t rmi_set_stream(rmi_ctx* ctx, void* cuda_stream);
int32_t rmi_sync(rmi_ctx* ctx);
/* on != 0: the kernels of a matmul / FFN / decode chain (activation quantizers, GEMVs, the tensor-core GEMM,
 * norm/quantize, attention, SiLU, the Q8_K quantizer and the Q4_K x Q8_K kernels) are launched with programmatic
 * stream serialization: a kernel may start while its predecessor in the stream drains, sets up its barriers and
 * tensor memory, fetches what no earlier kernel writes (its weights), and waits (griddepcontrol.wait) before it
 * touches anything else.  Results are unchanged; chains of dependent kernels run closer together (the M=512 FFN
 * step: 57.7 -> 51.7 us).  Off by default, because a weight uploaded or re-laid-out on the same stream without a
 * synchronisation in between could be fetched before it is complete; the decode session turns it on for its own
 * captured step.  The reference's counterpart is the absence of
 * a launch gap between operators inside one thread-pool dispatch (src/core/thread_pool.rs:119-161). */
int32_t rmi_set_dependent_launch(rmi_ctx* ctx, int32_t on);
/* sm count, L2 bytes, total device memory */
int32_t rmi_device_info(rmi_ctx* ctx, int32_t* sm_count, size_t* l2_bytes, size_t* mem_bytes);
/* Number of kernels this library has launched on this context (for launch accounting). */
int32_t rmi_launch_count(rmi_ctx* ctx, uint64_t* count);

/* Per-kernel device timing for benchmarks (no counterpart in the reference; its --profile
 * flag accumulates wall-clock per phase, src/app/text.rs:238-245).  While enabled, CUDA event
 * pairs are recorded around the launches tagged "q8_gemv", "gemm_tc" and "gemm_tc_swiglu";
 * rmi_prof_read sums them.  Enabling resets the records.  Not for use inside graph capture. */
int32_t rmi_prof_enable(rmi_ctx* ctx, int32_t on);
int32_t rmi_prof_read(rmi_ctx* ctx, const char* tag, uint64_t* launches, float* total_ms);

/* Device buffers for callers that have no CUDA allocator of their own. */
int32_t rmi_dev_alloc(rmi_ctx* ctx, size_t bytes, void** dev_ptr);
int32_t rmi_dev_free(rmi_ctx* ctx, void* dev_ptr);
int32_t rmi_h2d(rmi_ctx* ctx, void* dst_dev, const void* src_host, size_t bytes);
int32_t rmi_d2h(rmi_ctx* ctx, void* dst_host, const void* src_dev, size_t bytes);
int32_t rmi_host_alloc_pinned(rmi_ctx* ctx, size_t bytes, void** host_ptr);
int32_t rmi_host_free_pinned(rmi_ctx* ctx, void* host_ptr);

/* ---- weights ------------------------------------------------------------------------
 * Replaces QuantizedTensor::from_bytes + into_kernel (src/ops/kernel/quantized_tensor.rs:
 * 120-189): called once per tensor at load with the raw GGUF bytes (row-major blocks,
 * row length n_in, n_out rows).  Rows [row_begin, row_end) are uploaded -- the
 * PlacementSlice::Rows of src/format/load_plan.rs:19-22 -- and re-laid out for the device
 * (16-row interleaved blocks: 32 B of f16 scales then 16 x 32 B of quants).  The host bytes are not
 * referenced after the call returns. */
int32_t rmi_weight_upload(rmi_ctx* ctx, int32_t ggml_type, const void* bytes, size_t nbytes,
                          size_t n_in, size_t n_out, size_t row_begin, size_t row_end,
                          rmi_weight** out);
int32_t rmi_weight_free(rmi_ctx* ctx, rmi_weight* w);
int32_t rmi_weight_info(const rmi_weight* w, int32_t* ggml_type, size_t* n_in, size_t* n_rows,
                        size_t* device_bytes);
/* fuse_vstack_q8_0 / fuse_vstack_q4_k (src/ops/quant/fuse.rs:25-63) and
 * QTensorOwned::fuse_vstack (src/ops/kernel/qtensor_owned.rs:138-164): rows of a, then rows
 * of b.  RMI_ERR_BAD_SHAPE when the row lengths differ (the reference returns None). */
int32_t rmi_weight_fuse_vstack(rmi_ctx* ctx, const rmi_weight* a, const rmi_weight* b,
                               rmi_weight** out);

/* ---- Q8_0 activation quantizer --------------------------------------------------------
 * quantize_q8_0_into (src/ops/quant/q8_0.rs:3-24), row-wise for m rows of length n:
 * q8[m*n] int8 as u8, scales[m*n/32] = f32(f16(amax/127)). */
int32_t rmi_quantize_q8_0(rmi_ctx* ctx, const float* x, size_t m, size_t n, uint8_t* q8,
                          float* scales);
int32_t rmi_quantize_q8_0_dev(rmi_ctx* ctx, const float* x, size_t m, size_t n, uint8_t* q8,
                              float* scales);

/* ---- Q8_0 matmul ------------------------------------------------------------------------
 * Kernel::forward_prequantized (src/ops/kernel/trait_.rs:19-29) ==
 * matmul_q8_0_quantized_parallel_rows (src/ops/kernel/q8_0/parallel.rs:102-139) and the
 * GPU hook ctx.matmul_q8_0 (src/vulkan.rs:347-355), for m activation rows:
 *   output[t*n_rows + r] for r in [row_begin,row_end) ; other elements are not touched. */
int32_t rmi_matmul_q8_0_prequantized(rmi_ctx* ctx, const rmi_weight* w, const uint8_t* q8,
                                     const float* scales, size_t m, float* output,
                                     size_t row_begin, size_t row_end);
int32_t rmi_matmul_q8_0_prequantized_dev(rmi_ctx* ctx, const rmi_weight* w, const uint8_t* q8,
                                         const float* scales, size_t m, float* output,
                                         size_t row_begin, size_t row_end);
/* Kernel::forward / forward_batched (src/ops/kernel/trait_.rs:57-109): per row quantize,
 * then the matmul.  m <= 32 runs the memory-bound GEMV kernels (NEON / SCALAR: swapped-operand GEMM
 * from 9 rows), m > 32 the tcgen05 GEMM. */
int32_t rmi_matmul_q8_0(rmi_ctx* ctx, const rmi_weight* w, const float* x, size_t m, float* output);
/* ops::matmul_q8_0, the legacy f32-input matmul (src/ops/kernel/q8_0/parallel.rs:317-341): the dequantized
 * weight times the f32 activation, no activation quantization.  RMI_SEM_AVX2 reproduces matmul_q8_0_avx2_range
 * (avx2.rs:180-217: two 8-lane accumulators, fma(d * f32(q), x, acc), hsum_ps); the other semantics reproduce
 * matmul_q8_0_fallback_range (scalar.rs:3-29), which is what the reference runs off x86.  output[t*n_rows + r],
 * m <= 65535 rows of x per call; _dev takes device pointers and returns before the kernel finishes. */
int32_t rmi_matmul_q8_0_f32(rmi_ctx* ctx, const rmi_weight* w, const float* x, size_t m, float* output);
int32_t rmi_matmul_q8_0_f32_dev(rmi_ctx* ctx, const rmi_weight* w, const float* x, size_t m, float* output);
int32_t rmi_matmul_q8_0_dev(rmi_ctx* ctx, const rmi_weight* w, const float* x, size_t m,
                            float* output);
/* No counterpart in the reference.  Same result as rmi_matmul_q8_0_dev for m <= 32, but the call
 * allocates nothing: the quantized activations live in a 576 KiB array compiled into the library
 * (held by every GPU that loads it) instead of context scratch obtained with cudaMalloc.  It is
 * meant for hosts whose own allocator already owns all device memory, or whose loops cannot take
 * the device-wide synchronisation of cudaMalloc/cudaFree.  Limits: m <= 32 and m * n_in <= 524288
 * (RMI_ERR_BAD_SHAPE beyond that); per-kernel timing must be off.  The first call on a device
 * resolves the array's address, so issue it before any stream capture begins.  All calls on a
 * device share the array: calls that overlap on the GPU race, the caller orders them. */
int32_t rmi_matmul_q8_0_dev_noalloc(rmi_ctx* ctx, const rmi_weight* w, const float* x, size_t m,
                                    float* output);
/* Exact int32 dot of every 32-block, sums[(t*n_rows + r)*(n_in/32) + b]; debug/parity aid
 * with no counterpart in the reference API (it is the integer part of
 * src/ops/kernel/q8_0/scalar.rs:49-55).  use_tensor_cores != 0 routes through the
 * tcgen05 int8 MMA path (m is padded to the tile internally). */
int32_t rmi_q8_0_block_sums(rmi_ctx* ctx, const rmi_weight* w, const uint8_t* q8, size_t m,
                            int32_t* sums, int32_t use_tensor_cores);

/* ---- fused SwiGLU FFN -------------------------------------------------------------------
 * src/models/qwen3.rs:981-1046 for m tokens: quantize x, gate and up projections (one
 * pass over the v-stacked weight), up * silu(gate), re-quantize, down projection.
 * w_gate_up must come from rmi_weight_fuse_vstack(gate, up).  x [m,n_embd] -> out [m,n_embd]. */
int32_t rmi_ffn_swiglu_q8_0(rmi_ctx* ctx, const rmi_weight* w_gate_up, const rmi_weight* w_down,
                            const float* x, size_t m, float* out);
int32_t rmi_ffn_swiglu_q8_0_dev(rmi_ctx* ctx, const rmi_weight* w_gate_up,
                                const rmi_weight* w_down, const float* x, size_t m, float* out);
/* A run of n_batches FFN calls (batch i: weights wgu[i]/wd[i], host input x[i] [m, n_embd], host
 * output out[i] [m, n_embd]; all batches the same m and widths) with the host<->device copies of
 * neighbouring batches overlapped with the arithmetic on three streams.  Results are those of
 * n_batches calls of rmi_ffn_swiglu_q8_0.  Pinned host buffers are needed for the overlap;
 * pageable ones still give correct results.  No counterpart in the reference, whose FFN works
 * in host memory (src/models/qwen3.rs:968-1052). */
int32_t rmi_ffn_swiglu_q8_0_pipelined(rmi_ctx* ctx, const rmi_weight* const* w_gate_up,
                                      const rmi_weight* const* w_down, const float* const* x,
                                      float* const* out, size_t n_batches, size_t m);
/* silu_mul_inplace (src/ops/activation/mod.rs:137-151): up[i] *= gate[i]/(1+exp(-gate[i])) */
int32_t rmi_silu_mul(rmi_ctx* ctx, const float* gate, float* up, size_t n);

/* ---- Q4_K -------------------------------------------------------------------------------
 * BlockQ8K (src/ops/quant/mod.rs:36-40) as three arrays: d[nb], qs[nb*256], bsums[nb*16].
 * quantize_row_q8_k_into (src/ops/quant/mod.rs:52-61). */
int32_t rmi_quantize_q8_k(rmi_ctx* ctx, const float* x, size_t m, size_t n, float* d, int8_t* qs,
                          int16_t* bsums);
/* Q4_KKernel::forward_prepared (src/ops/kernel/q4_k.rs:56-93): Q8_K activation, then
 * vec_dot_q4k_q8k per row (src/ops/quant/mod.rs:202-289, :701-799). */
int32_t rmi_matmul_q4_k_q8k(rmi_ctx* ctx, const rmi_weight* w, const float* x, size_t m,
                            float* output, size_t row_begin, size_t row_end);
/* QuantizedLinear::forward_dequant / Layer::forward (src/core/model.rs:65-93): dequantized
 * f32 weights times the f32 input.  No 64 MiB scratch: weights are decoded in registers. */
/* Device-pointer variant of rmi_matmul_q4_k_q8k over all rows: x [m, n_in] f32 and output [m, n_rows] f32 on the
 * device; quantizes to Q8_K and multiplies, stream-ordered, no synchronisation. */
int32_t rmi_matmul_q4_k_q8k_dev(rmi_ctx* ctx, const rmi_weight* w, const float* x, size_t m,
                                float* output);
int32_t rmi_matmul_q4_k_dequant(rmi_ctx* ctx, const rmi_weight* w, const float* x, size_t m,
                                float* output);
int32_t rmi_matmul_q4_k_dequant_dev(rmi_ctx* ctx, const rmi_weight* w, const float* x, size_t m,
                                    float* output);
/* dequantize_q4_k_weight (src/ops/quant/mod.rs:492-508) */
int32_t rmi_dequantize_q4_k(rmi_ctx* ctx, const rmi_weight* w, float* output);

/* ---- Q4_0 (rmi_weight_upload with ggml type 2; 18-byte blocks) -------------------------------
 * Q4_0Kernel::forward_prequantized (src/ops/kernel/q4_0/mod.rs:29-80, scalar.rs:13-53; the AVX2 kernel is
 * bit-identical by contract): exact block dots with the Q8_0 activation (q8 [m, n_in], scales [m, n_in/32]),
 * sum += (f32(dot) * d) * scale in block order; rows [row_begin, row_end) of output [m, n_rows].  Bit-exact. */
int32_t rmi_matmul_q4_0_prequantized(rmi_ctx* ctx, const rmi_weight* w, const uint8_t* q8,
                                     const float* scales, size_t m, float* output,
                                     size_t row_begin, size_t row_end);
/* Kernel::forward for Q4_0 (src/ops/kernel/trait_.rs:57-76): quantize x to Q8_0 with the context's
 * semantics, then the call above over all rows. */
int32_t rmi_matmul_q4_0(rmi_ctx* ctx, const rmi_weight* w, const float* x, size_t m, float* output);

/* ---- Q6_K (rmi_weight_upload with ggml type 14; 210-byte super-blocks) ------------------------
 * Q6_KKernel::forward_prepared (src/ops/kernel/q6_k.rs:44-80): Q8_K-quantize every row of x, then
 * vec_dot_q6k_q8k per weight row (src/ops/quant/mod.rs:640-692 scalar, :964-1064 AVX2), rows
 * [row_begin, row_end) of output [m, n_rows].  Bit-exact under AVX2 and SCALAR semantics. */
int32_t rmi_matmul_q6_k_q8k(rmi_ctx* ctx, const rmi_weight* w, const float* x, size_t m,
                            float* output, size_t row_begin, size_t row_end);
/* Q6_KKernel::forward_prequantized = matmul_q6_k_scalar_range (src/ops/kernel/q6_k.rs:83-115): the
 * Q8_0 activation (q8 [m, n_in], scales [m, n_in/32]) dequantized, times the dequantized row
 * (src/ops/quant/mod.rs:530-569); f32 within 1e-4 of the reference's sequential sum. */
int32_t rmi_matmul_q6_k_prequantized(rmi_ctx* ctx, const rmi_weight* w, const uint8_t* q8,
                                     const float* scales, size_t m, float* output,
                                     size_t row_begin, size_t row_end);
/* dequant_q6k_weight (src/ops/quant/mod.rs:571-583): all rows to f32 [n_rows, n_in], bit-exact. */
int32_t rmi_dequantize_q6_k(rmi_ctx* ctx, const rmi_weight* w, float* output);

/* ---- embedding lookup --------------------------------------------------------------------
 * embedding_lookup (src/ops/embedding.rs:3-47) for a Q8_0, Q4_0 or Q6_K table uploaded with
 * rmi_weight_upload: rows token_ids[0..m) dequantized to output [m, n_in], bit-exact.  Ids outside the
 * table are rejected (RMI_ERR_BAD_SHAPE) instead of panicking on the slice as the reference does. */
int32_t rmi_embedding_lookup(rmi_ctx* ctx, const rmi_weight* w, const uint32_t* token_ids, size_t m,
                             float* output);

/* ---- GGUF -------------------------------------------------------------------------------
 * GGUFLoader::from_file / tensor_info / tensor_slice / metadata (src/core/loader.rs:211-395):
 * mmap + header, KV and tensor-table parse with the same range checks. */
int32_t rmi_gguf_open(const char* path, rmi_gguf** out);
int32_t rmi_gguf_close(rmi_gguf* g);
int32_t rmi_gguf_n_tensors(const rmi_gguf* g, size_t* n);
int32_t rmi_gguf_tensor(const rmi_gguf* g, const char* name, int32_t* ggml_type, uint64_t dims[4],
                        int32_t* n_dims, const void** data, size_t* nbytes);
int32_t rmi_gguf_meta_u64(const rmi_gguf* g, const char* key, uint64_t* value);
int32_t rmi_gguf_meta_f64(const rmi_gguf* g, const char* key, double* value);
int32_t rmi_gguf_meta_str(const rmi_gguf* g, const char* key, char* buf, size_t buf_len);
/* tensor_slice -> device layout in one step ("GGUF mmap weight upload") */
int32_t rmi_weight_upload_gguf(rmi_ctx* ctx, const rmi_gguf* g, const char* name,
                               size_t row_begin, size_t row_end, rmi_weight** out);

/* ---- Qwen3 decode -----------------------------------------------------------------------
 * Qwen3Model::from_source (src/models/qwen3.rs:246-400): checks dims/types per tensor and
 * uploads every weight once. */
int32_t rmi_qwen3_load(rmi_ctx* ctx, const char* gguf_path, rmi_qwen3** out);
int32_t rmi_qwen3_free(rmi_ctx* ctx, rmi_qwen3* model);
int32_t rmi_qwen3_config(const rmi_qwen3* model, size_t* n_embd, size_t* n_layer, size_t* n_head,
                         size_t* n_head_kv, size_t* head_dim, size_t* n_ff, size_t* vocab);
/* Qwen3Session::new (src/models/qwen3.rs:440-550) for `batch` independent sequences:
 * F16 KV cache [batch][n_layer][capacity][n_head_kv*head_dim] x2 in HBM plus all scratch.  Any
 * capacity in 1..=n_ctx is accepted, as in the reference (:442-447): up to a few thousand positions the
 * attention kernels keep their score rows in shared memory, beyond that the same arithmetic runs with
 * the rows in a global scratch area (6 bytes per head and position). */
int32_t rmi_session_create(rmi_ctx* ctx, const rmi_qwen3* model, size_t batch, size_t capacity,
                           rmi_session** out);
int32_t rmi_session_free(rmi_ctx* ctx, rmi_session* s);
/* Which of the reference's copies of the Qwen3 forward the session reproduces:
 * RMI_FORWARD_QWEN3_SESSION (default) = Qwen3Session::generate_inner (src/models/qwen3.rs:581-1158): f16 query,
 *   scores buffer + softmax, first maximal index as the greedy token;
 * RMI_FORWARD_APP_TEXT = the CLI's loop (src/app/text.rs:257-648): f32 query against the f16 keys
 *   (dot_f16_f32), online soft-max with a running maximum starting at 0, vec_mad_f16_f32 / vec_scale_f32 on
 *   the output row, and the last maximal index as the greedy token (:664-670);
 * RMI_FORWARD_APP_TEXT_F32KV = the same loop with `--kv-cache f32` (src/app/text.rs:183-186, :393-405, :458-496):
 *   K and V kept in f32, scores by dot_f32, soft-max over the scores padded to a multiple of 256, one dot_f32
 *   over the positions per output element.  The F32 caches are allocated by this call on first use; sessions
 *   longer than 512 positions are rejected (RMI_ERR_BAD_SHAPE; the reference's 512-entry value array panics).
 * RMI_FORWARD_APP_LOGITS / RMI_FORWARD_APP_LOGITS_F32KV = the logits tool's loop (src/app/logits.rs:474-560) over the
 *   F16 / F32 cache: scores by dot_f16_f32 / dot_f32, soft-max over the cached positions, then one sequential
 *   chain per output element (val += p_t * v_t, separate multiply and add), first maximal index as the
 *   reported token (:766-773); no 512-position limit.
 * The server's loop (src/bin/server.rs:595-641) is the F16 branch of the text loop statement for statement
 * (RMI_FORWARD_APP_TEXT). */
enum {
  RMI_FORWARD_QWEN3_SESSION = 0,
  RMI_FORWARD_APP_TEXT = 1,
  RMI_FORWARD_APP_TEXT_F32KV = 2,
  RMI_FORWARD_APP_LOGITS = 3,
  RMI_FORWARD_APP_LOGITS_F32KV = 4
};
int32_t rmi_session_set_forward(rmi_ctx* ctx, rmi_session* s, int32_t forward);
/* How the prompt positions before the last one are processed (their logits are never read):
 *   RMI_PREFILL_BATCHED (default)  all positions of a sequence as rows through every operator of a layer
 *     (matmuls with M = positions, causal attention per position over the cache rows written on the way).
 *     Every operator of the reference's step works on one row and positions only meet in the K/V cache, so
 *     every cache row carries the bits of the reference's token loop (src/models/qwen3.rs:657-689): under
 *     NEON/SCALAR semantics the matmuls run on the tensor cores, under AVX2 on the bit-exact CUDA-core
 *     kernels.  Used for the default forward and prompts of 17 positions or more; otherwise the token loop.
 *   RMI_PREFILL_TOKEN_LOOP         one position per step, as the reference does.
 *   RMI_PREFILL_BATCHED_TENSOR     as BATCHED, but AVX2 semantics also take the tensor cores: cache rows are
 *     then within the 1e-5 matmul contract of the eight-lane order instead of bit-equal to it. */
enum { RMI_PREFILL_BATCHED = 0, RMI_PREFILL_TOKEN_LOOP = 1, RMI_PREFILL_BATCHED_TENSOR = 2 };
int32_t rmi_session_set_prefill(rmi_ctx* ctx, rmi_session* s, int32_t mode);
/* Qwen3Session::generate greedy path (src/models/qwen3.rs:581-1158): processes the prompts (see
 * rmi_session_set_prefill), then generates n_gen tokens per sequence; the whole step runs on the
 * device.  prompts [batch, n_prompt] u32, out_tokens [batch, n_gen] u32.  EOS handling is
 * the caller's (there is no tokenizer here).  gen_ms (optional) receives the device time of
 * the n_gen generation steps, prefill_ms that of the prompt steps. */
int32_t rmi_session_generate(rmi_ctx* ctx, rmi_session* s, const uint32_t* prompts,
                             size_t n_prompt, size_t n_gen, uint32_t* out_tokens, float* prefill_ms,
                             float* gen_ms);
/* The same step for hosts that sample themselves -- one iteration of the loop in Qwen3Session::generate_inner
 * (src/models/qwen3.rs:657-1158; the reference hands the logits to its sampler, src/ops/sampler.rs) per call:
 *   rmi_session_reset     position 0 (required before the calls below, and after rmi_session_generate)
 *   rmi_session_prefill   tokens [batch, n_tokens] for positions 0..n_tokens-1 whose logits nobody needs (a
 *                         prompt without its last token); batched or token loop per rmi_session_set_prefill
 *   rmi_session_step      tokens [batch] at the current position; returns the greedy choice per sequence
 *                         (next_tokens [batch], may be NULL) and, if logits_opt is not NULL, the logits
 *                         [batch, vocab] for the host's own sampler.  Synchronous.  RMI_ERR_NONFINITE as in
 *                         the reference ("Cannot sample non-finite logits").
 *   rmi_session_position  the next position to be computed
 * All pointers are host pointers. */
int32_t rmi_session_reset(rmi_ctx* ctx, rmi_session* s);
int32_t rmi_session_prefill(rmi_ctx* ctx, rmi_session* s, const uint32_t* tokens, size_t n_tokens);
int32_t rmi_session_step(rmi_ctx* ctx, rmi_session* s, const uint32_t* tokens, uint32_t* next_tokens,
                         float* logits_opt);
int32_t rmi_session_position(const rmi_session* s, size_t* position);
/* Debug/parity reads after a generate call: hidden state of the last step [batch, n_embd]
 * and logits of the last step [batch, vocab]. */
int32_t rmi_session_read_hidden(rmi_ctx* ctx, rmi_session* s, float* hidden);
int32_t rmi_session_read_logits(rmi_ctx* ctx, rmi_session* s, float* logits);

/* ---- column-sharded matmul --------------------------------------------------------------
 * New for multi-GPU (the reference only plans row splits: src/format/load_plan.rs:208-330).
 * After each rank computed y_r [m, n/g] and an all-gather produced gathered [g, m, n/g],
 * this restores row-major [m, n] on the device. */
int32_t rmi_unshard_cols_dev(rmi_ctx* ctx, const float* gathered, size_t g, size_t m,
                             size_t n_per_rank, float* out);

/* Fused alternative to all-gather + un-shard (no counterpart in the reference; it realises the
 * same Rows placement, src/format/load_plan.rs:19-22): the matmul stores every f32 result into
 * each of `n_outs` (1..8) buffers of identical layout [m][out_stride], at columns
 * [col_offset, col_offset + n_rows of w).  outs[0] is normally this rank's own final buffer and
 * the others are peers' buffers mapped with rmi_ipc_open, so each rank writes its column slice
 * straight into every rank's [m, n] result over NVLink (plain stores, no multicast).  Device
 * pointers; returns after enqueueing. */
int32_t rmi_matmul_q8_0_fanout_dev(rmi_ctx* ctx, const rmi_weight* w, const float* x, size_t m,
                                   float* const* outs, int32_t n_outs, size_t out_stride,
                                   size_t col_offset);
/* CUDA IPC for buffers from rmi_dev_alloc (one process per GPU, same node): a 64-byte handle
 * to send to the peers, and the peer's mapping of it (peer access is enabled on open). */
int32_t rmi_ipc_export(rmi_ctx* ctx, const void* dev_ptr, uint8_t* handle64);
int32_t rmi_ipc_open(rmi_ctx* ctx, const uint8_t* handle64, void** out_ptr);
int32_t rmi_ipc_close(rmi_ctx* ctx, void* ptr);
/* Closes one exchange round.  flags[p] is rank p's flag array (`world` uint32, zero-initialised;
 * flags[rank] is this rank's own, the others are IPC mappings).  Enqueues a kernel that writes
 * `epoch` into slot `rank` of every array after all earlier stores of this stream, then waits
 * until all slots of its own array reached `epoch`.  Epochs must increase by one per round.
 * The wait gives up after the context's wait limit (two seconds unless rmi_set_wait_limit_ms changed
 * it) and records RMI_ERR_TIMEOUT in the context's device status, which rmi_check_status reports.
 * Every rank must run on its own GPU. */
int32_t rmi_peer_signal_wait_dev(rmi_ctx* ctx, uint32_t* const* flags, int32_t world, int32_t rank,
                                 uint32_t epoch);
/* Synchronises the stream and returns RMI_ERR_TIMEOUT if a device-side wait gave up since the
 * last check (the `_dev` entry points return before their kernels finish). */
int32_t rmi_check_status(rmi_ctx* ctx);
/* Time limit of every bounded device-side wait of this context (flag rounds between ranks, the GEMM's
 * barrier waits): 1..60000 ms, default 2000.  The reference's only wait of this kind, the thread pool's
 * spin barrier (src/core/thread_pool.rs:136-157), has no limit. */
int32_t rmi_set_wait_limit_ms(rmi_ctx* ctx, uint32_t ms);

/* ---- row-sharded matmul with its exchange (one context per GPU, ranks on one node) ----------------
 * The multi-GPU form of matmul_q8_0_quantized_parallel_rows (src/ops/kernel/q8_0/parallel.rs:102-139):
 * rank r of `world` holds weight rows [r*n_out/world, (r+1)*n_out/world) (rmi_weight_upload with that
 * row range, the PlacementSlice::Rows of src/format/load_plan.rs:19-22), x is replicated, and every
 * rank ends up with the whole row-major y [m, n_out] in its own result buffer.
 *   rmi_shard_group_create   allocates this rank's two result buffers [m_max, n_out] (they alternate
 *                            by round) and its flag array
 *   rmi_shard_group_export   192 bytes of CUDA IPC handles to send to every other rank
 *   rmi_shard_group_connect  all ranks' handles, 192 bytes each, ordered by rank (the own entry is
 *                            ignored); maps the peers' buffers.  All ranks must have connected before
 *                            the first matmul (a host-side barrier).
 *   rmi_matmul_q8_0_sharded_dev  x [m, n_in] on the device; enqueues the shard's matmul and the exchange
 *                            and returns this round's result buffer, complete once the enqueued work
 *                            has run.  RMI_EXCHANGE_FUSED_STORES: the matmul's epilogue stores its
 *                            columns into every rank's buffer over NVLink (best for small m);
 *                            RMI_EXCHANGE_PEER_COPY: m is cut into slabs of rows and the copy engines
 *                            push slab i to the peers while slab i+1 is computed (best for large m).
 *                            RMI_EXCHANGE_PEER_PUSH: the same slabs, pushed by a small kernel with plain
 *                            peer stores (a third of the SMs, all peers at once) instead of the copy engines.
 *                            All ranks must make the same sequence of calls.  Reads of round k's
 *                            result must be enqueued on the context's stream before round k+1 is
 *                            called; the buffer is then safe until round k+2 is called.  A rank that
 *                            does not show up makes the others' flag wait run out:
 *                            rmi_check_status reports RMI_ERR_TIMEOUT.
 *   rmi_shard_group_free     after a host-side barrier (no peer may still be writing). */
typedef struct rmi_shard_group rmi_shard_group;
enum { RMI_EXCHANGE_FUSED_STORES = 0, RMI_EXCHANGE_PEER_COPY = 1, RMI_EXCHANGE_PEER_PUSH = 2 };
int32_t rmi_shard_group_create(rmi_ctx* ctx, int32_t world, int32_t rank, size_t n_out, size_t m_max,
                               rmi_shard_group** out);
int32_t rmi_shard_group_export(rmi_ctx* ctx, const rmi_shard_group* g, uint8_t* handles192);
int32_t rmi_shard_group_connect(rmi_ctx* ctx, rmi_shard_group* g, const uint8_t* all_handles);
int32_t rmi_shard_group_epoch(const rmi_shard_group* g, uint32_t* epoch);
int32_t rmi_matmul_q8_0_sharded_dev(rmi_ctx* ctx, rmi_shard_group* g, const rmi_weight* w_shard, const float* x,
                                    size_t m, int32_t exchange, float** result);
int32_t rmi_shard_group_free(rmi_ctx* ctx, rmi_shard_group* g);

/* The NCCL form of the same exchange: all-gather of every rank's y_local [m, n_per_rank] (device) with the
 * caller's communicator (an ncclComm_t), then the un-shard into out [m, world * n_per_rank], enqueued on
 * the context's stream.  `gathered` is a device staging buffer of world*m*n_per_rank floats (may be null
 * for m == 1, where the shards are already contiguous pieces of the result).  NCCL is resolved at run
 * time from the libnccl.so.2 the process has loaded.  No counterpart in the reference (its devices are
 * planned, src/format/load_plan.rs:208-330, never executed). */
int32_t rmi_allgather_cols_dev(rmi_ctx* ctx, void* nccl_comm, const float* y_local, size_t m, size_t n_per_rank,
                               int32_t world, float* gathered, float* out);
/* For hosts without a communicator of their own: rank 0 obtains a 128-byte id (ncclGetUniqueId), sends it
 * to the other ranks by any means, and every rank creates its communicator (ncclCommInitRank on the
 * context's device). */
int32_t rmi_nccl_unique_id(uint8_t* id128);
int32_t rmi_nccl_comm_create(rmi_ctx* ctx, const uint8_t* id128, int32_t world, int32_t rank, void** comm);
int32_t rmi_nccl_comm_destroy(void* comm);

#ifdef __cplusplus
}
#endif
#endif
