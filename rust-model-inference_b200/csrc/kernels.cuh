// Launchers shared between translation units of librmi_cuda.so.
#pragma once
#include "common.cuh"

// q8_0.cu
int32_t launch_q8_repack_tile16(rmi_ctx* ctx, const uint8_t* raw, uint8_t* dst, size_t n_rows, size_t blocks);
int32_t launch_q8_copy_rows_tile16(rmi_ctx* ctx, const uint8_t* src, uint8_t* dst, size_t n_rows, size_t blocks, size_t row_off);
int32_t launch_q8_build_umma(rmi_ctx* ctx, const uint8_t* t16, uint8_t* uq, float* us, size_t n_rows, size_t blocks, size_t n_ff_perm);
int32_t launch_q8_quantize(rmi_ctx* ctx, const float* x, size_t m, size_t n, uint8_t* q8, float* scales, int out_mode);
int32_t launch_q8_gemv(rmi_ctx* ctx, const rmi_weight* w, const uint8_t* xq, const float* xs, size_t m,
                       float* out, size_t out_stride, size_t row_begin, size_t row_end);
bool q8_gemv_fused_norm_eligible(const rmi_ctx* ctx, const rmi_weight* w, size_t m);
// x = x_in (+ add); rms_norm(x, norm_w, eps); quantize; out = W x.  x is also written to x_out (!= x_in).
int32_t launch_q8_matmul_f32(rmi_ctx* ctx, const rmi_weight* w, const float* x, size_t m, float* out);
int32_t launch_q8_gemv_fused_norm(rmi_ctx* ctx, const rmi_weight* w, const float* x_in, const float* add,
                                  const float* norm_w, float eps, float* x_out, size_t m, float* out, size_t out_stride);
int32_t launch_q8_block_sums(rmi_ctx* ctx, const rmi_weight* w, const uint8_t* xq, size_t m, int32_t* sums);
int32_t launch_silu_mul_quantize(rmi_ctx* ctx, const float* gate, const float* up, size_t in_stride, size_t m,
                                 size_t n_ff, float* act, uint8_t* q8, float* scales);

// gemm_tc.cu (tcgen05 int8 MMA)
enum { GEMM_EPI_F32 = 0, GEMM_EPI_SWIGLU_Q8 = 1, GEMM_EPI_BLOCK_SUMS = 2 };
struct gemm_tc_args {
  const uint8_t* a_img;  // activations, tcgen05 A images [m_tiles][slabs][16 KiB]
  const float* a_scales; // [m_tiles][blocks][128]
  const rmi_weight* w;   // umma layout must be built
  size_t m;              // valid rows
  size_t col_begin, col_end;  // weight rows (= output columns) to compute
  int epilogue;
  float* out;            // F32: [m][out_stride]
  size_t out_stride;
  // SWIGLU_Q8: gate rows [0,n_ff), up rows [n_ff,2n_ff) of w; writes the re-quantized
  // activation as A images for the down projection plus its scales, and optionally f32 act
  size_t n_ff;
  uint8_t* act_img;
  float* act_scales;
  float* act_f32;
  int32_t* sums;         // BLOCK_SUMS: [m][n_rows][blocks]
  bool swap_ab;          // F32, all rows: weight as the 128-row operand, activation rows as tile columns
};
int32_t launch_gemm_tc(rmi_ctx* ctx, const gemm_tc_args& a);
int32_t ensure_umma_layout(rmi_ctx* ctx, const rmi_weight* w, bool gate_up_interleaved = false);

// api.cu: quantize + matmul / fused FFN on device buffers (caller holds ctx->mu); dout [m][out_stride],
// out_stride 0 = n_rows.  Uses the context's scratch slots 0..4.
int32_t matmul_q8_0_device(rmi_ctx* ctx, const rmi_weight* w, const float* dx, size_t m, float* dout,
                           size_t out_stride = 0);
int32_t ffn_device(rmi_ctx* ctx, const rmi_weight* wgu, const rmi_weight* wd, const float* dx, size_t m, float* dout);

// peer.cu: writes `epoch` into slot `rank` of every flag array, then waits (at most ctx->wait_limit_ns) until
// all `world` slots of flags[rank] reached it; on `stream`
int32_t launch_peer_push(rmi_ctx* ctx, cudaStream_t stream, const float* src, float* const* dsts, int n_peers, size_t n_rows,
                         size_t n_cols, size_t stride);
int32_t launch_peer_signal_wait(rmi_ctx* ctx, cudaStream_t stream, uint32_t* const* flags, int world, int rank,
                                uint32_t epoch);

// embedding lookups (q8_0.cu, q4_0.cu, q6k.cu): ids and out on the device
int32_t launch_q8_embedding(rmi_ctx* ctx, const rmi_weight* w, const uint32_t* ids, size_t m, float* out);
int32_t launch_q4_0_embedding(rmi_ctx* ctx, const rmi_weight* w, const uint32_t* ids, size_t m, float* out);
int32_t launch_q6k_embedding(rmi_ctx* ctx, const rmi_weight* w, const uint32_t* ids, size_t m, float* out);

// q4_0.cu
size_t q4_0_device_block_bytes();
int32_t launch_q4_0_matmul(rmi_ctx* ctx, const rmi_weight* w, const uint8_t* xq, const float* xs, size_t m, float* out,
                           size_t row_begin, size_t row_end);

// q6k.cu
size_t q6k_device_block_bytes();
int32_t launch_q6k_q8k_matmul(rmi_ctx* ctx, const rmi_weight* w, const float* d8, const int8_t* qs, const int16_t* bsums,
                              size_t m, float* out, size_t row_begin, size_t row_end);
int32_t launch_q6k_prequant_matmul(rmi_ctx* ctx, const rmi_weight* w, const uint8_t* xq, const float* xs, size_t m,
                                   float* out, size_t row_begin, size_t row_end);
int32_t launch_q6k_dequantize(rmi_ctx* ctx, const rmi_weight* w, float* out);

// q4k.cu
int32_t launch_q8k_quantize(rmi_ctx* ctx, const float* x, size_t m, size_t n, float* d, int8_t* qs, int16_t* bsums);
int32_t launch_q4k_q8k_matmul(rmi_ctx* ctx, const rmi_weight* w, const float* d8, const int8_t* qs, const int16_t* bsums,
                              size_t m, float* out, size_t row_begin, size_t row_end);
int32_t launch_q4k_dequant_matmul(rmi_ctx* ctx, const rmi_weight* w, const float* x, size_t m, float* out);
int32_t launch_q4k_dequantize(rmi_ctx* ctx, const rmi_weight* w, float* out);

// sharded.cu: 16-byte vectorised variant (falls back to the scalar kernel for unaligned shapes)
int32_t launch_unshard_cols_vec(rmi_ctx* ctx, const float* gathered, size_t g, size_t m, size_t npr, float* out);

// decode.cu
int32_t launch_unshard_cols(rmi_ctx* ctx, const float* gathered, size_t g, size_t m, size_t npr, float* out);
