// Host- and device-pointer entry points of the Q4_K paths.
#include "common.cuh"
#include "kernels.cuh"

extern "C" int32_t rmi_quantize_q8_k(rmi_ctx* ctx, const float* x, size_t m, size_t n, float* d, int8_t* qs,
                                     int16_t* bsums) {
  RMI_TRY(rmi_check_ctx(ctx));
  RMI_REQUIRE(n % 256 == 0, RMI_ERR_BAD_SHAPE, "n=%zu is not a multiple of 256", n);
  if (m * n == 0) return RMI_OK;
  RMI_REQUIRE(x && d && qs && bsums, RMI_ERR_BAD_HANDLE, "rmi_quantize_q8_k: null buffer");
  RMI_REQUIRE(ctx->sem != RMI_SEM_NEON, RMI_ERR_UNSUPPORTED, "the reference has no NEON Q8_K quantizer; use AVX2 or SCALAR");
  std::lock_guard<std::mutex> lock(ctx->mu);
  const size_t nb = m * n / 256;
  float *dx, *dd;
  int8_t* dq;
  int16_t* db;
  RMI_TRY(rmi_scratch(ctx, 5, m * n * 4, (void**)&dx));
  RMI_TRY(rmi_scratch(ctx, 0, m * n, (void**)&dq));
  RMI_TRY(rmi_scratch(ctx, 1, nb * 4, (void**)&dd));
  RMI_TRY(rmi_scratch(ctx, 4, nb * 32, (void**)&db));
  RMI_CUDA_CHECK(cudaMemcpyAsync(dx, x, m * n * 4, cudaMemcpyHostToDevice, ctx->stream));
  RMI_TRY(launch_q8k_quantize(ctx, dx, m, n, dd, dq, db));
  RMI_CUDA_CHECK(cudaMemcpyAsync(d, dd, nb * 4, cudaMemcpyDeviceToHost, ctx->stream));
  RMI_CUDA_CHECK(cudaMemcpyAsync(qs, dq, m * n, cudaMemcpyDeviceToHost, ctx->stream));
  RMI_CUDA_CHECK(cudaMemcpyAsync(bsums, db, nb * 32, cudaMemcpyDeviceToHost, ctx->stream));
  RMI_CUDA_CHECK(cudaStreamSynchronize(ctx->stream));
  return RMI_OK;
}

extern "C" int32_t rmi_matmul_q4_k_q8k(rmi_ctx* ctx, const rmi_weight* w, const float* x, size_t m, float* output,
                                       size_t row_begin, size_t row_end) {
  RMI_TRY(rmi_check_ctx(ctx));
  RMI_TRY(rmi_check_weight(w, RMI_GGML_Q4_K));
  RMI_REQUIRE(row_begin <= row_end && row_end <= w->n_rows, RMI_ERR_BAD_SHAPE, "row range [%zu,%zu) outside [0,%zu)",
              row_begin, row_end, w->n_rows);
  if (m == 0 || row_begin == row_end) return RMI_OK;
  RMI_REQUIRE(x && output, RMI_ERR_BAD_HANDLE, "rmi_matmul_q4_k_q8k: null buffer");
  RMI_REQUIRE(ctx->sem != RMI_SEM_NEON, RMI_ERR_UNSUPPORTED, "the reference has no NEON Q4_K x Q8_K kernel; use AVX2 or SCALAR");
  std::lock_guard<std::mutex> lock(ctx->mu);
  const size_t n = w->n_in, nb = m * n / 256, nr = row_end - row_begin;
  float *dx, *dd, *dout;
  int8_t* dq;
  int16_t* db;
  RMI_TRY(rmi_scratch(ctx, 5, m * n * 4, (void**)&dx));
  RMI_TRY(rmi_scratch(ctx, 0, m * n, (void**)&dq));
  RMI_TRY(rmi_scratch(ctx, 1, nb * 4, (void**)&dd));
  RMI_TRY(rmi_scratch(ctx, 4, nb * 32, (void**)&db));
  RMI_TRY(rmi_scratch(ctx, 6, m * w->n_rows * 4, (void**)&dout));
  RMI_CUDA_CHECK(cudaMemcpyAsync(dx, x, m * n * 4, cudaMemcpyHostToDevice, ctx->stream));
  RMI_TRY(launch_q8k_quantize(ctx, dx, m, n, dd, dq, db));
  RMI_TRY(launch_q4k_q8k_matmul(ctx, w, dd, dq, db, m, dout, row_begin, row_end));
  RMI_CUDA_CHECK(cudaMemcpy2DAsync(output + row_begin, w->n_rows * 4, dout + row_begin, w->n_rows * 4, nr * 4, m,
                                   cudaMemcpyDeviceToHost, ctx->stream));
  RMI_CUDA_CHECK(cudaStreamSynchronize(ctx->stream));
  return RMI_OK;
}

extern "C" int32_t rmi_matmul_q4_k_q8k_dev(rmi_ctx* ctx, const rmi_weight* w, const float* x, size_t m, float* output) {
  RMI_TRY(rmi_check_ctx(ctx));
  RMI_TRY(rmi_check_weight(w, RMI_GGML_Q4_K));
  if (m == 0 || w->n_rows == 0) return RMI_OK;
  RMI_REQUIRE(x && output, RMI_ERR_BAD_HANDLE, "rmi_matmul_q4_k_q8k_dev: null buffer");
  RMI_REQUIRE(ctx->sem != RMI_SEM_NEON, RMI_ERR_UNSUPPORTED, "the reference has no NEON Q4_K x Q8_K kernel; use AVX2 or SCALAR");
  std::lock_guard<std::mutex> lock(ctx->mu);
  const size_t n = w->n_in, nb = m * n / 256;
  float* dd;
  int8_t* dq;
  int16_t* db;
  RMI_TRY(rmi_scratch(ctx, 0, m * n, (void**)&dq));
  RMI_TRY(rmi_scratch(ctx, 1, nb * 4, (void**)&dd));
  RMI_TRY(rmi_scratch(ctx, 4, nb * 32, (void**)&db));
  RMI_TRY(launch_q8k_quantize(ctx, x, m, n, dd, dq, db));
  return launch_q4k_q8k_matmul(ctx, w, dd, dq, db, m, output, 0, w->n_rows);
}

extern "C" int32_t rmi_matmul_q4_k_dequant_dev(rmi_ctx* ctx, const rmi_weight* w, const float* x, size_t m,
                                               float* output) {
  RMI_TRY(rmi_check_ctx(ctx));
  RMI_TRY(rmi_check_weight(w, RMI_GGML_Q4_K));
  RMI_REQUIRE(((uintptr_t)x & 15) == 0, RMI_ERR_BAD_SHAPE, "device input must be 16-byte aligned");
  return launch_q4k_dequant_matmul(ctx, w, x, m, output);
}

extern "C" int32_t rmi_matmul_q4_k_dequant(rmi_ctx* ctx, const rmi_weight* w, const float* x, size_t m, float* output) {
  RMI_TRY(rmi_check_ctx(ctx));
  RMI_TRY(rmi_check_weight(w, RMI_GGML_Q4_K));
  if (m == 0 || w->n_rows == 0) return RMI_OK;
  RMI_REQUIRE(x && output, RMI_ERR_BAD_HANDLE, "rmi_matmul_q4_k_dequant: null buffer");
  std::lock_guard<std::mutex> lock(ctx->mu);
  float *dx, *dout;
  RMI_TRY(rmi_scratch(ctx, 5, m * w->n_in * 4, (void**)&dx));
  RMI_TRY(rmi_scratch(ctx, 6, m * w->n_rows * 4, (void**)&dout));
  RMI_CUDA_CHECK(cudaMemcpyAsync(dx, x, m * w->n_in * 4, cudaMemcpyHostToDevice, ctx->stream));
  RMI_TRY(launch_q4k_dequant_matmul(ctx, w, dx, m, dout));
  RMI_CUDA_CHECK(cudaMemcpyAsync(output, dout, m * w->n_rows * 4, cudaMemcpyDeviceToHost, ctx->stream));
  RMI_CUDA_CHECK(cudaStreamSynchronize(ctx->stream));
  return RMI_OK;
}

extern "C" int32_t rmi_dequantize_q4_k(rmi_ctx* ctx, const rmi_weight* w, float* output) {
  RMI_TRY(rmi_check_ctx(ctx));
  RMI_TRY(rmi_check_weight(w, RMI_GGML_Q4_K));
  if (w->n_rows == 0) return RMI_OK;
  RMI_REQUIRE(output != nullptr, RMI_ERR_BAD_HANDLE, "rmi_dequantize_q4_k: null buffer");
  std::lock_guard<std::mutex> lock(ctx->mu);
  float* dout;
  RMI_TRY(rmi_scratch(ctx, 6, w->n_rows * w->n_in * 4, (void**)&dout));
  RMI_TRY(launch_q4k_dequantize(ctx, w, dout));
  RMI_CUDA_CHECK(cudaMemcpyAsync(output, dout, w->n_rows * w->n_in * 4, cudaMemcpyDeviceToHost, ctx->stream));
  RMI_CUDA_CHECK(cudaStreamSynchronize(ctx->stream));
  return RMI_OK;
}

// ---------------------------------------------------------------- Q6_K

extern "C" int32_t rmi_matmul_q6_k_q8k(rmi_ctx* ctx, const rmi_weight* w, const float* x, size_t m, float* output,
                                       size_t row_begin, size_t row_end) {
  RMI_TRY(rmi_check_ctx(ctx));
  RMI_TRY(rmi_check_weight(w, RMI_GGML_Q6_K));
  RMI_REQUIRE(row_begin <= row_end && row_end <= w->n_rows, RMI_ERR_BAD_SHAPE, "row range [%zu,%zu) outside [0,%zu)",
              row_begin, row_end, w->n_rows);
  if (m == 0 || row_begin == row_end) return RMI_OK;
  RMI_REQUIRE(x && output, RMI_ERR_BAD_HANDLE, "rmi_matmul_q6_k_q8k: null buffer");
  RMI_REQUIRE(ctx->sem != RMI_SEM_NEON, RMI_ERR_UNSUPPORTED, "the reference has no NEON Q6_K x Q8_K kernel; use AVX2 or SCALAR");
  std::lock_guard<std::mutex> lock(ctx->mu);
  const size_t n = w->n_in, nb = m * n / 256, nr = row_end - row_begin;
  float *dx, *dd, *dout;
  int8_t* dq;
  int16_t* db;
  RMI_TRY(rmi_scratch(ctx, 5, m * n * 4, (void**)&dx));
  RMI_TRY(rmi_scratch(ctx, 0, m * n, (void**)&dq));
  RMI_TRY(rmi_scratch(ctx, 1, nb * 4, (void**)&dd));
  RMI_TRY(rmi_scratch(ctx, 4, nb * 32, (void**)&db));
  RMI_TRY(rmi_scratch(ctx, 6, m * w->n_rows * 4, (void**)&dout));
  RMI_CUDA_CHECK(cudaMemcpyAsync(dx, x, m * n * 4, cudaMemcpyHostToDevice, ctx->stream));
  RMI_TRY(launch_q8k_quantize(ctx, dx, m, n, dd, dq, db));
  RMI_TRY(launch_q6k_q8k_matmul(ctx, w, dd, dq, db, m, dout, row_begin, row_end));
  RMI_CUDA_CHECK(cudaMemcpy2DAsync(output + row_begin, w->n_rows * 4, dout + row_begin, w->n_rows * 4, nr * 4, m,
                                   cudaMemcpyDeviceToHost, ctx->stream));
  RMI_CUDA_CHECK(cudaStreamSynchronize(ctx->stream));
  return RMI_OK;
}

extern "C" int32_t rmi_matmul_q6_k_prequantized(rmi_ctx* ctx, const rmi_weight* w, const uint8_t* q8, const float* scales,
                                                size_t m, float* output, size_t row_begin, size_t row_end) {
  RMI_TRY(rmi_check_ctx(ctx));
  RMI_TRY(rmi_check_weight(w, RMI_GGML_Q6_K));
  RMI_REQUIRE(row_begin <= row_end && row_end <= w->n_rows, RMI_ERR_BAD_SHAPE, "row range [%zu,%zu) outside [0,%zu)",
              row_begin, row_end, w->n_rows);
  if (m == 0 || row_begin == row_end) return RMI_OK;
  RMI_REQUIRE(q8 && scales && output, RMI_ERR_BAD_HANDLE, "rmi_matmul_q6_k_prequantized: null buffer");
  std::lock_guard<std::mutex> lock(ctx->mu);
  const size_t n = w->n_in, nr = row_end - row_begin;
  uint8_t* dq;
  float *ds, *dout;
  RMI_TRY(rmi_scratch(ctx, 0, m * n, (void**)&dq));
  RMI_TRY(rmi_scratch(ctx, 1, m * (n / 32) * 4, (void**)&ds));
  RMI_TRY(rmi_scratch(ctx, 6, m * w->n_rows * 4, (void**)&dout));
  RMI_CUDA_CHECK(cudaMemcpyAsync(dq, q8, m * n, cudaMemcpyHostToDevice, ctx->stream));
  RMI_CUDA_CHECK(cudaMemcpyAsync(ds, scales, m * (n / 32) * 4, cudaMemcpyHostToDevice, ctx->stream));
  RMI_TRY(launch_q6k_prequant_matmul(ctx, w, dq, ds, m, dout, row_begin, row_end));
  RMI_CUDA_CHECK(cudaMemcpy2DAsync(output + row_begin, w->n_rows * 4, dout + row_begin, w->n_rows * 4, nr * 4, m,
                                   cudaMemcpyDeviceToHost, ctx->stream));
  RMI_CUDA_CHECK(cudaStreamSynchronize(ctx->stream));
  return RMI_OK;
}

extern "C" int32_t rmi_dequantize_q6_k(rmi_ctx* ctx, const rmi_weight* w, float* output) {
  RMI_TRY(rmi_check_ctx(ctx));
  RMI_TRY(rmi_check_weight(w, RMI_GGML_Q6_K));
  if (w->n_rows == 0) return RMI_OK;
  RMI_REQUIRE(output != nullptr, RMI_ERR_BAD_HANDLE, "rmi_dequantize_q6_k: null buffer");
  std::lock_guard<std::mutex> lock(ctx->mu);
  float* dout;
  RMI_TRY(rmi_scratch(ctx, 6, w->n_rows * w->n_in * 4, (void**)&dout));
  RMI_TRY(launch_q6k_dequantize(ctx, w, dout));
  RMI_CUDA_CHECK(cudaMemcpyAsync(output, dout, w->n_rows * w->n_in * 4, cudaMemcpyDeviceToHost, ctx->stream));
  RMI_CUDA_CHECK(cudaStreamSynchronize(ctx->stream));
  return RMI_OK;
}

// ---------------------------------------------------------------- Q4_0

extern "C" int32_t rmi_matmul_q4_0_prequantized(rmi_ctx* ctx, const rmi_weight* w, const uint8_t* q8, const float* scales,
                                                size_t m, float* output, size_t row_begin, size_t row_end) {
  RMI_TRY(rmi_check_ctx(ctx));
  RMI_TRY(rmi_check_weight(w, RMI_GGML_Q4_0));
  RMI_REQUIRE(row_begin <= row_end && row_end <= w->n_rows, RMI_ERR_BAD_SHAPE, "row range [%zu,%zu) outside [0,%zu)",
              row_begin, row_end, w->n_rows);
  if (m == 0 || row_begin == row_end) return RMI_OK;
  RMI_REQUIRE(q8 && scales && output, RMI_ERR_BAD_HANDLE, "rmi_matmul_q4_0_prequantized: null buffer");
  std::lock_guard<std::mutex> lock(ctx->mu);
  const size_t n = w->n_in, nr = row_end - row_begin;
  uint8_t* dq;
  float *ds, *dout;
  RMI_TRY(rmi_scratch(ctx, 0, m * n, (void**)&dq));
  RMI_TRY(rmi_scratch(ctx, 1, m * (n / 32) * 4, (void**)&ds));
  RMI_TRY(rmi_scratch(ctx, 6, m * w->n_rows * 4, (void**)&dout));
  RMI_CUDA_CHECK(cudaMemcpyAsync(dq, q8, m * n, cudaMemcpyHostToDevice, ctx->stream));
  RMI_CUDA_CHECK(cudaMemcpyAsync(ds, scales, m * (n / 32) * 4, cudaMemcpyHostToDevice, ctx->stream));
  RMI_TRY(launch_q4_0_matmul(ctx, w, dq, ds, m, dout, row_begin, row_end));
  RMI_CUDA_CHECK(cudaMemcpy2DAsync(output + row_begin, w->n_rows * 4, dout + row_begin, w->n_rows * 4, nr * 4, m,
                                   cudaMemcpyDeviceToHost, ctx->stream));
  RMI_CUDA_CHECK(cudaStreamSynchronize(ctx->stream));
  return RMI_OK;
}

extern "C" int32_t rmi_matmul_q4_0(rmi_ctx* ctx, const rmi_weight* w, const float* x, size_t m, float* output) {
  RMI_TRY(rmi_check_ctx(ctx));
  RMI_TRY(rmi_check_weight(w, RMI_GGML_Q4_0));
  if (m == 0 || w->n_rows == 0) return RMI_OK;
  RMI_REQUIRE(x && output, RMI_ERR_BAD_HANDLE, "rmi_matmul_q4_0: null buffer");
  std::lock_guard<std::mutex> lock(ctx->mu);
  const size_t n = w->n_in;
  uint8_t* dq;
  float *dx, *ds, *dout;
  RMI_TRY(rmi_scratch(ctx, 5, m * n * 4, (void**)&dx));
  RMI_TRY(rmi_scratch(ctx, 0, m * n, (void**)&dq));
  RMI_TRY(rmi_scratch(ctx, 1, m * (n / 32) * 4, (void**)&ds));
  RMI_TRY(rmi_scratch(ctx, 6, m * w->n_rows * 4, (void**)&dout));
  RMI_CUDA_CHECK(cudaMemcpyAsync(dx, x, m * n * 4, cudaMemcpyHostToDevice, ctx->stream));
  RMI_TRY(launch_q8_quantize(ctx, dx, m, n, dq, ds, 0));
  RMI_TRY(launch_q4_0_matmul(ctx, w, dq, ds, m, dout, 0, w->n_rows));
  RMI_CUDA_CHECK(cudaMemcpyAsync(output, dout, m * w->n_rows * 4, cudaMemcpyDeviceToHost, ctx->stream));
  RMI_CUDA_CHECK(cudaStreamSynchronize(ctx->stream));
  return RMI_OK;
}

// ---------------------------------------------------------------- embedding lookup

extern "C" int32_t rmi_embedding_lookup(rmi_ctx* ctx, const rmi_weight* w, const uint32_t* token_ids, size_t m,
                                        float* output) {
  RMI_TRY(rmi_check_ctx(ctx));
  RMI_TRY(rmi_check_weight(w, -1));
  RMI_REQUIRE(w->ggml_type == RMI_GGML_Q8_0 || w->ggml_type == RMI_GGML_Q4_0 || w->ggml_type == RMI_GGML_Q6_K,
              RMI_ERR_UNSUPPORTED, "unsupported embedding type %d (Q8_0, Q4_0 and Q6_K are handled)", w->ggml_type);
  if (m == 0 || w->n_in == 0) return RMI_OK;
  RMI_REQUIRE(token_ids && output, RMI_ERR_BAD_HANDLE, "rmi_embedding_lookup: null buffer");
  for (size_t i = 0; i < m; i++)
    RMI_REQUIRE(token_ids[i] < w->n_rows, RMI_ERR_BAD_SHAPE, "token id %u at position %zu is outside the table of %zu rows",
                token_ids[i], i, w->n_rows);
  std::lock_guard<std::mutex> lock(ctx->mu);
  uint32_t* dids;
  float* dout;
  RMI_TRY(rmi_scratch(ctx, 0, m * 4, (void**)&dids));
  RMI_TRY(rmi_scratch(ctx, 6, m * w->n_in * 4, (void**)&dout));
  RMI_CUDA_CHECK(cudaMemcpyAsync(dids, token_ids, m * 4, cudaMemcpyHostToDevice, ctx->stream));
  if (w->ggml_type == RMI_GGML_Q8_0) RMI_TRY(launch_q8_embedding(ctx, w, dids, m, dout));
  else if (w->ggml_type == RMI_GGML_Q4_0) RMI_TRY(launch_q4_0_embedding(ctx, w, dids, m, dout));
  else RMI_TRY(launch_q6k_embedding(ctx, w, dids, m, dout));
  RMI_CUDA_CHECK(cudaMemcpyAsync(output, dout, m * w->n_in * 4, cudaMemcpyDeviceToHost, ctx->stream));
  RMI_CUDA_CHECK(cudaStreamSynchronize(ctx->stream));
  return RMI_OK;
}
