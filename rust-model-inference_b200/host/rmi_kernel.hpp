// C++ mirror of the reference's kernel interface over the C ABI (include/rmi_cuda.h).
//
// The reference is Rust; this header states the same interface in C++ so that a compiled host
// can drive the library exactly the way the Rust shim would:
//   trait Kernel                          src/ops/kernel/trait_.rs:15-110
//   Q8Kernel                              src/ops/kernel/q8_0/mod.rs:22-56
//   Q4_KKernel                            src/ops/kernel/q4_k.rs:7-93
//   QuantizedLinear                       src/core/model.rs:12-104
//   quantize_q8_0_into                    src/ops/quant/q8_0.rs:3-24
//   matmul_q8_0_quantized_parallel_rows   src/ops/kernel/q8_0/parallel.rs:102-139
//   matmul_q8_0 (legacy f32 input)        src/ops/kernel/q8_0/parallel.rs:317-341
// Error convention: the trait methods return nothing; a failing device call throws
// rmi::Error (the Rust shim panics, like `.expect("GPU matmul failed")` in dispatch.rs:47-48).
#pragma once

#include <cstdint>
#include <memory>
#include <stdexcept>
#include <string>
#include <vector>

#include "../../include/rmi_cuda.h"

namespace rmi {

struct Error : std::runtime_error {
  int32_t status;
  Error(int32_t s, const std::string& m) : std::runtime_error(m), status(s) {}
};

inline void check(int32_t status) {
  if (status != RMI_OK) throw Error(status, rmi_last_error());
}

// Process-wide context, created on first use (src/ops/float.rs:44-58); failure throws.
inline rmi_ctx* context(int device = 0) {
  static rmi_ctx* ctx = nullptr;
  if (!ctx) check(rmi_init(device, &ctx));
  return ctx;
}

// quantize_q8_0_into(input, n, q8, scales)
inline void quantize_q8_0_into(const float* input, size_t n, uint8_t* q8, float* scales) {
  check(rmi_quantize_q8_0(context(), input, 1, n, q8, scales));
}

class Weight {
 public:
  Weight(int32_t ggml_type, const void* bytes, size_t nbytes, size_t n_in, size_t n_out) : n_in_(n_in), n_out_(n_out) {
    check(rmi_weight_upload(context(), ggml_type, bytes, nbytes, n_in, n_out, 0, n_out, &w_));
  }
  ~Weight() {
    if (w_) rmi_weight_free(context(), w_);
  }
  Weight(const Weight&) = delete;
  Weight& operator=(const Weight&) = delete;
  rmi_weight* handle() const { return w_; }
  size_t n_in() const { return n_in_; }
  size_t n_out() const { return n_out_; }

 private:
  rmi_weight* w_ = nullptr;
  size_t n_in_, n_out_;
};

// matmul_q8_0_quantized_parallel_rows(weight, input_q8, input_scales, output, n_in, n_out, ith, nth)
inline void matmul_q8_0_quantized_parallel_rows(const Weight& weight, const uint8_t* input_q8, const float* input_scales,
                                                float* output, size_t /*n_in*/, size_t n_out, size_t ith, size_t nth) {
  size_t s = 0, e = n_out;
  if (nth > 1 && n_out != 0) {
    const size_t per = (n_out + nth - 1) / nth;
    s = ith * per;
    e = s + per < n_out ? s + per : n_out;
    if (s >= e) return;
  }
  check(rmi_matmul_q8_0_prequantized(context(), weight.handle(), input_q8, input_scales, 1, output, s, e));
}

// matmul_q8_0(weight, input, output, n_in, n_out): the legacy f32-input matmul, one activation row, no activation
// quantization; accumulation order by the context's semantics (AVX2 or the scalar fallback).
inline void matmul_q8_0(const Weight& weight, const float* input, float* output, size_t /*n_in*/, size_t /*n_out*/) {
  check(rmi_matmul_q8_0_f32(context(), weight.handle(), input, 1, output));
}

// trait Kernel
class Kernel {
 public:
  virtual ~Kernel() = default;
  virtual void forward_prequantized(const uint8_t* input_q8, const float* input_scales, float* output, size_t n_in,
                                    size_t n_out, size_t ith, size_t nth) const = 0;
  // default: drop the f32 view and the Q8_K blocks (trait_.rs:39-54)
  virtual void forward_prepared(const float* /*input_f32*/, const uint8_t* input_q8, const float* input_scales,
                                float* output, size_t n_in, size_t n_out, size_t ith, size_t nth) const {
    forward_prequantized(input_q8, input_scales, output, n_in, n_out, ith, nth);
  }
  // quantize, then forward_prepared(.., 0, 1) (trait_.rs:57-75)
  virtual void forward(const float* input, float* output, size_t n_in, size_t n_out) const {
    std::vector<uint8_t> q8(n_in);
    std::vector<float> scales((n_in + 31) / 32);
    quantize_q8_0_into(input, n_in, q8.data(), scales.data());
    forward_prepared(input, q8.data(), scales.data(), output, n_in, n_out, 0, 1);
  }
  // per-token loop (trait_.rs:78-109)
  virtual void forward_batched(const float* input, size_t n_tokens, float* output, size_t n_in, size_t n_out) const {
    for (size_t t = 0; t < n_tokens; t++) forward(input + t * n_in, output + t * n_out, n_in, n_out);
  }
};

class Q8Kernel : public Kernel {
 public:
  Q8Kernel(const void* weight, size_t nbytes, size_t n_in, size_t n_out)
      : w_(std::make_unique<Weight>(RMI_GGML_Q8_0, weight, nbytes, n_in, n_out)) {}
  void forward_prequantized(const uint8_t* input_q8, const float* input_scales, float* output, size_t n_in, size_t n_out,
                            size_t ith, size_t nth) const override {
    matmul_q8_0_quantized_parallel_rows(*w_, input_q8, input_scales, output, n_in, n_out, ith, nth);
  }
  // one device call for all tokens (GEMV kernels up to 32 rows, tcgen05 GEMM above)
  void forward_batched(const float* input, size_t n_tokens, float* output, size_t, size_t) const override {
    check(rmi_matmul_q8_0(context(), w_->handle(), input, n_tokens, output));
  }
  const Weight& weight() const { return *w_; }

 private:
  std::unique_ptr<Weight> w_;
};

class Q4_KKernel : public Kernel {
 public:
  Q4_KKernel(const void* data, size_t nbytes, size_t n_in, size_t n_out)
      : w_(std::make_unique<Weight>(RMI_GGML_Q4_K, data, nbytes, n_in, n_out)) {}
  // q4_k.rs:20-54: Q8_0 activation dequantized to f32, dequantized weight rows, f32 dot
  void forward_prequantized(const uint8_t* input_q8, const float* input_scales, float* output, size_t n_in, size_t n_out,
                            size_t ith, size_t nth) const override {
    const size_t per = (n_out + nth - 1) / nth, s = ith * per, e = s + per < n_out ? s + per : n_out;
    if (s >= e) return;
    std::vector<float> x(n_in), full(n_out);
    for (size_t i = 0; i < n_in; i++) x[i] = (float)(int8_t)input_q8[i] * input_scales[i / 32];
    check(rmi_matmul_q4_k_dequant(context(), w_->handle(), x.data(), 1, full.data()));
    for (size_t r = s; r < e; r++) output[r] = full[r];
  }
  // q4_k.rs:56-93: Q8_K activation, vec_dot_q4k_q8k per row
  void forward_prepared(const float* input_f32, const uint8_t*, const float*, float* output, size_t, size_t n_out,
                        size_t ith, size_t nth) const override {
    const size_t per = (n_out + nth - 1) / nth, s = ith * per, e = s + per < n_out ? s + per : n_out;
    if (s >= e) return;
    check(rmi_matmul_q4_k_q8k(context(), w_->handle(), input_f32, 1, output, s, e));
  }

 private:
  std::unique_ptr<Weight> w_;
};

// QuantizedLinear<'a>: Q4_K dequantize-and-matmul Layer (src/core/model.rs:12-104)
class QuantizedLinear {
 public:
  static QuantizedLinear from_weight_slice(const void* weight, size_t nbytes, size_t in_features, size_t out_features,
                                           std::string name) {
    return QuantizedLinear(std::make_shared<Weight>(RMI_GGML_Q4_K, weight, nbytes, in_features, out_features),
                           std::move(name));
  }
  void forward_dequant(const float* input, float* output) const {
    check(rmi_matmul_q4_k_dequant(context(), w_->handle(), input, 1, output));
  }
  void forward(const float* input, float* output) const { forward_dequant(input, output); }
  size_t input_dim() const { return w_->n_in(); }
  size_t output_dim() const { return w_->n_out(); }
  const std::string& name() const { return name_; }

 private:
  QuantizedLinear(std::shared_ptr<Weight> w, std::string n) : w_(std::move(w)), name_(std::move(n)) {}
  std::shared_ptr<Weight> w_;
  std::string name_;
};

}  // namespace rmi
