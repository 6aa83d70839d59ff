// The reference's own Q8Kernel unit tests (src/ops/kernel/q8_0/mod.rs:58-157) and the Q4_K
// known answer (tests/quantized_inference.rs:233-249), written against the C++ mirror of the
// trait and run on the device.  Exit code 0 = all passed.
#include <cmath>
#include <cstdio>
#include <cstring>
#include <vector>

#include "../../rust-model-inference_b200/host/rmi_kernel.hpp"

static int failures = 0;
#define EXPECT(cond)                                         \
  do {                                                       \
    if (!(cond)) {                                           \
      std::printf("FAIL %s:%d %s\n", __FILE__, __LINE__, #cond); \
      failures++;                                            \
    }                                                        \
  } while (0)

static uint16_t f16_bits(float v) {  // exact for the powers of two used here
  uint32_t u;
  std::memcpy(&u, &v, 4);
  return (uint16_t)(((u >> 16) & 0x8000) | ((((u >> 23) & 0xff) - 112) << 10) | ((u >> 13) & 0x3ff));
}

static std::vector<uint8_t> q8_0_uniform_row(int8_t value, float scale) {
  std::vector<uint8_t> row(34, (uint8_t)value);
  uint16_t b = f16_bits(scale);
  std::memcpy(row.data(), &b, 2);
  return row;
}

// The session's per-step interface from a compiled host: the host samples (first maximal index) from the logits
// the library returns and must agree with the library's own greedy choice.
static void session_checks(const char* gguf_path) {
  rmi_ctx* ctx = rmi::context();
  rmi_qwen3* model = nullptr;
  rmi::check(rmi_qwen3_load(ctx, gguf_path, &model));
  size_t vocab = 0;
  rmi::check(rmi_qwen3_config(model, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, &vocab));
  rmi_session* s = nullptr;
  const size_t batch = 2;
  rmi::check(rmi_session_create(ctx, model, batch, 32, &s));
  rmi::check(rmi_session_reset(ctx, s));
  const uint32_t prompt[2][3] = {{1, 2, 3}, {7, 5, 3}};
  rmi::check(rmi_session_prefill(ctx, s, &prompt[0][0], 3));
  size_t pos = 99;
  rmi::check(rmi_session_position(s, &pos));
  EXPECT(pos == 3);
  std::vector<uint32_t> tok = {4, 9}, next(batch);
  std::vector<float> logits(batch * vocab);
  for (int step = 0; step < 4; step++) {
    rmi::check(rmi_session_step(ctx, s, tok.data(), next.data(), logits.data()));
    for (size_t b = 0; b < batch; b++) {
      size_t best = 0;
      for (size_t i = 1; i < vocab; i++)
        if (logits[b * vocab + i] > logits[b * vocab + best]) best = i;
      EXPECT(best == next[b]);
    }
    tok = next;
  }
  rmi::check(rmi_session_position(s, &pos));
  EXPECT(pos == 7);
  rmi::check(rmi_session_free(ctx, s));
  rmi::check(rmi_qwen3_free(ctx, model));
}

// One rank of the row-sharded matmul (world = 1): both exchanges of the shard group and the NCCL entry point must
// reproduce the plain matmul bit for bit.
static void sharded_checks() {
  rmi_ctx* ctx = rmi::context();
  const size_t n = 64, k = 64, m = 5;
  std::vector<uint8_t> w;
  for (size_t r = 0; r < n; r++)
    for (size_t b = 0; b < k / 32; b++) {
      auto blk = q8_0_uniform_row((int8_t)(1 + (r + b) % 5), 0.5f);
      w.insert(w.end(), blk.begin(), blk.end());
    }
  rmi_weight* wt = nullptr;
  rmi::check(rmi_weight_upload(ctx, RMI_GGML_Q8_0, w.data(), w.size(), k, n, 0, n, &wt));
  std::vector<float> x(m * k), ref(m * n), got(m * n);
  for (size_t i = 0; i < x.size(); i++) x[i] = 0.01f * (float)(i % 37) - 0.2f;
  rmi::check(rmi_matmul_q8_0(ctx, wt, x.data(), m, ref.data()));
  void* dx = nullptr;
  rmi::check(rmi_dev_alloc(ctx, x.size() * 4, &dx));
  rmi::check(rmi_h2d(ctx, dx, x.data(), x.size() * 4));
  rmi_shard_group* g = nullptr;
  rmi::check(rmi_shard_group_create(ctx, 1, 0, n, 8, &g));
  uint8_t handles[192];
  rmi::check(rmi_shard_group_export(ctx, g, handles));
  rmi::check(rmi_shard_group_connect(ctx, g, handles));
  for (int exchange : {RMI_EXCHANGE_FUSED_STORES, RMI_EXCHANGE_PEER_COPY, RMI_EXCHANGE_PEER_PUSH}) {
    float* result = nullptr;
    rmi::check(rmi_matmul_q8_0_sharded_dev(ctx, g, wt, (const float*)dx, m, exchange, &result));
    rmi::check(rmi_check_status(ctx));
    rmi::check(rmi_d2h(ctx, got.data(), result, got.size() * 4));
    EXPECT(std::memcmp(got.data(), ref.data(), got.size() * 4) == 0);
  }
  uint32_t epoch = 0;
  rmi::check(rmi_shard_group_epoch(g, &epoch));
  EXPECT(epoch == 3);
  rmi::check(rmi_shard_group_free(ctx, g));
  // NCCL entry point with a one-rank communicator created through the library
  uint8_t id[128];
  void* comm = nullptr;
  rmi::check(rmi_nccl_unique_id(id));
  rmi::check(rmi_nccl_comm_create(ctx, id, 1, 0, &comm));
  void *dy = nullptr, *dgath = nullptr, *dout = nullptr;
  rmi::check(rmi_dev_alloc(ctx, got.size() * 4, &dy));
  rmi::check(rmi_dev_alloc(ctx, got.size() * 4, &dgath));
  rmi::check(rmi_dev_alloc(ctx, got.size() * 4, &dout));
  rmi::check(rmi_matmul_q8_0_dev(ctx, wt, (const float*)dx, m, (float*)dy));
  rmi::check(rmi_allgather_cols_dev(ctx, comm, (const float*)dy, m, n, 1, (float*)dgath, (float*)dout));
  rmi::check(rmi_d2h(ctx, got.data(), dout, got.size() * 4));
  EXPECT(std::memcmp(got.data(), ref.data(), got.size() * 4) == 0);
  rmi::check(rmi_nccl_comm_destroy(comm));
  for (void* p : {dx, dy, dgath, dout}) rmi::check(rmi_dev_free(ctx, p));
  rmi::check(rmi_weight_free(ctx, wt));
}

int main(int argc, char** argv) {
  try {
    std::vector<uint8_t> q8(32, 1);
    std::vector<float> sc(1, 1.0f);
    {  // q8_kernel_uniform_weights_sum_to_dot_product / multi_row / scale_applied
      auto w = q8_0_uniform_row(1, 1.0f);
      rmi::Q8Kernel k(w.data(), w.size(), 32, 1);
      float out[1] = {0};
      k.forward_prequantized(q8.data(), sc.data(), out, 32, 1, 0, 1);
      EXPECT(out[0] == 32.0f);
      auto w2 = w;
      w2.insert(w2.end(), w.begin(), w.end());
      rmi::Q8Kernel k2(w2.data(), w2.size(), 32, 2);
      float out2[2] = {0, 0};
      k2.forward_prequantized(q8.data(), sc.data(), out2, 32, 2, 0, 1);
      EXPECT(out2[0] == 32.0f && out2[1] == 32.0f);
      auto wh = q8_0_uniform_row(1, 0.5f);
      rmi::Q8Kernel k3(wh.data(), wh.size(), 32, 1);
      k3.forward_prequantized(q8.data(), sc.data(), out, 32, 1, 0, 1);
      EXPECT(out[0] == 16.0f);
      // q8_kernel_forward_quantizes_internally
      std::vector<float> ones(32, 1.0f);
      k.forward(ones.data(), out, 32, 1);
      EXPECT(std::fabs(out[0] - 32.0f) < 5e-3f);
    }
    {  // legacy f32-input matmul: uniform weight 1 * 0.5 against an exactly representable activation row
      auto w = q8_0_uniform_row(1, 0.5f);
      rmi::Weight wt(RMI_GGML_Q8_0, w.data(), w.size(), 32, 1);
      std::vector<float> x(32);
      float expect = 0.0f;
      for (int i = 0; i < 32; i++) {
        x[i] = 0.25f * (float)(i - 7);
        expect += 0.5f * x[i];
      }
      float out[1] = {0};
      rmi::matmul_q8_0(wt, x.data(), out, 32, 1);
      EXPECT(out[0] == expect);  // every partial sum is a small multiple of 1/8: exact in any order
    }
    {  // q8_kernel_thread_partition
      std::vector<uint8_t> w;
      for (int i = 0; i < 4; i++) {
        auto r = q8_0_uniform_row(1, 1.0f);
        w.insert(w.end(), r.begin(), r.end());
      }
      rmi::Q8Kernel k(w.data(), w.size(), 32, 4);
      float a[4] = {0, 0, 0, 0}, b[4] = {0, 0, 0, 0};
      k.forward_prequantized(q8.data(), sc.data(), a, 32, 4, 0, 2);
      k.forward_prequantized(q8.data(), sc.data(), b, 32, 4, 1, 2);
      EXPECT(a[0] == 32.0f && a[1] == 32.0f && a[2] == 0.0f && a[3] == 0.0f);
      EXPECT(b[0] == 0.0f && b[1] == 0.0f && b[2] == 32.0f && b[3] == 32.0f);
      // forward_batched == per-token forward, bit for bit
      std::vector<float> x(3 * 32), o1(12), o2(12);
      for (size_t i = 0; i < x.size(); i++) x[i] = 0.013f * (float)i - 1.0f;
      k.forward_batched(x.data(), 3, o1.data(), 32, 4);
      for (int t = 0; t < 3; t++) k.forward(x.data() + 32 * t, o2.data() + 4 * t, 32, 4);
      EXPECT(std::memcmp(o1.data(), o2.data(), 48) == 0);
    }
    {  // q4_k_kernel_multiplies_uniform_block + QuantizedLinear
      std::vector<uint8_t> w(144, 0);
      uint16_t one = f16_bits(1.0f);
      std::memcpy(w.data(), &one, 2);
      const uint8_t scales[12] = {1, 1, 1, 1, 0, 0, 0, 0, 1, 1, 1, 1};
      std::memcpy(w.data() + 4, scales, 12);
      std::memset(w.data() + 16, 0x11, 128);
      rmi::Q4_KKernel k(w.data(), w.size(), 256, 1);
      std::vector<uint8_t> q(256, 1);
      std::vector<float> s(8, 1.0f);
      float out[1] = {0};
      k.forward_prequantized(q.data(), s.data(), out, 256, 1, 0, 1);
      EXPECT(out[0] == 256.0f);
      auto lin = rmi::QuantizedLinear::from_weight_slice(w.data(), w.size(), 256, 1, "uniform");
      std::vector<float> ones(256, 1.0f);
      lin.forward(ones.data(), out);
      EXPECT(out[0] == 256.0f && lin.input_dim() == 256 && lin.output_dim() == 1 && lin.name() == "uniform");
    }
    {  // error convention: shape errors surface as exceptions with the library's status code
      bool threw = false;
      try {
        std::vector<uint8_t> w(34);
        rmi::Q8Kernel bad(w.data(), w.size(), 33, 1);
      } catch (const rmi::Error& e) {
        threw = e.status == RMI_ERR_BAD_SHAPE;
      }
      EXPECT(threw);
    }
    sharded_checks();
    if (argc > 1) session_checks(argv[1]);
  } catch (const std::exception& e) {
    std::printf("FAIL exception: %s\n", e.what());
    failures++;
  }
  std::printf(failures ? "%d failure(s)\n" : "all kernel-trait checks passed\n", failures);
  return failures ? 1 : 0;
}
