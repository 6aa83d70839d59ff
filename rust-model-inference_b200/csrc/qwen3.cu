// Qwen3-architecture model and decode session on the device.
//
// Restates Qwen3Model::from_source (src/models/qwen3.rs:246-400) and
// Qwen3Session::{new, generate_inner} (src/models/qwen3.rs:440-550, :581-1158) of the
// reference for `batch` independent sequences.  One decode step is a fixed sequence of
// kernels captured once into a CUDA graph; the position lives in device memory and is
// advanced by the last node, so the same graph is replayed for every step.
#include <math.h>
#include <stdlib.h>
#include <string.h>

#include <new>
#include <string>
#include <utility>
#include <vector>

#include "common.cuh"
#include "decode.cuh"
#include "kernels.cuh"

static constexpr uint32_t RMI_MODEL_MAGIC = 0x524d494d;
static constexpr uint32_t RMI_SESSION_MAGIC = 0x524d4953;

struct layer_weights {
  float *attn_norm, *ffn_norm, *q_norm, *k_norm;
  rmi_weight *wqkv, *wo, *wgu, *wdown;
};

struct rmi_qwen3 {
  uint32_t magic;
  decode_dims d;  // batch / capacity unused here
  float freq_base;
  size_t n_ctx;
  std::vector<layer_weights> layers;
  float* output_norm;
  rmi_weight* token_embd;
  rmi_weight* output;  // == token_embd when tied
  size_t weight_bytes;
};

struct rmi_session {
  uint32_t magic;
  const rmi_qwen3* model;
  decode_dims d;
  uint16_t *k_cache, *v_cache;
  float *x, *x2, *qkv, *proj, *gu, *logits, *rope, *attn_dbg;  // x2: second residual buffer of the fused-norm path
  bool fused_norm;
  void* attn_scratch;  // score / probability rows of attention_seq_kernel when they do not fit in shared memory
  int forward;    // RMI_FORWARD_*: which of the reference's copies of the forward this session reproduces
  float* q32;     // f32 query after norm + rotation (CLI forward)
  float *k32_cache, *v32_cache;  // F32 caches of the CLI forward with `--kv-cache f32`; allocated on first use
  bool seq_attention;  // one CTA per (sequence, kv head) instead of a cluster: large batches
  bool fused_qk;  // q/k norm + rotation + cache write inside the attention kernel
  uint16_t* q16;
  uint8_t* q8;
  float* xs;
  uint32_t *prompts, *gen;
  size_t prompts_cap, gen_cap;
  int *d_step, *d_flag;
  float* argmax_v;
  uint32_t* argmax_i;
  // batched prompt processing (rows = sequences of a group x prompt positions); buffers allocated on first use
  // per-step interface (rmi_session_reset / _prefill / _step): tokens live in the ring gen[batch][capacity + 1]
  bool step_mode;
  size_t pos;        // next position to be computed
  int prefill_mode;  // RMI_PREFILL_*
  size_t pf_rows;
  float *pf_x, *pf_xn, *pf_qkv, *pf_attn, *pf_proj;
  uint16_t* pf_q16;
  cudaGraph_t graph_body, graph_full;
  cudaGraphExec_t exec_body, exec_full;
  size_t graph_n_prompt, graph_n_gen;
  int graph_sem;
  cudaStream_t graph_stream;
};

static int32_t check_model(const rmi_qwen3* m) {
  RMI_REQUIRE(m != nullptr && m->magic == RMI_MODEL_MAGIC, RMI_ERR_BAD_HANDLE, "invalid rmi_qwen3 handle");
  return RMI_OK;
}
static int32_t check_session(const rmi_session* s) {
  RMI_REQUIRE(s != nullptr && s->magic == RMI_SESSION_MAGIC, RMI_ERR_BAD_HANDLE, "invalid rmi_session handle");
  return RMI_OK;
}

// load_f32_tensor (src/models/qwen3.rs:1338-1348) + checked_tensor (:1350-1380)
static int32_t load_f32(rmi_ctx* ctx, const rmi_gguf* g, const std::string& name, size_t n, float** out) {
  int32_t type, nd;
  uint64_t dims[4];
  const void* data;
  size_t nbytes;
  RMI_TRY(rmi_gguf_tensor(g, name.c_str(), &type, dims, &nd, &data, &nbytes));
  RMI_REQUIRE(type == RMI_GGML_F32 && nd == 1 && dims[0] == n, RMI_ERR_FORMAT,
              "Invalid tensor %s: expected F32 [%zu]", name.c_str(), n);
  RMI_CUDA_CHECK(cudaMalloc(out, n * 4));
  RMI_CUDA_CHECK(cudaMemcpy(*out, data, n * 4, cudaMemcpyHostToDevice));
  return RMI_OK;
}

static int32_t load_q8(rmi_ctx* ctx, const rmi_gguf* g, const std::string& name, size_t n_in, size_t n_out,
                       rmi_weight** out) {
  int32_t type, nd;
  uint64_t dims[4];
  RMI_TRY(rmi_gguf_tensor(g, name.c_str(), &type, dims, &nd, nullptr, nullptr));
  RMI_REQUIRE(type == RMI_GGML_Q8_0 && nd == 2 && dims[0] == n_in && dims[1] == n_out, RMI_ERR_FORMAT,
              "Invalid tensor %s: shape [%llu,%llu] type %d; expected [%zu,%zu] Q8_0", name.c_str(),
              (unsigned long long)dims[0], (unsigned long long)(nd > 1 ? dims[1] : 0), type, n_in, n_out);
  return rmi_weight_upload_gguf(ctx, g, name.c_str(), 0, (size_t)-1, out);
}

static void free_model(rmi_ctx* ctx, rmi_qwen3* m) {
  if (!m) return;
  for (auto& l : m->layers) {
    cudaFree(l.attn_norm); cudaFree(l.ffn_norm); cudaFree(l.q_norm); cudaFree(l.k_norm);
    if (l.wqkv) rmi_weight_free(ctx, l.wqkv);
    if (l.wo) rmi_weight_free(ctx, l.wo);
    if (l.wgu) rmi_weight_free(ctx, l.wgu);
    if (l.wdown) rmi_weight_free(ctx, l.wdown);
  }
  cudaFree(m->output_norm);
  if (m->output && m->output != m->token_embd) rmi_weight_free(ctx, m->output);
  if (m->token_embd) rmi_weight_free(ctx, m->token_embd);
  m->magic = 0;
  delete m;
}

static size_t wbytes(const rmi_weight* w) {
  size_t b = 0;
  rmi_weight_info(w, nullptr, nullptr, nullptr, &b);
  return b;
}

static int32_t load_model(rmi_ctx* ctx, const rmi_gguf* g, rmi_qwen3* m) {
  char arch[64];
  RMI_TRY(rmi_gguf_meta_str(g, "general.architecture", arch, sizeof(arch)));
  RMI_REQUIRE(strcmp(arch, "qwen3") == 0, RMI_ERR_UNSUPPORTED, "Unsupported architecture: %s (this path handles qwen3)", arch);
  auto u = [&](const char* key, size_t* v) -> int32_t {
    uint64_t t;
    RMI_TRY(rmi_gguf_meta_u64(g, (std::string("qwen3.") + key).c_str(), &t));
    *v = (size_t)t;
    return RMI_OK;
  };
  decode_dims& d = m->d;
  RMI_TRY(u("embedding_length", &d.n_embd));
  RMI_TRY(u("block_count", &d.n_layer));
  RMI_TRY(u("attention.head_count", &d.n_head));
  RMI_TRY(u("attention.head_count_kv", &d.n_head_kv));
  RMI_TRY(u("feed_forward_length", &d.n_ff));
  RMI_TRY(u("context_length", &m->n_ctx));
  RMI_REQUIRE(d.n_head > 0 && d.n_embd % d.n_head == 0, RMI_ERR_FORMAT, "Invalid qwen3 head shape");
  uint64_t t;
  d.hd = d.n_embd / d.n_head;
  if (rmi_gguf_meta_u64(g, "qwen3.attention.key_length", &t) == RMI_OK) d.hd = (size_t)t;
  if (rmi_gguf_meta_u64(g, "qwen3.attention.value_length", &t) == RMI_OK)
    RMI_REQUIRE((size_t)t == d.hd, RMI_ERR_UNSUPPORTED, "key_length != value_length is not handled");
  RMI_REQUIRE(d.n_head_kv > 0 && d.n_head % d.n_head_kv == 0 && d.hd % 2 == 0 && d.hd > 0, RMI_ERR_FORMAT,
              "Invalid qwen3 attention shape");
  double f;
  m->freq_base = 1000000.0f;
  if (rmi_gguf_meta_f64(g, "qwen3.rope.freq_base", &f) == RMI_OK) m->freq_base = (float)f;
  RMI_TRY(rmi_gguf_meta_f64(g, "qwen3.attention.layer_norm_rms_epsilon", &f));
  d.eps = (float)f;
  {
    int32_t type, nd;
    uint64_t dims[4];
    RMI_TRY(rmi_gguf_tensor(g, "token_embd.weight", &type, dims, &nd, nullptr, nullptr));
    RMI_REQUIRE(nd == 2 && dims[0] == d.n_embd, RMI_ERR_FORMAT, "Invalid tensor token_embd.weight");
    d.vocab = (size_t)dims[1];
    if (rmi_gguf_meta_u64(g, "qwen3.vocab_size", &t) == RMI_OK)
      RMI_REQUIRE((size_t)t == d.vocab, RMI_ERR_FORMAT, "qwen3.vocab_size does not match token_embd.weight");
  }
  const size_t nq = d.n_head * d.hd, nk = d.n_head_kv * d.hd;
  RMI_REQUIRE(d.n_embd % 32 == 0 && nq % 32 == 0 && nk % 32 == 0 && d.n_ff % 32 == 0, RMI_ERR_BAD_SHAPE,
              "Q8_0 needs every matmul width to be a multiple of 32");
  RMI_TRY(load_f32(ctx, g, "output_norm.weight", d.n_embd, &m->output_norm));
  RMI_TRY(load_q8(ctx, g, "token_embd.weight", d.n_embd, d.vocab, &m->token_embd));
  m->weight_bytes += wbytes(m->token_embd);
  m->output = m->token_embd;
  if (rmi_gguf_tensor(g, "output.weight", nullptr, nullptr, nullptr, nullptr, nullptr) == RMI_OK) {
    RMI_TRY(load_q8(ctx, g, "output.weight", d.n_embd, d.vocab, &m->output));
    m->weight_bytes += wbytes(m->output);
  }
  m->layers.resize(d.n_layer);
  for (auto& l : m->layers) memset(&l, 0, sizeof(l));
  for (size_t i = 0; i < d.n_layer; i++) {
    layer_weights& l = m->layers[i];
    const std::string p = "blk." + std::to_string(i) + ".";
    RMI_TRY(load_f32(ctx, g, p + "attn_norm.weight", d.n_embd, &l.attn_norm));
    RMI_TRY(load_f32(ctx, g, p + "ffn_norm.weight", d.n_embd, &l.ffn_norm));
    // has_qk_norm for "qwen3" (src/core/loader.rs:556)
    RMI_TRY(load_f32(ctx, g, p + "attn_q_norm.weight", d.hd, &l.q_norm));
    RMI_TRY(load_f32(ctx, g, p + "attn_k_norm.weight", d.hd, &l.k_norm));
    rmi_weight *wq = nullptr, *wk = nullptr, *wv = nullptr, *wqk = nullptr, *wg = nullptr, *wu = nullptr;
    int32_t st = load_q8(ctx, g, p + "attn_q.weight", d.n_embd, nq, &wq);
    if (st == RMI_OK) st = load_q8(ctx, g, p + "attn_k.weight", d.n_embd, nk, &wk);
    if (st == RMI_OK) st = load_q8(ctx, g, p + "attn_v.weight", d.n_embd, nk, &wv);
    // q, k and v share the activation: one v-stacked weight, one GEMV (fuse.rs:1-8)
    if (st == RMI_OK) st = rmi_weight_fuse_vstack(ctx, wq, wk, &wqk);
    if (st == RMI_OK) st = rmi_weight_fuse_vstack(ctx, wqk, wv, &l.wqkv);
    if (wq) rmi_weight_free(ctx, wq);
    if (wk) rmi_weight_free(ctx, wk);
    if (wv) rmi_weight_free(ctx, wv);
    if (wqk) rmi_weight_free(ctx, wqk);
    RMI_TRY(st);
    RMI_TRY(load_q8(ctx, g, p + "attn_output.weight", nq, d.n_embd, &l.wo));
    st = load_q8(ctx, g, p + "ffn_gate.weight", d.n_embd, d.n_ff, &wg);
    if (st == RMI_OK) st = load_q8(ctx, g, p + "ffn_up.weight", d.n_embd, d.n_ff, &wu);
    if (st == RMI_OK) st = rmi_weight_fuse_vstack(ctx, wg, wu, &l.wgu);
    if (wg) rmi_weight_free(ctx, wg);
    if (wu) rmi_weight_free(ctx, wu);
    RMI_TRY(st);
    RMI_TRY(load_q8(ctx, g, p + "ffn_down.weight", d.n_ff, d.n_embd, &l.wdown));
    m->weight_bytes += wbytes(l.wqkv) + wbytes(l.wo) + wbytes(l.wgu) + wbytes(l.wdown);
  }
  return RMI_OK;
}

extern "C" int32_t rmi_qwen3_load(rmi_ctx* ctx, const char* gguf_path, rmi_qwen3** out) {
  RMI_TRY(rmi_check_ctx(ctx));
  RMI_REQUIRE(out && gguf_path, RMI_ERR_BAD_HANDLE, "rmi_qwen3_load: null argument");
  *out = nullptr;
  rmi_gguf* g = nullptr;
  RMI_TRY(rmi_gguf_open(gguf_path, &g));
  rmi_qwen3* m = new (std::nothrow) rmi_qwen3();
  if (!m) {
    rmi_gguf_close(g);
    rmi_set_error("host allocation failed");
    return RMI_ERR_OOM;
  }
  m->magic = RMI_MODEL_MAGIC;
  m->output_norm = nullptr;
  m->token_embd = m->output = nullptr;
  m->weight_bytes = 0;
  memset(&m->d, 0, sizeof(m->d));
  int32_t st = load_model(ctx, g, m);
  std::string err = rmi_last_error();
  rmi_gguf_close(g);
  if (st != RMI_OK) {
    free_model(ctx, m);
    rmi_set_error("%s", err.c_str());
    return st;
  }
  *out = m;
  return RMI_OK;
}

extern "C" int32_t rmi_qwen3_free(rmi_ctx* ctx, rmi_qwen3* model) {
  RMI_TRY(rmi_check_ctx(ctx));
  RMI_TRY(check_model(model));
  RMI_CUDA_CHECK(cudaStreamSynchronize(ctx->stream));
  free_model(ctx, model);
  return RMI_OK;
}

extern "C" int32_t rmi_qwen3_config(const rmi_qwen3* m, size_t* n_embd, size_t* n_layer, size_t* n_head,
                                    size_t* n_head_kv, size_t* head_dim, size_t* n_ff, size_t* vocab) {
  RMI_TRY(check_model(m));
  if (n_embd) *n_embd = m->d.n_embd;
  if (n_layer) *n_layer = m->d.n_layer;
  if (n_head) *n_head = m->d.n_head;
  if (n_head_kv) *n_head_kv = m->d.n_head_kv;
  if (head_dim) *head_dim = m->d.hd;
  if (n_ff) *n_ff = m->d.n_ff;
  if (vocab) *vocab = m->d.vocab;
  return RMI_OK;
}

// ---------------------------------------------------------------- session

static void drop_graphs(rmi_session* s) {
  if (s->exec_body) cudaGraphExecDestroy(s->exec_body);
  if (s->exec_full) cudaGraphExecDestroy(s->exec_full);
  if (s->graph_body) cudaGraphDestroy(s->graph_body);
  if (s->graph_full) cudaGraphDestroy(s->graph_full);
  s->exec_body = s->exec_full = nullptr;
  s->graph_body = s->graph_full = nullptr;
}

static void free_session(rmi_session* s) {
  if (!s) return;
  drop_graphs(s);
  cudaFree(s->k_cache); cudaFree(s->v_cache); cudaFree(s->x); cudaFree(s->x2); cudaFree(s->qkv); cudaFree(s->proj);
  cudaFree(s->gu); cudaFree(s->logits); cudaFree(s->rope); cudaFree(s->q16); cudaFree(s->q8); cudaFree(s->attn_scratch);
  cudaFree(s->xs); cudaFree(s->prompts); cudaFree(s->gen); cudaFree(s->d_step); cudaFree(s->d_flag);
  cudaFree(s->attn_dbg);
  cudaFree(s->q32);
  cudaFree(s->k32_cache);
  cudaFree(s->v32_cache);
  cudaFree(s->argmax_v);
  cudaFree(s->argmax_i);
  cudaFree(s->pf_x); cudaFree(s->pf_xn); cudaFree(s->pf_qkv); cudaFree(s->pf_attn); cudaFree(s->pf_proj); cudaFree(s->pf_q16);
  s->magic = 0;
  delete s;
}

extern "C" int32_t rmi_session_free(rmi_ctx* ctx, rmi_session* s) {
  RMI_TRY(rmi_check_ctx(ctx));
  RMI_TRY(check_session(s));
  RMI_CUDA_CHECK(cudaStreamSynchronize(ctx->stream));
  free_session(s);
  return RMI_OK;
}

static bool is_cli_forward(int forward) { return forward != RMI_FORWARD_QWEN3_SESSION; }
static bool uses_f32_cache(int forward) {
  return forward == RMI_FORWARD_APP_TEXT_F32KV || forward == RMI_FORWARD_APP_LOGITS_F32KV;
}

extern "C" int32_t rmi_session_set_forward(rmi_ctx* ctx, rmi_session* s, int32_t forward) {
  RMI_TRY(rmi_check_ctx(ctx));
  RMI_TRY(check_session(s));
  RMI_REQUIRE(forward >= RMI_FORWARD_QWEN3_SESSION && forward <= RMI_FORWARD_APP_LOGITS_F32KV, RMI_ERR_UNSUPPORTED,
              "unknown forward variant %d", forward);
  std::lock_guard<std::mutex> lock(ctx->mu);
  if (s->forward == forward) return RMI_OK;
  RMI_CUDA_CHECK(cudaStreamSynchronize(ctx->stream));
  // the text loop gathers a column of V into a 512-entry array (src/app/text.rs:478) and panics beyond it
  RMI_REQUIRE(forward != RMI_FORWARD_APP_TEXT_F32KV || (s->d.capacity + 255) / 256 * 256 <= 512, RMI_ERR_BAD_SHAPE,
              "the text loop's F32 cache holds at most 512 positions, session capacity is %zu", s->d.capacity);
  // the CLI variants keep a score row per head in shared memory: refuse a capacity that cannot run before anything is captured
  RMI_REQUIRE(!is_cli_forward(forward) || cli_attention_smem_bytes(s->d, forward) <= ctx->smem_optin, RMI_ERR_UNSUPPORTED,
              "forward variant %d needs %zu B of shared memory per attention CTA at capacity %zu (limit %zu)", forward,
              cli_attention_smem_bytes(s->d, forward), s->d.capacity, ctx->smem_optin);
  if (uses_f32_cache(forward) && !s->k32_cache) {
    const size_t kv = s->d.batch * s->d.n_layer * s->d.capacity * s->d.n_head_kv * s->d.hd * 4;
    float *k32 = nullptr, *v32 = nullptr;
    if (cudaMalloc((void**)&k32, kv) != cudaSuccess || cudaMalloc((void**)&v32, kv) != cudaSuccess) {
      (void)cudaGetLastError();
      cudaFree(k32);
      rmi_set_error("allocation of the F32 caches (2 x %zu bytes) failed", kv);
      return RMI_ERR_OOM;
    }
    cudaMemset(k32, 0, kv);
    cudaMemset(v32, 0, kv);
    s->k32_cache = k32;
    s->v32_cache = v32;
  }
  drop_graphs(s);  // the captured step belongs to the other variant
  s->forward = forward;
  return RMI_OK;
}

#define SESSION_ALLOC(ptr, bytes)                                                             \
  do {                                                                                        \
    const size_t _n = (size_t)(bytes);                                                        \
    cudaError_t _e = cudaMalloc((void**)&(ptr), _n != 0 ? _n : 16);                           \
    if (_e != cudaSuccess) {                                                                  \
      (void)cudaGetLastError();                                                               \
      rmi_set_error("session allocation of %zu bytes failed: %s", _n, cudaGetErrorString(_e)); \
      free_session(s);                                                                        \
      return RMI_ERR_OOM;                                                                     \
    }                                                                                         \
  } while (0)

extern "C" int32_t rmi_session_create(rmi_ctx* ctx, const rmi_qwen3* model, size_t batch, size_t capacity,
                                      rmi_session** out) {
  RMI_TRY(rmi_check_ctx(ctx));
  RMI_TRY(check_model(model));
  RMI_REQUIRE(out != nullptr, RMI_ERR_BAD_HANDLE, "rmi_session_create: out is null");
  *out = nullptr;
  // src/models/qwen3.rs:442-447
  RMI_REQUIRE(capacity > 0 && capacity <= model->n_ctx, RMI_ERR_BAD_SHAPE,
              "Session capacity %zu must be within 1..=%zu", capacity, model->n_ctx);
  RMI_REQUIRE(batch > 0 && batch <= 65535, RMI_ERR_BAD_SHAPE, "batch %zu out of range", batch);
  rmi_session* s = new (std::nothrow) rmi_session();
  RMI_REQUIRE(s != nullptr, RMI_ERR_OOM, "host allocation failed");
  memset(s, 0, sizeof(*s));
  s->magic = RMI_SESSION_MAGIC;
  s->model = model;
  s->d = model->d;
  s->d.batch = batch;
  s->d.capacity = capacity;
  const decode_dims& d = s->d;
  // Attention kernel of the session forward: the cluster kernel (score rows and this CTA's K/V chunk in shared
  // memory) for few sequences, the single-CTA kernel for many; when the capacity's score rows do not fit in shared
  // memory (beyond a few thousand positions) the single-CTA kernel keeps them in a global scratch area instead, so
  // any capacity up to the model's context length is accepted (src/models/qwen3.rs:442-447).
  bool seq_attention = attention_seq_eligible(d), long_attention = false;
  if (seq_attention ? attention_seq_smem_bytes(d, false) > ctx->smem_optin : attention_smem_bytes(d) > ctx->smem_optin) {
    if (!attention_seq_shape_ok(d) || attention_seq_smem_bytes(d, true) > ctx->smem_optin) {
      rmi_set_error("capacity %zu needs %zu B of shared memory per attention CTA (limit %zu) and the head shape has no "
                    "long-context kernel", capacity, attention_smem_bytes(d), ctx->smem_optin);
      free_session(s);
      return RMI_ERR_UNSUPPORTED;
    }
    seq_attention = long_attention = true;
  }
  const size_t nq = d.n_head * d.hd, nk = d.n_head_kv * d.hd;
  const size_t max_n_in = nq > d.n_ff ? (nq > d.n_embd ? nq : d.n_embd) : (d.n_ff > d.n_embd ? d.n_ff : d.n_embd);
  const size_t kv = batch * d.n_layer * capacity * nk * 2;
  SESSION_ALLOC(s->k_cache, kv);
  SESSION_ALLOC(s->v_cache, kv);
  SESSION_ALLOC(s->x, batch * d.n_embd * 4);
  SESSION_ALLOC(s->x2, batch * d.n_embd * 4);
  SESSION_ALLOC(s->qkv, batch * (nq + 2 * nk) * 4);
  SESSION_ALLOC(s->proj, batch * d.n_embd * 4);
  SESSION_ALLOC(s->gu, batch * 2 * d.n_ff * 4);
  SESSION_ALLOC(s->logits, batch * d.vocab * 4);
  SESSION_ALLOC(s->rope, capacity * d.hd * 4);
  SESSION_ALLOC(s->q16, batch * nq * 2);
  SESSION_ALLOC(s->q8, batch * max_n_in);
  SESSION_ALLOC(s->xs, batch * (max_n_in / 32) * 4);
  SESSION_ALLOC(s->d_step, 4);
  SESSION_ALLOC(s->d_flag, 4);
  SESSION_ALLOC(s->attn_dbg, batch * nq * 4);
  SESSION_ALLOC(s->argmax_v, argmax_scratch_floats(batch) * 4);
  SESSION_ALLOC(s->argmax_i, argmax_scratch_floats(batch) * 4);
  s->forward = RMI_FORWARD_QWEN3_SESSION;
  s->k32_cache = s->v32_cache = nullptr;
  s->seq_attention = seq_attention;
  if (long_attention) SESSION_ALLOC(s->attn_scratch, attention_seq_scratch_bytes(d));
  SESSION_ALLOC(s->q32, batch * nq * 4);
  s->fused_norm = true;
  s->fused_qk = batch <= 4 && !seq_attention;  // measured: a loss at batch 32; the single-CTA kernel has no fused form
  for (const auto& l : model->layers) {
    s->fused_norm = s->fused_norm && q8_gemv_fused_norm_eligible(ctx, l.wqkv, batch) && q8_gemv_fused_norm_eligible(ctx, l.wgu, batch);
  }
  cudaMemset(s->k_cache, 0, kv);
  cudaMemset(s->v_cache, 0, kv);
  // rope_neox (src/ops/rope.rs:21-37): theta_0 = pos, theta_{i+1} = theta_i * base^(-2/d) in f32,
  // cos/sin from this host's libm so that the table equals what the CPU path evaluates.
  {
    std::vector<float> tab(capacity * d.hd);
    const float theta_scale = powf(model->freq_base, -2.0f / (float)d.hd);
    for (size_t pos = 0; pos < capacity; pos++) {
      float theta = (float)pos;
      for (size_t i = 0; i < d.hd / 2; i++) {
        tab[pos * d.hd + 2 * i] = cosf(theta);
        tab[pos * d.hd + 2 * i + 1] = sinf(theta);
        theta = theta * theta_scale;
      }
    }
    if (cudaMemcpy(s->rope, tab.data(), tab.size() * 4, cudaMemcpyHostToDevice) != cudaSuccess) {
      rmi_set_error("rope table upload failed");
      free_session(s);
      return RMI_ERR_CUDA;
    }
  }
  *out = s;
  return RMI_OK;
}

// One decode step for every sequence of the batch.  with_logits = false skips the output
// projection (prompt positions whose logits nobody reads).
static int32_t enqueue_step(rmi_ctx* ctx, rmi_session* s, size_t n_prompt, size_t n_gen, bool with_logits) {
  const rmi_qwen3* m = s->model;
  const decode_dims& d = s->d;
  const size_t B = d.batch, nq = d.n_head * d.hd, nk = d.n_head_kv * d.hd;
  RMI_TRY(launch_embed(ctx, m->token_embd, s->prompts, n_prompt, s->gen, n_gen, s->d_step, s->x, B));
  const float* pending = nullptr;  // residual branch still to be added to x
  float* xc = s->x;                  // current residual stream (ping-pongs with x2 on the fused path)
  float* xn = s->x2;
  for (size_t l = 0; l < d.n_layer; l++) {
    const layer_weights& w = m->layers[l];
    if (s->fused_norm) {
      // residual add + rms_norm + quantize happen inside the GEMV's prologue; it writes the updated x to xn
      RMI_TRY(launch_q8_gemv_fused_norm(ctx, w.wqkv, xc, pending, w.attn_norm, d.eps, xn, B, s->qkv, nq + 2 * nk));
      std::swap(xc, xn);
    } else {
      RMI_TRY(launch_rmsnorm_quant(ctx, xc, pending, w.attn_norm, d.n_embd, d.eps, s->q8, s->xs, B));
      RMI_TRY(launch_q8_gemv(ctx, w.wqkv, s->q8, s->xs, B, s->qkv, nq + 2 * nk, 0, nq + 2 * nk));
    }
    if (uses_f32_cache(s->forward)) {
      // src/app/text.rs:393-405, :458-496: f32 query and F32 cache, padded soft-max, one dot per output element;
      // src/app/logits.rs:513-560: the same scores and soft-max, then a sequential chain per output element
      RMI_TRY(launch_qk_norm_rope_kv(ctx, d, s->qkv, w.q_norm, w.k_norm, s->rope, s->d_step, s->q16, s->k_cache,
                                     s->v_cache, l, s->q32, s->k32_cache, s->v32_cache));
      RMI_TRY(launch_attention_f32kv(ctx, d, s->q32, s->k32_cache, s->v32_cache, s->d_step, l, s->attn_dbg, s->q8, s->xs,
                                     s->forward == RMI_FORWARD_APP_LOGITS_F32KV));
    } else if (s->forward == RMI_FORWARD_APP_LOGITS) {
      // src/app/logits.rs:474-512: f32 query x F16 cache scores, soft-max, sequential chain per output element
      RMI_TRY(launch_qk_norm_rope_kv(ctx, d, s->qkv, w.q_norm, w.k_norm, s->rope, s->d_step, s->q16, s->k_cache,
                                     s->v_cache, l, s->q32));
      RMI_TRY(launch_attention_scores_f16kv(ctx, d, s->q32, s->k_cache, s->v_cache, s->d_step, l, s->attn_dbg, s->q8, s->xs));
    } else if (s->forward == RMI_FORWARD_APP_TEXT) {
      // src/app/text.rs:257-648: f32 query, online soft-max over the F16 cache
      RMI_TRY(launch_qk_norm_rope_kv(ctx, d, s->qkv, w.q_norm, w.k_norm, s->rope, s->d_step, s->q16, s->k_cache,
                                     s->v_cache, l, s->q32));
      RMI_TRY(launch_attention_online(ctx, d, s->q32, s->k_cache, s->v_cache, s->d_step, l, s->attn_dbg, s->q8, s->xs));
    } else if (s->fused_qk) {
      // q/k norm, rotation and the cache write happen inside the attention kernel
      RMI_TRY(launch_attention(ctx, d, s->q16, s->k_cache, s->v_cache, s->d_step, l, s->attn_dbg, s->q8, s->xs, s->qkv,
                               w.q_norm, w.k_norm, s->rope));
    } else {
      RMI_TRY(launch_qk_norm_rope_kv(ctx, d, s->qkv, w.q_norm, w.k_norm, s->rope, s->d_step, s->q16, s->k_cache,
                                     s->v_cache, l));
      if (s->seq_attention)
        RMI_TRY(launch_attention_seq(ctx, d, s->q16, s->k_cache, s->v_cache, s->d_step, l, s->attn_dbg, s->q8, s->xs, s->attn_scratch));
      else
        RMI_TRY(launch_attention(ctx, d, s->q16, s->k_cache, s->v_cache, s->d_step, l, s->attn_dbg, s->q8, s->xs));
    }
    RMI_TRY(launch_q8_gemv(ctx, w.wo, s->q8, s->xs, B, s->proj, d.n_embd, 0, d.n_embd));
    if (s->fused_norm) {
      RMI_TRY(launch_q8_gemv_fused_norm(ctx, w.wgu, xc, s->proj, w.ffn_norm, d.eps, xn, B, s->gu, 2 * d.n_ff));
      std::swap(xc, xn);
    } else {
      RMI_TRY(launch_rmsnorm_quant(ctx, xc, s->proj, w.ffn_norm, d.n_embd, d.eps, s->q8, s->xs, B));
      RMI_TRY(launch_q8_gemv(ctx, w.wgu, s->q8, s->xs, B, s->gu, 2 * d.n_ff, 0, 2 * d.n_ff));
    }
    RMI_TRY(launch_silu_mul_quantize(ctx, s->gu, s->gu + d.n_ff, 2 * d.n_ff, B, d.n_ff, nullptr, s->q8, s->xs));
    RMI_TRY(launch_q8_gemv(ctx, w.wdown, s->q8, s->xs, B, s->proj, d.n_embd, 0, d.n_embd));
    pending = s->proj;
  }
  // x += last down projection; output norm; logits; greedy token.  After an even number of swaps the
  // stream is back in s->x, which is what rmi_session_read_hidden returns.
  RMI_TRY(launch_rmsnorm_quant(ctx, xc, pending, m->output_norm, d.n_embd, d.eps, s->q8, s->xs, B));
  if (with_logits) {
    RMI_TRY(launch_q8_gemv(ctx, m->output, s->q8, s->xs, B, s->logits, d.vocab, 0, d.vocab));
    RMI_TRY(launch_argmax(ctx, s->logits, d.vocab, s->d_step, n_prompt, s->gen, n_gen, s->d_flag, B, s->argmax_v, s->argmax_i,
                          s->forward == RMI_FORWARD_APP_TEXT || s->forward == RMI_FORWARD_APP_TEXT_F32KV));
  }
  return launch_step_inc(ctx, s->d_step);
}

static int32_t build_graphs(rmi_ctx* ctx, rmi_session* s, size_t n_prompt, size_t n_gen) {
  if (s->exec_full && s->graph_n_prompt == n_prompt && s->graph_n_gen == n_gen && s->graph_sem == ctx->sem &&
      s->graph_stream == ctx->stream)
    return RMI_OK;
  drop_graphs(s);
  for (int which = 0; which < 2; which++) {
    RMI_CUDA_CHECK(cudaStreamBeginCapture(ctx->stream, cudaStreamCaptureModeThreadLocal));
    // programmatic dependent launch along the step's kernel chain: the next kernel's weight copy
    // overlaps the tail of the current one.  Measured gain for small batches only (large grids lose).
    const bool pdl_before = ctx->pdl;
    ctx->pdl = s->d.batch <= 16;  // measured on the 0.6B step: +6 % at batch 8, +3 % at 16, -8 % at 32
    int32_t st = enqueue_step(ctx, s, n_prompt, n_gen, which == 1);
    ctx->pdl = pdl_before;
    cudaGraph_t g = nullptr;
    cudaError_t e = cudaStreamEndCapture(ctx->stream, &g);
    if (st != RMI_OK) {
      if (g) cudaGraphDestroy(g);
      return st;
    }
    if (e != cudaSuccess) {
      rmi_set_error("graph capture of the decode step failed: %s", cudaGetErrorString(e));
      return RMI_ERR_CUDA;
    }
    cudaGraphExec_t ex = nullptr;
    e = cudaGraphInstantiate(&ex, g, 0);
    if (e != cudaSuccess) {
      cudaGraphDestroy(g);
      rmi_set_error("graph instantiation failed: %s", cudaGetErrorString(e));
      return RMI_ERR_CUDA;
    }
    if (which == 0) {
      s->graph_body = g;
      s->exec_body = ex;
    } else {
      s->graph_full = g;
      s->exec_full = ex;
    }
  }
  s->graph_n_prompt = n_prompt;
  s->graph_n_gen = n_gen;
  s->graph_sem = ctx->sem;
  s->graph_stream = ctx->stream;
  return RMI_OK;
}

extern "C" int32_t rmi_session_set_prefill(rmi_ctx* ctx, rmi_session* s, int32_t mode) {
  RMI_TRY(rmi_check_ctx(ctx));
  RMI_TRY(check_session(s));
  RMI_REQUIRE(mode >= RMI_PREFILL_BATCHED && mode <= RMI_PREFILL_BATCHED_TENSOR, RMI_ERR_UNSUPPORTED, "unknown prefill mode %d",
              mode);
  std::lock_guard<std::mutex> lock(ctx->mu);
  s->prefill_mode = mode;
  return RMI_OK;
}

// Prompt positions 0..P-1 of every sequence as rows through each operator (see prefill.cu).  Only the default
// forward is batched; the app-loop variants keep the token loop.
static const size_t PREFILL_MIN_POSITIONS = 16;
static const size_t PREFILL_MAX_ROWS = 8192;

static bool prefill_batched(const rmi_ctx* ctx, const rmi_session* s, size_t P) {
  return s->prefill_mode != RMI_PREFILL_TOKEN_LOOP && s->forward == RMI_FORWARD_QWEN3_SESSION && P >= PREFILL_MIN_POSITIONS &&
         prefill_supported(ctx, s->d, P);
}

static int32_t ensure_prefill_buffers(rmi_session* s, size_t rows) {
  if (s->pf_rows >= rows) return RMI_OK;
  const decode_dims& d = s->d;
  const size_t nq = d.n_head * d.hd, nk = d.n_head_kv * d.hd;
  cudaFree(s->pf_x); cudaFree(s->pf_xn); cudaFree(s->pf_qkv); cudaFree(s->pf_attn); cudaFree(s->pf_proj); cudaFree(s->pf_q16);
  s->pf_x = s->pf_xn = s->pf_qkv = s->pf_attn = s->pf_proj = nullptr;
  s->pf_q16 = nullptr;
  s->pf_rows = 0;
  cudaError_t e = cudaMalloc((void**)&s->pf_x, rows * d.n_embd * 4);
  if (e == cudaSuccess) e = cudaMalloc((void**)&s->pf_xn, rows * d.n_embd * 4);
  if (e == cudaSuccess) e = cudaMalloc((void**)&s->pf_qkv, rows * (nq + 2 * nk) * 4);
  if (e == cudaSuccess) e = cudaMalloc((void**)&s->pf_attn, rows * nq * 4);
  if (e == cudaSuccess) e = cudaMalloc((void**)&s->pf_proj, rows * d.n_embd * 4);
  if (e == cudaSuccess) e = cudaMalloc((void**)&s->pf_q16, rows * nq * 2);
  if (e != cudaSuccess) {
    (void)cudaGetLastError();
    rmi_set_error("allocation of the prefill buffers (%zu rows) failed: %s", rows, cudaGetErrorString(e));
    return RMI_ERR_OOM;
  }
  s->pf_rows = rows;
  return RMI_OK;
}

static size_t prefill_group_seqs(const rmi_session* s, size_t P) {
  const size_t per_group = P >= PREFILL_MAX_ROWS ? 1 : PREFILL_MAX_ROWS / P;
  return s->d.batch < per_group ? s->d.batch : per_group;
}

static bool prefill_on_tensor_cores(const rmi_ctx* ctx, const rmi_session* s) {
  return ctx->sem != RMI_SEM_AVX2 || s->prefill_mode == RMI_PREFILL_BATCHED_TENSOR;
}

// Everything that allocates (row buffers, the context's matmul scratch, tcgen05 weight layouts), done before the
// timed region of a generate call.
static int32_t prepare_prefill(rmi_ctx* ctx, rmi_session* s, size_t P) {
  const rmi_qwen3* m = s->model;
  const decode_dims& d = s->d;
  const size_t rows = prefill_group_seqs(s, P) * P;
  RMI_TRY(ensure_prefill_buffers(s, rows));
  const size_t nq = d.n_head * d.hd;
  const size_t widest = nq > d.n_ff ? (nq > d.n_embd ? nq : d.n_embd) : (d.n_ff > d.n_embd ? d.n_ff : d.n_embd);
  const size_t rows_pad = (rows + 127) / 128 * 128, wide_pad = (widest + 127) / 128 * 128;
  void* unused;
  RMI_TRY(rmi_scratch(ctx, 0, rows_pad * wide_pad, &unused));                 // quantized rows (row-major or images)
  RMI_TRY(rmi_scratch(ctx, 1, rows_pad * (wide_pad / 32) * 4, &unused));      // their scales
  RMI_TRY(rmi_scratch(ctx, 3, rows_pad * wide_pad, &unused));
  RMI_TRY(rmi_scratch(ctx, 4, rows_pad * (wide_pad / 32) * 4, &unused));
  if (prefill_on_tensor_cores(ctx, s)) {
    for (const auto& l : m->layers) {
      RMI_TRY(ensure_umma_layout(ctx, l.wqkv));
      RMI_TRY(ensure_umma_layout(ctx, l.wo));
      RMI_TRY(ensure_umma_layout(ctx, l.wgu, true));
      RMI_TRY(ensure_umma_layout(ctx, l.wdown));
    }
  } else {
    RMI_TRY(rmi_scratch(ctx, 2, rows * 2 * d.n_ff * 4, &unused));             // gate | up rows of the CUDA-core FFN
  }
  return RMI_OK;
}

static int32_t enqueue_prefill(rmi_ctx* ctx, rmi_session* s, size_t n_prompt, size_t P) {
  const rmi_qwen3* m = s->model;
  const decode_dims& d = s->d;
  const size_t nq = d.n_head * d.hd;
  const size_t group_seqs = prefill_group_seqs(s, P);
  RMI_TRY(ensure_prefill_buffers(s, group_seqs * P));
  // AVX2 semantics: the eight-lane accumulation order is reproduced bit for bit by the CUDA-core kernels, which
  // keeps every cache row identical to the token loop's; RMI_PREFILL_BATCHED_TENSOR trades that for the tensor cores
  const bool exact_before = ctx->prefill_exact;
  if (ctx->sem == RMI_SEM_AVX2) ctx->prefill_exact = s->prefill_mode != RMI_PREFILL_BATCHED_TENSOR;
  int32_t st = RMI_OK;
  for (size_t b0 = 0; b0 < d.batch && st == RMI_OK; b0 += group_seqs) {
    const size_t nb = d.batch - b0 < group_seqs ? d.batch - b0 : group_seqs, rows = nb * P;
    st = launch_embed_rows(ctx, m->token_embd, s->prompts, n_prompt, P, b0, rows, s->pf_x);
    const float* pending = nullptr;
    for (size_t l = 0; l < d.n_layer && st == RMI_OK; l++) {
      const layer_weights& w = m->layers[l];
      st = launch_rmsnorm_rows(ctx, s->pf_x, pending, w.attn_norm, d.n_embd, d.eps, s->pf_xn, rows);
      if (st == RMI_OK) st = matmul_q8_0_device(ctx, w.wqkv, s->pf_xn, rows, s->pf_qkv);
      if (st == RMI_OK)
        st = launch_qk_norm_rope_kv_rows(ctx, d, s->pf_qkv, w.q_norm, w.k_norm, s->rope, P, b0, rows, s->pf_q16, s->k_cache,
                                         s->v_cache, l);
      if (l + 1 == d.n_layer) break;  // the last layer only has to fill its cache rows: nobody reads these positions' output
      if (st == RMI_OK) st = launch_attention_prefill(ctx, d, s->pf_q16, s->k_cache, s->v_cache, l, P, b0, nb, s->pf_attn);
      if (st == RMI_OK) st = matmul_q8_0_device(ctx, w.wo, s->pf_attn, rows, s->pf_proj);
      if (st == RMI_OK) st = launch_rmsnorm_rows(ctx, s->pf_x, s->pf_proj, w.ffn_norm, d.n_embd, d.eps, s->pf_xn, rows);
      if (st == RMI_OK) st = ffn_device(ctx, w.wgu, w.wdown, s->pf_xn, rows, s->pf_proj);
      pending = s->pf_proj;
    }
  }
  ctx->prefill_exact = exact_before;
  RMI_TRY(st);
  (void)nq;
  return launch_set_step(ctx, s->d_step, (int)P);
}

extern "C" int32_t rmi_session_generate(rmi_ctx* ctx, rmi_session* s, const uint32_t* prompts, size_t n_prompt,
                                        size_t n_gen, uint32_t* out_tokens, float* prefill_ms, float* gen_ms) {
  RMI_TRY(rmi_check_ctx(ctx));
  RMI_TRY(check_session(s));
  const decode_dims& d = s->d;
  RMI_REQUIRE(prompts != nullptr && n_prompt > 0, RMI_ERR_BAD_SHAPE, "Cannot generate from an empty prompt");
  // src/models/qwen3.rs:569-578
  RMI_REQUIRE(n_prompt + n_gen <= d.capacity, RMI_ERR_BAD_SHAPE, "Generation requires capacity %zu; session has %zu",
              n_prompt + n_gen, d.capacity);
  RMI_REQUIRE(n_gen == 0 || out_tokens != nullptr, RMI_ERR_BAD_HANDLE, "out_tokens is null");
  for (size_t i = 0; i < d.batch * n_prompt; i++)
    RMI_REQUIRE(prompts[i] < d.vocab, RMI_ERR_BAD_SHAPE, "token id %u outside the vocabulary (%zu)", prompts[i], d.vocab);
  std::lock_guard<std::mutex> lock(ctx->mu);
  s->step_mode = false;
  if (s->prompts_cap < d.batch * n_prompt) {
    cudaFree(s->prompts);
    s->prompts = nullptr;
    RMI_CUDA_CHECK(cudaMalloc(&s->prompts, d.batch * n_prompt * 4));
    s->prompts_cap = d.batch * n_prompt;
    drop_graphs(s);
  }
  if (s->gen_cap < d.batch * (n_gen ? n_gen : 1)) {
    cudaFree(s->gen);
    s->gen = nullptr;
    RMI_CUDA_CHECK(cudaMalloc(&s->gen, d.batch * (n_gen ? n_gen : 1) * 4));
    s->gen_cap = d.batch * (n_gen ? n_gen : 1);
    drop_graphs(s);
  }
  RMI_CUDA_CHECK(cudaMemcpyAsync(s->prompts, prompts, d.batch * n_prompt * 4, cudaMemcpyHostToDevice, ctx->stream));
  RMI_CUDA_CHECK(cudaMemsetAsync(s->gen, 0, s->gen_cap * 4, ctx->stream));
  RMI_CUDA_CHECK(cudaMemsetAsync(s->d_step, 0, 4, ctx->stream));
  RMI_CUDA_CHECK(cudaMemsetAsync(s->d_flag, 0, 4, ctx->stream));
  RMI_CUDA_CHECK(cudaStreamSynchronize(ctx->stream));
  RMI_TRY(build_graphs(ctx, s, n_prompt, n_gen));
  const bool batched = n_prompt >= 2 && prefill_batched(ctx, s, n_prompt - 1);
  if (batched) {
    RMI_TRY(prepare_prefill(ctx, s, n_prompt - 1));
    RMI_CUDA_CHECK(cudaStreamSynchronize(ctx->stream));
  }
  cudaEvent_t e0, e1, e2;
  RMI_CUDA_CHECK(cudaEventCreate(&e0));
  RMI_CUDA_CHECK(cudaEventCreate(&e1));
  RMI_CUDA_CHECK(cudaEventCreate(&e2));
  // steps 0 .. n_prompt+n_gen-2 (src/models/qwen3.rs:118-126); logits from step n_prompt-1 on
  const size_t steps = n_prompt + n_gen - 1;
  // kernels per graph: the GEMV launcher issues one kernel per pass of 8/4/2/1 activation rows
  uint64_t passes = 0;
  for (size_t rem = d.batch, p2 = 8; p2 >= 1; p2 >>= 1)
    if (rem >= p2) {
      passes++;
      rem %= p2;
    }
  const uint64_t per_layer = 4 * passes + 1 + (s->fused_norm ? 0 : 2) + ((s->fused_qk && !is_cli_forward(s->forward)) ? 0 : 1) + 1;
  const uint64_t launches_per_body = 3 + d.n_layer * per_layer, launches_full = launches_per_body + passes + 2;
  RMI_CUDA_CHECK(cudaEventRecord(e0, ctx->stream));
  cudaError_t ce = cudaSuccess;
  size_t first_step = 0;
  if (batched) {
    const int32_t pst = enqueue_prefill(ctx, s, n_prompt, n_prompt - 1);
    if (pst != RMI_OK) {
      cudaStreamSynchronize(ctx->stream);
      cudaEventDestroy(e0);
      cudaEventDestroy(e1);
      cudaEventDestroy(e2);
      return pst;
    }
    first_step = n_prompt - 1;
  }
  for (size_t st = first_step; st < steps && ce == cudaSuccess; st++) {
    if (st == n_prompt - 1) ce = cudaEventRecord(e1, ctx->stream);
    const bool full = st + 1 >= n_prompt && n_gen > 0;
    if (ce == cudaSuccess) ce = cudaGraphLaunch(full ? s->exec_full : s->exec_body, ctx->stream);
    ctx->launches.fetch_add(full ? launches_full : launches_per_body, std::memory_order_relaxed);
  }
  if (ce == cudaSuccess && steps < n_prompt) ce = cudaEventRecord(e1, ctx->stream);
  if (ce == cudaSuccess) ce = cudaEventRecord(e2, ctx->stream);
  if (ce == cudaSuccess) ce = cudaStreamSynchronize(ctx->stream);
  float t_pre = 0.0f, t_gen = 0.0f;
  if (ce == cudaSuccess) {
    cudaEventElapsedTime(&t_pre, e0, e1);
    cudaEventElapsedTime(&t_gen, e1, e2);
  }
  cudaEventDestroy(e0);
  cudaEventDestroy(e1);
  cudaEventDestroy(e2);
  if (ce != cudaSuccess) {
    rmi_set_error("decode step failed: %s", cudaGetErrorString(ce));
    return RMI_ERR_CUDA;
  }
  if (prefill_ms) *prefill_ms = t_pre;
  if (gen_ms) *gen_ms = t_gen;
  int flag = 0;
  RMI_CUDA_CHECK(cudaMemcpy(&flag, s->d_flag, 4, cudaMemcpyDeviceToHost));
  if (n_gen) RMI_CUDA_CHECK(cudaMemcpy(out_tokens, s->gen, d.batch * n_gen * 4, cudaMemcpyDeviceToHost));
  RMI_REQUIRE(flag == 0, RMI_ERR_NONFINITE, "Cannot sample non-finite logits");
  return RMI_OK;
}

// ---------------------------------------------------------------- per-step interface
//
// The host feeds one token per sequence and position and samples itself.  Tokens are kept in a device ring
// gen[batch][capacity + 1]: the step at position p reads column p and its greedy choice lands in column p + 1
// (where the next step reads it unless the host writes its own token there first).

static int32_t ensure_step_mode(rmi_ctx* ctx, rmi_session* s) {
  const decode_dims& d = s->d;
  const size_t n_gen = d.capacity + 1;
  if (s->gen_cap < d.batch * n_gen) {
    RMI_CUDA_CHECK(cudaStreamSynchronize(ctx->stream));
    cudaFree(s->gen);
    s->gen = nullptr;
    s->gen_cap = 0;
    RMI_CUDA_CHECK(cudaMalloc(&s->gen, d.batch * n_gen * 4));
    s->gen_cap = d.batch * n_gen;
    drop_graphs(s);
  }
  return build_graphs(ctx, s, 0, n_gen);
}

extern "C" int32_t rmi_session_reset(rmi_ctx* ctx, rmi_session* s) {
  RMI_TRY(rmi_check_ctx(ctx));
  RMI_TRY(check_session(s));
  std::lock_guard<std::mutex> lock(ctx->mu);
  RMI_TRY(ensure_step_mode(ctx, s));
  RMI_CUDA_CHECK(cudaMemsetAsync(s->gen, 0, s->gen_cap * 4, ctx->stream));
  RMI_CUDA_CHECK(cudaMemsetAsync(s->d_step, 0, 4, ctx->stream));
  RMI_CUDA_CHECK(cudaMemsetAsync(s->d_flag, 0, 4, ctx->stream));
  s->pos = 0;
  s->step_mode = true;
  return RMI_OK;
}

extern "C" int32_t rmi_session_position(const rmi_session* s, size_t* position) {
  RMI_TRY(check_session(s));
  RMI_REQUIRE(position != nullptr, RMI_ERR_BAD_HANDLE, "rmi_session_position: null argument");
  *position = s->step_mode ? s->pos : 0;
  return RMI_OK;
}

extern "C" int32_t rmi_session_prefill(rmi_ctx* ctx, rmi_session* s, const uint32_t* tokens, size_t n_tokens) {
  RMI_TRY(rmi_check_ctx(ctx));
  RMI_TRY(check_session(s));
  const decode_dims& d = s->d;
  RMI_REQUIRE(s->step_mode, RMI_ERR_BAD_HANDLE, "call rmi_session_reset before the per-step interface");
  RMI_REQUIRE(s->pos == 0, RMI_ERR_BAD_SHAPE, "rmi_session_prefill starts at position 0; the session is at %zu", s->pos);
  RMI_REQUIRE(tokens != nullptr || n_tokens == 0, RMI_ERR_BAD_HANDLE, "rmi_session_prefill: null tokens");
  RMI_REQUIRE(n_tokens <= d.capacity, RMI_ERR_BAD_SHAPE, "%zu positions exceed the session capacity %zu", n_tokens, d.capacity);
  for (size_t i = 0; i < d.batch * n_tokens; i++)
    RMI_REQUIRE(tokens[i] < d.vocab, RMI_ERR_BAD_SHAPE, "token id %u outside the vocabulary (%zu)", tokens[i], d.vocab);
  if (n_tokens == 0) return RMI_OK;
  std::lock_guard<std::mutex> lock(ctx->mu);
  const size_t n_gen = d.capacity + 1;
  RMI_CUDA_CHECK(cudaMemcpy2DAsync(s->gen, n_gen * 4, tokens, n_tokens * 4, n_tokens * 4, d.batch, cudaMemcpyHostToDevice,
                                   ctx->stream));
  if (prefill_batched(ctx, s, n_tokens)) {
    RMI_TRY(prepare_prefill(ctx, s, n_tokens));
    // the rows kernels read token (b, p) at prompts[b * stride + p]: the ring with its row stride
    uint32_t* saved = s->prompts;
    s->prompts = s->gen;
    const int32_t st = enqueue_prefill(ctx, s, n_gen, n_tokens);
    s->prompts = saved;
    RMI_TRY(st);
  } else {
    for (size_t p = 0; p < n_tokens; p++) {
      RMI_CUDA_CHECK(cudaGraphLaunch(s->exec_body, ctx->stream));
      ctx->launches.fetch_add(1, std::memory_order_relaxed);
    }
  }
  s->pos = n_tokens;
  return RMI_OK;
}

extern "C" int32_t rmi_session_step(rmi_ctx* ctx, rmi_session* s, const uint32_t* tokens, uint32_t* next_tokens,
                                    float* logits_opt) {
  RMI_TRY(rmi_check_ctx(ctx));
  RMI_TRY(check_session(s));
  const decode_dims& d = s->d;
  RMI_REQUIRE(s->step_mode, RMI_ERR_BAD_HANDLE, "call rmi_session_reset before the per-step interface");
  RMI_REQUIRE(s->pos < d.capacity, RMI_ERR_BAD_SHAPE, "session is full (%zu positions)", d.capacity);
  RMI_REQUIRE(tokens != nullptr, RMI_ERR_BAD_HANDLE, "rmi_session_step: null tokens");
  for (size_t b = 0; b < d.batch; b++)
    RMI_REQUIRE(tokens[b] < d.vocab, RMI_ERR_BAD_SHAPE, "token id %u outside the vocabulary (%zu)", tokens[b], d.vocab);
  std::lock_guard<std::mutex> lock(ctx->mu);
  const size_t n_gen = d.capacity + 1;
  RMI_CUDA_CHECK(cudaMemcpy2DAsync(s->gen + s->pos, n_gen * 4, tokens, 4, 4, d.batch, cudaMemcpyHostToDevice, ctx->stream));
  RMI_CUDA_CHECK(cudaGraphLaunch(s->exec_full, ctx->stream));
  ctx->launches.fetch_add(1, std::memory_order_relaxed);
  if (next_tokens)
    RMI_CUDA_CHECK(cudaMemcpy2DAsync(next_tokens, 4, s->gen + s->pos + 1, n_gen * 4, 4, d.batch, cudaMemcpyDeviceToHost,
                                     ctx->stream));
  if (logits_opt)
    RMI_CUDA_CHECK(cudaMemcpyAsync(logits_opt, s->logits, d.batch * d.vocab * 4, cudaMemcpyDeviceToHost, ctx->stream));
  int flag = 0;
  RMI_CUDA_CHECK(cudaMemcpyAsync(&flag, s->d_flag, 4, cudaMemcpyDeviceToHost, ctx->stream));
  RMI_CUDA_CHECK(cudaStreamSynchronize(ctx->stream));
  s->pos += 1;
  RMI_REQUIRE(flag == 0, RMI_ERR_NONFINITE, "Cannot sample non-finite logits");
  return RMI_OK;
}

extern "C" int32_t rmi_session_read_hidden(rmi_ctx* ctx, rmi_session* s, float* hidden) {
  RMI_TRY(rmi_check_ctx(ctx));
  RMI_TRY(check_session(s));
  RMI_CUDA_CHECK(cudaStreamSynchronize(ctx->stream));
  RMI_CUDA_CHECK(cudaMemcpy(hidden, s->x, s->d.batch * s->d.n_embd * 4, cudaMemcpyDeviceToHost));
  return RMI_OK;
}

extern "C" int32_t rmi_session_read_logits(rmi_ctx* ctx, rmi_session* s, float* logits) {
  RMI_TRY(rmi_check_ctx(ctx));
  RMI_TRY(check_session(s));
  RMI_CUDA_CHECK(cudaStreamSynchronize(ctx->stream));
  RMI_CUDA_CHECK(cudaMemcpy(logits, s->logits, s->d.batch * s->d.vocab * 4, cudaMemcpyDeviceToHost));
  return RMI_OK;
}
