// C ABI glue of librmi_cuda.so: context, device memory, weight upload / v-stack, and the
// host-pointer and device-pointer entry points of the Q8_0 path.
#include <stdarg.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <new>

#include "common.cuh"
#include "kernels.cuh"

// ---------------------------------------------------------------- errors

static thread_local char g_err[512] = "";

void rmi_set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
}

extern "C" const char* rmi_last_error(void) { return g_err; }

int32_t rmi_check_ctx(rmi_ctx* ctx) {
  RMI_REQUIRE(ctx != nullptr && ctx->magic == RMI_CTX_MAGIC, RMI_ERR_BAD_HANDLE, "invalid rmi_ctx handle");
  cudaError_t e = cudaSetDevice(ctx->device);
  if (e != cudaSuccess) {
    rmi_set_error("cudaSetDevice(%d) failed: %s", ctx->device, cudaGetErrorString(e));
    return RMI_ERR_CUDA;
  }
  return RMI_OK;
}

int32_t rmi_check_weight(const rmi_weight* w, int ggml_type) {
  RMI_REQUIRE(w != nullptr && w->magic == RMI_WEIGHT_MAGIC, RMI_ERR_BAD_HANDLE, "invalid rmi_weight handle");
  RMI_REQUIRE(ggml_type < 0 || w->ggml_type == ggml_type, RMI_ERR_UNSUPPORTED,
              "weight has ggml type %d, this entry point needs %d", w->ggml_type, ggml_type);
  return RMI_OK;
}

int32_t rmi_post_launch(rmi_ctx* ctx, const char* what) {
  ctx->launches.fetch_add(1, std::memory_order_relaxed);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    rmi_set_error("launch of %s failed: %s", what, cudaGetErrorString(e));
    return RMI_ERR_CUDA;
  }
  return RMI_OK;
}

int32_t rmi_check_dev_status(rmi_ctx* ctx, const char* what) {
  RMI_CUDA_CHECK(cudaMemcpyAsync(ctx->h_status, ctx->d_status, sizeof(rmi_dev_status), cudaMemcpyDeviceToHost, ctx->stream));
  RMI_CUDA_CHECK(cudaStreamSynchronize(ctx->stream));
  if (ctx->h_status->code != 0) {
    rmi_set_error("%s: device-side wait gave up (site %d, detail %d)", what, ctx->h_status->where,
                  ctx->h_status->detail);
    RMI_CUDA_CHECK(cudaMemsetAsync(ctx->d_status, 0, RMI_STATUS_CLEAR_BYTES, ctx->stream));
    return RMI_ERR_TIMEOUT;
  }
  return RMI_OK;
}

int32_t rmi_scratch(rmi_ctx* ctx, int slot, size_t bytes, void** out) {
  if (bytes == 0) bytes = 16;
  if (ctx->scratch_bytes[slot] < bytes) {
    if (ctx->scratch[slot]) {
      // the old buffer may still be read by enqueued work
      RMI_CUDA_CHECK(cudaStreamSynchronize(ctx->stream));
      RMI_CUDA_CHECK(cudaFree(ctx->scratch[slot]));
      ctx->scratch[slot] = nullptr;
      ctx->scratch_bytes[slot] = 0;
    }
    size_t cap = (bytes + (1 << 20) - 1) & ~((size_t)(1 << 20) - 1);
    cudaError_t e = cudaMalloc(&ctx->scratch[slot], cap);
    if (e != cudaSuccess) {
      (void)cudaGetLastError();
      rmi_set_error("device allocation of %zu bytes failed: %s", cap, cudaGetErrorString(e));
      return RMI_ERR_OOM;
    }
    ctx->scratch_bytes[slot] = cap;
  }
  *out = ctx->scratch[slot];
  return RMI_OK;
}

// ---------------------------------------------------------------- per-kernel timing

int rmi_prof_begin(rmi_ctx* ctx, const char* tag) {
  if (!ctx->prof_on || ctx->prof.size() >= 16384) return -1;
  rmi_prof_rec r;
  r.tag = tag;
  if (cudaEventCreate(&r.a) != cudaSuccess) return -1;
  if (cudaEventCreate(&r.b) != cudaSuccess) {
    cudaEventDestroy(r.a);
    return -1;
  }
  cudaEventRecord(r.a, ctx->stream);
  ctx->prof.push_back(r);
  return (int)ctx->prof.size() - 1;
}

void rmi_prof_end(rmi_ctx* ctx, int idx) {
  if (idx >= 0) cudaEventRecord(ctx->prof[idx].b, ctx->stream);
}

static void prof_clear(rmi_ctx* ctx) {
  for (auto& r : ctx->prof) {
    cudaEventDestroy(r.a);
    cudaEventDestroy(r.b);
  }
  ctx->prof.clear();
}

extern "C" int32_t rmi_prof_enable(rmi_ctx* ctx, int32_t on) {
  RMI_TRY(rmi_check_ctx(ctx));
  RMI_CUDA_CHECK(cudaStreamSynchronize(ctx->stream));
  prof_clear(ctx);
  ctx->prof_on = on != 0;
  return RMI_OK;
}

extern "C" int32_t rmi_prof_read(rmi_ctx* ctx, const char* tag, uint64_t* launches, float* total_ms) {
  RMI_TRY(rmi_check_ctx(ctx));
  RMI_CUDA_CHECK(cudaStreamSynchronize(ctx->stream));
  uint64_t n = 0;
  double ms = 0.0;
  for (auto& r : ctx->prof) {
    if (strcmp(r.tag, tag) != 0) continue;
    float t = 0.0f;
    if (cudaEventElapsedTime(&t, r.a, r.b) == cudaSuccess) {
      ms += t;
      n++;
    }
  }
  if (launches) *launches = n;
  if (total_ms) *total_ms = (float)ms;
  return RMI_OK;
}

// ---------------------------------------------------------------- context

extern "C" int32_t rmi_init(int32_t device, rmi_ctx** out) {
  RMI_REQUIRE(out != nullptr, RMI_ERR_BAD_HANDLE, "rmi_init: out is null");
  *out = nullptr;
  int n = 0;
  cudaError_t e = cudaGetDeviceCount(&n);
  if (e != cudaSuccess || n == 0) {
    rmi_set_error("no usable CUDA device: %s", e == cudaSuccess ? "device count is 0" : cudaGetErrorString(e));
    (void)cudaGetLastError();
    return RMI_ERR_CUDA;
  }
  RMI_REQUIRE(device >= 0 && device < n, RMI_ERR_BAD_SHAPE, "device %d out of range (have %d)", device, n);
  RMI_CUDA_CHECK(cudaSetDevice(device));
  cudaDeviceProp prop;
  RMI_CUDA_CHECK(cudaGetDeviceProperties(&prop, device));
  RMI_REQUIRE(prop.major == 10, RMI_ERR_UNSUPPORTED,
              "device %d is sm_%d%d; this library is built for sm_100a (B200) only", device, prop.major, prop.minor);
  rmi_ctx* c = new (std::nothrow) rmi_ctx();
  RMI_REQUIRE(c != nullptr, RMI_ERR_OOM, "host allocation failed");
  c->magic = RMI_CTX_MAGIC;
  c->device = device;
  c->sm_count = prop.multiProcessorCount;
  c->l2_bytes = (size_t)prop.l2CacheSize;
  c->mem_bytes = prop.totalGlobalMem;
  c->smem_optin = prop.sharedMemPerBlockOptin;
  c->sem = RMI_SEM_AVX2;
  c->prefill_exact = false;
  c->wait_limit_ns = 2000000000ull;
  c->launches = 0;
  c->prof_on = false;
  c->pdl = false;
  c->fanout = out_fanout{};
  c->pipe_ready = false;
  for (int i = 0; i < 8; i++) {
    c->scratch[i] = nullptr;
    c->scratch_bytes[i] = 0;
  }
  if (cudaStreamCreateWithFlags(&c->own_stream, cudaStreamNonBlocking) != cudaSuccess ||
      cudaMalloc(&c->d_status, sizeof(rmi_dev_status)) != cudaSuccess ||
      cudaMallocHost(&c->h_status, sizeof(rmi_dev_status)) != cudaSuccess ||
      cudaMemset(c->d_status, 0, sizeof(rmi_dev_status)) != cudaSuccess ||
      cudaMemcpy(&c->d_status->limit_ns, &c->wait_limit_ns, 8, cudaMemcpyHostToDevice) != cudaSuccess) {
    rmi_set_error("context setup failed: %s", cudaGetErrorString(cudaGetLastError()));
    delete c;
    return RMI_ERR_CUDA;
  }
  c->stream = c->own_stream;
  *out = c;
  return RMI_OK;
}

extern "C" int32_t rmi_destroy(rmi_ctx* ctx) {
  RMI_TRY(rmi_check_ctx(ctx));
  cudaStreamSynchronize(ctx->stream);
  prof_clear(ctx);
  for (int i = 0; i < 8; i++)
    if (ctx->scratch[i]) cudaFree(ctx->scratch[i]);
  cudaFree(ctx->d_status);
  cudaFreeHost(ctx->h_status);
  if (ctx->pipe_ready) {
    cudaStreamDestroy(ctx->copy_in);
    cudaStreamDestroy(ctx->copy_out);
    for (int i = 0; i < 2; i++) {
      cudaEventDestroy(ctx->ev_in[i]);
      cudaEventDestroy(ctx->ev_compute[i]);
      cudaEventDestroy(ctx->ev_out[i]);
    }
  }
  cudaStreamDestroy(ctx->own_stream);
  ctx->magic = 0;
  delete ctx;
  return RMI_OK;
}

extern "C" int32_t rmi_set_semantics(rmi_ctx* ctx, int32_t sem) {
  RMI_TRY(rmi_check_ctx(ctx));
  RMI_REQUIRE(sem >= RMI_SEM_AVX2 && sem <= RMI_SEM_SCALAR, RMI_ERR_UNSUPPORTED, "unknown semantics %d", sem);
  ctx->sem = sem;
  return RMI_OK;
}

extern "C" int32_t rmi_set_prefill_exact(rmi_ctx* ctx, int32_t on) {
  RMI_TRY(rmi_check_ctx(ctx));
  ctx->prefill_exact = on != 0;
  return RMI_OK;
}

extern "C" int32_t rmi_set_dependent_launch(rmi_ctx* ctx, int32_t on) {
  RMI_TRY(rmi_check_ctx(ctx));
  std::lock_guard<std::mutex> lock(ctx->mu);
  ctx->pdl = on != 0;
  return RMI_OK;
}

extern "C" int32_t rmi_set_wait_limit_ms(rmi_ctx* ctx, uint32_t ms) {
  RMI_TRY(rmi_check_ctx(ctx));
  RMI_REQUIRE(ms >= 1 && ms <= 60000, RMI_ERR_BAD_SHAPE, "wait limit must be within 1..60000 ms, got %u", ms);
  std::lock_guard<std::mutex> lock(ctx->mu);
  RMI_CUDA_CHECK(cudaStreamSynchronize(ctx->stream));
  ctx->wait_limit_ns = (uint64_t)ms * 1000000ull;
  RMI_CUDA_CHECK(cudaMemcpy(&ctx->d_status->limit_ns, &ctx->wait_limit_ns, 8, cudaMemcpyHostToDevice));
  return RMI_OK;
}

extern "C" int32_t rmi_get_semantics(rmi_ctx* ctx, int32_t* sem) {
  RMI_TRY(rmi_check_ctx(ctx));
  *sem = ctx->sem;
  return RMI_OK;
}

extern "C" int32_t rmi_set_stream(rmi_ctx* ctx, void* cuda_stream) {
  RMI_TRY(rmi_check_ctx(ctx));
  RMI_CUDA_CHECK(cudaStreamSynchronize(ctx->stream));
  ctx->stream = cuda_stream ? (cudaStream_t)cuda_stream : ctx->own_stream;
  return RMI_OK;
}

extern "C" int32_t rmi_sync(rmi_ctx* ctx) {
  RMI_TRY(rmi_check_ctx(ctx));
  RMI_CUDA_CHECK(cudaStreamSynchronize(ctx->stream));
  return RMI_OK;
}

extern "C" int32_t rmi_device_info(rmi_ctx* ctx, int32_t* sm_count, size_t* l2_bytes, size_t* mem_bytes) {
  RMI_TRY(rmi_check_ctx(ctx));
  if (sm_count) *sm_count = ctx->sm_count;
  if (l2_bytes) *l2_bytes = ctx->l2_bytes;
  if (mem_bytes) *mem_bytes = ctx->mem_bytes;
  return RMI_OK;
}

extern "C" int32_t rmi_launch_count(rmi_ctx* ctx, uint64_t* count) {
  RMI_TRY(rmi_check_ctx(ctx));
  *count = ctx->launches.load();
  return RMI_OK;
}

extern "C" int32_t rmi_dev_alloc(rmi_ctx* ctx, size_t bytes, void** dev_ptr) {
  RMI_TRY(rmi_check_ctx(ctx));
  cudaError_t e = cudaMalloc(dev_ptr, bytes ? bytes : 16);
  if (e != cudaSuccess) {
    (void)cudaGetLastError();
    rmi_set_error("device allocation of %zu bytes failed: %s", bytes, cudaGetErrorString(e));
    return RMI_ERR_OOM;
  }
  return RMI_OK;
}

extern "C" int32_t rmi_dev_free(rmi_ctx* ctx, void* dev_ptr) {
  RMI_TRY(rmi_check_ctx(ctx));
  RMI_CUDA_CHECK(cudaStreamSynchronize(ctx->stream));
  RMI_CUDA_CHECK(cudaFree(dev_ptr));
  return RMI_OK;
}

extern "C" int32_t rmi_h2d(rmi_ctx* ctx, void* dst_dev, const void* src_host, size_t bytes) {
  RMI_TRY(rmi_check_ctx(ctx));
  RMI_CUDA_CHECK(cudaMemcpyAsync(dst_dev, src_host, bytes, cudaMemcpyHostToDevice, ctx->stream));
  RMI_CUDA_CHECK(cudaStreamSynchronize(ctx->stream));
  return RMI_OK;
}

extern "C" int32_t rmi_d2h(rmi_ctx* ctx, void* dst_host, const void* src_dev, size_t bytes) {
  RMI_TRY(rmi_check_ctx(ctx));
  RMI_CUDA_CHECK(cudaMemcpyAsync(dst_host, src_dev, bytes, cudaMemcpyDeviceToHost, ctx->stream));
  RMI_CUDA_CHECK(cudaStreamSynchronize(ctx->stream));
  return RMI_OK;
}

extern "C" int32_t rmi_host_alloc_pinned(rmi_ctx* ctx, size_t bytes, void** host_ptr) {
  RMI_TRY(rmi_check_ctx(ctx));
  cudaError_t e = cudaMallocHost(host_ptr, bytes ? bytes : 16);
  if (e != cudaSuccess) {
    (void)cudaGetLastError();
    rmi_set_error("pinned host allocation of %zu bytes failed: %s", bytes, cudaGetErrorString(e));
    return RMI_ERR_OOM;
  }
  return RMI_OK;
}

extern "C" int32_t rmi_host_free_pinned(rmi_ctx* ctx, void* host_ptr) {
  RMI_TRY(rmi_check_ctx(ctx));
  RMI_CUDA_CHECK(cudaFreeHost(host_ptr));
  return RMI_OK;
}

// ---------------------------------------------------------------- weights

static int32_t dev_malloc(void** p, size_t bytes) {
  cudaError_t e = cudaMalloc(p, bytes ? bytes : 16);
  if (e != cudaSuccess) {
    (void)cudaGetLastError();
    rmi_set_error("device allocation of %zu bytes failed: %s", bytes, cudaGetErrorString(e));
    return RMI_ERR_OOM;
  }
  return RMI_OK;
}

static rmi_weight* new_weight(int type, size_t n_in, size_t n_rows) {
  rmi_weight* w = new (std::nothrow) rmi_weight();
  if (!w) return nullptr;
  memset(w, 0, sizeof(*w));
  w->magic = RMI_WEIGHT_MAGIC;
  w->ggml_type = type;
  w->n_in = n_in;
  w->n_rows = n_rows;
  w->n_tiles16 = (n_rows + 15) / 16;
  return w;
}

static void free_weight(rmi_weight* w) {
  if (!w) return;
  if (w->d_tile16) cudaFree(w->d_tile16);
  if (w->d_umma_q) cudaFree(w->d_umma_q);
  if (w->d_umma_s) cudaFree(w->d_umma_s);
  if (w->d_umma_gu_q) cudaFree(w->d_umma_gu_q);
  if (w->d_umma_gu_s) cudaFree(w->d_umma_gu_s);
  if (w->d_raw) cudaFree(w->d_raw);
  w->magic = 0;
  delete w;
}

extern "C" int32_t rmi_weight_upload(rmi_ctx* ctx, int32_t ggml_type, const void* bytes, size_t nbytes,
                                     size_t n_in, size_t n_out, size_t row_begin, size_t row_end,
                                     rmi_weight** out) {
  RMI_TRY(rmi_check_ctx(ctx));
  RMI_REQUIRE(out != nullptr && bytes != nullptr, RMI_ERR_BAD_HANDLE, "rmi_weight_upload: null argument");
  *out = nullptr;
  RMI_REQUIRE(ggml_type == RMI_GGML_Q8_0 || ggml_type == RMI_GGML_Q4_K || ggml_type == RMI_GGML_Q6_K ||
                  ggml_type == RMI_GGML_Q4_0,
              RMI_ERR_UNSUPPORTED,
              "ggml type %d is not handled by this path (Q4_0 = 2, Q8_0 = 8, Q4_K = 12 and Q6_K = 14 are)", ggml_type);
  const size_t be = (ggml_type == RMI_GGML_Q8_0 || ggml_type == RMI_GGML_Q4_0) ? 32 : 256;
  const size_t bb = ggml_type == RMI_GGML_Q8_0 ? 34 : (ggml_type == RMI_GGML_Q4_0 ? 18 : (ggml_type == RMI_GGML_Q4_K ? 144 : 210));
  RMI_REQUIRE(n_in > 0 && n_in % be == 0, RMI_ERR_BAD_SHAPE, "n_in=%zu is not a multiple of %zu", n_in, be);
  RMI_REQUIRE(row_begin <= row_end && row_end <= n_out, RMI_ERR_BAD_SHAPE,
              "row range [%zu,%zu) outside [0,%zu)", row_begin, row_end, n_out);
  const size_t row_bytes = n_in / be * bb;
  RMI_REQUIRE(nbytes >= n_out * row_bytes, RMI_ERR_BAD_SHAPE,
              "weight buffer has %zu bytes, %zu rows x %zu bytes need %zu", nbytes, n_out, row_bytes, n_out * row_bytes);
  std::lock_guard<std::mutex> lock(ctx->mu);
  const size_t n_rows = row_end - row_begin;
  rmi_weight* w = new_weight(ggml_type, n_in, n_rows);
  RMI_REQUIRE(w != nullptr, RMI_ERR_OOM, "host allocation failed");
  const uint8_t* src = (const uint8_t*)bytes + row_begin * row_bytes;
  int32_t st = RMI_OK;
  if (ggml_type == RMI_GGML_Q6_K || ggml_type == RMI_GGML_Q4_0) {
    // 210-byte super-blocks / 18-byte blocks padded to an aligned device stride
    const bool q6 = ggml_type == RMI_GGML_Q6_K;
    const size_t nsb = n_rows * (n_in / be), stride = q6 ? q6k_device_block_bytes() : q4_0_device_block_bytes();
    w->raw_bytes = nsb * stride;
    std::vector<uint8_t> staged(w->raw_bytes ? w->raw_bytes : 1, 0);
    for (size_t i = 0; i < nsb; i++) {
      if (q6) {
        memcpy(staged.data() + i * stride, src + i * 210, 210);
      } else {  // f16 d | pad | nibbles
        memcpy(staged.data() + i * stride, src + i * 18, 2);
        memcpy(staged.data() + i * stride + 4, src + i * 18 + 2, 16);
      }
    }
    st = dev_malloc((void**)&w->d_raw, w->raw_bytes);
    if (st == RMI_OK && w->raw_bytes) {
      cudaError_t e = cudaMemcpyAsync(w->d_raw, staged.data(), w->raw_bytes, cudaMemcpyHostToDevice, ctx->stream);
      if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->stream);
      if (e != cudaSuccess) {
        rmi_set_error("weight upload failed: %s", cudaGetErrorString(e));
        st = RMI_ERR_CUDA;
      }
    }
  } else if (ggml_type == RMI_GGML_Q4_K) {
    w->raw_bytes = n_rows * row_bytes;
    st = dev_malloc((void**)&w->d_raw, w->raw_bytes);
    if (st == RMI_OK && w->raw_bytes) {
      cudaError_t e = cudaMemcpyAsync(w->d_raw, src, w->raw_bytes, cudaMemcpyHostToDevice, ctx->stream);
      if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->stream);
      if (e != cudaSuccess) {
        rmi_set_error("weight upload failed: %s", cudaGetErrorString(e));
        st = RMI_ERR_CUDA;
      }
    }
  } else {
    const size_t blocks = n_in / 32;
    w->tile16_bytes = w->n_tiles16 * blocks * Q8_REC_BYTES;
    uint8_t* d_raw = nullptr;
    st = dev_malloc((void**)&w->d_tile16, w->tile16_bytes);
    if (st == RMI_OK) st = dev_malloc((void**)&d_raw, n_rows * row_bytes);
    if (st == RMI_OK && n_rows) {
      cudaError_t e = cudaMemsetAsync(w->d_tile16, 0, w->tile16_bytes, ctx->stream);
      if (e == cudaSuccess) e = cudaMemcpyAsync(d_raw, src, n_rows * row_bytes, cudaMemcpyHostToDevice, ctx->stream);
      if (e != cudaSuccess) {
        rmi_set_error("weight upload failed: %s", cudaGetErrorString(e));
        st = RMI_ERR_CUDA;
      }
      if (st == RMI_OK) st = launch_q8_repack_tile16(ctx, d_raw, w->d_tile16, n_rows, blocks);
      if (st == RMI_OK && cudaStreamSynchronize(ctx->stream) != cudaSuccess) {
        rmi_set_error("weight re-layout failed: %s", cudaGetErrorString(cudaGetLastError()));
        st = RMI_ERR_CUDA;
      }
    }
    if (d_raw) cudaFree(d_raw);
  }
  if (st != RMI_OK) {
    free_weight(w);
    return st;
  }
  *out = w;
  return RMI_OK;
}

extern "C" int32_t rmi_weight_free(rmi_ctx* ctx, rmi_weight* w) {
  RMI_TRY(rmi_check_ctx(ctx));
  RMI_TRY(rmi_check_weight(w, -1));
  std::lock_guard<std::mutex> lock(ctx->mu);
  RMI_CUDA_CHECK(cudaStreamSynchronize(ctx->stream));
  free_weight(w);
  return RMI_OK;
}

extern "C" int32_t rmi_weight_info(const rmi_weight* w, int32_t* ggml_type, size_t* n_in, size_t* n_rows,
                                   size_t* device_bytes) {
  RMI_TRY(rmi_check_weight(w, -1));
  if (ggml_type) *ggml_type = w->ggml_type;
  if (n_in) *n_in = w->n_in;
  if (n_rows) *n_rows = w->n_rows;
  if (device_bytes) *device_bytes = w->tile16_bytes + w->raw_bytes + w->umma_bytes;
  return RMI_OK;
}

extern "C" int32_t rmi_weight_fuse_vstack(rmi_ctx* ctx, const rmi_weight* a, const rmi_weight* b,
                                          rmi_weight** out) {
  RMI_TRY(rmi_check_ctx(ctx));
  RMI_TRY(rmi_check_weight(a, -1));
  RMI_TRY(rmi_check_weight(b, -1));
  RMI_REQUIRE(out != nullptr, RMI_ERR_BAD_HANDLE, "rmi_weight_fuse_vstack: out is null");
  *out = nullptr;
  RMI_REQUIRE(a->ggml_type == b->ggml_type && a->n_in == b->n_in, RMI_ERR_BAD_SHAPE,
              "cannot v-stack: types %d/%d, row lengths %zu/%zu", a->ggml_type, b->ggml_type, a->n_in, b->n_in);
  std::lock_guard<std::mutex> lock(ctx->mu);
  rmi_weight* w = new_weight(a->ggml_type, a->n_in, a->n_rows + b->n_rows);
  RMI_REQUIRE(w != nullptr, RMI_ERR_OOM, "host allocation failed");
  w->n_rows_a = a->n_rows;
  int32_t st = RMI_OK;
  if (a->ggml_type != RMI_GGML_Q8_0) {
    w->raw_bytes = a->raw_bytes + b->raw_bytes;
    st = dev_malloc((void**)&w->d_raw, w->raw_bytes);
    if (st == RMI_OK) {
      cudaError_t e = cudaMemcpyAsync(w->d_raw, a->d_raw, a->raw_bytes, cudaMemcpyDeviceToDevice, ctx->stream);
      if (e == cudaSuccess) e = cudaMemcpyAsync(w->d_raw + a->raw_bytes, b->d_raw, b->raw_bytes, cudaMemcpyDeviceToDevice, ctx->stream);
      if (e != cudaSuccess) {
        rmi_set_error("v-stack copy failed: %s", cudaGetErrorString(e));
        st = RMI_ERR_CUDA;
      }
    }
  } else {
    const size_t blocks = a->n_in / 32;
    w->tile16_bytes = w->n_tiles16 * blocks * Q8_REC_BYTES;
    st = dev_malloc((void**)&w->d_tile16, w->tile16_bytes);
    if (st == RMI_OK) {
      if (cudaMemsetAsync(w->d_tile16, 0, w->tile16_bytes, ctx->stream) != cudaSuccess) st = RMI_ERR_CUDA;
      if (st == RMI_OK) st = launch_q8_copy_rows_tile16(ctx, a->d_tile16, w->d_tile16, a->n_rows, blocks, 0);
      if (st == RMI_OK) st = launch_q8_copy_rows_tile16(ctx, b->d_tile16, w->d_tile16, b->n_rows, blocks, a->n_rows);
    }
  }
  if (st == RMI_OK && cudaStreamSynchronize(ctx->stream) != cudaSuccess) {
    rmi_set_error("v-stack failed: %s", cudaGetErrorString(cudaGetLastError()));
    st = RMI_ERR_CUDA;
  }
  if (st != RMI_OK) {
    free_weight(w);
    return st;
  }
  *out = w;
  return RMI_OK;
}

int32_t ensure_umma_layout(rmi_ctx* ctx, const rmi_weight* cw, bool gate_up_interleaved) {
  rmi_weight* w = const_cast<rmi_weight*>(cw);
  if (gate_up_interleaved ? w->d_umma_gu_q != nullptr : w->d_umma_q != nullptr) return RMI_OK;
  RMI_REQUIRE(!gate_up_interleaved || (w->n_rows_a * 2 == w->n_rows && w->n_rows_a % 32 == 0), RMI_ERR_BAD_SHAPE,
              "gate/up interleaving needs a v-stack of two equal halves with n_ff a multiple of 32");
  const size_t blocks = w->n_in / 32;
  const size_t n_slabs = (w->n_in + 127) / 128;
  const size_t tiles = (w->n_rows + 127) / 128;
  size_t qb = tiles * n_slabs * 16384, sb = tiles * blocks * 128 * sizeof(float);
  uint8_t* q = nullptr;
  float* s = nullptr;
  RMI_TRY(dev_malloc((void**)&q, qb));
  int32_t st = dev_malloc((void**)&s, sb);
  if (st == RMI_OK && cudaMemsetAsync(s, 0, sb, ctx->stream) != cudaSuccess) st = RMI_ERR_CUDA;
  if (st == RMI_OK)
    st = launch_q8_build_umma(ctx, w->d_tile16, q, s, w->n_rows, blocks, gate_up_interleaved ? w->n_rows_a : 0);
  if (st != RMI_OK) {
    cudaFree(q);
    if (s) cudaFree(s);
    return st;
  }
  if (gate_up_interleaved) {
    w->d_umma_gu_q = q;
    w->d_umma_gu_s = s;
  } else {
    w->d_umma_q = q;
    w->d_umma_s = s;
  }
  w->umma_bytes += qb + sb;
  return RMI_OK;
}

// ---------------------------------------------------------------- Q8_0 entry points

// Up to this many activation rows the GEMM runs with swapped operands (32 activation rows per tile column
// block instead of a 128-row tile that is mostly padding).
constexpr size_t SWAP_AB_MAX_M = 96;

static bool use_tensor_cores(const rmi_ctx* ctx, size_t m) {
  // Prefill-shaped calls (m > 32) run on the tcgen05 GEMM.  It produces exact whole-block int32 sums
  // and accumulates them as sum = fma(f32(dot), wd*xs, sum): bit-exact for the NEON and SCALAR
  // variants of the reference.  The AVX2 variant accumulates eight partial sums per block
  // (avx2.rs:96-153), which the tensor core cannot deliver; for it the GEMM keeps the AVX2 quantizer
  // (activation bytes and scale bits unchanged), the exact block sums, and the whole-block chain,
  // whose f32 result is within 1e-5 of the eight-lane order.  rmi_set_prefill_exact(ctx, 1) keeps
  // AVX2 calls of every m on the bit-exact CUDA-core kernels instead.
  return m > 32 && !(ctx->sem == RMI_SEM_AVX2 && ctx->prefill_exact);
}

// Plain matmuls (no fused epilogue) also take the tensor cores for 8 < m <= 32, with swapped operands,
// where that is bit-exact (NEON and SCALAR); AVX2 calls of m <= 32 stay on the GEMV kernels, so the
// decode path is bit-exact under every setting.
static bool matmul_on_tensor_cores(const rmi_ctx* ctx, size_t m) {
  if (use_tensor_cores(ctx, m)) return true;
  return m > 8 && m <= SWAP_AB_MAX_M && ctx->sem != RMI_SEM_AVX2;
}

extern "C" int32_t rmi_quantize_q8_0_dev(rmi_ctx* ctx, const float* x, size_t m, size_t n, uint8_t* q8,
                                         float* scales) {
  RMI_TRY(rmi_check_ctx(ctx));
  RMI_REQUIRE(n % 32 == 0, RMI_ERR_BAD_SHAPE, "n=%zu is not a multiple of 32", n);
  RMI_REQUIRE(x && q8 && scales, RMI_ERR_BAD_HANDLE, "rmi_quantize_q8_0: null buffer");
  return launch_q8_quantize(ctx, x, m, n, q8, scales, 0);
}

extern "C" int32_t rmi_quantize_q8_0(rmi_ctx* ctx, const float* x, size_t m, size_t n, uint8_t* q8,
                                     float* scales) {
  RMI_TRY(rmi_check_ctx(ctx));
  RMI_REQUIRE(n % 32 == 0, RMI_ERR_BAD_SHAPE, "n=%zu is not a multiple of 32", n);
  RMI_REQUIRE((x && q8 && scales) || m * n == 0, RMI_ERR_BAD_HANDLE, "rmi_quantize_q8_0: null buffer");
  if (m * n == 0) return RMI_OK;
  std::lock_guard<std::mutex> lock(ctx->mu);
  float *dx, *ds;
  uint8_t* dq;
  RMI_TRY(rmi_scratch(ctx, 5, m * n * 4, (void**)&dx));
  RMI_TRY(rmi_scratch(ctx, 0, m * n, (void**)&dq));
  RMI_TRY(rmi_scratch(ctx, 1, m * (n / 32) * 4, (void**)&ds));
  RMI_CUDA_CHECK(cudaMemcpyAsync(dx, x, m * n * 4, cudaMemcpyHostToDevice, ctx->stream));
  RMI_TRY(launch_q8_quantize(ctx, dx, m, n, dq, ds, 0));
  RMI_CUDA_CHECK(cudaMemcpyAsync(q8, dq, m * n, cudaMemcpyDeviceToHost, ctx->stream));
  RMI_CUDA_CHECK(cudaMemcpyAsync(scales, ds, m * (n / 32) * 4, cudaMemcpyDeviceToHost, ctx->stream));
  RMI_CUDA_CHECK(cudaStreamSynchronize(ctx->stream));
  return RMI_OK;
}

static int32_t check_rows(const rmi_weight* w, size_t row_begin, size_t row_end) {
  RMI_REQUIRE(row_begin <= row_end && row_end <= w->n_rows, RMI_ERR_BAD_SHAPE,
              "row range [%zu,%zu) outside [0,%zu)", row_begin, row_end, w->n_rows);
  return RMI_OK;
}

extern "C" int32_t rmi_matmul_q8_0_prequantized_dev(rmi_ctx* ctx, const rmi_weight* w, const uint8_t* q8,
                                                    const float* scales, size_t m, float* output,
                                                    size_t row_begin, size_t row_end) {
  RMI_TRY(rmi_check_ctx(ctx));
  RMI_TRY(rmi_check_weight(w, RMI_GGML_Q8_0));
  RMI_TRY(check_rows(w, row_begin, row_end));
  RMI_REQUIRE(((uintptr_t)q8 & 15) == 0, RMI_ERR_BAD_SHAPE, "device q8 buffer must be 16-byte aligned");
  return launch_q8_gemv(ctx, w, q8, scales, m, output, w->n_rows, row_begin, row_end);
}

extern "C" int32_t rmi_matmul_q8_0_prequantized(rmi_ctx* ctx, const rmi_weight* w, const uint8_t* q8,
                                                const float* scales, size_t m, float* output,
                                                size_t row_begin, size_t row_end) {
  RMI_TRY(rmi_check_ctx(ctx));
  RMI_TRY(rmi_check_weight(w, RMI_GGML_Q8_0));
  RMI_TRY(check_rows(w, row_begin, row_end));
  if (m == 0 || row_begin == row_end) return RMI_OK;
  RMI_REQUIRE(q8 && scales && output, RMI_ERR_BAD_HANDLE, "rmi_matmul_q8_0_prequantized: null buffer");
  std::lock_guard<std::mutex> lock(ctx->mu);
  const size_t blocks = w->n_in / 32, n = w->n_rows, nr = row_end - row_begin;
  uint8_t* dq;
  float *ds, *dout;
  RMI_TRY(rmi_scratch(ctx, 0, m * w->n_in, (void**)&dq));
  RMI_TRY(rmi_scratch(ctx, 1, m * blocks * 4, (void**)&ds));
  RMI_TRY(rmi_scratch(ctx, 6, m * n * 4, (void**)&dout));
  RMI_CUDA_CHECK(cudaMemcpyAsync(dq, q8, m * w->n_in, cudaMemcpyHostToDevice, ctx->stream));
  RMI_CUDA_CHECK(cudaMemcpyAsync(ds, scales, m * blocks * 4, cudaMemcpyHostToDevice, ctx->stream));
  RMI_TRY(launch_q8_gemv(ctx, w, dq, ds, m, dout, n, row_begin, row_end));
  // only [row_begin,row_end) of each output row is written back (parallel.rs:131-138)
  RMI_CUDA_CHECK(cudaMemcpy2DAsync(output + row_begin, n * 4, dout + row_begin, n * 4, nr * 4, m,
                                   cudaMemcpyDeviceToHost, ctx->stream));
  RMI_CUDA_CHECK(cudaStreamSynchronize(ctx->stream));
  return RMI_OK;
}

// dout: [m][out_stride] f32, the weight's rows land in columns [0, n_rows); out_stride 0 = n_rows
int32_t matmul_q8_0_device(rmi_ctx* ctx, const rmi_weight* w, const float* dx, size_t m, float* dout,
                           size_t out_stride) {
  const size_t blocks = w->n_in / 32;
  if (out_stride == 0) out_stride = w->n_rows;
  if (matmul_on_tensor_cores(ctx, m)) {
    RMI_TRY(ensure_umma_layout(ctx, w));
    const size_t m_tiles = (m + 127) / 128, n_slabs = (w->n_in + 127) / 128;
    uint8_t* a_img;
    float* a_sc;
    RMI_TRY(rmi_scratch(ctx, 0, m_tiles * n_slabs * 16384, (void**)&a_img));
    RMI_TRY(rmi_scratch(ctx, 1, m_tiles * blocks * 128 * 4, (void**)&a_sc));
    if (m % 128 != 0 || w->n_in % 128 != 0) {
      RMI_CUDA_CHECK(cudaMemsetAsync(a_img, 0, m_tiles * n_slabs * 16384, ctx->stream));
      RMI_CUDA_CHECK(cudaMemsetAsync(a_sc, 0, m_tiles * blocks * 128 * 4, ctx->stream));
    }
    RMI_TRY(launch_q8_quantize(ctx, dx, m, w->n_in, a_img, a_sc, 1));
    gemm_tc_args g = {};
    g.a_img = a_img;
    g.a_scales = a_sc;
    g.w = w;
    g.m = m;
    g.col_begin = 0;
    g.col_end = w->n_rows;
    g.epilogue = GEMM_EPI_F32;
    g.out = dout;
    g.out_stride = out_stride;
    g.swap_ab = m <= SWAP_AB_MAX_M;
    return launch_gemm_tc(ctx, g);
  }
  uint8_t* dq;
  float* ds;
  RMI_TRY(rmi_scratch(ctx, 0, m * w->n_in, (void**)&dq));
  RMI_TRY(rmi_scratch(ctx, 1, m * blocks * 4, (void**)&ds));
  RMI_TRY(launch_q8_quantize(ctx, dx, m, w->n_in, dq, ds, 0));
  return launch_q8_gemv(ctx, w, dq, ds, m, dout, out_stride, 0, w->n_rows);
}

extern "C" int32_t rmi_matmul_q8_0_fanout_dev(rmi_ctx* ctx, const rmi_weight* w, const float* x, size_t m,
                                              float* const* outs, int32_t n_outs, size_t out_stride,
                                              size_t col_offset) {
  RMI_TRY(rmi_check_ctx(ctx));
  RMI_TRY(rmi_check_weight(w, RMI_GGML_Q8_0));
  RMI_REQUIRE(outs && n_outs >= 1 && n_outs <= RMI_MAX_FANOUT, RMI_ERR_BAD_SHAPE,
              "rmi_matmul_q8_0_fanout_dev: between 1 and %d output buffers", RMI_MAX_FANOUT);
  RMI_REQUIRE(out_stride >= col_offset + w->n_rows, RMI_ERR_BAD_SHAPE,
              "rmi_matmul_q8_0_fanout_dev: out_stride %zu < col_offset %zu + %zu rows", out_stride, col_offset, w->n_rows);
  for (int32_t i = 0; i < n_outs; i++)
    RMI_REQUIRE(outs[i] != nullptr && (reinterpret_cast<uintptr_t>(outs[i]) & 3) == 0, RMI_ERR_BAD_HANDLE,
                "rmi_matmul_q8_0_fanout_dev: output %d is null or misaligned", i);
  if (m == 0 || w->n_rows == 0) return RMI_OK;
  RMI_REQUIRE(x != nullptr, RMI_ERR_BAD_HANDLE, "rmi_matmul_q8_0_fanout_dev: null input");
  std::lock_guard<std::mutex> lock(ctx->mu);
  ctx->fanout.n = n_outs - 1;
  for (int32_t i = 1; i < n_outs; i++)
    ctx->fanout.delta[i - 1] = (long long)(reinterpret_cast<const char*>(outs[i]) - reinterpret_cast<const char*>(outs[0]));
  const int32_t st = matmul_q8_0_device(ctx, w, x, m, outs[0] + col_offset, out_stride);
  ctx->fanout = out_fanout{};
  return st;
}

extern "C" int32_t rmi_matmul_q8_0_dev(rmi_ctx* ctx, const rmi_weight* w, const float* x, size_t m, float* output) {
  RMI_TRY(rmi_check_ctx(ctx));
  RMI_TRY(rmi_check_weight(w, RMI_GGML_Q8_0));
  if (m == 0) return RMI_OK;
  std::lock_guard<std::mutex> lock(ctx->mu);
  return matmul_q8_0_device(ctx, w, x, m, output);
}

extern "C" int32_t rmi_matmul_q8_0(rmi_ctx* ctx, const rmi_weight* w, const float* x, size_t m, float* output) {
  RMI_TRY(rmi_check_ctx(ctx));
  RMI_TRY(rmi_check_weight(w, RMI_GGML_Q8_0));
  if (m == 0 || w->n_rows == 0) return RMI_OK;
  RMI_REQUIRE(x && output, RMI_ERR_BAD_HANDLE, "rmi_matmul_q8_0: null buffer");
  std::lock_guard<std::mutex> lock(ctx->mu);
  float *dx, *dout;
  RMI_TRY(rmi_scratch(ctx, 5, m * w->n_in * 4, (void**)&dx));
  RMI_TRY(rmi_scratch(ctx, 6, m * w->n_rows * 4, (void**)&dout));
  RMI_CUDA_CHECK(cudaMemcpyAsync(dx, x, m * w->n_in * 4, cudaMemcpyHostToDevice, ctx->stream));
  RMI_TRY(matmul_q8_0_device(ctx, w, dx, m, dout));
  RMI_CUDA_CHECK(cudaMemcpyAsync(output, dout, m * w->n_rows * 4, cudaMemcpyDeviceToHost, ctx->stream));
  if (matmul_on_tensor_cores(ctx, m)) return rmi_check_dev_status(ctx, "rmi_matmul_q8_0");
  RMI_CUDA_CHECK(cudaStreamSynchronize(ctx->stream));
  return RMI_OK;
}

extern "C" int32_t rmi_matmul_q8_0_f32_dev(rmi_ctx* ctx, const rmi_weight* w, const float* x, size_t m, float* output) {
  RMI_TRY(rmi_check_ctx(ctx));
  RMI_TRY(rmi_check_weight(w, RMI_GGML_Q8_0));
  if (m == 0 || w->n_rows == 0) return RMI_OK;
  RMI_REQUIRE(x && output, RMI_ERR_BAD_HANDLE, "rmi_matmul_q8_0_f32_dev: null buffer");
  RMI_REQUIRE(m <= 65535, RMI_ERR_BAD_SHAPE, "rmi_matmul_q8_0_f32_dev: at most 65535 rows per call, got %zu", m);
  std::lock_guard<std::mutex> lock(ctx->mu);
  return launch_q8_matmul_f32(ctx, w, x, m, output);
}

extern "C" int32_t rmi_matmul_q8_0_f32(rmi_ctx* ctx, const rmi_weight* w, const float* x, size_t m, float* output) {
  RMI_TRY(rmi_check_ctx(ctx));
  RMI_TRY(rmi_check_weight(w, RMI_GGML_Q8_0));
  if (m == 0 || w->n_rows == 0) return RMI_OK;
  RMI_REQUIRE(x && output, RMI_ERR_BAD_HANDLE, "rmi_matmul_q8_0_f32: null buffer");
  RMI_REQUIRE(m <= 65535, RMI_ERR_BAD_SHAPE, "rmi_matmul_q8_0_f32: at most 65535 rows per call, got %zu", m);
  std::lock_guard<std::mutex> lock(ctx->mu);
  float *dx, *dout;
  RMI_TRY(rmi_scratch(ctx, 5, m * w->n_in * 4, (void**)&dx));
  RMI_TRY(rmi_scratch(ctx, 6, m * w->n_rows * 4, (void**)&dout));
  RMI_CUDA_CHECK(cudaMemcpyAsync(dx, x, m * w->n_in * 4, cudaMemcpyHostToDevice, ctx->stream));
  RMI_TRY(launch_q8_matmul_f32(ctx, w, dx, m, dout));
  RMI_CUDA_CHECK(cudaMemcpyAsync(output, dout, m * w->n_rows * 4, cudaMemcpyDeviceToHost, ctx->stream));
  RMI_CUDA_CHECK(cudaStreamSynchronize(ctx->stream));
  return RMI_OK;
}

extern "C" int32_t rmi_q8_0_block_sums(rmi_ctx* ctx, const rmi_weight* w, const uint8_t* q8, size_t m,
                                       int32_t* sums, int32_t use_tc) {
  RMI_TRY(rmi_check_ctx(ctx));
  RMI_TRY(rmi_check_weight(w, RMI_GGML_Q8_0));
  if (m == 0 || w->n_rows == 0) return RMI_OK;
  RMI_REQUIRE(q8 && sums, RMI_ERR_BAD_HANDLE, "rmi_q8_0_block_sums: null buffer");
  std::lock_guard<std::mutex> lock(ctx->mu);
  const size_t blocks = w->n_in / 32, total = m * w->n_rows * blocks;
  uint8_t* dq;
  int32_t* dsum;
  RMI_TRY(rmi_scratch(ctx, 0, m * w->n_in, (void**)&dq));
  RMI_TRY(rmi_scratch(ctx, 7, total * 4, (void**)&dsum));
  RMI_CUDA_CHECK(cudaMemcpyAsync(dq, q8, m * w->n_in, cudaMemcpyHostToDevice, ctx->stream));
  if (!use_tc) {
    RMI_TRY(launch_q8_block_sums(ctx, w, dq, m, dsum));
  } else {
    // re-tile the given quants into A images with a tiny kernel-free path: dequantize is not
    // needed, the quantizer's image layout is produced on the host side here.
    RMI_TRY(ensure_umma_layout(ctx, w));
    const size_t m_tiles = (m + 127) / 128, n_slabs = (w->n_in + 127) / 128;
    size_t img_bytes = m_tiles * n_slabs * 16384;
    uint8_t* h_img = (uint8_t*)calloc(img_bytes, 1);
    RMI_REQUIRE(h_img != nullptr, RMI_ERR_OOM, "host allocation failed");
    for (size_t r = 0; r < m; r++)
      for (size_t k = 0; k < w->n_in; k++) {
        size_t tile = r / 128, rr = r % 128, slab = k / 128, c = (k % 128) / 16, byte = k % 16;
        h_img[(tile * n_slabs + slab) * 16384 + (rr / 8) * 1024 + c * 128 + (rr % 8) * 16 + byte] = q8[r * w->n_in + k];
      }
    uint8_t* a_img;
    int32_t st = rmi_scratch(ctx, 3, img_bytes, (void**)&a_img);
    if (st == RMI_OK && cudaMemcpyAsync(a_img, h_img, img_bytes, cudaMemcpyHostToDevice, ctx->stream) != cudaSuccess) st = RMI_ERR_CUDA;
    if (st == RMI_OK && cudaStreamSynchronize(ctx->stream) != cudaSuccess) st = RMI_ERR_CUDA;
    free(h_img);
    RMI_TRY(st);
    gemm_tc_args g = {};
    g.a_img = a_img;
    g.a_scales = nullptr;
    g.w = w;
    g.m = m;
    g.col_begin = 0;
    g.col_end = w->n_rows;
    g.epilogue = GEMM_EPI_BLOCK_SUMS;
    g.sums = dsum;
    RMI_TRY(launch_gemm_tc(ctx, g));
  }
  RMI_CUDA_CHECK(cudaMemcpyAsync(sums, dsum, total * 4, cudaMemcpyDeviceToHost, ctx->stream));
  if (use_tc) return rmi_check_dev_status(ctx, "rmi_q8_0_block_sums");
  RMI_CUDA_CHECK(cudaStreamSynchronize(ctx->stream));
  return RMI_OK;
}

// ---------------------------------------------------------------- fused SwiGLU FFN

int32_t ffn_device(rmi_ctx* ctx, const rmi_weight* wgu, const rmi_weight* wd, const float* dx, size_t m,
                   float* dout) {
  const size_t n_embd = wgu->n_in, n_ff = wgu->n_rows / 2;
  RMI_REQUIRE(wgu->n_rows_a * 2 == wgu->n_rows && wgu->n_rows_a > 0, RMI_ERR_BAD_SHAPE,
              "w_gate_up must be rmi_weight_fuse_vstack(gate, up) of equal row counts");
  RMI_REQUIRE(wd->n_in == n_ff && wd->n_rows == n_embd, RMI_ERR_BAD_SHAPE,
              "w_down is [%zu,%zu], expected [%zu,%zu]", wd->n_rows, wd->n_in, n_embd, n_ff);
  RMI_REQUIRE(n_ff % 32 == 0, RMI_ERR_BAD_SHAPE, "n_ff=%zu is not a multiple of 32", n_ff);
  const size_t b1 = n_embd / 32, b2 = n_ff / 32;
  if (use_tensor_cores(ctx, m)) {
    RMI_TRY(ensure_umma_layout(ctx, wgu, true));
    RMI_TRY(ensure_umma_layout(ctx, wd));
    const size_t m_tiles = (m + 127) / 128;
    const size_t s1 = (n_embd + 127) / 128, s2 = (n_ff + 127) / 128;
    uint8_t *a1, *a2;
    float *sc1, *sc2;
    RMI_TRY(rmi_scratch(ctx, 0, m_tiles * s1 * 16384, (void**)&a1));
    RMI_TRY(rmi_scratch(ctx, 1, m_tiles * b1 * 128 * 4, (void**)&sc1));
    RMI_TRY(rmi_scratch(ctx, 3, m_tiles * s2 * 16384, (void**)&a2));
    RMI_TRY(rmi_scratch(ctx, 4, m_tiles * b2 * 128 * 4, (void**)&sc2));
    if (m % 128 != 0 || n_embd % 128 != 0) {
      RMI_CUDA_CHECK(cudaMemsetAsync(a1, 0, m_tiles * s1 * 16384, ctx->stream));
      RMI_CUDA_CHECK(cudaMemsetAsync(sc1, 0, m_tiles * b1 * 128 * 4, ctx->stream));
    }
    if (n_ff % 128 != 0) RMI_CUDA_CHECK(cudaMemsetAsync(a2, 0, m_tiles * s2 * 16384, ctx->stream));
    RMI_TRY(launch_q8_quantize(ctx, dx, m, n_embd, a1, sc1, 1));
    gemm_tc_args g = {};
    g.a_img = a1;
    g.a_scales = sc1;
    g.w = wgu;
    g.m = m;
    g.col_begin = 0;
    g.col_end = n_ff;  // FFN columns; each tile computes 32 gate columns and the matching up columns
    g.epilogue = GEMM_EPI_SWIGLU_Q8;
    g.n_ff = n_ff;
    g.act_img = a2;
    g.act_scales = sc2;
    RMI_TRY(launch_gemm_tc(ctx, g));
    gemm_tc_args d = {};
    d.a_img = a2;
    d.a_scales = sc2;
    d.w = wd;
    d.m = m;
    d.col_begin = 0;
    d.col_end = n_embd;
    d.epilogue = GEMM_EPI_F32;
    d.out = dout;
    d.out_stride = n_embd;
    return launch_gemm_tc(ctx, d);
  }
  uint8_t *q1, *q2;
  float *sc1, *sc2, *gu;
  RMI_TRY(rmi_scratch(ctx, 0, m * n_embd, (void**)&q1));
  RMI_TRY(rmi_scratch(ctx, 1, m * b1 * 4, (void**)&sc1));
  RMI_TRY(rmi_scratch(ctx, 2, m * 2 * n_ff * 4, (void**)&gu));
  RMI_TRY(rmi_scratch(ctx, 3, m * n_ff, (void**)&q2));
  RMI_TRY(rmi_scratch(ctx, 4, m * b2 * 4, (void**)&sc2));
  RMI_TRY(launch_q8_quantize(ctx, dx, m, n_embd, q1, sc1, 0));
  RMI_TRY(launch_q8_gemv(ctx, wgu, q1, sc1, m, gu, 2 * n_ff, 0, 2 * n_ff));
  RMI_TRY(launch_silu_mul_quantize(ctx, gu, gu + n_ff, 2 * n_ff, m, n_ff, nullptr, q2, sc2));
  return launch_q8_gemv(ctx, wd, q2, sc2, m, dout, n_embd, 0, n_embd);
}

extern "C" int32_t rmi_ffn_swiglu_q8_0_dev(rmi_ctx* ctx, const rmi_weight* wgu, const rmi_weight* wd,
                                           const float* x, size_t m, float* out) {
  RMI_TRY(rmi_check_ctx(ctx));
  RMI_TRY(rmi_check_weight(wgu, RMI_GGML_Q8_0));
  RMI_TRY(rmi_check_weight(wd, RMI_GGML_Q8_0));
  if (m == 0) return RMI_OK;
  std::lock_guard<std::mutex> lock(ctx->mu);
  return ffn_device(ctx, wgu, wd, x, m, out);
}

extern "C" int32_t rmi_ffn_swiglu_q8_0(rmi_ctx* ctx, const rmi_weight* wgu, const rmi_weight* wd, const float* x,
                                       size_t m, float* out) {
  RMI_TRY(rmi_check_ctx(ctx));
  RMI_TRY(rmi_check_weight(wgu, RMI_GGML_Q8_0));
  RMI_TRY(rmi_check_weight(wd, RMI_GGML_Q8_0));
  if (m == 0) return RMI_OK;
  RMI_REQUIRE(x && out, RMI_ERR_BAD_HANDLE, "rmi_ffn_swiglu_q8_0: null buffer");
  std::lock_guard<std::mutex> lock(ctx->mu);
  float *dx, *dout;
  RMI_TRY(rmi_scratch(ctx, 5, m * wgu->n_in * 4, (void**)&dx));
  RMI_TRY(rmi_scratch(ctx, 6, m * wd->n_rows * 4, (void**)&dout));
  RMI_CUDA_CHECK(cudaMemcpyAsync(dx, x, m * wgu->n_in * 4, cudaMemcpyHostToDevice, ctx->stream));
  RMI_TRY(ffn_device(ctx, wgu, wd, dx, m, dout));
  RMI_CUDA_CHECK(cudaMemcpyAsync(out, dout, m * wd->n_rows * 4, cudaMemcpyDeviceToHost, ctx->stream));
  if (use_tensor_cores(ctx, m)) return rmi_check_dev_status(ctx, "rmi_ffn_swiglu_q8_0");
  RMI_CUDA_CHECK(cudaStreamSynchronize(ctx->stream));
  return RMI_OK;
}

static int32_t ensure_pipe(rmi_ctx* ctx) {
  if (ctx->pipe_ready) return RMI_OK;
  RMI_CUDA_CHECK(cudaStreamCreateWithFlags(&ctx->copy_in, cudaStreamNonBlocking));
  RMI_CUDA_CHECK(cudaStreamCreateWithFlags(&ctx->copy_out, cudaStreamNonBlocking));
  for (int i = 0; i < 2; i++) {
    RMI_CUDA_CHECK(cudaEventCreateWithFlags(&ctx->ev_in[i], cudaEventDisableTiming));
    RMI_CUDA_CHECK(cudaEventCreateWithFlags(&ctx->ev_compute[i], cudaEventDisableTiming));
    RMI_CUDA_CHECK(cudaEventCreateWithFlags(&ctx->ev_out[i], cudaEventDisableTiming));
  }
  ctx->pipe_ready = true;
  return RMI_OK;
}

// A run of FFN calls with the copies of neighbouring batches overlapped with the arithmetic:
// batch i is copied in on one stream while batch i-1 is computed on the context's stream and
// batch i-2 is copied out on a third (two device buffers per direction, events between them).
extern "C" int32_t rmi_ffn_swiglu_q8_0_pipelined(rmi_ctx* ctx, const rmi_weight* const* wgu,
                                                 const rmi_weight* const* wd, const float* const* x,
                                                 float* const* out, size_t n_batches, size_t m) {
  RMI_TRY(rmi_check_ctx(ctx));
  if (n_batches == 0 || m == 0) return RMI_OK;
  RMI_REQUIRE(wgu && wd && x && out, RMI_ERR_BAD_HANDLE, "rmi_ffn_swiglu_q8_0_pipelined: null argument");
  for (size_t i = 0; i < n_batches; i++) {
    RMI_TRY(rmi_check_weight(wgu[i], RMI_GGML_Q8_0));
    RMI_TRY(rmi_check_weight(wd[i], RMI_GGML_Q8_0));
    RMI_REQUIRE(x[i] && out[i], RMI_ERR_BAD_HANDLE, "rmi_ffn_swiglu_q8_0_pipelined: null buffer in batch %zu", i);
    RMI_REQUIRE(wgu[i]->n_in == wgu[0]->n_in && wd[i]->n_rows == wd[0]->n_rows, RMI_ERR_BAD_SHAPE,
                "rmi_ffn_swiglu_q8_0_pipelined: batch %zu has a different width", i);
  }
  std::lock_guard<std::mutex> lock(ctx->mu);
  RMI_TRY(ensure_pipe(ctx));
  const size_t in_bytes = m * wgu[0]->n_in * 4, out_bytes = m * wd[0]->n_rows * 4;
  const size_t in_slot = (in_bytes + 255) & ~(size_t)255, out_slot = (out_bytes + 255) & ~(size_t)255;
  uint8_t *dx, *dout;
  RMI_TRY(rmi_scratch(ctx, 5, 2 * in_slot, (void**)&dx));
  RMI_TRY(rmi_scratch(ctx, 6, 2 * out_slot, (void**)&dout));
  // work already queued on the context's stream may still use the scratch buffers
  RMI_CUDA_CHECK(cudaEventRecord(ctx->ev_compute[0], ctx->stream));
  RMI_CUDA_CHECK(cudaStreamWaitEvent(ctx->copy_in, ctx->ev_compute[0], 0));
  for (size_t i = 0; i < n_batches; i++) {
    const int b = (int)(i & 1);
    // dx[b] was read by the arithmetic of batch i-2
    if (i >= 2) RMI_CUDA_CHECK(cudaStreamWaitEvent(ctx->copy_in, ctx->ev_compute[b], 0));
    RMI_CUDA_CHECK(cudaMemcpyAsync(dx + b * in_slot, x[i], in_bytes, cudaMemcpyHostToDevice, ctx->copy_in));
    RMI_CUDA_CHECK(cudaEventRecord(ctx->ev_in[b], ctx->copy_in));
    RMI_CUDA_CHECK(cudaStreamWaitEvent(ctx->stream, ctx->ev_in[b], 0));
    // dout[b] was copied out for batch i-2
    if (i >= 2) RMI_CUDA_CHECK(cudaStreamWaitEvent(ctx->stream, ctx->ev_out[b], 0));
    RMI_TRY(ffn_device(ctx, wgu[i], wd[i], reinterpret_cast<const float*>(dx + b * in_slot), m,
                       reinterpret_cast<float*>(dout + b * out_slot)));
    RMI_CUDA_CHECK(cudaEventRecord(ctx->ev_compute[b], ctx->stream));
    RMI_CUDA_CHECK(cudaStreamWaitEvent(ctx->copy_out, ctx->ev_compute[b], 0));
    RMI_CUDA_CHECK(cudaMemcpyAsync(out[i], dout + b * out_slot, out_bytes, cudaMemcpyDeviceToHost, ctx->copy_out));
    RMI_CUDA_CHECK(cudaEventRecord(ctx->ev_out[b], ctx->copy_out));
  }
  RMI_CUDA_CHECK(cudaStreamSynchronize(ctx->copy_out));
  return rmi_check_dev_status(ctx, "rmi_ffn_swiglu_q8_0_pipelined");
}

extern "C" int32_t rmi_silu_mul(rmi_ctx* ctx, const float* gate, float* up, size_t n) {
  RMI_TRY(rmi_check_ctx(ctx));
  if (n == 0) return RMI_OK;
  RMI_REQUIRE(gate && up, RMI_ERR_BAD_HANDLE, "rmi_silu_mul: null buffer");
  std::lock_guard<std::mutex> lock(ctx->mu);
  size_t np = (n + 31) / 32 * 32;
  float *dg, *du;
  RMI_TRY(rmi_scratch(ctx, 5, np * 4, (void**)&dg));
  RMI_TRY(rmi_scratch(ctx, 6, np * 4, (void**)&du));
  RMI_CUDA_CHECK(cudaMemsetAsync(dg, 0, np * 4, ctx->stream));
  RMI_CUDA_CHECK(cudaMemsetAsync(du, 0, np * 4, ctx->stream));
  RMI_CUDA_CHECK(cudaMemcpyAsync(dg, gate, n * 4, cudaMemcpyHostToDevice, ctx->stream));
  RMI_CUDA_CHECK(cudaMemcpyAsync(du, up, n * 4, cudaMemcpyHostToDevice, ctx->stream));
  float* dact;
  RMI_TRY(rmi_scratch(ctx, 2, np * 4, (void**)&dact));
  RMI_TRY(launch_silu_mul_quantize(ctx, dg, du, np, 1, np, dact, nullptr, nullptr));
  RMI_CUDA_CHECK(cudaMemcpyAsync(up, dact, n * 4, cudaMemcpyDeviceToHost, ctx->stream));
  RMI_CUDA_CHECK(cudaStreamSynchronize(ctx->stream));
  return RMI_OK;
}

extern "C" int32_t rmi_unshard_cols_dev(rmi_ctx* ctx, const float* gathered, size_t g, size_t m, size_t npr,
                                        float* out) {
  RMI_TRY(rmi_check_ctx(ctx));
  RMI_REQUIRE(gathered && out, RMI_ERR_BAD_HANDLE, "rmi_unshard_cols_dev: null buffer");
  return launch_unshard_cols_vec(ctx, gathered, g, m, npr, out);
}
