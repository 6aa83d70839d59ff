// Row-sharded Q8_0 matmul across the GPUs of one node, one process (one context) per GPU.
//
// Rank r of g holds weight rows [r*N/g, (r+1)*N/g) -- the partition the reference uses across
// threads (src/ops/kernel/q8_0/parallel.rs:124-139) and plans across devices (PlacementSlice::Rows,
// src/format/load_plan.rs:19-22) -- and computes columns [r*N/g, (r+1)*N/g) of y [M, N].  Every rank
// ends up with the whole row-major [M, N] result.  Three exchanges are provided:
//
//   fused stores   the matmul's epilogue stores its column slice into every rank's result buffer
//                  through peer-mapped pointers (plain stores over NVLink); one flag round closes it.
//                  Best for small M (one launch, no copy).
//   peer copies    M is cut into slabs of rows; the matmul of slab i+1 runs on the context's stream
//                  while the copy engines push slab i's [rows, N/g] column slice into every peer's
//                  result buffer (2-D copies, no SM involved); one flag round at the end.
//   NCCL           ncclAllGather of the [M, N/g] shards into [g, M, N/g] followed by a local
//                  un-shard copy (rmi_allgather_cols_dev) with a communicator the host hands in.
//
// Result buffers alternate by round (two per rank).  A peer starts writing round k+2 into the buffer
// of round k only after it has seen this rank's flag of round k+1, and that flag is sent in stream
// order after everything this rank enqueued before its call of round k+1.  So a caller that
// enqueues its reads of round k's result on the context's stream before it calls round k+1 is safe
// without any further acknowledgement.
//
// No cluster-multicast load or store appears anywhere; peers' memory is touched by plain stores, by
// copy-engine copies and by NCCL only.
#include <dlfcn.h>

#include <cstring>
#include <new>

#include <cmath>
#include "common.cuh"
#include "kernels.cuh"

// ---------------------------------------------------------------- shard group

static constexpr uint32_t RMI_GROUP_MAGIC = 0x524d4947;  // "RMIG"
static constexpr int MAX_SLABS = 16;
static constexpr size_t HANDLE_BYTES = 64;
static constexpr size_t GROUP_HANDLE_BYTES = 3 * HANDLE_BYTES;  // result buffer 0, result buffer 1, flags

struct rmi_shard_group {
  uint32_t magic;
  int world, rank;
  size_t n_out, m_max;
  float* out[2];                        // this rank's result buffers [m_max, n_out]
  uint32_t* flags;                      // this rank's flag array (64 words, slot p written by rank p)
  float* peer_out[2][RMI_MAX_FANOUT];   // by rank; own entries are the local pointers
  uint32_t* peer_flags[RMI_MAX_FANOUT];
  bool connected;
  uint32_t epoch;
  cudaStream_t copy_stream;
  cudaEvent_t ev_slab[MAX_SLABS], ev_done;
};

static int32_t check_group(const rmi_shard_group* g) {
  RMI_REQUIRE(g != nullptr && g->magic == RMI_GROUP_MAGIC, RMI_ERR_BAD_HANDLE, "invalid rmi_shard_group handle");
  return RMI_OK;
}

static void free_group(rmi_shard_group* g, bool close_peers) {
  if (!g) return;
  if (close_peers && g->connected) {
    for (int p = 0; p < g->world; p++) {
      if (p == g->rank) continue;
      for (int b = 0; b < 2; b++)
        if (g->peer_out[b][p]) cudaIpcCloseMemHandle(g->peer_out[b][p]);
      if (g->peer_flags[p]) cudaIpcCloseMemHandle(g->peer_flags[p]);
    }
  }
  cudaFree(g->out[0]);
  cudaFree(g->out[1]);
  cudaFree(g->flags);
  if (g->copy_stream) cudaStreamDestroy(g->copy_stream);
  for (int i = 0; i < MAX_SLABS; i++)
    if (g->ev_slab[i]) cudaEventDestroy(g->ev_slab[i]);
  if (g->ev_done) cudaEventDestroy(g->ev_done);
  g->magic = 0;
  delete g;
}

extern "C" int32_t rmi_shard_group_create(rmi_ctx* ctx, int32_t world, int32_t rank, size_t n_out, size_t m_max,
                                          rmi_shard_group** out) {
  RMI_TRY(rmi_check_ctx(ctx));
  RMI_REQUIRE(out != nullptr, RMI_ERR_BAD_HANDLE, "rmi_shard_group_create: out is null");
  *out = nullptr;
  RMI_REQUIRE(world >= 1 && world <= RMI_MAX_FANOUT && rank >= 0 && rank < world, RMI_ERR_BAD_SHAPE,
              "world %d (1..%d) / rank %d", world, RMI_MAX_FANOUT, rank);
  RMI_REQUIRE(n_out > 0 && m_max > 0 && n_out % (size_t)world == 0, RMI_ERR_BAD_SHAPE,
              "n_out=%zu must be a positive multiple of the world size %d (equal shards)", n_out, world);
  rmi_shard_group* g = new (std::nothrow) rmi_shard_group();
  RMI_REQUIRE(g != nullptr, RMI_ERR_OOM, "host allocation failed");
  memset(g, 0, sizeof(*g));
  g->magic = RMI_GROUP_MAGIC;
  g->world = world;
  g->rank = rank;
  g->n_out = n_out;
  g->m_max = m_max;
  const size_t bytes = m_max * n_out * sizeof(float);
  cudaError_t e = cudaMalloc((void**)&g->out[0], bytes);
  if (e == cudaSuccess) e = cudaMalloc((void**)&g->out[1], bytes);
  if (e == cudaSuccess) e = cudaMalloc((void**)&g->flags, 256);
  if (e == cudaSuccess) e = cudaMemset(g->flags, 0, 256);
  if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&g->copy_stream, cudaStreamNonBlocking);
  for (int i = 0; i < MAX_SLABS && e == cudaSuccess; i++) e = cudaEventCreateWithFlags(&g->ev_slab[i], cudaEventDisableTiming);
  if (e == cudaSuccess) e = cudaEventCreateWithFlags(&g->ev_done, cudaEventDisableTiming);
  if (e != cudaSuccess) {
    (void)cudaGetLastError();
    rmi_set_error("shard group setup (2 x %zu bytes) failed: %s", bytes, cudaGetErrorString(e));
    free_group(g, false);
    return e == cudaErrorMemoryAllocation ? RMI_ERR_OOM : RMI_ERR_CUDA;
  }
  g->peer_out[0][rank] = g->out[0];
  g->peer_out[1][rank] = g->out[1];
  g->peer_flags[rank] = g->flags;
  g->connected = world == 1;
  *out = g;
  return RMI_OK;
}

extern "C" int32_t rmi_shard_group_export(rmi_ctx* ctx, const rmi_shard_group* g, uint8_t* handles192) {
  RMI_TRY(rmi_check_ctx(ctx));
  RMI_TRY(check_group(g));
  RMI_REQUIRE(handles192 != nullptr, RMI_ERR_BAD_HANDLE, "rmi_shard_group_export: null buffer");
  static_assert(sizeof(cudaIpcMemHandle_t) == HANDLE_BYTES, "IPC handle size");
  const void* ptrs[3] = {g->out[0], g->out[1], g->flags};
  for (int i = 0; i < 3; i++) {
    cudaIpcMemHandle_t h;
    RMI_CUDA_CHECK(cudaIpcGetMemHandle(&h, const_cast<void*>(ptrs[i])));
    memcpy(handles192 + i * HANDLE_BYTES, &h, HANDLE_BYTES);
  }
  return RMI_OK;
}

extern "C" int32_t rmi_shard_group_connect(rmi_ctx* ctx, rmi_shard_group* g, const uint8_t* all_handles) {
  RMI_TRY(rmi_check_ctx(ctx));
  RMI_TRY(check_group(g));
  RMI_REQUIRE(all_handles != nullptr, RMI_ERR_BAD_HANDLE, "rmi_shard_group_connect: null buffer");
  RMI_REQUIRE(!g->connected || g->world == 1, RMI_ERR_BAD_HANDLE, "shard group is already connected");
  for (int p = 0; p < g->world; p++) {
    if (p == g->rank) continue;
    const uint8_t* hp = all_handles + (size_t)p * GROUP_HANDLE_BYTES;
    void* mapped[3] = {nullptr, nullptr, nullptr};
    for (int i = 0; i < 3; i++) {
      cudaIpcMemHandle_t h;
      memcpy(&h, hp + i * HANDLE_BYTES, HANDLE_BYTES);
      cudaError_t e = cudaIpcOpenMemHandle(&mapped[i], h, cudaIpcMemLazyEnablePeerAccess);
      if (e != cudaSuccess) {
        (void)cudaGetLastError();
        rmi_set_error("mapping rank %d's buffer %d failed: %s", p, i, cudaGetErrorString(e));
        return RMI_ERR_CUDA;
      }
    }
    g->peer_out[0][p] = static_cast<float*>(mapped[0]);
    g->peer_out[1][p] = static_cast<float*>(mapped[1]);
    g->peer_flags[p] = static_cast<uint32_t*>(mapped[2]);
  }
  g->connected = true;
  return RMI_OK;
}

extern "C" int32_t rmi_shard_group_free(rmi_ctx* ctx, rmi_shard_group* g) {
  RMI_TRY(rmi_check_ctx(ctx));
  RMI_TRY(check_group(g));
  RMI_CUDA_CHECK(cudaStreamSynchronize(ctx->stream));
  RMI_CUDA_CHECK(cudaStreamSynchronize(g->copy_stream));
  free_group(g, true);
  return RMI_OK;
}

extern "C" int32_t rmi_shard_group_epoch(const rmi_shard_group* g, uint32_t* epoch) {
  RMI_TRY(check_group(g));
  if (epoch) *epoch = g->epoch;
  return RMI_OK;
}

// Slabs of the peer-copy exchange.  The matmul of a slab runs in whole waves of 128 x 64 tiles over the SMs, a slab's
// copies start when its matmul and the previous slab's copies are done, and the copy of the last slab is the part
// of the exchange that nothing overlaps.  The schedule is equal slabs of S row tiles (128 rows each) with the
// remainder last, S chosen by running that pipeline on a small cost model: waves(slab) = ceil(row tiles * column
// tiles / SMs), a wave = n_in / 128 K-slabs of 0.87 us, 12 us per launch, peer copies at 600 GB/s.
// (8 GPUs, M = 4096, 4096 columns per rank: 9 + 9 + 9 + 5 row tiles = 15 waves instead of the 16 of four 1024-row
// slabs, and a 640-row tail instead of a 1024-row one.)  Returns the number of slabs; rows[i] are their sizes.
static size_t slab_schedule(size_t m, size_t npr, size_t n_in, int world, size_t sm_count, size_t* rows) {
  const size_t mt = (m + 127) / 128;   // row tiles
  if (m <= 512 || mt < 8) {
    rows[0] = m;
    return 1;
  }
  const double col_tiles = (double)((npr + 63) / 64);
  const double wave_us = (double)((n_in + 127) / 128) * 0.87, launch_us = 12.0;
  const double copy_us_per_tile = 128.0 * (double)npr * 4.0 * (double)(world - 1) / 600e3;
  size_t best_s = mt;
  double best_end = 1e30;
  for (size_t S = 4; S <= mt; S++) {
    const size_t n_full = mt / S, rem = mt % S;
    if (n_full + (rem ? 1 : 0) > (size_t)MAX_SLABS) continue;
    double t = 0.0, copy_end = 0.0;
    for (size_t i = 0; i < n_full + (rem ? 1 : 0); i++) {
      const size_t tiles = i < n_full ? S : rem;
      t += std::ceil((double)tiles * col_tiles / (double)sm_count - 1e-9) * wave_us + launch_us;
      copy_end = (t > copy_end ? t : copy_end) + (double)tiles * copy_us_per_tile;
    }
    if (copy_end < best_end - 1e-9) {
      best_end = copy_end;
      best_s = S;
    }
  }
  size_t n = 0, left = m;
  while (left > 0) {
    const size_t take = left < best_s * 128 ? left : best_s * 128;
    rows[n++] = take;
    left -= take;
  }
  return n;
}

extern "C" int32_t rmi_matmul_q8_0_sharded_dev(rmi_ctx* ctx, rmi_shard_group* g, const rmi_weight* w, const float* x,
                                               size_t m, int32_t exchange, float** result) {
  RMI_TRY(rmi_check_ctx(ctx));
  RMI_TRY(check_group(g));
  RMI_TRY(rmi_check_weight(w, RMI_GGML_Q8_0));
  RMI_REQUIRE(g->connected, RMI_ERR_BAD_HANDLE, "shard group is not connected (rmi_shard_group_connect)");
  RMI_REQUIRE(exchange == RMI_EXCHANGE_FUSED_STORES || exchange == RMI_EXCHANGE_PEER_COPY || exchange == RMI_EXCHANGE_PEER_PUSH,
              RMI_ERR_UNSUPPORTED, "unknown exchange %d", exchange);
  const size_t npr = g->n_out / (size_t)g->world;
  RMI_REQUIRE(w->n_rows == npr, RMI_ERR_BAD_SHAPE, "weight shard has %zu rows, the group expects %zu", w->n_rows, npr);
  RMI_REQUIRE(m >= 1 && m <= g->m_max, RMI_ERR_BAD_SHAPE, "m=%zu outside 1..%zu", m, g->m_max);
  RMI_REQUIRE(x != nullptr, RMI_ERR_BAD_HANDLE, "rmi_matmul_q8_0_sharded_dev: null input");
  std::lock_guard<std::mutex> lock(ctx->mu);
  const uint32_t epoch = g->epoch + 1;
  const int par = (int)(epoch & 1);
  float* own = g->out[par];
  const size_t col_off = (size_t)g->rank * npr;
  if (exchange == RMI_EXCHANGE_FUSED_STORES || g->world == 1) {
    // own buffer first (the primary store), then the peers starting at rank+1 so that the ranks do not all
    // write to the same peer at the same time
    ctx->fanout.n = g->world - 1;
    for (int i = 1; i < g->world; i++) {
      const float* peer = g->peer_out[par][(g->rank + i) % g->world];
      ctx->fanout.delta[i - 1] = (long long)(reinterpret_cast<const char*>(peer) - reinterpret_cast<const char*>(own));
    }
    const int32_t st = matmul_q8_0_device(ctx, w, x, m, own + col_off, g->n_out);
    ctx->fanout = out_fanout{};
    RMI_TRY(st);
    RMI_TRY(launch_peer_signal_wait(ctx, ctx->stream, g->peer_flags, g->world, g->rank, epoch));
  } else {
    size_t rows[MAX_SLABS];
    const size_t n_slabs = slab_schedule(m, npr, w->n_in, g->world, (size_t)ctx->sm_count, rows);
    size_t r0 = 0;
    for (size_t s = 0; s < n_slabs; s++) {
      const size_t nr = rows[s];
      RMI_TRY(matmul_q8_0_device(ctx, w, x + r0 * w->n_in, nr, own + r0 * g->n_out + col_off, g->n_out));
      RMI_CUDA_CHECK(cudaEventRecord(g->ev_slab[s], ctx->stream));
      RMI_CUDA_CHECK(cudaStreamWaitEvent(g->copy_stream, g->ev_slab[s], 0));
      if (exchange == RMI_EXCHANGE_PEER_PUSH && npr % 4 == 0 && g->n_out % 4 == 0) {
        // one kernel stores the slab into all peers at once (peers in rank order starting after this rank)
        float* dsts[RMI_MAX_FANOUT];
        for (int i = 1; i < g->world; i++) dsts[i - 1] = g->peer_out[par][(g->rank + i) % g->world] + r0 * g->n_out + col_off;
        RMI_TRY(launch_peer_push(ctx, g->copy_stream, own + r0 * g->n_out + col_off, dsts, g->world - 1, nr, npr, g->n_out));
      } else {
        for (int i = 1; i < g->world; i++) {
          float* peer = g->peer_out[par][(g->rank + i) % g->world];
          RMI_CUDA_CHECK(cudaMemcpy2DAsync(peer + r0 * g->n_out + col_off, g->n_out * sizeof(float),
                                           own + r0 * g->n_out + col_off, g->n_out * sizeof(float), npr * sizeof(float), nr,
                                           cudaMemcpyDeviceToDevice, g->copy_stream));
        }
      }
      r0 += nr;
    }
    RMI_TRY(launch_peer_signal_wait(ctx, g->copy_stream, g->peer_flags, g->world, g->rank, epoch));
    RMI_CUDA_CHECK(cudaEventRecord(g->ev_done, g->copy_stream));
    RMI_CUDA_CHECK(cudaStreamWaitEvent(ctx->stream, g->ev_done, 0));
  }
  g->epoch = epoch;
  if (result) *result = own;
  return RMI_OK;
}

// ---------------------------------------------------------------- un-shard

namespace {

// gathered [g][m][npr] -> out [m][g*npr]; one CTA row per (rank, row), 16-byte accesses when aligned
__global__ void unshard_cols_vec_kernel(const float* __restrict__ gathered, size_t g, size_t m, size_t npr,
                                        float* __restrict__ out) {
  const size_t row = blockIdx.y, rank = blockIdx.z;
  const float* src = gathered + (rank * m + row) * npr;
  float* dst = out + row * (g * npr) + rank * npr;
  const size_t i = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * 4;
  if (i + 4 <= npr) {
    *reinterpret_cast<float4*>(dst + i) = *reinterpret_cast<const float4*>(src + i);
  } else {
    for (size_t k = i; k < npr; k++) dst[k] = src[k];
  }
}

}  // namespace

int32_t launch_unshard_cols_vec(rmi_ctx* ctx, const float* gathered, size_t g, size_t m, size_t npr, float* out) {
  if (g * m * npr == 0) return RMI_OK;
  if (npr % 4 != 0 || m > 65535 || (reinterpret_cast<uintptr_t>(gathered) & 15) || (reinterpret_cast<uintptr_t>(out) & 15))
    return launch_unshard_cols(ctx, gathered, g, m, npr, out);
  dim3 grid((unsigned)((npr / 4 + 255) / 256), (unsigned)m, (unsigned)g);
  unshard_cols_vec_kernel<<<grid, 256, 0, ctx->stream>>>(gathered, g, m, npr, out);
  return rmi_post_launch(ctx, "unshard_cols");
}

// ---------------------------------------------------------------- NCCL (resolved at run time)
//
// The library is not linked against NCCL: the few entry points used are looked up in the libnccl.so.2
// the process has already loaded (a host that owns a communicator has one), else loaded by name.  The
// declarations below restate NCCL's public C API (nccl.h): ncclResult_t 0 = success, ncclFloat32 = 7.

namespace {

struct nccl_unique_id {
  char internal[128];
};
typedef void* nccl_comm_t;
typedef int (*fn_get_unique_id)(nccl_unique_id*);
typedef int (*fn_comm_init_rank)(nccl_comm_t*, int, nccl_unique_id, int);
typedef int (*fn_comm_destroy)(nccl_comm_t);
typedef int (*fn_all_gather)(const void*, void*, size_t, int, nccl_comm_t, cudaStream_t);
typedef const char* (*fn_get_error_string)(int);

struct nccl_api {
  void* handle;
  fn_get_unique_id get_unique_id;
  fn_comm_init_rank comm_init_rank;
  fn_comm_destroy comm_destroy;
  fn_all_gather all_gather;
  fn_get_error_string error_string;
};

std::mutex g_nccl_mu;
nccl_api g_nccl = {};

int32_t nccl_load(const nccl_api** out) {
  std::lock_guard<std::mutex> lock(g_nccl_mu);
  if (!g_nccl.handle) {
    void* h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_NOLOAD);
    if (!h) h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
    if (!h) h = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
    RMI_REQUIRE(h != nullptr, RMI_ERR_UNSUPPORTED, "libnccl.so.2 could not be loaded: %s", dlerror());
    nccl_api a = {};
    a.handle = h;
    a.get_unique_id = (fn_get_unique_id)dlsym(h, "ncclGetUniqueId");
    a.comm_init_rank = (fn_comm_init_rank)dlsym(h, "ncclCommInitRank");
    a.comm_destroy = (fn_comm_destroy)dlsym(h, "ncclCommDestroy");
    a.all_gather = (fn_all_gather)dlsym(h, "ncclAllGather");
    a.error_string = (fn_get_error_string)dlsym(h, "ncclGetErrorString");
    RMI_REQUIRE(a.get_unique_id && a.comm_init_rank && a.comm_destroy && a.all_gather && a.error_string, RMI_ERR_UNSUPPORTED,
                "libnccl.so.2 lacks an expected entry point");
    g_nccl = a;
  }
  *out = &g_nccl;
  return RMI_OK;
}

}  // namespace

#define RMI_NCCL_CHECK(api, expr)                                                    \
  do {                                                                               \
    int _r = (expr);                                                                 \
    if (_r != 0) {                                                                   \
      rmi_set_error("%s failed: %s", #expr, (api)->error_string(_r));                \
      return RMI_ERR_CUDA;                                                           \
    }                                                                                \
  } while (0)

extern "C" int32_t rmi_nccl_unique_id(uint8_t* id128) {
  RMI_REQUIRE(id128 != nullptr, RMI_ERR_BAD_HANDLE, "rmi_nccl_unique_id: null buffer");
  const nccl_api* api;
  RMI_TRY(nccl_load(&api));
  nccl_unique_id id;
  RMI_NCCL_CHECK(api, api->get_unique_id(&id));
  memcpy(id128, &id, 128);
  return RMI_OK;
}

extern "C" int32_t rmi_nccl_comm_create(rmi_ctx* ctx, const uint8_t* id128, int32_t world, int32_t rank, void** comm) {
  RMI_TRY(rmi_check_ctx(ctx));  // makes the context's device current, which is what ncclCommInitRank binds to
  RMI_REQUIRE(id128 && comm, RMI_ERR_BAD_HANDLE, "rmi_nccl_comm_create: null argument");
  RMI_REQUIRE(world >= 1 && rank >= 0 && rank < world, RMI_ERR_BAD_SHAPE, "world %d / rank %d", world, rank);
  const nccl_api* api;
  RMI_TRY(nccl_load(&api));
  nccl_unique_id id;
  memcpy(&id, id128, 128);
  nccl_comm_t c = nullptr;
  RMI_NCCL_CHECK(api, api->comm_init_rank(&c, world, id, rank));
  *comm = c;
  return RMI_OK;
}

extern "C" int32_t rmi_nccl_comm_destroy(void* comm) {
  if (!comm) return RMI_OK;
  const nccl_api* api;
  RMI_TRY(nccl_load(&api));
  RMI_NCCL_CHECK(api, api->comm_destroy(comm));
  return RMI_OK;
}

extern "C" int32_t rmi_allgather_cols_dev(rmi_ctx* ctx, void* nccl_comm, const float* y_local, size_t m, size_t n_per_rank,
                                          int32_t world, float* gathered, float* out) {
  RMI_TRY(rmi_check_ctx(ctx));
  RMI_REQUIRE(nccl_comm && y_local && out, RMI_ERR_BAD_HANDLE, "rmi_allgather_cols_dev: null argument");
  RMI_REQUIRE(world >= 1, RMI_ERR_BAD_SHAPE, "world %d", world);
  if (m == 0 || n_per_rank == 0) return RMI_OK;
  RMI_REQUIRE(m == 1 || gathered != nullptr, RMI_ERR_BAD_HANDLE,
              "rmi_allgather_cols_dev: m > 1 needs the [world, m, n_per_rank] staging buffer");
  const nccl_api* api;
  RMI_TRY(nccl_load(&api));
  std::lock_guard<std::mutex> lock(ctx->mu);
  // one row: the shards are already contiguous pieces of the result
  float* dst = m == 1 ? out : gathered;
  RMI_NCCL_CHECK(api, api->all_gather(y_local, dst, m * n_per_rank, /* ncclFloat32 */ 7, nccl_comm, ctx->stream));
  if (m == 1) return RMI_OK;
  return launch_unshard_cols_vec(ctx, gathered, (size_t)world, m, n_per_rank, out);
}
