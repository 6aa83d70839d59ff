// Peer-memory plumbing for the row-sharded matmul: one process per GPU on one node.
//
// Each rank owns the final [M, N] output buffer and a small flag array, both exported through
// CUDA IPC; every rank maps its peers' buffers and the matmul stores its column slice straight
// into all of them (rmi_matmul_q8_0_fanout_dev).  The exchange is closed by a flag round:
// rank r writes the epoch into slot r of every peer's flag array (release, system scope) and
// waits, with a time limit, until every slot of its own array shows the epoch.
#include "common.cuh"
#include "kernels.cuh"

#include <cstring>

namespace {

struct peer_flags {
  uint32_t* p[RMI_MAX_FANOUT];
};

struct peer_dsts {
  float* p[RMI_MAX_FANOUT];
};

// Pushes rows [0, n_rows) x columns [0, n_cols) of `src` (row stride `stride` floats; the caller has offset the
// pointers to the slab and to this rank's columns) into the same place of every peer's buffer with plain 16-byte
// stores over NVLink.  A few dozen CTAs next to the matmul of the next slab: the copy is bound by the links, not by
// the SMs.  blockIdx.y selects the peer, so the peers are written concurrently.
__global__ void __launch_bounds__(256)
    peer_push_kernel(const float* __restrict__ src, peer_dsts dst, size_t n_rows, size_t n_cols, size_t stride) {
  float* out = dst.p[blockIdx.y];
  const size_t c4 = n_cols / 4, total = n_rows * c4;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const size_t r = i / c4, c = (i % c4) * 4;
    const float4 v = *reinterpret_cast<const float4*>(src + r * stride + c);
    *reinterpret_cast<float4*>(out + r * stride + c) = v;
  }
}

__global__ void peer_signal_wait_kernel(peer_flags flags, int world, int rank, uint32_t epoch, uint64_t limit_ns,
                                        rmi_dev_status* status) {
  const int p = threadIdx.x;
  if (p >= world) return;
  // everything this GPU stored before this kernel (the matmul's peer stores) is ordered before the flag
  __threadfence_system();
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(flags.p[p] + rank), "r"(epoch) : "memory");
  uint64_t t0;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
  const uint32_t* mine = flags.p[rank] + p;
  for (;;) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(mine) : "memory");
    if ((int32_t)(v - epoch) >= 0) break;
    uint64_t now;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
    if (now - t0 > limit_ns) {  // give up: the host reads the status word
      if (atomicCAS(&status->code, 0, RMI_ERR_TIMEOUT) == 0) {
        status->where = 20;
        status->detail = p;
      }
      break;
    }
    __nanosleep(200);
  }
}

}  // namespace

extern "C" int32_t rmi_ipc_export(rmi_ctx* ctx, const void* dev_ptr, uint8_t* handle64) {
  RMI_TRY(rmi_check_ctx(ctx));
  RMI_REQUIRE(dev_ptr && handle64, RMI_ERR_BAD_HANDLE, "rmi_ipc_export: null argument");
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
  cudaIpcMemHandle_t h;
  RMI_CUDA_CHECK(cudaSetDevice(ctx->device));
  RMI_CUDA_CHECK(cudaIpcGetMemHandle(&h, const_cast<void*>(dev_ptr)));
  memcpy(handle64, &h, 64);
  return RMI_OK;
}

extern "C" int32_t rmi_ipc_open(rmi_ctx* ctx, const uint8_t* handle64, void** out_ptr) {
  RMI_TRY(rmi_check_ctx(ctx));
  RMI_REQUIRE(handle64 && out_ptr, RMI_ERR_BAD_HANDLE, "rmi_ipc_open: null argument");
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, 64);
  RMI_CUDA_CHECK(cudaSetDevice(ctx->device));
  RMI_CUDA_CHECK(cudaIpcOpenMemHandle(out_ptr, h, cudaIpcMemLazyEnablePeerAccess));
  return RMI_OK;
}

extern "C" int32_t rmi_ipc_close(rmi_ctx* ctx, void* ptr) {
  RMI_TRY(rmi_check_ctx(ctx));
  if (!ptr) return RMI_OK;
  RMI_CUDA_CHECK(cudaSetDevice(ctx->device));
  RMI_CUDA_CHECK(cudaIpcCloseMemHandle(ptr));
  return RMI_OK;
}

int32_t launch_peer_signal_wait(rmi_ctx* ctx, cudaStream_t stream, uint32_t* const* flags, int world, int rank,
                                uint32_t epoch) {
  RMI_REQUIRE(flags && world >= 1 && world <= RMI_MAX_FANOUT && rank >= 0 && rank < world, RMI_ERR_BAD_SHAPE,
              "peer flag round: world %d rank %d", world, rank);
  peer_flags f = {};
  for (int i = 0; i < world; i++) {
    RMI_REQUIRE(flags[i] != nullptr, RMI_ERR_BAD_HANDLE, "peer flag round: flag array %d is null", i);
    f.p[i] = flags[i];
  }
  peer_signal_wait_kernel<<<1, 32, 0, stream>>>(f, world, rank, epoch, ctx->wait_limit_ns, ctx->d_status);
  return rmi_post_launch(ctx, "peer_signal_wait");
}

extern "C" int32_t rmi_peer_signal_wait_dev(rmi_ctx* ctx, uint32_t* const* flags, int32_t world, int32_t rank,
                                            uint32_t epoch) {
  RMI_TRY(rmi_check_ctx(ctx));
  std::lock_guard<std::mutex> lock(ctx->mu);
  return launch_peer_signal_wait(ctx, ctx->stream, flags, world, rank, epoch);
}

extern "C" int32_t rmi_check_status(rmi_ctx* ctx) {
  RMI_TRY(rmi_check_ctx(ctx));
  std::lock_guard<std::mutex> lock(ctx->mu);
  return rmi_check_dev_status(ctx, "rmi_check_status");
}

// dsts: the peers' pointers to the same element as src (n_peers <= RMI_MAX_FANOUT - 1).  n_cols % 4 == 0, 16-byte aligned.
int32_t launch_peer_push(rmi_ctx* ctx, cudaStream_t stream, const float* src, float* const* dsts, int n_peers, size_t n_rows,
                         size_t n_cols, size_t stride) {
  if (n_peers <= 0 || n_rows == 0 || n_cols == 0) return RMI_OK;
  peer_dsts d = {};
  for (int i = 0; i < n_peers; i++) d.p[i] = dsts[i];
  // about a third of the SMs in total: enough loads in flight for the links, few enough to leave the matmul its issue slots
  unsigned per_peer = (unsigned)(ctx->sm_count / 3 / n_peers);
  if (per_peer < 4) per_peer = 4;
  peer_push_kernel<<<dim3(per_peer, (unsigned)n_peers), 256, 0, stream>>>(src, d, n_rows, n_cols, stride);
  return rmi_post_launch(ctx, "peer_push");
}
