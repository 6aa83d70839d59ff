// rmi_matmul_q8_0_dev_noalloc: the f32-activation Q8_0 matmul for callers that must not
// allocate device memory.
//
// Who needs this: a host program that has already handed the whole GPU to its own memory
// manager (a serving engine's KV-cache pool, a framework allocator sized to the device) has
// nothing left for a plug-in's cudaMalloc -- the call fails, or worse succeeds by taking memory
// the host counted on -- and a latency-critical loop cannot afford the device-wide
// synchronisation that cudaMalloc and cudaFree imply.  The regular entry point
// (rmi_matmul_q8_0_dev) keeps its quantized activations in context scratch that grows with
// cudaMalloc on demand; this variant keeps them in a fixed array that is part of the library
// image instead.
//
// The array is a file-scope __device__ object: every GPU that loads the library holds its
// 576 KiB until the process exits.  Host code may not pass the array's name to a kernel (on
// the host the name is only a handle for the runtime); the device address is looked up with
// cudaGetSymbolAddress, once per device, while that device is current, and that pointer is
// what the kernels receive.  The look-up happens inside the first call on each device, so make
// that first call outside any stream capture.
//
// All calls on a device share the one array and nothing in it is ever cleared: each call's
// quantizer writes every byte the same call's matmul reads, so stale contents of an earlier
// call are never observed.  For the same reason two calls that overlap on the GPU (different
// streams, or different contexts on one device) race on the array; callers must order them.
#include <mutex>

#include "common.cuh"
#include "kernels.cuh"

namespace {

constexpr size_t NOALLOC_MAX_Q8_BYTES = 512 * 1024;                 // m * n_in
constexpr size_t NOALLOC_SCALE_BYTES = NOALLOC_MAX_Q8_BYTES / 32 * 4;  // one f32 per 32 values
constexpr int NOALLOC_MAX_DEVICES = 64;

static __device__ __align__(256) uint8_t g_noalloc_scratch[NOALLOC_MAX_Q8_BYTES + NOALLOC_SCALE_BYTES];

std::mutex g_setup_mu;
uint8_t* g_scratch_dev_ptr[NOALLOC_MAX_DEVICES] = {};

// Device address of the array on `device` (which must be current); resolved once per device.
int32_t scratch_address(int device, uint8_t** out) {
  RMI_REQUIRE(device >= 0 && device < NOALLOC_MAX_DEVICES, RMI_ERR_UNSUPPORTED, "device index %d is not supported", device);
  std::lock_guard<std::mutex> lock(g_setup_mu);
  if (g_scratch_dev_ptr[device] == nullptr) {
    void* p = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
    if (e != cudaSuccess || p == nullptr) {
      rmi_set_error("cudaGetSymbolAddress for the fixed scratch array failed: %s", cudaGetErrorString(e));
      return RMI_ERR_CUDA;
    }
    g_scratch_dev_ptr[device] = static_cast<uint8_t*>(p);
  }
  *out = g_scratch_dev_ptr[device];
  return RMI_OK;
}

}  // namespace

extern "C" int32_t rmi_matmul_q8_0_dev_noalloc(rmi_ctx* ctx, const rmi_weight* w, const float* x, size_t m,
                                               float* output) {
  RMI_TRY(rmi_check_ctx(ctx));  // also makes the context's device current
  RMI_TRY(rmi_check_weight(w, RMI_GGML_Q8_0));
  if (m == 0 || w->n_rows == 0) return RMI_OK;
  RMI_REQUIRE(x != nullptr && output != nullptr, RMI_ERR_BAD_HANDLE, "rmi_matmul_q8_0_dev_noalloc: null buffer");
  RMI_REQUIRE(m <= 32, RMI_ERR_BAD_SHAPE, "the allocation-free matmul handles at most 32 activation rows, got %zu", m);
  RMI_REQUIRE(m * w->n_in <= NOALLOC_MAX_Q8_BYTES, RMI_ERR_BAD_SHAPE,
              "m * n_in = %zu exceeds the fixed scratch array (%zu values); use rmi_matmul_q8_0_dev", m * w->n_in,
              NOALLOC_MAX_Q8_BYTES);
  RMI_REQUIRE(!ctx->prof_on, RMI_ERR_UNSUPPORTED, "per-kernel timing creates CUDA events; disable it for the allocation-free call");
  uint8_t* scratch = nullptr;
  RMI_TRY(scratch_address(ctx->device, &scratch));
  uint8_t* q8 = scratch;
  float* scales = reinterpret_cast<float*>(scratch + NOALLOC_MAX_Q8_BYTES);
  std::lock_guard<std::mutex> lock(ctx->mu);
  RMI_TRY(launch_q8_quantize(ctx, x, m, w->n_in, q8, scales, 0));
  return launch_q8_gemv(ctx, w, q8, scales, m, output, w->n_rows, 0, w->n_rows);
}
