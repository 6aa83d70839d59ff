// Shared host/device helpers for librmi_cuda.so (sm_100a only).
//
// The whole library is compiled with -fmad=false: the reference (Rust) never fuses a*b+c
// unless it calls mul_add, and its bit patterns depend on that.  Every intended fused
// multiply-add is written as __fmaf_rn / fma().
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>
#include <mutex>
#include <string>
#include <vector>

#include "../../include/rmi_cuda.h"

// ---------------------------------------------------------------- errors

void rmi_set_error(const char* fmt, ...);

#define RMI_CUDA_CHECK(expr)                                                              \
  do {                                                                                    \
    cudaError_t _e = (expr);                                                              \
    if (_e != cudaSuccess) {                                                              \
      rmi_set_error("%s failed: %s (%s:%d)", #expr, cudaGetErrorString(_e), __FILE__,      \
                    __LINE__);                                                            \
      return RMI_ERR_CUDA;                                                                \
    }                                                                                     \
  } while (0)

#define RMI_REQUIRE(cond, code, ...) \
  do {                               \
    if (!(cond)) {                   \
      rmi_set_error(__VA_ARGS__);    \
      return (code);                 \
    }                                \
  } while (0)

#define RMI_TRY(expr)              \
  do {                             \
    int32_t _s = (expr);           \
    if (_s != RMI_OK) return _s;   \
  } while (0)

// ---------------------------------------------------------------- handles

static constexpr uint32_t RMI_CTX_MAGIC = 0x524d4943;     // "RMIC"
static constexpr uint32_t RMI_WEIGHT_MAGIC = 0x524d4957;  // "RMIW"

// Device-side status word written by kernels that contain bounded waits.
struct rmi_dev_status {
  int32_t code;    // 0 = ok
  int32_t where;   // site id of the wait that gave up
  int32_t detail;  // e.g. tile index
  int32_t pad;
  unsigned long long limit_ns;  // time limit of a bounded wait; written by the host, kept across clears
};
static constexpr size_t RMI_STATUS_CLEAR_BYTES = 16;  // code, where, detail, pad

struct rmi_prof_rec {
  const char* tag;
  cudaEvent_t a, b;
};

// Extra copies of every f32 output store of a matmul: `delta[i]` is the byte offset from the primary
// output buffer to copy i (another buffer of the same layout, possibly in a peer GPU's memory).
constexpr int RMI_MAX_FANOUT = 8;
struct out_fanout {
  int n;
  long long delta[RMI_MAX_FANOUT - 1];
};

struct rmi_ctx {
  uint32_t magic;
  int device;
  int sm_count;
  size_t l2_bytes;
  size_t mem_bytes;
  size_t smem_optin;
  cudaStream_t own_stream;
  cudaStream_t stream;
  int sem;
  bool prefill_exact;  // AVX2 semantics: keep m > 32 on the bit-exact CUDA-core kernels
  uint64_t wait_limit_ns;  // time limit of every bounded device-side wait (default 2 s)
  std::atomic<uint64_t> launches;
  std::mutex mu;
  rmi_dev_status* d_status;  // device
  rmi_dev_status* h_status;  // pinned host mirror
  // growable scratch owned by the context (activations in quantized form etc.)
  void* scratch[8];
  size_t scratch_bytes[8];
  // optional per-kernel timing (rmi_prof_*): event pairs recorded around tagged launches
  bool prof_on;
  std::vector<rmi_prof_rec> prof;
  // decode chain: launch kernels with programmatic stream serialization (see pdl_wait below)
  bool pdl;
  // set by rmi_matmul_q8_0_fanout_dev for the duration of its launches
  out_fanout fanout;
  // copy streams and events of the pipelined host entry point (created on first use)
  cudaStream_t copy_in, copy_out;
  cudaEvent_t ev_in[2], ev_compute[2], ev_out[2];
  bool pipe_ready;
};

// Q8_0 / Q4_K weight resident in HBM.
//
// Q8_0 "tile16" layout: rows are grouped in tiles of 16.  For tile t and 32-block b the
// record at ((t * blocks + b) * 544) holds 16 f16 scales (32 B, row r at +2r) followed by
// 16 rows x 32 int8 (row r at 32 + 32r).  A warp streams records linearly: every 16-byte
// lane load is aligned and each 544-byte record is one contiguous burst.  Rows beyond
// n_rows inside the last tile are zero.
//
// Q8_0 "umma" layout (built on first use by the tcgen05 GEMM): per (128-row tile, 128-byte
// K slab) one 16 KiB image in the tcgen05 K-major no-swizzle core-matrix order
// (8 rows x 16 B core matrices, LBO 128 B along K, SBO 1024 B along rows), plus f32 scales
// [n_tiles][blocks][128].
//
// Q4_K layout: the 144-byte super-blocks unchanged, row-major (already 16-byte aligned).
struct rmi_weight {
  uint32_t magic;
  int ggml_type;
  size_t n_in;
  size_t n_rows;
  size_t n_tiles16;
  uint8_t* d_tile16;   // Q8_0
  size_t tile16_bytes;
  uint8_t* d_umma_q;   // Q8_0, lazily built
  float* d_umma_s;
  uint8_t* d_umma_gu_q;  // v-stacked gate|up weight in gate/up-interleaved row order (lazily built)
  float* d_umma_gu_s;
  size_t umma_bytes;
  uint8_t* d_raw;      // Q4_K
  size_t raw_bytes;
  // v-stack provenance (rows of a then rows of b); n_rows_a == 0 when not fused
  size_t n_rows_a;
};

static constexpr int Q8_REC_BYTES = 544;  // 32 B scales + 16 x 32 B quants

int32_t rmi_check_ctx(rmi_ctx* ctx);
int32_t rmi_check_weight(const rmi_weight* w, int ggml_type);
int32_t rmi_scratch(rmi_ctx* ctx, int slot, size_t bytes, void** out);
int32_t rmi_post_launch(rmi_ctx* ctx, const char* what);
int32_t rmi_check_dev_status(rmi_ctx* ctx, const char* what);
// Returns a record index (or -1 when timing is off); pass it to rmi_prof_end after the launch.
int rmi_prof_begin(rmi_ctx* ctx, const char* tag);
void rmi_prof_end(rmi_ctx* ctx, int idx);

// ---------------------------------------------------------------- device helpers

#ifdef __CUDACC__

// Programmatic dependent launch.  A kernel launched with the programmatic-serialization
// attribute may start while its predecessor in the stream is still running; it must call
// pdl_wait() before it touches anything the predecessor writes (or still reads).  Code before
// the wait may only read data that no kernel of the chain writes (weights) and use shared
// memory.  Without the launch attribute both calls are no-ops.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// Launch through cudaLaunchKernelEx so that the attribute can be attached when ctx->pdl is set.
template <typename... KArgs, typename... Args>
static inline cudaError_t rmi_launch(const rmi_ctx* ctx, void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                     Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = ctx->stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = ctx->pdl ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);
}

// One f32 result to the primary output and to every extra copy.
__device__ __forceinline__ void store_fanout(float* o, float v, const out_fanout& fo) {
  *o = v;
  if (fo.n == 0) return;
  // static indices: a dynamically indexed by-value struct would be copied to local memory in every thread
#pragma unroll
  for (int i = 0; i < RMI_MAX_FANOUT - 1; i++)
    if (i < fo.n) *reinterpret_cast<float*>(reinterpret_cast<char*>(o) + fo.delta[i]) = v;
}

// IEEE f16 -> f32 (exact)
__device__ __forceinline__ float f16_bits_to_f32(uint16_t h) {
  return __half2float(__ushort_as_half(h));
}
// f32 -> f16 round-to-nearest-even -> f32
__device__ __forceinline__ float f16_round_trip(float v) {
  return __half2float(__float2half_rn(v));
}
__device__ __forceinline__ uint16_t f32_to_f16_bits(float v) {
  return __half_as_ushort(__float2half_rn(v));
}

// Correctly rounded f32 exponential: exp in double, one rounding to f32.
__device__ __forceinline__ float exp_cr(float x) { return (float)exp((double)x); }

// int32 -> f32 for |v| < 2^22 without the conversion pipe: 0x4B400000 is 12582912.0f and
// adding a small integer to its bit pattern stays exact.
__device__ __forceinline__ float small_int_to_f32(int v) {
  return __fsub_rn(__int_as_float(v + 0x4B400000), 12582912.0f);
}

__device__ __forceinline__ int dp4a_s8(int a, int b, int c) { return __dp4a(a, b, c); }

// src/ops/quant/q8_0.rs: one value of a 32-block given the block's inverse scale
template <int SEM>
__device__ __forceinline__ int q8_quant_value(float x, float inv) {
  if (SEM == RMI_SEM_AVX2) {
    float r = rintf(__fmul_rn(x, inv));
    r = fminf(fmaxf(r, -128.0f), 127.0f);
    return (int)r;
  } else if (SEM == RMI_SEM_NEON) {
    float c = fminf(fmaxf(__fmul_rn(x, inv), -127.0f), 127.0f);
    int r = __float2int_rn(c);
    return max(-127, min(127, r));
  } else {
    float r = roundf(__fmul_rn(x, inv));
    r = fminf(fmaxf(r, -128.0f), 127.0f);
    return (int)r;
  }
}
// (d stored as f16, inverse used for rounding) from the block's amax
template <int SEM>
__device__ __forceinline__ void q8_scale_pair(float amax, float* d, float* inv) {
  if (SEM == RMI_SEM_AVX2) {
    *d = amax == 0.0f ? 0.0f : __fdiv_rn(amax, 127.0f);
    *inv = amax == 0.0f ? 0.0f : __fdiv_rn(127.0f, amax);
  } else if (SEM == RMI_SEM_NEON) {
    *d = __fdiv_rn(amax, 127.0f);
    *inv = *d > 0.0f ? __fdiv_rn(1.0f, *d) : 0.0f;
  } else {
    *d = amax == 0.0f ? 0.0f : __fdiv_rn(amax, 127.0f);
    *inv = *d == 0.0f ? 0.0f : __fdiv_rn(1.0f, *d);
  }
}

#endif  // __CUDACC__
