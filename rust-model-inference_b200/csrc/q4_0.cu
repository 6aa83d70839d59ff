// Q4_0 x Q8_0 matmul: exact int32 block dots of (nibble - 8) with the Q8_0 activation and the reference's
// f32 chain  sum += (f32(dot) * d) * scale  in block order.
//
// Reference (paths inside the reference project): src/ops/kernel/q4_0/scalar.rs:13-53; the AVX2 kernel
// (q4_0/avx2.rs:25-108) is bit-identical to it by contract (no FMA, block-by-block accumulation), so there is
// one semantics.  src/ops/kernel/q4_0/mod.rs:29-80 is the Kernel impl with its (ith, nth) partition.
//
// Device layout: the 18-byte blocks (f16 d | 16 nibble bytes), 2-byte aligned in a GGUF file, are padded to
// 20 bytes at upload (f16 d | 2 pad bytes | 16 nibble bytes) so that the nibble words are 4-byte aligned.
#include "common.cuh"
#include "kernels.cuh"

namespace {

constexpr int Q4_0_DEV_BYTES = 20;

// One warp per weight row.  The blocks are taken 32 at a time: lane l computes the product of block b0 + l
// (all 32 values: eight dp4a), then lane 0 adds the 32 products to the row sum in block order.
__global__ void q4_0_matmul_kernel(const uint8_t* __restrict__ w, size_t blocks, size_t n_rows,
                                   const uint8_t* __restrict__ xq, const float* __restrict__ xs,
                                   float* __restrict__ out, size_t row_begin, size_t row_end) {
  const size_t row = row_begin + ((size_t)blockIdx.x * blockDim.x + threadIdx.x) / 32;
  const int lane = threadIdx.x & 31;
  const size_t t = blockIdx.y;
  if (row >= row_end) return;
  const uint8_t* wrow = w + row * blocks * Q4_0_DEV_BYTES;
  const uint8_t* xrow = xq + t * blocks * 32;
  const float* srow = xs + t * blocks;
  float sum = 0.0f;
  for (size_t b0 = 0; b0 < blocks; b0 += 32) {
    const size_t b = b0 + lane;
    float prod = 0.0f;
    if (b < blocks) {
      const uint8_t* blk = wrow + b * Q4_0_DEV_BYTES;
      const float d = f16_bits_to_f32(*reinterpret_cast<const uint16_t*>(blk));
      const uint32_t* qw = reinterpret_cast<const uint32_t*>(blk + 4);
      const int* y = reinterpret_cast<const int*>(xrow + b * 32);
      int dot = 0, ysum = 0;
#pragma unroll
      for (int k = 0; k < 4; k++) {
        const uint32_t q = qw[k];
        const int ylo = y[k], yhi = y[4 + k];
        dot = dp4a_s8((int)(q & 0x0F0F0F0Fu), ylo, dot);         // values 4k..4k+3: low nibbles
        dot = dp4a_s8((int)((q >> 4) & 0x0F0F0F0Fu), yhi, dot);  // values 16+4k..: high nibbles
        ysum = dp4a_s8(0x01010101, ylo, ysum);
        ysum = dp4a_s8(0x01010101, yhi, ysum);
      }
      dot -= 8 * ysum;  // sum (nibble - 8) * y
      prod = __fmul_rn(__fmul_rn((float)dot, d), srow[b]);
    }
    const int n = blocks - b0 < 32 ? (int)(blocks - b0) : 32;
    for (int l = 0; l < n; l++) sum = __fadd_rn(sum, __shfl_sync(0xffffffffu, prod, l));
  }
  if (lane == 0) out[t * n_rows + row] = sum;
}

// embedding_lookup_q4_0 (src/ops/embedding.rs:24-38): one CTA per requested row, ((nibble as f32) - 8) * d
__global__ void q4_0_embedding_kernel(const uint8_t* __restrict__ w, size_t blocks, const uint32_t* __restrict__ ids,
                                      float* __restrict__ out) {
  const uint8_t* row = w + (size_t)ids[blockIdx.x] * blocks * Q4_0_DEV_BYTES;
  for (size_t i = threadIdx.x; i < blocks * 16; i += blockDim.x) {
    const uint8_t* blk = row + (i / 16) * Q4_0_DEV_BYTES;
    const float d = f16_bits_to_f32(*reinterpret_cast<const uint16_t*>(blk));
    const uint8_t q = blk[4 + (i % 16)];
    float* o = out + (size_t)blockIdx.x * blocks * 32 + (i / 16) * 32 + (i % 16);
    o[0] = __fmul_rn(__fsub_rn((float)(q & 0x0F), 8.0f), d);
    o[16] = __fmul_rn(__fsub_rn((float)(q >> 4), 8.0f), d);
  }
}

}  // namespace

int32_t launch_q4_0_embedding(rmi_ctx* ctx, const rmi_weight* w, const uint32_t* ids, size_t m, float* out) {
  if (m == 0) return RMI_OK;
  q4_0_embedding_kernel<<<(unsigned)m, 256, 0, ctx->stream>>>(w->d_raw, w->n_in / 32, ids, out);
  return rmi_post_launch(ctx, "q4_0_embedding");
}

size_t q4_0_device_block_bytes() { return Q4_0_DEV_BYTES; }

int32_t launch_q4_0_matmul(rmi_ctx* ctx, const rmi_weight* w, const uint8_t* xq, const float* xs, size_t m, float* out,
                           size_t row_begin, size_t row_end) {
  if (m == 0 || row_begin >= row_end) return RMI_OK;
  dim3 grid((unsigned)((row_end - row_begin + 3) / 4), (unsigned)m);
  q4_0_matmul_kernel<<<grid, 128, 0, ctx->stream>>>(w->d_raw, w->n_in / 32, w->n_rows, xq, xs, out, row_begin, row_end);
  return rmi_post_launch(ctx, "q4_0_matmul");
}
