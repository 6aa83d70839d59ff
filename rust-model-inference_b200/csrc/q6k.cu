// Q6_K paths: the Q6_K x Q8_K row dot (exact integer sums, the reference's AVX2 or scalar f32 order), the
// Q8_0-activation path (dequantized row x dequantized activation) and the row dequantizer.
//
// Reference (paths inside the reference project):
//   src/ops/quant/mod.rs:530-569 (dequantize_row_q6_k), :640-692 and :964-1064 (vec_dot_q6k_q8k scalar / AVX2),
//   src/ops/kernel/q6_k.rs:22-80 (Kernel impl), :83-115 (matmul_q6_k_scalar_range).
//
// Device layout: the 210-byte super-blocks (ql[128] | qh[64] | i8 scales[16] | f16 d), which are only 2-byte
// aligned in a GGUF file, are padded to 224 bytes at upload so that every word load is aligned.
#include "common.cuh"
#include "kernels.cuh"

namespace {

constexpr int Q6K_DEV_BYTES = 224;

// four 6-bit values (0..63) as bytes of one word: positions 4L..4L+3 of vector (j, k) of a super-block
__device__ __forceinline__ uint32_t q6k_word(const uint8_t* blk, int j, int k, int L) {
  const uint32_t qlw = *reinterpret_cast<const uint32_t*>(blk + 64 * j + 32 * (k & 1) + 4 * L);
  const uint32_t qhw = *reinterpret_cast<const uint32_t*>(blk + 128 + 32 * j + 4 * L);
  return ((qlw >> (4 * (k >> 1))) & 0x0F0F0F0Fu) | (((qhw >> (2 * k)) & 0x03030303u) << 4);
}

// vec_dot_q6k_q8k for one weight row per warp, MP activation rows per pass.  Lane = (vq, L): L = lane % 8 is
// the AVX2 int32 lane (bytes 4L..4L+3 of every 32-byte vector), vq = lane / 8 the vectors vq and vq + 4.
template <int SEM, int MP>
__global__ void q6k_q8k_matmul_kernel(const uint8_t* __restrict__ w, size_t nb, size_t n_rows,
                                      const float* __restrict__ d8, const int8_t* __restrict__ q8,
                                      const int16_t* __restrict__ bs, float* __restrict__ out, size_t row_begin,
                                      size_t row_end) {
  const size_t warp = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) / 32;
  const int lane = threadIdx.x & 31;
  const size_t row = row_begin + warp;
  const size_t t0 = (size_t)blockIdx.y * MP;
  if (row >= row_end) return;
  const int L = lane & 7, vq = lane >> 3;
  const uint8_t* wrow = w + row * nb * Q6K_DEV_BYTES;
  float acc[MP], accs[MP][4];
#pragma unroll
  for (int m = 0; m < MP; m++) {
    acc[m] = 0.0f;
#pragma unroll
    for (int k = 0; k < 4; k++) accs[m][k] = 0.0f;
  }
  for (size_t i = 0; i < nb; i++) {
    const uint8_t* blk = wrow + i * Q6K_DEV_BYTES;
    const uint32_t qa = q6k_word(blk, 0, vq, L), qb = q6k_word(blk, 1, vq, L);   // vectors vq and vq + 4
    const int8_t* sc = reinterpret_cast<const int8_t*>(blk + 192);
    const int sca = sc[2 * vq + (L >= 4)], scb = sc[8 + 2 * vq + (L >= 4)];
    const int sub_a = sc[2 * L], sub_b = sc[2 * L + 1];
    const float dw = f16_bits_to_f32(*reinterpret_cast<const uint16_t*>(blk + 208));
#pragma unroll
    for (int m = 0; m < MP; m++) {
      const size_t t = t0 + m;
      const int8_t* q8b = q8 + (t * nb + i) * 256;
      const int xa = *reinterpret_cast<const int*>(q8b + 32 * vq + 4 * L);
      const int xb = *reinterpret_cast<const int*>(q8b + 128 + 32 * vq + 4 * L);
      const float d = __fmul_rn(dw, d8[t * nb + i]);
      if (SEM != RMI_SEM_SCALAR) {
        // mod.rs:998-1062
        int v = sca * dp4a_s8((int)qa, xa, 0) + scb * dp4a_s8((int)qb, xb, 0);
        v += __shfl_xor_sync(0xffffffffu, v, 8);
        v += __shfl_xor_sync(0xffffffffu, v, 16);
        const int16_t* bsb = bs + (t * nb + i) * 16;
        const int sumi = v - 32 * ((int)bsb[2 * L] * sub_a + (int)bsb[2 * L + 1] * sub_b);
        acc[m] = __fmaf_rn(d, (float)sumi, acc[m]);
      } else {
        // mod.rs:675-687: aux32[e % 8] with e % 8 = 4 (L % 2) + byte
        int v[4];
#pragma unroll
        for (int k = 0; k < 4; k++) {
          const int a6 = (int)((qa >> (8 * k)) & 0xff) - 32, b6 = (int)((qb >> (8 * k)) & 0xff) - 32;
          const int a8 = (int)(int8_t)((xa >> (8 * k)) & 0xff), b8 = (int)(int8_t)((xb >> (8 * k)) & 0xff);
          v[k] = sca * a8 * a6 + scb * b8 * b6;
        }
#pragma unroll
        for (int k = 0; k < 4; k++) {
          v[k] += __shfl_xor_sync(0xffffffffu, v[k], 2);
          v[k] += __shfl_xor_sync(0xffffffffu, v[k], 4);
          v[k] += __shfl_xor_sync(0xffffffffu, v[k], 8);
          v[k] += __shfl_xor_sync(0xffffffffu, v[k], 16);
        }
#pragma unroll
        for (int k = 0; k < 4; k++) accs[m][k] = __fadd_rn(accs[m][k], __fmul_rn(d, (float)v[k]));
      }
    }
  }
#pragma unroll
  for (int m = 0; m < MP; m++) {
    float r;
    if (SEM != RMI_SEM_SCALAR) {
      // hsum_ps over the eight lanes (dot.rs:447-456)
      const float s = __fadd_rn(__shfl_xor_sync(0xffffffffu, acc[m], 4), acc[m]);
      const float u = __fadd_rn(s, __shfl_xor_sync(0xffffffffu, s, 1));
      r = __fadd_rn(u, __shfl_xor_sync(0xffffffffu, u, 2));
    } else {
      // sumf = sums[0] + ... + sums[7]: lane 0 holds sums[0..3], lane 1 sums[4..7]
      float hi[4];
#pragma unroll
      for (int k = 0; k < 4; k++) hi[k] = __shfl_sync(0xffffffffu, accs[m][k], 1);
      r = 0.0f;
#pragma unroll
      for (int k = 0; k < 4; k++) r = __fadd_rn(r, accs[m][k]);
#pragma unroll
      for (int k = 0; k < 4; k++) r = __fadd_rn(r, hi[k]);
    }
    if (lane == 0) out[(t0 + m) * n_rows + row] = r;
  }
}

// matmul_q6_k_scalar_range: dequantized row (d*sc)*q times the dequantized Q8_0 activation q8*scale, summed by a
// warp tree (the reference sums sequentially in f32; tolerance 1e-4).  One warp per weight row.
__global__ void q6k_prequant_matmul_kernel(const uint8_t* __restrict__ w, size_t nb, size_t n_rows,
                                           const uint8_t* __restrict__ xq, const float* __restrict__ xs,
                                           float* __restrict__ out, size_t row_begin, size_t row_end) {
  const size_t row = row_begin + ((size_t)blockIdx.x * blockDim.x + threadIdx.x) / 32;
  const int lane = threadIdx.x & 31;
  const size_t t = blockIdx.y;
  if (row >= row_end) return;
  const int L = lane & 7, vq = lane >> 3;
  const size_t K = nb * 256;
  const uint8_t* wrow = w + row * nb * Q6K_DEV_BYTES;
  float acc = 0.0f;
  for (size_t i = 0; i < nb; i++) {
    const uint8_t* blk = wrow + i * Q6K_DEV_BYTES;
    const int8_t* sc = reinterpret_cast<const int8_t*>(blk + 192);
    const float dw = f16_bits_to_f32(*reinterpret_cast<const uint16_t*>(blk + 208));
#pragma unroll
    for (int j = 0; j < 2; j++) {
      const uint32_t q = q6k_word(blk, j, vq, L);
      const int e0 = 128 * j + 32 * vq + 4 * L;
      const float ds = __fmul_rn(dw, (float)sc[e0 / 16]);
      const int xw = *reinterpret_cast<const int*>(xq + t * K + i * 256 + e0);
      const float xsc = xs[t * (K / 32) + (i * 256 + e0) / 32];
#pragma unroll
      for (int k = 0; k < 4; k++) {
        const float wv = __fmul_rn(ds, (float)((int)((q >> (8 * k)) & 0xff) - 32));
        const float xv = __fmul_rn((float)(int)(int8_t)((xw >> (8 * k)) & 0xff), xsc);
        acc = __fmaf_rn(wv, xv, acc);
      }
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if (lane == 0) out[t * n_rows + row] = acc;
}

__global__ void q6k_dequantize_kernel(const uint8_t* __restrict__ w, size_t n_superblocks, float* __restrict__ out) {
  const size_t sb = (size_t)blockIdx.x;
  if (sb >= n_superblocks) return;
  const uint8_t* blk = w + sb * Q6K_DEV_BYTES;
  const int e = threadIdx.x;  // 256 threads: one value each
  const int j = e / 128, r = e % 128, k = r / 32, l = r % 32;
  const uint8_t qlb = blk[64 * j + 32 * (k & 1) + l], qhb = blk[128 + 32 * j + l];
  const int q = (int)(((qlb >> (4 * (k >> 1))) & 0xF) | (((qhb >> (2 * k)) & 3) << 4)) - 32;
  const float d = f16_bits_to_f32(*reinterpret_cast<const uint16_t*>(blk + 208));
  const float sc = (float)(int)(int8_t)blk[192 + e / 16];
  out[sb * 256 + e] = __fmul_rn(__fmul_rn(d, sc), (float)q);
}

// embedding_lookup_q6_k (src/ops/embedding.rs:40-47): dequantize_row_q6_k of the requested rows;
// grid (super-blocks per row, rows), 256 threads = one value each
__global__ void q6k_embedding_kernel(const uint8_t* __restrict__ w, size_t nb, const uint32_t* __restrict__ ids,
                                     float* __restrict__ out) {
  const uint8_t* blk = w + ((size_t)ids[blockIdx.y] * nb + blockIdx.x) * Q6K_DEV_BYTES;
  const int e = threadIdx.x;
  const int j = e / 128, r = e % 128, k = r / 32, l = r % 32;
  const uint8_t qlb = blk[64 * j + 32 * (k & 1) + l], qhb = blk[128 + 32 * j + l];
  const int q = (int)(((qlb >> (4 * (k >> 1))) & 0xF) | (((qhb >> (2 * k)) & 3) << 4)) - 32;
  const float d = f16_bits_to_f32(*reinterpret_cast<const uint16_t*>(blk + 208));
  const float sc = (float)(int)(int8_t)blk[192 + e / 16];
  out[((size_t)blockIdx.y * nb + blockIdx.x) * 256 + e] = __fmul_rn(__fmul_rn(d, sc), (float)q);
}

template <int MP>
void q6k_q8k_launch(rmi_ctx* ctx, const rmi_weight* w, const float* d8, const int8_t* qs, const int16_t* bsums,
                    size_t groups, float* out, size_t row_begin, size_t row_end) {
  const size_t rows = row_end - row_begin, nb = w->n_in / 256;
  dim3 grid((unsigned)((rows + 3) / 4), (unsigned)groups);
  if (ctx->sem == RMI_SEM_SCALAR)
    q6k_q8k_matmul_kernel<RMI_SEM_SCALAR, MP><<<grid, 128, 0, ctx->stream>>>(w->d_raw, nb, w->n_rows, d8, qs, bsums, out, row_begin, row_end);
  else
    q6k_q8k_matmul_kernel<RMI_SEM_AVX2, MP><<<grid, 128, 0, ctx->stream>>>(w->d_raw, nb, w->n_rows, d8, qs, bsums, out, row_begin, row_end);
}

}  // namespace

size_t q6k_device_block_bytes() { return Q6K_DEV_BYTES; }

int32_t launch_q6k_embedding(rmi_ctx* ctx, const rmi_weight* w, const uint32_t* ids, size_t m, float* out) {
  if (m == 0) return RMI_OK;
  q6k_embedding_kernel<<<dim3((unsigned)(w->n_in / 256), (unsigned)m), 256, 0, ctx->stream>>>(w->d_raw, w->n_in / 256, ids, out);
  return rmi_post_launch(ctx, "q6k_embedding");
}

int32_t launch_q6k_q8k_matmul(rmi_ctx* ctx, const rmi_weight* w, const float* d8, const int8_t* qs,
                              const int16_t* bsums, size_t m, float* out, size_t row_begin, size_t row_end) {
  if (m == 0 || row_begin >= row_end) return RMI_OK;
  const size_t nb = w->n_in / 256;
  size_t t = 0;
  if (m >= 4) {
    q6k_q8k_launch<4>(ctx, w, d8, qs, bsums, m / 4, out, row_begin, row_end);
    RMI_TRY(rmi_post_launch(ctx, "q6k_q8k_matmul"));
    t = m / 4 * 4;
  }
  if (t < m) {
    q6k_q8k_launch<1>(ctx, w, d8 + t * nb, qs + t * nb * 256, bsums + t * nb * 16, m - t, out + t * w->n_rows, row_begin, row_end);
    RMI_TRY(rmi_post_launch(ctx, "q6k_q8k_matmul"));
  }
  return RMI_OK;
}

int32_t launch_q6k_prequant_matmul(rmi_ctx* ctx, const rmi_weight* w, const uint8_t* xq, const float* xs, size_t m,
                                   float* out, size_t row_begin, size_t row_end) {
  if (m == 0 || row_begin >= row_end) return RMI_OK;
  dim3 grid((unsigned)((row_end - row_begin + 3) / 4), (unsigned)m);
  q6k_prequant_matmul_kernel<<<grid, 128, 0, ctx->stream>>>(w->d_raw, w->n_in / 256, w->n_rows, xq, xs, out, row_begin, row_end);
  return rmi_post_launch(ctx, "q6k_prequant_matmul");
}

int32_t launch_q6k_dequantize(rmi_ctx* ctx, const rmi_weight* w, float* out) {
  const size_t nsb = w->n_rows * (w->n_in / 256);
  if (nsb == 0) return RMI_OK;
  q6k_dequantize_kernel<<<(unsigned)nsb, 256, 0, ctx->stream>>>(w->d_raw, nsb, out);
  return rmi_post_launch(ctx, "q6k_dequantize");
}
