// Q4_K paths: Q8_K activation quantizer, the Q4_K x Q8_K row dot (exact integer sums and
// the reference's f32 accumulation order), dequantize-and-matmul, and the row dequantizer.
//
// Reference (paths inside the reference project):
//   src/ops/quant/mod.rs:25-33 (6-bit scale/min unpack), :82-200 (Q8_K quantizer),
//   :210-289 and :701-799 (vec_dot_q4k_q8k scalar / AVX2), :456-508 (dequantize),
//   src/ops/kernel/q4_k.rs:56-93, src/core/model.rs:65-85 (forward_dequant).
#include "common.cuh"
#include "kernels.cuh"

namespace {

// sc[j], mn[j] of sub-block j (0..7) from the 12 scale bytes (mod.rs:25-33)
__device__ __forceinline__ void scale_min_k4(const uint8_t* s, int j, int* sc, int* mn) {
  if (j < 4) {
    *sc = s[j] & 63;
    *mn = s[j + 4] & 63;
  } else {
    *sc = (s[j + 4] & 0xF) | ((s[j - 4] >> 6) << 4);
    *mn = (s[j + 4] >> 4) | ((s[j] >> 6) << 4);
  }
}

// One CTA of 256 threads per super-block of 256 values.
template <int SEM>
__global__ void q8k_quantize_kernel(const float* __restrict__ x, size_t n_blocks_total, float* __restrict__ d,
                                    int8_t* __restrict__ qs, int16_t* __restrict__ bsums) {
  __shared__ float s_ax[8];
  __shared__ int s_idx[8];
  __shared__ float s_maxval;
  const size_t blk = blockIdx.x;
  if (blk >= n_blocks_total) return;
  const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
  const float v = x[blk * 256 + t];
  // first element with the largest |x| (mod.rs:90-97: strict '>' keeps the earliest)
  float ax = fabsf(v);
  int idx = t;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    float oa = __shfl_xor_sync(0xffffffffu, ax, o);
    int oi = __shfl_xor_sync(0xffffffffu, idx, o);
    if (oa > ax || (oa == ax && oi < idx)) {
      ax = oa;
      idx = oi;
    }
  }
  if (lane == 0) {
    s_ax[warp] = ax;
    s_idx[warp] = idx;
  }
  __syncthreads();
  if (t == 0) {
    float best = s_ax[0];
    int bi = s_idx[0];
    for (int w = 1; w < 8; w++)
      if (s_ax[w] > best || (s_ax[w] == best && s_idx[w] < bi)) {
        best = s_ax[w];
        bi = s_idx[w];
      }
    s_maxval = best == 0.0f ? 0.0f : x[blk * 256 + bi];
  }
  __syncthreads();
  const float max_val = s_maxval;
  int q = 0;
  float dd = 0.0f;
  if (max_val != 0.0f) {
    const float iscale = __fdiv_rn(-127.0f, max_val);
    if (SEM == RMI_SEM_SCALAR) {
      q = min(127, (int)rintf(__fmul_rn(iscale, v)));  // nearest_int (mod.rs:75-80) is round-half-even
    } else {
      q = max(-127, min(127, (int)rintf(__fmul_rn(v, iscale))));
    }
    dd = __fdiv_rn(1.0f, iscale);
  }
  qs[blk * 256 + t] = (int8_t)q;
  int s = q;
#pragma unroll
  for (int o = 8; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  if ((t & 15) == 0) bsums[blk * 16 + t / 16] = (int16_t)s;
  if (t == 0) d[blk] = dd;
}

// One warp per (weight row, activation row).  Lane l owns bytes 4l..4l+3 of the 128 quant
// bytes: group j = l/8 (sub-blocks 2j and 2j+1) and AVX2 lane L = l%8.
template <int SEM>
__global__ void q4k_q8k_matmul_kernel(const uint8_t* __restrict__ w, size_t nb, size_t n_rows,
                                      const float* __restrict__ d8, const int8_t* __restrict__ q8,
                                      const int16_t* __restrict__ bs, float* __restrict__ out, size_t row_begin,
                                      size_t row_end) {
  const size_t warp = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) / 32;
  const int lane = threadIdx.x & 31;
  const size_t row = row_begin + warp;
  const size_t t = blockIdx.y;
  if (row >= row_end) return;
  const int j = lane / 8, L = lane % 8;
  const uint8_t* wrow = w + row * nb * 144;
  float acc = 0.0f;    // AVX2: lane L of the eight f32 lanes; SCALAR: sums[4*(L%2)+k] live in accs[]
  float acc_m = 0.0f;  // AVX2: lane (lane%4) of the four min lanes
  float accs[4] = {0.0f, 0.0f, 0.0f, 0.0f};
  float sumf = 0.0f;
  for (size_t i = 0; i < nb; i++) {
    const uint8_t* blk = wrow + i * 144;
    const float dq = d8[t * nb + i];
    const float dw = f16_bits_to_f32(*reinterpret_cast<const uint16_t*>(blk));
    const float dminw = f16_bits_to_f32(*reinterpret_cast<const uint16_t*>(blk + 2));
    int sc0, mn0, sc1, mn1;
    scale_min_k4(blk + 4, 2 * j, &sc0, &mn0);
    scale_min_k4(blk + 4, 2 * j + 1, &sc1, &mn1);
    const uint32_t wq = *reinterpret_cast<const uint32_t*>(blk + 16 + 4 * lane);
    const int8_t* q8b = q8 + (t * nb + i) * 256;
    const int xlo = *reinterpret_cast<const int*>(q8b + 64 * j + 4 * L);
    const int xhi = *reinterpret_cast<const int*>(q8b + 64 * j + 32 + 4 * L);
    const int16_t* bsb = bs + (t * nb + i) * 16;
    if (SEM != RMI_SEM_SCALAR) {
      // mod.rs:759-783
      int v = sc0 * dp4a_s8((int)(wq & 0x0F0F0F0Fu), xlo, 0) + sc1 * dp4a_s8((int)((wq >> 4) & 0x0F0F0F0Fu), xhi, 0);
      v += __shfl_xor_sync(0xffffffffu, v, 8);
      v += __shfl_xor_sync(0xffffffffu, v, 16);
      const float dd = __fmul_rn(dw, dq);
      acc = __fmaf_rn(dd, (float)v, acc);
      // mod.rs:749-756: hadd_epi16 (wrapping i16) then madd_epi16 with the mins
      const int tt = lane & 3;
      int ma, mb, dummy;
      scale_min_k4(blk + 4, 2 * tt, &dummy, &ma);
      scale_min_k4(blk + 4, 2 * tt + 1, &dummy, &mb);
      const int s0 = (int)(int16_t)(bsb[4 * tt] + bsb[4 * tt + 1]);
      const int s1 = (int)(int16_t)(bsb[4 * tt + 2] + bsb[4 * tt + 3]);
      const float dmin = __fmul_rn(-dminw, dq);
      acc_m = __fmaf_rn(dmin, (float)(ma * s0 + mb * s1), acc_m);
    } else {
      // mod.rs:266-286: aux32[e%8] over all 256 elements, then sums[l] += dd*aux32[l]
      int v[4];
#pragma unroll
      for (int k = 0; k < 4; k++) {
        const int wl = (wq >> (8 * k)) & 0xF, wh = (wq >> (8 * k + 4)) & 0xF;
        const int a = (int)(int8_t)((xlo >> (8 * k)) & 0xff), b = (int)(int8_t)((xhi >> (8 * k)) & 0xff);
        v[k] = sc0 * wl * a + sc1 * wh * b;
      }
#pragma unroll
      for (int k = 0; k < 4; k++) {
        v[k] += __shfl_xor_sync(0xffffffffu, v[k], 2);
        v[k] += __shfl_xor_sync(0xffffffffu, v[k], 4);
        v[k] += __shfl_xor_sync(0xffffffffu, v[k], 8);
        v[k] += __shfl_xor_sync(0xffffffffu, v[k], 16);
      }
      const float dd = __fmul_rn(dw, dq);
#pragma unroll
      for (int k = 0; k < 4; k++) accs[k] = __fadd_rn(accs[k], __fmul_rn(dd, (float)v[k]));
      int sumi = 0;
      for (int jj = 0; jj < 16; jj++) {
        int mm, dummy;
        scale_min_k4(blk + 4, jj / 2, &dummy, &mm);
        sumi += (int)bsb[jj] * mm;
      }
      sumf = __fsub_rn(sumf, __fmul_rn(__fmul_rn(dminw, dq), (float)sumi));
    }
  }
  float r;
  if (SEM != RMI_SEM_SCALAR) {
    // hsum_ps over lanes L = 0..7 (dot.rs:447-456), mins: (m0+m2)+(m1+m3) (mod.rs:792-794)
    const float s = __fadd_rn(__shfl_xor_sync(0xffffffffu, acc, 4), acc);
    const float u = __fadd_rn(s, __shfl_xor_sync(0xffffffffu, s, 1));
    const float main_val = __fadd_rn(u, __shfl_xor_sync(0xffffffffu, u, 2));
    const float m02 = __fadd_rn(acc_m, __shfl_xor_sync(0xffffffffu, acc_m, 2));
    const float min_val = __fadd_rn(m02, __shfl_xor_sync(0xffffffffu, m02, 1));
    r = __fadd_rn(main_val, min_val);
  } else {
    // sumf += sums[0..7] in order: lane 0 holds sums[0..3] (elements e%8 = k), lane 1 sums[4..7]
    float hi[4];
#pragma unroll
    for (int k = 0; k < 4; k++) hi[k] = __shfl_sync(0xffffffffu, accs[k], 1);
    r = sumf;
#pragma unroll
    for (int k = 0; k < 4; k++) r = __fadd_rn(r, accs[k]);
#pragma unroll
    for (int k = 0; k < 4; k++) r = __fadd_rn(r, hi[k]);
  }
  if (lane == 0) out[t * n_rows + row] = r;
}

// forward_dequant: w = (d*sc)*q - (dmin*m) in f32 (mod.rs:471-486), dotted with the f32 input.
// One warp per weight row, MP activation rows per pass.
template <int MP>
__global__ void q4k_dequant_matmul_kernel(const uint8_t* __restrict__ w, size_t nb, size_t n_rows,
                                          const float* __restrict__ x, float* __restrict__ out) {
  const size_t row = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) / 32;
  const int lane = threadIdx.x & 31;
  if (row >= n_rows) return;
  const int j = lane / 8, L = lane % 8;
  const size_t K = nb * 256;
  const uint8_t* wrow = w + row * nb * 144;
  float acc[MP];
#pragma unroll
  for (int m = 0; m < MP; m++) acc[m] = 0.0f;
  for (size_t i = 0; i < nb; i++) {
    const uint8_t* blk = wrow + i * 144;
    const float dw = f16_bits_to_f32(*reinterpret_cast<const uint16_t*>(blk));
    const float dminw = f16_bits_to_f32(*reinterpret_cast<const uint16_t*>(blk + 2));
    int sc0, mn0, sc1, mn1;
    scale_min_k4(blk + 4, 2 * j, &sc0, &mn0);
    scale_min_k4(blk + 4, 2 * j + 1, &sc1, &mn1);
    const float d1 = __fmul_rn(dw, (float)sc0), m1 = __fmul_rn(dminw, (float)mn0);
    const float d2 = __fmul_rn(dw, (float)sc1), m2 = __fmul_rn(dminw, (float)mn1);
    const uint32_t wq = __ldg(reinterpret_cast<const uint32_t*>(blk + 16 + 4 * lane));
    float wl[4], wh[4];
#pragma unroll
    for (int k = 0; k < 4; k++) {
      wl[k] = __fsub_rn(__fmul_rn(d1, (float)((wq >> (8 * k)) & 0xF)), m1);
      wh[k] = __fsub_rn(__fmul_rn(d2, (float)((wq >> (8 * k + 4)) & 0xF)), m2);
    }
#pragma unroll
    for (int m = 0; m < MP; m++) {
      const float* xp = x + m * K + i * 256 + 64 * j + 4 * L;
      const float4 a = __ldg(reinterpret_cast<const float4*>(xp));
      const float4 b = __ldg(reinterpret_cast<const float4*>(xp + 32));
      float s = acc[m];
      s = __fmaf_rn(wl[0], a.x, s); s = __fmaf_rn(wl[1], a.y, s); s = __fmaf_rn(wl[2], a.z, s); s = __fmaf_rn(wl[3], a.w, s);
      s = __fmaf_rn(wh[0], b.x, s); s = __fmaf_rn(wh[1], b.y, s); s = __fmaf_rn(wh[2], b.z, s); s = __fmaf_rn(wh[3], b.w, s);
      acc[m] = s;
    }
  }
#pragma unroll
  for (int m = 0; m < MP; m++) {
    float s = acc[m];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if (lane == 0) out[m * n_rows + row] = s;
  }
}

__global__ void q4k_dequantize_kernel(const uint8_t* __restrict__ w, size_t n_superblocks, float* __restrict__ out) {
  const size_t warp = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) / 32;
  const int lane = threadIdx.x & 31;
  if (warp >= n_superblocks) return;
  const int j = lane / 8, L = lane % 8;
  const uint8_t* blk = w + warp * 144;
  const float dw = f16_bits_to_f32(*reinterpret_cast<const uint16_t*>(blk));
  const float dminw = f16_bits_to_f32(*reinterpret_cast<const uint16_t*>(blk + 2));
  int sc0, mn0, sc1, mn1;
  scale_min_k4(blk + 4, 2 * j, &sc0, &mn0);
  scale_min_k4(blk + 4, 2 * j + 1, &sc1, &mn1);
  const float d1 = __fmul_rn(dw, (float)sc0), m1 = __fmul_rn(dminw, (float)mn0);
  const float d2 = __fmul_rn(dw, (float)sc1), m2 = __fmul_rn(dminw, (float)mn1);
  const uint32_t wq = *reinterpret_cast<const uint32_t*>(blk + 16 + 4 * lane);
  float* o = out + warp * 256 + 64 * j + 4 * L;
#pragma unroll
  for (int k = 0; k < 4; k++) {
    o[k] = __fsub_rn(__fmul_rn(d1, (float)((wq >> (8 * k)) & 0xF)), m1);
    o[32 + k] = __fsub_rn(__fmul_rn(d2, (float)((wq >> (8 * k + 4)) & 0xF)), m2);
  }
}

}  // namespace

int32_t launch_q8k_quantize(rmi_ctx* ctx, const float* x, size_t m, size_t n, float* d, int8_t* qs, int16_t* bsums) {
  size_t nb = m * (n / 256);
  if (nb == 0) return RMI_OK;
  if (ctx->sem == RMI_SEM_SCALAR)
    q8k_quantize_kernel<RMI_SEM_SCALAR><<<(unsigned)nb, 256, 0, ctx->stream>>>(x, nb, d, qs, bsums);
  else
    q8k_quantize_kernel<RMI_SEM_AVX2><<<(unsigned)nb, 256, 0, ctx->stream>>>(x, nb, d, qs, bsums);
  return rmi_post_launch(ctx, "q8k_quantize");
}

int32_t launch_q4k_q8k_matmul(rmi_ctx* ctx, const rmi_weight* w, const float* d8, const int8_t* qs,
                              const int16_t* bsums, size_t m, float* out, size_t row_begin, size_t row_end) {
  if (m == 0 || row_begin >= row_end) return RMI_OK;
  const size_t rows = row_end - row_begin, nb = w->n_in / 256;
  dim3 grid((unsigned)((rows + 7) / 8), (unsigned)m);
  if (ctx->sem == RMI_SEM_SCALAR)
    q4k_q8k_matmul_kernel<RMI_SEM_SCALAR><<<grid, 256, 0, ctx->stream>>>(w->d_raw, nb, w->n_rows, d8, qs, bsums, out, row_begin, row_end);
  else
    q4k_q8k_matmul_kernel<RMI_SEM_AVX2><<<grid, 256, 0, ctx->stream>>>(w->d_raw, nb, w->n_rows, d8, qs, bsums, out, row_begin, row_end);
  return rmi_post_launch(ctx, "q4k_q8k_matmul");
}

int32_t launch_q4k_dequant_matmul(rmi_ctx* ctx, const rmi_weight* w, const float* x, size_t m, float* out) {
  if (m == 0 || w->n_rows == 0) return RMI_OK;
  const size_t nb = w->n_in / 256;
  const unsigned grid = (unsigned)((w->n_rows + 7) / 8);
  size_t t = 0;
  while (t < m) {
    const size_t left = m - t;
    const float* xp = x + t * w->n_in;
    float* op = out + t * w->n_rows;
    if (left >= 8) {
      q4k_dequant_matmul_kernel<8><<<grid, 256, 0, ctx->stream>>>(w->d_raw, nb, w->n_rows, xp, op);
      t += 8;
    } else if (left >= 4) {
      q4k_dequant_matmul_kernel<4><<<grid, 256, 0, ctx->stream>>>(w->d_raw, nb, w->n_rows, xp, op);
      t += 4;
    } else if (left >= 2) {
      q4k_dequant_matmul_kernel<2><<<grid, 256, 0, ctx->stream>>>(w->d_raw, nb, w->n_rows, xp, op);
      t += 2;
    } else {
      q4k_dequant_matmul_kernel<1><<<grid, 256, 0, ctx->stream>>>(w->d_raw, nb, w->n_rows, xp, op);
      t += 1;
    }
    RMI_TRY(rmi_post_launch(ctx, "q4k_dequant_matmul"));
  }
  return RMI_OK;
}

int32_t launch_q4k_dequantize(rmi_ctx* ctx, const rmi_weight* w, float* out) {
  const size_t nsb = w->n_rows * (w->n_in / 256);
  if (nsb == 0) return RMI_OK;
  q4k_dequantize_kernel<<<(unsigned)((nsb + 7) / 8), 256, 0, ctx->stream>>>(w->d_raw, nsb, out);
  return rmi_post_launch(ctx, "q4k_dequantize");
}
