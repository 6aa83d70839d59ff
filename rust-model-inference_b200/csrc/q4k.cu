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
// The 16-byte header of a super-block as four words (d | dmin<<16, then the 12 scale bytes) and the 6-bit
// unpack of mod.rs:25-33 on those words.
__device__ __forceinline__ void scale_min_w(uint32_t w1, uint32_t w2, uint32_t w3, int j, int* sc, int* mn) {
  // bytes 0..3 = w1, 4..7 = w2, 8..11 = w3.  j < 4: sc = q[j] & 63, mn = q[j+4] & 63;
  // j >= 4: sc = (q[j+4] & 15) | ((q[j-4] >> 6) << 4), mn = (q[j+4] >> 4) | ((q[j] >> 6) << 4)
  const int sh = 8 * (j & 3);
  const uint32_t a = w1 >> sh, b = w2 >> sh, c = w3 >> sh;
  const int sc_lo = (int)(a & 63u), mn_lo = (int)(b & 63u);
  const int sc_hi = (int)((c & 0xFu) | ((a >> 2) & 0x30u)), mn_hi = (int)(((c >> 4) & 0xFu) | ((b >> 2) & 0x30u));
  *sc = j < 4 ? sc_lo : sc_hi;
  *mn = j < 4 ? mn_lo : mn_hi;
}

// Super-blocks of a row are fetched Q4K_U at a time: lane h loads the 16-byte header of super-block i0+h (one
// load instead of a dozen dependent byte loads) and every lane its 4 quant bytes of each of the Q4K_U blocks,
// all issued before the first use; the header fields reach the lanes by shuffle (Q4K_U = q4k_batch<MP>::U).
#ifndef RMI_Q4K_ROWS8
#define RMI_Q4K_ROWS8 2
#endif

template <int MP>
struct q4k_batch {
  static constexpr int U = MP >= 4 ? 8 : 16;  // fewer blocks in flight when the accumulators need the registers
};

// Q4_K x Q8_K (vec_dot_q4k_q8k): one warp per weight row, MP activation rows per pass.  Lane = 4 quant bytes
// (j = lane/8 selects the 64-value group, L = lane%8 the AVX2 f32 lane).
template <int SEM, int MP>
__global__ void q4k_q8k_matmul_kernel(const uint8_t* __restrict__ w, size_t nb, size_t n_rows,
                                      const float* __restrict__ d8, const int8_t* __restrict__ q8,
                                      const int16_t* __restrict__ bs, float* __restrict__ out, size_t row_begin,
                                      size_t row_end) {
  constexpr int Q4K_U = q4k_batch<MP>::U;
  const size_t warp = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) / 32;
  const int lane = threadIdx.x & 31;
  const size_t row = row_begin + warp;
  const size_t t0 = (size_t)blockIdx.y * MP;
  if (row >= row_end) return;
  const int j = lane / 8, L = lane % 8;
  const uint8_t* wrow = w + row * nb * 144;
  float acc[MP], acc_m[MP], accs[MP][4], sumf[MP];
#pragma unroll
  for (int m = 0; m < MP; m++) {
    acc[m] = acc_m[m] = sumf[m] = 0.0f;
#pragma unroll
    for (int k = 0; k < 4; k++) accs[m][k] = 0.0f;
  }
  for (size_t i0 = 0; i0 < nb; i0 += Q4K_U) {
    uint4 hdr = make_uint4(0u, 0u, 0u, 0u);
    if (lane < Q4K_U && i0 + lane < nb) hdr = __ldg(reinterpret_cast<const uint4*>(wrow + (i0 + lane) * 144));
    uint32_t wqs[Q4K_U];
#pragma unroll
    for (int u = 0; u < Q4K_U; u++)
      wqs[u] = i0 + u < nb ? __ldg(reinterpret_cast<const uint32_t*>(wrow + (i0 + u) * 144 + 16 + 4 * lane)) : 0u;
#pragma unroll
    for (int u = 0; u < Q4K_U; u++) {
      if (i0 + u >= nb) break;  // warp-uniform
      const size_t i = i0 + u;
      const uint32_t h0 = __shfl_sync(0xffffffffu, hdr.x, u), h1 = __shfl_sync(0xffffffffu, hdr.y, u);
      const uint32_t h2 = __shfl_sync(0xffffffffu, hdr.z, u), h3 = __shfl_sync(0xffffffffu, hdr.w, u);
      const float dw = f16_bits_to_f32((uint16_t)(h0 & 0xffffu));
      const float dminw = f16_bits_to_f32((uint16_t)(h0 >> 16));
      int sc0, mn0, sc1, mn1;
      scale_min_w(h1, h2, h3, 2 * j, &sc0, &mn0);
      scale_min_w(h1, h2, h3, 2 * j + 1, &sc1, &mn1);
      const uint32_t wq = wqs[u];
      const int tt = lane & 3;
      int ma = 0, mb = 0, dummy;
      if (SEM != RMI_SEM_SCALAR) {
        scale_min_w(h1, h2, h3, 2 * tt, &dummy, &ma);
        scale_min_w(h1, h2, h3, 2 * tt + 1, &dummy, &mb);
      }
#pragma unroll
      for (int m = 0; m < MP; m++) {
        const size_t t = t0 + m;
        const float dq = d8[t * nb + i];
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
          acc[m] = __fmaf_rn(dd, (float)v, acc[m]);
          // mod.rs:749-756: hadd_epi16 (wrapping i16) then madd_epi16 with the mins
          const int2 b4 = *reinterpret_cast<const int2*>(bsb + 4 * tt);  // four i16 sums
          const int s0 = (int)(int16_t)((int16_t)(b4.x & 0xffff) + (int16_t)(b4.x >> 16));
          const int s1 = (int)(int16_t)((int16_t)(b4.y & 0xffff) + (int16_t)(b4.y >> 16));
          const float dmin = __fmul_rn(-dminw, dq);
          acc_m[m] = __fmaf_rn(dmin, (float)(ma * s0 + mb * s1), acc_m[m]);
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
          for (int k = 0; k < 4; k++) accs[m][k] = __fadd_rn(accs[m][k], __fmul_rn(dd, (float)v[k]));
          int sumi = 0;
#pragma unroll
          for (int jj = 0; jj < 16; jj++) {
            int mm;
            scale_min_w(h1, h2, h3, jj / 2, &dummy, &mm);
            sumi += (int)bsb[jj] * mm;
          }
          sumf[m] = __fsub_rn(sumf[m], __fmul_rn(__fmul_rn(dminw, dq), (float)sumi));
        }
      }
    }
  }
#pragma unroll
  for (int m = 0; m < MP; m++) {
    float r;
    if (SEM != RMI_SEM_SCALAR) {
      // hsum_ps over lanes L = 0..7 (dot.rs:447-456), mins: (m0+m2)+(m1+m3) (mod.rs:792-794)
      const float s = __fadd_rn(__shfl_xor_sync(0xffffffffu, acc[m], 4), acc[m]);
      const float u = __fadd_rn(s, __shfl_xor_sync(0xffffffffu, s, 1));
      const float main_val = __fadd_rn(u, __shfl_xor_sync(0xffffffffu, u, 2));
      const float m02 = __fadd_rn(acc_m[m], __shfl_xor_sync(0xffffffffu, acc_m[m], 2));
      const float min_val = __fadd_rn(m02, __shfl_xor_sync(0xffffffffu, m02, 1));
      r = __fadd_rn(main_val, min_val);
    } else {
      // sumf += sums[0..7] in order: lane 0 holds sums[0..3] (elements e%8 = k), lane 1 sums[4..7]
      float hi[4];
#pragma unroll
      for (int k = 0; k < 4; k++) hi[k] = __shfl_sync(0xffffffffu, accs[m][k], 1);
      r = sumf[m];
#pragma unroll
      for (int k = 0; k < 4; k++) r = __fadd_rn(r, accs[m][k]);
#pragma unroll
      for (int k = 0; k < 4; k++) r = __fadd_rn(r, hi[k]);
    }
    if (lane == 0) out[(t0 + m) * n_rows + row] = r;
  }
}

// forward_dequant: w = (d*sc)*q - (dmin*m) in f32 (mod.rs:471-486), dotted with the f32 input.
// One warp per R consecutive weight rows, MP activation rows per pass: the activation values fetched for a
// super-block are used for all R rows (at MP = 8 the activation reads through L1, not the weights, set the pace).
template <int MP, int R>
__global__ void q4k_dequant_matmul_kernel(const uint8_t* __restrict__ w, size_t nb, size_t n_rows,
                                          const float* __restrict__ x, float* __restrict__ out) {
  constexpr int Q4K_U = R > 1 ? 4 : q4k_batch<MP>::U;
  const size_t row0 = (((size_t)blockIdx.x * blockDim.x + threadIdx.x) / 32) * R;
  const int lane = threadIdx.x & 31;
  if (row0 >= n_rows) return;
  const int j = lane / 8, L = lane % 8;
  const size_t K = nb * 256;
  float acc[R][MP];
#pragma unroll
  for (int r = 0; r < R; r++)
#pragma unroll
    for (int m = 0; m < MP; m++) acc[r][m] = 0.0f;
  for (size_t i0 = 0; i0 < nb; i0 += Q4K_U) {
    uint4 hdr[R];
    uint32_t wqs[R][Q4K_U];
#pragma unroll
    for (int r = 0; r < R; r++) {
      const bool row_ok = row0 + r < n_rows;
      const uint8_t* wrow = w + (row0 + r) * nb * 144;
      hdr[r] = make_uint4(0u, 0u, 0u, 0u);
      if (row_ok && lane < Q4K_U && i0 + lane < nb) hdr[r] = __ldg(reinterpret_cast<const uint4*>(wrow + (i0 + lane) * 144));
#pragma unroll
      for (int u = 0; u < Q4K_U; u++)
        wqs[r][u] = row_ok && i0 + u < nb ? __ldg(reinterpret_cast<const uint32_t*>(wrow + (i0 + u) * 144 + 16 + 4 * lane)) : 0u;
    }
#pragma unroll
    for (int u = 0; u < Q4K_U; u++) {
      if (i0 + u >= nb) break;  // warp-uniform
      const size_t i = i0 + u;
      float wl[R][4], wh[R][4];
#pragma unroll
      for (int r = 0; r < R; r++) {
        const uint32_t h0 = __shfl_sync(0xffffffffu, hdr[r].x, u), h1 = __shfl_sync(0xffffffffu, hdr[r].y, u);
        const uint32_t h2 = __shfl_sync(0xffffffffu, hdr[r].z, u), h3 = __shfl_sync(0xffffffffu, hdr[r].w, u);
        const float dw = f16_bits_to_f32((uint16_t)(h0 & 0xffffu));
        const float dminw = f16_bits_to_f32((uint16_t)(h0 >> 16));
        int sc0, mn0, sc1, mn1;
        scale_min_w(h1, h2, h3, 2 * j, &sc0, &mn0);
        scale_min_w(h1, h2, h3, 2 * j + 1, &sc1, &mn1);
        const float d1 = __fmul_rn(dw, (float)sc0), m1 = __fmul_rn(dminw, (float)mn0);
        const float d2 = __fmul_rn(dw, (float)sc1), m2 = __fmul_rn(dminw, (float)mn1);
        const uint32_t wq = wqs[r][u];
#pragma unroll
        for (int k = 0; k < 4; k++) {
          wl[r][k] = __fsub_rn(__fmul_rn(d1, (float)((wq >> (8 * k)) & 0xF)), m1);
          wh[r][k] = __fsub_rn(__fmul_rn(d2, (float)((wq >> (8 * k + 4)) & 0xF)), m2);
        }
      }
#pragma unroll
      for (int m = 0; m < MP; m++) {
        const float* xp = x + m * K + i * 256 + 64 * j + 4 * L;
        const float4 a = __ldg(reinterpret_cast<const float4*>(xp));
        const float4 b = __ldg(reinterpret_cast<const float4*>(xp + 32));
#pragma unroll
        for (int r = 0; r < R; r++) {
          float sacc = acc[r][m];
          sacc = __fmaf_rn(wl[r][0], a.x, sacc); sacc = __fmaf_rn(wl[r][1], a.y, sacc);
          sacc = __fmaf_rn(wl[r][2], a.z, sacc); sacc = __fmaf_rn(wl[r][3], a.w, sacc);
          sacc = __fmaf_rn(wh[r][0], b.x, sacc); sacc = __fmaf_rn(wh[r][1], b.y, sacc);
          sacc = __fmaf_rn(wh[r][2], b.z, sacc); sacc = __fmaf_rn(wh[r][3], b.w, sacc);
          acc[r][m] = sacc;
        }
      }
    }
  }
#pragma unroll
  for (int r = 0; r < R; r++)
#pragma unroll
    for (int m = 0; m < MP; m++) {
      float sacc = acc[r][m];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) sacc += __shfl_xor_sync(0xffffffffu, sacc, o);
      if (lane == 0 && row0 + r < n_rows) out[m * n_rows + row0 + r] = sacc;
    }
}

// forward_dequant for many activation rows (compute-bound in f32): a register-tiled f32 GEMM whose weight tile
// is decoded from the Q4_K bytes on the way into shared memory (same w = (d*sc)*q - dmin*m arithmetic as above,
// mod.rs:471-486).  CTA tile 128 weight rows x 64 activation rows, K chunks of 32 values (one half of a 64-value
// group: the low or the high nibbles of 32 quant bytes, one 6-bit scale/min pair), 256 threads with 8 x 4
// accumulators each, two shared-memory stages.
constexpr int Q4G_BN = 128, Q4G_BM = 64, Q4G_BK = 32, Q4G_PAD = 4;

__global__ void __launch_bounds__(256)
    q4k_dequant_gemm_kernel(const uint8_t* __restrict__ w, size_t nb, size_t n_rows, const float* __restrict__ x,
                            size_t m_rows, float* __restrict__ out) {
  extern __shared__ __align__(16) uint8_t q4g_smem[];
  float (*Ws)[Q4G_BK][Q4G_BN + Q4G_PAD] = reinterpret_cast<float (*)[Q4G_BK][Q4G_BN + Q4G_PAD]>(q4g_smem);
  float (*Xs)[Q4G_BK][Q4G_BM + Q4G_PAD] =
      reinterpret_cast<float (*)[Q4G_BK][Q4G_BM + Q4G_PAD]>(q4g_smem + 2 * Q4G_BK * (Q4G_BN + Q4G_PAD) * 4);
  const int tid = threadIdx.x;
  const size_t n0 = (size_t)blockIdx.x * Q4G_BN, m0 = (size_t)blockIdx.y * Q4G_BM;
  const size_t K = nb * 256;
  const int n_chunks = (int)(nb * 8);
  // loader roles: weights - thread (row tid/2, 16 of the chunk's 32 values); activations - thread (row tid/4, 8 values)
  const int wr = tid >> 1, wh = tid & 1;
  const int xr = tid >> 2, xq = tid & 3;
  const bool w_ok = n0 + wr < n_rows, x_ok = m0 + xr < m_rows;
  const uint8_t* wrow = w + (n0 + wr) * nb * 144;
  const float* xrow = x + (m0 + xr) * K;
  // compute roles: tx = 8 consecutive weight rows, ty = 4 consecutive activation rows
  const int tx = tid & 15, ty = tid >> 4;
  float acc[4][8];
#pragma unroll
  for (int a = 0; a < 4; a++)
#pragma unroll
    for (int b = 0; b < 8; b++) acc[a][b] = 0.0f;

  uint4 qv = make_uint4(0u, 0u, 0u, 0u), hv = make_uint4(0u, 0u, 0u, 0u);
  float4 xa = make_float4(0.f, 0.f, 0.f, 0.f), xb = xa;
  auto fetch = [&](int c) {
    const int sb = c >> 3, cc = c & 7, grp = cc >> 1;
    if (w_ok) {
      const uint8_t* blk = wrow + (size_t)sb * 144;
      hv = __ldg(reinterpret_cast<const uint4*>(blk));
      qv = __ldg(reinterpret_cast<const uint4*>(blk + 16 + 32 * grp + 16 * wh));
    }
    if (x_ok) {
      const float* xp = xrow + (size_t)c * Q4G_BK + xq * 8;
      xa = __ldg(reinterpret_cast<const float4*>(xp));
      xb = __ldg(reinterpret_cast<const float4*>(xp + 4));
    }
  };
  auto stash = [&](int c, int st) {
    const int cc = c & 7, hi = cc & 1;
    int sc, mn;
    scale_min_w(hv.y, hv.z, hv.w, cc, &sc, &mn);
    const float d1 = __fmul_rn(f16_bits_to_f32((uint16_t)(hv.x & 0xffffu)), (float)sc);
    const float m1 = __fmul_rn(f16_bits_to_f32((uint16_t)(hv.x >> 16)), (float)mn);
    const uint32_t q[4] = {qv.x, qv.y, qv.z, qv.w};
#pragma unroll
    for (int v = 0; v < 16; v++) {
      const uint32_t byte = (q[v >> 2] >> (8 * (v & 3))) & 0xffu;
      const float qf = (float)(hi ? (byte >> 4) : (byte & 0xFu));
      Ws[st][wh * 16 + v][wr] = w_ok ? __fsub_rn(__fmul_rn(d1, qf), m1) : 0.0f;
    }
    const float xv[8] = {xa.x, xa.y, xa.z, xa.w, xb.x, xb.y, xb.z, xb.w};
#pragma unroll
    for (int v = 0; v < 8; v++) Xs[st][xq * 8 + v][xr] = x_ok ? xv[v] : 0.0f;
  };

  fetch(0);
  stash(0, 0);
  __syncthreads();
  for (int c = 0; c < n_chunks; c++) {
    const int st = c & 1;
    if (c + 1 < n_chunks) fetch(c + 1);
#pragma unroll
    for (int k = 0; k < Q4G_BK; k++) {
      const float4 a0 = *reinterpret_cast<const float4*>(&Ws[st][k][tx * 8]);
      const float4 a1 = *reinterpret_cast<const float4*>(&Ws[st][k][tx * 8 + 4]);
      const float4 b0 = *reinterpret_cast<const float4*>(&Xs[st][k][ty * 4]);
      const float av[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
      const float bv[4] = {b0.x, b0.y, b0.z, b0.w};
#pragma unroll
      for (int a = 0; a < 4; a++)
#pragma unroll
        for (int b = 0; b < 8; b++) acc[a][b] = __fmaf_rn(av[b], bv[a], acc[a][b]);
    }
    if (c + 1 < n_chunks) stash(c + 1, st ^ 1);
    __syncthreads();
  }
#pragma unroll
  for (int a = 0; a < 4; a++) {
    const size_t mrow = m0 + ty * 4 + a;
    if (mrow >= m_rows) continue;
    float* o = out + mrow * n_rows + n0 + tx * 8;
    if (n0 + tx * 8 + 8 <= n_rows && (n_rows & 3) == 0) {
      *reinterpret_cast<float4*>(o) = make_float4(acc[a][0], acc[a][1], acc[a][2], acc[a][3]);
      *reinterpret_cast<float4*>(o + 4) = make_float4(acc[a][4], acc[a][5], acc[a][6], acc[a][7]);
    } else {
#pragma unroll
      for (int b = 0; b < 8; b++)
        if (n0 + tx * 8 + b < n_rows) o[b] = acc[a][b];
    }
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

template <int MP>
static void q4k_q8k_launch(rmi_ctx* ctx, const rmi_weight* w, const float* d8, const int8_t* qs, const int16_t* bsums,
                           size_t groups, float* out, size_t row_begin, size_t row_end) {
  const size_t rows = row_end - row_begin, nb = w->n_in / 256;
  dim3 grid((unsigned)((rows + 3) / 4), (unsigned)groups);
  if (ctx->sem == RMI_SEM_SCALAR)
    q4k_q8k_matmul_kernel<RMI_SEM_SCALAR, MP><<<grid, 128, 0, ctx->stream>>>(w->d_raw, nb, w->n_rows, d8, qs, bsums, out, row_begin, row_end);
  else
    q4k_q8k_matmul_kernel<RMI_SEM_AVX2, MP><<<grid, 128, 0, ctx->stream>>>(w->d_raw, nb, w->n_rows, d8, qs, bsums, out, row_begin, row_end);
}

int32_t launch_q4k_q8k_matmul(rmi_ctx* ctx, const rmi_weight* w, const float* d8, const int8_t* qs,
                              const int16_t* bsums, size_t m, float* out, size_t row_begin, size_t row_end) {
  if (m == 0 || row_begin >= row_end) return RMI_OK;
  const size_t nb = w->n_in / 256;
  // groups of 4 activation rows share one pass over the weights (all groups in one launch), then the remainder
  size_t t = 0;
  if (m >= 4) {
    q4k_q8k_launch<4>(ctx, w, d8, qs, bsums, m / 4, out, row_begin, row_end);
    RMI_TRY(rmi_post_launch(ctx, "q4k_q8k_matmul"));
    t = m / 4 * 4;
  }
  if (t < m) {
    q4k_q8k_launch<1>(ctx, w, d8 + t * nb, qs + t * nb * 256, bsums + t * nb * 16, m - t, out + t * w->n_rows, row_begin, row_end);
    RMI_TRY(rmi_post_launch(ctx, "q4k_q8k_matmul"));
  }
  return RMI_OK;
}

int32_t launch_q4k_dequant_matmul(rmi_ctx* ctx, const rmi_weight* w, const float* x, size_t m, float* out) {
  if (m == 0 || w->n_rows == 0) return RMI_OK;
  const size_t nb = w->n_in / 256;
  if (m >= 32) {  // compute-bound: tiled f32 GEMM with on-the-fly decode
    dim3 g2((unsigned)((w->n_rows + Q4G_BN - 1) / Q4G_BN), (unsigned)((m + Q4G_BM - 1) / Q4G_BM));
    constexpr size_t smem = 2 * Q4G_BK * (Q4G_BN + Q4G_PAD + Q4G_BM + Q4G_PAD) * 4;
    if (cudaFuncSetAttribute(q4k_dequant_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) {
      rmi_set_error("cudaFuncSetAttribute(%zu B shared) failed", smem);
      return RMI_ERR_CUDA;
    }
    q4k_dequant_gemm_kernel<<<g2, 256, smem, ctx->stream>>>(w->d_raw, nb, w->n_rows, x, m, out);
    return rmi_post_launch(ctx, "q4k_dequant_gemm");
  }
  size_t t = 0;
  while (t < m) {
    const size_t left = m - t;
    const float* xp = x + t * w->n_in;
    float* op = out + t * w->n_rows;
    if (left >= 8) {
      constexpr int R = RMI_Q4K_ROWS8;
      q4k_dequant_matmul_kernel<8, R><<<(unsigned)((w->n_rows + 4 * R - 1) / (4 * R)), 128, 0, ctx->stream>>>(w->d_raw, nb, w->n_rows, xp, op);
      t += 8;
    } else if (left >= 4) {
      q4k_dequant_matmul_kernel<4, 2><<<(unsigned)((w->n_rows + 7) / 8), 128, 0, ctx->stream>>>(w->d_raw, nb, w->n_rows, xp, op);
      t += 4;
    } else if (left >= 2) {
      q4k_dequant_matmul_kernel<2, 1><<<(unsigned)((w->n_rows + 3) / 4), 128, 0, ctx->stream>>>(w->d_raw, nb, w->n_rows, xp, op);
      t += 2;
    } else {
      q4k_dequant_matmul_kernel<1, 1><<<(unsigned)((w->n_rows + 3) / 4), 128, 0, ctx->stream>>>(w->d_raw, nb, w->n_rows, xp, op);
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
