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
  pdl_wait();               // x may come from the preceding kernel of a dependent launch
  pdl_launch_dependents();  // the matmul that follows fetches its weights meanwhile
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

// Q4_K x Q8_K for many activation rows: a tiled kernel instead of one pass over the weights per group of rows.
// CTA tile: 32 weight rows x 16 activation rows, one super-block (256 values) per step, two shared-memory stages
// filled with cp.async.  Thread = (4 weight rows 4tn..4tn+3 x 4 activation rows tm, tm+4, tm+8, tm+12, AVX2 lane L): for every pair of its
// tile it forms lane L's integer sum  v_L = sum_j sc[2j] * dot4(lo nibbles) + sc[2j+1] * dot4(hi nibbles)  over
// the four 64-value groups (exact; mod.rs:759-783) and accumulates acc_L = fma(d_w * d_x, f32(v_L), acc_L) over
// the super-blocks in order, plus the mins term of lane L & 3 (mod.rs:749-756) -- the same per-lane chains as the
// row kernel above, so the f32 result is bit-identical; the eight lanes of a pair sit in eight neighbouring
// threads and are combined at the end exactly as hsum_ps does (dot.rs:447-456).
constexpr int Q4T_TN = 32, Q4T_TM = 16;
// activation rows padded to 288 B (16-byte aligned for cp.async; 72 words, so the four row groups of a warp, one row
// apart, fall into different banks)
constexpr int Q4T_XSTRIDE = 288;

struct q4t_stage {
  uint8_t wq[Q4T_TN][144];            // raw super-blocks of the weight rows
  int8_t xq[Q4T_TM][Q4T_XSTRIDE];     // quantized activations
  int16_t xb[Q4T_TM][16];             // bsums
  float xd[Q4T_TM];                   // d
};

__global__ void __launch_bounds__(256)
    q4k_q8k_tiled_kernel(const uint8_t* __restrict__ w, size_t nb, size_t n_rows, const float* __restrict__ d8,
                         const int8_t* __restrict__ q8, const int16_t* __restrict__ bs, size_t m_rows,
                         float* __restrict__ out, size_t row_begin, size_t row_end) {
  __shared__ __align__(16) q4t_stage stg[2];
  __shared__ int s_sc[2][Q4T_TN][8], s_mn[2][Q4T_TN][8];   // 6-bit scales and mins, decoded once per (row, super-block)
  __shared__ float s_wd[2][Q4T_TN][2];                     // d, dmin
  __shared__ int s_xs[2][Q4T_TM][8];                       // pairwise bsum sums (i16 wrap): [tt][0], [tt][1]
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int L = lane & 7, tm = lane >> 3, tn = warp;       // 4 activation-row tiles per warp share the weight tile
  const size_t n0 = row_begin + (size_t)blockIdx.x * Q4T_TN, m0 = (size_t)blockIdx.y * Q4T_TM;

  auto load_stage = [&](int st, size_t i) {
    // weights: 32 rows x 144 B = 288 16-byte pieces; activations: 16 rows x 256 B = 256 pieces; bsums 16 x 32 B
    for (int p = tid; p < Q4T_TN * 9; p += 256) {
      const int r = p / 9, c = p % 9;
      const size_t row = n0 + r < row_end ? n0 + r : row_end - 1;  // rows past the range repeat the last one (never stored)
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(&stg[st].wq[r][c * 16])),
                   "l"(w + (row * nb + i) * 144 + c * 16)
                   : "memory");
    }
    {
      const int r = tid / 16, c = tid % 16;
      const size_t t = m0 + r < m_rows ? m0 + r : m_rows - 1;
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(&stg[st].xq[r][c * 16])),
                   "l"(q8 + (t * nb + i) * 256 + c * 16)
                   : "memory");
    }
    if (tid < Q4T_TM * 2) {
      const int r = tid / 2, c = tid % 2;
      const size_t t = m0 + r < m_rows ? m0 + r : m_rows - 1;
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(&stg[st].xb[r][c * 8])),
                   "l"(bs + (t * nb + i) * 16 + c * 8)
                   : "memory");
    }
    if (tid < Q4T_TM) {
      const size_t t = m0 + tid < m_rows ? m0 + tid : m_rows - 1;
      stg[st].xd[tid] = d8[t * nb + i];
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  auto decode_stage = [&](int st) {
    if (tid < Q4T_TN * 8) {
      const int r = tid >> 3, jj = tid & 7;
      const uint32_t* h = reinterpret_cast<const uint32_t*>(stg[st].wq[r]);
      int sc, mn;
      scale_min_w(h[1], h[2], h[3], jj, &sc, &mn);
      s_sc[st][r][jj] = sc;
      s_mn[st][r][jj] = mn;
      if (jj == 0) {
        s_wd[st][r][0] = f16_bits_to_f32((uint16_t)(h[0] & 0xffffu));
        s_wd[st][r][1] = f16_bits_to_f32((uint16_t)(h[0] >> 16));
      }
    }
    if (tid < Q4T_TM * 8) {
      const int r = tid >> 3, k = tid & 7;   // k = 2 * tt + which
      const int16_t* b = stg[st].xb[r] + 2 * k;
      s_xs[st][r][k] = (int)(int16_t)(b[0] + b[1]);  // hadd_epi16 wraps to i16 (mod.rs:749-752)
    }
  };

  float acc[4][4], accm[4][4];
#pragma unroll
  for (int a = 0; a < 4; a++)
#pragma unroll
    for (int b = 0; b < 4; b++) acc[a][b] = accm[a][b] = 0.0f;

  load_stage(0, 0);
  for (size_t i = 0; i < nb; i++) {
    const int st = (int)(i & 1);
    if (i + 1 < nb) load_stage(st ^ 1, i + 1);
    if (i + 1 < nb) asm volatile("cp.async.wait_group 1;" ::: "memory");
    else asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncthreads();
    decode_stage(st);
    __syncthreads();
    const q4t_stage& S = stg[st];
    int v[4][4];
#pragma unroll
    for (int a = 0; a < 4; a++)
#pragma unroll
      for (int b = 0; b < 4; b++) v[a][b] = 0;
#pragma unroll
    for (int j = 0; j < 4; j++) {
      int xlo[4], xhi[4];
#pragma unroll
      for (int b = 0; b < 4; b++) {
        xlo[b] = *reinterpret_cast<const int*>(&S.xq[tm + 4 * b][64 * j + 4 * L]);
        xhi[b] = *reinterpret_cast<const int*>(&S.xq[tm + 4 * b][64 * j + 32 + 4 * L]);
      }
#pragma unroll
      for (int a = 0; a < 4; a++) {
        const int r = tn * 4 + a;
        const uint32_t wq = *reinterpret_cast<const uint32_t*>(&S.wq[r][16 + 32 * j + 4 * L]);
        const int sc0 = s_sc[st][r][2 * j], sc1 = s_sc[st][r][2 * j + 1];
        const int wlo = (int)(wq & 0x0F0F0F0Fu), whi = (int)((wq >> 4) & 0x0F0F0F0Fu);
#pragma unroll
        for (int b = 0; b < 4; b++) v[a][b] += sc0 * dp4a_s8(wlo, xlo[b], 0) + sc1 * dp4a_s8(whi, xhi[b], 0);
      }
    }
    const int tt = L & 3;
#pragma unroll
    for (int a = 0; a < 4; a++) {
      const int r = tn * 4 + a;
      const float dw = s_wd[st][r][0], dminw = s_wd[st][r][1];
      const int ma = s_mn[st][r][2 * tt], mb = s_mn[st][r][2 * tt + 1];
#pragma unroll
      for (int b = 0; b < 4; b++) {
        const int t = tm + 4 * b;
        const float dq = S.xd[t];
        acc[a][b] = __fmaf_rn(__fmul_rn(dw, dq), (float)v[a][b], acc[a][b]);
        accm[a][b] = __fmaf_rn(__fmul_rn(-dminw, dq), (float)(ma * s_xs[st][t][2 * tt] + mb * s_xs[st][t][2 * tt + 1]), accm[a][b]);
      }
    }
    __syncthreads();  // the stage is refilled by the loads issued in the next iteration
  }
#pragma unroll
  for (int a = 0; a < 4; a++)
#pragma unroll
    for (int b = 0; b < 4; b++) {
      // hsum_ps over lanes L = 0..7 (dot.rs:447-456), mins: (m0+m2)+(m1+m3) (mod.rs:792-794)
      const float s1 = __fadd_rn(__shfl_xor_sync(0xffffffffu, acc[a][b], 4), acc[a][b]);
      const float u = __fadd_rn(s1, __shfl_xor_sync(0xffffffffu, s1, 1));
      const float main_val = __fadd_rn(u, __shfl_xor_sync(0xffffffffu, u, 2));
      const float m02 = __fadd_rn(accm[a][b], __shfl_xor_sync(0xffffffffu, accm[a][b], 2));
      const float min_val = __fadd_rn(m02, __shfl_xor_sync(0xffffffffu, m02, 1));
      const size_t row = n0 + tn * 4 + a, t = m0 + tm + 4 * b;
      if (L == 0 && row < row_end && t < m_rows) out[t * n_rows + row] = __fadd_rn(main_val, min_val);
    }
}

// The sixteen 6-bit fields of a super-block header (mod.rs:25-33) unpacked four at a time on whole words:
// h1..h3 are the 12 scale bytes; the results hold sc[0..3], sc[4..7], mn[0..3], mn[4..7] as bytes.
struct q4k_fields {
  uint32_t sc_lo, sc_hi, mn_lo, mn_hi;
};
__device__ __forceinline__ q4k_fields unpack_fields(uint32_t h1, uint32_t h2, uint32_t h3) {
  q4k_fields f;
  f.sc_lo = h1 & 0x3F3F3F3Fu;
  f.mn_lo = h2 & 0x3F3F3F3Fu;
  f.sc_hi = (h3 & 0x0F0F0F0Fu) | ((h1 >> 2) & 0x30303030u);
  f.mn_hi = ((h3 >> 4) & 0x0F0F0F0Fu) | ((h2 >> 2) & 0x30303030u);
  return f;
}

// 2^23 + (byte k of word) as f32: 0x4B0000bb
__device__ __forceinline__ float byte_plus_2p23(uint32_t word, int k) {
  return __uint_as_float(__byte_perm(word, 0x4B000000u, 0x7440u + (uint32_t)k));
}

// Q4_K x Q8_K for 4 or 8 activation rows (decode batches): the weight rows stream through shared-memory rings filled
// with bulk copies, so the bytes in flight do not depend on registers or on how many warps are resident.  Each warp
// owns four consecutive weight rows and a private ring (a stage holds Q4S_SB consecutive super-blocks of each of its
// rows, one bulk copy per row), so warps never wait for one another after the prologue.  Lane = (quad q, AVX2 lane
// L): quad q owns weight row q of the warp's four, and its eight L-lanes own bytes 4L..4L+3 of each of the four
// 32-byte groups of a super-block, i.e. f32 lane L of vec_dot_q4k_q8k's accumulator (mod.rs:759-783): the per-lane
// integer sum needs no shuffle and the 6-bit fields are unpacked four at a time on whole words.  Every thread
// carries all MB activation rows; they are staged once per CTA, permuted so that a lane finds its eight words of a
// super-block in two 16-byte pieces, with the wrapped pairwise bsums (mod.rs:749-752) already formed.  Per-lane
// chains acc = fma(d_w*d_x, f32(v), acc) and the mins chain of lane L&3 run over the super-blocks in order and are
// combined as hsum_ps does, as in the kernels above.
constexpr int Q4S_WARPS = 4, Q4S_TN = 4 * Q4S_WARPS, Q4S_SB = 4, Q4S_S = 3;
constexpr int Q4S_ROW_BYTES = Q4S_SB * 144 + 32;       // 152 words: the four rows of a warp start 24 banks apart
constexpr int Q4S_STAGE_BYTES = 4 * Q4S_ROW_BYTES;     // one warp, one stage
constexpr int Q4S_RING_BYTES = Q4S_WARPS * Q4S_S * Q4S_STAGE_BYTES;

// Shared memory: rings | barriers (128 B) | per activation row: permuted quants (256 B per super-block), bsum pairs
// (int2 per super-block and lane L&3), d.
__host__ __device__ inline size_t q4s_smem_bytes(size_t mb, size_t nb) {
  return (size_t)Q4S_RING_BYTES + 128 + mb * nb * (256 + 32 + 4);
}

// Bounded wait on a shared-memory mbarrier phase; false when the limit ran out.
__device__ __forceinline__ bool mbar_wait_limited(uint32_t bar, uint32_t parity, uint64_t limit_ns) {
  uint64_t t0 = 0;
  for (uint32_t i = 0; i < (1u << 26); i++) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity), "r"(20000u)
        : "memory");
    if (ok) return true;
    if ((i & 15) == 15) {
      uint64_t now;
      asm volatile("mov.u64 %0, %globaltimer;" : "=l"(now));
      if (t0 == 0) t0 = now;
      else if (now - t0 > limit_ns) return false;
    }
  }
  return false;
}

template <int MB>
__global__ void __launch_bounds__(32 * Q4S_WARPS)
    q4k_q8k_stream_kernel(const uint8_t* __restrict__ w, size_t nb, size_t n_rows, const float* __restrict__ d8,
                          const int8_t* __restrict__ q8, const int16_t* __restrict__ bs, float* __restrict__ out,
                          size_t row_begin, size_t row_end, size_t n_tiles, rmi_dev_status* status) {
  extern __shared__ __align__(128) uint8_t q4s_smem[];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int L = lane & 7, q = lane >> 3, tt = L & 3;
  uint8_t* ring = q4s_smem + warp * (Q4S_S * Q4S_STAGE_BYTES);                   // this warp's stages
  uint64_t* bar = reinterpret_cast<uint64_t*>(q4s_smem + Q4S_RING_BYTES) + warp * Q4S_S;
  int* xq_s = reinterpret_cast<int*>(q4s_smem + Q4S_RING_BYTES + 128);           // [MB][nb][2][8][4] words
  int2* xb_s = reinterpret_cast<int2*>(xq_s + (size_t)MB * nb * 64);             // [MB][nb][4]
  float* xd_s = reinterpret_cast<float*>(xb_s + (size_t)MB * nb * 4);            // [MB][nb]
  const uint32_t bar_a = (uint32_t)__cvta_generic_to_shared(bar);
  const uint32_t ring_a = (uint32_t)__cvta_generic_to_shared(ring);
  const int n_chunks = (int)((nb + Q4S_SB - 1) / Q4S_SB);
  const size_t my_tiles = blockIdx.x < n_tiles ? (n_tiles - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
  const size_t n_items = my_tiles * (size_t)n_chunks;   // (tile, chunk) pairs of this warp, in order
  const size_t t0 = (size_t)blockIdx.y * MB;

  // item j -> stage j % Q4S_S of this warp's ring (lane r < 4 copies the warp's row r)
  auto issue = [&](size_t j) {
    const size_t tile = blockIdx.x + (j / n_chunks) * gridDim.x;
    const size_t i0 = (size_t)(j % n_chunks) * Q4S_SB;
    const uint32_t n = (uint32_t)(nb - i0 < (size_t)Q4S_SB ? nb - i0 : (size_t)Q4S_SB);
    const uint32_t st = (uint32_t)(j % Q4S_S), bytes = n * 144u;
    if (lane == 0)
      asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar_a + 8 * st), "r"(bytes * 4u) : "memory");
    __syncwarp();
    if (lane < 4) {
      size_t row = row_begin + tile * Q4S_TN + warp * 4 + lane;
      if (row >= row_end) row = row_end - 1;   // rows past the range repeat the last one (never stored)
      asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                       ring_a + st * (uint32_t)Q4S_STAGE_BYTES + (uint32_t)lane * Q4S_ROW_BYTES),
                   "l"(w + (row * nb + i0) * 144), "r"(bytes), "r"(bar_a + 8 * st)
                   : "memory");
    }
  };
  if (lane == 0) {
    for (int i = 0; i < Q4S_S; i++) asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(bar_a + 8 * i));
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncwarp();
  for (size_t j = 0; j < n_items && j < (size_t)Q4S_S; j++) issue(j);

  // the MB activation rows of this pass, once per CTA.  Word 16 jg + 8 h + l of a super-block (group jg, low / high
  // half h, lane l) goes to word 32 (jg / 2) + 4 l + 2 (jg % 2) + h: lane l then reads words 4l..4l+3 of two pieces.
  {
    // asynchronous 4-byte copies straight to the permuted place: all of a thread's copies are in flight at once (a
    // load-store loop through registers would pay one memory round trip per batch of loads)
    const int* src = reinterpret_cast<const int*>(q8 + t0 * nb * 256);
    for (size_t idx = tid; idx < (size_t)MB * nb * 64; idx += 32 * Q4S_WARPS) {
      const size_t rb = idx >> 6;   // (activation row, super-block)
      const int ws = (int)(idx & 63), jg = ws >> 4, h = (ws >> 3) & 1, l = ws & 7;
      asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((uint32_t)__cvta_generic_to_shared(
                       xq_s + rb * 64 + 32 * (jg >> 1) + 4 * l + 2 * (jg & 1) + h)),
                   "l"(src + idx)
                   : "memory");
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
    for (size_t idx = tid; idx < (size_t)MB * nb * 4; idx += 32 * Q4S_WARPS) {
      // mod.rs:749-756: hadd_epi16 (wrapping i16) of neighbouring bsums, the two pairs of lane idx % 4
      const int2 b4 = __ldg(reinterpret_cast<const int2*>(bs + t0 * nb * 16) + idx);
      xb_s[idx] = make_int2((int)(int16_t)((int16_t)(b4.x & 0xffff) + (int16_t)(b4.x >> 16)),
                            (int)(int16_t)((int16_t)(b4.y & 0xffff) + (int16_t)(b4.y >> 16)));
    }
    for (size_t idx = tid; idx < (size_t)MB * nb; idx += 32 * Q4S_WARPS) xd_s[idx] = __ldg(d8 + t0 * nb + idx);
    asm volatile("cp.async.wait_group 0;" ::: "memory");
  }
  __syncthreads();

  const uint64_t limit_ns = status->limit_ns;
  float acc[MB], accm[MB];
  for (size_t j = 0; j < n_items; j++) {
    const int c = (int)(j % n_chunks);
    const uint32_t st = (uint32_t)(j % Q4S_S), parity = (uint32_t)((j / Q4S_S) & 1);
    if (c == 0) {
#pragma unroll
      for (int b = 0; b < MB; b++) acc[b] = accm[b] = 0.0f;
    }
    if (!mbar_wait_limited(bar_a + 8 * st, parity, limit_ns)) {
      // the copies in flight target this CTA's own shared memory and are dropped with it
      if (atomicCAS(&status->code, 0, RMI_ERR_TIMEOUT) == 0) {
        status->where = 12;
        status->detail = (int)j;
      }
      return;
    }
    const size_t i0 = (size_t)c * Q4S_SB;
    const int n = (int)(nb - i0 < (size_t)Q4S_SB ? nb - i0 : (size_t)Q4S_SB);
    const uint8_t* row_s = ring + (size_t)st * Q4S_STAGE_BYTES + (size_t)q * Q4S_ROW_BYTES;
#pragma unroll
    for (int u = 0; u < Q4S_SB; u++) {
      if (u >= n) break;  // uniform
      const size_t i = i0 + u;
      const uint8_t* blk = row_s + u * 144;
      const uint4 h = *reinterpret_cast<const uint4*>(blk);
      const float dw = f16_bits_to_f32((uint16_t)(h.x & 0xffffu));
      const float ndminw = -f16_bits_to_f32((uint16_t)(h.x >> 16));
      // the sixteen 6-bit fields of mod.rs:25-33, four per word: sc[0..3], sc[4..7], mn[0..3], mn[4..7]
      const uint32_t sc_lo = h.y & 0x3F3F3F3Fu, mn_lo = h.z & 0x3F3F3F3Fu;
      const uint32_t sc_hi = (h.w & 0x0F0F0F0Fu) | ((h.y >> 2) & 0x30303030u);
      const uint32_t mn_hi = ((h.w >> 4) & 0x0F0F0F0Fu) | ((h.z >> 2) & 0x30303030u);
      int sc[8], wlo[4], whi[4];
#pragma unroll
      for (int k = 0; k < 4; k++) {
        sc[k] = (int)((sc_lo >> (8 * k)) & 0xffu);
        sc[4 + k] = (int)((sc_hi >> (8 * k)) & 0xffu);
      }
#pragma unroll
      for (int jg = 0; jg < 4; jg++) {
        const uint32_t wq = *reinterpret_cast<const uint32_t*>(blk + 16 + 32 * jg + 4 * L);
        wlo[jg] = (int)(wq & 0x0F0F0F0Fu);
        whi[jg] = (int)((wq >> 4) & 0x0F0F0F0Fu);
      }
      const uint32_t mw = tt < 2 ? mn_lo : mn_hi;
      const int ma = (int)((mw >> (16 * (tt & 1))) & 0xffu), mb = (int)((mw >> (16 * (tt & 1) + 8)) & 0xffu);
#pragma unroll
      for (int b = 0; b < MB; b++) {
        const size_t rb = (size_t)b * nb + i;
        const int4 x01 = *reinterpret_cast<const int4*>(xq_s + rb * 64 + 4 * L);        // lo0 hi0 lo1 hi1
        const int4 x23 = *reinterpret_cast<const int4*>(xq_s + rb * 64 + 32 + 4 * L);   // lo2 hi2 lo3 hi3
        const int2 ss = xb_s[rb * 4 + tt];
        const float dq = xd_s[rb];
        int v = sc[0] * dp4a_s8(wlo[0], x01.x, 0) + sc[1] * dp4a_s8(whi[0], x01.y, 0);
        v += sc[2] * dp4a_s8(wlo[1], x01.z, 0) + sc[3] * dp4a_s8(whi[1], x01.w, 0);
        v += sc[4] * dp4a_s8(wlo[2], x23.x, 0) + sc[5] * dp4a_s8(whi[2], x23.y, 0);
        v += sc[6] * dp4a_s8(wlo[3], x23.z, 0) + sc[7] * dp4a_s8(whi[3], x23.w, 0);
        acc[b] = __fmaf_rn(__fmul_rn(dw, dq), (float)v, acc[b]);
        accm[b] = __fmaf_rn(__fmul_rn(ndminw, dq), (float)(ma * ss.x + mb * ss.y), accm[b]);
      }
    }
    __syncwarp();  // every lane is done with the stage
    if (j + Q4S_S < n_items) issue(j + Q4S_S);
    if (c == n_chunks - 1) {
      const size_t tile = blockIdx.x + (j / n_chunks) * gridDim.x;
      const size_t row = row_begin + tile * Q4S_TN + warp * 4 + q;
#pragma unroll
      for (int b = 0; b < MB; b++) {
        // hsum_ps over lanes L = 0..7 (dot.rs:447-456), mins: (m0+m2)+(m1+m3) (mod.rs:792-794)
        const float s = __fadd_rn(__shfl_xor_sync(0xffffffffu, acc[b], 4), acc[b]);
        const float uu = __fadd_rn(s, __shfl_xor_sync(0xffffffffu, s, 1));
        const float main_val = __fadd_rn(uu, __shfl_xor_sync(0xffffffffu, uu, 2));
        const float m02 = __fadd_rn(accm[b], __shfl_xor_sync(0xffffffffu, accm[b], 2));
        const float min_val = __fadd_rn(m02, __shfl_xor_sync(0xffffffffu, m02, 1));
        if (L == 0 && row < row_end) out[(t0 + b) * n_rows + row] = __fadd_rn(main_val, min_val);
      }
    }
  }
}

// Q4_K x Q8_K for 1..8 activation rows with the super-blocks of a row split over the warps of a CTA, for the matrices
// of a decode step (a few thousand rows): a CTA owns four weight rows, warp w the chunks w, w + 4, ... of
// Q4S_SB super-blocks, so a 4096 x 4096 weight runs on 4096 warps instead of 1024.  Lane = (quad q = weight row,
// AVX2 lane L) as in the streaming kernel.  What can run in any order runs in parallel: for every (activation row,
// weight row, super-block, L) the exact integer sum v and the mins sum, converted to f32, and the two products
// d_w * d_x and -dmin_w * d_x go to shared memory.  What the reference orders runs in order: after a CTA barrier one
// lane per (activation row, weight row, L) folds its super-blocks in sequence, acc = fma(d_w*d_x, f32(v), acc) and
// the mins chain of lane L&3, and the eight lanes are combined as hsum_ps does -- the same operations on the same
// values as the kernels above.  The weight chunks are fetched by bulk copies issued before the wait on the
// preceding kernel of a dependent launch, so they overlap the quantizer that produces the activations.
constexpr int Q4P_S = 2;
constexpr int Q4P_RING_BYTES = Q4S_WARPS * Q4P_S * Q4S_STAGE_BYTES;
__host__ __device__ inline size_t q4p_smem_bytes(size_t mb, size_t nb) {
  return (size_t)Q4P_RING_BYTES + 128 + mb * 4 * nb * (8 * 8 + 8);
}

template <int MB>
__global__ void __launch_bounds__(32 * Q4S_WARPS)
    q4k_q8k_ksplit_kernel(const uint8_t* __restrict__ w, size_t nb, size_t n_rows, const float* __restrict__ d8,
                          const int8_t* __restrict__ q8, const int16_t* __restrict__ bs, float* __restrict__ out,
                          size_t row_begin, size_t row_end, rmi_dev_status* status) {
  extern __shared__ __align__(128) uint8_t q4p_smem[];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int L = lane & 7, q = lane >> 3, tt = L & 3;
  uint8_t* ring = q4p_smem + warp * (Q4P_S * Q4S_STAGE_BYTES);
  uint64_t* bar = reinterpret_cast<uint64_t*>(q4p_smem + Q4P_RING_BYTES) + warp * Q4P_S;
  float2* part_f = reinterpret_cast<float2*>(q4p_smem + Q4P_RING_BYTES + 128);   // [MB][4][nb][8]: f32(v), f32(mins sum)
  float2* part_p = part_f + (size_t)MB * 4 * nb * 8;                               // [MB][4][nb]: d_w*d_x, -dmin_w*d_x
  const uint32_t bar_a = (uint32_t)__cvta_generic_to_shared(bar);
  const uint32_t ring_a = (uint32_t)__cvta_generic_to_shared(ring);
  const int n_chunks = (int)((nb + Q4S_SB - 1) / Q4S_SB);
  const int n_my = warp < n_chunks ? (n_chunks - warp + Q4S_WARPS - 1) / Q4S_WARPS : 0;   // chunks warp, warp + 4, ...
  const size_t row0 = row_begin + (size_t)blockIdx.x * 4, t0 = (size_t)blockIdx.y * MB;

  auto issue = [&](int k) {
    const size_t i0 = (size_t)(warp + Q4S_WARPS * k) * Q4S_SB;
    const uint32_t n = (uint32_t)(nb - i0 < (size_t)Q4S_SB ? nb - i0 : (size_t)Q4S_SB);
    const uint32_t st = (uint32_t)(k % Q4P_S), bytes = n * 144u;
    if (lane == 0)
      asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar_a + 8 * st), "r"(bytes * 4u) : "memory");
    __syncwarp();
    if (lane < 4) {
      size_t row = row0 + lane;
      if (row >= row_end) row = row_end - 1;   // rows past the range repeat the last one (never stored)
      asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                       ring_a + st * (uint32_t)Q4S_STAGE_BYTES + (uint32_t)lane * Q4S_ROW_BYTES),
                   "l"(w + (row * nb + i0) * 144), "r"(bytes), "r"(bar_a + 8 * st)
                   : "memory");
    }
  };
  if (lane == 0) {
    for (int i = 0; i < Q4P_S; i++) asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(bar_a + 8 * i));
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncwarp();
  for (int k = 0; k < n_my && k < Q4P_S; k++) issue(k);   // weights: no kernel of a chain writes them
  pdl_wait();                                             // the activations come from the preceding kernel
  pdl_launch_dependents();

  const uint64_t limit_ns = status->limit_ns;
  for (int k = 0; k < n_my; k++) {
    const uint32_t st = (uint32_t)(k % Q4P_S), parity = (uint32_t)((k / Q4P_S) & 1);
    if (!mbar_wait_limited(bar_a + 8 * st, parity, limit_ns)) {
      // give up on this warp's chunks; the CTA still meets at the barrier below and the host reads the status
      if (atomicCAS(&status->code, 0, RMI_ERR_TIMEOUT) == 0) {
        status->where = 13;
        status->detail = k;
      }
      break;
    }
    const size_t i0 = (size_t)(warp + Q4S_WARPS * k) * Q4S_SB;
    const int n = (int)(nb - i0 < (size_t)Q4S_SB ? nb - i0 : (size_t)Q4S_SB);
    const uint8_t* row_s = ring + (size_t)st * Q4S_STAGE_BYTES + (size_t)q * Q4S_ROW_BYTES;
#pragma unroll
    for (int u = 0; u < Q4S_SB; u++) {
      if (u >= n) break;  // uniform
      const size_t i = i0 + u;
      const uint8_t* blk = row_s + u * 144;
      const uint4 h = *reinterpret_cast<const uint4*>(blk);
      const float dw = f16_bits_to_f32((uint16_t)(h.x & 0xffffu));
      const float ndminw = -f16_bits_to_f32((uint16_t)(h.x >> 16));
      const q4k_fields f = unpack_fields(h.y, h.z, h.w);
      int sc[8], wlo[4], whi[4];
#pragma unroll
      for (int kk = 0; kk < 4; kk++) {
        sc[kk] = (int)((f.sc_lo >> (8 * kk)) & 0xffu);
        sc[4 + kk] = (int)((f.sc_hi >> (8 * kk)) & 0xffu);
      }
#pragma unroll
      for (int jg = 0; jg < 4; jg++) {
        const uint32_t wq = *reinterpret_cast<const uint32_t*>(blk + 16 + 32 * jg + 4 * L);
        wlo[jg] = (int)(wq & 0x0F0F0F0Fu);
        whi[jg] = (int)((wq >> 4) & 0x0F0F0F0Fu);
      }
      const uint32_t mw = tt < 2 ? f.mn_lo : f.mn_hi;
      const int ma = (int)((mw >> (16 * (tt & 1))) & 0xffu), mb = (int)((mw >> (16 * (tt & 1) + 8)) & 0xffu);
#pragma unroll
      for (int b = 0; b < MB; b++) {
        const size_t xb = (t0 + b) * nb + i;
        const int* xw = reinterpret_cast<const int*>(q8 + xb * 256) + L;
        int v = 0;
#pragma unroll
        for (int jg = 0; jg < 4; jg++)
          v += sc[2 * jg] * dp4a_s8(wlo[jg], __ldg(xw + 16 * jg), 0) + sc[2 * jg + 1] * dp4a_s8(whi[jg], __ldg(xw + 16 * jg + 8), 0);
        // mod.rs:749-756: hadd_epi16 (wrapping i16) of neighbouring bsums, then madd_epi16 with the mins
        const int2 b4 = __ldg(reinterpret_cast<const int2*>(bs + xb * 16 + 4 * tt));
        const int s0 = (int)(int16_t)((int16_t)(b4.x & 0xffff) + (int16_t)(b4.x >> 16));
        const int s1 = (int)(int16_t)((int16_t)(b4.y & 0xffff) + (int16_t)(b4.y >> 16));
        const size_t pi = ((size_t)b * 4 + q) * nb + i;
        part_f[pi * 8 + L] = make_float2((float)v, (float)(ma * s0 + mb * s1));
        if (L == 0) {
          const float dq = __ldg(d8 + xb);
          part_p[pi] = make_float2(__fmul_rn(dw, dq), __fmul_rn(ndminw, dq));
        }
      }
    }
    __syncwarp();  // every lane is done with the stage
    if (k + Q4P_S < n_my) issue(k + Q4P_S);
  }
  __syncthreads();
  // the ordered part: one lane per (activation row b, weight row q, L); b = warp, warp + 4, ...
  for (int b = warp; b < MB; b += Q4S_WARPS) {
    const float2* pf = part_f + ((size_t)b * 4 + q) * nb * 8 + L;
    const float2* pp = part_p + ((size_t)b * 4 + q) * nb;
    float acc = 0.0f, accm = 0.0f;
    for (size_t i = 0; i < nb; i++) {
      const float2 fv = pf[i * 8], pv = pp[i];
      acc = __fmaf_rn(pv.x, fv.x, acc);
      accm = __fmaf_rn(pv.y, fv.y, accm);
    }
    // hsum_ps over lanes L = 0..7 (dot.rs:447-456), mins: (m0+m2)+(m1+m3) (mod.rs:792-794)
    const float s = __fadd_rn(__shfl_xor_sync(0xffffffffu, acc, 4), acc);
    const float uu = __fadd_rn(s, __shfl_xor_sync(0xffffffffu, s, 1));
    const float main_val = __fadd_rn(uu, __shfl_xor_sync(0xffffffffu, uu, 2));
    const float m02 = __fadd_rn(accm, __shfl_xor_sync(0xffffffffu, accm, 2));
    const float min_val = __fadd_rn(m02, __shfl_xor_sync(0xffffffffu, m02, 1));
    const size_t row = row0 + q;
    if (L == 0 && row < row_end) out[(t0 + b) * n_rows + row] = __fadd_rn(main_val, min_val);
  }
}

// forward_dequant: w = (d*sc)*q - (dmin*m) in f32 (mod.rs:471-486), dotted with the f32 input.
// One warp per R consecutive weight rows, MP activation rows per pass; lane = 4 quant bytes (group j = lane/8,
// bytes 4L..4L+3, L = lane%8).  Super-blocks go U at a time.  Each (row, super-block, group) of a batch has one
// provider lane that loads the 16-byte header and forms d*sc and dmin*m of the group's two sub-blocks once; the
// lanes that need them fetch them by shuffle.  A nibble becomes the f32 2^23 + q by a byte permute, and
// fma(d*sc, 2^23 + q, -(d*sc)*2^23) is the correctly rounded (d*sc)*q of the reference because the product and the
// power-of-two term are exact inside the fma.
template <int MP, int R>
__global__ void q4k_dequant_matmul_kernel(const uint8_t* __restrict__ w, size_t nb, size_t n_rows,
                                          const float* __restrict__ x, float* __restrict__ out) {
  constexpr int U = R > 1 ? 4 : 8;
  constexpr int SLOTS = R * U * 4 / 32;   // provider slots per lane
  static_assert(R * U * 4 % 32 == 0, "provider slots must fill the warp");
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
  for (size_t i0 = 0; i0 < nb; i0 += U) {
    // provider slot s = (r * U + u) * 4 + g lives in lane s % 32, register s / 32
    float pd1[SLOTS], pm1[SLOTS], pd2[SLOTS], pm2[SLOTS];
#pragma unroll
    for (int sl = 0; sl < SLOTS; sl++) {
      const int s = sl * 32 + lane, g = s & 3, u = (s >> 2) % U, r = s / (4 * U);
      pd1[sl] = pm1[sl] = pd2[sl] = pm2[sl] = 0.0f;
      if (row0 + r < n_rows && i0 + u < nb) {
        const uint4 h = __ldg(reinterpret_cast<const uint4*>(w + ((row0 + r) * nb + i0 + u) * 144));
        const q4k_fields f = unpack_fields(h.y, h.z, h.w);
        const uint32_t scw = g < 2 ? f.sc_lo : f.sc_hi, mnw = g < 2 ? f.mn_lo : f.mn_hi;
        const float dw = f16_bits_to_f32((uint16_t)(h.x & 0xffffu)), dminw = f16_bits_to_f32((uint16_t)(h.x >> 16));
        const float s0 = __fsub_rn(g & 1 ? byte_plus_2p23(scw, 2) : byte_plus_2p23(scw, 0), 8388608.0f);
        const float s1 = __fsub_rn(g & 1 ? byte_plus_2p23(scw, 3) : byte_plus_2p23(scw, 1), 8388608.0f);
        const float n0 = __fsub_rn(g & 1 ? byte_plus_2p23(mnw, 2) : byte_plus_2p23(mnw, 0), 8388608.0f);
        const float n1 = __fsub_rn(g & 1 ? byte_plus_2p23(mnw, 3) : byte_plus_2p23(mnw, 1), 8388608.0f);
        pd1[sl] = __fmul_rn(dw, s0);
        pm1[sl] = __fmul_rn(dminw, n0);
        pd2[sl] = __fmul_rn(dw, s1);
        pm2[sl] = __fmul_rn(dminw, n1);
      }
    }
    uint32_t wqs[R][U];
#pragma unroll
    for (int r = 0; r < R; r++)
#pragma unroll
      for (int u = 0; u < U; u++)
        wqs[r][u] = row0 + r < n_rows && i0 + u < nb
                        ? __ldg(reinterpret_cast<const uint32_t*>(w + ((row0 + r) * nb + i0 + u) * 144 + 16 + 4 * lane))
                        : 0u;
#pragma unroll
    for (int u = 0; u < U; u++) {
      if (i0 + u >= nb) break;  // warp-uniform
      const size_t i = i0 + u;
      float wl[R][4], wh[R][4];
#pragma unroll
      for (int r = 0; r < R; r++) {
        const int s = (r * U + u) * 4;          // + j: the provider of this lane's group
        const int sl = s / 32, src = (s % 32) + j;
        const float d1 = __shfl_sync(0xffffffffu, pd1[sl], src), m1 = __shfl_sync(0xffffffffu, pm1[sl], src);
        const float d2 = __shfl_sync(0xffffffffu, pd2[sl], src), m2 = __shfl_sync(0xffffffffu, pm2[sl], src);
        const float c1 = -__fmul_rn(d1, 8388608.0f), c2 = -__fmul_rn(d2, 8388608.0f);
        const uint32_t wq = wqs[r][u];
        const uint32_t lo = wq & 0x0F0F0F0Fu, hi = (wq >> 4) & 0x0F0F0F0Fu;
#pragma unroll
        for (int k = 0; k < 4; k++) {
          wl[r][k] = __fsub_rn(__fmaf_rn(d1, byte_plus_2p23(lo, k), c1), m1);
          wh[r][k] = __fsub_rn(__fmaf_rn(d2, byte_plus_2p23(hi, k), c2), m2);
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
// Two groups of 256 threads share a tile and take alternate K chunks (each with its own pair of shared-memory
// stages and its own named barrier), so that a CTA brings 16 warps to an SM: a 4096 x 4096 weight with 256
// activation rows is only 128 tiles, and 8 warps per SM leave the FMA pipe idle most of the time.  The two
// partial tiles are added at the end (group 0 + group 1); forward_dequant carries a tolerance, not an order.
constexpr int Q4G_KGROUPS = 2;
constexpr size_t Q4G_GROUP_SMEM = 2 * Q4G_BK * (Q4G_BN + Q4G_PAD + Q4G_BM + Q4G_PAD) * 4;

__global__ void __launch_bounds__(256 * Q4G_KGROUPS)
    q4k_dequant_gemm_kernel(const uint8_t* __restrict__ w, size_t nb, size_t n_rows, const float* __restrict__ x,
                            size_t m_rows, float* __restrict__ out) {
  extern __shared__ __align__(16) uint8_t q4g_smem[];
  const int kg = threadIdx.x >> 8, tid = threadIdx.x & 255;
  uint8_t* gsm = q4g_smem + (size_t)kg * Q4G_GROUP_SMEM;
  float (*Ws)[Q4G_BK][Q4G_BN + Q4G_PAD] = reinterpret_cast<float (*)[Q4G_BK][Q4G_BN + Q4G_PAD]>(gsm);
  float (*Xs)[Q4G_BK][Q4G_BM + Q4G_PAD] =
      reinterpret_cast<float (*)[Q4G_BK][Q4G_BM + Q4G_PAD]>(gsm + 2 * Q4G_BK * (Q4G_BN + Q4G_PAD) * 4);
  const size_t n0 = (size_t)blockIdx.x * Q4G_BN, m0 = (size_t)blockIdx.y * Q4G_BM;
  const size_t K = nb * 256;
  const int n_chunks = (int)(nb * 8);   // a multiple of 8: both groups walk the same number of chunks
  auto group_sync = [&]() { asm volatile("bar.sync %0, 256;" ::"r"(1 + kg) : "memory"); };
  // loader roles: weights - thread (row tid/2, 16 of the chunk's 32 values); activations - thread (row tid/4, 8 values)
  const int wr = tid >> 1, wh = tid & 1;
  const int xr = tid >> 2, xq = tid & 3;
  const bool w_ok = n0 + wr < n_rows, x_ok = m0 + xr < m_rows;
  const uint8_t* wrow = w + (n0 + wr) * nb * 144;
  const float* xrow = x + (m0 + xr) * K;
  // compute roles: tx = weight rows 4tx..4tx+3 and 64+4tx..64+4tx+3 (the sixteen tx of a warp read 256 contiguous
  // bytes per load: no bank conflict), ty = 4 consecutive activation rows
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
    const float c1 = -__fmul_rn(d1, 8388608.0f);
    const uint32_t q[4] = {qv.x, qv.y, qv.z, qv.w};
#pragma unroll
    for (int v4 = 0; v4 < 4; v4++) {
      const uint32_t nib = hi ? (q[v4] >> 4) & 0x0F0F0F0Fu : q[v4] & 0x0F0F0F0Fu;
#pragma unroll
      for (int v = 0; v < 4; v++)   // (d*sc)*q as fma(d*sc, 2^23 + q, -(d*sc)*2^23): exact product, one rounding
        Ws[st][wh * 16 + 4 * v4 + v][wr] = w_ok ? __fsub_rn(__fmaf_rn(d1, byte_plus_2p23(nib, v), c1), m1) : 0.0f;
    }
    const float xv[8] = {xa.x, xa.y, xa.z, xa.w, xb.x, xb.y, xb.z, xb.w};
#pragma unroll
    for (int v = 0; v < 8; v++) Xs[st][xq * 8 + v][xr] = x_ok ? xv[v] : 0.0f;
  };

  fetch(kg);
  stash(kg, 0);
  group_sync();
  for (int c = kg, it = 0; c < n_chunks; c += Q4G_KGROUPS, it++) {
    const int st = it & 1;
    if (c + Q4G_KGROUPS < n_chunks) fetch(c + Q4G_KGROUPS);
#pragma unroll
    for (int k = 0; k < Q4G_BK; k++) {
      const float4 a0 = *reinterpret_cast<const float4*>(&Ws[st][k][tx * 4]);
      const float4 a1 = *reinterpret_cast<const float4*>(&Ws[st][k][64 + tx * 4]);
      const float4 b0 = *reinterpret_cast<const float4*>(&Xs[st][k][ty * 4]);
      const float av[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
      const float bv[4] = {b0.x, b0.y, b0.z, b0.w};
#pragma unroll
      for (int a = 0; a < 4; a++)
#pragma unroll
        for (int b = 0; b < 8; b++) acc[a][b] = __fmaf_rn(av[b], bv[a], acc[a][b]);
    }
    if (c + Q4G_KGROUPS < n_chunks) stash(c + Q4G_KGROUPS, st ^ 1);
    group_sync();
  }
  // group 1 hands its partial tile over through its own (now idle) stages: [32 values][256 threads]
  float* hand = reinterpret_cast<float*>(q4g_smem + Q4G_GROUP_SMEM);
  if (kg == 1) {
#pragma unroll
    for (int a = 0; a < 4; a++)
#pragma unroll
      for (int b = 0; b < 8; b++) hand[(a * 8 + b) * 256 + tid] = acc[a][b];
  }
  __syncthreads();
  if (kg != 0) return;
#pragma unroll
  for (int a = 0; a < 4; a++)
#pragma unroll
    for (int b = 0; b < 8; b++) acc[a][b] = __fadd_rn(acc[a][b], hand[(a * 8 + b) * 256 + tid]);
#pragma unroll
  for (int a = 0; a < 4; a++) {
    const size_t mrow = m0 + ty * 4 + a;
    if (mrow >= m_rows) continue;
    float* o = out + mrow * n_rows + n0 + tx * 4;   // columns 4tx..4tx+3, then 64 further on
    if (n0 + 64 + tx * 4 + 4 <= n_rows && (n_rows & 3) == 0) {
      *reinterpret_cast<float4*>(o) = make_float4(acc[a][0], acc[a][1], acc[a][2], acc[a][3]);
      *reinterpret_cast<float4*>(o + 64) = make_float4(acc[a][4], acc[a][5], acc[a][6], acc[a][7]);
    } else {
#pragma unroll
      for (int b = 0; b < 8; b++) {
        const size_t col = n0 + tx * 4 + (b < 4 ? b : 60 + b);
        if (col < n_rows) out[mrow * n_rows + col] = acc[a][b];
      }
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
  cudaError_t le = ctx->sem == RMI_SEM_SCALAR
                       ? rmi_launch(ctx, q8k_quantize_kernel<RMI_SEM_SCALAR>, dim3((unsigned)nb), dim3(256), 0, x, nb, d, qs, bsums)
                       : rmi_launch(ctx, q8k_quantize_kernel<RMI_SEM_AVX2>, dim3((unsigned)nb), dim3(256), 0, x, nb, d, qs, bsums);
  if (le != cudaSuccess) {
    rmi_set_error("launch of q8k_quantize failed: %s", cudaGetErrorString(le));
    return RMI_ERR_CUDA;
  }
  return rmi_post_launch(ctx, "q8k_quantize");
}

template <int MP>
static void q4k_q8k_launch(rmi_ctx* ctx, const rmi_weight* w, const float* d8, const int8_t* qs, const int16_t* bsums,
                           size_t groups, float* out, size_t row_begin, size_t row_end) {
  const size_t rows = row_end - row_begin, nb = w->n_in / 256;
  dim3 grid((unsigned)((rows + 3) / 4), (unsigned)groups);
  // only the scalar order runs here; the AVX2 order has the kernels above
  q4k_q8k_matmul_kernel<RMI_SEM_SCALAR, MP><<<grid, 128, 0, ctx->stream>>>(w->d_raw, nb, w->n_rows, d8, qs, bsums, out, row_begin, row_end);
}

// One launch of the split-K kernel over `groups` groups of mb (1 or 2) activation rows.
static int32_t q4k_ksplit_launch(rmi_ctx* ctx, const rmi_weight* w, size_t mb, const float* d8, const int8_t* qs,
                                 const int16_t* bsums, size_t groups, float* out, size_t row_begin, size_t row_end) {
  const size_t nb = w->n_in / 256, smem = q4p_smem_bytes(mb, nb);
  auto kern = mb == 2 ? q4k_q8k_ksplit_kernel<2> : q4k_q8k_ksplit_kernel<1>;
  if (smem > 48 * 1024 && cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) {
    rmi_set_error("cudaFuncSetAttribute(%zu B shared) failed", smem);
    return RMI_ERR_CUDA;
  }
  const dim3 grid((unsigned)((row_end - row_begin + 3) / 4), (unsigned)groups);
  cudaError_t le = rmi_launch(ctx, kern, grid, dim3(32 * Q4S_WARPS), smem, w->d_raw, nb, w->n_rows, d8, qs, bsums, out, row_begin,
                              row_end, ctx->d_status);
  if (le != cudaSuccess) {
    rmi_set_error("launch of q4k_q8k_ksplit failed: %s", cudaGetErrorString(le));
    return RMI_ERR_CUDA;
  }
  return rmi_post_launch(ctx, "q4k_q8k_ksplit");
}

// One launch of the streaming kernel over `groups` groups of mb (4 or 8) activation rows.
static int32_t q4k_stream_launch(rmi_ctx* ctx, const rmi_weight* w, size_t mb, const float* d8, const int8_t* qs,
                                 const int16_t* bsums, size_t groups, float* out, size_t row_begin, size_t row_end) {
  const size_t nb = w->n_in / 256, smem = q4s_smem_bytes(mb, nb);
  const size_t n_tiles = (row_end - row_begin + Q4S_TN - 1) / Q4S_TN;
  auto kern = mb == 8 ? q4k_q8k_stream_kernel<8> : q4k_q8k_stream_kernel<4>;
  if (smem > 48 * 1024 && cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) {
    rmi_set_error("cudaFuncSetAttribute(%zu B shared) failed", smem);
    return RMI_ERR_CUDA;
  }
  size_t per_sm = (ctx->smem_optin + 1024) / (smem + 1024);
  if (per_sm > 6) per_sm = 6;
  if (per_sm < 1) per_sm = 1;
  size_t grid = (size_t)ctx->sm_count * per_sm;
  if (grid > n_tiles) grid = n_tiles;
  const size_t tiles_per_cta = (n_tiles + grid - 1) / grid;
  grid = (n_tiles + tiles_per_cta - 1) / tiles_per_cta;   // every CTA walks the same number of tiles
  kern<<<dim3((unsigned)grid, (unsigned)groups), 32 * Q4S_WARPS, smem, ctx->stream>>>(w->d_raw, nb, w->n_rows, d8, qs, bsums, out,
                                                                                       row_begin, row_end, n_tiles, ctx->d_status);
  return rmi_post_launch(ctx, "q4k_q8k_stream");
}

int32_t launch_q4k_q8k_matmul(rmi_ctx* ctx, const rmi_weight* w, const float* d8, const int8_t* qs,
                              const int16_t* bsums, size_t m, float* out, size_t row_begin, size_t row_end) {
  if (m == 0 || row_begin >= row_end) return RMI_OK;
  const size_t nb = w->n_in / 256;
  if (m >= 32 && ctx->sem != RMI_SEM_SCALAR) {
    // many rows: tiled kernel, every weight super-block is fetched once per 16 activation rows
    dim3 grid((unsigned)((row_end - row_begin + Q4T_TN - 1) / Q4T_TN), (unsigned)((m + Q4T_TM - 1) / Q4T_TM));
    q4k_q8k_tiled_kernel<<<grid, 256, 0, ctx->stream>>>(w->d_raw, nb, w->n_rows, d8, qs, bsums, m, out, row_begin, row_end);
    return rmi_post_launch(ctx, "q4k_q8k_tiled");
  }
  if (ctx->sem != RMI_SEM_SCALAR) {
    // few rows: groups of 8 / 4 activation rows through the streaming kernel (16-row tiles, whole rows per warp),
    // groups of 2 / 1 through the split-K kernel (4-row tiles, the super-blocks of a row over four warps)
    size_t t = 0;
    while (t < m) {
      const size_t left = m - t;
      size_t mb = left >= 8 ? 8 : (left >= 4 ? 4 : (left >= 2 ? 2 : 1));
      while (mb >= 4 && q4s_smem_bytes(mb, nb) > ctx->smem_optin - 1024) mb >>= 1;
      RMI_REQUIRE(mb >= 4 || q4p_smem_bytes(mb, nb) <= ctx->smem_optin - 1024, RMI_ERR_UNSUPPORTED,
                  "n_in=%zu does not fit the Q4_K x Q8_K shared-memory buffers", w->n_in);
      const size_t groups = left / mb;
      const float* dp = d8 + t * nb;
      const int8_t* qp = qs + t * nb * 256;
      const int16_t* bp = bsums + t * nb * 16;
      float* op = out + t * w->n_rows;
      if (mb >= 4) RMI_TRY(q4k_stream_launch(ctx, w, mb, dp, qp, bp, groups, op, row_begin, row_end));
      else RMI_TRY(q4k_ksplit_launch(ctx, w, mb, dp, qp, bp, groups, op, row_begin, row_end));
      t += mb * groups;
    }
    return RMI_OK;
  }
  // scalar order: groups of 4 activation rows share one pass over the weights (all groups in one launch), then the remainder
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
    constexpr size_t smem = Q4G_KGROUPS * Q4G_GROUP_SMEM;
    if (cudaFuncSetAttribute(q4k_dequant_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) {
      rmi_set_error("cudaFuncSetAttribute(%zu B shared) failed", smem);
      return RMI_ERR_CUDA;
    }
    q4k_dequant_gemm_kernel<<<g2, 256 * Q4G_KGROUPS, smem, ctx->stream>>>(w->d_raw, nb, w->n_rows, x, m, out);
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
