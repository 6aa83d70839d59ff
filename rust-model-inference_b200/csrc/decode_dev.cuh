// Device helpers shared by the decode-step kernels (decode.cu) and the batched prefill (prefill.cu).
#pragma once
#include "common.cuh"

namespace {

__device__ __forceinline__ void cp_async16(void* dst_smem, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(dst_smem)), "l"(src)
               : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

// Copying `rows` rows of `row16` 16-byte pieces (global rows src_stride bytes apart, shared rows dst_stride bytes
// apart) with cp.async, the pieces dealt to the CTA's threads in order.  The (row, piece) of a thread advances by a
// fixed step, so the plan costs two 32-bit divisions per kernel and the copy loops none.
struct row_copy_plan {
  unsigned r0, c0, dr, dc, row16;
};
__device__ __forceinline__ row_copy_plan make_row_copy_plan(unsigned row16) {
  row_copy_plan p;
  p.row16 = row16;
  p.r0 = threadIdx.x / row16;
  p.c0 = threadIdx.x - p.r0 * row16;
  p.dr = blockDim.x / row16;
  p.dc = blockDim.x - p.dr * row16;
  return p;
}
__device__ __forceinline__ void cp_async_rows(const row_copy_plan& p, uint8_t* dst, size_t dst_stride, const void* src,
                                              size_t src_stride, unsigned rows) {
  const uint8_t* s = static_cast<const uint8_t*>(src);
  unsigned r = p.r0, c = p.c0;
  while (r < rows) {
    cp_async16(dst + r * dst_stride + c * 16, s + r * src_stride + c * 16);
    r += p.dr;
    c += p.dc;
    if (c >= p.row16) {
      c -= p.row16;
      r++;
    }
  }
}

__device__ __forceinline__ double warp_sum_f64(double v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// One head (hd values at src) by one warp: optional rms norm with weights nw (norm.rs:3-11), NeoX
// rotation with the (cos, sin) pairs of `tab` (rope.rs:21-37), f16 result (RNE) at dst.
__device__ __forceinline__ void norm_rope_head_f16(const float* __restrict__ src, const float* __restrict__ nw, float eps,
                                                   const float* __restrict__ tab, size_t hd, int lane, uint16_t* dst,
                                                   float* dst32 = nullptr) {
  const size_t half = hd / 2;
  if (dst32) {  // f32 result (the CLI forward keeps the query in f32): plain loops
    double part32 = 0.0;
    for (size_t i = lane; i < hd; i += 32) part32 += (double)__fmul_rn(src[i], src[i]);
    part32 = warp_sum_f64(part32);
    float sc32 = 1.0f;
    if (nw) sc32 = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn((float)(part32 / (double)hd), eps)));
    for (size_t i = lane; i < half; i += 32) {
      float x0 = src[i], x1 = src[i + half];
      if (nw) {
        x0 = __fmul_rn(__fmul_rn(x0, sc32), nw[i]);
        x1 = __fmul_rn(__fmul_rn(x1, sc32), nw[i + half]);
      }
      const float c = tab[2 * i], sn = tab[2 * i + 1];
      dst32[i] = __fmaf_rn(x0, c, __fmul_rn(x1, -sn));
      dst32[i + half] = __fmaf_rn(x0, sn, __fmul_rn(x1, c));
    }
    return;
  }
  if (hd == 128) {
    // the usual head size: every global load (values, norm weights, cos/sin) is issued before the first use
    float xv[4], wv[4];
#pragma unroll
    for (int u = 0; u < 4; u++) {
      xv[u] = src[lane + 32 * u];
      wv[u] = nw ? nw[lane + 32 * u] : 1.0f;
    }
    const float2 cs0 = *reinterpret_cast<const float2*>(tab + 2 * lane);
    const float2 cs1 = *reinterpret_cast<const float2*>(tab + 2 * (lane + 32));
    double part = 0.0;
#pragma unroll
    for (int u = 0; u < 4; u++) part += (double)__fmul_rn(xv[u], xv[u]);
    part = warp_sum_f64(part);
    if (nw) {
      const float mean_sq = (float)(part / 128.0);
      const float sc = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(mean_sq, eps)));
#pragma unroll
      for (int u = 0; u < 4; u++) xv[u] = __fmul_rn(__fmul_rn(xv[u], sc), wv[u]);
    }
#pragma unroll
    for (int u = 0; u < 2; u++) {  // pairs (i, i + 64), i = lane + 32 u
      const float x0 = xv[u], x1 = xv[u + 2];
      const float c = u == 0 ? cs0.x : cs1.x, sn = u == 0 ? cs0.y : cs1.y;
      dst[lane + 32 * u] = f32_to_f16_bits(__fmaf_rn(x0, c, __fmul_rn(x1, -sn)));
      dst[lane + 32 * u + 64] = f32_to_f16_bits(__fmaf_rn(x0, sn, __fmul_rn(x1, c)));
    }
    return;
  }
  double part = 0.0;
  for (size_t i = lane; i < hd; i += 32) part += (double)__fmul_rn(src[i], src[i]);
  part = warp_sum_f64(part);
  float sc = 1.0f;
  if (nw) {
    const float mean_sq = (float)(part / (double)hd);
    sc = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(mean_sq, eps)));
  }
  for (size_t i = lane; i < half; i += 32) {
    float x0 = src[i], x1 = src[i + half];
    if (nw) {
      x0 = __fmul_rn(__fmul_rn(x0, sc), nw[i]);
      x1 = __fmul_rn(__fmul_rn(x1, sc), nw[i + half]);
    }
    const float c = tab[2 * i], s = tab[2 * i + 1];
    const float r0 = __fmaf_rn(x0, c, __fmul_rn(x1, -s));
    const float r1 = __fmaf_rn(x0, s, __fmul_rn(x1, c));
    dst[i] = f32_to_f16_bits(r0);
    dst[i + half] = f32_to_f16_bits(r1);
  }
}


}  // namespace
