// Q8_0 hot path on CUDA cores: weight re-layout, activation quantizer, the memory-bound
// GEMV family (1 <= M <= 8 activation rows per pass), exact block sums, SiLU*mul.
//
// Reference semantics reproduced bit for bit (paths inside the reference project):
//   quantizer  src/ops/quant/q8_0.rs:49-71 (scalar) :75-165 (NEON) :176-230 (AVX2)
//   GEMV       src/ops/kernel/q8_0/scalar.rs:31-58, neon.rs:49-73, avx2.rs:53-174
//   hsum       src/ops/dot.rs:447-456
#include "common.cuh"
#include "kernels.cuh"

// ---------------------------------------------------------------- weight re-layout

// raw GGUF rows ([f16 d][32 x i8] blocks, row stride blocks*34) -> tile16 records.
// One thread per (row, block); rows >= n_rows inside the last tile were zeroed by memset.
__global__ void q8_repack_tile16_kernel(const uint8_t* __restrict__ raw, uint8_t* __restrict__ dst,
                                        size_t n_rows, size_t blocks) {
  size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= n_rows * blocks) return;
  size_t row = idx / blocks, b = idx % blocks;
  const uint8_t* src = raw + (row * blocks + b) * 34;
  uint8_t* rec = dst + ((row / 16) * blocks + b) * Q8_REC_BYTES;
  size_t r = row % 16;
  rec[2 * r] = src[0];
  rec[2 * r + 1] = src[1];
  uint8_t* q = rec + 32 + 32 * r;
#pragma unroll
  for (int i = 0; i < 32; i++) q[i] = src[2 + i];
}

// tile16 rows of `src` appended after `row_off` rows of dst (v-stack); row_off % 16 may be != 0.
__global__ void q8_copy_rows_tile16_kernel(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst,
                                           size_t n_rows, size_t blocks, size_t row_off) {
  size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= n_rows * blocks) return;
  size_t row = idx / blocks, b = idx % blocks;
  const uint8_t* srec = src + ((row / 16) * blocks + b) * Q8_REC_BYTES;
  size_t drow = row + row_off;
  uint8_t* drec = dst + ((drow / 16) * blocks + b) * Q8_REC_BYTES;
  size_t rs = row % 16, rd = drow % 16;
  *reinterpret_cast<uint16_t*>(drec + 2 * rd) = *reinterpret_cast<const uint16_t*>(srec + 2 * rs);
  const int4* s = reinterpret_cast<const int4*>(srec + 32 + 32 * rs);
  int4* d = reinterpret_cast<int4*>(drec + 32 + 32 * rd);
  d[0] = s[0];
  d[1] = s[1];
}

// tile16 -> tcgen05 K-major core-matrix images + f32 scales [tile128][block][128].
__global__ void q8_build_umma_kernel(const uint8_t* __restrict__ t16, uint8_t* __restrict__ uq,
                                     float* __restrict__ us, size_t n_rows, size_t blocks,
                                     size_t n_slabs, size_t n_ff_perm) {
  // one thread per (row, 16-byte chunk)
  size_t chunks = blocks * 2;
  size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  size_t rows_pad = (n_rows + 127) / 128 * 128;
  if (idx >= rows_pad * n_slabs * 8) return;
  size_t row = idx / (n_slabs * 8), c_all = idx % (n_slabs * 8);
  size_t slab = c_all / 8, c = c_all % 8;
  int4 v = make_int4(0, 0, 0, 0);
  size_t b = c_all / 2;
  float s = 0.0f;
  // n_ff_perm != 0: destination rows [64t,64t+32) take gate rows 32t.., [64t+32,64t+64) the up
  // rows n_ff+32t.. of the v-stacked source
  size_t srow = row;
  if (n_ff_perm) srow = (row % 64 < 32) ? (row / 64) * 32 + row % 64 : n_ff_perm + (row / 64) * 32 + (row % 64 - 32);
  if (row < n_rows && srow < n_rows && c_all < chunks) {
    const uint8_t* rec = t16 + ((srow / 16) * blocks + b) * Q8_REC_BYTES;
    v = *reinterpret_cast<const int4*>(rec + 32 + 32 * (srow % 16) + 16 * (c_all & 1));
    s = f16_bits_to_f32(*reinterpret_cast<const uint16_t*>(rec + 2 * (srow % 16)));
  }
  size_t tile = row / 128, r = row % 128;
  uint8_t* img = uq + (tile * n_slabs + slab) * 16384;
  *reinterpret_cast<int4*>(img + (r / 8) * 1024 + c * 128 + (r % 8) * 16) = v;
  if ((c_all & 1) == 0 && b < blocks) us[(tile * blocks + b) * 128 + r] = s;
}

// ---------------------------------------------------------------- activation quantizer

// One warp per 32-block.  out_mode 0: q8 row-major [m][n], scales [m][n/32].
// out_mode 1: q8 in tcgen05 A-operand images ([tile128][slab][16 KiB]) and scales
// [tile128][block][128]; rows m..pad are written as zeros by the caller's memset.
template <int SEM>
__global__ void q8_quantize_kernel(const float* __restrict__ x, size_t m, size_t n,
                                   uint8_t* __restrict__ q8, float* __restrict__ scales,
                                   int out_mode) {
  pdl_wait();               // x may come from the preceding kernel of a dependent launch
  pdl_launch_dependents();
  size_t blocks = n / 32;
  size_t warp = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) / 32;
  int lane = threadIdx.x & 31;
  if (warp >= m * blocks) return;
  size_t row = warp / blocks, b = warp % blocks;
  float v = x[row * n + b * 32 + lane];
  float a = fabsf(v);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, o));
  float d, inv;
  q8_scale_pair<SEM>(a, &d, &inv);
  int q = q8_quant_value<SEM>(v, inv);
  float sc = f16_round_trip(d);
  if (out_mode == 0) {
    q8[row * n + b * 32 + lane] = (uint8_t)(int8_t)q;
    if (lane == 0) scales[row * blocks + b] = sc;
  } else {
    size_t n_slabs = (n + 127) / 128;
    size_t tile = row / 128, r = row % 128, k = b * 32 + lane;
    size_t slab = k / 128, c = (k % 128) / 16, byte = k % 16;
    q8[(tile * n_slabs + slab) * 16384 + (r / 8) * 1024 + c * 128 + (r % 8) * 16 + byte] =
        (uint8_t)(int8_t)q;
    if (lane == 0) scales[(tile * blocks + b) * 128 + r] = sc;
  }
}

// ---------------------------------------------------------------- GEMV

// LB bytes of each row's 32-byte block per lane; a warp covers LB rows of one 16-row tile.
// MP activation rows are processed per pass with the weights read once.  Weights are fetched
// in register batches of U blocks, two batches in flight (the next one is requested before the
// current one is consumed), so a warp keeps 2*U*32*LB bytes outstanding.
template <int LB>
struct gemv_batch {
  static constexpr int NL = LB / 4;
  static constexpr int U = LB == 16 ? 4 : (LB == 8 ? 8 : 16);
  int wq[U][NL];
  uint16_t wd[U];
};

template <int LB>
__device__ __forceinline__ void gemv_load_batch(gemv_batch<LB>& t, const uint8_t* qp, const uint8_t* sp, size_t b0,
                                                size_t blocks) {
  constexpr int U = gemv_batch<LB>::U;
#pragma unroll
  for (int u = 0; u < U; u++) {
    if (b0 + u < blocks) {
      const uint8_t* p = qp + (b0 + u) * Q8_REC_BYTES;
      if constexpr (LB == 16) {
        const int4 v = __ldg(reinterpret_cast<const int4*>(p));
        t.wq[u][0] = v.x; t.wq[u][1] = v.y; t.wq[u][2] = v.z; t.wq[u][3] = v.w;
      } else if constexpr (LB == 8) {
        const int2 v = __ldg(reinterpret_cast<const int2*>(p));
        t.wq[u][0] = v.x; t.wq[u][1] = v.y;
      } else {
        t.wq[u][0] = __ldg(reinterpret_cast<const int*>(p));
      }
      t.wd[u] = __ldg(reinterpret_cast<const uint16_t*>(sp + (b0 + u) * Q8_REC_BYTES));
    }
  }
}

template <int SEM, int LB, int MP>
__device__ __forceinline__ void gemv_consume_batch(const gemv_batch<LB>& t, size_t b0, size_t blocks, const int8_t* xq_s,
                                                   const float* xs_s, size_t K, int part,
                                                   float (&acc)[MP][SEM == RMI_SEM_AVX2 ? LB / 4 : 1]) {
  constexpr int U = gemv_batch<LB>::U, NL = LB / 4, LPR = 32 / LB;
#pragma unroll
  for (int u = 0; u < U; u++) {
    if (b0 + u < blocks) {
      const size_t b = b0 + u;
      const float wd = f16_bits_to_f32(t.wd[u]);
#pragma unroll
      for (int m = 0; m < MP; m++) {
        const int* xp = reinterpret_cast<const int*>(xq_s + m * K + b * 32 + part * LB);
        int xv[NL];
        if constexpr (LB == 16) {
          const int4 v = *reinterpret_cast<const int4*>(xp);
          xv[0] = v.x; xv[1] = v.y; xv[2] = v.z; xv[3] = v.w;
        } else if constexpr (LB == 8) {
          const int2 v = *reinterpret_cast<const int2*>(xp);
          xv[0] = v.x; xv[1] = v.y;
        } else {
          xv[0] = *xp;
        }
        const float da = __fmul_rn(wd, xs_s[m * blocks + b]);
        if constexpr (SEM == RMI_SEM_AVX2) {
          // avx2.rs:96-148: eight partial sums of four products, one FMA each
#pragma unroll
          for (int j = 0; j < NL; j++) {
            const int p = dp4a_s8(t.wq[u][j], xv[j], 0x4B400000);
            const float f = __fsub_rn(__int_as_float(p), 12582912.0f);
            acc[m][j] = __fmaf_rn(da, f, acc[m][j]);
          }
        } else {
          int dot = 0;
#pragma unroll
          for (int j = 0; j < NL; j++) dot = dp4a_s8(t.wq[u][j], xv[j], dot);
#pragma unroll
          for (int o = LPR / 2; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
          const float f = small_int_to_f32(dot);
          if constexpr (SEM == RMI_SEM_NEON) {
            acc[m][0] = __fmaf_rn(f, da, acc[m][0]);  // neon.rs:69
          } else {
            acc[m][0] = __fadd_rn(acc[m][0], __fmul_rn(da, f));  // scalar.rs:55
          }
        }
      }
    }
  }
}

// Short rows (K <= 2048) of a large single-row GEMV, e.g. the logits projection: a warp's whole job is one
// 16-row tile of 8..16 load batches, so the plain "load a batch, consume it" loop with eight warps per CTA
// (one activation staging per 128 rows) streams better than the double-buffered kernel below
// (measured 87 % against 75 % of the copy bandwidth at 151936 x 1024).
#ifndef RMI_GEMV_SHORT_MINB
#define RMI_GEMV_SHORT_MINB 1
#endif
template <int SEM, int LB, int MP>
__global__ void __launch_bounds__(256, RMI_GEMV_SHORT_MINB)
    q8_gemv_short_kernel(const uint8_t* __restrict__ w, size_t blocks, const uint8_t* __restrict__ xq,
                   const float* __restrict__ xs, float* __restrict__ out, size_t out_stride,
                   size_t row_begin, size_t row_end, size_t first_tile, const out_fanout fo) {
  constexpr int LPR = 32 / LB;      // lanes per row
  constexpr int NL = LB / 4;        // AVX2 lanes (dp4a groups) per thread
  constexpr int WPT = 16 / LB;      // warps per 16-row tile
  constexpr int U = LB == 16 ? 4 : 8;
  extern __shared__ __align__(128) uint8_t smem[];
  const size_t K = blocks * 32;
  int8_t* xq_s = reinterpret_cast<int8_t*>(smem);
  float* xs_s = reinterpret_cast<float*>(smem + MP * K);

  pdl_wait();
  pdl_launch_dependents();
  // stage the quantized activations (shared by every row)
  {
    const int4* src = reinterpret_cast<const int4*>(xq);
    int4* dst = reinterpret_cast<int4*>(xq_s);
    for (size_t i = threadIdx.x; i < MP * K / 16; i += blockDim.x) dst[i] = src[i];
    for (size_t i = threadIdx.x; i < MP * blocks; i += blockDim.x) xs_s[i] = xs[i];
  }
  __syncthreads();

  const int lane = threadIdx.x & 31;
  const size_t gw = (size_t)blockIdx.x * (blockDim.x / 32) + threadIdx.x / 32;
  const size_t tile = first_tile + gw / WPT;
  const int sub = (int)(gw % WPT);
  const int rit = sub * LB + lane / LPR;  // row in tile
  const int part = lane % LPR;
  const size_t row = tile * 16 + rit;
  if (tile * 16 >= row_end) return;  // whole warp out of range (uniform)

  const uint8_t* rec0 = w + tile * blocks * Q8_REC_BYTES;
  const uint8_t* qp = rec0 + 32 + rit * 32 + part * LB;
  const uint8_t* sp = rec0 + 2 * rit;

  float acc[MP][SEM == RMI_SEM_AVX2 ? NL : 1];
#pragma unroll
  for (int m = 0; m < MP; m++)
#pragma unroll
    for (int j = 0; j < (SEM == RMI_SEM_AVX2 ? NL : 1); j++) acc[m][j] = 0.0f;

  for (size_t b0 = 0; b0 < blocks; b0 += U) {
    int wq[U][NL];
    uint16_t wd_bits[U];
#pragma unroll
    for (int u = 0; u < U; u++) {
      if (b0 + u < blocks) {
        const uint8_t* p = qp + (b0 + u) * Q8_REC_BYTES;
        if (LB == 16) {
          int4 v = __ldg(reinterpret_cast<const int4*>(p));
          wq[u][0] = v.x; wq[u][NL > 1 ? 1 : 0] = v.y; wq[u][NL > 2 ? 2 : 0] = v.z; wq[u][NL > 3 ? 3 : 0] = v.w;
        } else if (LB == 8) {
          int2 v = __ldg(reinterpret_cast<const int2*>(p));
          wq[u][0] = v.x; wq[u][NL > 1 ? 1 : 0] = v.y;
        } else {
          wq[u][0] = __ldg(reinterpret_cast<const int*>(p));
        }
        wd_bits[u] = __ldg(reinterpret_cast<const uint16_t*>(sp + (b0 + u) * Q8_REC_BYTES));
      }
    }
#pragma unroll
    for (int u = 0; u < U; u++) {
      if (b0 + u < blocks) {
        const size_t b = b0 + u;
        const float wd = f16_bits_to_f32(wd_bits[u]);
#pragma unroll
        for (int m = 0; m < MP; m++) {
          const int* xp = reinterpret_cast<const int*>(xq_s + m * K + b * 32 + part * LB);
          const float da = __fmul_rn(wd, xs_s[m * blocks + b]);
          if (SEM == RMI_SEM_AVX2) {
            // avx2.rs:96-148: eight partial sums of four products, one FMA each
#pragma unroll
            for (int j = 0; j < NL; j++) {
              int p = dp4a_s8(wq[u][j], xp[j], 0x4B400000);
              float f = __fsub_rn(__int_as_float(p), 12582912.0f);
              acc[m][j] = __fmaf_rn(da, f, acc[m][j]);
            }
          } else {
            int dot = 0;
#pragma unroll
            for (int j = 0; j < NL; j++) dot = dp4a_s8(wq[u][j], xp[j], dot);
#pragma unroll
            for (int o = LPR / 2; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
            float f = small_int_to_f32(dot);
            if (SEM == RMI_SEM_NEON) {
              acc[m][0] = __fmaf_rn(f, da, acc[m][0]);  // neon.rs:69
            } else {
              acc[m][0] = __fadd_rn(acc[m][0], __fmul_rn(da, f));  // scalar.rs:55
            }
          }
        }
      }
    }
  }

#pragma unroll
  for (int m = 0; m < MP; m++) {
    float r;
    if (SEM == RMI_SEM_AVX2) {
      // dot.rs:447-456: s_i = a[i+4] + a[i]; (s0 + s1) + (s2 + s3)
      if (LB == 16) {
        float s[4];
#pragma unroll
        for (int j = 0; j < 4; j++)
          s[j] = __fadd_rn(__shfl_xor_sync(0xffffffffu, acc[m][j % NL], 1), acc[m][j % NL]);
        r = __fadd_rn(__fadd_rn(s[0], s[1]), __fadd_rn(s[2], s[3]));
      } else if (LB == 8) {
        float s0 = __fadd_rn(__shfl_xor_sync(0xffffffffu, acc[m][0], 2), acc[m][0]);
        float s1 = __fadd_rn(__shfl_xor_sync(0xffffffffu, acc[m][NL > 1 ? 1 : 0], 2), acc[m][NL > 1 ? 1 : 0]);
        float t = __fadd_rn(s0, s1);  // part 0: s0+s1, part 1: s2+s3
        float o = __shfl_xor_sync(0xffffffffu, t, 1);
        r = __fadd_rn(t, o);          // part 0: (s0+s1)+(s2+s3)
      } else {
        float s = __fadd_rn(__shfl_xor_sync(0xffffffffu, acc[m][0], 4), acc[m][0]);  // parts 0..3: s_part
        float t = __fadd_rn(s, __shfl_xor_sync(0xffffffffu, s, 1));                  // part 0: s0+s1, part 2: s2+s3
        r = __fadd_rn(t, __shfl_xor_sync(0xffffffffu, t, 2));                        // part 0: final
      }
    } else {
      r = acc[m][0];
    }
    if (part == 0 && row >= row_begin && row < row_end) store_fanout(out + m * out_stride + row, r, fo);
  }
}

template <int SEM, int LB, int MP>
__global__ void __launch_bounds__(256)
    q8_gemv_kernel(const uint8_t* __restrict__ w, size_t blocks, const uint8_t* __restrict__ xq,
                   const float* __restrict__ xs, float* __restrict__ out, size_t out_stride,
                   size_t row_begin, size_t row_end, size_t first_tile, const out_fanout fo) {
  constexpr int LPR = 32 / LB;      // lanes per row
  constexpr int NL = LB / 4;        // AVX2 lanes (dp4a groups) per thread
  constexpr int WPT = 16 / LB;      // warps per 16-row tile
  constexpr int U = gemv_batch<LB>::U;
  extern __shared__ __align__(128) uint8_t smem[];
  const size_t K = blocks * 32;
  int8_t* xq_s = reinterpret_cast<int8_t*>(smem);
  float* xs_s = reinterpret_cast<float*>(smem + MP * K);
  // blockIdx.y selects a group of MP activation rows: all groups stream the weights concurrently
  xq += (size_t)blockIdx.y * MP * K;
  xs += (size_t)blockIdx.y * MP * blocks;
  out += (size_t)blockIdx.y * MP * out_stride;

  const int lane = threadIdx.x & 31;
  const size_t gw = (size_t)blockIdx.x * (blockDim.x / 32) + threadIdx.x / 32;
  const size_t tile = first_tile + gw / WPT;
  const int sub = (int)(gw % WPT);
  const int rit = sub * LB + lane / LPR;  // row in tile
  const int part = lane % LPR;
  const size_t row = tile * 16 + rit;
  const bool active = tile * 16 < row_end;  // warp-uniform
  const uint8_t* rec0 = w + tile * blocks * Q8_REC_BYTES;
  const uint8_t* qp = rec0 + 32 + rit * 32 + part * LB;
  const uint8_t* sp = rec0 + 2 * rit;

  // first weight batch is requested before the activations are staged
  gemv_batch<LB> ba, bb;
  if (active) gemv_load_batch<LB>(ba, qp, sp, 0, blocks);
  pdl_wait();
  pdl_launch_dependents();
  {
    // asynchronous copies straight into shared memory, all of a thread's pieces in flight at once: a load / store
    // loop through registers waits for each batch in turn
    for (size_t i = threadIdx.x; i < MP * K / 16; i += blockDim.x)
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(xq_s + i * 16)),
                   "l"(xq + i * 16)
                   : "memory");
    for (size_t i = threadIdx.x; i < MP * blocks; i += blockDim.x)
      asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((uint32_t)__cvta_generic_to_shared(xs_s + i)),
                   "l"(xs + i)
                   : "memory");
    asm volatile("cp.async.commit_group;" ::: "memory");
    asm volatile("cp.async.wait_group 0;" ::: "memory");
  }
  __syncthreads();
  if (!active) return;

  float acc[MP][SEM == RMI_SEM_AVX2 ? NL : 1];
#pragma unroll
  for (int m = 0; m < MP; m++)
#pragma unroll
    for (int j = 0; j < (SEM == RMI_SEM_AVX2 ? NL : 1); j++) acc[m][j] = 0.0f;

  for (size_t b0 = 0; b0 < blocks; b0 += 2 * U) {
    if (b0 + U < blocks) gemv_load_batch<LB>(bb, qp, sp, b0 + U, blocks);
    gemv_consume_batch<SEM, LB, MP>(ba, b0, blocks, xq_s, xs_s, K, part, acc);
    if (b0 + 2 * U < blocks) gemv_load_batch<LB>(ba, qp, sp, b0 + 2 * U, blocks);
    if (b0 + U < blocks) gemv_consume_batch<SEM, LB, MP>(bb, b0 + U, blocks, xq_s, xs_s, K, part, acc);
  }

#pragma unroll
  for (int m = 0; m < MP; m++) {
    float r;
    if (SEM == RMI_SEM_AVX2) {
      // dot.rs:447-456: s_i = a[i+4] + a[i]; (s0 + s1) + (s2 + s3)
      if (LB == 16) {
        float s[4];
#pragma unroll
        for (int j = 0; j < 4; j++)
          s[j] = __fadd_rn(__shfl_xor_sync(0xffffffffu, acc[m][j % NL], 1), acc[m][j % NL]);
        r = __fadd_rn(__fadd_rn(s[0], s[1]), __fadd_rn(s[2], s[3]));
      } else if (LB == 8) {
        float s0 = __fadd_rn(__shfl_xor_sync(0xffffffffu, acc[m][0], 2), acc[m][0]);
        float s1 = __fadd_rn(__shfl_xor_sync(0xffffffffu, acc[m][NL > 1 ? 1 : 0], 2), acc[m][NL > 1 ? 1 : 0]);
        float t = __fadd_rn(s0, s1);  // part 0: s0+s1, part 1: s2+s3
        float o = __shfl_xor_sync(0xffffffffu, t, 1);
        r = __fadd_rn(t, o);          // part 0: (s0+s1)+(s2+s3)
      } else {
        float s = __fadd_rn(__shfl_xor_sync(0xffffffffu, acc[m][0], 4), acc[m][0]);  // parts 0..3: s_part
        float t = __fadd_rn(s, __shfl_xor_sync(0xffffffffu, s, 1));                  // part 0: s0+s1, part 2: s2+s3
        r = __fadd_rn(t, __shfl_xor_sync(0xffffffffu, t, 2));                        // part 0: final
      }
    } else {
      r = acc[m][0];
    }
    if (part == 0 && row >= row_begin && row < row_end) store_fanout(out + m * out_stride + row, r, fo);
  }
}

// ---------------------------------------------------------------- GEMV, small problems

// Latency-bound shapes (a few hundred 16-row tiles): one CTA of 128 threads per tile fetches the
// tile's whole record stream (blocks * 544 contiguous bytes) with a single bulk async copy, so
// the tile costs one memory round trip; thread (row r, lane l) then runs the reference's
// per-lane chain over the blocks out of shared memory.
//
// FUSED: the activations are not read pre-quantized; every CTA derives them itself while its
// weight copy is in flight: x = x_in (+ add), rms_norm(x, norm_w) (src/ops/norm.rs:3-11), Q8_0
// quantization.  The updated residual stream is written to x_out by the CTAs of tile 0 only
// (x_out must not alias x_in: other CTAs are still reading it).
struct gemv_norm_args {
  const float* x_in;
  const float* add;     // may be null
  const float* norm_w;
  float* x_out;         // may be null
  float eps;
};

template <int SEM, int MP, bool FUSED>
__global__ void __launch_bounds__(128)
    q8_gemv_staged_kernel(const uint8_t* __restrict__ w, size_t blocks, const uint8_t* __restrict__ xq,
                          const float* __restrict__ xs, float* __restrict__ out, size_t out_stride, size_t row_begin,
                          size_t row_end, size_t first_tile, rmi_dev_status* status, gemv_norm_args na,
                          const out_fanout fo) {
  extern __shared__ __align__(128) uint8_t smem[];
  const size_t K = blocks * 32;
  uint64_t* bar = reinterpret_cast<uint64_t*>(smem);
  uint8_t* wt = smem + 128;                                   // [blocks][544]
  int8_t* xq_s = reinterpret_cast<int8_t*>(wt + blocks * Q8_REC_BYTES);  // [MP][K]
  float* xs_s = reinterpret_cast<float*>(xq_s + MP * K);      // [MP][blocks]
  float* xf = xs_s + MP * blocks;                             // [MP][K], FUSED only
  if (!FUSED) {
    xq += (size_t)blockIdx.y * MP * K;
    xs += (size_t)blockIdx.y * MP * blocks;
  }
  out += (size_t)blockIdx.y * MP * out_stride;
  const size_t tile = first_tile + blockIdx.x;
  const uint32_t bar_a = (uint32_t)__cvta_generic_to_shared(bar);
  const uint32_t bytes = (uint32_t)(blocks * Q8_REC_BYTES);

  if (threadIdx.x == 0) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(bar_a));
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar_a), "r"(bytes) : "memory");
    // bulk copies are limited in size: issue 32 KiB pieces
    for (uint32_t off = 0; off < bytes; off += 32768) {
      const uint32_t n = bytes - off < 32768 ? bytes - off : 32768;
      asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                       (uint32_t)__cvta_generic_to_shared(wt + off)),
                   "l"(w + tile * blocks * Q8_REC_BYTES + off), "r"(n), "r"(bar_a)
                   : "memory");
    }
  }
  // the norm weight is a model weight like the tile: the first batch of it (the only one up to 1024 columns) is
  // requested before the wait as well, instead of after the two barriers of the norm below
  constexpr int NB = 8;
  float nw_pre[FUSED ? NB : 1];
  if (FUSED) {
#pragma unroll
    for (int u = 0; u < NB; u++) {
      const size_t blk = (threadIdx.x >> 5) + 4 * u;
      nw_pre[FUSED ? u : 0] = blk < blocks ? __ldg(na.norm_w + blk * 32 + (threadIdx.x & 31)) : 0.0f;
    }
  }
  pdl_wait();  // the weight copy above is in flight; everything below depends on the previous kernel
  pdl_launch_dependents();
  if (!FUSED) {
    // activations, in parallel with the weight copy: asynchronous copies straight into shared memory, all of a
    // thread's pieces in flight at once (a load / store loop through registers waits for each batch in turn)
    for (size_t i = threadIdx.x; i < MP * K / 16; i += blockDim.x)
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(xq_s + i * 16)),
                   "l"(xq + i * 16)
                   : "memory");
    for (size_t i = threadIdx.x; i < MP * blocks; i += blockDim.x)
      asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((uint32_t)__cvta_generic_to_shared(xs_s + i)),
                   "l"(xs + i)
                   : "memory");
    asm volatile("cp.async.commit_group;" ::: "memory");
    asm volatile("cp.async.wait_group 0;" ::: "memory");
  } else {
    __shared__ double s_part[MP][4];
    __shared__ float s_scale[MP];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const size_t seq0 = (size_t)blockIdx.y * MP;
    // Warp w owns the 32-blocks w, w+4, ...; they are handled NB at a time with every global load of a batch
    // (input, residual, norm weight) issued before the first use: loads inside a rolled loop would be serialised.
#pragma unroll
    for (int m = 0; m < MP; m++) {
      const float* xi = na.x_in + (seq0 + m) * K;
      const float* ad = na.add ? na.add + (seq0 + m) * K : nullptr;
      double part = 0.0;
      for (size_t b0 = warp; b0 < blocks; b0 += 4 * NB) {
        float v[NB], a2[NB];
#pragma unroll
        for (int u = 0; u < NB; u++) {
          const size_t blk = b0 + 4 * u;
          v[u] = blk < blocks ? __ldg(xi + blk * 32 + lane) : 0.0f;
          a2[u] = (ad && blk < blocks) ? __ldg(ad + blk * 32 + lane) : 0.0f;
        }
#pragma unroll
        for (int u = 0; u < NB; u++) {
          const size_t blk = b0 + 4 * u;
          if (blk < blocks) {
            const float val = ad ? __fadd_rn(v[u], a2[u]) : v[u];
            xf[m * K + blk * 32 + lane] = val;
            if (na.x_out && blockIdx.x == 0) na.x_out[(seq0 + m) * K + blk * 32 + lane] = val;
            part += (double)__fmul_rn(val, val);
          }
        }
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
      if (lane == 0) s_part[m][warp] = part;
    }
    __syncthreads();
    if (threadIdx.x < MP) {
      const double sum = s_part[threadIdx.x][0] + s_part[threadIdx.x][1] + s_part[threadIdx.x][2] + s_part[threadIdx.x][3];
      const float mean_sq = (float)(sum / (double)K);
      s_scale[threadIdx.x] = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(mean_sq, na.eps)));
    }
    __syncthreads();
    for (size_t b0 = warp; b0 < blocks; b0 += 4 * NB) {
      float nw[NB];
#pragma unroll
      for (int u = 0; u < NB; u++)
        nw[u] = b0 == (size_t)warp ? nw_pre[FUSED ? u : 0]
                                   : (b0 + 4 * u < blocks ? __ldg(na.norm_w + (b0 + 4 * u) * 32 + lane) : 0.0f);
#pragma unroll
      for (int m = 0; m < MP; m++) {
        const float sc = s_scale[m];
#pragma unroll
        for (int u = 0; u < NB; u++) {
          const size_t blk = b0 + 4 * u;
          if (blk < blocks) {
            const float v = __fmul_rn(__fmul_rn(xf[m * K + blk * 32 + lane], sc), nw[u]);
            float a = fabsf(v);
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, o));
            float d, inv;
            q8_scale_pair<SEM>(a, &d, &inv);
            xq_s[m * K + blk * 32 + lane] = (int8_t)q8_quant_value<SEM>(v, inv);
            if (lane == 0) xs_s[m * blocks + blk] = f16_round_trip(d);
          }
        }
      }
    }
  }
  __syncthreads();  // barrier initialised and activations staged
  {
    // bounded wait for the bulk copy (the context's wait limit), all threads observe the phase themselves
    const uint64_t limit_ns = status->limit_ns;
    uint64_t t0 = 0;
    bool done = false;
    for (uint32_t i = 0; i < (1u << 26) && !done; i++) {
      uint32_t ok;
      asm volatile(
          "{\n\t.reg .pred p;\n\t"
          "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
          "selp.u32 %0, 1, 0, p;\n\t}"
          : "=r"(ok)
          : "r"(bar_a), "r"(0u), "r"(20000u)
          : "memory");
      done = ok != 0;
      if (!done && (i & 15) == 15) {
        uint64_t now;
        asm volatile("mov.u64 %0, %globaltimer;" : "=l"(now));
        if (t0 == 0) t0 = now;
        else if (now - t0 > limit_ns) break;
      }
    }
    if (!done) {
      if (atomicCAS(&status->code, 0, RMI_ERR_TIMEOUT) == 0) {
        status->where = 10;
        status->detail = (int)tile;
      }
      return;
    }
  }

  const int rit = threadIdx.x >> 3, l = threadIdx.x & 7;
  const size_t row = tile * 16 + rit;
  float acc[MP];
#pragma unroll
  for (int m = 0; m < MP; m++) acc[m] = 0.0f;
  const uint8_t* qp = wt + 32 + rit * 32 + l * 4;
  const uint8_t* sp = wt + 2 * rit;
#pragma unroll 4
  for (size_t b = 0; b < blocks; b++) {
    const int wq = *reinterpret_cast<const int*>(qp + b * Q8_REC_BYTES);
    const float wd = f16_bits_to_f32(*reinterpret_cast<const uint16_t*>(sp + b * Q8_REC_BYTES));
#pragma unroll
    for (int m = 0; m < MP; m++) {
      const int xv = *reinterpret_cast<const int*>(xq_s + m * K + b * 32 + l * 4);
      const float da = __fmul_rn(wd, xs_s[m * blocks + b]);
      if (SEM == RMI_SEM_AVX2) {
        const float f = __fsub_rn(__int_as_float(dp4a_s8(wq, xv, 0x4B400000)), 12582912.0f);
        acc[m] = __fmaf_rn(da, f, acc[m]);  // avx2.rs:96-148, lane l of the eight
      } else {
        int dot = dp4a_s8(wq, xv, 0);
        dot += __shfl_xor_sync(0xffffffffu, dot, 1);
        dot += __shfl_xor_sync(0xffffffffu, dot, 2);
        dot += __shfl_xor_sync(0xffffffffu, dot, 4);
        const float f = small_int_to_f32(dot);
        if (SEM == RMI_SEM_NEON) acc[m] = __fmaf_rn(f, da, acc[m]);   // neon.rs:69
        else acc[m] = __fadd_rn(acc[m], __fmul_rn(da, f));            // scalar.rs:55
      }
    }
  }
#pragma unroll
  for (int m = 0; m < MP; m++) {
    float r = acc[m];
    if (SEM == RMI_SEM_AVX2) {  // dot.rs:447-456
      const float s = __fadd_rn(__shfl_xor_sync(0xffffffffu, r, 4), r);
      const float t = __fadd_rn(s, __shfl_xor_sync(0xffffffffu, s, 1));
      r = __fadd_rn(t, __shfl_xor_sync(0xffffffffu, t, 2));
    }
    if (l == 0 && row >= row_begin && row < row_end) store_fanout(out + m * out_stride + row, r, fo);
  }
}

// ---------------------------------------------------------------- GEMV, long streams

// Bandwidth-bound shapes with one or two activation rows and more 16-row tiles than the staged kernel takes
// (the config-5 shard at M = 1, the logits projection): persistent CTAs walk the tiles
// blockIdx.x, blockIdx.x + gridDim.x, ...  A tile's record stream (blocks * 544 contiguous bytes) is cut into
// chunks of STREAM_CB blocks that travel through a ring of STREAM_S shared-memory stages as bulk async copies
// (one elected thread, mbarrier transaction counts), so a CTA keeps STREAM_S * 17 KiB of reads in flight with
// no register staging, across tile boundaries.  64 threads per CTA: thread (row r, part p) owns bytes 8p..8p+7
// of every block of row r, i.e. two of the reference's eight per-lane chains, and runs them over the blocks in
// order out of shared memory.
// Measured on W [32768, 8192], M = 1 (fractions of the copy bandwidth): chunks of 8 / 16 / 32 / 48 / 64 blocks with
// 6 / 4 / 2 / 2 / 2 stages reach 0.50 / 0.77 / 0.88 / 0.83 / 0.64: large copies stream better as long as five CTAs
// still fit on an SM.
constexpr int STREAM_CB = 32;  // blocks per chunk: 32 * 544 = 17408 bytes
constexpr int STREAM_S = 2;    // stages
constexpr int STREAM_THREADS = 64;  // 16 rows x 4 lanes, 8 bytes of every block per lane

template <int SEM, int MP>
__global__ void __launch_bounds__(STREAM_THREADS)
    q8_gemv_stream_kernel(const uint8_t* __restrict__ w, size_t blocks, const uint8_t* __restrict__ xq,
                          const float* __restrict__ xs, float* __restrict__ out, size_t out_stride, size_t row_begin,
                          size_t row_end, size_t first_tile, size_t n_tiles, rmi_dev_status* status, const out_fanout fo) {
  extern __shared__ __align__(128) uint8_t smem[];
  const size_t K = blocks * 32;
  uint64_t* bar = reinterpret_cast<uint64_t*>(smem);                    // [STREAM_S]
  uint8_t* ring = smem + 128;                                           // [STREAM_S][STREAM_CB * 544]
  int8_t* xq_s = reinterpret_cast<int8_t*>(ring + STREAM_S * STREAM_CB * Q8_REC_BYTES);  // [MP][K]
  float* xs_s = reinterpret_cast<float*>(xq_s + MP * K);                // [MP][blocks]
  const uint32_t bar_a = (uint32_t)__cvta_generic_to_shared(bar);
  const uint32_t ring_a = (uint32_t)__cvta_generic_to_shared(ring);
  const int n_chunks = (int)((blocks + STREAM_CB - 1) / STREAM_CB);
  const size_t my_tiles = blockIdx.x < n_tiles ? (n_tiles - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
  const size_t n_items = my_tiles * (size_t)n_chunks;                   // (tile, chunk) pairs of this CTA, in order

  // item j -> stage j % STREAM_S; issued by thread 0 only
  auto issue = [&](size_t j) {
    const size_t tile = first_tile + blockIdx.x + (j / n_chunks) * gridDim.x;
    const int c = (int)(j % n_chunks);
    const size_t b0 = (size_t)c * STREAM_CB;
    const uint32_t nb = (uint32_t)(blocks - b0 < (size_t)STREAM_CB ? blocks - b0 : (size_t)STREAM_CB);
    const uint32_t bytes = nb * Q8_REC_BYTES;
    const uint32_t st = (uint32_t)(j % STREAM_S);
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar_a + 8 * st), "r"(bytes) : "memory");
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     ring_a + st * (uint32_t)(STREAM_CB * Q8_REC_BYTES)),
                 "l"(w + (tile * blocks + b0) * Q8_REC_BYTES), "r"(bytes), "r"(bar_a + 8 * st)
                 : "memory");
  };
  if (threadIdx.x == 0) {
    for (int i = 0; i < STREAM_S; i++) asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(bar_a + 8 * i));
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    for (size_t j = 0; j < n_items && j < (size_t)STREAM_S; j++) issue(j);   // weights: nobody in the chain writes them
  }
  pdl_wait();  // everything below depends on the previous kernel
  pdl_launch_dependents();
  {
    const int4* src = reinterpret_cast<const int4*>(xq);
    int4* dst = reinterpret_cast<int4*>(xq_s);
    for (size_t i = threadIdx.x; i < MP * K / 16; i += blockDim.x) dst[i] = __ldg(src + i);
    for (size_t i = threadIdx.x; i < MP * blocks; i += blockDim.x) xs_s[i] = __ldg(xs + i);
  }
  __syncthreads();  // barriers initialised, activations staged

  const int rit = threadIdx.x >> 2, part = threadIdx.x & 3;   // row in tile, which 8 bytes of the block
  const uint64_t limit_ns = status->limit_ns;
  float acc[MP][SEM == RMI_SEM_AVX2 ? 2 : 1];
  for (size_t j = 0; j < n_items; j++) {
    const int c = (int)(j % n_chunks);
    const uint32_t st = (uint32_t)(j % STREAM_S), parity = (uint32_t)((j / STREAM_S) & 1);
    if (c == 0) {
#pragma unroll
      for (int m = 0; m < MP; m++)
#pragma unroll
        for (int q = 0; q < (SEM == RMI_SEM_AVX2 ? 2 : 1); q++) acc[m][q] = 0.0f;
    }
    {
      // bounded wait for the chunk; every thread observes the phase itself
      uint64_t t0 = 0;
      bool done = false;
      for (uint32_t i = 0; i < (1u << 26) && !done; i++) {
        uint32_t ok;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(ok)
            : "r"(bar_a + 8 * st), "r"(parity), "r"(20000u)
            : "memory");
        done = ok != 0;
        if (!done && (i & 15) == 15) {
          uint64_t now;
          asm volatile("mov.u64 %0, %globaltimer;" : "=l"(now));
          if (t0 == 0) t0 = now;
          else if (now - t0 > limit_ns) break;
        }
      }
      if (!done) {  // the copies in flight target this CTA's own shared memory and are dropped with it
        if (atomicCAS(&status->code, 0, RMI_ERR_TIMEOUT) == 0) {
          status->where = 11;
          status->detail = (int)j;
        }
        return;
      }
    }
    const size_t b0 = (size_t)c * STREAM_CB;
    const int nb = (int)(blocks - b0 < (size_t)STREAM_CB ? blocks - b0 : (size_t)STREAM_CB);
    const uint8_t* wt = ring + st * (STREAM_CB * Q8_REC_BYTES);
    const uint8_t* qp = wt + 32 + rit * 32 + part * 8;
    const uint8_t* sp = wt + 2 * rit;
#pragma unroll 4
    for (int bi = 0; bi < nb; bi++) {
      const size_t b = b0 + bi;
      const int2 wq = *reinterpret_cast<const int2*>(qp + bi * Q8_REC_BYTES);
      const float wd = f16_bits_to_f32(*reinterpret_cast<const uint16_t*>(sp + bi * Q8_REC_BYTES));
#pragma unroll
      for (int m = 0; m < MP; m++) {
        const int2 xv = *reinterpret_cast<const int2*>(xq_s + m * K + b * 32 + part * 8);
        const float da = __fmul_rn(wd, xs_s[m * blocks + b]);
        if (SEM == RMI_SEM_AVX2) {
          // avx2.rs:96-148: lanes 2*part and 2*part+1 of the eight partial sums
          const float f0 = __fsub_rn(__int_as_float(dp4a_s8(wq.x, xv.x, 0x4B400000)), 12582912.0f);
          const float f1 = __fsub_rn(__int_as_float(dp4a_s8(wq.y, xv.y, 0x4B400000)), 12582912.0f);
          acc[m][0] = __fmaf_rn(da, f0, acc[m][0]);
          acc[m][SEM == RMI_SEM_AVX2 ? 1 : 0] = __fmaf_rn(da, f1, acc[m][SEM == RMI_SEM_AVX2 ? 1 : 0]);
        } else {
          int dot = dp4a_s8(wq.y, xv.y, dp4a_s8(wq.x, xv.x, 0));
          dot += __shfl_xor_sync(0xffffffffu, dot, 1);
          dot += __shfl_xor_sync(0xffffffffu, dot, 2);
          const float f = small_int_to_f32(dot);
          if (SEM == RMI_SEM_NEON) acc[m][0] = __fmaf_rn(f, da, acc[m][0]);   // neon.rs:69
          else acc[m][0] = __fadd_rn(acc[m][0], __fmul_rn(da, f));            // scalar.rs:55
        }
      }
    }
    __syncthreads();  // every thread is done with the stage
    if (threadIdx.x == 0 && j + STREAM_S < n_items) issue(j + STREAM_S);
    if (c == n_chunks - 1) {
      const size_t tile = first_tile + blockIdx.x + (j / n_chunks) * gridDim.x;
      const size_t row = tile * 16 + rit;
#pragma unroll
      for (int m = 0; m < MP; m++) {
        float r = acc[m][0];
        if (SEM == RMI_SEM_AVX2) {  // dot.rs:447-456: s_i = a[i+4] + a[i]; (s0 + s1) + (s2 + s3)
          const float a0 = acc[m][0], a1 = acc[m][SEM == RMI_SEM_AVX2 ? 1 : 0];
          const float s0 = __fadd_rn(__shfl_xor_sync(0xffffffffu, a0, 2), a0);
          const float s1 = __fadd_rn(__shfl_xor_sync(0xffffffffu, a1, 2), a1);
          const float t = __fadd_rn(s0, s1);  // part 0: s0+s1, part 1: s2+s3
          r = __fadd_rn(t, __shfl_xor_sync(0xffffffffu, t, 1));
        }
        if (part == 0 && row >= row_begin && row < row_end) store_fanout(out + m * out_stride + row, r, fo);
      }
    }
  }
}

// ---------------------------------------------------------------- exact block sums

__global__ void q8_block_sums_kernel(const uint8_t* __restrict__ w, size_t blocks, size_t n_rows,
                                     const uint8_t* __restrict__ xq, size_t m,
                                     int32_t* __restrict__ sums) {
  size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= m * n_rows * blocks) return;
  size_t b = idx % blocks, row = (idx / blocks) % n_rows, t = idx / (blocks * n_rows);
  const int* wp = reinterpret_cast<const int*>(w + ((row / 16) * blocks + b) * Q8_REC_BYTES + 32 + 32 * (row % 16));
  const int* xp = reinterpret_cast<const int*>(xq + t * blocks * 32 + b * 32);
  int dot = 0;
#pragma unroll
  for (int j = 0; j < 8; j++) dot = dp4a_s8(wp[j], xp[j], dot);
  sums[idx] = dot;
}

// ---------------------------------------------------------------- SiLU * mul (+ quantize)

// gate_up [m][2*n_ff] (gate columns first, then up).  act = up * (g / (1 + exp(-g)))
// (src/ops/activation/mod.rs:137-151), optionally written as f32 and/or re-quantized.
// One warp per 32-block of n_ff.
template <int SEM>
__global__ void silu_mul_quantize_kernel(const float* __restrict__ gate, const float* __restrict__ up,
                                         size_t in_stride, size_t m, size_t n_ff,
                                         float* __restrict__ act, uint8_t* __restrict__ q8,
                                         float* __restrict__ scales) {
  pdl_wait();
  pdl_launch_dependents();
  size_t blocks = n_ff / 32;
  size_t warp = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) / 32;
  int lane = threadIdx.x & 31;
  if (warp >= m * blocks) return;
  size_t row = warp / blocks, b = warp % blocks;
  float g = gate[row * in_stride + b * 32 + lane];
  float u = up[row * in_stride + b * 32 + lane];
  float s = __fdiv_rn(g, __fadd_rn(1.0f, exp_cr(-g)));
  float v = __fmul_rn(u, s);
  if (act) act[row * n_ff + b * 32 + lane] = v;
  if (q8) {
    float a = fabsf(v);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, o));
    float d, inv;
    q8_scale_pair<SEM>(a, &d, &inv);
    q8[row * n_ff + b * 32 + lane] = (uint8_t)(int8_t)q8_quant_value<SEM>(v, inv);
    if (lane == 0) scales[row * blocks + b] = f16_round_trip(d);
  }
}

// ---------------------------------------------------------------- f32-input matmul (ops::matmul_q8_0)

// Dequantized weight x f32 activation without activation quantization (src/ops/kernel/q8_0/parallel.rs:317-341).
// AVX2 (avx2.rs:180-217): two 8-lane accumulators per row; per block acc0 takes elements 0..7 and 16..23, acc1
// 8..15 and 24..31, each term fma(d * f32(q), x, acc); acc0 + acc1 lane by lane, then hsum_ps.  Thread (row r of
// the 16-row tile, chain c of 16) owns elements c and 16 + c of every block, which is lane c % 8 of acc c / 8.
// Every other instruction set runs scalar.rs:3-29: per block local += f32(q) * x over the 32 elements in order
// (separate multiply and add), sum += d * local; one thread per row.
template <int SEM>
__global__ void __launch_bounds__(256)
    q8_matmul_f32_kernel(const uint8_t* __restrict__ w, size_t blocks, size_t n_rows, const float* __restrict__ x,
                         float* __restrict__ out) {
  const int rit = threadIdx.x >> 4, c = threadIdx.x & 15;
  const size_t tile = blockIdx.x, row = tile * 16 + rit, K = blocks * 32;
  const float* xr = x + (size_t)blockIdx.y * K;
  const uint8_t* rec = w + tile * blocks * Q8_REC_BYTES;
  if (SEM == RMI_SEM_AVX2) {
    float acc = 0.0f;
    for (size_t b = 0; b < blocks; b++) {
      const uint8_t* r = rec + b * Q8_REC_BYTES;
      const float d = f16_bits_to_f32(*reinterpret_cast<const uint16_t*>(r + 2 * rit));
      const int8_t* q = reinterpret_cast<const int8_t*>(r + 32 + rit * 32);
      acc = __fmaf_rn(__fmul_rn(d, (float)q[c]), __ldg(xr + b * 32 + c), acc);
      acc = __fmaf_rn(__fmul_rn(d, (float)q[16 + c]), __ldg(xr + b * 32 + 16 + c), acc);
    }
    // acc0[L] + acc1[L], then dot.rs:447-456: s_i = a[i+4] + a[i]; (s0 + s1) + (s2 + s3)
    const float a = __fadd_rn(acc, __shfl_xor_sync(0xffffffffu, acc, 8));
    const float s = __fadd_rn(__shfl_xor_sync(0xffffffffu, a, 4), a);
    const float t = __fadd_rn(s, __shfl_xor_sync(0xffffffffu, s, 1));
    const float res = __fadd_rn(t, __shfl_xor_sync(0xffffffffu, t, 2));
    if (c == 0 && row < n_rows) out[(size_t)blockIdx.y * n_rows + row] = res;
  } else {
    if (c != 0 || row >= n_rows) return;
    float sum = 0.0f;
    for (size_t b = 0; b < blocks; b++) {
      const uint8_t* r = rec + b * Q8_REC_BYTES;
      const float d = f16_bits_to_f32(*reinterpret_cast<const uint16_t*>(r + 2 * rit));
      const int8_t* q = reinterpret_cast<const int8_t*>(r + 32 + rit * 32);
      float local = 0.0f;
      for (int k = 0; k < 32; k++) local = __fadd_rn(local, __fmul_rn((float)q[k], __ldg(xr + b * 32 + k)));
      sum = __fadd_rn(sum, __fmul_rn(d, local));
    }
    out[(size_t)blockIdx.y * n_rows + row] = sum;
  }
}

// ---------------------------------------------------------------- host launchers

int32_t launch_q8_repack_tile16(rmi_ctx* ctx, const uint8_t* raw, uint8_t* dst, size_t n_rows,
                                size_t blocks) {
  size_t n = n_rows * blocks;
  if (n == 0) return RMI_OK;
  q8_repack_tile16_kernel<<<(unsigned)((n + 255) / 256), 256, 0, ctx->stream>>>(raw, dst, n_rows, blocks);
  return rmi_post_launch(ctx, "q8_repack_tile16");
}

int32_t launch_q8_copy_rows_tile16(rmi_ctx* ctx, const uint8_t* src, uint8_t* dst, size_t n_rows,
                                   size_t blocks, size_t row_off) {
  size_t n = n_rows * blocks;
  if (n == 0) return RMI_OK;
  q8_copy_rows_tile16_kernel<<<(unsigned)((n + 255) / 256), 256, 0, ctx->stream>>>(src, dst, n_rows, blocks, row_off);
  return rmi_post_launch(ctx, "q8_copy_rows_tile16");
}

int32_t launch_q8_build_umma(rmi_ctx* ctx, const uint8_t* t16, uint8_t* uq, float* us, size_t n_rows,
                             size_t blocks, size_t n_ff_perm) {
  size_t n_slabs = (blocks * 32 + 127) / 128;
  size_t rows_pad = (n_rows + 127) / 128 * 128;
  size_t n = rows_pad * n_slabs * 8;
  if (n == 0) return RMI_OK;
  q8_build_umma_kernel<<<(unsigned)((n + 255) / 256), 256, 0, ctx->stream>>>(t16, uq, us, n_rows, blocks, n_slabs, n_ff_perm);
  return rmi_post_launch(ctx, "q8_build_umma");
}

int32_t launch_q8_quantize(rmi_ctx* ctx, const float* x, size_t m, size_t n, uint8_t* q8, float* scales,
                           int out_mode) {
  size_t warps = m * (n / 32);
  if (warps == 0) return RMI_OK;
  unsigned grid = (unsigned)((warps + 7) / 8);
  auto kern = ctx->sem == RMI_SEM_AVX2 ? q8_quantize_kernel<RMI_SEM_AVX2>
                                       : (ctx->sem == RMI_SEM_NEON ? q8_quantize_kernel<RMI_SEM_NEON> : q8_quantize_kernel<RMI_SEM_SCALAR>);
  const cudaError_t le = rmi_launch(ctx, kern, dim3(grid), dim3(256), 0, x, m, n, q8, scales, out_mode);
  if (le != cudaSuccess) {
    rmi_set_error("launch of q8_quantize failed: %s", cudaGetErrorString(le));
    return RMI_ERR_CUDA;
  }
  return rmi_post_launch(ctx, "q8_quantize");
}

template <int SEM, int LB, int MP>
static int32_t gemv_launch_one(rmi_ctx* ctx, const rmi_weight* w, const uint8_t* xq, const float* xs,
                               float* out, size_t out_stride, size_t row_begin, size_t row_end, size_t n_groups) {
  const size_t blocks = w->n_in / 32;
  const size_t first_tile = row_begin / 16;
  const size_t last_tile = (row_end + 15) / 16;
  const size_t warps = (last_tile - first_tile) * (16 / LB);
  const size_t smem = (size_t)MP * w->n_in + (size_t)MP * blocks * 4;
  const bool short_rows = MP == 1 && n_groups == 1 && blocks <= 64 && warps >= (size_t)ctx->sm_count * 16;
  auto kern = short_rows ? q8_gemv_short_kernel<SEM, LB, MP> : q8_gemv_kernel<SEM, LB, MP>;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) {
      rmi_set_error("cudaFuncSetAttribute(%zu B shared) failed: %s", smem, cudaGetErrorString(e));
      return RMI_ERR_CUDA;
    }
  }
  // fewer warps per CTA when the problem is small so that more SMs take part
  // several activation rows per pass: fatter CTAs share one staging of the MP*K activation bytes between more
  // weight rows (a 2-warp CTA would stage as many activation bytes as it reads weight bytes)
  int wpc = short_rows ? 8 : (warps * n_groups >= (size_t)ctx->sm_count * 8 ? 4 : 2);
  if (MP >= 4 && wpc == 2) wpc = 4;
  dim3 grid((unsigned)((warps + wpc - 1) / wpc), (unsigned)n_groups);
  const int pr = rmi_prof_begin(ctx, "q8_gemv");
  cudaError_t le = rmi_launch(ctx, kern, grid, dim3(wpc * 32), smem, w->d_tile16, blocks, xq, xs, out, out_stride,
                              row_begin, row_end, first_tile, ctx->fanout);
  rmi_prof_end(ctx, pr);
  if (le != cudaSuccess) {
    rmi_set_error("launch of q8_gemv failed: %s", cudaGetErrorString(le));
    return RMI_ERR_CUDA;
  }
  return rmi_post_launch(ctx, "q8_gemv");
}

#ifndef RMI_STREAM_MIN_BLOCKS
#define RMI_STREAM_MIN_BLOCKS 64
#endif

template <int SEM, int MP>
static int32_t gemv_dispatch_lb(rmi_ctx* ctx, const rmi_weight* w, const uint8_t* xq, const float* xs, float* out,
                                size_t out_stride, size_t row_begin, size_t row_end, size_t n_groups) {
  // Enough warps to keep every SM streaming: a pass over MP activation rows does MP times the
  // arithmetic per weight byte, so fewer (fatter) warps are needed as MP grows.
  {
    // small problem (up to six CTAs per SM): one CTA per tile and group of MP rows with the tile staged by a single
    // bulk copy, so a row's weights cost one memory round trip instead of one per register batch.  Measured on the
    // 0.6B decode step: batch 4 / 8 / 16 / 32 go from 2.08 / 3.37 / 5.73 / 9.42 to 3.03 / 3.92 / 6.19 / 9.93 k tok/s
    // with the passes of 4 and 8 rows included; twelve CTAs per SM is slower again (9.28 k at batch 32).
    const size_t t1 = (row_end + 15) / 16 - row_begin / 16, blocks = w->n_in / 32;
    const size_t smem = 128 + blocks * Q8_REC_BYTES + (size_t)MP * (w->n_in + blocks * 4);
    // wider passes only while two CTAs fit on an SM (an 8192-column tile with eight activation rows takes a whole SM
    // and ran slower than the register-staged kernel: 92 against 55 us for 4096 x 8192 at M = 16)
    if (t1 * n_groups <= (size_t)ctx->sm_count * 6 && smem <= ctx->smem_optin - 1024 && (MP <= 2 || smem <= 100 * 1024)) {
      auto kern = q8_gemv_staged_kernel<SEM, MP, false>;
      if (smem > 48 * 1024 &&
          cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) {
        rmi_set_error("cudaFuncSetAttribute(%zu B shared) failed", smem);
        return RMI_ERR_CUDA;
      }
      dim3 grid((unsigned)t1, (unsigned)n_groups);
      const int pr = rmi_prof_begin(ctx, "q8_gemv");
      cudaError_t le = rmi_launch(ctx, kern, grid, dim3(128), smem, w->d_tile16, blocks, xq, xs, out, out_stride,
                                  row_begin, row_end, row_begin / 16, ctx->d_status, gemv_norm_args{}, ctx->fanout);
      rmi_prof_end(ctx, pr);
      if (le != cudaSuccess) {
        rmi_set_error("launch of q8_gemv_staged failed: %s", cudaGetErrorString(le));
        return RMI_ERR_CUDA;
      }
      return rmi_post_launch(ctx, "q8_gemv_staged");
    }
  }
  {
    // many tiles, one or two activation rows: persistent CTAs stream the records through a ring of bulk copies
    const size_t t1 = (row_end + 15) / 16 - row_begin / 16, blocks = w->n_in / 32;
    const size_t smem = 128 + (size_t)STREAM_S * STREAM_CB * Q8_REC_BYTES + (size_t)MP * (w->n_in + blocks * 4);
    if (MP <= 2 && n_groups == 1 && blocks >= RMI_STREAM_MIN_BLOCKS && smem <= ctx->smem_optin - 1024) {
      auto kern = q8_gemv_stream_kernel<SEM, MP>;
      if (smem > 48 * 1024 &&
          cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) {
        rmi_set_error("cudaFuncSetAttribute(%zu B shared) failed", smem);
        return RMI_ERR_CUDA;
      }
      size_t per_sm = (ctx->smem_optin + 1024) / (smem + 1024);   // resident CTAs by shared memory
      if (per_sm > 8) per_sm = 8;
      if (per_sm < 1) per_sm = 1;
      // as many CTAs as can be resident, then trimmed so that every CTA walks the same number of tiles
      size_t grid = (size_t)ctx->sm_count * per_sm;
      if (grid > t1) grid = t1;
      const size_t tiles_per_cta = (t1 + grid - 1) / grid;
      grid = (t1 + tiles_per_cta - 1) / tiles_per_cta;
      const int pr = rmi_prof_begin(ctx, "q8_gemv");
      cudaError_t le = rmi_launch(ctx, kern, dim3((unsigned)grid), dim3(STREAM_THREADS), smem, w->d_tile16, blocks, xq, xs, out,
                                  out_stride, row_begin, row_end, row_begin / 16, t1, ctx->d_status, ctx->fanout);
      rmi_prof_end(ctx, pr);
      if (le != cudaSuccess) {
        rmi_set_error("launch of q8_gemv_stream failed: %s", cudaGetErrorString(le));
        return RMI_ERR_CUDA;
      }
      return rmi_post_launch(ctx, "q8_gemv_stream");
    }
  }
  const size_t tiles = ((row_end + 15) / 16 - row_begin / 16) * n_groups;
  const size_t per_sm = MP >= 8 ? 6 : (MP >= 4 ? 8 : 16);
  const size_t want = (size_t)ctx->sm_count * per_sm;
  if (tiles >= want) return gemv_launch_one<SEM, 16, MP>(ctx, w, xq, xs, out, out_stride, row_begin, row_end, n_groups);
  if (tiles * 2 >= want) return gemv_launch_one<SEM, 8, MP>(ctx, w, xq, xs, out, out_stride, row_begin, row_end, n_groups);
  return gemv_launch_one<SEM, 4, MP>(ctx, w, xq, xs, out, out_stride, row_begin, row_end, n_groups);
}

template <int SEM>
static int32_t gemv_dispatch_mp(rmi_ctx* ctx, const rmi_weight* w, const uint8_t* xq, const float* xs,
                                size_t m, float* out, size_t out_stride, size_t row_begin,
                                size_t row_end) {
  const size_t blocks = w->n_in / 32;
  size_t t = 0;
  // largest pass whose staged activations fit in shared memory
  size_t max_mp = 8;
  while (max_mp > 1 && max_mp * (w->n_in + blocks * 4) > ctx->smem_optin - 1024) max_mp >>= 1;
  RMI_REQUIRE(w->n_in + blocks * 4 <= ctx->smem_optin - 1024, RMI_ERR_UNSUPPORTED,
              "n_in=%zu does not fit the GEMV activation staging buffer", w->n_in);
  while (t < m) {
    size_t left = m - t;
    size_t mp = left >= 8 ? 8 : (left >= 4 ? 4 : (left >= 2 ? 2 : 1));
    if (mp > max_mp) mp = max_mp;
    const size_t groups = left / mp;  // all full groups of this width in one launch
    const uint8_t* q = xq + t * w->n_in;
    const float* s = xs + t * blocks;
    float* o = out + t * out_stride;
    int32_t st;
    switch (mp) {
      case 8: st = gemv_dispatch_lb<SEM, 8>(ctx, w, q, s, o, out_stride, row_begin, row_end, groups); break;
      case 4: st = gemv_dispatch_lb<SEM, 4>(ctx, w, q, s, o, out_stride, row_begin, row_end, groups); break;
      case 2: st = gemv_dispatch_lb<SEM, 2>(ctx, w, q, s, o, out_stride, row_begin, row_end, groups); break;
      default: st = gemv_dispatch_lb<SEM, 1>(ctx, w, q, s, o, out_stride, row_begin, row_end, groups); break;
    }
    if (st != RMI_OK) return st;
    t += mp * groups;
  }
  return RMI_OK;
}

// ---- rms_norm + quantize fused into the staged GEMV (decode, one or two sequences) ----
static size_t gemv_fused_smem(const rmi_weight* w, size_t mp) {
  const size_t blocks = w->n_in / 32;
  return 128 + blocks * Q8_REC_BYTES + mp * (w->n_in + blocks * 4) + mp * w->n_in * 4;
}

bool q8_gemv_fused_norm_eligible(const rmi_ctx* ctx, const rmi_weight* w, size_t m) {
  return (m == 1 || m == 2) && w->n_tiles16 <= (size_t)ctx->sm_count * 6 && gemv_fused_smem(w, m) <= ctx->smem_optin - 1024;
}

template <int SEM, int MP>
static int32_t gemv_fused_launch(rmi_ctx* ctx, const rmi_weight* w, const gemv_norm_args& na, float* out, size_t out_stride) {
  const size_t smem = gemv_fused_smem(w, MP), blocks = w->n_in / 32;
  auto kern = q8_gemv_staged_kernel<SEM, MP, true>;
  if (smem > 48 * 1024 && cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) {
    rmi_set_error("cudaFuncSetAttribute(%zu B shared) failed", smem);
    return RMI_ERR_CUDA;
  }
  const int pr = rmi_prof_begin(ctx, "q8_gemv");
  cudaError_t le = rmi_launch(ctx, kern, dim3((unsigned)w->n_tiles16, 1), dim3(128), smem, w->d_tile16, blocks,
                              (const uint8_t*)nullptr, (const float*)nullptr, out, out_stride, (size_t)0, w->n_rows,
                              (size_t)0, ctx->d_status, na, out_fanout{});
  rmi_prof_end(ctx, pr);
  if (le != cudaSuccess) {
    rmi_set_error("launch of q8_gemv_fused_norm failed: %s", cudaGetErrorString(le));
    return RMI_ERR_CUDA;
  }
  return rmi_post_launch(ctx, "q8_gemv_fused_norm");
}

int32_t launch_q8_gemv_fused_norm(rmi_ctx* ctx, const rmi_weight* w, const float* x_in, const float* add,
                                  const float* norm_w, float eps, float* x_out, size_t m, float* out, size_t out_stride) {
  RMI_REQUIRE(q8_gemv_fused_norm_eligible(ctx, w, m), RMI_ERR_UNSUPPORTED, "fused norm GEMV: shape not eligible");
  gemv_norm_args na = {x_in, add, norm_w, x_out, eps};
#define RMI_FUSED(SEMV) (m == 1 ? gemv_fused_launch<SEMV, 1>(ctx, w, na, out, out_stride) : gemv_fused_launch<SEMV, 2>(ctx, w, na, out, out_stride))
  switch (ctx->sem) {
    case RMI_SEM_AVX2: return RMI_FUSED(RMI_SEM_AVX2);
    case RMI_SEM_NEON: return RMI_FUSED(RMI_SEM_NEON);
    default: return RMI_FUSED(RMI_SEM_SCALAR);
  }
#undef RMI_FUSED
}

int32_t launch_q8_gemv(rmi_ctx* ctx, const rmi_weight* w, const uint8_t* xq, const float* xs, size_t m,
                       float* out, size_t out_stride, size_t row_begin, size_t row_end) {
  if (row_begin >= row_end || m == 0) return RMI_OK;
  switch (ctx->sem) {
    case RMI_SEM_AVX2: return gemv_dispatch_mp<RMI_SEM_AVX2>(ctx, w, xq, xs, m, out, out_stride, row_begin, row_end);
    case RMI_SEM_NEON: return gemv_dispatch_mp<RMI_SEM_NEON>(ctx, w, xq, xs, m, out, out_stride, row_begin, row_end);
    default: return gemv_dispatch_mp<RMI_SEM_SCALAR>(ctx, w, xq, xs, m, out, out_stride, row_begin, row_end);
  }
}

// embedding_lookup_q8_0 (src/ops/embedding.rs:12-22) from the tile16 layout: one CTA per requested row
__global__ void q8_embedding_kernel(const uint8_t* __restrict__ w, size_t blocks, const uint32_t* __restrict__ ids,
                                    float* __restrict__ out) {
  const uint32_t tok = ids[blockIdx.x];
  const uint8_t* base = w + (size_t)(tok / 16) * blocks * Q8_REC_BYTES;
  const int r = tok % 16;
  for (size_t i = threadIdx.x; i < blocks * 32; i += blockDim.x) {
    const uint8_t* rec = base + (i / 32) * Q8_REC_BYTES;
    const float d = f16_bits_to_f32(*reinterpret_cast<const uint16_t*>(rec + 2 * r));
    out[(size_t)blockIdx.x * blocks * 32 + i] = __fmul_rn(d, (float)(int8_t)rec[32 + 32 * r + (i & 31)]);
  }
}

int32_t launch_q8_embedding(rmi_ctx* ctx, const rmi_weight* w, const uint32_t* ids, size_t m, float* out) {
  if (m == 0) return RMI_OK;
  q8_embedding_kernel<<<(unsigned)m, 256, 0, ctx->stream>>>(w->d_tile16, w->n_in / 32, ids, out);
  return rmi_post_launch(ctx, "q8_embedding");
}

int32_t launch_q8_block_sums(rmi_ctx* ctx, const rmi_weight* w, const uint8_t* xq, size_t m,
                             int32_t* sums) {
  size_t n = m * w->n_rows * (w->n_in / 32);
  if (n == 0) return RMI_OK;
  q8_block_sums_kernel<<<(unsigned)((n + 255) / 256), 256, 0, ctx->stream>>>(w->d_tile16, w->n_in / 32,
                                                                            w->n_rows, xq, m, sums);
  return rmi_post_launch(ctx, "q8_block_sums");
}

int32_t launch_silu_mul_quantize(rmi_ctx* ctx, const float* gate, const float* up, size_t in_stride,
                                 size_t m, size_t n_ff, float* act, uint8_t* q8, float* scales) {
  size_t warps = m * (n_ff / 32);
  if (warps == 0) return RMI_OK;
  unsigned grid = (unsigned)((warps + 7) / 8);
  auto kern = ctx->sem == RMI_SEM_AVX2 ? silu_mul_quantize_kernel<RMI_SEM_AVX2>
                                       : (ctx->sem == RMI_SEM_NEON ? silu_mul_quantize_kernel<RMI_SEM_NEON>
                                                                   : silu_mul_quantize_kernel<RMI_SEM_SCALAR>);
  if (rmi_launch(ctx, kern, dim3(grid), dim3(256), 0, gate, up, in_stride, m, n_ff, act, q8, scales) != cudaSuccess) {
    rmi_set_error("launch of silu_mul_quantize failed: %s", cudaGetErrorString(cudaGetLastError()));
    return RMI_ERR_CUDA;
  }
  return rmi_post_launch(ctx, "silu_mul_quantize");
}

int32_t launch_q8_matmul_f32(rmi_ctx* ctx, const rmi_weight* w, const float* x, size_t m, float* out) {
  if (m == 0 || w->n_rows == 0) return RMI_OK;
  const dim3 grid((unsigned)w->n_tiles16, (unsigned)m);
  if (ctx->sem == RMI_SEM_AVX2)
    q8_matmul_f32_kernel<RMI_SEM_AVX2><<<grid, 256, 0, ctx->stream>>>(w->d_tile16, w->n_in / 32, w->n_rows, x, out);
  else
    q8_matmul_f32_kernel<RMI_SEM_SCALAR><<<grid, 256, 0, ctx->stream>>>(w->d_tile16, w->n_in / 32, w->n_rows, x, out);
  return rmi_post_launch(ctx, "q8_matmul_f32");
}
