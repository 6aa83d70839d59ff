// Element-wise and attention kernels of the Qwen3 decode step, each reproducing the
// reference's x86 arithmetic (paths inside the reference project):
//   embedding row        src/ops/embedding.rs:12-22
//   rms_norm             src/ops/norm.rs:3-19        (f32 squares summed in f64)
//   rope_neox            src/ops/rope.rs:21-37       (cos/sin come from a host-built table)
//   K/V -> f16 cache     src/models/qwen3.rs:851-870
//   attention            src/models/qwen3.rs:876-933 (f16 q/k/v/p, f64 dot accumulation,
//                        sequential f32 softmax sum: src/ops/attention.rs:28-38)
//   greedy argmax        src/models/qwen3.rs:172-191 (first maximum, non-finite -> error)
#include <cooperative_groups.h>

#include "common.cuh"
#include "decode.cuh"
#include "decode_dev.cuh"
#include "kernels.cuh"

namespace {

// x[b][:] = f16(d) * q of the token's embedding row (tile16 layout).
__global__ void embed_kernel(const uint8_t* __restrict__ emb, size_t blocks, const uint32_t* __restrict__ prompts,
                             size_t n_prompt, const uint32_t* __restrict__ gen, size_t n_gen,
                             const int* __restrict__ d_step, float* __restrict__ x, uint32_t vocab) {
  pdl_wait();
  pdl_launch_dependents();
  const size_t b = blockIdx.x;
  const int step = *d_step;
  uint32_t tok = (size_t)step < n_prompt ? prompts[b * n_prompt + step] : gen[b * n_gen + (step - n_prompt)];
  if (tok >= vocab) tok = 0;  // out-of-range ids are rejected on the host before the first step
  const uint8_t* base = emb + (size_t)(tok / 16) * blocks * Q8_REC_BYTES;
  const int r = tok % 16;
  for (size_t i = threadIdx.x; i < blocks * 32; i += blockDim.x) {
    const uint8_t* rec = base + (i / 32) * Q8_REC_BYTES;
    const float d = f16_bits_to_f32(*reinterpret_cast<const uint16_t*>(rec + 2 * r));
    x[b * blocks * 32 + i] = __fmul_rn(d, (float)(int8_t)rec[32 + 32 * r + (i & 31)]);
  }
}

// Optional residual add (x += add), rms_norm(x, weight) and Q8_0 quantization of the result.
// One CTA of 256 threads per sequence; warp w owns 32-blocks w, w+8, ...
template <int SEM>
__global__ void rmsnorm_quant_kernel(float* __restrict__ x, const float* __restrict__ add,
                                     const float* __restrict__ weight, size_t n, float eps,
                                     uint8_t* __restrict__ q8, float* __restrict__ scales) {
  __shared__ double s_part[8];
  __shared__ float s_scale;
  pdl_wait();
  pdl_launch_dependents();
  const size_t b = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const size_t blocks = n / 32;
  float* xr = x + b * n;
  double part = 0.0;
  constexpr int NB = 4;  // blocks per batch: all loads of a batch are issued before the first use
  for (size_t b0 = warp; b0 < blocks; b0 += 8 * NB) {
    float v[NB], a2[NB];
#pragma unroll
    for (int u = 0; u < NB; u++) {
      const size_t blk = b0 + 8 * u;
      v[u] = blk < blocks ? xr[blk * 32 + lane] : 0.0f;
      a2[u] = (add && blk < blocks) ? add[b * n + blk * 32 + lane] : 0.0f;
    }
#pragma unroll
    for (int u = 0; u < NB; u++) {
      const size_t blk = b0 + 8 * u;
      if (blk < blocks) {
        float val = v[u];
        if (add) {
          val = __fadd_rn(val, a2[u]);
          xr[blk * 32 + lane] = val;
        }
        part += (double)__fmul_rn(val, val);
      }
    }
  }
  part = warp_sum_f64(part);
  if (lane == 0) s_part[warp] = part;
  __syncthreads();
  if (threadIdx.x == 0) {
    double s = 0.0;
    for (int w = 0; w < 8; w++) s += s_part[w];
    const float mean_sq = (float)(s / (double)n);
    s_scale = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(mean_sq, eps)));
  }
  __syncthreads();
  const float sc = s_scale;
  for (size_t b0 = warp; b0 < blocks; b0 += 8 * NB) {
    float xv[NB], wv[NB];
#pragma unroll
    for (int u = 0; u < NB; u++) {
      const size_t blk = b0 + 8 * u;
      xv[u] = blk < blocks ? xr[blk * 32 + lane] : 0.0f;
      wv[u] = blk < blocks ? weight[blk * 32 + lane] : 0.0f;
    }
#pragma unroll
    for (int u = 0; u < NB; u++) {
      const size_t blk = b0 + 8 * u;
      if (blk < blocks) {
        const float v = __fmul_rn(__fmul_rn(xv[u], sc), wv[u]);
        float a = fabsf(v);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, o));
        float d, inv;
        q8_scale_pair<SEM>(a, &d, &inv);
        q8[b * n + blk * 32 + lane] = (uint8_t)(int8_t)q8_quant_value<SEM>(v, inv);
        if (lane == 0) scales[b * blocks + blk] = f16_round_trip(d);
      }
    }
  }
}

// Per-head q/k rms_norm, NeoX rope, f16 conversion; K and V appended to the cache.
// grid (batch, n_head + 2*n_head_kv), one warp per head.
__global__ void qk_norm_rope_kv_kernel(const float* __restrict__ qkv, size_t n_head, size_t n_head_kv, size_t hd,
                                       const float* __restrict__ q_norm, const float* __restrict__ k_norm, float eps,
                                       const float* __restrict__ rope, const int* __restrict__ d_step,
                                       uint16_t* __restrict__ q16, uint16_t* __restrict__ k_cache,
                                       uint16_t* __restrict__ v_cache, size_t layer, size_t n_layer,
                                       size_t capacity, float* __restrict__ q32, float* __restrict__ k32_cache,
                                       float* __restrict__ v32_cache) {
  pdl_wait();
  pdl_launch_dependents();
  const size_t b = blockIdx.x, head = blockIdx.y;
  const int lane = threadIdx.x;
  const int step = *d_step;
  const size_t nq = n_head * hd, nk = n_head_kv * hd;
  const float* src = qkv + b * (nq + 2 * nk) + head * hd;
  const size_t cache_row = ((b * n_layer + layer) * capacity + (size_t)step) * nk;
  if (head >= n_head + n_head_kv) {  // V: straight f16 conversion, or an f32 copy (text.rs:393-405)
    const size_t kvh = head - n_head - n_head_kv;
    if (v32_cache) {
      for (size_t i = lane; i < hd; i += 32) v32_cache[cache_row + kvh * hd + i] = src[i];
      return;
    }
    for (size_t i = lane; i < hd; i += 32) v_cache[cache_row + kvh * hd + i] = f32_to_f16_bits(src[i]);
    return;
  }
  if (k32_cache && head >= n_head) {  // K kept in f32
    norm_rope_head_f16(src, k_norm, eps, rope + (size_t)step * hd, hd, lane, nullptr,
                       k32_cache + cache_row + (head - n_head) * hd);
    return;
  }
  const bool is_q = head < n_head;
  uint16_t* dst = is_q ? q16 + b * nq + head * hd : k_cache + cache_row + (head - n_head) * hd;
  norm_rope_head_f16(src, is_q ? q_norm : k_norm, eps, rope + (size_t)step * hd, hd, lane, dst,
                     (is_q && q32) ? q32 + b * nq + head * hd : nullptr);
}

// Attention for one (sequence, kv head) by a thread-block cluster of CL CTAs; the `group`
// query heads that share the kv head are processed together.  CTA r owns the time steps
// [r*chunk, (r+1)*chunk): it stages its K and V rows in shared memory (cp.async, V overlapped
// with the score pass), computes its scores with the reference's sequential f64 dot, and
// publishes them into every CTA's score array through distributed shared memory.  After a
// cluster barrier each CTA evaluates the soft-max over all T scores (max, exp, the
// reference's sequential f32 sum, divide, f16), forms the f64 partial of P.V over its own
// steps and sends it to CTA 0, which adds the partials in rank order, re-quantizes the
// group*hd outputs to Q8_0 for the Wo projection and writes them.
//
// With fq.qkv set the kernel also does the step's q/k norm + rotation and cache write itself
// (qwen3.rs:851-870): every CTA derives the group's f16 query heads from the f32 projection, and
// the CTA that owns the current time step derives the new K and V rows, keeps them in its staged
// tiles and stores them into the caches.
struct attn_fused_qk {
  const float* qkv;     // [batch][nq + 2 nk] f32 projections of this step, or null
  const float* q_norm;  // may be null
  const float* k_norm;  // may be null
  const float* rope;    // [pos][hd/2][2]
  float eps;
};

template <int SEM, bool FQ>
__global__ void __launch_bounds__(256)
    attention_kernel(const uint16_t* __restrict__ q16, uint16_t* __restrict__ k_cache,
                     uint16_t* __restrict__ v_cache, const int* __restrict__ d_step, size_t n_head,
                     size_t n_head_kv, size_t hd, size_t layer, size_t n_layer, size_t capacity, size_t chunk,
                     float* __restrict__ attn_out, uint8_t* __restrict__ q8, float* __restrict__ scales,
                     const attn_fused_qk fq) {
  namespace cg = cooperative_groups;
  cg::cluster_group cluster = cg::this_cluster();
  const unsigned CL = cluster.num_blocks(), rank = cluster.block_rank();
  extern __shared__ __align__(16) uint8_t smem[];
  // Dependent launch.  Without the fused q/k part everything below reads what the preceding kernel wrote (the
  // query heads and the newest cache rows).  With it (FQ) the step counter and the cache rows of earlier positions
  // were written at least two kernels ago (the counter at the end of the previous step, the rows in earlier steps;
  // the predecessor of this kernel has passed its own wait, so all of that is complete and visible): the K/V staging
  // below is issued first and the wait comes just before the q|k|v projection is read.
  if (!FQ) pdl_wait();
  pdl_launch_dependents();
  // Distributed shared memory of another CTA may only be touched once that CTA is known to run: every CTA
  // arrives here and waits just before its first remote store (the staging below overlaps the barrier).
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  const size_t b = blockIdx.y, kvh = blockIdx.x / CL;
  const size_t group = n_head / n_head_kv, nq = n_head * hd, nk = n_head_kv * hd;
  const int T = *d_step + 1;
  const size_t cs = (capacity + 3) & ~(size_t)3;  // score row stride (keeps 16-byte alignment)
  const size_t kstride = hd * 2 + 16;  // bytes; the pad spreads rows over the banks
  // layout (all offsets multiples of 16 bytes)
  double* part = reinterpret_cast<double*>(smem);                            // [CL][group*hd] (used on rank 0)
  float* sc = reinterpret_cast<float*>(part + (size_t)CL * group * hd);      // [group][capacity]
  float* outv = sc + group * cs;                                       // [group*hd]
  float* red = outv + group * hd;                                            // [group] sums
  uint16_t* qs = reinterpret_cast<uint16_t*>(red + ((group + 3) & ~(size_t)3));  // [group][hd]
  uint16_t* p16 = qs + group * hd;                                           // [group][chunk]
  uint8_t* kbuf = reinterpret_cast<uint8_t*>(p16 + ((group * chunk + 7) & ~(size_t)7));  // [chunk][kstride]
  uint8_t* vbuf = kbuf + chunk * kstride;                                    // [chunk][hd*2]

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nwarp = blockDim.x >> 5;
  const int t0 = (int)(rank * chunk);
  const int n_t = T > t0 ? (T - t0 < (int)chunk ? T - t0 : (int)chunk) : 0;
  const float kq_scale = __fdiv_rn(1.0f, __fsqrt_rn((float)hd));
  const uint16_t* kbase = k_cache + ((b * n_layer + layer) * capacity + t0) * nk + kvh * hd;
  const uint16_t* vbase = v_cache + ((b * n_layer + layer) * capacity + t0) * nk + kvh * hd;

  // stage q, K (group 0) and V (group 1) with 16-byte async copies
  const size_t row16 = hd / 8;  // 16-byte pieces per row
  constexpr bool fused = FQ;
  const bool owner = fused && n_t > 0 && t0 + n_t == T;  // this CTA holds the current time step
  const int n_ld = owner ? n_t - 1 : n_t;                 // rows that already sit in the caches
  if (!fused)
    for (size_t i = tid; i < group * row16; i += blockDim.x)
      cp_async16(qs + i * 8, q16 + b * nq + kvh * group * hd + i * 8);
  const row_copy_plan plan = make_row_copy_plan((unsigned)row16);
  cp_async_rows(plan, kbuf, kstride, kbase, nk * 2, (unsigned)n_ld);
  cp_async_commit();
  cp_async_rows(plan, vbuf, hd * 2, vbase, nk * 2, (unsigned)n_ld);
  cp_async_commit();
  if (fused) {
    pdl_wait();
    const float* proj = fq.qkv + b * (nq + 2 * nk);
    const float* tab = fq.rope + (size_t)(T - 1) * hd;
    for (size_t unit = warp; unit < group + 2; unit += nwarp) {
      if (unit < group) {
        norm_rope_head_f16(proj + (kvh * group + unit) * hd, fq.q_norm, fq.eps, tab, hd, lane, qs + unit * hd);
      } else if (owner) {
        const size_t tl = (size_t)n_t - 1;
        const size_t cache_off = (size_t)tl * nk;  // relative to kbase / vbase
        if (unit == group) {
          uint16_t* krow = reinterpret_cast<uint16_t*>(kbuf + tl * kstride);
          norm_rope_head_f16(proj + nq + kvh * hd, fq.k_norm, fq.eps, tab, hd, lane, krow);
          __syncwarp();
          uint16_t* kg = k_cache + ((b * n_layer + layer) * capacity + t0) * nk + kvh * hd + cache_off;
          for (size_t i = lane; i < hd; i += 32) kg[i] = krow[i];
        } else {
          uint16_t* vrow = reinterpret_cast<uint16_t*>(vbuf) + tl * hd;
          uint16_t* vg = v_cache + ((b * n_layer + layer) * capacity + t0) * nk + kvh * hd + cache_off;
          const float* vsrc = proj + nq + nk + kvh * hd;
          for (size_t i0 = lane; i0 < hd; i0 += 128) {  // four loads in flight per lane
            float vv[4];
#pragma unroll
            for (int u = 0; u < 4; u++) vv[u] = i0 + 32 * u < hd ? vsrc[i0 + 32 * u] : 0.0f;
#pragma unroll
            for (int u = 0; u < 4; u++) {
              const size_t i = i0 + 32 * u;
              if (i < hd) {
                const uint16_t h = f32_to_f16_bits(vv[u]);
                vrow[i] = h;
                vg[i] = h;
              }
            }
          }
        }
      }
    }
  }
  cp_async_wait<1>();
  __syncthreads();
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");  // all CTAs of the cluster have started

  // scores[g][t] = f32(sum_f64 q*k) * kq_scale, sequential over the head dimension (dot.rs:115-118)
  const unsigned grp = (unsigned)group, hdu = (unsigned)hd;
  for (unsigned item = tid; item < (unsigned)n_t * grp; item += blockDim.x) {
    const unsigned tl = item / grp, g = item - tl * grp;
    const uint32_t* kr = reinterpret_cast<const uint32_t*>(kbuf + tl * kstride);
    const uint32_t* qr = reinterpret_cast<const uint32_t*>(qs + g * hd);
    double s = 0.0;
    for (size_t i = 0; i < hd / 2; i++) {
      const uint32_t kk = kr[i], qq = qr[i];
      s += (double)__fmul_rn(f16_bits_to_f32((uint16_t)(qq & 0xffff)), f16_bits_to_f32((uint16_t)(kk & 0xffff)));
      s += (double)__fmul_rn(f16_bits_to_f32((uint16_t)(qq >> 16)), f16_bits_to_f32((uint16_t)(kk >> 16)));
    }
    const float v = __fmul_rn((float)s, kq_scale);
    for (unsigned rr = 0; rr < CL; rr++) cluster.map_shared_rank(sc, rr)[g * cs + t0 + tl] = v;
  }
  cluster.sync();

  if (n_t > 0) {
    // max, exp, sequential f32 sum (attention.rs:28-38), divide, f16 for this CTA's steps
    for (size_t g = warp; g < group; g += nwarp) {
      float mx = -INFINITY;
      for (int t = lane; t < T; t += 32) mx = fmaxf(mx, sc[g * cs + t]);
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
      if (lane == 0) red[g] = mx;
    }
    __syncthreads();
    for (unsigned i = tid; i < grp * (unsigned)T; i += blockDim.x) {
      const unsigned g = i / (unsigned)T, t = i - g * (unsigned)T;
      sc[g * cs + t] = exp_cr(__fsub_rn(sc[g * cs + t], red[g]));
    }
    __syncthreads();
    for (size_t g = warp; g < group; g += nwarp) {
      if (lane == 0) {
        float sum = 0.0f;
        const float* e = sc + g * cs;
        for (int t = 0; t < T; t++) sum = __fadd_rn(sum, e[t]);
        red[g] = sum;
      }
    }
    __syncthreads();
    for (unsigned i = tid; i < grp * (unsigned)n_t; i += blockDim.x) {
      const unsigned g = i / (unsigned)n_t, tl = i - g * (unsigned)n_t;
      float pv = sc[g * cs + t0 + tl];
      if (red[g] > 0.0f) pv = __fdiv_rn(pv, red[g]);
      p16[g * chunk + tl] = f32_to_f16_bits(pv);
    }
  }
  cp_async_wait<0>();
  __syncthreads();

  // partial[g][d] = sum_f64 over this CTA's steps of v[t][d] * p[g][t]  -> rank 0
  double* part0 = cluster.map_shared_rank(part, 0);
  for (unsigned o = tid; o < grp * hdu; o += blockDim.x) {
    const unsigned g = o / hdu, d = o - g * hdu;
    const uint16_t* vc = reinterpret_cast<const uint16_t*>(vbuf) + d;
    const uint16_t* pr = p16 + g * chunk;
    double s = 0.0;
    for (int tl = 0; tl < n_t; tl++)
      s += (double)__fmul_rn(f16_bits_to_f32(vc[(size_t)tl * hd]), f16_bits_to_f32(pr[tl]));
    part0[(size_t)rank * group * hd + o] = s;
  }
  cluster.sync();
  if (rank != 0) return;

  for (size_t o = tid; o < group * hd; o += blockDim.x) {
    double s = 0.0;
    for (unsigned rr = 0; rr < CL; rr++) s += part[(size_t)rr * group * hd + o];
    outv[o] = (float)s;
  }
  __syncthreads();
  // write f32 (debug) and Q8_0 blocks of this kv head's group*hd outputs
  const size_t out0 = kvh * group * hd;  // heads kvh*group .. are contiguous in attn_out
  for (size_t blk = warp; blk < group * hd / 32; blk += nwarp) {
    const float v = outv[blk * 32 + lane];
    if (attn_out) attn_out[b * nq + out0 + blk * 32 + lane] = v;
    float a = fabsf(v);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, o));
    float d, inv;
    q8_scale_pair<SEM>(a, &d, &inv);
    q8[b * nq + out0 + blk * 32 + lane] = (uint8_t)(int8_t)q8_quant_value<SEM>(v, inv);
    if (lane == 0) scales[b * (nq / 32) + (out0 / 32) + blk] = f16_round_trip(d);
  }
}

// The CLI forward's attention (src/app/text.rs:414-453) for one (sequence, head) per CTA: f32 query against the
// f16 keys in the lane order of the selected instruction set (dot.rs:79-97, :241-276), an online soft-max whose
// running maximum starts at 0, vec_mad_f16_f32 / vec_scale_f32 on the output row.  The recurrence over the
// cached positions is evaluated exactly but in three parallel steps:
//   scores (all t in parallel)  ->  running maximum, rescale factors exp(ms_{t-1} - s_t) (1 where the maximum
//   does not move: multiplying by 1 is the identity) and weights exp(s_t - ms_t)  ->  per output element the
//   sequential chain over t (out = out * r_t; out = fma(w_t, v_t, out)), 128 chains side by side.
// Attention for one (sequence, kv head) by a single CTA: the variant for large batches, where there are enough
// (sequence, kv head) pairs to fill the GPU and a cluster per pair only adds synchronisation.  Same arithmetic as
// attention_kernel (sequential f64 dots of f16 values, soft-max with the sequential f32 sum, f16 probabilities,
// sequential f64 P.V); K and V stream through two shared-memory tiles of SEQ_TILE positions.
constexpr int SEQ_TILE = 128;

// GS: the score and probability rows ([group][capacity] f32 and f16) live in a global scratch area instead of shared
// memory (g_sc / g_p16, one slice per CTA), for capacities whose rows do not fit: only this CTA touches its slice and
// the phases are separated by CTA barriers, so the arithmetic and its order are unchanged.
// G > 0: the group has exactly G query heads of 128 elements.  Every cached value is then converted once for all
// heads of the group, by SEQ_THREADS_G threads: a thread of the score pass takes one position and one of QS slices of
// the head dimension for the G heads (G independent chains), a thread of the P.V pass takes two adjacent output
// columns and one of PS slices of each tile's positions for the G heads (2 G chains).  The f64 partial sums are added
// in ascending slice order: like the tree sums of the other f64 accumulations, exact whenever no f64 rounding occurs,
// which the products of two f16 values make the overwhelmingly common case.  G == 0: any group and head size.
constexpr int SEQ_THREADS_G = 512;
template <int SEM, bool GS, int G>
__global__ void __launch_bounds__(G > 0 ? SEQ_THREADS_G : 256)
    attention_seq_kernel(const uint16_t* __restrict__ q16, const uint16_t* __restrict__ k_cache,
                         const uint16_t* __restrict__ v_cache, const int* __restrict__ d_step, size_t n_head,
                         size_t n_head_kv, size_t hd, size_t layer, size_t n_layer, size_t capacity,
                         float* __restrict__ attn_out, uint8_t* __restrict__ q8, float* __restrict__ scales,
                         float* __restrict__ g_sc, double* __restrict__ g_pd) {
  extern __shared__ __align__(16) uint8_t smem[];
  pdl_wait();
  pdl_launch_dependents();
  const size_t kvh = blockIdx.x, b = blockIdx.y;
  const size_t group = n_head / n_head_kv, nq = n_head * hd, nk = n_head_kv * hd;
  const int T = *d_step + 1;
  const size_t cs = (capacity + 7) & ~(size_t)7;  // keeps every array 16-byte aligned
  const size_t slice = (b * n_head_kv + kvh) * group * cs;         // GS: this CTA's rows in the scratch area
  // f64 copies of the query rows and of the f16 probabilities: a product of two f16 values is exact in f32 and in
  // f64, so s + f64(f32(q) * f32(k)) (dot.rs:115-118) equals fma(f64(q), f64(k), s) bit for bit
  double* qd = reinterpret_cast<double*>(smem);                     // [group][hd]
  double* pd = GS ? g_pd + slice : qd + group * hd;                 // [group][cs]
  float* sc = GS ? g_sc + slice : reinterpret_cast<float*>(pd + group * cs);   // [group][cs]
  float* red = GS ? reinterpret_cast<float*>(qd + group * hd) : sc + group * cs;  // [group] (padded to 4)
  uint8_t* tiles = reinterpret_cast<uint8_t*>(red + ((group + 3) & ~(size_t)3));  // 2 x SEQ_TILE rows (16-byte aligned)
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nwarp = blockDim.x >> 5;
  const unsigned grp = (unsigned)group;
  constexpr int HD = 128;  // head size of the G > 0 variants
  constexpr int QS = SEQ_THREADS_G / SEQ_TILE, PS = SEQ_THREADS_G / (HD / 2);  // slices of the two passes
  constexpr int GA = G > 0 ? G : 1;
  // K rows are padded by 16 bytes: the threads of a warp read the same words of different rows, and rows of exactly
  // hd * 2 = 256 bytes would all start in the same bank
  const size_t row_bytes = hd * 2, k_stride = row_bytes + 16, tile_bytes = SEQ_TILE * k_stride, row16 = hd / 8;
  const int n_tiles = (T + SEQ_TILE - 1) / SEQ_TILE;
  const float kq_scale = __fdiv_rn(1.0f, __fsqrt_rn((float)hd));
  const uint16_t* kbase = k_cache + ((b * n_layer + layer) * capacity) * nk + kvh * hd;
  const uint16_t* vbase = v_cache + ((b * n_layer + layer) * capacity) * nk + kvh * hd;
  const row_copy_plan plan = make_row_copy_plan((unsigned)row16);
  auto stage = [&](const uint16_t* base, int tile, int buf, size_t stride) {
    const int t0 = tile * SEQ_TILE, nt = min(SEQ_TILE, T - t0);
    cp_async_rows(plan, tiles + (size_t)buf * tile_bytes, stride, base + (size_t)t0 * nk, nk * 2, (unsigned)nt);
    cp_async_commit();
  };
  for (size_t i = tid; i < group * hd; i += blockDim.x)
    qd[i] = (double)f16_bits_to_f32(q16[b * nq + kvh * group * hd + i]);
  stage(kbase, 0, 0, k_stride);
  // scores[g][t] = f32(sum_f64 q*k) * kq_scale (dot.rs:115-118)
  // One barrier per tile: after it the tile's rows are visible and every thread is done with the previous tile, so
  // the other tile buffer may be refilled and (G > 0) the previous tile's partial sums may be folded.
  double* qk_parts = reinterpret_cast<double*>(tiles + 2 * tile_bytes);  // G > 0: [2][QS][G][SEQ_TILE]
  auto fold_scores = [&](int tile) {
    const double* part = qk_parts + (size_t)(tile & 1) * (QS * GA * SEQ_TILE);
    const int t0 = tile * SEQ_TILE, nt = min(SEQ_TILE, T - t0);
    for (int item = tid; item < GA * SEQ_TILE; item += blockDim.x) {
      const int g = item >> 7, t = item & (SEQ_TILE - 1);
      if (t < nt) {
        double s = part[g * SEQ_TILE + t];
#pragma unroll
        for (int h = 1; h < QS; h++) s += part[(h * GA + g) * SEQ_TILE + t];
        sc[g * cs + t0 + t] = __fmul_rn((float)s, kq_scale);
      }
    }
  };
  for (int tile = 0; tile < n_tiles; tile++) {
    cp_async_wait<0>();
    __syncthreads();
    if (tile + 1 < n_tiles) stage(kbase, tile + 1, (tile + 1) & 1, k_stride);
    const uint8_t* kt = tiles + (size_t)(tile & 1) * tile_bytes;
    const int t0 = tile * SEQ_TILE, nt = min(SEQ_TILE, T - t0);
    if constexpr (G > 0) {
      if (tile > 0) fold_scores(tile - 1);
      double* qk_part = qk_parts + (size_t)(tile & 1) * (QS * G * SEQ_TILE);
      const int tl = tid & (SEQ_TILE - 1), h = tid >> 7;                    // four warps per slice
      if (tl < nt) {
        const uint4* kr = reinterpret_cast<const uint4*>(kt + tl * k_stride) + h * (HD / QS / 8);
        const double2* qr = reinterpret_cast<const double2*>(qd + h * (HD / QS));
        double s[G];
#pragma unroll
        for (int g = 0; g < G; g++) s[g] = 0.0;
#pragma unroll 2
        for (int i = 0; i < HD / QS / 8; i++) {
          const uint4 kv = kr[i];
          const uint32_t kw[4] = {kv.x, kv.y, kv.z, kv.w};
#pragma unroll
          for (int e = 0; e < 4; e++) {
            const double k0 = (double)f16_bits_to_f32((uint16_t)(kw[e] & 0xffff));
            const double k1 = (double)f16_bits_to_f32((uint16_t)(kw[e] >> 16));
#pragma unroll
            for (int g = 0; g < G; g++) {
              const double2 q2 = qr[g * (HD / 2) + i * 4 + e];
              s[g] = fma(q2.x, k0, s[g]);
              s[g] = fma(q2.y, k1, s[g]);
            }
          }
        }
#pragma unroll
        for (int g = 0; g < G; g++) qk_part[(h * G + g) * SEQ_TILE + tl] = s[g];
      }
    } else {
      for (unsigned item = tid; item < (unsigned)nt * grp; item += blockDim.x) {
        const unsigned tl = item / grp, g = item - tl * grp;
        const uint4* kr = reinterpret_cast<const uint4*>(kt + tl * k_stride);
        const double2* qr = reinterpret_cast<const double2*>(qd + g * hd);
        double s = 0.0;
        for (size_t i = 0; i < hd / 8; i++) {
          const uint4 kv = kr[i];
          const uint32_t kw[4] = {kv.x, kv.y, kv.z, kv.w};
#pragma unroll
          for (int e = 0; e < 4; e++) {
            const double2 q2 = qr[i * 4 + e];
            s = fma(q2.x, (double)f16_bits_to_f32((uint16_t)(kw[e] & 0xffff)), s);
            s = fma(q2.y, (double)f16_bits_to_f32((uint16_t)(kw[e] >> 16)), s);
          }
        }
        sc[g * cs + t0 + tl] = __fmul_rn((float)s, kq_scale);
      }
    }
  }
  __syncthreads();
  stage(vbase, 0, 0, row_bytes);  // the first V tile travels while the soft-max is evaluated
  // max, exp, sequential f32 sum (attention.rs:28-38), divide, f16
  if constexpr (G > 0) {
    fold_scores(n_tiles - 1);
    __syncthreads();
    // every warp finds the G maxima itself (a maximum does not depend on the order): no hand-over through shared memory
    float mx[G];
#pragma unroll
    for (int g = 0; g < G; g++) {
      float m = -INFINITY;
      for (int t = lane; t < T; t += 32) m = fmaxf(m, sc[g * cs + t]);
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
      mx[g] = m;
    }
    __syncthreads();  // all maxima taken before any score is overwritten
#pragma unroll
    for (int g = 0; g < G; g++)
      for (int t = tid; t < T; t += blockDim.x) sc[g * cs + t] = exp_cr(__fsub_rn(sc[g * cs + t], mx[g]));
  } else {
    for (size_t g = warp; g < group; g += nwarp) {
      float mx = -INFINITY;
      for (int t = lane; t < T; t += 32) mx = fmaxf(mx, sc[g * cs + t]);
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
      if (lane == 0) red[g] = mx;
    }
    __syncthreads();
    for (unsigned i = tid; i < grp * (unsigned)T; i += blockDim.x) {
      const unsigned g = i / (unsigned)T, t = i - g * (unsigned)T;
      sc[g * cs + t] = exp_cr(__fsub_rn(sc[g * cs + t], red[g]));
    }
  }
  __syncthreads();
  for (size_t g = warp; g < group; g += nwarp) {
    if (lane == 0) {
      float sum = 0.0f;
      const float* e = sc + g * cs;
      for (int t = 0; t < T; t++) sum = __fadd_rn(sum, e[t]);
      red[g] = sum;
    }
  }
  __syncthreads();
  for (unsigned i = tid; i < grp * (unsigned)T; i += blockDim.x) {
    const unsigned g = i / (unsigned)T, t = i - g * (unsigned)T;
    float pv = sc[g * cs + t];
    if (red[g] > 0.0f) pv = __fdiv_rn(pv, red[g]);
    pd[g * cs + t] = (double)f16_round_trip(pv);
  }
  // out[g][d] = f32(sum_f64 over t of v[t][d] * p[g][t]), one output element per thread and pass
  double accv[2] = {0.0, 0.0};
  size_t pv_row[2], pv_col[2];  // probability row start and V column of this thread's two outputs
#pragma unroll
  for (int pass = 0; pass < 2; pass++) {
    const unsigned o = tid + pass * blockDim.x, g = o / (unsigned)hd;
    pv_row[pass] = g * cs;
    pv_col[pass] = o - g * (unsigned)hd;
  }
  double acc2[GA][2];  // G > 0: columns 2 * pair and 2 * pair + 1 of the G heads over this thread's slice of the positions
#pragma unroll
  for (int g = 0; g < GA; g++) acc2[g][0] = acc2[g][1] = 0.0;
  for (int tile = 0; tile < n_tiles; tile++) {
    cp_async_wait<0>();
    __syncthreads();  // the tile (and, first time, the probabilities) visible; everyone is done with the previous tile
    if (tile + 1 < n_tiles) stage(vbase, tile + 1, (tile + 1) & 1, row_bytes);
    const uint16_t* vt = reinterpret_cast<const uint16_t*>(tiles + (size_t)(tile & 1) * tile_bytes);
    const int t0 = tile * SEQ_TILE, nt = min(SEQ_TILE, T - t0);
    if constexpr (G > 0) {
      const int pair = tid & 63, slice = tid >> 6;
      const uint32_t* vw = reinterpret_cast<const uint32_t*>(vt) + pair;
      const double* pr = pd + t0;
      const int t_end = min(nt, slice * (SEQ_TILE / PS) + SEQ_TILE / PS);
#pragma unroll 4
      for (int tl = slice * (SEQ_TILE / PS); tl < t_end; tl++) {
        const uint32_t w = vw[tl * (HD / 2)];
        const double v0 = (double)f16_bits_to_f32((uint16_t)(w & 0xffff)), v1 = (double)f16_bits_to_f32((uint16_t)(w >> 16));
#pragma unroll
        for (int g = 0; g < G; g++) {
          const double pg = pr[g * cs + tl];
          acc2[g][0] = fma(v0, pg, acc2[g][0]);
          acc2[g][1] = fma(v1, pg, acc2[g][1]);
        }
      }
    } else {
#pragma unroll
      for (int pass = 0; pass < 2; pass++) {
        if (tid + pass * blockDim.x >= group * hd) break;
        const double* pr = pd + pv_row[pass] + t0;
        const uint16_t* vc = vt + pv_col[pass];
        double s = accv[pass];
        for (int tl = 0; tl < nt; tl++) s = fma((double)f16_bits_to_f32(vc[(size_t)tl * hd]), pr[tl], s);
        accv[pass] = s;
      }
    }
  }
  if constexpr (G > 0) {  // the PS slices of every output, added in order (the tiles are free by now)
    double* pv_part = reinterpret_cast<double*>(tiles);  // [PS][G * HD]
    const int pair = tid & 63, slice = tid >> 6;
    __syncthreads();  // every thread is done with the last tile
#pragma unroll
    for (int g = 0; g < G; g++) {
      pv_part[slice * (G * HD) + g * HD + 2 * pair] = acc2[g][0];
      pv_part[slice * (G * HD) + g * HD + 2 * pair + 1] = acc2[g][1];
    }
    __syncthreads();
    if (tid < G * HD) {  // G * HD <= SEQ_THREADS_G: one output per thread
      double s = pv_part[tid];
#pragma unroll
      for (int q = 1; q < PS; q++) s += pv_part[q * (G * HD) + tid];
      accv[0] = s;
    }
  }
  // f32 (debug) and Q8_0 blocks of this kv head's group*hd outputs: 32 consecutive outputs per warp and pass
  const size_t out0 = kvh * group * hd;
  int pass = 0;
  for (size_t o = tid; o < group * hd && pass < 2; o += blockDim.x, pass++) {
    const float v = (float)accv[pass];
    if (attn_out) attn_out[b * nq + out0 + o] = v;
    float a = fabsf(v);
#pragma unroll
    for (int sft = 16; sft > 0; sft >>= 1) a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, sft));
    float dsc, inv;
    q8_scale_pair<SEM>(a, &dsc, &inv);
    q8[b * nq + out0 + o] = (uint8_t)(int8_t)q8_quant_value<SEM>(v, inv);
    if (lane == 0) scales[(b * nq + out0 + o) / 32] = f16_round_trip(dsc);
  }
}

constexpr int ATT_TILE = 64;

template <int SEM>
__global__ void __launch_bounds__(256)
    attention_online_kernel(const float* __restrict__ q32, const uint16_t* __restrict__ k_cache,
                            const uint16_t* __restrict__ v_cache, const int* __restrict__ d_step, size_t n_head,
                            size_t n_head_kv, size_t hd, size_t layer, size_t n_layer, size_t capacity,
                            float* __restrict__ attn_out, uint8_t* __restrict__ q8, float* __restrict__ scales) {
  constexpr int LN = SEM == RMI_SEM_AVX2 ? 8 : (SEM == RMI_SEM_NEON ? 4 : 1);
  extern __shared__ __align__(16) uint8_t smem[];
  pdl_wait();
  pdl_launch_dependents();
  const size_t head = blockIdx.x, b = blockIdx.y, kvh = head / (n_head / n_head_kv);
  const size_t nq = n_head * hd, nk = n_head_kv * hd;
  const int T = *d_step + 1;
  float* sc = reinterpret_cast<float*>(smem);  // [capacity] scores, then weights
  const size_t cap4 = (capacity + 3) & ~(size_t)3;
  float* rs = sc + cap4;                       // [capacity] rescale factors
  float* qs = rs + cap4;                       // [hd]
  float* seg = qs + hd;                        // [256] segment maxima
  const int tid = threadIdx.x, lane = tid & 31;
  const uint16_t* kbase = k_cache + ((b * n_layer + layer) * capacity) * nk + kvh * hd;
  const uint16_t* vbase = v_cache + ((b * n_layer + layer) * capacity) * nk + kvh * hd;
  for (size_t i = tid; i < hd; i += blockDim.x) qs[i] = q32[b * nq + head * hd + i];
  __syncthreads();
  const float kq_scale = __fdiv_rn(1.0f, __fsqrt_rn((float)hd));

  // K and V rows are staged through two shared-memory tiles of ATT_TILE positions with cp.async (the next
  // tile is in flight while the current one is used): a chain must not wait on global memory every few steps
  uint8_t* tiles = reinterpret_cast<uint8_t*>(seg + 256);
  const size_t row_bytes = hd * 2, tile_bytes = ATT_TILE * row_bytes, row16 = hd / 8;
  const int n_tiles = (T + ATT_TILE - 1) / ATT_TILE;
  const row_copy_plan plan = make_row_copy_plan((unsigned)row16);
  auto stage = [&](const uint16_t* base, int tile, int buf) {
    const int t0 = tile * ATT_TILE, nt = min(ATT_TILE, T - t0);
    cp_async_rows(plan, tiles + (size_t)buf * tile_bytes, row_bytes, base + (size_t)t0 * nk, nk * 2, (unsigned)nt);
    cp_async_commit();
  };

  // scores: a group of LN threads per position, thread l takes elements l, l + LN, ... (one SIMD lane)
  {
    const int l = tid % LN, grp = tid / LN, n_grp = 256 / LN;
    stage(kbase, 0, 0);
    for (int tile = 0; tile < n_tiles; tile++) {
      if (tile + 1 < n_tiles) stage(kbase, tile + 1, (tile + 1) & 1);
      if (tile + 1 < n_tiles) cp_async_wait<1>(); else cp_async_wait<0>();
      __syncthreads();
      const uint8_t* kt = tiles + (size_t)(tile & 1) * tile_bytes;
      const int t0 = tile * ATT_TILE, nt = min(ATT_TILE, T - t0);
      for (int tl = grp; tl < ((nt + n_grp - 1) / n_grp) * n_grp; tl += n_grp) {  // whole warps stay converged for the shuffles
        float acc = 0.0f;
        if (tl < nt) {
          const uint16_t* kr = reinterpret_cast<const uint16_t*>(kt + (size_t)tl * row_bytes);
          for (size_t i = l; i < hd; i += LN) {
            const float kv = f16_bits_to_f32(kr[i]);
            acc = SEM == RMI_SEM_SCALAR ? __fadd_rn(acc, __fmul_rn(qs[i], kv)) : __fmaf_rn(qs[i], kv, acc);
          }
        }
        if (SEM == RMI_SEM_AVX2) {  // hsum_ps (dot.rs:447-456)
          acc = __fadd_rn(__shfl_xor_sync(0xffffffffu, acc, 4), acc);
          acc = __fadd_rn(acc, __shfl_xor_sync(0xffffffffu, acc, 1));
          acc = __fadd_rn(acc, __shfl_xor_sync(0xffffffffu, acc, 2));
        } else if (SEM == RMI_SEM_NEON) {  // vaddvq_f32
          acc = __fadd_rn(acc, __shfl_xor_sync(0xffffffffu, acc, 1));
          acc = __fadd_rn(acc, __shfl_xor_sync(0xffffffffu, acc, 2));
        }
        if (l == 0 && tl < nt) sc[t0 + tl] = __fmul_rn(acc, kq_scale);
      }
      __syncthreads();  // the tile may be overwritten by the copy issued in the next iteration
    }
  }

  // running maximum (starts at 0): thread i owns the positions [i*S, (i+1)*S)
  const int S = (T + 255) / 256;
  const int t_lo = tid * S, t_hi = min(T, t_lo + S);
  float mx = 0.0f;
  for (int t = t_lo; t < t_hi; t++) mx = fmaxf(mx, sc[t]);
  seg[tid] = mx;
  __syncthreads();
  float ms = 0.0f;  // maximum over all earlier segments
  for (int i = 0; i < tid; i++) ms = fmaxf(ms, seg[i]);
  for (int t = t_lo; t < t_hi; t++) {
    const float s = sc[t];
    float r = 1.0f;
    if (s > ms) {
      r = exp_cr(__fsub_rn(ms, s));
      ms = s;
    }
    rs[t] = r;
    sc[t] = exp_cr(__fsub_rn(s, ms));
  }
  __syncthreads();

  // the chains over t, one per output element; every thread also carries s_sum
  float out = 0.0f, s_sum = 0.0f;
  stage(vbase, 0, 0);
  for (int tile = 0; tile < n_tiles; tile++) {
    if (tile + 1 < n_tiles) stage(vbase, tile + 1, (tile + 1) & 1);
    if (tile + 1 < n_tiles) cp_async_wait<1>(); else cp_async_wait<0>();
    __syncthreads();
    if ((size_t)tid < hd) {
      const uint16_t* vt = reinterpret_cast<const uint16_t*>(tiles + (size_t)(tile & 1) * tile_bytes) + tid;
      const int t0 = tile * ATT_TILE, nt = min(ATT_TILE, T - t0);
      for (int tl = 0; tl < nt; tl++) {
        const float r = rs[t0 + tl], wgt = sc[t0 + tl], vf = f16_bits_to_f32(vt[(size_t)tl * hd]);
        out = __fmul_rn(out, r);
        s_sum = __fmul_rn(s_sum, r);
        out = SEM == RMI_SEM_SCALAR ? __fadd_rn(out, __fmul_rn(wgt, vf)) : __fmaf_rn(wgt, vf, out);
        s_sum = __fadd_rn(s_sum, wgt);
      }
    }
    __syncthreads();
  }
  if ((size_t)tid < hd) {
    out = __fmul_rn(out, __fdiv_rn(1.0f, s_sum));
    // this head's output, f32 (debug) and Q8_0 (one block per warp) for the Wo projection
    const size_t o = b * nq + head * hd + tid;
    if (attn_out) attn_out[o] = out;
    float a = fabsf(out);
#pragma unroll
    for (int sft = 16; sft > 0; sft >>= 1) a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, sft));
    float dsc, inv;
    q8_scale_pair<SEM>(a, &dsc, &inv);
    q8[o] = (uint8_t)(int8_t)q8_quant_value<SEM>(out, inv);
    if (lane == 0) scales[o / 32] = f16_round_trip(dsc);
  }
}

// Score-buffer attention of the CLI forwards, one CTA per (head, sequence), over an F32 or an F16 cache:
//   * `--kv-cache f32` of the text loop (src/app/text.rs:458-496; KV16 = false, SEQ_PV = false): scores =
//     dot_f32(q, k_t) * scale in the lane order of the selected instruction set (src/ops/dot.rs:8-76: eight AVX2
//     lanes; four NEON accumulators of four lanes, combined (acc0+acc2)+(acc1+acc3) then pairwise; one scalar chain
//     with separate multiply and add), the soft-max of src/ops/attention.rs:28-38 (the -inf padding to a multiple
//     of 256 adds exact zeros), then out[d] = dot_f32(V[:, d], weights) in the same lane order over the positions:
//     chain l of element d takes the positions l, l + LN, ...; the chains of one element are combined through
//     shared memory.  Padded positions multiply a zero by a zero weight and leave every chain unchanged.
//   * the logits tool (src/app/logits.rs:474-560; SEQ_PV = true): scores by dot_f16_f32 over the F16 cache
//     (KV16 = true: eight AVX2 lanes, four NEON lanes, src/ops/dot.rs:79-97, :241-276) or dot_f32 over the F32
//     cache, the same soft-max, then one sequential chain per output element, val += p_t * v_t with separate
//     multiply and add in every instruction set.
template <bool KV16>
struct kv_elem { using type = float; };
template <>
struct kv_elem<true> { using type = uint16_t; };
__device__ __forceinline__ float kv_val(const float* p) { return *p; }
__device__ __forceinline__ float kv_val(const uint16_t* p) { return f16_bits_to_f32(*p); }

// K and V pass through two shared-memory tiles of SM_TILE positions (cp.async, the next tile in flight while the
// current one is used; rows padded by 16 bytes against bank conflicts): a chain must not wait on global memory.
constexpr int SM_TILE = 64;

template <int SEM, bool KV16, bool SEQ_PV>
__global__ void __launch_bounds__(256)
    attention_softmax_kernel(const float* __restrict__ q32, const typename kv_elem<KV16>::type* __restrict__ k_cache,
                             const typename kv_elem<KV16>::type* __restrict__ v_cache, const int* __restrict__ d_step,
                             size_t n_head, size_t n_head_kv, size_t hd, size_t layer, size_t n_layer, size_t capacity,
                             float* __restrict__ attn_out, uint8_t* __restrict__ q8, float* __restrict__ scales) {
  using kv_t = typename kv_elem<KV16>::type;
  constexpr int LN = SEM == RMI_SEM_AVX2 ? 8 : (SEM == RMI_SEM_NEON ? (KV16 ? 4 : 16) : 1);  // score lanes
  constexpr int LP = SEQ_PV ? 1 : LN;                                                        // chains per element
  constexpr bool PV_FMA = !SEQ_PV && SEM != RMI_SEM_SCALAR;
  constexpr int MAX_ITEMS = LP;  // LP * hd / 256 chains per thread with hd <= 256
  extern __shared__ __align__(16) uint8_t smem[];
  pdl_wait();
  pdl_launch_dependents();
  const size_t head = blockIdx.x, b = blockIdx.y, kvh = head / (n_head / n_head_kv);
  const size_t nq = n_head * hd, nk = n_head_kv * hd;
  const int T = *d_step + 1;
  const size_t cap4 = (capacity + 3) & ~(size_t)3;
  float* sc = reinterpret_cast<float*>(smem);  // [capacity] scores, then weights
  float* qs = sc + cap4;                       // [hd]
  float* part = qs + hd;                       // [16][hd] chain results
  float* red = part + 16 * hd;                 // [32]
  uint8_t* tiles = reinterpret_cast<uint8_t*>(red + 32);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const kv_t* kbase = k_cache + ((b * n_layer + layer) * capacity) * nk + kvh * hd;
  const kv_t* vbase = v_cache + ((b * n_layer + layer) * capacity) * nk + kvh * hd;
  for (size_t i = tid; i < hd; i += blockDim.x) qs[i] = q32[b * nq + head * hd + i];
  const float kq_scale = __fdiv_rn(1.0f, __fsqrt_rn((float)hd));

  const size_t row_bytes = hd * sizeof(kv_t), row_stride = row_bytes + 16, tile_bytes = SM_TILE * row_stride;
  const size_t row16 = row_bytes / 16;
  const int n_tiles = (T + SM_TILE - 1) / SM_TILE;
  const row_copy_plan plan = make_row_copy_plan((unsigned)row16);
  auto stage = [&](const kv_t* base, int tile, int buf) {
    const int t0 = tile * SM_TILE, nt = min(SM_TILE, T - t0);
    cp_async_rows(plan, tiles + (size_t)buf * tile_bytes, row_stride, base + (size_t)t0 * nk, nk * sizeof(kv_t),
                  (unsigned)nt);
    cp_async_commit();
  };

  {  // scores: LN threads per position, thread l takes elements l, l + LN, ... (one SIMD lane)
    const int l = tid % LN, grp = tid / LN, n_grp = 256 / LN;
    stage(kbase, 0, 0);
    for (int tile = 0; tile < n_tiles; tile++) {
      if (tile + 1 < n_tiles) stage(kbase, tile + 1, (tile + 1) & 1);
      if (tile + 1 < n_tiles) cp_async_wait<1>(); else cp_async_wait<0>();
      __syncthreads();  // also orders the staging of qs before its first use
      const uint8_t* kt = tiles + (size_t)(tile & 1) * tile_bytes;
      const int t0 = tile * SM_TILE, nt = min(SM_TILE, T - t0);
      for (int tl = grp; tl < ((nt + n_grp - 1) / n_grp) * n_grp; tl += n_grp) {  // whole warps stay converged
        float acc = 0.0f;
        if (tl < nt) {
          const kv_t* kr = reinterpret_cast<const kv_t*>(kt + (size_t)tl * row_stride);
          for (size_t i = l; i < hd; i += LN) {
            const float kv = kv_val(kr + i);
            acc = SEM == RMI_SEM_SCALAR ? __fadd_rn(acc, __fmul_rn(qs[i], kv)) : __fmaf_rn(qs[i], kv, acc);
          }
        }
        if (SEM == RMI_SEM_AVX2) {  // hsum_ps
          acc = __fadd_rn(__shfl_xor_sync(0xffffffffu, acc, 4), acc);
          acc = __fadd_rn(acc, __shfl_xor_sync(0xffffffffu, acc, 1));
          acc = __fadd_rn(acc, __shfl_xor_sync(0xffffffffu, acc, 2));
        } else if (SEM == RMI_SEM_NEON) {
          if (!KV16) {  // (acc0 + acc2) + (acc1 + acc3)
            acc = __fadd_rn(acc, __shfl_xor_sync(0xffffffffu, acc, 8));
            acc = __fadd_rn(acc, __shfl_xor_sync(0xffffffffu, acc, 4));
          }
          acc = __fadd_rn(acc, __shfl_xor_sync(0xffffffffu, acc, 1));  // vaddvq_f32
          acc = __fadd_rn(acc, __shfl_xor_sync(0xffffffffu, acc, 2));
        }
        if (l == 0 && tl < nt) sc[t0 + tl] = __fmul_rn(acc, kq_scale);
      }
      __syncthreads();  // the tile may be overwritten by the copy issued in the next iteration
    }
  }
  stage(vbase, 0, 0);  // the first V tile arrives during the soft-max

  // soft-max: maximum, exp, sequential f32 sum, divide
  float mx = -INFINITY;
  for (int t = tid; t < T; t += 256) mx = fmaxf(mx, sc[t]);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  if (lane == 0) red[warp] = mx;
  __syncthreads();
  mx = red[0];
  for (int w = 1; w < 8; w++) mx = fmaxf(mx, red[w]);
  __syncthreads();
  for (int t = tid; t < T; t += 256) sc[t] = exp_cr(__fsub_rn(sc[t], mx));
  __syncthreads();
  if (tid == 0) {
    float sum = 0.0f;
    for (int t = 0; t < T; t++) sum = __fadd_rn(sum, sc[t]);
    red[16] = sum;
  }
  __syncthreads();
  const float sum = red[16];
  if (sum > 0.0f)
    for (int t = tid; t < T; t += 256) sc[t] = __fdiv_rn(sc[t], sum);

  // chains: item = l * hd + d (a warp reads 32 consecutive elements of one V row); chain l of element d takes the
  // positions l, l + LP, ...; SM_TILE is a multiple of LP, so inside every tile chain l starts at local position l
  float acc[MAX_ITEMS];
#pragma unroll
  for (int it = 0; it < MAX_ITEMS; it++) acc[it] = 0.0f;
  for (int tile = 0; tile < n_tiles; tile++) {
    if (tile + 1 < n_tiles) stage(vbase, tile + 1, (tile + 1) & 1);
    if (tile + 1 < n_tiles) cp_async_wait<1>(); else cp_async_wait<0>();
    __syncthreads();  // also orders the weights written above before their first use
    const uint8_t* vt = tiles + (size_t)(tile & 1) * tile_bytes;
    const int t0 = tile * SM_TILE, nt = min(SM_TILE, T - t0);
#pragma unroll
    for (int it = 0; it < MAX_ITEMS; it++) {
      const size_t item = (size_t)tid + 256 * (size_t)it;
      if (item < (size_t)LP * hd) {
        const int l = (int)(item / hd);
        const kv_t* vc = reinterpret_cast<const kv_t*>(vt) + item % hd;
        float a = acc[it];
        for (int tl = l; tl < nt; tl += LP) {
          const float vv = kv_val(reinterpret_cast<const kv_t*>(reinterpret_cast<const uint8_t*>(vc) + (size_t)tl * row_stride));
          const float wgt = sc[t0 + tl];
          a = PV_FMA ? __fmaf_rn(vv, wgt, a) : __fadd_rn(a, __fmul_rn(vv, wgt));
        }
        acc[it] = a;
      }
    }
    __syncthreads();
  }
#pragma unroll
  for (int it = 0; it < MAX_ITEMS; it++) {
    const size_t item = (size_t)tid + 256 * (size_t)it;
    if (item < (size_t)LP * hd) part[item] = acc[it];
  }
  __syncthreads();
  if ((size_t)tid < hd) {
    float out;
    const float* p = part + tid;
    if (LP == 8) {
      const float s0 = __fadd_rn(p[4 * hd], p[0]), s1 = __fadd_rn(p[5 * hd], p[hd]);
      const float s2 = __fadd_rn(p[6 * hd], p[2 * hd]), s3 = __fadd_rn(p[7 * hd], p[3 * hd]);
      out = __fadd_rn(__fadd_rn(s0, s1), __fadd_rn(s2, s3));
    } else if (LP == 16) {
      float c[4];
#pragma unroll
      for (int i = 0; i < 4; i++)
        c[i] = __fadd_rn(__fadd_rn(p[(size_t)i * hd], p[(size_t)(8 + i) * hd]),
                         __fadd_rn(p[(size_t)(4 + i) * hd], p[(size_t)(12 + i) * hd]));
      out = __fadd_rn(__fadd_rn(c[0], c[1]), __fadd_rn(c[2], c[3]));
    } else {
      out = p[0];
    }
    const size_t o = b * nq + head * hd + tid;
    if (attn_out) attn_out[o] = out;
    float a = fabsf(out);
#pragma unroll
    for (int sft = 16; sft > 0; sft >>= 1) a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, sft));
    float dsc, inv;
    q8_scale_pair<SEM>(a, &dsc, &inv);
    q8[o] = (uint8_t)(int8_t)q8_quant_value<SEM>(out, inv);
    if (lane == 0) scales[o / 32] = f16_round_trip(dsc);
  }
}

// Greedy token in two stages: ARGMAX_SLICES CTAs per sequence each reduce a slice of the logits to
// (value, first index), then one CTA per sequence combines the slices.  Larger value wins, equal
// values keep the lower index (first maximum); a non-finite logit raises *flag.
constexpr int ARGMAX_SLICES = 64;

// LAST = false: equal values keep the lower index (Qwen3Session, qwen3.rs:172-191); LAST = true: the higher
// index (Iterator::max_by in the CLI forward, src/app/text.rs:664-670).  0xffffffff marks "no candidate yet".
template <bool LAST>
__device__ __forceinline__ void argmax_combine(float& best, uint32_t& bi, float ov, uint32_t oi) {
  if (oi == 0xffffffffu) return;
  const bool tie_wins = LAST ? oi > bi : oi < bi;
  if (bi == 0xffffffffu || ov > best || (ov == best && tie_wins)) {
    best = ov;
    bi = oi;
  }
}

template <bool LAST>
__device__ __forceinline__ void argmax_block_reduce(float& best, uint32_t& bi, float* s_v, uint32_t* s_i) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const uint32_t oi = __shfl_xor_sync(0xffffffffu, bi, o);
    argmax_combine<LAST>(best, bi, ov, oi);
  }
  if (lane == 0) {
    s_v[warp] = best;
    s_i[warp] = bi;
  }
  __syncthreads();
  if (threadIdx.x == 0)
    for (int w = 1; w < (int)(blockDim.x >> 5); w++) argmax_combine<LAST>(best, bi, s_v[w], s_i[w]);
}

template <bool LAST>
__global__ void argmax_partial_kernel(const float* __restrict__ logits, size_t vocab, float* __restrict__ part_v,
                                      uint32_t* __restrict__ part_i, int* __restrict__ flag) {
  __shared__ float s_v[32];
  __shared__ uint32_t s_i[32];
  pdl_wait();
  pdl_launch_dependents();
  const size_t b = blockIdx.y, slice = blockIdx.x;
  const size_t per = (vocab + ARGMAX_SLICES - 1) / ARGMAX_SLICES;
  const size_t lo = slice * per, hi = lo + per < vocab ? lo + per : vocab;
  const float* l = logits + b * vocab;
  float best = -INFINITY;
  uint32_t bi = 0xffffffffu;
  bool bad = false;
  for (size_t i = lo + threadIdx.x; i < hi; i += blockDim.x) {
    const float v = l[i];
    if (!isfinite(v)) bad = true;
    argmax_combine<LAST>(best, bi, v, (uint32_t)i);
  }
  if (bad) atomicExch(flag, 1);
  argmax_block_reduce<LAST>(best, bi, s_v, s_i);
  if (threadIdx.x == 0) {
    part_v[b * ARGMAX_SLICES + slice] = best;
    part_i[b * ARGMAX_SLICES + slice] = bi;
  }
}

template <bool LAST>
__global__ void argmax_final_kernel(const float* __restrict__ part_v, const uint32_t* __restrict__ part_i,
                                    const int* __restrict__ d_step, size_t n_prompt, uint32_t* __restrict__ gen,
                                    size_t n_gen) {
  __shared__ float s_v[32];
  __shared__ uint32_t s_i[32];
  pdl_wait();
  pdl_launch_dependents();
  const size_t b = blockIdx.x;
  float best = -INFINITY;
  uint32_t bi = 0xffffffffu;
  if (threadIdx.x < ARGMAX_SLICES) {
    best = part_v[b * ARGMAX_SLICES + threadIdx.x];
    bi = part_i[b * ARGMAX_SLICES + threadIdx.x];
  }
  argmax_block_reduce<LAST>(best, bi, s_v, s_i);
  if (threadIdx.x == 0) {
    const int step = *d_step;
    const size_t gi = (size_t)step + 1 - n_prompt;  // step >= n_prompt-1 when this kernel runs
    if (gi < n_gen) gen[b * n_gen + gi] = bi == 0xffffffffu ? 0u : bi;
  }
}

__global__ void step_inc_kernel(int* d_step) {
  pdl_wait();
  pdl_launch_dependents();
  *d_step += 1;
}

__global__ void unshard_cols_kernel(const float* __restrict__ gathered, size_t g, size_t m, size_t npr,
                                    float* __restrict__ out) {
  const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= g * m * npr) return;
  const size_t c = idx % npr, r = (idx / npr) % m, rank = idx / (npr * m);
  out[r * (g * npr) + rank * npr + c] = gathered[idx];
}

}  // namespace

int32_t launch_unshard_cols(rmi_ctx* ctx, const float* gathered, size_t g, size_t m, size_t npr, float* out) {
  const size_t n = g * m * npr;
  if (n == 0) return RMI_OK;
  unshard_cols_kernel<<<(unsigned)((n + 255) / 256), 256, 0, ctx->stream>>>(gathered, g, m, npr, out);
  return rmi_post_launch(ctx, "unshard_cols");
}

int32_t launch_embed(rmi_ctx* ctx, const rmi_weight* emb, const uint32_t* prompts, size_t n_prompt, const uint32_t* gen,
                     size_t n_gen, const int* d_step, float* x, size_t batch) {
  if (rmi_launch(ctx, embed_kernel, dim3((unsigned)batch), dim3(256), 0, emb->d_tile16, emb->n_in / 32, prompts, n_prompt,
                 gen, n_gen, d_step, x, (uint32_t)emb->n_rows) != cudaSuccess) {
    rmi_set_error("launch of embed failed: %s", cudaGetErrorString(cudaGetLastError()));
    return RMI_ERR_CUDA;
  }
  return rmi_post_launch(ctx, "embed");
}

int32_t launch_rmsnorm_quant(rmi_ctx* ctx, float* x, const float* add, const float* weight, size_t n, float eps,
                             uint8_t* q8, float* scales, size_t batch) {
  auto kern = ctx->sem == RMI_SEM_AVX2 ? rmsnorm_quant_kernel<RMI_SEM_AVX2>
                                       : (ctx->sem == RMI_SEM_NEON ? rmsnorm_quant_kernel<RMI_SEM_NEON>
                                                                   : rmsnorm_quant_kernel<RMI_SEM_SCALAR>);
  if (rmi_launch(ctx, kern, dim3((unsigned)batch), dim3(256), 0, x, add, weight, n, eps, q8, scales) != cudaSuccess) {
    rmi_set_error("launch of rmsnorm_quant failed: %s", cudaGetErrorString(cudaGetLastError()));
    return RMI_ERR_CUDA;
  }
  return rmi_post_launch(ctx, "rmsnorm_quant");
}

int32_t launch_qk_norm_rope_kv(rmi_ctx* ctx, const decode_dims& d, const float* qkv, const float* q_norm,
                               const float* k_norm, const float* rope, const int* d_step, uint16_t* q16,
                               uint16_t* k_cache, uint16_t* v_cache, size_t layer, float* q32, float* k32_cache,
                               float* v32_cache) {
  dim3 grid((unsigned)d.batch, (unsigned)(d.n_head + 2 * d.n_head_kv));
  if (rmi_launch(ctx, qk_norm_rope_kv_kernel, grid, dim3(32), 0, qkv, d.n_head, d.n_head_kv, d.hd, q_norm, k_norm, d.eps,
                 rope, d_step, q16, k_cache, v_cache, layer, d.n_layer, d.capacity, q32, k32_cache, v32_cache) !=
      cudaSuccess) {
    rmi_set_error("launch of qk_norm_rope_kv failed: %s", cudaGetErrorString(cudaGetLastError()));
    return RMI_ERR_CUDA;
  }
  return rmi_post_launch(ctx, "qk_norm_rope_kv");
}

// Cluster size: up to 8 CTAs per (sequence, kv head), at least 16 time steps per CTA.
static unsigned attention_cluster(const decode_dims& d) {
  unsigned cl = 1;
  while (cl < 8 && d.capacity / (cl * 2) >= 16) cl *= 2;
  return cl;
}

size_t attention_smem_bytes(const decode_dims& d) {
  const size_t group = d.n_head / d.n_head_kv, cl = attention_cluster(d);
  const size_t chunk = (d.capacity + cl - 1) / cl;
  size_t b = cl * group * d.hd * 8;                           // partials
  b += (group * ((d.capacity + 3) & ~(size_t)3) + group * d.hd + ((group + 3) & ~(size_t)3)) * 4;  // scores, out, sums
  b += (group * d.hd + ((group * chunk + 7) & ~(size_t)7)) * 2;  // q, p
  b += chunk * (d.hd * 2 + 16) + chunk * d.hd * 2;            // K, V
  return b + 32;
}

int32_t launch_attention(rmi_ctx* ctx, const decode_dims& d, const uint16_t* q16, uint16_t* k_cache,
                         uint16_t* v_cache, const int* d_step, size_t layer, float* attn_out, uint8_t* q8,
                         float* scales, const float* qkv, const float* q_norm, const float* k_norm,
                         const float* rope) {
  RMI_REQUIRE(d.hd % 8 == 0 && (d.n_head / d.n_head_kv) * d.hd % 32 == 0, RMI_ERR_UNSUPPORTED,
              "attention needs head_dim %% 8 == 0 and group*head_dim %% 32 == 0");
  const size_t smem = attention_smem_bytes(d);
  const unsigned cl = attention_cluster(d);
  const size_t chunk = (d.capacity + cl - 1) / cl;
  void (*kern)(const uint16_t*, uint16_t*, uint16_t*, const int*, size_t, size_t, size_t, size_t, size_t,
               size_t, size_t, float*, uint8_t*, float*, const attn_fused_qk) =
      qkv ? (ctx->sem == RMI_SEM_AVX2 ? attention_kernel<RMI_SEM_AVX2, true>
                                      : (ctx->sem == RMI_SEM_NEON ? attention_kernel<RMI_SEM_NEON, true>
                                                                  : attention_kernel<RMI_SEM_SCALAR, true>))
          : (ctx->sem == RMI_SEM_AVX2 ? attention_kernel<RMI_SEM_AVX2, false>
                                      : (ctx->sem == RMI_SEM_NEON ? attention_kernel<RMI_SEM_NEON, false>
                                                                  : attention_kernel<RMI_SEM_SCALAR, false>));
  if (smem > 48 * 1024 && cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) {
    (void)cudaGetLastError();
    rmi_set_error("attention needs %zu B of shared memory", smem);
    return RMI_ERR_UNSUPPORTED;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(d.n_head_kv * cl), (unsigned)d.batch, 1);
  cfg.blockDim = dim3(256, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = ctx->stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = cl;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = ctx->pdl ? 2 : 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, kern, q16, k_cache, v_cache, d_step, d.n_head, d.n_head_kv, d.hd, layer,
                                     d.n_layer, d.capacity, chunk, attn_out, q8, scales,
                                     attn_fused_qk{qkv, q_norm, k_norm, rope, d.eps});
  if (e != cudaSuccess) {
    rmi_set_error("attention launch failed: %s", cudaGetErrorString(e));
    return RMI_ERR_CUDA;
  }
  return rmi_post_launch(ctx, "attention");
}

// One CTA per (kv head, sequence); needs group * head_dim <= 512 (two outputs per thread).
bool attention_seq_shape_ok(const decode_dims& d) {
  const size_t group = d.n_head / d.n_head_kv;
  return group * d.hd <= 512 && (group * d.hd) % 32 == 0 && d.hd % 8 == 0;
}

// ... and preferred over the cluster kernel when there are enough (sequence, kv head) pairs to fill the GPU
bool attention_seq_eligible(const decode_dims& d) { return attention_seq_shape_ok(d) && d.batch * d.n_head_kv >= 64; }

// Shared memory of attention_seq_kernel; global_scores: without the [group][capacity] score and probability rows.
size_t attention_seq_smem_bytes(const decode_dims& d, bool global_scores) {
  const size_t group = d.n_head / d.n_head_kv, cs = (d.capacity + 7) & ~(size_t)7;
  return (global_scores ? 0 : group * cs * 4 + group * cs * 8) + ((group + 3) & ~(size_t)3) * 4 + group * d.hd * 8 +
         2 * (size_t)SEQ_TILE * (d.hd * 2 + 16) + 2 * (SEQ_THREADS_G / SEQ_TILE) * group * SEQ_TILE * 8;  // last: slices of the score dots, two tiles
}

// Bytes of global scratch for the score rows (f32) and the probability rows (f64 copies of the f16 values) of all CTAs.
size_t attention_seq_scratch_bytes(const decode_dims& d) {
  const size_t cs = (d.capacity + 7) & ~(size_t)7;
  return d.batch * d.n_head * cs * 12;
}

using attention_seq_fn = void (*)(const uint16_t*, const uint16_t*, const uint16_t*, const int*, size_t, size_t, size_t,
                                 size_t, size_t, size_t, float*, uint8_t*, float*, float*, double*);
template <int SEM, bool GS>
static attention_seq_fn attention_seq_pick_g(int g) {
  return g == 2 ? attention_seq_kernel<SEM, GS, 2> : (g == 4 ? attention_seq_kernel<SEM, GS, 4> : attention_seq_kernel<SEM, GS, 0>);
}
template <int SEM>
static attention_seq_fn attention_seq_pick_gs(bool gs, int g) {
  return gs ? attention_seq_pick_g<SEM, true>(g) : attention_seq_pick_g<SEM, false>(g);
}
static attention_seq_fn attention_seq_pick(int sem, bool gs, int g) {
  return sem == RMI_SEM_AVX2 ? attention_seq_pick_gs<RMI_SEM_AVX2>(gs, g)
                             : (sem == RMI_SEM_NEON ? attention_seq_pick_gs<RMI_SEM_NEON>(gs, g)
                                                    : attention_seq_pick_gs<RMI_SEM_SCALAR>(gs, g));
}

int32_t launch_attention_seq(rmi_ctx* ctx, const decode_dims& d, const uint16_t* q16, const uint16_t* k_cache,
                             const uint16_t* v_cache, const int* d_step, size_t layer, float* attn_out, uint8_t* q8,
                             float* scales, void* score_scratch) {
  const size_t cs = (d.capacity + 7) & ~(size_t)7;
  const bool gs = score_scratch != nullptr;
  const size_t smem = attention_seq_smem_bytes(d, gs);
  double* g_pd = reinterpret_cast<double*>(score_scratch);   // doubles first: 8-byte alignment
  float* g_sc = gs ? reinterpret_cast<float*>(g_pd + d.batch * d.n_head * cs) : nullptr;
  const size_t group = d.n_head / d.n_head_kv;
  const int gv = d.hd == 128 && (group == 2 || group == 4) ? (int)group : 0;  // conversions shared by the group's heads
  auto kern = attention_seq_pick(ctx->sem, gs, gv);
  if (smem > 48 * 1024 && cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) {
    (void)cudaGetLastError();
    rmi_set_error("attention needs %zu B of shared memory", smem);
    return RMI_ERR_UNSUPPORTED;
  }
  if (rmi_launch(ctx, kern, dim3((unsigned)d.n_head_kv, (unsigned)d.batch), dim3(gv ? SEQ_THREADS_G : 256), smem, q16, k_cache, v_cache, d_step,
                 d.n_head, d.n_head_kv, d.hd, layer, d.n_layer, d.capacity, attn_out, q8, scales, g_sc, g_pd) != cudaSuccess) {
    rmi_set_error("launch of attention_seq failed: %s", cudaGetErrorString(cudaGetLastError()));
    return RMI_ERR_CUDA;
  }
  return rmi_post_launch(ctx, "attention_seq");
}

// The CLI forward's attention: one CTA per (head, sequence).
int32_t launch_attention_online(rmi_ctx* ctx, const decode_dims& d, const float* q32, const uint16_t* k_cache,
                                const uint16_t* v_cache, const int* d_step, size_t layer, float* attn_out, uint8_t* q8,
                                float* scales) {
  RMI_REQUIRE(d.hd % 32 == 0 && d.hd <= 256, RMI_ERR_UNSUPPORTED, "online attention needs head_dim %% 32 == 0 and <= 256");
  const size_t smem = (2 * ((d.capacity + 3) & ~(size_t)3) + d.hd + 256) * 4 + 2 * ATT_TILE * d.hd * 2;
  auto kern = ctx->sem == RMI_SEM_AVX2 ? attention_online_kernel<RMI_SEM_AVX2>
                                       : (ctx->sem == RMI_SEM_NEON ? attention_online_kernel<RMI_SEM_NEON>
                                                                   : attention_online_kernel<RMI_SEM_SCALAR>);
  if (smem > 48 * 1024 && cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) {
    (void)cudaGetLastError();
    rmi_set_error("online attention needs %zu B of shared memory", smem);
    return RMI_ERR_UNSUPPORTED;
  }
  if (rmi_launch(ctx, kern, dim3((unsigned)d.n_head, (unsigned)d.batch), dim3(256), smem, q32, k_cache, v_cache, d_step,
                 d.n_head, d.n_head_kv, d.hd, layer, d.n_layer, d.capacity, attn_out, q8, scales) != cudaSuccess) {
    rmi_set_error("launch of attention_online failed: %s", cudaGetErrorString(cudaGetLastError()));
    return RMI_ERR_CUDA;
  }
  return rmi_post_launch(ctx, "attention_online");
}

template <bool KV16, bool SEQ_PV>
static int32_t launch_attention_softmax_t(rmi_ctx* ctx, const decode_dims& d, const float* q32,
                                          const typename kv_elem<KV16>::type* k_cache,
                                          const typename kv_elem<KV16>::type* v_cache, const int* d_step, size_t layer,
                                          float* attn_out, uint8_t* q8, float* scales) {
  RMI_REQUIRE(d.hd % 32 == 0 && d.hd <= 256, RMI_ERR_UNSUPPORTED, "score-buffer attention needs head_dim %% 32 == 0 and <= 256");
  const size_t smem = (((d.capacity + 3) & ~(size_t)3) + d.hd + 16 * d.hd + 32) * 4 +
                      2 * SM_TILE * (d.hd * sizeof(typename kv_elem<KV16>::type) + 16);
  auto kern = ctx->sem == RMI_SEM_AVX2 ? attention_softmax_kernel<RMI_SEM_AVX2, KV16, SEQ_PV>
                                       : (ctx->sem == RMI_SEM_NEON ? attention_softmax_kernel<RMI_SEM_NEON, KV16, SEQ_PV>
                                                                   : attention_softmax_kernel<RMI_SEM_SCALAR, KV16, SEQ_PV>);
  if (smem > 48 * 1024 && cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) {
    (void)cudaGetLastError();
    rmi_set_error("score-buffer attention needs %zu B of shared memory", smem);
    return RMI_ERR_UNSUPPORTED;
  }
  if (rmi_launch(ctx, kern, dim3((unsigned)d.n_head, (unsigned)d.batch), dim3(256), smem, q32, k_cache, v_cache, d_step,
                 d.n_head, d.n_head_kv, d.hd, layer, d.n_layer, d.capacity, attn_out, q8, scales) != cudaSuccess) {
    rmi_set_error("launch of attention_softmax failed: %s", cudaGetErrorString(cudaGetLastError()));
    return RMI_ERR_CUDA;
  }
  return rmi_post_launch(ctx, "attention_softmax");
}

int32_t launch_attention_f32kv(rmi_ctx* ctx, const decode_dims& d, const float* q32, const float* k_cache,
                               const float* v_cache, const int* d_step, size_t layer, float* attn_out, uint8_t* q8,
                               float* scales, bool sequential_pv) {
  return sequential_pv
             ? launch_attention_softmax_t<false, true>(ctx, d, q32, k_cache, v_cache, d_step, layer, attn_out, q8, scales)
             : launch_attention_softmax_t<false, false>(ctx, d, q32, k_cache, v_cache, d_step, layer, attn_out, q8, scales);
}

int32_t launch_attention_scores_f16kv(rmi_ctx* ctx, const decode_dims& d, const float* q32, const uint16_t* k_cache,
                                      const uint16_t* v_cache, const int* d_step, size_t layer, float* attn_out,
                                      uint8_t* q8, float* scales) {
  return launch_attention_softmax_t<true, true>(ctx, d, q32, k_cache, v_cache, d_step, layer, attn_out, q8, scales);
}

size_t cli_attention_smem_bytes(const decode_dims& d, int forward) {
  const size_t cap4 = (d.capacity + 3) & ~(size_t)3;
  if (forward == RMI_FORWARD_APP_TEXT) return (2 * cap4 + d.hd + 256) * 4 + 2 * ATT_TILE * d.hd * 2;
  const size_t elem = (forward == RMI_FORWARD_APP_LOGITS) ? 2 : 4;   // F16 cache, else one of the F32-cache variants
  return (cap4 + d.hd + 16 * d.hd + 32) * 4 + 2 * SM_TILE * (d.hd * elem + 16);
}

size_t argmax_scratch_floats(size_t batch) { return batch * ARGMAX_SLICES; }

int32_t launch_argmax(rmi_ctx* ctx, const float* logits, size_t vocab, const int* d_step, size_t n_prompt, uint32_t* gen,
                      size_t n_gen, int* flag, size_t batch, float* part_v, uint32_t* part_i, bool last_index) {
  dim3 grid(ARGMAX_SLICES, (unsigned)batch);
  auto k1 = last_index ? argmax_partial_kernel<true> : argmax_partial_kernel<false>;
  auto k2 = last_index ? argmax_final_kernel<true> : argmax_final_kernel<false>;
  if (rmi_launch(ctx, k1, grid, dim3(256), 0, logits, vocab, part_v, part_i, flag) != cudaSuccess ||
      rmi_launch(ctx, k2, dim3((unsigned)batch), dim3(64), 0, part_v, part_i, d_step, n_prompt, gen, n_gen) !=
          cudaSuccess) {
    rmi_set_error("launch of argmax failed: %s", cudaGetErrorString(cudaGetLastError()));
    return RMI_ERR_CUDA;
  }
  ctx->launches.fetch_add(1, std::memory_order_relaxed);
  return rmi_post_launch(ctx, "argmax");
}

int32_t launch_step_inc(rmi_ctx* ctx, int* d_step) {
  if (rmi_launch(ctx, step_inc_kernel, dim3(1), dim3(1), 0, d_step) != cudaSuccess) {
    rmi_set_error("launch of step_inc failed: %s", cudaGetErrorString(cudaGetLastError()));
    return RMI_ERR_CUDA;
  }
  return rmi_post_launch(ctx, "step_inc");
}
