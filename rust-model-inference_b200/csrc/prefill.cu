// Batched prompt processing for the Qwen3 session.
//
// The reference feeds the prompt one position at a time (src/models/qwen3.rs:657-689); every operator of a
// step works on one row, and the only coupling between positions is the K/V cache that attention reads.  So
// the prompt positions 0..P-1 of a sequence can run as P rows through each operator -- the matmuls as
// M = P calls of the same per-row kernels (src/ops/kernel/trait_.rs:78-109 defines an M-row matmul as exactly
// that loop), attention causally per position over the cache rows written by the same launch sequence -- and
// every value (cache rows, hidden state) carries the bits the token loop would have produced.  Only the
// position P = n_prompt-1, whose logits are needed, then runs through the regular decode step.
//
// Kernels here: embedding rows, rms_norm rows (f32 out), per-head q/k norm + rotation + cache append for all
// rows, and causal attention for many query positions.  Their arithmetic restates the same reference code as
// the decode-step kernels (paths inside the reference project):
//   rms_norm       src/ops/norm.rs:3-19           f32 squares summed in f64
//   rope / cache   src/ops/rope.rs:21-37, src/models/qwen3.rs:851-870
//   attention      src/models/qwen3.rs:876-933    f16 q/k/v/p, sequential f64 dots (src/ops/dot.rs:99-119),
//                                                 softmax with the sequential f32 sum (src/ops/attention.rs:28-38)
#include "common.cuh"
#include "decode.cuh"
#include "decode_dev.cuh"
#include "kernels.cuh"

namespace {

// x[r][:] = f16(d) * q of row prompts[b][p]; r = b_local * P + p
__global__ void embed_rows_kernel(const uint8_t* __restrict__ emb, size_t blocks, const uint32_t* __restrict__ prompts,
                                  size_t n_prompt, size_t P, size_t b0, float* __restrict__ x, uint32_t vocab) {
  const size_t r = blockIdx.x, b = b0 + r / P, p = r % P;
  uint32_t tok = prompts[b * n_prompt + p];
  if (tok >= vocab) tok = 0;  // rejected on the host before the first launch
  const uint8_t* base = emb + (size_t)(tok / 16) * blocks * Q8_REC_BYTES;
  const int rr = tok % 16;
  for (size_t i = threadIdx.x; i < blocks * 32; i += blockDim.x) {
    const uint8_t* rec = base + (i / 32) * Q8_REC_BYTES;
    const float d = f16_bits_to_f32(*reinterpret_cast<const uint16_t*>(rec + 2 * rr));
    x[r * blocks * 32 + i] = __fmul_rn(d, (float)(int8_t)rec[32 + 32 * rr + (i & 31)]);
  }
}

// x += add (optional); out = rms_norm(x) * weight.  One CTA of 256 threads per row.
__global__ void rmsnorm_rows_kernel(float* __restrict__ x, const float* __restrict__ add, const float* __restrict__ weight,
                                    size_t n, float eps, float* __restrict__ out) {
  __shared__ double s_part[8];
  __shared__ float s_scale;
  const size_t r = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  float* xr = x + r * n;
  double part = 0.0;
  for (size_t i = threadIdx.x; i < n; i += blockDim.x) {
    float v = xr[i];
    if (add) {
      v = __fadd_rn(v, add[r * n + i]);
      xr[i] = v;
    }
    part += (double)__fmul_rn(v, v);
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
  for (size_t i = threadIdx.x; i < n; i += blockDim.x) out[r * n + i] = __fmul_rn(__fmul_rn(xr[i], sc), weight[i]);
}

// grid (rows, n_head + 2 n_head_kv), one warp per head: q -> q16[r], k/v -> cache row (b, layer, p)
__global__ void qk_norm_rope_kv_rows_kernel(const float* __restrict__ qkv, size_t n_head, size_t n_head_kv, size_t hd,
                                            const float* __restrict__ q_norm, const float* __restrict__ k_norm, float eps,
                                            const float* __restrict__ rope, size_t P, size_t b0,
                                            uint16_t* __restrict__ q16, uint16_t* __restrict__ k_cache,
                                            uint16_t* __restrict__ v_cache, size_t layer, size_t n_layer, size_t capacity) {
  const size_t r = blockIdx.x, head = blockIdx.y, b = b0 + r / P, p = r % P;
  const int lane = threadIdx.x;
  const size_t nq = n_head * hd, nk = n_head_kv * hd;
  const float* src = qkv + r * (nq + 2 * nk) + head * hd;
  const size_t cache_row = ((b * n_layer + layer) * capacity + p) * nk;
  if (head >= n_head + n_head_kv) {  // V: straight f16 conversion
    const size_t kvh = head - n_head - n_head_kv;
    for (size_t i = lane; i < hd; i += 32) v_cache[cache_row + kvh * hd + i] = f32_to_f16_bits(src[i]);
    return;
  }
  const bool is_q = head < n_head;
  uint16_t* dst = is_q ? q16 + r * nq + head * hd : k_cache + cache_row + (head - n_head) * hd;
  norm_rope_head_f16(src, is_q ? q_norm : k_norm, eps, rope + p * hd, hd, lane, dst);
}

// Causal attention of QT consecutive query positions of one (sequence, kv head): the `group` query heads that
// share the kv head are processed together, so a CTA owns QT * group query rows.  K and V stream through two
// shared-memory tiles; the scores of all rows stay in shared memory (row stride = positions visible to the last
// query of the CTA).  Per row the arithmetic is that of one decode step: sequential f64 dot over the head
// dimension, f32 score * 1/sqrt(hd), max, exp, sequential f32 sum over the positions, divide, f16, then per
// output element the f64 sum over the positions in ascending order.
constexpr int PF_TILE = 64;

template <int HD>
__global__ void __launch_bounds__(256)
    attention_prefill_kernel(const uint16_t* __restrict__ q16, const uint16_t* __restrict__ k_cache,
                             const uint16_t* __restrict__ v_cache, size_t n_head, size_t n_head_kv, size_t layer,
                             size_t n_layer, size_t capacity, size_t P, size_t b0, int QT, float* __restrict__ attn_out) {
  extern __shared__ __align__(16) uint8_t smem[];
  const size_t kvh = blockIdx.y, bl = blockIdx.z, b = b0 + bl;
  const int t_first = (int)blockIdx.x * QT;
  const int nqp = min(QT, (int)P - t_first);        // query positions of this CTA
  const int t_last = t_first + nqp - 1;
  const int T = t_last + 1;                          // cache positions any row of the CTA may see
  const int group = (int)(n_head / n_head_kv);
  const int rows = nqp * group;                      // row = qp * group + g
  const size_t nq = n_head * HD, nk = n_head_kv * HD;
  const size_t cs = ((size_t)T + 7) & ~(size_t)7;
  float* sc = reinterpret_cast<float*>(smem);                                   // [QT*group][cs] scores, then weights
  uint16_t* p16 = reinterpret_cast<uint16_t*>(sc + (size_t)QT * group * cs);    // [QT*group][cs]
  uint16_t* qs = p16 + (size_t)QT * group * cs;                                 // [QT*group][HD + 2] (row stride of 65 words: conflict-free)
  // 2 x PF_TILE x HD f16 tiles behind the query rows, on a 16-byte boundary
  uint8_t* tiles = smem + (((size_t)(reinterpret_cast<uint8_t*>(qs + (size_t)QT * group * (HD + 2)) - smem) + 15) & ~(size_t)15);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  constexpr size_t row_bytes = HD * 2, tile_bytes = PF_TILE * row_bytes, row16 = HD / 8;
  const int n_tiles = (T + PF_TILE - 1) / PF_TILE;
  const float kq_scale = __fdiv_rn(1.0f, __fsqrt_rn((float)HD));
  const uint16_t* kbase = k_cache + ((b * n_layer + layer) * capacity) * nk + kvh * HD;
  const uint16_t* vbase = v_cache + ((b * n_layer + layer) * capacity) * nk + kvh * HD;
  auto stage = [&](const uint16_t* base, int tile, int buf) {
    const int t0 = tile * PF_TILE, nt = min(PF_TILE, T - t0);
    uint8_t* dst = tiles + (size_t)buf * tile_bytes;
    for (size_t i = tid; i < (size_t)nt * row16; i += blockDim.x)
      cp_async16(dst + (i / row16) * row_bytes + (i % row16) * 16, base + (size_t)(t0 + i / row16) * nk + (i % row16) * 8);
    cp_async_commit();
  };
  // query rows: q16 row (bl * P + t) holds all heads of position t
  for (size_t i = tid; i < (size_t)rows * (HD / 2); i += blockDim.x) {
    const int row = (int)(i / (HD / 2)), w = (int)(i % (HD / 2));
    const int qp = row / group, g = row % group;
    const uint32_t* src = reinterpret_cast<const uint32_t*>(q16 + (bl * P + t_first + qp) * nq + (kvh * group + g) * HD);
    reinterpret_cast<uint32_t*>(qs + (size_t)row * (HD + 2))[w] = src[w];
  }
  stage(kbase, 0, 0);
  // scores[row][t] = f32(sum_f64 q*k) * kq_scale for t <= position of the row (dot.rs:115-118)
  for (int tile = 0; tile < n_tiles; tile++) {
    if (tile + 1 < n_tiles) stage(kbase, tile + 1, (tile + 1) & 1);
    if (tile + 1 < n_tiles) cp_async_wait<1>(); else cp_async_wait<0>();
    __syncthreads();
    const uint8_t* kt = tiles + (size_t)(tile & 1) * tile_bytes;
    const int t0 = tile * PF_TILE, nt = min(PF_TILE, T - t0);
    for (int item = tid; item < nt * rows; item += blockDim.x) {
      const int tl = item / rows, row = item % rows;
      const int t = t0 + tl, tq = t_first + row / group;
      if (t > tq) continue;  // causal: a query sees positions 0..its own
      const uint32_t* kr = reinterpret_cast<const uint32_t*>(kt + (size_t)tl * row_bytes);
      const uint32_t* qr = reinterpret_cast<const uint32_t*>(qs + (size_t)row * (HD + 2));
      double s = 0.0;
#pragma unroll 8
      for (int i = 0; i < HD / 2; i++) {
        const uint32_t kk = kr[i], qq = qr[i];
        s += (double)__fmul_rn(f16_bits_to_f32((uint16_t)(qq & 0xffff)), f16_bits_to_f32((uint16_t)(kk & 0xffff)));
        s += (double)__fmul_rn(f16_bits_to_f32((uint16_t)(qq >> 16)), f16_bits_to_f32((uint16_t)(kk >> 16)));
      }
      sc[(size_t)row * cs + t] = __fmul_rn((float)s, kq_scale);
    }
    __syncthreads();
  }
  stage(vbase, 0, 0);  // the first V tile travels while the soft-max is evaluated
  // per row: max, exp, sequential f32 sum (attention.rs:28-38), divide, f16
  for (int row = warp; row < rows; row += 8) {
    const int Tr = t_first + row / group + 1;
    float* e = sc + (size_t)row * cs;
    float mx = -INFINITY;
    for (int t = lane; t < Tr; t += 32) mx = fmaxf(mx, e[t]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    for (int t = lane; t < Tr; t += 32) e[t] = exp_cr(__fsub_rn(e[t], mx));
    __syncwarp();
    float sum = 0.0f;
    if (lane == 0) {
      for (int t = 0; t < Tr; t++) sum = __fadd_rn(sum, e[t]);
    }
    sum = __shfl_sync(0xffffffffu, sum, 0);
    uint16_t* pr = p16 + (size_t)row * cs;
    for (int t = lane; t < Tr; t += 32) {
      float pv = e[t];
      if (sum > 0.0f) pv = __fdiv_rn(pv, sum);
      pr[t] = f32_to_f16_bits(pv);
    }
  }
  __syncthreads();
  // out[row][d] = f32(sum_f64 over t ascending of v[t][d] * p[row][t]); thread -> (row, d) pairs, HD consecutive
  // threads share a row so that p is a broadcast and v a conflict-free row read
  constexpr int MAXO = 16;  // outputs per thread: QT * group * HD <= 256 * MAXO
  double accv[MAXO];
#pragma unroll
  for (int u = 0; u < MAXO; u++) accv[u] = 0.0;
  const int n_out = rows * HD;
  for (int tile = 0; tile < n_tiles; tile++) {
    if (tile + 1 < n_tiles) stage(vbase, tile + 1, (tile + 1) & 1);
    if (tile + 1 < n_tiles) cp_async_wait<1>(); else cp_async_wait<0>();
    __syncthreads();
    const uint16_t* vt = reinterpret_cast<const uint16_t*>(tiles + (size_t)(tile & 1) * tile_bytes);
    const int t0 = tile * PF_TILE, nt = min(PF_TILE, T - t0);
#pragma unroll
    for (int u = 0; u < MAXO; u++) {
      const int o = tid + u * 256;
      if (o < n_out) {
        const int row = o / HD, dd = o % HD;
        const int lim = min(nt, t_first + row / group + 1 - t0);  // positions of this tile the row may see
        const uint16_t* pr = p16 + (size_t)row * cs + t0;
        double s = accv[u];
        for (int tl = 0; tl < lim; tl++)
          s += (double)__fmul_rn(f16_bits_to_f32(vt[(size_t)tl * HD + dd]), f16_bits_to_f32(pr[tl]));
        accv[u] = s;
      }
    }
    __syncthreads();
  }
#pragma unroll
  for (int u = 0; u < MAXO; u++) {
    const int o = tid + u * 256;
    if (o < n_out) {
      const int row = o / HD, dd = o % HD;
      const int qp = row / group, g = row % group;
      attn_out[(bl * P + t_first + qp) * nq + (kvh * group + g) * HD + dd] = (float)accv[u];
    }
  }
}

__global__ void set_step_kernel(int* d_step, int value) { *d_step = value; }

size_t prefill_attention_smem(int QT, int group, size_t T, size_t hd) {
  const size_t cs = (T + 7) & ~(size_t)7, rows = (size_t)QT * group;
  return rows * cs * 4 + rows * cs * 2 + rows * (hd + 2) * 2 + 16 + 2 * (size_t)PF_TILE * hd * 2;
}

}  // namespace

// Largest number of query positions per CTA (a power of two up to 16) whose score rows fit in shared memory and
// whose outputs fit the per-thread accumulators; 0 when even one position does not fit.
int prefill_attention_qt(const rmi_ctx* ctx, const decode_dims& d, size_t P) {
  const int group = (int)(d.n_head / d.n_head_kv);
  // first choice: three CTAs per SM (their work grows with the query position, more CTAs even it out)
  for (size_t limit : {(size_t)74 * 1024, ctx->smem_optin}) {
    for (int qt = 16; qt >= 1; qt >>= 1) {
      if ((size_t)qt * group * d.hd > 256 * 16) continue;
      if (prefill_attention_smem(qt, group, P, d.hd) <= limit) return qt;
    }
  }
  return 0;
}

bool prefill_supported(const rmi_ctx* ctx, const decode_dims& d, size_t P) {
  return (d.hd == 128 || d.hd == 64 || d.hd == 32) && d.n_head % d.n_head_kv == 0 && prefill_attention_qt(ctx, d, P) > 0;
}

int32_t launch_embed_rows(rmi_ctx* ctx, const rmi_weight* emb, const uint32_t* prompts, size_t n_prompt, size_t P, size_t b0,
                          size_t rows, float* x) {
  embed_rows_kernel<<<(unsigned)rows, 256, 0, ctx->stream>>>(emb->d_tile16, emb->n_in / 32, prompts, n_prompt, P, b0, x,
                                                           (uint32_t)emb->n_rows);
  return rmi_post_launch(ctx, "embed_rows");
}

int32_t launch_rmsnorm_rows(rmi_ctx* ctx, float* x, const float* add, const float* weight, size_t n, float eps, float* out,
                            size_t rows) {
  rmsnorm_rows_kernel<<<(unsigned)rows, 256, 0, ctx->stream>>>(x, add, weight, n, eps, out);
  return rmi_post_launch(ctx, "rmsnorm_rows");
}

int32_t launch_qk_norm_rope_kv_rows(rmi_ctx* ctx, const decode_dims& d, const float* qkv, const float* q_norm,
                                    const float* k_norm, const float* rope, size_t P, size_t b0, size_t rows, uint16_t* q16,
                                    uint16_t* k_cache, uint16_t* v_cache, size_t layer) {
  dim3 grid((unsigned)rows, (unsigned)(d.n_head + 2 * d.n_head_kv));
  qk_norm_rope_kv_rows_kernel<<<grid, 32, 0, ctx->stream>>>(qkv, d.n_head, d.n_head_kv, d.hd, q_norm, k_norm, d.eps, rope, P,
                                                            b0, q16, k_cache, v_cache, layer, d.n_layer, d.capacity);
  return rmi_post_launch(ctx, "qk_norm_rope_kv_rows");
}

int32_t launch_attention_prefill(rmi_ctx* ctx, const decode_dims& d, const uint16_t* q16, const uint16_t* k_cache,
                                 const uint16_t* v_cache, size_t layer, size_t P, size_t b0, size_t n_seq, float* attn_out) {
  const int qt = prefill_attention_qt(ctx, d, P);
  RMI_REQUIRE(qt > 0, RMI_ERR_UNSUPPORTED, "prompt of %zu positions does not fit the prefill attention kernel", P);
  const int group = (int)(d.n_head / d.n_head_kv);
  const size_t smem = prefill_attention_smem(qt, group, P, d.hd);
  void (*kern)(const uint16_t*, const uint16_t*, const uint16_t*, size_t, size_t, size_t, size_t, size_t, size_t, size_t, int,
               float*) = d.hd == 128 ? attention_prefill_kernel<128>
                                     : (d.hd == 64 ? attention_prefill_kernel<64> : attention_prefill_kernel<32>);
  if (smem > 48 * 1024 && cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) {
    (void)cudaGetLastError();
    rmi_set_error("prefill attention needs %zu B of shared memory", smem);
    return RMI_ERR_UNSUPPORTED;
  }
  dim3 grid((unsigned)((P + qt - 1) / qt), (unsigned)d.n_head_kv, (unsigned)n_seq);
  kern<<<grid, 256, smem, ctx->stream>>>(q16, k_cache, v_cache, d.n_head, d.n_head_kv, layer, d.n_layer, d.capacity, P, b0, qt,
                                         attn_out);
  return rmi_post_launch(ctx, "attention_prefill");
}

int32_t launch_set_step(rmi_ctx* ctx, int* d_step, int value) {
  set_step_kernel<<<1, 1, 0, ctx->stream>>>(d_step, value);
  return rmi_post_launch(ctx, "set_step");
}
